// Differential attention: two softmax maps a head over the same values, combined as a1 - lambda a2.
//
// The cache holds one vector per token, [k: kv_heads x 2 x dim | v: kv_heads x vdim] (after norm and rotation), in
// pages: cache[page][offset][width].
//
//   diff_qk_prepare          per row: RMS norm (one weight vector for all heads and maps) and rotation of every q and k
//                            map; q is changed in place, k and v go to the row's slot of the cache
//   diff_attention_generic   a warp a (row, head): keys in chunks of 32 at fixed places (a lane a key for the scores,
//                            a lane a value column for the sums), both maps side by side, 32-bit throughout; the
//                            result does not depend on the step's make-up by a single bit
#include "common.cuh"

namespace pih {

constexpr int kDiffMaxPerLane = 8;          // dim, vdim <= 256

template <typename T>
__global__ void __launch_bounds__(128)
diff_qk_prepare_kernel(T* __restrict__ qkv, long long ld, const float* __restrict__ q_norm, const float* __restrict__ k_norm,
                       float eps, const float* __restrict__ freq, int rot, const int* __restrict__ positions,
                       const int* __restrict__ slot_mapping, T* __restrict__ cache, long long cache_slots, int heads,
                       int kv_heads, int dim, int vdim, int write_kv, uint32_t* __restrict__ error) {
  extern __shared__ float smem[];
  wait_for_prior_kernels();
  launch_dependents();
  const int row = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  float* buf = smem + warp * dim;
  const int nq = heads * 2, nk = write_kv ? kv_heads * 2 : 0;
  const long long width = static_cast<long long>(kv_heads) * (2 * dim + vdim);
  int slot = write_kv ? slot_mapping[row] : 0;
  if (write_kv && slot != kPaddingSlot && (slot < 0 || slot >= cache_slots)) {
    if (threadIdx.x == 0) publish_error(error, kRowWithoutPage);
    slot = kPaddingSlot;
  }
  const float pos = static_cast<float>(positions[row]);
  const int half = rot >> 1;
  T* x = qkv + row * ld;
  for (int unit = warp; unit < nq + nk; unit += warps) {
    T* xu = x + static_cast<long long>(unit) * dim;
    const float* w = unit < nq ? q_norm : k_norm;
    float ss = 0.0f;
    for (int e = lane; e < dim; e += 32) {
      const float v = to_float<T>(xu[e]);
      buf[e] = v;
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float inv = w != nullptr ? 1.0f / sqrtf(ss / static_cast<float>(dim) + eps) : 1.0f;
    __syncwarp();
    for (int e = lane; e < dim; e += 32) buf[e] = w != nullptr ? buf[e] * inv * w[e] : buf[e];
    __syncwarp();
    T* dst = unit < nq ? xu : (slot >= 0 ? cache + slot * width + static_cast<long long>(unit - nq) * dim : nullptr);
    for (int e = lane; e < dim; e += 32) {
      float o;
      if (e < rot) {
        const int pair = e < half ? e : e - half;
        float sn, cs;
        sincosf(pos * freq[pair], &sn, &cs);
        const float u = buf[pair], v = buf[pair + half];
        o = e < half ? u * cs - v * sn : v * cs + u * sn;
      } else {
        o = buf[e];
      }
      if (dst != nullptr) dst[e] = from_float<T>(o);
    }
    __syncwarp();
  }
  if (write_kv && slot >= 0) {
    const T* v = x + static_cast<long long>(nq + nk) * dim;
    T* dst = cache + slot * width + static_cast<long long>(nk) * dim;
    for (int e = threadIdx.x; e < kv_heads * vdim; e += blockDim.x) dst[e] = v[e];
  }
}

// What follows the two maps' sums of a (row, head): o = a1 / l1 - lambda a2 / l2, divided by its root mean square over
// vdim, times out_scale.  A lane holds columns lane + 32 e.
template <typename T>
__device__ __forceinline__ void diff_finish(const float* a1, const float* a2, float l1, float l2, float lam, float eps,
                                            float out_scale, int vdim, int lane, T* __restrict__ out) {
  float o[kDiffMaxPerLane];
  float ss = 0.0f;
  const float i1 = 1.0f / l1, i2 = 1.0f / l2;
#pragma unroll
  for (int e = 0; e < kDiffMaxPerLane; ++e) {
    o[e] = (lane + 32 * e < vdim) ? a1[e] * i1 - lam * (a2[e] * i2) : 0.0f;
    ss = fmaf(o[e], o[e], ss);
  }
  ss = warp_sum(ss);
  const float inv = out_scale / sqrtf(ss / static_cast<float>(vdim) + eps);
#pragma unroll
  for (int e = 0; e < kDiffMaxPerLane; ++e)
    if (lane + 32 * e < vdim) out[lane + 32 * e] = from_float<T>(o[e] * inv);
}

template <typename T>
__global__ void __launch_bounds__(128)
diff_attention_generic_kernel(const T* __restrict__ qkv, long long ld, T* __restrict__ out, const T* __restrict__ cache,
                              const int* __restrict__ block_table, int table_width, const int* __restrict__ request_of_row,
                              const int* __restrict__ positions, int rows, int heads, int kv_heads, int dim, int vdim,
                              int page_size, int num_pages, float scale, float lam, float out_scale, float eps, int window,
                              uint32_t* __restrict__ error) {
  extern __shared__ float smem[];
  wait_for_prior_kernels();
  launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long unit = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + warp;
  if (unit >= static_cast<long long>(rows) * heads) return;
  const int row = static_cast<int>(unit / heads), head = static_cast<int>(unit % heads);
  const int req = request_of_row[row];
  if (req < 0) {                                           // a row of padding: zeros, so that nothing unset travels on
    T* o = out + static_cast<long long>(row) * heads * vdim + static_cast<long long>(head) * vdim;
    for (int e = lane; e < vdim; e += 32) o[e] = from_float<T>(0.0f);
    return;
  }
  const int g = head / (heads / kv_heads);
  const long long width = static_cast<long long>(kv_heads) * (2 * dim + vdim);
  float* q = smem + warp * 2 * dim;                        // map 1 | map 2
  const T* qr = qkv + row * ld + static_cast<long long>(head) * 2 * dim;
  for (int e = lane; e < 2 * dim; e += 32) q[e] = to_float<T>(qr[e]);
  __syncwarp();
  const int pos = positions[row];
  const int first = window > 0 ? max(0, pos - window + 1) : 0;
  const int* table = block_table + static_cast<long long>(req) * table_width;
  float a1[kDiffMaxPerLane], a2[kDiffMaxPerLane];
#pragma unroll
  for (int e = 0; e < kDiffMaxPerLane; ++e) a1[e] = a2[e] = 0.0f;
  float m1 = -INFINITY, m2 = -INFINITY, l1 = 0.0f, l2 = 0.0f;
  for (int j0 = first & ~31; j0 <= pos; j0 += 32) {
    const int j = j0 + lane;
    const bool live = j >= first && j <= pos;
    long long at = -1;
    if (live) {
      const int page = table[j / page_size];
      if (page < 0 || page >= num_pages) publish_error(error, kRowWithoutPage);
      else at = (static_cast<long long>(page) * page_size + j % page_size) * width;
    }
    float s1 = -INFINITY, s2 = -INFINITY;
    if (at >= 0) {
      const T* k = cache + at + static_cast<long long>(g) * 2 * dim;
      float d1 = 0.0f, d2 = 0.0f;
      for (int e = 0; e < dim; ++e) {
        d1 = fmaf(q[e], to_float<T>(k[e]), d1);
        d2 = fmaf(q[dim + e], to_float<T>(k[dim + e]), d2);
      }
      s1 = d1 * scale;
      s2 = d2 * scale;
    }
    const float n1 = fmaxf(m1, warp_max(s1)), n2 = fmaxf(m2, warp_max(s2));
    if (n1 == -INFINITY) continue;                          // (no live key in the chunk: cannot happen for j0 <= pos)
    const float p1 = at >= 0 ? expf(s1 - n1) : 0.0f, p2 = at >= 0 ? expf(s2 - n2) : 0.0f;
    const float c1 = expf(m1 - n1), c2 = expf(m2 - n2);    // exp(-inf) = 0 at the first chunk
    l1 = fmaf(l1, c1, warp_sum(p1));
    l2 = fmaf(l2, c2, warp_sum(p2));
    m1 = n1;
    m2 = n2;
#pragma unroll
    for (int e = 0; e < kDiffMaxPerLane; ++e) { a1[e] *= c1; a2[e] *= c2; }
    const long long v_at = at >= 0 ? at + static_cast<long long>(kv_heads) * 2 * dim + static_cast<long long>(g) * vdim : -1;
    for (int jj = 0; jj < 32; ++jj) {
      const long long va = __shfl_sync(0xffffffffu, v_at, jj);
      const float w1 = __shfl_sync(0xffffffffu, p1, jj), w2 = __shfl_sync(0xffffffffu, p2, jj);
      if (va < 0) continue;
      const T* v = cache + va;
#pragma unroll
      for (int e = 0; e < kDiffMaxPerLane; ++e) {
        if (lane + 32 * e < vdim) {
          const float x = to_float<T>(v[lane + 32 * e]);
          a1[e] = fmaf(w1, x, a1[e]);
          a2[e] = fmaf(w2, x, a2[e]);
        }
      }
    }
  }
  if (!(l1 > 0.0f) || !(l2 > 0.0f) || l1 > 3.0e38f || l2 > 3.0e38f) {
    if (lane == 0) publish_error(error, kAttentionDenominator);
    l1 = l2 = 1.0f;
  }
  diff_finish<T>(a1, a2, l1, l2, lam, eps, out_scale, vdim, lane,
                 out + static_cast<long long>(row) * heads * vdim + static_cast<long long>(head) * vdim);
}

}  // namespace pih

using namespace pih;
typedef __nv_bfloat16 bf16;

// qkv [rows, ld]: q [heads, 2, dim] | k [kv_heads, 2, dim] | v [kv_heads, vdim] (k and v only with write_kv);
// q_norm, k_norm fp32 [dim] or null; freq fp32 [rot / 2]; cache [num_pages, page_size, kv_heads (2 dim + vdim)].
extern "C" int pih_diff_qk_prepare(int dtype, void* qkv, long long ld, const void* q_norm, const void* k_norm, float eps,
                                   const void* freq, int rot, const void* positions, const void* slot_mapping, void* cache,
                                   int page_size, int num_pages, int rows, int heads, int kv_heads, int dim, int vdim,
                                   int write_kv, void* error, void* stream) {
  if (rows <= 0) return 0;
  if (rot < 0 || rot > dim || (rot & 1) || (rot > 0 && freq == nullptr) || heads < 1 || kv_heads < 1) return PIH_ERR_BAD_ARGUMENT;
  if (dim > 4096) return PIH_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t smem = 4 * static_cast<size_t>(dim) * sizeof(float);
  const long long slots = static_cast<long long>(num_pages) * page_size;
#define PIH_DQK(T)                                                                                                     \
  launch_kernel(diff_qk_prepare_kernel<T>, dim3(rows), dim3(128), smem, s, static_cast<T*>(qkv), ld,                   \
                static_cast<const float*>(q_norm), static_cast<const float*>(k_norm), eps, static_cast<const float*>(freq), \
                rot, static_cast<const int*>(positions), static_cast<const int*>(slot_mapping), static_cast<T*>(cache), \
                slots, heads, kv_heads, dim, vdim, write_kv, static_cast<uint32_t*>(error))
  if (dtype == PIH_F32) PIH_DQK(float);
  else if (dtype == PIH_BF16) PIH_DQK(bf16);
  else return PIH_ERR_BAD_ARGUMENT;
#undef PIH_DQK
  PIH_LAUNCH_CHECK();
  return 0;
}

extern "C" int pih_diff_attention_generic(int dtype, const void* qkv, long long ld, void* out, const void* cache,
                                          const void* block_table, int table_width, const void* request_of_row,
                                          const void* positions, int rows, int heads, int kv_heads, int dim, int vdim,
                                          int page_size, int num_pages, float scale, float lam, float out_scale, float eps,
                                          int window, void* error, void* stream) {
  if (rows <= 0) return 0;
  if (dim > 32 * kDiffMaxPerLane * 4 || vdim > 32 * kDiffMaxPerLane || heads % kv_heads) return PIH_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long units = static_cast<long long>(rows) * heads;
  const size_t smem = 4 * 2 * static_cast<size_t>(dim) * sizeof(float);
#define PIH_DAG(T)                                                                                                     \
  launch_kernel(diff_attention_generic_kernel<T>, dim3(static_cast<unsigned>((units + 3) / 4)), dim3(128), smem, s,    \
                static_cast<const T*>(qkv), ld, static_cast<T*>(out), static_cast<const T*>(cache),                    \
                static_cast<const int*>(block_table), table_width, static_cast<const int*>(request_of_row),            \
                static_cast<const int*>(positions), rows, heads, kv_heads, dim, vdim, page_size, num_pages, scale, lam, \
                out_scale, eps, window, static_cast<uint32_t*>(error))
  if (dtype == PIH_F32) PIH_DAG(float);
  else if (dtype == PIH_BF16) PIH_DAG(bf16);
  else return PIH_ERR_BAD_ARGUMENT;
#undef PIH_DAG
  PIH_LAUNCH_CHECK();
  return 0;
}
