// Retention: linear attention with a fixed decay a head and a matrix state per (request, head).
//
//   retention_prepare      q and k of every row rotated by the row's position (angles formed in 32-bit from the
//                          frequencies), k then scaled: 32-bit copies [rows, heads, dim]
//   retention_recurrence   per token  S <- S + (decay - 1) S + k v^T,  o = S^T q,  from the request's state slot
//
// The order of the additions of a read-out is fixed by the kernel: it does not depend on how a sequence is cut into
// steps or on what else a step holds.
#include "common.cuh"

namespace pih {

// A thread an element of q and of k.  Rotate-half over the first ``rot`` columns: column i < rot / 2 pairs with
// i + rot / 2; (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = position * freq[i].
template <typename T>
__global__ void __launch_bounds__(256)
retention_prepare_kernel(const T* __restrict__ qk, long long ld, const float* __restrict__ freq,
                         const int* __restrict__ positions, float* __restrict__ qf, float* __restrict__ kf, int rows,
                         int heads, int dim, int rot, float key_scale) {
  wait_for_prior_kernels();
  launch_dependents();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long per_row = static_cast<long long>(heads) * dim;
  if (i >= rows * per_row) return;
  const int row = static_cast<int>(i / per_row);
  const int e = static_cast<int>(i % dim);
  const long long head_at = (i - static_cast<long long>(row) * per_row) - e;        // head * dim
  const T* q = qk + row * ld + head_at;
  const T* k = q + per_row;
  float qo, ko;
  const int half = rot >> 1;
  if (e < rot) {
    const int pair = e < half ? e : e - half;
    float sn, cs;
    sincosf(static_cast<float>(positions[row]) * freq[pair], &sn, &cs);
    const float qu = to_float<T>(q[pair]), qv = to_float<T>(q[pair + half]);
    const float ku = to_float<T>(k[pair]), kv = to_float<T>(k[pair + half]);
    if (e < half) {
      qo = qu * cs - qv * sn;
      ko = ku * cs - kv * sn;
    } else {
      qo = qv * cs + qu * sn;
      ko = kv * cs + ku * sn;
    }
  } else {
    qo = to_float<T>(q[e]);
    ko = to_float<T>(k[e]);
  }
  qf[i] = qo;
  kf[i] = ko * key_scale;
}

// Block (request, head, slab of value columns); thread j owns column v0 + j of S (all ``dim`` rows, in shared memory:
// S[i][j]).  The next token's k and q are fetched into registers while this token is computed.  Any dim.
template <typename T>
__global__ void retention_recurrence_kernel(const float* __restrict__ qf, const float* __restrict__ kf,
                                            const T* __restrict__ v, long long ldv, const float* __restrict__ decay_m1,
                                            float* __restrict__ out, float* __restrict__ state, long long state_stride,
                                            const int* __restrict__ cu_q, const int* __restrict__ state_slots, int heads,
                                            int dim, int vdim) {
  extern __shared__ float smem[];
  wait_for_prior_kernels();
  launch_dependents();
  const int r = blockIdx.x, h = blockIdx.y;
  const int cols = blockDim.x;
  const int j = threadIdx.x, col = blockIdx.z * cols + j;
  const int lo = cu_q[r], hi = cu_q[r + 1];
  const int slot = state_slots[r];
  if (hi <= lo || slot < 0) return;
  float* S = smem;                          // [dim][cols]
  float* kq = smem + dim * cols;            // [2 buffers][k: dim | q: dim]
  const bool live = col < vdim;
  float* Sg = state + slot * state_stride + (static_cast<long long>(h) * dim) * vdim;
  for (int i = 0; i < dim; ++i) S[i * cols + j] = live ? Sg[static_cast<long long>(i) * vdim + col] : 0.0f;
  const float dm1 = decay_m1[h];
  const int per = (2 * dim + cols - 1) / cols;                   // numbers of k|q a thread fetches
  auto fetch = [&](int t, int e) -> float {
    const int idx = j + e * cols;
    if (idx >= 2 * dim) return 0.0f;
    const float* src = idx < dim ? kf : qf;
    return src[(static_cast<long long>(t) * heads + h) * dim + (idx < dim ? idx : idx - dim)];
  };
  constexpr int kMaxPer = 32;               // dim <= 16 * cols
  float nxt[kMaxPer];
#pragma unroll
  for (int e = 0; e < kMaxPer; ++e) nxt[e] = e < per ? fetch(lo, e) : 0.0f;
  for (int t = lo; t < hi; ++t) {
    float* cur = kq + (t & 1) * 2 * dim;
#pragma unroll
    for (int e = 0; e < kMaxPer; ++e)
      if (e < per && j + e * cols < 2 * dim) cur[j + e * cols] = nxt[e];
    __syncthreads();
    if (t + 1 < hi) {
#pragma unroll
      for (int e = 0; e < kMaxPer; ++e) nxt[e] = e < per ? fetch(t + 1, e) : 0.0f;
    }
    const float vj = live ? to_float<T>(v[static_cast<long long>(t) * ldv + static_cast<long long>(h) * vdim + col]) : 0.0f;
    const float* k = cur;
    const float* q = cur + dim;
    float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
    int i = 0;
    for (; i + 4 <= dim; i += 4) {
      const float s0 = fmaf(k[i + 0], vj, fmaf(dm1, S[(i + 0) * cols + j], S[(i + 0) * cols + j]));
      const float s1 = fmaf(k[i + 1], vj, fmaf(dm1, S[(i + 1) * cols + j], S[(i + 1) * cols + j]));
      const float s2 = fmaf(k[i + 2], vj, fmaf(dm1, S[(i + 2) * cols + j], S[(i + 2) * cols + j]));
      const float s3 = fmaf(k[i + 3], vj, fmaf(dm1, S[(i + 3) * cols + j], S[(i + 3) * cols + j]));
      S[(i + 0) * cols + j] = s0; S[(i + 1) * cols + j] = s1; S[(i + 2) * cols + j] = s2; S[(i + 3) * cols + j] = s3;
      o0 = fmaf(s0, q[i + 0], o0); o1 = fmaf(s1, q[i + 1], o1); o2 = fmaf(s2, q[i + 2], o2); o3 = fmaf(s3, q[i + 3], o3);
    }
    for (; i < dim; ++i) {
      const float s0 = fmaf(k[i], vj, fmaf(dm1, S[i * cols + j], S[i * cols + j]));
      S[i * cols + j] = s0;
      o0 = fmaf(s0, q[i], o0);
    }
    if (live) out[(static_cast<long long>(t) * heads + h) * vdim + col] = (o0 + o1) + (o2 + o3);
  }
  if (live)
    for (int i = 0; i < dim; ++i) Sg[static_cast<long long>(i) * vdim + col] = S[i * cols + j];
}

}  // namespace pih

using namespace pih;
typedef __nv_bfloat16 bf16;

// qk [rows, ld]: q heads then k heads ([heads, dim] each); v [rows, ldv]: [heads, vdim]; freq fp32 [rot / 2] (null: no
// rotation); decay_m1 fp32 [heads]: decay - 1; scratch fp32 [2 * rows * heads * dim]; out fp32 [rows, heads, vdim];
// state fp32: S of (slot, head) at state + slot * state_stride + head * dim * vdim, [dim, vdim].
extern "C" int pih_retention(int dtype, const void* qk, long long ld, const void* v, long long ldv, const void* freq, int rot,
                             const void* positions, const void* decay_m1, float key_scale, void* scratch, void* out,
                             void* state, long long state_stride, const void* cu_q, const void* state_slots, int rows,
                             int requests, int heads, int dim, int vdim, void* stream) {
  if (rows <= 0 || requests <= 0) return 0;
  if (rot < 0 || rot > dim || (rot & 1) || (rot > 0 && freq == nullptr)) return PIH_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int cols = vdim >= 64 ? 64 : 32;
  if (dim > 16 * cols) return PIH_ERR_UNSUPPORTED;
  const size_t smem = (static_cast<size_t>(dim) * cols + 4 * dim) * sizeof(float);
  if (smem > 200 * 1024) return PIH_ERR_UNSUPPORTED;
  float* qf = static_cast<float*>(scratch);
  float* kf = qf + static_cast<long long>(rows) * heads * dim;
  const long long n = static_cast<long long>(rows) * heads * dim;
  const dim3 grid(requests, heads, (vdim + cols - 1) / cols);
#define PIH_RET(T)                                                                                                     \
  do {                                                                                                                 \
    launch_kernel(retention_prepare_kernel<T>, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, s,          \
                  static_cast<const T*>(qk), ld, static_cast<const float*>(freq), static_cast<const int*>(positions),  \
                  qf, kf, rows, heads, dim, rot, key_scale);                                                           \
    PIH_LAUNCH_CHECK();                                                                                                \
    if (smem > 48 * 1024)                                                                                              \
      cudaFuncSetAttribute(retention_recurrence_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,                \
                           static_cast<int>(smem));                                                                    \
    launch_kernel(retention_recurrence_kernel<T>, grid, dim3(cols), smem, s, static_cast<const float*>(qf),            \
                  static_cast<const float*>(kf), static_cast<const T*>(v), ldv, static_cast<const float*>(decay_m1),   \
                  static_cast<float*>(out), static_cast<float*>(state), state_stride, static_cast<const int*>(cu_q),   \
                  static_cast<const int*>(state_slots), heads, dim, vdim);                                             \
  } while (0)
  if (dtype == PIH_F32) PIH_RET(float);
  else if (dtype == PIH_BF16) PIH_RET(bf16);
  else return PIH_ERR_BAD_ARGUMENT;
#undef PIH_RET
  PIH_LAUNCH_CHECK();
  return 0;
}
