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
//   diff_attention_tile      bf16, tensor cores (mma.sync m16n8k16), requests of more than 16 rows: a warp 16 rows and
//                            one map of a (request, head), a block 8 such warps that share tiles of 64 keys fetched by
//                            cp.async into two buffers; scores, softmax and sums 32-bit; the weights enter the product
//                            with the values as a bf16 pair (rounding and remainder), so that they count with 16 bits
//   diff_attention_split     requests of at most 16 rows: the keys of a (row, head) cut into parts side by side (the
//                            generic kernel's loop over a stretch of keys), then diff_attention_merge in order
#include "common.cuh"
#include "mma.cuh"

namespace pih {

constexpr int kDiffMaxPerLane = 16;         // value columns a lane at most: vdim <= 512 (instances: 2, 4, 8, 16)

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
  for (int unit = blockIdx.y * warps + warp; unit < nq + nk; unit += gridDim.y * warps) {
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
  if (write_kv && slot >= 0 && blockIdx.y == 0) {
    const T* v = x + static_cast<long long>(nq + nk) * dim;
    T* dst = cache + slot * width + static_cast<long long>(nk) * dim;
    for (int e = threadIdx.x; e < kv_heads * vdim; e += blockDim.x) dst[e] = v[e];
  }
}

// What follows the two maps' sums of a (row, head): o = a1 / l1 - lambda a2 / l2, divided by its root mean square over
// vdim, times out_scale.  A lane holds columns lane + 32 e.
template <typename T, int PL>
__device__ __forceinline__ void diff_finish(const float* a1, const float* a2, float l1, float l2, float lam, float eps,
                                            float out_scale, int vdim, int lane, T* __restrict__ out) {
  float o[PL];
  float ss = 0.0f;
  const float i1 = 1.0f / l1, i2 = 1.0f / l2;
#pragma unroll
  for (int e = 0; e < PL; ++e) {
    o[e] = (lane + 32 * e < vdim) ? a1[e] * i1 - lam * (a2[e] * i2) : 0.0f;
    ss = fmaf(o[e], o[e], ss);
  }
  ss = warp_sum(ss);
  const float inv = out_scale / sqrtf(ss / static_cast<float>(vdim) + eps);
#pragma unroll
  for (int e = 0; e < PL; ++e)
    if (lane + 32 * e < vdim) out[lane + 32 * e] = from_float<T>(o[e] * inv);
}

// The sums of both maps of one (row, head) over the keys first .. last (absolute places; chunks of 32 at multiples of
// 32): a lane a key for the scores, a lane a value column (lane + 32 e) for the sums.  q: 32-bit, [map 1 | map 2].
template <typename T, int PL>
__device__ __forceinline__ void diff_stretch(const float* q, const T* __restrict__ cache, const int* __restrict__ table,
                                             int first, int last, int g, int kv_heads, int dim, int vdim, int page_size,
                                             int num_pages, float scale, int lane, float (&a1)[PL],
                                             float (&a2)[PL], float& m1, float& m2, float& l1, float& l2,
                                             uint32_t* __restrict__ error) {
  const long long width = static_cast<long long>(kv_heads) * (2 * dim + vdim);
  for (int j0 = first & ~31; j0 <= last; j0 += 32) {
    const int j = j0 + lane;
    const bool live = j >= first && j <= last;
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
      constexpr int kVec = 16 / sizeof(T);
      if (dim % kVec == 0 && width % kVec == 0) {           // 16-byte loads; the additions in the same order
        // four pieces of each map are asked for before the first is used: a lane has up to eight loads in flight
        for (int e0 = 0; e0 < dim; e0 += 4 * kVec) {
          uint4 r1[4], r2[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int e = min(e0 + u * kVec, dim - kVec);     // (a piece beyond the end: the last one again, not used)
            r1[u] = *reinterpret_cast<const uint4*>(k + e);
            r2[u] = *reinterpret_cast<const uint4*>(k + dim + e);
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int e = e0 + u * kVec;
            if (e < dim) {
              const T* k1 = reinterpret_cast<const T*>(&r1[u]);
              const T* k2 = reinterpret_cast<const T*>(&r2[u]);
#pragma unroll
              for (int i = 0; i < kVec; ++i) {
                d1 = fmaf(q[e + i], to_float<T>(k1[i]), d1);
                d2 = fmaf(q[dim + e + i], to_float<T>(k2[i]), d2);
              }
            }
          }
        }
      } else {
        for (int e = 0; e < dim; ++e) {
          d1 = fmaf(q[e], to_float<T>(k[e]), d1);
          d2 = fmaf(q[dim + e], to_float<T>(k[dim + e]), d2);
        }
      }
      s1 = d1 * scale;
      s2 = d2 * scale;
    }
    const float n1 = fmaxf(m1, warp_max(s1)), n2 = fmaxf(m2, warp_max(s2));
    if (n1 == -INFINITY) continue;                          // no live key in the chunk
    const float p1 = at >= 0 ? expf(s1 - n1) : 0.0f, p2 = at >= 0 ? expf(s2 - n2) : 0.0f;
    const float c1 = expf(m1 - n1), c2 = expf(m2 - n2);    // exp(-inf) = 0 at the first chunk
    l1 = fmaf(l1, c1, warp_sum(p1));
    l2 = fmaf(l2, c2, warp_sum(p2));
    m1 = n1;
    m2 = n2;
#pragma unroll
    for (int e = 0; e < PL; ++e) { a1[e] *= c1; a2[e] *= c2; }
    const long long v_at = at >= 0 ? at + static_cast<long long>(kv_heads) * 2 * dim + static_cast<long long>(g) * vdim : -1;
    // The values of kBatch keys are asked for together (a key without a place reads the cache's first row and counts as
    // zeros): shuffles first, then all loads, then the sums in the keys' order.
    constexpr int kBatch = PL <= 4 ? 8 : (PL <= 8 ? 4 : 2);
    for (int j8 = 0; j8 < 32; j8 += kBatch) {
      long long va[kBatch];
      float w1[kBatch], w2[kBatch], x[kBatch][PL];
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
        va[b] = __shfl_sync(0xffffffffu, v_at, j8 + b);
        w1[b] = __shfl_sync(0xffffffffu, p1, j8 + b);
        w2[b] = __shfl_sync(0xffffffffu, p2, j8 + b);
      }
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
        const T* v = cache + (va[b] >= 0 ? va[b] : 0);
#pragma unroll
        for (int e = 0; e < PL; ++e) x[b][e] = (lane + 32 * e < vdim) ? to_float<T>(v[lane + 32 * e]) : 0.0f;
      }
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
        const bool there = va[b] >= 0;
#pragma unroll
        for (int e = 0; e < PL; ++e) {
          const float xv = there ? x[b][e] : 0.0f;
          a1[e] = fmaf(w1[b], xv, a1[e]);
          a2[e] = fmaf(w2[b], xv, a2[e]);
        }
      }
    }
  }
}

// A warp a (row, head) and a part of its keys.  splits == 1: the whole row, finished here (``partial`` unused).  More:
// part ``blockIdx.y`` of the keys of rows whose request brings at most ``small_rows`` rows (the others are the tile
// kernel's), its sums to ``partial`` [row][head][split][4 + 2 vdim]: m1, l1, m2, l2, a1, a2.
template <typename T, int PL>
__global__ void __launch_bounds__(128)
diff_attention_generic_kernel(const T* __restrict__ qkv, long long ld, T* __restrict__ out, const T* __restrict__ cache,
                              const int* __restrict__ block_table, int table_width, const int* __restrict__ request_of_row,
                              const int* __restrict__ positions, const int* __restrict__ cu_q, int rows, int heads,
                              int kv_heads, int dim, int vdim, int page_size, int num_pages, float scale, float lam,
                              float out_scale, float eps, int window, int splits, int small_rows,
                              float* __restrict__ partial, uint32_t* __restrict__ error) {
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
    if (blockIdx.y == 0)
      for (int e = lane; e < vdim; e += 32) o[e] = from_float<T>(0.0f);
    return;
  }
  if (splits > 1 && cu_q[req + 1] - cu_q[req] > small_rows) return;
  const int g = head / (heads / kv_heads);
  float* q = smem + warp * 2 * dim;                        // map 1 | map 2
  const T* qr = qkv + row * ld + static_cast<long long>(head) * 2 * dim;
  for (int e = lane; e < 2 * dim; e += 32) q[e] = to_float<T>(qr[e]);
  __syncwarp();
  const int pos = positions[row];
  int first = window > 0 ? max(0, pos - window + 1) : 0, last = pos;
  if (splits > 1) {                                        // equal stretches of whole chunks
    const int chunk0 = first >> 5, chunks = (pos >> 5) - chunk0 + 1;
    const int per = (chunks + splits - 1) / splits;
    const int c_lo = chunk0 + static_cast<int>(blockIdx.y) * per;
    first = max(first, c_lo << 5);
    last = min(pos, ((c_lo + per) << 5) - 1);
  }
  const int* table = block_table + static_cast<long long>(req) * table_width;
  float a1[PL], a2[PL];
#pragma unroll
  for (int e = 0; e < PL; ++e) a1[e] = a2[e] = 0.0f;
  float m1 = -INFINITY, m2 = -INFINITY, l1 = 0.0f, l2 = 0.0f;
  if (first <= last)
    diff_stretch<T, PL>(q, cache, table, first, last, g, kv_heads, dim, vdim, page_size, num_pages, scale, lane, a1, a2, m1, m2,
                    l1, l2, error);
  if (splits > 1) {
    float* p = partial + ((static_cast<long long>(row) * heads + head) * splits + blockIdx.y) * (4 + 2 * vdim);
    if (lane == 0) { p[0] = m1; p[1] = l1; p[2] = m2; p[3] = l2; }
#pragma unroll
    for (int e = 0; e < PL; ++e)
      if (lane + 32 * e < vdim) { p[4 + lane + 32 * e] = a1[e]; p[4 + vdim + lane + 32 * e] = a2[e]; }
    return;
  }
  if (!(l1 > 0.0f) || !(l2 > 0.0f) || l1 > 3.0e38f || l2 > 3.0e38f) {
    if (lane == 0) publish_error(error, kAttentionDenominator);
    l1 = l2 = 1.0f;
  }
  diff_finish<T, PL>(a1, a2, l1, l2, lam, eps, out_scale, vdim, lane,
                 out + static_cast<long long>(row) * heads * vdim + static_cast<long long>(head) * vdim);
}

// A warp a (row, head): the parts' sums folded in order, then the combination and the head's norm.
template <typename T, int PL>
__global__ void __launch_bounds__(128)
diff_attention_merge_kernel(const float* __restrict__ partial, T* __restrict__ out, const int* __restrict__ request_of_row,
                            const int* __restrict__ cu_q, int rows, int heads, int vdim, int splits, int small_rows,
                            float lam, float out_scale, float eps, uint32_t* __restrict__ error) {
  wait_for_prior_kernels();
  launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long unit = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + warp;
  if (unit >= static_cast<long long>(rows) * heads) return;
  const int row = static_cast<int>(unit / heads);
  const int req = request_of_row[row];
  if (req < 0 || cu_q[req + 1] - cu_q[req] > small_rows) return;
  // the parts' maxima and sums first (a lane a part), then every part's factor, then the sums with all loads in flight
  const float* base = partial + unit * splits * (4 + 2 * vdim);
  float pm1 = -INFINITY, pm2 = -INFINITY, pl1 = 0.0f, pl2 = 0.0f;
  if (lane < splits) {
    const float* p = base + static_cast<long long>(lane) * (4 + 2 * vdim);
    pm1 = p[0]; pl1 = p[1]; pm2 = p[2]; pl2 = p[3];
  }
  const float m1 = warp_max(pm1), m2 = warp_max(pm2);
  const float f1 = pm1 == -INFINITY ? 0.0f : expf(pm1 - m1), f2 = pm2 == -INFINITY ? 0.0f : expf(pm2 - m2);
  float l1 = warp_sum(pl1 * f1), l2 = warp_sum(pl2 * f2);
  float a1[PL], a2[PL];
#pragma unroll
  for (int e = 0; e < PL; ++e) a1[e] = a2[e] = 0.0f;
#pragma unroll 4
  for (int s = 0; s < splits; ++s) {
    const float* p = base + static_cast<long long>(s) * (4 + 2 * vdim);
    const float d1 = __shfl_sync(0xffffffffu, f1, s), d2 = __shfl_sync(0xffffffffu, f2, s);
#pragma unroll
    for (int e = 0; e < PL; ++e)
      if (lane + 32 * e < vdim) {
        a1[e] = fmaf(p[4 + lane + 32 * e], d1, a1[e]);
        a2[e] = fmaf(p[4 + vdim + lane + 32 * e], d2, a2[e]);
      }
  }
  if (!(l1 > 0.0f) || !(l2 > 0.0f) || l1 > 3.0e38f || l2 > 3.0e38f) {
    if (lane == 0) publish_error(error, kAttentionDenominator);
    l1 = l2 = 1.0f;
  }
  diff_finish<T, PL>(a1, a2, l1, l2, lam, eps, out_scale, vdim, lane, out + unit * vdim);
}

// Tensor cores for requests of more than ``small_rows`` rows (bf16).  A block is 64 consecutive rows of one request and
// one head (found on the device from cu_q: block x of the grid is the x-th such tile of the step, blocks beyond the
// last leave); its eight warps are 16 rows x one MAP each (warps 0-3 the first map, 4-7 the second), so that the two
// softmax streams of a row run side by side.  Key tiles of 64 (both maps' keys and the values of the head's key/value
// head) come by cp.async into two buffers; columns beyond dim / vdim up to the instance's DIM / VDIM are zeros.  Per
// warp: S = Q K^T (32-bit), the running maximum and sum of a row in the exp2 domain, P as a bf16 pair (rounding,
// remainder) into O += P V.  At the end the second map's warps hand lambda O2 / l2 over through shared memory and the
// first map's form o = O1 / l1 - lambda O2 / l2, its norm over vdim, out_scale.
template <int DIM, int VDIM>
__global__ void __launch_bounds__(256, (DIM <= 64 ? 2 : 1))
diff_attention_tile_kernel(const __nv_bfloat16* __restrict__ qkv, long long ld, __nv_bfloat16* __restrict__ out,
                           const __nv_bfloat16* __restrict__ cache, const int* __restrict__ block_table, int table_width,
                           const int* __restrict__ cu_q, const int* __restrict__ q_start, int requests, int heads,
                           int kv_heads, int dim, int vdim, int page_size, int num_pages, float scale, float lam,
                           float out_scale, float eps, int window, int small_rows, uint32_t* __restrict__ error) {
  typedef __nv_bfloat16 bf16;
  constexpr int QLD = 2 * DIM + 8, VLD = VDIM + 8;           // row strides that keep ldmatrix free of bank conflicts
  constexpr int QC = 2 * DIM / 8, VC = VDIM / 8, PER = QC + VC;   // 16-byte pieces of a row of q or k, of v, of a key
  constexpr int XLD = VDIM + 4;                               // of the hand-over of the second map's sums (32-bit)
  static_assert(64 * XLD * 4 <= 2 * 64 * (QLD + VLD) * 2, "the hand-over fits the key and value buffers");
  extern __shared__ __align__(16) unsigned char diff_tile_smem[];
  bf16* Qs = reinterpret_cast<bf16*>(diff_tile_smem);         // [64][QLD]
  bf16* Ks = Qs + 64 * QLD;                                   // [2][64][QLD]
  bf16* Vs = Ks + 2 * 64 * QLD;                               // [2][64][VLD]
  __shared__ int tile_info[2];
  wait_for_prior_kernels();
  launch_dependents();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) {
    int t = blockIdx.x, found = -1, at = 0;
    for (int r = 0; r < requests; ++r) {
      const int n = cu_q[r + 1] - cu_q[r];
      if (n <= small_rows) continue;
      const int tiles = (n + 63) >> 6;
      if (t < tiles) { found = r; at = cu_q[r] + t * 64; break; }
      t -= tiles;
    }
    tile_info[0] = found;
    tile_info[1] = at;
  }
  __syncthreads();
  const int req = tile_info[0];
  if (req < 0) return;
  const int row0 = tile_info[1];
  const int nrows = min(64, cu_q[req + 1] - row0);
  const int pos0 = q_start[req] + (row0 - cu_q[req]);
  const int head = blockIdx.y, g = head / (heads / kv_heads);
  const long long width = static_cast<long long>(kv_heads) * (2 * dim + vdim);
  const int* table = block_table + static_cast<long long>(req) * table_width;
  const int key_last = pos0 + nrows - 1;
  const int key_first = window > 0 ? max(0, pos0 - window + 1) : 0;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

  for (int c = tid; c < 64 * QC; c += 256) {
    const int rr = c / QC, cc = c % QC, map = cc / (DIM / 8), col = (cc % (DIM / 8)) * 8;
    bf16* dst = Qs + rr * QLD + map * DIM + col;
    if (rr < nrows && col < dim)
      mma::copy_async_16(dst, qkv + (row0 + rr) * ld + static_cast<long long>(head) * 2 * dim + map * dim + col);
    else
      *reinterpret_cast<uint4*>(dst) = zero;
  }
  // four threads a key: the key's place in the cache is looked up once, its pieces are dealt round
  auto load_keys = [&](int buf, int j0) {
    const int key = tid >> 2, j = j0 + key;
    bf16* kb = Ks + (buf * 64 + key) * QLD;
    bf16* vb = Vs + (buf * 64 + key) * VLD;
    long long at = -1;
    if (j >= key_first && j <= key_last) {
      const int page = table[j / page_size];
      if (page < 0 || page >= num_pages) publish_error(error, kRowWithoutPage);
      else at = (static_cast<long long>(page) * page_size + j % page_size) * width;
    }
    const bf16* ksrc = cache + at + static_cast<long long>(g) * 2 * dim;
    const bf16* vsrc = cache + at + static_cast<long long>(kv_heads) * 2 * dim + static_cast<long long>(g) * vdim;
#pragma unroll
    for (int cc = (tid & 3); cc < PER; cc += 4) {
      if (cc < QC) {
        const int map = cc / (DIM / 8), col = (cc % (DIM / 8)) * 8;
        if (at >= 0 && col < dim) mma::copy_async_16(kb + map * DIM + col, ksrc + map * dim + col);
        else *reinterpret_cast<uint4*>(kb + map * DIM + col) = zero;
      } else {
        const int col = (cc - QC) * 8;
        if (at >= 0 && col < vdim) mma::copy_async_16(vb + col, vsrc + col);
        else *reinterpret_cast<uint4*>(vb + col) = zero;
      }
    }
    mma::copy_async_commit();
  };
  const int tile_lo = key_first >> 6, tile_hi = key_last >> 6;
  load_keys(0, tile_lo * 64);                                 // (the group also holds the copies of q)

  const int map = warp >> 2, wr0 = (warp & 3) * 16;
  const int ra = wr0 + (lane >> 2), rb = ra + 8;
  const int pos_a = ra < nrows ? pos0 + ra : -1, pos_b = rb < nrows ? pos0 + rb : -1;
  const int warp_first = pos0 + wr0, warp_last = pos0 + min(wr0 + 15, nrows - 1);
  const float to_exp2 = scale * 1.4426950408889634f;
  float O[VDIM / 8][4];
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;
#pragma unroll
  for (int n = 0; n < VDIM / 8; ++n) O[n][0] = O[n][1] = O[n][2] = O[n][3] = 0.0f;
  for (int it = tile_lo; it <= tile_hi; ++it) {
    const int buf = (it - tile_lo) & 1;
    if (it < tile_hi) {
      load_keys(buf ^ 1, (it + 1) * 64);
      mma::copy_async_wait<1>();
    } else {
      mma::copy_async_wait<0>();
    }
    __syncthreads();
    const int j0 = it * 64;
    if (wr0 < nrows && j0 <= warp_last) {
      const bf16* kb = Ks + buf * 64 * QLD + map * DIM;
      const bf16* vb = Vs + buf * 64 * VLD;
      float S[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) S[n][0] = S[n][1] = S[n][2] = S[n][3] = 0.0f;
#pragma unroll
      for (int kk = 0; kk < DIM / 16; ++kk) {
        uint32_t a[4];
        mma::load_matrices(a, Qs + (wr0 + (lane & 15)) * QLD + map * DIM + kk * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t b[4];
          mma::load_matrices(b, kb + (np * 16 + (lane >> 4) * 8 + (lane & 7)) * QLD + kk * 16 + ((lane >> 3) & 1) * 8);
          mma::multiply_add(S[2 * np], a, b[0], b[1]);
          mma::multiply_add(S[2 * np + 1], a, b[2], b[3]);
        }
      }
      // a tile that every row of the warp sees whole needs no mask
      const bool whole = j0 + 63 <= warp_first && (window <= 0 || j0 > warp_last - window);
      float top_a = -INFINITY, top_b = -INFINITY;
#pragma unroll
      for (int n = 0; n < 8; ++n) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int key = j0 + n * 8 + 2 * (lane & 3) + c;
          const bool see_a = whole || (key <= pos_a && (window <= 0 || key > pos_a - window));
          const bool see_b = whole || (key <= pos_b && (window <= 0 || key > pos_b - window));
          S[n][c] = see_a ? S[n][c] * to_exp2 : -INFINITY;
          S[n][2 + c] = see_b ? S[n][2 + c] * to_exp2 : -INFINITY;
          top_a = fmaxf(top_a, S[n][c]);
          top_b = fmaxf(top_b, S[n][2 + c]);
        }
      }
      top_a = fmaxf(top_a, __shfl_xor_sync(0xffffffffu, top_a, 1));
      top_a = fmaxf(top_a, __shfl_xor_sync(0xffffffffu, top_a, 2));
      top_b = fmaxf(top_b, __shfl_xor_sync(0xffffffffu, top_b, 1));
      top_b = fmaxf(top_b, __shfl_xor_sync(0xffffffffu, top_b, 2));
      const float new_a = fmaxf(m_a, top_a), new_b = fmaxf(m_b, top_b);
      const float ref_a = new_a == -INFINITY ? 0.0f : new_a, ref_b = new_b == -INFINITY ? 0.0f : new_b;
      const float fix_a = exp2f(m_a - ref_a), fix_b = exp2f(m_b - ref_b);
      m_a = new_a;
      m_b = new_b;
      float sum_a = 0.0f, sum_b = 0.0f;
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        S[n][0] = exp2f(S[n][0] - ref_a);
        S[n][1] = exp2f(S[n][1] - ref_a);
        S[n][2] = exp2f(S[n][2] - ref_b);
        S[n][3] = exp2f(S[n][3] - ref_b);
        sum_a += S[n][0] + S[n][1];
        sum_b += S[n][2] + S[n][3];
      }
      l_a = fmaf(l_a, fix_a, sum_a);
      l_b = fmaf(l_b, fix_b, sum_b);
#pragma unroll
      for (int n = 0; n < VDIM / 8; ++n) {
        O[n][0] *= fix_a;
        O[n][1] *= fix_a;
        O[n][2] *= fix_b;
        O[n][3] *= fix_b;
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {                        // 16 keys a step
        uint32_t hi[4], lo[4];
        hi[0] = mma::pack(S[2 * kk][0], S[2 * kk][1]);
        hi[1] = mma::pack(S[2 * kk][2], S[2 * kk][3]);
        hi[2] = mma::pack(S[2 * kk + 1][0], S[2 * kk + 1][1]);
        hi[3] = mma::pack(S[2 * kk + 1][2], S[2 * kk + 1][3]);
        lo[0] = mma::pack_remainder(S[2 * kk][0], S[2 * kk][1]);
        lo[1] = mma::pack_remainder(S[2 * kk][2], S[2 * kk][3]);
        lo[2] = mma::pack_remainder(S[2 * kk + 1][0], S[2 * kk + 1][1]);
        lo[3] = mma::pack_remainder(S[2 * kk + 1][2], S[2 * kk + 1][3]);
#pragma unroll
        for (int vp = 0; vp < VDIM / 16; ++vp) {
          uint32_t b[4];
          mma::load_matrices_transposed(b, vb + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * VLD + vp * 16 + (lane >> 4) * 8);
          mma::multiply_add(O[2 * vp], hi, b[0], b[1]);
          mma::multiply_add(O[2 * vp + 1], hi, b[2], b[3]);
          mma::multiply_add(O[2 * vp], lo, b[0], b[1]);
          mma::multiply_add(O[2 * vp + 1], lo, b[2], b[3]);
        }
      }
    }
    __syncthreads();
  }
  // the second map's warps hand lambda O2 / l2 over (the buffers are free: every warp is past the last barrier)
  float* X = reinterpret_cast<float*>(Ks);                    // [64][XLD], over the key and value buffers
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  const bool bad = (ra < nrows && (!(l_a > 0.0f) || l_a > 3.0e38f)) || (rb < nrows && (!(l_b > 0.0f) || l_b > 3.0e38f));
  if (bad) publish_error(error, kAttentionDenominator);
  const float i_a = l_a > 0.0f ? 1.0f / l_a : 0.0f, i_b = l_b > 0.0f ? 1.0f / l_b : 0.0f;
  if (map == 1) {
#pragma unroll
    for (int n = 0; n < VDIM / 8; ++n) {
      const int col = n * 8 + 2 * (lane & 3);
      *reinterpret_cast<float2*>(X + ra * XLD + col) = make_float2(lam * (O[n][0] * i_a), lam * (O[n][1] * i_a));
      *reinterpret_cast<float2*>(X + rb * XLD + col) = make_float2(lam * (O[n][2] * i_b), lam * (O[n][3] * i_b));
    }
  }
  __syncthreads();
  if (map == 1 || wr0 >= nrows) return;
  float ss_a = 0.0f, ss_b = 0.0f;
#pragma unroll
  for (int n = 0; n < VDIM / 8; ++n) {
    const int col = n * 8 + 2 * (lane & 3);
    const float2 xa = *reinterpret_cast<const float2*>(X + ra * XLD + col);
    const float2 xb = *reinterpret_cast<const float2*>(X + rb * XLD + col);
    O[n][0] = O[n][0] * i_a - xa.x;                           // (columns beyond vdim are zeros)
    O[n][1] = O[n][1] * i_a - xa.y;
    O[n][2] = O[n][2] * i_b - xb.x;
    O[n][3] = O[n][3] * i_b - xb.y;
    ss_a = fmaf(O[n][0], O[n][0], fmaf(O[n][1], O[n][1], ss_a));
    ss_b = fmaf(O[n][2], O[n][2], fmaf(O[n][3], O[n][3], ss_b));
  }
  ss_a += __shfl_xor_sync(0xffffffffu, ss_a, 1);
  ss_a += __shfl_xor_sync(0xffffffffu, ss_a, 2);
  ss_b += __shfl_xor_sync(0xffffffffu, ss_b, 1);
  ss_b += __shfl_xor_sync(0xffffffffu, ss_b, 2);
  const float inv_a = out_scale / sqrtf(ss_a / static_cast<float>(vdim) + eps);
  const float inv_b = out_scale / sqrtf(ss_b / static_cast<float>(vdim) + eps);
#pragma unroll
  for (int n = 0; n < VDIM / 8; ++n) {
    const int col = n * 8 + 2 * (lane & 3);
    if (col >= vdim) continue;                                // vdim is a multiple of 8: the pair is inside
    if (ra < nrows)
      *reinterpret_cast<__nv_bfloat162*>(out + (static_cast<long long>(row0 + ra) * heads + head) * vdim + col) =
          __floats2bfloat162_rn(O[n][0] * inv_a, O[n][1] * inv_a);
    if (rb < nrows)
      *reinterpret_cast<__nv_bfloat162*>(out + (static_cast<long long>(row0 + rb) * heads + head) * vdim + col) =
          __floats2bfloat162_rn(O[n][2] * inv_b, O[n][3] * inv_b);
  }
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
  if (dim > 2048) return PIH_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t smem = 4 * static_cast<size_t>(dim) * sizeof(float);
  const long long slots = static_cast<long long>(num_pages) * page_size;
  // few rows: a warp a map, side by side; many rows: a block a row
  const int units = 2 * heads + (write_kv ? 2 * kv_heads : 0);
  const unsigned units_y = rows <= 64 ? static_cast<unsigned>((units + 3) / 4) : 1u;
#define PIH_DQK(T)                                                                                                     \
  launch_kernel(diff_qk_prepare_kernel<T>, dim3(rows, units_y), dim3(128), smem, s, static_cast<T*>(qkv), ld,          \
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

template <int DIM, int VDIM>
static int launch_diff_tile(cudaStream_t s, unsigned tiles, const void* qkv, long long ld, void* out, const void* cache,
                            const void* block_table, int table_width, const void* cu_q, const void* q_start, int requests,
                            int heads, int kv_heads, int dim, int vdim, int page_size, int num_pages, float scale, float lam,
                            float out_scale, float eps, int window, int small_rows, void* error) {
  const size_t smem = (static_cast<size_t>(3) * 64 * (2 * DIM + 8) + 2 * 64 * (VDIM + 8)) * sizeof(bf16);
  static bool raised = false;
  if (!raised && smem > 48 * 1024) {
    cudaFuncSetAttribute(diff_attention_tile_kernel<DIM, VDIM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         static_cast<int>(smem));
    raised = true;
  }
  launch_kernel(diff_attention_tile_kernel<DIM, VDIM>, dim3(tiles, heads), dim3(256), smem, s, static_cast<const bf16*>(qkv),
                ld, static_cast<bf16*>(out), static_cast<const bf16*>(cache), static_cast<const int*>(block_table),
                table_width, static_cast<const int*>(cu_q), static_cast<const int*>(q_start), requests, heads, kv_heads, dim,
                vdim, page_size, num_pages, scale, lam, out_scale, eps, window, small_rows, static_cast<uint32_t*>(error));
  PIH_LAUNCH_CHECK();
  return 0;
}

// 1 when the tensor-core kernel has an instance for these sizes (bf16; dim and vdim multiples of 8 up to 128).
extern "C" int pih_diff_attention_tile_takes(int dim, int vdim) {
  return dim >= 8 && vdim >= 8 && dim % 8 == 0 && vdim % 8 == 0 && dim <= 128 && vdim <= 128;
}

// The attention of the step's rows.  ``tile`` (bf16 only, sizes that pih_diff_attention_tile_takes): requests of more
// than 16 rows run on the tensor-core kernel.  ``small``: the other rows (all rows without ``tile``) run on the warp
// kernel, their keys cut into ``splits`` parts (1: uncut, the row's result does not depend on the step's make-up by a
// bit) through ``partial`` (fp32 [rows, heads, splits, 4 + 2 vdim]).
extern "C" int pih_diff_attention(int dtype, const void* qkv, long long ld, void* out, const void* cache,
                                  const void* block_table, int table_width, const void* request_of_row,
                                  const void* positions, const void* cu_q, const void* q_start, int rows, int requests,
                                  int heads, int kv_heads, int dim, int vdim, int page_size, int num_pages, float scale,
                                  float lam, float out_scale, float eps, int window, int tile, int small, int splits,
                                  void* partial, void* error, void* stream) {
  if (rows <= 0) return 0;
  if (dim > 1024 || vdim > 32 * kDiffMaxPerLane || heads % kv_heads || splits < 1) return PIH_ERR_UNSUPPORTED;
  if (tile && (dtype != PIH_BF16 || !pih_diff_attention_tile_takes(dim, vdim) || ld % 8)) return PIH_ERR_UNSUPPORTED;
  if (splits > 32 || (splits > 1 && partial == nullptr)) return PIH_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int small_rows = tile ? 16 : 0x7fffffff;
  if (tile) {
    const unsigned tiles = static_cast<unsigned>((rows + 63) / 64 + requests);
    int rc;
#define PIH_TILE(D, V)                                                                                                 \
  rc = launch_diff_tile<D, V>(s, tiles, qkv, ld, out, cache, block_table, table_width, cu_q, q_start, requests, heads, \
                              kv_heads, dim, vdim, page_size, num_pages, scale, lam, out_scale, eps, window, small_rows, error)
    if (dim <= 32) { if (vdim <= 64) PIH_TILE(32, 64); else PIH_TILE(32, 128); }
    else if (dim <= 64) { if (vdim <= 64) PIH_TILE(64, 64); else PIH_TILE(64, 128); }
    else { if (vdim <= 64) PIH_TILE(128, 64); else PIH_TILE(128, 128); }
#undef PIH_TILE
    if (rc != 0) return rc;
  }
  if (!small) return 0;
  const long long units = static_cast<long long>(rows) * heads;
  const size_t smem = 4 * 2 * static_cast<size_t>(dim) * sizeof(float);
  const dim3 grid(static_cast<unsigned>((units + 3) / 4), splits);
#define PIH_DAG_PL(T, PL)                                                                                              \
  do {                                                                                                                 \
    launch_kernel(diff_attention_generic_kernel<T, PL>, grid, dim3(128), smem, s, static_cast<const T*>(qkv), ld,      \
                  static_cast<T*>(out), static_cast<const T*>(cache), static_cast<const int*>(block_table), table_width, \
                  static_cast<const int*>(request_of_row), static_cast<const int*>(positions),                         \
                  static_cast<const int*>(cu_q), rows, heads, kv_heads, dim, vdim, page_size, num_pages, scale, lam,   \
                  out_scale, eps, window, splits, small_rows, static_cast<float*>(partial), static_cast<uint32_t*>(error)); \
    PIH_LAUNCH_CHECK();                                                                                                \
    if (splits > 1)                                                                                                    \
      launch_kernel(diff_attention_merge_kernel<T, PL>, dim3(grid.x), dim3(128), 0, s,                                 \
                    static_cast<const float*>(partial), static_cast<T*>(out), static_cast<const int*>(request_of_row), \
                    static_cast<const int*>(cu_q), rows, heads, vdim, splits, small_rows, lam, out_scale, eps,         \
                    static_cast<uint32_t*>(error));                                                                    \
  } while (0)
#define PIH_DAG(T)                                                                                                     \
  do {                                                                                                                 \
    if (vdim <= 64) PIH_DAG_PL(T, 2);                                                                                  \
    else if (vdim <= 128) PIH_DAG_PL(T, 4);                                                                            \
    else if (vdim <= 256) PIH_DAG_PL(T, 8);                                                                            \
    else PIH_DAG_PL(T, 16);                                                                                            \
  } while (0)
  if (dtype == PIH_F32) PIH_DAG(float);
  else if (dtype == PIH_BF16) PIH_DAG(bf16);
  else return PIH_ERR_BAD_ARGUMENT;
#undef PIH_DAG_PL
#undef PIH_DAG
  PIH_LAUNCH_CHECK();
  return 0;
}
