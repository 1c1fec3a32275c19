// Retention: linear attention with a fixed decay a head and a matrix state per (request, head).
//
//   retention_prepare      q and k of every row rotated by the row's position (angles formed in 32-bit from the
//                          frequencies), k then scaled: 32-bit copies [rows, heads, dim]
//   retention_recurrence   per token  S <- S + (decay - 1) S + k v^T,  o = S^T q,  from the request's state slot; S in
//                          shared memory (any key size), or in registers for the key sizes that have an instance
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

// The same recurrence with S in registers, for the key sizes that have an instance.  Block (request, head, 32 value
// columns); a column of S is held by kParts threads (thread (column c = tid / kParts, part p = tid % kParts) the rows
// p * kDim / kParts ...), so the parts of a column sit in neighbouring lanes and meet through shuffles.  What the
// recurrence reads of a token (k, q, the block's 32 values) is staged in shared memory a chunk of tokens at a time, two
// buffers: the next chunk's numbers are copied asynchronously while this chunk is computed, so no load from memory
// and only one barrier a chunk lie on the chain from token to token.  The order of the additions is fixed by the
// kernel, not by the step's make-up or by where a chunk begins.
__device__ __forceinline__ void retention_copy_16(void* smem_dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))), "l"(src));
}

template <typename T, int kDim>
__global__ void __launch_bounds__(kDim >= 64 ? 256 : (kDim >= 32 ? 128 : 64))
retention_recurrence_reg_kernel(const float* __restrict__ qf, const float* __restrict__ kf, const T* __restrict__ v,
                                long long ldv, const float* __restrict__ decay_m1, float* __restrict__ out,
                                float* __restrict__ state, long long state_stride, const int* __restrict__ cu_q,
                                const int* __restrict__ state_slots, int heads, int vdim) {
  constexpr int kParts = kDim >= 64 ? 8 : (kDim >= 32 ? 4 : 2);   // threads a column of S
  constexpr int kThreads = 32 * kParts;
  constexpr int kRows = kDim / kParts;                    // rows of S a thread holds (a multiple of 4)
  constexpr int kSeg = kRows + 4;                         // a part's stretch of k (or q) in the staging buffer: the parts'
                                                          // 16-byte reads fall into different banks
  constexpr int kChunk = kDim <= 128 ? 16 : 8;            // tokens staged at a time
  constexpr int kVWords = 32 * sizeof(T) / 4;             // the block's 32 values of a token, in 32-bit words
  constexpr int kTok = 2 * kParts * kSeg + kVWords;       // words staged a token: k | q | values
  constexpr int kCopies = 2 * (kDim / 4) + kVWords / 4;   // 16-byte copies a token
  extern __shared__ __align__(16) float stage[];          // [2][kChunk][kTok]
  wait_for_prior_kernels();
  launch_dependents();
  const int r = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * 32;
  const int lo = cu_q[r], hi = cu_q[r + 1];
  const int slot = state_slots[r];
  if (hi <= lo || slot < 0) return;
  const int tid = threadIdx.x, c = tid / kParts, p = tid % kParts;
  float* Sg = state + slot * state_stride + (static_cast<long long>(h) * kDim + p * kRows) * vdim + col0 + c;
  float S[kRows];
#pragma unroll
  for (int i = 0; i < kRows; ++i) S[i] = Sg[static_cast<long long>(i) * vdim];
  const float dm1 = decay_m1[h];
  auto fetch = [&](int buf, int t0) {
    const int n = min(kChunk, hi - t0);
    for (int e = tid; e < n * kCopies; e += kThreads) {
      const int tok = e / kCopies, piece = e % kCopies;
      float* dst = stage + (buf * kChunk + tok) * kTok;
      const long long t = t0 + tok;
      if (piece < 2 * (kDim / 4)) {
        const int which = piece / (kDim / 4), at = (piece % (kDim / 4)) * 4;       // k or q; the element
        const float* src = (which == 0 ? kf : qf) + (t * heads + h) * kDim + at;
        retention_copy_16(dst + which * kParts * kSeg + (at / kRows) * kSeg + at % kRows, src);
      } else {
        const int w = piece - 2 * (kDim / 4);
        retention_copy_16(dst + 2 * kParts * kSeg + w * 4,
                          reinterpret_cast<const float*>(v + t * ldv + static_cast<long long>(h) * vdim + col0) + w * 4);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  fetch(0, lo);
  int buf = 0;
  for (int t0 = lo; t0 < hi; t0 += kChunk, buf ^= 1) {
    if (t0 + kChunk < hi) {
      fetch(buf ^ 1, t0 + kChunk);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const int n = min(kChunk, hi - t0);
#pragma unroll 4                                           // (a token's shuffles and store run under the next tokens' FMAs)
    for (int tok = 0; tok < n; ++tok) {
      const float* cur = stage + (buf * kChunk + tok) * kTok;
      const float4* k4 = reinterpret_cast<const float4*>(cur + p * kSeg);
      const float4* q4 = reinterpret_cast<const float4*>(cur + kParts * kSeg + p * kSeg);
      const float vj = to_float<T>(reinterpret_cast<const T*>(cur + 2 * kParts * kSeg)[c]);
      float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
#pragma unroll
      for (int i = 0; i < kRows / 4; ++i) {
        const float4 k = k4[i], q = q4[i];
        S[4 * i + 0] = fmaf(k.x, vj, fmaf(dm1, S[4 * i + 0], S[4 * i + 0]));
        S[4 * i + 1] = fmaf(k.y, vj, fmaf(dm1, S[4 * i + 1], S[4 * i + 1]));
        S[4 * i + 2] = fmaf(k.z, vj, fmaf(dm1, S[4 * i + 2], S[4 * i + 2]));
        S[4 * i + 3] = fmaf(k.w, vj, fmaf(dm1, S[4 * i + 3], S[4 * i + 3]));
        o0 = fmaf(S[4 * i + 0], q.x, o0);
        o1 = fmaf(S[4 * i + 1], q.y, o1);
        o2 = fmaf(S[4 * i + 2], q.z, o2);
        o3 = fmaf(S[4 * i + 3], q.w, o3);
      }
      float o = (o0 + o1) + (o2 + o3);
#pragma unroll
      for (int d = 1; d < kParts; d <<= 1) o += __shfl_xor_sync(0xffffffffu, o, d);
      if (p == 0) out[((static_cast<long long>(t0) + tok) * heads + h) * vdim + col0 + c] = o;
    }
    __syncthreads();                                       // the buffer is free for the chunk after the next
  }
#pragma unroll
  for (int i = 0; i < kRows; ++i) Sg[static_cast<long long>(i) * vdim] = S[i];
}

}  // namespace pih

using namespace pih;
typedef __nv_bfloat16 bf16;

template <typename T, int D>
static void launch_retention_in_registers(cudaStream_t s, const float* qf, const float* kf, const void* v, long long ldv,
                                          const void* decay_m1, void* out, void* state, long long state_stride,
                                          const void* cu_q, const void* state_slots, int requests, int heads, int vdim) {
  constexpr int parts = D >= 64 ? 8 : (D >= 32 ? 4 : 2);
  constexpr int chunk = D <= 128 ? 16 : 8;
  constexpr size_t needed = 2 * chunk * (2 * parts * (D / parts + 4) + 32 * sizeof(T) / 4) * sizeof(float);
  // The token loop is bound by the SM's shared-memory reads: two blocks on one SM each run at half speed.  With fewer
  // blocks than SMs, every block asks for more than half of an SM's shared memory and so gets an SM alone.
  const bool alone = static_cast<long long>(requests) * heads * (vdim / 32) <= 148;
  const size_t bytes = alone && needed < 116 * 1024 ? 116 * 1024 : needed;
  if (bytes > 48 * 1024)
    cudaFuncSetAttribute(retention_recurrence_reg_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         static_cast<int>(bytes));
  launch_kernel(retention_recurrence_reg_kernel<T, D>, dim3(requests, heads, vdim / 32), dim3(32 * parts), bytes, s, qf, kf,
                static_cast<const T*>(v), ldv, static_cast<const float*>(decay_m1), static_cast<float*>(out),
                static_cast<float*>(state), state_stride, static_cast<const int*>(cu_q),
                static_cast<const int*>(state_slots), heads, vdim);
}

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
  // S in registers: the key sizes with an instance, value columns in whole slabs of 32, and everything that is copied
  // in 16-byte pieces on a 16-byte boundary
  const size_t esize = dtype == PIH_F32 ? 4 : 2;
  const bool in_registers = (dim == 16 || dim == 32 || dim == 64 || dim == 128 || dim == 256) && vdim % 32 == 0 &&
                            (reinterpret_cast<uintptr_t>(v) % 16 == 0) && (ldv * esize) % 16 == 0 &&
                            (vdim * esize) % 16 == 0 && (reinterpret_cast<uintptr_t>(scratch) % 16 == 0);
#define PIH_RET_ARGS s, qf, kf, v, ldv, decay_m1, out, state, state_stride, cu_q, state_slots, requests, heads, vdim
#define PIH_RET(T)                                                                                                     \
  do {                                                                                                                 \
    launch_kernel(retention_prepare_kernel<T>, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, s,          \
                  static_cast<const T*>(qk), ld, static_cast<const float*>(freq), static_cast<const int*>(positions),  \
                  qf, kf, rows, heads, dim, rot, key_scale);                                                           \
    PIH_LAUNCH_CHECK();                                                                                                \
    if (in_registers) {                                                                                                \
      switch (dim) {                                                                                                   \
        case 16: launch_retention_in_registers<T, 16>(PIH_RET_ARGS); break;                                           \
        case 32: launch_retention_in_registers<T, 32>(PIH_RET_ARGS); break;                                           \
        case 64: launch_retention_in_registers<T, 64>(PIH_RET_ARGS); break;                                           \
        case 128: launch_retention_in_registers<T, 128>(PIH_RET_ARGS); break;                                         \
        default: launch_retention_in_registers<T, 256>(PIH_RET_ARGS); break;                                          \
      }                                                                                                                \
      break;                                                                                                           \
    }                                                                                                                  \
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
#undef PIH_RET_ARGS
  PIH_LAUNCH_CHECK();
  return 0;
}
