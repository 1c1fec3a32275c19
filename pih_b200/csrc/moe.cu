// Mixture of experts: routing and the experts' products over rows grouped by expert.
//
//   moe_route      per row: the ``top`` largest router logits (32-bit), softmax over the chosen ones, and the row's
//                  place among the rows of each chosen expert
//   moe_plan       per expert: where its rows start, and where its row tiles start (one block)
//   moe_scatter    (row, choice) -> a position in expert order, and back
//   moe_gate_up    grouped product: act[pos] = silu(x[row] . Wg_e^T) * (x[row] . Wu_e^T)
//   moe_down       grouped product: y[pos] = act[pos] . Wd_e^T  (32-bit)
//   moe_combine    out[row] = sum_k weight[row][k] * y[pos(row, k)], k ascending
//
// Nothing returns to the host: a grouped product is launched for the most row tiles that the step could need
// (ceil(rows * top / 64) + experts), a block looks up its expert and rows in the plan, and blocks beyond the plan
// leave.  Every output element is accumulated by one thread in ascending k exactly as the single product does, and a
// row's result depends on that row alone: the rows an expert happens to share a tile with change no bit.
#include "common.cuh"

namespace pih {

constexpr int kMoeTile = 64;

// One warp a row.  A logit that is not a number counts as the smallest; ties go to the smaller index.
__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, int rows, int experts, int top, int* __restrict__ expert_of,
                 float* __restrict__ weight_of, int* __restrict__ rank_of, int* __restrict__ counts) {
  wait_for_prior_kernels();
  launch_dependents();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  constexpr int kPer = 32;                                       // experts <= 1024
  float v[kPer];
  uint32_t taken = 0;
#pragma unroll
  for (int e = 0; e < kPer; ++e) {
    const int i = lane + 32 * e;
    float a = (e * 32 < experts && i < experts) ? logits[static_cast<long long>(row) * experts + i] : -INFINITY;
    v[e] = (a == a) ? a : -INFINITY;
  }
  float first = 0.0f, denom = 0.0f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int best_i = 0x7fffffff;
#pragma unroll
    for (int e = 0; e < kPer; ++e) {
      const int i = lane + 32 * e;
      if (e * 32 < experts && i < experts && !((taken >> e) & 1u) && (v[e] > best || best_i == 0x7fffffff)) {
        best = v[e];
        best_i = i;
      }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, d);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, d);
      if (oi != 0x7fffffff && (best_i == 0x7fffffff || ob > best || (ob == best && oi < best_i))) { best = ob; best_i = oi; }
    }
    if ((best_i & 31) == lane) taken |= 1u << (best_i >> 5);
    if (k == 0) first = best;
    const float e_k = (best == -INFINITY) ? (first == -INFINITY ? 1.0f : 0.0f) : expf(best - first);
    denom += e_k;
    if (lane == 0) {
      expert_of[static_cast<long long>(row) * top + k] = best_i;
      weight_of[static_cast<long long>(row) * top + k] = e_k;
      rank_of[static_cast<long long>(row) * top + k] = atomicAdd(&counts[best_i], 1);
    }
  }
  __syncwarp();
  if (lane < top) {
    for (int k = lane; k < top; k += 32) weight_of[static_cast<long long>(row) * top + k] /= denom;
  }
}

// plan: [0 .. experts] first position of an expert's rows; [experts+1 .. 2 experts+1] first tile of an expert.
__global__ void moe_plan_kernel(const int* __restrict__ counts, int experts, int* __restrict__ plan) {
  wait_for_prior_kernels();
  launch_dependents();
  if (threadIdx.x != 0) return;
  int pos = 0, tile = 0;
  for (int e = 0; e < experts; ++e) {
    plan[e] = pos;
    plan[experts + 1 + e] = tile;
    pos += counts[e];
    tile += (counts[e] + kMoeTile - 1) / kMoeTile;
  }
  plan[experts] = pos;
  plan[2 * experts + 1] = tile;
}

__global__ void moe_scatter_kernel(const int* __restrict__ expert_of, const int* __restrict__ rank_of,
                                   const int* __restrict__ plan, int slots, int top, int* __restrict__ pos_of,
                                   int* __restrict__ row_of) {
  wait_for_prior_kernels();
  launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= slots) return;
  const int pos = plan[expert_of[i]] + rank_of[i];
  pos_of[i] = pos;
  row_of[pos] = i / top;
}

// The grouped product.  kGated: two weight matrices per expert and silu(a) * b in the epilogue.  A's rows are
// gathered through ``row_of`` when it is given (else row = position).  W: [experts, N, K] contiguous.
template <typename TA, typename TC, bool kGated>
__global__ void __launch_bounds__(256)
moe_grouped_kernel(const TA* __restrict__ A, long long lda, const int* __restrict__ row_of, const TA* __restrict__ W0,
                   const TA* __restrict__ W1, TC* __restrict__ C, long long ldc, const int* __restrict__ plan,
                   int experts, int N, int K) {
  constexpr int BM = kMoeTile, BN = 64, BK = 16, TM = 4, TN = 4;
  wait_for_prior_kernels();
  launch_dependents();
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[kGated ? 2 : 1][BK][BN + 4];
  __shared__ int rows_s[BM];
  __shared__ int info[3];
  const int tid = threadIdx.x;
  if (tid == 0) {
    const int tile = blockIdx.y;
    const int* tiles = plan + experts + 1;
    int e = -1;
    if (tile < tiles[experts]) {
      int lo = 0, hi = experts - 1;                              // the last expert whose first tile is <= tile and that has tiles
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (tiles[mid] <= tile) lo = mid; else hi = mid - 1;
      }
      e = lo;
    }
    info[0] = e;
    if (e >= 0) {
      info[1] = plan[e] + (tile - tiles[e]) * BM;                // first position of the tile
      info[2] = min(BM, plan[e + 1] - info[1]);                  // its rows
    }
  }
  __syncthreads();
  const int e = info[0];
  if (e < 0) return;
  const int p0 = info[1], m_rows = info[2];
  if (tid < BM) rows_s[tid] = tid < m_rows ? (row_of != nullptr ? row_of[p0 + tid] : p0 + tid) : -1;
  __syncthreads();
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  const int n0 = blockIdx.x * BN;
  const TA* w0 = W0 + static_cast<long long>(e) * N * K;
  const TA* w1 = kGated ? W1 + static_cast<long long>(e) * N * K : nullptr;
  float acc[kGated ? 2 : 1][TM][TN];
#pragma unroll
  for (int g = 0; g < (kGated ? 2 : 1); ++g)
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[g][i][j] = 0.0f;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int el = tid + i * 256;
      const int r = el / BK, c = el % BK;
      const int gk = k0 + c, gn = n0 + r;
      const int src = rows_s[r];
      As[c][r] = (src >= 0 && gk < K) ? to_float<TA>(A[static_cast<long long>(src) * lda + gk]) : 0.0f;
      Ws[0][c][r] = (gn < N && gk < K) ? to_float<TA>(w0[static_cast<long long>(gn) * K + gk]) : 0.0f;
      if (kGated) Ws[1][c][r] = (gn < N && gk < K) ? to_float<TA>(w1[static_cast<long long>(gn) * K + gk]) : 0.0f;
    }
    __syncthreads();
    float part[kGated ? 2 : 1][TM][TN];
#pragma unroll
    for (int g = 0; g < (kGated ? 2 : 1); ++g)
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) part[g][i][j] = 0.0f;
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
      for (int g = 0; g < (kGated ? 2 : 1); ++g) {
        float w[TN];
#pragma unroll
        for (int j = 0; j < TN; ++j) w[j] = Ws[g][k][tx * TN + j];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
          for (int j = 0; j < TN; ++j) part[g][i][j] = fmaf(a[i], w[j], part[g][i][j]);
      }
    }
#pragma unroll
    for (int g = 0; g < (kGated ? 2 : 1); ++g)
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[g][i][j] += part[g][i][j];
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = ty * TM + i;
    if (m >= m_rows) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn >= N) continue;
      float val;
      if (kGated) {
        // the two products are rounded to the storage type before the activation, as separate products would be
        const float a = round_to<TA>(acc[0][i][j]), b = round_to<TA>(acc[kGated ? 1 : 0][i][j]);
        val = (a / (1.0f + expf(-a))) * b;
      } else {
        val = acc[0][i][j];
      }
      C[static_cast<long long>(p0 + m) * ldc + gn] = from_float<TC>(val);
    }
  }
}

template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ pos_of,
                                   const float* __restrict__ weight_of, T* __restrict__ out, int rows, int hidden, int top) {
  wait_for_prior_kernels();
  launch_dependents();
  const int row = blockIdx.x;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float acc = 0.0f;
    for (int k = 0; k < top; ++k) {
      const long long i = static_cast<long long>(row) * top + k;
      acc = fmaf(weight_of[i], y[static_cast<long long>(pos_of[i]) * hidden + c], acc);
    }
    out[static_cast<long long>(row) * hidden + c] = from_float<T>(acc);
  }
}

}  // namespace pih

using namespace pih;
typedef __nv_bfloat16 bf16;

// ints: expert_of[slots] | rank_of[slots] | pos_of[slots] | row_of[slots] | counts[experts] | plan[2 experts + 2];
// the caller zeroes counts.  weight_of: fp32 [slots].
extern "C" long long pih_moe_route_words(int rows, int experts, int top) {
  return 4LL * rows * top + experts + 2LL * experts + 2;
}

extern "C" int pih_moe_route(const void* logits, int rows, int experts, int top, void* ints, void* weight_of, void* stream) {
  if (rows <= 0) return 0;
  if (experts < 1 || experts > 1024 || top < 1 || top > experts) return PIH_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long slots = static_cast<long long>(rows) * top;
  int* expert_of = static_cast<int*>(ints);
  int* rank_of = expert_of + slots;
  int* pos_of = rank_of + slots;
  int* row_of = pos_of + slots;
  int* counts = row_of + slots;
  int* plan = counts + experts;
  launch_kernel(moe_route_kernel, dim3((rows + 3) / 4), dim3(128), 0, s, static_cast<const float*>(logits), rows, experts,
                top, expert_of, static_cast<float*>(weight_of), rank_of, counts);
  PIH_LAUNCH_CHECK();
  launch_kernel(moe_plan_kernel, dim3(1), dim3(32), 0, s, static_cast<const int*>(counts), experts, plan);
  PIH_LAUNCH_CHECK();
  launch_kernel(moe_scatter_kernel, dim3(static_cast<unsigned>((slots + 255) / 256)), dim3(256), 0, s,
                static_cast<const int*>(expert_of), static_cast<const int*>(rank_of), static_cast<const int*>(plan),
                static_cast<int>(slots), top, pos_of, row_of);
  PIH_LAUNCH_CHECK();
  return 0;
}

// x [rows, lda]; w_gate, w_up [experts, ff, hidden]; w_down [experts, hidden, ff]; act [slots, ff] (storage type);
// y fp32 [slots, hidden]; out [rows, hidden] (storage type).
extern "C" int pih_moe_experts(int dtype, const void* x, long long lda, const void* w_gate, const void* w_up,
                               const void* w_down, void* act, void* y, void* out, const void* ints, const void* weight_of,
                               int rows, int experts, int top, int hidden, int ff, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long slots = static_cast<long long>(rows) * top;
  const int* expert_of = static_cast<const int*>(ints);
  const int* pos_of = expert_of + 2 * slots;
  const int* row_of = pos_of + slots;
  const int* plan = row_of + slots + experts;
  const unsigned tiles = static_cast<unsigned>((slots + kMoeTile - 1) / kMoeTile + experts);
  if (tiles > 65535) return PIH_ERR_UNSUPPORTED;
#define PIH_MOE(T)                                                                                                     \
  do {                                                                                                                 \
    launch_kernel(moe_grouped_kernel<T, T, true>, dim3((ff + 63) / 64, tiles), dim3(256), 0, s,                        \
                  static_cast<const T*>(x), lda, row_of, static_cast<const T*>(w_gate), static_cast<const T*>(w_up),   \
                  static_cast<T*>(act), static_cast<long long>(ff), plan, experts, ff, hidden);                        \
    PIH_LAUNCH_CHECK();                                                                                                \
    launch_kernel(moe_grouped_kernel<T, float, false>, dim3((hidden + 63) / 64, tiles), dim3(256), 0, s,               \
                  static_cast<const T*>(act), static_cast<long long>(ff), static_cast<const int*>(nullptr),            \
                  static_cast<const T*>(w_down), static_cast<const T*>(nullptr), static_cast<float*>(y),               \
                  static_cast<long long>(hidden), plan, experts, hidden, ff);                                          \
    PIH_LAUNCH_CHECK();                                                                                                \
    launch_kernel(moe_combine_kernel<T>, dim3(rows), dim3(hidden >= 256 ? 256 : 128), 0, s,                            \
                  static_cast<const float*>(y), pos_of, static_cast<const float*>(weight_of), static_cast<T*>(out),    \
                  rows, hidden, top);                                                                                  \
  } while (0)
  if (dtype == PIH_F32) PIH_MOE(float);
  else if (dtype == PIH_BF16) PIH_MOE(bf16);
  else return PIH_ERR_BAD_ARGUMENT;
#undef PIH_MOE
  PIH_LAUNCH_CHECK();
  return 0;
}
