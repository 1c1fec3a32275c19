// Attention over a cached latent: every token caches ONE vector c of ``rank`` numbers, and a head's key and value
// are products of c with that head's matrices.  Because both are linear in c, the head's key matrix is folded into
// the query (q' = W_k^T q, ``rank`` numbers) and its value matrix is applied after the weighted sum of latents:
//
//   score_j = (q' . c_j) * scale        o' = sum_j p_j c_j        head output = W_v o'
//
// so the kernels here see one shared "key = value = c_j" for all heads (the folded products are batched matrix
// products outside).  The softmax denominator may hold a sink: a learned logit per head that has no key and no value;
// it is the state the running softmax starts from (maximum = sink, sum = 1, accumulator = 0).  A sigmoid gate per
// (row, head) may scale the output.  Scores, weights and sums are 32-bit; keys are visited in ascending position, so a
// row's result does not depend on how its prompt was cut or batched.
//
//   latent_write              c = rmsnorm(raw latent) * w  ->  the paged cache [pages, page_size, rank]
//   latent_attention_generic  one warp a (row, head), any rank up to 512, float or bf16 storage
#include "common.cuh"

namespace pih {

template <typename T>
__global__ void __launch_bounds__(128)
latent_write_kernel(const T* __restrict__ raw, long long ld, const float* __restrict__ weight, float eps,
                    T* __restrict__ cache, const int* __restrict__ slot_mapping, int rows, int rank, long long cache_rows,
                    uint32_t* err) {
  wait_for_prior_kernels();
  launch_dependents();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int slot = slot_mapping[row];
  if (slot == kPaddingSlot) return;
  if (slot < 0 || slot >= cache_rows) {
    if (lane == 0) publish_error(err, kRowWithoutPage);
    return;
  }
  const T* src = raw + static_cast<long long>(row) * ld;
  float ss = 0.0f;
  for (int i = lane; i < rank; i += 32) { const float a = to_float<T>(src[i]); ss = fmaf(a, a, ss); }
  ss = warp_sum(ss);
  const float scale = 1.0f / sqrtf(ss / static_cast<float>(rank) + eps);
  T* dst = cache + static_cast<long long>(slot) * rank;
  for (int i = lane; i < rank; i += 32) dst[i] = from_float<T>(to_float<T>(src[i]) * scale * weight[i]);
}

constexpr int kLatentPerLane = 16;          // rank <= 32 * 16

// q: [rows, heads, rank] (the folded queries); gate: [rows, ldg] logits, column h, or null; sink: fp32 [heads] or null.
template <typename T, int kPerLane>
__global__ void __launch_bounds__(128)
latent_attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ gate, long long ldg,
                                const float* __restrict__ sink, const T* __restrict__ cache,
                                const int* __restrict__ block_table, int table_width, const int* __restrict__ request_of_row,
                                const int* __restrict__ positions, T* __restrict__ out, int rows, int heads, int rank,
                                int page_size, int num_pages, float scale, int window, uint32_t* err) {
  wait_for_prior_kernels();
  launch_dependents();
  const long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= static_cast<long long>(rows) * heads) return;
  const int lane = threadIdx.x & 31;
  const int row = static_cast<int>(item / heads), h = static_cast<int>(item % heads);
  const int req = request_of_row[row];
  if (req < 0) return;                                           // a row of padding
  const int pos = positions[row];
  float qr[kPerLane], acc[kPerLane];
#pragma unroll
  for (int e = 0; e < kPerLane; ++e) {
    const int i = lane + 32 * e;
    qr[e] = i < rank ? to_float<T>(q[item * rank + i]) : 0.0f;
    acc[e] = 0.0f;
  }
  float m = sink != nullptr ? sink[h] : -INFINITY;
  float l = sink != nullptr ? 1.0f : 0.0f;
  const int first = window > 0 ? max(0, pos - window + 1) : 0;
  const int* table = block_table + static_cast<long long>(req) * table_width;
  bool bad = false;
  for (int j = first; j <= pos; ++j) {
    const int pi = j / page_size;
    const int page = pi < table_width ? table[pi] : -1;
    if (page < 0 || page >= num_pages) { bad = true; continue; }
    const T* c = cache + (static_cast<long long>(page) * page_size + (j - pi * page_size)) * rank;
    float cr[kPerLane];
    float s = 0.0f;
#pragma unroll
    for (int e = 0; e < kPerLane; ++e) {
      const int i = lane + 32 * e;
      cr[e] = (e * 32 < rank && i < rank) ? to_float<T>(c[i]) : 0.0f;
      s = fmaf(qr[e], cr[e], s);
    }
    s = warp_sum(s) * scale;
    const float m_new = fmaxf(m, s);
    const float corr = expf(m - m_new);                          // exp(-inf) = 0 at the first key without a sink
    const float p = expf(s - m_new);
    l = fmaf(l, corr, p);
#pragma unroll
    for (int e = 0; e < kPerLane; ++e) acc[e] = fmaf(acc[e], corr, p * cr[e]);
    m = m_new;
  }
  if (bad && lane == 0) publish_error(err, kRowWithoutPage);
  if (!(l > 0.0f) || !isfinite(l)) {
    if (lane == 0) publish_error(err, kAttentionDenominator);
    l = 1.0f;
  }
  float factor = 1.0f / l;
  if (gate != nullptr) {
    const float z = to_float<T>(gate[static_cast<long long>(row) * ldg + h]);
    factor *= 1.0f / (1.0f + expf(-z));
  }
#pragma unroll
  for (int e = 0; e < kPerLane; ++e) {
    const int i = lane + 32 * e;
    if (i < rank) out[item * rank + i] = from_float<T>(acc[e] * factor);
  }
}

}  // namespace pih

using namespace pih;
typedef __nv_bfloat16 bf16;

extern "C" int pih_latent_write(int dtype, const void* raw, long long ld, const void* weight, float eps, void* cache,
                                const void* slot_mapping, int rows, int rank, int page_size, int num_pages, void* err,
                                void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long cache_rows = static_cast<long long>(page_size) * num_pages;
#define PIH_LW(T)                                                                                                      \
  launch_kernel(latent_write_kernel<T>, dim3((rows + 3) / 4), dim3(128), 0, s, static_cast<const T*>(raw), ld,         \
                static_cast<const float*>(weight), eps, static_cast<T*>(cache), static_cast<const int*>(slot_mapping), \
                rows, rank, cache_rows, static_cast<uint32_t*>(err))
  if (dtype == PIH_F32) PIH_LW(float);
  else if (dtype == PIH_BF16) PIH_LW(bf16);
  else return PIH_ERR_BAD_ARGUMENT;
#undef PIH_LW
  PIH_LAUNCH_CHECK();
  return 0;
}

extern "C" int pih_latent_attention_generic(int dtype, const void* q, const void* gate, long long ldg, const void* sink,
                                            const void* cache, const void* block_table, int table_width,
                                            const void* request_of_row, const void* positions, void* out, int rows,
                                            int heads, int rank, int page_size, int num_pages, float scale, int window,
                                            void* err, void* stream) {
  if (rows <= 0) return 0;
  if (rank > 32 * kLatentPerLane) return PIH_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long items = static_cast<long long>(rows) * heads;
  dim3 grid(static_cast<unsigned>((items + 3) / 4));
#define PIH_LA1(T, NE)                                                                                                 \
  launch_kernel(latent_attention_generic_kernel<T, NE>, grid, dim3(128), 0, s, static_cast<const T*>(q),                   \
                static_cast<const T*>(gate), ldg, static_cast<const float*>(sink), static_cast<const T*>(cache),       \
                static_cast<const int*>(block_table), table_width, static_cast<const int*>(request_of_row),            \
                static_cast<const int*>(positions), static_cast<T*>(out), rows, heads, rank, page_size, num_pages,     \
                scale, window, static_cast<uint32_t*>(err))
#define PIH_LA(T)                                                                                                      \
  do {                                                                                                                 \
    if (rank <= 64) PIH_LA1(T, 2);                                                                                     \
    else if (rank <= 128) PIH_LA1(T, 4);                                                                               \
    else if (rank <= 256) PIH_LA1(T, 8);                                                                               \
    else PIH_LA1(T, 16);                                                                                               \
  } while (0)
  if (dtype == PIH_F32) PIH_LA(float);
  else if (dtype == PIH_BF16) PIH_LA(bf16);
  else return PIH_ERR_BAD_ARGUMENT;
#undef PIH_LA
#undef PIH_LA1
  PIH_LAUNCH_CHECK();
  return 0;
}
