// Latent attention, the step between the down-projections and what follows them: the query latent
// and the key/value latent of every token are RMS-normed (32-bit statistics, weight inside the single
// rounding); the query latent goes on as a matrix for the up-projection, the key/value latent goes to
// the token's place in its sequence's pages, where it serves as key and as value at once.
//
// Input: the 32-bit sums of the stacked down-projections, row stride ld, the query latent at column
// q_col, the key/value latent at column kv_col.  Page layout: [page][slot][kv_rank] (one "head").
#include "common.cuh"

namespace lb {

template <typename T>
__global__ void latent_norm_kernel(const float* __restrict__ pre, long long ld, int q_col, int kv_col, int q_rank,
                                   int kv_rank, const float* __restrict__ q_w, const float* __restrict__ kv_w,
                                   T* __restrict__ q_out, T* __restrict__ pages, const int* __restrict__ positions,
                                   const int* __restrict__ token_seq, const int* __restrict__ block_table,
                                   int page_size, int max_pages, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const bool is_q = blockIdx.y == 0;
  const int n = is_q ? q_rank : kv_rank;
  const float* src = pre + (size_t)t * ld + (is_q ? q_col : kv_col);
  const float* w = is_q ? q_w : kv_w;
  T* dst;
  if (is_q) {
    dst = q_out + (size_t)t * q_rank;
  } else {
    const int pos = positions[t];
    const int page = block_table[(size_t)token_seq[t] * max_pages + pos / page_size];
    if (page < 0) return;                                   // an entry that owns no page: uniform over the block
    dst = pages + ((size_t)page * page_size + pos % page_size) * kv_rank;
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) { const float v = src[i]; ss += v * v; }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) dst[i] = from_f32<T>(src[i] * inv * w[i]);
}

}  // namespace lb

LB_EXPORT int lb_latent_norm(int dtype, const float* pre, long long ld, int q_col, int kv_col, int q_rank, int kv_rank,
                             const float* q_w, const float* kv_w, void* q_out, void* pages, const int* positions,
                             const int* token_seq, const int* block_table, int num_tokens, int page_size, int max_pages,
                             float eps, cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(dtype), "latent_norm: bad dtype %d", dtype);
  LB_CHECK_ARG(num_tokens >= 0 && q_rank > 0 && kv_rank > 0 && page_size > 0 && max_pages > 0, "latent_norm: bad sizes");
  LB_CHECK_ARG(pre && q_w && kv_w && q_out && pages && positions && token_seq && block_table, "latent_norm: null argument");
  if (num_tokens == 0) return 0;
  const int widest = q_rank > kv_rank ? q_rank : kv_rank;
  const int threads = widest >= 1024 ? 256 : (widest >= 256 ? 128 : 64);
  LB_DISPATCH_DTYPE(dtype, T, {
    lb::launch(lb::latent_norm_kernel<T>, dim3(num_tokens, 2), dim3(threads), 0, stream, pre, ld, q_col, kv_col, q_rank,
               kv_rank, q_w, kv_w, (T*)q_out, (T*)pages, positions, token_seq, block_table, page_size, max_pages, eps);
  })
  LB_CHECK_LAUNCH("latent_norm");
  return 0;
}
