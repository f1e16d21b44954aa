// Row-wise causal attention over the paged cache: one warp per (new token, query head).
//
// This is the attention of the true float32 path (and the fallback for head sizes the
// tensor-core kernels do not take). Its arithmetic for one (token, head) is a fixed sequence of
// float32 operations that depends only on that query, the keys and values of its own request and
// their absolute positions: keys are taken in tiles of 32 aligned to absolute position, each
// lane owns one key of the tile, scores are a sequential dot product, the tile's maximum and sum
// go through a fixed lane tree, and the running (max, sum, output) are updated tile by tile.
// So the result is the same bit for bit whether the token came in a whole prompt, in a portion,
// alone as a decode token, or beside other requests.
//
// Formula: softmax(q k^T * d^-0.5 + causal mask) v with query head h reading kv head
// h / (heads / kv_heads) (miniserve/model/attention.py:60-67, miniserve/model/qwen3.py:133-135);
// a query at absolute position p sees keys 0..p of its request, or p-window+1..p with a window.
#include <cfloat>

#include "common.cuh"

namespace ms {

constexpr int ROWWISE_MAX_D = 256;

template <typename T>
__global__ void __launch_bounds__(128)
attention_rowwise_kernel(T* __restrict__ out,            // [T, nq, d]
                         const T* __restrict__ q,        // [T, nq, d]
                         const T* __restrict__ k_pool,   // [pages, nkv, page_size, d]
                         const T* __restrict__ v_pool,
                         const int* __restrict__ positions, const int* __restrict__ row_of_token,
                         const int* __restrict__ page_indptr, const int* __restrict__ page_indices,
                         int num_tokens, int nq, int nkv, int d, float scale, int window, int page_shift,
                         int num_pages, int* __restrict__ status) {
  extern __shared__ float q_smem[];  // [warps][d]
  pdl_prologue();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (item >= (long long)num_tokens * nq) return;
  const int t = (int)(item / nq), h = (int)(item - (long long)t * nq);
  const int kvh = h / (nq / nkv);
  const int qpos = positions[t];
  const int row = row_of_token[t];
  const int* pages = page_indices + page_indptr[row];
  const int page_size = 1 << page_shift;
  const int lo = window > 0 ? max(0, qpos - window + 1) : 0;

  float* qs = q_smem + warp * d;
  const T* qsrc = q + ((size_t)t * nq + h) * d;
  for (int c = lane; c < d; c += 32) qs[c] = Elem<T>::load(qsrc + c);
  __syncwarp();

  float m = -INFINITY, l = 0.f;
  float acc[ROWWISE_MAX_D / 32];
#pragma unroll
  for (int i = 0; i < ROWWISE_MAX_D / 32; ++i) acc[i] = 0.f;

  for (int tile = (lo >> 5) << 5; tile <= qpos; tile += 32) {
    const int kj = tile + lane;
    const bool valid = kj >= lo && kj <= qpos;
    float s = -INFINITY;
    size_t base = 0;
    if (valid) {
      const int page = pages[kj >> page_shift];
      bool usable = page >= 0;
      if (!usable) atomicExch(status, 3);
      MS_DEBUG_ONLY(if (usable && (page >= num_pages || row < 0)) {
        atomicExch(status, 5);
        usable = false;
      })
      if (usable) {
        base = (((size_t)page * nkv + kvh) * page_size + (kj & (page_size - 1))) * d;
        const T* kr = k_pool + base;
        float dot = 0.f;
        for (int c = 0; c < d; ++c) dot = fmaf(qs[c], Elem<T>::load(kr + c), dot);
        s = dot * scale;
      }
    }
    const float m_tile = warp_max(s);
    const float m_new = fmaxf(m, m_tile);
    const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
    const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int i = 0; i < ROWWISE_MAX_D / 32; ++i) acc[i] *= alpha;
    const int j_lo = max(lo - tile, 0), j_hi = min(qpos - tile, 31);
    for (int j = j_lo; j <= j_hi; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const unsigned long long bj = __shfl_sync(0xffffffffu, (unsigned long long)base, j);
      const T* vr = v_pool + bj;
#pragma unroll
      for (int i = 0; i < ROWWISE_MAX_D / 32; ++i) {
        const int c = lane + 32 * i;
        if (c < d) acc[i] = fmaf(pj, Elem<T>::load(vr + c), acc[i]);
      }
    }
    m = m_new;
  }
  T* o = out + ((size_t)t * nq + h) * d;
#pragma unroll
  for (int i = 0; i < ROWWISE_MAX_D / 32; ++i) {
    const int c = lane + 32 * i;
    if (c < d) Elem<T>::store(o + c, acc[i] / l);
  }
}

}  // namespace ms

using namespace ms;

MS_EXPORT int ms_attention_rowwise(void* out, const void* q, const void* k_pool, const void* v_pool,
                                   const int* positions, const int* row_of_token, const int* page_indptr,
                                   const int* page_indices, int num_tokens, int nq, int nkv, int head_dim, float scale,
                                   int window, int page_size, int num_pages, int* status, int dtype, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  MS_CHECK_ARG(nq > 0 && nkv > 0 && nq % nkv == 0, "attention: %d query heads are not a multiple of %d kv heads", nq, nkv);
  MS_CHECK_ARG(head_dim > 0 && head_dim <= ROWWISE_MAX_D, "attention: head_dim=%d is outside 1..%d", head_dim, ROWWISE_MAX_D);
  MS_CHECK_ARG(page_size > 0 && (page_size & (page_size - 1)) == 0, "attention: page_size=%d must be a power of two", page_size);
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  const int warps = 4;
  const long long items = (long long)num_tokens * nq;
  const unsigned blocks = (unsigned)((items + warps - 1) / warps);
  const size_t smem = (size_t)warps * head_dim * sizeof(float);
  if (dtype == MS_F32)
    MS_LAUNCH(attention_rowwise_kernel<float>, blocks, warps * 32, smem, stream,
        (float*)out, (const float*)q, (const float*)k_pool, (const float*)v_pool, positions, row_of_token, page_indptr,
        page_indices, num_tokens, nq, nkv, head_dim, scale, window, page_shift, num_pages, status);
  else
    MS_LAUNCH(attention_rowwise_kernel<__nv_bfloat16>, blocks, warps * 32, smem, stream,
        (__nv_bfloat16*)out, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool,
        positions, row_of_token, page_indptr, page_indices, num_tokens, nq, nkv, head_dim, scale, window, page_shift,
        num_pages, status);
  return 0;
}
