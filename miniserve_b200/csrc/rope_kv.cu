// Per-head RMSNorm of q and k, rotate-half position encoding, and the write of the new keys
// and values into the paged cache, in one pass over the fused q|k|v projection output.
//
// Formulas: miniserve/model/qwen3.py:118-123 (q/k norm over head_dim with the model's eps,
// before the rotation; rotate_half(x) = cat(-x[d/2:], x[:d/2]); out = x*cos + rotate_half(x)*sin),
// :98-108 (angle = float(position) * inv_freq[j], inv_freq in float32), and
// miniserve/cache/kv_pool.py:46-50 (new k after norm and rotation, and v as projected, stored at
// the token's slot before attention runs). The cosine and sine are taken in float32 and the
// result is rounded once.
//
// Cache layout (ours): K and V pools are [pages, kv_heads, page_size, head_dim] per cache entry,
// so that one page of one kv head is a contiguous tile.
#include "common.cuh"

namespace ms {

template <typename T>
__global__ void qk_norm_rope_kv_kernel(
    T* __restrict__ q_out,            // [T, nq, d]
    T* __restrict__ k_pool,           // [pages, nkv, page_size, d] (may be null: this entry reads another's cache)
    T* __restrict__ v_pool,
    const T* __restrict__ qkv,        // [T, (nq + 2*nkv) * d]  (or [T, nq*d] when k_pool is null)
    const T* __restrict__ q_norm_w,   // [d] or null (no q/k norm)
    const T* __restrict__ k_norm_w,
    const float* __restrict__ inv_freq,  // [rot/2] or null (no rotation)
    const float* __restrict__ cos_sin,   // [T, rot]: cos then sin of every (token, pair), or null (computed here)
    const int* __restrict__ positions, const int* __restrict__ row_of_token,
    const int* __restrict__ page_indptr, const int* __restrict__ page_indices,
    int num_tokens, int nq, int nkv, int d, int rot, float eps, int page_shift, int* __restrict__ status) {
  pdl_prologue();
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int heads_total = nq + (k_pool ? 2 * nkv : 0);
  const long long item = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  if (item >= (long long)num_tokens * heads_total) return;
  const int t = (int)(item / heads_total);
  const int h = (int)(item - (long long)t * heads_total);
  const int row_width = heads_total * d;
  const T* src = qkv + (size_t)t * row_width + (size_t)h * d;
  const int pos = positions[t];

  T* dst;
  const T* nw = nullptr;
  bool rotate = inv_freq != nullptr;
  if (h < nq) {
    dst = q_out + ((size_t)t * nq + h) * d;
    nw = q_norm_w;
  } else {
    const int kvh = (h - nq) % nkv;
    const bool is_v = (h - nq) >= nkv;
    const int row = row_of_token[t];
    const int page_size = 1 << page_shift;
    const int page = page_indices[page_indptr[row] + (pos >> page_shift)];
    if (page < 0) {  // a page the window has already given back, or a table that is too short
      if (lane == 0) atomicExch(status, 2);
      return;
    }
    T* pool = is_v ? v_pool : k_pool;
    dst = pool + (((size_t)page * nkv + kvh) * page_size + (pos & (page_size - 1))) * d;
    if (is_v) {
      for (int c = lane; c < d; c += 32) dst[c] = src[c];
      return;
    }
    nw = k_norm_w;
  }

  // sum of squares over the head, lanes in a fixed tree
  float inv = 1.f;
  if (nw) {
    float ss = 0.f;
    for (int c = lane; c < d; c += 32) {
      const float x = Elem<T>::load(src + c);
      ss += x * x;
    }
    ss = warp_sum(ss);
    inv = 1.0f / sqrtf(ss / (float)d + eps);
  }
  const int half = rot >> 1;
  for (int j = lane; j < half; j += 32) {
    float lo = Elem<T>::load(src + j), hi = Elem<T>::load(src + j + half);
    if (nw) {
      lo = (lo * inv) * Elem<T>::load(nw + j);
      hi = (hi * inv) * Elem<T>::load(nw + j + half);
    }
    if (rotate) {
      float sn, cs;
      if (cos_sin) {
        cs = cos_sin[(size_t)t * rot + j];
        sn = cos_sin[(size_t)t * rot + half + j];
      } else {
        sincosf((float)pos * inv_freq[j], &sn, &cs);
      }
      const float olo = lo * cs - hi * sn;
      const float ohi = hi * cs + lo * sn;
      lo = olo;
      hi = ohi;
    }
    Elem<T>::store(dst + j, lo);
    Elem<T>::store(dst + j + half, hi);
  }
  // dimensions beyond the rotated part (rot < d) pass through normalised
  for (int c = rot + lane; c < d; c += 32) {
    float x = Elem<T>::load(src + c);
    if (nw) x = (x * inv) * Elem<T>::load(nw + c);
    Elem<T>::store(dst + c, x);
  }
}

// cos and sin of every (token, rotation pair) of a step: table[t, j] = cos(pos_t * inv_freq_j),
// table[t, rot/2 + j] = sin(...). Made once per step and read by every layer's q/k kernel.
__global__ void rope_table_kernel(float* __restrict__ table, const int* __restrict__ positions,
                                  const float* __restrict__ inv_freq, int num_tokens, int rot) {
  pdl_prologue();
  const int half = rot >> 1;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)num_tokens * half) return;
  const int t = (int)(idx / half), j = (int)(idx - (long long)t * half);
  float sn, cs;
  sincosf((float)positions[t] * inv_freq[j], &sn, &cs);
  table[(size_t)t * rot + j] = cs;
  table[(size_t)t * rot + half + j] = sn;
}

}  // namespace ms

using namespace ms;

MS_EXPORT int ms_rope_table(float* table, const int* positions, const float* inv_freq, int num_tokens, int rotary_dim,
                            cudaStream_t stream) {
  if (num_tokens == 0 || rotary_dim == 0) return 0;
  MS_CHECK_ARG(rotary_dim > 0 && rotary_dim % 2 == 0, "rope_table: rotary_dim=%d must be even", rotary_dim);
  const long long items = (long long)num_tokens * (rotary_dim / 2);
  MS_LAUNCH(rope_table_kernel, (unsigned)((items + 255) / 256), 256, 0, stream, table, positions, inv_freq, num_tokens,
            rotary_dim);
  return 0;
}

MS_EXPORT int ms_qk_norm_rope_kv(void* q_out, void* k_pool, void* v_pool, const void* qkv, const void* q_norm_w,
                                 const void* k_norm_w, const float* inv_freq, const float* cos_sin, const int* positions,
                                 const int* row_of_token, const int* page_indptr, const int* page_indices,
                                 int num_tokens, int nq, int nkv, int head_dim, int rotary_dim, float eps,
                                 int page_size, int* status, int dtype, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  MS_CHECK_ARG(nq > 0 && nkv > 0 && head_dim > 0, "qk_norm_rope_kv: bad sizes nq=%d nkv=%d d=%d", nq, nkv, head_dim);
  MS_CHECK_ARG(rotary_dim >= 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0,
               "qk_norm_rope_kv: rotary_dim=%d must be even and at most head_dim=%d", rotary_dim, head_dim);
  MS_CHECK_ARG(page_size > 0 && (page_size & (page_size - 1)) == 0, "qk_norm_rope_kv: page_size=%d must be a power of two", page_size);
  MS_CHECK_ARG((k_pool == nullptr) == (v_pool == nullptr), "qk_norm_rope_kv: give both pools or neither");
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  const long long items = (long long)num_tokens * (nq + (k_pool ? 2 * nkv : 0));
  const int warps = 8;
  const unsigned blocks = (unsigned)((items + warps - 1) / warps);
  if (dtype == MS_F32)
    MS_LAUNCH(qk_norm_rope_kv_kernel<float>, blocks, warps * 32, 0, stream,
        (float*)q_out, (float*)k_pool, (float*)v_pool, (const float*)qkv, (const float*)q_norm_w, (const float*)k_norm_w,
        inv_freq, cos_sin, positions, row_of_token, page_indptr, page_indices, num_tokens, nq, nkv, head_dim, rotary_dim, eps,
        page_shift, status);
  else
    MS_LAUNCH(qk_norm_rope_kv_kernel<__nv_bfloat16>, blocks, warps * 32, 0, stream,
        (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, (const __nv_bfloat16*)qkv,
        (const __nv_bfloat16*)q_norm_w, (const __nv_bfloat16*)k_norm_w, inv_freq, cos_sin, positions, row_of_token, page_indptr,
        page_indices, num_tokens, nq, nkv, head_dim, rotary_dim, eps, page_shift, status);
  return 0;
}
