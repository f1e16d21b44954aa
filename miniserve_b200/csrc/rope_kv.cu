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
    int num_tokens, int nq, int nkv, int d, int rot, float eps, int page_shift, int num_pages, int* __restrict__ status) {
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
    MS_DEBUG_ONLY(if (page >= num_pages || row < 0) {
      if (lane == 0) atomicExch(status, 5);
      return;
    })
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

// bfloat16 fast path for head sizes 128 and 256 with the whole head rotated: one block per token,
// D/16 lanes per head. A lane holds 8 consecutive elements of the head's first half and the 8 of
// the second half that rotate with them (two 16-byte loads), so the rotation needs no exchange
// between lanes; only the sum of squares goes round the head's lanes. What depends on the token
// alone (position, page, cos/sin, norm weights) is fetched once per lane, and the loads of two
// passes over the heads are in flight together.
template <int D>
__global__ void __launch_bounds__(128)
qk_norm_rope_kv_bf16_token_kernel(
    __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool,
    const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ q_norm_w,
    const __nv_bfloat16* __restrict__ k_norm_w, const float* __restrict__ inv_freq, const float* __restrict__ cos_sin,
    const int* __restrict__ positions, const int* __restrict__ row_of_token, const int* __restrict__ page_indptr,
    const int* __restrict__ page_indices, int nq, int nkv, float eps, int page_shift, int num_pages, int* __restrict__ status) {
  constexpr int LPH = D / 16;     // lanes per head
  constexpr int HPW = 32 / LPH;   // heads per warp and pass
  constexpr int HALF = D / 2;
  constexpr int BATCH = 2;        // passes whose loads are issued together
  pdl_prologue();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int sub = lane % LPH, slot = lane / LPH, j0 = sub * 8;
  const int pos = positions[t];
  const bool has_kv = k_pool != nullptr;
  const int heads_total = nq + (has_kv ? 2 * nkv : 0);
  const __nv_bfloat16* row_in = qkv + (size_t)t * heads_total * D;
  // The page of the token hangs on a chain of three dependent loads; the first values of the
  // token are asked for before the chain is followed, so that both are in flight together.
  const int request = has_kv ? row_of_token[t] : 0;
  const int stride = nwarps * HPW;  // heads per pass of the block
  uint4 lo_raw[BATCH], hi_raw[BATCH];
  auto fetch = [&](int base) {
#pragma unroll
    for (int b = 0; b < BATCH; ++b) {
      const int h = min(base + warp * HPW + slot + b * stride, heads_total - 1);  // past the end: the last head again, unused
      const __nv_bfloat16* src = row_in + (size_t)h * D;
      lo_raw[b] = *reinterpret_cast<const uint4*>(src + j0);
      hi_raw[b] = *reinterpret_cast<const uint4*>(src + HALF + j0);
    }
  };
  fetch(0);
  float cs[8], sn[8];
  if (inv_freq == nullptr) {
#pragma unroll
    for (int i = 0; i < 8; ++i) { cs[i] = 1.f; sn[i] = 0.f; }
  } else if (cos_sin) {
    const float4* c4 = reinterpret_cast<const float4*>(cos_sin + (size_t)t * D + j0);
    const float4* s4 = reinterpret_cast<const float4*>(cos_sin + (size_t)t * D + HALF + j0);
    const float4 a = c4[0], b = c4[1], c = s4[0], d4 = s4[1];
    cs[0] = a.x; cs[1] = a.y; cs[2] = a.z; cs[3] = a.w; cs[4] = b.x; cs[5] = b.y; cs[6] = b.z; cs[7] = b.w;
    sn[0] = c.x; sn[1] = c.y; sn[2] = c.z; sn[3] = c.w; sn[4] = d4.x; sn[5] = d4.y; sn[6] = d4.z; sn[7] = d4.w;
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) sincosf((float)pos * inv_freq[j0 + i], &sn[i], &cs[i]);
  }
  // the norm weights of this lane's elements, the same for every head of a kind
  const bool normed = q_norm_w != nullptr;
  uint4 wq_lo = make_uint4(0u, 0u, 0u, 0u), wq_hi = wq_lo, wk_lo = wq_lo, wk_hi = wq_lo;
  if (normed) {
    wq_lo = *reinterpret_cast<const uint4*>(q_norm_w + j0);
    wq_hi = *reinterpret_cast<const uint4*>(q_norm_w + HALF + j0);
    if (has_kv) {
      wk_lo = *reinterpret_cast<const uint4*>(k_norm_w + j0);
      wk_hi = *reinterpret_cast<const uint4*>(k_norm_w + HALF + j0);
    }
  }
  size_t slot_base = 0;
  if (has_kv) {
    const int page = page_indices[page_indptr[request] + (pos >> page_shift)];
    if (page < 0) {
      if (threadIdx.x == 0) atomicExch(status, 2);
      return;
    }
    MS_DEBUG_ONLY(if (page >= num_pages || request < 0) {
      if (threadIdx.x == 0) atomicExch(status, 5);
      return;
    })
    const int page_size = 1 << page_shift;
    slot_base = ((size_t)page * nkv * page_size + (pos & (page_size - 1))) * D;  // + kvh * page_size * D
  }
  for (int base = 0; base < heads_total; base += BATCH * stride) {  // the same trips for every lane: they exchange sums
    const int h0 = base + warp * HPW + slot;
    if (base > 0) fetch(base);
#pragma unroll
    for (int b = 0; b < BATCH; ++b) {
      const int h = h0 + b * stride;
      const bool live = h < heads_total;
      const bool is_v = h >= nq + nkv, is_q = h < nq;
      float lo[8], hi[8];
      bf16x8_to_float(lo_raw[b], lo);
      bf16x8_to_float(hi_raw[b], hi);
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += lo[i] * lo[i] + hi[i] * hi[i];
      // every lane takes part in the exchange, also those past the last head
#pragma unroll
      for (int off = LPH / 2; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
      uint4 out_lo = lo_raw[b], out_hi = hi_raw[b];  // a value head is stored as it came
      if (!is_v) {
        float wl[8], wh[8];
        float inv = 1.f;
        if (normed) {
          inv = 1.0f / sqrtf(ss / (float)D + eps);
          bf16x8_to_float(is_q ? wq_lo : wk_lo, wl);
          bf16x8_to_float(is_q ? wq_hi : wk_hi, wh);
        }
        float ol[8], oh[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float l = normed ? (lo[i] * inv) * wl[i] : lo[i];
          const float hgh = normed ? (hi[i] * inv) * wh[i] : hi[i];
          ol[i] = l * cs[i] - hgh * sn[i];
          oh[i] = hgh * cs[i] + l * sn[i];
        }
        out_lo = float_to_bf16x8(ol);
        out_hi = float_to_bf16x8(oh);
      }
      if (live) {
        __nv_bfloat16* dst = is_q ? q_out + ((size_t)t * nq + h) * D
                                  : (is_v ? v_pool + slot_base + ((size_t)(h - nq - nkv) << page_shift) * D
                                          : k_pool + slot_base + ((size_t)(h - nq) << page_shift) * D);
        *reinterpret_cast<uint4*>(dst + j0) = out_lo;
        *reinterpret_cast<uint4*>(dst + HALF + j0) = out_hi;
      }
    }
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

// The same table laid out for a reader that walks 128 tokens at a time, eight rotation pairs at a time (the
// q|k|v product's epilogue in gemm_tc.cu fetches such a piece with one bulk copy):
// tiled[tile of 128 tokens][eighth of the 64 pairs][cos, sin][token within the tile][pair within the eighth].
// Tokens beyond the last one (the last tile's unused rows) are left as they are.
__global__ void rope_table_tile_kernel(float* __restrict__ tiled, const float* __restrict__ table, int num_tokens) {
  pdl_prologue();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)num_tokens * 128) return;
  const int t = (int)(idx >> 7), col = (int)(idx & 127);
  const int is_sin = col >> 6, pair = col & 63;
  tiled[((((size_t)(t >> 7) * 8 + (pair >> 3)) * 2 + is_sin) * 128 + (t & 127)) * 8 + (pair & 7)] = table[idx];
}

}  // namespace ms

using namespace ms;

// table: float32 [T, 128] (64 cosines then 64 sines per token); tiled: float32 [ceil(T / 128), 8, 2, 128, 8]
MS_EXPORT int ms_rope_table_tile(float* tiled, const float* table, int num_tokens, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  const long long items = (long long)num_tokens * 128;
  MS_LAUNCH(rope_table_tile_kernel, (unsigned)((items + 255) / 256), 256, 0, stream, tiled, table, num_tokens);
  return 0;
}

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
                                 int page_size, int num_pages, int* status, int dtype, cudaStream_t stream) {
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
  if (dtype == MS_BF16 && head_dim % 128 == 0 && head_dim <= 256 && (rotary_dim == head_dim || inv_freq == nullptr) &&
      (k_pool == nullptr || (q_norm_w != nullptr) == (k_norm_w != nullptr)) && ((uintptr_t)qkv % 16 == 0) &&
      ((uintptr_t)q_out % 16 == 0) && ((uintptr_t)k_pool % 16 == 0) && ((uintptr_t)v_pool % 16 == 0) &&
      ((uintptr_t)q_norm_w % 16 == 0) && ((uintptr_t)k_norm_w % 16 == 0) && (cos_sin == nullptr || (uintptr_t)cos_sin % 16 == 0)) {
    if (head_dim == 128)
      MS_LAUNCH(qk_norm_rope_kv_bf16_token_kernel<128>, num_tokens, 128, 0, stream, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool,
                (__nv_bfloat16*)v_pool, (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)q_norm_w, (const __nv_bfloat16*)k_norm_w,
                inv_freq, inv_freq ? cos_sin : (const float*)nullptr, positions, row_of_token, page_indptr, page_indices, nq, nkv,
                eps, page_shift, num_pages, status);
    else
      MS_LAUNCH(qk_norm_rope_kv_bf16_token_kernel<256>, num_tokens, 128, 0, stream, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool,
                (__nv_bfloat16*)v_pool, (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)q_norm_w, (const __nv_bfloat16*)k_norm_w,
                inv_freq, inv_freq ? cos_sin : (const float*)nullptr, positions, row_of_token, page_indptr, page_indices, nq, nkv,
                eps, page_shift, num_pages, status);
    return 0;
  }
  if (dtype == MS_F32)
    MS_LAUNCH(qk_norm_rope_kv_kernel<float>, blocks, warps * 32, 0, stream,
        (float*)q_out, (float*)k_pool, (float*)v_pool, (const float*)qkv, (const float*)q_norm_w, (const float*)k_norm_w,
        inv_freq, cos_sin, positions, row_of_token, page_indptr, page_indices, num_tokens, nq, nkv, head_dim, rotary_dim, eps,
        page_shift, num_pages, status);
  else
    MS_LAUNCH(qk_norm_rope_kv_kernel<__nv_bfloat16>, blocks, warps * 32, 0, stream,
        (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, (const __nv_bfloat16*)qkv,
        (const __nv_bfloat16*)q_norm_w, (const __nv_bfloat16*)k_norm_w, inv_freq, cos_sin, positions, row_of_token, page_indptr,
        page_indices, num_tokens, nq, nkv, head_dim, rotary_dim, eps, page_shift, num_pages, status);
  return 0;
}
