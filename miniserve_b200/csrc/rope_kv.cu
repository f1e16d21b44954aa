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

// bfloat16 fast path for head sizes that are multiples of 64 with the whole head rotated: one
// block per token, every warp takes a share of the heads, two adjacent elements per lane. What
// depends on the token alone (position, page, cos/sin, norm weights) is fetched once per warp.
template <int PER_LANE>
__global__ void __launch_bounds__(128)
qk_norm_rope_kv_bf16_token_kernel(
    __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool,
    const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ q_norm_w,
    const __nv_bfloat16* __restrict__ k_norm_w, const float* __restrict__ inv_freq, const float* __restrict__ cos_sin,
    const int* __restrict__ positions, const int* __restrict__ row_of_token, const int* __restrict__ page_indptr,
    const int* __restrict__ page_indices, int nq, int nkv, int d, float eps, int page_shift, int* __restrict__ status) {
  pdl_prologue();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int half = d >> 1;
  constexpr int per_lane = PER_LANE;  // iterations of 64 pairs (2 per lane): head size 128 or 256
  const int pos = positions[t];
  const bool has_kv = k_pool != nullptr;
  const int heads_total = nq + (has_kv ? 2 * nkv : 0);
  const __nv_bfloat16* row_in = qkv + (size_t)t * heads_total * d;
  size_t slot_base = 0;
  if (has_kv) {
    const int page = page_indices[page_indptr[row_of_token[t]] + (pos >> page_shift)];
    if (page < 0) {
      if (threadIdx.x == 0) atomicExch(status, 2);
      return;
    }
    const int page_size = 1 << page_shift;
    slot_base = ((size_t)page * nkv * page_size + (pos & (page_size - 1))) * d;  // + kvh * page_size * d
  }
  // per-lane constants: cos/sin of its two pairs per iteration (at most 2 iterations: d <= 256)
  float cs[per_lane][2], sn[per_lane][2];
#pragma unroll
  for (int it = 0; it < per_lane; ++it) {
    const int j = it * 64 + 2 * lane;
    if (inv_freq == nullptr) {
      cs[it][0] = cs[it][1] = 1.f;
      sn[it][0] = sn[it][1] = 0.f;
    } else if (cos_sin) {
      const float2 c = *reinterpret_cast<const float2*>(cos_sin + (size_t)t * d + j);
      const float2 s2 = *reinterpret_cast<const float2*>(cos_sin + (size_t)t * d + half + j);
      cs[it][0] = c.x; cs[it][1] = c.y; sn[it][0] = s2.x; sn[it][1] = s2.y;
    } else {
      sincosf((float)pos * inv_freq[j], &sn[it][0], &cs[it][0]);
      sincosf((float)pos * inv_freq[j + 1], &sn[it][1], &cs[it][1]);
    }
  }
  // the norm weights of this lane's elements, the same for every head of a kind
  __nv_bfloat162 wq[per_lane][2], wk[per_lane][2];
  const bool normed = q_norm_w != nullptr;
#pragma unroll
  for (int it = 0; it < per_lane; ++it) {
    if (!normed) continue;
    const int j = it * 64 + 2 * lane;
    wq[it][0] = *reinterpret_cast<const __nv_bfloat162*>(q_norm_w + j);
    wq[it][1] = *reinterpret_cast<const __nv_bfloat162*>(q_norm_w + half + j);
    if (has_kv) {
      wk[it][0] = *reinterpret_cast<const __nv_bfloat162*>(k_norm_w + j);
      wk[it][1] = *reinterpret_cast<const __nv_bfloat162*>(k_norm_w + half + j);
    }
  }
  // Heads in batches of four per warp: all loads of a batch are issued before the first is
  // used, so that a warp keeps several cache lines in flight instead of one head's two.
  constexpr int HB = 4;
  for (int h0 = warp; h0 < heads_total; h0 += HB * nwarps) {
    __nv_bfloat162 raw[HB][per_lane][2];
#pragma unroll
    for (int b = 0; b < HB; ++b) {
      const int h = min(h0 + b * nwarps, heads_total - 1);  // past the end: the last head again, unused
      const __nv_bfloat16* src = row_in + (size_t)h * d;
#pragma unroll
      for (int it = 0; it < per_lane; ++it) {
        const int j = it * 64 + 2 * lane;
        raw[b][it][0] = *reinterpret_cast<const __nv_bfloat162*>(src + j);
        raw[b][it][1] = *reinterpret_cast<const __nv_bfloat162*>(src + half + j);
      }
    }
#pragma unroll
    for (int b = 0; b < HB; ++b) {
      const int h = h0 + b * nwarps;
      if (h >= heads_total) continue;
      if (h >= nq + nkv) {  // a value head: copied as it is
        __nv_bfloat16* dst = v_pool + slot_base + ((size_t)(h - nq - nkv) << page_shift) * d;
#pragma unroll
        for (int it = 0; it < per_lane; ++it) {
          const int j = it * 64 + 2 * lane;
          *reinterpret_cast<__nv_bfloat162*>(dst + j) = raw[b][it][0];
          *reinterpret_cast<__nv_bfloat162*>(dst + half + j) = raw[b][it][1];
        }
        continue;
      }
      const bool is_q = h < nq;
      __nv_bfloat16* dst = is_q ? q_out + ((size_t)t * nq + h) * d : k_pool + slot_base + ((size_t)(h - nq) << page_shift) * d;
      float lo[per_lane][2], hi[per_lane][2];
      float ss = 0.f;
#pragma unroll
      for (int it = 0; it < per_lane; ++it) {
        const float2 a = __bfloat1622float2(raw[b][it][0]);
        const float2 c = __bfloat1622float2(raw[b][it][1]);
        lo[it][0] = a.x; lo[it][1] = a.y; hi[it][0] = c.x; hi[it][1] = c.y;
        ss += a.x * a.x + a.y * a.y + c.x * c.x + c.y * c.y;
      }
      float inv = 1.f;
      if (normed) {
        ss = warp_sum(ss);
        inv = 1.0f / sqrtf(ss / (float)d + eps);
      }
#pragma unroll
      for (int it = 0; it < per_lane; ++it) {
        const int j = it * 64 + 2 * lane;
        float wl[2] = {1.f, 1.f}, wh[2] = {1.f, 1.f};
        if (normed) {
          const float2 a = __bfloat1622float2(is_q ? wq[it][0] : wk[it][0]);
          const float2 c = __bfloat1622float2(is_q ? wq[it][1] : wk[it][1]);
          wl[0] = a.x; wl[1] = a.y; wh[0] = c.x; wh[1] = c.y;
        }
        float ol[2], oh[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float l = normed ? (lo[it][e] * inv) * wl[e] : lo[it][e];
          const float hgh = normed ? (hi[it][e] * inv) * wh[e] : hi[it][e];
          ol[e] = l * cs[it][e] - hgh * sn[it][e];
          oh[e] = hgh * cs[it][e] + l * sn[it][e];
        }
        *reinterpret_cast<__nv_bfloat162*>(dst + j) = __floats2bfloat162_rn(ol[0], ol[1]);
        *reinterpret_cast<__nv_bfloat162*>(dst + half + j) = __floats2bfloat162_rn(oh[0], oh[1]);
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
  if (dtype == MS_BF16 && head_dim % 128 == 0 && head_dim <= 256 && (rotary_dim == head_dim || inv_freq == nullptr) &&
      (k_pool == nullptr || (q_norm_w != nullptr) == (k_norm_w != nullptr)) && ((uintptr_t)qkv % 8 == 0) &&
      ((uintptr_t)q_out % 8 == 0) && ((uintptr_t)k_pool % 8 == 0) && ((uintptr_t)v_pool % 8 == 0) &&
      (cos_sin == nullptr || (uintptr_t)cos_sin % 8 == 0)) {
    if (head_dim == 128)
      MS_LAUNCH(qk_norm_rope_kv_bf16_token_kernel<1>, num_tokens, 128, 0, stream, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool,
                (__nv_bfloat16*)v_pool, (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)q_norm_w, (const __nv_bfloat16*)k_norm_w,
                inv_freq, inv_freq ? cos_sin : (const float*)nullptr, positions, row_of_token, page_indptr, page_indices, nq, nkv,
                head_dim, eps, page_shift, status);
    else
      MS_LAUNCH(qk_norm_rope_kv_bf16_token_kernel<2>, num_tokens, 128, 0, stream, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool,
                (__nv_bfloat16*)v_pool, (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)q_norm_w, (const __nv_bfloat16*)k_norm_w,
                inv_freq, inv_freq ? cos_sin : (const float*)nullptr, positions, row_of_token, page_indptr, page_indices, nq, nkv,
                head_dim, eps, page_shift, status);
    return 0;
  }
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
