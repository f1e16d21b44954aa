// Embedding gather, RMSNorm (with the residual add and an optional row gather fused in),
// and SiLU-and-multiply. One templated kernel each for float32 and bfloat16 activations;
// the residual stream is float32 in both modes and every statistic is computed in float32.
//
// Formulas follow miniserve/model/qwen3.py:78-82 (RMSNorm: x * rsqrt(mean(x^2) + eps), then
// times the weight), :211 (embedding), :128-131 (SiLU(gate) * up) and the fused operator list
// of miniserve/model/fused.py:160-211 (residual add + norm in one pass).
#include "common.cuh"

namespace ms {

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embed_gather_kernel(float* __restrict__ residual, const T* __restrict__ table,
                                    const int* __restrict__ ids, int hidden, int vocab) {
  pdl_prologue();
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);  // ids are validated on the host; stay in bounds anyway
  const T* src = table + (size_t)id * hidden;
  float* dst = residual + (size_t)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = Elem<T>::load(src + i);
}

// bfloat16 rows that are a multiple of 8 wide: eight elements per thread (a 16-byte load, two 16-byte stores)
__global__ void embed_gather_bf16x8_kernel(float* __restrict__ residual, const __nv_bfloat16* __restrict__ table,
                                           const int* __restrict__ ids, int hidden8, int vocab, int tokens) {
  pdl_prologue();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)tokens * hidden8) return;
  const int t = (int)(idx / hidden8), c = (int)(idx - (long long)t * hidden8);
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  float v[8];
  bf16x8_to_float(reinterpret_cast<const uint4*>(table + (size_t)id * hidden8 * 8)[c], v);
  float4* dst = reinterpret_cast<float4*>(residual + (size_t)t * hidden8 * 8) + 2 * c;
  dst[0] = make_float4(v[0], v[1], v[2], v[3]);
  dst[1] = make_float4(v[4], v[5], v[6], v[7]);
}

// ---------------------------------------------------------------- (add +) RMSNorm (+ gather)
// For output row i: r = rows ? rows[i] : i.
//   h = residual[r] (+ delta[r] if delta)            float32
//   if (write_residual) residual[r] = h              (only without a gather)
//   out[i] = h / sqrt(mean(h^2) + eps) * w           rounded once to T
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS)
add_rmsnorm_kernel(T* __restrict__ out, float* __restrict__ residual, const T* __restrict__ delta,
                   const T* __restrict__ w, const int* __restrict__ rows, float eps, int hidden,
                   int write_residual) {
  extern __shared__ float row_buf[];  // hidden floats
  __shared__ float red[32];
  pdl_prologue();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* res = residual + (size_t)r * hidden;
  const T* dl = delta ? delta + (size_t)r * hidden : nullptr;
  float ss = 0.f;
  for (int c = threadIdx.x; c < hidden; c += THREADS) {
    float h = res[c];
    if (dl) h += Elem<T>::load(dl + c);
    row_buf[c] = h;
    ss += h * h;
  }
  const float total = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
  T* o = out + (size_t)i * hidden;
  for (int c = threadIdx.x; c < hidden; c += THREADS) {
    const float h = row_buf[c];
    if (write_residual && dl) res[c] = h;
    Elem<T>::store(o + c, (h * inv) * Elem<T>::load(w + c));
  }
}

// The same for bfloat16 activations whose rows are a multiple of 8 wide: eight elements per thread
// and trip (two 16-byte loads of the residual, one of the addend), the sum kept in registers when
// a row is at most 8 * THREADS wide, else in shared memory.
template <int THREADS>
__global__ void __launch_bounds__(THREADS)
add_rmsnorm_bf16x8_kernel(__nv_bfloat16* __restrict__ out, float* __restrict__ residual,
                          const __nv_bfloat16* __restrict__ delta, const __nv_bfloat16* __restrict__ w,
                          const int* __restrict__ rows, float eps, int hidden, int write_residual) {
  extern __shared__ float row_buf[];  // hidden floats, used only by rows wider than 8 * THREADS
  __shared__ float red[32];
  pdl_prologue();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* res = residual + (size_t)r * hidden;
  const __nv_bfloat16* dl = delta ? delta + (size_t)r * hidden : nullptr;
  const int chunks = hidden >> 3;
  const bool in_regs = chunks <= THREADS;
  float h[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  float ss = 0.f;
  for (int c = threadIdx.x; c < chunks; c += THREADS) {
    const float4 a = *reinterpret_cast<const float4*>(res + 8 * c), b = *reinterpret_cast<const float4*>(res + 8 * c + 4);
    h[0] = a.x; h[1] = a.y; h[2] = a.z; h[3] = a.w; h[4] = b.x; h[5] = b.y; h[6] = b.z; h[7] = b.w;
    if (dl) {
      float d[8];
      bf16x8_to_float(*reinterpret_cast<const uint4*>(dl + 8 * c), d);
#pragma unroll
      for (int e = 0; e < 8; ++e) h[e] += d[e];
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += h[e] * h[e];
    if (!in_regs) {
      *reinterpret_cast<float4*>(row_buf + 8 * c) = make_float4(h[0], h[1], h[2], h[3]);
      *reinterpret_cast<float4*>(row_buf + 8 * c + 4) = make_float4(h[4], h[5], h[6], h[7]);
    }
  }
  const float total = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
  __nv_bfloat16* o = out + (size_t)i * hidden;
  const bool store_sum = write_residual && dl;
  float* sum_to = res;
  for (int c = threadIdx.x; c < chunks; c += THREADS) {
    if (!in_regs) {
      const float4 a = *reinterpret_cast<const float4*>(row_buf + 8 * c), b = *reinterpret_cast<const float4*>(row_buf + 8 * c + 4);
      h[0] = a.x; h[1] = a.y; h[2] = a.z; h[3] = a.w; h[4] = b.x; h[5] = b.y; h[6] = b.z; h[7] = b.w;
    }
    if (store_sum) {
      *reinterpret_cast<float4*>(sum_to + 8 * c) = make_float4(h[0], h[1], h[2], h[3]);
      *reinterpret_cast<float4*>(sum_to + 8 * c + 4) = make_float4(h[4], h[5], h[6], h[7]);
    }
    float wv[8], y[8];
    bf16x8_to_float(*reinterpret_cast<const uint4*>(w + 8 * c), wv);
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = (h[e] * inv) * wv[e];
    *reinterpret_cast<uint4*>(o + 8 * c) = float_to_bf16x8(y);
  }
}

// ---------------------------------------------------------------- SiLU(gate) * up
template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int inter, size_t total) {
  pdl_prologue();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / inter;
  const int c = (int)(idx - t * inter);
  const float g = Elem<T>::load(gate_up + t * 2 * inter + c);
  const float u = Elem<T>::load(gate_up + t * 2 * inter + inter + c);
  const float s = g / (1.0f + expf(-g));
  Elem<T>::store(out + idx, s * u);
}

// bfloat16, 8 elements per thread (inter % 8 == 0)
__global__ void silu_mul_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gate_up,
                                       int inter8, size_t total8) {
  pdl_prologue();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total8) return;
  const size_t t = idx / inter8;
  const int c = (int)(idx - t * inter8);
  const uint4 gv = reinterpret_cast<const uint4*>(gate_up)[t * 2 * inter8 + c];
  const uint4 uv = reinterpret_cast<const uint4*>(gate_up)[t * 2 * inter8 + inter8 + c];
  const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
  const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
  uint4 ov;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 g = __bfloat1622float2(g2[k]);
    const float2 u = __bfloat1622float2(u2[k]);
    float2 r;
    r.x = g.x / (1.0f + expf(-g.x)) * u.x;
    r.y = g.y / (1.0f + expf(-g.y)) * u.y;
    o2[k] = __float22bfloat162_rn(r);
  }
  reinterpret_cast<uint4*>(out)[idx] = ov;
}

// ---------------------------------------------------------------- float32 <- T copy (logits of a bf16 GEMM)
template <typename T>
__global__ void to_float_kernel(float* __restrict__ out, const T* __restrict__ in, size_t n) {
  pdl_prologue();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = Elem<T>::load(in + i);
}

// token_ids[dst[i]] = tokens[src[i]]: input ids that were sampled by the step before and have not
// been read back to the host (miniserve/engine/model_runner.py:263-277 does this with index_copy).
__global__ void fill_tokens_kernel(int* __restrict__ token_ids, const int* __restrict__ dst, const int* __restrict__ tokens,
                                   const int* __restrict__ src, int n) {
  pdl_prologue();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) token_ids[dst[i]] = tokens[src[i]];
}

}  // namespace ms

using namespace ms;

MS_EXPORT int ms_fill_tokens(int* token_ids, const int* dst, const int* tokens, const int* src, int n, cudaStream_t stream) {
  if (n == 0) return 0;
  MS_LAUNCH(fill_tokens_kernel, (n + 127) / 128, 128, 0, stream, token_ids, dst, tokens, src, n);
  return 0;
}

MS_EXPORT int ms_embed_gather(void* residual_f32, const void* table, const int* ids, int tokens, int hidden,
                              int vocab, int dtype, cudaStream_t stream) {
  if (tokens == 0) return 0;
  MS_CHECK_ARG(tokens > 0 && hidden > 0 && vocab > 0, "embed_gather: bad sizes T=%d H=%d V=%d", tokens, hidden, vocab);
  const int threads = hidden >= 256 ? 256 : 64;
  if (dtype == MS_F32) {
    MS_LAUNCH(embed_gather_kernel<float>, tokens, threads, 0, stream, (float*)residual_f32, (const float*)table, ids, hidden, vocab);
  } else if (hidden % 8 == 0 && (uintptr_t)table % 16 == 0 && (uintptr_t)residual_f32 % 16 == 0) {
    const long long items = (long long)tokens * (hidden / 8);
    MS_LAUNCH(embed_gather_bf16x8_kernel, (unsigned)((items + 255) / 256), 256, 0, stream, (float*)residual_f32, (const __nv_bfloat16*)table, ids,
              hidden / 8, vocab, tokens);
  } else {
    MS_LAUNCH(embed_gather_kernel<__nv_bfloat16>, tokens, threads, 0, stream, (float*)residual_f32, (const __nv_bfloat16*)table, ids, hidden, vocab);
  }
  return 0;
}

// delta: an addend in the activation dtype, or null; it is added to the residual before the norm.
MS_EXPORT int ms_add_rmsnorm(void* out, void* residual_f32, const void* delta, const void* weight, const int* rows,
                             float eps, int num_out_rows, int hidden, int write_residual, int dtype,
                             cudaStream_t stream) {
  if (num_out_rows == 0) return 0;
  MS_CHECK_ARG(num_out_rows > 0 && hidden > 0, "add_rmsnorm: bad sizes rows=%d H=%d", num_out_rows, hidden);
  MS_CHECK_ARG(!(rows && write_residual), "add_rmsnorm: a gathered norm cannot write the residual back");
  const size_t smem = (size_t)hidden * sizeof(float);
  MS_CHECK_ARG(smem <= 200 * 1024, "add_rmsnorm: hidden size %d needs %zu bytes of shared memory (limit 204800)", hidden, smem);
  constexpr int THREADS = 256;
  if (dtype == MS_F32) {
    auto k = add_rmsnorm_kernel<float, THREADS>;
    if (smem > 48 * 1024) MS_CHECK_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MS_LAUNCH(k, num_out_rows, THREADS, smem, stream, (float*)out, (float*)residual_f32, (const float*)delta, (const float*)weight, rows, eps, hidden, write_residual);
  } else if (hidden % 8 == 0 && ((uintptr_t)out % 16 == 0) && ((uintptr_t)residual_f32 % 16 == 0) &&
             ((uintptr_t)delta % 16 == 0) && ((uintptr_t)weight % 16 == 0)) {
    if (hidden <= 8 * 128) {
      MS_LAUNCH((add_rmsnorm_bf16x8_kernel<128>), num_out_rows, 128, 0, stream, (__nv_bfloat16*)out, (float*)residual_f32, (const __nv_bfloat16*)delta, (const __nv_bfloat16*)weight, rows, eps, hidden, write_residual);
    } else {
      auto k = add_rmsnorm_bf16x8_kernel<256>;
      const size_t need = hidden <= 8 * 256 ? 0 : smem;
      if (need > 48 * 1024) MS_CHECK_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)need));
      MS_LAUNCH(k, num_out_rows, 256, need, stream, (__nv_bfloat16*)out, (float*)residual_f32, (const __nv_bfloat16*)delta, (const __nv_bfloat16*)weight, rows, eps, hidden, write_residual);
    }
  } else {
    auto k = add_rmsnorm_kernel<__nv_bfloat16, THREADS>;
    if (smem > 48 * 1024) MS_CHECK_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MS_LAUNCH(k, num_out_rows, THREADS, smem, stream, (__nv_bfloat16*)out, (float*)residual_f32, (const __nv_bfloat16*)delta, (const __nv_bfloat16*)weight, rows, eps, hidden, write_residual);
  }
  return 0;
}

MS_EXPORT int ms_silu_mul(void* out, const void* gate_up, int tokens, int inter, int dtype, cudaStream_t stream) {
  if (tokens == 0) return 0;
  MS_CHECK_ARG(tokens > 0 && inter > 0, "silu_mul: bad sizes T=%d I=%d", tokens, inter);
  const size_t total = (size_t)tokens * inter;
  if (dtype == MS_F32) {
    MS_LAUNCH(silu_mul_kernel<float>, (unsigned)((total + 255) / 256), 256, 0, stream, (float*)out, (const float*)gate_up, inter, total);
  } else if (inter % 8 == 0 && ((uintptr_t)out % 16 == 0) && ((uintptr_t)gate_up % 16 == 0)) {
    const size_t total8 = total / 8;
    MS_LAUNCH(silu_mul_bf16x8_kernel, (unsigned)((total8 + 255) / 256), 256, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)gate_up, inter / 8, total8);
  } else {
    MS_LAUNCH(silu_mul_kernel<__nv_bfloat16>, (unsigned)((total + 255) / 256), 256, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)gate_up, inter, total);
  }
  return 0;
}

MS_EXPORT int ms_to_float(void* out_f32, const void* in, long long n, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  if (dtype == MS_F32)
    MS_LAUNCH(to_float_kernel<float>, (unsigned)((n + 255) / 256), 256, 0, stream, (float*)out_f32, (const float*)in, (size_t)n);
  else
    MS_LAUNCH(to_float_kernel<__nv_bfloat16>, (unsigned)((n + 255) / 256), 256, 0, stream, (float*)out_f32, (const __nv_bfloat16*)in, (size_t)n);
  return 0;
}
