// Weight-streaming matrix product for a handful of tokens (decode steps):
// C[M, N] = X[M, K] * W[N, K]^T with M <= 16, bfloat16 operands, float32 accumulation.
//
// At these sizes the product is bound by reading W once from HBM (about M flops per byte), so the
// kernel is built around the weight stream: a CTA owns 16 rows of W and a slice of K; each of its
// eight warps streams its part of that slice straight from global memory into tensor-core
// fragments with 16-byte loads (eight in flight per lane), multiplies it with the matching
// activations from shared memory, and the warps' partial sums are added in shared memory in a
// fixed order. With `splits` > 1 the K dimension is also cut across CTAs and each split writes
// float32 partial sums [splits, M, N]; the consumer (the fused residual-add + RMSNorm kernel) adds
// them, so narrow outputs (N = hidden) still fill the machine without atomics.
// Stands where the reference's decode step calls F.linear (miniserve/model/qwen3.py:115-131,186).
#include "common.cuh"

namespace ms {

constexpr int SK_WARPS = 8, SK_THREADS = SK_WARPS * 32, SK_ROWS = 16, SK_UNROLL = 4;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// What the kernel does while it stages its activations (the weights are already in flight):
//   PRO_PLAIN  X is bf16 [M, K], copied as it is;
//   PRO_NORM   X = rmsnorm(res_in + delta) * norm_w, the fused residual-add + RMSNorm
//              (miniserve/model/fused.py:170,192: fused_add_rmsnorm): every CTA recomputes the M rows
//              (a few KB), the first CTA also stores the sum to res_out (a buffer other than res_in,
//              since other CTAs still read res_in);
//   PRO_SILU   X = silu(gate) * up of a stacked [M, 2K] gate|up tensor (miniserve/model/qwen3.py:128-131).
enum SkinnyPrologue : int { PRO_PLAIN = 0, PRO_NORM = 1, PRO_SILU = 2 };

struct SkinnyFused {
  const float* res_in;           // PRO_NORM: [M, K] float32
  const __nv_bfloat16* delta;    // PRO_NORM: [M, K] addend or null
  float* res_out;                // PRO_NORM: [M, K] receives res_in + delta (may be null: not stored)
  const __nv_bfloat16* norm_w;   // PRO_NORM: [K]
  float eps;
};


// MODE 0: bf16 out [M, N]; 1: float32 out [M, N]; 2: float32 partials [splits, M, N];
// MODE 3: W is a stacked gate|up weight [2N, K] and out [M, N] = silu(x Wg^T) * (x Wu^T) in bf16
// (miniserve/model/qwen3.py:128-131): the CTA takes 8 gate rows as the lower half of its fragments
// and the 8 up rows that belong to them as the upper half, so both factors of an output meet in it.
// Both products are rounded to bfloat16 before the activation, as when they are stored in between.
template <int MT, int MODE, int PRO>
__global__ void __launch_bounds__(SK_THREADS)
gemm_skinny_kernel(void* __restrict__ out, const __nv_bfloat16* __restrict__ X, const __nv_bfloat16* __restrict__ W,
                   int M, int N, int K, int k_per_split, SkinnyFused fused) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * (MODE == 3 ? 8 : SK_ROWS);
  const int k_begin = blockIdx.y * k_per_split, k_end = min(K, k_begin + k_per_split);
  const int k_len = k_end - k_begin;
  const int xs_stride = k_per_split + 32;  // bf16 elements: rows 64 bytes apart modulo 128, so 16-byte reads of two rows do not collide
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);

  // this warp's part of the slice, in chunks of 32 k (8 per lane of a quad)
  const int per_warp = ((k_len + SK_WARPS * 32 - 1) / (SK_WARPS * 32)) * 32;
  const int wk_begin = warp * per_warp, wk_end = min(k_len, wk_begin + per_warp);
  const int upper = MODE == 3 ? N : 8;  // where the fragments' upper rows come from, relative to the lower ones
  const bool row_a = n0 + g < N, row_b = MODE == 3 ? row_a : n0 + g + 8 < N;
  const __nv_bfloat16* wa_ptr = W + (size_t)(n0 + (row_a ? g : 0)) * K + k_begin + 8 * t;
  const __nv_bfloat16* wb_ptr = W + (size_t)(n0 + (row_b ? g + upper : 0)) * K + k_begin + 8 * t;

  uint4 wa[SK_UNROLL], wb[SK_UNROLL];
  auto fetch = [&](int k) {
#pragma unroll
    for (int u = 0; u < SK_UNROLL; ++u) {
      const int kk = k + 32 * u;
      const bool in = kk + 8 * t < wk_end;
      wa[u] = (in && row_a) ? ldg_stream(wa_ptr + kk) : make_uint4(0u, 0u, 0u, 0u);
      wb[u] = (in && row_b) ? ldg_stream(wb_ptr + kk) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  // the weights do not depend on anything this step computed: their stream starts before the
  // wait for the kernels launched earlier (which produce X)
  pdl_launch_dependents();
  fetch(wk_begin);
  // what does not fit into the registers is asked into L2 meanwhile (one 128-byte line = 64 k of a row)
  if (t == 0) {
    for (int kk = wk_begin + 32 * SK_UNROLL; kk < wk_end; kk += 64) {
      if (row_a) asm volatile("prefetch.global.L2 [%0];\n" ::"l"(wa_ptr + kk));
      if (row_b) asm volatile("prefetch.global.L2 [%0];\n" ::"l"(wb_ptr + kk));
    }
  }
  pdl_wait();

  // activations of this K slice: [MT * 8][k_len], rows past M are zero
  const int chunks = k_len >> 3;
  if (PRO == PRO_NORM) {
    // one warp per row (rows warp, warp + 8); K is whole here (no split)
    for (int row = warp; row < MT * 8; row += SK_WARPS) {
      if (row >= M) {
        for (int c = lane; c < chunks; c += 32) *reinterpret_cast<uint4*>(xs + row * xs_stride + c * 8) = make_uint4(0u, 0u, 0u, 0u);
        continue;
      }
      const float* rin = fused.res_in + (size_t)row * K;
      const __nv_bfloat16* dl = fused.delta ? fused.delta + (size_t)row * K : nullptr;
      float ss = 0.f;
      for (int c = lane; c < chunks; c += 32) {
        float h[8], d[8];
        *reinterpret_cast<float4*>(h) = *reinterpret_cast<const float4*>(rin + c * 8);
        *reinterpret_cast<float4*>(h + 4) = *reinterpret_cast<const float4*>(rin + c * 8 + 4);
        if (dl) {
          bf16x8_to_float(*reinterpret_cast<const uint4*>(dl + c * 8), d);
#pragma unroll
          for (int i = 0; i < 8; ++i) h[i] += d[i];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += h[i] * h[i];
        if (blockIdx.x == 0 && fused.res_out) {
          *reinterpret_cast<float4*>(fused.res_out + (size_t)row * K + c * 8) = *reinterpret_cast<float4*>(h);
          *reinterpret_cast<float4*>(fused.res_out + (size_t)row * K + c * 8 + 4) = *reinterpret_cast<float4*>(h + 4);
        }
      }
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)K + fused.eps);
      for (int c = lane; c < chunks; c += 32) {
        float h[8], d[8], wv[8];
        *reinterpret_cast<float4*>(h) = *reinterpret_cast<const float4*>(rin + c * 8);
        *reinterpret_cast<float4*>(h + 4) = *reinterpret_cast<const float4*>(rin + c * 8 + 4);
        if (dl) {
          bf16x8_to_float(*reinterpret_cast<const uint4*>(dl + c * 8), d);
#pragma unroll
          for (int i = 0; i < 8; ++i) h[i] += d[i];
        }
        bf16x8_to_float(*reinterpret_cast<const uint4*>(fused.norm_w + c * 8), wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) h[i] = (h[i] * inv) * wv[i];
        *reinterpret_cast<uint4*>(xs + row * xs_stride + c * 8) = float_to_bf16x8(h);
      }
    }
  } else {
    for (int idx = tid; idx < MT * 8 * chunks; idx += SK_THREADS) {
      const int row = idx / chunks, c = idx - row * chunks;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (row < M) {
        if (PRO == PRO_SILU) {
          // X is the stacked gate|up tensor [M, 2K]: silu(gate) * up in float32, rounded once
          float gt[8], up[8];
          bf16x8_to_float(*reinterpret_cast<const uint4*>(X + (size_t)row * 2 * K + k_begin + c * 8), gt);
          bf16x8_to_float(*reinterpret_cast<const uint4*>(X + (size_t)row * 2 * K + K + k_begin + c * 8), up);
#pragma unroll
          for (int i = 0; i < 8; ++i) gt[i] = gt[i] / (1.0f + expf(-gt[i])) * up[i];
          v = float_to_bf16x8(gt);
        } else {
          v = *reinterpret_cast<const uint4*>(X + (size_t)row * K + k_begin + c * 8);
        }
      }
      *reinterpret_cast<uint4*>(xs + row * xs_stride + c * 8) = v;
    }
  }
  __syncthreads();

  float acc[MT][4];
#pragma unroll
  for (int j = 0; j < MT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

  for (int k = wk_begin; k < wk_end; k += 32 * SK_UNROLL) {
    uint4 ca[SK_UNROLL], cb[SK_UNROLL];
#pragma unroll
    for (int u = 0; u < SK_UNROLL; ++u) {
      ca[u] = wa[u];
      cb[u] = wb[u];
    }
    if (k + 32 * SK_UNROLL < wk_end) fetch(k + 32 * SK_UNROLL);  // next group in flight while this one is used
#pragma unroll
    for (int u = 0; u < SK_UNROLL; ++u) {
      const int kk = k + 32 * u;
      if (kk >= wk_end) break;
      const bool in = kk + 8 * t < wk_end;
#pragma unroll
      for (int j = 0; j < MT; ++j) {
        uint4 xb = make_uint4(0u, 0u, 0u, 0u);
        if (in) xb = *reinterpret_cast<const uint4*>(xs + (8 * j + g) * xs_stride + kk + 8 * t);
        mma_bf16_16816(acc[j], ca[u].x, cb[u].x, ca[u].y, cb[u].y, xb.x, xb.y);
        mma_bf16_16816(acc[j], ca[u].z, cb[u].z, ca[u].w, cb[u].w, xb.z, xb.w);
      }
    }
  }

  // add the warps' partial sums in warp order
  __syncthreads();
  float* red = reinterpret_cast<float*>(smem_raw);  // [warps][16 rows][MT * 8 tokens]
  constexpr int TOK = MT * 8;
#pragma unroll
  for (int j = 0; j < MT; ++j) {
    float* base = red + (size_t)warp * SK_ROWS * TOK;
    base[g * TOK + 8 * j + 2 * t] = acc[j][0];
    base[g * TOK + 8 * j + 2 * t + 1] = acc[j][1];
    base[(g + 8) * TOK + 8 * j + 2 * t] = acc[j][2];
    base[(g + 8) * TOK + 8 * j + 2 * t + 1] = acc[j][3];
  }
  __syncthreads();
  if (MODE == 3) {
    for (int idx = tid; idx < 8 * TOK; idx += SK_THREADS) {
      const int tok = idx >> 3, row = idx & 7;
      if (tok >= M || n0 + row >= N) continue;
      float sg = 0.f, su = 0.f;
#pragma unroll
      for (int w = 0; w < SK_WARPS; ++w) {
        sg += red[(size_t)w * SK_ROWS * TOK + row * TOK + tok];
        su += red[(size_t)w * SK_ROWS * TOK + (row + 8) * TOK + tok];
      }
      const float gt = __bfloat162float(__float2bfloat16_rn(sg)), up = __bfloat162float(__float2bfloat16_rn(su));
      reinterpret_cast<__nv_bfloat16*>(out)[(size_t)tok * N + n0 + row] = __float2bfloat16_rn(gt / (1.0f + expf(-gt)) * up);
    }
  } else
  for (int idx = tid; idx < SK_ROWS * TOK; idx += SK_THREADS) {
    const int tok = idx / SK_ROWS, row = idx - tok * SK_ROWS;  // consecutive threads: consecutive n
    if (tok >= M || n0 + row >= N) continue;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < SK_WARPS; ++w) s += red[(size_t)w * SK_ROWS * TOK + row * TOK + tok];
    const size_t o = (size_t)tok * N + n0 + row;
    if (MODE == 0) {
      reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(s);
    } else if (MODE == 1) {
      reinterpret_cast<float*>(out)[o] = s;
    } else {
      reinterpret_cast<float*>(out)[(size_t)blockIdx.y * M * N + o] = s;
    }
  }
}

// The same product for an output with many more row tiles than the GPU holds CTAs (the head over
// the vocabulary: 9,496 tiles): a CTA stages X once and walks the tiles blockIdx.x, + gridDim.x, ...
// The weights of the next tile (or of the tile's next k group) are requested before the current
// ones are multiplied, so a CTA always has a tile's rows in flight, and the staging of X and the
// start of a CTA are paid once per CTA instead of once per tile. The sums are formed in the same
// order as in gemm_skinny_kernel, so both kernels give the same bits.
// MODE 0: bfloat16 out [M, N]; 1: float32 out [M, N].
template <int MT, int MODE>
__global__ void __launch_bounds__(SK_THREADS)
gemm_skinny_stream_kernel(void* __restrict__ out, const __nv_bfloat16* __restrict__ X, const __nv_bfloat16* __restrict__ W,
                          int M, int N, int K) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int TOK = MT * 8;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int xs_stride = K + 32;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  // two areas for the warps' partial sums, taken in turn: a tile's sums are still being read while the next tile's are written
  float* red = reinterpret_cast<float*>(smem_raw + (size_t)TOK * xs_stride * 2);
  const int n_tiles = (N + SK_ROWS - 1) / SK_ROWS;
  const int per_warp = ((K + SK_WARPS * 32 - 1) / (SK_WARPS * 32)) * 32;
  const int wk_begin = warp * per_warp, wk_end = min(K, wk_begin + per_warp);

  uint4 wa[SK_UNROLL], wb[SK_UNROLL];
  auto fetch = [&](int tile, int k) {
    const int n0 = tile * SK_ROWS;
    const bool row_a = n0 + g < N, row_b = n0 + g + 8 < N;
    const __nv_bfloat16* pa = W + (size_t)(n0 + (row_a ? g : 0)) * K + 8 * t;
    const __nv_bfloat16* pb = W + (size_t)(n0 + (row_b ? g + 8 : 0)) * K + 8 * t;
#pragma unroll
    for (int u = 0; u < SK_UNROLL; ++u) {
      const int kk = k + 32 * u;
      const bool in = kk + 8 * t < wk_end;
      wa[u] = (in && row_a) ? ldg_stream(pa + kk) : make_uint4(0u, 0u, 0u, 0u);
      wb[u] = (in && row_b) ? ldg_stream(pb + kk) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  int tile = blockIdx.x;  // the grid never has more CTAs than there are tiles
  pdl_launch_dependents();
  fetch(tile, wk_begin);
  pdl_wait();

  const int chunks = K >> 3;
  for (int idx = tid; idx < TOK * chunks; idx += SK_THREADS) {
    const int row = idx / chunks, c = idx - row * chunks;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row < M) v = *reinterpret_cast<const uint4*>(X + (size_t)row * K + c * 8);
    *reinterpret_cast<uint4*>(xs + row * xs_stride + c * 8) = v;
  }
  __syncthreads();

  int turn = 0;
  for (; tile < n_tiles; tile += gridDim.x) {
    float acc[MT][4];
#pragma unroll
    for (int j = 0; j < MT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    for (int k = wk_begin; k < wk_end; k += 32 * SK_UNROLL) {
      uint4 ca[SK_UNROLL], cb[SK_UNROLL];
#pragma unroll
      for (int u = 0; u < SK_UNROLL; ++u) {
        ca[u] = wa[u];
        cb[u] = wb[u];
      }
      if (k + 32 * SK_UNROLL < wk_end) {
        fetch(tile, k + 32 * SK_UNROLL);
      } else if (tile + (int)gridDim.x < n_tiles) {
        fetch(tile + (int)gridDim.x, wk_begin);
      }
#pragma unroll
      for (int u = 0; u < SK_UNROLL; ++u) {
        const int kk = k + 32 * u;
        if (kk >= wk_end) break;
        const bool in = kk + 8 * t < wk_end;
#pragma unroll
        for (int j = 0; j < MT; ++j) {
          uint4 xb = make_uint4(0u, 0u, 0u, 0u);
          if (in) xb = *reinterpret_cast<const uint4*>(xs + (8 * j + g) * xs_stride + kk + 8 * t);
          mma_bf16_16816(acc[j], ca[u].x, cb[u].x, ca[u].y, cb[u].y, xb.x, xb.y);
          mma_bf16_16816(acc[j], ca[u].z, cb[u].z, ca[u].w, cb[u].w, xb.z, xb.w);
        }
      }
    }
    float* mine = red + (size_t)turn * SK_WARPS * SK_ROWS * TOK;
#pragma unroll
    for (int j = 0; j < MT; ++j) {
      float* base = mine + (size_t)warp * SK_ROWS * TOK;
      base[g * TOK + 8 * j + 2 * t] = acc[j][0];
      base[g * TOK + 8 * j + 2 * t + 1] = acc[j][1];
      base[(g + 8) * TOK + 8 * j + 2 * t] = acc[j][2];
      base[(g + 8) * TOK + 8 * j + 2 * t + 1] = acc[j][3];
    }
    __syncthreads();  // also: everyone has finished reading the other area (the tile before)
    const int n0 = tile * SK_ROWS;
    for (int idx = tid; idx < SK_ROWS * TOK; idx += SK_THREADS) {
      const int tok = idx / SK_ROWS, row = idx - tok * SK_ROWS;  // consecutive threads: consecutive n
      if (tok >= M || n0 + row >= N) continue;
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < SK_WARPS; ++w) s += mine[(size_t)w * SK_ROWS * TOK + row * TOK + tok];
      const size_t o = (size_t)tok * N + n0 + row;
      if (MODE == 0) {
        reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(s);
      } else {
        reinterpret_cast<float*>(out)[o] = s;
      }
    }
    turn ^= 1;
  }
}

// Outputs with at least this many row tiles per SM go to the kernel that walks tiles.
constexpr int SK_STREAM_TILES_PER_SM = 8;
static int g_stream_mode = 1;  // 0: off; 1: on; 2 (measurements only): on, launched with the programmatic-dependent-launch attribute

template <int MT, int MODE>
static int launch_skinny_stream(void* out, const void* X, const void* W, int M, int N, int K, int sm_count, cudaStream_t stream) {
  const size_t smem = (size_t)MT * 8 * (K + 32) * 2 + 2 * (size_t)SK_WARPS * SK_ROWS * MT * 8 * 4;
  MS_CHECK_ARG(smem <= 200 * 1024, "gemm_skinny: K=%d needs %zu bytes of shared memory", K, smem);
  auto kernel = gemm_skinny_stream_kernel<MT, MODE>;
  static size_t configured = 0;
  static int per_sm = 0;
  if (smem > configured) {
    if (smem > 48 * 1024) MS_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
    per_sm = 0;
  }
  if (per_sm == 0) {
    // CTAs that are resident together for the largest shared-memory size seen so far
    MS_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, SK_THREADS, configured));
    MS_CHECK_ARG(per_sm > 0, "gemm_skinny: the kernel does not fit an SM with %zu bytes of shared memory", configured);
  }
  const long long tiles = ceil_div(N, SK_ROWS), resident = (long long)sm_count * per_sm;
  // Launched without the programmatic-dependent-launch attribute (the kernel's griddepcontrol
  // instructions then do nothing and it starts when the kernel before it has completed): its
  // CTAs fill every SM's registers for the whole of its time, and when they became resident
  // early, behind the last layers' kernels, the step was slower than with no overlap at all
  // (a decode step of Qwen3-0.6B at batch 8: 1.359 ms with the attribute, 1.301 ms without,
  // 1.329 ms with one row tile per CTA).
  const int pdl_was = pdl_switch();
  if (g_stream_mode != 2) pdl_switch() = 0;
  const cudaError_t err = launch(kernel, dim3((unsigned)(tiles < resident ? tiles : resident)), dim3(SK_THREADS), smem, stream, out,
                                (const __nv_bfloat16*)X, (const __nv_bfloat16*)W, M, N, K);
  pdl_switch() = pdl_was;
  MS_CHECK_CUDA(err);
  return 0;
}

template <int MT, int MODE, int PRO>
static int launch_skinny(void* out, const void* X, const void* W, int M, int N, int K, int splits, const SkinnyFused& fused,
                         cudaStream_t stream) {
  // whole multiples of 8 warps x 32 k per split keep every warp's range aligned
  int k_per_split = ceil_div(ceil_div(K, splits), 32) * 32;
  const int used_splits = ceil_div(K, k_per_split);
  MS_CHECK_ARG(used_splits == splits, "gemm_skinny: %d splits leave some without work (K=%d)", splits, K);
  const size_t smem_x = (size_t)MT * 8 * (k_per_split + 32) * 2;
  const size_t smem_red = (size_t)SK_WARPS * SK_ROWS * MT * 8 * 4;
  const size_t smem = smem_x > smem_red ? smem_x : smem_red;
  MS_CHECK_ARG(smem <= 200 * 1024, "gemm_skinny: K slice of %d needs %zu bytes of shared memory", k_per_split, smem);
  auto kernel = gemm_skinny_kernel<MT, MODE, PRO>;
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    MS_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  dim3 grid(ceil_div(N, MODE == 3 ? 8 : SK_ROWS), splits);
  MS_LAUNCH(kernel, grid, SK_THREADS, smem, stream, out, (const __nv_bfloat16*)X, (const __nv_bfloat16*)W, M, N, K, k_per_split, fused);
  return 0;
}

}  // namespace ms

using namespace ms;

static int check_skinny(const void* W, int M, int N, int K, int splits, int out_mode) {
  MS_CHECK_ARG(M > 0 && M <= 16, "gemm_skinny: M=%d is outside 1..16", M);
  MS_CHECK_ARG(K > 0 && K % 8 == 0, "gemm_skinny: K=%d must be a multiple of 8", K);
  MS_CHECK_ARG((uintptr_t)W % 16 == 0, "gemm_skinny: the weight must be 16-byte aligned");
  MS_CHECK_ARG(splits >= 1 && (splits == 1 || out_mode == 2), "gemm_skinny: only partial sums can be split over K");
  MS_CHECK_ARG(out_mode >= 0 && out_mode <= 2, "gemm_skinny: bad output mode %d", out_mode);
  MS_CHECK_ARG(ceil_div(N, SK_ROWS) <= 2147483647 && splits <= 65535, "gemm_skinny: grid too large");
  return 0;
}

#define MS_SK_DISPATCH(PRO)                                                                                   \
  do {                                                                                                        \
    const bool wide = M > 8;                                                                                  \
    if (out_mode == 0) return wide ? launch_skinny<2, 0, PRO>(out, X, W, M, N, K, splits, fused, stream)      \
                                   : launch_skinny<1, 0, PRO>(out, X, W, M, N, K, splits, fused, stream);     \
    if (out_mode == 1) return wide ? launch_skinny<2, 1, PRO>(out, X, W, M, N, K, splits, fused, stream)      \
                                   : launch_skinny<1, 1, PRO>(out, X, W, M, N, K, splits, fused, stream);     \
    return wide ? launch_skinny<2, 2, PRO>(out, X, W, M, N, K, splits, fused, stream)                         \
                : launch_skinny<1, 2, PRO>(out, X, W, M, N, K, splits, fused, stream);                        \
  } while (0)

// Tuning and tests: 0 keeps outputs with very many row tiles on the kernel with one tile per CTA;
// 2 launches the tile-walking kernel with the dependent-launch attribute (see launch_skinny_stream).
MS_EXPORT void ms_gemm_skinny_set_stream(int mode) { ms::g_stream_mode = mode; }

// out_mode 0: bfloat16 [M, N]; 1: float32 [M, N]; 2: float32 partials [splits, M, N].
MS_EXPORT int ms_gemm_skinny_bf16(void* out, const void* X, const void* W, int M, int N, int K, int splits, int out_mode,
                                  cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (int rc = check_skinny(W, M, N, K, splits, out_mode)) return rc;
  MS_CHECK_ARG((uintptr_t)X % 16 == 0, "gemm_skinny: the activations must be 16-byte aligned");
  if (splits == 1 && out_mode != 2) {
    static int sm_count = 0;
    if (sm_count == 0) {
      int dev = 0;
      MS_CHECK_CUDA(cudaGetDevice(&dev));
      MS_CHECK_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
    }
    if (g_stream_mode != 0 && ceil_div(N, SK_ROWS) >= (long long)SK_STREAM_TILES_PER_SM * sm_count) {
      const bool wide = M > 8;
      if (out_mode == 0) return wide ? launch_skinny_stream<2, 0>(out, X, W, M, N, K, sm_count, stream)
                                     : launch_skinny_stream<1, 0>(out, X, W, M, N, K, sm_count, stream);
      return wide ? launch_skinny_stream<2, 1>(out, X, W, M, N, K, sm_count, stream)
                  : launch_skinny_stream<1, 1>(out, X, W, M, N, K, sm_count, stream);
    }
  }
  const SkinnyFused fused = {};
  MS_SK_DISPATCH(PRO_PLAIN);
}

// out [M, N] bfloat16 = silu(X Wg^T) * (X Wu^T) for the stacked weight W = [Wg; Wu] of 2N rows.
MS_EXPORT int ms_gemm_skinny_gate_up_bf16(void* out, const void* X, const void* W, int M, int N, int K, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (int rc = check_skinny(W, M, N, K, 1, 0)) return rc;
  MS_CHECK_ARG((uintptr_t)X % 16 == 0, "gemm_skinny: the activations must be 16-byte aligned");
  const SkinnyFused fused = {};
  return M > 8 ? launch_skinny<2, 3, PRO_PLAIN>(out, X, W, M, N, K, 1, fused, stream)
               : launch_skinny<1, 3, PRO_PLAIN>(out, X, W, M, N, K, 1, fused, stream);
}

// out = rmsnorm(res_in + delta) * norm_w times W^T; res_out (a buffer other than res_in, or null)
// receives res_in + delta. delta may be null.
MS_EXPORT int ms_gemm_skinny_norm_bf16(void* out, const float* res_in, const void* delta, float* res_out, const void* norm_w,
                                       float eps, const void* W, int M, int N, int K, int out_mode, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  const int splits = 1;
  if (int rc = check_skinny(W, M, N, K, splits, out_mode)) return rc;
  MS_CHECK_ARG(out_mode != 2, "gemm_skinny: the fused norm needs the whole K in one CTA (no partial sums)");
  MS_CHECK_ARG(res_in != nullptr && norm_w != nullptr && res_out != res_in, "gemm_skinny: the fused norm needs res_in, norm_w and a separate res_out");
  MS_CHECK_ARG(((uintptr_t)res_in % 16 == 0) && ((uintptr_t)delta % 16 == 0) && ((uintptr_t)res_out % 16 == 0) && ((uintptr_t)norm_w % 16 == 0),
               "gemm_skinny: fused-norm operands must be 16-byte aligned");
  const void* X = nullptr;
  const SkinnyFused fused = {res_in, (const __nv_bfloat16*)delta, res_out, (const __nv_bfloat16*)norm_w, eps};
  MS_SK_DISPATCH(PRO_NORM);
}

// out = (silu(gate_up[:, :K]) * gate_up[:, K:]) times W^T for gate_up [M, 2K].
MS_EXPORT int ms_gemm_skinny_silu_bf16(void* out, const void* gate_up, const void* W, int M, int N, int K, int splits,
                                       int out_mode, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (int rc = check_skinny(W, M, N, K, splits, out_mode)) return rc;
  MS_CHECK_ARG((uintptr_t)gate_up % 16 == 0, "gemm_skinny: the activations must be 16-byte aligned");
  const void* X = gate_up;
  const SkinnyFused fused = {};
  MS_SK_DISPATCH(PRO_SILU);
}
