// Weight-streaming matrix product for a handful of tokens (decode steps):
// C[M, N] = X[M, K] * W[N, K]^T with M <= 16, bfloat16 operands, float32 accumulation.
//
// At these sizes the product is bound by reading W once from HBM (about M flops per byte), so the
// kernel is built around the weight stream: a CTA owns 16 rows of W and a slice of K; each of its
// eight warps streams its part of that slice straight from global memory into tensor-core
// fragments with 16-byte loads (eight in flight per lane), multiplies it with the matching
// activations from shared memory, and the warps' partial sums are added in shared memory in a
// fixed order.
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

// MODE 0: bf16 out [M, N]; 1: float32 out [M, N];
// MODE 3: W is a stacked gate|up weight [2N, K] and out [M, N] = silu(x Wg^T) * (x Wu^T) in bf16
// (miniserve/model/qwen3.py:128-131): the CTA takes 8 gate rows as the lower half of its fragments
// and the 8 up rows that belong to them as the upper half, so both factors of an output meet in it.
// Both products are rounded to bfloat16 before the activation, as when they are stored in between.
template <int MT, int MODE>
__global__ void __launch_bounds__(SK_THREADS)
gemm_skinny_kernel(void* __restrict__ out, const __nv_bfloat16* __restrict__ X, const __nv_bfloat16* __restrict__ W,
                   int M, int N, int K) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * (MODE == 3 ? 8 : SK_ROWS);
  const int k_begin = 0, k_len = K;
  const int xs_stride = K + 32;  // bf16 elements: rows 64 bytes apart modulo 128, so 16-byte reads of two rows do not collide
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
  for (int idx = tid; idx < MT * 8 * chunks; idx += SK_THREADS) {
    const int row = idx / chunks, c = idx - row * chunks;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row < M) v = *reinterpret_cast<const uint4*>(X + (size_t)row * K + c * 8);
    *reinterpret_cast<uint4*>(xs + row * xs_stride + c * 8) = v;
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
    } else {
      reinterpret_cast<float*>(out)[o] = s;
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
static int g_stream_mode = 1;  // 0: off (one row tile per CTA); 1: on

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
  pdl_switch() = 0;
  const cudaError_t err = launch(kernel, dim3((unsigned)(tiles < resident ? tiles : resident)), dim3(SK_THREADS), smem, stream, out,
                                (const __nv_bfloat16*)X, (const __nv_bfloat16*)W, M, N, K);
  pdl_switch() = pdl_was;
  MS_CHECK_CUDA(err);
  return 0;
}

template <int MT, int MODE>
static int launch_skinny(void* out, const void* X, const void* W, int M, int N, int K, cudaStream_t stream) {
  const size_t smem_x = (size_t)MT * 8 * (K + 32) * 2;
  const size_t smem_red = (size_t)SK_WARPS * SK_ROWS * MT * 8 * 4;
  const size_t smem = smem_x > smem_red ? smem_x : smem_red;
  MS_CHECK_ARG(smem <= 200 * 1024, "gemm_skinny: K=%d needs %zu bytes of shared memory", K, smem);
  auto kernel = gemm_skinny_kernel<MT, MODE>;
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    MS_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  dim3 grid(ceil_div(N, MODE == 3 ? 8 : SK_ROWS));
  MS_LAUNCH(kernel, grid, SK_THREADS, smem, stream, out, (const __nv_bfloat16*)X, (const __nv_bfloat16*)W, M, N, K);
  return 0;
}

}  // namespace ms

using namespace ms;

static int check_skinny(const void* W, int M, int N, int K, int out_mode) {
  MS_CHECK_ARG(M > 0 && M <= 16, "gemm_skinny: M=%d is outside 1..16", M);
  MS_CHECK_ARG(K > 0 && K % 8 == 0, "gemm_skinny: K=%d must be a multiple of 8", K);
  MS_CHECK_ARG((uintptr_t)W % 16 == 0, "gemm_skinny: the weight must be 16-byte aligned");
  MS_CHECK_ARG(out_mode == 0 || out_mode == 1, "gemm_skinny: bad output mode %d", out_mode);
  MS_CHECK_ARG(ceil_div(N, SK_ROWS) <= 2147483647, "gemm_skinny: grid too large");
  return 0;
}

// 0 keeps outputs with very many row tiles on the kernel with one tile per CTA (tests compare the two).
MS_EXPORT void ms_gemm_skinny_set_stream(int mode) { ms::g_stream_mode = mode; }

// out_mode 0: bfloat16 [M, N]; 1: float32 [M, N].
MS_EXPORT int ms_gemm_skinny_bf16(void* out, const void* X, const void* W, int M, int N, int K, int out_mode,
                                  cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (int rc = check_skinny(W, M, N, K, out_mode)) return rc;
  MS_CHECK_ARG((uintptr_t)X % 16 == 0, "gemm_skinny: the activations must be 16-byte aligned");
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    MS_CHECK_CUDA(cudaGetDevice(&dev));
    MS_CHECK_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
  }
  const bool wide = M > 8;
  if (g_stream_mode != 0 && ceil_div(N, SK_ROWS) >= (long long)SK_STREAM_TILES_PER_SM * sm_count) {
    if (out_mode == 0) return wide ? launch_skinny_stream<2, 0>(out, X, W, M, N, K, sm_count, stream)
                                   : launch_skinny_stream<1, 0>(out, X, W, M, N, K, sm_count, stream);
    return wide ? launch_skinny_stream<2, 1>(out, X, W, M, N, K, sm_count, stream)
                : launch_skinny_stream<1, 1>(out, X, W, M, N, K, sm_count, stream);
  }
  if (out_mode == 0) return wide ? launch_skinny<2, 0>(out, X, W, M, N, K, stream) : launch_skinny<1, 0>(out, X, W, M, N, K, stream);
  return wide ? launch_skinny<2, 1>(out, X, W, M, N, K, stream) : launch_skinny<1, 1>(out, X, W, M, N, K, stream);
}

// out [M, N] bfloat16 = silu(X Wg^T) * (X Wu^T) for the stacked weight W = [Wg; Wu] of 2N rows.
MS_EXPORT int ms_gemm_skinny_gate_up_bf16(void* out, const void* X, const void* W, int M, int N, int K, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (int rc = check_skinny(W, M, N, K, 0)) return rc;
  MS_CHECK_ARG((uintptr_t)X % 16 == 0, "gemm_skinny: the activations must be 16-byte aligned");
  return M > 8 ? launch_skinny<2, 3>(out, X, W, M, N, K, stream) : launch_skinny<1, 3>(out, X, W, M, N, K, stream);
}
