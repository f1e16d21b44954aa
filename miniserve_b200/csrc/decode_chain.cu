// A chain of weight-streaming matrix products for a handful of tokens (decode steps), run by ONE
// persistent kernel: C_p[M, N_p] = X_p[M, K_p] * W_p[N_p, K_p]^T for p = 0, 1, ... with M <= 16,
// bfloat16 operands, float32 accumulation, and what lies between two products of a decoder layer
// (residual add, RMSNorm, SiLU * up) in the epilogues.
//
// Why one kernel: at these sizes a product is one trip to HBM long, and a layer run as separate
// kernels (norm, q|k|v, o, norm, gate|up, down) is a chain of such trips with a launch between
// each. Here one CTA per SM stays resident for the whole chain. A producer warp streams the CTA's
// share of EVERY phase's weights through a ring of shared-memory slots with bulk copies, without
// regard to phase boundaries: weights do not depend on the step, so while the eight consumer
// warps wait at the grid-wide barrier between two phases the next phase's weights are already
// arriving. The consumers stage the phase's activations (a few KB, from L2), multiply slot by
// slot with mma.sync, add the warps' partial sums in a fixed order and run the epilogue.
//
// RMSNorm across phases: the phase that closes a residual branch (o, down) writes the new
// residual r = residual + delta in float32, xw = bfloat16(r * norm_weight) and, per token and
// output tile, the sum of r^2. The next phase multiplies xw and scales its result by
// rsqrt(mean(r^2) + eps) per token: the norm's row scale commutes with the product, so no CTA has
// to see a whole row before the weights are used (miniserve/model/qwen3.py:78-82 computes the same
// value with the scale applied first; both round the normalised activation to bfloat16 once).
//
// Every wait (mbarrier, grid barrier) is bounded: when a limit runs out the CTA raises the status
// word, marks the chain aborted for the other CTAs, lets its copies in flight land and returns.
// The grid barrier needs all CTAs resident together: the kernel is launched cooperatively with at
// most one CTA per SM.
//
// Stands where the reference's decode step calls F.linear, rmsnorm and silu-and-mul one after the
// other (miniserve/model/qwen3.py:110-131, miniserve/model/fused.py:173-211).
#include "common.cuh"

namespace ms {

constexpr int CH_CWARPS = 8, CH_CTHREADS = CH_CWARPS * 32, CH_THREADS = CH_CTHREADS + 32;
constexpr int CH_MAX_PHASES = 8;
constexpr int CH_SLOT_ELEMS = 16 * 1024;  // weight elements of one ring slot: 16 rows x 1,024 or 8 rows x 2,048
constexpr int CH_PAD = 32;                // padding of a shared-memory row, in elements: rows 64 bytes apart modulo 128
constexpr int CH_SLOT_BYTES = (CH_SLOT_ELEMS + 16 * CH_PAD) * 2;
constexpr uint32_t CH_WAIT_LIMIT = 1u << 22;

enum ChainEpilogue : int { CH_OUT_BF16 = 0, CH_OUT_F32 = 1, CH_SILU_MUL = 2, CH_RESIDUAL = 3 };

// One product of the chain. All pointers are device pointers; activations are row-major [M, width].
struct ChainPhase {
  const __nv_bfloat16* W;    // [N, K]; CH_SILU_MUL: [2N, K], gate rows then up rows
  const __nv_bfloat16* X;    // [M, K]
  const float* sumsq_in;     // [M, parts_in] partial sums of squares of the rows X was made from, or null (no row scale)
  void* out;                 // CH_OUT_BF16 / CH_SILU_MUL: bf16 [M, N]; CH_OUT_F32: float [M, N]; CH_RESIDUAL: unused
  float* residual;           // CH_RESIDUAL: [M, N] float32, read and written in place
  const __nv_bfloat16* norm_w;  // CH_RESIDUAL: [N], the weight of the norm that follows
  __nv_bfloat16* xw_out;     // CH_RESIDUAL: [M, N] = bf16(residual * norm_w)
  float* sumsq_out;          // CH_RESIDUAL: [M, tiles] sum of residual^2 over each tile's columns
  int N, K;
  int parts_in;
  int epilogue;
  int wrows;                 // weight rows per slot: 16 or 8 (8: narrow outputs, so that every SM has a tile)
  float eps;                 // of the norm whose row scale this phase applies
};

struct ChainProgram {
  int num_phases;
  int M;
  const __nv_bfloat16* prefetch;  // weights the NEXT kernel in the stream reads first: asked into L2 at the end (or null)
  long long prefetch_bytes;
  ChainPhase phase[CH_MAX_PHASES];
};

__device__ __forceinline__ uint32_t ch_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ch_mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(ch_smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void ch_mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(ch_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void ch_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(ch_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool ch_mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(done) : "r"(ch_smem_u32(bar)), "r"(parity) : "memory");
  return done != 0;
}
// global -> shared bulk copy, completion counted in bytes on an mbarrier of this CTA
__device__ __forceinline__ void ch_bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
               ::"r"(ch_smem_u32(dst)), "l"(src), "r"(bytes), "r"(ch_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void ch_consumer_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(CH_CTHREADS) : "memory"); }
__device__ __forceinline__ unsigned ch_ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void ch_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct ChainGeo {
  int wrows, cols, kc, chunks, tiles;
};
__host__ __device__ inline ChainGeo chain_geo(const ChainPhase& ph) {
  ChainGeo g;
  g.wrows = ph.wrows;
  g.cols = ph.epilogue == CH_SILU_MUL ? 8 : ph.wrows;  // output columns of a tile
  g.kc = CH_SLOT_ELEMS / ph.wrows;
  g.chunks = (ph.K + g.kc - 1) / g.kc;
  g.tiles = (ph.N + g.cols - 1) / g.cols;
  return g;
}

// barrier state in global memory (int32 words): [0..1] a 64-bit count of arrivals that only grows (every barrier
// adds gridDim.x, so between barriers it is a multiple of gridDim.x), [2] abort flag
struct ChainSync {
  unsigned* state;
  int* status;
  volatile int* cta_abort;  // shared memory: set when this CTA gave up
};

__device__ __forceinline__ void chain_give_up(const ChainSync& s, int code) {
  atomicCAS(s.status, 0, code);
  atomicExch(s.state + 2, 1u);
  *s.cta_abort = 1;
}

__device__ __forceinline__ unsigned long long ch_ld_acquire64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];\n" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// Grid-wide barrier of the consumer warps: thread 0 of each CTA arrives (a release after the CTA's
// own barrier, which makes the stores of all its threads visible) and polls with acquire loads. The
// count an arrival returns tells which barrier it belongs to: the next multiple of gridDim.x is its target.
__device__ __forceinline__ void chain_grid_barrier(const ChainSync& s) {
  ch_consumer_sync();
  if (threadIdx.x == 0 && !*s.cta_abort) {
    unsigned long long* count = reinterpret_cast<unsigned long long*>(s.state);
    unsigned long long old;
    asm volatile("atom.acq_rel.gpu.global.add.u64 %0, [%1], 1;\n" : "=l"(old) : "l"(count) : "memory");
    const unsigned long long target = (old / gridDim.x + 1) * gridDim.x;
    if (old + 1 < target) {
      uint32_t it = 0;
      while (ch_ld_acquire64(count) < target) {
        if (++it > CH_WAIT_LIMIT || ((it & 255u) == 0 && ch_ld_acquire(s.state + 2) != 0)) {
          chain_give_up(s, 41);
          break;
        }
        if (it > 64) __nanosleep(32);
      }
    }
  }
  ch_consumer_sync();
}

__device__ __forceinline__ void ch_cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;  // 0: the 16 bytes are zero-filled and nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(ch_smem_u32(dst)), "l"(src), "r"(n));
}


// Stage a phase's activations X [M, K] into shared memory rows of `xs_stride` elements (rows past M
// zero) with asynchronous 16-byte copies through L2, all in flight at once, and compute the row
// scale of the norm before the phase from its partial sums of squares. `tid`/`nthreads`: the
// calling group (its warps whole); the caller synchronises the group afterwards.
template <int TOK>
__device__ __forceinline__ void chain_stage(const ChainPhase& ph, int M, __nv_bfloat16* xs, int xs_stride, float* row_scale,
                                            int tid, int nthreads) {
  const int K = ph.K, chunks = K >> 3;
  for (int row = 0; row < TOK; ++row) {
    const bool live = row < M;
    const __nv_bfloat16* src = ph.X + (size_t)(live ? row : 0) * K;
    for (int c = tid; c < chunks; c += nthreads) ch_cp_async16(xs + (size_t)row * xs_stride + c * 8, src + c * 8, live);
  }
  asm volatile("cp.async.commit_group;\n" ::);
  const int warp = tid >> 5, lane = tid & 31, nwarps = nthreads >> 5;
  // rows warp, warp + nwarps: every load of both rows is asked for before any is used (a lane takes four
  // consecutive partial sums with one 16-byte load where the row allows it)
  const int parts = ph.parts_in;
  const bool vec = ph.sumsq_in != nullptr && (parts & 3) == 0 && ((uintptr_t)ph.sumsq_in & 15) == 0;
  float ss[2] = {0.f, 0.f};
  if (ph.sumsq_in != nullptr) {
    for (int base = 0; base < parts; base += vec ? 512 : 128) {
      float4 v[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int row = warp + j * nwarps;
        if (row >= M) continue;
        const float* src = ph.sumsq_in + (size_t)row * parts + base;
        if (vec) {
          if (base + 4 * lane < parts) v[j] = __ldcg(reinterpret_cast<const float4*>(src) + lane);
        } else {
          if (base + lane < parts) v[j].x = __ldcg(src + lane);
          if (base + 32 + lane < parts) v[j].y = __ldcg(src + 32 + lane);
          if (base + 64 + lane < parts) v[j].z = __ldcg(src + 64 + lane);
          if (base + 96 + lane < parts) v[j].w = __ldcg(src + 96 + lane);
        }
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) ss[j] += (v[j].x + v[j].y) + (v[j].z + v[j].w);
    }
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int row = warp + j * nwarps;
    if (row >= 16) continue;
    float scale = 1.f;
    if (ph.sumsq_in != nullptr && row < M) scale = 1.0f / sqrtf(warp_sum(ss[j]) / (float)K + ph.eps);
    if (lane == 0) row_scale[row] = scale;
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
}

// What a thread of the epilogue needs from global memory besides the product: asked for before the
// product is formed, used after.
struct ChainEpiIn {
  float residual;
  float norm_w;
};
template <int TOK>
__device__ __forceinline__ ChainEpiIn chain_epilogue_fetch(const ChainPhase& ph, int cols, int tile, int M, int tid) {
  ChainEpiIn in{0.f, 0.f};
  if (ph.epilogue == CH_RESIDUAL && tid < cols * TOK) {
    const int tok = tid / cols, n = tile * cols + (tid - tok * cols);
    if (tok < M && n < ph.N) {
      in.residual = __ldcg(ph.residual + (size_t)tok * ph.N + n);
      in.norm_w = __bfloat162float(ph.norm_w[n]);
    }
  }
  return in;
}

// The epilogue of one output tile: thread tid < cols * TOK owns (token tid / cols, column tid % cols),
// adds the warps' partial sums `mine` [warps][16][TOK] in warp order and stores what the phase asks for.
template <int TOK, int WARPS>
__device__ __forceinline__ void chain_epilogue(const ChainPhase& ph, int cols, int tiles, int tile, int M, int tid,
                                               const float* mine, const float* row_scale, const ChainEpiIn& in) {
  if (tid >= cols * TOK) return;  // whole warps: cols * TOK is a multiple of 64
  const int N = ph.N;
  const int tok = tid / cols, col = tid - tok * cols;
  const int n = tile * cols + col;
  const bool live = tok < M && n < N;
  float s = 0.f, s2 = 0.f;
#pragma unroll
  for (int w = 0; w < WARPS; ++w) s += mine[(size_t)w * 16 * TOK + col * TOK + tok];
  const float rs = row_scale[tok];
  if (ph.epilogue == CH_SILU_MUL) {
#pragma unroll
    for (int w = 0; w < WARPS; ++w) s2 += mine[(size_t)w * 16 * TOK + (col + 8) * TOK + tok];
    const float gt = __bfloat162float(__float2bfloat16_rn(s * rs)), up = __bfloat162float(__float2bfloat16_rn(s2 * rs));
    if (live) reinterpret_cast<__nv_bfloat16*>(ph.out)[(size_t)tok * N + n] = __float2bfloat16_rn(gt / (1.0f + expf(-gt)) * up);
  } else if (ph.epilogue == CH_OUT_BF16) {
    if (live) reinterpret_cast<__nv_bfloat16*>(ph.out)[(size_t)tok * N + n] = __float2bfloat16_rn(s * rs);
  } else if (ph.epilogue == CH_OUT_F32) {
    if (live) reinterpret_cast<float*>(ph.out)[(size_t)tok * N + n] = s * rs;
  } else {
    // a residual branch closes: r = residual + bf16(delta), and what the next norm needs of r
    float r = 0.f;
    if (live) {
      const size_t o = (size_t)tok * N + n;
      r = in.residual + __bfloat162float(__float2bfloat16_rn(s * rs));
      ph.residual[o] = r;
      ph.xw_out[o] = __float2bfloat16_rn(r * in.norm_w);
    }
    float ss = r * r;
    for (int off = 1; off < cols; off <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if (col == 0 && tok < M) ph.sumsq_out[(size_t)tok * tiles + tile] = ss;
  }
}

template <int MT>
__global__ void __launch_bounds__(CH_THREADS, 1)
decode_chain_kernel(const ChainProgram prog, unsigned* __restrict__ sync_state, int* __restrict__ status, int num_slots,
                    int xs_elems) {
  constexpr int TOK = MT * 8;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  // layout: ring slots | activations | two areas of partial sums | row scales | mbarriers | flags
  unsigned char* ring = smem_raw;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(ring + (size_t)num_slots * CH_SLOT_BYTES);
  float* red = reinterpret_cast<float*>(xs + xs_elems);
  float* row_scale = red + 2 * CH_CWARPS * 16 * TOK;
  uint64_t* full = reinterpret_cast<uint64_t*>(row_scale + 16);
  uint64_t* empty = full + num_slots;
  volatile int* cta_abort = reinterpret_cast<volatile int*>(empty + num_slots);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < num_slots; ++s) {
      ch_mbar_init(full + s, 1);
      ch_mbar_init(empty + s, CH_CWARPS);
    }
    *cta_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();
  pdl_launch_dependents();
  const int M = prog.M;

  if (warp == CH_CWARPS) {
    // ---------------------------------------------------------------- producer: one warp streams the weights
    // lane 0 waits for a free slot and announces the bytes; lane r then issues the copy of the slot's row r
    uint32_t seq = 0;
    bool ok = true;
    for (int p = 0; p < prog.num_phases && ok; ++p) {
      const ChainPhase& ph = prog.phase[p];
      const ChainGeo geo = chain_geo(ph);
      const int row_stride = geo.kc + CH_PAD;
      const bool paired = ph.epilogue == CH_SILU_MUL;
      for (int tile = blockIdx.x; tile < geo.tiles && ok; tile += gridDim.x) {
        const int n0 = tile * geo.cols;
        const int n = paired ? (lane < 8 ? n0 + lane : ph.N + n0 + lane - 8) : n0 + lane;
        const bool valid = lane < geo.wrows && (paired ? (n0 + (lane & 7) < ph.N) : (n < ph.N));
        const int rows = __popc(__ballot_sync(0xffffffffu, valid));
        for (int c = 0; c < geo.chunks && ok; ++c, ++seq) {
          const int slot = seq % num_slots;
          const uint32_t round = seq / num_slots;
          const int k0 = c * geo.kc, klen = min(geo.kc, ph.K - k0);
          const uint32_t row_bytes = (uint32_t)klen * 2;
          if (lane == 0) {
            if (round > 0) {
              uint32_t it = 0;
              while (!ch_mbar_try(empty + slot, (round - 1) & 1)) {
                if (++it > CH_WAIT_LIMIT || *cta_abort) {
                  ok = false;
                  break;
                }
                if (it > 1024) __nanosleep(64);
              }
            }
            if (ok) ch_mbar_expect_tx(full + slot, row_bytes * rows);
          }
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
          if (!ok) break;
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(ring + (size_t)slot * CH_SLOT_BYTES);
          if (valid) ch_bulk_load(dst + (size_t)lane * row_stride, ph.W + (size_t)n * ph.K + k0, row_bytes, full + slot);
        }
      }
    }
    if (lane == 0) {
      if (!ok && !*cta_abort) {
        ChainSync s{sync_state, status, cta_abort};
        chain_give_up(s, 42);
      }
      // copies already issued land in this CTA's shared memory: after giving up, wait (bounded) for the
      // last fill of every slot, which the consumers may not have waited for
      if (*cta_abort) {
        for (int s = 0; s < num_slots && (uint32_t)s < seq; ++s) {
          // the last fill of slot s has sequence number: the largest q < seq with q % num_slots == s
          const uint32_t last = ((seq - 1 - s) / num_slots) * num_slots + s;
          uint32_t it = 0;
          while (!ch_mbar_try(full + s, (last / num_slots) & 1) && ++it < CH_WAIT_LIMIT) {
          }
        }
      }
    }
    return;
  }

  // ------------------------------------------------------------------ consumers
  const int g = lane >> 2, t = lane & 3;
  ChainSync sync{sync_state, status, cta_abort};
  pdl_wait();  // everything before this kernel in the stream has completed: activations may be read
  uint32_t seq = 0;
  int turn = 0;

  for (int p = 0; p < prog.num_phases; ++p) {
    const ChainPhase& ph = prog.phase[p];
    const ChainGeo geo = chain_geo(ph);
    const int K = ph.K;
    const int xs_stride = K + CH_PAD;
    if (p > 0) chain_grid_barrier(sync);

    // activations of this phase: [TOK][K], rows past M zero; and the row scale of the norm before it
    chain_stage<TOK>(ph, M, xs, xs_stride, row_scale, tid, CH_CTHREADS);
    ch_consumer_sync();

    const int row_stride = geo.kc + CH_PAD;
    for (int tile = blockIdx.x; tile < geo.tiles; tile += gridDim.x) {
      float acc[MT][4];
#pragma unroll
      for (int j = 0; j < MT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
      const ChainEpiIn epi_in = chain_epilogue_fetch<TOK>(ph, geo.cols, tile, M, tid);
      for (int c = 0; c < geo.chunks; ++c, ++seq) {
        const int slot = seq % num_slots;
        const uint32_t parity = (seq / num_slots) & 1;
        {
          // A CTA that gave up keeps walking its tiles without waiting (its results no longer matter), so
          // that all of its warps still meet at every barrier below and none is left behind.
          uint32_t it = 0;
          while (!*cta_abort && !ch_mbar_try(full + slot, parity)) {
            if (++it > CH_WAIT_LIMIT) {
              chain_give_up(sync, 43);
              break;
            }
          }
        }
        const __nv_bfloat16* ws = reinterpret_cast<const __nv_bfloat16*>(ring + (size_t)slot * CH_SLOT_BYTES);
        const int k0 = c * geo.kc, klen = min(geo.kc, K - k0);
        const int per_warp = ((klen + CH_CWARPS * 32 - 1) / (CH_CWARPS * 32)) * 32;
        const int wk_begin = warp * per_warp, wk_end = min(klen, wk_begin + per_warp);
        const __nv_bfloat16* wlo = ws + (size_t)g * row_stride + 8 * t;
        const __nv_bfloat16* whi = ws + (size_t)(g + 8) * row_stride + 8 * t;
        const __nv_bfloat16* xrow = xs + (size_t)g * xs_stride + k0 + 8 * t;
        const bool upper = geo.wrows == 16;
#pragma unroll 4
        for (int kk = wk_begin; kk < wk_end; kk += 32) {
          const bool in = kk + 8 * t < wk_end;
          uint4 a = make_uint4(0u, 0u, 0u, 0u), b = a;
          if (in) {
            a = *reinterpret_cast<const uint4*>(wlo + kk);
            if (upper) b = *reinterpret_cast<const uint4*>(whi + kk);
          }
#pragma unroll
          for (int j = 0; j < MT; ++j) {
            uint4 xb = make_uint4(0u, 0u, 0u, 0u);
            if (in) xb = *reinterpret_cast<const uint4*>(xrow + (size_t)8 * j * xs_stride + kk);
            ch_mma(acc[j], a.x, b.x, a.y, b.y, xb.x, xb.y);
            ch_mma(acc[j], a.z, b.z, a.w, b.w, xb.z, xb.w);
          }
        }
        __syncwarp();
        if (lane == 0) ch_mbar_arrive(empty + slot);  // this warp has read the slot
      }

      // the warps' partial sums, added in warp order
      float* mine = red + (size_t)turn * CH_CWARPS * 16 * TOK;
      {
        float* base = mine + (size_t)warp * 16 * TOK;
#pragma unroll
        for (int j = 0; j < MT; ++j) {
          base[g * TOK + 8 * j + 2 * t] = acc[j][0];
          base[g * TOK + 8 * j + 2 * t + 1] = acc[j][1];
          base[(g + 8) * TOK + 8 * j + 2 * t] = acc[j][2];
          base[(g + 8) * TOK + 8 * j + 2 * t + 1] = acc[j][3];
        }
      }
      ch_consumer_sync();
      chain_epilogue<TOK, CH_CWARPS>(ph, geo.cols, geo.tiles, tile, M, tid, mine, row_scale, epi_in);
      turn ^= 1;
    }
  }

  // the weights that the next kernel in the stream reads first, asked into L2 while this one drains
  if (prog.prefetch != nullptr && !*cta_abort) {
    const long long lines = (prog.prefetch_bytes + 127) >> 7;
    const char* base = reinterpret_cast<const char*>(prog.prefetch);
    for (long long i = (long long)blockIdx.x * CH_CTHREADS + tid; i < lines; i += (long long)gridDim.x * CH_CTHREADS)
      asm volatile("prefetch.global.L2 [%0];\n" ::"l"(base + (i << 7)));
  }
}


// The same phase as a kernel of its own: one CTA per output tile, the tile's weights streamed from
// global memory straight into tensor-core fragments (their loads start before the wait on the kernel
// before), the same staging, summation order and epilogue as in the persistent kernel. A chain
// launched phase by phase trades the grid-wide barriers for kernel boundaries, which programmatic
// dependent launch makes cheap.
constexpr int CP_UNROLL = 4;

__device__ __forceinline__ uint4 ch_ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

template <int MT, int WROWS>
__global__ void __launch_bounds__(CH_CTHREADS)
chain_phase_kernel(const ChainPhase ph, int M) {
  constexpr int TOK = MT * 8;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int K = ph.K, N = ph.N;
  const bool paired = ph.epilogue == CH_SILU_MUL;
  const int cols = paired ? 8 : WROWS, tiles = (N + cols - 1) / cols, tile = blockIdx.x;
  const int n0 = tile * cols;
  const int xs_stride = K + CH_PAD;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  float* red = reinterpret_cast<float*>(xs + (size_t)TOK * xs_stride);
  float* row_scale = red + CH_CWARPS * 16 * TOK;

  // fragment rows: g from the tile's first eight weight rows, g + 8 from its second eight (the up rows of a
  // gate|up pair tile); with eight weight rows per tile the second half stays zero
  const bool row_a = n0 + g < N, row_b = WROWS == 16 && (paired ? row_a : n0 + g + 8 < N);
  const __nv_bfloat16* wa_ptr = ph.W + (size_t)(n0 + (row_a ? g : 0)) * K + 8 * t;
  const __nv_bfloat16* wb_ptr = ph.W + (size_t)(row_b ? (paired ? N + n0 + g : n0 + g + 8) : 0) * K + 8 * t;
  // K is walked as the persistent kernel walks it, so that both add in the same order: in chunks of one
  // ring slot (kc), each chunk cut across the eight warps, a warp's part taken in groups of CP_UNROLL steps
  constexpr int kc = CH_SLOT_ELEMS / WROWS;
  const int chunks = (K + kc - 1) / kc;
  int it_c = 0, it_k = -1, it_end = 0;  // the next group: chunk, offset in the chunk, end of this warp's part of it
  auto seek = [&]() {
    while (it_c < chunks) {
      const int klen = min(kc, K - it_c * kc);
      const int per_warp = ((klen + CH_CWARPS * 32 - 1) / (CH_CWARPS * 32)) * 32;
      it_end = min(klen, warp * per_warp + per_warp);
      if (it_k < 0) it_k = warp * per_warp;
      if (it_k < it_end) return;
      ++it_c;
      it_k = -1;
    }
  };
  uint4 wa[CP_UNROLL], wb[CP_UNROLL];
  auto fetch = [&]() {  // the group at the iterator, which then moves on
    const int base = it_c * kc;
#pragma unroll
    for (int u = 0; u < CP_UNROLL; ++u) {
      const int kk = it_k + 32 * u;
      const bool in = kk + 8 * t < it_end;
      wa[u] = (in && row_a) ? ch_ldg_stream(wa_ptr + base + kk) : make_uint4(0u, 0u, 0u, 0u);
      wb[u] = (in && row_b) ? ch_ldg_stream(wb_ptr + base + kk) : make_uint4(0u, 0u, 0u, 0u);
    }
    it_k += 32 * CP_UNROLL;
    seek();
  };
  // weights do not depend on the step: their stream starts before the wait for the kernels before
  pdl_launch_dependents();
  seek();
  int cur_c = it_c, cur_k = it_k, cur_end = it_end;
  if (it_c < chunks) fetch();
  if (t == 0) {  // what does not fit into the registers is asked into L2 meanwhile (one 128-byte line = 64 k of a row)
    const int per_warp_all = ((K + CH_CWARPS * 32 - 1) / (CH_CWARPS * 32)) * 32;
    for (int kk = warp * per_warp_all; kk < min(K, (warp + 1) * per_warp_all); kk += 64) {
      if (row_a) asm volatile("prefetch.global.L2 [%0];\n" ::"l"(wa_ptr - 8 * t + kk));
      if (row_b) asm volatile("prefetch.global.L2 [%0];\n" ::"l"(wb_ptr - 8 * t + kk));
    }
  }
  pdl_wait();
  const ChainEpiIn epi_in = chain_epilogue_fetch<TOK>(ph, cols, tile, M, tid);
  chain_stage<TOK>(ph, M, xs, xs_stride, row_scale, tid, CH_CTHREADS);
  __syncthreads();

  float acc[MT][4];
#pragma unroll
  for (int j = 0; j < MT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  while (cur_c < chunks) {
    uint4 ca[CP_UNROLL], cb[CP_UNROLL];
#pragma unroll
    for (int u = 0; u < CP_UNROLL; ++u) {
      ca[u] = wa[u];
      cb[u] = wb[u];
    }
    const int use_c = cur_c, use_k = cur_k, use_end = cur_end;
    cur_c = it_c, cur_k = it_k, cur_end = it_end;
    if (it_c < chunks) fetch();  // next group in flight while this one is used
#pragma unroll
    for (int u = 0; u < CP_UNROLL; ++u) {
      const int kk = use_k + 32 * u;
      if (kk >= use_end) break;
      const bool in = kk + 8 * t < use_end;
#pragma unroll
      for (int j = 0; j < MT; ++j) {
        uint4 xb = make_uint4(0u, 0u, 0u, 0u);
        if (in) xb = *reinterpret_cast<const uint4*>(xs + (size_t)(8 * j + g) * xs_stride + use_c * kc + kk + 8 * t);
        ch_mma(acc[j], ca[u].x, cb[u].x, ca[u].y, cb[u].y, xb.x, xb.y);
        ch_mma(acc[j], ca[u].z, cb[u].z, ca[u].w, cb[u].w, xb.z, xb.w);
      }
    }
  }
  {
    float* base = red + (size_t)warp * 16 * TOK;
#pragma unroll
    for (int j = 0; j < MT; ++j) {
      base[g * TOK + 8 * j + 2 * t] = acc[j][0];
      base[g * TOK + 8 * j + 2 * t + 1] = acc[j][1];
      base[(g + 8) * TOK + 8 * j + 2 * t] = acc[j][2];
      base[(g + 8) * TOK + 8 * j + 2 * t + 1] = acc[j][3];
    }
  }
  __syncthreads();
  chain_epilogue<TOK, CH_CWARPS>(ph, cols, tiles, tile, M, tid, red, row_scale, epi_in);
}

// residual[t] = float(table[ids[t]]); xw[t] = bf16(residual[t] * norm_w); sumsq[t] = sum of residual[t]^2:
// the start of a chain (miniserve/model/qwen3.py:211 followed by the first layer's input norm).
__global__ void __launch_bounds__(256)
chain_embed_kernel(float* __restrict__ residual, __nv_bfloat16* __restrict__ xw, float* __restrict__ sumsq,
                   const __nv_bfloat16* __restrict__ table, const int* __restrict__ ids, const __nv_bfloat16* __restrict__ norm_w,
                   int hidden, int vocab) {
  pdl_prologue();
  __shared__ float scratch[32];
  const int tkn = blockIdx.x;
  int id = ids[tkn];
  id = min(max(id, 0), vocab - 1);
  const __nv_bfloat16* src = table + (size_t)id * hidden;
  float ss = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float r = __bfloat162float(src[c]);
    residual[(size_t)tkn * hidden + c] = r;
    xw[(size_t)tkn * hidden + c] = __float2bfloat16_rn(r * __bfloat162float(norm_w[c]));
    ss += r * r;
  }
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0) sumsq[tkn] = ss;
}

}  // namespace ms

using namespace ms;

static size_t chain_smem_bytes(int mt, int num_slots, int xs_elems) {
  return (size_t)num_slots * CH_SLOT_BYTES + (size_t)xs_elems * 2 + (size_t)2 * CH_CWARPS * 16 * mt * 8 * 4 + 16 * 4 +
         (size_t)2 * num_slots * 8 + 16;
}

// Weight rows per ring slot for an output of N columns on `grid` CTAs: 16, or 8 when 16-row tiles
// would leave CTAs without one.
MS_EXPORT int ms_decode_chain_wrows(int N, int epilogue, int grid) {
  if (epilogue == CH_SILU_MUL) return 16;
  return ceil_div(N, 16) >= grid ? 16 : 8;
}

// Tiles of a phase (the number of partial sums of squares a CH_RESIDUAL phase writes per token).
MS_EXPORT int ms_decode_chain_tiles(int N, int epilogue, int wrows) {
  return ceil_div(N, epilogue == CH_SILU_MUL ? 8 : wrows);
}

// CTAs the chain runs on: one per SM.
MS_EXPORT int ms_decode_chain_grid(int* grid) {
  int dev = 0;
  MS_CHECK_CUDA(cudaGetDevice(&dev));
  MS_CHECK_CUDA(cudaDeviceGetAttribute(grid, cudaDevAttrMultiProcessorCount, dev));
  return 0;
}

// Whether a chain with these sizes fits a CTA's shared memory (at least two ring slots).
MS_EXPORT int ms_decode_chain_fits(int M, int max_k) {
  if (M < 1 || M > 16 || max_k < 8) return 0;
  const int mt = M > 8 ? 2 : 1;
  return chain_smem_bytes(mt, 2, mt * 8 * (max_k + CH_PAD)) <= 227 * 1024 ? 1 : 0;
}

template <int MT>
static int launch_chain(const ChainProgram& prog, unsigned* sync_state, int* status, int grid, int max_k, cudaStream_t stream) {
  const int xs_elems = MT * 8 * (max_k + CH_PAD);
  int slots = 8;
  while (slots > 2 && chain_smem_bytes(MT, slots, xs_elems) > 227 * 1024) --slots;
  const size_t smem = chain_smem_bytes(MT, slots, xs_elems);
  MS_CHECK_ARG(smem <= 227 * 1024, "decode_chain: K=%d needs %zu bytes of shared memory", max_k, smem);
  auto kernel = decode_chain_kernel<MT>;
  static size_t configured[64] = {};
  int dev = 0;
  MS_CHECK_CUDA(cudaGetDevice(&dev));
  MS_CHECK_ARG(dev >= 0 && dev < 64, "decode_chain: device index %d is not supported", dev);
  if (smem > configured[dev]) {
    MS_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev] = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(CH_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  // Cooperative: the launch fails instead of deadlocking if the CTAs cannot all be resident. Programmatic
  // stream serialisation: the CTAs may become resident, and the producer may start the weight stream,
  // while the kernel before this one drains. If the driver refuses the pair, the second attribute is dropped.
  static int pdl_with_cooperative = 1;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pdl_switch() && pdl_with_cooperative) ? 2 : 1;
  cudaError_t err = cudaLaunchKernelEx(&cfg, kernel, prog, sync_state, status, slots, xs_elems);
  if (err != cudaSuccess && cfg.numAttrs == 2) {
    (void)cudaGetLastError();
    pdl_with_cooperative = 0;
    cfg.numAttrs = 1;
    err = cudaLaunchKernelEx(&cfg, kernel, prog, sync_state, status, slots, xs_elems);
  }
  MS_CHECK_CUDA(err);
  return 0;
}


template <int MT, int WROWS>
static int launch_phase(const ChainPhase& ph, int M, cudaStream_t stream) {
  const size_t smem = (size_t)MT * 8 * (ph.K + CH_PAD) * 2 + (size_t)CH_CWARPS * 16 * MT * 8 * 4 + 16 * 4;
  MS_CHECK_ARG(smem <= 200 * 1024, "decode_chain: K=%d needs %zu bytes of shared memory", ph.K, smem);
  auto kernel = chain_phase_kernel<MT, WROWS>;
  static size_t configured[64] = {};
  int dev = 0;
  MS_CHECK_CUDA(cudaGetDevice(&dev));
  MS_CHECK_ARG(dev >= 0 && dev < 64, "decode_chain: device index %d is not supported", dev);
  if (smem > 48 * 1024 && smem > configured[dev]) {
    MS_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev] = smem;
  }
  const int cols = ph.epilogue == CH_SILU_MUL ? 8 : WROWS;
  MS_LAUNCH(kernel, ceil_div(ph.N, cols), CH_CTHREADS, smem, stream, ph, M);
  return 0;
}

static int launch_phases(const ChainProgram& prog, cudaStream_t stream) {
  for (int p = 0; p < prog.num_phases; ++p) {
    const ChainPhase& ph = prog.phase[p];
    int rc;
    if (prog.M > 8) rc = ph.wrows == 16 ? launch_phase<2, 16>(ph, prog.M, stream) : launch_phase<2, 8>(ph, prog.M, stream);
    else rc = ph.wrows == 16 ? launch_phase<1, 16>(ph, prog.M, stream) : launch_phase<1, 8>(ph, prog.M, stream);
    if (rc) return rc;
  }
  return 0;
}

// Run the chain. `sync_state`: 4 ints of device memory (8-byte aligned), zero before the first launch and
// left consistent by every launch that did not give up (after a raised status word: zero it again).
// `persistent` 1: one cooperative kernel with grid-wide barriers between the phases; 0: one kernel per
// phase. Both add in the same order and give the same bits.
MS_EXPORT int ms_decode_chain(const ChainProgram* prog, unsigned* sync_state, int* status, int persistent, cudaStream_t stream) {
  MS_CHECK_ARG(prog != nullptr && prog->num_phases >= 1 && prog->num_phases <= CH_MAX_PHASES, "decode_chain: 1 to %d phases", CH_MAX_PHASES);
  MS_CHECK_ARG(prog->M >= 1 && prog->M <= 16, "decode_chain: M=%d is outside 1..16", prog->M);
  MS_CHECK_ARG(sync_state != nullptr && status != nullptr && (uintptr_t)sync_state % 8 == 0,
               "decode_chain: needs the barrier state (8-byte aligned) and the status word");
  int grid = 0;
  if (int rc = ms_decode_chain_grid(&grid)) return rc;
  int max_k = 0;
  for (int p = 0; p < prog->num_phases; ++p) {
    const ChainPhase& ph = prog->phase[p];
    MS_CHECK_ARG(ph.N > 0 && ph.K > 0 && ph.K % 8 == 0, "decode_chain: phase %d has N=%d, K=%d (K must be a multiple of 8)", p, ph.N, ph.K);
    MS_CHECK_ARG(ph.wrows == 8 || ph.wrows == 16, "decode_chain: phase %d has %d weight rows per slot", p, ph.wrows);
    MS_CHECK_ARG(ph.epilogue != CH_SILU_MUL || ph.wrows == 16, "decode_chain: phase %d: gate and up rows fill a 16-row slot", p);
    MS_CHECK_ARG(ph.epilogue >= 0 && ph.epilogue <= CH_RESIDUAL, "decode_chain: phase %d has epilogue %d", p, ph.epilogue);
    MS_CHECK_ARG((uintptr_t)ph.W % 16 == 0 && (uintptr_t)ph.X % 16 == 0, "decode_chain: phase %d: operands must be 16-byte aligned", p);
    MS_CHECK_ARG(ph.W != nullptr && ph.X != nullptr, "decode_chain: phase %d lacks an operand", p);
    if (ph.epilogue == CH_RESIDUAL)
      MS_CHECK_ARG(ph.residual && ph.norm_w && ph.xw_out && ph.sumsq_out, "decode_chain: phase %d lacks a residual operand", p);
    else
      MS_CHECK_ARG(ph.out != nullptr, "decode_chain: phase %d has no output", p);
    MS_CHECK_ARG(ph.sumsq_in == nullptr || ph.parts_in > 0, "decode_chain: phase %d has row sums without a count", p);
    max_k = ph.K > max_k ? ph.K : max_k;
  }
  if (!persistent) return launch_phases(*prog, stream);
  return prog->M > 8 ? launch_chain<2>(*prog, sync_state, status, grid, max_k, stream)
                     : launch_chain<1>(*prog, sync_state, status, grid, max_k, stream);
}

MS_EXPORT int ms_chain_embed(float* residual, void* xw, float* sumsq, const void* table, const int* ids, const void* norm_w,
                             int num_tokens, int hidden, int vocab, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  MS_LAUNCH(chain_embed_kernel, num_tokens, 256, 0, stream, residual, (__nv_bfloat16*)xw, sumsq, (const __nv_bfloat16*)table, ids,
            (const __nv_bfloat16*)norm_w, hidden, vocab);
  return 0;
}
