// bfloat16 matrix product on the 5th-generation tensor cores:
// C[M, N] = A[M, K] * W[N, K]^T (both operands K-major), float32 accumulation in tensor memory.
//
// One CTA computes a 128 x BN tile of C. Roles by warp:
//   warp 0   one elected lane streams A and W tiles (128 x 64 and BN x 64 bf16, 128-byte swizzle)
//            into a ring of shared-memory stages with TMA (cp.async.bulk.tensor) and mbarriers;
//   warp 1   allocates tensor memory; one elected lane issues tcgen05.mma (M=128, N=BN, K=16, four
//            per stage) on shared-memory descriptors and releases each stage with tcgen05.commit;
//   warps 2-5 read the accumulator back with tcgen05.ld (each warp its own 32 lanes), apply the
//            epilogue and store: plain (bf16 or float32 out), or SiLU(gate) * up for the stacked
//            gate|up projection, which then never writes the 2 x intermediate tensor.
// Every wait on an mbarrier is bounded: after a limit the kernel raises a status word, stops
// waiting, frees its tensor memory and returns.
//
// Stands where the reference calls F.linear on cuBLAS (miniserve/model/qwen3.py:115-131) and, for
// the fused epilogue, flashinfer.silu_and_mul after the gate_up product (miniserve/model/fused.py:195).
#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

namespace ms {

constexpr int TC_BM = 128, TC_BK = 64;
constexpr int TC_THREADS = 192;

enum TcEpilogue : int { TC_OUT_BF16 = 0, TC_OUT_F32 = 1, TC_SILU_MUL = 2, TC_QKV_ROPE = 3 };

// What the q|k|v epilogue (TC_QKV_ROPE) needs besides the product: per-head RMSNorm of q and k, rotation
// by position and the write of q to [T, nq, 128] and of k, v into their cache pages, as the separate
// kernel of rope_kv.cu does (miniserve/model/qwen3.py:118-123, miniserve/model/attention.py:139). Head size 128.
struct QkvEpilogue {
  __nv_bfloat16* k_pool;            // [pages + 1, nkv, page_size, 128]
  __nv_bfloat16* v_pool;
  const __nv_bfloat16* q_norm_w;    // [128] or null (no norm)
  const __nv_bfloat16* k_norm_w;
  const float* cos_sin;             // the rotation table by tiles of 128 tokens (rope_kv.cu, ms_rope_table_tile), or null (no rotation)
  const int* positions;
  const int* row_of_token;
  const int* page_indptr;
  const int* page_indices;
  int nq, nkv, page_shift;
  float eps;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity. Returns false if the time limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) { return mbar_wait_bounded(smem_u32(bar), parity); }
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(pred));
  return pred != 0;
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 bf16) wide, laid
// out by TMA with the 128-byte swizzle: 8-row groups are 1024 bytes apart (stride byte offset),
// the leading byte offset is unused for swizzled K-major tiles (set to 1), version 1, layout 2.
__device__ __forceinline__ uint64_t make_smem_desc(const void* tile) {
  const uint32_t addr = smem_u32(tile);
  uint64_t desc = 0;
  desc |= (uint64_t)((addr & 0x3FFFF) >> 4);  // start address, 16-byte units
  desc |= (uint64_t)1 << 16;                  // leading byte offset (ignored)
  desc |= (uint64_t)(1024 >> 4) << 32;        // stride byte offset
  desc |= (uint64_t)1 << 46;                  // descriptor version for this architecture
  desc |= (uint64_t)2 << 61;                  // SWIZZLE_128B
  return desc;
}

// kind::f16 instruction descriptor: D float32, A and B bfloat16, both K-major, M x N.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}

template <int BN>
struct TcSmem {
  static constexpr int a_bytes = TC_BM * TC_BK * 2;
  static constexpr int b_bytes = BN * TC_BK * 2;
  static constexpr int stage_bytes = a_bytes + b_bytes;
};

// grid: (ceil(N_out / (BN or BN/2 for SiLU)), ceil(M / 128)). For TC_SILU_MUL, W is [2 * inter, K]
// (gate rows, then up rows), BN is 256 and a CTA computes 128 gate and the matching 128 up columns.
template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(TC_THREADS, (STAGES * (TC_BM + BN) * TC_BK * 2 + 2048 <= 110 * 1024) ? 2 : 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, void* __restrict__ out,
               int M, int N_out, int K, int up_row_offset, int* __restrict__ status) {
  extern __shared__ unsigned char smem_dyn[];
  // 128-byte swizzled tiles want 1024-byte alignment
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], accum_bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int gave_up;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int COLS = EPI == TC_SILU_MUL ? BN / 2 : BN;  // output columns per CTA
  const int n0 = blockIdx.x * COLS, m0 = blockIdx.y * TC_BM;
  const int k_iters = (K + TC_BK - 1) / TC_BK;
  constexpr uint32_t TMEM_COLS = BN <= 32 ? 32 : BN <= 64 ? 64 : BN <= 128 ? 128 : 256;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&accum_bar, 1);
    gave_up = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;

  // everything above touches nothing an earlier kernel wrote; A does
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    if (elect_one()) {
      for (int it = 0; it < k_iters; ++it) {
        const int s = it % STAGES;
        if (it >= STAGES && !mbar_wait(&empty_bar[s], ((it / STAGES) - 1) & 1)) {
          atomicExch(status, 11);
          gave_up = 1;
          break;
        }
        unsigned char* a_tile = smem + (size_t)s * TcSmem<BN>::stage_bytes;
        unsigned char* b_tile = a_tile + TcSmem<BN>::a_bytes;
        mbar_expect_tx(&full_bar[s], TcSmem<BN>::stage_bytes);
        tma_load_2d(a_tile, &map_a, &full_bar[s], it * TC_BK, m0);
        if (EPI == TC_SILU_MUL) {
          tma_load_2d(b_tile, &map_w, &full_bar[s], it * TC_BK, n0);
          tma_load_2d(b_tile + TcSmem<BN>::b_bytes / 2, &map_w, &full_bar[s], it * TC_BK, up_row_offset + n0);
        } else {
          tma_load_2d(b_tile, &map_w, &full_bar[s], it * TC_BK, n0);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc(TC_BM, BN);
      bool ok = true;
      for (int it = 0; it < k_iters && ok; ++it) {
        const int s = it % STAGES;
        if (!mbar_wait(&full_bar[s], (it / STAGES) & 1)) {
          atomicExch(status, 12);
          gave_up = 1;
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const unsigned char* a_tile = smem + (size_t)s * TcSmem<BN>::stage_bytes;
        const unsigned char* b_tile = a_tile + TcSmem<BN>::a_bytes;
        const uint64_t da = make_smem_desc(a_tile), db = make_smem_desc(b_tile);
#pragma unroll
        for (int k = 0; k < TC_BK / 16; ++k) {
          // 16 bf16 = 32 bytes further along K inside the swizzle atom: 2 units of 16 bytes
          umma_bf16(tmem_base, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (it | k) != 0);
        }
        umma_commit(&empty_bar[s]);  // arrives when the MMAs that read this stage are done
      }
      umma_commit(&accum_bar);  // arrives when every MMA issued so far is done
    }
  } else {
    // epilogue warps 2..5: warp w may touch tensor-memory lanes 32 * (w % 4) .. + 31
    const int quad = warp & 3;
    const int row = m0 + quad * 32 + lane;
    bool ok = mbar_wait(&accum_bar, 0);
    if (!ok) {
      atomicExch(status, 13);
      gave_up = 1;
    }
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    if (ok) {
      const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < COLS; c += 32) {
        uint32_t acc[32];
        tmem_ld32(lane_addr + (uint32_t)c, acc);
        uint32_t up[32];
        if (EPI == TC_SILU_MUL) tmem_ld32(lane_addr + (uint32_t)(COLS + c), up);
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
        if (row < M) {
          const int col0 = n0 + c;
          if (EPI == TC_OUT_F32) {
            float* dst = reinterpret_cast<float*>(out) + (size_t)row * N_out + col0;
            if (col0 + 32 <= N_out && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<uint4*>(dst + j) = make_uint4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
            } else {
              for (int j = 0; j < 32 && col0 + j < N_out; ++j) dst[j] = __uint_as_float(acc[j]);
            }
          } else {
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              float x = __uint_as_float(acc[j]);
              if (EPI == TC_SILU_MUL) x = x / (1.0f + expf(-x)) * __uint_as_float(up[j]);
              v[j] = x;
            }
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)row * N_out + col0;
            if (col0 + 32 <= N_out && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 pk;
                __nv_bfloat162 p0 = __floats2bfloat162_rn(v[j], v[j + 1]), p1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
                __nv_bfloat162 p2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]), p3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
                pk.x = *reinterpret_cast<uint32_t*>(&p0);
                pk.y = *reinterpret_cast<uint32_t*>(&p1);
                pk.z = *reinterpret_cast<uint32_t*>(&p2);
                pk.w = *reinterpret_cast<uint32_t*>(&p3);
                *reinterpret_cast<uint4*>(dst + j) = pk;
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < N_out; ++j) dst[j] = __float2bfloat16_rn(v[j]);
            }
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// One 32-column chunk of a row of the accumulator (and of the up half for SiLU * up), to global memory.
// SiLU with the fast exponential and division: both are good to about two float32 ulps, far inside
// the bfloat16 rounding that follows. For x below -88 the exponential overflows to infinity and the
// quotient is -0, the limit of SiLU there.
__device__ __forceinline__ float silu_fast(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

template <int EPI>
__device__ __forceinline__ void store_chunk(void* __restrict__ out, const uint32_t (&acc)[32], const uint32_t (&up)[32], int row,
                                            int col0, int N_out) {
  if (EPI == TC_OUT_F32) {
    float* dst = reinterpret_cast<float*>(out) + (size_t)row * N_out + col0;
    if (col0 + 32 <= N_out && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) *reinterpret_cast<uint4*>(dst + j) = make_uint4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
    } else {
      for (int j = 0; j < 32 && col0 + j < N_out; ++j) dst[j] = __uint_as_float(acc[j]);
    }
  } else {
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    float x = __uint_as_float(acc[j]);
    if (EPI == TC_SILU_MUL) x = x / (1.0f + expf(-x)) * __uint_as_float(up[j]);
    v[j] = x;
  }
  __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)row * N_out + col0;
  if (col0 + 32 <= N_out && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      uint4 pk;
      __nv_bfloat162 p0 = __floats2bfloat162_rn(v[j], v[j + 1]), p1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
      __nv_bfloat162 p2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]), p3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
      pk.x = *reinterpret_cast<uint32_t*>(&p0);
      pk.y = *reinterpret_cast<uint32_t*>(&p1);
      pk.z = *reinterpret_cast<uint32_t*>(&p2);
      pk.w = *reinterpret_cast<uint32_t*>(&p3);
      *reinterpret_cast<uint4*>(dst + j) = pk;
    }
  } else {
    for (int j = 0; j < 32 && col0 + j < N_out; ++j) dst[j] = __float2bfloat16_rn(v[j]);
  }
  }
}

// The persistent form: one CTA per SM walks over tiles (tile = CTA index, + grid size, ...), the
// ring of shared-memory stages keeps running from one tile into the next, and tensor memory holds
// two accumulators, so that the epilogue of a tile overlaps the products of the next one.
template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                          void* __restrict__ out, int M, int N_out, int K, int up_row_offset, int* __restrict__ status) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  static_assert(BN <= 256, "two accumulators of BN columns must fit 512 columns of tensor memory");
  constexpr uint32_t ACC_COLS = BN <= 64 ? 64 : BN <= 128 ? 128 : 256;  // columns of one accumulator
  constexpr int COLS = EPI == TC_SILU_MUL ? BN / 2 : BN;                // output columns per tile

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_iters = (K + TC_BK - 1) / TC_BK;
  const int n_tiles = (N_out + COLS - 1) / COLS, m_tiles = (M + TC_BM - 1) / TC_BM;
  const int num_tiles = n_tiles * m_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 128);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base_slot)), "r"(2 * ACC_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;

  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    if (elect_one()) {
      int kb = 0;  // k-blocks loaded so far, over all tiles: the ring does not restart between tiles
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        const int n0 = (tile % n_tiles) * COLS, m0 = (tile / n_tiles) * TC_BM;
        bool ok = true;
        for (int it = 0; it < k_iters; ++it, ++kb) {
          const int s = kb % STAGES;
          if (kb >= STAGES && !mbar_wait(&empty_bar[s], ((kb / STAGES) - 1) & 1)) {
            atomicExch(status, 11);
            ok = false;
            break;
          }
          unsigned char* a_tile = smem + (size_t)s * TcSmem<BN>::stage_bytes;
          unsigned char* b_tile = a_tile + TcSmem<BN>::a_bytes;
          mbar_expect_tx(&full_bar[s], TcSmem<BN>::stage_bytes);
          tma_load_2d(a_tile, &map_a, &full_bar[s], it * TC_BK, m0);
          if (EPI == TC_SILU_MUL) {
            tma_load_2d(b_tile, &map_w, &full_bar[s], it * TC_BK, n0);
            tma_load_2d(b_tile + TcSmem<BN>::b_bytes / 2, &map_w, &full_bar[s], it * TC_BK, up_row_offset + n0);
          } else {
            tma_load_2d(b_tile, &map_w, &full_bar[s], it * TC_BK, n0);
          }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc(TC_BM, BN);
      int kb = 0, tc = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tc) {
        const int buf = tc & 1;
        // the epilogue warps must have read this accumulator's previous tile
        if (tc >= 2 && !mbar_wait(&acc_empty[buf], ((tc >> 1) - 1) & 1)) {
          atomicExch(status, 14);
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t tmem_acc = tmem_base + (uint32_t)buf * ACC_COLS;
        for (int it = 0; it < k_iters; ++it, ++kb) {
          const int s = kb % STAGES;
          if (!mbar_wait(&full_bar[s], (kb / STAGES) & 1)) {
            atomicExch(status, 12);
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const unsigned char* a_tile = smem + (size_t)s * TcSmem<BN>::stage_bytes;
          const unsigned char* b_tile = a_tile + TcSmem<BN>::a_bytes;
          const uint64_t da = make_smem_desc(a_tile), db = make_smem_desc(b_tile);
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k) umma_bf16(tmem_acc, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (it | k) != 0);
          umma_commit(&empty_bar[s]);
        }
        if (ok) umma_commit(&acc_full[buf]);
      }
    }
  } else {
    // epilogue warps 2..5: warp w may touch tensor-memory lanes 32 * (w % 4) .. + 31
    const int quad = warp & 3;
    int tc = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tc) {
      const int buf = tc & 1;
      const int n0 = (tile % n_tiles) * COLS, m0 = (tile / n_tiles) * TC_BM;
      const int row = m0 + quad * 32 + lane;
      if (!mbar_wait(&acc_full[buf], (tc >> 1) & 1)) {
        atomicExch(status, 13);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const uint32_t lane_addr = tmem_base + (uint32_t)buf * ACC_COLS + ((uint32_t)(quad * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < COLS; c += 32) {
        uint32_t acc[32];
        tmem_ld32(lane_addr + (uint32_t)c, acc);
        if constexpr (EPI == TC_SILU_MUL) {
          uint32_t up[32];
          tmem_ld32(lane_addr + (uint32_t)(COLS + c), up);
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
          if (row < M) store_chunk<EPI>(out, acc, up, row, n0 + c, N_out);
        } else {
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
          if (row < M) store_chunk<EPI>(out, acc, acc, row, n0 + c, N_out);
        }
      }
      // this accumulator may be overwritten by the tile after the next
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      mbar_arrive(&acc_empty[buf]);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(2 * ACC_COLS) : "memory");
  }
}

// ---------------------------------------------------------------- two CTAs per tile (cta_group::2)
// A pair of CTAs (a cluster of two, on neighbouring SMs) computes one 256 x 256 tile: each CTA
// loads its own 128 rows of A and 128 of the tile's 256 rows of W, the tensor cores of both read
// both halves of W (the peer's through distributed shared memory), and each accumulates its own
// 128 x 256 half in its own tensor memory. An SM thus stages 32 KB per k-block of 64 instead of
// 48 KB for the same products. The first CTA of the pair issues the products for both and owns
// the "stage is full" barriers, which the TMA copies of both CTAs report to; "stage is empty"
// and "accumulator is full" reach both CTAs at once (tcgen05.commit with a cluster mask).
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// TMA copy whose bytes are reported to the barrier of the pair's first CTA (address bit 24 cleared)
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar) & 0xFEFFFFFFu), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u;
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
}
// arrives on this barrier in both CTAs of the pair when the products issued so far are done
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
               ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}
// arrive on the same barrier in the pair's first CTA
__device__ __forceinline__ void mbar_arrive_first_cta(uint64_t* bar) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(smem_u32(bar)), "r"(0u));
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(remote) : "memory");
}

// ---------------------------------------------------------------- decode products with a long k
// out[M, N] = X[M, K] W[N, K]^T for a handful of tokens (M <= 64), with the operands swapped: 128 rows
// of W are the instruction's M, the tokens its N (16, 32 or 64 columns of tensor memory). Such a
// product is a stream of weights; here TMA keeps it coming, eight to eleven stages of 16 KB per CTA in
// flight (some 180 KB a CTA against the 32 KB of registers a CTA of gemm_skinny.cu has in flight), and
// one thread issues the products. K is cut into slices, the CTAs of a thread-block cluster (along x),
// so that a narrow output still gives every SM a CTA; their partial sums meet in shared memory,
// every CTA of the cluster adding up the tokens that fall to it, in the order of the slices.
// The weights of the first stages are asked for before the wait on the kernels launched earlier
// (they do not depend on them), the activations after it.
template <int BT, int STAGES>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_decode_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                      __nv_bfloat16* __restrict__ out, int M, int N, int K, int slices, int iters_per_slice,
                      int* __restrict__ status) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], accum_bar;
  __shared__ uint32_t tmem_base_slot;
  constexpr int W_BYTES = TC_BM * TC_BK * 2, X_BYTES = BT * TC_BK * 2, STAGE_BYTES = W_BYTES + X_BYTES;
  constexpr uint32_t TMEM_COLS = BT <= 32 ? 32 : 64;
  float* part = reinterpret_cast<float*>(smem + (size_t)STAGES * STAGE_BYTES);  // [BT tokens][128 rows of W]: this slice's sums

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = (int)cluster_ctarank();
  const int n0 = ((int)blockIdx.x / slices) * TC_BM;
  const int k_iters = (K + TC_BK - 1) / TC_BK;
  const int it0 = min(k_iters, rank * iters_per_slice), n_it = min(k_iters, it0 + iters_per_slice) - it0;

  // Thread 0 is the producer. It sets the barriers up and asks for the weights of the first stages at
  // once, before tensor memory is allocated and before the wait on the kernels launched earlier: the
  // weights depend on neither.
  const int ahead = min(n_it, STAGES);
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&accum_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    for (int i = 0; i < ahead; ++i) {
      mbar_expect_tx(&full_bar[i], STAGE_BYTES);
      tma_load_2d(smem + (size_t)i * STAGE_BYTES, &map_w, &full_bar[i], (it0 + i) * TC_BK, n0);
    }
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;
  pdl_launch_dependents();

  if (warp == 0) {
    if (threadIdx.x == 0) {
      pdl_wait();
      for (int i = 0; i < ahead; ++i) tma_load_2d(smem + (size_t)i * STAGE_BYTES + W_BYTES, &map_x, &full_bar[i], (it0 + i) * TC_BK, 0);
      for (int i = ahead; i < n_it; ++i) {
        const int s = i % STAGES;
        if (!mbar_wait(&empty_bar[s], ((i / STAGES) - 1) & 1)) {
          atomicExch(status, 16);
          break;
        }
        mbar_expect_tx(&full_bar[s], STAGE_BYTES);
        tma_load_2d(smem + (size_t)s * STAGE_BYTES, &map_w, &full_bar[s], (it0 + i) * TC_BK, n0);
        tma_load_2d(smem + (size_t)s * STAGE_BYTES + W_BYTES, &map_x, &full_bar[s], (it0 + i) * TC_BK, 0);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc(TC_BM, BT);
      for (int i = 0; i < n_it; ++i) {
        const int s = i % STAGES;
        if (!mbar_wait(&full_bar[s], (i / STAGES) & 1)) {
          atomicExch(status, 17);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const unsigned char* w_tile = smem + (size_t)s * STAGE_BYTES;
        const uint64_t da = make_smem_desc(w_tile), db = make_smem_desc(w_tile + W_BYTES);
#pragma unroll
        for (int k = 0; k < TC_BK / 16; ++k) umma_bf16(tmem_base, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (i | k) != 0);
        umma_commit(&empty_bar[s]);
      }
      umma_commit(&accum_bar);
    }
  } else {
    // warps 2..5: warp w may touch tensor-memory lanes 32 * (w % 4) .. + 31, i.e. rows of W
    pdl_wait();
    const int quad = warp & 3, l = quad * 32 + lane;
    bool ok = true;
    if (n_it > 0) {
      ok = mbar_wait(&accum_bar, 0);
      if (!ok) atomicExch(status, 18);
    }
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
#pragma unroll 1
    for (int c = 0; c < BT; c += 32) {
      uint32_t acc[32];
      if (n_it > 0 && ok) {
        tmem_ld32(lane_addr + (uint32_t)c, acc);
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = 0u;
      }
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (c + j < BT) part[(c + j) * TC_BM + l] = __uint_as_float(acc[j]);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  cluster_sync_all();  // every slice's sums are in its shared memory
  if (warp >= 2) {
    const int l = (warp & 3) * 32 + lane;
    if (n0 + l < N) {
      // the tokens rank, rank + slices, ...: all slices' sums of a token are asked for together (eight
      // loads from the cluster's shared memory in flight), then added in the order of the slices
      uint32_t peer[8];
#pragma unroll
      for (int sl = 0; sl < 8; ++sl)
        asm("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(peer[sl]) : "r"(smem_u32(part + l)), "r"((uint32_t)(sl < slices ? sl : 0)));
      for (int tok = rank; tok < M; tok += slices) {
        float v[8];
#pragma unroll
        for (int sl = 0; sl < 8; ++sl) {
          v[sl] = 0.f;
          if (sl < slices) asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v[sl]) : "r"(peer[sl] + (uint32_t)(tok * TC_BM * 4)));
        }
        float sum = 0.f;
#pragma unroll
        for (int sl = 0; sl < 8; ++sl) sum += v[sl];
        out[(size_t)tok * N + n0 + l] = __float2bfloat16_rn(sum);
      }
    }
  }
  cluster_sync_all();  // nobody's shared memory goes away while another CTA may still read it
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// AND of a flag over the 128 threads of a group of epilogue warps (hardware barrier `id`), and their plain barrier
__device__ __forceinline__ bool epilogue_all(int id, bool flag) {
  uint32_t res;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %2, 0;\n\t"
      "bar.red.and.pred q, %1, 128, p;\n\tselp.u32 %0, 1, 0, q;\n\t}\n"
      : "=r"(res) : "r"(id), "r"((uint32_t)flag) : "memory");
  return res != 0;
}
__device__ __forceinline__ void epilogue_sync(int id) { asm volatile("bar.sync %0, 128;\n" ::"r"(id) : "memory"); }

// The q|k|v epilogue's ring for the rotation table: four slots of [128 tokens][8 cosines] then
// [128 tokens][8 sines] (float32), one quarter of a half head each, read by both groups of epilogue warps
// (a tile's two heads are of one kind and of the same tokens).
constexpr int CS_SLOTS = 4;
constexpr int CS_SLOT_BYTES = 2 * TC_BM * 8 * 4;
constexpr int CS_RING_BYTES = CS_SLOTS * CS_SLOT_BYTES;  // 32 KB
// `bytes` contiguous bytes (a multiple of 16, both addresses 16-byte aligned) from global to this CTA's shared memory
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

constexpr int PAIR_THREADS = 320;  // TMA warp, MMA warp, eight epilogue warps
constexpr int PAIR_BN = 256;                    // the wide tile; outputs too narrow for it take 128 columns
constexpr int PAIR_OUT_BYTES = TC_BM * 64 * 2;  // one [128][64] bfloat16 tile of the epilogue's four
// per CTA and stage: 128 rows of A and half of the tile's BN rows of W, 64 k each
__host__ __device__ constexpr int pair_stage_bytes(int bn) { return (TC_BM + bn / 2) * TC_BK * 2; }

template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(PAIR_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_out, void* __restrict__ out,
                    int M, int N_out, int K, int up_row_offset, int* __restrict__ status, const QkvEpilogue qe) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int row_dst[2][TC_BM];  // TC_QKV_ROPE: the pool row (page, kv head, slot) each row of a k or v head goes to (-1: none)
  __shared__ uint64_t cs_full[CS_SLOTS], cs_empty[CS_SLOTS];  // TC_QKV_ROPE: a slot of the cos/sin ring has landed / has been read by all eight warps
  constexpr int COLS = EPI == TC_SILU_MUL ? BN / 2 : BN;  // output columns per tile
  constexpr int STAGE_BYTES = pair_stage_bytes(BN);
  constexpr uint32_t TMEM_COLS = 2 * BN;             // two accumulators (512 or 256 columns)
  constexpr int A_BYTES = TC_BM * TC_BK * 2;

  unsigned char* smem_cs = smem + (size_t)STAGES * STAGE_BYTES + 4 * PAIR_OUT_BYTES;  // TC_QKV_ROPE only
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0: the CTA that issues the products
  const int k_iters = (K + TC_BK - 1) / TC_BK;
  const int n_tiles = (N_out + COLS - 1) / COLS, m_tiles = (M + 2 * TC_BM - 1) / (2 * TC_BM);
  const int num_tiles = n_tiles * m_tiles;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  // Tiles that run at the same time share the larger operand: with fewer rows in A than in W the
  // row tiles change fastest, so that a tile of W is fetched from memory once and serves every row
  // tile while it is in L2 (24,576 x 4,096 weights do not fit L2; walking them once per row tile
  // took 339 us against the library's 271 for 2,048 rows).
  const bool m_fastest = M <= N_out;
  auto tile_m = [&](int tile) { return m_fastest ? tile % m_tiles : tile / n_tiles; };
  auto tile_n = [&](int tile) { return m_fastest ? tile / m_tiles : tile % n_tiles; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 16);  // one arrival per epilogue warp of both CTAs
    }
    for (int i = 0; i < CS_SLOTS; ++i) {
      mbar_init(&cs_full[i], 1);
      mbar_init(&cs_empty[i], 8);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything is reported to them
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;

  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    if (elect_one()) {
      int kb = 0;
      for (int tile = pair; tile < num_tiles; tile += num_pairs) {
        const int n0 = tile_n(tile) * COLS, m0 = tile_m(tile) * 2 * TC_BM + (int)rank * TC_BM;
        // this CTA's 128 of the tile's 256 rows of W: for SiLU * up the first CTA brings the gate rows, the second the up rows
        const int w_row = EPI == TC_SILU_MUL ? (rank == 0 ? n0 : up_row_offset + n0) : n0 + (int)rank * (BN / 2);
        bool ok = true;
        for (int it = 0; it < k_iters; ++it, ++kb) {
          const int s = kb % STAGES;
          if (kb >= STAGES && !mbar_wait(&empty_bar[s], ((kb / STAGES) - 1) & 1)) {
            atomicExch(status, 11);
            ok = false;
            break;
          }
          unsigned char* a_tile = smem + (size_t)s * STAGE_BYTES;
          if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * STAGE_BYTES);  // both CTAs' bytes
          tma_load_2d_pair(a_tile, &map_a, &full_bar[s], it * TC_BK, m0);
          tma_load_2d_pair(a_tile + A_BYTES, &map_w, &full_bar[s], it * TC_BK, w_row);
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    if (rank == 0 && elect_one()) {
      constexpr uint32_t idesc = make_idesc(2 * TC_BM, BN);
      int kb = 0, tc = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++tc) {
        const int buf = tc & 1;
        if (tc >= 2 && !mbar_wait(&acc_empty[buf], ((tc >> 1) - 1) & 1)) {
          atomicExch(status, 14);
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t tmem_acc = tmem_base + (uint32_t)buf * BN;
        for (int it = 0; it < k_iters; ++it, ++kb) {
          const int s = kb % STAGES;
          if (!mbar_wait(&full_bar[s], (kb / STAGES) & 1)) {
            atomicExch(status, 12);
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const unsigned char* a_tile = smem + (size_t)s * STAGE_BYTES;
          const uint64_t da = make_smem_desc(a_tile), db = make_smem_desc(a_tile + A_BYTES);
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k) umma_bf16_pair(tmem_acc, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (it | k) != 0);
          umma_commit_pair(&empty_bar[s]);
        }
        if (ok) umma_commit_pair(&acc_full[buf]);
      }
    }
  } else {
    // eight epilogue warps in two groups of four; a group's warps cover the 128 lanes of tensor
    // memory (warp w may touch lanes 32 * (w % 4) .. + 31) and the groups share out the columns
    const int quad = warp & 3, eg = (warp - 2) >> 2;
    const bool issuer = (int)threadIdx.x == 64 + 128 * eg;
    int tc = 0, out_buf = 0;
    uint32_t cs_count = 0;  // TC_QKV_ROPE: quarters of the cos/sin table that have been through the ring before this tile
    const bool tma_out = EPI != TC_OUT_F32 && EPI != TC_QKV_ROPE && N_out % 8 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++tc) {
      const int buf = tc & 1;
      const int n0 = tile_n(tile) * COLS, m0 = tile_m(tile) * 2 * TC_BM + (int)rank * TC_BM;
      const int row = m0 + quad * 32 + lane;
      // TC_QKV_ROPE: the rotation's cosines and sines of the tile's 128 tokens come through a ring of four
      // slots filled by bulk copies, a quarter of a half head (8 pairs) per slot, asked for four quarters
      // ahead by the first thread of the first group. Every thread reads its token's 32 + 32 bytes of a
      // slot. Read from a [T, 128] table in global memory instead (512 bytes apart from thread to thread)
      // the same values took 3 to 7 us of a tile's epilogue, more than the tile's products; fetched from
      // that table by TMA in boxes of 128 x 32 bytes still 2 to 5 us (a request per token and box).
      bool qkv_rotated = false;
      const bool cs_producer = issuer && eg == 0;
      auto cs_issue = [&](uint32_t fill, int quarter) {  // the producer thread only
        const uint32_t slot = fill % CS_SLOTS;
        if (fill >= CS_SLOTS && !mbar_wait(&cs_empty[slot], ((fill / CS_SLOTS) - 1) & 1u)) atomicExch(status, 15);
        mbar_expect_tx(&cs_full[slot], CS_SLOT_BYTES);
        // the table is laid out by tiles of 128 tokens and quarters, so a slot's worth is one contiguous block
        bulk_load(smem_cs + (size_t)slot * CS_SLOT_BYTES, qe.cos_sin + ((size_t)(m0 / TC_BM) * 8 + quarter) * (CS_SLOT_BYTES / 4),
                  CS_SLOT_BYTES, &cs_full[slot]);
      };
      if constexpr (EPI == TC_QKV_ROPE) {
        qkv_rotated = qe.cos_sin != nullptr && n0 / 128 < qe.nq + qe.nkv;  // q and k heads; the same for both groups
        if (qkv_rotated && cs_producer) {
          for (int ahead = 0; ahead < CS_SLOTS; ++ahead) cs_issue(cs_count + ahead, ahead);  // before the accumulator is waited for
        }
      }
      // the four epilogue warps go on together or stop together (they meet at barriers below)
      if (!epilogue_all(1 + eg, mbar_wait(&acc_full[buf], (tc >> 1) & 1))) {
        atomicExch(status, 13);
        if (qkv_rotated && cs_producer) {
          // what was asked for above must have landed before this CTA's shared memory may go away
          for (int ahead = 0; ahead < CS_SLOTS; ++ahead) mbar_wait(&cs_full[(cs_count + ahead) % CS_SLOTS], ((cs_count + ahead) / CS_SLOTS) & 1u);
        }
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const uint32_t lane_addr = tmem_base + (uint32_t)buf * BN + ((uint32_t)(quad * 32) << 16);
      if constexpr (EPI == TC_QKV_ROPE) {
        // A tile's 256 columns are two whole heads; each group of warps takes one. A thread owns a
        // token's row of its head: it reads the 128 values from tensor memory once, keeps them as 64
        // pairs of bfloat16 (the product is rounded to bfloat16 first, as when it is stored) and
        // gives the accumulator back at once; then it normalises and rotates from registers, puts
        // the result into the group's two swizzled [128][64] tiles, and the tiles leave by TMA (q) or
        // by row copies into the token's cache page (k, v). Reads of tensor memory are slow while
        // the next tile's products run (0.6 us for the 128 columns with the tensor cores idle, 1.7 busy).
        const int r = quad * 32 + lane, tok = m0 + r;
        const int head = n0 / 128 + eg;
        const bool is_q = head < qe.nq, is_v = head >= qe.nq + qe.nkv;
        const __nv_bfloat16* nw = is_v ? nullptr : (is_q ? qe.q_norm_w : qe.k_norm_w);
        const uint32_t head_addr = lane_addr + (uint32_t)(128 * eg);
        unsigned char* stage_lo = smem + (size_t)STAGES * STAGE_BYTES + (size_t)(2 * eg) * PAIR_OUT_BYTES;
        unsigned char* stage_hi = stage_lo + PAIR_OUT_BYTES;
        uint32_t packed[64];  // elements 2 i and 2 i + 1 of the head
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t acc[32];
          tmem_ld32(head_addr + (uint32_t)(32 * c), acc);
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const __nv_bfloat162 p = __floats2bfloat162_rn(__uint_as_float(acc[i]), __uint_as_float(acc[i + 1]));
            const uint32_t u = *reinterpret_cast<const uint32_t*>(&p);
            const float x0 = __uint_as_float(u << 16), x1 = __uint_as_float(u & 0xFFFF0000u);
            ss += x0 * x0;
            ss += x1 * x1;
            packed[16 * c + (i >> 1)] = u;
          }
        }
        // the accumulator is free for the tile after the next one
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive_first_cta(&acc_empty[buf]);
        const float inv = nw ? 1.0f / sqrtf(ss / 128.f + qe.eps) : 1.f;
        if (issuer) asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");  // the stores of the tile before have read both tiles
        epilogue_sync(1 + eg);
        bool cs_ok = true;
#pragma unroll
        for (int qi = 0; qi < 8; ++qi) {  // eight rotation pairs at a time: elements 8 qi .. + 7 of the head's first half, and of its second
          float l[8], h[8];
#pragma unroll
          for (int e = 0; e < 8; e += 2) {
            const uint32_t ul = packed[(8 * qi + e) >> 1], uh = packed[(64 + 8 * qi + e) >> 1];
            l[e] = __uint_as_float(ul << 16);
            l[e + 1] = __uint_as_float(ul & 0xFFFF0000u);
            h[e] = __uint_as_float(uh << 16);
            h[e + 1] = __uint_as_float(uh & 0xFFFF0000u);
          }
          if (nw) {
            float wl[8], wh[8];
            bf16x8_to_float(*reinterpret_cast<const uint4*>(nw + 8 * qi), wl);
            bf16x8_to_float(*reinterpret_cast<const uint4*>(nw + 64 + 8 * qi), wh);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              l[e] = (l[e] * inv) * wl[e];
              h[e] = (h[e] * inv) * wh[e];
            }
          }
          float cs[8] = {1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f}, sn[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          if (qkv_rotated) {
            const uint32_t fill = cs_count + (uint32_t)qi, slot = fill % CS_SLOTS;
            cs_ok = cs_ok && mbar_wait(&cs_full[slot], (fill / CS_SLOTS) & 1u);
            const float4* mine = reinterpret_cast<const float4*>(smem_cs + (size_t)slot * CS_SLOT_BYTES + r * 32);
            const float4 c0 = mine[0], c1 = mine[1], s0 = mine[CS_SLOT_BYTES / 32], s1 = mine[CS_SLOT_BYTES / 32 + 1];
            cs[0] = c0.x; cs[1] = c0.y; cs[2] = c0.z; cs[3] = c0.w; cs[4] = c1.x; cs[5] = c1.y; cs[6] = c1.z; cs[7] = c1.w;
            sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
            // this warp has its values; when all eight warps have, the slot takes the quarter four further on
            __syncwarp();
            if (lane == 0) mbar_arrive(&cs_empty[slot]);
            if (cs_producer && qi + CS_SLOTS < 8) cs_issue(fill + CS_SLOTS, qi + CS_SLOTS);
          }
          float ol[8], oh[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            ol[e] = l[e] * cs[e] - h[e] * sn[e];
            oh[e] = h[e] * cs[e] + l[e] * sn[e];
          }
          *reinterpret_cast<uint4*>(stage_lo + r * 128 + ((qi ^ (r & 7)) << 4)) = float_to_bf16x8(ol);
          *reinterpret_cast<uint4*>(stage_hi + r * 128 + ((qi ^ (r & 7)) << 4)) = float_to_bf16x8(oh);
        }
        if (qkv_rotated) cs_count += 8;
        if (!cs_ok) atomicExch(status, 15);
        if (!is_q) {
          // where this token's row of the head goes in the pool
          int dst = -1;
          if (tok < M) {
            const int pos = qe.positions[tok];
            const int page = qe.page_indices[qe.page_indptr[qe.row_of_token[tok]] + (pos >> qe.page_shift)];
            if (page < 0) {
              atomicExch(status, 2);
            } else {
              const int kvh = head - qe.nq - (is_v ? qe.nkv : 0);
              dst = ((page * qe.nkv + kvh) << qe.page_shift) + (pos & ((1 << qe.page_shift) - 1));
            }
          }
          row_dst[eg][r] = dst;
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        epilogue_sync(1 + eg);
        if (is_q) {
          if (issuer) {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];\n"
                         ::"l"(&map_out), "r"(smem_u32(stage_lo)), "r"(head * 128), "r"(m0) : "memory");
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];\n"
                         ::"l"(&map_out), "r"(smem_u32(stage_hi)), "r"(head * 128 + 64), "r"(m0) : "memory");
            asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
          }
        } else {
          // two rows per warp and trip: 16 lanes copy a row's 256 bytes (8 chunks from each tile) in whole lines
          __nv_bfloat16* pool = is_v ? qe.v_pool : qe.k_pool;
          const int sub = lane & 15, c = sub & 7;
          const unsigned char* from = sub < 8 ? stage_lo : stage_hi;
#pragma unroll 4
          for (int trip = 0; trip < 16; ++trip) {
            const int rr = quad * 32 + 2 * trip + (lane >> 4);
            const int dst = row_dst[eg][rr];
            if (dst >= 0)
              *reinterpret_cast<uint4*>(pool + (size_t)dst * 128 + (sub >> 3) * 64 + c * 8) = *reinterpret_cast<const uint4*>(from + rr * 128 + ((c ^ (rr & 7)) << 4));
          }
        }
      } else if constexpr (EPI == TC_OUT_F32) {
#pragma unroll 1
        for (int c = 32 * eg; c < COLS; c += 64) {
          uint32_t acc[32];
          tmem_ld32(lane_addr + (uint32_t)c, acc);
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
          if (row < M) store_chunk<EPI>(out, acc, acc, row, n0 + c, N_out);
        }
      } else if (!tma_out) {
#pragma unroll 1
        for (int c = 32 * eg; c < COLS; c += 64) {
          uint32_t acc[32];
          tmem_ld32(lane_addr + (uint32_t)c, acc);
          if constexpr (EPI == TC_SILU_MUL) {
            uint32_t up[32];
            tmem_ld32(lane_addr + (uint32_t)(COLS + c), up);
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            if (row < M) store_chunk<EPI>(out, acc, up, row, n0 + c, N_out);
          } else {
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            if (row < M) store_chunk<EPI>(out, acc, acc, row, n0 + c, N_out);
          }
        }
      } else {
        // bfloat16 out: 64 columns at a time go through a swizzled shared-memory tile [128][64] and
        // leave with one TMA store, which writes whole lines and clips at the matrix's edge; each
        // group of warps has two such tiles that take turns, so that a store is still reading one
        // while the next is being filled
        const int r = quad * 32 + lane;
#pragma unroll 1
        for (int cb = 64 * eg; cb < COLS; cb += 128) {
          unsigned char* stage_out = smem + (size_t)STAGES * STAGE_BYTES + (size_t)(2 * eg + out_buf) * PAIR_OUT_BYTES;
          if (issuer) asm volatile("cp.async.bulk.wait_group.read 1;\n" ::: "memory");  // this tile's last store has read it
          epilogue_sync(1 + eg);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t acc[32];
            float v[32];
            tmem_ld32(lane_addr + (uint32_t)(cb + 32 * h), acc);
            if constexpr (EPI == TC_SILU_MUL) {
              uint32_t up[32];
              tmem_ld32(lane_addr + (uint32_t)(COLS + cb + 32 * h), up);
              asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
              for (int q = 0; q < 32; ++q) {
                const float x = __uint_as_float(acc[q]);
                v[q] = silu_fast(x) * __uint_as_float(up[q]);
              }
            } else {
              asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
              for (int q = 0; q < 32; ++q) v[q] = __uint_as_float(acc[q]);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 pk;
              __nv_bfloat162 p0 = __floats2bfloat162_rn(v[8 * q], v[8 * q + 1]), p1 = __floats2bfloat162_rn(v[8 * q + 2], v[8 * q + 3]);
              __nv_bfloat162 p2 = __floats2bfloat162_rn(v[8 * q + 4], v[8 * q + 5]), p3 = __floats2bfloat162_rn(v[8 * q + 6], v[8 * q + 7]);
              pk.x = *reinterpret_cast<uint32_t*>(&p0);
              pk.y = *reinterpret_cast<uint32_t*>(&p1);
              pk.z = *reinterpret_cast<uint32_t*>(&p2);
              pk.w = *reinterpret_cast<uint32_t*>(&p3);
              const int chunk = 4 * h + q;  // 16-byte chunk of the 128-byte row; the swizzle XORs it with the row
              *reinterpret_cast<uint4*>(stage_out + r * 128 + ((chunk ^ (r & 7)) << 4)) = pk;
            }
          }
          asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
          epilogue_sync(1 + eg);
          if (issuer) {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];\n"
                         ::"l"(&map_out), "r"(smem_u32(stage_out)), "r"(n0 + cb), "r"(m0) : "memory");
            asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
          }
          out_buf ^= 1;
        }
      }
      if constexpr (EPI != TC_QKV_ROPE) {  // (that epilogue has given the accumulator back already)
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive_first_cta(&acc_empty[buf]);
      }
    }
    if (issuer) asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory");  // every store has landed
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  cluster_sync_all();  // neither CTA's shared or tensor memory goes away while the other may still use it
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------- host side
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int get_encode(EncodeFn* out) {
  static EncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    MS_CHECK_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres));
    MS_CHECK_ARG(ptr != nullptr && qres == cudaDriverEntryPointSuccess, "gemm_tc: the driver has no cuTensorMapEncodeTiled");
    fn = reinterpret_cast<EncodeFn>(ptr);
  }
  *out = fn;
  return 0;
}

// A 2-D bfloat16 tensor [rows, cols] (cols contiguous), boxes of box_rows x 64 columns, 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows) {
  EncodeFn encode;
  if (int rc = get_encode(&encode)) return rc;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult res = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  MS_CHECK_ARG(res == CUDA_SUCCESS, "gemm_tc: cuTensorMapEncodeTiled failed with code %d (rows=%lld cols=%lld)", (int)res, rows, cols);
  return 0;
}

template <int BN, int STAGES, int EPI>
static int launch_tc(void* out, const void* A, const void* W, int M, int N_out, int w_rows, int K, int up_row_offset,
                     int* status, cudaStream_t stream) {
  CUtensorMap map_a, map_w;
  if (int rc = make_map(&map_a, A, M, K, TC_BM)) return rc;
  if (int rc = make_map(&map_w, W, w_rows, K, EPI == TC_SILU_MUL ? BN / 2 : BN)) return rc;
  constexpr size_t smem = (size_t)STAGES * TcSmem<BN>::stage_bytes + 1024;
  auto kernel = gemm_tc_kernel<BN, STAGES, EPI>;
  static bool configured = false;
  if (!configured) {
    MS_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  constexpr int COLS = EPI == TC_SILU_MUL ? BN / 2 : BN;
  dim3 grid(ceil_div(N_out, COLS), ceil_div(M, TC_BM));
  MS_LAUNCH(kernel, grid, TC_THREADS, smem, stream, map_a, map_w, out, M, N_out, K, up_row_offset, status);
  return 0;
}

template <int BN, int STAGES, int EPI>
static int launch_tc_persistent(void* out, const void* A, const void* W, int M, int N_out, int w_rows, int K, int up_row_offset,
                                int* status, cudaStream_t stream) {
  CUtensorMap map_a, map_w;
  if (int rc = make_map(&map_a, A, M, K, TC_BM)) return rc;
  if (int rc = make_map(&map_w, W, w_rows, K, EPI == TC_SILU_MUL ? BN / 2 : BN)) return rc;
  constexpr size_t smem = (size_t)STAGES * TcSmem<BN>::stage_bytes + 1024;
  static_assert(smem <= 227 * 1024, "the ring does not fit shared memory");
  auto kernel = gemm_tc_persistent_kernel<BN, STAGES, EPI>;
  static bool configured = false;
  static int sm_count = 0;
  if (!configured) {
    MS_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int dev = 0;
    MS_CHECK_CUDA(cudaGetDevice(&dev));
    MS_CHECK_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
    configured = true;
  }
  constexpr int COLS = EPI == TC_SILU_MUL ? BN / 2 : BN;
  const long long tiles = (long long)ceil_div(N_out, COLS) * ceil_div(M, TC_BM);
  MS_CHECK_ARG(tiles < (1LL << 30), "gemm_tc: too many tiles (%lld)", tiles);
  const unsigned grid = (unsigned)(tiles < sm_count ? tiles : sm_count);
  MS_LAUNCH(kernel, grid, TC_THREADS, smem, stream, map_a, map_w, out, M, N_out, K, up_row_offset, status);
  return 0;
}

template <int BN, int STAGES, int EPI>
static int launch_tc_pair(void* out, const void* A, const void* W, int M, int N_out, int w_rows, int K, int up_row_offset,
                          int* status, cudaStream_t stream, const QkvEpilogue& qe = QkvEpilogue{}) {
  CUtensorMap map_a, map_w, map_out;
  if (int rc = make_map(&map_a, A, M, K, TC_BM)) return rc;
  if (int rc = make_map(&map_w, W, w_rows, K, BN / 2)) return rc;
  map_out = map_a;  // a valid map also when the kernel does not store through it (float32 out, odd widths)
  if (EPI == TC_QKV_ROPE) {
    if (int rc = make_map(&map_out, out, M, (long long)qe.nq * 128, TC_BM)) return rc;  // q alone goes out through it
  } else if (EPI != TC_OUT_F32 && N_out % 8 == 0 && (uintptr_t)out % 16 == 0) {
    if (int rc = make_map(&map_out, out, M, N_out, TC_BM)) return rc;
  }
  constexpr size_t smem = (size_t)STAGES * pair_stage_bytes(BN) + 4 * PAIR_OUT_BYTES + (EPI == TC_QKV_ROPE ? CS_RING_BYTES : 0) + 1024;
  static_assert(smem <= 227 * 1024, "the ring does not fit shared memory");
  auto kernel = gemm_tc_pair_kernel<BN, STAGES, EPI>;
  static bool configured = false;
  static int sm_count = 0;
  if (!configured) {
    MS_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int dev = 0;
    MS_CHECK_CUDA(cudaGetDevice(&dev));
    MS_CHECK_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
    configured = true;
  }
  constexpr int COLS = EPI == TC_SILU_MUL ? BN / 2 : BN;
  const long long tiles = (long long)ceil_div(N_out, COLS) * ceil_div(M, 2 * TC_BM);
  MS_CHECK_ARG(tiles < (1LL << 30), "gemm_tc: too many tiles (%lld)", tiles);
  const long long pairs = tiles < sm_count / 2 ? tiles : sm_count / 2;
  MS_LAUNCH_CLUSTERED(kernel, (unsigned)(2 * pairs), PAIR_THREADS, smem, stream, 2, map_a, map_w, map_out, out, M, N_out, K,
                      up_row_offset, status, qe);
  return 0;
}

template <int BT, int STAGES>
static int launch_tc_decode(void* out, const void* X, const void* W, int M, int N, int K, int* status, cudaStream_t stream) {
  CUtensorMap map_w, map_x;
  if (int rc = make_map(&map_w, W, N, K, TC_BM)) return rc;
  if (int rc = make_map(&map_x, X, M, K, BT)) return rc;
  constexpr size_t smem = (size_t)STAGES * (TC_BM + BT) * TC_BK * 2 + (size_t)BT * TC_BM * 4 + 1024;
  static_assert(smem <= 227 * 1024, "the ring does not fit shared memory");
  auto kernel = gemm_tc_decode_kernel<BT, STAGES>;
  static bool configured = false;
  static int sm_count = 0;
  if (!configured) {
    MS_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int dev = 0;
    MS_CHECK_CUDA(cudaGetDevice(&dev));
    MS_CHECK_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
    configured = true;
  }
  // Slices of k: as many as still let every cluster be resident at once (clusters are placed within a
  // group of SMs, so fewer fit than SMs / size), each of at least four k-blocks, at most eight.
  static int fit[9] = {0};  // how many clusters of each size the device holds at once
  if (fit[1] == 0) {
    for (int size = 1; size <= 8; ++size) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3((unsigned)(size * sm_count));
      cfg.blockDim = dim3(TC_THREADS);
      cfg.dynamicSmemBytes = smem;
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = (unsigned)size;
      attr.val.clusterDim.y = attr.val.clusterDim.z = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) n = sm_count / size / 2;
      fit[size] = n;
    }
  }
  const int tiles = ceil_div(N, TC_BM), k_iters = ceil_div(K, TC_BK);
  int slices = 1;
  for (int size = 2; size <= 8 && size <= k_iters / 4; ++size)
    if (fit[size] >= tiles) slices = size;
  const int iters_per_slice = ceil_div(k_iters, slices);
  MS_LAUNCH_CLUSTERED(kernel, (unsigned)(tiles * slices), TC_THREADS, smem, stream, slices, map_w, map_x, (__nv_bfloat16*)out, M, N, K, slices,
                      iters_per_slice, status);
  return 0;
}

}  // namespace ms

using namespace ms;

MS_DEFINE_LAST_ERROR(ms_gemm_tc_last_error)
MS_DEFINE_PDL_SWITCH(ms_gemm_tc_set_pdl)

// epilogue 0: out bf16 [M, N]; 1: out float32 [M, N]; 2: W is [2 * N, K] (gate rows then up rows),
// out bf16 [M, N] = silu(A gate^T) * (A up^T). status: a device int the kernel raises if a wait ran out.
static int g_tc_config = 0;
// Which of the kernel's forms runs: 0 = chosen from the shape (what serving uses); the tests force each form at
// every shape: 5 = one CTA per tile, 10 / 11 = persistent with 256- / 128-column tiles, 20 / 21 = pairs of CTAs on
// 256- / 128-column tiles.
MS_EXPORT void ms_gemm_tc_set_config(int config) { g_tc_config = config; }

// 1 if this package's kernel is the faster choice for the product (measured on B200 against
// cuBLAS): bfloat16 out, at least one 256 x 256 tile for every pair of SMs, and rounds of tiles
// that are mostly full of output. Then the 2-CTA kernel runs 2048 x 4096 x 1024 in 16.0 us
// (cuBLAS 16.3), 2048 x 6144 x 1024 in 21.5 (22.8), 2048 x 24576 x 4096 in 261 (272) and
// 8192 x 4096 x 4096 in 167 (180). A narrow output (2048 x 1024: 32 tiles) leaves SMs idle and
// the library's smaller tiles win (14.2 against 8.9 us), as they do for 1,000 rows (4 row tiles,
// the last a quarter full: 56 against 42 us at 6144 x 4096).
MS_EXPORT int ms_gemm_tc_prefers(int M, int N, int K, int epilogue) {
  int dev = 0, sm_count = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  if (epilogue == TC_OUT_F32 || K % 8 != 0 || N % 8 != 0) return 0;
  // SiLU * up: a tile's 256 columns are 128 gate and 128 up columns, i.e. 128 columns of output; the fused
  // kernel beats the library's product followed by the activation kernel by more (28 against 34 us for
  // 2048 x 2*3072 x 1024, 261 against 295 us for 2048 x 2*12288 x 4096)
  const int cols = epilogue == TC_SILU_MUL ? PAIR_BN / 2 : PAIR_BN;
  const long long pairs = sm_count / 2, tiles = (long long)ceil_div(M, 2 * TC_BM) * ceil_div(N, cols);
  const long long rounds = (tiles + pairs - 1) / pairs;
  // the share of the tiles' area that is output, and of the rounds' slots that hold a tile
  const double useful = (double)M * N / ((double)tiles * 2 * TC_BM * cols), filled = (double)tiles / (double)(rounds * pairs);
  const double need = epilogue == TC_SILU_MUL ? 0.7 : (K > 8192 ? 0.95 : 0.8);
  // a long k with a half-empty last round: the library cuts k there and wins (145 against 130 us for 2100 x 4096 x 12288)
  return tiles >= pairs && useful * filled >= need;
}

// q_out [M, nq, 128], k_pool / v_pool [pages + 1, nkv, page_size, 128] from x [M, K] and the stacked
// weight [(nq + 2 nkv) * 128, K]: the q|k|v product with the per-head norm, the rotation and the cache
// write in its epilogue (the 2-CTA kernel). nq and nkv even, head size 128, the whole head rotated.
MS_EXPORT int ms_gemm_tc_qkv_bf16(void* q_out, const void* x, const void* w_qkv, int M, int K, int nq, int nkv, void* k_pool,
                                  void* v_pool, const void* q_norm_w, const void* k_norm_w, const float* cos_sin,
                                  const int* positions, const int* row_of_token, const int* page_indptr,
                                  const int* page_indices, int page_size, float eps, int* status, cudaStream_t stream) {
  if (M == 0) return 0;
  MS_CHECK_ARG(M > 0 && K > 0 && K % 8 == 0, "gemm_tc: bad sizes M=%d K=%d", M, K);
  MS_CHECK_ARG(nq > 0 && nkv > 0 && nq % 2 == 0 && nkv % 2 == 0, "gemm_tc: the q|k|v epilogue takes even head counts, not %d and %d", nq, nkv);
  MS_CHECK_ARG(page_size > 0 && (page_size & (page_size - 1)) == 0, "gemm_tc: page_size=%d must be a power of two", page_size);
  MS_CHECK_ARG((q_norm_w != nullptr) == (k_norm_w != nullptr), "gemm_tc: q and k are normed together or not at all");
  MS_CHECK_ARG(((uintptr_t)x % 16 == 0) && ((uintptr_t)w_qkv % 16 == 0) && ((uintptr_t)q_out % 16 == 0) && ((uintptr_t)k_pool % 16 == 0) &&
                   ((uintptr_t)v_pool % 16 == 0) && ((uintptr_t)q_norm_w % 16 == 0) && ((uintptr_t)k_norm_w % 16 == 0) &&
                   ((uintptr_t)cos_sin % 16 == 0),
               "gemm_tc: operands must be 16-byte aligned");
  MS_CHECK_ARG(status != nullptr && k_pool != nullptr && v_pool != nullptr, "gemm_tc: the q|k|v epilogue needs the pools and a status word");
  int shift = 0;
  while ((1 << shift) < page_size) ++shift;
  const QkvEpilogue qe = {(__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, (const __nv_bfloat16*)q_norm_w, (const __nv_bfloat16*)k_norm_w,
                          cos_sin, positions, row_of_token, page_indptr, page_indices, nq, nkv, shift, eps};
  const int n_total = (nq + 2 * nkv) * 128;
  return launch_tc_pair<256, 4, TC_QKV_ROPE>(q_out, x, w_qkv, M, n_total, n_total, K, 0, status, stream, qe);
}

MS_EXPORT int ms_gemm_tc_bf16(void* out, const void* A, const void* W, int M, int N, int K, int epilogue, int* status,
                              cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  MS_CHECK_ARG(M > 0 && N > 0 && K > 0, "gemm_tc: bad sizes M=%d N=%d K=%d", M, N, K);
  MS_CHECK_ARG(K % 8 == 0, "gemm_tc: K=%d must be a multiple of 8 (rows must be 16-byte multiples for TMA)", K);
  MS_CHECK_ARG(((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0), "gemm_tc: operands must be 16-byte aligned");
  MS_CHECK_ARG(status != nullptr, "gemm_tc: needs a status word");
  MS_CHECK_ARG(ceil_div(M, TC_BM) <= 65535, "gemm_tc: M=%d too large for one launch", M);
  // Enough 128 x 256 tiles to give every SM one: the persistent kernel (measured on B200: 1,366 against
  // 1,093 TFLOP/s for 8192 x 4096 x 4096, 740 against 582 for 2048 x 4096 x 1024; cuBLAS: 1,527 and
  // 1,048). Fewer: one CTA per 128 x 128 tile, which spreads a narrow output over more SMs.
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    MS_CHECK_CUDA(cudaGetDevice(&dev));
    MS_CHECK_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
  }
  const bool wide = (long long)ceil_div(M, TC_BM) * ceil_div(N, 256) >= sm_count;           // a 128 x 256 tile per SM
  const bool pairs = (long long)ceil_div(M, 2 * TC_BM) * ceil_div(N, PAIR_BN) >= sm_count / 2;  // a 256 x 256 tile per pair of SMs
  switch (epilogue) {
    case TC_OUT_BF16:
      if (g_tc_config == 5) return launch_tc<128, 5, TC_OUT_BF16>(out, A, W, M, N, N, K, 0, status, stream);
      if (g_tc_config == 10) return launch_tc_persistent<256, 4, TC_OUT_BF16>(out, A, W, M, N, N, K, 0, status, stream);
      if (g_tc_config == 11) return launch_tc_persistent<128, 6, TC_OUT_BF16>(out, A, W, M, N, N, K, 0, status, stream);
      if (g_tc_config == 21) return launch_tc_pair<128, 6, TC_OUT_BF16>(out, A, W, M, N, N, K, 0, status, stream);
      if (g_tc_config == 20 || pairs) return launch_tc_pair<256, 5, TC_OUT_BF16>(out, A, W, M, N, N, K, 0, status, stream);
      return launch_tc<128, 5, TC_OUT_BF16>(out, A, W, M, N, N, K, 0, status, stream);
    case TC_OUT_F32:
      if (g_tc_config == 5) return launch_tc<128, 5, TC_OUT_F32>(out, A, W, M, N, N, K, 0, status, stream);
      if (g_tc_config == 20) return launch_tc_pair<256, 5, TC_OUT_F32>(out, A, W, M, N, N, K, 0, status, stream);
      if (g_tc_config == 10 || wide) return launch_tc_persistent<256, 4, TC_OUT_F32>(out, A, W, M, N, N, K, 0, status, stream);
      return launch_tc<128, 5, TC_OUT_F32>(out, A, W, M, N, N, K, 0, status, stream);
    case TC_SILU_MUL:
      if (g_tc_config == 5) return launch_tc<256, 4, TC_SILU_MUL>(out, A, W, M, N, 2 * N, K, N, status, stream);
      if (g_tc_config == 10) return launch_tc_persistent<256, 4, TC_SILU_MUL>(out, A, W, M, N, 2 * N, K, N, status, stream);
      if (g_tc_config == 20 || (long long)ceil_div(M, 2 * TC_BM) * ceil_div(N, PAIR_BN / 2) >= sm_count / 2)
        return launch_tc_pair<256, 5, TC_SILU_MUL>(out, A, W, M, N, 2 * N, K, N, status, stream);
      return launch_tc_persistent<256, 4, TC_SILU_MUL>(out, A, W, M, N, 2 * N, K, N, status, stream);
    default: return fail("gemm_tc: unknown epilogue %d", epilogue);
  }
}

// out [M, N] bfloat16 = X [M, K] W [N, K]^T for M <= 64 tokens (decode steps), see gemm_tc_decode_kernel.
MS_EXPORT int ms_gemm_tc_decode_bf16(void* out, const void* X, const void* W, int M, int N, int K, int* status, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  MS_CHECK_ARG(M > 0 && M <= 64 && N > 0 && K > 0, "gemm_tc: a decode product takes 1..64 rows, not M=%d (N=%d K=%d)", M, N, K);
  MS_CHECK_ARG(K % 8 == 0, "gemm_tc: K=%d must be a multiple of 8 (rows must be 16-byte multiples for TMA)", K);
  MS_CHECK_ARG(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0), "gemm_tc: operands must be 16-byte aligned");
  MS_CHECK_ARG(status != nullptr, "gemm_tc: needs a status word");
  if (M <= 16) return launch_tc_decode<16, 11>(out, X, W, M, N, K, status, stream);
  if (M <= 32) return launch_tc_decode<32, 10>(out, X, W, M, N, K, status, stream);
  return launch_tc_decode<64, 8>(out, X, W, M, N, K, status, stream);
}
