// Causal grouped-query attention for prompts and mixed steps on the 5th-generation tensor cores,
// for head size 128 and bfloat16: S = Q K^T and O += P V are tcgen05.mma instructions with the
// accumulators in tensor memory, operands staged by TMA straight out of the paged cache.
//
// Formula as in attention_bf16.cu (miniserve/model/attention.py:60-67,125-133): a query row at
// absolute position p sees keys 0..p of its request (or the last `window`), query head h reads kv
// head h / (heads / kv_heads), softmax in float32 with scale head_dim^-0.5.
//
// One CTA owns 128 query rows: G query heads of one kv head x 128/G consecutive tokens, so that
// the G heads share every K/V tile. Roles by warp:
//   warps 0-3  softmax: thread r owns row r (tensor-memory lane r). Per key tile it reads its row
//              of S with tcgen05.ld, masks, keeps a running maximum and sum, writes P (bf16) into
//              shared memory in the tensor core's K-major swizzled layout, and rescales O in tensor
//              memory only when the maximum has grown by more than 2^8 (the stale maximum is exact
//              in the end because the same one scales the sum);
//   warp 4     one lane issues all TMA loads: Q once, then K and V tiles (128 keys) page by page
//              into a two-stage ring;
//   warp 5     allocates tensor memory; one lane issues the MMAs: S(j+1) is issued before P(j) is
//              ready so that the tensor cores work while the softmax of tile j runs.
// Every mbarrier wait is bounded; on a timeout the kernel raises the status word and winds down.
#include <cuda.h>

#include <cfloat>
#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

namespace ms {

constexpr int AT_D = 128, AT_ROWS = 128, AT_KEYS = 128;
constexpr int AT_THREADS = 192;
constexpr uint32_t AT_WAIT_LIMIT = 1u << 24;
constexpr float AT_LOG2E = 1.4426950408889634f;
constexpr int AT_BLOCK = 128 * 64 * 2;  // one [128 rows][64 bf16] swizzled block: 16 KB

__device__ __forceinline__ uint32_t at_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void at_mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(at_smem(bar)), "r"(count));
}
__device__ __forceinline__ void at_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(at_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void at_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(at_smem(bar)) : "memory");
}
__device__ __forceinline__ bool at_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = at_smem(bar);
  for (uint32_t i = 0; i < AT_WAIT_LIMIT; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void at_tma_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
      ::"r"(at_smem(dst)), "l"(map), "r"(at_smem(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void at_tma_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
      ::"r"(at_smem(dst)), "l"(map), "r"(at_smem(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ bool at_elect() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}\n" : "=r"(pred));
  return pred != 0;
}
// Shared-memory matrix descriptor, 128-byte swizzle: leading / stride byte offsets in bytes.
__device__ __forceinline__ uint64_t at_desc(const void* tile, uint32_t lbo, uint32_t sbo) {
  uint64_t d = (uint64_t)((at_smem(tile) & 0x3FFFF) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(sbo >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__device__ __forceinline__ void at_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u;
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void at_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(at_smem(bar)) : "memory");
}
__device__ __forceinline__ void at_tmem_ld32(uint32_t taddr, float (&r)[32]) {
  uint32_t* u = reinterpret_cast<uint32_t*>(r);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
        "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]), "=r"(u[16]),
        "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]), "=r"(u[24]),
        "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
      : "r"(taddr));
}
__device__ __forceinline__ void at_tmem_st32(uint32_t taddr, const float (&r)[32]) {
  const uint32_t* u = reinterpret_cast<const uint32_t*>(r);
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
      ::"r"(taddr), "r"(u[0]), "r"(u[1]), "r"(u[2]), "r"(u[3]), "r"(u[4]), "r"(u[5]), "r"(u[6]), "r"(u[7]), "r"(u[8]),
        "r"(u[9]), "r"(u[10]), "r"(u[11]), "r"(u[12]), "r"(u[13]), "r"(u[14]), "r"(u[15]), "r"(u[16]), "r"(u[17]),
        "r"(u[18]), "r"(u[19]), "r"(u[20]), "r"(u[21]), "r"(u[22]), "r"(u[23]), "r"(u[24]), "r"(u[25]), "r"(u[26]),
        "r"(u[27]), "r"(u[28]), "r"(u[29]), "r"(u[30]), "r"(u[31])
      : "memory");
}
__device__ __forceinline__ float at_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
#define AT_FENCE_BEFORE() asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory")
#define AT_FENCE_AFTER() asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory")

// D float32, A and B bfloat16, 128 x 128; b_mn: B is MN-major (V: [key][d] with d contiguous).
__host__ __device__ constexpr uint32_t at_idesc(bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

struct AtSmem {
  // offsets from a 1024-byte aligned base
  static constexpr int q = 0;                         // 2 blocks
  static constexpr int kv = 2 * AT_BLOCK;             // 2 stages x (K: 2 blocks, V: 2 blocks)
  static constexpr int stage = 4 * AT_BLOCK;
  static constexpr int p = kv + 2 * stage;            // 2 buffers x 2 blocks
  static constexpr int total = p + 4 * AT_BLOCK;      // 14 blocks = 224 KB
};

__global__ void __launch_bounds__(AT_THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                       const int* __restrict__ cu_q, const int* __restrict__ q_start, const int* __restrict__ page_indptr,
                       const int* __restrict__ page_indices, int nq, int nkv, float scale_log2, int window,
                       int page_shift, int G, int* __restrict__ status, int dbg) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t q_full, kv_full[2], kv_empty[2], s_full[2], s_empty[2], p_full, pv_done[2];
  __shared__ uint32_t tmem_slot;

  pdl_prologue();
  const int r = blockIdx.y;
  const int tok0 = cu_q[r], q_len = cu_q[r + 1] - tok0;
  const int tpc = AT_ROWS / G;  // tokens per CTA
  const int m0 = (gridDim.x - 1 - blockIdx.x) * tpc;  // later tiles see more keys: start them first
  if (m0 >= q_len) return;  // uniform for the CTA, before any barrier or allocation
  const int start = q_start[r], kv_len = start + q_len;
  const int head0 = blockIdx.z * G, kvh = head0 / (nq / nkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int q_first = start + m0, q_last = start + min(m0 + tpc, q_len) - 1;
  const int hi = min(kv_len, q_last + 1);
  const int lo = window > 0 ? max(0, q_first - window + 1) : 0;
  const int lo_max = window > 0 ? max(0, q_last - window + 1) : 0;  // the highest lower bound among the rows
  const int tile_begin = lo / AT_KEYS, tile_end = (hi + AT_KEYS - 1) / AT_KEYS;
  const int n_tiles = tile_end - tile_begin;

  if (threadIdx.x == 0) {
    at_mbar_init(&q_full, 1);
    for (int i = 0; i < 2; ++i) {
      at_mbar_init(&kv_full[i], 1);
      at_mbar_init(&kv_empty[i], 1);
      at_mbar_init(&s_full[i], 1);
      at_mbar_init(&s_empty[i], 128);
    }
    at_mbar_init(&p_full, 128);
    at_mbar_init(&pv_done[0], 1);
    at_mbar_init(&pv_done[1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(at_smem(&tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  AT_FENCE_BEFORE();
  __syncthreads();
  AT_FENCE_AFTER();
  const uint32_t tmem = tmem_slot;
  const uint32_t tmem_s[2] = {tmem, tmem + 128u};
  const uint32_t tmem_o = tmem + 256u;

  if (warp == 4) {
    // ------------------------------------------------------------ TMA producer
    // Lane 0 issues every copy; all lanes fetch the tile's page ids together (one coalesced load
    // instead of a chain of dependent ones).
    if (lane == 0) {
      at_expect_tx(&q_full, 2 * AT_BLOCK);
      at_tma_3d(smem + AtSmem::q, &map_q, &q_full, 0, head0, tok0 + m0);
      at_tma_3d(smem + AtSmem::q + AT_BLOCK, &map_q, &q_full, 64, head0, tok0 + m0);
    }
    const int* pages = page_indices + page_indptr[r];
    const int page_size = 1 << page_shift;
    const int box_rows = min(page_size, AT_KEYS);
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int s = j & 1;
      const int key0 = (tile_begin + j) * AT_KEYS;
      const int boxes = min(AT_KEYS, ((kv_len - key0 + box_rows - 1) / box_rows) * box_rows) / box_rows;  // pages that exist
      int my_row = 0;
      if (lane < boxes) {
        const int key = key0 + lane * box_rows;
        const int page = pages[key >> page_shift];
        my_row = (max(page, 0) * nkv + kvh) * page_size + (key & (page_size - 1));
      }
      if (j >= 2) {
        if (lane == 0) ok = at_wait(&kv_empty[s], ((j >> 1) - 1) & 1);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
          if (lane == 0) atomicExch(status, 21);
          break;
        }
      }
      unsigned char* kt = smem + AtSmem::kv + s * AtSmem::stage;
      unsigned char* vt = kt + 2 * AT_BLOCK;
      if (lane == 0) at_expect_tx(&kv_full[s], (uint32_t)boxes * box_rows * 128 * ((dbg & 8) ? 2 : 4));
      __syncwarp();  // the expected byte count is posted before any copy can complete
      if (lane < boxes) {  // every lane issues the four copies of its own page
        const int off = lane * box_rows * 128;
        at_tma_2d(kt + off, &map_k, &kv_full[s], 0, my_row);
        at_tma_2d(kt + AT_BLOCK + off, &map_k, &kv_full[s], 64, my_row);
        if (!(dbg & 8)) {
          at_tma_2d(vt + off, &map_v, &kv_full[s], 0, my_row);
          at_tma_2d(vt + AT_BLOCK + off, &map_v, &kv_full[s], 64, my_row);
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------ MMA issuer
    if (at_elect()) {
      constexpr uint32_t idesc_s = at_idesc(false), idesc_o = at_idesc(true);
      bool ok = at_wait(&q_full, 0);
      if (!ok) atomicExch(status, 22);
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        if (!at_wait(&kv_full[s], (j >> 1) & 1)) return false;
        if (j >= 2 && !at_wait(&s_empty[s], ((j >> 1) - 1) & 1)) return false;
        AT_FENCE_AFTER();
        const unsigned char* kt = smem + AtSmem::kv + s * AtSmem::stage;
#pragma unroll
        for (int kk = 0; kk < AT_D / 16; ++kk) {
          const uint64_t da = at_desc(smem + AtSmem::q + (kk >> 2) * AT_BLOCK, 16, 1024) + (uint64_t)(2 * (kk & 3));
          const uint64_t db = at_desc(kt + (kk >> 2) * AT_BLOCK, 16, 1024) + (uint64_t)(2 * (kk & 3));
          at_mma(tmem_s[s], da, db, idesc_s, kk != 0);
        }
        at_commit(&s_full[s]);
        return true;
      };
      if (ok && n_tiles > 0) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) ok = issue_s(j + 1);
        if (!ok) break;
        if (!at_wait(&p_full, j & 1)) {
          ok = false;
          break;
        }
        AT_FENCE_AFTER();
        const int s = j & 1;
        const unsigned char* vt = smem + AtSmem::kv + s * AtSmem::stage + 2 * AT_BLOCK;
#pragma unroll
        for (int kk = 0; kk < AT_KEYS / 16; ++kk) {
          // A = P [rows][keys], K-major: 16 keys = 32 bytes along the row; B = V [keys][d], MN-major:
          // the two 64-wide halves of d are one block apart, 8-key groups 1024 bytes apart
          const uint64_t da = at_desc(smem + AtSmem::p + (s * 2 + (kk >> 2)) * AT_BLOCK, 16, 1024) + (uint64_t)(2 * (kk & 3));
          const uint64_t db = at_desc(vt + kk * 2048, AT_BLOCK, 1024);
          at_mma(tmem_o, da, db, idesc_o, (j | kk) != 0);
        }
        at_commit(&kv_empty[s]);
        at_commit(&pv_done[s]);
      }
      if (!ok) atomicExch(status, 23);
    }
  } else {
    // ------------------------------------------------------------ softmax, thread = row
    const int row = threadIdx.x;                    // 0..127, also the tensor-memory lane
    const int tok = row / G, hd = row - tok * G;    // rows are ordered token-major, head-minor
    const int qpos = start + m0 + tok;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    float m_used = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int b = j & 1;
      if (!at_wait(&s_full[b], (j >> 1) & 1)) { ok = false; break; }
      AT_FENCE_AFTER();
      float sv[4][32];
      if (!(dbg & 4)) {
#pragma unroll
      for (int c = 0; c < 4; ++c) at_tmem_ld32(tmem_s[b] + lane_base + (uint32_t)(c * 32), sv[c]);
      } else {
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i) sv[c][i] = (float)(i + c);
      }
      asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
      AT_FENCE_BEFORE();
      at_arrive(&s_empty[b]);
      const int key0 = (tile_begin + j) * AT_KEYS;
      // Only tiles that touch the diagonal, the window's edge or the end of the request need the
      // mask; the maximum is tracked on the raw scores (the scale is positive).
      const bool interior = key0 + AT_KEYS - 1 <= q_first && key0 >= lo_max;
      float m_tile = -INFINITY;
      if (dbg & 2) {
        m_tile = sv[0][0];
      } else if (interior) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) m_tile = fmaxf(m_tile, sv[c][i]);
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = key0 + c * 32 + i;
            const bool valid = key <= qpos && key >= lo && (window <= 0 || key > qpos - window);
            sv[c][i] = valid ? sv[c][i] : -INFINITY;
            m_tile = fmaxf(m_tile, sv[c][i]);
          }
      }
      const float m_new = fmaxf(m_used, m_tile);
      float alpha = 1.f;
      bool rescale = false;
      if (m_used == -INFINITY) {
        m_used = m_new;  // nothing accumulated yet for this row
      } else if ((m_new - m_used) * scale_log2 > 8.f) {
        alpha = at_ex2((m_used - m_new) * scale_log2);
        m_used = m_new;
        rescale = true;
      }
      if (__any_sync(0xffffffffu, rescale)) {
        // O may only be touched once the PV product of the previous tile has completed
        if (!at_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1)) { ok = false; break; }
        AT_FENCE_AFTER();
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          float ov[32];
          at_tmem_ld32(tmem_o + lane_base + (uint32_t)(c * 32), ov);
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] *= alpha;
          at_tmem_st32(tmem_o + lane_base + (uint32_t)(c * 32), ov);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
        l_sum *= alpha;
      }
      // this tile's P buffer was last read by the PV product two tiles ago
      if (j >= 2 && !at_wait(&pv_done[b], ((j >> 1) - 1) & 1)) { ok = false; break; }
      const float m_sub = (m_used == -INFINITY ? 0.f : m_used) * scale_log2;
      float part[4] = {0.f, 0.f, 0.f, 0.f};
      unsigned char* p_row = smem + AtSmem::p + b * 2 * AT_BLOCK + row * 128;
      if (!(dbg & 1))
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          float e[8];
#pragma unroll
          for (int x = 0; x < 8; ++x) {
            e[x] = at_ex2(fmaf(sv[c][i + x], scale_log2, -m_sub));  // ex2(-inf) = 0 for masked keys
            part[x & 3] += e[x];
          }
          uint4 pk;
          __nv_bfloat162 p0 = __floats2bfloat162_rn(e[0], e[1]), p1 = __floats2bfloat162_rn(e[2], e[3]);
          __nv_bfloat162 p2 = __floats2bfloat162_rn(e[4], e[5]), p3 = __floats2bfloat162_rn(e[6], e[7]);
          pk.x = *reinterpret_cast<uint32_t*>(&p0);
          pk.y = *reinterpret_cast<uint32_t*>(&p1);
          pk.z = *reinterpret_cast<uint32_t*>(&p2);
          pk.w = *reinterpret_cast<uint32_t*>(&p3);
          const int chunk = c * 4 + (i >> 3);  // 16 chunks of 8 keys
          *reinterpret_cast<uint4*>(p_row + (chunk >> 3) * AT_BLOCK + (((chunk & 7) ^ (row & 7)) << 4)) = pk;
        }
      const float row_sum = (part[0] + part[1]) + (part[2] + part[3]);
      l_sum += row_sum;
      // keys past the end of the request in this tile: their V rows may hold anything (even NaN);
      // P is zero there, but 0 * NaN is NaN, so zero those rows of V
      const int valid_keys = kv_len - key0;
      if (valid_keys < AT_KEYS && row >= valid_keys) {
        unsigned char* vt = smem + AtSmem::kv + b * AtSmem::stage + 2 * AT_BLOCK;
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int cc = 0; cc < 8; ++cc) *reinterpret_cast<uint4*>(vt + h * AT_BLOCK + row * 128 + cc * 16) = make_uint4(0u, 0u, 0u, 0u);
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      AT_FENCE_BEFORE();
      at_arrive(&p_full);
    }
    if (ok && n_tiles > 0) ok = at_wait(&pv_done[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1);
    if (!ok) atomicExch(status, 24);
    AT_FENCE_AFTER();
    if (ok) {
      const bool store = m0 + tok < q_len;  // rows of the tile past the end of the request are dropped
      const float inv = 1.0f / l_sum;
      __nv_bfloat16* dst = out + ((size_t)(tok0 + m0 + (store ? tok : 0)) * nq + head0 + hd) * AT_D;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        float ov[32];
        at_tmem_ld32(tmem_o + lane_base + (uint32_t)(c * 32), ov);  // warp-wide: every lane takes part
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
        if (store) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 pk;
            __nv_bfloat162 p0 = __floats2bfloat162_rn(ov[i] * inv, ov[i + 1] * inv), p1 = __floats2bfloat162_rn(ov[i + 2] * inv, ov[i + 3] * inv);
            __nv_bfloat162 p2 = __floats2bfloat162_rn(ov[i + 4] * inv, ov[i + 5] * inv), p3 = __floats2bfloat162_rn(ov[i + 6] * inv, ov[i + 7] * inv);
            pk.x = *reinterpret_cast<uint32_t*>(&p0);
            pk.y = *reinterpret_cast<uint32_t*>(&p1);
            pk.z = *reinterpret_cast<uint32_t*>(&p2);
            pk.w = *reinterpret_cast<uint32_t*>(&p3);
            *reinterpret_cast<uint4*>(dst + c * 32 + i) = pk;
          }
        }
      }
    }
  }
  AT_FENCE_BEFORE();
  __syncthreads();
  if (warp == 5) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512u) : "memory");
  }
}

// ---------------------------------------------------------------- host side
using AtEncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int at_get_encode(AtEncodeFn* out) {
  static AtEncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    MS_CHECK_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres));
    MS_CHECK_ARG(ptr != nullptr && qres == cudaDriverEntryPointSuccess, "attention_tc: the driver has no cuTensorMapEncodeTiled");
    fn = reinterpret_cast<AtEncodeFn>(ptr);
  }
  *out = fn;
  return 0;
}

}  // namespace ms

using namespace ms;

MS_DEFINE_LAST_ERROR(ms_attn_tc_last_error)
MS_DEFINE_PDL_SWITCH(ms_attn_tc_set_pdl)

// 1 if this kernel takes the shape: head size 128, pages of 8..128 tokens (powers of two).
MS_EXPORT int ms_attn_tc_supports(int head_dim, int page_size, int nq, int nkv) {
  return head_dim == AT_D && page_size >= 8 && page_size <= 128 && (page_size & (page_size - 1)) == 0 && nq % nkv == 0;
}

MS_EXPORT int ms_attn_tc_prefill(void* out, const void* q, const void* k_pool, const void* v_pool, const int* cu_q,
                                 const int* q_start, const int* page_indptr, const int* page_indices, int num_rows,
                                 int num_tokens, int max_q_len, int nq, int nkv, long long pool_pages, float scale,
                                 int window, int page_size, int* status, cudaStream_t stream) {
  if (num_rows == 0) return 0;
  MS_CHECK_ARG(ms_attn_tc_supports(AT_D, page_size, nq, nkv), "attention_tc: unsupported shape (page_size=%d)", page_size);
  MS_CHECK_ARG(num_rows <= 65535, "attention_tc: too many rows (%d) for one launch", num_rows);
  MS_CHECK_ARG(((uintptr_t)q % 16 == 0) && ((uintptr_t)k_pool % 16 == 0) && ((uintptr_t)v_pool % 16 == 0), "attention_tc: operands must be 16-byte aligned");
  const int group = nq / nkv;
  int G = 1;
  while (G * 2 <= 8 && group % (G * 2) == 0) G *= 2;  // heads per CTA: the largest power of two up to 8 that divides the group
  const int tpc = AT_ROWS / G;
  AtEncodeFn encode;
  if (int rc = at_get_encode(&encode)) return rc;
  CUtensorMap map_q, map_k, map_v;
  {
    const cuuint64_t dims[3] = {(cuuint64_t)AT_D, (cuuint64_t)nq, (cuuint64_t)num_tokens};
    const cuuint64_t strides[2] = {(cuuint64_t)AT_D * 2, (cuuint64_t)nq * AT_D * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)tpc};
    const cuuint32_t elem[3] = {1, 1, 1};
    const CUresult res = encode(&map_q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, elem,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    MS_CHECK_ARG(res == CUDA_SUCCESS, "attention_tc: encoding the query map failed with code %d", (int)res);
  }
  const cuuint64_t rows = (cuuint64_t)pool_pages * nkv * page_size;
  const cuuint64_t kdims[2] = {(cuuint64_t)AT_D, rows};
  const cuuint64_t kstrides[1] = {(cuuint64_t)AT_D * 2};
  const cuuint32_t kbox[2] = {64, (cuuint32_t)(page_size < AT_KEYS ? page_size : AT_KEYS)};
  const cuuint32_t kelem[2] = {1, 1};
  for (int i = 0; i < 2; ++i) {
    const CUresult res = encode(i == 0 ? &map_k : &map_v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                                const_cast<void*>(i == 0 ? k_pool : v_pool), kdims, kstrides, kbox, kelem,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    MS_CHECK_ARG(res == CUDA_SUCCESS, "attention_tc: encoding the cache map failed with code %d", (int)res);
  }
  constexpr size_t smem = AtSmem::total + 1024;
  static bool configured = false;
  if (!configured) {
    MS_CHECK_CUDA(cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  static const int dbg = getenv("MINISERVE_ATTN_TC_DEBUG") ? atoi(getenv("MINISERVE_ATTN_TC_DEBUG")) : 0;  // timing experiments only
  dim3 grid(ceil_div(max_q_len, tpc), num_rows, nq / G);
  MS_LAUNCH(attn_prefill_tc_kernel, grid, AT_THREADS, smem, stream, map_q, map_k, map_v, (__nv_bfloat16*)out, cu_q, q_start,
            page_indptr, page_indices, nq, nkv, scale * AT_LOG2E, window, page_shift, G, status, dbg);
  return 0;
}
