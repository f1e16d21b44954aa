// Causal grouped-query attention for prompts and mixed steps on the 5th-generation tensor cores,
// for head size 128 and bfloat16: S = Q K^T and O += P V are tcgen05.mma instructions with the
// accumulators in tensor memory, operands staged by TMA straight out of the paged cache.
//
// Formula as in attention_bf16.cu (miniserve/model/attention.py:60-67,125-133): a query row at
// absolute position p sees keys 0..p of its request (or the last `window`), query head h reads kv
// head h / (heads / kv_heads), softmax in float32 with scale head_dim^-0.5.
//
// One CTA owns 256 query rows in two groups of 128 (G query heads of one kv head x 128/G
// consecutive tokens each), so that every K/V tile is fetched once for all of them. Thread r of a
// softmax group owns row r (tensor-memory lane r): per key tile it reads its row of S with
// tcgen05.ld, masks it if the tile touches the diagonal, a window's edge or the request's end,
// keeps a running maximum and sum, stores P (bfloat16) back into tensor memory, and rescales O
// only when the maximum has grown by more than 2^8 (the stale maximum is exact in the end because
// the same one scales the sum).
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
__device__ __forceinline__ bool at_wait(uint64_t* bar, uint32_t parity) { return mbar_wait_bounded(at_smem(bar), parity); }
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
// 2^x on the FMA pipes (for x <= 8): round to the nearest integer with the 1.5 * 2^23 trick, a
// cubic for 2^fraction on [-0.5, 0.5] (relative error 1e-4, far below the bfloat16 rounding of P),
// and the integer part added to the exponent bits. Used for a share of the elements so that the
// special-function unit (16 ex2 per clock per SM) would not limit the softmax. Measured on B200 it
// is not the limit here (0, 2, 3 or 4 of every 8 emulated: 411, 427, 421, 431 us for 8,192 tokens).
__device__ __forceinline__ float at_ex2_poly(float x) {
  x = fmaxf(x, -125.f);
  const float t = x + 12582912.f;
  const float f = x - (t - 12582912.f);
  float p = fmaf(f, 0.0558382829f, 0.2426394785f);
  p = fmaf(p, f, 0.6931367339f);
  p = fmaf(p, f, 0.9999245570f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}
#ifndef AT_EMULATED_OF_8
#define AT_EMULATED_OF_8 0  // of every 8 exponentials, this many go to the FMA pipes (measured: no gain, so none)
#endif
#define AT_FENCE_BEFORE() asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory")
#define AT_FENCE_AFTER() asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory")

// D float32, A and B bfloat16, 128 x 128; b_mn: B is MN-major (V: [key][d] with d contiguous).
__host__ __device__ constexpr uint32_t at_idesc(bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

// The kernel: 256 query rows per CTA as two groups of 128 that take turns on the tensor cores.
// Both groups (A: tokens m0 .. m0+tpc-1, B: the next tpc tokens; G heads each) attend over the
// same K/V tiles, so every tile is fetched once for twice the rows. While group A's softmax
// warps work on tile j, the tensor cores run group B's products, and the other way round. P never
// goes through shared memory: the softmax threads store it (bfloat16, two per 32-bit column) into
// the tensor-memory columns its S tile occupied, and the second product takes its A operand from
// there. Tensor memory: S/P of A [0,128), S/P of B [128,256), O of A [256,384), O of B [384,512).
// Warps 0-3: softmax A, 4-7: softmax B, 8: TMA, 9: MMA, 10-11: idle (registers are handed over by groups of four warps).
constexpr int AT_THREADS = 384;  // 8 softmax warps, 1 TMA warp, 1 MMA warp, 2 warps that only make up the third group of four

struct AtSmem {
  static constexpr int q = 0;                     // group A: 2 blocks, group B: 2 blocks
  static constexpr int kv = 4 * AT_BLOCK;         // 2 stages x (K: 2 blocks, V: 2 blocks)
  static constexpr int stage = 4 * AT_BLOCK;
  static constexpr int total = kv + 2 * stage;    // 12 blocks = 192 KB
};

__device__ __forceinline__ void at_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u;
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void at_tmem_st16(uint32_t taddr, const uint32_t (&u)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n"
      ::"r"(taddr), "r"(u[0]), "r"(u[1]), "r"(u[2]), "r"(u[3]), "r"(u[4]), "r"(u[5]), "r"(u[6]), "r"(u[7]), "r"(u[8]),
        "r"(u[9]), "r"(u[10]), "r"(u[11]), "r"(u[12]), "r"(u[13]), "r"(u[14]), "r"(u[15])
      : "memory");
}

// eight float32 scaled by `inv`, as eight bfloat16
__device__ __forceinline__ uint4 at_pack8(const float* v, float inv) {
  __nv_bfloat162 p0 = __floats2bfloat162_rn(v[0] * inv, v[1] * inv), p1 = __floats2bfloat162_rn(v[2] * inv, v[3] * inv);
  __nv_bfloat162 p2 = __floats2bfloat162_rn(v[4] * inv, v[5] * inv), p3 = __floats2bfloat162_rn(v[6] * inv, v[7] * inv);
  uint4 pk;
  pk.x = *reinterpret_cast<uint32_t*>(&p0);
  pk.y = *reinterpret_cast<uint32_t*>(&p1);
  pk.z = *reinterpret_cast<uint32_t*>(&p2);
  pk.w = *reinterpret_cast<uint32_t*>(&p3);
  return pk;
}
// barriers of one softmax group (128 threads, hardware barrier `id`): plain, and with an OR over a flag
__device__ __forceinline__ void at_group_sync(int id) { asm volatile("bar.sync %0, 128;\n" ::"r"(id) : "memory"); }
__device__ __forceinline__ bool at_group_any(int id, bool flag) {
  uint32_t res;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %2, 0;\n\t"
      "bar.red.or.pred q, %1, 128, p;\n\tselp.u32 %0, 1, 0, q;\n\t}\n"
      : "=r"(res) : "r"(id), "r"((uint32_t)flag) : "memory");
  return res != 0;
}

// A new running maximum for a row: the stale one is kept while the new one exceeds it by at most
// 2^8 after scaling (the same maximum scales the sum, so the result stays exact); returns the factor
// that what was accumulated so far has to be scaled by (1: nothing to do).
__device__ __forceinline__ float at_new_maximum(float m_tile, float& m_used, float scale_log2) {
  const float m_new = fmaxf(m_used, m_tile);
  if (m_used == -INFINITY) {
    m_used = m_new;
  } else if ((m_new - m_used) * scale_log2 > 8.f) {
    const float alpha = at_ex2((m_used - m_new) * scale_log2);
    m_used = m_new;
    return alpha;
  }
  return 1.f;
}
// O *= alpha for this thread's row. Called when S(j) is complete, so the product P(j-1) V(j-1) issued
// before it is complete too: O is quiet.
__device__ __forceinline__ void at_rescale(uint32_t t_o, float alpha) {
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {
    float ov[32];
    at_tmem_ld32(t_o + (uint32_t)(c * 32), ov);
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) ov[i] *= alpha;
    at_tmem_st32(t_o + (uint32_t)(c * 32), ov);
  }
}
// The softmax step of one row for a tile in which the row sees only the keys at offsets
// [seen_lo, seen_hi]. The scores are read twice, 32 columns at a time: once for the maximum, once for
// the exponentials (chunk c of P, 16 columns, lies below chunk c + 1 of S, so chunks are read and
// written in turn). A function of its own: inlined beside the all-in-registers form of interior tiles
// it cost that form its registers. The one-pass form (the whole row in registers here too) was tried in
// this function and measured slower inside a prompt step (3.60 against 3.53 ms for 2,048 tokens): its
// 128 live values cost the kernel around the call more than the second read costs here.
// Returns the sum of the row's exponentials.
__device__ __noinline__ float at_softmax_masked(uint32_t t_s, uint32_t t_o, int seen_lo, int seen_hi, float scale_log2,
                                                float& m_used, float& l_sum) {
  float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {
    float v[32];
    at_tmem_ld32(t_s + (uint32_t)(c * 32), v);
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const int off = c * 32 + i;
      mx[i & 3] = fmaxf(mx[i & 3], off <= seen_hi && off >= seen_lo ? v[i] : -INFINITY);
    }
  }
  const float alpha = at_new_maximum(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), m_used, scale_log2);
  if (__any_sync(0xffffffffu, alpha != 1.f)) {
    at_rescale(t_o, alpha);
    l_sum *= alpha;
  }
  const float m_sub = (m_used == -INFINITY ? 0.f : m_used) * scale_log2;
  float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {
    float v[32];
    at_tmem_ld32(t_s + (uint32_t)(c * 32), v);
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
    uint32_t pk[16];
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      const int off = c * 32 + i;
      const float e0 = off <= seen_hi && off >= seen_lo ? at_ex2(fmaf(v[i], scale_log2, -m_sub)) : 0.f;
      const float e1 = off + 1 <= seen_hi && off + 1 >= seen_lo ? at_ex2(fmaf(v[i + 1], scale_log2, -m_sub)) : 0.f;
      part[(i >> 1) & 3] += e0 + e1;
      __nv_bfloat162 p2 = __floats2bfloat162_rn(e0, e1);
      pk[i >> 1] = *reinterpret_cast<uint32_t*>(&p2);
    }
    at_tmem_st16(t_s + (uint32_t)(c * 16), pk);
  }
  return (part[0] + part[1]) + (part[2] + part[3]);
}

// What one work item (a tile of 2 x 128 query rows, one group of heads, one split of the keys)
// has to do. All threads of a CTA compute it from the item's index; the scheduler warp also
// uses it to tell empty items from real ones.
struct AtItem {
  int r, rank, tok0, q_len, m0, start, kv_len, head0, split;
  int n_tiles[2], q_first[2], q_last[2], lo_g[2], lo_max[2], shares[2];
  int tile_begin, n_all;
  bool has_b;
};

struct AtGrid {
  int q_tiles, rows, head_groups, splits, max_tiles_per_item, window, G;
  __device__ __forceinline__ int total() const { return q_tiles * rows * head_groups * splits; }
};

// Items are numbered so that the tiles with the most keys (the last tiles of the longest rows)
// come first: tile rank, then row, then head group, then split.
__device__ __forceinline__ bool at_item(AtItem& it, int idx, const AtGrid& gr, const int* __restrict__ cu_q,
                                        const int* __restrict__ q_start) {
  it.split = idx % gr.splits;
  idx /= gr.splits;
  it.head0 = (idx % gr.head_groups) * gr.G;
  idx /= gr.head_groups;
  it.r = idx % gr.rows;
  it.rank = idx / gr.rows;
  const int tpc = AT_ROWS / gr.G;  // tokens per group
  it.tok0 = cu_q[it.r];
  it.q_len = cu_q[it.r + 1] - it.tok0;
  it.m0 = (gr.q_tiles - 1 - it.rank) * 2 * tpc;
  if (it.m0 >= it.q_len) return false;
  it.start = q_start[it.r];
  it.kv_len = it.start + it.q_len;
  // per group: the key tiles it needs (B needs at least as many as A; B may have no rows at all)
  it.has_b = it.m0 + tpc < it.q_len;
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    it.q_first[g] = it.start + it.m0 + g * tpc;
    it.q_last[g] = it.start + min(it.m0 + (g + 1) * tpc, it.q_len) - 1;
    it.lo_g[g] = gr.window > 0 ? max(0, it.q_first[g] - gr.window + 1) : 0;
    it.lo_max[g] = gr.window > 0 ? max(0, it.q_last[g] - gr.window + 1) : 0;
  }
  it.tile_begin = it.lo_g[0] / AT_KEYS;
  it.n_tiles[0] = (min(it.kv_len, it.q_last[0] + 1) + AT_KEYS - 1) / AT_KEYS - it.tile_begin;
  it.n_tiles[1] = it.has_b ? (min(it.kv_len, it.q_last[1] + 1) + AT_KEYS - 1) / AT_KEYS - it.tile_begin : 0;
  // Key ranges longer than `max_tiles_per_item` are cut into pieces of that length (the last one
  // shorter; measured faster than equal pieces, whose items all start late in the queue's order)
  // that other items take, at most `splits` of them: this one keeps `per_split` key tiles from its
  // piece's first. A group whose keys lie in more than one piece leaves a partial result
  // (unnormalised O, the maximum it is scaled by, the sum), and the last of them to finish adds
  // the partial results up in the order of the pieces.
  const int n_full = max(it.n_tiles[0], it.n_tiles[1]);
  const int per_split = max(gr.max_tiles_per_item, (n_full + gr.splits - 1) / gr.splits);
  if (it.split * per_split >= n_full) return false;
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    it.shares[g] = (it.n_tiles[g] + per_split - 1) / per_split;  // in how many splits the group has keys
    it.n_tiles[g] = min(max(it.n_tiles[g] - it.split * per_split, 0), per_split);
  }
  it.tile_begin += it.split * per_split;
  it.n_all = max(it.n_tiles[0], it.n_tiles[1]);
  return true;
}

// The scheduler (all lanes of one warp): the CTA's first item is the one with its own number, the
// others come off a counter in global memory. Empty items (tiles past a short row's end, splits
// past a short key range) are stepped over: the lanes look at the 32 items from the claimed one
// on, so a run of empty items costs one round trip. When nothing is left, the CTA signs off on a
// second counter, and the last one to do so puts both back to zero for the next launch.
__device__ __forceinline__ int at_claim(int* __restrict__ queue, const AtGrid& gr, const int* __restrict__ cu_q,
                                        const int* __restrict__ q_start, int lane, bool first) {
  const int total = gr.total();
  for (;;) {
    int idx = (int)blockIdx.x;
    if (!first) {
      if (lane == 0) idx = (int)gridDim.x + atomicAdd(queue, 1);
      idx = __shfl_sync(0xffffffffu, idx, 0);
    }
    if (idx >= total) {
      if (lane == 0 && atomicAdd(queue + 1, 1) == (int)gridDim.x - 1) {
        queue[0] = 0;
        queue[1] = 0;
      }
      return -1;
    }
    AtItem probe;
    const bool work = idx + lane < total && at_item(probe, idx + lane, gr, cu_q, q_start);
    const unsigned mask = __ballot_sync(0xffffffffu, work);
    if (mask & 1u) return idx;
    const int run = mask ? __ffs(mask) - 1 : 32;  // this many items from idx on are empty
    if (!first && lane == 0 && run > 1) atomicMax(queue, idx + run - (int)gridDim.x);
    first = false;
  }
}

// Persistent: one CTA per SM takes items off a queue until none is left.
__global__ void __launch_bounds__(AT_THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                        const int* __restrict__ cu_q, const int* __restrict__ q_start, const int* __restrict__ page_indptr,
                        const int* __restrict__ page_indices, int nq, int nkv, float scale_log2, int page_shift,
                        const AtGrid gr_given, int* __restrict__ status,
                        float* __restrict__ part_o, float2* __restrict__ part_ml, int* __restrict__ queue,
                        int* __restrict__ tickets, const int* __restrict__ plan) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t q_full, kv_full[2], kv_empty[2], s_full[2], p_full[2], o_final[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int ticket_of[2];
  __shared__ int item_slot;       // the item the CTA works on (-1: none left)
  __shared__ int failed;          // a bounded wait gave up somewhere: the CTA winds down
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  pdl_prologue();
  // A launch that was captured into a CUDA graph takes what follows from the rows' lengths (tiles per
  // row, rows, key splits) from device memory, where the host puts it before every replay: the
  // launch itself (a CTA per SM, these arguments) is then the same for every step of its size.
  AtGrid gr = gr_given;
  if (plan != nullptr) {
    gr.q_tiles = plan[0];
    gr.rows = plan[1];
    gr.splits = plan[2];
    gr.max_tiles_per_item = plan[3];
    part_ml = reinterpret_cast<float2*>(part_o + (size_t)gr.q_tiles * gr.rows * gr.head_groups * 2 * gr.splits * (AT_ROWS * AT_D));
  }
  const int G = gr.G, window = gr.window;
  const int tpc = AT_ROWS / G;
  int next_item = -1;  // held by the scheduler warp
  if (warp == 8) {
    next_item = at_claim(queue, gr, cu_q, q_start, lane, true);
    if (lane == 0) item_slot = next_item;
  }
  auto init_barriers = [&]() {
    at_mbar_init(&q_full, 1);
    for (int i = 0; i < 2; ++i) {
      at_mbar_init(&kv_full[i], 1);
      at_mbar_init(&kv_empty[i], 1);
      at_mbar_init(&s_full[i], 1);
      at_mbar_init(&p_full[i], 128);
      at_mbar_init(&o_final[i], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  };
  if (threadIdx.x == 0) {
    failed = 0;
    init_barriers();
  }
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(at_smem(&tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  AT_FENCE_BEFORE();
  __syncthreads();
  AT_FENCE_AFTER();
  const uint32_t tmem = tmem_slot;

  // The roles part for good here, each with its own loop over the items, because they part in registers
  // too: 12 warps of 168 registers fill the register file, the softmax warps (a whole row of scores each,
  // 128 values) want more and the two warps that issue copies and products, and their two idle
  // companions, need few. Warps 8 to 11 give theirs up, warps 0 to 7 take them.
  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;\n");
    for (;;) {
      const int cur = item_slot;
      if (cur < 0) break;
      AtItem it;
      at_item(it, cur, gr, cu_q, q_start);
      const int r = it.r, tok0 = it.tok0, m0 = it.m0, kv_len = it.kv_len;
      const int head0 = it.head0, kvh = head0 / (nq / nkv), tile_begin = it.tile_begin, n_all = it.n_all;
      const bool has_b = it.has_b;
      if (warp == 8) {
        // ---------------------------------------------------------- TMA producer (and scheduler)
        if (lane == 0) {
          at_expect_tx(&q_full, (has_b ? 4 : 2) * AT_BLOCK);
          at_tma_3d(smem + AtSmem::q, &map_q, &q_full, 0, head0, tok0 + m0);
          at_tma_3d(smem + AtSmem::q + AT_BLOCK, &map_q, &q_full, 64, head0, tok0 + m0);
          if (has_b) {
            at_tma_3d(smem + AtSmem::q + 2 * AT_BLOCK, &map_q, &q_full, 0, head0, tok0 + m0 + tpc);
            at_tma_3d(smem + AtSmem::q + 3 * AT_BLOCK, &map_q, &q_full, 64, head0, tok0 + m0 + tpc);
          }
        }
        const int* pages = page_indices + page_indptr[r];
        const int page_size = 1 << page_shift;
        const int box_rows = min(page_size, AT_KEYS);
        bool ok = true;
        for (int j = 0; j < n_all; ++j) {
          const int s = j & 1;
          const int key0 = (tile_begin + j) * AT_KEYS;
          const int boxes = min(AT_KEYS, ((kv_len - key0 + box_rows - 1) / box_rows) * box_rows) / box_rows;
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
              if (lane == 0) {
                atomicExch(status, 31);
                failed = 1;
              }
              break;
            }
          }
          unsigned char* kt = smem + AtSmem::kv + s * AtSmem::stage;
          unsigned char* vt = kt + 2 * AT_BLOCK;
          if (lane == 0) at_expect_tx(&kv_full[s], (uint32_t)boxes * box_rows * 128 * 4);
          __syncwarp();
          if (lane < boxes) {
            const int off = lane * box_rows * 128;
            at_tma_2d(kt + off, &map_k, &kv_full[s], 0, my_row);
            at_tma_2d(kt + AT_BLOCK + off, &map_k, &kv_full[s], 64, my_row);
            at_tma_2d(vt + off, &map_v, &kv_full[s], 0, my_row);
            at_tma_2d(vt + AT_BLOCK + off, &map_v, &kv_full[s], 64, my_row);
          }
        }
        // all loads of this item are on their way: find the next one while the others compute
        __syncwarp();
        next_item = at_claim(queue, gr, cu_q, q_start, lane, false);
      } else if (warp == 9) {
        // ---------------------------------------------------------- MMA issuer
        if (at_elect()) {
          constexpr uint32_t idesc_s = at_idesc(false), idesc_o = at_idesc(true);
          bool ok = at_wait(&q_full, 0);
          int kv_ready = -1;  // the last tile whose kv_full this thread has waited for
          auto need_kv = [&](int j) -> bool {
            if (j <= kv_ready) return true;
            if (!at_wait(&kv_full[j & 1], (j >> 1) & 1)) return false;
            kv_ready = j;
            AT_FENCE_AFTER();
            return true;
          };
          auto issue_s = [&](int g, int j) -> bool {
            if (!need_kv(j)) return false;
            const unsigned char* kt = smem + AtSmem::kv + (j & 1) * AtSmem::stage;
            const unsigned char* qt = smem + AtSmem::q + g * 2 * AT_BLOCK;
  #pragma unroll
            for (int kk = 0; kk < AT_D / 16; ++kk) {
              const uint64_t da = at_desc(qt + (kk >> 2) * AT_BLOCK, 16, 1024) + (uint64_t)(2 * (kk & 3));
              const uint64_t db = at_desc(kt + (kk >> 2) * AT_BLOCK, 16, 1024) + (uint64_t)(2 * (kk & 3));
              at_mma(tmem + (uint32_t)(g * 128), da, db, idesc_s, kk != 0);
            }
            at_commit(&s_full[g]);
            return true;
          };
          if (ok && it.n_tiles[0] > 0) ok = issue_s(0, 0);
          if (ok && it.n_tiles[1] > 0) ok = issue_s(1, 0);
          for (int j = 0; j < n_all && ok; ++j) {
            const unsigned char* vt = smem + AtSmem::kv + (j & 1) * AtSmem::stage + 2 * AT_BLOCK;
  #pragma unroll 1
            for (int g = 0; g < 2 && ok; ++g) {
              if (j >= it.n_tiles[g]) continue;
              if (!at_wait(&p_full[g], j & 1)) { ok = false; break; }
              AT_FENCE_AFTER();
  #pragma unroll
              for (int kk = 0; kk < AT_KEYS / 16; ++kk) {
                // A = P of this group in tensor memory: 16 keys = 8 columns of packed bf16 pairs;
                // B = V [keys][d], MN-major
                const uint64_t db = at_desc(vt + kk * 2048, AT_BLOCK, 1024);
                at_mma_ts(tmem + (uint32_t)(256 + g * 128), tmem + (uint32_t)(g * 128 + kk * 8), db, idesc_o, (j | kk) != 0);
              }
              if (j + 1 < it.n_tiles[g]) {
                ok = issue_s(g, j + 1);  // overwrites this group's S/P columns: ordered after the product above
              } else {
                at_commit(&o_final[g]);
              }
            }
            // the producer waits for this only before tile j + 2: an arrival that nobody waits for
            // must not be in flight when the barriers are set up again for the next item
            if (ok && j + 2 < n_all) at_commit(&kv_empty[j & 1]);
          }
          if (!ok) {
            atomicExch(status, 33);
            failed = 1;
          }
        }
      }
      // ------------------------------------------------------------ between items
      // Everything of this item is over: every product has completed (the softmax groups waited for
      // the last ones), every arrival that was asked for has been waited for. The barriers start
      // again from phase 0 and the scheduler publishes the next item.
      AT_FENCE_BEFORE();
      __syncthreads();
      if (failed) break;
      if (threadIdx.x == 0) init_barriers();
      if (warp == 8 && lane == 0) item_slot = next_item;
      __syncthreads();
      AT_FENCE_AFTER();
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;\n");
    for (;;) {
      const int cur = item_slot;
      if (cur < 0) break;
      AtItem it;
      at_item(it, cur, gr, cu_q, q_start);
      const int r = it.r, tok0 = it.tok0, q_len = it.q_len, m0 = it.m0, start = it.start, kv_len = it.kv_len;
      const int head0 = it.head0, split = it.split, tile_begin = it.tile_begin;
      {
        // ---------------------------------------------------------- softmax, thread = row of its group
        const int g = warp >> 2;
        const int row = threadIdx.x & 127;                // row within the group = tensor-memory lane
        const int tok = row / G, hd = row - tok * G;
        const int tok_in_req = m0 + g * tpc + tok;
        const int qpos = start + tok_in_req;
        const int lo_mine = it.lo_g[g], lo_max_mine = it.lo_max[g], q_first_mine = it.q_first[g];
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t t_s = tmem + (uint32_t)(g * 128) + lane_base, t_o = tmem + (uint32_t)(256 + g * 128) + lane_base;
        const int n_mine = it.n_tiles[g];
        float m_used = -INFINITY, l_sum = 0.f;
        bool ok = true;
        for (int j = 0; j < n_mine && ok; ++j) {
          if (!at_wait(&s_full[g], j & 1)) { ok = false; break; }
          AT_FENCE_AFTER();
          const int key0 = (tile_begin + j) * AT_KEYS;
          const bool interior = key0 + AT_KEYS - 1 <= q_first_mine && key0 >= lo_max_mine;
          float part[4] = {0.f, 0.f, 0.f, 0.f};
          if (interior) {
            // every key of the tile is seen by every row of the group: the whole row of scores in
            // registers, four loads in flight, one wait
            float sv[4][32];
  #pragma unroll
            for (int c = 0; c < 4; ++c) at_tmem_ld32(t_s + (uint32_t)(c * 32), sv[c]);
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
  #pragma unroll
            for (int c = 0; c < 4; ++c)
  #pragma unroll
              for (int i = 0; i < 32; ++i) mx[i & 3] = fmaxf(mx[i & 3], sv[c][i]);
            const float alpha = at_new_maximum(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), m_used, scale_log2);
            if (__any_sync(0xffffffffu, alpha != 1.f)) {
              at_rescale(t_o, alpha);
              l_sum *= alpha;
            }
            // P = 2^(s * scale - max), packed two bf16 per column into the columns S came from
            const float m_sub = (m_used == -INFINITY ? 0.f : m_used) * scale_log2;
  #pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t pk[16];
  #pragma unroll
              for (int i = 0; i < 32; i += 2) {
                const float x0 = fmaf(sv[c][i], scale_log2, -m_sub), x1 = fmaf(sv[c][i + 1], scale_log2, -m_sub);
                const float e0 = (i & 7) < AT_EMULATED_OF_8 ? at_ex2_poly(x0) : at_ex2(x0);
                const float e1 = ((i + 1) & 7) < AT_EMULATED_OF_8 ? at_ex2_poly(x1) : at_ex2(x1);
                part[(i >> 1) & 3] += e0 + e1;
                __nv_bfloat162 p2 = __floats2bfloat162_rn(e0, e1);
                pk[i >> 1] = *reinterpret_cast<uint32_t*>(&p2);
              }
              at_tmem_st16(t_s + (uint32_t)(c * 16), pk);
            }
          } else {
            // a tile on the diagonal, at a window's edge or at the request's end: the keys of the tile
            // that this row sees are those at offsets [seen_lo, seen_hi]
            const int seen_hi = qpos - key0;
            const int seen_lo = max(lo_mine, window > 0 ? qpos - window + 1 : 0) - key0;
            part[0] = at_softmax_masked(t_s, t_o, seen_lo, seen_hi, scale_log2, m_used, l_sum);
          }
          l_sum += (part[0] + part[1]) + (part[2] + part[3]);
          const int valid_keys = kv_len - key0;
          if (valid_keys < AT_KEYS && row >= valid_keys) {
            unsigned char* vt = smem + AtSmem::kv + (j & 1) * AtSmem::stage + 2 * AT_BLOCK;
  #pragma unroll
            for (int h = 0; h < 2; ++h)
  #pragma unroll
              for (int cc = 0; cc < 8; ++cc) *reinterpret_cast<uint4*>(vt + h * AT_BLOCK + row * 128 + cc * 16) = make_uint4(0u, 0u, 0u, 0u);
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
          }
          asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
          AT_FENCE_BEFORE();
          at_arrive(&p_full[g]);
        }
        if (ok && n_mine > 0) ok = at_wait(&o_final[g], 0);
        if (!ok) {
          atomicExch(status, 34);
          failed = 1;
        }
        AT_FENCE_AFTER();
        const bool store = tok_in_req < q_len;
        const size_t item = (size_t)(tok0 + (store ? tok_in_req : 0)) * nq + head0 + hd;  // (token, head) of this row
        __nv_bfloat16* dst = out + item * AT_D;
        if (it.shares[g] <= 1) {
          if (ok && n_mine > 0) {
            const float inv = 1.0f / l_sum;
  #pragma unroll 1
            for (int c = 0; c < 4; ++c) {
              float ov[32];
              at_tmem_ld32(t_o + (uint32_t)(c * 32), ov);
              asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
              if (store) {
  #pragma unroll
                for (int i = 0; i < 32; i += 8) *reinterpret_cast<uint4*>(dst + c * 32 + i) = at_pack8(ov + i, inv);
              }
            }
          }
        } else if (n_mine > 0) {
          // One of several splits of this group's keys. Each takes a ticket when it is done. All but the
          // last leave their partial result (unnormalised O, the maximum it is scaled by, the sum) and
          // count themselves done; the last waits until the others are (they took their tickets before
          // it and depend on nothing of it, so this is a wait for writes in flight), then adds the
          // partial results up in the order of the splits, its own from tensor memory, and writes the
          // rows. Partial results are laid out [group of rows][split][4 columns][row], so that the 128
          // threads of a group (one row each) write and read whole 512-byte lines together.
          const size_t unit = ((size_t)(it.rank * gr.rows + r) * gr.head_groups + head0 / G) * 2 + g;
          float4* po = reinterpret_cast<float4*>(part_o) + (unit * gr.splits + split) * (32 * 128) + row;
          float2* pml = part_ml + unit * gr.splits * 128 + row;
          int* ticket = tickets + unit;
          int* done = tickets + (size_t)gr.q_tiles * gr.rows * gr.head_groups * 2 + unit;
          // all 128 threads of the group meet here, also after a wait that gave up: then nobody takes a ticket
          const bool bad = at_group_any(1 + g, !ok);
          if (row == 0 && !bad) ticket_of[g] = atomicAdd(ticket, 1);
          at_group_sync(1 + g);
          const bool last = !bad && ticket_of[g] == it.shares[g] - 1;
          if (!bad && !last) {
  #pragma unroll 1
            for (int c = 0; c < 4; ++c) {
              float ov[32];
              at_tmem_ld32(t_o + (uint32_t)(c * 32), ov);
              asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
  #pragma unroll
              for (int i = 0; i < 8; ++i) po[(c * 8 + i) * 128] = make_float4(ov[4 * i], ov[4 * i + 1], ov[4 * i + 2], ov[4 * i + 3]);
            }
            pml[split * 128] = make_float2(m_used, l_sum);
            __threadfence();
            at_group_sync(1 + g);
            if (row == 0) atomicAdd(done, 1);
          } else if (last) {
            if (row == 0) {
              // bounded like every wait: a split that took its ticket and never finishes is an error, not a hang
              unsigned long long began = 0;
              bool there = false;
              for (uint32_t polls = 1; !there; ++polls) {
                there = *reinterpret_cast<volatile int*>(done) >= it.shares[g] - 1;
                if (!there && (polls & 63u) == 0) {
                  unsigned long long now;
                  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(now));
                  if (began == 0) began = now;
                  else if (now - began > MS_WAIT_NS) break;
                }
              }
              if (!there) atomicExch(status, 35);
              *ticket = 0;  // both left as they were found, for the next launch
              *done = 0;
              __threadfence();
            }
            at_group_sync(1 + g);
            const float4* pall = reinterpret_cast<const float4*>(part_o) + unit * gr.splits * (32 * 128) + row;
            float m_all = m_used;
            for (int sp = 0; sp < it.shares[g]; ++sp)
              if (sp != split) m_all = fmaxf(m_all, __ldcg(&pml[sp * 128]).x);
            float l_all = 0.f;
            for (int sp = 0; sp < it.shares[g]; ++sp) {
              const float2 ml = sp == split ? make_float2(m_used, l_sum) : __ldcg(&pml[sp * 128]);
              l_all += ml.y == 0.f ? 0.f : at_ex2((ml.x - m_all) * scale_log2) * ml.y;
            }
            const float inv = 1.0f / l_all;
  #pragma unroll 1
            for (int c = 0; c < 4; ++c) {
              float own[32], acc[32];
              at_tmem_ld32(t_o + (uint32_t)(c * 32), own);
              asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
  #pragma unroll
              for (int i = 0; i < 32; ++i) acc[i] = 0.f;
              for (int sp = 0; sp < it.shares[g]; ++sp) {
                if (sp == split) {
                  const float w = l_sum == 0.f ? 0.f : at_ex2((m_used - m_all) * scale_log2);
  #pragma unroll
                  for (int i = 0; i < 32; ++i) acc[i] = fmaf(w, own[i], acc[i]);
                } else {
                  const float2 ml = __ldcg(&pml[sp * 128]);
                  const float w = ml.y == 0.f ? 0.f : at_ex2((ml.x - m_all) * scale_log2);
                  const float4* src = pall + (size_t)sp * (32 * 128) + (c * 8) * 128;
  #pragma unroll
                  for (int i = 0; i < 8; ++i) {
                    const float4 v = __ldcg(src + i * 128);
                    acc[4 * i] = fmaf(w, v.x, acc[4 * i]);
                    acc[4 * i + 1] = fmaf(w, v.y, acc[4 * i + 1]);
                    acc[4 * i + 2] = fmaf(w, v.z, acc[4 * i + 2]);
                    acc[4 * i + 3] = fmaf(w, v.w, acc[4 * i + 3]);
                  }
                }
              }
              if (store) {
  #pragma unroll
                for (int i = 0; i < 32; i += 8) *reinterpret_cast<uint4*>(dst + c * 32 + i) = at_pack8(acc + i, inv);
              }
            }
          }
          at_group_sync(1 + g);  // ticket_of[g] is free for the next item
        }
      }
      // ------------------------------------------------------------ between items
      // Everything of this item is over: every product has completed (the softmax groups waited for
      // the last ones), every arrival that was asked for has been waited for. The barriers start
      // again from phase 0 and the scheduler publishes the next item.
      AT_FENCE_BEFORE();
      __syncthreads();
      if (failed) break;
      if (threadIdx.x == 0) init_barriers();
      __syncthreads();
      AT_FENCE_AFTER();
    }
  }
  AT_FENCE_BEFORE();
  __syncthreads();
  if (warp == 9) {
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

static int at_heads_per_cta(int nq, int nkv) {
  const int group = nq / nkv;
  int G = 1;
  while (G * 2 <= 8 && group % (G * 2) == 0) G *= 2;  // the largest power of two up to 8 that divides the group
  return G;
}

constexpr int AT_MIN_TILES = 8;  // the least number of key tiles that a split keeps

// How the keys of a tile of queries are shared out, from the step's geometry on the host (q_start
// and q_len of the rows the launch covers): key ranges longer than *min_tiles key tiles are cut into
// pieces of that length, at most *splits of them. One CTA fills an SM, so a step with at most one query tile per SM cannot even its load
// out through the queue (nor can one with up to two): the last tiles of a long prompt, or the few tiles of a portion far into a
// long context, walk many more keys than the rest while other SMs idle. Then key ranges longer
// than about 1.2 times the work per SM are cut. With many more tiles than SMs the queue evens the
// load out by itself and splits only add partial results.
// Measured on B200, 16 heads in 8 groups: 256 tokens behind 30,000: 645 us whole, 109 us cut;
// 512 behind 8,192: 193 -> 72 us; one prompt of 2,048 (128 tiles, the last 16 key tiles long):
// 57 us whole, 47 us with ranges over 8 tiles cut in two, 42 us with ranges over 9.
// ms_attn_tc_scratch says how much scratch the splits need.
MS_EXPORT void ms_attn_tc_plan(const int* q_start, const int* q_len, int num_rows, int nq, int nkv, int window, int sm_count,
                               int* splits, int* min_tiles) {
  *splits = 1;
  *min_tiles = AT_MIN_TILES;
  const int G = at_heads_per_cta(nq, nkv), span = 2 * (AT_ROWS / G), head_groups = nq / G;
  long long ctas = 0, steps = 0;
  int longest = 0;
  for (int r = 0; r < num_rows; ++r) {
    for (int m0 = 0; m0 < q_len[r]; m0 += span) {
      const int last = q_start[r] + (m0 + span < q_len[r] ? m0 + span : q_len[r]) - 1;
      const int lo = window > 0 && q_start[r] + m0 - window + 1 > 0 ? q_start[r] + m0 - window + 1 : 0;
      const int n = (last + AT_KEYS) / AT_KEYS - lo / AT_KEYS;
      ctas += head_groups;
      steps += (long long)n * head_groups;
      longest = n > longest ? n : longest;
    }
  }
  if (ctas == 0 || ctas > 2LL * sm_count) return;
  const long long fair = (steps * 12 + 10LL * sm_count - 1) / (10LL * sm_count);  // 1.2 x the work per SM, rounded up
  *min_tiles = (int)(fair < 4 ? 4 : fair);
  const int want = ceil_div(longest, *min_tiles);
  *splits = want < 1 ? 1 : (want > 16 ? 16 : want);
}

// What a launch needs besides its operands: float32 for the partial results of split key ranges
// (none for one split) and int32 for the work queue and the merge tickets; the int32 must be zero
// before the first launch and are left zero by every launch.
MS_EXPORT void ms_attn_tc_scratch(int max_q_len, int num_rows, int nq, int nkv, int splits, long long* partial_floats,
                                  long long* queue_ints) {
  const int G = at_heads_per_cta(nq, nkv);
  const long long units = (long long)ceil_div(max_q_len, 2 * (AT_ROWS / G)) * num_rows * (nq / G) * 2;  // groups of 128 rows
  *partial_floats = splits > 1 ? units * splits * (AT_ROWS * AT_D + AT_ROWS * 2) : 0;
  *queue_ints = 2 + 2 * units;  // the queue's two counters, a ticket and a count of finished splits per group of rows
}

MS_EXPORT int ms_attn_tc_prefill(void* out, const void* q, const void* k_pool, const void* v_pool, const int* cu_q,
                                 const int* q_start, const int* page_indptr, const int* page_indices, int num_rows,
                                 int num_tokens, int max_q_len, int nq, int nkv, long long pool_pages, float scale,
                                 int window, int page_size, int* status, int splits, int min_tiles, float* partials,
                                 int* queue, const int* plan, cudaStream_t stream) {
  // plan: null, or four device ints (tiles of queries per row, rows, key splits, least key tiles per split) that
  // ms_attn_tc_write_plan fills before the launch runs; num_rows, max_q_len, splits and min_tiles are then unused
  if (num_rows == 0 && plan == nullptr) return 0;
  if (plan != nullptr) {
    num_rows = 1;
    max_q_len = num_tokens;
    splits = 2;  // (only says that there is scratch for partial results)
    min_tiles = 1;
  }
  MS_CHECK_ARG(splits >= 1 && splits <= 64 && min_tiles >= 1, "attention_tc: %d key splits of at least %d tiles", splits, min_tiles);
  // partials and queue: sized by ms_attn_tc_scratch (the work queue's two counters, then the tickets
  // of the groups whose keys are split)
  MS_CHECK_ARG(queue != nullptr, "attention_tc: the work queue is missing");
  MS_CHECK_ARG(splits == 1 || (partials != nullptr && (uintptr_t)partials % 16 == 0),
               "attention_tc: key splits need scratch for the partial results");
  MS_CHECK_ARG(ms_attn_tc_supports(AT_D, page_size, nq, nkv), "attention_tc: unsupported shape (page_size=%d)", page_size);
  MS_CHECK_ARG(((uintptr_t)q % 16 == 0) && ((uintptr_t)k_pool % 16 == 0) && ((uintptr_t)v_pool % 16 == 0), "attention_tc: operands must be 16-byte aligned");
  const int G = at_heads_per_cta(nq, nkv);
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
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  constexpr size_t smem_bytes = AtSmem::total + 1024;
  static bool configured = false;
  if (!configured) {
    MS_CHECK_CUDA(cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
    configured = true;
  }
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    MS_CHECK_CUDA(cudaGetDevice(&dev));
    MS_CHECK_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
  }
  const AtGrid gr = {ceil_div(max_q_len, 2 * tpc), num_rows, nq / G, splits, min_tiles, window, G};
  const long long total = (long long)gr.q_tiles * gr.rows * gr.head_groups * gr.splits;
  MS_CHECK_ARG(total < (1LL << 30), "attention_tc: %lld work items are too many for one launch", total);
  // one CTA fills an SM (192 KB of shared memory, all of tensor memory) and takes items until none is left
  const unsigned grid = (unsigned)(plan == nullptr && total < sm_count ? total : sm_count);
  MS_LAUNCH(attn_prefill_tc_kernel, grid, AT_THREADS, smem_bytes, stream, map_q, map_k, map_v, (__nv_bfloat16*)out, cu_q,
            q_start, page_indptr, page_indices, nq, nkv, scale * AT_LOG2E, page_shift, gr, status,
            partials, reinterpret_cast<float2*>(partials + (total / gr.splits) * 2 * gr.splits * (AT_ROWS * AT_D)), queue,
            queue + 2, plan);
  return 0;
}

namespace ms {
__global__ void attn_tc_plan_kernel(int* __restrict__ plan, int q_tiles, int rows, int splits, int min_tiles) {
  pdl_prologue();
  plan[0] = q_tiles;
  plan[1] = rows;
  plan[2] = splits;
  plan[3] = min_tiles;
}
}  // namespace ms

// Plans a step's attention as ms_attn_tc_plan does and puts the plan where a captured launch reads it
// (a one-thread kernel in stream order: its arguments travel with the launch, so no host buffer has to
// outlive the call). The key splits are cut down until their partial results fit partial_floats; the
// work queue must hold queue_ints.
MS_EXPORT int ms_attn_tc_write_plan(int* plan, const int* q_start, const int* q_len, int num_rows, int max_q_len, int nq, int nkv,
                                    int window, int sm_count, long long partial_floats, long long queue_ints, cudaStream_t stream) {
  MS_CHECK_ARG(plan != nullptr && num_rows > 0 && max_q_len > 0, "attention_tc: a plan needs rows");
  int splits = 1, min_tiles = AT_MIN_TILES;
  ms_attn_tc_plan(q_start, q_len, num_rows, nq, nkv, window, sm_count, &splits, &min_tiles);
  long long need_f = 0, need_i = 0;
  for (;; --splits) {
    ms_attn_tc_scratch(max_q_len, num_rows, nq, nkv, splits, &need_f, &need_i);
    if (splits == 1 || need_f <= partial_floats) break;
  }
  MS_CHECK_ARG(need_i <= queue_ints, "attention_tc: the work queue holds %lld entries, the step needs %lld", queue_ints, need_i);
  const int G = at_heads_per_cta(nq, nkv);
  MS_LAUNCH(attn_tc_plan_kernel, 1, 1, 0, stream, plan, ceil_div(max_q_len, 2 * (AT_ROWS / G)), num_rows, splits, min_tiles);
  return 0;
}
