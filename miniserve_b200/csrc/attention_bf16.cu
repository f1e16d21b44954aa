// bfloat16 attention over the paged cache on the tensor cores, compiled for ONE head size
// (-DMS_HEAD_DIM=D, a multiple of 16 up to 256): a causal grouped-query kernel for prompts and
// mixed steps, and a split-K kernel plus merge for decode-only steps.
//
// Formula: softmax(q k^T * scale + causal mask) v, query head h reading kv head h / (heads /
// kv_heads) (miniserve/model/attention.py:60-67,125-133; miniserve/model/qwen3.py:133-135). A query
// row r of a request sits at absolute position q_start + r and sees keys 0 .. that position (or the
// last `window` of them). These kernels stand where the reference calls FlashInfer's batch
// prefill and batch decode wrappers (miniserve/model/attention.py:97-101,136-140).
//
// Scores, the running maximum and sum, and the output accumulator are float32; probabilities are
// rounded to bfloat16 for the second product. Keys and values come from pages
// [pages, kv_heads, page_size, D] through cp.async into padded shared-memory tiles; rows past the
// end of a request are zero-filled, never read.
#include <cfloat>

#include <cooperative_groups.h>

#include "common.cuh"

#ifndef MS_HEAD_DIM
#error "compile with -DMS_HEAD_DIM=<head size>"
#endif

namespace ms {

constexpr int D = MS_HEAD_DIM;
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head size must be a multiple of 16 up to 256");
constexpr int DPAD = D + 8;          // row stride in shared memory (bf16): conflict-free ldmatrix
constexpr int KSTEPS = D / 16;       // k-steps of q k^T
constexpr int DTILES = D / 8;        // n-tiles of p v
constexpr int CHUNKS = D / 8;        // 16-byte chunks per row
constexpr bool Q_IN_REGS = D <= 128;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;  // 0: the 16 bytes are zero-filled and nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

struct PagedKV {
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const int* pages;  // this request's page ids
  int kv_head, nkv, page_shift;
  __device__ __forceinline__ size_t row_offset(int key) const {
    const int page = pages[key >> page_shift];
    const int page_size = 1 << page_shift;
    return (((size_t)max(page, 0) * nkv + kv_head) * page_size + (key & (page_size - 1))) * D;
  }
};

// Copy keys [key0, key0 + ROWS) of K and V into padded tiles; rows outside [lo, hi) are zero-filled.
template <int ROWS, int THREADS>
__device__ __forceinline__ void load_kv_tile(__nv_bfloat16* ks, __nv_bfloat16* vs, const PagedKV& kv, int key0, int lo,
                                             int hi, int tid) {
  for (int idx = tid; idx < ROWS * CHUNKS; idx += THREADS) {
    const int row = idx / CHUNKS, chunk = idx - row * CHUNKS;
    const int key = key0 + row;
    const bool valid = key >= lo && key < hi;
    const size_t off = valid ? kv.row_offset(key) + chunk * 8 : 0;
    cp_async16(ks + row * DPAD + chunk * 8, kv.k + off, valid);
    cp_async16(vs + row * DPAD + chunk * 8, kv.v + off, valid);
  }
}

// ------------------------------------------------------------------ prompts and mixed steps
constexpr int PF_BM = 64, PF_BN = 64, PF_THREADS = 128;

__global__ void __launch_bounds__(PF_THREADS)
attn_prefill_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ q,
                    const __nv_bfloat16* __restrict__ k_pool, const __nv_bfloat16* __restrict__ v_pool,
                    const int* __restrict__ cu_q, const int* __restrict__ q_start, const int* __restrict__ page_indptr,
                    const int* __restrict__ page_indices, int nq, int nkv, float scale_log2, int window,
                    int page_shift) {
  pdl_prologue();
  const int r = blockIdx.y, head = blockIdx.z;
  const int tok0 = cu_q[r], q_len = cu_q[r + 1] - tok0;
  const int m0 = blockIdx.x * PF_BM;
  if (m0 >= q_len) return;
  const int start = q_start[r];
  const int kv_len = start + q_len;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;

  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [BM][DPAD]
  __nv_bfloat16* ks = qs + PF_BM * DPAD;                            // [2][BN][DPAD]
  __nv_bfloat16* vs = ks + 2 * PF_BN * DPAD;                        // [2][BN][DPAD]

  PagedKV kv{k_pool, v_pool, page_indices + page_indptr[r], head / (nq / nkv), nkv, page_shift};

  // key range this tile of queries can see
  const int q_first = start + m0, q_last = start + min(m0 + PF_BM, q_len) - 1;
  const int hi = min(kv_len, q_last + 1);
  const int lo = window > 0 ? max(0, q_first - window + 1) : 0;
  const int tile_begin = lo / PF_BN, tile_end = (hi + PF_BN - 1) / PF_BN;

  // q tile
  for (int idx = tid; idx < PF_BM * CHUNKS; idx += PF_THREADS) {
    const int row = idx / CHUNKS, chunk = idx - row * CHUNKS;
    const bool valid = m0 + row < q_len;
    const __nv_bfloat16* src = q + ((size_t)(tok0 + (valid ? m0 + row : 0)) * nq + head) * D + chunk * 8;
    cp_async16(qs + row * DPAD + chunk * 8, src, valid);
  }
  load_kv_tile<PF_BN, PF_THREADS>(ks, vs, kv, tile_begin * PF_BN, lo, hi, tid);
  cp_async_commit();

  uint32_t qf[Q_IN_REGS ? KSTEPS : 1][4];
  float o[DTILES][4];
#pragma unroll
  for (int i = 0; i < DTILES; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int qpos[2] = {start + m0 + warp * 16 + g, start + m0 + warp * 16 + g + 8};

  for (int tile = tile_begin; tile < tile_end; ++tile) {
    const int stage = (tile - tile_begin) & 1;
    if (tile + 1 < tile_end)
      load_kv_tile<PF_BN, PF_THREADS>(ks + (stage ^ 1) * PF_BN * DPAD, vs + (stage ^ 1) * PF_BN * DPAD, kv,
                                      (tile + 1) * PF_BN, lo, hi, tid);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (Q_IN_REGS && tile == tile_begin) {
#pragma unroll
      for (int kk = 0; kk < (Q_IN_REGS ? KSTEPS : 1); ++kk)
        ldmatrix_x4(qf[kk], qs + (warp * 16 + (lane & 15)) * DPAD + kk * 16 + (lane >> 4) * 8);
    }
    const __nv_bfloat16* kt = ks + stage * PF_BN * DPAD;
    const __nv_bfloat16* vt = vs + stage * PF_BN * DPAD;

    float s[PF_BN / 8][4];
#pragma unroll
    for (int i = 0; i < PF_BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      uint32_t a[4];
      if (Q_IN_REGS) {
        a[0] = qf[kk][0]; a[1] = qf[kk][1]; a[2] = qf[kk][2]; a[3] = qf[kk][3];
      } else {
        ldmatrix_x4(a, qs + (warp * 16 + (lane & 15)) * DPAD + kk * 16 + (lane >> 4) * 8);
      }
#pragma unroll
      for (int np = 0; np < PF_BN / 16; ++np) {
        uint32_t b[4];
        ldmatrix_x4(b, kt + (np * 16 + (lane & 7) + ((lane >> 4) << 3)) * DPAD + kk * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[2 * np], a, b[0], b[1]);
        mma_bf16(s[2 * np + 1], a, b[2], b[3]);
      }
    }
    // mask, then the running softmax of rows g and g + 8
    const int key_base = tile * PF_BN + 2 * t;
    float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
    for (int nt = 0; nt < PF_BN / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key_base + nt * 8 + (e & 1);
        const int qp = qpos[e >> 1];
        const bool ok = key <= qp && key >= lo && (window <= 0 || key > qp - window);
        s[nt][e] = ok ? s[nt][e] * scale_log2 : -INFINITY;
        m_new[e >> 1] = fmaxf(m_new[e >> 1], s[nt][e]);
      }
    float alpha[2], m_use[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      m_new[i] = quad_max(m_new[i]);
      m_use[i] = m_new[i] == -INFINITY ? 0.f : m_new[i];
      alpha[i] = exp2f(m_run[i] - m_use[i]);  // m_run = -inf gives 0
      m_run[i] = m_new[i];
    }
    float row_sum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < PF_BN / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        s[nt][e] = exp2f(s[nt][e] - m_use[e >> 1]);
        row_sum[e >> 1] += s[nt][e];
      }
#pragma unroll
    for (int i = 0; i < 2; ++i) l_run[i] = l_run[i] * alpha[i] + row_sum[i];
#pragma unroll
    for (int dt = 0; dt < DTILES; ++dt) {
      o[dt][0] *= alpha[0]; o[dt][1] *= alpha[0]; o[dt][2] *= alpha[1]; o[dt][3] *= alpha[1];
    }
#pragma unroll
    for (int kk = 0; kk < PF_BN / 16; ++kk) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int dp = 0; dp < DTILES / 2; ++dp) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * DPAD + dp * 16 + (lane >> 4) * 8);
        mma_bf16(o[2 * dp], a, b[0], b[1]);
        mma_bf16(o[2 * dp + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();  // everyone is done with this stage before it is loaded again
  }
  cp_async_wait<0>();
#pragma unroll
  for (int i = 0; i < 2; ++i) l_run[i] = quad_sum(l_run[i]);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = m0 + warp * 16 + g + 8 * i;
    if (row >= q_len) continue;
    const float inv = 1.0f / l_run[i];
    __nv_bfloat16* dst = out + ((size_t)(tok0 + row) * nq + head) * D + 2 * t;
#pragma unroll
    for (int dt = 0; dt < DTILES; ++dt)
      *reinterpret_cast<uint32_t*>(dst + dt * 8) = pack_bf16(o[dt][2 * i] * inv, o[dt][2 * i + 1] * inv);
  }
}

// ------------------------------------------------------------------ decode: split-K over the keys
// One CTA per (split, request, kv head x 16 query heads of its group). The four warps take
// 16-key slices of the CTA's key range in turn; each warp runs its own cp.async pipeline into
// its own shared memory, so no block-wide barrier sits in the loop. At the end the warps' partial
// (max, sum, output) lie in shared memory. Splits that run as one thread-block cluster add up all
// warps' partials of all splits from there, each CTA its share of the output; otherwise the CTA
// merges its warps and writes one partial per split, or the final output when there is a single split.
constexpr int DC_WARPS = 4, DC_THREADS = DC_WARPS * 32, DC_STAGES = 3, DC_SLICE = 16;

struct DecodeSmem {
  static constexpr int q_elems = 16 * DPAD;
  static constexpr int stage_elems = 2 * DC_SLICE * DPAD;  // K slice then V slice
  static constexpr int pipe_elems = DC_WARPS * DC_STAGES * stage_elems;
  static constexpr size_t bytes_pipe = (size_t)(q_elems + pipe_elems) * 2;
  static constexpr size_t bytes_merge = (size_t)DC_WARPS * 16 * (D + 2) * 4 + (size_t)q_elems * 2;
  static constexpr size_t bytes = bytes_pipe > bytes_merge ? bytes_pipe : bytes_merge;
};

__global__ void __launch_bounds__(DC_THREADS)
attn_decode_kernel(__nv_bfloat16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                   const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                   const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ kv_len_ptr,
                   const int* __restrict__ page_indptr, const int* __restrict__ page_indices, int nq, int nkv,
                   float scale_log2, int window, int page_shift, int num_splits, int* __restrict__ counters,
                   int cluster_merge) {
  // Until pdl_wait() below, only data written before this step is touched: the step's metadata and
  // the keys and values of older tokens. So the CTA may start streaming them while the kernels
  // before it (the q/k/v projection, the rotation and cache write) are still running.
  pdl_launch_dependents();
  const int split = blockIdx.x, r = blockIdx.y;
  const int group = nq / nkv, chunks_per_group = (group + 15) / 16;
  const int kvh = blockIdx.z / chunks_per_group, head0 = kvh * group + (blockIdx.z % chunks_per_group) * 16;
  const int heads_here = min(16, kvh * group + group - head0);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int kv_len = kv_len_ptr[r];
  const int lo = window > 0 ? max(0, kv_len - window) : 0;
  // the key range of this split, in whole slices
  const int first_slice = lo / DC_SLICE, end_slice = (kv_len + DC_SLICE - 1) / DC_SLICE;
  const int per_split = (end_slice - first_slice + num_splits - 1) / num_splits;
  const int s_begin = first_slice + split * per_split, s_end = min(end_slice, s_begin + per_split);

  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* pipe = qs + DecodeSmem::q_elems + warp * DC_STAGES * DecodeSmem::stage_elems;

  PagedKV kv{k_pool, v_pool, page_indices + page_indptr[r], kvh, nkv, page_shift};

  float o[DTILES][4];
#pragma unroll
  for (int i = 0; i < DTILES; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  // this warp's slices: s_begin + warp, + DC_WARPS, ...
  const int my_first = s_begin + warp;
  const int my_count = my_first < s_end ? (s_end - my_first + DC_WARPS - 1) / DC_WARPS : 0;
  auto issue = [&](int i) {
    if (i < my_count) {
      __nv_bfloat16* st = pipe + (i % DC_STAGES) * DecodeSmem::stage_elems;
      const int key0 = (my_first + i * DC_WARPS) * DC_SLICE;
      if (page_shift >= 4) {
        // pages of at least 16 tokens: the whole slice lies in one page, one lookup per slice
        const int page = kv.pages[key0 >> page_shift];
        const size_t base = ((((size_t)max(page, 0) * nkv + kvh) << page_shift) + (key0 & ((1 << page_shift) - 1))) * D;
#pragma unroll
        for (int it = 0; it < DC_SLICE * CHUNKS / 32; ++it) {
          const int idx = it * 32 + lane, row = idx / CHUNKS, chunk = idx - row * CHUNKS;
          const bool valid = key0 + row >= lo && key0 + row < kv_len;
          const size_t off = valid ? base + row * D + chunk * 8 : 0;
          cp_async16(st + row * DPAD + chunk * 8, kv.k + off, valid);
          cp_async16(st + (DC_SLICE + row) * DPAD + chunk * 8, kv.v + off, valid);
        }
      } else {
        load_kv_tile<DC_SLICE, 32>(st, st + DC_SLICE * DPAD, kv, key0, lo, kv_len, lane);
      }
    }
    cp_async_commit();
  };
  // Fill the pipeline with slices of older tokens; the slice that holds this step's own token
  // (written by the kernel before this one) and the queries come after the wait.
  const int newest_slice = (kv_len - 1) / DC_SLICE;
  int issued = 0;
  for (; issued < DC_STAGES - 1; ++issued) {
    if (issued < my_count && my_first + issued * DC_WARPS >= newest_slice) break;
    issue(issued);
  }
  pdl_wait();
  for (int idx = tid; idx < 16 * CHUNKS; idx += DC_THREADS) {
    const int row = idx / CHUNKS, chunk = idx - row * CHUNKS;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row < heads_here) v = *reinterpret_cast<const uint4*>(q + ((size_t)r * nq + head0 + row) * D + chunk * 8);
    *reinterpret_cast<uint4*>(qs + row * DPAD + chunk * 8) = v;
  }
  for (; issued < DC_STAGES - 1; ++issued) issue(issued);
  __syncthreads();
  uint32_t qf[Q_IN_REGS ? KSTEPS : 1][4];
  if (Q_IN_REGS) {
#pragma unroll
    for (int kk = 0; kk < (Q_IN_REGS ? KSTEPS : 1); ++kk)
      ldmatrix_x4(qf[kk], qs + (lane & 15) * DPAD + kk * 16 + (lane >> 4) * 8);
  }

  for (int i = 0; i < my_count; ++i) {
    issue(i + DC_STAGES - 1);
    cp_async_wait<DC_STAGES - 1>();
    __syncwarp();
    const __nv_bfloat16* kt = pipe + (i % DC_STAGES) * DecodeSmem::stage_elems;
    const __nv_bfloat16* vt = kt + DC_SLICE * DPAD;
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      uint32_t a[4], b[4];
      if (Q_IN_REGS) {
        a[0] = qf[kk][0]; a[1] = qf[kk][1]; a[2] = qf[kk][2]; a[3] = qf[kk][3];
      } else {
        ldmatrix_x4(a, qs + (lane & 15) * DPAD + kk * 16 + (lane >> 4) * 8);
      }
      ldmatrix_x4(b, kt + ((lane & 7) + ((lane >> 4) << 3)) * DPAD + kk * 16 + ((lane >> 3) & 1) * 8);
      mma_bf16(s[0], a, b[0], b[1]);
      mma_bf16(s[1], a, b[2], b[3]);
    }
    const int key_base = (my_first + i * DC_WARPS) * DC_SLICE + 2 * t;
    float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key_base + nt * 8 + (e & 1);
        const bool ok = key >= lo && key < kv_len;
        s[nt][e] = ok ? s[nt][e] * scale_log2 : -INFINITY;
        m_new[e >> 1] = fmaxf(m_new[e >> 1], s[nt][e]);
      }
    float alpha[2], m_use[2], row_sum[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      m_new[j] = quad_max(m_new[j]);
      m_use[j] = m_new[j] == -INFINITY ? 0.f : m_new[j];
      alpha[j] = exp2f(m_run[j] - m_use[j]);
      m_run[j] = m_new[j];
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        s[nt][e] = exp2f(s[nt][e] - m_use[e >> 1]);
        row_sum[e >> 1] += s[nt][e];
      }
#pragma unroll
    for (int j = 0; j < 2; ++j) l_run[j] = l_run[j] * alpha[j] + row_sum[j];
    uint32_t a[4];
    a[0] = pack_bf16(s[0][0], s[0][1]);
    a[1] = pack_bf16(s[0][2], s[0][3]);
    a[2] = pack_bf16(s[1][0], s[1][1]);
    a[3] = pack_bf16(s[1][2], s[1][3]);
    // the running maximum rarely moves after the first slices: rescale only when it did
    if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
      for (int dt = 0; dt < DTILES; ++dt) {
        o[dt][0] *= alpha[0]; o[dt][1] *= alpha[0]; o[dt][2] *= alpha[1]; o[dt][3] *= alpha[1];
      }
    }
#pragma unroll
    for (int dp = 0; dp < DTILES / 2; ++dp) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, vt + ((lane & 7) + ((lane >> 3) & 1) * 8) * DPAD + dp * 16 + (lane >> 4) * 8);
      mma_bf16(o[2 * dp], a, b[0], b[1]);
      mma_bf16(o[2 * dp + 1], a, b[2], b[3]);
    }
    __syncwarp();
  }
  cp_async_wait<0>();
#pragma unroll
  for (int j = 0; j < 2; ++j) l_run[j] = quad_sum(l_run[j]);
  __syncthreads();  // the pipelines are drained: shared memory becomes the merge area

  float* merge = reinterpret_cast<float*>(smem_raw + (size_t)DecodeSmem::q_elems * 2);  // [warps][16][D + 2]
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    if (g + 8 * j >= heads_here) continue;  // rows of the tile that stand for no query head
    float* row = merge + ((size_t)warp * 16 + g + 8 * j) * (D + 2);
#pragma unroll
    for (int dt = 0; dt < DTILES; ++dt) {
      row[dt * 8 + 2 * t] = o[dt][2 * j];
      row[dt * 8 + 2 * t + 1] = o[dt][2 * j + 1];
    }
    if (t == 0) {
      row[D] = m_run[j];
      row[D + 1] = l_run[j];
    }
  }
  if (num_splits > 1 && cluster_merge) {
    // The splits of a (request, head group) are one thread-block cluster. Every warp's partial result
    // stays in its CTA's shared memory; after one cluster barrier each CTA adds up its share of the
    // output's elements over all warps of all splits through distributed shared memory:
    // out = sum_p w_p O_p / sum_p w_p l_p with w_p = 2^(m_p - max m). All of a batch's values are asked
    // for together (one trip to the other CTAs' shared memory), four splits to a batch.
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    const int total = heads_here * D, share = (total + num_splits - 1) / num_splits;
    const int first = (int)cluster.block_rank() * share, last = min(total, first + share);
    for (int idx = first + tid; idx < last; idx += DC_THREADS) {
      const int row = idx / D, c = idx - row * D;
      float acc = 0.f, l = 0.f, m = -INFINITY;
      for (int s0 = 0; s0 < num_splits; s0 += 4) {
        float ms[4 * DC_WARPS], ls[4 * DC_WARPS], os[4 * DC_WARPS];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const bool in = s0 + i < num_splits;
          const float* base = cluster.map_shared_rank(merge, in ? s0 + i : 0) + (size_t)row * (D + 2);
#pragma unroll
          for (int w = 0; w < DC_WARPS; ++w) {
            const float* src = base + (size_t)w * 16 * (D + 2);
            ms[i * DC_WARPS + w] = in ? src[D] : -INFINITY;
            ls[i * DC_WARPS + w] = in ? src[D + 1] : 0.f;
            os[i * DC_WARPS + w] = in ? src[c] : 0.f;
          }
        }
        float m_new = m;
#pragma unroll
        for (int i = 0; i < 4 * DC_WARPS; ++i) m_new = fmaxf(m_new, ms[i]);
        if (m_new == -INFINITY) continue;
        const float keep = m == -INFINITY ? 0.f : exp2f(m - m_new);
        acc *= keep;
        l *= keep;
        m = m_new;
#pragma unroll
        for (int i = 0; i < 4 * DC_WARPS; ++i) {
          const float wgt = ms[i] == -INFINITY ? 0.f : exp2f(ms[i] - m);
          acc += wgt * os[i];
          l += wgt * ls[i];
        }
      }
      out[((size_t)r * nq + head0 + row) * D + c] = __float2bfloat16_rn(acc / l);
    }
    cluster.sync();  // shared memory lives until every CTA of the cluster has read it
    return;
  }
  __syncthreads();
  for (int idx = tid; idx < heads_here * D; idx += DC_THREADS) {
    const int row = idx / D, c = idx - row * D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < DC_WARPS; ++w) m = fmaxf(m, merge[((size_t)w * 16 + row) * (D + 2) + D]);
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < DC_WARPS; ++w) {
      const float* src = merge + ((size_t)w * 16 + row) * (D + 2);
      const float wgt = src[D] == -INFINITY ? 0.f : exp2f(src[D] - m);
      acc += wgt * src[c];
      l += wgt * src[D + 1];
    }
    const int head = head0 + row;
    if (num_splits == 1) {
      out[((size_t)r * nq + head) * D + c] = __float2bfloat16_rn(acc / l);
    } else {
      const size_t p = ((size_t)r * nq + head) * num_splits + split;
      part_o[p * D + c] = acc;
      if (c == 0) {
        part_ml[2 * p] = m;
        part_ml[2 * p + 1] = l;
      }
    }
  }
  if (num_splits == 1 || counters == nullptr) return;
  // The split that finishes last merges them all (a ticket per (request, head chunk); no waiting):
  // out = sum_s w_s O_s / sum_s w_s l_s with w_s = 2^(m_s - max m).
  __shared__ int last_one;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    int* ticket = counters + (size_t)r * gridDim.z + blockIdx.z;
    const int prev = atomicAdd(ticket, 1);
    last_one = prev == num_splits - 1;
    if (last_one) *ticket = 0;  // ready for the next launch
  }
  __syncthreads();
  if (!last_one) return;
  __threadfence();
  for (int idx = tid; idx < heads_here * D; idx += DC_THREADS) {
    const int row = idx / D, c = idx - row * D;
    const size_t item = (size_t)r * nq + head0 + row;
    const float2* ml = reinterpret_cast<const float2*>(part_ml) + item * num_splits;
    const float* po = part_o + item * num_splits * D + c;
    float acc = 0.f, l = 0.f, m = -INFINITY;
    // splits in groups of eight: the loads of a group are in flight together (they are what this
    // tail waits for); the result is rescaled when a later group raises the maximum
    for (int s0 = 0; s0 < num_splits; s0 += 8) {
      float2 mls[8];
      float os[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const bool in = s0 + i < num_splits;
        mls[i] = in ? __ldcg(ml + s0 + i) : make_float2(-INFINITY, 0.f);
        os[i] = in ? __ldcg(po + (size_t)(s0 + i) * D) : 0.f;
      }
      float m_new = m;
#pragma unroll
      for (int i = 0; i < 8; ++i) m_new = fmaxf(m_new, mls[i].x);
      if (m_new == -INFINITY) continue;
      const float keep = m == -INFINITY ? 0.f : exp2f(m - m_new);
      acc *= keep;
      l *= keep;
      m = m_new;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float wgt = mls[i].x == -INFINITY ? 0.f : exp2f(mls[i].x - m);
        acc += wgt * os[i];
        l += wgt * mls[i].y;
      }
    }
    out[item * D + c] = __float2bfloat16_rn(acc / l);
  }
}

// out[r, head] = sum_s w_s O_s / sum_s w_s l_s with w_s = 2^(m_s - max m)
__global__ void attn_decode_merge_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ part_o,
                                         const float* __restrict__ part_ml, int num_splits) {
  pdl_prologue();
  const size_t item = blockIdx.x;  // r * nq + head
  const float* ml = part_ml + item * num_splits * 2;
  float m = -INFINITY;
  for (int s = 0; s < num_splits; ++s) m = fmaxf(m, ml[2 * s]);
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    float acc = 0.f, l = 0.f;
    for (int s = 0; s < num_splits; ++s) {
      const float ms_ = ml[2 * s];
      const float wgt = ms_ == -INFINITY ? 0.f : exp2f(ms_ - m);
      acc += wgt * part_o[(item * num_splits + s) * D + c];
      l += wgt * ml[2 * s + 1];
    }
    out[item * D + c] = __float2bfloat16_rn(acc / l);
  }
}

}  // namespace ms

using namespace ms;

#define MS_CAT2(a, b) a##b
#define MS_CAT(a, b) MS_CAT2(a, b)
#define MS_ATTN_FN(name) MS_CAT(MS_CAT(MS_CAT(ms_attn_bf16_d, MS_HEAD_DIM), _), name)

MS_DEFINE_LAST_ERROR(MS_ATTN_FN(last_error))
MS_DEFINE_PDL_SWITCH(MS_ATTN_FN(set_pdl))

MS_EXPORT int MS_ATTN_FN(head_dim)() { return D; }

static int shift_of(int page_size) {
  int s = 0;
  while ((1 << s) < page_size) ++s;
  return s;
}

MS_EXPORT int MS_ATTN_FN(prefill)(void* out, const void* q, const void* k_pool, const void* v_pool, const int* cu_q,
                                  const int* q_start, const int* page_indptr, const int* page_indices, int num_rows,
                                  int max_q_len, int nq, int nkv, float scale, int window, int page_size,
                                  cudaStream_t stream) {
  if (num_rows == 0) return 0;
  MS_CHECK_ARG(nq > 0 && nkv > 0 && nq % nkv == 0, "attention: %d query heads are not a multiple of %d kv heads", nq, nkv);
  MS_CHECK_ARG(page_size > 0 && (page_size & (page_size - 1)) == 0, "attention: page_size=%d must be a power of two", page_size);
  MS_CHECK_ARG(num_rows <= 65535 && nq <= 65535, "attention: too many rows (%d) or heads (%d) for one launch", num_rows, nq);
  const size_t smem = (size_t)(PF_BM + 4 * PF_BN) * DPAD * 2;
  static bool configured[64] = {};  // the attribute belongs to a device
  int dev = 0;
  MS_CHECK_CUDA(cudaGetDevice(&dev));
  MS_CHECK_ARG(dev >= 0 && dev < 64, "attention: device index %d is not supported", dev);
  if (!configured[dev]) {
    MS_CHECK_CUDA(cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev] = true;
  }
  dim3 grid(ceil_div(max_q_len, PF_BM), num_rows, nq);
  MS_LAUNCH(attn_prefill_kernel, grid, PF_THREADS, smem, stream,
      (__nv_bfloat16*)out, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, cu_q,
      q_start, page_indptr, page_indices, nq, nkv, scale * LOG2E, window, shift_of(page_size));
  MS_CHECK_LAUNCH();
  return 0;
}

MS_EXPORT int MS_ATTN_FN(decode_fused)(void* out, void* part_o, void* part_ml, int* counters, const void* q,
                                       const void* k_pool, const void* v_pool, const int* kv_len,
                                       const int* page_indptr, const int* page_indices, int num_rows, int nq, int nkv,
                                       float scale, int window, int page_size, int num_splits, cudaStream_t stream);

// The decode kernel's shared-memory attribute belongs to a device: set once for each.
static int configure_decode() {
  static bool configured[64] = {};
  int dev = 0;
  MS_CHECK_CUDA(cudaGetDevice(&dev));
  MS_CHECK_ARG(dev >= 0 && dev < 64, "attention: device index %d is not supported", dev);
  if (!configured[dev]) {
    MS_CHECK_CUDA(cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DecodeSmem::bytes));
    configured[dev] = true;
  }
  return 0;
}

// Scratch for num_splits > 1: part_o [rows, nq, splits, D] floats and part_ml [rows, nq, splits, 2] floats.
MS_EXPORT int MS_ATTN_FN(decode)(void* out, void* part_o, void* part_ml, const void* q, const void* k_pool,
                                 const void* v_pool, const int* kv_len, const int* page_indptr,
                                 const int* page_indices, int num_rows, int nq, int nkv, float scale, int window,
                                 int page_size, int num_splits, cudaStream_t stream) {
  return MS_ATTN_FN(decode_fused)(out, part_o, part_ml, nullptr, q, k_pool, v_pool, kv_len, page_indptr, page_indices,
                                  num_rows, nq, nkv, scale, window, page_size, num_splits, stream);
}

// As above; with `counters` (num_rows * kv_heads * ceil(group / 16) ints, zero before the first
// launch, left zero by every launch) the split that finishes last merges the partial results
// inside the same kernel and no second kernel is launched.
MS_EXPORT int MS_ATTN_FN(decode_fused)(void* out, void* part_o, void* part_ml, int* counters, const void* q,
                                       const void* k_pool, const void* v_pool, const int* kv_len,
                                       const int* page_indptr, const int* page_indices, int num_rows, int nq, int nkv,
                                       float scale, int window, int page_size, int num_splits, cudaStream_t stream) {
  if (num_rows == 0) return 0;
  MS_CHECK_ARG(nq > 0 && nkv > 0 && nq % nkv == 0, "attention: %d query heads are not a multiple of %d kv heads", nq, nkv);
  MS_CHECK_ARG(page_size > 0 && (page_size & (page_size - 1)) == 0, "attention: page_size=%d must be a power of two", page_size);
  MS_CHECK_ARG(num_splits >= 1 && num_splits <= 65535, "attention: bad split count %d", num_splits);
  MS_CHECK_ARG(num_splits == 1 || (part_o != nullptr && part_ml != nullptr), "attention: splits need scratch memory");
  MS_CHECK_ARG(num_rows <= 65535, "attention: too many rows (%d) for one launch", num_rows);
  const int group = nq / nkv;
  if (int rc = configure_decode()) return rc;
  dim3 grid(num_splits, num_rows, nkv * ceil_div(group, 16));
  MS_LAUNCH(attn_decode_kernel, grid, DC_THREADS, DecodeSmem::bytes, stream,
      (__nv_bfloat16*)out, (float*)part_o, (float*)part_ml, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool,
      (const __nv_bfloat16*)v_pool, kv_len, page_indptr, page_indices, nq, nkv, scale * LOG2E, window,
      shift_of(page_size), num_splits, counters, 0);
  if (num_splits > 1 && counters == nullptr) {
    MS_LAUNCH(attn_decode_merge_kernel, num_rows * nq, D >= 128 ? 128 : 64, 0, stream, (__nv_bfloat16*)out,
              (const float*)part_o, (const float*)part_ml, num_splits);
  }
  return 0;
}

// The same with the splits of a (request, head group) as one thread-block cluster (2 to 8 splits):
// partial results stay in shared memory and the cluster's first CTA adds them up through
// distributed shared memory, so no scratch, no fence and no ticket are needed.
MS_EXPORT int MS_ATTN_FN(decode_cluster)(void* out, const void* q, const void* k_pool, const void* v_pool, const int* kv_len,
                                         const int* page_indptr, const int* page_indices, int num_rows, int nq, int nkv,
                                         float scale, int window, int page_size, int num_splits, cudaStream_t stream) {
  if (num_rows == 0) return 0;
  MS_CHECK_ARG(nq > 0 && nkv > 0 && nq % nkv == 0, "attention: %d query heads are not a multiple of %d kv heads", nq, nkv);
  MS_CHECK_ARG(page_size > 0 && (page_size & (page_size - 1)) == 0, "attention: page_size=%d must be a power of two", page_size);
  MS_CHECK_ARG(num_splits >= 2 && num_splits <= 8, "attention: a cluster takes 2 to 8 splits, not %d", num_splits);
  MS_CHECK_ARG(num_rows <= 65535, "attention: too many rows (%d) for one launch", num_rows);
  const int group = nq / nkv;
  if (int rc = configure_decode()) return rc;
  dim3 grid(num_splits, num_rows, nkv * ceil_div(group, 16));
  MS_LAUNCH_CLUSTERED(attn_decode_kernel, grid, DC_THREADS, DecodeSmem::bytes, stream, num_splits,
      (__nv_bfloat16*)out, (float*)nullptr, (float*)nullptr, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool,
      (const __nv_bfloat16*)v_pool, kv_len, page_indptr, page_indices, nq, nkv, scale * LOG2E, window,
      shift_of(page_size), num_splits, (int*)nullptr, 1);
  return 0;
}

// How many clusters of `num_splits` CTAs of the decode kernel this device holds at a time (a cluster
// lies within one GPC, so this is not SM count x 2 / num_splits). A launch with more (request, head
// group) items than that runs in two rounds.
MS_EXPORT int MS_ATTN_FN(decode_clusters_resident)(int num_splits, int* out) {
  MS_CHECK_ARG(num_splits >= 1 && num_splits <= 8, "attention: a cluster takes up to 8 splits, not %d", num_splits);
  static int cached[64][9] = {};
  int dev = 0;
  MS_CHECK_CUDA(cudaGetDevice(&dev));
  MS_CHECK_ARG(dev >= 0 && dev < 64, "attention: device index %d is not supported", dev);
  if (cached[dev][num_splits] == 0) {
    if (int rc = configure_decode()) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(num_splits, 1024, 1);
    cfg.blockDim = dim3(DC_THREADS);
    cfg.dynamicSmemBytes = DecodeSmem::bytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = num_splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    MS_CHECK_CUDA(cudaOccupancyMaxActiveClusters(&n, attn_decode_kernel, &cfg));
    cached[dev][num_splits] = n > 0 ? n : -1;
  }
  *out = cached[dev][num_splits] > 0 ? cached[dev][num_splits] : 0;
  return 0;
}

// ------------------------------------------------------------------ decode without allocation
// See attention_noalloc.h: the same computation as the decode entry point above, with the
// split-K scratch in a file-scope device array instead of caller-provided memory.
#include "attention_noalloc.h"

static __device__ __align__(256) float g_noalloc_scratch[MS_ATTN_NOALLOC_SCRATCH_FLOATS];

// Device address of g_noalloc_scratch per device. In host code the array's name is only a
// stand-in for the symbol, not a device pointer, so the address is looked up once per device
// (with that device current) and passed to the kernels as an ordinary argument.
static int noalloc_scratch_address(float** out) {
  constexpr int MAX_DEVICES = 64;
  static float* address[MAX_DEVICES] = {};
  int device = 0;
  MS_CHECK_CUDA(cudaGetDevice(&device));
  MS_CHECK_ARG(device >= 0 && device < MAX_DEVICES, "decode_noalloc: device index %d is not supported", device);
  if (address[device] == nullptr) {
    void* ptr = nullptr;
    MS_CHECK_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
    MS_CHECK_ARG(ptr != nullptr, "decode_noalloc: the scratch array has no device address");
    address[device] = static_cast<float*>(ptr);
  }
  *out = address[device];
  return 0;
}

MS_EXPORT int MS_ATTN_FN(decode_noalloc)(void* out, const void* q, const void* k_pool, const void* v_pool,
                                         const int* kv_len, const int* page_indptr, const int* page_indices,
                                         int num_rows, int nq, int nkv, float scale, int window, int page_size,
                                         int num_splits, cudaStream_t stream) {
  if (num_rows == 0) return 0;
  MS_CHECK_ARG(num_rows > 0 && nq > 0 && num_splits >= 1, "decode_noalloc: bad sizes rows=%d heads=%d splits=%d", num_rows, nq,
               num_splits);
  float* part_o = nullptr;
  float* part_ml = nullptr;
  if (num_splits > 1) {
    const long long items = (long long)num_rows * nq * num_splits;
    const long long need = items * (D + 2);
    MS_CHECK_ARG(need <= (long long)MS_ATTN_NOALLOC_SCRATCH_FLOATS,
                 "decode_noalloc: rows * heads * splits * (D + 2) = %lld floats of scratch, the built-in array holds %d; "
                 "use fewer splits or rows, or the allocating entry point",
                 need, MS_ATTN_NOALLOC_SCRATCH_FLOATS);
    float* base = nullptr;
    if (int rc = noalloc_scratch_address(&base)) return rc;
    part_o = base;               // [rows, heads, splits, D]
    part_ml = base + items * D;  // [rows, heads, splits, 2]
  }
  return MS_ATTN_FN(decode)(out, part_o, part_ml, q, k_pool, v_pool, kv_len, page_indptr, page_indices, num_rows, nq, nkv,
                            scale, window, page_size, num_splits, stream);
}
