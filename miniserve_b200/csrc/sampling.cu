// Token selection on the device from float32 logits [rows, vocab]: greedy argmax (first maximal
// index wins), temperature sampling by the Gumbel-max trick with hashed noise, and nucleus
// (top-p) masking.
//
// Restates miniserve/engine/sampler.py: :91 (argmax), :95 (z = logits / T in float32), :29-46 (noise:
// u = ((mix32((key + v*0x9E3779B9) mod 2^32) >> 8) + 0.5) / 2^24, key = mix32(seed ^ mix32(counter)),
// mix32 = two rounds of x = ((x >> 16) ^ x) * 0x45D9F3B, then (x >> 16) ^ x), :98-99
// (g = -log(-log u), argmax(z + g)), :102-112 (keep the most likely tokens while the probability
// mass before them is below top_p; ties keep index order). The noise is a pure function of
// (seed, counter, vocabulary index), so a row samples the same token wherever it sits in a batch.
#include <cfloat>

#include <cooperative_groups.h>

#include "common.cuh"

namespace ms {

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x = ((x >> 16) ^ x) * 0x45D9F3Bu;
  x = ((x >> 16) ^ x) * 0x45D9F3Bu;
  return (x >> 16) ^ x;
}

__device__ __forceinline__ float gumbel(uint32_t key, uint32_t v) {
  const uint32_t h = mix32(key + v * 0x9E3779B9u);
  const float u = ((float)(h >> 8) + 0.5f) * (1.0f / 16777216.0f);
  return -logf(-logf(u));
}

struct Best {
  float val;
  int idx;
};
__device__ __forceinline__ Best better(Best a, Best b) {
  // larger value wins; on equal values the lower index wins
  if (b.val > a.val || (b.val == a.val && b.idx < a.idx)) return b;
  return a;
}
__device__ __forceinline__ Best block_best(Best b, Best* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other;
    other.val = __shfl_xor_sync(0xffffffffu, b.val, o);
    other.idx = __shfl_xor_sync(0xffffffffu, b.idx, o);
    b = better(b, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = b;
  __syncthreads();
  Best r = scratch[0];
  for (int w = 1; w < nwarps; ++w) r = better(r, scratch[w]);
  return r;
}

// Per row nucleus description written by nucleus_kernel and read by sample_kernel.
struct Nucleus {
  float zmax;     // max of z = logit / T
  float sum;      // sum of exp(z - zmax)
  float cut;      // smallest probability that is kept
  int ties_kept;  // how many tokens with probability == cut are kept, in index order
};

__device__ __forceinline__ float prob_of(float logit, float inv_t, const Nucleus& n) {
  return expf(logit * inv_t - n.zmax) / n.sum;
}

// One block per row. 31-step search over the bit pattern of the cut probability.
__global__ void __launch_bounds__(1024)
nucleus_kernel(Nucleus* __restrict__ out, const float* __restrict__ logits, const float* __restrict__ temperature,
               const float* __restrict__ top_p, int vocab) {
  __shared__ float red[32];
  pdl_prologue();
  const int r = blockIdx.x;
  const float t = temperature[r], tp = top_p[r];
  Nucleus n;
  n.zmax = 0.f; n.sum = 1.f; n.cut = 0.f; n.ties_kept = 0x7fffffff;
  if (!(t > 0.f) || tp >= 1.f) {  // greedy row or whole distribution: nothing to mask
    if (threadIdx.x == 0) out[r] = n;
    return;
  }
  const float inv_t = 1.0f / t;
  const float* lg = logits + (size_t)r * vocab;
  float mx = -INFINITY;
  for (int v = threadIdx.x; v < vocab; v += blockDim.x) mx = fmaxf(mx, lg[v] * inv_t);
  mx = warp_max(mx);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = red[0];
  for (int w = 1; w < (int)(blockDim.x >> 5); ++w) mx = fmaxf(mx, red[w]);
  float s = 0.f;
  for (int v = threadIdx.x; v < vocab; v += blockDim.x) s += expf(lg[v] * inv_t - mx);
  n.zmax = mx;
  n.sum = block_sum(s, red);
  // smallest x (as float bits) with f(x) = sum of probabilities greater than x  <  top_p
  uint32_t lo = 0u, hi = 0x3f800000u;  // f(1.0) = 0 < top_p always holds at hi
  while (lo < hi) {
    const uint32_t mid = lo + ((hi - lo) >> 1);
    const float x = __uint_as_float(mid);
    float f = 0.f;
    for (int v = threadIdx.x; v < vocab; v += blockDim.x) {
      const float p = prob_of(lg[v], inv_t, n);
      if (p > x) f += p;
    }
    f = block_sum(f, red);
    if (f < tp) hi = mid; else lo = mid + 1;
  }
  n.cut = __uint_as_float(lo);
  float f = 0.f;
  for (int v = threadIdx.x; v < vocab; v += blockDim.x) {
    const float p = prob_of(lg[v], inv_t, n);
    if (p > n.cut) f += p;
  }
  f = block_sum(f, red);
  // the k-th tie (k = 0, 1, ...) is kept while f + k*cut < top_p
  int k = 1;
  if (n.cut > 0.f) {
    const float room = (tp - f) / n.cut;
    k = room >= 2147483000.f ? 0x7fffffff : max(1, (int)ceilf(room));
  } else {
    k = 0x7fffffff;
  }
  n.ties_kept = k;
  if (threadIdx.x == 0) out[r] = n;
}

// One block per row: tokens[r] = argmax(logits) if temperature == 0, else argmax(z + gumbel) over
// the tokens the nucleus keeps.
__global__ void __launch_bounds__(1024)
sample_kernel(int* __restrict__ tokens, const float* __restrict__ logits, const float* __restrict__ temperature,
              const long long* __restrict__ seed, const long long* __restrict__ counter,
              const Nucleus* __restrict__ nucleus, int vocab) {
  __shared__ Best scratch[32];
  __shared__ int tie_base[33];
  pdl_prologue();
  const int r = blockIdx.x;
  const float* lg = logits + (size_t)r * vocab;
  const float t = temperature ? temperature[r] : 0.f;
  Best b;
  b.val = -INFINITY;
  b.idx = 0x7fffffff;
  if (!(t > 0.f)) {
    for (int v = threadIdx.x; v < vocab; v += blockDim.x) {
      const float x = lg[v];
      if (x > b.val) { b.val = x; b.idx = v; }
    }
  } else {
    const float inv_t = 1.0f / t;
    const uint32_t key = mix32((uint32_t)seed[r] ^ mix32((uint32_t)counter[r]));
    const bool masked = nucleus != nullptr && nucleus[r].ties_kept != 0x7fffffff;
    if (!masked) {
      for (int v = threadIdx.x; v < vocab; v += blockDim.x) {
        const float x = lg[v] / t + gumbel(key, (uint32_t)v);
        if (x > b.val) { b.val = x; b.idx = v; }
      }
    } else {
      // Each warp owns a contiguous stretch of the vocabulary so that ties at the cut can be
      // ranked in index order.
      const Nucleus n = nucleus[r];
      const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
      const int per_warp = ((vocab + nwarps - 1) / nwarps + 31) / 32 * 32;
      const int begin = min(warp * per_warp, vocab), end = min(begin + per_warp, vocab);
      int ties = 0;
      for (int v0 = begin; v0 < end; v0 += 32) {
        const int v = v0 + lane;
        const bool tie = v < end && prob_of(lg[v], inv_t, n) == n.cut;
        ties += __popc(__ballot_sync(0xffffffffu, tie));
      }
      if (lane == 0) tie_base[warp + 1] = ties;
      __syncthreads();
      if (threadIdx.x == 0) {
        tie_base[0] = 0;
        for (int w = 0; w < nwarps; ++w) tie_base[w + 1] += tie_base[w];
      }
      __syncthreads();
      int rank0 = tie_base[warp];
      for (int v0 = begin; v0 < end; v0 += 32) {
        const int v = v0 + lane;
        float p = -1.f;
        if (v < end) p = prob_of(lg[v], inv_t, n);
        const bool tie = v < end && p == n.cut;
        const unsigned ballot = __ballot_sync(0xffffffffu, tie);
        const int rank = rank0 + __popc(ballot & ((1u << lane) - 1u));
        rank0 += __popc(ballot);
        const bool keep = v < end && (p > n.cut || (tie && rank < n.ties_kept));
        if (keep) {
          const float x = lg[v] / t + gumbel(key, (uint32_t)v);
          if (x > b.val || (x == b.val && v < b.idx)) { b.val = x; b.idx = v; }
        }
      }
    }
  }
  b = block_best(b, scratch);
  if (threadIdx.x == 0) tokens[r] = b.idx == 0x7fffffff ? 0 : b.idx;
}

// Two-stage selection for rows without a nucleus: stage one takes the best of a stretch of the
// vocabulary per block (so a few rows still use the whole machine), stage two the best of those.
__global__ void __launch_bounds__(256)
sample_partial_kernel(Best* __restrict__ partial, const float* __restrict__ logits,
                      const float* __restrict__ temperature, const long long* __restrict__ seed,
                      const long long* __restrict__ counter, int vocab, int per_block) {
  __shared__ Best scratch[32];
  pdl_prologue();
  const int r = blockIdx.y;
  const float* lg = logits + (size_t)r * vocab;
  const float t = temperature ? temperature[r] : 0.f;
  const int begin = blockIdx.x * per_block, end = min(vocab, begin + per_block);
  Best b;
  b.val = -INFINITY;
  b.idx = 0x7fffffff;
  if (!(t > 0.f)) {
    for (int v = begin + threadIdx.x; v < end; v += blockDim.x) {
      const float x = lg[v];
      if (x > b.val) { b.val = x; b.idx = v; }
    }
  } else {
    const uint32_t key = mix32((uint32_t)seed[r] ^ mix32((uint32_t)counter[r]));
    for (int v = begin + threadIdx.x; v < end; v += blockDim.x) {
      const float x = lg[v] / t + gumbel(key, (uint32_t)v);
      if (x > b.val) { b.val = x; b.idx = v; }
    }
  }
  b = block_best(b, scratch);
  if (threadIdx.x == 0) partial[(size_t)r * gridDim.x + blockIdx.x] = b;
}

__global__ void __launch_bounds__(256)
sample_final_kernel(int* __restrict__ tokens, const Best* __restrict__ partial, int num_partials) {
  __shared__ Best scratch[32];
  pdl_prologue();
  const int r = blockIdx.x;
  Best b;
  b.val = -INFINITY;
  b.idx = 0x7fffffff;
  for (int i = threadIdx.x; i < num_partials; i += blockDim.x) b = better(b, partial[(size_t)r * num_partials + i]);
  b = block_best(b, scratch);
  if (threadIdx.x == 0) tokens[r] = b.idx == 0x7fffffff ? 0 : b.idx;
}

// ------------------------------------------------------------------ rows with a nucleus: a cluster per row
// The two kernels above walk a row's whole vocabulary 33 times with one CTA, an exponential and a division
// per token each time (1.3 ms at 151,936 tokens, whatever the number of rows). Here a row belongs to a
// thread-block cluster: every CTA keeps its stretch of the row's probabilities in shared memory, computed
// once, and the search for the cut becomes rounds of a pass over shared memory and one sum across the
// cluster. The search takes three thresholds a round (two bits of the cut's bit pattern instead of one).
// The same CTAs then rank the ties at the cut in index order, mask and select. Same formulas, same
// kept set as nucleus_kernel + sample_kernel; sums are taken in a fixed order (lanes, warps, CTAs).
constexpr int NC_THREADS = 512, NC_WARPS = NC_THREADS / 32, NC_MAX_CTAS = 8;

struct NcShared {
  float red[NC_WARPS][4];
  float xchg[2][NC_MAX_CTAS][4];  // values of every CTA of the cluster, double buffered
  Best best[NC_MAX_CTAS];
  Best scratch[32];
  int ties[NC_MAX_CTAS];
  int tie_base[NC_WARPS + 1];
};

// v[i] summed (or the maximum taken) over all threads of all CTAs of the cluster, the same bits in every thread.
template <int N, bool MAX>
__device__ __forceinline__ void nc_all_reduce(float (&v)[N], NcShared& sh, int& buf,
                                              cooperative_groups::cluster_group& cluster, int rank, int ctas) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int i = 0; i < N; ++i) v[i] = MAX ? warp_max(v[i]) : warp_sum(v[i]);
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < N; ++i) sh.red[warp][i] = v[i];
  }
  __syncthreads();
  if (warp == 0) {
    // the warps' values meet in the first warp (lane w holds warp w's), whose lanes then each tell one CTA
    float a[N];
#pragma unroll
    for (int i = 0; i < N; ++i) {
      a[i] = lane < NC_WARPS ? sh.red[lane][i] : (MAX ? -INFINITY : 0.f);
      a[i] = MAX ? warp_max(a[i]) : warp_sum(a[i]);
    }
    if (lane < ctas) {
      float* dst = cluster.map_shared_rank(&sh.xchg[buf][rank][0], lane);
#pragma unroll
      for (int i = 0; i < N; ++i) dst[i] = a[i];
    }
  }
  cluster.sync();
#pragma unroll
  for (int i = 0; i < N; ++i) {
    float a = sh.xchg[buf][0][i];
    for (int c = 1; c < ctas; ++c) a = MAX ? fmaxf(a, sh.xchg[buf][c][i]) : a + sh.xchg[buf][c][i];
    v[i] = a;
  }
  buf ^= 1;
}

// Grid: rows x ctas CTAs in clusters of `ctas` along x; CTA `rank` of a cluster owns tokens
// [rank * slice, (rank + 1) * slice) of its row. Dynamic shared memory: slice floats.
__global__ void __launch_bounds__(NC_THREADS)
sample_cluster_kernel(int* __restrict__ tokens, const float* __restrict__ logits, const float* __restrict__ temperature,
                      const float* __restrict__ top_p, const long long* __restrict__ seed,
                      const long long* __restrict__ counter, int vocab, int slice) {
  extern __shared__ float nc_probs[];
  __shared__ NcShared sh;
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  const int ctas = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
  const int r = blockIdx.x / ctas;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_prologue();
  const float* lg = logits + (size_t)r * vocab;
  const float t = temperature[r], tp = top_p[r];
  const int begin = min(rank * slice, vocab), n = min(slice, vocab - begin);
  int buf = 0;
  Best b;
  b.val = -INFINITY;
  b.idx = 0x7fffffff;
  if (!(t > 0.f)) {
    for (int i = tid; i < n; i += NC_THREADS) {
      const float x = lg[begin + i];
      if (x > b.val) { b.val = x; b.idx = begin + i; }
    }
  } else if (tp >= 1.f) {
    const uint32_t key = mix32((uint32_t)seed[r] ^ mix32((uint32_t)counter[r]));
    for (int i = tid; i < n; i += NC_THREADS) {
      const float x = lg[begin + i] / t + gumbel(key, (uint32_t)(begin + i));
      if (x > b.val) { b.val = x; b.idx = begin + i; }
    }
  } else {
    const float inv_t = 1.0f / t;
    Nucleus nu;
    float one[1] = {-INFINITY};
    for (int i = tid; i < n; i += NC_THREADS) one[0] = fmaxf(one[0], lg[begin + i] * inv_t);
    nc_all_reduce<1, true>(one, sh, buf, cluster, rank, ctas);
    nu.zmax = one[0];
    one[0] = 0.f;
    for (int i = tid; i < n; i += NC_THREADS) {
      const float e = expf(lg[begin + i] * inv_t - nu.zmax);
      nc_probs[i] = e;
      one[0] += e;
    }
    nc_all_reduce<1, false>(one, sh, buf, cluster, rank, ctas);
    nu.sum = one[0];
    for (int i = tid; i < n; i += NC_THREADS) nc_probs[i] = nc_probs[i] / nu.sum;  // prob_of(), once per token
    // smallest x (as float bits) with f(x) = sum of probabilities greater than x  <  top_p
    uint32_t lo = 0u, hi = 0x3f800000u;  // f(1.0) = 0 < top_p always holds at hi
    while (lo < hi) {
      const uint32_t span = hi - lo;
      const uint32_t m1 = lo + (span >> 2), m2 = lo + (span >> 1), m3 = m2 + (span >> 2);
      const float x1 = __uint_as_float(m1), x2 = __uint_as_float(m2), x3 = __uint_as_float(m3);
      float f[3] = {0.f, 0.f, 0.f};
      for (int i = tid; i < n; i += NC_THREADS) {
        const float p = nc_probs[i];
        f[0] += p > x1 ? p : 0.f;
        f[1] += p > x2 ? p : 0.f;
        f[2] += p > x3 ? p : 0.f;
      }
      nc_all_reduce<3, false>(f, sh, buf, cluster, rank, ctas);
      if (f[0] < tp) {
        hi = m1;
      } else if (f[1] < tp) {
        lo = m1 + 1;
        hi = m2;
      } else if (f[2] < tp) {
        lo = m2 + 1;
        hi = m3;
      } else {
        lo = m3 + 1;
      }
    }
    nu.cut = __uint_as_float(lo);
    one[0] = 0.f;
    for (int i = tid; i < n; i += NC_THREADS) {
      const float p = nc_probs[i];
      one[0] += p > nu.cut ? p : 0.f;
    }
    nc_all_reduce<1, false>(one, sh, buf, cluster, rank, ctas);
    // the k-th tie (k = 0, 1, ...) is kept while f + k*cut < top_p
    nu.ties_kept = 0x7fffffff;
    if (nu.cut > 0.f) {
      const float room = (tp - one[0]) / nu.cut;
      nu.ties_kept = room >= 2147483000.f ? 0x7fffffff : max(1, (int)ceilf(room));
    }
    // Ties at the cut are ranked in index order: CTAs own consecutive stretches of the row, and inside a
    // CTA every warp owns a consecutive stretch of the CTA's.
    const int per_warp = ((n + NC_WARPS - 1) / NC_WARPS + 31) / 32 * 32;
    const int wb = min(warp * per_warp, n), we = min(wb + per_warp, n);
    int ties = 0;
    for (int i0 = wb; i0 < we; i0 += 32) {
      const int i = i0 + lane;
      ties += __popc(__ballot_sync(0xffffffffu, i < we && nc_probs[i] == nu.cut));
    }
    if (lane == 0) sh.tie_base[warp + 1] = ties;
    __syncthreads();
    if (tid == 0) {
      sh.tie_base[0] = 0;
      for (int w = 0; w < NC_WARPS; ++w) sh.tie_base[w + 1] += sh.tie_base[w];
      for (int c = 0; c < ctas; ++c) *cluster.map_shared_rank(&sh.ties[rank], c) = sh.tie_base[NC_WARPS];
    }
    cluster.sync();
    int rank0 = sh.tie_base[warp];
    for (int c = 0; c < rank; ++c) rank0 += sh.ties[c];
    const uint32_t key = mix32((uint32_t)seed[r] ^ mix32((uint32_t)counter[r]));
    for (int i0 = wb; i0 < we; i0 += 32) {
      const int i = i0 + lane;
      const float p = i < we ? nc_probs[i] : -1.f;
      const bool tie = i < we && p == nu.cut;
      const unsigned ballot = __ballot_sync(0xffffffffu, tie);
      const int tie_rank = rank0 + __popc(ballot & ((1u << lane) - 1u));
      rank0 += __popc(ballot);
      if (i < we && (p > nu.cut || (tie && tie_rank < nu.ties_kept))) {
        const int v = begin + i;
        const float x = lg[v] / t + gumbel(key, (uint32_t)v);
        if (x > b.val || (x == b.val && v < b.idx)) { b.val = x; b.idx = v; }
      }
    }
  }
  b = block_best(b, sh.scratch);
  if (tid == 0) *cluster.map_shared_rank(&sh.best[rank], 0) = b;
  cluster.sync();
  if (rank == 0 && tid == 0) {
    Best a = sh.best[0];
    for (int c = 1; c < ctas; ++c) a = better(a, sh.best[c]);
    tokens[r] = a.idx == 0x7fffffff ? 0 : a.idx;
  }
}

}  // namespace ms

using namespace ms;

// Bytes of scratch the two-stage path needs for `rows` rows of `vocab` logits (0: one stage).
static int partial_blocks(int vocab) { return vocab >= 16384 ? ceil_div(vocab, 4096) : 0; }
MS_EXPORT long long ms_sample_scratch_bytes(int rows, int vocab) {
  return (long long)rows * partial_blocks(vocab) * (long long)sizeof(Best);
}

MS_EXPORT int ms_nucleus_bytes() { return (int)sizeof(Nucleus); }

// partial_scratch: ms_sample_scratch_bytes(rows, vocab) bytes, or null to select in one stage.
MS_EXPORT int ms_sample(int* tokens, const float* logits, const float* temperature, const float* top_p,
                        const long long* seed, const long long* counter, void* nucleus_scratch, void* partial_scratch,
                        int rows, int vocab, cudaStream_t stream) {
  if (rows == 0) return 0;
  MS_CHECK_ARG(rows > 0 && vocab > 0, "sample: bad sizes rows=%d vocab=%d", rows, vocab);
  MS_CHECK_ARG(temperature == nullptr || (seed != nullptr && counter != nullptr), "sample: temperature rows need seeds and counters");
  const int threads = vocab >= 8192 ? 1024 : 256;
  if (top_p != nullptr) {
    MS_CHECK_ARG(nucleus_scratch != nullptr && temperature != nullptr, "sample: top_p needs scratch and temperatures");
    // a cluster per row, the row's probabilities in the cluster's shared memory, if they fit there
    const int ctas = vocab >= 16384 ? NC_MAX_CTAS : 1;
    const int slice = ceil_div(ceil_div(vocab, ctas), 32) * 32;
    const size_t smem = (size_t)slice * sizeof(float);
    if (smem <= 200 * 1024 && (long long)rows * ctas <= 0x7fffffffLL) {
      static size_t configured[64] = {};  // the attribute belongs to a device
      int dev = 0;
      MS_CHECK_CUDA(cudaGetDevice(&dev));
      MS_CHECK_ARG(dev >= 0 && dev < 64, "sample: device index %d is not supported", dev);
      if (configured[dev] < smem) {
        MS_CHECK_CUDA(cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured[dev] = smem;
      }
      MS_LAUNCH_CLUSTERED(sample_cluster_kernel, rows * ctas, NC_THREADS, smem, stream, ctas, tokens, logits, temperature, top_p,
                          seed, counter, vocab, slice);
      return 0;
    }
    MS_LAUNCH(nucleus_kernel, rows, threads, 0, stream, (Nucleus*)nucleus_scratch, logits, temperature, top_p, vocab);
  } else if (partial_scratch != nullptr && partial_blocks(vocab) > 0) {
    const int nblk = partial_blocks(vocab);
    MS_CHECK_ARG(rows <= 65535, "sample: too many rows (%d) for one launch", rows);
    MS_LAUNCH(sample_partial_kernel, dim3(nblk, rows), 256, 0, stream, (Best*)partial_scratch, logits, temperature, seed,
              counter, vocab, ceil_div(vocab, nblk));
    MS_LAUNCH(sample_final_kernel, rows, 256, 0, stream, tokens, (const Best*)partial_scratch, nblk);
    return 0;
  }
  MS_LAUNCH(sample_kernel, rows, threads, 0, stream, tokens, logits, temperature, seed, counter,
            top_p ? (const Nucleus*)nucleus_scratch : (const Nucleus*)nullptr, vocab);
  return 0;
}
