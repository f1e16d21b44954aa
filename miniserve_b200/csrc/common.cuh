// Shared helpers for every kernel file: element types, error reporting, small device utilities.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>
#include <cstring>

namespace ms {

// Last error message of this thread; every shared library exports it under its own name
// (MS_DEFINE_LAST_ERROR) so Python can turn a non-zero return code into an exception.
inline char* error_buffer() {
  static thread_local char buf[1024];
  return buf;
}

inline int fail(const char* fmt, ...) __attribute__((format(printf, 1, 2)));

#define MS_CHECK_ARG(cond, ...)                         \
  do {                                                  \
    if (!(cond)) return ::ms::fail(__VA_ARGS__);        \
  } while (0)

#define MS_CHECK_CUDA(expr)                                                                  \
  do {                                                                                       \
    cudaError_t err__ = (expr);                                                              \
    if (err__ != cudaSuccess)                                                                \
      return ::ms::fail("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(err__), __FILE__, \
                        __LINE__);                                                           \
  } while (0)

#define MS_CHECK_LAUNCH() MS_CHECK_CUDA(cudaGetLastError())

template <typename T>
struct Elem;
template <>
struct Elem<float> {
  static __device__ __forceinline__ float load(const float* p) { return *p; }
  static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
};
template <>
struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a whole block in a fixed order (lane tree, then warps in index order), so the
// result depends only on the values and the block size.
template <int MAX_WARPS = 32>
__device__ __forceinline__ float block_sum(float v, float* scratch /* MAX_WARPS floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < nwarps; ++w) total += scratch[w];
  return total;
}

// eight bfloat16 in a 16-byte word, to and from float32
__device__ __forceinline__ void bf16x8_to_float(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x = __bfloat1622float2(h[i]);
    f[2 * i] = x.x;
    f[2 * i + 1] = x.y;
  }
}
__device__ __forceinline__ uint4 float_to_bf16x8(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// ---- programmatic dependent launch
// Every kernel of this package starts with pdl_prologue(): it lets the next kernel in the stream
// begin launching (its CTAs become resident and may fetch what does not depend on earlier
// kernels, i.e. weights), then waits until everything launched before it has completed and is
// visible. Because every kernel waits before it touches activations or the cache, completion
// order stays the launch order and no kernel reads or overwrites data too early. Launched
// without the attribute (or when the switch below is off) both instructions do nothing.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_prologue() {
  pdl_launch_dependents();
  pdl_wait();
}

// ---- bounded wait on an mbarrier
// Waits for the phase of the given parity of the mbarrier at shared-memory address `bar`, for at
// most MS_WAIT_NS of the global timer (looked at every 64 failed polls; a poll itself may block
// for a while inside the hardware). A wait that ends this way returns false: the caller raises the
// device status word and winds its pipeline down, so a protocol error or a lost arrival costs a
// couple of seconds and an error on the host, not a GPU that no longer answers.
constexpr unsigned long long MS_WAIT_NS = 2000000000ull;
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, unsigned long long limit_ns = MS_WAIT_NS) {
  unsigned long long began = 0;
  for (uint32_t polls = 1;; ++polls) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    if ((polls & 63u) == 0) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(now));
      if (began == 0) began = now;
      else if (now - began > limit_ns) return false;
    }
  }
}

inline int& pdl_switch() {
  static int on = 1;
  return on;
}

// cluster_x > 1: thread-block clusters of that many CTAs along x (the grid's x must be a multiple).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_clustered(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    unsigned cluster_x, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (pdl_switch()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          Args&&... args) {
  return launch_clustered(kernel, grid, block, smem, stream, 1u, static_cast<Args&&>(args)...);
}

}  // namespace ms

#include <cstdarg>
inline int ms::fail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(ms::error_buffer(), 1024, fmt, ap);
  va_end(ap);
  return 1;
}

// Checks that only a debug build carries (MINISERVE_DEBUG=1 compiles the libraries with
// -DMS_DEBUG_CHECKS under names of their own): indices that the host is trusted to have got right
// are checked against their bounds, and a kernel that finds one out of range raises the status word
// (code 5) and skips the access instead of making it.
#ifdef MS_DEBUG_CHECKS
#define MS_DEBUG_ONLY(...) __VA_ARGS__
#else
#define MS_DEBUG_ONLY(...)
#endif

// dtype codes shared with Python
enum MsDtype : int { MS_F32 = 0, MS_BF16 = 1 };

#define MS_EXPORT extern "C" __attribute__((visibility("default")))
#define MS_DEFINE_LAST_ERROR(name) \
  MS_EXPORT const char* name() { return ::ms::error_buffer(); }
// The per-library switch for programmatic dependent launch (1: on, the default).
#define MS_DEFINE_PDL_SWITCH(name) \
  MS_EXPORT void name(int on) { ::ms::pdl_switch() = on; }
#define MS_LAUNCH(kernel, grid, block, smem, stream, ...) \
  MS_CHECK_CUDA(::ms::launch(kernel, dim3(grid), dim3(block), (size_t)(smem), stream, __VA_ARGS__))
#define MS_LAUNCH_CLUSTERED(kernel, grid, block, smem, stream, cluster_x, ...) \
  MS_CHECK_CUDA(::ms::launch_clustered(kernel, dim3(grid), dim3(block), (size_t)(smem), stream, (unsigned)(cluster_x), __VA_ARGS__))
