// Small runtime services of the kernel library: the error string, a device status word that
// kernels raise instead of faulting, and device queries.
#include "common.cuh"

MS_DEFINE_LAST_ERROR(ms_kernels_last_error)
MS_DEFINE_PDL_SWITCH(ms_kernels_set_pdl)

MS_EXPORT int ms_device_sm_count(int device, int* out) {
  MS_CHECK_CUDA(cudaDeviceGetAttribute(out, cudaDevAttrMultiProcessorCount, device));
  return 0;
}

MS_EXPORT int ms_device_arch(int device, int* major, int* minor) {
  MS_CHECK_CUDA(cudaDeviceGetAttribute(major, cudaDevAttrComputeCapabilityMajor, device));
  MS_CHECK_CUDA(cudaDeviceGetAttribute(minor, cudaDevAttrComputeCapabilityMinor, device));
  return 0;
}

// What a bounded wait does when nothing ever arrives, shown on purpose: one thread waits on an mbarrier
// that nobody arrives on, for at most limit_ns, then raises the status word to `code` and returns. The
// kernel ends by itself and the context stays usable; the host reads the word. (The pipelines of
// gemm_tc.cu and attention_tc.cu give up the same way, after MS_WAIT_NS.)
namespace ms {
__global__ void wait_selftest_kernel(int* __restrict__ status, unsigned long long limit_ns, int code) {
  __shared__ uint64_t bar;
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(&bar);
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(addr), "r"(1u));
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  if (!mbar_wait_bounded(addr, 0, limit_ns)) atomicExch(status, code);
}
}  // namespace ms

MS_EXPORT int ms_wait_selftest(int* status, long long limit_ns, int code, cudaStream_t stream) {
  MS_CHECK_ARG(status != nullptr && limit_ns > 0 && limit_ns <= 1000000000LL, "wait_selftest: a limit of up to a second, and a status word");
  ms::wait_selftest_kernel<<<1, 1, 0, stream>>>(status, (unsigned long long)limit_ns, code);
  MS_CHECK_CUDA(cudaGetLastError());
  return 0;
}
