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
