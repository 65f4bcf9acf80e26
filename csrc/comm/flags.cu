// Bounded device-side waits on flags written by a peer GPU or by the host.
//
// Every fused compute+collective kernel in this library waits on peer flags
// through wait_flag_ge(): a wait that exceeds its time budget latches
// PB_TIMEOUT_FLAG into a status word and returns, so a missing peer can never
// hang the GPU. pb_wait_flag_probe exposes that primitive on its own: the host
// (or a test) points it at a flag nobody sets and reads the status back, which
// is how failure detection is exercised without faulting or hanging a device.
#include "common.cuh"

namespace pb {

__global__ void wait_flag_probe_kernel(const uint32_t* flag, uint32_t want, uint64_t budget_ns,
                                       int* status) {
  if (threadIdx.x == 0 && blockIdx.x == 0) wait_flag_ge(flag, want, budget_ns, status);
}

__global__ void set_flag_kernel(uint32_t* flag, uint32_t value) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    __threadfence_system();
    st_release_sys(flag, value);
  }
}

}  // namespace pb

using namespace pb;

// Waits until *flag >= want or budget_ns elapsed (status <- 2 on time-out).
PB_API int pb_wait_flag_probe(const void* flag, int want, long budget_ns, void* status,
                              cudaStream_t st) {
  if (budget_ns <= 0 || budget_ns > 5000000000L) return PB_BAD_ARG;  // at most 5 s
  wait_flag_probe_kernel<<<1, 32, 0, st>>>(static_cast<const uint32_t*>(flag),
                                           static_cast<uint32_t>(want),
                                           static_cast<uint64_t>(budget_ns),
                                           static_cast<int*>(status));
  return cudaGetLastError();
}

PB_API int pb_set_flag(void* flag, int value, cudaStream_t st) {
  set_flag_kernel<<<1, 32, 0, st>>>(static_cast<uint32_t*>(flag), static_cast<uint32_t>(value));
  return cudaGetLastError();
}
