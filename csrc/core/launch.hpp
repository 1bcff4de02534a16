// One door for every kernel launch.
//
//   MCCL_LAUNCH(kernel, grid, block, smem, stream, args...)
//
// launches `kernel`, reads the launch status (cudaGetLastError, so a bad configuration is reported at
// the site that caused it and a stale error of an unrelated call is not carried along), counts the
// launch under the kernel's name, and at log level TRACE prints site, grid, block, shared memory and
// stream.  The expression's value is the cudaError_t of the launch.  A kernel name that contains commas
// (template arguments) goes in parentheses: MCCL_LAUNCH((gemm<BN, ST>), ...).
//
// The reference wraps every Metal command-buffer commit the same way (MCCL_COMMIT(site, ...):
// csrc/metal/CommitTrace.hpp:15-26) so that a stalled or failed commit names its call site.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <map>
#include <string>

namespace mccl {

// Status of the launch just made (clears the error state) plus bookkeeping; see MCCL_LAUNCH.
cudaError_t launch_record(const char* kernel, const char* file, int line, dim3 grid, dim3 block, size_t smem, cudaStream_t stream);
// First failure among the launches this thread made through MCCL_LAUNCH since the last call (cudaSuccess when
// none); clears it.  Launchers that enqueue several kernels end with `return launch_status();`.
cudaError_t launch_status();
// Launches per kernel name since the process started (or since launch_counts_reset()).
std::map<std::string, uint64_t> launch_counts();
void launch_counts_reset();
uint64_t launch_total();

// Programmatic dependent launch (sm_90+).  A kernel launched with MCCL_LAUNCH_PDL may begin while the kernel before
// it in the stream is still draining: its CTAs become resident, do their set-up (barrier init, tensor-memory
// allocation, descriptor prefetch, index arithmetic) and then block in pdl_wait() until every earlier kernel of the
// stream has finished and its memory is visible.  Such a kernel must call pdl_wait() before its first access to
// global memory, read or write.  pdl_trigger() tells the hardware that the kernels after this one may start their
// set-up; kernels that never call it release their dependents when they exit.  The launch attribute is only set with
// MCCL_PDL=1 (without it the device calls are no-ops and the stream serialises as usual): measured on the training
// step it did not pay, so it is an option, not the default.
bool pdl_enabled();
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#if defined(__CUDACC__)
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

}  // namespace mccl

#define MCCL_LAUNCH_PDL(kernel, grid, block, smem, stream, ...)                                                 \
  (::mccl::launch_pdl((kernel), dim3(grid), dim3(block), static_cast<size_t>(smem), (stream), __VA_ARGS__),     \
   ::mccl::launch_record(#kernel, __FILE__, __LINE__, dim3(grid), dim3(block), static_cast<size_t>(smem), (stream)))

#define MCCL_LAUNCH(kernel, grid, block, smem, stream, ...)                                                     \
  ((kernel)<<<(grid), (block), (smem), (stream)>>>(__VA_ARGS__),                                               \
   ::mccl::launch_record(#kernel, __FILE__, __LINE__, dim3(grid), dim3(block), static_cast<size_t>(smem), (stream)))
