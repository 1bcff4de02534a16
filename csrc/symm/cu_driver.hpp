// Lazily resolved table of CUDA driver entry points (virtual memory
// management and NVLink multicast).
//
// The extension must import on a machine without a GPU driver (CPU tests, the
// build check), so it never links libcuda: the functions are looked up with
// dlopen/dlsym on first use, and a missing library or symbol only disables the
// feature that needs it.  Parity: the reference resolves its optional RDMA
// library the same way, probing once and disabling the transport when
// anything is missing (csrc/transport/rdma/IbvWrapper.cpp:31-81).
#pragma once

#include <cuda.h>

#include <string>

namespace mccl {

struct CuDriver {
  bool loaded = false;      // libcuda found and the VMM entry points resolved
  bool multicast = false;   // cuMulticast* entry points resolved
  std::string why;          // reason when !loaded

  CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
  CUresult (*DeviceGet)(CUdevice*, int) = nullptr;
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) = nullptr;
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long) = nullptr;
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags) = nullptr;

  CUresult (*CtxGetCurrent)(CUcontext*) = nullptr;
  CUresult (*CtxSetCurrent)(CUcontext) = nullptr;
  CUresult (*DevicePrimaryCtxRetain)(CUcontext*, CUdevice) = nullptr;
  // Driver calls need a context bound to the calling thread; threads that have
  // only used cached allocations so far (autograd workers) may have none yet.
  // Binds the primary context of `device` when the thread has no context.
  void ensure_context(int device) const;

  // TMA descriptors (optional; absent only on very old drivers)
  CUresult (*TensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill) = nullptr;

  std::string error_string(CUresult r) const;

  // Process-wide table; resolution happens once.
  static const CuDriver& get();
};

}  // namespace mccl

// Throws CudaError with the driver's message when a CUresult is not success.
#define MCCL_CU_CHECK(expr)                                                                    \
  do {                                                                                         \
    CUresult _mccl_cu = (expr);                                                                \
    MCCL_CHECK_T(_mccl_cu == CUDA_SUCCESS, CudaError,                                          \
                 #expr << " failed: " << ::mccl::CuDriver::get().error_string(_mccl_cu));      \
  } while (0)

#define MCCL_CUDA_CHECK(expr)                                                                  \
  do {                                                                                         \
    cudaError_t _mccl_rt = (expr);                                                             \
    MCCL_CHECK_T(_mccl_rt == cudaSuccess, CudaError, #expr << " failed: " << cudaGetErrorString(_mccl_rt)); \
  } while (0)
