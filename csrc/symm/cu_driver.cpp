#include "cu_driver.hpp"

#include <dlfcn.h>

#include "../core/log.hpp"

namespace mccl {

namespace {

template <typename Fn>
bool resolve(void* lib, const char* name, Fn& out) {
  out = reinterpret_cast<Fn>(dlsym(lib, name));
  return out != nullptr;
}

CuDriver build_table() {
  CuDriver d;
  void* lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) lib = dlopen("libcuda.so", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) {
    d.why = "libcuda.so.1 not found (no NVIDIA driver on this machine)";
    return d;
  }
  bool ok = true;
  ok &= resolve(lib, "cuGetErrorString", d.GetErrorString);
  ok &= resolve(lib, "cuDeviceGet", d.DeviceGet);
  ok &= resolve(lib, "cuDeviceGetAttribute", d.DeviceGetAttribute);
  ok &= resolve(lib, "cuMemGetAllocationGranularity", d.MemGetAllocationGranularity);
  ok &= resolve(lib, "cuMemCreate", d.MemCreate);
  ok &= resolve(lib, "cuMemRelease", d.MemRelease);
  ok &= resolve(lib, "cuMemExportToShareableHandle", d.MemExportToShareableHandle);
  ok &= resolve(lib, "cuMemImportFromShareableHandle", d.MemImportFromShareableHandle);
  ok &= resolve(lib, "cuMemAddressReserve", d.MemAddressReserve);
  ok &= resolve(lib, "cuMemAddressFree", d.MemAddressFree);
  ok &= resolve(lib, "cuMemMap", d.MemMap);
  ok &= resolve(lib, "cuMemUnmap", d.MemUnmap);
  ok &= resolve(lib, "cuMemSetAccess", d.MemSetAccess);
  if (!ok) {
    d.why = "libcuda is missing a virtual-memory-management entry point";
    return d;
  }
  d.loaded = true;
  resolve(lib, "cuTensorMapEncodeTiled", d.TensorMapEncodeTiled);
  resolve(lib, "cuCtxGetCurrent", d.CtxGetCurrent);
  resolve(lib, "cuCtxSetCurrent", d.CtxSetCurrent);
  resolve(lib, "cuDevicePrimaryCtxRetain", d.DevicePrimaryCtxRetain);
  bool mc = true;
  mc &= resolve(lib, "cuMulticastCreate", d.MulticastCreate);
  mc &= resolve(lib, "cuMulticastAddDevice", d.MulticastAddDevice);
  mc &= resolve(lib, "cuMulticastBindMem", d.MulticastBindMem);
  mc &= resolve(lib, "cuMulticastUnbind", d.MulticastUnbind);
  mc &= resolve(lib, "cuMulticastGetGranularity", d.MulticastGetGranularity);
  d.multicast = mc;
  MCCL_DEBUG("cuda driver table resolved (multicast entry points: " << (mc ? "yes" : "no") << ")");
  return d;
}

}  // namespace

const CuDriver& CuDriver::get() {
  static const CuDriver table = build_table();
  return table;
}

void CuDriver::ensure_context(int device) const {
  if (!CtxGetCurrent || !CtxSetCurrent || !DevicePrimaryCtxRetain || !DeviceGet) return;
  CUcontext ctx = nullptr;
  if (CtxGetCurrent(&ctx) == CUDA_SUCCESS && ctx != nullptr) return;
  CUdevice dev;
  if (DeviceGet(&dev, device) != CUDA_SUCCESS) return;
  // The primary context is never released by this process, so the extra
  // reference taken here costs nothing.
  if (DevicePrimaryCtxRetain(&ctx, dev) == CUDA_SUCCESS) CtxSetCurrent(ctx);
}

std::string CuDriver::error_string(CUresult r) const {
  const char* s = nullptr;
  if (GetErrorString && GetErrorString(r, &s) == CUDA_SUCCESS && s) return std::string(s) + " (CUresult " + std::to_string(r) + ")";
  return "CUresult " + std::to_string(static_cast<int>(r));
}

}  // namespace mccl
