// The CUDA driver API, resolved at run time from libcuda.so.1. The library links no driver
// symbol, so it loads (and serves host buffers) on machines without a GPU, and a host-only
// program never creates a CUDA context through it.
#pragma once
#include <cuda.h>

#include <string>

namespace hx {

struct CuDriver {
  bool ok = false;  // library found, every entry resolved, cuInit succeeded
  std::string why;  // reason when !ok

  CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
  CUresult (*CtxGetCurrent)(CUcontext*) = nullptr;
  CUresult (*CtxGetDevice)(CUdevice*) = nullptr;
  CUresult (*DeviceGetCount)(int*) = nullptr;
  CUresult (*DeviceGet)(CUdevice*, int) = nullptr;
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
  CUresult (*DevicePrimaryCtxGetState)(CUdevice, unsigned*, int*) = nullptr;
  CUresult (*PointerGetAttribute)(void*, CUpointer_attribute, CUdeviceptr) = nullptr;
  CUresult (*PointerGetAttributes)(unsigned, CUpointer_attribute*, void**, CUdeviceptr) = nullptr;
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*,
                                          CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*,
                        unsigned long long) = nullptr;
  CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr,
                                unsigned long long) = nullptr;
  CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle,
                     unsigned long long) = nullptr;
  CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle,
                                         CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*,
                                           CUmemAllocationHandleType) = nullptr;
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) = nullptr;
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle,
                               size_t, size_t, unsigned long long) = nullptr;
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*,
                                      CUmulticastGranularity_flags) = nullptr;

  std::string err(CUresult r) const;
};

// Loads the driver on first use; never creates a context.
const CuDriver& cu();

}  // namespace hx
