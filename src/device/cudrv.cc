#include "device/cudrv.h"

#include <dlfcn.h>

#include <cstdio>
#include <cstdlib>
#include <mutex>

namespace hx {
namespace {

using GetProc = CUresult (*)(const char*, void**, int, cuuint64_t, CUdriverProcAddressQueryResult*);

// The multicast entry points arrived with CUDA 12.1; ask for the 12.4 view of the API.
constexpr int kApiVersion = 12040;

template <typename F>
bool bind(GetProc gp, const char* name, F* slot, std::string* why) {
  void* fn = nullptr;
  CUdriverProcAddressQueryResult q;
  if (gp(name, &fn, kApiVersion, CU_GET_PROC_ADDRESS_DEFAULT, &q) != CUDA_SUCCESS || !fn) {
    *why = std::string("the CUDA driver has no ") + name;
    return false;
  }
  *slot = reinterpret_cast<F>(fn);
  return true;
}

CuDriver load() {
  CuDriver d;
  void* lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) {
    d.why = "libcuda.so.1 is not available";
    return d;
  }
  auto init = reinterpret_cast<CUresult (*)(unsigned)>(dlsym(lib, "cuInit"));
  auto gp = reinterpret_cast<GetProc>(dlsym(lib, "cuGetProcAddress_v2"));
  if (!init || !gp) {
    d.why = "libcuda.so.1 lacks cuInit / cuGetProcAddress_v2";
    return d;
  }
  if (init(0) != CUDA_SUCCESS) {
    d.why = "cuInit failed (no usable GPU)";
    return d;
  }
  bool ok = true;
#define HX_BIND(NAME) ok = ok && bind(gp, "cu" #NAME, &d.NAME, &d.why)
  HX_BIND(GetErrorString);
  HX_BIND(CtxGetCurrent);
  HX_BIND(CtxGetDevice);
  HX_BIND(DeviceGetCount);
  HX_BIND(DeviceGet);
  HX_BIND(DeviceGetAttribute);
  HX_BIND(DevicePrimaryCtxGetState);
  HX_BIND(PointerGetAttribute);
  HX_BIND(PointerGetAttributes);
  HX_BIND(MemGetAllocationGranularity);
  HX_BIND(MemCreate);
  HX_BIND(MemRelease);
  HX_BIND(MemAddressReserve);
  HX_BIND(MemAddressFree);
  HX_BIND(MemMap);
  HX_BIND(MemUnmap);
  HX_BIND(MemSetAccess);
  HX_BIND(MemExportToShareableHandle);
  HX_BIND(MemImportFromShareableHandle);
  HX_BIND(MulticastCreate);
  HX_BIND(MulticastAddDevice);
  HX_BIND(MulticastBindMem);
  HX_BIND(MulticastUnbind);
  HX_BIND(MulticastGetGranularity);
#undef HX_BIND
  d.ok = ok;
  return d;
}

}  // namespace

std::string CuDriver::err(CUresult r) const {
  const char* s = nullptr;
  if (GetErrorString && GetErrorString(r, &s) == CUDA_SUCCESS && s) return s;
  return "CUDA driver error " + std::to_string(int(r));
}

const CuDriver& cu() {
  static const CuDriver d = [] {
    CuDriver x = load();
    if (!x.ok && std::getenv("HXCCL_DEBUG"))
      std::fprintf(stderr, "hxccl: CUDA driver unavailable (%s); every buffer is treated as host memory\n",
                   x.why.c_str());
    return x;
  }();
  return d;
}

}  // namespace hx
