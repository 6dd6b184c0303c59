// Where a pointer lives and whether this process has a CUDA context, both asked of the driver
// API, which (unlike the runtime API) never creates a context as a side effect. A program that
// only passes host buffers therefore stays context-free, as the reference guarantees
// (src/memspace_cuda.cc:13-53, tests/gpu_host_no_context.cc).
#include "core/devpath.h"
#include "device/cudrv.h"

namespace hx {

// One driver call per pointer on the path of every collective: memory type, managed flag and
// device ordinal together. Unknown pointers (plain host memory) make the call fail or leave the
// type zero.
MemKind classify_on(const void* p, int* ordinal) {
  *ordinal = -1;
  if (!p) return MemKind::Null;
  const CuDriver& d = cu();
  if (!d.ok) return MemKind::Host;
  unsigned type = 0, managed = 0;
  int where = -1;
  CUpointer_attribute what[3] = {CU_POINTER_ATTRIBUTE_MEMORY_TYPE, CU_POINTER_ATTRIBUTE_IS_MANAGED,
                                 CU_POINTER_ATTRIBUTE_DEVICE_ORDINAL};
  void* into[3] = {&type, &managed, &where};
  if (d.PointerGetAttributes(3, what, into, reinterpret_cast<CUdeviceptr>(p)) != CUDA_SUCCESS) return MemKind::Host;
  if (type == CU_MEMORYTYPE_DEVICE || type == CU_MEMORYTYPE_UNIFIED || managed) {
    *ordinal = where;
    return MemKind::Device;
  }
  return MemKind::Host;  // ordinary, pinned or registered host memory
}

MemKind classify(const void* p) {
  if (!p) return MemKind::Null;
  const CuDriver& d = cu();
  if (!d.ok) return MemKind::Host;
  unsigned type = 0;
  if (d.PointerGetAttribute(&type, CU_POINTER_ATTRIBUTE_MEMORY_TYPE,
                            reinterpret_cast<CUdeviceptr>(p)) != CUDA_SUCCESS)
    return MemKind::Host;  // unknown to CUDA: ordinary host memory
  if (type == CU_MEMORYTYPE_DEVICE) return MemKind::Device;
  if (type == CU_MEMORYTYPE_UNIFIED) return MemKind::Device;  // managed memory
  unsigned managed = 0;
  if (d.PointerGetAttribute(&managed, CU_POINTER_ATTRIBUTE_IS_MANAGED,
                            reinterpret_cast<CUdeviceptr>(p)) == CUDA_SUCCESS && managed)
    return MemKind::Device;
  return MemKind::Host;  // pinned / registered host memory
}

int device_ordinal_of(const void* p) {
  const CuDriver& d = cu();
  if (!p || !d.ok) return -1;
  int ordinal = -1;
  if (d.PointerGetAttribute(&ordinal, CU_POINTER_ATTRIBUTE_DEVICE_ORDINAL, reinterpret_cast<CUdeviceptr>(p)) !=
      CUDA_SUCCESS)
    return -1;
  return ordinal;
}

bool cuda_context_exists() {
  const CuDriver& d = cu();
  if (!d.ok) return false;
  CUcontext cur = nullptr;
  if (d.CtxGetCurrent(&cur) == CUDA_SUCCESS && cur) return true;
  int n = 0;
  if (d.DeviceGetCount(&n) != CUDA_SUCCESS) return false;
  for (int i = 0; i < n; ++i) {
    CUdevice dev;
    unsigned flags = 0;
    int active = 0;
    if (d.DeviceGet(&dev, i) == CUDA_SUCCESS &&
        d.DevicePrimaryCtxGetState(dev, &flags, &active) == CUDA_SUCCESS && active)
      return true;
  }
  return false;
}

}  // namespace hx
