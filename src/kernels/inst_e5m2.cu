#include "kernels/inst.cuh"
namespace hx {
HX_INSTANTIATE_TYPE(hx::e5m2)
}
