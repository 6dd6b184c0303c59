#include "kernels/inst.cuh"
namespace hx {
HX_INSTANTIATE_TYPE(uint32_t)
}
