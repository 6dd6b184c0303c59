#include "kernels/inst.cuh"
namespace hx {
HX_INSTANTIATE_TYPE(uint8_t)
}
