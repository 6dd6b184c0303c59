#include "kernels/inst.cuh"
namespace hx {
HX_INSTANTIATE_TYPE(int8_t)
}
