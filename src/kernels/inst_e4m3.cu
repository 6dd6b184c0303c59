#include "kernels/inst.cuh"
namespace hx {
HX_INSTANTIATE_TYPE(hx::e4m3)
}
