#include "kernels/inst.cuh"
namespace hx {
HX_INSTANTIATE_TYPE(hx::bf16)
template cudaError_t launch_twoshot_cast_t<hx::bf16>(const TwoShotArgs*, LaunchShape, cudaStream_t);
}
