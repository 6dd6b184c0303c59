// Host-callable launchers of the sm_100a kernels. `world` > 1 launches the single-GPU
// "whole world in one grid" form: args then points to `world` argument blocks in device
// memory and blockIdx.y selects the rank (cooperative launch, so all ranks' CTAs are
// co-resident and can wait on one another). world == 0 launches the production form with
// the one argument block passed by value.
#pragma once
#include <cuda_runtime.h>

#include "device/proto.h"

namespace hx {

struct LaunchShape {
  int ctas;
  int threads;
  int world;  // 0 = production (one rank per GPU)
};

cudaError_t launch_xchg_copy(const XchgArgs* args, LaunchShape s, cudaStream_t st);
cudaError_t launch_xchg_fold(int dt, const XchgArgs* args, LaunchShape s, cudaStream_t st);
cudaError_t launch_twoshot(int dt, const TwoShotArgs* args, LaunchShape s, cudaStream_t st);
// fp32 buffers with wire_dt (hxcclFloat16 / hxcclBfloat16) on the wire; args as for two-shot, bytes of wire_dt
cudaError_t launch_twoshot_cast(int wire_dt, const TwoShotArgs* args, LaunchShape s, cudaStream_t st);
// three-role pipeline for large messages (grid = 3 * lanes)
cudaError_t launch_twoshot_roles(int dt, const TwoShotArgs* args, LaunchShape s, cudaStream_t st);
// neighbour ring (reduce-scatter + all-gather around the ring); args->steps = rounds
cudaError_t launch_ring(int dt, const TwoShotArgs* args, LaunchShape s, cudaStream_t st);
// small messages: flag inside the data, no hand-shake (threads must be 256)
cudaError_t launch_ll(int dt, const LLArgs* args, LaunchShape s, cudaStream_t st);
// production only; roles = three-role pipeline
cudaError_t launch_nvls(const NvlsArgs* args, LaunchShape s, cudaStream_t st, bool roles = false);
cudaError_t launch_p2p(const P2pArgs* args, LaunchShape s, cudaStream_t st);

// dst[0, bytes) = src[0, bytes) at memory speed (the single-rank collectives)
cudaError_t launch_copy(void* dst, const void* src, size_t bytes, cudaStream_t st);

// standalone elementwise kernels (dst op= src, dst = src*scalar, buf /= divisor)
cudaError_t launch_reduce(void* dst, const void* src, size_t count, int dt, int op, cudaStream_t st);
cudaError_t launch_scale(void* dst, const void* src, size_t count, int dt, const void* scalar_host,
                         cudaStream_t st);
cudaError_t launch_divide(void* buf, size_t count, int dt, int divisor, cudaStream_t st);

// largest grid of `threads`-wide CTAs of the widest collective kernel that is co-resident
int max_resident_ctas(int threads);

}  // namespace hx
