// Kernel launch with the programmatic-dependent-launch attribute (see pdl_prologue in common.cuh).
#pragma once
#include <cuda_runtime.h>
#include <stdlib.h>

namespace rtp {

// RTP_PDL=1 lets a kernel start while its predecessor drains (off by default: on the training step the kernels fill
// the SMs' registers and shared memory, so a successor rarely finds room before its predecessor has left)
inline bool pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("RTP_PDL");
    on = (e && e[0] == '1') ? 1 : 0;
  }
  return on == 1;
}

// Raises the dynamic shared-memory limit of kernel `Kern` on the current device, once per (kernel, device): the
// attribute belongs to the kernel on one device, so a process that drives several GPUs sets it on each.
template <auto Kern>
cudaError_t ensure_smem(int bytes) {
  constexpr int kMaxDev = 64;
  static bool done[kMaxDev] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= kMaxDev) dev = 0;
  if (done[dev]) return cudaSuccess;
  cudaError_t e = cudaFuncSetAttribute(Kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) done[dev] = true;
  return e;
}

template <typename... KArgs, typename... Args>
cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Same, with thread-block clusters of `cluster` CTAs.
template <typename... KArgs, typename... Args>
cudaError_t launch_kc(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, dim3 cluster,
                      Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  at[1].id = cudaLaunchAttributeClusterDimension;
  at[1].val.clusterDim.x = cluster.x;
  at[1].val.clusterDim.y = cluster.y;
  at[1].val.clusterDim.z = cluster.z;
  cfg.attrs = at;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace rtp
