// Host-side access to cuTensorMapEncodeTiled without linking libcuda: the entry point is looked up through the
// runtime once per process.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <mutex>

namespace rtp {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled is a driver call and needs a current context.  A thread that has only used the runtime API so
// far (for instance an autograd worker thread whose first CUDA work is a tensor-map encode) may not have one bound
// yet; a context-requiring runtime call binds the primary context.  Done once per thread.
inline void ensure_context_on_this_thread() {
  static thread_local bool done = false;
  if (!done) {
    cudaFree(nullptr);
    done = true;
  }
}

inline EncodeTiledFn get_encode_tiled() {
  ensure_context_on_this_thread();
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

}  // namespace rtp
