// Host-side access to cuTensorMapEncodeTiled without linking libcuda: the entry point is looked up through the
// runtime once per process.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <mutex>
#include <string.h>

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

// Host stand-in for the encoder, used by the program lint (rtp_lint_*), which builds rotation programs on a machine
// without a GPU: it records what the builder asked for in the 128 opaque bytes, where the lint reads it back.
struct HostTensorMap {
  unsigned long long magic;            // kHostMapMagic
  unsigned long long base;
  unsigned int rank, swizzle;
  unsigned long long dims[3];          // elements, innermost first
  unsigned long long strides[2];       // bytes, of dims[1] and dims[2]
  unsigned int box[3];
};
static_assert(sizeof(HostTensorMap) <= sizeof(CUtensorMap), "host record must fit the opaque tensor map");
constexpr unsigned long long kHostMapMagic = 0x52545048544d4150ull;
inline bool& host_tmap_mode() {
  static bool on = false;
  return on;
}
inline CUresult host_encode_tiled(CUtensorMap* m, CUtensorMapDataType, cuuint32_t rank, void* ptr, const cuuint64_t* dims,
                                  const cuuint64_t* strides, const cuuint32_t* box, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle sw, CUtensorMapL2promotion, CUtensorMapFloatOOBfill) {
  HostTensorMap h = {};
  h.magic = kHostMapMagic;
  h.base = reinterpret_cast<unsigned long long>(ptr);
  h.rank = rank;
  h.swizzle = (unsigned int)sw;
  for (cuuint32_t i = 0; i < rank && i < 3; ++i) { h.dims[i] = dims[i]; h.box[i] = box[i]; }
  for (cuuint32_t i = 0; i + 1 < rank && i < 2; ++i) h.strides[i] = strides[i];
  memset(m, 0, sizeof(*m));
  memcpy(m, &h, sizeof(h));
  return CUDA_SUCCESS;
}

inline EncodeTiledFn get_encode_tiled() {
  if (host_tmap_mode()) return &host_encode_tiled;
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
