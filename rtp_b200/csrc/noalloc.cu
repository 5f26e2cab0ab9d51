// See noalloc.h.  The scratch array, the lookup of its device address and the entry point live in this file.
#include <cuda_runtime.h>
#include <string>
#include "api.h"
#include "gemm_program.h"
#include "kernels.h"
#include "noalloc.h"

namespace {

// [0, RTP_FLAG_BYTES): flag/status block of the rotation kernel.  [RTP_FLAG_BYTES, ...): fp32 column sums of dy.
// In host code this name is only a handle for cudaGetSymbolAddress; it is not a device pointer.
static_assert(RTP_NOALLOC_SCRATCH_BYTES >= RTP_FLAG_BYTES + 4 * RTP_NOALLOC_MAX_OUT_FEATURES, "scratch too small");
static __device__ __align__(256) unsigned char g_noalloc_scratch[RTP_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {nullptr};
thread_local std::string g_msg;

int nfail(const std::string& s) {
  g_msg = s;
  return -1;
}

// Once per device, with that device current: resolve the device address of the array.
int scratch_for_current_device(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return nfail(std::string("cudaGetDevice: ") + cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return nfail("device index out of range");
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p) return nfail(std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e));
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return 0;
}

}  // namespace

extern "C" {

const char* rtp_noalloc_last_error(void) { return g_msg.c_str(); }

int rtp_noalloc_status(void* stream, unsigned long long* host_out) {
  if (!host_out) return nfail("rtp_noalloc_status: null output pointer");
  void* scratch = nullptr;
  if (scratch_for_current_device(&scratch)) return -1;
  const RtpFlagBlock* fb = reinterpret_cast<const RtpFlagBlock*>(scratch);
  cudaError_t e = cudaMemcpyAsync(host_out, &fb->status.v, sizeof(unsigned long long), cudaMemcpyDeviceToHost,
                                  (cudaStream_t)stream);
  if (e != cudaSuccess) return nfail(std::string("status copy: ") + cudaGetErrorString(e));
  e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return nfail(std::string("status sync: ") + cudaGetErrorString(e));
  return 0;
}

int rtp_linear_bwd_noalloc(const void* x, long long ldx, const void* dy, long long ldy, const void* w,
                           long long bias_off, int M, int in_features, int out_features, void* dx, long long lddx,
                           void* grad_flat, void* stream) {
  if (out_features > RTP_NOALLOC_MAX_OUT_FEATURES)
    return nfail("rtp_linear_bwd_noalloc: out_features " + std::to_string(out_features) + " exceeds the built-in scratch (max " +
                 std::to_string(RTP_NOALLOC_MAX_OUT_FEATURES) + ")");
  if (M <= 0 || in_features <= 0 || out_features <= 0) return nfail("rtp_linear_bwd_noalloc: empty problem");
  void* scratch = nullptr;
  if (scratch_for_current_device(&scratch)) return -1;
  cudaStream_t s = (cudaStream_t)stream;
  // the flag/status block must start at zero; the column sums are zeroed by rtp_colsum itself
  cudaError_t e = cudaMemsetAsync(scratch, 0, RTP_FLAG_BYTES, s);
  if (e != cudaSuccess) return nfail(std::string("cudaMemsetAsync: ") + cudaGetErrorString(e));
  float* dbias = reinterpret_cast<float*>(static_cast<unsigned char*>(scratch) + RTP_FLAG_BYTES);
  if (bias_off >= 0) {
    if (rtp_colsum(dy, ldy, M, out_features, dbias, stream)) return nfail(rtp_kernels_last_error());
  }
  RtpRing ring = {};
  ring.rank = 0;
  ring.world = 1;
  ring.ws[0] = scratch;
  ring.slot_bytes = 0;
  ring.ctas = rtp_sm_count();
  ring.timeout_ns = 2000000000ull;
  RtpLinearBwd op = {};
  op.mode = 0;
  op.M = M;
  op.in_features = in_features;
  op.out_features = out_features;
  op.home = w;
  op.bias_off = bias_off;
  op.shard_bytes = 0;
  op.x = x; op.ldx = ldx;
  op.dy = dy; op.ldy = ldy;
  op.dx = dx; op.lddx = lddx;
  op.grad_home = grad_flat;
  op.dbias_full = bias_off >= 0 ? dbias : nullptr;
  if (rtp_linear_bwd(&ring, &op, stream)) return nfail(rtp_last_error());
  return 0;
}

}  // extern "C"
