// In-place ring shift: every rank's buffer is replaced by its neighbour's, through a small staging ring in peer-mapped
// memory instead of a second full-size buffer.  This is the transport of the memory-lean ("in-place") rotation mode
// and the library's rotate-only kernel (reference: the blocking exchange of rtp/inplace/module/collectives.py:173-225
// and rtp/rotated_tensor_parallel.py:241-271, which receive into a full-size temporary).
//
// Each CTA owns a contiguous range of the buffer and a private lane of the staging area (kDepth chunks) on the
// destination rank.  Per chunk: wait until the destination has consumed what the lane's slot held before, push the own
// chunk with NVLink P2P stores, signal "arrived"; then wait for the chunk coming from the source rank, copy it over the
// (already pushed) own chunk and return the credit.  Counters only ever grow, across calls too, so nothing is reset
// between launches; the two directions have separate lanes and counters because their writers differ.  All waits are
// bounded: on expiry the CTA records a status code and returns.
#include <cuda_runtime.h>
#include <cooperative_groups.h>
#include <stdint.h>

#include <string>

#include "api.h"
#include "common.cuh"

namespace {
using namespace rtp;

constexpr int kShiftThreads = 256;
constexpr int kDepth = 2;                               // chunks per lane
constexpr unsigned long long kChunk = 32768;            // bytes per chunk
constexpr int kMaxLanes = 64;                           // CTAs per rank
constexpr int kMaxEmu = 4;

// Layout of a staging area (one per rank, peer-mapped):
//   [flags: 2 directions x kMaxLanes x {arrive, credit, sent} x 128 B][data: 2 directions x lanes x kDepth x kChunk]
// with `lanes` fixed when the area is created (every launch on it must use the same value).
constexpr unsigned long long kFlagStride = 128;
constexpr unsigned long long kFlagsBytes = 2ull * kMaxLanes * 3 * kFlagStride;
__host__ __device__ inline unsigned long long* flag_ptr(void* base, int dir, int lane, int which) {
  return reinterpret_cast<unsigned long long*>(reinterpret_cast<uint8_t*>(base) +
                                               ((unsigned long long)(dir * kMaxLanes + lane) * 3 + which) * kFlagStride);
}
__host__ __device__ inline uint8_t* data_ptr(void* base, int dir, int lane, int slot, int lanes) {
  return reinterpret_cast<uint8_t*>(base) + kFlagsBytes + ((unsigned long long)(dir * lanes + lane) * kDepth + slot) * kChunk;
}

struct ShiftRank {
  void* buf;                 // local buffer that is replaced
  unsigned long long bytes;  // multiple of 16
  void* mine;                // this rank's staging area
  void* dst;                 // staging area of the rank this one sends to
  void* src;                 // staging area of the rank this one receives from
  int dir;                   // 0 = down (send to r-1), 1 = up
  unsigned long long* status;
  unsigned long long timeout_ns;
};
struct ShiftParams {
  ShiftRank r[kMaxEmu];
  int lanes;                 // CTAs per rank
};

__global__ void __launch_bounds__(kShiftThreads) ring_shift_kernel(const __grid_constant__ ShiftParams p) {
  const int vr = (int)blockIdx.x / p.lanes, lane = (int)blockIdx.x % p.lanes;
  const ShiftRank& R = p.r[vr];
  __shared__ uint32_t abort_flag;
  __shared__ uint32_t s_ok;
  if (threadIdx.x == 0) abort_flag = 0;
  __syncthreads();
  // this lane's range of the buffer, in chunks
  const unsigned long long nchunks = (R.bytes + kChunk - 1) / kChunk;
  const unsigned long long per = (nchunks + p.lanes - 1) / p.lanes;
  const unsigned long long c_lo = per * lane, c_hi = c_lo + per < nchunks ? c_lo + per : nchunks;
  unsigned long long* my_arrive = flag_ptr(R.mine, R.dir, lane, 0);    // bumped by my source
  unsigned long long* my_credit = flag_ptr(R.mine, R.dir, lane, 1);    // bumped by my destination
  unsigned long long* my_sent = flag_ptr(R.mine, R.dir, lane, 2);      // chunks this lane has pushed so far (local only)
  unsigned long long* dst_arrive = flag_ptr(R.dst, R.dir, lane, 0);
  unsigned long long* src_credit = flag_ptr(R.src, R.dir, lane, 1);
  const unsigned long long base = *my_sent;
  uint8_t* buf = reinterpret_cast<uint8_t*>(R.buf);
  unsigned long long m = base;                         // cumulative index of the chunk being moved
  for (unsigned long long c = c_lo; c < c_hi; ++c, ++m) {
    const int slot = (int)(m % kDepth);
    const unsigned long long off = c * kChunk;
    const unsigned long long n = (R.bytes - off < kChunk ? R.bytes - off : kChunk) >> 4;   // 16-byte units
    if (threadIdx.x == 0) {
      // the slot's previous content (my chunk m - kDepth) has been consumed by the destination
      uint32_t ok = 1;
      if (m >= (unsigned long long)kDepth)
        ok = wait_counter_ge(my_credit, m - kDepth + 1, &abort_flag, R.status, R.timeout_ns, ST_TIMEOUT_CREDIT) ? 1u : 0u;
      s_ok = ok;
    }
    __syncthreads();
    if (!s_ok) break;
    {
      const uint4* s = reinterpret_cast<const uint4*>(buf + off);
      uint4* d = reinterpret_cast<uint4*>(data_ptr(R.dst, R.dir, lane, slot, p.lanes));
      for (unsigned long long i = threadIdx.x; i < n; i += kShiftThreads) d[i] = s[i];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      red_relaxed_sys_add(dst_arrive, 1ull);
      s_ok = wait_counter_ge(my_arrive, m + 1, &abort_flag, R.status, R.timeout_ns, ST_TIMEOUT_ARRIVAL) ? 1u : 0u;
    }
    __syncthreads();
    if (!s_ok) break;
    {
      const uint4* s = reinterpret_cast<const uint4*>(data_ptr(R.mine, R.dir, lane, slot, p.lanes));
      uint4* d = reinterpret_cast<uint4*>(buf + off);
      for (unsigned long long i = threadIdx.x; i < n; i += kShiftThreads) d[i] = __ldcv(s + i);
    }
    __syncthreads();
    if (threadIdx.x == 0) red_relaxed_sys_add(src_credit, 1ull);   // "read done": nothing of mine has to be visible first
  }
  if (threadIdx.x == 0) *my_sent = base + (c_hi > c_lo ? c_hi - c_lo : 0);
}

thread_local std::string g_serr;
int sfail(const std::string& s) { g_serr = s; return -1; }

}  // namespace

extern "C" {

const char* rtp_shift_last_error(void) { return g_serr.c_str(); }

// bytes of one staging area for `lanes` CTAs per rank
unsigned long long rtp_shift_staging_bytes(int lanes) {
  if (lanes < 1) lanes = 1;
  if (lanes > kMaxLanes) lanes = kMaxLanes;
  return kFlagsBytes + 2ull * lanes * kDepth * kChunk;
}
// cudaMalloc of a staging area with zeroed counters (its handle is exchanged with rtp_ws_ipc_get / rtp_ws_ipc_open)
int rtp_shift_staging_create(int lanes, void** out) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, rtp_shift_staging_bytes(lanes));
  if (e != cudaSuccess) return sfail(std::string("cudaMalloc staging: ") + cudaGetErrorString(e));
  e = cudaMemset(p, 0, kFlagsBytes);
  if (e != cudaSuccess) { cudaFree(p); return sfail("cudaMemset staging failed"); }
  *out = p;
  return 0;
}
int rtp_shift_staging_destroy(void* p) { return cudaFree(p) == cudaSuccess ? 0 : sfail("cudaFree failed"); }
int rtp_shift_max_lanes(void) { return kMaxLanes; }

// Shifts `world_emulated` ranks at once (1 for a real multi-GPU ring: every process launches its own rank's kernel;
// 2..4 to emulate a ring on one GPU in a cooperative launch).  staging[e] / buf[e] belong to emulated rank e;
// dst_staging[e] / src_staging[e] are the staging areas of the ranks it sends to / receives from, as mapped here.
int rtp_ring_shift(int world_emulated, void* const* buf, unsigned long long bytes, void* const* staging,
                   void* const* dst_staging, void* const* src_staging, int direction, int lanes,
                   unsigned long long* const* status, unsigned long long timeout_ns, void* stream) {
  if (world_emulated < 1 || world_emulated > kMaxEmu) return sfail("ring_shift: 1 to 4 ranks per launch");
  if (bytes % 16) return sfail("ring_shift: bytes must be a multiple of 16");
  if (lanes < 1 || lanes > kMaxLanes) return sfail("ring_shift: lanes out of range");
  if (direction != 0 && direction != 1) return sfail("ring_shift: direction must be 0 (down) or 1 (up)");
  static thread_local ShiftParams P;
  for (int e = 0; e < world_emulated; ++e) {
    if ((reinterpret_cast<uintptr_t>(buf[e]) & 15) != 0) return sfail("ring_shift: buffer must be 16-byte aligned");
    P.r[e].buf = buf[e]; P.r[e].bytes = bytes;
    P.r[e].mine = staging[e]; P.r[e].dst = dst_staging[e]; P.r[e].src = src_staging[e];
    P.r[e].dir = direction;
    P.r[e].status = status[e];
    P.r[e].timeout_ns = timeout_ns ? timeout_ns : 2000000000ull;
  }
  P.lanes = lanes;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(lanes * world_emulated);
  cfg.blockDim = dim3(kShiftThreads);
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeCooperative;
  at[0].val.cooperative = world_emulated > 1 ? 1 : 0;    // emulated ranks wait on one another: all CTAs must be resident
  cfg.attrs = at;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, ring_shift_kernel, P);
  if (e != cudaSuccess) return sfail(std::string("ring_shift launch: ") + cudaGetErrorString(e));
  return 0;
}

}  // extern "C"
