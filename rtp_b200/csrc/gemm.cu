// Host side of the rotation GEMM kernel: tensor-map encoding, program builders for the plain GEMM and
// for the rotated (column/row) linear layers in forward and backward, and the launchers.
//
// Rotation schedule (forward): rank r uses shard (r+i)%N at step i, the same visiting order as the
// reference's ColumnParallelLinear.forward (rtp/module/linear.py:204-236).  Because NVSwitch gives
// every pair of GPUs the same bandwidth, a shard is not forwarded hop by hop: its owner pushes it from
// its (read-only) home buffer straight into the slot of the rank that needs it next, so no rank ever
// waits for a neighbour to finish forwarding.  Backward visits shards in the order r-1, r-2, ..., r
// (rtp/module/collectives.py:281-317), weights again pushed by their owners.  The gradient of a shard
// does not travel from rank to rank either: every rank stores its contribution straight into a gradient
// slot of the owner (one slot per contributing rank) and the owner adds the N contributions in a last
// phase: a reduce-scatter done as one all-to-all hop instead of N-1 dependent ones.
// Sums over visiting shards (row-mode forward, column-mode input gradient) are ONE K-segmented phase whose
// contraction walks over the shards in their order of arrival, so their output is written once.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cooperative_groups.h>
#include <mutex>
#include <string>
#include <vector>
#include <algorithm>
#include <cstring>
#include <cstdio>
#include <cstdlib>
#include "api.h"
#include "gemm_kernel.cuh"
#include "launch.h"
#include "tmap.h"

namespace {

thread_local std::string g_err;
int fail(const std::string& s) { g_err = s; return -1; }

using rtp::EncodeTiledFn;
EncodeTiledFn get_encode() { return rtp::get_encode_tiled(); }

// 2-D bf16 tensor map over a row-major [outer, inner] view with row pitch `ld` elements.
// box = [box_outer rows, 64 elements], 128-byte swizzle, zero fill outside the tensor.
int make_map(CUtensorMap* m, const void* ptr, long long inner, long long outer, long long ld, int box_outer) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return fail("cuTensorMapEncodeTiled entry point not found");
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0) return fail("TMA operand base is not 16-byte aligned");
  if ((ld * 2) % 16 != 0) return fail("TMA operand row pitch is not a multiple of 16 bytes");
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  return 0;
}
// operand stored [rows, k] row-major (K-major)
int make_map_k(CUtensorMap* m, const void* ptr, long long rows, long long k, long long ld, int box_rows = 128) {
  return make_map(m, ptr, k, rows, ld, box_rows);
}
// operand stored [k, mn] row-major (MN-major): boxes of [64 k rows, 64 mn]
int make_map_mn(CUtensorMap* m, const void* ptr, long long mn, long long k, long long ld) {
  return make_map(m, ptr, mn, k, ld, 64);
}
// Same operand as a 3-D tensor {64 mn, k, mn / 64} with box {64, 64, nblk}: ONE copy per stage delivers the nblk 64-wide
// column blocks side by side, exactly the shared-memory layout the UMMA descriptors expect (the producer thread is
// issue-bound, so halving its copies per k-block matters).  Needs mn % 64 == 0; *is3d tells which form was built
// (falls back to the 2-D map otherwise, also if the driver rejects the encoding).
int make_map_mn3(CUtensorMap* m, const void* ptr, long long mn, long long k, long long ld, int nblk, unsigned char* is3d) {
  *is3d = 0;
  EncodeTiledFn enc = get_encode();
  if (enc && nblk >= 1 && mn % 64 == 0 && (reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && (ld * 2) % 16 == 0) {
    cuuint64_t dims[3] = {64u, (cuuint64_t)k, (cuuint64_t)(mn / 64)};
    cuuint64_t strides[2] = {(cuuint64_t)ld * 2, 128u};
    cuuint32_t box[3] = {64u, 64u, (cuuint32_t)nblk};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) { *is3d = 1; return 0; }
  }
  return make_map_mn(m, ptr, mn, k, ld);
}

// Per-device facts are cached per device: one process may drive several GPUs.
constexpr int kMaxDevices = 64;
int current_device() {
  int dev = 0;
  cudaGetDevice(&dev);
  return (dev >= 0 && dev < kMaxDevices) ? dev : 0;
}
int sm_count() {
  static int n[kMaxDevices] = {0};
  const int dev = current_device();
  if (!n[dev]) cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
  return n[dev];
}

void init_phase(RtpPhase& ph) {
  memset(&ph, 0, sizeof(ph));
  for (int w = 0; w < RTP_MAX_WAITS; ++w) { ph.wait_ctr[w] = -1; ph.done_ctr[w] = -1; }
  ph.credit_ctr = -1;
  ph.bn = 128;
  ph.batch = 1;
  ph.batch_inner = 1;
  ph.b_box = 128;
  ph.alpha = 1.f;
}
void set_peers(const RtpRing& R, RtpProgram& P) {
  P.rank = R.rank;
  P.world = R.world;
  for (int t = 0; t < RTP_FLAG_MAX_WORLD; ++t)
    P.peer_flags[t] = (t < R.world && R.ws[t]) ? reinterpret_cast<RtpFlagBlock*>(R.ws[t]) : nullptr;
}
void init_program(RtpProgram& p) {
  memset(&p, 0, sizeof(p));
  p.timeout_ns = 2000000000ull;
}

bool aligned16(const void* p, long long ld_elems, int elem_bytes) {
  return (reinterpret_cast<uintptr_t>(p) & 15) == 0 && ((ld_elems * elem_bytes) & 15) == 0;
}
void set_vec_ok(RtpPhase& ph) {
  bool ok = aligned16(ph.d, ph.ldd, ph.d_fp32 ? 4 : 2);
  if (ph.c) ok = ok && aligned16(ph.c, ph.ldc, ph.c_fp32 ? 4 : 2);
  if (ph.mask) ok = ok && aligned16(ph.mask, ph.ldmask, 2);
  ph.vec_ok = ok ? 1 : 0;
}
// CTA-pair mode (cta_group::2).  Policy: 1 = always (launches with an even grid), 0 = never, -1 = automatic: pairs are
// used when the output has at least one 256 x 256 tile per CTA, which is where halving the B traffic per SM pays for
// the cluster launch.  RTP_PAIR=0/1 or rtp_set_pair_mode() override; the decision is taken once per program, before
// its tensor maps are built.
int g_pair = -2;                 // -2: environment not read yet
thread_local bool t_pair = false;
int pair_policy() {
  if (g_pair == -2) {
    const char* e = getenv("RTP_PAIR");
    g_pair = (e && e[0] == '1') ? 1 : (e && e[0] == '0') ? 0 : -1;
  }
  return g_pair;
}
void decide_pair(long long M, long long N, int ctas, bool eligible = true) {
  const int pol = pair_policy();
  const long long t256 = ((M + 255) / 256) * ((N + 255) / 256);
  t_pair = eligible && (pol == 1 || (pol == -1 && M >= 512 && t256 >= ctas));
}
bool pair_mode() { return t_pair; }
int pick_bn(int M, int N, int ctas) {
  if (pair_mode()) {
    long long t256 = (long long)((M + 255) / 256) * ((N + 255) / 256);
    return (t256 >= ctas / 2) ? 256 : 128;
  }
  long long t256 = (long long)((M + 127) / 128) * ((N + 255) / 256);
  return (t256 >= ctas) ? 256 : 128;
}
uint32_t drop_threshold(float p) {
  if (p <= 0.f) return 0;
  double t = (double)p * 4294967296.0;
  if (t > 4294967295.0) t = 4294967295.0;
  return (uint32_t)t;
}

// Pipeline geometry: the stage must hold the widest B tile of the program; narrower tiles get more stages.
int g_force_stages = 0;
unsigned long long* g_trace = nullptr;   // tuning aid, see rtp_debug_set_trace
// CTAs reserved for the push jobs of a launch (they own no GEMM tile, so their copy engine is not shared with a tile
// pipeline and their tile memory becomes a deep copy ring).  RTP_PUSH_CTAS overrides; 0 = every CTA pushes a share.
int g_push_ctas = -2;
int push_cta_policy(int ctas) {
  if (g_push_ctas == -2) {
    const char* e = getenv("RTP_PUSH_CTAS");
    g_push_ctas = e ? atoi(e) : -1;
  }
  // default 0: measured on two B200s, an SM sends to a peer at a limited rate, so a launch moves more when every CTA
  // pushes a share than when a few reserved CTAs push everything
  int r = g_push_ctas >= 0 ? g_push_ctas : 0;
  if (r >= ctas) r = 0;
  return r;
}
// How the pusher warp moves a shard (RTP_PUSH_RING; unset = chosen per launch): 2 = plain loads and peer stores through registers; bulk
// copies through a shared-memory ring per CTA: 0 / 3 = four 3840-byte chunks, completion awaited 3 / 12 copies behind the
// issue point; 1 / 4 = two 7680-byte chunks, 1 / 8 copies behind.
int push_ring_policy(const RtpProgram& P) {
  static int v = -2;
  if (v == -2) {
    const char* e = getenv("RTP_PUSH_RING");
    v = e ? atoi(e) : -1;
    if (v < -1 || v > 4) v = -1;
  }
  if (v >= 0) return v;
  // Automatic: plain stores, except for a launch with one very large job (a ring of two ranks with big layers), where
  // the bulk copies are faster and their one completion wait costs nothing.  (GPT-1.3B on 2 GPUs with bulk copies for
  // every push, RTP_PUSH_RING=0: 187 ms per step against 222 ms with plain stores.)
  if (P.n_pushes == 1 && P.pushes[0].bytes >= (32ull << 20)) return 0;
  return 2;
}
void finalize_program(RtpProgram& P, int ctas, bool pair) {
  const int tm = pair ? 256 : 128;
  P.push_ring = push_ring_policy(P);
  int reserved = P.n_pushes > 0 ? push_cta_policy(ctas) : 0;
  if (pair) reserved &= ~1;
  P.n_compute = ctas - reserved;
  ctas = P.n_compute;
  if (pair) ctas /= 2;
  // Tile t of a phase runs on CTA (t + cta_off) % ctas.  Successive phases start where the previous one ended, so
  // that small per-step GEMMs fill the whole grid.  A phase that accumulates into the output of an earlier phase
  // (C == that phase's D) must keep that phase's mapping: the read-modify-write of a tile then stays inside one CTA,
  // ordered by program order.
  long long acc = 0;
  for (int i = 0; i < P.n_phases; ++i) {
    RtpPhase& ph = P.phases[i];
    if (ph.kind != RTP_KIND_GEMM) { ph.cta_off = 0; continue; }
    const long long tiles = (long long)((ph.M + tm - 1) / tm) * ((ph.N + ph.bn - 1) / ph.bn) * ph.batch;
    int chained = -1;
    if (ph.c)
      for (int k = 0; k < i; ++k)
        if (P.phases[k].kind == RTP_KIND_GEMM && P.phases[k].d == ph.c && P.phases[k].M == ph.M &&
            P.phases[k].N == ph.N && P.phases[k].bn == ph.bn)
          chained = k;
    if (chained >= 0) {
      ph.cta_off = P.phases[chained].cta_off;
    } else {
      ph.cta_off = (int)(acc % ctas);
      acc += tiles;
    }
  }
  int bn = pair ? 64 : 128;   // widest B tile staged by ONE CTA
  for (int i = 0; i < P.n_phases; ++i) {
    const int w = pair ? P.phases[i].bn / 2 : P.phases[i].bn;
    if (P.phases[i].kind == RTP_KIND_GEMM && w > bn) bn = w;
  }
  P.stage_bytes = rtp::kABytes + bn * rtp::kBK * 2;
  P.n_stages = rtp::kTileBytes / P.stage_bytes;
  if (P.n_stages > rtp::kMaxStages) P.n_stages = rtp::kMaxStages;
  if (g_force_stages > 0 && g_force_stages < P.n_stages) P.n_stages = g_force_stages;
}

template <int NEMU, bool PAIR>
int launch_impl(const rtp::GemmParams<NEMU>& params, int grid, bool cooperative, cudaStream_t stream) {
  // the shared-memory limit is an attribute of the kernel on ONE device: set once per (instantiation, device)
  static bool attr_set[kMaxDevices] = {false};
  const int dev = current_device();
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(rtp::rtp_gemm_kernel<NEMU, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         rtp::kSmemBytes);
    if (e != cudaSuccess) return fail(std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(rtp::kNumThreads);
  cfg.dynamicSmemBytes = rtp::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute at[3];
  int nat = 0;
  if (cooperative) {
    at[nat].id = cudaLaunchAttributeCooperative;
    at[nat].val.cooperative = 1;
    ++nat;
  } else if (rtp::pdl_enabled()) {
    // the kernel waits for its predecessor (griddepcontrol.wait) after its shared-memory / TMEM set-up
    at[nat].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[nat].val.programmaticStreamSerializationAllowed = 1;
    ++nat;
  }
  if (PAIR) {
    at[nat].id = cudaLaunchAttributeClusterDimension;
    at[nat].val.clusterDim.x = 2;
    at[nat].val.clusterDim.y = 1;
    at[nat].val.clusterDim.z = 1;
    ++nat;
  }
  cfg.attrs = at;
  cfg.numAttrs = nat;
  if (NEMU == 1) finalize_program(const_cast<RtpProgram&>(params.prog[0]), params.ctas_per_rank, PAIR);
  cudaError_t e = cudaLaunchKernelEx(&cfg, rtp::rtp_gemm_kernel<NEMU, PAIR>, params);
  if (e != cudaSuccess) return fail(std::string("launch rtp_gemm_kernel: ") + cudaGetErrorString(e));
  return 0;
}
// `allow_pair`: the caller built the program with pair-compatible tensor maps and tile widths
template <int NEMU>
int launch(const rtp::GemmParams<NEMU>& params, int grid, bool cooperative, cudaStream_t stream, bool allow_pair = false) {
  if (NEMU == 1 && allow_pair && pair_mode() && grid % 2 == 0 && params.ctas_per_rank % 2 == 0)
    return launch_impl<1, true>(reinterpret_cast<const rtp::GemmParams<1>&>(params), grid, cooperative, stream);
  return launch_impl<NEMU, false>(params, grid, cooperative, stream);
}

// ------------------------------------------------------------------------------------------------
// workspace layout
// ------------------------------------------------------------------------------------------------
constexpr unsigned long long kFlagBytes = RTP_FLAG_BYTES;
static_assert(sizeof(RtpFlagBlock) <= kFlagBytes, "flag block too large");
RtpFlagBlock* ws_flags(void* ws) { return reinterpret_cast<RtpFlagBlock*>(ws); }
// Physical layout of a workspace of a ring of `world` ranks: [flag block][bank 0: world-1 weight slots][bank 1: world-1
// weight slots][world gradient slots].  `i` is the logical weight slot (bank * RTP_NUM_SLOTS + index in the bank).
uint8_t* ws_wslot(void* ws, unsigned long long slot_bytes, int i, int world) {
  const int bank = i / RTP_NUM_SLOTS, idx = i % RTP_NUM_SLOTS;
  return reinterpret_cast<uint8_t*>(ws) + kFlagBytes + (unsigned long long)(bank * (world - 1) + idx) * slot_bytes;
}
uint8_t* ws_gslot(void* ws, unsigned long long slot_bytes, int i, int world) {
  return reinterpret_cast<uint8_t*>(ws) + kFlagBytes +
         (unsigned long long)(RTP_NUM_WBANKS * (world - 1) + i) * slot_bytes;
}
int mod(int a, int n) { return ((a % n) + n) % n; }

// Cross-launch prefetch: pushes the home shard of the NEXT rotated linear into weight-slot bank `bank` of the ranks
// that will read it there (kind 0: forward visiting order, 1: backward visiting order).  The fills are counted by the
// launch that consumes them.
int add_prefetch_pushes(const RtpRing& R, RtpProgram& P, const void* home, unsigned long long bytes, int bank, int kind) {
  const int N = R.world, r = R.rank;
  if (!home || N == 1) return 0;
  if (bytes > R.slot_bytes) return fail("prefetched shard larger than workspace slot");
  if (bytes % 16) return fail("next_bytes must be a multiple of 16");
  if (bank < 0 || bank >= RTP_NUM_WBANKS) return fail("bank out of range");
  for (int s = 0; s + 1 < N; ++s) {
    if (P.n_pushes >= RTP_MAX_PUSHES) return fail("too many pushes");
    RtpPush& pu = P.pushes[P.n_pushes++];
    memset(&pu, 0, sizeof(pu));
    const int t = kind == 0 ? mod(r - (s + 1), N) : mod(r + 1 + s, N);
    const int slot = bank * RTP_NUM_SLOTS + s;
    pu.src = home;
    pu.dst = ws_wslot(R.ws[t], R.slot_bytes, slot, R.world);
    pu.bytes = bytes;
    pu.credit_ptr = &ws_flags(R.ws[R.rank])->credit[t][RTP_CTR_W0 + slot].v;
    pu.credit_ctr = RTP_CTR_W0 + slot;
    pu.credit_rel = 0;
    pu.arrive_ptr = &ws_flags(R.ws[t])->arrive[RTP_CTR_W0 + slot].v;
  }
  return 0;
}

// Tile-segmented phases (one phase for all shards of a column-mode forward / weight gradient) can be switched off
// with RTP_SEG_TILES=0: the builders then emit one phase per shard.
bool seg_tiles_ok() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("RTP_SEG_TILES");
    v = (e && atoi(e) == 0) ? 0 : 1;
  }
  return v == 1;
}

// ------------------------------------------------------------------------------------------------
// program builders
// ------------------------------------------------------------------------------------------------
int build_linear_fwd(const RtpRing& R, const RtpLinearFwd& op, RtpProgram& P) {
  init_program(P);
  const int N = R.world, r = R.rank;
  if (N < 1 || N > RTP_MAX_WORLD) return fail("world size out of range");
  if (N > RTP_MAX_PHASES) return fail("too many phases");
  const bool col = op.mode == 0;
  if (col ? (op.out_features % N) : (op.in_features % N)) return fail("features not divisible by world size");
  const int Os = col ? op.out_features / N : op.out_features;  // rows of a weight shard
  const int Ks = col ? op.in_features : op.in_features / N;    // columns of a weight shard
  if (N > 1 && op.shard_bytes > R.slot_bytes) return fail("shard larger than workspace slot");
  if (op.shard_bytes % 16) return fail("shard_bytes must be a multiple of 16");
  if (op.bank < 0 || op.bank >= RTP_NUM_WBANKS) return fail("bank out of range");
  const int wb = op.bank * RTP_NUM_SLOTS;   // first weight slot of the bank this launch reads
  void* ws = R.ws[r];
  P.flags = ws ? ws_flags(ws) : nullptr;
  set_peers(R, P);
  P.status = ws ? &ws_flags(ws)->status.v : nullptr;
  P.timeout_ns = R.timeout_ns ? R.timeout_ns : 2000000000ull;

  // maps: 0 = x, 1 = home, 1+i = weight slot i-1 (read at step i)
  if (make_map_k(&P.maps[0], op.x, op.M, op.in_features, op.ldx)) return -1;
  const int bn = pick_bn(op.M, col ? Os : op.out_features, R.ctas);
  const int b_box = pair_mode() ? bn / 2 : 128;
  if (make_map_k(&P.maps[1], op.home, Os, Ks, Ks, b_box)) return -1;
  for (int i = 1; i < N; ++i)
    if (make_map_k(&P.maps[1 + i], ws_wslot(ws, R.slot_bytes, wb + i - 1, R.world), Os, Ks, Ks, b_box)) return -1;
  if (!col && N > 1) {
    // Row mode on a ring: y = sum_j x[:, block j] W_j^T + sum_j b_j is ONE phase whose contraction walks over the shards
    // in their order of arrival (own shard first), so the output is written once instead of N read-modify-write passes.
    P.n_phases = 1;
    RtpPhase& ph = P.phases[0];
    init_phase(ph);
    ph.a_map = 0; ph.b_map = 1;
    ph.M = op.M; ph.N = Os; ph.K = Ks;
    ph.bn = bn; ph.b_box = b_box;
    ph.ldd = op.ldy; ph.d = op.y;
    ph.nseg = N;
    for (int i = 0; i < N; ++i) {
      const int j = mod(r + i, N);
      const int slot = wb + i - 1;
      const uint8_t* src = (i == 0) ? reinterpret_cast<const uint8_t*>(op.home) : ws_wslot(ws, R.slot_bytes, slot, R.world);
      ph.seg_a_off_k[i] = j * Ks;
      ph.seg_b_map[i] = (i == 0) ? 1 : 1 + i;
      if (i > 0) {
        ph.wait_ctr[i] = RTP_CTR_W0 + slot; ph.wait_rel[i] = 0;
        ph.done_ctr[i] = RTP_CTR_W0 + slot;
        P.uses_inc[RTP_CTR_W0 + slot] = 1;
      }
      if (op.bias_off >= 0) {
        const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(src) + op.bias_off;
        if (i == 0) ph.bias = b; else ph.bias_more[ph.n_bias_more++] = b;
      }
    }
    ph.act = op.act;
    ph.drop_thresh = drop_threshold(op.drop_p);
    ph.drop_scale = op.drop_p > 0.f ? 1.f / (1.f - op.drop_p) : 1.f;
    ph.drop_seed = op.seed; ph.drop_offset = op.offset; ph.drop_step_ptr = op.step_ptr;
    set_vec_ok(ph);
  } else if (col && N > 1 && seg_tiles_ok() && Os % bn == 0) {
    // Column mode on a ring: y[:, block j] = x W_j^T + b_j for every shard is ONE phase whose output columns fall into N
    // segments in the order of arrival of the shards (own shard first); a tile reads its shard's tensor map once the
    // shard has arrived.
    P.n_phases = 1;
    RtpPhase& ph = P.phases[0];
    init_phase(ph);
    RtpSegTable& st = P.segtab[0];
    ph.a_map = 0; ph.b_map = 1;
    ph.M = op.M; ph.N = op.out_features; ph.K = Ks;
    ph.bn = bn; ph.b_box = b_box;
    ph.ldd = op.ldy; ph.d = op.y;
    ph.tseg = 1; ph.tseg_len = Os; ph.tseg_n = N; ph.tseg_tab = 0;
    for (int i = 0; i < N; ++i) {
      const int j = mod(r + i, N);
      const int slot = wb + i - 1;
      const uint8_t* src = (i == 0) ? reinterpret_cast<const uint8_t*>(op.home) : ws_wslot(ws, R.slot_bytes, slot, R.world);
      st.map[i] = (i == 0) ? 1 : 1 + i;
      st.off_mn[i] = 0;
      st.drop_add[i] = j;
      st.d[i] = reinterpret_cast<__nv_bfloat16*>(op.y) + (long long)j * Os;
      st.bias[i] = op.bias_off >= 0 ? reinterpret_cast<const __nv_bfloat16*>(src) + op.bias_off : nullptr;
      if (i > 0) {
        ph.wait_ctr[i] = RTP_CTR_W0 + slot; ph.wait_rel[i] = 0;
        ph.done_ctr[i] = RTP_CTR_W0 + slot;
        P.uses_inc[RTP_CTR_W0 + slot] = 1;
      }
    }
    ph.act = op.act;
    ph.drop_thresh = drop_threshold(op.drop_p);
    ph.drop_scale = op.drop_p > 0.f ? 1.f / (1.f - op.drop_p) : 1.f;
    ph.drop_seed = op.seed; ph.drop_offset = op.offset; ph.drop_step_ptr = op.step_ptr;
    set_vec_ok(ph);
  } else {
  P.n_phases = N;
  for (int i = 0; i < N; ++i) {
    RtpPhase& ph = P.phases[i];
    init_phase(ph);
    const int j = mod(r + i, N);
    const int slot = wb + i - 1;   // step i reads weight slot i-1 of the bank (filled once by the owner of shard j)
    const uint8_t* src = (i == 0) ? reinterpret_cast<const uint8_t*>(op.home) : ws_wslot(ws, R.slot_bytes, slot, R.world);
    ph.a_map = 0;
    ph.b_map = (i == 0) ? 1 : 1 + i;
    ph.M = op.M;
    ph.N = Os;
    ph.K = Ks;
    ph.bn = bn;
    ph.b_box = b_box;
    ph.ldd = op.ldy;
    ph.d = reinterpret_cast<__nv_bfloat16*>(op.y) + (col ? (long long)j * Os : 0);
    if (!col) {
      ph.a_off_k = j * Ks;
      if (i > 0) { ph.c = op.y; ph.ldc = op.ldy; }
    }
    if (op.bias_off >= 0) ph.bias = reinterpret_cast<const __nv_bfloat16*>(src) + op.bias_off;
    // activation / dropout act on the finished output: every step in column mode, the last one in row mode
    if (col || i == N - 1) {
      ph.act = op.act;
      ph.drop_thresh = drop_threshold(op.drop_p);
      ph.drop_scale = op.drop_p > 0.f ? 1.f / (1.f - op.drop_p) : 1.f;
      ph.drop_seed = op.seed;
      ph.drop_offset = op.offset + (unsigned long long)(col ? j : 0);
      ph.drop_step_ptr = op.step_ptr;
    }
    if (i > 0) {
      ph.wait_ctr[0] = RTP_CTR_W0 + slot;
      ph.wait_rel[0] = 0;
      ph.done_ctr[0] = RTP_CTR_W0 + slot;
      P.uses_inc[RTP_CTR_W0 + slot] = 1;
    }
    set_vec_ok(ph);
  }
  }
  P.n_pushes = op.no_self_push ? 0 : N - 1;
  for (int i = 0; i + 1 < N && !op.no_self_push; ++i) {
    RtpPush& pu = P.pushes[i];
    memset(&pu, 0, sizeof(pu));
    const int t = mod(r - (i + 1), N);
    const int slot = wb + i;
    pu.src = op.home;
    pu.dst = ws_wslot(R.ws[t], R.slot_bytes, slot, R.world);
    pu.bytes = op.shard_bytes;
    pu.credit_ptr = &ws_flags(R.ws[R.rank])->credit[t][RTP_CTR_W0 + slot].v;
    pu.credit_ctr = RTP_CTR_W0 + slot;
    pu.credit_rel = 0;
    pu.arrive_ptr = &ws_flags(R.ws[t])->arrive[RTP_CTR_W0 + slot].v;
  }
  return add_prefetch_pushes(R, P, op.next_home, op.next_bytes, 1 - op.bank, op.next_kind);
}

// Whether a backward launch computes its bias gradient as a GEMM phase of its own (see RtpLinearBwd::ones).  Needs the
// pair decision of the launch to have been made (decide_pair).
bool folds_bias(const RtpRing& R, const RtpLinearBwd& op) {
  return R.world == 1 && !pair_mode() && op.M % 8 == 0 && op.out_features % 8 == 0 &&
         (reinterpret_cast<uintptr_t>(op.ones) & 15) == 0;
}

int build_linear_bwd(const RtpRing& R, const RtpLinearBwd& op, RtpProgram& P) {
  // Backward on a ring of N ranks.  Rank r visits the shards in the order r-1, r-2, ..., r (step s handles shard
  // j = r-1-s; weights are pushed by their owners into weight slot s).  The weight gradient of shard j computed here
  // does not hop around the ring: NVSwitch makes every peer equally near, so it is stored straight into gradient slot
  // number s of the OWNER j (each owner receives N-1 slots, one per peer, plus its own contribution in a local slot)
  // and the owner adds the N contributions in one last phase.  No phase waits for another rank's compute, so all 2N
  // GEMM phases of a launch are free to run concurrently across the grid.
  init_program(P);
  const int N = R.world, r = R.rank;
  if (N < 1 || N > RTP_MAX_WORLD || 2 * N + 2 > RTP_MAX_PHASES) return fail("world size out of range");
  const bool col = op.mode == 0;
  if (col ? (op.out_features % N) : (op.in_features % N)) return fail("features not divisible by world size");
  const int Os = col ? op.out_features / N : op.out_features;
  const int Ks = col ? op.in_features : op.in_features / N;
  if (N > 1 && op.shard_bytes > R.slot_bytes) return fail("shard larger than workspace slot");
  // shards pushed ahead by the previous launch must be read here: nobody else returns their slots' credits
  if (N > 1 && op.no_self_push && !op.dx)
    return fail("a backward launch whose weight shards were pushed ahead has to compute the input gradient (dx is null)");
  if (op.grad_accumulate && N > 1) return fail("grad_accumulate is only supported on a 1-rank ring");
  if (op.bank < 0 || op.bank >= RTP_NUM_WBANKS) return fail("bank out of range");
  const int wb = op.bank * RTP_NUM_SLOTS;   // first weight slot of the bank this launch reads
  void* ws = R.ws[r];
  P.flags = ws ? ws_flags(ws) : nullptr;
  set_peers(R, P);
  P.status = ws ? &ws_flags(ws)->status.v : nullptr;
  P.timeout_ns = R.timeout_ns ? R.timeout_ns : 2000000000ull;

  // maps: 0 = dy (MN-major view: k = tokens), 1 = x (MN-major view), 2 = dy (K-major view: k = out),
  //       3 = home W (MN-major view: k = shard rows), 4+s = weight slot s
  // MN-major operands travel as 3-D maps (one copy per operand and k-block) when every tile offset is a multiple of 64
  const bool m3 = Os % 64 == 0 && Ks % 64 == 0;
  const int bn_w = pick_bn(Os, Ks, R.ctas), bn_d = pick_bn(op.M, Ks, R.ctas);
  const int nb_w = (pair_mode() ? bn_w / 2 : bn_w) / 64, nb_d = (pair_mode() ? bn_d / 2 : bn_d) / 64;
  if (make_map_mn3(&P.maps[0], op.dy, op.out_features, op.M, op.ldy, m3 ? 2 : 0, &P.map3d[0])) return -1;
  if (make_map_mn3(&P.maps[1], op.x, op.in_features, op.M, op.ldx, m3 ? nb_w : 0, &P.map3d[1])) return -1;
  if (op.dx) {
    if (make_map_k(&P.maps[2], op.dy, op.M, op.out_features, op.ldy)) return -1;
    if (make_map_mn3(&P.maps[3], op.home, Ks, Os, Ks, m3 ? nb_d : 0, &P.map3d[3])) return -1;
    for (int s = 0; s + 1 < N; ++s)
      if (make_map_mn3(&P.maps[4 + s], ws_wslot(ws, R.slot_bytes, wb + s, R.world), Ks, Os, Ks, m3 ? nb_d : 0,
                       &P.map3d[4 + s]))
        return -1;
  }
  int np = 0;
  const int bn_wg = pick_bn(Os, Ks, R.ctas);
  const int tm = pair_mode() ? 256 : 128;
  if (col && N > 1 && seg_tiles_ok() && Os % tm == 0) {
    // ---- wgrad of every shard as ONE phase: dW[N * Os, Ks] = dy^T x, whose output rows fall into N segments, one per
    //      owner: the tiles of segment s go to gradient slot s of owner j (local slot N-1 for the own shard).
    RtpPhase& ph = P.phases[np++];
    init_phase(ph);
    RtpSegTable& st = P.segtab[0];
    ph.a_map = 0; ph.a_mn = 1;
    ph.b_map = 1; ph.b_mn = 1;
    ph.M = op.out_features; ph.N = Ks; ph.K = op.M;
    ph.bn = bn_wg;
    ph.ldd = Ks;
    ph.tseg = 2; ph.tseg_len = Os; ph.tseg_n = N; ph.tseg_tab = 0;
    for (int s = 0; s < N; ++s) {
      const int j = mod(r - 1 - s, N);
      uint8_t* dst = ws_gslot(R.ws[j], R.slot_bytes, s, R.world);
      st.map[s] = -1;
      st.off_mn[s] = j * Os;
      st.d[s] = dst;
      st.bias[s] = nullptr;
      st.credit_ptr[s] = &ws_flags(R.ws[R.rank])->credit[j][RTP_CTR_G0 + s].v;
      st.credit_ctr[s] = RTP_CTR_G0 + s;
      st.arrive_ptr[s] = &ws_flags(R.ws[j])->arrive[RTP_CTR_G0 + s].v;
      if (op.bias_off >= 0 && op.dbias_full) {
        st.vec_out[s] = reinterpret_cast<__nv_bfloat16*>(dst) + op.bias_off;
        st.vec_off[s] = (long long)j * Os;
      }
    }
    ph.d = st.d[0];
    ph.arrive_ptr = st.arrive_ptr[0];     // marks the phase as one that announces its output
    if (op.bias_off >= 0 && op.dbias_full) { ph.vec_add = op.dbias_full; ph.vec_len = Os; }
    set_vec_ok(ph);
  } else if (!col && N > 1 && seg_tiles_ok() && Ks % bn_wg == 0) {
    // ---- row mode: dW_j = dy^T x[:, block j] for every shard as ONE phase whose output COLUMNS fall into N segments
    RtpPhase& ph = P.phases[np++];
    init_phase(ph);
    RtpSegTable& st = P.segtab[0];
    ph.a_map = 0; ph.a_mn = 1;
    ph.b_map = 1; ph.b_mn = 1;
    ph.M = Os; ph.N = op.in_features; ph.K = op.M;
    ph.bn = bn_wg;
    ph.ldd = Ks;
    ph.tseg = 1; ph.tseg_len = Ks; ph.tseg_n = N; ph.tseg_tab = 0;
    for (int s = 0; s < N; ++s) {
      const int j = mod(r - 1 - s, N);
      uint8_t* dst = ws_gslot(R.ws[j], R.slot_bytes, s, R.world);
      st.map[s] = -1;
      st.off_mn[s] = j * Ks;
      st.d[s] = dst;
      st.bias[s] = nullptr;
      st.credit_ptr[s] = &ws_flags(R.ws[R.rank])->credit[j][RTP_CTR_G0 + s].v;
      st.credit_ctr[s] = RTP_CTR_G0 + s;
      st.arrive_ptr[s] = &ws_flags(R.ws[j])->arrive[RTP_CTR_G0 + s].v;
      if (op.bias_off >= 0 && op.dbias_full) {
        st.vec_out[s] = reinterpret_cast<__nv_bfloat16*>(dst) + op.bias_off;
        st.vec_off[s] = 0;
      }
    }
    ph.d = st.d[0];
    ph.arrive_ptr = st.arrive_ptr[0];     // marks the phase as one that announces its output
    if (op.bias_off >= 0 && op.dbias_full) { ph.vec_add = op.dbias_full; ph.vec_len = Os; }
    set_vec_ok(ph);
  } else
  for (int s = 0; s < N; ++s) {
    const int j = mod(r - 1 - s, N);
    // ---- wgrad: dW_j = dy_j^T x  -> gradient slot s of owner j (own shard: straight into the home gradient when
    //      the ring has one rank, else into the local slot N-1 that the final reduce reads)
    {
      RtpPhase& ph = P.phases[np++];
      init_phase(ph);
      ph.a_map = 0; ph.a_mn = 1;
      ph.b_map = 1; ph.b_mn = 1;
      ph.M = Os; ph.N = Ks; ph.K = op.M;
      if (col) ph.a_off_mn = j * Os; else ph.b_off_mn = j * Ks;
      ph.bn = pick_bn(ph.M, ph.N, R.ctas);
      uint8_t* dst;
      if (N == 1) dst = reinterpret_cast<uint8_t*>(op.grad_home);
      else dst = ws_gslot(R.ws[j], R.slot_bytes, s, R.world);
      ph.d = dst; ph.ldd = Ks;
      if (op.grad_accumulate && N == 1) { ph.c = op.grad_home; ph.ldc = Ks; }
      if (N > 1) {
        ph.credit_ptr = &ws_flags(R.ws[R.rank])->credit[j][RTP_CTR_G0 + s].v;
        ph.credit_ctr = RTP_CTR_G0 + s; ph.credit_rel = 0;
        ph.arrive_ptr = &ws_flags(R.ws[j])->arrive[RTP_CTR_G0 + s].v;
      }
      if (op.bias_off >= 0 && op.dbias_full) {
        ph.vec_out = reinterpret_cast<__nv_bfloat16*>(dst) + op.bias_off;
        ph.vec_in = (op.grad_accumulate && N == 1) ? reinterpret_cast<const __nv_bfloat16*>(op.grad_home) + op.bias_off : nullptr;
        ph.vec_add = op.dbias_full + (col ? (long long)j * Os : 0);
        ph.vec_len = Os;
      }
      set_vec_ok(ph);
    }
  }
  if (op.bias_off >= 0 && !op.dbias_full && op.ones && folds_bias(R, op)) {
    // ---- bias gradient as a GEMM: db[1, out] = ones[1, M] dy[M, out].  One row of A is real, the rest of the 128-row
    //      tile is zero fill; the few extra tiles ride in the grid beside the weight-gradient tiles.
    if (make_map_k(&P.maps[4], op.ones, 1, op.M, op.M)) return -1;
    if (make_map_mn3(&P.maps[5], op.dy, op.out_features, op.M, op.ldy, (op.out_features % 64 == 0) ? 2 : 0, &P.map3d[5]))
      return -1;
    RtpPhase& ph = P.phases[np++];
    init_phase(ph);
    ph.a_map = 4; ph.a_mn = 0;
    ph.b_map = 5; ph.b_mn = 1;
    ph.M = 1; ph.N = op.out_features; ph.K = op.M;
    ph.bn = 128;
    __nv_bfloat16* db = reinterpret_cast<__nv_bfloat16*>(op.grad_home) + op.bias_off;
    ph.d = db; ph.ldd = op.out_features;
    if (op.grad_accumulate) { ph.c = db; ph.ldc = op.out_features; }
    set_vec_ok(ph);
  }
  // The weight-gradient phases need only local operands, so they all come first and cover the time the weight shards
  // are in flight; the input-gradient phases follow, own shard first, then the visiting shards in order of arrival.
  if (col && N > 1 && op.dx) {
    // Column mode on a ring: dx = sum_j dy[:, block j] W_j is ONE phase whose contraction walks over the shards, own
    // shard first, then the visiting ones in their order of arrival; dx is written once.
    RtpPhase& ph = P.phases[np++];
    init_phase(ph);
    ph.a_map = 2; ph.a_mn = 0;
    ph.b_map = 3; ph.b_mn = 1;
    ph.M = op.M; ph.N = Ks; ph.K = Os;
    ph.bn = pick_bn(ph.M, ph.N, R.ctas);
    ph.ldd = op.lddx; ph.d = op.dx;
    if (op.dx_accumulate) { ph.c = op.dx; ph.ldc = op.lddx; }
    if (op.mask) { ph.mask = op.mask; ph.ldmask = op.ldmask; ph.mask_scale = op.mask_scale; }
    ph.nseg = N;
    for (int q = 0; q < N; ++q) {
      const int s = (q == 0) ? N - 1 : q - 1;
      const int j = mod(r - 1 - s, N);
      const bool last = s == N - 1;   // own shard
      ph.seg_a_off_k[q] = j * Os;
      ph.seg_b_map[q] = last ? 3 : 4 + s;
      if (!last) {
        ph.wait_ctr[q] = RTP_CTR_W0 + wb + s; ph.wait_rel[q] = 0;
        ph.done_ctr[q] = RTP_CTR_W0 + wb + s;
        P.uses_inc[RTP_CTR_W0 + wb + s] = 1;
      }
    }
    set_vec_ok(ph);
  } else if (!col && N > 1 && op.dx && !op.mask && !op.dx_accumulate && seg_tiles_ok() &&
             Ks % pick_bn(op.M, Ks, R.ctas) == 0) {
    // Row mode on a ring: dx[:, block j] = dy W_j for every shard is ONE phase whose output columns fall into N segments
    // in the order of arrival of the shards (own shard first).
    RtpPhase& ph = P.phases[np++];
    init_phase(ph);
    RtpSegTable& st = P.segtab[1];
    ph.a_map = 2; ph.a_mn = 0;
    ph.b_map = 3; ph.b_mn = 1;
    ph.M = op.M; ph.N = op.in_features; ph.K = Os;
    ph.bn = pick_bn(op.M, Ks, R.ctas);
    ph.ldd = op.lddx; ph.d = op.dx;
    ph.tseg = 1; ph.tseg_len = Ks; ph.tseg_n = N; ph.tseg_tab = 1;
    for (int q = 0; q < N; ++q) {
      const int s = (q == 0) ? N - 1 : q - 1;
      const int j = mod(r - 1 - s, N);
      const bool last = s == N - 1;   // own shard
      st.map[q] = last ? 3 : 4 + s;
      st.off_mn[q] = 0;
      st.d[q] = reinterpret_cast<__nv_bfloat16*>(op.dx) + (long long)j * Ks;
      st.bias[q] = nullptr;
      if (!last) {
        ph.wait_ctr[q] = RTP_CTR_W0 + wb + s; ph.wait_rel[q] = 0;
        ph.done_ctr[q] = RTP_CTR_W0 + wb + s;
        P.uses_inc[RTP_CTR_W0 + wb + s] = 1;
      }
    }
    set_vec_ok(ph);
  } else {
  for (int q = 0; q < N && op.dx; ++q) {
    const int s = (q == 0) ? N - 1 : q - 1;
    const int j = mod(r - 1 - s, N);
    const bool last = s == N - 1;   // own shard
    const bool first_emitted = q == 0, final_emitted = q == N - 1;
    // ---- dgrad: column: dx += dy_j W_j ; row: dx_j = dy W_j
    {
      RtpPhase& ph = P.phases[np++];
      init_phase(ph);
      ph.a_map = 2; ph.a_mn = 0;
      ph.b_map = last ? 3 : 4 + s; ph.b_mn = 1;
      ph.M = op.M; ph.N = Ks; ph.K = Os;
      if (col) ph.a_off_k = j * Os;
      ph.bn = pick_bn(ph.M, ph.N, R.ctas);
      ph.ldd = op.lddx;
      ph.d = reinterpret_cast<__nv_bfloat16*>(op.dx) + (col ? 0 : (long long)j * Ks);
      if (col && (!first_emitted || op.dx_accumulate)) { ph.c = op.dx; ph.ldc = op.lddx; }
      if (!col && op.dx_accumulate) { ph.c = ph.d; ph.ldc = op.lddx; }
      if (op.mask && (!col || final_emitted)) {
        ph.mask = reinterpret_cast<const __nv_bfloat16*>(op.mask) + (col ? 0 : (long long)j * Ks);
        ph.ldmask = op.ldmask; ph.mask_scale = op.mask_scale;
      }
      if (!last) {
        ph.wait_ctr[0] = RTP_CTR_W0 + wb + s; ph.wait_rel[0] = 0;
        ph.done_ctr[0] = RTP_CTR_W0 + wb + s;
        P.uses_inc[RTP_CTR_W0 + wb + s] = 1;
      }
      set_vec_ok(ph);
    }
  }
  }
  // ---- owner-side sum of the N gradient slots (slot s was written by rank r+1+s; slot N-1 by this rank)
  if (N > 1) {
    RtpPhase& ph = P.phases[np++];
    init_phase(ph);
    ph.kind = RTP_KIND_REDUCE;
    ph.M = ph.N = ph.K = 0;
    ph.d = op.grad_home;
    ph.r_nsrc = N;
    ph.r_n = (long long)(op.shard_bytes / 2) & ~7ll;
    for (int s = 0; s < N; ++s) {
      ph.r_src[s] = ws_gslot(ws, R.slot_bytes, s, R.world);
      ph.wait_ctr[s] = RTP_CTR_G0 + s; ph.wait_rel[s] = 0;
      ph.done_ctr[s] = RTP_CTR_G0 + s;
      P.uses_inc[RTP_CTR_G0 + s] = 1;
    }
  }
  P.n_phases = np;
  // weight pushes: the owner q sends its home shard to rank q+1+s, which uses it at its step s (weight slot s)
  P.n_pushes = (op.dx && !op.no_self_push) ? N - 1 : 0;
  for (int s = 0; s + 1 < N && op.dx && !op.no_self_push; ++s) {
    RtpPush& pu = P.pushes[s];
    memset(&pu, 0, sizeof(pu));
    const int t = mod(r + 1 + s, N);
    pu.src = op.home;
    pu.dst = ws_wslot(R.ws[t], R.slot_bytes, wb + s, R.world);
    pu.bytes = op.shard_bytes;
    pu.credit_ptr = &ws_flags(R.ws[R.rank])->credit[t][RTP_CTR_W0 + wb + s].v;
    pu.credit_ctr = RTP_CTR_W0 + wb + s;
    pu.credit_rel = 0;
    pu.arrive_ptr = &ws_flags(R.ws[t])->arrive[RTP_CTR_W0 + wb + s].v;
  }
  return add_prefetch_pushes(R, P, op.next_home, op.next_bytes, 1 - op.bank, op.next_kind);
}

int build_expert_fwd(const RtpRing& R, const RtpExpertFwd& op, RtpProgram& P) {
  init_program(P);
  const int N = R.world, r = R.rank, L = op.n_local;
  if (N < 1 || N > RTP_MAX_WORLD || L < 1) return fail("world size out of range");
  if (N * L > RTP_MAX_PHASES || 1 + N * L > RTP_MAX_MAPS) return fail("too many experts for one launch");
  if (N > 1 && op.shard_bytes > R.slot_bytes) return fail("shard larger than workspace slot");
  if (op.shard_bytes % 16) return fail("shard_bytes must be a multiple of 16");
  void* ws = R.ws[r];
  P.flags = ws ? ws_flags(ws) : nullptr;
  set_peers(R, P);
  P.status = ws ? &ws_flags(ws)->status.v : nullptr;
  P.timeout_ns = R.timeout_ns ? R.timeout_ns : 2000000000ull;
  const long long rows = (long long)N * L * op.cap;
  if (make_map_k(&P.maps[0], op.x, rows, op.in_features, op.ldx)) return -1;
  const int bn = pick_bn(op.cap, op.out_features, R.ctas);
  const int b_box = pair_mode() ? bn / 2 : 128;
  int np = 0;
  for (int i = 0; i < N; ++i) {
    const int j = mod(r + i, N);
    const uint8_t* src = (i == 0) ? reinterpret_cast<const uint8_t*>(op.home) : ws_wslot(ws, R.slot_bytes, i - 1, R.world);
    for (int e = 0; e < L; ++e) {
      const int g = j * L + e;
      const __nv_bfloat16* w = reinterpret_cast<const __nv_bfloat16*>(src) + (long long)e * op.expert_stride;
      const int mi = 1 + i * L + e;
      if (make_map_k(&P.maps[mi], w, op.out_features, op.in_features, op.in_features, b_box)) return -1;
      RtpPhase& ph = P.phases[np++];
      init_phase(ph);
      ph.a_map = 0; ph.b_map = mi;
      ph.a_off_mn = g * op.cap;
      ph.M = op.cap; ph.N = op.out_features; ph.K = op.in_features;
      ph.bn = bn; ph.b_box = b_box;
      ph.d = reinterpret_cast<__nv_bfloat16*>(op.y) + (long long)g * op.cap * op.ldy;
      ph.ldd = op.ldy;
      if (op.bias_off >= 0) ph.bias = w + op.bias_off;
      ph.act = op.act;
      if (i > 0) {
        ph.wait_ctr[0] = RTP_CTR_W0 + (i - 1); ph.wait_rel[0] = 0;
        if (e == L - 1) ph.done_ctr[0] = RTP_CTR_W0 + (i - 1);
      }
      set_vec_ok(ph);
    }
  }
  P.n_phases = np;
  P.n_pushes = N - 1;
  for (int i = 0; i + 1 < N; ++i) {
    RtpPush& pu = P.pushes[i];
    memset(&pu, 0, sizeof(pu));
    const int t = mod(r - (i + 1), N);
    pu.src = op.home;
    pu.dst = ws_wslot(R.ws[t], R.slot_bytes, i, R.world);
    pu.bytes = op.shard_bytes;
    pu.credit_ptr = &ws_flags(R.ws[R.rank])->credit[t][RTP_CTR_W0 + i].v;
    pu.credit_ctr = RTP_CTR_W0 + i;
    pu.credit_rel = 0;
    pu.arrive_ptr = &ws_flags(R.ws[t])->arrive[RTP_CTR_W0 + i].v;
    P.uses_inc[RTP_CTR_W0 + i] = 1;
  }
  return 0;
}

int build_expert_bwd(const RtpRing& R, const RtpExpertBwd& op, RtpProgram& P) {
  init_program(P);
  const int N = R.world, r = R.rank, L = op.n_local;
  if (N < 1 || N > RTP_MAX_WORLD || L < 1) return fail("world size out of range");
  if (2 * N * L + 1 > RTP_MAX_PHASES || 3 + N * L > RTP_MAX_MAPS) return fail("too many experts for one launch");
  if (N > 1 && op.shard_bytes > R.slot_bytes) return fail("shard larger than workspace slot");
  void* ws = R.ws[r];
  P.flags = ws ? ws_flags(ws) : nullptr;
  set_peers(R, P);
  P.status = ws ? &ws_flags(ws)->status.v : nullptr;
  P.timeout_ns = R.timeout_ns ? R.timeout_ns : 2000000000ull;
  const long long rows = (long long)N * L * op.cap;
  // maps: 0 = dy (tokens are k), 1 = x (tokens are k), 2 = dy (out is k), 3.. = expert weights (home / slots)
  if (make_map_mn(&P.maps[0], op.dy, op.out_features, rows, op.ldy)) return -1;
  if (make_map_mn(&P.maps[1], op.x, op.in_features, rows, op.ldx)) return -1;
  if (op.dx && make_map_k(&P.maps[2], op.dy, rows, op.out_features, op.ldy)) return -1;
  int np = 0;
  for (int s = 0; s < N; ++s) {
    const int j = mod(r - 1 - s, N);
    const bool last = s == N - 1;
    const uint8_t* wsrc = last ? reinterpret_cast<const uint8_t*>(op.home) : ws_wslot(ws, R.slot_bytes, s, R.world);
    uint8_t* gdst = (N == 1) ? reinterpret_cast<uint8_t*>(op.grad_home) : ws_gslot(R.ws[j], R.slot_bytes, s, R.world);
    for (int e = 0; e < L; ++e) {
      const int g = j * L + e;
      {  // wgrad of expert g
        RtpPhase& ph = P.phases[np++];
        init_phase(ph);
        ph.a_map = 0; ph.a_mn = 1; ph.a_off_k = g * op.cap;
        ph.b_map = 1; ph.b_mn = 1; ph.b_off_k = g * op.cap;
        ph.M = op.out_features; ph.N = op.in_features; ph.K = op.cap;
        ph.bn = pick_bn(ph.M, ph.N, R.ctas);
        __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(gdst) + (long long)e * op.expert_stride;
        ph.d = d; ph.ldd = op.in_features;
        if (N > 1) {
          ph.credit_ptr = &ws_flags(R.ws[R.rank])->credit[j][RTP_CTR_G0 + s].v;
          ph.credit_ctr = RTP_CTR_G0 + s; ph.credit_rel = 0;
          if (e == L - 1) ph.arrive_ptr = &ws_flags(R.ws[j])->arrive[RTP_CTR_G0 + s].v;
        }
        if (op.bias_off >= 0 && op.dbias_full) {
          ph.vec_out = d + op.bias_off;
          ph.vec_add = op.dbias_full + (long long)g * op.out_features;
          ph.vec_len = op.out_features;
        }
        set_vec_ok(ph);
      }
      if (op.dx) {  // dgrad of expert g
        const int mi = 3 + s * L + e;
        const __nv_bfloat16* w = reinterpret_cast<const __nv_bfloat16*>(wsrc) + (long long)e * op.expert_stride;
        if (make_map_mn(&P.maps[mi], w, op.in_features, op.out_features, op.in_features)) return -1;
        RtpPhase& ph = P.phases[np++];
        init_phase(ph);
        ph.a_map = 2; ph.a_off_mn = g * op.cap;
        ph.b_map = mi; ph.b_mn = 1;
        ph.M = op.cap; ph.N = op.in_features; ph.K = op.out_features;
        ph.bn = pick_bn(ph.M, ph.N, R.ctas);
        ph.d = reinterpret_cast<__nv_bfloat16*>(op.dx) + (long long)g * op.cap * op.lddx;
        ph.ldd = op.lddx;
        if (op.mask) {
          ph.mask = reinterpret_cast<const __nv_bfloat16*>(op.mask) + (long long)g * op.cap * op.ldmask;
          ph.ldmask = op.ldmask; ph.mask_scale = op.mask_scale;
        }
        if (!last) {
          ph.wait_ctr[0] = RTP_CTR_W0 + s; ph.wait_rel[0] = 0;
          if (e == L - 1) ph.done_ctr[0] = RTP_CTR_W0 + s;
        }
        set_vec_ok(ph);
      }
    }
  }
  if (N > 1) {
    RtpPhase& ph = P.phases[np++];
    init_phase(ph);
    ph.kind = RTP_KIND_REDUCE;
    ph.M = ph.N = ph.K = 0;
    ph.d = op.grad_home;
    ph.r_nsrc = N;
    ph.r_n = (long long)(op.shard_bytes / 2) & ~7ll;
    for (int s = 0; s < N; ++s) {
      ph.r_src[s] = ws_gslot(ws, R.slot_bytes, s, R.world);
      ph.wait_ctr[s] = RTP_CTR_G0 + s; ph.wait_rel[s] = 0;
      ph.done_ctr[s] = RTP_CTR_G0 + s;
      P.uses_inc[RTP_CTR_G0 + s] = 1;
    }
  }
  P.n_phases = np;
  P.n_pushes = op.dx ? N - 1 : 0;
  for (int s = 0; s + 1 < N && op.dx; ++s) {
    RtpPush& pu = P.pushes[s];
    memset(&pu, 0, sizeof(pu));
    const int t = mod(r + 1 + s, N);
    pu.src = op.home;
    pu.dst = ws_wslot(R.ws[t], R.slot_bytes, s, R.world);
    pu.bytes = op.shard_bytes;
    pu.credit_ptr = &ws_flags(R.ws[R.rank])->credit[t][RTP_CTR_W0 + s].v;
    pu.credit_ctr = RTP_CTR_W0 + s;
    pu.credit_rel = 0;
    pu.arrive_ptr = &ws_flags(R.ws[t])->arrive[RTP_CTR_W0 + s].v;
    P.uses_inc[RTP_CTR_W0 + s] = 1;
  }
  return 0;
}

int build_embed_fwd(const RtpRing& R, const RtpEmbedFwd& op, RtpProgram& P) {
  init_program(P);
  const int N = R.world, r = R.rank;
  if (N < 1 || N > RTP_MAX_WORLD) return fail("world size out of range");
  if (op.Ds % 8 || op.Ds * N != op.D) return fail("embedding: D must be N * Ds with Ds a multiple of 8");
  if (N > 1 && op.shard_bytes > R.slot_bytes) return fail("shard larger than workspace slot");
  if (op.shard_bytes % 16) return fail("shard_bytes must be a multiple of 16");
  void* ws = R.ws[r];
  P.flags = ws ? ws_flags(ws) : nullptr;
  set_peers(R, P);
  P.status = ws ? &ws_flags(ws)->status.v : nullptr;
  P.timeout_ns = R.timeout_ns ? R.timeout_ns : 2000000000ull;
  P.n_phases = N;
  for (int i = 0; i < N; ++i) {
    RtpPhase& ph = P.phases[i];
    init_phase(ph);
    const int j = mod(r + i, N);
    const int slot = i - 1;
    ph.kind = RTP_KIND_GATHER;
    ph.M = ph.N = ph.K = 0;
    ph.g_table = (i == 0) ? op.home : ws_wslot(ws, R.slot_bytes, slot, R.world);
    ph.g_ids = op.ids;
    ph.g_tokens = op.T; ph.g_cols = op.Ds; ph.g_dim = op.D; ph.g_col_off = j * op.Ds; ph.g_tpp = op.tokens_per_pos;
    ph.g_scale = op.scale; ph.g_pe = op.pe; ph.g_ldpe = op.ld_pe;
    ph.d = reinterpret_cast<__nv_bfloat16*>(op.out) + (long long)j * op.Ds;
    ph.ldd = op.ld_out;
    ph.drop_thresh = drop_threshold(op.drop_p);
    ph.drop_scale = op.drop_p > 0.f ? 1.f / (1.f - op.drop_p) : 1.f;
    ph.drop_seed = op.seed; ph.drop_offset = op.offset; ph.drop_step_ptr = op.step_ptr;
    if (i > 0) {
      ph.wait_ctr[0] = RTP_CTR_W0 + slot;
      ph.wait_rel[0] = 0;
      ph.done_ctr[0] = RTP_CTR_W0 + slot;
    }
  }
  P.n_pushes = N - 1;
  for (int i = 0; i + 1 < N; ++i) {
    RtpPush& pu = P.pushes[i];
    memset(&pu, 0, sizeof(pu));
    const int t = mod(r - (i + 1), N);
    const int slot = i;
    pu.src = op.home;
    pu.dst = ws_wslot(R.ws[t], R.slot_bytes, slot, R.world);
    pu.bytes = op.shard_bytes;
    pu.credit_ptr = &ws_flags(R.ws[R.rank])->credit[t][RTP_CTR_W0 + slot].v;
    pu.credit_ctr = RTP_CTR_W0 + slot;
    pu.credit_rel = 0;
    pu.arrive_ptr = &ws_flags(R.ws[t])->arrive[RTP_CTR_W0 + slot].v;
    P.uses_inc[RTP_CTR_W0 + slot] = 1;
  }
  return 0;
}

int build_reduce_scatter(const RtpRing& R, const RtpReduceScatter& op, RtpProgram& P) {
  init_program(P);
  const int N = R.world, r = R.rank;
  if (N < 1 || N > RTP_MAX_WORLD) return fail("world size out of range");
  if (op.cols % 8 || op.ld % 8) return fail("reduce_scatter: cols and ld must be multiples of 8");
  if (N > 1 && (unsigned long long)op.rows * op.cols * 2 > R.slot_bytes) return fail("block larger than workspace slot");
  void* ws = R.ws[r];
  P.flags = ws ? ws_flags(ws) : nullptr;
  set_peers(R, P);
  P.status = ws ? &ws_flags(ws)->status.v : nullptr;
  P.timeout_ns = R.timeout_ns ? R.timeout_ns : 2000000000ull;
  const int up = mod(r + 1, N);
  P.n_phases = N;
  for (int s = 0; s < N; ++s) {
    RtpPhase& ph = P.phases[s];
    init_phase(ph);
    const int j = mod(r - 1 - s, N);
    const int gin = (s - 1) & 1, gout = s & 1;
    const bool last = s == N - 1;
    ph.kind = RTP_KIND_VECADD;
    ph.M = ph.N = ph.K = 0;
    ph.v_src = reinterpret_cast<const __nv_bfloat16*>(op.src) + (long long)j * op.cols;
    ph.v_ld = op.ld; ph.v_rows = op.rows; ph.v_cols = op.cols;
    ph.d = last ? op.out : (void*)ws_gslot(R.ws[up], R.slot_bytes, gout, R.world);
    if (s > 0) {
      ph.c = ws_gslot(ws, R.slot_bytes, gin, R.world);
      ph.wait_ctr[0] = RTP_CTR_G0 + gin; ph.wait_rel[0] = (s - 1) / 2;
      ph.done_ctr[0] = RTP_CTR_G0 + gin;
    }
    if (!last) {
      ph.credit_ptr = &ws_flags(R.ws[R.rank])->credit[up][RTP_CTR_G0 + gout].v;
      ph.credit_ctr = RTP_CTR_G0 + gout; ph.credit_rel = s / 2;
      ph.arrive_ptr = &ws_flags(R.ws[up])->arrive[RTP_CTR_G0 + gout].v;
    }
  }
  P.uses_inc[RTP_CTR_G0] = N / 2;
  P.uses_inc[RTP_CTR_G0 + 1] = (N - 1) / 2;
  return 0;
}

// Reduce-scatter of N contiguous blocks as ONE hop: rank r pushes block j (j != r) of its block-major buffer straight
// into a gradient slot of owner j (bulk copies over NVLink, all peers at once), and sums the N-1 blocks it receives with
// its own block r.  Slot s of an owner is written by rank owner + 1 + s, the same convention as the weight gradients.
int build_reduce_blocks(const RtpRing& R, const RtpReduceBlocks& op, RtpProgram& P) {
  init_program(P);
  const int N = R.world, r = R.rank;
  if (N < 1 || N > RTP_MAX_WORLD) return fail("world size out of range");
  if (op.block_elems % 8) return fail("reduce_blocks: block_elems must be a multiple of 8");
  const unsigned long long bytes = (unsigned long long)op.block_elems * 2;
  if (N > 1 && bytes > R.slot_bytes) return fail("block larger than workspace slot");
  void* ws = R.ws[r];
  P.flags = ws ? ws_flags(ws) : nullptr;
  set_peers(R, P);
  P.status = ws ? &ws_flags(ws)->status.v : nullptr;
  P.timeout_ns = R.timeout_ns ? R.timeout_ns : 2000000000ull;
  const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(op.src);
  RtpPhase& ph = P.phases[0];
  init_phase(ph);
  ph.kind = RTP_KIND_REDUCE;
  ph.M = ph.N = ph.K = 0;
  ph.d = op.out;
  ph.r_nsrc = N;
  ph.r_n = op.block_elems;
  for (int s = 0; s + 1 < N; ++s) {
    ph.r_src[s] = ws_gslot(ws, R.slot_bytes, s, R.world);
    ph.wait_ctr[s] = RTP_CTR_G0 + s; ph.wait_rel[s] = 0;
    ph.done_ctr[s] = RTP_CTR_G0 + s;
    P.uses_inc[RTP_CTR_G0 + s] = 1;
  }
  ph.r_src[N - 1] = src + (long long)r * op.block_elems;      // own block: read in place
  P.n_phases = 1;
  P.n_pushes = N - 1;
  for (int s = 0; s + 1 < N; ++s) {
    RtpPush& pu = P.pushes[s];
    memset(&pu, 0, sizeof(pu));
    const int j = mod(r - 1 - s, N);                           // owner that receives my block j in its slot s
    pu.src = src + (long long)j * op.block_elems;
    pu.dst = ws_gslot(R.ws[j], R.slot_bytes, s, R.world);
    pu.bytes = bytes;
    pu.credit_ptr = &ws_flags(R.ws[R.rank])->credit[j][RTP_CTR_G0 + s].v;
    pu.credit_ctr = RTP_CTR_G0 + s;
    pu.credit_rel = 0;
    pu.arrive_ptr = &ws_flags(R.ws[j])->arrive[RTP_CTR_G0 + s].v;
  }
  return 0;
}

template <int NEMU, class Op, class Builder>
int run_emu(const RtpRing* rings, const Op* ops, Builder build, cudaStream_t stream) {
  decide_pair(0, 0, 0, false);   // emulated ranks share one cooperative launch without clusters
  static RtpProgram progs[RTP_MAX_EMU_RANKS];
  static rtp::GemmParams<NEMU> params;
  for (int e = 0; e < NEMU; ++e) {
    if (build(rings[e], ops[e], progs[e])) return -1;
    finalize_program(progs[e], rings[0].ctas, false);
  }
  cudaError_t err = cudaMemcpyToSymbolAsync(rtp::c_emu_progs, progs, sizeof(RtpProgram) * NEMU, 0,
                                            cudaMemcpyHostToDevice, stream);
  if (err != cudaSuccess) return fail(std::string("copy of emulated programs: ") + cudaGetErrorString(err));
  // the host array is reused by the next call: wait until the copy has read it
  err = cudaStreamSynchronize(stream);
  if (err != cudaSuccess) return fail(std::string("stream sync: ") + cudaGetErrorString(err));
  params.ctas_per_rank = rings[0].ctas;
  return launch<NEMU>(params, rings[0].ctas * NEMU, true, stream);
}


// ------------------------------------------------------------------------------------------------
// Program lint: builds the programs of ALL ranks of a ring on the host (no GPU needed: tensor maps are recorded by a
// stand-in encoder, workspaces and operands are made-up addresses) and checks what the kernel relies on:
//   * every tiled copy starts on a 16-byte boundary of its innermost coordinate and inside its tensor;
//   * tile segments divide the output evenly and no two tiles of non-accumulating phases write the same bytes;
//   * the cross-rank protocol is consistent: every arrival counter a rank waits on has exactly ONE producer on the
//     ring (a push job or a phase / segment that announces its output), that producer waits for the matching credit in
//     its own flag block and writes inside the slot the counter belongs to, the consumer reports the slot `done`, and
//     the per-slot fill counts advance identically on every rank.
// The tile arithmetic mirrors rtp_gemm_kernel's producer and epilogue.
// ------------------------------------------------------------------------------------------------
struct Lint {
  std::string rep;
  int problems = 0;
  void bad(const std::string& s) {
    ++problems;
    if (rep.size() < 6000) rep += s + "\n";
  }
};
std::string lstr(long long v) { return std::to_string(v); }

const rtp::HostTensorMap* host_map(const CUtensorMap* m) {
  const rtp::HostTensorMap* h = reinterpret_cast<const rtp::HostTensorMap*>(m);
  return h->magic == rtp::kHostMapMagic ? h : nullptr;
}

// one tiled copy of operand `which` ('A' / 'B') of phase p: coordinate (mn, k) in elements
// (`may_be_outside`: the second CTA of a pair may start past a ragged edge; such a copy reads the fill value)
void lint_copy(Lint& L, int rank, int p, char which, const RtpProgram& P, int map, bool mn_major, long long mn, long long k,
               bool may_be_outside) {
  const rtp::HostTensorMap* h = host_map(&P.maps[map]);
  const std::string at = "rank " + lstr(rank) + " phase " + lstr(p) + " operand " + which + " (map " + lstr(map) + "): ";
  if (!h) { L.bad(at + "tensor map was never encoded"); return; }
  if (mn < 0 || k < 0) { L.bad(at + "negative coordinate (" + lstr(mn) + ", " + lstr(k) + ")"); return; }
  if (P.map3d[map]) {
    if (mn % 64) L.bad(at + "3-D map needs the mn coordinate to be a multiple of 64, got " + lstr(mn));
    if (!may_be_outside && ((unsigned long long)(mn / 64) >= h->dims[2] || (unsigned long long)k >= h->dims[1]))
      L.bad(at + "copy starts outside the tensor: (mn " + lstr(mn) + ", k " + lstr(k) + ")");
  } else {
    const long long x = mn_major ? mn : k, y = mn_major ? k : mn;
    if (x % 8) L.bad(at + "innermost coordinate " + lstr(x) + " is not a multiple of 8 elements (16 bytes)");
    if (!may_be_outside && ((unsigned long long)x >= h->dims[0] || (unsigned long long)y >= h->dims[1]))
      L.bad(at + "copy starts outside the tensor: (x " + lstr(x) + ", y " + lstr(y) + ")");
  }
}

struct LintRect {
  unsigned long long base;   // address of the tile's first element
  long long rows, cols, pitch;   // cols and pitch in bytes
  int rank, phase;
};
bool rects_overlap(const LintRect& a, const LintRect& b) {
  if (a.pitch != b.pitch) {
    const unsigned long long a1 = a.base + (a.rows - 1) * a.pitch + a.cols, b1 = b.base + (b.rows - 1) * b.pitch + b.cols;
    return a.base < b1 && b.base < a1;   // cannot decompose: report any intersection of the spans
  }
  const long long P = a.pitch;
  long long d = (long long)(b.base - a.base);
  long long q = d >= 0 ? d / P : -((-d + P - 1) / P);
  const long long rem = d - q * P;   // 0 <= rem < P
  auto rows_meet = [&](long long off) {   // row i of a meets row j of b with i = j + off
    const long long lo = off < 0 ? -off : 0, hi = std::min(b.rows - 1, a.rows - 1 - off);
    return lo <= hi;
  };
  if (rem < a.cols && rows_meet(q)) return true;
  if (rem - P + b.cols > 0 && rows_meet(q + 1)) return true;
  return false;
}

void lint_program(Lint& L, const RtpRing& R, int rank, const RtpProgram& P, bool pair, std::vector<LintRect>& rects) {
  const int TM = pair ? 256 : 128;
  for (int p = 0; p < P.n_phases; ++p) {
    const RtpPhase& ph = P.phases[p];
    if (ph.kind != RTP_KIND_GEMM) continue;
    const std::string at = "rank " + lstr(rank) + " phase " + lstr(p) + ": ";
    if (ph.bn != 128 && ph.bn != 256) L.bad(at + "tile width " + lstr(ph.bn));
    if (ph.batch != 1) continue;   // batched windows (attention) are not part of the rotation programs
    const RtpSegTable& st = P.segtab[ph.tseg_tab];
    if (ph.tseg) {
      const int unit = ph.tseg == 1 ? ph.bn : TM;
      if (ph.tseg_len % unit) L.bad(at + "segment length " + lstr(ph.tseg_len) + " is not a multiple of the tile (" + lstr(unit) + ")");
      if ((long long)ph.tseg_n * ph.tseg_len != (ph.tseg == 1 ? ph.N : ph.M)) L.bad(at + "segments do not add up to the phase's extent");
      if (ph.tseg_n < 1 || ph.tseg_n > RTP_MAX_WAITS) L.bad(at + "segment count " + lstr(ph.tseg_n));
    }
    const int tiles_m = (ph.M + TM - 1) / TM, tiles_n = (ph.N + ph.bn - 1) / ph.bn;
    const int nseg = ph.nseg > 1 ? ph.nseg : 1;
    for (int tn = 0; tn < tiles_n; ++tn)
      for (int tm = 0; tm < tiles_m; ++tm)
        for (int half = 0; half < (pair ? 2 : 1); ++half) {
          int m0u = tm * TM, n0 = tn * ph.bn;
          const int bn_local = pair ? ph.bn / 2 : ph.bn;
          long long a_mn = m0u + half * 128 + ph.a_off_mn, b_mn = n0 + half * bn_local + ph.b_off_mn;
          int a_map = ph.a_map, b_map = ph.b_map;
          int sg = 0;
          long long e_M = ph.M, e_N = ph.N;
          unsigned long long d = reinterpret_cast<unsigned long long>(ph.d);
          if (ph.tseg) {
            sg = (ph.tseg == 1 ? n0 : m0u) / ph.tseg_len;
            if (sg >= ph.tseg_n) { L.bad(at + "tile outside the segments"); continue; }
            if (ph.tseg == 1) {
              b_mn += st.off_mn[sg] - (long long)sg * ph.tseg_len;
              if (st.map[sg] >= 0) b_map = st.map[sg];
              n0 -= sg * ph.tseg_len; e_N = ph.tseg_len;
            } else {
              a_mn += st.off_mn[sg] - (long long)sg * ph.tseg_len;
              if (st.map[sg] >= 0) a_map = st.map[sg];
              m0u -= sg * ph.tseg_len; e_M = ph.tseg_len;
            }
            d = reinterpret_cast<unsigned long long>(st.d[sg]);
            if (!st.d[sg]) L.bad(at + "segment " + lstr(sg) + " has no destination");
          }
          for (int s = 0; s < nseg; ++s) {
            const long long a_k = ph.a_off_k + (nseg > 1 ? ph.seg_a_off_k[s] : 0);
            lint_copy(L, rank, p, 'A', P, a_map, ph.a_mn != 0, a_mn, a_k, half == 1);
            lint_copy(L, rank, p, 'B', P, nseg > 1 ? ph.seg_b_map[s] : b_map, ph.b_mn != 0, b_mn, ph.b_off_k, half == 1);
          }
          {
            const long long m0 = m0u + half * 128;
            if (m0 >= e_M) continue;
            const int elt = ph.d_fp32 ? 4 : 2;
            LintRect r;
            r.base = d + ((unsigned long long)m0 * ph.ldd + n0) * elt;
            r.rows = std::min<long long>(128, e_M - m0);
            r.cols = std::min<long long>(ph.bn, e_N - n0) * elt;
            r.pitch = ph.ldd * elt;
            r.rank = rank; r.phase = p;
            if (!ph.c) rects.push_back(r);
          }
        }
  }
  (void)R;
}

// which (rank, counter) does an arrival pointer belong to?
bool find_arrive(const RtpRing& R, const unsigned long long* ptr, int* t_out, int* c_out) {
  for (int t = 0; t < R.world; ++t)
    for (int c = 0; c < RTP_NUM_CTR; ++c)
      if (ptr == &ws_flags(R.ws[t])->arrive[c].v) { *t_out = t; *c_out = c; return true; }
  return false;
}
void slot_range(const RtpRing& R, int t, int c, unsigned long long* lo, unsigned long long* hi) {
  uint8_t* base = c < RTP_CTR_G0 ? ws_wslot(R.ws[t], R.slot_bytes, c - RTP_CTR_W0, R.world)
                                 : ws_gslot(R.ws[t], R.slot_bytes, c - RTP_CTR_G0, R.world);
  *lo = reinterpret_cast<unsigned long long>(base);
  *hi = *lo + R.slot_bytes;
}

struct LintProducer { int rank; int t, c; const unsigned long long* credit_ptr; int credit_ctr; unsigned long long lo, hi; std::string what; };

void lint_ring(Lint& L, const std::vector<RtpRing>& rings, const std::vector<RtpProgram>& progs) {
  const int N = (int)rings.size();
  std::vector<LintProducer> prods;
  for (int r = 0; r < N; ++r) {
    const RtpProgram& P = progs[r];
    for (int j = 0; j < P.n_pushes; ++j) {
      const RtpPush& pu = P.pushes[j];
      LintProducer pr{r, -1, -1, pu.credit_ptr, pu.credit_ctr, reinterpret_cast<unsigned long long>(pu.dst),
                      reinterpret_cast<unsigned long long>(pu.dst) + pu.bytes, "push " + lstr(j)};
      if (!pu.arrive_ptr || !find_arrive(rings[r], pu.arrive_ptr, &pr.t, &pr.c))
        L.bad("rank " + lstr(r) + " push " + lstr(j) + ": arrival pointer is not an arrival counter of the ring");
      else prods.push_back(pr);
    }
    for (int p = 0; p < P.n_phases; ++p) {
      const RtpPhase& ph = P.phases[p];
      if (!ph.arrive_ptr) continue;
      if (ph.tseg) {
        const RtpSegTable& st = P.segtab[ph.tseg_tab];
        for (int i = 0; i < ph.tseg_n; ++i) {
          if (!st.arrive_ptr[i]) continue;
          const unsigned long long d = reinterpret_cast<unsigned long long>(st.d[i]);
          const long long rows = ph.tseg == 2 ? ph.tseg_len : ph.M, cols = ph.tseg == 1 ? ph.tseg_len : ph.N;
          LintProducer pr{r, -1, -1, st.credit_ptr[i], st.credit_ctr[i], d, d + ((rows - 1) * ph.ldd + cols) * 2,
                          "phase " + lstr(p) + " segment " + lstr(i)};
          if (!find_arrive(rings[r], st.arrive_ptr[i], &pr.t, &pr.c))
            L.bad("rank " + lstr(r) + " " + pr.what + ": arrival pointer is not an arrival counter of the ring");
          else prods.push_back(pr);
        }
      } else {
        const unsigned long long d = reinterpret_cast<unsigned long long>(ph.d);
        LintProducer pr{r, -1, -1, ph.credit_ptr, ph.credit_ctr, d, d + (((long long)ph.M - 1) * ph.ldd + ph.N) * (ph.d_fp32 ? 4 : 2),
                        "phase " + lstr(p)};
        if (ph.kind != RTP_KIND_GEMM) { pr.lo = pr.hi = 0; }
        if (!find_arrive(rings[r], ph.arrive_ptr, &pr.t, &pr.c))
          L.bad("rank " + lstr(r) + " phase " + lstr(p) + ": arrival pointer is not an arrival counter of the ring");
        else prods.push_back(pr);
      }
    }
  }
  // consumers
  for (int t = 0; t < N; ++t) {
    const RtpProgram& P = progs[t];
    bool waits[RTP_NUM_CTR] = {false}, dones[RTP_NUM_CTR] = {false};
    for (int p = 0; p < P.n_phases; ++p)
      for (int w = 0; w < RTP_MAX_WAITS; ++w) {
        if (P.phases[p].wait_ctr[w] >= 0) waits[P.phases[p].wait_ctr[w]] = true;
        if (P.phases[p].done_ctr[w] >= 0) dones[P.phases[p].done_ctr[w]] = true;
      }
    for (int c = 0; c < RTP_NUM_CTR; ++c) {
      int n = 0;
      for (const LintProducer& pr : prods) n += (pr.t == t && pr.c == c);
      const std::string at = "rank " + lstr(t) + " counter " + lstr(c) + ": ";
      if (waits[c] && n != 1) L.bad(at + "waited on, but " + lstr(n) + " producers announce it (must be exactly one)");
      if (!waits[c] && n > 0) L.bad(at + lstr(n) + " producer(s) announce it, nobody waits");
      if (waits[c] && !dones[c]) L.bad(at + "waited on but never reported done (its credit would never return)");
      if (waits[c] != (P.uses_inc[c] != 0)) L.bad(at + "fill count and waits disagree (uses_inc " + lstr(P.uses_inc[c]) + ")");
      if (P.uses_inc[c] != progs[0].uses_inc[c]) L.bad(at + "fill count advances differently from rank 0");
    }
  }
  for (const LintProducer& pr : prods) {
    const std::string at = "rank " + lstr(pr.rank) + " " + pr.what + " -> rank " + lstr(pr.t) + " counter " + lstr(pr.c) + ": ";
    if (pr.credit_ptr != &ws_flags(rings[pr.rank].ws[pr.rank])->credit[pr.t][pr.c].v || pr.credit_ctr != pr.c)
      L.bad(at + "does not wait for the matching credit in its own flag block");
    unsigned long long lo, hi;
    slot_range(rings[pr.rank], pr.t, pr.c, &lo, &hi);
    if (pr.hi > pr.lo && (pr.lo < lo || pr.hi > hi)) L.bad(at + "writes outside the slot the counter belongs to");
  }
}

// Self-test of the lint: damages rank 0's program the way a builder bug would.
void lint_inject(RtpProgram& P, int what) {
  if (what == 1 && P.n_pushes >= 2) P.pushes[0].arrive_ptr = P.pushes[1].arrive_ptr;   // two producers for one counter
  if (what == 2) P.phases[0].a_off_k += 4;                                               // a copy off its 16-byte boundary
  if (what == 3 && P.n_pushes >= 1) P.pushes[0].credit_ctr += 1;                          // waits for the wrong credit
  if (what == 4 && P.phases[0].tseg && P.phases[0].tseg_n >= 2)                          // two segments, one destination
    P.segtab[P.phases[0].tseg_tab].d[1] = P.segtab[P.phases[0].tseg_tab].d[0];
  if (what == 5 && P.n_pushes >= 1) P.pushes[0].bytes += 1ull << 33;                      // a push that leaves its slot
}

// made-up addresses: workspaces 64 GB apart, operands of rank r in a region of their own
void* fake_ws(int t) { return reinterpret_cast<void*>((unsigned long long)(t + 1) << 36); }
void* fake_buf(int r, int which) { return reinterpret_cast<void*>(((unsigned long long)(0x100 + r) << 36) + ((unsigned long long)which << 32)); }

void fake_rings(std::vector<RtpRing>& rings, int world, int ctas, unsigned long long slot_bytes) {
  rings.assign(world, RtpRing{});
  for (int r = 0; r < world; ++r) {
    rings[r].rank = r; rings[r].world = world; rings[r].slot_bytes = slot_bytes; rings[r].ctas = ctas;
    for (int t = 0; t < world; ++t) rings[r].ws[t] = fake_ws(t);
  }
}

int lint_finish(Lint& L, std::vector<LintRect>& rects, char* report, int cap) {
  // tiles of non-accumulating phases must not write the same bytes (per rank: other ranks write other memory)
  for (size_t i = 0; i < rects.size() && L.problems < 64; ++i)
    for (size_t j = i + 1; j < rects.size(); ++j)
      if (rects[i].rank == rects[j].rank && rects_overlap(rects[i], rects[j])) {
        L.bad("rank " + lstr(rects[i].rank) + ": a tile of phase " + lstr(rects[i].phase) + " and a tile of phase " +
              lstr(rects[j].phase) + " write the same bytes");
        break;
      }
  if (report && cap > 0) {
    const size_t n = std::min<size_t>(L.rep.size(), (size_t)cap - 1);
    memcpy(report, L.rep.data(), n);
    report[n] = 0;
  }
  return L.problems;
}

}  // namespace

extern "C" {

const char* rtp_last_error(void) { return g_err.c_str(); }
void rtp_debug_force_stages(int n) { g_force_stages = n; }
void rtp_set_push_ctas(int n) { g_push_ctas = n < 0 ? -1 : n; }
void rtp_set_pair_mode(int on) { g_pair = on < 0 ? -1 : (on ? 1 : 0); }
void rtp_debug_set_trace(unsigned long long* device_buffer_1024_words) { g_trace = device_buffer_1024_words; }
int rtp_sm_count(void) { return sm_count(); }

int rtp_gemm(const RtpGemmArgs* a, void* stream) {
  static thread_local rtp::GemmParams<1> params;
  RtpProgram& P = params.prog[0];
  init_program(P);
  if (a->M <= 0 || a->N <= 0 || a->K <= 0) return fail("empty GEMM");
  if (a->a_mn ? make_map_mn3(&P.maps[0], a->a, a->M, a->K, a->lda, 2, &P.map3d[0]) : make_map_k(&P.maps[0], a->a, a->M, a->K, a->lda))
    return -1;
  const int ctas = a->num_ctas > 0 ? a->num_ctas : sm_count();
  decide_pair(a->M, a->N, ctas);
  const int bn_sel = a->bn ? a->bn : pick_bn(a->M, a->N, ctas);
  if (bn_sel != 128 && bn_sel != 256) return fail("bn must be 128 or 256");
  const bool pair = pair_mode();
  const int b_box = pair ? bn_sel / 2 : 128;   // a pair stages half of the B tile per CTA
  if (a->b_mn ? make_map_mn3(&P.maps[1], a->b, a->N, a->K, a->ldb, (pair ? bn_sel / 2 : bn_sel) / 64, &P.map3d[1])
              : make_map_k(&P.maps[1], a->b, a->N, a->K, a->ldb, b_box))
    return -1;
  RtpPhase& ph = P.phases[0];
  init_phase(ph);
  ph.a_map = 0; ph.b_map = 1; ph.a_mn = a->a_mn; ph.b_mn = a->b_mn;
  ph.M = a->M; ph.N = a->N; ph.K = a->K;
  ph.bn = bn_sel;
  ph.b_box = b_box;
  ph.d = a->d; ph.ldd = a->ldd; ph.d_fp32 = a->d_fp32;
  ph.c = a->c; ph.ldc = a->ldc; ph.c_fp32 = a->c_fp32;
  ph.bias = a->bias; ph.act = a->act;
  ph.mask = a->mask; ph.ldmask = a->ldmask; ph.mask_scale = a->mask_scale;
  ph.drop_thresh = drop_threshold(a->drop_p);
  ph.drop_scale = a->drop_p > 0.f ? 1.f / (1.f - a->drop_p) : 1.f;
  ph.drop_seed = a->seed; ph.drop_offset = a->offset; ph.drop_step_ptr = a->step_ptr;
  set_vec_ok(ph);
  P.n_phases = 1;
  P.status = a->status;
  P.trace = g_trace;
  if (!P.status) return fail("status word required");
  params.ctas_per_rank = ctas;
  const int tiles = pair ? 2 * ((a->M + 255) / 256) * ((a->N + ph.bn - 1) / ph.bn)
                         : ((a->M + 127) / 128) * ((a->N + ph.bn - 1) / ph.bn);
  int grid = tiles < ctas ? tiles : ctas;
  if (pair) grid &= ~1;
  params.ctas_per_rank = grid;
  return launch<1>(params, grid, false, (cudaStream_t)stream, pair);
}

int rtp_gemm_batched(const RtpGemmBatched* a, void* stream) {
  static thread_local rtp::GemmParams<1> params;
  RtpProgram& P = params.prog[0];
  init_program(P);
  if (a->M <= 0 || a->N <= 0 || a->K <= 0 || a->batch <= 0 || a->batch_inner <= 0) return fail("empty batched GEMM");
  const int bn = a->bn ? a->bn : (a->N <= 64 ? 64 : (a->N <= 128 ? 128 : 256));
  if (bn != 64 && bn != 128 && bn != 256) return fail("bn must be 64, 128 or 256");
  const int b_box = bn == 64 ? 64 : 128;
  if (a->a_mn ? make_map_mn(&P.maps[0], a->a, a->a_cols, a->a_rows, a->lda)
              : make_map_k(&P.maps[0], a->a, a->a_rows, a->a_cols, a->lda))
    return -1;
  if (a->b_mn ? make_map_mn(&P.maps[1], a->b, a->b_cols, a->b_rows, a->ldb)
              : make_map_k(&P.maps[1], a->b, a->b_rows, a->b_cols, a->ldb, b_box))
    return -1;
  RtpPhase& ph = P.phases[0];
  init_phase(ph);
  ph.a_map = 0; ph.b_map = 1; ph.a_mn = a->a_mn; ph.b_mn = a->b_mn;
  ph.M = a->M; ph.N = a->N; ph.K = a->K; ph.bn = bn; ph.b_box = b_box;
  ph.batch = a->batch; ph.batch_inner = a->batch_inner;
  ph.a_bo_mn = a->a_bo_mn; ph.a_bo_k = a->a_bo_k; ph.a_bi_mn = a->a_bi_mn; ph.a_bi_k = a->a_bi_k;
  ph.b_bo_mn = a->b_bo_mn; ph.b_bo_k = a->b_bo_k; ph.b_bi_mn = a->b_bi_mn; ph.b_bi_k = a->b_bi_k;
  ph.d = a->d; ph.ldd = a->ldd; ph.d_bo = a->d_bo; ph.d_bi = a->d_bi;
  ph.causal = a->causal; ph.alpha = a->alpha;
  set_vec_ok(ph);
  if ((a->d_bo | a->d_bi) & 7) ph.vec_ok = 0;
  P.n_phases = 1;
  P.status = a->status;
  if (!P.status) return fail("status word required");
  const long long tiles = (long long)((a->M + 127) / 128) * ((a->N + bn - 1) / bn) * a->batch;
  const int ctas = sm_count();
  const int grid = tiles < ctas ? (int)tiles : ctas;
  params.ctas_per_rank = grid;
  return launch<1>(params, grid, false, (cudaStream_t)stream);
}

int rtp_linear_fwd(const RtpRing* ring, const RtpLinearFwd* op, void* stream) {
  static thread_local rtp::GemmParams<1> params;
  // CTA pairs by size, on any ring (the pair protocol is local to one GPU; checked against an fp32 oracle on real rings)
  decide_pair(op->M, ring->world > 1 && op->mode == 0 ? op->out_features / ring->world : op->out_features, ring->ctas);
  if (build_linear_fwd(*ring, *op, params.prog[0])) return -1;
  params.prog[0].trace = g_trace;
  if (!params.prog[0].status) return fail("ring workspace required");
  params.ctas_per_rank = ring->ctas;
  return launch<1>(params, ring->ctas, false, (cudaStream_t)stream, true);
}
int rtp_linear_bwd(const RtpRing* ring, const RtpLinearBwd* op, void* stream) {
  static thread_local rtp::GemmParams<1> params;
  // CTA pairs by the size of the input-gradient GEMM [M, in-per-shard], on any ring
  decide_pair(op->M, op->mode == 0 ? op->in_features : op->in_features / ring->world, ring->ctas);
  if (build_linear_bwd(*ring, *op, params.prog[0])) return -1;
  params.prog[0].trace = g_trace;
  if (!params.prog[0].status) return fail("ring workspace required");
  params.ctas_per_rank = ring->ctas;
  return launch<1>(params, ring->ctas, false, (cudaStream_t)stream, true);
}
int rtp_linear_bwd_folds_bias(const RtpRing* ring, const RtpLinearBwd* op) {
  decide_pair(op->M, op->mode == 0 ? op->in_features : op->in_features / ring->world, ring->ctas);
  return (op->bias_off >= 0 && op->ones && folds_bias(*ring, *op)) ? 1 : 0;
}
int rtp_expert_fwd(const RtpRing* ring, const RtpExpertFwd* op, void* stream) {
  static thread_local rtp::GemmParams<1> params;
  decide_pair(0, 0, ring->ctas);   // pairs only when forced
  if (build_expert_fwd(*ring, *op, params.prog[0])) return -1;
  if (!params.prog[0].status) return fail("ring workspace required");
  params.ctas_per_rank = ring->ctas;
  return launch<1>(params, ring->ctas, false, (cudaStream_t)stream, true);
}
int rtp_expert_bwd(const RtpRing* ring, const RtpExpertBwd* op, void* stream) {
  static thread_local rtp::GemmParams<1> params;
  decide_pair(0, 0, ring->ctas);   // pairs only when forced
  if (build_expert_bwd(*ring, *op, params.prog[0])) return -1;
  if (!params.prog[0].status) return fail("ring workspace required");
  params.ctas_per_rank = ring->ctas;
  return launch<1>(params, ring->ctas, false, (cudaStream_t)stream, true);
}
int rtp_expert_fwd_emu(const RtpRing* rings, const RtpExpertFwd* ops, int world, void* stream) {
  if (world == 2) return run_emu<2>(rings, ops, build_expert_fwd, (cudaStream_t)stream);
  if (world == 4) return run_emu<4>(rings, ops, build_expert_fwd, (cudaStream_t)stream);
  return fail("emulation supports 2 or 4 ranks");
}
int rtp_expert_bwd_emu(const RtpRing* rings, const RtpExpertBwd* ops, int world, void* stream) {
  if (world == 2) return run_emu<2>(rings, ops, build_expert_bwd, (cudaStream_t)stream);
  if (world == 4) return run_emu<4>(rings, ops, build_expert_bwd, (cudaStream_t)stream);
  return fail("emulation supports 2 or 4 ranks");
}
int rtp_embed_fwd_rot(const RtpRing* ring, const RtpEmbedFwd* op, void* stream) {
  static thread_local rtp::GemmParams<1> params;
  if (build_embed_fwd(*ring, *op, params.prog[0])) return -1;
  if (!params.prog[0].status) return fail("ring workspace required");
  params.ctas_per_rank = ring->ctas;
  return launch<1>(params, ring->ctas, false, (cudaStream_t)stream);
}
int rtp_reduce_scatter_cols(const RtpRing* ring, const RtpReduceScatter* op, void* stream) {
  static thread_local rtp::GemmParams<1> params;
  if (build_reduce_scatter(*ring, *op, params.prog[0])) return -1;
  if (!params.prog[0].status) return fail("ring workspace required");
  params.ctas_per_rank = ring->ctas;
  return launch<1>(params, ring->ctas, false, (cudaStream_t)stream);
}
int rtp_reduce_blocks(const RtpRing* ring, const RtpReduceBlocks* op, void* stream) {
  static thread_local rtp::GemmParams<1> params;
  if (build_reduce_blocks(*ring, *op, params.prog[0])) return -1;
  if (!params.prog[0].status) return fail("ring workspace required");
  params.ctas_per_rank = ring->ctas;
  return launch<1>(params, ring->ctas, false, (cudaStream_t)stream);
}
int rtp_reduce_blocks_emu(const RtpRing* rings, const RtpReduceBlocks* ops, int world, void* stream) {
  if (world == 2) return run_emu<2>(rings, ops, build_reduce_blocks, (cudaStream_t)stream);
  if (world == 4) return run_emu<4>(rings, ops, build_reduce_blocks, (cudaStream_t)stream);
  return fail("emulation supports 2 or 4 ranks");
}
int rtp_embed_fwd_rot_emu(const RtpRing* rings, const RtpEmbedFwd* ops, int world, void* stream) {
  if (world == 2) return run_emu<2>(rings, ops, build_embed_fwd, (cudaStream_t)stream);
  if (world == 4) return run_emu<4>(rings, ops, build_embed_fwd, (cudaStream_t)stream);
  return fail("emulation supports 2 or 4 ranks");
}
int rtp_reduce_scatter_cols_emu(const RtpRing* rings, const RtpReduceScatter* ops, int world, void* stream) {
  if (world == 2) return run_emu<2>(rings, ops, build_reduce_scatter, (cudaStream_t)stream);
  if (world == 4) return run_emu<4>(rings, ops, build_reduce_scatter, (cudaStream_t)stream);
  return fail("emulation supports 2 or 4 ranks");
}
int rtp_linear_fwd_emu(const RtpRing* rings, const RtpLinearFwd* ops, int world, void* stream) {
  if (world == 2) return run_emu<2>(rings, ops, build_linear_fwd, (cudaStream_t)stream);
  if (world == 4) return run_emu<4>(rings, ops, build_linear_fwd, (cudaStream_t)stream);
  return fail("emulation supports 2 or 4 ranks");
}
int rtp_linear_bwd_emu(const RtpRing* rings, const RtpLinearBwd* ops, int world, void* stream) {
  if (world == 2) return run_emu<2>(rings, ops, build_linear_bwd, (cudaStream_t)stream);
  if (world == 4) return run_emu<4>(rings, ops, build_linear_bwd, (cudaStream_t)stream);
  return fail("emulation supports 2 or 4 ranks");
}

// ------------------------------------------------------------------------------------- workspace
// bytes of a workspace that serves rings of exactly `world` ranks
unsigned long long rtp_ws_bytes_world(unsigned long long slot_bytes, int world) {
  if (world < 1) world = 1;
  return kFlagBytes + (unsigned long long)(RTP_NUM_WBANKS * (world - 1) + world) * slot_bytes;
}
int rtp_ws_create_world(unsigned long long slot_bytes, int world, void** out) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, rtp_ws_bytes_world(slot_bytes, world));
  if (e != cudaSuccess) return fail(std::string("cudaMalloc workspace: ") + cudaGetErrorString(e));
  e = cudaMemset(p, 0, kFlagBytes);
  if (e != cudaSuccess) { cudaFree(p); return fail("cudaMemset workspace failed"); }
  *out = p;
  return 0;
}
int rtp_ws_destroy(void* ws) { return cudaFree(ws) == cudaSuccess ? 0 : fail("cudaFree failed"); }
int rtp_ws_reset(void* ws, void* stream) {
  return cudaMemsetAsync(ws, 0, kFlagBytes, (cudaStream_t)stream) == cudaSuccess ? 0 : fail("memset failed");
}
int rtp_ws_ipc_get(void* ws, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ws);
  if (e != cudaSuccess) return fail(std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(e));
  static_assert(sizeof(h) == 64, "ipc handle size");
  memcpy(handle64, &h, 64);
  return 0;
}
int rtp_ws_ipc_open(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  cudaError_t e = cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fail(std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e));
  return 0;
}
int rtp_ws_ipc_close(void* mapped) {
  return cudaIpcCloseMemHandle(mapped) == cudaSuccess ? 0 : fail("cudaIpcCloseMemHandle failed");
}
int rtp_ws_status(void* ws, unsigned long long* host_out, void* stream) {
  cudaError_t e = cudaMemcpyAsync(host_out, &ws_flags(ws)->status.v, 8, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (e != cudaSuccess) return fail(std::string("status copy: ") + cudaGetErrorString(e));
  e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return fail(std::string("status sync: ") + cudaGetErrorString(e));
  return 0;
}
int rtp_ws_num_counters(void) { return RTP_NUM_CTR; }
int rtp_ws_counters(void* ws, unsigned long long* host_out, void* stream) {
  // arrive[], done[], uses[] of this rank's flag block, RTP_NUM_CTR words each (the words sit 128 bytes apart)
  const RtpFlagBlock* f = ws_flags(ws);
  const RtpFlagWord* src[3] = {f->arrive, f->done, f->uses};
  for (int k = 0; k < 3; ++k) {
    cudaError_t e = cudaMemcpy2DAsync(host_out + k * RTP_NUM_CTR, 8, src[k], sizeof(RtpFlagWord), 8, RTP_NUM_CTR,
                                      cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(std::string("counter copy: ") + cudaGetErrorString(e));
  }
  cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return fail(std::string("counter sync: ") + cudaGetErrorString(e));
  return 0;
}
void* rtp_ws_wslot(void* ws, unsigned long long slot_bytes, int i, int world) { return ws_wslot(ws, slot_bytes, i, world); }
void* rtp_ws_gslot(void* ws, unsigned long long slot_bytes, int i, int world) { return ws_gslot(ws, slot_bytes, i, world); }


// ---- program lint (host only; see the comment above lint_program) -------------------------------------------------
int rtp_lint_linear(int world, int ctas, unsigned long long slot_bytes, int mode, int M, int in_features, int out_features,
                    int has_bias, int backward, int need_dx, int inject, char* report, int cap) {
  rtp::host_tmap_mode() = true;
  Lint L;
  std::vector<RtpRing> rings;
  fake_rings(rings, world, ctas, slot_bytes);
  std::vector<RtpProgram> progs(world);
  std::vector<LintRect> rects;
  const bool col = mode == 0;
  const long long Os = col ? out_features / world : out_features, Ks = col ? in_features : in_features / world;
  int rc = 0;
  for (int r = 0; r < world && rc == 0; ++r) {
    bool pair;
    if (!backward) {
      RtpLinearFwd op = {};
      op.mode = mode; op.M = M; op.in_features = in_features; op.out_features = out_features;
      op.home = fake_buf(r, 0); op.bias_off = has_bias ? Os * Ks : -1;
      op.shard_bytes = (unsigned long long)((Os * Ks + (has_bias ? Os : 0)) * 2 + 15) & ~15ull;
      op.x = fake_buf(r, 1); op.ldx = in_features; op.y = fake_buf(r, 2); op.ldy = out_features;
      decide_pair(op.M, (world > 1 && col) ? out_features / world : out_features, ctas);
      pair = pair_mode();
      rc = build_linear_fwd(rings[r], op, progs[r]);
    } else {
      RtpLinearBwd op = {};
      op.mode = mode; op.M = M; op.in_features = in_features; op.out_features = out_features;
      op.home = fake_buf(r, 0); op.bias_off = has_bias ? Os * Ks : -1;
      op.shard_bytes = (unsigned long long)((Os * Ks + (has_bias ? Os : 0)) * 2 + 15) & ~15ull;
      op.x = fake_buf(r, 1); op.ldx = in_features; op.dy = fake_buf(r, 2); op.ldy = out_features;
      if (need_dx) { op.dx = fake_buf(r, 3); op.lddx = in_features; }
      op.grad_home = fake_buf(r, 4);
      if (has_bias) op.dbias_full = reinterpret_cast<const float*>(fake_buf(r, 5));
      decide_pair(op.M, col ? in_features : in_features / world, ctas);
      pair = pair_mode();
      rc = build_linear_bwd(rings[r], op, progs[r]);
    }
    if (rc) { L.bad("rank " + lstr(r) + ": builder refused: " + g_err); break; }
    finalize_program(progs[r], ctas, pair);
    if (r == 0) lint_inject(progs[0], inject);
    lint_program(L, rings[r], r, progs[r], pair, rects);
  }
  if (rc == 0 && world > 1) lint_ring(L, rings, progs);
  rtp::host_tmap_mode() = false;
  return lint_finish(L, rects, report, cap);
}

int rtp_lint_experts(int world, int ctas, unsigned long long slot_bytes, int n_local, int cap_tokens, int in_features,
                     int out_features, int has_bias, int backward, int need_dx, char* report, int cap) {
  rtp::host_tmap_mode() = true;
  Lint L;
  std::vector<RtpRing> rings;
  fake_rings(rings, world, ctas, slot_bytes);
  std::vector<RtpProgram> progs(world);
  std::vector<LintRect> rects;
  const long long block = (long long)out_features * in_features + (has_bias ? out_features : 0);
  const long long stride = (block + 7) & ~7ll;
  int rc = 0;
  for (int r = 0; r < world && rc == 0; ++r) {
    decide_pair(0, 0, ctas);
    if (!backward) {
      RtpExpertFwd op = {};
      op.cap = cap_tokens; op.n_local = n_local; op.in_features = in_features; op.out_features = out_features;
      op.home = fake_buf(r, 0); op.expert_stride = stride; op.bias_off = has_bias ? (long long)out_features * in_features : -1;
      op.shard_bytes = (unsigned long long)(stride * n_local * 2 + 15) & ~15ull;
      op.x = fake_buf(r, 1); op.ldx = in_features; op.y = fake_buf(r, 2); op.ldy = out_features;
      rc = build_expert_fwd(rings[r], op, progs[r]);
    } else {
      RtpExpertBwd op = {};
      op.cap = cap_tokens; op.n_local = n_local; op.in_features = in_features; op.out_features = out_features;
      op.home = fake_buf(r, 0); op.expert_stride = stride; op.bias_off = has_bias ? (long long)out_features * in_features : -1;
      op.shard_bytes = (unsigned long long)(stride * n_local * 2 + 15) & ~15ull;
      op.x = fake_buf(r, 1); op.ldx = in_features; op.dy = fake_buf(r, 2); op.ldy = out_features;
      if (need_dx) { op.dx = fake_buf(r, 3); op.lddx = in_features; }
      op.grad_home = fake_buf(r, 4);
      if (has_bias) op.dbias_full = reinterpret_cast<const float*>(fake_buf(r, 5));
      rc = build_expert_bwd(rings[r], op, progs[r]);
    }
    if (rc) { L.bad("rank " + lstr(r) + ": builder refused: " + g_err); break; }
    finalize_program(progs[r], ctas, pair_mode());
    lint_program(L, rings[r], r, progs[r], pair_mode(), rects);
  }
  if (rc == 0 && world > 1) lint_ring(L, rings, progs);
  rtp::host_tmap_mode() = false;
  return lint_finish(L, rects, report, cap);
}


// Chain lint: the rotated linears of a training step as the fused trainer issues them.  Launch k reads its visiting
// shards from weight-slot bank k & 1; launch 0 pushes its own shards, every later launch finds them pushed by its
// predecessor, and every launch but the last pushes the home shard of its successor into the other bank.  `spec` holds
// 7 ints per launch: mode, M, in_features, out_features, has_bias, backward, need_dx.  Checked per launch, with the
// producers of a launch taken to be its own pushes into its bank plus the predecessor's pushes into that bank: the
// same ring rules as rtp_lint_linear (one producer per awaited counter, matching credit, writes inside the slot, slot
// reported done, identical fill counts), and in addition that a launch never pushes ahead into a bank it fills or reads
// itself and that the last launch pushes nothing ahead.  `flip_bank_at` >= 0 builds that launch with the wrong bank (a
// self-test: the lint must complain).
int rtp_lint_linear_chain(int world, int ctas, unsigned long long slot_bytes, int n_launches, const int* spec,
                          int flip_bank_at, char* report, int cap) {
  rtp::host_tmap_mode() = true;
  Lint L;
  std::vector<RtpRing> rings;
  fake_rings(rings, world, ctas, slot_bytes);
  std::vector<LintRect> rects;     // per-launch tile overlap is the business of rtp_lint_linear: not collected here
  std::vector<std::vector<RtpProgram>> progs(n_launches, std::vector<RtpProgram>(world));
  auto shard_elems = [&](const int* sp) {
    const bool col = sp[0] == 0;
    const long long Os = col ? sp[3] / world : sp[3], Ks = col ? sp[2] : sp[2] / world;
    return Os * Ks + (sp[4] ? Os : 0);
  };
  int rc = 0;
  for (int k = 0; k < n_launches && rc == 0; ++k) {
    const int* sp = spec + 7 * k;
    const int* nx = k + 1 < n_launches ? spec + 7 * (k + 1) : nullptr;
    const bool col = sp[0] == 0;
    const long long Os = col ? sp[3] / world : sp[3], Ks = col ? sp[2] : sp[2] / world;
    const int bank = (k & 1) ^ (k == flip_bank_at ? 1 : 0);
    for (int r = 0; r < world && rc == 0; ++r) {
      const void* next_home = nx ? fake_buf(r, 8 + ((k + 1) & 7)) : nullptr;
      const unsigned long long next_bytes = nx ? (unsigned long long)(shard_elems(nx) * 2 + 15) & ~15ull : 0;
      bool pair;
      if (!sp[5]) {
        RtpLinearFwd op = {};
        op.mode = sp[0]; op.M = sp[1]; op.in_features = sp[2]; op.out_features = sp[3];
        op.home = fake_buf(r, 8 + (k & 7)); op.bias_off = sp[4] ? Os * Ks : -1;
        op.shard_bytes = (unsigned long long)(shard_elems(sp) * 2 + 15) & ~15ull;
        op.x = fake_buf(r, 1); op.ldx = sp[2]; op.y = fake_buf(r, 2); op.ldy = sp[3];
        op.bank = bank; op.no_self_push = k > 0;
        op.next_home = next_home; op.next_bytes = next_bytes; op.next_kind = nx ? nx[5] : 0;
        decide_pair(op.M, (world > 1 && col) ? sp[3] / world : sp[3], ctas);
        pair = pair_mode();
        rc = build_linear_fwd(rings[r], op, progs[k][r]);
      } else {
        RtpLinearBwd op = {};
        op.mode = sp[0]; op.M = sp[1]; op.in_features = sp[2]; op.out_features = sp[3];
        op.home = fake_buf(r, 8 + (k & 7)); op.bias_off = sp[4] ? Os * Ks : -1;
        op.shard_bytes = (unsigned long long)(shard_elems(sp) * 2 + 15) & ~15ull;
        op.x = fake_buf(r, 1); op.ldx = sp[2]; op.dy = fake_buf(r, 2); op.ldy = sp[3];
        if (sp[6]) { op.dx = fake_buf(r, 3); op.lddx = sp[2]; }
        op.grad_home = fake_buf(r, 4);
        if (sp[4]) op.dbias_full = reinterpret_cast<const float*>(fake_buf(r, 5));
        op.bank = bank; op.no_self_push = k > 0;
        op.next_home = next_home; op.next_bytes = next_bytes; op.next_kind = nx ? nx[5] : 0;
        decide_pair(op.M, col ? sp[2] : sp[2] / world, ctas);
        pair = pair_mode();
        rc = build_linear_bwd(rings[r], op, progs[k][r]);
      }
      if (rc) { L.bad("launch " + lstr(k) + " rank " + lstr(r) + ": builder refused: " + g_err); break; }
      finalize_program(progs[k][r], ctas, pair);
    }
  }
  auto w_bank = [](int ctr) { return (ctr >= RTP_CTR_W0 && ctr < RTP_CTR_G0) ? (ctr - RTP_CTR_W0) / RTP_NUM_SLOTS : -1; };
  for (int k = 0; k < n_launches && rc == 0 && world > 1; ++k) {
    const int bank = k & 1;          // the bank the chain rule gives this launch, whatever it was built with
    std::vector<RtpProgram> merged(world);
    const size_t before = L.rep.size();
    for (int r = 0; r < world; ++r) {
      const RtpProgram& P = progs[k][r];
      RtpProgram& Q = merged[r];
      Q = P;
      Q.n_pushes = 0;
      for (int j = 0; j < P.n_pushes; ++j) {
        const int b = w_bank(P.pushes[j].credit_ctr);
        if (b == bank || b < 0) Q.pushes[Q.n_pushes++] = P.pushes[j];
        else {
          if (k + 1 == n_launches) L.bad("launch " + lstr(k) + " rank " + lstr(r) + ": the last launch pushes ahead");
          if (P.uses_inc[P.pushes[j].credit_ctr])
            L.bad("launch " + lstr(k) + " rank " + lstr(r) + " push " + lstr(j) + ": pushes ahead into a slot that the launch fills itself");
        }
      }
      if (k > 0) {
        const RtpProgram& B = progs[k - 1][r];
        for (int j = 0; j < B.n_pushes; ++j)
          if (w_bank(B.pushes[j].credit_ctr) == bank) {
            if (Q.n_pushes >= RTP_MAX_PUSHES) { L.bad("launch " + lstr(k) + ": too many producers"); break; }
            Q.pushes[Q.n_pushes++] = B.pushes[j];
          }
      }
      for (int p = 0; p < P.n_phases; ++p)
        for (int w = 0; w < RTP_MAX_WAITS; ++w) {
          const int b = w_bank(P.phases[p].wait_ctr[w]);
          if (b >= 0 && b != bank)
            L.bad("launch " + lstr(k) + " rank " + lstr(r) + " phase " + lstr(p) + ": reads bank " + lstr(b) + ", the chain gives it bank " + lstr(bank));
        }
    }
    lint_ring(L, rings, merged);
    if (L.rep.size() > before) L.rep.insert(before, "launch " + lstr(k) + ":\n");
  }
  rtp::host_tmap_mode() = false;
  return lint_finish(L, rects, report, cap);
}


// The programs without GEMM tiles: kind 0 = rotated embedding lookup (a = V, b = D, c = tokens), 1 = one-hop reduce of
// `world` blocks of a elements.  Only the ring rules apply (there are no tiled copies).  The hop-by-hop reduce-scatter
// (rtp_reduce_scatter_cols) fills the same slot several times per launch, which these one-fill-per-launch rules do not
// describe: it is not linted.
int rtp_lint_transport(int world, int ctas, unsigned long long slot_bytes, int kind, long long a, long long b, long long c,
                       char* report, int cap) {
  if (kind != 0 && kind != 1) return fail("rtp_lint_transport: kind must be 0 or 1");
  rtp::host_tmap_mode() = true;
  Lint L;
  std::vector<RtpRing> rings;
  fake_rings(rings, world, ctas, slot_bytes);
  std::vector<RtpProgram> progs(world);
  std::vector<LintRect> rects;
  int rc = 0;
  for (int r = 0; r < world && rc == 0; ++r) {
    decide_pair(0, 0, 0, false);
    if (kind == 0) {
      RtpEmbedFwd op = {};
      op.V = (int)a; op.D = (int)b; op.Ds = (int)(b / world); op.T = (int)c;
      op.home = fake_buf(r, 0); op.shard_bytes = ((unsigned long long)a * (unsigned long long)op.Ds * 2 + 15) & ~15ull;
      op.ids = reinterpret_cast<const long long*>(fake_buf(r, 1));
      op.out = fake_buf(r, 2); op.ld_out = b; op.scale = 1.f; op.tokens_per_pos = 1;
      rc = build_embed_fwd(rings[r], op, progs[r]);
    } else {
      RtpReduceBlocks op = {};
      op.src = fake_buf(r, 0); op.block_elems = a; op.out = fake_buf(r, 2);
      rc = build_reduce_blocks(rings[r], op, progs[r]);
    }
    if (rc) { L.bad("rank " + lstr(r) + ": builder refused: " + g_err); break; }
    finalize_program(progs[r], ctas, false);
  }
  if (rc == 0 && world > 1) lint_ring(L, rings, progs);
  rtp::host_tmap_mode() = false;
  return lint_finish(L, rects, report, cap);
}

}  // extern "C"
