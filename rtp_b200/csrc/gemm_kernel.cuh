// The rotation GEMM kernel: a persistent, warp-specialised tcgen05 kernel that runs an RtpProgram.
//
//   warp 0      TMA producer: streams 128x64 (A) and bn x 64 (B) bf16 tiles into a 4-stage smem ring
//   warp 1      UMMA issuer: one elected thread issues tcgen05.mma into one of two TMEM accumulators
//   warps 2-5   epilogue: tcgen05.ld the accumulator, apply bias/activation/mask/dropout/accumulate,
//               store to local or peer global memory, then bump the phase's counters
//   warp 6      pusher: copies this rank's home shard into a peer's workspace slot with bulk asynchronous copies (bulk
//               load from local memory into a two-slot shared-memory ring, bulk store from there into the peer's memory
//               over NVLink), bounded by the peer's slot-free counter, then bumps the peer's arrival counter
//   warp 7      signaller: release fence + "data arrived" signal of phases whose output goes to another rank, so that the
//               epilogue warps never wait for their NVLink stores to be acknowledged
//
// All cross-rank waits are on 64-bit counters with an iteration/time limit; on expiry the CTA marks
// the status word, drains what it has in flight, frees its TMEM and returns.
#pragma once
#include "common.cuh"
#include "gemm_program.h"

namespace rtp {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kMaxStages = 8;
constexpr int kABytes = kBM * kBK * 2;          // 16 KB
constexpr int kTileBytes = 196608;              // smem ring: 4 stages of 48 KB (bn 256) or 6 stages of 32 KB (bn 128)
constexpr int kTmemCols = 512;
constexpr int kNumThreads = 256;
constexpr int kStagePitch = 144;                // bytes per staged output row: 64 bf16 + 16 pad (conflict-free 16 B writes)
constexpr int kStagingBytes = 4 * 32 * kStagePitch;
// Push rings.  A CTA that also runs GEMM tiles has a small ring of its own (its shared memory belongs to the tile
// pipeline); a CTA reserved for pushing uses the idle tile pipeline's memory as a deep ring.
// A transfer to a peer costs a fixed 3 to 4 microseconds (measured on two B200s: 1 MB in 7 us, 8 MB in 18 us, 64 MB in
// 100 us = 670 GB/s, whatever issues the copies).  What matters is therefore never to wait for one job's stores
// before starting the next: four small chunks per CTA are outstanding at any time and a job is announced while the
// stores of the following jobs are already on the link.
constexpr int kPushChunk = 3840;                // small ring: bytes per bulk copy
constexpr int kPushSlots = 4;
constexpr int kPushRingBytes = kPushSlots * kPushChunk;
constexpr int kBigPushChunk = 16384;            // deep ring: 12 slots in the tile area
constexpr int kMaxPushSlots = 12;
static_assert(kMaxPushSlots * kBigPushChunk <= 196608, "deep push ring must fit the tile area");
constexpr int kCtlBytes = 768;                  // barriers and CTA-wide words
constexpr int kSmemBytes = kTileBytes + 1024 /*align slack*/ + kCtlBytes + kStagingBytes + kPushRingBytes;
static_assert(kSmemBytes <= 232448, "over the 227 KB of shared memory a CTA can have");

struct SmemCtrl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t peer_full[kMaxStages];   // pair mode, leader only: "the other CTA's half of this stage has landed"
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t drain;
  uint64_t push_full[kMaxPushSlots];   // push ring: "the bulk load into slot s has landed"
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t handed;                  // phases the epilogue warps have handed to the signaller warp
  uint32_t jobs_issued;             // push jobs whose stores the pusher warp has issued (store-pusher mode)
  // Copy of the flag block's uses[] (completed fills per slot; constant while a launch runs).  Every wait target is
  // computed from it; read from global memory it cost a dependent ~0.7 us load in front of every counter poll.
  unsigned long long uses[RTP_NUM_CTR];
};

static_assert(sizeof(SmemCtrl) <= kCtlBytes, "control block outgrew its shared-memory slot");

// One rank per launch: the program travels as a kernel parameter.  Emulated ranks (several programs in one
// cooperative launch on one GPU) read their programs from constant memory instead, which is large enough for four.
template <int NEMU>
struct GemmParams {
  RtpProgram prog[NEMU == 1 ? 1 : 1];
  int ctas_per_rank;
};
__device__ RtpProgram c_emu_progs[RTP_MAX_EMU_RANKS];   // global, not constant memory: four programs exceed the 64 KB constant bank

__device__ __forceinline__ unsigned long long fill_target(const unsigned long long* uses, int ctr, int rel, int plus,
                                                          int G) {
  // counters count one unit per CTA per fill of the slot
  return (uses[ctr] + (unsigned long long)(rel + plus)) * (unsigned long long)G;
}

// a slot may be written again once `uses + rel` of its fills have been read completely (credits count whole fills)
__device__ __forceinline__ unsigned long long credit_target(const unsigned long long* uses, int ctr, int rel) {
  return uses[ctr] + (unsigned long long)rel;
}

// ------------------------------------------------------------------------------------------------------------------
// Push jobs of one CTA: its share (index / sharers) of every job moves through a ring of NS shared-memory slots with
// bulk asynchronous copies: bulk load from local memory, then bulk store into the peer's slot over NVLink.  All chunks
// of all jobs form one software pipeline: NS - 1 loads are in flight while stores leave; at most LAG + 1 stores are
// outstanding, and a job is signalled ("data arrived") once its last store is complete.
// ------------------------------------------------------------------------------------------------------------------
struct PushCtx {
  const RtpProgram* P;
  int G, cta, index, sharers;
  uint8_t* ring;
  uint64_t* bars;
  const unsigned long long* uses;   // the CTA's copy of the slot fill counts
  volatile uint32_t* abort_flag;
  unsigned long long* status;
  unsigned long long wait_ns, timeout_ns;
};

// Store-pusher: the whole warp streams this CTA's share of every job with plain loads and peer stores through
// registers (16 x 16 bytes per lane in flight).  Peer stores are posted: the warp never waits for one, so all jobs of a
// launch are on the link back to back.  A job whose stores have been ISSUED is handed to the signaller warp, which makes
// them visible with its (batched) system fence and announces the job.  Measured on 8 B200s this is what keeps NVLink
// busy: with the bulk-copy pusher below, the issuing thread has to wait for the completion of its own copies before it
// may announce a job, and under an 8-way exchange a completion takes ~10 us, during which it issues nothing (7 x 1 MB
// took 66 us: 106 GB/s).
__device__ __noinline__ void run_pushes_stores(const PushCtx& c, SmemCtrl* ctl, int lane) {
  const RtpProgram& P = *c.P;
  bool ok = true;
  for (int j = 0; j < P.n_pushes; ++j) {
    const RtpPush& pu = P.pushes[j];
    const bool tr = P.trace && c.cta == 0 && lane == 0 && j < 8;
    if (tr) P.trace[3 * 256 + 200 + j * 4 + 0] = globaltimer_ns();
    uint32_t good = ok ? 1u : 0u;
    if (ok && lane == 0 && pu.credit_ptr)
      good = wait_counter_ge(pu.credit_ptr, credit_target(c.uses, pu.credit_ctr, pu.credit_rel), c.abort_flag, c.status,
                             c.wait_ns, ST_TIMEOUT_CREDIT) ? 1u : 0u;
    good = __shfl_sync(0xffffffffu, good, 0);
    if (!good) ok = false;
    if (tr) P.trace[3 * 256 + 200 + j * 4 + 1] = globaltimer_ns();
    if (ok) {
      const unsigned long long units = pu.bytes >> 4;
      const unsigned long long per = (units + c.sharers - 1) / c.sharers;
      const unsigned long long lo = per * (unsigned long long)c.index;
      unsigned long long hi = lo + per;
      if (hi > units) hi = units;
      const uint4* src = reinterpret_cast<const uint4*>(pu.src);
      uint4* dst = reinterpret_cast<uint4*>(pu.dst);
      unsigned long long i = lo + lane;
      for (; i + 32 * 15 < hi; i += 32 * 16) {
        uint4 v[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) v[u] = __ldg(src + i + 32 * u);
#pragma unroll
        for (int u = 0; u < 16; ++u) dst[i + 32 * u] = v[u];
      }
      for (; i < hi; i += 32) dst[i] = __ldg(src + i);
    }
    // every lane's stores are ordered before lane 0's release of the counter
    __syncwarp();
    if (lane == 0) {
      __threadfence_block();
      atomicAdd(&ctl->jobs_issued, 1u);
    }
    if (tr) P.trace[3 * 256 + 200 + j * 4 + 3] = globaltimer_ns();
  }
}

template <int NS, int CHUNK, int LAG>
__device__ __noinline__ void run_pushes(const PushCtx& c) {
  const RtpProgram& P = *c.P;
  const uint32_t ring_s = smem_u32(c.ring);
  const uint32_t pf_s = smem_u32(c.bars);
  bool ok = true;
  uint32_t ph_bits = 0;                 // parity of the next completion of every slot's barrier
  // byte range of job j that this CTA moves
  auto job_range = [&](int j, unsigned long long& lo, unsigned long long& hi) {
    const unsigned long long units = P.pushes[j].bytes >> 4;
    const unsigned long long per = (units + c.sharers - 1) / c.sharers;
    lo = per * (unsigned long long)c.index;
    hi = lo + per;
    if (hi > units) hi = units;
    if (lo > hi) lo = hi;
    lo <<= 4; hi <<= 4;
  };
  auto signal_job = [&](int j) {
    if (P.trace && c.cta == P.n_compute % c.G && j < 8) P.trace[3 * 256 + 200 + j * 4 + 3] = globaltimer_ns();
    // the job's stores are complete: make them visible system-wide, then count this CTA in
    fence_proxy_async();
    __threadfence_system();
    if (P.pushes[j].arrive_ptr) red_relaxed_sys_add(P.pushes[j].arrive_ptr, 1ull);
    if (P.trace && c.cta == P.n_compute % c.G && j < 8) P.trace[3 * 256 + 200 + j * 4 + 2] = globaltimer_ns();
  };
  // chunk cursor of the loader
  int lj = 0;
  unsigned long long loff = 0, lhi = 0;
  bool lvalid = false;
  auto next_chunk = [&]() {
    lvalid = false;
    while (lj < P.n_pushes) {
      if (loff < lhi) { lvalid = true; return; }
      ++lj;
      if (lj < P.n_pushes) job_range(lj, loff, lhi);
    }
  };
  job_range(0, loff, lhi);
  next_chunk();
  // per ring slot: what was loaded there
  uint32_t s_bytes[NS];
  int s_job[NS];
  unsigned long long s_off[NS];
  bool s_start[NS], s_last[NS];
  for (int i = 0; i < NS; ++i) s_job[i] = -1;
  auto issue_load = [&](int s) {
    const RtpPush& pu = P.pushes[lj];
    const unsigned long long n = (lhi - loff) < (unsigned long long)CHUNK ? (lhi - loff) : (unsigned long long)CHUNK;
    unsigned long long jlo, jhi;
    job_range(lj, jlo, jhi);
    s_bytes[s] = (uint32_t)n; s_job[s] = lj; s_off[s] = loff;
    s_start[s] = loff == jlo; s_last[s] = loff + n == lhi;
    mbar_arrive_expect_tx_s(pf_s + s * 8, (uint32_t)n);
    bulk_load_s(ring_s + s * CHUNK, reinterpret_cast<const uint8_t*>(pu.src) + loff, (uint32_t)n, pf_s + s * 8);
    loff += n;
    next_chunk();
  };
  // jobs whose last store has been committed but not yet signalled, in commit order: (job, index of its last store)
  int q_job[RTP_MAX_PUSHES], q_at[RTP_MAX_PUSHES];
  int q_head = 0, q_tail = 0;
  bool counted[RTP_MAX_PUSHES];
  for (int j = 0; j < RTP_MAX_PUSHES; ++j) counted[j] = false;
  int n_loaded = 0, n_stored = 0;
  for (; n_loaded < NS - 1 && lvalid; ++n_loaded) issue_load(n_loaded % NS);
  while (n_stored < n_loaded && ok) {
    const int s = n_stored % NS;
    const int j = s_job[s];
    const RtpPush& pu = P.pushes[j];
    if (s_start[s]) {
      if (P.trace && c.cta == P.n_compute % c.G && j < 8) P.trace[3 * 256 + 200 + j * 4 + 0] = globaltimer_ns();
      if (pu.credit_ptr && !wait_counter_ge(pu.credit_ptr, credit_target(c.uses, pu.credit_ctr, pu.credit_rel), c.abort_flag,
                                            c.status, c.wait_ns, ST_TIMEOUT_CREDIT)) {
        ok = false;
        break;
      }
      if (P.trace && c.cta == P.n_compute % c.G && j < 8) P.trace[3 * 256 + 200 + j * 4 + 1] = globaltimer_ns();
    }
    // the load of this chunk has landed (a copy from local memory always completes; the limit guards a logic error)
    if (!mbar_wait_s(pf_s + s * 8, (ph_bits >> s) & 1u, c.abort_flag, c.status, c.timeout_ns)) { ok = false; break; }
    ph_bits ^= 1u << s;
    s_job[s] = -1;
    bulk_store_s(reinterpret_cast<uint8_t*>(pu.dst) + s_off[s], ring_s + s * CHUNK, s_bytes[s]);
    bulk_commit();
    if (s_last[s]) { q_job[q_tail] = j; q_at[q_tail] = n_stored; ++q_tail; }
    ++n_stored;
    // the store before this one has read its slot: that slot takes the next load
    bulk_wait_read<1>();
    if (lvalid) { issue_load(n_loaded % NS); ++n_loaded; }
    // jobs whose last store is complete are announced
    if (q_head < q_tail && q_at[q_head] < n_stored - LAG) {
      bulk_wait<LAG>();
      while (q_head < q_tail && q_at[q_head] < n_stored - LAG) {
        signal_job(q_job[q_head]);
        counted[q_job[q_head]] = true;
        ++q_head;
      }
    }
  }
  bulk_wait<0>();
  if (!ok) {
    // loads may still be in flight into the ring: let them land before the CTA can exit
    for (int s = 0; s < NS; ++s) {
      if (s_job[s] < 0) continue;
      const unsigned long long t0 = globaltimer_ns();
      while (!mbar_try_wait(c.bars + s, (ph_bits >> s) & 1u)) {
        if (globaltimer_ns() - t0 > 2000000ull) break;
      }
    }
  }
  while (q_head < q_tail) {
    if (ok) signal_job(q_job[q_head]);
    counted[q_job[q_head]] = true;
    ++q_head;
  }
  // jobs in which this CTA had nothing to move
  for (int j = 0; j < P.n_pushes && ok; ++j)
    if (!counted[j] && P.pushes[j].arrive_ptr) red_relaxed_sys_add(P.pushes[j].arrive_ptr, 1ull);
}

// PAIR = true: launched with clusters of two CTAs; one UMMA (cta_group::2, M = 256) spans the pair.
template <int NEMU, bool PAIR>
__global__ void __launch_bounds__(kNumThreads, 1) rtp_gemm_kernel(const __grid_constant__ GemmParams<NEMU> params) {
  extern __shared__ uint8_t smem_raw[];
  const int G = params.ctas_per_rank;
  const uint32_t crank = PAIR ? cluster_ctarank() : 0u;   // 0 = leader of the pair
  constexpr int TM = PAIR ? 2 * kBM : kBM;                 // rows of an output tile of one scheduling unit
  const int vrank = (NEMU == 1) ? 0 : (int)(blockIdx.x / G);
  const int cta = (NEMU == 1) ? (int)blockIdx.x : (int)(blockIdx.x % G);
  const RtpProgram& P = (NEMU == 1) ? params.prog[0] : c_emu_progs[vrank];

  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SmemCtrl* ctl = reinterpret_cast<SmemCtrl*>(tiles + kTileBytes);
  uint8_t* staging = tiles + kTileBytes + kCtlBytes;
  const int kStages = P.n_stages;          // uniform for the launch: set by the host from the widest tile
  const int kStageBytes = P.stage_bytes;
  volatile uint32_t* abort_flag = &ctl->abort_flag;
  unsigned long long* status = P.status;
  const unsigned long long wait_ns = P.timeout_ns;           // cross-rank counter waits
  const unsigned long long timeout_ns = 2 * P.timeout_ns;   // CTA-internal mbarrier waits (report the root cause first)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // scheduling unit = CTA, or CTA pair; GU units per rank
  const int unit = PAIR ? (cta >> 1) : cta;
  // CTAs [0, n_comp) own GEMM tiles; the rest (if any) are reserved for the push jobs of the launch
  const int n_comp = (P.n_compute > 0 && P.n_compute < G) ? P.n_compute : G;
  const bool tile_cta = cta < n_comp;
  const int GU = PAIR ? (n_comp >> 1) : n_comp;

  pdl_launch_dependents();
#define GEMM_STAMP(i) do { if (P.trace && cta == 0) P.trace[3 * 256 + 64 + (i)] = globaltimer_ns(); } while (0)
  if (threadIdx.x == 0) GEMM_STAMP(0);
  if (warp == 0) {
    // one barrier set per lane
    if (lane < kStages) {
      mbar_init(&ctl->full[lane], 1);
      mbar_init(&ctl->empty[lane], 1);
      mbar_init(&ctl->peer_full[lane], 1);
    } else if (lane < kMaxStages + 2) {
      const int a = lane - kMaxStages;
      if (a >= 0) {
        mbar_init(&ctl->tmem_full[a], 1);
        mbar_init(&ctl->tmem_empty[a], PAIR ? 8 : 4);  // pair: the epilogue warps of both CTAs arrive on the leader's barrier
      }
    } else if (lane == kMaxStages + 2) {
      mbar_init(&ctl->drain, 1);
      for (int i = 0; i < kMaxPushSlots; ++i) mbar_init(&ctl->push_full[i], 1);
      ctl->abort_flag = 0;
      ctl->handed = 0;
      ctl->jobs_issued = 0;
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    if (PAIR) { tmem_alloc_pair(&ctl->tmem_base, kTmemCols); tmem_relinquish_pair(); }
    else { tmem_alloc(&ctl->tmem_base, kTmemCols); tmem_relinquish(); }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();      // the peer's barriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  // everything above touched only shared memory and TMEM; from here on the previous kernel of the stream must be complete
  pdl_wait();
  // the previous launch has published its fill counts: one parallel read for all later wait targets (nothing waits
  // on a ring of one rank)
  if (P.flags && P.world != 1) {
    if (threadIdx.x >= 96 && threadIdx.x < 96 + RTP_NUM_CTR) ctl->uses[threadIdx.x - 96] = __ldcg(&P.flags->uses[threadIdx.x - 96].v);
    __syncthreads();
  }
  if (threadIdx.x == 0) GEMM_STAMP(1);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (tile_cta && elect_one()) {     // elect.sync, not lane == 0: lets the compiler treat the TMA operands as warp-uniform
      int stage = 0;
      uint32_t phase = 0;
      uint32_t issued_mask = 0, issued_parity = 0;   // bit s: stage s has been filled / parity of its last fill
      int tr_n = 0;
      const uint32_t tiles_s = smem_u32(tiles);
      const uint32_t full_s = smem_u32(&ctl->full[0]);
      const uint32_t empty_s = smem_u32(&ctl->empty[0]);

      bool ok = true;
      for (int p = 0; p < P.n_phases && ok; ++p) {
        const RtpPhase& ph = P.phases[p];
        const int tiles_m = (ph.M + TM - 1) / TM;
        const int tiles_n = (ph.N + ph.bn - 1) >> (31 - __clz(ph.bn));   // bn is a power of two
        const int per_batch = tiles_m * tiles_n;
        const int total = per_batch * ph.batch;
        if ((unit - ph.cta_off + GU) % GU >= total) continue;
        const int nseg = ph.nseg > 1 ? ph.nseg : 1;
        bool any_wait = false;
        for (int w = 0; w < RTP_MAX_WAITS && ok && nseg == 1 && !ph.tseg; ++w) {
          if (ph.wait_ctr[w] >= 0) {
            any_wait = true;
            ok = wait_counter_ge(&P.flags->arrive[ph.wait_ctr[w]].v,
                                 fill_target(ctl->uses, ph.wait_ctr[w], ph.wait_rel[w], 1, G), abort_flag, status,
                                 wait_ns, ST_TIMEOUT_ARRIVAL);
          }
        }
        if (!ok) break;
        if (any_wait) fence_proxy_async();
        uint32_t seg_ready = 0;          // segments whose shard has been seen to have arrived
        const unsigned long long ma = reinterpret_cast<unsigned long long>(&P.maps[ph.a_map]);
        unsigned long long mb = reinterpret_cast<unsigned long long>(&P.maps[ph.b_map]);
        const int kblocks_full = (ph.K + kBK - 1) / kBK;
        const int p_a_mn = ph.a_mn;
        const int p_b_mn = ph.b_mn;
        const int p_bn = ph.bn;
        const int p_causal = ph.causal;
        const int p_batch_inner = ph.batch_inner;
        const bool p_batch1 = ph.batch == 1;
        const int p_a_off_mn = ph.a_off_mn;
        const int p_a_off_k = ph.a_off_k;
        const int p_b_off_mn = ph.b_off_mn;
        const int p_b_off_k = ph.b_off_k;
        const int p_a_bo_mn = ph.a_bo_mn;
        const int p_a_bo_k = ph.a_bo_k;
        const int p_a_bi_mn = ph.a_bi_mn;
        const int p_a_bi_k = ph.a_bi_k;
        const int p_b_bo_mn = ph.b_bo_mn;
        const int p_b_bo_k = ph.b_bo_k;
        const int p_b_bi_mn = ph.b_bi_mn;
        const int p_b_bi_k = ph.b_bi_k;
        const int p_cta_off = ph.cta_off;
        const int bn_local = PAIR ? p_bn / 2 : p_bn;     // B rows staged by this CTA
        const uint32_t tx = kABytes + bn_local * kBK * 2;
        // One stage = na boxes of A and nb boxes of B.  Coordinates are kept as (x, y) of the tensor map, so the
        // k-loop only adds constants: a K-major operand advances x by 64 per k-block, an MN-major one advances y.
        const int na = p_a_mn ? 2 : 1;                                   // MN-major A: two 64-wide boxes
        const int nb = p_b_mn ? bn_local / 64 : bn_local / ph.b_box;
        const int a_dx = p_a_mn ? 0 : kBK, a_dy = p_a_mn ? kBK : 0;      // per k-block
        const int b_dx = p_b_mn ? 0 : kBK, b_dy = p_b_mn ? kBK : 0;
        const int b_ix = p_b_mn ? 64 : 0, b_iy = p_b_mn ? 0 : ph.b_box;  // per box inside a stage
        const uint32_t b_ismem = p_b_mn ? 8192u : (uint32_t)ph.b_box * 128u;
        bool a3 = p_a_mn && P.map3d[ph.a_map];
        bool b3 = p_b_mn && P.map3d[ph.b_map];
        const int p_tseg = ph.tseg, p_tseg_len = ph.tseg_len;
        const RtpSegTable& segs = P.segtab[ph.tseg_tab];
        unsigned long long ma_t = ma;
        if (p == 0) GEMM_STAMP(2);
        for (int t = (unit - p_cta_off + GU) % GU; t < total && ok; t += GU) {
          // unbatched phases (the common case) skip the divisions by the batch geometry
          const int z = p_batch1 ? 0 : t / per_batch, tt = p_batch1 ? t : t - z * per_batch;
          const int tn = tt / tiles_m;
          const int m0u = (tt - tn * tiles_m) * TM;          // first row of the unit's tile
          const int m0 = m0u + (int)crank * kBM;            // first row of this CTA's half
          const int n0 = tn * p_bn;
          if (p_causal == 1 && n0 > m0u + TM - 1) continue;
          const int kblocks = p_causal == 2 ? min(kblocks_full, (m0u + TM + kBK - 1) / kBK) : kblocks_full;
          const int kb0 = p_causal == 3 ? m0u / kBK : 0;   // contraction index = query, output row = key: queries before the key contribute nothing
          const int zo = p_batch1 ? 0 : z / p_batch_inner, zi = p_batch1 ? 0 : z - zo * p_batch_inner;
          int a_mn0 = m0 + p_a_off_mn + zo * p_a_bo_mn + zi * p_a_bi_mn;
          const int a_k0 = p_a_off_k + zo * p_a_bo_k + zi * p_a_bi_k;
          int b_mn0 = n0 + (int)crank * bn_local + p_b_off_mn + zo * p_b_bo_mn + zi * p_b_bi_mn;
          const int b_k0 = p_b_off_k + zo * p_b_bo_k + zi * p_b_bi_k;
          if (p_tseg) {
            // the tile belongs to one segment: its shard must have arrived; operand coordinates are local to the shard
            const int sgt = (p_tseg == 1 ? n0 : m0u) / p_tseg_len;
            if (!((seg_ready >> sgt) & 1u)) {
              if (ph.wait_ctr[sgt] >= 0) {
                ok = wait_counter_ge(&P.flags->arrive[ph.wait_ctr[sgt]].v,
                                     fill_target(ctl->uses, ph.wait_ctr[sgt], ph.wait_rel[sgt], 1, G), abort_flag, status,
                                     wait_ns, ST_TIMEOUT_ARRIVAL);
                if (!ok) break;
                fence_proxy_async();
              }
              seg_ready |= 1u << sgt;
            }
            if (p_tseg == 1) {
              b_mn0 += segs.off_mn[sgt] - sgt * p_tseg_len;
              if (segs.map[sgt] >= 0) {
                mb = reinterpret_cast<unsigned long long>(&P.maps[segs.map[sgt]]);
                b3 = p_b_mn && P.map3d[segs.map[sgt]];
              }
            } else {
              a_mn0 += segs.off_mn[sgt] - sgt * p_tseg_len;
              if (segs.map[sgt] >= 0) {
                ma_t = reinterpret_cast<unsigned long long>(&P.maps[segs.map[sgt]]);
                a3 = p_a_mn && P.map3d[segs.map[sgt]];
              }
            }
          }
          int ax = (p_a_mn ? a_mn0 : a_k0) + kb0 * a_dx, ay = (p_a_mn ? a_k0 : a_mn0) + kb0 * a_dy;
          int bx = (p_b_mn ? b_mn0 : b_k0) + kb0 * b_dx, by = (p_b_mn ? b_k0 : b_mn0) + kb0 * b_dy;
          // Self-check: a tiled copy must start on a 16-byte boundary in its innermost coordinate (8 elements; a whole
          // 64-element block for the 3-D maps).  A violation is recorded with the phase and the coordinate and the
          // copy is never issued.
          if (((a3 ? (ax & 63) : (ax & 7)) | (b3 ? (bx & 63) : (bx & 7))) != 0) {
            atomicCAS(status, (unsigned long long)ST_OK,
                      (unsigned long long)ST_BAD_ARGUMENT | ((unsigned long long)(p & 0xff) << 8) |
                          ((unsigned long long)(uint32_t)(ax & 0xfffff) << 16) | ((unsigned long long)(uint32_t)(bx & 0xfffff) << 40));
            *abort_flag = 1;
            ok = false;
            break;
          }
          if (P.trace && cta == 0 && tr_n < 60) P.trace[0 * 256 + tr_n * 4 + 0] = globaltimer_ns();
          for (int sg = 0; sg < nseg && ok; ++sg) {
          if (nseg > 1) {
            // next shard of the contraction: its own tensor map, A moves to the matching k-range
            if (!((seg_ready >> sg) & 1u)) {
              if (ph.wait_ctr[sg] >= 0) {
                ok = wait_counter_ge(&P.flags->arrive[ph.wait_ctr[sg]].v,
                                     fill_target(ctl->uses, ph.wait_ctr[sg], ph.wait_rel[sg], 1, G), abort_flag, status,
                                     wait_ns, ST_TIMEOUT_ARRIVAL);
                if (!ok) break;
                fence_proxy_async();
              }
              seg_ready |= 1u << sg;
            }
            mb = reinterpret_cast<unsigned long long>(&P.maps[ph.seg_b_map[sg]]);
            b3 = p_b_mn && P.map3d[ph.seg_b_map[sg]];
            const int ak = a_k0 + ph.seg_a_off_k[sg];
            ax = p_a_mn ? a_mn0 : ak; ay = p_a_mn ? ak : a_mn0;
            bx = p_b_mn ? b_mn0 : b_k0; by = p_b_mn ? b_k0 : b_mn0;
          }
          for (int kb = kb0; kb < kblocks; ++kb) {
            if (!mbar_wait_s(empty_s + stage * 8, phase ^ 1, abort_flag, status, timeout_ns)) { ok = false; break; }
            const uint32_t sa = tiles_s + stage * kStageBytes;
            const uint32_t sb = sa + kABytes;
            issued_mask |= 1u << stage;
            issued_parity = (issued_parity & ~(1u << stage)) | (phase << stage);
            {
              // every CTA (also in a pair) copies into its own shared memory and completes its own barrier
              const uint32_t bar = full_s + stage * 8;
              mbar_arrive_expect_tx_s(bar, tx);
              if (a3) {
                tma_load_3d_s(sa, ma_t, 0, ay, ax >> 6, bar);     // both 64-wide halves of A in one copy
              } else {
                tma_load_2d_s(sa, ma_t, ax, ay, bar);
                if (na == 2) tma_load_2d_s(sa + 8192, ma_t, ax + 64, ay, bar);
              }
              if (b3) {
                tma_load_3d_s(sb, mb, 0, by, bx >> 6, bar);       // all 64-wide column blocks of B in one copy
              } else {
                for (int i = 0; i < nb; ++i) tma_load_2d_s(sb + i * b_ismem, mb, bx + i * b_ix, by + i * b_iy, bar);
              }
            }
            ax += a_dx; ay += a_dy; bx += b_dx; by += b_dy;
            if (++stage == kStages) { stage = 0; phase ^= 1; }
          }
          }
          if (P.trace && cta == 0 && tr_n < 60) P.trace[0 * 256 + tr_n * 4 + 1] = globaltimer_ns();
          ++tr_n;
        }
      }
      if (!ok) {
        // gave up: wait (bounded) until every copy this thread issued has landed before the CTA exits
        {
          for (int s = 0; s < kStages; ++s) {
            if (!((issued_mask >> s) & 1u)) continue;
            unsigned long long t0 = globaltimer_ns();
            while (!mbar_try_wait(&ctl->full[s], (issued_parity >> s) & 1u)) {
              if (globaltimer_ns() - t0 > 2000000ull) break;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ UMMA issuer
    if (!tile_cta) {
      // reserved for pushing: no tiles
    } else if (crank == 0 && elect_one()) {     // in a pair only the leader issues; its UMMAs drive both SMs
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      bool issued_any = false;
      int tr_m = 0;
      const uint32_t tiles_s = smem_u32(tiles);
      const uint32_t full_s = smem_u32(&ctl->full[0]);
      const uint32_t peer_full_s = smem_u32(&ctl->peer_full[0]);
      (void)peer_full_s;
      for (int p = 0; p < P.n_phases && ok; ++p) {
        const RtpPhase& ph = P.phases[p];
        const int tiles_m = (ph.M + TM - 1) / TM;
        const int tiles_n = (ph.N + ph.bn - 1) >> (31 - __clz(ph.bn));   // bn is a power of two
        const int per_batch = tiles_m * tiles_n;
        const int total = per_batch * ph.batch;
        const int kblocks_full = (ph.K + kBK - 1) / kBK;
        const uint32_t idesc = make_idesc_bf16(TM, ph.bn, ph.a_mn, ph.b_mn);
        const uint32_t a_lbo = ph.a_mn ? 8192u : 16u, b_lbo = ph.b_mn ? 8192u : 16u;
        const uint32_t a_kstep16 = ph.a_mn ? 128u : 2u, b_kstep16 = ph.b_mn ? 128u : 2u;   // k-step of 16 elements, in 16-byte units
        const uint64_t da0 = make_smem_desc(0, a_lbo, 1024), db0 = make_smem_desc(0, b_lbo, 1024);
        for (int t = (unit - ph.cta_off + GU) % GU; t < total && ok; t += GU) {
          const int tt = ph.batch == 1 ? t : t % per_batch;
          const int tn = tt / tiles_m;
          const int m0 = (tt - tn * tiles_m) * TM;
          const int n0 = tn * ph.bn;
          if (ph.causal == 1 && n0 > m0 + TM - 1) continue;
          const int kblocks = (ph.causal == 2 ? min(kblocks_full, (m0 + TM + kBK - 1) / kBK) : kblocks_full) *
                              (ph.nseg > 1 ? ph.nseg : 1);      // K-segmented: the segments follow one another
          const int kb0 = ph.causal == 3 ? m0 / kBK : 0;
          if (P.trace && cta == 0 && tr_m < 60) P.trace[1 * 256 + tr_m * 4 + 0] = globaltimer_ns();
          if (!mbar_wait(&ctl->tmem_empty[acc], acc_phase ^ 1, abort_flag, status, timeout_ns)) { ok = false; break; }
          if (P.trace && cta == 0 && tr_m < 60) P.trace[1 * 256 + tr_m * 4 + 1] = globaltimer_ns();
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)(acc * 256);
          for (int kb = kb0; kb < kblocks; ++kb) {
            if (!mbar_wait_s(full_s + stage * 8, phase, abort_flag, status, timeout_ns)) { ok = false; break; }
            if (PAIR && !mbar_try_wait_cluster_s(peer_full_s + stage * 8, phase)) {
              // bounded: the slow path spins on the plain form, then the acquire is repeated once it has flipped
              if (!mbar_wait_slow_s(peer_full_s + stage * 8, phase, abort_flag, status, timeout_ns)) { ok = false; break; }
              mbar_try_wait_cluster_s(peer_full_s + stage * 8, phase);
            }
            tc_fence_after();
            const uint32_t sa = (tiles_s + stage * kStageBytes) >> 4;   // descriptors hold the address in 16-byte units
            const uint32_t sb = sa + (kABytes >> 4);
#pragma unroll
            for (int kk = 0; kk < kBK / 16; ++kk) {
              const uint64_t da = da0 + (uint64_t)(sa + kk * a_kstep16);
              const uint64_t db = db0 + (uint64_t)(sb + kk * b_kstep16);
              if (PAIR) umma_bf16_pair(d_tmem, da, db, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
              else umma_bf16(d_tmem, da, db, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
            }
            issued_any = true;
            // frees the smem stage (in both CTAs of a pair) once these MMAs have read it
            if (PAIR) umma_commit_pair(&ctl->empty[stage]); else umma_commit(&ctl->empty[stage]);
            if (++stage == kStages) { stage = 0; phase ^= 1; }
          }
          if (!ok) break;
          if (PAIR) umma_commit_pair(&ctl->tmem_full[acc]); else umma_commit(&ctl->tmem_full[acc]);
          if (P.trace && cta == 0 && tr_m < 60) P.trace[1 * 256 + tr_m * 4 + 2] = globaltimer_ns();
          ++tr_m;
          if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
      }
      if (!ok && issued_any) {
        // make sure no MMA is still reading smem / writing TMEM before tear-down (a kernel keeps ONE cta_group for all of
        // its tcgen05 instructions: in a pair the commit is the pair form; the second CTA's drain barrier takes the
        // other arrival and nobody waits on it)
        if (PAIR) umma_commit_pair(&ctl->drain); else umma_commit(&ctl->drain);
        unsigned long long t0 = globaltimer_ns();
        while (!mbar_try_wait(&ctl->drain, 0)) {
          if (globaltimer_ns() - t0 > 2000000ull) break;
        }
      }
    } else if (PAIR && crank != 0 && elect_one()) {
      // Relay of the second CTA of a pair: its copies complete its own barriers; one arrive per stage tells the leader's
      // UMMA issuer that this half of the stage is in place.  Walks the same (phase, tile, k-block) sequence.
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint32_t full_s = smem_u32(&ctl->full[0]);
      const uint32_t lead_peer_full = mapa_u32(smem_u32(&ctl->peer_full[0]), 0);
      for (int p = 0; p < P.n_phases && ok; ++p) {
        const RtpPhase& ph = P.phases[p];
        const int tiles_m = (ph.M + TM - 1) / TM;
        const int tiles_n = (ph.N + ph.bn - 1) >> (31 - __clz(ph.bn));   // bn is a power of two
        const int per_batch = tiles_m * tiles_n;
        const int total = per_batch * ph.batch;
        const int kblocks_full = (ph.K + kBK - 1) / kBK;
        for (int t = (unit - ph.cta_off + GU) % GU; t < total && ok; t += GU) {
          const int tt = ph.batch == 1 ? t : t % per_batch;
          const int tn = tt / tiles_m;
          const int m0 = (tt - tn * tiles_m) * TM;
          const int n0 = tn * ph.bn;
          if (ph.causal == 1 && n0 > m0 + TM - 1) continue;
          const int kblocks = (ph.causal == 2 ? min(kblocks_full, (m0 + TM + kBK - 1) / kBK) : kblocks_full) *
                              (ph.nseg > 1 ? ph.nseg : 1);
          const int kb0 = ph.causal == 3 ? m0 / kBK : 0;
          for (int kb = kb0; kb < kblocks; ++kb) {
            if (!mbar_wait_s(full_s + stage * 8, phase, abort_flag, status, timeout_ns)) { ok = false; break; }
            mbar_arrive_cluster(lead_peer_full + stage * 8);   // plain arrive: a cluster-scope release costs about a microsecond here
            if (++stage == kStages) { stage = 0; phase ^= 1; }
          }
        }
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue (4 warps)
    const int quad = warp & 3;  // TMEM lane quadrant this warp may access
    const int epi_tid = (warp - 2) * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    int tr_e = 0;
    for (int p = 0; p < P.n_phases; ++p) {
      const RtpPhase& ph = P.phases[p];
      const int tiles_m = (ph.M + TM - 1) / TM;
      const int tiles_n = (ph.N + ph.bn - 1) >> (31 - __clz(ph.bn));   // bn is a power of two
      const int per_batch = tiles_m * tiles_n;
      const int total = per_batch * ph.batch;
      const bool has_tiles = cta < total;
      const unsigned long long drop_off =
          ph.drop_offset + (ph.drop_step_ptr ? __ldg(ph.drop_step_ptr) * 65536ull : 0ull);
      const bool does_vec = (ph.vec_out != nullptr) && cta == 0;
      (void)has_tiles;
      if (P.trace && cta == 0 && warp == 2 && lane == 0 && p < 16) P.trace[3 * 256 + 128 + p * 4 + 0] = globaltimer_ns();
      if (ok) {
        // Operands of the accumulate / bias reads must have arrived and the destination slot must be free.
        // A CTA without tiles waits too: the counters only mean "every CTA is past fill u" if no CTA
        // publishes its signal for fill u+1 before fill u+1 exists.
        uint32_t good = 1;
        // (a tile-segmented phase waits per tile: the producer for the tile's shard, this warp for the tile's destination)
        if (lane == 0 && !ph.tseg) {
          for (int w = 0; w < RTP_MAX_WAITS && good; ++w)
            if (ph.wait_ctr[w] >= 0)
              good = wait_counter_ge(&P.flags->arrive[ph.wait_ctr[w]].v,
                                     fill_target(ctl->uses, ph.wait_ctr[w], ph.wait_rel[w], 1, G), abort_flag, status,
                                     wait_ns, ST_TIMEOUT_ARRIVAL);
          if (good && ph.credit_ptr)
            good = wait_counter_ge(ph.credit_ptr, credit_target(ctl->uses, ph.credit_ctr, ph.credit_rel),
                                   abort_flag, status, wait_ns, ST_TIMEOUT_CREDIT);
        }
        good = __shfl_sync(0xffffffffu, good, 0);
        if (!good) ok = false;
      }
      if (P.trace && cta == 0 && warp == 2 && lane == 0 && p < 16) P.trace[3 * 256 + 128 + p * 4 + 1] = globaltimer_ns();
      if (ok && ph.kind == RTP_KIND_GATHER) {
        // embedding rows of the visiting table shard -> column block of the output
        const int per_row = ph.g_cols >> 3;
        const long long items = (long long)ph.g_tokens * per_row;
        const __nv_bfloat16* table = reinterpret_cast<const __nv_bfloat16*>(ph.g_table);
        const __nv_bfloat16* pe = reinterpret_cast<const __nv_bfloat16*>(ph.g_pe);
        __nv_bfloat16* outp = reinterpret_cast<__nv_bfloat16*>(ph.d);
        for (long long it = (long long)cta * 128 + epi_tid; it < items; it += (long long)G * 128) {
          const int t = (int)(it / per_row), c = (int)(it % per_row) * 8;
          uint4 raw = __ldcg(reinterpret_cast<const uint4*>(table + (size_t)ph.g_ids[t] * ph.g_cols + c));
          float v[8] = {bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y),
                        bf16_lo(raw.z), bf16_hi(raw.z), bf16_lo(raw.w), bf16_hi(raw.w)};
#pragma unroll
          for (int k = 0; k < 8; ++k) v[k] *= ph.g_scale;
          if (pe) {
            uint4 pr = *reinterpret_cast<const uint4*>(pe + (size_t)(t / ph.g_tpp) * ph.g_ldpe + ph.g_col_off + c);
            v[0] += bf16_lo(pr.x); v[1] += bf16_hi(pr.x); v[2] += bf16_lo(pr.y); v[3] += bf16_hi(pr.y);
            v[4] += bf16_lo(pr.z); v[5] += bf16_hi(pr.z); v[6] += bf16_lo(pr.w); v[7] += bf16_hi(pr.w);
          }
          if (ph.drop_thresh) {
            const unsigned long long e = (unsigned long long)t * ph.g_dim + ph.g_col_off + c;
            uint4 r0 = philox4x32(ph.drop_seed, drop_off, e >> 2), r1 = philox4x32(ph.drop_seed, drop_off, (e >> 2) + 1);
            const uint32_t rw[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = rw[k] >= ph.drop_thresh ? v[k] * ph.drop_scale : 0.f;
          }
          *reinterpret_cast<uint4*>(outp + (size_t)t * ph.ldd + c) =
              make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
        }
      } else if (ok && ph.kind == RTP_KIND_VECADD) {
        const int per_row = ph.v_cols >> 3;
        const long long items = (long long)ph.v_rows * per_row;
        const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(ph.v_src);
        const __nv_bfloat16* cin = reinterpret_cast<const __nv_bfloat16*>(ph.c);
        __nv_bfloat16* outp = reinterpret_cast<__nv_bfloat16*>(ph.d);
        for (long long it = (long long)cta * 128 + epi_tid; it < items; it += (long long)G * 128) {
          const long long r = it / per_row;
          const int c = (int)(it % per_row) * 8;
          uint4 a = *reinterpret_cast<const uint4*>(src + r * ph.v_ld + c);
          float v[8] = {bf16_lo(a.x), bf16_hi(a.x), bf16_lo(a.y), bf16_hi(a.y),
                        bf16_lo(a.z), bf16_hi(a.z), bf16_lo(a.w), bf16_hi(a.w)};
          if (cin) {
            uint4 b = __ldcg(reinterpret_cast<const uint4*>(cin + r * ph.v_cols + c));
            v[0] += bf16_lo(b.x); v[1] += bf16_hi(b.x); v[2] += bf16_lo(b.y); v[3] += bf16_hi(b.y);
            v[4] += bf16_lo(b.z); v[5] += bf16_hi(b.z); v[6] += bf16_lo(b.w); v[7] += bf16_hi(b.w);
          }
          *reinterpret_cast<uint4*>(outp + r * ph.v_cols + c) =
              make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
        }
      }
      if (ok && ph.kind == RTP_KIND_REDUCE) {
        const long long items = ph.r_n >> 3;
        __nv_bfloat16* outp = reinterpret_cast<__nv_bfloat16*>(ph.d);
        const int nsrc = ph.r_nsrc;
        const uint4* srcs[RTP_NUM_SLOTS];
#pragma unroll
        for (int k = 0; k < RTP_NUM_SLOTS; ++k) srcs[k] = reinterpret_cast<const uint4*>(ph.r_src[k < nsrc ? k : 0]);
        // two items per thread and every source in flight at once (the loads are predicated, not looped over)
        const long long stride = (long long)G * 128;
        for (long long it = (long long)cta * 128 + epi_tid; it < items; it += 2 * stride) {
          const long long it1 = it + stride;
          const bool two = it1 < items;
          uint4 a[RTP_NUM_SLOTS], b[RTP_NUM_SLOTS];
#pragma unroll
          for (int k = 0; k < RTP_NUM_SLOTS; ++k) {
            a[k] = make_uint4(0u, 0u, 0u, 0u);
            b[k] = make_uint4(0u, 0u, 0u, 0u);
            if (k < nsrc) {
              a[k] = __ldcg(srcs[k] + it);
              if (two) b[k] = __ldcg(srcs[k] + it1);
            }
          }
          float s0[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, s1[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int k = 0; k < RTP_NUM_SLOTS; ++k) {
            s0[0] += bf16_lo(a[k].x); s0[1] += bf16_hi(a[k].x); s0[2] += bf16_lo(a[k].y); s0[3] += bf16_hi(a[k].y);
            s0[4] += bf16_lo(a[k].z); s0[5] += bf16_hi(a[k].z); s0[6] += bf16_lo(a[k].w); s0[7] += bf16_hi(a[k].w);
            s1[0] += bf16_lo(b[k].x); s1[1] += bf16_hi(b[k].x); s1[2] += bf16_lo(b[k].y); s1[3] += bf16_hi(b[k].y);
            s1[4] += bf16_lo(b[k].z); s1[5] += bf16_hi(b[k].z); s1[6] += bf16_lo(b[k].w); s1[7] += bf16_hi(b[k].w);
          }
          *reinterpret_cast<uint4*>(outp + it * 8) = make_uint4(pack_bf16(s0[0], s0[1]), pack_bf16(s0[2], s0[3]),
                                                                 pack_bf16(s0[4], s0[5]), pack_bf16(s0[6], s0[7]));
          if (two)
            *reinterpret_cast<uint4*>(outp + it1 * 8) = make_uint4(pack_bf16(s1[0], s1[1]), pack_bf16(s1[2], s1[3]),
                                                                    pack_bf16(s1[4], s1[5]), pack_bf16(s1[6], s1[7]));
        }
      }
      // phase fields used per element live in registers (reading them from parameter space inside the loops costs a
      // dependent constant load each time)
      const int p_M = ph.M;
      const int p_N = ph.N;
      const int e_bn = ph.bn;
      const int p_tseg = ph.tseg, p_tseg_len = ph.tseg_len;
      const RtpSegTable& segs = P.segtab[ph.tseg_tab];
      uint32_t cred_ready = 0;        // segments whose destination has been seen to be free
      const float e_alpha = ph.alpha;
      const const void* e_c = ph.c;
      const long long e_ldc = ph.ldc;
      const int e_c_fp32 = ph.c_fp32;
      const void* const p_bias = ph.bias;
      const int e_nbias_more = ph.n_bias_more;
      const int e_act = ph.act;
      const const void* e_mask = ph.mask;
      const long long e_ldmask = ph.ldmask;
      const float e_mask_scale = ph.mask_scale;
      const uint32_t e_drop_thresh = ph.drop_thresh;
      const float e_drop_scale = ph.drop_scale;
      const unsigned long long e_drop_seed = ph.drop_seed;
      void* const p_d = ph.d;
      const long long e_ldd = ph.ldd;
      const int e_d_fp32 = ph.d_fp32;
      const int e_vec_ok = ph.vec_ok;
      const int e_causal = ph.causal;
      const int e_batch_inner = ph.batch_inner;
      const long long e_d_bo = ph.d_bo;
      const long long e_d_bi = ph.d_bi;
      const long long e_c_bo = ph.c_bo;
      const long long e_c_bi = ph.c_bi;
      const int e_cta_off = ph.cta_off;
      // vector accesses of the straight-line path: operands 16-byte aligned (vec_ok), bias too, dropout index a multiple of 4
      bool e_bias_al = !p_bias || (reinterpret_cast<uintptr_t>(p_bias) & 15) == 0;
      for (int nb = 0; nb < e_nbias_more; ++nb) e_bias_al = e_bias_al && (reinterpret_cast<uintptr_t>(ph.bias_more[nb]) & 15) == 0;
      if (p_tseg)
        for (int sgi = 0; sgi < ph.tseg_n; ++sgi)
          e_bias_al = e_bias_al && (reinterpret_cast<uintptr_t>(segs.bias[sgi]) & 15) == 0 &&
                      (reinterpret_cast<uintptr_t>(segs.d[sgi]) & 15) == 0;
      const bool e_fast_ok = e_vec_ok && e_bias_al && (!e_drop_thresh || ((p_tseg == 1 ? p_tseg_len : p_N) & 3) == 0);
      for (int t = tile_cta ? (unit - e_cta_off + GU) % GU : total; t < total && ok; t += GU) {
        const bool e_batch1 = e_batch_inner == 1 && per_batch == total;
        const int z = e_batch1 ? 0 : t / per_batch, tt = e_batch1 ? t : t - z * per_batch;
        const int tn = tt / tiles_m;
        int m0u = (tt - tn * tiles_m) * TM;
        int n0 = tn * e_bn;
        if (e_causal == 1 && n0 > m0u + TM - 1) continue;
        // Tile-segmented phase: from here on the tile lives in its segment's coordinates (local row / column, the
        // segment's destination, bias and extent).
        int e_M = p_M, e_N = p_N;
        void* e_d = p_d;
        const void* e_bias = p_bias;
        unsigned long long drop_off_t = drop_off;
        int sgt = 0;
        if (p_tseg) {
          sgt = (p_tseg == 1 ? n0 : m0u) / p_tseg_len;
          if (p_tseg == 1) { n0 -= sgt * p_tseg_len; e_N = p_tseg_len; }
          else { m0u -= sgt * p_tseg_len; e_M = p_tseg_len; }
          e_d = segs.d[sgt];
          e_bias = segs.bias[sgt];
          drop_off_t += (unsigned long long)segs.drop_add[sgt];
        }
        const int m0 = m0u + (int)crank * kBM;
        const long long zoff_d = e_batch1 ? 0ll : (long long)(z / e_batch_inner) * e_d_bo + (long long)(z % e_batch_inner) * e_d_bi;
        const long long zoff_c = e_batch1 ? 0ll : (long long)(z / e_batch_inner) * e_c_bo + (long long)(z % e_batch_inner) * e_c_bi;
        uint32_t good = 1;
        const bool tr_on = P.trace && cta == 0 && warp == 2 && lane == 0 && tr_e < 60;
        if (tr_on) P.trace[2 * 256 + tr_e * 4 + 0] = globaltimer_ns();
        if (lane == 0) good = mbar_wait(&ctl->tmem_full[acc], acc_phase, abort_flag, status, timeout_ns);
        good = __shfl_sync(0xffffffffu, good, 0);
        if (!good) { ok = false; break; }
        if (p_tseg && segs.credit_ptr[sgt] && !((cred_ready >> sgt) & 1u)) {
          // first tile of this CTA for the segment: the destination slot must have been read by its owner
          if (lane == 0)
            good = wait_counter_ge(segs.credit_ptr[sgt], credit_target(ctl->uses, segs.credit_ctr[sgt], 0), abort_flag, status,
                                   wait_ns, ST_TIMEOUT_CREDIT);
          good = __shfl_sync(0xffffffffu, good, 0);
          if (!good) { ok = false; break; }
          cred_ready |= 1u << sgt;
        }
        tc_fence_after();
        if (tr_on) P.trace[2 * 256 + tr_e * 4 + 1] = globaltimer_ns();
        const int row = m0 + quad * 32 + lane;
        const bool row_ok = row < e_M;
        const bool interior = (m0 + kBM <= e_M) && (n0 + e_bn <= e_N);
        const bool fast = interior && e_fast_ok;
        const bool staged = !fast && !e_d_fp32 && e_vec_ok && (e_N & 7) == 0;
        uint8_t* stg = staging + (warp - 2) * (32 * kStagePitch);
        for (int cb = 0; cb < e_bn / 32; ++cb) {
          uint32_t r[32];
          __syncwarp();
          const bool tr_cb = tr_on && tr_e == 1 && cb < 8;
          if (tr_cb) P.trace[3 * 256 + cb * 4 + 0] = globaltimer_ns();
          tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * 256 + cb * 32), r);
          tmem_ld_wait();
          if (tr_cb) P.trace[3 * 256 + cb * 4 + 1] = globaltimer_ns();
          const int col0 = n0 + cb * 32;
          if (fast) {
            // Interior tile with 16-byte aligned operands: straight-line code on the whole 32-column chunk, one branch
            // per epilogue feature.  (The per-group code below handles edges and unaligned operands.)
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * e_alpha;
            if (e_c) {
              if (e_c_fp32) {
                const float4* cp = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(e_c) + zoff_c +
                                                                   (long long)row * e_ldc + col0);
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                  const float4 c = __ldcg(cp + q);
                  v[4 * q] += c.x; v[4 * q + 1] += c.y; v[4 * q + 2] += c.z; v[4 * q + 3] += c.w;
                }
              } else {
                const uint4* cp = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(e_c) + zoff_c +
                                                                 (long long)row * e_ldc + col0);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const uint4 c = __ldcg(cp + q);
                  v[8 * q] += bf16_lo(c.x); v[8 * q + 1] += bf16_hi(c.x); v[8 * q + 2] += bf16_lo(c.y);
                  v[8 * q + 3] += bf16_hi(c.y); v[8 * q + 4] += bf16_lo(c.z); v[8 * q + 5] += bf16_hi(c.z);
                  v[8 * q + 6] += bf16_lo(c.w); v[8 * q + 7] += bf16_hi(c.w);
                }
              }
            }
            if (e_bias) {
              for (int nb = 0; nb <= e_nbias_more; ++nb) {
                const void* bsrc = nb == 0 ? e_bias : ph.bias_more[nb - 1];
                const uint4* bp = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(bsrc) + col0);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const uint4 b = __ldcg(bp + q);
                  v[8 * q] += bf16_lo(b.x); v[8 * q + 1] += bf16_hi(b.x); v[8 * q + 2] += bf16_lo(b.y);
                  v[8 * q + 3] += bf16_hi(b.y); v[8 * q + 4] += bf16_lo(b.z); v[8 * q + 5] += bf16_hi(b.z);
                  v[8 * q + 6] += bf16_lo(b.w); v[8 * q + 7] += bf16_hi(b.w);
                }
              }
            }
            if (e_act == 1) {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = fmaxf(v[i], 0.f);
            } else if (e_act == 2) {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = 0.5f * v[i] * (1.f + erff(v[i] * 0.70710678118654752f));
            }
            if (e_mask) {
              const uint4* mp = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(e_mask) +
                                                               (long long)row * e_ldmask + col0);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint4 m = __ldcg(mp + q);
                const uint32_t mw[4] = {m.x, m.y, m.z, m.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  v[8 * q + 2 * i] = bf16_lo(mw[i]) > 0.f ? v[8 * q + 2 * i] * e_mask_scale : 0.f;
                  v[8 * q + 2 * i + 1] = bf16_hi(mw[i]) > 0.f ? v[8 * q + 2 * i + 1] * e_mask_scale : 0.f;
                }
              }
            }
            if (e_drop_thresh) {
              const unsigned long long e4 =
                  ((unsigned long long)row * (unsigned long long)e_N + (unsigned long long)col0) >> 2;
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                const uint4 rr = philox4x32(e_drop_seed, drop_off_t, e4 + q);
                v[4 * q] = rr.x >= e_drop_thresh ? v[4 * q] * e_drop_scale : 0.f;
                v[4 * q + 1] = rr.y >= e_drop_thresh ? v[4 * q + 1] * e_drop_scale : 0.f;
                v[4 * q + 2] = rr.z >= e_drop_thresh ? v[4 * q + 2] * e_drop_scale : 0.f;
                v[4 * q + 3] = rr.w >= e_drop_thresh ? v[4 * q + 3] * e_drop_scale : 0.f;
              }
            }
            if (e_d_fp32) {
              float4* dp = reinterpret_cast<float4*>(reinterpret_cast<float*>(e_d) + zoff_d + (long long)row * e_ldd + col0);
#pragma unroll
              for (int q = 0; q < 8; ++q) dp[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            } else {
              uint8_t* sp = stg + lane * kStagePitch + (cb & 1) * 64;
#pragma unroll
              for (int q = 0; q < 4; ++q)
                *reinterpret_cast<uint4*>(sp + q * 16) =
                    make_uint4(pack_bf16(v[8 * q], v[8 * q + 1]), pack_bf16(v[8 * q + 2], v[8 * q + 3]),
                               pack_bf16(v[8 * q + 4], v[8 * q + 5]), pack_bf16(v[8 * q + 6], v[8 * q + 7]));
            }
          } else if (row_ok && col0 < e_N) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {  // groups of 8 columns
            const int col = col0 + g * 8;
            if (col >= e_N) break;
            const int nvalid = min(8, e_N - col);
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[g * 8 + i]) * e_alpha;
            const bool vec = e_vec_ok && nvalid == 8;
            if (e_c) {
              if (e_c_fp32) {
                const float* cp = reinterpret_cast<const float*>(e_c) + zoff_c + (long long)row * e_ldc + col;
                if (vec) {
                  float4 c0 = __ldcg(reinterpret_cast<const float4*>(cp));
                  float4 c1 = __ldcg(reinterpret_cast<const float4*>(cp) + 1);
                  v[0] += c0.x; v[1] += c0.y; v[2] += c0.z; v[3] += c0.w;
                  v[4] += c1.x; v[5] += c1.y; v[6] += c1.z; v[7] += c1.w;
                } else {
                  for (int i = 0; i < nvalid; ++i) v[i] += __ldcg(cp + i);
                }
              } else {
                const __nv_bfloat16* cp = reinterpret_cast<const __nv_bfloat16*>(e_c) + zoff_c + (long long)row * e_ldc + col;
                if (vec) {
                  uint4 c = __ldcg(reinterpret_cast<const uint4*>(cp));
                  v[0] += bf16_lo(c.x); v[1] += bf16_hi(c.x); v[2] += bf16_lo(c.y); v[3] += bf16_hi(c.y);
                  v[4] += bf16_lo(c.z); v[5] += bf16_hi(c.z); v[6] += bf16_lo(c.w); v[7] += bf16_hi(c.w);
                } else {
                  for (int i = 0; i < nvalid; ++i)
                    v[i] += __bfloat162float(__ldcg(cp + i));
                }
              }
            }
            if (e_bias) {
              for (int nb = 0; nb <= e_nbias_more; ++nb) {
                const __nv_bfloat16* bp = reinterpret_cast<const __nv_bfloat16*>(nb == 0 ? e_bias : ph.bias_more[nb - 1]) + col;
                if (nvalid == 8 && (reinterpret_cast<uintptr_t>(bp) & 15) == 0) {
                  const uint4 b = __ldcg(reinterpret_cast<const uint4*>(bp));   // one 16-byte load for 8 columns
                  v[0] += bf16_lo(b.x); v[1] += bf16_hi(b.x); v[2] += bf16_lo(b.y); v[3] += bf16_hi(b.y);
                  v[4] += bf16_lo(b.z); v[5] += bf16_hi(b.z); v[6] += bf16_lo(b.w); v[7] += bf16_hi(b.w);
                } else {
                  for (int i = 0; i < nvalid; ++i) v[i] += __bfloat162float(__ldcg(bp + i));
                }
              }
            }
            if (e_act == 1) {
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] = fmaxf(v[i], 0.f);
            } else if (e_act == 2) {
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] = 0.5f * v[i] * (1.f + erff(v[i] * 0.70710678118654752f));
            }
            if (e_mask) {
              const __nv_bfloat16* mp = reinterpret_cast<const __nv_bfloat16*>(e_mask) + (long long)row * e_ldmask + col;
              if (vec) {
                uint4 m = __ldcg(reinterpret_cast<const uint4*>(mp));
                const uint32_t mw[4] = {m.x, m.y, m.z, m.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  v[2 * i] = bf16_lo(mw[i]) > 0.f ? v[2 * i] * e_mask_scale : 0.f;
                  v[2 * i + 1] = bf16_hi(mw[i]) > 0.f ? v[2 * i + 1] * e_mask_scale : 0.f;
                }
              } else {
                for (int i = 0; i < nvalid; ++i)
                  v[i] = __bfloat162float(__ldcg(mp + i)) > 0.f ? v[i] * e_mask_scale : 0.f;
              }
            }
            if (e_drop_thresh) {
              // element index = position in the logical [M, N] output; 8 | col so two philox calls cover the group
              const unsigned long long e = (unsigned long long)row * (unsigned long long)e_N + (unsigned long long)col;
              uint4 r0 = philox4x32(e_drop_seed, drop_off_t, e >> 2);
              uint4 r1 = philox4x32(e_drop_seed, drop_off_t, (e >> 2) + 1);
              const uint32_t rw[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] = rw[i] >= e_drop_thresh ? v[i] * e_drop_scale : 0.f;
            }
            if (e_d_fp32) {
              float* dp = reinterpret_cast<float*>(e_d) + zoff_d + (long long)row * e_ldd + col;
              if (vec) {
                reinterpret_cast<float4*>(dp)[0] = make_float4(v[0], v[1], v[2], v[3]);
                reinterpret_cast<float4*>(dp)[1] = make_float4(v[4], v[5], v[6], v[7]);
              } else {
                for (int i = 0; i < nvalid; ++i) dp[i] = v[i];
              }
            } else if (staged) {
              // park the 16 bytes in this warp's staging rows; they leave the SM as full 128-byte lines below
              *reinterpret_cast<uint4*>(stg + lane * kStagePitch + (cb & 1) * 64 + g * 16) =
                  make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
            } else {
              __nv_bfloat16* dp = reinterpret_cast<__nv_bfloat16*>(e_d) + zoff_d + (long long)row * e_ldd + col;
              if (vec) {
                *reinterpret_cast<uint4*>(dp) =
                    make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
              } else {
                for (int i = 0; i < nvalid; ++i) dp[i] = __float2bfloat16(v[i]);
              }
            }
          }
          }
          if (tr_cb) P.trace[3 * 256 + cb * 4 + 2] = globaltimer_ns();
          if (fast && !e_d_fp32 && (cb & 1)) {
            // coalesced write-out of 32 rows x 64 columns: 8 lanes cover one row's 128 bytes, 4 rows per instruction
            __syncwarp();
            __nv_bfloat16* dp = reinterpret_cast<__nv_bfloat16*>(e_d) + zoff_d +
                                (long long)(m0 + quad * 32 + (lane >> 3)) * e_ldd + n0 + (cb - 1) * 32 + (lane & 7) * 8;
            const uint8_t* sp = stg + (lane >> 3) * kStagePitch + (lane & 7) * 16;
#pragma unroll
            for (int k = 0; k < 8; ++k)
              *reinterpret_cast<uint4*>(dp + (long long)(k * 4) * e_ldd) =
                  *reinterpret_cast<const uint4*>(sp + k * 4 * kStagePitch);
            __syncwarp();
          } else if (staged && (cb & 1)) {
            __syncwarp();
            const int pair_col0 = n0 + (cb - 1) * 32;
            __nv_bfloat16* dbase = reinterpret_cast<__nv_bfloat16*>(e_d) + zoff_d;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const int rr = k * 4 + (lane >> 3);
              const int grow = m0 + quad * 32 + rr;
              const int gcol = pair_col0 + (lane & 7) * 8;
              if (grow < e_M && gcol < e_N) {
                const uint4 val = *reinterpret_cast<const uint4*>(stg + rr * kStagePitch + (lane & 7) * 16);
                *reinterpret_cast<uint4*>(dbase + (long long)grow * e_ldd + gcol) = val;
              }
            }
            __syncwarp();
          }
          if (tr_cb) P.trace[3 * 256 + cb * 4 + 3] = globaltimer_ns();
        }
        tc_fence_before();
        __syncwarp();
        if (tr_on) P.trace[2 * 256 + tr_e * 4 + 2] = globaltimer_ns();
        ++tr_e;
        if (lane == 0) {
          if (PAIR && crank != 0) mbar_arrive_cluster(mapa_u32(smem_u32(&ctl->tmem_empty[acc]), 0));
          else mbar_arrive(&ctl->tmem_empty[acc]);
        }
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      // small vector job (bias-gradient hop) by CTA 0
      if (ok && cta == 0 && p_tseg) {
        // bias-gradient rows of every segment (fp32 column sums -> the segment's destination)
        for (int sgi = 0; sgi < ph.tseg_n; ++sgi) {
          if (!segs.vec_out[sgi]) continue;
          if (segs.credit_ptr[sgi] && !((cred_ready >> sgi) & 1u)) {
            uint32_t good = 1;
            if (lane == 0)
              good = wait_counter_ge(segs.credit_ptr[sgi], credit_target(ctl->uses, segs.credit_ctr[sgi], 0), abort_flag, status,
                                     wait_ns, ST_TIMEOUT_CREDIT);
            good = __shfl_sync(0xffffffffu, good, 0);
            if (!good) { ok = false; break; }
            cred_ready |= 1u << sgi;
          }
          __nv_bfloat16* vo = reinterpret_cast<__nv_bfloat16*>(segs.vec_out[sgi]);
          const float* va = ph.vec_add + segs.vec_off[sgi];
          for (int i = epi_tid; i < ph.vec_len; i += 128) vo[i] = __float2bfloat16(va[i]);
        }
      }
      if (ok && does_vec) {
        for (int i = epi_tid; i < ph.vec_len; i += 128) {
          float x = ph.vec_add[i];
          if (ph.vec_in) {
            x += ph.vec_fp32 ? __ldcg(reinterpret_cast<const float*>(ph.vec_in) + i)
                             : __bfloat162float(__ldcg(reinterpret_cast<const __nv_bfloat16*>(ph.vec_in) + i));
          }
          if (ph.vec_fp32) reinterpret_cast<float*>(ph.vec_out)[i] = x;
          else reinterpret_cast<__nv_bfloat16*>(ph.vec_out)[i] = __float2bfloat16(x);
        }
      }
      if (P.trace && cta == 0 && warp == 2 && lane == 0 && p < 16) P.trace[3 * 256 + 128 + p * 4 + 2] = globaltimer_ns();
      // phase end: publish "read done" / "data arrived". Every CTA signals, also one without tiles.
      bool signals = ph.arrive_ptr != nullptr;
      for (int w = 0; w < RTP_MAX_WAITS; ++w) signals = signals || ph.done_ctr[w] >= 0;
      if (signals) {
        // All four epilogue warps are through with the phase.
        asm volatile("bar.sync 1, 128;" ::: "memory");
        // "read done": the operands have been consumed, nothing written by this CTA has to be visible first
        // The CTA that completes the count of a fill (every CTA reports once per fill) tells all other ranks: whoever
        // writes this slot next finds the credit in its own memory.
        if (epi_tid == 0 && ok)
          for (int w = 0; w < RTP_MAX_WAITS; ++w)
            if (ph.done_ctr[w] >= 0) {
              const int c = ph.done_ctr[w];
              const unsigned long long old = atomicAdd(&P.flags->done[c].v, 1ull);
              if ((old + 1ull) % (unsigned long long)G == 0ull)
                for (int t = 0; t < P.world; ++t)     // this rank included: it may be the next writer of its own slot
                  red_relaxed_sys_add(&P.peer_flags[t]->credit[P.rank][c].v, 1ull);
            }
        // "data arrived": the tiles stored by this CTA (possibly into a peer's memory) must be visible first.  Waiting
        // for the NVLink stores to be acknowledged costs microseconds, so the release fence and the signal are handed
        // to the signaller warp through a CTA-wide counter (a counter, not a barrier: this warp may be several phases
        // ahead of the signaller).  The chain "stores of the four warps -> bar.sync 1 -> release of the counter ->
        // acquire by the signaller" orders them before its fence.
        if (ph.arrive_ptr && epi_tid == 0) {
          __threadfence_block();
          atomicAdd(&ctl->handed, 1u);
        }
      }
      if (P.trace && cta == 0 && warp == 2 && lane == 0 && p < 16) P.trace[3 * 256 + 128 + p * 4 + 3] = globaltimer_ns();
    }
  } else if (warp == 6) {
    // ------------------------------------------------------------------ pusher (one elected thread)
    // CTAs [n_compute, G) are reserved for pushing when the program has push jobs: they own no GEMM tile, so their copy
    // engine is not shared with a tile pipeline and their tile memory serves as a deep ring.  Without reserved CTAs
    // every CTA moves 1/G of each job through its small ring.
    if (P.n_pushes > 0 && P.push_ring == 2 && !(P.n_compute > 0 && P.n_compute < G)) {
      PushCtx pc;
      pc.P = &P; pc.G = G; pc.cta = cta;
      pc.abort_flag = abort_flag; pc.status = status; pc.wait_ns = wait_ns; pc.timeout_ns = timeout_ns;
      pc.uses = ctl->uses;
      pc.bars = nullptr; pc.ring = nullptr; pc.index = cta; pc.sharers = G;
      run_pushes_stores(pc, ctl, lane);
    } else if (elect_one() && P.n_pushes > 0) {
      const int n_comp = P.n_compute > 0 ? P.n_compute : G;
      PushCtx pc;
      pc.P = &P; pc.G = G; pc.cta = cta;
      pc.abort_flag = abort_flag; pc.status = status; pc.wait_ns = wait_ns; pc.timeout_ns = timeout_ns;
      pc.uses = ctl->uses;
      pc.bars = &ctl->push_full[0];
      if (n_comp < G) {
        if (cta < n_comp) {
          // nothing to move: count this CTA in for every fill right away (the fill is complete only when the CTAs that
          // do write have counted themselves in, after their stores)
          for (int j = 0; j < P.n_pushes; ++j)
            if (P.pushes[j].arrive_ptr) red_relaxed_sys_add(P.pushes[j].arrive_ptr, 1ull);
        } else {
          pc.ring = tiles; pc.index = cta - n_comp; pc.sharers = G - n_comp;
          run_pushes<kMaxPushSlots, kBigPushChunk, 6>(pc);
        }
      } else {
        pc.ring = staging + kStagingBytes; pc.index = cta; pc.sharers = G;
        // LAG = how many newer copies may be outstanding when a job's completion is awaited.  The wait blocks the one
        // issuing thread, so a small LAG stalls the stream whenever a completion is slow (8-way exchange: ~10 us); a
        // large one announces small jobs only after everything has been issued.
        if (P.push_ring == 1) run_pushes<2, 2 * kPushChunk, 1>(pc);
        else if (P.push_ring == 3) run_pushes<kPushSlots, kPushChunk, 12>(pc);
        else if (P.push_ring == 4) run_pushes<2, 2 * kPushChunk, 8>(pc);
        else run_pushes<kPushSlots, kPushChunk, kPushSlots - 1>(pc);
      }
    }
  }
  else if (warp == 7) {
    // ------------------------------------------------------------------ signaller
    // For every phase that announces its output to another rank: wait until the epilogue warps have handed the phase
    // over, issue ONE cumulative system-scope release fence (it completes when the CTA's stores, NVLink ones included,
    // have been acknowledged) and bump the consumer's arrival counter.  The epilogue warps are already at work on the
    // next phase meanwhile.
    if (lane == 0) {
      // phases that announce their output, in program order
      int n_sig = 0;
      for (int p = 0; p < P.n_phases; ++p) n_sig += P.phases[p].arrive_ptr != nullptr;
      // push jobs come this way too when the pusher warp works with plain stores (it only ISSUES them)
      const int n_jobs = (P.push_ring == 2 && !(P.n_compute > 0 && P.n_compute < G)) ? P.n_pushes : 0;
      int next_p = 0;         // next phase index to look at
      uint32_t sent = 0;      // announcing phases signalled so far
      uint32_t jsent = 0;     // push jobs signalled so far
      while ((int)sent < n_sig || (int)jsent < n_jobs) {
        // bounded: the epilogue warps hand every such phase over and the pusher warp every job, also after an abort
        const unsigned long long t0 = globaltimer_ns();
        uint32_t have = 0, jhave = 0;
        bool got = true;
        while (true) {
          have = *reinterpret_cast<volatile uint32_t*>(&ctl->handed);
          jhave = *reinterpret_cast<volatile uint32_t*>(&ctl->jobs_issued);
          if (have > sent || jhave > jsent) break;
          if (globaltimer_ns() - t0 > 2 * timeout_ns) { got = false; break; }
          __nanosleep(32);
        }
        if (!got) break;
        __threadfence_block();
        // ONE fence covers every phase handed over so far (a fence waits a link round trip: never one per phase)
        const bool live = !*abort_flag;
        if (live) __threadfence_system();
        while (sent < have) {
          while (P.phases[next_p].arrive_ptr == nullptr) ++next_p;
          const RtpPhase& sp = P.phases[next_p];
          if (live) {
            if (sp.tseg) {
              // a tile-segmented phase announces every segment's destination
              const RtpSegTable& st = P.segtab[sp.tseg_tab];
              for (int i = 0; i < sp.tseg_n; ++i)
                if (st.arrive_ptr[i]) red_relaxed_sys_add(st.arrive_ptr[i], 1ull);
            } else {
              red_relaxed_sys_add(sp.arrive_ptr, 1ull);
            }
          }
          ++next_p;
          ++sent;
        }
        for (; jsent < jhave; ++jsent) {
          if (live && P.pushes[jsent].arrive_ptr) red_relaxed_sys_add(P.pushes[jsent].arrive_ptr, 1ull);
          if (P.trace && cta == 0 && jsent < 8) P.trace[3 * 256 + 200 + jsent * 4 + 2] = globaltimer_ns();
        }
      }
    }
  }

  // ---------------------------------------------------------------------- tear-down
  if (threadIdx.x == 64) GEMM_STAMP(4);
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) GEMM_STAMP(5);
  if (PAIR) cluster_sync_all();      // neither CTA leaves while the other may still signal its barriers or read its smem
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, kTmemCols); else tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 32) GEMM_STAMP(6);
  if (threadIdx.x == 0 && P.flags) {
    __threadfence();
    unsigned long long prev = atomicAdd(&P.flags->done_ctas.v, 1ull);
    if (prev == (unsigned long long)(G - 1)) {
      for (int k = 0; k < RTP_NUM_CTR; ++k) P.flags->uses[k].v += (unsigned long long)P.uses_inc[k];
      P.flags->done_ctas.v = 0;
      __threadfence();
    }
  }
}

}  // namespace rtp
