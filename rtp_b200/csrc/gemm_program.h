// Host/device description of one launch of the rotation GEMM kernel.
//
// A launch executes a small *program*: an ordered list of GEMM phases (each a tiled
// D = epilogue(A * B^T) over tcgen05 tensor cores) and an ordered list of push jobs (bulk copies of a
// weight shard into a peer GPU's workspace slot).  Phases and pushes synchronise with other ranks
// only through monotonically increasing 64-bit counters that live in each rank's peer-mapped flag
// block; a plain single-GPU GEMM is a program with one phase, no pushes and no counters.
#pragma once
#include <cuda.h>
#include <stdint.h>

#define RTP_MAX_MAPS 12
#define RTP_MAX_PHASES 18
#define RTP_MAX_PUSHES 16
#define RTP_MAX_EMU_RANKS 4

// indices into FlagBlock::arrive / ::done / ::uses
#define RTP_NUM_SLOTS 8            // slots per bank: two banks of weight slots (W0..W7, W8..W15) and gradient slots G0..G7
#define RTP_NUM_WBANKS 2           // a launch reads the weight shards of one bank while the next launch's shards arrive in the other
#define RTP_CTR_W0 0
#define RTP_CTR_G0 (RTP_NUM_WBANKS * RTP_NUM_SLOTS)
#define RTP_NUM_CTR (RTP_CTR_G0 + RTP_NUM_SLOTS)
#define RTP_FLAG_BYTES 65536       // bytes reserved for the flag block at the start of a workspace
#define RTP_FLAG_MAX_WORLD 8
#define RTP_MAX_WAITS 8

// Per-rank flag block (peer-mapped). Every word sits in its own 128-byte line.
struct alignas(128) RtpFlagWord {
  unsigned long long v;
  unsigned long long pad[15];
};
struct RtpFlagBlock {
  RtpFlagWord arrive[RTP_NUM_CTR];  // bumped by the producer's CTAs after their stores into the slot
  RtpFlagWord done[RTP_NUM_CTR];    // bumped (locally) by this rank's CTAs once they finished reading the slot
  RtpFlagWord uses[RTP_NUM_CTR];    // number of completed fills of the slot (same on every rank)
  // credit[t][c]: how many fills of slot c of RANK t have been read completely.  Written by rank t (the CTA that
  // completes a fill's `done` count tells every other rank), read by whoever wants to write that slot next: a producer
  // polls its OWN memory, never a peer's (a load from peer memory is an NVLink round trip of microseconds).
  RtpFlagWord credit[RTP_FLAG_MAX_WORLD][RTP_NUM_CTR];
  RtpFlagWord done_ctas;            // CTAs of the running launch that have finished
  RtpFlagWord status;               // 0 = ok, else first error code
};

#define RTP_KIND_GEMM 0
#define RTP_KIND_GATHER 1   // embedding lookup from a visiting table shard
#define RTP_KIND_VECADD 2   // out[r, c] = src[r, c] (+ in[r, c]): one hop of a ring reduce-scatter
#define RTP_KIND_REDUCE 3   // out[i] = sum_k src_k[i] over r_nsrc flat bf16 buffers (owner-side sum of gradient slots)

// Field order matters for speed: a phase is read from the kernel-parameter bank, where the first touch of a line
// costs a few hundred nanoseconds on the critical path of a short GEMM.  The fields that the TMA producer and the UMMA
// issuer need come first, the epilogue's next, the ones of the rarer phase kinds last.
struct RtpPhase {
  int kind;
  // operands (bf16). *_mn = 1: the operand is stored with its M (or N) index contiguous.
  int a_map, b_map;
  int a_mn, b_mn;
  int M, N, K;
  int bn;  // tile width: 64, 128 or 256
  int b_box;      // rows per TMA box of a K-major B operand (64 or 128)
  int causal;     // 1: skip tiles entirely above the diagonal (n0 > m0 + 127); 2: stop the k loop at the diagonal; 3: start it at the tile's first row (transposed products)
  int cta_off;  // tile t of this phase runs on CTA (t + cta_off) % G, so that successive phases fill different SMs
  // batching: `batch` independent GEMMs whose operands are windows of the same 2-D tensors.  Batch z = (zo, zi) with
  // zi = z % batch_inner; the window of operand X starts at (mn, k) += zo * x_bo_{mn,k} + zi * x_bi_{mn,k} and the
  // output / accumulate pointers move by zo * d_bo + zi * d_bi elements.
  int batch, batch_inner;
  int a_off_mn, a_off_k;  // element offsets added to the tile coordinates
  int b_off_mn, b_off_k;
  int a_bo_mn, a_bo_k, a_bi_mn, a_bi_k;
  int b_bo_mn, b_bo_k, b_bi_mn, b_bi_k;
  // K-segmented phase (nseg > 1): the contraction runs over nseg segments of K elements each; segment i reads A at
  // k-offset seg_a_off_k[i] and B through tensor map seg_b_map[i] (from k = 0), after local arrival counter wait_ctr[i]
  // (if >= 0).  One accumulator, one epilogue: a sum over visiting weight shards needs no read-modify-write of D.
  int nseg;
  int seg_a_off_k[RTP_MAX_WAITS];
  int seg_b_map[RTP_MAX_WAITS];
  // Tile-segmented phase (tseg != 0): the OUTPUT falls into tseg_n segments of tseg_len columns (tseg = 1) or rows
  // (tseg = 2), one per weight shard; M / N of the phase span all segments.  Per-segment operands, destinations and
  // counters come from RtpProgram::segtab[tseg_tab] (wait_ctr[i] / done_ctr[i] of this phase belong to segment i).
  // One phase instead of one per shard: the fixed cost of a phase (counter polls, hand-off, done reports: ~3 us) is
  // paid once per launch instead of N times.
  int tseg, tseg_len, tseg_n, tseg_tab;
  // synchronisation (all optional)
  int wait_ctr[RTP_MAX_WAITS];  // local arrival counters that must reach fill (uses + rel + 1) before operands are read
  int wait_rel[RTP_MAX_WAITS];
  // epilogue
  void* d;
  long long ldd;
  const void* c;  // optional accumulate source (same shape as d)
  long long ldc;
  const void* bias;    // optional bf16[N]
  const void* bias_more[RTP_MAX_WAITS - 1];  // further bias vectors added on top (K-segmented row-mode forward: one per shard)
  int n_bias_more;
  const void* mask;    // optional bf16 [M, N]: out = mask > 0 ? out * mask_scale : 0
  long long ldmask;
  int d_fp32;
  int vec_ok;  // 1: 16-byte vector accesses of d/c/mask rows are aligned
  int c_fp32;
  int act;             // 0 none, 1 relu, 2 gelu(erf)
  float alpha;    // accumulator scale applied first in the epilogue
  float mask_scale;
  uint32_t drop_thresh;  // 0: no dropout. keep element if philox word >= thresh
  float drop_scale;
  unsigned long long drop_seed, drop_offset;
  const unsigned long long* drop_step_ptr;  // optional device counter: offset += *ptr * 65536 (graph replays get fresh masks)
  long long d_bo, d_bi, c_bo, c_bi;
  unsigned long long* credit_ptr;  // local credit counter of the destination (rank, slot): must reach uses + rel before d is written
  int credit_ctr;
  int credit_rel;
  int done_ctr[RTP_MAX_WAITS];     // local `done` counters bumped when this CTA has finished the phase
  unsigned long long* arrive_ptr;  // remote `arrive` counter bumped when this CTA has finished the phase
  // optional vector job done by CTA 0 at the end of the phase: vec_out[i] = vec_in[i] + vec_add[i] (bf16/fp32 per flags)
  void* vec_out;
  const void* vec_in;
  const float* vec_add;
  int vec_len;
  int vec_fp32;  // dtype of vec_out / vec_in
  // ---- RTP_KIND_GATHER: out[t, c] = dropout(table[ids[t], c] * scale + pe[t / tpp, col_off + c]); out = d (pitch ldd)
  const void* g_table;       // [V, g_cols] bf16, home shard or a workspace slot
  const long long* g_ids;
  int g_tokens, g_cols, g_dim, g_col_off, g_tpp;
  float g_scale;
  const void* g_pe;
  long long g_ldpe;
  // ---- RTP_KIND_VECADD: d[r, c] = v_src[r * v_ld + c] (+ c[r, c]);  d and c are dense [v_rows, v_cols]
  const void* v_src;
  long long v_ld;
  int v_rows, v_cols;
  // ---- RTP_KIND_REDUCE
  const void* r_src[RTP_NUM_SLOTS];
  int r_nsrc;
  long long r_n;  // elements, multiple of 8
};

// Per-segment data of a tile-segmented phase (see RtpPhase::tseg).  Segment order = order of arrival of the shards.
struct RtpSegTable {
  int map[RTP_MAX_WAITS];        // tensor map of the segmented operand (B if tseg = 1, A if tseg = 2); -1: the phase's own
  int off_mn[RTP_MAX_WAITS];     // mn offset of that operand for the segment (tile coordinates are local to the segment)
  int drop_add[RTP_MAX_WAITS];   // added to the phase's dropout offset
  void* d[RTP_MAX_WAITS];        // output base of the segment (pitch = the phase's ldd)
  const void* bias[RTP_MAX_WAITS];
  unsigned long long* credit_ptr[RTP_MAX_WAITS];   // local credit counter that must reach uses + 0 before d[i] is written
  int credit_ctr[RTP_MAX_WAITS];
  unsigned long long* arrive_ptr[RTP_MAX_WAITS];   // remote arrival counter bumped once per CTA when the phase is done
  void* vec_out[RTP_MAX_WAITS];                    // per-segment vector job: vec_out[i][k] = vec_add[vec_off[i] + k], k < vec_len
  long long vec_off[RTP_MAX_WAITS];
};
#define RTP_MAX_SEGTABS 3

struct RtpPush {
  const void* src;
  void* dst;  // peer memory
  unsigned long long bytes;  // multiple of 16
  unsigned long long* credit_ptr;  // local credit counter of the destination (rank, slot)
  int credit_ctr;
  int credit_rel;
  unsigned long long* arrive_ptr;  // remote `arrive` counter of the destination slot
};

struct alignas(64) RtpProgram {
  int n_phases, n_pushes;
  int n_stages, stage_bytes;  // smem pipeline geometry (host: finalize_program)
  int n_compute;              // CTAs [0, n_compute) run GEMM tiles, [n_compute, grid) only push (0 / grid: none reserved)
  int push_ring;              // pusher: 2 = plain loads + peer stores by the whole warp (default); bulk copies through a
                              // shared-memory ring by one thread: 0 / 3 = four 3840-byte chunks, 1 / 4 = two of 7680 (see gemm.cu)
  RtpFlagBlock* flags;  // this rank's flag block (may be null when nothing synchronises)
  RtpFlagBlock* peer_flags[RTP_FLAG_MAX_WORLD];  // every rank's flag block as mapped here (credits are written there)
  int rank, world;
  unsigned long long* status;  // status word (flags->status or a plain device word)
  unsigned long long timeout_ns;
  unsigned long long* trace;  // optional debug timeline of CTA 0: [role][tile][event] globaltimer stamps (see gemm_kernel.cuh)
  int uses_inc[RTP_NUM_CTR];  // added to flags->uses[] by the last CTA of the launch
  unsigned char map3d[RTP_MAX_MAPS];  // 1: the map of an MN-major operand is 3-D {64 mn, k, mn / 64}: one copy fetches all
                                      // 64-wide column blocks of a stage (coordinates {0, k, mn / 64})
  alignas(64) CUtensorMap maps[RTP_MAX_MAPS];
  RtpPhase phases[RTP_MAX_PHASES];
  RtpPush pushes[RTP_MAX_PUSHES];
  RtpSegTable segtab[RTP_MAX_SEGTABS];
};

