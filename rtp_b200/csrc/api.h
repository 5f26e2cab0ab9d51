// C ABI of librtp_b200.so. Every function takes raw device pointers and a CUDA stream, returns 0 on
// success or a negative error code, and never synchronises the device. Python binds these with ctypes.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RTP_MAX_WORLD 8

// ------------------------------------------------------------------------------------------- GEMM
// D[M,N] = epilogue( A * B^T (+ C) ),  bf16 operands, fp32 accumulation on tcgen05 tensor cores.
typedef struct {
  const void* a; long long lda; int a_mn;  // a_mn = 0: A is [M,K] row-major. 1: A is stored [K,M] row-major.
  const void* b; long long ldb; int b_mn;  // b_mn = 0: B is [N,K] row-major. 1: B is stored [K,N] row-major.
  int M, N, K;
  void* d; long long ldd; int d_fp32;
  const void* c; long long ldc; int c_fp32;   // optional accumulate source
  const void* bias;                           // optional bf16 [N]
  int act;                                    // 0 none, 1 relu, 2 gelu
  const void* mask; long long ldmask; float mask_scale;  // optional: out = mask > 0 ? out * scale : 0
  float drop_p; unsigned long long seed, offset;          // dropout on the output when drop_p > 0
  const unsigned long long* step_ptr;                     // optional device step counter mixed into the dropout offset
  unsigned long long* status;                 // device status word (0 = ok)
  int num_ctas;                               // 0 = one CTA per SM
  int bn;                                     // 0 = auto, else 128 or 256
} RtpGemmArgs;
int rtp_gemm(const RtpGemmArgs* args, void* stream);

// Batched GEMM over windows of two 2-D tensors: batch z = (zo, zi), zi = z % batch_inner.  Operand X (stored
// [x_rows, x_cols] row-major, pitch ldx) is read at row/column offsets zo * x_bo_* + zi * x_bi_* (in the operand's
// own (mn, k) coordinates); the output moves by zo * d_bo + zi * d_bi elements.  Used for attention, where the
// per-head matrices are column windows of [B*S, H*hd] projections.
typedef struct {
  const void* a; long long lda; int a_mn; long long a_rows, a_cols;
  const void* b; long long ldb; int b_mn; long long b_rows, b_cols;
  int M, N, K, batch, batch_inner;
  int a_bo_mn, a_bo_k, a_bi_mn, a_bi_k;
  int b_bo_mn, b_bo_k, b_bi_mn, b_bi_k;
  void* d; long long ldd, d_bo, d_bi;
  float alpha;
  int causal;      // 1: skip tiles above the diagonal; 2: stop the contraction at the diagonal; 3: start it at the tile's first row
  int bn;          // 0 = auto
  unsigned long long* status;
} RtpGemmBatched;
int rtp_gemm_batched(const RtpGemmBatched* args, void* stream);

// ---------------------------------------------------------------------------- rotated linear layers
// Workspace of one rank (peer-mapped): [flag block][W slot 0][W slot 1][G slot 0][G slot 1].
typedef struct {
  int rank, world;
  void* ws[RTP_MAX_WORLD];         // workspace base of every rank, as mapped in this process
  unsigned long long slot_bytes;   // capacity of each of the four slots
  int ctas;                        // CTAs per rank (same value on every rank)
  unsigned long long timeout_ns;
} RtpRing;

typedef struct {
  int mode;                 // 0: column (shard [out/N, in], outputs concatenated); 1: row (shard [out, in/N], summed)
  int M;                    // rows (tokens) of this rank's batch
  int in_features, out_features;  // of the full layer
  const void* home;         // this rank's flat shard: weight, then (optionally) bias at bias_off
  long long bias_off;       // element offset of the bias inside the flat shard, -1: no bias
  unsigned long long shard_bytes;  // bytes of the flat shard that travel (multiple of 16)
  const void* x; long long ldx;    // [M, in]
  void* y; long long ldy;          // [M, out]
  int act;                         // activation applied to y (column mode only)
  float drop_p; unsigned long long seed, offset;  // dropout applied to y after the activation
  const unsigned long long* step_ptr;             // optional device step counter mixed into the dropout offset
  // Cross-launch prefetch (all zero = every launch pushes the shards it needs itself).  The launch reads visiting shards
  // from weight-slot bank `bank`; with no_self_push = 1 they were pushed there by the previous launch.  If next_home is
  // set, this launch also pushes that shard (the home shard of the NEXT rotated linear on this stream, which must read
  // bank 1 - bank with no_self_push = 1) to the ranks that will use it: next_kind 0 = forward order, 1 = backward order.
  int bank, no_self_push;
  const void* next_home; unsigned long long next_bytes; int next_kind;
} RtpLinearFwd;
int rtp_linear_fwd(const RtpRing* ring, const RtpLinearFwd* op, void* stream);

typedef struct {
  int mode, M, in_features, out_features;
  const void* home; long long bias_off; unsigned long long shard_bytes;
  const void* x; long long ldx;    // saved input [M, in]
  const void* dy; long long ldy;   // [M, out]
  void* dx; long long lddx;        // [M, in], may be null (first layer)
  void* grad_home;                 // flat gradient of the home shard (same layout as home), bf16
  const float* dbias_full;         // fp32 column sums of dy: [out] (may be null when there is no bias)
  const void* mask; long long ldmask; float mask_scale;  // optional mask applied to dx (activation/dropout backward)
  int dx_accumulate;               // 1: add the input gradient to what dx already holds
  int grad_accumulate;             // 1: add the weight gradient to what grad_home already holds
  int bank, no_self_push;          // cross-launch prefetch, see RtpLinearFwd
  const void* next_home; unsigned long long next_bytes; int next_kind;
  // Optional row of M ones (bf16).  Where rtp_linear_bwd_folds_bias() says yes and dbias_full is null, the bias gradient
  // is one more GEMM phase of the launch (ones[1, M] x dy[M, out], fp32 accumulation) and needs no column-sum kernel.
  const void* ones;
} RtpLinearBwd;
int rtp_linear_bwd(const RtpRing* ring, const RtpLinearBwd* op, void* stream);
// 1 if the launch described by `op` computes the bias gradient itself from op->ones (1-rank ring, tiles on single CTAs,
// M a multiple of 8), 0 if the caller has to supply the column sums in dbias_full.
int rtp_linear_bwd_folds_bias(const RtpRing* ring, const RtpLinearBwd* op);

// Rotating experts (MoE): rank r owns n_local whole experts; x / y hold the dispatched tokens expert-major
// ([world*n_local*cap, features], expert g = rows [g*cap, (g+1)*cap)).  One launch applies ONE linear of every
// expert (y_g = act(x_g W_g^T + b_g)) while the flat range that holds the local experts' (weight, bias) blocks
// visits every rank.  Tokens never leave their GPU.
typedef struct {
  int cap, n_local, in_features, out_features;
  const void* home;                    // n_local blocks: weight [out, in] at e*expert_stride, bias at + bias_off
  long long expert_stride, bias_off;   // elements (bias_off -1: no bias)
  unsigned long long shard_bytes;
  const void* x; long long ldx;
  void* y; long long ldy;
  int act;
} RtpExpertFwd;
int rtp_expert_fwd(const RtpRing* ring, const RtpExpertFwd* op, void* stream);
typedef struct {
  int cap, n_local, in_features, out_features;
  const void* home; long long expert_stride, bias_off; unsigned long long shard_bytes;
  const void* x; long long ldx;
  const void* dy; long long ldy;
  void* dx; long long lddx;            // may be null
  void* grad_home;                     // same layout as home
  const float* dbias_full;             // fp32 [world*n_local, out] per-expert column sums of dy (null: no bias)
  const void* mask; long long ldmask; float mask_scale;   // optional activation backward applied to dx
} RtpExpertBwd;
int rtp_expert_bwd(const RtpRing* ring, const RtpExpertBwd* op, void* stream);
int rtp_expert_fwd_emu(const RtpRing* rings, const RtpExpertFwd* ops, int world, void* stream);
int rtp_expert_bwd_emu(const RtpRing* rings, const RtpExpertBwd* ops, int world, void* stream);

// Rotated embedding lookup: the table is sharded along the embedding dim ([V, D/N] per rank); shard j fills
// columns [j*D/N, (j+1)*D/N) of out.  out = dropout(table[ids] * scale + pe[t / tokens_per_pos]).
typedef struct {
  const void* home; unsigned long long shard_bytes;
  int V, Ds, D;
  const long long* ids; int T;
  void* out; long long ld_out;
  float scale;
  const void* pe; long long ld_pe; int tokens_per_pos;
  float drop_p; unsigned long long seed, offset; const unsigned long long* step_ptr;
} RtpEmbedFwd;
int rtp_embed_fwd_rot(const RtpRing* ring, const RtpEmbedFwd* op, void* stream);

// Ring reduce-scatter over column blocks: every rank holds a dense [rows, N*cols] bf16 matrix `src` (pitch ld);
// rank r ends up with sum over ranks of column block r in `out` (dense [rows, cols]).  Used for the gradient of
// the rotated embedding table.
typedef struct {
  const void* src; long long ld;
  int rows, cols;
  void* out;
} RtpReduceScatter;
int rtp_reduce_scatter_cols(const RtpRing* ring, const RtpReduceScatter* op, void* stream);
// The same reduction as ONE hop (all-to-all): `src` holds N contiguous blocks of block_elems bf16 each (block j is what
// this rank contributes to owner j); every block travels straight to its owner and the owner adds the N contributions.
typedef struct {
  const void* src;
  long long block_elems;     // multiple of 8
  void* out;                 // [block_elems] bf16: sum over ranks of block `rank`
} RtpReduceBlocks;
int rtp_reduce_blocks(const RtpRing* ring, const RtpReduceBlocks* op, void* stream);
int rtp_reduce_blocks_emu(const RtpRing* rings, const RtpReduceBlocks* ops, int world, void* stream);
int rtp_embed_fwd_rot_emu(const RtpRing* rings, const RtpEmbedFwd* ops, int world, void* stream);
int rtp_reduce_scatter_cols_emu(const RtpRing* rings, const RtpReduceScatter* ops, int world, void* stream);

// Single-GPU emulation of `world` ranks in one cooperative launch (for tests with fewer GPUs than ranks).
int rtp_linear_fwd_emu(const RtpRing* rings, const RtpLinearFwd* ops, int world, void* stream);
int rtp_linear_bwd_emu(const RtpRing* rings, const RtpLinearBwd* ops, int world, void* stream);

// ------------------------------------------------------------------------------- in-place ring shift
// Replaces every rank's buffer by its neighbour's through a small peer-mapped staging area (no second full-size buffer):
// the transport of the memory-lean in-place rotation mode, and the library's rotate-only kernel.  direction 0 = "down"
// (send to rank r-1, receive from r+1), 1 = "up".  world_emulated = 1 on a real ring (each process launches its own
// rank); 2..4 emulate that many ranks on one GPU in one cooperative launch.
unsigned long long rtp_shift_staging_bytes(int lanes);
int rtp_shift_staging_create(int lanes, void** out);     // cudaMalloc + zeroed counters; IPC handle via rtp_ws_ipc_get
int rtp_shift_staging_destroy(void* staging);
int rtp_shift_max_lanes(void);
int rtp_ring_shift(int world_emulated, void* const* buf, unsigned long long bytes, void* const* staging,
                   void* const* dst_staging, void* const* src_staging, int direction, int lanes,
                   unsigned long long* const* status, unsigned long long timeout_ns, void* stream);
const char* rtp_shift_last_error(void);

// ------------------------------------------------------------------------------------- workspace
unsigned long long rtp_ws_bytes_world(unsigned long long slot_bytes, int world);
int rtp_ws_create_world(unsigned long long slot_bytes, int world, void** out);   // sized for rings of exactly `world` ranks
int rtp_ws_destroy(void* ws);
int rtp_ws_reset(void* ws, void* stream);                        // zero the flag block
int rtp_ws_ipc_get(void* ws, void* handle64);                    // 64-byte cudaIpcMemHandle
int rtp_ws_ipc_open(const void* handle64, void** out);
int rtp_ws_ipc_close(void* mapped);
int rtp_ws_status(void* ws, unsigned long long* host_out, void* stream);  // reads the status word (synchronises stream)
// Race-detection aid: copies the arrive[], done[] and uses[] counters of this rank's flag block to host_out
// (3 * rtp_ws_num_counters() words; synchronises the stream).  At a quiescent point uses[] must be the same on every
// rank of the ring and arrive[c] == done[c] == uses[c] * CTAs for every slot counter c.
// Program lint (host only, no GPU needed): builds the rotation programs of every rank of a made-up ring and checks copy
// alignment, tile segments, overlapping output tiles and the cross-rank counter protocol (one producer per arrival
// counter, matching credit, writes inside the slot, `done` reports, equal fill counts).  Returns the number of problems;
// `report` receives one line per problem.
// `inject` (0 = off) damages rank 0's program in one of five ways so that the lint can be tested itself.
int rtp_lint_linear(int world, int ctas, unsigned long long slot_bytes, int mode, int M, int in_features, int out_features,
                    int has_bias, int backward, int need_dx, int inject, char* report, int cap);
int rtp_lint_experts(int world, int ctas, unsigned long long slot_bytes, int n_local, int cap_tokens, int in_features,
                     int out_features, int has_bias, int backward, int need_dx, char* report, int cap);
// The same for a chain of rotated linears with cross-launch prefetch, as the fused trainer issues them: `spec` holds 7
// ints per launch (mode, M, in_features, out_features, has_bias, backward, need_dx); launch k reads bank k & 1 and pushes
// the shards of launch k + 1 into the other bank.  `flip_bank_at` >= 0 builds that launch with the wrong bank (self-test).
int rtp_lint_linear_chain(int world, int ctas, unsigned long long slot_bytes, int n_launches, const int* spec,
                          int flip_bank_at, char* report, int cap);
// And for the programs without GEMM tiles: kind 0 = rotated embedding lookup (a = V, b = D, c = tokens), 1 = one-hop
// reduce of `world` blocks (a = elements per block).
int rtp_lint_transport(int world, int ctas, unsigned long long slot_bytes, int kind, long long a, long long b, long long c,
                       char* report, int cap);
int rtp_ws_num_counters(void);
int rtp_ws_counters(void* ws, unsigned long long* host_out, void* stream);
void* rtp_ws_wslot(void* ws, unsigned long long slot_bytes, int i, int world);   // logical weight slot i = bank * 8 + index
void* rtp_ws_gslot(void* ws, unsigned long long slot_bytes, int i, int world);
int rtp_sm_count(void);
const char* rtp_last_error(void);
void rtp_set_pair_mode(int on);        // CTA pairs (cta_group::2 UMMA, half of the B tile per SM): 1 always, 0 never, -1 automatic (default; env RTP_PAIR=0/1 overrides)
void rtp_set_push_ctas(int n);         // CTAs per launch reserved for pushing shards to peers (default 0: every CTA pushes a share; env RTP_PUSH_CTAS)
void rtp_debug_set_trace(unsigned long long* device_buffer_1024_words);  // tuning aid: globaltimer timeline of CTA 0 of rtp_gemm launches (null = off)
void rtp_debug_force_stages(int n);   // tuning aid: cap the smem pipeline depth (0 = automatic)

#ifdef __cplusplus
}
#endif
