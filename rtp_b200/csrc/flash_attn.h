// C ABI of the flash-attention kernels (flash_attn.cu): softmax(scale * Q K^T + mask) V with online softmax on tcgen05
// tensor cores, forward and backward, for any sequence length and head_dim 64 or 128.  Nothing of size S x S is ever
// written to global memory: forward keeps one fp32 log-sum-exp per query row, backward recomputes the probabilities.
//
// Replaces the attention inside the reference's vendored multi_head_attention_forward
// (rtp/module/functional.py:785-792 explicit softmax path, :825 scaled_dot_product_attention path).
#pragma once
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

// A [batch, seq, heads, head_dim] bf16 operand described by strides, so that packed projections ([tokens, 3 * D] with
// the q / k / v blocks of every head-shard side by side) and both token orders ([B, S] and [S, B]) need no copy.
// Element (b, s, h, d) lives at ptr + b * sb + s * ss + col(h) + d, with
//     col(h) = col_base + (h / hpg) * gstride + (h % hpg) * hstride          (all in elements).
// `width` is the number of valid columns of a row (the extent the tensor map is built over).
typedef struct {
  void* ptr;
  long long sb, ss;
  long long width;
  int col_base, hpg, gstride, hstride;
} RtpFlashRef;

typedef struct {
  RtpFlashRef q, k, v, o;       // o: output of forward, input of backward
  RtpFlashRef dout, dq, dk, dv; // backward only
  float* lse;                   // [B * H, Sq] log-sum-exp of the scaled scores in log2 units (written by forward)
  float* delta;                 // [B * H, Sq] scratch of backward: rowsum(dO * O)
  int B, H, Sq, Sk, head_dim;
  int causal;                   // 1: key j is visible to query i only if j <= i (needs Sq == Sk)
  const void* mask;             // optional additive mask [Sq, Sk] shared by all batches and heads (-inf = masked)
  long long mask_ld; int mask_fp32;   // row pitch in elements; dtype fp32 (1) or bf16 (0)
  const unsigned char* kpm;     // optional key-padding mask [B, Sk], non-zero = key is ignored
  long long kpm_ld;
  float sm_scale;
  float drop_p; unsigned long long seed, offset;   // dropout on the probabilities (regenerated in backward)
  const unsigned long long* step_ptr;              // optional device counter mixed into the dropout offset
  unsigned long long* status;   // device status word (0 = ok; a bounded wait that ran out writes its code)
} RtpFlashArgs;

int rtp_flash_fwd(const RtpFlashArgs* a, void* stream);
int rtp_flash_bwd(const RtpFlashArgs* a, void* stream);   // two launches: dQ (+ delta), then dK / dV
const char* rtp_flash_last_error(void);
// Tuning aid: while a device buffer of 512 64-bit words is set, CTA 0 of the forward kernel stamps the SM clock at the
// steps of its first 16 key blocks (row warps 0 and 4: words 0..255, UMMA issuer: 256..383).  Null switches it off.
void rtp_flash_debug_set_trace(long long* device_buffer_512_words);

#ifdef __cplusplus
}
#endif
