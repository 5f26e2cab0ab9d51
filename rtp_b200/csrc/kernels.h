// C ABI of the memory-bound kernels (see kernels.cu). Same conventions as api.h.
#pragma once
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
  void* p;        // bf16 parameter
  const void* g;  // bf16 gradient
  void* m;        // first moment (fp32 or bf16)
  void* v;        // second moment
  long long n;
  float lr_mult;  // 1/N for biases that are stored as b/N on every rank
  int state_fp32;
} RtpAdamTensor;

const char* rtp_kernels_last_error(void);
int rtp_norm_fwd(const void* x, const void* sub, const void* gamma, const void* beta, void* h_out, void* y,
                 float* mean, float* rstd, int M, int D, float eps, int rms, float drop_p, unsigned long long seed,
                 unsigned long long offset, const unsigned long long* step_ptr, void* stream);
int rtp_norm_bwd(const void* dy, const void* h, const void* gamma, const float* mean, const float* rstd, void* dx,
                 void* dsub, float* dgamma, float* dbeta, int M, int D, int rms, float drop_p,
                 unsigned long long seed, unsigned long long offset, const void* dres,
                 const unsigned long long* step_ptr, void* stream);
int rtp_cross_entropy(void* logits, long long ld, const long long* target, float* loss, int M, int V, float grad_scale,
                      long long ignore_index, int write_grad, void* stream);
// Same, but the gradient goes to `grad` (row pitch ldg) and the logits stay as they are; grad = null: in place.
int rtp_cross_entropy_to(void* logits, long long ld, const long long* target, float* loss, int M, int V, float grad_scale,
                         long long ignore_index, int write_grad, void* grad, long long ldg, void* stream);
int rtp_embed_fwd(const void* table, const long long* ids, const void* pe, long long ld_pe, int tokens_per_pos,
                  void* out, long long ld_out, int col_off, int T, int Ds, int D, float scale, float drop_p,
                  unsigned long long seed, unsigned long long offset, const unsigned long long* step_ptr,
                  void* stream);
int rtp_embed_bwd(void* gtable, const long long* ids, const void* dy, long long ld_dy, int col_off, int T, int Ds,
                  int D, float scale, float drop_p, unsigned long long seed, unsigned long long offset,
                  const unsigned long long* step_ptr, void* stream);
// Same scatter-add into a block-major gradient [Ds / blk_cols][V][blk_cols]: one contiguous [V, blk_cols] block per owner
// of an embedding-dim shard, ready to be pushed to that owner.
int rtp_embed_bwd_blocks(void* gtable, const long long* ids, const void* dy, long long ld_dy, int col_off, int T, int Ds,
                         int D, float scale, float drop_p, unsigned long long seed, unsigned long long offset,
                         const unsigned long long* step_ptr, int blk_cols, int V, void* stream);
// Tensor-core (tcgen05) kernels for S = 32 / 64, head_dim 64 (attn_tc.cu); rtp_attn_small_* route to them when they
// apply.  rtp_set_attn_tc(0) forces the scalar kernels (A/B comparison).
int rtp_attn_tc_supported(int S, int heads, int nshard);
int rtp_attn_tc_error(void);
int rtp_attn_tc_set_trace(unsigned long long* device_buffer);
const char* rtp_attn_tc_last_error(void);
void rtp_set_attn_tc(int on);
int rtp_attn_tc_fwd(const void* qkv, void* out, int S, int B, int heads, int nshard, int causal, float sm_scale,
                    float drop_p, unsigned long long seed, unsigned long long offset,
                    const unsigned long long* step_ptr, void* stream);
int rtp_attn_tc_bwd(const void* qkv, const void* dout, void* dqkv, int S, int B, int heads, int nshard, int causal,
                    float sm_scale, float drop_p, unsigned long long seed, unsigned long long offset,
                    const unsigned long long* step_ptr, void* stream);
int rtp_attn_small_fwd(const void* qkv, void* out, int S, int B, int heads, int nshard, int causal, float sm_scale,
                       float drop_p, unsigned long long seed, unsigned long long offset,
                       const unsigned long long* step_ptr, void* stream);
int rtp_attn_small_bwd(const void* qkv, const void* dout, void* dqkv, int S, int B, int heads, int nshard, int causal,
                       float sm_scale, float drop_p, unsigned long long seed, unsigned long long offset,
                       const unsigned long long* step_ptr, void* stream);
// Top-2 MoE gating on [S, E] fp32 logits (E <= 64) and its gradient; rotary position embedding (gate_rope.cu).
const char* rtp_gate_last_error(void);
int rtp_top2_gate_fwd(const float* logits, const float* noise, float* gates, int* idx, int* loc, float* gate_w,
                      unsigned char* valid, float* me_sum, float* ce, float* l_aux, int S, int E, int capacity,
                      void* stream);
int rtp_top2_gate_bwd(const float* gates, const int* idx, const unsigned char* valid, const float* ce,
                      const float* d_gate_w, const float* d_l_aux, float* dlogits, int S, int E, void* stream);
int rtp_rope(const void* x, void* y, const float* cosv, const float* sinv, long long T, int H, int hd, int S, int inner,
             int backward, void* stream);
// Convolution as GEMM: patch matrix of an NCHW bf16 input and its adjoint (im2col.cu).
const char* rtp_im2col_last_error(void);
int rtp_im2col(const void* x, void* cols, int B, int C, int H, int W, int KH, int KW, int sh, int sw, int ph, int pw,
               int dh, int dw, int Kp, void* stream);
int rtp_col2im(const void* dcols, void* dx, int B, int C, int H, int W, int KH, int KW, int sh, int sw, int ph, int pw,
               int dh, int dw, int Kp, void* stream);
int rtp_colsum(const void* x, long long ld, int M, int N, float* out, void* stream);
int rtp_adam(const RtpAdamTensor* tensors_dev, const int* block_start_dev, int ntensors, int total_blocks,
             const long long* step_dev, float lr, float beta1, float beta2, float eps, float weight_decay, int adamw,
             float clip_value, float grad_scale, const int* block_tensor_dev /* optional: tensor index of every block */,
             void* stream);
int rtp_causal_softmax(void* s, long long rows, int S, float scale, void* stream);
int rtp_causal_softmax_bwd(const void* p, void* dp, long long rows, int S, float scale, void* stream);
int rtp_gelu_fwd(const void* x, void* y, long long n, void* stream);
int rtp_gelu_bwd(const void* x, const void* dy, void* dx, long long n, void* stream);
int rtp_swiglu_fwd(const void* g, const void* u, long long ld, void* y, long long rows, int cols, void* stream);
int rtp_swiglu_bwd(const void* g, const void* u, long long ld, const void* dy, void* dg, void* du, long long ldo,
                   long long rows, int cols, void* stream);
int rtp_moe_scatter(const void* src, const int* slot, const float* scale, void* dst, int S, int M, long long dst_rows,
                    void* stream);
int rtp_moe_gather(const void* src, const int* slot, const float* scale, void* dst, int S, int M, void* stream);
int rtp_moe_rowdot(const void* a, const void* b, const int* slot, float* out, int S, int M, void* stream);
int rtp_add(const void* a, const void* b, void* out, long long n, void* stream);
int rtp_cast_f32_bf16(const float* in, void* out, long long n, float scale, void* stream);
int rtp_sum_f32(const float* in, float* out, int n, float scale, void* stream);

#ifdef __cplusplus
}
#endif
