// Top-2 gating (MoE router) and rotary position embedding kernels.
//
// Gating, for logits [S, E] with E <= 64 (reference semantics: rtp/module/top2gate.py:43-105):
//   gate_rows_kernel   one warp per token: fp32 softmax, top-1, top-2 of (logits + noise) with the top-1 expert masked,
//                      and the column sums of the softmax (for the load-balancing loss)
//   gate_slots_kernel  one block: token-order slot of every token inside its two experts (second choices queue behind
//                      all first choices), capacity mask, normalised gate weights, l_aux
//   gate_bwd_kernel    one warp per token: gradient of (gate weights, l_aux) with respect to the logits
// The [S, E, C] one-hot tensors of the reference are never formed.
//
// RoPE: rotates the pairs (x[2i], x[2i+1]) of every head by the angle of the token's position; the backward pass is
// the same kernel with the sine negated.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "common.cuh"
#include "kernels.h"

namespace {
using namespace rtp;

std::string g_err;
int fail(const char* what, cudaError_t e) {
  g_err = std::string(what) + ": " + cudaGetErrorString(e);
  return -1;
}

constexpr int kMaxE = 64;

__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// arg max over (value, index) pairs of a warp; ties go to the smaller index (torch.argmax returns the first maximum)
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

// logits: [S, E] fp32.  noise: [S, E] fp32 or null (then no noise is added: deterministic second choice).
// gates: [S, E] fp32 softmax.  idx: [S, 2].  me_sum: [E] column sums of the softmax (zeroed by the caller).
__global__ void gate_rows_kernel(const float* __restrict__ logits, const float* __restrict__ noise,
                                 float* __restrict__ gates, int* __restrict__ idx, float* __restrict__ me_sum, int S,
                                 int E) {
  __shared__ float s_me[kMaxE];
  for (int i = threadIdx.x; i < E; i += blockDim.x) s_me[i] = 0.f;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int s = blockIdx.x * nw + warp; s < S; s += gridDim.x * nw) {
    float x[2], n[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int e = lane + 32 * k;
      x[k] = e < E ? logits[(size_t)s * E + e] : -INFINITY;
      n[k] = (e < E && noise) ? noise[(size_t)s * E + e] : 0.f;
    }
    const float mx = warp_max_f(fmaxf(x[0], x[1]));
    float p[2];
    p[0] = lane < E ? __expf(x[0] - mx) : 0.f;
    p[1] = lane + 32 < E ? __expf(x[1] - mx) : 0.f;
    const float inv = 1.f / warp_sum_f(p[0] + p[1]);
    p[0] *= inv;
    p[1] *= inv;
    // top-1 of the softmax
    float v1 = p[0] >= p[1] ? p[0] : p[1];
    int i1 = p[0] >= p[1] ? lane : lane + 32;
    if (lane >= E) { v1 = -INFINITY; i1 = 1 << 30; }
    warp_argmax(v1, i1);
    // top-2: arg max of logits + noise with the first choice removed
    float y0 = (lane < E && lane != i1) ? x[0] + n[0] : -INFINITY;
    float y1 = (lane + 32 < E && lane + 32 != i1) ? x[1] + n[1] : -INFINITY;
    float v2 = y0 >= y1 ? y0 : y1;
    int i2 = y0 >= y1 ? lane : lane + 32;
    if (v2 == -INFINITY) i2 = 1 << 30;
    warp_argmax(v2, i2);
    if (i2 >= E) i2 = i1;   // E == 1
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int e = lane + 32 * k;
      if (e < E) {
        gates[(size_t)s * E + e] = p[k];
        atomicAdd(&s_me[e], p[k]);
      }
    }
    if (lane == 0) {
      idx[2 * s] = i1;
      idx[2 * s + 1] = i2;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < E; i += blockDim.x) atomicAdd(&me_sum[i], s_me[i]);
}

// One block of 1024 threads walks the tokens in order, 1024 at a time.  Position of a token among the earlier tokens
// with the same expert = (count in earlier chunks) + (count in earlier warps of the chunk) + (rank inside the warp).
__device__ __forceinline__ void ranked_pass(const int* __restrict__ idx, int which, int S, int E, int* s_base,
                                            int (*s_warp)[kMaxE], int* __restrict__ loc) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int c0 = 0; c0 < S; c0 += 1024) {
    const int s = c0 + threadIdx.x;
    const int e = s < S ? idx[2 * s + which] : -1;
    for (int i = threadIdx.x; i < 32 * kMaxE; i += 1024) (&s_warp[0][0])[i] = 0;
    __syncthreads();
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    if (e >= 0 && rank == 0) s_warp[warp][e] = __popc(peers);
    __syncthreads();
    if (threadIdx.x < E) {
      int run = s_base[threadIdx.x];
      for (int w = 0; w < 32; ++w) {
        const int t = s_warp[w][threadIdx.x];
        s_warp[w][threadIdx.x] = run;
        run += t;
      }
      s_base[threadIdx.x] = run;
    }
    __syncthreads();
    if (e >= 0) loc[2 * s + which] = s_warp[warp][e] + rank;
    __syncthreads();
  }
}

__global__ void __launch_bounds__(1024) gate_slots_kernel(const float* __restrict__ gates, const int* __restrict__ idx,
                                                          const float* __restrict__ me_sum, int* __restrict__ loc,
                                                          float* __restrict__ gate_w, unsigned char* __restrict__ valid,
                                                          float* __restrict__ ce_out, float* __restrict__ l_aux, int S,
                                                          int E, int capacity) {
  __shared__ int s_base[kMaxE];
  __shared__ int s_warp[32][kMaxE];
  __shared__ float s_red[kMaxE];
  if (threadIdx.x < kMaxE) s_base[threadIdx.x] = 0;
  __syncthreads();
  ranked_pass(idx, 0, S, E, s_base, s_warp, loc);
  // s_base now holds the number of first choices per expert: second choices start behind them
  if (threadIdx.x < E) {
    const float ce = (float)s_base[threadIdx.x] / (float)S;
    ce_out[threadIdx.x] = ce;
    s_red[threadIdx.x] = (me_sum[threadIdx.x] / (float)S) * ce;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int e = 0; e < E; ++e) t += s_red[e];
    *l_aux = t / (float)E;
  }
  ranked_pass(idx, 1, S, E, s_base, s_warp, loc);
  for (int s = threadIdx.x; s < S; s += 1024) {
    const int e1 = idx[2 * s], e2 = idx[2 * s + 1];
    const int l1 = loc[2 * s], l2 = loc[2 * s + 1];
    const bool ok1 = l1 < capacity, ok2 = l2 < capacity && e2 != e1;
    const float g1 = ok1 ? gates[(size_t)s * E + e1] : 0.f;
    const float g2 = ok2 ? gates[(size_t)s * E + e2] : 0.f;
    const float d = fmaxf(g1 + g2, 1.1920929e-07f);
    gate_w[2 * s] = g1 / d;
    gate_w[2 * s + 1] = g2 / d;
    valid[2 * s] = ok1;
    valid[2 * s + 1] = ok2;
    if (!ok1) loc[2 * s] = 0;
    if (!ok2) loc[2 * s + 1] = 0;
  }
}

// dlogits = softmax'(dgates), with dgates[e] = d_l_aux * ce[e] / (E * S) + the gradient through the two normalised
// gate weights of the token.
__global__ void gate_bwd_kernel(const float* __restrict__ gates, const int* __restrict__ idx,
                                const unsigned char* __restrict__ valid, const float* __restrict__ ce,
                                const float* __restrict__ d_gate_w, const float* __restrict__ d_l_aux,
                                float* __restrict__ dlogits, int S, int E) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const float dl = d_l_aux ? *d_l_aux : 0.f;
  for (int s = blockIdx.x * nw + warp; s < S; s += gridDim.x * nw) {
    const int e1 = idx[2 * s], e2 = idx[2 * s + 1];
    const bool ok1 = valid[2 * s] != 0, ok2 = valid[2 * s + 1] != 0;
    const float g1 = ok1 ? gates[(size_t)s * E + e1] : 0.f;
    const float g2 = ok2 ? gates[(size_t)s * E + e2] : 0.f;
    const float sum = g1 + g2;
    const bool clamped = sum <= 1.1920929e-07f;
    const float d = fmaxf(sum, 1.1920929e-07f);
    const float do1 = d_gate_w[2 * s], do2 = d_gate_w[2 * s + 1];
    // out1 = g1 / d, out2 = g2 / d
    float dg1, dg2;
    if (clamped) {
      dg1 = do1 / d;
      dg2 = do2 / d;
    } else {
      dg1 = (do1 - do2) * g2 / (d * d);
      dg2 = (do2 - do1) * g1 / (d * d);
    }
    if (!ok1) dg1 = 0.f;
    if (!ok2) dg2 = 0.f;
    float p[2], dgt[2];
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int e = lane + 32 * k;
      p[k] = 0.f;
      dgt[k] = 0.f;
      if (e < E) {
        p[k] = gates[(size_t)s * E + e];
        dgt[k] = dl * ce[e] / ((float)E * (float)S);
        if (e == e1) dgt[k] += dg1;
        if (e == e2 && ok2) dgt[k] += dg2;
        dot += dgt[k] * p[k];
      }
    }
    dot = warp_sum_f(dot);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int e = lane + 32 * k;
      if (e < E) dlogits[(size_t)s * E + e] = p[k] * (dgt[k] - dot);
    }
  }
}

// x, y: [T, H, hd] bf16; token t sits at position (t / inner) % S: inner = 1 for a [B, S] token order, inner = B for
// [S, B].
__global__ void rope_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                            const float* __restrict__ cosv, const float* __restrict__ sinv, long long T, int H, int hd,
                            int S, int inner, float sin_sign) {
  const int half = hd >> 1;
  const long long total = T * H * (half >> 2);   // 4 pairs (8 elements, 16 bytes) per item
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int q = (int)(i % (half >> 2));
    const long long th = i / (half >> 2);
    const long long t = th / H;
    const int pos = (int)((t / inner) % S);
    const uint4 raw = *reinterpret_cast<const uint4*>(x + th * hd + q * 8);
    const float4 c = *reinterpret_cast<const float4*>(cosv + (size_t)pos * half + q * 4);
    float4 sn = *reinterpret_cast<const float4*>(sinv + (size_t)pos * half + q * 4);
    sn.x *= sin_sign; sn.y *= sin_sign; sn.z *= sin_sign; sn.w *= sin_sign;
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    const float cs[4] = {c.x, c.y, c.z, c.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float a = __uint_as_float(w[k] << 16), b = __uint_as_float(w[k] & 0xffff0000u);
      const __nv_bfloat162 r = __floats2bfloat162_rn(a * cs[k] - b * ss[k], a * ss[k] + b * cs[k]);
      o[k] = *reinterpret_cast<const uint32_t*>(&r);
    }
    *reinterpret_cast<uint4*>(y + th * hd + q * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace

extern "C" {

const char* rtp_gate_last_error(void) { return g_err.c_str(); }

int rtp_top2_gate_fwd(const float* logits, const float* noise, float* gates, int* idx, int* loc, float* gate_w,
                      unsigned char* valid, float* me_sum, float* ce, float* l_aux, int S, int E, int capacity,
                      void* stream) {
  if (E < 1 || E > kMaxE) { g_err = "top2 gate: number of experts must be in [1, 64]"; return -1; }
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(me_sum, 0, sizeof(float) * E, st);
  if (e != cudaSuccess) return fail("top2 gate memset", e);
  int grid = (S + 7) / 8;
  if (grid > 148 * 4) grid = 148 * 4;
  gate_rows_kernel<<<grid, 256, 0, st>>>(logits, noise, gates, idx, me_sum, S, E);
  gate_slots_kernel<<<1, 1024, 0, st>>>(gates, idx, me_sum, loc, gate_w, valid, ce, l_aux, S, E, capacity);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail("top2 gate", e);
  return 0;
}

int rtp_top2_gate_bwd(const float* gates, const int* idx, const unsigned char* valid, const float* ce,
                      const float* d_gate_w, const float* d_l_aux, float* dlogits, int S, int E, void* stream) {
  if (E < 1 || E > kMaxE) { g_err = "top2 gate: number of experts must be in [1, 64]"; return -1; }
  int grid = (S + 7) / 8;
  if (grid > 148 * 4) grid = 148 * 4;
  gate_bwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(gates, idx, valid, ce, d_gate_w, d_l_aux, dlogits, S, E);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail("top2 gate backward", e);
  return 0;
}

// x, y: [T, H, hd] bf16 (may alias); cos, sin: [S, hd / 2] fp32; position of token t = (t / inner) % S.
// backward = 1 applies the inverse rotation (the gradient of the forward map).
int rtp_rope(const void* x, void* y, const float* cosv, const float* sinv, long long T, int H, int hd, int S, int inner,
             int backward, void* stream) {
  if (hd % 16) { g_err = "rope: head_dim must be a multiple of 16"; return -1; }
  if (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(cosv) |
        reinterpret_cast<uintptr_t>(sinv)) & 15) != 0) { g_err = "rope: operands must be 16-byte aligned"; return -1; }
  const long long total = T * H * (hd / 16);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) return 0;
  rope_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, cosv, sinv, T,
                                                                 H, hd, S, inner, backward ? -1.f : 1.f);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail("rope", e);
  return 0;
}

}  // extern "C"
