// Memory-bound kernels of the training step, written for sm_100a: fused dropout+residual+LayerNorm
// (and RMSNorm), softmax cross-entropy (loss and logit gradient in one pass over the row), rotated
// embedding gather/scatter, short-sequence causal attention, column sums for bias gradients,
// multi-tensor Adam(W) with value clipping, and small elementwise helpers.
// All tensors are bf16 unless stated; statistics and reductions are fp32.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <string>
#include <cooperative_groups.h>
#include "common.cuh"
#include "launch.h"
#include "kernels.h"

using namespace rtp;

namespace {
thread_local std::string k_err;
int kfail(const char* what, cudaError_t e) {
  k_err = std::string(what) + ": " + cudaGetErrorString(e);
  return -1;
}
#define LAUNCH_CHECK(name)                                 \
  do {                                                     \
    cudaError_t e__ = cudaGetLastError();                  \
    if (e__ != cudaSuccess) return kfail(name, e__);       \
  } while (0)

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// block-wide sum over up to 1024 threads; `red` is a 32-float smem scratch
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
  if (w == 0) t = warp_sum(t);
  if (threadIdx.x == 0) red[0] = t;
  __syncthreads();
  return red[0];
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < nw) ? red[threadIdx.x] : -INFINITY;
  if (w == 0) t = warp_max(t);
  if (threadIdx.x == 0) red[0] = t;
  __syncthreads();
  return red[0];
}
__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  f[0] = bf16_lo(u.x); f[1] = bf16_hi(u.x); f[2] = bf16_lo(u.y); f[3] = bf16_hi(u.y);
  f[4] = bf16_lo(u.z); f[5] = bf16_hi(u.z); f[6] = bf16_lo(u.w); f[7] = bf16_hi(u.w);
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
}
// dropout keep flags for 8 consecutive elements starting at e (e % 8 == 0)
__device__ __forceinline__ void keep8(uint64_t seed, uint64_t offset, uint64_t e, uint32_t thresh, bool* k) {
  uint4 r0 = philox4x32(seed, offset, e >> 2), r1 = philox4x32(seed, offset, (e >> 2) + 1);
  k[0] = r0.x >= thresh; k[1] = r0.y >= thresh; k[2] = r0.z >= thresh; k[3] = r0.w >= thresh;
  k[4] = r1.x >= thresh; k[5] = r1.y >= thresh; k[6] = r1.z >= thresh; k[7] = r1.w >= thresh;
}
uint32_t host_thresh(float p) {
  if (p <= 0.f) return 0;
  double t = (double)p * 4294967296.0;
  if (t > 4294967295.0) t = 4294967295.0;
  return (uint32_t)t;
}

// ------------------------------------------------------------------------------------------------
// h = x + dropout(sub);  y = norm(h) * gamma (+ beta).  rms = 0: LayerNorm, 1: RMSNorm.
// One 256-thread block per row; the row lives in registers (NG groups of 8 columns per thread, D <= 2048 * NG), so
// global memory is touched exactly once per tensor.  Saves h (bf16) and the row statistics for backward.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float2 block_sum2(float a, float b, float2* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  a = warp_sum(a);
  b = warp_sum(b);
  __syncthreads();
  if (lane == 0) red[w] = make_float2(a, b);
  __syncthreads();
  float2 t = (lane < nw) ? red[lane] : make_float2(0.f, 0.f);
  t.x = warp_sum(t.x);
  t.y = warp_sum(t.y);
  return t;
}

template <int NG>
__global__ void __launch_bounds__(256) norm_fwd_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ sub, const __nv_bfloat16* __restrict__ gamma,
    const __nv_bfloat16* __restrict__ beta, __nv_bfloat16* __restrict__ h_out, __nv_bfloat16* __restrict__ y,
    float* __restrict__ mean_out, float* __restrict__ rstd_out, int M, int D, float eps, int rms, uint32_t thresh,
    float drop_scale, uint64_t seed, uint64_t offset, const unsigned long long* __restrict__ step_ptr) {
  __shared__ float2 red[32];
  if (step_ptr) offset += __ldg(step_ptr) * 65536ull;
  float g[NG][8], bt[NG][8];
#pragma unroll
  for (int q = 0; q < NG; ++q) {
    const int c = (q * 256 + threadIdx.x) * 8;
    if (c < D) {
      unpack8(*reinterpret_cast<const uint4*>(gamma + c), g[q]);
      if (beta) unpack8(*reinterpret_cast<const uint4*>(beta + c), bt[q]);
      else {
#pragma unroll
        for (int i = 0; i < 8; ++i) bt[q][i] = 0.f;
      }
    }
  }
  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    const size_t base = (size_t)row * D;
    float v[NG][8];
    float s = 0.f;
#pragma unroll
    for (int q = 0; q < NG; ++q) {
      const int c = (q * 256 + threadIdx.x) * 8;
      if (c < D) {
        unpack8(__ldcs(reinterpret_cast<const uint4*>(x + base + c)), v[q]);
        if (sub) {
          float u[8];
          unpack8(__ldcs(reinterpret_cast<const uint4*>(sub + base + c)), u);
          if (thresh) {
            bool k[8];
            keep8(seed, offset, base + c, thresh, k);
#pragma unroll
            for (int i = 0; i < 8; ++i) u[i] = k[i] ? u[i] * drop_scale : 0.f;
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) v[q][i] += u[i];
        }
        const uint4 hp = pack8(v[q]);   // round to bf16 first: backward sees exactly the saved h
        unpack8(hp, v[q]);
        if (h_out) *reinterpret_cast<uint4*>(h_out + base + c) = hp;
#pragma unroll
        for (int i = 0; i < 8; ++i) s += v[q][i];
      }
    }
    float mean = 0.f;
    if (!rms) mean = block_sum2(s, 0.f, red).x / D;
    float qq = 0.f;
#pragma unroll
    for (int q = 0; q < NG; ++q) {
      const int c = (q * 256 + threadIdx.x) * 8;
      if (c < D) {
#pragma unroll
        for (int i = 0; i < 8; ++i) { const float d = v[q][i] - mean; qq += d * d; }
      }
    }
    const float var = block_sum2(qq, 0.f, red).x / D;
    const float rstd = rsqrtf(var + eps);
    if (threadIdx.x == 0) {
      if (mean_out) mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
#pragma unroll
    for (int q = 0; q < NG; ++q) {
      const int c = (q * 256 + threadIdx.x) * 8;
      if (c < D) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = (v[q][i] - mean) * rstd * g[q][i] + bt[q][i];
        *reinterpret_cast<uint4*>(y + base + c) = pack8(o);
      }
    }
  }
}

// Backward: dh = d(norm)/dh (+ dres); dx = dh; dsub = dropout_mask * dh.  Per-thread dgamma / dbeta partials stay in
// registers across the rows of the block and are added to the fp32 outputs with one atomic per column at the end.
template <int NG>
__global__ void __launch_bounds__(256) norm_bwd_kernel(
    const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ gamma,
    const float* __restrict__ mean_in, const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
    __nv_bfloat16* __restrict__ dsub, float* __restrict__ dgamma, float* __restrict__ dbeta, int M, int D, int rms,
    uint32_t thresh, float drop_scale, uint64_t seed, uint64_t offset, const __nv_bfloat16* __restrict__ dres,
    const unsigned long long* __restrict__ step_ptr, int vec_atomics) {
  __shared__ float2 red[32];
  if (step_ptr) offset += __ldg(step_ptr) * 65536ull;
  float g[NG][8], pg[NG][8], pb[NG][8];
#pragma unroll
  for (int q = 0; q < NG; ++q) {
    const int c = (q * 256 + threadIdx.x) * 8;
    if (c < D) unpack8(*reinterpret_cast<const uint4*>(gamma + c), g[q]);
#pragma unroll
    for (int i = 0; i < 8; ++i) { pg[q][i] = 0.f; pb[q][i] = 0.f; }
  }
  // raw rows are fetched one row ahead, so that the loads of row i+1 are in flight during the block reduction of row i
  uint4 nd[NG], nh[NG];
  if (blockIdx.x < M) {
#pragma unroll
    for (int q = 0; q < NG; ++q) {
      const int c = (q * 256 + threadIdx.x) * 8;
      if (c < D) {
        nd[q] = __ldcs(reinterpret_cast<const uint4*>(dy + (size_t)blockIdx.x * D + c));
        nh[q] = __ldcs(reinterpret_cast<const uint4*>(h + (size_t)blockIdx.x * D + c));
      }
    }
  }
  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    const size_t base = (size_t)row * D;
    const float mean = rms ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    float d[NG][8], xh[NG][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int q = 0; q < NG; ++q) {
      const int c = (q * 256 + threadIdx.x) * 8;
      if (c < D) {
        float hv[8];
        unpack8(nd[q], d[q]);
        unpack8(nh[q], hv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[q][i] = (hv[i] - mean) * rstd;
          const float dg = d[q][i] * g[q][i];
          s1 += dg;
          s2 += dg * xh[q][i];
          pg[q][i] += d[q][i] * xh[q][i];
          pb[q][i] += d[q][i];
        }
      }
    }
    const int nrow = row + gridDim.x;
    if (nrow < M) {
#pragma unroll
      for (int q = 0; q < NG; ++q) {
        const int c = (q * 256 + threadIdx.x) * 8;
        if (c < D) {
          nd[q] = __ldcs(reinterpret_cast<const uint4*>(dy + (size_t)nrow * D + c));
          nh[q] = __ldcs(reinterpret_cast<const uint4*>(h + (size_t)nrow * D + c));
        }
      }
    }
    const float2 t = block_sum2(s1, s2, red);
    s1 = rms ? 0.f : t.x / D;
    s2 = t.y / D;
#pragma unroll
    for (int q = 0; q < NG; ++q) {
      const int c = (q * 256 + threadIdx.x) * 8;
      if (c < D) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = (d[q][i] * g[q][i] - s1 - xh[q][i] * s2) * rstd;
        if (dres) {   // gradient that reaches h along a second path (pre-norm residual stream)
          float e[8];
          unpack8(__ldcs(reinterpret_cast<const uint4*>(dres + base + c)), e);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += e[i];
        }
        *reinterpret_cast<uint4*>(dx + base + c) = pack8(o);
        if (dsub) {
          if (thresh) {
            bool k[8];
            keep8(seed, offset, base + c, thresh, k);
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = k[i] ? o[i] * drop_scale : 0.f;
          }
          *reinterpret_cast<uint4*>(dsub + base + c) = pack8(o);
        }
      }
    }
  }
#pragma unroll
  for (int q = 0; q < NG; ++q) {
    const int c = (q * 256 + threadIdx.x) * 8;
    if (c < D) {
      if (!vec_atomics) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          atomicAdd(dgamma + c + i, pg[q][i]);
          if (dbeta) atomicAdd(dbeta + c + i, pb[q][i]);
        }
        continue;
      }
      // 16-byte vector reductions: four columns per atomic
      atomicAdd(reinterpret_cast<float4*>(dgamma + c), make_float4(pg[q][0], pg[q][1], pg[q][2], pg[q][3]));
      atomicAdd(reinterpret_cast<float4*>(dgamma + c + 4), make_float4(pg[q][4], pg[q][5], pg[q][6], pg[q][7]));
      if (dbeta) {
        atomicAdd(reinterpret_cast<float4*>(dbeta + c), make_float4(pb[q][0], pb[q][1], pb[q][2], pb[q][3]));
        atomicAdd(reinterpret_cast<float4*>(dbeta + c + 4), make_float4(pb[q][4], pb[q][5], pb[q][6], pb[q][7]));
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Softmax cross-entropy over rows of bf16 logits [M, V] (row pitch ld). Writes the per-row loss (fp32)
// and overwrites the logits with grad_scale * (softmax - onehot), i.e. the gradient of
// grad_scale * sum_rows(loss). Rows whose target equals ignore_index give zero loss and gradient.
// ------------------------------------------------------------------------------------------------
__global__ void ce_kernel(__nv_bfloat16* logits, long long ld, const long long* __restrict__ target,
                          float* __restrict__ loss, int M, int V, float grad_scale, long long ignore_index,
                          int write_grad, __nv_bfloat16* grad, long long ldg) {
  __shared__ float red[32];
  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    __nv_bfloat16* lp = logits + (size_t)row * ld;
    __nv_bfloat16* gp = grad ? grad + (size_t)row * ldg : lp;   // the gradient may go to a buffer of its own
    const long long t = target[row];
    float mx = -INFINITY;
    for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
      float v[8];
      unpack8(*reinterpret_cast<const uint4*>(lp + c), v);
#pragma unroll
      for (int i = 0; i < 8; ++i) mx = fmaxf(mx, v[i]);
    }
    mx = block_max(mx, red);
    float se = 0.f;
    for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
      float v[8];
      unpack8(*reinterpret_cast<const uint4*>(lp + c), v);
#pragma unroll
      for (int i = 0; i < 8; ++i) se += __expf(v[i] - mx);
    }
    se = block_sum(se, red);
    const float lse = mx + __logf(se);
    const bool ignored = (t == ignore_index) || t < 0 || t >= V;
    if (threadIdx.x == 0) loss[row] = ignored ? 0.f : lse - __bfloat162float(lp[t]);
    __syncthreads();
    if (write_grad) {
      const float inv = 1.f / se;
      for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
        float v[8];
        unpack8(*reinterpret_cast<const uint4*>(lp + c), v);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float p = __expf(v[i] - mx) * inv;
          if (c + i == t) p -= 1.f;
          v[i] = ignored ? 0.f : p * grad_scale;
        }
        *reinterpret_cast<uint4*>(gp + c) = pack8(v);
      }
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------------------------
// Embedding gather for one visiting table shard [V, Ds]: out[t, col_off + c] =
//   dropout(table[ids[t], c] * scale + pe[t / tokens_per_pos, col_off + c])
// ------------------------------------------------------------------------------------------------
__global__ void embed_fwd_kernel(const __nv_bfloat16* __restrict__ table, const long long* __restrict__ ids,
                                 const __nv_bfloat16* __restrict__ pe, long long ld_pe, int tokens_per_pos,
                                 __nv_bfloat16* __restrict__ out, long long ld_out, int col_off, int T, int Ds, int D,
                                 float scale, uint32_t thresh, float drop_scale, uint64_t seed, uint64_t offset,
                                 const unsigned long long* __restrict__ step_ptr) {
  if (step_ptr) offset += __ldg(step_ptr) * 65536ull;
  const int per_row = Ds / 8;
  const long long total = (long long)T * per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / per_row), c = (int)(i % per_row) * 8;
    float v[8];
    unpack8(*reinterpret_cast<const uint4*>(table + (size_t)ids[t] * Ds + c), v);
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] *= scale;
    if (pe) {
      float p[8];
      unpack8(*reinterpret_cast<const uint4*>(pe + (size_t)(t / tokens_per_pos) * ld_pe + col_off + c), p);
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] += p[k];
    }
    if (thresh) {
      bool kp[8];
      keep8(seed, offset, (uint64_t)t * D + col_off + c, thresh, kp);
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] = kp[k] ? v[k] * drop_scale : 0.f;
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * ld_out + col_off + c) = pack8(v);
  }
}
// Scatter-add of the output gradient into a (zeroed or incoming) table-shard gradient [V, Ds].
// blk_cols > 0: gtable is block-major, [Ds / blk_cols][V][blk_cols] (one contiguous [V, blk_cols] block per owner of an
// embedding-dim shard); blk_cols = 0: plain [V, Ds].
__global__ void embed_bwd_kernel(__nv_bfloat16* __restrict__ gtable, const long long* __restrict__ ids,
                                 const __nv_bfloat16* __restrict__ dy, long long ld_dy, int col_off, int T, int Ds,
                                 int D, float scale, uint32_t thresh, float drop_scale, uint64_t seed, uint64_t offset,
                                 const unsigned long long* __restrict__ step_ptr, int blk_cols, int V) {
  if (step_ptr) offset += __ldg(step_ptr) * 65536ull;
  const int per_row = Ds / 8;
  const long long total = (long long)T * per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / per_row), c = (int)(i % per_row) * 8;
    float v[8];
    unpack8(*reinterpret_cast<const uint4*>(dy + (size_t)t * ld_dy + col_off + c), v);
    if (thresh) {
      bool kp[8];
      keep8(seed, offset, (uint64_t)t * D + col_off + c, thresh, kp);
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] = kp[k] ? v[k] * drop_scale : 0.f;
    }
    __nv_bfloat162* g = blk_cols > 0
        ? reinterpret_cast<__nv_bfloat162*>(gtable + ((size_t)(c / blk_cols) * V + (size_t)ids[t]) * blk_cols + (c % blk_cols))
        : reinterpret_cast<__nv_bfloat162*>(gtable + (size_t)ids[t] * Ds + c);
#pragma unroll
    for (int k = 0; k < 4; ++k) atomicAdd(g + k, __floats2bfloat162_rn(v[2 * k] * scale, v[2 * k + 1] * scale));
  }
}

// ------------------------------------------------------------------------------------------------
// Short-sequence attention (S <= 128, head_dim 64) on packed projections.
// qkv: [T, 3*D] with T = S*B tokens (token = s*B + b). The projection comes out of a column-rotated
// linear, so its columns are grouped per shard: shard j holds [q_j | k_j | v_j], each D/nshard wide.
// out: [T, D], column = head*64 + d. One block per (batch, head).
// ------------------------------------------------------------------------------------------------
constexpr int kHd = 64;
__device__ __forceinline__ int qkv_col(int head, int which, int D, int nshard, int heads) {
  const int hps = heads / nshard;  // heads per shard
  const int j = head / hps, hl = head % hps;
  return j * (3 * (D / nshard)) + which * (D / nshard) + hl * kHd;
}

__global__ void attn_small_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ out, int S,
                                      int B, int heads, int nshard, int causal, float sm_scale, uint32_t thresh,
                                      float drop_scale, uint64_t seed, uint64_t offset,
                                      const unsigned long long* __restrict__ step_ptr) {
  extern __shared__ float smf[];
  if (step_ptr) offset += __ldg(step_ptr) * 65536ull;
  const int D = heads * kHd;
  const int b = blockIdx.x / heads, h = blockIdx.x % heads;
  float* q = smf;                 // [S][65]
  float* k = q + S * 65;
  float* v = k + S * 65;
  float* p = v + S * 65;          // [S][S+1]
  const int cq = qkv_col(h, 0, D, nshard, heads), ck = qkv_col(h, 1, D, nshard, heads), cv = qkv_col(h, 2, D, nshard, heads);
  for (int i = threadIdx.x; i < S * 8; i += blockDim.x) {
    const int s = i / 8, c = (i % 8) * 8;
    const size_t rowp = (size_t)(s * B + b) * (3 * D);
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(qkv + rowp + cq + c), f);
    for (int e = 0; e < 8; ++e) q[s * 65 + c + e] = f[e] * sm_scale;
    unpack8(*reinterpret_cast<const uint4*>(qkv + rowp + ck + c), f);
    for (int e = 0; e < 8; ++e) k[s * 65 + c + e] = f[e];
    unpack8(*reinterpret_cast<const uint4*>(qkv + rowp + cv + c), f);
    for (int e = 0; e < 8; ++e) v[s * 65 + c + e] = f[e];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) {
    const int r = i / S, c = i % S;
    float acc = -INFINITY;
    if (!causal || c <= r) {
      acc = 0.f;
#pragma unroll 16
      for (int e = 0; e < kHd; ++e) acc += q[r * 65 + e] * k[c * 65 + e];
    }
    p[r * (S + 1) + c] = acc;
  }
  __syncthreads();
  // softmax per row: one warp per row
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int r = warp; r < S; r += nw) {
    float mx = -INFINITY;
    for (int c = lane; c < S; c += 32) mx = fmaxf(mx, p[r * (S + 1) + c]);
    mx = warp_max(mx);
    float se = 0.f;
    for (int c = lane; c < S; c += 32) {
      float e = __expf(p[r * (S + 1) + c] - mx);
      p[r * (S + 1) + c] = e;
      se += e;
    }
    se = warp_sum(se);
    const float inv = 1.f / se;
    for (int c = lane; c < S; c += 32) {
      float pv = p[r * (S + 1) + c] * inv;
      if (thresh) {
        const uint64_t e = ((uint64_t)blockIdx.x * S + r) * S + c;
        pv = dropout_keep(seed, offset, e, thresh) ? pv * drop_scale : 0.f;
      }
      p[r * (S + 1) + c] = pv;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < S * kHd; i += blockDim.x) {
    const int r = i / kHd, e = i % kHd;
    float acc = 0.f;
    const int lim = causal ? r + 1 : S;
    for (int c = 0; c < lim; ++c) acc += p[r * (S + 1) + c] * v[c * 65 + e];
    out[(size_t)(r * B + b) * D + h * kHd + e] = __float2bfloat16(acc);
  }
}

__global__ void attn_small_bwd_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ dout,
                                      __nv_bfloat16* __restrict__ dqkv, int S, int B, int heads, int nshard,
                                      int causal, float sm_scale, uint32_t thresh, float drop_scale, uint64_t seed,
                                      uint64_t offset, const unsigned long long* __restrict__ step_ptr) {
  extern __shared__ float smf[];
  if (step_ptr) offset += __ldg(step_ptr) * 65536ull;
  const int D = heads * kHd;
  const int b = blockIdx.x / heads, h = blockIdx.x % heads;
  float* q = smf;                 // [S][65] (pre-scaled)
  float* k = q + S * 65;
  float* v = k + S * 65;
  float* go = v + S * 65;         // dO
  float* p = go + S * 65;         // [S][S+1] softmax probabilities (no dropout)
  float* ds = p + S * (S + 1);    // [S][S+1] dP then dS
  const int cq = qkv_col(h, 0, D, nshard, heads), ck = qkv_col(h, 1, D, nshard, heads), cv = qkv_col(h, 2, D, nshard, heads);
  for (int i = threadIdx.x; i < S * 8; i += blockDim.x) {
    const int s = i / 8, c = (i % 8) * 8;
    const size_t rowp = (size_t)(s * B + b) * (3 * D);
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(qkv + rowp + cq + c), f);
    for (int e = 0; e < 8; ++e) q[s * 65 + c + e] = f[e] * sm_scale;
    unpack8(*reinterpret_cast<const uint4*>(qkv + rowp + ck + c), f);
    for (int e = 0; e < 8; ++e) k[s * 65 + c + e] = f[e];
    unpack8(*reinterpret_cast<const uint4*>(qkv + rowp + cv + c), f);
    for (int e = 0; e < 8; ++e) v[s * 65 + c + e] = f[e];
    unpack8(*reinterpret_cast<const uint4*>(dout + (size_t)(s * B + b) * D + h * kHd + c), f);
    for (int e = 0; e < 8; ++e) go[s * 65 + c + e] = f[e];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) {
    const int r = i / S, c = i % S;
    float acc = -INFINITY, dp = 0.f;
    if (!causal || c <= r) {
      acc = 0.f;
#pragma unroll 16
      for (int e = 0; e < kHd; ++e) {
        acc += q[r * 65 + e] * k[c * 65 + e];
        dp += go[r * 65 + e] * v[c * 65 + e];
      }
    }
    p[r * (S + 1) + c] = acc;
    ds[r * (S + 1) + c] = dp;   // dP of the dropped probabilities
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int r = warp; r < S; r += nw) {
    float mx = -INFINITY;
    for (int c = lane; c < S; c += 32) mx = fmaxf(mx, p[r * (S + 1) + c]);
    mx = warp_max(mx);
    float se = 0.f;
    for (int c = lane; c < S; c += 32) {
      float e = __expf(p[r * (S + 1) + c] - mx);
      p[r * (S + 1) + c] = e;
      se += e;
    }
    se = warp_sum(se);
    const float inv = 1.f / se;
    float dot = 0.f;
    for (int c = lane; c < S; c += 32) {
      const float pv = p[r * (S + 1) + c] * inv;
      float m = 1.f;
      if (thresh) {
        const uint64_t e = ((uint64_t)blockIdx.x * S + r) * S + c;
        m = dropout_keep(seed, offset, e, thresh) ? drop_scale : 0.f;
      }
      const float dpv = ds[r * (S + 1) + c] * m;  // gradient wrt the un-dropped probability
      p[r * (S + 1) + c] = pv;
      ds[r * (S + 1) + c] = dpv;
      dot += dpv * pv;
    }
    dot = warp_sum(dot);
    for (int c = lane; c < S; c += 32) {
      const float pv = p[r * (S + 1) + c];
      const float dsv = pv * (ds[r * (S + 1) + c] - dot);
      // keep the dropped probability in p for dV
      float m = 1.f;
      if (thresh) {
        const uint64_t e = ((uint64_t)blockIdx.x * S + r) * S + c;
        m = dropout_keep(seed, offset, e, thresh) ? drop_scale : 0.f;
      }
      p[r * (S + 1) + c] = pv * m;
      ds[r * (S + 1) + c] = dsv;
    }
  }
  __syncthreads();
  // dQ = dS K * scale ; dK = dS^T Q(pre-scaled) ; dV = Pd^T dO
  for (int i = threadIdx.x; i < S * kHd; i += blockDim.x) {
    const int r = i / kHd, e = i % kHd;
    float dq = 0.f, dk = 0.f, dv = 0.f;
    for (int c = 0; c < S; ++c) {
      dq += ds[r * (S + 1) + c] * k[c * 65 + e];
      dk += ds[c * (S + 1) + r] * q[c * 65 + e];
      dv += p[c * (S + 1) + r] * go[c * 65 + e];
    }
    const size_t rowp = (size_t)(r * B + b) * (3 * D);
    dqkv[rowp + cq + e] = __float2bfloat16(dq * sm_scale);
    dqkv[rowp + ck + e] = __float2bfloat16(dk);
    dqkv[rowp + cv + e] = __float2bfloat16(dv);
  }
}

// ------------------------------------------------------------------------------------------------
// Column sums of a bf16 matrix [M, N] (pitch ld) into fp32 out[N] (must be zeroed by the caller).
// ------------------------------------------------------------------------------------------------
__global__ void colsum_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int M, int N, float* __restrict__ out,
                              int rows_per_block) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (c >= N) return;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(M, r0 + rows_per_block);
  float a0 = 0.f, a1 = 0.f;
  for (int r = r0; r < r1; ++r) {
    const uint32_t u = *reinterpret_cast<const uint32_t*>(x + (size_t)r * ld + c);
    a0 += bf16_lo(u);
    a1 += bf16_hi(u);
  }
  atomicAdd(out + c, a0);
  atomicAdd(out + c + 1, a1);
}

// Vector variant: a block of 256 threads owns 64 columns (8 column lanes x 16 bytes) and a range of rows (32 row lanes,
// up to 8 loads in flight per thread); the row lanes are combined in shared memory.  The blocks that share a column
// group form a thread-block cluster along y: each leaves its 64 partial sums in its own shared memory, and the first
// block of the cluster adds them up through distributed shared memory and stores the result (no atomics, no zero-fill).
__global__ void __launch_bounds__(256) colsum_vec_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int M, int N,
                                                         float* __restrict__ out, int rows_per_block, int atomic) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ float red[32][65];
  __shared__ float part[64];
  const int cl = threadIdx.x & 7, rl = threadIdx.x >> 3;
  const int c = blockIdx.x * 64 + cl * 8;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(M, r0 + rows_per_block);
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  if (c < N) {
    int r = r0 + rl;
    for (; r + 7 * 32 < r1; r += 8 * 32) {
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = __ldcs(reinterpret_cast<const uint4*>(x + (size_t)(r + u * 32) * ld + c));
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        float f[8];
        unpack8(v[u], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += f[i];
      }
    }
    for (; r + 3 * 32 < r1; r += 4 * 32) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = __ldcs(reinterpret_cast<const uint4*>(x + (size_t)(r + u * 32) * ld + c));
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float f[8];
        unpack8(v[u], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += f[i];
      }
    }
    for (; r < r1; r += 32) {
      float f[8];
      unpack8(__ldcs(reinterpret_cast<const uint4*>(x + (size_t)r * ld + c)), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[rl][cl * 8 + i] = acc[i];
  __syncthreads();
  if (threadIdx.x < 64) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 32; ++k) t += red[k][threadIdx.x];
    part[threadIdx.x] = t;
  }
  cluster.sync();
  if (cluster.block_rank() == 0 && threadIdx.x < 64) {
    const int col = blockIdx.x * 64 + threadIdx.x;
    float t = 0.f;
    for (unsigned k = 0; k < cluster.num_blocks(); ++k) t += cluster.map_shared_rank(part, k)[threadIdx.x];
    if (col < N) {
      if (atomic) atomicAdd(out + col, t); else out[col] = t;
    }
  }
  cluster.sync();   // no block leaves while its shared memory may still be read
}

// ------------------------------------------------------------------------------------------------
// Multi-tensor Adam / AdamW with optional gradient value clipping.
// ------------------------------------------------------------------------------------------------
struct AdamRegs {
  float pv[8], gv[8], mv[8], vv[8];
  long long i0;
  int cnt;
  bool vec, svec;
};
// loads of one group of up to 8 elements (issued for both groups of a thread before either is updated)
__device__ __forceinline__ void adam_load(const RtpAdamTensor& t, long long i0, AdamRegs& r) {
  r.i0 = i0;
  r.cnt = i0 < t.n ? (int)min((long long)8, t.n - i0) : 0;
  if (r.cnt == 0) return;
  const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(t.p) + i0;
  const __nv_bfloat16* g = reinterpret_cast<const __nv_bfloat16*>(t.g) + i0;
  r.vec = r.cnt == 8 && ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g)) & 15) == 0;
  if (r.vec) {
    unpack8(__ldcs(reinterpret_cast<const uint4*>(p)), r.pv);
    unpack8(__ldcs(reinterpret_cast<const uint4*>(g)), r.gv);
  } else {
    _Pragma("unroll") for (int i = 0; i < 8; ++i) if (i < r.cnt) { r.pv[i] = __bfloat162float(p[i]); r.gv[i] = __bfloat162float(g[i]); }
  }
  // state_fp32: 0 = both moments bf16, 1 = both fp32, 2 = first moment bf16, second moment fp32
  r.svec = r.cnt == 8 && ((reinterpret_cast<uintptr_t>(t.m) | reinterpret_cast<uintptr_t>(t.v)) & 15) == 0;
  if (t.state_fp32 == 1) {
    const float* m = reinterpret_cast<const float*>(t.m) + i0;
    if (r.svec) {
      const float4 a = __ldcs(reinterpret_cast<const float4*>(m)), b = __ldcs(reinterpret_cast<const float4*>(m) + 1);
      r.mv[0] = a.x; r.mv[1] = a.y; r.mv[2] = a.z; r.mv[3] = a.w; r.mv[4] = b.x; r.mv[5] = b.y; r.mv[6] = b.z; r.mv[7] = b.w;
    } else {
      _Pragma("unroll") for (int i = 0; i < 8; ++i) if (i < r.cnt) r.mv[i] = m[i];
    }
  } else {
    const __nv_bfloat16* m = reinterpret_cast<const __nv_bfloat16*>(t.m) + i0;
    if (r.svec) unpack8(__ldcs(reinterpret_cast<const uint4*>(m)), r.mv);
    else { _Pragma("unroll") for (int i = 0; i < 8; ++i) if (i < r.cnt) r.mv[i] = __bfloat162float(m[i]); }
  }
  if (t.state_fp32 >= 1) {
    const float* v = reinterpret_cast<const float*>(t.v) + i0;
    if (r.svec) {
      const float4 c = __ldcs(reinterpret_cast<const float4*>(v)), d = __ldcs(reinterpret_cast<const float4*>(v) + 1);
      r.vv[0] = c.x; r.vv[1] = c.y; r.vv[2] = c.z; r.vv[3] = c.w; r.vv[4] = d.x; r.vv[5] = d.y; r.vv[6] = d.z; r.vv[7] = d.w;
    } else {
      _Pragma("unroll") for (int i = 0; i < 8; ++i) if (i < r.cnt) r.vv[i] = v[i];
    }
  } else {
    const __nv_bfloat16* v = reinterpret_cast<const __nv_bfloat16*>(t.v) + i0;
    if (r.svec) unpack8(__ldcs(reinterpret_cast<const uint4*>(v)), r.vv);
    else { _Pragma("unroll") for (int i = 0; i < 8; ++i) if (i < r.cnt) r.vv[i] = __bfloat162float(v[i]); }
  }
}
__device__ __forceinline__ void adam_update_store(const RtpAdamTensor& t, AdamRegs& r, float lr, float beta1, float beta2,
                                                  float eps, float weight_decay, int adamw, float clip_value,
                                                  float grad_scale, float step_size, float inv_sqrt_bc2) {
  if (r.cnt == 0) return;
  _Pragma("unroll") for (int i = 0; i < 8; ++i) if (i < r.cnt) {
    float gg = r.gv[i] * grad_scale;
    if (clip_value > 0.f) gg = fminf(fmaxf(gg, -clip_value), clip_value);
    if (weight_decay != 0.f) {
      if (adamw) r.pv[i] *= 1.f - lr * t.lr_mult * weight_decay; else gg += weight_decay * r.pv[i];
    }
    r.mv[i] = beta1 * r.mv[i] + (1.f - beta1) * gg;
    r.vv[i] = beta2 * r.vv[i] + (1.f - beta2) * gg * gg;
    r.pv[i] -= step_size * r.mv[i] / (sqrtf(r.vv[i]) * inv_sqrt_bc2 + eps);
  }
  __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(t.p) + r.i0;
  if (r.vec) __stcs(reinterpret_cast<uint4*>(p), pack8(r.pv));
  else { _Pragma("unroll") for (int i = 0; i < 8; ++i) if (i < r.cnt) p[i] = __float2bfloat16(r.pv[i]); }
  if (t.state_fp32 == 1) {
    float* m = reinterpret_cast<float*>(t.m) + r.i0;
    if (r.svec) {
      __stcs(reinterpret_cast<float4*>(m), make_float4(r.mv[0], r.mv[1], r.mv[2], r.mv[3]));
      __stcs(reinterpret_cast<float4*>(m) + 1, make_float4(r.mv[4], r.mv[5], r.mv[6], r.mv[7]));
    } else {
      _Pragma("unroll") for (int i = 0; i < 8; ++i) if (i < r.cnt) m[i] = r.mv[i];
    }
  } else {
    __nv_bfloat16* m = reinterpret_cast<__nv_bfloat16*>(t.m) + r.i0;
    if (r.svec) __stcs(reinterpret_cast<uint4*>(m), pack8(r.mv));
    else { _Pragma("unroll") for (int i = 0; i < 8; ++i) if (i < r.cnt) m[i] = __float2bfloat16(r.mv[i]); }
  }
  if (t.state_fp32 >= 1) {
    float* v = reinterpret_cast<float*>(t.v) + r.i0;
    if (r.svec) {
      __stcs(reinterpret_cast<float4*>(v), make_float4(r.vv[0], r.vv[1], r.vv[2], r.vv[3]));
      __stcs(reinterpret_cast<float4*>(v) + 1, make_float4(r.vv[4], r.vv[5], r.vv[6], r.vv[7]));
    } else {
      _Pragma("unroll") for (int i = 0; i < 8; ++i) if (i < r.cnt) v[i] = r.vv[i];
    }
  } else {
    __nv_bfloat16* v = reinterpret_cast<__nv_bfloat16*>(t.v) + r.i0;
    if (r.svec) __stcs(reinterpret_cast<uint4*>(v), pack8(r.vv));
    else { _Pragma("unroll") for (int i = 0; i < 8; ++i) if (i < r.cnt) v[i] = __float2bfloat16(r.vv[i]); }
  }
}

// One block = kAdamGroups x 2048 elements of one tensor; every thread owns one group of 8 elements in each 2048-element
// sub-chunk and has the loads of all its groups in flight before it updates the first.
constexpr int kAdamGroups = 2;
__global__ void __launch_bounds__(256, 4) adam_kernel(const RtpAdamTensor* __restrict__ tensors,
                                                   const int* __restrict__ block_start, int ntensors,
                                                   const long long* __restrict__ step_ptr, float lr, float beta1,
                                                   float beta2, float eps, float weight_decay, int adamw,
                                                   float clip_value, float grad_scale,
                                                   const int* __restrict__ block_tensor) {
  // locate the tensor this block works on: one load from the per-block table when the caller provides it
  int lo = 0, hi = ntensors - 1;
  if (block_tensor) {
    lo = block_tensor[blockIdx.x];
  } else {
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (block_start[mid] <= (int)blockIdx.x) lo = mid; else hi = mid - 1;
    }
  }
  const RtpAdamTensor t = tensors[lo];
  const long long step = *step_ptr;
  const float bc1 = 1.f - powf(beta1, (float)step);
  const float bc2 = 1.f - powf(beta2, (float)step);
  const float step_size = lr * t.lr_mult / bc1;
  const float inv_sqrt_bc2 = rsqrtf(bc2);
  const long long base = (long long)((int)blockIdx.x - block_start[lo]) * (256 * 8 * kAdamGroups);
  AdamRegs r[kAdamGroups];
#pragma unroll
  for (int u = 0; u < kAdamGroups; ++u) adam_load(t, base + u * (256 * 8) + threadIdx.x * 8, r[u]);
#pragma unroll
  for (int u = 0; u < kAdamGroups; ++u)
    adam_update_store(t, r[u], lr, beta1, beta2, eps, weight_decay, adamw, clip_value, grad_scale, step_size, inv_sqrt_bc2);
}

// ------------------------------------------------------------------------------------------------
// Causal softmax over rows of a score matrix stack [rows_total, S] (row r belongs to query i = r % S).
// In place: p[i, j] = softmax_j(scale * s[i, j]) for j <= i, 0 for j > i (those entries may hold anything).
// ------------------------------------------------------------------------------------------------
__global__ void causal_softmax_kernel(__nv_bfloat16* __restrict__ s, long long rows, int S, float scale) {
  __shared__ float red[32];
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    __nv_bfloat16* p = s + row * S;
    const int i = (int)(row % S);
    float mx = -INFINITY;
    for (int c = threadIdx.x * 8; c <= i; c += blockDim.x * 8) {
      float v[8];
      unpack8(*reinterpret_cast<const uint4*>(p + c), v);
#pragma unroll
      for (int k = 0; k < 8; ++k) if (c + k <= i) mx = fmaxf(mx, v[k] * scale);
    }
    mx = block_max(mx, red);
    float se = 0.f;
    for (int c = threadIdx.x * 8; c <= i; c += blockDim.x * 8) {
      float v[8];
      unpack8(*reinterpret_cast<const uint4*>(p + c), v);
#pragma unroll
      for (int k = 0; k < 8; ++k) if (c + k <= i) se += __expf(v[k] * scale - mx);
    }
    se = block_sum(se, red);
    const float inv = 1.f / se;
    for (int c = threadIdx.x * 8; c < S; c += blockDim.x * 8) {
      float v[8];
      if (c <= i) unpack8(*reinterpret_cast<const uint4*>(p + c), v);
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] = (c + k <= i) ? __expf(v[k] * scale - mx) * inv : 0.f;
      *reinterpret_cast<uint4*>(p + c) = pack8(v);
    }
    __syncthreads();
  }
}
// dS = scale * P * (dP - sum_j P dP), written over dP; entries above the diagonal become 0.
__global__ void causal_softmax_bwd_kernel(const __nv_bfloat16* __restrict__ pm, __nv_bfloat16* __restrict__ dp,
                                          long long rows, int S, float scale) {
  __shared__ float red[32];
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* p = pm + row * S;
    __nv_bfloat16* d = dp + row * S;
    const int i = (int)(row % S);
    float dot = 0.f;
    for (int c = threadIdx.x * 8; c <= i; c += blockDim.x * 8) {
      float a[8], b[8];
      unpack8(*reinterpret_cast<const uint4*>(p + c), a);
      unpack8(*reinterpret_cast<const uint4*>(d + c), b);
#pragma unroll
      for (int k = 0; k < 8; ++k) if (c + k <= i) dot += a[k] * b[k];
    }
    dot = block_sum(dot, red);
    for (int c = threadIdx.x * 8; c < S; c += blockDim.x * 8) {
      float a[8], b[8], o[8];
      if (c <= i) {
        unpack8(*reinterpret_cast<const uint4*>(p + c), a);
        unpack8(*reinterpret_cast<const uint4*>(d + c), b);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) o[k] = (c + k <= i) ? scale * a[k] * (b[k] - dot) : 0.f;
      *reinterpret_cast<uint4*>(d + c) = pack8(o);
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------------------------
// Activations (n % 8 == 0).  mode 0: y = gelu(x) (erf form).  mode 1: y = silu(g) * u with g, u the two column halves
// selected by pointers.  Backward kernels recompute from the saved pre-activations.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float gelu_f(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }
__device__ __forceinline__ float gelu_grad_f(float x) {
  const float cdf = 0.5f * (1.f + erff(x * 0.70710678118654752f));
  return cdf + x * 0.3989422804014327f * __expf(-0.5f * x * x);
}
__global__ void gelu_fwd_kernel(const __nv_bfloat16* x, __nv_bfloat16* y, long long n) {
  const long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;
  float v[8];
  unpack8(*reinterpret_cast<const uint4*>(x + i), v);
#pragma unroll
  for (int k = 0; k < 8; ++k) v[k] = gelu_f(v[k]);
  *reinterpret_cast<uint4*>(y + i) = pack8(v);
}
__global__ void gelu_bwd_kernel(const __nv_bfloat16* x, const __nv_bfloat16* dy, __nv_bfloat16* dx, long long n) {
  const long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;
  float v[8], g[8];
  unpack8(*reinterpret_cast<const uint4*>(x + i), v);
  unpack8(*reinterpret_cast<const uint4*>(dy + i), g);
#pragma unroll
  for (int k = 0; k < 8; ++k) v[k] = g[k] * gelu_grad_f(v[k]);
  *reinterpret_cast<uint4*>(dx + i) = pack8(v);
}
// g, u: [rows, cols] windows with pitch ld (elements); y dense [rows, cols]
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* g, const __nv_bfloat16* u, long long ld, __nv_bfloat16* y,
                                  long long rows, int cols) {
  const long long it = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const int per = cols / 8;
  if (it >= rows * per) return;
  const long long r = it / per;
  const int c = (int)(it % per) * 8;
  float a[8], b[8];
  unpack8(*reinterpret_cast<const uint4*>(g + r * ld + c), a);
  unpack8(*reinterpret_cast<const uint4*>(u + r * ld + c), b);
#pragma unroll
  for (int k = 0; k < 8; ++k) a[k] = a[k] / (1.f + __expf(-a[k])) * b[k];
  *reinterpret_cast<uint4*>(y + r * cols + c) = pack8(a);
}
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* g, const __nv_bfloat16* u, long long ld, const __nv_bfloat16* dy,
                                  __nv_bfloat16* dg, __nv_bfloat16* du, long long ldo, long long rows, int cols) {
  const long long it = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const int per = cols / 8;
  if (it >= rows * per) return;
  const long long r = it / per;
  const int c = (int)(it % per) * 8;
  float a[8], b[8], d[8], og[8], ou[8];
  unpack8(*reinterpret_cast<const uint4*>(g + r * ld + c), a);
  unpack8(*reinterpret_cast<const uint4*>(u + r * ld + c), b);
  unpack8(*reinterpret_cast<const uint4*>(dy + r * cols + c), d);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float sg = 1.f / (1.f + __expf(-a[k]));
    const float silu = a[k] * sg;
    ou[k] = d[k] * silu;
    og[k] = d[k] * b[k] * (sg + silu * (1.f - sg));
  }
  *reinterpret_cast<uint4*>(dg + r * ldo + c) = pack8(og);
  *reinterpret_cast<uint4*>(du + r * ldo + c) = pack8(ou);
}

// ------------------------------------------------------------------------------------------------
// MoE token movement by index (top-2): slot[s, k] is the destination row (expert * capacity + position) of choice k
// of token s, or -1.  One warp per (token, choice).  M % 8 == 0.
// ------------------------------------------------------------------------------------------------
__global__ void moe_scatter_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ slot,
                                   const float* __restrict__ scale, __nv_bfloat16* __restrict__ dst, int S, int M) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= 2 * S) return;
  const int sl = slot[w];
  if (sl < 0) return;
  const float sc = scale ? scale[w] : 1.f;
  const __nv_bfloat16* a = src + (size_t)(w >> 1) * M;
  __nv_bfloat16* d = dst + (size_t)sl * M;
  for (int c = lane * 8; c < M; c += 256) {
    float v[8];
    unpack8(*reinterpret_cast<const uint4*>(a + c), v);
    if (scale) {
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] *= sc;
    }
    *reinterpret_cast<uint4*>(d + c) = pack8(v);
  }
}
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ slot,
                                  const float* __restrict__ scale, __nv_bfloat16* __restrict__ dst, int S, int M) {
  const int s = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (s >= S) return;
  const int s0 = slot[2 * s], s1 = slot[2 * s + 1];
  const float g0 = scale ? scale[2 * s] : 1.f, g1 = scale ? scale[2 * s + 1] : 1.f;
  for (int c = lane * 8; c < M; c += 256) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, v[8];
    if (s0 >= 0) {
      unpack8(*reinterpret_cast<const uint4*>(src + (size_t)s0 * M + c), v);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += g0 * v[k];
    }
    if (s1 >= 0) {
      unpack8(*reinterpret_cast<const uint4*>(src + (size_t)s1 * M + c), v);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += g1 * v[k];
    }
    *reinterpret_cast<uint4*>(dst + (size_t)s * M + c) = pack8(acc);
  }
}
// out[s, k] = <a[s, :], b[slot[s, k], :]>
__global__ void moe_rowdot_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                  const int* __restrict__ slot, float* __restrict__ out, int S, int M) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= 2 * S) return;
  const int sl = slot[w];
  float acc = 0.f;
  if (sl >= 0) {
    const __nv_bfloat16* x = a + (size_t)(w >> 1) * M;
    const __nv_bfloat16* y = b + (size_t)sl * M;
    for (int c = lane * 8; c < M; c += 256) {
      float u[8], v[8];
      unpack8(*reinterpret_cast<const uint4*>(x + c), u);
      unpack8(*reinterpret_cast<const uint4*>(y + c), v);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc += u[k] * v[k];
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) out[w] = acc;
}

// out = a + b (bf16), n % 8 == 0 handled vectorised, tail scalar
__global__ void add_kernel(const __nv_bfloat16* a, const __nv_bfloat16* b, __nv_bfloat16* out, long long n) {
  const long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 8;
  if (i + 8 <= n) {
    float x[8], y[8];
    unpack8(*reinterpret_cast<const uint4*>(a + i), x);
    unpack8(*reinterpret_cast<const uint4*>(b + i), y);
    for (int k = 0; k < 8; ++k) x[k] += y[k];
    *reinterpret_cast<uint4*>(out + i) = pack8(x);
  } else {
    for (long long k = i; k < n; ++k) out[k] = __float2bfloat16(__bfloat162float(a[k]) + __bfloat162float(b[k]));
  }
}
// fp32 vector -> bf16 (used for LayerNorm parameter gradients accumulated in fp32)
__global__ void cast_f32_bf16_kernel(const float* in, __nv_bfloat16* out, long long n, float scale) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i < n) out[i] = __float2bfloat16(in[i] * scale);
}
// sum of fp32 vector * scale -> out[0] (single block)
__global__ void sum_kernel(const float* in, float* out, int n, float scale) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += in[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) out[0] = s * scale;
}

}  // namespace

extern "C" {

const char* rtp_kernels_last_error(void) { return k_err.c_str(); }

int rtp_norm_fwd(const void* x, const void* sub, const void* gamma, const void* beta, void* h_out, void* y,
                 float* mean, float* rstd, int M, int D, float eps, int rms, float drop_p, unsigned long long seed,
                 unsigned long long offset, const unsigned long long* step_ptr, void* stream) {
  if (D % 8 || D > 8192) { k_err = "norm: D must be a multiple of 8 and at most 8192"; return -1; }
  const int grid = M < 148 * 8 ? M : 148 * 8;
  const float ds = drop_p > 0.f ? 1.f / (1.f - drop_p) : 1.f;
  const int ng = (D + 2047) / 2048;
#define RTP_NORM_FWD(NG)                                                                                              \
  norm_fwd_kernel<NG><<<grid, 256, 0, (cudaStream_t)stream>>>(                                                       \
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)sub, (const __nv_bfloat16*)gamma, (const __nv_bfloat16*)beta,    \
      (__nv_bfloat16*)h_out, (__nv_bfloat16*)y, mean, rstd, M, D, eps, rms, host_thresh(drop_p), ds, seed, offset,    \
      step_ptr)
  if (ng == 1) RTP_NORM_FWD(1); else if (ng == 2) RTP_NORM_FWD(2); else if (ng == 3) RTP_NORM_FWD(3); else RTP_NORM_FWD(4);
#undef RTP_NORM_FWD
  LAUNCH_CHECK("norm_fwd");
  return 0;
}
int rtp_norm_bwd(const void* dy, const void* h, const void* gamma, const float* mean, const float* rstd, void* dx,
                 void* dsub, float* dgamma, float* dbeta, int M, int D, int rms, float drop_p,
                 unsigned long long seed, unsigned long long offset, const void* dres,
                 const unsigned long long* step_ptr, void* stream) {
  if (D % 8 || D > 8192) { k_err = "norm: D must be a multiple of 8 and at most 8192"; return -1; }
  int grid = 148 * 2;   // few blocks: every block ends with one vector atomic per 4 columns of dgamma / dbeta
  if (grid > M) grid = M;
  const float ds = drop_p > 0.f ? 1.f / (1.f - drop_p) : 1.f;
  const int ng = (D + 2047) / 2048;
  const int vec_atomics = ((reinterpret_cast<uintptr_t>(dgamma) | reinterpret_cast<uintptr_t>(dbeta)) & 15) == 0;
#define RTP_NORM_BWD(NG)                                                                                              \
  norm_bwd_kernel<NG><<<grid, 256, 0, (cudaStream_t)stream>>>(                                                       \
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)h, (const __nv_bfloat16*)gamma, mean, rstd, (__nv_bfloat16*)dx, \
      (__nv_bfloat16*)dsub, dgamma, dbeta, M, D, rms, host_thresh(drop_p), ds, seed, offset,                          \
      (const __nv_bfloat16*)dres, step_ptr, vec_atomics)
  if (ng == 1) RTP_NORM_BWD(1); else if (ng == 2) RTP_NORM_BWD(2); else if (ng == 3) RTP_NORM_BWD(3); else RTP_NORM_BWD(4);
#undef RTP_NORM_BWD
  LAUNCH_CHECK("norm_bwd");
  return 0;
}
int rtp_cross_entropy(void* logits, long long ld, const long long* target, float* loss, int M, int V, float grad_scale,
                      long long ignore_index, int write_grad, void* stream) {
  return rtp_cross_entropy_to(logits, ld, target, loss, M, V, grad_scale, ignore_index, write_grad, nullptr, 0, stream);
}
int rtp_cross_entropy_to(void* logits, long long ld, const long long* target, float* loss, int M, int V, float grad_scale,
                         long long ignore_index, int write_grad, void* grad, long long ldg, void* stream) {
  if (V % 8 || ld % 8 || (grad && ldg % 8)) { k_err = "cross_entropy: V and the row pitches must be multiples of 8"; return -1; }
  const int grid = M < 148 * 8 ? M : 148 * 8;
  ce_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)logits, ld, target, loss, M, V, grad_scale,
                                                    ignore_index, write_grad, (__nv_bfloat16*)grad, ldg);
  LAUNCH_CHECK("cross_entropy");
  return 0;
}
int rtp_embed_fwd(const void* table, const long long* ids, const void* pe, long long ld_pe, int tokens_per_pos,
                  void* out, long long ld_out, int col_off, int T, int Ds, int D, float scale, float drop_p,
                  unsigned long long seed, unsigned long long offset, const unsigned long long* step_ptr,
                  void* stream) {
  if (Ds % 8 || col_off % 8 || ld_out % 8) { k_err = "embed: widths must be multiples of 8"; return -1; }
  const long long total = (long long)T * (Ds / 8);
  int grid = (int)((total + 255) / 256);
  if (grid > 148 * 16) grid = 148 * 16;
  const float ds = drop_p > 0.f ? 1.f / (1.f - drop_p) : 1.f;
  embed_fwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)table, ids, (const __nv_bfloat16*)pe,
                                                           ld_pe, tokens_per_pos, (__nv_bfloat16*)out, ld_out, col_off,
                                                           T, Ds, D, scale, host_thresh(drop_p), ds, seed, offset,
                                                           step_ptr);
  LAUNCH_CHECK("embed_fwd");
  return 0;
}
int rtp_embed_bwd(void* gtable, const long long* ids, const void* dy, long long ld_dy, int col_off, int T, int Ds,
                  int D, float scale, float drop_p, unsigned long long seed, unsigned long long offset,
                  const unsigned long long* step_ptr, void* stream) {
  return rtp_embed_bwd_blocks(gtable, ids, dy, ld_dy, col_off, T, Ds, D, scale, drop_p, seed, offset, step_ptr, 0, 0, stream);
}
int rtp_embed_bwd_blocks(void* gtable, const long long* ids, const void* dy, long long ld_dy, int col_off, int T, int Ds,
                         int D, float scale, float drop_p, unsigned long long seed, unsigned long long offset,
                         const unsigned long long* step_ptr, int blk_cols, int V, void* stream) {
  if (Ds % 8 || col_off % 8 || ld_dy % 8 || blk_cols % 8 || (blk_cols > 0 && Ds % blk_cols)) {
    k_err = "embed: widths must be multiples of 8";
    return -1;
  }
  const long long total = (long long)T * (Ds / 8);
  int grid = (int)((total + 255) / 256);
  if (grid > 148 * 16) grid = 148 * 16;
  const float ds = drop_p > 0.f ? 1.f / (1.f - drop_p) : 1.f;
  embed_bwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)gtable, ids, (const __nv_bfloat16*)dy, ld_dy,
                                                           col_off, T, Ds, D, scale, host_thresh(drop_p), ds, seed,
                                                           offset, step_ptr, blk_cols, V);
  LAUNCH_CHECK("embed_bwd");
  return 0;
}
static int g_attn_tc = 1;
void rtp_set_attn_tc(int on) { g_attn_tc = on ? 1 : 0; }
static size_t attn_smem(int S, bool bwd) {
  size_t f = (size_t)(bwd ? 4 : 3) * S * 65 + (size_t)(bwd ? 2 : 1) * S * (S + 1);
  return f * sizeof(float);
}
int rtp_attn_small_fwd(const void* qkv, void* out, int S, int B, int heads, int nshard, int causal, float sm_scale,
                       float drop_p, unsigned long long seed, unsigned long long offset,
                       const unsigned long long* step_ptr, void* stream) {
  if (g_attn_tc && rtp_attn_tc_supported(S, heads, nshard)) {
    const int rc = rtp_attn_tc_fwd(qkv, out, S, B, heads, nshard, causal, sm_scale, drop_p, seed, offset, step_ptr, stream);
    if (rc) k_err = rtp_attn_tc_last_error();
    return rc;
  }
  if (S > 128 || heads % nshard) { k_err = "attn_small: S must be <= 128 and heads divisible by shards"; return -1; }
  const size_t smem = attn_smem(S, false);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(attn_small_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return kfail("attn fwd attr", e);
  }
  const float ds = drop_p > 0.f ? 1.f / (1.f - drop_p) : 1.f;
  attn_small_fwd_kernel<<<B * heads, 128, smem, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)qkv, (__nv_bfloat16*)out, S, B, heads, nshard, causal, sm_scale, host_thresh(drop_p), ds,
      seed, offset, step_ptr);
  LAUNCH_CHECK("attn_small_fwd");
  return 0;
}
int rtp_attn_small_bwd(const void* qkv, const void* dout, void* dqkv, int S, int B, int heads, int nshard, int causal,
                       float sm_scale, float drop_p, unsigned long long seed, unsigned long long offset,
                       const unsigned long long* step_ptr, void* stream) {
  if (g_attn_tc && rtp_attn_tc_supported(S, heads, nshard)) {
    const int rc = rtp_attn_tc_bwd(qkv, dout, dqkv, S, B, heads, nshard, causal, sm_scale, drop_p, seed, offset, step_ptr,
                                   stream);
    if (rc) k_err = rtp_attn_tc_last_error();
    return rc;
  }
  if (heads % nshard) { k_err = "attn_small: heads must be divisible by shards"; return -1; }
  const size_t smem = attn_smem(S, true);
  if (smem > 227 * 1024) { k_err = "attn_small backward: sequence too long for shared memory (S <= 96)"; return -1; }
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(attn_small_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return kfail("attn bwd attr", e);
  }
  const float ds = drop_p > 0.f ? 1.f / (1.f - drop_p) : 1.f;
  attn_small_bwd_kernel<<<B * heads, 128, smem, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dqkv, S, B, heads, nshard, causal,
      sm_scale, host_thresh(drop_p), ds, seed, offset, step_ptr);
  LAUNCH_CHECK("attn_small_bwd");
  return 0;
}
int rtp_colsum(const void* x, long long ld, int M, int N, float* out, void* stream) {
  if (N % 2 || ld % 2) { k_err = "colsum: N and ld must be even"; return -1; }
  if (N % 8 == 0 && ld % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    // clusters of up to 8 blocks split the rows (at least 128 rows per block); very tall matrices get several
    // clusters per column group, whose sums meet in the zeroed output by atomics
    int cy = 8;
    while (cy > 1 && M < cy * 128) cy >>= 1;
    int groups = 1;
    while (groups < 64 && M / (cy * groups) > 1024) groups <<= 1;
    const int rows = (M + cy * groups - 1) / (cy * groups);
    if (groups > 1) {
      cudaError_t e = cudaMemsetAsync(out, 0, (size_t)N * sizeof(float), (cudaStream_t)stream);
      if (e != cudaSuccess) return kfail("colsum memset", e);
    }
    rtp::launch_kc(colsum_vec_kernel, dim3((N + 63) / 64, cy * groups), dim3(256), 0, (cudaStream_t)stream, dim3(1, cy, 1),
                   (const __nv_bfloat16*)x, ld, M, N, out, rows, groups > 1 ? 1 : 0);
    LAUNCH_CHECK("colsum");
    return 0;
  }
  cudaError_t e = cudaMemsetAsync(out, 0, (size_t)N * sizeof(float), (cudaStream_t)stream);
  if (e != cudaSuccess) return kfail("colsum memset", e);
  const int rows_per_block = 64;
  dim3 grid((N / 2 + 127) / 128, (M + rows_per_block - 1) / rows_per_block);
  colsum_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ld, M, N, out, rows_per_block);
  LAUNCH_CHECK("colsum");
  return 0;
}
int rtp_adam(const RtpAdamTensor* tensors_dev, const int* block_start_dev, int ntensors, int total_blocks,
             const long long* step_dev, float lr, float beta1, float beta2, float eps, float weight_decay, int adamw,
             float clip_value, float grad_scale, const int* block_tensor_dev, void* stream) {
  if (ntensors <= 0 || total_blocks <= 0) return 0;
  adam_kernel<<<total_blocks, 256, 0, (cudaStream_t)stream>>>(tensors_dev, block_start_dev, ntensors, step_dev, lr,
                                                              beta1, beta2, eps, weight_decay, adamw, clip_value,
                                                              grad_scale, block_tensor_dev);
  LAUNCH_CHECK("adam");
  return 0;
}
int rtp_causal_softmax(void* s, long long rows, int S, float scale, void* stream) {
  if (S % 8) { k_err = "causal_softmax: S must be a multiple of 8"; return -1; }
  const int grid = rows < 148 * 16 ? (int)rows : 148 * 16;
  causal_softmax_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)s, rows, S, scale);
  LAUNCH_CHECK("causal_softmax");
  return 0;
}
int rtp_causal_softmax_bwd(const void* p, void* dp, long long rows, int S, float scale, void* stream) {
  if (S % 8) { k_err = "causal_softmax_bwd: S must be a multiple of 8"; return -1; }
  const int grid = rows < 148 * 16 ? (int)rows : 148 * 16;
  causal_softmax_bwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)p, (__nv_bfloat16*)dp, rows, S,
                                                                   scale);
  LAUNCH_CHECK("causal_softmax_bwd");
  return 0;
}
int rtp_gelu_fwd(const void* x, void* y, long long n, void* stream) {
  if (n % 8) { k_err = "gelu: n must be a multiple of 8"; return -1; }
  gelu_fwd_kernel<<<(unsigned)((n / 8 + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, n);
  LAUNCH_CHECK("gelu_fwd");
  return 0;
}
int rtp_gelu_bwd(const void* x, const void* dy, void* dx, long long n, void* stream) {
  if (n % 8) { k_err = "gelu: n must be a multiple of 8"; return -1; }
  gelu_bwd_kernel<<<(unsigned)((n / 8 + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy,
                                                                                 (__nv_bfloat16*)dx, n);
  LAUNCH_CHECK("gelu_bwd");
  return 0;
}
int rtp_swiglu_fwd(const void* g, const void* u, long long ld, void* y, long long rows, int cols, void* stream) {
  if (cols % 8 || ld % 8) { k_err = "swiglu: cols and ld must be multiples of 8"; return -1; }
  const long long items = rows * (cols / 8);
  swiglu_fwd_kernel<<<(unsigned)((items + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)g, (const __nv_bfloat16*)u, ld,
                                                                                   (__nv_bfloat16*)y, rows, cols);
  LAUNCH_CHECK("swiglu_fwd");
  return 0;
}
int rtp_swiglu_bwd(const void* g, const void* u, long long ld, const void* dy, void* dg, void* du, long long ldo,
                   long long rows, int cols, void* stream) {
  if (cols % 8 || ld % 8 || ldo % 8) { k_err = "swiglu: cols and ld must be multiples of 8"; return -1; }
  const long long items = rows * (cols / 8);
  swiglu_bwd_kernel<<<(unsigned)((items + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)g, (const __nv_bfloat16*)u, ld, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dg, (__nv_bfloat16*)du, ldo, rows,
      cols);
  LAUNCH_CHECK("swiglu_bwd");
  return 0;
}
int rtp_moe_scatter(const void* src, const int* slot, const float* scale, void* dst, int S, int M, long long dst_rows,
                    void* stream) {
  if (M % 8) { k_err = "moe: M must be a multiple of 8"; return -1; }
  cudaError_t e = cudaMemsetAsync(dst, 0, (size_t)dst_rows * M * 2, (cudaStream_t)stream);
  if (e != cudaSuccess) return kfail("moe memset", e);
  const long long threads = 2ll * S * 32;
  moe_scatter_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)src, slot, scale, (__nv_bfloat16*)dst, S, M);
  LAUNCH_CHECK("moe_scatter");
  return 0;
}
int rtp_moe_gather(const void* src, const int* slot, const float* scale, void* dst, int S, int M, void* stream) {
  if (M % 8) { k_err = "moe: M must be a multiple of 8"; return -1; }
  const long long threads = (long long)S * 32;
  moe_gather_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)src, slot, scale, (__nv_bfloat16*)dst, S, M);
  LAUNCH_CHECK("moe_gather");
  return 0;
}
int rtp_moe_rowdot(const void* a, const void* b, const int* slot, float* out, int S, int M, void* stream) {
  if (M % 8) { k_err = "moe: M must be a multiple of 8"; return -1; }
  const long long threads = 2ll * S * 32;
  moe_rowdot_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, slot, out, S, M);
  LAUNCH_CHECK("moe_rowdot");
  return 0;
}
int rtp_add(const void* a, const void* b, void* out, long long n, void* stream) {
  const long long blocks = (n + 2047) / 2048;
  add_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                                                 (__nv_bfloat16*)out, n);
  LAUNCH_CHECK("add");
  return 0;
}
int rtp_cast_f32_bf16(const float* in, void* out, long long n, float scale, void* stream) {
  cast_f32_bf16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(in, (__nv_bfloat16*)out, n, scale);
  LAUNCH_CHECK("cast");
  return 0;
}
int rtp_sum_f32(const float* in, float* out, int n, float scale, void* stream) {
  sum_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(in, out, n, scale);
  LAUNCH_CHECK("sum");
  return 0;
}

}  // extern "C"
