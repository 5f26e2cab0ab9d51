// Short-sequence attention (S = 32 or 64, head_dim 64) on tcgen05 tensor cores.
//
// One CTA of 128 threads handles 128 / S (batch, head) pairs at once: their query rows are stacked into one
// 128-row operand, so that every product is an M = 128 UMMA.  Each head gets its own chain of UMMAs against its own
// K / V rows and its own TMEM columns; thread t owns stacked row t (TMEM lane t), so the softmax of a row and the
// dS algebra of the backward pass run entirely in that thread's registers, without shuffles.
//
//   forward :  S_q = Q K_q^T  ->  P = dropout(softmax(scale * S))  ->  O_q = P K-compact x V_q
//   backward:  S_q, dP_q = dO V_q^T  ->  dS  ->  dQ_q = dS x K_q ;  dK = dS^T x Q ;  dV = P_drop^T x dO
//
// dS^T and P_drop^T are written to shared memory as block-diagonal [128 x 128] MN-major A operands (row t of the
// stack writes k-row t, 16-byte stores), so dK and dV of all stacked heads come out of one chain of eight UMMAs each.
// Operands are fetched with plain 16-byte loads into 128-byte-swizzled tiles (the strided token order s*B + b of the
// packed projection needs no tensor map); "fence.proxy.async" publishes them to the tensor core.
//
// Same data layout and dropout stream as the scalar kernels in kernels.cu (attn_small_*), which remain the path for
// every other sequence length.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "common.cuh"
#include "kernels.h"
#include "launch.h"

namespace {
using namespace rtp;

constexpr int kHd = 64;
constexpr int kRows = 128;                 // stacked rows per CTA
constexpr int kTile = kRows * 128;         // one [128 x 64] bf16 operand tile, 128-byte rows: 16 KB

__device__ unsigned int g_attn_tc_error;        // set when a bounded wait for the CTA's own UMMAs ran out
__device__ unsigned long long* g_attn_trace;   // tuning aid: timeline of CTA 0 (16 words), null = off
#define ATT_STAMP(i) do { if (g_attn_trace && blockIdx.x == 0 && threadIdx.x == 0) g_attn_trace[i] = globaltimer_ns(); } while (0)

struct Ctl {
  uint64_t bar[2];
  uint32_t tmem_base;
  int valid[4];
  int b[4];
  int h[4];
  int cq[4], ck[4], cv[4];
};

__device__ __forceinline__ int qkv_col(int head, int which, int D, int nshard, int heads) {
  const int hps = heads / nshard;  // heads per shard
  const int j = head / hps, hl = head % hps;
  return j * (3 * (D / nshard)) + which * (D / nshard) + hl * kHd;
}
// byte offset of 16-byte chunk `chunk` of row `row` in a 128-byte-swizzled tile of 128-byte rows
__device__ __forceinline__ uint32_t sw128(int row, int chunk) {
  return (uint32_t)row * 128u + (uint32_t)((chunk ^ (row & 7)) << 4);
}
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  while (!mbar_try_wait(bar, parity)) {
    if (globaltimer_ns() - t0 > 1000000000ull) {
      atomicExch(&g_attn_tc_error, 1u);
      return false;
    }
  }
  return true;
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }

// Stacks rows [q * S_T + s] = token (s, b_q), columns col[q] .. col[q] + 64 of `src` (row pitch ld) into swizzled tiles.
// A thread's eight 16-byte loads per tile are all issued before the first shared-memory store, so that they overlap
// (a store in between would order them: the compiler cannot prove that the tile and the control block do not alias).
struct HeadRef {
  int valid, b, col;
};
template <int S_T>
__device__ __forceinline__ void fetch_stack(uint4 (&v)[8], const __nv_bfloat16* __restrict__ src, long long ld, int B,
                                            const HeadRef (&hr)[kRows / S_T], int tid) {
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int i = it * 128 + tid;
    const int row = i >> 3, c = i & 7;
    const int q = row / S_T, s = row % S_T;
    v[it] = make_uint4(0u, 0u, 0u, 0u);
    if (hr[q].valid) v[it] = __ldg(reinterpret_cast<const uint4*>(src + (size_t)(s * B + hr[q].b) * ld + hr[q].col + c * 8));
  }
}
__device__ __forceinline__ void store_stack(uint8_t* dst, const uint4 (&v)[8], int tid) {
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int i = it * 128 + tid;
    *reinterpret_cast<uint4*>(dst + sw128(i >> 3, i & 7)) = v[it];
  }
}

template <int S_T>
__device__ __forceinline__ void setup(Ctl* ctl, int tid, int warp, int B, int heads, int nshard, int n_bh,
                                      uint32_t tmem_cols) {
  constexpr int HPC = kRows / S_T;
  const int D = heads * kHd;
  pdl_launch_dependents();
  if (tid < HPC) {
    const int bh = blockIdx.x * HPC + tid;
    const int ok = bh < n_bh;
    const int b = ok ? bh / heads : 0, h = ok ? bh % heads : 0;
    ctl->valid[tid] = ok;
    ctl->b[tid] = b;
    ctl->h[tid] = h;
    ctl->cq[tid] = qkv_col(h, 0, D, nshard, heads);
    ctl->ck[tid] = qkv_col(h, 1, D, nshard, heads);
    ctl->cv[tid] = qkv_col(h, 2, D, nshard, heads);
  }
  if (tid == 0) {
    mbar_init(&ctl->bar[0], 1);
    mbar_init(&ctl->bar[1], 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&ctl->tmem_base, tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();   // set-up touched shared memory and TMEM only; the loads below need the previous kernel's output
}

// Row t of the score matrix out of TMEM, scaled; masked entries become -inf.
template <int S_T>
__device__ __forceinline__ void load_row(uint32_t taddr, float (&x)[S_T]) {
#pragma unroll
  for (int j = 0; j < S_T / 32; ++j) {
    uint32_t r[32];
    tmem_ld_32x32(taddr + j * 32, r);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; ++i) x[j * 32 + i] = __uint_as_float(r[i]);
  }
}

template <int S_T>
__global__ void __launch_bounds__(128) attn_tc_fwd_kernel(const __nv_bfloat16* __restrict__ qkv,
                                                          __nv_bfloat16* __restrict__ out, int B, int heads, int nshard,
                                                          int causal, float sm_scale, uint32_t thresh, float drop_scale,
                                                          uint64_t seed, uint64_t offset,
                                                          const unsigned long long* __restrict__ step_ptr, int n_bh) {
  constexpr int HPC = kRows / S_T;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = sm;
  uint8_t* sK = sm + kTile;
  uint8_t* sV = sm + 2 * kTile;
  uint8_t* sP = sm + 3 * kTile;
  Ctl* ctl = reinterpret_cast<Ctl*>(sm + 4 * kTile);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int D = heads * kHd;
  ATT_STAMP(0);
  setup<S_T>(ctl, tid, warp, B, heads, nshard, n_bh, 256);
  ATT_STAMP(1);
  if (step_ptr) offset += __ldg(step_ptr) * 65536ull;
  const uint32_t tmem = ctl->tmem_base;

  {
    HeadRef hq[HPC], hk[HPC], hv[HPC];
#pragma unroll
    for (int qq = 0; qq < HPC; ++qq) {
      hq[qq] = {ctl->valid[qq], ctl->b[qq], ctl->cq[qq]};
      hk[qq] = {ctl->valid[qq], ctl->b[qq], ctl->ck[qq]};
      hv[qq] = {ctl->valid[qq], ctl->b[qq], ctl->cv[qq]};
    }
    uint4 va[8], vb[8], vc[8];
    fetch_stack<S_T>(va, qkv, 3 * D, B, hq, tid);
    fetch_stack<S_T>(vb, qkv, 3 * D, B, hk, tid);
    fetch_stack<S_T>(vc, qkv, 3 * D, B, hv, tid);
    store_stack(sQ, va, tid);
    store_stack(sK, vb, tid);
    store_stack(sV, vc, tid);
  }
  fence_proxy_async_smem();
  __syncthreads();
  ATT_STAMP(2);

  if (warp == 0 && elect_one()) {
    const uint32_t idesc = make_idesc_bf16(128, S_T, 0, 0);
    const uint32_t aq = smem_u32(sQ), bk = smem_u32(sK);
#pragma unroll
    for (int q = 0; q < HPC; ++q)
#pragma unroll
      for (int kk = 0; kk < kHd / 16; ++kk)
        umma_bf16(tmem + q * S_T, make_smem_desc(aq + kk * 32, 16, 1024),
                  make_smem_desc(bk + q * S_T * 128 + kk * 32, 16, 1024), idesc, kk > 0 ? 1u : 0u);
    umma_commit(&ctl->bar[0]);
  }
  wait_bar(&ctl->bar[0], 0);
  tc_fence_after();
  ATT_STAMP(3);

  const int q = tid / S_T, s = tid % S_T;
  const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
  {
    float x[S_T];
    load_row<S_T>(lane_addr + q * S_T, x);
    float mx = -INFINITY;
#pragma unroll
    for (int c = 0; c < S_T; ++c) {
      x[c] = (causal && c > s) ? -INFINITY : x[c] * sm_scale;
      mx = fmaxf(mx, x[c]);
    }
    float sum = 0.f;
#pragma unroll
    for (int c = 0; c < S_T; ++c) {
      x[c] = __expf(x[c] - mx);
      sum += x[c];
    }
    const float inv = 1.f / sum;
    const int bh = blockIdx.x * HPC + q;
    const uint64_t e0 = ((uint64_t)bh * S_T + s) * S_T;
#pragma unroll
    for (int c4 = 0; c4 < S_T / 4; ++c4) {
      float m0 = inv, m1 = inv, m2 = inv, m3 = inv;
      if (thresh) {
        const uint4 rr = philox4x32(seed, offset, (e0 >> 2) + c4);
        m0 = rr.x >= thresh ? inv * drop_scale : 0.f;
        m1 = rr.y >= thresh ? inv * drop_scale : 0.f;
        m2 = rr.z >= thresh ? inv * drop_scale : 0.f;
        m3 = rr.w >= thresh ? inv * drop_scale : 0.f;
      }
      x[4 * c4] *= m0; x[4 * c4 + 1] *= m1; x[4 * c4 + 2] *= m2; x[4 * c4 + 3] *= m3;
    }
#pragma unroll
    for (int c8 = 0; c8 < S_T / 8; ++c8)
      *reinterpret_cast<uint4*>(sP + sw128(tid, c8)) =
          make_uint4(pack2(x[8 * c8], x[8 * c8 + 1]), pack2(x[8 * c8 + 2], x[8 * c8 + 3]),
                     pack2(x[8 * c8 + 4], x[8 * c8 + 5]), pack2(x[8 * c8 + 6], x[8 * c8 + 7]));
  }
  ATT_STAMP(4);
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();   // every row of S has been read: its TMEM columns are reused for O
  ATT_STAMP(5);

  if (warp == 0 && elect_one()) {
    tc_fence_after();
    const uint32_t idesc = make_idesc_bf16(128, kHd, 0, 1);
    const uint32_t ap = smem_u32(sP), bv = smem_u32(sV);
#pragma unroll
    for (int qq = 0; qq < HPC; ++qq)
#pragma unroll
      for (int kk = 0; kk < S_T / 16; ++kk)
        umma_bf16(tmem + qq * kHd, make_smem_desc(ap + kk * 32, 16, 1024),
                  make_smem_desc(bv + qq * S_T * 128 + kk * 2048, 8192, 1024), idesc, kk > 0 ? 1u : 0u);
    umma_commit(&ctl->bar[1]);
  }
  wait_bar(&ctl->bar[1], 0);
  tc_fence_after();
  ATT_STAMP(6);
  {
    float o[kHd];
    load_row<kHd>(lane_addr + q * kHd, o);
    if (ctl->valid[q]) {
      uint4* dst = reinterpret_cast<uint4*>(out + (size_t)(s * B + ctl->b[q]) * D + ctl->h[q] * kHd);
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8)
        dst[c8] = make_uint4(pack2(o[8 * c8], o[8 * c8 + 1]), pack2(o[8 * c8 + 2], o[8 * c8 + 3]),
                             pack2(o[8 * c8 + 4], o[8 * c8 + 5]), pack2(o[8 * c8 + 6], o[8 * c8 + 7]));
    }
  }
  ATT_STAMP(7);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
  ATT_STAMP(8);
}

template <int S_T>
__global__ void __launch_bounds__(128) attn_tc_bwd_kernel(const __nv_bfloat16* __restrict__ qkv,
                                                          const __nv_bfloat16* __restrict__ dout,
                                                          __nv_bfloat16* __restrict__ dqkv, int B, int heads, int nshard,
                                                          int causal, float sm_scale, uint32_t thresh, float drop_scale,
                                                          uint64_t seed, uint64_t offset,
                                                          const unsigned long long* __restrict__ step_ptr, int n_bh) {
  constexpr int HPC = kRows / S_T;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = sm;
  uint8_t* sK = sm + kTile;
  uint8_t* sV = sm + 2 * kTile;
  uint8_t* sG = sm + 3 * kTile;            // dO
  uint8_t* sS = sm + 4 * kTile;            // dS, compact K-major [128 x S_T]
  uint8_t* sTS = sm + 5 * kTile;           // dS^T, block-diagonal MN-major A [k = stacked row][m = stacked key]: 32 KB
  uint8_t* sTP = sm + 7 * kTile;           // P_drop^T, same form: 32 KB
  Ctl* ctl = reinterpret_cast<Ctl*>(sm + 9 * kTile);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int D = heads * kHd;
  ATT_STAMP(0);
  setup<S_T>(ctl, tid, warp, B, heads, nshard, n_bh, 512);
  ATT_STAMP(1);
  if (step_ptr) offset += __ldg(step_ptr) * 65536ull;
  const uint32_t tmem = ctl->tmem_base;

  {
    HeadRef hq[HPC], hk[HPC], hv[HPC], hg[HPC];
#pragma unroll
    for (int qq = 0; qq < HPC; ++qq) {
      hq[qq] = {ctl->valid[qq], ctl->b[qq], ctl->cq[qq]};
      hk[qq] = {ctl->valid[qq], ctl->b[qq], ctl->ck[qq]};
      hv[qq] = {ctl->valid[qq], ctl->b[qq], ctl->cv[qq]};
      hg[qq] = {ctl->valid[qq], ctl->b[qq], ctl->h[qq] * kHd};   // dO has [T, D] layout: column of head h is h * 64
    }
    uint4 va[8], vb[8], vc[8], vd[8];
    fetch_stack<S_T>(va, qkv, 3 * D, B, hq, tid);
    fetch_stack<S_T>(vb, qkv, 3 * D, B, hk, tid);
    fetch_stack<S_T>(vc, qkv, 3 * D, B, hv, tid);
    fetch_stack<S_T>(vd, dout, D, B, hg, tid);
    // the off-diagonal blocks of the transposed operands stay zero (filled while the loads are in flight)
#pragma unroll 4
    for (int i = tid; i < 4 * kTile / 16; i += 128) reinterpret_cast<uint4*>(sTS)[i] = make_uint4(0u, 0u, 0u, 0u);
    store_stack(sQ, va, tid);
    store_stack(sK, vb, tid);
    store_stack(sV, vc, tid);
    store_stack(sG, vd, tid);
  }
  fence_proxy_async_smem();
  __syncthreads();
  ATT_STAMP(2);

  if (warp == 0 && elect_one()) {
    const uint32_t idesc = make_idesc_bf16(128, S_T, 0, 0);
    const uint32_t aq = smem_u32(sQ), bk = smem_u32(sK), ag = smem_u32(sG), bv = smem_u32(sV);
#pragma unroll
    for (int qq = 0; qq < HPC; ++qq)
#pragma unroll
      for (int kk = 0; kk < kHd / 16; ++kk)
        umma_bf16(tmem + qq * S_T, make_smem_desc(aq + kk * 32, 16, 1024),
                  make_smem_desc(bk + qq * S_T * 128 + kk * 32, 16, 1024), idesc, kk > 0 ? 1u : 0u);
#pragma unroll
    for (int qq = 0; qq < HPC; ++qq)
#pragma unroll
      for (int kk = 0; kk < kHd / 16; ++kk)
        umma_bf16(tmem + 128 + qq * S_T, make_smem_desc(ag + kk * 32, 16, 1024),
                  make_smem_desc(bv + qq * S_T * 128 + kk * 32, 16, 1024), idesc, kk > 0 ? 1u : 0u);
    umma_commit(&ctl->bar[0]);
  }
  wait_bar(&ctl->bar[0], 0);
  tc_fence_after();
  ATT_STAMP(3);

  const int q = tid / S_T, s = tid % S_T;
  const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
  {
    float x[S_T], dp[S_T];
    load_row<S_T>(lane_addr + q * S_T, x);
    load_row<S_T>(lane_addr + 128 + q * S_T, dp);
    float mx = -INFINITY;
#pragma unroll
    for (int c = 0; c < S_T; ++c) {
      x[c] = (causal && c > s) ? -INFINITY : x[c] * sm_scale;
      mx = fmaxf(mx, x[c]);
    }
    float sum = 0.f;
#pragma unroll
    for (int c = 0; c < S_T; ++c) {
      x[c] = __expf(x[c] - mx);
      sum += x[c];
    }
    const float inv = 1.f / sum;
    const int bh = blockIdx.x * HPC + q;
    const uint64_t e0 = ((uint64_t)bh * S_T + s) * S_T;
    // x <- P, dp <- m * dP (gradient wrt the un-dropped probability); the mask m is kept as a bit set
    uint64_t keep = ~0ull;
    float dot = 0.f;
#pragma unroll
    for (int c4 = 0; c4 < S_T / 4; ++c4) {
      uint32_t k4 = 0xfu;
      if (thresh) {
        const uint4 rr = philox4x32(seed, offset, (e0 >> 2) + c4);
        k4 = (rr.x >= thresh ? 1u : 0u) | (rr.y >= thresh ? 2u : 0u) | (rr.z >= thresh ? 4u : 0u) |
             (rr.w >= thresh ? 8u : 0u);
        keep = (keep & ~(0xfull << (4 * c4))) | ((uint64_t)k4 << (4 * c4));
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = 4 * c4 + i;
        x[c] *= inv;
        dp[c] = ((k4 >> i) & 1u) ? dp[c] * drop_scale : 0.f;
        dot += dp[c] * x[c];
      }
    }
    // dS (into dp) and the dropped probabilities (into x)
#pragma unroll
    for (int c = 0; c < S_T; ++c) {
      dp[c] = x[c] * (dp[c] - dot);
      x[c] = ((keep >> c) & 1ull) ? x[c] * drop_scale : 0.f;
    }
    // compact dS row, and row t of both transposed operands (k-row t; columns of this head's keys)
    const int m0 = q * S_T;
    uint8_t* ts = sTS + (tid >> 6) * 16384 + (m0 >> 6) * 8192;
    uint8_t* tp = sTP + (tid >> 6) * 16384 + (m0 >> 6) * 8192;
    const int kr = tid & 63, cb = (m0 & 63) >> 3;
#pragma unroll
    for (int c8 = 0; c8 < S_T / 8; ++c8) {
      const uint4 vs = make_uint4(pack2(dp[8 * c8], dp[8 * c8 + 1]), pack2(dp[8 * c8 + 2], dp[8 * c8 + 3]),
                                  pack2(dp[8 * c8 + 4], dp[8 * c8 + 5]), pack2(dp[8 * c8 + 6], dp[8 * c8 + 7]));
      const uint4 vp = make_uint4(pack2(x[8 * c8], x[8 * c8 + 1]), pack2(x[8 * c8 + 2], x[8 * c8 + 3]),
                                  pack2(x[8 * c8 + 4], x[8 * c8 + 5]), pack2(x[8 * c8 + 6], x[8 * c8 + 7]));
      *reinterpret_cast<uint4*>(sS + sw128(tid, c8)) = vs;
      *reinterpret_cast<uint4*>(ts + sw128(kr, cb + c8)) = vs;
      *reinterpret_cast<uint4*>(tp + sw128(kr, cb + c8)) = vp;
    }
  }
  ATT_STAMP(4);
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();   // S and dP have been read everywhere: their TMEM columns are reused for dQ
  ATT_STAMP(5);

  if (warp == 0 && elect_one()) {
    tc_fence_after();
    const uint32_t as = smem_u32(sS), bk = smem_u32(sK), bq = smem_u32(sQ), bg = smem_u32(sG);
    const uint32_t ats = smem_u32(sTS), atp = smem_u32(sTP);
    const uint32_t id_q = make_idesc_bf16(128, kHd, 0, 1), id_t = make_idesc_bf16(128, kHd, 1, 1);
#pragma unroll
    for (int qq = 0; qq < HPC; ++qq)
#pragma unroll
      for (int kk = 0; kk < S_T / 16; ++kk)
        umma_bf16(tmem + qq * kHd, make_smem_desc(as + kk * 32, 16, 1024),
                  make_smem_desc(bk + qq * S_T * 128 + kk * 2048, 8192, 1024), id_q, kk > 0 ? 1u : 0u);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      umma_bf16(tmem + 256, make_smem_desc(ats + (j >> 2) * 16384 + (j & 3) * 2048, 8192, 1024),
                make_smem_desc(bq + j * 2048, 8192, 1024), id_t, j > 0 ? 1u : 0u);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      umma_bf16(tmem + 320, make_smem_desc(atp + (j >> 2) * 16384 + (j & 3) * 2048, 8192, 1024),
                make_smem_desc(bg + j * 2048, 8192, 1024), id_t, j > 0 ? 1u : 0u);
    umma_commit(&ctl->bar[1]);
  }
  wait_bar(&ctl->bar[1], 0);
  tc_fence_after();
  ATT_STAMP(6);
  if (ctl->valid[q]) {
    __nv_bfloat16* rowp = dqkv + (size_t)(s * B + ctl->b[q]) * (3 * D);
    float o[kHd];
    load_row<kHd>(lane_addr + q * kHd, o);
    uint4* dst = reinterpret_cast<uint4*>(rowp + ctl->cq[q]);
#pragma unroll
    for (int c8 = 0; c8 < 8; ++c8)
      dst[c8] = make_uint4(pack2(o[8 * c8] * sm_scale, o[8 * c8 + 1] * sm_scale),
                           pack2(o[8 * c8 + 2] * sm_scale, o[8 * c8 + 3] * sm_scale),
                           pack2(o[8 * c8 + 4] * sm_scale, o[8 * c8 + 5] * sm_scale),
                           pack2(o[8 * c8 + 6] * sm_scale, o[8 * c8 + 7] * sm_scale));
    load_row<kHd>(lane_addr + 256, o);
    dst = reinterpret_cast<uint4*>(rowp + ctl->ck[q]);
#pragma unroll
    for (int c8 = 0; c8 < 8; ++c8)
      dst[c8] = make_uint4(pack2(o[8 * c8] * sm_scale, o[8 * c8 + 1] * sm_scale),
                           pack2(o[8 * c8 + 2] * sm_scale, o[8 * c8 + 3] * sm_scale),
                           pack2(o[8 * c8 + 4] * sm_scale, o[8 * c8 + 5] * sm_scale),
                           pack2(o[8 * c8 + 6] * sm_scale, o[8 * c8 + 7] * sm_scale));
    load_row<kHd>(lane_addr + 320, o);
    dst = reinterpret_cast<uint4*>(rowp + ctl->cv[q]);
#pragma unroll
    for (int c8 = 0; c8 < 8; ++c8)
      dst[c8] = make_uint4(pack2(o[8 * c8], o[8 * c8 + 1]), pack2(o[8 * c8 + 2], o[8 * c8 + 3]),
                           pack2(o[8 * c8 + 4], o[8 * c8 + 5]), pack2(o[8 * c8 + 6], o[8 * c8 + 7]));
  } else {
    // tcgen05.ld is warp-collective: rows without a head still take part
    float o[kHd];
    load_row<kHd>(lane_addr + q * kHd, o);
    load_row<kHd>(lane_addr + 256, o);
    load_row<kHd>(lane_addr + 320, o);
  }
  ATT_STAMP(7);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
  ATT_STAMP(8);
}

std::string g_err;
constexpr int kFwdSmem = 4 * kTile + 1024 + 256;
constexpr int kBwdSmem = 9 * kTile + 1024 + 256;
uint32_t thresh_of(float p) {
  if (p <= 0.f) return 0u;
  double t = (double)p * 4294967296.0;
  if (t > 4294967295.0) t = 4294967295.0;
  return (uint32_t)t;
}
template <auto Kern>
int set_smem(int bytes) {
  cudaError_t e = rtp::ensure_smem<Kern>(bytes);
  if (e != cudaSuccess) {
    g_err = std::string("attn_tc: cudaFuncSetAttribute: ") + cudaGetErrorString(e);
    return -1;
  }
  return 0;
}
}  // namespace

extern "C" {

const char* rtp_attn_tc_last_error(void) { return g_err.c_str(); }

// tuning aid: device buffer of 16 words that receives globaltimer stamps of CTA 0 (null switches it off)
int rtp_attn_tc_set_trace(unsigned long long* device_buffer) {
  return cudaMemcpyToSymbol(g_attn_trace, &device_buffer, sizeof(device_buffer)) == cudaSuccess ? 0 : -1;
}

int rtp_attn_tc_supported(int S, int heads, int nshard) { return (S == 32 || S == 64) && heads % nshard == 0; }

// 1 if a bounded wait inside one of the kernels ran out since the last call (and clears the flag); synchronises.
int rtp_attn_tc_error(void) {
  unsigned int v = 0, z = 0;
  if (cudaMemcpyFromSymbol(&v, g_attn_tc_error, sizeof(v)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_attn_tc_error, &z, sizeof(z));
  return (int)v;
}

int rtp_attn_tc_fwd(const void* qkv, void* out, int S, int B, int heads, int nshard, int causal, float sm_scale,
                    float drop_p, unsigned long long seed, unsigned long long offset,
                    const unsigned long long* step_ptr, void* stream) {
  if (!rtp_attn_tc_supported(S, heads, nshard)) { g_err = "attn_tc: S must be 32 or 64"; return -1; }
  const int n_bh = B * heads;
  const float ds = drop_p > 0.f ? 1.f / (1.f - drop_p) : 1.f;
  const int hpc = 128 / S;
  const int grid = (n_bh + hpc - 1) / hpc;
  if (S == 32) {
    if (set_smem<attn_tc_fwd_kernel<32>>(kFwdSmem)) return -1;
    rtp::launch_k(attn_tc_fwd_kernel<32>, dim3(grid), dim3(128), kFwdSmem, (cudaStream_t)stream, 
        (const __nv_bfloat16*)qkv, (__nv_bfloat16*)out, B, heads, nshard, causal, sm_scale, thresh_of(drop_p), ds, seed,
        offset, step_ptr, n_bh);
  } else {
    if (set_smem<attn_tc_fwd_kernel<64>>(kFwdSmem)) return -1;
    rtp::launch_k(attn_tc_fwd_kernel<64>, dim3(grid), dim3(128), kFwdSmem, (cudaStream_t)stream, 
        (const __nv_bfloat16*)qkv, (__nv_bfloat16*)out, B, heads, nshard, causal, sm_scale, thresh_of(drop_p), ds, seed,
        offset, step_ptr, n_bh);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { g_err = std::string("attn_tc_fwd: ") + cudaGetErrorString(e); return -1; }
  return 0;
}

int rtp_attn_tc_bwd(const void* qkv, const void* dout, void* dqkv, int S, int B, int heads, int nshard, int causal,
                    float sm_scale, float drop_p, unsigned long long seed, unsigned long long offset,
                    const unsigned long long* step_ptr, void* stream) {
  if (!rtp_attn_tc_supported(S, heads, nshard)) { g_err = "attn_tc: S must be 32 or 64"; return -1; }
  const int n_bh = B * heads;
  const float ds = drop_p > 0.f ? 1.f / (1.f - drop_p) : 1.f;
  const int hpc = 128 / S;
  const int grid = (n_bh + hpc - 1) / hpc;
  if (S == 32) {
    if (set_smem<attn_tc_bwd_kernel<32>>(kBwdSmem)) return -1;
    rtp::launch_k(attn_tc_bwd_kernel<32>, dim3(grid), dim3(128), kBwdSmem, (cudaStream_t)stream, 
        (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dqkv, B, heads, nshard, causal, sm_scale,
        thresh_of(drop_p), ds, seed, offset, step_ptr, n_bh);
  } else {
    if (set_smem<attn_tc_bwd_kernel<64>>(kBwdSmem)) return -1;
    rtp::launch_k(attn_tc_bwd_kernel<64>, dim3(grid), dim3(128), kBwdSmem, (cudaStream_t)stream, 
        (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dqkv, B, heads, nshard, causal, sm_scale,
        thresh_of(drop_p), ds, seed, offset, step_ptr, n_bh);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { g_err = std::string("attn_tc_bwd: ") + cudaGetErrorString(e); return -1; }
  return 0;
}

}  // extern "C"
