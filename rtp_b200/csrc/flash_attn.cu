// Flash attention on tcgen05 tensor cores: forward, dQ and dK/dV kernels (see flash_attn.h for the interface).
//
// One CTA = 128 query rows (forward, dQ) or 128 keys (dK/dV) of one (batch, head).  Ten warps:
//   warps 0-7  "row" threads, two per row of the tile: thread (t, h) reads TMEM lane t and owns the key columns
//              [64 h, 64 h + 64) of the 128-key block (warps w and w + 4 may both access lanes 32 (w % 4) ..).  The online
//              softmax of a row (forward) and the dS algebra (backward) run in registers without shuffles; the two
//              threads of a row exchange one partial maximum per block through shared memory (forward only).
//   warp 8     TMA producer: Q / K / V / dO tiles, 128 rows x 64 columns per copy, 128-byte swizzle, local memory only.
//   warp 9     UMMA issuer (one elected thread).
//
// Forward, per block of 128 keys:  S = Q K^T (TMEM, double-buffered)  ->  row threads: scale, masks, running max,
// P = exp2(S - m) as bf16 into a shared tile  ->  O += P V with O resident in TMEM.  O is rescaled in TMEM only when a
// row's maximum has grown by more than 2^8 since the last rescale (the sum l carries the same offset, so the final
// O / l is exact); most blocks skip the rescale.  Output: O / l and the row's log-sum-exp (log2 units).
//
// Backward recomputes P from Q, K and the saved log-sum-exp; nothing of size S x S touches global memory.
//   dQ kernel   (CTA = query block): delta = rowsum(dO * O);  per key block: S, dP = dO V^T -> dS = P (dP - delta)
//               -> dQ += dS K.
//   dK/dV kernel (CTA = key block): per query block: S, dP -> P, dS tiles -> dV += P^T dO, dK += dS^T Q.  The P / dS
//               tiles are written row-per-thread once and read by the UMMA as MN-major A operands (= transposed).
// Each kernel is compiled in four variants (additive / key-padding masks yes or no, dropout yes or no): the mask and
// Philox code unrolled over a row's registers is several times larger than the plain softmax and, when merely branched
// over, slowed the row threads down through instruction fetch alone.
// Every mbarrier wait is bounded; on expiry the CTA records a status code, drains its copies and UMMAs, frees its TMEM
// and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include <string>

#include "common.cuh"
#include "flash_attn.h"
#include "launch.h"
#include "tmap.h"

namespace {
using namespace rtp;

constexpr int kBlk = 128;              // rows of Q per CTA = keys per block
constexpr int kSub = 16384;            // one [128 x 64] bf16 sub-tile with 128-byte rows
constexpr int kThreads = 320;
constexpr int kRowThreads = 256;
constexpr int kProducerWarp = 8, kMmaWarp = 9;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleGap = 8.f;     // rescale O when a row maximum grew by more than 2^8

struct DRef {                          // device copy of an RtpFlashRef
  void* ptr;
  long long sb, ss;
  int col_base, hpg, gstride, hstride;
};
__device__ __forceinline__ int head_col(const DRef& r, int h) {
  return r.col_base + (h / r.hpg) * r.gstride + (h % r.hpg) * r.hstride;
}
__device__ __forceinline__ __nv_bfloat16* row_ptr(const DRef& r, int b, int s, int h) {
  return reinterpret_cast<__nv_bfloat16*>(r.ptr) + (long long)b * r.sb + (long long)s * r.ss + head_col(r, h);
}

struct MaskArgs {
  const void* mask; long long mask_ld; int mask_fp32;
  const unsigned char* kpm; long long kpm_ld;
  int causal, Sq, Sk;
  float scale_log2, sm_scale;
  uint32_t thresh; float drop_scale;
  unsigned long long seed, offset;
  const unsigned long long* step_ptr;
};

struct alignas(64) FlashParams {
  CUtensorMap mq, mk, mv, mdo;         // 3-D maps {columns, dim1, dim2}; *_seq1 tells which of dim1 / dim2 is the sequence
  CUtensorMap mq64, mdo64, mk64, mv64; // the same tensors with boxes of 64 rows (backward kernels)
  int q_seq1, k_seq1, v_seq1, do_seq1;
  DRef q, k, v, o, dout, dq, dk, dv;
  float* lse;
  float* delta;
  int B, H;
  MaskArgs m;
  unsigned long long* status;
  unsigned long long timeout_ns;
  long long* trace;                    // tuning aid (rtp_flash_debug_set_trace): SM clock stamps of CTA 0, else null
};

struct Ctl {
  uint64_t bar[24];
  uint32_t tmem_base;
  uint32_t abort_flag;
};
// Exchange area of the two threads of a row (forward): per block one partial row maximum each way, double-buffered by
// block parity.  The two warps that share 32 rows meet at an mbarrier of their own (64 arrivals per exchange).
struct Xchg {
  float val[2][2][128];
};

__device__ __forceinline__ uint32_t sw128(int row, int chunk) {
  return (uint32_t)row * 128u + (uint32_t)((chunk ^ (row & 7)) << 4);
}
__device__ __forceinline__ void tmem_ld32f(uint32_t taddr, float* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]),
        "=f"(r[8]), "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15]),
        "=f"(r[16]), "=f"(r[17]), "=f"(r[18]), "=f"(r[19]), "=f"(r[20]), "=f"(r[21]), "=f"(r[22]), "=f"(r[23]),
        "=f"(r[24]), "=f"(r[25]), "=f"(r[26]), "=f"(r[27]), "=f"(r[28]), "=f"(r[29]), "=f"(r[30]), "=f"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32f(uint32_t taddr, const float* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "f"(r[0]), "f"(r[1]), "f"(r[2]), "f"(r[3]), "f"(r[4]), "f"(r[5]), "f"(r[6]), "f"(r[7]),
        "f"(r[8]), "f"(r[9]), "f"(r[10]), "f"(r[11]), "f"(r[12]), "f"(r[13]), "f"(r[14]), "f"(r[15]),
        "f"(r[16]), "f"(r[17]), "f"(r[18]), "f"(r[19]), "f"(r[20]), "f"(r[21]), "f"(r[22]), "f"(r[23]),
        "f"(r[24]), "f"(r[25]), "f"(r[26]), "f"(r[27]), "f"(r[28]), "f"(r[29]), "f"(r[30]), "f"(r[31])
      : "memory");
}

// Loads one [128 rows x 64 * SUB columns] tile of a (batch, head) into SUB swizzled sub-tiles.
template <int SUB>
__device__ __forceinline__ void load_tile(uint32_t dst, const CUtensorMap* map, int seq1, int col, int b, int s0,
                                          uint32_t bar) {
  const unsigned long long m = reinterpret_cast<unsigned long long>(map);
#pragma unroll
  for (int u = 0; u < SUB; ++u) {
    if (seq1) tma_load_3d_s(dst + u * kSub, m, col + u * 64, s0, b, bar);
    else tma_load_3d_s(dst + u * kSub, m, col + u * 64, b, s0, bar);
  }
}

// The backward kernels walk the other sequence in sub-blocks of 64 rows, three stages deep.
constexpr int kHalf = 64;                 // rows per sub-block
constexpr int kHalfTile = kHalf * 128;    // one [64 x 64] bf16 sub-tile with 128-byte rows
constexpr int kBwdStages = 3;
template <int SUB>
__device__ __forceinline__ void load_tile64(uint32_t dst, const CUtensorMap* map, int seq1, int col, int b, int s0,
                                            uint32_t bar) {
  const unsigned long long m = reinterpret_cast<unsigned long long>(map);
#pragma unroll
  for (int u = 0; u < SUB; ++u) {
    if (seq1) tma_load_3d_s(dst + u * kHalfTile, m, col + u * 64, s0, b, bar);
    else tma_load_3d_s(dst + u * kHalfTile, m, col + u * 64, b, s0, bar);
  }
}

// x[i] = log2-domain score of (row, col0 + i): scale, additive mask, key padding, causal and sequence bounds.
// Masked entries become -inf.  `plain` = nothing but the scale applies to this block.
template <int NC, bool MSK>
__device__ __forceinline__ void score_chunk(float* x, int row, int col0, int b, const MaskArgs& m, bool plain) {
#pragma unroll
  for (int i = 0; i < NC; ++i) x[i] *= m.scale_log2;
  if (plain) return;
  if constexpr (MSK) {
  if (m.mask && row < m.Sq) {
    if (m.mask_fp32) {
      const float* mp = reinterpret_cast<const float*>(m.mask) + (long long)row * m.mask_ld + col0;
      if (col0 + NC <= m.Sk && (reinterpret_cast<uintptr_t>(mp) & 15) == 0) {
#pragma unroll
        for (int q = 0; q < NC / 4; ++q) {
          const float4 v = __ldg(reinterpret_cast<const float4*>(mp) + q);
          x[4 * q] += v.x * kLog2e; x[4 * q + 1] += v.y * kLog2e; x[4 * q + 2] += v.z * kLog2e; x[4 * q + 3] += v.w * kLog2e;
        }
      } else {
#pragma unroll
        for (int i = 0; i < NC; ++i) if (col0 + i < m.Sk) x[i] += __ldg(mp + i) * kLog2e;
      }
    } else {
      const __nv_bfloat16* mp = reinterpret_cast<const __nv_bfloat16*>(m.mask) + (long long)row * m.mask_ld + col0;
      if (col0 + NC <= m.Sk && (reinterpret_cast<uintptr_t>(mp) & 15) == 0) {
#pragma unroll
        for (int q = 0; q < NC / 8; ++q) {
          const uint4 v = __ldg(reinterpret_cast<const uint4*>(mp) + q);
          x[8 * q] += bf16_lo(v.x) * kLog2e; x[8 * q + 1] += bf16_hi(v.x) * kLog2e;
          x[8 * q + 2] += bf16_lo(v.y) * kLog2e; x[8 * q + 3] += bf16_hi(v.y) * kLog2e;
          x[8 * q + 4] += bf16_lo(v.z) * kLog2e; x[8 * q + 5] += bf16_hi(v.z) * kLog2e;
          x[8 * q + 6] += bf16_lo(v.w) * kLog2e; x[8 * q + 7] += bf16_hi(v.w) * kLog2e;
        }
      } else {
#pragma unroll
        for (int i = 0; i < NC; ++i) if (col0 + i < m.Sk) x[i] += __bfloat162float(__ldg(mp + i)) * kLog2e;
      }
    }
  }
  if (m.kpm) {
    const unsigned char* kp = m.kpm + (long long)b * m.kpm_ld + col0;
#pragma unroll
    for (int i = 0; i < NC; ++i) if (col0 + i < m.Sk && __ldg(kp + i)) x[i] = -INFINITY;
  }
  }
  if (m.causal && col0 + NC - 1 > row) {
#pragma unroll
    for (int i = 0; i < NC; ++i) if (col0 + i > row) x[i] = -INFINITY;
  }
  if (col0 + NC > m.Sk) {
#pragma unroll
    for (int i = 0; i < NC; ++i) if (col0 + i >= m.Sk) x[i] = -INFINITY;
  }
}
// keep bits of the NC probabilities (row, col0 ..) of head-batch bh: bit i set = kept.  Needs Sk % 4 == 0.
template <int NC>
__device__ __forceinline__ uint32_t keep_bits(const MaskArgs& m, unsigned long long offset, long long bh, int row, int col0) {
  static_assert(NC <= 32, "keep mask is one word");
  const unsigned long long e4 = (((unsigned long long)bh * m.Sq + row) * (unsigned long long)m.Sk + col0) >> 2;
  uint32_t bits = 0;
#pragma unroll
  for (int g = 0; g < NC / 4; ++g) {
    const uint4 r = philox4x32(m.seed, offset, e4 + g);
    bits |= ((r.x >= m.thresh ? 1u : 0u) | (r.y >= m.thresh ? 2u : 0u) | (r.z >= m.thresh ? 4u : 0u) |
             (r.w >= m.thresh ? 8u : 0u)) << (4 * g);
  }
  return bits;
}
__device__ __forceinline__ uint4 pack8f(const float* v) {
  return make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
}

// Common set-up: barriers, TMEM, abort flag.  Returns the TMEM base.
__device__ __forceinline__ uint32_t setup_cta(Ctl* ctl, const int* counts, int nbar, int warp, int lane) {
  pdl_launch_dependents();
  if (warp == kProducerWarp) {
    if (lane < nbar) mbar_init(&ctl->bar[lane], counts[lane]);
    if (lane == 31) ctl->abort_flag = 0;
    mbar_fence_init();
    __syncwarp();
    tmem_alloc(&ctl->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  return ctl->tmem_base;
}
__device__ __forceinline__ void teardown_cta(uint32_t tmem, int warp) {
  tc_fence_before();
  __syncthreads();
  if (warp == kProducerWarp) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}
// Publishes `v` to the other thread of the row and returns the partner's value; `n` counts the exchanges of this row
// group from 0.  The arrive releases the value, the (bounded) wait acquires the partner's.
__device__ __forceinline__ float xchg_row(Xchg* x, uint64_t* xbar, int wg, int rt, uint32_t n, float v,
                                          volatile uint32_t* abort_flag, unsigned long long* status,
                                          unsigned long long timeout_ns, bool& ok) {
  x->val[n & 1][wg][rt] = v;
  mbar_arrive(xbar);
  if (!mbar_wait(xbar, n & 1u, abort_flag, status, timeout_ns)) { ok = false; return v; }
  return x->val[n & 1][wg ^ 1][rt];
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max64(const float* s) {
  float m0 = s[0], m1 = s[1], m2 = s[2], m3 = s[3];
#pragma unroll
  for (int i = 4; i < 64; i += 4) {
    m0 = fmaxf(m0, s[i]); m1 = fmaxf(m1, s[i + 1]); m2 = fmaxf(m2, s[i + 2]); m3 = fmaxf(m3, s[i + 3]);
  }
  return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}
// After an abort: wait (bounded) for the copies this thread has issued, so that none lands in a dead CTA.
__device__ __forceinline__ void drain_loads(uint64_t* const* bars, const uint32_t* parity, const bool* issued, int n) {
  for (int i = 0; i < n; ++i) {
    if (!issued[i]) continue;
    const unsigned long long t0 = globaltimer_ns();
    while (!mbar_try_wait(bars[i], parity[i])) {
      if (globaltimer_ns() - t0 > 2000000ull) break;
    }
  }
}
__device__ __forceinline__ void drain_mma(uint64_t* bar) {
  umma_commit(bar);
  const unsigned long long t0 = globaltimer_ns();
  while (!mbar_try_wait(bar, 0)) {
    if (globaltimer_ns() - t0 > 2000000ull) break;
  }
}

// =====================================================================================================  forward
// barriers
enum { F_QFULL = 0, F_KFULL = 1, F_KEMPTY = 3, F_VFULL = 5, F_VEMPTY = 7, F_SFULL = 9, F_SEMPTY = 11, F_PFULL = 13,
       F_PVDONE = 14, F_DRAIN = 15, F_XCHG = 16 /* .. 19: one per group of 32 rows */ };

template <int HD, bool MSK, bool DRP>
__global__ void __launch_bounds__(kThreads, 1) flash_fwd_kernel(const __grid_constant__ FlashParams p) {
  constexpr int SUB = HD / 64;
  constexpr int TILE = SUB * kSub;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = sm;
  uint8_t* sK = sQ + TILE;            // 2 stages
  uint8_t* sV = sK + 2 * TILE;        // 2 stages
  uint8_t* sP = sV + 2 * TILE;        // [128 x 128] bf16: two sub-tiles
  Ctl* ctl = reinterpret_cast<Ctl*>(sP + 2 * kSub);
  Xchg* xc = reinterpret_cast<Xchg*>(sP + 2 * kSub + 256);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const MaskArgs& M = p.m;
  const int nqb = (M.Sq + kBlk - 1) / kBlk;
  const int BH = p.B * p.H;
  // heaviest (last) query blocks first
  const int qb = nqb - 1 - (int)(blockIdx.x / BH);
  const int bh = (int)(blockIdx.x % BH);
  const int b = bh / p.H, h = bh % p.H;
  const int q0 = qb * kBlk;
  int nkb = (M.Sk + kBlk - 1) / kBlk;
  if (M.causal) nkb = min(nkb, qb + 1);

  // counts by barrier index: Q/K/V full and empty 1 each, S full 1, S empty 8 (one per row warp), P full 256, drain 1,
  // row exchange 64 (two warps)
  const int counts[20] = {1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 8, 8, kRowThreads, 1, 1, 64, 64, 64, 64};
  const uint32_t tmem = setup_cta(ctl, counts, 20, warp, lane);
  volatile uint32_t* abort_flag = &ctl->abort_flag;
  unsigned long long* status = p.status;
  const unsigned long long tmo = p.timeout_ns;
  uint64_t* bar = ctl->bar;

  if (warp == kProducerWarp) {
    // ---------------------------------------------------------------------------------- TMA producer
    if (elect_one()) {
      const int cq = head_col(p.q, h), ck = head_col(p.k, h), cv = head_col(p.v, h);
      bool ok = true;
      uint64_t* dbar[5]; uint32_t dpar[5]; bool dis[5] = {false, false, false, false, false};
      mbar_arrive_expect_tx(&bar[F_QFULL], TILE);
      load_tile<SUB>(smem_u32(sQ), &p.mq, p.q_seq1, cq, b, q0, smem_u32(&bar[F_QFULL]));
      dbar[0] = &bar[F_QFULL]; dpar[0] = 0; dis[0] = true;
      for (int j = 0; j < nkb && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        if (!mbar_wait(&bar[F_KEMPTY + st], ph ^ 1u, abort_flag, status, tmo)) { ok = false; break; }
        mbar_arrive_expect_tx(&bar[F_KFULL + st], TILE);
        load_tile<SUB>(smem_u32(sK + st * TILE), &p.mk, p.k_seq1, ck, b, j * kBlk, smem_u32(&bar[F_KFULL + st]));
        dbar[1 + st] = &bar[F_KFULL + st]; dpar[1 + st] = ph; dis[1 + st] = true;
        if (!mbar_wait(&bar[F_VEMPTY + st], ph ^ 1u, abort_flag, status, tmo)) { ok = false; break; }
        mbar_arrive_expect_tx(&bar[F_VFULL + st], TILE);
        load_tile<SUB>(smem_u32(sV + st * TILE), &p.mv, p.v_seq1, cv, b, j * kBlk, smem_u32(&bar[F_VFULL + st]));
        dbar[3 + st] = &bar[F_VFULL + st]; dpar[3 + st] = ph; dis[3 + st] = true;
      }
      if (!ok || *abort_flag) drain_loads(dbar, dpar, dis, 5);
    }
  } else if (warp == kMmaWarp) {
    // ---------------------------------------------------------------------------------- UMMA issuer
    if (elect_one()) {
      const uint32_t id_s = make_idesc_bf16(128, 128, 0, 0), id_o = make_idesc_bf16(128, HD, 0, 1);
      const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV), aP = smem_u32(sP);
      bool ok = true, issued = false;
      auto issue_s = [&](int j) {
        const uint32_t kb = aK + (j & 1) * TILE, d = tmem + (uint32_t)((j & 1) * 128);
#pragma unroll
        for (int u = 0; u < SUB; ++u)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_bf16(d, make_smem_desc(aQ + u * kSub + kk * 32, 16, 1024), make_smem_desc(kb + u * kSub + kk * 32, 16, 1024),
                      id_s, (u | kk) ? 1u : 0u);
        umma_commit(&bar[F_KEMPTY + (j & 1)]);
        umma_commit(&bar[F_SFULL + (j & 1)]);
      };
      ok = mbar_wait(&bar[F_QFULL], 0, abort_flag, status, tmo);
      if (ok && nkb > 0) ok = mbar_wait(&bar[F_KFULL], 0, abort_flag, status, tmo);
      if (ok && nkb > 0) { tc_fence_after(); issue_s(0); issued = true; }
      for (int j = 0; j < nkb && ok; ++j) {
        if (j + 1 < nkb) {
          const int n = j + 1, st = n & 1;
          const uint32_t ph = (uint32_t)(n >> 1) & 1u;
          if (!mbar_wait(&bar[F_KFULL + st], ph, abort_flag, status, tmo)) { ok = false; break; }
          if (!mbar_wait(&bar[F_SEMPTY + st], ph ^ 1u, abort_flag, status, tmo)) { ok = false; break; }
          tc_fence_after();
          issue_s(n);
        }
        const int st = j & 1;
        long long* tm = (p.trace && blockIdx.x == 0 && j < 16) ? p.trace + 256 + j * 8 : nullptr;
        if (tm) tm[0] = clock64();                       // S of the next block issued
        if (!mbar_wait(&bar[F_VFULL + st], (uint32_t)(j >> 1) & 1u, abort_flag, status, tmo)) { ok = false; break; }
        if (tm) tm[1] = clock64();                       // V landed
        if (!mbar_wait(&bar[F_PFULL], (uint32_t)j & 1u, abort_flag, status, tmo)) { ok = false; break; }
        if (tm) tm[2] = clock64();                       // P written
        tc_fence_after();
        const uint32_t vb = aV + st * TILE;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_bf16(tmem + 256, make_smem_desc(aP + (kk >> 2) * kSub + (kk & 3) * 32, 16, 1024),
                    make_smem_desc(vb + kk * 2048, kSub, 1024), id_o, (j > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&bar[F_VEMPTY + st]);
        umma_commit(&bar[F_PVDONE]);
        if (tm) tm[3] = clock64();                       // P V issued
      }
      if (!ok && issued) drain_mma(&bar[F_DRAIN]);
    }
  } else {
    // ---------------------------------------------------------------------------------- row threads
    const int wg = warp >> 2, rt = tid & 127;          // column half and row of this thread
    const int row = q0 + rt;
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const unsigned long long offset = M.offset + (M.step_ptr ? __ldg(M.step_ptr) * 65536ull : 0ull);
    constexpr int OC = HD / 64;                        // 32-column chunks of O per thread
    float m_used = -INFINITY, l = 0.f;                  // l: this thread's half of the row sum
    bool ok = true;
    // stamps of two row warps of CTA 0: [warp 0 | warp 4][block < 16][event < 8]
    long long* tr = (p.trace && blockIdx.x == 0 && lane == 0 && (warp & 3) == 0) ? p.trace + (warp >> 2) * 128 : nullptr;
    for (int j = 0; j < nkb; ++j) {
      const int buf = j & 1;
      if (tr && j < 16) tr[j * 8 + 0] = clock64();
      uint32_t good = mbar_wait(&bar[F_SFULL + buf], (uint32_t)(j >> 1) & 1u, abort_flag, status, tmo) ? 1u : 0u;
      if (!__all_sync(0xffffffffu, good)) { ok = false; break; }
      tc_fence_after();
      if (tr && j < 16) tr[j * 8 + 1] = clock64();
      float s[64];
#pragma unroll
      for (int c = 0; c < 2; ++c) tmem_ld32f(lane_addr + (uint32_t)(buf * 128 + wg * 64 + c * 32), s + 32 * c);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar[F_SEMPTY + buf]);
      if (tr && j < 16) tr[j * 8 + 2] = clock64();
      const int col0 = j * kBlk + wg * 64;
      const bool plain = !(MSK && (M.mask || M.kpm)) && !(M.causal && j == qb) && (j * kBlk + kBlk <= M.Sk);
      // a block that only needs the scale keeps the raw scores: the scale rides in the exponent's multiply-add
      if (!plain) {
#pragma unroll
        for (int c = 0; c < 2; ++c) score_chunk<32, MSK>(s + 32 * c, row, col0 + 32 * c, b, M, false);
      }
      float mx = max64(s);
      if (plain) mx *= M.scale_log2;      // the scale is positive: the maximum commutes with it
      // both threads of the row must scale with the same reference: exchange the partial maxima
      bool xok = true;
      mx = fmaxf(mx, xchg_row(xc, &bar[F_XCHG + (warp & 3)], wg, rt, (uint32_t)j, mx, abort_flag, status, tmo, xok));
      if (!__all_sync(0xffffffffu, xok ? 1u : 0u)) { ok = false; break; }
      if (tr && j < 16) tr[j * 8 + 3] = clock64();
      const float cand = fmaxf(m_used, mx);
      const bool need = cand > m_used + kRescaleGap;
      const float m_new = need ? cand : m_used;
      const float mref = (m_new == -INFINITY) ? 0.f : m_new;
      const float mul = plain ? M.scale_log2 : 1.f;
      if (j > 0) {
        // P V of the previous block must be complete before the P tile is overwritten and before O is rescaled (it was
        // issued a whole block ago: this wait is almost always over at once)
        good = mbar_wait(&bar[F_PVDONE], (uint32_t)(j - 1) & 1u, abort_flag, status, tmo) ? 1u : 0u;
        if (!__all_sync(0xffffffffu, good)) { ok = false; break; }
        tc_fence_after();
        if (__any_sync(0xffffffffu, need)) {
          const float alpha = need ? ex2_approx(m_used - cand) : 1.f;
#pragma unroll
          for (int c = 0; c < OC; ++c) {
            float o[32];
            tmem_ld32f(lane_addr + (uint32_t)(256 + (wg * OC + c) * 32), o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] *= alpha;
            tmem_st32f(lane_addr + (uint32_t)(256 + (wg * OC + c) * 32), o);
          }
          tmem_st_wait();
          l *= alpha;
        }
      }
      if (tr && j < 16) tr[j * 8 + 4] = clock64();
      // exponentials and the stores of P, eight columns at a time: the stores of one group issue while the special-
      // function unit works on the next (the 64 ex2 of a thread are what bounds this loop)
      float r0 = 0.f, r1 = 0.f, r2 = 0.f, r3 = 0.f;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float* e = s + 8 * c;
#pragma unroll
        for (int i = 0; i < 8; ++i) e[i] = ex2_approx(fmaf(e[i], mul, -mref));
        r0 += e[0] + e[4]; r1 += e[1] + e[5]; r2 += e[2] + e[6]; r3 += e[3] + e[7];
        if constexpr (DRP) {
          const uint32_t keep = keep_bits<8>(M, offset, bh, min(row, M.Sq - 1), col0 + 8 * c);
#pragma unroll
          for (int i = 0; i < 8; ++i) e[i] = ((keep >> i) & 1u) ? e[i] * M.drop_scale : 0.f;
        }
        *reinterpret_cast<uint4*>(sP + wg * kSub + sw128(rt, c)) = pack8f(e);
      }
      m_used = m_new;
      l += (r0 + r1) + (r2 + r3);
      if (tr && j < 16) tr[j * 8 + 5] = clock64();
      if (tr && j < 16) tr[j * 8 + 6] = clock64();
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&bar[F_PFULL]);
      if (tr && j < 16) tr[j * 8 + 7] = clock64();
    }
    if (ok && nkb > 0) {
      uint32_t good = mbar_wait(&bar[F_PVDONE], (uint32_t)(nkb - 1) & 1u, abort_flag, status, tmo) ? 1u : 0u;
      if (!__all_sync(0xffffffffu, good)) ok = false;
    }
    if (ok) {
      bool xok = true;
      const float l_all = l + xchg_row(xc, &bar[F_XCHG + (warp & 3)], wg, rt, (uint32_t)nkb, l, abort_flag, status, tmo, xok);
      if (!__all_sync(0xffffffffu, xok ? 1u : 0u)) ok = false;
      if (ok) {
        tc_fence_after();
        const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
        __nv_bfloat16* dst = row < M.Sq ? row_ptr(p.o, b, row, h) : nullptr;
#pragma unroll
        for (int c = 0; c < OC; ++c) {
          const int cc = wg * OC + c;
          float o[32];
          if (nkb > 0) {
            tmem_ld32f(lane_addr + (uint32_t)(256 + cc * 32), o);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = 0.f;
          }
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] *= inv;
          if (dst) {
#pragma unroll
            for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(dst + cc * 32 + q * 8) = pack8f(o + 8 * q);
          }
        }
        if (wg == 0 && row < M.Sq && p.lse) {
          const float mref = (m_used == -INFINITY) ? 0.f : m_used;
          p.lse[(long long)bh * M.Sq + row] = l_all > 0.f ? mref + log2f(l_all) : INFINITY;
        }
      }
    }
  }
  teardown_cta(tmem, warp);
}

// =====================================================================================================  dQ
// CTA = 128 queries of one (batch, head); the keys are walked in sub-blocks of 64, three stages of K / V deep:
//   S = Q K^T and dP = dO V^T      [128 queries x 64 keys] each, in TMEM, double-buffered
//   row threads (TMEM lane = query, two threads per query with 32 keys each): dS = P (dP - delta) as bf16 into a
//                                  [128 x 64] K-major shared tile
//   dQ += dS K                     contraction over the 64 keys; B = the K stage read MN-major
// The products of sub-block i+1 run while the row threads work on sub-block i.
enum { Q_QFULL = 0, Q_KVFULL = 1 /* 3 stages */, Q_KVEMPTY = 4 /* 3 stages */, Q_SDPFULL = 7 /* 2 */, Q_SDPEMPTY = 9 /* 2 */,
       Q_DSFULL = 11, Q_DSEMPTY = 12, Q_DONE = 13, Q_DRAIN = 14 };

template <int HD, bool MSK, bool DRP>
__global__ void __launch_bounds__(kThreads, 1) flash_dq_kernel(const __grid_constant__ FlashParams p) {
  constexpr int SUB = HD / 64;
  constexpr int TILE = SUB * kSub;          // Q or dO: 128 rows
  constexpr int KT = SUB * kHalfTile;       // one stage of K or V: 64 rows
  constexpr int NS = kBwdStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = sm;
  uint8_t* sG = sQ + TILE;            // dO
  uint8_t* sK = sG + TILE;            // NS stages
  uint8_t* sV = sK + NS * KT;         // NS stages
  uint8_t* sS = sV + NS * KT;         // dS [128 queries x 64 keys] bf16
  Ctl* ctl = reinterpret_cast<Ctl*>(sS + kSub);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const MaskArgs& M = p.m;
  const int nqb = (M.Sq + kBlk - 1) / kBlk;
  const int BH = p.B * p.H;
  const int qb = nqb - 1 - (int)(blockIdx.x / BH);
  const int bh = (int)(blockIdx.x % BH);
  const int b = bh / p.H, h = bh % p.H;
  const int q0 = qb * kBlk;
  int nsb = (M.Sk + kHalf - 1) / kHalf;                 // key sub-blocks
  if (M.causal) nsb = min(nsb, 2 * (qb + 1));
  // counts by barrier index: Q/dO full 1; K/V stage full and empty 1; S/dP full 1, S/dP empty 8 (one per row warp);
  // dS full 256; the rest 1
  const int counts[15] = {1, 1, 1, 1, 1, 1, 1, 1, 1, 8, 8, kRowThreads, 1, 1, 1};
  const uint32_t tmem = setup_cta(ctl, counts, 15, warp, lane);
  volatile uint32_t* abort_flag = &ctl->abort_flag;
  unsigned long long* status = p.status;
  const unsigned long long tmo = p.timeout_ns;
  uint64_t* bar = ctl->bar;

  if (warp == kProducerWarp) {
    if (elect_one()) {
      const int cq = head_col(p.q, h), ck = head_col(p.k, h), cv = head_col(p.v, h), cg = head_col(p.dout, h);
      bool ok = true;
      uint64_t* dbar[1 + NS]; uint32_t dpar[1 + NS]; bool dis[1 + NS];
      for (int i = 0; i < 1 + NS; ++i) dis[i] = false;
      mbar_arrive_expect_tx(&bar[Q_QFULL], 2 * TILE);
      load_tile<SUB>(smem_u32(sQ), &p.mq, p.q_seq1, cq, b, q0, smem_u32(&bar[Q_QFULL]));
      load_tile<SUB>(smem_u32(sG), &p.mdo, p.do_seq1, cg, b, q0, smem_u32(&bar[Q_QFULL]));
      dbar[0] = &bar[Q_QFULL]; dpar[0] = 0; dis[0] = true;
      for (int j = 0; j < nsb && ok; ++j) {
        const int st = j % NS;
        const uint32_t ph = (uint32_t)(j / NS) & 1u;
        if (!mbar_wait(&bar[Q_KVEMPTY + st], ph ^ 1u, abort_flag, status, tmo)) { ok = false; break; }
        mbar_arrive_expect_tx(&bar[Q_KVFULL + st], 2 * KT);
        load_tile64<SUB>(smem_u32(sK + st * KT), &p.mk64, p.k_seq1, ck, b, j * kHalf, smem_u32(&bar[Q_KVFULL + st]));
        load_tile64<SUB>(smem_u32(sV + st * KT), &p.mv64, p.v_seq1, cv, b, j * kHalf, smem_u32(&bar[Q_KVFULL + st]));
        dbar[1 + st] = &bar[Q_KVFULL + st]; dpar[1 + st] = ph; dis[1 + st] = true;
      }
      if (!ok || *abort_flag) drain_loads(dbar, dpar, dis, 1 + NS);
    }
  } else if (warp == kMmaWarp) {
    if (elect_one()) {
      const uint32_t id_s = make_idesc_bf16(128, kHalf, 0, 0), id_q = make_idesc_bf16(128, HD, 0, 1);
      const uint32_t aQ = smem_u32(sQ), aG = smem_u32(sG), aK = smem_u32(sK), aV = smem_u32(sV), aS = smem_u32(sS);
      bool ok = mbar_wait(&bar[Q_QFULL], 0, abort_flag, status, tmo);
      bool issued = false;
      // S = Q K^T (columns 0..63 of the buffer), dP = dO V^T (columns 64..127)
      auto issue_sdp = [&](int n) {
        const uint32_t ks = aK + (n % NS) * KT, vs = aV + (n % NS) * KT, d = tmem + (uint32_t)((n & 1) * 128);
#pragma unroll
        for (int u = 0; u < SUB; ++u)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_bf16(d, make_smem_desc(aQ + u * kSub + kk * 32, 16, 1024), make_smem_desc(ks + u * kHalfTile + kk * 32, 16, 1024),
                      id_s, (u | kk) ? 1u : 0u);
#pragma unroll
        for (int u = 0; u < SUB; ++u)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_bf16(d + 64, make_smem_desc(aG + u * kSub + kk * 32, 16, 1024),
                      make_smem_desc(vs + u * kHalfTile + kk * 32, 16, 1024), id_s, (u | kk) ? 1u : 0u);
        umma_commit(&bar[Q_SDPFULL + (n & 1)]);
      };
      if (ok && nsb > 0) ok = mbar_wait(&bar[Q_KVFULL], 0, abort_flag, status, tmo);
      if (ok && nsb > 0) { tc_fence_after(); issue_sdp(0); issued = true; }
      for (int j = 0; j < nsb && ok; ++j) {
        if (j + 1 < nsb) {
          const int n = j + 1;
          if (!mbar_wait(&bar[Q_KVFULL + n % NS], (uint32_t)(n / NS) & 1u, abort_flag, status, tmo)) { ok = false; break; }
          if (!mbar_wait(&bar[Q_SDPEMPTY + (n & 1)], ((uint32_t)(n >> 1) & 1u) ^ 1u, abort_flag, status, tmo)) { ok = false; break; }
          tc_fence_after();
          issue_sdp(n);
        }
        if (!mbar_wait(&bar[Q_DSFULL], (uint32_t)j & 1u, abort_flag, status, tmo)) { ok = false; break; }
        tc_fence_after();
        // dQ += dS K   (A = dS, K-major over the 64 keys; B = the K stage read MN-major)
        const uint32_t ks = aK + (j % NS) * KT;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16(tmem + 256, make_smem_desc(aS + kk * 32, 16, 1024), make_smem_desc(ks + kk * 2048, kHalfTile, 1024), id_q,
                    (j > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&bar[Q_KVEMPTY + j % NS]);
        umma_commit(&bar[Q_DSEMPTY]);
        if (j == nsb - 1) umma_commit(&bar[Q_DONE]);
      }
      if (!ok && issued) drain_mma(&bar[Q_DRAIN]);
    }
  } else {
    const int wg = warp >> 2, rt = tid & 127;          // key half and query row of this thread
    const int row = q0 + rt;
    const bool live = row < M.Sq;
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const unsigned long long offset = M.offset + (M.step_ptr ? __ldg(M.step_ptr) * 65536ull : 0ull);
    // delta = rowsum(dO * O), kept for the dK / dV kernel as well (both threads of a row compute it, one stores it)
    float delta = 0.f, lse2 = INFINITY;
    if (live) {
      const uint4* op = reinterpret_cast<const uint4*>(row_ptr(p.o, b, row, h));
      const uint4* gp = reinterpret_cast<const uint4*>(row_ptr(p.dout, b, row, h));
#pragma unroll
      for (int c = 0; c < HD / 8; ++c) {
        const uint4 a = __ldg(op + c), g = __ldg(gp + c);
        delta += bf16_lo(a.x) * bf16_lo(g.x) + bf16_hi(a.x) * bf16_hi(g.x) + bf16_lo(a.y) * bf16_lo(g.y) +
                 bf16_hi(a.y) * bf16_hi(g.y) + bf16_lo(a.z) * bf16_lo(g.z) + bf16_hi(a.z) * bf16_hi(g.z) +
                 bf16_lo(a.w) * bf16_lo(g.w) + bf16_hi(a.w) * bf16_hi(g.w);
      }
      if (wg == 0) p.delta[(long long)bh * M.Sq + row] = delta;
      lse2 = p.lse[(long long)bh * M.Sq + row];
    }
    bool ok = true;
    for (int j = 0; j < nsb; ++j) {
      const int buf = j & 1;
      uint32_t good = mbar_wait(&bar[Q_SDPFULL + buf], (uint32_t)(j >> 1) & 1u, abort_flag, status, tmo) ? 1u : 0u;
      if (!__all_sync(0xffffffffu, good)) { ok = false; break; }
      tc_fence_after();
      float x[32], dp[32];
      tmem_ld32f(lane_addr + (uint32_t)(buf * 128 + wg * 32), x);
      tmem_ld32f(lane_addr + (uint32_t)(buf * 128 + 64 + wg * 32), dp);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar[Q_SDPEMPTY + buf]);
      const int col0 = j * kHalf + wg * 32;
      // the diagonal crosses the last two sub-blocks of a causal query block
      const bool plain = !(MSK && (M.mask || M.kpm)) && !(M.causal && j >= 2 * qb) && (j * kHalf + kHalf <= M.Sk);
      score_chunk<32, MSK>(x, row, col0, b, M, plain);
      uint32_t keep = 0xffffffffu;
      if constexpr (DRP) keep = keep_bits<32>(M, offset, bh, min(row, M.Sq - 1), col0);
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float pr = ex2_approx(x[i] - lse2);
        const float d = ((keep >> i) & 1u) ? dp[i] * M.drop_scale : 0.f;
        x[i] = pr * (d - delta);
      }
      if (j > 0) {
        // the product of the previous sub-block must have read the dS tile
        good = mbar_wait(&bar[Q_DSEMPTY], (uint32_t)(j - 1) & 1u, abort_flag, status, tmo) ? 1u : 0u;
        if (!__all_sync(0xffffffffu, good)) { ok = false; break; }
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(sS + sw128(rt, wg * 4 + c)) = pack8f(x + 8 * c);
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&bar[Q_DSFULL]);
    }
    if (ok && nsb > 0) {
      uint32_t good = mbar_wait(&bar[Q_DONE], 0, abort_flag, status, tmo) ? 1u : 0u;
      if (!__all_sync(0xffffffffu, good)) ok = false;
    }
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* dst = live ? row_ptr(p.dq, b, row, h) : nullptr;
#pragma unroll
      for (int cc = 0; cc < HD / 64; ++cc) {
        const int c = wg * (HD / 64) + cc;
        float o[32];
        if (nsb > 0) {
          tmem_ld32f(lane_addr + (uint32_t)(256 + c * 32), o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] *= M.sm_scale;
        if (dst) {
#pragma unroll
          for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(dst + c * 32 + q * 8) = pack8f(o + 8 * q);
        }
      }
    }
  }
  teardown_cta(tmem, warp);
}

// =====================================================================================================  dK / dV
// CTA = 128 keys of one (batch, head).  The rows of every product are KEYS (transposed formulation), and the queries are
// walked in sub-blocks of 64:
//   S^T = K Q^T and dP^T = V dO^T            [128 keys x 64 queries] each, in TMEM, double-buffered
//   row threads (TMEM lane = key, two threads per key with 32 queries each): P^T and dS^T as bf16 into two
//                                            [128 x 64] K-major shared tiles
//   dV += P^T dO,  dK += dS^T Q              contraction over the 64 queries; B = the dO / Q stage read MN-major
// With 64-query stages three of them fit beside K and V also at head_dim 128, and the double-buffered S^T / dP^T let the
// products of sub-block i+1 run while the row threads work on sub-block i.  The per-query statistics (log-sum-exp and
// delta) of a stage are put into shared memory by the producer warp and read as broadcasts.
enum { K_KVFULL = 0, K_QGFULL = 1 /* 3 stages */, K_QGEMPTY = 4 /* 3 stages */, K_SDPFULL = 7 /* 2 */, K_SDPEMPTY = 9 /* 2 */,
       K_DSFULL = 11, K_DSEMPTY = 12, K_DONE = 13, K_DRAIN = 14 };

template <int HD, bool MSK, bool DRP>
__global__ void __launch_bounds__(kThreads, 1) flash_dkv_kernel(const __grid_constant__ FlashParams p) {
  constexpr int SUB = HD / 64;
  constexpr int TILE = SUB * kSub;          // K or V: 128 rows
  constexpr int QT = SUB * kHalfTile;       // one stage of Q or dO: 64 rows
  constexpr int NS = kBwdStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = sm;
  uint8_t* sV = sK + TILE;
  uint8_t* sQ = sV + TILE;            // NS stages
  uint8_t* sG = sQ + NS * QT;         // NS stages (dO)
  uint8_t* sP = sG + NS * QT;         // dropped probabilities, transposed: [keys][64 queries]
  uint8_t* sS = sP + kSub;            // dS transposed
  Ctl* ctl = reinterpret_cast<Ctl*>(sS + kSub);
  float* sStat = reinterpret_cast<float*>(sS + kSub + 256);   // per stage: 64 log-sum-exp values, 64 deltas
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const MaskArgs& M = p.m;
  const int nsub = (M.Sq + kHalf - 1) / kHalf;
  const int BH = p.B * p.H;
  // with a causal mask the first key blocks see the most query blocks: they go first
  const int kb = (int)(blockIdx.x / BH);
  const int bh = (int)(blockIdx.x % BH);
  const int b = bh / p.H, h = bh % p.H;
  const int k0 = kb * kBlk;
  const int s_begin = M.causal ? k0 / kHalf : 0;
  const int nit = max(nsub - s_begin, 0);
  // counts by barrier index: K/V full 1; stage full 33 (the copy's issuer + 32 lanes that wrote the statistics); stage
  // empty 1; S/dP full 1, S/dP empty 8 (one per row warp); dS full 256; the rest 1
  const int counts[15] = {1, 33, 33, 33, 1, 1, 1, 1, 1, 8, 8, kRowThreads, 1, 1, 1};
  const uint32_t tmem = setup_cta(ctl, counts, 15, warp, lane);
  volatile uint32_t* abort_flag = &ctl->abort_flag;
  unsigned long long* status = p.status;
  const unsigned long long tmo = p.timeout_ns;
  uint64_t* bar = ctl->bar;

  if (warp == kProducerWarp) {
    // the whole warp walks the stages: lane 0 issues the copies, every lane fetches the statistics of two queries
    const int cq = head_col(p.q, h), ck = head_col(p.k, h), cv = head_col(p.v, h), cg = head_col(p.dout, h);
    bool ok = true;
    uint64_t* dbar[1 + NS]; uint32_t dpar[1 + NS]; bool dis[1 + NS];
    for (int i = 0; i < 1 + NS; ++i) dis[i] = false;
    if (lane == 0) {
      mbar_arrive_expect_tx(&bar[K_KVFULL], 2 * TILE);
      load_tile<SUB>(smem_u32(sK), &p.mk, p.k_seq1, ck, b, k0, smem_u32(&bar[K_KVFULL]));
      load_tile<SUB>(smem_u32(sV), &p.mv, p.v_seq1, cv, b, k0, smem_u32(&bar[K_KVFULL]));
      dbar[0] = &bar[K_KVFULL]; dpar[0] = 0; dis[0] = true;
    }
    for (int it = 0; it < nit; ++it) {
      const int st = it % NS;
      const uint32_t ph = (uint32_t)(it / NS) & 1u;
      const uint32_t good = mbar_wait(&bar[K_QGEMPTY + st], ph ^ 1u, abort_flag, status, tmo) ? 1u : 0u;
      if (!__all_sync(0xffffffffu, good)) { ok = false; break; }
      const int q0 = (s_begin + it) * kHalf;
      if (lane == 0) {
        mbar_arrive_expect_tx(&bar[K_QGFULL + st], 2 * QT);
        load_tile64<SUB>(smem_u32(sQ + st * QT), &p.mq64, p.q_seq1, cq, b, q0, smem_u32(&bar[K_QGFULL + st]));
        load_tile64<SUB>(smem_u32(sG + st * QT), &p.mdo64, p.do_seq1, cg, b, q0, smem_u32(&bar[K_QGFULL + st]));
        dbar[1 + st] = &bar[K_QGFULL + st]; dpar[1 + st] = ph; dis[1 + st] = true;
      }
      float2 ls = make_float2(INFINITY, INFINITY), dl = make_float2(0.f, 0.f);
      const int q = q0 + 2 * lane;
      const long long base = (long long)bh * M.Sq;
      if (q < M.Sq) { ls.x = __ldg(p.lse + base + q); dl.x = __ldg(p.delta + base + q); }
      if (q + 1 < M.Sq) { ls.y = __ldg(p.lse + base + q + 1); dl.y = __ldg(p.delta + base + q + 1); }
      float* stat = sStat + st * 2 * kHalf;
      *reinterpret_cast<float2*>(stat + 2 * lane) = ls;
      *reinterpret_cast<float2*>(stat + kHalf + 2 * lane) = dl;
      mbar_arrive(&bar[K_QGFULL + st]);
    }
    if (lane == 0 && (!ok || *abort_flag)) drain_loads(dbar, dpar, dis, 1 + NS);
  } else if (warp == kMmaWarp) {
    if (elect_one()) {
      const uint32_t id_s = make_idesc_bf16(128, kHalf, 0, 0), id_t = make_idesc_bf16(128, HD, 0, 1);
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ), aG = smem_u32(sG);
      const uint32_t aP = smem_u32(sP), aS = smem_u32(sS);
      bool ok = mbar_wait(&bar[K_KVFULL], 0, abort_flag, status, tmo);
      bool issued = false;
      // S^T = K Q^T (columns 0..63 of the buffer), dP^T = V dO^T (columns 64..127): rows = keys
      auto issue_sdp = [&](int n) {
        const uint32_t qs = aQ + (n % NS) * QT, gs = aG + (n % NS) * QT, d = tmem + (uint32_t)((n & 1) * 128);
#pragma unroll
        for (int u = 0; u < SUB; ++u)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_bf16(d, make_smem_desc(aK + u * kSub + kk * 32, 16, 1024), make_smem_desc(qs + u * kHalfTile + kk * 32, 16, 1024),
                      id_s, (u | kk) ? 1u : 0u);
#pragma unroll
        for (int u = 0; u < SUB; ++u)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_bf16(d + 64, make_smem_desc(aV + u * kSub + kk * 32, 16, 1024),
                      make_smem_desc(gs + u * kHalfTile + kk * 32, 16, 1024), id_s, (u | kk) ? 1u : 0u);
        umma_commit(&bar[K_SDPFULL + (n & 1)]);
      };
      if (ok && nit > 0) ok = mbar_wait(&bar[K_QGFULL], 0, abort_flag, status, tmo);
      if (ok && nit > 0) { tc_fence_after(); issue_sdp(0); issued = true; }
      for (int it = 0; it < nit && ok; ++it) {
        if (it + 1 < nit) {
          const int n = it + 1;
          if (!mbar_wait(&bar[K_QGFULL + n % NS], (uint32_t)(n / NS) & 1u, abort_flag, status, tmo)) { ok = false; break; }
          if (!mbar_wait(&bar[K_SDPEMPTY + (n & 1)], ((uint32_t)(n >> 1) & 1u) ^ 1u, abort_flag, status, tmo)) { ok = false; break; }
          tc_fence_after();
          issue_sdp(n);
        }
        long long* tm = (p.trace && blockIdx.x == 0 && it < 16) ? p.trace + 256 + it * 8 : nullptr;
        if (tm) tm[0] = clock64();                       // S / dP of the next sub-block issued
        if (!mbar_wait(&bar[K_DSFULL], (uint32_t)it & 1u, abort_flag, status, tmo)) { ok = false; break; }
        if (tm) tm[1] = clock64();                       // dS written
        tc_fence_after();
        const uint32_t qs = aQ + (it % NS) * QT, gs = aG + (it % NS) * QT;
        // dV += P^T dO, dK += dS^T Q: A = the transposed tiles (K-major over the 64 queries), B = the stage, MN-major
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16(tmem + 256, make_smem_desc(aP + kk * 32, 16, 1024), make_smem_desc(gs + kk * 2048, kHalfTile, 1024), id_t,
                    (it > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16(tmem + 256 + HD, make_smem_desc(aS + kk * 32, 16, 1024), make_smem_desc(qs + kk * 2048, kHalfTile, 1024),
                    id_t, (it > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&bar[K_QGEMPTY + it % NS]);
        umma_commit(&bar[K_DSEMPTY]);
        if (it == nit - 1) umma_commit(&bar[K_DONE]);
        if (tm) tm[2] = clock64();                       // dV / dK issued
      }
      if (!ok && issued) drain_mma(&bar[K_DRAIN]);
    }
  } else {
    const int wg = warp >> 2, rt = tid & 127;          // query half and key row of this thread
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const unsigned long long offset = M.offset + (M.step_ptr ? __ldg(M.step_ptr) * 65536ull : 0ull);
    const int key = k0 + rt;
    bool key_dead = key >= M.Sk;
    if constexpr (MSK) key_dead = key_dead || (M.kpm && __ldg(M.kpm + (long long)b * M.kpm_ld + key));
    const bool keys_plain = !(MSK && (M.mask || M.kpm)) && (k0 + kBlk <= M.Sk);
    bool ok = true;
    long long* tr = (p.trace && blockIdx.x == 0 && lane == 0 && (warp & 3) == 0) ? p.trace + (warp >> 2) * 128 : nullptr;
    for (int it = 0; it < nit; ++it) {
      const int st = it % NS, buf = it & 1;
      const int qbase = (s_begin + it) * kHalf + wg * 32;      // first query of this thread
      if (tr && it < 16) tr[it * 8 + 0] = clock64();
      uint32_t good = mbar_wait(&bar[K_QGFULL + st], (uint32_t)(it / NS) & 1u, abort_flag, status, tmo) ? 1u : 0u;
      if (tr && it < 16) tr[it * 8 + 1] = clock64();
      if (good) good = mbar_wait(&bar[K_SDPFULL + buf], (uint32_t)(it >> 1) & 1u, abort_flag, status, tmo) ? 1u : 0u;
      if (!__all_sync(0xffffffffu, good)) { ok = false; break; }
      tc_fence_after();
      if (tr && it < 16) tr[it * 8 + 2] = clock64();
      float x[32], dp[32];
      tmem_ld32f(lane_addr + (uint32_t)(buf * 128 + wg * 32), x);
      tmem_ld32f(lane_addr + (uint32_t)(buf * 128 + 64 + wg * 32), dp);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar[K_SDPEMPTY + buf]);
      if (tr && it < 16) tr[it * 8 + 3] = clock64();
      // the diagonal crosses the first two sub-blocks of a causal key block
      const bool plain = keys_plain && !(M.causal && it < 2);
      const float4* lse4 = reinterpret_cast<const float4*>(sStat + st * 2 * kHalf + wg * 32);
      const float4* del4 = reinterpret_cast<const float4*>(sStat + st * 2 * kHalf + kHalf + wg * 32);
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        const float4 L4 = lse4[g], D4 = del4[g];
        const float lse_[4] = {L4.x, L4.y, L4.z, L4.w}, del_[4] = {D4.x, D4.y, D4.z, D4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = 4 * g + e;
          const int q = qbase + i;
          float xs = x[i] * M.scale_log2;
          if (!plain) {
            if constexpr (MSK) {
              if (M.mask && q < M.Sq && key < M.Sk) {
                const long long mi = (long long)q * M.mask_ld + key;
                xs += (M.mask_fp32 ? __ldg(reinterpret_cast<const float*>(M.mask) + mi)
                                   : __bfloat162float(__ldg(reinterpret_cast<const __nv_bfloat16*>(M.mask) + mi))) * kLog2e;
              }
            }
            if (key_dead || (M.causal && key > q)) xs = -INFINITY;
          }
          const float pr = ex2_approx(xs - lse_[e]);
          bool kp = true;
          if constexpr (DRP) {
            const unsigned long long idx = ((unsigned long long)bh * M.Sq + min(q, M.Sq - 1)) * (unsigned long long)M.Sk + key;
            kp = dropout_keep(M.seed, offset, idx, M.thresh);
          }
          const float d = kp ? dp[i] * M.drop_scale : 0.f;
          dp[i] = pr * (d - del_[e]);             // dS
          x[i] = kp ? pr * M.drop_scale : 0.f;    // dropped probability
        }
      }
      if (tr && it < 16) tr[it * 8 + 4] = clock64() + (x[0] == 12345.f ? 1 : 0);
      if (it > 0) {
        // the products of the previous sub-block must have read the two tiles
        good = mbar_wait(&bar[K_DSEMPTY], (uint32_t)(it - 1) & 1u, abort_flag, status, tmo) ? 1u : 0u;
        if (!__all_sync(0xffffffffu, good)) { ok = false; break; }
      }
      if (tr && it < 16) tr[it * 8 + 5] = clock64();
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t off = sw128(rt, wg * 4 + c);
        *reinterpret_cast<uint4*>(sP + off) = pack8f(x + 8 * c);
        *reinterpret_cast<uint4*>(sS + off) = pack8f(dp + 8 * c);
      }
      if (tr && it < 16) tr[it * 8 + 6] = clock64();
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&bar[K_DSFULL]);
      if (tr && it < 16) tr[it * 8 + 7] = clock64();
    }
    if (ok && nit > 0) {
      uint32_t good = mbar_wait(&bar[K_DONE], 0, abort_flag, status, tmo) ? 1u : 0u;
      if (!__all_sync(0xffffffffu, good)) ok = false;
    }
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* dvp = key < M.Sk ? row_ptr(p.dv, b, key, h) : nullptr;
      __nv_bfloat16* dkp = key < M.Sk ? row_ptr(p.dk, b, key, h) : nullptr;
#pragma unroll
      for (int cc = 0; cc < HD / 64; ++cc) {
        const int c = wg * (HD / 64) + cc;
        float o[32];
        if (nit > 0) { tmem_ld32f(lane_addr + (uint32_t)(256 + c * 32), o); tmem_ld_wait(); }
        else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0.f;
        }
        if (dvp) {
#pragma unroll
          for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(dvp + c * 32 + q * 8) = pack8f(o + 8 * q);
        }
        if (nit > 0) { tmem_ld32f(lane_addr + (uint32_t)(256 + HD + c * 32), o); tmem_ld_wait(); }
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] *= M.sm_scale;
        if (dkp) {
#pragma unroll
          for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(dkp + c * 32 + q * 8) = pack8f(o + 8 * q);
        }
      }
    }
  }
  teardown_cta(tmem, warp);
}

// =====================================================================================================  host
thread_local std::string g_ferr;
long long* g_flash_trace = nullptr;
int ffail(const std::string& s) { g_ferr = s; return -1; }

uint32_t thresh_of(float pdrop) {
  if (pdrop <= 0.f) return 0u;
  double t = (double)pdrop * 4294967296.0;
  if (t > 4294967295.0) t = 4294967295.0;
  return (uint32_t)t;
}

// 3-D map {width columns, dim1, dim2} over a [batch, seq, width] view; the dimension with the smaller stride comes first.
int make_map3(CUtensorMap* m, int* seq1, const RtpFlashRef& r, int B, int S, const char* what, unsigned rows = 128u) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return ffail("cuTensorMapEncodeTiled entry point not found");
  if ((reinterpret_cast<uintptr_t>(r.ptr) & 15) != 0) return ffail(std::string(what) + ": base is not 16-byte aligned");
  if ((r.sb * 2) % 16 || (r.ss * 2) % 16) return ffail(std::string(what) + ": strides must be multiples of 16 bytes");
  if (r.width <= 0) return ffail(std::string(what) + ": width missing");
  const bool s_first = r.ss <= r.sb || B == 1;
  *seq1 = s_first ? 1 : 0;
  cuuint64_t dims[3] = {(cuuint64_t)r.width, (cuuint64_t)(s_first ? S : B), (cuuint64_t)(s_first ? B : S)};
  cuuint64_t strides[2] = {(cuuint64_t)(s_first ? r.ss : r.sb) * 2, (cuuint64_t)(s_first ? r.sb : r.ss) * 2};
  if (B == 1) strides[1] = strides[0] * (cuuint64_t)S;   // a single batch: any legal pitch
  cuuint32_t box[3] = {64u, s_first ? rows : 1u, s_first ? 1u : rows};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  CUresult rc = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, r.ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return ffail(std::string(what) + ": cuTensorMapEncodeTiled failed with code " + std::to_string((int)rc));
  return 0;
}
DRef dref(const RtpFlashRef& r) {
  DRef d;
  d.ptr = r.ptr; d.sb = r.sb; d.ss = r.ss;
  d.col_base = r.col_base; d.hpg = r.hpg > 0 ? r.hpg : 1; d.gstride = r.gstride; d.hstride = r.hstride;
  return d;
}
int check_ref(const RtpFlashRef& r, const char* what, int hd) {
  if (!r.ptr) return ffail(std::string(what) + ": null pointer");
  if ((reinterpret_cast<uintptr_t>(r.ptr) & 15) || (r.sb % 8) || (r.ss % 8) || (r.col_base % 8) || (r.gstride % 8) ||
      (r.hstride % 8))
    return ffail(std::string(what) + ": rows of a head must be 16-byte aligned");
  (void)hd;
  return 0;
}
int fill_common(const RtpFlashArgs* a, FlashParams& P) {
  if (a->head_dim != 64 && a->head_dim != 128) return ffail("flash attention: head_dim must be 64 or 128");
  if (a->B <= 0 || a->H <= 0 || a->Sq <= 0 || a->Sk <= 0) return ffail("flash attention: empty problem");
  if (a->causal && a->Sq != a->Sk) return ffail("flash attention: a causal mask needs Sq == Sk");
  if (a->drop_p > 0.f && a->Sk % 4) return ffail("flash attention: dropout needs Sk to be a multiple of 4");
  if (!a->status) return ffail("flash attention: status word required");
  P.B = a->B; P.H = a->H;
  P.m.mask = a->mask; P.m.mask_ld = a->mask_ld; P.m.mask_fp32 = a->mask_fp32;
  P.m.kpm = a->kpm; P.m.kpm_ld = a->kpm_ld;
  P.m.causal = a->causal; P.m.Sq = a->Sq; P.m.Sk = a->Sk;
  P.m.sm_scale = a->sm_scale; P.m.scale_log2 = a->sm_scale * kLog2e;
  P.m.thresh = thresh_of(a->drop_p);
  P.m.drop_scale = a->drop_p > 0.f ? 1.f / (1.f - a->drop_p) : 1.f;
  P.m.seed = a->seed; P.m.offset = a->offset; P.m.step_ptr = a->step_ptr;
  P.status = a->status;
  P.timeout_ns = 2000000000ull;
  P.trace = g_flash_trace;
  P.lse = a->lse;
  P.delta = a->delta;
  if (check_ref(a->q, "q", a->head_dim) || check_ref(a->k, "k", a->head_dim) || check_ref(a->v, "v", a->head_dim) ||
      check_ref(a->o, "o", a->head_dim))
    return -1;
  if (make_map3(&P.mq, &P.q_seq1, a->q, a->B, a->Sq, "q")) return -1;
  if (make_map3(&P.mk, &P.k_seq1, a->k, a->B, a->Sk, "k")) return -1;
  if (make_map3(&P.mv, &P.v_seq1, a->v, a->B, a->Sk, "v")) return -1;
  P.q = dref(a->q); P.k = dref(a->k); P.v = dref(a->v); P.o = dref(a->o);
  return 0;
}
constexpr int smem_fwd(int hd) { return 1024 + (hd / 64) * kSub * 5 + 2 * kSub + 256 + (int)sizeof(Xchg); }
constexpr int smem_dq(int hd) { return 1024 + (hd / 64) * (2 * kSub + 2 * kBwdStages * kHalfTile) + kSub + 256; }
constexpr int smem_dkv(int hd) {
  return 1024 + (hd / 64) * (2 * kSub + 2 * kBwdStages * kHalfTile) + 2 * kSub + 256 + kBwdStages * 2 * kHalf * 4;
}
static_assert(sizeof(Ctl) <= 256, "control block");
static_assert(smem_dq(128) <= 232448 && smem_dkv(128) <= 232448 && smem_fwd(128) <= 232448, "shared memory budget");

template <auto Kern>
int launch_flash(const FlashParams& P, int grid, int smem, cudaStream_t stream, const char* what) {
  cudaError_t e = ensure_smem<Kern>(smem);
  if (e != cudaSuccess) return ffail(std::string(what) + ": cudaFuncSetAttribute: " + cudaGetErrorString(e));
  e = launch_k(Kern, dim3(grid), dim3(kThreads), smem, stream, P);
  if (e != cudaSuccess) return ffail(std::string(what) + ": " + cudaGetErrorString(e));
  return 0;
}

}  // namespace

extern "C" {

const char* rtp_flash_last_error(void) { return g_ferr.c_str(); }
void rtp_flash_debug_set_trace(long long* device_buffer_512_words) { g_flash_trace = device_buffer_512_words; }

int rtp_flash_fwd(const RtpFlashArgs* a, void* stream) {
  static thread_local FlashParams P;
  if (fill_common(a, P)) return -1;
  if (!a->lse) return ffail("flash attention: lse buffer required");
  const int grid = ((a->Sq + kBlk - 1) / kBlk) * a->B * a->H;
  cudaStream_t s = (cudaStream_t)stream;
  const bool msk = a->mask || a->kpm, drp = P.m.thresh != 0;
#define RTP_FWD(HD, MSK, DRP) launch_flash<flash_fwd_kernel<HD, MSK, DRP>>(P, grid, smem_fwd(HD), s, "flash_fwd")
#define RTP_FWD_HD(HD) (msk ? (drp ? RTP_FWD(HD, true, true) : RTP_FWD(HD, true, false)) \
                            : (drp ? RTP_FWD(HD, false, true) : RTP_FWD(HD, false, false)))
  return a->head_dim == 64 ? RTP_FWD_HD(64) : RTP_FWD_HD(128);
#undef RTP_FWD_HD
#undef RTP_FWD
}

int rtp_flash_bwd(const RtpFlashArgs* a, void* stream) {
  static thread_local FlashParams P;
  if (fill_common(a, P)) return -1;
  if (!a->lse || !a->delta) return ffail("flash attention backward: lse and delta buffers required");
  if (check_ref(a->dout, "dout", a->head_dim) || check_ref(a->dq, "dq", a->head_dim) || check_ref(a->dk, "dk", a->head_dim) ||
      check_ref(a->dv, "dv", a->head_dim))
    return -1;
  if (make_map3(&P.mdo, &P.do_seq1, a->dout, a->B, a->Sq, "dout")) return -1;
  if (make_map3(&P.mq64, &P.q_seq1, a->q, a->B, a->Sq, "q", 64u)) return -1;
  if (make_map3(&P.mdo64, &P.do_seq1, a->dout, a->B, a->Sq, "dout", 64u)) return -1;
  if (make_map3(&P.mk64, &P.k_seq1, a->k, a->B, a->Sk, "k", 64u)) return -1;
  if (make_map3(&P.mv64, &P.v_seq1, a->v, a->B, a->Sk, "v", 64u)) return -1;
  P.dout = dref(a->dout); P.dq = dref(a->dq); P.dk = dref(a->dk); P.dv = dref(a->dv);
  const int gq = ((a->Sq + kBlk - 1) / kBlk) * a->B * a->H;
  const int gk = ((a->Sk + kBlk - 1) / kBlk) * a->B * a->H;
  cudaStream_t s = (cudaStream_t)stream;
  const bool msk = a->mask || a->kpm, drp = P.m.thresh != 0;
#define RTP_BWD(HD, MSK, DRP)                                                                              \
  (launch_flash<flash_dq_kernel<HD, MSK, DRP>>(P, gq, smem_dq(HD), s, "flash_dq")                          \
       ? -1                                                                                                \
       : launch_flash<flash_dkv_kernel<HD, MSK, DRP>>(P, gk, smem_dkv(HD), s, "flash_dkv"))
#define RTP_BWD_HD(HD) (msk ? (drp ? RTP_BWD(HD, true, true) : RTP_BWD(HD, true, false)) \
                            : (drp ? RTP_BWD(HD, false, true) : RTP_BWD(HD, false, false)))
  return a->head_dim == 64 ? RTP_BWD_HD(64) : RTP_BWD_HD(128);
#undef RTP_BWD_HD
#undef RTP_BWD
}

}  // extern "C"
