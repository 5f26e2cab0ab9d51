// Patch matrices for convolution as GEMM: a rotated Conv2d (output channels sharded, reference rtp/module/conv.py:103-114)
// runs on the rotation GEMM kernels as a column-parallel linear over the unfolded input.
//   im2col : x [B, C, H, W] bf16  ->  cols [B*OH*OW, Kp] bf16, column (c, kh, kw) = c*KH*KW + kh*KW + kw, zero padded to Kp
//   col2im : dcols [B*OH*OW, Kp]  ->  dx [B, C, H, W]  (gather form: every input element sums the patch entries that
//            read it, so there are no atomics and the result does not depend on scheduling)
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "kernels.h"

namespace {

std::string g_err;

struct ConvGeom {
  int B, C, H, W, KH, KW, OH, OW, sh, sw, ph, pw, dh, dw, Kp;
};

// One thread per (output position m, input channel c): the position is decoded once and the thread writes the channel's
// KH*KW consecutive patch entries (adjacent threads write adjacent channels, so a warp's stores are contiguous).
// Threads with c == C fill the zero padding of the row up to Kp.
__global__ void im2col_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ cols, ConvGeom g) {
  const int KK = g.KH * g.KW;
  const int K = g.C * KK;
  const int cpr = g.C + (g.Kp > K ? 1 : 0);          // work items per output row
  const long long total = (long long)g.B * g.OH * g.OW * cpr;
  const __nv_bfloat16 zero = __float2bfloat16(0.f);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % cpr);
    const long long m = i / cpr;
    __nv_bfloat16* dst = cols + m * g.Kp;
    if (c == g.C) {
      for (int k = K; k < g.Kp; ++k) dst[k] = zero;
      continue;
    }
    const int ow = (int)(m % g.OW), oh = (int)((m / g.OW) % g.OH), b = (int)(m / ((long long)g.OW * g.OH));
    const __nv_bfloat16* src = x + ((long long)b * g.C + c) * g.H * g.W;
    dst += c * KK;
    const int h0 = oh * g.sh - g.ph, w0 = ow * g.sw - g.pw;
    for (int kh = 0; kh < g.KH; ++kh) {
      const int h = h0 + kh * g.dh;
      const bool hok = h >= 0 && h < g.H;
      for (int kw = 0; kw < g.KW; ++kw) {
        const int w = w0 + kw * g.dw;
        dst[kh * g.KW + kw] = (hok && w >= 0 && w < g.W) ? src[(long long)h * g.W + w] : zero;
      }
    }
  }
}

__global__ void col2im_kernel(const __nv_bfloat16* __restrict__ dcols, __nv_bfloat16* __restrict__ dx, ConvGeom g) {
  const long long total = (long long)g.B * g.C * g.H * g.W;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int w = (int)(i % g.W), h = (int)((i / g.W) % g.H), c = (int)((i / ((long long)g.W * g.H)) % g.C);
    const int b = (int)(i / ((long long)g.W * g.H * g.C));
    float acc = 0.f;
    for (int kh = 0; kh < g.KH; ++kh) {
      const int hn = h + g.ph - kh * g.dh;
      if (hn < 0 || hn % g.sh) continue;
      const int oh = hn / g.sh;
      if (oh >= g.OH) continue;
      for (int kw = 0; kw < g.KW; ++kw) {
        const int wn = w + g.pw - kw * g.dw;
        if (wn < 0 || wn % g.sw) continue;
        const int ow = wn / g.sw;
        if (ow >= g.OW) continue;
        const long long m = ((long long)b * g.OH + oh) * g.OW + ow;
        acc += __bfloat162float(dcols[m * g.Kp + (c * g.KH + kh) * g.KW + kw]);
      }
    }
    dx[i] = __float2bfloat16(acc);
  }
}

int launch_geom(ConvGeom& g, int B, int C, int H, int W, int KH, int KW, int sh, int sw, int ph, int pw, int dh, int dw,
                int Kp) {
  g.B = B; g.C = C; g.H = H; g.W = W; g.KH = KH; g.KW = KW; g.sh = sh; g.sw = sw; g.ph = ph; g.pw = pw; g.dh = dh; g.dw = dw;
  g.OH = (H + 2 * ph - dh * (KH - 1) - 1) / sh + 1;
  g.OW = (W + 2 * pw - dw * (KW - 1) - 1) / sw + 1;
  g.Kp = Kp;
  if (g.OH <= 0 || g.OW <= 0 || Kp < C * KH * KW) { g_err = "im2col: bad geometry"; return -1; }
  return 0;
}

}  // namespace

extern "C" {

const char* rtp_im2col_last_error(void) { return g_err.c_str(); }

int rtp_im2col(const void* x, void* cols, int B, int C, int H, int W, int KH, int KW, int sh, int sw, int ph, int pw,
               int dh, int dw, int Kp, void* stream) {
  ConvGeom g;
  if (launch_geom(g, B, C, H, W, KH, KW, sh, sw, ph, pw, dh, dw, Kp)) return -1;
  const long long total = (long long)g.B * g.OH * g.OW * (g.C + 1);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  im2col_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)cols, g);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { g_err = std::string("im2col: ") + cudaGetErrorString(e); return -1; }
  return 0;
}

int rtp_col2im(const void* dcols, void* dx, int B, int C, int H, int W, int KH, int KW, int sh, int sw, int ph, int pw,
               int dh, int dw, int Kp, void* stream) {
  ConvGeom g;
  if (launch_geom(g, B, C, H, W, KH, KW, sh, sw, ph, pw, dh, dw, Kp)) return -1;
  const long long total = (long long)g.B * g.C * g.H * g.W;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  col2im_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)dcols, (__nv_bfloat16*)dx, g);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { g_err = std::string("col2im: ") + cudaGetErrorString(e); return -1; }
  return 0;
}

}  // extern "C"
