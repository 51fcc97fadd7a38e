// Convolution as GEMM for channels-last bf16 activations (sm_100a): im2col gathers
// the K = KH*KW*Cin patch of every output pixel into a row (tap-major, channels
// fastest, 16-byte copies), the tcgen05 GEMM does the product, and col2im folds the
// patch gradients back as a gather over the taps that touch an input pixel (no
// atomics, deterministic). Covers 3x3, 7x7 and strided 1x1 convolutions with
// Cin a multiple of 8. Replaces the cuDNN convolutions of the reference's ResNet
// (hw/models/resenet.py:14,79,113).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gcow {
namespace conv {

typedef __nv_bfloat16 bf16;

struct Geo {
  int N, H, W, C, KH, KW, stride, pad, OH, OW;
};

// col[(n,oh,ow)][(kh,kw,c)] = x[n][oh*s-p+kh][ow*s-p+kw][c] or 0
__global__ void im2col_kernel(const bf16* __restrict__ x, bf16* __restrict__ col, Geo g) {
  const int cg = g.C / 8, taps = g.KH * g.KW;
  const int64_t total = (int64_t)g.N * g.OH * g.OW * taps * cg;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int c8 = (int)(t % cg);
    int64_t r = t / cg;
    const int tap = (int)(r % taps);
    int64_t p = r / taps;
    const int ow = (int)(p % g.OW); p /= g.OW;
    const int oh = (int)(p % g.OH);
    const int n = (int)(p / g.OH);
    const int ih = oh * g.stride - g.pad + tap / g.KW, iw = ow * g.stride - g.pad + tap % g.KW;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (ih >= 0 && ih < g.H && iw >= 0 && iw < g.W)
      v = *reinterpret_cast<const uint4*>(x + (((int64_t)n * g.H + ih) * g.W + iw) * g.C + c8 * 8);
    *reinterpret_cast<uint4*>(col + t * 8) = v;
  }
}

// dx[n][ih][iw][c] = sum over taps (kh,kw) and outputs (oh,ow) with oh*s-p+kh == ih, ow*s-p+kw == iw of dcol
__global__ void col2im_kernel(const bf16* __restrict__ dcol, bf16* __restrict__ dx, Geo g) {
  const int cg = g.C / 8, taps = g.KH * g.KW;
  const int64_t total = (int64_t)g.N * g.H * g.W * cg;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int c8 = (int)(t % cg);
    int64_t p = t / cg;
    const int iw = (int)(p % g.W); p /= g.W;
    const int ih = (int)(p % g.H);
    const int n = (int)(p / g.H);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int kh = 0; kh < g.KH; kh++) {
      const int a = ih + g.pad - kh;
      if (a < 0 || a % g.stride) continue;
      const int oh = a / g.stride;
      if (oh >= g.OH) continue;
      for (int kw = 0; kw < g.KW; kw++) {
        const int b = iw + g.pad - kw;
        if (b < 0 || b % g.stride) continue;
        const int ow = b / g.stride;
        if (ow >= g.OW) continue;
        const int64_t row = ((int64_t)n * g.OH + oh) * g.OW + ow;
        const uint4 u = *reinterpret_cast<const uint4*>(dcol + ((row * taps + kh * g.KW + kw) * cg + c8) * 8);
        const __nv_bfloat162* q = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; i++) { float2 f = __bfloat1622float2(q[i]); acc[2 * i] += f.x; acc[2 * i + 1] += f.y; }
      }
    }
    uint4 o;
    __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int i = 0; i < 4; i++) ob[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
    *reinterpret_cast<uint4*>(dx + t * 8) = o;
  }
}

// Patch matrix for an input whose channel count is not a multiple of 8 (the 3-channel image in front of
// the stem): row length Kp >= KH*KW*C is a multiple of 8, element kk of a row is tap kk / C, channel kk % C,
// columns past KH*KW*C are zero. A CTA serves kTileW consecutive output pixels of one output row: it stages the
// KH input-row segments they touch in shared memory (coalesced reads, zero fill outside the image), then every
// thread assembles eight elements of a patch row from there and stores them as 16 bytes, so the patch matrix -
// by far the larger side - is written in whole, consecutive rows.
constexpr int kTileW = 32;
__global__ void __launch_bounds__(256)
im2col_anyc_kernel(const bf16* __restrict__ x, bf16* __restrict__ col, Geo g, int Kp, int tiles_w) {
  extern __shared__ bf16 patch[];                          // [KH][span][C]
  const int span = (kTileW - 1) * g.stride + g.KW;         // input pixels per row segment
  const int rowlen = span * g.C, RC = g.KW * g.C, K = g.KH * RC;
  int b = blockIdx.x;
  const int tw = b % tiles_w; b /= tiles_w;
  const int oh = b % g.OH;
  const int n = b / g.OH;
  const int ow0 = tw * kTileW;
  const int h0 = oh * g.stride - g.pad, w0 = ow0 * g.stride - g.pad;
  for (int i = threadIdx.x; i < g.KH * rowlen; i += blockDim.x) {
    const int kh = i / rowlen, r = i - kh * rowlen;
    const int ih = h0 + kh, iw = w0 + r / g.C;
    bf16 e = __float2bfloat16(0.0f);
    if (ih >= 0 && ih < g.H && iw >= 0 && iw < g.W) e = x[(((int64_t)n * g.H + ih) * g.W + w0) * g.C + r];
    patch[i] = e;
  }
  __syncthreads();
  const int groups = Kp / 8;
  const int npix = min(kTileW, g.OW - ow0);
  bf16* out = col + (((int64_t)n * g.OH + oh) * g.OW + ow0) * Kp;
  for (int t = threadIdx.x; t < npix * groups; t += blockDim.x) {
    const int p = t / groups, k0 = (t - p * groups) * 8;
    __align__(16) bf16 v[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const int kk = k0 + i;
      bf16 e = __float2bfloat16(0.0f);
      if (kk < K) {
        const int kh = kk / RC, j = kk - kh * RC;
        e = patch[kh * rowlen + p * g.stride * g.C + j];
      }
      v[i] = e;
    }
    *reinterpret_cast<uint4*>(out + (int64_t)t * 8) = *reinterpret_cast<const uint4*>(v);
  }
}

// The same for a geometry known at compile time (the 7x7 / 2 stem over 3-channel images): every division and
// remainder of the generic kernel has a run-time divisor and costs about twenty integer instructions, which made that
// kernel instruction-bound at an eighth of the memory roofline; here they are multiplications by constants.
template <int C, int KH, int KW, int S, int TILEW>
__global__ void __launch_bounds__(256)
im2col_fixed_kernel(const bf16* __restrict__ x, bf16* __restrict__ col, Geo g, int tiles_w) {
  constexpr int SPAN = (TILEW - 1) * S + KW, ROWLEN = SPAN * C, RC = KW * C, K = KH * RC, KP = (K + 7) / 8 * 8;
  constexpr int GROUPS = KP / 8;
  __shared__ bf16 patch[KH * ROWLEN];
  int b = blockIdx.x;
  const int tw = b % tiles_w; b /= tiles_w;
  const int oh = b % g.OH;
  const int n = b / g.OH;
  const int ow0 = tw * TILEW;
  const int h0 = oh * S - g.pad, w0 = ow0 * S - g.pad;
  const bf16 zero = __float2bfloat16(0.0f);
  for (int i = threadIdx.x; i < KH * ROWLEN; i += 256) {
    const int kh = i / ROWLEN, r = i - kh * ROWLEN;
    const int ih = h0 + kh, iw = w0 + r / C;
    bf16 e = zero;
    if (ih >= 0 && ih < g.H && iw >= 0 && iw < g.W) e = x[(((int64_t)n * g.H + ih) * g.W + w0) * C + r];
    patch[i] = e;
  }
  __syncthreads();
  const int npix = min(TILEW, g.OW - ow0);
  bf16* out = col + (((int64_t)n * g.OH + oh) * g.OW + ow0) * KP;
  // Every thread keeps ONE group of eight patch-row elements for its whole life: where they sit relative to the pixel's
  // first staged element is fixed, so the offsets are computed once; threads then stride over the pixels. Consecutive
  // threads write consecutive 16-byte groups of consecutive rows.
  constexpr int SLOTS = 256 / GROUPS;                        // pixels in flight per pass
  const int grp = threadIdx.x % GROUPS, slot = threadIdx.x / GROUPS;
  if (slot < SLOTS) {
    int off[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const int kk = grp * 8 + i;
      const int kh = kk / RC, j = kk - kh * RC;
      off[i] = kk < K ? kh * ROWLEN + j : -1;
    }
    for (int p = slot; p < npix; p += SLOTS) {
      const bf16* src = patch + p * S * C;
      __align__(16) bf16 v[8];
#pragma unroll
      for (int i = 0; i < 8; i++) v[i] = off[i] >= 0 ? src[off[i]] : zero;
      *reinterpret_cast<uint4*>(out + ((int64_t)p * GROUPS + grp) * 8) = *reinterpret_cast<const uint4*>(v);
    }
  }
}

// Pixel subsample in front of a strided 1x1 convolution: y[n][oh][ow][:] = x[n][oh*s][ow*s][:], 16 bytes per thread;
// and its gradient, which puts g back at the sampled pixels and zeros everywhere else in one pass.
__global__ void subsample_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, int N, int H, int W, int C, int s,
                                 int OH, int OW) {
  const int cg = C / 8;
  const int64_t total = (int64_t)N * OH * OW * cg;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int c8 = (int)(t % cg);
    int64_t p = t / cg;
    const int ow = (int)(p % OW); p /= OW;
    const int oh = (int)(p % OH);
    const int n = (int)(p / OH);
    *reinterpret_cast<uint4*>(y + t * 8) =
        *reinterpret_cast<const uint4*>(x + ((((int64_t)n * H + (int64_t)oh * s) * W + (int64_t)ow * s) * cg + c8) * 8);
  }
}
__global__ void subsample_grad_kernel(const bf16* __restrict__ g, bf16* __restrict__ dx, int N, int H, int W, int C, int s,
                                      int OH, int OW) {
  const int cg = C / 8;
  const int64_t total = (int64_t)N * H * W * cg;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int c8 = (int)(t % cg);
    int64_t p = t / cg;
    const int w = (int)(p % W); p /= W;
    const int h = (int)(p % H);
    const int n = (int)(p / H);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (h % s == 0 && w % s == 0 && h / s < OH && w / s < OW)
      v = *reinterpret_cast<const uint4*>(g + ((((int64_t)n * OH + h / s) * OW + w / s) * cg + c8) * 8);
    *reinterpret_cast<uint4*>(dx + t * 8) = v;
  }
}

inline int grid1d(int64_t items) { int64_t b = (items + 255) / 256; return (int)(b > 148 * 16 ? 148 * 16 : (b < 1 ? 1 : b)); }

}  // namespace conv
}  // namespace gcow

using namespace gcow::conv;

extern "C" {

int gcow_im2col(const void* x, void* col, int N, int H, int W, int C, int KH, int KW, int stride, int pad, void* stream) {
  if (C % 8 || stride < 1) return -1;
  Geo g{N, H, W, C, KH, KW, stride, pad, (H + 2 * pad - KH) / stride + 1, (W + 2 * pad - KW) / stride + 1};
  const int64_t total = (int64_t)N * g.OH * g.OW * KH * KW * (C / 8);
  im2col_kernel<<<grid1d(total), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)col, g);
  return (int)cudaGetLastError();
}

// Any channel count; `Kp` (row length of col) is a multiple of 8 and at least KH*KW*C.
int gcow_im2col_anyc(const void* x, void* col, int N, int H, int W, int C, int KH, int KW, int stride, int pad, int Kp,
                     void* stream) {
  if (Kp % 8 || Kp < KH * KW * C || stride < 1) return -1;
  Geo g{N, H, W, C, KH, KW, stride, pad, (H + 2 * pad - KH) / stride + 1, (W + 2 * pad - KW) / stride + 1};
  const int tiles_w = (g.OW + kTileW - 1) / kTileW;
  const int64_t ctas = (int64_t)N * g.OH * tiles_w;
  const size_t smem = (size_t)KH * ((kTileW - 1) * stride + KW) * C * sizeof(bf16);
  if (ctas > 0x7fffffffLL || smem > 48 * 1024) return -1;
  if (C == 3 && KH == 7 && KW == 7 && stride == 2 && Kp == 152) {
    constexpr int TW = 112;                                            // a whole output row of the 224 x 224 stem per CTA
    const int tw = (g.OW + TW - 1) / TW;
    im2col_fixed_kernel<3, 7, 7, 2, TW><<<(unsigned)((int64_t)N * g.OH * tw), 256, 0, (cudaStream_t)stream>>>(
        (const bf16*)x, (bf16*)col, g, tw);
    return (int)cudaGetLastError();
  }
  if (C == 3 && KH == 3 && KW == 3 && stride == 1 && Kp == 32) {       // the 3x3 stem of the CIFAR variant
    im2col_fixed_kernel<3, 3, 3, 1, kTileW><<<(unsigned)ctas, 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)col, g, tiles_w);
    return (int)cudaGetLastError();
  }
  im2col_anyc_kernel<<<(unsigned)ctas, 256, smem, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)col, g, Kp, tiles_w);
  return (int)cudaGetLastError();
}

// y[N][OH][OW][C] = x[N][::s][::s][C] with OH = ceil(H/s), OW = ceil(W/s); C a multiple of 8. grad != 0: the gradient
// (x is then the [N][OH][OW][C] upstream gradient and y the [N][H][W][C] result, zero off the sampled pixels).
int gcow_subsample(const void* x, void* y, int N, int H, int W, int C, int s, int grad, void* stream) {
  if (C % 8 || s < 1) return -1;
  const int OH = (H + s - 1) / s, OW = (W + s - 1) / s;
  if (grad) subsample_grad_kernel<<<grid1d((int64_t)N * H * W * (C / 8)), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)x, (bf16*)y, N, H, W, C, s, OH, OW);
  else subsample_kernel<<<grid1d((int64_t)N * OH * OW * (C / 8)), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)x, (bf16*)y, N, H, W, C, s, OH, OW);
  return (int)cudaGetLastError();
}

int gcow_col2im(const void* dcol, void* dx, int N, int H, int W, int C, int KH, int KW, int stride, int pad, void* stream) {
  if (C % 8 || stride < 1) return -1;
  Geo g{N, H, W, C, KH, KW, stride, pad, (H + 2 * pad - KH) / stride + 1, (W + 2 * pad - KW) / stride + 1};
  col2im_kernel<<<grid1d((int64_t)N * H * W * (C / 8)), 256, 0, (cudaStream_t)stream>>>((const bf16*)dcol, (bf16*)dx, g);
  return (int)cudaGetLastError();
}

}  // extern "C"
