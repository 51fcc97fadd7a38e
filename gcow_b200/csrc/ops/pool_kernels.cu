// Pooling for channels-last bf16 activations (sm_100a): 3x3 stride-2 pad-1 max
// pooling and global average pooling, forward and backward. A thread owns 8
// consecutive channels of one output (or input) pixel. The max-pool forward
// stores which of the 9 taps won (one byte per element); the backward is a
// gather over the at most four windows that cover an input pixel, so it needs no
// atomics and is deterministic. Replaces nn.MaxPool2d(3, 2, 1) and
// nn.AdaptiveAvgPool2d(1) of the reference's ResNet (hw/models/resenet.py:82,89).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "pdl.cuh"

namespace gcow {
namespace pool {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void load8(const bf16* p, float (&v)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; i++) { float2 f = __bfloat1622float2(b[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
__device__ __forceinline__ void store8(bf16* p, const float (&v)[8]) {
  uint4 u;
  __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; i++) b[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

// One CTA per output row (forward) or input row (backward): the row's base addresses are computed once, and the
// position inside the row splits into (pixel, channel group) with a shift when the group count is a power of two.
// The earlier flat index with three run-time divisions per element made both kernels instruction-bound.
__device__ __forceinline__ void split_index(int i, int groups, int& pix, int& g) {
  if ((groups & (groups - 1)) == 0) { const int sh = 31 - __clz(groups); pix = i >> sh; g = i & (groups - 1); }
  else { pix = i / groups; g = i - pix * groups; }
}

__global__ void __launch_bounds__(256)
maxpool_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, uint8_t* __restrict__ idx,
                   int N, int H, int W, int C, int OH, int OW) {
  pdl_wait();
  const int groups = C / 8;
  const int oh = blockIdx.x % OH, n = blockIdx.x / OH;
  const bf16* xin = x + (int64_t)n * H * W * C;
  const int64_t orow = ((int64_t)n * OH + oh) * OW * C;
  for (int i = threadIdx.x; i < OW * groups; i += blockDim.x) {
    int ow, g;
    split_index(i, groups, ow, g);
    float best[8];
    uint8_t arg[8];
#pragma unroll
    for (int k = 0; k < 8; k++) { best[k] = -INFINITY; arg[k] = 0; }
#pragma unroll
    for (int k = 0; k < 9; k++) {
      const int ih = oh * 2 - 1 + k / 3, iw = ow * 2 - 1 + k % 3;
      if (ih < 0 || ih >= H || iw < 0 || iw >= W) continue;
      float v[8];
      load8(xin + ((int64_t)ih * W + iw) * C + g * 8, v);
#pragma unroll
      for (int e = 0; e < 8; e++) if (v[e] > best[e] || best[e] == -INFINITY) { best[e] = v[e]; arg[e] = (uint8_t)k; }
    }
    const int64_t off = orow + (int64_t)ow * C + g * 8;
    store8(y + off, best);
    *reinterpret_cast<uint2*>(idx + off) = *reinterpret_cast<const uint2*>(arg);
  }
}

__global__ void __launch_bounds__(256)
maxpool_bwd_kernel(const bf16* __restrict__ dy, const uint8_t* __restrict__ idx, bf16* __restrict__ dx,
                   int N, int H, int W, int C, int OH, int OW) {
  pdl_wait();
  const int groups = C / 8;
  const int ih = blockIdx.x % H, n = blockIdx.x / H;
  const int64_t obase = (int64_t)n * OH * OW * C;
  bf16* drow = dx + ((int64_t)n * H + ih) * W * C;
  // the one or two output rows whose windows cover this input row
  const int oh0 = ih / 2, oh1 = (ih + 1) / 2;
  for (int i = threadIdx.x; i < W * groups; i += blockDim.x) {
    int iw, g;
    split_index(i, groups, iw, g);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int oh = oh0; oh <= oh1 && oh < OH; oh++) {
      const int kh = ih - (oh * 2 - 1);
      if (kh < 0 || kh > 2) continue;
      for (int ow = iw / 2; ow <= (iw + 1) / 2 && ow < OW; ow++) {
        const int kw = iw - (ow * 2 - 1);
        if (kw < 0 || kw > 2) continue;
        const int64_t off = obase + ((int64_t)oh * OW + ow) * C + g * 8;
        float gv[8];
        load8(dy + off, gv);
        const uint2 a = *reinterpret_cast<const uint2*>(idx + off);
        const uint8_t* arg = reinterpret_cast<const uint8_t*>(&a);
        const uint8_t k = (uint8_t)(kh * 3 + kw);
#pragma unroll
        for (int e = 0; e < 8; e++) if (arg[e] == k) acc[e] += gv[e];
      }
    }
    store8(drow + (int64_t)iw * C + g * 8, acc);
  }
}

// y[n][c] = mean over HW of x[n][hw][c]; one CTA per (n, 64-channel chunk)
__global__ void __launch_bounds__(256)
avgpool_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, int HW, int C) {
  __shared__ float sm[32][65];
  const int n = blockIdx.y, c0 = blockIdx.x * 64, cg = threadIdx.x % 8, r0 = threadIdx.x / 8;   // 8 groups x 32 row lanes
  float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (c0 + cg * 8 < C)
    for (int r = r0; r < HW; r += 32) {
      float v[8];
      load8(x + ((int64_t)n * HW + r) * C + c0 + cg * 8, v);
#pragma unroll
      for (int i = 0; i < 8; i++) s[i] += v[i];
    }
#pragma unroll
  for (int i = 0; i < 8; i++) sm[r0][cg * 8 + i] = s[i];
  __syncthreads();
  if (threadIdx.x < 64 && c0 + threadIdx.x < C) {
    float t = 0;
    for (int j = 0; j < 32; j++) t += sm[j][threadIdx.x];
    y[(int64_t)n * C + c0 + threadIdx.x] = __float2bfloat16(t / HW);
  }
}

__global__ void avgpool_bwd_kernel(const bf16* __restrict__ dy, bf16* __restrict__ dx, int N, int HW, int C) {
  const int groups = C / 8;
  const int64_t total = (int64_t)N * HW * groups;
  const float inv = 1.0f / HW;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int g = (int)(t % groups);
    const int64_t p = t / groups;
    const int n = (int)(p / HW);
    float v[8];
    load8(dy + (int64_t)n * C + g * 8, v);
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] *= inv;
    store8(dx + p * C + g * 8, v);
  }
}

inline int grid1d(int64_t items) { int64_t g = (items + 255) / 256; return (int)(g > 148 * 16 ? 148 * 16 : (g < 1 ? 1 : g)); }

}  // namespace pool
}  // namespace gcow

using namespace gcow::pool;

extern "C" {

int gcow_maxpool3x3s2_fwd(const void* x, void* y, void* idx, int N, int H, int W, int C, void* stream) {
  if (C % 8) return -1;
  const int OH = (H + 2 - 3) / 2 + 1, OW = (W + 2 - 3) / 2 + 1;
  if ((int64_t)N * OH > 0x7fffffffLL) return -1;
  gcow::launch_dependent(maxpool_fwd_kernel, dim3((unsigned)(N * OH)), dim3(256), 0, (cudaStream_t)stream,
                         (const bf16*)x, (bf16*)y, (uint8_t*)idx, N, H, W, C, OH, OW);
  return (int)cudaGetLastError();
}
int gcow_maxpool3x3s2_bwd(const void* dy, const void* idx, void* dx, int N, int H, int W, int C, void* stream) {
  if (C % 8) return -1;
  const int OH = (H + 2 - 3) / 2 + 1, OW = (W + 2 - 3) / 2 + 1;
  if ((int64_t)N * H > 0x7fffffffLL) return -1;
  gcow::launch_dependent(maxpool_bwd_kernel, dim3((unsigned)(N * H)), dim3(256), 0, (cudaStream_t)stream,
                         (const bf16*)dy, (const uint8_t*)idx, (bf16*)dx, N, H, W, C, OH, OW);
  return (int)cudaGetLastError();
}
int gcow_avgpool_fwd(const void* x, void* y, int N, int HW, int C, void* stream) {
  if (C % 8) return -1;
  dim3 grid((C + 63) / 64, N);
  avgpool_fwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)y, HW, C);
  return (int)cudaGetLastError();
}
int gcow_avgpool_bwd(const void* dy, void* dx, int N, int HW, int C, void* stream) {
  if (C % 8) return -1;
  avgpool_bwd_kernel<<<grid1d((int64_t)N * HW * (C / 8)), 256, 0, (cudaStream_t)stream>>>((const bf16*)dy, (bf16*)dx, N, HW, C);
  return (int)cudaGetLastError();
}

}  // extern "C"
