// Fused BatchNorm2d (+ residual add) (+ ReLU) for channels-last bf16 activations
// (sm_100a), forward and backward, training and inference statistics.
//
// x is viewed as R = N*H*W rows of C channels. A thread owns 8 consecutive
// channels (one 16-byte access) of every (256*8/C)-th row, keeps its partial
// sums in fp32 registers and the CTA folds them per channel; per-CTA partials
// are summed in a fixed order by a second small kernel, which also derives the
// per-channel scale/shift and updates the running statistics. The normalise
// pass then applies y = x*scale + shift (+ residual), optional ReLU, in one
// read-modify-write sweep, so the add and the activation never touch memory on
// their own, and records the ReLU outcome as one bit per element (one byte per
// thread and row). Backward mirrors it: one sweep for dgamma/dbeta (reading that
// bit mask instead of the activations, and writing the masked gradient out when a
// residual branch needs it), one sweep for dx.
//
// The reference's ResNet uses nn.BatchNorm2d + ReLU + add as separate ATen /
// cuDNN operators (hw/models/resenet.py:12-22,28-40,80-89).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "pdl.cuh"
#include <stdlib.h>
#include <stdint.h>

namespace gcow {
namespace bn {



typedef __nv_bfloat16 bf16;
constexpr int kThreads = 256;

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

// Fold per-thread sums a[8], b[8] over the threads that share a channel group and
// write them to part[blockIdx.x][0][C] / [1][C].
__device__ __forceinline__ void cta_fold(const float (&a)[8], const float (&b)[8], int C, float* __restrict__ part) {
  __shared__ float sm[kThreads * 17];          // 16 values per thread, padded against bank conflicts
  const int groups = C / 8, tid = threadIdx.x;
  float* mine = sm + tid * 17;
#pragma unroll
  for (int i = 0; i < 8; i++) { mine[i] = a[i]; mine[8 + i] = b[i]; }
  __syncthreads();
  const int lanes = kThreads / groups;          // threads per channel group (>= 1)
  for (int idx = tid; idx < groups * 16; idx += kThreads) {
    const int g = idx / 16, k = idx % 16;
    float s = 0;
    for (int j = 0; j < lanes; j++) s += sm[(j * groups + g) * 17 + k];
    const int c = g * 8 + (k & 7);
    part[(size_t)blockIdx.x * 2 * C + (k < 8 ? 0 : C) + c] = s;
  }
}

// ---- forward statistics: partial sum(x), sum(x^2)
__global__ void __launch_bounds__(kThreads)
stats_kernel(const bf16* __restrict__ x, float* __restrict__ part, int64_t R, int C) {
  pdl_trigger();
  pdl_wait();       // launched under the tail of the kernel that writes x
  const int groups = C / 8, g = threadIdx.x % groups, r0 = threadIdx.x / groups, rstep = kThreads / groups;
  float s[8] = {0, 0, 0, 0, 0, 0, 0, 0}, q[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll 4
  for (int64_t r = (int64_t)blockIdx.x * rstep + r0; r < R; r += (int64_t)gridDim.x * rstep) {
    float v[8];
    load8(x + r * C + g * 8, v);
#pragma unroll
    for (int i = 0; i < 8; i++) { s[i] += v[i]; q[i] += v[i] * v[i]; }
  }
  cta_fold(s, q, C, part);
}

// Sum the per-CTA partials of 32 channels with a 32 x 8 thread block: thread (cx, py)
// adds partials py, py+8, ... of channel c (coalesced across cx), then the 8 rows are
// added in a fixed order, so the result does not depend on scheduling.
constexpr int kFinX = 32, kFinY = 32;
__device__ __forceinline__ void fold_partials(const float* __restrict__ part, int parts, int C, int c, double& s_out,
                                              double& q_out) {
  __shared__ double sm_s[kFinY][kFinX + 1], sm_q[kFinY][kFinX + 1];
  const int cx = threadIdx.x, py = threadIdx.y;
  double s = 0, q = 0;   // the variance is a difference of two large sums: fold in double
  if (c < C)
    for (int p = py; p < parts; p += kFinY) { s += part[(size_t)p * 2 * C + c]; q += part[(size_t)p * 2 * C + C + c]; }
  sm_s[py][cx] = s; sm_q[py][cx] = q;
  __syncthreads();
  s = 0; q = 0;
#pragma unroll
  for (int j = 0; j < kFinY; j++) { s += sm_s[j][cx]; q += sm_q[j][cx]; }
  s_out = s; q_out = q;
}

// ---- finalize forward: mean/rstd, scale/shift, running statistics
__global__ void __launch_bounds__(kFinX * kFinY)
finalize_fwd_kernel(const float* __restrict__ part, int parts, int C, int64_t R, float eps, float momentum,
                    const float* __restrict__ gamma, const float* __restrict__ beta,
                    float* __restrict__ mean, float* __restrict__ rstd, float* __restrict__ scale,
                    float* __restrict__ shift, float* __restrict__ run_mean, float* __restrict__ run_var) {
  pdl_wait();
  pdl_trigger();
  const int c = blockIdx.x * kFinX + threadIdx.x;
  double s, q;
  fold_partials(part, parts, C, c, s, q);
  if (c >= C || threadIdx.y != 0) return;
  const double mu = s / (double)R;
  double var = q / (double)R - mu * mu;
  if (var < 0) var = 0;
  const float rs = rsqrtf((float)var + eps);
  mean[c] = (float)mu; rstd[c] = rs;
  const float sc = gamma[c] * rs;
  scale[c] = sc; shift[c] = beta[c] - (float)mu * sc;
  if (run_mean) {
    const double unbiased = R > 1 ? var * (double)R / (double)(R - 1) : var;
    run_mean[c] = (1.0f - momentum) * run_mean[c] + momentum * (float)mu;
    run_var[c] = (1.0f - momentum) * run_var[c] + momentum * (float)unbiased;
  }
}

// scale/shift from given (running) statistics, for inference
__global__ void affine_from_stats_kernel(const float* __restrict__ gamma, const float* __restrict__ beta,
                                         const float* __restrict__ mean_in, const float* __restrict__ var_in, float eps,
                                         int C, float* __restrict__ scale, float* __restrict__ shift) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const float sc = gamma[c] * rsqrtf(var_in[c] + eps);
  scale[c] = sc; shift[c] = beta[c] - mean_in[c] * sc;
}

// ---- normalise: y = x*scale + shift (+ residual) (ReLU)
__global__ void __launch_bounds__(kThreads)
apply_kernel(const bf16* __restrict__ x, const bf16* __restrict__ residual, bf16* __restrict__ y,
             uint8_t* __restrict__ mask, const float* __restrict__ scale, const float* __restrict__ shift, int64_t R,
             int C, int relu) {
  pdl_wait();
  pdl_trigger();    // the consumer of y may set itself up meanwhile
  const int groups = C / 8, g = threadIdx.x % groups, r0 = threadIdx.x / groups, rstep = kThreads / groups;
  float sc[8], sh[8];
#pragma unroll
  for (int i = 0; i < 8; i++) { sc[i] = scale[g * 8 + i]; sh[i] = shift[g * 8 + i]; }
#pragma unroll 4
  for (int64_t r = (int64_t)blockIdx.x * rstep + r0; r < R; r += (int64_t)gridDim.x * rstep) {
    const int64_t off = r * C + g * 8;
    float v[8];
    load8(x + off, v);
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = v[i] * sc[i] + sh[i];
    if (residual) {
      float w[8];
      load8(residual + off, w);
#pragma unroll
      for (int i = 0; i < 8; i++) v[i] += w[i];
    }
    if (relu) {
      uint32_t bits = 0;
#pragma unroll
      for (int i = 0; i < 8; i++) { bits |= (v[i] > 0.0f ? 1u : 0u) << i; v[i] = fmaxf(v[i], 0.0f); }
      if (mask) mask[r * groups + g] = (uint8_t)bits;      // bit i: channel g*8+i passed the ReLU
    }
    store8(y + off, v);
  }
}

// ---- backward sweep 1: partial sum(g), sum(g*xhat); g = dy (+ dy2) masked by (y > 0) when relu.
// dy2 (nullable) is a second gradient of the same output (the output feeds two consumers): adding it here saves
// the separate addition kernel and its three passes over the tensor.
// When gmask_out is given, the masked gradient is written there (the residual branch's gradient).
__global__ void __launch_bounds__(kThreads)
bwd_reduce_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ dy2, const uint8_t* __restrict__ mask,
                  const bf16* __restrict__ x,
                  const float* __restrict__ mean, const float* __restrict__ rstd, bf16* __restrict__ gmask_out,
                  float* __restrict__ part, int64_t R, int C, int relu) {
  pdl_trigger();
  pdl_wait();
  const int groups = C / 8, g = threadIdx.x % groups, r0 = threadIdx.x / groups, rstep = kThreads / groups;
  float mu[8], rs[8], s[8] = {0, 0, 0, 0, 0, 0, 0, 0}, q[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
  for (int i = 0; i < 8; i++) { mu[i] = mean[g * 8 + i]; rs[i] = rstd[g * 8 + i]; }
#pragma unroll 4
  for (int64_t r = (int64_t)blockIdx.x * rstep + r0; r < R; r += (int64_t)gridDim.x * rstep) {
    const int64_t off = r * C + g * 8;
    float gv[8], xv[8];
    load8(dy + off, gv);
    load8(x + off, xv);
    if (dy2) {
      float w[8];
      load8(dy2 + off, w);
#pragma unroll
      for (int i = 0; i < 8; i++) gv[i] += w[i];
    }
    if (relu) {
      const uint32_t bits = mask[r * groups + g];
#pragma unroll
      for (int i = 0; i < 8; i++) gv[i] = (bits >> i) & 1u ? gv[i] : 0.0f;
    }
    if (gmask_out) store8(gmask_out + off, gv);
#pragma unroll
    for (int i = 0; i < 8; i++) { s[i] += gv[i]; q[i] += gv[i] * (xv[i] - mu[i]) * rs[i]; }
  }
  cta_fold(s, q, C, part);
}

// ---- finalize backward: dbeta = sum g, dgamma = sum g*xhat (fixed order)
__global__ void __launch_bounds__(kFinX * kFinY)
finalize_bwd_kernel(const float* __restrict__ part, int parts, int C, float* __restrict__ dgamma,
                    float* __restrict__ dbeta) {
  pdl_wait();
  pdl_trigger();
  const int c = blockIdx.x * kFinX + threadIdx.x;
  double s, q;
  fold_partials(part, parts, C, c, s, q);
  if (c >= C || threadIdx.y != 0) return;
  dbeta[c] = (float)s; dgamma[c] = (float)q;
}

// ---- backward sweep 2: dx = gamma*rstd * (g - dbeta/R - xhat*dgamma/R)
__global__ void __launch_bounds__(kThreads)
bwd_dx_kernel(const bf16* __restrict__ dy, const uint8_t* __restrict__ mask, const bf16* __restrict__ x,
              const float* __restrict__ gamma, const float* __restrict__ mean, const float* __restrict__ rstd,
              const float* __restrict__ dgamma, const float* __restrict__ dbeta, bf16* __restrict__ dx, int64_t R, int C,
              int relu) {
  pdl_wait();
  pdl_trigger();
  const int groups = C / 8, g = threadIdx.x % groups, r0 = threadIdx.x / groups, rstep = kThreads / groups;
  float mu[8], rs[8], k0[8], k1[8], k2[8];
  const float invR = 1.0f / (float)R;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int c = g * 8 + i;
    mu[i] = mean[c]; rs[i] = rstd[c];
    k0[i] = gamma[c] * rs[i];
    k1[i] = dbeta[c] * invR;
    k2[i] = dgamma[c] * invR;
  }
#pragma unroll 4
  for (int64_t r = (int64_t)blockIdx.x * rstep + r0; r < R; r += (int64_t)gridDim.x * rstep) {
    const int64_t off = r * C + g * 8;
    float gv[8], xv[8];
    load8(dy + off, gv);
    load8(x + off, xv);
    if (relu) {
      const uint32_t bits = mask[r * groups + g];
#pragma unroll
      for (int i = 0; i < 8; i++) gv[i] = (bits >> i) & 1u ? gv[i] : 0.0f;
    }
#pragma unroll
    for (int i = 0; i < 8; i++) gv[i] = k0[i] * (gv[i] - k1[i] - (xv[i] - mu[i]) * rs[i] * k2[i]);
    store8(dx + off, gv);
  }
}

inline int grid_for(int64_t R, int C) {
  const int rstep = kThreads / (C / 8);
  int64_t g = (R + rstep - 1) / rstep;
  if (g > 148 * 3) g = 148 * 3;
  return (int)(g < 1 ? 1 : g);
}
inline bool shape_ok(int C) { return C % 8 == 0 && C >= 8 && C <= 2048 && kThreads % (C / 8) == 0; }

}  // namespace bn
}  // namespace gcow

using namespace gcow::bn;

extern "C" {

int gcow_bn_supported(int C) { return shape_ok(C) ? 1 : 0; }
int gcow_bn_parts(int64_t R, int C) { return shape_ok(C) ? grid_for(R, C) : 0; }

// Training forward. part: gcow_bn_parts * 2 * C floats of scratch. stats: 4*C floats out
// (mean, rstd, scale, shift). run_mean/run_var may be null. mask: R*C/8 bytes out (ReLU
// outcome, one bit per element), required when relu != 0 and a backward pass will follow.
int gcow_bn_fwd_train(const void* x, const void* residual, void* y, void* mask, const float* gamma, const float* beta,
                      float* run_mean, float* run_var, float* stats, float* part, int64_t R, int C, float eps,
                      float momentum, int relu, void* stream) {
  if (!shape_ok(C) || R <= 0) return -1;
  cudaStream_t s = (cudaStream_t)stream;
  const int g = grid_for(R, C);
  float *mean = stats, *rstd = stats + C, *scale = stats + 2 * C, *shift = stats + 3 * C;
  gcow::launch_dependent(stats_kernel, dim3(g), dim3(kThreads), 0, s, (const bf16*)x, part, R, C);
  gcow::launch_dependent(finalize_fwd_kernel, dim3((C + kFinX - 1) / kFinX), dim3(kFinX, kFinY), 0, s, part, g, C, R, eps, momentum, gamma,
                   beta, mean, rstd, scale, shift, run_mean, run_var);
  gcow::launch_dependent(apply_kernel, dim3(g), dim3(kThreads), 0, s, (const bf16*)x, (const bf16*)residual, (bf16*)y, (uint8_t*)mask,
                   (const float*)scale, (const float*)shift, R, C, relu);
  return (int)cudaGetLastError();
}

// Inference forward with given statistics; scratch: 2*C floats.
int gcow_bn_fwd_eval(const void* x, const void* residual, void* y, const float* gamma, const float* beta,
                     const float* run_mean, const float* run_var, float* scratch, int64_t R, int C, float eps, int relu,
                     void* stream) {
  if (!shape_ok(C) || R <= 0) return -1;
  cudaStream_t s = (cudaStream_t)stream;
  affine_from_stats_kernel<<<(C + 127) / 128, 128, 0, s>>>(gamma, beta, run_mean, run_var, eps, C, scratch, scratch + C);
  apply_kernel<<<grid_for(R, C), kThreads, 0, s>>>((const bf16*)x, (const bf16*)residual, (bf16*)y, nullptr, scratch, scratch + C, R, C, relu);
  return (int)cudaGetLastError();
}

// Backward. stats and mask as written by the forward. dres (nullable) receives the gradient
// of the residual input (the ReLU-masked dy). dgb: 2*C floats out (dgamma, dbeta).
// dy2 (nullable): a second gradient of the same output, added to dy on the fly; it needs dres (any buffer of the
// tensor's size) to carry the masked sum to the second sweep.
// dgamma and dbeta (C floats each) may lie anywhere, e.g. in the two parameters' gradient tensors.
int gcow_bn_bwd3(const void* dy, const void* dy2, const void* mask, const void* x, const float* gamma, const float* stats,
                 void* dx, void* dres, float* dgamma, float* dbeta, float* part, int64_t R, int C, int relu, void* stream) {
  if (!shape_ok(C) || R <= 0 || (dy2 && !dres)) return -1;
  cudaStream_t s = (cudaStream_t)stream;
  const int g = grid_for(R, C);
  const float *mean = stats, *rstd = stats + C;
  gcow::launch_dependent(bwd_reduce_kernel, dim3(g), dim3(kThreads), 0, s, (const bf16*)dy, (const bf16*)dy2, (const uint8_t*)mask,
                         (const bf16*)x, mean, rstd, (bf16*)dres, part, R, C, relu);
  gcow::launch_dependent(finalize_bwd_kernel, dim3((C + kFinX - 1) / kFinX), dim3(kFinX, kFinY), 0, s, (const float*)part, g, C, dgamma, dbeta);
  // the second sweep applies the mask again, or reads the masked gradient if it was written
  gcow::launch_dependent(bwd_dx_kernel, dim3(g), dim3(kThreads), 0, s, (const bf16*)(dres ? dres : dy), (const uint8_t*)mask, (const bf16*)x,
                   gamma, mean, rstd, (const float*)dgamma, (const float*)dbeta, (bf16*)dx, R, C, dres ? 0 : relu);
  return (int)cudaGetLastError();
}

int gcow_bn_bwd2(const void* dy, const void* dy2, const void* mask, const void* x, const float* gamma, const float* stats,
                 void* dx, void* dres, float* dgb, float* part, int64_t R, int C, int relu, void* stream) {
  return gcow_bn_bwd3(dy, dy2, mask, x, gamma, stats, dx, dres, dgb, dgb + C, part, R, C, relu, stream);
}

int gcow_bn_bwd(const void* dy, const void* mask, const void* x, const float* gamma, const float* stats, void* dx,
                void* dres, float* dgb, float* part, int64_t R, int C, int relu, void* stream) {
  return gcow_bn_bwd2(dy, nullptr, mask, x, gamma, stats, dx, dres, dgb, part, R, C, relu, stream);
}

}  // extern "C"
