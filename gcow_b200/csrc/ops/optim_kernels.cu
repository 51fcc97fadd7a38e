// Multi-tensor optimizer steps (sm_100a): one launch updates every parameter.
//
// The host builds, once, a device table of chunks {param, grad, state..., n};
// each CTA walks chunks grid-stride and applies the update with 128-bit loads.
// With DDP's gradient-as-bucket-view the grad pointers are the all-reduced
// bucket memory itself, so the step consumes the decoded gradients in place.
//
// SGD follows torch.optim.SGD as the reference configures it (lr 0.1, momentum
// 0.9, weight decay 1e-4: hw/models/train_imagenet.py:251-253,
// hw/models/train_resnet_cifar10.py:156-158):
//   g += wd * p;  buf = first ? g : mu * buf + (1 - damp) * g;
//   g  = nesterov ? g + mu * buf : buf;  p -= lr * g
// AdamW is the decoupled-weight-decay Adam used for BERT pre-training.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gcow {

struct OptChunk {
  float* p;
  const float* g;
  float* s0;   // momentum buffer / exp_avg
  float* s1;   // exp_avg_sq (AdamW) or nullptr
  uint32_t n;
  uint32_t pad;
  __nv_bfloat16* shadow;   // bf16 copy of the updated parameter in the same element order, or nullptr: what the
                           // GEMM and convolution kernels read, so no cast kernel runs in the next forward pass
};

constexpr int kOptThreads = 256;

// four consecutive bf16 values (the chunk starts 16-byte aligned in fp32, so 8-byte aligned here)
__device__ __forceinline__ void store_shadow4(__nv_bfloat16* dst, const float4& p) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(p.x, p.y), hi = __floats2bfloat162_rn(p.z, p.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&lo);
  u.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = u;
}

template <class F>
__device__ __forceinline__ void for_each4(const OptChunk& c, F f) {
  const bool al = ((((uintptr_t)c.p) | ((uintptr_t)c.g) | ((uintptr_t)c.s0) | ((uintptr_t)c.s1)) & 15) == 0;
  const uint32_t n4 = al ? c.n / 4 : 0;
  for (uint32_t i = threadIdx.x; i < n4; i += blockDim.x) f(i * 4, 4);
  for (uint32_t i = n4 * 4 + threadIdx.x; i < c.n; i += blockDim.x) f(i, 1);
}

__global__ void __launch_bounds__(kOptThreads)
sgd_kernel(const OptChunk* __restrict__ chunks, uint32_t nchunks, float lr, float mu, float wd, float damp,
           int nesterov, int first, float grad_scale) {
  for (uint32_t ci = blockIdx.x; ci < nchunks; ci += gridDim.x) {
    const OptChunk c = chunks[ci];
    for_each4(c, [&](uint32_t i, int w) {
      if (w == 4) {
        float4 p = *reinterpret_cast<float4*>(c.p + i);
        float4 g = *reinterpret_cast<const float4*>(c.g + i);
        float4 b = first || !c.s0 ? make_float4(0, 0, 0, 0) : *reinterpret_cast<float4*>(c.s0 + i);
        float* pp = &p.x; float* gg = &g.x; float* bb = &b.x;
#pragma unroll
        for (int k = 0; k < 4; k++) {
          float gk = gg[k] * grad_scale + wd * pp[k];
          if (c.s0) {
            bb[k] = first ? gk : mu * bb[k] + (1.0f - damp) * gk;
            gk = nesterov ? gk + mu * bb[k] : bb[k];
          }
          pp[k] -= lr * gk;
        }
        *reinterpret_cast<float4*>(c.p + i) = p;
        if (c.s0) *reinterpret_cast<float4*>(c.s0 + i) = b;
        if (c.shadow) store_shadow4(c.shadow + i, p);
      } else {
        float gk = c.g[i] * grad_scale + wd * c.p[i];
        if (c.s0) {
          float b = first ? gk : mu * c.s0[i] + (1.0f - damp) * gk;
          c.s0[i] = b;
          gk = nesterov ? gk + mu * b : b;
        }
        c.p[i] -= lr * gk;
        if (c.shadow) c.shadow[i] = __float2bfloat16(c.p[i]);
      }
    });
  }
}

__global__ void __launch_bounds__(kOptThreads)
adamw_kernel(const OptChunk* __restrict__ chunks, uint32_t nchunks, float lr, float b1, float b2, float eps,
             float wd, float bc1, float bc2_sqrt, float grad_scale) {
  // bc1 = 1 - b1^t ; bc2_sqrt = sqrt(1 - b2^t)
  const float step = lr / bc1;
  for (uint32_t ci = blockIdx.x; ci < nchunks; ci += gridDim.x) {
    const OptChunk c = chunks[ci];
    auto upd = [&](float& p, float g, float& m, float& v) {
      g *= grad_scale;
      p *= 1.0f - lr * wd;
      m = b1 * m + (1.0f - b1) * g;
      v = b2 * v + (1.0f - b2) * g * g;
      const float denom = sqrtf(v) / bc2_sqrt + eps;
      p -= step * (m / denom);
    };
    for_each4(c, [&](uint32_t i, int w) {
      if (w == 4) {
        float4 p = *reinterpret_cast<float4*>(c.p + i), m = *reinterpret_cast<float4*>(c.s0 + i),
               v = *reinterpret_cast<float4*>(c.s1 + i);
        const float4 g = *reinterpret_cast<const float4*>(c.g + i);
        upd(p.x, g.x, m.x, v.x); upd(p.y, g.y, m.y, v.y); upd(p.z, g.z, m.z, v.z); upd(p.w, g.w, m.w, v.w);
        *reinterpret_cast<float4*>(c.p + i) = p;
        *reinterpret_cast<float4*>(c.s0 + i) = m;
        *reinterpret_cast<float4*>(c.s1 + i) = v;
        if (c.shadow) store_shadow4(c.shadow + i, p);
      } else {
        upd(c.p[i], c.g[i], c.s0[i], c.s1[i]);
        if (c.shadow) c.shadow[i] = __float2bfloat16(c.p[i]);
      }
    });
  }
}

}  // namespace gcow

using namespace gcow;

extern "C" {

uint32_t gcow_opt_chunk_bytes() { return (uint32_t)sizeof(OptChunk); }

int gcow_sgd_step(const void* chunks, uint32_t nchunks, float lr, float mu, float wd, float damp, int nesterov,
                  int first, float grad_scale, void* stream) {
  if (!nchunks) return 0;
  int grid = nchunks < 148u * 8 ? (int)nchunks : 148 * 8;
  sgd_kernel<<<grid, kOptThreads, 0, (cudaStream_t)stream>>>((const OptChunk*)chunks, nchunks, lr, mu, wd, damp,
                                                             nesterov, first, grad_scale);
  return (int)cudaGetLastError();
}

int gcow_adamw_step(const void* chunks, uint32_t nchunks, float lr, float b1, float b2, float eps, float wd,
                    float bc1, float bc2_sqrt, float grad_scale, void* stream) {
  if (!nchunks) return 0;
  int grid = nchunks < 148u * 8 ? (int)nchunks : 148 * 8;
  adamw_kernel<<<grid, kOptThreads, 0, (cudaStream_t)stream>>>((const OptChunk*)chunks, nchunks, lr, b1, b2, eps,
                                                               wd, bc1, bc2_sqrt, grad_scale);
  return (int)cudaGetLastError();
}

}  // extern "C"
