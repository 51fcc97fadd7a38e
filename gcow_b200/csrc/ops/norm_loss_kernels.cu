// Memory-bound training kernels (sm_100a): LayerNorm forward/backward, exact-erf
// GELU forward/backward, fused softmax cross-entropy (loss + in-place gradient),
// column sums (bias gradients) and the uint8 -> bf16 image normalisation.
// All of them stream their operands once with 16-byte accesses and keep row
// statistics in fp32; reductions that cross CTAs are two-stage with a fixed
// order, so results are run-to-run deterministic.
//
// The reference's models get these from ATen/cuDNN through PyTorch
// (hw/models/resenet.py:12-22,80-89; cross-entropy at hw/models/train_imagenet.py:249).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "pdl.cuh"
#include <stdint.h>

namespace gcow {
namespace nl {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int d = 16; d; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int d = 16; d; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
  return v;
}
__device__ __forceinline__ void load8(const bf16* p, float (&v)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; i++) { float2 f = __bfloat1622float2(b[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
__device__ __forceinline__ void unpack8(const uint4& u, float (&v)[8]) {
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

// ------------------------------------------------------------------ LayerNorm
// One warp per row; H a multiple of 8. The row (a few KB) is re-read from L1.
__global__ void __launch_bounds__(128)
layernorm_fwd_kernel(const bf16* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                     bf16* __restrict__ y, float* __restrict__ mean, float* __restrict__ rstd, int rows, int H,
                     float eps) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  for (int r = blockIdx.x * 4 + (threadIdx.x >> 5); r < rows; r += gridDim.x * 4) {
    const bf16* xr = x + (size_t)r * H;
    float s = 0;
    for (int c = lane * 8; c < H; c += 256) { float v[8]; load8(xr + c, v);
#pragma unroll
      for (int i = 0; i < 8; i++) s += v[i]; }
    const float mu = warp_sum(s) / H;
    float q = 0;
    for (int c = lane * 8; c < H; c += 256) { float v[8]; load8(xr + c, v);
#pragma unroll
      for (int i = 0; i < 8; i++) { float d = v[i] - mu; q += d * d; } }
    const float rs = rsqrtf(warp_sum(q) / H + eps);
    if (lane == 0) { mean[r] = mu; rstd[r] = rs; }
    bf16* yr = y + (size_t)r * H;
    for (int c = lane * 8; c < H; c += 256) {
      float v[8];
      load8(xr + c, v);
      const float4 g0 = *reinterpret_cast<const float4*>(gamma + c), g1 = *reinterpret_cast<const float4*>(gamma + c + 4);
      const float4 b0 = *reinterpret_cast<const float4*>(beta + c), b1 = *reinterpret_cast<const float4*>(beta + c + 4);
      const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
      const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; i++) v[i] = (v[i] - mu) * rs * g[i] + b[i];
      store8(yr + c, v);
    }
  }
}

// dx per row; per-CTA partial sums of dgamma/dbeta go to part[blockIdx.x][2][H].
// A lane always works on the same columns (lane*8 + 256*k), so its dgamma/dbeta
// contributions stay in registers across all rows of the warp (CH = H/256 chunks of
// 8 columns, CH <= 4) and touch shared memory once at the end; wider rows (CH == 0)
// accumulate in shared memory.
template <int CH>
__global__ void __launch_bounds__(128, CH > 0 ? 3 : 1)
layernorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const float* __restrict__ gamma,
                     const float* __restrict__ mean, const float* __restrict__ rstd, bf16* __restrict__ dx,
                     float* __restrict__ part, int rows, int H) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float sm[];          // [4 warps][2][H]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* dg = sm + (size_t)warp * 2 * H;
  float* db = dg + H;
  constexpr int NR = CH > 0 ? CH : 1;
  float rg[NR][8], rb[NR][8];
  if (CH > 0) {
    // gamma lives in shared memory (one copy per CTA): 32 registers less per thread buy a third CTA per SM
    for (int c = threadIdx.x; c < 256 * NR; c += blockDim.x) sm[c] = c < H ? gamma[c] : 0.0f;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < NR; k++)
#pragma unroll
      for (int i = 0; i < 8; i++) { rg[k][i] = 0; rb[k][i] = 0; }
  } else {
    for (int c = lane; c < H; c += 32) { dg[c] = 0; db[c] = 0; }
    __syncwarp();
  }
  if (CH > 0) {
    // One row per warp and turn; the next row's 2 x CH 16-byte loads are issued before this row's arithmetic, so a
    // warp always has a row in flight (without that the kernel ran at a quarter of the memory roofline: load, reduce
    // across the warp, store, and only then the next load).
    const int stride = gridDim.x * 4;
    int r = blockIdx.x * 4 + warp;
    uint4 nx[NR], ng[NR];
    float nmu = 0.0f, nrs = 0.0f;
    auto fetch = [&](int row) {
      const bf16* xr = x + (size_t)row * H;
      const bf16* gr = dy + (size_t)row * H;
#pragma unroll
      for (int k = 0; k < NR; k++) {
        const int c = lane * 8 + 256 * k;
        if (c < H) {
          nx[k] = *reinterpret_cast<const uint4*>(xr + c);
          ng[k] = *reinterpret_cast<const uint4*>(gr + c);
        }
      }
      nmu = mean[row]; nrs = rstd[row];
    };
    if (r < rows) fetch(r);
    for (; r < rows; r += stride) {
      uint4 cx[NR], cgv[NR];
#pragma unroll
      for (int k = 0; k < NR; k++) { cx[k] = nx[k]; cgv[k] = ng[k]; }
      const float mu = nmu, rs = nrs;
      if (r + stride < rows) fetch(r + stride);
      float s1 = 0, s2 = 0;
#pragma unroll
      for (int k = 0; k < NR; k++) {
        const int c = lane * 8 + 256 * k;
        if (c < H) {
          float xv[8], gv[8], gam[8];
          unpack8(cx[k], xv); unpack8(cgv[k], gv);
          *reinterpret_cast<float4*>(gam) = *reinterpret_cast<const float4*>(sm + c);
          *reinterpret_cast<float4*>(gam + 4) = *reinterpret_cast<const float4*>(sm + c + 4);
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const float xh = (xv[i] - mu) * rs, gg = gv[i] * gam[i];
            s1 += gg; s2 += gg * xh;
            rg[k][i] += gv[i] * xh;
            rb[k][i] += gv[i];
          }
        }
      }
      s1 = warp_sum(s1) / H; s2 = warp_sum(s2) / H;
      bf16* dr = dx + (size_t)r * H;
      // the row is still in registers as packed bf16: unpacking it again is cheaper than keeping 2 x 8 x CH floats
#pragma unroll
      for (int k = 0; k < NR; k++) {
        const int c = lane * 8 + 256 * k;
        if (c < H) {
          float xv[8], gv[8], gam[8], o[8];
          unpack8(cx[k], xv); unpack8(cgv[k], gv);
          *reinterpret_cast<float4*>(gam) = *reinterpret_cast<const float4*>(sm + c);
          *reinterpret_cast<float4*>(gam + 4) = *reinterpret_cast<const float4*>(sm + c + 4);
#pragma unroll
          for (int i = 0; i < 8; i++) o[i] = rs * (gv[i] * gam[i] - s1 - (xv[i] - mu) * rs * s2);
          store8(dr + c, o);
        }
      }
    }
  }
  for (int r = blockIdx.x * 4 + warp; CH == 0 && r < rows; r += gridDim.x * 4) {
    const bf16* xr = x + (size_t)r * H;
    const bf16* gr = dy + (size_t)r * H;
    const float mu = mean[r], rs = rstd[r];
    float s1 = 0, s2 = 0;
    for (int c = lane * 8; c < H; c += 256) {
      float xv[8], gv[8];
      load8(xr + c, xv); load8(gr + c, gv);
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const float xh = (xv[i] - mu) * rs, gg = gv[i] * gamma[c + i];
        s1 += gg; s2 += gg * xh;
        dg[c + i] += gv[i] * xh;
        db[c + i] += gv[i];
      }
    }
    s1 = warp_sum(s1) / H; s2 = warp_sum(s2) / H;
    bf16* dr = dx + (size_t)r * H;
    for (int c = lane * 8; c < H; c += 256) {
      float xv[8], gv[8], o[8];
      load8(xr + c, xv); load8(gr + c, gv);
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const float xh = (xv[i] - mu) * rs;
        o[i] = rs * (gv[i] * gamma[c + i] - s1 - xh * s2);
      }
      store8(dr + c, o);
    }
  }
  if (CH > 0) {
    __syncthreads();      // every warp is done with the gamma copy that these sums overwrite
#pragma unroll
    for (int k = 0; k < NR; k++)
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const int c = lane * 8 + 256 * k + i;
        if (c < H) { dg[c] = rg[k][i]; db[c] = rb[k][i]; }
      }
  }
  __syncthreads();
  float* out = part + (size_t)blockIdx.x * 2 * H;
  for (int c = threadIdx.x; c < 2 * H; c += blockDim.x)
    out[c] = sm[c] + sm[2 * H + c] + sm[4 * H + c] + sm[6 * H + c];
}

// out[c] = sum_p part[p][c]  (fixed order)
__global__ void reduce_partials_kernel(const float* __restrict__ part, float* __restrict__ out, int parts, int n) {
  pdl_wait();       // launched as a dependent of the kernel that writes `part`
  pdl_trigger();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= n) return;
  float s = 0;
  for (int p = 0; p < parts; p++) s += part[(size_t)p * n + c];
  out[c] = s;
}

// The same for many partials of a short vector (LayerNorm's 444 x 2H): 32 x 32 threads per 32 columns, thread (cx, py)
// adds partials py, py + 32, ..., then the 32 rows are added in a fixed order. One thread per column walking all the
// partials serially took longer than the LayerNorm backward sweep it follows.
__global__ void __launch_bounds__(1024)
reduce_partials_tall_kernel(const float* __restrict__ part, float* __restrict__ out, int parts, int n) {
  pdl_wait();
  pdl_trigger();
  __shared__ float sm[32][33];
  const int cx = threadIdx.x, py = threadIdx.y;
  const int c = blockIdx.x * 32 + cx;
  float s = 0;
  if (c < n)
    for (int p = py; p < parts; p += 32) s += part[(size_t)p * n + c];
  sm[py][cx] = s;
  __syncthreads();
  if (py == 0 && c < n) {
    float t = 0;
#pragma unroll
    for (int j = 0; j < 32; j++) t += sm[j][cx];
    out[c] = t;
  }
}

// ----------------------------------------------------------------------- GELU
__device__ __forceinline__ float gelu_f(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f)); }
__device__ __forceinline__ float gelu_grad_f(float x) {
  const float cdf = 0.5f * (1.0f + erff(x * 0.70710678118654752f));
  return cdf + x * 0.3989422804014327f * __expf(-0.5f * x * x);
}
__global__ void gelu_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, size_t n8) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    float v[8];
    load8(x + i * 8, v);
#pragma unroll
    for (int k = 0; k < 8; k++) v[k] = gelu_f(v[k]);
    store8(y + i * 8, v);
  }
}
__global__ void gelu_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, bf16* __restrict__ dx, size_t n8) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    float v[8], g[8];
    load8(x + i * 8, v); load8(dy + i * 8, g);
#pragma unroll
    for (int k = 0; k < 8; k++) g[k] *= gelu_grad_f(v[k]);
    store8(dx + i * 8, g);
  }
}

// ------------------------------------------------------- softmax cross-entropy
// One CTA per row of `logits` [rows, ld] (V valid columns, bf16). Writes the
// row loss (0 for ignored rows) and overwrites the row with
// (softmax - onehot) * scale, scale = 1 / max(1, *valid_count).
__global__ void __launch_bounds__(256)
softmax_xent_kernel(bf16* __restrict__ logits, const int64_t* __restrict__ target, float* __restrict__ row_loss,
                    const float* __restrict__ valid_count, int V, int ld, int ignore_index) {
  __shared__ float red[16];
  const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  bf16* row = logits + (size_t)r * ld;
  const int64_t t = target[r];
  const int V8 = V & ~7;
  if (t == ignore_index) {
    for (int c = tid * 8; c < ld; c += 256 * 8) *reinterpret_cast<uint4*>(row + c) = make_uint4(0, 0, 0, 0);
    if (tid == 0) row_loss[r] = 0;
    return;
  }
  float mx = -INFINITY;
  for (int c = tid * 8; c < V8; c += 256 * 8) { float v[8]; load8(row + c, v);
#pragma unroll
    for (int i = 0; i < 8; i++) mx = fmaxf(mx, v[i]); }
  for (int c = V8 + tid; c < V; c += 256) mx = fmaxf(mx, __bfloat162float(row[c]));
  mx = warp_max(mx);
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = red[0];
#pragma unroll
  for (int i = 1; i < 8; i++) mx = fmaxf(mx, red[i]);
  float s = 0;
  for (int c = tid * 8; c < V8; c += 256 * 8) { float v[8]; load8(row + c, v);
#pragma unroll
    for (int i = 0; i < 8; i++) s += __expf(v[i] - mx); }
  for (int c = V8 + tid; c < V; c += 256) s += __expf(__bfloat162float(row[c]) - mx);
  s = warp_sum(s);
  if (lane == 0) red[8 + warp] = s;
  __syncthreads();
  s = 0;
#pragma unroll
  for (int i = 0; i < 8; i++) s += red[8 + i];
  const float lse = mx + __logf(s);
  const float scale = 1.0f / fmaxf(1.0f, *valid_count);
  const float inv = scale / s;
  if (tid == 0) row_loss[r] = (lse - __bfloat162float(row[t])) * scale;
  __syncthreads();   // row[t] read before it is overwritten
  for (int c = tid * 8; c < V8; c += 256 * 8) {
    float v[8];
    load8(row + c, v);
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = __expf(v[i] - mx) * inv - ((int64_t)(c + i) == t ? scale : 0.0f);
    store8(row + c, v);
  }
  for (int c = V8 + tid; c < ld; c += 256)
    row[c] = c < V ? __float2bfloat16(__expf(__bfloat162float(row[c]) - mx) * inv - ((int64_t)c == t ? scale : 0.0f))
                   : __float2bfloat16(0.0f);
}

// -------------------------------------------------------------------- softmax
// Row softmax of scale * x (one warp per row, the row is re-read from L1), and its
// backward ds = scale * p * (dp - sum(dp * p)). Used by the unfused attention path.
__global__ void __launch_bounds__(128)
softmax_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, int64_t rows, int S, float scale) {
  const int lane = threadIdx.x & 31;
  for (int64_t r = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5); r < rows; r += (int64_t)gridDim.x * 4) {
    const bf16* xr = x + r * S;
    float mx = -INFINITY;
    for (int c = lane * 8; c < S; c += 256) { float v[8]; load8(xr + c, v);
#pragma unroll
      for (int i = 0; i < 8; i++) mx = fmaxf(mx, v[i]); }
    mx = warp_max(mx) * scale;
    float sum = 0;
    for (int c = lane * 8; c < S; c += 256) { float v[8]; load8(xr + c, v);
#pragma unroll
      for (int i = 0; i < 8; i++) sum += __expf(v[i] * scale - mx); }
    const float inv = 1.0f / warp_sum(sum);
    bf16* yr = y + r * S;
    for (int c = lane * 8; c < S; c += 256) {
      float v[8];
      load8(xr + c, v);
#pragma unroll
      for (int i = 0; i < 8; i++) v[i] = __expf(v[i] * scale - mx) * inv;
      store8(yr + c, v);
    }
  }
}
__global__ void __launch_bounds__(128)
softmax_bwd_kernel(const bf16* __restrict__ dp, const bf16* __restrict__ p, bf16* __restrict__ ds, int64_t rows, int S,
                   float scale) {
  const int lane = threadIdx.x & 31;
  for (int64_t r = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5); r < rows; r += (int64_t)gridDim.x * 4) {
    const bf16 *gr = dp + r * S, *pr = p + r * S;
    float dot = 0;
    for (int c = lane * 8; c < S; c += 256) { float g[8], q[8]; load8(gr + c, g); load8(pr + c, q);
#pragma unroll
      for (int i = 0; i < 8; i++) dot += g[i] * q[i]; }
    dot = warp_sum(dot);
    bf16* dr = ds + r * S;
    for (int c = lane * 8; c < S; c += 256) {
      float g[8], q[8];
      load8(gr + c, g); load8(pr + c, q);
#pragma unroll
      for (int i = 0; i < 8; i++) g[i] = scale * q[i] * (g[i] - dot);
      store8(dr + c, g);
    }
  }
}

// -------------------------------------------------------------- column sums
// part[blockIdx.y][c] = sum over this CTA's row range of g[r][c]  (bf16 in, fp32 out)
__global__ void __launch_bounds__(256)
colsum_partial_kernel(const bf16* __restrict__ g, float* __restrict__ part, int rows, int cols, int ld, int rows_per) {
  pdl_trigger();
  pdl_wait();
  const int c = (blockIdx.x * 256 + threadIdx.x) * 2;
  if (c >= cols) return;
  const int r0 = blockIdx.y * rows_per, r1 = min(rows, r0 + rows_per);
  float s0 = 0, s1 = 0;
  for (int r = r0; r < r1; r++) {
    const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(g + (size_t)r * ld + c);
    const float2 f = __bfloat1622float2(v);
    s0 += f.x; s1 += f.y;
  }
  part[(size_t)blockIdx.y * cols + c] = s0;
  if (c + 1 < cols) part[(size_t)blockIdx.y * cols + c + 1] = s1;
}

// Wide variant: 16-byte loads (8 columns per thread), 8 row lanes per CTA with independent accumulators,
// folded through shared memory. One CTA covers 256 columns x rows_per rows.
__global__ void __launch_bounds__(256)
colsum_partial8_kernel(const bf16* __restrict__ g, float* __restrict__ part, int rows, int cols, int ld, int rows_per) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[8][256 + 8];
  const int cg = threadIdx.x & 31, rl = threadIdx.x >> 5;       // column group (8 columns), row lane
  const int c = blockIdx.x * 256 + cg * 8;
  const int r0 = blockIdx.y * rows_per, r1 = min(rows, r0 + rows_per);
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; j++) acc[j] = 0.0f;
  if (c < cols) {
#pragma unroll 4
    for (int r = r0 + rl; r < r1; r += 8) {
      const uint4 v = *reinterpret_cast<const uint4*>(g + (size_t)r * ld + c);
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int e = 0; e < 4; e++) { const float2 f = __bfloat1622float2(b[e]); acc[2 * e] += f.x; acc[2 * e + 1] += f.y; }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; j++) red[rl][cg * 8 + j] = acc[j];
  __syncthreads();
  const int col = blockIdx.x * 256 + threadIdx.x;
  if (col < cols) {
    float s = 0.0f;
#pragma unroll
    for (int l = 0; l < 8; l++) s += red[l][threadIdx.x];     // fixed order
    part[(size_t)blockIdx.y * cols + col] = s;
  }
}

// ------------------------------------------------------- image normalisation
// uint8 NHWC [n, 3] pixels -> bf16 NHWC padded to `cpad` channels (extra channels 0):
// y = (x - mean_c) / std_c with mean/std given in 0..255 units.
__global__ void u8_to_bf16_norm_kernel(const uint8_t* __restrict__ x, bf16* __restrict__ y, size_t pixels, int cpad,
                                       float m0, float m1, float m2, float i0, float i1, float i2) {
  for (size_t p = (size_t)blockIdx.x * blockDim.x + threadIdx.x; p < pixels; p += (size_t)gridDim.x * blockDim.x) {
    const uint8_t* s = x + p * 3;
    bf16* d = y + p * cpad;
    d[0] = __float2bfloat16(((float)s[0] - m0) * i0);
    d[1] = __float2bfloat16(((float)s[1] - m1) * i1);
    d[2] = __float2bfloat16(((float)s[2] - m2) * i2);
    for (int c = 3; c < cpad; c++) d[c] = __float2bfloat16(0.0f);
  }
}

}  // namespace nl
}  // namespace gcow

using namespace gcow::nl;

extern "C" {

int gcow_layernorm_fwd(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd,
                       int rows, int H, float eps, void* stream) {
  if (H % 8 || rows <= 0) return -1;
  int grid = (rows + 3) / 4; if (grid > 148 * 16) grid = 148 * 16;
  gcow::launch_dependent(layernorm_fwd_kernel, dim3(grid), dim3(128), 0, (cudaStream_t)stream, (const bf16*)x, gamma, beta, (bf16*)y, mean, rstd, rows, H, eps);
  return (int)cudaGetLastError();
}

// Number of partial rows the backward writes; `part` must hold parts * 2 * H floats.
int gcow_layernorm_bwd_parts(int rows) { int g = (rows + 3) / 4; return g < 148 * 3 ? g : 148 * 3; }   // three CTAs per SM are resident

int gcow_layernorm_bwd(const void* dy, const void* x, const float* gamma, const float* mean, const float* rstd,
                       void* dx, float* part, float* dgamma_dbeta, int rows, int H, void* stream) {
  if (H % 8 || rows <= 0 || H > 4096) return -1;
  const int parts = gcow_layernorm_bwd_parts(rows);
  const size_t smem = (size_t)8 * H * sizeof(float);
  static bool attr = false;
  if (!attr) { cudaFuncSetAttribute(layernorm_bwd_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 4096 * 4); attr = true; }
  const int ch = (H + 255) / 256;
#define GCOW_LN_BWD(CH) gcow::launch_dependent(layernorm_bwd_kernel<CH>, dim3(parts), dim3(128), smem, (cudaStream_t)stream, (const bf16*)dy, (const bf16*)x, gamma, mean, rstd, (bf16*)dx, part, rows, H)
  switch (ch) {
    case 1: GCOW_LN_BWD(1); break;
    case 2: GCOW_LN_BWD(2); break;
    case 3: GCOW_LN_BWD(3); break;
    case 4: GCOW_LN_BWD(4); break;
    default: GCOW_LN_BWD(0); break;
  }
#undef GCOW_LN_BWD
  gcow::launch_dependent(reduce_partials_tall_kernel, dim3((2 * H + 31) / 32), dim3(32, 32), 0, (cudaStream_t)stream, (const float*)part,
                   dgamma_dbeta, parts, 2 * H);
  return (int)cudaGetLastError();
}

int gcow_gelu_fwd(const void* x, void* y, uint64_t n, void* stream) {
  if (n % 8) return -1;
  if (!n) return 0;
  uint64_t n8 = n / 8; int grid = (int)((n8 + 255) / 256 < 148 * 16 ? (n8 + 255) / 256 : 148 * 16);
  gelu_fwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)y, n8);
  return (int)cudaGetLastError();
}
int gcow_gelu_bwd(const void* dy, const void* x, void* dx, uint64_t n, void* stream) {
  if (n % 8) return -1;
  if (!n) return 0;
  uint64_t n8 = n / 8; int grid = (int)((n8 + 255) / 256 < 148 * 16 ? (n8 + 255) / 256 : 148 * 16);
  gelu_bwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const bf16*)dy, (const bf16*)x, (bf16*)dx, n8);
  return (int)cudaGetLastError();
}

int gcow_softmax_xent(void* logits, const int64_t* target, float* row_loss, const float* valid_count, int rows,
                      int V, int ld, int ignore_index, void* stream) {
  if (ld % 8 || V > ld || rows <= 0) return -1;
  softmax_xent_kernel<<<rows, 256, 0, (cudaStream_t)stream>>>((bf16*)logits, target, row_loss, valid_count, V, ld, ignore_index);
  return (int)cudaGetLastError();
}

// out[i] = sum_p part[p * n + i] in a fixed order (split-K partial products, bias partials).
int gcow_reduce_partials(const float* part, float* out, int parts, int64_t n, void* stream) {
  if (n <= 0 || parts <= 0 || n > 0x7fffffff) return -1;
  if (parts >= 64 && n <= 65536)
    gcow::launch_dependent(reduce_partials_tall_kernel, dim3((unsigned)((n + 31) / 32)), dim3(32, 32), 0, (cudaStream_t)stream, part, out,
                     parts, (int)n);
  else
    gcow::launch_dependent(reduce_partials_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, part, out, parts,
                     (int)n);
  return (int)cudaGetLastError();
}

int gcow_softmax_fwd(const void* x, void* y, int64_t rows, int S, float scale, void* stream) {
  if (S % 8 || rows <= 0) return -1;
  int64_t g = (rows + 3) / 4; if (g > 148 * 16) g = 148 * 16;
  softmax_fwd_kernel<<<(int)g, 128, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)y, rows, S, scale);
  return (int)cudaGetLastError();
}
int gcow_softmax_bwd(const void* dp, const void* p, void* ds, int64_t rows, int S, float scale, void* stream) {
  if (S % 8 || rows <= 0) return -1;
  int64_t g = (rows + 3) / 4; if (g > 148 * 16) g = 148 * 16;
  softmax_bwd_kernel<<<(int)g, 128, 0, (cudaStream_t)stream>>>((const bf16*)dp, (const bf16*)p, (bf16*)ds, rows, S, scale);
  return (int)cudaGetLastError();
}

// Column sums of a bf16 [rows, cols] matrix (ld even, cols even) into fp32 out[cols];
// `part` must hold gcow_colsum_parts(rows) * cols floats.
int gcow_colsum_parts(int rows) { int p = (rows + 127) / 128; return p < 128 ? (p < 1 ? 1 : p) : 128; }
int gcow_colsum(const void* g, float* part, float* out, int rows, int cols, int ld, void* stream) {
  if (cols % 2 || ld % 2 || rows <= 0) return -1;
  const int parts = gcow_colsum_parts(rows);
  const int rows_per = (rows + parts - 1) / parts;
  if (cols % 8 == 0 && ld % 8 == 0 && ((uintptr_t)g & 15) == 0) {
    dim3 grid((cols + 255) / 256, parts);
    gcow::launch_dependent(colsum_partial8_kernel, grid, dim3(256), 0, (cudaStream_t)stream, (const bf16*)g, part, rows, cols, ld, rows_per);
  } else {
    dim3 grid((cols / 2 + 255) / 256, parts);
    gcow::launch_dependent(colsum_partial_kernel, grid, dim3(256), 0, (cudaStream_t)stream, (const bf16*)g, part, rows, cols, ld, rows_per);
  }
  if (parts >= 64)
    gcow::launch_dependent(reduce_partials_tall_kernel, dim3((cols + 31) / 32), dim3(32, 32), 0, (cudaStream_t)stream, (const float*)part,
                     out, parts, cols);
  else
    gcow::launch_dependent(reduce_partials_kernel, dim3((cols + 255) / 256), dim3(256), 0, (cudaStream_t)stream, (const float*)part, out,
                     parts, cols);
  return (int)cudaGetLastError();
}

int gcow_u8_to_bf16_norm(const void* x, void* y, uint64_t pixels, int cpad, const float* mean3, const float* std3,
                         void* stream) {
  if (!pixels) return 0;
  int grid = (int)((pixels + 255) / 256 < 148 * 16 ? (pixels + 255) / 256 : 148 * 16);
  u8_to_bf16_norm_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)x, (bf16*)y, pixels, cpad, mean3[0], mean3[1],
                                                                 mean3[2], 1.0f / std3[0], 1.0f / std3[1], 1.0f / std3[2]);
  return (int)cudaGetLastError();
}

}  // extern "C"
