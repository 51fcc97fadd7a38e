// Fused multi-head self-attention on the 5th-generation tensor cores (sm_100a), head dimension 64,
// sequence length a multiple of 128 up to 512, no mask, no dropout: forward and backward.
//
// All three kernels read the packed projection qkv [B][S][3][H][64] (bf16) in place through 4-D
// tensor maps {d, h, s, b} - a box is 128 sequence positions of one head, 128-byte rows with the
// 128-byte swizzle - and write the context / gradients in the layouts the neighbouring GEMMs use
// ([B][S][H][64] and [B][S][3][H][64]), so no transposed copy of Q, K or V exists.
//
//  forward   one CTA per (128 queries, head): S = Q K^T for ALL keys lands in tensor memory (up to
//            512 fp32 columns, one row per thread), the row maximum and the exponentials are taken
//            straight from there, P goes to shared memory as bf16 in the MMA's K-major layout and
//            O = P V accumulates in the tensor-memory columns that S has vacated. exp(S - max)
//            needs no running rescale because the whole row is present. Also stores the row's
//            log2-sum-exp for the backward pass.
//  backward  recomputes P from Q, K and the stored log-sum-exp.
//     dK/dV  one CTA per (128 keys, head), loop over the query tiles: S and dP = dO V^T in tensor
//            memory, P and dS = P (dP - delta) to shared memory in the MN-major layout so that
//            P^T dO and dS^T Q need no transpose, dV and dK accumulate in tensor memory.
//     dQ     one CTA per (128 queries, head), loop over the key tiles: same S, dP, dS, then
//            dQ += dS K. Recomputing S and dP here instead of adding dQ with atomics keeps the
//            gradients deterministic.
//  delta = rowsum(dO * O) comes from a small elementwise kernel.
//
// 512 threads per CTA: four threads share an accumulator row (the four warps that may read a
// tensor-memory lane quarter each take a quarter of the columns), which is what hides the latency
// of the exponentials; thread 0 issues the TMA loads and the MMAs. Every mbarrier wait is bounded: after a fixed number of polls the CTA records an error
// code, leaves its loops, waits (bounded) for outstanding MMAs, frees its tensor memory and
// returns. No load uses cluster multicast. The reference's models are CNNs
// (hw/models/train_imagenet.py:199-202); this kernel serves the BERT configuration.
#include <stdio.h>
#include <mutex>

#include "tc_common.cuh"

namespace gcow {
namespace attn {

using namespace gcow::tc;

constexpr int D = 64;                 // head dimension: one 128-byte row
constexpr int TILE = 128;             // rows of a query / key tile
constexpr int TILE_BYTES = TILE * D * 2;   // 16 KB
constexpr int MAX_S = 512;
constexpr int NT = 512;               // threads per CTA: 4 column groups x 128 rows

struct Params {
  __nv_bfloat16* out;      // forward: context [B][S][H][64]
  float* lse;              // [B][H][S] log2-sum-exp of the scaled scores
  const float* delta;      // backward: [B][H][S] rowsum(dO * O)
  __nv_bfloat16* dqkv;     // backward: [B][S][3][H][64]
  int B, S, H;
  float scale_log2;        // softmax scale * log2(e)
  float scale;             // softmax scale
  uint32_t* error;
};

struct Bars {
  uint64_t a, b, c, d, e[2], f[2], drain;
  uint32_t tmem_base;
  volatile uint32_t abort;
  float red[4][TILE];      // per-row partial maxima / sums of the four column groups
};

__device__ __forceinline__ uint32_t idesc_f16(int n, bool a_mn, bool b_mn) {
  // fp32 accumulate, bf16 x bf16, operand major-ness, N, M = 128
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ bool wait(Bars* bs, uint64_t* bar, uint32_t parity, uint32_t* error, uint32_t code) {
  return mbar_wait_abortable(&bs->abort, bar, parity, error, code);
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
// Byte offset of the 16-byte chunk holding elements 8j..8j+7 of row r in a [rows][64] bf16 tile with
// 128-byte rows and the 128-byte swizzle (the layout TMA writes and the K-major descriptor reads).
__device__ __forceinline__ uint32_t sw128(int r, int j) { return (uint32_t)(r * 128 + ((j ^ (r & 7)) << 4)); }

// Store 32 consecutive fp32 values of this thread's row as bf16 into a K-major operand: the row has `64`
// elements per 16 KB block, the 32 values are elements e0..e0+31 of the row (e0 a multiple of 32).
__device__ __forceinline__ void store_kmajor32(uint8_t* tile, int row, int e0, const float (&v)[32]) {
  uint8_t* blk = tile + (e0 >> 6) * TILE_BYTES;
  const int j0 = (e0 & 63) >> 3;
#pragma unroll
  for (int j = 0; j < 4; j++) {
    uint4 o = make_uint4(pack2(v[8 * j], v[8 * j + 1]), pack2(v[8 * j + 2], v[8 * j + 3]),
                         pack2(v[8 * j + 4], v[8 * j + 5]), pack2(v[8 * j + 6], v[8 * j + 7]));
    *reinterpret_cast<uint4*>(blk + sw128(row, j0 + j)) = o;
  }
}
// Store 32 consecutive values of this thread's row into an MN-major operand whose reduction index is the ROW
// (this thread) and whose M/N index is the column: [k-block = row / 64][box = col / 64][row % 64][64 cols].
__device__ __forceinline__ void store_mnmajor32(uint8_t* tile, int row, int c0, const float (&v)[32]) {
  uint8_t* box = tile + (row >> 6) * 16384 + (c0 >> 6) * 8192;
  const int r = row & 63, j0 = (c0 & 63) >> 3;
#pragma unroll
  for (int j = 0; j < 4; j++) {
    uint4 o = make_uint4(pack2(v[8 * j], v[8 * j + 1]), pack2(v[8 * j + 2], v[8 * j + 3]),
                         pack2(v[8 * j + 4], v[8 * j + 5]), pack2(v[8 * j + 6], v[8 * j + 7]));
    *reinterpret_cast<uint4*>(box + sw128(r, j0 + j)) = o;
  }
}

__device__ __forceinline__ void tmem_alloc(Bars* bs, int warp) {
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bs->tmem_base)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
}
__device__ __forceinline__ void tmem_free(uint32_t base, int warp) {
  if (warp == 0) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(512u) : "memory");
  }
}
// All MMAs issued by this thread have completed (bounded), so tensor memory and the operands may go.
__device__ __forceinline__ void drain(Bars* bs) {
  tc_commit(&bs->drain);
  for (uint32_t it = 0; it < kSpinLimit; it++) if (mbar_try_wait(&bs->drain, 0)) break;
}

// A [128 x 64k] K-major (rows x reduction) times B: 4 k-steps per 64 reduction elements.
__device__ __forceinline__ void mma_kk(uint32_t d_tmem, uint32_t a_smem, uint32_t b_smem, int n, bool acc) {
  const uint32_t id = idesc_f16(n, false, false);
  const uint64_t da = smem_desc_sw128(a_smem), db = smem_desc_sw128(b_smem);
#pragma unroll
  for (int k = 0; k < 4; k++) tc_mma(d_tmem, da + 2 * k, db + 2 * k, id, acc || k);
}

// ------------------------------------------------------------------------------ forward
__global__ void __launch_bounds__(NT, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                const __grid_constant__ CUtensorMap tv, const Params p) {
  extern __shared__ uint8_t raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = base;                       // 16 KB
  uint8_t* sK = sQ + TILE_BYTES;            // S/128 tiles; P of the first 256 keys overwrites it
  uint8_t* sV = sK + 4 * TILE_BYTES;
  uint8_t* sP1 = sV + 4 * TILE_BYTES;       // P of keys 256..511
  Bars* bs = reinterpret_cast<Bars*>(sP1 + 4 * TILE_BYTES);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int row = (warp & 3) * 32 + (tid & 31), cg = warp >> 2;      // accumulator row, column group 0..3
  const int q0 = blockIdx.x * TILE, h = blockIdx.y, b = blockIdx.z;
  const int nk = p.S, ntile = nk / TILE;
  const int half0 = nk < 256 ? nk : 256, half1 = nk - half0;

  if (tid == 0) {
    mbar_init(&bs->a, 1); mbar_init(&bs->b, 1); mbar_init(&bs->c, 1); mbar_init(&bs->d, 1); mbar_init(&bs->drain, 1);
    bs->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  tmem_alloc(bs, warp);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bs->tmem_base;
  const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
  bool ok = true;

  if (tid == 0) {
    mbar_expect_tx(&bs->a, TILE_BYTES + nk * 128);
    tma_load_4d(smem_u32(sQ), &tq, smem_u32(&bs->a), 0, h, q0, b);
    for (int t = 0; t < ntile; t++) tma_load_4d(smem_u32(sK + t * TILE_BYTES), &tk, smem_u32(&bs->a), 0, h, t * TILE, b);
    mbar_expect_tx(&bs->b, nk * 128);
    for (int t = 0; t < ntile; t++) tma_load_4d(smem_u32(sV + t * TILE_BYTES), &tv, smem_u32(&bs->b), 0, h, t * TILE, b);
    ok = wait(bs, &bs->a, 0, p.error, 21);
    if (ok) {
      tc_fence_after();
      mma_kk(tmem, smem_u32(sQ), smem_u32(sK), half0, false);                       // S[:, 0:half0]
      if (half1) mma_kk(tmem + 256, smem_u32(sQ), smem_u32(sK + 2 * TILE_BYTES), half1, false);
      tc_commit(&bs->c);
    }
  }
  ok = wait(bs, &bs->c, 0, p.error, 22);
  ok = __syncthreads_and(ok);
  if (ok) {
    tc_fence_after();
    // pass 1: row maximum over every key; this thread scans its quarter of the columns
    float m = -INFINITY;
    {
      // tensor-memory loads two chunks ahead of the arithmetic
      const int c0 = cg * (nk / 128), c1 = (cg + 1) * (nk / 128);
      uint32_t ra[32], rb[32];
      tc_ld32(lane_addr + c0 * 32, ra);
      for (int c = c0; c < c1; c += 2) {
        tc_wait_ld();
        if (c + 1 < c1) tc_ld32(lane_addr + (c + 1) * 32, rb);
#pragma unroll
        for (int j = 0; j < 32; j++) m = fmaxf(m, __uint_as_float(ra[j]));
        if (c + 1 < c1) {
          tc_wait_ld();
          if (c + 2 < c1) tc_ld32(lane_addr + (c + 2) * 32, ra);
#pragma unroll
          for (int j = 0; j < 32; j++) m = fmaxf(m, __uint_as_float(rb[j]));
        }
      }
    }
    bs->red[cg][row] = m;
    __syncthreads();
    m = fmaxf(fmaxf(bs->red[0][row], bs->red[1][row]), fmaxf(bs->red[2][row], bs->red[3][row]));
    __syncthreads();                        // red is reused for the row sums below
    const float ms = m * p.scale_log2;
    float l = 0.0f;
    // pass 2: exponentials, row sum, P as bf16 in the A-operand layout; then O += P V for that half
    for (int hf = 0; hf < 2; hf++) {      // same trip count for every thread: the loop body holds barriers
      const int keys = hf ? half1 : half0;
      if (!keys) break;
      uint8_t* sP = hf ? sP1 : sK;
      {
        // this thread's one or two chunks of the half: both loads are issued before the first is used
        const int c0 = cg * (keys / 128), two = keys / 128 == 2;
        uint32_t ra[32], rb[32];
        tc_ld32(lane_addr + hf * 256 + c0 * 32, ra);
        if (two) tc_ld32(lane_addr + hf * 256 + (c0 + 1) * 32, rb);
        tc_wait_ld();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; j++) {
          v[j] = exp2f(fmaf(__uint_as_float(ra[j]), p.scale_log2, -ms));
          l += v[j];
        }
        store_kmajor32(sP, row, c0 * 32, v);
        if (two) {
#pragma unroll
          for (int j = 0; j < 32; j++) {
            v[j] = exp2f(fmaf(__uint_as_float(rb[j]), p.scale_log2, -ms));
            l += v[j];
          }
          store_kmajor32(sP, row, (c0 + 1) * 32, v);
        }
      }
      proxy_fence();
      tc_fence_before();
      __syncthreads();
      if (tid == 0) {
        if (hf == 0 && ok) ok = wait(bs, &bs->b, 0, p.error, 23);
        if (ok) {
          tc_fence_after();
          const uint32_t id = idesc_f16(D, false, true);
          for (int blk = 0; blk < keys / 64; blk++) {
            const uint64_t da = smem_desc_sw128(smem_u32(sP + blk * TILE_BYTES));
            const uint64_t db = smem_desc_mn_sw128(smem_u32(sV + (hf * 256 + blk * 64) * 128));
#pragma unroll
            for (int k = 0; k < 4; k++) tc_mma(tmem, da + 2 * k, db + (2048 >> 4) * k, id, (hf | blk | k) != 0);
          }
          if (hf == 1 || !half1) tc_commit(&bs->d);
        }
      }
    }
    bs->red[cg][row] = l;
    ok = ok && wait(bs, &bs->d, 0, p.error, 24);
    ok = __syncthreads_and(ok);
    if (ok) {
      tc_fence_after();
      l = (bs->red[0][row] + bs->red[1][row]) + (bs->red[2][row] + bs->red[3][row]);
      const float inv = 1.0f / l;
      const size_t orow = (((size_t)b * p.S + q0 + row) * p.H + h) * D;
      if (cg < 2) {                          // 64 output columns: column groups 0 and 1 take 32 each
        const int c = cg;
        uint32_t r[32];
        tc_ld32(lane_addr + c * 32, r);
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 4; j++) {
          uint4 o = make_uint4(pack2(__uint_as_float(r[8 * j]) * inv, __uint_as_float(r[8 * j + 1]) * inv),
                               pack2(__uint_as_float(r[8 * j + 2]) * inv, __uint_as_float(r[8 * j + 3]) * inv),
                               pack2(__uint_as_float(r[8 * j + 4]) * inv, __uint_as_float(r[8 * j + 5]) * inv),
                               pack2(__uint_as_float(r[8 * j + 6]) * inv, __uint_as_float(r[8 * j + 7]) * inv));
          *reinterpret_cast<uint4*>(p.out + orow + c * 32 + j * 8) = o;
        }
      }
      if (cg == 0) p.lse[((size_t)b * p.H + h) * p.S + q0 + row] = ms + log2f(l);
    }
  }
  if (tid == 0) drain(bs);
  tc_fence_before();
  __syncthreads();
  tmem_free(tmem, warp);
}

// delta[b][h][s] = sum_d dO[b][s][h][d] * O[b][s][h][d]; one thread per row.
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ go,
                                  float* __restrict__ delta, int B, int S, int H) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;       // over b, s, h
  if (i >= (size_t)B * S * H) return;
  const int h = (int)(i % H);
  const size_t bs = i / H;
  const int s = (int)(bs % S), b = (int)(bs / S);
  const uint4* po = reinterpret_cast<const uint4*>(o + i * D);
  const uint4* pg = reinterpret_cast<const uint4*>(go + i * D);
  float acc = 0.0f;
#pragma unroll
  for (int k = 0; k < D / 8; k++) {
    const uint4 x = po[k], y = pg[k];
    const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&x);
    const __nv_bfloat162* yb = reinterpret_cast<const __nv_bfloat162*>(&y);
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const float2 a = __bfloat1622float2(xb[e]), c = __bfloat1622float2(yb[e]);
      acc = fmaf(a.x, c.x, fmaf(a.y, c.y, acc));
    }
  }
  delta[((size_t)b * H + h) * S + s] = acc;
}

// P and dS of one 128 x 128 tile from S (tensor-memory columns 0..127) and dP (columns 128..255): this thread's
// row. WRITE_P: also emit P. MN: operands go to the MN-major layout (reduction over rows), else K-major.
template <bool WRITE_P, bool MN>
__device__ __forceinline__ void softmax_grad_tile(uint32_t lane_addr, int row, int c, float lse, float delta, const Params& p,
                                                  uint8_t* sP, uint8_t* sdS) {
  {                                          // this thread's 32-column chunk c of the row
    uint32_t rs[32], rd[32];
    tc_ld32(lane_addr + c * 32, rs);
    tc_ld32(lane_addr + 128 + c * 32, rd);
    tc_wait_ld();
    float pv[32], ds[32];
#pragma unroll
    for (int j = 0; j < 32; j++) {
      pv[j] = exp2f(fmaf(__uint_as_float(rs[j]), p.scale_log2, -lse));
      ds[j] = pv[j] * (__uint_as_float(rd[j]) - delta) * p.scale;
    }
    if (MN) {
      if (WRITE_P) store_mnmajor32(sP, row, c * 32, pv);
      store_mnmajor32(sdS, row, c * 32, ds);
    } else {
      if (WRITE_P) store_kmajor32(sP, row, c * 32, pv);
      store_kmajor32(sdS, row, c * 32, ds);
    }
  }
}

// Write this thread's row of a 64-column fp32 accumulator (tensor-memory column `col`) as bf16 to `dst`.
__device__ __forceinline__ void store_acc_row(uint32_t lane_addr, int col, int c, __nv_bfloat16* dst) {
  {                                          // chunk c (0 or 1) of the 64 columns
    uint32_t r[32];
    tc_ld32(lane_addr + col + c * 32, r);
    tc_wait_ld();
#pragma unroll
    for (int j = 0; j < 4; j++) {
      uint4 o = make_uint4(pack2(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1])),
                           pack2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3])),
                           pack2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5])),
                           pack2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7])));
      *reinterpret_cast<uint4*>(dst + c * 32 + j * 8) = o;
    }
  }
}

// ------------------------------------------------------------------- backward: dK and dV
__global__ void __launch_bounds__(NT, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                     const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo, const Params p) {
  extern __shared__ uint8_t raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sK = base;                        // 16 KB each
  uint8_t* sV = sK + TILE_BYTES;
  uint8_t* sQ = sV + TILE_BYTES;             // two buffers
  uint8_t* sdO = sQ + 2 * TILE_BYTES;        // two buffers
  uint8_t* sP = sdO + 2 * TILE_BYTES;        // 32 KB, MN-major
  uint8_t* sdS = sP + 2 * TILE_BYTES;        // 32 KB, MN-major
  Bars* bs = reinterpret_cast<Bars*>(sdS + 2 * TILE_BYTES);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int row = (warp & 3) * 32 + (tid & 31), cg = warp >> 2;
  const int k0 = blockIdx.x * TILE, h = blockIdx.y, b = blockIdx.z;
  const int nq = p.S / TILE;

  if (tid == 0) {
    mbar_init(&bs->a, 1); mbar_init(&bs->c, 1); mbar_init(&bs->d, 1); mbar_init(&bs->drain, 1);
    mbar_init(&bs->e[0], 1); mbar_init(&bs->e[1], 1);
    bs->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  tmem_alloc(bs, warp);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bs->tmem_base;
  const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
  constexpr uint32_t COL_S = 0, COL_DV = 256, COL_DK = 320;      // dP sits at COL_S + 128
  bool ok = true;

  if (tid == 0) {
    mbar_expect_tx(&bs->a, 2 * TILE_BYTES);
    tma_load_4d(smem_u32(sK), &tk, smem_u32(&bs->a), 0, h, k0, b);
    tma_load_4d(smem_u32(sV), &tv, smem_u32(&bs->a), 0, h, k0, b);
    mbar_expect_tx(&bs->e[0], 2 * TILE_BYTES);
    tma_load_4d(smem_u32(sQ), &tq, smem_u32(&bs->e[0]), 0, h, 0, b);
    tma_load_4d(smem_u32(sdO), &tdo, smem_u32(&bs->e[0]), 0, h, 0, b);
    ok = wait(bs, &bs->a, 0, p.error, 31);
  }
  for (int i = 0; i < nq; i++) {
    const int buf = i & 1;
    uint8_t* q = sQ + buf * TILE_BYTES;
    uint8_t* go = sdO + buf * TILE_BYTES;
    if (tid == 0 && ok) {
      // the other buffer was last read by the MMAs of iteration i-1, whose completion (bar d) is awaited
      // below before this point is reached again; start fetching tile i+1 into it now
      if (i + 1 < nq) {
        if (i >= 1) ok = wait(bs, &bs->d, (i - 1) & 1, p.error, 32);
        if (ok) {
          mbar_expect_tx(&bs->e[buf ^ 1], 2 * TILE_BYTES);
          tma_load_4d(smem_u32(sQ + (buf ^ 1) * TILE_BYTES), &tq, smem_u32(&bs->e[buf ^ 1]), 0, h, (i + 1) * TILE, b);
          tma_load_4d(smem_u32(sdO + (buf ^ 1) * TILE_BYTES), &tdo, smem_u32(&bs->e[buf ^ 1]), 0, h, (i + 1) * TILE, b);
        }
      }
      ok = ok && wait(bs, &bs->e[buf], (i >> 1) & 1, p.error, 33);
      if (ok) {
        tc_fence_after();
        mma_kk(tmem + COL_S, smem_u32(q), smem_u32(sK), TILE, false);            // S  = Q_i K_j^T
        mma_kk(tmem + COL_S + 128, smem_u32(go), smem_u32(sV), TILE, false);     // dP = dO_i V_j^T
        tc_commit(&bs->c);
      }
    }
    const size_t stat = ((size_t)b * p.H + h) * p.S + i * TILE + row;
    const float lse = p.lse[stat], delta = p.delta[stat];
    ok = wait(bs, &bs->c, i & 1, p.error, 34);
    // P / dS of iteration i-1 must have been consumed by its MMAs before they are overwritten
    if (i >= 1) ok = ok && wait(bs, &bs->d, (i - 1) & 1, p.error, 35);
    ok = __syncthreads_and(ok);
    if (!ok) break;
    tc_fence_after();
    softmax_grad_tile<true, true>(lane_addr + COL_S, row, cg, lse, delta, p, sP, sdS);
    proxy_fence();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      const uint32_t id = idesc_f16(D, true, true);                 // A = P^T / dS^T (MN-major), B = dO / Q as [q][d]
      for (int kb = 0; kb < 2; kb++) {
        const uint64_t dap = smem_desc_mn_sw128(smem_u32(sP + kb * 16384));
        const uint64_t dad = smem_desc_mn_sw128(smem_u32(sdS + kb * 16384));
        const uint64_t dbo = smem_desc_mn_sw128(smem_u32(go + kb * 8192));
        const uint64_t dbq = smem_desc_mn_sw128(smem_u32(q + kb * 8192));
#pragma unroll
        for (int k = 0; k < 4; k++) {
          tc_mma(tmem + COL_DV, dap + (2048 >> 4) * k, dbo + (2048 >> 4) * k, id, (i | kb | k) != 0);
          tc_mma(tmem + COL_DK, dad + (2048 >> 4) * k, dbq + (2048 >> 4) * k, id, (i | kb | k) != 0);
        }
      }
      tc_commit(&bs->d);
    }
  }
  ok = ok && wait(bs, &bs->d, (nq - 1) & 1, p.error, 36);
  ok = __syncthreads_and(ok);
  if (ok) {
    tc_fence_after();
    const size_t orow = ((((size_t)b * p.S + k0 + row) * 3) * p.H + h) * D;     // [b][s][which][h][d], which = 0
    // column groups 0, 1: the two halves of dK's row; 2, 3: of dV's row
    store_acc_row(lane_addr, cg < 2 ? COL_DK : COL_DV, cg & 1, p.dqkv + orow + (size_t)(cg < 2 ? 1 : 2) * p.H * D);
  }
  if (tid == 0) drain(bs);
  tc_fence_before();
  __syncthreads();
  tmem_free(tmem, warp);
}

// ------------------------------------------------------------------------ backward: dQ
__global__ void __launch_bounds__(NT, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                   const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo, const Params p) {
  extern __shared__ uint8_t raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = base;
  uint8_t* sdO = sQ + TILE_BYTES;
  uint8_t* sK = sdO + TILE_BYTES;            // two buffers
  uint8_t* sV = sK + 2 * TILE_BYTES;         // two buffers
  uint8_t* sdS = sV + 2 * TILE_BYTES;        // 32 KB, K-major: [128 queries][128 keys] as two 64-key blocks
  Bars* bs = reinterpret_cast<Bars*>(sdS + 2 * TILE_BYTES);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int row = (warp & 3) * 32 + (tid & 31), cg = warp >> 2;
  const int q0 = blockIdx.x * TILE, h = blockIdx.y, b = blockIdx.z;
  const int nkv = p.S / TILE;

  if (tid == 0) {
    mbar_init(&bs->a, 1); mbar_init(&bs->c, 1); mbar_init(&bs->d, 1); mbar_init(&bs->drain, 1);
    mbar_init(&bs->e[0], 1); mbar_init(&bs->e[1], 1);
    bs->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  tmem_alloc(bs, warp);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bs->tmem_base;
  const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
  constexpr uint32_t COL_S = 0, COL_DQ = 256;
  bool ok = true;
  const size_t stat = ((size_t)b * p.H + h) * p.S + q0 + row;
  const float lse = p.lse[stat], delta = p.delta[stat];

  if (tid == 0) {
    mbar_expect_tx(&bs->a, 2 * TILE_BYTES);
    tma_load_4d(smem_u32(sQ), &tq, smem_u32(&bs->a), 0, h, q0, b);
    tma_load_4d(smem_u32(sdO), &tdo, smem_u32(&bs->a), 0, h, q0, b);
    mbar_expect_tx(&bs->e[0], 2 * TILE_BYTES);
    tma_load_4d(smem_u32(sK), &tk, smem_u32(&bs->e[0]), 0, h, 0, b);
    tma_load_4d(smem_u32(sV), &tv, smem_u32(&bs->e[0]), 0, h, 0, b);
    ok = wait(bs, &bs->a, 0, p.error, 41);
  }
  for (int j = 0; j < nkv; j++) {
    const int buf = j & 1;
    uint8_t* kt = sK + buf * TILE_BYTES;
    uint8_t* vt = sV + buf * TILE_BYTES;
    if (tid == 0 && ok) {
      if (j + 1 < nkv) {
        if (j >= 1) ok = wait(bs, &bs->d, (j - 1) & 1, p.error, 42);      // K of tile j-1 is still read by its dQ MMAs
        if (ok) {
          mbar_expect_tx(&bs->e[buf ^ 1], 2 * TILE_BYTES);
          tma_load_4d(smem_u32(sK + (buf ^ 1) * TILE_BYTES), &tk, smem_u32(&bs->e[buf ^ 1]), 0, h, (j + 1) * TILE, b);
          tma_load_4d(smem_u32(sV + (buf ^ 1) * TILE_BYTES), &tv, smem_u32(&bs->e[buf ^ 1]), 0, h, (j + 1) * TILE, b);
        }
      }
      ok = ok && wait(bs, &bs->e[buf], (j >> 1) & 1, p.error, 43);
      if (ok) {
        tc_fence_after();
        mma_kk(tmem + COL_S, smem_u32(sQ), smem_u32(kt), TILE, false);           // S  = Q_i K_j^T
        mma_kk(tmem + COL_S + 128, smem_u32(sdO), smem_u32(vt), TILE, false);    // dP = dO_i V_j^T
        tc_commit(&bs->c);
      }
    }
    ok = wait(bs, &bs->c, j & 1, p.error, 44);
    if (j >= 1) ok = ok && wait(bs, &bs->d, (j - 1) & 1, p.error, 45);           // dS of tile j-1 consumed
    ok = __syncthreads_and(ok);
    if (!ok) break;
    tc_fence_after();
    softmax_grad_tile<false, false>(lane_addr + COL_S, row, cg, lse, delta, p, nullptr, sdS);
    proxy_fence();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      const uint32_t id = idesc_f16(D, false, true);                // A = dS (K-major), B = K_j as [key][d] (MN-major)
      for (int blk = 0; blk < 2; blk++) {
        const uint64_t da = smem_desc_sw128(smem_u32(sdS + blk * TILE_BYTES));
        const uint64_t db = smem_desc_mn_sw128(smem_u32(kt + blk * 8192));
#pragma unroll
        for (int k = 0; k < 4; k++) tc_mma(tmem + COL_DQ, da + 2 * k, db + (2048 >> 4) * k, id, (j | blk | k) != 0);
      }
      tc_commit(&bs->d);
    }
  }
  ok = ok && wait(bs, &bs->d, (nkv - 1) & 1, p.error, 46);
  ok = __syncthreads_and(ok);
  if (ok) {
    tc_fence_after();
    const size_t orow = ((((size_t)b * p.S + q0 + row) * 3) * p.H + h) * D;
    if (cg < 2) store_acc_row(lane_addr, COL_DQ, cg, p.dqkv + orow);
  }
  if (tid == 0) drain(bs);
  tc_fence_before();
  __syncthreads();
  tmem_free(tmem, warp);
}

// ------------------------------------------------------------------------------ host side
// One of Q / K / V inside qkv [B][S][3][H][64] (which = 0, 1, 2), or a plain [B][S][H][64] tensor (which = -1):
// dims {d, h, s, b}, box = 64 x 1 x 128 x 1 (128 rows of one head).
static int make_map(CUtensorMap* map, const void* ptr, int B, int S, int H, int which) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return -10;
  const uint64_t row = (which >= 0 ? 3ull : 1ull) * H * D;          // elements between consecutive sequence positions
  const char* basep = (const char*)ptr + (which > 0 ? (size_t)which * H * D * 2 : 0);
  if ((uintptr_t)basep & 15) return -11;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)D * 2, row * 2, row * 2 * (cuuint64_t)S};
  cuuint32_t box[4] = {(cuuint32_t)D, 1, (cuuint32_t)TILE, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<char*>(basep), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "gcow attention: cuTensorMapEncodeTiled failed with CUresult %d (B %d S %d H %d which %d)\n", (int)r, B, S, H, which);
    return -12;
  }
  return 0;
}

constexpr size_t kFwdSmem = TILE_BYTES * 13 + sizeof(Bars) + 1024;      // Q + 4 K + 4 V + 4 P
constexpr size_t kBwdSmem = TILE_BYTES * 10 + sizeof(Bars) + 1024;      // K, V, 2 Q, 2 dO, P (2), dS (2)
constexpr size_t kDqSmem = TILE_BYTES * 8 + sizeof(Bars) + 1024;        // Q, dO, 2 K, 2 V, dS (2)

static int check_shape(int B, int S, int H, int d) {
  if (d != D || S % TILE || S <= 0 || S > MAX_S || B <= 0 || H <= 0 || H > 65535 || B > 65535) return -1;
  return 0;
}

static void set_attrs() {
  static std::once_flag once;
  std::call_once(once, [] {
    cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFwdSmem);
    cudaFuncSetAttribute(attn_bwd_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kBwdSmem);
    cudaFuncSetAttribute(attn_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDqSmem);
  });
}

}  // namespace attn
}  // namespace gcow

using namespace gcow::attn;

extern "C" {

// 1 if the fused kernels cover this problem (head dimension 64, S a multiple of 128 up to 512).
int gcow_attention_supported(int B, int S, int H, int d) { return check_shape(B, S, H, d) == 0; }

// out[B][S][H][64] = softmax(scale * Q K^T) V per head, qkv [B][S][3][H][64] bf16; lse [B][H][S] fp32 receives the
// log2-sum-exp of the scaled scores (kept for the backward pass). `error`: device word, set if a wait gave up.
int gcow_attention_fwd(const void* qkv, void* out, float* lse, int B, int S, int H, int d, float scale,
                       uint32_t* error, void* stream) {
  if (check_shape(B, S, H, d)) return -1;
  set_attrs();
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_map(&tq, qkv, B, S, H, 0)) || (rc = make_map(&tk, qkv, B, S, H, 1)) || (rc = make_map(&tv, qkv, B, S, H, 2)))
    return rc;
  Params p = {};
  p.out = (__nv_bfloat16*)out; p.lse = lse; p.B = B; p.S = S; p.H = H;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f; p.error = error;
  attn_fwd_kernel<<<dim3(S / TILE, H, B), NT, kFwdSmem, (cudaStream_t)stream>>>(tq, tk, tv, p);
  return (int)cudaGetLastError();
}

// dqkv[B][S][3][H][64] from qkv, the forward's out and lse, and dout [B][S][H][64]; delta [B][H][S] fp32 is scratch.
int gcow_attention_bwd(const void* qkv, const void* out, const void* dout, const float* lse, float* delta, void* dqkv,
                       int B, int S, int H, int d, float scale, uint32_t* error, void* stream) {
  if (check_shape(B, S, H, d)) return -1;
  set_attrs();
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  if ((rc = make_map(&tq, qkv, B, S, H, 0)) || (rc = make_map(&tk, qkv, B, S, H, 1)) || (rc = make_map(&tv, qkv, B, S, H, 2)) ||
      (rc = make_map(&tdo, dout, B, S, H, -1)))
    return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t rows = (size_t)B * S * H;
  attn_delta_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)out, (const __nv_bfloat16*)dout, delta, B, S, H);
  Params p = {};
  p.lse = const_cast<float*>(lse); p.delta = delta; p.dqkv = (__nv_bfloat16*)dqkv; p.B = B; p.S = S; p.H = H;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f; p.error = error;
  attn_bwd_dkdv_kernel<<<dim3(S / TILE, H, B), NT, kBwdSmem, st>>>(tq, tk, tv, tdo, p);
  attn_bwd_dq_kernel<<<dim3(S / TILE, H, B), NT, kDqSmem, st>>>(tq, tk, tv, tdo, p);
  return (int)cudaGetLastError();
}

}  // extern "C"
