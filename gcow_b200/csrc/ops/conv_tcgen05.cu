// Implicit-GEMM convolution on the 5th-generation tensor cores (sm_100a), NHWC bf16,
// stride 1 or 2, any odd or even filter size with zero padding. No im2col matrix is ever
// written: the TMA unit gathers the shifted input window of every filter tap
// straight from the activation tensor, and its out-of-bounds zero fill IS the padding.
//
//   forward   Y[n,h,w,co] = sum_{r,s,ci} X[n, h+r-ph, w+s-pw, ci] * Wt[co,r,s,ci]
//             GEMM view: M = output pixels, N = Co, K = (r,s,ci).
//             An M tile is a box of bw x bh x bn output pixels (<= 256 rows) of a 4-D tensor
//             map {C, W, H, N}; for tap (r,s) the same box is fetched at (w0+s-pw, h0+r-ph).
//             Rows of the box land in shared memory as 128-byte channel rows with the
//             128-byte swizzle, exactly the K-major operand layout of tcgen05.mma.
//             Stride 2: the tensor map steps two elements along W and H (elementStrides), so the box holds every
//             second input pixel and the same code runs on the half-size output grid.
//   dgrad     the same kernel on dY with the filter flipped and its channel roles swapped
//             (flip_weights_kernel), padding k-1-p. Stride 2 (3x3, padding 1): the input gradient splits by the
//             parity of its pixel coordinates into four stride-1 convolutions of dY with 1, 2, 2 and 4 of the nine
//             taps (phase_weights_kernel); each writes every second pixel of every second row of dX.
//   wgrad     dW[co, (r,s,ci)] = sum_pixels dY[pixel, co] * X[pixel + (r,s) - p, ci]
//             GEMM view: M = Co, N = taps*Ci, K = pixels. Both operands are MN-major:
//             64-pixel boxes of dY (A) and of the shifted X (B, one 64-channel box per
//             (tap, channel chunk) column group, each with its own shift). The pixel
//             range is split over CTAs; fp32 partial results are summed by a second
//             kernel in a fixed order.
//
// Same structure as the GEMM kernel: persistent CTAs, warp 0 issues TMA loads into an
// mbarrier ring, one thread of warp 1 issues tcgen05.mma into TMEM accumulators, eight
// epilogue warps read them back with tcgen05.ld. No multicast; every wait is bounded and
// gives up by raising an error word.
//
// What sets the speed (measured): a TMA copy costs a few hundred cycles per instruction
// on top of its bytes, and an M128 x N x K16 MMA takes about as long for N = 64 as for
// N = 256. So a stage is fetched with as few, as large boxes as possible - the forward
// tile is one box of up to 256 pixels (two 128-row accumulators that share the filter
// tile), the weight gradient folds its 64-channel groups into a fifth box dimension -
// and the launcher picks the tile from a small cost model of those two effects.
//
// Replaces the cuDNN 3x3 convolutions behind nn.Conv2d in the reference's models
// (hw/models/resenet.py:14,48-50).
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <mutex>

#include "pdl.cuh"
#include "tc_common.cuh"

namespace gcow {
namespace conv {

using namespace gcow::tc;

constexpr int BK = 64, UMMA_K = 16, MAX_STAGES = 8;
constexpr int HALF_BYTES = 128 * BK * 2;       // one 128-row operand tile: 128 rows (or two 64-column boxes) of 128 bytes
constexpr int EPI_WARPS = 8, THREADS = 64 + 32 * EPI_WARPS;
constexpr uint32_t TMEM_COLS = 512;
constexpr int kSmemBudget = 200 * 1024;

enum Flags : int { kBias = 2 };

struct Params {
  void* out;            // forward: bf16 [N, H, W, Co]; wgrad: fp32 partials [split][Co][taps * Ci]
  const float* bias;    // forward only, [Co] or nullptr
  int N, H, W;          // extents of the output pixels (forward) / of dY (wgrad)
  int Ci, Co;           // forward: reduction channels and output channels; wgrad: channels of X and of dY
  int kh, kw, pad_h, pad_w;
  int bw, bh, bn;       // pixel box of one TMA load
  int tiles_w, tiles_h, tiles_n;   // number of pixel boxes along W, H, N
  int bn_cols;          // GEMM N of one tile: 64, 128 or 256
  int stages;
  int split, chunks_per_split;     // wgrad: CTA groups over the pixel range
  int b_chunks;         // wgrad: 64-channel groups of X fetched by one copy (1, 2 or 4)
  int flags;
  int stride;           // step of the input window per output pixel (forward) / per dY pixel (wgrad): 1 or 2
  int swap;             // forward, two accumulators, 128 output channels: the channels are the MMA's M, the 256 pixels its N
  int out_step, out_off_h, out_off_w, out_H, out_W;   // forward: tile pixel (h, w) is stored at (h * out_step + out_off_h,
                                                      // w * out_step + out_off_w) of a [N, out_H, out_W, Co] tensor
  uint32_t* error;
};

struct Smem {
  uint64_t full[MAX_STAGES], empty[MAX_STAGES], tmem_full[2], tmem_empty[4], drain;
  uint32_t tmem_base;
  volatile uint32_t abort;
};

// HALVES: 128-row accumulators per tile
template <bool WGRAD, int HALVES>
__global__ void __launch_bounds__(THREADS, 1)
conv_igemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int A_BYTES = HALVES * HALF_BYTES;
  const int b_bytes = p.bn_cols * BK * 2;
  const int stage_bytes = A_BYTES + b_bytes;
  const int STAGES = p.stages;
  Smem* sm = reinterpret_cast<Smem*>(base + STAGES * stage_bytes);
  // per-warp staging buffers of the epilogue, 16-byte aligned behind the barriers
  uint8_t* stage_base = reinterpret_cast<uint8_t*>(((uintptr_t)(sm + 1) + 15) & ~(uintptr_t)15);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int taps = p.kh * p.kw;
  const int cchunks = p.Ci / BK;
  const int pix_tiles = p.tiles_w * p.tiles_h * p.tiles_n;
  // forward: tiles over (pixel box, Co tile), reduction over (tap, channel chunk)
  // wgrad:   tiles over (split, Co tile, column tile of taps*Ci), reduction over pixel boxes
  const int tiles_c = WGRAD ? (p.Co + 128 * HALVES - 1) / (128 * HALVES) : (p.Co + p.bn_cols - 1) / p.bn_cols;
  const int col_groups = taps * cchunks;                          // wgrad: 64-column groups of N
  const int tiles_col = (col_groups * BK + p.bn_cols - 1) / p.bn_cols;
  const int num_tiles = WGRAD ? p.split * tiles_c * tiles_col : pix_tiles * tiles_c;
  // Accumulators: tile t uses buffer b = t & 1 when two tiles fit in the 512 columns, else always buffer 0;
  // half h of buffer b sits at column b * 256 + h * (columns per half).
  const bool dbuf = HALVES * p.bn_cols <= 256;
  const uint32_t half_cols = dbuf ? (uint32_t)p.bn_cols : 256u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(&sm->full[s], 1); mbar_init(&sm->empty[s], 1); }
    for (int a = 0; a < 2; a++) mbar_init(&sm->tmem_full[a], 1);
    for (int a = 0; a < 4; a++) mbar_init(&sm->tmem_empty[a], EPI_WARPS * 32);
    mbar_init(&sm->drain, 1);
    sm->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm->tmem_base)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm->tmem_base;
  // a kernel launched as a programmatic dependent (the ordered sum of split partial results) may be scheduled
  // from here on; it waits for this grid to complete before it reads anything
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // this grid's own set-up ran under the tail of its predecessor; global memory only after that one has completed
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // reduction length of a tile (wgrad: the pixel boxes of its split)
  auto tile_kblocks = [&](int tile) -> int {
    if (!WGRAD) return taps * cchunks;
    const int sp = tile / (tiles_c * tiles_col);
    const int first = sp * p.chunks_per_split;
    int last = first + p.chunks_per_split;
    if (last > pix_tiles) last = pix_tiles;
    return last - first;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t s = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!WGRAD) {
          const int tcn = tile % tiles_c, pt = tile / tiles_c;
          const int w0 = (pt % p.tiles_w) * p.bw, h0 = ((pt / p.tiles_w) % p.tiles_h) * p.bh;
          const int n0 = (pt / (p.tiles_w * p.tiles_h)) * p.bn;
          const int co0 = tcn * p.bn_cols;
          const uint32_t a_tx = (uint32_t)(p.bw * p.bh * p.bn) * 128u;
          for (int tap = 0; tap < taps && ok; tap++) {
            const int r = tap / p.kw, sx = tap - r * p.kw;
            for (int cc = 0; cc < cchunks; cc++) {
              if (!(ok = mbar_wait_abortable(&sm->abort, &sm->empty[s], phase ^ 1, p.error, 1))) break;
              mbar_expect_tx(&sm->full[s], a_tx + (uint32_t)b_bytes);
              const uint32_t bar = smem_u32(&sm->full[s]);
              uint8_t* st = base + s * stage_bytes;
              tma_load_4d(smem_u32(st), &map_a, bar, cc * BK, w0 * p.stride + sx - p.pad_w, h0 * p.stride + r - p.pad_h, n0);
              tma_load_2d(smem_u32(st + A_BYTES), &map_b, bar, tap * p.Ci + cc * BK, co0);
              if (++s == (uint32_t)STAGES) { s = 0; phase ^= 1; }
            }
          }
        } else {
          const int tcol = tile % tiles_col;
          int rest = tile / tiles_col;
          const int tco = rest % tiles_c, sp = rest / tiles_c;
          const int g0 = tcol * (p.bn_cols / BK);                 // first 64-column group of this tile
          const int first = sp * p.chunks_per_split, nk = tile_kblocks(tile);
          for (int kb = 0; kb < nk; kb++) {
            const int chunk = first + kb;
            const int w0 = (chunk % p.tiles_w) * p.bw, h0 = ((chunk / p.tiles_w) % p.tiles_h) * p.bh;
            const int n0 = (chunk / (p.tiles_w * p.tiles_h)) * p.bn;
            if (!(ok = mbar_wait_abortable(&sm->abort, &sm->empty[s], phase ^ 1, p.error, 1))) break;
            mbar_expect_tx(&sm->full[s], (uint32_t)(A_BYTES + b_bytes));
            const uint32_t bar = smem_u32(&sm->full[s]);
            uint8_t* st = base + s * stage_bytes;
            // dY: every 64-channel group of the tile's rows in one copy (groups past Co read zeros)
            tma_load_5d(smem_u32(st), &map_a, bar, 0, w0, h0, n0, tco * 2 * HALVES);
            // X: runs of b_chunks channel groups share a filter tap, hence a shift, hence a copy
            for (int i = 0; i < p.bn_cols / BK; i += p.b_chunks) {
              const int g = g0 + i;
              int tap = g / cchunks, ch = g - tap * cchunks;
              if (g >= col_groups) { tap = 0; ch = cchunks; }     // past the last column group: zeros
              const int r = tap / p.kw, sx = tap - r * p.kw;
              tma_load_5d(smem_u32(st + A_BYTES + i * 8192), &map_b, bar, 0, w0 * p.stride + sx - p.pad_w,
                          h0 * p.stride + r - p.pad_h, n0, ch);
            }
            if (++s == (uint32_t)STAGES) { s = 0; phase ^= 1; }
          }
        }
      }
      if (!ok) {
        // giving up: let copies already in flight land before the CTA's shared memory is released
        for (int i = 0; i < 1000; i++) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      // instruction descriptor: fp32 accumulate, bf16 x bf16, operand major-ness, N = bn_cols, M = 128
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)WGRAD << 15) | ((uint32_t)WGRAD << 16) |
                             ((uint32_t)(p.bn_cols >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      constexpr uint64_t kstep = WGRAD ? (2048 >> 4) : (32 >> 4);
      uint32_t s = 0, phase = 0, t = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, t++) {
        const uint32_t buf = dbuf ? (t & 1) : 0, use = dbuf ? (t >> 1) : t;
        const int nk = tile_kblocks(tile);
        for (int kb = 0; kb < nk && ok; kb++) {
          if (!(ok = mbar_wait_abortable(&sm->abort, &sm->full[s], phase, p.error, 3))) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(base + s * stage_bytes), sb = sa + A_BYTES;
          const uint64_t db = WGRAD ? smem_desc_mn_sw128(sb) : smem_desc_sw128(sb);
          if (!WGRAD && HALVES == 2 && p.swap) {
            // D[co][pixel]: the filter tile is A, both pixel halves (contiguous in shared memory) are one 256-row B
            if (kb == 0) {
              for (int h = 0; h < 2 && ok; h++) ok = mbar_wait_abortable(&sm->abort, &sm->tmem_empty[buf * 2 + h], (use & 1) ^ 1, p.error, 2);
              if (!ok) break;
              tc_fence_after();
            }
            const uint32_t idesc_swap = (1u << 4) | (1u << 7) | (1u << 10) | ((256u >> 3) << 17) | ((128u >> 4) << 24);
            const uint64_t dpix = smem_desc_sw128(sa);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; k++)
              tc_mma(tmem_base + buf * 256, db + kstep * k, dpix + kstep * k, idesc_swap, (kb | k) != 0);
            tc_commit(&sm->empty[s]);
            if (++s == (uint32_t)STAGES) { s = 0; phase ^= 1; }
            continue;
          }
#pragma unroll
          for (int h = 0; h < HALVES; h++) {
            if (kb == 0) {   // first write to this accumulator: its previous contents must have been read out
              if (!(ok = mbar_wait_abortable(&sm->abort, &sm->tmem_empty[buf * 2 + h], (use & 1) ^ 1, p.error, 2))) break;
              tc_fence_after();
            }
            const uint64_t da = WGRAD ? smem_desc_mn_sw128(sa + h * HALF_BYTES) : smem_desc_sw128(sa + h * HALF_BYTES);
            const uint32_t d_tmem = tmem_base + buf * 256 + h * half_cols;
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; k++)
              tc_mma(d_tmem, da + kstep * k, db + kstep * k, idesc, (kb | k) != 0);
          }
          if (!ok) break;
          tc_commit(&sm->empty[s]);
          if (++s == (uint32_t)STAGES) { s = 0; phase ^= 1; }
        }
        if (ok) tc_commit(&sm->tmem_full[buf]);
      }
      // drain: everything issued by this thread has finished before TMEM is freed
      tc_commit(&sm->drain);
      for (uint32_t it = 0; it < kSpinLimit; it++) if (mbar_try_wait(&sm->drain, 0)) break;
    }
  } else {
    // ----------------------------------------------------------------- epilogue
    const int q = warp & 3;                       // TMEM lane quarter this warp may read
    const int ew = warp - 2;
    const int cols = p.bn_cols / 2;               // columns of each accumulator this warp drains
    const int col0 = (ew / 4) * cols;
    const int nch = cols / 32;                    // 1, 2 or 4 chunks of 32 columns
    uint32_t t = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, t++) {
      const uint32_t buf = dbuf ? (t & 1) : 0, use = dbuf ? (t >> 1) : t;
      ok = mbar_wait_abortable(&sm->abort, &sm->tmem_full[buf], use & 1, p.error, 4);
      ok = __all_sync(0xffffffffu, ok);   // the tensor-memory loads below need the whole warp
      if (!ok) break;
      tc_fence_after();
      if (!WGRAD && HALVES == 2 && p.swap) {
        // lane = output channel q * 32 + lane, column = tile pixel: 32-pixel chunks pass through the warp's staging
        // buffer as [pixel][32 channels] and leave as 16-byte pieces, four lanes per pixel
        const int tcn = tile % tiles_c, pt = tile / tiles_c;
        const int w0 = (pt % p.tiles_w) * p.bw, h0 = ((pt / p.tiles_w) % p.tiles_h) * p.bh;
        const int n0 = (pt / (p.tiles_w * p.tiles_h)) * p.bn;
        const int co = tcn * p.bn_cols + q * 32;
        const int hsel = ew / 4;
        const float bias = (p.flags & kBias) && co + lane < p.Co ? __ldg(p.bias + co + lane) : 0.0f;
        uint8_t* stg = stage_base + ew * kStageWarpBytes;
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * 256 + hsel * 128;
        __nv_bfloat16* outp = reinterpret_cast<__nv_bfloat16*>(p.out) + co + (lane & 3) * 8;
        const bool co_ok = co + (lane & 3) * 8 + 8 <= p.Co;
        auto emit = [&](const uint32_t (&r)[32], int c) {
#pragma unroll
          for (int e = 0; e < 32; e++)
            *reinterpret_cast<__nv_bfloat16*>(stg + e * 64 + lane * 2) = __float2bfloat16(__uint_as_float(r[e]) + bias);
          __syncwarp();
#pragma unroll
          for (int e0 = 0; e0 < 32; e0 += 8) {
            const int row = hsel * 128 + c * 32 + e0 + (lane >> 2);
            const int iw = row % p.bw, ih = (row / p.bw) % p.bh, in = row / (p.bw * p.bh);
            const int w = w0 + iw, hh = h0 + ih, n = n0 + in;
            const int oh = hh * p.out_step + p.out_off_h, ow = w * p.out_step + p.out_off_w;
            const uint4 v = *reinterpret_cast<const uint4*>(stg + (e0 + (lane >> 2)) * 64 + (lane & 3) * 16);
            if (co_ok && in < p.bn && w < p.W && hh < p.H && n < p.N && oh < p.out_H && ow < p.out_W)
              *reinterpret_cast<uint4*>(outp + (((size_t)n * p.out_H + oh) * p.out_W + ow) * (size_t)p.Co) = v;
          }
          __syncwarp();
        };
        uint32_t ra[32], rb[32];
        tc_ld32(taddr, ra);
        tc_wait_ld();
        tc_ld32(taddr + 32, rb);
        emit(ra, 0);
        tc_wait_ld();
        tc_ld32(taddr + 64, ra);
        emit(rb, 1);
        tc_wait_ld();
        tc_ld32(taddr + 96, rb);
        emit(ra, 2);
        tc_wait_ld();
        tc_fence_before();
        mbar_arrive(&sm->tmem_empty[buf * 2]);
        mbar_arrive(&sm->tmem_empty[buf * 2 + 1]);
        emit(rb, 3);
        continue;
      }
#pragma unroll 1
      for (int h = 0; h < HALVES; h++) {
        const int row = h * 128 + q * 32 + lane;    // tile row of this thread
        // where this thread's row goes
        bool row_ok;
        size_t row_off;        // element offset of the row's first column of this tile
        int n_first, n_limit;  // first column index of this tile, and the column bound
        if (!WGRAD) {
          const int tcn = tile % tiles_c, pt = tile / tiles_c;
          const int iw = row % p.bw, ih = (row / p.bw) % p.bh, in = row / (p.bw * p.bh);
          const int w = (pt % p.tiles_w) * p.bw + iw, hh = ((pt / p.tiles_w) % p.tiles_h) * p.bh + ih;
          const int n = (pt / (p.tiles_w * p.tiles_h)) * p.bn + in;
          const int oh = hh * p.out_step + p.out_off_h, ow = w * p.out_step + p.out_off_w;
          row_ok = in < p.bn && w < p.W && hh < p.H && n < p.N && oh < p.out_H && ow < p.out_W;
          n_first = tcn * p.bn_cols;
          n_limit = p.Co;
          row_off = (((size_t)n * p.out_H + oh) * p.out_W + ow) * (size_t)p.Co;
        } else {
          const int tcol = tile % tiles_col;
          int rest = tile / tiles_col;
          const int tco = rest % tiles_c, sp = rest / tiles_c;
          const int co = tco * 128 * HALVES + row;
          const int ncols = col_groups * BK;
          row_ok = co < p.Co;
          n_first = tcol * p.bn_cols;
          n_limit = ncols;
          row_off = ((size_t)sp * p.Co + co) * (size_t)ncols;
        }
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * 256 + h * half_cols + col0;
        auto process = [&](const uint32_t (&r)[32], int c) {
          const int n = n_first + col0 + c * 32;
          if (!WGRAD && p.bn_cols == 256 && n + 32 <= n_limit) {
            // wide rows, whole 32-channel chunk (warp-uniform): coalesced store through the warp's staging buffer
            // (measured: a gain at 256 output channels per tile, a loss at 64 and 128, where rows are short anyway)
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[j]);
            if (p.flags & kBias) {
#pragma unroll
              for (int j = 0; j < 32; j++) v[j] += __ldg(p.bias + n + j);
            }
            warp_store_rows_bf16(stage_base + ew * kStageWarpBytes, lane, v, reinterpret_cast<__nv_bfloat16*>(p.out),
                                 row_off + n, row_ok);
            return;
          }
          if (row_ok && n < n_limit) {
            if (WGRAD) {
              float* C = reinterpret_cast<float*>(p.out) + row_off + n;
              if (n + 32 <= n_limit) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                  *reinterpret_cast<float4*>(C + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                                  __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
              } else {
#pragma unroll
                for (int j = 0; j < 32; j++) if (n + j < n_limit) C[j] = __uint_as_float(r[j]);
              }
            } else {
              float v[32];
#pragma unroll
              for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[j]);
              if (p.flags & kBias) {
#pragma unroll
                for (int j = 0; j < 32; j++) if (n + j < n_limit) v[j] += __ldg(p.bias + n + j);
              }
              __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(p.out) + row_off + n;
              if (n + 32 <= n_limit) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  uint4 o;
                  __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                  for (int e = 0; e < 4; e++) ob[e] = __floats2bfloat162_rn(v[j + 2 * e], v[j + 2 * e + 1]);
                  *reinterpret_cast<uint4*>(C + j) = o;
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; j++) if (n + j < n_limit) C[j] = __float2bfloat16(v[j]);
              }
            }
          }
        };
        uint32_t ra[32], rb[32];
        tc_ld32(taddr, ra);
#pragma unroll 1
        for (int c = 0; c < nch; c += 2) {
          tc_wait_ld();
          if (c + 1 < nch) tc_ld32(taddr + (c + 1) * 32, rb);
          process(ra, c);
          if (c + 1 < nch) {
            tc_wait_ld();
            if (c + 2 < nch) tc_ld32(taddr + (c + 2) * 32, ra);
            process(rb, c + 1);
          }
        }
        // this accumulator has been read out: the MMA warp may overwrite it
        tc_fence_before();
        mbar_arrive(&sm->tmem_empty[buf * 2 + h]);
      }
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------------------
// Weight-stationary forward for 64 -> 64 channels, 3x3, stride 1, padding 1 (the first stage of ResNet-50).
// With 64 output channels as the MMA's N the instruction above uses a quarter of the array's width. Here the
// roles are swapped: D[co][pixel] = sum_taps W_tap[co][ci] * X[pixel + tap][ci], the pixels are the 256-wide N
// and the filter is the A operand. The 72 KB filter is fetched once per CTA and stays in shared memory. Per
// tile ONE copy brings the pixel rows with their halo - (rows + 2) x (W + 2) pixels of 128 bytes, zero filled
// outside the image - and the nine taps read it in place: pixel slot n = i * (W + 2) + j of the tile is smem row
// n + r * (W + 2) + s for tap (r, s), so a tap is the same operand descriptor moved by whole 128-byte rows.
// Slots with j >= W or i >= rows hold sums nobody needs and are not stored. Against nine copies per tile this
// reads each pixel from L2 once (plus the halo) instead of nine times.
// The MMA is M = 64 x N = 256: accumulator row r (an output channel) sits in lane (r / 16) * 32 + r % 16 of the
// tensor memory, so each of the four lane quarters holds 16 channels and all eight epilogue warps have work
// (measured: 80 us against 100 us with M = 128 and the upper 64 rows unused; an MMA takes about 150 cycles
// either way). A descriptor whose start is not 1024-byte aligned needs no base offset: the 128-byte swizzle
// is a function of the absolute shared-memory address, for the TMA's writes and the MMA's reads alike.
struct WsParams {
  __nv_bfloat16* out;   // [N, H, W, 64]
  const float* bias;    // [64] or nullptr
  int N, H, W;
  int pitch;            // W + 2: pixel slots per image row
  int rows;             // image rows per tile
  int nslots;           // N of the MMA: rows * pitch rounded up to 16 (an MMA's time grows with its N)
  int tiles_h;
  int stages, stage_bytes;
  uint32_t* error;
};

constexpr int WS_TAPS = 9, WS_W_BYTES = WS_TAPS * 64 * 128;
constexpr int kWsSmemMax = 227 * 1024;

struct WsSmem {
  uint64_t full[4], empty[4], tmem_full[2], tmem_empty[2], wfull, drain;
  uint32_t tmem_base;
  volatile uint32_t abort;
};

__global__ void __launch_bounds__(THREADS, 1)
conv_ws_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const WsParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* stage0 = base + WS_W_BYTES;
  WsSmem* sm = reinterpret_cast<WsSmem*>(stage0 + p.stages * p.stage_bytes);
  uint8_t* stage_base = reinterpret_cast<uint8_t*>(((uintptr_t)(sm + 1) + 15) & ~(uintptr_t)15);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = p.N * p.tiles_h;
  const int STAGES = p.stages;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(&sm->full[s], 1); mbar_init(&sm->empty[s], 1); }
    for (int a = 0; a < 2; a++) { mbar_init(&sm->tmem_full[a], 1); mbar_init(&sm->tmem_empty[a], EPI_WARPS * 32); }
    mbar_init(&sm->wfull, 1);
    mbar_init(&sm->drain, 1);
    sm->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm->tmem_base)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm->tmem_base;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(&sm->wfull, (uint32_t)WS_W_BYTES);
      for (int tap = 0; tap < WS_TAPS; tap++)
        tma_load_2d(smem_u32(base + tap * 8192), &map_w, smem_u32(&sm->wfull), tap * 64, 0);
      const uint32_t tx = (uint32_t)(p.pitch * (p.rows + 2)) * 128u;
      uint32_t s = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int n = tile / p.tiles_h, h0 = (tile - n * p.tiles_h) * p.rows;
        if (!(ok = mbar_wait_abortable(&sm->abort, &sm->empty[s], phase ^ 1, p.error, 1))) break;
        mbar_expect_tx(&sm->full[s], tx);
        tma_load_4d(smem_u32(stage0 + s * p.stage_bytes), &map_x, smem_u32(&sm->full[s]), 0, -1, h0 - 1, n);
        if (++s == (uint32_t)STAGES) { s = 0; phase ^= 1; }
      }
      if (!ok) {
        for (int i = 0; i < 1000; i++) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.nslots >> 3) << 17) | ((64u >> 4) << 24);
      bool ok = mbar_wait_abortable(&sm->abort, &sm->wfull, 0, p.error, 5);
      tc_fence_after();
      const uint32_t wsm = smem_u32(base);
      uint32_t s = 0, phase = 0, t = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, t++) {
        const uint32_t buf = t & 1, use = t >> 1;
        if (!(ok = mbar_wait_abortable(&sm->abort, &sm->full[s], phase, p.error, 3))) break;
        if (!(ok = mbar_wait_abortable(&sm->abort, &sm->tmem_empty[buf], (use & 1) ^ 1, p.error, 2))) break;
        tc_fence_after();
        const uint32_t xs = smem_u32(stage0 + s * p.stage_bytes);
        const uint32_t d_tmem = tmem_base + buf * 256;
#pragma unroll 1
        for (int tap = 0; tap < WS_TAPS; tap++) {
          const int r = tap / 3, sx = tap - 3 * r;
          const uint32_t xb = xs + (uint32_t)(r * p.pitch + sx) * 128u;
          uint64_t db = smem_desc_sw128(xb);
          const uint64_t da = smem_desc_sw128(wsm + tap * 8192);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; k++) tc_mma(d_tmem, da + 2 * k, db + 2 * k, idesc, (tap | k) != 0);
        }
        tc_commit(&sm->empty[s]);
        tc_commit(&sm->tmem_full[buf]);
        if (++s == (uint32_t)STAGES) { s = 0; phase ^= 1; }
      }
      tc_commit(&sm->drain);
      for (uint32_t it = 0; it < kSpinLimit; it++) if (mbar_try_wait(&sm->drain, 0)) break;
    }
  } else {
    // Lane = output channel, column = pixel slot, but memory wants the channels of a pixel side by side: every
    // 32-slot chunk passes through the warp's staging buffer as [slot][channel] and leaves in 16-byte pieces.
    const int q = warp & 3, ew = warp - 2, half = ew / 4;
    constexpr int nco = 16;                        // channels this warp owns: lanes 0..15 of its quarter
    const int co0 = q * nco;
    const bool lane_useful = lane < nco;
    const float bias = (lane_useful && p.bias) ? __ldg(p.bias + co0 + lane) : 0.0f;
    uint8_t* stg = stage_base + ew * kStageWarpBytes;
    constexpr int row_bytes = nco * 2;             // 32 bytes of one slot
    constexpr int lanes_per_slot = row_bytes / 16, slots_per_pass = 32 / lanes_per_slot;
    const int my_slot = lane / lanes_per_slot, my_piece = lane % lanes_per_slot;
    uint32_t t = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, t++) {
      const uint32_t buf = t & 1, use = t >> 1;
      ok = mbar_wait_abortable(&sm->abort, &sm->tmem_full[buf], use & 1, p.error, 4);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int n = tile / p.tiles_h, h0 = (tile - n * p.tiles_h) * p.rows;
      {
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * 256 + half * 128;
        __nv_bfloat16* img = p.out + ((size_t)n * p.H + h0) * p.W * 64 + co0 + my_piece * 8;
        // (i, j) of the first slot this lane stores
        int i = (half * 128 + my_slot) / p.pitch, j = half * 128 + my_slot - i * p.pitch;
        auto process = [&](const uint32_t (&r)[32]) {
          if (lane_useful) {
#pragma unroll
            for (int e = 0; e < 32; e++)
              *reinterpret_cast<__nv_bfloat16*>(stg + e * row_bytes + lane * 2) = __float2bfloat16(__uint_as_float(r[e]) + bias);
          }
          __syncwarp();
          for (int e0 = 0; e0 < 32; e0 += slots_per_pass) {
            const uint4 v = *reinterpret_cast<const uint4*>(stg + (e0 + my_slot) * row_bytes + my_piece * 16);
            if (j < p.W && i < p.rows && h0 + i < p.H) *reinterpret_cast<uint4*>(img + ((size_t)i * p.W + j) * 64) = v;
            j += slots_per_pass;
            while (j >= p.pitch) { j -= p.pitch; i++; }
          }
          __syncwarp();
        };
        // the next chunk's tensor-memory load is in flight while this one is staged and stored
        uint32_t ra[32], rb[32];
        tc_ld32(taddr, ra);
        tc_wait_ld();
        tc_ld32(taddr + 32, rb);
        process(ra);
        tc_wait_ld();
        tc_ld32(taddr + 64, ra);
        process(rb);
        tc_wait_ld();
        tc_ld32(taddr + 96, rb);
        process(ra);
        tc_wait_ld();
        // everything of this accumulator is in registers: the MMA warp may overwrite it
        tc_fence_before();
        mbar_arrive(&sm->tmem_empty[buf]);
        process(rb);
      }
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------------------
// Halo-tile forward for Ci -> 128 channels, 3x3, stride 1, padding 1 (Ci a multiple of 64): the same idea as the
// weight-stationary kernel with the filter streamed instead of resident. The 128 output channels are the MMA's M,
// the pixel slots (rows x (W + 2), rounded up to 16) its N. Per tile one halo box per 64-channel chunk of the input
// (all chunks on one barrier) serves the nine taps; the filter tiles [128][64] of (chunk, tap) run through a ring
// of their own. Against the general kernel (a 32 KB pixel box per tap and chunk) the pixel traffic from L2 falls
// ninefold; the filter traffic per tile is the same.
struct HaloParams {
  __nv_bfloat16* out;   // [N, H, W, 128]
  const float* bias;
  int N, H, W, Ci;
  int pitch, rows, tiles_h;
  int nslots;           // N of the MMA: rows * pitch rounded up to 16
  int chunk_bytes;      // shared-memory region of one 64-channel chunk of a tile (1024-byte multiple)
  int a_stages, b_stages;
  uint32_t* error;
};

struct HaloSmem {
  uint64_t a_full[2], a_empty[2], b_full[8], b_empty[8], tmem_full[2], tmem_empty[2], drain;
  uint32_t tmem_base;
  volatile uint32_t abort;
};

constexpr int HALO_B_BYTES = 128 * 64 * 2;

__global__ void __launch_bounds__(THREADS, 1)
conv_halo_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const HaloParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int cchunks = p.Ci / 64;
  const int a_stage_bytes = cchunks * p.chunk_bytes;
  uint8_t* bring = base + p.a_stages * a_stage_bytes;
  HaloSmem* sm = reinterpret_cast<HaloSmem*>(bring + p.b_stages * HALO_B_BYTES);
  uint8_t* stage_base = reinterpret_cast<uint8_t*>(((uintptr_t)(sm + 1) + 15) & ~(uintptr_t)15);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = p.N * p.tiles_h;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; s++) { mbar_init(&sm->a_full[s], 1); mbar_init(&sm->a_empty[s], 1); }
    for (int s = 0; s < 8; s++) { mbar_init(&sm->b_full[s], 1); mbar_init(&sm->b_empty[s], 1); }
    for (int a = 0; a < 2; a++) { mbar_init(&sm->tmem_full[a], 1); mbar_init(&sm->tmem_empty[a], EPI_WARPS * 32); }
    mbar_init(&sm->drain, 1);
    sm->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm->tmem_base)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm->tmem_base;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == 0) {
    if (lane == 0) {
      const uint32_t a_tx = (uint32_t)(cchunks * p.pitch * (p.rows + 2)) * 128u;
      uint32_t sa = 0, pa = 0, sb = 0, pb = 0;
      bool ok = true;
      auto load_a = [&](int tile) {
        const int n = tile / p.tiles_h, h0 = (tile - n * p.tiles_h) * p.rows;
        if (!(ok = mbar_wait_abortable(&sm->abort, &sm->a_empty[sa], pa ^ 1, p.error, 1))) return;
        mbar_expect_tx(&sm->a_full[sa], a_tx);
        for (int c = 0; c < cchunks; c++)
          tma_load_4d(smem_u32(base + sa * a_stage_bytes + c * p.chunk_bytes), &map_x, smem_u32(&sm->a_full[sa]), c * 64, -1,
                      h0 - 1, n);
        if (++sa == (uint32_t)p.a_stages) { sa = 0; pa ^= 1; }
      };
      // the pixel tile of the next tile is requested in the middle of this tile's filter tiles
      if (blockIdx.x < num_tiles) load_a(blockIdx.x);
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < cchunks * WS_TAPS && ok; kb++) {
          // once the ring has wrapped within this tile the previous tile's MMAs are done and its pixel stage is free
          if (kb == p.b_stages && tile + (int)gridDim.x < num_tiles) { load_a(tile + gridDim.x); if (!ok) break; }
          const int c = kb / WS_TAPS, tap = kb - c * WS_TAPS;
          if (!(ok = mbar_wait_abortable(&sm->abort, &sm->b_empty[sb], pb ^ 1, p.error, 6))) break;
          mbar_expect_tx(&sm->b_full[sb], (uint32_t)HALO_B_BYTES);
          tma_load_2d(smem_u32(bring + sb * HALO_B_BYTES), &map_w, smem_u32(&sm->b_full[sb]), tap * p.Ci + c * 64, 0);
          if (++sb == (uint32_t)p.b_stages) { sb = 0; pb ^= 1; }
        }
      }
      if (!ok) {
        for (int i = 0; i < 1000; i++) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.nslots >> 3) << 17) | ((128u >> 4) << 24);
      uint32_t sa = 0, pa = 0, sb = 0, pb = 0, t = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, t++) {
        const uint32_t buf = t & 1, use = t >> 1;
        if (!(ok = mbar_wait_abortable(&sm->abort, &sm->a_full[sa], pa, p.error, 3))) break;
        if (!(ok = mbar_wait_abortable(&sm->abort, &sm->tmem_empty[buf], (use & 1) ^ 1, p.error, 2))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * 256;
        for (int kb = 0; kb < cchunks * WS_TAPS && ok; kb++) {
          const int c = kb / WS_TAPS, tap = kb - c * WS_TAPS;
          const int r = tap / 3, sx = tap - 3 * r;
          if (!(ok = mbar_wait_abortable(&sm->abort, &sm->b_full[sb], pb, p.error, 7))) break;
          tc_fence_after();
          const uint64_t da = smem_desc_sw128(smem_u32(bring + sb * HALO_B_BYTES));
          const uint64_t db = smem_desc_sw128(smem_u32(base + sa * a_stage_bytes + c * p.chunk_bytes) +
                                              (uint32_t)(r * p.pitch + sx) * 128u);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; k++) tc_mma(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
          tc_commit(&sm->b_empty[sb]);
          if (++sb == (uint32_t)p.b_stages) { sb = 0; pb ^= 1; }
        }
        if (!ok) break;
        tc_commit(&sm->a_empty[sa]);
        tc_commit(&sm->tmem_full[buf]);
        if (++sa == (uint32_t)p.a_stages) { sa = 0; pa ^= 1; }
      }
      tc_commit(&sm->drain);
      for (uint32_t it = 0; it < kSpinLimit; it++) if (mbar_try_wait(&sm->drain, 0)) break;
    }
  } else {
    // lane = output channel q * 32 + lane, column = pixel slot; 32-slot chunks turn around in the staging buffer
    const int q = warp & 3, ew = warp - 2, half = ew / 4;
    const int co0 = q * 32;
    const float bias = p.bias ? __ldg(p.bias + co0 + lane) : 0.0f;
    uint8_t* stg = stage_base + ew * kStageWarpBytes;
    const int my_slot = lane >> 2, my_piece = lane & 3;
    uint32_t t = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, t++) {
      const uint32_t buf = t & 1, use = t >> 1;
      ok = mbar_wait_abortable(&sm->abort, &sm->tmem_full[buf], use & 1, p.error, 4);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int n = tile / p.tiles_h, h0 = (tile - n * p.tiles_h) * p.rows;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * 256 + half * 128;
      __nv_bfloat16* img = p.out + ((size_t)n * p.H + h0) * p.W * 128 + co0 + my_piece * 8;
      int i = (half * 128 + my_slot) / p.pitch, j = half * 128 + my_slot - i * p.pitch;
      auto process = [&](const uint32_t (&r)[32]) {
#pragma unroll
        for (int e = 0; e < 32; e++)
          *reinterpret_cast<__nv_bfloat16*>(stg + e * 64 + lane * 2) = __float2bfloat16(__uint_as_float(r[e]) + bias);
        __syncwarp();
#pragma unroll
        for (int e0 = 0; e0 < 32; e0 += 8) {
          const uint4 v = *reinterpret_cast<const uint4*>(stg + (e0 + my_slot) * 64 + my_piece * 16);
          if (j < p.W && i < p.rows && h0 + i < p.H) *reinterpret_cast<uint4*>(img + ((size_t)i * p.W + j) * 128) = v;
          j += 8;
          while (j >= p.pitch) { j -= p.pitch; i++; }
        }
        __syncwarp();
      };
      // columns at and past nslots were not written by the MMA: their slots lie past the tile's rows and are skipped
      uint32_t ra[32], rb[32];
      tc_ld32(taddr, ra);
      tc_wait_ld();
      tc_ld32(taddr + 32, rb);
      process(ra);
      tc_wait_ld();
      tc_ld32(taddr + 64, ra);
      process(rb);
      tc_wait_ld();
      tc_ld32(taddr + 96, rb);
      process(ra);
      tc_wait_ld();
      tc_fence_before();
      mbar_arrive(&sm->tmem_empty[buf]);
      process(rb);
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------------------
// Weight gradient of the same layers (64 -> 64 channels, 3x3, stride 1, padding 1) from halo tiles.
//   dW[co][(r, s), ci] = sum over pixels of dY[pixel][co] * X[pixel + (r - 1, s - 1)][ci]
// A tile is four image rows in slots of pitch 64: one copy brings six rows of dY (rows h0-1 .. h0+4, columns
// 0..63, zero filled past the image) and one copy six rows of X (the same rows, columns -1..62). With dY slot
// d = (row - h0 + 1) * 64 + col the X pixel of tap (r, s) is slot d + (r - 1) * 64 + s. Both operands are
// MN-major (a slot is a 128-byte row of 64 channels, slots are the reduction), so a tap is again a start
// address moved by whole rows, and the descriptor's leading offset - the distance between consecutive 64-wide
// blocks of M or N - does two more things:
//   B: N = 192 = the three taps of a filter row, leading offset one slot (128 bytes): block n is tap s = n;
//   A: M = 128 = dY and dY one image row further down (leading offset 64 slots): the upper 64 accumulator
//      rows get the filter row r, the lower 64 the filter row r - 1 of the dY row below.
// Two MMAs per 16 slots: {r = 1 above, r = 0 below} into columns 0..191 and {r = 2 above} into columns
// 192..383 (its lower half repeats r = 1 and is not read). The lower half sees dY rows h0+1 .. h0+4; the
// first tile of an image runs four more steps (slots of row h0-1, zero for the upper half) so that it also
// sees row 0. Against the general kernel (one 8 KB copy of shifted X per tap and 64 pixels, three column
// tiles that each re-read dY) a tile of 224 pixels costs two 48 KB copies and 32 MMAs.
// Every CTA sums a contiguous range of tiles in tensor memory and writes one fp32 partial [64][576].
struct WsWgradParams {
  float* part;          // [gridDim.x][64][576]
  int N, H, W;
  int tiles_h, num_tiles, per;
  uint32_t* error;
};

constexpr int WG_X_ROWS = 392, WG_DY_ROWS = 384, WG_STAGE_BYTES = (WG_X_ROWS + WG_DY_ROWS) * 128, WG_STAGES = 2;
constexpr uint32_t WG_BOX_BYTES = 64 * 6 * 128;

__device__ __forceinline__ uint64_t smem_desc_mn_lbo(uint32_t saddr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3ffffu) >> 4);
  d |= (uint64_t)(lbo_bytes >> 4) << 16;
  d |= (uint64_t)(1024u >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__global__ void __launch_bounds__(THREADS, 1)
conv_wgrad_ws_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_dy,
                     const WsWgradParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  WsSmem* sm = reinterpret_cast<WsSmem*>(base + WG_STAGES * WG_STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int first = blockIdx.x * p.per;
  int last = first + p.per;
  if (last > p.num_tiles) last = p.num_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < WG_STAGES; s++) { mbar_init(&sm->full[s], 1); mbar_init(&sm->empty[s], 1); }
    mbar_init(&sm->tmem_full[0], 1);
    mbar_init(&sm->drain, 1);
    sm->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm->tmem_base)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // the eight rows behind each X box are read by the last taps against zero dY: they must hold finite numbers
  if (threadIdx.x < WG_STAGES * 64) {
    const int s = threadIdx.x / 64, i = threadIdx.x % 64;
    *reinterpret_cast<uint4*>(base + s * WG_STAGE_BYTES + 384 * 128 + i * 16) = make_uint4(0, 0, 0, 0);
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm->tmem_base;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == 0) {
    if (lane == 0) {
      uint32_t s = 0, phase = 0;
      bool ok = true;
      for (int tile = first; tile < last && ok; tile++) {
        const int n = tile / p.tiles_h, h0 = (tile - n * p.tiles_h) * 4;
        if (!(ok = mbar_wait_abortable(&sm->abort, &sm->empty[s], phase ^ 1, p.error, 1))) break;
        mbar_expect_tx(&sm->full[s], 2 * WG_BOX_BYTES);
        uint8_t* st = base + s * WG_STAGE_BYTES;
        tma_load_4d(smem_u32(st), &map_x, smem_u32(&sm->full[s]), 0, -1, h0 - 1, n);
        tma_load_4d(smem_u32(st + WG_X_ROWS * 128), &map_dy, smem_u32(&sm->full[s]), 0, 0, h0 - 1, n);
        if (++s == WG_STAGES) { s = 0; phase ^= 1; }
      }
      if (!ok) {
        for (int i = 0; i < 1000; i++) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // fp32 accumulate, bf16 x bf16, both operands MN-major, N = 192, M = 128
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) | ((192u >> 3) << 17) | ((128u >> 4) << 24);
      uint32_t s = 0, phase = 0, acc = 0;
      bool ok = true;
      for (int tile = first; tile < last && ok; tile++) {
        const int n = tile / p.tiles_h, h0 = (tile - n * p.tiles_h) * 4;
        if (!(ok = mbar_wait_abortable(&sm->abort, &sm->full[s], phase, p.error, 3))) break;
        tc_fence_after();
        const uint32_t xs = smem_u32(base + s * WG_STAGE_BYTES), ds = xs + WG_X_ROWS * 128;
#pragma unroll 1
        for (int k = (h0 == 0 ? 0 : 4); k < 20; k++) {
          const uint32_t off = (uint32_t)k * 16u * 128u;
          const uint64_t da = smem_desc_mn_lbo(ds + off, 64u * 128u);
          tc_mma(tmem_base, da, smem_desc_mn_lbo(xs + off, 128u), idesc, acc);
          tc_mma(tmem_base + 192, da, smem_desc_mn_lbo(xs + off + 64u * 128u, 128u), idesc, acc);
          acc = 1;
        }
        tc_commit(&sm->empty[s]);
        if (++s == WG_STAGES) { s = 0; phase ^= 1; }
      }
      if (ok) tc_commit(&sm->tmem_full[0]);
      tc_commit(&sm->drain);
      for (uint32_t it = 0; it < kSpinLimit; it++) if (mbar_try_wait(&sm->drain, 0)) break;
    }
  } else {
    const int q = warp & 3, ew = warp - 2, half = ew / 4;     // half 0: columns 0..191, half 1: columns 192..383
    bool ok = mbar_wait_abortable(&sm->abort, &sm->tmem_full[0], 0, p.error, 4);
    ok = __all_sync(0xffffffffu, ok);
    if (ok && !(half == 1 && q >= 2)) {
      tc_fence_after();
      const int row = q * 32 + lane;
      const int co = row & 63;
      const int r = half == 1 ? 2 : (row < 64 ? 1 : 0);        // filter row of this accumulator half
      float* dst = p.part + ((size_t)blockIdx.x * 64 + co) * 576 + r * 192;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + half * 192;
#pragma unroll 1
      for (int c = 0; c < 6; c++) {
        uint32_t v[32];
        tc_ld32(taddr + c * 32, v);
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(dst + c * 32 + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                                     __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
      }
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------------------
// Halo-tile weight gradient for channel counts that are multiples of 128, 3x3, stride 1, padding 1. The scheme of
// conv_wgrad_ws_kernel with real channels in both halves of M: per tile of R image rows in slots of pitch P (16, 32 or 64) one box of dY per
// 64 output channels (rows h0 .. h0+R-1, columns 0..P-1) and one box of X per 64 input channels (rows h0-1 .. h0+R,
// columns -1..P-2); X slot = dY slot + r * P + s. A: dY, M = 128 = the two channel boxes (leading offset = one
// box); B: X of one channel chunk, N = 192 = the three taps of filter row r (leading offset one slot). The
// accumulators of one filter row and 128 x 128 channels are 2 x 192 columns, so a CTA serves ONE (filter row, 128 input
// channels, 128 output channels) group (blockIdx.y) over its range of tiles; the groups re-read the tiles, which are
// cheap (with 128 channels each tensor crosses L2 three times instead of nine).
struct WgHaloParams {
  float* part;          // [gridDim.x][Co][9 * Ci]
  int N, H, W, Ci, Co;
  int P, R;             // slot pitch, image rows per tile
  int tiles_h, num_tiles, per;
  int x_chunk_bytes, dy_chunk_bytes;
  uint32_t* error;
};

__global__ void __launch_bounds__(THREADS, 1)
conv_wgrad_halo_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_dy,
                       const WgHaloParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int stage_bytes = 2 * p.x_chunk_bytes + 2 * p.dy_chunk_bytes;
  WsSmem* sm = reinterpret_cast<WsSmem*>(base + WG_STAGES * stage_bytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int first = blockIdx.x * p.per;
  int last = first + p.per;
  if (last > p.num_tiles) last = p.num_tiles;
  const int frow = blockIdx.y % 3;                // filter row of this CTA,
  const int cig = (blockIdx.y / 3) % (p.Ci / 128), cog = blockIdx.y / 3 / (p.Ci / 128);   // its 128 input and output channels
  const int x_box = p.P * (p.R + 2) * 128;        // bytes of one X box; the bytes behind it up to x_chunk_bytes are zero

  if (threadIdx.x == 0) {
    for (int s = 0; s < WG_STAGES; s++) { mbar_init(&sm->full[s], 1); mbar_init(&sm->empty[s], 1); }
    mbar_init(&sm->tmem_full[0], 1);
    mbar_init(&sm->drain, 1);
    sm->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm->tmem_base)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // the last taps read a few slots behind each X box against zero dY: those bytes must hold finite numbers
  {
    const int pad16 = (p.x_chunk_bytes - x_box) / 16;
    for (int i = threadIdx.x; i < WG_STAGES * 2 * pad16; i += blockDim.x) {
      const int region = i / pad16, j = i - region * pad16;
      *reinterpret_cast<uint4*>(base + (region / 2) * stage_bytes + (region % 2) * p.x_chunk_bytes + x_box + j * 16) = make_uint4(0, 0, 0, 0);
    }
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm->tmem_base;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == 0) {
    if (lane == 0) {
      const uint32_t tx = 2u * (uint32_t)x_box + 2u * (uint32_t)(p.P * p.R * 128);
      uint32_t s = 0, phase = 0;
      bool ok = true;
      for (int tile = first; tile < last && ok; tile++) {
        const int n = tile / p.tiles_h, h0 = (tile - n * p.tiles_h) * p.R;
        if (!(ok = mbar_wait_abortable(&sm->abort, &sm->empty[s], phase ^ 1, p.error, 1))) break;
        mbar_expect_tx(&sm->full[s], tx);
        uint8_t* st = base + s * stage_bytes;
        const uint32_t bar = smem_u32(&sm->full[s]);
        for (int c = 0; c < 2; c++) {
          tma_load_4d(smem_u32(st + c * p.x_chunk_bytes), &map_x, bar, cig * 128 + c * 64, -1, h0 - 1, n);
          tma_load_4d(smem_u32(st + 2 * p.x_chunk_bytes + c * p.dy_chunk_bytes), &map_dy, bar, cog * 128 + c * 64, 0, h0, n);
        }
        if (++s == WG_STAGES) { s = 0; phase ^= 1; }
      }
      if (!ok) {
        for (int i = 0; i < 1000; i++) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) | ((192u >> 3) << 17) | ((128u >> 4) << 24);
      const int ksteps = p.P * p.R / 16;
      uint32_t s = 0, phase = 0, acc = 0;
      bool ok = true;
      for (int tile = first; tile < last && ok; tile++) {
        if (!(ok = mbar_wait_abortable(&sm->abort, &sm->full[s], phase, p.error, 3))) break;
        tc_fence_after();
        const uint32_t xs = smem_u32(base + s * stage_bytes), ds = xs + 2 * p.x_chunk_bytes;
#pragma unroll 1
        for (int k = 0; k < ksteps; k++) {
          const uint32_t off = (uint32_t)k * 16u * 128u;
          const uint64_t da = smem_desc_mn_lbo(ds + off, (uint32_t)p.dy_chunk_bytes);
          const uint32_t xo = off + (uint32_t)(frow * p.P) * 128u;
          tc_mma(tmem_base, da, smem_desc_mn_lbo(xs + xo, 128u), idesc, acc);
          tc_mma(tmem_base + 192, da, smem_desc_mn_lbo(xs + p.x_chunk_bytes + xo, 128u), idesc, acc);
          acc = 1;
        }
        tc_commit(&sm->empty[s]);
        if (++s == WG_STAGES) { s = 0; phase ^= 1; }
      }
      if (ok) tc_commit(&sm->tmem_full[0]);
      tc_commit(&sm->drain);
      for (uint32_t it = 0; it < kSpinLimit; it++) if (mbar_try_wait(&sm->drain, 0)) break;
    }
  } else {
    const int q = warp & 3, ew = warp - 2, half = ew / 4;     // half = input-channel chunk: columns half * 192 ..
    bool ok = mbar_wait_abortable(&sm->abort, &sm->tmem_full[0], 0, p.error, 4);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      const int co = q * 32 + lane;
      // column c * 32 + j of this half is tap s = (c * 32 + j) / 64, input channel cig * 128 + half * 64 + (c * 32 + j) % 64
      float* dst = p.part + ((size_t)blockIdx.x * p.Co + cog * 128 + co) * (size_t)(9 * p.Ci) + (size_t)frow * 3 * p.Ci + cig * 128 + half * 64;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + half * 192;
#pragma unroll 1
      for (int c = 0; c < 6; c++) {
        uint32_t v[32];
        tc_ld32(taddr + c * 32, v);
        tc_wait_ld();
        float* o = dst + (c >> 1) * p.Ci + (c & 1) * 32;
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(o + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                          __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
      }
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// wt[ci][kh-1-r][kw-1-s][co] = w[co][r][s][ci]: the filter of the data-gradient convolution
__global__ void flip_weights_kernel(const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ wt, int Co, int kh,
                                    int kw, int Ci) {
  const size_t total = (size_t)Co * kh * kw * Ci;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    // i indexes the destination, so that writes are coalesced
    const int co = (int)(i % Co);
    size_t rest = i / Co;
    const int s = (int)(rest % kw); rest /= kw;
    const int r = (int)(rest % kh);
    const int ci = (int)(rest / kh);
    wt[i] = w[(((size_t)co * kh + (kh - 1 - r)) * kw + (kw - 1 - s)) * Ci + ci];
  }
}

// Filters of the four parity phases of the input gradient of a 3x3, stride-2, padding-1 convolution.
// w [Co][3][3][Ci] -> wp: phase (a, b) (a = row parity of the dX pixel, b = column parity) is a dense
// (1 + a) x (1 + b) filter [Ci][1 + a][1 + b][Co], its tap (u, v) reading dY at offset (+u, +v); the four
// filters lie behind one another at element offsets {0, 1, 3, 5} * Ci * Co.
__global__ void __launch_bounds__(256)
phase_weights_kernel(const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ wp, int Co, int Ci) {
  const size_t per = (size_t)Ci * Co;
  const size_t total = 9 * per;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    // i indexes wp: find the phase, then (ci, u, v, co)
    const size_t blk = i / per;                       // 0 | 1,2 | 3,4 | 5..8
    const int ph = blk < 1 ? 0 : (blk < 3 ? 1 : (blk < 5 ? 2 : 3));
    const int a = ph >> 1, b = ph & 1, kh = 1 + a, kw = 1 + b;
    const size_t base = (ph == 0 ? 0 : (ph == 1 ? 1 : (ph == 2 ? 3 : 5))) * per;
    size_t j = i - base;
    const int co = (int)(j % Co); j /= Co;
    const int v = (int)(j % kw); j /= kw;
    const int u = (int)(j % kh); j /= kh;
    const int ci = (int)j;
    const int r = a == 0 ? 1 : (u == 0 ? 2 : 0), sx = b == 0 ? 1 : (v == 0 ? 2 : 0);
    wp[i] = w[(((size_t)co * 3 + r) * 3 + sx) * Ci + ci];
  }
}

// ------------------------------------------------------------------- host side
// bf16 NHWC tensor as {C, W, H, N}; box = 64 channels x bw x bh x bn pixels.
// chunks > 0: five dimensions {64, W, H, N, C / 64}, the box also spans `chunks` 64-channel groups,
// which land 64 * bw * bh * bn * 2 bytes apart in shared memory (C must be a multiple of 64).
// step > 1: the box holds every step-th pixel along W and H (the map's element strides); its traversed extent is then
// (bw - 1) * step + 1 by (bh - 1) * step + 1.
static int make_map_nhwc(CUtensorMap* map, const void* ptr, uint64_t N, uint64_t H, uint64_t W, uint64_t C, uint32_t bw,
                         uint32_t bh, uint32_t bn, uint32_t chunks, uint32_t step = 1) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return -10;
  if (((uintptr_t)ptr & 15) || (C * 2) % 16) return -11;
  const uint32_t tw = (bw - 1) * step + 1, th = (bh - 1) * step + 1;
  if (tw > 256 || th > 256 || bn > 256 || (chunks && C % 64) || step < 1 || step > 8) return -11;
  cuuint64_t dims[5] = {chunks ? 64 : C, W, H, N, C / 64};
  cuuint64_t strides[4] = {C * 2, W * C * 2, H * W * C * 2, 128};
  cuuint32_t box[5] = {(cuuint32_t)BK, tw, th, bn, chunks};
  cuuint32_t estr[5] = {1, step, step, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, chunks ? 5 : 4, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -12;
}

// 2-D bf16 [rows][cols] row-major, box = 64 columns x box_rows
static int make_map_2d(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return -10;
  if (((uintptr_t)ptr & 15) || (cols * 2) % 16) return -11;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -12;
}

// Pixel box bw x bh x bn covering a W x H x N grid with the fewest wasted rows.
// `exact` != 0: the box must hold exactly `rows` pixels (wgrad: 64); else at most `rows`.
// Ties go to the longer contiguous run (larger bw, then bh). Returns the fraction of fetched rows that are pixels.
static double pick_box(int W, int H, int N, int rows, int exact, int* obw, int* obh, int* obn) {
  double best = -1.0, best_eff = 0.0;
  *obw = 1; *obh = 1; *obn = rows > 256 ? 256 : rows;
  for (int bw = 1; bw <= rows && bw <= 256; bw++) {
    if (bw > W + 7) break;
    for (int bh = 1; bw * bh <= rows && bh <= 256; bh++) {
      if (bh > H + 7) break;
      int bn = rows / (bw * bh);
      if (bn > N) bn = N;
      if (bn > 256) bn = 256;
      if (bn < 1) continue;
      if (exact && bw * bh * bn != rows) continue;
      const double covered = (double)((W + bw - 1) / bw) * bw * ((H + bh - 1) / bh) * bh * ((N + bn - 1) / bn) * bn;
      const double eff = ((double)W * H * N / covered) * ((double)(bw * bh * bn) / rows);
      const double score = eff + 1e-4 * bw + 1e-6 * bh;
      if (score > best) { best = score; best_eff = eff; *obw = bw; *obh = bh; *obn = bn; }
    }
  }
  return best_eff;
}

static size_t smem_for(int halves, int bn_cols, int stages) {
  return (size_t)stages * (halves * HALF_BYTES + bn_cols * BK * 2) + sizeof(Smem) + 16 + EPI_WARPS * kStageWarpBytes + 1024;
}

static int device_sms() {
  static std::once_flag once;
  static int sms = 148;
  std::call_once(once, [] {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int cap = kSmemBudget + 2048 + EPI_WARPS * kStageWarpBytes;
    cudaFuncSetAttribute(conv_igemm_kernel<false, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap);
    cudaFuncSetAttribute(conv_igemm_kernel<false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap);
    cudaFuncSetAttribute(conv_igemm_kernel<true, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap);
    cudaFuncSetAttribute(conv_igemm_kernel<true, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap);
    cudaFuncSetAttribute(conv_ws_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kWsSmemMax);
    cudaFuncSetAttribute(conv_wgrad_ws_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kWsSmemMax);
    cudaFuncSetAttribute(conv_halo_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kWsSmemMax);
    cudaFuncSetAttribute(conv_wgrad_halo_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kWsSmemMax);
  });
  return sms;
}

static int stages_for(int halves, int bn_cols) {
  int st = kSmemBudget / (halves * HALF_BYTES + bn_cols * BK * 2);
  st = st > MAX_STAGES ? MAX_STAGES : st;
  return st;
}

// Cycles of one reduction step as measured on B200: every TMA copy costs about 220 cycles plus its bytes at
// about 100 bytes per cycle, every M128 x N x K16 MMA about 128 cycles whatever N; the slower side wins.
static double step_cycles(int copies, double bytes, int mmas) {
  const double tma = 220.0 * copies + bytes / 100.0, mma = 128.0 * mmas;
  return tma > mma ? tma : mma;
}

// One or two 128-row accumulators per forward tile: fewer, larger copies against fewer tiles to spread over the SMs.
static int fwd_halves(int Wo, int Ho, int N, int tiles_c, int ksteps, int bn_cols, int sms) {
  double cost[3] = {0, 0, 0};
  for (int hv = 1; hv <= 2; hv++) {
    int bw, bh, bn;
    pick_box(Wo, Ho, N, 128 * hv, 0, &bw, &bh, &bn);
    const long long tiles = (long long)((Wo + bw - 1) / bw) * ((Ho + bh - 1) / bh) * ((N + bn - 1) / bn) * tiles_c;
    const long long waves = (tiles + sms - 1) / sms;
    cost[hv] = (double)waves * ksteps * step_cycles(2, hv * HALF_BYTES + bn_cols * 128.0, 4 * hv);
  }
  // two 256-column accumulators fill the tensor memory: the epilogue no longer overlaps the next tile, and the
  // 64 KB stages leave a ring of three (measured: 1.45 x the modelled step)
  if (bn_cols == 256) cost[2] *= 1.45;
  int halves = cost[2] < cost[1] ? 2 : 1;
  return halves;
}

struct WgradPlan { int bw, bh, bn, tiles_w, tiles_h, tiles_n, split, per, b_chunks, halves; };

static WgradPlan wgrad_plan(int N, int Ho, int Wo, int Ci, int Co, int taps, int sms) {
  WgradPlan q;
  pick_box(Wo, Ho, N, 64, 1, &q.bw, &q.bh, &q.bn);
  q.tiles_w = (Wo + q.bw - 1) / q.bw; q.tiles_h = (Ho + q.bh - 1) / q.bh; q.tiles_n = (N + q.bn - 1) / q.bn;
  const int chunks = q.tiles_w * q.tiles_h * q.tiles_n;
  q.halves = Co >= 256 ? 2 : 1;                                 // 256 output rows per tile share each X box
  const int base = ((Co + 128 * q.halves - 1) / (128 * q.halves)) * ((taps * Ci + 255) / 256);
  int split = sms / base;                                       // one wave: never more tiles than SMs
  if (split > (chunks + 7) / 8) split = (chunks + 7) / 8;      // at least 8 pixel boxes per CTA
  if (split < 1) split = 1;
  q.per = (chunks + split - 1) / split;
  q.split = (chunks + q.per - 1) / q.per;                       // no empty split
  const int cchunks = Ci / 64;
  q.b_chunks = cchunks % 4 == 0 ? 4 : (cchunks % 2 == 0 ? 2 : 1);
  return q;
}

}  // namespace conv
}  // namespace gcow

using namespace gcow::conv;

extern "C" {

// Whether forward tiles of 256 pixels x 128 channels take the operand-swapped MMA (default) or the plain one; the two
// agree up to the order of the fp32 sums, which is what the tests use this for.
static int g_swap_enabled = 1;
void gcow_conv_set_swap(int on) { g_swap_enabled = on ? 1 : 0; }

// The forward kernel in full generality: input window step `stride` (1 or 2), an output grid of Ho x Wo tile pixels
// whose pixel (h, w) is stored at (h * out_step + out_off_h, w * out_step + out_off_w) of y [N, out_H, out_W, Co].
static int conv_fwd_launch(const void* x, const void* w, void* y, const float* bias, int N, int Hin, int Win, int Ci, int Co,
                           int kh, int kw, int pad_h, int pad_w, int stride, int Ho, int Wo, int out_step, int out_off_h,
                           int out_off_w, int out_H, int out_W, uint32_t* error, void* stream) {
  if (N <= 0 || Ho <= 0 || Wo <= 0) return 0;
  if (Ci % 64 || Co % 8 || kh < 1 || kw < 1 || pad_h < 0 || pad_w < 0 || stride < 1 || stride > 2 || out_step < 1) return -1;
  if ((uintptr_t)y & 15) return -1;
  const int sms = device_sms();
  Params p{};
  p.bn_cols = Co <= 64 ? 64 : (Co <= 128 ? 128 : 256);
  const int tiles_c = (Co + p.bn_cols - 1) / p.bn_cols;
  const int ksteps = kh * kw * (Ci / 64);
  const int halves = fwd_halves(Wo, Ho, N, tiles_c, ksteps, p.bn_cols, sms);
  pick_box(Wo, Ho, N, 128 * halves, 0, &p.bw, &p.bh, &p.bn);
  p.tiles_w = (Wo + p.bw - 1) / p.bw; p.tiles_h = (Ho + p.bh - 1) / p.bh; p.tiles_n = (N + p.bn - 1) / p.bn;
  p.stages = stages_for(halves, p.bn_cols);
  p.out = y; p.bias = bias; p.N = N; p.H = Ho; p.W = Wo; p.Ci = Ci; p.Co = Co;
  p.kh = kh; p.kw = kw; p.pad_h = pad_h; p.pad_w = pad_w;
  p.split = 1; p.chunks_per_split = 0; p.b_chunks = 1;
  p.flags = bias ? kBias : 0;
  p.stride = stride;
  p.swap = (halves == 2 && p.bn_cols == 128 && Co % 8 == 0 && g_swap_enabled) ? 1 : 0;
  p.out_step = out_step; p.out_off_h = out_off_h; p.out_off_w = out_off_w; p.out_H = out_H; p.out_W = out_W;
  p.error = error;
  CUtensorMap ma, mb;
  int rc = make_map_nhwc(&ma, x, (uint64_t)N, (uint64_t)Hin, (uint64_t)Win, (uint64_t)Ci, p.bw, p.bh, p.bn, 0, (uint32_t)stride);
  if (rc) return rc;
  rc = make_map_2d(&mb, w, (uint64_t)Co, (uint64_t)kh * kw * Ci, (uint32_t)p.bn_cols);
  if (rc) return rc;
  const long long tiles = (long long)p.tiles_w * p.tiles_h * p.tiles_n * tiles_c;
  const int grid = (int)(tiles < sms ? tiles : sms);
  const size_t smem = smem_for(halves, p.bn_cols, p.stages);
  if (halves == 2) gcow::launch_dependent(conv_igemm_kernel<false, 2>, dim3(grid), dim3(THREADS), smem, (cudaStream_t)stream, ma, mb, p);
  else gcow::launch_dependent(conv_igemm_kernel<false, 1>, dim3(grid), dim3(THREADS), smem, (cudaStream_t)stream, ma, mb, p);
  return (int)cudaGetLastError();
}

// y[N,Ho,Wo,Co] = conv(x[N,Hin,Win,Ci], w[Co,kh,kw,Ci]) (+ bias), stride 1, zero padding (pad_h, pad_w);
// Ho = Hin + 2*pad_h - kh + 1. bf16, NHWC; Ci a multiple of 64, Co a multiple of 8.
// `error` is a device word that stays 0 unless a wait gave up. Returns 0, a negative argument error or a CUDA error.
int gcow_conv_fwd(const void* x, const void* w, void* y, const float* bias, int N, int Hin, int Win, int Ci, int Co,
                  int kh, int kw, int pad_h, int pad_w, uint32_t* error, void* stream) {
  const int Ho = Hin + 2 * pad_h - kh + 1, Wo = Win + 2 * pad_w - kw + 1;
  return conv_fwd_launch(x, w, y, bias, N, Hin, Win, Ci, Co, kh, kw, pad_h, pad_w, 1, Ho, Wo, 1, 0, 0, Ho, Wo, error, stream);
}

// The same with the window moved `stride` (1 or 2) input pixels per output pixel: Ho = (Hin + 2*pad_h - kh) / stride + 1.
int gcow_conv_fwd_strided(const void* x, const void* w, void* y, const float* bias, int N, int Hin, int Win, int Ci, int Co,
                          int kh, int kw, int pad_h, int pad_w, int stride, uint32_t* error, void* stream) {
  if (stride < 1 || stride > 2) return -1;
  const int Ho = (Hin + 2 * pad_h - kh) / stride + 1, Wo = (Win + 2 * pad_w - kw) / stride + 1;
  return conv_fwd_launch(x, w, y, bias, N, Hin, Win, Ci, Co, kh, kw, pad_h, pad_w, stride, Ho, Wo, 1, 0, 0, Ho, Wo, error, stream);
}

// Whether gcow_conv_fwd_ws takes these extents (64 -> 64 channels, 3x3, stride 1, padding 1 are implied).
int gcow_conv_ws_usable(int N, int H, int W) {
  return N > 0 && H > 0 && W >= 6 && W + 2 <= 128;
}

// y[N,H,W,64] = conv3x3(x[N,H,W,64], w[64,3,3,64]) (+ bias), stride 1, padding 1, on the weight-stationary kernel
// (pixels as the MMA's N). With w = the flipped filter [ci][2-r][2-s][co] and x = dY it is the input gradient.
int gcow_conv_fwd_ws(const void* x, const void* w, void* y, const float* bias, int N, int H, int W, uint32_t* error,
                     void* stream) {
  if (!gcow_conv_ws_usable(N, H, W)) return -1;
  if (((uintptr_t)y & 1) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return -1;
  const int sms = device_sms();
  WsParams p{};
  p.out = (__nv_bfloat16*)y; p.bias = bias; p.N = N; p.H = H; p.W = W;
  p.pitch = W + 2;
  p.rows = 256 / p.pitch;
  if (p.rows > H) p.rows = H;
  p.nslots = (p.rows * p.pitch + 15) & ~15;
  p.tiles_h = (H + p.rows - 1) / p.rows;
  // a stage holds the copied box; the taps of the last pixel slots read up to 2 * pitch + 2 rows further, into the
  // next stage or the epilogue's staging buffers: sums of slots that are never stored
  p.stage_bytes = (p.pitch * (p.rows + 2) * 128 + 1023) & ~1023;
  const int tail = 16 + EPI_WARPS * kStageWarpBytes;
  const int reach = (256 + 2 * p.pitch + 2) * 128 - tail;        // what the last stage itself must cover
  if (p.stage_bytes < reach) p.stage_bytes = (reach + 1023) & ~1023;
  int st = (kWsSmemMax - 1024 - WS_W_BYTES - (int)sizeof(WsSmem) - tail) / p.stage_bytes;
  if (st > 4) st = 4;
  if (st < 2) return -1;
  p.stages = st;
  p.error = error;
  CUtensorMap mx, mw;
  int rc = make_map_nhwc(&mx, x, (uint64_t)N, (uint64_t)H, (uint64_t)W, 64, (uint32_t)p.pitch, (uint32_t)(p.rows + 2), 1, 0);
  if (rc) return rc;
  rc = make_map_2d(&mw, w, 64, (uint64_t)WS_TAPS * 64, 64);
  if (rc) return rc;
  const long long tiles = (long long)N * p.tiles_h;
  const int grid = (int)(tiles < sms ? tiles : sms);
  const size_t smem = 1024 + WS_W_BYTES + (size_t)st * p.stage_bytes + sizeof(WsSmem) + tail;
  gcow::launch_dependent(conv_ws_kernel, dim3(grid), dim3(THREADS), smem, (cudaStream_t)stream, mx, mw, p);
  return (int)cudaGetLastError();
}

// Tile geometry of the halo-tile forward for Ci -> 128 channels; false when it does not apply or does not fit.
static bool halo_plan(int N, int H, int W, int Ci, HaloParams* p) {
  if (N <= 0 || H <= 0 || W < 6 || W + 2 > 128 || Ci < 64 || Ci % 64) return false;
  p->N = N; p->H = H; p->W = W; p->Ci = Ci;
  p->pitch = W + 2;
  // image rows per tile: the fewest MMA columns over the whole image
  long best = -1;
  for (int rows = 1; rows * p->pitch <= 256 && rows <= H; rows++) {
    const int ns = (rows * p->pitch + 15) & ~15;
    const long cost = (long)((H + rows - 1) / rows) * ns;
    if (best < 0 || cost <= best) { best = cost; p->rows = rows; p->nslots = ns; }
  }
  if (best < 0) return false;
  p->tiles_h = (H + p->rows - 1) / p->rows;
  p->chunk_bytes = ((p->nslots + 2 * p->pitch + 2) * 128 + 1023) & ~1023;
  p->a_stages = 2;
  const int fixed = 1024 + (int)sizeof(HaloSmem) + 16 + EPI_WARPS * kStageWarpBytes;
  const int left = kWsSmemMax - fixed - p->a_stages * (Ci / 64) * p->chunk_bytes;
  p->b_stages = left / HALO_B_BYTES;
  if (p->b_stages > 8) p->b_stages = 8;
  return p->b_stages >= 3;
}

int gcow_conv_halo_usable(int N, int H, int W, int Ci) {
  HaloParams p{};
  return halo_plan(N, H, W, Ci, &p) ? 1 : 0;
}

// y[N,H,W,128] = conv3x3(x[N,H,W,Ci], w[128,3,3,Ci]) (+ bias), stride 1, padding 1, on the halo-tile kernel.
int gcow_conv_fwd_halo(const void* x, const void* w, void* y, const float* bias, int N, int H, int W, int Ci, uint32_t* error,
                       void* stream) {
  HaloParams p{};
  if (!halo_plan(N, H, W, Ci, &p) || ((uintptr_t)y & 15)) return -1;
  const int sms = device_sms();
  p.out = (__nv_bfloat16*)y; p.bias = bias; p.error = error;
  CUtensorMap mx, mw;
  int rc = make_map_nhwc(&mx, x, (uint64_t)N, (uint64_t)H, (uint64_t)W, (uint64_t)Ci, (uint32_t)p.pitch, (uint32_t)(p.rows + 2), 1, 0);
  if (rc) return rc;
  rc = make_map_2d(&mw, w, 128, (uint64_t)WS_TAPS * Ci, 128);
  if (rc) return rc;
  const long long tiles = (long long)N * p.tiles_h;
  const int grid = (int)(tiles < sms ? tiles : sms);
  const size_t smem = 1024 + (size_t)p.a_stages * (Ci / 64) * p.chunk_bytes + (size_t)p.b_stages * HALO_B_BYTES +
                      sizeof(HaloSmem) + 16 + EPI_WARPS * kStageWarpBytes;
  gcow::launch_dependent(conv_halo_kernel, dim3(grid), dim3(THREADS), smem, (cudaStream_t)stream, mx, mw, p);
  return (int)cudaGetLastError();
}

// Whether gcow_conv_wgrad_ws takes these extents, and how many partial results it writes (0: not usable).
int gcow_conv_wgrad_ws_split(int N, int H, int W) {
  if (N <= 0 || H <= 0 || W < 1 || W + 2 > 64) return 0;
  const int sms = device_sms();
  const long long tiles = (long long)N * ((H + 3) / 4);
  if (tiles > (1ll << 30)) return 0;
  const int per = (int)((tiles + sms - 1) / sms);
  return (int)((tiles + per - 1) / per);
}

// part[split][64][9 * 64] (fp32) = partial sums of dy[N,H,W,64]^T * shifted x[N,H,W,64] for a 3x3 filter with padding 1,
// split = gcow_conv_wgrad_ws_split(N, H, W); the caller adds the slices (gcow_reduce_partials).
int gcow_conv_wgrad_ws(const void* dy, const void* x, float* part, int N, int H, int W, uint32_t* error, void* stream) {
  const int split = gcow_conv_wgrad_ws_split(N, H, W);
  if (split <= 0 || ((uintptr_t)part & 15)) return -1;
  WsWgradParams p{};
  p.part = part; p.N = N; p.H = H; p.W = W;
  p.tiles_h = (H + 3) / 4;
  p.num_tiles = N * p.tiles_h;
  p.per = (p.num_tiles + split - 1) / split;
  p.error = error;
  CUtensorMap mx, md;
  int rc = make_map_nhwc(&mx, x, (uint64_t)N, (uint64_t)H, (uint64_t)W, 64, 64, 6, 1, 0);
  if (rc) return rc;
  rc = make_map_nhwc(&md, dy, (uint64_t)N, (uint64_t)H, (uint64_t)W, 64, 64, 6, 1, 0);
  if (rc) return rc;
  const size_t smem = 1024 + (size_t)WG_STAGES * WG_STAGE_BYTES + sizeof(WsSmem) + 64;
  gcow::launch_dependent(conv_wgrad_ws_kernel, dim3(split), dim3(THREADS), smem, (cudaStream_t)stream, mx, md, p);
  return (int)cudaGetLastError();
}

// Geometry of the halo-tile weight gradient for channel counts that are multiples of 128; split = 0: not usable.
static int wgrad_halo_plan(int N, int H, int W, int Ci, int Co, WgHaloParams* p) {
  if (N <= 0 || H <= 0 || W < 1 || W + 2 > 64 || Ci < 128 || Ci % 128 || Co < 128 || Co % 128) return 0;
  p->N = N; p->H = H; p->W = W; p->Ci = Ci; p->Co = Co;
  p->P = W + 2 <= 16 ? 16 : (W + 2 <= 32 ? 32 : 64);
  p->R = p->P == 16 ? 7 : (p->P == 32 ? 4 : 2);   // two stages of two X and two dY boxes fit the shared memory
  p->tiles_h = (H + p->R - 1) / p->R;
  const long long tiles = (long long)N * p->tiles_h;
  if (tiles > (1ll << 30)) return 0;
  p->num_tiles = (int)tiles;
  const int per_tile = 3 * (Ci / 128) * (Co / 128);   // CTAs per range of tiles: filter rows x channel blocks
  if (per_tile > 65535) return 0;
  int groups = device_sms() / per_tile;
  if (groups < 1) groups = 1;
  p->per = (int)((tiles + groups - 1) / groups);
  p->x_chunk_bytes = (p->P * (p->R + 2) * 128 + 256 + 1023) & ~1023;
  p->dy_chunk_bytes = p->P * p->R * 128;
  return (int)((tiles + p->per - 1) / p->per);
}

int gcow_conv_wgrad_halo_split(int N, int H, int W, int Ci, int Co) {
  WgHaloParams p{};
  return wgrad_halo_plan(N, H, W, Ci, Co, &p);
}

// part[split][Co][9 * Ci] (fp32) = partial sums of dy[N,H,W,Co]^T * shifted x[N,H,W,Ci], 3x3, padding 1;
// split = gcow_conv_wgrad_halo_split(N, H, W, Ci, Co); the caller adds the slices.
int gcow_conv_wgrad_halo(const void* dy, const void* x, float* part, int N, int H, int W, int Ci, int Co, uint32_t* error,
                         void* stream) {
  WgHaloParams p{};
  const int split = wgrad_halo_plan(N, H, W, Ci, Co, &p);
  if (split <= 0 || ((uintptr_t)part & 15)) return -1;
  p.part = part; p.error = error;
  CUtensorMap mx, md;
  int rc = make_map_nhwc(&mx, x, (uint64_t)N, (uint64_t)H, (uint64_t)W, (uint64_t)Ci, (uint32_t)p.P, (uint32_t)(p.R + 2), 1, 0);
  if (rc) return rc;
  rc = make_map_nhwc(&md, dy, (uint64_t)N, (uint64_t)H, (uint64_t)W, (uint64_t)Co, (uint32_t)p.P, (uint32_t)p.R, 1, 0);
  if (rc) return rc;
  const size_t smem = 1024 + (size_t)WG_STAGES * (2 * p.x_chunk_bytes + 2 * p.dy_chunk_bytes) + sizeof(WsSmem) + 64;
  if (smem > (size_t)kWsSmemMax) return -1;
  gcow::launch_dependent(conv_wgrad_halo_kernel, dim3(split, 3 * (Ci / 128) * (Co / 128)), dim3(THREADS), smem, (cudaStream_t)stream, mx, md, p);
  return (int)cudaGetLastError();
}

// Input gradient of a 3x3, stride-2, padding-1 convolution with even input extents: dx[N,Hin,Win,Ci] from
// dy[N,Hin/2,Win/2,Co] and w[Co,3,3,Ci]. `wp` is scratch of 9*Ci*Co bf16 for the four phase filters. Four launches of
// the forward kernel, one per parity of the dx pixel; together they write every pixel of dx exactly once.
int gcow_conv_dgrad_s2(const void* dy, const void* w, void* wp, void* dx, int N, int Hin, int Win, int Ci, int Co,
                       uint32_t* error, void* stream) {
  if (Hin % 2 || Win % 2 || Ci % 64 || Co % 64 || N <= 0) return -1;
  const int Ho = Hin / 2, Wo = Win / 2;
  const size_t per = (size_t)Ci * Co;
  int blocks = (int)((9 * per + 255) / 256);
  if (blocks > 1184) blocks = 1184;
  phase_weights_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)w, (__nv_bfloat16*)wp, Co, Ci);
  int rc = (int)cudaGetLastError();
  if (rc) return rc;
  const size_t off[4] = {0, 1, 3, 5};
  for (int ph = 0; ph < 4; ph++) {
    const int a = ph >> 1, b = ph & 1;
    // dY is the input (its channels Co are reduced), dX's channels Ci are the outputs; taps read dY at (+u, +v)
    rc = conv_fwd_launch(dy, (const __nv_bfloat16*)wp + off[ph] * per, dx, nullptr, N, Ho, Wo, Co, Ci, 1 + a, 1 + b, 0, 0, 1,
                         Ho, Wo, 2, a, b, Hin, Win, error, stream);
    if (rc) return rc;
  }
  return 0;
}

// Input gradient of a 1x1 convolution with stride 2: dx[N,Hin,Win,Ci] is dy[N,Ho,Wo,Co] * wt at the sampled pixels
// (every second pixel of every second row) and zero elsewhere. wt [Ci][Co] is the transposed filter.
int gcow_conv_dgrad_1x1_s2(const void* dy, const void* wt, void* dx, int N, int Hin, int Win, int Ci, int Co,
                           uint32_t* error, void* stream) {
  if (Ci % 8 || Co % 64 || N <= 0 || Hin <= 0 || Win <= 0) return -1;
  const int Ho = (Hin - 1) / 2 + 1, Wo = (Win - 1) / 2 + 1;
  int rc = (int)cudaMemsetAsync(dx, 0, (size_t)N * Hin * Win * Ci * 2, (cudaStream_t)stream);
  if (rc) return rc;
  return conv_fwd_launch(dy, wt, dx, nullptr, N, Ho, Wo, Co, Ci, 1, 1, 0, 0, 1, Ho, Wo, 2, 0, 0, Hin, Win, error, stream);
}

// Number of fp32 partial results gcow_conv_wgrad writes for these extents (the first dimension of `part`).
int gcow_conv_wgrad_split_strided(int N, int Hin, int Win, int Ci, int Co, int kh, int kw, int pad_h, int pad_w, int stride) {
  if (stride < 1 || stride > 2) return 0;
  const int Ho = (Hin + 2 * pad_h - kh) / stride + 1, Wo = (Win + 2 * pad_w - kw) / stride + 1;
  if (N <= 0 || Ho <= 0 || Wo <= 0) return 0;
  return wgrad_plan(N, Ho, Wo, Ci, Co, kh * kw, device_sms()).split;
}
int gcow_conv_wgrad_split(int N, int Hin, int Win, int Ci, int Co, int kh, int kw, int pad_h, int pad_w) {
  return gcow_conv_wgrad_split_strided(N, Hin, Win, Ci, Co, kh, kw, pad_h, pad_w, 1);
}

// part[split][Co][kh*kw*Ci] (fp32) = partial sums over pixel ranges of dy[N,Ho,Wo,Co]^T * shifted x[N,Hin,Win,Ci];
// the caller adds the `split` slices (gcow_reduce_partials). Ci and Co multiples of 64.
int gcow_conv_wgrad_strided(const void* dy, const void* x, float* part, int N, int Hin, int Win, int Ci, int Co, int kh, int kw,
                            int pad_h, int pad_w, int stride, uint32_t* error, void* stream) {
  if (stride < 1 || stride > 2) return -1;
  const int Ho = (Hin + 2 * pad_h - kh) / stride + 1, Wo = (Win + 2 * pad_w - kw) / stride + 1;
  if (N <= 0 || Ho <= 0 || Wo <= 0) return 0;
  if (Ci % 64 || Co % 64 || kh < 1 || kw < 1 || pad_h < 0 || pad_w < 0) return -1;
  if ((uintptr_t)part & 15) return -1;
  const int sms = device_sms();
  const WgradPlan q = wgrad_plan(N, Ho, Wo, Ci, Co, kh * kw, sms);
  Params p{};
  p.bw = q.bw; p.bh = q.bh; p.bn = q.bn; p.tiles_w = q.tiles_w; p.tiles_h = q.tiles_h; p.tiles_n = q.tiles_n;
  p.bn_cols = 256;
  p.stages = stages_for(q.halves, p.bn_cols);
  p.out = part; p.bias = nullptr; p.N = N; p.H = Ho; p.W = Wo; p.Ci = Ci; p.Co = Co;
  p.kh = kh; p.kw = kw; p.pad_h = pad_h; p.pad_w = pad_w;
  p.split = q.split; p.chunks_per_split = q.per; p.b_chunks = q.b_chunks;
  p.flags = 0;
  p.stride = stride;
  p.out_step = 1; p.out_off_h = 0; p.out_off_w = 0; p.out_H = Ho; p.out_W = Wo;
  p.error = error;
  CUtensorMap ma, mb;
  int rc = make_map_nhwc(&ma, dy, (uint64_t)N, (uint64_t)Ho, (uint64_t)Wo, (uint64_t)Co, q.bw, q.bh, q.bn, 2u * q.halves);
  if (rc) return rc;
  rc = make_map_nhwc(&mb, x, (uint64_t)N, (uint64_t)Hin, (uint64_t)Win, (uint64_t)Ci, q.bw, q.bh, q.bn, (uint32_t)q.b_chunks,
                     (uint32_t)stride);
  if (rc) return rc;
  const long long tiles = (long long)q.split * ((Co + 128 * q.halves - 1) / (128 * q.halves)) * ((kh * kw * Ci + 255) / 256);
  const int grid = (int)(tiles < sms ? tiles : sms);
  const size_t smem = smem_for(q.halves, p.bn_cols, p.stages);
  if (q.halves == 2) gcow::launch_dependent(conv_igemm_kernel<true, 2>, dim3(grid), dim3(THREADS), smem, (cudaStream_t)stream, ma, mb, p);
  else gcow::launch_dependent(conv_igemm_kernel<true, 1>, dim3(grid), dim3(THREADS), smem, (cudaStream_t)stream, ma, mb, p);
  return (int)cudaGetLastError();
}

int gcow_conv_wgrad(const void* dy, const void* x, float* part, int N, int Hin, int Win, int Ci, int Co, int kh, int kw,
                    int pad_h, int pad_w, uint32_t* error, void* stream) {
  return gcow_conv_wgrad_strided(dy, x, part, N, Hin, Win, Ci, Co, kh, kw, pad_h, pad_w, 1, error, stream);
}

// wt[Ci][kh][kw][Co] = w[Co][kh][kw][Ci] rotated by 180 degrees: with it, the gradient with respect to the input of a
// stride-1 convolution is gcow_conv_fwd(dy, wt, ..., Ci = Co, Co = Ci, pad = k - 1 - pad).
int gcow_conv_flip_weights(const void* w, void* wt, int Co, int kh, int kw, int Ci, void* stream) {
  const size_t total = (size_t)Co * kh * kw * Ci;
  if (!total) return 0;
  int blocks = (int)((total + 255) / 256);
  if (blocks > 1184) blocks = 1184;
  flip_weights_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)w, (__nv_bfloat16*)wt, Co, kh, kw, Ci);
  return (int)cudaGetLastError();
}

// The forward tiling the launcher would choose on a device with `sms` SMs: out = {accumulators per tile (1 or 2),
// columns per tile, bw, bh, bn, pipeline stages}. For tests and tuning; needs no GPU.
void gcow_conv_fwd_plan(int N, int Hin, int Win, int Ci, int Co, int kh, int kw, int pad_h, int pad_w, int sms, int* out) {
  const int Ho = Hin + 2 * pad_h - kh + 1, Wo = Win + 2 * pad_w - kw + 1;
  const int bn_cols = Co <= 64 ? 64 : (Co <= 128 ? 128 : 256);
  const int halves = fwd_halves(Wo, Ho, N, (Co + bn_cols - 1) / bn_cols, kh * kw * (Ci / 64), bn_cols, sms);
  out[0] = halves; out[1] = bn_cols;
  pick_box(Wo, Ho, N, 128 * halves, 0, &out[2], &out[3], &out[4]);
  out[5] = stages_for(halves, bn_cols);
}

// The pixel box chosen for given extents: out = {bw, bh, bn}. For tests of the tiling rule.
void gcow_conv_pick_box(int W, int H, int N, int rows, int exact, int* out) {
  pick_box(W, H, N, rows, exact, &out[0], &out[1], &out[2]);
}

}  // extern "C"
