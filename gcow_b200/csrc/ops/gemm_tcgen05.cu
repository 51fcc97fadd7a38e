// bf16 GEMM on the 5th-generation tensor cores (sm_100a): C[M,N] = A[M,K] * B[N,K]^T
// with fp32 accumulation in tensor memory and a fused epilogue.
//
// Persistent, warp-specialised kernel, one CTA per SM, in two tile shapes:
//   256x256 (default): A 256x64 + B 256x64 per stage (64 KB, 3 stages). Each K step issues
//            two M128 N256 K16 MMAs that share the B tile, one per 128-row half; the two
//            fp32 accumulators fill all 512 TMEM columns. Twice the flops per byte fetched
//            from L2 compared with 128x256 - the kernel is bound by the per-SM L2->shared
//            bandwidth, not by the tensor pipe. Eight epilogue warps drain half 0 then half
//            1, releasing each half separately so the next tile's MMAs restart early.
//   128x256 (small M): A 128x64 + B 256x64 per stage (48 KB, 4 stages), two 128x256
//            accumulators used alternately so the epilogue fully overlaps the next tile.
//   warp 0      TMA producer: cp.async.bulk.tensor tiles, 128-byte swizzle, mbarrier tx counts;
//   warp 1      allocates the 512 TMEM columns; one elected thread issues tcgen05.mma
//               (kind::f16) from shared-memory descriptors; tcgen05.commit releases ring
//               stages and publishes finished accumulators;
//   warps 2+    epilogue: tcgen05.ld their 32-lane quarter of the accumulator, add bias /
//               residual, optional GELU, convert and store.
// Each operand may be K-major (stored [rows][K], the layout of activations and
// of nn.Linear / 1x1-convolution weights in the forward product) or MN-major
// (stored [K][rows]); the backward products dX = dY*W and dW = dY^T*X read the
// same tensors with the other major-ness, so no transposed copy is ever made.
// An MN-major tile is fetched as 64-column boxes of 64 K-rows each (8 KB apart).
// No TMA multicast is used anywhere. Every mbarrier wait is bounded: after a fixed
// number of polls the CTA raises an error word, all roles leave their loops,
// outstanding MMAs are drained (bounded), TMEM is freed and the kernel returns.
//
// Replaces the cuBLAS GEMMs behind nn.Linear / 1x1 convolutions in the
// reference's models (hw/models/resenet.py:11,17,90).
#include <stdio.h>
#include <string.h>
#include <stdlib.h>
#include <mutex>

#include "pdl.cuh"
#include "tc_common.cuh"

namespace gcow {
namespace gemm {

constexpr int BN = 256, BK = 64, UMMA_K = 16;
constexpr int B_BYTES = BN * BK * 2;
constexpr int MAX_STAGES = 4;
constexpr uint32_t TMEM_COLS = 512;

template <int BM_> struct Shape {
  static constexpr int BM = BM_;
  static constexpr int HALVES = BM_ / 128;                 // 128-row accumulators per tile
  static constexpr int STAGES = BM_ == 256 ? 3 : 4;
  static constexpr int A_BYTES = BM_ * BK * 2;
  static constexpr int EPI_WARPS = 8;                      // two warps per TMEM lane quarter, half the columns each
  static constexpr int THREADS = 64 + 32 * EPI_WARPS;
  static constexpr size_t SMEM = (size_t)STAGES * (A_BYTES + B_BYTES);
};

enum Flags : int { kOutF32 = 1, kBias = 2, kGelu = 4, kResidual = 8, kAccumulate = 16,
                   kAuxOut = 32,     // bf16 output only: also store the value before GELU to aux (what the GELU gradient needs)
                   kGeluGrad = 64 }; // bf16 output only: multiply by GELU'(aux) - the gradient through a fused GELU

struct Params {
  void* C;                 // bf16 or fp32 [M, ldc]
  const float* bias;       // [N] fp32 or nullptr
  const void* residual;    // same type/ld as C or nullptr
  void* aux;               // bf16, same shape/ld as C: written (kAuxOut) or read (kGeluGrad)
  int M, N, K, ldc, flags;
  int batch;               // number of independent products (operands are 3-D tensor maps when > 1)
  int a_merged, b_merged;  // MN-major operand fetched as ONE box per stage (its row length is a multiple of 64)
  int a_chunks, b_chunks;  // 64-row groups of the A / B tile that exist in the matrix (a narrow operand is fetched with
  uint32_t stage_tx;       // a smaller box: the rest of its tile is never read back); bytes both copies of a stage bring
  int tma_store;           // bf16 C without residual / aux: the epilogue hands 32 x 32 boxes to the TMA (tmap_c is valid)
  long long stride_c;      // elements between consecutive C (and residual) matrices
  uint32_t* error;         // device word, set non-zero when a wait gave up
};

struct Smem {
  uint64_t full[MAX_STAGES], empty[MAX_STAGES], tmem_full[2], tmem_empty[2], drain;
  uint32_t tmem_base;
  volatile uint32_t abort;
};

using namespace gcow::tc;

// Merged MN-major fetch: the matrix [K][rows] is described as {64 elements, K, rows / 64 (, batch)}, so one
// box {64, 64, tile rows / 64} brings every 64-column group of the tile, 8 KB apart, in a single copy.
__device__ __forceinline__ void tma_load_mn(uint32_t dst, const CUtensorMap* map, uint32_t bar, int k, int chunk, int z,
                                            bool batched) {
  if (batched) tma_load_4d(dst, map, bar, 0, k, chunk, z);
  else tma_load_3d(dst, map, bar, 0, k, chunk);
}

__device__ __forceinline__ bool mbar_wait(Smem* sm, uint64_t* bar, uint32_t parity, uint32_t* error, uint32_t code) {
  return mbar_wait_abortable(&sm->abort, bar, parity, error, code);
}

template <int BM_, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(Shape<BM_>::THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_c, const Params p) {
  using S = Shape<BM_>;
  constexpr int BM = S::BM, STAGES = S::STAGES, A_BYTES = S::A_BYTES, HALVES = S::HALVES, EPI_WARPS = S::EPI_WARPS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* smA = base;
  uint8_t* smB = base + STAGES * A_BYTES;
  Smem* sm = reinterpret_cast<Smem*>(base + STAGES * (A_BYTES + B_BYTES));
  // per-warp staging buffers of the epilogue (two each) behind the barriers; 512-byte aligned, because their layout
  // (tc::stage_offset) is the 64-byte swizzle of the output tensor map, which is a function of the address
  uint8_t* stage_base = reinterpret_cast<uint8_t*>(((uintptr_t)(sm + 1) + 511) & ~(uintptr_t)511);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
  const int tiles_mn = tiles_m * tiles_n;
  const int num_tiles = tiles_mn * p.batch;
  const bool batched = p.batch > 1;
  const int kblocks = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(&sm->full[s], 1); mbar_init(&sm->empty[s], 1); }
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
  // a kernel launched as a programmatic dependent (the ordered sum of split partial results) may be scheduled
  // from here on; it waits for this grid to complete before it reads anything
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // ... and this grid, when it was launched the same way, has come this far (barriers, tensor memory) under the tail
  // of ITS predecessor: nothing in global memory is touched before that one has completed
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t s = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int bz = tile / tiles_mn, tmn = tile - bz * tiles_mn;
        const int m0 = (tmn % tiles_m) * BM, n0 = (tmn / tiles_m) * BN;
        for (int kb = 0; kb < kblocks; kb++) {
          if (!(ok = mbar_wait(sm, &sm->empty[s], phase ^ 1, p.error, 1))) break;
          mbar_expect_tx(&sm->full[s], p.stage_tx);
          const uint32_t bar = smem_u32(&sm->full[s]);
          if (!A_MN) {
            tma_load(smem_u32(smA + s * A_BYTES), &tmap_a, bar, kb * BK, m0, bz, batched);
          } else if (p.a_merged) {
            tma_load_mn(smem_u32(smA + s * A_BYTES), &tmap_a, bar, kb * BK, m0 / 64, bz, batched);
          } else {
            for (int i = 0; i < p.a_chunks; i++)
              tma_load(smem_u32(smA + s * A_BYTES + i * 8192), &tmap_a, bar, m0 + 64 * i, kb * BK, bz, batched);
          }
          if (!B_MN) {
            tma_load(smem_u32(smB + s * B_BYTES), &tmap_b, bar, kb * BK, n0, bz, batched);
          } else if (p.b_merged) {
            tma_load_mn(smem_u32(smB + s * B_BYTES), &tmap_b, bar, kb * BK, n0 / 64, bz, batched);
          } else {
            for (int i = 0; i < p.b_chunks; i++)
              tma_load(smem_u32(smB + s * B_BYTES + i * 8192), &tmap_b, bar, n0 + 64 * i, kb * BK, bz, batched);
          }
          if (++s == STAGES) { s = 0; phase ^= 1; }
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
      // instruction descriptor: fp32 accumulate, bf16 x bf16, operand major-ness, N256 M128
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)A_MN << 15) | ((uint32_t)B_MN << 16) |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      uint32_t s = 0, phase = 0, t = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, t++) {
        // HALVES == 1: accumulators alternate per tile. HALVES == 2: both are used by every tile.
        const uint32_t acc0 = HALVES == 1 ? (t & 1) : 0, aphase = HALVES == 1 ? ((t >> 1) & 1) : (t & 1);
        for (int kb = 0; kb < kblocks && ok; kb++) {
          if (!(ok = mbar_wait(sm, &sm->full[s], phase, p.error, 3))) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smA + s * A_BYTES), sb = smem_u32(smB + s * B_BYTES);
          const uint64_t db = B_MN ? smem_desc_mn_sw128(sb) : smem_desc_sw128(sb);
          // one K step of 16: 32 bytes along a K-major row, 16 rows (2048 bytes) of an MN-major tile
          constexpr uint64_t ka = A_MN ? (2048 >> 4) : (32 >> 4), kbs = B_MN ? (2048 >> 4) : (32 >> 4);
#pragma unroll
          for (int h = 0; h < HALVES; h++) {
            if (kb == 0) {   // first write to this accumulator: its previous contents must have been read out
              if (!(ok = mbar_wait(sm, &sm->tmem_empty[acc0 + h], aphase ^ 1, p.error, 2))) break;
              tc_fence_after();
            }
            // 128 rows of A are 16 KB in either layout (128 rows x 128 B, or two 64-column boxes)
            const uint64_t da = A_MN ? smem_desc_mn_sw128(sa + h * 16384) : smem_desc_sw128(sa + h * 16384);
            const uint32_t d_tmem = tmem_base + (acc0 + h) * BN;
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; k++)
              tc_mma(d_tmem, da + ka * k, db + kbs * k, idesc, (kb | k) != 0);
          }
          if (!ok) break;
          tc_commit(&sm->empty[s]);
          if (++s == STAGES) { s = 0; phase ^= 1; }
        }
        if (ok) tc_commit(&sm->tmem_full[acc0]);
      }
      // drain: everything issued by this thread has finished before TMEM is freed
      tc_commit(&sm->drain);
      for (uint32_t it = 0; it < kSpinLimit; it++) if (mbar_try_wait(&sm->drain, 0)) break;
    }
  } else {
    // ----------------------------------------------------------------- epilogue
    const int q = warp & 3;                       // TMEM lane quarter this warp may read
    const int ew = warp - 2;                      // 0 .. EPI_WARPS-1
    constexpr int COLS = BN / (EPI_WARPS / 4);    // columns of each accumulator this warp drains
    const int col0 = (ew / 4) * COLS;
    uint32_t t = 0;
    int sbuf = 0;                                 // staging buffer of the next TMA store
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, t++) {
      const int bz = tile / tiles_mn, tmn = tile - bz * tiles_mn;
      const int m0 = (tmn % tiles_m) * BM, n0 = (tmn / tiles_m) * BN;
      const uint32_t acc0 = HALVES == 1 ? (t & 1) : 0, aphase = HALVES == 1 ? ((t >> 1) & 1) : (t & 1);
      ok = mbar_wait(sm, &sm->tmem_full[acc0], aphase, p.error, 4);
      ok = __all_sync(0xffffffffu, ok);   // the tensor-memory loads below need the whole warp
      if (!ok) break;
      tc_fence_after();
#pragma unroll 1
      for (int h = 0; h < HALVES; h++) {
        const int m = m0 + h * 128 + q * 32 + lane;
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (acc0 + h) * BN + col0;
        // Tensor-memory loads are software pipelined: the load of chunk c+1 is in flight
        // while chunk c is converted and stored.
        auto process = [&](const uint32_t (&r)[32], int c) {
          const int n = n0 + col0 + c * 32;
          if (p.tma_store && n + 32 <= p.N && m0 + h * 128 + q * 32 < p.M) {
            // The warp's 32 x 32 block goes to its staging buffer in the output map's swizzle and one lane hands it to
            // the TMA, which clips rows past M. Two buffers alternate: a buffer is rewritten only after the store
            // issued from it two blocks ago has finished reading it.
            uint8_t* stg = stage_base + (ew * 2 + sbuf) * kStageWarpBytes;
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[j]);
            if (p.flags & kBias) {
#pragma unroll
              for (int j = 0; j < 32; j++) v[j] += __ldg(p.bias + n + j);
            }
            if (p.flags & kGelu) {
#pragma unroll
              for (int j = 0; j < 32; j++) v[j] = gelu_f(v[j]);
            }
#pragma unroll
            for (int k = 0; k < 4; k++) {
              uint4 o;
              __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
              for (int e = 0; e < 4; e++) ob[e] = __floats2bfloat162_rn(v[8 * k + 2 * e], v[8 * k + 2 * e + 1]);
              *reinterpret_cast<uint4*>(stg + stage_offset(lane, k)) = o;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                           ::"l"((uint64_t)&tmap_c), "r"(smem_u32(stg)), "r"(n), "r"(m0 + h * 128 + q * 32), "r"(bz) : "memory");
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
              asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            }
            __syncwarp();
            sbuf ^= 1;
            return;
          }
          if (!(p.flags & kOutF32) && n + 32 <= p.N && m0 + h * 128 + q * 32 < p.M) {
            // bf16 output, whole 32-column chunk (warp-uniform): every global access goes through the
            // warp's staging buffer so that it is coalesced
            uint8_t* stg = stage_base + ew * 2 * kStageWarpBytes;
            const bool row_ok = m < p.M;
            const size_t off = (size_t)bz * (size_t)p.stride_c + (size_t)m * p.ldc + n;
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[j]);
            if (p.flags & kBias) {
#pragma unroll
              for (int j = 0; j < 32; j++) v[j] += __ldg(p.bias + n + j);
            }
            if (p.flags & kAuxOut) warp_store_rows_bf16(stg, lane, v, reinterpret_cast<__nv_bfloat16*>(p.aux), off, row_ok);
            if (p.flags & kGeluGrad) {
              float x[32];
              warp_load_rows_bf16<false>(stg, lane, reinterpret_cast<const __nv_bfloat16*>(p.aux), off, row_ok, x);
#pragma unroll
              for (int j = 0; j < 32; j++) v[j] *= gelu_grad_f(x[j]);
            }
            if (p.flags & kGelu) {
#pragma unroll
              for (int j = 0; j < 32; j++) v[j] = gelu_f(v[j]);
            }
            if (p.flags & kResidual)
              warp_load_rows_bf16<true>(stg, lane, reinterpret_cast<const __nv_bfloat16*>(p.residual), off, row_ok, v);
            warp_store_rows_bf16(stg, lane, v, reinterpret_cast<__nv_bfloat16*>(p.C), off, row_ok);
            return;
          }
          if (m < p.M && n < p.N) {
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[j]);
            if (p.flags & kBias) {
#pragma unroll
              for (int j = 0; j < 32; j++) if (n + j < p.N) v[j] += __ldg(p.bias + n + j);
            }
            const size_t off = (size_t)bz * (size_t)p.stride_c + (size_t)m * p.ldc + n;
            if (p.flags & kGelu) {
#pragma unroll
              for (int j = 0; j < 32; j++) v[j] = gelu_f(v[j]);
            }
            if (p.flags & kOutF32) {
              float* C = reinterpret_cast<float*>(p.C) + off;
              const float* R = reinterpret_cast<const float*>(p.residual) + off;
              if (n + 32 <= p.N) {
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                  float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                  if (p.flags & kResidual) { float4 x = *reinterpret_cast<const float4*>(R + j); o.x += x.x; o.y += x.y; o.z += x.z; o.w += x.w; }
                  if (p.flags & kAccumulate) { float4 x = *reinterpret_cast<const float4*>(C + j); o.x += x.x; o.y += x.y; o.z += x.z; o.w += x.w; }
                  *reinterpret_cast<float4*>(C + j) = o;
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; j++) {     // unrolled with a predicate: v[] stays in registers
                  if (n + j < p.N) {
                    float o = v[j];
                    if (p.flags & kResidual) o += R[j];
                    if (p.flags & kAccumulate) o += C[j];
                    C[j] = o;
                  }
                }
              }
            } else {
              __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(p.C) + off;
              const __nv_bfloat16* R = reinterpret_cast<const __nv_bfloat16*>(p.residual) + off;
              if (n + 32 <= p.N) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  if (p.flags & kResidual) {
                    uint4 x = *reinterpret_cast<const uint4*>(R + j);
                    const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
                    for (int e = 0; e < 4; e++) { float2 f = __bfloat1622float2(xb[e]); v[j + 2 * e] += f.x; v[j + 2 * e + 1] += f.y; }
                  }
                  uint4 o;
                  __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                  for (int e = 0; e < 4; e++) ob[e] = __floats2bfloat162_rn(v[j + 2 * e], v[j + 2 * e + 1]);
                  *reinterpret_cast<uint4*>(C + j) = o;
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; j++) {
                  if (n + j < p.N) {
                    float o = v[j];
                    if (p.flags & kResidual) o += __bfloat162float(R[j]);
                    C[j] = __float2bfloat16(o);
                  }
                }
              }
            }
          }
        };
        constexpr int NCH = COLS / 32;
        uint32_t ra[32], rb[32];
        tc_ld32(taddr, ra);
#pragma unroll 1
        for (int c = 0; c < NCH; c += 2) {
          tc_wait_ld();
          if (c + 1 < NCH) tc_ld32(taddr + (c + 1) * 32, rb);
          process(ra, c);
          if (c + 1 < NCH) {
            tc_wait_ld();
            if (c + 2 < NCH) tc_ld32(taddr + (c + 2) * 32, ra);
            process(rb, c + 1);
          }
        }
        // this accumulator has been read out: the MMA warp may overwrite it
        tc_fence_before();
        mbar_arrive(&sm->tmem_empty[acc0 + h]);
      }
    }
    // the stores this lane handed to the TMA have completed before the CTA's shared memory goes away
    if (p.tma_store && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
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

// ------------------------------------------------------------------- host side
static EncodeTiledFn encode_fn() { return encode_tiled_fn(); }

// Says on stderr why a tensor map was refused (the launcher then returns -12): rank, extents, strides and box.
static int map_refused(CUresult r, int rank, const cuuint64_t* dims, const cuuint64_t* strides, const cuuint32_t* box) {
  fprintf(stderr, "gcow gemm: cuTensorMapEncodeTiled failed with CUresult %d; rank %d, dims", (int)r, rank);
  for (int i = 0; i < rank; i++) fprintf(stderr, " %llu", (unsigned long long)dims[i]);
  fprintf(stderr, ", byte strides");
  for (int i = 0; i + 1 < rank; i++) fprintf(stderr, " %llu", (unsigned long long)strides[i]);
  fprintf(stderr, ", box");
  for (int i = 0; i < rank; i++) fprintf(stderr, " %u", (unsigned)box[i]);
  fprintf(stderr, "\n");
  return -12;
}

// 2-D bf16 row-major [rows, cols] with leading dimension ld (elements); box = 64 columns x box_rows.
static int make_map(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -10;
  if (((uintptr_t)ptr & 15) || (ld * 2) % 16) return -11;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : map_refused(r, 2, dims, strides, box);
}

// 3-D variant: `batch` matrices, `bstride` elements apart; box = 64 columns x box_rows x 1.
static int make_map3(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint64_t batch,
                     uint64_t bstride, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -10;
  if (((uintptr_t)ptr & 15) || (ld * 2) % 16 || (bstride * 2) % 16) return -11;
  cuuint64_t dims[3] = {cols, rows, batch};
  cuuint64_t strides[2] = {ld * 2, bstride * 2};
  cuuint32_t box[3] = {(cuuint32_t)BK, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : map_refused(r, 3, dims, strides, box);
}

// Output map of the TMA-store epilogue: bf16 [batch][rows][cols], box = 32 columns x 32 rows in the 64-byte swizzle.
static int make_map_store(CUtensorMap* map, void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint64_t batch,
                          uint64_t bstride) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -10;
  if (((uintptr_t)ptr & 15) || (ld * 2) % 16 || (bstride * 2) % 16) return -11;
  cuuint64_t dims[3] = {cols, rows, batch};
  cuuint64_t strides[2] = {ld * 2, bstride * 2};
  cuuint32_t box[3] = {32, 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : map_refused(r, 3, dims, strides, box);
}

// MN-major matrix [K][cols] (cols a multiple of 64) as {64, K, cols / 64 (, batch)}; box = 64 x 64 x chunks.
static int make_map_mn(CUtensorMap* map, const void* ptr, uint64_t K, uint64_t cols, uint64_t ld, uint64_t batch,
                       uint64_t bstride, uint32_t chunks) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -10;
  if (((uintptr_t)ptr & 15) || (ld * 2) % 16 || (bstride * 2) % 16 || cols % 64) return -11;
  const cuuint32_t rank = batch > 1 ? 4 : 3;
  cuuint64_t dims[4] = {64, K, cols / 64, batch};
  cuuint64_t strides[3] = {ld * 2, 128, bstride * 2};
  cuuint32_t box[4] = {64, 64, chunks, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : map_refused(r, (int)rank, dims, strides, box);
}

template <int BM_> constexpr size_t smem_bytes() {
  return Shape<BM_>::SMEM + sizeof(Smem) + 512 + (size_t)Shape<BM_>::EPI_WARPS * 2 * kStageWarpBytes + 1024;
}

}  // namespace gemm

namespace tc {
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  // The encoder is a driver-API call and needs a current context on the calling thread. A thread that has made no
  // runtime-API call yet has none (autograd's backward threads reach a launcher this way when their first
  // allocation is served from PyTorch's cache), and the call fails with CUDA_ERROR_INVALID_CONTEXT. Binding the
  // runtime's device once per thread makes its primary context current.
  thread_local bool bound = false;
  if (!bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaSetDevice(dev) == cudaSuccess) bound = true;
  }
  return fn;
}
}  // namespace tc
}  // namespace gcow

using namespace gcow::gemm;

extern "C" {

// C[M,N] (+)= op(A) * op(B)^T  (+ bias[N]) (GELU) (+ residual[M,N]).
// a_mn == 0: A is stored [M][K] (lda = row length); a_mn == 1: A is stored [K][M].
// b_mn == 0: B is stored [N][K];                    b_mn == 1: B is stored [K][N].
// bf16 operands, leading dimensions multiples of 8, 16-byte aligned bases; C bf16 or fp32 (flags & 1) with ldc a multiple of 8 (bf16) or
// 4 (fp32). `error` is a device word that stays 0 unless a wait gave up.
// tile_rows: 128 or 256 to force a tile shape, anything else lets the launcher choose.
// Returns 0, a negative argument error, or a CUDA error code.
static int gemm_launch(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                       const float* bias, const void* residual, void* aux, int flags, uint32_t* error, int max_ctas,
                       int a_mn, int b_mn, int tile_rows, int batch, long long stride_a, long long stride_b,
                       long long stride_c, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return 0;
  if (batch > 1 && (stride_a % 8 || stride_b % 8 || stride_c % 8)) return -1;
  if (lda % 8 || ldb % 8) return -1;
  if ((!a_mn || !b_mn) && K % 8) return -1;   // a K-major operand has K as its row length
  if ((flags & kOutF32) ? (ldc % 4) : (ldc % 8)) return -1;
  if ((uintptr_t)C & 15) return -1;
  if ((flags & kBias) && !bias) return -1;
  if ((flags & kResidual) && (!residual || ((uintptr_t)residual & 15))) return -1;
  if ((flags & (kAuxOut | kGeluGrad)) && (!aux || ((uintptr_t)aux & 15) || N % 32 || (flags & kOutF32))) return -1;
  if ((flags & kAuxOut) && (flags & kGeluGrad)) return -1;
  CUtensorMap ma, mb, mc;
  memset(&mc, 0, sizeof(mc));
  static std::once_flag once;
  static int sms = 148;
  std::call_once(once, [] {
#define GCOW_GEMM_ATTR(BM_, A, B) cudaFuncSetAttribute(gemm_bf16_kernel<BM_, A, B>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes<BM_>())
    GCOW_GEMM_ATTR(128, false, false); GCOW_GEMM_ATTR(128, false, true); GCOW_GEMM_ATTR(128, true, false); GCOW_GEMM_ATTR(128, true, true);
    GCOW_GEMM_ATTR(256, false, false); GCOW_GEMM_ATTR(256, false, true); GCOW_GEMM_ATTR(256, true, false); GCOW_GEMM_ATTR(256, true, true);
#undef GCOW_GEMM_ATTR
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  });
  // 256-row tiles halve the L2 traffic per flop; keep 128-row tiles when they are needed to fill the SMs
  const int tiles256 = ((M + 255) / 256) * ((N + BN - 1) / BN) * batch;
  // ... and for short reductions, where the epilogue of a 256-row tile (which cannot overlap the next tile's
  // first MMAs) would dominate
  // ... and for very short reductions, where the step is bound by memory and the 256-row tile fetches the B tile
  // half as often (measured on the 1x1 layers of ResNet-50)
  const int bm = (tile_rows == 128 || tile_rows == 256) ? tile_rows
                 : ((tiles256 >= (sms * 4) / 5 && (K >= 2048 || K < 256)) ? 256 : 128);
  // K-major: matrix [rows][K], box 64 x tile rows. MN-major: matrix [K][rows], box 64 x 64.
  // An operand with fewer rows than its tile (64 output channels against the 256-column B tile) is fetched with a box of
  // its own height: the rest of the tile's shared memory keeps stale bytes, which only reach accumulator rows or
  // columns that are never stored.
  const int a_rows = bm < (M + 63) / 64 * 64 ? bm : (M + 63) / 64 * 64;
  const int b_rows = BN < (N + 63) / 64 * 64 ? BN : (N + 63) / 64 * 64;
  int rc;
  // an MN-major operand whose row length is a multiple of 64 is fetched with one copy per stage
  const int a_merged = a_mn && M % 64 == 0, b_merged = b_mn && N % 64 == 0;
  if (a_merged || b_merged) {
    rc = a_merged ? make_map_mn(&ma, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, (uint64_t)batch, (uint64_t)stride_a, (uint32_t)a_rows / 64)
         : batch == 1 ? (a_mn ? make_map(&ma, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, 64)
                              : make_map(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, (uint32_t)a_rows))
                      : (a_mn ? make_map3(&ma, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, (uint64_t)batch, (uint64_t)stride_a, 64)
                              : make_map3(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, (uint64_t)batch, (uint64_t)stride_a, (uint32_t)a_rows));
    if (rc) return rc;
    rc = b_merged ? make_map_mn(&mb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, (uint64_t)batch, (uint64_t)stride_b, (uint32_t)b_rows / 64)
         : batch == 1 ? (b_mn ? make_map(&mb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, 64)
                              : make_map(&mb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, (uint32_t)b_rows))
                      : (b_mn ? make_map3(&mb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, (uint64_t)batch, (uint64_t)stride_b, 64)
                              : make_map3(&mb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, (uint64_t)batch, (uint64_t)stride_b, (uint32_t)b_rows));
  } else if (batch == 1) {
    rc = a_mn ? make_map(&ma, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, 64)
              : make_map(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, (uint32_t)a_rows);
    if (rc) return rc;
    rc = b_mn ? make_map(&mb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, 64)
              : make_map(&mb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, (uint32_t)b_rows);
  } else {
    rc = a_mn ? make_map3(&ma, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, (uint64_t)batch, (uint64_t)stride_a, 64)
              : make_map3(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, (uint64_t)batch, (uint64_t)stride_a, (uint32_t)a_rows);
    if (rc) return rc;
    rc = b_mn ? make_map3(&mb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, (uint64_t)batch, (uint64_t)stride_b, 64)
              : make_map3(&mb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, (uint64_t)batch, (uint64_t)stride_b, (uint32_t)b_rows);
  }
  if (rc) return rc;
  Params p;
  p.C = C; p.bias = bias; p.residual = residual; p.aux = aux;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.flags = flags; p.error = error;
  p.batch = batch; p.stride_c = batch > 1 ? stride_c : 0;
  p.a_merged = a_merged; p.b_merged = b_merged;
  p.a_chunks = a_rows / 64; p.b_chunks = b_rows / 64;
  p.stage_tx = (uint32_t)(a_rows + b_rows) * 128u;
  // plain bf16 results (bias and GELU allowed) leave through the TMA; N must be whole 32-column blocks
  p.tma_store = !(flags & (kOutF32 | kResidual | kAccumulate | kAuxOut | kGeluGrad)) && N % 32 == 0;
  if (p.tma_store) {
    const uint64_t bs = batch > 1 ? (uint64_t)stride_c : (uint64_t)M * (uint64_t)ldc;
    if (make_map_store(&mc, C, (uint64_t)M, (uint64_t)N, (uint64_t)ldc, (uint64_t)batch, bs)) p.tma_store = 0;
  }
  const int tiles = ((M + bm - 1) / bm) * ((N + BN - 1) / BN) * batch;
  int grid = tiles < sms ? tiles : sms;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  cudaStream_t st = (cudaStream_t)stream;
#define GCOW_GEMM_LAUNCH(BM_, A, B) gcow::launch_dependent(gemm_bf16_kernel<BM_, A, B>, dim3(grid), dim3(Shape<BM_>::THREADS), smem_bytes<BM_>(), st, ma, mb, mc, p)
  if (bm == 256) {
    if (!a_mn && !b_mn) GCOW_GEMM_LAUNCH(256, false, false);
    else if (!a_mn && b_mn) GCOW_GEMM_LAUNCH(256, false, true);
    else if (a_mn && !b_mn) GCOW_GEMM_LAUNCH(256, true, false);
    else GCOW_GEMM_LAUNCH(256, true, true);
  } else {
    if (!a_mn && !b_mn) GCOW_GEMM_LAUNCH(128, false, false);
    else if (!a_mn && b_mn) GCOW_GEMM_LAUNCH(128, false, true);
    else if (a_mn && !b_mn) GCOW_GEMM_LAUNCH(128, true, false);
    else GCOW_GEMM_LAUNCH(128, true, true);
  }
#undef GCOW_GEMM_LAUNCH
  return (int)cudaGetLastError();
}

int gcow_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                   const float* bias, const void* residual, int flags, uint32_t* error, int max_ctas,
                   int a_mn, int b_mn, int tile_rows, void* stream) {
  return gemm_launch(A, B, C, M, N, K, lda, ldb, ldc, bias, residual, nullptr, flags, error, max_ctas, a_mn, b_mn, tile_rows,
                     1, 0, 0, 0, stream);
}

// As gcow_gemm_bf16 with a bf16 side tensor `aux` of C's shape and leading dimension (N a multiple of 32, bf16 C):
// flags & 32: aux receives the value before GELU (acc + bias) while C gets GELU of it;
// flags & 64: the result is multiplied by GELU'(aux) before the residual is added - the backward of that GELU.
int gcow_gemm_bf16_aux(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                       const float* bias, const void* residual, void* aux, int flags, uint32_t* error, int a_mn, int b_mn,
                       int tile_rows, void* stream) {
  return gemm_launch(A, B, C, M, N, K, lda, ldb, ldc, bias, residual, aux, flags, error, 0, a_mn, b_mn, tile_rows,
                     1, 0, 0, 0, stream);
}

// `batch` independent products; matrix i of A/B/C (and residual) starts stride_a/b/c elements
// (multiples of 8) after matrix i-1. Everything else as gcow_gemm_bf16.
int gcow_gemm_bf16_batched(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                           int batch, long long stride_a, long long stride_b, long long stride_c, const float* bias,
                           const void* residual, int flags, uint32_t* error, int a_mn, int b_mn, int tile_rows,
                           void* stream) {
  return gemm_launch(A, B, C, M, N, K, lda, ldb, ldc, bias, residual, nullptr, flags, error, 0, a_mn, b_mn, tile_rows, batch,
                     stride_a, stride_b, stride_c, stream);
}

}  // extern "C"
