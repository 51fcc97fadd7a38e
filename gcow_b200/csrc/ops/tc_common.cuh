// Inline-PTX building blocks shared by the tcgen05 kernels (GEMM and implicit-GEMM
// convolution): mbarrier operations with bounded waits, TMA tile loads, tcgen05
// MMA / commit / tensor-memory loads and the shared-memory matrix descriptors of
// the 128-byte-swizzled tile layouts. No load here uses cluster multicast.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gcow {
namespace tc {

constexpr uint32_t kSpinLimit = 1u << 26;   // polls before a wait gives up

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok;
}
// Bounded wait. Returns false when the CTA is aborting (this or another role gave up):
// after kSpinLimit polls the abort word is raised and `code` is recorded in *error.
__device__ __forceinline__ bool mbar_wait_abortable(volatile uint32_t* abort, uint64_t* bar, uint32_t parity,
                                                    uint32_t* error, uint32_t code) {
  for (uint32_t it = 0; it < kSpinLimit; it++) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort) return false;
  }
  *abort = 1;
  atomicCAS(error, 0u, code);
  return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(x), "r"(y) : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z, int w) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
               ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z, int w, int v) {
  asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
               ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w), "r"(v) : "memory");
}
// x = innermost coordinate, y = row coordinate, z = batch index (used only by batched launches)
__device__ __forceinline__ void tma_load(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z, bool batched) {
  if (batched) tma_load_3d(dst, map, bar, x, y, z);
  else tma_load_2d(dst, map, bar, x, y);
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile stored as rows of 128 bytes
// with the 128-byte swizzle: 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3ffffu) >> 4);        // start address
  d |= (uint64_t)(1024u >> 4) << 32;               // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                          // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                          // layout: 128-byte swizzle
  return d;
}

// MN-major tile: boxes of [64 K-rows][64 elements = 128 bytes], 128-byte swizzle.
// Groups of 8 K-rows are 1024 bytes apart (stride offset); the next 64 elements
// along M/N start one box (8192 bytes) later (leading offset).
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3ffffu) >> 4);
  d |= (uint64_t)(8192u >> 4) << 16;
  d |= (uint64_t)(1024u >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// GELU pieces for GEMM epilogues, where eight warps do the elementwise math of a whole tile and libm's erff
// (a long dependent chain) would take longer than the tile's main loop. Phi(x) = 0.5 (1 + erf(x / sqrt 2)) from
// the rational approximation erf(z) = 1 - (a1 t + ... + a5 t^5) exp(-z^2), t = 1 / (1 + p z) (Abramowitz &
// Stegun 7.1.26, absolute error below 1.5e-7); exp(-z^2) = exp(-x^2 / 2) is also what the derivative needs.
__device__ __forceinline__ void gelu_parts(float x, float& cdf, float& gauss) {
  const float z = fabsf(x) * 0.70710678118654752f;
  const float t = __fdividef(1.0f, fmaf(0.3275911f, z, 1.0f));
  gauss = __expf(-0.5f * x * x);
  float q = fmaf(1.061405429f, t, -1.453152027f);
  q = fmaf(q, t, 1.421413741f);
  q = fmaf(q, t, -0.284496736f);
  q = fmaf(q, t, 0.254829592f);
  q = 0.5f * q * t * gauss;
  cdf = x >= 0.0f ? 1.0f - q : q;
}
__device__ __forceinline__ float gelu_f(float x) {
  float cdf, g;
  gelu_parts(x, cdf, g);
  return x * cdf;
}
// d/dx of x Phi(x) = Phi(x) + x phi(x)
__device__ __forceinline__ float gelu_grad_f(float x) {
  float cdf, g;
  gelu_parts(x, cdf, g);
  return fmaf(x * 0.3989422804014327f, g, cdf);
}

// Coalesced bf16 rows for epilogues. After tcgen05.ld a lane owns one row of the tile (32 consecutive columns),
// so a direct 16-byte store per lane touches 32 different rows per instruction: 32 memory transactions of 16
// useful bytes. These helpers pass the warp's 32 x 32 block through a private shared-memory buffer of 32 rows
// x 64 bytes so that four lanes cover the 64 bytes of one row and an instruction touches 8 rows: a quarter of the
// transactions, all of them whole sectors. The 16-byte chunk k of row r sits at chunk k ^ ((r >> 1) & 3), which keeps
// both access patterns free of bank conflicts without padding (the 2 KB per warp matter: with eight of them a GEMM
// CTA still leaves room on its SM for one CTA of the all-reduce kernel).
// row_off: element offset of the lane's own row start (column 0 of the block), row_ok: whether that row exists.
constexpr int kStageRowBytes = 64, kStageWarpBytes = 32 * kStageRowBytes;
__device__ __forceinline__ int stage_offset(int row, int chunk) { return row * kStageRowBytes + ((chunk ^ ((row >> 1) & 3)) << 4); }

__device__ __forceinline__ void warp_store_rows_bf16(uint8_t* stg, int lane, const float (&v)[32], __nv_bfloat16* base,
                                                     size_t row_off, bool row_ok) {
#pragma unroll
  for (int k = 0; k < 4; k++) {
    uint4 o;
    __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; e++) ob[e] = __floats2bfloat162_rn(v[8 * k + 2 * e], v[8 * k + 2 * e + 1]);
    *reinterpret_cast<uint4*>(stg + stage_offset(lane, k)) = o;
  }
  __syncwarp();
#pragma unroll
  for (int it = 0; it < 4; it++) {
    const int row = it * 8 + (lane >> 2), ch = lane & 3;
    const unsigned long long off = __shfl_sync(0xffffffffu, (unsigned long long)row_off, row);
    const int ok = __shfl_sync(0xffffffffu, (int)row_ok, row);
    const uint4 x = *reinterpret_cast<const uint4*>(stg + stage_offset(row, ch));
    if (ok) *reinterpret_cast<uint4*>(base + off + ch * 8) = x;
  }
  __syncwarp();
}

// out[j] (+)= the lane's own row of a bf16 tensor, fetched with the same coalesced pattern
template <bool ADD>
__device__ __forceinline__ void warp_load_rows_bf16(uint8_t* stg, int lane, const __nv_bfloat16* base, size_t row_off,
                                                    bool row_ok, float (&out)[32]) {
#pragma unroll
  for (int it = 0; it < 4; it++) {
    const int row = it * 8 + (lane >> 2), ch = lane & 3;
    const unsigned long long off = __shfl_sync(0xffffffffu, (unsigned long long)row_off, row);
    const int ok = __shfl_sync(0xffffffffu, (int)row_ok, row);
    uint4 x = make_uint4(0, 0, 0, 0);
    if (ok) x = *reinterpret_cast<const uint4*>(base + off + ch * 8);
    *reinterpret_cast<uint4*>(stg + stage_offset(row, ch)) = x;
  }
  __syncwarp();
#pragma unroll
  for (int k = 0; k < 4; k++) {
    const uint4 x = *reinterpret_cast<const uint4*>(stg + stage_offset(lane, k));
    const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const float2 f = __bfloat1622float2(xb[e]);
      if (ADD) { out[8 * k + 2 * e] += f.x; out[8 * k + 2 * e + 1] += f.y; }
      else { out[8 * k + 2 * e] = f.x; out[8 * k + 2 * e + 1] = f.y; }
    }
  }
  __syncwarp();
}

// Host side: the driver's tensor-map encoder, looked up once through the runtime.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn();

}  // namespace tc
}  // namespace gcow
