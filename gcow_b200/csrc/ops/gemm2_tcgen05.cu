// bf16 GEMM on CTA pairs (tcgen05 cta_group::2): C[M,N] = A[M,K] * B[N,K]^T, K-major operands, fp32 accumulation in
// tensor memory, fused epilogue (bias, GELU, residual, side tensor for the GELU gradient).
//
// Two CTAs on neighbouring SMs (a cluster of 2) compute one 256 x 256 tile. CTA r loads rows r*128.. of the A tile
// and rows r*128.. of the B tile (half of each), so per flop every SM fetches two thirds of what the one-CTA
// 128 x 256 tile needs; one thread of CTA 0 issues M256 x N256 x K16 MMAs that read both CTAs' shared memory, and
// each CTA ends up with its 128 rows x 256 columns in its own tensor memory - which leaves room for two
// accumulators, so the epilogue of a tile overlaps the main loop of the next.
// A stage holds 128 K-elements: the tensor maps describe an operand as {64, rows, K/64}, so ONE 32 KB box per
// operand brings both 64-wide K chunks (a TMA copy costs a few hundred cycles per instruction besides its bytes).
//
// Signalling inside the pair (no multicast qualifier anywhere; remote barriers are addressed with mapa):
//   full[s]       lives in CTA 0; armed by CTA 0's producer with the bytes of both CTAs' copies, which both
//                 complete on it (cp.async.bulk.tensor ... .cta_group::2 with CTA 0's barrier address);
//   empty[s]      one per CTA; the MMA thread commits to its own and to the peer's;
//   tmem_full[a]  one per CTA, same; tmem_empty[a] lives in CTA 0, both CTAs' epilogue threads arrive on it.
// Every wait is bounded; a CTA that gives up raises the error word, and its peer's waits then run out too.
//
// Replaces the cuBLAS GEMMs behind nn.Linear in the forward pass of the transformer models trained by the
// benchmark (no counterpart in the reference, whose GEMMs are library calls: hw/models/resenet.py:90).
#include <stdlib.h>
#include <mutex>

#include "tc_common.cuh"

namespace gcow {
namespace gemm2 {

using namespace gcow::tc;

constexpr int BM = 256, BN = 256, UMMA_K = 16;
constexpr int BK = 128;                               // K elements per stage: two 64-wide chunks
constexpr int CHUNK_BYTES = 128 * 64 * 2;             // 128 rows x 128 bytes
constexpr int OPER_BYTES = 2 * CHUNK_BYTES;           // one CTA's half of an operand, one stage
constexpr int STAGE_BYTES = 2 * OPER_BYTES;           // 64 KB
constexpr int STAGES = 3;
constexpr int EPI_WARPS = 8, THREADS = 64 + 32 * EPI_WARPS;
constexpr uint32_t TMEM_COLS = 512;

enum Flags : int { kBias = 2, kGelu = 4, kResidual = 8, kAuxOut = 32, kGeluGrad = 64 };

struct Params {
  __nv_bfloat16* C;
  const float* bias;
  const __nv_bfloat16* residual;
  __nv_bfloat16* aux;
  int M, N, K, ldc, flags;
  uint32_t* error;
};

struct Smem {
  uint64_t full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], drain;
  uint32_t tmem_base;
  volatile uint32_t abort;
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the copy lands in this CTA's shared memory; its bytes complete on the barrier at cluster address `bar`
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

// MN-major operand tile fetched as ONE box {64 columns, 128 K-rows, 2 column groups}: each 64-column group is
// 128 K-rows x 128 bytes = 16 KB, so groups are 16 KB apart (leading offset) and 8-row groups 1 KB (stride offset).
__device__ __forceinline__ uint64_t smem_desc_mn_sw128_16k(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3ffffu) >> 4);
  d |= (uint64_t)(16384u >> 4) << 16;
  d |= (uint64_t)(1024u >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// B_MN: B is stored [K][N] (the data-gradient product dX = dY * W reads the weight matrix in place)
template <bool B_MN>
__global__ void __launch_bounds__(THREADS, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  Smem* sm = reinterpret_cast<Smem*>(base + STAGES * STAGE_BYTES);
  uint8_t* stage_base = reinterpret_cast<uint8_t*>(((uintptr_t)(sm + 1) + 15) & ~(uintptr_t)15);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();               // 0: issues the MMAs and owns full / tmem_empty
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int kblocks = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(&sm->full[s], 1); mbar_init(&sm->empty[s], 1); }
    for (int a = 0; a < 2; a++) { mbar_init(&sm->tmem_full[a], 1); mbar_init(&sm->tmem_empty[a], 2 * EPI_WARPS * 32); }
    mbar_init(&sm->drain, 1);
    sm->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm->tmem_base)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();            // both CTAs' barriers are initialised before either signals the other
  tc_fence_after();
  const uint32_t tmem_base = sm->tmem_base;
  // programmatic dependent launch: the next kernel of the stream may set itself up from here on, and this one, when
  // launched the same way, has set itself up under the tail of its predecessor; global memory only after that
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t s = 0, phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += pairs) {
        const int m0 = (tile % tiles_m) * BM + (int)rank * 128, n0 = (tile / tiles_m) * BN + (int)rank * 128;
        for (int kb = 0; kb < kblocks; kb++) {
          if (!(ok = mbar_wait_abortable(&sm->abort, &sm->empty[s], phase ^ 1, p.error, 1))) break;
          if (rank == 0) mbar_expect_tx(&sm->full[s], 2 * STAGE_BYTES);
          const uint32_t bar = map_to_cta(smem_u32(&sm->full[s]), 0);
          uint8_t* st = base + s * STAGE_BYTES;
          tma_load_3d_pair(smem_u32(st), &tmap_a, bar, 0, m0, kb * 2);
          if (B_MN) tma_load_3d_pair(smem_u32(st + OPER_BYTES), &tmap_b, bar, 0, kb * BK, n0 / 64);
          else tma_load_3d_pair(smem_u32(st + OPER_BYTES), &tmap_b, bar, 0, n0, kb * 2);
          if (++s == STAGES) { s = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // giving up: let copies already in flight land before the CTA's shared memory is released
        for (int i = 0; i < 1000; i++) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer (CTA 0 only)
    if (lane == 0 && rank == 0) {
      // instruction descriptor: fp32 accumulate, bf16 x bf16, K-major operands, N 256, M 256 (128 rows per CTA)
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)B_MN << 16) | ((uint32_t)(BN >> 3) << 17) |
                             ((uint32_t)(BM >> 4) << 24);
      uint32_t s = 0, phase = 0, t = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += pairs, t++) {
        const uint32_t acc = t & 1, aphase = (t >> 1) & 1;
        if (!(ok = mbar_wait_abortable(&sm->abort, &sm->tmem_empty[acc], aphase ^ 1, p.error, 2))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kblocks; kb++) {
          if (!(ok = mbar_wait_abortable(&sm->abort, &sm->full[s], phase, p.error, 3))) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(base + s * STAGE_BYTES), sb = sa + OPER_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; k++) {
            const uint32_t off = (k >> 2) * CHUNK_BYTES + (k & 3) * 32;     // 64-wide chunk, then 32 bytes per K step
            // MN-major B: 16 K-rows of 128 bytes per step, 128 rows contiguous within a column group
            const uint64_t db = B_MN ? smem_desc_mn_sw128_16k(sb + k * 2048) : smem_desc_sw128(sb + off);
            tc_mma_pair(d_tmem, smem_desc_sw128(sa + off), db, idesc, (kb | k) != 0);
          }
          const uint32_t eb = smem_u32(&sm->empty[s]);
          tc_commit_pair(map_to_cta(eb, 0));
          tc_commit_pair(map_to_cta(eb, 1));
          if (++s == STAGES) { s = 0; phase ^= 1; }
        }
        if (ok) {
          const uint32_t fb = smem_u32(&sm->tmem_full[acc]);
          tc_commit_pair(map_to_cta(fb, 0));
          tc_commit_pair(map_to_cta(fb, 1));
        }
      }
      // drain: everything issued by this thread has finished before tensor memory is freed
      tc_commit_pair(map_to_cta(smem_u32(&sm->drain), 0));
      for (uint32_t it = 0; it < kSpinLimit; it++) if (mbar_try_wait(&sm->drain, 0)) break;
    }
  } else {
    // ----------------------------------------------------------------- epilogue (both CTAs, own 128 rows)
    const int q = warp & 3, ew = warp - 2;
    constexpr int COLS = BN / (EPI_WARPS / 4);
    const int col0 = (ew / 4) * COLS;
    uint8_t* stg = stage_base + ew * kStageWarpBytes;
    uint32_t t = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += pairs, t++) {
      const int m0 = (tile % tiles_m) * BM + (int)rank * 128, n0 = (tile / tiles_m) * BN;
      const uint32_t acc = t & 1, aphase = (t >> 1) & 1;
      ok = mbar_wait_abortable(&sm->abort, &sm->tmem_full[acc], aphase, p.error, 4);
      ok = __all_sync(0xffffffffu, ok);   // the tensor-memory loads below need the whole warp
      if (!ok) break;
      tc_fence_after();
      const int m = m0 + q * 32 + lane;
      const bool row_ok = m < p.M;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + col0;
      auto process = [&](const uint32_t (&r)[32], int c) {
        const int n = n0 + col0 + c * 32;
        if (n >= p.N || m0 + q * 32 >= p.M) return;       // warp-uniform; the launcher guarantees N % 32 == 0
        const size_t off = (size_t)m * p.ldc + n;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[j]);
        if (p.flags & kBias) {
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] += __ldg(p.bias + n + j);
        }
        if (p.flags & kAuxOut) warp_store_rows_bf16(stg, lane, v, p.aux, off, row_ok);
        if (p.flags & kGeluGrad) {
          float x[32];
          warp_load_rows_bf16<false>(stg, lane, p.aux, off, row_ok, x);
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] *= gelu_grad_f(x[j]);
        }
        if (p.flags & kGelu) {
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] = gelu_f(v[j]);
        }
        if (p.flags & kResidual) warp_load_rows_bf16<true>(stg, lane, p.residual, off, row_ok, v);
        warp_store_rows_bf16(stg, lane, v, p.C, off, row_ok);
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
      // this CTA's half of the accumulator has been read out: tell the MMA thread in CTA 0
      tc_fence_before();
      mbar_arrive_cluster(map_to_cta(smem_u32(&sm->tmem_empty[acc]), 0));
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  cluster_sync();            // the peer no longer reads this CTA's shared memory or signals its barriers
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// K-major matrix [rows][K] (K a multiple of 64) as {64, rows, K / 64}; box = 64 x 128 rows x 2 chunks (32 KB).
static int make_map_kfold(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t K, uint64_t ld) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return -10;
  if (((uintptr_t)ptr & 15) || (ld * 2) % 16 || K % 64) return -11;
  cuuint64_t dims[3] = {64, rows, K / 64};
  cuuint64_t strides[2] = {ld * 2, 128};
  cuuint32_t box[3] = {64, 128, 2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -12;
}

// MN-major matrix [K][cols] (cols a multiple of 64) as {64, K, cols / 64}; box = 64 x 128 K-rows x 2 column groups (32 KB).
static int make_map_mnfold(CUtensorMap* map, const void* ptr, uint64_t K, uint64_t cols, uint64_t ld) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return -10;
  if (((uintptr_t)ptr & 15) || (ld * 2) % 16 || cols % 64) return -11;
  cuuint64_t dims[3] = {64, K, cols / 64};
  cuuint64_t strides[2] = {ld * 2, 128};
  cuuint32_t box[3] = {64, 128, 2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -12;
}

constexpr size_t kSmemBytes = (size_t)STAGES * STAGE_BYTES + sizeof(Smem) + 16 + (size_t)EPI_WARPS * kStageWarpBytes + 1024;

}  // namespace gemm2
}  // namespace gcow

using namespace gcow::gemm2;

extern "C" {

// Number of CTA pairs that can run at once on the current device (0: cluster launches are not possible).
int gcow_gemm2_max_pairs() {
  static std::once_flag once;
  static int pairs = 0;
  std::call_once(once, [] {
    if (cudaFuncSetAttribute(gemm2_bf16_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes) != cudaSuccess ||
        cudaFuncSetAttribute(gemm2_bf16_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes) != cudaSuccess) {
      cudaGetLastError();
      return;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2, 1, 1);
    cfg.blockDim = dim3(THREADS, 1, 1);
    cfg.dynamicSmemBytes = kSmemBytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm2_bf16_kernel<false>, &cfg) == cudaSuccess) pairs = n;
    else cudaGetLastError();
  });
  return pairs;
}

// C[M,N] = A[M,K] * op(B) (+ bias) (GELU) (+ residual), bf16 in and out, on CTA pairs. A is K-major [M][K]; B is
// [N][K] (b_mn == 0) or [K][N] (b_mn == 1, N a multiple of 64).
// K a multiple of 64, N a multiple of 32, lda/ldb/ldc multiples of 8, 16-byte aligned bases.
// flags as gcow_gemm_bf16 (2 bias, 4 GELU, 8 residual, 32 aux receives the pre-GELU value, 64 multiply by GELU'(aux)).
// Returns 0, a negative argument error (-2: not supported here, use the one-CTA kernel) or a CUDA error code.
int gcow_gemm2_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                    const float* bias, const void* residual, void* aux, int flags, uint32_t* error, int b_mn, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % 64 || N % 32 || lda % 8 || ldb % 8 || ldc % 8 || ((uintptr_t)C & 15) || (b_mn && N % 64)) return -2;
  if (flags & ~(kBias | kGelu | kResidual | kAuxOut | kGeluGrad)) return -2;
  if ((flags & kBias) && !bias) return -1;
  if ((flags & kResidual) && (!residual || ((uintptr_t)residual & 15))) return -1;
  if ((flags & (kAuxOut | kGeluGrad)) && (!aux || ((uintptr_t)aux & 15))) return -1;
  const int max_pairs = gcow_gemm2_max_pairs();
  if (max_pairs <= 0) return -2;
  CUtensorMap ma, mb;
  int rc = make_map_kfold(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda);
  if (rc) return rc;
  rc = b_mn ? make_map_mnfold(&mb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb)
            : make_map_kfold(&mb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb);
  if (rc) return rc;
  Params p;
  p.C = (__nv_bfloat16*)C; p.bias = bias; p.residual = (const __nv_bfloat16*)residual; p.aux = (__nv_bfloat16*)aux;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.flags = flags; p.error = error;
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  static const bool pdl = [] { const char* e = getenv("GCOW_PDL"); return !(e && e[0] == '0'); }();
  cfg.attrs = attr; cfg.numAttrs = pdl ? 2 : 1;
  if (b_mn) return (int)cudaLaunchKernelEx(&cfg, gemm2_bf16_kernel<true>, ma, mb, p);
  return (int)cudaLaunchKernelEx(&cfg, gemm2_bf16_kernel<false>, ma, mb, p);
}

}  // extern "C"
