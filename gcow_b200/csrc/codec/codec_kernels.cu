// Stand-alone encode / decode kernels of the ZFP float32 block codec (sm_100a).
//
// One thread owns one block and runs every stage in registers (zfp_block.cuh);
// the 128 processing elements and the serial burst writer of the FPGA design
// (hw/src/zfp.cpp:31-76, hw/src/io.cpp:185-320) become a grid of threads that
// store at computed bit offsets:
//   * fixed rate, 1-D, 16/32/64/128 bits per block: table-driven coder, one
//     aligned store per block, fully coalesced ("fast" kernels);
//   * every other case (1-D odd rates such as the 9-bit floor, 2-D in any mode,
//     fixed accuracy / precision): blocks are encoded into a scratch slot, the
//     slot lengths are prefix-summed, and a second pass ORs each slot into the
//     stream at its bit offset ("generic" kernels).
// Array walk and partial edge blocks follow sw/src/zfp.c:31-56,79-103 and
// sw/src/encode.c:41-88; per-stage debug kernels mirror hw/stages/*.cpp.
#include <cuda_runtime.h>
#include <stdint.h>
#include "zfp_block.cuh"

namespace gcow {

constexpr int kThreads = 256;

// Coder tables live in global memory (filled once per device by the host, see
// gcow_codec_tables) and are copied into shared memory by every CTA.
__device__ __align__(16) uint16_t g_enc_table[kEncTabSize];
__device__ __align__(16) uint16_t g_dec_table[kDecBudgetTabSize];
__device__ __align__(16) uint32_t g_enc_pair_table[kEncPairTabSize];
__device__ __align__(16) uint32_t g_dec_loop_table[kDecLoopTabSize];

__device__ __forceinline__ void load_enc_table(uint16_t* etab, const uint16_t* __restrict__ src) {
  for (int i = threadIdx.x; i < kEncTabSize / 2; i += blockDim.x)
    reinterpret_cast<uint32_t*>(etab)[i] = reinterpret_cast<const uint32_t*>(src)[i];
}
__device__ __forceinline__ void load_dec_table(uint16_t* dtab, const uint16_t* __restrict__ src) {
  for (int i = threadIdx.x; i < kDecBudgetTabSize / 8; i += blockDim.x)
    reinterpret_cast<uint4*>(dtab)[i] = reinterpret_cast<const uint4*>(src)[i];
}

__device__ __forceinline__ void load_pair_table(uint32_t* epair, const uint32_t* __restrict__ src) {
  for (int i = threadIdx.x; i < kEncPairTabSize / 4; i += blockDim.x)
    reinterpret_cast<uint4*>(epair)[i] = reinterpret_cast<const uint4*>(src)[i];
}

__device__ __forceinline__ void load_loop_table(uint32_t* dloop, const uint32_t* __restrict__ src) {
  for (int i = threadIdx.x; i < kDecLoopTabSize / 4; i += blockDim.x)
    reinterpret_cast<uint4*>(dloop)[i] = reinterpret_cast<const uint4*>(src)[i];
}

// Load block b of a 1-D array of n floats (tail block padded).
__device__ __forceinline__ void load_block_1d(float* f, const float* __restrict__ in, uint64_t n,
                                              uint64_t b, bool aligned) {
  uint64_t x0 = 4 * b;
  if (x0 + 4 <= n) {
    if (aligned) {
      float4 v = __ldg(reinterpret_cast<const float4*>(in) + b);
      f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    } else {
      f[0] = in[x0]; f[1] = in[x0 + 1]; f[2] = in[x0 + 2]; f[3] = in[x0 + 3];
    }
  } else {
    uint32_t c = (uint32_t)(n - x0);
    f[0] = f[1] = f[2] = f[3] = 0;
    for (uint32_t i = 0; i < c; i++) f[i] = in[x0 + i];
    pad_partial(f, c, 1);
  }
}
__device__ __forceinline__ void store_block_1d(const float* f, float* __restrict__ out, uint64_t n,
                                               uint64_t b, bool aligned) {
  uint64_t x0 = 4 * b;
  if (x0 + 4 <= n) {
    if (aligned) reinterpret_cast<float4*>(out)[b] = make_float4(f[0], f[1], f[2], f[3]);
    else { out[x0] = f[0]; out[x0 + 1] = f[1]; out[x0 + 2] = f[2]; out[x0 + 3] = f[3]; }
  } else {
    for (uint64_t i = 0; x0 + i < n; i++) out[x0 + i] = f[i];
  }
}

template <int BITS> struct CodeIO;
template <> struct CodeIO<16> {
  static constexpr int NW = 1;
  static __device__ __forceinline__ void store(void* out, uint64_t b, const uint32_t (&w)[1]) { ((uint16_t*)out)[b] = (uint16_t)w[0]; }
  static __device__ __forceinline__ void load(const void* in, uint64_t b, uint32_t (&w)[1]) { w[0] = ((const uint16_t*)in)[b]; }
};
template <> struct CodeIO<32> {
  static constexpr int NW = 1;
  static __device__ __forceinline__ void store(void* out, uint64_t b, const uint32_t (&w)[1]) { ((uint32_t*)out)[b] = w[0]; }
  static __device__ __forceinline__ void load(const void* in, uint64_t b, uint32_t (&w)[1]) { w[0] = ((const uint32_t*)in)[b]; }
};
template <> struct CodeIO<64> {
  static constexpr int NW = 2;
  static __device__ __forceinline__ void store(void* out, uint64_t b, const uint32_t (&w)[2]) { ((uint2*)out)[b] = make_uint2(w[0], w[1]); }
  static __device__ __forceinline__ void load(const void* in, uint64_t b, uint32_t (&w)[2]) { uint2 v = ((const uint2*)in)[b]; w[0] = v.x; w[1] = v.y; }
};
template <> struct CodeIO<128> {
  static constexpr int NW = 4;
  static __device__ __forceinline__ void store(void* out, uint64_t b, const uint32_t (&w)[4]) { ((uint4*)out)[b] = make_uint4(w[0], w[1], w[2], w[3]); }
  static __device__ __forceinline__ void load(const void* in, uint64_t b, uint32_t (&w)[4]) { uint4 v = ((const uint4*)in)[b]; w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w; }
};

template <int BITS>
__global__ void __launch_bounds__(kThreads)
encode_1d_fixed_kernel(const float* __restrict__ in, uint64_t n, void* __restrict__ out, int aligned,
                       const uint16_t* __restrict__ tab, const uint32_t* __restrict__ pair_tab) {
  __shared__ __align__(16) uint32_t epair[kEncPairTabSize];
  load_pair_table(epair, pair_tab);
  __syncthreads();
  const LeanTables lt = {tab, nullptr, epair, nullptr};      // the plane-by-plane table is read from global memory (rare path)
  const uint64_t blocks = num_blocks_1d(n);
  for (uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; b < blocks;
       b += (uint64_t)gridDim.x * blockDim.x) {
    float f[4];
    load_block_1d(f, in, n, b, aligned);
    uint32_t w[CodeIO<BITS>::NW];
    encode_block_1d_lean<BITS>(f, lt, w);
    CodeIO<BITS>::store(out, b, w);
  }
}

template <int BITS>
__global__ void __launch_bounds__(kThreads)
decode_1d_fixed_kernel(const void* __restrict__ in, float* __restrict__ out, uint64_t n, int shift,
                       int aligned, const uint16_t* __restrict__ tab, const uint32_t* __restrict__ loop_tab) {
  __shared__ __align__(16) uint32_t dloop[kDecLoopTabSize];
  load_loop_table(dloop, loop_tab);
  __syncthreads();
  const LeanTables lt = {nullptr, tab, nullptr, dloop};      // the plane-by-plane table is read from global memory (rare path)
  const uint64_t blocks = num_blocks_1d(n);
  for (uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; b < blocks;
       b += (uint64_t)gridDim.x * blockDim.x) {
    uint32_t w[CodeIO<BITS>::NW];
    CodeIO<BITS>::load(in, b, w);
    float f[4];
    decode_block_1d_lean<BITS>(f, lt, w, shift);
    store_block_1d(f, out, n, b, aligned);
  }
}

// ------------------------------------------------------------ generic path
// Sink that writes word j of this thread's slot at slot[j * stride]: slots of
// neighbouring blocks interleave, so a warp's stores coalesce.
struct StridedSink {
  uint64_t* out;
  uint64_t stride;
  uint64_t acc;
  uint32_t fill;
  uint32_t nw;
  __device__ __forceinline__ StridedSink(uint64_t* o, uint64_t s) : out(o), stride(s), acc(0), fill(0), nw(0) {}
  __device__ __forceinline__ void put(uint64_t v, uint32_t n) {
    if (!n) return;
    acc |= v << fill;
    uint32_t tot = fill + n;
    if (tot >= 64) {
      out[(uint64_t)nw * stride] = acc; nw++;
      acc = fill ? (v >> (64 - fill)) : 0;
      tot -= 64;
    }
    fill = tot;
  }
  __device__ __forceinline__ void pad(uint32_t n) {
    while (n) { uint32_t c = n < 64 ? n : 64; put(0, c); n -= c; }
  }
  __device__ __forceinline__ void finish() { if (fill) { out[(uint64_t)nw * stride] = acc; nw++; fill = 0; acc = 0; } }
};

template <int DIM>
__device__ __forceinline__ void gather_block(float* f, const float* __restrict__ in, uint64_t nx,
                                             uint64_t ny, uint64_t b) {
  if (DIM == 1) { load_block_1d(f, in, nx, b, false); return; }
  uint64_t bx = (nx + 3) / 4;
  uint64_t x0 = 4 * (b % bx), y0 = 4 * (b / bx);
  uint32_t cx = (uint32_t)(nx - x0 < 4 ? nx - x0 : 4), cy = (uint32_t)(ny - y0 < 4 ? ny - y0 : 4);
#pragma unroll
  for (int i = 0; i < 16; i++) f[i] = 0;
#pragma unroll
  for (uint32_t y = 0; y < 4; y++) {
    if (y < cy) {
#pragma unroll
      for (uint32_t x = 0; x < 4; x++) if (x < cx) f[4 * y + x] = in[(y0 + y) * nx + x0 + x];
      if (cx < 4) pad_partial(f + 4 * y, cx, 1);
    }
  }
  if (cy < 4) {
#pragma unroll
    for (int x = 0; x < 4; x++) pad_partial(f + x, cy, 4);
  }
}

template <int DIM>
__device__ __forceinline__ void scatter_block(const float* f, float* __restrict__ out, uint64_t nx,
                                              uint64_t ny, uint64_t b) {
  if (DIM == 1) { store_block_1d(f, out, nx, b, false); return; }
  uint64_t bx = (nx + 3) / 4;
  uint64_t x0 = 4 * (b % bx), y0 = 4 * (b / bx);
  uint32_t cx = (uint32_t)(nx - x0 < 4 ? nx - x0 : 4), cy = (uint32_t)(ny - y0 < 4 ? ny - y0 : 4);
#pragma unroll
  for (uint32_t y = 0; y < 4; y++)
#pragma unroll
    for (uint32_t x = 0; x < 4; x++)
      if (y < cy && x < cx) out[(y0 + y) * nx + x0 + x] = f[4 * y + x];
}

// Pass 1: encode block b into scratch slot b (word j at slots[j*blocks + b]),
// record its bit length.
template <int DIM>
__global__ void __launch_bounds__(kThreads)
encode_slots_kernel(const float* __restrict__ in, uint64_t nx, uint64_t ny, ZfpParams p,
                    uint64_t blocks, uint64_t* __restrict__ slots, uint32_t* __restrict__ lens) {
  for (uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; b < blocks;
       b += (uint64_t)gridDim.x * blockDim.x) {
    float f[1 << (2 * DIM)];
    gather_block<DIM>(f, in, nx, ny, b);
    StridedSink sink(slots + b, blocks);
    uint32_t bits = encode_block<DIM>(f, p, sink);
    sink.finish();
    lens[b] = bits;
  }
}

// Fixed rate with a whole number of 64-bit words per block (any DIM): block b owns
// words [b*W, (b+1)*W) of the stream, so every thread packs straight into them and
// no scratch, offset table or second pass is needed.
template <int DIM>
__global__ void __launch_bounds__(kThreads)
encode_fixed_direct_kernel(const float* __restrict__ in, uint64_t nx, uint64_t ny, ZfpParams p, uint64_t blocks,
                           uint64_t* __restrict__ out) {
  const uint32_t W = p.maxbits / 64;
  for (uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; b < blocks;
       b += (uint64_t)gridDim.x * blockDim.x) {
    float f[1 << (2 * DIM)];
    gather_block<DIM>(f, in, nx, ny, b);
    WordSink sink(out + b * W);
    encode_block<DIM>(f, p, sink);     // pads to minbits = maxbits, i.e. exactly W words
    sink.finish();
  }
}

// Exclusive prefix sum of block lengths -> bit offsets (blocks + 1 entries).
// Three steps: per-tile sums, scan of the tile sums by one CTA, per-tile scan.
constexpr int kScanTile = 2048;  // elements per CTA (256 threads x 8)

__device__ __forceinline__ uint64_t cta_exclusive_scan(uint64_t v, uint64_t* total) {
  __shared__ uint64_t warp_sums[kThreads / 32];
  __shared__ uint64_t cta_total;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  uint64_t x = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    uint64_t y = __shfl_up_sync(0xffffffffu, x, d);
    if (lane >= d) x += y;
  }
  if (lane == 31) warp_sums[wid] = x;
  __syncthreads();
  if (wid == 0) {
    uint64_t s = lane < kThreads / 32 ? warp_sums[lane] : 0;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      uint64_t y = __shfl_up_sync(0xffffffffu, s, d);
      if (lane >= d) s += y;
    }
    if (lane < kThreads / 32) warp_sums[lane] = s;
    if (lane == kThreads / 32 - 1) cta_total = s;
  }
  __syncthreads();
  uint64_t base = wid ? warp_sums[wid - 1] : 0;
  if (total) *total = cta_total;
  uint64_t r = base + x - v;
  __syncthreads();
  return r;
}

__global__ void __launch_bounds__(kThreads)
scan_tile_sums_kernel(const uint32_t* __restrict__ lens, uint64_t blocks, uint64_t* __restrict__ tile_sums) {
  uint64_t base = (uint64_t)blockIdx.x * kScanTile;
  uint64_t s = 0;
  for (int i = 0; i < kScanTile / kThreads; i++) {
    uint64_t idx = base + (uint64_t)i * kThreads + threadIdx.x;
    if (idx < blocks) s += lens[idx];
  }
  uint64_t total;
  cta_exclusive_scan(s, &total);
  if (threadIdx.x == 0) tile_sums[blockIdx.x] = total;
}

__global__ void __launch_bounds__(kThreads)
scan_tile_offsets_kernel(uint64_t* __restrict__ tile_sums, uint64_t tiles) {
  // single CTA: sequential over chunks of kThreads tiles, carry in a register
  uint64_t carry = 0;
  for (uint64_t t0 = 0; t0 < tiles; t0 += kThreads) {
    uint64_t idx = t0 + threadIdx.x;
    uint64_t v = idx < tiles ? tile_sums[idx] : 0;
    uint64_t total;
    uint64_t ex = cta_exclusive_scan(v, &total);
    if (idx < tiles) tile_sums[idx] = carry + ex;
    carry += total;
  }
}

__global__ void __launch_bounds__(kThreads)
scan_apply_kernel(const uint32_t* __restrict__ lens, uint64_t blocks, const uint64_t* __restrict__ tile_offs,
                  uint64_t* __restrict__ block_bits) {
  // each thread owns 8 consecutive elements of the tile
  constexpr int PER = kScanTile / kThreads;
  uint64_t base = (uint64_t)blockIdx.x * kScanTile + (uint64_t)threadIdx.x * PER;
  uint32_t v[PER];
  uint64_t s = 0;
#pragma unroll
  for (int i = 0; i < PER; i++) { v[i] = base + i < blocks ? lens[base + i] : 0; s += v[i]; }
  uint64_t ex = cta_exclusive_scan(s, nullptr) + tile_offs[blockIdx.x];
#pragma unroll
  for (int i = 0; i < PER; i++) {
    if (base + i < blocks) block_bits[base + i] = ex;
    ex += v[i];
    if (base + i == blocks - 1) block_bits[blocks] = ex;
  }
}

__global__ void __launch_bounds__(kThreads)
fixed_offsets_kernel(uint64_t blocks, uint32_t maxbits, uint64_t* __restrict__ block_bits) {
  for (uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; b <= blocks;
       b += (uint64_t)gridDim.x * blockDim.x)
    block_bits[b] = b * maxbits;
}

// Pass 2: OR slot b into the (zeroed) stream at bit offset block_bits[b].
__global__ void __launch_bounds__(kThreads)
scatter_slots_kernel(const uint64_t* __restrict__ slots, const uint32_t* __restrict__ lens,
                     const uint64_t* __restrict__ block_bits, uint64_t blocks,
                     unsigned long long* __restrict__ out) {
  for (uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; b < blocks;
       b += (uint64_t)gridDim.x * blockDim.x) {
    uint64_t pos = block_bits[b];
    uint32_t len = lens[b];
    uint32_t nw = (len + 63) / 64;
    uint32_t o = (uint32_t)(pos & 63);
    uint64_t wi = pos >> 6;
    uint64_t carry = 0;
    for (uint32_t j = 0; j < nw; j++) {
      uint64_t v = slots[(uint64_t)j * blocks + b];
      uint64_t lo = carry | (v << o);
      carry = o ? (v >> (64 - o)) : 0;
      if (lo) atomicOr(out + wi + j, (unsigned long long)lo);
    }
    if (carry) atomicOr(out + wi + nw, (unsigned long long)carry);
  }
}

template <int DIM>
__global__ void __launch_bounds__(kThreads)
decode_generic_kernel(const uint64_t* __restrict__ in, float* __restrict__ out, uint64_t nx, uint64_t ny,
                      ZfpParams p, uint64_t blocks, const uint64_t* __restrict__ block_bits, int shift) {
  for (uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; b < blocks;
       b += (uint64_t)gridDim.x * blockDim.x) {
    uint64_t pos = block_bits ? block_bits[b] : b * (uint64_t)p.maxbits;
    WordSrc src(in, pos);
    float f[1 << (2 * DIM)];
    decode_block<DIM>(f, p, src, shift);
    scatter_block<DIM>(f, out, nx, ny, b);
  }
}

// ------------------------------------------------------ stage debug kernels
template <int DIM>
__global__ void dbg_emax_kernel(const float* __restrict__ blocks, uint64_t nb, int* __restrict__ emax) {
  constexpr int N = 1 << (2 * DIM);
  uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nb) return;
  float f[N];
#pragma unroll
  for (int i = 0; i < N; i++) f[i] = blocks[b * N + i];
  emax[b] = block_emax<N>(f);
}
template <int DIM>
__global__ void dbg_cast_kernel(const float* __restrict__ blocks, uint64_t nb, const int* __restrict__ emax,
                                int32_t* __restrict__ q) {
  constexpr int N = 1 << (2 * DIM);
  uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nb) return;
  float f[N]; int32_t r[N];
#pragma unroll
  for (int i = 0; i < N; i++) f[i] = blocks[b * N + i];
  fwd_cast<N>(r, f, emax[b]);
#pragma unroll
  for (int i = 0; i < N; i++) q[b * N + i] = r[i];
}
template <int DIM>
__global__ void dbg_inv_cast_kernel(const int32_t* __restrict__ q, uint64_t nb, const int* __restrict__ emax,
                                    int shift, float* __restrict__ blocks) {
  constexpr int N = 1 << (2 * DIM);
  uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nb) return;
  float f[N]; int32_t r[N];
#pragma unroll
  for (int i = 0; i < N; i++) r[i] = q[b * N + i];
  inv_cast<N>(f, r, emax[b], shift);
#pragma unroll
  for (int i = 0; i < N; i++) blocks[b * N + i] = f[i];
}
template <int DIM>
__global__ void dbg_xform_kernel(int32_t* __restrict__ q, uint64_t nb, int inverse) {
  constexpr int N = 1 << (2 * DIM);
  uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nb) return;
  int32_t r[N];
#pragma unroll
  for (int i = 0; i < N; i++) r[i] = q[b * N + i];
  if (inverse) Xform<DIM>::inv(r); else Xform<DIM>::fwd(r);
#pragma unroll
  for (int i = 0; i < N; i++) q[b * N + i] = r[i];
}
template <int DIM>
__global__ void dbg_reorder_kernel(const int32_t* __restrict__ q, uint32_t* __restrict__ u, uint64_t nb) {
  constexpr int N = 1 << (2 * DIM);
  uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nb) return;
  int32_t r[N]; uint32_t v[N];
#pragma unroll
  for (int i = 0; i < N; i++) r[i] = q[b * N + i];
  fwd_reorder<DIM>(v, r);
#pragma unroll
  for (int i = 0; i < N; i++) u[b * N + i] = v[i];
}
// Plane coder alone: block b's code goes to out[b * words_per_block ...],
// preceded by a 9-bit header when header >= 0.
template <int DIM>
__global__ void dbg_planes_kernel(const uint32_t* __restrict__ u, uint64_t nb, uint32_t budget, uint32_t prec,
                                  int header, uint32_t words_per_block, uint64_t* __restrict__ out,
                                  uint32_t* __restrict__ bits) {
  constexpr int N = 1 << (2 * DIM);
  uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nb) return;
  uint32_t v[N];
#pragma unroll
  for (int i = 0; i < N; i++) v[i] = u[b * N + i];
  WordSink sink(out + b * words_per_block);
  if (header >= 0) sink.put((uint64_t)header, 9);
  encode_planes<N>(v, budget, prec, sink);
  bits[b] = (uint32_t)sink.bit_count();
  sink.finish();
}

// Block formation alone (the FPGA design's gather / chunk stage): block b of the
// array, padded at the edges, to blocks[b * 4^DIM ...].
template <int DIM>
__global__ void dbg_gather_kernel(const float* __restrict__ data, uint64_t nx, uint64_t ny, uint64_t nb,
                                  float* __restrict__ blocks) {
  constexpr int N = 1 << (2 * DIM);
  uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nb) return;
  float f[N];
  gather_block<DIM>(f, data, nx, ny, b);
#pragma unroll
  for (int i = 0; i < N; i++) blocks[b * N + i] = f[i];
}
// One whole block (header + planes + padding) per thread into its own words.
template <int DIM>
__global__ void dbg_encode_block_kernel(const float* __restrict__ blocks, uint64_t nb, ZfpParams p,
                                        uint32_t words_per_block, uint64_t* __restrict__ out, uint32_t* __restrict__ bits) {
  constexpr int N = 1 << (2 * DIM);
  uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nb) return;
  float f[N];
#pragma unroll
  for (int i = 0; i < N; i++) f[i] = blocks[b * N + i];
  WordSink sink(out + b * words_per_block);
  bits[b] = encode_block<DIM>(f, p, sink);
  sink.finish();
}

inline int grid_for(uint64_t items, int per_cta = kThreads, int cap = 148 * 16) {
  uint64_t g = (items + per_cta - 1) / per_cta;
  if (g < 1) g = 1;
  if (g > (uint64_t)cap) g = cap;
  return (int)g;
}

inline ZfpParams load_params(const int32_t* p) {
  ZfpParams z;
  z.minbits = (uint32_t)p[0]; z.maxbits = (uint32_t)p[1]; z.maxprec = (uint32_t)p[2]; z.minexp = p[3];
  return z;
}

}  // namespace gcow

using namespace gcow;

#include <mutex>

extern "C" {

// Device pointers of the coder tables on the current device; the tables are
// built on the host and uploaded on the first call per device (a synchronous
// copy, so make that first call outside any stream capture).
int gcow_codec_tables4(const void** etab, const void** dtab, const void** epair, const void** dloop) {
  static std::mutex mu;
  static const void* e_addr[64] = {};
  static const void* d_addr[64] = {};
  static const void* p_addr[64] = {};
  static const void* l_addr[64] = {};
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess || dev < 0 || dev >= 64) return err ? (int)err : -1;
  std::lock_guard<std::mutex> lock(mu);
  if (!e_addr[dev]) {
    static uint16_t he[kEncTabSize], hd[kDecBudgetTabSize];
    static uint32_t hp[kEncPairTabSize], hl[kDecLoopTabSize];
    build_codec_tables(he, hd);
    build_pair_table(hp);
    build_dec_loop_table(hl);
    if ((err = cudaMemcpyToSymbol(g_dec_loop_table, hl, sizeof hl)) != cudaSuccess) return (int)err;
    void* pl = nullptr;
    if ((err = cudaGetSymbolAddress(&pl, g_dec_loop_table)) != cudaSuccess) return (int)err;
    l_addr[dev] = pl;
    if ((err = cudaMemcpyToSymbol(g_enc_table, he, sizeof he)) != cudaSuccess) return (int)err;
    if ((err = cudaMemcpyToSymbol(g_dec_table, hd, sizeof hd)) != cudaSuccess) return (int)err;
    if ((err = cudaMemcpyToSymbol(g_enc_pair_table, hp, sizeof hp)) != cudaSuccess) return (int)err;
    void *pe = nullptr, *pd = nullptr, *pp = nullptr;
    if ((err = cudaGetSymbolAddress(&pe, g_enc_table)) != cudaSuccess) return (int)err;
    if ((err = cudaGetSymbolAddress(&pd, g_dec_table)) != cudaSuccess) return (int)err;
    if ((err = cudaGetSymbolAddress(&pp, g_enc_pair_table)) != cudaSuccess) return (int)err;
    p_addr[dev] = pp;
    d_addr[dev] = pd;
    e_addr[dev] = pe;
  }
  *etab = e_addr[dev];
  *dtab = d_addr[dev];
  *epair = p_addr[dev];
  *dloop = l_addr[dev];
  return 0;
}

int gcow_codec_tables(const void** etab, const void** dtab) {
  const void *pair, *loop;
  return gcow_codec_tables4(etab, dtab, &pair, &loop);
}

// Fixed-rate 1-D encode; maxbits in {16, 32, 64, 128}. `out` holds
// blocks*maxbits/8 bytes (caller rounds the buffer up to 8 bytes).
int gcow_encode_1d_fixed(const float* in, uint64_t n, int maxbits, void* out, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  uint64_t blocks = num_blocks_1d(n);
  if (!blocks) return 0;
  int aligned = ((uintptr_t)in & 15) == 0;
  int g = grid_for(blocks);
  const void *etp, *dtp, *ptp, *ltp;
  if (int rc = gcow_codec_tables4(&etp, &dtp, &ptp, &ltp)) return rc;
  const uint16_t* et = (const uint16_t*)etp;
  const uint32_t* pt = (const uint32_t*)ptp;
  switch (maxbits) {
    case 16: encode_1d_fixed_kernel<16><<<g, kThreads, 0, s>>>(in, n, out, aligned, et, pt); break;
    case 32: encode_1d_fixed_kernel<32><<<g, kThreads, 0, s>>>(in, n, out, aligned, et, pt); break;
    case 64: encode_1d_fixed_kernel<64><<<g, kThreads, 0, s>>>(in, n, out, aligned, et, pt); break;
    case 128: encode_1d_fixed_kernel<128><<<g, kThreads, 0, s>>>(in, n, out, aligned, et, pt); break;
    default: return -1;
  }
  return (int)cudaGetLastError();
}

int gcow_decode_1d_fixed(const void* in, float* out, uint64_t n, int maxbits, int shift, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  uint64_t blocks = num_blocks_1d(n);
  if (!blocks) return 0;
  int aligned = ((uintptr_t)out & 15) == 0;
  int g = grid_for(blocks);
  const void *etp, *dtp, *ptp, *ltp;
  if (int rc = gcow_codec_tables4(&etp, &dtp, &ptp, &ltp)) return rc;
  const uint32_t* lt = (const uint32_t*)ltp;
  const uint16_t* dt = (const uint16_t*)dtp;
  switch (maxbits) {
    case 16: decode_1d_fixed_kernel<16><<<g, kThreads, 0, s>>>(in, out, n, shift, aligned, dt, lt); break;
    case 32: decode_1d_fixed_kernel<32><<<g, kThreads, 0, s>>>(in, out, n, shift, aligned, dt, lt); break;
    case 64: decode_1d_fixed_kernel<64><<<g, kThreads, 0, s>>>(in, out, n, shift, aligned, dt, lt); break;
    case 128: decode_1d_fixed_kernel<128><<<g, kThreads, 0, s>>>(in, out, n, shift, aligned, dt, lt); break;
    default: return -1;
  }
  return (int)cudaGetLastError();
}

// Launch sequence of the generic encoder, shared by the entry point that takes the caller's scratch and the one
// that uses the library's built-in array: slots -> per-block lengths -> prefix sum -> bit-offset scatter.
static int launch_encode_generic(const float* in, uint64_t nx, uint64_t ny, const ZfpParams& p, uint64_t blocks,
                                 uint64_t* out, uint64_t out_bytes, void* scratch, uint64_t* block_bits,
                                 cudaStream_t s) {
  const int dim = ny ? 2 : 1;
  const uint64_t wpb = (max_block_bits(p, dim) + 63) / 64;
  uint64_t* slots = (uint64_t*)scratch;
  uint32_t* lens = (uint32_t*)(slots + wpb * blocks);
  uint64_t* tile_sums = (uint64_t*)((char*)lens + ((blocks * 4 + 7) & ~7ull));
  const uint64_t tiles = (blocks + kScanTile - 1) / kScanTile;
  cudaMemsetAsync(out, 0, out_bytes, s);   // the scatter pass ORs into the stream
  const int g = grid_for(blocks);
  if (dim == 1) encode_slots_kernel<1><<<g, kThreads, 0, s>>>(in, nx, ny, p, blocks, slots, lens);
  else encode_slots_kernel<2><<<g, kThreads, 0, s>>>(in, nx, ny, p, blocks, slots, lens);
  if (is_fixed_rate(p)) {
    fixed_offsets_kernel<<<grid_for(blocks + 1), kThreads, 0, s>>>(blocks, p.maxbits, block_bits);
  } else {
    scan_tile_sums_kernel<<<(unsigned)tiles, kThreads, 0, s>>>(lens, blocks, tile_sums);
    scan_tile_offsets_kernel<<<1, kThreads, 0, s>>>(tile_sums, tiles);
    scan_apply_kernel<<<(unsigned)tiles, kThreads, 0, s>>>(lens, blocks, tile_sums, block_bits);
  }
  scatter_slots_kernel<<<g, kThreads, 0, s>>>(slots, lens, block_bits, blocks, (unsigned long long*)out);
  return (int)cudaGetLastError();
}

// Scratch requirements of the generic encoder, in bytes, for `blocks` blocks.
// Layout: slots (words_per_block * blocks u64) | lens (blocks u32, padded) |
// tile sums (tiles u64).
uint64_t gcow_encode_generic_scratch_bytes(const int32_t* params, uint64_t blocks, int dim) {
  ZfpParams p = load_params(params);
  uint64_t wpb = (max_block_bits(p, dim) + 63) / 64;
  uint64_t tiles = (blocks + kScanTile - 1) / kScanTile;
  return wpb * blocks * 8 + ((blocks * 4 + 7) & ~7ull) + tiles * 8 + 64;
}

// Generic encode (any mode, dim 1 or 2). `out` must hold max_output_bytes and
// is zeroed here; `block_bits` (blocks + 1 u64, device) receives every block's
// start bit and, last, the total bit count. The stream length in bytes is
// ceil(total/64)*8.
int gcow_encode_generic(const float* in, uint64_t nx, uint64_t ny, const int32_t* params, uint64_t* out,
                        uint64_t out_bytes, void* scratch, uint64_t* block_bits, void* stream) {
  ZfpParams p = load_params(params);
  uint64_t blocks = ny ? num_blocks_2d(nx, ny) : num_blocks_1d(nx);
  if (!blocks) return 0;
  return launch_encode_generic(in, nx, ny, p, blocks, out, out_bytes, scratch, block_bits, (cudaStream_t)stream);
}

// Fixed-rate encode without scratch; maxbits must be a multiple of 64 (e.g. 2-D at
// 4, 8, 16 bits/value; 1-D at 16 bits/value and up). `out` holds blocks*maxbits/8 bytes.
int gcow_encode_fixed_direct(const float* in, uint64_t nx, uint64_t ny, const int32_t* params, uint64_t* out,
                             void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  ZfpParams p = load_params(params);
  if (!is_fixed_rate(p) || p.maxbits % 64) return -1;
  uint64_t blocks = ny ? num_blocks_2d(nx, ny) : num_blocks_1d(nx);
  if (!blocks) return 0;
  int g = grid_for(blocks);
  if (ny) encode_fixed_direct_kernel<2><<<g, kThreads, 0, s>>>(in, nx, ny, p, blocks, out);
  else encode_fixed_direct_kernel<1><<<g, kThreads, 0, s>>>(in, nx, ny, p, blocks, out);
  return (int)cudaGetLastError();
}

// Generic decode. block_bits == nullptr means fixed rate (offset b*maxbits).
int gcow_decode_generic(const uint64_t* in, float* out, uint64_t nx, uint64_t ny, const int32_t* params,
                        const uint64_t* block_bits, int shift, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  ZfpParams p = load_params(params);
  uint64_t blocks = ny ? num_blocks_2d(nx, ny) : num_blocks_1d(nx);
  if (!blocks) return 0;
  if (!block_bits && !is_fixed_rate(p)) return -2;
  int g = grid_for(blocks);
  if (ny) decode_generic_kernel<2><<<g, kThreads, 0, s>>>(in, out, nx, ny, p, blocks, block_bits, shift);
  else decode_generic_kernel<1><<<g, kThreads, 0, s>>>(in, out, nx, ny, p, blocks, block_bits, shift);
  return (int)cudaGetLastError();
}

// Stage debug kernels: which = 0 emax, 1 cast, 2 forward transform, 3 inverse
// transform, 4 reorder to negabinary, 5 inverse cast. Arrays hold nb blocks of
// 4^dim values each.
int gcow_dbg_stage(int which, int dim, uint64_t nb, const void* a, void* b, const int* emax, int shift,
                   void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  int g = (int)((nb + 127) / 128);
  if (!nb) return 0;
#define GCOW_DISPATCH(K, ...) do { if (dim == 1) K<1><<<g, 128, 0, s>>>(__VA_ARGS__); else K<2><<<g, 128, 0, s>>>(__VA_ARGS__); } while (0)
  switch (which) {
    case 0: GCOW_DISPATCH(dbg_emax_kernel, (const float*)a, nb, (int*)b); break;
    case 1: GCOW_DISPATCH(dbg_cast_kernel, (const float*)a, nb, emax, (int32_t*)b); break;
    case 2: GCOW_DISPATCH(dbg_xform_kernel, (int32_t*)b, nb, 0); break;
    case 3: GCOW_DISPATCH(dbg_xform_kernel, (int32_t*)b, nb, 1); break;
    case 4: GCOW_DISPATCH(dbg_reorder_kernel, (const int32_t*)a, (uint32_t*)b, nb); break;
    case 5: GCOW_DISPATCH(dbg_inv_cast_kernel, (const int32_t*)a, nb, emax, shift, (float*)b); break;
    default: return -1;
  }
  return (int)cudaGetLastError();
}
int gcow_dbg_gather(int dim, const float* data, uint64_t nx, uint64_t ny, uint64_t nb, float* blocks, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  int g = (int)((nb + 127) / 128);
  if (!nb) return 0;
  GCOW_DISPATCH(dbg_gather_kernel, data, nx, ny, nb, blocks);
  return (int)cudaGetLastError();
}
// out must be zero-initialised by the caller (words_per_block u64 per block).
int gcow_dbg_encode_block(int dim, const float* blocks, uint64_t nb, const int32_t* params, uint32_t words_per_block,
                          uint64_t* out, uint32_t* bits, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  int g = (int)((nb + 127) / 128);
  if (!nb) return 0;
  ZfpParams p = load_params(params);
  GCOW_DISPATCH(dbg_encode_block_kernel, blocks, nb, p, words_per_block, out, bits);
  return (int)cudaGetLastError();
}
int gcow_dbg_planes(int dim, uint64_t nb, const uint32_t* u, uint32_t budget, uint32_t prec, int header,
                    uint32_t words_per_block, uint64_t* out, uint32_t* bits, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  int g = (int)((nb + 127) / 128);
  if (!nb) return 0;
  GCOW_DISPATCH(dbg_planes_kernel, u, nb, budget, prec, header, words_per_block, out, bits);
  return (int)cudaGetLastError();
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Allocation-free variant of gcow_encode_generic (see gcow_static_api.h).
// ---------------------------------------------------------------------------
#include <mutex>
#include <stdio.h>
#include "gcow_static_api.h"

namespace {

constexpr uint64_t kStaticScratchBytes = 8ull << 20;

// Scratch shared by every call on a device. In host code this name is only a
// stand-in for the symbol, not a device address: the address handed to kernels
// comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
void* g_static_addr[kMaxDevices] = {};
thread_local char g_static_err[256] = "";

int static_fail(int code, const char* fmt, unsigned long long a = 0, unsigned long long b = 0) {
  snprintf(g_static_err, sizeof g_static_err, fmt, a, b);
  return code;
}

// Device address of the scratch on the current device; looked up once per device.
int static_scratch_ptr(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return static_fail(GCOW_STATIC_SETUP_FAILED, "cannot identify the current device (cuda error %llu)", (unsigned long long)e);
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (!g_static_addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_static_scratch);
    if (e != cudaSuccess || !p)
      return static_fail(GCOW_STATIC_SETUP_FAILED, "cudaGetSymbolAddress failed with cuda error %llu", (unsigned long long)e);
    g_static_addr[dev] = p;
  }
  *out = g_static_addr[dev];
  return GCOW_STATIC_OK;
}

}  // namespace

extern "C" {

uint64_t gcow_encode_generic_static_capacity(void) { return kStaticScratchBytes; }

const char* gcow_encode_generic_static_error(void) { return g_static_err; }

int gcow_encode_generic_static(const float* in, uint64_t nx, uint64_t ny, const int32_t* params,
                               uint64_t* out, uint64_t out_bytes, uint64_t* block_bits, void* stream) {
  g_static_err[0] = 0;
  if (!in || !params || !out || !block_bits)
    return static_fail(GCOW_STATIC_BAD_ARGS, "null argument");
  ZfpParams p = load_params(params);
  const int dim = ny ? 2 : 1;
  // Every block needs at least 8 bytes of scratch, so a block count beyond capacity / 8 can be refused before
  // any size is multiplied out; extents are bounded first so that the 2-D block count itself cannot wrap.
  const uint64_t max_blocks = kStaticScratchBytes / 8;
  const uint64_t bx = nx / 4 + (nx % 4 != 0), by = ny ? ny / 4 + (ny % 4 != 0) : 1;
  if (bx > max_blocks || by > max_blocks || bx * by > max_blocks)
    return static_fail(GCOW_STATIC_TOO_LARGE,
                       "%llu x %llu values are far beyond what the built-in scratch array can hold; "
                       "split the input or use gcow_encode_generic with your own scratch",
                       (unsigned long long)nx, (unsigned long long)ny);
  const uint64_t blocks = ny ? num_blocks_2d(nx, ny) : num_blocks_1d(nx);
  if (!blocks) return GCOW_STATIC_OK;
  const uint64_t need = gcow_encode_generic_scratch_bytes(params, blocks, dim);
  if (need > kStaticScratchBytes)
    return static_fail(GCOW_STATIC_TOO_LARGE,
                       "request needs %llu bytes of scratch but the built-in array holds %llu; "
                       "split the input or use gcow_encode_generic with your own scratch",
                       (unsigned long long)need, (unsigned long long)kStaticScratchBytes);
  if (out_bytes < max_output_bytes(p, blocks, dim))
    return static_fail(GCOW_STATIC_BAD_ARGS, "output buffer of %llu bytes is smaller than the worst case %llu",
                       (unsigned long long)out_bytes, (unsigned long long)max_output_bytes(p, blocks, dim));
  void* scratch = nullptr;
  int rc = static_scratch_ptr(&scratch);
  if (rc != GCOW_STATIC_OK) return rc;

  const int e = launch_encode_generic(in, nx, ny, p, blocks, out, out_bytes, scratch, block_bits, (cudaStream_t)stream);
  if (e != 0) return static_fail(e, "kernel launch failed with cuda error %llu", (unsigned long long)e);
  return GCOW_STATIC_OK;
}

}  // extern "C"
