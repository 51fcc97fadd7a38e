// Compression parameters and size arithmetic of the ZFP float32 block codec.
//
// The four "expert" parameters (minbits, maxbits, maxprec, minexp) and the
// helpers derived from them are shared by the CUDA kernels, the host launchers
// and the CPU oracle, so every implementation sizes and cuts blocks identically.
//
// Parity with the reference CPU codec:
//   sw/include/common.h:10-13   default parameter values
//   sw/src/common.c:6-21        accuracy mode (minexp from frexp(tolerance) - 1)
//   sw/src/common.c:187-224     worst-case output size
//   sw/src/common.c:226-229     precision of a block from its exponent
//   sw/src/common.c:232-236     "budget can cut this block" predicate
// Fixed-rate and fixed-precision setters follow the upstream ZFP rule (the
// reference only lists those modes in an enum, sw/include/types.h:29-36).
#pragma once
#include <stdint.h>
#include <math.h>

#if defined(__CUDACC__)
#define GCOW_HD __host__ __device__ __forceinline__
#else
#define GCOW_HD inline
#endif

namespace gcow {

constexpr uint32_t kMinBits = 1;       // minimum bits per block
constexpr uint32_t kMaxBits = 16658;   // maximum bits per block
constexpr uint32_t kMaxPrec = 64;      // maximum bit-plane count
constexpr int32_t  kMinExp  = -1074;   // smallest bit-plane exponent kept
constexpr uint32_t kHeaderMaxBits = 148;  // header allowance in the size bound (never written)
constexpr int kEBits = 8;              // exponent bits of float32
constexpr int kEBias = 127;            // exponent bias of float32
constexpr uint32_t kNbMask = 0xaaaaaaaau;  // negabinary conversion mask
constexpr int kHeaderBits = 1 + kEBits;    // non-zero flag + biased exponent

struct ZfpParams {
  uint32_t minbits;
  uint32_t maxbits;
  uint32_t maxprec;
  int32_t  minexp;
};

GCOW_HD ZfpParams default_params() {
  ZfpParams p;
  p.minbits = kMinBits; p.maxbits = kMaxBits; p.maxprec = kMaxPrec; p.minexp = kMinExp;
  return p;
}

// Fixed rate: `rate` bits per value, `dim` in {1,2}. A block can never be
// shorter than its 9-bit header, so low rates are floored at 9 bits/block
// (the reference would underflow `maxbits - 9`, sw/src/encode.c:479-480).
inline ZfpParams params_rate(double rate, int dim) {
  ZfpParams p = default_params();
  uint32_t n = 1u << (2 * dim);
  uint32_t bits = (uint32_t)floor(n * rate + 0.5);
  if (bits < (uint32_t)kHeaderBits) bits = kHeaderBits;
  p.minbits = p.maxbits = bits;
  return p;
}

// Fixed accuracy: absolute error tolerance. 2^minexp <= tolerance < 2^(minexp+1).
inline ZfpParams params_accuracy(double tolerance) {
  ZfpParams p = default_params();
  if (tolerance > 0) {
    int e;
    (void)frexp(tolerance, &e);
    p.minexp = e - 1;
  }
  return p;
}

// Fixed precision: keep `prec` most significant bit planes of every block.
inline ZfpParams params_precision(uint32_t prec) {
  ZfpParams p = default_params();
  p.maxprec = prec < kMaxPrec ? prec : kMaxPrec;
  return p;
}

GCOW_HD bool is_fixed_rate(const ZfpParams& p) { return p.minbits == p.maxbits; }

// Number of bit planes kept for a block whose common exponent is `emax`.
GCOW_HD uint32_t block_precision(int emax, uint32_t maxprec, int minexp, int dim) {
  int v = emax - minexp + 2 * dim + 2;
  if (v < 0) v = 0;
  return maxprec < (uint32_t)v ? maxprec : (uint32_t)v;
}

// True when a block coded at `maxprec` planes can run past `maxbits`.
GCOW_HD bool budget_can_cut(uint32_t maxbits, uint32_t maxprec, uint32_t size) {
  return (maxprec + 1) * size - 1 > maxbits;
}

// Largest possible encoding of one float32 block, in bits.
GCOW_HD uint32_t max_block_bits(const ZfpParams& p, int dim) {
  uint32_t n = 1u << (2 * dim);
  uint32_t prec = p.maxprec < 32u ? p.maxprec : 32u;
  uint32_t bits = kHeaderBits + (n - 1) + n * prec;
  if (bits > p.maxbits) bits = p.maxbits;
  if (bits < p.minbits) bits = p.minbits;
  return bits;
}

GCOW_HD uint64_t num_blocks_1d(uint64_t n) { return (n + 3) / 4; }
GCOW_HD uint64_t num_blocks_2d(uint64_t nx, uint64_t ny) { return ((nx + 3) / 4) * ((ny + 3) / 4); }

// Worst-case stream size in bytes, rounded up to a 64-bit word; includes the
// reference's 148-bit header allowance so buffers sized by either agree.
GCOW_HD uint64_t max_output_bytes(const ZfpParams& p, uint64_t blocks, int dim) {
  uint64_t bits = kHeaderMaxBits + blocks * (uint64_t)max_block_bits(p, dim);
  return ((bits + 63) & ~(uint64_t)63) / 8;
}

// Exact stream size in bytes of a fixed-rate stream (no header), word aligned.
GCOW_HD uint64_t fixed_rate_bytes(const ZfpParams& p, uint64_t blocks) {
  uint64_t bits = blocks * (uint64_t)p.maxbits;
  return ((bits + 63) & ~(uint64_t)63) / 8;
}

}  // namespace gcow
