// Per-block stages of the ZFP float32 codec as host+device inline functions.
//
// One CUDA thread (or one CPU loop iteration) owns one block of 4^DIM values
// and runs every stage in registers: common exponent, block-floating-point
// cast, decorrelating lift, negabinary reorder and the embedded bit-plane
// coder. The same functions compile for the host, so the fast formulation used
// by the kernels is checked on the CPU against the serial oracle.
//
// Stage semantics follow the reference CPU codec:
//   sw/src/encode.c:41-88     gather and padding of partial blocks
//   sw/src/encode.c:128-152   block exponent (frexp, subnormal clamp)
//   sw/src/encode.c:162-187   cast: (int32)(2^(30-emax) * f), C truncation
//   sw/src/encode.c:189-260   forward lift, rows then columns
//   sw/src/encode.c:263-275   negabinary + coefficient order (sw/include/types.h:71-97)
//   sw/src/encode.c:279-339   budgeted embedded coder (group test + unary runs)
//   sw/src/encode.c:457-495   block header: flag bit + 8-bit biased exponent
//   sw/src/decode.c:12-25,44-183,220-253  the inverses
// The budgeted coder emits a prefix of the unbudgeted one (every emitted bit
// depends only on the plane and on the running count n), so encoding is
// "concatenate per-plane codes, cut at the budget".
#pragma once
#include <math.h>
#include <stdint.h>
#include <string.h>
#include "zfp_params.h"

namespace gcow {

// ---------------------------------------------------------------- bit casts
GCOW_HD uint32_t f32_bits(float f) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(f);
#else
  uint32_t u; memcpy(&u, &f, 4); return u;
#endif
}
GCOW_HD float bits_f32(uint32_t u) {
#if defined(__CUDA_ARCH__)
  return __uint_as_float(u);
#else
  float f; memcpy(&f, &u, 4); return f;
#endif
}
GCOW_HD int ctz32(uint32_t x) {  // x != 0
#if defined(__CUDA_ARCH__)
  return __ffs((int)x) - 1;
#else
  return __builtin_ctz(x);
#endif
}
GCOW_HD uint32_t low_mask32(uint32_t n) { return n >= 32 ? 0xffffffffu : ((1u << n) - 1u); }
GCOW_HD uint64_t low_mask64(uint32_t n) { return n >= 64 ? ~0ull : ((1ull << n) - 1ull); }

// 2^e as float32: exact for -149 <= e <= 127, +inf above, 0 below (what
// ldexpf(1, e) returns).
GCOW_HD float pow2f(int e) {
  if (e > 127) return bits_f32(0x7f800000u);
  if (e >= -126) return bits_f32((uint32_t)(e + 127) << 23);
  if (e >= -149) return bits_f32(1u << (e + 149));
  return 0.0f;
}

// float -> int32 with truncation; out-of-range and NaN give INT32_MIN, which
// is what the x86 conversion the reference relies on produces.
GCOW_HD int32_t trunc_to_i32(float v) {
  float a = v < 0 ? -v : v;
  if (!(a < 2147483648.0f)) return (int32_t)0x80000000u;
#if defined(__CUDA_ARCH__)
  return __float2int_rz(v);
#else
  return (int32_t)v;
#endif
}

// ------------------------------------------------------------------ stages
// Exponent e of m >= 0 with m = f * 2^e, 0.5 <= f < 1; -127 for zero, clamped
// to -126 for subnormals. Non-finite input is clamped to the largest exponent.
GCOW_HD int scalar_exponent(float m) {
  if (!(m > 0)) return -kEBias;
  uint32_t ex = (f32_bits(m) >> 23) & 0xffu;
  if (ex == 0) return 1 - kEBias;
  if (ex == 255) ex = 254;
  return (int)ex - 126;
}

template <int N>
GCOW_HD int block_emax(const float* f) {
  float m = 0;
#pragma unroll
  for (int i = 0; i < N; i++) {
    float a = f[i] < 0 ? -f[i] : f[i];
    if (m < a) m = a;
  }
  return scalar_exponent(m);
}

template <int N>
GCOW_HD void fwd_cast(int32_t* q, const float* f, int emax) {
  float scale = pow2f(30 - emax);
#pragma unroll
  for (int i = 0; i < N; i++) q[i] = trunc_to_i32(scale * f[i]);
}

// `shift` folds an exact division by 2^shift into the scale (averaging over a
// power-of-two number of ranks).
template <int N>
GCOW_HD void inv_cast(float* f, const int32_t* q, int emax, int shift = 0) {
  float scale = pow2f(emax - 30 - shift);
#pragma unroll
  for (int i = 0; i < N; i++) f[i] = scale * (float)q[i];
}

GCOW_HD uint32_t asr1(uint32_t v) { return (uint32_t)((int32_t)v >> 1); }

// Forward lift of one 4-vector; wrapping arithmetic, arithmetic shifts.
GCOW_HD void fwd_lift(int32_t& x_, int32_t& y_, int32_t& z_, int32_t& w_) {
  uint32_t x = (uint32_t)x_, y = (uint32_t)y_, z = (uint32_t)z_, w = (uint32_t)w_;
  x += w; x = asr1(x); w -= x;
  z += y; z = asr1(z); y -= z;
  x += z; x = asr1(x); z -= x;
  w += y; w = asr1(w); y -= w;
  w += asr1(y); y -= asr1(w);
  x_ = (int32_t)x; y_ = (int32_t)y; z_ = (int32_t)z; w_ = (int32_t)w;
}

GCOW_HD void inv_lift(int32_t& x_, int32_t& y_, int32_t& z_, int32_t& w_) {
  uint32_t x = (uint32_t)x_, y = (uint32_t)y_, z = (uint32_t)z_, w = (uint32_t)w_;
  y += asr1(w); w -= asr1(y);
  y += w; w <<= 1; w -= y;
  z += x; x <<= 1; x -= z;
  y += z; z <<= 1; z -= y;
  w += x; x <<= 1; x -= w;
  x_ = (int32_t)x; y_ = (int32_t)y; z_ = (int32_t)z; w_ = (int32_t)w;
}

template <int DIM> struct Xform;
template <> struct Xform<1> {
  static GCOW_HD void fwd(int32_t* q) { fwd_lift(q[0], q[1], q[2], q[3]); }
  static GCOW_HD void inv(int32_t* q) { inv_lift(q[0], q[1], q[2], q[3]); }
  static GCOW_HD constexpr int perm(int i) { return i; }
};
template <> struct Xform<2> {
  static GCOW_HD void fwd(int32_t* q) {
#pragma unroll
    for (int y = 0; y < 4; y++) fwd_lift(q[4 * y], q[4 * y + 1], q[4 * y + 2], q[4 * y + 3]);
#pragma unroll
    for (int x = 0; x < 4; x++) fwd_lift(q[x], q[x + 4], q[x + 8], q[x + 12]);
  }
  static GCOW_HD void inv(int32_t* q) {
#pragma unroll
    for (int x = 0; x < 4; x++) inv_lift(q[x], q[x + 4], q[x + 8], q[x + 12]);
#pragma unroll
    for (int y = 0; y < 4; y++) inv_lift(q[4 * y], q[4 * y + 1], q[4 * y + 2], q[4 * y + 3]);
  }
  // Coefficients ordered by total degree i+j, then i^2+j^2.
  static GCOW_HD constexpr int perm(int i) {
    constexpr int P[16] = {0, 1, 4, 5, 2, 8, 6, 9, 3, 12, 10, 7, 13, 11, 14, 15};
    return P[i];
  }
};

GCOW_HD uint32_t int2nb(int32_t x) { return ((uint32_t)x + kNbMask) ^ kNbMask; }
GCOW_HD int32_t nb2int(uint32_t u) { return (int32_t)((u ^ kNbMask) - kNbMask); }

template <int DIM>
GCOW_HD void fwd_reorder(uint32_t* u, const int32_t* q) {
#pragma unroll
  for (int i = 0; i < (1 << (2 * DIM)); i++) u[i] = int2nb(q[Xform<DIM>::perm(i)]);
}
template <int DIM>
GCOW_HD void inv_reorder(int32_t* q, const uint32_t* u) {
#pragma unroll
  for (int i = 0; i < (1 << (2 * DIM)); i++) q[Xform<DIM>::perm(i)] = nb2int(u[i]);
}

// Fill positions n..3 of a 4-vector with stride s: 0 -> zeros, 1 -> a a a a,
// 2 -> a b b a, 3 -> a b c a.
GCOW_HD void pad_partial(float* b, uint32_t n, int s) {
  if (n == 0) b[0] = 0;
  if (n <= 1) b[s] = b[0];
  if (n <= 2) b[2 * s] = b[s];
  if (n <= 3) b[3 * s] = b[0];
}

// --------------------------------------------------------- plane transposes
template <int N>
GCOW_HD uint32_t extract_plane(const uint32_t* u, int k) {
  uint32_t x = 0;
#pragma unroll
  for (int i = 0; i < N; i++) x |= ((u[i] >> k) & 1u) << i;
  return x;
}
template <int N>
GCOW_HD void deposit_plane(uint32_t* u, uint32_t x, int k) {
#pragma unroll
  for (int i = 0; i < N; i++) u[i] |= ((x >> i) & 1u) << k;
}

// ------------------------------------------------------ embedded plane coder
// Code of one bit plane `x` (N bits) given that the first `n` coefficients are
// already significant: n verbatim bits, then group tests and unary runs. `n`
// is advanced. Runs of zeros are skipped with a count-trailing-zeros.
template <int N>
GCOW_HD void encode_plane(uint32_t x, uint32_t& n, uint64_t& code, uint32_t& len) {
  code = x & low_mask32(n);
  len = n;
  x = n >= 32 ? 0 : x >> n;
  while (n < (uint32_t)N) {
    if (!x) { len++; break; }            // negative group test: one 0 bit
    code |= 1ull << len; len++;          // positive group test
    uint32_t z = (uint32_t)ctz32(x);     // z zeros precede the next one-bit
    if (n + z < (uint32_t)N - 1) { code |= 1ull << (len + z); len += z + 1; }
    else len += z;                       // last position: the one-bit is implied
    x >>= z; x >>= 1;
    n += z + 1;
  }
}

// Encode planes 31..kmin into `sink` until `budget` bits are used.
template <int N, class Sink>
GCOW_HD uint32_t encode_planes(const uint32_t* u, uint32_t budget, uint32_t prec, Sink& sink) {
  uint32_t kmin = prec < 32 ? 32 - prec : 0;
  uint32_t bits = budget, n = 0;
  for (uint32_t k = 32; bits && k-- > kmin;) {
    uint32_t x = extract_plane<N>(u, (int)k);
    uint64_t code; uint32_t len;
    encode_plane<N>(x, n, code, len);
    if (len > bits) { len = bits; code &= low_mask64(len); }
    sink.put(code, len);
    bits -= len;
  }
  return budget - bits;
}

// Decode planes k-1..kmin from `src` with `bits` of budget, starting with `n`
// significant coefficients; `u` accumulates. When the budget ends inside a
// unary run the pending one-bit is still placed at the position reached, which
// is what the serial decoder of the reference does.
template <int N, class Src>
GCOW_HD uint32_t decode_planes_from(uint32_t* u, uint32_t bits, uint32_t kmin, uint32_t k,
                                    uint32_t n, Src& src) {
  uint32_t start = bits;
  while (bits && k-- > kmin) {
    uint32_t m = n < bits ? n : bits;
    bits -= m;
    uint32_t x = (uint32_t)src.get(m);
    for (; bits && n < (uint32_t)N; n++) {
      bits--;
      if (src.get(1)) {
        for (; bits && n < (uint32_t)N - 1; n++) {
          bits--;
          if (src.get(1)) break;
        }
        x += 1u << n;
      } else {
        break;
      }
    }
    deposit_plane<N>(u, x, (int)k);
  }
  return start - bits;
}

template <int N, class Src>
GCOW_HD uint32_t decode_planes(uint32_t* u, uint32_t budget, uint32_t prec, Src& src) {
#pragma unroll
  for (int i = 0; i < N; i++) u[i] = 0;
  uint32_t kmin = prec < 32 ? 32 - prec : 0;
  return decode_planes_from<N>(u, budget, kmin, 32, 0, src);
}

// ------------------------------------------------------- memory bit streams
// LSB-first packer into 64-bit words (sw/src/stream.c:61-138 semantics).
struct WordSink {
  uint64_t* out;
  uint64_t acc;
  uint32_t fill;
  uint32_t nw;
  GCOW_HD explicit WordSink(uint64_t* o) : out(o), acc(0), fill(0), nw(0) {}
  GCOW_HD void put(uint64_t v, uint32_t n) {  // 0 <= n <= 64, v < 2^n
    if (!n) return;
    acc |= v << fill;
    uint32_t tot = fill + n;
    if (tot >= 64) {
      out[nw++] = acc;
      acc = fill ? (v >> (64 - fill)) : 0;
      tot -= 64;
    }
    fill = tot;
  }
  GCOW_HD void pad(uint32_t n) {
    while (n) { uint32_t c = n < 64 ? n : 64; put(0, c); n -= c; }
  }
  GCOW_HD uint64_t bit_count() const { return (uint64_t)nw * 64 + fill; }
  GCOW_HD void finish() { if (fill) { out[nw++] = acc; acc = 0; fill = 0; } }
};

// Random-access LSB-first reader over 64-bit words.
struct WordSrc {
  const uint64_t* in;
  uint64_t pos;
  GCOW_HD WordSrc(const uint64_t* i, uint64_t p) : in(i), pos(p) {}
  GCOW_HD uint64_t get(uint32_t n) {  // 0 <= n <= 32
    if (!n) return 0;
    uint32_t o = (uint32_t)(pos & 63);
    uint64_t w = in[pos >> 6] >> o;
    if (o + n > 64) w |= in[(pos >> 6) + 1] << (64 - o);
    pos += n;
    return w & low_mask64(n);
  }
  GCOW_HD void skip(uint64_t n) { pos += n; }
};

// ------------------------------------------------------ generic block codec
// Encode one block of 4^DIM floats. Returns the number of bits emitted,
// including zero padding up to minbits.
template <int DIM, class Sink>
GCOW_HD uint32_t encode_block(const float* f, const ZfpParams& p, Sink& sink) {
  constexpr int N = 1 << (2 * DIM);
  int emax = block_emax<N>(f);
  uint32_t prec = block_precision(emax, p.maxprec, p.minexp, DIM);
  uint32_t biased = prec ? (uint32_t)(emax + kEBias) : 0;
  uint32_t bits;
  if (biased) {
    sink.put(2 * biased + 1, kHeaderBits);
    int32_t q[N];
    uint32_t u[N];
    fwd_cast<N>(q, f, emax);
    Xform<DIM>::fwd(q);
    fwd_reorder<DIM>(u, q);
    bits = kHeaderBits + encode_planes<N>(u, p.maxbits - kHeaderBits, prec, sink);
  } else {
    sink.put(0, 1);
    bits = 1;
  }
  if (bits < p.minbits) { sink.pad(p.minbits - bits); bits = p.minbits; }
  return bits;
}

// Decode one block; the source is advanced by the block's full length
// (including padding up to minbits). `shift` divides the result by 2^shift.
template <int DIM, class Src>
GCOW_HD uint32_t decode_block(float* f, const ZfpParams& p, Src& src, int shift = 0) {
  constexpr int N = 1 << (2 * DIM);
  uint32_t bits = 1;
  if (src.get(1)) {
    int emax = (int)src.get(kEBits) - kEBias;
    bits += kEBits;
    uint32_t prec = block_precision(emax, p.maxprec, p.minexp, DIM);
    uint32_t u[N];
    int32_t q[N];
    bits += decode_planes<N>(u, p.maxbits - kHeaderBits, prec, src);
    inv_reorder<DIM>(q, u);
    Xform<DIM>::inv(q);
    inv_cast<N>(f, q, emax, shift);
  } else {
#pragma unroll
    for (int i = 0; i < N; i++) f[i] = 0;
  }
  if (bits < p.minbits) { src.skip(p.minbits - bits); bits = p.minbits; }
  return bits;
}

// ------------------------------------------- table-driven 1-D block codec
// For blocks of 4 a plane has 16 values and the running count n has 5, so one
// plane is one table lookup. Encoder entry: code (7 bits) | len << 7 | n' << 10.
// Decoder entry, indexed by (n, next 7 stream bits): plane | len << 4 | n' << 7.
constexpr int kEncTabSize = 5 * 16;
constexpr int kDecTabSize = 5 * 128;

GCOW_HD uint16_t make_enc_entry(uint32_t n, uint32_t x) {
  uint64_t code; uint32_t len;
  encode_plane<4>(x, n, code, len);
  return (uint16_t)(code | (len << 7) | (n << 10));
}

struct TinySrc {  // reads from a small integer
  uint32_t v, used;
  GCOW_HD uint64_t get(uint32_t n) {
    uint32_t r = n ? (v & low_mask32(n)) : 0;
    v = n >= 32 ? 0 : v >> n;
    used += n;
    return r;
  }
};

GCOW_HD uint16_t make_dec_entry(uint32_t n, uint32_t peek) {
  uint32_t u[4] = {0, 0, 0, 0};
  TinySrc s{peek, 0};
  // one plane (k = 1 -> plane 0), effectively unlimited budget
  uint32_t m = n;
  uint32_t x = (uint32_t)s.get(m);
  for (; n < 4; n++) {
    if (s.get(1)) {
      for (; n < 3; n++) if (s.get(1)) break;
      x += 1u << n;
    } else break;
  }
  (void)u;
  return (uint16_t)(x | (s.used << 4) | (n << 7));
}

// Decoder entry for a plane when only `a` bits of budget remain (a = 7 stands for
// "7 or more"): index ((n * 8 + a) * 128 + next bits masked to a). When the
// budget ends inside a unary run the pending one-bit lands where the run
// stopped, exactly as in the serial decoder, so one table serves whole planes
// and the ragged end of a block alike. Entry: plane | used << 4 | n' << 7.
constexpr int kDecBudgetTabSize = 5 * 8 * 128;
GCOW_HD uint16_t make_dec_budget_entry(uint32_t n, uint32_t a, uint32_t peek) {
  TinySrc s{peek, 0};
  uint32_t bits = a;
  uint32_t m = n < bits ? n : bits;
  bits -= m;
  uint32_t x = (uint32_t)s.get(m);
  for (; bits && n < 4; n++) {
    bits--;
    if (s.get(1)) {
      for (; bits && n < 3; n++) {
        bits--;
        if (s.get(1)) break;
      }
      x += 1u << n;
    } else {
      break;
    }
  }
  return (uint16_t)(x | ((a - bits) << 4) | (n << 7));
}

// OR the bits of v (up to 32) in at bit `pos` of a little-endian array of NW
// 32-bit words; bits past the array fall off.
template <int NW>
GCOW_HD void reg_put(uint32_t (&w)[NW], uint32_t pos, uint32_t v) {
#pragma unroll
  for (int i = 0; i < NW; i++) {
    int lo = (int)pos - 32 * i;
    if (lo >= 0 && lo < 32) w[i] |= v << lo;
    else if (lo < 0 && lo > -32) w[i] |= v >> (-lo);
  }
}
// The 32 bits starting at bit `pos` (zeros past the array).
template <int NW>
GCOW_HD uint32_t reg_peek(const uint32_t (&w)[NW], uint32_t pos) {
  uint32_t r = 0;
#pragma unroll
  for (int i = 0; i < NW; i++) {
    int lo = (int)pos - 32 * i;
    if (lo >= 0 && lo < 32) r |= w[i] >> lo;
    else if (lo < 0 && lo > -32) r |= w[i] << (-lo);
  }
  return r;
}
template <int NW>
struct RegSrc {
  const uint32_t (&w)[NW];
  uint32_t pos;
  GCOW_HD uint64_t get(uint32_t n) {  // n <= 7 here
    if (!n) return 0;
    uint32_t r = reg_peek<NW>(w, pos) & low_mask32(n);
    pos += n;
    return r;
  }
};

GCOW_HD uint32_t brev32(uint32_t x) {
#if defined(__CUDA_ARCH__)
  return __brev(x);
#else
  x = ((x >> 1) & 0x55555555u) | ((x & 0x55555555u) << 1);
  x = ((x >> 2) & 0x33333333u) | ((x & 0x33333333u) << 2);
  x = ((x >> 4) & 0x0f0f0f0fu) | ((x & 0x0f0f0f0fu) << 4);
  x = ((x >> 8) & 0x00ff00ffu) | ((x & 0x00ff00ffu) << 8);
  return (x >> 16) | (x << 16);
#endif
}
GCOW_HD uint32_t clz32(uint32_t x) {  // x != 0
#if defined(__CUDA_ARCH__)
  return (uint32_t)__clz((int)x);
#else
  return (uint32_t)__builtin_clz(x);
#endif
}
// low 8 bits -> every 4th bit, and back
GCOW_HD uint32_t spread4(uint32_t x) {
  x &= 0xffu;
  x = (x | (x << 12)) & 0x000f000fu;
  x = (x | (x << 6)) & 0x03030303u;
  x = (x | (x << 3)) & 0x11111111u;
  return x;
}
GCOW_HD uint32_t compact4(uint32_t x) {
  x &= 0x11111111u;
  x = (x | (x >> 3)) & 0x03030303u;
  x = (x | (x >> 6)) & 0x000f000fu;
  x = (x | (x >> 12)) & 0xffu;
  return x;
}
// Bit planes k-1 .. k-8 of four values as eight nibbles in stream order
// (plane k-1 in the low nibble, value i in bit i of a nibble); 1 <= k <= 32.
GCOW_HD uint32_t plane_group(const uint32_t* u, uint32_t k) {
  const uint32_t s = 32 - k;
  return spread4(brev32(u[0] << s)) | (spread4(brev32(u[1] << s)) << 1) |
         (spread4(brev32(u[2] << s)) << 2) | (spread4(brev32(u[3] << s)) << 3);
}
GCOW_HD void deposit_group(uint32_t* u, uint32_t T, uint32_t k) {
  const uint32_t s = 32 - k;
#pragma unroll
  for (int i = 0; i < 4; i++) u[i] |= brev32(compact4(T >> i)) >> s;
}

// Encode one block of 4 into NW 32-bit words (maxbits <= 32*NW). Returns the
// bit count including padding to minbits.
//
// Three shortcuts over the plane-by-plane loop, all bit-identical to it:
// leading all-zero planes cost one 0 bit each and are skipped with a
// count-leading-zeros; planes are transposed eight at a time (plane_group);
// and once all four coefficients are significant every further plane is four
// verbatim bits, i.e. the rest of the transposed group is appended as is.
template <int NW>
GCOW_HD uint32_t encode_block_1d_fast(const float* f, const ZfpParams& p, const uint16_t* etab,
                                      uint32_t (&w)[NW]) {
#pragma unroll
  for (int i = 0; i < NW; i++) w[i] = 0;
  int emax = block_emax<4>(f);
  uint32_t prec = block_precision(emax, p.maxprec, p.minexp, 1);
  uint32_t pos;
  if (prec && emax + kEBias) {
    w[0] = 2u * (uint32_t)(emax + kEBias) + 1u;
    pos = kHeaderBits;
    int32_t q[4];
    uint32_t u[4];
    fwd_cast<4>(q, f, emax);
    fwd_lift(q[0], q[1], q[2], q[3]);
#pragma unroll
    for (int i = 0; i < 4; i++) u[i] = int2nb(q[i]);
    const uint32_t kmin = prec < 32 ? 32 - prec : 0;
    const uint32_t end = p.maxbits;
    uint32_t n = 0, k = 32;
    const uint32_t m = u[0] | u[1] | u[2] | u[3];
    uint32_t z = m ? clz32(m) : 32u;
    if (z > 32 - kmin) z = 32 - kmin;
    pos += z;  // one 0 bit per all-zero plane
    k -= z;
    while (pos < end && k > kmin) {
      const uint32_t T = plane_group(u, k);
      const uint32_t cnt = k - kmin < 8 ? k - kmin : 8;
      uint32_t j = 0;
      while (n < 4 && j < cnt && pos < end) {
        uint32_t e = etab[n * 16 + ((T >> (4 * j)) & 15u)];
        reg_put<NW>(w, pos, e & 0x7fu);
        pos += (e >> 7) & 7u;
        n = e >> 10;
        j++;
      }
      if (j < cnt && pos < end) {  // n == 4: the remaining planes of the group are verbatim
        uint32_t nb = 4 * (cnt - j);
        reg_put<NW>(w, pos, (T >> (4 * j)) & low_mask32(nb));
        pos += nb;
      }
      k -= cnt;
    }
    if (pos > end) {  // cut the last code at the budget
#pragma unroll
      for (int i = 0; i < NW; i++) {
        if (end <= 32u * i) w[i] = 0;
        else if (end < 32u * (i + 1)) w[i] &= low_mask32(end - 32u * i);
      }
      pos = end;
    }
  } else {
    pos = 1;
  }
  return pos < p.minbits ? p.minbits : pos;
}

// Decode one block of 4 held in NW 32-bit words; mirror of the encoder's
// shortcuts. Codes are looked up whole only while at least 7 bits of budget
// remain; the last few bits before all coefficients are significant go through
// the serial routine, which has the exact semantics at the budget edge.
template <int NW>
GCOW_HD void decode_block_1d_fast(float* f, const ZfpParams& p, const uint16_t* dtab,
                                  const uint32_t (&w)[NW], int shift = 0) {
  if (!(w[0] & 1u)) {
    f[0] = f[1] = f[2] = f[3] = 0;
    return;
  }
  int emax = (int)((w[0] >> 1) & 0xffu) - kEBias;
  uint32_t prec = block_precision(emax, p.maxprec, p.minexp, 1);
  const uint32_t kmin = prec < 32 ? 32 - prec : 0;
  uint32_t u[4] = {0, 0, 0, 0};
  uint32_t pos = kHeaderBits, n = 0, k = 32;
  const uint32_t end = p.maxbits;
  {  // leading all-zero planes
    uint32_t avail = end - pos;
    uint32_t S = reg_peek<NW>(w, pos) & low_mask32(avail);
    uint32_t z = S ? (uint32_t)ctz32(S) : 32u;
    if (z > avail) z = avail;
    if (z > 32 - kmin) z = 32 - kmin;
    pos += z;
    k -= z;
  }
  while (pos < end && k > kmin) {
    const uint32_t cnt = k - kmin < 8 ? k - kmin : 8;
    uint32_t T = 0, j = 0;
    while (n < 4 && j < cnt && end - pos >= 7) {
      uint32_t e = dtab[n * 128 + (reg_peek<NW>(w, pos) & 127u)];
      T |= (e & 15u) << (4 * j);
      pos += (e >> 4) & 7u;
      n = e >> 7;
      j++;
    }
    if (n == 4 && j < cnt && pos < end) {  // verbatim planes
      uint32_t nb = 4 * (cnt - j), avail = end - pos;
      uint32_t take = nb < avail ? nb : avail;
      T |= (reg_peek<NW>(w, pos) & low_mask32(take)) << (4 * j);
      pos += take;
      j = cnt;
    }
    if (T) deposit_group(u, T, k);
    if (j < cnt) {  // budget nearly spent before all coefficients became significant
      RegSrc<NW> src{w, pos};
      decode_planes_from<4>(u, end - pos, kmin, k - j, n, src);
      break;
    }
    k -= cnt;
  }
  int32_t q[4];
#pragma unroll
  for (int i = 0; i < 4; i++) q[i] = nb2int(u[i]);
  inv_lift(q[0], q[1], q[2], q[3]);
  inv_cast<4>(f, q, emax, shift);
}

// ------------------------------------------- fixed-rate 1-D block codec
// Specialisation of the table-driven coder for fixed rate with BITS bits per
// block (16, 32, 64 or 128). In fixed-rate mode minexp is -1074, so every block
// keeps all 32 planes (kmin = 0) and only the bit budget ends a block. The
// exponent arithmetic is done on the float's bit pattern, and eight planes of
// the four coefficients are transposed at once with byte permutes, one bit
// reversal and four delta swaps.
GCOW_HD uint32_t byte_perm(uint32_t x, uint32_t y, uint32_t sel) {
#if defined(__CUDA_ARCH__)
  return __byte_perm(x, y, sel);
#else
  uint64_t v = ((uint64_t)y << 32) | x;
  uint32_t r = 0;
  for (int i = 0; i < 4; i++) r |= (uint32_t)((v >> (8 * ((sel >> (4 * i)) & 7))) & 0xff) << (8 * i);
  return r;
#endif
}
GCOW_HD uint32_t delta_swap(uint32_t x, uint32_t mask, int d) {
  uint32_t t = ((x >> d) ^ x) & mask;
  return x ^ t ^ (t << d);
}
// Planes k-1 .. k-8 of u[0..3] as eight nibbles in stream order (see plane_group).
GCOW_HD uint32_t plane_group8(const uint32_t* u, uint32_t k) {
  const uint32_t s = 32 - k;
  // top bytes, value 3 in the low byte
  uint32_t t0 = byte_perm(u[3] << s, u[2] << s, 0x0073);
  uint32_t t1 = byte_perm(u[1] << s, u[0] << s, 0x0073);
  uint32_t r = brev32(byte_perm(t0, t1, 0x5410));   // bit 8i+j = plane k-1-j of value i
  r = delta_swap(r, 0x0000f0f0u, 12);               // 4x8 -> 8x4 bit-matrix transpose
  r = delta_swap(r, 0x00cc00ccu, 6);
  r = delta_swap(r, 0x0a0a0a0au, 3);
  r = delta_swap(r, 0x22222222u, 1);
  return r;
}
GCOW_HD void deposit_group8(uint32_t* u, uint32_t T, uint32_t k) {
  const uint32_t s = 32 - k;
  T = delta_swap(T, 0x22222222u, 1);
  T = delta_swap(T, 0x0a0a0a0au, 3);
  T = delta_swap(T, 0x00cc00ccu, 6);
  T = delta_swap(T, 0x0000f0f0u, 12);
  const uint32_t pk = brev32(T);                    // byte 3-i = top byte of value i
  u[0] |= (pk & 0xff000000u) >> s;
  u[1] |= ((pk << 8) & 0xff000000u) >> s;
  u[2] |= ((pk << 16) & 0xff000000u) >> s;
  u[3] |= (pk << 24) >> s;
}

template <int BITS>
GCOW_HD void encode_block_1d_rate(const float* f, const uint16_t* etab, uint32_t (&w)[(BITS + 31) / 32]) {
  constexpr int NW = (BITS + 31) / 32;
#pragma unroll
  for (int i = 0; i < NW; i++) w[i] = 0;
  float m = 0;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    float a = f[i] < 0 ? -f[i] : f[i];
    if (m < a) m = a;
  }
  const uint32_t mb = f32_bits(m);
  if (mb == 0) return;                           // all zero: a single 0 bit
  uint32_t ex = mb >> 23;                        // emax = ex - 126 (subnormals: ex = 0 -> -126)
  if (ex > 254) ex = 254;
  w[0] = 2u * ex + 3u;                           // flag bit + biased exponent (emax + 127 = ex + 1)
  const float scale = bits_f32(ex >= 29 ? (283u - ex) << 23 : 0x7f800000u);   // 2^(30 - emax)
  int32_t q[4];
  uint32_t u[4];
#pragma unroll
  for (int i = 0; i < 4; i++) q[i] = trunc_to_i32(scale * f[i]);
  fwd_lift(q[0], q[1], q[2], q[3]);
#pragma unroll
  for (int i = 0; i < 4; i++) u[i] = int2nb(q[i]);
  const uint32_t mm = u[0] | u[1] | u[2] | u[3];
  const uint32_t z = mm ? clz32(mm) : 32u;
  uint32_t pos = kHeaderBits + z, k = 32 - z, n = 0;
  while (pos < (uint32_t)BITS && k > 0) {
    uint32_t T = plane_group8(u, k);
    const uint32_t cnt = k < 8 ? k : 8;
    // one table row per significance count, including n = 4 (four verbatim bits)
    for (uint32_t j = 0; j < cnt && pos < (uint32_t)BITS; j++, T >>= 4) {
      if (NW > 1 && n == 4) {                    // long blocks: append the rest of the group at once
        reg_put<NW>(w, pos, T);
        pos += 4 * (cnt - j);
        break;
      }
      const uint32_t e = etab[n * 16 + (T & 15u)];
      if (NW == 1) w[0] |= (e & 0x7fu) << pos; else reg_put<NW>(w, pos, e & 0x7fu);
      pos += (e >> 7) & 7u;
      n = e >> 10;
    }
    k -= cnt;
  }
  if (BITS < 32 * NW) w[NW - 1] &= low_mask32(BITS - 32 * (NW - 1));
}

// `dtab` is the budget-aware table (kDecBudgetTabSize entries).
template <int BITS>
GCOW_HD void decode_block_1d_rate(float* f, const uint16_t* dtab, const uint32_t (&w)[(BITS + 31) / 32],
                                  int shift = 0, uint32_t kmin = 0) {
  constexpr int NW = (BITS + 31) / 32;
  if (!(w[0] & 1u)) {
    f[0] = f[1] = f[2] = f[3] = 0;
    return;
  }
  const uint32_t planemask = 0xffffffffu << kmin;               // planes below kmin are not part of the block
  const int emax = (int)((w[0] >> 1) & 0xffu) - kEBias;
  uint32_t u[4] = {0, 0, 0, 0};
  uint32_t pos = kHeaderBits, n = 0, k = 32;
  constexpr uint32_t end = BITS;
  {
    const uint32_t avail = end - pos;
    const uint32_t S = (NW == 1 ? (w[0] >> pos) : reg_peek<NW>(w, pos)) & low_mask32(avail);
    uint32_t z = S ? (uint32_t)ctz32(S) : 32u;
    if (z > avail) z = avail;
    pos += z;
    k -= z;
  }
  while (pos < end && k > 0) {
    const uint32_t cnt = k < 8 ? k : 8;
    uint32_t T = 0;
    for (uint32_t j = 0; j < cnt && pos < end; j++) {
      const uint32_t avail = end - pos;
      const uint32_t pk = NW == 1 ? (w[0] >> pos) : reg_peek<NW>(w, pos);
      if (NW > 1 && n == 4) {                    // verbatim planes of a long block in one go
        const uint32_t nb = 4 * (cnt - j);
        const uint32_t take = nb < avail ? nb : avail;
        T |= (pk & low_mask32(take)) << (4 * j);
        pos += take;
        break;
      }
      const uint32_t a = avail < 7 ? avail : 7;
      const uint32_t e = dtab[((n * 8 + a) << 7) + (pk & low_mask32(a))];
      T |= (e & 15u) << (4 * j);
      pos += (e >> 4) & 7u;
      n = e >> 7;
    }
    if (T) deposit_group8(u, T, k);
    k -= cnt;
  }
  int32_t q[4];
#pragma unroll
  for (int i = 0; i < 4; i++) q[i] = nb2int(u[i] & planemask);
  inv_lift(q[0], q[1], q[2], q[3]);
  inv_cast<4>(f, q, emax, shift);
}

// Host-side construction of both tables (the kernels copy them from global memory).
inline void build_codec_tables(uint16_t* etab, uint16_t* dtab_budget) {
  for (uint32_t i = 0; i < (uint32_t)kEncTabSize; i++) etab[i] = make_enc_entry(i >> 4, i & 15);
  for (uint32_t i = 0; i < (uint32_t)kDecBudgetTabSize; i++) {
    const uint32_t n = i >> 10, a = (i >> 7) & 7, pk = i & 127;
    dtab_budget[i] = make_dec_budget_entry(n, a, pk & low_mask32(a));
  }
}

// ------------------------------------------- lean fixed-rate 1-D block codec
// The coder above walks a block plane by plane with a data-dependent trip count, so
// the 32 lanes of a warp (one block each) spend much of their time waiting for the
// slowest lane. The functions below produce the same bits with warp-uniform control
// flow and fewer integer instructions:
//
//  * encoder: the top eight bit planes are coded two planes per table lookup, four
//    lookups for every lane. The table index (two planes of four coefficients) is
//    gathered from the top bytes with one mask and one multiply, so no bit-matrix
//    transpose is needed. A plane at significance count n >= 3 is always the four
//    coefficient bits verbatim (with n = 3 the group-test bit IS bit 3), so longer
//    blocks append the remaining planes as transposed nibbles.
//  * decoder: planes are looked up one at a time only until n reaches 3; the rest of
//    the block is verbatim nibbles taken from the stream in one shift.
//
// Inputs the fast path does not cover (a non-finite or vanishing block maximum, a NaN
// member, data so smooth that eight planes do not reach n >= 3 or fill the budget)
// return to encode_block_1d_rate / decode_block_1d_rate above, which stay the
// definition. The serial oracle and the reference build are the tests' yardstick for
// both (sw/src/encode.c:279-339,457-495; sw/src/decode.c:141-183,220-253).

// Two planes per lookup: index n * 256 + g, where bit 7-2i of g is coefficient i's
// bit in the first (higher) plane and bit 6-2i its bit in the second plane.
// Entry: code (14 bits) | length << 16 | (n' - n) << 24, so that adding an entry to a
// packed state [junk:16 | position:8 | n:8] advances position and n at once.
constexpr int kEncPairTabSize = 5 * 256;
GCOW_HD uint32_t make_enc_pair_entry(uint32_t n, uint32_t g) {
  uint32_t x1 = 0, x2 = 0;
  for (int i = 0; i < 4; i++) {
    x1 |= ((g >> (7 - 2 * i)) & 1u) << i;
    x2 |= ((g >> (6 - 2 * i)) & 1u) << i;
  }
  const uint32_t n0 = n;
  uint64_t c1, c2; uint32_t l1, l2;
  encode_plane<4>(x1, n, c1, l1);
  encode_plane<4>(x2, n, c2, l2);
  return (uint32_t)(c1 | (c2 << l1)) | ((l1 + l2) << 16) | ((n - n0) << 24);
}

GCOW_HD uint32_t shl_sat(uint32_t v, uint32_t s) {   // v << s, 0 for s >= 32
#if defined(__CUDA_ARCH__)
  uint32_t r; asm("shl.b32 %0, %1, %2;" : "=r"(r) : "r"(v), "r"(s)); return r;
#else
  return s < 32 ? v << s : 0u;
#endif
}
GCOW_HD uint32_t shr_sat(uint32_t v, uint32_t s) {   // v >> s, 0 for s >= 32
#if defined(__CUDA_ARCH__)
  uint32_t r; asm("shr.u32 %0, %1, %2;" : "=r"(r) : "r"(v), "r"(s)); return r;
#else
  return s < 32 ? v >> s : 0u;
#endif
}

// BITS bits held in registers, addressed by bit position.
template <int NW> struct BitBuf;
template <> struct BitBuf<1> {
  uint32_t a;
  GCOW_HD void clear() { a = 0; }
  GCOW_HD void load(const uint32_t (&w)[1]) { a = w[0]; }
  GCOW_HD void store(uint32_t (&w)[1]) const { w[0] = a; }
  GCOW_HD void put(uint32_t pos, uint32_t v) { a |= shl_sat(v, pos); }
  GCOW_HD uint32_t peek(uint32_t pos) const { return shr_sat(a, pos); }
};
template <> struct BitBuf<2> {
  uint64_t a;
  GCOW_HD void clear() { a = 0; }
  GCOW_HD void load(const uint32_t (&w)[2]) { a = (uint64_t)w[0] | ((uint64_t)w[1] << 32); }
  GCOW_HD void store(uint32_t (&w)[2]) const { w[0] = (uint32_t)a; w[1] = (uint32_t)(a >> 32); }
  GCOW_HD void put(uint32_t pos, uint32_t v) { if (pos < 64) a |= (uint64_t)v << pos; }
  GCOW_HD uint32_t peek(uint32_t pos) const { return pos < 64 ? (uint32_t)(a >> pos) : 0u; }
};
template <> struct BitBuf<4> {
  uint64_t lo, hi;
  GCOW_HD void clear() { lo = hi = 0; }
  GCOW_HD void load(const uint32_t (&w)[4]) {
    lo = (uint64_t)w[0] | ((uint64_t)w[1] << 32); hi = (uint64_t)w[2] | ((uint64_t)w[3] << 32);
  }
  GCOW_HD void store(uint32_t (&w)[4]) const {
    w[0] = (uint32_t)lo; w[1] = (uint32_t)(lo >> 32); w[2] = (uint32_t)hi; w[3] = (uint32_t)(hi >> 32);
  }
  GCOW_HD void put(uint32_t pos, uint32_t v) {
    if (pos < 64) {
      lo |= (uint64_t)v << pos;
      if (pos > 32) hi |= (uint64_t)v >> (64 - pos);
    } else if (pos < 128) {
      hi |= (uint64_t)v << (pos - 64);
    }
  }
  GCOW_HD uint32_t peek(uint32_t pos) const {
    if (pos < 64) {
      uint64_t r = lo >> pos;
      if (pos > 32) r |= hi << (64 - pos);
      return (uint32_t)r;
    }
    return pos < 128 ? (uint32_t)(hi >> (pos - 64)) : 0u;
  }
};

// Decoder loop table: one plane per lookup while fewer than three coefficients are significant.
// Byte offset n * 4096 + a * 512 + peek * 4 (n = 0..2, a = remaining budget capped at 7, peek = next 7
// stream bits). Entry: plane nibble | bits used << 8 | (n' * 4096) << 16 - the last field is the row
// offset of the next lookup, and n' >= 3 ends the loop.
constexpr int kDecLoopTabSize = 3 * 8 * 128;
GCOW_HD uint32_t make_dec_loop_entry(uint32_t n, uint32_t a, uint32_t peek) {
  const uint32_t e = make_dec_budget_entry(n, a, peek & low_mask32(a));      // plane | used << 4 | n' << 7
  return (e & 15u) | (((e >> 4) & 7u) << 8) | ((e >> 7) << 28);
}

GCOW_HD uint32_t funnel_r(uint32_t lo, uint32_t hi, uint32_t s) {   // low word of (hi:lo) >> s, 0 < s < 32
#if defined(__CUDA_ARCH__)
  return __funnelshift_r(lo, hi, s);
#else
  return (lo >> s) | (hi << (32 - s));
#endif
}

struct LeanTables {
  const uint16_t* etab;    // kEncTabSize: one plane per lookup (definition path; rarely used, may be global memory)
  const uint16_t* dtab;    // kDecBudgetTabSize: budget-aware, one plane per lookup (definition path, likewise)
  const uint32_t* epair;   // kEncPairTabSize: two planes per lookup
  const uint32_t* dloop;   // kDecLoopTabSize: decoder loop while n < 3
};

template <int BITS>
GCOW_HD void encode_block_1d_lean(const float* f, const LeanTables& t, uint32_t (&w)[(BITS + 31) / 32],
                                  uint32_t kmin = 0) {   // planes below kmin need not be coded (what follows them is ignored)
  constexpr int NW = (BITS + 31) / 32;
  const float a01 = fmaxf(fabsf(f[0]), fabsf(f[1])), a23 = fmaxf(fabsf(f[2]), fabsf(f[3]));
  const uint32_t mb = f32_bits(fmaxf(a01, a23));
  if (mb == 0) {
#pragma unroll
    for (int i = 0; i < NW; i++) w[i] = 0;
    return;
  }
  const uint32_t ex = mb >> 23;
  if (ex < 29 || ex > 254) { encode_block_1d_rate<BITS>(f, t.etab, w); return; }
  const float scale = bits_f32((283u - ex) << 23);           // 2^(30 - emax), emax = ex - 126
  const float p0 = scale * f[0], p1 = scale * f[1], p2 = scale * f[2], p3 = scale * f[3];
  if (!(fabsf((p0 + p1) + (p2 + p3)) < 8.0e9f)) { encode_block_1d_rate<BITS>(f, t.etab, w); return; }   // a NaN member
  int32_t q[4];
#if defined(__CUDA_ARCH__)
  q[0] = __float2int_rz(p0); q[1] = __float2int_rz(p1); q[2] = __float2int_rz(p2); q[3] = __float2int_rz(p3);
#else
  q[0] = (int32_t)p0; q[1] = (int32_t)p1; q[2] = (int32_t)p2; q[3] = (int32_t)p3;
#endif
  fwd_lift(q[0], q[1], q[2], q[3]);
  uint32_t u[4];
#pragma unroll
  for (int i = 0; i < 4; i++) u[i] = int2nb(q[i]);
  const uint32_t mm = u[0] | u[1] | u[2] | u[3];
  uint32_t z = mm ? clz32(mm) : 32u;
  if (z > 24) z = 24;                                         // further zero planes go through the table (one 0 bit each)
  const uint32_t sh = 24 - z;
  const uint32_t R = (u[0] >> sh) | ((u[1] >> sh) << 8) | ((u[2] >> sh) << 16) | ((u[3] >> sh) << 24);
  BitBuf<NW> buf;
  buf.clear();
  buf.put(0, 2u * ex + 3u);                                   // flag bit + biased exponent (emax + 127 = ex + 1)
  uint32_t S = (kHeaderBits + z) << 16;                       // [junk:16 | position:8 | n:8]
  constexpr int kPairs = BITS == 16 ? 2 : 4;                  // 16-bit blocks: four planes always exceed 7 payload bits
#pragma unroll
  for (int j = 0; j < kPairs; j++) {
    const uint32_t x = (R >> (6 - 2 * j)) & 0x03030303u;
    const uint32_t g = (x * 0x40100401u) >> 24;               // the four 2-bit fields side by side
    const uint32_t e = t.epair[(S >> 24) * 256u + g];
    buf.put((S >> 16) & 0xffu, e & 0x3fffu);
    S += e;
  }
  uint32_t pos = (S >> 16) & 0xffu, n = S >> 24, k = 32 - z - 2 * kPairs;
  if (NW > 1) {
    // the remaining planes are verbatim nibbles once n >= 3
    while (n >= 3 && pos < (uint32_t)BITS && k > kmin) {
      buf.put(pos, plane_group8(u, k));
      const uint32_t cnt = k < 8 ? k : 8;
      pos += 4 * cnt;
      k -= cnt;
    }
  }
  if (pos < (uint32_t)BITS && k > kmin) { encode_block_1d_rate<BITS>(f, t.etab, w); return; }   // very smooth block
  buf.store(w);
  if (BITS < 32 * NW) w[NW - 1] &= low_mask32(BITS - 32 * (NW - 1));
}

template <int BITS>
GCOW_HD void decode_block_1d_lean(float* f, const LeanTables& t, const uint32_t (&w)[(BITS + 31) / 32],
                                  int shift = 0, uint32_t kmin = 0) {
  constexpr int NW = (BITS + 31) / 32;
  if (!(w[0] & 1u)) {
    f[0] = f[1] = f[2] = f[3] = 0;
    return;
  }
  const uint32_t planemask = 0xffffffffu << kmin;               // planes below kmin are not part of the block
  const uint32_t e8 = (w[0] >> 1) & 0xffu;                     // biased exponent, emax + 127
  BitBuf<NW> buf;
  buf.load(w);
  constexpr uint32_t end = BITS;
  // leading all-zero planes: one 0 bit each; a sentinel bit ends the count at the budget (or at 32 planes)
  constexpr uint32_t kPayload = end - kHeaderBits;
  const uint32_t lead = buf.peek(kHeaderBits);
  const uint32_t z = kPayload < 32 ? (uint32_t)ctz32(lead | (1u << (kPayload < 32 ? kPayload : 0)))
                                   : (lead ? (uint32_t)ctz32(lead) : 32u);
  uint32_t pos = kHeaderBits + z;
  const uint32_t ktop = 32 - z;                                // planes ktop-1 .. 0 remain
  // planes with n < 3: one budget-aware lookup each, at most eight of them here
  uint32_t nrow = 0, j4 = 0, T = 0;                            // nrow = n * 4096, the table row's byte offset
#pragma unroll
  for (int c = 0; c < 8; c++) {
    if (!(nrow < 3u * 4096u && pos < end && (NW == 1 || (uint32_t)c < ktop))) break;
    const uint32_t avail = end - pos;
    const uint32_t a = avail < 7 ? avail : 7;
    const uint32_t pk = buf.peek(pos) & 127u;                  // bits past the block's end read as 0
    const uint32_t e = *reinterpret_cast<const uint32_t*>(reinterpret_cast<const char*>(t.dloop) + nrow + a * 512u + pk * 4u);
    T = funnel_r(T, e, 4);                                     // newest plane enters at the top nibble
    pos += (e >> 8) & 0xffu;
    nrow = e >> 16;
    j4 += 4;
  }
  if (nrow < 3u * 4096u && pos < end && j4 < 4 * ktop && ktop - (j4 >> 2) > kmin) {   // very smooth block
    decode_block_1d_rate<BITS>(f, t.dtab, w, shift, kmin);
    return;
  }
  T = shr_sat(T, 32 - j4);                                     // first plane in the low nibble
  uint32_t u[4] = {0, 0, 0, 0};
  uint32_t k = ktop;
  if (NW == 1) {
    // the rest of the block is verbatim nibbles: at most 16 planes in all, two transposed words
    const uint32_t tail = buf.peek(pos);
    T |= shl_sat(tail, j4);
    const uint32_t T1 = j4 ? shr_sat(tail, 32 - j4) : 0u;
    deposit_group8(u, T, k);
    if (T1 && k > 8) deposit_group8(u, T1, k - 8);
  } else {
    if (T) deposit_group8(u, T, k);
    k -= j4 >> 2;
    while (pos < end && k > kmin) {
      deposit_group8(u, buf.peek(pos), k);           // bits past the block's end read as 0
      pos += 32;
      k = k > 8 ? k - 8 : 0;
    }
  }
  int32_t q[4];
#pragma unroll
  for (int i = 0; i < 4; i++) q[i] = nb2int(u[i] & planemask);
  inv_lift(q[0], q[1], q[2], q[3]);
  // 2^(emax - 30 - shift): a normal float unless the block is tiny
  const int ef = (int)e8 - 30 - shift;
  const float scale = (ef >= 1 && ef <= 254) ? bits_f32((uint32_t)ef << 23) : pow2f((int)e8 - kEBias - 30 - shift);
#pragma unroll
  for (int i = 0; i < 4; i++) f[i] = scale * (float)q[i];
}

// Fixed accuracy with a bit cap (minexp from the tolerance, maxbits = BITS, minbits = 1): a block keeps the planes
// 31 .. 32 - prec, prec = block_precision(emax, ., minexp, 1), as far as the cap allows. The embedded code of those
// planes is a prefix of the fixed-rate code, so the fixed-rate encoder serves unchanged and the decoder only has to
// drop what it read of the planes below: `kmin` of the coders above (which also keeps them on their fast path when
// the planes that count end before the bit budget does). A block with prec = 0 (everything below
// the tolerance) or all zeros is a single 0 bit in the stream; callers send nothing for it.
// Lowest plane kept, from a kept block's header word (32 - prec, at most 31).
GCOW_HD uint32_t accuracy_kmin(uint32_t w0, int minexp) {
  const int emax = (int)((w0 >> 1) & 0xffu) - kEBias;
  return 32u - block_precision(emax, 32, minexp, 1);
}
// Lowest plane kept for the block f, or 32 when the block is dropped.
GCOW_HD uint32_t accuracy_kmin_of(const float* f, int minexp) {
  const int emax = block_emax<4>(f);
  return emax == -kEBias ? 32u : 32u - block_precision(emax, 32, minexp, 1);
}

// Host-side construction of the pair table.
inline void build_pair_table(uint32_t* epair) {
  for (uint32_t i = 0; i < (uint32_t)kEncPairTabSize; i++) epair[i] = make_enc_pair_entry(i >> 8, i & 255u);
}
inline void build_dec_loop_table(uint32_t* dloop) {
  for (uint32_t i = 0; i < (uint32_t)kDecLoopTabSize; i++) dloop[i] = make_dec_loop_entry(i >> 10, (i >> 7) & 7u, i & 127u);
}

}  // namespace gcow
