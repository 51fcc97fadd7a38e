// CPU oracle of the ZFP float32 block codec (1-D blocks of 4, 2-D blocks of 4x4).
//
// A deliberately plain restatement: a bit-at-a-time stream, libm frexp/ldexp
// for the float stages and the serial group-test coder. It shares no code with
// the table-driven / register-packed formulation in zfp_block.cuh, so agreement
// between the two (and with the reference build) is meaningful. The library
// also exports the header's fast path compiled for the host, the individual
// stages for golden-vector tests, and the host model of the compressed
// all-reduce used to check the fused GPU kernels.
//
// Behaviour parity: sw/src/stream.c (bit order, 64-bit words, flush),
// sw/src/encode.c and sw/src/decode.c (stages; the decoder is used with the
// block size where the reference passes the dimension, sw/src/decode.c:193-202),
// sw/src/zfp.c:31-56,79-103 (row-major walk over blocks, partial edge blocks).
#include <stdint.h>
#include <stddef.h>
#include <string.h>
#include <math.h>
#include <algorithm>
#include <thread>
#include <vector>

#include "zfp_block.cuh"

namespace {

using gcow::ZfpParams;

// ------------------------------------------------------------ bit stream
class BitStream {
 public:
  BitStream(uint64_t* words, uint64_t bit_offset = 0)
      : w_(words), idx_(bit_offset >> 6), buf_(0), nbuf_(0) {
    uint32_t o = (uint32_t)(bit_offset & 63);
    if (o) {  // resume inside a word (used when threads start mid-stream)
      buf_ = w_[idx_] & ((1ull << o) - 1);
      nbuf_ = o;
    }
  }
  void write_bit(uint32_t b) {
    buf_ |= (uint64_t)(b & 1u) << nbuf_;
    if (++nbuf_ == 64) { w_[idx_++] = buf_; buf_ = 0; nbuf_ = 0; }
  }
  void write_bits(uint64_t v, uint32_t n) {
    for (uint32_t i = 0; i < n; i++) write_bit((uint32_t)((v >> i) & 1u));
  }
  void pad(uint64_t n) { for (uint64_t i = 0; i < n; i++) write_bit(0); }
  // zero-fill to the next word boundary
  void flush() { while (nbuf_) write_bit(0); }
  // write the partial word without disturbing bits above the cursor
  void flush_partial() {
    if (nbuf_) {
      uint64_t keep = w_[idx_] & ~((1ull << nbuf_) - 1);
      w_[idx_] = keep | buf_;
    }
  }
  uint64_t wpos() const { return idx_ * 64 + nbuf_; }

 private:
  uint64_t* w_;
  uint64_t idx_;
  uint64_t buf_;
  uint32_t nbuf_;
};

class BitReader {
 public:
  BitReader(const uint64_t* words, uint64_t bit_offset = 0) : w_(words), pos_(bit_offset) {}
  uint32_t read_bit() {
    uint32_t b = (uint32_t)((w_[pos_ >> 6] >> (pos_ & 63)) & 1u);
    pos_++;
    return b;
  }
  uint64_t read_bits(uint32_t n) {
    uint64_t v = 0;
    for (uint32_t i = 0; i < n; i++) v |= (uint64_t)read_bit() << i;
    return v;
  }
  void skip(uint64_t n) { pos_ += n; }
  uint64_t rpos() const { return pos_; }

 private:
  const uint64_t* w_;
  uint64_t pos_;
};

// ------------------------------------------------------------ stages (libm)
int o_scalar_exponent(float x) {
  int e = -127;
  if (x > 0) {
    if (isinf(x)) return 128;
    (void)frexpf(x, &e);
    e = std::max(e, -126);
  }
  return e;
}
int o_block_exponent(const float* f, int n) {
  float m = 0;
  for (int i = 0; i < n; i++) { float a = fabsf(f[i]); if (m < a) m = a; }
  return o_scalar_exponent(m);
}
int32_t o_trunc(float v) {
  if (!(fabsf(v) < 2147483648.0f)) return INT32_MIN;
  return (int32_t)v;
}
void o_fwd_cast(int32_t* q, const float* f, int n, int emax) {
  float scale = ldexpf(1.0f, 30 - emax);
  for (int i = 0; i < n; i++) q[i] = o_trunc(scale * f[i]);
}
void o_inv_cast(float* f, const int32_t* q, int n, int emax, int shift) {
  float scale = ldexpf(1.0f, emax - 30 - shift);
  for (int i = 0; i < n; i++) f[i] = scale * (float)q[i];
}
inline int32_t sar(int32_t v) { return v >> 1; }
inline int32_t wadd(int32_t a, int32_t b) { return (int32_t)((uint32_t)a + (uint32_t)b); }
inline int32_t wsub(int32_t a, int32_t b) { return (int32_t)((uint32_t)a - (uint32_t)b); }
inline int32_t wshl(int32_t a) { return (int32_t)((uint32_t)a << 1); }
void o_fwd_lift(int32_t* p, int s) {
  int32_t x = p[0], y = p[s], z = p[2 * s], w = p[3 * s];
  x = wadd(x, w); x = sar(x); w = wsub(w, x);
  z = wadd(z, y); z = sar(z); y = wsub(y, z);
  x = wadd(x, z); x = sar(x); z = wsub(z, x);
  w = wadd(w, y); w = sar(w); y = wsub(y, w);
  w = wadd(w, sar(y)); y = wsub(y, sar(w));
  p[0] = x; p[s] = y; p[2 * s] = z; p[3 * s] = w;
}
void o_inv_lift(int32_t* p, int s) {
  int32_t x = p[0], y = p[s], z = p[2 * s], w = p[3 * s];
  y = wadd(y, sar(w)); w = wsub(w, sar(y));
  y = wadd(y, w); w = wshl(w); w = wsub(w, y);
  z = wadd(z, x); x = wshl(x); x = wsub(x, z);
  y = wadd(y, z); z = wshl(z); z = wsub(z, y);
  w = wadd(w, x); x = wshl(x); x = wsub(x, w);
  p[0] = x; p[s] = y; p[2 * s] = z; p[3 * s] = w;
}
void o_fwd_xform(int32_t* q, int dim) {
  if (dim == 1) { o_fwd_lift(q, 1); return; }
  for (int y = 0; y < 4; y++) o_fwd_lift(q + 4 * y, 1);
  for (int x = 0; x < 4; x++) o_fwd_lift(q + x, 4);
}
void o_inv_xform(int32_t* q, int dim) {
  if (dim == 1) { o_inv_lift(q, 1); return; }
  for (int x = 0; x < 4; x++) o_inv_lift(q + x, 4);
  for (int y = 0; y < 4; y++) o_inv_lift(q + 4 * y, 1);
}
const int kPerm1[4] = {0, 1, 2, 3};
const int kPerm2[16] = {0, 1, 4, 5, 2, 8, 6, 9, 3, 12, 10, 7, 13, 11, 14, 15};
const int* o_perm(int dim) { return dim == 1 ? kPerm1 : kPerm2; }
void o_fwd_reorder(uint32_t* u, const int32_t* q, int dim) {
  int n = 1 << (2 * dim);
  const int* perm = o_perm(dim);
  for (int i = 0; i < n; i++) u[i] = ((uint32_t)q[perm[i]] + 0xaaaaaaaau) ^ 0xaaaaaaaau;
}
void o_inv_reorder(int32_t* q, const uint32_t* u, int dim) {
  int n = 1 << (2 * dim);
  const int* perm = o_perm(dim);
  for (int i = 0; i < n; i++) q[perm[i]] = (int32_t)((u[i] ^ 0xaaaaaaaau) - 0xaaaaaaaau);
}

uint32_t o_encode_planes(BitStream& s, const uint32_t* u, uint32_t maxbits, uint32_t maxprec,
                         uint32_t size) {
  uint32_t kmin = 32 > maxprec ? 32 - maxprec : 0;
  uint32_t bits = maxbits, n = 0;
  for (uint32_t k = 32; bits && k-- > kmin;) {
    uint64_t x = 0;
    for (uint32_t i = 0; i < size; i++) x += (uint64_t)((u[i] >> k) & 1u) << i;
    uint32_t m = std::min(n, bits);
    bits -= m;
    s.write_bits(x, m);
    x >>= m;
    for (; bits && n < size; x >>= 1, n++) {
      bits--;
      uint32_t t = x != 0;
      s.write_bit(t);
      if (!t) break;
      for (; bits && n < size - 1; x >>= 1, n++) {
        bits--;
        uint32_t b = (uint32_t)(x & 1u);
        s.write_bit(b);
        if (b) break;
      }
    }
  }
  return maxbits - bits;
}

uint32_t o_decode_planes(BitReader& s, uint32_t* u, uint32_t maxbits, uint32_t maxprec,
                         uint32_t size) {
  uint32_t kmin = 32 > maxprec ? 32 - maxprec : 0;
  uint32_t bits = maxbits, n = 0;
  for (uint32_t i = 0; i < size; i++) u[i] = 0;
  for (uint32_t k = 32; bits && k-- > kmin;) {
    uint32_t m = std::min(n, bits);
    bits -= m;
    uint64_t x = s.read_bits(m);
    for (; bits && n < size; n++) {
      bits--;
      if (s.read_bit()) {
        for (; bits && n < size - 1; n++) {
          bits--;
          if (s.read_bit()) break;
        }
        x += (uint64_t)1 << n;
      } else {
        break;
      }
    }
    for (uint32_t i = 0; x; i++, x >>= 1) u[i] += (uint32_t)(x & 1u) << k;
  }
  return maxbits - bits;
}

uint32_t o_encode_block(BitStream& s, const float* f, const ZfpParams& p, int dim) {
  int size = 1 << (2 * dim);
  int emax = o_block_exponent(f, size);
  uint32_t prec = gcow::block_precision(emax, p.maxprec, p.minexp, dim);
  uint32_t biased = prec ? (uint32_t)(emax + 127) : 0;
  uint32_t bits = 1;
  if (biased) {
    int32_t q[16];
    uint32_t u[16];
    bits += 8;
    s.write_bits(2 * biased + 1, bits);
    o_fwd_cast(q, f, size, emax);
    o_fwd_xform(q, dim);
    o_fwd_reorder(u, q, dim);
    bits += o_encode_planes(s, u, p.maxbits - bits, prec, (uint32_t)size);
  } else {
    s.write_bit(0);
  }
  if (bits < p.minbits) { s.pad(p.minbits - bits); bits = p.minbits; }
  return bits;
}

uint32_t o_decode_block(BitReader& s, float* f, const ZfpParams& p, int dim, int shift) {
  int size = 1 << (2 * dim);
  uint32_t bits = 1;
  if (s.read_bit()) {
    int32_t q[16];
    uint32_t u[16];
    bits += 8;
    int emax = (int)s.read_bits(8) - 127;
    uint32_t prec = gcow::block_precision(emax, p.maxprec, p.minexp, dim);
    bits += o_decode_planes(s, u, p.maxbits - bits, prec, (uint32_t)size);
    o_inv_reorder(q, u, dim);
    o_inv_xform(q, dim);
    o_inv_cast(f, q, size, emax, shift);
  } else {
    for (int i = 0; i < size; i++) f[i] = 0;
  }
  if (bits < p.minbits) { s.skip(p.minbits - bits); bits = p.minbits; }
  return bits;
}

void o_pad(float* b, uint32_t n, int s) {
  switch (n) {
    case 0: b[0] = 0;            /* fallthrough */
    case 1: b[s] = b[0];         /* fallthrough */
    case 2: b[2 * s] = b[s];     /* fallthrough */
    case 3: b[3 * s] = b[0];     /* fallthrough */
    default: break;
  }
}

// gather block `b` of an (nx, ny) array; ny == 0 means 1-D
void o_gather(float* blk, const float* data, uint64_t nx, uint64_t ny, uint64_t b) {
  if (ny == 0) {
    uint64_t x0 = 4 * b;
    uint32_t n = (uint32_t)std::min<uint64_t>(4, nx - x0);
    for (uint32_t i = 0; i < n; i++) blk[i] = data[x0 + i];
    if (n < 4) o_pad(blk, n, 1);
    return;
  }
  uint64_t bx = (nx + 3) / 4;
  uint64_t x0 = 4 * (b % bx), y0 = 4 * (b / bx);
  uint32_t cx = (uint32_t)std::min<uint64_t>(4, nx - x0), cy = (uint32_t)std::min<uint64_t>(4, ny - y0);
  for (uint32_t y = 0; y < cy; y++) {
    for (uint32_t x = 0; x < cx; x++) blk[4 * y + x] = data[(y0 + y) * nx + x0 + x];
    if (cx < 4) o_pad(blk + 4 * y, cx, 1);
  }
  if (cy < 4) for (uint32_t x = 0; x < 4; x++) o_pad(blk + x, cy, 4);
}

void o_scatter(const float* blk, float* data, uint64_t nx, uint64_t ny, uint64_t b) {
  if (ny == 0) {
    uint64_t x0 = 4 * b;
    uint32_t n = (uint32_t)std::min<uint64_t>(4, nx - x0);
    for (uint32_t i = 0; i < n; i++) data[x0 + i] = blk[i];
    return;
  }
  uint64_t bx = (nx + 3) / 4;
  uint64_t x0 = 4 * (b % bx), y0 = 4 * (b / bx);
  uint32_t cx = (uint32_t)std::min<uint64_t>(4, nx - x0), cy = (uint32_t)std::min<uint64_t>(4, ny - y0);
  for (uint32_t y = 0; y < cy; y++)
    for (uint32_t x = 0; x < cx; x++) data[(y0 + y) * nx + x0 + x] = blk[4 * y + x];
}

uint64_t total_blocks(uint64_t nx, uint64_t ny) {
  return ny ? gcow::num_blocks_2d(nx, ny) : gcow::num_blocks_1d(nx);
}

ZfpParams load_params(const int32_t* p) {
  ZfpParams z;
  z.minbits = (uint32_t)p[0]; z.maxbits = (uint32_t)p[1]; z.maxprec = (uint32_t)p[2]; z.minexp = p[3];
  return z;
}

template <class F>
void parallel_blocks(uint64_t blocks, uint64_t grain, int threads, F fn) {
  if (threads <= 1 || blocks <= grain) { fn(0, blocks); return; }
  uint64_t per = ((blocks + threads - 1) / threads + grain - 1) / grain * grain;
  std::vector<std::thread> pool;
  for (uint64_t b0 = 0; b0 < blocks; b0 += per) {
    uint64_t b1 = std::min(blocks, b0 + per);
    pool.emplace_back([=] { fn(b0, b1); });
  }
  for (auto& t : pool) t.join();
}

}  // namespace

extern "C" {

// ------------------------------------------------------------ parameters
void gcow_params_rate(double rate, int dim, int32_t* out) {
  ZfpParams p = gcow::params_rate(rate, dim);
  out[0] = (int32_t)p.minbits; out[1] = (int32_t)p.maxbits; out[2] = (int32_t)p.maxprec; out[3] = p.minexp;
}
void gcow_params_accuracy(double tol, int32_t* out) {
  ZfpParams p = gcow::params_accuracy(tol);
  out[0] = (int32_t)p.minbits; out[1] = (int32_t)p.maxbits; out[2] = (int32_t)p.maxprec; out[3] = p.minexp;
}
void gcow_params_precision(uint32_t prec, int32_t* out) {
  ZfpParams p = gcow::params_precision(prec);
  out[0] = (int32_t)p.minbits; out[1] = (int32_t)p.maxbits; out[2] = (int32_t)p.maxprec; out[3] = p.minexp;
}
uint64_t gcow_max_output_bytes(const int32_t* params, uint64_t nx, uint64_t ny) {
  return gcow::max_output_bytes(load_params(params), total_blocks(nx, ny), ny ? 2 : 1);
}
uint32_t gcow_block_precision(int emax, uint32_t maxprec, int minexp, int dim) {
  return gcow::block_precision(emax, maxprec, minexp, dim);
}

// ------------------------------------------------------------ oracle codec
// Compress an (nx, ny) row-major float array (ny == 0: 1-D of nx values).
// `out` must hold gcow_max_output_bytes(). If `block_bits` is non-null it
// receives the start bit of every block plus the end (blocks + 1 entries).
// Returns the stream size in bytes (padded to a 64-bit word).
uint64_t gcow_oracle_compress(const float* data, uint64_t nx, uint64_t ny, const int32_t* params,
                              uint64_t* out, uint64_t* block_bits, int threads) {
  ZfpParams p = load_params(params);
  int dim = ny ? 2 : 1;
  uint64_t blocks = total_blocks(nx, ny);
  if (gcow::is_fixed_rate(p)) {
    // block b starts at bit b*maxbits; ranges of 64 blocks start on a word
    parallel_blocks(blocks, 64, threads, [&](uint64_t b0, uint64_t b1) {
      BitStream s(out + (b0 * p.maxbits) / 64);
      float blk[16];
      for (uint64_t b = b0; b < b1; b++) {
        if (block_bits) block_bits[b] = b * p.maxbits;
        o_gather(blk, data, nx, ny, b);
        o_encode_block(s, blk, p, dim);
      }
      s.flush();
    });
    if (block_bits) block_bits[blocks] = blocks * p.maxbits;
    return gcow::fixed_rate_bytes(p, blocks);
  }
  BitStream s(out);
  float blk[16];
  for (uint64_t b = 0; b < blocks; b++) {
    if (block_bits) block_bits[b] = s.wpos();
    o_gather(blk, data, nx, ny, b);
    o_encode_block(s, blk, p, dim);
  }
  if (block_bits) block_bits[blocks] = s.wpos();
  s.flush();
  return s.wpos() / 8;
}

// Decompress into an (nx, ny) array; every value is divided by 2^shift.
// Returns the number of stream bits consumed.
uint64_t gcow_oracle_decompress(const uint64_t* in, float* data, uint64_t nx, uint64_t ny,
                                const int32_t* params, int shift, int threads) {
  ZfpParams p = load_params(params);
  int dim = ny ? 2 : 1;
  uint64_t blocks = total_blocks(nx, ny);
  if (gcow::is_fixed_rate(p)) {
    parallel_blocks(blocks, 64, threads, [&](uint64_t b0, uint64_t b1) {
      BitReader s(in, b0 * p.maxbits);
      float blk[16];
      for (uint64_t b = b0; b < b1; b++) {
        o_decode_block(s, blk, p, dim, shift);
        o_scatter(blk, data, nx, ny, b);
      }
    });
    return blocks * p.maxbits;
  }
  BitReader s(in);
  float blk[16];
  for (uint64_t b = 0; b < blocks; b++) {
    o_decode_block(s, blk, p, dim, shift);
    o_scatter(blk, data, nx, ny, b);
  }
  return s.rpos();
}

// ------------------------------------- header fast path compiled for the host
// Generic path (WordSink / WordSrc + run-skipping plane coder), any mode.
uint64_t gcow_header_compress(const float* data, uint64_t nx, uint64_t ny, const int32_t* params,
                              uint64_t* out) {
  ZfpParams p = load_params(params);
  uint64_t blocks = total_blocks(nx, ny);
  gcow::WordSink sink(out);
  float blk[16];
  for (uint64_t b = 0; b < blocks; b++) {
    o_gather(blk, data, nx, ny, b);
    if (ny) gcow::encode_block<2>(blk, p, sink); else gcow::encode_block<1>(blk, p, sink);
  }
  uint64_t bits = sink.bit_count();
  sink.finish();
  return ((bits + 63) / 64) * 8;
}
uint64_t gcow_header_decompress(const uint64_t* in, float* data, uint64_t nx, uint64_t ny,
                                const int32_t* params, int shift) {
  ZfpParams p = load_params(params);
  uint64_t blocks = total_blocks(nx, ny);
  gcow::WordSrc src(in, 0);
  float blk[16];
  for (uint64_t b = 0; b < blocks; b++) {
    if (ny) gcow::decode_block<2>(blk, p, src, shift); else gcow::decode_block<1>(blk, p, src, shift);
    o_scatter(blk, data, nx, ny, b);
  }
  return src.pos;
}

// Table-driven 1-D fixed-rate paths (rate-specialised, general, and the warp-uniform
// formulation the kernels run); all are run and must agree (-2 otherwise). maxbits
// must be 16, 32, 64 or 128.
namespace {
struct HostLeanTables {
  std::vector<uint16_t> etab, btab;
  std::vector<uint32_t> epair, dloop;
  gcow::LeanTables t;
  HostLeanTables() : etab(gcow::kEncTabSize), btab(gcow::kDecBudgetTabSize), epair(gcow::kEncPairTabSize),
                     dloop(gcow::kDecLoopTabSize) {
    gcow::build_codec_tables(etab.data(), btab.data());
    gcow::build_pair_table(epair.data());
    gcow::build_dec_loop_table(dloop.data());
    t.etab = etab.data(); t.dtab = btab.data(); t.epair = epair.data(); t.dloop = dloop.data();
  }
};
const gcow::LeanTables& host_lean_tables() {
  static HostLeanTables h;
  return h.t;
}
}  // namespace

// Fixed accuracy with a bit cap through the lean coders (as the sparse all-reduce kernel uses them) against the
// definition path: out = D(E(x)) from the lean pair, and the return value counts the blocks whose result differs from
// decode_block(encode_block(x)) at {minbits 1, maxbits bits, maxprec 64, minexp}. 0 means they agree everywhere.
int64_t gcow_lean_accuracy_check(const float* data, uint64_t n, int bits, int minexp, float* out) {
  const gcow::LeanTables& lt = host_lean_tables();
  ZfpParams p;
  p.minbits = 1; p.maxbits = (uint32_t)bits; p.maxprec = 64; p.minexp = minexp;
  uint64_t blocks = gcow::num_blocks_1d(n);
  int64_t bad = 0;
  std::vector<uint64_t> buf(8);
  for (uint64_t b = 0; b < blocks; b++) {
    float blk[4], want[4], got[4] = {0, 0, 0, 0};
    o_gather(blk, data, n, 0, b);
    std::fill(buf.begin(), buf.end(), 0);
    BitStream s(buf.data());
    o_encode_block(s, blk, p, 1);
    s.flush();
    BitReader rd(buf.data());
    o_decode_block(rd, want, p, 1, 0);
    const uint32_t kmin = gcow::accuracy_kmin_of(blk, minexp);
    if (kmin < 32) {
      switch (bits) {
        case 16: { uint32_t w[1]; gcow::encode_block_1d_lean<16>(blk, lt, w, kmin); gcow::decode_block_1d_lean<16>(got, lt, w, 0, gcow::accuracy_kmin(w[0], minexp)); break; }
        case 32: { uint32_t w[1]; gcow::encode_block_1d_lean<32>(blk, lt, w, kmin); gcow::decode_block_1d_lean<32>(got, lt, w, 0, gcow::accuracy_kmin(w[0], minexp)); break; }
        case 64: { uint32_t w[2]; gcow::encode_block_1d_lean<64>(blk, lt, w, kmin); gcow::decode_block_1d_lean<64>(got, lt, w, 0, gcow::accuracy_kmin(w[0], minexp)); break; }
        case 128: { uint32_t w[4]; gcow::encode_block_1d_lean<128>(blk, lt, w, kmin); gcow::decode_block_1d_lean<128>(got, lt, w, 0, gcow::accuracy_kmin(w[0], minexp)); break; }
        default: return -1;
      }
    }
    bad += memcmp(want, got, sizeof(want)) != 0;
    o_scatter(got, out, n, 0, b);
  }
  return bad;
}

int gcow_fast1d_compress(const float* data, uint64_t n, const int32_t* params, void* out) {
  ZfpParams p = load_params(params);
  uint16_t etab[gcow::kEncTabSize];
  for (uint32_t i = 0; i < (uint32_t)gcow::kEncTabSize; i++) etab[i] = gcow::make_enc_entry(i / 16, i % 16);
  const gcow::LeanTables& lt = host_lean_tables();
  uint64_t blocks = gcow::num_blocks_1d(n);
  float blk[4];
  for (uint64_t b = 0; b < blocks; b++) {
    o_gather(blk, data, n, 0, b);
    switch (p.maxbits) {
      case 16: { uint32_t w[1], v[1], l[1]; gcow::encode_block_1d_rate<16>(blk, etab, w); gcow::encode_block_1d_fast<1>(blk, p, etab, v); gcow::encode_block_1d_lean<16>(blk, lt, l); if (memcmp(w, v, 4) || memcmp(w, l, 4)) return -2; ((uint16_t*)out)[b] = (uint16_t)w[0]; break; }
      case 32: { uint32_t w[1], v[1], l[1]; gcow::encode_block_1d_rate<32>(blk, etab, w); gcow::encode_block_1d_fast<1>(blk, p, etab, v); gcow::encode_block_1d_lean<32>(blk, lt, l); if (memcmp(w, v, 4) || memcmp(w, l, 4)) return -2; ((uint32_t*)out)[b] = w[0]; break; }
      case 64: { uint32_t w[2], v[2], l[2]; gcow::encode_block_1d_rate<64>(blk, etab, w); gcow::encode_block_1d_fast<2>(blk, p, etab, v); gcow::encode_block_1d_lean<64>(blk, lt, l); if (memcmp(w, v, 8) || memcmp(w, l, 8)) return -2; memcpy((uint32_t*)out + 2 * b, w, 8); break; }
      case 128: { uint32_t w[4], v[4], l[4]; gcow::encode_block_1d_rate<128>(blk, etab, w); gcow::encode_block_1d_fast<4>(blk, p, etab, v); gcow::encode_block_1d_lean<128>(blk, lt, l); if (memcmp(w, v, 16) || memcmp(w, l, 16)) return -2; memcpy((uint32_t*)out + 4 * b, w, 16); break; }
      default: return -1;
    }
  }
  return 0;
}
int gcow_fast1d_decompress(const void* in, float* data, uint64_t n, const int32_t* params, int shift) {
  ZfpParams p = load_params(params);
  std::vector<uint16_t> dtab(gcow::kDecTabSize), btab(gcow::kDecBudgetTabSize), etab(gcow::kEncTabSize);
  for (uint32_t i = 0; i < (uint32_t)gcow::kDecTabSize; i++) dtab[i] = gcow::make_dec_entry(i / 128, i % 128);
  gcow::build_codec_tables(etab.data(), btab.data());
  uint64_t blocks = gcow::num_blocks_1d(n);
  float blk[4], alt[4], lean[4];
  const gcow::LeanTables& lt = host_lean_tables();
  for (uint64_t b = 0; b < blocks; b++) {
    switch (p.maxbits) {
      case 16: { uint32_t w[1] = {((const uint16_t*)in)[b]}; gcow::decode_block_1d_rate<16>(blk, btab.data(), w, shift); gcow::decode_block_1d_fast<1>(alt, p, dtab.data(), w, shift); gcow::decode_block_1d_lean<16>(lean, lt, w, shift); break; }
      case 32: { uint32_t w[1] = {((const uint32_t*)in)[b]}; gcow::decode_block_1d_rate<32>(blk, btab.data(), w, shift); gcow::decode_block_1d_fast<1>(alt, p, dtab.data(), w, shift); gcow::decode_block_1d_lean<32>(lean, lt, w, shift); break; }
      case 64: { uint32_t w[2]; memcpy(w, (const uint32_t*)in + 2 * b, 8); gcow::decode_block_1d_rate<64>(blk, btab.data(), w, shift); gcow::decode_block_1d_fast<2>(alt, p, dtab.data(), w, shift); gcow::decode_block_1d_lean<64>(lean, lt, w, shift); break; }
      case 128: { uint32_t w[4]; memcpy(w, (const uint32_t*)in + 4 * b, 16); gcow::decode_block_1d_rate<128>(blk, btab.data(), w, shift); gcow::decode_block_1d_fast<4>(alt, p, dtab.data(), w, shift); gcow::decode_block_1d_lean<128>(lean, lt, w, shift); break; }
      default: return -1;
    }
    if (memcmp(blk, alt, 16) || memcmp(blk, lean, 16)) return -2;   // the table-driven formulations must agree
    o_scatter(blk, data, n, 0, b);
  }
  return 0;
}

// ------------------------------------------------------------ single stages
// which: 0 = oracle (libm), 1 = header (bit arithmetic)
int gcow_stage_emax(const float* f, int n, int which) {
  if (which == 0) return o_block_exponent(f, n);
  return n == 4 ? gcow::block_emax<4>(f) : gcow::block_emax<16>(f);
}
void gcow_stage_cast(const float* f, int32_t* q, int n, int emax, int which) {
  if (which == 0) { o_fwd_cast(q, f, n, emax); return; }
  if (n == 4) gcow::fwd_cast<4>(q, f, emax); else gcow::fwd_cast<16>(q, f, emax);
}
void gcow_stage_inv_cast(const int32_t* q, float* f, int n, int emax, int shift, int which) {
  if (which == 0) { o_inv_cast(f, q, n, emax, shift); return; }
  if (n == 4) gcow::inv_cast<4>(f, q, emax, shift); else gcow::inv_cast<16>(f, q, emax, shift);
}
void gcow_stage_xform(int32_t* q, int dim, int inverse, int which) {
  if (which == 0) { if (inverse) o_inv_xform(q, dim); else o_fwd_xform(q, dim); return; }
  if (dim == 1) { if (inverse) gcow::Xform<1>::inv(q); else gcow::Xform<1>::fwd(q); }
  else { if (inverse) gcow::Xform<2>::inv(q); else gcow::Xform<2>::fwd(q); }
}
void gcow_stage_reorder(const int32_t* q, uint32_t* u, int dim, int which) {
  if (which == 0) { o_fwd_reorder(u, q, dim); return; }
  if (dim == 1) gcow::fwd_reorder<1>(u, q); else gcow::fwd_reorder<2>(u, q);
}
void gcow_stage_inv_reorder(const uint32_t* u, int32_t* q, int dim, int which) {
  if (which == 0) { o_inv_reorder(q, u, dim); return; }
  if (dim == 1) gcow::inv_reorder<1>(q, u); else gcow::inv_reorder<2>(q, u);
}
// Encode `reps` copies of one coefficient block after an optional 9-bit header
// value (header < 0: none). Returns total bits; `out` is flushed to a word.
uint64_t gcow_stage_encode_planes(const uint32_t* u, int size, uint32_t budget, uint32_t prec,
                                  int header, int reps, uint64_t* out, int which) {
  if (which == 0) {
    BitStream s(out);
    for (int r = 0; r < reps; r++) {
      if (header >= 0) s.write_bits((uint64_t)header, 9);
      o_encode_planes(s, u, budget, prec, (uint32_t)size);
    }
    uint64_t bits = s.wpos();
    s.flush();
    return bits;
  }
  gcow::WordSink sink(out);
  for (int r = 0; r < reps; r++) {
    if (header >= 0) sink.put((uint64_t)header, 9);
    if (size == 4) gcow::encode_planes<4>(u, budget, prec, sink);
    else gcow::encode_planes<16>(u, budget, prec, sink);
  }
  uint64_t bits = sink.bit_count();
  sink.finish();
  return bits;
}
uint32_t gcow_stage_decode_planes(const uint64_t* in, uint64_t bit_offset, uint32_t* u, int size,
                                  uint32_t budget, uint32_t prec, int which) {
  if (which == 0) {
    BitReader s(in, bit_offset);
    return o_decode_planes(s, u, budget, prec, (uint32_t)size);
  }
  gcow::WordSrc src(in, bit_offset);
  if (size == 4) return gcow::decode_planes<4>(u, budget, prec, src);
  return gcow::decode_planes<16>(u, budget, prec, src);
}
// Raw stream writes: values[i] with nbits[i] each; returns words written.
uint64_t gcow_stage_stream_write(const uint64_t* values, const uint32_t* nbits, int count,
                                 uint64_t* out, int which) {
  if (which == 0) {
    BitStream s(out);
    for (int i = 0; i < count; i++) s.write_bits(values[i], nbits[i]);
    s.flush();
    return s.wpos() / 64;
  }
  gcow::WordSink sink(out);
  for (int i = 0; i < count; i++)
    sink.put(nbits[i] >= 64 ? values[i] : (values[i] & ((1ull << nbits[i]) - 1)), nbits[i]);
  sink.finish();
  return sink.nw;
}
void gcow_stage_gather(const float* data, uint64_t nx, uint64_t ny, uint64_t b, float* blk) {
  o_gather(blk, data, nx, ny, b);
}

// ---------------------------------------------- host model of the all-reduce
// xs: P contiguous arrays of n floats (rank-major). variant 0 (two-shot):
// out = D(E( sum_r D(E(x_r)) )) / 2^shift ; variant 1 (one-shot):
// out = ( sum_r D(E(x_r)) ) / 2^shift. Sums run in ascending rank order in
// fp32. 1-D blocks of 4, fixed-rate parameters.
void gcow_oracle_allreduce(const float* xs, int P, uint64_t n, const int32_t* params, int variant,
                           int shift, float* out, int threads) {
  ZfpParams p = load_params(params);
  uint64_t blocks = gcow::num_blocks_1d(n);
  float inv = ldexpf(1.0f, -shift);
  parallel_blocks(blocks, 64, threads, [&](uint64_t b0, uint64_t b1) {
    std::vector<uint64_t> buf((p.maxbits + 63) / 64 + 2);
    for (uint64_t b = b0; b < b1; b++) {
      float acc[4] = {0, 0, 0, 0}, blk[4], dec[4];
      for (int r = 0; r < P; r++) {
        o_gather(blk, xs + (uint64_t)r * n, n, 0, b);
        std::fill(buf.begin(), buf.end(), 0);
        BitStream s(buf.data());
        o_encode_block(s, blk, p, 1);
        s.flush();
        BitReader rd(buf.data());
        o_decode_block(rd, dec, p, 1, 0);
        for (int i = 0; i < 4; i++) acc[i] = r == 0 ? dec[i] : acc[i] + dec[i];
      }
      if (variant == 0) {
        std::fill(buf.begin(), buf.end(), 0);
        BitStream s(buf.data());
        o_encode_block(s, acc, p, 1);
        s.flush();
        BitReader rd(buf.data());
        o_decode_block(rd, dec, p, 1, shift);
      } else {
        for (int i = 0; i < 4; i++) dec[i] = acc[i] * inv;
      }
      o_scatter(dec, out, n, 0, b);
    }
  });
}

}  // extern "C"
