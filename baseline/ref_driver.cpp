// C-ABI shim around the UNMODIFIED reference CPU codec (sw/src/*.c compiled as
// C++ exactly as sw/Makefile:4-5 does). Nothing here re-implements a stage:
// every function below only calls the reference's own exported functions.
//
//  * 2-D: zfp_compress() itself (sw/src/zfp.c:10-28).
//  * 1-D: the reference has no 1-D driver, so blocks of 4 are pushed through
//    the same sequence encode_fblock/encode_iblock perform (sw/src/encode.c:
//    412-495) with block size 4 and the identity coefficient order.
//  * decode: decode_iblock passes the dimension where the block size is needed
//    (sw/src/decode.c:193-202), so the decoder is composed from the reference's
//    stage functions with the block size passed explicitly.
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include "types.h"
#include "common.h"
#include "stream.h"
#include "encode.h"
#include "decode.h"
#include "zfp.h"

// Non-static reference functions that the reference headers do not declare.
float quantize_scaler(float x, int e);
void fwd_lift_vector(int32* p, ptrdiff_t s);
uint32 twoscomplement_to_negabinary(int32 x);
void pad_partial_block(float* block, size_t n, ptrdiff_t s);
int exceeded_maxbits(uint maxbits, uint maxprec, uint size);
void bwd_cast_block(const int32* iblock, float* fblock, uint n, int emax);
int32 negabinary_to_twoscomplement(uint32 x);
void bwd_lift_vector(int32* p, ptrdiff_t s);
void bwd_decorrelate_2d_block(int32* iblock);
uint decode_partial_bitplanes(stream* const s, uint32* const ublock, uint maxbits, uint maxprec,
                              uint block_size);
uint decode_full_bitplanes(stream* s, uint32* const ublock, uint maxprec, uint block_size);
void bwd_reorder_uint2int(const uint32* ublock, int32* iblock, const uchar* perm, uint n);

static const uchar kPerm1[5] = {0, 1, 2, 3, 0};  // 5th entry: the reference loop runs n+1 times
static uchar kPerm2[17];

static void set_params(zfp_output* o, const int32_t* p) {
  o->minbits = (uint)p[0]; o->maxbits = (uint)p[1]; o->maxprec = (uint)p[2]; o->minexp = p[3];
}

extern "C" {

uint64_t ref_compress_2d(const float* data, uint64_t nx, uint64_t ny, const int32_t* params,
                         void* out, uint64_t cap) {
  zfp_input in;
  memset(&in, 0, sizeof in);
  in.dtype = dtype_float; in.data = (void*)data; in.nx = nx; in.ny = ny;
  zfp_output o;
  set_params(&o, params);
  memset(out, 0, cap);
  o.data = stream_init(out, cap);
  stream_rewind(o.data);
  uint64_t bytes = zfp_compress(&o, &in);
  free(o.data);
  return bytes;
}

uint64_t ref_compress_1d(const float* data, uint64_t n, const int32_t* params, void* out,
                         uint64_t cap) {
  zfp_output o;
  set_params(&o, params);
  memset(out, 0, cap);
  stream* s = stream_init(out, cap);
  stream_rewind(s);
  for (uint64_t x = 0; x < n; x += 4) {
    float f[4];
    uint32_t c = n - x < 4 ? (uint32_t)(n - x) : 4;
    for (uint32_t i = 0; i < c; i++) f[i] = data[x + i];
    if (c < 4) pad_partial_block(f, c, 1);
    uint bits = 1;
    int emax = get_block_exponent(f, 4);
    uint maxprec = get_precision(emax, o.maxprec, o.minexp, 1);
    uint biased = maxprec ? (uint)(emax + EBIAS) : 0;
    if (biased) {
      int32 q[4];
      uint32 u[5];
      bits += EBITS;
      stream_write_bits(s, 2 * biased + 1, bits);
      fwd_cast_block(q, f, 4, emax);
      fwd_lift_vector(q, 1);
      fwd_reorder_int2uint(u, q, kPerm1, 4);
      uint enc;
      uint maxbits = o.maxbits - bits;
      uint minbits = o.minbits - MIN(bits, o.minbits);
      if (exceeded_maxbits(maxbits, maxprec, 4)) enc = encode_partial_bitplanes(s, u, maxbits, maxprec, 4);
      else enc = encode_all_bitplanes(s, u, maxprec, 4);
      if (enc < minbits) { stream_pad(s, minbits - enc); enc = minbits; }
      bits += enc;
    } else {
      stream_write_bit(s, 0);
      if (o.minbits > bits) { stream_pad(s, o.minbits - bits); bits = o.minbits; }
    }
  }
  stream_flush(s);
  uint64_t bytes = stream_size_bytes(s);
  free(s);
  return bytes;
}

static void ref_decode_block(stream* s, const zfp_output* o, float* f, int dim) {
  uint size = BLOCK_SIZE(dim);
  uint bits = 1;
  if (stream_read_bit(s)) {
    int32 q[17];
    uint32 u[17];
    bits += EBITS;
    int emax = (int)stream_read_bits(s, EBITS) - EBIAS;
    uint maxprec = get_precision(emax, o->maxprec, o->minexp, dim);
    uint maxbits = o->maxbits - bits;
    uint minbits = o->minbits - MIN(bits, o->minbits);
    uint dec;
    if (exceeded_maxbits(maxbits, maxprec, size)) dec = decode_partial_bitplanes(s, u, maxbits, maxprec, size);
    else dec = decode_full_bitplanes(s, u, maxprec, size);
    if (dec < minbits) { stream_skip(s, minbits - dec); dec = minbits; }
    if (dim == 2) {
      bwd_reorder_uint2int(u, q, PERM_2D, size);
      bwd_decorrelate_2d_block(q);
    } else {
      bwd_reorder_uint2int(u, q, kPerm1, size);
      bwd_lift_vector(q, 1);
    }
    bwd_cast_block(q, f, size, emax);
  } else {
    for (uint i = 0; i < size; i++) f[i] = 0;
    if (o->minbits > bits) stream_skip(s, o->minbits - bits);
  }
}

void ref_decompress(const void* in, uint64_t in_bytes, float* data, uint64_t nx, uint64_t ny,
                    const int32_t* params) {
  zfp_output o;
  set_params(&o, params);
  stream* s = stream_init((void*)in, in_bytes);
  stream_rewind(s);
  if (ny == 0) {
    for (uint64_t x = 0; x < nx; x += 4) {
      float f[4];
      ref_decode_block(s, &o, f, 1);
      for (uint64_t i = 0; i < 4 && x + i < nx; i++) data[x + i] = f[i];
    }
  } else {
    for (uint64_t y = 0; y < ny; y += 4)
      for (uint64_t x = 0; x < nx; x += 4) {
        float f[16];
        ref_decode_block(s, &o, f, 2);
        float* raw = data + y * nx + x;
        if (nx - x < 4 || ny - y < 4)
          scatter_partial_2d_block(f, raw, MIN(nx - x, 4u), MIN(ny - y, 4u), 1, (ptrdiff_t)nx);
        else
          scatter_2d_block(f, raw, 1, (ptrdiff_t)nx);
      }
  }
  free(s);
}

void ref_set_accuracy(double tol, int32_t* params) {
  zfp_output o;
  set_zfp_output_accuracy(&o, tol);
  params[0] = (int32_t)o.minbits; params[1] = (int32_t)o.maxbits; params[2] = (int32_t)o.maxprec; params[3] = o.minexp;
}

int ref_stage_emax(const float* f, int n) { return get_block_exponent(f, (uint)n); }
void ref_stage_cast(const float* f, int32_t* q, int n, int emax) { fwd_cast_block((int32*)q, f, (uint)n, emax); }
void ref_stage_xform(int32_t* q, int dim) {
  if (dim == 2) fwd_decorrelate_2d_block((int32*)q); else fwd_lift_vector((int32*)q, 1);
}
void ref_stage_reorder(const int32_t* q, uint32_t* u17, int dim) {
  if (!kPerm2[1]) { memcpy(kPerm2, PERM_2D, 16); kPerm2[16] = 0; }
  fwd_reorder_int2uint((uint32*)u17, (const int32*)q, dim == 2 ? kPerm2 : kPerm1, dim == 2 ? 16 : 4);
}
uint32_t ref_get_precision(int emax, uint32_t maxprec, int minexp, int dim) {
  return get_precision(emax, maxprec, minexp, dim);
}

}  // extern "C"
