/* C interface of the gcow_b200 codec libraries.
 *
 * libgcow_cpu.so  - the host codec (serial / multi-threaded oracle), no CUDA needed;
 * libgcow_cuda.so - the sm_100a kernels; pointers are device pointers, `stream` is a cudaStream_t.
 *
 * Counterpart of the reference's sw/include/zfp.h + common.h (zfp_compress / zfp_decompress on a zfp_input /
 * zfp_output pair with the four parameters set by hand or by set_zfp_output_accuracy): here the four parameters
 * travel as int32_t[4] = {minbits, maxbits, maxprec, minexp} and arrays as (pointer, nx, ny), ny == 0 meaning a
 * one-dimensional array cut into blocks of 4 instead of 4 x 4. Streams are header-less, LSB-first, padded to a
 * 64-bit word, byte-identical to the reference's for two-dimensional input.
 */
#ifndef GCOW_H_
#define GCOW_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- parameters (both libraries export these from the host side: libgcow_cpu.so) */
void gcow_params_rate(double bits_per_value, int dim, int32_t* params_out);
void gcow_params_accuracy(double tolerance, int32_t* params_out);      /* sw/src/common.c:6-21 */
void gcow_params_precision(uint32_t planes, int32_t* params_out);
uint64_t gcow_max_output_bytes(const int32_t* params, uint64_t nx, uint64_t ny);   /* sw/src/common.c:187-224 */
uint32_t gcow_block_precision(int emax, uint32_t maxprec, int minexp, int dim);

/* ---- host codec (libgcow_cpu.so) */
/* Compress; `out` holds gcow_max_output_bytes(); block_bits (nullable) receives blocks + 1 bit offsets.
 * Returns the stream size in bytes. Fixed-rate streams are encoded by `threads` threads. */
uint64_t gcow_oracle_compress(const float* data, uint64_t nx, uint64_t ny, const int32_t* params, uint64_t* out,
                              uint64_t* block_bits, int threads);
/* Decompress; every value is divided by 2^shift. `in` must be readable one word past the stream.
 * Returns the number of stream bits consumed. */
uint64_t gcow_oracle_decompress(const uint64_t* in, float* data, uint64_t nx, uint64_t ny, const int32_t* params,
                                int shift, int threads);
/* out = D(E(sum_r D(E(x_r)))) / 2^shift (variant 0, 2) or (sum_r D(E(x_r))) / 2^shift (variant 1) for P arrays of n
 * values stored back to back, fp32 sums in ascending rank order: the result every rank of the fused all-reduce
 * must produce, bit for bit. One-dimensional blocks, fixed-rate parameters. */
void gcow_oracle_allreduce(const float* xs, int P, uint64_t n, const int32_t* params, int variant, int shift,
                           float* out, int threads);

/* ---- device codec (libgcow_cuda.so); all return 0 or a CUDA error code */
int gcow_encode_1d_fixed(const float* in, uint64_t n, int maxbits, void* out, void* stream);   /* maxbits 16/32/64/128 */
int gcow_decode_1d_fixed(const void* in, float* out, uint64_t n, int maxbits, int shift, void* stream);
uint64_t gcow_encode_generic_scratch_bytes(const int32_t* params, uint64_t blocks, int dim);
int gcow_encode_generic(const float* in, uint64_t nx, uint64_t ny, const int32_t* params, uint64_t* out,
                        uint64_t out_bytes, void* scratch, uint64_t* block_bits, void* stream);
int gcow_encode_fixed_direct(const float* in, uint64_t nx, uint64_t ny, const int32_t* params, uint64_t* out,
                             void* stream);                                                  /* maxbits % 64 == 0 */
int gcow_decode_generic(const uint64_t* in, float* out, uint64_t nx, uint64_t ny, const int32_t* params,
                        const uint64_t* block_bits, int shift, void* stream);

#ifdef __cplusplus
}
#endif
#endif  /* GCOW_H_ */
