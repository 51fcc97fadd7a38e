// Allocation-free variant of the generic encoder.
//
// This entry point has no counterpart in the reference codec: it exists for
// callers of this library that are not in a position to allocate device memory.
// Typical cases: a process whose whole device memory has already been handed to
// a pool or caching allocator, so a cudaMalloc would fail or fragment it; a
// latency-critical loop that cannot afford the implicit device-wide
// synchronisation of cudaMalloc/cudaFree; and embedding code (plugins, language
// bindings) that is only allowed to pass buffers it was given. Such callers
// cannot use gcow_encode_generic(), which needs a caller-allocated scratch area
// sized by gcow_encode_generic_scratch_bytes().
//
// gcow_encode_generic_static() performs the same two-pass encode (per-block
// slots, prefix sum of the block lengths, bit-offset scatter) but keeps its
// scratch in a fixed array inside the library. Consequences the caller must
// know:
//   * Capacity is fixed: the scratch a call needs (the value
//     gcow_encode_generic_scratch_bytes() would return) must not exceed
//     gcow_encode_generic_static_capacity() = 8 MiB, e.g. up to about 109 000
//     4x4 blocks in accuracy mode or 1 000 000 blocks of 4 at 16 bits. Larger
//     requests are refused with GCOW_STATIC_TOO_LARGE and nothing is launched.
//   * Every GPU that loads the library holds those 8 MiB until the process exits.
//   * The first call on each device looks up the array's device address (no
//     allocation, but a runtime call); make that first call before starting any
//     stream capture.
//   * All calls on a device share the one array, which keeps the previous
//     call's contents. The encoder overwrites every word it later reads, so no
//     clearing is needed between calls, but two calls that overlap in time on the
//     same device (different streams, or different host threads) race on the
//     scratch and corrupt each other's output: serialise them on one stream.
//   * It calls no cudaMalloc, cudaFree or other allocating routine. Inputs and
//     outputs (`in`, `out`, `block_bits`) are still the caller's buffers.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  GCOW_STATIC_OK = 0,
  GCOW_STATIC_TOO_LARGE = -3,   // request needs more scratch than the built-in array holds
  GCOW_STATIC_BAD_ARGS = -1,
  GCOW_STATIC_SETUP_FAILED = -4 // the array's device address could not be obtained
};

// Bytes of built-in scratch (the fixed maximum).
uint64_t gcow_encode_generic_static_capacity(void);

// Same contract as gcow_encode_generic() minus the scratch argument:
//   in         device pointer, nx*max(ny,1) floats (ny == 0: 1-D of nx values)
//   params     host pointer to {minbits, maxbits, maxprec, minexp}
//   out        device buffer of out_bytes >= max_output_bytes; zeroed by the call
//   block_bits device buffer of blocks+1 uint64: start bit of every block, then the total
//   stream     cudaStream_t
// Returns GCOW_STATIC_OK, one of the codes above, or a positive CUDA error code.
// On a non-zero return, gcow_encode_generic_static_error() describes the reason.
int gcow_encode_generic_static(const float* in, uint64_t nx, uint64_t ny, const int32_t* params,
                               uint64_t* out, uint64_t out_bytes, uint64_t* block_bits, void* stream);

// Message for the last non-zero return on the calling thread ("" if none).
const char* gcow_encode_generic_static_error(void);

#ifdef __cplusplus
}
#endif
