// Work partition and symmetric-arena layout of the fused compressed all-reduce.
//
// Shared by the CUDA kernels, their launcher and the CPU thread model of the
// flag protocol, so all of them agree on who writes what where.
//
// A bucket of n floats is NB = ceil(n/4) blocks. It is cut into P shards of
// SB blocks (rank j owns shard j) and every shard into G slices (CTA i of every
// rank works on slice i of every shard in every phase). One flag exists per
// (phase, source rank, CTA): "source rank's CTA i has delivered its slice".
//
// Arena of every rank (same layout, mapped into all peers):
//   [ flags: 2 parities x 2 phases x kMaxRanks x kMaxCtas u32 ]
//   [ data region, parity 0 ][ data region, parity 1 ]
// Data region, two-shot:  recv slots [P][SB codes] then gather slots [P][SB codes]
//              one-shot:  recv slots [P][P*SB codes]
//              sparse two-shot (fixed accuracy with a bit cap): the same recv and gather slots, each followed by a
//              bitmap of SB bits. A slice is cut into kSparseChunks chunks; a chunk's kept blocks ("1" in the bitmap)
//              are packed from the chunk's first code position on, dropped blocks send nothing.
// Calls alternate parity. A rank that starts call k+2 has finished call k+1,
// whose last phase waited for every peer's phase 2 of call k+1, which a peer
// only reaches after its call k has fully completed - so parity k%2 is free.
//
// The reference has no collective of its own (its gradients go through stock
// DDP/NCCL and then a host codec, hw/models/train_imagenet.py:219,449-475);
// this partition is what replaces that pair.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define GCOW_LAYOUT_HD __host__ __device__ __forceinline__
#else
#define GCOW_LAYOUT_HD inline
#endif

namespace gcow {

constexpr int kMaxRanks = 8;
constexpr int kMaxCtas = 2048;
constexpr uint64_t kFlagBytes = 2ull * 2 * kMaxRanks * kMaxCtas * 4;

enum ArVariant : int { kTwoShot = 0, kOneShot = 1, kTwoShotNvls = 2, kTwoShotSparse = 3 };
constexpr int kSparseChunks = 8;   // packed ranges per slice: one per warp of the owner's CTA

// status codes written by a kernel that gave up waiting
enum ArStatus : uint32_t { kArOk = 0, kArTimeout = 1, kArAborted = 2, kArBadArgs = 3 };

struct ArLayout {
  uint64_t blocks;        // NB
  uint64_t shard_blocks;  // SB, multiple of 64
  uint64_t slice_blocks;  // blocks per CTA slice, multiple of 32 (of 32 * kSparseChunks in the sparse variant)
  uint32_t code_bytes;    // bytes per compressed block
  uint64_t slot_bytes;    // bytes of one source's slot in the recv area
  uint64_t recv_bytes;    // P * slot_bytes
  uint64_t gather_bytes;  // P * SB * code_bytes (two-shot), 0 (one-shot)
  uint64_t region_bytes;  // recv + gather
  uint64_t bitmap_off;    // sparse variant: byte offset of a slot's bitmap (after its SB code positions), else 0
};

GCOW_LAYOUT_HD uint64_t round_up_u64(uint64_t v, uint64_t m) { return (v + m - 1) / m * m; }

GCOW_LAYOUT_HD ArLayout ar_layout(uint64_t n, int P, int G, int bits, int variant) {
  ArLayout L;
  L.blocks = (n + 3) / 4;
  L.shard_blocks = round_up_u64((L.blocks + P - 1) / P, 64);
  if (L.shard_blocks == 0) L.shard_blocks = 64;
  const bool sparse = variant == kTwoShotSparse;
  L.slice_blocks = round_up_u64((L.shard_blocks + G - 1) / G, sparse ? 32 * kSparseChunks : 32);
  L.code_bytes = (uint32_t)bits / 8;
  uint64_t shard_bytes = L.shard_blocks * L.code_bytes;
  L.bitmap_off = 0;
  if (sparse) {
    L.bitmap_off = shard_bytes;
    shard_bytes += round_up_u64(L.shard_blocks / 8, 16);
  }
  if (variant == kOneShot) {
    L.slot_bytes = shard_bytes * P;
    L.gather_bytes = 0;
  } else {
    L.slot_bytes = shard_bytes;
    L.gather_bytes = shard_bytes * P;
  }
  L.recv_bytes = L.slot_bytes * P;
  L.region_bytes = L.recv_bytes + L.gather_bytes;
  return L;
}

// byte offset of the flag of (parity, phase, source rank, cta)
GCOW_LAYOUT_HD uint64_t flag_offset(int parity, int phase, int src, int cta) {
  return ((((uint64_t)parity * 2 + phase) * kMaxRanks + src) * kMaxCtas + cta) * 4;
}

GCOW_LAYOUT_HD uint64_t arena_bytes_for(uint64_t region_bytes) {
  return kFlagBytes + 2 * round_up_u64(region_bytes, 256);
}

GCOW_LAYOUT_HD uint64_t region_offset(int parity, uint64_t region_cap) {
  return kFlagBytes + (uint64_t)parity * round_up_u64(region_cap, 256);
}

}  // namespace gcow
