// Fused compressed all-reduce over NVLink peer memory (sm_100a).
//
// One persistent kernel per rank does the whole collective; there is no NCCL
// call and no separate codec launch. With P ranks, rank r:
//   phase 1  encodes its bucket block by block in registers and stores every
//            compressed block straight into the owner's receive slot over
//            NVLink (plain peer st.global), then releases one flag per
//            (destination, CTA);
//   phase 2  (owner of shard r) waits for the P flags of its slice, decodes the
//            P copies of each block, adds them in ascending rank order in fp32,
//            re-encodes and stores the result into every rank's gather slot -
//            P peer stores, or one multimem.st through the NVSwitch multicast
//            mapping in the NVLS variant - then releases the gather flags;
//   phase 3  waits for each shard's gather flag and decodes into the fp32
//            output, folding the division by P into the block exponent.
// The one-shot variant pushes every block to every rank in phase 1 and sums the
// P decoded copies locally (no re-encode, one network hop).
// The sparse variant is the two-shot protocol at fixed accuracy with a bit cap: a block whose values all lie below the
// tolerance is one bit in a bitmap and sends no code, the others are packed behind one another (ballot + popcount
// give each its position), so the bytes on the wire follow the data.
//
// Every wait is bounded by a globaltimer deadline and an iteration count; a CTA
// that gives up records {code, phase, peer, cta, expected, seen}, raises the
// abort flag for its siblings and returns. Nothing traps and nothing spins
// forever, so a missing peer costs a time-out, not the GPU.
//
// Replaces the reference's "NCCL all-reduce, then copy the whole gradient to
// the host, zfpy round trip, copy back" (hw/models/train_imagenet.py:219,449-475).
#include <cuda_runtime.h>
#include <stdint.h>
#include "zfp_block.cuh"
#include "ar_layout.h"

namespace gcow {

constexpr int kArThreads = 256;

struct ArArgs {
  const float* in;
  float* out;
  uint64_t n;
  int rank, world, variant, shift;
  float postscale;
  uint8_t* arena[kMaxRanks];  // every rank's arena as mapped here; arena[rank] is local memory
  uint8_t* mc_arena;          // multicast mapping of all arenas (NVLS) or nullptr
  uint64_t region_off;        // byte offset of this call's data region
  int parity;
  uint32_t epoch;
  uint64_t timeout_ns;
  uint32_t* status;           // 8 words, see record_failure
  uint32_t* abort_flag;       // local device word
  unsigned long long* stamps; // optional [gridDim.x][4] globaltimer stamps, or nullptr
  const uint16_t* enc_table;  // coder tables in global memory (see gcow_codec_tables3)
  const uint16_t* dec_table;
  const uint32_t* pair_table;
  const uint32_t* loop_table;
  float* residual;            // error feedback: added to the input before encoding, then set to x - D(E(x)); or nullptr
  int minexp;                 // sparse variant: smallest bit-plane exponent kept (fixed-accuracy rule)
  unsigned long long* wire;   // sparse variant: += codes this rank stored into other ranks' memory, or nullptr
  ArLayout L;
};

// ------------------------------------------------------------- primitives
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void mc_st_release_u32(uint32_t* p, uint32_t v) {
  asm volatile("multimem.st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
template <int BYTES> struct McStore;
template <> struct McStore<2> {  // two 16-bit codes are paired by the caller into 32 bits
  static __device__ __forceinline__ void st(void* p, const uint32_t* w) {
    asm volatile("multimem.st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(w[0]) : "memory");
  }
};
template <> struct McStore<4> {
  static __device__ __forceinline__ void st(void* p, const uint32_t* w) {
    asm volatile("multimem.st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(w[0]) : "memory");
  }
};
template <> struct McStore<8> {
  static __device__ __forceinline__ void st(void* p, const uint32_t* w) {
    uint64_t v = (uint64_t)w[0] | ((uint64_t)w[1] << 32);
    asm volatile("multimem.st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
  }
};
template <> struct McStore<16> {
  static __device__ __forceinline__ void st(void* p, const uint32_t* w) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p),
                 "f"(__uint_as_float(w[0])), "f"(__uint_as_float(w[1])), "f"(__uint_as_float(w[2])),
                 "f"(__uint_as_float(w[3]))
                 : "memory");
  }
};

// First failure wins the status record; everyone learns through abort_flag.
__device__ __forceinline__ void record_failure(const ArArgs& a, uint32_t code, int phase, int peer,
                                               uint32_t expected, uint32_t seen) {
  if (atomicCAS(a.status, 0u, code) == 0u) {
    a.status[1] = (uint32_t)phase;
    a.status[2] = (uint32_t)peer;
    a.status[3] = blockIdx.x;
    a.status[4] = expected;
    a.status[5] = seen;
    a.status[6] = a.epoch;
    __threadfence_system();
  }
  atomicExch(a.abort_flag, 1u);
}

// Bounded wait until *flag reaches `epoch`. Returns false on time-out / abort.
__device__ __forceinline__ bool wait_flag(const ArArgs& a, const uint32_t* flag, int phase, int peer) {
  const uint64_t deadline = global_ns() + a.timeout_ns;
  const uint64_t max_iters = a.timeout_ns / 8 + 4096;
  uint32_t seen = 0;
  for (uint64_t it = 0; it < max_iters; it++) {
    seen = ld_acquire_sys(flag);
    if ((int32_t)(seen - a.epoch) >= 0) return true;
    if ((it & 63) == 63) {
      if (ld_volatile_u32(a.abort_flag)) { record_failure(a, kArAborted, phase, peer, a.epoch, seen); return false; }
      if (global_ns() > deadline) break;
    }
    __nanosleep(40);
  }
  record_failure(a, kArTimeout, phase, peer, a.epoch, seen);
  return false;
}

__device__ __forceinline__ uint32_t* flag_ptr(uint8_t* arena, int parity, int phase, int src, int cta) {
  return reinterpret_cast<uint32_t*>(arena + flag_offset(parity, phase, src, cta));
}

template <int BITS> struct Code;
template <> struct Code<16> {
  static constexpr int NW = 1, BYTES = 2;
  static __device__ __forceinline__ void st(void* base, uint64_t b, const uint32_t (&w)[1]) { ((uint16_t*)base)[b] = (uint16_t)w[0]; }
  static __device__ __forceinline__ void ld(const void* base, uint64_t b, uint32_t (&w)[1]) { w[0] = ((const volatile uint16_t*)base)[b]; }
};
template <> struct Code<32> {
  static constexpr int NW = 1, BYTES = 4;
  static __device__ __forceinline__ void st(void* base, uint64_t b, const uint32_t (&w)[1]) { ((uint32_t*)base)[b] = w[0]; }
  static __device__ __forceinline__ void ld(const void* base, uint64_t b, uint32_t (&w)[1]) { w[0] = __ldcg((const uint32_t*)base + b); }
};
template <> struct Code<64> {
  static constexpr int NW = 2, BYTES = 8;
  static __device__ __forceinline__ void st(void* base, uint64_t b, const uint32_t (&w)[2]) { ((uint2*)base)[b] = make_uint2(w[0], w[1]); }
  static __device__ __forceinline__ void ld(const void* base, uint64_t b, uint32_t (&w)[2]) { uint2 v = __ldcg((const uint2*)base + b); w[0] = v.x; w[1] = v.y; }
};
template <> struct Code<128> {
  static constexpr int NW = 4, BYTES = 16;
  static __device__ __forceinline__ void st(void* base, uint64_t b, const uint32_t (&w)[4]) { ((uint4*)base)[b] = make_uint4(w[0], w[1], w[2], w[3]); }
  static __device__ __forceinline__ void ld(const void* base, uint64_t b, uint32_t (&w)[4]) { uint4 v = __ldcg((const uint4*)base + b); w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w; }
};

__device__ __forceinline__ void load_block(float* f, const float* __restrict__ in, uint64_t n, uint64_t gb, bool aligned) {
  uint64_t x0 = 4 * gb;
  if (x0 + 4 <= n) {
    if (aligned) { float4 v = reinterpret_cast<const float4*>(in)[gb]; f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w; }
    else { f[0] = in[x0]; f[1] = in[x0 + 1]; f[2] = in[x0 + 2]; f[3] = in[x0 + 3]; }
  } else {
    uint32_t c = (uint32_t)(n - x0);
    f[0] = f[1] = f[2] = f[3] = 0;
    for (uint32_t i = 0; i < c; i++) f[i] = in[x0 + i];
    pad_partial(f, c, 1);
  }
}
__device__ __forceinline__ void store_block(const float* f, float* __restrict__ out, uint64_t n, uint64_t gb, bool aligned) {
  uint64_t x0 = 4 * gb;
  if (x0 + 4 <= n) {
    if (aligned) reinterpret_cast<float4*>(out)[gb] = make_float4(f[0], f[1], f[2], f[3]);
    else { out[x0] = f[0]; out[x0 + 1] = f[1]; out[x0 + 2] = f[2]; out[x0 + 3] = f[3]; }
  } else {
    for (uint64_t i = 0; x0 + i < n; i++) out[x0 + i] = f[i];
  }
}

// Error feedback around the encoder: f += r, and after encoding r = f - D(E(f)) (what this rank's code lost).
template <int BITS, int NW>
__device__ __forceinline__ void encode_with_feedback(float (&f)[4], const ArArgs& a, uint64_t gb, const LeanTables& lt,
                                                     uint32_t (&w)[NW]) {
  const bool al = ((uintptr_t)a.residual & 15) == 0;
  float r[4];
  load_block(r, a.residual, a.n, gb, al);
  const uint64_t x0 = 4 * gb;
  if (x0 + 4 > a.n) {          // load_block pads a partial block with copies; the residual of the padding is not data
    for (uint64_t i = a.n > x0 ? a.n - x0 : 0; i < 4; i++) r[i] = 0;
  }
#pragma unroll
  for (int i = 0; i < 4; i++) f[i] += r[i];
  encode_block_1d_lean<BITS>(f, lt, w);
  float d[4];
  decode_block_1d_lean<BITS>(d, lt, w, 0);
#pragma unroll
  for (int i = 0; i < 4; i++) r[i] = f[i] - d[i];
  store_block(r, a.residual, a.n, gb, al);
}

__device__ __forceinline__ void stamp(const ArArgs& a, int slot) {
  if (a.stamps && threadIdx.x == 0) a.stamps[(uint64_t)blockIdx.x * 4 + slot] = global_ns();
}

template <int BITS>
__global__ void __launch_bounds__(kArThreads, 6)
allreduce_fused_kernel(const ArArgs a) {
  using C = Code<BITS>;
  constexpr int NW = C::NW;
  __shared__ __align__(16) uint32_t epair[kEncPairTabSize];
  __shared__ __align__(16) uint32_t dloop[kDecLoopTabSize];
  __shared__ int s_ok;
  for (int i = threadIdx.x; i < kDecLoopTabSize / 4; i += blockDim.x)
    reinterpret_cast<uint4*>(dloop)[i] = reinterpret_cast<const uint4*>(a.loop_table)[i];
  for (int i = threadIdx.x; i < kEncPairTabSize / 4; i += blockDim.x)
    reinterpret_cast<uint4*>(epair)[i] = reinterpret_cast<const uint4*>(a.pair_table)[i];
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  // the plane-by-plane tables serve the rare blocks that leave the fast path and stay in global memory
  const LeanTables lt = {a.enc_table, a.dec_table, epair, dloop};

  const int P = a.world, r = a.rank, cta = blockIdx.x, tid = threadIdx.x;
  const ArLayout& L = a.L;
  const uint64_t SB = L.shard_blocks, NB = L.blocks;
  const uint64_t s0 = (uint64_t)cta * L.slice_blocks;
  const uint64_t s1 = s0 + L.slice_blocks < SB ? s0 + L.slice_blocks : SB;
  const bool in_al = ((uintptr_t)a.in & 15) == 0, out_al = ((uintptr_t)a.out & 15) == 0;
  // Loops over (shard, block of the slice) give each warp one shard, so that short
  // slices still keep P warps busy: warp w works on shard slot w % P and, when the
  // 8 warps outnumber the shards evenly, on every (8/P)-th group of 32 blocks.
  const int warp = tid >> 5, lane = tid & 31, nwarps = kArThreads / 32;
  const int wps = (nwarps % P == 0) ? nwarps / P : 1;        // warps per shard
  const int slot = warp % P, sub = warp / P;
  const bool has_slot = warp < P * wps;
  const uint64_t b_first = s0 + (uint64_t)sub * 32 + lane, b_step = (uint64_t)wps * 32;
  uint8_t* const local = a.arena[r];
  stamp(a, 0);

  if (a.variant == kOneShot) {
    // ---- phase 1: encode once, store to every rank's slot for this source
    if (has_slot) {
      const int k = slot;
      for (uint64_t b = b_first; b < s1; b += b_step) {
        uint64_t gb = (uint64_t)k * SB + b;
        if (gb >= NB) break;
        float f[4];
        load_block(f, a.in, a.n, gb, in_al);
        uint32_t w[NW];
        if (a.residual) encode_with_feedback<BITS, NW>(f, a, gb, lt, w);
        else encode_block_1d_lean<BITS>(f, lt, w);
        for (int step = 0; step < P; step++) {
          int j = (r + 1 + step) % P;
          C::st(a.arena[j] + a.region_off + (uint64_t)r * L.slot_bytes, gb, w);
        }
      }
    }
    __syncthreads();
    if (tid < P) {
      __threadfence_system();
      st_release_sys(flag_ptr(a.arena[tid], a.parity, 0, r, cta), a.epoch);
    }
    stamp(a, 1);
    // ---- phase 2: wait for every source, decode P copies, sum, write fp32
    if (tid < P) {
      if (!wait_flag(a, flag_ptr(local, a.parity, 0, tid, cta), 1, tid)) s_ok = 0;
    }
    __syncthreads();
    if (!s_ok) return;
    stamp(a, 2);
    if (has_slot) {
      const int k = slot;
      for (uint64_t b = b_first; b < s1; b += b_step) {
        uint64_t gb = (uint64_t)k * SB + b;
        if (gb >= NB) break;
        float acc[4];
        for (int s = 0; s < P; s++) {
          uint32_t w[NW];
          C::ld(local + a.region_off + (uint64_t)s * L.slot_bytes, gb, w);
          float d[4];
          decode_block_1d_lean<BITS>(d, lt, w, 0);
          if (s == 0) { acc[0] = d[0]; acc[1] = d[1]; acc[2] = d[2]; acc[3] = d[3]; }
          else { acc[0] += d[0]; acc[1] += d[1]; acc[2] += d[2]; acc[3] += d[3]; }
        }
#pragma unroll
        for (int i = 0; i < 4; i++) acc[i] *= a.postscale;
        store_block(acc, a.out, a.n, gb, out_al);
      }
    }
    stamp(a, 3);
    return;
  }

  // ------------------------------------------------------------- two-shot
  const uint64_t shard_bytes = SB * C::BYTES;
  // ---- phase 1: encode shard j, store into owner j's slot for source r
  if (has_slot) {
    const int j = (r + 1 + slot) % P;
    uint8_t* dst = a.arena[j] + a.region_off + (uint64_t)r * L.slot_bytes;
    for (uint64_t b = b_first; b < s1; b += b_step) {
      uint64_t gb = (uint64_t)j * SB + b;
      if (gb >= NB) break;
      float f[4];
      load_block(f, a.in, a.n, gb, in_al);
      uint32_t w[NW];
      if (a.residual) encode_with_feedback<BITS, NW>(f, a, gb, lt, w);
      else encode_block_1d_lean<BITS>(f, lt, w);
      C::st(dst, b, w);
    }
  }
  __syncthreads();
  if (tid < P) {
    __threadfence_system();
    st_release_sys(flag_ptr(a.arena[tid], a.parity, 0, r, cta), a.epoch);
  }
  stamp(a, 1);

  // ---- phase 2: reduce my shard's slice, broadcast the re-encoded result
  if (tid < P) {
    if (!wait_flag(a, flag_ptr(local, a.parity, 0, tid, cta), 1, tid)) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return;
  {
    const uint64_t gather_off = a.region_off + L.recv_bytes + (uint64_t)r * shard_bytes;
    // slice bounds are multiples of 32, so a warp enters and leaves this loop
    // together; blocks past the end of the bucket are skipped by predicate
    for (uint64_t b = s0 + tid; b < s1; b += blockDim.x) {
      const uint64_t gb = (uint64_t)r * SB + b;
      const bool valid = gb < NB;
      uint32_t w[NW];
#pragma unroll
      for (int i = 0; i < NW; i++) w[i] = 0;
      if (valid) {
        // the next source's code is in flight while this one is decoded
        float acc[4];
        uint32_t c[NW], nxt[NW];
        C::ld(local + a.region_off, b, c);
        for (int s = 0; s < P; s++) {
          if (s + 1 < P) C::ld(local + a.region_off + (uint64_t)(s + 1) * L.slot_bytes, b, nxt);
          float d[4];
          decode_block_1d_lean<BITS>(d, lt, c, 0);
          if (s == 0) { acc[0] = d[0]; acc[1] = d[1]; acc[2] = d[2]; acc[3] = d[3]; }
          else { acc[0] += d[0]; acc[1] += d[1]; acc[2] += d[2]; acc[3] += d[3]; }
#pragma unroll
          for (int i = 0; i < NW; i++) c[i] = nxt[i];
        }
        encode_block_1d_lean<BITS>(acc, lt, w);
      }
      if (a.variant == kTwoShotNvls) {
        if (BITS == 16) {
          // pair two 16-bit codes so the multicast store is 32 bits wide
          uint32_t other = __shfl_down_sync(0xffffffffu, w[0], 1);
          if ((tid & 1) == 0 && valid) {
            uint32_t pair[1] = {(w[0] & 0xffffu) | (other << 16)};
            McStore<4>::st(a.mc_arena + gather_off + b * 2, pair);
          }
        } else if (valid) {
          McStore<C::BYTES>::st(a.mc_arena + gather_off + b * C::BYTES, w);
        }
      } else if (valid) {
        for (int step = 0; step < P; step++) {
          int j = (r + 1 + step) % P;
          C::st(a.arena[j] + gather_off, b, w);
        }
      }
    }
    __syncthreads();
    if (a.variant == kTwoShotNvls) {
      if (tid == 0) {
        __threadfence_system();
        mc_st_release_u32(flag_ptr(a.mc_arena, a.parity, 1, r, cta), a.epoch);
      }
    } else if (tid < P) {
      __threadfence_system();
      st_release_sys(flag_ptr(a.arena[tid], a.parity, 1, r, cta), a.epoch);
    }
  }
  stamp(a, 2);

  // ---- phase 3: decode every shard's slice into the output. All P flags are
  // awaited before the first write, so a CTA that gives up leaves `out` alone.
  if (tid < P) {
    if (!wait_flag(a, flag_ptr(local, a.parity, 1, tid, cta), 2, tid)) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return;
  if (has_slot) {
    const int j = slot;
    const uint8_t* src = local + a.region_off + L.recv_bytes + (uint64_t)j * shard_bytes;
    for (uint64_t b = b_first; b < s1; b += b_step) {
      uint64_t gb = (uint64_t)j * SB + b;
      if (gb >= NB) break;
      uint32_t w[NW];
      C::ld(src, b, w);
      float d[4];
      decode_block_1d_lean<BITS>(d, lt, w, a.shift);
      if (a.postscale != 1.0f) {
#pragma unroll
        for (int i = 0; i < 4; i++) d[i] *= a.postscale;
      }
      store_block(d, a.out, a.n, gb, out_al);
    }
  }
  stamp(a, 3);
}


// ------------------------------------------------- sparse two-shot (fixed accuracy with a bit cap)
// Encodes one block under the accuracy rule; false = dropped (decodes to zeros, nothing is sent). With error feedback
// the residual is added first and then set to what the code (or the drop) lost.
template <int BITS, int NW>
__device__ __forceinline__ bool sparse_encode(float (&f)[4], const ArArgs& a, uint64_t gb, const LeanTables& lt,
                                              uint32_t (&w)[NW]) {
  float r[4];
  const bool al = ((uintptr_t)a.residual & 15) == 0;
  if (a.residual) {
    load_block(r, a.residual, a.n, gb, al);
    const uint64_t x0 = 4 * gb;
    if (x0 + 4 > a.n) {
      for (uint64_t i = a.n > x0 ? a.n - x0 : 0; i < 4; i++) r[i] = 0;
    }
#pragma unroll
    for (int i = 0; i < 4; i++) f[i] += r[i];
  }
  const uint32_t kmin = accuracy_kmin_of(f, a.minexp);
  const bool keep = kmin < 32;
  if (keep) encode_block_1d_lean<BITS>(f, lt, w, kmin);
  if (a.residual) {
    float d[4] = {0, 0, 0, 0};
    if (keep) decode_block_1d_lean<BITS>(d, lt, w, 0, kmin);
#pragma unroll
    for (int i = 0; i < 4; i++) r[i] = f[i] - d[i];
    store_block(r, a.residual, a.n, gb, al);
  }
  return keep;
}

template <int BITS>
__global__ void __launch_bounds__(kArThreads, 5)
allreduce_sparse_kernel(const ArArgs a) {
  using C = Code<BITS>;
  constexpr int NW = C::NW;
  static_assert(kSparseChunks == kArThreads / 32, "one chunk per warp of the owner's CTA");
  __shared__ __align__(16) uint32_t epair[kEncPairTabSize];
  __shared__ __align__(16) uint32_t dloop[kDecLoopTabSize];
  __shared__ int s_ok;
  __shared__ uint32_t s_run[kArThreads / 32][kMaxRanks];
  for (int i = threadIdx.x; i < kDecLoopTabSize / 4; i += blockDim.x)
    reinterpret_cast<uint4*>(dloop)[i] = reinterpret_cast<const uint4*>(a.loop_table)[i];
  for (int i = threadIdx.x; i < kEncPairTabSize / 4; i += blockDim.x)
    reinterpret_cast<uint4*>(epair)[i] = reinterpret_cast<const uint4*>(a.pair_table)[i];
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  const LeanTables lt = {a.enc_table, a.dec_table, epair, dloop};

  const int P = a.world, r = a.rank, cta = blockIdx.x, tid = threadIdx.x;
  const ArLayout& L = a.L;
  const uint64_t SB = L.shard_blocks, NB = L.blocks;
  const uint64_t s0 = (uint64_t)cta * L.slice_blocks;
  const uint64_t s1 = s0 + L.slice_blocks < SB ? s0 + L.slice_blocks : SB;
  const uint64_t CL = L.slice_blocks / kSparseChunks;          // chunk length, a multiple of 32
  const bool in_al = ((uintptr_t)a.in & 15) == 0, out_al = ((uintptr_t)a.out & 15) == 0;
  const int warp = tid >> 5, lane = tid & 31, nwarps = kArThreads / 32;
  const uint32_t below = (1u << lane) - 1u;                    // lanes before this one
  // phases 1 and 3: warp w works on shard slot w % P and on a contiguous run of the slice's chunks
  const int wps = (nwarps % P == 0) ? nwarps / P : 1;
  const int slot = warp % P, sub = warp / P;
  const bool has_slot = warp < P * wps;
  const int cpp = kSparseChunks / wps;                         // chunks per warp: wps is 1, 2, 4 or 8
  uint8_t* const local = a.arena[r];
  unsigned long long sent = 0;
  stamp(a, 0);

  // ---- phase 1: encode shard j; kept blocks go, packed per chunk, into owner j's slot for source r
  if (has_slot) {
    const int j = (r + 1 + slot) % P;
    uint8_t* dst = a.arena[j] + a.region_off + (uint64_t)r * L.slot_bytes;
    uint32_t* dst_bm = reinterpret_cast<uint32_t*>(dst + L.bitmap_off);
    for (int c = sub * cpp; c < (sub + 1) * cpp; c++) {
      const uint64_t c0 = s0 + (uint64_t)c * CL;
      if (c0 >= s1) break;
      const uint64_t c1 = c0 + CL < s1 ? c0 + CL : s1;
      uint64_t run = 0;
      for (uint64_t base = c0; base < c1; base += 32) {
        const uint64_t b = base + lane, gb = (uint64_t)j * SB + b;
        bool keep = false;
        uint32_t w[NW];
        if (b < c1 && gb < NB) {
          float f[4];
          load_block(f, a.in, a.n, gb, in_al);
          keep = sparse_encode<BITS, NW>(f, a, gb, lt, w);
        }
        const uint32_t word = __ballot_sync(0xffffffffu, keep);
        if (keep) C::st(dst, c0 + run + __popc(word & below), w);
        if (lane == 0) dst_bm[base >> 5] = word;
        run += __popc(word);
      }
      if (j != r) sent += run;
    }
  }
  __syncthreads();
  if (tid < P) {
    __threadfence_system();
    st_release_sys(flag_ptr(a.arena[tid], a.parity, 0, r, cta), a.epoch);
  }
  stamp(a, 1);

  // ---- phase 2: warp w reduces chunk w of my shard's slice and sends the re-encoded result to every rank
  if (tid < P) {
    if (!wait_flag(a, flag_ptr(local, a.parity, 0, tid, cta), 1, tid)) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return;
  {
    const uint64_t goff = a.region_off + L.recv_bytes + (uint64_t)r * L.slot_bytes;
    const uint64_t c0 = s0 + (uint64_t)warp * CL;
    if (c0 < s1) {
      const uint64_t c1 = c0 + CL < s1 ? c0 + CL : s1;
      // packed position reached in every source's chunk: one counter per (warp, source) in shared memory, so that the
      // loop over the sources stays a loop (eight inlined copies of the decoder would not fit the instruction cache)
      if (lane < kMaxRanks) s_run[warp][lane] = 0;
      __syncwarp();
      uint64_t run_out = 0;
      for (uint64_t base = c0; base < c1; base += 32) {
        const uint64_t b = base + lane, gb = (uint64_t)r * SB + b;
        float acc[4] = {0, 0, 0, 0};                            // 0 + d is d: the sum is in ascending rank order
#pragma unroll 1
        for (int s = 0; s < P; s++) {
          const uint8_t* src = local + a.region_off + (uint64_t)s * L.slot_bytes;
          const uint32_t word = __ldcg(reinterpret_cast<const uint32_t*>(src + L.bitmap_off) + (base >> 5));
          const uint32_t run = s_run[warp][s];
          if ((word >> lane) & 1u) {
            uint32_t w[NW];
            C::ld(src, c0 + run + __popc(word & below), w);
            float d[4];
            decode_block_1d_lean<BITS>(d, lt, w, 0, accuracy_kmin(w[0], a.minexp));
#pragma unroll
            for (int i = 0; i < 4; i++) acc[i] += d[i];
          }
          __syncwarp();
          if (lane == 0) s_run[warp][s] = run + __popc(word);
        }
        __syncwarp();
        bool keep = false;
        uint32_t w[NW];
        if (b < c1 && gb < NB) {
          const uint32_t kmin = accuracy_kmin_of(acc, a.minexp);
          keep = kmin < 32;
          if (keep) encode_block_1d_lean<BITS>(acc, lt, w, kmin);
        }
        const uint32_t word = __ballot_sync(0xffffffffu, keep);
        const uint64_t at = c0 + run_out + __popc(word & below);
        for (int step = 0; step < P; step++) {
          uint8_t* g = a.arena[(r + 1 + step) % P] + goff;
          if (keep) C::st(g, at, w);
          if (lane == 0) reinterpret_cast<uint32_t*>(g + L.bitmap_off)[base >> 5] = word;
        }
        run_out += __popc(word);
      }
      sent += run_out * (uint64_t)(P - 1);
    }
    __syncthreads();
    if (tid < P) {
      __threadfence_system();
      st_release_sys(flag_ptr(a.arena[tid], a.parity, 1, r, cta), a.epoch);
    }
  }
  stamp(a, 2);

  // ---- phase 3: decode every shard's slice into the output (dropped blocks are zeros)
  if (tid < P) {
    if (!wait_flag(a, flag_ptr(local, a.parity, 1, tid, cta), 2, tid)) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return;
  if (has_slot) {
    const int j = slot;
    const uint8_t* src = local + a.region_off + L.recv_bytes + (uint64_t)j * L.slot_bytes;
    const uint32_t* bm = reinterpret_cast<const uint32_t*>(src + L.bitmap_off);
    for (int c = sub * cpp; c < (sub + 1) * cpp; c++) {
      const uint64_t c0 = s0 + (uint64_t)c * CL;
      if (c0 >= s1) break;
      const uint64_t c1 = c0 + CL < s1 ? c0 + CL : s1;
      uint64_t run = 0;
      for (uint64_t base = c0; base < c1; base += 32) {
        const uint64_t b = base + lane, gb = (uint64_t)j * SB + b;
        const uint32_t word = __ldcg(bm + (base >> 5));
        float d[4] = {0, 0, 0, 0};
        if ((word >> lane) & 1u) {
          uint32_t w[NW];
          C::ld(src, c0 + run + __popc(word & below), w);
          decode_block_1d_lean<BITS>(d, lt, w, a.shift, accuracy_kmin(w[0], a.minexp));
          if (a.postscale != 1.0f) {
#pragma unroll
            for (int i = 0; i < 4; i++) d[i] *= a.postscale;
          }
        }
        if (b < c1 && gb < NB) store_block(d, a.out, a.n, gb, out_al);
        run += __popc(word);
      }
    }
  }
  if (a.wire && lane == 0 && sent) atomicAdd(a.wire, sent);
  stamp(a, 3);
}

// Copy src -> dst only if no call so far has failed (status word still 0), and
// record the verdict for the host. With the all-reduce writing to a side buffer,
// a bucket whose collective gave up keeps its original local gradient.
__global__ void __launch_bounds__(256)
commit_kernel(const uint32_t* __restrict__ status, const float* __restrict__ src, float* __restrict__ dst,
              uint64_t n, uint32_t* __restrict__ verdict) {
  const bool ok = *status == 0;
  if (blockIdx.x == 0 && threadIdx.x == 0) *verdict = ok ? 1u : 2u;
  if (!ok) return;
  const bool al = ((((uintptr_t)src) | ((uintptr_t)dst)) & 15) == 0;
  const uint64_t n4 = al ? n / 4 : 0;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (uint64_t)gridDim.x * blockDim.x)
    reinterpret_cast<float4*>(dst)[i] = reinterpret_cast<const float4*>(src)[i];
  for (uint64_t i = n4 * 4 + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
    dst[i] = src[i];
}

// A flag wait on its own: lets the host-visible time-out path be exercised
// without a peer (the flag is one that nothing sets).
__global__ void wait_probe_kernel(const ArArgs a, const uint32_t* flag) {
  if (threadIdx.x == 0) wait_flag(a, flag, 9, 0);
}

template <int BITS>
int max_coresident_ctas(int device, bool sparse = false) {
  int per_sm = 0, sms = 0;
  if (sparse) cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, allreduce_sparse_kernel<BITS>, kArThreads, 0);
  else cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, allreduce_fused_kernel<BITS>, kArThreads, 0);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  return per_sm * sms;
}

}  // namespace gcow

using namespace gcow;

extern "C" int gcow_codec_tables4(const void** etab, const void** dtab, const void** epair, const void** dloop);

extern "C" {

uint64_t gcow_ar_arena_bytes(uint64_t region_bytes) { return arena_bytes_for(region_bytes); }
uint64_t gcow_ar_flag_bytes() { return kFlagBytes; }

// Bytes of data region one call needs (to be checked against the arena's capacity).
uint64_t gcow_ar_region_bytes(uint64_t n, int world, int ctas, int bits, int variant) {
  return ar_layout(n, world, ctas, bits, variant).region_bytes;
}

// Largest grid that is guaranteed co-resident (the flag protocol needs it).
int gcow_ar_max_ctas_v(int bits, int variant) {
  int dev = 0;
  cudaGetDevice(&dev);
  const bool sp = variant == kTwoShotSparse;
  int m = 0;
  switch (bits) {
    case 16: m = max_coresident_ctas<16>(dev, sp); break;
    case 32: m = max_coresident_ctas<32>(dev, sp); break;
    case 64: m = max_coresident_ctas<64>(dev, sp); break;
    case 128: m = max_coresident_ctas<128>(dev, sp); break;
    default: return -1;
  }
  return m < kMaxCtas ? m : kMaxCtas;
}
int gcow_ar_max_ctas(int bits) { return gcow_ar_max_ctas_v(bits, kTwoShot); }

// Launch the fused all-reduce on `stream`. `residual` (n floats, or null) enables error feedback inside the kernel: the
// encoder sees in + residual, and residual becomes what this rank's code of that sum dropped.
//   arenas: `world` device pointers (every rank's arena as mapped in this process)
//   mc_arena: multicast mapping or null; region_cap: bytes of one parity's data region
//   status: 8 u32 (device-visible); abort_flag: 1 u32; stamps: optional ctas*4 u64
// Returns 0, a CUDA error code, or -1 / -2 for bad arguments / insufficient arena.
static int ar_launch_impl(const float* in, float* out, uint64_t n, int rank, int world, int variant, int bits,
                          int ctas, int shift, float postscale, void* const* arenas, void* mc_arena,
                          uint64_t region_cap, uint32_t epoch, uint64_t timeout_ns, uint32_t* status,
                          uint32_t* abort_flag, unsigned long long* stamps, float* residual, int minexp,
                          unsigned long long* wire, void* stream) {
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || ctas < 1 || ctas > kMaxCtas) return -1;
  if (variant == kTwoShotNvls && !mc_arena) return -1;
  ArArgs a;
  a.in = in; a.out = out; a.n = n;
  a.rank = rank; a.world = world; a.variant = variant; a.shift = shift; a.postscale = postscale;
  for (int i = 0; i < kMaxRanks; i++) a.arena[i] = i < world ? (uint8_t*)arenas[i] : nullptr;
  a.mc_arena = (uint8_t*)mc_arena;
  a.parity = (int)(epoch & 1);
  a.region_off = region_offset(a.parity, region_cap);
  a.epoch = epoch;
  a.timeout_ns = timeout_ns;
  a.status = status; a.abort_flag = abort_flag; a.stamps = stamps;
  a.residual = residual;
  a.minexp = minexp;
  a.wire = wire;
  a.L = ar_layout(n, world, ctas, bits, variant);
  if (a.L.region_bytes > region_cap) return -2;
  const void *etp, *dtp, *ptp, *ltp;
  if (int rc = gcow_codec_tables4(&etp, &dtp, &ptp, &ltp)) return rc;
  a.enc_table = (const uint16_t*)etp;
  a.dec_table = (const uint16_t*)dtp;
  a.pair_table = (const uint32_t*)ptp;
  a.loop_table = (const uint32_t*)ltp;
  if (n == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (variant == kTwoShotSparse) {
    switch (bits) {
      case 16: allreduce_sparse_kernel<16><<<ctas, kArThreads, 0, s>>>(a); break;
      case 32: allreduce_sparse_kernel<32><<<ctas, kArThreads, 0, s>>>(a); break;
      case 64: allreduce_sparse_kernel<64><<<ctas, kArThreads, 0, s>>>(a); break;
      case 128: allreduce_sparse_kernel<128><<<ctas, kArThreads, 0, s>>>(a); break;
      default: return -1;
    }
    return (int)cudaGetLastError();
  }
  switch (bits) {
    case 16: allreduce_fused_kernel<16><<<ctas, kArThreads, 0, s>>>(a); break;
    case 32: allreduce_fused_kernel<32><<<ctas, kArThreads, 0, s>>>(a); break;
    case 64: allreduce_fused_kernel<64><<<ctas, kArThreads, 0, s>>>(a); break;
    case 128: allreduce_fused_kernel<128><<<ctas, kArThreads, 0, s>>>(a); break;
    default: return -1;
  }
  return (int)cudaGetLastError();
}

int gcow_ar_launch_ef(const float* in, float* out, uint64_t n, int rank, int world, int variant, int bits,
                      int ctas, int shift, float postscale, void* const* arenas, void* mc_arena,
                      uint64_t region_cap, uint32_t epoch, uint64_t timeout_ns, uint32_t* status,
                      uint32_t* abort_flag, unsigned long long* stamps, float* residual, void* stream) {
  if (variant == kTwoShotSparse) return -1;
  return ar_launch_impl(in, out, n, rank, world, variant, bits, ctas, shift, postscale, arenas, mc_arena, region_cap,
                        epoch, timeout_ns, status, abort_flag, stamps, residual, 0, nullptr, stream);
}

// The sparse variant: fixed accuracy (planes below 2^minexp are dropped, blocks wholly below it send nothing) with a cap
// of `bits` per block. `wire` (device, or null) is incremented by the number of codes stored into other ranks' memory.
int gcow_ar_launch_sparse(const float* in, float* out, uint64_t n, int rank, int world, int bits, int ctas, int shift,
                          float postscale, void* const* arenas, uint64_t region_cap, uint32_t epoch,
                          uint64_t timeout_ns, uint32_t* status, uint32_t* abort_flag, unsigned long long* stamps,
                          float* residual, int minexp, unsigned long long* wire, void* stream) {
  return ar_launch_impl(in, out, n, rank, world, kTwoShotSparse, bits, ctas, shift, postscale, arenas, nullptr,
                        region_cap, epoch, timeout_ns, status, abort_flag, stamps, residual, minexp, wire, stream);
}

int gcow_ar_launch(const float* in, float* out, uint64_t n, int rank, int world, int variant, int bits,
                   int ctas, int shift, float postscale, void* const* arenas, void* mc_arena,
                   uint64_t region_cap, uint32_t epoch, uint64_t timeout_ns, uint32_t* status,
                   uint32_t* abort_flag, unsigned long long* stamps, void* stream) {
  return gcow_ar_launch_ef(in, out, n, rank, world, variant, bits, ctas, shift, postscale, arenas, mc_arena, region_cap,
                           epoch, timeout_ns, status, abort_flag, stamps, nullptr, stream);
}

// Conditional commit of an out-of-place all-reduce result (see commit_kernel).
// verdict receives 1 (copied) or 2 (a call had failed; dst left untouched).
int gcow_ar_commit(const uint32_t* status, const float* src, float* dst, uint64_t n, uint32_t* verdict,
                   int ctas, void* stream) {
  if (!n) return 0;
  uint64_t g = (n / 4 + 255) / 256;
  if (g < 1) g = 1;
  if (g > (uint64_t)(ctas > 0 ? ctas : 148)) g = ctas > 0 ? ctas : 148;
  commit_kernel<<<(unsigned)g, 256, 0, (cudaStream_t)stream>>>(status, src, dst, n, verdict);
  return (int)cudaGetLastError();
}

// Wait (bounded) on one flag word that the caller chooses; used to test that a
// wait that is never satisfied ends with a status record instead of a hang.
int gcow_ar_wait_probe(const uint32_t* flag, uint32_t epoch, uint64_t timeout_ns, uint32_t* status,
                       uint32_t* abort_flag, void* stream) {
  ArArgs a = {};
  a.epoch = epoch; a.timeout_ns = timeout_ns; a.status = status; a.abort_flag = abort_flag;
  wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(a, flag);
  return (int)cudaGetLastError();
}

}  // extern "C"
