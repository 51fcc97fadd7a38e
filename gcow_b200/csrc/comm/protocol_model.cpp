// CPU thread model of the fused all-reduce's flag protocol.
//
// P host threads play the ranks and G "CTAs" per rank are played in sequence by
// that thread, running the same three phases, the same arena layout
// (ar_layout.h) and the same block codec (zfp_block.cuh, host build) as the
// CUDA kernel. Flags are std::atomic<uint32_t> with release/acquire ordering
// and every wait has a deadline. The model exists to test what must never be
// tested by faulting a GPU: a rank that never joins, a late rank, a dropped
// flag, a stale epoch left in a flag, parity reuse across calls. It is also
// what runs under ThreadSanitizer (build.py: sanitize="thread").
//
// The reference has no distributed failure handling to mirror (its host code
// exits on any OpenCL error, hw/include/host.hpp:18-24).
#include <stdint.h>
#include <string.h>
#include <atomic>
#include <chrono>
#include <thread>
#include <vector>

#include "../codec/zfp_block.cuh"
#include "ar_layout.h"

namespace {

using namespace gcow;
using Clock = std::chrono::steady_clock;

struct Fault {
  int skip_rank;        // this rank never runs (-1: none)
  int delay_rank;       // this rank starts late (-1: none)
  int delay_ms;
  int drop_src, drop_dst, drop_phase;  // flag (src -> dst, phase) is never written (-1: none)
};

struct Model {
  int P, G, bits, variant, shift, minexp;
  uint64_t n, region_cap;
  ArLayout L;
  std::vector<std::vector<uint8_t>> arena;  // one per rank
  std::vector<uint16_t> etab, dtab;
};

std::atomic<uint32_t>* flag_at(Model& m, int rank, int parity, int phase, int src, int cta) {
  return reinterpret_cast<std::atomic<uint32_t>*>(m.arena[rank].data() + flag_offset(parity, phase, src, cta));
}

bool wait_flag(std::atomic<uint32_t>* f, uint32_t epoch, int timeout_ms, uint32_t* seen) {
  auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
  for (;;) {
    uint32_t v = f->load(std::memory_order_acquire);
    *seen = v;
    if ((int32_t)(v - epoch) >= 0) return true;
    if (Clock::now() > deadline) return false;
    std::this_thread::yield();
  }
}

template <int NW>
void put_code(uint8_t* base, uint64_t b, const uint32_t (&w)[NW], int bytes) {
  memcpy(base + b * bytes, w, bytes);
}
template <int NW>
void get_code(const uint8_t* base, uint64_t b, uint32_t (&w)[NW], int bytes) {
  for (int i = 0; i < NW; i++) w[i] = 0;
  memcpy(w, base + b * bytes, bytes);
}

void load_block(float* f, const float* in, uint64_t n, uint64_t gb) {
  uint64_t x0 = 4 * gb;
  uint32_t c = (uint32_t)(n - x0 < 4 ? n - x0 : 4);
  f[0] = f[1] = f[2] = f[3] = 0;
  for (uint32_t i = 0; i < c; i++) f[i] = in[x0 + i];
  if (c < 4) pad_partial(f, c, 1);
}
void store_block(const float* f, float* out, uint64_t n, uint64_t gb) {
  uint64_t x0 = 4 * gb;
  for (uint64_t i = 0; i < 4 && x0 + i < n; i++) out[x0 + i] = f[i];
}

// status: [0] code, [1] phase, [2] peer, [3] cta, [4] expected, [5] seen
template <int BITS>
void run_rank(Model& m, int r, const float* in, float* out, uint32_t epoch, int timeout_ms,
              const Fault& ft, uint32_t* status) {
  constexpr int NW = (BITS + 31) / 32;
  const int P = m.P, G = m.G, parity = (int)(epoch & 1), bytes = m.bits / 8;
  const ArLayout& L = m.L;
  const uint64_t SB = L.shard_blocks, NB = L.blocks;
  const uint64_t roff = region_offset(parity, m.region_cap);
  auto fail = [&](int phase, int peer, int cta, uint32_t seen) {
    if (status[0] == 0) { status[0] = kArTimeout; status[1] = phase; status[2] = peer; status[3] = cta; status[4] = epoch; status[5] = seen; }
  };
  auto signal = [&](int dst, int phase, int cta) {
    if (ft.drop_src == r && ft.drop_dst == dst && ft.drop_phase == phase) return;
    flag_at(m, dst, parity, phase, r, cta)->store(epoch, std::memory_order_release);
  };
  const uint64_t shard_bytes = SB * bytes;

  // phase 1 for every CTA
  for (int cta = 0; cta < G; cta++) {
    uint64_t s0 = (uint64_t)cta * L.slice_blocks, s1 = std::min<uint64_t>(s0 + L.slice_blocks, SB);
    if (m.variant == kOneShot) {
      for (int k = 0; k < P; k++)
        for (uint64_t b = s0; b < s1; b++) {
          uint64_t gb = (uint64_t)k * SB + b;
          if (gb >= NB) break;
          float f[4]; uint32_t w[NW];
          load_block(f, in, m.n, gb);
          encode_block_1d_rate<BITS>(f, m.etab.data(), w);
          for (int j = 0; j < P; j++) put_code<NW>(m.arena[j].data() + roff + (uint64_t)r * L.slot_bytes, gb, w, bytes);
        }
      for (int j = 0; j < P; j++) signal(j, 0, cta);
    } else {
      for (int step = 0; step < P; step++) {
        int j = (r + 1 + step) % P;
        for (uint64_t b = s0; b < s1; b++) {
          uint64_t gb = (uint64_t)j * SB + b;
          if (gb >= NB) break;
          float f[4]; uint32_t w[NW];
          load_block(f, in, m.n, gb);
          encode_block_1d_rate<BITS>(f, m.etab.data(), w);
          put_code<NW>(m.arena[j].data() + roff + (uint64_t)r * L.slot_bytes, b, w, bytes);
        }
        signal(j, 0, cta);
      }
    }
  }
  // phase 2
  const float inv = 1.0f / (float)(1u << m.shift);
  for (int cta = 0; cta < G; cta++) {
    uint64_t s0 = (uint64_t)cta * L.slice_blocks, s1 = std::min<uint64_t>(s0 + L.slice_blocks, SB);
    for (int s = 0; s < P; s++) {
      uint32_t seen;
      if (!wait_flag(flag_at(m, r, parity, 0, s, cta), epoch, timeout_ms, &seen)) { fail(1, s, cta, seen); return; }
    }
    const uint8_t* local = m.arena[r].data();
    if (m.variant == kOneShot) {
      for (int k = 0; k < P; k++)
        for (uint64_t b = s0; b < s1; b++) {
          uint64_t gb = (uint64_t)k * SB + b;
          if (gb >= NB) break;
          float acc[4] = {0, 0, 0, 0};
          for (int s = 0; s < P; s++) {
            uint32_t w[NW]; float d[4];
            get_code<NW>(local + roff + (uint64_t)s * L.slot_bytes, gb, w, bytes);
            decode_block_1d_rate<BITS>(d, m.dtab.data(), w, 0);
            for (int i = 0; i < 4; i++) acc[i] = s == 0 ? d[i] : acc[i] + d[i];
          }
          for (int i = 0; i < 4; i++) acc[i] *= inv;
          store_block(acc, out, m.n, gb);
        }
      continue;
    }
    for (uint64_t b = s0; b < s1; b++) {
      uint64_t gb = (uint64_t)r * SB + b;
      if (gb >= NB) break;
      float acc[4] = {0, 0, 0, 0};
      for (int s = 0; s < P; s++) {
        uint32_t w[NW]; float d[4];
        get_code<NW>(local + roff + (uint64_t)s * L.slot_bytes, b, w, bytes);
        decode_block_1d_rate<BITS>(d, m.dtab.data(), w, 0);
        for (int i = 0; i < 4; i++) acc[i] = s == 0 ? d[i] : acc[i] + d[i];
      }
      uint32_t w[NW];
      encode_block_1d_rate<BITS>(acc, m.etab.data(), w);
      for (int j = 0; j < P; j++)
        put_code<NW>(m.arena[j].data() + roff + L.recv_bytes + (uint64_t)r * shard_bytes, b, w, bytes);
    }
    for (int j = 0; j < P; j++) signal(j, 1, cta);
  }
  if (m.variant == kOneShot) return;
  // phase 3
  for (int cta = 0; cta < G; cta++) {
    uint64_t s0 = (uint64_t)cta * L.slice_blocks, s1 = std::min<uint64_t>(s0 + L.slice_blocks, SB);
    for (int j = 0; j < P; j++) {
      uint32_t seen;
      if (!wait_flag(flag_at(m, r, parity, 1, j, cta), epoch, timeout_ms, &seen)) { fail(2, j, cta, seen); return; }
    }
    for (int j = 0; j < P; j++) {
      const uint8_t* src = m.arena[r].data() + roff + L.recv_bytes + (uint64_t)j * shard_bytes;
      for (uint64_t b = s0; b < s1; b++) {
        uint64_t gb = (uint64_t)j * SB + b;
        if (gb >= NB) break;
        uint32_t w[NW]; float d[4];
        get_code<NW>(src, b, w, bytes);
        decode_block_1d_rate<BITS>(d, m.dtab.data(), w, m.shift);
        store_block(d, out, m.n, gb);
      }
    }
  }
}

// The sparse variant (fixed accuracy with a bit cap): the same flags, with the kept blocks of every chunk packed
// behind one another and a bitmap beside them, exactly as allreduce_sparse_kernel lays them out.
template <int BITS>
void run_rank_sparse(Model& m, int r, const float* in, float* out, uint32_t epoch, int timeout_ms,
                     const Fault& ft, uint32_t* status) {
  constexpr int NW = (BITS + 31) / 32;
  const int P = m.P, G = m.G, parity = (int)(epoch & 1), bytes = m.bits / 8;
  const ArLayout& L = m.L;
  const uint64_t SB = L.shard_blocks, NB = L.blocks, CL = L.slice_blocks / kSparseChunks;
  const uint64_t roff = region_offset(parity, m.region_cap);
  auto fail = [&](int phase, int peer, int cta, uint32_t seen) {
    if (status[0] == 0) { status[0] = kArTimeout; status[1] = phase; status[2] = peer; status[3] = cta; status[4] = epoch; status[5] = seen; }
  };
  auto signal = [&](int dst, int phase, int cta) {
    if (ft.drop_src == r && ft.drop_dst == dst && ft.drop_phase == phase) return;
    flag_at(m, dst, parity, phase, r, cta)->store(epoch, std::memory_order_release);
  };
  auto set_bit = [](uint8_t* slot_bitmap, uint64_t b, bool v) {
    uint32_t* wd = reinterpret_cast<uint32_t*>(slot_bitmap) + (b >> 5);
    if ((b & 31) == 0) *wd = 0;
    if (v) *wd |= 1u << (b & 31);
  };
  auto get_bit = [](const uint8_t* slot_bitmap, uint64_t b) {
    return (reinterpret_cast<const uint32_t*>(slot_bitmap)[b >> 5] >> (b & 31)) & 1u;
  };
  // phase 1
  for (int cta = 0; cta < G; cta++) {
    uint64_t s0 = (uint64_t)cta * L.slice_blocks, s1 = std::min<uint64_t>(s0 + L.slice_blocks, SB);
    for (int step = 0; step < P; step++) {
      int j = (r + 1 + step) % P;
      uint8_t* dst = m.arena[j].data() + roff + (uint64_t)r * L.slot_bytes;
      for (uint64_t c0 = s0; c0 < s1; c0 += CL) {
        uint64_t c1 = std::min<uint64_t>(c0 + CL, s1), run = 0;
        for (uint64_t b = c0; b < c1; b++) {
          uint64_t gb = (uint64_t)j * SB + b;
          bool keep = false;
          uint32_t w[NW];
          if (gb < NB) {
            float f[4];
            load_block(f, in, m.n, gb);
            keep = accuracy_kmin_of(f, m.minexp) < 32;
            if (keep) encode_block_1d_rate<BITS>(f, m.etab.data(), w);
          }
          if (keep) put_code<NW>(dst, c0 + run++, w, bytes);
          set_bit(dst + L.bitmap_off, b, keep);
        }
      }
      signal(j, 0, cta);
    }
  }
  // phase 2
  for (int cta = 0; cta < G; cta++) {
    uint64_t s0 = (uint64_t)cta * L.slice_blocks, s1 = std::min<uint64_t>(s0 + L.slice_blocks, SB);
    for (int s = 0; s < P; s++) {
      uint32_t seen;
      if (!wait_flag(flag_at(m, r, parity, 0, s, cta), epoch, timeout_ms, &seen)) { fail(1, s, cta, seen); return; }
    }
    const uint8_t* local = m.arena[r].data();
    const uint64_t goff = roff + L.recv_bytes + (uint64_t)r * L.slot_bytes;
    for (uint64_t c0 = s0; c0 < s1; c0 += CL) {
      uint64_t c1 = std::min<uint64_t>(c0 + CL, s1), run_out = 0;
      std::vector<uint64_t> run_in(P, 0);
      for (uint64_t b = c0; b < c1; b++) {
        uint64_t gb = (uint64_t)r * SB + b;
        float acc[4] = {0, 0, 0, 0};
        for (int s = 0; s < P; s++) {
          const uint8_t* src = local + roff + (uint64_t)s * L.slot_bytes;
          if (!get_bit(src + L.bitmap_off, b)) continue;
          uint32_t w[NW]; float d[4];
          get_code<NW>(src, c0 + run_in[s]++, w, bytes);
          decode_block_1d_rate<BITS>(d, m.dtab.data(), w, 0, accuracy_kmin(w[0], m.minexp));
          for (int i = 0; i < 4; i++) acc[i] += d[i];
        }
        bool keep = false;
        uint32_t w[NW];
        if (gb < NB) {
          keep = accuracy_kmin_of(acc, m.minexp) < 32;
          if (keep) encode_block_1d_rate<BITS>(acc, m.etab.data(), w);
        }
        for (int j = 0; j < P; j++) {
          uint8_t* g = m.arena[j].data() + goff;
          if (keep) put_code<NW>(g, c0 + run_out, w, bytes);
          set_bit(g + L.bitmap_off, b, keep);
        }
        run_out += keep;
      }
    }
    for (int j = 0; j < P; j++) signal(j, 1, cta);
  }
  // phase 3
  for (int cta = 0; cta < G; cta++) {
    uint64_t s0 = (uint64_t)cta * L.slice_blocks, s1 = std::min<uint64_t>(s0 + L.slice_blocks, SB);
    for (int j = 0; j < P; j++) {
      uint32_t seen;
      if (!wait_flag(flag_at(m, r, parity, 1, j, cta), epoch, timeout_ms, &seen)) { fail(2, j, cta, seen); return; }
    }
    for (int j = 0; j < P; j++) {
      const uint8_t* src = m.arena[r].data() + roff + L.recv_bytes + (uint64_t)j * L.slot_bytes;
      for (uint64_t c0 = s0; c0 < s1; c0 += CL) {
        uint64_t c1 = std::min<uint64_t>(c0 + CL, s1), run = 0;
        for (uint64_t b = c0; b < c1; b++) {
          uint64_t gb = (uint64_t)j * SB + b;
          float d[4] = {0, 0, 0, 0};
          if (get_bit(src + L.bitmap_off, b)) {
            uint32_t w[NW];
            get_code<NW>(src, c0 + run++, w, bytes);
            decode_block_1d_rate<BITS>(d, m.dtab.data(), w, m.shift, accuracy_kmin(w[0], m.minexp));
          }
          if (gb < NB) store_block(d, out, m.n, gb);
        }
      }
    }
  }
}

}  // namespace

extern "C" {

// Run `calls` consecutive all-reduces of P ranks x n floats on host threads.
// xs: [calls][P][n] inputs; outs: [calls][P][n] outputs; status: [P][8] words
// (first failure per rank over all calls). The fault applies to call
// `fault_call` only; stale_epoch >= 0 pre-seeds every flag with that value
// before the first call. Returns the number of ranks that reported a failure.
// `minexp` matters to the sparse variant (3) only: the fixed-accuracy rule's smallest bit-plane exponent.
int gcow_protocol_model2(const float* xs, float* outs, int P, uint64_t n, int G, int bits, int variant,
                         int shift, int calls, int timeout_ms, int fault_call, int skip_rank,
                         int delay_rank, int delay_ms, int drop_src, int drop_dst, int drop_phase,
                         int stale_epoch, uint32_t* status, int minexp) {
  Model m;
  m.P = P; m.G = G; m.bits = bits; m.variant = variant; m.shift = shift; m.n = n; m.minexp = minexp;
  m.L = ar_layout(n, P, G, bits, variant);
  m.region_cap = m.L.region_bytes;
  m.arena.assign(P, std::vector<uint8_t>(arena_bytes_for(m.region_cap), 0));
  m.etab.resize(kEncTabSize);
  m.dtab.resize(kDecBudgetTabSize);
  build_codec_tables(m.etab.data(), m.dtab.data());
  if (stale_epoch >= 0)
    for (int r = 0; r < P; r++)
      for (uint64_t o = 0; o < kFlagBytes; o += 4) *reinterpret_cast<uint32_t*>(m.arena[r].data() + o) = (uint32_t)stale_epoch;
  memset(status, 0, sizeof(uint32_t) * 8 * P);
  uint32_t first_epoch = stale_epoch >= 0 ? (uint32_t)stale_epoch + 1 : 1;
  for (int c = 0; c < calls; c++) {
    Fault ft = {-1, -1, 0, -1, -1, -1};
    if (c == fault_call) ft = {skip_rank, delay_rank, delay_ms, drop_src, drop_dst, drop_phase};
    std::vector<std::thread> th;
    for (int r = 0; r < P; r++) {
      if (ft.skip_rank == r) continue;
      th.emplace_back([&, r, c, ft] {
        if (ft.delay_rank == r) std::this_thread::sleep_for(std::chrono::milliseconds(ft.delay_ms));
        const float* in = xs + ((uint64_t)c * P + r) * n;
        float* out = outs + ((uint64_t)c * P + r) * n;
        uint32_t epoch = first_epoch + (uint32_t)c;
        if (variant == kTwoShotSparse) {
          switch (bits) {
            case 16: run_rank_sparse<16>(m, r, in, out, epoch, timeout_ms, ft, status + 8 * r); break;
            case 32: run_rank_sparse<32>(m, r, in, out, epoch, timeout_ms, ft, status + 8 * r); break;
            case 64: run_rank_sparse<64>(m, r, in, out, epoch, timeout_ms, ft, status + 8 * r); break;
            default: run_rank_sparse<128>(m, r, in, out, epoch, timeout_ms, ft, status + 8 * r); break;
          }
          return;
        }
        switch (bits) {
          case 16: run_rank<16>(m, r, in, out, epoch, timeout_ms, ft, status + 8 * r); break;
          case 32: run_rank<32>(m, r, in, out, epoch, timeout_ms, ft, status + 8 * r); break;
          case 64: run_rank<64>(m, r, in, out, epoch, timeout_ms, ft, status + 8 * r); break;
          default: run_rank<128>(m, r, in, out, epoch, timeout_ms, ft, status + 8 * r); break;
        }
      });
    }
    for (auto& t : th) t.join();
  }
  int failed = 0;
  for (int r = 0; r < P; r++) failed += status[8 * r] != 0;
  return failed;
}

int gcow_protocol_model(const float* xs, float* outs, int P, uint64_t n, int G, int bits, int variant,
                        int shift, int calls, int timeout_ms, int fault_call, int skip_rank,
                        int delay_rank, int delay_ms, int drop_src, int drop_dst, int drop_phase,
                        int stale_epoch, uint32_t* status) {
  return gcow_protocol_model2(xs, outs, P, n, G, bits, variant, shift, calls, timeout_ms, fault_call, skip_rank,
                              delay_rank, delay_ms, drop_src, drop_dst, drop_phase, stale_epoch, status, -1074);
}

}  // extern "C"
