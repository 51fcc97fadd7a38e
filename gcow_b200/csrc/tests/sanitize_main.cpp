// Stand-alone driver for the host-side sanitizer runs (AddressSanitizer +
// UndefinedBehaviorSanitizer, or ThreadSanitizer): exercises the CPU oracle on
// awkward sizes and the thread model of the all-reduce protocol, including an
// injected failure. compute-sanitizer is not available for the GPU kernels, so
// the code they share with the host (zfp_block.cuh, ar_layout.h) is checked here.
// The reference builds with -Wall -Wextra only (sw/Makefile:5).
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>
#include <vector>

extern "C" {
void gcow_params_rate(double rate, int dim, int32_t* out);
void gcow_params_accuracy(double tol, int32_t* out);
uint64_t gcow_max_output_bytes(const int32_t* params, uint64_t nx, uint64_t ny);
uint64_t gcow_oracle_compress(const float* data, uint64_t nx, uint64_t ny, const int32_t* params, uint64_t* out,
                              uint64_t* block_bits, int threads);
uint64_t gcow_oracle_decompress(const uint64_t* in, float* data, uint64_t nx, uint64_t ny, const int32_t* params,
                                int shift, int threads);
uint64_t gcow_header_compress(const float* data, uint64_t nx, uint64_t ny, const int32_t* params, uint64_t* out);
int gcow_fast1d_compress(const float* data, uint64_t n, const int32_t* params, void* out);
int gcow_fast1d_decompress(const void* in, float* data, uint64_t n, const int32_t* params, int shift);
void gcow_oracle_allreduce(const float* xs, int P, uint64_t n, const int32_t* params, int variant, int shift,
                           float* out, int threads);
int gcow_protocol_model(const float* xs, float* outs, int P, uint64_t n, int G, int bits, int variant, int shift,
                        int calls, int timeout_ms, int fault_call, int skip_rank, int delay_rank, int delay_ms,
                        int drop_src, int drop_dst, int drop_phase, int stale_epoch, uint32_t* status);
}

static float frand(uint32_t& s) { s = s * 1664525u + 1013904223u; return ((int32_t)s) * (1e-3f / 2147483648.0f); }

#define CHECK(c) do { if (!(c)) { fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #c); return 1; } } while (0)

int main() {
  uint32_t seed = 1;
  // codec on sizes that leave partial blocks and partial words
  const uint64_t sizes1[] = {1, 3, 4, 5, 63, 64, 65, 4099};
  for (uint64_t n : sizes1) {
    std::vector<float> x(n), y(n);
    for (auto& v : x) v = frand(seed);
    for (double rate : {2.0, 4.0, 8.0, 16.0, 32.0}) {
      int32_t p[4];
      gcow_params_rate(rate, 1, p);
      std::vector<uint64_t> out(gcow_max_output_bytes(p, n, 0) / 8 + 1, 0), out2(out.size(), 0);
      uint64_t bytes = gcow_oracle_compress(x.data(), n, 0, p, out.data(), nullptr, 3);
      uint64_t bytes2 = gcow_header_compress(x.data(), n, 0, p, out2.data());
      CHECK(bytes == bytes2 && !memcmp(out.data(), out2.data(), bytes));
      gcow_oracle_decompress(out.data(), y.data(), n, 0, p, 0, 3);
      if (p[1] == 16 || p[1] == 32 || p[1] == 64 || p[1] == 128) {
        std::vector<uint8_t> fast(bytes + 16, 0);
        CHECK(gcow_fast1d_compress(x.data(), n, p, fast.data()) == 0);
        CHECK(!memcmp(fast.data(), out.data(), ((n + 3) / 4) * p[1] / 8));
        std::vector<float> z(n);
        CHECK(gcow_fast1d_decompress(fast.data(), z.data(), n, p, 1) == 0);
      }
    }
  }
  {  // 2-D accuracy mode with ragged edges
    const uint64_t nx = 13, ny = 9;
    std::vector<float> x(nx * ny), y(nx * ny);
    for (auto& v : x) v = frand(seed) * 1000;
    int32_t p[4];
    gcow_params_accuracy(1e-3, p);
    std::vector<uint64_t> out(gcow_max_output_bytes(p, nx, ny) / 8 + 1, 0);
    std::vector<uint64_t> idx(((nx + 3) / 4) * ((ny + 3) / 4) + 1);
    gcow_oracle_compress(x.data(), nx, ny, p, out.data(), idx.data(), 1);
    gcow_oracle_decompress(out.data(), y.data(), nx, ny, p, 0, 1);
    for (size_t i = 0; i < x.size(); i++) CHECK(fabsf(x[i] - y[i]) <= 1e-3f);
  }
  // protocol model: healthy calls must equal the arithmetic oracle; then a dropped flag
  {
    const int P = 4, calls = 3;
    const uint64_t n = 4 * 700 + 1;
    std::vector<float> xs((size_t)calls * P * n), outs(xs.size()), ref(n);
    for (auto& v : xs) v = frand(seed);
    uint32_t status[8 * P];
    int32_t p[4];
    gcow_params_rate(8, 1, p);
    int failed = gcow_protocol_model(xs.data(), outs.data(), P, n, 3, 32, 0, 2, calls, 2000, -1, -1, -1, 0, -1, -1, -1, -1, status);
    CHECK(failed == 0);
    for (int c = 0; c < calls; c++) {
      gcow_oracle_allreduce(xs.data() + (size_t)c * P * n, P, n, p, 0, 2, ref.data(), 2);
      for (int r = 0; r < P; r++) CHECK(!memcmp(ref.data(), outs.data() + ((size_t)c * P + r) * n, n * 4));
    }
    failed = gcow_protocol_model(xs.data(), outs.data(), P, n, 3, 32, 0, 2, 2, 100, 0, -1, -1, 0, 1, 2, 0, -1, status);
    CHECK(failed == P);
    failed = gcow_protocol_model(xs.data(), outs.data(), P, n, 2, 32, 1, 2, 1, 2000, -1, -1, -1, 0, -1, -1, -1, 7, status);
    CHECK(failed == 0);
  }
  printf("sanitize_main: ok\n");
  return 0;
}
