/* Plain-C user of the host library through gcow.h: the reference's zfp_compress call sequence
 * (sw/tests/test_zfp.cpp: field exp(-(x^2+y^2)), tolerance 1e-3, compare with the golden stream) without Python.
 * usage: capi_main n golden.zfp   -> exit 0 when the stream equals the golden file and the round trip is within
 * the tolerance. */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "gcow.h"

int main(int argc, char** argv) {
  if (argc < 3) return 2;
  const uint64_t n = (uint64_t)atoll(argv[1]);
  float* field = (float*)malloc(n * n * sizeof(float));
  for (uint64_t y = 0; y < n; y++)
    for (uint64_t x = 0; x < n; x++) {
      const double fx = 2.0 * (double)x / (double)n, fy = 2.0 * (double)y / (double)n;
      field[y * n + x] = (float)exp(-(fx * fx + fy * fy));
    }
  int32_t params[4];
  gcow_params_accuracy(1e-3, params);
  const uint64_t cap = gcow_max_output_bytes(params, n, n);
  uint64_t* out = (uint64_t*)calloc(cap / 8 + 2, 8);
  const uint64_t bytes = gcow_oracle_compress(field, n, n, params, out, NULL, 1);
  FILE* f = fopen(argv[2], "rb");
  if (!f) return 3;
  unsigned char* gold = (unsigned char*)malloc(cap + 16);
  const size_t got = fread(gold, 1, cap + 16, f);
  fclose(f);
  if (got != bytes || memcmp(gold, out, bytes) != 0) { printf("stream differs: %llu vs %zu bytes\n", (unsigned long long)bytes, got); return 1; }
  float* back = (float*)malloc(n * n * sizeof(float));
  gcow_oracle_decompress(out, back, n, n, params, 0, 1);
  double worst = 0;
  for (uint64_t i = 0; i < n * n; i++) { const double e = fabs((double)back[i] - (double)field[i]); if (e > worst) worst = e; }
  printf("bytes %llu max_abs_error %.3g\n", (unsigned long long)bytes, worst);
  return worst <= 1e-3 ? 0 : 4;
}
