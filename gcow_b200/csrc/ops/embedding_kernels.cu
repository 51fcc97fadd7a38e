// Embedding kernels of the BERT input layer: y = tok[ids] + pos[position] + typ[type_ids] in one pass, and its
// deterministic backward (no atomics): position and type gradients are ordered sums over the batch, the token
// gradient is a segmented sum over the tokens sorted by id, one CTA per distinct id.
//
// Not in the reference (its models are CNNs); needed by the BERT-large configuration of the benchmark.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gcow {
namespace emb {

typedef __nv_bfloat16 bf16;

// one CTA per token, H / 4 threads, float4 table reads, 8-byte bf16 stores
__global__ void embed3_fwd_kernel(const int64_t* __restrict__ ids, const int64_t* __restrict__ type_ids,
                                  const float* __restrict__ tok, const float* __restrict__ pos, const float* __restrict__ typ,
                                  bf16* __restrict__ y, int S, int H) {
  const int t = blockIdx.x;
  const int64_t id = ids[t], ty = type_ids[t];
  const int s = t % S;
  for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
    const float4 a = *reinterpret_cast<const float4*>(tok + (size_t)id * H + c);
    const float4 b = *reinterpret_cast<const float4*>(pos + (size_t)s * H + c);
    const float4 d = *reinterpret_cast<const float4*>(typ + (size_t)ty * H + c);
    __nv_bfloat162 lo = __floats2bfloat162_rn(a.x + b.x + d.x, a.y + b.y + d.y);
    __nv_bfloat162 hi = __floats2bfloat162_rn(a.z + b.z + d.z, a.w + b.w + d.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&lo);
    o.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(y + (size_t)t * H + c) = o;
  }
}

// dpos[s, :] = sum over the batch of gy[b, s, :], in batch order. grid = S, block = H / 2 threads (bf16 pairs).
__global__ void embed_pos_bwd_kernel(const bf16* __restrict__ gy, float* __restrict__ dpos, int B, int S, int H) {
  const int s = blockIdx.x;
  for (int c = threadIdx.x * 2; c < H; c += blockDim.x * 2) {
    float a0 = 0.0f, a1 = 0.0f;
    for (int b = 0; b < B; b++) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gy + ((size_t)b * S + s) * H + c));
      a0 += f.x; a1 += f.y;
    }
    dpos[(size_t)s * H + c] = a0;
    dpos[(size_t)s * H + c + 1] = a1;
  }
}

// part[p][k][c] = sum over tokens t in slab p with type_ids[t] == k of gy[t][c]; slabs are added by reduce_partials.
// grid = (H / 512, parts), block 256 threads x 2 columns; `types` <= 4 accumulators per thread.
__global__ void embed_type_bwd_kernel(const bf16* __restrict__ gy, const int64_t* __restrict__ type_ids,
                                      float* __restrict__ part, int T, int H, int types, int rows_per) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (c >= H) return;
  const int t0 = blockIdx.y * rows_per, t1 = min(T, t0 + rows_per);
  float acc[4][2] = {{0, 0}, {0, 0}, {0, 0}, {0, 0}};
  for (int t = t0; t < t1; t++) {
    const int k = (int)type_ids[t];
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gy + (size_t)t * H + c));
#pragma unroll
    for (int j = 0; j < 4; j++) if (j == k) { acc[j][0] += f.x; acc[j][1] += f.y; }
  }
  for (int k = 0; k < types; k++) {
    float* o = part + ((size_t)blockIdx.y * types + k) * H + c;
    o[0] = acc[k][0]; o[1] = acc[k][1];
  }
}

// Token gradient. `order` lists the token positions sorted by id (stable). CTA i looks at sorted position i; if it
// starts a run of equal ids it adds the run's rows of gy in sorted order and writes the row of that id.
// Rows of ids that do not occur are left untouched (the caller zero-fills the table).
__global__ void embed_tok_bwd_kernel(const bf16* __restrict__ gy, const int64_t* __restrict__ ids,
                                     const int64_t* __restrict__ order, float* __restrict__ dtok, int T, int H) {
  const int i = blockIdx.x;
  const int64_t id = ids[order[i]];
  if (i > 0 && ids[order[i - 1]] == id) return;            // not the first of its run
  for (int c = threadIdx.x * 2; c < H; c += blockDim.x * 2) {
    float a0 = 0.0f, a1 = 0.0f;
    for (int j = i; j < T; j++) {
      const int64_t t = order[j];
      if (ids[t] != id) break;
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gy + (size_t)t * H + c));
      a0 += f.x; a1 += f.y;
    }
    dtok[(size_t)id * H + c] = a0;
    dtok[(size_t)id * H + c + 1] = a1;
  }
}

}  // namespace emb
}  // namespace gcow

using namespace gcow::emb;

extern "C" {

// y[T, H] (bf16) = tok[ids] + pos[t mod S] + typ[type_ids]; fp32 tables, int64 indices, H a multiple of 4.
int gcow_embed3_fwd(const int64_t* ids, const int64_t* type_ids, const float* tok, const float* pos, const float* typ,
                    void* y, int T, int S, int H, void* stream) {
  if (T <= 0) return 0;
  if (H % 4 || S <= 0) return -1;
  int threads = H / 4 < 256 ? ((H / 4 + 31) / 32) * 32 : 256;
  embed3_fwd_kernel<<<T, threads, 0, (cudaStream_t)stream>>>(ids, type_ids, tok, pos, typ, (bf16*)y, S, H);
  return (int)cudaGetLastError();
}

int gcow_embed_type_parts(int T) { int p = (T + 255) / 256; return p < 1 ? 1 : (p > 128 ? 128 : p); }

// Gradients of the three tables from gy[T = B*S, H] (bf16). dtok [V, H] must be zero-filled by the caller; dpos gets
// its first S rows written; type_part must hold gcow_embed_type_parts(T) * types * H floats, and the caller adds its
// slabs into dtyp [types, H] (gcow_reduce_partials). `order`: token positions sorted by id. types <= 4, H even.
int gcow_embed3_bwd(const void* gy, const int64_t* ids, const int64_t* type_ids, const int64_t* order, float* dtok,
                    float* dpos, float* type_part, int B, int S, int H, int types, void* stream) {
  const int T = B * S;
  if (T <= 0) return 0;
  if (H % 2 || types < 1 || types > 4) return -1;
  cudaStream_t st = (cudaStream_t)stream;
  const int threads = H / 2 < 256 ? ((H / 2 + 31) / 32) * 32 : 256;
  embed_tok_bwd_kernel<<<T, threads, 0, st>>>((const bf16*)gy, ids, order, dtok, T, H);
  embed_pos_bwd_kernel<<<S, threads, 0, st>>>((const bf16*)gy, dpos, B, S, H);
  const int parts = gcow_embed_type_parts(T), rows_per = (T + parts - 1) / parts;
  dim3 grid((H / 2 + 255) / 256, parts);
  embed_type_bwd_kernel<<<grid, 256, 0, st>>>((const bf16*)gy, type_ids, type_part, T, H, types, rows_per);
  return (int)cudaGetLastError();
}

}  // extern "C"
