// Multi-stream residual ("hyper-connections") of the token-sequence decoders.  The residual of a token is S fp32 rows
// x_1..x_S (xs [T, S, D]).  A sub-layer reads the combination u = sum_s a_s x_s through an RMS norm, and its output y rebuilds
// every stream from the old ones:  x_t <- sum_s M[s, t] x_s + b_t y.
//
//   pg_embed_streams     every stream of a token starts as its embedding row
//   pg_stream_mix_norm   one pass per row that (1) applies the write-back of the sub-layer that just finished (y, M, b) and
//                        (2) forms the read u of the next sub-layer, normalises it and leaves it in the activation type --
//                        either half may be absent (first read of a step; last write-back; stream sum + final norm)
//
// All sums, the norm statistics and the streams are fp32.
#include "common.cuh"
#include "paligemma_b200.h"

using bf16 = __nv_bfloat16;

#define PG_ST(s) reinterpret_cast<cudaStream_t>(s)

namespace {

constexpr int MAX_STREAMS = 16;

template <typename T>
__device__ __forceinline__ float ld_t(const T* p, long long i);
template <>
__device__ __forceinline__ float ld_t<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ld_t<bf16>(const bf16* p, long long i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void st_t(float* p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void st_t(bf16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }

template <typename TI>
__global__ void embed_streams_kernel(const int* __restrict__ tokens, const TI* __restrict__ table, long long ld, float* __restrict__ xs, int S, int D,
                                     float scale) {
  const long long t = blockIdx.x;
  const long long row = tokens[t];
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const float v = ld_t(table, row * ld + d) * scale;
    for (int s = 0; s < S; ++s) xs[(t * S + s) * D + d] = v;
  }
}

// One CTA per token row.  A thread holds V consecutive columns of all S streams (V = 4: 16-byte accesses): the write-back is
// column-wise, so it is done in place.  u goes to shared memory for the second pass after the block-wide mean square.
// SMAX = 4, 8 or 16 bounds the unrolled stream loops.
template <int V>
struct VecF;
template <>
struct VecF<1> {
  float v[1];
  __device__ __forceinline__ void load(const float* p) { v[0] = *p; }
  __device__ __forceinline__ void store(float* p) const { *p = v[0]; }
};
template <>
struct VecF<4> {
  float v[4];
  __device__ __forceinline__ void load(const float* p) { const float4 t = *reinterpret_cast<const float4*>(p); v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
  __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
__device__ __forceinline__ void st_vec(float* p, const float* v, int n) {
  if (n == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  else p[0] = v[0];
}
__device__ __forceinline__ void st_vec(bf16* p, const float* v, int n) {
  if (n == 4) {
    uint2 u;
    u.x = pg::pack_bf16(v[0], v[1]);
    u.y = pg::pack_bf16(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = u;
  } else {
    p[0] = __float2bfloat16_rn(v[0]);
  }
}

template <typename TO, int V, int SMAX>
__global__ void __launch_bounds__(256) stream_mix_norm_kernel(float* __restrict__ xs, const float* __restrict__ y, long long ldy,
                                                              const float* __restrict__ mix, const float* __restrict__ wr,
                                                              const float* __restrict__ rd, const float* __restrict__ norm_w,
                                                              TO* __restrict__ out_act, int S, int D, float eps) {
  extern __shared__ __align__(16) float sm[];  // u[D], then 32 partial sums
  float* us = sm;
  float* red = sm + D;
  __shared__ float Ms[MAX_STREAMS * MAX_STREAMS], bs[MAX_STREAMS], as[MAX_STREAMS];
  const long long t = blockIdx.x;
  if (threadIdx.x < MAX_STREAMS * MAX_STREAMS) {
    const int from = threadIdx.x / MAX_STREAMS, to = threadIdx.x % MAX_STREAMS;
    Ms[threadIdx.x] = (mix != nullptr && from < S && to < S) ? mix[from * S + to] : 0.f;
  }
  if (threadIdx.x < MAX_STREAMS) {
    bs[threadIdx.x] = (wr != nullptr && threadIdx.x < S) ? wr[threadIdx.x] : 0.f;
    as[threadIdx.x] = (rd != nullptr && threadIdx.x < S) ? rd[threadIdx.x] : 0.f;
  }
  __syncthreads();
  float* xr = xs + t * S * D;
  float ss = 0.f;
  for (int d = threadIdx.x * V; d < D; d += 256 * V) {
    VecF<V> x[SMAX];
#pragma unroll
    for (int s = 0; s < SMAX; ++s) {
      if (s < S) x[s].load(xr + (long long)s * D + d);
      else {
#pragma unroll
        for (int j = 0; j < V; ++j) x[s].v[j] = 0.f;
      }
    }
    if (y != nullptr) {
      VecF<V> yv, nx[SMAX];
      yv.load(y + t * ldy + d);
#pragma unroll
      for (int to = 0; to < SMAX; ++to)
#pragma unroll
        for (int j = 0; j < V; ++j) {
          float acc = 0.f;
#pragma unroll
          for (int s = 0; s < SMAX; ++s) acc = fmaf(Ms[s * MAX_STREAMS + to], x[s].v[j], acc);  // rows / columns past S are zero
          nx[to].v[j] = fmaf(bs[to], yv.v[j], acc);
        }
#pragma unroll
      for (int s = 0; s < SMAX; ++s)
        if (s < S) { x[s] = nx[s]; nx[s].store(xr + (long long)s * D + d); }
    }
    if (rd != nullptr) {
#pragma unroll
      for (int j = 0; j < V; ++j) {
        float u = 0.f;
#pragma unroll
        for (int s = 0; s < SMAX; ++s) u = fmaf(as[s], x[s].v[j], u);
        us[d + j] = u;
        ss = fmaf(u, u, ss);
      }
    }
  }
  if (rd == nullptr) return;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) tot += red[w];
  const float inv = 1.0f / sqrtf(tot / (float)D + eps);
  for (int d = threadIdx.x * V; d < D; d += 256 * V) {
    float v[V];
#pragma unroll
    for (int j = 0; j < V; ++j) v[j] = us[d + j] * inv * (norm_w != nullptr ? norm_w[d + j] : 1.0f);
    st_vec(out_act + t * D + d, v, V);
  }
}

template <typename TO, int V, int SMAX>
int launch_stream(float* xs, const float* y, long long ldy, const float* mix, const float* wr, const float* rd, const float* norm_w, void* out_act,
                  int rows, int S, int D, float eps, size_t smem, cudaStream_t st) {
  auto kern = stream_mix_norm_kernel<TO, V, SMAX>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return PG_ERR_CUDA;
  kern<<<rows, 256, smem, st>>>(xs, y, ldy, mix, wr, rd, norm_w, static_cast<TO*>(out_act), S, D, eps);
  pg_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? PG_OK : PG_ERR_CUDA;
}

}  // namespace

extern "C" int pg_embed_streams(const int* tokens, const void* table, long long ld, float* xs, int rows, int S, int D, float scale, int table_f32,
                                void* stream) {
  if (rows <= 0 || D <= 0 || S <= 0) return PG_ERR_ARG;
  if (table_f32)
    embed_streams_kernel<float><<<rows, 128, 0, PG_ST(stream)>>>(tokens, static_cast<const float*>(table), ld, xs, S, D, scale);
  else
    embed_streams_kernel<bf16><<<rows, 128, 0, PG_ST(stream)>>>(tokens, static_cast<const bf16*>(table), ld, xs, S, D, scale);
  pg_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? PG_OK : PG_ERR_CUDA;
}

extern "C" int pg_stream_mix_norm(float* xs, const float* y, long long ldy, const float* mix, const float* write_coef, const float* read_coef,
                                  const float* norm_w, void* out_act, int rows, int S, int D, float eps, int out_f32, void* stream) {
  if (rows <= 0 || D <= 0 || S <= 0 || S > MAX_STREAMS || xs == nullptr) return PG_ERR_ARG;
  if ((y != nullptr) != (mix != nullptr) || (y != nullptr) != (write_coef != nullptr)) return PG_ERR_ARG;
  if ((read_coef != nullptr) != (out_act != nullptr)) return PG_ERR_ARG;
  const size_t smem = ((size_t)D + 32) * sizeof(float);
  if (smem > 200 * 1024) return PG_ERR_ARG;
  cudaStream_t st = PG_ST(stream);
  // 16-byte accesses: rows of the streams, of y and of the output start on 16-byte boundaries (8 for a bf16 output)
  const bool vec = D % 4 == 0 && ldy % 4 == 0 && ((reinterpret_cast<uintptr_t>(xs) | reinterpret_cast<uintptr_t>(y)) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(out_act) & (out_f32 ? 15 : 7)) == 0;
#define PG_STREAM(TO, V, SM) return launch_stream<TO, V, SM>(xs, y, ldy, mix, write_coef, read_coef, norm_w, out_act, rows, S, D, eps, smem, st)
  if (out_f32) {
    if (S > 8) PG_STREAM(float, 1, 16);
    if (vec && S <= 4) PG_STREAM(float, 4, 4);
    if (vec) PG_STREAM(float, 4, 8);
    if (S <= 4) PG_STREAM(float, 1, 4);
    PG_STREAM(float, 1, 8);
  }
  if (S > 8) PG_STREAM(bf16, 1, 16);
  if (vec && S <= 4) PG_STREAM(bf16, 4, 4);
  if (vec) PG_STREAM(bf16, 4, 8);
  if (S <= 4) PG_STREAM(bf16, 1, 4);
  PG_STREAM(bf16, 1, 8);
#undef PG_STREAM
}
