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

constexpr int MAX_STREAMS = 8;

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

// One CTA per token row.  Column d of all S streams lives in one thread: the write-back is column-wise, so it is done in
// place.  u goes to shared memory for the second pass after the block-wide mean square.
template <typename TO>
__global__ void __launch_bounds__(256) stream_mix_norm_kernel(float* __restrict__ xs, const float* __restrict__ y, long long ldy,
                                                              const float* __restrict__ mix, const float* __restrict__ wr,
                                                              const float* __restrict__ rd, const float* __restrict__ norm_w,
                                                              TO* __restrict__ out_act, int S, int D, float eps) {
  extern __shared__ float sm[];  // u[D], then 32 partial sums
  float* us = sm;
  float* red = sm + D;
  __shared__ float Ms[MAX_STREAMS * MAX_STREAMS], bs[MAX_STREAMS], as[MAX_STREAMS];
  const long long t = blockIdx.x;
  if (threadIdx.x < S * S && mix != nullptr) Ms[threadIdx.x] = mix[threadIdx.x];
  if (threadIdx.x < S) {
    bs[threadIdx.x] = wr != nullptr ? wr[threadIdx.x] : 0.f;
    as[threadIdx.x] = rd != nullptr ? rd[threadIdx.x] : 0.f;
  }
  __syncthreads();
  float* xr = xs + t * S * D;
  float ss = 0.f;
  for (int d = threadIdx.x; d < D; d += 256) {
    float x[MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < MAX_STREAMS; ++s) x[s] = s < S ? xr[(long long)s * D + d] : 0.f;
    if (y != nullptr) {
      const float yv = y[t * ldy + d];
      float nx[MAX_STREAMS];
#pragma unroll
      for (int to = 0; to < MAX_STREAMS; ++to) {
        float acc = 0.f;
#pragma unroll
        for (int s = 0; s < MAX_STREAMS; ++s)
          if (s < S && to < S) acc = fmaf(Ms[s * S + to], x[s], acc);
        nx[to] = fmaf(bs[to < S ? to : 0], yv, acc);
      }
#pragma unroll
      for (int s = 0; s < MAX_STREAMS; ++s)
        if (s < S) { x[s] = nx[s]; xr[(long long)s * D + d] = nx[s]; }
    }
    if (rd != nullptr) {
      float u = 0.f;
#pragma unroll
      for (int s = 0; s < MAX_STREAMS; ++s)
        if (s < S) u = fmaf(as[s], x[s], u);
      us[d] = u;
      ss = fmaf(u, u, ss);
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
  for (int d = threadIdx.x; d < D; d += 256) {
    float v = us[d] * inv;
    if (norm_w != nullptr) v *= norm_w[d];
    st_t(out_act, t * D + d, v);
  }
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
  if (out_f32) {
    auto kern = stream_mix_norm_kernel<float>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return PG_ERR_CUDA;
    kern<<<rows, 256, smem, st>>>(xs, y, ldy, mix, write_coef, read_coef, norm_w, static_cast<float*>(out_act), S, D, eps);
  } else {
    auto kern = stream_mix_norm_kernel<bf16>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return PG_ERR_CUDA;
    kern<<<rows, 256, smem, st>>>(xs, y, ldy, mix, write_coef, read_coef, norm_w, static_cast<bf16*>(out_act), S, D, eps);
  }
  pg_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? PG_OK : PG_ERR_CUDA;
}
