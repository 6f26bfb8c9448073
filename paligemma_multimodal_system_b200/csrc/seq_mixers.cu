// Token mixers of the token-sequence decoders over a RAGGED step: the rows of a step are the new tokens of several
// requests ("entries"), each entry a run of n consecutive rows that continues a sequence whose first `ctx` tokens are
// already in the paged cache / the recurrent state.  A whole prompt, a portion of one and a single decoded token are
// the same case with different n and ctx, so the arithmetic of a position never depends on how its sequence was cut.
//
//   pg_attn_prepare        q/k RMS norm (shared per-head weight), interleaved partial rotation, weightless value norm;
//                          k and v rows go to their cache pages, q to a dense buffer
//   pg_attn_ragged         causal softmax attention of the new rows over the paged cache (grouped k/v heads, tanh soft cap,
//                          sigmoid output gate); scores, probabilities and the output accumulation in fp32
//   pg_linear_attn_scan    decayed outer-product recurrence S <- a S + k v^T, o = S^T q with the state in fp32,
//                          token by token (decode, short portions)
//   pg_linear_attn_chunked the same recurrence in blocks of 32 tokens (prompt portions)
#include "common.cuh"
#include "paligemma_b200.h"

using bf16 = __nv_bfloat16;

#define PG_ST(s) reinterpret_cast<cudaStream_t>(s)
#define PG_RET()                                                    \
  do {                                                              \
    pg_count_launch(1);                                             \
    return cudaGetLastError() == cudaSuccess ? PG_OK : PG_ERR_CUDA; \
  } while (0)

namespace {

template <typename T>
__device__ __forceinline__ float ldf(const T* p, long long i);
template <>
__device__ __forceinline__ float ldf<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ldf<bf16>(const bf16* p, long long i) { return __bfloat162float(p[i]); }
template <typename T>
__device__ __forceinline__ void stf(T* p, long long i, float v);
template <>
__device__ __forceinline__ void stf<float>(float* p, long long i, float v) { p[i] = v; }
template <>
__device__ __forceinline__ void stf<bf16>(bf16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float wmax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float sigmoidf(float z) { return 1.0f / (1.0f + expf(-z)); }

// ---------------------------------------------------------------------------------------------------------------------
// One CTA per token row.  The cos / sin of the token's rot_dims/2 angles are computed once (angle = position * frequency
// in double, so that a position in the thousands loses nothing to the product's rounding) and shared by every head.
// ---------------------------------------------------------------------------------------------------------------------
template <typename TA>
__global__ void __launch_bounds__(128) attn_prepare_kernel(const TA* __restrict__ qkv, long long ld, const int* __restrict__ pos,
                                                           const int* __restrict__ row_entry, const int* __restrict__ page_table, int max_pages,
                                                           int page, const double* __restrict__ freq, const float* __restrict__ qn,
                                                           const float* __restrict__ kn, TA* __restrict__ q_out, TA* __restrict__ k_pages,
                                                           TA* __restrict__ v_pages, int H, int G, int dim, int vdim, int rot, float eps) {
  extern __shared__ float cs[];  // cos[rot/2], sin[rot/2]
  const long long t = blockIdx.x;
  const int p = pos[t];
  for (int i = threadIdx.x; i < rot / 2; i += blockDim.x) {
    double s, c;
    sincos((double)p * freq[i], &s, &c);
    cs[i] = (float)c;
    cs[rot / 2 + i] = (float)s;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const long long pg_row = (long long)page_table[(long long)row_entry[t] * max_pages + p / page] * page + p % page;
  const TA* row = qkv + t * ld;
  for (int vec = warp; vec < H + 2 * G; vec += nw) {
    const bool is_q = vec < H, is_k = !is_q && vec < H + G;
    const int n = (is_q || is_k) ? dim : vdim;
    const long long off = is_q ? (long long)vec * dim : is_k ? (long long)H * dim + (long long)(vec - H) * dim
                                                            : (long long)(H + G) * dim + (long long)(vec - H - G) * vdim;
    float ss = 0.f;
    for (int d = lane; d < n; d += 32) { const float v = ldf(row, off + d); ss = fmaf(v, v, ss); }
    ss = wsum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
    if (is_q || is_k) {
      const float* w = is_q ? qn : kn;
      TA* dst = is_q ? q_out + t * ((long long)H * dim) + (long long)vec * dim
                     : k_pages + pg_row * ((long long)G * dim) + (long long)(vec - H) * dim;
      for (int d = lane; d < n; d += 32) {
        float a = ldf(row, off + d) * inv * w[d];
        if (d < rot) {
          const float b = ldf(row, off + (d ^ 1)) * inv * w[d ^ 1];
          const float c = cs[d >> 1], s = cs[rot / 2 + (d >> 1)];
          a = (d & 1) ? a * c + b * s : a * c - b * s;
        }
        stf(dst, d, a);
      }
    } else {
      TA* dst = v_pages + pg_row * ((long long)G * vdim) + (long long)(vec - H - G) * vdim;
      for (int d = lane; d < n; d += 32) stf(dst, d, ldf(row, off + d) * inv);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Causal attention of an entry's new rows over its paged keys / values.  CTA = 32 query rows (token x query head of one
// k/v head) of one entry; 8 warps x 4 rows.  Keys pass in tiles of 32 through shared memory (fp32); per tile lane j scores
// key j for the warp's 4 rows, the warp keeps a running max / sum per row and accumulates P V with lane <-> value columns.
// VC = ceil(vdim / 32) value columns per lane.
// ---------------------------------------------------------------------------------------------------------------------
template <typename TA, int VC>
__global__ void __launch_bounds__(256) attn_ragged_kernel(const TA* __restrict__ q, const TA* __restrict__ k_pages, const TA* __restrict__ v_pages,
                                                          const TA* __restrict__ gate, long long ldg, TA* __restrict__ out,
                                                          const int* __restrict__ entry_row0, const int* __restrict__ entry_n,
                                                          const int* __restrict__ entry_ctx, const int* __restrict__ page_table, int max_pages,
                                                          int page, int H, int G, int dim, int vdim, float scale, float softcap) {
  const int e = blockIdx.z, g = blockIdx.y, gsz = H / G;
  const int n = entry_n[e], ctx = entry_ctx[e], row0 = entry_row0[e];
  const int rows = n * gsz;
  const int r0 = blockIdx.x * 32;
  if (r0 >= rows) return;
  const int dimp = (dim + 3) & ~3, ks = dimp + 4;
  extern __shared__ __align__(16) float sm[];
  float* Qs = sm;                    // [32][dimp]
  float* Ks = Qs + 32 * dimp;        // [32][ks]
  float* Vs = Ks + 32 * ks;          // [32][vdim]
  float* Ps = Vs + 32 * vdim;        // [8][4][32]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // query rows: r -> token r / gsz, head g * gsz + r % gsz
  for (int i = threadIdx.x; i < 32 * dimp; i += 256) {
    const int r = i / dimp, d = i % dimp, rr = r0 + r;
    float v = 0.f;
    if (rr < rows && d < dim) v = ldf(q, (long long)(row0 + rr / gsz) * ((long long)H * dim) + (long long)(g * gsz + rr % gsz) * dim + d);
    Qs[i] = v;
  }
  float m[4], l[4], o[4][VC];
  int lim[4];  // last visible key of the row (-1: row does not exist)
  int wlim = -1;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m[i] = -INFINITY; l[i] = 0.f;
#pragma unroll
    for (int c = 0; c < VC; ++c) o[i][c] = 0.f;
    const int rr = r0 + warp * 4 + i;
    lim[i] = rr < rows ? ctx + rr / gsz : -1;
    wlim = max(wlim, lim[i]);
  }
  const int last_row = min(rows, r0 + 32) - 1;
  const int kmax = ctx + last_row / gsz;  // last key any row of this CTA sees
  const int* pt = page_table + (long long)e * max_pages;
  for (int k0 = 0; k0 <= kmax; k0 += 32) {
    __syncthreads();
    for (int i = threadIdx.x; i < 32 * dimp; i += 256) {
      const int r = i / dimp, d = i % dimp, j = k0 + r;
      float v = 0.f;
      if (j <= kmax && d < dim) v = ldf(k_pages, ((long long)pt[j / page] * page + j % page) * ((long long)G * dim) + (long long)g * dim + d);
      Ks[r * ks + d] = v;
    }
    for (int i = threadIdx.x; i < 32 * vdim; i += 256) {
      const int r = i / vdim, d = i % vdim, j = k0 + r;
      float v = 0.f;
      if (j <= kmax) v = ldf(v_pages, ((long long)pt[j / page] * page + j % page) * ((long long)G * vdim) + (long long)g * vdim + d);
      Vs[i] = v;
    }
    __syncthreads();
    if (k0 > wlim) continue;  // every row of this warp is past its causal limit
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    const float* kr = Ks + lane * ks;
    const float* qw = Qs + warp * 4 * dimp;
    for (int d = 0; d < dimp; d += 4) {
      const float4 kv = *reinterpret_cast<const float4*>(kr + d);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 qv = *reinterpret_cast<const float4*>(qw + i * dimp + d);
        s[i] = fmaf(qv.x, kv.x, s[i]); s[i] = fmaf(qv.y, kv.y, s[i]); s[i] = fmaf(qv.z, kv.z, s[i]); s[i] = fmaf(qv.w, kv.w, s[i]);
      }
    }
    float* pw = Ps + warp * 128;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float sc = s[i] * scale;
      if (softcap > 0.f) sc = softcap * tanhf(sc / softcap);
      const bool vis = k0 + lane <= lim[i];
      sc = vis ? sc : -INFINITY;
      const float mn = fmaxf(m[i], wmax(sc));
      float pr = 0.f, corr = 1.f;
      if (mn > -INFINITY) {
        pr = vis ? expf(sc - mn) : 0.f;
        corr = expf(m[i] - mn);  // m = -inf on the first visible tile: exp(-inf) = 0
      }
      l[i] = l[i] * corr + wsum(pr);
      m[i] = mn;
#pragma unroll
      for (int c = 0; c < VC; ++c) o[i][c] *= corr;
      pw[i * 32 + lane] = pr;
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      for (int j = 0; j < 32; j += 4) {
        const float4 p4 = *reinterpret_cast<const float4*>(pw + i * 32 + j);
        const float pv[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
        for (int jj = 0; jj < 4; ++jj)
#pragma unroll
          for (int c = 0; c < VC; ++c) {
            const int col = lane + 32 * c;
            if (col < vdim) o[i][c] = fmaf(pv[jj], Vs[(j + jj) * vdim + col], o[i][c]);
          }
      }
    }
    __syncwarp();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int rr = r0 + warp * 4 + i;
    if (rr >= rows) continue;
    const long long t = row0 + rr / gsz;
    const int head = g * gsz + rr % gsz;
    const float inv = 1.0f / l[i];
#pragma unroll
    for (int c = 0; c < VC; ++c) {
      const int col = lane + 32 * c;
      if (col < vdim) {
        float v = o[i][c] * inv;
        if (gate != nullptr) v *= sigmoidf(ldf(gate, t * ldg + (long long)head * vdim + col));
        stf(out, t * ((long long)H * vdim) + (long long)head * vdim + col, v);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Decayed linear attention, token by token.  CTA = (value-column block of VB columns, head, entry); thread = one value
// column x one slice of DC key dimensions, its part of the state in registers.  q, k, v = silu(projection) are formed
// in fp32 from the activation-type projections; state, decay and output are fp32.
// ---------------------------------------------------------------------------------------------------------------------
template <typename TA, int DCMAX>
__global__ void __launch_bounds__(256) linear_attn_scan_kernel(const TA* __restrict__ qkv, long long ld, float* __restrict__ state,
                                                               const float* __restrict__ decay, float* __restrict__ out,
                                                               const int* __restrict__ entry_row0, const int* __restrict__ entry_n,
                                                               const int* __restrict__ entry_ctx, const int* __restrict__ entry_slot, int H,
                                                               int dim, int vdim, int VB) {
  const int e = blockIdx.z, h = blockIdx.y, vb = blockIdx.x;
  const int n = entry_n[e], row0 = entry_row0[e];
  const int nchunk = 256 / VB, DC = (dim + nchunk - 1) / nchunk;
  const int vl = threadIdx.x % VB, chunk = threadIdx.x / VB;
  const int v = vb * VB + vl;
  const bool v_ok = v < vdim;
  extern __shared__ float sm[];
  float* qs = sm;              // [dim]
  float* ksm = qs + dim;       // [dim]
  float* red = ksm + dim;      // [nchunk][VB]
  float S[DCMAX];
  float* st = state + (((long long)entry_slot[e] * H + h) * dim) * vdim;
  const bool fresh = entry_ctx[e] == 0;
#pragma unroll
  for (int i = 0; i < DCMAX; ++i) {
    const int d = chunk * DC + i;
    S[i] = (!fresh && i < DC && d < dim && v_ok) ? st[(long long)d * vdim + v] : 0.f;
  }
  const float a = decay[h];
  const long long qo = (long long)h * dim, ko = (long long)H * dim + (long long)h * dim, vo = 2LL * H * dim + (long long)h * vdim;
  for (int t = 0; t < n; ++t) {
    const TA* row = qkv + (long long)(row0 + t) * ld;
    for (int d = threadIdx.x; d < dim; d += 256) {
      qs[d] = silu(ldf(row, qo + d));
      ksm[d] = silu(ldf(row, ko + d));
    }
    const float vv = v_ok ? silu(ldf(row, vo + v)) : 0.f;
    __syncthreads();
    float part = 0.f;
#pragma unroll
    for (int i = 0; i < DCMAX; ++i) {
      const int d = chunk * DC + i;
      if (i < DC && d < dim) {
        S[i] = fmaf(a, S[i], ksm[d] * vv);
        part = fmaf(S[i], qs[d], part);
      }
    }
    red[chunk * VB + vl] = part;
    __syncthreads();
    if (chunk == 0 && v_ok) {
      float o = 0.f;
      for (int c = 0; c < nchunk; ++c) o += red[c * VB + vl];
      out[(long long)(row0 + t) * ((long long)H * vdim) + (long long)h * vdim + v] = o;
    }
  }
#pragma unroll
  for (int i = 0; i < DCMAX; ++i) {
    const int d = chunk * DC + i;
    if (i < DC && d < dim && v_ok) st[(long long)d * vdim + v] = S[i];
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// The same recurrence advanced 32 tokens at a time.  With a = decay, block rows i, j = 0 .. c-1 and S the state before the block:
//   o_i = sum_{j <= i} a^(i-j) (q_i . k_j) v_j  +  a^(i+1) S^T q_i        S' = a^c S + sum_j a^(c-1-j) k_j v_j^T
// CTA = (value-column block, head, entry); the state block [dim][VB] lives in shared memory for the whole entry.
// Thread = value column x row group for the outputs, value column x key-dimension slice for the state update.
// ---------------------------------------------------------------------------------------------------------------------
template <typename TA>
__global__ void __launch_bounds__(256) linear_attn_chunked_kernel(const TA* __restrict__ qkv, long long ld, float* __restrict__ state,
                                                                  const float* __restrict__ decay, float* __restrict__ out,
                                                                  const int* __restrict__ entry_row0, const int* __restrict__ entry_n,
                                                                  const int* __restrict__ entry_ctx, const int* __restrict__ entry_slot, int H,
                                                                  int dim, int vdim, int VB) {
  constexpr int C = 32;
  const int e = blockIdx.z, h = blockIdx.y, vb = blockIdx.x;
  const int n = entry_n[e], row0 = entry_row0[e];
  const int ngrp = 256 / VB, rpt = C / ngrp;  // row groups; rows per thread (<= 8 because VB <= 64)
  const int vl = threadIdx.x % VB, grp = threadIdx.x / VB;
  const int v = vb * VB + vl;
  const bool v_ok = v < vdim;
  const int kd = dim + 1;
  extern __shared__ float sm[];
  float* Qs = sm;                 // [C][kd]
  float* Ks = Qs + C * kd;        // [C][kd]
  float* Vs = Ks + C * kd;        // [C][VB]
  float* As = Vs + C * VB;        // [C][C]
  float* Ss = As + C * C;         // [dim][VB]
  float* ap = Ss + dim * VB;      // a^0 .. a^C
  float* st = state + (((long long)entry_slot[e] * H + h) * dim) * vdim;
  const bool fresh = entry_ctx[e] == 0;
  for (int i = threadIdx.x; i < dim * VB; i += 256) {
    const int d = i / VB, c = vb * VB + i % VB;
    Ss[i] = (!fresh && c < vdim) ? st[(long long)d * vdim + c] : 0.f;
  }
  const double a = (double)decay[h];
  for (int i = threadIdx.x; i <= C; i += 256) ap[i] = (float)pow(a, (double)i);
  const long long qo = (long long)h * dim, ko = (long long)H * dim + (long long)h * dim, vo = 2LL * H * dim + (long long)h * vdim;
  for (int t0 = 0; t0 < n; t0 += C) {
    const int cn = min(C, n - t0);
    __syncthreads();
    for (int i = threadIdx.x; i < C * dim; i += 256) {
      const int r = i / dim, d = i % dim;
      float qv = 0.f, kv = 0.f;
      if (r < cn) {
        const TA* row = qkv + (long long)(row0 + t0 + r) * ld;
        qv = silu(ldf(row, qo + d));
        kv = silu(ldf(row, ko + d));
      }
      Qs[r * kd + d] = qv;
      Ks[r * kd + d] = kv;
    }
    for (int i = threadIdx.x; i < C * VB; i += 256) {
      const int r = i / VB, c = vb * VB + i % VB;
      Vs[i] = (r < cn && c < vdim) ? silu(ldf(qkv + (long long)(row0 + t0 + r) * ld, vo + c)) : 0.f;
    }
    __syncthreads();
    // A[i][j] = a^(i-j) q_i . k_j  (j <= i)
    for (int idx = threadIdx.x; idx < C * C; idx += 256) {
      const int i = idx / C, j = idx % C;
      float s = 0.f;
      if (j <= i) {
        for (int d = 0; d < dim; ++d) s = fmaf(Qs[i * kd + d], Ks[j * kd + d], s);
        s *= ap[i - j];
      }
      As[idx] = s;
    }
    __syncthreads();
    // outputs of the thread's rows i = grp * rpt + r
    float acc[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) acc[r] = 0.f;
    for (int d = 0; d < dim; ++d) {
      const float sv = Ss[d * VB + vl];
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < rpt) acc[r] = fmaf(Qs[(grp * rpt + r) * kd + d], sv, acc[r]);
    }
#pragma unroll
    for (int r = 0; r < 8; ++r)
      if (r < rpt) acc[r] *= ap[grp * rpt + r + 1];
    for (int j = 0; j < C; ++j) {
      const float vv = Vs[j * VB + vl];
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < rpt) acc[r] = fmaf(As[(grp * rpt + r) * C + j], vv, acc[r]);
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const int i = grp * rpt + r;
      if (r < rpt && i < cn && v_ok) out[(long long)(row0 + t0 + i) * ((long long)H * vdim) + (long long)h * vdim + v] = acc[r];
    }
    __syncthreads();  // every read of the old state is done
    // state: thread = value column x key dimensions d = grp, grp + ngrp, ...
    float vw[C];
#pragma unroll
    for (int j = 0; j < C; ++j) vw[j] = j < cn ? Vs[j * VB + vl] * ap[cn - 1 - j] : 0.f;
    const float ac = ap[cn];
    for (int d = grp; d < dim; d += ngrp) {
      float s = ac * Ss[d * VB + vl];
#pragma unroll
      for (int j = 0; j < C; ++j) s = fmaf(Ks[j * kd + d], vw[j], s);
      Ss[d * VB + vl] = s;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < dim * VB; i += 256) {
    const int d = i / VB, c = vb * VB + i % VB;
    if (c < vdim) st[(long long)d * vdim + c] = Ss[i];
  }
}

}  // namespace

extern "C" int pg_attn_prepare(const void* qkv, long long ld, const int* pos, const int* row_entry, const int* page_table, int max_pages,
                               int page, const double* freq, const float* q_norm, const float* k_norm, void* q_out, void* k_pages,
                               void* v_pages, int rows, int H, int G, int dim, int vdim, int rot_dims, float eps, int act_f32, void* stream) {
  if (rows <= 0 || H <= 0 || G <= 0 || dim <= 0 || vdim <= 0 || rot_dims < 0 || rot_dims > dim || (rot_dims & 1) || page <= 0) return PG_ERR_ARG;
  const size_t smem = (size_t)(rot_dims + 2) * sizeof(float);
  if (act_f32)
    attn_prepare_kernel<float><<<rows, 128, smem, PG_ST(stream)>>>(static_cast<const float*>(qkv), ld, pos, row_entry, page_table, max_pages, page, freq,
                                                                  q_norm, k_norm, static_cast<float*>(q_out), static_cast<float*>(k_pages),
                                                                  static_cast<float*>(v_pages), H, G, dim, vdim, rot_dims, eps);
  else
    attn_prepare_kernel<bf16><<<rows, 128, smem, PG_ST(stream)>>>(static_cast<const bf16*>(qkv), ld, pos, row_entry, page_table, max_pages, page, freq,
                                                                 q_norm, k_norm, static_cast<bf16*>(q_out), static_cast<bf16*>(k_pages),
                                                                 static_cast<bf16*>(v_pages), H, G, dim, vdim, rot_dims, eps);
  PG_RET();
}

template <typename TA, int VC>
static int launch_attn_ragged(const void* q, const void* kp, const void* vp, const void* gate, long long ldg, void* out, const int* row0,
                              const int* n, const int* ctx, const int* pt, int max_pages, int page, int entries, int max_n, int H, int G,
                              int dim, int vdim, float scale, float softcap, cudaStream_t st) {
  const int dimp = (dim + 3) & ~3;
  const size_t smem = ((size_t)32 * dimp + 32 * (dimp + 4) + 32 * vdim + 8 * 128) * sizeof(float);
  if (smem > 220 * 1024) return PG_ERR_ARG;
  auto kern = attn_ragged_kernel<TA, VC>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return PG_ERR_CUDA;
  dim3 grid((max_n * (H / G) + 31) / 32, G, entries);
  kern<<<grid, 256, smem, st>>>(static_cast<const TA*>(q), static_cast<const TA*>(kp), static_cast<const TA*>(vp), static_cast<const TA*>(gate), ldg,
                                static_cast<TA*>(out), row0, n, ctx, pt, max_pages, page, H, G, dim, vdim, scale, softcap);
  PG_RET();
}

extern "C" int pg_attn_ragged(const void* q, const void* k_pages, const void* v_pages, const void* gate, long long ldg, void* out,
                              const int* entry_row0, const int* entry_n, const int* entry_ctx, const int* page_table, int max_pages, int page,
                              int entries, int max_n, int H, int G, int dim, int vdim, float scale, float softcap, int act_f32, void* stream) {
  if (entries <= 0 || max_n <= 0 || H <= 0 || G <= 0 || (H % G) != 0 || dim <= 0 || vdim <= 0 || vdim > 256 || entries > 65535 || G > 65535)
    return PG_ERR_ARG;
  cudaStream_t st = PG_ST(stream);
#define PG_ATTN(TA, VC) \
  return launch_attn_ragged<TA, VC>(q, k_pages, v_pages, gate, ldg, out, entry_row0, entry_n, entry_ctx, page_table, max_pages, page, entries, max_n, \
                                    H, G, dim, vdim, scale, softcap, st)
  if (act_f32) {
    if (vdim <= 64) PG_ATTN(float, 2);
    if (vdim <= 128) PG_ATTN(float, 4);
    PG_ATTN(float, 8);
  }
  if (vdim <= 64) PG_ATTN(bf16, 2);
  if (vdim <= 128) PG_ATTN(bf16, 4);
  PG_ATTN(bf16, 8);
#undef PG_ATTN
}

template <typename TA, int DCMAX>
static int launch_scan(const void* qkv, long long ld, float* state, const float* decay, float* out, const int* row0, const int* n, const int* ctx,
                       const int* slot, int entries, int H, int dim, int vdim, int VB, cudaStream_t st) {
  const int nchunk = 256 / VB;
  const size_t smem = ((size_t)2 * dim + (size_t)nchunk * VB) * sizeof(float);
  dim3 grid((vdim + VB - 1) / VB, H, entries);
  linear_attn_scan_kernel<TA, DCMAX><<<grid, 256, smem, st>>>(static_cast<const TA*>(qkv), ld, state, decay, out, row0, n, ctx, slot, H, dim, vdim, VB);
  PG_RET();
}

extern "C" int pg_linear_attn_scan(const void* qkv, long long ld, float* state, const float* decay, float* out, const int* entry_row0,
                                   const int* entry_n, const int* entry_ctx, const int* entry_slot, int entries, int H, int dim, int vdim,
                                   int act_f32, void* stream) {
  if (entries <= 0 || H <= 0 || dim <= 0 || vdim <= 0 || dim > 1024 || entries > 65535 || H > 65535) return PG_ERR_ARG;
  cudaStream_t st = PG_ST(stream);
  // VB value columns per CTA (a power of two <= 64); the 256 / VB thread groups split the key dimensions
  int VB = 64;
  while (VB > 8 && VB / 2 >= vdim) VB /= 2;
  const int DC = (dim + 256 / VB - 1) / (256 / VB);
#define PG_SCAN(TA, DCM) return launch_scan<TA, DCM>(qkv, ld, state, decay, out, entry_row0, entry_n, entry_ctx, entry_slot, entries, H, dim, vdim, VB, st)
  if (act_f32) {
    if (DC <= 16) PG_SCAN(float, 16);
    if (DC <= 64) PG_SCAN(float, 64);
    PG_SCAN(float, 256);
  }
  if (DC <= 16) PG_SCAN(bf16, 16);
  if (DC <= 64) PG_SCAN(bf16, 64);
  PG_SCAN(bf16, 256);
#undef PG_SCAN
}

extern "C" int pg_linear_attn_chunked(const void* qkv, long long ld, float* state, const float* decay, float* out, const int* entry_row0,
                                      const int* entry_n, const int* entry_ctx, const int* entry_slot, int entries, int H, int dim, int vdim,
                                      int act_f32, void* stream) {
  if (entries <= 0 || H <= 0 || dim <= 0 || vdim <= 0 || entries > 65535 || H > 65535) return PG_ERR_ARG;
  int VB = 64;
  while (VB > 8 && VB / 2 >= vdim) VB /= 2;
  auto bytes = [&](int vb) { return ((size_t)2 * 32 * (dim + 1) + 32 * vb + 32 * 32 + (size_t)dim * vb + 33) * sizeof(float); };
  while (VB > 8 && bytes(VB) > 200 * 1024) VB /= 2;
  const size_t smem = bytes(VB);
  if (smem > 200 * 1024) return PG_ERR_ARG;
  dim3 grid((vdim + VB - 1) / VB, H, entries);
  cudaStream_t st = PG_ST(stream);
  if (act_f32) {
    auto kern = linear_attn_chunked_kernel<float>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return PG_ERR_CUDA;
    kern<<<grid, 256, smem, st>>>(static_cast<const float*>(qkv), ld, state, decay, out, entry_row0, entry_n, entry_ctx, entry_slot, H, dim, vdim, VB);
  } else {
    auto kern = linear_attn_chunked_kernel<bf16>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return PG_ERR_CUDA;
    kern<<<grid, 256, smem, st>>>(static_cast<const bf16*>(qkv), ld, state, decay, out, entry_row0, entry_n, entry_ctx, entry_slot, H, dim, vdim, VB);
  }
  PG_RET();
}
