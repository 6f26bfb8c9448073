// Causal attention of prompt portions over the paged bf16 cache on the tensor cores, with the probabilities kept at fp32
// precision.
//
// The design asks for scores and probabilities in 32 bits.  q and k are bf16 here (they are stored so), so S = Q K^T from
// bf16 x bf16 products accumulated in fp32 is exact to fp32 rounding.  The probabilities P = exp(s - m) stay fp32 in
// registers; for P V each is cut into THREE bf16 terms p = p1 + p2 + p3 (8 + 8 + 8 mantissa bits) and the product is three
// tensor-core passes over the same bf16 V tile accumulated in fp32 -- the result carries fp32 P, not a bf16 rounding of it.
// Soft cap, running max / sum and the output gate are fp32 SIMT code on the accumulator fragments.
//
// CTA = 64 query rows (token x query head of one k/v head) of one entry, 4 warps x 16 rows; keys in tiles of 64.
// mma.sync.m16n8k16 fragments: S accumulators of two adjacent 8-key blocks are, element for element, the A operand of one
// 16-key step of P V, so P never leaves the registers.  (tcgen05 would want P in shared or tensor memory as bf16; three
// passes from there cost the round trips this kernel avoids.)
#include "common.cuh"
#include "paligemma_b200.h"

using bf16 = __nv_bfloat16;

namespace {

__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// tanh to fp32 accuracy without the library's slow path: odd series below 0.1 (next term 17 x^7 / 315 < 6e-10), else
// 1 - 2 / (exp(2|x|) + 1), whose absolute error of ~1e-7 is relative there as well
__device__ __forceinline__ float tanh32(float x) {
  const float ax = fabsf(x), x2 = x * x;
  const float small = x * fmaf(x2, fmaf(x2, 0.13333333f, -0.33333334f), 1.0f);
  const float big = copysignf(1.0f - __fdividef(2.0f, exp2f(ax * 2.885390082f) + 1.0f), x);
  return ax < 0.1f ? small : big;
}

// p = hi + mid + lo with bf16 terms (round to nearest each time; the remainders are exact in fp32)
__device__ __forceinline__ void split3(float p, float q, uint32_t& hi, uint32_t& mid, uint32_t& lo) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(p, q);
  const float2 hf = __bfloat1622float2(h);
  const float rp = p - hf.x, rq = q - hf.y;
  const __nv_bfloat162 m = __floats2bfloat162_rn(rp, rq);
  const float2 mf = __bfloat1622float2(m);
  const __nv_bfloat162 l = __floats2bfloat162_rn(rp - mf.x, rq - mf.y);
  hi = *reinterpret_cast<const uint32_t*>(&h);
  mid = *reinterpret_cast<const uint32_t*>(&m);
  lo = *reinterpret_cast<const uint32_t*>(&l);
}

template <int DIM, int VDIM>
__global__ void __launch_bounds__(128, (DIM + VDIM <= 128) ? 4 : 2) attn_ragged_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                                                              const bf16* __restrict__ gate, long long ldg, bf16* __restrict__ out,
                                                              const int* __restrict__ entry_row0, const int* __restrict__ entry_n,
                                                              const int* __restrict__ entry_ctx, const int* __restrict__ page_table, int max_pages,
                                                              int page, int H, int G, float scale, float softcap, int skip_single, int gate_per_head) {
  constexpr int KS = DIM / 16, NV = VDIM / 8, QP = DIM + 8, VP = 64 + 8;
  const int e = blockIdx.z, g = blockIdx.y, gsz = H / G;
  const int n = entry_n[e], ctx = entry_ctx[e], row0 = entry_row0[e];
  if (skip_single && n == 1) return;
  const int rows = n * gsz;
  const int r0 = blockIdx.x * 64;
  if (r0 >= rows) return;
  extern __shared__ __align__(16) unsigned char smraw[];
  bf16* Qs = reinterpret_cast<bf16*>(smraw);  // [64][QP]
  bf16* Ks = Qs + 64 * QP;                    // [64][QP]
  bf16* Vt = Ks + 64 * QP;                    // [VDIM][VP]  (transposed: value column x key)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gq = lane >> 2, tq = lane & 3;
  // Q tile (zero rows past the end)
  for (int id = threadIdx.x; id < 64 * (DIM / 8); id += 128) {
    const int r = id / (DIM / 8), cc = id % (DIM / 8), rr = r0 + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (rr < rows) v = *reinterpret_cast<const uint4*>(q + (long long)(row0 + rr / gsz) * ((long long)H * DIM) + (long long)(g * gsz + rr % gsz) * DIM + cc * 8);
    *reinterpret_cast<uint4*>(Qs + r * QP + cc * 8) = v;
  }
  __syncthreads();
  uint32_t qa[KS][4];
  const int rl = warp * 16 + gq, rh = rl + 8;
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    qa[ks][0] = *reinterpret_cast<const uint32_t*>(Qs + rl * QP + ks * 16 + 2 * tq);
    qa[ks][1] = *reinterpret_cast<const uint32_t*>(Qs + rh * QP + ks * 16 + 2 * tq);
    qa[ks][2] = *reinterpret_cast<const uint32_t*>(Qs + rl * QP + ks * 16 + 8 + 2 * tq);
    qa[ks][3] = *reinterpret_cast<const uint32_t*>(Qs + rh * QP + ks * 16 + 8 + 2 * tq);
  }
  const int lim_l = r0 + rl < rows ? ctx + (r0 + rl) / gsz : -1;  // last visible key of the lane's two rows
  const int lim_h = r0 + rh < rows ? ctx + (r0 + rh) / gsz : -1;
  const int wrow_last = min(rows - 1, r0 + warp * 16 + 15);
  const int wlim = r0 + warp * 16 < rows ? ctx + wrow_last / gsz : -1;
  const int kmax = ctx + (min(rows, r0 + 64) - 1) / gsz;
  float oacc[NV][4];
#pragma unroll
  for (int i = 0; i < NV; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;
  float m_l = -INFINITY, m_h = -INFINITY, l_l = 0.f, l_h = 0.f;
  const float inv_cap = softcap > 0.f ? 1.0f / softcap : 0.f;
  const int* pt = page_table + (long long)e * max_pages;
  const long long krow = (long long)G * DIM, vrow = (long long)G * VDIM;
  for (int k0 = 0; k0 <= kmax; k0 += 64) {
    __syncthreads();
    for (int id = threadIdx.x; id < 64 * (DIM / 8); id += 128) {
      const int r = id / (DIM / 8), cc = id % (DIM / 8), j = k0 + r;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (j <= kmax) v = *reinterpret_cast<const uint4*>(k_pages + ((long long)pt[j / page] * page + j % page) * krow + (long long)g * DIM + cc * 8);
      *reinterpret_cast<uint4*>(Ks + r * QP + cc * 8) = v;
    }
    for (int id = threadIdx.x; id < 64 * (VDIM / 8); id += 128) {
      const int r = id % 64, cc = id / 64, j = k0 + r;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (j <= kmax) v = *reinterpret_cast<const uint4*>(v_pages + ((long long)pt[j / page] * page + j % page) * vrow + (long long)g * VDIM + cc * 8);
      const bf16* pv = reinterpret_cast<const bf16*>(&v);
#pragma unroll
      for (int x = 0; x < 8; ++x) Vt[(cc * 8 + x) * VP + r] = pv[x];
    }
    __syncthreads();
    if (k0 > wlim) continue;
    float sacc[8][4];
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
      sacc[nb][0] = sacc[nb][1] = sacc[nb][2] = sacc[nb][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(Ks + (nb * 8 + gq) * QP + ks * 16 + 2 * tq);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(Ks + (nb * 8 + gq) * QP + ks * 16 + 8 + 2 * tq);
        mma16816(sacc[nb], qa[ks], b0, b1);
      }
    }
    // scores -> probabilities (fp32), running max / sum per row; the four lanes of a quad share a row
    float mx_l = -INFINITY, mx_h = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < 8; ++nb)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float sc = sacc[nb][c] * scale;
        if (softcap > 0.f) sc = softcap * tanh32(sc * inv_cap);
        sc *= 1.4426950408889634f;  // base-2 exponentials below
        const int key = k0 + nb * 8 + 2 * tq + (c & 1);
        const bool vis = key <= ((c & 2) ? lim_h : lim_l);
        sc = vis ? sc : -INFINITY;
        sacc[nb][c] = sc;
        if (c & 2) mx_h = fmaxf(mx_h, sc); else mx_l = fmaxf(mx_l, sc);
      }
    mx_l = fmaxf(mx_l, __shfl_xor_sync(0xffffffffu, mx_l, 1)); mx_l = fmaxf(mx_l, __shfl_xor_sync(0xffffffffu, mx_l, 2));
    mx_h = fmaxf(mx_h, __shfl_xor_sync(0xffffffffu, mx_h, 1)); mx_h = fmaxf(mx_h, __shfl_xor_sync(0xffffffffu, mx_h, 2));
    const float mn_l = fmaxf(m_l, mx_l), mn_h = fmaxf(m_h, mx_h);
    const float ml_safe = mn_l > -INFINITY ? mn_l : 0.f, mh_safe = mn_h > -INFINITY ? mn_h : 0.f;  // rows that see no key yet
    const float corr_l = exp2f(m_l - ml_safe), corr_h = exp2f(m_h - mh_safe);
    float sum_l = 0.f, sum_h = 0.f;
#pragma unroll
    for (int nb = 0; nb < 8; ++nb)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float p = exp2f(sacc[nb][c] - ((c & 2) ? mh_safe : ml_safe));  // exp2(-inf) = 0 for masked keys
        sacc[nb][c] = p;
        if (c & 2) sum_h += p; else sum_l += p;
      }
    l_l = l_l * corr_l + sum_l;  // per-lane partial sums; the quad is added up at the end
    l_h = l_h * corr_h + sum_h;
    m_l = mn_l;
    m_h = mn_h;
#pragma unroll
    for (int nv = 0; nv < NV; ++nv) {
      oacc[nv][0] *= corr_l; oacc[nv][1] *= corr_l; oacc[nv][2] *= corr_h; oacc[nv][3] *= corr_h;
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t a1[4], a2[4], a3[4];
      split3(sacc[2 * kk][0], sacc[2 * kk][1], a1[0], a2[0], a3[0]);
      split3(sacc[2 * kk][2], sacc[2 * kk][3], a1[1], a2[1], a3[1]);
      split3(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1], a1[2], a2[2], a3[2]);
      split3(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3], a1[3], a2[3], a3[3]);
#pragma unroll
      for (int nv = 0; nv < NV; ++nv) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(Vt + (nv * 8 + gq) * VP + kk * 16 + 2 * tq);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(Vt + (nv * 8 + gq) * VP + kk * 16 + 8 + 2 * tq);
        mma16816(oacc[nv], a1, b0, b1);
        mma16816(oacc[nv], a2, b0, b1);
        mma16816(oacc[nv], a3, b0, b1);
      }
    }
  }
  l_l += __shfl_xor_sync(0xffffffffu, l_l, 1); l_l += __shfl_xor_sync(0xffffffffu, l_l, 2);
  l_h += __shfl_xor_sync(0xffffffffu, l_h, 1); l_h += __shfl_xor_sync(0xffffffffu, l_h, 2);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int rr = r0 + (half ? rh : rl);
    if (rr >= rows) continue;
    const long long t = row0 + rr / gsz;
    const int head = g * gsz + rr % gsz;
    const float inv = 1.0f / (half ? l_h : l_l);
#pragma unroll
    for (int nv = 0; nv < NV; ++nv) {
      const int col = nv * 8 + 2 * tq;
      float v0 = oacc[nv][2 * half] * inv, v1 = oacc[nv][2 * half + 1] * inv;
      if (gate != nullptr) {
        float2 gg;
        if (gate_per_head) gg.x = gg.y = __bfloat162float(gate[t * ldg + head]);  // one scalar gate per head
        else gg = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gate + t * ldg + (long long)head * VDIM + col));
        v0 *= 1.0f / (1.0f + expf(-gg.x));
        v1 *= 1.0f / (1.0f + expf(-gg.y));
      }
      *reinterpret_cast<__nv_bfloat162*>(out + t * ((long long)H * VDIM) + (long long)head * VDIM + col) = __floats2bfloat162_rn(v0, v1);
    }
  }
}

template <int DIM, int VDIM>
int launch(const void* q, const void* kp, const void* vp, const void* gate, long long ldg, void* out, const int* row0, const int* n, const int* ctx,
           const int* pt, int max_pages, int page, int entries, int max_n, int H, int G, float scale, float softcap, int skip_single, int gate_per_head, cudaStream_t st) {
  const size_t smem = ((size_t)2 * 64 * (DIM + 8) + (size_t)VDIM * 72) * sizeof(bf16);
  auto kern = attn_ragged_mma_kernel<DIM, VDIM>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return PG_ERR_CUDA;
  dim3 grid((max_n * (H / G) + 63) / 64, G, entries);
  kern<<<grid, 128, smem, st>>>(static_cast<const bf16*>(q), static_cast<const bf16*>(kp), static_cast<const bf16*>(vp), static_cast<const bf16*>(gate), ldg,
                                static_cast<bf16*>(out), row0, n, ctx, pt, max_pages, page, H, G, scale, softcap, skip_single, gate_per_head);
  pg_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? PG_OK : PG_ERR_CUDA;
}

}  // namespace

extern "C" int pg_attn_ragged_mma(const void* q, const void* k_pages, const void* v_pages, const void* gate, long long ldg, void* out,
                                  const int* entry_row0, const int* entry_n, const int* entry_ctx, const int* page_table, int max_pages, int page,
                                  int entries, int max_n, int H, int G, int dim, int vdim, float scale, float softcap, int skip_single, int gate_per_head,
                                  void* stream) {
  if (entries <= 0 || max_n <= 0 || H <= 0 || G <= 0 || (H % G) != 0 || entries > 65535 || G > 65535) return PG_ERR_ARG;
  // 16-byte row loads and bf16x2 gate / output accesses
  if (((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_pages) | reinterpret_cast<uintptr_t>(v_pages) | reinterpret_cast<uintptr_t>(out)) & 15) ||
      (gate != nullptr && !gate_per_head && ((reinterpret_cast<uintptr_t>(gate) & 3) || (ldg & 1))))
    return PG_ERR_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define PG_MMA(D, V) \
  if (dim == D && vdim == V) \
    return launch<D, V>(q, k_pages, v_pages, gate, ldg, out, entry_row0, entry_n, entry_ctx, page_table, max_pages, page, entries, max_n, H, G, scale, \
                        softcap, skip_single, gate_per_head, st)
  PG_MMA(32, 32);
  PG_MMA(96, 64);    // explicit-head form of latent attention: [plain | rotated] keys
  PG_MMA(192, 128);
  PG_MMA(64, 64);
  PG_MMA(128, 128);
  PG_MMA(64, 128);
  PG_MMA(128, 64);
#undef PG_MMA
  return PG_ERR_ARG;  // other head sizes: pg_attn_ragged
}
