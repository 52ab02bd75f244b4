// HBM-bound kernels around the projection GEMMs and the attention (bf16 tensors, fp32 arithmetic):
//
//   add_layernorm_fwd / _bwd   s = a x + b r, y = LayerNorm(s) gamma + beta  — the residual-and-norm glue of the Pre-LN layer
//                              (a = b = 1; modules.py:179-195 of the reference) and of the muS layer (a = sqrt(1 - tau),
//                              b = sqrt(tau); mu_scaling/layer.py:259-280); without gamma it is the scaled residual add alone.
//   gelu_bwd_colsum            dz = dy * gelu'(z) and the bias gradient sum_rows(dz) in the same pass; without z the column
//                              sum of dy alone (bias gradient of a plain projection).
//   qkv_grad_pack              gradients of the head-major q, k, v (B,H,T,D) -> one row-major [T*B][3E] matrix for the
//                              dgrad / wgrad products: un-rotates dq and dk of the self pathway (transpose of the RoPE
//                              rotation) and applies the q scale.
//
// Every kernel reads each input once and writes each output once, 16 bytes per thread and access, rows walked by whole warps.
#include <cuda_fp8.h>

#include "common.cuh"

namespace mintb {
namespace {

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

__device__ __forceinline__ uint2 pack8_e4m3(const float (&f)[8], float inv) {
  uint2 u;
  __nv_fp8x2_storage_t* h = reinterpret_cast<__nv_fp8x2_storage_t*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __nv_cvt_float2_to_fp8x2(make_float2(f[2 * i] * inv, f[2 * i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
  return u;
}

// eight values -> e5m2 (saturating at +-57344) after multiplication by inv; `f` is overwritten with the values the
// 8-bit numbers stand for, times `scale` (an e5m2 number is the upper byte of the fp16 number with the same value)
__device__ __forceinline__ uint2 pack8_e5m2_roundtrip(float (&f)[8], float inv, float scale) {
  uint2 u;
  __nv_fp8x2_storage_t* h = reinterpret_cast<__nv_fp8x2_storage_t*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    h[i] = __nv_cvt_float2_to_fp8x2(make_float2(f[2 * i] * inv, f[2 * i + 1] * inv), __NV_SATFINITE, __NV_E5M2);
    const unsigned short lo = static_cast<unsigned short>((h[i] & 0xffu) << 8), hi = static_cast<unsigned short>(h[i] & 0xff00u);
    f[2 * i] = __half2float(__ushort_as_half(lo)) * scale;
    f[2 * i + 1] = __half2float(__ushort_as_half(hi)) * scale;
  }
  return u;
}

__device__ __forceinline__ float ld_param(const void* p, int dtype, int i) {
  return dtype == MINTB_F32 ? static_cast<const float*>(p)[i] : __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}

constexpr int kLnWarps = 4;
constexpr int kLnMaxE = 2560;   // widest row the LayerNorm kernels take

struct LnParams {
  const __nv_bfloat16 *x, *r;       // r may be null (then s = a x)
  float a, b;
  const void *gamma, *beta;         // null: no normalisation, only s
  int param_dtype;                  // MINTB_F32 or MINTB_BF16
  __nv_bfloat16 *s_out, *y_out;     // either may be null
  __nv_fp8_storage_t* q_out;        // e4m3 copy of the main result (y with gamma, else s), sat(value * q_inv); may be null
  float q_inv;
  float2* stats;                    // [rows] (mean, rstd); written by forward, read by backward
  const __nv_bfloat16 *dy, *ds_in;  // backward inputs (either may be null)
  __nv_bfloat16 *dx, *dr;           // backward outputs (dr may be null)
  float* partial;                   // backward: [gridDim.x][2][E] sums of dy * xhat and of dy
  int rows, E;
  float eps;
};

// MAXV: 16-byte vectors per lane (E <= MAXV * 256)
template <int MAXV>
__global__ void __launch_bounds__(kLnWarps * 32) add_layernorm_fwd_kernel(LnParams p) {
  __shared__ __align__(16) float s_gamma[kLnMaxE], s_beta[kLnMaxE];   // the parameters as fp32, read back 16 bytes at a time
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int nvec = p.E / 8;
  const float inv_e = 1.f / float(p.E);
  if (p.gamma != nullptr) {
    for (int i = threadIdx.x; i < p.E; i += kLnWarps * 32) {
      s_gamma[i] = ld_param(p.gamma, p.param_dtype, i);
      s_beta[i] = p.beta != nullptr ? ld_param(p.beta, p.param_dtype, i) : 0.f;
    }
    __syncthreads();
  }
  for (int row = blockIdx.x * kLnWarps + warp; row < p.rows; row += gridDim.x * kLnWarps) {
    const uint4* xr = reinterpret_cast<const uint4*>(p.x + size_t(row) * p.E);
    const uint4* rr = p.r != nullptr ? reinterpret_cast<const uint4*>(p.r + size_t(row) * p.E) : nullptr;
    // every load of the row is issued before the first use (a store between two loads would order them)
    uint4 xq[MAXV], rq[MAXV];
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int vi = lane + 32 * k;
      xq[k] = rq[k] = make_uint4(0u, 0u, 0u, 0u);
      if (vi < nvec) {
        xq[k] = __ldg(xr + vi);
        if (rr != nullptr) rq[k] = __ldg(rr + vi);
      }
    }
    float v[MAXV][8];
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      float xv[8], rv[8];
      unpack8(xq[k], xv);
      unpack8(rq[k], rv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[k][j] = rr != nullptr ? fmaf(p.a, xv[j], p.b * rv[j]) : p.a * xv[j];
        sum += v[k][j];
      }
    }
    if (p.s_out != nullptr) {
#pragma unroll
      for (int k = 0; k < MAXV; ++k) {
        const int vi = lane + 32 * k;
        if (vi < nvec) {
          const uint4 packed = pack8(v[k]);
          reinterpret_cast<uint4*>(p.s_out + size_t(row) * p.E)[vi] = packed;
          if (p.q_out != nullptr && p.gamma == nullptr) {   // the e4m3 copy is taken from the rounded bf16 values
            float rb[8];
            unpack8(packed, rb);
            reinterpret_cast<uint2*>(p.q_out + size_t(row) * p.E)[vi] = pack8_e4m3(rb, p.q_inv);
          }
        }
      }
    }
    if (p.gamma == nullptr) continue;
    const float mean = warp_sum_f(sum) * inv_e;
    float sq = 0.f;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      if (lane + 32 * k < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d = v[k][j] - mean;
          sq = fmaf(d, d, sq);
        }
      }
    }
    const float rstd = rsqrtf(warp_sum_f(sq) * inv_e + p.eps);
    if (lane == 0 && p.stats != nullptr) p.stats[row] = make_float2(mean, rstd);
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int vi = lane + 32 * k;
      if (vi < nvec) {
        float o[8], gm[8], bt[8];
        *reinterpret_cast<float4*>(gm) = *reinterpret_cast<const float4*>(s_gamma + vi * 8);
        *reinterpret_cast<float4*>(gm + 4) = *reinterpret_cast<const float4*>(s_gamma + vi * 8 + 4);
        *reinterpret_cast<float4*>(bt) = *reinterpret_cast<const float4*>(s_beta + vi * 8);
        *reinterpret_cast<float4*>(bt + 4) = *reinterpret_cast<const float4*>(s_beta + vi * 8 + 4);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = fmaf((v[k][j] - mean) * rstd, gm[j], bt[j]);
        const uint4 packed = pack8(o);
        reinterpret_cast<uint4*>(p.y_out + size_t(row) * p.E)[vi] = packed;
        if (p.q_out != nullptr) {
          float rb[8];
          unpack8(packed, rb);
          reinterpret_cast<uint2*>(p.q_out + size_t(row) * p.E)[vi] = pack8_e4m3(rb, p.q_inv);
        }
      }
    }
  }
}

// ds = LayerNorm'(dy) + ds_in;  dx = a ds;  dr = b ds;  per-CTA partial sums for dgamma / dbeta.
// LayerNorm backward per row: g = dy gamma, xhat = (s - mean) rstd, ds = rstd (g - mean(g) - xhat mean(g xhat)).
//
// A CTA spans one row: thread i owns the 8 columns of 16-byte vector i for every row the CTA walks, so its share of
// dgamma / dbeta stays in 16 registers and no thread ever adds into another thread's columns.  kLnBwdRows rows are in
// flight at a time (up to 16 loads of 16 bytes per thread before the first use); their 2 x kLnBwdRows row sums are reduced
// by warp shuffles, then across the warps through a double-buffered shared-memory slot with ONE barrier per batch of rows.
#ifndef MINTB_LN_BWD_ROWS
#define MINTB_LN_BWD_ROWS 4
#endif
#ifndef MINTB_LN_BWD_PER_SM
#define MINTB_LN_BWD_PER_SM 3
#endif
constexpr int kLnBwdRows = MINTB_LN_BWD_ROWS;
static_assert(kLnBwdRows % 2 == 0, "row sums travel as float4");
constexpr int kLnBwdMaxWarps = kLnMaxE / 8 / 32;   // 10

// NW: warps per CTA (E <= NW * 256); MINB: CTAs per SM the register budget is cut for.
template <int NW, int MINB>
__global__ void __launch_bounds__(NW * 32, MINB) add_layernorm_bwd_kernel(LnParams p) {
  __shared__ __align__(16) float red[2][NW][2 * kLnBwdRows];
  const int vi = threadIdx.x, warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int nvec = p.E / 8;
  constexpr int nwarps = NW;
  const bool live = vi < nvec;
  const bool norm = p.gamma != nullptr;
  const float inv_e = 1.f / float(p.E);
  float gm[8], rg[8], rb[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    gm[j] = (norm && live) ? ld_param(p.gamma, p.param_dtype, vi * 8 + j) : 0.f;
    rg[j] = rb[j] = 0.f;
  }
  int parity = 0;
  for (int row0 = blockIdx.x * kLnBwdRows; row0 < p.rows; row0 += gridDim.x * kLnBwdRows, parity ^= 1) {
    uint4 xq[kLnBwdRows], dq[kLnBwdRows], rq[kLnBwdRows];
    float2 st[kLnBwdRows];
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int r = 0; r < kLnBwdRows; ++r) {
      const int row = row0 + r;
      const bool ok = live && row < p.rows;
      const size_t off = size_t(row) * p.E;
      xq[r] = dq[r] = rq[r] = zero4;
      st[r] = make_float2(0.f, 0.f);
      if (ok && norm) {
        xq[r] = __ldg(reinterpret_cast<const uint4*>(p.x + off) + vi);
        dq[r] = __ldg(reinterpret_cast<const uint4*>(p.dy + off) + vi);
        if (p.r != nullptr) rq[r] = __ldg(reinterpret_cast<const uint4*>(p.r + off) + vi);
        st[r] = __ldg(p.stats + row);
      }
    }
    float c[2 * kLnBwdRows];
    if (norm) {
#pragma unroll
      for (int r = 0; r < kLnBwdRows; ++r) {
        float xv[8], dyv[8], rv[8];
        unpack8(xq[r], xv);
        unpack8(dq[r], dyv);
        unpack8(rq[r], rv);
        float c1 = 0.f, c2 = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xhat = (fmaf(p.a, xv[j], p.b * rv[j]) - st[r].x) * st[r].y;   // rows past the end: all zeros
          const float g = dyv[j] * gm[j];
          c1 += g;
          c2 = fmaf(g, xhat, c2);
          rg[j] = fmaf(dyv[j], xhat, rg[j]);
          rb[j] += dyv[j];
        }
        c[2 * r] = warp_sum_f(c1);
        c[2 * r + 1] = warp_sum_f(c2);
      }
      if (lane == 0) {
#pragma unroll
        for (int i = 0; i < 2 * kLnBwdRows; i += 4)
          *reinterpret_cast<float4*>(&red[parity][warp][i]) = make_float4(c[i], c[i + 1], c[i + 2], c[i + 3]);
      }
      __syncthreads();   // the slot of the other parity is free again once every thread is past this barrier
#pragma unroll
      for (int i = 0; i < 2 * kLnBwdRows; ++i) c[i] = 0.f;
#pragma unroll
      for (int w = 0; w < nwarps; ++w) {   // same order in every thread: all of them hold identical sums
#pragma unroll
        for (int i = 0; i < 2 * kLnBwdRows; i += 4) {
          const float4 t = *reinterpret_cast<const float4*>(&red[parity][w][i]);
          c[i] += t.x; c[i + 1] += t.y; c[i + 2] += t.z; c[i + 3] += t.w;
        }
      }
    }
    // The second pass unpacks the rows again instead of keeping 2 x 8 x kLnBwdRows fp32 values alive across the barrier;
    // the empty statements stop the compiler from undoing that.
#pragma unroll
    for (int r = 0; r < kLnBwdRows; ++r) {
      asm volatile("" : "+r"(xq[r].x), "+r"(xq[r].y), "+r"(xq[r].z), "+r"(xq[r].w));
      asm volatile("" : "+r"(dq[r].x), "+r"(dq[r].y), "+r"(dq[r].z), "+r"(dq[r].w));
      asm volatile("" : "+r"(rq[r].x), "+r"(rq[r].y), "+r"(rq[r].z), "+r"(rq[r].w));
    }
    uint4 eq[kLnBwdRows];   // the gradient that reaches s directly (the residual branch of a Pre-LN layer), or zeros
#pragma unroll
    for (int r = 0; r < kLnBwdRows; ++r)
      eq[r] = (p.ds_in != nullptr && live && row0 + r < p.rows)
                  ? __ldg(reinterpret_cast<const uint4*>(p.ds_in + size_t(row0 + r) * p.E) + vi) : zero4;
#pragma unroll
    for (int r = 0; r < kLnBwdRows; ++r) {
      const int row = row0 + r;
      if (!(live && row < p.rows)) continue;
      const size_t off = size_t(row) * p.E;
      float ds[8];
      unpack8(eq[r], ds);
      if (norm) {
        float xv[8], dyv[8], rv[8];
        unpack8(xq[r], xv);
        unpack8(dq[r], dyv);
        unpack8(rq[r], rv);
        const float c1 = c[2 * r] * inv_e, c2 = c[2 * r + 1] * inv_e;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xhat = (fmaf(p.a, xv[j], p.b * rv[j]) - st[r].x) * st[r].y;
          ds[j] += st[r].y * (dyv[j] * gm[j] - c1 - xhat * c2);
        }
      }
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = p.a * ds[j];
      reinterpret_cast<uint4*>(p.dx + off)[vi] = pack8(o);
      if (p.dr != nullptr) {
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = p.b * ds[j];
        reinterpret_cast<uint4*>(p.dr + off)[vi] = pack8(o);
      }
    }
  }
  if (norm && live && p.partial != nullptr) {
    float* dst = p.partial + size_t(blockIdx.x) * 2 * p.E + vi * 8;
    *reinterpret_cast<float4*>(dst) = make_float4(rg[0], rg[1], rg[2], rg[3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(rg[4], rg[5], rg[6], rg[7]);
    *reinterpret_cast<float4*>(dst + p.E) = make_float4(rb[0], rb[1], rb[2], rb[3]);
    *reinterpret_cast<float4*>(dst + p.E + 4) = make_float4(rb[4], rb[5], rb[6], rb[7]);
  }
}

// dgamma[e] = sum over CTAs of partial[c][0][e], dbeta likewise; fixed order.  CTA = 32 columns x 8 row lanes: each lane
// adds every 8th partial, the 8 sums meet in shared memory.
__global__ void __launch_bounds__(256) ln_param_grad_kernel(const float* __restrict__ partial, int n_parts, int E, float* __restrict__ dgamma,
                                                            float* __restrict__ dbeta) {
  __shared__ float red[8][33];
  const int cl = threadIdx.x % 32, rl = threadIdx.x / 32;
  const int i = blockIdx.x * 32 + cl;
  float t = 0.f;
  if (i < 2 * E)
    for (int c = rl; c < n_parts; c += 8) t += partial[size_t(c) * 2 * E + i];
  red[rl][cl] = t;
  __syncthreads();
  if (rl == 0 && i < 2 * E) {
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) sum += red[k][cl];
    if (i < E) dgamma[i] = sum; else dbeta[i - E] = sum;
  }
}

// ------------------------------------------------------------------------------------------------ GELU backward + column sums
constexpr int kColRows = 256;   // rows per CTA strip of the gradient pack
constexpr int kSumRows = 64;    // rows per CTA strip of the column sums: every thread has its 8 rows in flight at once, and
                                // the grid is many waves deep (a 256-row strip left 1.6 to 2.2 waves at 32768 rows)
constexpr int kColLanes = 8;    // threads that share a column group, each taking every 8th row of the strip

// d/dz [z/2 (1 + erf(z / sqrt 2))] = (1 + erf(z / sqrt 2)) / 2 + z exp(-z^2 / 2) / sqrt(2 pi).  erf comes from the
// rational-exponential form 1 - (a1 t + ... + a5 t^5) exp(-u^2), t = 1 / (1 + p u), u = |z| / sqrt 2 (absolute error below
// 1.5e-7), which needs the very exponential the second term needs: one exp2 and one reciprocal per element.
__device__ __forceinline__ float gelu_erf_grad(float z) {
  const float u = fabsf(z) * 0.70710678118654752f;
  float t, e;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f, u, 1.f)));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-0.72134752044448170f * z * z));   // exp(-z^2 / 2)
  float poly = fmaf(1.061405429f, t, -1.453152027f);
  poly = fmaf(poly, t, 1.421413741f);
  poly = fmaf(poly, t, -0.284496736f);
  poly = fmaf(poly, t, 0.254829592f);
  const float erf_abs = fmaf(-poly * t, e, 1.f);                   // erf(|z| / sqrt 2)
  const float cdf = 0.5f + copysignf(0.5f * erf_abs, z);
  return fmaf(z * 0.3989422804014327f, e, cdf);
}

// the same with gelu(z) = z cdf(z) as a second result
__device__ __forceinline__ float gelu_erf_grad_val(float z, float& val) {
  const float u = fabsf(z) * 0.70710678118654752f;
  float t, e;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f, u, 1.f)));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-0.72134752044448170f * z * z));
  float poly = fmaf(1.061405429f, t, -1.453152027f);
  poly = fmaf(poly, t, 1.421413741f);
  poly = fmaf(poly, t, -0.284496736f);
  poly = fmaf(poly, t, 0.254829592f);
  const float erf_abs = fmaf(-poly * t, e, 1.f);
  const float cdf = 0.5f + copysignf(0.5f * erf_abs, z);
  val = z * cdf;
  return fmaf(z * 0.3989422804014327f, e, cdf);
}

// CTA = 32 column groups (8 columns each: 256 columns) x 8 row lanes over a strip of kSumRows rows; a warp reads 512
// contiguous bytes of one row.  A thread issues the loads of all its rows of the strip (in two halves when z is read as
// well) before it touches the first value.  The 8 partial column sums meet in shared memory; db gets one atomicAdd per
// column and CTA.
template <bool HAS_Z>
__global__ void __launch_bounds__(256) gelu_bwd_colsum_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ z,
                                                              __nv_bfloat16* __restrict__ dz, float* __restrict__ db, int M, int N,
                                                              __nv_bfloat16* __restrict__ act, __nv_fp8_storage_t* __restrict__ q8,
                                                              float q_inv, float q_scale) {
  __shared__ float part[kColLanes][32][8];
  const int cl = threadIdx.x % 32, rl = threadIdx.x / 32;
  const int cg = blockIdx.x * 32 + cl;   // column group
  const bool live = cg * 8 < N;
  const int m0 = blockIdx.y * kSumRows;
  constexpr int kPerThread = kSumRows / kColLanes;        // 8 rows of the strip per thread
  constexpr int kBatch = HAS_Z ? kPerThread / 2 : kPerThread;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (live) {
#pragma unroll
    for (int h = 0; h < kPerThread / kBatch; ++h) {
      uint4 gq[kBatch], zq[HAS_Z ? kBatch : 1];
#pragma unroll
      for (int i = 0; i < kBatch; ++i) {
        const int m = m0 + rl + (h * kBatch + i) * kColLanes;
        const size_t off = size_t(m) * N + size_t(cg) * 8;
        gq[i] = make_uint4(0u, 0u, 0u, 0u);
        if (HAS_Z) zq[i] = gq[i];
        if (m < M) {
          gq[i] = __ldg(reinterpret_cast<const uint4*>(dy + off));
          if (HAS_Z) zq[i] = __ldg(reinterpret_cast<const uint4*>(z + off));
        }
      }
#pragma unroll
      for (int i = 0; i < kBatch; ++i) {
        const int m = m0 + rl + (h * kBatch + i) * kColLanes;
        float g[8];
        unpack8(gq[i], g);
        if (HAS_Z) {
          float zv[8];
          unpack8(zq[i], zv);
          if (act != nullptr) {   // gelu(z) itself as well: the activation the next product's weight gradient needs
            float a[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) g[j] *= gelu_erf_grad_val(zv[j], a[j]);
            if (m < M) *reinterpret_cast<uint4*>(act + size_t(m) * N + size_t(cg) * 8) = pack8(a);
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) g[j] *= gelu_erf_grad(zv[j]);
          }
          if (dz != nullptr) {
            const uint4 packed = pack8(g);
            if (m < M) *reinterpret_cast<uint4*>(dz + size_t(m) * N + size_t(cg) * 8) = packed;
            if (q8 == nullptr) unpack8(packed, g);   // the bias gradient sums what the products will read
          }
        }
        if (q8 != nullptr) {   // the e5m2 operand of the 8-bit dgrad / wgrad products; the bias gradient sums these very numbers
          const uint2 pk = pack8_e5m2_roundtrip(g, q_inv, q_scale);
          if (m < M) *reinterpret_cast<uint2*>(q8 + size_t(m) * N + size_t(cg) * 8) = pk;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += g[j];   // rows past the end hold zeros
      }
    }
  }
  if (db == nullptr) return;
#pragma unroll
  for (int j = 0; j < 8; ++j) part[rl][cl][j] = acc[j];
  __syncthreads();
  // 256 threads <-> 256 columns of the CTA
  const int c = threadIdx.x;
  const int col = blockIdx.x * 256 + c;
  if (col < N) {
    float t = 0.f;
#pragma unroll
    for (int r = 0; r < kColLanes; ++r) t += part[r][c / 8][c % 8];
    atomicAdd(db + col, t);
  }
}

// ------------------------------------------------------------------------------------------------ QKV gradient pack
// g[(t * B + b)][which * E + h * D + d] = f(dsrc[which][b][h][t][d]), f = q scale and the transposed rotation for dq, dk;
// db[col] = sum over rows of g (the bias gradient of the fused projection) in the same pass.
// CTA = 32 column groups (8 columns each: 256 columns of g) x 8 row lanes over a strip of kColRows rows; a thread's column
// group — pathway third, head, 8 dimensions — is fixed, only (t, b) changes from row to row.
template <int D>
__global__ void __launch_bounds__(256) qkv_grad_pack_kernel(const __nv_bfloat16* __restrict__ dq, const __nv_bfloat16* __restrict__ dk,
                                                            const __nv_bfloat16* __restrict__ dv, __nv_bfloat16* __restrict__ g,
                                                            float* __restrict__ db, const float* __restrict__ cos_tab,
                                                            const float* __restrict__ sin_tab, const int32_t* __restrict__ row_map,
                                                            int M, int T, int B, int H, float q_scale) {
  __shared__ float part[kColLanes][32][8];
  constexpr int VPH = D / 8, hd = D / 2;             // vectors per head; rotation pairs dimension d with d + hd
  const int E = H * D, N = 3 * E;
  const int cl = threadIdx.x % 32, rl = threadIdx.x / 32;
  const int cg = blockIdx.x * 32 + cl;               // column group
  const bool live = cg * 8 < N;
  const int col = live ? cg * 8 : 0;
  const int which = col / E, e = col % E, h = e / D, dv8 = (e % D) / 8;
  const __nv_bfloat16* src = which == 0 ? dq : (which == 1 ? dk : dv);
  const bool rot = cos_tab != nullptr && which < 2;
  const bool upper = dv8 * 8 >= hd;
  const int pv = upper ? dv8 - VPH / 2 : dv8 + VPH / 2;   // the vector holding the partner dimensions
  const int f0 = upper ? dv8 * 8 - hd : dv8 * 8;
  const float scale = which == 0 ? q_scale : 1.f;
  const int m0 = blockIdx.y * kColRows, m1 = min(M, m0 + kColRows);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (live) {
#pragma unroll 4
    for (int m = m0 + rl; m < m1; m += kColLanes) {
      const int mo = row_map != nullptr ? row_map[m] : m;   // packed rows: output row m is token mo = t * B + b
      const int t = mo / B, b = mo % B;
      const uint4* row = reinterpret_cast<const uint4*>(src + ((size_t(b) * H + h) * T + t) * D);
      float v[8];
      unpack8(__ldg(row + dv8), v);
      if (rot) {
        // y = R x rotated forward: y_lo = x_lo c - x_hi s, y_hi = x_hi c + x_lo s; the gradient takes the transpose:
        // dx_lo = dy_lo c + dy_hi s, dx_hi = dy_hi c - dy_lo s
        float o[8], c[8], sn[8];
        unpack8(__ldg(row + pv), o);
        const float4* c4 = reinterpret_cast<const float4*>(cos_tab + size_t(t) * hd + f0);
        const float4* s4 = reinterpret_cast<const float4*>(sin_tab + size_t(t) * hd + f0);
        *reinterpret_cast<float4*>(c) = __ldg(c4); *reinterpret_cast<float4*>(c + 4) = __ldg(c4 + 1);
        *reinterpret_cast<float4*>(sn) = __ldg(s4); *reinterpret_cast<float4*>(sn + 4) = __ldg(s4 + 1);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = upper ? v[j] * c[j] - o[j] * sn[j] : v[j] * c[j] + o[j] * sn[j];
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] *= scale;
      const uint4 packed = pack8(v);
      *reinterpret_cast<uint4*>(g + size_t(m) * N + col) = packed;
      unpack8(packed, v);   // the bias gradient sums what the products will read
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += v[j];
    }
  }
  if (db == nullptr) return;
#pragma unroll
  for (int j = 0; j < 8; ++j) part[rl][cl][j] = acc[j];
  __syncthreads();
  const int c = threadIdx.x;
  const int ocol = blockIdx.x * 256 + c;
  if (ocol < N) {
    float t = 0.f;
#pragma unroll
    for (int r = 0; r < kColLanes; ++r) t += part[r][c / 8][c % 8];
    atomicAdd(db + ocol, t);
  }
}

int fail(const char* what, cudaError_t e) {
  set_error("%s: %s", what, cudaGetErrorString(e));
  return MINTB_ECUDA;
}

int ln_maxv(int E) { return E <= 512 ? 2 : (E <= 1280 ? 5 : (E <= 2560 ? 10 : 0)); }

// Upper bound of the backward grid (sizes the partial-sum workspace); the launch takes min(this, 148 x resident CTAs per SM).
int ln_bwd_grid_max(int rows) {
  const int want = (rows + kLnBwdRows - 1) / kLnBwdRows;
  return want < 148 * 8 ? want : 148 * 8;
}

}  // namespace
}  // namespace mintb

extern "C" {

using namespace mintb;

int mintb_add_layernorm_fwd_q(const void* x, const void* r, float a, float b, const void* gamma, const void* beta, int param_dtype,
                              void* s_out, void* y_out, float* stats, int rows, int E, float eps, void* q_out, float q_inv_scale,
                              void* stream) {
  if (x == nullptr || rows <= 0 || E <= 0 || (E % 8) != 0 || ln_maxv(E) == 0) {
    set_error("mintb_add_layernorm_fwd: x is required, rows > 0, E a multiple of 8 and at most 2560 (got rows %d, E %d)", rows, E);
    return x == nullptr || rows <= 0 || E <= 0 ? MINTB_EINVAL : MINTB_EUNSUPPORTED;
  }
  if ((gamma != nullptr && y_out == nullptr) || (gamma == nullptr && s_out == nullptr) ||
      (param_dtype != MINTB_F32 && param_dtype != MINTB_BF16)) {
    set_error("mintb_add_layernorm_fwd: y_out is required with gamma, s_out without; parameters are f32 or bf16");
    return MINTB_EINVAL;
  }
  LnParams p{};
  p.x = static_cast<const __nv_bfloat16*>(x); p.r = static_cast<const __nv_bfloat16*>(r);
  p.a = a; p.b = b; p.gamma = gamma; p.beta = beta; p.param_dtype = param_dtype;
  p.s_out = static_cast<__nv_bfloat16*>(s_out); p.y_out = static_cast<__nv_bfloat16*>(y_out);
  p.stats = reinterpret_cast<float2*>(stats); p.rows = rows; p.E = E; p.eps = eps;
  p.q_out = static_cast<__nv_fp8_storage_t*>(q_out); p.q_inv = q_inv_scale;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int want = (rows + kLnWarps - 1) / kLnWarps;
  const int grid = want < 148 * 16 ? want : 148 * 16;   // rows are walked with a grid stride
  switch (ln_maxv(E)) {
    case 2: add_layernorm_fwd_kernel<2><<<grid, kLnWarps * 32, 0, st>>>(p); break;
    case 5: add_layernorm_fwd_kernel<5><<<grid, kLnWarps * 32, 0, st>>>(p); break;
    default: add_layernorm_fwd_kernel<10><<<grid, kLnWarps * 32, 0, st>>>(p); break;
  }
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? MINTB_OK : fail("mintb_add_layernorm_fwd launch", e);
}

int mintb_add_layernorm_fwd(const void* x, const void* r, float a, float b, const void* gamma, const void* beta, int param_dtype,
                            void* s_out, void* y_out, float* stats, int rows, int E, float eps, void* stream) {
  return mintb_add_layernorm_fwd_q(x, r, a, b, gamma, beta, param_dtype, s_out, y_out, stats, rows, E, eps, nullptr, 1.f, stream);
}

size_t mintb_add_layernorm_bwd_workspace_bytes(int rows, int E) {
  if (rows <= 0 || E <= 0) return 0;
  return align256(size_t(ln_bwd_grid_max(rows)) * 2 * E * sizeof(float));
}

int mintb_add_layernorm_bwd(const void* dy, const void* ds_in, const void* x, const void* r, float a, float b, const void* gamma,
                            int param_dtype, const float* stats, void* dx, void* dr, float* dgamma, float* dbeta, void* workspace,
                            size_t workspace_bytes, int rows, int E, void* stream) {
  if (rows <= 0 || E <= 0 || (E % 8) != 0 || ln_maxv(E) == 0) {
    set_error("mintb_add_layernorm_bwd: rows > 0, E a multiple of 8 and at most 2560 (got rows %d, E %d)", rows, E);
    return rows <= 0 || E <= 0 ? MINTB_EINVAL : MINTB_EUNSUPPORTED;
  }
  const bool norm = gamma != nullptr;
  if (dx == nullptr || (norm && (dy == nullptr || x == nullptr || stats == nullptr || (dgamma == nullptr) != (dbeta == nullptr))) ||
      (!norm && ds_in == nullptr)) {
    set_error("mintb_add_layernorm_bwd: missing pointer (with gamma: dy, x, stats, dgamma and dbeta or neither; without: ds_in; always dx)");
    return MINTB_EINVAL;
  }
  const bool param_grads = norm && dgamma != nullptr;   // frozen parameters: no partial sums, no second pass
  if (param_grads && (workspace == nullptr || workspace_bytes < mintb_add_layernorm_bwd_workspace_bytes(rows, E))) {
    set_error("mintb_add_layernorm_bwd: workspace of %zu bytes required", mintb_add_layernorm_bwd_workspace_bytes(rows, E));
    return MINTB_EWORKSPACE;
  }
  LnParams p{};
  p.x = static_cast<const __nv_bfloat16*>(x); p.r = static_cast<const __nv_bfloat16*>(r);
  p.a = a; p.b = b; p.gamma = gamma; p.param_dtype = param_dtype;
  p.stats = const_cast<float2*>(reinterpret_cast<const float2*>(stats));
  p.dy = static_cast<const __nv_bfloat16*>(dy); p.ds_in = static_cast<const __nv_bfloat16*>(ds_in);
  p.dx = static_cast<__nv_bfloat16*>(dx); p.dr = static_cast<__nv_bfloat16*>(dr);
  p.partial = param_grads ? static_cast<float*>(workspace) : nullptr; p.rows = rows; p.E = E;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // one 16-byte vector of the row per thread; ONE wave of CTAs, each walking its share of the rows
  const int nw = ln_maxv(E);   // 2, 5 or 10 warps
  const int per_sm = nw == 2 ? 8 : (nw == 5 ? MINTB_LN_BWD_PER_SM : 1);
  const int grid_max = ln_bwd_grid_max(rows);
  const int grid = grid_max < 148 * per_sm ? grid_max : 148 * per_sm;
  switch (nw) {
    case 2: add_layernorm_bwd_kernel<2, 8><<<grid, 64, 0, st>>>(p); break;
    case 5: add_layernorm_bwd_kernel<5, MINTB_LN_BWD_PER_SM><<<grid, 160, 0, st>>>(p); break;
    default: add_layernorm_bwd_kernel<10, 1><<<grid, 320, 0, st>>>(p); break;
  }
  cudaError_t e = cudaSuccess;
  if (e != cudaSuccess) return fail("mintb_add_layernorm_bwd", e);
  count_launches(1);
  if (param_grads) {
    ln_param_grad_kernel<<<(2 * E + 31) / 32, 256, 0, st>>>(p.partial, grid, E, dgamma, dbeta);
    count_launches(1);
  }
  e = cudaGetLastError();
  return e == cudaSuccess ? MINTB_OK : fail("mintb_add_layernorm_bwd launch", e);
}

int mintb_gelu_bwd_colsum_f8(const void* dy, const void* z, void* dz, void* act, float* db, void* dz_e5m2, float e5m2_scale, int M,
                             int N, void* stream) {
  if (dy == nullptr || M <= 0 || N <= 0 || (N % 8) != 0 || (z != nullptr && dz == nullptr && dz_e5m2 == nullptr) ||
      (z == nullptr && db == nullptr && dz_e5m2 == nullptr) || (z == nullptr && act != nullptr) || (dz_e5m2 != nullptr && !(e5m2_scale > 0.f))) {
    set_error("mintb_gelu_bwd_colsum: dy required, N a multiple of 8, a result to write (dz / dz_e5m2 with z, db / dz_e5m2 without), "
              "act only with z, a positive e5m2_scale with dz_e5m2");
    return MINTB_EINVAL;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (db != nullptr) {
    cudaError_t e = cudaMemsetAsync(db, 0, size_t(N) * sizeof(float), st);
    if (e != cudaSuccess) return fail("mintb_gelu_bwd_colsum memset", e);
  }
  dim3 grid((N + 255) / 256, (M + kSumRows - 1) / kSumRows);
  __nv_fp8_storage_t* q8 = static_cast<__nv_fp8_storage_t*>(dz_e5m2);
  const float q_inv = q8 != nullptr ? 1.f / e5m2_scale : 1.f, q_scale = q8 != nullptr ? e5m2_scale : 1.f;
  if (z != nullptr)
    gelu_bwd_colsum_kernel<true><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(z),
                                                       static_cast<__nv_bfloat16*>(dz), db, M, N, static_cast<__nv_bfloat16*>(act), q8,
                                                       q_inv, q_scale);
  else
    gelu_bwd_colsum_kernel<false><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(dy), nullptr, nullptr, db, M, N, nullptr, q8,
                                                        q_inv, q_scale);
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? MINTB_OK : fail("mintb_gelu_bwd_colsum launch", e);
}

int mintb_gelu_bwd_colsum_act(const void* dy, const void* z, void* dz, void* act, float* db, int M, int N, void* stream) {
  if ((z != nullptr && dz == nullptr) || (z == nullptr && db == nullptr)) {
    set_error("mintb_gelu_bwd_colsum: dy required, N a multiple of 8, dz with z, db without z, act only with z");
    return MINTB_EINVAL;
  }
  return mintb_gelu_bwd_colsum_f8(dy, z, dz, act, db, nullptr, 1.f, M, N, stream);
}

int mintb_gelu_bwd_colsum(const void* dy, const void* z, void* dz, float* db, int M, int N, void* stream) {
  return mintb_gelu_bwd_colsum_act(dy, z, dz, nullptr, db, M, N, stream);
}

int mintb_qkv_grad_pack(const void* dq, const void* dk, const void* dv, void* g, float* db, const float* rope_cos,
                        const float* rope_sin, const int32_t* row_map, int n_rows, int T, int B, int H, int D, float q_scale,
                        void* stream) {
  if (dq == nullptr || dk == nullptr || dv == nullptr || g == nullptr || T <= 0 || B <= 0 || H <= 0 ||
      (rope_cos == nullptr) != (rope_sin == nullptr)) {
    set_error("mintb_qkv_grad_pack: null pointer or non-positive size");
    return MINTB_EINVAL;
  }
  if (D != 16 && D != 32 && D != 64) {
    set_error("mintb_qkv_grad_pack: head_dim %d is not one of 16, 32, 64", D);
    return MINTB_EUNSUPPORTED;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int N = 3 * H * D, M = row_map != nullptr ? n_rows : T * B;
  if (M <= 0) {
    set_error("mintb_qkv_grad_pack: no rows");
    return MINTB_EINVAL;
  }
  if (db != nullptr) {
    cudaError_t e = cudaMemsetAsync(db, 0, size_t(N) * sizeof(float), st);
    if (e != cudaSuccess) return fail("mintb_qkv_grad_pack memset", e);
  }
  dim3 grid((N + 255) / 256, (M + kColRows - 1) / kColRows);
  const __nv_bfloat16 *q = static_cast<const __nv_bfloat16*>(dq), *k = static_cast<const __nv_bfloat16*>(dk),
                      *v = static_cast<const __nv_bfloat16*>(dv);
  __nv_bfloat16* o = static_cast<__nv_bfloat16*>(g);
  switch (D) {
    case 16: qkv_grad_pack_kernel<16><<<grid, 256, 0, st>>>(q, k, v, o, db, rope_cos, rope_sin, row_map, M, T, B, H, q_scale); break;
    case 32: qkv_grad_pack_kernel<32><<<grid, 256, 0, st>>>(q, k, v, o, db, rope_cos, rope_sin, row_map, M, T, B, H, q_scale); break;
    default: qkv_grad_pack_kernel<64><<<grid, 256, 0, st>>>(q, k, v, o, db, rope_cos, rope_sin, row_map, M, T, B, H, q_scale); break;
  }
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? MINTB_OK : fail("mintb_qkv_grad_pack launch", e);
}

}  // extern "C"
