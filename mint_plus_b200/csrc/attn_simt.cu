// fp32 CUDA-core kernels for the combined-softmax multimer attention (forward, dQ, dK/dV).
//
// They serve the fp32 configuration (bit-level agreement with the PyTorch path to ~1e-6) and head sizes the
// tensor-core kernels do not cover.  Every result is produced in a fixed order: no atomics.
//
// Work split: G = D/8 threads share one row (query row in forward and dQ, key row in dK/dV); each owns 8
// consecutive head dimensions of the row's vectors and accumulators, dot products are completed with
// xor-shuffles inside the group.  A block of 128 threads covers 128/G rows and walks the other sequence
// axis in tiles of 32 staged in shared memory (32 = one word of the packed mask).
#include "common.cuh"

namespace mintb {

constexpr int kSimtThreads = 128;
constexpr int kSimtTile = 32;

template <int G>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = G / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Loads row `t` of x[T][D] (head already selected) into dst[D] (shared), rotating it if cos/sin are given:
// y[d] = x[d] cos - x[d+h] sin (d < h), y[d] = x[d] cos + x[d-h] sin (d >= h)   (rotary_embedding.py:16-24).
template <typename T, int D>
__device__ __forceinline__ void stage_row(const T* __restrict__ x, int t, int Tlen, const float* cos_tab,
                                          const float* sin_tab, float* dst, int lane, int nlanes, size_t row_stride = D) {
  constexpr int h = D / 2;
  for (int d = lane; d < D; d += nlanes) {
    float v = 0.f;
    if (t < Tlen) {
      v = ld_f(x + size_t(t) * row_stride + d);
      if (cos_tab != nullptr) {
        int f = d < h ? d : d - h;
        float c = cos_tab[size_t(t) * h + f], s = sin_tab[size_t(t) * h + f];
        float partner = d < h ? -ld_f(x + size_t(t) * row_stride + d + h) : ld_f(x + size_t(t) * row_stride + d - h);
        v = v * c + partner * s;
      }
    }
    dst[d] = v;
  }
}

struct SimtParams {
  const void *q_s, *k_s, *v_s, *q_c, *k_c, *v_c;
  const uint32_t *bits, *bitsT, *kpad;
  const float *cos_tab, *sin_tab;
  void* out;
  float* lse;
  const void* d_out;
  void *dq_s, *dk_s, *dv_s, *dq_c, *dk_c, *dv_c;
  float* delta;  // [B][H][T]
  int B, H, T, TW;
  float scale;
  size_t o_row, o_bh;   // element strides of out and d_out: between queries, between (batch, head) pairs
  int sqrt_sm;  // square-root softmax: out = sum_j sqrt(p_j) v_j (mu_scaling/layer.py:162-163)
};

// ------------------------------------------------------------------------------------------------ forward
template <typename T, int D>
__global__ void __launch_bounds__(kSimtThreads) attn_fwd_simt_kernel(SimtParams p) {
  constexpr int G = D / 8, R = kSimtThreads / G, KT = kSimtTile;
  __shared__ __align__(16) float sq_s[R][D], sq_c[R][D];
  __shared__ __align__(16) float sk_s[KT][D], sk_c[KT][D], sv_s[KT][D], sv_c[KT][D];

  const int bh = blockIdx.y, b = bh / p.H;
  const int r = threadIdx.x / G, g = threadIdx.x % G;
  const int i = blockIdx.x * R + r;
  const size_t head = size_t(bh) * p.T * D;
  const T* q_s = static_cast<const T*>(p.q_s) + head;
  const T* k_s = static_cast<const T*>(p.k_s) + head;
  const T* v_s = static_cast<const T*>(p.v_s) + head;
  const T* q_c = static_cast<const T*>(p.q_c) + head;
  const T* k_c = static_cast<const T*>(p.k_c) + head;
  const T* v_c = static_cast<const T*>(p.v_c) + head;

  stage_row<T, D>(q_s, i, p.T, p.cos_tab, p.sin_tab, sq_s[r], g, G);
  stage_row<T, D>(q_c, i, p.T, nullptr, nullptr, sq_c[r], g, G);
  __syncwarp();
  float qs[8], qc[8], acc[8];
#pragma unroll
  for (int d = 0; d < 8; ++d) {
    qs[d] = sq_s[r][g * 8 + d];
    qc[d] = sq_c[r][g * 8 + d];
    acc[d] = 0.f;
  }
  const float c2 = p.scale * kLog2e;
  float m = -INFINITY, l = 0.f;
  const int irow = i < p.T ? i : p.T - 1;  // rows past T compute on a valid row and are not stored
  const uint32_t* mrow = p.bits + (size_t(b) * p.T + irow) * p.TW;

  for (int j0 = 0; j0 < p.T; j0 += KT) {
    const uint32_t valid = ~p.kpad[size_t(b) * p.TW + j0 / 32];
    if (valid == 0u) continue;  // block-uniform: every key of the tile is padded
    __syncthreads();
    for (int jj = threadIdx.x / 32; jj < KT; jj += kSimtThreads / 32) {
      const int lane = threadIdx.x % 32;
      stage_row<T, D>(k_s, j0 + jj, p.T, p.cos_tab, p.sin_tab, sk_s[jj], lane, 32);
      stage_row<T, D>(k_c, j0 + jj, p.T, nullptr, nullptr, sk_c[jj], lane, 32);
      stage_row<T, D>(v_s, j0 + jj, p.T, nullptr, nullptr, sv_s[jj], lane, 32);
      stage_row<T, D>(v_c, j0 + jj, p.T, nullptr, nullptr, sv_c[jj], lane, 32);
    }
    __syncthreads();
    const uint32_t cross = mrow[j0 / 32];
    float s[KT];
    float tmax = -INFINITY;
#pragma unroll
    for (int jj = 0; jj < KT; ++jj) {
      const bool x = (cross >> jj) & 1u;
      const float* kk = x ? &sk_c[jj][g * 8] : &sk_s[jj][g * 8];
      float part = 0.f;
#pragma unroll
      for (int d = 0; d < 8; ++d) part = fmaf(x ? qc[d] : qs[d], kk[d], part);
      part = group_sum<G>(part);
      s[jj] = ((valid >> jj) & 1u) ? part * c2 : -INFINITY;
      tmax = fmaxf(tmax, s[jj]);
    }
    const float m_new = fmaxf(m, tmax);  // tile has at least one valid key, so m_new is finite
    // square-root softmax accumulates sqrt(p) v: the terms are exp2((s - m) / 2), the row sum stays sum exp2(s - m)
    const float alpha = exp2f(m - m_new);
    const float alpha_acc = p.sqrt_sm ? exp2f(0.5f * (m - m_new)) : alpha;
    l *= alpha;
#pragma unroll
    for (int d = 0; d < 8; ++d) acc[d] *= alpha_acc;
#pragma unroll
    for (int jj = 0; jj < KT; ++jj) {
      float pj;
      if (p.sqrt_sm) {
        pj = exp2f(0.5f * (s[jj] - m_new));
        l = fmaf(pj, pj, l);
      } else {
        pj = exp2f(s[jj] - m_new);
        l += pj;
      }
      const float* vv = ((cross >> jj) & 1u) ? &sv_c[jj][g * 8] : &sv_s[jj][g * 8];
#pragma unroll
      for (int d = 0; d < 8; ++d) acc[d] = fmaf(pj, vv[d], acc[d]);
    }
    m = m_new;
  }
  if (i < p.T) {
    // A row whose keys are all padded gives 0/0 = NaN, as the softmax of an all -inf row does in PyTorch.
    const float inv = p.sqrt_sm ? rsqrtf(l) : 1.f / l;
    T* o = static_cast<T*>(p.out) + size_t(bh) * p.o_bh + size_t(i) * p.o_row + g * 8;
#pragma unroll
    for (int d = 0; d < 8; ++d) st_f(o + d, acc[d] * inv);
    if (g == 0) p.lse[size_t(bh) * p.T + i] = (m + log2f(l)) * kLn2;
  }
}

// ------------------------------------------------------------------------------------------------ dQ (+ delta)
// Per query row i: delta_i = dO_i . O_i;  for each key j: p = exp(s - lse), dp = dO_i . V_sel(j),
// ds = p (dp - delta);  dq~_sel += ds * k~_sel(j).  Then dq_self = scale * R^T dq~_self, dq_cross = scale * dq~_cross.
template <typename T, int D>
__global__ void __launch_bounds__(kSimtThreads) attn_bwd_dq_simt_kernel(SimtParams p) {
  constexpr int G = D / 8, R = kSimtThreads / G, KT = kSimtTile, h = D / 2;
  __shared__ __align__(16) float sq_s[R][D], sq_c[R][D];
  __shared__ __align__(16) float sk_s[KT][D], sk_c[KT][D], sv_s[KT][D], sv_c[KT][D];

  const int bh = blockIdx.y, b = bh / p.H;
  const int r = threadIdx.x / G, g = threadIdx.x % G;
  const int i = blockIdx.x * R + r;
  const size_t head = size_t(bh) * p.T * D;
  const T* q_s = static_cast<const T*>(p.q_s) + head;
  const T* k_s = static_cast<const T*>(p.k_s) + head;
  const T* v_s = static_cast<const T*>(p.v_s) + head;
  const T* q_c = static_cast<const T*>(p.q_c) + head;
  const T* k_c = static_cast<const T*>(p.k_c) + head;
  const T* v_c = static_cast<const T*>(p.v_c) + head;
  const T* o = static_cast<const T*>(p.out) + size_t(bh) * p.o_bh;
  const T* dO = static_cast<const T*>(p.d_out) + size_t(bh) * p.o_bh;

  stage_row<T, D>(q_s, i, p.T, p.cos_tab, p.sin_tab, sq_s[r], g, G);
  stage_row<T, D>(q_c, i, p.T, nullptr, nullptr, sq_c[r], g, G);
  __syncwarp();
  const int irow = i < p.T ? i : p.T - 1;
  float qs[8], qc[8], go[8], dqs[8], dqc[8];
  float dpart = 0.f;
#pragma unroll
  for (int d = 0; d < 8; ++d) {
    qs[d] = sq_s[r][g * 8 + d];
    qc[d] = sq_c[r][g * 8 + d];
    go[d] = ld_f(dO + size_t(irow) * p.o_row + g * 8 + d);
    dpart = fmaf(go[d], ld_f(o + size_t(irow) * p.o_row + g * 8 + d), dpart);
    dqs[d] = 0.f;
    dqc[d] = 0.f;
  }
  const float delta = group_sum<G>(dpart);
  const float c2 = p.scale * kLog2e;
  const float lse2 = p.lse[size_t(bh) * p.T + irow] * kLog2e;
  if (i < p.T && g == 0) p.delta[size_t(bh) * p.T + i] = delta;
  const uint32_t* mrow = p.bits + (size_t(b) * p.T + irow) * p.TW;

  for (int j0 = 0; j0 < p.T; j0 += KT) {
    const uint32_t valid = ~p.kpad[size_t(b) * p.TW + j0 / 32];
    if (valid == 0u) continue;
    __syncthreads();
    for (int jj = threadIdx.x / 32; jj < KT; jj += kSimtThreads / 32) {
      const int lane = threadIdx.x % 32;
      stage_row<T, D>(k_s, j0 + jj, p.T, p.cos_tab, p.sin_tab, sk_s[jj], lane, 32);
      stage_row<T, D>(k_c, j0 + jj, p.T, nullptr, nullptr, sk_c[jj], lane, 32);
      stage_row<T, D>(v_s, j0 + jj, p.T, nullptr, nullptr, sv_s[jj], lane, 32);
      stage_row<T, D>(v_c, j0 + jj, p.T, nullptr, nullptr, sv_c[jj], lane, 32);
    }
    __syncthreads();
    const uint32_t cross = mrow[j0 / 32];
#pragma unroll 4
    for (int jj = 0; jj < KT; ++jj) {
      if (!((valid >> jj) & 1u)) continue;  // group-uniform
      const bool x = (cross >> jj) & 1u;
      const float* kk = x ? &sk_c[jj][g * 8] : &sk_s[jj][g * 8];
      const float* vv = x ? &sv_c[jj][g * 8] : &sv_s[jj][g * 8];
      float sp = 0.f, dp = 0.f;
#pragma unroll
      for (int d = 0; d < 8; ++d) {
        sp = fmaf(x ? qc[d] : qs[d], kk[d], sp);
        dp = fmaf(go[d], vv[d], dp);
      }
      sp = group_sum<G>(sp);
      dp = group_sum<G>(dp);
      // softmax: ds = p (dp - delta).  square-root softmax, r = sqrt(p): ds = r (dp - r delta) / 2
      float ds;
      if (p.sqrt_sm) {
        const float rj = exp2f(0.5f * (sp * c2 - lse2));
        ds = 0.5f * rj * (dp - rj * delta);
      } else {
        ds = exp2f(sp * c2 - lse2) * (dp - delta);
      }
      if (x) {
#pragma unroll
        for (int d = 0; d < 8; ++d) dqc[d] = fmaf(ds, kk[d], dqc[d]);
      } else {
#pragma unroll
        for (int d = 0; d < 8; ++d) dqs[d] = fmaf(ds, kk[d], dqs[d]);
      }
    }
  }
  // Un-rotate the self-pathway gradient through shared memory (the partner dimension lives in another thread).
  __syncthreads();
#pragma unroll
  for (int d = 0; d < 8; ++d) sq_s[r][g * 8 + d] = dqs[d];
  __syncwarp();
  if (i < p.T) {
    T* oq_s = static_cast<T*>(p.dq_s) + head + size_t(i) * D;
    T* oq_c = static_cast<T*>(p.dq_c) + head + size_t(i) * D;
#pragma unroll
    for (int d = 0; d < 8; ++d) {
      const int dd = g * 8 + d;
      float v = dqs[d];
      if (p.cos_tab != nullptr) {
        const int f = dd < h ? dd : dd - h;
        const float c = p.cos_tab[size_t(i) * h + f], s = p.sin_tab[size_t(i) * h + f];
        v = dd < h ? v * c + sq_s[r][dd + h] * s : v * c - sq_s[r][dd - h] * s;
      }
      st_f(oq_s + dd, v * p.scale);
      st_f(oq_c + dd, dqc[d] * p.scale);
    }
  }
}

// ------------------------------------------------------------------------------------------------ dK, dV
// Per key row j, looping over query tiles:  dv_sel += p * dO_i;  dk~_sel += ds * scale * q~_sel(i).
template <typename T, int D>
__global__ void __launch_bounds__(kSimtThreads) attn_bwd_dkv_simt_kernel(SimtParams p) {
  constexpr int G = D / 8, R = kSimtThreads / G, QT = kSimtTile, h = D / 2;
  __shared__ __align__(16) float sk_s[R][D], sk_c[R][D];
  __shared__ __align__(16) float sq_s[QT][D], sq_c[QT][D], sdo[QT][D];
  __shared__ float slse2[QT], sdelta[QT];

  const int bh = blockIdx.y, b = bh / p.H;
  const int r = threadIdx.x / G, g = threadIdx.x % G;
  const int j = blockIdx.x * R + r;
  const size_t head = size_t(bh) * p.T * D;
  const T* q_s = static_cast<const T*>(p.q_s) + head;
  const T* k_s = static_cast<const T*>(p.k_s) + head;
  const T* v_s = static_cast<const T*>(p.v_s) + head;
  const T* q_c = static_cast<const T*>(p.q_c) + head;
  const T* k_c = static_cast<const T*>(p.k_c) + head;
  const T* v_c = static_cast<const T*>(p.v_c) + head;
  const T* dO = static_cast<const T*>(p.d_out) + size_t(bh) * p.o_bh;

  stage_row<T, D>(k_s, j, p.T, p.cos_tab, p.sin_tab, sk_s[r], g, G);
  stage_row<T, D>(k_c, j, p.T, nullptr, nullptr, sk_c[r], g, G);
  __syncwarp();
  const int jrow = j < p.T ? j : p.T - 1;
  float ks[8], kc[8], vs[8], vc[8], dks[8], dkc[8], dvs[8], dvc[8];
#pragma unroll
  for (int d = 0; d < 8; ++d) {
    ks[d] = sk_s[r][g * 8 + d];
    kc[d] = sk_c[r][g * 8 + d];
    vs[d] = ld_f(v_s + size_t(jrow) * D + g * 8 + d);
    vc[d] = ld_f(v_c + size_t(jrow) * D + g * 8 + d);
    dks[d] = dkc[d] = dvs[d] = dvc[d] = 0.f;
  }
  const float c2 = p.scale * kLog2e;
  const bool key_valid = (j < p.T) && !((p.kpad[size_t(b) * p.TW + jrow / 32] >> (jrow % 32)) & 1u);
  const uint32_t* mrow = p.bitsT + (size_t(b) * p.T + jrow) * p.TW;

  for (int i0 = 0; i0 < p.T; i0 += QT) {
    __syncthreads();
    for (int ii = threadIdx.x / 32; ii < QT; ii += kSimtThreads / 32) {
      const int lane = threadIdx.x % 32;
      stage_row<T, D>(q_s, i0 + ii, p.T, p.cos_tab, p.sin_tab, sq_s[ii], lane, 32);
      stage_row<T, D>(q_c, i0 + ii, p.T, nullptr, nullptr, sq_c[ii], lane, 32);
      stage_row<T, D>(dO, i0 + ii, p.T, nullptr, nullptr, sdo[ii], lane, 32, p.o_row);
    }
    if (threadIdx.x < QT) {
      const int i = i0 + threadIdx.x;
      slse2[threadIdx.x] = i < p.T ? p.lse[size_t(bh) * p.T + i] * kLog2e : INFINITY;  // p = exp2(-inf) = 0
      sdelta[threadIdx.x] = i < p.T ? p.delta[size_t(bh) * p.T + i] : 0.f;
    }
    __syncthreads();
    const uint32_t cross = mrow[i0 / 32];
#pragma unroll 4
    for (int ii = 0; ii < QT; ++ii) {
      const bool x = (cross >> ii) & 1u;
      const float* qq = x ? &sq_c[ii][g * 8] : &sq_s[ii][g * 8];
      const float* gg = &sdo[ii][g * 8];
      float sp = 0.f, dp = 0.f;
#pragma unroll
      for (int d = 0; d < 8; ++d) {
        sp = fmaf(qq[d], x ? kc[d] : ks[d], sp);
        dp = fmaf(gg[d], x ? vc[d] : vs[d], dp);
      }
      sp = group_sum<G>(sp);
      dp = group_sum<G>(dp);
      // A padded key has probability zero; every thread still takes part in the shuffles above.
      // (pj multiplies dO in dV: p for the softmax, sqrt(p) for the square-root softmax)
      float pj, ds;
      if (p.sqrt_sm) {
        pj = key_valid ? exp2f(0.5f * (sp * c2 - slse2[ii])) : 0.f;
        ds = 0.5f * pj * (dp - pj * sdelta[ii]) * p.scale;
      } else {
        pj = key_valid ? exp2f(sp * c2 - slse2[ii]) : 0.f;
        ds = pj * (dp - sdelta[ii]) * p.scale;
      }
      if (x) {
#pragma unroll
        for (int d = 0; d < 8; ++d) {
          dvc[d] = fmaf(pj, gg[d], dvc[d]);
          dkc[d] = fmaf(ds, qq[d], dkc[d]);
        }
      } else {
#pragma unroll
        for (int d = 0; d < 8; ++d) {
          dvs[d] = fmaf(pj, gg[d], dvs[d]);
          dks[d] = fmaf(ds, qq[d], dks[d]);
        }
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int d = 0; d < 8; ++d) sk_s[r][g * 8 + d] = dks[d];
  __syncwarp();
  if (j < p.T) {
    const size_t off = head + size_t(j) * D;
#pragma unroll
    for (int d = 0; d < 8; ++d) {
      const int dd = g * 8 + d;
      float v = dks[d];
      if (p.cos_tab != nullptr) {
        const int f = dd < h ? dd : dd - h;
        const float c = p.cos_tab[size_t(j) * h + f], s = p.sin_tab[size_t(j) * h + f];
        v = dd < h ? v * c + sk_s[r][dd + h] * s : v * c - sk_s[r][dd - h] * s;
      }
      st_f(static_cast<T*>(p.dk_s) + off + dd, v);
      st_f(static_cast<T*>(p.dk_c) + off + dd, dkc[d]);
      st_f(static_cast<T*>(p.dv_s) + off + dd, dvs[d]);
      st_f(static_cast<T*>(p.dv_c) + off + dd, dvc[d]);
    }
  }
}

// ------------------------------------------------------------------------------------------------ launchers
static SimtParams make_params(const AttnArgs& a) {
  SimtParams p{};
  p.q_s = a.q_s; p.k_s = a.k_s; p.v_s = a.v_s; p.q_c = a.q_c; p.k_c = a.k_c; p.v_c = a.v_c;
  p.bits = a.meta.bits; p.bitsT = a.meta.bitsT; p.kpad = a.meta.kpad;
  p.cos_tab = a.rope ? a.rope_cos : nullptr;
  p.sin_tab = a.rope ? a.rope_sin : nullptr;
  p.out = a.out; p.lse = a.lse; p.d_out = a.d_out;
  p.dq_s = a.dq_s; p.dk_s = a.dk_s; p.dv_s = a.dv_s; p.dq_c = a.dq_c; p.dk_c = a.dk_c; p.dv_c = a.dv_c;
  p.delta = static_cast<float*>(a.workspace);
  p.B = a.B; p.H = a.H; p.T = a.T; p.TW = a.meta.TW;
  p.scale = a.scale;
  p.sqrt_sm = a.sqrt_softmax ? 1 : 0;
  p.o_row = out_row_stride(a);
  p.o_bh = out_bh_stride(a);
  return p;
}

size_t simt_bwd_workspace_bytes(int B, int H, int T, int D) { return align256(size_t(B) * H * T * sizeof(float)); }

template <typename T, int D>
static cudaError_t fwd_t(const AttnArgs& a) {
  constexpr int R = kSimtThreads / (D / 8);
  dim3 grid((a.T + R - 1) / R, a.B * a.H);
  attn_fwd_simt_kernel<T, D><<<grid, kSimtThreads, 0, a.stream>>>(make_params(a));
  count_launches(1);
  return cudaGetLastError();
}

template <typename T, int D>
static cudaError_t bwd_t(const AttnArgs& a) {
  constexpr int R = kSimtThreads / (D / 8);
  dim3 grid((a.T + R - 1) / R, a.B * a.H);
  SimtParams p = make_params(a);
  attn_bwd_dq_simt_kernel<T, D><<<grid, kSimtThreads, 0, a.stream>>>(p);
  attn_bwd_dkv_simt_kernel<T, D><<<grid, kSimtThreads, 0, a.stream>>>(p);
  count_launches(2);
  return cudaGetLastError();
}

#define MINTB_SIMT_DISPATCH(FN)                                                        \
  if (a.dtype == MINTB_F32) {                                                          \
    switch (a.D) {                                                                     \
      case 16: return FN<float, 16>(a);                                                \
      case 32: return FN<float, 32>(a);                                                \
      case 64: return FN<float, 64>(a);                                                \
    }                                                                                  \
  } else {                                                                             \
    switch (a.D) {                                                                     \
      case 16: return FN<__nv_bfloat16, 16>(a);                                        \
      case 32: return FN<__nv_bfloat16, 32>(a);                                        \
      case 64: return FN<__nv_bfloat16, 64>(a);                                        \
    }                                                                                  \
  }                                                                                    \
  return cudaErrorInvalidValue;

cudaError_t launch_attn_fwd_simt(const AttnArgs& a) { MINTB_SIMT_DISPATCH(fwd_t) }
cudaError_t launch_attn_bwd_simt(const AttnArgs& a) { MINTB_SIMT_DISPATCH(bwd_t) }

}  // namespace mintb
