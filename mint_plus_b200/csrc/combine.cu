// Combine from materialised logits: select by chain mask -> row softmax -> split -> two weighted sums, and its
// backward.  HBM-bound on the two (B,H,T,T) logit tensors; one warp per query row, fixed summation order.
#include "common.cuh"

namespace mintb {

template <typename T>
__device__ __forceinline__ float sel_logit(const T* il, const T* el, const uint8_t* m, int j) {
  return m[j] ? ld_f(el + j) : ld_f(il + j);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Row statistics shared by forward and backward: m = max_j logit, l = sum_j exp(logit - m).
template <typename T>
__device__ __forceinline__ void row_stats(const T* il, const T* el, const uint8_t* m, int Tn, int lane, float& mx,
                                          float& l) {
  mx = -INFINITY;
  for (int j = lane; j < Tn; j += 32) mx = fmaxf(mx, sel_logit(il, el, m, j));
  mx = warp_max(mx);
  l = 0.f;
  for (int j = lane; j < Tn; j += 32) l += expf(sel_logit(il, el, m, j) - mx);
  l = warp_sum(l);
}

template <typename T, int D>
__global__ void __launch_bounds__(128) combine_fwd_kernel(const T* __restrict__ il, const T* __restrict__ el,
                                                           const uint8_t* __restrict__ mask,
                                                           const T* __restrict__ iv, const T* __restrict__ ev,
                                                           T* __restrict__ out, int B, int H, int Tn) {
  constexpr int NV = (D + 31) / 32;
  const size_t row = size_t(blockIdx.x) * 4 + threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  if (row >= size_t(B) * H * Tn) return;
  const int i = int(row % Tn);
  const size_t bh = row / Tn;
  const int b = int(bh / H);
  const T* ilr = il + row * Tn;
  const T* elr = el + row * Tn;
  const uint8_t* mr = mask + (size_t(b) * Tn + i) * Tn;
  const T* ivh = iv + bh * Tn * D;
  const T* evh = ev + bh * Tn * D;
  float mx, l;
  row_stats(ilr, elr, mr, Tn, lane, mx, l);
  const float inv = 1.f / l;
  float acc[NV];
#pragma unroll
  for (int k = 0; k < NV; ++k) acc[k] = 0.f;
  for (int j0 = 0; j0 < Tn; j0 += 32) {
    const int j = j0 + lane;
    float pj = 0.f;
    bool x = false;
    if (j < Tn) {
      x = mr[j] != 0;
      pj = expf((x ? ld_f(elr + j) : ld_f(ilr + j)) - mx) * inv;
    }
    const unsigned xs = __ballot_sync(0xffffffffu, x);
    const int n = min(32, Tn - j0);
    for (int jj = 0; jj < n; ++jj) {
      const float pb = __shfl_sync(0xffffffffu, pj, jj);
      const T* v = ((xs >> jj) & 1u) ? evh + size_t(j0 + jj) * D : ivh + size_t(j0 + jj) * D;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int d = lane + 32 * k;
        if (d < D) acc[k] = fmaf(pb, ld_f(v + d), acc[k]);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int d = lane + 32 * k;
    if (d < D) st_f(out + row * D + d, acc[k]);
  }
}

// Backward kernel 1, one warp per query row: stats -> dP_ij = dO_i . V_sel(j) -> delta = sum_j p dP -> dS = p (dP - delta),
// written to the selected pathway's logit gradient (zero in the other).  Stores (m, 1/l) for kernel 2.
template <typename T, int D>
__global__ void __launch_bounds__(128) combine_bwd_rows_kernel(const T* __restrict__ il, const T* __restrict__ el,
                                                                const uint8_t* __restrict__ mask,
                                                                const T* __restrict__ iv, const T* __restrict__ ev,
                                                                const T* __restrict__ dO, T* __restrict__ d_il,
                                                                T* __restrict__ d_el, float* __restrict__ stats, int B,
                                                                int H, int Tn) {
  const size_t row = size_t(blockIdx.x) * 4 + threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  if (row >= size_t(B) * H * Tn) return;
  const int i = int(row % Tn);
  const size_t bh = row / Tn;
  const int b = int(bh / H);
  const T* ilr = il + row * Tn;
  const T* elr = el + row * Tn;
  const uint8_t* mr = mask + (size_t(b) * Tn + i) * Tn;
  const T* ivh = iv + bh * Tn * D;
  const T* evh = ev + bh * Tn * D;
  float go[D];
#pragma unroll
  for (int d = 0; d < D; ++d) go[d] = ld_f(dO + row * D + d);
  float mx, l;
  row_stats(ilr, elr, mr, Tn, lane, mx, l);
  const float inv = 1.f / l;
  if (lane == 0) {
    stats[row * 2] = mx;
    stats[row * 2 + 1] = inv;
  }
  float delta = 0.f;
  for (int j = lane; j < Tn; j += 32) {
    const bool x = mr[j] != 0;
    const T* v = x ? evh + size_t(j) * D : ivh + size_t(j) * D;
    float dp = 0.f;
#pragma unroll
    for (int d = 0; d < D; ++d) dp = fmaf(go[d], ld_f(v + d), dp);
    delta = fmaf(expf((x ? ld_f(elr + j) : ld_f(ilr + j)) - mx) * inv, dp, delta);
  }
  delta = warp_sum(delta);
  for (int j = lane; j < Tn; j += 32) {
    const bool x = mr[j] != 0;
    const T* v = x ? evh + size_t(j) * D : ivh + size_t(j) * D;
    float dp = 0.f;
#pragma unroll
    for (int d = 0; d < D; ++d) dp = fmaf(go[d], ld_f(v + d), dp);
    const float pj = expf((x ? ld_f(elr + j) : ld_f(ilr + j)) - mx) * inv;
    const float ds = pj * (dp - delta);
    st_f(d_il + row * Tn + j, x ? 0.f : ds);
    st_f(d_el + row * Tn + j, x ? ds : 0.f);
  }
}

// Backward kernel 2: dV_intra[j] = sum_i (p o ~M)_ij dO_i, dV_inter[j] = sum_i (p o M)_ij dO_i.
// Block = 32 keys x 4 slices of D; walks the query rows in order (deterministic).
template <typename T, int D>
__global__ void __launch_bounds__(128) combine_bwd_values_kernel(const T* __restrict__ il, const T* __restrict__ el,
                                                                  const uint8_t* __restrict__ mask,
                                                                  const T* __restrict__ dO,
                                                                  const float* __restrict__ stats,
                                                                  T* __restrict__ d_iv, T* __restrict__ d_ev, int B,
                                                                  int H, int Tn) {
  constexpr int DS = D / 4;
  const int jj = threadIdx.x % 32, q = threadIdx.x / 32;
  const int j = blockIdx.x * 32 + jj;
  const size_t bh = blockIdx.y;
  const int b = int(bh / H);
  float ai[DS], ae[DS];
#pragma unroll
  for (int d = 0; d < DS; ++d) ai[d] = ae[d] = 0.f;
  if (j < Tn) {
    for (int i = 0; i < Tn; ++i) {
      const size_t row = bh * Tn + i;
      const bool x = mask[(size_t(b) * Tn + i) * Tn + j] != 0;
      const float lg = x ? ld_f(el + row * Tn + j) : ld_f(il + row * Tn + j);
      const float pj = expf(lg - stats[row * 2]) * stats[row * 2 + 1];
      const T* g = dO + row * D + q * DS;
      if (x) {
#pragma unroll
        for (int d = 0; d < DS; ++d) ae[d] = fmaf(pj, ld_f(g + d), ae[d]);
      } else {
#pragma unroll
        for (int d = 0; d < DS; ++d) ai[d] = fmaf(pj, ld_f(g + d), ai[d]);
      }
    }
    const size_t off = (bh * Tn + j) * D + q * DS;
#pragma unroll
    for (int d = 0; d < DS; ++d) {
      st_f(d_iv + off + d, ai[d]);
      st_f(d_ev + off + d, ae[d]);
    }
  }
}

template <typename T, int D>
static cudaError_t fwd_t(const void* il, const void* el, const uint8_t* mask, const void* iv, const void* ev, void* out,
                         int B, int H, int Tn, cudaStream_t s) {
  size_t rows = size_t(B) * H * Tn;
  combine_fwd_kernel<T, D><<<unsigned((rows + 3) / 4), 128, 0, s>>>(
      static_cast<const T*>(il), static_cast<const T*>(el), mask, static_cast<const T*>(iv), static_cast<const T*>(ev),
      static_cast<T*>(out), B, H, Tn);
  count_launches(1);
  return cudaGetLastError();
}

template <typename T, int D>
static cudaError_t bwd_t(const void* il, const void* el, const uint8_t* mask, const void* iv, const void* ev,
                         const void* d_out, void* d_il, void* d_el, void* d_iv, void* d_ev, float* stats, int B, int H,
                         int Tn, cudaStream_t s) {
  size_t rows = size_t(B) * H * Tn;
  combine_bwd_rows_kernel<T, D><<<unsigned((rows + 3) / 4), 128, 0, s>>>(
      static_cast<const T*>(il), static_cast<const T*>(el), mask, static_cast<const T*>(iv), static_cast<const T*>(ev),
      static_cast<const T*>(d_out), static_cast<T*>(d_il), static_cast<T*>(d_el), stats, B, H, Tn);
  dim3 grid((Tn + 31) / 32, B * H);
  combine_bwd_values_kernel<T, D><<<grid, 128, 0, s>>>(static_cast<const T*>(il), static_cast<const T*>(el), mask,
                                                       static_cast<const T*>(d_out), stats, static_cast<T*>(d_iv),
                                                       static_cast<T*>(d_ev), B, H, Tn);
  count_launches(2);
  return cudaGetLastError();
}

cudaError_t launch_combine_fwd(const void* il, const void* el, const uint8_t* mask, const void* iv, const void* ev,
                               void* out, int B, int H, int T, int D, int dtype, cudaStream_t s) {
#define CASE(TT, DD) return fwd_t<TT, DD>(il, el, mask, iv, ev, out, B, H, T, s)
  if (dtype == MINTB_F32) {
    if (D == 16) CASE(float, 16);
    if (D == 32) CASE(float, 32);
    if (D == 64) CASE(float, 64);
  } else {
    if (D == 16) CASE(__nv_bfloat16, 16);
    if (D == 32) CASE(__nv_bfloat16, 32);
    if (D == 64) CASE(__nv_bfloat16, 64);
  }
#undef CASE
  return cudaErrorInvalidValue;
}

cudaError_t launch_combine_bwd(const void* il, const void* el, const uint8_t* mask, const void* iv, const void* ev,
                               const void* d_out, void* d_il, void* d_el, void* d_iv, void* d_ev, float* stats, int B,
                               int H, int T, int D, int dtype, cudaStream_t s) {
#define CASE(TT, DD) return bwd_t<TT, DD>(il, el, mask, iv, ev, d_out, d_il, d_el, d_iv, d_ev, stats, B, H, T, s)
  if (dtype == MINTB_F32) {
    if (D == 16) CASE(float, 16);
    if (D == 32) CASE(float, 32);
    if (D == 64) CASE(float, 64);
  } else {
    if (D == 16) CASE(__nv_bfloat16, 16);
    if (D == 32) CASE(__nv_bfloat16, 32);
    if (D == 64) CASE(__nv_bfloat16, 64);
  }
#undef CASE
  return cudaErrorInvalidValue;
}

}  // namespace mintb
