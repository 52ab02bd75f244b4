// The two ends of the model around the layer stack, as HBM-bound kernels:
//   embed_fwd / embed_bwd   token embedding with the token-dropout rescale, <mask> and <pad> zeroing of MINT.forward and the
//                           (B,T,E) -> (T,B,E) layout change, in one pass; its weight gradient by per-CTA private sums
//   masked_ce_fwd / _bwd    the masked-language-model loss of the training step: cross-entropy over the vocabulary at the
//                           target positions, averaged over them, and its gradient with respect to the logits
#include "common.cuh"

namespace mintb {

namespace {

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Factor of token (b, t): 0 for <pad>, 0 for <mask> under token dropout, else the row's rescale
// (1 - mask_ratio_train) / (1 - masked / unpadded) under token dropout, else 1.
__device__ __forceinline__ float row_scale(int n_mask, int n_real, int token_dropout, float mask_ratio_train) {
  if (!token_dropout) return 1.f;
  const float observed = float(n_mask) / float(n_real);      // 0 / 0 -> NaN, as the tensor expression gives for an all-pad row
  return (1.f - mask_ratio_train) / (1.f - observed);
}

// One CTA per batch row: count <mask> and unpadded tokens, then write out[t][b][:] = W[tok] * factor for every t.
template <typename T>
__global__ void __launch_bounds__(256) embed_fwd_kernel(const long long* __restrict__ tokens, const T* __restrict__ w, T* __restrict__ out,
                                                       float* __restrict__ scales, int B, int Tn, int E, int V, int pad_idx,
                                                       int mask_idx, int token_dropout, float mask_ratio_train) {
  __shared__ int s_cnt[2];
  const int b = blockIdx.x;
  const long long* row = tokens + size_t(b) * Tn;
  if (threadIdx.x < 2) s_cnt[threadIdx.x] = 0;
  __syncthreads();
  int nm = 0, nr = 0;
  for (int t = threadIdx.x; t < Tn; t += blockDim.x) {
    const long long tok = row[t];
    nm += tok == mask_idx;
    nr += tok != pad_idx;
  }
  atomicAdd(&s_cnt[0], nm);
  atomicAdd(&s_cnt[1], nr);
  __syncthreads();
  const float scale = row_scale(s_cnt[0], s_cnt[1], token_dropout, mask_ratio_train);
  if (threadIdx.x == 0 && scales != nullptr) scales[b] = scale;
  constexpr int VEC = 16 / sizeof(T);
  const int nvec = E / VEC;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, nwarps = blockDim.x / 32;
  for (int t = warp; t < Tn; t += nwarps) {
    const long long tok = row[t];
    const bool zero = tok == pad_idx || (token_dropout && tok == mask_idx) || tok < 0 || tok >= V;
    const uint4* src = reinterpret_cast<const uint4*>(w + size_t(zero ? 0 : tok) * E);
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t(t) * B + b) * E);
    for (int v = lane; v < nvec; v += 32) {
      uint4 q = make_uint4(0u, 0u, 0u, 0u);
      if (!zero) {
        q = __ldg(src + v);
        if (scale != 1.f) {
          T* e = reinterpret_cast<T*>(&q);
#pragma unroll
          for (int j = 0; j < VEC; ++j) e[j] = from_f<T>(to_f<T>(e[j]) * scale);
        }
      }
      dst[v] = q;
    }
  }
}

// dW[v][:] += factor(b, t) * d_out[t][b][:] over the tokens with tok == v.  A CTA walks a slab of tokens of one batch row
// with a private [V][chunk] sum in shared memory (a thread owns its columns, so no two threads meet), then adds the slab's
// sums to the fp32 result with one atomic per element.  grid = (slabs, B, column chunks).
template <typename T>
__global__ void __launch_bounds__(256) embed_bwd_kernel(const long long* __restrict__ tokens, const T* __restrict__ d_out,
                                                       const float* __restrict__ scales, float* __restrict__ dw, int B, int Tn, int E,
                                                       int V, int pad_idx, int mask_idx, int token_dropout, int slab, int chunk) {
  extern __shared__ float s_acc[];   // [V][chunk]
  const int b = blockIdx.y, c0 = blockIdx.z * chunk;
  const int cols = min(chunk, E - c0);
  for (int i = threadIdx.x; i < V * chunk; i += blockDim.x) s_acc[i] = 0.f;
  __syncthreads();
  const float scale = scales[b];
  const int t0 = blockIdx.x * slab, t1 = min(Tn, t0 + slab);
  for (int t = t0; t < t1; ++t) {
    const long long tok = tokens[size_t(b) * Tn + t];
    if (tok == pad_idx || (token_dropout && tok == mask_idx) || tok < 0 || tok >= V) continue;   // uniform over the CTA
    const T* g = d_out + (size_t(t) * B + b) * E + c0;
    float* acc = s_acc + size_t(tok) * chunk;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) acc[c] += to_f<T>(g[c]) * scale;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < V * chunk; i += blockDim.x) {
    const int v = i / chunk, c = i % chunk;
    const float a = s_acc[i];
    if (c < cols && a != 0.f) atomicAdd(dw + size_t(v) * E + c0 + c, a);
  }
}

// One thread per token row of the logits [N][ld] (the first V columns count): log-sum-exp, the loss at the target where the
// row is a target position, and the two sums (loss, count) by one atomic per warp.
__global__ void __launch_bounds__(256) masked_ce_fwd_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets,
                                                           const unsigned char* __restrict__ mask, float* __restrict__ lse_out,
                                                           float* __restrict__ sums, int N, int ld, int V) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  float loss = 0.f, cnt = 0.f;
  if (i < N) {
    const __nv_bfloat16* row = logits + size_t(i) * ld;
    float m = -INFINITY;
    for (int v = 0; v < V; ++v) m = fmaxf(m, __bfloat162float(row[v]));
    float s = 0.f;
    for (int v = 0; v < V; ++v) s += __expf(__bfloat162float(row[v]) - m);
    const float lse = m + __logf(s);
    lse_out[i] = lse;
    if (mask[i]) {
      const long long tg = targets[i];
      loss = lse - (tg >= 0 && tg < V ? __bfloat162float(row[tg]) : 0.f);
      cnt = 1.f;
    }
  }
  for (int off = 16; off > 0; off >>= 1) {
    loss += __shfl_xor_sync(0xffffffffu, loss, off);
    cnt += __shfl_xor_sync(0xffffffffu, cnt, off);
  }
  if ((threadIdx.x % 32) == 0 && cnt > 0.f) {
    atomicAdd(sums, loss);
    atomicAdd(sums + 1, cnt);
  }
}

// d_logits[i][v] = (softmax(logits[i])[v] - [v == target]) * g / count at target rows, 0 elsewhere and in the pad columns.
__global__ void __launch_bounds__(256) masked_ce_bwd_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets,
                                                           const unsigned char* __restrict__ mask, const float* __restrict__ lse,
                                                           const float* __restrict__ sums, const float* __restrict__ g,
                                                           __nv_bfloat16* __restrict__ d_logits, int N, int ld, int V) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N) return;
  __nv_bfloat16* drow = d_logits + size_t(i) * ld;
  if (!mask[i]) {
    for (int v = 0; v < ld; ++v) drow[v] = __float2bfloat16_rn(0.f);
    return;
  }
  const float coef = g[0] / sums[1];
  const __nv_bfloat16* row = logits + size_t(i) * ld;
  const float l = lse[i];
  const long long tg = targets[i];
  for (int v = 0; v < ld; ++v) {
    float d = 0.f;
    if (v < V) d = (__expf(__bfloat162float(row[v]) - l) - (v == tg ? 1.f : 0.f)) * coef;
    drow[v] = __float2bfloat16_rn(d);
  }
}

}  // namespace
}  // namespace mintb

using namespace mintb;

static int el_fail(const char* what, cudaError_t e) {
  set_error("%s: %s", what, cudaGetErrorString(e));
  return MINTB_ECUDA;
}

extern "C" int mintb_embed_fwd(const long long* tokens, const void* weight, void* out, float* row_scales, int B, int T, int E, int V,
                               int dtype, int pad_idx, int mask_idx, int token_dropout, float mask_ratio_train, void* stream) {
  const int esz = dtype == MINTB_F32 ? 4 : 2;
  if (tokens == nullptr || weight == nullptr || out == nullptr || B <= 0 || T <= 0 || E <= 0 || V <= 0 ||
      (dtype != MINTB_F32 && dtype != MINTB_BF16) || (E * esz) % 16 != 0 || (reinterpret_cast<uintptr_t>(weight) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15)) {
    set_error("mintb_embed_fwd: tokens, weight, out, positive sizes, an f32 / bf16 weight with 16-byte rows and aligned pointers are required");
    return MINTB_EINVAL;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == MINTB_F32)
    embed_fwd_kernel<float><<<B, 256, 0, st>>>(tokens, static_cast<const float*>(weight), static_cast<float*>(out), row_scales, B, T, E, V,
                                               pad_idx, mask_idx, token_dropout, mask_ratio_train);
  else
    embed_fwd_kernel<__nv_bfloat16><<<B, 256, 0, st>>>(tokens, static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(out),
                                                       row_scales, B, T, E, V, pad_idx, mask_idx, token_dropout, mask_ratio_train);
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? MINTB_OK : el_fail("mintb_embed_fwd launch", e);
}

extern "C" int mintb_embed_bwd(const long long* tokens, const void* d_out, const float* row_scales, float* d_weight, int B, int T, int E,
                               int V, int dtype, int pad_idx, int mask_idx, int token_dropout, void* stream) {
  if (tokens == nullptr || d_out == nullptr || row_scales == nullptr || d_weight == nullptr || B <= 0 || T <= 0 || E <= 0 || V <= 0 ||
      V > 64 || (dtype != MINTB_F32 && dtype != MINTB_BF16)) {
    set_error("mintb_embed_bwd: tokens, d_out, row_scales, d_weight, positive sizes, a vocabulary of at most 64 and f32 / bf16 are required");
    return MINTB_EINVAL;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(d_weight, 0, size_t(V) * E * sizeof(float), st);
  if (e != cudaSuccess) return el_fail("mintb_embed_bwd memset", e);
  const int chunk = E < 512 ? E : 512;                 // V x 512 fp32 = at most 128 KB of shared memory
  const int slab = 128;
  const size_t smem = size_t(V) * chunk * sizeof(float);
  dim3 grid((T + slab - 1) / slab, B, (E + chunk - 1) / chunk);
  if (dtype == MINTB_F32) {
    e = cudaFuncSetAttribute(embed_bwd_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return el_fail("cudaFuncSetAttribute", e);
    embed_bwd_kernel<float><<<grid, 256, smem, st>>>(tokens, static_cast<const float*>(d_out), row_scales, d_weight, B, T, E, V, pad_idx,
                                                     mask_idx, token_dropout, slab, chunk);
  } else {
    e = cudaFuncSetAttribute(embed_bwd_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return el_fail("cudaFuncSetAttribute", e);
    embed_bwd_kernel<__nv_bfloat16><<<grid, 256, smem, st>>>(tokens, static_cast<const __nv_bfloat16*>(d_out), row_scales, d_weight, B, T, E,
                                                             V, pad_idx, mask_idx, token_dropout, slab, chunk);
  }
  count_launches(1);
  e = cudaGetLastError();
  return e == cudaSuccess ? MINTB_OK : el_fail("mintb_embed_bwd launch", e);
}

extern "C" int mintb_masked_ce_fwd(const void* logits, const long long* targets, const unsigned char* mask, float* lse, float* sums,
                                   int N, int ld, int V, void* stream) {
  if (logits == nullptr || targets == nullptr || mask == nullptr || lse == nullptr || sums == nullptr || N <= 0 || V <= 0 || ld < V) {
    set_error("mintb_masked_ce_fwd: logits (bf16 [N][ld], ld >= V), targets, mask, lse, sums and positive sizes are required");
    return MINTB_EINVAL;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(sums, 0, 2 * sizeof(float), st);
  if (e != cudaSuccess) return el_fail("mintb_masked_ce_fwd memset", e);
  masked_ce_fwd_kernel<<<(N + 255) / 256, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), targets, mask, lse, sums, N, ld, V);
  count_launches(1);
  e = cudaGetLastError();
  return e == cudaSuccess ? MINTB_OK : el_fail("mintb_masked_ce_fwd launch", e);
}

extern "C" int mintb_masked_ce_bwd(const void* logits, const long long* targets, const unsigned char* mask, const float* lse,
                                   const float* sums, const float* grad_loss, void* d_logits, int N, int ld, int V, void* stream) {
  if (logits == nullptr || targets == nullptr || mask == nullptr || lse == nullptr || sums == nullptr || grad_loss == nullptr ||
      d_logits == nullptr || N <= 0 || V <= 0 || ld < V) {
    set_error("mintb_masked_ce_bwd: every pointer and positive sizes (ld >= V) are required");
    return MINTB_EINVAL;
  }
  masked_ce_bwd_kernel<<<(N + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(logits), targets, mask, lse, sums, grad_loss, static_cast<__nv_bfloat16*>(d_logits), N, ld, V);
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? MINTB_OK : el_fail("mintb_masked_ce_bwd launch", e);
}
