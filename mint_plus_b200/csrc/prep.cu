// Mask metadata and RoPE tables: small memory-bound kernels run once per batch.
#include "common.cuh"

namespace mintb {

// One thread per 32-key word of one query row: bit = (chain_id[i] != chain_id[j]).
// The relation is symmetric, so the key-major copy (bitsT) holds the same words.
__global__ void meta_bits_from_chain_ids(const int32_t* __restrict__ chain_ids, uint32_t* __restrict__ bits,
                                         uint32_t* __restrict__ bitsT, int B, int T, int TW) {
  size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  size_t total = size_t(B) * T * TW;
  if (idx >= total) return;
  int w = int(idx % TW);
  size_t bi = idx / TW;
  int i = int(bi % T);
  int b = int(bi / T);
  const int32_t* row = chain_ids + size_t(b) * T;
  int32_t ci = row[i];
  uint32_t word = 0;
  int j0 = w * 32;
#pragma unroll 8
  for (int jj = 0; jj < 32; ++jj) {
    int j = j0 + jj;
    if (j < T && row[j] != ci) word |= (1u << jj);
  }
  bits[idx] = word;
  bitsT[idx] = word;
}

// Arbitrary (B,T,T) mask: row-major words, and the transposed relation for the key-major copy.
__global__ void meta_bits_from_mask(const uint8_t* __restrict__ mask, uint32_t* __restrict__ bits,
                                    uint32_t* __restrict__ bitsT, int B, int T, int TW) {
  size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  size_t total = size_t(B) * T * TW;
  if (idx >= total) return;
  int w = int(idx % TW);
  size_t bi = idx / TW;
  int i = int(bi % T);
  int b = int(bi / T);
  const uint8_t* m = mask + size_t(b) * T * T;
  uint32_t word = 0, wordT = 0;
  int j0 = w * 32;
  for (int jj = 0; jj < 32; ++jj) {
    int j = j0 + jj;
    if (j < T) {
      if (m[size_t(i) * T + j]) word |= (1u << jj);
      if (m[size_t(j) * T + i]) wordT |= (1u << jj);  // row i of bitsT is KEY i; bit jj is QUERY j
    }
  }
  bits[idx] = word;
  bitsT[idx] = wordT;
}

__global__ void meta_kpad(const uint8_t* __restrict__ key_pad, uint32_t* __restrict__ kpad, int B, int T, int TW) {
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * TW) return;
  int w = idx % TW, b = idx / TW;
  uint32_t word = 0;
  for (int jj = 0; jj < 32; ++jj) {
    int j = w * 32 + jj;
    bool padded = (j >= T) || (key_pad != nullptr && key_pad[size_t(b) * T + j] != 0);
    if (padded) word |= (1u << jj);
  }
  kpad[idx] = word;
}

// One warp per 64x64 tile: lanes stride over the 64 query rows, two words per row.
__global__ void meta_tile_class(const uint32_t* __restrict__ bits, const uint32_t* __restrict__ kpad,
                                uint8_t* __restrict__ cls, int B, int T, int TW, int NT) {
  int warp = (blockIdx.x * blockDim.x + threadIdx.x) / 32;
  int lane = threadIdx.x % 32;
  if (warp >= B * NT * NT) return;
  int kt = warp % NT, qt = (warp / NT) % NT, b = warp / (NT * NT);
  uint32_t pad0 = kpad[size_t(b) * TW + 2 * kt], pad1 = kpad[size_t(b) * TW + 2 * kt + 1];
  uint32_t intra = 0, inter = 0;
  for (int r = lane; r < kClassTile; r += 32) {
    int i = qt * kClassTile + r;
    if (i < T) {
      const uint32_t* row = bits + (size_t(b) * T + i) * TW + 2 * kt;
      uint32_t w0 = row[0], w1 = row[1];
      inter |= (w0 & ~pad0) | (w1 & ~pad1);
      intra |= (~w0 & ~pad0) | (~w1 & ~pad1);
    }
  }
  intra = __reduce_or_sync(0xffffffffu, intra);
  inter = __reduce_or_sync(0xffffffffu, inter);
  if (lane == 0) {
    uint8_t c = 0;
    if (intra) c |= kHasIntra;
    if (inter) c |= kHasInter;
    if (pad0 | pad1) c |= kHasPad;
    cls[warp] = c;
  }
}

static cudaError_t finish_meta(const uint8_t* key_pad, void* meta, int B, int T, cudaStream_t s) {
  MetaLayout L = meta_layout(B, T);
  char* p = static_cast<char*>(meta);
  uint32_t* bits = reinterpret_cast<uint32_t*>(p + L.off_bits);
  uint32_t* kpad = reinterpret_cast<uint32_t*>(p + L.off_kpad);
  uint8_t* cls = reinterpret_cast<uint8_t*>(p + L.off_cls);
  meta_kpad<<<(B * L.TW + 127) / 128, 128, 0, s>>>(key_pad, kpad, B, T, L.TW);
  int warps = B * L.NT * L.NT;
  meta_tile_class<<<(warps * 32 + 127) / 128, 128, 0, s>>>(bits, kpad, cls, B, T, L.TW, L.NT);
  count_launches(3);  // bits + kpad + class
  return cudaGetLastError();
}

cudaError_t launch_meta_from_chain_ids(const int32_t* chain_ids, const uint8_t* key_pad, void* meta, int B, int T,
                                       cudaStream_t s) {
  MetaLayout L = meta_layout(B, T);
  char* p = static_cast<char*>(meta);
  size_t total = size_t(B) * T * L.TW;
  meta_bits_from_chain_ids<<<unsigned((total + 255) / 256), 256, 0, s>>>(
      chain_ids, reinterpret_cast<uint32_t*>(p + L.off_bits), reinterpret_cast<uint32_t*>(p + L.off_bitsT), B, T, L.TW);
  return finish_meta(key_pad, meta, B, T, s);
}

cudaError_t launch_meta_from_mask(const uint8_t* mask, const uint8_t* key_pad, void* meta, int B, int T,
                                  cudaStream_t s) {
  MetaLayout L = meta_layout(B, T);
  char* p = static_cast<char*>(meta);
  size_t total = size_t(B) * T * L.TW;
  meta_bits_from_mask<<<unsigned((total + 255) / 256), 256, 0, s>>>(
      mask, reinterpret_cast<uint32_t*>(p + L.off_bits), reinterpret_cast<uint32_t*>(p + L.off_bitsT), B, T, L.TW);
  return finish_meta(key_pad, meta, B, T, s);
}

// cos/sin of float(position) * inv_freq[i], full-range accurate cosf/sinf (arguments reach ~T radians).
__global__ void rope_tables_kernel(const float* __restrict__ inv_freq, float* __restrict__ cos_tab,
                                   float* __restrict__ sin_tab, int T, int half) {
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T * half) return;
  int i = idx % half, t = idx / half;
  float ang = __fmul_rn(float(t), inv_freq[i]);
  cos_tab[idx] = cosf(ang);
  sin_tab[idx] = sinf(ang);
}

cudaError_t launch_rope_tables(const float* inv_freq, float* cos_tab, float* sin_tab, int T, int D, cudaStream_t s) {
  int n = T * (D / 2);
  rope_tables_kernel<<<(n + 255) / 256, 256, 0, s>>>(inv_freq, cos_tab, sin_tab, T, D / 2);
  count_launches(1);
  return cudaGetLastError();
}

}  // namespace mintb
