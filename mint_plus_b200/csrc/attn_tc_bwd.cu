// tcgen05 backward of the combined-softmax multimer attention (bf16 in, fp32 accumulate).
//
// With the forward log-sum-exp known, the two pathways are independent: the self pathway contributes
// P o ~M and the cross pathway P o M, each computed from its own Q, K, V.  The grid is
// (key tiles of 128, batch*head, pathway); a CTA owns dK and dV of its key tile in TMEM and walks the query
// tiles of 128 whose class holds pairs of its pathway:
//   S^T = K Q^T, dP^T = V dO^T            (lane = key, column = query; two halves of 64 queries, one TMEM buffer each)
//   P^T = exp2(S^T c - lse), masked       dS^T = P^T o (dP^T - delta)
//   dV += P^T dO, dK += dS^T Q            (A operands read from TMEM, aliased over S^T / dP^T)
//   dQ_tile = dS K                        (dS through shared memory), added to an fp32 accumulator in HBM
// Warp roles: warps 0-3 MMA issuers, one per family of products (warp 0 also issues the TMA loads), warps 4-19 compute
// (thread = key row x 16 query columns of the half in flight).  The halves ping-pong: while one is computed the tensor pipe refills the other buffer.
// TMEM (512 columns): dK, dV, two dQ tiles, then two (head_dim 64) or three (head_dim <= 32) buffers {S^T half, dP^T half}.
// dQ is accumulated across CTAs with fp32 atomics, so its low-order bits depend on arrival order;
// dK and dV are reduced inside one CTA in a fixed order.  All mbarrier waits are bounded.
#include "common.cuh"
#include "ptx.cuh"

namespace mintb {

using namespace ptx;

constexpr int kBwdTile = 128;       // keys per CTA and queries per step
constexpr int kHalf = 64;           // queries per compute group
constexpr int kBwdMaxTiles = 256;   // T <= 32768
constexpr unsigned kBwdStaggerNs = 250;   // initial offset between the two pairs of compute groups

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn bwd_encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// (B,H,T,D) tensors: dimensions (D, T, BH), box (D, rows, 1).  Sequence-first (T,B,H,D) tensors: dimensions (D, BH, T),
// box (D, 1, rows) — the same bytes land in shared memory, the two outer coordinates swap places.
static bool bwd_make_map(CUtensorMap* m, const void* ptr, int D, int T, int BH, int box_rows, bool seq_first = false) {
  EncodeTiledFn fn = bwd_encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[3] = {cuuint64_t(D), cuuint64_t(seq_first ? BH : T), cuuint64_t(seq_first ? T : BH)};
  cuuint64_t strides[2] = {cuuint64_t(D) * 2, cuuint64_t(seq_first ? BH : T) * D * 2};
  cuuint32_t box[3] = {cuuint32_t(D), cuuint32_t(seq_first ? 1 : box_rows), cuuint32_t(seq_first ? box_rows : 1)};
  cuuint32_t es[3] = {1, 1, 1};
  CUtensorMapSwizzle sw = D == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : D == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// fp32 dQ accumulator [BH][T][D] as a reduction target: box = (D / 4 columns, 32 rows, 1), i.e. what one compute warp
// drains from TMEM per query tile.
static bool bwd_make_dq_map(CUtensorMap* m, const void* ptr, int D, int T, int BH) {
  EncodeTiledFn fn = bwd_encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[3] = {cuuint64_t(D), cuuint64_t(T), cuuint64_t(BH)};
  cuuint64_t strides[2] = {cuuint64_t(D) * 4, cuuint64_t(T) * D * 4};
  cuuint32_t box[3] = {cuuint32_t(D / 4), 32, 1};
  cuuint32_t es[3] = {1, 1, 1};
  CUtensorMapSwizzle sw = D == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : D == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE;
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

__device__ __forceinline__ float bwd_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t bwd_pack(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint64_t pack2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t fadd2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t fmul2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ void named_barrier(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ------------------------------------------------------------------------------------------------ pre / post passes
// Per-query statistics for the backward pass: nl = -lse * log2 e and nd = -delta, delta = sum_d dO[i][d] * O[i][d], stored
// for each pair of queries (2p, 2p+1) of a (batch, head) as the 16 bytes (nl0, nl1, nd0, nd1).
// Rows are padded to a multiple of 128 per (batch, head); the pad entries are (-inf, 0), which makes exp2 give 0 there.
// The pass also clears the two fp32 dQ accumulators that the main kernel adds to.
// `factor` is 1, or 1/2 for the square-root softmax (whose kernel works with sqrt(p) = exp2((s c - lse) / 2) and delta / 2).
__global__ void __launch_bounds__(256) bwd_stats_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                                        const float* __restrict__ lse, float2* __restrict__ stats, int BH, int T,
                                                        int Tpad, int D, float factor, size_t row_stride, size_t bh_stride,
                                                        float* __restrict__ acc_s, float* __restrict__ acc_c) {
  griddep_launch();       // the main kernel's set-up may overlap this pass; it waits for it before it reads the statistics
  const int lpr = D / 8;  // lanes per row
  const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t prow = idx / lpr;          // row in the padded layout
  const int c = int(idx % lpr);
  const size_t bh = prow / Tpad;
  const int t = int(prow % Tpad);
  const bool live = bh < size_t(BH) && t < T;
  float acc = 0.f;
  if (live) {
    const size_t off = bh * bh_stride + size_t(t) * row_stride + c * 8;   // same layout for O and dO
    const uint4 a = *reinterpret_cast<const uint4*>(o + off);
    const uint4 b = *reinterpret_cast<const uint4*>(d_o + off);
    const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 x = __bfloat1622float2(ap[e]), y = __bfloat1622float2(bp[e]);
      acc = fmaf(x.x, y.x, acc);
      acc = fmaf(x.y, y.y, acc);
    }
    // this thread's eight columns of the row in the two fp32 dQ accumulators [b h][T][D] start at zero
    const size_t ao = (bh * T + t) * D + c * 8;
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    *reinterpret_cast<float4*>(acc_s + ao) = z;
    *reinterpret_cast<float4*>(acc_s + ao + 4) = z;
    *reinterpret_cast<float4*>(acc_c + ao) = z;
    *reinterpret_cast<float4*>(acc_c + ao + 4) = z;
  }
  for (int off = lpr / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (bh < size_t(BH) && c == 0) {
    // two queries share 16 bytes as (nl0, nl1, nd0, nd1): the kernel then reads each pair of like values as one
    // 64-bit register pair, ready for its packed fp32x2 arithmetic
    float* dst = reinterpret_cast<float*>(stats) + (prow / 2) * 4 + (prow % 2);
    dst[0] = live ? -lse[bh * T + t] * kLog2e * factor : -INFINITY;
    dst[2] = live ? -acc * factor : 0.f;
  }
}

// dq = scale * R^T(acc) for the self pathway (with tables), scale * acc for the cross pathway; fp32 -> bf16.
__global__ void __launch_bounds__(256) bwd_dq_convert_kernel(const float* __restrict__ acc_s, const float* __restrict__ acc_c,
                                                             __nv_bfloat16* __restrict__ dq_s, __nv_bfloat16* __restrict__ dq_c,
                                                             const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
                                                             size_t rows, int T, int D, float scale, int H, size_t g_row,
                                                             size_t g_b, size_t g_h, const int32_t* __restrict__ token_row, int B) {
  griddep_wait();   // launched while the main kernel may still be running: its additions have to be complete
  const int h = D / 2, cpr = h / 8;
  const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= rows * cpr) return;
  const int c = int(idx % cpr);
  const size_t row = idx / cpr;
  const int t = int(row % T);
  float lo[8], hi[8];
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    const float* src = (which == 0 ? acc_s : acc_c) + row * D + c * 8;
    // accumulators are [b][h][t][D]; the result goes to ptr + t * g_row + b * g_b + h * g_h (+ column), or, with a token
    // map, to row token_row[t * B + b] of the row-major matrix (g_b is its row length); tokens without a row are dropped
    const size_t bh_ = row / T;
    size_t base = size_t(t) * g_row + (bh_ / H) * g_b;
    if (token_row != nullptr) {
      const int tr = __ldg(token_row + size_t(t) * B + bh_ / H);
      if (tr < 0) return;
      base = size_t(tr) * g_b;
    }
    __nv_bfloat16* dst = (which == 0 ? dq_s : dq_c) + base + (bh_ % H) * g_h + c * 8;
    *reinterpret_cast<float4*>(lo) = *reinterpret_cast<const float4*>(src);
    *reinterpret_cast<float4*>(lo + 4) = *reinterpret_cast<const float4*>(src + 4);
    *reinterpret_cast<float4*>(hi) = *reinterpret_cast<const float4*>(src + h);
    *reinterpret_cast<float4*>(hi + 4) = *reinterpret_cast<const float4*>(src + h + 4);
    uint4 olo, ohi;
    __nv_bfloat16* olp = reinterpret_cast<__nv_bfloat16*>(&olo);
    __nv_bfloat16* ohp = reinterpret_cast<__nv_bfloat16*>(&ohi);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float a = lo[e], b = hi[e];
      if (which == 0 && cos_tab != nullptr) {  // R^T: dx_lo = dy_lo c + dy_hi s, dx_hi = dy_hi c - dy_lo s
        const float cs = cos_tab[size_t(t) * h + c * 8 + e], sn = sin_tab[size_t(t) * h + c * 8 + e];
        const float na = a * cs + b * sn, nb = b * cs - a * sn;
        a = na;
        b = nb;
      }
      olp[e] = __float2bfloat16_rn(a * scale);
      ohp[e] = __float2bfloat16_rn(b * scale);
    }
    *reinterpret_cast<uint4*>(dst) = olo;
    *reinterpret_cast<uint4*>(dst + h) = ohi;
  }
}

// ------------------------------------------------------------------------------------------------ main kernel
template <int D>
struct BwdCfg {
  static constexpr int kRowBytes = 2 * D;
  static constexpr int kTileBytes = kBwdTile * kRowBytes;       // K, V, Q_i, dO_i tiles
  static constexpr int kDsBlock = kBwdTile * 128;               // one half (64 queries) of dS: [128 key rows][128 B]
  static constexpr int kDsBytes = 2 * kDsBlock;
  // One CTA per SM, 16 compute warps, all 512 TMEM columns: dK, dV, two dQ tiles, then two (head_dim 64) or three
  // (head_dim <= 32) buffers of {S^T half (64 columns), dP^T half (64 columns)}; the third buffer lets the products run
  // two halves ahead of the compute warps.
  static constexpr int kCW = 16;                                // compute warps
  static constexpr int kThreads = 128 + 32 * kCW;
  static constexpr int kNBuf = D <= 32 ? 3 : 2;
  static constexpr int kNDq = 2;                                // dQ tiles in TMEM == dS tiles in shared memory
  static constexpr int kQStages = D <= 32 ? 3 : 2;              // stages of {Q_i, dO_i}
  static constexpr int kAcc = D <= 32 ? 32 : 64;                // columns reserved per accumulator
  static constexpr int kColDK = 0, kColDV = kAcc, kColDQ = 2 * kAcc, kColBuf = (2 + kNDq) * kAcc;
  static constexpr uint32_t kTmemCols = 512;
  static constexpr int kVPG = 16 / kCW;                         // 16-column query groups per thread and half
  static constexpr int kDqWarpBytes = 32 * (D / 4) * 4;          // staging of one warp's dQ slice: 32 queries x D/4 fp32 columns
  static constexpr int kDqStageBytes = kCW * kDqWarpBytes;
  static constexpr int kStatBytes = 128 * 8;                     // softmax statistics of one query tile: 128 x (-lse log2 e, -delta)
  static constexpr size_t kSmemBytes =
      1024 + 2 * kTileBytes + size_t(kQStages) * 2 * kTileBytes + size_t(kNDq) * kDsBytes + kDqStageBytes + kQStages * kStatBytes + 4096;
};

struct BwdParams {
  const uint32_t *bitsT, *kpad;
  const uint8_t* cls;
  const float2* stats;             // [B*H][Tpad / 2] x (nl0, nl1, nd0, nd1): -lse * log2 e and -delta of two queries, Tpad = T rounded up to 128
  const float *cos_tab, *sin_tab;  // null without rope
  float* dq_acc[2];                // fp32 [B*H][T][D] per pathway
  __nv_bfloat16 *dk[2], *dv[2];
  int H, T, Tpad, TW, NT;
  float scale, scale_log2;
  int* status;
  int do_seq_first;                // dO is laid out (T,B,H,D): its tensor map takes (0, bh, t) instead of (0, t, bh)
  int skip_pad_queries;            // query tiles that hold only padded positions are left out
  size_t g_row, g_b, g_h;          // element strides of dk / dv: between keys, batch entries, heads
  const int32_t* token_row;        // row of the row-major gradient matrices per token t * B + b (negative: none), or null
  int B;
};

// ring counter with phase bit: position in [0, N), phase flips on wrap
template <int N>
struct Ring {
  uint32_t pos = 0, phase = 0;
  __device__ __forceinline__ void advance() {
    if (++pos == N) { pos = 0; phase ^= 1; }
  }
};

template <int D, bool SQ>
__global__ void __launch_bounds__(BwdCfg<D>::kThreads, 1)
attn_bwd_tc_kernel(const __grid_constant__ CUtensorMap map_qs, const __grid_constant__ CUtensorMap map_ks,
                   const __grid_constant__ CUtensorMap map_vs, const __grid_constant__ CUtensorMap map_qc,
                   const __grid_constant__ CUtensorMap map_kc, const __grid_constant__ CUtensorMap map_vc,
                   const __grid_constant__ CUtensorMap map_do, const __grid_constant__ CUtensorMap map_dq_s,
                   const __grid_constant__ CUtensorMap map_dq_c, BwdParams p) {
  using Cfg = BwdCfg<D>;
  constexpr int RB = Cfg::kRowBytes, kNBuf = Cfg::kNBuf, kQStages = Cfg::kQStages, kNDq = Cfg::kNDq, kVPG = Cfg::kVPG;
  constexpr int kBwdThreads = Cfg::kThreads, kComputeThreads = 32 * Cfg::kCW;
  constexpr int kColDK = Cfg::kColDK, kColDV = Cfg::kColDV, kColDQ = Cfg::kColDQ, kColBuf = Cfg::kColBuf, kAcc = Cfg::kAcc;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sK = smem;
  unsigned char* sV = sK + Cfg::kTileBytes;
  unsigned char* sQ = sV + Cfg::kTileBytes;                          // [stage][0: Q_i, 1: dO_i]
  unsigned char* sDS = sQ + size_t(kQStages) * 2 * Cfg::kTileBytes;  // [buf][half][128 rows x 128 B]
  unsigned char* sDqStage = sDS + size_t(kNDq) * Cfg::kDsBytes;      // [compute warp][32 queries][D/4 fp32], swizzled
  unsigned char* sStats = sDqStage + Cfg::kDqStageBytes;             // [stage][64] x (nl0, nl1, nd0, nd1), loaded with the query tile
  unsigned char* tail = sStats + size_t(kQStages) * Cfg::kStatBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(tail);
  uint64_t* kv_full = bars;            // 1
  uint64_t* acc_full = bars + 1;       // 1
  uint64_t* q_full = bars + 2;         // [3]
  uint64_t* q_empty = bars + 5;        // [3]
  uint64_t* sdp_full = bars + 8;       // [3 buffers]
  uint64_t* pds_full = bars + 11;      // [3 buffers]
  uint64_t* buf_free = bars + 14;      // [3 buffers]
  uint64_t* dq_full = bars + 17;       // [2]
  uint64_t* dq_empty = bars + 19;      // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);
  uint8_t* tq = reinterpret_cast<uint8_t*>(tmem_slot + 2);  // per query tile: 0 skip, else 1 | (needs chain mask) << 1 | (pad) << 2

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int kt = blockIdx.x, bh = blockIdx.y, path = blockIdx.z, b = bh / p.H;
  const int k0 = kt * kBwdTile;
  const int nqt = (p.T + kBwdTile - 1) / kBwdTile;
  const uint8_t want = path == 0 ? kHasIntra : kHasInter;

  const CUtensorMap* mq = path == 0 ? &map_qs : &map_qc;
  const CUtensorMap* mk = path == 0 ? &map_ks : &map_kc;
  const CUtensorMap* mv = path == 0 ? &map_vs : &map_vc;

  // the gradients of a key tile without a single pair of this pathway are zero
  auto write_zero_gradients = [&]() {
    for (int idx = tid; idx < kBwdTile * (D / 8); idx += kBwdThreads) {
      const int row = idx / (D / 8), vec = idx % (D / 8);
      if (k0 + row < p.T) {
        size_t base = size_t(k0 + row) * p.g_row + size_t(b) * p.g_b;
        if (p.token_row != nullptr) {
          const int tr = __ldg(p.token_row + size_t(k0 + row) * p.B + b);
          if (tr < 0) continue;
          base = size_t(tr) * p.g_b;
        }
        const size_t off = base + size_t(bh % p.H) * p.g_h + vec * 8;
        *reinterpret_cast<uint4*>(p.dk[path] + off) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(p.dv[path] + off) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  };
  // Every key of the tile padded (padded batches have many such tiles): leave before any barrier, TMEM or copy is set up.
  {
    const uint32_t* w = p.kpad + size_t(b) * p.TW + 4 * kt;
    if ((w[0] & w[1] & w[2] & w[3]) == 0xffffffffu) {   // uniform over the CTA
      write_zero_gradients();
      return;
    }
  }
  if (tid == 0) {
    mbar_init(kv_full, 1);
    mbar_init(acc_full, 2);
    for (int s = 0; s < 3; ++s) {
      mbar_init(&q_full[s], 1); mbar_init(&q_empty[s], 2);      // released by the dV and the dK stream
      mbar_init(&sdp_full[s], 1); mbar_init(&pds_full[s], kComputeThreads);
      mbar_init(&buf_free[s], 2);                                // dV and dK of a half have read P^T, dS^T
    }
    for (int s = 0; s < 2; ++s) { mbar_init(&dq_full[s], 1); mbar_init(&dq_empty[s], kComputeThreads); }
    fence_mbar_init();
    // K and V of the tile do not depend on the query-tile scan below: their copies run while it does
    prefetch_tensormap(mk); prefetch_tensormap(mv);
    mbar_expect_tx(kv_full, 2 * Cfg::kTileBytes);
    tma_load_3d(sK, mk, kv_full, 0, k0, bh);
    tma_load_3d(sV, mv, kv_full, 0, k0, bh);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, Cfg::kTmemCols); tmem_relinquish(); }

  int any_active = 0;
  uint8_t my_flag = 0;   // flag of query tile `tid` (the loop below runs at most once per thread: nqt <= kBwdMaxTiles < kBwdThreads)
  for (int i = tid; i < nqt; i += kBwdThreads) {
    uint8_t c = 0;
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
      for (int e = 0; e < 2; ++e)
        if (2 * i + a < p.NT && 2 * kt + e < p.NT) c |= p.cls[(size_t(b) * p.NT + 2 * i + a) * p.NT + 2 * kt + e];
    uint8_t f = 0;
    if (c & want) f = 1 | (((c & 3) == 3) ? 2 : 0) | ((c & kHasPad) ? 4 : 0);
    if (p.skip_pad_queries) {   // the padding bits describe positions: words 4 i .. 4 i + 3 cover the queries of tile i
      const uint32_t* w = p.kpad + size_t(b) * p.TW + 4 * i;
      if ((w[0] & w[1] & w[2] & w[3]) == 0xffffffffu) f = 0;
    }
    tq[i] = f;
    any_active |= f;
    my_flag = f;
  }
  // The first query tile's Q and dO do not wait for the CTA-wide barrier below: warp 0 holds the flags of tiles 0..31 and
  // requests the first tile with work among them at once (the copy of its statistics follows after the wait for the pass
  // before this kernel).  A TMA round trip is about as long as the whole set-up, so the first products start that much
  // earlier.  Warp 0 remembers the tile; its loading loop then skips these two copies.
  int early_q = -1;
  if (warp == 0) {
    const unsigned act = __ballot_sync(0xffffffffu, my_flag != 0);
    if (act != 0u) {
      early_q = __ffs(act) - 1;
      if (lane == 0) {   // the thread that initialised the barriers
        prefetch_tensormap(mq); prefetch_tensormap(&map_do);
        mbar_expect_tx(&q_full[0], 2 * Cfg::kTileBytes + Cfg::kStatBytes);
        tma_load_3d(sQ, mq, &q_full[0], 0, early_q * kBwdTile, bh);
        if (p.do_seq_first) tma_load_3d(sQ + Cfg::kTileBytes, &map_do, &q_full[0], 0, bh, early_q * kBwdTile);
        else tma_load_3d(sQ + Cfg::kTileBytes, &map_do, &q_full[0], 0, early_q * kBwdTile, bh);
      }
    }
  }
  tc_fence_before();
  any_active = __syncthreads_or(any_active);
  tc_fence_after();
  // Up to here nothing that the pass before this kernel writes (the statistics, the cleared dQ accumulators) has been
  // touched, so all of it may overlap that pass; from here on it has to be complete.  The pass after this kernel (the dQ
  // conversion) may be scheduled once every CTA has come this far; it waits for the whole grid itself.
  griddep_wait();
  if (tid == 0) griddep_launch();
  const uint32_t tbase = *tmem_slot;
  if (any_active == 0) {
    // no query tile holds a pair of this pathway (every query on the other side of the mask): zero gradients; the copies of
    // K and V must have landed and TMEM must be given back before the CTA leaves
    write_zero_gradients();
    if (tid == 0) mbar_wait(kv_full, 0, p.status, 0x500);
    __syncthreads();
    if (warp == 1) {
      __syncwarp();
      tmem_dealloc(tbase, Cfg::kTmemCols);
    }
    return;
  }
  int n_active = 0;
  for (int i = 0; i < nqt; ++i) n_active += tq[i] != 0;
  n_active = __shfl_sync(0xffffffffu, n_active, 0);   // the same in every thread; the shuffle lets the compiler know it
  // The MMA warps below run their loops with all lanes and let one elected lane issue: with warp-uniform control flow and
  // operands the descriptors stay in uniform registers, which is what tcgen05.mma reads; issued from a divergent single-lane
  // region every instruction first has to move its operands there.
  auto wait_all = [&](uint64_t* bar, uint32_t parity, int code) -> bool {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity, p.status, code));
  };
  const uint32_t tbase_u = __shfl_sync(0xffffffffu, tbase, 0);
  const int n_sub = 2 * n_active;   // 64-query halves, numbered u = 2 * tile + half; half u lives in buffer u % kNBuf

  if (warp == 1) {
    // ---------------------------------------------------------------- MMA stream A: S^T = K Q^T and dP^T = V dO^T
    // Issuing one tcgen05.mma costs its thread some 50 cycles whatever the tile size, and at small head sizes the
    // products are tiny, so the four families of products are issued by four warps in parallel (disjoint accumulators).
    if (n_active > 0) {
      const bool leader = elect_one();
      constexpr uint32_t idesc_s = idesc_bf16(kBwdTile, kHalf, false, false);   // M = 128 keys, N = 64 queries
      constexpr uint32_t kHi = desc_hi32(8 * RB, swizzle_for_row_bytes(RB));
      constexpr uint32_t kLbo = desc_lbo32(16);
      const uint32_t k_lo = desc_addr32(__shfl_sync(0xffffffffu, smem_u32(sK), 0)) + kLbo;
      const uint32_t v_lo = desc_addr32(__shfl_sync(0xffffffffu, smem_u32(sV), 0)) + kLbo;
      const uint32_t q_lo = desc_addr32(__shfl_sync(0xffffffffu, smem_u32(sQ), 0)) + kLbo;
      constexpr uint32_t kTileU = Cfg::kTileBytes >> 4, kHalfU = (kHalf * RB) >> 4;
      bool ok = wait_all(kv_full, 0, 0x501);
      Ring<kQStages> qr;     // query tile of the half being issued
      Ring<kNBuf> ib;        // buffer of the half being issued
      Ring<kNBuf> wb;        // buffer whose release is awaited next
      auto issue_sdp = [&](int u) -> bool {   // both products of half u
        const int h = u & 1;
        if (h == 0 && !wait_all(&q_full[qr.pos], qr.phase, 0x502)) return false;
        tc_fence_after();
        const uint32_t qs = q_lo + qr.pos * 2 * kTileU + h * kHalfU;
        const uint32_t dos = qs + kTileU;
        const uint32_t col = tbase_u + kColBuf + ib.pos * 128;
        if (leader) {
#pragma unroll
          for (int k = 0; k < D / 16; ++k) umma_ss(col, make_desc(kHi, k_lo + 2 * k), make_desc(kHi, qs + 2 * k), idesc_s, k > 0);
#pragma unroll
          for (int k = 0; k < D / 16; ++k) umma_ss(col + 64, make_desc(kHi, v_lo + 2 * k), make_desc(kHi, dos + 2 * k), idesc_s, k > 0);
          umma_commit(&sdp_full[ib.pos]);
        }
        __syncwarp();
        ib.advance();
        if (h == 1) qr.advance();
        return true;
      };
      int issued = 0;
      for (; issued < kNBuf && issued < n_sub && ok; ++issued) ok = issue_sdp(issued);
      for (int u = 0; issued < n_sub && ok; ++u, ++issued) {
        ok = wait_all(&buf_free[wb.pos], wb.phase, 0x505);   // dV and dK of half u have consumed P^T, dS^T
        if (!ok) break;
        wb.advance();
        ok = issue_sdp(issued);
      }
    }
  } else if (warp == 2 || warp == 3) {
    // ---------------------------------------------------------------- MMA streams V and K: dV += P^T dO, dK += dS^T Q
    if (n_active > 0) {
      const bool leader = elect_one();
      constexpr uint32_t idesc_acc = idesc_bf16(kBwdTile, D, false, true);      // A from TMEM, B rows of dO / Q (N = D contiguous)
      constexpr uint32_t kHi = desc_hi32(8 * RB, swizzle_for_row_bytes(RB));
      constexpr uint32_t kLbo = desc_lbo32(8 * RB);
      constexpr uint32_t kTileU = Cfg::kTileBytes >> 4, kHalfU = (kHalf * RB) >> 4, kStep = (16 * RB) >> 4;
      const bool is_v = __shfl_sync(0xffffffffu, warp, 0) == 2;
      // dV reads P^T (over S^T) and dO; dK reads dS^T (over dP^T, 64 columns further) and Q
      const uint32_t b_lo = desc_addr32(__shfl_sync(0xffffffffu, smem_u32(sQ), 0)) + kLbo + (is_v ? kTileU : 0u);
      const uint32_t a_col = tbase_u + kColBuf + (is_v ? 0u : 64u);
      const uint32_t d_col = tbase_u + (is_v ? kColDV : kColDK);
      bool ok = true;
      Ring<kQStages> qr;
      Ring<kNBuf> br;
      for (int it = 0; it < n_active && ok; ++it) {
        ok = wait_all(&q_full[qr.pos], qr.phase, 0x511);
        for (int h = 0; h < 2 && ok; ++h) {
          ok = wait_all(&pds_full[br.pos], br.phase, 0x512);
          if (!ok) break;
          tc_fence_after();
          const uint32_t rows = b_lo + qr.pos * 2 * kTileU + h * kHalfU;
          if (leader) {
#pragma unroll
            for (int k = 0; k < kHalf / 16; ++k)
              umma_ts(d_col, a_col + br.pos * 128 + k * 16, make_desc(kHi, rows + k * kStep), idesc_acc, it > 0 || h > 0 || k > 0);
            umma_commit(&buf_free[br.pos]);
          }
          __syncwarp();
          br.advance();
        }
        if (ok && leader) umma_commit(&q_empty[qr.pos]);
        __syncwarp();
        qr.advance();
      }
      if (ok && leader) umma_commit(acc_full);
    }
  } else if (warp == 0) {
    // ---------------------------------------------------------------- TMA loads and MMA stream Q: dQ tile = dS K
    // One thread does both: it loads K, V and the first query tiles, then per tile issues the dQ product and
    // refills the stage that tile has just released with the tile kQStages steps ahead.
    if (n_active > 0) {
      const bool leader = elect_one();
      constexpr uint32_t idesc_dq = idesc_bf16(kBwdTile, D, true, true);        // A = dS (queries contiguous), B = K (D contiguous)
      constexpr uint32_t kHiA = desc_hi32(8 * 128, kSw128), kHiB = desc_hi32(8 * RB, swizzle_for_row_bytes(RB));
      const uint32_t ds_lo = desc_addr32(__shfl_sync(0xffffffffu, smem_u32(sDS), 0)) + desc_lbo32(Cfg::kDsBlock);
      const uint32_t kb_lo = desc_addr32(__shfl_sync(0xffffffffu, smem_u32(sK), 0)) + desc_lbo32(8 * RB);
      constexpr uint32_t kDsU = Cfg::kDsBytes >> 4, kAStep = (16 * 128) >> 4, kBStep = (16 * RB) >> 4;
      if (leader) { prefetch_tensormap(mq); prefetch_tensormap(&map_do); }      // (K and V were requested before the query-tile scan)
      int next_q = 0;        // next query tile index to look at (the elected lane's copy is the one that counts)
      Ring<kQStages> lr;     // stage the next load goes to (likewise)
      auto load_next = [&]() {   // issue the loads of the next active query tile; called by the elected lane only
        while (next_q < nqt && tq[next_q] == 0) ++next_q;
        if (next_q >= nqt) return;
        unsigned char* dst = sQ + size_t(lr.pos) * 2 * Cfg::kTileBytes;
        const bool early = next_q == early_q;   // Q and dO of this tile (the first one, stage 0) were requested during the set-up
        if (!early) mbar_expect_tx(&q_full[lr.pos], 2 * Cfg::kTileBytes + Cfg::kStatBytes);
        bulk_load_1d(sStats + size_t(lr.pos) * Cfg::kStatBytes, p.stats + size_t(bh) * p.Tpad + size_t(next_q) * kBwdTile,
                     Cfg::kStatBytes, &q_full[lr.pos]);
        if (!early) {
          tma_load_3d(dst, mq, &q_full[lr.pos], 0, next_q * kBwdTile, bh);
          if (p.do_seq_first) tma_load_3d(dst + Cfg::kTileBytes, &map_do, &q_full[lr.pos], 0, bh, next_q * kBwdTile);
          else tma_load_3d(dst + Cfg::kTileBytes, &map_do, &q_full[lr.pos], 0, next_q * kBwdTile, bh);
        }
        ++next_q;
        lr.advance();
      };
      if (leader) {
        for (int s = 0; s < kQStages; ++s) load_next();
      }
      __syncwarp();
      bool ok = wait_all(kv_full, 0, 0x521);
      Ring<kNBuf> br;        // buffers of the two halves of the tile
      Ring<kQStages> er;     // stage released by the tile
      for (int it = 0; it < n_active && ok; ++it) {
        ok = wait_all(&pds_full[br.pos], br.phase, 0x522);
        br.advance();
        if (ok) ok = wait_all(&pds_full[br.pos], br.phase, 0x523);
        br.advance();
        if (ok) ok = wait_all(&dq_empty[it % kNDq], ((it / kNDq) & 1) ^ 1, 0x524);   // buffer drained kNDq tiles ago
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_lo = ds_lo + uint32_t(it % kNDq) * kDsU;
        if (leader) {
#pragma unroll
          for (int k = 0; k < kBwdTile / 16; ++k)
            umma_ss(tbase_u + kColDQ + (it % kNDq) * kAcc, make_desc(kHiA, a_lo + k * kAStep), make_desc(kHiB, kb_lo + k * kBStep), idesc_dq, k > 0);
          umma_commit(&dq_full[it % kNDq]);
        }
        __syncwarp();
        if (it + kQStages < n_active) {   // this tile's stage is released by its dV and dK streams
          ok = wait_all(&q_empty[er.pos], er.phase, 0x525);
          if (ok && leader) load_next();
          __syncwarp();
        }
        er.advance();
      }
    }
  } else {
    // ---------------------------------------------------------------- compute warps (lane = key row)
    // 16 warps work on ONE 64-query half at a time: thread = key row x 16 query columns (group grp = 0..3).  The
    // products run up to kNBuf halves ahead, and groups 2,3 start a fraction of a half later than groups 0,1 so that the
    // exp2-heavy part of one pair of groups overlaps the TMEM traffic and barrier work of the other.
    // Everything here is elementwise: no exchange between threads.
    const int cwp = warp - 4;                     // 0..kCW-1
    const int grp = cwp / 4;                      // physical group; it covers the 16-column groups vg = grp * kVPG + v
    const int quarter = warp % 4;
    const int r = quarter * 32 + lane;            // key row in the tile == TMEM lane
    const int kj = k0 + r;
    const int krow = kj < p.T ? kj : p.T - 1;
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    const uint32_t tBuf = tbase + lane_base + kColBuf;   // + 128 * buffer + 16 * vg: S^T columns of this thread; dP^T 64 further
    const bool key_valid = kj < p.T && !((p.kpad[size_t(b) * p.TW + krow / 32] >> (krow % 32)) & 1u);
    const uint32_t* mrow = p.bitsT + (size_t(b) * p.T + krow) * p.TW;
    const uint32_t flip = path == 0 ? 0xffffu : 0u;   // keep-bit = mask bit XOR flip
    const uint64_t c22 = pack2(p.scale_log2, p.scale_log2);
    bool ok = true;
    int it = 0;
    Ring<kNBuf> br;
    Ring<kQStages> sr;     // stage that holds the current tile's statistics

    // dQ of a tile leaves through shared memory: each compute warp stages its 32 queries x NC columns and one lane adds
    // them to the fp32 accumulator in HBM with ONE bulk reduction (instead of a 16-byte atomic per thread and 4 columns).
    const CUtensorMap* mdq = path == 0 ? &map_dq_s : &map_dq_c;
    unsigned char* my_stage = sDqStage + size_t(cwp) * Cfg::kDqWarpBytes;
    auto drain_dq = [&](int jt, int qtile) -> bool {   // add dQ of active tile jt (query tile qtile) to HBM
      if (!mbar_wait(&dq_full[jt % kNDq], (jt / kNDq) & 1, p.status, 0x601)) return false;
      tc_fence_after();
      constexpr int NC = D / 4 * kVPG;   // columns per thread
      constexpr int kRowB = NC * 4;      // bytes per staged row: 64, 32 or 16
      uint32_t v[NC];
      tmem_ld_n<NC>(tbase + lane_base + kColDQ + (jt % kNDq) * kAcc + grp * NC, v);
      if (lane == 0) bulk_wait_read_all();   // the previous reduction of this warp has read the staging rows
      __syncwarp();
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&dq_empty[jt % kNDq]);
#pragma unroll
      for (int e = 0; e < NC; e += 4) {
        const uint32_t off = kRowB == 16 ? uint32_t(lane) * 16u : swizzled_offset(lane, e / 4, kRowB);
        *reinterpret_cast<uint4*>(my_stage + off) = make_uint4(v[e], v[e + 1], v[e + 2], v[e + 3]);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0 && qtile * kBwdTile + quarter * 32 < p.T) {   // rows past T inside the box are dropped by the copy engine
        tma_reduce_add_3d(mdq, my_stage, grp * NC, qtile * kBwdTile + quarter * 32, bh);
        bulk_commit_group();
      }
      return true;
    };

    int prev_tile = -1;
    for (int i = 0; i < nqt && ok; ++i) {
      const uint8_t f = tq[i];
      if (f == 0) continue;
      // mask bits of the tile for this key row: half `sub`, 16-column group vg -> word 2 sub + vg / 2, bits 16 (vg & 1)...
#pragma unroll 1
      for (int sub = 0; sub < 2 && ok; ++sub) {
        ok = mbar_wait(&sdp_full[br.pos], br.phase, p.status, 0x602);
        if (!ok) break;
        if (sub == 0) {   // the tile's loads have landed long ago (its products are done): this only orders the reads below
          ok = mbar_wait(&q_full[sr.pos], sr.phase, p.status, 0x604);
          if (!ok) break;
        }
        if (it == 0 && sub == 0 && grp >= 2) __nanosleep(kBwdStaggerNs);
        tc_fence_after();
        unsigned char* ds_row = sDS + size_t(it % kNDq) * Cfg::kDsBytes + size_t(sub) * Cfg::kDsBlock;
#pragma unroll
        for (int v = 0; v < kVPG; ++v) {
          const int vg = grp * kVPG + v;
          // statistics of this thread's 16 queries, from the copy that arrived in shared memory with the query tile
          const float4* st = reinterpret_cast<const float4*>(sStats + size_t(sr.pos) * Cfg::kStatBytes) + (sub * kHalf + 16 * vg) / 2;
          float4 sq[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) sq[j] = st[j];
          uint32_t keep = 0xffffu;
          if (f & 2) keep = ((__ldg(mrow + 4 * i + 2 * sub + vg / 2) >> (16 * (vg & 1))) & 0xffffu) ^ flip;
          if (!key_valid) keep = 0u;
          const bool all = keep == 0xffffu;
          const uint32_t tS = tBuf + br.pos * 128 + 16 * vg;
          uint32_t sv[16], dpv[16];
          tmem_ld16(tS, sv);
          tmem_ld16(tS + 64, dpv);
          tmem_ld_wait();
          uint32_t pp[8], dd[8];
#pragma unroll
          for (int j = 0; j < 16; j += 2) {
            const float4 q2 = sq[j / 2];   // (nl0, nl1, nd0, nd1)
            float p0, p1;
            unpack2(ffma2(pack2(__uint_as_float(sv[j]), __uint_as_float(sv[j + 1])), c22, pack2(q2.x, q2.y)), p0, p1);
            p0 = bwd_ex2(p0);
            p1 = bwd_ex2(p1);
            if (!all) {
              if (!((keep >> j) & 1u)) p0 = 0.f;
              if (!((keep >> (j + 1)) & 1u)) p1 = 0.f;
            }
            float d0, d1;
            const uint64_t p2 = pack2(p0, p1), dp2 = pack2(__uint_as_float(dpv[j]), __uint_as_float(dpv[j + 1])), nd2 = pack2(q2.z, q2.w);
            if (SQ)   // r = sqrt(p) is what p0, p1 hold: dS = r (dP / 2 - r delta / 2), and r itself multiplies dO in dV
              unpack2(fmul2(p2, ffma2(p2, nd2, fmul2(dp2, pack2(0.5f, 0.5f)))), d0, d1);
            else      // dS = p (dP - delta)
              unpack2(fmul2(p2, fadd2(dp2, nd2)), d0, d1);
            pp[j / 2] = bwd_pack(p0, p1);
            dd[j / 2] = bwd_pack(d0, d1);
          }
          tmem_st8(tS, pp);         // P^T over the S^T columns this thread has read
          tmem_st8(tS + 64, dd);    // dS^T likewise
          // and dS into shared memory for the dQ product: 2 chunks of 8 queries in block `sub` of the dS tile
          *reinterpret_cast<uint4*>(ds_row + swizzled_offset(r, 2 * vg, 128)) = make_uint4(dd[0], dd[1], dd[2], dd[3]);
          *reinterpret_cast<uint4*>(ds_row + swizzled_offset(r, 2 * vg + 1, 128)) = make_uint4(dd[4], dd[5], dd[6], dd[7]);
        }
        tmem_st_wait();
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(&pds_full[br.pos]);
        br.advance();
      }
      if (!ok) break;
      if (prev_tile >= 0) ok = drain_dq(it - 1, prev_tile);
      prev_tile = i;
      sr.advance();
      ++it;
    }
    if (ok && prev_tile >= 0) ok = drain_dq(it - 1, prev_tile);
    if (lane == 0) bulk_wait_read_all();   // the reductions have read their staging rows (their additions may still be under way)

    // ---- epilogue: 16-column groups vg 0,1 write the two column halves of dK (scaled, un-rotated for the self pathway),
    //      vg 2,3 those of dV
    if (n_active > 0) {
      if (ok) ok = mbar_wait(acc_full, 0, p.status, 0x603);
      tc_fence_after();
    }
    ok = __all_sync(0xffffffffu, ok);   // the stores below exchange rows between the lanes of the warp
    if (ok) {
      constexpr int hD = D / 2;
      constexpr int kPieces = hD / 8;   // 16-byte pieces of a thread's half row: 4, 2 or 1
      if (kPieces > 1) {                // the staging rows of the dQ reductions are reused below
        if (lane == 0) bulk_wait_read_all();
        __syncwarp();
      }
#pragma unroll
      for (int v = 0; v < kVPG; ++v) {
        const int vg = grp * kVPG + v;
        const bool is_dk = vg < 2;
        const int half_col = vg & 1;
        float lo[hD], hi[hD];   // lower / upper half of the row (dK needs both for the rotation; dV only its own)
        if (n_active > 0) {
          const uint32_t src = tbase + lane_base + (is_dk ? kColDK : kColDV);
          uint32_t t0[hD], t1[hD];
          if (is_dk || half_col == 0) tmem_ld_n<hD>(src, t0);
          if (is_dk || half_col == 1) tmem_ld_n<hD>(src + hD, t1);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < hD; ++j) { lo[j] = __uint_as_float(t0[j]); hi[j] = __uint_as_float(t1[j]); }
        } else {
#pragma unroll
          for (int j = 0; j < hD; ++j) lo[j] = hi[j] = 0.f;
        }
        // element offset of this thread's half row in dk / dv, negative when the key has no row (past T, or dropped token)
        long long row_off = -1;
        if (kj < p.T) {
          row_off = static_cast<long long>(size_t(kj) * p.g_row + size_t(b) * p.g_b);
          if (p.token_row != nullptr) {
            const int tr = __ldg(p.token_row + size_t(kj) * p.B + b);
            row_off = tr < 0 ? -1 : static_cast<long long>(size_t(tr) * p.g_b);
          }
          if (row_off >= 0) row_off += static_cast<long long>(size_t(bh % p.H) * p.g_h + half_col * hD);
        }
        float outv[hD];
        if (is_dk) {
          const bool rot = path == 0 && p.cos_tab != nullptr;
          if (rot) {   // R^T: dx_lo = dy_lo c + dy_hi s, dx_hi = dy_hi c - dy_lo s; table rows read 16 bytes at a time
            const float4* c4 = reinterpret_cast<const float4*>(p.cos_tab + size_t(krow) * hD);
            const float4* s4 = reinterpret_cast<const float4*>(p.sin_tab + size_t(krow) * hD);
#pragma unroll
            for (int d = 0; d < hD; d += 4) {
              const float4 cs = __ldg(c4 + d / 4), sn = __ldg(s4 + d / 4);
              const float cv[4] = {cs.x, cs.y, cs.z, cs.w}, sv4[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
              for (int e = 0; e < 4; ++e)
                outv[d + e] = (half_col == 0 ? lo[d + e] * cv[e] + hi[d + e] * sv4[e] : hi[d + e] * cv[e] - lo[d + e] * sv4[e]) * p.scale;
            }
          } else {
#pragma unroll
            for (int d = 0; d < hD; ++d) outv[d] = (half_col == 0 ? lo[d] : hi[d]) * p.scale;
          }
        } else {
#pragma unroll
          for (int d = 0; d < hD; ++d) outv[d] = half_col == 0 ? lo[d] : hi[d];
        }
        __nv_bfloat16* base = is_dk ? p.dk[path] : p.dv[path];
        if constexpr (kPieces == 1) {
          if (row_off >= 0)
            *reinterpret_cast<uint4*>(base + row_off) = make_uint4(bwd_pack(outv[0], outv[1]), bwd_pack(outv[2], outv[3]),
                                                                   bwd_pack(outv[4], outv[5]), bwd_pack(outv[6], outv[7]));
        } else {
          // Rows of different keys lie far apart (row-major gradients) or 2 hD elements apart: staged per warp and read back
          // so that kPieces neighbouring lanes write one row's contiguous 16 hD bytes, a store instruction covers whole runs.
          constexpr int kRowB = hD * 2;   // 64 or 32 bytes
#pragma unroll
          for (int j = 0; j < hD; j += 8)
            *reinterpret_cast<uint4*>(my_stage + swizzled_offset(lane, j / 8, kRowB)) =
                make_uint4(bwd_pack(outv[j], outv[j + 1]), bwd_pack(outv[j + 2], outv[j + 3]), bwd_pack(outv[j + 4], outv[j + 5]),
                           bwd_pack(outv[j + 6], outv[j + 7]));
          __syncwarp();
          const int piece = lane % kPieces;
#pragma unroll
          for (int i = 0; i < kPieces; ++i) {
            const int r = i * (32 / kPieces) + lane / kPieces;
            const long long ro = __shfl_sync(0xffffffffu, row_off, r);
            const uint4 q = *reinterpret_cast<const uint4*>(my_stage + swizzled_offset(r, piece, kRowB));
            if (ro >= 0) *reinterpret_cast<uint4*>(base + ro + piece * 8) = q;
          }
          __syncwarp();
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tbase, Cfg::kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------------ host side
static size_t bwd_rot_bytes(int B, int H, int T, int D) { return align256(size_t(B) * H * T * D * 2); }
static size_t bwd_acc_bytes(int B, int H, int T, int D) { return align256(size_t(B) * H * T * D * 4); }
static int bwd_tpad(int T) { return (T + kBwdTile - 1) / kBwdTile * kBwdTile; }
static size_t bwd_stats_bytes(int B, int H, int T) { return align256(size_t(B) * H * bwd_tpad(T) * 8); }

// Workspace: [rotated Q_self | rotated K_self] (rope only) | stats | dQ accumulator self | dQ accumulator cross
size_t tc_bwd_workspace_bytes(int B, int H, int T, int D, bool rope) {
  return (rope ? 2 * bwd_rot_bytes(B, H, T, D) : 0) + bwd_stats_bytes(B, H, T) + 2 * bwd_acc_bytes(B, H, T, D);
}

void launch_rope_rotate(const AttnArgs& a, __nv_bfloat16* qr, __nv_bfloat16* kr);  // attn_tc.cu

template <int D, bool SQ>
static int bwd_tc_t(const AttnArgs& a, const void* q_s, const void* k_s, const float2* stats, float* acc_s, float* acc_c) {
  using Cfg = BwdCfg<D>;
  const int BH = a.B * a.H;
  CUtensorMap mqs, mks, mvs, mqc, mkc, mvc, mdo;
  if (!bwd_make_map(&mqs, q_s, D, a.T, BH, kBwdTile) || !bwd_make_map(&mks, k_s, D, a.T, BH, kBwdTile) ||
      !bwd_make_map(&mvs, a.v_s, D, a.T, BH, kBwdTile) || !bwd_make_map(&mqc, a.q_c, D, a.T, BH, kBwdTile) ||
      !bwd_make_map(&mkc, a.k_c, D, a.T, BH, kBwdTile) || !bwd_make_map(&mvc, a.v_c, D, a.T, BH, kBwdTile) ||
      !bwd_make_map(&mdo, a.d_out, D, a.T, BH, kBwdTile, a.out_seq_first)) {
    set_error("mintb_attn_bwd: cuTensorMapEncodeTiled failed");
    return MINTB_ECUDA;
  }
  CUtensorMap mdq_s, mdq_c;
  if (!bwd_make_dq_map(&mdq_s, acc_s, D, a.T, BH) || !bwd_make_dq_map(&mdq_c, acc_c, D, a.T, BH)) {
    set_error("mintb_attn_bwd: cuTensorMapEncodeTiled failed for the dQ accumulators");
    return MINTB_ECUDA;
  }
  cudaError_t e = cudaFuncSetAttribute(attn_bwd_tc_kernel<D, SQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(Cfg::kSmemBytes));
  if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return MINTB_ECUDA; }
  BwdParams p{};
  p.bitsT = a.meta.bitsT; p.kpad = a.meta.kpad; p.cls = a.meta.cls;
  p.stats = stats;
  p.cos_tab = a.rope ? a.rope_cos : nullptr;
  p.sin_tab = a.rope ? a.rope_sin : nullptr;
  p.dq_acc[0] = acc_s; p.dq_acc[1] = acc_c;
  p.dk[0] = static_cast<__nv_bfloat16*>(a.dk_s); p.dk[1] = static_cast<__nv_bfloat16*>(a.dk_c);
  p.dv[0] = static_cast<__nv_bfloat16*>(a.dv_s); p.dv[1] = static_cast<__nv_bfloat16*>(a.dv_c);
  p.H = a.H; p.T = a.T; p.Tpad = bwd_tpad(a.T); p.TW = a.meta.TW; p.NT = a.meta.NT;
  p.scale = a.scale;
  p.scale_log2 = a.scale * kLog2e * (SQ ? 0.5f : 1.f);   // multiplies the logits inside exp2
  p.status = a.dev_status;
  p.do_seq_first = a.out_seq_first ? 1 : 0;
  p.skip_pad_queries = a.skip_pad_queries ? 1 : 0;
  p.g_row = grad_row_stride(a); p.g_b = grad_b_stride(a); p.g_h = grad_h_stride(a);
  p.token_row = a.token_row; p.B = a.B;
  dim3 grid((a.T + kBwdTile - 1) / kBwdTile, BH, 2);
  e = launch_dependent(attn_bwd_tc_kernel<D, SQ>, grid, dim3(Cfg::kThreads), Cfg::kSmemBytes, a.stream, mqs, mks, mvs, mqc, mkc, mvc, mdo, mdq_s, mdq_c, p);
  count_launches(1);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("attention backward launch: %s", cudaGetErrorString(e)); return MINTB_ECUDA; }
  return MINTB_OK;
}

int launch_attn_bwd_tc(const AttnArgs& a) {
  if ((a.T + kBwdTile - 1) / kBwdTile > kBwdMaxTiles) { set_error("mintb_attn_bwd: T = %d is too long", a.T); return MINTB_EUNSUPPORTED; }
  char* ws = static_cast<char*>(a.workspace);
  const void* q_s = a.q_s;
  const void* k_s = a.k_s;
  const size_t rows = size_t(a.B) * a.H * a.T;
  if (a.rope && !a.qk_prerotated) {
    __nv_bfloat16* qr = reinterpret_cast<__nv_bfloat16*>(ws);
    __nv_bfloat16* kr = reinterpret_cast<__nv_bfloat16*>(ws + bwd_rot_bytes(a.B, a.H, a.T, a.D));
    if (!a.rot_saved) launch_rope_rotate(a, qr, kr);
    q_s = qr;
    k_s = kr;
    ws += 2 * bwd_rot_bytes(a.B, a.H, a.T, a.D);
  }
  float2* stats = reinterpret_cast<float2*>(ws);
  ws += bwd_stats_bytes(a.B, a.H, a.T);
  float* acc_s = reinterpret_cast<float*>(ws);
  float* acc_c = reinterpret_cast<float*>(ws + bwd_acc_bytes(a.B, a.H, a.T, a.D));
  {
    const int tpad = bwd_tpad(a.T);
    const size_t n = size_t(a.B) * a.H * tpad * (a.D / 8);
    bwd_stats_kernel<<<unsigned((n + 255) / 256), 256, 0, a.stream>>>(static_cast<const __nv_bfloat16*>(a.out),
                                                                     static_cast<const __nv_bfloat16*>(a.d_out), a.lse, stats,
                                                                     a.B * a.H, a.T, tpad, a.D, a.sqrt_softmax ? 0.5f : 1.f, out_row_stride(a),
                                                                     out_bh_stride(a), acc_s, acc_c);
    count_launches(1);
  }
  int rc = MINTB_EUNSUPPORTED;
  switch (a.D) {
#define MINTB_BWD_CASE(DD)                                                                                       \
  case DD:                                                                                                       \
    rc = a.sqrt_softmax ? bwd_tc_t<DD, true>(a, q_s, k_s, stats, acc_s, acc_c) : bwd_tc_t<DD, false>(a, q_s, k_s, stats, acc_s, acc_c); \
    break;
    MINTB_BWD_CASE(16)
    MINTB_BWD_CASE(32)
    MINTB_BWD_CASE(64)
#undef MINTB_BWD_CASE
    default: set_error("mintb_attn_bwd: unsupported head_dim %d", a.D);
  }
  if (rc != MINTB_OK) return rc;
  {
    const size_t n = rows * (a.D / 16);
    cudaError_t le = launch_dependent(bwd_dq_convert_kernel, dim3(unsigned((n + 255) / 256)), dim3(256), 0, a.stream,
        acc_s, acc_c, static_cast<__nv_bfloat16*>(a.dq_s), static_cast<__nv_bfloat16*>(a.dq_c),
        a.rope ? a.rope_cos : nullptr, a.rope ? a.rope_sin : nullptr, rows, a.T, a.D, a.scale, a.H, grad_row_stride(a),
        grad_b_stride(a), grad_h_stride(a), a.token_row, a.B);
    count_launches(1);
    if (le != cudaSuccess) { set_error("attention backward launch: %s", cudaGetErrorString(le)); return MINTB_ECUDA; }
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("attention backward launch: %s", cudaGetErrorString(e)); return MINTB_ECUDA; }
  return MINTB_OK;
}

}  // namespace mintb
