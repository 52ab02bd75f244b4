// tcgen05 kernels of the combined-softmax multimer attention (bf16 in, fp32 accumulate), forward pass.
//
// One CTA owns a tile of 128 query rows of one (batch, head) and walks the key tiles of 64.  Warp roles:
//   warp 0     TMA producer: Q tiles once, then per key tile only the K/V tiles its class needs
//              (intra-only: K_self,V_self; inter-only: K_cross,V_cross; mixed: all four)
//   warp 1     tcgen05.mma issuer: S = Q K^T into a TMEM buffer, then O += P V with P read from TMEM
//   warps 2-5  softmax: one thread per query row (TMEM lane), online softmax over the combined logits,
//              P written back into the S buffer as packed bf16, lazy rescale of O, epilogue
// TMEM (256 columns, two CTAs per SM): O [0,64), S/P buffer 0 [64,128), buffer 1 [128,192).
// A pure tile uses one buffer (alternating, so the next QK^T overlaps this tile's softmax); a mixed tile
// puts the self logits in buffer 0 and the cross logits in buffer 1 and issues two P V products.
// Every wait on an mbarrier is bounded; on expiry the role records a code in *dev_status and unwinds.
#include <mutex>

#include "common.cuh"
#include "ptx.cuh"

namespace mintb {

using namespace ptx;

constexpr int kBM = 128;          // query rows per CTA
constexpr int kBN = 64;           // keys per tile
constexpr int kTcThreads = 192;
constexpr int kTmemCols = 256;
constexpr int kColO = 0, kColS0 = 64, kColS1 = 128;
constexpr int kMaxKeyTiles = 512;  // T <= 32768
constexpr float kRescaleThreshold = 8.f;  // log2 units: P stays below 2^8 between rescales

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// [B*H][T][D] bf16 tensor viewed as a 3-D map (D, T, B*H) with a box of (D, rows, 1); rows past T read as zero.
static bool make_map(CUtensorMap* m, const void* ptr, int D, int T, int BH, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[3] = {cuuint64_t(D), cuuint64_t(T), cuuint64_t(BH)};
  cuuint64_t strides[2] = {cuuint64_t(D) * 2, cuuint64_t(T) * D * 2};
  cuuint32_t box[3] = {cuuint32_t(D), cuuint32_t(box_rows), 1};
  cuuint32_t es[3] = {1, 1, 1};
  CUtensorMapSwizzle sw = D == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : D == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// ------------------------------------------------------------------------------------------------ RoPE pre-pass
// y = R(x) for the self pathway's Q and K, written as bf16 to the workspace.  One thread rotates 8 dims of the lower
// half together with their partners in the upper half (16-byte loads and stores, rows contiguous in memory).
__global__ void __launch_bounds__(256) rope_rotate_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                                          __nv_bfloat16* __restrict__ qr, __nv_bfloat16* __restrict__ kr,
                                                          const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
                                                          size_t rows, int T, int D) {
  const int h = D / 2, cpr = h / 8;  // chunks per row
  const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= rows * cpr) return;
  const int c = int(idx % cpr);
  const size_t row = idx / cpr;
  const int t = int(row % T);
  const float4* ct = reinterpret_cast<const float4*>(cos_tab + size_t(t) * h + c * 8);
  const float4* st = reinterpret_cast<const float4*>(sin_tab + size_t(t) * h + c * 8);
  const float4 c0 = ct[0], c1 = ct[1], s0 = st[0], s1 = st[1];
  const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
  const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    const __nv_bfloat16* src = (which == 0 ? q : k) + row * D + c * 8;
    __nv_bfloat16* dst = (which == 0 ? qr : kr) + row * D + c * 8;
    uint4 lo = *reinterpret_cast<const uint4*>(src), hi = *reinterpret_cast<const uint4*>(src + h);
    const __nv_bfloat16* lp = reinterpret_cast<const __nv_bfloat16*>(&lo);
    const __nv_bfloat16* hp = reinterpret_cast<const __nv_bfloat16*>(&hi);
    uint4 olo, ohi;
    __nv_bfloat16* olp = reinterpret_cast<__nv_bfloat16*>(&olo);
    __nv_bfloat16* ohp = reinterpret_cast<__nv_bfloat16*>(&ohi);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float a = __bfloat162float(lp[e]), b = __bfloat162float(hp[e]);
      olp[e] = __float2bfloat16_rn(a * cs[e] - b * sn[e]);
      ohp[e] = __float2bfloat16_rn(b * cs[e] + a * sn[e]);
    }
    *reinterpret_cast<uint4*>(dst) = olo;
    *reinterpret_cast<uint4*>(dst + h) = ohi;
  }
}

// ------------------------------------------------------------------------------------------------ forward
template <int D>
struct FwdCfg {
  static constexpr int kStages = D == 64 ? 2 : 3;
  static constexpr int kRowBytes = 2 * D;
  static constexpr int kQBytes = kBM * kRowBytes;
  static constexpr int kKvBytes = kBN * kRowBytes;
  static constexpr size_t kSmemBytes = 1024 /*align slack*/ + 2 * kQBytes + size_t(kStages) * 4 * kKvBytes + 1024 /*barriers, tile classes*/;
};

struct FwdParams {
  const uint32_t *bits, *kpad;
  const uint8_t* cls;
  __nv_bfloat16* out;
  float* lse;
  int H, T, TW, NT;
  float scale_log2;  // scale * log2(e)
  int* status;
};

template <int D>
__global__ void __launch_bounds__(kTcThreads, 2)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_qs, const __grid_constant__ CUtensorMap map_ks,
                   const __grid_constant__ CUtensorMap map_vs, const __grid_constant__ CUtensorMap map_qc,
                   const __grid_constant__ CUtensorMap map_kc, const __grid_constant__ CUtensorMap map_vc, FwdParams p) {
  using Cfg = FwdCfg<D>;
  constexpr int kStages = Cfg::kStages, RB = Cfg::kRowBytes;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sQs = smem;
  unsigned char* sQc = smem + Cfg::kQBytes;
  unsigned char* sKV = smem + 2 * Cfg::kQBytes;  // [stage][slot: 0 K_self, 1 K_cross, 2 V_self, 3 V_cross]
  unsigned char* tail = sKV + size_t(kStages) * 4 * Cfg::kKvBytes;
  uint64_t* bar_q = reinterpret_cast<uint64_t*>(tail);
  uint64_t* kv_full = bar_q + 1;
  uint64_t* kv_empty = kv_full + kStages;
  uint64_t* s_full = kv_empty + kStages;  // [2]
  uint64_t* p_full = s_full + 2;          // [2]
  uint64_t* o_ready = p_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_ready + 1);
  uint8_t* tcls = reinterpret_cast<uint8_t*>(tmem_slot + 2);  // class per key tile, 0 = skip

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int qt = blockIdx.x, bh = blockIdx.y, b = bh / p.H;
  const int q0 = qt * kBM;
  const int nkt = p.NT;  // key tiles of 64 == class-table columns

  // tile classes of this query tile: OR of its two 64-row halves
  for (int kt = tid; kt < nkt; kt += kTcThreads) {
    const uint8_t* row0 = p.cls + (size_t(b) * p.NT + 2 * qt) * p.NT;
    uint8_t c = row0[kt];
    if (2 * qt + 1 < p.NT) c |= row0[p.NT + kt];
    tcls[kt] = (c & (kHasIntra | kHasInter)) ? c : 0;
  }
  if (tid == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < kStages; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    mbar_init(&s_full[0], 1); mbar_init(&s_full[1], 1);
    mbar_init(&p_full[0], 128); mbar_init(&p_full[1], 128);
    mbar_init(o_ready, 1);
    fence_mbar_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      prefetch_tensormap(&map_qs); prefetch_tensormap(&map_qc);
      prefetch_tensormap(&map_ks); prefetch_tensormap(&map_vs);
      prefetch_tensormap(&map_kc); prefetch_tensormap(&map_vc);
      mbar_expect_tx(bar_q, 2 * Cfg::kQBytes);
      tma_load_3d(sQs, &map_qs, bar_q, 0, q0, bh);
      tma_load_3d(sQc, &map_qc, bar_q, 0, q0, bh);
      int it = 0;
      for (int kt = 0; kt < nkt; ++kt) {
        const uint8_t c = tcls[kt];
        if (c == 0) continue;
        const int stage = it % kStages;
        if (!mbar_wait(&kv_empty[stage], ((it / kStages) & 1) ^ 1, p.status, 0x101)) break;
        unsigned char* slot = sKV + size_t(stage) * 4 * Cfg::kKvBytes;
        const int n = ((c & kHasIntra) ? 2 : 0) + ((c & kHasInter) ? 2 : 0);
        mbar_expect_tx(&kv_full[stage], n * Cfg::kKvBytes);
        if (c & kHasIntra) {
          tma_load_3d(slot + 0 * Cfg::kKvBytes, &map_ks, &kv_full[stage], 0, kt * kBN, bh);
          tma_load_3d(slot + 2 * Cfg::kKvBytes, &map_vs, &kv_full[stage], 0, kt * kBN, bh);
        }
        if (c & kHasInter) {
          tma_load_3d(slot + 1 * Cfg::kKvBytes, &map_kc, &kv_full[stage], 0, kt * kBN, bh);
          tma_load_3d(slot + 3 * Cfg::kKvBytes, &map_vc, &kv_full[stage], 0, kt * kBN, bh);
        }
        ++it;
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = idesc_bf16(kBM, kBN, false, false);
      constexpr uint32_t idesc_pv = idesc_bf16(kBM, D, false, true);
      const uint32_t qs_addr = smem_u32(sQs), qc_addr = smem_u32(sQc), kv_addr = smem_u32(sKV);
      const uint32_t col_s[2] = {tbase + kColS0, tbase + kColS1};
      bool ok = mbar_wait(bar_q, 0, p.status, 0x201);
      tc_fence_after();

      // issue S = Q K^T of active tile `it` (class c); the stage must be full
      auto issue_qk = [&](int it, uint8_t c) -> bool {
        const int stage = it % kStages;
        if (!mbar_wait(&kv_full[stage], (it / kStages) & 1, p.status, 0x202)) return false;
        tc_fence_after();
        const uint32_t slot = kv_addr + uint32_t(stage) * 4 * Cfg::kKvBytes;
        const bool mixed = (c & 3) == 3;
        if (mixed || (c & kHasIntra)) {
          const int buf = mixed ? 0 : (it & 1);
#pragma unroll
          for (int k = 0; k < D / 16; ++k)
            umma_ss(col_s[buf], desc_k_major(qs_addr + k * 32, RB), desc_k_major(slot + 0 * Cfg::kKvBytes + k * 32, RB), idesc_qk, k > 0);
          umma_commit(&s_full[buf]);
        }
        if (mixed || (c & kHasInter)) {
          const int buf = mixed ? 1 : (it & 1);
#pragma unroll
          for (int k = 0; k < D / 16; ++k)
            umma_ss(col_s[buf], desc_k_major(qc_addr + k * 32, RB), desc_k_major(slot + 1 * Cfg::kKvBytes + k * 32, RB), idesc_qk, k > 0);
          umma_commit(&s_full[buf]);
        }
        return true;
      };

      // next active tile after kt (or nkt)
      auto next_active = [&](int kt) { while (kt < nkt && tcls[kt] == 0) ++kt; return kt; };
      int kt = next_active(0);
      int it = 0;
      uint32_t p_uses[2] = {0, 0};
      bool qk_issued = false;  // S of tile `it` already issued
      while (ok && kt < nkt) {
        const uint8_t c = tcls[kt];
        const bool mixed = (c & 3) == 3;
        if (!qk_issued) ok = issue_qk(it, c);
        if (!ok) break;
        const int kt_next = next_active(kt + 1);
        const uint8_t c_next = kt_next < nkt ? tcls[kt_next] : 0;
        const bool next_mixed = (c_next & 3) == 3;
        qk_issued = false;
        if (c_next != 0 && !mixed && !next_mixed) {  // other buffer is free: overlap next QK^T with this softmax
          ok = issue_qk(it + 1, c_next);
          qk_issued = true;
          if (!ok) break;
        }
        // O += P V
        const int stage = it % kStages;
        const uint32_t slot = kv_addr + uint32_t(stage) * 4 * Cfg::kKvBytes;
        bool acc = it > 0;
        if (mixed || (c & kHasIntra)) {
          const int buf = mixed ? 0 : (it & 1);
          ok = mbar_wait(&p_full[buf], p_uses[buf] & 1, p.status, 0x203);
          if (!ok) break;
          ++p_uses[buf];
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < kBN / 16; ++k) {
            umma_ts(tbase + kColO, col_s[buf] + k * 8, desc_mn_major(slot + 2 * Cfg::kKvBytes + k * 16 * RB, RB, 8 * RB), idesc_pv, acc);
            acc = true;
          }
        }
        if (mixed || (c & kHasInter)) {
          const int buf = mixed ? 1 : (it & 1);
          ok = mbar_wait(&p_full[buf], p_uses[buf] & 1, p.status, 0x204);
          if (!ok) break;
          ++p_uses[buf];
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < kBN / 16; ++k) {
            umma_ts(tbase + kColO, col_s[buf] + k * 8, desc_mn_major(slot + 3 * Cfg::kKvBytes + k * 16 * RB, RB, 8 * RB), idesc_pv, acc);
            acc = true;
          }
        }
        umma_commit(&kv_empty[stage]);
        umma_commit(o_ready);
        kt = kt_next;
        ++it;
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax warps (one thread per query row)
    const int quarter = warp % 4;                 // TMEM lane quarter this warp may access
    const int row = quarter * 32 + lane;          // row within the query tile == TMEM lane
    const int qi = q0 + row;
    const int qrow = qi < p.T ? qi : p.T - 1;
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    const uint32_t tO = tbase + lane_base + kColO;
    const uint32_t tS[2] = {tbase + lane_base + kColS0, tbase + lane_base + kColS1};
    const uint32_t* mrow = p.bits + (size_t(b) * p.T + qrow) * p.TW;
    const uint32_t* prow = p.kpad + size_t(b) * p.TW;
    const float c2 = p.scale_log2;
    float m_ref = -INFINITY, l = 0.f;
    uint32_t s_uses[2] = {0, 0};
    int it = 0;
    bool ok = true;
    for (int kt = 0; kt < nkt && ok; ++kt) {
      const uint8_t c = tcls[kt];
      if (c == 0) continue;
      const bool mixed = (c & 3) == 3;
      float s[kBN];
      if (!mixed) {
        const int buf = it & 1;
        ok = mbar_wait(&s_full[buf], s_uses[buf] & 1, p.status, 0x301);
        if (!ok) break;
        ++s_uses[buf];
        tc_fence_after();
        uint32_t r0[32], r1[32];
        tmem_ld32(tS[buf], r0);
        tmem_ld32(tS[buf] + 32, r1);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) { s[j] = __uint_as_float(r0[j]); s[32 + j] = __uint_as_float(r1[j]); }
      } else {
        ok = mbar_wait(&s_full[0], s_uses[0] & 1, p.status, 0x302) && mbar_wait(&s_full[1], s_uses[1] & 1, p.status, 0x303);
        if (!ok) break;
        ++s_uses[0]; ++s_uses[1];
        tc_fence_after();
        const uint2 cw = *reinterpret_cast<const uint2*>(mrow + 2 * kt);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t rs[32], rc[32];
          tmem_ld32(tS[0] + 32 * half, rs);
          tmem_ld32(tS[1] + 32 * half, rc);
          tmem_ld_wait();
          const uint32_t w = half == 0 ? cw.x : cw.y;
#pragma unroll
          for (int j = 0; j < 32; ++j) s[32 * half + j] = __uint_as_float(((w >> j) & 1u) ? rc[j] : rs[j]);
        }
      }
      if (c & kHasPad) {
        const uint2 pw = *reinterpret_cast<const uint2*>(prow + 2 * kt);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if ((pw.x >> j) & 1u) s[j] = -INFINITY;
          if ((pw.y >> j) & 1u) s[32 + j] = -INFINITY;
        }
      }
      float tmax = s[0];
#pragma unroll
      for (int j = 1; j < kBN; ++j) tmax = fmaxf(tmax, s[j]);
      const float m_tile = tmax * c2;  // c2 > 0; -inf only if every key of the tile is padded for this row's mask
      float alpha = 1.f;
      bool rescale = false;
      if (it == 0) {
        m_ref = m_tile;
      } else if (m_tile > m_ref + kRescaleThreshold) {
        alpha = ex2(m_ref - m_tile);   // m_ref = -inf (nothing seen yet) gives 0
        m_ref = m_tile;
        l *= alpha;
        rescale = true;
      }
      // Every phase of o_ready is observed, tile by tile (a parity wait cannot tell phases two apart):
      // early when O has to be rescaled, otherwise just before P is handed over.
      bool o_seen = it == 0;
      if (it > 0 && __any_sync(0xffffffffu, rescale)) {
        ok = mbar_wait(o_ready, (it - 1) & 1, p.status, 0x304);
        if (!ok) break;
        o_seen = true;
        tc_fence_after();
        if constexpr (D >= 32) {
#pragma unroll
          for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t o[32];
            tmem_ld32(tO + c0, o);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
            tmem_st32(tO + c0, o);
          }
        } else {
          uint32_t o[16];
          tmem_ld16(tO, o);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
          tmem_st16(tO, o);
        }
      }
      // A row that has seen only padded keys so far keeps m_ref = -inf; use 0 as the reference so exp2 gives 0, not NaN.
      const float mr = m_ref == -INFINITY ? 0.f : m_ref;
      float lsum = 0.f;
      if (!mixed) {
        uint32_t pk[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float p0 = ex2(fmaf(s[2 * j], c2, -mr)), p1 = ex2(fmaf(s[2 * j + 1], c2, -mr));
          lsum += p0 + p1;
          pk[j] = pack_bf16(p0, p1);
        }
        tmem_st32(tS[it & 1], pk);
      } else {
        const uint2 cw = *reinterpret_cast<const uint2*>(mrow + 2 * kt);
        uint32_t pi[32], pe[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float p0 = ex2(fmaf(s[2 * j], c2, -mr)), p1 = ex2(fmaf(s[2 * j + 1], c2, -mr));
          lsum += p0 + p1;
          const uint32_t w = (2 * j) < 32 ? cw.x : cw.y;
          const bool x0 = (w >> ((2 * j) & 31)) & 1u, x1 = (w >> ((2 * j + 1) & 31)) & 1u;
          pi[j] = pack_bf16(x0 ? 0.f : p0, x1 ? 0.f : p1);
          pe[j] = pack_bf16(x0 ? p0 : 0.f, x1 ? p1 : 0.f);
        }
        tmem_st32(tS[0], pi);
        tmem_st32(tS[1], pe);
      }
      l += lsum;
      tmem_st_wait();
      if (!o_seen) {
        ok = mbar_wait(o_ready, (it - 1) & 1, p.status, 0x306);
        if (!ok) break;
      }
      tc_fence_before();
      if (!mixed) {
        mbar_arrive(&p_full[it & 1]);
      } else {
        mbar_arrive(&p_full[0]);
        mbar_arrive(&p_full[1]);
      }
      ++it;
    }
    // ---- epilogue: O / l -> bf16, lse
    if (ok && it > 0) ok = mbar_wait(o_ready, (it - 1) & 1, p.status, 0x305);
    tc_fence_after();
    if (ok) {
      const float inv = 1.f / l;  // no unpadded key at all: l = 0 and the row becomes NaN, as in the PyTorch path
      __nv_bfloat16* orow = p.out + (size_t(bh) * p.T + qi) * D;
      if (it == 0) {
        if (qi < p.T) {
          const uint32_t nan2 = 0x7FC07FC0u;
#pragma unroll
          for (int d = 0; d < D; d += 8) *reinterpret_cast<uint4*>(orow + d) = make_uint4(nan2, nan2, nan2, nan2);
          p.lse[size_t(bh) * p.T + qi] = -INFINITY;
        }
      } else {
        if constexpr (D >= 32) {
#pragma unroll
          for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t o[32];
            tmem_ld32(tO + c0, o);
            tmem_ld_wait();
            if (qi < p.T) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 v;
                v.x = pack_bf16(__uint_as_float(o[j + 0]) * inv, __uint_as_float(o[j + 1]) * inv);
                v.y = pack_bf16(__uint_as_float(o[j + 2]) * inv, __uint_as_float(o[j + 3]) * inv);
                v.z = pack_bf16(__uint_as_float(o[j + 4]) * inv, __uint_as_float(o[j + 5]) * inv);
                v.w = pack_bf16(__uint_as_float(o[j + 6]) * inv, __uint_as_float(o[j + 7]) * inv);
                *reinterpret_cast<uint4*>(orow + c0 + j) = v;
              }
            }
          }
        } else {
          uint32_t o[16];
          tmem_ld16(tO, o);
          tmem_ld_wait();
          if (qi < p.T) {
#pragma unroll
            for (int j = 0; j < 16; j += 8) {
              uint4 v;
              v.x = pack_bf16(__uint_as_float(o[j + 0]) * inv, __uint_as_float(o[j + 1]) * inv);
              v.y = pack_bf16(__uint_as_float(o[j + 2]) * inv, __uint_as_float(o[j + 3]) * inv);
              v.z = pack_bf16(__uint_as_float(o[j + 4]) * inv, __uint_as_float(o[j + 5]) * inv);
              v.w = pack_bf16(__uint_as_float(o[j + 6]) * inv, __uint_as_float(o[j + 7]) * inv);
              *reinterpret_cast<uint4*>(orow + j) = v;
            }
          }
        }
        if (qi < p.T) p.lse[size_t(bh) * p.T + qi] = (m_ref + log2f(l)) * kLn2;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tbase, kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------------ host side
bool tc_supported(int D, int dtype) { return dtype == MINTB_BF16 && (D == 16 || D == 32 || D == 64); }

static size_t rot_bytes(int B, int H, int T, int D) { return align256(size_t(B) * H * T * D * 2); }

size_t tc_fwd_workspace_bytes(int B, int H, int T, int D, bool rope) { return rope ? 2 * rot_bytes(B, H, T, D) : 0; }

template <int D>
static int fwd_tc_t(const AttnArgs& a, const void* q_s, const void* k_s) {
  using Cfg = FwdCfg<D>;
  const int BH = a.B * a.H;
  CUtensorMap mqs, mks, mvs, mqc, mkc, mvc;
  if (!make_map(&mqs, q_s, D, a.T, BH, kBM) || !make_map(&mks, k_s, D, a.T, BH, kBN) ||
      !make_map(&mvs, a.v_s, D, a.T, BH, kBN) || !make_map(&mqc, a.q_c, D, a.T, BH, kBM) ||
      !make_map(&mkc, a.k_c, D, a.T, BH, kBN) || !make_map(&mvc, a.v_c, D, a.T, BH, kBN)) {
    set_error("mintb_attn_fwd: cuTensorMapEncodeTiled failed");
    return MINTB_ECUDA;
  }
  {  // per device and cheap, so set on every call
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(Cfg::kSmemBytes));
    if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return MINTB_ECUDA; }
  }
  FwdParams p{a.meta.bits, a.meta.kpad, a.meta.cls, static_cast<__nv_bfloat16*>(a.out), a.lse, a.H, a.T, a.meta.TW, a.meta.NT,
              a.scale * kLog2e, a.dev_status};
  dim3 grid((a.T + kBM - 1) / kBM, BH);
  attn_fwd_tc_kernel<D><<<grid, kTcThreads, Cfg::kSmemBytes, a.stream>>>(mqs, mks, mvs, mqc, mkc, mvc, p);
  count_launches(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("attention forward launch: %s", cudaGetErrorString(e)); return MINTB_ECUDA; }
  return MINTB_OK;
}

// Rotated copies of the self pathway's Q and K (shared by the forward and backward launchers).
void launch_rope_rotate(const AttnArgs& a, __nv_bfloat16* qr, __nv_bfloat16* kr) {
  const size_t rows = size_t(a.B) * a.H * a.T;
  const size_t n = rows * (a.D / 16);
  rope_rotate_kernel<<<unsigned((n + 255) / 256), 256, 0, a.stream>>>(
      static_cast<const __nv_bfloat16*>(a.q_s), static_cast<const __nv_bfloat16*>(a.k_s), qr, kr, a.rope_cos, a.rope_sin, rows, a.T, a.D);
  count_launches(1);
}

int launch_attn_fwd_tc(const AttnArgs& a) {
  if (a.meta.NT > kMaxKeyTiles) { set_error("mintb_attn_fwd: T = %d exceeds %d", a.T, kMaxKeyTiles * kBN); return MINTB_EUNSUPPORTED; }
  const void* q_s = a.q_s;
  const void* k_s = a.k_s;
  if (a.rope) {
    char* ws = static_cast<char*>(a.workspace);
    __nv_bfloat16* qr = reinterpret_cast<__nv_bfloat16*>(ws);
    __nv_bfloat16* kr = reinterpret_cast<__nv_bfloat16*>(ws + rot_bytes(a.B, a.H, a.T, a.D));
    launch_rope_rotate(a, qr, kr);
    q_s = qr;
    k_s = kr;
  }
  switch (a.D) {
    case 16: return fwd_tc_t<16>(a, q_s, k_s);
    case 32: return fwd_tc_t<32>(a, q_s, k_s);
    case 64: return fwd_tc_t<64>(a, q_s, k_s);
  }
  set_error("mintb_attn_fwd: unsupported head_dim %d", a.D);
  return MINTB_EUNSUPPORTED;
}

// ------------------------------------------------------------------------------------------------ no-allocation forward
// Scratch for mintb_attn_fwd_static: the rotated copies of Q_self and K_self that the forward pass with RoPE reads.
// It is part of the loaded module, so every GPU that loads this library holds these bytes until the process exits.
static __device__ __align__(256) unsigned char g_fwd_static_scratch[MINTB_STATIC_SCRATCH_BYTES];

// `g_fwd_static_scratch` names the array for DEVICE code only.  Host code must ask the runtime for the array's address on
// the device that is current; the answer differs per device and is cached here after the first call on each device.
static int static_scratch_ptr(void** out) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static void* ptrs[kMaxDevices] = {};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_error("mintb_attn_fwd_static: cudaGetDevice failed or device index %d is out of range", dev);
    return MINTB_ECUDA;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_fwd_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_error("mintb_attn_fwd_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return MINTB_ECUDA;
    }
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return MINTB_OK;
}

}  // namespace mintb

extern "C" int mintb_attn_fwd_static(const void* q_self, const void* k_self, const void* v_self, const void* q_cross,
                                     const void* k_cross, const void* v_cross, const void* meta, const float* rope_cos,
                                     const float* rope_sin, void* out, float* lse, int B, int H, int T, int D, int dtype,
                                     unsigned flags, float scale, void* stream, int* dev_status) {
  using namespace mintb;
  if (dtype != MINTB_BF16 || (flags & MINTB_FLAG_FORCE_SIMT)) {
    set_error("mintb_attn_fwd_static: only the bf16 tensor-core forward has a no-allocation variant");
    return MINTB_EUNSUPPORTED;
  }
  AttnArgs a{};
  // the shared argument checks first (no workspace is passed in, so none is checked there)
  int rc = check_attn_args(a, "mintb_attn_fwd_static", q_self, k_self, v_self, q_cross, k_cross, v_cross, meta, rope_cos,
                           rope_sin, nullptr, 0, 0, B, H, T, D, dtype, flags, scale, stream, dev_status);
  if (rc != MINTB_OK) return rc;
  if (out == nullptr || lse == nullptr || (reinterpret_cast<uintptr_t>(out) & 15) != 0) {
    set_error("mintb_attn_fwd_static: out (16-byte aligned) and lse are required");
    return MINTB_EINVAL;
  }
  const size_t need = tc_fwd_workspace_bytes(B, H, T, D, a.rope);
  if (need > size_t(MINTB_STATIC_SCRATCH_BYTES)) {
    set_error("mintb_attn_fwd_static: B*H*T*D = %zu needs %zu bytes of scratch, the built-in array holds %zu; "
              "use mintb_attn_fwd with a caller-provided workspace",
              size_t(B) * H * T * D, need, size_t(MINTB_STATIC_SCRATCH_BYTES));
    return MINTB_EWORKSPACE;
  }
  void* scratch = nullptr;
  rc = static_scratch_ptr(&scratch);
  if (rc != MINTB_OK) return rc;
  a.out = out;
  a.lse = lse;
  a.workspace = scratch;   // every byte the kernels read from it is written by the rotation pass of this same call
  a.workspace_bytes = size_t(MINTB_STATIC_SCRATCH_BYTES);
  return launch_attn_fwd_tc(a);
}
