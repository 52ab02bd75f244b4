// tcgen05 kernels of the combined-softmax multimer attention (bf16 in, fp32 accumulate), forward pass.
//
// One CTA owns a tile of 128 query rows of one (batch, head) and walks a list of key runs ("entries") that share a class:
// pure entries (one pathway) of up to 128 keys (64 at head_dim 64), mixed entries of 64 (32) keys.  Warp roles:
//   warp 0     TMA producer: Q tiles once, then per entry only the K/V tiles its class needs
//              (intra-only: K_self,V_self; inter-only: K_cross,V_cross; mixed: all four)
//   warp 1     tcgen05.mma issuer: S = Q K^T into TMEM, then O += P V with P read from TMEM
//   warps 2-9  softmax: two threads per query row (TMEM lane), each with its own online-softmax state over one half of
//              the entry's keys and its own O accumulator; lazy rescale of O; the halves are merged in the epilogue
// TMEM (256 columns, two CTAs per SM): S (logits, fp32), P (probabilities, packed bf16), O half 0, O half 1.
// S is released as soon as the softmax threads have read it, so the next Q K^T overlaps this entry's exponentials;
// a mixed entry holds the self logits in the low half of S and the cross logits in the high half.
// Every wait on an mbarrier is bounded; on expiry the role records a code in *dev_status and unwinds.
#include <mutex>

#include "common.cuh"
#include "ptx.cuh"

namespace mintb {

using namespace ptx;

constexpr int kBM = 128;          // query rows per CTA
constexpr int kTcThreads = 320;   // producer warp, MMA warp, 8 softmax warps
constexpr int kTmemCols = 256;
constexpr int kMaxKeyTiles = 512;  // entries per query tile (T <= 16384)
constexpr unsigned kStaggerNs = 350;       // initial offset between the two softmax groups of a CTA
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

// Packed fp32x2 arithmetic (two lanes per instruction on the FMA pipe) and the three-input maximum.
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
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// ------------------------------------------------------------------------------------------------ RoPE pre-pass
// y = R(x) for the self pathway's Q and K, written as bf16 to the workspace.  One thread rotates 8 dims of the lower
// half together with their partners in the upper half (16-byte loads and stores, rows contiguous in memory).
__global__ void __launch_bounds__(256) rope_rotate_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                                          __nv_bfloat16* __restrict__ qr, __nv_bfloat16* __restrict__ kr,
                                                          const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
                                                          size_t rows, int T, int D) {
  griddep_launch();   // the attention kernel's set-up may overlap this pass
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
// Work list of one CTA: runs of keys ("entries") that share a class.  A pure entry (one pathway) covers kN keys when two
// adjacent 64-key tiles of the same pathway can be merged, else kN/2... see build below; a mixed entry covers kBox keys and
// holds the self logits in S columns [0, kBox) and the cross logits in [kBox, 2 kBox).
template <int D>
struct FwdCfg {
  static constexpr int kN = D == 64 ? 64 : 128;    // most keys per entry (S columns)
  static constexpr int kBox = kN / 2;              // keys per TMA box; keys of a mixed entry
  static constexpr int kStages = 4;
  static constexpr int kRowBytes = 2 * D;
  static constexpr int kQBytes = kBM * kRowBytes;
  static constexpr int kBoxBytes = kBox * kRowBytes;
  // A stage holds [K | V] of a pure entry (kN rows each) or [K_self, K_cross | V_self, V_cross] of a mixed one (kBox rows each)
  static constexpr int kSlotBytes = kN * kRowBytes;
  static constexpr int kStageBytes = 2 * kSlotBytes;
  static constexpr int kColS = 0, kColP = kN;                // S: kN fp32 columns; P: kN/2 columns of packed bf16
  static constexpr int kColO = D == 64 ? 128 : 192;          // O of key-half 0, then O of key-half 1
  static constexpr int kOStride = D == 64 ? 64 : 32;
  static constexpr size_t kSmemBytes = 1024 /*align slack*/ + 2 * kQBytes + size_t(kStages) * kStageBytes + 8192 /*tail: barriers, items, statistics, two entry lists*/;
};

struct FwdParams {
  const uint32_t *bits, *kpad;
  const uint8_t* cls;
  __nv_bfloat16* out;
  float* lse;
  int H, T, TW, NT;
  float scale_log2;  // scale * log2(e)
  int* status;
  size_t out_row_stride, out_bh_stride;   // elements between consecutive queries / (batch, head) pairs of `out`
  int skip_pad_queries;                   // leave out query tiles that hold only padded positions
  int* sched;                             // work counter pair of this launch (common.cuh)
  int NQ, n_items;                        // query tiles per (batch, head); items = NQ * B * H, item = bh * NQ + qt
};

// entry flags (low three bits are the class bits kHasIntra | kHasInter | kHasPad)
constexpr uint8_t kEntryFull = 8;   // covers kN keys (else kBox)

// One chunk of W (32 or 16) logits of one query row: mask, running max, lazy rescale, exp2, row sum, packed bf16 out.
// `s` holds the selected logits on entry.  Returns the packed probabilities in `pk` (W / 2 words).
// With SQ (square-root softmax, out = sum_j sqrt(p_j) v_j) the stored terms are exp2((s c - m_ref) / 2) — `c22` then holds
// c / 2 — the row sum adds their squares, and `alpha_out`, which rescales O and terms already packed, is the square root
// of the factor applied to the row sum.
template <int W, bool SQ>
__device__ __forceinline__ void softmax_chunk(float (&s)[W], uint32_t pad_bits, bool has_pad, float c2, uint64_t c22,
                                              float& m_ref, float& l, float& alpha_out, bool& rescale_out,
                                              uint32_t (&pk)[W / 2]) {
  if (has_pad) {
#pragma unroll
    for (int j = 0; j < W; ++j)
      if ((pad_bits >> j) & 1u) s[j] = -INFINITY;
  }
  float m0 = fmaxf(s[0], s[1]), m1 = fmaxf(s[2], s[3]), m2 = fmaxf(s[4], s[5]), m3 = fmaxf(s[6], s[7]);
#pragma unroll
  for (int j = 8; j < W; j += 8) {
    m0 = fmax3(m0, s[j], s[j + 1]); m1 = fmax3(m1, s[j + 2], s[j + 3]);
    m2 = fmax3(m2, s[j + 4], s[j + 5]); m3 = fmax3(m3, s[j + 6], s[j + 7]);
  }
  const float m_tile = fmaxf(fmax3(m0, m1, m2), m3) * c2;   // c2 > 0; -inf if every key of the chunk is padded
  alpha_out = 1.f;
  rescale_out = false;
  if (m_tile > m_ref + kRescaleThreshold) {   // also the first finite maximum (m_ref = -inf)
    const float a = ex2(m_ref - m_tile);       // 0 when nothing has been accumulated yet
    alpha_out = SQ ? ex2(0.5f * (m_ref - m_tile)) : a;
    m_ref = m_tile;
    l *= a;
    rescale_out = true;
  }
  // exp2(s c - m_ref); while every key seen so far is padded (m_ref = -inf) use 0 as reference: exp2(-inf) = 0
  const float nm = m_ref == -INFINITY ? 0.f : (SQ ? -0.5f * m_ref : -m_ref);
  const uint64_t nm2 = pack2(nm, nm);
  uint64_t la = pack2(0.f, 0.f), lb = la;
#pragma unroll
  for (int j = 0; j < W / 2; j += 2) {
    float p0, p1, p2, p3;
    unpack2(ffma2(pack2(s[2 * j], s[2 * j + 1]), c22, nm2), p0, p1);
    unpack2(ffma2(pack2(s[2 * j + 2], s[2 * j + 3]), c22, nm2), p2, p3);
    p0 = ex2(p0); p1 = ex2(p1); p2 = ex2(p2); p3 = ex2(p3);
    if (SQ) {
      const uint64_t a = pack2(p0, p1), b = pack2(p2, p3);
      la = ffma2(a, a, la);
      lb = ffma2(b, b, lb);
    } else {
      la = fadd2(la, pack2(p0, p1));
      lb = fadd2(lb, pack2(p2, p3));
    }
    pk[j] = pack_bf16(p0, p1);
    pk[j + 1] = pack_bf16(p2, p3);
  }
  float l0, l1;
  unpack2(fadd2(la, lb), l0, l1);
  l += l0 + l1;
}

// A work item of the persistent forward kernel as the producer warp hands it to the other roles.
struct FwdItem {
  int qt, bh;
  int n_ent;    // entries of the item; kItemEnd: no more work; kItemSkip: a query tile that is left out (nothing to write)
};
constexpr int kItemEnd = -1, kItemSkip = -2;

// Persistent CTAs (two per SM) take (query tile, batch * head) items from a counter in global memory.  The producer warp
// runs one item ahead: while the other roles work on item i it fetches item i + 1, builds its entry list (double buffered)
// and, as soon as the last Q K^T of item i has read the Q tiles, loads the next Q tiles and the first K/V stages, so that
// the set-up of an item hides behind the tail of its predecessor, and a CTA that drew a cheap item simply draws the next.
template <int D, bool SQ>
__global__ void __launch_bounds__(kTcThreads, 2)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_qs, const __grid_constant__ CUtensorMap map_ks,
                   const __grid_constant__ CUtensorMap map_vs, const __grid_constant__ CUtensorMap map_qc,
                   const __grid_constant__ CUtensorMap map_kc, const __grid_constant__ CUtensorMap map_vc, FwdParams p) {
  using Cfg = FwdCfg<D>;
  constexpr int kStages = Cfg::kStages, RB = Cfg::kRowBytes, kN = Cfg::kN, kBox = Cfg::kBox;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sQs = smem;
  unsigned char* sQc = smem + Cfg::kQBytes;
  unsigned char* sKV = smem + 2 * Cfg::kQBytes;  // [stage][K slot | V slot]
  unsigned char* tail = sKV + size_t(kStages) * Cfg::kStageBytes;
  uint64_t* bar_q = reinterpret_cast<uint64_t*>(tail);   // producer -> MMA: the Q tiles of the item have landed
  uint64_t* q_free = bar_q + 1;           // MMA -> producer: the item's last Q K^T has completed, the Q tiles may be overwritten
  uint64_t* kv_full = q_free + 1;         // [kStages]
  uint64_t* kv_empty = kv_full + kStages; // [kStages]
  uint64_t* s_full = kv_empty + kStages;  // MMA -> softmax: logits of the entry are in TMEM
  uint64_t* s_free = s_full + 1;          // softmax -> MMA: every thread has read its logits (256 arrivals)
  uint64_t* p_full = s_free + 1;          // softmax -> MMA: probabilities are in TMEM (256 arrivals)
  uint64_t* o_ready = p_full + 1;         // MMA -> softmax: P V of the entry has completed
  uint64_t* item_full = o_ready + 1;      // [2] producer -> MMA, softmax: the item and its entry list are in shared memory
  uint64_t* item_free = item_full + 2;    // [2] MMA, softmax -> producer: the slot may be overwritten (257 arrivals)
  uint64_t* h_full = item_free + 2;       // softmax -> softmax: both halves' statistics of the item are written (256 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(h_full + 1);
  FwdItem* items = reinterpret_cast<FwdItem*>(tmem_slot + 2);     // [2]
  float* hstat = reinterpret_cast<float*>(items + 2);              // per item slot: [2][128] running maxima, [2][128] row sums
  uint16_t* ent_k = reinterpret_cast<uint16_t*>(hstat + 2 * 512);  // [2][kMaxKeyTiles] first key of the entry / 32
  uint8_t* ent_c = reinterpret_cast<uint8_t*>(ent_k + 2 * kMaxKeyTiles);   // [2][kMaxKeyTiles]

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int nkt = p.NT;  // key tiles of 64 == class-table columns

  if (tid == 0) {
    mbar_init(bar_q, 1);
    mbar_init(q_free, 1);
    for (int s = 0; s < kStages; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    mbar_init(s_full, 1);
    mbar_init(s_free, 256);
    mbar_init(p_full, 256);
    mbar_init(o_ready, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&item_full[s], 1); mbar_init(&item_free[s], 257); }
    mbar_init(h_full, 256);
    fence_mbar_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  griddep_wait();   // the set-up above may overlap the rotation pass before this kernel; its copies are read from here on
  const uint32_t tbase = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- producer: scheduler, entry lists, TMA
    if (lane == 0) {
      prefetch_tensormap(&map_qs); prefetch_tensormap(&map_qc);
      prefetch_tensormap(&map_ks); prefetch_tensormap(&map_vs);
      prefetch_tensormap(&map_kc); prefetch_tensormap(&map_vc);
    }
    uint32_t item_no = 0, q_no = 0, g_it = 0;   // items drawn, Q loads issued, entries loaded (over all items of this CTA)
    bool ok = true;
    for (;;) {
      const int slot = item_no & 1;
      int item = 0;
      if (lane == 0) item = item_no == 0 ? int(blockIdx.x) : int(gridDim.x) + atomicAdd(p.sched, 1);   // the first item is the CTA's own number
      item = __shfl_sync(0xffffffffu, item, 0);
      const bool have = item < p.n_items;
      if (item_no >= 2) {   // the slot was last used by item item_no - 2: the other roles must have left it
        ok = __all_sync(0xffffffffu, mbar_wait(&item_free[slot], ((item_no >> 1) - 1) & 1, p.status, 0x102));
        if (!ok) break;
      }
      const int qt = have ? item % p.NQ : 0, bh = have ? item / p.NQ : 0, b = bh / p.H;
      int n = kItemEnd;
      if (have) {
        bool skip = false;
        if (p.skip_pad_queries) {   // the padding bits describe positions, so they cover the query rows of this tile as well
          const uint32_t* w = p.kpad + size_t(b) * p.TW + 4 * qt;
          skip = (w[0] & w[1] & w[2] & w[3]) == 0xffffffffu;
        }
        if (skip) {
          n = kItemSkip;
        } else {
          // tile classes of this query tile (OR of its two 64-row halves) turned into the entry list, 32 key tiles per pass
          uint16_t* ek = ent_k + slot * kMaxKeyTiles;
          uint8_t* ec = ent_c + slot * kMaxKeyTiles;
          const uint8_t* row0 = p.cls + (size_t(b) * p.NT + 2 * qt) * p.NT;
          const bool two_rows = 2 * qt + 1 < p.NT;
          n = 0;
          for (int base = 0; base < nkt; base += 32) {
            const int kt = base + lane;
            uint8_t c = 0;
            if (kt < nkt) {
              c = row0[kt];
              if (two_rows) c |= row0[p.NT + kt];
              if (!(c & (kHasIntra | kHasInter))) c = 0;
            }
            uint8_t cn = uint8_t(__shfl_down_sync(0xffffffffu, unsigned(c), 1));   // a pass boundary also ends a run
            uint8_t cp = uint8_t(__shfl_up_sync(0xffffffffu, unsigned(c), 1));
            if (lane == 31) cn = 0;
            if (lane == 0) cp = 0;
            const bool mixed = (c & 3) == 3, pure = c != 0 && !mixed;
            // runs of pure tiles of one pathway: a tile starts a run unless its predecessor is a pure tile of the same pathway
            const bool run_start = pure && !(cp != 0 && (cp & 3) == (c & 3));
            const unsigned starts = __ballot_sync(0xffffffffu, run_start);
            const unsigned below = starts & (0xffffffffu >> (31 - lane));               // run starts at or before this lane
            const int off = pure ? lane - (31 - __clz(below)) : 0;                      // position inside the run
            const bool can_pair = kN == 128 && pure && cn != 0 && (cn & 3) == (c & 3);
            int cnt = 0;
            uint8_t flags = c;
            if (mixed) cnt = kN == 128 ? 1 : 2;
            else if (pure) {
              if constexpr (kN == 128) {
                if ((off & 1) == 0) { cnt = 1; if (can_pair) flags = uint8_t(c | cn | kEntryFull); }
              } else {
                cnt = 1;
                flags = uint8_t(c | kEntryFull);
              }
            }
            // exclusive prefix sum of cnt over the lanes (cnt is 0, 1 or 2)
            const unsigned b1 = __ballot_sync(0xffffffffu, cnt & 1), b2 = __ballot_sync(0xffffffffu, cnt & 2);
            const unsigned lt = (1u << lane) - 1u;
            const int pos = n + __popc(b1 & lt) + 2 * __popc(b2 & lt);
            if (cnt >= 1) { ek[pos] = uint16_t(2 * kt); ec[pos] = flags; }
            if (cnt == 2) { ek[pos + 1] = uint16_t(2 * kt + 1); ec[pos + 1] = flags; }
            n += __popc(b1) + 2 * __popc(b2);
          }
        }
      }
      if (lane == 0) items[slot] = FwdItem{qt, bh, n};
      __syncwarp();
      if (lane == 0) mbar_arrive(&item_full[slot]);
      if (!have) break;
      if (n > 0) {
        if (lane == 0) {
          if (q_no > 0) ok = mbar_wait(q_free, (q_no - 1) & 1, p.status, 0x103);   // the previous item's Q tiles are no longer read
          if (ok) {
            mbar_expect_tx(bar_q, 2 * Cfg::kQBytes);
            tma_load_3d(sQs, &map_qs, bar_q, 0, qt * kBM, bh);
            tma_load_3d(sQc, &map_qc, bar_q, 0, qt * kBM, bh);
            const uint16_t* ek = ent_k + slot * kMaxKeyTiles;
            const uint8_t* ec = ent_c + slot * kMaxKeyTiles;
            for (int it = 0; it < n; ++it, ++g_it) {
              const int stage = g_it % kStages;
              if (!mbar_wait(&kv_empty[stage], ((g_it / kStages) & 1) ^ 1, p.status, 0x101)) { ok = false; break; }
              const uint8_t c = ec[it];
              const int k0 = int(ek[it]) * 32;
              unsigned char* kslot = sKV + size_t(stage) * Cfg::kStageBytes;
              unsigned char* vslot = kslot + Cfg::kSlotBytes;
              if ((c & 3) == 3) {   // mixed: one box of each of the four tensors
                mbar_expect_tx(&kv_full[stage], 4 * Cfg::kBoxBytes);
                tma_load_3d(kslot, &map_ks, &kv_full[stage], 0, k0, bh);
                tma_load_3d(kslot + Cfg::kBoxBytes, &map_kc, &kv_full[stage], 0, k0, bh);
                tma_load_3d(vslot, &map_vs, &kv_full[stage], 0, k0, bh);
                tma_load_3d(vslot + Cfg::kBoxBytes, &map_vc, &kv_full[stage], 0, k0, bh);
              } else {
                const CUtensorMap* mk = (c & kHasIntra) ? &map_ks : &map_kc;
                const CUtensorMap* mv = (c & kHasIntra) ? &map_vs : &map_vc;
                const int boxes = (c & kEntryFull) ? 2 : 1;
                mbar_expect_tx(&kv_full[stage], 2 * boxes * Cfg::kBoxBytes);
                for (int bx = 0; bx < boxes; ++bx) {
                  tma_load_3d(kslot + bx * Cfg::kBoxBytes, mk, &kv_full[stage], 0, k0 + bx * kBox, bh);
                  tma_load_3d(vslot + bx * Cfg::kBoxBytes, mv, &kv_full[stage], 0, k0 + bx * kBox, bh);
                }
              }
            }
          }
        }
        ok = __shfl_sync(0xffffffffu, int(ok), 0) != 0;
        g_it = __shfl_sync(0xffffffffu, g_it, 0);
        ++q_no;
        if (!ok) break;
      }
      ++item_no;
    }
    if (lane == 0) leave_tile_counter(p.sched, int(gridDim.x));   // (after this CTA's last draw, whichever way the loop ended)
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    // The whole warp runs this loop and one elected lane issues: with warp-uniform control flow and operands the compiler
    // keeps the descriptors in uniform registers, which is what the MMA instruction reads; issued from a divergent
    // single-lane region every instruction first moves its operands there, and that, not the tensor pipe, set the pace.
    // Values read from shared memory are made provably uniform with a lane-0 shuffle.  Order per entry: as soon as the
    // softmax threads have READ S of the entry before, the next Q K^T is issued into the same columns (P lives
    // elsewhere) - also across items -, then P V of this entry once its probabilities have arrived.
    {
      const bool leader = elect_one();
      constexpr uint32_t idesc_qk_full = idesc_bf16(kBM, kN, false, false);
      constexpr uint32_t idesc_qk_half = idesc_bf16(kBM, kBox, false, false);
      constexpr uint32_t idesc_pv = idesc_bf16(kBM, D, false, true);
      constexpr uint32_t kHi = desc_hi32(8 * RB, swizzle_for_row_bytes(RB));      // K-major and MN-major tiles alike
      constexpr uint32_t kLboK = desc_lbo32(16), kLboV = desc_lbo32(8 * RB);
      constexpr uint32_t kSlot = Cfg::kSlotBytes >> 4, kBoxU = Cfg::kBoxBytes >> 4, kStageUnits = Cfg::kStageBytes >> 4;
      constexpr uint32_t kVStep = (16 * RB) >> 4;
      const uint32_t smem_base = __shfl_sync(0xffffffffu, smem_u32(smem), 0);
      const uint32_t tb = __shfl_sync(0xffffffffu, tbase, 0);
      const uint32_t lo_qs = desc_addr32(smem_base) + kLboK, lo_qc = desc_addr32(smem_base + Cfg::kQBytes) + kLboK;
      const uint32_t lo_kv = desc_addr32(smem_base + 2 * Cfg::kQBytes);
      const uint32_t col_s = tb + Cfg::kColS, col_p = tb + Cfg::kColP, col_o = tb + Cfg::kColO;
      uint32_t item_no = 0, q_no = 0, g_it = 0;   // g_it: entries whose P V has been issued (over all items)
      bool ok = true;
      auto wait_all = [&](uint64_t* bar, uint32_t parity, int code) -> bool {
        return __all_sync(0xffffffffu, mbar_wait(bar, parity, p.status, code));
      };

      // Q K^T of entry number g (over all items), class byte c; S must have been read by the softmax threads of entry g - 1
      auto issue_qk = [&](uint32_t g, uint32_t c) -> bool {
        if (g > 0 && !wait_all(s_free, (g - 1) & 1, 0x205)) return false;
        const uint32_t stage = g % kStages;
        if (!wait_all(&kv_full[stage], (g / kStages) & 1, 0x202)) return false;
        tc_fence_after();
        const uint32_t slot = lo_kv + stage * kStageUnits + kLboK;
        if ((c & 3) == 3) {   // mixed: self logits in columns [0, kBox), cross logits in [kBox, 2 kBox)
          if (leader) {
#pragma unroll
            for (int k = 0; k < D / 16; ++k)
              umma_ss(col_s, make_desc(kHi, lo_qs + 2 * k), make_desc(kHi, slot + 2 * k), idesc_qk_half, k > 0);
#pragma unroll
            for (int k = 0; k < D / 16; ++k)
              umma_ss(col_s + kBox, make_desc(kHi, lo_qc + 2 * k), make_desc(kHi, slot + kBoxU + 2 * k), idesc_qk_half, k > 0);
          }
        } else {
          const uint32_t a_lo = (c & kHasIntra) ? lo_qs : lo_qc;
          const uint32_t idesc = (c & kEntryFull) ? idesc_qk_full : idesc_qk_half;
          if (leader) {
#pragma unroll
            for (int k = 0; k < D / 16; ++k) umma_ss(col_s, make_desc(kHi, a_lo + 2 * k), make_desc(kHi, slot + 2 * k), idesc, k > 0);
          }
        }
        if (leader) umma_commit(s_full);
        __syncwarp();
        return true;
      };

      for (;;) {
        const int slot = item_no & 1;
        ok = wait_all(&item_full[slot], (item_no >> 1) & 1, 0x206);
        if (!ok) break;
        const int n_ent = __shfl_sync(0xffffffffu, items[slot].n_ent, 0);
        if (n_ent == kItemEnd) break;
        if (n_ent > 0) {
          const uint8_t* ec = ent_c + slot * kMaxKeyTiles;
          ok = wait_all(bar_q, q_no & 1, 0x201);
          if (!ok) break;
          tc_fence_after();
          uint32_t c_next = __shfl_sync(0xffffffffu, uint32_t(ec[0]), 0);
          ok = issue_qk(g_it, c_next);
          if (ok && n_ent == 1 && leader) umma_commit(q_free);
          for (int it = 0; it < n_ent && ok; ++it, ++g_it) {
            const uint32_t c = c_next;
            if (it + 1 < n_ent) {
              c_next = __shfl_sync(0xffffffffu, uint32_t(ec[it + 1]), 0);
              ok = issue_qk(g_it + 1, c_next);
              if (!ok) break;
              if (it + 2 == n_ent && leader) umma_commit(q_free);   // that was the item's last Q K^T
            }
            ok = wait_all(p_full, g_it & 1, 0x203);
            if (!ok) break;
            tc_fence_after();
            const uint32_t v_lo = lo_kv + uint32_t(g_it % kStages) * kStageUnits + kSlot + kLboV;
            const bool acc = it > 0;
            if ((c & 3) == 3) {
              // keys [0, kBox/2) of the entry belong to softmax half 0 (O half 0), the rest to half 1
              if (leader) {
#pragma unroll
                for (int k = 0; k < kBox / 16; ++k)
                  umma_ts(col_o + (k >= kBox / 32 ? Cfg::kOStride : 0), col_p + k * 8, make_desc(kHi, v_lo + k * kVStep), idesc_pv,
                          acc || (k % (kBox / 32)) != 0);
#pragma unroll
                for (int k = 0; k < kBox / 16; ++k)
                  umma_ts(col_o + (k >= kBox / 32 ? Cfg::kOStride : 0), col_p + kBox / 2 + k * 8,
                          make_desc(kHi, v_lo + kBoxU + k * kVStep), idesc_pv, true);
              }
            } else if (c & kEntryFull) {
              if (leader) {
#pragma unroll
                for (int k = 0; k < kN / 16; ++k)
                  umma_ts(col_o + (k >= kN / 32 ? Cfg::kOStride : 0), col_p + k * 8, make_desc(kHi, v_lo + k * kVStep), idesc_pv,
                          acc || (k % (kN / 32)) != 0);
              }
            } else {
              if (leader) {
#pragma unroll
                for (int k = 0; k < kBox / 16; ++k)
                  umma_ts(col_o + (k >= kBox / 32 ? Cfg::kOStride : 0), col_p + k * 8, make_desc(kHi, v_lo + k * kVStep), idesc_pv,
                          acc || (k % (kBox / 32)) != 0);
              }
            }
            if (leader) {
              umma_commit(o_ready);
              umma_commit(&kv_empty[g_it % kStages]);
            }
            __syncwarp();
          }
          if (!ok) break;
          ++q_no;
        }
        if (leader) mbar_arrive(&item_free[slot]);
        ++item_no;
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax warps: two threads per query row
    // Thread (row, ch) owns half ch of the keys of every entry of its row, with its OWN running maximum, row sum and O
    // accumulator (the P V product of key-half ch lands in O half ch), so the two threads of a row never synchronise inside
    // the loop; the two partial softmax states are merged once per item, in its epilogue.
    const int sw = warp - 2;                      // 0..7
    const int quarter = warp % 4;                 // TMEM lane quarter this warp may access
    const int ch = sw / 4;                        // key half
    const int row = quarter * 32 + lane;          // row within the query tile == TMEM lane
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    const uint32_t tO = tbase + lane_base + Cfg::kColO + Cfg::kOStride * ch;
    const uint32_t tS = tbase + lane_base + Cfg::kColS;
    const uint32_t tP = tbase + lane_base + Cfg::kColP;
    const float c2 = p.scale_log2;
    const uint64_t c22 = SQ ? pack2(0.5f * c2, 0.5f * c2) : pack2(c2, c2);   // multiplies the logits inside exp2
    uint32_t item_no = 0, g_it = 0, h_no = 0;   // items seen, entries done, items whose statistics were merged
    bool ok = true;

    // rescale this thread's O accumulator by alpha (rare: the running maximum grew by more than the threshold)
    auto rescale_o = [&](float alpha) {
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 16) {
        uint32_t o[16];
        tmem_ld16(tO + c0, o);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
        tmem_st16(tO + c0, o);
      }
    };

    for (;;) {
      const int slot = item_no & 1;
      ok = mbar_wait(&item_full[slot], (item_no >> 1) & 1, p.status, 0x306);
      if (!ok) break;
      const FwdItem item = items[slot];
      if (item.n_ent == kItemEnd) break;
      const int n_ent = item.n_ent, bh = item.bh, b = bh / p.H;
      const int qi = item.qt * kBM + row;
      const int qrow = qi < p.T ? qi : p.T - 1;
      if (n_ent != kItemSkip) {
      const uint16_t* ent_k_i = ent_k + slot * kMaxKeyTiles;
      const uint8_t* ent_c_i = ent_c + slot * kMaxKeyTiles;
      const uint32_t* mrow = p.bits + (size_t(b) * p.T + qrow) * p.TW;
      const uint32_t* prow = p.kpad + size_t(b) * p.TW;
      float m_ref = -INFINITY, l = 0.f;

      for (int it = 0; it < n_ent && ok; ++it, ++g_it) {
        const uint8_t c = ent_c_i[it];
        const int kw = int(ent_k_i[it]);              // first key of the entry / 32
        const bool mixed = (c & 3) == 3;
        const bool has_pad = (c & kHasPad) != 0;
        ok = mbar_wait(s_full, g_it & 1, p.status, 0x301);
        if (!ok) break;
        if (it == 0 && ch == 1) __nanosleep(kStaggerNs);   // the two key halves run out of phase (see kStaggerNs)
        tc_fence_after();
        // Every phase of o_ready is observed, entry by entry (a parity wait cannot tell phases two apart): before O is
        // rescaled or, at the latest, before P (single-buffered) is overwritten.
        bool o_seen = it == 0;
        auto see_o = [&]() -> bool {
          if (o_seen) return true;
          o_seen = true;
          if (!mbar_wait(o_ready, (g_it - 1) & 1, p.status, 0x304)) return false;
          tc_fence_after();
          return true;
        };

        if (!mixed && (c & kEntryFull) && kN == 128) {
          // 128 keys: this thread's 64 logits in two chunks of 32
          float alpha; bool resc;
          uint32_t pk[16];
          {
            float s[32];
            uint32_t r[32];
            tmem_ld32(tS + 64 * ch, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) s[j] = __uint_as_float(r[j]);
            softmax_chunk<32, SQ>(s, has_pad ? prow[kw + 2 * ch] : 0u, has_pad, c2, c22, m_ref, l, alpha, resc, pk);
          }
          if (__any_sync(0xffffffffu, resc && it > 0)) { ok = see_o(); if (!ok) break; rescale_o(alpha); }
          uint32_t pk2[16];
          {
            float s[32];
            uint32_t r[32];
            tmem_ld32(tS + 64 * ch + 32, r);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(s_free);                       // both chunks are in registers: S may be overwritten
#pragma unroll
            for (int j = 0; j < 32; ++j) s[j] = __uint_as_float(r[j]);
            softmax_chunk<32, SQ>(s, has_pad ? prow[kw + 2 * ch + 1] : 0u, has_pad, c2, c22, m_ref, l, alpha, resc, pk2);
          }
          // a rescale decided by the second chunk also applies to what the first chunk contributes: fold it into pk
          if (__any_sync(0xffffffffu, resc)) {
            if (it > 0) { ok = see_o(); if (!ok) break; rescale_o(alpha); }
            if (resc) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float a0 = __uint_as_float(pk[j] << 16) * alpha, a1 = __uint_as_float(pk[j] & 0xffff0000u) * alpha;
                pk[j] = pack_bf16(a0, a1);
              }
            }
          }
          ok = see_o();
          if (!ok) break;
          tmem_st16(tP + 32 * ch, pk);
          tmem_st16(tP + 32 * ch + 16, pk2);
        } else if (!mixed) {
          // kBox (D <= 32: 64) or kN (D = 64: 64) keys: 32 logits per thread;  D = 64 half entries do not occur for pure tiles
          constexpr int W = 32;
          float alpha; bool resc;
          uint32_t pk[W / 2];
          {
            float s[W];
            uint32_t r[W];
            tmem_ld32(tS + W * ch, r);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(s_free);
#pragma unroll
            for (int j = 0; j < W; ++j) s[j] = __uint_as_float(r[j]);
            softmax_chunk<W, SQ>(s, has_pad ? prow[kw + ch] : 0u, has_pad, c2, c22, m_ref, l, alpha, resc, pk);
          }
          if (__any_sync(0xffffffffu, resc && it > 0)) { ok = see_o(); if (!ok) break; rescale_o(alpha); }
          ok = see_o();
          if (!ok) break;
          tmem_st16(tP + (W / 2) * ch, pk);
        } else {
          // mixed entry of kBox keys: W = kBox / 2 logits per thread, selected between the self and cross logits
          constexpr int W = kBox / 2;   // 32 (D <= 32) or 16 (D = 64)
          float alpha; bool resc;
          uint32_t pk[W / 2];
          // mask and padding bits of this thread's W keys: key index of bit 0 is 32 kw + W ch
          const int bit0 = W * ch;                       // offset inside the entry (entry starts on a 32-key boundary)
          const uint32_t cw = (mrow[kw + bit0 / 32] >> (bit0 % 32)) & (W == 32 ? 0xffffffffu : 0xffffu);
          const uint32_t pw = has_pad ? (prow[kw + bit0 / 32] >> (bit0 % 32)) : 0u;
          {
            float s[W];
            uint32_t rs[W], rc[W];
            tmem_ld_n<W>(tS + W * ch, rs);
            tmem_ld_n<W>(tS + kBox + W * ch, rc);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(s_free);
#pragma unroll
            for (int j = 0; j < W; ++j) s[j] = __uint_as_float(((cw >> j) & 1u) ? rc[j] : rs[j]);
            softmax_chunk<W, SQ>(s, pw, has_pad, c2, c22, m_ref, l, alpha, resc, pk);
          }
          if (__any_sync(0xffffffffu, resc && it > 0)) { ok = see_o(); if (!ok) break; rescale_o(alpha); }
          // split by pathway: P o ~M multiplies V_self, P o M multiplies V_cross
          uint32_t pi[W / 2], pe[W / 2];
#pragma unroll
          for (int j = 0; j < W / 2; ++j) {
            const uint32_t lo_x = (cw >> (2 * j)) & 1u, hi_x = (cw >> (2 * j + 1)) & 1u;
            const uint32_t keep_e = (lo_x ? 0x0000ffffu : 0u) | (hi_x ? 0xffff0000u : 0u);
            pe[j] = pk[j] & keep_e;
            pi[j] = pk[j] & ~keep_e;
          }
          ok = see_o();
          if (!ok) break;
          tmem_st_n<W / 2>(tP + (W / 2) * ch, pi);
          tmem_st_n<W / 2>(tP + kBox / 2 + (W / 2) * ch, pe);
        }
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(p_full);
      }
      if (!ok) break;
      // ---- epilogue of the item: merge the two softmax states of each row, O / l -> bf16, lse
      // (the statistics are double buffered: every merge passes the h_full barrier, so a thread is at most one merge ahead of
      // its row's other thread; the wait is an mbarrier so that it is bounded)
      float* hm = hstat + (h_no & 1) * 512;   // [2][128] running maxima
      float* hl = hm + 256;             // [2][128] row sums
      hm[ch * 128 + row] = m_ref;
      hl[ch * 128 + row] = l;
      mbar_arrive(h_full);
      ok = mbar_wait(h_full, h_no & 1, p.status, 0x307);
      ++h_no;
      if (!ok) break;
      const float m_other = hm[(ch ^ 1) * 128 + row], l_other = hl[(ch ^ 1) * 128 + row];
      if (n_ent > 0) ok = mbar_wait(o_ready, (g_it - 1) & 1, p.status, 0x305);
      tc_fence_after();
      if (ok) {
        constexpr int NC = D / 2;   // output columns written by this thread
        __nv_bfloat16* orow = p.out + size_t(bh) * p.out_bh_stride + size_t(qi) * p.out_row_stride + ch * NC;
        if (n_ent == 0) {
          if (qi < p.T) {   // no unpadded key at all: NaN, as the softmax of an all -inf row gives in the PyTorch path
            const uint32_t nan2 = 0x7FC07FC0u;
#pragma unroll
            for (int d = 0; d < NC; d += 8) *reinterpret_cast<uint4*>(orow + d) = make_uint4(nan2, nan2, nan2, nan2);
            if (ch == 0) p.lse[size_t(bh) * p.T + qi] = -INFINITY;
          }
        } else {
          const float m_all = fmaxf(m_ref, m_other);                 // finite: an active tile has an unpadded key
          const float w_self = ex2(m_ref - m_all), w_other = ex2(m_other - m_all);   // exp2(-inf) = 0 for an empty half
          const float l_all = l * w_self + l_other * w_other;
          // softmax: O / l.  square-root softmax: the accumulators hold sum exp2((s - m) / 2) v, so they are brought to the
          // common maximum by the square roots of the weights and divided by sqrt(l)
          const float inv = SQ ? rsqrtf(l_all) : 1.f / l_all;
          const float f_self = (SQ ? ex2(0.5f * (m_ref - m_all)) : w_self) * inv;
          const float f_other = (SQ ? ex2(0.5f * (m_other - m_all)) : w_other) * inv;
          constexpr int CH = NC > 16 ? 16 : NC;   // columns per pass (keeps the register footprint small)
#pragma unroll
          for (int c0 = 0; c0 < NC; c0 += CH) {
            uint32_t oa[CH], ob[CH];
            tmem_ld_n<CH>(tO + ch * NC + c0, oa);                                                              // own accumulator
            tmem_ld_n<CH>(tbase + lane_base + Cfg::kColO + Cfg::kOStride * (ch ^ 1) + ch * NC + c0, ob);       // the other half's
            tmem_ld_wait();
            if (qi < p.T) {
              float v[CH];
#pragma unroll
              for (int j = 0; j < CH; ++j) {
                // an empty half holds whatever was in TMEM: its weight is exactly 0, but 0 * NaN must not leak
                const float a = w_self > 0.f ? __uint_as_float(oa[j]) * f_self : 0.f;
                const float bb = w_other > 0.f ? __uint_as_float(ob[j]) * f_other : 0.f;
                v[j] = a + bb;
              }
#pragma unroll
              for (int j = 0; j < CH; j += 8)
                *reinterpret_cast<uint4*>(orow + c0 + j) = make_uint4(pack_bf16(v[j], v[j + 1]), pack_bf16(v[j + 2], v[j + 3]),
                                                                      pack_bf16(v[j + 4], v[j + 5]), pack_bf16(v[j + 6], v[j + 7]));
            }
          }
          if (qi < p.T) {
            if (ch == 0) p.lse[size_t(bh) * p.T + qi] = (m_all + log2f(l_all)) * kLn2;
          }
        }
      }
      if (!ok) break;
      }
      // O and the entry list of this slot are no longer read by this thread
      tc_fence_before();
      mbar_arrive(&item_free[slot]);
      ++item_no;
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

// [rotated Q_self | rotated K_self] (with in-kernel RoPE only)
size_t tc_fwd_workspace_bytes(int B, int H, int T, int D, bool rope) { return rope ? 2 * rot_bytes(B, H, T, D) : 0; }

template <int D, bool SQ>
static int fwd_tc_t(const AttnArgs& a, const void* q_s, const void* k_s) {
  using Cfg = FwdCfg<D>;
  const int BH = a.B * a.H;
  CUtensorMap mqs, mks, mvs, mqc, mkc, mvc;
  if (!make_map(&mqs, q_s, D, a.T, BH, kBM) || !make_map(&mks, k_s, D, a.T, BH, Cfg::kBox) ||
      !make_map(&mvs, a.v_s, D, a.T, BH, Cfg::kBox) || !make_map(&mqc, a.q_c, D, a.T, BH, kBM) ||
      !make_map(&mkc, a.k_c, D, a.T, BH, Cfg::kBox) || !make_map(&mvc, a.v_c, D, a.T, BH, Cfg::kBox)) {
    set_error("mintb_attn_fwd: cuTensorMapEncodeTiled failed");
    return MINTB_ECUDA;
  }
  {  // per device and cheap, so set on every call
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_tc_kernel<D, SQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(Cfg::kSmemBytes));
    if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return MINTB_ECUDA; }
  }
  int* sched = nullptr;   // the launch's work counter pair (common.cuh)
  if (int rc = next_tile_counter(&sched); rc != MINTB_OK) return rc;
  const int NQ = (a.T + kBM - 1) / kBM;
  const long long n_items = (long long)NQ * BH;
  if (n_items > 0x7fff0000LL) { set_error("mintb_attn_fwd: %lld work items exceed the counter's range", n_items); return MINTB_EUNSUPPORTED; }
  FwdParams p{a.meta.bits, a.meta.kpad, a.meta.cls, static_cast<__nv_bfloat16*>(a.out), a.lse, a.H, a.T, a.meta.TW, a.meta.NT,
              a.scale * kLog2e, a.dev_status, out_row_stride(a), out_bh_stride(a), a.skip_pad_queries ? 1 : 0,
              sched, NQ, int(n_items)};
  static int n_ctas = 0;   // two persistent CTAs per SM
  if (n_ctas == 0) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    n_ctas = 2 * (sms > 0 ? sms : 148);
  }
  const unsigned grid = unsigned(n_items < n_ctas ? n_items : n_ctas);
  cudaError_t e = launch_dependent(attn_fwd_tc_kernel<D, SQ>, dim3(grid), dim3(kTcThreads), Cfg::kSmemBytes, a.stream, mqs, mks, mvs, mqc, mkc, mvc, p);
  count_launches(1);
  if (e == cudaSuccess) e = cudaGetLastError();
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
  if (2 * a.meta.NT > kMaxKeyTiles) { set_error("mintb_attn_fwd: T = %d exceeds %d", a.T, kMaxKeyTiles * 32); return MINTB_EUNSUPPORTED; }
  const void* q_s = a.q_s;
  const void* k_s = a.k_s;
  if (a.rope && !a.qk_prerotated) {
    char* ws = static_cast<char*>(a.workspace);
    __nv_bfloat16* qr = reinterpret_cast<__nv_bfloat16*>(ws);
    __nv_bfloat16* kr = reinterpret_cast<__nv_bfloat16*>(ws + rot_bytes(a.B, a.H, a.T, a.D));
    launch_rope_rotate(a, qr, kr);
    q_s = qr;
    k_s = kr;
  }
  switch (a.D) {
    case 16: return a.sqrt_softmax ? fwd_tc_t<16, true>(a, q_s, k_s) : fwd_tc_t<16, false>(a, q_s, k_s);
    case 32: return a.sqrt_softmax ? fwd_tc_t<32, true>(a, q_s, k_s) : fwd_tc_t<32, false>(a, q_s, k_s);
    case 64: return a.sqrt_softmax ? fwd_tc_t<64, true>(a, q_s, k_s) : fwd_tc_t<64, false>(a, q_s, k_s);
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
  const size_t need = tc_fwd_workspace_bytes(B, H, T, D, a.rope && !a.qk_prerotated);
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
