// tcgen05 GEMM for the projections around the attention: out = epilogue(alpha * x W^T + bias).
//
//   x [M][K] and W [N][K] are both K-contiguous (nn.Linear layout), bf16 (kind::f16) or e4m3 (kind::f8f6f4), fp32 accumulate.
//   Persistent CTAs walk 128 x 256 output tiles (N fastest, so the CTAs running together share rows of x in L2).
//   warp 0  TMA producer: 128-byte-wide K slabs of x (128 rows) and W (256 rows) into a 4-stage ring, 128B swizzle
//   warp 1  MMA issuer: four tcgen05.mma (M128 N256) per slab into one of two 256-column TMEM accumulators
//   warps 2-9  epilogue: two threads per output row (one per half of the tile's columns); 32 columns at a time: alpha, bias, erf-GELU, cast, store —
//              row-major, or scattered head-major into (B,H,T,D) q/k/v with optional scale and RoPE (the QKV projection),
//              while the MMA warp already fills the other accumulator.
// Every mbarrier wait is bounded (see ptx.cuh).
#include "common.cuh"
#include "ptx.cuh"

#include <cuda_fp8.h>

namespace mintb {

using namespace ptx;

constexpr int kGM = 128, kGN = 256, kGStages = 4;
constexpr int kGEpiWarps = 8, kGEpiThreads = 32 * kGEpiWarps, kGThreads = 64 + kGEpiThreads;   // TMA warp, MMA warp, epilogue warps
constexpr int kSlabBytes = 128;                       // bytes of K per stage and row (64 bf16 or 128 e4m3)
constexpr int kABytes = kGM * kSlabBytes, kBBytes = kGN * kSlabBytes, kGStageBytes = kABytes + kBBytes;
constexpr int kGStageOutBytes = 32 * 64 + 32 * 32;   // one epilogue warp's staging: 32 rows x 32 bf16 columns, then 32 rows x 32 e4m3 columns, for bulk stores
constexpr int kGTileRing = 4;   // tile numbers travel from the loading warp to the other roles through a ring this deep
constexpr size_t kGemmSmem = 1024 + size_t(kGStages) * kGStageBytes + kGEpiWarps * kGStageOutBytes + 256 + 2 * kGN * sizeof(float);

enum GemmEpilogue : int { kEpiBias = 0, kEpiBiasGelu = 1, kEpiHeadMajor = 2 };

struct GemmParams {
  int M, N, K;                 // K in elements
  int in_dtype;                // MINTB_BF16 or MINTB_E4M3
  int out_dtype;               // MINTB_BF16 or MINTB_E4M3 (row-major epilogues)
  int bias_dtype;              // MINTB_F32 or MINTB_BF16
  int epilogue;
  float alpha;                 // multiplies the accumulator (product of the operands' dequantisation scales)
  float alpha2;                // head-major epilogue with two pathways: the multiplier of the second pathway's columns (n >= 3E)
  const __nv_bfloat16* resid;  // row-major epilogues: when non-null the result is res_a * resid[m][n] + res_b * (alpha x w^T + bias)
  float res_a, res_b;
  float out_scale;             // multiplies the result before the cast to e4m3
  const void* bias;            // [N] or null
  void* out;                   // row-major [M][N]
  __nv_bfloat16* preact;       // when non-null, the value before the activation / the e4m3 cast is also stored here (bf16 [M][N])
  // head-major scatter: row m = t * B + b, column n = which * E + h * D + d  ->  dst[which][((b * H + h) * T + t) * D + d]
  __nv_bfloat16* qkv[6];       // q, k, v of the first pathway, then (two-pathway projection) of the second
  int B, T, H, D;
  float q_scale;               // multiplies the q third (1 to leave the scaling to the attention kernel)
  const float *rope_cos, *rope_sin;   // [T][D/2]; rotate the q and k thirds when non-null
  const int32_t* row_map;             // packed input rows: row m of x is token row_map[m] = t * B + b (null: m itself)
  int use_bulk_store;          // bf16 row-major outputs leave through shared memory and bulk tensor stores
  int use_bulk_f8;        // the e4m3 result leaves as bulk tensor stores too (32 x 32-byte boxes)
  int alt_stores;         // every chunk issues a bf16 bulk store (pre-activation copy) AND an e4m3 one: they alternate between two staging areas
  int* status;
  int* sched;                  // work counter pair of this launch (common.cuh)
};

// erf-GELU x/2 (1 + erf(x / sqrt 2)) with erf from the rational-exponential form 1 - (a1 t + ... + a5 t^5) exp(-z^2),
// t = 1 / (1 + p z) (absolute error below 1.5e-7, far inside the bf16 / e4m3 output precision): two special-function
// operations and a short Horner chain per element keep the epilogue shorter than the products of a K = 1280 tile.
// two fp32 values in one 64-bit register for the packed fp32 instructions of sm_100
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
__device__ __forceinline__ uint64_t fmul2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

// erf-GELU of two values: x/2 (1 + erf(x / sqrt 2)) = max(x, 0) - a 2^s(a), a = min(|x|, 5.75), where
// s(a) = log2(erfc(a / sqrt 2)) - 1 is replaced by a polynomial of degree 6 (least squares on Chebyshev nodes of [0, 5.75],
// weighted by the result's sensitivity a 2^s ln 2 and re-weighted towards the largest error).  Against the exact function in
// fp32 arithmetic: largest absolute error 5.1e-7, largest error relative to max(|gelu|, 1e-3) 5.2e-5 (the Abramowitz-Stegun
// 7.1.26 form it replaces: 6.6e-7 and 2.7e-4, with two MUFU operations and 16 instructions per value instead of one and 7).
// Beyond 5.75 the subtracted term is below 6e-8 |x|.
__device__ __forceinline__ void gelu_erf2(float& x0, float& x1) {
  const float a0 = fminf(fabsf(x0), 5.75f), a1 = fminf(fabsf(x1), 5.75f);
  const uint64_t a = pack2(a0, a1);
  uint64_t s = ffma2(pack2(3.309347236e-05f, 3.309347236e-05f), a, pack2(-7.692253187e-04f, -7.692253187e-04f));
  s = ffma2(s, a, pack2(8.080734485e-03f, 8.080734485e-03f));
  s = ffma2(s, a, pack2(-5.341213111e-02f, -5.341213111e-02f));
  s = ffma2(s, a, pack2(-4.587709539e-01f, -4.587709539e-01f));
  s = ffma2(s, a, pack2(-1.151201708e+00f, -1.151201708e+00f));
  s = ffma2(s, a, pack2(-9.999930604e-01f, -9.999930604e-01f));
  float s0, s1, e0, e1;
  unpack2(s, s0, s1);
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(s0));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(s1));
  x0 = fmaf(-a0, e0, fmaxf(x0, 0.f));
  x1 = fmaf(-a1, e1, fmaxf(x1, 0.f));
}

__device__ __forceinline__ float load_bias(const void* bias, int dtype, int n) {
  return dtype == MINTB_F32 ? static_cast<const float*>(bias)[n] : __bfloat162float(static_cast<const __nv_bfloat16*>(bias)[n]);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// EPI: epilogue kind; HD: head_dim of the head-major epilogue (0 otherwise)
template <int EPI, int HD>
__global__ void __launch_bounds__(kGThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_out, const __grid_constant__ CUtensorMap map_pre, GemmParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* s_out = smem + size_t(kGStages) * kGStageBytes;   // [epilogue warp][32 rows][64 B], 64B swizzle
  unsigned char* tail = s_out + kGEpiWarps * kGStageOutBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(tail);   // [kGStages]
  uint64_t* empty = full + kGStages;                     // [kGStages]
  uint64_t* acc_full = empty + kGStages;                 // [2]
  uint64_t* acc_empty = acc_full + 2;                    // [2]
  uint64_t* tr_full = acc_empty + 2;                     // [kGTileRing] loading warp -> MMA, epilogue: a tile number is in the ring
  uint64_t* tr_empty = tr_full + kGTileRing;             // [kGTileRing] MMA thread and one lane per epilogue warp have read it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tr_empty + kGTileRing);
  int* tile_ring = reinterpret_cast<int*>(tmem_slot + 2);    // [kGTileRing] tile number, negative = no more tiles
  float* s_bias = reinterpret_cast<float*>(tail + 256);   // [2][kGN] bias of the tile in flight (double buffered), 16-byte aligned
  static_assert((2 * kGStages + 4 + 2 * kGTileRing) * 8 + 8 + kGTileRing * 4 <= 256, "barrier area of the shared-memory tail");

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int tiles_m = (p.M + kGM - 1) / kGM, tiles_n = (p.N + kGN - 1) / kGN;
  const int n_tiles = tiles_m * tiles_n;
  const int elems_per_slab = p.in_dtype == MINTB_E4M3 ? 128 : 64;
  const int n_slabs = (p.K + elems_per_slab - 1) / elems_per_slab;

  if (tid == 0) {
    for (int s = 0; s < kGStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], kGEpiThreads); }
    for (int s = 0; s < kGTileRing; ++s) { mbar_init(&tr_full[s], 1); mbar_init(&tr_empty[s], 1 + kGEpiWarps); }
    fence_mbar_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tensormap(&map_a);
      prefetch_tensormap(&map_b);
      // Tiles are drawn from the launch's work counter (the first one is the CTA's own number), so a CTA that shares its SM
      // with another kernel for a while - a collective of the gradient exchange, say - simply takes fewer tiles instead of
      // holding the whole grid up.  The tile numbers reach the other roles through a small ring.
      uint32_t stage = 0, phase = 0, n_drawn = 0;
      bool ok = true;
      for (;;) {
        const uint32_t slot = n_drawn % kGTileRing;
        ok = mbar_wait(&tr_empty[slot], ((n_drawn / kGTileRing) & 1) ^ 1, p.status, 0x705);
        if (!ok) break;
        int t = n_drawn == 0 ? int(blockIdx.x) : int(gridDim.x) + atomicAdd(p.sched, 1);
        if (t >= n_tiles) t = -1;
        tile_ring[slot] = t;
        mbar_arrive(&tr_full[slot]);
        ++n_drawn;
        if (t < 0) break;
        const int m0 = (t / tiles_n) * kGM, n0 = (t % tiles_n) * kGN;
        for (int kb = 0; kb < n_slabs; ++kb) {
          ok = mbar_wait(&empty[stage], phase ^ 1, p.status, 0x701);
          if (!ok) break;
          unsigned char* a = smem + size_t(stage) * kGStageBytes;
          mbar_expect_tx(&full[stage], kGStageBytes);
          tma_load_2d(a, &map_a, &full[stage], kb * elems_per_slab, m0);
          tma_load_2d(a + kABytes, &map_b, &full[stage], kb * elems_per_slab, n0);
          if (++stage == kGStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
      }
      leave_tile_counter(p.sched, int(gridDim.x));
    }
  } else if (warp == 1) {
    // All lanes run the loop and one elected lane issues: with warp-uniform control flow and operands the descriptors stay
    // in uniform registers, which is what tcgen05.mma reads; issued from a single-lane region every instruction first has
    // to move its operands there, and at 8-bit rates (one 128 x 256 x 32-byte instruction per 128 cycles) the issuing
    // thread is then the bottleneck.
    const bool leader = elect_one();
    auto wait_all = [&](uint64_t* bar, uint32_t parity, int code) -> bool {
      return __all_sync(0xffffffffu, mbar_wait(bar, parity, p.status, code));
    };
    const bool f8 = p.in_dtype == MINTB_E4M3;
    const uint32_t idesc = f8 ? idesc_e4m3(kGM, kGN) : idesc_bf16(kGM, kGN, false, false);
    constexpr uint32_t kHi = desc_hi32(8 * kSlabBytes, kSw128);
    const uint32_t a_lo0 = desc_addr32(__shfl_sync(0xffffffffu, smem_u32(smem), 0)) + desc_lbo32(16);
    const uint32_t tbase_u = __shfl_sync(0xffffffffu, tbase, 0);
    uint32_t stage = 0, phase = 0, ab = 0, ab_phase = 0, n_seen = 0;
    bool ok = true;
    for (;;) {
      const uint32_t slot = n_seen % kGTileRing;
      ok = wait_all(&tr_full[slot], (n_seen / kGTileRing) & 1, 0x706);
      if (!ok) break;
      const int t = __shfl_sync(0xffffffffu, tile_ring[slot], 0);
      if (leader) mbar_arrive(&tr_empty[slot]);
      ++n_seen;
      if (t < 0) break;
      ok = wait_all(&acc_empty[ab], ab_phase ^ 1, 0x702);
      if (!ok) break;
      tc_fence_after();
      const uint32_t d = tbase_u + ab * kGN;
      for (int kb = 0; kb < n_slabs; ++kb) {
        ok = wait_all(&full[stage], phase, 0x703);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_lo = a_lo0 + stage * (kGStageBytes >> 4), b_lo = a_lo + (kABytes >> 4);
        if (leader) {
          if (f8) {
#pragma unroll
            for (int k = 0; k < 4; ++k) umma_ss_f8(d, make_desc(kHi, a_lo + 2 * k), make_desc(kHi, b_lo + 2 * k), idesc, kb > 0 || k > 0);
          } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) umma_ss(d, make_desc(kHi, a_lo + 2 * k), make_desc(kHi, b_lo + 2 * k), idesc, kb > 0 || k > 0);
          }
          umma_commit(&empty[stage]);
        }
        __syncwarp();
        if (++stage == kGStages) { stage = 0; phase ^= 1; }
      }
      if (!ok) break;
      if (leader) umma_commit(&acc_full[ab]);
      __syncwarp();
      if (++ab == 2) { ab = 0; ab_phase ^= 1; }
    }
  } else {
    // eight warps: warp w works on TMEM lanes 32 (w % 4) ... (the quarter it may access) and on column half (w - 2) / 4
    const int quarter = warp % 4;
    const int chalf = (warp - 2) / 4;
    const int row = quarter * 32 + lane;
    const int et = (warp - 2) * 32 + lane;   // thread index among the epilogue threads
    unsigned char* my_out = s_out + size_t(warp - 2) * kGStageOutBytes;   // bf16 rows (1024-byte aligned: 64-byte swizzle)
    unsigned char* my_out8 = my_out + 32 * 64;                            // e4m3 rows
    // 32 columns of this warp's 32 rows as bf16 -> shared memory (row = lane) -> one bulk tensor store: whole 64-byte row
    // pieces reach L2 instead of one 16-byte piece per lane and instruction; rows / columns past the matrix are dropped.
    // With an e4m3 result beside a bf16 one the two stores of a chunk alternate between the two staging areas, so each
    // waits only for the store before the last one (its own area's previous use), not for the one just issued.
    auto bulk_store32 = [&](const CUtensorMap* map, const float (&val)[32], int n, int row0) {
      if (lane == 0) {   // the previous store from these staging rows has read them
        if (p.alt_stores) bulk_wait_read_but_one(); else bulk_wait_read_all();
      }
      __syncwarp();
#pragma unroll
      for (int j = 0; j < 32; j += 8)
        *reinterpret_cast<uint4*>(my_out + swizzled_offset(lane, j / 8, 64)) =
            make_uint4(pack_bf16x2(val[j], val[j + 1]), pack_bf16x2(val[j + 2], val[j + 3]), pack_bf16x2(val[j + 4], val[j + 5]),
                       pack_bf16x2(val[j + 6], val[j + 7]));
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(map, my_out, n, row0);
        bulk_commit_group();
      }
    };
    // the same for an e4m3 result: 32 rows x 32 bytes, rows unswizzled
    auto bulk_store32_f8 = [&](const CUtensorMap* map, const float (&val)[32], int n, int row0) {
      if (lane == 0) {
        if (p.alt_stores) bulk_wait_read_but_one(); else bulk_wait_read_all();
      }
      __syncwarp();
      uint4 o[2];
      __nv_fp8x2_storage_t* op = reinterpret_cast<__nv_fp8x2_storage_t*>(o);
      const uint64_t os2 = pack2(p.out_scale, p.out_scale);
#pragma unroll
      for (int j = 0; j < 32; j += 2) {   // the conversion itself saturates at +-448
        float a, b;
        unpack2(fmul2(pack2(val[j], val[j + 1]), os2), a, b);
        op[j / 2] = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
      }
      *reinterpret_cast<uint4*>(my_out8 + lane * 32) = o[0];
      *reinterpret_cast<uint4*>(my_out8 + lane * 32 + 16) = o[1];
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(map, my_out8, n, row0);
        bulk_commit_group();
      }
    };
    // Head-major outputs: the 32 columns (64 bytes) of a row go to one place of q / k / v, rows lie far apart.  Staged like
    // above and read back so that four neighbouring lanes write the four 16-byte pieces of one row: every store instruction
    // covers whole 64-byte runs (eight rows) instead of one 16-byte piece of each of 32 rows.  `row_off` is this lane's row
    // offset in elements (negative: row not stored), `col_off` what the chunk adds; HD = 16 splits the chunk over two heads
    // (`head_step` elements apart).
    auto scatter_store32 = [&](__nv_bfloat16* base, const float (&val)[32], long long row_off, size_t col_off, size_t head_step) {
      // (the head-major kernels issue no bulk stores, so nothing else reads the staging rows)
#pragma unroll
      for (int j = 0; j < 32; j += 8)
        *reinterpret_cast<uint4*>(my_out + swizzled_offset(lane, j / 8, 64)) =
            make_uint4(pack_bf16x2(val[j], val[j + 1]), pack_bf16x2(val[j + 2], val[j + 3]), pack_bf16x2(val[j + 4], val[j + 5]),
                       pack_bf16x2(val[j + 6], val[j + 7]));
      __syncwarp();
      const int piece = lane % 4;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = i * 8 + lane / 4;
        const long long ro = __shfl_sync(0xffffffffu, row_off, r);
        const uint4 q = *reinterpret_cast<const uint4*>(my_out + swizzled_offset(r, piece, 64));
        if (ro >= 0) {
          const size_t within = HD == 16 ? size_t(piece / 2) * head_step + size_t(piece % 2) * 8 : size_t(piece) * 8;
          *reinterpret_cast<uint4*>(base + size_t(ro) + col_off + within) = q;
        }
      }
      __syncwarp();
    };
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    uint32_t ab = 0, ab_phase = 0, n_seen = 0;
    bool ok = true;
    for (;;) {
      const uint32_t slot = n_seen % kGTileRing;
      ok = mbar_wait(&tr_full[slot], (n_seen / kGTileRing) & 1, p.status, 0x707);
      if (!ok) break;
      const int t = tile_ring[slot];
      __syncwarp();
      if (lane == 0) mbar_arrive(&tr_empty[slot]);
      ++n_seen;
      if (t < 0) break;
      const int m0 = (t / tiles_n) * kGM, n0 = (t % tiles_n) * kGN;
      const int m = m0 + row;
      float* bias_t = s_bias + ab * kGN;
      for (int j = et; j < kGN; j += kGEpiThreads) bias_t[j] = (p.bias != nullptr && n0 + j < p.N) ? load_bias(p.bias, p.bias_dtype, n0 + j) : 0.f;
      named_bar_sync(1, kGEpiThreads);
      ok = mbar_wait(&acc_full[ab], ab_phase, p.status, 0x704);
      if (!ok) break;
      tc_fence_after();
      const uint32_t tacc = tbase + lane_base + ab * kGN;
      int hm_b = 0, hm_t = 0;   // head-major: decode the row once
      long long hm_row = -1;    // element offset of (b, head 0, t, 0) in q / k / v, negative for rows past M
      if constexpr (EPI == kEpiHeadMajor) {
        // rows past M (the ragged last tile) compute on token 0 and are not stored: their table reads stay in range
        const int mo = m < p.M ? (p.row_map != nullptr ? p.row_map[m] : m) : 0;
        hm_t = mo / p.B;
        hm_b = mo % p.B;
        if (m < p.M) hm_row = (static_cast<long long>(hm_b) * p.H * p.T + hm_t) * HD;
      }
      // one chunk of 32 columns, its accumulator values already in registers
      auto do_chunk = [&](const int c0, const uint32_t (&r)[32]) {
        float v[32];
        // (two-pathway QKV projection: the columns of the second pathway carry their own multiplier)
        const float al = (EPI == kEpiHeadMajor && n0 + c0 >= 3 * p.H * HD) ? p.alpha2 : p.alpha;
        {
          const uint64_t al2 = pack2(al, al);
          const float4* b4 = reinterpret_cast<const float4*>(bias_t + c0);
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const float4 bb = b4[j / 4];
            unpack2(ffma2(pack2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), al2, pack2(bb.x, bb.y)), v[j], v[j + 1]);
            unpack2(ffma2(pack2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])), al2, pack2(bb.z, bb.w)), v[j + 2], v[j + 3]);
          }
        }
        if constexpr (EPI == kEpiHeadMajor) {
          // column n = which * E + h * HD + d, which = 0..2 (q, k, v of the first pathway) or 3..5 (of the second, never
          // rotated).  E is a multiple of 32 (of 64 when HD = 64), so a 32-column chunk lies in one third and covers whole
          // heads (HD = 16: two, HD = 32: one) or one half of a head (HD = 64).
          const int E = p.H * HD;
          const int n = n0 + c0;
          const int which = n / E, e = n % E;
          const bool rot = p.rope_cos != nullptr && which < 2;
          if (which == 0 || which == 3) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= p.q_scale;
          }
          if constexpr (HD <= 32) {
            constexpr int hd = HD / 2;
            if (rot) {
#pragma unroll
              for (int j = 0; j < hd; j += 4) {   // table rows are read 16 bytes at a time
                const float4 c4 = __ldg(reinterpret_cast<const float4*>(p.rope_cos + size_t(hm_t) * hd + j));
                const float4 s4 = __ldg(reinterpret_cast<const float4*>(p.rope_sin + size_t(hm_t) * hd + j));
                const float cs[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                for (int h0 = 0; h0 < 32; h0 += HD) {
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float a = v[h0 + j + e], bb = v[h0 + j + e + hd];
                    v[h0 + j + e] = a * cs[e] - bb * sn[e];
                    v[h0 + j + e + hd] = bb * cs[e] + a * sn[e];
                  }
                }
              }
            }
            // the chunk starts at head e / HD (HD = 16: and covers the next one too), heads are T * HD elements apart
            scatter_store32(p.qkv[which], v, hm_row, size_t(e / HD) * p.T * HD, size_t(p.T) * HD);
          }
          // (head size 64 does not come here: its loop below works on whole heads)
        } else {
          const int n = n0 + c0;
          if (p.resid != nullptr) {   // res_a * resid + res_b * (projection): the residual sum of the layer, formed here
            if (m < p.M) {
              const __nv_bfloat16* rr = p.resid + size_t(m) * p.N + n;
              if (n + 32 <= p.N) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  const uint4 q = __ldg(reinterpret_cast<const uint4*>(rr + j));
                  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 f = __bfloat1622float2(h2[e]);
                    v[j + 2 * e] = fmaf(p.res_a, f.x, p.res_b * v[j + 2 * e]);
                    v[j + 2 * e + 1] = fmaf(p.res_a, f.y, p.res_b * v[j + 2 * e + 1]);
                  }
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (n + j < p.N) v[j] = fmaf(p.res_a, __bfloat162float(rr[j]), p.res_b * v[j]);
              }
            }
          }
          if constexpr (EPI == kEpiBias) {
            // the value itself in bf16 beside an e4m3 result (the bf16 copy the layer keeps, the e4m3 copy the next projection reads)
            if (p.preact != nullptr) {
              if (p.use_bulk_store) {
                bulk_store32(&map_pre, v, n, m0 + quarter * 32);
              } else if (m < p.M) {
                __nv_bfloat16* dst = p.preact + size_t(m) * p.N + n;
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (n + j < p.N) dst[j] = __float2bfloat16_rn(v[j]);
              }
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = __bfloat162float(__float2bfloat16_rn(v[j]));   // the e4m3 copy is taken from the bf16 values
            }
          }
          if constexpr (EPI == kEpiBiasGelu) {
            if (p.preact != nullptr && p.use_bulk_store) {
              bulk_store32(&map_pre, v, n, m0 + quarter * 32);
            } else if (p.preact != nullptr && m < p.M) {   // the backward pass reads the pre-activation instead of recomputing it
              __nv_bfloat16* dst = p.preact + size_t(m) * p.N + n;
              if (n + 32 <= p.N) {
#pragma unroll
                for (int j = 0; j < 32; j += 8)
                  *reinterpret_cast<uint4*>(dst + j) = make_uint4(pack_bf16x2(v[j], v[j + 1]), pack_bf16x2(v[j + 2], v[j + 3]),
                                                                  pack_bf16x2(v[j + 4], v[j + 5]), pack_bf16x2(v[j + 6], v[j + 7]));
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (n + j < p.N) dst[j] = __float2bfloat16_rn(v[j]);
              }
            }
#pragma unroll
            for (int j = 0; j < 32; j += 2) gelu_erf2(v[j], v[j + 1]);
          }
          if (p.use_bulk_store && p.out_dtype == MINTB_BF16) {
            bulk_store32(&map_out, v, n, m0 + quarter * 32);
          } else if (p.use_bulk_f8) {
            bulk_store32_f8(&map_out, v, n, m0 + quarter * 32);
          } else if (m < p.M) {
            if (p.out_dtype == MINTB_BF16) {
              __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + size_t(m) * p.N + n;
              if (n + 32 <= p.N) {
#pragma unroll
                for (int j = 0; j < 32; j += 8)
                  *reinterpret_cast<uint4*>(dst + j) = make_uint4(pack_bf16x2(v[j], v[j + 1]), pack_bf16x2(v[j + 2], v[j + 3]),
                                                                  pack_bf16x2(v[j + 4], v[j + 5]), pack_bf16x2(v[j + 6], v[j + 7]));
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (n + j < p.N) dst[j] = __float2bfloat16_rn(v[j]);
              }
            } else {
              __nv_fp8_storage_t* dst = static_cast<__nv_fp8_storage_t*>(p.out) + size_t(m) * p.N + n;
              if (n + 32 <= p.N && (p.N & 15) == 0) {   // 16-byte stores need 16-byte aligned rows
                uint4 o[2];
                __nv_fp8_storage_t* op = reinterpret_cast<__nv_fp8_storage_t*>(o);
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  op[j] = __nv_cvt_float_to_fp8(v[j] * p.out_scale, __NV_SATFINITE, __NV_E4M3);
                *reinterpret_cast<uint4*>(dst) = o[0];
                *reinterpret_cast<uint4*>(dst + 16) = o[1];
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (n + j < p.N)
                    dst[j] = __nv_cvt_float_to_fp8(v[j] * p.out_scale, __NV_SATFINITE, __NV_E4M3);
              }
            }
          }
        }
      };
      // The TMEM load of the next chunk is issued before the arithmetic and the stores of the current one (head size 64
      // has its own loop).
      const int cbeg = chalf * (kGN / 2), cend = (chalf + 1) * (kGN / 2);
      if constexpr (EPI == kEpiHeadMajor && HD == 64) {
        // One head (64 columns: the lower and the upper half the rotation pairs up) of q, k or v per step: both halves
        // arrive with one TMEM round trip and the table rows are on their way while it lasts.  (E is a multiple of 64 and
        // the tile's columns start at a multiple of 256, so a step never straddles a head or a third.)
#pragma unroll 1
        for (int c0 = cbeg; c0 < cend; c0 += 64) {
          if (n0 + c0 >= p.N) break;   // uniform
          uint32_t ra[32], rb[32];
          tmem_ld32(tacc + c0, ra);
          tmem_ld32(tacc + c0 + 32, rb);
          const int E = p.H * 64;
          const int n = n0 + c0;
          const int which = n / E, e = n % E;
          const bool rot = p.rope_cos != nullptr && which < 2;
          const float al = n >= 3 * E ? p.alpha2 : p.alpha;
          // the first halves of the token's two table rows (128 bytes each) now, the second halves (then in L1) when needed
          const float4* cos4 = reinterpret_cast<const float4*>(p.rope_cos + size_t(hm_t) * 32);
          const float4* sin4 = reinterpret_cast<const float4*>(p.rope_sin + size_t(hm_t) * 32);
          float4 cs[4], sn[4];
          if (rot) {
#pragma unroll
            for (int j = 0; j < 4; ++j) { cs[j] = __ldg(cos4 + j); sn[j] = __ldg(sin4 + j); }
          }
          tmem_ld_wait();
          float lo[32], hi[32];
          {
            const float mul = (which == 0 || which == 3) ? p.q_scale : 1.f;   // (x al + b) q_scale
            const uint64_t al2 = pack2(al * mul, al * mul), m2 = pack2(mul, mul);
            const float4* b4 = reinterpret_cast<const float4*>(bias_t + c0);
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              const float4 bl = b4[j / 4], bh = b4[8 + j / 4];
              unpack2(ffma2(pack2(__uint_as_float(ra[j]), __uint_as_float(ra[j + 1])), al2, fmul2(pack2(bl.x, bl.y), m2)), lo[j], lo[j + 1]);
              unpack2(ffma2(pack2(__uint_as_float(ra[j + 2]), __uint_as_float(ra[j + 3])), al2, fmul2(pack2(bl.z, bl.w), m2)), lo[j + 2], lo[j + 3]);
              unpack2(ffma2(pack2(__uint_as_float(rb[j]), __uint_as_float(rb[j + 1])), al2, fmul2(pack2(bh.x, bh.y), m2)), hi[j], hi[j + 1]);
              unpack2(ffma2(pack2(__uint_as_float(rb[j + 2]), __uint_as_float(rb[j + 3])), al2, fmul2(pack2(bh.z, bh.w), m2)), hi[j + 2], hi[j + 3]);
            }
          }
          if (rot) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              if (half == 1) {
#pragma unroll
                for (int j = 0; j < 4; ++j) { cs[j] = __ldg(cos4 + 4 + j); sn[j] = __ldg(sin4 + 4 + j); }
              }
#pragma unroll
              for (int j = 0; j < 16; j += 4) {
                const float c4[4] = {cs[j / 4].x, cs[j / 4].y, cs[j / 4].z, cs[j / 4].w};
                const float s4[4] = {sn[j / 4].x, sn[j / 4].y, sn[j / 4].z, sn[j / 4].w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const float a = lo[16 * half + j + q], bb = hi[16 * half + j + q];
                  lo[16 * half + j + q] = a * c4[q] - bb * s4[q];
                  hi[16 * half + j + q] = bb * c4[q] + a * s4[q];
                }
              }
            }
          }
          scatter_store32(p.qkv[which], lo, hm_row, size_t(e / 64) * p.T * 64, 0);
          scatter_store32(p.qkv[which], hi, hm_row, size_t(e / 64) * p.T * 64 + 32, 0);
        }
      } else {
        uint32_t ra[32], rb[32];
        tmem_ld32(tacc + cbeg, ra);
#pragma unroll 1
        for (int c0 = cbeg; c0 < cend; c0 += 64) {
          if (n0 + c0 >= p.N) break;   // uniform
          tmem_ld_wait();
          tmem_ld32(tacc + c0 + 32, rb);
          do_chunk(c0, ra);
          if (n0 + c0 + 32 >= p.N) break;   // uniform
          tmem_ld_wait();
          if (c0 + 64 < cend) tmem_ld32(tacc + c0 + 64, ra);
          do_chunk(c0 + 32, rb);
        }
        tmem_ld_wait();   // (a load issued ahead of a chunk that was not processed)
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[ab]);
      if (++ab == 2) { ab = 0; ab_phase ^= 1; }
    }
    if (lane == 0) bulk_wait_read_all();   // the bulk stores have read their staging rows (the kernel boundary orders their writes)
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tbase, 512);
  }
}

// x (bf16) -> e4m3 with a per-tensor scale: q = sat(x * inv_scale); 16 elements per thread.  The conversion saturates
// finite values at +-448 and keeps a NaN a NaN (an explicit clamp would turn it into -448 and hide a diverged run).
__global__ void __launch_bounds__(256) quantize_e4m3_kernel(const __nv_bfloat16* __restrict__ x, __nv_fp8_storage_t* __restrict__ out,
                                                            size_t n, float inv_scale) {
  const size_t i = (size_t(blockIdx.x) * blockDim.x + threadIdx.x) * 16;
  if (i >= n) return;
  if (i + 16 <= n) {
    const uint4 a = *reinterpret_cast<const uint4*>(x + i), b = *reinterpret_cast<const uint4*>(x + i + 8);
    const __nv_bfloat16* ap = reinterpret_cast<const __nv_bfloat16*>(&a);
    const __nv_bfloat16* bp = reinterpret_cast<const __nv_bfloat16*>(&b);
    uint4 o;
    __nv_fp8_storage_t* op = reinterpret_cast<__nv_fp8_storage_t*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      op[j] = __nv_cvt_float_to_fp8(__bfloat162float(ap[j]) * inv_scale, __NV_SATFINITE, __NV_E4M3);
      op[8 + j] = __nv_cvt_float_to_fp8(__bfloat162float(bp[j]) * inv_scale, __NV_SATFINITE, __NV_E4M3);
    }
    *reinterpret_cast<uint4*>(out + i) = o;
  } else {
    for (size_t j = i; j < n; ++j)
      out[j] = __nv_cvt_float_to_fp8(__bfloat162float(x[j]) * inv_scale, __NV_SATFINITE, __NV_E4M3);
  }
}

// ------------------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn gemm_encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// [rows][K] matrix, K contiguous; box = (128 bytes of K, box_rows); out-of-range parts read as zero.
static bool gemm_map(CUtensorMap* m, const void* ptr, int rows, int K, int dtype, int box_rows) {
  EncodeTiledFn fn = gemm_encode_fn();
  if (fn == nullptr) return false;
  const int esz = dtype == MINTB_E4M3 ? 1 : 2;
  cuuint64_t dims[2] = {cuuint64_t(K), cuuint64_t(rows)};
  cuuint64_t strides[1] = {cuuint64_t(K) * esz};
  cuuint32_t box[2] = {cuuint32_t(kSlabBytes / esz), cuuint32_t(box_rows)};
  cuuint32_t es[2] = {1, 1};
  return fn(m, dtype == MINTB_E4M3 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims,
            strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// bf16 [rows][N] output, box = (32 columns, 32 rows) with 64B swizzle: the unit one epilogue warp stores at a time
static bool gemm_out_map(CUtensorMap* m, const void* ptr, int rows, int N) {
  EncodeTiledFn fn = gemm_encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {cuuint64_t(N), cuuint64_t(rows)};
  cuuint64_t strides[1] = {cuuint64_t(N) * 2};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t es[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// e4m3 [rows][N] output, box = (32 bytes, 32 rows), no swizzle
static bool gemm_out_map_f8(CUtensorMap* m, const void* ptr, int rows, int N) {
  EncodeTiledFn fn = gemm_encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {cuuint64_t(N), cuuint64_t(rows)};
  cuuint64_t strides[1] = {cuuint64_t(N)};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t es[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int launch_gemm(const GemmParams& p_in, const void* x, const void* w, cudaStream_t stream) {
  GemmParams p = p_in;
  CUtensorMap ma, mb;
  if (!gemm_map(&ma, x, p.M, p.K, p.in_dtype, kGM) || !gemm_map(&mb, w, p.N, p.K, p.in_dtype, kGN)) {
    set_error("mintb gemm: cuTensorMapEncodeTiled failed");
    return MINTB_ECUDA;
  }
  // row-major bf16 outputs (and the pre-activation copy) go out as bulk tensor stores when their rows are 16-byte multiples
  CUtensorMap mo = ma, mp = ma;   // placeholders when unused
  p.use_bulk_store = 0;
  // (with an e4m3 result only the bf16 pre-activation copy takes this route)
  if (p.epilogue != kEpiHeadMajor && p.N % 8 == 0 && (p.out_dtype == MINTB_BF16 || p.preact != nullptr)) {
    if ((p.out_dtype == MINTB_BF16 && !gemm_out_map(&mo, p.out, p.M, p.N)) ||
        (p.preact != nullptr && !gemm_out_map(&mp, p.preact, p.M, p.N))) {
      set_error("mintb gemm: cuTensorMapEncodeTiled failed for the output");
      return MINTB_ECUDA;
    }
    p.use_bulk_store = 1;
  }
  p.use_bulk_f8 = 0;
  if (p.epilogue != kEpiHeadMajor && p.out_dtype == MINTB_E4M3 && p.N % 16 == 0) {
    if (!gemm_out_map_f8(&mo, p.out, p.M, p.N)) {
      set_error("mintb gemm: cuTensorMapEncodeTiled failed for the e4m3 output");
      return MINTB_ECUDA;
    }
    p.use_bulk_f8 = 1;
  }
  p.alt_stores = (p.use_bulk_f8 && p.use_bulk_store && p.preact != nullptr) ? 1 : 0;
  void (*kern)(CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, GemmParams) = nullptr;
  if (p.epilogue == kEpiBias) kern = gemm_tc_kernel<kEpiBias, 0>;
  else if (p.epilogue == kEpiBiasGelu) kern = gemm_tc_kernel<kEpiBiasGelu, 0>;
  else if (p.D == 16) kern = gemm_tc_kernel<kEpiHeadMajor, 16>;
  else if (p.D == 32) kern = gemm_tc_kernel<kEpiHeadMajor, 32>;
  else kern = gemm_tc_kernel<kEpiHeadMajor, 64>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kGemmSmem));
  if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return MINTB_ECUDA; }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int tiles = ((p.M + kGM - 1) / kGM) * ((p.N + kGN - 1) / kGN);
  const int grid = tiles < sms ? tiles : sms;
  if (int rc = next_tile_counter(&p.sched); rc != MINTB_OK) return rc;
  kern<<<grid, kGThreads, kGemmSmem, stream>>>(ma, mb, mo, mp, p);
  count_launches(1);
  e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("gemm launch: %s", cudaGetErrorString(e)); return MINTB_ECUDA; }
  return MINTB_OK;
}

cudaError_t launch_quantize_e4m3(const void* x, void* out, size_t n, float inv_scale, cudaStream_t s) {
  const size_t threads = (n + 15) / 16;
  quantize_e4m3_kernel<<<unsigned((threads + 255) / 256), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x),
                                                                     static_cast<__nv_fp8_storage_t*>(out), n, inv_scale);
  count_launches(1);
  return cudaGetLastError();
}

}  // namespace mintb

using namespace mintb;

static int check_gemm(const char* who, const void* x, const void* w, int M, int N, int K, int in_dtype) {
  if (x == nullptr || w == nullptr || M <= 0 || N <= 0 || K <= 0) {
    set_error("%s: x, w and positive M, N, K are required", who);
    return MINTB_EINVAL;
  }
  if (in_dtype != MINTB_BF16 && in_dtype != MINTB_E4M3) {
    set_error("%s: operands must be bf16 or e4m3", who);
    return MINTB_EUNSUPPORTED;
  }
  const int esz = in_dtype == MINTB_E4M3 ? 1 : 2;
  if ((size_t(K) * esz) % 16 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) {
    set_error("%s: rows of x and w must be 16-byte aligned (K * element size a multiple of 16)", who);
    return MINTB_EINVAL;
  }
  return MINTB_OK;
}

extern "C" int mintb_linear_fwd(const void* x, const void* w, const void* bias, void* out, void* preact_out, int M, int N, int K,
                                int in_dtype, int bias_dtype, int out_dtype, int gelu, float alpha, float out_scale, void* stream,
                                int* dev_status) {
  int rc = check_gemm("mintb_linear_fwd", x, w, M, N, K, in_dtype);
  if (rc != MINTB_OK) return rc;
  if (out == nullptr || (out_dtype != MINTB_BF16 && out_dtype != MINTB_E4M3) || (reinterpret_cast<uintptr_t>(out) & 15) ||
      (out_dtype == MINTB_BF16 && N % 8 != 0)) {
    set_error("mintb_linear_fwd: out must be a 16-byte aligned bf16 (N a multiple of 8) or e4m3 buffer");
    return MINTB_EINVAL;
  }
  if (preact_out != nullptr && (!gelu || N % 8 != 0 || (reinterpret_cast<uintptr_t>(preact_out) & 15))) {
    set_error("mintb_linear_fwd: preact_out goes with gelu, N a multiple of 8 and a 16-byte aligned buffer");
    return MINTB_EINVAL;
  }
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.in_dtype = in_dtype; p.out_dtype = out_dtype; p.bias_dtype = bias_dtype;
  p.epilogue = gelu ? kEpiBiasGelu : kEpiBias;
  p.alpha = alpha; p.out_scale = out_scale; p.bias = bias; p.out = out; p.status = dev_status;
  p.preact = static_cast<__nv_bfloat16*>(preact_out);
  return launch_gemm(p, x, w, static_cast<cudaStream_t>(stream));
}

extern "C" int mintb_qkv_fwd(const void* x, const void* w, const void* bias, void* q, void* k, void* v, int T, int B, int H, int D,
                             int in_dtype, int bias_dtype, float alpha, float q_scale, const float* rope_cos,
                             const float* rope_sin, const int32_t* row_map, int n_rows, void* stream, int* dev_status) {
  const int E = H * D;
  const int M = row_map != nullptr ? n_rows : T * B;
  int rc = check_gemm("mintb_qkv_fwd", x, w, M, 3 * E, E, in_dtype);
  if (rc != MINTB_OK) return rc;
  if (q == nullptr || k == nullptr || v == nullptr || (D != 16 && D != 32 && D != 64) || T <= 0 || B <= 0 || H <= 0 ||
      E % (D == 64 ? 64 : 32) != 0) {
    set_error("mintb_qkv_fwd: q, k, v, head_dim 16, 32 or 64 and H * D a multiple of 32 (64 at head_dim 64) are required");
    return MINTB_EINVAL;
  }
  if ((rope_cos == nullptr) != (rope_sin == nullptr)) {
    set_error("mintb_qkv_fwd: give both RoPE tables or neither");
    return MINTB_EINVAL;
  }
  GemmParams p{};
  p.M = M; p.N = 3 * E; p.K = E; p.in_dtype = in_dtype; p.out_dtype = MINTB_BF16; p.bias_dtype = bias_dtype;
  p.epilogue = kEpiHeadMajor;
  p.row_map = row_map;
  p.alpha = alpha; p.alpha2 = alpha; p.out_scale = 1.f; p.bias = bias; p.out = nullptr;
  p.qkv[0] = static_cast<__nv_bfloat16*>(q); p.qkv[1] = static_cast<__nv_bfloat16*>(k); p.qkv[2] = static_cast<__nv_bfloat16*>(v);
  p.B = B; p.T = T; p.H = H; p.D = D; p.q_scale = q_scale; p.rope_cos = rope_cos; p.rope_sin = rope_sin;
  p.status = dev_status;
  return launch_gemm(p, x, w, static_cast<cudaStream_t>(stream));
}

extern "C" int mintb_linear_res_fwd(const void* x, const void* w, const void* bias, const void* resid, float res_a, float res_b, void* out,
                                    void* bf16_copy_out, int M, int N, int K, int in_dtype, int bias_dtype, int out_dtype, float alpha,
                                    float out_scale, void* stream, int* dev_status) {
  int rc = check_gemm("mintb_linear_res_fwd", x, w, M, N, K, in_dtype);
  if (rc != MINTB_OK) return rc;
  if (out == nullptr || (out_dtype != MINTB_BF16 && out_dtype != MINTB_E4M3) || (reinterpret_cast<uintptr_t>(out) & 15) || N % 8 != 0 ||
      (reinterpret_cast<uintptr_t>(resid) & 15) || (reinterpret_cast<uintptr_t>(bf16_copy_out) & 15) ||
      (bf16_copy_out != nullptr && out_dtype != MINTB_E4M3)) {
    set_error("mintb_linear_res_fwd: out must be a 16-byte aligned bf16 or e4m3 buffer, N a multiple of 8, resid and bf16_copy_out "
              "16-byte aligned, and bf16_copy_out goes with an e4m3 out");
    return MINTB_EINVAL;
  }
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.in_dtype = in_dtype; p.out_dtype = out_dtype; p.bias_dtype = bias_dtype;
  p.epilogue = kEpiBias;
  p.alpha = alpha; p.out_scale = out_scale; p.bias = bias; p.out = out; p.status = dev_status;
  p.preact = static_cast<__nv_bfloat16*>(bf16_copy_out);
  p.resid = static_cast<const __nv_bfloat16*>(resid); p.res_a = res_a; p.res_b = res_b;
  return launch_gemm(p, x, w, static_cast<cudaStream_t>(stream));
}

extern "C" int mintb_qkv2_fwd(const void* x, const void* w, const void* bias, void* q1, void* k1, void* v1, void* q2, void* k2, void* v2,
                              int T, int B, int H, int D, int in_dtype, int bias_dtype, float alpha1, float alpha2, float q_scale,
                              const float* rope_cos, const float* rope_sin, const int32_t* row_map, int n_rows, void* stream,
                              int* dev_status) {
  const int E = H * D;
  const int M = row_map != nullptr ? n_rows : T * B;
  int rc = check_gemm("mintb_qkv2_fwd", x, w, M, 6 * E, E, in_dtype);
  if (rc != MINTB_OK) return rc;
  if (q1 == nullptr || k1 == nullptr || v1 == nullptr || q2 == nullptr || k2 == nullptr || v2 == nullptr ||
      (D != 16 && D != 32 && D != 64) || T <= 0 || B <= 0 || H <= 0 || E % (D == 64 ? 64 : 32) != 0) {
    set_error("mintb_qkv2_fwd: six outputs, head_dim 16, 32 or 64 and H * D a multiple of 32 (64 at head_dim 64) are required");
    return MINTB_EINVAL;
  }
  if ((rope_cos == nullptr) != (rope_sin == nullptr)) {
    set_error("mintb_qkv2_fwd: give both RoPE tables or neither");
    return MINTB_EINVAL;
  }
  GemmParams p{};
  p.M = M; p.N = 6 * E; p.K = E; p.in_dtype = in_dtype; p.out_dtype = MINTB_BF16; p.bias_dtype = bias_dtype;
  p.epilogue = kEpiHeadMajor;
  p.row_map = row_map;
  p.alpha = alpha1; p.alpha2 = alpha2; p.out_scale = 1.f; p.bias = bias; p.out = nullptr;
  void* outs[6] = {q1, k1, v1, q2, k2, v2};
  for (int i = 0; i < 6; ++i) p.qkv[i] = static_cast<__nv_bfloat16*>(outs[i]);
  p.B = B; p.T = T; p.H = H; p.D = D; p.q_scale = q_scale; p.rope_cos = rope_cos; p.rope_sin = rope_sin;
  p.status = dev_status;
  return launch_gemm(p, x, w, static_cast<cudaStream_t>(stream));
}

extern "C" int mintb_quantize_e4m3(const void* x, void* out, size_t n, float inv_scale, void* stream) {
  if (x == nullptr || out == nullptr || n == 0 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) {
    set_error("mintb_quantize_e4m3: 16-byte aligned x and out and n > 0 are required");
    return MINTB_EINVAL;
  }
  cudaError_t e = launch_quantize_e4m3(x, out, n, inv_scale, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) { set_error("quantize launch: %s", cudaGetErrorString(e)); return MINTB_ECUDA; }
  return MINTB_OK;
}
