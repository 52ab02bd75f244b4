// tcgen05 GEMMs of the projections' backward pass (the products torch.autograd forms for nn.Linear / te.Linear):
//
//   dgrad   dx[M][K] = alpha (dz[M][N] w[N][K] + dz2[M][N2] w2[N2][K])      (the second pair is optional: two projections of
//                                                                            one activation add their input gradients here)
//   wgrad   dw[N][K] = alpha dz^T[N][M] x[M][K]
//
// Every matrix is row-major as the forward pass left it; nothing is transposed in memory.  A reduction index that is NOT the
// contiguous one of its matrix (w in dgrad; dz and x in wgrad) is fed to the tensor core as an "MN-major" operand: the copy
// engine loads [reduction rows][128 bytes of the other index] boxes with the 128-byte swizzle and the shared-memory
// descriptor names the block stride, so tcgen05.mma reads the tile transposed.  Operands are bf16 (kind::f16) or 8-bit
// floats (kind::f8f6f4: e5m2 gradients against e4m3 activations / weights), fp32 accumulation in TMEM.
//
// Persistent CTAs, one per SM, 128 x 256 output tiles, the roles of the forward GEMM: warp 0 TMA producer (4-stage ring of
// 128-byte reduction slabs), warp 1 MMA issuer (two 256-column accumulators), warps 2-9 epilogue.  dgrad stores bf16 through
// shared memory and bulk tensor stores.  wgrad reduces over the tokens, tens of thousands of them against a few hundred
// output tiles, so its reduction is cut into S aligned splits (S chosen on the host so that tiles x S fills the SMs
// evenly); every unit adds its fp32 partial tile to a zeroed fp32 matrix with bulk tensor reductions, and a small pass
// converts that matrix when the gradient is wanted in bf16.  Units of one split run together, so the CTAs march through
// the same token range at the same time and share their operand tiles in L2.  Every mbarrier wait is bounded.
#include "common.cuh"
#include "ptx.cuh"

namespace mintb {

using namespace ptx;

constexpr int kBM = 128, kBN = 256, kBStages = 4;
constexpr int kBABytes = kBM * 128, kBBBytes = kBN * 128, kBStageBytes = kBABytes + kBBBytes;
constexpr int kBEpiWarps = 8, kBEpiThreads = 32 * kBEpiWarps, kBThreads = 64 + kBEpiThreads;
constexpr int kBOutStageBytes = 32 * 128;   // one epilogue warp's staging: 32 rows x 128 bytes
constexpr size_t kBwdGemmSmem = 1024 + size_t(kBStages) * kBStageBytes + kBEpiWarps * kBOutStageBytes + 256;

enum BwdGemmMode : int { kDgrad = 0, kWgrad = 1 };

struct BwdGemmParams {
  int rows, cols;        // the output matrix
  int red1, red2;        // reduction lengths (elements) of the first and the second operand pair (red2 = 0: one pair)
  int f8;                // operands are 8-bit floats (else bf16)
  uint32_t idesc;        // instruction descriptor (formats, majors, M = 128, N = 256)
  int splits;            // aligned cuts of the reduction (wgrad); 1 for dgrad
  int n_full, pieces;    // the first n_full (split, tile) units run whole, the others in `pieces` aligned pieces (UnitMap)
  float alpha;
  int* status;
  int* sched;            // work counter pair of this launch (common.cuh)
};

// 2-D tiled reduction shared memory -> global (fp32 add); rows / columns outside the tensor are dropped.
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* m, const void* src, int c0, int c1) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(src)), "r"(c0), "r"(c1)
               : "memory");
}

__device__ __forceinline__ uint32_t bwd_pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// Work unit u: split = u / n_tiles (so the units of one split run together), tile = u % n_tiles with the column index
// fastest.  The loading warp draws unit numbers from the launch's work counter (the first one is the CTA's own number) and
// hands them to the other roles through a small ring, so a CTA that shares its SM with another kernel for a while simply
// takes fewer units instead of holding the whole grid up.
constexpr int kBUnitRing = 4;
// The units in launch order: first the n_full "large" units - (split, tile) pairs, split-major, each a tile's reduction over one
// of `splits` aligned cuts - then the remaining large units cut once more into `pieces` aligned pieces each (piece-major, so
// that the pieces in flight at one time cover the same reduction range).  The host chooses n_full as a whole number of
// rounds of the grid and `pieces` so that the last, partial round of large units becomes rounds of short ones.
struct UnitMap {
  int n_units, n_tiles, n_slabs, per_split, n_full, rem, sub;
  __device__ UnitMap(int n_tiles_, int n_slabs_, int splits, int n_full_, int pieces) {
    n_tiles = n_tiles_; n_slabs = n_slabs_;
    per_split = (n_slabs + splits - 1) / splits;
    const int n_large = n_tiles * splits;
    n_full = n_full_ < n_large ? n_full_ : n_large;
    rem = n_large - n_full;
    sub = (per_split + pieces - 1) / pieces;
    n_units = n_full + rem * pieces;
  }
  // false for a unit past the end of the reduction (it holds nothing)
  __device__ bool decode(int u, int& tile, int& kb0, int& kb1) const {
    int large = u, piece = -1;
    if (u >= n_full) { large = n_full + (u - n_full) % rem; piece = (u - n_full) / rem; }
    tile = large % n_tiles;
    kb0 = (large / n_tiles) * per_split;
    kb1 = kb0 + per_split < n_slabs ? kb0 + per_split : n_slabs;
    if (piece >= 0) {
      kb0 += piece * sub;
      kb1 = kb0 + sub < kb1 ? kb0 + sub : kb1;
    }
    return kb0 < kb1;
  }
};

template <int MODE>
__global__ void __launch_bounds__(kBThreads, 1)
gemm_bwd_kernel(const __grid_constant__ CUtensorMap map_a1, const __grid_constant__ CUtensorMap map_b1,
                const __grid_constant__ CUtensorMap map_a2, const __grid_constant__ CUtensorMap map_b2,
                const __grid_constant__ CUtensorMap map_out, BwdGemmParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* s_out = smem + size_t(kBStages) * kBStageBytes;   // [epilogue warp][32 rows][128 B]
  unsigned char* tail = s_out + kBEpiWarps * kBOutStageBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(tail);   // [kBStages]
  uint64_t* empty = full + kBStages;                     // [kBStages]
  uint64_t* acc_full = empty + kBStages;                 // [2]
  uint64_t* acc_empty = acc_full + 2;                    // [2]
  uint64_t* ur_full = acc_empty + 2;                     // [kBUnitRing] loading warp -> MMA, epilogue: a unit number is in the ring
  uint64_t* ur_empty = ur_full + kBUnitRing;             // [kBUnitRing] MMA thread and one lane per epilogue warp have read it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ur_empty + kBUnitRing);
  int* unit_ring = reinterpret_cast<int*>(tmem_slot + 2);   // [kBUnitRing] unit number, negative = no more units

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int tiles_n = (p.cols + kBN - 1) / kBN;
  const int n_tiles = ((p.rows + kBM - 1) / kBM) * tiles_n;
  const int epb = p.f8 ? 128 : 64;                       // operand elements per 128 bytes
  const int slabs1 = (p.red1 + epb - 1) / epb, slabs2 = (p.red2 + epb - 1) / epb;
  const int n_slabs = slabs1 + slabs2;
  const uint32_t blk_bytes = uint32_t(epb) * 128u;       // one block of an MN-major tile: epb reduction rows x 128 bytes

  if (tid == 0) {
    for (int s = 0; s < kBStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], kBEpiThreads); }
    for (int s = 0; s < kBUnitRing; ++s) { mbar_init(&ur_full[s], 1); mbar_init(&ur_empty[s], 1 + kBEpiWarps); }
    fence_mbar_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tensormap(&map_a1);
      prefetch_tensormap(&map_b1);
      uint32_t stage = 0, phase = 0, n_drawn = 0;
      bool ok = true, first = true;
      const UnitMap um(n_tiles, n_slabs, p.splits, p.n_full, p.pieces);
      int tile = 0, kb0 = 0, kb1 = 0;
      for (;;) {
        const uint32_t slot = n_drawn % kBUnitRing;
        ok = mbar_wait(&ur_empty[slot], ((n_drawn / kBUnitRing) & 1) ^ 1, p.status, 0x805);
        if (!ok) break;
        int u;
        do {   // the next unit that holds something
          u = first ? int(blockIdx.x) : int(gridDim.x) + atomicAdd(p.sched, 1);
          first = false;
        } while (u < um.n_units && !um.decode(u, tile, kb0, kb1));
        if (u >= um.n_units) u = -1;
        unit_ring[slot] = u;
        mbar_arrive(&ur_full[slot]);
        ++n_drawn;
        if (u < 0) break;
        const int m0 = (tile / tiles_n) * kBM, n0 = (tile % tiles_n) * kBN;
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(&empty[stage], phase ^ 1, p.status, 0x801);
          if (!ok) break;
          const bool second = kb >= slabs1;
          const CUtensorMap* ma = second ? &map_a2 : &map_a1;
          const CUtensorMap* mb = second ? &map_b2 : &map_b1;
          const int kk = (second ? kb - slabs1 : kb) * epb;       // first reduction element of the slab
          unsigned char* a = smem + size_t(stage) * kBStageBytes;
          unsigned char* b = a + kBABytes;
          mbar_expect_tx(&full[stage], kBStageBytes);
          if (MODE == kDgrad) {
            tma_load_2d(a, ma, &full[stage], kk, m0);             // rows of dz: reduction index contiguous
          } else {
            for (int blk = 0; blk < kBM / epb; ++blk)             // dz^T: [tokens][128 bytes of output rows]
              tma_load_2d(a + blk * blk_bytes, ma, &full[stage], m0 + blk * epb, kk);
          }
          for (int blk = 0; blk < kBN / epb; ++blk)               // w / x: [reduction rows][128 bytes of output columns]
            tma_load_2d(b + blk * blk_bytes, mb, &full[stage], n0 + blk * epb, kk);
          if (++stage == kBStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
      }
      leave_tile_counter(p.sched, int(gridDim.x));
    }
  } else if (warp == 1) {
    // All lanes run the loop and one elected lane issues (warp-uniform control flow and operands keep the descriptors in
    // uniform registers; from a single-lane region the issuing thread is the bottleneck at 8-bit rates).
    const bool leader = elect_one();
    auto wait_all = [&](uint64_t* bar, uint32_t parity, int code) -> bool {
      return __all_sync(0xffffffffu, mbar_wait(bar, parity, p.status, code));
    };
    constexpr uint32_t kHi = desc_hi32(8 * 128, kSw128);        // eight 128-byte rows per swizzle atom, either major
    const uint32_t lo0 = desc_addr32(__shfl_sync(0xffffffffu, smem_u32(smem), 0));
    const uint32_t tbase_u = __shfl_sync(0xffffffffu, tbase, 0);
    const uint32_t lbo_k = desc_lbo32(16), lbo_mn = desc_lbo32(blk_bytes);
    const uint32_t step_mn = p.f8 ? (32u * 128u) >> 4 : (16u * 128u) >> 4;   // one MMA consumes 32 (8-bit) or 16 reduction rows
    uint32_t stage = 0, phase = 0, ab = 0, ab_phase = 0, n_seen = 0;
    bool ok = true;
    const UnitMap um(n_tiles, n_slabs, p.splits, p.n_full, p.pieces);
    int tile, kb0, kb1;
    for (;;) {
      const uint32_t slot = n_seen % kBUnitRing;
      ok = wait_all(&ur_full[slot], (n_seen / kBUnitRing) & 1, 0x806);
      if (!ok) break;
      const int u = __shfl_sync(0xffffffffu, unit_ring[slot], 0);
      if (leader) mbar_arrive(&ur_empty[slot]);
      ++n_seen;
      if (u < 0) break;
      um.decode(u, tile, kb0, kb1);
      ok = wait_all(&acc_empty[ab], ab_phase ^ 1, 0x802);
      if (!ok) break;
      tc_fence_after();
      const uint32_t d = tbase_u + ab * kBN;
      for (int kb = kb0; kb < kb1; ++kb) {
        ok = wait_all(&full[stage], phase, 0x803);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_lo = lo0 + stage * (kBStageBytes >> 4), b_lo = a_lo + (kBABytes >> 4);
        if (leader) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t da = MODE == kDgrad ? make_desc(kHi, a_lo + lbo_k + 2 * k) : make_desc(kHi, a_lo + lbo_mn + k * step_mn);
            const uint64_t db = make_desc(kHi, b_lo + lbo_mn + k * step_mn);
            if (p.f8) umma_ss_f8(d, da, db, p.idesc, kb > kb0 || k > 0);
            else umma_ss(d, da, db, p.idesc, kb > kb0 || k > 0);
          }
          umma_commit(&empty[stage]);
        }
        __syncwarp();
        if (++stage == kBStages) { stage = 0; phase ^= 1; }
      }
      if (!ok) break;
      if (leader) umma_commit(&acc_full[ab]);
      __syncwarp();
      if (++ab == 2) { ab = 0; ab_phase ^= 1; }
    }
  } else {
    // eight warps: warp w works on TMEM lanes 32 (w % 4) ... and on column half (w - 2) / 4 of the tile
    const int quarter = warp % 4;
    const int chalf = (warp - 2) / 4;
    unsigned char* my_out = s_out + size_t(warp - 2) * kBOutStageBytes;
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    uint32_t ab = 0, ab_phase = 0, n_seen = 0;
    bool ok = true;
    const UnitMap um(n_tiles, n_slabs, p.splits, p.n_full, p.pieces);
    int tile, kb0, kb1;
    for (;;) {
      const uint32_t slot = n_seen % kBUnitRing;
      ok = __all_sync(0xffffffffu, mbar_wait(&ur_full[slot], (n_seen / kBUnitRing) & 1, p.status, 0x807));
      if (!ok) break;
      const int u = unit_ring[slot];
      __syncwarp();
      if (lane == 0) mbar_arrive(&ur_empty[slot]);
      ++n_seen;
      if (u < 0) break;
      um.decode(u, tile, kb0, kb1);
      const int m0 = (tile / tiles_n) * kBM, n0 = (tile % tiles_n) * kBN;
      ok = __all_sync(0xffffffffu, mbar_wait(&acc_full[ab], ab_phase, p.status, 0x804));
      if (!ok) break;
      tc_fence_after();
      const uint32_t tacc = tbase + lane_base + ab * kBN;
#pragma unroll 1
      for (int c0 = chalf * (kBN / 2); c0 < (chalf + 1) * (kBN / 2); c0 += 32) {
        if (n0 + c0 >= p.cols) break;   // uniform
        uint32_t r[32];
        tmem_ld32(tacc + c0, r);
        tmem_ld_wait();
        if (lane == 0) bulk_wait_read_all();   // the previous bulk operation of this warp has read the staging rows
        __syncwarp();
        if (MODE == kDgrad) {
          // 32 columns of this warp's 32 rows as bf16 -> shared memory (row = lane, 64-byte swizzle) -> one bulk tensor store
#pragma unroll
          for (int j = 0; j < 32; j += 8)
            *reinterpret_cast<uint4*>(my_out + swizzled_offset(lane, j / 8, 64)) = make_uint4(
                bwd_pack_bf16x2(__uint_as_float(r[j]) * p.alpha, __uint_as_float(r[j + 1]) * p.alpha),
                bwd_pack_bf16x2(__uint_as_float(r[j + 2]) * p.alpha, __uint_as_float(r[j + 3]) * p.alpha),
                bwd_pack_bf16x2(__uint_as_float(r[j + 4]) * p.alpha, __uint_as_float(r[j + 5]) * p.alpha),
                bwd_pack_bf16x2(__uint_as_float(r[j + 6]) * p.alpha, __uint_as_float(r[j + 7]) * p.alpha));
        } else {
          // 32 fp32 columns (128-byte rows, 128-byte swizzle) -> one bulk tensor reduction into the fp32 matrix
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(my_out + swizzled_offset(lane, j / 4, 128)) =
                make_float4(__uint_as_float(r[j]) * p.alpha, __uint_as_float(r[j + 1]) * p.alpha, __uint_as_float(r[j + 2]) * p.alpha,
                            __uint_as_float(r[j + 3]) * p.alpha);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (MODE == kDgrad) tma_store_2d(&map_out, my_out, n0 + c0, m0 + quarter * 32);
          else tma_reduce_add_2d(&map_out, my_out, n0 + c0, m0 + quarter * 32);
          bulk_commit_group();
        }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[ab]);
      if (++ab == 2) { ab = 0; ab_phase ^= 1; }
    }
    if (lane == 0) bulk_wait_read_all();   // the bulk operations have read their staging rows (the kernel boundary orders their writes)
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tbase, 512);
  }
}

// out[i] = bf16(acc[i]): the fp32 sum of the wgrad units as the bf16 gradient; 8 elements per thread.
__global__ void __launch_bounds__(256) wgrad_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ out, size_t n) {
  const size_t i = (size_t(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;
  if (i + 8 <= n) {
    const float4 a = *reinterpret_cast<const float4*>(acc + i), b = *reinterpret_cast<const float4*>(acc + i + 4);
    *reinterpret_cast<uint4*>(out + i) =
        make_uint4(bwd_pack_bf16x2(a.x, a.y), bwd_pack_bf16x2(a.z, a.w), bwd_pack_bf16x2(b.x, b.y), bwd_pack_bf16x2(b.z, b.w));
  } else {
    for (size_t j = i; j < n; ++j) out[j] = __float2bfloat16_rn(acc[j]);
  }
}

// ------------------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn bwd_gemm_encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Row-major [rows][cols] matrix of 1- or 2-byte elements, box = (128 bytes of columns, box_rows), 128-byte swizzle;
// out-of-range parts read as zero.
static bool operand_map(CUtensorMap* m, const void* ptr, int rows, int cols, int esz, int box_rows) {
  EncodeTiledFn fn = bwd_gemm_encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
  cuuint64_t strides[1] = {cuuint64_t(cols) * esz};
  cuuint32_t box[2] = {cuuint32_t(128 / esz), cuuint32_t(box_rows)};
  cuuint32_t es[2] = {1, 1};
  return fn(m, esz == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box,
            es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// [rows][cols] output, box = (32 columns, 32 rows): bf16 with the 64-byte swizzle, fp32 with the 128-byte swizzle
static bool result_map(CUtensorMap* m, const void* ptr, int rows, int cols, bool f32) {
  EncodeTiledFn fn = bwd_gemm_encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
  cuuint64_t strides[1] = {cuuint64_t(cols) * (f32 ? 4 : 2)};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t es[2] = {1, 1};
  return fn(m, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, f32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// kind::f16 / kind::f8f6f4 instruction descriptor: fp32 accumulate, operand formats (bf16: 1; e4m3: 0, e5m2: 1), majors, N, M
static uint32_t bwd_idesc(int a_fmt, int b_fmt, bool a_mn, bool b_mn) {
  return (1u << 4) | (uint32_t(a_fmt) << 7) | (uint32_t(b_fmt) << 10) | (uint32_t(a_mn) << 15) | (uint32_t(b_mn) << 16) |
         (uint32_t(kBN >> 3) << 17) | (uint32_t(kBM >> 4) << 24);
}

static int sm_count() {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

static int fmt_code(int dtype) { return dtype == MINTB_E5M2 ? 1 : dtype == MINTB_E4M3 ? 0 : 1; }   // bf16 is code 1 of kind::f16
static bool is_f8(int dtype) { return dtype == MINTB_E4M3 || dtype == MINTB_E5M2; }

template <int MODE>
static int launch_bwd_gemm(const CUtensorMap& a1, const CUtensorMap& b1, const CUtensorMap& a2, const CUtensorMap& b2,
                           const CUtensorMap& out, const BwdGemmParams& p_in, int grid, cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(gemm_bwd_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kBwdGemmSmem));
  if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return MINTB_ECUDA; }
  BwdGemmParams p = p_in;
  if (int rc = next_tile_counter(&p.sched); rc != MINTB_OK) return rc;
  gemm_bwd_kernel<MODE><<<grid, kBThreads, kBwdGemmSmem, stream>>>(a1, b1, a2, b2, out, p);
  count_launches(1);
  e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("backward gemm launch: %s", cudaGetErrorString(e)); return MINTB_ECUDA; }
  return MINTB_OK;
}

// Plan of a weight-gradient launch: n_tiles output tiles, a reduction of n_slabs slabs, `sms` CTAs.  A tile's reduction is cut
// into `splits` aligned parts (large units); as many large units as fill whole rounds of the grid run as they are, and the
// left-over ones - which would occupy a round of their own with part of the grid idle - are cut again into `pieces` pieces
// each, so that they spread over the whole grid as short units.  Cost model in slab-times on the busiest CTA: a round of
// large units costs its slabs (the epilogue of a unit overlaps the next unit's products), a round of short units at least
// an epilogue (six slab-times), one epilogue at the end.  At most 16 splits and 32 pieces, units of at least 8 slabs.
struct WgradPlan { int splits, n_full, pieces; long long units; };
static WgradPlan plan_wgrad(int n_tiles, int n_slabs, int sms) {
  WgradPlan best{1, n_tiles, 1, n_tiles};
  long long best_cost = -1;
  for (int s = 1; s <= 16; ++s) {
    const int per = (n_slabs + s - 1) / s;
    if (s > 1 && per < 8) break;
    const int s_eff = (n_slabs + per - 1) / per;                 // cuts that hold something
    const long long large = static_cast<long long>(n_tiles) * s_eff;
    const long long full_rounds = large / sms, rem = large - full_rounds * sms;
    for (int m = 1; m <= 32; ++m) {
      const int sub = (per + m - 1) / m;
      if (m > 1 && (sub < 8 || rem == 0)) break;
      const int m_eff = (per + sub - 1) / sub;
      const long long short_rounds = (rem * m_eff + sms - 1) / sms;
      const long long cost = full_rounds * per + short_rounds * (sub > 6 ? sub : 6) + 6;
      const long long units = full_rounds * sms + rem * m_eff;
      if (best_cost < 0 || cost < best_cost || (cost == best_cost && units < best.units)) {
        best_cost = cost;
        best = WgradPlan{s_eff, int(full_rounds * sms), m_eff, units};
      }
    }
  }
  return best;
}

}  // namespace mintb

using namespace mintb;

static bool bwd_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

extern "C" int mintb_linear_dgrad(const void* dz, const void* w, const void* dz2, const void* w2, void* dx, int M, int N, int K,
                                  int N2, int dz_dtype, int w_dtype, float alpha, void* stream, int* dev_status) {
  const bool f8 = is_f8(dz_dtype);
  if (dz == nullptr || w == nullptr || dx == nullptr || M <= 0 || N <= 0 || K <= 0 || N2 < 0 || ((dz2 == nullptr) != (N2 == 0)) ||
      ((w2 == nullptr) != (N2 == 0))) {
    set_error("mintb_linear_dgrad: dz, w, dx and positive M, N, K are required; dz2, w2 and N2 come together");
    return MINTB_EINVAL;
  }
  if (!(dz_dtype == MINTB_BF16 && w_dtype == MINTB_BF16) && !(is_f8(dz_dtype) && is_f8(w_dtype))) {
    set_error("mintb_linear_dgrad: operands are both bf16 or both 8-bit floats (e4m3 / e5m2)");
    return MINTB_EUNSUPPORTED;
  }
  const int esz = f8 ? 1 : 2;
  if ((size_t(N) * esz) % 16 || (size_t(N2) * esz) % 16 || (size_t(K) * esz) % 16 || K % 8 || !bwd_aligned16(dz) || !bwd_aligned16(w) ||
      !bwd_aligned16(dz2) || !bwd_aligned16(w2) || !bwd_aligned16(dx)) {
    set_error("mintb_linear_dgrad: rows of dz, w and dx must be 16-byte multiples and the pointers 16-byte aligned");
    return MINTB_EINVAL;
  }
  const int epb = 128 / esz;
  CUtensorMap a1, b1, a2, b2, mo;
  bool ok = operand_map(&a1, dz, M, N, esz, kBM) && operand_map(&b1, w, N, K, esz, epb) && result_map(&mo, dx, M, K, false);
  a2 = a1; b2 = b1;
  if (ok && N2 > 0) ok = operand_map(&a2, dz2, M, N2, esz, kBM) && operand_map(&b2, w2, N2, K, esz, epb);
  if (!ok) { set_error("mintb_linear_dgrad: cuTensorMapEncodeTiled failed"); return MINTB_ECUDA; }
  BwdGemmParams p{};
  p.rows = M; p.cols = K; p.red1 = N; p.red2 = N2; p.f8 = f8 ? 1 : 0;
  p.idesc = bwd_idesc(fmt_code(dz_dtype), fmt_code(w_dtype), false, true);
  p.splits = 1; p.pieces = 1; p.alpha = alpha; p.status = dev_status;
  const int tiles = ((M + kBM - 1) / kBM) * ((K + kBN - 1) / kBN);
  p.n_full = tiles;
  const int sms = sm_count();
  return launch_bwd_gemm<kDgrad>(a1, b1, a2, b2, mo, p, tiles < sms ? tiles : sms, static_cast<cudaStream_t>(stream));
}

extern "C" size_t mintb_linear_wgrad_workspace_bytes(int N, int K, int out_dtype) {
  return out_dtype == MINTB_F32 ? 0 : align256(size_t(N) * K * 4);
}

extern "C" int mintb_linear_wgrad(const void* dz, const void* x, void* dw, void* workspace, size_t workspace_bytes, int M, int N,
                                  int K, int dz_dtype, int x_dtype, int out_dtype, float alpha, void* stream, int* dev_status) {
  const bool f8 = is_f8(dz_dtype);
  if (dz == nullptr || x == nullptr || dw == nullptr || M <= 0 || N <= 0 || K <= 0) {
    set_error("mintb_linear_wgrad: dz, x, dw and positive M, N, K are required");
    return MINTB_EINVAL;
  }
  if (!(dz_dtype == MINTB_BF16 && x_dtype == MINTB_BF16) && !(is_f8(dz_dtype) && is_f8(x_dtype))) {
    set_error("mintb_linear_wgrad: operands are both bf16 or both 8-bit floats (e4m3 / e5m2)");
    return MINTB_EUNSUPPORTED;
  }
  if (out_dtype != MINTB_BF16 && out_dtype != MINTB_F32) {
    set_error("mintb_linear_wgrad: dw is bf16 or fp32");
    return MINTB_EINVAL;
  }
  const int esz = f8 ? 1 : 2;
  if ((size_t(N) * esz) % 16 || (size_t(K) * esz) % 16 || K % 4 || !bwd_aligned16(dz) || !bwd_aligned16(x) || !bwd_aligned16(dw) ||
      !bwd_aligned16(workspace)) {
    set_error("mintb_linear_wgrad: rows of dz and x must be 16-byte multiples, K a multiple of 4, and the pointers 16-byte aligned");
    return MINTB_EINVAL;
  }
  const size_t need = mintb_linear_wgrad_workspace_bytes(N, K, out_dtype);
  if (need > 0 && (workspace == nullptr || workspace_bytes < need)) {
    set_error("mintb_linear_wgrad: workspace of %zu bytes required, %zu given", need, workspace_bytes);
    return MINTB_EWORKSPACE;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* acc = out_dtype == MINTB_F32 ? static_cast<float*>(dw) : static_cast<float*>(workspace);
  cudaError_t e = cudaMemsetAsync(acc, 0, size_t(N) * K * 4, s);
  if (e != cudaSuccess) { set_error("cudaMemsetAsync: %s", cudaGetErrorString(e)); return MINTB_ECUDA; }
  const int epb = 128 / esz;
  CUtensorMap a1, b1, mo;
  if (!operand_map(&a1, dz, M, N, esz, epb) || !operand_map(&b1, x, M, K, esz, epb) || !result_map(&mo, acc, N, K, true)) {
    set_error("mintb_linear_wgrad: cuTensorMapEncodeTiled failed");
    return MINTB_ECUDA;
  }
  BwdGemmParams p{};
  p.rows = N; p.cols = K; p.red1 = M; p.red2 = 0; p.f8 = f8 ? 1 : 0;
  p.idesc = bwd_idesc(fmt_code(dz_dtype), fmt_code(x_dtype), true, true);
  p.alpha = alpha; p.status = dev_status;
  const int tiles = ((N + kBM - 1) / kBM) * ((K + kBN - 1) / kBN);
  const int sms = sm_count();
  const WgradPlan plan = plan_wgrad(tiles, (M + epb - 1) / epb, sms);
  p.splits = plan.splits; p.n_full = plan.n_full; p.pieces = plan.pieces;
  const long long units = plan.units;
  int rc = launch_bwd_gemm<kWgrad>(a1, b1, a1, b1, mo, p, units < sms ? int(units) : sms, s);
  if (rc != MINTB_OK) return rc;
  if (out_dtype == MINTB_BF16) {
    const size_t n = size_t(N) * K;
    wgrad_convert_kernel<<<unsigned((n / 8 + 255) / 256 + 1), 256, 0, s>>>(acc, static_cast<__nv_bfloat16*>(dw), n);
    count_launches(1);
    e = cudaGetLastError();
    if (e != cudaSuccess) { set_error("wgrad convert launch: %s", cudaGetErrorString(e)); return MINTB_ECUDA; }
  }
  return MINTB_OK;
}
