// Shared declarations of the mintb library: parameter blocks, mask-metadata layout, host launchers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

#include "../../include/mintb.h"

namespace mintb {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr int kClassTile = 64;  // granularity of the tile-class table

enum TileClass : uint8_t { kHasIntra = 1, kHasInter = 2, kHasPad = 4 };

// Layout of the caller-allocated mask-metadata blob for (B, T); all offsets are multiples of 256 bytes.
//   bits   uint32 [B][T][TW]   bit (i, j): 1 -> cross pathway for query i, key j         (row = query)
//   bitsT  uint32 [B][T][TW]   bit (j, i): the same relation, row = key                   (for dK/dV)
//   kpad   uint32 [B][TW]      bit j: 1 -> key j is padded or j >= T
//   cls    uint8  [B][NT][NT]  class byte of the 64x64 tile (query tile, key tile)
struct MetaLayout {
  int TW;  // words per row: ceil(T/32) rounded up to a multiple of 4 (so a 128-key tile is one 16-byte load)
  int NT;  // ceil(T/64)
  size_t off_bits, off_bitsT, off_kpad, off_cls, total;
};

__host__ __device__ inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

__host__ __device__ inline MetaLayout meta_layout(int B, int T) {
  MetaLayout L;
  L.TW = (((T + 31) / 32) + 3) & ~3;
  L.NT = (T + kClassTile - 1) / kClassTile;
  size_t bits = align256(size_t(B) * T * L.TW * 4);
  L.off_bits = 0;
  L.off_bitsT = bits;
  L.off_kpad = 2 * bits;
  L.off_cls = L.off_kpad + align256(size_t(B) * L.TW * 4);
  L.total = L.off_cls + align256(size_t(B) * L.NT * L.NT);
  return L;
}

struct MetaPtrs {
  const uint32_t* bits;
  const uint32_t* bitsT;
  const uint32_t* kpad;
  const uint8_t* cls;
  int TW, NT;
};

inline MetaPtrs meta_ptrs(const void* meta, int B, int T) {
  MetaLayout L = meta_layout(B, T);
  const char* p = static_cast<const char*>(meta);
  return MetaPtrs{reinterpret_cast<const uint32_t*>(p + L.off_bits), reinterpret_cast<const uint32_t*>(p + L.off_bitsT),
                  reinterpret_cast<const uint32_t*>(p + L.off_kpad), reinterpret_cast<const uint8_t*>(p + L.off_cls),
                  L.TW, L.NT};
}

// Arguments of one attention call, shared by every kernel family.
struct AttnArgs {
  const void *q_s, *k_s, *v_s, *q_c, *k_c, *v_c;
  MetaPtrs meta;
  const float *rope_cos, *rope_sin;  // [T][D/2], only with rope
  void* out;                         // fwd: written; bwd: read
  float* lse;                        // fwd: written; bwd: read
  const void* d_out;
  void *dq_s, *dk_s, *dv_s, *dq_c, *dk_c, *dv_c;
  void* workspace;
  size_t workspace_bytes;
  int B, H, T, D;
  int dtype;
  bool rope;
  bool sqrt_softmax;
  bool out_seq_first;                // out / d_out laid out (T,B,H,D) instead of (B,H,T,D)
  bool rot_saved;                    // backward: the workspace already starts with the rotated Q_self, K_self
  bool skip_pad_queries;             // query tiles holding only padded positions are left out
  bool qk_prerotated;                // q_self / k_self arrive rotated; only the gradients are (un-)rotated
  bool grad_rowmajor;                // gradients go into [T*B][3E] row-major matrices
  const int32_t* token_row;          // with grad_rowmajor: row of those matrices that belongs to token t*B + b, negative = none
                                     // (the matrices then hold only the listed rows); null = row t*B + b
  float scale;
  cudaStream_t stream;
  int* dev_status;
};

// element strides of out / d_out: row (query) stride and (batch, head) stride
inline size_t out_row_stride(const AttnArgs& a) { return a.out_seq_first ? size_t(a.B) * a.H * a.D : size_t(a.D); }
inline size_t out_bh_stride(const AttnArgs& a) { return a.out_seq_first ? size_t(a.D) : size_t(a.T) * a.D; }

// element strides of the six gradient tensors: between rows (t), batch entries and heads
inline size_t grad_row_stride(const AttnArgs& a) { return a.grad_rowmajor ? size_t(a.B) * 3 * a.H * a.D : size_t(a.D); }
inline size_t grad_b_stride(const AttnArgs& a) { return a.grad_rowmajor ? size_t(3) * a.H * a.D : size_t(a.H) * a.T * a.D; }
inline size_t grad_h_stride(const AttnArgs& a) { return a.grad_rowmajor ? size_t(a.D) : size_t(a.T) * a.D; }

void set_error(const char* fmt, ...);
// Launch `kern` so that it may start while the kernel before it in the stream is still running (programmatic dependent
// launch); the kernel calls ptx::griddep_wait() before it touches anything that kernel writes.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}
void count_launches(int n);  // process-wide tally of kernels launched by this library

// Work counters of the persistent kernels.  A launch takes the next {next unit, CTAs that have left} pair of a pool in the
// library image (zero when it gets it); its CTAs draw work units from the first word, and the last CTA to leave clears the
// pair again, so no launch needs a clearing pass.  Launches that can run at the same time hold different pairs as long as
// fewer than kTileCounterSlots launches lie between them; launches on one stream run one after the other and may share.
constexpr int kTileCounterSlots = 4096;
int next_tile_counter(int** out);      // MINTB_OK or an error code
// (device side, in ptx.cuh: leave_tile_counter)

// api.cu
int check_attn_args(AttnArgs& a, const char* who, const void* q_s, const void* k_s, const void* v_s, const void* q_c,
                    const void* k_c, const void* v_c, const void* meta, const float* rope_cos, const float* rope_sin,
                    void* workspace, size_t workspace_bytes, size_t need, int B, int H, int T, int D, int dtype,
                    unsigned flags, float scale, void* stream, int* dev_status);

// prep.cu
cudaError_t launch_meta_from_chain_ids(const int32_t* chain_ids, const uint8_t* key_pad, void* meta, int B, int T,
                                       cudaStream_t s);
cudaError_t launch_meta_from_mask(const uint8_t* mask, const uint8_t* key_pad, void* meta, int B, int T,
                                  cudaStream_t s);
cudaError_t launch_rope_tables(const float* inv_freq, float* cos_tab, float* sin_tab, int T, int D, cudaStream_t s);

// attn_simt.cu — fp32 CUDA-core kernels (any dtype in, fp32 arithmetic)
size_t simt_bwd_workspace_bytes(int B, int H, int T, int D);
cudaError_t launch_attn_fwd_simt(const AttnArgs& a);
cudaError_t launch_attn_bwd_simt(const AttnArgs& a);

// attn_tc_fwd.cu / attn_tc_bwd.cu — tcgen05 kernels (bf16, D in {32, 64})
bool tc_supported(int D, int dtype);
size_t tc_fwd_workspace_bytes(int B, int H, int T, int D, bool rope);
size_t tc_bwd_workspace_bytes(int B, int H, int T, int D, bool rope);
int launch_attn_fwd_tc(const AttnArgs& a);  // returns a MINTB_* code
int launch_attn_bwd_tc(const AttnArgs& a);

// combine.cu
cudaError_t launch_combine_fwd(const void* il, const void* el, const uint8_t* mask, const void* iv, const void* ev,
                               void* out, int B, int H, int T, int D, int dtype, cudaStream_t s);
cudaError_t launch_combine_bwd(const void* il, const void* el, const uint8_t* mask, const void* iv, const void* ev,
                               const void* d_out, void* d_il, void* d_el, void* d_iv, void* d_ev, float* stats, int B,
                               int H, int T, int D, int dtype, cudaStream_t s);

// ---- element access helpers -------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float ld_f(const T* p);
template <>
__device__ __forceinline__ float ld_f<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ld_f<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename T>
__device__ __forceinline__ void st_f(T* p, float v);
template <>
__device__ __forceinline__ void st_f<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void st_f<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

}  // namespace mintb
