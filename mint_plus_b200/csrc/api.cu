// extern "C" entry points of libmintb: host-side validation and dispatch.  See include/mintb.h.
#include <atomic>
#include <mutex>
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace mintb {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

static std::atomic<unsigned long long> g_launches{0};
// the pool of work counters (see common.cuh); zero-initialised with the module, each pair cleared again by its last user
static __device__ int g_tile_counters[2 * kTileCounterSlots];

int next_tile_counter(int** out) {
  constexpr int kMaxDevices = 64;
  static std::atomic<unsigned> next{0};
  static std::mutex mu;
  static int* base[kMaxDevices] = {};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_error("work counters: cudaGetDevice failed or device index %d is out of range", dev);
    return MINTB_ECUDA;
  }
  int* b = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (base[dev] == nullptr) {   // the symbol's address differs per device; look it up once with that device current
      void* ptr = nullptr;
      e = cudaGetSymbolAddress(&ptr, g_tile_counters);
      if (e != cudaSuccess || ptr == nullptr) {
        set_error("work counters: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        return MINTB_ECUDA;
      }
      base[dev] = static_cast<int*>(ptr);
    }
    b = base[dev];
  }
  *out = b + 2 * (next.fetch_add(1, std::memory_order_relaxed) % kTileCounterSlots);
  return MINTB_OK;
}

void count_launches(int n) { g_launches.fetch_add(static_cast<unsigned long long>(n), std::memory_order_relaxed); }

static int cuda_fail(cudaError_t e, const char* what) {
  set_error("%s: %s", what, cudaGetErrorString(e));
  return MINTB_ECUDA;
}

static bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

static int check_shape(int B, int H, int T, int D, int dtype, const char* who) {
  if (B <= 0 || H <= 0 || T <= 0) {
    set_error("%s: B, H, T must be positive (got %d, %d, %d)", who, B, H, T);
    return MINTB_EINVAL;
  }
  if (dtype != MINTB_F32 && dtype != MINTB_BF16) {
    set_error("%s: dtype must be MINTB_F32 or MINTB_BF16 (got %d)", who, dtype);
    return MINTB_EINVAL;
  }
  if (D != 16 && D != 32 && D != 64) {
    set_error("%s: head_dim %d is not supported (16, 32 or 64)", who, D);
    return MINTB_EUNSUPPORTED;
  }
  if (size_t(B) * H > 65535u * 32u) {
    set_error("%s: B*H = %zu is too large", who, size_t(B) * H);
    return MINTB_EINVAL;
  }
  return MINTB_OK;
}

static bool use_tc(int D, int dtype, unsigned flags) {
  return !(flags & MINTB_FLAG_FORCE_SIMT) && tc_supported(D, dtype);
}

}  // namespace mintb

using namespace mintb;

extern "C" {

// Clears every work counter of the current device.  Needed only after a kernel gave up on a bounded wait (a device status
// was raised): its CTAs may not all have left their counter.  Synchronises the device.
int mintb_reset_work_counters(void) {
  int* first = nullptr;
  int rc = next_tile_counter(&first);
  if (rc != MINTB_OK) return rc;
  cudaError_t e = cudaDeviceSynchronize();
  int* base = nullptr;
  if (e == cudaSuccess) e = cudaGetSymbolAddress(reinterpret_cast<void**>(&base), g_tile_counters);
  if (e == cudaSuccess) e = cudaMemset(base, 0, sizeof(int) * 2 * kTileCounterSlots);
  return e == cudaSuccess ? MINTB_OK : cuda_fail(e, "mintb_reset_work_counters");
}

int mintb_version(void) { return 100; }

const char* mintb_last_error(void) { return g_err; }

unsigned long long mintb_kernel_launches(void) { return g_launches.load(std::memory_order_relaxed); }

size_t mintb_mask_meta_bytes(int B, int T) {
  if (B <= 0 || T <= 0) return 0;
  return meta_layout(B, T).total;
}

int mintb_mask_meta_from_chain_ids(const int32_t* chain_ids, const uint8_t* key_pad, void* meta, int B, int T,
                                   void* stream) {
  if (B <= 0 || T <= 0 || chain_ids == nullptr || meta == nullptr || !aligned(meta, 256)) {
    set_error("mintb_mask_meta_from_chain_ids: need B, T > 0, chain_ids, and a 256-byte aligned meta buffer");
    return MINTB_EINVAL;
  }
  cudaError_t e = launch_meta_from_chain_ids(chain_ids, key_pad, meta, B, T, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? MINTB_OK : cuda_fail(e, "mask metadata launch");
}

int mintb_mask_meta_from_mask(const uint8_t* chain_mask, const uint8_t* key_pad, void* meta, int B, int T,
                              void* stream) {
  if (B <= 0 || T <= 0 || chain_mask == nullptr || meta == nullptr || !aligned(meta, 256)) {
    set_error("mintb_mask_meta_from_mask: need B, T > 0, chain_mask, and a 256-byte aligned meta buffer");
    return MINTB_EINVAL;
  }
  cudaError_t e = launch_meta_from_mask(chain_mask, key_pad, meta, B, T, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? MINTB_OK : cuda_fail(e, "mask metadata launch");
}

int mintb_rope_tables(const float* inv_freq, float* cos_tab, float* sin_tab, int T, int D, void* stream) {
  if (T <= 0 || D <= 0 || (D & 1) || inv_freq == nullptr || cos_tab == nullptr || sin_tab == nullptr) {
    set_error("mintb_rope_tables: need T > 0, even D > 0 and non-null pointers");
    return MINTB_EINVAL;
  }
  cudaError_t e = launch_rope_tables(inv_freq, cos_tab, sin_tab, T, D, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? MINTB_OK : cuda_fail(e, "rope table launch");
}

size_t mintb_attn_fwd_workspace_bytes(int B, int H, int T, int D, int dtype, unsigned flags) {
  if (check_shape(B, H, T, D, dtype, "mintb_attn_fwd_workspace_bytes") != MINTB_OK) return 0;
  if (use_tc(D, dtype, flags))
    return tc_fwd_workspace_bytes(B, H, T, D, (flags & MINTB_FLAG_ROPE) != 0 && !(flags & MINTB_FLAG_QK_PREROTATED));
  return 0;
}

size_t mintb_attn_bwd_workspace_bytes(int B, int H, int T, int D, int dtype, unsigned flags) {
  if (check_shape(B, H, T, D, dtype, "mintb_attn_bwd_workspace_bytes") != MINTB_OK) return 0;
  if (use_tc(D, dtype, flags))
    return tc_bwd_workspace_bytes(B, H, T, D, (flags & MINTB_FLAG_ROPE) != 0 && !(flags & MINTB_FLAG_QK_PREROTATED));
  return simt_bwd_workspace_bytes(B, H, T, D);
}

static int fill_common(AttnArgs& a, const char* who, const void* q_s, const void* k_s, const void* v_s,
                       const void* q_c, const void* k_c, const void* v_c, const void* meta, const float* rope_cos,
                       const float* rope_sin, void* workspace, size_t workspace_bytes, size_t need, int B, int H,
                       int T, int D, int dtype, unsigned flags, float scale, void* stream, int* dev_status) {
  int rc = check_shape(B, H, T, D, dtype, who);
  if (rc != MINTB_OK) return rc;
  if (flags & ~(MINTB_FLAG_ROPE | MINTB_FLAG_SQRT_SOFTMAX | MINTB_FLAG_FORCE_SIMT | MINTB_FLAG_OUT_SEQ_FIRST | MINTB_FLAG_ROT_SAVED |
                MINTB_FLAG_SKIP_PAD_QUERIES | MINTB_FLAG_QK_PREROTATED | MINTB_FLAG_GRAD_ROWMAJOR)) {
    set_error("%s: unknown flag bits 0x%x", who, flags);
    return MINTB_EINVAL;
  }
  const void* ptrs[] = {q_s, k_s, v_s, q_c, k_c, v_c};
  for (const void* p : ptrs) {
    if (p == nullptr || !aligned(p, 16)) {
      set_error("%s: q/k/v pointers must be non-null and 16-byte aligned", who);
      return MINTB_EINVAL;
    }
  }
  if (meta == nullptr || !aligned(meta, 256)) {
    set_error("%s: meta must be a 256-byte aligned buffer built by mintb_mask_meta_*", who);
    return MINTB_EINVAL;
  }
  if ((flags & MINTB_FLAG_ROPE) && (rope_cos == nullptr || rope_sin == nullptr)) {
    set_error("%s: MINTB_FLAG_ROPE needs rope_cos and rope_sin tables", who);
    return MINTB_EINVAL;
  }
  if (!(scale > 0.f) || scale > 1e6f) {
    set_error("%s: scale must be a positive finite number (got %g)", who, double(scale));
    return MINTB_EINVAL;
  }
  if (need > 0 && (workspace == nullptr || workspace_bytes < need || !aligned(workspace, 256))) {
    set_error("%s: workspace of %zu bytes (256-byte aligned) required, got %zu", who, need, workspace_bytes);
    return MINTB_EWORKSPACE;
  }
  a.q_s = q_s; a.k_s = k_s; a.v_s = v_s; a.q_c = q_c; a.k_c = k_c; a.v_c = v_c;
  a.meta = meta_ptrs(meta, B, T);
  a.rope_cos = rope_cos; a.rope_sin = rope_sin;
  a.workspace = workspace; a.workspace_bytes = workspace_bytes;
  a.B = B; a.H = H; a.T = T; a.D = D; a.dtype = dtype;
  a.rope = (flags & MINTB_FLAG_ROPE) != 0;
  a.sqrt_softmax = (flags & MINTB_FLAG_SQRT_SOFTMAX) != 0;
  a.out_seq_first = (flags & MINTB_FLAG_OUT_SEQ_FIRST) != 0;
  a.rot_saved = (flags & MINTB_FLAG_ROT_SAVED) != 0;
  a.skip_pad_queries = (flags & MINTB_FLAG_SKIP_PAD_QUERIES) != 0;
  a.qk_prerotated = (flags & MINTB_FLAG_QK_PREROTATED) != 0;
  a.grad_rowmajor = (flags & MINTB_FLAG_GRAD_ROWMAJOR) != 0;
  if ((a.qk_prerotated || a.grad_rowmajor) && !use_tc(D, dtype, flags)) {
    set_error("%s: pre-rotated inputs / row-major gradients are served by the bf16 tensor-core kernels only", who);
    return MINTB_EUNSUPPORTED;
  }
  if (a.qk_prerotated && !a.rope) {
    set_error("%s: MINTB_FLAG_QK_PREROTATED goes with MINTB_FLAG_ROPE and the tables", who);
    return MINTB_EINVAL;
  }
  a.scale = scale;
  a.stream = static_cast<cudaStream_t>(stream);
  a.dev_status = dev_status;
  return MINTB_OK;
}

}  // extern "C"

namespace mintb {
// The argument checks of mintb_attn_fwd for entry points defined in other files.
int check_attn_args(AttnArgs& a, const char* who, const void* q_s, const void* k_s, const void* v_s, const void* q_c,
                    const void* k_c, const void* v_c, const void* meta, const float* rope_cos, const float* rope_sin,
                    void* workspace, size_t workspace_bytes, size_t need, int B, int H, int T, int D, int dtype,
                    unsigned flags, float scale, void* stream, int* dev_status) {
  return fill_common(a, who, q_s, k_s, v_s, q_c, k_c, v_c, meta, rope_cos, rope_sin, workspace, workspace_bytes, need, B,
                     H, T, D, dtype, flags, scale, stream, dev_status);
}
}  // namespace mintb

extern "C" {

int mintb_attn_fwd(const void* q_self, const void* k_self, const void* v_self, const void* q_cross,
                   const void* k_cross, const void* v_cross, const void* meta, const float* rope_cos,
                   const float* rope_sin, void* out, float* lse, void* workspace, size_t workspace_bytes, int B,
                   int H, int T, int D, int dtype, unsigned flags, float scale, void* stream, int* dev_status) {
  AttnArgs a{};
  size_t need = mintb_attn_fwd_workspace_bytes(B, H, T, D, dtype, flags);
  int rc = fill_common(a, "mintb_attn_fwd", q_self, k_self, v_self, q_cross, k_cross, v_cross, meta, rope_cos,
                       rope_sin, workspace, workspace_bytes, need, B, H, T, D, dtype, flags, scale, stream, dev_status);
  if (rc != MINTB_OK) return rc;
  if (out == nullptr || lse == nullptr || !aligned(out, 16)) {
    set_error("mintb_attn_fwd: out (16-byte aligned) and lse are required");
    return MINTB_EINVAL;
  }
  a.out = out;
  a.lse = lse;
  if (use_tc(D, dtype, flags)) return launch_attn_fwd_tc(a);
  cudaError_t e = launch_attn_fwd_simt(a);
  return e == cudaSuccess ? MINTB_OK : cuda_fail(e, "attention forward launch");
}

int mintb_attn_bwd_rows(const void* q_self, const void* k_self, const void* v_self, const void* q_cross,
                        const void* k_cross, const void* v_cross, const void* meta, const float* rope_cos,
                        const float* rope_sin, const void* out, const float* lse, const void* d_out, void* dq_self,
                        void* dk_self, void* dv_self, void* dq_cross, void* dk_cross, void* dv_cross, void* workspace,
                        size_t workspace_bytes, int B, int H, int T, int D, int dtype, unsigned flags, float scale,
                        void* stream, int* dev_status, const int32_t* token_row) {
  AttnArgs a{};
  size_t need = mintb_attn_bwd_workspace_bytes(B, H, T, D, dtype, flags);
  int rc = fill_common(a, "mintb_attn_bwd", q_self, k_self, v_self, q_cross, k_cross, v_cross, meta, rope_cos,
                       rope_sin, workspace, workspace_bytes, need, B, H, T, D, dtype, flags, scale, stream, dev_status);
  if (rc != MINTB_OK) return rc;
  const void* ptrs[] = {out, lse, d_out, dq_self, dk_self, dv_self, dq_cross, dk_cross, dv_cross};
  for (const void* p : ptrs) {
    if (p == nullptr || !aligned(p, 16)) {
      set_error("mintb_attn_bwd: out, lse, d_out and the six gradient buffers must be non-null, 16-byte aligned");
      return MINTB_EINVAL;
    }
  }
  if (token_row != nullptr && !a.grad_rowmajor) {
    set_error("mintb_attn_bwd_rows: a token-row map needs MINTB_FLAG_GRAD_ROWMAJOR");
    return MINTB_EINVAL;
  }
  a.token_row = token_row;
  a.out = const_cast<void*>(out);
  a.lse = const_cast<float*>(lse);
  a.d_out = d_out;
  a.dq_s = dq_self; a.dk_s = dk_self; a.dv_s = dv_self; a.dq_c = dq_cross; a.dk_c = dk_cross; a.dv_c = dv_cross;
  if (use_tc(D, dtype, flags)) return launch_attn_bwd_tc(a);
  cudaError_t e = launch_attn_bwd_simt(a);
  return e == cudaSuccess ? MINTB_OK : cuda_fail(e, "attention backward launch");
}

int mintb_attn_bwd(const void* q_self, const void* k_self, const void* v_self, const void* q_cross,
                   const void* k_cross, const void* v_cross, const void* meta, const float* rope_cos,
                   const float* rope_sin, const void* out, const float* lse, const void* d_out, void* dq_self,
                   void* dk_self, void* dv_self, void* dq_cross, void* dk_cross, void* dv_cross, void* workspace,
                   size_t workspace_bytes, int B, int H, int T, int D, int dtype, unsigned flags, float scale,
                   void* stream, int* dev_status) {
  return mintb_attn_bwd_rows(q_self, k_self, v_self, q_cross, k_cross, v_cross, meta, rope_cos, rope_sin, out, lse, d_out,
                             dq_self, dk_self, dv_self, dq_cross, dk_cross, dv_cross, workspace, workspace_bytes, B, H, T,
                             D, dtype, flags, scale, stream, dev_status, nullptr);
}

int mintb_combine_fwd(const void* intra_logits, const void* inter_logits, const uint8_t* chain_mask,
                      const void* intra_values, const void* inter_values, void* out, int B, int H, int T, int D,
                      int dtype, void* stream) {
  int rc = check_shape(B, H, T, D, dtype, "mintb_combine_fwd");
  if (rc != MINTB_OK) return rc;
  if (!intra_logits || !inter_logits || !chain_mask || !intra_values || !inter_values || !out) {
    set_error("mintb_combine_fwd: null pointer");
    return MINTB_EINVAL;
  }
  cudaError_t e = launch_combine_fwd(intra_logits, inter_logits, chain_mask, intra_values, inter_values, out, B, H, T,
                                     D, dtype, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? MINTB_OK : cuda_fail(e, "combine forward launch");
}

size_t mintb_combine_bwd_workspace_bytes(int B, int H, int T) {
  if (B <= 0 || H <= 0 || T <= 0) return 0;
  return align256(size_t(B) * H * T * 2 * sizeof(float));
}

int mintb_combine_bwd(const void* intra_logits, const void* inter_logits, const uint8_t* chain_mask,
                      const void* intra_values, const void* inter_values, const void* d_out, void* d_intra_logits,
                      void* d_inter_logits, void* d_intra_values, void* d_inter_values, void* workspace,
                      size_t workspace_bytes, int B, int H, int T, int D, int dtype, void* stream) {
  int rc = check_shape(B, H, T, D, dtype, "mintb_combine_bwd");
  if (rc != MINTB_OK) return rc;
  if (workspace == nullptr || workspace_bytes < mintb_combine_bwd_workspace_bytes(B, H, T)) {
    set_error("mintb_combine_bwd: workspace of %zu bytes required", mintb_combine_bwd_workspace_bytes(B, H, T));
    return MINTB_EWORKSPACE;
  }
  if (!intra_logits || !inter_logits || !chain_mask || !intra_values || !inter_values || !d_out ||
      !d_intra_logits || !d_inter_logits || !d_intra_values || !d_inter_values) {
    set_error("mintb_combine_bwd: null pointer");
    return MINTB_EINVAL;
  }
  cudaError_t e = launch_combine_bwd(intra_logits, inter_logits, chain_mask, intra_values, inter_values, d_out,
                                     d_intra_logits, d_inter_logits, d_intra_values, d_inter_values,
                                     static_cast<float*>(workspace), B, H, T, D, dtype,
                                     static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? MINTB_OK : cuda_fail(e, "combine backward launch");
}

}  // extern "C"
