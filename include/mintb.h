/*
 * mintb — C ABI of the B200 (sm_100a) implementation of MINT's two-pathway combined-softmax
 * multimer attention and the kernels either side of it.
 *
 * The reference (molecular-william/mint_plus) is pure Python + Triton and has no FFI for this path:
 * its boundary is a set of Python call signatures.  Each entry point below names the reference
 * function whose device work it replaces (path within the mint_plus checkout : lines).
 *
 * Conventions
 *   - Plain pointers and sizes only.  Every pointer is a DEVICE pointer unless stated otherwise.
 *   - The caller owns every buffer (inputs, outputs, mask metadata, workspaces); nothing is allocated
 *     or freed here.  Inputs are read-only.
 *   - Tensors are contiguous, row-major: q/k/v/out/grad [B][H][T][D]; lse [B][H][T] (float);
 *     chain_ids [B][T] (int32); key_pad [B][T] (uint8, non-zero = padded key); chain_mask [B][T][T]
 *     (uint8, non-zero = the two positions belong to different chains -> cross pathway).
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).  No entry point
 *     synchronises the host with the device.
 *   - Return value: MINTB_OK, or a negative MINTB_E* code for an argument rejected on the host before
 *     anything was launched; mintb_last_error() then holds a message for the calling thread.
 *   - `dev_status` (device int32, caller-zeroed, may be NULL): kernels with bounded waits store a
 *     non-zero code there if a wait ran out, and return; they never trap and never spin forever.
 */
#ifndef MINTB_H_
#define MINTB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define MINTB_API __attribute__((visibility("default")))
#else
#define MINTB_API
#endif

#define MINTB_OK 0
#define MINTB_EINVAL (-1)       /* bad shape / null pointer / misaligned pointer                   */
#define MINTB_EUNSUPPORTED (-2) /* valid request this library does not implement (fails loudly)    */
#define MINTB_EWORKSPACE (-3)   /* workspace smaller than the matching *_workspace_bytes() answer  */
#define MINTB_ECUDA (-4)        /* a CUDA runtime/driver call failed (launch, descriptor encode)   */

/* dtype of q/k/v/out/grads */
#define MINTB_F32 0
#define MINTB_BF16 1
#define MINTB_E4M3 2 /* operands / outputs of the projection GEMMs only */
#define MINTB_E5M2 3 /* gradient operand of the backward projection GEMMs only */

/* flags */
#define MINTB_FLAG_ROPE 1u         /* rotate Q and K of the SELF pathway (rotary_embedding.py:47-55)                */
#define MINTB_FLAG_SQRT_SOFTMAX 2u /* sqrt(softmax) coefficients (mu_scaling/layer.py:162-163)                       */
#define MINTB_FLAG_FORCE_SIMT 4u   /* run the fp32 CUDA-core kernels even where the tcgen05 kernels apply (checking) */
#define MINTB_FLAG_ROT_SAVED 16u    /* mintb_attn_bwd only, with MINTB_FLAG_ROPE: `workspace` is the very buffer mintb_attn_fwd was
                                      given for the same inputs (sized for the backward pass), so the rotated copies of Q_self and
                                      K_self at its start are reused instead of being computed again */
#define MINTB_FLAG_SKIP_PAD_QUERIES 32u /* query tiles of 128 rows that hold only padded positions are not computed: their rows of
                                      `out` / `lse` stay unwritten and contribute nothing to the gradients (their d_out rows are
                                      ignored).  For callers that drop padded tokens from the token-wise work */
#define MINTB_FLAG_QK_PREROTATED 64u /* with MINTB_FLAG_ROPE: q_self and k_self are given already rotated (the fused QKV product rotates
                                      them in its epilogue); they are used as they are, and the gradients come back with respect to
                                      the un-rotated projections (the transposed rotation is applied to dq_self, dk_self) */
#define MINTB_FLAG_GRAD_ROWMAJOR 128u /* mintb_attn_bwd: the six gradients are written straight into the [T*B][3E] row-major input
                                      gradient of a fused QKV projection: element (t,b,h,d) of a gradient goes to
                                      ptr[(t*B + b)*3E + h*D + d]; the caller passes dq = G, dk = G + E, dv = G + 2E per pathway */
#define MINTB_FLAG_OUT_SEQ_FIRST 8u /* `out` and `d_out` are laid out (T,B,H,D) — the layer's (T,B,E) — instead of (B,H,T,D):
                                      saves the permute copy before out_proj (modules.py:146-150) and the one of its gradient */

MINTB_API int mintb_version(void);
MINTB_API const char* mintb_last_error(void);
/* Number of CUDA kernels this library has launched in this process so far (instrumentation; the reference
 * has no counterpart). */
MINTB_API unsigned long long mintb_kernel_launches(void);

/* Self-test of the bounded waits (no counterpart in the reference).  Launches a one-CTA kernel with the set-up of the
 * tensor-core kernels whose consumer waits on a barrier that is never completed; after limit_ns (at most 1e9) the wait
 * gives up, *dev_status receives 0x901 (if it was 0), TMEM is released and the kernel returns - nothing traps, nothing
 * spins on.  trail (device int[2], may be NULL) receives {2, 1}: the wait gave up, and TMEM was released after it. */
MINTB_API int mintb_selftest_wait(unsigned long long limit_ns, int* dev_status, int* trail, void* stream);

/* The persistent kernels (attention forward, the GEMMs) draw their work units from counters in the library image; the last
 * CTA of a launch clears the launch's counter again.  After a launch gave up on a bounded wait (a device status was raised)
 * some CTAs may not have left their counter: call this before launching again.  It synchronises the device. */
MINTB_API int mintb_reset_work_counters(void);

/* ---------------------------------------------------------------------------------------------------
 * Mask metadata.  Replaces the (B,T,T) bool tensor the reference builds every step (esm2.py:89) and
 * re-reads per head (modules.py:129-141; multi_pathway_attention.py:101-128): one bit per (query,key)
 * pair, one bit per key for padding (attention.py:230-236), and a class byte per 64x64 tile
 * (bit0: has an intra-chain pair, bit1: has an inter-chain pair, bit2: has a padded key).
 * `meta` must hold mintb_mask_meta_bytes(B,T) bytes, 256-byte aligned; build it once per batch.
 * key_pad may be NULL (no padding).
 */
MINTB_API size_t mintb_mask_meta_bytes(int B, int T);
MINTB_API int mintb_mask_meta_from_chain_ids(const int32_t* chain_ids, const uint8_t* key_pad, void* meta, int B, int T,
                                   void* stream);
MINTB_API int mintb_mask_meta_from_mask(const uint8_t* chain_mask, const uint8_t* key_pad, void* meta, int B, int T,
                              void* stream);

/* RoPE tables cos/sin [T][D/2] (float) from inv_freq [D/2] (float, device), as rotary_embedding.py:47-53
 * computes them: angle = float(position) * inv_freq. */
MINTB_API int mintb_rope_tables(const float* inv_freq, float* cos_tab, float* sin_tab, int T, int D, void* stream);

/* ---------------------------------------------------------------------------------------------------
 * Attention forward.  Replaces fused_multi_pathway_attention (kernels/multi_pathway_attention.py:184-280)
 * and the PyTorch path it mirrors (modules.py:94-154): out = (P o ~M) V_self + (P o M) V_cross with
 * P = softmax_keys(where(M, scale*Q_cross K_cross^T, scale*R(Q_self) R(K_self)^T)), padded keys -inf.
 * With MINTB_FLAG_ROPE the kernel rotates the self pathway (rope_cos/rope_sin required) — pass raw
 * projections and scale = D^-0.5; without it the caller has already scaled and rotated
 * (multi_pathway_attention.py:199-202) — pass scale = 1.
 * lse [B][H][T] receives log(sum_j exp(logit_ij)) for the backward pass.
 * The workspace holds the rotated copies of q_self and k_self (MINTB_FLAG_ROPE only; otherwise none is needed).
 */
MINTB_API size_t mintb_attn_fwd_workspace_bytes(int B, int H, int T, int D, int dtype, unsigned flags);
MINTB_API int mintb_attn_fwd(const void* q_self, const void* k_self, const void* v_self, const void* q_cross,
                   const void* k_cross, const void* v_cross, const void* meta, const float* rope_cos,
                   const float* rope_sin, void* out, float* lse, void* workspace, size_t workspace_bytes, int B,
                   int H, int T, int D, int dtype, unsigned flags, float scale, void* stream, int* dev_status);

/* No-allocation forward.  It has no counterpart in the reference.  Some callers of this library cannot allocate device
 * memory at the point where they call it: code that runs while a CUDA graph is being captured, real-time or
 * fixed-memory-budget hosts that forbid cudaMalloc after start-up, and host languages whose bindings hand over
 * pre-pinned buffers only.  For them this variant of mintb_attn_fwd (bf16 tensor-core path) keeps the scratch it needs
 * with MINTB_FLAG_ROPE - the rotated copies of q_self and k_self - in an array of MINTB_STATIC_SCRATCH_BYTES inside the
 * library image, so the caller passes inputs and outputs only and nothing is allocated or freed, here or in any
 * library routine it calls.  Limits and rules:
 *   - 2 * B*H*T*D * 2 bytes must fit the array (B*H*T*D <= 8 Mi elements with rope); larger calls return
 *     MINTB_EWORKSPACE with a message and launch nothing.  Every GPU that loads the library holds the array until exit.
 *   - The first call on each device looks the array's device address up (with that device current); make that first
 *     call outside any stream capture.
 *   - All calls on a device share the one array.  Nothing in it has to start at zero (each call rewrites what it
 *     reads), but two calls that overlap on the GPU - different streams, or threads - race on it: serialise them.
 */
#define MINTB_STATIC_SCRATCH_BYTES (32u << 20)
MINTB_API int mintb_attn_fwd_static(const void* q_self, const void* k_self, const void* v_self, const void* q_cross,
                                    const void* k_cross, const void* v_cross, const void* meta, const float* rope_cos,
                                    const float* rope_sin, void* out, float* lse, int B, int H, int T, int D, int dtype,
                                    unsigned flags, float scale, void* stream, int* dev_status);

/* Attention backward.  Replaces fused_multi_pathway_attention_bwd (kernels/multi_pathway_attention_bwd.py:15-59)
 * with what torch.autograd computes through modules.py:129-144: probabilities are recomputed from lse;
 * dq/dk of the self pathway are un-rotated and dq is multiplied by scale, so the six results are the
 * gradients w.r.t. the tensors that were passed to mintb_attn_fwd.
 * Reproducibility: dk and dv are reduced in a fixed order and are bit-identical from run to run; on the bf16 tensor-core
 * path dq is summed over key tiles in fp32 in the order the CTAs happen to arrive (one rounding to bf16 at the end), so
 * its last bf16 bit may differ between two runs on the same inputs.  The fp32 path (and MINTB_FLAG_FORCE_SIMT) is
 * bit-reproducible for all six. */
MINTB_API size_t mintb_attn_bwd_workspace_bytes(int B, int H, int T, int D, int dtype, unsigned flags);
MINTB_API int mintb_attn_bwd(const void* q_self, const void* k_self, const void* v_self, const void* q_cross,
                   const void* k_cross, const void* v_cross, const void* meta, const float* rope_cos,
                   const float* rope_sin, const void* out, const float* lse, const void* d_out, void* dq_self,
                   void* dk_self, void* dv_self, void* dq_cross, void* dk_cross, void* dv_cross, void* workspace,
                   size_t workspace_bytes, int B, int H, int T, int D, int dtype, unsigned flags, float scale,
                   void* stream, int* dev_status);
/* mintb_attn_bwd for callers whose token-wise tensors hold only the unpadded tokens (the reference pads every batch to
 * its longest pair, data/data.py:63-129, and has no such mode).  With MINTB_FLAG_GRAD_ROWMAJOR the two gradient matrices
 * then have one row per kept token, [n_rows][3E]: token_row[t*B + b] (int32, device) is the row of token (t, b), negative
 * for a token without a row, whose gradients are dropped.  token_row == NULL is mintb_attn_bwd. */
MINTB_API int mintb_attn_bwd_rows(const void* q_self, const void* k_self, const void* v_self, const void* q_cross,
                   const void* k_cross, const void* v_cross, const void* meta, const float* rope_cos,
                   const float* rope_sin, const void* out, const float* lse, const void* d_out, void* dq_self,
                   void* dk_self, void* dv_self, void* dq_cross, void* dk_cross, void* dv_cross, void* workspace,
                   size_t workspace_bytes, int B, int H, int T, int D, int dtype, unsigned flags, float scale,
                   void* stream, int* dev_status, const int32_t* token_row);

/* ---------------------------------------------------------------------------------------------------
 * Combine from materialised logits.  Replaces fused_multimer_combine / fused_multimer_combine_bwd
 * (kernels/__init__.py:179-286): logits [B][H][T][T] of both pathways already hold -inf on padded keys.
 * Backward follows autograd: d_intra_logits is zero where the mask selects the cross pathway and vice versa;
 * its workspace holds the per-row softmax statistics between its two kernels.
 */
MINTB_API int mintb_combine_fwd(const void* intra_logits, const void* inter_logits, const uint8_t* chain_mask,
                      const void* intra_values, const void* inter_values, void* out, int B, int H, int T, int D,
                      int dtype, void* stream);
MINTB_API size_t mintb_combine_bwd_workspace_bytes(int B, int H, int T);
MINTB_API int mintb_combine_bwd(const void* intra_logits, const void* inter_logits, const uint8_t* chain_mask,
                      const void* intra_values, const void* inter_values, const void* d_out, void* d_intra_logits,
                      void* d_inter_logits, void* d_intra_values, void* d_inter_values, void* workspace,
                      size_t workspace_bytes, int B, int H, int T, int D, int dtype, void* stream);

/* ---------------------------------------------------------------------------------------------------
 * Projection GEMMs (tcgen05, bf16 or e4m3 operands, fp32 accumulate) with fused epilogues.
 * x [M][K] and w [N][K] are K-contiguous (nn.Linear layout); K * element size must be a multiple of 16 bytes.
 *
 * mintb_linear_fwd: out[M][N] = act(alpha * x w^T + bias), act = erf-GELU if `gelu` (modules.py:16-23,323-335), stored as
 * bf16 or, multiplied by out_scale and saturated to +-448, as e4m3.  Replaces nn.Linear / te.Linear forward for out_proj,
 * fc1(+GELU), fc2 (attention.py:68, modules.py:326-334, mu_scaling/__init__.py:83-124).  For e4m3 operands alpha is the
 * product of the two per-tensor dequantisation scales times any static output multiplier (alt/munit_scaling.py:22-34).
 * With `gelu`, a non-null `preact_out` (bf16 [M][N]) also receives alpha * x w^T + bias, which the GELU backward reads.
 *
 * mintb_qkv_fwd: the fused QKV projection of one pathway (attention.py:97-117, 304-323): x is (T,B,E) flattened to
 * [T*B][E], w [3E][E] with rows ordered [Q;K;V]; q, k, v are written head-major (B,H,T,D) directly (no permute copy),
 * the q third multiplied by q_scale, and the q and k thirds rotated by RoPE when the tables are given.  With padding
 * dropped from the token-wise work (variable-length packing) x holds only the n_rows unpadded tokens and row_map[m] = t * B + b
 * names the token of row m; positions that no row maps to are left untouched in q, k, v (row_map null: all T * B rows).
 *
 * mintb_quantize_e4m3: out[i] = saturate(x[i] * inv_scale) from bf16 (the per-tensor scaled cast of the FP8 path).
 */
MINTB_API int mintb_linear_fwd(const void* x, const void* w, const void* bias, void* out, void* preact_out, int M, int N, int K,
                               int in_dtype, int bias_dtype, int out_dtype, int gelu, float alpha, float out_scale, void* stream,
                               int* dev_status);
MINTB_API int mintb_qkv_fwd(const void* x, const void* w, const void* bias, void* q, void* k, void* v, int T, int B, int H,
                            int D, int in_dtype, int bias_dtype, float alpha, float q_scale, const float* rope_cos,
                            const float* rope_sin, const int32_t* row_map, int n_rows, void* stream, int* dev_status);
MINTB_API int mintb_quantize_e4m3(const void* x, void* out, size_t n, float inv_scale, void* stream);
/* mintb_linear_res_fwd: mintb_linear_fwd without activation and with the layer's residual sum formed in the epilogue:
 * out[M][N] = res_a * resid[M][N] + res_b * (alpha * x w^T + bias) - x + out_proj(attention) of the Pre-LN layer
 * (modules.py:183-186: res_a = res_b = 1) and sqrt(1 - tau) x + sqrt(tau) out_proj(attention) of the muS layer
 * (mu_scaling/layer.py:262-266).  resid bf16 (NULL: no residual).  With an e4m3 `out` (the operand of the projection that
 * reads the sum next) bf16_copy_out, when non-null, receives the sum in bf16 and the e4m3 numbers are cast from those bf16
 * values.
 * mintb_qkv2_fwd: mintb_qkv_fwd for BOTH pathways of a layer in one product: w is [6E][E] with rows [Q1;K1;V1;Q2;K2;V2],
 * bias [6E]; the first pathway's q and k are rotated when the tables are given, the second pathway's never; alpha1 / alpha2
 * multiply the two pathways' columns (their weights carry separate e4m3 scales); q_scale multiplies both q thirds.  The
 * activation is read once instead of twice (modules.py:179-195 computes the two projections as separate Linears). */
MINTB_API int mintb_linear_res_fwd(const void* x, const void* w, const void* bias, const void* resid, float res_a, float res_b,
                                   void* out, void* bf16_copy_out, int M, int N, int K, int in_dtype, int bias_dtype,
                                   int out_dtype, float alpha, float out_scale, void* stream, int* dev_status);
MINTB_API int mintb_qkv2_fwd(const void* x, const void* w, const void* bias, void* q1, void* k1, void* v1, void* q2, void* k2,
                             void* v2, int T, int B, int H, int D, int in_dtype, int bias_dtype, float alpha1, float alpha2,
                             float q_scale, const float* rope_cos, const float* rope_sin, const int32_t* row_map, int n_rows,
                             void* stream, int* dev_status);

/* Backward of the projections: the two products torch.autograd forms for y = x w^T (attention.py:68, modules.py:326-334;
 * te.Linear's backward under mu_scaling/__init__.py:83-124; alt/munit_scaling.py:36-55 states the 8-bit variant: gradient
 * in e5m2 against e4m3 weights / activations).  All matrices are row-major as the forward pass left them - none is
 * transposed in memory.  Operands are both bf16, or both 8-bit floats (MINTB_E4M3 / MINTB_E5M2 per operand); fp32 accumulate.
 *
 * mintb_linear_dgrad: dx[M][K] = alpha * (dz[M][N] w[N][K] + dz2[M][N2] w2[N2][K]), stored as bf16.  The second pair is
 *   optional (dz2 = w2 = NULL, N2 = 0): two projections of one activation (the self and cross QKV products) add their input
 *   gradients in one accumulator instead of a separate pass.  For 8-bit operands alpha carries the dequantisation scales.
 * mintb_linear_wgrad: dw[N][K] = alpha * dz^T x with dz[M][N], x[M][K]; dw is fp32 or bf16.  The reduction over the M
 *   tokens is cut into aligned splits that add fp32 partial tiles into one fp32 matrix: dw itself when it is fp32, else
 *   `workspace` (mintb_linear_wgrad_workspace_bytes), which a final pass converts to bf16.  The order of those additions is
 *   not fixed, so the last bits of dw may differ from run to run when more than one split is used.
 */
MINTB_API int mintb_linear_dgrad(const void* dz, const void* w, const void* dz2, const void* w2, void* dx, int M, int N, int K,
                                 int N2, int dz_dtype, int w_dtype, float alpha, void* stream, int* dev_status);
MINTB_API size_t mintb_linear_wgrad_workspace_bytes(int N, int K, int out_dtype);
MINTB_API int mintb_linear_wgrad(const void* dz, const void* x, void* dw, void* workspace, size_t workspace_bytes, int M, int N,
                                 int K, int dz_dtype, int x_dtype, int out_dtype, float alpha, void* stream, int* dev_status);

/* ---------------------------------------------------------------------------------------------------
 * HBM-bound glue of the layer around the GEMMs and the attention (bf16 tensors [rows][E] / [M][N], fp32 arithmetic).
 *
 * mintb_add_layernorm_fwd: s = a x + b r (r may be null), y = LayerNorm(s) * gamma + beta over the last dimension.
 *   Replaces the residual add + ESM1bLayerNorm pairs of the Pre-LN layer (modules.py:179-195: a = b = 1) and the weighted
 *   residuals + final norm of the muS layer (mu_scaling/layer.py:259-280: a = sqrt(1 - tau), b = sqrt(tau)).  gamma null:
 *   no normalisation, only s_out is written.  Otherwise y_out is written, s_out if non-null, and stats[rows] = (mean, rstd)
 *   (2 floats per row) if non-null.  E must be a multiple of 8, at most 2560; gamma / beta are f32 or bf16 (param_dtype).
 * mintb_add_layernorm_bwd: ds = dLayerNorm(dy) + ds_in (either part may be absent), dx = a ds, dr = b ds (dr may be null),
 *   dgamma / dbeta (fp32 [E]) summed in a fixed order through the workspace; both null (frozen parameters) skips them and
 *   needs no workspace.
 * mintb_gelu_bwd_colsum: with z: dz = dy * gelu'(z) (erf form, modules.py:16-23) and db[N] = column sums of dz (db may be
 *   null); without z: db = column sums of dy (the bias gradient of a projection).  N a multiple of 8.
 *   mintb_gelu_bwd_colsum_act also writes act = gelu(z) (bf16 [M][N], may be null) in the same pass: the forward pass of an
 *   FFN whose fc1 hands its result to fc2 as e4m3 keeps only z, and fc2's weight gradient reads this copy.
 * mintb_qkv_grad_pack: the gradients of head-major q, k, v (B,H,T,D) gathered into one [T*B][3E] matrix with columns
 *   [dQ | dK | dV], dq multiplied by q_scale and dq, dk un-rotated (transpose of the RoPE rotation) when tables are given:
 *   the inverse of mintb_qkv_fwd's epilogue, feeding the dgrad / wgrad products of the fused QKV projection; a non-null
 *   db (fp32 [3E]) receives the column sums of that matrix, the bias gradient, from the same pass.
 */
MINTB_API int mintb_add_layernorm_fwd(const void* x, const void* r, float a, float b, const void* gamma, const void* beta,
                                      int param_dtype, void* s_out, void* y_out, float* stats, int rows, int E, float eps,
                                      void* stream);
/* the same, also writing an e4m3 copy q_out[rows][E] = sat(result * q_inv_scale) of the main result (y with gamma, else s):
 * the operand of the next e4m3 projection without a separate cast pass */
MINTB_API int mintb_add_layernorm_fwd_q(const void* x, const void* r, float a, float b, const void* gamma, const void* beta,
                                        int param_dtype, void* s_out, void* y_out, float* stats, int rows, int E, float eps,
                                        void* q_out, float q_inv_scale, void* stream);
MINTB_API size_t mintb_add_layernorm_bwd_workspace_bytes(int rows, int E);
MINTB_API int mintb_add_layernorm_bwd(const void* dy, const void* ds_in, const void* x, const void* r, float a, float b,
                                      const void* gamma, int param_dtype, const float* stats, void* dx, void* dr, float* dgamma,
                                      float* dbeta, void* workspace, size_t workspace_bytes, int rows, int E, void* stream);
MINTB_API int mintb_gelu_bwd_colsum(const void* dy, const void* z, void* dz, float* db, int M, int N, void* stream);
MINTB_API int mintb_gelu_bwd_colsum_act(const void* dy, const void* z, void* dz, void* act, float* db, int M, int N,
                                        void* stream);
/* mintb_gelu_bwd_colsum_act with an 8-bit copy of the result for the 8-bit dgrad / wgrad products: dz_e5m2[M][N] =
 * saturate_e5m2(dz / e5m2_scale) (alt/munit_scaling.py:41-45 of the reference: the gradient is scaled, clamped to +-57344
 * and cast to e5m2), written by the same pass; dz (bf16) may then be NULL.  db then sums the e5m2 numbers times e5m2_scale,
 * the very values the products read (alt/munit_scaling.py:55). */
MINTB_API int mintb_gelu_bwd_colsum_f8(const void* dy, const void* z, void* dz, void* act, float* db, void* dz_e5m2,
                                       float e5m2_scale, int M, int N, void* stream);
MINTB_API int mintb_qkv_grad_pack(const void* dq, const void* dk, const void* dv, void* g, float* db, const float* rope_cos,
                                  const float* rope_sin, const int32_t* row_map, int n_rows, int T, int B, int H, int D,
                                  float q_scale, void* stream);

/* ---------------------------------------------------------------------------------------------------
 * The two ends of the model around the layer stack (HBM-bound, one pass each).
 *
 * mintb_embed_fwd: the prologue of MINT.forward (esm2.py:91-104): out[t][b][:] = weight[tokens[b][t]][:] * f(b, t), written
 *   sequence-first (T,B,E); f = 0 for <pad>, 0 for <mask> when token_dropout, else the row's rescale
 *   (1 - mask_ratio_train) / (1 - masked_b / unpadded_b) when token_dropout, else 1.  tokens int64 [B][T]; weight and out
 *   f32 or bf16 (dtype); row_scales[B] (may be NULL) receives the rescale of each row for the backward pass.
 * mintb_embed_bwd: d_weight[V][E] (fp32, overwritten) = sum over tokens of f(b, t) * d_out[t][b][:] into row tokens[b][t]
 *   (private sums per CTA, then fp32 atomics: the order of the additions is not fixed).  V <= 64.
 * mintb_masked_ce_fwd: the loss of the masked-language-model step (training/wrapper.py:77-80): sums[0] = sum over rows with
 *   mask != 0 of (logsumexp(logits[i][:V]) - logits[i][targets[i]]), sums[1] = number of such rows, lse[i] for the backward
 *   pass; logits bf16 [N][ld] (ld >= V: row stride in elements), fp32 arithmetic.  The mean is sums[0] / sums[1].
 * mintb_masked_ce_bwd: d_logits[N][ld] (bf16) = (softmax(logits[i]) - onehot(targets[i])) * grad_loss[0] / sums[1] at the
 *   masked rows, 0 elsewhere and in the columns past V.
 */
MINTB_API int mintb_embed_fwd(const long long* tokens, const void* weight, void* out, float* row_scales, int B, int T, int E, int V,
                              int dtype, int pad_idx, int mask_idx, int token_dropout, float mask_ratio_train, void* stream);
MINTB_API int mintb_embed_bwd(const long long* tokens, const void* d_out, const float* row_scales, float* d_weight, int B, int T,
                              int E, int V, int dtype, int pad_idx, int mask_idx, int token_dropout, void* stream);
MINTB_API int mintb_masked_ce_fwd(const void* logits, const long long* targets, const unsigned char* mask, float* lse, float* sums,
                                  int N, int ld, int V, void* stream);
MINTB_API int mintb_masked_ce_bwd(const void* logits, const long long* targets, const unsigned char* mask, const float* lse,
                                  const float* sums, const float* grad_loss, void* d_logits, int N, int ld, int V, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MINTB_H_ */
