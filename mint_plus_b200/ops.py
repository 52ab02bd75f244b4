"""Tensor-facing operators over libmintb: mask metadata, RoPE tables, and the autograd function of the
combined-softmax multimer attention.  PyTorch supplies device memory, streams and autograd glue only;
every computation runs in the CUDA library (there is no eager fallback).
"""
from __future__ import annotations

import weakref
from typing import Optional, Tuple

import torch

from . import _lib as L

_DTYPES = {torch.float32: L.F32, torch.bfloat16: L.BF16}


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("mint_plus_b200 operators run on CUDA tensors only (no CPU fallback)")


class _NoCtx:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_CTX = _NoCtx()


def _on(device):
    """Context that makes `device` the current CUDA device for a library call; free when it already is (the usual case:
    switching costs several microseconds of host time per call, and a training step makes thousands of calls)."""
    return _NO_CTX if torch.cuda.current_device() == device.index else torch.cuda.device(device)


def _workspace(nbytes: int, device) -> Optional[torch.Tensor]:
    # torch's caching allocator hands out 512-byte aligned blocks
    return torch.empty(nbytes, dtype=torch.uint8, device=device) if nbytes else None


# ----------------------------------------------------------------------------------------------- status word
_status = {}


def _dev_status(device) -> torch.Tensor:
    key = torch.device(device).index
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def check_device_status(device=None) -> None:
    """Synchronise and raise if a kernel reported a bounded wait that ran out."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    code = int(_dev_status(device).item())
    if code != 0:
        _dev_status(device).zero_()
        with _on(device):
            L.lib().mintb_reset_work_counters()   # CTAs that gave up may not have left their work counter
        raise L.MintbError(f"a mintb kernel gave up a bounded wait (device status 0x{code:x})")


# ----------------------------------------------------------------------------------------------- mask metadata
class MaskMeta:
    """Packed chain/padding mask of one batch (see include/mintb.h): build once, use for every layer and head."""

    def __init__(self, buf: torch.Tensor, B: int, T: int):
        self.buf, self.B, self.T = buf, B, T


def _key_pad_u8(key_padding_mask, B, T):
    if key_padding_mask is None:
        return None
    if tuple(key_padding_mask.shape) != (B, T):
        raise ValueError(f"key_padding_mask must be (B, T) = ({B}, {T}), got {tuple(key_padding_mask.shape)}")
    return key_padding_mask.to(torch.uint8).contiguous()


def mask_meta_from_chain_ids(chain_ids: torch.Tensor, key_padding_mask: Optional[torch.Tensor] = None) -> MaskMeta:
    """chain_ids (B,T) integer; key_padding_mask (B,T) bool, True = padded key (esm2.py:85,89)."""
    _require_cuda(chain_ids, key_padding_mask)
    B, T = chain_ids.shape
    cid = chain_ids.to(torch.int32).contiguous()
    pad = _key_pad_u8(key_padding_mask, B, T)
    buf = torch.empty(L.lib().mintb_mask_meta_bytes(B, T), dtype=torch.uint8, device=cid.device)
    with _on(cid.device):
        L.check(L.lib().mintb_mask_meta_from_chain_ids(_ptr(cid), _ptr(pad), _ptr(buf), B, T, _stream()),
                "mask_meta_from_chain_ids")
    return MaskMeta(buf, B, T)


def mask_meta_from_mask(chain_mask: torch.Tensor, key_padding_mask: Optional[torch.Tensor] = None) -> MaskMeta:
    """chain_mask (B,T,T) bool, True = different chains (cross pathway)."""
    _require_cuda(chain_mask, key_padding_mask)
    if chain_mask.dim() != 3 or chain_mask.shape[1] != chain_mask.shape[2]:
        raise ValueError(f"chain_mask must be (B, T, T), got {tuple(chain_mask.shape)}")
    B, T, _ = chain_mask.shape
    m = chain_mask.to(torch.uint8).contiguous() if chain_mask.dtype != torch.bool else chain_mask.contiguous().view(torch.uint8)
    pad = _key_pad_u8(key_padding_mask, B, T)
    buf = torch.empty(L.lib().mintb_mask_meta_bytes(B, T), dtype=torch.uint8, device=m.device)
    with _on(m.device):
        L.check(L.lib().mintb_mask_meta_from_mask(_ptr(m), _ptr(pad), _ptr(buf), B, T, _stream()), "mask_meta_from_mask")
    return MaskMeta(buf, B, T)


_meta_cache = []  # [(weakref(mask), version, weakref(pad) | None, pad version, MaskMeta)], newest first


def cached_mask_meta(chain_mask: torch.Tensor, key_padding_mask: Optional[torch.Tensor] = None) -> MaskMeta:
    """Metadata for a (B,T,T) mask, reused while the same tensor objects are passed again (every layer of a
    forward pass receives the same mask, esm2.py:124-132)."""
    for ref_m, ver_m, ref_p, ver_p, meta in _meta_cache:
        if ref_m() is chain_mask and ver_m == chain_mask._version:
            if key_padding_mask is None and ref_p is None:
                return meta
            if key_padding_mask is not None and ref_p is not None and ref_p() is key_padding_mask \
                    and ver_p == key_padding_mask._version:
                return meta
    meta = mask_meta_from_mask(chain_mask, key_padding_mask)
    _meta_cache.insert(0, (weakref.ref(chain_mask), chain_mask._version,
                           None if key_padding_mask is None else weakref.ref(key_padding_mask),
                           0 if key_padding_mask is None else key_padding_mask._version, meta))
    del _meta_cache[4:]
    return meta


# ----------------------------------------------------------------------------------------------- RoPE tables
_rope_cache = {}


def default_inv_freq(D: int, device) -> torch.Tensor:
    """rotary_embedding.py:43: 1 / 10000^(2i/D), fp32."""
    return (1.0 / (10000 ** (torch.arange(0, D, 2).float() / D))).to(device)


def rope_tables(T: int, D: int, device,
                inv_freq: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """(cos, sin, inv_freq): the cos/sin tables (T, D/2) fp32 on `device`, cached per (T, D, device, inv_freq contents); the
    third entry is the caller's inv_freq (None for the default frequencies), held so that the cache key stays valid."""
    device = torch.device(device)
    key = (T, D, device.index, inv_freq.data_ptr() if inv_freq is not None else 0,
           inv_freq._version if inv_freq is not None else 0)
    hit = _rope_cache.get(key)
    if hit is not None:
        return hit
    inv = default_inv_freq(D, device) if inv_freq is None else inv_freq.detach().to(device=device, dtype=torch.float32).contiguous()
    if inv.numel() != D // 2:
        raise ValueError(f"inv_freq must have D/2 = {D // 2} entries")
    cos = torch.empty(T, D // 2, dtype=torch.float32, device=device)
    sin = torch.empty_like(cos)
    with _on(device):
        L.check(L.lib().mintb_rope_tables(_ptr(inv), _ptr(cos), _ptr(sin), T, D, _stream()), "rope_tables")
    if len(_rope_cache) > 16:
        _rope_cache.clear()
    _rope_cache[key] = (cos, sin, inv_freq)   # keeps the buffer alive so its address cannot be reused under this key
    return _rope_cache[key]


# ----------------------------------------------------------------------------------------------- attention
class _MultimerAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q_s, k_s, v_s, q_c, k_c, v_c, meta: MaskMeta, cos, sin, scale: float, flags: int, grad_tabs=None):
        B, H, T, D = q_s.shape
        dt = _DTYPES[q_s.dtype]
        lib = L.lib()
        # sequence-first result: (T,B,H,D), which the layer views as its (T,B,E) activations without a copy
        out = torch.empty((T, B, H, D) if flags & L.FLAG_OUT_SEQ_FIRST else (B, H, T, D), dtype=q_s.dtype, device=q_s.device)
        lse = torch.empty(B, H, T, dtype=torch.float32, device=q_s.device)
        ws_bytes = lib.mintb_attn_fwd_workspace_bytes(B, H, T, D, dt, flags)
        # With in-kernel RoPE the forward pass leaves rotated copies of Q_self and K_self at the start of its workspace.  When a
        # backward pass will follow, the workspace is sized for it and kept, so that pass starts from those copies.
        keep_ws = bool(flags & L.FLAG_ROPE) and not (flags & L.FLAG_QK_PREROTATED) and any(ctx.needs_input_grad[:6])
        if keep_ws:
            ws_bytes = max(ws_bytes, lib.mintb_attn_bwd_workspace_bytes(B, H, T, D, dt, flags))
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q_s.device)
        else:
            ws = _workspace(ws_bytes, q_s.device)
        ctx.fwd_ws = ws if keep_ws else None
        with _on(q_s.device):
            rc = lib.mintb_attn_fwd(_ptr(q_s), _ptr(k_s), _ptr(v_s), _ptr(q_c), _ptr(k_c), _ptr(v_c), _ptr(meta.buf),
                                    _ptr(cos), _ptr(sin), _ptr(out), _ptr(lse), _ptr(ws), ws_bytes, B, H, T, D, dt,
                                    flags, scale, _stream(), _ptr(_dev_status(q_s.device)))
        L.check(rc, "mintb_attn_fwd")
        ctx.save_for_backward(q_s, k_s, v_s, q_c, k_c, v_c, out, lse, cos, sin)
        ctx.meta, ctx.scale, ctx.flags = meta, scale, flags
        ctx.grad_tabs = grad_tabs
        return out

    @staticmethod
    def backward(ctx, d_out):
        grads, _, _ = _attention_backward(ctx, d_out)
        return (*grads, None, None, None, None, None, None)


def _attention_backward(ctx, d_out, pack=None):
    """Backward pass of `_MultimerAttentionFn` for a context `ctx` of its forward pass.  Returns (the six gradients as
    (B,H,T,D) tensors or views, g_self, g_cross); the last two are the row-major [rows][3E] matrices [dQ | dK | dV] when the
    context asked for them (`grad_tabs`), else None.  With `pack` those matrices hold only the unpadded tokens' rows (the
    kernels drop the others), and the six per-tensor gradients are not formed (None)."""
    q_s, k_s, v_s, q_c, k_c, v_c, out, lse, cos, sin = ctx.saved_tensors
    B, H, T, D = q_s.shape
    dt = _DTYPES[q_s.dtype]
    lib = L.lib()
    d_out = d_out.contiguous()
    flags = ctx.flags
    rowmajor = ctx.grad_tabs is not None
    g_s = g_c = None
    if rowmajor:
        # The inputs came from the fused QKV products (q, k of the self pathway already rotated there): the gradients are
        # written straight into the [rows][3E] matrices those products' backward passes consume — un-rotated, no gather pass.
        E = H * D
        n_rows = pack.n if pack is not None else T * B
        g_s, g_c = (torch.empty(n_rows, 3 * E, dtype=q_s.dtype, device=q_s.device) for _ in range(2))
        grads = [g_s[:, :E], g_s[:, E:2 * E], g_s[:, 2 * E:], g_c[:, :E], g_c[:, E:2 * E], g_c[:, 2 * E:]]
        if ctx.grad_tabs[0] is not None:
            cos, sin = ctx.grad_tabs
            flags |= L.FLAG_ROPE | L.FLAG_QK_PREROTATED
        flags |= L.FLAG_GRAD_ROWMAJOR
    else:
        if pack is not None:
            raise ValueError("packed gradient rows need the row-major gradient layout")
        grads = [torch.empty_like(q_s) for _ in range(6)]
    ws_bytes = lib.mintb_attn_bwd_workspace_bytes(B, H, T, D, dt, flags)
    if ctx.fwd_ws is not None:
        ws, ws_bytes, flags = ctx.fwd_ws, ctx.fwd_ws.numel(), flags | L.FLAG_ROT_SAVED
    else:
        ws = _workspace(ws_bytes, q_s.device)
    with _on(q_s.device):
        rc = lib.mintb_attn_bwd_rows(_ptr(q_s), _ptr(k_s), _ptr(v_s), _ptr(q_c), _ptr(k_c), _ptr(v_c), _ptr(ctx.meta.buf),
                                     _ptr(cos), _ptr(sin), _ptr(out), _ptr(lse), _ptr(d_out), *[_ptr(g) for g in grads],
                                     _ptr(ws), ws_bytes, B, H, T, D, dt, flags, ctx.scale, _stream(),
                                     _ptr(_dev_status(q_s.device)), _ptr(pack.inv32) if pack is not None else None)
    L.check(rc, "mintb_attn_bwd")
    if pack is not None:
        grads = [None] * 6
    elif rowmajor:   # hand each gradient back as the (B,H,T,D) view of its third of the row-major matrix
        grads = [g.view(T, B, H, D).permute(1, 2, 0, 3) for g in grads]
    return grads, g_s, g_c


def multimer_attention(q_self, k_self, v_self, q_cross, k_cross, v_cross, *, meta: Optional[MaskMeta] = None,
                       chain_ids=None, chain_mask=None, key_padding_mask=None, rope: bool = True,
                       inv_freq: Optional[torch.Tensor] = None, scale: Optional[float] = None,
                       sqrt_softmax: bool = False, force_simt: bool = False, out_seq_first: bool = False,
                       skip_pad_queries: bool = False, grad_rowmajor_tabs=None) -> torch.Tensor:
    """Two-pathway combined-softmax attention on (B,H,T,D) projections; differentiable.  The result is (B,H,T,D), or
    (T,B,H,D) with out_seq_first=True (the layout of the layer's (T,B,E) activations: no permute copy before out_proj).
    skip_pad_queries=True leaves out 128-row query tiles that hold only padded positions: their output rows stay unwritten.
    grad_rowmajor_tabs = (cos, sin) or (None, None): for inputs that came from `qkv_project` (q, k of the self pathway rotated
    there with these tables, rope=False here): the backward pass writes the gradients straight into the [T*B][3E] matrices
    the projections' backward passes consume, un-rotating dq_self / dk_self on the way (bf16 tensor-core path only).


    out = (P o ~M) V_self + (P o M) V_cross,  P = softmax_j where(M, s*Qc Kc^T, s*R(Qs) R(Ks)^T), padded keys -inf
    (modules.py:94-154 of the reference).  With rope=True the raw projections are passed and the kernels rotate
    the self pathway and apply `scale` (default D^-0.5); with rope=False and scale=1 the caller has done both,
    which is the calling convention of the reference's fused kernel (multi_pathway_attention.py:199-202).
    The mask comes from exactly one of `meta`, `chain_ids` (B,T) or `chain_mask` (B,T,T).
    """
    ts = (q_self, k_self, v_self, q_cross, k_cross, v_cross)
    _require_cuda(*ts)
    if q_self.dim() != 4 or any(t.shape != q_self.shape for t in ts):
        raise ValueError("q/k/v of both pathways must share one (B, H, T, D) shape")
    if q_self.dtype not in _DTYPES or any(t.dtype != q_self.dtype for t in ts):
        raise TypeError("q/k/v must all be float32 or all be bfloat16")
    B, H, T, D = q_self.shape
    if meta is None:
        if (chain_ids is None) == (chain_mask is None):
            raise ValueError("give exactly one of meta, chain_ids, chain_mask")
        meta = mask_meta_from_chain_ids(chain_ids, key_padding_mask) if chain_ids is not None \
            else cached_mask_meta(chain_mask, key_padding_mask)
    elif chain_ids is not None or chain_mask is not None or key_padding_mask is not None:
        raise ValueError("meta already carries the chain and padding masks")
    if (meta.B, meta.T) != (B, T):
        raise ValueError(f"mask metadata is for (B, T) = ({meta.B}, {meta.T}), tensors have ({B}, {T})")
    flags = ((L.FLAG_ROPE if rope else 0) | (L.FLAG_SQRT_SOFTMAX if sqrt_softmax else 0) | (L.FLAG_FORCE_SIMT if force_simt else 0)
             | (L.FLAG_OUT_SEQ_FIRST if out_seq_first else 0) | (L.FLAG_SKIP_PAD_QUERIES if skip_pad_queries else 0))
    cos = sin = None
    if rope:
        cos, sin, _ = rope_tables(T, D, q_self.device, inv_freq)
    if scale is None:
        scale = D ** -0.5
    ts = tuple(t.contiguous() for t in ts)
    if grad_rowmajor_tabs is not None and (rope or force_simt or q_self.dtype != torch.bfloat16 or D not in (16, 32, 64)):
        grad_rowmajor_tabs = None      # served by the bf16 tensor-core kernels on pre-rotated inputs only
    return _MultimerAttentionFn.apply(*ts, meta, cos, sin, float(scale), int(flags), grad_rowmajor_tabs)


# ----------------------------------------------------------------------------------------------- combine from logits
class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, il, el, mask_u8, iv, ev):
        B, H, T, D = iv.shape
        out = torch.empty_like(iv)
        with _on(iv.device):
            rc = L.lib().mintb_combine_fwd(_ptr(il), _ptr(el), _ptr(mask_u8), _ptr(iv), _ptr(ev), _ptr(out), B, H, T, D,
                                          _DTYPES[iv.dtype], _stream())
        L.check(rc, "mintb_combine_fwd")
        ctx.save_for_backward(il, el, mask_u8, iv, ev)
        return out

    @staticmethod
    def backward(ctx, d_out):
        il, el, mask_u8, iv, ev = ctx.saved_tensors
        B, H, T, D = iv.shape
        d_out = d_out.contiguous()
        d_il, d_el, d_iv, d_ev = torch.empty_like(il), torch.empty_like(el), torch.empty_like(iv), torch.empty_like(ev)
        lib = L.lib()
        ws_bytes = lib.mintb_combine_bwd_workspace_bytes(B, H, T)
        ws = _workspace(ws_bytes, iv.device)
        with _on(iv.device):
            rc = lib.mintb_combine_bwd(_ptr(il), _ptr(el), _ptr(mask_u8), _ptr(iv), _ptr(ev), _ptr(d_out), _ptr(d_il),
                                       _ptr(d_el), _ptr(d_iv), _ptr(d_ev), _ptr(ws), ws_bytes, B, H, T, D,
                                       _DTYPES[iv.dtype], _stream())
        L.check(rc, "mintb_combine_bwd")
        return d_il, d_el, None, d_iv, d_ev


def multimer_combine(intra_logits, inter_logits, chain_mask, intra_values, inter_values) -> torch.Tensor:
    """Combine from materialised (B,H,T,T) logits (kernels/__init__.py:179-242 of the reference); differentiable."""
    ts = (intra_logits, inter_logits, intra_values, inter_values)
    _require_cuda(*ts, chain_mask)
    B, H, T, D = intra_values.shape
    if tuple(intra_logits.shape) != (B, H, T, T) or inter_logits.shape != intra_logits.shape \
            or inter_values.shape != intra_values.shape or tuple(chain_mask.shape) != (B, T, T):
        raise ValueError("expected logits (B,H,T,T) x2, chain_mask (B,T,T), values (B,H,T,D) x2")
    if intra_values.dtype not in _DTYPES or any(t.dtype != intra_values.dtype for t in ts):
        raise TypeError("logits and values must all be float32 or all be bfloat16")
    m = chain_mask.contiguous().view(torch.uint8) if chain_mask.dtype == torch.bool else chain_mask.to(torch.uint8).contiguous()
    return _CombineFn.apply(intra_logits.contiguous(), inter_logits.contiguous(), m, intra_values.contiguous(),
                            inter_values.contiguous())


# ----------------------------------------------------------------------------------------------- projection GEMMs
_BIAS_DT = {torch.float32: L.F32, torch.bfloat16: L.BF16}


def _bias_arg(bias):
    if bias is None:
        return None, L.F32
    if bias.dtype not in _BIAS_DT:
        raise TypeError("bias must be float32 or bfloat16")
    return bias.contiguous(), _BIAS_DT[bias.dtype]


def gemm_bf16(x2d: torch.Tensor, w: torch.Tensor, bias=None, gelu: bool = False, save_preact: bool = False):
    """act(x2d @ w.T + bias) on the tcgen05 GEMM: x2d [M,K] bf16, w [N,K] bf16 -> [M,N] bf16 (no autograd).
    With gelu and save_preact the pre-activation is returned as well: (out, z)."""
    _require_cuda(x2d, w, bias)
    M, K = x2d.shape
    N = w.shape[0]
    b, bdt = _bias_arg(bias)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=x2d.device)
    z = torch.empty(M, N, dtype=torch.bfloat16, device=x2d.device) if (gelu and save_preact) else None
    with _on(x2d.device):
        rc = L.lib().mintb_linear_fwd(_ptr(x2d), _ptr(w), _ptr(b), _ptr(out), _ptr(z), M, N, K, L.BF16, bdt, L.BF16, int(gelu),
                                      1.0, 1.0, _stream(), _ptr(_dev_status(x2d.device)))
    L.check(rc, "mintb_linear_fwd")
    return (out, z) if save_preact else out


def quantize_e4m3(x: torch.Tensor, scale: float) -> torch.Tensor:
    """Per-tensor scaled cast bf16 -> e4m3: saturate(x / scale) (no autograd)."""
    _require_cuda(x)
    x = x.contiguous()
    out = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
    with _on(x.device):
        L.check(L.lib().mintb_quantize_e4m3(_ptr(x), _ptr(out), x.numel(), 1.0 / scale, _stream()), "mintb_quantize_e4m3")
    return out


def attach_e4m3(t: torch.Tensor, q8: torch.Tensor, scale: float) -> None:
    """Hand the e4m3 copy of `t` (cast with `scale`) to whoever receives `t` next: the copy rides on the tensor object itself.
    The pass that produced `t` (a fused residual + LayerNorm) wrote it for the e4m3 projections that read `t` next."""
    t._mintb_e4m3 = (q8, float(scale), t._version)


def e4m3_of(t: torch.Tensor, scale: float) -> torch.Tensor:
    """The e4m3 operand of a projection that reads the (rows, E) view of `t`: the copy attached by the pass that produced `t`
    when there is one with this scale and `t` has not been written since, else a cast pass."""
    hit = getattr(t, "_mintb_e4m3", None)
    if hit is not None and hit[1] == float(scale) and hit[2] == t._version and hit[0].numel() == t.numel():
        return hit[0].view(-1, t.shape[-1])
    return quantize_e4m3(t.reshape(-1, t.shape[-1]), scale)


def gemm_e4m3(xq: torch.Tensor, wq: torch.Tensor, alpha: float, bias=None, gelu: bool = False,
              out_e4m3_scale: Optional[float] = None, save_preact: bool = False):
    """act(alpha * xq @ wq.T + bias) with e4m3 operands; bf16 result, or e4m3 (result / out_e4m3_scale, saturated).
    With gelu and save_preact the bf16 pre-activation is returned as well: (out, z)."""
    _require_cuda(xq, wq, bias)
    M, K = xq.shape
    N = wq.shape[0]
    b, bdt = _bias_arg(bias)
    to_f8 = out_e4m3_scale is not None
    out = torch.empty(M, N, dtype=torch.float8_e4m3fn if to_f8 else torch.bfloat16, device=xq.device)
    z = torch.empty(M, N, dtype=torch.bfloat16, device=xq.device) if (gelu and save_preact) else None
    with _on(xq.device):
        rc = L.lib().mintb_linear_fwd(_ptr(xq), _ptr(wq), _ptr(b), _ptr(out), _ptr(z), M, N, K, L.E4M3, bdt,
                                      L.E4M3 if to_f8 else L.BF16, int(gelu), float(alpha),
                                      1.0 / out_e4m3_scale if to_f8 else 1.0, _stream(), _ptr(_dev_status(xq.device)))
    L.check(rc, "mintb_linear_fwd")
    return (out, z) if save_preact else out


def gemm_res(x_op: torch.Tensor, w_op: torch.Tensor, alpha: float, bias, resid: torch.Tensor, a: float, b: float,
             quant_scale: Optional[float] = None):
    """a * resid + b * (alpha * x_op @ w_op.T + bias) on the tcgen05 GEMM, the residual sum formed in its epilogue: operands
    bf16 or e4m3 (both alike), resid bf16 [M,N] -> bf16 [M,N].  With quant_scale the pass also leaves the e4m3 copy
    saturate(result / quant_scale) for the projection that reads the sum next: returns (sum, copy), else (sum, None)."""
    _require_cuda(x_op, w_op, bias, resid)
    M, K = x_op.shape
    N = w_op.shape[0]
    bt, bdt = _bias_arg(bias)
    in_dt = L.E4M3 if x_op.dtype == torch.float8_e4m3fn else L.BF16
    out = torch.empty(M, N, dtype=torch.bfloat16, device=x_op.device)
    q8 = torch.empty(M, N, dtype=torch.float8_e4m3fn, device=x_op.device) if quant_scale else None
    resid = resid.contiguous()
    with _on(x_op.device):
        rc = L.lib().mintb_linear_res_fwd(_ptr(x_op), _ptr(w_op), _ptr(bt), _ptr(resid), float(a), float(b),
                                          _ptr(q8) if q8 is not None else _ptr(out), _ptr(out) if q8 is not None else None, M, N, K,
                                          in_dt, bdt, L.E4M3 if q8 is not None else L.BF16, float(alpha),
                                          1.0 / quant_scale if quant_scale else 1.0, _stream(), _ptr(_dev_status(x_op.device)))
    L.check(rc, "mintb_linear_res_fwd")
    return out, q8


_GEMM_DT = {torch.bfloat16: L.BF16, torch.float8_e4m3fn: L.E4M3, torch.float8_e5m2: L.E5M2}


def gemm_dgrad(dz: torch.Tensor, w: torch.Tensor, dz2: Optional[torch.Tensor] = None, w2: Optional[torch.Tensor] = None,
               alpha: float = 1.0) -> torch.Tensor:
    """dx = alpha (dz @ w + dz2 @ w2) on the tcgen05 GEMM: dz [M,N], w [N,K] (the nn.Linear weight as stored) -> bf16 [M,K].
    Operands are all bf16, or all 8-bit floats (e5m2 gradients, e4m3 weights; alpha then carries the scales).  The optional
    second pair adds another projection's input gradient in the same accumulator (no autograd)."""
    _require_cuda(dz, w, dz2, w2)
    M, N = dz.shape
    K = w.shape[1]
    if w.shape[0] != N or (dz2 is None) != (w2 is None):
        raise ValueError("gemm_dgrad: dz [M,N] needs w [N,K]; dz2 and w2 come together")
    N2 = 0 if dz2 is None else dz2.shape[1]
    if dz2 is not None and (dz2.shape[0] != M or tuple(w2.shape) != (N2, K) or dz2.dtype != dz.dtype or w2.dtype != w.dtype):
        raise ValueError("gemm_dgrad: the second operand pair must match the first in rows, K and dtypes")
    if dz.dtype not in _GEMM_DT or w.dtype not in _GEMM_DT:
        raise TypeError("gemm_dgrad takes bfloat16 or float8 operands")
    dz, w = dz.contiguous(), w.contiguous()
    dz2, w2 = (None, None) if dz2 is None else (dz2.contiguous(), w2.contiguous())
    dx = torch.empty(M, K, dtype=torch.bfloat16, device=dz.device)
    with _on(dz.device):
        rc = L.lib().mintb_linear_dgrad(_ptr(dz), _ptr(w), _ptr(dz2), _ptr(w2), _ptr(dx), M, N, K, N2, _GEMM_DT[dz.dtype],
                                        _GEMM_DT[w.dtype], float(alpha), _stream(), _ptr(_dev_status(dz.device)))
    L.check(rc, "mintb_linear_dgrad")
    return dx


def gemm_wgrad(dz: torch.Tensor, x: torch.Tensor, alpha: float = 1.0, out_dtype=torch.bfloat16) -> torch.Tensor:
    """dw = alpha dz^T @ x on the tcgen05 GEMM: dz [M,N], x [M,K] -> [N,K] in bf16 or fp32 (fp32 accumulation over the M rows
    either way).  Operands are both bf16, or both 8-bit floats (no autograd)."""
    _require_cuda(dz, x)
    M, N = dz.shape
    if x.shape[0] != M:
        raise ValueError("gemm_wgrad: dz [M,N] and x [M,K] must have the same number of rows")
    K = x.shape[1]
    if dz.dtype not in _GEMM_DT or x.dtype not in _GEMM_DT:
        raise TypeError("gemm_wgrad takes bfloat16 or float8 operands")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise TypeError("gemm_wgrad writes bfloat16 or float32")
    dz, x = dz.contiguous(), x.contiguous()
    odt = L.F32 if out_dtype == torch.float32 else L.BF16
    dw = torch.empty(N, K, dtype=out_dtype, device=dz.device)
    lib = L.lib()
    wsb = lib.mintb_linear_wgrad_workspace_bytes(N, K, odt)
    ws = _workspace(wsb, dz.device)
    with _on(dz.device):
        rc = lib.mintb_linear_wgrad(_ptr(dz), _ptr(x), _ptr(dw), _ptr(ws), wsb, M, N, K, _GEMM_DT[dz.dtype], _GEMM_DT[x.dtype], odt,
                                    float(alpha), _stream(), _ptr(_dev_status(dz.device)))
    L.check(rc, "mintb_linear_wgrad")
    return dw


def gelu_bwd_colsum(dy: torch.Tensor, z: Optional[torch.Tensor], want_db: bool = True, want_act: bool = False):
    """(dz, db): dz = dy * gelu'(z) (bf16 [M,N]; dy itself when z is None) and db = column sums of dz (fp32 [N]) in one pass.
    With want_act the same pass also writes gelu(z) in bf16 and the result is (dz, db, act)."""
    _require_cuda(dy, z)
    dy = dy.contiguous()
    M, N = dy.shape
    dz = torch.empty_like(dy) if z is not None else dy
    db = torch.empty(N, dtype=torch.float32, device=dy.device) if want_db else None
    act = torch.empty_like(dy) if (want_act and z is not None) else None
    if z is None and not want_db:
        return (dz, None, None) if want_act else (dz, None)
    with _on(dy.device):
        rc = L.lib().mintb_gelu_bwd_colsum_act(_ptr(dy), _ptr(z), _ptr(dz) if z is not None else None, _ptr(act), _ptr(db), M, N,
                                               _stream())
    L.check(rc, "mintb_gelu_bwd_colsum")
    return (dz, db, act) if want_act else (dz, db)


E5M2_MAX = 57344.0
GRAD_HEADROOM = 16.0     # the largest gradient seen at calibration lands this far below the e5m2 maximum


class GradScale:
    """Static scale of the e5m2 cast of one projection's output gradient: g8 = saturate_e5m2(dz / scale)
    (mint_plus/models/alt/munit_scaling.py:41-45 states the cast with a fixed multiplier).  `scale` None means "not
    measured yet": the first backward pass that meets it measures amax(dz) once (one host read) and fixes
    scale = amax * GRAD_HEADROOM / 57344, so that gradients GRAD_HEADROOM times larger still fit and e5m2's 2^-30 range
    below that covers the small ones.  Set `scale` by hand, or back to None to measure again."""

    def __init__(self, scale: Optional[float] = None):
        self.scale = scale

    def fix(self, amax: float) -> float:
        self.scale = max(float(amax), 1e-30) * GRAD_HEADROOM / E5M2_MAX
        return self.scale


def grad_colsum_f8(dy: torch.Tensor, z: Optional[torch.Tensor], want_db: bool, scale: float, want_dz: bool = False):
    """(dz8, db, dz): dz = dy * gelu'(z) (dy itself without z) as e5m2 numbers dz8 = saturate(dz / scale) [M,N], the bias
    gradient db (fp32 [N], the column sums of the e5m2 numbers times scale) and, with want_dz, dz in bf16 — one pass."""
    _require_cuda(dy, z)
    dy = dy.contiguous()
    M, N = dy.shape
    dz8 = torch.empty(M, N, dtype=torch.float8_e5m2, device=dy.device)
    db = torch.empty(N, dtype=torch.float32, device=dy.device) if want_db else None
    dz = torch.empty_like(dy) if (want_dz and z is not None) else None
    with _on(dy.device):
        rc = L.lib().mintb_gelu_bwd_colsum_f8(_ptr(dy), _ptr(z), _ptr(dz), None, _ptr(db), _ptr(dz8), float(scale), M, N, _stream())
    L.check(rc, "mintb_gelu_bwd_colsum_f8")
    return dz8, db, (dz if z is not None else (dy if want_dz else None))


def f8_output_grad(dy: torch.Tensor, z: Optional[torch.Tensor], want_db: bool, holder: "GradScale"):
    """The e5m2 operand of a projection's 8-bit backward products from its upstream gradient: (dz8, db, scale).  Measures
    the holder's scale on first use."""
    if holder.scale is None:
        dz = gelu_bwd_colsum(dy, z, False)[0] if z is not None else dy
        holder.fix(float(dz.detach().abs().amax()))
    dz8, db, _ = grad_colsum_f8(dy, z, want_db, holder.scale)
    return dz8, db, holder.scale


def _gelu_erf_grad(z: torch.Tensor) -> torch.Tensor:
    zf = z.float()
    return 0.5 * (1.0 + torch.erf(zf * 0.7071067811865476)) + zf * torch.exp(-0.5 * zf * zf) * 0.3989422804014327


def linear_backward(dy, x2d, w, bias, z, needs, out_scale: float = 1.0, db=None, want_dx=True):
    """Gradients of y = act(out_scale * x W^T + b): the GELU derivative and the bias gradient come from one fused pass
    (or the bias gradient is handed in as `db` by the pass that produced dy); dgrad (dz W) and wgrad (dz^T x) run on the
    tcgen05 GEMMs of the library from the row-major matrices as they are, bf16 operands, with the static output multiplier
    as their alpha.  Returns (dx, dW, dbias, dz); `want_dx` False leaves dx to the caller (who adds several projections'
    input gradients in one product, `gemm_dgrad` with two operand pairs)."""
    want_db = bias is not None and needs[2]
    if db is not None:
        dz = dy
    else:
        dz, db = gelu_bwd_colsum(dy, z, want_db)
    dx = dw = None
    if needs[0] and want_dx:
        dx = gemm_dgrad(dz, _as_bf16(w), alpha=out_scale)
    if needs[1]:
        dw = gemm_wgrad(dz, x2d, alpha=out_scale, out_dtype=torch.float32 if w.dtype == torch.float32 else torch.bfloat16)
        if dw.dtype != w.dtype:
            dw = dw.to(w.dtype)
    return dx, dw, (db.to(bias.dtype) if want_db else None), dz


def _as_bf16(w: torch.Tensor) -> torch.Tensor:
    return (w if w.dtype == torch.bfloat16 else w.to(torch.bfloat16)).contiguous()


class _LinearFn(torch.autograd.Function):
    """y = act(x W^T + b) with the forward on the tcgen05 GEMM.  With GELU the pre-activation is written by the same GEMM
    epilogue and kept for the backward pass."""

    @staticmethod
    def forward(ctx, x2d, w, bias, gelu):
        wb = (w if w.dtype == torch.bfloat16 else w.to(torch.bfloat16)).contiguous()
        keep = gelu and any(ctx.needs_input_grad[:3])
        res = gemm_bf16(x2d, wb, bias, gelu, save_preact=keep)
        out, z = res if keep else (res, None)
        ctx.save_for_backward(x2d, w, bias, z)
        return out

    @staticmethod
    def backward(ctx, dy):
        x2d, w, bias, z = ctx.saved_tensors
        dx, dw, db, _ = linear_backward(dy, x2d, w, bias, z, ctx.needs_input_grad)
        return dx, dw, db, None


class _LinearResFn(torch.autograd.Function):
    """s = a r + b (x W^T + bias) with the residual sum formed in the GEMM epilogue (bf16 operands); optionally also the e4m3
    copy of s for the projection that reads it next (second output, not differentiable)."""

    @staticmethod
    def forward(ctx, x2d, w, bias, resid2d, a, b, quant_scale):
        out, q8 = gemm_res(x2d, _as_bf16(w), 1.0, bias, resid2d, a, b, quant_scale)
        ctx.save_for_backward(x2d, w, bias)
        ctx.ab = (float(a), float(b))
        if q8 is not None:
            ctx.mark_non_differentiable(q8)
        return out, q8

    @staticmethod
    def backward(ctx, dy, _dq8=None):
        x2d, w, bias = ctx.saved_tensors
        a, b = ctx.ab
        n = ctx.needs_input_grad
        dy = dy.contiguous()
        dx, dw, db, _ = linear_backward(dy, x2d, w, bias, None, n, out_scale=b)
        if db is not None and b != 1.0:
            db = db * b
        d_res = (dy if a == 1.0 else dy * a) if n[3] else None
        return dx, dw, db, d_res, None, None, None


def linear_res(x: torch.Tensor, weight: torch.Tensor, bias, resid: torch.Tensor, a: float, b: float,
               quant_scale: Optional[float] = None) -> torch.Tensor:
    """a * resid + b * nn.Linear(x) for bf16 CUDA activations, one pass (the residual add rides in the GEMM epilogue);
    differentiable.  With quant_scale the e4m3 copy of the result is attached to it for the next e4m3 projection."""
    if x.dtype != torch.bfloat16 or resid.dtype != torch.bfloat16:
        raise TypeError("ops.linear_res takes bfloat16 activations")
    x2d = x.reshape(-1, x.shape[-1]).contiguous()
    out, q8 = _LinearResFn.apply(x2d, weight, bias, resid.reshape(-1, weight.shape[0]), float(a), float(b), quant_scale)
    out = out.view(*x.shape[:-1], weight.shape[0])
    if q8 is not None:
        attach_e4m3(out, q8, quant_scale)
    return out


class _LoraLinearFn(torch.autograd.Function):
    """y = x (W + s B A)^T + b on ONE product with the merged weight; the adapters get their gradients through thin
    products (dA = s (dy B)^T x, dB = s dy^T (x A^T)), the frozen W none unless it asks for one."""

    @staticmethod
    def forward(ctx, x2d, w, bias, lora_a, lora_b, scaling):
        with torch.no_grad():
            w_used = (w + scaling * (lora_b.to(w.dtype) @ lora_a.to(w.dtype))).to(torch.bfloat16).contiguous()
        out = gemm_bf16(x2d, w_used, bias, False)
        ctx.save_for_backward(x2d, w, bias, lora_a, lora_b)
        ctx.scaling = float(scaling)
        return out

    @staticmethod
    def backward(ctx, dy):
        x2d, w, bias, lora_a, lora_b = ctx.saved_tensors
        s, needs, dt = ctx.scaling, ctx.needs_input_grad, x2d.dtype
        dy = dy.contiguous()
        dx = dw = db = d_a = d_b = None
        if needs[0]:
            dx = gemm_dgrad(dy, _as_bf16(w + s * (lora_b.to(w.dtype) @ lora_a.to(w.dtype))))
        if needs[1]:
            dw = gemm_wgrad(dy, x2d).to(w.dtype)
        if bias is not None and needs[2]:
            db = gelu_bwd_colsum(dy, None, True)[1].to(bias.dtype)
        if needs[3]:
            d_a = (((dy @ lora_b.to(dt)).t() @ x2d) * s).to(lora_a.dtype)
        if needs[4]:
            d_b = ((dy.t() @ (x2d @ lora_a.to(dt).t())) * s).to(lora_b.dtype)
        return dx, dw, db, d_a, d_b, None


def lora_linear(x: torch.Tensor, weight: torch.Tensor, bias, lora_a: torch.Tensor, lora_b: torch.Tensor, scaling: float) -> torch.Tensor:
    """A Linear with LoRA adapters A (r, in), B (out, r) for bf16 CUDA activations: x (W + scaling B A)^T + b; differentiable."""
    if x.dtype != torch.bfloat16:
        raise TypeError("ops.lora_linear takes bfloat16 activations")
    x2d = x.reshape(-1, x.shape[-1]).contiguous()
    y = _LoraLinearFn.apply(x2d, weight, bias, lora_a, lora_b, float(scaling))
    return y.view(*x.shape[:-1], weight.shape[0])


def linear(x: torch.Tensor, weight: torch.Tensor, bias=None, gelu: bool = False) -> torch.Tensor:
    """nn.Linear forward (optionally followed by erf-GELU) for bf16 CUDA activations; differentiable."""
    if x.dtype != torch.bfloat16:
        raise TypeError("ops.linear takes bfloat16 activations")
    x2d = x.reshape(-1, x.shape[-1]).contiguous()
    y = _LinearFn.apply(x2d, weight, bias, gelu)
    return y.view(*x.shape[:-1], weight.shape[0])


# ----------------------------------------------------------------------------------------------- variable-length packing
class PackInfo:
    """Which rows of the (T*B) token grid hold a token: `rows64` / `rows32` list them (row = t * B + b) in increasing order.
    Token-wise work (projections, norms, FFN) then runs on those rows only; the attention keeps the padded (B,H,T,D) grid."""

    def __init__(self, padding_mask: torch.Tensor):
        B, T = padding_mask.shape
        keep = ~padding_mask.t().reshape(-1)               # (T, B) order, like the layer's activations
        self.rows64 = torch.nonzero(keep, as_tuple=False).squeeze(1)
        self.rows32 = self.rows64.to(torch.int32)
        self.T, self.B, self.n = T, B, int(self.rows64.numel())
        # the inverse: packed row of token t * B + b, -1 where the position holds no token
        self.inv32 = torch.full((T * B,), -1, dtype=torch.int32, device=padding_mask.device)
        self.inv32[self.rows64] = torch.arange(self.n, dtype=torch.int32, device=padding_mask.device)


# ----------------------------------------------------------------------------------------------- residual + LayerNorm
class _AddLayerNormFn(torch.autograd.Function):
    """(s, y) with s = a x + b r and y = LayerNorm(s) gamma + beta, in one pass over x and r; `need_s` False drops s,
    gamma None drops the normalisation (then only s).  Replaces the residual add + LayerNorm pairs of the layers."""

    @staticmethod
    def forward(ctx, x, r, a, b, gamma, beta, eps, need_s, quant_scale=None):
        E = x.shape[-1]
        x2 = x.reshape(-1, E).contiguous()
        r2 = r.reshape(-1, E).contiguous() if r is not None else None
        rows = x2.shape[0]
        norm = gamma is not None
        s = torch.empty_like(x2) if (need_s or not norm) else None
        y = torch.empty_like(x2) if norm else None
        stats = torch.empty(rows, 2, dtype=torch.float32, device=x.device) if norm else None
        pdt = _BIAS_DT[gamma.dtype] if norm else L.F32
        # the e4m3 copy of the main result for the e4m3 projection that consumes it next (same values as quantize_e4m3)
        q8 = torch.empty(rows, E, dtype=torch.float8_e4m3fn, device=x.device) if quant_scale else None
        with _on(x.device):
            rc = L.lib().mintb_add_layernorm_fwd_q(_ptr(x2), _ptr(r2), float(a), float(b), _ptr(gamma), _ptr(beta), pdt, _ptr(s), _ptr(y),
                                                   _ptr(stats), rows, E, float(eps), _ptr(q8),
                                                   1.0 / quant_scale if quant_scale else 1.0, _stream())
        L.check(rc, "mintb_add_layernorm_fwd")
        ctx.save_for_backward(x2, r2, gamma, stats)
        ctx.cfg = (float(a), float(b), x.shape, pdt, beta is not None)
        ctx.mark_non_differentiable(*([q8] if q8 is not None else []))
        return s.view(x.shape) if s is not None else None, y.view(x.shape) if y is not None else None, q8

    @staticmethod
    def backward(ctx, ds_in, dy, _dq8=None):
        x2, r2, gamma, stats = ctx.saved_tensors
        a, b, shape, pdt, has_beta = ctx.cfg
        rows, E = x2.shape
        norm = gamma is not None
        if not norm and ds_in is None:
            return (None,) * 9
        dy2 = dy.reshape(rows, E).contiguous() if (norm and dy is not None) else None
        if norm and dy2 is None:
            dy2 = torch.zeros_like(x2)
        ds2 = ds_in.reshape(rows, E).contiguous() if ds_in is not None else None
        dx = torch.empty_like(x2)
        dr = torch.empty_like(x2) if r2 is not None else None
        want_pg = norm and (ctx.needs_input_grad[4] or ctx.needs_input_grad[5])   # frozen norm parameters: no sums at all
        dgamma = torch.empty(E, dtype=torch.float32, device=x2.device) if want_pg else None
        dbeta = torch.empty(E, dtype=torch.float32, device=x2.device) if want_pg else None
        lib = L.lib()
        wsb = lib.mintb_add_layernorm_bwd_workspace_bytes(rows, E) if want_pg else 0
        ws = torch.empty(wsb, dtype=torch.uint8, device=x2.device) if wsb else None
        with _on(x2.device):
            rc = lib.mintb_add_layernorm_bwd(_ptr(dy2), _ptr(ds2), _ptr(x2), _ptr(r2), a, b, _ptr(gamma), pdt, _ptr(stats), _ptr(dx),
                                             _ptr(dr), _ptr(dgamma), _ptr(dbeta), _ptr(ws), wsb, rows, E, _stream())
        L.check(rc, "mintb_add_layernorm_bwd")
        return (dx.view(shape), dr.view(shape) if dr is not None else None, None, None,
                dgamma.to(gamma.dtype) if want_pg else None, dbeta.to(gamma.dtype) if (want_pg and has_beta) else None, None, None, None)


def add_layernorm(x, r, a: float, b: float, norm: Optional[torch.nn.LayerNorm], need_s: bool = True,
                  quant_scale: Optional[float] = None):
    """(s, y): s = a x + b r (r may be None), y = norm(s).  bf16 CUDA tensors; `norm` None returns (s, None).
    `quant_scale`: the activation scale of the e4m3 projection that reads the main result (y, or s without `norm`) next:
    the kernel then writes that projection's e4m3 operand in the same pass; the copy rides on the returned tensor
    (`attach_e4m3`) and the projection takes it from there (`e4m3_of`) instead of casting."""
    if x.dtype != torch.bfloat16 or not x.is_cuda:
        raise TypeError("add_layernorm takes bfloat16 CUDA tensors")
    if norm is None:
        s, y, q8 = _AddLayerNormFn.apply(x, r, a, b, None, None, 0.0, True, quant_scale)
    else:
        s, y, q8 = _AddLayerNormFn.apply(x, r, a, b, norm.weight, norm.bias, norm.eps, need_s, quant_scale)
    if q8 is not None:
        attach_e4m3(y if y is not None else s, q8, quant_scale)
    return s, y


def _rope_rotate_torch(t, cos, sin, inverse=False):
    """(B,H,T,D) rotation with (T, D/2) tables; inverse applies the transpose."""
    h = t.shape[-1] // 2
    lo, hi = t[..., :h].float(), t[..., h:].float()
    s = -sin if inverse else sin
    return torch.cat((lo * cos - hi * s, hi * cos + lo * s), dim=-1).to(t.dtype)


def _lora_merged(w, lora_a, lora_b, scaling):
    """W + s [B_q A_q; B_k A_k; B_v A_v] for a [3E, E] weight with adapters A (3, r, E), B (3, E, r); W itself without."""
    if lora_a is None:
        return w
    with torch.no_grad():
        delta = torch.bmm(lora_b.to(w.dtype), lora_a.to(w.dtype)).reshape(w.shape)
        return w + scaling * delta


def _lora_grads(g, x2d, lora_a, lora_b, scaling, E, wanted):
    """The adapters' gradients through thin products only (no E x E weight gradient): for each of q, k, v
    dB = s g^T (x A^T), dA = s (g B)^T x."""
    if lora_a is None or not wanted:
        return None, None
    # four launches for the three adapters together: x A^T for all of them in one product, the two per-adapter products
    # as batched ones on strided views of g (no copies of g), and (g B)^T x again as one product
    M_, r = g.shape[0], lora_a.shape[1]
    dt = x2d.dtype
    g3 = g.view(M_, 3, E)
    xa = (x2d @ lora_a.to(dt).reshape(3 * r, -1).t()).view(M_, 3, r)                 # [M, 3, r]
    d_b = torch.bmm(g3.permute(1, 2, 0), xa.permute(1, 0, 2))                         # (3, E, M) x (3, M, r) -> (3, E, r)
    gb = torch.bmm(g3.permute(1, 0, 2), lora_b.to(dt))                                # (3, M, E) x (3, E, r) -> (3, M, r)
    d_a = (gb.permute(1, 0, 2).reshape(M_, 3 * r).t() @ x2d).view(3, r, -1)            # (3r, M) x (M, E) -> (3, r, E)
    return (d_a * scaling).to(lora_a.dtype), (d_b * scaling).to(lora_b.dtype)


def _rowmajor_base(dq, dk, dv, T, B, H, D):
    """If dq, dk, dv are the (B,H,T,D) views of the three thirds of ONE contiguous [T*B][3E] matrix (what the attention
    backward pass hands back when it writes row-major), return that matrix, else None."""
    E = H * D
    want_stride = (3 * E, D, B * 3 * E, 1)
    ts = (dq, dk, dv)
    if any(t.dtype != torch.bfloat16 or tuple(t.shape) != (B, H, T, D) or tuple(t.stride()) != want_stride for t in ts):
        return None
    st = dq.untyped_storage()
    if any(t.untyped_storage().data_ptr() != st.data_ptr() for t in ts):
        return None
    o = dq.storage_offset()
    if dk.storage_offset() != o + E or dv.storage_offset() != o + 2 * E:
        return None
    return torch.as_strided(dq, (T * B, 3 * E), (3 * E, 1), o)


class _QkvFn(torch.autograd.Function):
    """Fused QKV projection of one pathway with head-major outputs (and RoPE on q, k when tables are given)."""

    @staticmethod
    def forward(ctx, x, w, bias, H, cos, sin, q_scale, wq=None, w_scale=1.0, x_scale=1.0, out_scale=1.0, gs=None, pack=None,
                lora_a=None, lora_b=None, lora_scaling=1.0):
        if pack is None:
            T, B, E = x.shape
            x2d = x.reshape(T * B, E).contiguous()
        else:                       # x holds the unpadded tokens only; pack.rows names the (t, b) position of each
            (T, B), E = (pack.T, pack.B), x.shape[-1]
            x2d = x.reshape(-1, E).contiguous()
        D = E // H
        b, bdt = _bias_arg(bias)
        if wq is None:      # bf16 operands
            w_used = _lora_merged(w, lora_a, lora_b, lora_scaling)
            a_op, b_op, in_dt, alpha = x2d, (w_used if w_used.dtype == torch.bfloat16 else w_used.to(torch.bfloat16)).contiguous(), L.BF16, 1.0
        else:               # e4m3 operands, one scale per tensor; the product of the scales is folded into alpha
            a_op, b_op, in_dt, alpha = e4m3_of(x, x_scale), wq, L.E4M3, float(x_scale) * float(w_scale) * float(out_scale)
        # packed: positions without a token are never written, and keys there are masked but still multiplied by a zero
        # probability, so they must hold finite numbers
        alloc = torch.zeros if pack is not None else torch.empty
        q, k, v = (alloc(B, H, T, D, dtype=torch.bfloat16, device=x.device) for _ in range(3))
        with _on(x.device):
            rc = L.lib().mintb_qkv_fwd(_ptr(a_op), _ptr(b_op), _ptr(b), _ptr(q), _ptr(k), _ptr(v), T, B, H, D, in_dt, bdt,
                                       float(alpha), float(q_scale), _ptr(cos), _ptr(sin),
                                       _ptr(pack.rows32) if pack is not None else None, x2d.shape[0], _stream(),
                                       _ptr(_dev_status(x.device)))
        L.check(rc, "mintb_qkv_fwd")
        ctx.save_for_backward(x2d, w, bias, cos, sin, lora_a, lora_b)
        # 8-bit backward products (e5m2 gradient against these e4m3 operands): (xq, wq, weight scale, activation scale, GradScale)
        ctx.f8 = (a_op, b_op, float(w_scale), float(x_scale), gs) if (wq is not None and gs is not None) else None
        ctx.lora_scaling = float(lora_scaling)
        ctx.pack = pack
        ctx.x_shape = tuple(x.shape)
        ctx.dims = (T, B, H, D, q_scale, float(out_scale))
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        x2d, w, bias, cos, sin, lora_a, lora_b = ctx.saved_tensors
        T, B, H, D, q_scale, out_scale = ctx.dims
        E = H * D
        pack = ctx.pack
        n_rows = x2d.shape[0]
        want_db = bias is not None and ctx.needs_input_grad[2]
        g = _rowmajor_base(dq, dk, dv, T, B, H, D) if (pack is None and q_scale == 1.0) else None
        db = None
        if g is None:
            # (B,H,T,D) x3 -> [rows, 3E] with the rotation undone and the q scale applied, in one pass
            g = torch.empty(n_rows, 3 * E, dtype=torch.bfloat16, device=x2d.device)
            db = torch.empty(3 * E, dtype=torch.float32, device=x2d.device) if want_db else None
            with _on(x2d.device):
                rc = L.lib().mintb_qkv_grad_pack(_ptr(dq.contiguous()), _ptr(dk.contiguous()), _ptr(dv.contiguous()), _ptr(g), _ptr(db),
                                                 _ptr(cos), _ptr(sin), _ptr(pack.rows32) if pack is not None else None, n_rows,
                                                 T, B, H, D, float(q_scale), _stream())
            L.check(rc, "mintb_qkv_grad_pack")
        # else: the attention backward pass has already written [dQ | dK | dV] row-major (and un-rotated): no gather pass
        dx, dw, db, d_a, d_b, _ = _qkv_backward_from_g(ctx, g, db)
        return (dx, dw, db, None, None, None, None, None, None, None, None, None, None, d_a, d_b, None)


def _qkv_backward_from_g(ctx, g, db=None, want_dx=True, f8_scale=None):
    """Gradients of one fused QKV projection (context `ctx` of `_QkvFn.forward`) from the row-major gradient matrix
    g = [dQ | dK | dV] of its output: (dx shaped like the input or None, dW, dbias, dA, dB of the LoRA adapters, and the
    (gradient operand, weight operand, multiplier) its dgrad product takes).  A projection that ran on e4m3 operands with
    8-bit gradients enabled casts g to e5m2 (scale `f8_scale`, else its own GradScale) and runs both products in 8 bits."""
    x2d, w, bias, _, _, lora_a, lora_b = ctx.saved_tensors
    T, B, H, D, q_scale, out_scale = ctx.dims
    needs = ctx.needs_input_grad
    if getattr(ctx, "f8", None) is not None:
        xq, wq, w_scale, x_scale, gs = ctx.f8
        want_db = bias is not None and needs[2] and db is None
        if f8_scale is None:
            g8, db8, f8_scale = f8_output_grad(g, None, want_db, gs)
        else:
            g8, db8, _ = grad_colsum_f8(g, None, want_db, f8_scale)
        if want_db:
            db = db8
        dx = dw = None
        if needs[0] and want_dx:
            dx = gemm_dgrad(g8, wq, alpha=f8_scale * w_scale * out_scale).view(ctx.x_shape)
        if needs[1]:
            dw = gemm_wgrad(g8, xq, alpha=f8_scale * x_scale * out_scale,
                            out_dtype=torch.float32 if w.dtype == torch.float32 else torch.bfloat16)
            if dw.dtype != w.dtype:
                dw = dw.to(w.dtype)
        db_out = db.to(bias.dtype) if (bias is not None and needs[2] and db is not None) else None
        return dx, dw, db_out, None, None, (g8, wq, f8_scale * w_scale * out_scale)
    w_used = _lora_merged(w, lora_a, lora_b, ctx.lora_scaling)
    dx, dw, db, _ = linear_backward(g, x2d, w_used, bias, None, needs, out_scale, db=db, want_dx=want_dx)
    d_a, d_b = _lora_grads(g, x2d, lora_a, lora_b, ctx.lora_scaling, H * D, needs[13] or needs[14])
    return (dx.view(ctx.x_shape) if dx is not None else None), dw, db, d_a, d_b, (g, _as_bf16(w_used), out_scale)


class _SubCtx:
    """Stand-in for an autograd context when one Function runs the forward and backward code of another as plain calls."""

    def __init__(self, needs_input_grad):
        self.needs_input_grad = tuple(needs_input_grad)
        self.saved_tensors = ()

    def save_for_backward(self, *tensors):
        self.saved_tensors = tensors


def _qkv2_forward(cs, cc, x, w_s, b_s, w_c, b_c, H, cos, sin, q_scale, fp8_s, fp8_c, pack, w6, b6):
    """Both pathways' fused QKV projections as ONE product on the [6E][E] operand `w6` (rows [Q;K;V] of the self pathway, then
    of the cross pathway): x is read once, the epilogue writes the six head-major tensors and rotates q, k of the self pathway.
    Fills the two sub-contexts exactly as two `_QkvFn.forward` calls would."""
    if pack is None:
        T, B, E = x.shape
        x2d = x.reshape(T * B, E).contiguous()
    else:
        (T, B), E = (pack.T, pack.B), x.shape[-1]
        x2d = x.reshape(-1, E).contiguous()
    D = E // H
    b6t, bdt = _bias_arg(b6)
    wq_s, ws_s, xs_s, os_s, gs_s = fp8_s
    wq_c, ws_c, xs_c, os_c, gs_c = fp8_c
    if wq_s is None:
        a_op, in_dt, al1, al2 = x2d, L.BF16, 1.0, 1.0
    else:
        a_op, in_dt = e4m3_of(x, xs_s), L.E4M3
        al1, al2 = float(xs_s) * float(ws_s) * float(os_s), float(xs_c) * float(ws_c) * float(os_c)
    alloc = torch.zeros if pack is not None else torch.empty     # packed: positions without a token must hold finite numbers
    outs = [alloc(B, H, T, D, dtype=torch.bfloat16, device=x.device) for _ in range(6)]
    with _on(x.device):
        rc = L.lib().mintb_qkv2_fwd(_ptr(a_op), _ptr(w6), _ptr(b6t), *[_ptr(t) for t in outs], T, B, H, D, in_dt, bdt, al1, al2,
                                    float(q_scale), _ptr(cos), _ptr(sin), _ptr(pack.rows32) if pack is not None else None,
                                    x2d.shape[0], _stream(), _ptr(_dev_status(x.device)))
    L.check(rc, "mintb_qkv2_fwd")
    for c, w, b, tabs, wq, ws, xs, os_, gs in ((cs, w_s, b_s, (cos, sin), wq_s, ws_s, xs_s, os_s, gs_s),
                                                (cc, w_c, b_c, (None, None), wq_c, ws_c, xs_c, os_c, gs_c)):
        c.save_for_backward(x2d, w, b, tabs[0], tabs[1], None, None)
        c.f8 = (a_op, wq, float(ws), float(xs), gs) if (wq is not None and gs is not None) else None
        c.lora_scaling, c.pack, c.x_shape = 1.0, pack, tuple(x.shape)
        c.dims = (T, B, H, D, q_scale, float(os_))
    return outs


class _QkvAttentionFn(torch.autograd.Function):
    """Both fused QKV projections of a layer and its two-pathway attention as ONE differentiable step: x -> attention output.

    Between the three products nothing but the kernels' own layouts exists: q, k, v head-major from the GEMM epilogues, and
    on the way back the attention kernels write [dQ | dK | dV] of each pathway row-major (only the unpadded tokens' rows when
    packed), which the dgrad / wgrad products read as they are; the second pathway's input gradient is accumulated into the
    first's by its own product."""

    @staticmethod
    def forward(ctx, x, w_s, b_s, la_s, lb_s, w_c, b_c, la_c, lb_c, H, cos, sin, q_scale, fp8_s, fp8_c, ls_s, ls_c, pack,
                meta, scale, flags, fused6=None):
        n = ctx.needs_input_grad
        f = (False,) * 10
        cs = _SubCtx((n[0], n[1], n[2]) + f + (n[3], n[4], False))
        cc = _SubCtx((n[0], n[5], n[6]) + f + (n[7], n[8], False))
        ca = _SubCtx((any(n[:9]),) * 6 + (False,) * 6)
        one_product = (fused6 is not None and la_s is None and la_c is None and (fp8_s[0] is None) == (fp8_c[0] is None)
                       and (fp8_s[0] is None or fp8_s[2] == fp8_c[2]) and (b_s is None) == (b_c is None))
        if one_product:
            q_s, k_s, v_s, q_c, k_c, v_c = _qkv2_forward(cs, cc, x, w_s, b_s, w_c, b_c, H, cos, sin, q_scale, fp8_s, fp8_c, pack, *fused6)
        else:
            q_s, k_s, v_s = _QkvFn.forward(cs, x, w_s, b_s, H, cos, sin, q_scale, *fp8_s, pack, la_s, lb_s, ls_s)
            q_c, k_c, v_c = _QkvFn.forward(cc, x, w_c, b_c, H, None, None, q_scale, *fp8_c, pack, la_c, lb_c, ls_c)
        out = _MultimerAttentionFn.forward(ca, q_s, k_s, v_s, q_c, k_c, v_c, meta, None, None, scale, flags, (cos, sin))
        ctx.subs = (cs, cc, ca)
        ctx.counts = tuple(len(c.saved_tensors) for c in ctx.subs)
        ctx.save_for_backward(*cs.saved_tensors, *cc.saved_tensors, *ca.saved_tensors)
        for c in ctx.subs:
            c.saved_tensors = ()
        ctx.pack = pack
        return out

    @staticmethod
    def backward(ctx, d_out):
        cs, cc, ca = ctx.subs
        saved, off = ctx.saved_tensors, 0
        for c, k in zip(ctx.subs, ctx.counts):
            c.saved_tensors = saved[off:off + k]
            off += k
        _, g_s, g_c = _attention_backward(ca, d_out, ctx.pack)
        scale_c = None
        if getattr(cs, "f8", None) is not None and getattr(cc, "f8", None) is not None:
            # 8-bit products for both pathways.  Their input gradients share ONE accumulator, hence one multiplier: the cross
            # pathway's e5m2 cast takes the scale that makes its multiplier equal the self pathway's.
            (_, _, ws_s, _, gs_s), (_, _, ws_c, _, _) = cs.f8, cc.f8
            ratio = (ws_s * cs.dims[5]) / (ws_c * cc.dims[5])
            if gs_s.scale is None:
                gs_s.fix(max(float(g_s.abs().amax()), float(g_c.abs().amax()) / ratio))
            scale_c = gs_s.scale * ratio
        _, dw_s, db_s, da_s, dlb_s, (ga_s, wb_s, al_s) = _qkv_backward_from_g(cs, g_s, want_dx=False)
        _, dw_c, db_c, da_c, dlb_c, (ga_c, wb_c, al_c) = _qkv_backward_from_g(cc, g_c, want_dx=False, f8_scale=scale_c)
        dx = None
        if ctx.needs_input_grad[0]:
            # both projections read the same x: their input gradients are ONE product over the concatenated reduction
            if ga_s.dtype == ga_c.dtype and abs(al_s - al_c) <= 1e-6 * abs(al_s):
                dx = gemm_dgrad(ga_s, wb_s, ga_c, wb_c, alpha=al_s)
            else:
                dx = gemm_dgrad(ga_s, wb_s, alpha=al_s) + gemm_dgrad(ga_c, wb_c, alpha=al_c)
            dx = dx.view(cs.x_shape)
        for c in ctx.subs:
            c.saved_tensors = ()
        return (dx, dw_s, db_s, da_s, dlb_s, dw_c, db_c, da_c, dlb_c) + (None,) * 13


def qkv_attention(x: torch.Tensor, proj_self, proj_cross, num_heads: int, meta: "MaskMeta", rope=None, scale: float = 1.0,
                  sqrt_softmax: bool = False, pack=None, skip_pad_queries: bool = False, fused6=None) -> torch.Tensor:
    """Attention output (T,B,H,D) of a layer from its input x (T,B,E) (or the packed rows of one, with `pack`): both fused
    QKV projections (`qkv_project`'s arithmetic; `proj_*` = (weight (3E,E), bias, fp8 operands or None, lora or None)) and
    `multimer_attention` on their head-major results, differentiable as one step (attention.py:87-117,188-323 and
    modules.py:94-154 of the reference).  `rope` = (cos, sin) rotates q, k of the self pathway in the GEMM epilogue;
    `scale` multiplies the logits of both pathways inside the attention kernels.  Head sizes 16, 32, 64.
    `fused6` = (the [6E][E] operand holding both pathways' weights — bf16, or e4m3 when the projections are FP8 — and the
    [6E] bias): both projections then run as ONE product that reads x once."""
    if x.dtype != torch.bfloat16 or not x.is_cuda or (pack is None and x.dim() != 3):
        raise TypeError("qkv_attention takes a (T, B, E) bfloat16 CUDA tensor (or the packed rows of one, with `pack`)")
    cos, sin = rope if rope is not None else (None, None)

    def unpack(proj):
        w, b, fp8, lora = proj
        la, lb, ls = lora if lora is not None else (None, None, 1.0)
        return w, b, la, lb, (tuple(fp8) + (None,) * (5 - len(fp8)) if fp8 is not None else (None, 1.0, 1.0, 1.0, None)), ls

    w_s, b_s, la_s, lb_s, f_s, ls_s = unpack(proj_self)
    w_c, b_c, la_c, lb_c, f_c, ls_c = unpack(proj_cross)
    flags = (L.FLAG_OUT_SEQ_FIRST | (L.FLAG_SQRT_SOFTMAX if sqrt_softmax else 0)
             | (L.FLAG_SKIP_PAD_QUERIES if skip_pad_queries else 0))
    return _QkvAttentionFn.apply(x, w_s, b_s, la_s, lb_s, w_c, b_c, la_c, lb_c, num_heads, cos, sin, 1.0, f_s, f_c, ls_s, ls_c,
                                 pack, meta, float(scale), int(flags), fused6)


def qkv_project(x: torch.Tensor, weight: torch.Tensor, bias, num_heads: int, rope: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                q_scale: float = 1.0, fp8: Optional[Tuple[torch.Tensor, float, float, float]] = None, pack=None,
                lora: Optional[Tuple[torch.Tensor, torch.Tensor, float]] = None):
    """x (T,B,E) bf16, weight (3E,E) with rows [Q;K;V] -> q, k, v (B,H,T,D) bf16, written head-major by the GEMM epilogue
    (attention.py:97-117, 304-323 of the reference without the three permute copies).  `rope` = (cos, sin) tables rotates q, k.
    `lora` = (A (3,r,E), B (3,E,r), alpha / r) adds frozen-base LoRA adapters of q, k, v: the product runs on the merged
    weight, the adapters get their gradients through thin products.
    `fp8` = (e4m3 weight, weight scale, activation scale, static output multiplier[, GradScale]) runs the product on e4m3
    operands; `weight` stays the master copy that receives the gradient.  With a GradScale the backward products run in 8 bits
    as well (e5m2 gradient against the e4m3 operands), else in bf16 on the master weight."""
    if x.dtype != torch.bfloat16 or (pack is None and x.dim() != 3):
        raise TypeError("qkv_project takes a (T, B, E) bfloat16 tensor (or the packed rows of one, with `pack`)")
    cos, sin = rope if rope is not None else (None, None)
    wq, w_scale, x_scale, out_scale, gs = (tuple(fp8) + (None,) * (5 - len(fp8))) if fp8 is not None else (None, 1.0, 1.0, 1.0, None)
    la, lb, ls = lora if lora is not None else (None, None, 1.0)
    return _QkvFn.apply(x, weight, bias, num_heads, cos, sin, q_scale, wq, w_scale, x_scale, out_scale, gs, pack, la, lb, ls)


# ----------------------------------------------------------------------------------------------- model prologue / epilogue
class _EmbedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, weight, pad_idx, mask_idx, token_dropout, mask_ratio_train):
        B, T = tokens.shape
        V, E = weight.shape
        out = torch.empty(T, B, E, dtype=weight.dtype, device=weight.device)
        scales = torch.empty(B, dtype=torch.float32, device=weight.device)
        w = weight.contiguous()
        with _on(weight.device):
            rc = L.lib().mintb_embed_fwd(_ptr(tokens), _ptr(w), _ptr(out), _ptr(scales), B, T, E, V, _DTYPES[weight.dtype], int(pad_idx),
                                         int(mask_idx), int(bool(token_dropout)), float(mask_ratio_train), _stream())
        L.check(rc, "mintb_embed_fwd")
        ctx.save_for_backward(tokens, scales)
        ctx.cfg = (V, E, weight.dtype, int(pad_idx), int(mask_idx), int(bool(token_dropout)))
        return out

    @staticmethod
    def backward(ctx, d_out):
        tokens, scales = ctx.saved_tensors
        V, E, dt, pad_idx, mask_idx, td = ctx.cfg
        B, T = tokens.shape
        d_out = d_out.contiguous()
        dw = torch.empty(V, E, dtype=torch.float32, device=d_out.device)
        with _on(d_out.device):
            rc = L.lib().mintb_embed_bwd(_ptr(tokens), _ptr(d_out), _ptr(scales), _ptr(dw), B, T, E, V, _DTYPES[dt], pad_idx, mask_idx, td,
                                         _stream())
        L.check(rc, "mintb_embed_bwd")
        return None, dw.to(dt), None, None, None, None


def embed_tokens(tokens: torch.Tensor, weight: torch.Tensor, pad_idx: int, mask_idx: int, token_dropout: bool,
                 mask_ratio_train: float = 0.12) -> torch.Tensor:
    """The model's prologue in one pass (esm2.py:91-104 of the reference): x = W[tokens]; under token dropout <mask> rows are
    zeroed and every row of sample b is multiplied by (1 - mask_ratio_train) / (1 - masked_b / unpadded_b); <pad> rows are
    zeroed; the result is written sequence-first, (T, B, E), the layout of the layer stack.  tokens (B, T) int64 on the
    device; weight (V, E) fp32 or bf16; differentiable with respect to the weight."""
    _require_cuda(tokens, weight)
    if tokens.dtype != torch.int64 or tokens.dim() != 2 or weight.dtype not in _DTYPES:
        raise TypeError("embed_tokens takes int64 tokens (B, T) and an fp32 or bf16 weight (V, E)")
    return _EmbedFn.apply(tokens.contiguous(), weight, pad_idx, mask_idx, token_dropout, mask_ratio_train)


class _MaskedCeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rows, targets, mask_u8, V):
        N, ld = rows.shape[0], rows.stride(0)
        lse = torch.empty(N, dtype=torch.float32, device=rows.device)
        sums = torch.empty(2, dtype=torch.float32, device=rows.device)
        with _on(rows.device):
            rc = L.lib().mintb_masked_ce_fwd(_ptr(rows), _ptr(targets), _ptr(mask_u8), _ptr(lse), _ptr(sums), N, ld, V, _stream())
        L.check(rc, "mintb_masked_ce_fwd")
        ctx.save_for_backward(rows, targets, mask_u8, lse, sums)
        ctx.V = V
        return sums[0] / sums[1]

    @staticmethod
    def backward(ctx, g):
        rows, targets, mask_u8, lse, sums = ctx.saved_tensors
        N, ld = rows.shape[0], rows.stride(0)
        d_pad = torch.empty(N, ld, dtype=torch.bfloat16, device=rows.device)
        g32 = g.detach().to(torch.float32).reshape(1).contiguous()
        with _on(rows.device):
            rc = L.lib().mintb_masked_ce_bwd(_ptr(rows), _ptr(targets), _ptr(mask_u8), _ptr(lse), _ptr(sums), _ptr(g32), _ptr(d_pad), N, ld,
                                             ctx.V, _stream())
        L.check(rc, "mintb_masked_ce_bwd")
        return d_pad[:, :rows.shape[1]], None, None, None


def masked_cross_entropy(logits: torch.Tensor, targets: torch.Tensor, target_mask: torch.Tensor) -> torch.Tensor:
    """mean over the target positions of cross_entropy(logits, targets) (training/wrapper.py:77-80 of the reference) in one
    pass over the logits, fp32 arithmetic: logits (B, T, V) bf16 on the device — a (T, B)-ordered or (B, T)-ordered view of
    rows with 16-byte aligned stride is read in place — targets (B, T) int64, target_mask (B, T) bool.  Differentiable with
    respect to the logits."""
    _require_cuda(logits, targets, target_mask)
    if logits.dtype != torch.bfloat16 or logits.dim() != 3 or logits.stride(-1) != 1:
        raise TypeError("masked_cross_entropy takes bfloat16 logits (B, T, V) with a contiguous last dimension")
    B, T, V = logits.shape
    if logits.stride(0) == T * logits.stride(1):                         # rows in (B, T) order
        rows = torch.as_strided(logits, (B * T, V), (logits.stride(1), 1), logits.storage_offset())
        tg, mk = targets, target_mask
    elif logits.stride(1) == B * logits.stride(0):                       # rows in (T, B) order: a transposed view
        rows = torch.as_strided(logits, (T * B, V), (logits.stride(0), 1), logits.storage_offset())
        tg, mk = targets.t(), target_mask.t()
    else:
        c = logits.contiguous()
        rows, tg, mk = c.view(B * T, V), targets, target_mask
    return _MaskedCeFn.apply(rows, tg.contiguous().view(-1), mk.contiguous().view(-1).to(torch.uint8), V)
