"""TransformerLayer_MINT_plus / build_mint_plus / enable_fused_multi_pathway with the reference's interface
(mint_plus/models/modules_plus.py:20-305, mint_plus/models/modules.py:323-335, 398-417).

The layer always takes the fused CUDA attention — in training as well as in eval, since the fused
operator is differentiable — and passes the key-padding mask to it.  `_use_fused_multi_pathway` is kept
as an attribute for code that toggles it; False selects the materialised-logits combine kernel.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from . import ops
from .attention import MultiHeadAttention, MultimerAttention
from .kernels import fused_multimer_combine


def _linear(mod, x, gelu=False):
    """A projection module applied to a bf16 CUDA tensor: Fp8Linear on the e4m3 GEMM, nn.Linear on the bf16 GEMM."""
    from .mu_scaling import Fp8Linear
    if isinstance(mod, Fp8Linear):
        return mod(x, gelu=gelu)
    if type(mod) is not nn.Linear:          # a wrapped projection (e.g. LoRA adapters): its own forward decides
        y = mod(x)
        return gelu_erf(y) if gelu else y
    return ops.linear(x, mod.weight, mod.bias, gelu=gelu)


import os as _os
# the two whole-layer fusions (module-level switches; both on by default)
FUSE_QKV6 = _os.environ.get("MINTB_FUSE_QKV6", "1") != "0"              # both pathways' QKV projections as one product
_QKV6_MAX_BYTES = 40 << 20
FUSE_OUT_RESIDUAL = _os.environ.get("MINTB_FUSE_OUT_RESIDUAL", "1") != "0"   # residual sum in the output projection's epilogue


def _linear_res(mod, x, resid, a, b, quant_scale=None):
    """a * resid + b * mod(x) for bf16 CUDA tensors: in the projection's GEMM epilogue for nn.Linear / Fp8Linear, as a
    separate fused pass for wrapped projections (e.g. LoRA adapters)."""
    from .mu_scaling import Fp8Linear
    if isinstance(mod, Fp8Linear):
        return mod.forward_res(x, resid, a, b, quant_scale)
    if type(mod) is nn.Linear:
        return ops.linear_res(x, mod.weight, mod.bias, resid, a, b, quant_scale)
    s, _ = ops.add_layernorm(resid, mod(x), a, b, None, quant_scale=quant_scale)
    return s


def gelu_erf(x):
    return x * 0.5 * (1.0 + torch.erf(x / math.sqrt(2.0)))


class VanillaFeedForward(nn.Module):
    def __init__(self, embed_dim, ffn_embed_dim, use_erf_gelu: bool = False):
        super().__init__()
        self.fc1 = nn.Linear(embed_dim, ffn_embed_dim)
        self.fc2 = nn.Linear(ffn_embed_dim, embed_dim)
        self.use_erf_gelu = use_erf_gelu

    def forward(self, x):
        # bf16 on the GPU: both projections run on the tcgen05 GEMM, bias and erf-GELU in its epilogue
        # (F.gelu's default is the exact erf form too, so both flags give the same function)
        if x.is_cuda and x.dtype == torch.bfloat16:
            from .mu_scaling import Fp8Linear, fp8_ffn
            if isinstance(self.fc1, Fp8Linear) and isinstance(self.fc2, Fp8Linear):
                return fp8_ffn(self.fc1, self.fc2, x)    # fc1 hands gelu(.) to fc2 as e4m3: no bf16 copy, no cast pass
            return _linear(self.fc2, _linear(self.fc1, x, gelu=True))
        x = gelu_erf(self.fc1(x)) if self.use_erf_gelu else F.gelu(self.fc1(x))
        return self.fc2(x)


def _qkv_operands(attn):
    """(weight [3E,E], bias, fp8 tuple or None, lora tuple or None) of one pathway's Q/K/V projections, whether the module
    holds one fused Linear or three separate ones (rows ordered [Q;K;V] either way), or None when the modules are of mixed kinds."""
    from .lora import LoRALinear
    from .mu_scaling import Fp8Linear, fused_fp8_weight
    fused = getattr(attn, "fused_qkv", None)
    mods = [fused] if fused is not None else [attn.q_proj, attn.k_proj, attn.v_proj]
    if len(mods) == 3 and all(isinstance(m, LoRALinear) and type(m.base) is nn.Linear and not isinstance(m.dropout, nn.Dropout)
                              for m in mods) and len({(m.r, m.scaling) for m in mods}) == 1:
        # frozen base + LoRA adapters on q, k, v: one fused product on the merged weight
        w = torch.cat([m.base.weight for m in mods], dim=0)
        b = torch.cat([m.base.bias for m in mods], dim=0) if mods[0].base.bias is not None else None
        lora = (torch.stack([m.lora_A for m in mods]), torch.stack([m.lora_B for m in mods]), mods[0].scaling)
        return w, b, None, lora
    if all(isinstance(m, Fp8Linear) for m in mods):
        kind = "fp8"
    elif all(type(m) is nn.Linear for m in mods):
        kind = "bf16"
    else:
        return None
    if len(mods) == 1:
        w, b = mods[0].weight, mods[0].bias
    else:
        w = torch.cat([m.weight for m in mods], dim=0)
        b = torch.cat([m.bias for m in mods], dim=0) if mods[0].bias is not None else None
    return w, b, (fused_fp8_weight(attn, mods) if kind == "fp8" else None), None


def _qkv_params(attn):
    fused = getattr(attn, "fused_qkv", None)
    mods = [fused] if fused is not None else [attn.q_proj, attn.k_proj, attn.v_proj]
    mods = [getattr(m, "base", m) for m in mods]
    return [p for m in mods for p in (m.weight, m.bias) if p is not None]


def _fused6_operands(layer, ops_s, ops_c):
    """The [6E][E] weight operand (bf16, or e4m3 for FP8 projections) and [6E] bias of BOTH pathways' QKV projections for
    the one-product QKV GEMM, cached on the layer until one of the underlying parameters changes; None when the two
    pathways cannot share a product (adapters, mixed kinds)."""
    (w_s, b_s, f8_s, lora_s), (w_c, b_c, f8_c, lora_c) = ops_s, ops_c
    if lora_s is not None or lora_c is not None or (f8_s is None) != (f8_c is None) or (b_s is None) != (b_c is None):
        return None
    if f8_s is not None and f8_s[2] != f8_c[2]:
        return None
    if 6 * w_s.shape[1] * w_s.shape[1] * (1 if f8_s is not None else 2) > _QKV6_MAX_BYTES:
        return None       # a [6E][E] operand this large pushes the activation rows out of L2 between column tiles (measured slower)
    key = tuple((p.data_ptr(), p._version) for p in _qkv_params(layer.self_attn) + _qkv_params(layer.multimer_attn)) + (f8_s is not None,)
    cached = getattr(layer, "_qkv6_cache", None)
    if cached is not None and cached[0] == key:
        return cached[1], cached[2]
    with torch.no_grad():
        if f8_s is not None:
            w6 = torch.cat([f8_s[0].view(torch.uint8), f8_c[0].view(torch.uint8)], dim=0).view(torch.float8_e4m3fn)
        else:
            w6 = torch.cat([w_s.detach().to(torch.bfloat16), w_c.detach().to(torch.bfloat16)], dim=0)
        b6 = torch.cat([b_s.detach().float(), b_c.detach().float()], dim=0) if b_s is not None else None
    layer._qkv6_cache = (key, w6, b6)
    return w6, b6


class _TwoPathwayLayer(nn.Module):
    """The attention half shared by the Pre-LN layers and the muS layer: both QKV projections, the fused two-pathway
    attention (or the materialised-logits combine when `_use_fused_multi_pathway` is False), the output projection."""

    _use_sqrt_softmax = False

    def _standard_attention(self, x, attn_mask, padding_mask):
        return self.self_attn(x=x, key_padding_mask=padding_mask, attn_mask=attn_mask)

    def _multimer_attention_plus(self, x, chain_mask, padding_mask, chain_ids=None, pack=None):
        if self._use_fused_multi_pathway:
            return self._multimer_attention_superfused(x, chain_mask, padding_mask, chain_ids, pack)
        if pack is not None:
            raise NotImplementedError("packed tokens need the fused attention (enable_fused_multi_pathway)")
        if self._use_sqrt_softmax:
            raise NotImplementedError("square-root softmax needs the fused attention (enable_fused_multi_pathway)")
        T, B, E = x.shape
        sa, ma = self.self_attn, self.multimer_attn
        if chain_mask is None:
            chain_mask = chain_ids.unsqueeze(-1) != chain_ids.unsqueeze(-2)
        intra_logits, intra_values = sa(x=x, key_padding_mask=padding_mask, before_softmax=True)
        inter_logits, inter_values = ma(x=x, key_padding_mask=padding_mask, before_softmax=True)
        attn_out = fused_multimer_combine(intra_logits.type_as(intra_values), inter_logits.type_as(inter_values),
                                          chain_mask, intra_values, inter_values)
        attn_out = attn_out.permute(2, 0, 1, 3).reshape(T, B, E)
        return sa.out_proj(attn_out), None

    def _multimer_attention_superfused(self, x, chain_mask, padding_mask, chain_ids=None, pack=None, residual=None, quant_scale=None):
        """x (T,B,E) -> (T,B,E): both QKV projections, fused two-pathway attention, output projection.  With `pack`
        (ops.PackInfo) x is (N,1,E), the N unpadded tokens only: the projections run on those rows, the attention on the
        padded grid with fully padded query tiles left out, and its result is gathered back to the N rows.
        `residual` = (r, a, b) (bf16 on the GPU only): the result is a r + b out_proj(attention), the sum formed in the output
        projection's GEMM epilogue; `quant_scale` then also attaches the e4m3 copy of that sum for the next e4m3 projection."""
        if pack is None:
            T, B, E = x.shape
        else:
            (T, B), E = (pack.T, pack.B), x.shape[-1]
        sa, ma = self.self_attn, self.multimer_attn
        if sa.head_dim not in (16, 32, 64):
            raise NotImplementedError(f"head size {sa.head_dim}: the CUDA attention kernels take head sizes 16, 32 and 64 "
                                      "(there is no eager fallback)")
        if chain_ids is not None and chain_mask is None:
            mask_kw = dict(meta=_cached_ids_meta(chain_ids, padding_mask))
        else:
            mask_kw = dict(chain_mask=chain_mask, key_padding_mask=padding_mask)
        rope = sa.rot_emb is not None
        sqrt_sm = bool(self._use_sqrt_softmax)
        ops_s = ops_c = None
        if x.is_cuda and x.dtype == torch.bfloat16:
            ops_s, ops_c = _qkv_operands(sa), _qkv_operands(ma)
        if ops_s is not None and ops_c is not None:
            # bf16 activations on the GPU: the QKV GEMMs (bf16 or e4m3 operands) write q, k, v head-major and rotate the self
            # pathway in their epilogue, so the attention kernel gets ready-made operands (no permute copies, no rotation pass)
            tabs = ops.rope_tables(T, sa.head_dim, x.device, sa.rot_emb.inv_freq)[:2] if rope else None
            # projections and attention as one differentiable step: on the way back the attention kernels write
            # [dQ | dK | dV] row-major (only the unpadded tokens' rows when packed) for the projections' products
            meta = mask_kw["meta"] if "meta" in mask_kw else ops.cached_mask_meta(chain_mask, padding_mask)
            attn_out = ops.qkv_attention(x, ops_s, ops_c, sa.num_heads, meta, rope=tabs, scale=sa.scaling,
                                         sqrt_softmax=sqrt_sm, pack=pack, skip_pad_queries=pack is not None,
                                         fused6=_fused6_operands(self, ops_s, ops_c) if FUSE_QKV6 else None)
        elif pack is not None:
            raise NotImplementedError("packed tokens need bfloat16 CUDA activations and nn.Linear / Fp8Linear projections")
        else:
            q_s, k_s, v_s = sa.project_qkv_4d(x)
            q_c, k_c, v_c = ma.project_qkv_4d(x)
            attn_out = ops.multimer_attention(q_s, k_s, v_s, q_c, k_c, v_c, rope=rope,
                                              inv_freq=sa.rot_emb.inv_freq if rope else None, scale=sa.scaling,
                                              sqrt_softmax=sqrt_sm, out_seq_first=True, **mask_kw)
        attn_out = attn_out.reshape(T, B, E)      # the kernels wrote (T,B,H,D): a view, no permute copy
        if pack is not None:
            attn_out = attn_out.view(T * B, E).index_select(0, pack.rows64).unsqueeze(1)
        if x.is_cuda and x.dtype == torch.bfloat16:
            if residual is not None:
                return _linear_res(sa.out_proj, attn_out, residual[0], residual[1], residual[2], quant_scale), None
            return _linear(sa.out_proj, attn_out), None
        if residual is not None:
            raise NotImplementedError("the residual epilogue needs bfloat16 CUDA activations")
        return sa.out_proj(attn_out), None

    # the PyTorch-named entry of the reference resolves to the same fused path
    def _multimer_attention(self, x, chain_mask, padding_mask):
        return self._multimer_attention_plus(x, chain_mask, padding_mask)


class _PreLnLayer(_TwoPathwayLayer):
    """x -> LN -> attention -> +residual -> LN -> FFN -> +residual (modules.py:179-195, modules_plus.py:72-96)."""

    def _init_common(self, embed_dim, ffn_embed_dim, attention_heads, use_rotary_embeddings, use_multimer, use_rmsnorm,
                     use_erf_gelu):
        self.embed_dim = embed_dim
        self.ffn_embed_dim = ffn_embed_dim
        self.attention_heads = attention_heads
        self.use_rotary_embeddings = use_rotary_embeddings
        self.use_multimer = use_multimer
        self.use_rmsnorm = use_rmsnorm
        self.use_erf_gelu = use_erf_gelu
        self._use_fused_multi_pathway = True
        self.feed_forward = VanillaFeedForward(embed_dim, ffn_embed_dim, use_erf_gelu=use_erf_gelu)
        norm = (lambda: nn.RMSNorm(embed_dim)) if use_rmsnorm else (lambda: nn.LayerNorm(embed_dim))
        self.self_attn_layer_norm = norm()
        self.final_layer_norm = norm()

    def forward(self, x, self_attn_mask=None, self_attn_padding_mask=None, chain_ids=None, pack=None):
        if x.is_cuda and x.dtype == torch.bfloat16 and isinstance(self.final_layer_norm, nn.LayerNorm):
            # bf16 on the GPU: each residual add is fused with the LayerNorm that follows it (one pass over the activations)
            _, h = ops.add_layernorm(x, None, 1.0, 0.0, self.self_attn_layer_norm, need_s=False)
            if self.use_multimer and self._use_fused_multi_pathway and FUSE_OUT_RESIDUAL:
                # x + out_proj(attention): the residual add rides in the output projection's GEMM epilogue
                x, attn = self._multimer_attention_superfused(h, self_attn_mask, self_attn_padding_mask, chain_ids, pack,
                                                              residual=(x, 1.0, 1.0))
                _, h = ops.add_layernorm(x, None, 1.0, 0.0, self.final_layer_norm, need_s=False)
                return x + self.feed_forward(h), attn
            if self.use_multimer:
                h, attn = self._multimer_attention_plus(h, self_attn_mask, self_attn_padding_mask, chain_ids, pack)
            else:
                h, attn = self._standard_attention(h, self_attn_mask, self_attn_padding_mask)
            x, h = ops.add_layernorm(x, h, 1.0, 1.0, self.final_layer_norm, need_s=True)
            return x + self.feed_forward(h), attn
        if pack is not None:
            raise NotImplementedError("packed tokens need bfloat16 CUDA activations")
        residual = x
        x = self.self_attn_layer_norm(x)
        if self.use_multimer:
            x, attn = self._multimer_attention_plus(x, self_attn_mask, self_attn_padding_mask, chain_ids)
        else:
            x, attn = self._standard_attention(x, self_attn_mask, self_attn_padding_mask)
        x = residual + x
        residual = x
        x = self.final_layer_norm(x)
        x = self.feed_forward(x)
        x = residual + x
        return x, attn


class TransformerLayer_MINT_plus(_PreLnLayer):
    """Pre-LN layer with one fused Linear(E, 3E) per pathway (modules_plus.py:20-64)."""

    def __init__(self, embed_dim, ffn_embed_dim, attention_heads, use_rotary_embeddings: bool = True,
                 use_multimer: bool = False, use_rmsnorm: bool = False, use_erf_gelu: bool = False):
        super().__init__()
        self.self_attn = MultiHeadAttention(embed_dim, attention_heads, use_rotary_embeddings=use_rotary_embeddings,
                                            use_fused_qkv=True)
        if use_multimer:
            self.multimer_attn = MultimerAttention(embed_dim, attention_heads)
        self._init_common(embed_dim, ffn_embed_dim, attention_heads, use_rotary_embeddings, use_multimer, use_rmsnorm,
                          use_erf_gelu)


_ids_meta_cache = []


def _cached_ids_meta(chain_ids, padding_mask):
    for ids, ver, pad, meta in _ids_meta_cache:
        if ids is chain_ids and ver == chain_ids._version and pad is padding_mask:
            return meta
    meta = ops.mask_meta_from_chain_ids(chain_ids, padding_mask)
    _ids_meta_cache.insert(0, (chain_ids, chain_ids._version, padding_mask, meta))
    del _ids_meta_cache[2:]
    return meta


def build_mint_plus(model: nn.Module) -> nn.Module:
    """Replace every layer of `model.layers` by a TransformerLayer_MINT_plus, concatenating the separate
    q/k/v projection weights of both pathways into fused [Q;K;V] matrices; out_proj, rotary buffer, FFN and
    norms are shared by reference (modules_plus.py:240-305)."""
    for i, old in enumerate(model.layers):
        new = TransformerLayer_MINT_plus(
            embed_dim=old.embed_dim, ffn_embed_dim=old.ffn_embed_dim, attention_heads=old.attention_heads,
            use_rotary_embeddings=old.use_rotary_embeddings, use_multimer=old.use_multimer,
            use_rmsnorm=getattr(old, "use_rmsnorm", False), use_erf_gelu=getattr(old, "use_erf_gelu", False))
        ref = old.self_attn.out_proj.weight if old.self_attn.out_proj is not None else next(old.parameters())
        new.to(device=ref.device, dtype=ref.dtype)

        def fuse(dst: nn.Linear, src):
            if getattr(src, "fused_qkv", None) is not None and getattr(src, "q_proj", None) is None:
                dst.weight.data.copy_(src.fused_qkv.weight.data)
                if src.fused_qkv.bias is not None:
                    dst.bias.data.copy_(src.fused_qkv.bias.data)
                return
            dst.weight.data.copy_(torch.cat([src.q_proj.weight, src.k_proj.weight, src.v_proj.weight], dim=0))
            if src.q_proj.bias is not None:
                dst.bias.data.copy_(torch.cat([src.q_proj.bias, src.k_proj.bias, src.v_proj.bias], dim=0))

        fuse(new.self_attn.fused_qkv, old.self_attn)
        new.self_attn.out_proj = old.self_attn.out_proj
        new.self_attn.rot_emb = old.self_attn.rot_emb
        if hasattr(old, "multimer_attn") and old.multimer_attn is not None and new.use_multimer:
            fuse(new.multimer_attn.fused_qkv, old.multimer_attn)
        new.feed_forward = old.feed_forward
        new.self_attn_layer_norm = old.self_attn_layer_norm
        new.final_layer_norm = old.final_layer_norm
        new.train(old.training)
        model.layers[i] = new
    return model


def enable_fused_multi_pathway(model: nn.Module, enabled: bool = True):
    """Toggle the fused (no materialised logits) attention on every layer, including layers wrapped in blocks
    that expose `.layers` (modules.py:398-417)."""
    for layer in model.layers:
        for sub in (layer.layers if hasattr(layer, "layers") else [layer]):
            sub._use_fused_multi_pathway = enabled
