"""MINT model with the reference's constructor, forward signature, outputs and state-dict keys
(mint_plus/models/esm2.py:14-145, 146-256; registry mint_plus/models/__init__.py:4-60).

What differs from the reference forward: the (B,T,T) chain mask is not built when every layer is a two-pathway layer
of this package — the layers get `chain_ids` and derive the compact mask metadata from them once per batch — and
`layer_factory` lets a builder choose the layer class.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional

import torch
from torch import nn
from torch.utils.checkpoint import checkpoint

from .modules import RobertaLMHead, TransformerLayer_MINT
from .modules_plus import _TwoPathwayLayer

MODEL_REGISTRY = {
    "8M": dict(name="esm2_t6_8M_UR50D", num_layers=6, embed_dim=320, attention_heads=20, intermediate_size=1280),
    "35M": dict(name="esm2_t12_35M_UR50D", num_layers=12, embed_dim=480, attention_heads=20, intermediate_size=1920),
    "150M": dict(name="esm2_t30_150M_UR50D", num_layers=30, embed_dim=640, attention_heads=20, intermediate_size=2560),
    "650M": dict(name="esm2_t33_650M_UR50D", num_layers=33, embed_dim=1280, attention_heads=20, intermediate_size=5120),
    "3B": dict(name="esm2_t36_3B_UR50D", num_layers=36, embed_dim=1792, attention_heads=16, intermediate_size=7168),
    "15B": dict(name="esm2_t48_15B_UR50D", num_layers=48, embed_dim=5120, attention_heads=20, intermediate_size=20480),
}

# Head sizes the CUDA attention kernels take, and the widest rows the fused residual + LayerNorm kernels take.  The
# registry's "35M" (head size 24), "3B" (head size 112) and "15B" (head size 256, rows of 5120) entries are kept for their names and shapes
# (state dicts can be inspected on the CPU); running them on the GPU raises NotImplementedError.
SUPPORTED_HEAD_DIMS = (16, 32, 64)
MAX_EMBED_DIM = 2560


def check_supported_shape(embed_dim: int, attention_heads: int) -> None:
    """Raise NotImplementedError for a model shape the CUDA path cannot run (there is no eager fallback)."""
    head_dim = embed_dim // attention_heads
    if head_dim not in SUPPORTED_HEAD_DIMS or embed_dim > MAX_EMBED_DIM:
        raise NotImplementedError(
            f"embed_dim={embed_dim}, attention_heads={attention_heads} (head size {head_dim}) is outside what the CUDA kernels "
            f"of this package run: head sizes {SUPPORTED_HEAD_DIMS}, embed_dim <= {MAX_EMBED_DIM}")


class Alphabet:
    """The ESM-1b token table: 33 entries, <cls>=0, <pad>=1, <eos>=2, <unk>=3, amino acids from 4, <mask>=32."""

    toks = ["<cls>", "<pad>", "<eos>", "<unk>", "L", "A", "G", "V", "S", "E", "R", "T", "I", "D", "P", "K", "Q", "N", "F",
            "Y", "M", "H", "W", "C", "X", "B", "U", "Z", "O", ".", "-", "<null_1>", "<mask>"]

    def __init__(self):
        self.tok_to_idx = {t: i for i, t in enumerate(self.toks)}
        self.padding_idx, self.cls_idx, self.eos_idx = 1, 0, 2
        self.unk_idx, self.mask_idx = 3, 32
        self.prepend_bos = self.append_eos = True

    def __len__(self):
        return len(self.toks)

    @classmethod
    def from_architecture(cls, name: str) -> "Alphabet":
        if name not in ("ESM-1b", "roberta_large"):
            raise ValueError(f"unknown alphabet {name!r}")
        return cls()

    def encode(self, sequence: str) -> List[int]:
        return [self.tok_to_idx.get(ch, self.unk_idx) for ch in sequence]


class MINT(nn.Module):
    def __init__(self, num_layers: int = 33, embed_dim: int = 1280, attention_heads: int = 20, alphabet="ESM-1b",
                 token_dropout: bool = True, use_multimer: bool = True, use_rmsnorm: bool = False,
                 use_erf_gelu: bool = False, fp8: bool = False,
                 layer_factory: Optional[Callable[[], nn.Module]] = None):
        super().__init__()
        self.num_layers, self.embed_dim, self.attention_heads = num_layers, embed_dim, attention_heads
        if not isinstance(alphabet, Alphabet):
            alphabet = Alphabet.from_architecture(alphabet)
        self.alphabet = alphabet
        self.alphabet_size = len(alphabet)
        self.padding_idx, self.mask_idx = alphabet.padding_idx, alphabet.mask_idx
        self.cls_idx, self.eos_idx = alphabet.cls_idx, alphabet.eos_idx
        self.prepend_bos, self.append_eos = alphabet.prepend_bos, alphabet.append_eos
        self.token_dropout = token_dropout
        self.use_multimer = use_multimer
        self.use_rmsnorm = use_rmsnorm
        self.use_erf_gelu = use_erf_gelu
        # True / False, or "auto": checkpoint per layer (as the reference always does, esm2.py:124-132) only when the
        # activations of all layers would not fit in the free device memory — on a 180 GB part they usually do
        self.checkpoint_layers = "auto"
        # Variable-length packing: padded positions are dropped from the token-wise work (projections, norms, FFN) and
        # query tiles that hold only padding are left out of the attention.  Non-padded positions get the same values; padded
        # positions of the outputs are zero instead of the values the reference computes there.  bfloat16 on the GPU only.
        self.pack_padding = False
        self._init_submodules(layer_factory)

    def _init_submodules(self, layer_factory=None):
        self.embed_tokens = nn.Embedding(self.alphabet_size, self.embed_dim, padding_idx=self.padding_idx)
        if layer_factory is None:
            def layer_factory():
                return TransformerLayer_MINT(self.embed_dim, 4 * self.embed_dim, self.attention_heads,
                                             use_rmsnorm=self.use_rmsnorm, use_rotary_embeddings=True,
                                             use_multimer=self.use_multimer, use_erf_gelu=self.use_erf_gelu)
        self.layers = nn.ModuleList([layer_factory() for _ in range(self.num_layers)])
        self.emb_layer_norm_after = nn.RMSNorm(self.embed_dim) if self.use_rmsnorm else nn.LayerNorm(self.embed_dim)
        self.lm_head = RobertaLMHead(embed_dim=self.embed_dim, output_dim=self.alphabet_size,
                                     weight=self.embed_tokens.weight)

    def _needs_dense_mask(self) -> bool:
        """The (B,T,T) mask is only built for layers that cannot take chain ids (foreign layer classes, single-pathway
        layers, or the materialised-logits combine)."""
        for layer in self.layers:
            for sub in (layer.layers if hasattr(layer, "layers") else [layer]):
                if not (isinstance(sub, _TwoPathwayLayer) and sub.use_multimer and sub._use_fused_multi_pathway):
                    return True
        return False

    def forward(self, tokens: torch.Tensor, chain_ids: Optional[torch.Tensor] = None,
                repr_layers: List[int] = []) -> Dict[str, torch.Tensor]:
        assert tokens.ndim == 2
        padding_mask = tokens.eq(self.padding_idx)                    # B, T
        if chain_ids is None:
            chain_ids = torch.zeros_like(tokens)
        self_attn_mask = None
        if self._needs_dense_mask():
            self_attn_mask = ~torch.eq(chain_ids.unsqueeze(-1), chain_ids.unsqueeze(-2))      # B, T, T; True = other chain
            if not self.use_multimer:
                self_attn_mask = None                                 # a single-pathway model attends everywhere

        repr_layers = set(repr_layers)
        hidden_representations = {}
        w_emb = self.embed_tokens.weight
        if tokens.is_cuda and w_emb.dtype in (torch.float32, torch.bfloat16) and (self.embed_dim * w_emb.element_size()) % 16 == 0:
            # on the GPU: lookup, token-dropout rescale, <mask> / <pad> zeroing and the (B,T,E) -> (T,B,E) layout change in one pass
            from . import ops
            x = ops.embed_tokens(tokens, w_emb, self.padding_idx, self.mask_idx, bool(self.token_dropout and self.training), 0.15 * 0.8)
            if 0 in repr_layers:
                hidden_representations[0] = x.transpose(0, 1)
        else:
            x = self.embed_tokens(tokens)
            if self.token_dropout and self.training:
                x = x.masked_fill((tokens == self.mask_idx).unsqueeze(-1), 0.0)
                mask_ratio_train = 0.15 * 0.8
                src_lengths = (~padding_mask).sum(-1)
                mask_ratio_observed = (tokens == self.mask_idx).sum(-1).to(x.dtype) / src_lengths
                x = x * (1 - mask_ratio_train) / (1 - mask_ratio_observed)[:, None, None]
            x = x * (1 - padding_mask.unsqueeze(-1).type_as(x))
            if 0 in repr_layers:
                hidden_representations[0] = x
            x = x.transpose(0, 1).contiguous()                         # (B,T,E) -> (T,B,E), laid out sequence-first
        pack = None
        if self.pack_padding:
            if self_attn_mask is not None or not (x.is_cuda and x.dtype == torch.bfloat16):
                raise NotImplementedError("pack_padding needs bfloat16 CUDA activations and the fused two-pathway layers")
            from .ops import PackInfo
            pack = PackInfo(padding_mask)
            T_, B_, E_ = x.shape
            x = x.view(T_ * B_, E_).index_select(0, pack.rows64).unsqueeze(1)      # (N,1,E): the unpadded tokens

        def unpack(t):                                                 # (N,1,E) -> (T,B,E), zeros at padded positions
            if pack is None:
                return t
            full = t.new_zeros(pack.T * pack.B, t.shape[-1])
            return full.index_copy(0, pack.rows64, t.squeeze(1)).view(pack.T, pack.B, t.shape[-1])

        use_ckpt = self.training and torch.is_grad_enabled() and self._want_checkpoint(x)
        self.last_forward_checkpointed = use_ckpt
        if use_ckpt and not x.requires_grad:
            x.requires_grad_(True)
        layer_idx = -1
        for layer_idx, layer in enumerate(self.layers):
            if hasattr(layer, "_next_x_scale"):   # lets the layer's last pass write the next layer's e4m3 QKV operand
                from .mu_scaling import qkv_activation_scale
                layer._next_x_scale = qkv_activation_scale(self.layers[layer_idx + 1]) if layer_idx + 1 < len(self.layers) else None
            kw = dict(self_attn_padding_mask=padding_mask, self_attn_mask=self_attn_mask, chain_ids=chain_ids)
            if pack is not None:
                kw["pack"] = pack
            if use_ckpt:
                x, _ = checkpoint(layer, x, use_reentrant=False, **kw)
            else:
                x, _ = layer(x, **kw)
            if (layer_idx + 1) in repr_layers:
                hidden_representations[layer_idx + 1] = unpack(x).transpose(0, 1)

        if x.is_cuda and x.dtype == torch.bfloat16 and isinstance(self.emb_layer_norm_after, nn.LayerNorm):
            from . import ops
            _, x = ops.add_layernorm(x, None, 1.0, 0.0, self.emb_layer_norm_after, need_s=False)
            x = unpack(x)
        else:
            x = unpack(self.emb_layer_norm_after(x))
        if (layer_idx + 1) in repr_layers:
            hidden_representations[layer_idx + 1] = x.transpose(0, 1)
        # the head runs on the sequence-first rows as they are; (T,B,V) -> (B,T,V) is a copy of the small logits tensor only
        # (contiguous, as the reference returns them: callers reshape them with .view)
        logits = self.lm_head(x).transpose(0, 1).contiguous()
        return {"logits": logits, "representations": hidden_representations}

    def _want_checkpoint(self, x: torch.Tensor) -> bool:
        if self.checkpoint_layers != "auto":
            return bool(self.checkpoint_layers)
        if not x.is_cuda:
            return True
        # what one layer keeps for its backward pass: about 11 tensors of the size of x (the layer input, both pathways'
        # q, k, v, the attention output twice, the two residual sums) plus two 4E-wide FFN tensors; 22 x with some margin
        per_layer = 22 * x.numel() * x.element_size()
        free, _ = torch.cuda.mem_get_info(x.device)
        free += torch.cuda.memory_reserved(x.device) - torch.cuda.memory_allocated(x.device)   # cached blocks are reusable
        return per_layer * len(self.layers) > 0.7 * free

    @classmethod
    def from_config(cls, model_size: str, fp8: bool = False, use_erf_gelu: bool = False) -> "MINT":
        if model_size not in MODEL_REGISTRY:
            raise ValueError(f"Unknown model size: {model_size}. Available: {list(MODEL_REGISTRY)}")
        cfg = MODEL_REGISTRY[model_size]
        check_supported_shape(cfg["embed_dim"], cfg["attention_heads"])
        return cls(num_layers=cfg["num_layers"], embed_dim=cfg["embed_dim"], attention_heads=cfg["attention_heads"],
                   fp8=fp8, use_erf_gelu=use_erf_gelu)

    def _upgrade_state_dict(self, state_dict: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        """Map HuggingFace-ESM key names (`esm.encoder.layer.N.attention.self.query...`) to this model's
        (esm2.py:205-246 of the reference)."""
        rules = (("attention.self.query", "self_attn.q_proj"), ("attention.self.key", "self_attn.k_proj"),
                 ("attention.self.value", "self_attn.v_proj"), ("attention.output.dense", "self_attn.out_proj"),
                 ("attention.Layer", "self_attn_layer_norm"), ("LayerNorm", "final_layer_norm"),
                 ("intermediate", "feed_forward.fc1"), ("output", "feed_forward.fc2"))
        out = {}
        for key, value in state_dict.items():
            new_key = key
            for prefix in ("esm.", "encoder."):
                if new_key.startswith(prefix):
                    new_key = new_key[len(prefix):]
            parts = new_key.split(".")
            if len(parts) > 1 and parts[0] in ("layer", "layers") and parts[1].isdigit():
                for pattern, target in rules:
                    if pattern in new_key:
                        new_key = f"layers.{parts[1]}.{target}.{parts[-1]}"
                        break
            elif "word_embeddings.weight" in new_key:
                new_key = "embed_tokens.weight"
            elif "lm_head.decoder.weight" in new_key:
                new_key = "lm_head.weight"
            out[new_key] = value
        return out

    def load_pretrained_weights(self, checkpoint_path: str, strict: bool = False, dtype: torch.dtype = torch.float32,
                                alternating: bool = False):
        ckpt = torch.load(checkpoint_path, map_location="cpu")
        state_dict = ckpt.get("model", ckpt.get("state_dict", ckpt)) if isinstance(ckpt, dict) else ckpt
        state_dict = self._upgrade_state_dict(state_dict)
        if dtype != torch.float32:
            state_dict = {k: v.to(dtype=dtype) for k, v in state_dict.items()}
        if "lm_head.decoder.weight" in state_dict and "lm_head.weight" not in state_dict:
            state_dict["lm_head.weight"] = state_dict["lm_head.decoder.weight"]
        return self.load_state_dict(state_dict, strict=strict)
