"""mint_plus_b200 — B200 (sm_100a) implementation of MINT's two-pathway combined-softmax attention path.

Host code is Python/PyTorch with the reference's call signatures; the arithmetic runs in libmintb.so
(hand-written CUDA behind the C ABI of include/mintb.h).
"""
from .kernels import (differentiable_multi_pathway_attention, differentiable_multimer_combine,
                      fused_multi_pathway_attention, fused_multimer_combine)
from .ops import (MaskMeta, check_device_status, mask_meta_from_chain_ids, mask_meta_from_mask,
                  multimer_attention, multimer_combine, rope_tables)
from .attention import MultiHeadAttention, MultimerAttention
from .modules_plus import (TransformerLayer_MINT_plus, VanillaFeedForward, build_mint_plus,
                           enable_fused_multi_pathway)
from .modules import CheckpointedBlock, RobertaLMHead, TransformerLayer_MINT, build_checkpointed_model
from .esm2 import MINT, MODEL_REGISTRY, SUPPORTED_HEAD_DIMS, Alphabet
from .training import GraphedTrainStep, mlm_corrupt, shared_step
from .rotary_embedding import RotaryEmbedding
from .mu_scaling import (Fp8Linear, TransformerLayer_MINT_mu, apply_fp8_to_model, build_mint_fp8, build_mint_mu,
                         calibrate_fp8, compute_tau, refresh_fp8_weights, Fp8WeightScaler, set_unit_output_scales, unit_variance_init_)

__all__ = [
    "fused_multi_pathway_attention", "differentiable_multi_pathway_attention", "fused_multimer_combine",
    "differentiable_multimer_combine", "multimer_attention", "multimer_combine", "MaskMeta",
    "mask_meta_from_chain_ids", "mask_meta_from_mask", "rope_tables", "check_device_status",
    "MultiHeadAttention", "MultimerAttention", "TransformerLayer_MINT_plus", "VanillaFeedForward",
    "build_mint_plus", "enable_fused_multi_pathway", "RotaryEmbedding", "Fp8Linear", "apply_fp8_to_model", "calibrate_fp8",
    "unit_variance_init_", "TransformerLayer_MINT", "TransformerLayer_MINT_mu", "RobertaLMHead", "MINT", "MODEL_REGISTRY",
    "Alphabet", "build_mint_mu", "build_mint_fp8", "compute_tau", "mlm_corrupt", "shared_step", "GraphedTrainStep", "CheckpointedBlock",
    "build_checkpointed_model", "set_unit_output_scales", "SUPPORTED_HEAD_DIMS", "refresh_fp8_weights", "Fp8WeightScaler",
]
