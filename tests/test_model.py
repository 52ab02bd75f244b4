"""Whole-model parity: the MINT mirror against logits the reference MINT produced on the same name-seeded weights
(tests/golden/mint8m_*.npz, made by tests/golden/make_golden.py).

CPU tests route the attention call to the oracle (test infrastructure) to check the host logic around it — embedding,
pad zeroing, layer glue, LM head, state-dict names; GPU tests run the product path end to end."""
import os

import numpy as np
import pytest
import torch

import mint_plus_b200 as M
from mint_plus_b200 import modules_plus, ops
from oracle import multimer_attention as O
from oracle.seeded_weights import c1_batch, fill_state_dict_

# Six layers of fp32 arithmetic whose sums run in another order than the reference's CPU kernels (tiled attention with an
# online softmax, warp-shuffle LayerNorm sums, split-K-free but differently blocked matrix products).
FP32_MODEL_RTOL = 4e-5
GOLD = os.path.join(os.path.dirname(__file__), "golden")
CASES = ["mint8m_small", "mint8m_mu", "mint8m_mu_sqrt", "mint8m_c1"]


def _load(name):
    z = np.load(os.path.join(GOLD, name + ".npz"))
    seed, batch_seed, B, T, lo, hi, sqrt_sm = (int(v) for v in z["meta"])
    tokens, chain_ids = c1_batch(batch_seed, B, T, lo, hi)
    assert np.array_equal(tokens.numpy(), z["tokens"].astype(np.int64))          # the batch is reproducible from its seed
    assert np.array_equal(chain_ids.numpy(), z["chain_ids"].astype(np.int64))
    return z, seed, tokens, chain_ids, bool(sqrt_sm)


def _build(name, seed, sqrt_sm):
    if "_mu" in name:
        model = M.build_mint_mu("8M", use_sqrt_softmax=sqrt_sm)
    else:
        model = M.MINT(num_layers=6, embed_dim=320, attention_heads=20, use_multimer=True, use_erf_gelu=True)
    fill_state_dict_(model, seed)
    return model.eval()


@pytest.fixture
def oracle_attention(monkeypatch):
    """Replace the CUDA attention by the oracle so that the model's host logic can run without a GPU."""
    def fake_meta(chain_ids, padding_mask):
        return chain_ids, padding_mask

    def fake_attention(q_s, k_s, v_s, q_c, k_c, v_c, *, meta=None, chain_mask=None, key_padding_mask=None, rope=True,
                       inv_freq=None, scale=None, sqrt_softmax=False, out_seq_first=False, **kw):
        if meta is not None:
            ids, key_padding_mask = meta
            chain_mask = ids.unsqueeze(-1) != ids.unsqueeze(-2)
        out = O.multimer_attention(q_s, k_s, v_s, q_c, k_c, v_c, chain_mask, key_padding_mask, scale=scale, rope=rope,
                                   sqrt_softmax=sqrt_softmax)
        return out.permute(2, 0, 1, 3).contiguous() if out_seq_first else out

    monkeypatch.setattr(modules_plus, "_cached_ids_meta", fake_meta)
    monkeypatch.setattr(ops, "multimer_attention", fake_attention)


@pytest.mark.parametrize("name", CASES)
def test_state_dict_keys_equal_the_reference_models(name):
    z, seed, _, _, sqrt_sm = _load(name)
    assert sorted(_build(name, seed, sqrt_sm).state_dict().keys()) == [str(k) for k in z["keys"]]


@pytest.mark.parametrize("name", CASES[:3])
def test_host_logic_matches_reference_logits_with_oracle_attention(name, oracle_attention):
    z, seed, tokens, chain_ids, sqrt_sm = _load(name)
    model = _build(name, seed, sqrt_sm)
    with torch.no_grad():
        res = model(tokens, chain_ids, repr_layers=[3, 6])
    np.testing.assert_allclose(res["logits"].numpy(), z["logits"], rtol=1e-4, atol=2e-5)
    np.testing.assert_allclose(res["representations"][3][:, ::8].numpy(), z["repr3"], rtol=1e-4, atol=2e-5)
    np.testing.assert_allclose(res["representations"][6][:, ::8].numpy(), z["repr6"], rtol=1e-4, atol=2e-5)


def test_product_path_refuses_cpu_tensors():
    model = _build("mint8m_small", 1, False)
    tokens, chain_ids = c1_batch(7, 1, 32, 4, 8)
    with pytest.raises((RuntimeError, ValueError, TypeError)):
        model(tokens, chain_ids)


def test_token_dropout_rescale_and_checkpointing_in_training_mode(oracle_attention):
    torch.manual_seed(0)
    model = M.MINT(num_layers=2, embed_dim=64, attention_heads=4, use_multimer=True).train()
    tokens, chain_ids = c1_batch(9, 2, 48, 5, 15)
    tokens[0, 3] = model.mask_idx
    out = model(tokens, chain_ids)["logits"]
    out.float().pow(2).mean().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in model.parameters())
    # rows that hold a <mask> are rescaled by (1 - 0.12) / (1 - observed ratio) (esm2.py:94-99 of the reference)
    emb = model.embed_tokens(tokens)
    n = (tokens[0] != model.padding_idx).sum()
    x0 = emb[0, 0] * (1 - 0.12) / (1 - 1.0 / n)
    rep = model(tokens, chain_ids, repr_layers=[0])["representations"][0]
    torch.testing.assert_close(rep[0, 0], x0)
    assert rep[0, 3].abs().max() == 0


# ------------------------------------------------------------------------------------------------ GPU

@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_model_fp32_matches_reference_logits(name):
    z, seed, tokens, chain_ids, sqrt_sm = _load(name)
    model = _build(name, seed, sqrt_sm).cuda()
    with torch.no_grad():
        res = model(tokens.cuda(), chain_ids.cuda(), repr_layers=[3, 6])
    ops.check_device_status()
    got, want = res["logits"].cpu().numpy(), z["logits"]
    # fp32 tolerance: 1e-5 relative to the logits' scale (values are O(1..5))
    rel = np.abs(got - want).max() / max(1.0, np.abs(want).max())
    print(f"{name}: fp32 logits max err / scale = {rel:.3g}")
    assert rel <= FP32_MODEL_RTOL, rel
    np.testing.assert_allclose(res["representations"][6][:, ::8].cpu().numpy(), z["repr6"], rtol=1e-4, atol=4e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_model_bf16_tracks_reference_logits(name):
    z, seed, tokens, chain_ids, sqrt_sm = _load(name)
    model = _build(name, seed, sqrt_sm).cuda().to(torch.bfloat16)
    for layer in model.layers:                       # rotary tables stay fp32, as under bf16-mixed training
        layer.self_attn.rot_emb.inv_freq = layer.self_attn.rot_emb.inv_freq.float()
    with torch.no_grad():
        res = model(tokens.cuda(), chain_ids.cuda())
    ops.check_device_status()
    got, want = res["logits"].float().cpu().numpy(), z["logits"]
    valid = (tokens != 1).numpy()
    err = np.abs(got - want)[valid]
    assert err.max() < 0.25 and err.mean() < 0.03, (err.max(), err.mean())


@pytest.mark.gpu
def test_model_bf16_training_step_gives_finite_gradients():
    torch.manual_seed(0)
    model = M.MINT(num_layers=2, embed_dim=320, attention_heads=20, use_multimer=True).cuda().to(torch.bfloat16).train()
    tokens, chain_ids = c1_batch(11, 2, 256, 30, 100)
    out = model(tokens.cuda(), chain_ids.cuda())["logits"]
    loss = torch.nn.functional.cross_entropy(out.float().view(-1, 33), tokens.cuda().view(-1), ignore_index=1)
    loss.backward()
    ops.check_device_status()
    assert torch.isfinite(loss)
    for n, p in model.named_parameters():
        assert p.grad is not None and torch.isfinite(p.grad).all(), n


@pytest.mark.gpu
def test_checkpointed_layers_give_the_same_gradients():
    """Per-layer activation checkpointing (esm2.py:117-127 of the reference always checkpoints) recomputes the fused
    projection + attention step in the backward pass: same loss, and gradients equal up to the order of the dQ reductions."""
    torch.manual_seed(0)
    model = M.MINT(num_layers=2, embed_dim=320, attention_heads=20, use_multimer=True).cuda().to(torch.bfloat16).train()
    tokens, chain_ids = c1_batch(13, 2, 256, 30, 100)
    tokens, chain_ids = tokens.cuda(), chain_ids.cuda()
    results = []
    for ckpt in (False, True):
        model.checkpoint_layers = ckpt
        model.zero_grad(set_to_none=True)
        out = model(tokens, chain_ids)["logits"]
        loss = torch.nn.functional.cross_entropy(out.float().view(-1, 33), tokens.view(-1), ignore_index=1)
        loss.backward()
        assert model.last_forward_checkpointed == ckpt
        results.append((loss.detach().clone(), {n: p.grad.detach().float().clone() for n, p in model.named_parameters()}))
    ops.check_device_status()
    (l0, g0), (l1, g1) = results
    assert torch.equal(l0, l1)
    for n in g0:
        scale = g0[n].abs().max().item()
        assert (g0[n] - g1[n]).abs().max().item() <= 2e-2 * scale + 1e-6, n


def test_shared_step_masks_only_residues_and_gives_a_finite_loss(oracle_attention):
    """The MLM step of the reference wrapper (training/wrapper.py:48-86): targets are non-special positions only."""
    torch.manual_seed(3)
    model = M.MINT(num_layers=1, embed_dim=64, attention_heads=4, use_multimer=True).train()
    tokens, chain_ids = c1_batch(21, 3, 80, 10, 30)
    g = torch.Generator().manual_seed(5)
    inp, target = M.mlm_corrupt(tokens, 0, model.eos_idx, model.padding_idx, model.mask_idx, g)
    special = (tokens == 0) | (tokens == model.eos_idx) | (tokens == model.padding_idx)
    assert not (target & special).any() and target.any()
    assert torch.equal(inp[~target], tokens[~target])                      # untouched outside the targets
    changed = inp[target] != tokens[target]
    assert ((inp[target] == model.mask_idx) | ~changed | ((inp[target] >= 4) & (inp[target] < 24))).all()
    loss, ppl = M.shared_step(model, (tokens, chain_ids), generator=torch.Generator().manual_seed(6))
    loss.backward()
    assert torch.isfinite(loss.detach()) and torch.isfinite(ppl) and abs(float(ppl) - float(torch.exp(loss.detach()))) < 1e-4


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["base", "mu_fp8"])
def test_packed_tokens_give_the_same_values_at_unpadded_positions(kind):
    """pack_padding drops padded positions from the token-wise work and padded query tiles from the attention: logits
    at real positions and all parameter gradients must agree with the unpacked run (same kernels, same row arithmetic)."""
    torch.manual_seed(0)
    if kind == "base":
        model = M.MINT(num_layers=2, embed_dim=128, attention_heads=4, use_multimer=True)
    else:
        model = M.build_mint_mu("8M", num_layers=2, embed_dim=128, attention_heads=4, use_fp8=True, use_sqrt_softmax=True)
    fill_state_dict_(model, 3)
    model = model.cuda().to(torch.bfloat16).train()
    model.token_dropout = False
    for layer in model.layers:
        layer.self_attn.rot_emb.inv_freq = layer.self_attn.rot_emb.inv_freq.float()
    tokens, chain_ids = c1_batch(31, 3, 384, 20, 60)          # 384 positions, at most 124 real: whole query tiles are padding
    tokens, chain_ids = tokens.cuda(), chain_ids.cuda()
    valid = tokens != 1

    def run(pack):
        model.pack_padding = pack
        model.zero_grad()
        logits = model(tokens, chain_ids)["logits"].float()
        (logits[valid].square().mean()).backward()
        ops.check_device_status()
        return logits.detach(), {n: p.grad.detach().float().clone() for n, p in model.named_parameters() if p.grad is not None}

    want, wgrads = run(False)
    got, ggrads = run(True)
    assert torch.equal(got[valid], want[valid])                # identical arithmetic row by row
    assert (got[~valid] == model.lm_head(torch.zeros(1, 128, device="cuda", dtype=torch.bfloat16)).float()).all()
    assert ggrads.keys() == wgrads.keys()
    for n in wgrads:
        scale = wgrads[n].abs().max().item()
        assert (ggrads[n] - wgrads[n]).abs().max().item() <= 2e-2 * scale + 1e-6, n


@pytest.mark.gpu
def test_lora_adapters_on_the_fused_projection_match_the_module_by_module_path(monkeypatch):
    """Frozen base + LoRA on q/k/v/out: the fused QKV product on the merged weight (adapter gradients through thin
    products) against the plain LoRALinear modules called one by one."""
    from mint_plus_b200.lora import apply_lora
    torch.manual_seed(0)
    model = fill_state_dict_(M.MINT(num_layers=2, embed_dim=128, attention_heads=4, use_multimer=True), 9)
    model = model.cuda().to(torch.bfloat16)
    for layer in model.layers:
        layer.self_attn.rot_emb.inv_freq = layer.self_attn.rot_emb.inv_freq.float()
    apply_lora(model, r=8, alpha=16.0)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if n.endswith("lora_B"):
                p.normal_(0.0, 0.05)
    model.train()
    model.token_dropout = False
    tokens, chain_ids = c1_batch(41, 2, 160, 20, 60)
    tokens, chain_ids = tokens.cuda(), chain_ids.cuda()

    def run():
        model.zero_grad()
        logits = model(tokens, chain_ids)["logits"].float()
        logits.square().mean().backward()
        ops.check_device_status()
        return logits.detach(), {n: p.grad.float().clone() for n, p in model.named_parameters() if p.requires_grad}

    fast, fgrads = run()
    monkeypatch.setattr(modules_plus, "_qkv_operands", lambda attn: None)       # module-by-module projections
    slow, sgrads = run()
    # the merged weight is rounded to bf16 once, the module path rounds base and adapter outputs separately
    assert (fast - slow).abs().max().item() < 0.15 and (fast - slow).abs().mean().item() < 0.03
    assert fgrads.keys() == sgrads.keys() and len(fgrads) == 2 * 2 * 7
    for n in sgrads:
        scale = sgrads[n].abs().max().item()
        assert (fgrads[n] - sgrads[n]).abs().max().item() <= 0.08 * scale + 1e-5, n
