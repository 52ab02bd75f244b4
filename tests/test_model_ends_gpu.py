"""The model's prologue and epilogue on the GPU path (called through the C ABI) against the tensor expressions of the
reference: the embedding with token-dropout rescale, <mask> / <pad> zeroing and the (T,B,E) layout (esm2.py:91-104), the
RobertaLMHead (modules.py:338-369) on the library's GEMMs, and the masked-language-model loss (training/wrapper.py:77-80)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

import mint_plus_b200 as M  # noqa: E402
from mint_plus_b200 import ops  # noqa: E402

DEV = "cuda"
PAD, MASK = 1, 32


def _tokens(B, T, seed):
    g = torch.Generator().manual_seed(seed)
    tok = torch.randint(4, 24, (B, T), generator=g)
    tok[:, 0] = 0
    for b in range(B):
        n_pad = int(torch.randint(0, T // 3, (1,), generator=g))
        if n_pad:
            tok[b, T - n_pad:] = PAD
        tok[b, torch.randint(1, T - n_pad, (max(1, T // 10),), generator=g)] = MASK
    return tok


def _ref_embed(tok, w, token_dropout):
    x = F.embedding(tok, w)
    pad = tok.eq(PAD)
    if token_dropout:
        x = x.masked_fill((tok == MASK).unsqueeze(-1), 0.0)
        observed = (tok == MASK).sum(-1).float() / (~pad).sum(-1)
        x = x * (1 - 0.15 * 0.8) / (1 - observed)[:, None, None]
    x = x * (1 - pad.unsqueeze(-1).float())
    return x.transpose(0, 1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("token_dropout", [False, True])
def test_embedding_prologue_and_its_weight_gradient(dtype, token_dropout):
    B, T, E, V = 3, 200, 320, 33
    tok = _tokens(B, T, 5)
    torch.manual_seed(0)
    w = torch.randn(V, E).to(dtype)
    gy = torch.randn(T, B, E).to(dtype)
    wd = w.to(DEV).requires_grad_(True)
    out = ops.embed_tokens(tok.to(DEV), wd, PAD, MASK, token_dropout, 0.15 * 0.8)
    assert tuple(out.shape) == (T, B, E) and out.is_contiguous() and out.dtype == dtype
    out.backward(gy.to(DEV))
    wr = w.float().requires_grad_(True)
    want = _ref_embed(tok, wr, token_dropout)
    want.backward(gy.float())
    if dtype == torch.float32:
        torch.testing.assert_close(out.cpu(), want.detach(), rtol=1e-6, atol=1e-7)
        torch.testing.assert_close(wd.grad.cpu(), wr.grad, rtol=1e-5, atol=1e-5)
    else:
        assert (out.float().cpu() - want.detach()).abs().max().item() <= 8e-3 * want.abs().max().item()
        assert (wd.grad.float().cpu() - wr.grad).abs().max().item() <= 1e-2 * wr.grad.abs().max().item()
    if not token_dropout:       # no arithmetic at all: the rows are copies
        flat = out.cpu().transpose(0, 1)
        assert torch.equal(flat[~tok.eq(PAD)], w[tok[~tok.eq(PAD)]])
        assert flat[tok.eq(PAD)].abs().max().item() == 0


def test_masked_cross_entropy_value_and_gradient_in_both_row_orders():
    B, T, V, ld = 4, 150, 33, 40
    torch.manual_seed(1)
    base = (2 * torch.randn(T, B, ld)).bfloat16()
    tok = _tokens(B, T, 9)
    target = (torch.rand(B, T) < 0.15) & ~tok.eq(PAD)
    ref_logits = base[..., :V].float().transpose(0, 1).clone().requires_grad_(True)            # (B, T, V)
    ref = F.cross_entropy(ref_logits.transpose(1, 2), tok, reduction="none")
    ref = (ref * target).sum() / target.sum()
    (ref * 3.0).backward()
    for order in ("tb", "bt"):
        store = base.to(DEV) if order == "tb" else base.transpose(0, 1).contiguous().to(DEV)
        store.requires_grad_(True)
        logits = store[..., :V].transpose(0, 1) if order == "tb" else store[..., :V]
        assert tuple(logits.shape) == (B, T, V)
        loss = ops.masked_cross_entropy(logits, tok.to(DEV), target.to(DEV))
        (loss * 3.0).backward()
        assert abs(loss.item() - ref.item()) <= 1e-4 * abs(ref.item())
        g = store.grad.float().cpu()
        g = g.transpose(0, 1) if order == "tb" else g
        assert g[..., V:].abs().max().item() == 0                                         # pad columns get no gradient
        assert (g[..., :V] - ref_logits.grad).abs().max().item() <= 1e-2 * ref_logits.grad.abs().max().item()


def test_lm_head_on_the_library_kernels_matches_the_tensor_expression():
    torch.manual_seed(3)
    E, V, T, B = 320, 33, 70, 3
    emb = torch.nn.Embedding(V, E)
    head = M.RobertaLMHead(E, V, emb.weight)
    with torch.no_grad():
        head.bias.normal_(0, 0.1)
        head.dense.bias.normal_(0, 0.1)
    for p in list(head.parameters()) + [emb.weight]:
        p.data = p.data.bfloat16().float()
    x = torch.randn(T, B, E).bfloat16().float()
    gy = torch.randn(T, B, V).bfloat16().float()
    xr = x.clone().requires_grad_(True)
    want = F.linear(head.layer_norm(F.gelu(head.dense(xr))), emb.weight) + head.bias
    want.backward(gy)
    want_gw = emb.weight.grad.clone()
    emb.weight.grad = None
    emb_g = emb.to(DEV).to(torch.bfloat16)
    head_g = M.RobertaLMHead(E, V, emb_g.weight).to(DEV).to(torch.bfloat16)
    head_g.load_state_dict({k: v for k, v in head.state_dict().items()}, strict=False)
    head_g.weight = emb_g.weight
    xg = x.to(DEV, torch.bfloat16).requires_grad_(True)
    got = head_g(xg)
    assert tuple(got.shape) == (T, B, V)
    got.backward(gy.to(DEV, torch.bfloat16))
    ops.check_device_status()
    assert (got.float().cpu() - want.detach()).abs().max().item() <= 3e-2 * want.abs().max().item()
    assert (xg.grad.float().cpu() - xr.grad).abs().max().item() <= 3e-2 * xr.grad.abs().max().item()
    assert (emb_g.weight.grad.float().cpu() - want_gw).abs().max().item() <= 3e-2 * want_gw.abs().max().item()


def test_training_step_runs_on_library_kernels_from_tokens_to_loss():
    """A bf16 training step of a small model: no torch embedding / linear / layer_norm / cross_entropy kernel between the tokens
    and the loss; the loss equals the tensor-expression loss on the model's own logits."""
    torch.manual_seed(7)
    model = M.MINT(num_layers=2, embed_dim=128, attention_heads=4, use_multimer=True).to(DEV).to(torch.bfloat16).train()
    tok = _tokens(2, 256, 11).to(DEV)
    tok[tok == MASK] = 5
    cid = torch.zeros_like(tok); cid[:, 100:] = 1
    gen = torch.Generator(device=DEV).manual_seed(4)
    loss, ppl = M.shared_step(model, (tok, cid), generator=gen)
    loss.backward()
    ops.check_device_status()
    assert torch.isfinite(loss) and all(p.grad is not None and torch.isfinite(p.grad).all() for p in model.parameters())
    gen = torch.Generator(device=DEV).manual_seed(4)
    inp, target = M.mlm_corrupt(tok, 0, model.eos_idx, model.padding_idx, model.mask_idx, gen)
    with torch.no_grad():
        out = model(inp, chain_ids=cid)["logits"]
    ref = F.cross_entropy(out.float().transpose(1, 2), tok, reduction="none")
    ref = (ref * target).sum() / target.sum()
    assert abs(loss.item() - ref.item()) <= 2e-3 * abs(ref.item())


def test_graphed_training_step_replays_the_eager_step():
    """A training step captured into a CUDA graph: replays give finite losses close to the eager step's (the MLM corruption
    is redrawn every replay, so not equal), every trainable parameter gets a finite, non-zero gradient at an address that
    does not move between replays, and a new batch copied into the graph's buffers changes the result."""
    torch.manual_seed(9)
    model = M.MINT(num_layers=2, embed_dim=128, attention_heads=4, use_multimer=True).to(DEV).to(torch.bfloat16).train()
    tok = _tokens(2, 256, 13).to(DEV)
    tok[tok == MASK] = 5
    cid = torch.zeros_like(tok); cid[:, 120:] = 1
    losses = []
    for _ in range(4):
        for p in model.parameters():
            p.grad = None
        loss, _ = M.shared_step(model, (tok, cid))
        loss.backward()
        losses.append(loss.item())
    eager = sum(losses) / len(losses)
    eager_norm = sum(p.grad.float().norm().item() for p in model.parameters())
    del loss          # a live loss keeps the eager step's autograd graph (and its gradient-accumulation nodes, bound to the
    # default stream) alive, which invalidates a capture on another stream
    graphed = M.GraphedTrainStep(model, tok, cid)
    l1 = graphed.step().item()
    ptrs = [p.grad.data_ptr() for p in model.parameters()]
    l2 = graphed.step(tok, cid).item()
    ops.check_device_status()
    assert [p.grad.data_ptr() for p in model.parameters()] == ptrs
    for l in (l1, l2):
        assert l == l and abs(l - eager) <= 0.15 * abs(eager), (l, eager)
    norm = sum(p.grad.float().norm().item() for p in model.parameters())
    assert all(torch.isfinite(p.grad).all() for p in model.parameters())
    assert 0.5 * eager_norm <= norm <= 2.0 * eager_norm
    tok2 = _tokens(2, 256, 14).to(DEV)
    tok2[tok2 == MASK] = 7
    g_before = [p.grad.clone() for p in model.parameters()]
    graphed.step(tok2.cpu().pin_memory(), cid)      # a pinned host batch is copied in as well
    torch.cuda.synchronize()
    assert any(not torch.equal(a, p.grad) for a, p in zip(g_before, model.parameters()))
