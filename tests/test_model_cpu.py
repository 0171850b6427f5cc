"""The decoder, router, checkpoint helpers and stats on CPU (fp32, collective transport)."""

import torch

from chunked_ep_moe_b200.models.deepseek_tiny import DeepSeekTiny, DeepSeekTinyConfig
from chunked_ep_moe_b200.ops.striping import stripe_weights, unstripe_weights
from chunked_ep_moe_b200.utils import checkpoint as ckpt
from chunked_ep_moe_b200.utils import stats


def _tiny_cfg(**kw):
    base = dict(vocab_size=97, d_model=32, n_layers=3, n_heads=2, head_dim=16, dense_ffn=64, num_experts=4, moe_ffn=16,
                top_k=2, shared_ffn=16, slice_size=16, stripe_width=4, transport="emulated",
                expert_compute="reference")
    base.update(kw)
    return DeepSeekTinyConfig(**base)


def test_decoder_trains_on_cpu():
    torch.manual_seed(0)
    cfg = _tiny_cfg()
    model = DeepSeekTiny(cfg)
    model.init_weights(seed=1)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2)
    tokens = torch.randint(0, cfg.vocab_size, (2, 17))
    losses = []
    for _ in range(8):
        opt.zero_grad()
        ce, aux = model(tokens[:, :-1], tokens[:, 1:])
        (ce + aux).backward()
        opt.step()
        for r in model.routers():
            r.update_bias()
        losses.append(float(ce.detach()))
    assert all(p.grad is not None for p in model.parameters())
    assert losses[-1] < losses[0], losses
    assert float(aux) > 0


def test_slice_size_does_not_change_the_model():
    """Chunking is an execution detail: S=4 and S=1000 give the same loss and gradients."""
    tokens = torch.randint(0, 97, (2, 13), generator=torch.Generator().manual_seed(3))
    outs = []
    for s in (4, 1000):
        model = DeepSeekTiny(_tiny_cfg(slice_size=s))
        model.init_weights(seed=5)
        ce, aux = model(tokens[:, :-1], tokens[:, 1:])
        (ce + aux).backward()
        outs.append((ce.detach(), model.blocks[1].ffn.w_up.grad.clone(), model.embed.weight.grad.clone()))
    assert torch.allclose(outs[0][0], outs[1][0], atol=1e-6)
    assert torch.allclose(outs[0][1], outs[1][1], atol=1e-6)
    assert torch.allclose(outs[0][2], outs[1][2], atol=1e-6)


def test_checkpoint_roundtrip_and_unstriped_export(tmp_path):
    cfg = _tiny_cfg()
    model = DeepSeekTiny(cfg)
    model.init_weights(seed=2)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    tokens = torch.randint(0, cfg.vocab_size, (1, 9))
    ce, aux = model(tokens[:, :-1], tokens[:, 1:])
    (ce + aux).backward()
    opt.step()
    ckpt.save_checkpoint(str(tmp_path), model, opt, step=7, rank=0)

    other = DeepSeekTiny(cfg)
    other.init_weights(seed=99)
    opt2 = torch.optim.AdamW(other.parameters(), lr=1e-3)
    assert ckpt.load_checkpoint(str(tmp_path), other, opt2, rank=0) == 7
    for (n1, p1), (_, p2) in zip(model.state_dict().items(), other.state_dict().items()):
        assert torch.equal(p1, p2), n1

    exported = ckpt.export_unstriped(model.state_dict(), cfg.stripe_width)
    assert any(k.endswith("w_gate") for k in exported) and not any(k.endswith(".w_up") for k in exported)
    back = ckpt.import_unstriped(exported, cfg.stripe_width)
    for k, v in model.state_dict().items():
        assert torch.equal(back[k], v), k


def test_stripe_roundtrip():
    gate, up = torch.randn(3, 8, 12), torch.randn(3, 8, 12)
    for stripe in (1, 4, 12):
        w = stripe_weights(gate, up, stripe)
        assert w.shape == (3, 8, 24)
        g2, u2 = unstripe_weights(w, stripe)
        assert torch.equal(g2, gate) and torch.equal(u2, up)
        assert torch.equal(w[..., :stripe], gate[..., :stripe]) and torch.equal(w[..., stripe:2 * stripe], up[..., :stripe])


def test_stats_helpers():
    wb = stats.wire_bytes(1000, 7168, None, backward=False)
    assert wb["dispatch_bytes"] == 1000 * (7168 * 2 + 4) and wb["combine_bytes"] == 1000 * 7168 * 2
    wq = stats.wire_bytes(1000, 7168, "float8_e4m3fn", backward=True)
    assert wq["dispatch_bytes"] == 1000 * (2 * (7168 + 56 * 4) + 4)
    assert stats.layer_flops(10, 4, 2, False) == 10 * 4 * 2 * 6
    rl = stats.roofline_ms(23.09e12, 4.11e9, {"bf16_tflops_sustained": 1368.3, "bf16_tflops": 1629.7})
    assert abs(rl["compute_ms"] - 16.87) < 0.05 and rl["roofline_ms"] == rl["compute_ms"]
    hs = stats.header_stats([3, 20, 24, 5, 0, 16] + [0] * 10, 8)
    assert hs["my_active_slices"] == 3 and hs["my_padding_rows"] == 4


def _ep_step(rank, world, tokens):
    """One forward/backward + gradient reduction of the decoder on `world` expert-parallel data-parallel ranks."""
    from chunked_ep_moe_b200.train import reduce_gradients

    cfg = _tiny_cfg(aux_loss_coef=0.0)
    model = DeepSeekTiny(cfg)
    model.init_weights(seed=11, rank=rank)
    per = tokens.shape[0] // world
    mine = tokens[rank * per:(rank + 1) * per]
    ce, aux = model(mine[:, :-1], mine[:, 1:])
    (ce + aux).backward()
    reduce_gradients(model, world)
    dense = {n: p.grad.clone() for n, p in model.named_parameters() if not (n.endswith("w_up") or n.endswith("w_down"))}
    experts = {n: p.grad.clone() for n, p in model.named_parameters() if n.endswith("w_up") or n.endswith("w_down")}
    return {"loss": float(ce.detach()), "dense": dense, "experts": experts}


def test_two_ranks_give_the_gradients_of_one():
    """Splitting the batch over two ranks that each own half of the experts changes nothing: the mean loss, the
    (all-reduced) dense gradients and the concatenated expert gradients equal the single-rank step's."""
    from dist_utils import run_ranks

    tokens = torch.randint(0, 97, (4, 13), generator=torch.Generator().manual_seed(7))
    one = _ep_step(0, 1, tokens)
    two = run_ranks(_ep_step, 2, tokens, timeout=300)
    assert abs(one["loss"] - (two[0]["loss"] + two[1]["loss"]) / 2) < 1e-5
    for name, grad in one["dense"].items():
        for r in range(2):
            assert torch.allclose(two[r]["dense"][name], grad, rtol=1e-4, atol=1e-6), name
    for name, grad in one["experts"].items():  # [4 experts, ...] on one rank; [2 experts, ...] on each of two
        both = torch.cat([two[0]["experts"][name], two[1]["experts"][name]])
        assert torch.allclose(both, grad, rtol=1e-4, atol=1e-6), name


def test_router_balancing_state_survives_a_bf16_cast():
    """Casting the model to bf16 must leave the router's counts and selection bias in fp32: a bias of 0.5 still
    moves by 1e-3 per step and counts in the thousands stay exact."""
    from chunked_ep_moe_b200.models.deepseek_tiny import DeepSeekTinyConfig, Router

    cfg = DeepSeekTinyConfig(vocab_size=64, d_model=32, n_layers=2, n_heads=2, head_dim=16, dense_ffn=64,
                             num_experts=4, moe_ffn=32, top_k=2, shared_ffn=32, slice_size=16, transport="emulated",
                             expert_compute="reference")
    router = Router(cfg).to(dtype=torch.bfloat16)
    assert router.weight.dtype == torch.bfloat16
    assert router.routed_bias.dtype == torch.float32 and router.load_counts.dtype == torch.float32
    router.routed_bias.fill_(0.5)
    router.load_counts.copy_(torch.tensor([4097.0, 3.0, 2051.0, 1.0]))
    assert router.load_counts.tolist() == [4097.0, 3.0, 2051.0, 1.0]
    router.update_bias()
    moved = (router.routed_bias - 0.5).abs()
    assert torch.allclose(moved, torch.full_like(moved, cfg.bias_update_rate), rtol=1e-3), moved


def test_router_select_and_dense_swiglu_on_cpu():
    """The plain-torch branches of the fused decoder ops: what the router and the dense FFN compute, written out."""
    from chunked_ep_moe_b200.models import fused_ops

    gen = torch.Generator().manual_seed(3)
    logits = torch.randn(50, 12, generator=gen, requires_grad=True)
    bias = torch.zeros(12)
    bias[7] = 10.0  # the bias decides the selection but never enters the weights
    ids, weights, counts, score_sums = fused_ops.router_select(logits, bias, 3, 2.0)
    assert ids.dtype == torch.int32 and (ids[:, 0] == 7).all()
    scores = torch.sigmoid(logits.detach())
    chosen = torch.gather(scores, 1, ids.long())
    torch.testing.assert_close(weights.detach(), 2.0 * chosen / chosen.sum(-1, keepdim=True))
    torch.testing.assert_close(weights.sum(-1).detach(), torch.full((50,), 2.0))
    assert int(counts.sum()) == 150 and int(counts[7]) == 50
    torch.testing.assert_close(score_sums.sum().detach(), torch.tensor(50.0))  # normalised scores sum to 1 per token
    (weights.sum() + score_sums[0]).backward()
    assert torch.isfinite(logits.grad).all() and logits.grad.abs().sum() > 0

    gu = torch.randn(9, 32, generator=gen)
    gate, up = gu.chunk(2, dim=-1)
    torch.testing.assert_close(fused_ops.dense_swiglu(gu), torch.nn.functional.silu(gate) * up)
