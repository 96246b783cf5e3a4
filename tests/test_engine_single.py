"""Partitioned tiny Llama on one process vs the unpartitioned autograd oracle."""
import pytest
import torch

from kareus_b200.config import ParallelConfig, get_model_config
from kareus_b200.models.llama import GPTModel
from kareus_b200.models.oracle import OracleLlama, load_from_shards, shard_of_oracle_grad


def _batch(cfg, b, s, seed=0):
    g = torch.Generator().manual_seed(seed)
    tokens = torch.randint(0, cfg.vocab_size, (b, s), generator=g)
    labels = torch.randint(0, cfg.vocab_size, (b, s), generator=g)
    mask = (torch.rand(b, s, generator=g) > 0.1).float()
    return tokens, labels, mask


def _check(model, oracle, tp=1, rank=0, rtol=1e-6, atol=1e-8):
    for i, layer in enumerate(model.decoder.layers):
        for name, p in (("qkv", layer.qkv.weight), ("proj", layer.proj.weight), ("fc1", layer.fc1.weight),
                        ("fc2", layer.fc2.weight), ("input_norm", layer.input_norm.weight),
                        ("pre_mlp_norm", layer.pre_mlp_norm.weight)):
            want = shard_of_oracle_grad(oracle, name, i, tp, rank)
            torch.testing.assert_close(p.main_grad.to(want.dtype), want, rtol=rtol, atol=atol,
                                       msg=lambda m, n=name, i=i: f"layer {i} {n}: {m}")
    torch.testing.assert_close(model.embedding.weight.main_grad, shard_of_oracle_grad(oracle, "emb", -1, tp, rank),
                               rtol=rtol, atol=atol)
    torch.testing.assert_close(model.output_layer.weight.main_grad, shard_of_oracle_grad(oracle, "out", -1, tp, rank),
                               rtol=rtol, atol=atol)
    torch.testing.assert_close(model.final_norm.weight.main_grad, oracle.final_norm.grad, rtol=rtol, atol=atol)


@pytest.mark.parametrize("n", [1, 2, 4])
@pytest.mark.parametrize("recompute,rl", [(False, None), (True, None), (True, 1)])
def test_single_process_matches_oracle(n, recompute, rl):
    cfg = get_model_config("tiny")
    par = ParallelConfig(num_nanobatches=n, recompute=recompute)
    model = GPTModel(cfg, par, dtype="fp64", recompute_layers=rl)
    oracle = OracleLlama(cfg)
    load_from_shards(oracle, [model])
    tokens, labels, mask = _batch(cfg, 4, 32)
    loss = model(tokens, labels, mask)
    loss.backward()
    model.finalize_grads()
    ref_loss = oracle(tokens, labels, mask)
    ref_loss.backward()
    torch.testing.assert_close(loss.detach(), ref_loss.detach(), rtol=1e-9, atol=1e-10)
    _check(model, oracle)


def test_qk_layernorm_and_dropout_replay():
    cfg = get_model_config("tiny").replace(qk_layernorm=True, hidden_dropout=0.0)
    model = GPTModel(cfg, ParallelConfig(num_nanobatches=2, recompute=True), dtype="fp64")
    oracle = OracleLlama(cfg)
    load_from_shards(oracle, [model])
    tokens, labels, mask = _batch(cfg, 2, 16)
    loss = model(tokens, labels, mask)
    loss.backward()
    ref_loss = oracle(tokens, labels, mask)
    ref_loss.backward()
    torch.testing.assert_close(loss.detach(), ref_loss.detach(), rtol=1e-9, atol=1e-10)
    l0 = model.decoder.layers[0]
    torch.testing.assert_close(l0.qkv_post.q_norm_weight.main_grad, oracle.layers[0].q_norm.grad, rtol=1e-6, atol=1e-9)

    # dropout: recompute must reproduce the forward masks, so grads equal the non-recompute run
    cfg_d = get_model_config("tiny").replace(hidden_dropout=0.1)
    torch.manual_seed(0)
    grads = []
    for rec in (False, True):
        import kareus_b200.ops.basic as basic
        import itertools
        basic._SEED_COUNTER = itertools.count(1)
        m = GPTModel(cfg_d, ParallelConfig(num_nanobatches=2, recompute=rec), dtype="fp64")
        m(tokens, labels, mask).backward()
        grads.append(m.decoder.layers[0].fc1.weight.main_grad.clone())
    torch.testing.assert_close(grads[0], grads[1], rtol=1e-9, atol=1e-12)


@pytest.mark.parametrize("n,recompute", [(2, True), (4, False)])
def test_sequence_split_nanobatches(n, recompute):
    """MBS 1: nanobatches split the sequence; later nanobatches attend to earlier ones' keys and
    send dK/dV back (backward visits nanobatches last to first)."""
    cfg = get_model_config("tiny")
    par = ParallelConfig(num_nanobatches=n, recompute=recompute, nano_split_dim="seq")
    model = GPTModel(cfg, par, dtype="fp64")
    assert model.seq_split
    oracle = OracleLlama(cfg)
    load_from_shards(oracle, [model])
    tokens, labels, mask = _batch(cfg, 1, 64)
    loss = model(tokens, labels, mask)
    loss.backward()
    model.finalize_grads()
    ref_loss = oracle(tokens, labels, mask)
    ref_loss.backward()
    torch.testing.assert_close(loss.detach(), ref_loss.detach(), rtol=1e-9, atol=1e-10)
    _check(model, oracle)


def test_gelu_and_geglu_ops_match_autograd():
    from kareus_b200.engine.context import OpContext
    from kareus_b200.ops.activations import GegluOp, GeluOp
    for op, width in ((GeluOp(), 16), (GegluOp(), 32)):
        x = torch.randn(3, 5, width, dtype=torch.float64, requires_grad=True)
        ctx = OpContext()
        (y,) = op.forward(ctx, x.detach())
        if op.gated:
            a, b = x[..., :16], x[..., 16:]
            want = torch.nn.functional.gelu(a, approximate="tanh") * b
        else:
            want = torch.nn.functional.gelu(x, approximate="tanh")
        torch.testing.assert_close(y, want.detach(), rtol=1e-9, atol=1e-10)
        g = torch.randn_like(want)
        want.backward(g)
        (dx,) = op.backward(ctx, g)
        torch.testing.assert_close(dx, x.grad, rtol=1e-8, atol=1e-9)


def test_layernorm_and_bias_ops_match_autograd():
    from kareus_b200.engine.context import OpContext
    from kareus_b200.ops.extras import BiasOp, LayerNormOp, make_norm
    x = torch.randn(6, 3, 32, dtype=torch.float64, requires_grad=True)
    ln = make_norm("LayerNorm", 32, 1e-5, "ln", dtype=torch.float64)
    with torch.no_grad():
        ln.weight.mul_(1.3)
        ln.bias.add_(0.2)
    ctx = OpContext()
    (y,) = ln.forward(ctx, x.detach())
    want = torch.nn.functional.layer_norm(x, (32,), ln.weight.detach(), ln.bias.detach(), 1e-5)
    torch.testing.assert_close(y, want.detach(), rtol=1e-9, atol=1e-10)
    g = torch.randn_like(want)
    w_ref = ln.weight.detach().clone().requires_grad_(True)
    b_ref = ln.bias.detach().clone().requires_grad_(True)
    torch.nn.functional.layer_norm(x, (32,), w_ref, b_ref, 1e-5).backward(g)
    (dx,) = ln.backward(ctx, g)
    torch.testing.assert_close(dx, x.grad, rtol=1e-8, atol=1e-9)
    torch.testing.assert_close(ln.weight.main_grad, w_ref.grad, rtol=1e-8, atol=1e-9)
    torch.testing.assert_close(ln.bias.main_grad, b_ref.grad, rtol=1e-8, atol=1e-9)
    b = BiasOp(32, dtype=torch.float64)
    (z,) = b.forward(OpContext(), x.detach())
    torch.testing.assert_close(z, x.detach() + b.bias.detach())
    b.backward(OpContext(), g)
    torch.testing.assert_close(b.bias.main_grad, g.reshape(-1, 32).sum(0))
    assert type(make_norm("RMSNorm", 32, 1e-5, "n")).__name__ == "RMSNormOp"


@pytest.mark.parametrize("activation,skip", [(None, False), ("gelu", False), (None, True)])
def test_linear_bias_operator_matches_autograd(activation, skip):
    """Linear + bias (+ GELU): forward with and without gradients, all three gradients."""
    import torch.nn.functional as F
    from kareus_b200.engine.context import OpContext
    from kareus_b200.ops.extras import LinearBiasOp
    torch.manual_seed(0)
    op = LinearBiasOp(48, 40, activation=activation, skip_bias_add=skip, dtype=torch.float64, seed=3)
    op.bias.data.normal_()
    x = torch.randn(6, 2, 48, dtype=torch.float64, requires_grad=True)
    w = op.weight.detach().clone().requires_grad_(True)
    b = op.bias.detach().clone().requires_grad_(True)
    z = F.linear(x, w, None if skip else b)
    want = F.gelu(z, approximate="tanh") if activation else z
    ctx = OpContext()
    (y,) = op.forward(ctx, x.detach())
    torch.testing.assert_close(y, want.detach())
    nog = OpContext()
    nog.requires_grad = False
    torch.testing.assert_close(op.forward(nog, x.detach())[0], want.detach())     # the single-launch path
    dy = torch.randn_like(want)
    want.backward(dy)
    (dx,) = op.backward(ctx, dy)
    torch.testing.assert_close(dx, x.grad)
    torch.testing.assert_close(op.weight.main_grad, w.grad)
    if skip:
        assert getattr(op.bias, "main_grad", None) is None
    else:
        torch.testing.assert_close(op.bias.main_grad, b.grad)
