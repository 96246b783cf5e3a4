"""Launch lists: a region recorded once and replayed from C++ computes what the interpreter path computes."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _trainer(replay: bool, layers=8, chunk=4):
    from kareus_b200.config import ParallelConfig, TrainConfig, get_model_config
    from kareus_b200.train.trainer import Trainer, synthetic_batch
    cfg = get_model_config("tiny128").replace(num_layers=layers)
    tc = TrainConfig(micro_batch_size=2, global_batch_size=8, seq_len=256, warmup_steps=0, lr=1e-3)
    tr = Trainer(cfg, ParallelConfig(num_nanobatches=2, recompute=True), tc, device="cuda", recompute_layers=chunk)
    tr.model.decoder.engine.replay = replay
    batches = [synthetic_batch(cfg, tc, tr.num_microbatches, seed=s) for s in (0, 1)]
    return tr, batches


def test_replayed_steps_match_interpreted_steps():
    from kareus_b200.kernels import cuda as KC, launch_count
    runs = {}
    for replay in (False, True):
        tr, batches = _trainer(replay)
        l0 = launch_count()
        losses, norms = [], []
        for i in range(4):
            losses.append(tr.train_step(batches[i % 2]))
            norms.append(float(tr.optimizer.last_grad_norm))
        torch.cuda.synchronize()
        KC.check_status()
        runs[replay] = (losses, norms, launch_count() - l0, tr.model.decoder.engine.replayed_regions)
    (l_py, n_py, count_py, reg_py), (l_re, n_re, count_re, reg_re) = runs[False], runs[True]
    assert reg_py == 0
    # 4 microbatches per step: the first runs plainly, the second is recorded, all others replay
    # (1 forward region + 2 recompute/backward chunks each)
    assert reg_re == (4 * 4 - 2) * 3
    # a replay accounts for the kernels it launches (the interpreter path counts per wrapper call)
    assert abs(count_re - count_py) < 0.15 * count_py, (count_re, count_py)
    for a, b in zip(l_py, l_re):
        assert abs(a - b) < 2e-2, (l_py, l_re)           # attention backward adds dQ with fp32 atomics
    for a, b in zip(n_py, n_re):
        assert abs(a - b) < 2e-2 * max(1.0, abs(a)), (n_py, n_re)
    assert l_re[-1] < l_re[0]


def test_regions_with_per_call_state_stay_interpreted():
    """Dropout draws a new seed per call: such a block is never recorded."""
    tr, batches = _trainer(True, layers=2, chunk=2)
    for layer in tr.model.decoder.layers:
        layer.attn_bda.p = 0.1
    for i in range(3):
        tr.train_step(batches[i % 2])
    torch.cuda.synchronize()
    assert tr.model.decoder.engine.replayed_regions == 0


def test_rmsnorm_backward_accumulates_into_main_grad():
    from kareus_b200.kernels import cuda as KC, ref
    g = torch.Generator(device="cuda").manual_seed(3)
    for rows, H in [(1000, 3072), (257, 128)]:
        x = torch.randn(rows, H, device="cuda", generator=g).bfloat16()
        dy = torch.randn(rows, H, device="cuda", generator=g).bfloat16()
        w = torch.randn(H, device="cuda", generator=g).bfloat16()
        _, rstd = KC.rmsnorm_fwd(x, w, 1e-5)
        acc = torch.randn(H, device="cuda", generator=g)
        want_dx, want_dw = ref.rmsnorm_bwd(dy.float(), x.float(), rstd, w.float())
        want = acc + want_dw
        dx, none = KC.rmsnorm_bwd(dy, x, rstd, w, dw_accum=acc)
        assert none is None
        torch.testing.assert_close(acc, want, rtol=2e-3, atol=2e-2)
        torch.testing.assert_close(dx.float(), want_dx, rtol=2e-2, atol=2e-2)
