"""Trainer steps on CPU: single process, pipeline parallel and data parallel agree."""
import pytest
import torch
import torch.distributed as dist

from dist_utils import run_distributed


def _run_steps(tp, pp, dp, steps=2, n=2, tie=False, want_trainer=False):
    from kareus_b200.config import ParallelConfig, TrainConfig, get_model_config
    from kareus_b200.parallel.mesh import Mesh
    from kareus_b200.train.trainer import Trainer, synthetic_batch
    cfg = get_model_config("tiny")
    if tie:
        cfg = cfg.replace(tie_embeddings=True)
    par = ParallelConfig(tp=tp, pp=pp, dp=dp, num_nanobatches=n, recompute=True)
    tc = TrainConfig(micro_batch_size=2, global_batch_size=8, seq_len=32, lr=2e-3, warmup_steps=0, max_steps=10,
                     dtype="fp64")
    mesh = Mesh(tp=tp, pp=pp, dp=dp)
    tr = Trainer(cfg, par, tc, mesh=mesh, dtype="fp64")
    losses = []
    for i in range(steps):
        full = synthetic_batch(cfg, tc, tc.num_microbatches(1), seed=100, pin=False)
        share = tr.num_microbatches * tc.micro_batch_size
        lo = mesh.dp_rank * share
        batch = {k: v[lo:lo + share] for k, v in full.items()}
        losses.append(tr.train_step(batch, loss_denominator=float(full["loss_mask"].sum())))
    return (losses, tr) if want_trainer else losses


EXPECTED = {}


def test_single_process_trains():
    losses = _run_steps(1, 1, 1, steps=3)
    assert losses[0] > losses[-1]
    assert abs(losses[0] - 6.93) < 0.2       # ln(1024) at init


def _worker(rank, world, tp, pp, dp, want):
    got = _run_steps(tp, pp, dp)
    for a, b in zip(got, want):
        assert abs(a - b) < 1e-8, (got, want)


@pytest.mark.parametrize("tp,pp,dp", [(1, 2, 1), (1, 1, 2), (2, 2, 1)])
def test_parallel_layouts_match_single(tp, pp, dp):
    want = _run_steps(1, 1, 1)
    if tp > 1:
        pytest.skip("tp shards use rank-dependent init; covered by test_engine_distributed")
    run_distributed(_worker, tp * pp * dp, tp, pp, dp, want)


def _tied_worker(rank, world, want):
    got, tr = _run_steps(1, 2, 1, tie=True, want_trainer=True)
    for a, b in zip(got, want):
        assert abs(a - b) < 1e-8, (got, want)
    # both holders of the tied weight still carry the same values after the updates
    m = tr.model
    w = (m.embedding.weight if m.pre_process else m.output_layer.weight).detach().clone()
    both = [torch.empty_like(w) for _ in range(2)]
    dist.all_gather(both, w)
    assert torch.equal(both[0], both[1])
    assert m.tied_across_stages


def test_tied_embedding_across_pipeline_stages_matches_single():
    """Embedding and output weight tied (Qwen3-style) with the two on different pipeline stages: same
    losses as one stage holding one weight, which needs the same init, the summed gradient on both
    copies and the copy counted once in the gradient norm."""
    want = _run_steps(1, 1, 1, tie=True)
    run_distributed(_tied_worker, 2, want)


def _eval_then_train(tp, pp, dp):
    """(evaluation loss, loss of the training step on the same batch, evaluation loss after the step)."""
    from kareus_b200.config import ParallelConfig, TrainConfig, get_model_config
    from kareus_b200.parallel.mesh import Mesh
    from kareus_b200.train.trainer import Trainer, synthetic_batch
    cfg = get_model_config("tiny")
    par = ParallelConfig(tp=tp, pp=pp, dp=dp, num_nanobatches=2, recompute=True)
    tc = TrainConfig(micro_batch_size=2, global_batch_size=8, seq_len=32, lr=2e-3, warmup_steps=0, max_steps=10,
                     dtype="fp64")
    mesh = Mesh(tp=tp, pp=pp, dp=dp)
    tr = Trainer(cfg, par, tc, mesh=mesh, dtype="fp64")
    full = synthetic_batch(cfg, tc, tc.num_microbatches(1), seed=100, pin=False)
    share = tr.num_microbatches * tc.micro_batch_size
    batch = {k: v[mesh.dp_rank * share:(mesh.dp_rank + 1) * share] for k, v in full.items()}
    den = float(full["loss_mask"].sum())
    before = [p.detach().clone() for p in tr.model.parameters()]
    e0 = tr.evaluate(batch, loss_denominator=den)
    assert all(torch.equal(a, b) for a, b in zip(before, tr.model.parameters())) and tr.step_index == 0
    t0 = tr.train_step(batch, loss_denominator=den)
    e1 = tr.evaluate(batch, loss_denominator=den)
    return e0, t0, e1


def _eval_worker(rank, world, tp, pp, dp, want):
    got = _eval_then_train(tp, pp, dp)
    for a, b in zip(got, want):
        assert abs(a - b) < 1e-8, (got, want)


@pytest.mark.parametrize("tp,pp,dp", [(1, 2, 1), (1, 1, 2)])
def test_evaluation_pass(tp, pp, dp):
    """Forward-only evaluation gives the loss a training step reports for the same weights, changes nothing,
    and works through pipeline stages and data-parallel ranks."""
    want = _eval_then_train(1, 1, 1)
    assert abs(want[0] - want[1]) < 1e-10 and want[2] < want[0]
    run_distributed(_eval_worker, tp * pp * dp, tp, pp, dp, want)
