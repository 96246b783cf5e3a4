"""TP / SP / CP runs on gloo ranks vs the unpartitioned oracle (BASELINE config 1 plumbing)."""
import pytest
import torch
import torch.distributed as dist

from dist_utils import run_distributed


def _worker(rank, world, tp, cp, tp_comm, n, recompute, with_plan, cp_comm="all_gather", seq_split=False):
    from kareus_b200.config import ParallelConfig, get_model_config
    from kareus_b200.models.llama import GPTModel
    from kareus_b200.models.oracle import OracleLlama, load_from_shards, shard_of_oracle_grad
    from kareus_b200.parallel.mesh import Mesh
    from kareus_b200.parallel.collectives import dual_chunk_ids
    from kareus_b200.plan import PipelineCommScheduler, uniform_schedule, CommConfig

    cfg = get_model_config("tiny")
    par = ParallelConfig(tp=tp, cp=cp, num_nanobatches=n, tp_comm=tp_comm, recompute=recompute, cp_comm=cp_comm,
                         nano_split_dim="seq" if seq_split else "auto")
    mesh = Mesh(tp=tp, cp=cp)
    model = GPTModel(cfg, par, mesh=mesh, dtype="fp64", seed=0)
    assert model.seq_split == seq_split
    if with_plan:
        plan = uniform_schedule(1, ["forward", "backward"], CommConfig(("linear_0", "none"), (4, 256)),
                                context_parallel=False)
        sched = PipelineCommScheduler.from_parsed(plan, 0, 1, use_activation_checkpointing=True)
        model.decoder.set_scheduler(sched)

    # gather every TP rank's shards (cp ranks hold replicas) to build the oracle
    class Shell:  # minimal structure load_from_shards expects
        pass
    states = [None] * world
    dist.all_gather_object(states, {k: v.detach() for k, v in model.state_dict().items()})
    tp_models = []
    for r in range(tp):
        m = GPTModel(cfg, ParallelConfig(tp=1, num_nanobatches=n), dtype="fp64", seed=0)
        # rebuild a shard-shaped shell: load rank r's tensors by name
        shell = GPTModel.__new__(GPTModel)
        torch.nn.Module.__init__(shell)
        tp_models.append(states[r])
    oracle = OracleLlama(cfg)
    _load(oracle, tp_models, cfg)

    g = torch.Generator().manual_seed(1)
    b, s = 4, 32
    tokens = torch.randint(0, cfg.vocab_size, (b, s), generator=g)
    labels = torch.randint(0, cfg.vocab_size, (b, s), generator=g)
    mask = (torch.rand(b, s, generator=g) > 0.1).double()
    ref_loss = oracle(tokens, labels, mask)
    ref_loss.backward()

    if cp > 1:
        c = s // (2 * cp)
        a, bb = dual_chunk_ids(cp, mesh.cp_rank)
        idx = torch.cat([torch.arange(a * c, (a + 1) * c), torch.arange(bb * c, (bb + 1) * c)])
        tok_l, lab_l, mask_l = tokens[:, idx], labels[:, idx], mask[:, idx]
    else:
        tok_l, lab_l, mask_l = tokens, labels, mask
    if with_plan:
        sched.on_step_begin()
        sched.on_instruction_begin("forward")
    loss = model(tok_l, lab_l, mask_l, loss_denominator=float(mask.sum()))
    if with_plan:
        sched.on_instruction_begin("backward")
    loss.backward()
    if with_plan:
        sched.on_step_end()
    model.finalize_grads()
    total = loss.detach().clone()
    if cp > 1:
        dist.all_reduce(total, group=mesh.group("cp"))
        for p in model.parameters():
            dist.all_reduce(p.main_grad, group=mesh.group("cp"))
    torch.testing.assert_close(total, ref_loss.detach(), rtol=1e-8, atol=1e-10)
    r = mesh.tp_rank
    for i, layer in enumerate(model.decoder.layers):
        for name, p in (("qkv", layer.qkv.weight), ("proj", layer.proj.weight), ("fc1", layer.fc1.weight),
                        ("fc2", layer.fc2.weight), ("input_norm", layer.input_norm.weight),
                        ("pre_mlp_norm", layer.pre_mlp_norm.weight)):
            want = shard_of_oracle_grad(oracle, name, i, tp, r)
            torch.testing.assert_close(p.main_grad, want, rtol=1e-6, atol=1e-9,
                                       msg=lambda m, n=name, i=i: f"rank {rank} layer {i} {n}: {m}")
    torch.testing.assert_close(model.embedding.weight.main_grad,
                               shard_of_oracle_grad(oracle, "emb", -1, tp, r), rtol=1e-6, atol=1e-9)
    torch.testing.assert_close(model.output_layer.weight.main_grad,
                               shard_of_oracle_grad(oracle, "out", -1, tp, r), rtol=1e-6, atol=1e-9)
    torch.testing.assert_close(model.final_norm.weight.main_grad, oracle.final_norm.grad, rtol=1e-6, atol=1e-9)


def _load(oracle, states, cfg):
    """Assemble oracle weights from per-TP-rank state dicts."""
    def cat(key, dim):
        return torch.cat([s[key] for s in states], dim)
    with torch.no_grad():
        oracle.emb.copy_(cat("embedding.weight", 0))
        oracle.out.copy_(cat("output_layer.weight", 0))
        oracle.final_norm.copy_(states[0]["final_norm.weight"])
        for i, l in enumerate(oracle.layers):
            p = f"decoder.layers.{i}."
            l.input_norm.copy_(states[0][p + "input_norm.weight"])
            l.pre_mlp_norm.copy_(states[0][p + "pre_mlp_norm.weight"])
            l.qkv.copy_(cat(p + "qkv.weight", 0))
            l.proj.copy_(cat(p + "proj.weight", 1))
            gates = [s[p + "fc1.weight"].chunk(2, 0)[0] for s in states]
            ups = [s[p + "fc1.weight"].chunk(2, 0)[1] for s in states]
            l.fc1.copy_(torch.cat(gates + ups, 0))
            l.fc2.copy_(cat(p + "fc2.weight", 1))


@pytest.mark.parametrize("tp_comm,n,recompute,with_plan", [
    ("allreduce", 2, True, True),
    ("allreduce", 4, False, False),
    ("sp", 2, True, True),
    ("sp", 1, False, False),
])
def test_tp2(tp_comm, n, recompute, with_plan):
    run_distributed(_worker, 2, 2, 1, tp_comm, n, recompute, with_plan)


def test_cp2_all_gather():
    run_distributed(_worker, 2, 1, 2, "allreduce", 2, True, False)


def test_tp2_cp2_sp():
    run_distributed(_worker, 4, 2, 2, "sp", 2, True, False)


def test_cp2_ring_attention():
    """Pull-based ring attention (chunk schedule + log-sum-exp merge + dKV reduce-scatter) on gloo."""
    run_distributed(_worker, 2, 1, 2, "allreduce", 2, True, False, "ring")


def _cp_keys_worker(rank, world):
    from kareus_b200.config import ParallelConfig, get_model_config
    from kareus_b200.models.llama import GPTModel
    from kareus_b200.parallel.mesh import Mesh
    from kareus_b200.plan import FWD_KEYS_CP, BWD_KEYS_CP
    par = ParallelConfig(tp=2, cp=2, num_nanobatches=2, tp_comm="allreduce")
    m = GPTModel(get_model_config("tiny"), par, mesh=Mesh(tp=2, cp=2), dtype="fp32")
    eng = m.decoder.engine
    fk = [k for k in eng.full.fwd.expected_keys()]
    bk = [k for k in eng.full.bwd.expected_keys()]
    # the 5 forward and 7 backward keys of the reference's context-parallel plan files all occur
    assert set(FWD_KEYS_CP) <= set(fk), fk
    assert set(BWD_KEYS_CP) <= set(bk), bk
    # one layer: qkv_ar/qkv_ag, ao_ag/ao_ar, mlp/mlp (skipping the very first step, which carries nothing)
    assert fk[1:6] == ["fwd_qkv_ag", "fwd_ao_ag", "fwd_ao_ar", "fwd_mlp", "fwd_mlp"], fk[:8]


def test_cp_plan_keys_match_reference_vocabulary():
    run_distributed(_cp_keys_worker, 4)


@pytest.mark.parametrize("tp,recompute", [(1, True), (1, False), (2, True)])
def test_sequence_split_nanobatches_with_context_parallelism(tp, recompute):
    """Two nanobatches along the sequence on top of dual-chunk context parallelism (micro batches that cannot be
    split along the batch, e.g. one 16k sequence): nanobatch 0 is every rank's early chunk and gathers the first
    half of the keys, nanobatch 1 the late chunk and sees both halves; its backward hands the first half's dK/dV
    to nanobatch 0 before that one's reduce-scatter.  Loss and every gradient equal the unpartitioned oracle."""
    run_distributed(_worker, tp * 2, tp, 2, "allreduce", 2, recompute, False, "all_gather", True)
