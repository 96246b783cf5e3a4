"""Single-partition executor and the hardware evaluator on CPU with a simulated NVML."""
import pytest
import torch

from kareus_b200.config import ParallelConfig, get_model_config
from kareus_b200.energy import EnergyMonitor, FakeNVML, FrequencyController
from kareus_b200.profile.hardware import HardwareEvaluator
from kareus_b200.profile.nonpartition import build_cases, profile_nonpartition
from kareus_b200.profile.partition_executor import PartitionExecutor
from kareus_b200.profile.space import Config


@pytest.mark.parametrize("key", ["fwd_trail", "bwd_trail"])
def test_executor_runs_one_partition_repeatedly(key):
    cfg = get_model_config("tiny")
    ex = PartitionExecutor(cfg, ParallelConfig(num_nanobatches=2, recompute=False), key, 4, 32, dtype="fp32")
    assert "norm_0" in ex.slots() and "linear_0" in ex.slots()
    for _ in range(3):
        ex.execute(("linear_0", "none"), (8, 1024))
    with pytest.raises(KeyError):
        PartitionExecutor(cfg, ParallelConfig(num_nanobatches=2), "fwd_attn", 4, 32, dtype="fp32")  # needs tp > 1


def test_evaluator_and_nonpartition(tmp_path):
    class Clock:
        t = 0.0
        def __call__(self): return self.t
    clk = Clock()
    nv = FakeNVML(n=1, time_fn=clk)
    mon = EnergyMonitor([0], nvml=nv, sync_fn=lambda i: None, time_fn=clk)
    ctl = FrequencyController(0, "locked", nvml=nv)

    class Ex:
        def execute(self, ow, shape):
            clk.t += 0.01 * 1965 / (nv.sm_clock(0))

    ev = HardwareEvaluator(lambda nano: Ex(), mon, ctl, measurement_duration=0.2, cooldown_duration=0.0, settle_s=0.0,
                           sleep_fn=lambda s: None)
    res = ev([Config(1965, 6, ("norm_0", "none")), Config(1200, 6, ("norm_0", "none"))])
    ev.close()
    assert res[1][0] > res[0][0] and res[1][1] < res[0][1]       # slower and cheaper at the lower clock
    assert ev.samples[1]["sm_clock"] == 1200 and nv.calls[-1] == ("reset", 0)

    from kareus_b200.models.llama import GPTModel
    model = GPTModel(get_model_config("tiny"), ParallelConfig(), dtype="fp32")
    cases = build_cases(model, 4, 32, "cpu")
    wrapped = {k: (lambda f=f: (f(), setattr(clk, "t", clk.t + 0.001))[0]) for k, f in cases.items()}
    profile_nonpartition(wrapped, [1500, 1200], tmp_path, mon, measurement_duration=0.01, cooldown_duration=0.0,
                         sleep_fn=lambda s: None)
    txt = (tmp_path / "nonpartition" / "1500" / "loss_energy.csv").read_text().splitlines()
    assert txt[0] == "time (s),total_energy (J),per_rank_energy (J)" and len(txt[1].split(",")) == 3


def test_fused_sequence_parallel_partitions_name_real_slots():
    """Every partition of the fused sequence-parallel path exists as a step key and offers the launch
    slots its search space lists (checked on the unfused "sp" program, which has the same segments)."""
    from kareus_b200.config import ParallelConfig, get_model_config
    from kareus_b200.engine.block import _Chunk
    from kareus_b200.models.llama import TransformerLayer
    from kareus_b200.profile.space import SP_FUSED_SPACES, partition_space

    class Comm:
        heap = None

        def _args(self, axis):
            return (None, 2, 0) if axis == "tp" else (None, 1, 0)

        def make(self, cls, axis, name):
            g, w, r = self._args(axis)
            return cls(g, w, r, name=name)

    cfg = get_model_config("tiny")
    layer = TransformerLayer(cfg, ParallelConfig(tp=2, tp_comm="sp"), Comm(), 0, torch.float32, "cpu", seed=0)
    chunk = _Chunk(layer.operators(), 2, "partition_end")
    assert len(SP_FUSED_SPACES) == 8
    for key, (kind, space) in SP_FUSED_SPACES.items():
        prog = chunk.bwd if key.startswith("bwd_") else chunk.fwd
        steps = [s for s in prog.steps if s.key == key and s.compute and s.comm is not None]
        assert steps, key
        for slot, _ in space.overlap_windows:
            assert slot in steps[-1].slots, (key, slot, steps[-1].slots)
        assert partition_space(key, "sp_fused")[0] == kind
    assert partition_space("fwd_attn", "allreduce")[0] == "all_reduce"


def _cp_partition_worker(rank, world):
    """Context-parallel partitions on TP2 x CP2: one that only exists between two layers (a layer's first
    segment beside the previous layer's MLP all-reduce) and a backward one whose attention backward consumes
    re-gathered K/V, each executed several times as the profiler does."""
    import torch
    from kareus_b200.config import ParallelConfig, get_model_config
    from kareus_b200.parallel.collectives import CommFactory
    from kareus_b200.parallel.mesh import Mesh
    from kareus_b200.profile.partition_executor import PartitionExecutor
    cfg = get_model_config("tiny")
    mesh = Mesh(tp=2, cp=2, dp=1, pp=1)
    par = ParallelConfig(tp=2, cp=2, num_nanobatches=2, tp_comm="allreduce", comm_backend="nccl", recompute=False)
    for key in ("fwd_qkv_ar", "bwd_a_ag", "bwd_o_ar", "bwd_qkv_rs"):
        ex = PartitionExecutor(cfg, par, key, 2, 64, mesh=mesh, comm=CommFactory(mesh, "nccl"), device="cpu",
                               dtype="fp32")
        assert ex.step.key == key and ex.step.comm is not None, key
        slot = sorted(ex.slots())[0]
        for _ in range(3):
            ex.execute(overlap_window=(slot, "none"), resource_shape=(4, 1024))


def test_context_parallel_partitions_run_repeatedly():
    from dist_utils import run_distributed
    run_distributed(_cp_partition_worker, 4, timeout=300.0)
