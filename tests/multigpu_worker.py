"""Worker of the multi-GPU tests; launched with torch.distributed.run, one rank per GPU."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def test_heap_collectives(heap, rank, world, dev):
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    for shape in [(1024, 2, 512), (4096, 1, 3072), (333, 1, 8)]:
        x = torch.randn(shape, device=dev, generator=g).bfloat16()
        want = x.clone()
        dist.all_reduce(want)
        got = heap.all_reduce(x.clone(), nb=0, sm_num=8, block_size=512, tag=f"t_ar{shape[0]}")
        torch.cuda.synchronize()
        assert rel(got, want) < 2e-2, ("all_reduce", shape, rel(got, want))
        wg = torch.empty((shape[0] * world,) + shape[1:], device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(wg, x)
        gg = heap.all_gather(x, nb=1, sm_num=4, block_size=1024, tag=f"t_ag{shape[0]}")
        torch.cuda.synchronize()
        assert torch.equal(gg, wg), ("all_gather", shape)
        if shape[0] % world == 0:
            ws = torch.empty((shape[0] // world,) + shape[1:], device=dev, dtype=torch.bfloat16)
            dist.reduce_scatter_tensor(ws, x.clone())
            gs = heap.reduce_scatter(x, nb=0, sm_num=6, block_size=1024, tag=f"t_rs{shape[0]}")
            torch.cuda.synchronize()
            assert rel(gs, ws) < 2e-2, ("reduce_scatter", shape, rel(gs, ws))
    # repeated calls reuse buffers and flags (epochs grow)
    x = torch.ones(2048, 8, device=dev).bfloat16()
    for i in range(5):
        y = heap.all_reduce(x.clone(), nb=0, sm_num=3, tag="rep")
    torch.cuda.synchronize()
    assert torch.all(y == world)


def test_fused_gemm_collectives(heap, rank, world, dev, prefix=""):
    """all-gather→GEMM and GEMM→reduce-scatter kernels vs NCCL + fp32 matmul."""
    from types import SimpleNamespace
    from kareus_b200.engine.context import OpContext
    from kareus_b200.kernels import cuda as KC
    from kareus_b200.ops.fused import FusedAGDgrad, FusedAGGemm, FusedDgradRS, FusedGemmRS
    g = torch.Generator(device=dev).manual_seed(5 + rank)
    for (ms, k, n, sm) in [(256, 512, 384, 4), (1024, 3072, 640, 12), (512, 1024, 3072, 8)]:
        w = (torch.randn(n, k, device=dev, generator=g) * 0.05).bfloat16()
        lin = SimpleNamespace(name=f"{prefix}lin{ms}_{n}", out_features=n, in_features=k, weight=w)
        x = torch.randn(ms, 1, k, device=dev, generator=g).bfloat16()
        xs = torch.empty(ms * world, 1, k, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(xs, x)
        want = xs.float().reshape(-1, k) @ w.float().t()
        op = FusedAGGemm(lin, heap, 8)
        for rep in range(4):
            # with a backward pass to come the gathered input lands in a tensor of its own (kept for the
            # weight gradient); without, in the call site's heap buffer
            ctx = OpContext()
            ctx.requires_grad = rep != 1
            (y,) = op.run((x,), sm_num=sm, nb=0, ctx=ctx)
            torch.cuda.synchronize()
            KC.check_status()
            assert rel(y.reshape(-1, n), want) < 1e-2, ("ag_gemm", ms, k, n, rep, rel(y.reshape(-1, n), want))
            if ctx.requires_grad:
                assert torch.equal(ctx.saved_tensors[0], xs.reshape(-1, k))
        a = torch.randn(ms * world, 1, k, device=dev, generator=g).bfloat16()
        part = (a.float().reshape(-1, k) @ w.float().t())
        full = part.clone()
        dist.all_reduce(full)
        want_rs = full[rank * ms:(rank + 1) * ms]
        op2 = FusedGemmRS(lin, heap, 8)
        for rep in range(3):
            (o,) = op2.run((a,), sm_num=sm, nb=1, ctx=OpContext())
            torch.cuda.synchronize()
            KC.check_status()
            assert rel(o.reshape(-1, n), want_rs) < 2e-2, ("gemm_rs", ms, k, n, rep, rel(o.reshape(-1, n), want_rs))
        # backward mirrors (weight read as an MN-major operand): dgrad → reduce-scatter, all-gather → dgrad
        w.main_grad = torch.zeros(n, k, device=dev)
        dy = torch.randn(ms * world, 1, n, device=dev, generator=g).bfloat16()
        ctx = OpContext()
        ctx.save_for_backward(xs.reshape(-1, k))
        (dx,) = FusedDgradRS(lin, heap, 8).run((dy,), sm_num=sm, nb=0, ctx=ctx)
        torch.cuda.synchronize()
        KC.check_status()
        full = dy.float().reshape(-1, n) @ w.float()
        dist.all_reduce(full)
        assert rel(dx.reshape(-1, k), full[rank * ms:(rank + 1) * ms]) < 2e-2, ("dgrad_rs", ms, k, n)
        assert rel(w.main_grad, dy.float().reshape(-1, n).t() @ xs.float().reshape(-1, k)) < 2e-2
        w.main_grad.zero_()
        dys = torch.randn(ms, 1, n, device=dev, generator=g).bfloat16()
        dyg = torch.empty(ms * world, 1, n, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(dyg, dys)
        ctx = OpContext()
        ctx.save_for_backward(a.reshape(-1, k))
        (dxa,) = FusedAGDgrad(lin, heap, 8).run((dys,), sm_num=sm, nb=1, ctx=ctx)
        torch.cuda.synchronize()
        KC.check_status()
        assert rel(dxa.reshape(-1, k), dyg.float().reshape(-1, n) @ w.float()) < 2e-2, ("ag_dgrad", ms, k, n)
        assert rel(w.main_grad, dyg.float().reshape(-1, n).t() @ a.float().reshape(-1, k)) < 2e-2


def test_nvls_collectives(heap, rank, world, dev):
    """All-reduce and reduce-scatter through the NVLink switch (multimem) vs NCCL.  The multicast binding is
    always undone before the process ends."""
    from kareus_b200.kernels import cuda as KC
    if not heap.enable_nvls(512 << 20):
        if rank == 0:
            print("switch multicast not supported here: skipped", flush=True)
        return
    try:
        g = torch.Generator(device=dev).manual_seed(7 + rank)
        for shape in [(1024, 2, 512), (4096, 1, 3072), (world * 64, 8)]:
            x = torch.randn(shape, device=dev, generator=g).bfloat16()
            want = x.clone()
            dist.all_reduce(want)
            for rep in range(3):
                got = heap.all_reduce(x.clone(), nb=0, sm_num=8, block_size=512, tag=f"n_ar{shape[0]}")
                torch.cuda.synchronize()
                KC.check_status()
                assert rel(got, want) < 2e-2, ("nvls all_reduce", shape, rep, rel(got, want))
            ws = torch.empty((shape[0] // world,) + shape[1:], device=dev, dtype=torch.bfloat16)
            dist.reduce_scatter_tensor(ws, x.clone())
            gs = heap.reduce_scatter(x, nb=1, sm_num=6, block_size=1024, tag=f"n_rs{shape[0]}")
            torch.cuda.synchronize()
            KC.check_status()
            assert rel(gs, ws) < 2e-2, ("nvls reduce_scatter", shape, rel(gs, ws))
        # a producer writes straight into the collective's bound input buffer
        st = heap.staging("ar", "n_stage", 0, (2048, 8), torch.bfloat16)
        st.fill_(float(rank + 1))
        y = heap.all_reduce(st, nb=0, sm_num=4, tag="n_stage")
        torch.cuda.synchronize()
        assert torch.all(y == world * (world + 1) / 2)
        # the fused GEMM+collective kernels in their multicast variants (push through the switch, summed fetch)
        test_fused_gemm_collectives(heap, rank, world, dev, prefix="mc_")
    finally:
        heap.nvls.close()
        heap.nvls = None


def test_bounded_wait(heap, dev):
    from kareus_b200.kernels import cuda as KC
    heap.wait_flag_probe(limit_ns=100_000_000)
    torch.cuda.synchronize()
    try:
        KC.check_status()
        raise AssertionError("expected a peer-timeout status")
    except KC.KernelError as e:
        assert "peer" in str(e)
    assert torch.ones(3, device=dev).sum().item() == 3      # context still usable


def test_model_modes(heap, rank, world, dev):
    from kareus_b200.config import ParallelConfig, TrainConfig, get_model_config
    from kareus_b200.parallel.mesh import Mesh
    from kareus_b200.train.trainer import Trainer, synthetic_batch
    from kareus_b200.kernels import cuda as KC
    cfg = get_model_config("tiny128").replace(num_attention_heads=8, num_query_groups=max(4, world))
    tc = TrainConfig(micro_batch_size=4, global_batch_size=8, seq_len=512, warmup_steps=0, lr=1e-3)
    mesh = Mesh(tp=world)
    losses = {}
    for tp_comm, backend, replay in [("allreduce", "nccl", True), ("allreduce", "kernel", True), ("sp", "nccl", True),
                                     ("sp", "kernel", True), ("sp_fused", "kernel", False),
                                     ("sp_fused", "kernel", True)]:
        par = ParallelConfig(tp=world, num_nanobatches=2, tp_comm=tp_comm, comm_backend=backend, recompute=True)
        try:
            tr = Trainer(cfg, par, tc, mesh=mesh, device=dev, heap=heap,
                         sync=os.environ.get("KAREUS_SYNC", "partition_end"))
        except NotImplementedError:
            continue
        eng = tr.model.decoder.engine
        eng.default_shape = (8, 1024)
        eng.replay = replay
        batch = synthetic_batch(cfg, tc, tr.num_microbatches, seed=7)
        l = [tr.train_step(batch) for _ in range(4)]
        torch.cuda.synchronize()
        KC.check_status()
        losses[(tp_comm, backend, replay)] = l
        if tp_comm == "sp_fused":
            # with launch lists on, the fused path must really have been replayed from C++; NCCL
            # collectives can never be part of a list
            assert (eng.replayed_regions > 0) == replay, (tp_comm, replay, eng.replayed_regions)
        else:
            assert eng.replayed_regions == 0
        del tr
    base = losses[("allreduce", "nccl", True)]
    if rank == 0:
        print("losses:", {k: [round(x, 4) for x in v] for k, v in losses.items()}, flush=True)
    assert base[-1] < base[0]
    for k, v in losses.items():
        for a, b in zip(v, base):
            assert abs(a - b) < 0.05, (k, v, base)


def test_ring_attention(heap, rank, world, dev):
    """CP over the GPUs: K/V tiles of other ranks are read by the attention kernels from peer memory."""
    from kareus_b200.config import ParallelConfig, TrainConfig, get_model_config
    from kareus_b200.parallel.mesh import Mesh
    from kareus_b200.train.trainer import Trainer, synthetic_batch
    from kareus_b200.kernels import cuda as KC
    cfg = get_model_config("tiny128")
    seq = max(1024, 256 * world)         # sequence chunks (2 per rank) of at least one 128-row tile
    tc = TrainConfig(micro_batch_size=2, global_batch_size=4, seq_len=seq, warmup_steps=0, lr=1e-3)
    mesh = Mesh(cp=world)
    losses = {}
    for cp_comm in ("all_gather", "ring"):
        par = ParallelConfig(cp=world, num_nanobatches=2, recompute=True, cp_comm=cp_comm)
        tr = Trainer(cfg, par, tc, mesh=mesh, device=dev, heap_cp=heap if cp_comm == "ring" else None)
        batch = synthetic_batch(cfg, tc, tr.num_microbatches, seed=3, cp=world, cp_rank=mesh.cp_rank)
        losses[cp_comm] = [tr.train_step(batch, loss_denominator=float(4 * seq)) for _ in range(3)]
        torch.cuda.synchronize()
        KC.check_status()
        del tr
    if rank == 0:
        print("cp losses:", losses, flush=True)
    for a, b in zip(losses["ring"], losses["all_gather"]):
        assert abs(a - b) < 0.05, losses
    assert losses["ring"][-1] < losses["ring"][0]


def main():
    from kareus_b200.parallel.mesh import init_distributed
    from kareus_b200.parallel.symm_heap import SymmetricHeap
    rank, world, local = init_distributed(timeout_s=120)     # a rank that died must not hang the others for long
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    which = sys.argv[1] if len(sys.argv) > 1 else "all"
    heap = SymmetricHeap.create(dist.group.WORLD, dev, size_bytes=2 << 30)
    if which in ("all", "collectives"):
        test_heap_collectives(heap, rank, world, dev)
    if which in ("all", "fused"):
        test_fused_gemm_collectives(heap, rank, world, dev)
    if which in ("all", "ring"):
        test_ring_attention(heap, rank, world, dev)
    if which == "nvls":
        test_nvls_collectives(heap, rank, world, dev)
    if which in ("all", "wait"):
        test_bounded_wait(heap, dev)
    if which in ("all", "model"):
        test_model_modes(heap, rank, world, dev)
    dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        print(f"multigpu worker ok ({which}, world {world})", flush=True)
    heap.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
