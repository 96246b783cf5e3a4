"""Small, self-terminating workloads of each hot kernel for profiler captures.

    python -m kareus_b200.kernels.profile_cases gemm        # 8192 x 8192 x 8192 bf16, 3 launches
    python -m kareus_b200.kernels.profile_cases attn_fwd    # B4 H3 S4096 d128 causal, 3 launches
    python -m kareus_b200.kernels.profile_cases norm | swiglu | ce | adamw | rope

Each case touches more than the 126 MB L2 where DRAM figures matter but holds at most a few GB,
and launches its kernel a handful of times so a ``--set full`` capture ends within minutes.

Timing tables (CUDA events, no profiler; L2 flushed between launches):

    python -m kareus_b200.kernels.profile_cases gemm_table      # model GEMM shapes at TP 1 and TP 8, vs cuBLAS
    python -m kareus_b200.kernels.profile_cases attn_table      # flash attention forward/backward, vs the wheel
    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 \
        -m kareus_b200.kernels.profile_cases fused                # the eight fused GEMM+collective kernels at TP N
"""
from __future__ import annotations

import os
import sys

import torch


def _timed(fn, flush, iters: int = 7, skip: int = 3) -> float:
    """Median CUDA-event time in ms of ``fn()`` with the L2 flushed before every launch."""
    times = []
    for i in range(iters + skip):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda._sleep(2_000_000)          # the launch is enqueued while the GPU is still busy
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        if i >= skip:
            times.append(a.elapsed_time(b))
    times.sort()
    return times[len(times) // 2]


def gemm_table() -> None:
    """Forward, dgrad and wgrad GEMMs of one Llama-3.2-3B layer and the LM head at TP 1 and TP 8 shapes:
    this library's tcgen05 kernels vs cuBLAS (torch.matmul) on the same tensors."""
    from . import cuda as KC
    dev = "cuda"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    M = 16384
    rows = []
    for tp in (1, 8):
        shapes = {"qkv": (M, 5120 // tp, 3072), "proj": (M, 3072, 3072 // tp), "fc1": (M, 16384 // tp, 3072),
                  "fc2": (M, 3072, 8192 // tp)}
        if tp == 1:
            shapes["head"] = (M, 128256, 3072)
            shapes["square"] = (8192, 8192, 8192)
        for name, (m, n, k) in shapes.items():
            a = torch.randn(m, k, device=dev).bfloat16()
            w = torch.randn(n, k, device=dev).bfloat16()
            dy = torch.randn(m, n, device=dev).bfloat16()
            acc = torch.zeros(n, k, device=dev)
            flops = 2.0 * m * n * k
            cases = {"fprop": (lambda: KC.gemm(a, w), lambda: torch.matmul(a, w.t())),
                     "dgrad": (lambda: KC.gemm(dy, w, trans_b=False), lambda: torch.matmul(dy, w)),
                     "wgrad": (lambda: KC.gemm(dy, a, trans_a=True, trans_b=False, accumulate=acc),
                               lambda: torch.matmul(dy.t(), a))}
            for kind, (ours, lib_) in cases.items():
                t_o, t_l = _timed(ours, flush), _timed(lib_, flush)
                rows.append((f"tp{tp} {name} {kind}", m, n, k, flops / t_o / 1e9, flops / t_l / 1e9))
            del a, w, dy, acc
    KC.check_status()
    print("| GEMM | M | N | K | this library TFLOP/s | cuBLAS TFLOP/s |\n|---|---|---|---|---|---|")
    for r in rows:
        print(f"| {r[0]} | {r[1]} | {r[2]} | {r[3]} | {r[4]:.0f} | {r[5]:.0f} |")


def wgrad_sweep() -> None:
    """Weight-gradient GEMMs (fp32 accumulate, K = 16384 tokens) of the 3B layer at TP 1/2/8 with every
    tile (128 / 256 rows) and K split forced in turn; the last column is what the library picks by itself."""
    import ctypes
    from . import cuda as KC
    L = KC.lib()
    L.kb_gemm_accum_force.argtypes = [ctypes.c_int, ctypes.c_int]
    L.kb_gemm_accum_force.restype = None
    L.kb_gemm_accum_plan.argtypes = [ctypes.c_int] * 4 + [ctypes.POINTER(ctypes.c_int)] * 2
    L.kb_gemm_accum_plan.restype = None
    dev = "cuda"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    tokens = 16384
    splits = (1, 2, 3, 4, 6, 8)
    print("| wgrad | out x in | " + " | ".join(f"{t}/ks{k}" for t in (128, 256) for k in splits)
          + " | picked | picked TFLOP/s | cuBLAS TFLOP/s |")
    print("|---|---|" + "---|" * (2 * len(splits) + 3))
    for tp in (1, 2, 8):
        shapes = {"qkv": (5120 // tp, 3072), "proj": (3072, 3072 // tp), "fc1": (16384 // tp, 3072),
                  "fc2": (3072, 8192 // tp)}
        for name, (n_out, n_in) in shapes.items():
            dy = torch.randn(tokens, n_out, device=dev).bfloat16()
            x = torch.randn(tokens, n_in, device=dev).bfloat16()
            acc = torch.zeros(n_out, n_in, device=dev)
            flops = 2.0 * tokens * n_out * n_in
            run = lambda: KC.gemm(dy, x, trans_a=True, trans_b=False, accumulate=acc)
            cells = []
            for tile in (128, 256):
                for ks in splits:
                    L.kb_gemm_accum_force(tile, ks)
                    cells.append(flops / _timed(run, flush, iters=5, skip=2) / 1e9)
            L.kb_gemm_accum_force(0, 0)
            t_auto = _timed(run, flush)
            t_lib = _timed(lambda: torch.matmul(dy.t(), x), flush)
            tile_c, ks_c = ctypes.c_int(), ctypes.c_int()
            L.kb_gemm_accum_plan(n_out, n_in, tokens, KC.sm_count(),
                                 ctypes.byref(tile_c), ctypes.byref(ks_c))
            print(f"| tp{tp} {name} | {n_out} x {n_in} | " + " | ".join(f"{c:.0f}" for c in cells)
                  + f" | {tile_c.value}/ks{ks_c.value} | {flops / t_auto / 1e9:.0f} | {flops / t_lib / 1e9:.0f} |")
            del dy, x, acc
    KC.check_status()


def memory_table() -> None:
    """Every memory-bound kernel of a training step at the Llama-3.2-3B shapes: CUDA-event time, algorithmic
    bytes (each operand read or written once) and the fraction of the measured copy bandwidth."""
    import json
    from pathlib import Path
    from . import cuda as KC, ref
    dev = "cuda"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    peaks = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    hbm = json.loads(peaks.read_text())["hbm_gbs"] if peaks.exists() else 6650.0
    rows_, H, F, V = 32768, 3072, 8192, 128256
    x = torch.randn(rows_, H, device=dev).bfloat16()
    w = torch.ones(H, device=dev).bfloat16()
    y, rstd = KC.rmsnorm_fwd(x, w, 1e-5)
    dw = torch.zeros(H, device=dev)
    gu = torch.randn(rows_, 2 * F, device=dev).bfloat16()
    act = KC.swiglu_fwd(gu)
    qkv = torch.randn(4096, 8, 8, 5, 128, device=dev).bfloat16()
    fr = ref.rope_table(4096, 128, 500000.0, device=dev)
    logits = torch.randn(8192, V, device=dev).bfloat16()
    tgt = torch.randint(0, V, (8192,), device=dev)
    m, s_, t_ = KC.cross_entropy_local_stats(logits, tgt, 0)
    ones = torch.ones_like(m)
    n = 128 * 1024 * 1024
    g32, m32, v32, w32 = (torch.randn(n, device=dev) for _ in range(4))
    p16 = w32.bfloat16()
    emb = torch.randn(V, H, device=dev).bfloat16()
    tok = torch.randint(0, V, (4096, 8), device=dev)
    demb = torch.randn(4096, 8, H, device=dev).bfloat16()
    gemb = torch.zeros(V, H, device=dev)
    b2 = 2
    cases = [
        ("rmsnorm fwd", lambda: KC.rmsnorm_fwd(x, w, 1e-5), 2 * x.numel() * b2),
        ("rmsnorm bwd (+dw into the main gradient)", lambda: KC.rmsnorm_bwd(y, x, rstd, w, dw_accum=dw), 3 * x.numel() * b2),
        ("swiglu fwd", lambda: KC.swiglu_fwd(gu), (gu.numel() + act.numel()) * b2),
        ("swiglu bwd", lambda: KC.swiglu_bwd(act, gu), (act.numel() + 2 * gu.numel()) * b2),
        ("rope on q and k, in place", lambda: KC.rope_inplace(qkv[..., :3, :], qkv[..., 3, :], fr), 2 * qkv[..., :4, :].numel() * b2),
        ("dropout-add fwd (p = 0.1)", lambda: KC.dropout_add_fwd(x, y, 0.1, 7), 3 * x.numel() * b2),
        ("dropout bwd", lambda: KC.dropout_add_bwd(x, 0.1, 7), 2 * x.numel() * b2),
        ("residual add", lambda: KC.add(x, y), 3 * x.numel() * b2),
        ("cross entropy: max / sum / target logit", lambda: KC.cross_entropy_local_stats(logits, tgt, 0), logits.numel() * b2),
        ("cross entropy: gradient in place", lambda: KC.cross_entropy_finish(logits, tgt, 0, m, s_, ones), 2 * logits.numel() * b2),
        ("AdamW (fp32 master, moments; bf16 weights out)", lambda: KC.adamw_step(p16, g32, m32, v32, w32, 1e-4, 0.9, 0.98, 1e-8, 0.01, 3),
         n * (4 * 4 + 3 * 4 + 2)),
        ("sum of squares (gradient norm)", lambda: KC.sumsq(g32), n * 4),
        ("embedding gather", lambda: KC.embedding_fwd(tok, emb, 0), 2 * tok.numel() * H * b2),
        ("embedding scatter-add (fp32 gradient)", lambda: KC.embedding_bwd(demb, tok, gemb, 0), tok.numel() * H * (b2 + 8)),
    ]
    print(f"| kernel | us | algorithmic MB | GB/s | of measured copy ({hbm:.0f} GB/s) |\n|---|---|---|---|---|")
    for name, fn, nbytes in cases:
        t = _timed(fn, flush)
        gbs = nbytes / t / 1e6
        print(f"| {name} | {t * 1e3:.0f} | {nbytes / 1e6:.0f} | {gbs:.0f} | {gbs / hbm:.2f} |")
    KC.check_status()


def attn_table() -> None:
    """Causal GQA flash attention at the 3B shapes (per nanobatch of 4 sequences): TP 1 (24/8 heads) and
    TP 8 (3/1 heads), forward and backward, vs the flash-attention wheel when it is installed."""
    from . import attention_cuda, cuda as KC
    dev = "cuda"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    print("| case | this library ms | TFLOP/s | wheel ms | TFLOP/s |\n|---|---|---|---|---|")
    for (s, b, g, rep) in [(4096, 4, 8, 3), (4096, 4, 1, 3), (16384, 1, 2, 3)]:
        d = 128
        packed = torch.randn(s, b, g, (rep + 2) * d, device=dev).bfloat16()
        q = packed[..., : rep * d].unflatten(-1, (rep, d))
        k = packed[..., rep * d:(rep + 1) * d]
        v = packed[..., (rep + 1) * d:]
        o, lse = attention_cuda.forward(q, k, v, d ** -0.5)
        do = torch.randn_like(o)
        fl_f = 4.0 * s * s * d * g * rep * b / 2
        t_f = _timed(lambda: attention_cuda.forward(q, k, v, d ** -0.5), flush)
        t_b = _timed(lambda: attention_cuda.backward(do, q, k, v, o, lse, d ** -0.5), flush)
        try:
            ol, lsel = KC.attention_fwd_library(q, k, v, d ** -0.5)
            w_f = _timed(lambda: KC.attention_fwd_library(q, k, v, d ** -0.5), flush)
            w_b = _timed(lambda: KC.attention_bwd_library(do, q, k, v, ol, lsel, d ** -0.5), flush)
        except Exception:
            w_f = w_b = float("nan")
        tag = f"S{s} B{b} heads {g * rep}/{g}"
        print(f"| fwd {tag} | {t_f:.3f} | {fl_f / t_f / 1e9:.0f} | {w_f:.3f} | {fl_f / w_f / 1e9:.0f} |")
        print(f"| bwd {tag} | {t_b:.3f} | {2.5 * fl_f / t_b / 1e9:.0f} | {w_b:.3f} | {2.5 * fl_f / w_b / 1e9:.0f} |")
    KC.check_status()


def fused_table() -> None:
    """The eight fused GEMM+collective kernels (QKV, FC1, out-proj, FC2 and their backward mirrors) at
    the 3B layer shapes for TP = world size: time (CUDA events, max over ranks), GEMM TFLOP/s, NVLink
    GB/s per direction and the fraction of max(FLOPs / measured GEMM peak, bytes / 770 GB/s)."""
    import json
    import os
    from pathlib import Path
    from types import SimpleNamespace
    import torch.distributed as dist
    from ..engine.context import OpContext
    from ..ops.fused import FusedAGDgrad, FusedAGGemm, FusedDgradRS, FusedGemmRS
    from ..parallel.mesh import init_distributed
    from ..parallel.symm_heap import SymmetricHeap
    from . import cuda as KC
    rank, world, local = init_distributed(timeout_s=120)
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    heap = SymmetricHeap.create(dist.group.WORLD, dev, size_bytes=3 << 30)
    if os.environ.get("KAREUS_NVLS", "0") == "1":      # multicast variants of the kernels
        mc_on = heap.enable_nvls(3 << 30)
        if rank == 0:
            print(f"NVLink-switch multicast: {'on' if mc_on else 'not supported, peer loads/stores'}")
    peak = 1669.2e12
    pk = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if pk.exists():
        peak = float(json.loads(pk.read_text()).get("bf16_tflops", 1669.2)) * 1e12
    sm = int(os.environ.get("KAREUS_COMM_SM", "12" if world >= 4 else "16"))
    # per-rank shapes of tensor-parallel degree `tp` (default: the number of ranks; KAREUS_TABLE_TP runs
    # another degree's shapes on this many ranks, e.g. the TP8 shapes on two GPUs)
    tp = int(os.environ.get("KAREUS_TABLE_TP", str(world)))
    reps = int(os.environ.get("KAREUS_TABLE_REPS", "10"))
    M, H, F, HEADS, KV, D = 16384, 3072, 8192, 24, 8, 128
    q_out, f_out = (HEADS + 2 * KV) * D // tp, 2 * F // tp
    # name -> (in_features, out_features, class, kind of collective, is backward)
    cases = [("qkv fwd: AG->GEMM", H, q_out, FusedAGGemm, "ag"), ("fc1 fwd: AG->GEMM", H, f_out, FusedAGGemm, "ag"),
             ("proj fwd: GEMM->RS", HEADS * D // tp, H, FusedGemmRS, "rs"),
             ("fc2 fwd: GEMM->RS", F // tp, H, FusedGemmRS, "rs"),
             ("qkv bwd: dgrad->RS", H, q_out, FusedDgradRS, "rs"), ("fc1 bwd: dgrad->RS", H, f_out, FusedDgradRS, "rs"),
             ("proj bwd: AG->dgrad", HEADS * D // tp, H, FusedAGDgrad, "ag"),
             ("fc2 bwd: AG->dgrad", F // tp, H, FusedAGDgrad, "ag")]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    if rank == 0:
        print(f"| kernel (TP{tp} shapes on {world} ranks, M={M}, {sm} comm CTAs, {reps} calls back to back) | N | K | us | "
              "GEMM TFLOP/s | "
              "NVLink GB/s/dir | roofline us (gemm, link) | fraction | plain GEMM us |\n|---|---|---|---|---|---|---|---|---|")
    for name, k_in, n_out, cls, kind in cases:
        w = (torch.randn(n_out, k_in, device=dev) * 0.02).bfloat16()
        w.main_grad = torch.zeros(n_out, k_in, device=dev)
        lin = SimpleNamespace(name="prof_" + name.split(":")[0].replace(" ", "_"), out_features=n_out,
                              in_features=k_in, weight=w)
        op = cls(lin, heap, sm)
        bwd = cls in (FusedDgradRS, FusedAGDgrad)
        # GEMM dims of the fused kernel itself (the backward's wgrad GEMM is a separate plain launch and is
        # excluded by timing a variant without saved input)
        red, out = (n_out, k_in) if bwd else (k_in, n_out)      # reduction dim, output features
        rows_in = M // world if kind == "ag" else M
        x = torch.randn(rows_in, 1, red, device=dev).bfloat16()

        # KAREUS_TABLE_PLANNED=1: the driver count is used as given (a plan's value); otherwise the
        # all-gather kernels scale it by their output width as they do in an unplanned run
        planned = os.environ.get("KAREUS_TABLE_PLANNED", "0") == "1"

        def call():
            if not bwd:
                ctx = OpContext()
                ctx.requires_grad = False
                op.run((x,), sm_num=sm, nb=0, ctx=ctx, planned=planned)
            elif cls is FusedDgradRS:
                op._gemm_rs(x.reshape(-1, red), w, out, True, 0, 0)      # whole SM budget, none left free
            else:
                op._ag_gemm(x.reshape(-1, red), w, out, True, sm, 0, planned)

        # `reps` calls back to back per sample: the ranks' GPUs do not start a sample at the same instant
        # (host skew after the barrier), and with a single call the early ranks' wait for the late one
        # would be charged to the kernel.  Inputs and outputs (100 MB each) do not stay in L2 between calls.
        times = []
        for i in range(9):
            flush.zero_()
            dist.barrier()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda._sleep(3_000_000)
            call()                      # absorbs the start skew
            a.record()
            for _ in range(reps):
                call()
            b.record()
            torch.cuda.synchronize()
            t = torch.tensor([a.elapsed_time(b) / reps], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            if i >= 3:
                times.append(t.item())
        times.sort()
        ms = times[len(times) // 2]
        # the same GEMM without any collective (whole GPU), for the cost of the communication inside the kernel
        xa = torch.randn(M, red, device=dev).bfloat16()
        plain = _timed(lambda: KC.gemm(xa, w, trans_b=not bwd), flush) * 1e3
        del xa
        flops = 2.0 * M * out * red
        link = (world - 1) / world * M * (red if kind == "ag" else out) * 2
        t_gemm, t_link = flops / peak * 1e6, link / 770e9 * 1e6
        if rank == 0:
            print(f"| {name} | {out} | {red} | {ms * 1e3:.0f} | {flops / 1e9 / ms:.0f} | {link / 1e6 / ms:.0f} | "
                  f"{t_gemm:.0f}, {t_link:.0f} | {max(t_gemm, t_link) / (ms * 1e3):.2f} | {plain:.0f} |", flush=True)
        del w, x
    KC.check_status()
    dist.barrier()
    heap.close()
    dist.destroy_process_group()


def collectives_table() -> None:
    """The heap's all-pairs collectives (plain peer loads/stores, no GEMM) on one nanobatch-sized tensor
    (16384 x 3072 bf16 = 100 MB) over a grid of launch shapes: time per call (five calls back to back, max
    over ranks) and bytes crossing NVLink per direction per second.  Shows what CTA count and block size a
    kernel needs to fill the links."""
    import torch.distributed as dist
    from ..parallel.mesh import init_distributed
    from ..parallel.symm_heap import SymmetricHeap
    from . import cuda as KC
    rank, world, local = init_distributed(timeout_s=120)
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    heap = SymmetricHeap.create(dist.group.WORLD, dev, size_bytes=2 << 30)
    M, H = 16384, 3072
    link = (world - 1) / world * M * H * 2
    if rank == 0:
        print(f"| collective ({world} ranks, {M}x{H} bf16) | CTAs | threads | us | NVLink GB/s/dir |\n|---|---|---|---|---|")
    for kind, shape in (("all_gather", (M // world, H)), ("reduce_scatter", (M, H)), ("all_reduce", (M, H))):
        best, table = heap.auto_tune(kind, shape, sm_candidates=(8, 16, 32, 64), block_candidates=(512, 1024), iters=5)
        factor = 2.0 if kind == "all_reduce" else 1.0
        if rank == 0:
            for (sm, blk), ms in sorted(table.items()):
                print(f"| {kind} | {sm} | {blk} | {ms * 1e3:.0f} | {factor * link / 1e6 / ms:.0f} |", flush=True)
    # NCCL on the same tensors, for the rate the library reaches on this box
    x = torch.ones(M, H, dtype=torch.bfloat16, device=dev)
    shard = torch.ones(M // world, H, dtype=torch.bfloat16, device=dev)
    out_full = torch.empty(M, H, dtype=torch.bfloat16, device=dev)
    for kind, fn, factor in (("nccl all_gather", lambda: dist.all_gather_into_tensor(out_full, shard), 1.0),
                             ("nccl reduce_scatter", lambda: dist.reduce_scatter_tensor(shard, x), 1.0),
                             ("nccl all_reduce", lambda: dist.all_reduce(x), 2.0)):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(5):
            fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / 5], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            print(f"| {kind} | - | - | {t.item() * 1e3:.0f} | {factor * link / 1e6 / t.item():.0f} |", flush=True)
    KC.check_status()
    dist.barrier()
    heap.close()
    dist.destroy_process_group()


# every command of this module: tables (CUDA events) and single-kernel cases (for a profiler capture)
CASES = ("collectives", "memory_table", "wgrad_sweep", "gemm_table", "attn_table", "fused", "gemm", "gemm_wgrad",
         "attn_fwd", "attn_bwd", "norm", "swiglu", "rope", "ce", "adamw", "step")


def main(case: str, reps: int = 3) -> None:
    if case not in CASES:
        raise SystemExit(f"unknown case {case!r}; one of: {', '.join(CASES)}")
    from . import cuda as KC
    dev = "cuda"
    if case == "collectives":
        return collectives_table()
    if case == "memory_table":
        return memory_table()
    if case == "wgrad_sweep":
        return wgrad_sweep()
    if case == "gemm_table":
        return gemm_table()
    if case == "attn_table":
        return attn_table()
    if case == "fused":
        return fused_table()
    if case == "gemm":
        a = torch.randn(8192, 8192, device=dev).bfloat16()
        b = torch.randn(8192, 8192, device=dev).bfloat16()
        for _ in range(reps):
            KC.gemm(a, b)
    elif case == "gemm_wgrad":
        dy = torch.randn(16384, 3072, device=dev).bfloat16()
        x = torch.randn(16384, 8192, device=dev).bfloat16()
        acc = torch.zeros(3072, 8192, device=dev)
        for _ in range(reps):
            KC.gemm(dy, x, trans_a=True, trans_b=False, accumulate=acc)
    elif case in ("attn_fwd", "attn_bwd"):
        from . import attention_cuda
        s, b, g, rep, d = 4096, 4, 1, 3, 128
        packed = torch.randn(s, b, g, (rep + 2) * d, device=dev).bfloat16()
        q = packed[..., : rep * d].unflatten(-1, (rep, d))
        k = packed[..., rep * d:(rep + 1) * d]
        v = packed[..., (rep + 1) * d:]
        for _ in range(reps):
            o, lse = attention_cuda.forward(q, k, v, d ** -0.5)
        if case == "attn_bwd":
            do = torch.randn_like(o)
            for _ in range(reps):
                attention_cuda.backward(do, q, k, v, o, lse, d ** -0.5)
    elif case == "norm":
        x = torch.randn(65536, 3072, device=dev).bfloat16()
        w = torch.ones(3072, device=dev).bfloat16()
        for _ in range(reps):
            y, r = KC.rmsnorm_fwd(x, w, 1e-5)
            KC.rmsnorm_bwd(y, x, r, w)
    elif case == "swiglu":
        x = torch.randn(32768, 16384, device=dev).bfloat16()
        for _ in range(reps):
            y = KC.swiglu_fwd(x)
            KC.swiglu_bwd(y, x)
    elif case == "rope":
        t = torch.randn(4096, 8, 8, 5, 128, device=dev).bfloat16()
        from . import ref
        fr = ref.rope_table(4096, 128, 500000.0, device=dev)
        for _ in range(reps):
            KC.rope_inplace(t[..., :3, :], t[..., 3, :], fr)
    elif case == "ce":
        logits = torch.randn(8192, 128256, device=dev).bfloat16()
        tgt = torch.randint(0, 128256, (8192,), device=dev)
        for _ in range(reps):
            m, s_, t_ = KC.cross_entropy_local_stats(logits, tgt, 0)
            KC.cross_entropy_finish(logits, tgt, 0, m, s_, torch.ones_like(m))
    elif case == "adamw":
        n = 256 * 1024 * 1024
        g = torch.randn(n, device=dev)
        m = torch.zeros(n, device=dev)
        v = torch.zeros(n, device=dev)
        w = torch.randn(n, device=dev)
        p = w.bfloat16()
        for i in range(reps):
            KC.adamw_step(p, g, m, v, w, 1e-3, 0.9, 0.98, 1e-8, 0.01, i + 1)
    elif case == "step":
        # one training step of a 2-layer model with the 3B layer shape (1 microbatch of 8 x 4096)
        from ..config import ParallelConfig, TrainConfig, get_model_config
        from ..train.trainer import Trainer, synthetic_batch
        cfg = get_model_config("llama3.2_3b").replace(num_layers=2, vocab_size=32768)
        tc = TrainConfig(micro_batch_size=8, global_batch_size=8, seq_len=4096, warmup_steps=0)
        tr = Trainer(cfg, ParallelConfig(num_nanobatches=2, recompute=True), tc, device=dev, recompute_layers=2)
        batch = synthetic_batch(cfg, tc, 1, seed=0)
        for _ in range(reps):
            tr.train_step(batch)
    else:
        raise SystemExit(f"unknown case {case!r}")
    torch.cuda.synchronize()
    KC.check_status()
    print(f"{case}: ok")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "gemm")
