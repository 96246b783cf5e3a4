"""Small, self-terminating workloads of each hot kernel for profiler captures.

    python -m kareus_b200.kernels.profile_cases gemm        # 8192 x 8192 x 8192 bf16, 3 launches
    python -m kareus_b200.kernels.profile_cases attn_fwd    # B4 H3 S4096 d128 causal, 3 launches
    python -m kareus_b200.kernels.profile_cases norm | swiglu | ce | adamw | rope

Each case touches more than the 126 MB L2 where DRAM figures matter but holds at most a few GB,
and launches its kernel a handful of times so a ``--set full`` capture ends within minutes.
"""
from __future__ import annotations

import sys

import torch


def main(case: str, reps: int = 3) -> None:
    from . import cuda as KC
    dev = "cuda"
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
