"""Per-clock time/energy of the parts of a stage that are not transformer-layer partitions:
embedding forward/backward, final norm + output projection forward/backward, and the loss.

Output layout (reference ``tests/bayesian/nonpartition/profile_nonpartition.py:92-111,148-473``):
``nonpartition/<freq>/{preprocess,preprocess_backward,postprocess,postprocess_backward,loss}_energy.csv``
with header ``time (s),total_energy (J),per_rank_energy (J)``.
"""
from __future__ import annotations

from pathlib import Path
from typing import Callable, Dict, Optional, Sequence

import torch

from .. import kernels as K
from ..energy.monitor import EnergyMonitor, measure

FILES = {"preprocess": "preprocess_energy.csv", "preprocess_backward": "preprocess_backward_energy.csv",
         "postprocess": "postprocess_energy.csv", "postprocess_backward": "postprocess_backward_energy.csv",
         "loss": "loss_energy.csv"}


def build_cases(model, micro_batch_size: int, seq_len: int, device) -> Dict[str, Callable[[], None]]:
    """Closures over one nanobatch-sized input of ``model`` (a first+last stage ``GPTModel``)."""
    cfg, n = model.cfg, model.n
    b = max(1, micro_batch_size // n)
    tok = torch.randint(0, cfg.vocab_size, (seq_len, b), device=device)
    emb, head = model.embedding, model.output_layer
    h = torch.randn(seq_len, b, cfg.hidden_size, device=device).to(emb.weight.dtype)
    from ..ops.basic import ensure_main_grad
    gw_e, gw_h = ensure_main_grad(emb.weight), ensure_main_grad(head.weight)
    x2 = h.reshape(-1, cfg.hidden_size)
    logits = K.gemm(x2, head.weight, trans_b=True)
    tgt = tok.reshape(-1)
    ones = torch.ones(tgt.numel(), device=device)

    def preprocess():
        K.embedding_fwd(tok, emb.weight, emb.vocab_start)

    def preprocess_backward():
        K.embedding_bwd(h, tok, gw_e, emb.vocab_start)

    def postprocess():
        y, _ = K.rmsnorm_fwd(x2, model.final_norm.weight, cfg.norm_eps)
        K.gemm(y, head.weight, trans_b=True)

    def loss():
        m, s, t = K.cross_entropy_local_stats(logits, tgt, head.vocab_start)
        K.cross_entropy_finish(logits, tgt, head.vocab_start, m, s, ones)

    def postprocess_backward():
        K.gemm(logits, head.weight, trans_b=False)
        K.gemm(logits, x2, trans_a=True, trans_b=False, accumulate=gw_h)

    return {"preprocess": preprocess, "preprocess_backward": preprocess_backward, "postprocess": postprocess,
            "postprocess_backward": postprocess_backward, "loss": loss}


def profile_nonpartition(cases: Dict[str, Callable[[], None]], freqs: Sequence[int], out_dir, monitor: EnergyMonitor,
                         controller=None, world_size: int = 1, measurement_duration: float = 2.0,
                         cooldown_duration: float = 1.0, group=None, sleep_fn=None) -> None:
    import time
    sleep_fn = sleep_fn or time.sleep
    for f in freqs:
        if controller is not None:
            controller.set_frequency(f)
        d = Path(out_dir) / "nonpartition" / str(f)
        d.mkdir(parents=True, exist_ok=True)
        for name, fn in cases.items():
            tr = measure(fn, monitor, measurement_duration, cooldown_duration, group=group, sleep_fn=sleep_fn)
            (d / FILES[name]).write_text("time (s),total_energy (J),per_rank_energy (J)\n"
                                         f"{tr.time_per_iter},{tr.energy_per_iter},{tr.energy_per_iter / world_size}\n")
