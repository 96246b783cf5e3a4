"""Phase 2a: compose partition profiles into per-stage candidates (``profile_<model>_...csv``).

    python -m kareus_b200.cli.run_compose --model_name llama3.2_3b --tensor_parallel_size 8 \
        --context_parallel_size 1 --pipeline_parallel_size 2 --batch_size 8 --seq_len 4096
"""
from __future__ import annotations

import argparse


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model_name", required=True)
    ap.add_argument("--tensor_parallel_size", type=int, required=True)
    ap.add_argument("--context_parallel_size", type=int, default=1)
    ap.add_argument("--pipeline_parallel_size", type=int, default=1)
    ap.add_argument("--batch_size", type=int, required=True)
    ap.add_argument("--seq_len", type=int, required=True)
    ap.add_argument("--bayesian_profile_dir", default=".")
    ap.add_argument("--prepost_profile_dir", default=None)
    ap.add_argument("--output_dir", default=".")
    ap.add_argument("--gpu_type", default="B200")
    ap.add_argument("--no_activation_checkpointing", action="store_true")
    ap.add_argument("--no_scale_time_energy", action="store_true")
    ap.add_argument("--nanobatches", type=int, default=2)
    a = ap.parse_args(argv)
    from ..compose.composer import generate_profile_csv
    out = generate_profile_csv(a.model_name, a.tensor_parallel_size, a.context_parallel_size,
                               a.pipeline_parallel_size, a.batch_size, a.seq_len, a.bayesian_profile_dir,
                               a.prepost_profile_dir, a.output_dir, a.gpu_type, not a.no_activation_checkpointing,
                               not a.no_scale_time_energy, a.nanobatches)
    print(f"Profile CSV saved: {out}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
