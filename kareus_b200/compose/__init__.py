"""Offline plane, CPU only: frontier composer, time–cost solver, plan driver, comparison tools."""
from .composer import compose, generate_profile_csv, pareto_optimal, layers_per_stage, read_bo_jsonl
from .solver import ExecutionOption, PhillipsDessouky, plan_pipeline
from .driver import run_optimization
from .compare import compare_frontiers, dominates, frontier_from_plans, summarize_run
