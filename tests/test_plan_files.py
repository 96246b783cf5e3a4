"""Plan-file contracts: config strings, both layouts, emit∘parse identity, scheduler checks, and a
round trip over every plan file shipped with the reference (when that checkout is present)."""
import os
from pathlib import Path

import pytest

from kareus_b200.plan import (CommConfig, PipelineCommScheduler, emit_freqs_text, emit_schedule_text,
                              parse_config_string, parse_freqs_text, parse_schedule_text, read_trailer,
                              sample_frontier, uniform_schedule)

REF = Path(os.environ.get("KAREUS_REFERENCE_DIR", "/nonexistent")) / "tests"

SCHED = """
[
[('forward', 'norm_0-none-12-1024', 'norm_0-none-18-1024'), ('backward', 'attn_0-none-21-1024', 'norm_0-none-15-1024', 'rope_0-none-30-1024', 'activation_0-none-15-1024')],
[('forward', 'norm_0-none-27-1024', 'norm_0-none-27-1024'), ('backward', 'rope_0-none-6-1024', 'norm_0-none-21-1024', 'rope_0-none-21-1024', 'activation_0-none-15-1024')],
]
# Iteration 324 cost change: 0.0227579757019285
# Iteration 324 total cost: 1224.8441048803174
# Iteration 324 total cost with P2P: 2333.9241048803174
"""


def test_config_strings():
    c = parse_config_string("norm_0-none-12-1024")
    assert c == CommConfig(("norm_0", "none"), (12, 1024)) and c.to_string() == "norm_0-none-12-1024"
    assert parse_config_string("-1--1-16-1024") == CommConfig((-1, -1), (16, 1024))
    assert parse_config_string("0-8-16-1024").overlap_window == (0, 8)
    for bad in ("norm_0-12-1024", "a-b-c-d", ""):
        with pytest.raises(ValueError):
            parse_config_string(bad)


def test_checkpointing_layout_round_trip():
    plan = parse_schedule_text(SCHED, True, False)
    assert len(plan) == 2 and plan[0][0].kind == "forward" and plan[0][1].kind == "backward"
    assert plan[0][0].fwd_attn.sm_num == 12 and plan[0][0].bwd_mlp is None
    assert plan[0][1].bwd_attn.start == "rope_0" and plan[0][1].fwd_attn.start == "attn_0"     # recompute keys
    assert plan[1][0].fwd_trail.resource_shape == (20, 1024)
    tr = read_trailer(SCHED)
    text = emit_schedule_text(plan, True, int(tr["iteration"]), tr["cost_change"], tr["total_cost"], tr["total_cost_p2p"])
    assert parse_schedule_text(text, True, False) == plan
    assert read_trailer(text) == tr
    # sequence-parallel keys inherit the launch shape, not the slot, of their parent key
    ag = plan[0][0].get("fwd_attn_ag")
    assert ag.start == "first" and ag.resource_shape == (12, 1024)


def test_pair_layout_and_cp_layout():
    pair = "[[(('forward','norm_0-none-3-1024','norm_0-none-6-1024'),('backward','rope_0-none-9-1024','norm_0-none-3-1024'))]]"
    p = parse_schedule_text(pair, False, False)
    assert p[0][0].kind == "both" and p[0][0].bwd_attn.sm_num == 9
    assert parse_schedule_text(emit_schedule_text(p, False), False, False) == p
    cp = uniform_schedule(2, ["forward", "backward"], context_parallel=True)
    text = emit_schedule_text(cp, True)
    back = parse_schedule_text(text, True, True)
    assert back == cp and len(back[0][1].as_dict()) == 12
    with pytest.raises(TypeError):
        parse_schedule_text("[[('forward', 'norm_0-none-3-1024')]]", True, False)
    with pytest.raises(ValueError):
        parse_schedule_text("[[('sideways', 'a-b-1-2', 'a-b-1-2')]]", True, False)
    with pytest.raises(ValueError):
        parse_schedule_text("import os", True, False)          # not a literal: never evaluated


def test_scheduler_consumption_checks():
    plan = uniform_schedule(1, ["forward", "forward", "backward", "backward"])
    s = PipelineCommScheduler.from_parsed(plan, 0, 2, use_activation_checkpointing=True)
    s.on_instruction_begin("forward")
    with pytest.raises(RuntimeError):
        s.on_instruction_begin("backward")        # plan says forward
    s.on_instruction_begin("forward")
    with pytest.raises(RuntimeError):
        s.on_step_end()                            # two items left
    s.on_instruction_begin("backward"); s.on_instruction_begin("backward")
    s.on_step_end()
    with pytest.raises(ValueError):
        PipelineCommScheduler.from_parsed(plan, 0, 3, use_activation_checkpointing=True)
    with pytest.raises(IndexError):
        PipelineCommScheduler.from_parsed(plan, 1, 2, use_activation_checkpointing=True)


def test_frontier_sampling_rule():
    names = [f"freqs_pipeline_{i:05d}.py" for i in range(2496)]
    kept = sample_frontier(names)
    assert len(kept) == 10 and kept[-1] == "freqs_pipeline_02495.py"
    idx = [int(k[15:20]) for k in kept]
    assert idx == [324, 658, 992, 1326, 1660, 1827, 1994, 2161, 2328, 2495]       # the reference's shipped frontier


@pytest.mark.skipif(not REF.exists(), reason="reference checkout not present")
def test_round_trip_every_shipped_plan_file():
    files = sorted(REF.glob("*/schedules/**/*pipeline_*.py"))
    assert len(files) > 100
    n_sched = 0
    for f in files:
        text = f.read_text()
        tr = read_trailer(text)
        args = (int(tr["iteration"]), tr["cost_change"], tr["total_cost"], tr["total_cost_p2p"]) if tr else ()
        if f.name.startswith("freqs_"):
            plan = parse_freqs_text(text)
            assert parse_freqs_text(emit_freqs_text(plan, *args)) == plan
        else:
            cp = "cp2" in str(f)
            plan = parse_schedule_text(text, True, cp)
            assert parse_schedule_text(emit_schedule_text(plan, True, *args), True, cp) == plan
            n_sched += 1
        if tr:
            assert read_trailer(emit_freqs_text([[("forward", 900)]], *args)) == tr
    assert n_sched >= 10
