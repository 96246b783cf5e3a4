"""Online energy plane against a simulated NVML: windows, measure(), clock control, plan server."""
import json
import time

import pytest

from kareus_b200.energy import (EnergyMonitor, FakeNVML, FrequencyController, GpuStatsMonitor, PFOServer,
                                PipelineFrequencyOptimizer, PointSolution, PowerMonitor, measure)
from kareus_b200.energy.nvml import decode_throttle
from kareus_b200.plan import emit_freqs_text, parse_freqs_text


class Clock:
    def __init__(self):
        self.t = 0.0

    def __call__(self):
        return self.t


def test_windows_nest_and_log(tmp_path):
    clk = Clock()
    nv = FakeNVML(n=2, time_fn=clk)
    log = tmp_path / "zeus_monitor_global_rank-0_local_rank-0.txt"
    mon = EnergyMonitor([0, 1], log_file=str(log), nvml=nv, sync_fn=lambda idx: None, time_fn=clk)
    mon.begin_window("training_step")
    clk.t += 1.0
    mon.begin_window("training_step_fwd_bwd_step_call")
    clk.t += 2.0
    inner = mon.end_window("training_step_fwd_bwd_step_call")
    clk.t += 0.5
    outer = mon.end_window("training_step")
    assert inner.time == pytest.approx(2.0) and outer.time == pytest.approx(3.5)
    assert inner.gpu_energy[0] == pytest.approx(2000.0, rel=1e-3)       # 1000 W at max clock
    assert outer.total_energy == pytest.approx(7000.0, rel=1e-3)
    rows = log.read_text().strip().splitlines()
    assert rows[0] == "start_time,window_name,elapsed_time,gpu0_energy,gpu1_energy"
    assert rows[1].split(",")[1] == "training_step_fwd_bwd_step_call"
    with pytest.raises(ValueError):
        mon.end_window("never_opened")


def test_measure_counts_iterations():
    clk = Clock()
    nv = FakeNVML(n=1, time_fn=clk)
    mon = EnergyMonitor([0], nvml=nv, sync_fn=lambda idx: None, time_fn=clk)

    def work():
        clk.t += 0.25

    trial = measure(work, mon, measurement_duration=2.0, cooldown_duration=0.0)
    assert trial.iterations == 8
    assert trial.time_per_iter == pytest.approx(0.25)
    assert trial.energy_per_iter == pytest.approx(250.0, rel=1e-3)


def test_frequency_controller_modes():
    nv = FakeNVML(n=1)
    off = FrequencyController(0, "off", nvml=nv)
    off.set_frequency(1200)
    assert nv.calls == [] and off.history == []
    adv = FrequencyController(0, "advisory", nvml=nv)
    adv.set_frequency(1200)
    assert nv.calls == [] and adv.history[-1][1] == 1200
    with FrequencyController(0, "locked", nvml=nv) as ctl:
        ctl.set_frequency(1500)
        ctl.set_frequency(1350)
        assert ctl.wait_idle()
        assert nv.locked[0] == 1350
    assert nv.calls[-1] == ("reset", 0) and nv.locked[0] is None
    # lower clock => lower simulated power
    assert nv.power_w(0) == pytest.approx(1000.0)


def test_frequency_controller_without_permission_degrades():
    nv = FakeNVML(n=1, deny_clock_control=True)
    ctl = FrequencyController(0, "locked", nvml=nv)
    ctl.set_frequency(1200)
    ctl.wait_idle()
    time.sleep(0.05)
    assert ctl.mode == "advisory" and ctl.errors and nv.calls == []
    ctl.close()


PLAN = [[("forward", 1500), ("forward", 1400), ("backward", 1300), ("backward", 1200)],
        [("forward", 1100), ("backward", 1000), ("forward", 900), ("backward", 900)]]


def _client(pp_rank, ctl, **kw):
    return PipelineFrequencyOptimizer(rank=pp_rank, dp_rank=0, pp_rank=pp_rank, tp_rank=0, device_id=0, dp_degree=1,
                                      pp_degree=2, tp_degree=1, world_size=2, controller=ctl, **kw)


def test_pfo_in_process_and_http():
    text = emit_freqs_text(PLAN, iteration=7, cost_change=0.1, total_cost=10.0, total_cost_p2p=20.0)
    plan = parse_freqs_text(text)
    assert plan == PLAN
    sol = PointSolution(plan)
    ctl = FrequencyController(0, "advisory")
    c = _client(1, ctl, solution=sol)
    c.on_step_begin()
    for name in ("forward", "backward", "forward", "backward"):
        c.on_instruction_begin(name)
        c.on_instruction_end(name)
    c.on_step_end()
    assert [f for _, f in ctl.history] == [1100, 1000, 900, 900]
    c.on_step_begin()
    with pytest.raises(RuntimeError):
        c.on_instruction_begin("backward")        # plan says forward first

    srv = PFOServer(sol, port=0).start()
    try:
        ctl2 = FrequencyController(0, "advisory")
        h = _client(0, ctl2, server_url=srv.url)
        h.on_step_begin()
        h.on_instruction_begin("forward")
        assert ctl2.history[-1][1] == 1500 and 0 in sol.registered
    finally:
        srv.stop()


def test_pfo_server_down_falls_back_to_max_clock():
    ctl = FrequencyController(0, "advisory")
    c = _client(0, ctl, server_url="http://127.0.0.1:9", timeout_s=0.2)
    assert c.fallback
    c.on_step_begin()
    c.on_instruction_begin("forward")
    c.on_step_end()
    assert ctl.history == []


def test_samplers_record_change_points():
    nv = FakeNVML(n=1)
    pm = PowerMonitor(0, update_period=0.005, nvml=nv).start()
    gs = GpuStatsMonitor(0, period_s=0.005, nvml=nv).start()
    time.sleep(0.03)
    nv.set_locked_clocks(0, 1200, 1200)
    time.sleep(0.03)
    pm.stop(); gs.stop()
    assert len(pm.get_power_timeline()) >= 4
    assert [c for _, c in gs.clock_changes] == [1965, 1200]
    assert decode_throttle(0x4 | 0x40) == ["sw_power_cap", "hw_thermal_slowdown"]
