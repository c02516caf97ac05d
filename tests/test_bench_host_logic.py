"""Host-side arithmetic of bench.py that can be checked without a GPU: the per-layer roofline from a count
table, the clock sampler's window filter, the workload descriptions."""
import datetime
import time
import types

import torch

import bench


def test_layer_roofline_from_a_count_table():
    env = types.SimpleNamespace(world=2, peaks={"bf16_tflops_sustained": 1000.0, "hbm_gbs": 5000.0})
    c = bench.CONFIGS["c2"]
    d, h, E = c["d_model"], c["d_hidden"], c["experts_per_gpu"]
    # table[src, dst, expert]: rank 0 sends 2000 rows per expert to each rank, rank 1 sends 1000
    table = torch.zeros(2, 2, E, dtype=torch.int64)
    table[0] += 2000
    table[1] += 1000
    B = 3000 * E                                           # rows each GPU's experts process
    r = bench.layer_roofline(env, "c2", table, ms_per_step=1.0)
    assert r["busiest_gpu_rows"] == B
    assert abs(r["t_tensor_ms"] - 12.0 * B * d * h / 1e15 * 1e3) < 1e-12
    hbm = 2.0 * (8 * B * d + 8 * B * h) + 12.0 * E * d * h
    assert abs(r["t_hbm_ms"] - hbm / 5e12 * 1e3) < 1e-12
    # the busier direction of the busier GPU: rank 0 sends 2000 E rows away, rank 1 receives them
    assert abs(r["t_nvlink_ms"] - 4.0 * 2000 * E * d * 2.0 / (bench.NVLINK_GBS * 1e9) * 1e3) < 1e-12
    assert r["bound"] == "tensor" and abs(r["frac"] - r["t_tensor_ms"] / 1.0) < 1e-12
    single = bench.layer_roofline(types.SimpleNamespace(world=1, peaks=env.peaks), "c2", table[:1, :1], 1.0)
    assert single["t_nvlink_ms"] == 0.0
    small = bench.layer_roofline(env, "c2", table // 100, ms_per_step=1.0)
    assert small["bound"] == "hbm"                         # few rows: reading the weights dominates


class _Done:
    def terminate(self):
        pass

    def wait(self, timeout=None):
        pass

    def kill(self):
        pass


def _stamp(t):
    return datetime.datetime.fromtimestamp(t).strftime("%Y/%m/%d %H:%M:%S.%f")[:-3]


def test_clock_sampler_keeps_the_samples_of_the_timed_window():
    now = time.time()
    quiet = ["Not Active"] * 4
    s = bench.ClockSampler(0)
    s.proc = _Done()
    s.rows = [[_stamp(now - 2.0), "1200", "1965", "200"] + quiet,
              [_stamp(now - 0.5), "1800", "1965", "900", "Not Active", "Not Active", "Not Active", "Active"],
              [_stamp(now - 0.4), "1700", "1965", "950", "Not Active", "Not Active", "Not Active", "Active"],
              ["garbage"]]
    got = s.stop(now - 0.6, now)
    assert got == {"sm_mhz": 1750.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"], "samples": 2,
                   "window": "timed region"}
    s.proc = _Done()
    got = s.stop(now + 10, now + 11)                       # no sample inside: everything taken under load
    assert got["samples"] == 3 and got["window"] == "whole run under load" and got["sm_mhz"] == 1700.0
    s.proc, s.rows = _Done(), []
    assert s.stop(now - 1, now) is None


def test_workload_descriptions_name_no_model():
    for name in bench.CONFIGS:
        w = bench.workload_config(name, 8)
        assert "workload" in w and "model" not in w and w["parallelism"] == "ep8"
        assert w["tokens_per_gpu"] == bench.CONFIGS[name]["tokens_per_gpu"]
