"""CPU: the pieces of bench.py that do not need a GPU -- FLOP accounting, the peaks file, the clock sampler's parser."""
import importlib.util
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    m = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = m
    spec.loader.exec_module(m)
    return m


def test_algorithmic_flops_of_the_workload():
    b = _bench()
    w = b.WORKLOAD
    fl = b.alg_flops(w["B"], w["S"], w["H"], w["Dh"], w["E"], w["De"])
    assert fl == 18 * 32768 * 8 * 2816 * 128                      # 18 * T * H * I * d_h
    assert abs(fl - 1.70e12) / 1.70e12 < 0.01                      # the per-layer figure of the 370M configuration
    assert b.alg_flops(1, 1, 1, 1, 1, 1, passes=6) == 6


def test_peaks_have_the_three_denominators():
    p = _bench().measured_peaks()
    assert p["source"] in ("measured", "fallback")
    assert 1000 < p["sustained"] <= p["burst"] < 2300 and 5000 < p["hbm"] < 8100


def test_clock_sampler_parses_nvidia_smi_lines():
    b = _bench()
    s = b.ClockSampler(0)
    s.proc = type("P", (), {"terminate": lambda self: None})()
    s.lines = ["1965, 1965, 512.3, Not Active, Not Active, Not Active, Not Active",
               "1680, 1965, 998.1, Not Active, Not Active, Not Active, Active",
               "1665, 1965, 1001.7, Not Active, Not Active, Not Active, Active",
               "garbage line", "[N/A], 1965, 1.0, Not Active, Not Active, Not Active, Not Active"]
    r = s.stop()
    assert r["sm_mhz"] == 1680.0 and r["sm_max_mhz"] == 1965.0 and r["samples"] == 3
    assert r["reasons"] == ["sw_power_cap"] and r["power_w"] == 998.1
    s2 = b.ClockSampler(0)
    assert s2.stop()["sm_mhz"] is None                             # never started: reported as unavailable, not as zero
