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


def test_recorded_dram_traffic_is_tied_to_kernel_sources_and_workload(tmp_path, monkeypatch):
    """roofline.traffic comes from a recorded ncu capture; it is reported only for the kernel sources and workload it was taken
    from, otherwise None with the reason."""
    import json
    b = _bench()
    w = dict(b.WORKLOAD)
    rec = {"kernel_source_sha256": b.kernel_source_digest(), "workload": {k: w[k] for k in ("B", "S", "H", "Hkuv", "Dh", "E", "De")},
           "dram_bytes_per_launch": {"bwd_dw_kernel": 2.0e8}, "command": "ncu ..."}
    f = tmp_path / "t.json"
    f.write_text(json.dumps(rec))
    monkeypatch.setattr(b, "TRAFFIC_FILE", str(f))
    assert b.recorded_traffic("bwd_dw_kernel", w)[0] == 2.0e8
    assert b.recorded_traffic("fwd_kernel", w)[0] is None
    assert b.recorded_traffic("bwd_dw_kernel", dict(w, B=2)) == (None, "recorded capture is of another workload")
    rec["kernel_source_sha256"] = "0" * 64
    f.write_text(json.dumps(rec))
    assert b.recorded_traffic("bwd_dw_kernel", w) == (None, "recorded capture is of older kernel sources")
    assert b.choose_peak({"burst": 2.0, "sustained": 1.0}, 0.05) == ("burst", 2.0)
    assert b.choose_peak({"burst": 2.0, "sustained": 1.0}, 2.5) == ("sustained", 1.0)


def test_both_arms_print_the_same_config():
    b = _bench()
    assert b.workload_config(b.WORKLOAD, 1) == b.workload_config(dict(b.WORKLOAD), 1)
    assert "tokens_per_s" not in b.workload_config(b.WORKLOAD, 1)     # a description of the workload, no measured values
