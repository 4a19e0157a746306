"""Host-side pieces of bench.py that need no GPU: the operation count, the clock record and the choice of the
roofline denominator."""
import sys
import time
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
import bench  # noqa: E402


def test_attn_ops_counts_attended_keys_and_the_sink():
    # brute force over the mask of the reference's model (new_block.py:205-213): key j < i, j >= i - W', plus the sink
    for S, W in ((64, 0), (96, 16), (200, 48), (257, 40)):
        w = None if W == 0 else ((W - 1) // 16 + 1) * 16
        n = 0
        for i in range(S):
            lo = 0 if w is None else max(0, i - w)
            n += (i - lo) + 1
        assert bench.attn_ops(2, 3, 32, S, W) == 4.0 * 2 * 3 * 32 * n


def _sampler_with(nvml, smi_lines=()):
    s = bench.ClockSampler(0)
    s.nvml = list(nvml)
    s.lines = list(smi_lines)
    return s


def test_clock_record_uses_the_samples_inside_the_timed_region():
    t0 = time.time()
    cap = bench.ClockSampler.BITS["sw_power_cap"]
    nvml = [(t0 - 1.0, 1200, 1965, 300.0, bench.ClockSampler.BITS["hw_slowdown"]),   # before the region: ignored
            (t0 + 0.010, 1965, 1965, 700.0, 0),
            (t0 + 0.015, 1800, 1965, 740.0, cap),
            (t0 + 0.020, 1807, 1965, 742.0, cap),
            (t0 + 5.0, 900, 1965, 100.0, 0)]                                          # after it: ignored
    rec = _sampler_with(nvml).stop(t0, t0 + 0.03)
    assert rec["samples"] == 3 and rec["source"].startswith("nvml")
    assert rec["sm_mhz"] == 1807.0 and rec["sm_mhz_lowest"] == 1800.0 and rec["sm_mhz_highest"] == 1965.0
    assert rec["sm_max_mhz"] == 1965.0 and rec["power_w_max"] == 742.0
    assert rec["reasons"] == ["sw_power_cap"] and rec["nvml_reason_bits"] == hex(cap)


def test_clock_record_falls_back_to_nvidia_smi_lines():
    import datetime
    t0 = time.time()
    stamp = lambda t: datetime.datetime.fromtimestamp(t).strftime("%Y/%m/%d %H:%M:%S.%f")[:-3]
    lines = [f"{stamp(t0 + 0.01)}, 1965, 1965, 410.5, Not Active, Not Active, Not Active, Active",
             f"{stamp(t0 + 0.11)}, 1950, 1965, 420.0, Not Active, Not Active, Not Active, Not Active",
             "garbage"]
    rec = _sampler_with([], lines).stop(t0, t0 + 0.2)
    assert rec["samples"] == 2 and rec["samples_nvidia_smi"] == 2 and rec["source"].startswith("nvidia-smi")
    assert rec["sm_mhz"] == 1957.5 and rec["reasons"] == ["sw_power_cap"]


class _Tensor:
    bound, dtype, units = "tensor", "s8", 1


def test_roofline_denominator_follows_the_load_condition():
    peaks = {"hbm_gbs": 6540.8, "bf16_burst": 1670.8, "bf16_sustained": 1424.4, "source": "measured"}
    # short region, no cap in the clock record: burst
    r = bench.roofline(_Tensor(), 900.0, 0.03, peaks, {}, "none", {"reasons": []})
    assert r["peak"] == 2 * 1670.8 and "burst" in r["peak_source"]
    # the same region with the power cap active: sustained
    r = bench.roofline(_Tensor(), 845.0, 0.03, peaks, {}, "none", {"reasons": ["sw_power_cap"]})
    assert r["peak"] == 2 * 1424.4 and "sustained" in r["peak_source"]
    assert abs(r["frac"] - 845.0 / 2848.8) < 1e-12
    assert abs(r["frac_of_burst"] - 845.0 / 3341.6) < 1e-12 and abs(r["frac_of_sustained"] - r["frac"]) < 1e-12
    # a region that, with the load in front of it, lasts a second: sustained
    r = bench.roofline(_Tensor(), 845.0, 0.6, peaks, {}, "none", {"reasons": []})
    assert r["peak"] == 2 * 1424.4


def test_measured_peaks_file_or_fallback():
    p = bench.measured_peaks()
    assert p["hbm_gbs"] > 1000 and p["bf16_burst"] >= p["bf16_sustained"] > 100
    assert np.isfinite(p["bf16_burst"])
