"""Host logic of bench.py that needs no GPU: the summary of the clock samples."""
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _bench():
    argv, sys.argv = sys.argv, ["bench.py"]
    try:
        if str(ROOT) not in sys.path:
            sys.path.insert(0, str(ROOT))
        import bench
        return bench
    finally:
        sys.argv = argv


def test_clock_samples_are_summarised_over_the_timed_region_only():
    bench = _bench()
    s = bench.ClockSampler(0)            # no GPU here: neither NVML nor nvidia-smi deliver anything
    s.stop_flag = True
    t0 = time.time()
    assert s.inside(t0, t0 + 1) == 0
    assert s.stop(t0, t0 + 1)["samples"] == 0 and s.stop(t0, t0 + 1)["sm_mhz"] is None
    s.samples = [(t0 - 0.5, 300, 1965, []),                       # idle before the region: not counted
                 (t0 + 0.01, 1965, 1965, []), (t0 + 0.02, 1950, 1965, ["sw_power_cap"]), (t0 + 0.03, 1965, 1965, []),
                 (t0 + 2.0, 500, 1965, ["hw_slowdown"])]          # after it: not counted either
    assert s.inside(t0, t0 + 0.05) == 3
    out = s.stop(t0, t0 + 0.05, "note")
    assert out["sm_mhz"] == 1965 and out["sm_max_mhz"] == 1965 and out["samples"] == 3
    assert out["reasons"] == ["sw_power_cap"] and out["note"] == "note"
