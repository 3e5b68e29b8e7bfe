"""Host-side pieces of bench.py that need no GPU: the clock-record summary and the CPU answer."""
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("ka_bench", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class _Done:
    def terminate(self):
        pass

    def wait(self, timeout=None):
        return 0


def test_clock_summary_uses_samples_of_the_timed_window_and_names_reasons():
    bench = _bench()
    cs = bench.ClockSampler(0)
    cs.proc = _Done()
    cs.lines = [
        (10.0, "1965, 1965, 300.0, Not Active, Not Active, Not Active, Not Active"),     # before the window
        (20.0, "1350, 1965, 990.0, Not Active, Not Active, Not Active, Active"),
        (20.1, "1290, 1965, 1001.0, Not Active, Not Active, Not Active, Active"),
        (20.2, "1320, 1965, 998.0, Not Active, Not Active, Not Active, Active"),
        (30.0, "210, 1965, 150.0, Not Active, Not Active, Not Active, Not Active"),      # after it
    ]
    out = cs.stop(19.95, 20.25)
    assert out["sm_mhz"] == 1320.0 and out["sm_max_mhz"] == 1965.0 and out["samples"] == 3
    assert out["reasons"] == ["sw_power_cap"] and out["window"] == "timed region"


def test_clock_summary_falls_back_to_the_nearest_samples_for_a_short_window():
    bench = _bench()
    cs = bench.ClockSampler(0)
    cs.proc = _Done()
    cs.lines = [(t, f"{mhz}, 1965, 900.0, Not Active, Active, Not Active, Not Active")
                for t, mhz in ((1.0, 1900), (2.0, 1500), (3.0, 1400), (9.0, 300))]
    out = cs.stop(2.4, 2.45)       # no sample inside
    assert out["samples"] == 3 and out["sm_mhz"] == 1500.0
    assert out["reasons"] == ["hw_thermal_slowdown"] and out["window"].startswith("nearest samples")


def test_clock_summary_without_nvidia_smi():
    bench = _bench()
    cs = bench.ClockSampler(0)
    out = cs.stop()
    assert out["sm_mhz"] is None and out["reasons"] == ["nvidia-smi unavailable"]


def test_bench_without_a_gpu_prints_one_json_line_and_exits_zero():
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    for impl in ("own", "reference"):
        r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", impl, "--layout", "rows"],
                           capture_output=True, text=True, env=env, timeout=300)
        assert r.returncode == 0, r.stderr[-500:]
        line = json.loads(r.stdout.strip().splitlines()[-1])
        assert line["impl"] == impl and "unavailable" in line


def test_deadline_prints_the_line_on_rank_zero_and_ends_the_process_with_status_zero():
    code = (
        "import importlib.util, time, sys\n"
        f"spec = importlib.util.spec_from_file_location('ka_bench', {os.path.join(ROOT, 'bench.py')!r})\n"
        "m = importlib.util.module_from_spec(spec); spec.loader.exec_module(m)\n"
        "rank = int(sys.argv[1])\n"
        "m.Deadline(0.3, rank, lambda: {'value': 1.5, 'other_layout': {'unavailable': 'late'}}).start()\n"
        "time.sleep(20)\n"
        "print('not reached')\n"
    )
    for rank, want in ((0, {"value": 1.5, "other_layout": {"unavailable": "late"}}), (1, None)):
        r = subprocess.run([sys.executable, "-c", code, str(rank)], capture_output=True, text=True, timeout=120)
        assert r.returncode == 0 and "not reached" not in r.stdout
        if want is None:
            assert r.stdout.strip() == ""
        else:
            assert json.loads(r.stdout.strip()) == want


def test_deadline_cancelled_in_time_does_nothing():
    bench = _bench()
    d = bench.Deadline(0.2, 0, lambda: {"never": True}).start()
    d.cancel()
    import time

    time.sleep(0.5)   # the process is still here
