"""The arithmetic of bench.py that needs no GPU: how the decode trajectory is cut into timed
windows, the flop count of a prefill step, the clock sampler's reading of nvidia-smi lines, and
the answer to a request for more than one GPU."""

import importlib.util
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("steps", [1, 5, 16, 20, 31, 32, 79, 80, 200, 500, 10 ** 6])
def test_windows_cover_the_trajectory_and_count_every_step(bench, steps):
    prompt, context = 512, 1024
    steps = min(steps, bench.max_steps(prompt, context))    # as bench.py clamps --steps
    windows = bench.decode_windows(prompt, context, steps)
    assert sum(k for _f, k, _r in windows) == steps
    assert 1 <= len(windows) <= bench.N_WINDOWS
    last_end = prompt
    for first, k, reps in windows:
        assert k >= 1 and 1 <= reps <= 3
        assert first >= last_end                      # windows follow one another, no overlap
        assert first + reps * k <= context - 1        # the last timed step still fits the model
        last_end = first + reps * k
    if steps >= 16:                                   # a repeat starts from an idle GPU: never short
        assert min(k for _f, k, _r in windows) >= 16
    if steps >= 80:
        assert len(windows) == bench.N_WINDOWS


@pytest.mark.parametrize("steps", [20, 80, 500])
def test_the_timed_steps_sit_around_the_middle_of_the_trajectory(bench, steps):
    windows = bench.decode_windows(512, 1024, steps)
    mean = bench.windows_mean_context(windows)
    assert abs(mean - 768) < 40                       # 512 -> 1,024: mean context 768
    # by hand: a window of k steps repeated r times, first context f, has mean f + (r k - 1) / 2
    total = sum(k for _f, k, _r in windows)
    want = sum(k * (f + (r * k - 1) / 2) for f, k, r in windows) / total
    assert mean == pytest.approx(want)


def test_max_steps_is_what_the_windows_can_hold(bench):
    n = bench.max_steps(512, 1024)
    windows = bench.decode_windows(512, 1024, n)
    assert sum(k for _f, k, _r in windows) == n
    assert all(first + reps * k <= 1023 for first, k, reps in windows)


def test_prefill_flops_by_hand(bench):
    cfg = dict(n_embd=8, n_inner=None, n_layer=3, vocab_size=11)
    n_seqs, s, rows = 2, 5, 2
    T = n_seqs * s
    linear = 2 * T * 3 * (8 * 24 + 8 * 8 + 2 * 8 * 32) + 2 * rows * 8 * 11
    pairs = s * (s + 1) // 2                          # (query, visible key) pairs of a sequence
    attention = 3 * n_seqs * pairs * 2 * 2 * 8        # q.k and p.v, 2 flops a multiply-add, all heads
    assert bench.prefill_flops(cfg, n_seqs, s, rows) == linear + attention
    cfg["n_inner"] = 20
    assert bench.prefill_flops(cfg, 1, 1, 0) == 2 * 3 * (8 * 24 + 8 * 8 + 2 * 8 * 20) + 3 * 2 * 2 * 8


class _FakeSmi:
    def __init__(self, text):
        self.text = text

    def terminate(self):
        pass

    def kill(self):
        pass

    def communicate(self, timeout=None):
        return self.text, ""


def test_clock_sampler_reads_busy_samples_and_reasons(bench):
    lines = [
        "120, 1965, 210.0, Not Active, Not Active, Not Active, Not Active, 0",
        "1965, 1965, 600.0, Not Active, Not Active, Not Active, Active, 93",
        "1950, 1965, 610.0, Not Active, Not Active, Not Active, Not Active, 95",
        "1935, 1965, 620.0, Not Active, Not Active, Not Active, Not Active, 97",
        "garbage line",
        "[N/A], 1965, 1.0, Not Active, Not Active, Not Active, Not Active, 0",
    ]
    s = bench.ClockSampler()
    s.proc = _FakeSmi("\n".join(lines))
    got = s.stop()
    assert got["sm_mhz"] == 1950.0                    # the median of the three busy samples
    assert got["sm_max_mhz"] == 1965.0
    assert got["samples"] == 4 and got["samples_busy"] == 3
    assert got["reasons"] == ["sw_power_cap"]
    # a program that never keeps the GPU busy: the median of all samples stands
    s.proc = _FakeSmi("\n".join(lines[:1] * 3))
    got = s.stop()
    assert got["sm_mhz"] == 120.0 and got["samples_busy"] == 0
    # no nvidia-smi at all
    s.proc = None
    assert s.stop()["reasons"] == ["nvidia-smi unavailable"]


def test_more_than_one_gpu_is_refused_with_one_line_and_exit_code_2():
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--gpus", "2"],
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 2
    out = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(out) == 1 and "one GPU" in out[0]
