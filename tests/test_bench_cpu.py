"""The arithmetic behind the bench line, checked without a GPU: the algorithmic-bytes formulas of the
roofline figures against hand-computed values for the benchmark shapes, the sizing of the CPU sample,
and the argument defaults."""
import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


def test_forward_bytes_formula(bench):
    # 66,634 neurons, 5 channels, batch 5: 31 + 24*5 + 25/5 = 156 B per neuron-step of state, accumulator
    # and outputs; 9 B per delivered synapse, 8 B per active source row
    cnt = dict(rec_events=1000, lgn_events=200, bkg_events=50, rec_rows=10, lgn_rows=4, bkg_rows=1)
    got = bench.fwd_bytes_per_launch(cnt, 66634, 5, 5, 2500)
    assert got == 156.0 * 66634 * 5 * 2500 + 9.0 * 1250 + 8.0 * 15
    # per neuron-step at the benchmark's event rates (about 107 k synapse events per batch-step): ~170 B
    per_step = dict(rec_events=159000 * 2500, lgn_events=81000 * 2500, bkg_events=296000 * 2500,
                    rec_rows=7000 * 2500, lgn_rows=700 * 2500, bkg_rows=110 * 2500)
    b = bench.fwd_bytes_per_launch(per_step, 66634, 5, 5, 2500) / (66634 * 5 * 2500)
    assert 165.0 < b < 175.0


def test_backward_bytes_formula(bench):
    # 37 + 24*5 + 25/5 = 162 B per neuron-step, the recurrent synapse stream once per step (9 B per
    # synapse, shared by the batch), 17 B per weight-gradient event
    got = bench.bwd_bytes_per_launch(dict(dw_events=1000), 66634, 5, 5, 500, 7996080)
    assert got == 162.0 * 66634 * 5 * 500 + 9.0 * 7996080 * 500 + 17.0 * 1000
    per = bench.bwd_bytes_per_launch(dict(dw_events=238500 * 500), 66634, 5, 5, 500, 7996080) / (66634 * 5 * 500)
    assert 385.0 < per < 395.0          # the ~390 B per neuron-step of the configuration-4 roofline


def test_cpu_sample_is_sized_by_the_number_of_runs(bench):
    assert bench.bounded_cpu_steps(50, 2) == 50                  # the cpu_baseline leg: two samples of 50 ms
    assert 6 <= bench.bounded_cpu_steps(50, 8) <= 50             # the CPU arm's default: 5 timed + 3 warm-up
    assert bench.bounded_cpu_steps(50, 1000) == 6                # never below 6 simulated ms
