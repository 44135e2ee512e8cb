"""Calibration statistics of the quantization front-end (n2d2_b200/host/Calibration.hpp: RangeStats, Histogram,
MSE / KL-divergence / quantile thresholds, state files) against the REFERENCE's own code: the committed fixtures
were produced by the reference's Histogram / RangeStats sources compiled where they lie
(tests/golden/make_calibration_golden.py); where that compiled code is present, further seeded cases are compared
live.  Every value must be equal bit for bit."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, 'tests', 'host', 'test_calibration')
GOLDEN = os.path.join(ROOT, 'tests', 'golden', 'calibration_golden.txt')
STATE = os.path.join(ROOT, 'tests', 'golden', 'calibration_state')
NAMES = ['range min', 'range max', 'moment 0', 'moment 1', 'moment 2', 'bins', 'histogram min', 'histogram max',
         'bin checksum', 'MSE threshold', 'KL threshold', 'quantile 0.9999', 'quantile 0.5', 'bin centre']


def _build():
    src = os.path.join(ROOT, 'tests', 'host', 'test_calibration.cpp')
    deps = [src, os.path.join(ROOT, 'n2d2_b200', 'host', 'Calibration.hpp')]
    if os.path.exists(EXE) and all(os.path.getmtime(EXE) > os.path.getmtime(d) for d in deps):
        return
    env = {k: v for k, v in os.environ.items() if k not in ('CC', 'CXX')}
    # no fused multiply-adds: the reference's objects are built the same way
    subprocess.check_call(['g++', '-std=c++17', '-O2', '-ffp-contract=off', '-Wall', '-o', EXE, src], env=env)


def _value(s):
    return float.fromhex(s) if ('x' in s or 'X' in s) else int(s)


def _run_case(case):
    out = subprocess.run([EXE, 'case'] + [str(c) for c in case], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    return [_value(t) for t in out.stdout.split()]


def _golden_cases():
    cases = []
    for line in open(GOLDEN):
        if line.startswith('#') or not line.strip():
            continue
        left, right = line.split('|')
        cases.append((left.split(), [_value(t) for t in right.split()]))
    return cases


@pytest.mark.parametrize('case,want', _golden_cases(), ids=lambda c: '_'.join(c[:2] + c[4:6]) if isinstance(c[0], str) else None)
def test_thresholds_ranges_and_bins_equal_the_reference(case, want):
    _build()
    got = _run_case(case)
    assert len(got) == len(want) == len(NAMES)
    for name, g, w in zip(NAMES, got, want):
        assert g == w, f'{name}: {g!r} != {w!r} ({case})'


def test_state_files_equal_the_reference_byte_for_byte():
    _build()
    scratch = os.path.join(ROOT, 'tests', 'host', '_tmp')
    os.makedirs(scratch, exist_ok=True)
    out = subprocess.run([EXE, 'state', scratch], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    for f in ('hist.bin', 'range.bin'):
        assert open(os.path.join(scratch, f), 'rb').read() == open(os.path.join(STATE, f), 'rb').read(), f


def test_further_cases_against_the_compiled_reference():
    import importlib.util
    spec = importlib.util.spec_from_file_location('make_calibration_golden',
                                                  os.path.join(ROOT, 'tests', 'golden', 'make_calibration_golden.py'))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    if not os.path.exists(gen.SO):
        pytest.skip('the reference tree was not compiled here')
    _build()
    lib = gen.lib()
    for case in [('tail', 101, 6000, 0.5, 8, 'MSE'), ('relu', 102, 7000, 12.0, 6, 'KL-Divergence'),
                 ('bell', 103, 3000, 1.0, 3, 'MSE'), ('bell', 104, 8000, 250.0, 8, 'KL-Divergence')]:
        want = [_value(t) for t in gen.reference_case(lib, *case)]
        got = _run_case(case)
        for name, g, w in zip(NAMES, got, want):
            assert g == w, f'{name}: {g!r} != {w!r} ({case})'
