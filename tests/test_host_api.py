"""The C++ host classes with N2D2's names (n2d2_b200/host/N2D2.hpp): compiled against the C ABI and run
as the reference's cell tests are (build a net with the reference's constructors, compare every value)."""
import os
import subprocess

import pytest

from n2d2_b200 import runtime
from oracle import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, 'tests', 'host', 'test_host_api')


def _build():
    oracle.build()
    src = os.path.join(ROOT, 'tests', 'host', 'test_host_api.cpp')
    deps = [src, os.path.join(ROOT, 'n2d2_b200', 'host', 'N2D2.hpp'), os.path.join(ROOT, 'include', 'n2d2b.h')]
    if os.path.exists(EXE) and all(os.path.getmtime(EXE) > os.path.getmtime(d) for d in deps):
        return
    env = {k: v for k, v in os.environ.items() if k not in ('CC', 'CXX')}
    subprocess.check_call(['g++', '-std=c++17', '-O1', '-o', EXE, src, runtime.LIB_PATH,
                           os.path.join(ROOT, 'oracle', 'libn2d2_oracle.so'),
                           '-Wl,-rpath,' + os.path.join(ROOT, 'n2d2_b200'), '-Wl,-rpath,' + os.path.join(ROOT, 'oracle')], env=env)


def test_host_classes_compile_and_fail_loudly_without_a_gpu():
    import torch
    _build()
    if torch.cuda.is_available():
        pytest.skip('a GPU is present')
    out = subprocess.run([EXE, '--no-gpu'], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr


@pytest.mark.gpu
def test_host_classes_run_config1_bit_exact():
    _build()
    out = subprocess.run([EXE], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    assert ' 0 mismatches' in out.stdout
