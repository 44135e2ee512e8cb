"""The post-training quantization front-end (n2d2_b200/host/DeepNetQuantization.hpp): known answers of the
scaling approximations and of the ScalingCell rewrite rules on CPU; on a GPU, small float networks are
quantized from value-range calibration and the integer networks must track the float ones (relative
error and top-1 agreement: the accuracy-level criterion of the reference's own quantization tests,
tests/class_DeepNetQuantization.cpp)."""
import os
import subprocess

import pytest

from n2d2_b200 import runtime
from oracle import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, 'tests', 'host', 'test_quantization')


def _build():
    oracle.build()
    src = os.path.join(ROOT, 'tests', 'host', 'test_quantization.cpp')
    deps = [src, runtime.LIB_PATH, os.path.join(ROOT, 'include', 'n2d2b.h')] + [
        os.path.join(ROOT, 'n2d2_b200', 'host', f) for f in ('N2D2.hpp', 'DeepNetQuantization.hpp', 'Calibration.hpp')]
    if os.path.exists(EXE) and all(os.path.getmtime(EXE) > os.path.getmtime(d) for d in deps):
        return
    env = {k: v for k, v in os.environ.items() if k not in ('CC', 'CXX')}
    subprocess.check_call(['g++', '-std=c++17', '-O1', '-Wall', '-o', EXE, src, runtime.LIB_PATH,
                           os.path.join(ROOT, 'oracle', 'libn2d2_oracle.so'),
                           '-Wl,-rpath,' + os.path.join(ROOT, 'n2d2_b200'), '-Wl,-rpath,' + os.path.join(ROOT, 'oracle')], env=env)


def test_scaling_approximations_and_graph_rewrite_known_answers():
    _build()
    out = subprocess.run([EXE, '--kat'], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    assert 'known answers ok' in out.stdout


@pytest.mark.gpu
@pytest.mark.parametrize('per_channel', [0, 1])
@pytest.mark.parametrize('mode', ['fixed', 'single', 'double'])
def test_quantized_networks_track_the_float_networks(mode, per_channel):
    _build()
    out = subprocess.run([EXE, '--run', mode, str(per_channel)], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr


def test_statistics_driven_front_end_on_cpu():
    """Ranges and histograms fed batch by batch, the thresholds quantizeActivations asks for (a max pooling's
    statistics stand for the cell above it), weight clipping, state files."""
    _build()
    scratch = os.path.join(ROOT, 'tests', 'host', '_tmp')
    os.makedirs(scratch, exist_ok=True)
    out = subprocess.run([EXE, '--stats', scratch], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    assert 'statistics front-end ok' in out.stdout


@pytest.mark.gpu
@pytest.mark.parametrize('mode,per_channel,clip', [('fixed', 0, 1), ('double', 1, 1), ('fixed', 0, 2), ('single', 1, 2),
                                                   ('fixed', 1, 3)])
def test_networks_quantized_from_calibration_statistics(mode, per_channel, clip):
    # clip: 1 = statistics without clipping (must equal the value-range run), 2 = MSE, 3 = KL divergence
    _build()
    out = subprocess.run([EXE, '--run', mode, str(per_channel), str(clip)], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr


def test_scaling_approximations_equal_the_reference_on_committed_vectors():
    """approximateScalingWithPowerOf2Divs / approximateScalingWithFixedPoint against vectors produced by the reference's
    own functions (tests/golden/make_quantization_golden.py): exponents, precisions, fractional bits and fixed-point
    scalings bit for bit, including the fall-back from 16 to 32 bits and the case the reference rejects."""
    _build()
    out = subprocess.run([EXE, '--golden', os.path.join(ROOT, 'tests', 'golden', 'quantization_golden.txt')],
                         capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    assert 'golden cases ok' in out.stdout
