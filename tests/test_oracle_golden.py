"""The CPU oracle against vectors produced by the reference's own CPU kernels (tests/golden/
ref_vectors.npz, made by tests/golden/make_golden.py from the reference sources) and against
hand-derived known answers for every scaling mode."""
import json
import os

import numpy as np
import pytest

from oracle import oracle

GOLD = np.load(os.path.join(os.path.dirname(__file__), 'golden', 'ref_vectors.npz'))
CASES = json.loads(bytes(GOLD['cases']).decode())


def _ids(c):
    return f"{c['kind']}{c['id']}" + (f"_u{c['unsigned']}_b{c['bits']}" if c['kind'] == 'scaling' else '')


@pytest.mark.parametrize('case', [c for c in CASES if c['kind'] == 'conv'], ids=_ids)
@pytest.mark.parametrize('flavour', ['f32', 'i64'])
def test_conv_matches_reference_kernel(case, flavour):
    i = case['id']
    x, w, b, y = (GOLD[f'conv{i}_{k}'] for k in 'xwby')
    s, p, d, g = case['stride'], case['pad'], case['dil'], case['groups']
    got = oracle.conv(x, w, flavour, (s, s), (p, p, p, p), (d, d), g, bias=b, ref_quirks=True)
    assert np.array_equal(got.astype(np.float64), y.astype(np.float64))


@pytest.mark.parametrize('case', [c for c in CASES if c['kind'] == 'pool'], ids=_ids)
@pytest.mark.parametrize('flavour', ['f32', 'i64'])
def test_pool_matches_reference_kernel(case, flavour):
    i = case['id']
    x, y = GOLD[f'pool{i}_x'], GOLD[f'pool{i}_y']
    k, s, p = case['k'], case['stride'], case['pad']
    got = oracle.pool(x, case['pool'], (k, k), (s, s), (p, p), flavour)
    assert np.array_equal(got.astype(np.float64), y.astype(np.float64))


def _scaling_quant(case):
    i = case['id']
    q = {'mode': case['mode'], 'out_bits': case['bits'], 'out_unsigned': bool(case['unsigned']), 'act': 'linear',
         'frac_bits': case['frac_bits'], 'is_clipped': case['is_clipped']}
    for key in ('shift0', 'shift1', 'mult', 'fscale', 'clip'):
        if f'scal{i}_{key}' in GOLD:
            q[key] = GOLD[f'scal{i}_{key}']
    return q


@pytest.mark.parametrize('case', [c for c in CASES if c['kind'] == 'scaling'], ids=_ids)
@pytest.mark.parametrize('flavour', ['f32', 'i64'])
def test_scaling_matches_reference_kernel(case, flavour):
    y = GOLD[f"scal{case['id']}_{case['unsigned']}_{case['bits']}_y"]
    got = oracle.scaling(GOLD['scal_x'], _scaling_quant(case), flavour)
    assert np.array_equal(got.astype(np.float64), y.astype(np.float64))


# ---- hand-derived known answers (round-half-up shifts, half-away-from-zero float, saturation) ----
KAT = [
    # single shift: (x + 2^(s-1)) >> s, arithmetic shift = floor
    ({'mode': 'single', 'shift0': [1]}, False, [3, -3, 1, -1, 255, -257, 1000], [2, -1, 1, 0, 127, -128, 127]),
    ({'mode': 'single', 'shift0': [0]}, True, [3, -3, 255, 256], [3, 0, 255, 255]),
    ({'mode': 'single', 'shift0': [4]}, True, [8, 7, 24, 23, -8, 4088], [1, 0, 2, 1, 0, 255]),
    # double shift: (x + (x << a) + 2^(b-1)) >> b  = x * (1 + 2^a) / 2^b rounded half up
    ({'mode': 'double', 'shift0': [1], 'shift1': [2]}, False, [2, -2, 1, -1, 200], [2, -1, 1, -1, 127]),
    ({'mode': 'double', 'shift0': [2], 'shift1': [0]}, False, [3, -30], [15, -128]),
    # fixed point: (x * m + 2^(f-1)) >> f
    ({'mode': 'fixed32', 'mult': [3], 'frac_bits': 1}, False, [1, -1, 3, -3], [2, -1, 5, -4]),
    ({'mode': 'fixed32', 'mult': [-3], 'frac_bits': 1}, False, [1, -1], [-1, 2]),
    ({'mode': 'fixed32', 'mult': [1 << 15], 'frac_bits': 16}, True, [1, 3, 511, -5], [1, 2, 255, 0]),
    ({'mode': 'fixed32', 'mult': [1 << 16], 'frac_bits': 16, 'is_clipped': True, 'clip': [10.5]}, False,
     [-4, 0, 10, 11, 500], [0, 0, 10, 11, 11]),   # 11 > 10.5 -> clip -> round(10.5) = 11
    ({'mode': 'fixed32', 'mult': [1 << 16], 'frac_bits': 16, 'is_clipped': True, 'clip': [-10.5]}, False,
     [4, 0, -10, -11, -500], [0, 0, -10, -11, -11]),  # clip <= 0 clamps to [clip, 0]; round(-10.5) = -11
    # float: round half away from zero, then saturate
    ({'mode': 'float', 'fscale': [0.5]}, False, [1, -1, 3, -3, 1000, -1000], [1, -1, 2, -2, 127, -128]),
    ({'mode': 'float', 'fscale': [0.5]}, True, [1, -1, 3, 1000], [1, 0, 2, 255]),
    ({'mode': 'float', 'fscale': [0.25], 'is_clipped': True, 'clip': [9.0]}, False, [-5, 8, 9, 10, 99], [0, 2, 2, 2, 2]),
]


@pytest.mark.parametrize('flavour', ['f32', 'i64'])
@pytest.mark.parametrize('k', range(len(KAT)))
def test_scaling_known_answers(k, flavour):
    q, unsigned, xs, want = KAT[k]
    q = dict(q, out_bits=8, out_unsigned=unsigned, act='linear')
    x = np.array(xs).reshape(len(xs), 1, 1, 1)
    got = oracle.scaling(x, q, flavour).reshape(-1)
    assert got.astype(np.int64).tolist() == want


def test_integer_modes_reject_unquantized_cells():
    # FixedPoint/SingleShift/DoubleShift::propagate throw when nbBits == 0 (src/Scaling_Kernels.cpp:103-105)
    x = np.zeros((1, 1, 1, 1))
    assert oracle.lib().n2d2o_scaling_f32(oracle._p(np.zeros(1, np.float32)), oracle._p(np.zeros(1, np.float32)), 1, 1, 1,
                                          4, None, None, 0, None, oracle._p(np.zeros(1, np.uint8)), None, 0, None, 0, 0) == -1


def test_relu_and_order_of_operations():
    # scale -> saturate -> ReLU (src/Cell/ConvCell_Frame.cpp:449-468 + RectifierActivation_Frame.hpp:61-83)
    q = {'mode': 'single', 'shift0': [0], 'out_bits': 8, 'out_unsigned': False, 'act': 'relu'}
    x = np.array([-500, -3, 0, 3, 500]).reshape(5, 1, 1, 1)
    assert oracle.scaling(x, q, 'i64').reshape(-1).tolist() == [0, 0, 0, 3, 127]


def test_f32_and_i64_flavours_agree_below_2_24_and_part_above():
    rng = np.random.default_rng(5)
    x = rng.integers(0, 256, (1, 64, 6, 6))
    w = rng.integers(-127, 128, (4, 64, 3, 3))
    a = oracle.conv(x, w, 'f32', pad=(1, 1, 1, 1))
    b = oracle.conv(x, w, 'i64', pad=(1, 1, 1, 1))
    assert np.array_equal(a.astype(np.int64), b)       # 576 taps * 32385 < 2^24
    # all-maximal operands push the partial sums beyond 2^24: fp32 accumulation then rounds
    x = np.full((1, 1024, 3, 3), 255)
    w = np.full((1, 1024, 3, 3), 127)
    w[0, ::2] = 126
    a = oracle.conv(x, w, 'f32', pad=(1, 1, 1, 1))
    b = oracle.conv(x, w, 'i64', pad=(1, 1, 1, 1))
    assert b.max() > (1 << 24)
    assert not np.array_equal(a.astype(np.int64), b)


def test_average_pool_truncates_toward_zero():
    x = np.array([[-7, 0], [0, 0]]).reshape(1, 1, 2, 2)
    assert oracle.pool(x, 'avg', (2, 2), (2, 2), (0, 0), 'i64').item() == -1   # -7/4 -> -1, not -2
    assert oracle.pool(x, 'avg', (2, 2), (2, 2), (0, 0), 'f32').item() == -1
    # divisor counts padded taps (PoolCell_Frame.cpp:158-166)
    x = np.full((1, 1, 2, 2), 9)
    got = oracle.pool(x, 'avg', (3, 3), (2, 2), (1, 1), 'i64')
    assert got.reshape(-1).tolist() == [4]   # 4 in-image taps * 9 / 9


def test_max_pool_of_an_all_padding_window_is_zero():
    x = np.full((1, 1, 2, 2), -5)
    got = oracle.pool(x, 'max', (2, 2), (3, 3), (2, 2), 'i64')
    assert got.reshape(-1)[0] == 0
