"""Stand-alone Scaling::propagate on the GPU (n2d2b_scaling_propagate) against the golden vectors the
reference's own Scaling_Kernels produced, and against the hand-derived known answers."""
import json
import os

import numpy as np
import pytest

from n2d2_b200 import runtime

pytestmark = pytest.mark.gpu

GOLD = np.load(os.path.join(os.path.dirname(__file__), 'golden', 'ref_vectors.npz'))
CASES = [c for c in json.loads(bytes(GOLD['cases']).decode()) if c['kind'] == 'scaling']


def _gpu_scaling(x_nchw, q):
    import torch
    x = np.ascontiguousarray(np.transpose(x_nchw, (0, 2, 3, 1))).astype(np.int32)   # NHWC
    B, H, W, C = x.shape
    d_in = torch.from_numpy(x).cuda()
    d_out = torch.zeros((B, H, W, C), dtype=torch.int8, device='cuda')
    runtime.scaling_propagate(d_in.data_ptr(), d_out.data_ptr(), B * H * W, q, C)
    out = d_out.cpu().numpy()
    out = out.view(np.uint8) if q.get('out_unsigned') else out
    return np.transpose(out.astype(np.int64), (0, 3, 1, 2))


@pytest.mark.parametrize('case', CASES, ids=lambda c: f"{c['mode']}{c['id']}_u{c['unsigned']}_b{c['bits']}")
def test_scaling_matches_reference_vectors(case):
    i = case['id']
    q = {'mode': case['mode'], 'out_bits': case['bits'], 'out_unsigned': bool(case['unsigned']), 'act': 'linear',
         'frac_bits': case['frac_bits'], 'is_clipped': case['is_clipped']}
    for key in ('shift0', 'shift1', 'mult', 'fscale', 'clip'):
        if f'scal{i}_{key}' in GOLD:
            q[key] = GOLD[f'scal{i}_{key}']
    want = GOLD[f"scal{i}_{case['unsigned']}_{case['bits']}_y"].astype(np.int64)
    got = _gpu_scaling(GOLD['scal_x'], q)
    assert np.array_equal(got, want)


def test_scaling_known_answers_on_gpu():
    from test_oracle_golden import KAT
    for q, unsigned, xs, want in KAT:
        q = dict(q, out_bits=8, out_unsigned=unsigned, act='linear')
        x = np.array(xs).reshape(len(xs), 1, 1, 1)
        assert _gpu_scaling(x, q).reshape(-1).tolist() == want
