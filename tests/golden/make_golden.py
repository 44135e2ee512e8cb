"""Generates tests/golden/ref_vectors.npz from the reference's own CPU kernels (compiled by
oracle/refshim/Makefile into oracle/_ref/).  Needs the reference tree; run once, commit the output.

    make -C oracle/refshim && python tests/golden/make_golden.py

Every case stores its integer inputs and the reference's outputs; tests/test_oracle_golden.py replays
them through the oracle without needing the reference."""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle, refshim  # noqa: E402

rng = np.random.default_rng(20240611)
arrays = {}
cases = []

# convolutions: (C, H, W, O, k, stride, pad, dil, groups, value range)
CONVS = [(3, 9, 11, 8, 3, 1, 1, 1, 1), (8, 12, 12, 16, 3, 2, 1, 1, 1), (16, 7, 7, 16, 3, 1, 1, 1, 16),
         (4, 10, 10, 6, 5, 2, 2, 1, 1), (8, 9, 9, 8, 1, 2, 0, 1, 1), (6, 11, 11, 4, 3, 1, 2, 2, 1),
         (8, 8, 8, 8, 3, 1, 1, 1, 2), (1, 24, 24, 16, 4, 2, 0, 1, 1), (3, 15, 15, 4, 7, 2, 3, 1, 1),
         (512, 5, 5, 2, 3, 1, 1, 1, 1)]
for i, (C, H, W, O, k, s, p, d, g) in enumerate(CONVS):
    x = rng.integers(0, 256, (2, C, H, W)).astype(np.int32)
    w = rng.integers(-127, 128, (O, C // g, k, k)).astype(np.int32)
    b = rng.integers(-4096, 4097, O).astype(np.int32)
    y = refshim.conv(x, w, (s, s), (p, p, p, p), (d, d), oracle.group_map(O, C, g), b)
    arrays[f'conv{i}_x'], arrays[f'conv{i}_w'], arrays[f'conv{i}_b'], arrays[f'conv{i}_y'] = x.astype(np.uint8), w.astype(np.int8), b, y
    cases.append({'kind': 'conv', 'id': i, 'stride': s, 'pad': p, 'dil': d, 'groups': g})

POOLS = [('max', 4, 9, 9, 3, 2, 0), ('max', 4, 9, 9, 3, 2, 1), ('avg', 8, 7, 7, 7, 1, 0), ('avg', 3, 8, 10, 2, 2, 0),
         ('avg', 4, 9, 9, 3, 2, 1), ('max', 2, 5, 5, 2, 3, 2)]
for i, (kind, C, H, W, k, s, p) in enumerate(POOLS):
    x = rng.integers(-128, 256, (2, C, H, W)).astype(np.int32)
    y = refshim.pool(x, kind, (k, k), (s, s), (p, p), quantized=True)
    arrays[f'pool{i}_x'], arrays[f'pool{i}_y'] = x.astype(np.int16), y
    cases.append({'kind': 'pool', 'id': i, 'pool': kind, 'k': k, 'stride': s, 'pad': p})

C = 8
xs = rng.integers(-300000, 300000, (2, C, 5, 5)).astype(np.int32)
# hand-picked values on every channel: zero, +-1, ties at one half of every shift, large magnitudes
special = np.array([0, 1, -1, 2, -2, 3, -3, 127, 128, -128, -129, 255, 256, 32, -32, 31, -33, 64, -64, 1 << 20,
                    -(1 << 20), (1 << 24) - 1, -(1 << 24) + 1, 65535, -65536], np.int32)
xs[0] = np.broadcast_to(special.reshape(1, 5, 5), (C, 5, 5))
SCALINGS = [
    {'mode': 'single', 'shift0': np.array([0, 1, 2, 5, 6, 8, 12, 16], np.uint8)},
    {'mode': 'double', 'shift0': np.array([0, 1, 2, 3, 4, 1, 2, 3], np.uint8), 'shift1': np.array([0, 1, 4, 6, 8, 10, 12, 14], np.uint8)},
    {'mode': 'fixed32', 'mult': rng.integers(1 << 14, 1 << 15, C).astype(np.int32), 'frac_bits': 16},
    {'mode': 'fixed32', 'mult': rng.integers(-(1 << 15), 1 << 15, C).astype(np.int32), 'frac_bits': 24},
    {'mode': 'fixed32', 'mult': rng.integers(1, 1 << 30, C).astype(np.int32), 'frac_bits': 0},
    {'mode': 'fixed32', 'mult': rng.integers(1 << 14, 1 << 15, C).astype(np.int32), 'frac_bits': 16, 'is_clipped': True,
     'clip': np.array([100.5, 2000.25, -300.75, 65000.0, 0.0, 12.5, -1.5, 1e6], np.float32)},
    {'mode': 'float', 'fscale': rng.uniform(-0.01, 0.01, C).astype(np.float32)},
    {'mode': 'float', 'fscale': np.array([0.5, 0.25, 1.5, 2.5, 0.001, 0.0625, 1.0, 0.03125], np.float32)},
    {'mode': 'float', 'fscale': rng.uniform(0, 0.001, C).astype(np.float32), 'is_clipped': True,
     'clip': np.array([100.5, 2000.25, -300.75, 65000.0, 0.0, 12.5, -1.5, 1e6], np.float32)},
]
for i, q in enumerate(SCALINGS):
    for uns in (0, 1):
        for bits in (8, 4):
            qq = dict(q, out_bits=bits, out_unsigned=bool(uns))
            y = refshim.scaling(xs, qq)
            arrays[f'scal{i}_{uns}_{bits}_y'] = y
            meta = {'kind': 'scaling', 'id': i, 'unsigned': uns, 'bits': bits, 'mode': q['mode'],
                    'frac_bits': int(q.get('frac_bits', 0)), 'is_clipped': bool(q.get('is_clipped', False))}
            cases.append(meta)
    for key in ('shift0', 'shift1', 'mult', 'fscale', 'clip'):
        if key in q:
            arrays[f'scal{i}_{key}'] = q[key]
arrays['scal_x'] = xs

out = os.path.join(ROOT, 'tests', 'golden', 'ref_vectors.npz')
np.savez_compressed(out, cases=np.frombuffer(json.dumps(cases).encode(), np.uint8), **arrays)
print(out, os.path.getsize(out), 'bytes,', len(cases), 'cases')
