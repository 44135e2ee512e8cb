"""Host-side checks that need no GPU: the C-ABI library loads and exports every declared symbol,
fails loudly without a device, and the network descriptions have the reference's geometry."""
import ctypes
import os
import re

import numpy as np
import pytest

from n2d2_b200 import netdesc, runtime

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    syms = set()
    for f in os.listdir(os.path.join(ROOT, 'include')):
        if f.endswith('.h'):
            text = open(os.path.join(ROOT, 'include', f)).read()
            syms |= set(re.findall(r'\b(n2d2b_[a-z0-9_]+)\s*\(', text))
    return sorted(syms)


def test_library_exports_every_declared_entry_point():
    lib = ctypes.CDLL(runtime.LIB_PATH)
    syms = _declared_symbols()
    assert len(syms) >= 18
    for s in syms:
        assert hasattr(lib, s), f'{s} is declared in include/ but not exported'


def test_no_cpu_fallback_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip('a GPU is present')
    with pytest.raises(runtime.N2D2BError):
        runtime.QuantizedNet(netdesc.mnist24(), 4)


def test_product_never_touches_the_oracle():
    for dirpath, _, files in os.walk(os.path.join(ROOT, 'n2d2_b200')):
        for f in files:
            if f.endswith(('.py', '.cu', '.cuh', '.h', '.hpp', '.cpp')):
                text = open(os.path.join(dirpath, f)).read()
                assert 'oracle' not in text.lower(), f'{f} mentions the oracle'


def test_resnet50_geometry_and_work():
    net = netdesc.resnet50()
    macs, shapes = netdesc.layer_macs(net)
    convs = [m for l, m in zip(net['layers'], macs) if l['type'] == 'conv']
    assert len(convs) == 53
    assert shapes[1] == (64, 55, 55)                       # pool1 without padding: 112 -> 55
    assert abs(sum(convs) / 4.0599e9 - 1) < 1e-3
    assert macs[-1] == 2048 * 1000
    assert [l['type'] for l in net['layers']].count('sum') == 16


def test_resnet18_mobilenet_mnist_geometry():
    macs, shapes = netdesc.layer_macs(netdesc.resnet18())
    assert abs(sum(macs) / 1.810e9 - 1) < 5e-3
    net = netdesc.mobilenet_v1()
    macs, shapes = netdesc.layer_macs(net)
    assert abs(sum(macs) / 0.5687e9 - 1) < 5e-3
    dw = sum(m for l, m in zip(net['layers'], macs) if l['type'] == 'conv' and l['groups'] > 1)
    assert abs(dw / 17.4e6 - 1) < 2e-2
    net = netdesc.mnist24()
    macs, shapes = netdesc.layer_macs(net)
    assert sum(macs) == 243676
    assert shapes[0] == (16, 11, 11) and shapes[1] == (24, 4, 4)
    q = net['layers'][0]['quant']
    assert q['mode'] == 'single' and q['shift0'].min() >= 6 and q['shift0'].max() <= 12


def test_generators_are_seeded():
    a, b = netdesc.mnist24(seed=3), netdesc.mnist24(seed=3)
    assert all(np.array_equal(x['weights'], y['weights']) for x, y in zip(a['layers'], b['layers']))
    c = netdesc.mnist24(seed=4)
    assert not np.array_equal(a['layers'][0]['weights'], c['layers'][0]['weights'])


def test_int4_packing_puts_even_elements_in_the_high_nibble():
    w = np.array([[1, -2, 7, -7, 3]], np.int8)
    p = netdesc.pack_int4(w)
    assert p.tolist() == [[0x1E, 0x79, 0x30]]
