"""The oracle against the reference's own kernels compiled where they lie (oracle/_ref, built by
oracle/refshim/Makefile when the reference tree is present).  Skipped when the shim was never built."""
import numpy as np
import pytest

from n2d2_b200 import netdesc
from oracle import oracle, refshim

pytestmark = pytest.mark.skipif(not refshim.available(), reason='oracle/_ref/libn2d2_refshim.so not built')


def test_random_convolutions_match_the_reference_kernel():
    rng = np.random.default_rng(11)
    for _ in range(25):
        C = int(rng.choice([1, 3, 8, 16, 64]))
        g = int(rng.choice([1, C])) if C > 1 else 1
        O = g * int(rng.integers(1, 5)) if g > 1 else int(rng.integers(1, 20))
        k = int(rng.choice([1, 2, 3, 4, 5, 7]))
        s, d = int(rng.integers(1, 4)), int(rng.choice([1, 1, 2]))
        if k < 3:
            d = 1   # the reference's CPU kernel asserts on a dilated 2x2 kernel (its unrolled 3x3 branch reads tap 2)
        p = int(rng.integers(0, k))
        H, W = int(rng.integers(d * (k - 1) + 1, 20)), int(rng.integers(d * (k - 1) + 1, 20))
        x = rng.integers(-128, 256, (2, C, H, W))
        w = rng.integers(-127, 128, (O, C // g, k, k))
        b = rng.integers(-4096, 4097, O)
        want = refshim.conv(x, w, (s, s), (p, p, p, p), (d, d), oracle.group_map(O, C, g), b)
        got = oracle.conv(x, w, 'f32', (s, s), (p, p, p, p), (d, d), g, bias=b, ref_quirks=True)
        assert np.array_equal(got, want), (C, H, W, O, k, s, p, d, g)


def test_sparse_connection_maps_match_the_reference_kernel():
    # Cell mapping (the ini files' Mapping(...)): unconnected channels are skipped; with a map that is not made of
    # groups the weight tensor is indexed by the channel itself
    rng = np.random.default_rng(12)
    for _ in range(12):
        C, O = int(rng.choice([3, 8, 16, 24])), int(rng.integers(2, 30))
        k = int(rng.choice([1, 3, 5]))
        s = int(rng.integers(1, 3))
        p = int(rng.integers(0, k))
        H, W = int(rng.integers(k, 16)), int(rng.integers(k, 16))
        maps = (rng.random((O, C)) < 0.4).astype(np.uint8)
        maps[np.arange(O), rng.integers(0, C, O)] = 1            # every output keeps at least one channel
        x = rng.integers(-128, 256, (2, C, H, W))
        w = rng.integers(-127, 128, (O, C, k, k))
        b = rng.integers(-4096, 4097, O)
        want = refshim.conv(x, w, (s, s), (p, p, p, p), (1, 1), maps, b)
        got = oracle.conv(x, w, 'f32', (s, s), (p, p, p, p), (1, 1), 1, maps=maps, bias=b, ref_quirks=True)
        assert np.array_equal(got, want), (C, H, W, O, k, s, p)
        # the same integers from a dense convolution whose unconnected weights are zero (what the device runs)
        dense = oracle.conv(x, w * maps[:, :, None, None], 'i64', (s, s), (p, p, p, p), (1, 1), 1, bias=b)
        assert np.array_equal(dense, oracle.conv(x, w, 'i64', (s, s), (p, p, p, p), (1, 1), 1, maps=maps, bias=b))


def test_fp32_rounding_beyond_2_24_matches_the_reference_kernel():
    x = np.full((1, 1024, 5, 5), 255)
    w = np.full((2, 1024, 3, 3), 127)
    w[0, ::2] = 126
    want = refshim.conv(x, w, (1, 1), (1, 1, 1, 1))
    got = oracle.conv(x, w, 'f32', (1, 1), (1, 1, 1, 1))
    assert want.max() > (1 << 24)
    assert np.array_equal(got, want)


def test_whole_networks_match():
    for net, batch in ((netdesc.mnist24(), 8), (netdesc.resnet50(size=32, classes=10), 2),
                       (netdesc.mobilenet_v1(size=32, classes=10), 2),
                       (netdesc.resnet18(size=32, classes=10, scaling='float', clipped=True), 2)):
        x = netdesc.make_input(net, batch)
        want = refshim.run_net(net, x)
        got = oracle.run_net(net, x, 'f32')
        for l, a, b in zip(net['layers'], got, want):
            assert np.array_equal(a, b), l['name']
