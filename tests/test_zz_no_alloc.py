"""The first-layer convolution entry point that allocates no device memory
(n2d2b_first_conv_noalloc).

Who needs it: code that runs where cudaMalloc is off limits - a plugin inside a framework that owns
the device heap, a latency-bound loop that cannot take an allocation's device-wide synchronisation,
a process at its memory budget.  Its scratch is a fixed array inside the library, so the batch is
bounded and calls share state; this file checks that it returns exactly what the regular,
allocating path returns, on two calls in a row with different layers and inputs (the second call
must not see anything of the first), and that oversize requests are refused.

Collected last on purpose: if it fails, every other test has already run.
"""
import numpy as np
import pytest

from n2d2_b200 import netdesc, runtime
from oracle import oracle

from gpu_common import single_conv_net

pytestmark = pytest.mark.gpu


def _both_paths(net, batch, seed):
    import torch
    layer = net['layers'][0]
    i = net['input']
    x = netdesc.make_input(net, batch, seed=seed)
    # the existing entry points: a one-cell network, finalized (allocates), run on host buffers
    qn = runtime.QuantizedNet(net, batch)
    assert qn.engines() == ['stem-tcgen05']
    want = qn.forward_host(x)
    qn.close()
    # the allocation-free entry point on caller-owned device buffers
    d_in = torch.from_numpy(x.view(np.uint8)).cuda()
    d_out = torch.full((batch, want.shape[1]), 0x5A, dtype=torch.uint8, device='cuda')
    torch.cuda.synchronize()
    runtime.first_conv_noalloc(d_in.data_ptr(), batch, i['H'], i['W'], i['C'], i['unsigned'], layer, d_out.data_ptr())
    torch.cuda.synchronize()
    got = d_out.cpu().numpy().view(want.dtype)
    # both against the CPU restatement of the reference as well, not only against each other
    ref = oracle.run_net(net, x, 'i64')[-1].reshape(batch, -1)
    assert np.array_equal(want.astype(np.int64), ref), 'the allocating path differs from the oracle'
    assert np.array_equal(got.astype(np.int64), ref), 'the allocation-free entry point differs from the oracle'
    return got, want


def test_noalloc_first_conv_matches_the_allocating_path_twice_in_a_row():
    # call 1: a ResNet-style stem (3 channels, 7x7 stride 2, unsigned output after ReLU)
    net1 = single_conv_net(3, 64, 64, 64, 7, 2, 3, in_unsigned=True, mode='double', seed=21)
    got, want = _both_paths(net1, 4, seed=5)
    assert np.array_equal(got, want)          # integer path: bit-exact, no tolerance
    # call 2, straight after: other geometry, channel count, signedness, scaling mode and a smaller
    # output - anything left over from call 1 in the shared scratch would show
    net2 = single_conv_net(4, 19, 23, 32, 3, 1, 1, in_unsigned=False, act='linear', mode='single', seed=22)
    got, want = _both_paths(net2, 3, seed=6)
    assert np.array_equal(got, want)
    # and the first layer again, to make sure call 2 left nothing behind either
    got, want = _both_paths(net1, 2, seed=7)
    assert np.array_equal(got, want)


def test_noalloc_first_conv_rejects_what_it_cannot_hold():
    import torch
    net = single_conv_net(3, 64, 64, 64, 7, 2, 3, mode='double')
    layer = net['layers'][0]
    d = torch.zeros(16, dtype=torch.uint8, device='cuda')
    too_many = runtime.NOALLOC_MAX_PIXELS // (64 * 64) + 1
    with pytest.raises(runtime.N2D2BError, match='exceeds the fixed scratch'):
        runtime.first_conv_noalloc(d.data_ptr(), too_many, 64, 64, 3, True, layer, d.data_ptr())
    wide = single_conv_net(16, 16, 16, 64, 3, 1, 1, mode='double')['layers'][0]
    with pytest.raises(runtime.N2D2BError, match='first-layer kernel'):
        runtime.first_conv_noalloc(d.data_ptr(), 1, 16, 16, 16, True, wide, d.data_ptr())
