"""Helpers shared by the GPU parity tests: run a network description through the C ABI and compare
every readable tensor with the CPU oracle, bit for bit."""
import numpy as np

from n2d2_b200 import netdesc, runtime
from oracle import oracle

KEEP = runtime.KEEP_ALL_OUTPUTS | runtime.NO_FUSION


def single_conv_net(C, H, W, O, k, stride=1, pad=0, in_unsigned=True, act='relu', mode='single', seed=7, dil=1,
                    groups=1, bias=True, **builder_kw):
    b = netdesc.NetBuilder('single', C, H, W, seed, mode, input_unsigned=in_unsigned, weight_dist=('normal', 30),
                           **builder_kw)
    b.conv(-1, O, k, stride=stride, pad=pad, act=act, dil=dil, groups=groups, bias=bias, name='c')
    return b.net


def compare_net(net, batch, flags=KEEP, flavour='i64', x=None, want_engine=None, slices=0, ref=None):
    """Returns (number of compared layers, engines). Asserts bit-exact equality with the oracle."""
    if x is None:
        x = netdesc.make_input(net, batch)
    if ref is None:
        ref = oracle.run_net(net, x, flavour)
    qn = runtime.QuantizedNet(net, max(batch, 1), flags=flags)
    try:
        if slices:
            qn.set_slices(slices)
        out = qn.forward_host(x)
        eng = qn.engines()
        if want_engine is not None:
            wanted = (want_engine,) if isinstance(want_engine, str) else tuple(want_engine)
            assert any(w in eng for w in wanted), f'expected a {wanted} cell, got {sorted(set(eng))}'
        n = 0
        last = len(net['layers']) - 1
        assert np.array_equal(out.astype(np.int64), ref[last].reshape(batch, -1)), 'final output differs'
        for i, l in enumerate(net['layers']):
            if not qn.tensor_info(qn.tensor_of_layer[i]).readable:
                continue
            got = qn.read_layer(i, batch).astype(np.int64)
            bad = int((got != ref[i]).sum())
            assert bad == 0, f"layer {i} {l['name']} ({eng[i]}): {bad} of {ref[i].size} values differ"
            n += 1
        return n, eng
    finally:
        qn.close()
