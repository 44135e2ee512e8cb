"""Parity at the sizes the benchmark times: the five configurations at their real geometry
(3x224x224 inputs, the reference ini's unpadded pool1 -> 55x55 maps), through the C ABI, bit for bit.

Small batches are compared with the CPU oracle cell by cell and in the shipped configuration (fused
residual sums, shared buffers); the benchmark batches (1024 images of ResNet-50, 2048 of the 4-bit
ResNet-18) are checked through size-independent properties: the host-buffer, streaming and
device-buffer entry points must agree on every image, and images picked on both sides of every upload
slice boundary must equal the oracle's result for that image alone."""
import numpy as np
import pytest

from n2d2_b200 import netdesc, runtime
from oracle import oracle

from gpu_common import KEEP, compare_net

pytestmark = pytest.mark.gpu

FULL = {
    'resnet50_double': lambda: netdesc.resnet50(seed=4, size=224),
    'resnet18_fixed': lambda: netdesc.resnet18(seed=2, size=224),
    'mobilenet_single': lambda: netdesc.mobilenet_v1(seed=3, size=224),
    'resnet18_w4_clipped_fixed': lambda: netdesc.resnet18(seed=5, size=224, weight_bits=4, clipped=True),
}


@pytest.mark.parametrize('name', sorted(FULL))
def test_full_size_network_cell_by_cell_and_shipped(name):
    net = FULL[name]()
    x = netdesc.make_input(net, 3, seed=77)
    # the two oracle flavours: fp32 accumulation in the reference's loop order (what the reference computes)
    # and exact int64; stated mismatch count between them on this configuration: 0
    ref64 = oracle.run_net(net, x[:2], 'i64')
    ref32 = oracle.run_net(net, x[:2], 'f32')
    mismatches = sum(int((np.asarray(a).astype(np.int64) != np.asarray(b).astype(np.int64)).sum())
                     for a, b in zip(ref64, ref32))
    assert mismatches == 0, f'{name}: fp32 and int64 oracles differ in {mismatches} values'
    n, eng = compare_net(net, 2, flags=KEEP, x=x[:2], ref=ref64)
    assert n == len(net['layers'])
    compare_net(net, 2, flags=0, x=x[:2], ref=ref64)
    compare_net(net, 3, flags=0, x=x)     # an odd batch in the shipped configuration
    if 'resnet' in name:
        n, eng = compare_net(net, 2, flags=runtime.FUSE_FIRST_POOL, x=x[:2], ref=ref64)   # first layer + pooling as one kernel
        assert 'stem-pool-tcgen05' in eng


def _slice_bounds(batch, nslices):
    wsum = 2 * nslices - 1
    return [batch * 2 * k // wsum for k in range(1, nslices)]


def _entry_points_agree(net, batch, picks_extra=()):
    """forward (device buffers), forward_host (sliced upload) and submit_host / wait (streaming) on the same
    batch; oracle on picked images."""
    import torch
    x = netdesc.make_input(net, batch, seed=1234)
    qn = runtime.QuantizedNet(net, batch)
    try:
        h_in = torch.from_numpy(x.view(np.uint8)).pin_memory()
        d_in = h_in.cuda()
        d_out = torch.empty((batch, qn.out_elems), dtype=torch.int8, device='cuda')
        qn.forward_device(d_in.data_ptr(), batch, d_out.data_ptr(), 0)
        qn.check(0)
        dev = d_out.cpu().numpy()
        host = qn.forward_host(x).view(np.int8)
        assert np.array_equal(host, dev), 'host-buffer and device-buffer entry points differ'
        # streaming: three batches back to back through the two staging sets (third waits for the first)
        outs = [torch.empty((batch, qn.out_elems), dtype=torch.int8).pin_memory() for _ in range(3)]
        for o in outs:
            qn.submit_host_ptr(h_in.data_ptr(), batch, o.data_ptr(), 0)
        qn.wait()
        for o in outs:
            assert np.array_equal(o.numpy(), dev), 'streaming entry point differs'
    finally:
        qn.close()
    nslices = min(8, batch // 128) if batch >= 256 else 1
    picks = {0, batch - 1, *picks_extra}
    for b in _slice_bounds(batch, nslices):
        picks |= {b - 1, b}
    picks = sorted(picks)
    ref = oracle.run_net(net, x[picks], 'i64')[-1].reshape(len(picks), -1)
    assert np.array_equal(dev[picks].astype(np.int64), ref), 'picked images differ from the oracle'


def test_resnet50_two_upload_slices_at_batch_256():
    # the smallest batch that slices the upload: the leading cells (everything up to the second stage's first
    # 1x1) run once per slice at an image offset into shared buffers
    _entry_points_agree(FULL['resnet50_double'](), 256, picks_extra=(127, 128))


def test_resnet50_at_the_benchmark_batch():
    # 1024 images: eight upload slices, the 256-row variant on the large-K layers
    _entry_points_agree(FULL['resnet50_double'](), 1024)


def test_resnet18_w4_at_the_benchmark_batch():
    _entry_points_agree(FULL['resnet18_w4_clipped_fixed'](), 2048)
