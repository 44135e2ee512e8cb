"""Parity of the CUDA path with the CPU oracle, through the C ABI, bit for bit (integer work: no
tolerance).  Every network is compared cell by cell (KEEP_ALL_OUTPUTS | NO_FUSION) and again in the
shipped configuration (residual sums folded into the convolution epilogue, buffers reused)."""
import numpy as np
import pytest

from n2d2_b200 import netdesc, runtime
from oracle import oracle

from gpu_common import KEEP, compare_net, single_conv_net

# (C, H, W, O, k, pad, dilation, input unsigned): stride-1 layers small enough for resident weights
PATCH_CASES = [(64, 56, 56, 64, 3, 1, 1, True), (64, 20, 17, 64, 3, 1, 1, True), (32, 9, 9, 32, 3, 1, 1, False),
               (128, 12, 12, 64, 3, 1, 1, True), (32, 15, 15, 64, 5, 2, 1, True), (64, 20, 20, 64, 3, 2, 2, True),
               (64, 10, 10, 32, 3, 0, 1, True), (64, 6, 250, 64, 3, 1, 1, True), (64, 33, 29, 128, 2, 1, 1, False),
               (32, 40, 40, 96, 3, 1, 1, True),
               # weights beyond the resident limit: the tap blocks stream through a ring
               (128, 28, 28, 128, 3, 1, 1, True), (64, 14, 14, 128, 5, 2, 1, True), (128, 9, 33, 96, 3, 1, 1, False),
               (128, 5, 100, 96, 3, 1, 1, True),
               # streamed weights, bands of three and four tiles (one weight pass serves the whole band)
               (64, 30, 14, 128, 5, 2, 1, True), (128, 24, 28, 128, 3, 1, 1, False)]


@pytest.mark.parametrize('case', PATCH_CASES, ids=lambda c: 'C%d_%dx%d_O%d_k%d_p%d_d%d' % c[:7])
@pytest.mark.parametrize('mode', ['double', 'fixed'])
def test_stride1_patch_kernel(case, mode):
    C, H, W, O, k, p, d, uns = case
    net = single_conv_net(C, H, W, O, k, 1, p, in_unsigned=uns, mode=mode, dil=d)
    compare_net(net, 3, want_engine=None if mode == 'fixed' else 'patch-tcgen05')


def test_stride1_patch_kernel_many_bands_and_images():
    # more (image, band) items than SMs, a last band shorter than the others, linear activation (signed output)
    net = single_conv_net(64, 56, 56, 64, 3, 1, 1, in_unsigned=True, mode='single', act='linear')
    compare_net(net, 40, want_engine='patch-tcgen05')


def test_forced_im2col_keeps_the_implicit_gemm_kernel():
    net = single_conv_net(64, 20, 17, 64, 3, 1, 1, mode='double')
    compare_net(net, 2, flags=runtime.KEEP_ALL_OUTPUTS | runtime.FORCE_IM2COL, want_engine='tcgen05')


@pytest.mark.parametrize('slices', [2, 3, 5])
def test_host_entry_point_runs_the_leading_cells_slice_by_slice(slices):
    # at batch >= 256 the host-buffer entry point uploads the batch in slices and runs the leading cells
    # (here: all of them - im2col and 1x1 implicit GEMM, patch kernel, fused residual sum, pooling) per slice;
    # uneven slice sizes, every layer compared with the oracle
    b = netdesc.NetBuilder('sliced', 16, 48, 48, 11, 'double', weight_dist=('normal', 30))
    c0 = b.conv(-1, 64, 3, pad=1, name='c0')
    c1 = b.conv(c0, 64, 3, pad=1, name='c1')
    x4 = b.conv(c1, 128, 1, act='linear', name='x4')
    pj = b.conv(c0, 128, 1, act='linear', name='proj')
    sm = b.sum([x4, pj], act='relu', name='sum')
    b.pool(sm, 'max', 2, 2, name='pool')
    n, eng = compare_net(b.net, 261, flags=0, slices=slices)
    assert 'fused' in eng and 'patch-tcgen05' in eng and 'tcgen05' in eng
    compare_net(b.net, 261, slices=slices)     # and with every cell's output kept and compared


# (C, H, W, stride, pad, dilation, input unsigned, activation)
DW_CASES = [(32, 20, 20, 1, 1, 1, True, 'relu'), (64, 21, 19, 2, 1, 1, True, 'relu'), (16, 9, 9, 1, 0, 1, False, 'linear'),
            (128, 14, 14, 1, 1, 1, True, 'relu'), (512, 7, 9, 2, 1, 1, True, 'relu'), (1024, 7, 7, 1, 1, 1, True, 'linear'),
            (48, 13, 13, 1, 2, 2, True, 'relu'), (32, 5, 3, 1, 1, 1, False, 'relu')]


@pytest.mark.parametrize('case', DW_CASES, ids=lambda c: 'C%d_%dx%d_s%d_p%d_d%d' % c[:6])
@pytest.mark.parametrize('mode', ['single', 'double', 'fixed'])
def test_depthwise_3x3(case, mode):
    # the dot-product kernel (32-bit epilogue) and, with the exact-epilogue flag, the 64-bit kernel
    C, H, W, s, p, d, uns, act = case
    net = single_conv_net(C, H, W, C, 3, s, p, in_unsigned=uns, act=act, mode=mode, dil=d, groups=C)
    # layers with whole groups of 64 (or one of 32) channels, and stride-1 layers with groups of 32, run on the tensor
    # cores as block-diagonal groups
    on_tensor_cores = C % 64 == 0 or C == 32 or (s == 1 and C % 32 == 0)
    # (fixed-point scalings with wide shifts have no 32-bit epilogue and stay on the exact CUDA-core kernel)
    want = 'depthwise' if not on_tensor_cores else (('depthwise-tcgen05', 'depthwise') if mode == 'fixed' else 'depthwise-tcgen05')
    compare_net(net, 3, want_engine=want)
    compare_net(net, 3, flags=KEEP | R.FORCE_SIMT, want_engine='depthwise')
    compare_net(net, 3, flags=KEEP | R.EXACT64_EPILOGUE, want_engine='depthwise')


# (C, H, W, k, pad, dilation, batch): depthwise layers as block-diagonal groups on the tensor cores - several bands
# and images per CTA, more groups than fit the grid evenly, 5x5 and dilated filters, one group of 32
# (C, H, W, k, stride, pad, dilation, batch): the strided ones through im2col loads of the group's channel slice
DW_TC_STRIDED_CASES = [(64, 112, 112, 3, 2, 1, 1, 3), (128, 56, 56, 3, 2, 1, 1, 5), (256, 28, 28, 3, 2, 1, 1, 9),
                       (512, 14, 14, 3, 2, 1, 1, 37), (1024, 9, 7, 3, 2, 1, 1, 4), (32, 30, 30, 3, 2, 1, 1, 3),
                       (192, 17, 23, 5, 3, 2, 1, 3), (64, 40, 40, 3, 1, 0, 1, 2), (128, 9, 9, 3, 2, 1, 1, 1)]


@pytest.mark.parametrize('case', DW_TC_STRIDED_CASES, ids=lambda c: 'C%d_%dx%d_k%d_s%d_p%d_d%d_b%d' % c)
@pytest.mark.parametrize('mode', ['double', 'single'])
def test_strided_depthwise_as_block_diagonal_groups(case, mode):
    C, H, W, k, st, p, d, batch = case
    net = single_conv_net(C, H, W, C, k, st, p, mode=mode, dil=d, groups=C)
    compare_net(net, batch, want_engine='depthwise-tcgen05')


DW_TC_CASES = [(128, 56, 56, 3, 1, 1, 5), (512, 14, 14, 3, 1, 1, 37), (1024, 7, 7, 3, 1, 1, 9), (32, 112, 112, 3, 1, 1, 3),
               (96, 30, 17, 3, 1, 1, 4), (64, 20, 20, 5, 2, 1, 3), (192, 24, 24, 3, 2, 2, 3), (256, 28, 28, 3, 0, 1, 2),
               (64, 9, 9, 3, 1, 1, 1), (1024, 3, 3, 3, 1, 1, 1)]


@pytest.mark.parametrize('case', DW_TC_CASES, ids=lambda c: 'C%d_%dx%d_k%d_p%d_d%d_b%d' % c)
@pytest.mark.parametrize('mode', ['double', 'single'])
def test_depthwise_as_block_diagonal_groups_on_the_tensor_cores(case, mode):
    C, H, W, k, p, d, batch = case
    net = single_conv_net(C, H, W, C, k, 1, p, mode=mode, dil=d, groups=C)
    compare_net(net, batch, want_engine='depthwise-tcgen05')


# (C, H, W, O, k, stride, pad, input unsigned, builder keywords): layers the 256-row variant can take
# (weight blocks beyond the resident limit, 128-byte K slabs, 256-column tiles, no residual)
PAIR_CASES = [(512, 9, 9, 256, 1, 1, 0, True, {}), (256, 14, 14, 256, 3, 1, 1, True, {}),
              (128, 15, 15, 512, 3, 2, 1, True, {}), (512, 19, 19, 256, 1, 1, 0, False, {}),
              (1024, 7, 7, 512, 1, 1, 0, True, {'unsigned_relu': False}), (128, 20, 11, 256, 3, 1, 1, True, {})]


@pytest.mark.parametrize('case', PAIR_CASES, ids=lambda c: 'C%d_%dx%d_O%d_k%d_s%d' % c[:6])
@pytest.mark.parametrize('mode', ['double', 'single'])
def test_256_row_tiles(case, mode):
    C, H, W, O, k, s, p, uns, kw = case
    net = single_conv_net(C, H, W, O, k, s, p, in_unsigned=uns, mode=mode, **kw)
    compare_net(net, 3, flags=KEEP | R.FORCE_PAIR, want_engine='tcgen05-pair')
    compare_net(net, 5, flags=KEEP | R.FORCE_PAIR, want_engine='tcgen05-pair')   # another (odd) number of row tiles


pytestmark = pytest.mark.gpu
R = runtime


def test_config1_mnist24_single_shift_batch64():
    n, eng = compare_net(netdesc.mnist24(), 64)
    assert n == 4
    n, eng = compare_net(netdesc.mnist24(), 64, flags=KEEP | R.FORCE_SIMT)
    assert set(eng) == {'simt'}
    # the fp32-accumulating flavour (what the reference's CPU cells compute) gives the same integers here
    compare_net(netdesc.mnist24(), 64, flavour='f32')


@pytest.mark.parametrize('force', [0, R.FORCE_SIMT], ids=['tensor-core', 'cuda-core'])
@pytest.mark.parametrize('name', ['resnet50_double', 'resnet18_fixed', 'mobilenet_single', 'resnet18_w4_clipped_fixed',
                                  'resnet18_float_clipped', 'resnet18_signed', 'resnet18_per_channel_frac'])
def test_small_networks_cell_by_cell(name, force):
    net = {
        'resnet50_double': lambda: netdesc.resnet50(size=64, classes=100),
        'resnet18_fixed': lambda: netdesc.resnet18(size=64, classes=100),
        'mobilenet_single': lambda: netdesc.mobilenet_v1(size=64, classes=100),
        'resnet18_w4_clipped_fixed': lambda: netdesc.resnet18(size=64, classes=100, weight_bits=4, clipped=True),
        'resnet18_float_clipped': lambda: netdesc.resnet18(size=48, classes=10, scaling='float', clipped=True),
        'resnet18_signed': lambda: netdesc.resnet18(size=48, classes=10, unsigned_relu=False),
        'resnet18_per_channel_frac': lambda: netdesc.resnet18(size=48, classes=10, per_channel_frac=True),
    }[name]()
    n, eng = compare_net(net, 3, flags=KEEP | force)
    assert n == len(net['layers'])
    if not force and 'resnet' in name:
        assert any(e.startswith('tcgen05') for e in eng)


@pytest.mark.parametrize('name', ['resnet50', 'resnet18', 'mobilenet'])
def test_small_networks_shipped_configuration(name):
    net = {'resnet50': lambda: netdesc.resnet50(size=64, classes=100),
           'resnet18': lambda: netdesc.resnet18(size=64, classes=100),
           'mobilenet': lambda: netdesc.mobilenet_v1(size=64, classes=100)}[name]()
    n, eng = compare_net(net, 5, flags=0)
    if name != 'mobilenet':
        assert 'fused' in eng     # residual sums ride in the convolution epilogue


# (C, H, O, k, stride, pad, input unsigned, flags)
TC_CASES = [
    (64, 8, 64, 1, 1, 0, True, 0), (128, 8, 256, 1, 1, 0, True, 0), (256, 9, 64, 1, 1, 0, False, 0),
    (32, 8, 64, 1, 1, 0, True, 0), (16, 9, 32, 1, 1, 0, True, 0), (48, 9, 32, 3, 1, 1, True, 0),
    (512, 7, 2048, 1, 1, 0, True, 0), (64, 8, 64, 1, 1, 0, True, R.FORCE_IM2COL), (64, 8, 64, 3, 1, 1, True, 0),
    (128, 15, 128, 3, 2, 1, True, 0), (256, 14, 512, 1, 2, 0, False, 0), (64, 55, 64, 3, 1, 1, True, 0),
    (64, 28, 1000, 1, 1, 0, True, 0), (64, 13, 72, 3, 1, 1, True, 0), (192, 7, 96, 5, 2, 2, True, 0),
    (64, 12, 64, 3, 1, 2, True, 0),
]


@pytest.mark.parametrize('case', TC_CASES, ids=lambda c: 'C%d_H%d_O%d_k%d_s%d_p%d_%s_f%d' % (
    c[0], c[1], c[2], c[3], c[4], c[5], 'u8' if c[6] else 's8', c[7]))
def test_tensor_core_convolutions(case):
    C, H, O, k, s, p, uns, flags = case
    net = single_conv_net(C, H, H, O, k, s, p, in_unsigned=uns)
    # stride-1 layers with few channels and resident weights take the patch kernel unless im2col is forced
    patch = (s == 1 and k > 1 and C in (32, 64, 128) and O % 32 == 0 and O <= 128 and not flags & R.FORCE_IM2COL)
    compare_net(net, 3, flags=KEEP | flags, want_engine='patch-tcgen05' if patch else 'tcgen05')
    if patch:
        compare_net(net, 3, flags=KEEP | R.FORCE_IM2COL, want_engine='tcgen05')


@pytest.mark.parametrize('mode', ['double', 'single', 'fixed'])
@pytest.mark.parametrize('t_act', ['linear', 'relu'])
@pytest.mark.parametrize('r_act', ['linear', 'relu'])
def test_fused_residual_sum_all_sign_combinations(mode, t_act, r_act):
    # conv (signed or unsigned output) + residual operand (signed or unsigned) -> second requantisation,
    # folded into the convolution's epilogue; several widths so that every column slice size occurs
    for O in (64, 128, 256):
        b = netdesc.NetBuilder('res', 64, 9, 9, 5, mode, weight_dist=('normal', 30))
        r = b.conv(-1, O, 1, act=r_act)
        t = b.conv(r, O, 3, pad=1, act=t_act)
        b.sum([t, r], act='relu')
        n, eng = compare_net(b.net, 3, flags=0)
        assert 'fused' in eng
        compare_net(b.net, 3)     # and cell by cell, unfused


def test_exact64_epilogue_matches_too():
    # the tensor-core cells default to the 32-bit epilogue wherever it is provably exact; the 64-bit
    # form must give the same integers
    for net in (netdesc.resnet50(size=64, classes=100), netdesc.resnet18(size=64, classes=100, clipped=True)):
        compare_net(net, 3, flags=KEEP | R.EXACT64_EPILOGUE, want_engine='tcgen05')
        compare_net(net, 3, flags=R.EXACT64_EPILOGUE)


def test_wide_shifts_fall_back_to_the_exact_epilogue():
    # fractional bits beyond what 32-bit products can hold
    net = single_conv_net(64, 9, 9, 64, 3, 1, 1, mode='fixed')
    q = net['layers'][0]['quant']
    q['mult'] = (q['mult'].astype(np.int64) << 14).astype(np.int32)
    q['frac_bits'] = int(q['frac_bits']) + 14
    compare_net(net, 2, want_engine='tcgen05')


# (C, H, W, O, k, stride, pad, input unsigned)
STEM_CASES = [(3, 32, 32, 64, 7, 2, 3, True), (3, 224, 224, 64, 7, 2, 3, True), (3, 33, 29, 32, 3, 2, 1, True),
              (1, 24, 24, 32, 4, 2, 0, True), (4, 17, 19, 64, 5, 1, 2, False), (2, 16, 16, 96, 8, 3, 0, True),
              (3, 20, 20, 128, 3, 1, 1, True)]


@pytest.mark.parametrize('case', STEM_CASES, ids=lambda c: 'C%d_%dx%d_O%d_k%d_s%d_p%d' % c[:7])
@pytest.mark.parametrize('mode', ['double', 'single', 'fixed'])
def test_first_layer_tensor_core_kernel(case, mode):
    C, H, W, O, k, s, p, uns = case
    net = single_conv_net(C, H, W, O, k, s, p, in_unsigned=uns, mode=mode)
    # wide fixed-point shifts need 64-bit products: those cells take the exact CUDA-core kernel
    compare_net(net, 3, want_engine=None if mode == 'fixed' else 'stem-tcgen05')


def test_tensor_core_dilated_convolution():
    net = single_conv_net(64, 15, 15, 64, 3, 1, 2, dil=2)
    compare_net(net, 2, flags=KEEP | R.FORCE_IM2COL, want_engine='tcgen05')
    compare_net(net, 2, want_engine='patch-tcgen05')


@pytest.mark.parametrize('mode', ['single', 'double', 'fixed', 'float'])
@pytest.mark.parametrize('act', ['relu', 'linear'])
def test_every_scaling_mode_on_both_kernel_families(mode, act):
    for flags in (KEEP, KEEP | R.FORCE_SIMT):
        net = single_conv_net(64, 9, 9, 80, 3, 1, 1, mode=mode, act=act, clipped=(mode in ('fixed', 'float')))
        compare_net(net, 2, flags=flags)


def test_direct_kernels_odd_geometries():
    # few channels, groups, no bias, rectangular pooling, odd channel counts
    for net in (single_conv_net(3, 17, 13, 5, 3, 2, 1), single_conv_net(6, 9, 9, 9, 3, 1, 1, groups=3),
                single_conv_net(16, 9, 9, 16, 3, 1, 1, groups=16), single_conv_net(5, 8, 8, 7, 2, 2, 0, bias=False),
                single_conv_net(1, 24, 24, 16, 4, 2, 0)):
        compare_net(net, 2)
    b = netdesc.NetBuilder('pools', 5, 11, 9, 3, 'single')
    x = b.conv(-1, 7, 3, pad=1)
    b.pool(x, 'max', (3, 2), 2, pad=1)
    b.pool(x, 'avg', (2, 3), 1)
    compare_net(b.net, 2)


def test_scaling_cell_and_int32_outputs():
    # a cell without Scaling leaves int32 accumulators; a ScalingCell brings them back to 8 bits
    b = netdesc.NetBuilder('raw', 32, 6, 6, 11, 'fixed')
    x = b.conv(-1, 32, 3, pad=1, act='linear')
    b.net['layers'][0]['quant'] = {'mode': 'none', 'act': 'linear'}
    y = b.scaling(x, act='relu')
    b.net['layers'][1]['quant']['mult'] = (b.net['layers'][1]['quant']['mult'] // 4096).astype(np.int32) + 1
    b.net['layers'][1]['quant']['frac_bits'] = 14
    compare_net(b.net, 2)


def test_batch_edges_and_errors():
    net = netdesc.resnet18(size=32, classes=10)
    qn = runtime.QuantizedNet(net, 4)
    x = netdesc.make_input(net, 4)
    ref = oracle.run_net(net, x, 'i64')[-1].reshape(4, -1)
    full = qn.forward_host(x).astype(np.int64)
    assert np.array_equal(full, ref)
    one = qn.forward_host(x[:1]).astype(np.int64)           # ragged: fewer images than max_batch
    assert np.array_equal(one, ref[:1])
    assert qn.forward_host(x[:0]).shape[0] == 0              # empty batch is a no-op
    with pytest.raises(runtime.N2D2BError, match='exceeds'):
        qn.forward_host(netdesc.make_input(net, 5))
    qn.close()
    bad = netdesc.mnist24()
    bad['layers'][0]['groups'] = 3                           # does not divide 1 channel / 16 outputs
    with pytest.raises(runtime.N2D2BError, match='groups'):
        runtime.QuantizedNet(bad, 1)
    bad = netdesc.mnist24()
    bad['layers'][0]['quant']['out_bits'] = 12               # beyond what an 8-bit tensor holds
    with pytest.raises(runtime.N2D2BError, match='out_bits'):
        runtime.QuantizedNet(bad, 1)


def test_batch_invariance_at_a_large_batch():
    # size-independent property: an image's logits do not depend on what else is in the batch, so a
    # large batch can be checked image by image against small-batch oracle runs
    net = netdesc.resnet50(size=96, classes=100)
    big = 300
    x = netdesc.make_input(net, big)
    qn = runtime.QuantizedNet(net, big)
    out = qn.forward_host(x).astype(np.int64)
    qn.close()
    picks = [0, 1, 127, 128, 255, 299]
    ref = oracle.run_net(net, x[picks], 'i64')[-1].reshape(len(picks), -1)
    assert np.array_equal(out[picks], ref)


def _saturating(net, thr):
    """Turns every cell's activation into Saturation(+-thr) (signed outputs)."""
    for l in net['layers']:
        if 'quant' in l and l['quant']['mode'] != 'none':
            l['quant']['act'] = 'saturation'
            l['quant']['sat_thr'] = thr
            l['quant']['out_unsigned'] = False
    return net


# one case per kernel family: (what, builder of a one-cell network, engine expected in the shipped configuration)
SAT_CASES = [
    ('igemm', lambda m: single_conv_net(64, 9, 9, 80, 3, 1, 1, mode=m), 'tcgen05'),
    ('igemm_1x1_wide', lambda m: single_conv_net(128, 8, 8, 256, 1, 1, 0, mode=m), 'tcgen05'),
    ('patch', lambda m: single_conv_net(64, 20, 17, 64, 3, 1, 1, mode=m), 'patch-tcgen05'),
    ('stem_s2d', lambda m: single_conv_net(3, 32, 32, 64, 7, 2, 3, mode=m), 'stem-tcgen05'),
    ('stem_gather', lambda m: single_conv_net(4, 17, 19, 64, 5, 1, 2, mode=m), 'stem-tcgen05'),
    ('depthwise', lambda m: single_conv_net(48, 20, 20, 48, 3, 2, 1, mode=m, groups=48), 'depthwise'),
    ('depthwise-tc-strided', lambda m: single_conv_net(128, 20, 20, 128, 3, 2, 1, mode=m, groups=128), 'depthwise-tcgen05'),
    ('depthwise-tc', lambda m: single_conv_net(64, 20, 20, 64, 3, 1, 1, mode=m, groups=64), 'depthwise-tcgen05'),
    ('direct', lambda m: single_conv_net(3, 17, 13, 5, 3, 2, 1, mode=m), 'simt'),
]


@pytest.mark.parametrize('case', SAT_CASES, ids=lambda c: c[0])
@pytest.mark.parametrize('mode', ['single', 'double', 'fixed', 'float'])
def test_saturation_activation_on_every_kernel_family(case, mode):
    # SaturationActivation: Scaling (saturating to the output range) then a clamp to +-threshold
    # (include/Activation/SaturationActivation_Frame.hpp:55-80 of the reference)
    _, build, engine = case
    for thr in (50, 127):
        net = _saturating(build(mode), thr)
        # float scalings and wide fixed-point shifts take the exact 64-bit kernels, whatever the family
        exact_only = mode == 'float' or (mode == 'fixed' and engine in ('stem-tcgen05', 'patch-tcgen05', 'depthwise-tcgen05'))
        compare_net(net, 3, want_engine=None if exact_only else engine)
        compare_net(net, 3, flags=KEEP | R.FORCE_SIMT)
        ref = oracle.run_net(net, netdesc.make_input(net, 3), 'i64')[-1]
        assert int(np.abs(ref).max()) <= thr


def test_saturation_activation_in_a_network_with_fused_sums_fc_and_scaling_cell():
    b = netdesc.NetBuilder('sat', 64, 12, 12, 9, 'double', weight_dist=('normal', 30))
    r = b.conv(-1, 128, 1, act='linear')
    t = b.conv(r, 128, 3, pad=1, act='linear')
    s = b.sum([t, r], act='linear')
    y = b.scaling(s, act='linear', mode='fixed')
    p = b.pool(y, 'avg', (12, 12), 1)
    b.fc(p, 16, act='linear')
    net = _saturating(b.net, 90)
    n, eng = compare_net(net, 3, flags=0)
    assert 'fused' in eng
    compare_net(net, 3)


def test_a_bounded_wait_that_runs_out_is_reported_and_leaves_the_network_usable():
    # The device-side waits of the tensor-core kernels give up after a time limit instead of hanging.  A
    # test hook makes exactly that happen, harmlessly (a one-CTA kernel waits 1 ms on a barrier nobody
    # arrives at and returns): the asynchronous entry point cannot know, the check reports it once, and
    # the next forward pass is correct.
    net = netdesc.resnet50(size=64, classes=100)
    x = netdesc.make_input(net, 2)
    ref = oracle.run_net(net, x, 'i64')[-1].reshape(2, -1)
    qn = runtime.QuantizedNet(net, 2)
    try:
        assert np.array_equal(qn.forward_host(x).astype(np.int64), ref)
        qn.check(0)                                   # nothing pending
        qn.selftest_wait_timeout(1000, 0)
        with pytest.raises(runtime.N2D2BError, match='status -4'):
            qn.check(0)
        qn.check(0)                                   # reported once, then clear
        qn.selftest_wait_timeout(500, 0)
        with pytest.raises(runtime.N2D2BError, match='gave up waiting'):
            qn.forward_host(x)                        # the blocking entry points make the same check
        assert np.array_equal(qn.forward_host(x).astype(np.int64), ref)
    finally:
        qn.close()


def test_output_edge_estimated_labels_first_maximum_wins():
    # Target top-1 (src/Target/Target_CUDA_kernels.cu:88-104 of the reference): strict '>' while scanning the
    # classes in order, so the lowest index among equal scores wins; int8 logits tie often
    import torch
    net = netdesc.resnet18(size=32, classes=1000)
    batch = 7
    x = netdesc.make_input(net, batch)
    ref = oracle.run_net(net, x, 'i64')[-1].reshape(batch, -1)
    qn = runtime.QuantizedNet(net, batch)
    try:
        d_in = torch.from_numpy(x).cuda()
        d_out = torch.empty((batch, qn.out_elems), dtype=torch.int8, device='cuda')
        labels = torch.full((batch,), -1, dtype=torch.int32, device='cuda')
        values = torch.zeros((batch,), dtype=torch.int32, device='cuda')
        qn.forward_device(d_in.data_ptr(), batch, d_out.data_ptr(), 0)
        qn.estimated_labels(batch, labels.data_ptr(), values.data_ptr(), 0)
        qn.check(0)
        assert np.array_equal(d_out.cpu().numpy().astype(np.int64), ref)
        assert np.array_equal(labels.cpu().numpy(), ref.argmax(axis=1))       # numpy's argmax is first-maximum too
        assert np.array_equal(values.cpu().numpy(), ref.max(axis=1))
        assert (ref == ref.max(axis=1, keepdims=True)).sum(axis=1).max() > 1  # the case does contain ties
    finally:
        qn.close()


def test_input_edge_quantizes_float_stimuli_like_the_range_transform():
    # src/DeepNetQuantization.cpp:359-370: x * (2^n - 1) (unsigned) or x * (2^(n-1) - 1) (signed), truncated;
    # NCHW float in, NHWC 8-bit out
    import torch
    rng = np.random.Generator(np.random.PCG64(3))
    x = rng.integers(0, 256, size=(3, 3, 9, 7)).astype(np.float32) / np.float32(255.0)    # 8-bit images scaled to [0, 1]
    x[0, 0, 0, :4] = [0.5, 0.999, 1.5, -0.2]                                             # plus values that truncate / saturate
    d_in = torch.from_numpy(x).cuda()
    for unsigned, factor, lo, hi, dt in ((True, 255.0, 0, 255, np.uint8), (False, 127.0, -128, 127, np.int8)):
        xs = x if unsigned else x * 2 - 1
        d_in = torch.from_numpy(np.ascontiguousarray(xs)).cuda()
        d_out = torch.zeros((3, 9, 7, 3), dtype=torch.uint8, device='cuda')
        runtime.quantize_stimuli(d_in.data_ptr(), 3, 3, 9, 7, d_out.data_ptr(), 8, unsigned)
        torch.cuda.synchronize()
        want = np.clip(np.trunc(xs.astype(np.float32) * np.float32(factor)), lo, hi).astype(dt).transpose(0, 2, 3, 1)
        assert np.array_equal(d_out.cpu().numpy().view(dt), want)


# (C, H, O, k, stride, pad, input unsigned): 4-bit weights, packed two per byte in HBM and expanded in the kernel
W4_CASES = [(64, 8, 64, 1, 1, 0, True), (128, 8, 256, 1, 1, 0, True), (32, 9, 32, 3, 1, 1, True), (256, 14, 512, 1, 2, 0, False),
            (64, 30, 64, 3, 1, 1, True), (512, 7, 1024, 1, 1, 0, True), (128, 15, 128, 3, 2, 1, True), (256, 9, 256, 3, 1, 1, True)]


@pytest.mark.parametrize('case', W4_CASES, ids=lambda c: 'C%d_H%d_O%d_k%d_s%d' % c[:5])
@pytest.mark.parametrize('mode', ['double', 'fixed', 'single'])
def test_packed_int4_weights_on_the_tensor_cores(case, mode):
    C, H, O, k, s, p, uns = case
    for clipped in ((False, True) if mode == 'fixed' else (False,)):
        net = single_conv_net(C, H, H, O, k, s, p, in_unsigned=uns, mode=mode, weight_bits=4, clipped=clipped)
        compare_net(net, 3, want_engine='tcgen05-w4')
        compare_net(net, 3, flags=KEEP | R.EXACT64_EPILOGUE, want_engine='tcgen05-w4')


def test_packed_int4_rows_that_tma_cannot_address_are_widened():
    # a packed row of kH * kW * Cin / 2 bytes must be a multiple of 16 bytes for the tensor map; other cells hold int8
    net = single_conv_net(48, 9, 9, 32, 3, 1, 1, mode='double', weight_bits=4)
    n, eng = compare_net(net, 3)
    assert eng == ['tcgen05']


def test_packed_int4_weights_stay_packed_in_hbm_and_fuse_residuals():
    net = netdesc.resnet18(size=64, classes=100, weight_bits=4, clipped=True)
    n, eng = compare_net(net, 3, flags=0)
    assert 'fused' in eng
    qn = runtime.QuantizedNet(net, 3)
    try:
        total, packed = qn.weight_bytes()
        eng = qn.engines()
    finally:
        qn.close()
    w4 = [l for l, e in zip(net['layers'], eng) if e == 'tcgen05-w4']
    # every convolution but the three-channel first layer, and the classifier, hold half a byte per weight
    assert len(w4) == sum(1 for l in net['layers'] if l['type'] in ('conv', 'fc')) - 1
    assert packed == sum(int(l['weights'].size) for l in w4) // 2
    assert packed > 0.95 * total
    # a network given the same weights unpacked holds twice as much
    qn8 = runtime.QuantizedNet(net, 3, pack4=False)
    try:
        total8, packed8 = qn8.weight_bytes()
    finally:
        qn8.close()
    assert packed8 == 0 and total8 >= 2 * packed
    # residual sums in both signedness combinations, unclipped scalings (the dot-product epilogue)
    for mode in ('double', 'single'):
        net = netdesc.resnet18(size=48, classes=10, weight_bits=4, scaling=mode)
        n, eng = compare_net(net, 3, flags=0)
        assert 'fused' in eng and 'tcgen05-w4' in eng


# (C, H, W, O, k, pad, activation, pooling window, pooling stride, input unsigned)
STEM_POOL_CASES = [(3, 64, 64, 64, 7, 3, 'relu', 3, 2, True), (3, 224, 224, 64, 7, 3, 'relu', 3, 2, True),
                   (3, 33, 29, 32, 3, 1, 'relu', 2, 2, True), (1, 24, 24, 32, 4, 0, 'linear', 2, 2, True),
                   (4, 40, 36, 128, 5, 2, 'linear', 3, 2, False), (3, 50, 50, 96, 7, 3, 'relu', 3, 3, True),
                   (3, 31, 47, 64, 3, 1, 'relu', 2, 1, True), (2, 20, 20, 64, 8, 0, 'relu', 4, 2, True)]


@pytest.mark.parametrize('case', STEM_POOL_CASES, ids=lambda c: 'C%d_%dx%d_O%d_k%d_p%d_%s_pool%d_s%d' % c[:9])
@pytest.mark.parametrize('mode', ['double', 'single'])
def test_first_layer_with_the_max_pooling_folded_in(case, mode):
    # stride-2 first layer + max pooling as one kernel (opt-in): the pooled tensor is all that reaches HBM
    C, H, W, O, k, p, act, pk, ps, uns = case
    b = netdesc.NetBuilder('stempool', C, H, W, 13, mode, input_unsigned=uns, weight_dist=('normal', 30))
    c = b.conv(-1, O, k, stride=2, pad=p, act=act, name='conv1')
    b.pool(c, 'max', pk, ps, name='pool1')
    for batch in (1, 5):
        n, eng = compare_net(b.net, batch, flags=R.FUSE_FIRST_POOL)
        assert eng == ['stem-pool-tcgen05', 'fused']
    compare_net(b.net, 3)     # and as two cells, every output kept


@pytest.mark.parametrize('bits,unsigned', [(4, True), (4, False), (2, True), (5, False), (1, True)])
def test_activations_below_eight_bits(bits, unsigned):
    # mixed-precision networks of the QAT fusion carry their own activation bit width (the saturation range of the
    # Scaling, include/Activation/RectifierActivation_Frame.hpp:65-66): values stay one per byte on the device
    b = netdesc.NetBuilder('lowbits', 32, 10, 10, 17, 'fixed', weight_dist=('uniform', 7), weight_bits=4)
    c1 = b.conv(-1, 64, 3, pad=1, act='relu' if unsigned else 'linear', name='c1')
    c2 = b.conv(c1, 64, 1, act='relu' if unsigned else 'linear', name='c2')
    b.pool(c2, 'max', 2, 2, name='p')
    for l in b.net['layers'][:2]:
        l['quant']['out_bits'] = bits
        l['quant']['out_unsigned'] = unsigned
    x = netdesc.make_input(b.net, 3)
    ref = oracle.run_net(b.net, x, 'i64')
    lo, hi = (0, 2 ** bits - 1) if unsigned else (-2 ** (bits - 1), 2 ** (bits - 1) - 1)
    assert ref[1].min() >= lo and ref[1].max() <= hi and (ref[1].max() == hi or bits > 4)
    compare_net(b.net, 3, x=x, ref=ref)
    compare_net(b.net, 3, flags=0, x=x, ref=ref)


# (C, H, W, O, k, pad): output channels that are not a multiple of 32 (and of 16, and of 8)
ODD_O_CASES = [(64, 20, 20, 40, 1, 0), (64, 9, 9, 36, 1, 0), (32, 12, 12, 100, 3, 1), (128, 7, 7, 1000, 1, 0),
               (16, 10, 10, 7, 3, 1)]


@pytest.mark.parametrize('case', ODD_O_CASES, ids=lambda c: 'C%d_%dx%d_O%d_k%d' % c[:5])
@pytest.mark.parametrize('mode', ['double', 'fixed'])
def test_output_channels_that_tma_stores_cannot_address_run_padded(case, mode):
    # such a cell takes the 32-bit epilogue on zero-padded weight rows and a copy kernel drops the padding
    C, H, W, O, k, pad = case
    net = single_conv_net(C, H, W, O, k, 1, pad, mode=mode)
    n, eng = compare_net(net, 5)
    assert eng == ['tcgen05']
    qn = runtime.QuantizedNet(net, 5)
    try:
        assert qn.launches_per_forward() == 2
    finally:
        qn.close()
    # the exact 64-bit epilogue needs no padding
    n, eng = compare_net(net, 5, flags=KEEP | R.EXACT64_EPILOGUE)
    assert eng == ['tcgen05']


def test_padded_output_channels_in_upload_slices():
    net = single_conv_net(16, 48, 48, 24, 3, 1, 1, mode='double')
    compare_net(net, 7, slices=3)


@pytest.mark.parametrize('classes,top_n,size', [(1000, 5, 32), (10, 10, 32), (37, 3, 48), (1000, 1, 32)])
def test_output_edge_top_n_in_the_order_the_reference_sort_leaves(classes, top_n, size):
    # Target top-N (src/Target/Target_CUDA_kernels.cu:44-86): an exchange sort whose order among equal scores is
    # neither by class nor stable; the oracle replays it literally, the device evaluates it in closed form
    import torch
    net = netdesc.resnet18(size=size, classes=classes)
    batch = 9
    x = netdesc.make_input(net, batch)
    ref = oracle.run_net(net, x, 'i64')[-1].reshape(batch, -1)
    want_l, want_v = oracle.estimated_labels_topn(ref, top_n)
    qn = runtime.QuantizedNet(net, batch)
    try:
        d_in = torch.from_numpy(x).cuda()
        d_out = torch.empty((batch, qn.out_elems), dtype=torch.int8, device='cuda')
        labels = torch.full((batch, top_n), -1, dtype=torch.int32, device='cuda')
        values = torch.zeros((batch, top_n), dtype=torch.int32, device='cuda')
        qn.forward_device(d_in.data_ptr(), batch, d_out.data_ptr(), 0)
        qn.estimated_labels_topn(batch, top_n, labels.data_ptr(), values.data_ptr(), 0)
        qn.check(0)
        assert np.array_equal(values.cpu().numpy(), want_v)
        assert np.array_equal(labels.cpu().numpy(), want_l)
        if top_n > 1 and classes > 100:
            # the case does contain ties inside the top-N, and their order is not the ascending class order
            tied = [(want_v[b][:-1] == want_v[b][1:]).any() for b in range(batch)]
            assert any(tied)
        with pytest.raises(runtime.N2D2BError):
            qn.estimated_labels_topn(batch, classes + 1, labels.data_ptr(), values.data_ptr(), 0)
    finally:
        qn.close()


def test_output_edge_top_n_per_pixel_of_a_score_map():
    # a fully convolutional head: top-N per pixel, output [image][k][y][x]; int8 maps with few levels tie everywhere
    import torch
    net = single_conv_net(16, 12, 10, 21, 3, 1, 1, mode='single', act='linear')
    batch, top_n = 4, 4
    x = netdesc.make_input(net, batch)
    ref = oracle.run_net(net, x, 'i64')[-1]                      # [B][H][W][C]
    B, H, W, Cn = ref.shape
    assert (H, W, Cn) == (12, 10, 21)
    want_l, want_v = oracle.estimated_labels_topn(ref.reshape(B * H * W, Cn), top_n)
    qn = runtime.QuantizedNet(net, batch)
    try:
        qn.forward_host(x)
        labels = torch.full((B, top_n, H, W), -1, dtype=torch.int32, device='cuda')
        values = torch.zeros((B, top_n, H, W), dtype=torch.int32, device='cuda')
        qn.estimated_labels_topn(batch, top_n, labels.data_ptr(), values.data_ptr(), 0)
        qn.check(0)
        # the host-buffer form returns the same arrays
        host_l, host_v = qn.estimated_labels_topn_host(batch, top_n)
        assert np.array_equal(host_l, labels.cpu().numpy()) and np.array_equal(host_v, values.cpu().numpy())
        got_l = labels.cpu().numpy().transpose(0, 2, 3, 1).reshape(B * H * W, top_n)
        got_v = values.cpu().numpy().transpose(0, 2, 3, 1).reshape(B * H * W, top_n)
        assert np.array_equal(got_v, want_v)
        assert np.array_equal(got_l, want_l)
    finally:
        qn.close()


def _identity_scores_net(classes, H, W):
    """A network whose final tensor is its (signed 8-bit) input: a 1x1 convolution with identity weights, no bias and
    a shift of zero."""
    net = single_conv_net(classes, H, W, classes, 1, 1, 0, in_unsigned=False, act='linear', mode='single', bias=False)
    l = net['layers'][0]
    l['weights'] = np.eye(classes, dtype=np.int8).reshape(classes, 1, 1, classes)
    l['bias'] = None
    l['quant']['shift0'] = np.zeros(classes, np.uint8)
    l['quant']['out_unsigned'] = False
    return net


@pytest.mark.parametrize('classes,top_n,hw', [(1000, 5, (1, 1)), (10, 10, (1, 1)), (21, 4, (12, 10)), (150, 3, (5, 7))])
def test_top_n_order_against_the_reference_kernel_itself(classes, top_n, hw):
    # The reference's cudaGetEstimatedTarget kernel, compiled from the reference tree where that tree is, run here on
    # int8-like scores full of ties: the oracle's literal replay of its sort and the device's closed form must both
    # return its labels.
    from oracle import refshim
    if not refshim.target_available():
        pytest.skip('the reference tree was not compiled for this machine')
    import torch
    H, W = hw
    rng = np.random.default_rng(classes * 7 + top_n)
    B = 6
    levels = 9 if classes > 100 else 5                       # few score levels: ties in every top-N
    scores = rng.integers(-levels, levels + 1, (B, H, W, classes)).astype(np.int64)
    ref_l, ref_v = refshim.estimated_target(scores.transpose(0, 3, 1, 2).astype(np.float32), top_n)
    ora_l, ora_v = oracle.estimated_labels_topn(scores.reshape(B * H * W, classes), top_n)
    ora_l = ora_l.reshape(B, H, W, top_n).transpose(0, 3, 1, 2)
    ora_v = ora_v.reshape(B, H, W, top_n).transpose(0, 3, 1, 2)
    assert np.array_equal(ref_v.astype(np.int64), ora_v)
    assert np.array_equal(ref_l, ora_l)
    # the device entry point works on a network's final tensor: a 1x1 convolution that copies its input (identity
    # weights, unit scaling) puts exactly these scores there
    net = _identity_scores_net(classes, H, W)
    qn = runtime.QuantizedNet(net, B)
    try:
        out = qn.forward_host(scores.astype(np.int8))
        assert np.array_equal(out.reshape(B, H, W, classes).astype(np.int64), scores)
        got_l, got_v = qn.estimated_labels_topn_host(B, top_n)
        assert np.array_equal(got_v.astype(np.int64), ora_v)
        assert np.array_equal(got_l, ref_l)
    finally:
        qn.close()


@pytest.mark.parametrize('C,O,k', [(64, 96, 3), (16, 24, 5), (128, 128, 1), (3, 20, 3)])
def test_sparse_connection_map(C, O, k):
    # the reference's Cell mapping (Mapping(...) of its ini files): channels an output is not connected to are skipped
    # by its kernels; the device runs the dense layer with zero weights there
    net = single_conv_net(C, 14, 15, O, k, 1, k // 2, mode='double')
    rng = np.random.default_rng(C + O)
    maps = (rng.random((O, C)) < 0.35).astype(np.uint8)
    maps[np.arange(O), rng.integers(0, C, O)] = 1
    net['layers'][0]['maps'] = maps
    compare_net(net, 5)


@pytest.mark.parametrize('bits', [2, 1])
@pytest.mark.parametrize('case', [(64, 12, 12, 64, 3, 1, 1), (3, 15, 13, 10, 3, 2, 1), (32, 9, 9, 40, 1, 1, 0), (16, 8, 8, 24, 5, 1, 2)],
                         ids=lambda c: 'C%d_%dx%d_O%d_k%d' % c[:5])
def test_packed_two_bit_and_one_bit_weights(case, bits):
    # the export's data<2> / data<1> packing (four / eight weights per byte, first in the highest bits, rows starting on
    # a byte, 1-bit weights -1 / +1) through the C ABI; rows of 27 or 25 weights end in a partly filled byte
    C, H, W, O, k, s, p = case
    net = single_conv_net(C, H, W, O, k, s, p, mode='double', weight_bits=bits)
    w = net['layers'][0]['weights']
    assert w.min() >= (-2 if bits == 2 else -1) and w.max() <= 1 and (bits == 2 or not (w == 0).any())
    compare_net(net, 3)


def test_networks_with_two_bit_and_one_bit_weights():
    for bits in (2, 1):
        net = netdesc.resnet18(size=32, classes=10, weight_bits=bits, scaling='double')
        n, eng = compare_net(net, 3, flags=0)
        assert 'fused' in eng
