"""Import of the reference's on-disk forms (n2d2_b200/host/ExportImport.hpp): the per-cell headers of the
CPP_Quantization export and `.syntxt` parameter files.  The committed fixture
(tests/golden/export_fixture, written by tests/golden/make_export_fixture.py in the reference's format)
is read by a C++ program; what it reads must equal the network the fixture was written from, and the
network rebuilt from the headers must compute what the oracle computes for that network."""
import importlib.util
import os
import subprocess

import numpy as np
import pytest

from n2d2_b200 import netdesc, runtime

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, 'tests', 'host', 'test_export_import')
FIXTURE = os.path.join(ROOT, 'tests', 'golden', 'export_fixture')


def _fixture_net():
    spec = importlib.util.spec_from_file_location('make_export_fixture', os.path.join(ROOT, 'tests', 'golden', 'make_export_fixture.py'))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod, mod.fixture_net()


def _build():
    src = os.path.join(ROOT, 'tests', 'host', 'test_export_import.cpp')
    deps = [src, os.path.join(ROOT, 'n2d2_b200', 'host', 'N2D2.hpp'), os.path.join(ROOT, 'n2d2_b200', 'host', 'ExportImport.hpp'),
            os.path.join(ROOT, 'include', 'n2d2b.h'), runtime.LIB_PATH]
    if os.path.exists(EXE) and all(os.path.getmtime(EXE) > os.path.getmtime(d) for d in deps):
        return
    env = {k: v for k, v in os.environ.items() if k not in ('CC', 'CXX')}
    subprocess.check_call(['g++', '-std=c++17', '-O1', '-Wall', '-o', EXE, src, runtime.LIB_PATH,
                           '-Wl,-rpath,' + os.path.join(ROOT, 'n2d2_b200')], env=env)


def _parsed():
    _build()
    out = subprocess.run([EXE, '--parse', FIXTURE], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    d = {}
    for ln in out.stdout.splitlines():
        k, _, v = ln.partition(' ')
        d[k] = v.split()
    return d


def test_fixture_is_what_the_generator_writes():
    # the committed files are the generator's output for the seeded network (nobody edited one side only)
    mod, net = _fixture_net()
    _, shapes = netdesc.layer_macs(net)
    l = net['layers'][0]
    text = mod.conv_header(l, shapes[-1], shapes[0], l['quant']['out_unsigned'])
    assert text == open(os.path.join(FIXTURE, 'conv1.hpp')).read()
    # a few statements spelled as the reference's writers spell them (src/Export/CPP/CPP_CellExport.cpp:110-241,
    # src/Export/CellExport.cpp:100-117)
    assert 'static const N2D2_Export::SingleShiftScalingPerChannel<8> CONV1_SCALING = {' in text
    assert f"{int(l['bias'][0])} + {1 << (int(l['quant']['shift0'][0]) - 1)}, " in text
    w4 = open(os.path.join(FIXTURE, 'conv3_w4.hpp')).read()
    assert 'static const data<4> conv3_w4_weights[' in w4 and 'FixedPointClippingAndScalingPerChannel<16, ' in w4
    assert 'std::array<SUM_T, 3>{' in open(os.path.join(FIXTURE, 'conv2.hpp')).read()


def test_headers_and_syntxt_parse_to_the_network_they_were_written_from():
    _, net = _fixture_net()
    d = _parsed()
    ints = lambda k: np.array([int(v) for v in d[k]], np.int64)
    layers = {l['name']: l for l in net['layers']}
    for name in ('conv1', 'conv2', 'conv3_w4', 'fc1'):
        l = layers[name]
        assert np.array_equal(ints(f'{name}.weights'), np.asarray(l['weights']).reshape(-1).astype(np.int64)), name
        assert np.array_equal(ints(f'{name}.biases'), np.asarray(l['bias']).astype(np.int64)), name
    # the single-shift half is in the exported biases and out of the cell's own
    q1 = layers['conv1']['quant']
    half = (1 << (q1['shift0'].astype(np.int64) - 1))
    assert np.array_equal(ints('conv1.exportedBiases'), layers['conv1']['bias'].astype(np.int64) + half)
    assert d['conv1.activation'] == ['Rectifier'] and d['conv3_w4.activation'] == ['Linear']
    assert d['conv3_w4.weightBits'] == ['4'] and d['conv1.weightBits'] == ['8']
    # scalings: mode numbers follow include/ScalingMode.hpp (NONE 0 ... DOUBLE_SHIFT 5)
    assert d['conv1.mode'] == ['4'] and np.array_equal(ints('conv1.shift0'), q1['shift0'])
    q2 = layers['conv2']['quant']
    assert d['conv2.mode'] == ['5'] and np.array_equal(ints('conv2.shift0'), q2['shift0']) and np.array_equal(ints('conv2.shift1'), q2['shift1'])
    assert d['conv2.outputUnsigned'] == ['1']
    q3 = layers['conv3_w4']['quant']
    assert d['conv3_w4.mode'] == ['3'] and d['conv3_w4.isClipped'] == ['1'] and int(d['conv3_w4.fracBits'][0]) == q3['frac_bits']
    assert np.array_equal(ints('conv3_w4.mult'), q3['mult']) and np.array_equal(ints('conv3_w4.clip'), q3['clip'].astype(np.int64))
    qs = layers['sum1']['quant']
    assert d['sum1.mode'] == ['4'] and np.array_equal(ints('sum1.shift0'), qs['shift0']) and d['sum1.name.ELEM_OP'] == ['Sum']
    qf = layers['fc1']['quant']
    assert d['fc1.mode'] == ['3'] and np.array_equal(ints('fc1.mult'), qf['mult']) and int(d['fc1.fracBits'][0]) == qf['frac_bits']
    assert d['pool1.name.POOLING'] == ['Max'] and d['pool1.const.POOL_WIDTH'] == ['2'] and d['pool1.mode'] == ['0']
    # .syntxt: [output][channel][ky][kx]
    w = np.asarray(layers['conv1']['weights']).astype(np.int64)          # [O][kH][kW][C]
    assert np.array_equal(ints('syntxt.conv1.weights'), w.transpose(0, 3, 1, 2).reshape(-1))
    assert np.array_equal(ints('syntxt.conv1.biases'), layers['conv1']['bias'])
    assert d['malformed.threw'] == ['1']
    # sub-4-bit storage of the QAT export (src/Export/CPP/CPP_ConvCellExport.cpp:419-607)
    assert d['w2.weights'] == ['1', '-1', '0', '-2', '1'] and d['w1.weights'] == ['1', '-1', '-1', '1', '1', '-1', '1', '1', '1']


@pytest.mark.gpu
def test_network_rebuilt_from_the_headers_matches_the_oracle(tmp_path):
    from oracle import oracle
    _, net = _fixture_net()
    _build()
    batch = 5
    x = netdesc.make_input(net, batch, seed=8)
    ref = oracle.run_net(net, x, 'i64')[-1].reshape(batch, -1)
    stim, out = str(tmp_path / 'stimuli.bin'), str(tmp_path / 'logits.bin')
    x.tofile(stim)
    r = subprocess.run([EXE, '--run', FIXTURE, stim, str(batch), out], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    got = np.fromfile(out, np.int32).reshape(batch, -1)
    assert np.array_equal(got.astype(np.int64), ref)
