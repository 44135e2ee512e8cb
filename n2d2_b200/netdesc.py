"""Quantized-network descriptions: the cells DeepNetQuantization::quantizeNetwork leaves behind
(N2D2 src/DeepNetQuantization.cpp:285-388), as plain data, and seeded generators for the benchmark
topologies.

A network is a dict {'name', 'input': {C,H,W,unsigned}, 'layers': [...]}.  A layer is a dict with
'type' in {'conv','fc','pool','sum','scaling'}, 'inputs' (indices of producing layers, -1 = the
network input) and, depending on the type:

  conv     Cout, kH, kW, stride=(y,x), pad=(top,left,bottom,right), dil=(y,x), groups, weight_bits,
           weights int8 [Cout][kH][kW][Cin/groups], bias int32 [Cout] or None, quant
  fc       Cout, weight_bits, weights int8 [Cout][K] (K in NHWC order of the input), bias, quant
  pool     pool ('max'|'avg'), kH, kW, stride=(y,x), pad=(y,x)
  sum      quant                        (ElemWise Sum, unit weights)
  scaling  quant                        (ScalingCell)

quant = {'mode': 'none'|'float'|'fixed16'|'fixed32'|'single'|'double', 'act': 'linear'|'relu'|
'saturation', 'out_bits', 'out_unsigned', and the per-channel arrays of the mode: fscale | mult +
frac_bits (+ frac_bits_per_ch) | shift0 | shift0 + shift1, optional is_clipped + clip, sat_thr}.

Topologies restate models/mnist24_16c4s2_24c5s2_150_10.ini, models/ResNet-18.ini +
ResNet-block.ini.tpl, models/ResNet-50.ini + ResNet-bottleneck_block.ini.tpl and
models/MobileNet_v1.ini of the reference; weights, biases and scalings are seeded synthetic values.
"""
from __future__ import annotations

import math

import numpy as np

MODES = {'none': 0, 'float': 1, 'fixed16': 2, 'fixed32': 3, 'single': 4, 'double': 5}
ACTS = {'linear': 0, 'relu': 1, 'saturation': 2}


def conv_out_dim(n, k, stride, pad0, pad1, dil=1):
    # ConvCell_Frame_Kernels.cpp:37-45
    return int((n + pad0 + pad1 - dil * (k - 1) - 1 + stride) / float(stride))


def pool_out_dim(n, k, stride, pad):
    # PoolCell.cpp:233-239
    return int((n + 2 * pad - k + stride) / float(stride))


def pack_int4(w):
    """Pack int4 values (last axis flattened per output channel) two per byte, even element in the
    high nibble (export/CPP_Quantization/include/typedefs.hpp:359-375 of the reference)."""
    rows = w.reshape(w.shape[0], -1).astype(np.int16)
    if rows.shape[1] % 2:
        rows = np.concatenate([rows, np.zeros((rows.shape[0], 1), np.int16)], axis=1)
    hi = (rows[:, 0::2] & 0xF).astype(np.uint8)
    lo = (rows[:, 1::2] & 0xF).astype(np.uint8)
    return ((hi << 4) | lo).astype(np.uint8)


def pack_bits(w, bits):
    """Sub-byte weights [rows][...] as the export's data<N> stores them: 8 / bits values per byte, the first in the
    highest bits, every row starting on a byte; 1-bit weights store -1 as 0
    (export/CPP_Quantization/include/typedefs.hpp:359-517 of the reference)."""
    rows = np.asarray(w, np.int64).reshape(w.shape[0], -1)
    per = 8 // bits
    if bits == 1:
        if not np.isin(rows, (-1, 1)).all():
            raise ValueError('1-bit weights are -1 or +1')
        v = (rows > 0).astype(np.int64)
    else:
        v = rows & ((1 << bits) - 1)
    pad = (-rows.shape[1]) % per
    if pad:
        v = np.concatenate([v, np.zeros((rows.shape[0], pad), np.int64)], axis=1)
    v = v.reshape(rows.shape[0], -1, per)
    out = np.zeros(v.shape[:2], np.int64)
    for j in range(per):
        out |= v[:, :, j] << (8 - bits * (j + 1))
    return np.ascontiguousarray(out.astype(np.uint8))


class NetBuilder:
    """Builds a network description and draws seeded parameters.

    scaling: 'single' | 'double' | 'fixed' | 'float'.  `calibrate` picks each cell's scale from the
    expected accumulator spread so that activations neither vanish nor saturate everywhere (the
    per-channel draws stay inside the ranges the benchmark configurations name); with
    calibrate=False the raw ranges are used as given.
    """

    def __init__(self, name, C, H, W, seed, scaling, unsigned_relu=True, input_unsigned=True,
                 weight_dist=('uniform', 127), weight_bits=8, calibrate=True, shift_range=(6, 12),
                 clipped=False, per_channel_frac=False):
        self.net = {'name': name, 'input': {'C': C, 'H': H, 'W': W, 'unsigned': bool(input_unsigned)},
                    'layers': []}
        self.rng = np.random.Generator(np.random.PCG64(seed))
        self.scaling_mode = scaling
        self.unsigned_relu = unsigned_relu
        self.weight_dist = weight_dist
        self.weight_bits = weight_bits
        self.calibrate = calibrate
        self.shift_range = shift_range
        self.clipped = clipped
        self.per_channel_frac = per_channel_frac
        # per tensor: (C, H, W, rms estimate)
        in_rms = 147.0 if input_unsigned else 74.0
        self.shapes = {-1: (C, H, W, in_rms)}

    # ---- parameter draws -------------------------------------------------------------------
    def _weights(self, shape):
        kind, p = self.weight_dist
        if self.weight_bits == 4:
            return self.rng.integers(-7, 8, size=shape, dtype=np.int64).astype(np.int8)
        if self.weight_bits == 2:
            return self.rng.integers(-2, 2, size=shape, dtype=np.int64).astype(np.int8)
        if self.weight_bits == 1:
            return (2 * self.rng.integers(0, 2, size=shape, dtype=np.int64) - 1).astype(np.int8)
        if kind == 'uniform':
            return self.rng.integers(-p, p + 1, size=shape, dtype=np.int64).astype(np.int8)
        w = np.rint(self.rng.normal(0.0, p, size=shape))
        return np.clip(w, -127, 127).astype(np.int8)

    def _weight_sigma(self):
        kind, p = self.weight_dist
        if self.weight_bits == 4:
            return 4.3
        if self.weight_bits in (1, 2):
            return 1.1
        return p / math.sqrt(3.0) if kind == 'uniform' else float(p)

    def _quant(self, channels, act, acc_sigma, target_rms=45.0, mode=None):
        mode = mode or self.scaling_mode
        out_unsigned = bool(self.unsigned_relu and act == 'relu')
        q = {'mode': None, 'act': act, 'out_bits': 8, 'out_unsigned': out_unsigned}
        want = target_rms / max(acc_sigma, 1.0)   # desired multiplicative scale
        rng = self.rng
        if mode == 'single':
            q['mode'] = 'single'
            if self.calibrate:
                s0 = int(round(-math.log2(want)))
                sh = np.clip(s0 + rng.integers(-1, 2, size=channels), 0, 30)
            else:
                sh = rng.integers(self.shift_range[0], self.shift_range[1] + 1, size=channels)
            q['shift0'] = sh.astype(np.uint8)
        elif mode == 'double':
            q['mode'] = 'double'
            a = rng.integers(1, 5, size=channels)
            if self.calibrate:
                b = np.rint(np.log2((1.0 + 2.0 ** a) / want) + rng.uniform(-0.5, 0.5, size=channels))
                b = np.clip(b, 1, 30)
            else:
                b = rng.integers(8, 15, size=channels)
            q['shift0'] = a.astype(np.uint8)
            q['shift1'] = b.astype(np.uint8)
        elif mode == 'fixed':
            q['mode'] = 'fixed32'
            mult = rng.integers(1 << 14, 1 << 15, size=channels)
            if self.calibrate:
                f = int(np.clip(round(math.log2(24576.0 / want)), 1, 40))
            else:
                f = int(rng.integers(16, 25))
            q['mult'] = mult.astype(np.int32)
            q['frac_bits'] = f
            if self.per_channel_frac:
                q['frac_bits_per_ch'] = np.clip(f + rng.integers(-1, 2, size=channels), 1, 40).astype(np.uint8)
        elif mode == 'float':
            q['mode'] = 'float'
            q['fscale'] = (want * rng.uniform(0.7, 1.4, size=channels)).astype(np.float32)
        else:
            raise ValueError(mode)
        if self.clipped and q['mode'] in ('float', 'fixed32', 'fixed16'):
            # clip = a real-valued accumulator bound, as the QAT fusion produces
            q['is_clipped'] = True
            q['clip'] = (acc_sigma * rng.uniform(1.5, 3.0, size=channels)).astype(np.float32)
        return q

    def _out_rms(self, act):
        return 45.0 * (0.6 if act == 'relu' else 1.0)

    # ---- cells -----------------------------------------------------------------------------
    def conv(self, inp, Cout, k, stride=1, pad=0, act='relu', groups=1, dil=1, bias=True, name=None):
        C, H, W, rms = self.shapes[inp]
        kH = kW = k
        Cg = C // groups
        w = self._weights((Cout, kH, kW, Cg))
        b = self.rng.integers(-4096, 4097, size=Cout).astype(np.int32) if bias else None
        acc_sigma = math.sqrt(kH * kW * Cg) * self._weight_sigma() * rms
        layer = {'type': 'conv', 'name': name or f'conv{len(self.net["layers"])}', 'inputs': [inp],
                 'Cout': Cout, 'kH': kH, 'kW': kW, 'stride': (stride, stride), 'pad': (pad, pad, pad, pad),
                 'dil': (dil, dil), 'groups': groups, 'weight_bits': self.weight_bits,
                 'weights': w, 'bias': b, 'quant': self._quant(Cout, act, acc_sigma)}
        oH = conv_out_dim(H, kH, stride, pad, pad, dil)
        oW = conv_out_dim(W, kW, stride, pad, pad, dil)
        return self._push(layer, (Cout, oH, oW, self._out_rms(act)))

    def fc(self, inp, Cout, act='linear', bias=True, name=None):
        C, H, W, rms = self.shapes[inp]
        K = C * H * W
        w = self._weights((Cout, K))
        b = self.rng.integers(-4096, 4097, size=Cout).astype(np.int32) if bias else None
        acc_sigma = math.sqrt(K) * self._weight_sigma() * rms
        layer = {'type': 'fc', 'name': name or f'fc{len(self.net["layers"])}', 'inputs': [inp], 'Cout': Cout,
                 'weight_bits': self.weight_bits, 'weights': w, 'bias': b,
                 'quant': self._quant(Cout, act, acc_sigma)}
        return self._push(layer, (Cout, 1, 1, self._out_rms(act)))

    def pool(self, inp, kind, k, stride, pad=0, name=None):
        C, H, W, rms = self.shapes[inp]
        kH, kW = (k, k) if isinstance(k, int) else k
        layer = {'type': 'pool', 'name': name or f'pool{len(self.net["layers"])}', 'inputs': [inp], 'pool': kind,
                 'kH': kH, 'kW': kW, 'stride': (stride, stride), 'pad': (pad, pad)}
        return self._push(layer, (C, pool_out_dim(H, kH, stride, pad), pool_out_dim(W, kW, stride, pad), rms))

    def sum(self, inputs, act='relu', name=None, mode=None):
        C, H, W, _ = self.shapes[inputs[0]]
        rms = math.sqrt(sum(self.shapes[i][3] ** 2 for i in inputs))
        layer = {'type': 'sum', 'name': name or f'sum{len(self.net["layers"])}', 'inputs': list(inputs),
                 'quant': self._quant(C, act, rms, target_rms=min(rms, 60.0), mode=mode)}
        return self._push(layer, (C, H, W, self._out_rms(act)))

    def scaling(self, inp, act='linear', name=None, mode=None):
        C, H, W, rms = self.shapes[inp]
        layer = {'type': 'scaling', 'name': name or f'scaling{len(self.net["layers"])}', 'inputs': [inp],
                 'quant': self._quant(C, act, rms, target_rms=rms * 0.8, mode=mode)}
        return self._push(layer, (C, H, W, self._out_rms(act)))

    def _push(self, layer, shape):
        idx = len(self.net['layers'])
        self.net['layers'].append(layer)
        self.shapes[idx] = shape
        return idx


# ------------------------------------------------------------------------------------ topologies
def mnist24(seed=1, scaling='single', calibrate=False):
    """models/mnist24_16c4s2_24c5s2_150_10.ini made dense with biases: 8-bit, SingleShift,
    shifts U{6..12}, weights U{-127..127}, biases U{-4096..4096}."""
    b = NetBuilder('mnist24', 1, 24, 24, seed, scaling, calibrate=calibrate, shift_range=(6, 12))
    x = b.conv(-1, 16, 4, stride=2, name='conv1')
    x = b.conv(x, 24, 5, stride=2, name='conv2')
    x = b.fc(x, 150, act='relu', name='fc1')
    b.fc(x, 10, act='linear', name='fc2')
    return b.net


def resnet18(seed=2, size=224, scaling='fixed', weight_bits=8, unsigned_relu=True, pool_pad=0, width=64,
             classes=1000, clipped=False, per_channel_frac=False):
    """models/ResNet-18.ini: 7x7/2 stem, 3x3/2 max pool (no padding in the reference ini), basic blocks
    2-2-2-2 with a 1x1 projection on the first block of every stage, global average pool, fc."""
    dist = ('normal', 40) if weight_bits == 8 else ('uniform', 7)
    b = NetBuilder(f'resnet18_w{weight_bits}', 3, size, size, seed, scaling, unsigned_relu=unsigned_relu,
                   weight_dist=dist, weight_bits=weight_bits, clipped=clipped, per_channel_frac=per_channel_frac)
    x = b.conv(-1, width, 7, stride=2, pad=3, name='conv1')
    x = b.pool(x, 'max', 3, 2, pad=pool_pad, name='pool1')
    for stage, (f, blocks) in enumerate(zip([width, 2 * width, 4 * width, 8 * width], [2, 2, 2, 2])):
        for blk in range(blocks):
            stride = 2 if (stage > 0 and blk == 0) else 1
            nm = f'conv{stage + 2}.{blk + 1}'
            y = b.conv(x, f, 3, stride=stride, pad=1, name=nm + '_3x3_1')
            y = b.conv(y, f, 3, stride=1, pad=1, act='linear', name=nm + '_3x3_2')
            sc = x
            if blk == 0:
                sc = b.conv(x, f, 1, stride=stride, pad=0, act='linear', name=nm + '_1x1_proj')
            x = b.sum([y, sc], act='relu', name=nm + '_sum')
    C, H, W, _ = b.shapes[x]
    x = b.pool(x, 'avg', (H, W), 1, name='pool')
    b.fc(x, classes, act='linear', name='fc')
    return b.net


def resnet50(seed=4, size=224, scaling='double', unsigned_relu=True, pool_pad=0, width=64, classes=1000,
             blocks=(3, 4, 6, 3)):
    """models/ResNet-50.ini: bottleneck blocks 3-4-6-3 (1x1 -> 3x3 carrying the stride -> 1x1 x4,
    1x1 projection on the first block of every stage), global average pool, fc."""
    b = NetBuilder('resnet50', 3, size, size, seed, scaling, unsigned_relu=unsigned_relu,
                   weight_dist=('normal', 30))
    x = b.conv(-1, width, 7, stride=2, pad=3, name='conv1')
    x = b.pool(x, 'max', 3, 2, pad=pool_pad, name='pool1')
    for stage, (f, nb) in enumerate(zip([width, 2 * width, 4 * width, 8 * width], blocks)):
        for blk in range(nb):
            stride = 2 if (stage > 0 and blk == 0) else 1
            nm = f'conv{stage + 2}.{blk + 1}'
            y = b.conv(x, f, 1, name=nm + '_1x1')
            y = b.conv(y, f, 3, stride=stride, pad=1, name=nm + '_3x3')
            y = b.conv(y, 4 * f, 1, act='linear', name=nm + '_1x1_x4')
            sc = x
            if blk == 0:
                sc = b.conv(x, 4 * f, 1, stride=stride, act='linear', name=nm + '_1x1_proj')
            x = b.sum([y, sc], act='relu', name=nm + '_sum')
    C, H, W, _ = b.shapes[x]
    x = b.pool(x, 'avg', (H, W), 1, name='pool')
    b.fc(x, classes, act='linear', name='fc')
    return b.net


def mobilenet_v1(seed=3, size=224, scaling='single', alpha=1.0, classes=1000):
    """models/MobileNet_v1.ini at alpha = 1.0 / 224 px: 3x3/2 stem, 13 depthwise-separable blocks
    (3x3 depthwise + 1x1 pointwise), global average pool, fc."""
    b = NetBuilder('mobilenet_v1', 3, size, size, seed, scaling, weight_dist=('uniform', 127))
    c = lambda n: int(n * alpha)
    x = b.conv(-1, c(32), 3, stride=2, pad=1, name='conv1')
    cfg = [(64, 1), (128, 2), (128, 1), (256, 2), (256, 1), (512, 2)] + [(512, 1)] * 5 + [(1024, 2), (1024, 1)]
    for i, (f, s) in enumerate(cfg):
        C = b.shapes[x][0]
        x = b.conv(x, C, 3, stride=s, pad=1, groups=C, name=f'conv{i + 2}_3x3_dw')
        x = b.conv(x, c(f), 1, name=f'conv{i + 2}_1x1')
    C, H, W, _ = b.shapes[x]
    x = b.pool(x, 'avg', (H, W), 1, name='pool')
    b.fc(x, classes, act='linear', name='fc')
    return b.net


def make_input(net, batch, seed=1234):
    """Seeded uniform 8-bit stimuli, NHWC."""
    i = net['input']
    rng = np.random.Generator(np.random.PCG64(seed))
    if i['unsigned']:
        return rng.integers(0, 256, size=(batch, i['H'], i['W'], i['C']), dtype=np.int64).astype(np.uint8)
    return rng.integers(-128, 128, size=(batch, i['H'], i['W'], i['C']), dtype=np.int64).astype(np.int8)


def layer_macs(net):
    """Multiply-accumulates per image of every layer (padding taps counted, as in a dense GEMM)."""
    shapes = {-1: (net['input']['C'], net['input']['H'], net['input']['W'])}
    macs = []
    for idx, l in enumerate(net['layers']):
        C, H, W = shapes[l['inputs'][0]]
        if l['type'] == 'conv':
            oH = conv_out_dim(H, l['kH'], l['stride'][0], l['pad'][0], l['pad'][2], l['dil'][0])
            oW = conv_out_dim(W, l['kW'], l['stride'][1], l['pad'][1], l['pad'][3], l['dil'][1])
            macs.append(oH * oW * l['Cout'] * (C // l['groups']) * l['kH'] * l['kW'])
            shapes[idx] = (l['Cout'], oH, oW)
        elif l['type'] == 'fc':
            macs.append(C * H * W * l['Cout'])
            shapes[idx] = (l['Cout'], 1, 1)
        elif l['type'] == 'pool':
            shapes[idx] = (C, pool_out_dim(H, l['kH'], l['stride'][0], l['pad'][0]),
                           pool_out_dim(W, l['kW'], l['stride'][1], l['pad'][1]))
            macs.append(0)
        else:
            shapes[idx] = (C, H, W)
            macs.append(0)
    return macs, shapes
