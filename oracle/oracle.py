"""ctypes binding of the CPU oracle (oracle/n2d2_oracle.c) and a layer-by-layer runner for the
network descriptions of n2d2_b200/netdesc.py.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the benchmark's CPU-baseline
leg.  The product never imports it.

Two flavours: 'f32' accumulates in fp32 in the reference's loop order on NCHW float tensors (what
the reference's CPU cells do), 'i64' is the exact-integer arbiter.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

MODES = {'none': 0, 'float': 1, 'fixed16': 2, 'fixed32': 3, 'single': 4, 'double': 5}
ACTS = {'linear': 0, 'relu': 1, 'saturation': 2}


def build(force=False):
    so = os.path.join(_HERE, 'libn2d2_oracle.so')
    srcs = [os.path.join(_HERE, f) for f in ('n2d2_oracle.c', 'n2d2_oracle_impl.inc', 'n2d2_oracle.h')]
    if force or not os.path.exists(so) or any(os.path.getmtime(s) > os.path.getmtime(so) for s in srcs):
        subprocess.check_call(['make', '-C', _HERE, 'libn2d2_oracle.so'], stdout=subprocess.DEVNULL)
    return so


def lib():
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(build())
        _LIB.n2d2o_conv_out_dim.restype = C.c_int
        _LIB.n2d2o_pool_out_dim.restype = C.c_int
        _LIB.n2d2o_num_threads.restype = C.c_int
        _LIB.n2d2o_scaling_f32.restype = C.c_int
        _LIB.n2d2o_scaling_i64.restype = C.c_int
    return _LIB


def num_threads():
    return lib().n2d2o_num_threads()


def use_all_cores():
    """Makes the OpenMP runtime (shared with the reference shim) use every core this process may run on,
    whatever OMP_NUM_THREADS the launcher exported. Returns the thread count."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    lib().n2d2o_set_num_threads(n)
    return num_threads()


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _np_t(flavour):
    return np.float32 if flavour == 'f32' else np.int64


def _fn(name, flavour):
    return getattr(lib(), f'{name}_{flavour}')


def group_map(O, Cin, groups):
    """Boolean connection map of a grouped convolution, [O][Cin] (Cell mapping of the reference)."""
    if groups == 1:
        return None
    m = np.zeros((O, Cin), np.uint8)
    cg, og = Cin // groups, O // groups
    for g in range(groups):
        m[g * og:(g + 1) * og, g * cg:(g + 1) * cg] = 1
    return m


def conv(x, w_oihw, flavour, stride=(1, 1), pad=(0, 0, 0, 0), dil=(1, 1), groups=1, maps=None, bias=None,
         accumulate_into=None, ref_quirks=False):
    """x: [B][C][H][W]; w_oihw: [O][Cg][kH][kW]; pad = (top, left, bottom, right). Returns [B][O][oH][oW]."""
    t = _np_t(flavour)
    x = np.ascontiguousarray(x, t)
    w = np.ascontiguousarray(w_oihw, t)
    B, Cin, H, W = x.shape
    O, wC, kH, kW = w.shape
    oH = lib().n2d2o_conv_out_dim(H, kH, stride[0], pad[0], pad[2], dil[0])
    oW = lib().n2d2o_conv_out_dim(W, kW, stride[1], pad[1], pad[3], dil[1])
    if maps is None:
        maps = group_map(O, Cin, groups)
    nb_groups = groups
    out = accumulate_into if accumulate_into is not None else np.zeros((B, O, oH, oW), t)
    _fn('n2d2o_conv', flavour)(
        _p(x), W, H, Cin, B, _p(w), kW, kH, wC, O, _p(maps), nb_groups, stride[1], stride[0],
        pad[1], pad[0], pad[3], pad[2], dil[1], dil[0], 1 if accumulate_into is not None else 0,
        1 if ref_quirks else 0, _p(out))
    if bias is not None:
        bb = np.ascontiguousarray(bias, t)
        _fn('n2d2o_add_bias', flavour)(_p(out), oW, oH, O, B, _p(bb))
    return out


def fc(x, w, flavour, bias=None):
    """x: [B][K] (flattened NCHW like the reference); w: [O][K]."""
    t = _np_t(flavour)
    x = np.ascontiguousarray(x, t)
    w = np.ascontiguousarray(w, t)
    B, K = x.shape
    O = w.shape[0]
    bb = None if bias is None else np.ascontiguousarray(bias, t)
    out = np.zeros((B, O), t)
    _fn('n2d2o_fc', flavour)(_p(x), K, B, _p(w), _p(bb), O, _p(out))
    return out


def pool(x, kind, k, stride, pad, flavour, quantized=True):
    t = _np_t(flavour)
    x = np.ascontiguousarray(x, t)
    B, Cn, H, W = x.shape
    oH = lib().n2d2o_pool_out_dim(H, k[0], stride[0], pad[0])
    oW = lib().n2d2o_pool_out_dim(W, k[1], stride[1], pad[1])
    out = np.zeros((B, Cn, oH, oW), t)
    if kind == 'max':
        _fn('n2d2o_pool_max', flavour)(_p(x), W, H, Cn, B, k[1], k[0], stride[1], stride[0], pad[1], pad[0], _p(out))
    else:
        _fn('n2d2o_pool_avg', flavour)(_p(x), W, H, Cn, B, k[1], k[0], stride[1], stride[0], pad[1], pad[0],
                                       1 if quantized else 0, _p(out))
    return out


def elemwise_sum(xs, flavour):
    t = _np_t(flavour)
    xs = [np.ascontiguousarray(x, t) for x in xs]
    n = len(xs)
    ptrs = (C.c_void_p * n)(*[x.ctypes.data for x in xs])
    wts = np.ones(n, t)
    sh = np.zeros(n, t)
    out = np.zeros_like(xs[0])
    _fn('n2d2o_elemwise_sum', flavour)(ptrs, n, _p(wts), _p(sh), C.c_size_t(xs[0].size), _p(out))
    return out


def scaling(x, q, flavour):
    """x: [B][C][H][W] (or [B][C]); q: quant dict. Applies Scaling::propagate then the activation."""
    t = _np_t(flavour)
    x = np.ascontiguousarray(x, t)
    B, Cn = x.shape[0], x.shape[1]
    HW = int(np.prod(x.shape[2:])) if x.ndim > 2 else 1
    mode = MODES[q['mode']]
    f32 = lambda k: None if q.get(k) is None else np.ascontiguousarray(q[k], np.float32)
    i32 = lambda k: None if q.get(k) is None else np.ascontiguousarray(q[k], np.int32)
    u8 = lambda k: None if q.get(k) is None else np.ascontiguousarray(q[k], np.uint8)
    fscale, mult, s0, s1, clip, fpc = f32('fscale'), i32('mult'), u8('shift0'), u8('shift1'), f32('clip'), u8('frac_bits_per_ch')
    out = np.zeros_like(x)
    nbits = int(q.get('out_bits', 8)) if mode != 0 else 0
    rc = _fn('n2d2o_scaling', flavour)(
        _p(x), _p(out), B, Cn, HW, mode, _p(fscale), _p(mult), int(q.get('frac_bits', 0)), _p(fpc), _p(s0), _p(s1),
        1 if q.get('is_clipped') else 0, _p(clip), nbits, 1 if q.get('out_unsigned') else 0)
    if rc != 0:
        raise RuntimeError('scaling on a non-quantized cell (the reference throws here)')
    _fn('n2d2o_activation', flavour)(_p(out), C.c_size_t(out.size), ACTS[q.get('act', 'linear')],
                                     C.c_float(0.0), C.c_float(float(q.get('sat_thr', 0))))
    return out


def unpack_weights(layer):
    """int8 view of a layer's weights (int4 values are stored widened in the description)."""
    return np.asarray(layer['weights'], np.int8)


def estimated_labels_topn(scores, top_n):
    """Target top-N of the reference (src/Target/Target_CUDA_kernels.cu:44-104) on integer scores [pixels][classes]:
    returns (labels, values), each [pixels][top_n]."""
    sc = np.ascontiguousarray(scores, np.int64)
    pixels, nb_class = sc.shape
    labels = np.zeros((pixels, top_n), np.int32)
    values = np.zeros((pixels, top_n), np.int64)
    lib().n2d2o_estimated_labels_topn(sc.ctypes.data_as(C.c_void_p), C.c_size_t(pixels), nb_class, top_n,
                                      labels.ctypes.data_as(C.c_void_p), values.ctypes.data_as(C.c_void_p))
    return labels, values


def run_net(net, x_nhwc, flavour='f32'):
    """Runs the network on x_nhwc ([B][H][W][C], 8-bit) cell by cell. Returns the list of per-layer
    outputs as NHWC int64 arrays (exactly-integer values in both flavours)."""
    t = _np_t(flavour)
    x = np.ascontiguousarray(np.transpose(np.asarray(x_nhwc), (0, 3, 1, 2))).astype(t)
    outs = {-1: x}
    res = []
    for idx, l in enumerate(net['layers']):
        a = outs[l['inputs'][0]]
        if l['type'] == 'conv':
            w = unpack_weights(l)                      # [O][kH][kW][Cg]
            w_oihw = np.transpose(w, (0, 3, 1, 2))
            y = conv(a, w_oihw, flavour, l['stride'], l['pad'], l['dil'], l['groups'], maps=l.get('maps'), bias=l['bias'])
            y = scaling(y, l['quant'], flavour)
        elif l['type'] == 'fc':
            w = unpack_weights(l)                      # [O][K], K in NHWC order of the input
            B, Cn, H, W = a.shape
            w_nchw = w.reshape(-1, H, W, Cn).transpose(0, 3, 1, 2).reshape(w.shape[0], -1)
            y = fc(a.reshape(B, -1), w_nchw, flavour, bias=l['bias'])
            y = scaling(y, l['quant'], flavour).reshape(B, -1, 1, 1)
        elif l['type'] == 'pool':
            y = pool(a, l['pool'], (l['kH'], l['kW']), l['stride'], l['pad'], flavour)
        elif l['type'] == 'sum':
            y = elemwise_sum([outs[i] for i in l['inputs']], flavour)
            y = scaling(y, l['quant'], flavour)
        elif l['type'] == 'scaling':
            y = scaling(a, l['quant'], flavour)
        else:
            raise ValueError(l['type'])
        outs[idx] = y
        res.append(np.transpose(np.rint(y).astype(np.int64), (0, 2, 3, 1)))
    return res
