"""ctypes binding of oracle/_ref/libn2d2_refshim.so: the reference's own CPU kernels
(ConvCell_Frame_Kernels, PoolCell_Frame_Kernels, Scaling_Kernels) compiled from the reference tree by
oracle/refshim/Makefile.  TEST INFRASTRUCTURE ONLY.  Tensors are NCHW float32 like the reference's."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
SO = os.path.join(_HERE, '_ref', 'libn2d2_refshim.so')
_LIB = None


def available():
    return os.path.exists(SO)


def lib():
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(SO)
    return _LIB


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def conv(x, w_oihw, stride=(1, 1), pad=(0, 0, 0, 0), dil=(1, 1), maps=None, bias=None):
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w_oihw, np.float32)
    B, Cn, H, W = x.shape
    O, wC, kH, kW = w.shape
    oH = int((H + pad[0] + pad[2] - dil[0] * (kH - 1) - 1 + stride[0]) / float(stride[0]))
    oW = int((W + pad[1] + pad[3] - dil[1] * (kW - 1) - 1 + stride[1]) / float(stride[1]))
    out = np.zeros((B, O, oH, oW), np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, np.float32)
    m = None if maps is None else np.ascontiguousarray(maps, np.uint8)
    lib().refshim_conv(_p(x), W, H, Cn, B, _p(w), kW, kH, wC, O, _p(m), stride[1], stride[0], pad[1], pad[0], pad[3],
                       pad[2], dil[1], dil[0], _p(b), oW, oH, _p(out))
    return out


def pool(x, kind, k, stride, pad, quantized=True):
    x = np.ascontiguousarray(x, np.float32)
    B, Cn, H, W = x.shape
    oH = int((H + 2 * pad[0] - k[0] + stride[0]) / float(stride[0]))
    oW = int((W + 2 * pad[1] - k[1] + stride[1]) / float(stride[1]))
    out = np.zeros((B, Cn, oH, oW), np.float32)
    lib().refshim_pool(_p(x), W, H, Cn, B, k[1], k[0], stride[1], stride[0], pad[1], pad[0],
                       1 if kind == 'max' else 0, 1 if quantized else 0, oW, oH, _p(out))
    return out


def scaling(x, q):
    """Scaling only (no activation): q is a quant dict of n2d2_b200/netdesc.py."""
    x = np.ascontiguousarray(x, np.float32)
    B, Cn = x.shape[0], x.shape[1]
    H = x.shape[2] if x.ndim > 2 else 1
    W = x.shape[3] if x.ndim > 3 else 1
    mode = {'float': 1, 'fixed16': 2, 'fixed32': 2, 'single': 4, 'double': 5}[q['mode']]
    g = lambda k, t: None if q.get(k) is None else np.ascontiguousarray(q[k], t)
    fs, mu, s0, s1, cl = g('fscale', np.float32), g('mult', np.int32), g('shift0', np.uint8), g('shift1', np.uint8), g('clip', np.float32)
    out = np.zeros_like(x)
    lib().refshim_scaling(_p(x), _p(out), B, Cn, H, W, mode, _p(fs), _p(mu), int(q.get('frac_bits', 0)), _p(s0), _p(s1),
                          1 if q.get('is_clipped') else 0, _p(cl), int(q.get('out_bits', 8)),
                          1 if q.get('out_unsigned') else 0)
    return out


def run_net(net, x_nhwc):
    """The reference's CPU quantized path on a whole network: convolution, pooling and the Scaling
    kernels are the reference's own compiled code (this shim); fully-connected, element-wise sum and
    the ReLU after the scaling come from the oracle port (their reference sources need the whole
    library to build).  Returns the per-layer outputs as NHWC int64 arrays."""
    from . import oracle
    x = np.ascontiguousarray(np.transpose(np.asarray(x_nhwc), (0, 3, 1, 2))).astype(np.float32)
    outs = {-1: x}
    res = []

    def quantize(y, q):
        if q['mode'] != 'none':
            y = scaling(y, q)
        oracle._fn('n2d2o_activation', 'f32')(_p(y), C.c_size_t(y.size), oracle.ACTS[q.get('act', 'linear')],
                                              C.c_float(0.0), C.c_float(float(q.get('sat_thr', 0))))
        return y

    for idx, l in enumerate(net['layers']):
        a = outs[l['inputs'][0]]
        if l['type'] == 'conv':
            w = np.transpose(np.asarray(l['weights'], np.int8), (0, 3, 1, 2))
            maps = oracle.group_map(l['Cout'], a.shape[1], l['groups'])
            y = quantize(conv(a, w, l['stride'], l['pad'], l['dil'], maps, l['bias']), l['quant'])
        elif l['type'] == 'fc':
            w = np.asarray(l['weights'], np.int8)
            B, Cn, H, W = a.shape
            w_nchw = w.reshape(-1, H, W, Cn).transpose(0, 3, 1, 2).reshape(w.shape[0], -1)
            y = oracle.fc(a.reshape(B, -1), w_nchw, 'f32', bias=l['bias']).reshape(B, -1, 1, 1)
            y = quantize(y, l['quant'])
        elif l['type'] == 'pool':
            y = pool(a, l['pool'], (l['kH'], l['kW']), l['stride'], l['pad'])
        elif l['type'] == 'sum':
            y = quantize(oracle.elemwise_sum([outs[i] for i in l['inputs']], 'f32'), l['quant'])
        elif l['type'] == 'scaling':
            y = quantize(a.copy(), l['quant'])
        else:
            raise ValueError(l['type'])
        outs[idx] = y
        res.append(np.transpose(np.rint(y).astype(np.int64), (0, 2, 3, 1)))
    return res


# ---- the reference's Target top-N CUDA kernel (src/Target/Target_CUDA_kernels.cu), GPU boxes only -------------------
TARGET_SO = os.path.join(_HERE, '_ref', 'libn2d2_targetshim.so')
_TARGET_LIB = None


def target_available():
    return os.path.exists(TARGET_SO)


def estimated_target(scores_nchw, top_n):
    """cudaGetEstimatedTarget of the reference on float scores [batch][class][y][x] (run on the current GPU):
    returns (labels int32, values float32), each [batch][top_n][y][x]."""
    global _TARGET_LIB
    if _TARGET_LIB is None:
        _TARGET_LIB = C.CDLL(TARGET_SO)
    s = np.ascontiguousarray(scores_nchw, np.float32)
    B, Cn, H, W = s.shape
    labels = np.zeros((B, top_n, H, W), np.int32)
    values = np.zeros((B, top_n, H, W), np.float32)
    rc = _TARGET_LIB.refshim_estimated_target(top_n, Cn, H, W, B, _p(s), _p(values), _p(labels))
    if rc != 0:
        raise RuntimeError(f'refshim_estimated_target failed ({rc})')
    return labels, values
