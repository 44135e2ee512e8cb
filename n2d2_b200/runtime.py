"""ctypes binding of the C ABI (include/n2d2b.h, built into n2d2_b200/libn2d2b.so).

This is the Python harness over the boundary: it feeds a network description (netdesc.py) through
the same entry points the C++ host classes use.  There is no CPU path here: if the library is
missing or no B200 is present the calls raise.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from .netdesc import ACTS, MODES, pack_bits, pack_int4

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, 'libn2d2b.so')

KEEP_ALL_OUTPUTS = 1
NO_FUSION = 2
FORCE_SIMT = 4
FORCE_IM2COL = 8
FORCE_PAIR = 32
EXACT64_EPILOGUE = 16
FUSE_FIRST_POOL = 64


class N2D2BError(RuntimeError):
    pass


class Scaling(C.Structure):
    _fields_ = [('mode', C.c_int32), ('nb_channels', C.c_int32), ('fscale', C.c_void_p), ('mult', C.c_void_p),
                ('frac_bits', C.c_int32), ('frac_bits_per_channel', C.c_void_p), ('shift0', C.c_void_p),
                ('shift1', C.c_void_p), ('is_clipped', C.c_int32), ('clip', C.c_void_p)]


class Quant(C.Structure):
    _fields_ = [('scaling', Scaling), ('activation', C.c_int32), ('out_bits', C.c_int32),
                ('out_unsigned', C.c_int32), ('saturation_threshold', C.c_int32)]


class ConvDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        'input', 'nb_outputs', 'kernel_h', 'kernel_w', 'stride_y', 'stride_x', 'pad_top', 'pad_left',
        'pad_bottom', 'pad_right', 'dilation_y', 'dilation_x', 'groups', 'weight_bits')]


class PoolDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        'input', 'pooling', 'pool_h', 'pool_w', 'stride_y', 'stride_x', 'pad_y', 'pad_x')]


class TensorInfo(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        'channels', 'height', 'width', 'dtype', 'is_unsigned', 'producer', 'readable')]


_lib = None


def load():
    """Loads libn2d2b.so; raises if it has not been built (there is no fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise N2D2BError(f'{LIB_PATH} is missing: build it with `python -m n2d2_b200.build`')
        lib = C.CDLL(LIB_PATH)
        lib.n2d2b_last_error.restype = C.c_char_p
        lib.n2d2b_net_cell_engine.restype = C.c_char_p
        lib.n2d2b_net_cell_engine.argtypes = [C.c_void_p, C.c_int]
        lib.n2d2b_net_create.argtypes = [C.c_int, C.POINTER(C.c_void_p)]
        lib.n2d2b_net_destroy.argtypes = [C.c_void_p]
        lib.n2d2b_net_destroy.restype = None
        lib.n2d2b_net_set_input.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int)]
        lib.n2d2b_net_add_conv.argtypes = [C.c_void_p, C.POINTER(ConvDesc), C.c_void_p, C.c_void_p,
                                           C.POINTER(Quant), C.POINTER(C.c_int)]
        lib.n2d2b_net_add_fc.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                         C.POINTER(Quant), C.POINTER(C.c_int)]
        lib.n2d2b_net_add_pool.argtypes = [C.c_void_p, C.POINTER(PoolDesc), C.POINTER(C.c_int)]
        lib.n2d2b_net_add_elemwise_sum.argtypes = [C.c_void_p, C.POINTER(C.c_int), C.c_int, C.POINTER(Quant),
                                                   C.POINTER(C.c_int)]
        lib.n2d2b_net_add_scaling.argtypes = [C.c_void_p, C.c_int, C.POINTER(Quant), C.POINTER(C.c_int)]
        lib.n2d2b_net_finalize.argtypes = [C.c_void_p, C.c_int, C.c_uint]
        lib.n2d2b_net_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        lib.n2d2b_net_forward_host.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        lib.n2d2b_net_check.argtypes = [C.c_void_p, C.c_void_p]
        lib.n2d2b_net_set_slices.argtypes = [C.c_void_p, C.c_int]
        lib.n2d2b_net_submit_host.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        lib.n2d2b_net_wait.argtypes = [C.c_void_p]
        lib.n2d2b_net_selftest_wait_timeout.argtypes = [C.c_void_p, C.c_uint, C.c_void_p]
        lib.n2d2b_net_estimated_labels.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        lib.n2d2b_net_estimated_labels_topn.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        lib.n2d2b_net_estimated_labels_topn_host.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        lib.n2d2b_quantize_stimuli.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                               C.c_void_p, C.c_void_p]
        lib.n2d2b_net_num_tensors.argtypes = [C.c_void_p]
        lib.n2d2b_net_tensor_info.argtypes = [C.c_void_p, C.c_int, C.POINTER(TensorInfo)]
        lib.n2d2b_net_read_tensor.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_size_t]
        lib.n2d2b_net_launches_per_forward.argtypes = [C.c_void_p]
        lib.n2d2b_net_weight_bytes.argtypes = [C.c_void_p, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]
        lib.n2d2b_net_profile.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int,
                                          C.c_void_p]
        lib.n2d2b_scaling_propagate.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.POINTER(Quant),
                                                C.c_void_p]
        lib.n2d2b_probe_i8_mma_rate.argtypes = [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_double), C.POINTER(C.c_double)]
        lib.n2d2b_first_conv_noalloc.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                                 C.POINTER(ConvDesc), C.c_void_p, C.c_void_p, C.POINTER(Quant),
                                                 C.c_void_p, C.c_void_p]
        _lib = lib
    return _lib


def check(rc):
    if rc < 0:
        raise N2D2BError(f'n2d2b status {rc}: {load().n2d2b_last_error().decode()}')
    return rc


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def make_quant(q, channels):
    """Builds the C struct for a quant dict; returns (struct, keepalive list)."""
    keep = []

    def arr(key, dtype):
        v = q.get(key)
        if v is None:
            return None
        a = np.ascontiguousarray(v, dtype)
        keep.append(a)
        return _ptr(a)

    s = Scaling()
    s.mode = MODES[q['mode']]
    s.nb_channels = channels
    s.fscale = arr('fscale', np.float32)
    s.mult = arr('mult', np.int32)
    s.frac_bits = int(q.get('frac_bits', 0))
    s.frac_bits_per_channel = arr('frac_bits_per_ch', np.uint8)
    s.shift0 = arr('shift0', np.uint8)
    s.shift1 = arr('shift1', np.uint8)
    s.is_clipped = 1 if q.get('is_clipped') else 0
    s.clip = arr('clip', np.float32)
    qq = Quant()
    qq.scaling = s
    qq.activation = ACTS[q.get('act', 'linear')]
    qq.out_bits = int(q.get('out_bits', 8))
    qq.out_unsigned = 1 if q.get('out_unsigned') else 0
    qq.saturation_threshold = int(q.get('sat_thr', 0))
    return qq, keep


class QuantizedNet:
    """One quantized network on one GPU (an n2d2b_net)."""

    def __init__(self, net, max_batch, device=0, flags=0, pack4=True):
        self.lib = load()
        self.desc = net
        self.handle = C.c_void_p()
        check(self.lib.n2d2b_net_create(device, C.byref(self.handle)))
        self.device = device
        self.max_batch = max_batch
        i = net['input']
        tid = C.c_int()
        check(self.lib.n2d2b_net_set_input(self.handle, i['C'], i['H'], i['W'], 1 if i['unsigned'] else 0, C.byref(tid)))
        self.tensor_of_layer = {-1: tid.value}
        for idx, l in enumerate(net['layers']):
            ins = [self.tensor_of_layer[j] for j in l['inputs']]
            if l['type'] in ('conv', 'fc'):
                w = np.ascontiguousarray(l['weights'], np.int8)
                if l.get('maps') is not None:
                    # sparse connection map [Cout][Cin] of the reference's Cell mapping: unconnected channels get zero
                    # weights in the dense layer the device runs ([Cout][kH][kW][Cin])
                    if l['type'] != 'conv' or l['groups'] != 1:
                        raise ValueError('a connection map needs a convolution without groups')
                    w = np.ascontiguousarray(w * np.asarray(l['maps'], np.int8)[:, None, None, :])
                bits = int(l.get('weight_bits', 8))
                packed = pack4 and bits in (1, 2, 4)
                wbuf = (pack_int4(w) if bits == 4 else pack_bits(w, bits)) if packed else w
                wbits = bits if packed else 8
                b = None if l.get('bias') is None else np.ascontiguousarray(l['bias'], np.int32)
                q, keep = make_quant(l['quant'], l['Cout'])
                if l['type'] == 'conv':
                    d = ConvDesc(ins[0], l['Cout'], l['kH'], l['kW'], l['stride'][0], l['stride'][1], l['pad'][0],
                                 l['pad'][1], l['pad'][2], l['pad'][3], l['dil'][0], l['dil'][1], l['groups'], wbits)
                    check(self.lib.n2d2b_net_add_conv(self.handle, C.byref(d), _ptr(wbuf), _ptr(b), C.byref(q),
                                                      C.byref(tid)))
                else:
                    check(self.lib.n2d2b_net_add_fc(self.handle, ins[0], l['Cout'], wbits, _ptr(wbuf), _ptr(b),
                                                    C.byref(q), C.byref(tid)))
            elif l['type'] == 'pool':
                d = PoolDesc(ins[0], 0 if l['pool'] == 'max' else 1, l['kH'], l['kW'], l['stride'][0], l['stride'][1],
                             l['pad'][0], l['pad'][1])
                check(self.lib.n2d2b_net_add_pool(self.handle, C.byref(d), C.byref(tid)))
            elif l['type'] == 'sum':
                info = self.tensor_info(ins[0])
                q, keep = make_quant(l['quant'], info.channels)
                arr = (C.c_int * len(ins))(*ins)
                check(self.lib.n2d2b_net_add_elemwise_sum(self.handle, arr, len(ins), C.byref(q), C.byref(tid)))
            elif l['type'] == 'scaling':
                info = self.tensor_info(ins[0])
                q, keep = make_quant(l['quant'], info.channels)
                check(self.lib.n2d2b_net_add_scaling(self.handle, ins[0], C.byref(q), C.byref(tid)))
            else:
                raise ValueError(l['type'])
            self.tensor_of_layer[idx] = tid.value
        check(self.lib.n2d2b_net_finalize(self.handle, max_batch, flags))
        out = self.tensor_info(self.tensor_of_layer[len(net['layers']) - 1])
        self.out_info = out
        self.out_elems = out.channels * out.height * out.width
        self.out_dtype = np.int32 if out.dtype == 1 else (np.uint8 if out.is_unsigned else np.int8)
        self.in_elems = i['C'] * i['H'] * i['W']

    def close(self):
        if self.handle:
            self.lib.n2d2b_net_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def tensor_info(self, tid):
        info = TensorInfo()
        check(self.lib.n2d2b_net_tensor_info(self.handle, tid, C.byref(info)))
        return info

    def engines(self):
        return [self.lib.n2d2b_net_cell_engine(self.handle, i).decode() for i in range(len(self.desc['layers']))]

    def weight_bytes(self):
        """(bytes of weights in HBM, bytes among them that are packed 4-bit weights)."""
        total, packed = C.c_size_t(), C.c_size_t()
        check(self.lib.n2d2b_net_weight_bytes(self.handle, C.byref(total), C.byref(packed)))
        return total.value, packed.value

    def launches_per_forward(self):
        return check(self.lib.n2d2b_net_launches_per_forward(self.handle))

    def forward_device(self, d_in_ptr, batch, d_out_ptr, stream=0):
        """Raw device pointers (ints); asynchronous on `stream`."""
        check(self.lib.n2d2b_net_forward(self.handle, d_in_ptr, batch, d_out_ptr, stream))

    def forward_host(self, x, out=None, stream=0):
        """x: [batch][H][W][C] 8-bit numpy array (or any buffer with a ctypes pointer). Returns the
        last cell's output as [batch][out_elems]."""
        batch = x.shape[0]
        if out is None:
            out = np.empty((batch, self.out_elems), self.out_dtype)
        check(self.lib.n2d2b_net_forward_host(self.handle, _ptr(x), batch, _ptr(out), stream))
        return out

    def forward_host_ptr(self, h_in_ptr, batch, h_out_ptr, stream=0):
        check(self.lib.n2d2b_net_forward_host(self.handle, h_in_ptr, batch, h_out_ptr, stream))

    def estimated_labels_topn(self, batch, top_n, d_labels_ptr, d_values_ptr=None, stream=0):
        """Target top-N of the last forward pass: labels / values [batch][top_n][height][width] int32 on the device."""
        check(self.lib.n2d2b_net_estimated_labels_topn(self.handle, batch, top_n, d_labels_ptr, d_values_ptr, stream))

    def estimated_labels_topn_host(self, batch, top_n):
        """Target top-N of the last forward pass as numpy arrays (labels, values), each [batch][top_n][height][width]."""
        t = self.out_info
        labels = np.empty((batch, top_n, t.height, t.width), np.int32)
        values = np.empty((batch, top_n, t.height, t.width), np.int32)
        check(self.lib.n2d2b_net_estimated_labels_topn_host(self.handle, batch, top_n, _ptr(labels), _ptr(values)))
        return labels, values

    def estimated_labels(self, batch, d_labels_ptr, d_values_ptr=None, stream=0):
        """Top-1 class of the last forward pass's final tensor (first maximum wins), into device int32 buffers."""
        check(self.lib.n2d2b_net_estimated_labels(self.handle, batch, d_labels_ptr, d_values_ptr, stream))

    def check(self, stream=0):
        """Waits for `stream` and raises if a kernel of this network gave up on a bounded wait."""
        check(self.lib.n2d2b_net_check(self.handle, stream))

    def set_slices(self, n):
        check(self.lib.n2d2b_net_set_slices(self.handle, n))

    def submit_host_ptr(self, h_in_ptr, batch, h_out_ptr, stream=0):
        """Streaming form: returns at once; h_out is complete after wait()."""
        check(self.lib.n2d2b_net_submit_host(self.handle, h_in_ptr, batch, h_out_ptr, stream))

    def wait(self):
        check(self.lib.n2d2b_net_wait(self.handle))

    def selftest_wait_timeout(self, limit_us=1000, stream=0):
        check(self.lib.n2d2b_net_selftest_wait_timeout(self.handle, limit_us, stream))

    def read_layer(self, layer_idx, batch):
        """Output of layer `layer_idx` of the last forward as an NHWC integer array (needs KEEP_ALL_OUTPUTS
        unless it is the last layer)."""
        tid = self.tensor_of_layer[layer_idx]
        info = self.tensor_info(tid)
        dt = np.int32 if info.dtype == 1 else (np.uint8 if info.is_unsigned else np.int8)
        a = np.empty((batch, info.height, info.width, info.channels), dt)
        check(self.lib.n2d2b_net_read_tensor(self.handle, tid, batch, _ptr(a), a.nbytes))
        return a

    def profile(self, d_in_ptr, batch, d_out_ptr, stream=0):
        n = len(self.desc['layers'])
        ms = np.zeros(n, np.float32)
        check(self.lib.n2d2b_net_profile(self.handle, d_in_ptr, batch, d_out_ptr, _ptr(ms), n, stream))
        return ms


def scaling_propagate(x_i32_dev_ptr, out_dev_ptr, nb_pixels, q, channels, device=0, stream=0):
    qq, keep = make_quant(q, channels)
    check(load().n2d2b_scaling_propagate(device, x_i32_dev_ptr, out_dev_ptr, nb_pixels, C.byref(qq), stream))


def quantize_stimuli(d_in_ptr, batch, channels, height, width, d_out_ptr, nb_bits=8, env_unsigned=True, device=0, stream=0):
    """Float NCHW stimuli -> trunc(x * (2^n - 1 | 2^(n-1) - 1)) as 8-bit NHWC (the input edge of a quantized network)."""
    check(load().n2d2b_quantize_stimuli(device, d_in_ptr, batch, channels, height, width, nb_bits, 1 if env_unsigned else 0,
                                        d_out_ptr, stream))


def probe_i8_mma_rate(device=0, n=256, reps=40000):
    """Measured dense int8 tensor-pipe rate of the GPU: (TOP/s over the whole chip, SM cycles per 128 x n x 32 MMA)."""
    tops, cyc = C.c_double(), C.c_double()
    check(load().n2d2b_probe_i8_mma_rate(device, n, reps, C.byref(tops), C.byref(cyc)))
    return tops.value, cyc.value


NOALLOC_MAX_PIXELS = 8 * 1024 * 1024


def first_conv_noalloc(d_in_ptr, batch, height, width, channels, in_unsigned, layer, d_out_ptr, device=0, stream=0):
    """First-layer convolution through the entry point that allocates no device memory (its scratch is
    a fixed array inside the library; see include/n2d2b.h for the limits).  `layer` is a conv layer
    dict of netdesc.py; d_in_ptr / d_out_ptr are raw device pointers."""
    w = np.ascontiguousarray(layer['weights'], np.int8)
    b = None if layer.get('bias') is None else np.ascontiguousarray(layer['bias'], np.int32)
    q, keep = make_quant(layer['quant'], layer['Cout'])
    d = ConvDesc(0, layer['Cout'], layer['kH'], layer['kW'], layer['stride'][0], layer['stride'][1], layer['pad'][0],
                 layer['pad'][1], layer['pad'][2], layer['pad'][3], layer['dil'][0], layer['dil'][1], layer['groups'],
                 int(layer.get('weight_bits', 8)))
    check(load().n2d2b_first_conv_noalloc(device, d_in_ptr, batch, height, width, channels, 1 if in_unsigned else 0,
                                          C.byref(d), _ptr(w), _ptr(b), C.byref(q), d_out_ptr, stream))
