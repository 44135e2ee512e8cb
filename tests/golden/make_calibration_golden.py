"""Generates tests/golden/calibration_golden.txt and tests/golden/calibration_state/{hist,range}.bin from the
REFERENCE's own Histogram / RangeStats code (src/Histogram.cpp, src/RangeStats.cpp), compiled where it lies into
oracle/_ref/libn2d2_calibshim.so by oracle/refshim/Makefile.  Needs the reference tree, so it runs where that tree
is; the fixtures it writes are committed and are what tests/test_calibration.py replays everywhere else.

    make -C oracle/refshim REF=<reference tree> && python tests/golden/make_calibration_golden.py

A case = values from a 64-bit linear congruential generator through a fixed sequence of IEEE double operations
(repeated bit for bit by tests/host/test_calibration.cpp), fed in two batches: ranges first, then the histogram
created over the first batch's range and enlarged for the second, like reportOutputsRange / reportOutputsHistogram
(src/DeepNetQuantization.cpp:150-281)."""
import ctypes as C
import os
import struct

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
SO = os.path.join(ROOT, 'oracle', '_ref', 'libn2d2_calibshim.so')

# (kind, seed, n, scale, bits, mode)
CASES = [('bell', 1, 20000, 3.0, 8, 'MSE'), ('bell', 2, 20000, 0.02, 8, 'KL-Divergence'), ('relu', 3, 30000, 3.5, 8, 'MSE'),
         ('relu', 4, 30000, 100.0, 8, 'KL-Divergence'), ('tail', 5, 40000, 1.0, 8, 'MSE'), ('tail', 6, 40000, 1.0, 8, 'KL-Divergence'),
         ('bell', 7, 5000, 3.0, 4, 'MSE'), ('relu', 8, 5000, 1.0, 4, 'KL-Divergence'), ('tail', 9, 9000, 2.0, 5, 'MSE'),
         ('relu', 10, 50, 1.0, 8, 'MSE'), ('bell', 11, 12000, 7.0, 8, 'Quantile'), ('relu', 12, 2, 1.0, 8, 'KL-Divergence')]

MASK = (1 << 64) - 1


def nb_bins(bits, mode):
    return 65536 if mode == 'Quantile' else min((1 << bits) * 64, 65536)


def draw(kind, seed, n, scale):
    x = seed
    out = np.empty(n, np.float64)
    for i in range(n):
        u = []
        for _ in range(5):
            x = (x * 6364136223846793005 + 1442695040888963407) & MASK
            u.append(float(x >> 11) * (1.0 / 9007199254740992.0))
        b = (((u[0] + u[1]) + (u[2] + u[3])) - 2.0) * scale
        if kind == 'relu':
            b = b if b > 0.0 else 0.0
        if kind == 'tail':
            b = b * (1.0 + 8.0 * ((u[4] * u[4]) * (u[4] * u[4])))
        out[i] = float(np.float32(b))
    return out


def lib():
    l = C.CDLL(SO)
    l.calib_hist_new.restype = C.c_void_p
    l.calib_hist_new.argtypes = [C.c_double, C.c_double, C.c_size_t]
    l.calib_hist_free.argtypes = [C.c_void_p]
    l.calib_hist_add.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
    l.calib_hist_enlarge.argtypes = [C.c_void_p, C.c_double, C.c_int]
    for f in ('calib_hist_mse', 'calib_hist_kl'):
        getattr(l, f).restype = C.c_double
        getattr(l, f).argtypes = [C.c_void_p, C.c_size_t]
    l.calib_hist_quantile.restype = C.c_double
    l.calib_hist_quantile.argtypes = [C.c_void_p, C.c_double]
    l.calib_hist_nb_bins.restype = C.c_size_t
    l.calib_hist_nb_bins.argtypes = [C.c_void_p]
    for f in ('calib_hist_min', 'calib_hist_max'):
        getattr(l, f).restype = C.c_double
        getattr(l, f).argtypes = [C.c_void_p]
    l.calib_hist_bins.argtypes = [C.c_void_p, C.c_void_p]
    l.calib_hist_save.argtypes = [C.c_void_p, C.c_char_p, C.c_char_p]
    l.calib_range.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]
    l.calib_range_save.argtypes = [C.c_void_p, C.c_size_t, C.c_char_p, C.c_char_p]
    return l


def ptr(a):
    return a.ctypes.data_as(C.c_void_p)


def reference_case(l, kind, seed, n, scale, bits, mode):
    """The fields tests/host/test_calibration.cpp prints for the same case, from the reference's code."""
    v = draw(kind, seed, n, scale)
    h = n // 2
    r1 = np.zeros(5)
    r = np.zeros(5)
    first = np.ascontiguousarray(v[:h])
    l.calib_range(ptr(first), h, ptr(r1))
    l.calib_range(ptr(v), n, ptr(r))
    val = max(max(abs(r1[0]), abs(r1[1])), 0.1)
    hist = l.calib_hist_new(0.0 if kind == 'relu' else -val, val, nb_bins(bits, mode))
    assert hist
    assert l.calib_hist_add(hist, ptr(first), h) == 0
    lo = l.calib_hist_min(hist)
    l.calib_hist_enlarge(hist, max(abs(r[0]), abs(r[1])), 1 if lo < 0.0 else 0)
    rest = np.ascontiguousarray(v[h:])
    assert l.calib_hist_add(hist, ptr(rest), n - h) == 0
    nbins = l.calib_hist_nb_bins(hist)
    bins = np.zeros(nbins, np.uint64)
    l.calib_hist_bins(hist, ptr(bins))
    check = int(sum((i + 1) * int(b) for i, b in enumerate(bins)) & MASK)
    lo, hi = l.calib_hist_min(hist), l.calib_hist_max(hist)
    # centre of the bin the first value falls into (getBinValue(getBinIdx(v[0])))
    width = (hi - lo) / nbins
    clamped = min(max(v[0], lo), hi)
    idx = int((clamped - lo) / width + 1e-6)
    idx = idx - 1 if idx == nbins else idx
    centre = lo + (idx + 0.5) * width
    fields = [float(r[0]).hex(), float(r[1]).hex(), float(r[2]).hex(), float(r[3]).hex(), float(r[4]).hex(), str(nbins),
              lo.hex(), hi.hex(), str(check), l.calib_hist_mse(hist, bits).hex(), l.calib_hist_kl(hist, bits).hex(),
              l.calib_hist_quantile(hist, 0.9999).hex(), l.calib_hist_quantile(hist, 0.5).hex(), float(centre).hex()]
    l.calib_hist_free(hist)
    return fields


def main():
    l = lib()
    with open(os.path.join(HERE, 'calibration_golden.txt'), 'w') as f:
        f.write('# kind seed n scale bits mode | range min max m0 m1 m2 | bins min max checksum | MSE KL q0.9999 q0.5 centre\n')
        for case in CASES:
            f.write(' '.join(str(c) for c in case) + ' | ' + ' '.join(reference_case(l, *case)) + '\n')
    # state files of one histogram and one range, written by the reference's own save routines
    d = os.path.join(HERE, 'calibration_state')
    os.makedirs(d, exist_ok=True)
    v = draw('bell', 42, 4000, 3.0)
    r = np.zeros(5)
    l.calib_range(ptr(v), len(v), ptr(r))
    val = max(abs(r[0]), abs(r[1]))
    hist = l.calib_hist_new(-val, val, 64)
    assert l.calib_hist_add(hist, ptr(v), len(v)) == 0
    assert l.calib_hist_save(hist, b'conv1', os.path.join(d, 'hist.bin').encode()) == 0
    assert l.calib_range_save(ptr(v), len(v), b'conv1', os.path.join(d, 'range.bin').encode()) == 0
    l.calib_hist_free(hist)
    print('written', len(CASES), 'cases')


if __name__ == '__main__':
    main()
