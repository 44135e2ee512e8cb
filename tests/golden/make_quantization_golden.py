"""Generates tests/golden/quantization_golden.txt from the REFERENCE's own scaling approximations
(DeepNetQuantization::approximateScalingWithFixedPoint and ::approximateScalingWithPowerOf2Divs,
src/DeepNetQuantization.cpp:1043-1134), compiled where they lie into oracle/_ref/libn2d2_quantshim.so by
oracle/refshim/Makefile.  Needs the reference tree; the fixture it writes is committed and replayed by
tests/test_quantization.py everywhere else.

    make -C oracle/refshim REF=<reference tree> && python tests/golden/make_quantization_golden.py

Lines:  p2 <scaling as a hex float> <nbDivisions> | <precision as a hex double> <exponents...>
        fx <mode 2|3> <scalings as hex floats...> | <fractional bits or -1> <mode after> <fixed-point scalings...>"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
SO = os.path.join(ROOT, 'oracle', '_ref', 'libn2d2_quantshim.so')


def lib():
    l = C.CDLL(SO)
    l.quantshim_power_of_2_divs.restype = C.c_double
    l.quantshim_power_of_2_divs.argtypes = [C.c_float, C.c_size_t, C.c_void_p]
    l.quantshim_fixed_point.restype = C.c_int
    l.quantshim_fixed_point.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
    return l


def power_of_2_divs(l, scaling, nb):
    e = (C.c_ubyte * nb)()
    precision = l.quantshim_power_of_2_divs(C.c_float(scaling), nb, e)
    return precision, list(e)


def fixed_point(l, mode, scalings):
    sc = np.ascontiguousarray(scalings, np.float32)
    out = np.zeros(len(sc), np.int32)
    m = C.c_int(mode)
    frac = l.quantshim_fixed_point(C.byref(m), sc.ctypes.data_as(C.c_void_p), len(sc), out.ctypes.data_as(C.c_void_p))
    return frac, m.value, [int(v) for v in out]


def cases():
    rng = np.random.default_rng(20240611)
    p2 = [1.0, 0.5, 0.25, 0.2525, 0.0119, 0.01, 0.75, 0.999, 0.9801, 0.98, 0.51, 2.0 ** -20, 3e-5, 0.3333333, 0.6667]
    p2 += [float(np.float32(v)) for v in rng.uniform(1e-4, 1.0, 120)]
    p2 += [float(np.float32(2.0 ** -k * (1.0 + d))) for k in range(1, 12) for d in (-1e-3, 0.0, 1e-3, 0.02, 0.0205)]
    fx = []
    for mode in (2, 3):
        for n in (1, 3, 16):
            for scale in (1e-4, 0.01, 0.7, 1.5, 40.0, 3.0e4, 4.0e4, 1.0e9, 3.0e9):
                fx.append((mode, [float(np.float32(v)) for v in rng.uniform(0.1, 1.0, n) * scale]))
    return p2, fx


def main():
    l = lib()
    p2, fx = cases()
    with open(os.path.join(HERE, 'quantization_golden.txt'), 'w') as f:
        f.write('# written by make_quantization_golden.py from the reference\'s compiled code\n')
        for s in p2:
            for nb in (1, 2):
                if not (0.0 < s <= 1.0):
                    continue
                precision, e = power_of_2_divs(l, s, nb)
                f.write(f'p2 {float(np.float32(s)).hex()} {nb} | {precision.hex()} ' + ' '.join(str(x) for x in e) + '\n')
        for mode, sc in fx:
            frac, m, out = fixed_point(l, mode, sc)
            f.write(f'fx {mode} ' + ' '.join(float(v).hex() for v in sc) + f' | {frac} {m} ' + ' '.join(str(x) for x in out) + '\n')
    print('written', 2 * len(p2), '+', len(fx), 'cases')


if __name__ == '__main__':
    main()
