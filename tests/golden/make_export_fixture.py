"""Writes tests/golden/export_fixture/: a small quantized network in the two on-disk forms of the
reference - the per-cell headers of its CPP_Quantization export and `.syntxt` parameter files - for
the import tests (tests/test_export_import.py).

The text follows what the reference's writers emit, statement by statement:
  geometry defines      src/Export/CPP/CPP_ConvCellExport.cpp:75-135, CPP_FcCellExport.cpp:67-89,
                        CPP_PoolCellExport.cpp:74-94, CPP_ElemWiseCellExport.cpp:63-144
  biases                CPP_ConvCellExport.cpp:145-174 ("b + half" for single-shift cells,
                        src/Export/CellExport.cpp:100-117)
  weights               CPP_ConvCellExport.cpp:251-260 (OHWC), :419-607 (`data<4>` hex bytes, first
                        value in the high nibble), CPP_FcCellExport.cpp:143-161
  activation, scaling   src/Export/CPP/CPP_CellExport.cpp:53-83,110-241
  .syntxt               src/Cell/ConvCell.cpp:299-411 (one line per output, channel by channel, kernel
                        x-fastest; biases one per line)

Run from the repository root:  python tests/golden/make_export_fixture.py
The network itself comes from fixture_net() below (seeded), which the tests rebuild to know the
expected values.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from n2d2_b200 import netdesc  # noqa: E402

OUT = os.path.join(ROOT, 'tests', 'golden', 'export_fixture')


def fixture_net():
    b = netdesc.NetBuilder('export_fixture', 1, 12, 12, 31, 'single', weight_dist=('uniform', 127), calibrate=True)
    c1 = b.conv(-1, 8, 3, stride=1, pad=1, name='conv1')                       # single shift per channel
    p1 = b.pool(c1, 'max', 2, 2, name='pool1')
    b.scaling_mode = 'double'
    c2 = b.conv(p1, 16, 3, name='conv2')                                       # double shift per channel
    b.scaling_mode, b.weight_bits, b.clipped = 'fixed', 4, True
    c3 = b.conv(c2, 16, 1, act='linear', name='conv3_w4')                      # int4 weights, clipped fixed point
    # the export writes clipping values as int32 (CPP_CellExport.cpp:186-189): keep them integral so that the
    # header holds exactly what the cell computes with
    qc = b.net['layers'][c3]['quant']
    qc['clip'] = np.floor(qc['clip']).astype(np.float32)
    b.weight_bits, b.clipped = 8, False
    s = b.sum([c3, c2], act='relu', name='sum1', mode='single')
    q = b.net['layers'][s]['quant']
    q['shift0'] = np.full_like(q['shift0'], 1)                                 # uniform: the template form
    f = b.fc(s, 10, act='linear', name='fc1')
    q = b.net['layers'][f]['quant']
    q['mult'] = np.full_like(q['mult'], int(q['mult'][0]))                     # uniform multiplier: FixedPointScaling<m, f>
    return b.net


def _join(values, per_line):
    out, n = [], 0
    for v in values:
        out.append(f'{v}, ')
        n += 1
        if n % per_line == 0:
            out.append('\n')
    return ''.join(out)


def scaling_text(prefix, q, out_unsigned):
    m = q['mode']
    if m == 'none':
        return f'static const N2D2_Export::NoScaling {prefix}_SCALING;\n'
    if m == 'single':
        s = [int(v) for v in q['shift0']]
        if len(set(s)) == 1:
            return f'static const N2D2_Export::SingleShiftScaling<{s[0]}> {prefix}_SCALING;\n'
        return (f'static const N2D2_Export::SingleShiftScalingPerChannel<{len(s)}> {prefix}_SCALING = {{'
                + ''.join(f'{v}, ' for v in s) + '};\n')
    if m == 'double':
        a, b = [int(v) for v in q['shift0']], [int(v) for v in q['shift1']]
        if len(set(zip(a, b))) == 1:
            return f'static const N2D2_Export::DoubleShiftScaling<{a[0]}, {b[0]}> {prefix}_SCALING;\n'
        return (f'static const N2D2_Export::DoubleShiftScalingPerChannel<{len(a)}, {int(out_unsigned)}> {prefix}_SCALING = {{'
                + ''.join(f'std::array<SUM_T, 3>{{{x}, {y}, {1 << (y - 1)}}}, ' for x, y in zip(a, b)) + '};\n')
    if m in ('fixed16', 'fixed32'):
        mult, f = [int(v) for v in q['mult']], int(q['frac_bits'])
        if q.get('is_clipped'):
            clip = [int(v) for v in q['clip']]     # the reference writes the clipping values as int32
            return (f'static const N2D2_Export::FixedPointClippingAndScalingPerChannel<{len(mult)}, {f}> {prefix}_SCALING = {{{{'
                    + ','.join(map(str, mult)) + '}, {' + ','.join(map(str, clip)) + '}};\n')
        if len(set(mult)) == 1:
            return f'static const N2D2_Export::FixedPointScaling<{mult[0]}, {f}> {prefix}_SCALING;\n'
        return (f'static const N2D2_Export::FixedPointScalingPerChannel<{len(mult)}, {f}> {prefix}_SCALING = {{'
                + ','.join(map(str, mult)) + '};\n')
    raise ValueError(m)


def header_guard(name, body):
    up = name.upper()
    return (f'// N2D2 auto-generated file.\n\n#ifndef N2D2_EXPORTC_{up}_LAYER_H\n#define N2D2_EXPORTC_{up}_LAYER_H\n\n'
            '#include "../../include/typedefs.h"\n#include "../../include/utils.h"\n' + body
            + f'#endif // N2D2_EXPORTC_{up}_LAYER_H\n')


ACT = {'relu': 'Rectifier', 'linear': 'Linear', 'saturation': 'Saturation'}


def biases_text(name, l, size_macro):
    q = l['quant']
    items = []
    for o in range(l['Cout']):
        t = '0' if l.get('bias') is None else str(int(l['bias'][o]))
        if q['mode'] == 'single' and int(q['shift0'][o]) > 0:
            t += f" + {1 << (int(q['shift0'][o]) - 1)}"
        items.append(t + ', ')
    ctype = 'int16_t' if l.get('weight_bits', 8) <= 4 else 'int32_t'
    return (f'static const {ctype} {name}_biases[{size_macro}] N2D2_SECTION_ATTRIBUTE(N2D2_SECTION_NN_BIASSES) = {{'
            + ''.join(items) + '};\n\n')


def weights_text(name, prefix, l, order_comment):
    w = np.asarray(l['weights'])
    bits = int(l.get('weight_bits', 8))
    if bits == 8:
        return (order_comment + f'static const WDATA_T {name}_weights[{prefix}_WEIGHTS_SIZE] '
                'N2D2_SECTION_ATTRIBUTE(N2D2_SECTION_NN_WEIGHTS) = {' + _join([int(v) for v in w.reshape(-1)], 24) + '};\n\n')
    # sub-byte: every (output, ky, kx) run of channels packed into whole bytes, first value in the high bits
    runs = w.reshape(-1, w.shape[-1]).astype(np.int64)
    per = 8 // bits
    items = []
    for run in runs:
        vals = list(run) + [0] * ((-len(run)) % per)
        for k in range(0, len(vals), per):
            acc = 0
            for v in vals[k:k + per]:
                acc = (acc << bits) | (int(v) & ((1 << bits) - 1))
            items.append(f'0x{acc:02x}')
    return (order_comment + f'static const data<{bits}> {name}_weights[{prefix}_WEIGHTS_SIZE] '
            'N2D2_SECTION_ATTRIBUTE(N2D2_SECTION_NN_WEIGHTS) = {' + _join(items, 24) + '\n};\n\n')


def conv_header(l, shape_in, shape_out, out_unsigned):
    name, p = l['name'], l['name'].upper()
    C, H, W = shape_in
    O, oH, oW = shape_out
    d = [('NB_OUTPUTS', O), ('NB_CHANNELS', C), ('OUTPUTS_WIDTH', oW), ('OUTPUTS_HEIGHT', oH), ('OX_SIZE', oW), ('OY_SIZE', oH),
         ('CHANNELS_WIDTH', W), ('CHANNELS_HEIGHT', H), ('KERNEL_WIDTH', l['kW']), ('KERNEL_HEIGHT', l['kH']),
         ('SUB_SAMPLE_X', 1), ('SUB_SAMPLE_Y', 1), ('STRIDE_X', l['stride'][1]), ('STRIDE_Y', l['stride'][0]),
         ('PADDING_X', l['pad'][1]), ('PADDING_Y', l['pad'][0]), ('DILATION_X', l['dil'][1]), ('DILATION_Y', l['dil'][0]),
         ('NO_BIAS', 0 if l.get('bias') is not None else 1)]
    body = ''.join(f'#define {p}_{k} {v}\n' for k, v in d) + '\n'
    body += ('// Kernel size if dilation is included in weights\n'
             f"#define {p}_DILATED_KERNEL_WIDTH {l['dil'][1] * (l['kW'] - 1) + 1}\n"
             f"#define {p}_DILATED_KERNEL_HEIGHT {l['dil'][0] * (l['kH'] - 1) + 1}\n\n")
    body += f"#define {p}_ACTIVATION {ACT[l['quant']['act']]}\n"
    body += scaling_text(p, l['quant'], out_unsigned) + '\n'
    body += (f'#define {p}_OUTPUTS_SIZE ({p}_NB_OUTPUTS*{p}_OUTPUTS_WIDTH*{p}_OUTPUTS_HEIGHT)\n'
             f'#define {p}_CHANNELS_SIZE ({p}_NB_CHANNELS*{p}_CHANNELS_WIDTH*{p}_CHANNELS_HEIGHT)\n\n')
    body += biases_text(name, l, f'{p}_NB_OUTPUTS')
    body += f'#define {p}_WEIGHTS_SIZE ({p}_NB_OUTPUTS*{p}_KERNEL_WIDTH*{p}_KERNEL_HEIGHT*{p}_NB_CHANNELS)\n\n'
    body += weights_text(name, p, l, '// Flatten weights with the order [NB_OUTPUTS][KERNEL_HEIGHT][KERNEL_WIDTH][NB_CHANNELS]\n')
    return header_guard(name, body)


def fc_header(l, shape_in, out_unsigned):
    name, p = l['name'], l['name'].upper()
    C, H, W = shape_in
    d = [('NB_OUTPUTS', l['Cout']), ('NB_CHANNELS', C), ('OUTPUTS_WIDTH', 1), ('OUTPUTS_HEIGHT', 1), ('CHANNELS_WIDTH', W),
         ('CHANNELS_HEIGHT', H), ('NO_BIAS', 0 if l.get('bias') is not None else 1)]
    body = ''.join(f'#define {p}_{k} {v}\n' for k, v in d) + '\n'
    body += f"#define {p}_ACTIVATION {ACT[l['quant']['act']]}\n"
    body += scaling_text(p, l['quant'], out_unsigned) + '\n'
    body += (f'#define {p}_OUTPUTS_SIZE ({p}_NB_OUTPUTS*{p}_OUTPUTS_WIDTH*{p}_OUTPUTS_HEIGHT)\n'
             f'#define {p}_CHANNELS_SIZE ({p}_NB_CHANNELS*{p}_CHANNELS_WIDTH*{p}_CHANNELS_HEIGHT)\n\n')
    body += biases_text(name, l, f'{p}_OUTPUTS_SIZE')
    body += f'#define {p}_WEIGHTS_SIZE ({p}_OUTPUTS_SIZE*{p}_CHANNELS_SIZE)\n\n'
    body += weights_text(name, p, l, '// Flatten weights with the order[OUTPUTS_SIZE][CHANNELS_SIZE]. \n'
                         '// If the previous cell was a 2D cell, CHANNELS_SIZE is flatten in the '
                         '[CHANNELS_HEIGHT][CHANNELS_WIDTH][NB_CHANNELS] order.\n')
    return header_guard(name, body)


def pool_header(l, shape_in, shape_out):
    name, p = l['name'], l['name'].upper()
    C, H, W = shape_in
    O, oH, oW = shape_out
    d = [('NB_OUTPUTS', O), ('NB_CHANNELS', C), ('OUTPUTS_WIDTH', oW), ('OUTPUTS_HEIGHT', oH), ('CHANNELS_WIDTH', W),
         ('CHANNELS_HEIGHT', H)]
    body = ''.join(f'#define {p}_{k} {v}\n' for k, v in d) + '\n'
    body += (f'#define {p}_OUTPUTS_SIZE ({p}_NB_OUTPUTS*{p}_OUTPUTS_WIDTH*{p}_OUTPUTS_HEIGHT)\n'
             f'#define {p}_CHANNELS_SIZE ({p}_NB_CHANNELS*{p}_CHANNELS_WIDTH*{p}_CHANNELS_HEIGHT)\n\n')
    d = [('POOL_WIDTH', l['kW']), ('POOL_HEIGHT', l['kH']), ('PADDING_X', l['pad'][1]), ('PADDING_Y', l['pad'][0]),
         ('STRIDE_X', l['stride'][1]), ('STRIDE_Y', l['stride'][0]), ('POOLING', 'Max' if l['pool'] == 'max' else 'Average')]
    body += ''.join(f'#define {p}_{k} {v}\n' for k, v in d) + '\n'
    body += f'#define {p}_ACTIVATION Linear\nstatic const N2D2_Export::NoScaling {p}_SCALING;\n\n'
    return header_guard(name, body)


def sum_header(l, shape, out_unsigned):
    name, p = l['name'], l['name'].upper()
    C, H, W = shape
    d = [('NB_INPUTS', len(l['inputs'])), ('NB_OUTPUTS', C), ('NB_CHANNELS', C * len(l['inputs'])), ('OUTPUTS_WIDTH', W),
         ('OUTPUTS_HEIGHT', H), ('CHANNELS_WIDTH', W), ('CHANNELS_HEIGHT', H)]
    body = ''.join(f'#define {p}_{k} {v}\n' for k, v in d) + '\n'
    body += f"#define {p}_ACTIVATION {ACT[l['quant']['act']]}\n"
    body += scaling_text(p, l['quant'], out_unsigned) + '\n'
    body += f'#define {p}_ELEM_OP Sum\n#define {p}_ELEM_COEFF_MODE PerLayer\n\n'
    return header_guard(name, body)


def syntxt(l):
    """Conv weights in the reference's OCHW export format (our arrays are [O][kH][kW][C])."""
    w = np.asarray(l['weights']).astype(np.int64)
    O = w.shape[0]
    lines = []
    for o in range(O):
        vals = []
        for c in range(w.shape[3]):
            for y in range(w.shape[1]):
                for x in range(w.shape[2]):
                    vals.append(f'{int(w[o, y, x, c])} ')
        lines.append(''.join(vals) + '\n')
    biases = ''.join(f'{int(b)}\n' for b in l['bias'])
    return ''.join(lines), biases


def main():
    net = fixture_net()
    os.makedirs(OUT, exist_ok=True)
    _, shapes = netdesc.layer_macs(net)
    for i, l in enumerate(net['layers']):
        sin = shapes[l['inputs'][0]]
        q = l.get('quant', {})
        path = os.path.join(OUT, l['name'] + '.hpp')
        if l['type'] == 'conv':
            text = conv_header(l, sin, shapes[i], q.get('out_unsigned', False))
        elif l['type'] == 'fc':
            text = fc_header(l, sin, q.get('out_unsigned', False))
        elif l['type'] == 'pool':
            text = pool_header(l, sin, shapes[i])
        elif l['type'] == 'sum':
            text = sum_header(l, shapes[i], q.get('out_unsigned', False))
        else:
            raise ValueError(l['type'])
        open(path, 'w').write(text)
    w, b = syntxt(net['layers'][0])
    open(os.path.join(OUT, 'conv1_weights.syntxt'), 'w').write(w)
    open(os.path.join(OUT, 'conv1_biases.syntxt'), 'w').write(b)
    print('wrote', sorted(os.listdir(OUT)))


if __name__ == '__main__':
    main()
