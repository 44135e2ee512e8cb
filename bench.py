#!/usr/bin/env python
"""Benchmark of the quantized integer inference path: int8 ResNet-50 images/s.

    python bench.py --gpus N --steps K --warmup W          (N > 1: launched under torchrun)
    python bench.py --impl reference ...                   (the reference's CPU path, host cores)

    python bench.py --peak-probe                           (int8 tensor-pipe issue rate of this GPU)

One step = one forward pass of the quantized network over one batch of synthetic uint8 images.
Work is batch-sharded with no collective on the data path (the final int8 logits are all-gathered
once, outside the timed region): `--scaling weak` (default) gives every rank `--batch` images per
step, `--scaling strong` splits `--batch` images over the ranks.  Timing is CUDA events on the
launching stream, max over ranks, barrier + synchronize on both sides.  After the timed regions the
logits of a few images of the rank's own batch are compared with the CPU oracle and the three entry
points (device buffers, host buffers, streaming) with each other; any mismatch fails the run.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# DRAM bytes (dram__bytes_read + dram__bytes_write) of the 47 implicit-GEMM launches of one ResNet-50 forward
# pass at batch 256, from the ncu capture summarised under profiles/: reported as the batch-256 capture it is
# (at larger batches less of a layer's output is still in L2 when the next layer reads it).
IGEMM_DRAM_BYTES_B256_CAPTURE = 4671.13e6
IGEMM_LAUNCHES_B256_CAPTURE = 47

METRIC = 'int8_resnet50_images_per_sec'
UNIT = 'images/s'


def build_net(args):
    from n2d2_b200 import netdesc
    if args.workload == 'resnet50':
        return netdesc.resnet50(seed=4, size=224)
    if args.workload == 'resnet18':
        return netdesc.resnet18(seed=2, size=224)
    if args.workload == 'resnet18_w4':
        return netdesc.resnet18(seed=5, size=224, weight_bits=4, clipped=True)
    if args.workload == 'mobilenet_v1':
        return netdesc.mobilenet_v1(seed=3, size=224)
    if args.workload == 'mnist24':
        return netdesc.mnist24(seed=1)
    raise SystemExit(f'unknown workload {args.workload}')


def workload_config(args, net, world):
    names = {'resnet50': 'ResNet-50 (bottleneck 3-4-6-3, reference-ini geometry), 8-bit PTQ, DoubleShiftScaling, '
                         'int8 residual add with saturation, 3x224x224 uint8 input',
             'resnet18': 'ResNet-18, 8-bit PTQ, FixedPointScaling, 3x224x224 uint8 input',
             'resnet18_w4': 'ResNet-18, int4 weights / u8 activations, clipped FixedPointScaling',
             'mobilenet_v1': 'MobileNet v1 a=1.0, 8-bit PTQ, SingleShiftScaling',
             'mnist24': 'mnist24_16c4s2_24c5s2_150_10, 8-bit PTQ, SingleShiftScaling'}
    per_gpu = per_gpu_batch(args, world)
    return {'workload': names[args.workload], 'batch_per_gpu': per_gpu, 'global_batch': per_gpu * world,
            'parallelism': f'batch-sharded x{world}, no collective on the data path',
            'cache': 'inputs and activations larger than L2 (no flush needed)' if per_gpu >= 256
                     else 'L2 flushed between steps'}


def per_gpu_batch(args, world):
    if args.scaling == 'strong':
        if args.batch % world:
            raise SystemExit(f'--scaling strong: --batch {args.batch} is not a multiple of {world} ranks')
        return args.batch // world
    return args.batch


class ClockSampler:
    """Samples SM clocks and clock-event reasons while the timed region runs: NVML read-outs every few milliseconds
    from a thread (read-only queries), or nvidia-smi in a loop where the NVML binding is missing."""
    FIELDS = ('clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,'
              'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,'
              'clocks_event_reasons.sw_power_cap')
    REASONS = (('hw_slowdown', 0x8), ('hw_thermal_slowdown', 0x40), ('sw_thermal_slowdown', 0x20), ('sw_power_cap', 0x4))

    def __init__(self, index):
        self.index = index
        self.samples = []      # (time, sm MHz, max MHz, set of reasons)
        self.proc = None
        self.nvml = None
        self.stop_flag = False

    def start(self):
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            try:
                uuid = 'GPU-' + str(torch.cuda.get_device_properties(self.index).uuid)
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.nvml = pynvml
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ['nvidia-smi', '-i', str(self.index), f'--query-gpu={self.FIELDS}', '--format=csv,noheader,nounits',
                 '-lms', '100'], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _poll(self):
        n = self.nvml
        while not self.stop_flag:
            try:
                mhz = float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                get = getattr(n, 'nvmlDeviceGetCurrentClocksEventReasons', None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
                mask = int(get(self.handle))
                self.samples.append((time.time(), mhz, self.max_mhz, {name for name, bit in self.REASONS if mask & bit}))
            except Exception:
                pass
            time.sleep(0.004)

    def _read(self):
        for line in self.proc.stdout:
            p = [x.strip() for x in line.split(',')]
            try:
                reasons = {name for (name, _), v in zip(self.REASONS, p[3:7]) if v.lower().startswith('active')}
                self.samples.append((time.time(), float(p[0]), float(p[1]), reasons))
            except (ValueError, IndexError):
                continue

    def stop(self, t0, t1):
        if not self.proc and not self.nvml:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['no clock read-out available']}
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
        self.stop_flag = True
        rows = [r for r in self.samples if t0 <= r[0] <= t1] or self.samples[-3:]
        reasons = set()
        for r in rows:
            reasons |= r[3]
        sm = [r[1] for r in rows]
        return {'sm_mhz': statistics.median(sm) if sm else None, 'sm_max_mhz': max(r[2] for r in rows) if rows else None,
                'reasons': sorted(reasons), 'samples': len(sm), 'source': 'nvml' if self.nvml else 'nvidia-smi'}


def measured_peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        p = json.load(open(path))
        return {'bf16_sustained': p.get('bf16_tflops_sustained'), 'bf16_burst': p.get('bf16_tflops'),
                'hbm': p.get('hbm_gbs'), 'source': 'measured'}
    return {'bf16_sustained': 1400.0, 'bf16_burst': 1590.0, 'hbm': 6650.0, 'source': 'fallback'}


def cpu_baseline(net, seconds_budget=20.0):
    """The reference's CPU quantized path on the host cores, on a bounded sample of the workload."""
    from n2d2_b200 import netdesc
    from oracle import oracle, refshim
    use_ref = refshim.available()
    run = (lambda x: refshim.run_net(net, x)) if use_ref else (lambda x: oracle.run_net(net, x, 'f32'))
    cores = oracle.use_all_cores()
    x1 = netdesc.make_input(net, 1, seed=99)
    t = time.perf_counter(); run(x1); dt1 = time.perf_counter() - t
    n = int(max(1, min(64, seconds_budget / max(dt1, 1e-3) / 2)))
    x = netdesc.make_input(net, n, seed=100)
    t = time.perf_counter(); run(x); dt = time.perf_counter() - t
    line = {'value': n / dt, 'unit': UNIT, 'cores': cores, 'kind': 'reference' if use_ref else 'port',
            'sample': f'{n} images of the same network in one batch, {dt:.1f} s'
                      + (' (convolution, pooling and Scaling are the reference\'s own compiled kernels; '
                         'fc / sum / ReLU from the port)' if use_ref else '')}
    if use_ref:
        # the reference threads convolution, pooling and fc over batch x channels and runs Scaling on one thread
        # (src/Scaling_Kernels.cpp:70-88); the port threads every cell: both figures, the faithful one is `value`
        t = time.perf_counter(); oracle.run_net(net, x, 'f32'); dtp = time.perf_counter() - t
        line['fully_threaded_port'] = {'value': n / dtp, 'unit': UNIT, 'cores': cores,
                                       'sample': f'the same {n} images through the port, every cell threaded, {dtp:.1f} s'}
    return line


def launch_groups(net, engines):
    """One entry per kernel launch of a forward pass: (name, layer indices, ops per image, algorithmic bytes per
    image, weight bytes).  A sum folded into a convolution's epilogue belongs to that convolution's launch: the
    convolution's own output is never written, the residual operand is read once."""
    from n2d2_b200 import netdesc
    macs, shapes = netdesc.layer_macs(net)
    elems = {k: v[0] * v[1] * v[2] for k, v in shapes.items()}
    groups, owner = [], {}
    for i, l in enumerate(net['layers']):
        if engines[i] == 'fused' and l['type'] == 'pool':
            # a max pooling folded into the first-layer kernel: that launch writes the pooled tensor only
            conv = l['inputs'][0]
            g = groups[owner[conv]]
            g['layers'].append(i)
            g['bytes'] += elems[i] - elems[conv]
            g['name'] += '+' + l['name']
            owner[i] = owner[conv]
            continue
        if engines[i] == 'fused':
            conv = max(j for j in l['inputs'] if j >= 0 and net['layers'][j]['type'] == 'conv' and j in owner)
            g = groups[owner[conv]]
            other = [j for j in l['inputs'] if j != conv][0]
            g['layers'].append(i)
            g['bytes'] += elems[other] + elems[i] - elems[conv]
            g['name'] += '+sum'
            owner[i] = owner[conv]
            continue
        w = int(l['weights'].size) if 'weights' in l else 0
        if l.get('weight_bits', 8) == 4:
            w //= 2
        b = sum(elems[j] for j in l['inputs']) + elems[i]
        if l['type'] == 'conv':
            # a strided filter that skips pixels (1x1 stride 2) reads only the pixels it uses
            C = shapes[l['inputs'][0]][0]
            b = min(elems[l['inputs'][0]], shapes[i][1] * shapes[i][2] * l['kH'] * l['kW'] * C) + elems[i]
        owner[i] = len(groups)
        groups.append({'name': l['name'], 'layers': [i], 'ops': 2.0 * macs[i], 'bytes': float(b), 'wbytes': float(w),
                       'engine': engines[i]})
    return groups


def run_reference(args):
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    from n2d2_b200 import netdesc
    from oracle import oracle, refshim
    net = build_net(args)
    use_ref = refshim.available()
    cores = oracle.use_all_cores()
    run = (lambda x: refshim.run_net(net, x)) if use_ref else (lambda x: oracle.run_net(net, x, 'f32'))
    n = args.ref_images
    x = netdesc.make_input(net, n, seed=100)
    for _ in range(args.warmup):
        run(x[:1])
    t = time.perf_counter()
    for _ in range(args.steps):
        run(x)
    dt = time.perf_counter() - t
    value = n * args.steps / dt
    world = int(os.environ.get('WORLD_SIZE', '1'))
    line = {'impl': 'reference', 'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': args.gpus, 'steps': args.steps,
            'warmup': args.warmup, 'ms_per_step': dt / args.steps * 1e3, 'higher_is_better': True, 'scaling': args.scaling,
            'vs_baseline': None, 'dtype': 'f32 holding integers (reference CPU path)', 'data': 'synthetic',
            'config': dict(workload_config(args, net, world), sample_images_per_step=n),
            'cpu_baseline': {'value': value, 'unit': UNIT, 'cores': cores,
                             'kind': 'reference' if use_ref else 'port',
                             'sample': f'{n} images per step x {args.steps} steps'},
            'e2e': {'value': value, 'unit': UNIT, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
            'gpu_launches': 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='b200', choices=['b200', 'reference'])
    ap.add_argument('--workload', default='resnet50')
    ap.add_argument('--batch', type=int, default=1024,
                    help='images per GPU per step (weak scaling) or per step over all GPUs (strong scaling)')
    ap.add_argument('--scaling', default='weak', choices=['weak', 'strong'])
    ap.add_argument('--ref-images', type=int, default=8, help='images per step of the reference arm')
    ap.add_argument('--parity-images', type=int, default=4, help='images of the batch compared with the CPU oracle')
    ap.add_argument('--peak-probe', action='store_true', help='only measure the int8 tensor-pipe issue rate')
    ap.add_argument('--finalize-flags', type=int, default=0,
                    help='n2d2b_net_finalize flags (include/n2d2b.h), e.g. 64 = first layer and max pooling as one kernel')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--profile-out', default=None, help='write the per-cell device times here (JSON)')
    args = ap.parse_args()
    if args.impl == 'reference':
        return run_reference(args)
    if args.peak_probe:
        from n2d2_b200 import runtime
        out = {}
        for n in (64, 128, 256):
            tops, cyc = runtime.probe_i8_mma_rate(int(os.environ.get('LOCAL_RANK', '0')), n, 40000)
            out[f'n{n}'] = {'tops': tops, 'cycles_per_mma': cyc, 'mac_per_clk_per_sm': 128.0 * n * 32 / cyc}
        print(json.dumps({'probe': 'tcgen05.mma kind::i8 128 x n x 32 issued back to back on every SM', **out}))
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    from n2d2_b200 import netdesc, runtime
    from n2d2_b200.sharding import gather_outputs

    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    if world != args.gpus and world > 1:
        raise SystemExit(f'--gpus {args.gpus} but WORLD_SIZE={world}')
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group('nccl', device_id=torch.device('cuda', local_rank))

    net = build_net(args)
    B = per_gpu_batch(args, world)
    qn = runtime.QuantizedNet(net, B, device=local_rank, flags=args.finalize_flags)
    i = net['input']
    gen = torch.Generator(device='cuda').manual_seed(1000 + rank)
    d_in = torch.randint(0, 256, (B, i['H'], i['W'], i['C']), dtype=torch.uint8, device='cuda', generator=gen)
    d_out = torch.empty((B, qn.out_elems), dtype=torch.int8, device='cuda')
    h_in = torch.empty((B, i['H'], i['W'], i['C']), dtype=torch.uint8).pin_memory()
    h_in.copy_(d_in.cpu())
    h_out = [torch.empty((B, qn.out_elems), dtype=torch.int8).pin_memory() for _ in range(2)]
    stream = torch.cuda.current_stream()
    sptr = stream.cuda_stream
    flush = torch.empty(256 << 20, dtype=torch.uint8, device='cuda') if B < 256 else None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step_device():
        if flush is not None:
            flush.fill_(1)
        qn.forward_device(d_in.data_ptr(), B, d_out.data_ptr(), sptr)

    submitted = [0]

    def step_stream():
        # streaming entry point: upload of this step's images from pinned memory (copy stream, second staging
        # buffer), forward, download of its logits - all queued, nothing waited for until the end of the region
        k = submitted[0]
        submitted[0] += 1
        qn.submit_host_ptr(h_in.data_ptr(), B, h_out[k & 1].data_ptr(), sptr)

    def step_blocking():
        qn.forward_host_ptr(h_in.data_ptr(), B, h_out[0].data_ptr(), sptr)

    def timed(fn, steps, after=None):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        if after:
            after()
        barrier()
        t1 = time.time()
        ms = torch.tensor([e0.elapsed_time(e1)], device='cuda')
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()), t0, t1

    for _ in range(max(args.warmup, 3)):
        step_device()
    qn.check(sptr)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ms_total, t0, t1 = timed(step_device, args.steps)
    clocks = sampler.stop(t0, t1) if rank == 0 else None
    qn.check(sptr)      # a kernel that gave up on a bounded wait fails the run here
    if flush is not None:
        # the flush kernel runs inside the timed region; measure it alone and take it out
        fl_ms, _, _ = timed(lambda: flush.fill_(1), args.steps)
        ms_total = max(ms_total - fl_ms, 1e-6)
    ms_per_step = ms_total / args.steps
    value = B * world / (ms_per_step * 1e-3)

    # end to end through the host-buffer entry points: pinned H2D of every step's images, forward, D2H of its
    # logits, all inside the timed region.  Streaming (submit / wait): step k + 1's upload runs under step k's
    # forward pass.  Blocking (forward_host): one call per step, returns with the logits on the host.
    for _ in range(2):
        step_stream()
    qn.wait()
    e2e_ms, _, _ = timed(step_stream, args.steps, after=qn.wait)
    e2e_value = B * world / (e2e_ms / args.steps * 1e-3)
    streamed = h_out[(submitted[0] - 1) & 1].clone()
    for _ in range(2):
        step_blocking()
    blk_ms, _, _ = timed(step_blocking, args.steps)
    blk_value = B * world / (blk_ms / args.steps * 1e-3)

    # parity, outside the timed regions: the three entry points against each other on the whole batch, and a few
    # images of this rank's batch against the CPU oracle
    dev_logits = d_out.cpu()
    parity = {'host_equals_device': bool(torch.equal(h_out[0], dev_logits)),
              'streaming_equals_device': bool(torch.equal(streamed, dev_logits)), 'images': 0, 'mismatches': 0}
    if rank == 0 and args.parity_images > 0:
        from oracle import oracle
        n = min(args.parity_images, B)
        picks = sorted({0, B - 1, *(int(j * (B - 1) / max(n - 1, 1)) for j in range(n))})[:max(n, 1)]
        ref = oracle.run_net(net, h_in[picks].numpy(), 'i64')[-1].reshape(len(picks), -1)
        got = dev_logits[picks].numpy().astype(np.int64)
        parity['images'] = len(picks)
        parity['mismatches'] = int((got != ref).sum())
        parity['oracle'] = 'CPU restatement of the reference path, int64 accumulation'

    # final logits of all ranks (the one collective of the path, outside the timed region)
    logits = gather_outputs(d_out, B * world) if world > 1 else d_out
    checksum = int(logits.to(torch.int64).sum().item())

    # per-cell device times (CUDA events on the launching stream) -> roofline per launch and of the dominant kernel
    prof = np.zeros(len(net['layers']))
    reps = 3
    for _ in range(reps):
        prof += qn.profile(d_in.data_ptr(), B, d_out.data_ptr(), sptr)
    prof /= reps
    engines = qn.engines()
    macs, _ = netdesc.layer_macs(net)
    peaks = measured_peaks()
    probe_tops, probe_cyc = runtime.probe_i8_mma_rate(local_rank, 256, 40000)
    int8_peak = 2.0 * peaks['bf16_burst']
    hbm_peak = peaks['hbm']
    # the implicit-GEMM kernel and its 256-row variant (same file, same structure) count as one kernel family
    tc_ms = sum(m for m, e in zip(prof, engines) if e.startswith('tcgen05'))
    tc_ops = sum(2.0 * mc * B for mc, e in zip(macs, engines) if e.startswith('tcgen05'))
    tc_launches = sum(1 for e in engines if e.startswith('tcgen05'))
    achieved = tc_ops / (tc_ms * 1e-3) / 1e12 if tc_ms > 0 else 0.0
    # every launch against the roofline that bounds it: max(ops / int8 peak, algorithmic bytes / HBM peak)
    groups = launch_groups(net, engines)
    rows, bound_sum, meas_sum, tc_alg_bytes = [], 0.0, 0.0, 0.0
    by_kind = {}
    for g in groups:
        ms = float(sum(prof[j] for j in g['layers']))
        t_tensor = g['ops'] * B / (int8_peak * 1e12) * 1e3
        alg_bytes = g['bytes'] * B + g['wbytes']
        t_hbm = alg_bytes / (hbm_peak * 1e9) * 1e3
        bound = max(t_tensor, t_hbm)
        bound_sum += bound
        meas_sum += ms
        if g['engine'].startswith('tcgen05'):
            tc_alg_bytes += alg_bytes
        rows.append([g['name'], g['engine'], round(ms, 4), 'tensor' if t_tensor >= t_hbm else 'hbm',
                     round(bound / ms, 3) if ms > 0 else None])
        # the same per kind of launch: a residual sum folded into the epilogue is its own kind of the implicit-GEMM kernel
        kind = g['engine'] + (' + fused residual sum' if '+sum' in g['name'] else '')
        k = by_kind.setdefault(kind, [0, 0.0, 0.0])
        k[0] += 1; k[1] += ms; k[2] += bound
    roofline = {'bound': 'tensor', 'kernel': 'igemm_i8_tcgen05_kernel (with its 256-row variant igemm_pair_i8_tcgen05_kernel)',
                'achieved': achieved, 'peak': int8_peak, 'unit': 'TOP/s', 'frac': achieved / int8_peak,
                'peak_note': f"2 x {peaks['source']} burst bf16 cuBLAS TFLOP/s ({peaks['bf16_burst']}): the kind::i8 pipe "
                             'issues twice the bf16 rate and the timed region is a fraction of a second',
                'frac_of_2x_sustained_bf16': achieved / (2.0 * peaks['bf16_sustained']),
                'peak_probe': {'tops': probe_tops, 'cycles_per_mma_n256': probe_cyc, 'frac': achieved / probe_tops,
                               'what': 'tcgen05.mma kind::i8 128x256x32 issued back to back on every SM of this GPU, '
                                       'CUDA events (n2d2b_probe_i8_mma_rate)'},
                'traffic': IGEMM_DRAM_BYTES_B256_CAPTURE / IGEMM_LAUNCHES_B256_CAPTURE,
                'traffic_note': 'dram__bytes_read+write per launch of an ncu capture at batch 256 (47 launches of one '
                                'forward pass), reported at that batch; see profiles/',
                'traffic_batch': 256,
                'algorithmic_bytes_per_launch': tc_alg_bytes / max(tc_launches, 1),
                'launches_per_step': tc_launches, 'avg_launch_ms': tc_ms / max(tc_launches, 1),
                'share_of_step': tc_ms / float(prof.sum()) if prof.sum() > 0 else None,
                'per_launch': {'frac_time_weighted': bound_sum / meas_sum if meas_sum > 0 else None,
                               'what': 'sum over launches of max(ops / int8 peak, algorithmic bytes / measured HBM '
                                       f'{hbm_peak} GB/s) divided by the sum of measured launch times',
                               'rows': rows, 'columns': ['cell', 'engine', 'ms', 'bound', 'frac'],
                               'by_kind': [{'kind': kd, 'launches': v[0], 'ms': round(v[1], 4),
                                            'share_of_step': round(v[1] / meas_sum, 4) if meas_sum > 0 else None,
                                            'frac': round(v[2] / v[1], 3) if v[1] > 0 else None}
                                           for kd, v in sorted(by_kind.items(), key=lambda kv: -kv[1][1])]}}
    if args.profile_out and rank == 0:
        prows = [{'cell': l['name'], 'engine': e, 'ms': float(m), 'macs_per_image': int(mc)}
                 for l, e, m, mc in zip(net['layers'], engines, prof, macs)]
        json.dump({'batch': B, 'rows': prows}, open(args.profile_out, 'w'), indent=1)

    line = {'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': world, 'steps': args.steps,
            'warmup': max(args.warmup, 3), 'ms_per_step': ms_per_step, 'higher_is_better': True, 'scaling': args.scaling,
            'vs_baseline': None, 'dtype': 'u8/s8 operands, s32 accumulate', 'data': 'synthetic',
            'config': workload_config(args, net, world), 'clocks': clocks,
            'e2e': {'value': e2e_value, 'unit': UNIT, 'h2d_bytes_per_step': int(h_in.numel()) * world,
                    'd2h_bytes_per_step': int(h_out[0].numel()) * world,
                    'entry_point': 'n2d2b_net_submit_host / n2d2b_net_wait (streaming: the next upload runs under the '
                                   'current forward pass)',
                    'blocking_value': blk_value, 'blocking_entry_point': 'n2d2b_net_forward_host'},
            'gpu_launches': qn.launches_per_forward() * args.steps, 'roofline': roofline,
            'parity': parity, 'logits_checksum': checksum}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line['cpu_baseline'] = cpu_baseline(net)
    if rank == 0:
        print(json.dumps(line), flush=True)
    qn.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if parity['mismatches'] or not parity['host_equals_device'] or not parity['streaming_equals_device']:
        raise SystemExit(f'parity failure: {parity}')


if __name__ == '__main__':
    main()
