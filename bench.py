#!/usr/bin/env python
"""Benchmark of the quantized integer inference path: int8 ResNet-50 images/s.

    python bench.py --gpus N --steps K --warmup W          (N > 1: launched under torchrun)
    python bench.py --impl reference ...                   (the reference's CPU path, host cores)

One step = one forward pass of the quantized network over one batch of synthetic uint8 images.
Work is batch-sharded: every rank owns `--batch` images per step (weak scaling, no collective on the
data path; the final int8 logits are all-gathered once, outside the timed region).  Timing is CUDA
events on the launching stream, max over ranks, barrier + synchronize on both sides.
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

# DRAM bytes one launch of the implicit-GEMM kernel moves per image (average over the 53 launches of a
# ResNet-50 forward): 4950.6 MB / 53 launches / 256 images, from the ncu capture summarised under profiles/.
IGEMM_DRAM_BYTES_PER_IMAGE_PER_LAUNCH = 4668.37e6 / 47 / 256

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
    return {'workload': names[args.workload], 'batch_per_gpu': args.batch, 'global_batch': args.batch * world,
            'parallelism': f'batch-sharded x{world}, no collective on the data path',
            'cache': 'inputs and activations larger than L2 (no flush needed)' if args.batch >= 256
                     else 'L2 flushed between steps'}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ('clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,'
              'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,'
              'clocks_event_reasons.sw_power_cap')

    def __init__(self, index):
        self.index = index
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ['nvidia-smi', '-i', str(self.index), f'--query-gpu={self.FIELDS}', '--format=csv,noheader,nounits',
                 '-lms', '100'], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if not self.proc:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [l for (t, l) in self.samples if t0 <= t <= t1 + 0.1] or [l for (_, l) in self.samples[-3:]]
        sm, mx, reasons = [], [], set()
        for l in rows:
            p = [x.strip() for x in l.split(',')]
            try:
                sm.append(float(p[0])); mx.append(float(p[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap'), p[3:7]):
                if v.lower().startswith('active'):
                    reasons.add(name)
        return {'sm_mhz': statistics.median(sm) if sm else None, 'sm_max_mhz': max(mx) if mx else None,
                'reasons': sorted(reasons), 'samples': len(sm)}


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
    return {'value': n / dt, 'unit': UNIT, 'cores': cores, 'kind': 'reference' if use_ref else 'port',
            'sample': f'{n} images of the same network in one batch, {dt:.1f} s'
                      + (' (convolution, pooling and Scaling are the reference\'s own compiled kernels; '
                         'fc / sum / ReLU from the port)' if use_ref else '')}


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
            'warmup': args.warmup, 'ms_per_step': dt / args.steps * 1e3, 'higher_is_better': True, 'scaling': 'weak',
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
    ap.add_argument('--batch', type=int, default=1024, help='images per GPU per step')
    ap.add_argument('--ref-images', type=int, default=2, help='images per step of the reference arm')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--profile-out', default=None, help='write the per-cell device times here (JSON)')
    args = ap.parse_args()
    if args.impl == 'reference':
        return run_reference(args)

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
    B = args.batch
    qn = runtime.QuantizedNet(net, B, device=local_rank)
    i = net['input']
    gen = torch.Generator(device='cuda').manual_seed(1000 + rank)
    d_in = torch.randint(0, 256, (B, i['H'], i['W'], i['C']), dtype=torch.uint8, device='cuda', generator=gen)
    d_out = torch.empty((B, qn.out_elems), dtype=torch.int8, device='cuda')
    h_in = torch.empty((B, i['H'], i['W'], i['C']), dtype=torch.uint8).pin_memory()
    h_in.copy_(d_in.cpu())
    h_out = torch.empty((B, qn.out_elems), dtype=torch.int8).pin_memory()
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

    def step_host():
        qn.forward_host_ptr(h_in.data_ptr(), B, h_out.data_ptr(), sptr)

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        barrier()
        t1 = time.time()
        ms = torch.tensor([e0.elapsed_time(e1)], device='cuda')
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()), t0, t1

    for _ in range(max(args.warmup, 3)):
        step_device()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ms_total, t0, t1 = timed(step_device, args.steps)
    clocks = sampler.stop(t0, t1) if rank == 0 else None
    if flush is not None:
        # the flush kernel runs inside the timed region; measure it alone and take it out
        fl_ms, _, _ = timed(lambda: flush.fill_(1), args.steps)
        ms_total = max(ms_total - fl_ms, 1e-6)
    ms_per_step = ms_total / args.steps
    value = B * world / (ms_per_step * 1e-3)

    # end to end through the host-buffer entry point: pinned H2D of the step's images, forward, D2H of the logits
    for _ in range(2):
        step_host()
    e2e_ms, _, _ = timed(step_host, args.steps)
    e2e_value = B * world / (e2e_ms / args.steps * 1e-3)

    # final logits of all ranks (the one collective of the path, outside the timed region)
    logits = gather_outputs(d_out, B * world) if world > 1 else d_out
    checksum = int(logits.to(torch.int64).sum().item())

    # per-cell device times (CUDA events on the launching stream) -> roofline of the dominant kernel
    prof = np.zeros(len(net['layers']))
    reps = 3
    for _ in range(reps):
        prof += qn.profile(d_in.data_ptr(), B, d_out.data_ptr(), sptr)
    prof /= reps
    engines = qn.engines()
    macs, _ = netdesc.layer_macs(net)
    # the implicit-GEMM kernel and its 256-row variant (same file, same structure) count as one kernel family
    tc_ms = sum(m for m, e in zip(prof, engines) if e.startswith('tcgen05'))
    tc_ops = sum(2.0 * mc * B for mc, e in zip(macs, engines) if e.startswith('tcgen05'))
    tc_launches = sum(1 for e in engines if e.startswith('tcgen05'))
    peaks = measured_peaks()
    int8_peak = 2.0 * peaks['bf16_sustained']
    achieved = tc_ops / (tc_ms * 1e-3) / 1e12 if tc_ms > 0 else 0.0
    roofline = {'bound': 'tensor', 'kernel': 'igemm_i8_tcgen05_kernel (with its 256-row variant igemm_pair_i8_tcgen05_kernel)', 'achieved': achieved, 'peak': int8_peak,
                'unit': 'TOP/s', 'frac': achieved / int8_peak, 'traffic': IGEMM_DRAM_BYTES_PER_IMAGE_PER_LAUNCH * B,
                'traffic_note': 'dram__bytes_read+write per launch, averaged over the 47 launches of one forward; '
                                'captured with ncu at batch 256 and scaled by batch (traffic grows in proportion); '
                                'see profiles/igemm_i8_tcgen05_resnet50_b256_dram_per_launch.md',
                'launches_per_step': tc_launches, 'avg_launch_ms': tc_ms / max(tc_launches, 1),
                'share_of_step': tc_ms / float(prof.sum()) if prof.sum() > 0 else None,
                'peak_note': f"2 x {peaks['source']} sustained bf16 cuBLAS TFLOP/s ({peaks['bf16_sustained']}): "
                             'the kind::i8 pipe issues twice the bf16 rate; no int8 figure is measured on this pool'}
    if args.profile_out and rank == 0:
        rows = [{'cell': l['name'], 'engine': e, 'ms': float(m), 'macs_per_image': int(mc)}
                for l, e, m, mc in zip(net['layers'], engines, prof, macs)]
        json.dump({'batch': B, 'rows': rows}, open(args.profile_out, 'w'), indent=1)

    line = {'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': world, 'steps': args.steps,
            'warmup': max(args.warmup, 3), 'ms_per_step': ms_per_step, 'higher_is_better': True, 'scaling': 'weak',
            'vs_baseline': None, 'dtype': 'u8/s8 operands, s32 accumulate', 'data': 'synthetic',
            'config': workload_config(args, net, world), 'clocks': clocks,
            'e2e': {'value': e2e_value, 'unit': UNIT, 'h2d_bytes_per_step': int(h_in.numel()) * world,
                    'd2h_bytes_per_step': int(h_out.numel()) * world},
            'gpu_launches': qn.launches_per_forward() * args.steps, 'roofline': roofline,
            'logits_checksum': checksum}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line['cpu_baseline'] = cpu_baseline(net)
    if rank == 0:
        print(json.dumps(line), flush=True)
    qn.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
