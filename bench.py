"""Benchmark of the GPTQ hot path: one linear layer 4096 -> 4096 (bf16), 128 x 2048 calibration
tokens, W4 asymmetric g128, act-order, percdamp 0.01 (the single-layer GPTQ configuration).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A step = Hessian accumulation over every calibration sample (add_batch is called once per
sequence, the way the algorithm's forward hook delivers them; the plugin hands 8 sequences to
one lc_hessian_accum_multi launch) + the GPTQ layer solve.  Inputs are
seeded synthetic tensors with the configuration's shapes and value distributions.

N > 1 (launched by torch.distributed.run): calibration sequences are sharded over the ranks,
the raw Hessian is all-reduced once (NCCL), the rows of the layer are split over the ranks for
the solve and all-gathered.  Total work is fixed: strong scaling.

`--impl reference` times the CPU restatement of the reference (oracle/) on the host cores, on a
bounded sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

R, C, NS, T = 4096, 4096, 128, 2048
METRIC = 'GPTQ W4 g128 layers/sec'
UNIT = 'layers/s'
WORKLOAD = ('GPTQ single linear 4096x4096 bf16, calibration 128x2048x4096 N(0,1) with 1% outlier channels x20, '
            'W4 asym g128, blocksize 128, percdamp 0.01, act_order')


def peaks():
    p = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(p):
        d = json.load(open(p))
        return d['hbm_gbs'], d['bf16_tflops'], d['bf16_tflops_sustained'], 'measured'
    return 6650.0, 1590.0, 1400.0, 'fallback'


def make_inputs(n_seq, seed_offset=0, pin=False):
    import torch
    g = torch.Generator().manual_seed(2000)
    W = (torch.randn(R, C, generator=g) * 0.02).to(torch.bfloat16)
    ch = torch.randperm(C, generator=g)[:C // 100]
    gx = torch.Generator().manual_seed(2001 + seed_offset)
    X = torch.empty((n_seq, T, C), dtype=torch.bfloat16, pin_memory=pin)
    for i in range(n_seq):
        x = torch.randn(T, C, generator=gx)
        x[:, ch] *= 20
        X[i] = x.to(torch.bfloat16)
    if pin:
        W = W.pin_memory()
    return W, X


class ClockSampler:
    QUERY = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,'
             'clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
             'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, gpu_index):
        self.f = tempfile.NamedTemporaryFile('w+', suffix='.csv', delete=False)
        try:
            self.p = subprocess.Popen(['nvidia-smi', '-i', str(gpu_index), f'--query-gpu={self.QUERY}',
                                       '--format=csv,noheader,nounits', '-lms', '100'],
                                      stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self):
        if self.p is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        rows = [ln.split(',') for ln in open(self.f.name).read().strip().splitlines() if ln.count(',') >= 8]
        os.unlink(self.f.name)
        sm, mx, power, reasons = [], [], [], set()
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        for r in rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                power.append(float(r[3]))
            except ValueError:
                continue
            for n, v in zip(names, r[5:9]):
                if v.strip().lower().startswith('active'):
                    reasons.add(n)
        if not sm:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['no samples']}
        # median over the busier half of the samples (the sampler also sees idle gaps)
        busy = sorted(s for s, p in zip(sm, power) if p >= 0.5 * max(power)) or sorted(sm)
        return {'sm_mhz': busy[len(busy) // 2], 'sm_max_mhz': max(mx), 'power_w_max': max(power),
                'samples': len(sm), 'reasons': sorted(reasons)}


HESSIAN_BATCH = 8   # sequences handed to one Hessian launch (GPTQ special key `hessian_batch`)


def launches_per_step(n_seq):
    n_blocks = C // 128
    # hessian per batch of sequences + diag + (damp, permute H, permute W) + flip + block + trailing + un-permute
    return -(-n_seq // HESSIAN_BATCH) + 1 + 3 + 1 + n_blocks + (n_blocks - 1) + 1


def cpu_port(n_hess_samples=8, threads=None):
    """Times the oracle port on a bounded sample; returns (layers/s extrapolated, description, cores)."""
    import torch
    from oracle import gptq_ref
    cores = threads or os.cpu_count()
    torch.set_num_threads(cores)
    W, X = make_inputs(n_hess_samples)
    st = gptq_ref.hessian_init(C)
    t0 = time.perf_counter()
    for i in range(n_hess_samples):
        gptq_ref.add_batch(st, X[i:i + 1])
    t_h = (time.perf_counter() - t0) / n_hess_samples * NS
    # a well-conditioned stand-in for the full-data Hessian: the solver's cost does not depend on values
    t0 = time.perf_counter()
    gptq_ref.quantize_layer(W, st['H'] + 1e-3 * torch.eye(C) * float(st['H'].diagonal().mean()))
    t_s = time.perf_counter() - t0
    desc = (f'Hessian: {n_hess_samples} of {NS} samples timed and scaled x{NS // n_hess_samples}; '
            f'prepare + weight_transform: full 4096x4096 layer')
    return 1.0 / (t_h + t_s), desc, cores, t_h, t_s


def run_reference(args, rank):
    if rank != 0:
        return
    vals = []
    desc = cores = None
    for i in range(args.warmup + args.steps):
        v, desc, cores, t_h, t_s = cpu_port(4 if args.steps + args.warmup > 2 else 8)
        if i >= args.warmup:
            vals.append(v)
    v = sum(vals) / len(vals)
    line = {'impl': 'reference', 'metric': METRIC, 'value': v, 'unit': UNIT, 'n_gpus': args.gpus,
            'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': 1e3 / v, 'higher_is_better': True,
            'scaling': 'strong', 'vs_baseline': None, 'dtype': 'bf16 in / fp32 accumulate', 'data': 'synthetic',
            'config': {'workload': WORKLOAD},
            'cpu_baseline': {'value': v, 'unit': UNIT, 'cores': cores, 'kind': 'port', 'sample': desc},
            'e2e': {'value': v, 'unit': UNIT, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
            'gpu_launches': 0}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=5)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='b200', choices=['b200', 'reference'])
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-e2e', action='store_true')
    args = ap.parse_args()
    rank = int(os.environ.get('RANK', 0))
    local_rank = int(os.environ.get('LOCAL_RANK', 0))
    world = int(os.environ.get('WORLD_SIZE', 1))
    if args.impl == 'reference':
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    import lightcompress_b200 as lc
    from lightcompress_b200 import _lib as L

    torch.cuda.set_device(local_rank)
    dev = torch.device('cuda', local_rank)
    if world > 1:
        dist.init_process_group('nccl', device_id=dev)
    assert world == args.gpus, f'--gpus {args.gpus} but WORLD_SIZE={world}'
    assert NS % world == 0 and R % world == 0
    n_seq = NS // world
    hbm_peak, tf_burst, tf_sust, peak_kind = peaks()

    W_host, X_host = make_inputs(n_seq, seed_offset=rank, pin=not args.no_e2e)
    W = W_host.to(dev)
    X = X_host.to(dev)
    wq = lc.IntegerQuantizer(4, False, 'per_group', group_size=128)
    solver = lc.GPTQ(wq, {'actorder': True, 'percdamp': 0.01, 'blocksize': 128, 'emit_codes': True,
                          'hessian_batch': HESSIAN_BATCH})
    layer = torch.nn.Linear(C, R, bias=False, dtype=torch.bfloat16, device=dev)
    from lightcompress_b200 import parallel
    r0, r1 = parallel.row_shard(R)
    hess_ev = []

    def step(x_dev, record=False):
        layer.weight.data = W
        solver.layer_init(layer, 'l')
        if record:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        for i in range(n_seq):
            solver.add_batch(layer, 'l', x_dev[i:i + 1])
        if record:
            e1.record()
            hess_ev.append((e0, e1))
        if world == 1:
            res = solver.layer_transform(layer, 'l')
            out = res['weight']
        else:
            res = solver.layer_transform(layer, 'l', rows=(r0, r1))
            out = parallel.gather_rows(res['weight'], R)
        solver.free('l')
        return out, res

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps):
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        sync_all()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # ---- device-resident throughput ------------------------------------------------------------
    for _ in range(args.warmup):
        step(X)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    ms_total = timed(lambda: step(X, record=True), args.steps)
    ms_step = ms_total / args.steps
    value = 1e3 / ms_step
    hess_ms = sum(a.elapsed_time(b) for a, b in hess_ev) / len(hess_ev)
    n_hess_launches = -(-n_seq // HESSIAN_BATCH)
    hess_launch_ms = hess_ms / n_hess_launches
    tok_per_launch = T * n_seq / n_hess_launches

    # ---- end to end: host buffers in, host result out ------------------------------------------
    e2e = None
    if not args.no_e2e:
        copy_stream = torch.cuda.Stream(device=dev)
        x_stage = torch.empty_like(X)
        out_host = torch.empty((R // world, C), dtype=torch.float32).pin_memory()
        sc_host = torch.empty((R // world * (C // 128), 1), dtype=torch.float32).pin_memory()
        zr_host = torch.empty_like(sc_host).pin_memory()
        chunk = 8

        def e2e_step():
            main = torch.cuda.current_stream()
            copy_stream.wait_stream(main)       # previous step's readers of x_stage are done
            layer.weight.data = W_host.to(dev, non_blocking=True)
            solver.layer_init(layer, 'l')
            evs = []
            with torch.cuda.stream(copy_stream):
                for i in range(0, n_seq, chunk):
                    x_stage[i:i + chunk].copy_(X_host[i:i + chunk], non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(copy_stream)
                    evs.append(ev)
            for k, i in enumerate(range(0, n_seq, chunk)):
                main.wait_event(evs[k])
                for j in range(i, min(i + chunk, n_seq)):
                    solver.add_batch(layer, 'l', x_stage[j:j + 1])
            res = solver.layer_transform(layer, 'l', rows=None if world == 1 else (r0, r1))
            out_host.copy_(res['weight'], non_blocking=True)
            sc_host.copy_(res['buf_scales'], non_blocking=True)
            zr_host.copy_(res['buf_zeros'], non_blocking=True)
            solver.free('l')

        for _ in range(2):
            e2e_step()
        e2e_ms = timed(e2e_step, args.steps) / args.steps
        e2e = {'value': 1e3 / e2e_ms, 'unit': UNIT, 'ms_per_step': e2e_ms,
               'h2d_bytes_per_step': int(X_host.numel() * 2 + W_host.numel() * 2),
               'd2h_bytes_per_step': int(out_host.numel() * 4 + sc_host.numel() * 8)}
    clocks = sampler.stop() if sampler else None

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel (Hessian GEMM) ------------------------------------------
    alg_flops = 2.0 * tok_per_launch * C * C          # per launch: the full square the reference computes
    n_super = (C // 256) * (C // 256 + 1) // 2
    exe_flops = 2.0 * tok_per_launch * 256 * 256 * n_super   # 256x256 tiles actually issued (upper triangle)
    achieved = alg_flops / (hess_launch_ms * 1e-3) / 1e12
    peak = tf_sust
    roofline = {'bound': 'tensor', 'kernel': 'hessian_umma_kernel', 'achieved': achieved, 'peak': peak,
                'unit': 'TFLOP/s', 'frac': achieved / peak, 'peak_kind': f'{peak_kind} sustained cuBLAS bf16',
                'achieved_executed': exe_flops / (hess_launch_ms * 1e-3) / 1e12,
                'launch_ms': hess_launch_ms, 'launches_per_step': n_hess_launches,
                'tokens_per_launch': tok_per_launch, 'share_of_step': hess_ms / ms_step,
                'traffic': None}

    line = {'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': world, 'steps': args.steps,
            'warmup': args.warmup, 'ms_per_step': ms_step, 'higher_is_better': True, 'scaling': 'strong',
            'vs_baseline': None, 'dtype': 'bf16 in / fp32 accumulate', 'data': 'synthetic',
            'config': {'workload': WORKLOAD, 'l2': 'inputs (2.1 GB of activations per step) exceed the 126 MB L2',
                       'sharding': f'{n_seq} sequences and {R // world} rows per rank'},
            'roofline': roofline, 'gpu_launches': launches_per_step(n_seq) * args.steps, 'clocks': clocks}
    if e2e:
        line['e2e'] = e2e
    if not args.no_cpu_baseline and world == 1:
        v, desc, cores, t_h, t_s = cpu_port(8)
        line['cpu_baseline'] = {'value': v, 'unit': UNIT, 'cores': cores, 'kind': 'port', 'sample': desc,
                                'hessian_s': t_h, 'solver_s': t_s}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
