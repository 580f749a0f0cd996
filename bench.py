"""Benchmark of the GPTQ calibration hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload block|layer]

Default workload `block` (the end-to-end GPTQ configuration's unit of work): ONE Llama-2-7B-shape
decoder layer (hidden 4096, 32 heads, MLP 11008, bf16, weights N(0, 0.02^2)) quantised with GPTQ
W4A16 asymmetric g128, act-order, percdamp 0.01, true_sequential, quant_out, on 128 x 2048 tokens
of synthetic hidden states (N(0,1), 1 % outlier channels x20).  A step = the reference's
per-block schedule (5 forwards of the block over all sequences, 4 distinct Hessians, 7 layer
solves); value = decoder layers per second.

Workload `layer` (the single-linear GPTQ configuration): one 4096 -> 4096 linear, 128 x 2048 x 4096
calibration activations; a step = Hessian accumulation over all sequences + the layer solve.

N > 1 (launched by torch.distributed.run): calibration sequences are sharded over the ranks, each
Hessian is all-reduced once (NCCL), the (linear, row-range) solve units are dealt to the ranks.
Total work is fixed: strong scaling.

`--impl reference` times the CPU restatement of the reference (oracle/) on the host cores, on a
bounded sample of the same workload.
"""
import argparse
import copy
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

NS, T, HID, INTER, HEADS = 128, 2048, 4096, 11008, 32
METRIC = 'GPTQ W4 g128 decoder layers/sec'
UNIT = 'layers/s'
HESSIAN_BATCH = 8   # sequences handed to one Hessian launch (GPTQ special key `hessian_batch`)
SPECIAL = {'actorder': True, 'percdamp': 0.01, 'blocksize': 128, 'true_sequential': True,
           'static_groups': False, 'hessian_batch': HESSIAN_BATCH, 'emit_codes': True}
WORKLOADS = {
    'block': ('one Llama-2-7B-shape decoder layer (hidden 4096, 32 heads, MLP 11008, bf16 N(0,0.02^2)), GPTQ W4A16 '
              'asym g128, act_order, percdamp 0.01, true_sequential, quant_out; calibration 128x2048 tokens of '
              'hidden states N(0,1) with 1% outlier channels x20'),
    'layer': ('GPTQ single linear 4096x4096 bf16 N(0,0.02^2), calibration 128x2048x4096 N(0,1) with 1% outlier '
              'channels x20, W4 asym g128, blocksize 128, percdamp 0.01, act_order'),
}


def peaks():
    p = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(p):
        d = json.load(open(p))
        return d['hbm_gbs'], d['bf16_tflops'], d['bf16_tflops_sustained'], 'measured'
    return 6650.0, 1590.0, 1400.0, 'fallback'


# ---- synthetic inputs --------------------------------------------------------------------------
def make_activations(n_seq, seed, pin=False):
    """(n_seq, T, HID) bf16, N(0,1) with 1 % of the channels scaled x20 (same channels on every rank)."""
    import torch
    g = torch.Generator().manual_seed(2000)
    ch = torch.randperm(HID, generator=g)[:HID // 100]
    gx = torch.Generator().manual_seed(seed)
    X = torch.empty((n_seq, T, HID), dtype=torch.bfloat16, pin_memory=pin)
    for i in range(n_seq):
        x = torch.randn(T, HID, generator=gx)
        x[:, ch] *= 20
        X[i] = x.to(torch.bfloat16)
    return X


def make_linear_weight():
    import torch
    g = torch.Generator().manual_seed(2000)
    return (torch.randn(HID, HID, generator=g) * 0.02).to(torch.bfloat16)


def make_block(seq_len=T):
    """Random-init Llama decoder layer of the 7B shape from the installed transformers + forward kwargs."""
    import torch
    from transformers import LlamaConfig
    from transformers.models.llama.modeling_llama import LlamaDecoderLayer, LlamaRotaryEmbedding
    cfg = LlamaConfig(hidden_size=HID, intermediate_size=INTER, num_attention_heads=HEADS,
                      num_key_value_heads=HEADS, num_hidden_layers=1, vocab_size=32000,
                      max_position_embeddings=4096, rms_norm_eps=1e-5)
    cfg._attn_implementation = 'sdpa'
    g = torch.Generator().manual_seed(4000)
    block = LlamaDecoderLayer(cfg, 0).to(torch.bfloat16)
    for p in block.parameters():
        if p.dim() == 2:
            p.data = (torch.randn(p.shape, generator=g) * 0.02).to(torch.bfloat16)
    rot = LlamaRotaryEmbedding(cfg)
    pos = torch.arange(seq_len)[None]
    cos, sin = rot(torch.zeros(1, seq_len, HID, dtype=torch.bfloat16), pos)
    return block, {'position_embeddings': (cos, sin), 'attention_mask': None, 'position_ids': pos}


def kwargs_to(kwargs, dev):
    import torch
    out = {}
    for k, v in kwargs.items():
        if torch.is_tensor(v):
            out[k] = v.to(dev)
        elif isinstance(v, tuple):
            out[k] = tuple(t.to(dev) for t in v)
        else:
            out[k] = v
    return out


LINEAR_KEYS = ['q', 'k', 'v', 'o', 'gate', 'up', 'down']
LINEAR_SHAPES = [(HID, HID)] * 4 + [(INTER, HID)] * 2 + [(HID, INTER)]   # (rows, cols) of q,k,v,o,gate,up,down


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
        # median over the samples taken under load (the sampler also sees idle gaps between phases)
        busy = sorted(s for s, p in zip(sm, power) if p >= 0.5 * max(power)) or sorted(sm)
        return {'sm_mhz': busy[len(busy) // 2], 'sm_max_mhz': max(mx), 'power_w_max': max(power),
                'samples': len(sm), 'reasons': sorted(reasons)}


# ---- CPU port (oracle) on a bounded sample --------------------------------------------------------
def cpu_port_layer(n_hess_samples=8):
    import torch
    from oracle import gptq_ref
    cores = os.cpu_count()
    torch.set_num_threads(cores)
    W = make_linear_weight()
    X = make_activations(n_hess_samples, 2001)
    st = gptq_ref.hessian_init(HID)
    t0 = time.perf_counter()
    for i in range(n_hess_samples):
        gptq_ref.add_batch(st, X[i:i + 1])
    t_h = (time.perf_counter() - t0) / n_hess_samples * NS
    t0 = time.perf_counter()
    gptq_ref.quantize_layer(W, st['H'] + 1e-3 * torch.eye(HID) * float(st['H'].diagonal().mean()))
    t_s = time.perf_counter() - t0
    desc = (f'Hessian: {n_hess_samples} of {NS} sequences timed and scaled x{NS // n_hess_samples}; '
            f'prepare + weight_transform: the full 4096x4096 layer')
    return 1.0 / (t_h + t_s), desc, cores, {'hessian_s': t_h, 'solver_s': t_s}


def cpu_port_block():
    """One sequence through the reference schedule's five forwards with its Hessian hooks (scaled
    x128), plus the solver: prepare and weight_transform timed on a 4096x4096 linear and scaled to
    the seven linears by C^3 and rows*cols respectively."""
    import torch
    from oracle import gptq_block_ref, gptq_ref
    cores = os.cpu_count()
    torch.set_num_threads(cores)
    block, kwargs = make_block()
    x = make_activations(1, 2001)
    subsets = gptq_block_ref.llama_subsets(block)
    t0 = time.perf_counter()
    with torch.no_grad():
        for p in range(5):
            # pass 0 hooks all seven linears, passes 1-3 the next subset, pass 4 (quant_out) none
            items = [it for s in subsets for it in s] if p == 0 else (subsets[p] if p < 4 else [])
            states, hs = {}, []
            for name, parent, attr in items:
                layer = getattr(parent, attr)
                states[name] = gptq_ref.hessian_init(layer.weight.shape[1])

                def hook(m, inp, out, name=name, states=states):
                    gptq_ref.add_batch(states[name], inp[0].data)
                hs.append(layer.register_forward_hook(hook))
            block(x[0:1], **kwargs)
            for h in hs:
                h.remove()
    t_fwd = (time.perf_counter() - t0) * NS
    W = make_linear_weight()
    g = torch.Generator().manual_seed(1)
    Xs = torch.randn(8192, HID, generator=g)
    H = (Xs.t() @ Xs) * (2.0 / 4)
    t0 = time.perf_counter()
    Wp, U, perm, invperm = gptq_ref.prepare(W, H)
    t_prep = time.perf_counter() - t0
    t0 = time.perf_counter()
    gptq_ref.weight_transform(Wp, U)
    t_wt = time.perf_counter() - t0
    t_solver = sum(t_prep * (c / HID) ** 3 + t_wt * (r * c) / (HID * HID) for r, c in LINEAR_SHAPES)
    desc = (f'forwards + Hessian hooks: 1 of {NS} sequences through the 5 passes, scaled x{NS}; solver: prepare and '
            f'weight_transform timed on one 4096x4096 linear, scaled to the 7 linears by C^3 and rows*cols')
    return 1.0 / (t_fwd + t_solver), desc, cores, {'forward_hessian_s': t_fwd, 'solver_s': t_solver}


def run_reference(args, rank):
    if rank != 0:
        return
    fn = cpu_port_block if args.workload == 'block' else (lambda: cpu_port_layer(4))
    vals, desc, cores = [], None, None
    for i in range(args.warmup + args.steps):
        v, desc, cores, _ = fn()
        if i >= args.warmup:
            vals.append(v)
    v = sum(vals) / len(vals)
    print(json.dumps({
        'impl': 'reference', 'metric': METRIC, 'value': v, 'unit': UNIT, 'n_gpus': args.gpus, 'steps': args.steps,
        'warmup': args.warmup, 'ms_per_step': 1e3 / v, 'higher_is_better': True, 'scaling': 'strong',
        'vs_baseline': None, 'dtype': 'bf16 in / fp32 accumulate', 'data': 'synthetic',
        'config': {'workload': WORKLOADS[args.workload], 'name': args.workload},
        'cpu_baseline': {'value': v, 'unit': UNIT, 'cores': cores, 'kind': 'port', 'sample': desc},
        'e2e': {'value': v, 'unit': UNIT, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0}, 'gpu_launches': 0}))


# ---- GPU workloads ---------------------------------------------------------------------------------
class HessianTimer:
    """Brackets every Hessian launch with CUDA events on the launching stream."""

    def __init__(self, solver):
        self.pairs = []
        self.on = False
        orig = solver._flush

        def flush(st):
            if not self.on or not st['pending']:
                return orig(st)
            import torch
            cols = st['pending'][0].shape[1]
            toks = sum(x.shape[0] for x in st['pending'])
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            orig(st)
            e1.record()
            self.pairs.append((cols, toks, e0, e1))
        solver._flush = flush

    def summary(self):
        by_c = {}
        for cols, toks, e0, e1 in self.pairs:
            d = by_c.setdefault(cols, [0, 0.0, 0])
            d[0] += 1
            d[1] += e0.elapsed_time(e1)
            d[2] += toks
        return by_c


def rtn_aux(hbm_peak, dev):
    """quant_dequant GB/s of the RTN kernel on the configuration of the reference's CPU-runnable case
    (fp32 4096x4096, W4 asymmetric, groups of 128) and on a tensor far larger than L2; raw C-ABI calls,
    8 rotating buffers so that no launch finds its input in L2, CUDA events around 40 launches."""
    import torch
    from lightcompress_b200 import _lib as L
    out = {}
    for name, rows, cols, dt in (('rtn_w4_g128_fp32_4096x4096', 4096, 4096, torch.float32),
                                 ('rtn_w4_g128_fp32_16384x8192', 16384, 8192, torch.float32),
                                 ('rtn_w4_g128_bf16_16384x8192', 16384, 8192, torch.bfloat16)):
        n_buf = 8 if rows == 4096 else 2
        g = torch.Generator().manual_seed(1001)
        ws = [(torch.randn(rows, cols, generator=g) * 0.02).to(dt).to(dev) for _ in range(n_buf)]
        outs = [torch.empty_like(w) for w in ws]
        st = L.stream_of(ws[0])

        def run(i):
            L.call('lc_rtn_int_quant', L.ptr(ws[i % n_buf]), L.lc_dtype(ws[0]), rows, cols, 128, 4, 0, None, None,
                   L.ptr(outs[i % n_buf]), None, L.LC_CODES_NONE, None, None, st)
        for i in range(8):
            run(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(40):
            run(i)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) / 40 * 1e3
        nbytes = 2 * rows * cols * ws[0].element_size()
        gbs = nbytes / us / 1e3
        out[name] = {'us': us, 'algorithmic_bytes': nbytes, 'gb_s': gbs, 'frac_of_measured_hbm': gbs / hbm_peak}
        del ws, outs
    return out


def run_secondary(args):
    """`--workload awq`: AWQ scale + clip search of one Llama-2-7B-shape block on 128 x 512 calibration
    tokens in one batch (W4 asym g128, trans_version v2, clip_version v1).  `--workload moe`: FP8 e4m3
    fake quant of a 64-expert MoE layer (per-channel weights once, per-token activations per forward).
    Device-resident inputs, CUDA events, one JSON line with the configuration's own metric."""
    import torch
    import lightcompress_b200 as lc
    dev = torch.device('cuda', 0)
    torch.cuda.set_device(dev)
    hbm_peak = peaks()[0]
    if args.workload == 'awq':
        from lightcompress_b200.awq import Awq
        block_host, kwargs_host = make_block(seq_len=512)
        kwargs = kwargs_to(kwargs_host, dev)
        g = torch.Generator().manual_seed(3001)
        X = torch.randn(NS, 512, HID, generator=g)
        X[:, :, torch.randperm(HID, generator=g)[:41]] *= 20
        X = X.to(torch.bfloat16).to(dev)
        master = copy.deepcopy(block_host).to(dev)
        wq = lc.IntegerQuantizer(4, False, 'per_group', group_size=128)
        awq = Awq(wq, {'trans': True, 'trans_version': 'v2', 'weight_clip': True, 'clip_version': 'v1'},
                  calib_seq_len=512)

        def step():
            return awq.block_transform(copy.deepcopy(master), X, kwargs)
        metric, unit = 'AWQ W4 g128 scale+clip search blocks/sec', 'blocks/s'
        workload = ('one Llama-2-7B-shape decoder block, AWQ W4 asym g128, 20-point scale grid on 4 subsets + clip '
                    'search on 5 linears, 128x512 calibration tokens in one batch')
    else:
        from lightcompress_b200.moe_fp8 import Fp8FakeQuantMoE
        g = torch.Generator().manual_seed(5001)
        x = torch.randn(16384, 2048, generator=g).to(torch.bfloat16).to(dev)
        moe = Fp8FakeQuantMoE(device=dev)
        pristine = [t.clone() for t in (moe.w_gate, moe.w_up, moe.w_down, moe.s_gate, moe.s_up, moe.s_down)]

        def step():
            moe.w_gate, moe.w_up, moe.w_down, moe.s_gate, moe.s_up, moe.s_down = pristine
            moe.quantize_weights()
            return moe.forward(x)
        metric, unit = 'FP8 e4m3 fake-quant MoE layer passes/sec (weights quantised + one forward)', 'passes/s'
        workload = ('64 routed experts (1408 x 2048) + shared MLP, top-6, 16384 tokens, e4m3 per-channel weights, '
                    'per-token dynamic activations')
    for _ in range(max(1, args.warmup)):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    print(json.dumps({'metric': metric, 'value': 1e3 / ms, 'unit': unit, 'n_gpus': 1, 'steps': args.steps,
                      'warmup': args.warmup, 'ms_per_step': ms, 'higher_is_better': True, 'scaling': 'weak',
                      'vs_baseline': None, 'dtype': 'bf16', 'data': 'synthetic',
                      'config': {'workload': workload, 'name': args.workload}, 'hbm_peak_gbs': hbm_peak}))


def n_super(c):
    s = -(-c // 256)
    return s * (s + 1) // 2


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=3)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='b200', choices=['b200', 'reference'])
    ap.add_argument('--workload', default='block', choices=['block', 'layer', 'awq', 'moe'])
    ap.add_argument('--calib-bs', type=int, default=1,
                    help='sequences per block-forward call (calib.bs of the reference config; block workload)')
    ap.add_argument('--static-groups', action='store_true',
                    help='special.static_groups of the reference (its export configs); a side measurement')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-e2e', action='store_true')
    args = ap.parse_args()
    if args.static_groups:
        SPECIAL['static_groups'] = True
    rank = int(os.environ.get('RANK', 0))
    local_rank = int(os.environ.get('LOCAL_RANK', 0))
    world = int(os.environ.get('WORLD_SIZE', 1))
    if args.workload in ('awq', 'moe'):
        # secondary configurations (AWQ block search, FP8 MoE fake quant): one GPU, their own metric
        if rank == 0:
            run_secondary(args)
        return
    if args.impl == 'reference':
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    import lightcompress_b200 as lc
    from lightcompress_b200 import parallel

    torch.cuda.set_device(local_rank)
    dev = torch.device('cuda', local_rank)
    if world > 1:
        dist.init_process_group('nccl', device_id=dev)
    assert world == args.gpus, f'--gpus {args.gpus} but WORLD_SIZE={world}'
    s0, s1 = parallel.sequence_shard(NS)
    n_seq = s1 - s0
    hbm_peak, tf_burst, tf_sust, peak_kind = peaks()
    wq = lc.IntegerQuantizer(4, False, 'per_group', group_size=128)

    X_host = make_activations(n_seq, 2001 + rank, pin=not args.no_e2e)
    X = X_host.to(dev)

    if args.workload == 'block':
        block_host, kwargs_host = make_block()
        kwargs = kwargs_to(kwargs_host, dev)
        master = copy.deepcopy(block_host).to(dev)
        runner = lc.GPTQBlockwise(wq, SPECIAL, quant_out=True)
        solver = runner.solver
        timer = HessianTimer(solver)
        bs = max(1, min(args.calib_bs, n_seq))
        inputs = [X[i:i + bs] for i in range(0, n_seq, bs)]

        def step():
            block = copy.deepcopy(master)          # device copy of the bf16 block (the reference does block.cuda())
            outs = runner.block_opt(block, inputs, kwargs)
            return block, outs

        if not args.no_e2e:
            for p in block_host.parameters():
                p.data = p.data.pin_memory()
            x_stages = [torch.empty_like(X), torch.empty_like(X)]
            w_host = {n: torch.empty(rc, dtype=torch.float32).pin_memory()
                      for n, rc in zip(LINEAR_KEYS, LINEAR_SHAPES) if LINEAR_KEYS.index(n) % world == rank}

            host_params = [p.data for p in block_host.parameters()]
            copy_in, copy_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
            chunk = 8
            name_to_key = {'self_attn.q_proj': 'q', 'self_attn.k_proj': 'k', 'self_attn.v_proj': 'v',
                           'self_attn.o_proj': 'o', 'mlp.gate_proj': 'gate', 'mlp.up_proj': 'up',
                           'mlp.down_proj': 'down'}
            # steps_left: steps still to run in the current (warm-up or timed) sequence; pending: the
            # copy events of activations already on their way for the next step, and their buffer
            e2e_state = {'steps_left': 0, 'pending': None, 'buf': 0, 'prev_block': None}

            def start_input_copy(buf):
                evs = []
                with torch.cuda.stream(copy_in):
                    for i in range(0, n_seq, chunk):
                        x_stages[buf][i:i + chunk].copy_(X_host[i:i + chunk], non_blocking=True)
                        ev = torch.cuda.Event()
                        ev.record(copy_in)
                        evs.append(ev)
                return evs

            p_stages = [[torch.empty_like(p, device=dev) for p in host_params] for _ in range(2)] if rank == 0 else None

            def start_copies(buf):
                """Parameters (rank 0) and activations of one step, host -> staging buffers `buf`."""
                p_ev = None
                if rank == 0:
                    with torch.cuda.stream(copy_in):
                        for d, hp in zip(p_stages[buf], host_params):
                            d.copy_(hp, non_blocking=True)
                        p_ev = torch.cuda.Event()
                        p_ev.record(copy_in)
                return p_ev, start_input_copy(buf)

            def e2e_step():
                # Host -> device copies run on their own stream into one of two sets of staging buffers:
                # the block's parameters, then the activations chunk by chunk; the first stage of the block
                # waits for the chunk it is about to read.  While a step computes, the parameters and
                # activations of the NEXT step of the same sequence of steps are already copied into the
                # other set (a caller that streams a model's blocks through the GPU prefetches the same
                # way); the first step of a sequence copies its own inputs, the last one prefetches nothing
                # and waits for its results to reach the host, so every copy lies inside the timed region.
                # Each subset's quantised weights go back to the host on a third stream while the next
                # stage (or the next step) computes (the reference's block.cuda() / block.cpu()).
                main_s = torch.cuda.current_stream()
                copy_in.wait_stream(main_s)
                block = copy.deepcopy(master)
                if e2e_state['pending'] is None:
                    e2e_state['pending'] = start_copies(e2e_state['buf'])
                (p_ev, evs), buf = e2e_state['pending'], e2e_state['buf']
                # the block's parameters cross PCIe once (rank 0) and reach the other ranks over NVLink
                if rank == 0:
                    main_s.wait_event(p_ev)
                for i, p in enumerate(block.parameters()):
                    if rank == 0:
                        p.data.copy_(p_stages[buf][i], non_blocking=True)
                    if world > 1:
                        dist.broadcast(p.data, src=0)
                x_stage = x_stages[buf]
                e2e_state['steps_left'] -= 1
                if e2e_state['steps_left'] > 0:
                    e2e_state['buf'] = 1 - buf
                    e2e_state['pending'] = start_copies(1 - buf)
                else:
                    e2e_state['pending'] = None
                mods = dict(block.named_modules())

                def on_input(i):
                    if (i * bs) % chunk == 0:
                        main_s.wait_event(evs[min(len(evs) - 1, (i * bs) // chunk)])
                    if bs > chunk:
                        main_s.wait_event(evs[min(len(evs) - 1, ((i + 1) * bs - 1) // chunk)])

                def on_subset_done(names):
                    done = torch.cuda.Event()
                    done.record(main_s)
                    copy_out.wait_event(done)
                    with torch.cuda.stream(copy_out):
                        # every rank holds the same quantised weights; each linear goes back to the host
                        # from one rank only
                        for nme in names:
                            key = name_to_key[nme]
                            if LINEAR_KEYS.index(key) % world == rank:
                                w_host[key].copy_(mods[nme].weight, non_blocking=True)
                runner.on_input, runner.on_subset_done = on_input, on_subset_done
                outs = runner.block_opt(block, [x_stage[i:i + bs] for i in range(0, n_seq, bs)], kwargs)
                runner.on_input = runner.on_subset_done = None
                # the device-to-host copies of the last subset may still run while the next step starts; the
                # block they read from stays referenced until then.  The last step of a sequence waits.
                e2e_state['prev_block'] = block
                if e2e_state['steps_left'] <= 0:
                    main_s.wait_stream(copy_out)
                    e2e_state['prev_block'] = None
                return outs
            h2d = int(X_host.numel() * 2 * world + sum(p.numel() * 2 for p in block_host.parameters()))   # whole job
            d2h = int(sum(r * c * 4 for r, c in LINEAR_SHAPES))
        # kernels of this library per step (torch's own kernels -- cuBLAS GEMMs of the forward, cuSOLVER
        # potrf, SDPA, argsort, gathers -- are not counted):
        #   Hessian launches, 4 diag; per distinct Hessian (3 x C=4096, 1 x C=11008): damp + permute,
        #   low-part split, leaf inverse, flip, and 5 launches (2 GEMMs, 2 splits, 1 transpose) per internal
        #   node of the recursive triangular inverse (C/128 - 1 nodes);
        #   per subset (the rows of its linears are solved as one stacked matrix): permute W, un-permute, and
        #   per 128-column block the block kernel plus the eager / sub-panel / panel updates counted below;
        #   per linear the deploy-time fake quant;
        #   per sequence: 2 RMS norms, 2 rotary embeddings, 1 SiLU-gate.
        n_calls = -(-n_seq // bs)

        def solver_launches(c):
            # block kernels, eager FFMA updates (one per block that is not the last of its 256-column
            # sub-panel), K = 256 GEMMs (one per sub-panel that is not the last of its panel), K = 1024 GEMMs
            blocks, subs, panels = -(-c // 128), -(-c // 256), -(-c // 1024)
            return blocks + (blocks - subs) + (subs - panels) + (panels - 1)
        launches = (4 * -(-n_calls // HESSIAN_BATCH) + 4
                    + sum(2 + 1 + 1 + 1 + 5 * (c // 128 - 1) for c in (HID, HID, HID, INTER))
                    + sum(2 + solver_launches(c) for c in (HID, HID, HID, INTER)) + len(LINEAR_SHAPES)
                    + 5 * n_calls)
    else:
        W_host = make_linear_weight().pin_memory() if not args.no_e2e else make_linear_weight()
        W = W_host.to(dev)
        solver = lc.GPTQ(wq, SPECIAL)
        timer = HessianTimer(solver)
        layer = torch.nn.Linear(HID, HID, bias=False, dtype=torch.bfloat16, device=dev)
        r0, r1 = parallel.row_shard(HID)

        def run_layer(x_dev, w):
            layer.weight.data = w
            solver.layer_init(layer, 'l')
            for i in range(n_seq):
                solver.add_batch(layer, 'l', x_dev[i:i + 1])
            res = solver.layer_transform(layer, 'l', rows=None if world == 1 else (r0, r1))
            out = res['weight'] if world == 1 else parallel.gather_rows(res['weight'], HID)
            solver.free('l')
            return out, res

        def step():
            return run_layer(X, W)

        if not args.no_e2e:
            copy_stream = torch.cuda.Stream(device=dev)
            x_stage = torch.empty_like(X)
            rows_here = HID if world == 1 else r1 - r0
            out_host = torch.empty((rows_here, HID), dtype=torch.float32).pin_memory()
            sc_host = torch.empty((rows_here * (HID // 128), 1), dtype=torch.float32).pin_memory()
            zr_host = torch.empty_like(sc_host).pin_memory()

            def e2e_step():
                main_s = torch.cuda.current_stream()
                copy_stream.wait_stream(main_s)       # the previous step's readers of x_stage are done
                layer.weight.data = W_host.to(dev, non_blocking=True)
                solver.layer_init(layer, 'l')
                evs = []
                with torch.cuda.stream(copy_stream):
                    for i in range(0, n_seq, HESSIAN_BATCH):
                        x_stage[i:i + HESSIAN_BATCH].copy_(X_host[i:i + HESSIAN_BATCH], non_blocking=True)
                        ev = torch.cuda.Event()
                        ev.record(copy_stream)
                        evs.append(ev)
                for k, i in enumerate(range(0, n_seq, HESSIAN_BATCH)):
                    main_s.wait_event(evs[k])
                    for j in range(i, min(i + HESSIAN_BATCH, n_seq)):
                        solver.add_batch(layer, 'l', x_stage[j:j + 1])
                res = solver.layer_transform(layer, 'l', rows=None if world == 1 else (r0, r1))
                out_host.copy_(res['weight'], non_blocking=True)
                sc_host.copy_(res['buf_scales'], non_blocking=True)
                zr_host.copy_(res['buf_zeros'], non_blocking=True)
                solver.free('l')
            h2d = int(X_host.numel() * 2 + W_host.numel() * 2)
            d2h = int(out_host.numel() * 4 + sc_host.numel() * 8)
        launches = -(-n_seq // HESSIAN_BATCH) + 1 + 3 + 1 + 2 * (HID // 128) - 1 + 1

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
        step()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    timer.on = True
    ms_step = timed(step, args.steps) / args.steps
    timer.on = False
    value = 1e3 / ms_step
    hess = timer.summary()

    # ---- end to end: host buffers in, host result out ------------------------------------------
    e2e = None
    if not args.no_e2e:
        if args.workload == 'block':
            e2e_state['steps_left'] = 2
        for _ in range(2):
            e2e_step()
        if args.workload == 'block':
            e2e_state['steps_left'] = args.steps
        e2e_ms = timed(e2e_step, args.steps) / args.steps
        e2e = {'value': 1e3 / e2e_ms, 'unit': UNIT, 'ms_per_step': e2e_ms, 'h2d_bytes_per_step': h2d,
               'd2h_bytes_per_step': d2h,
               'overlap': ('copies on side streams; the parameters and activations of step s+1 are prefetched into '
                           'a second set of staging buffers while step s computes (not for the first step, none '
                           'after the last, which also waits for its results on the host: all copies lie inside '
                           'the timed region)') if args.workload == 'block' else 'none'}
    clocks = sampler.stop() if sampler else None

    # ---- the other two headline kernels, timed alone (HBM-bound family 1) ----------------------
    aux = None
    if rank == 0 and args.workload == 'block':
        aux = rtn_aux(hbm_peak, dev)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel of ours: the Hessian GEMM -------------------------------
    # algorithmic FLOPs = 2 * tokens * C^2 per launch (the full square the reference computes);
    # executed = the 256x256 tiles on/above the diagonal that are actually issued
    n_l = sum(d[0] for d in hess.values())
    ms_l = sum(d[1] for d in hess.values())
    alg = sum(2.0 * d[2] * c * c for c, d in hess.items())
    exe = sum(2.0 * d[2] * 256 * 256 * n_super(c) for c, d in hess.items())
    achieved = alg / (ms_l * 1e-3) / 1e12
    roofline = {'bound': 'tensor', 'kernel': 'hessian_umma_kernel', 'achieved': achieved, 'peak': tf_sust,
                'unit': 'TFLOP/s', 'frac': achieved / tf_sust,
                'peak_kind': f'{peak_kind} sustained cuBLAS bf16 (of measured)',
                'achieved_executed': exe / (ms_l * 1e-3) / 1e12, 'frac_executed': exe / (ms_l * 1e-3) / 1e12 / tf_sust,
                'launch_ms': ms_l / n_l, 'launches_per_step': n_l / args.steps,
                'share_of_step': ms_l / args.steps / ms_step,
                'per_cols': {str(c): {'launches_per_step': d[0] / args.steps, 'launch_ms': d[1] / d[0],
                                      'tokens_per_launch': d[2] / d[0]} for c, d in hess.items()},
                'traffic': None}
    # DRAM bytes per 16384-token launch from the ncu captures summarised under profiles/ (Hessian kernel)
    # (dram__bytes_read.sum + dram__bytes_write.sum); the bench launches the same shapes
    ncu_traffic = {4096: 213.7e6, 11008: 2833.0e6}
    if all(c in ncu_traffic and abs(d[2] / d[0] - 16384) < 1 for c, d in hess.items()):
        roofline['traffic'] = sum(d[0] * ncu_traffic[c] for c, d in hess.items()) / n_l
        roofline['traffic_source'] = 'ncu, per launch, weighted over the launch mix of the step'
        roofline['algorithmic_bytes'] = sum(d[0] * (2.0 * 16384 * c + 8.0 * c * c) for c, d in hess.items()) / n_l

    line = {'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': world, 'steps': args.steps,
            'warmup': args.warmup, 'ms_per_step': ms_step, 'higher_is_better': True, 'scaling': 'strong',
            'vs_baseline': None, 'dtype': 'bf16 in / fp32 accumulate', 'data': 'synthetic',
            'config': {'workload': WORKLOADS[args.workload], 'name': args.workload,
                       'l2': 'inputs (2.1 GB of activations per step) exceed the 126 MB L2',
                       'sharding': f'{n_seq} sequences per rank; solve units (linear, row range) dealt to the ranks',
                       'hessian_batch': HESSIAN_BATCH, 'calib_bs': args.calib_bs if args.workload == 'block' else 1,
                       'static_groups': bool(SPECIAL['static_groups'])},
            'roofline': roofline, 'gpu_launches': launches * args.steps, 'clocks': clocks}
    if e2e:
        line['e2e'] = e2e
    if aux:
        line['aux_kernels'] = aux
    if not args.no_cpu_baseline and world == 1:
        v, desc, cores, parts = (cpu_port_block() if args.workload == 'block' else cpu_port_layer(8))
        line['cpu_baseline'] = dict({'value': v, 'unit': UNIT, 'cores': cores, 'kind': 'port', 'sample': desc}, **parts)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
