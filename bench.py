"""Benchmark of the GPTQ calibration hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                    [--workload block|layer|model|awq|moe|kernel] [--case NAME --launches N]

Default workload `block` (the end-to-end GPTQ configuration's unit of work): ONE Llama-2-7B-shape
decoder layer (hidden 4096, 32 heads, MLP 11008, bf16, weights N(0, 0.02^2)) quantised with GPTQ
W4A16 asymmetric g128, act-order, percdamp 0.01, true_sequential, quant_out, on 128 x 2048 tokens
of synthetic hidden states (N(0,1), 1 % outlier channels x20).  A step = the reference's
per-block schedule (5 forwards of the block over all sequences, 4 distinct Hessians, 7 layer
solves); value = decoder layers per second.

Workload `layer` (the single-linear GPTQ configuration): one 4096 -> 4096 linear, 128 x 2048 x 4096
calibration activations; a step = Hessian accumulation over all sequences + the layer solve.

Workload `model` (the end-to-end configuration): a random-init 32-layer Llama-2-7B-shape model in host
memory, 128 x 2048 token ids -> embedding -> the block loop over all 32 layers with every block
streamed through the GPU (lightcompress_b200.HostStagedGPTQ.run_block_loop); a step = one pass over the
model, value = 32 / its duration.

Workload `kernel` (--case NAME): a small, self-terminating run of one kernel family sized for a
profiler capture (inputs larger than the 126 MB L2, a few hundred MB on the device, a handful of
launches); prints no benchmark line.

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
FACTORIZATION = 'native_full'   # `--workload kernel --case factor*`: this library's own blocked Cholesky + inverse
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


LINEAR_NAMES = ['self_attn.q_proj', 'self_attn.k_proj', 'self_attn.v_proj', 'self_attn.o_proj', 'mlp.gate_proj',
                'mlp.up_proj', 'mlp.down_proj']
# DRAM bytes per 16384-token Hessian launch by width, from the ncu captures under profiles/
HESSIAN_NCU_TRAFFIC = {4096: 310.4e6, 11008: 3511.0e6}
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


_SOLVER_CACHE = {}


def cpu_port_block(seq_index=0):
    """One sequence (number `seq_index` of the 128) through the reference schedule's five forwards with
    its Hessian hooks, scaled x128, plus the solver: prepare and weight_transform timed once per process
    on a 4096x4096 linear and scaled to the seven linears by C^3 and rows*cols respectively.
    Returns (layers/s extrapolated, description, cores, parts, seconds actually spent)."""
    import torch
    from oracle import gptq_block_ref, gptq_ref
    cores = os.cpu_count()
    torch.set_num_threads(cores)
    t_begin = time.perf_counter()
    block, kwargs = make_block()
    x = make_activations(seq_index + 1, 2001)[seq_index:seq_index + 1]
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
    if 'solver' not in _SOLVER_CACHE:
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
        _SOLVER_CACHE['solver'] = sum(t_prep * (c / HID) ** 3 + t_wt * (r * c) / (HID * HID) for r, c in LINEAR_SHAPES)
    t_solver = _SOLVER_CACHE['solver']
    desc = (f'forwards + Hessian hooks: 1 of {NS} sequences (a different one each step) through the 5 passes, scaled '
            f'x{NS}; solver: prepare and weight_transform timed once on one 4096x4096 linear, scaled to the 7 linears '
            f'by C^3 and rows*cols')
    return (1.0 / (t_fwd + t_solver), desc, cores, {'forward_hessian_s': t_fwd, 'solver_s': t_solver},
            time.perf_counter() - t_begin)


def run_reference(args, rank):
    """The reference arm: the CPU port of the reference on the host cores.  A full step of the workload
    takes over an hour on the host, so each step times a bounded sample and the value is an
    extrapolation, marked as such; `ms_per_step` is the time a step really took here."""
    if rank != 0:
        return
    vals, spent, desc, cores = [], [], None, None
    for i in range(args.warmup + args.steps):
        if args.workload == 'layer':
            t0 = time.perf_counter()
            v, desc, cores, _ = cpu_port_layer(4)
            dt = time.perf_counter() - t0
        else:
            v, desc, cores, _, dt = cpu_port_block(seq_index=i % NS)
        if i >= args.warmup:
            vals.append(v)
            spent.append(dt)
    v = sum(vals) / len(vals)
    name = 'layer' if args.workload == 'layer' else 'block'
    print(json.dumps({
        'impl': 'reference', 'metric': METRIC, 'value': v, 'unit': UNIT, 'n_gpus': args.gpus, 'steps': args.steps,
        'warmup': args.warmup, 'ms_per_step': 1e3 * sum(spent) / len(spent), 'higher_is_better': True,
        'scaling': 'strong', 'vs_baseline': None, 'dtype': 'bf16 in / fp32 accumulate', 'data': 'synthetic',
        'extrapolated': True, 'extrapolated_ms_per_step': 1e3 / v,
        'sample_fraction': {'sequences': 1.0 / NS if name == 'block' else 4.0 / NS,
                            'solver': 'one 4096x4096 linear of the seven' if name == 'block' else 'full'},
        'spread': {'min': min(vals), 'max': max(vals)},
        'config': {'workload': WORKLOADS[name], 'name': name},
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


def _time_launches(run, n=40, warm=8):
    import torch
    for i in range(warm):
        run(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(n):
        run(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n * 1e3


def rtn_aux(hbm_peak, dev):
    """quant_dequant GB/s of the RTN kernel.  The reference's CPU-runnable configuration as stated -- fp32
    4096x4096, W4 asymmetric, groups of 128, outputs: dequantised weight + packed int4 codes + scales +
    zeros (143.7 MB algorithmic) -- through the raw C ABI and through the IntegerQuantizer methods a
    caller uses; the dequantised weight alone (fake quant, 134.2 MB + parameters); and tensors far larger
    than L2.  8 rotating buffers at 4096x4096 so that no launch finds its input in L2, CUDA events around
    40 launches."""
    import torch
    import lightcompress_b200 as lc
    from lightcompress_b200 import _lib as L
    out = {}
    qz = lc.IntegerQuantizer(4, False, 'per_group', group_size=128)
    for name, rows, cols, dt in (('rtn_w4_g128_fp32_4096x4096', 4096, 4096, torch.float32),
                                 ('rtn_w4_g128_fp32_16384x8192', 16384, 8192, torch.float32),
                                 ('rtn_w4_g128_bf16_16384x8192', 16384, 8192, torch.bfloat16)):
        n_buf = 8 if rows == 4096 else 2
        g = torch.Generator().manual_seed(1001)
        ws = [(torch.randn(rows, cols, generator=g) * 0.02).to(dt).to(dev) for _ in range(n_buf)]
        outs = [torch.empty_like(w) for w in ws]
        st = L.stream_of(ws[0])
        esz = ws[0].element_size()
        n_grp = rows * cols // 128

        def fake_only(i):
            L.call('lc_rtn_int_quant', L.ptr(ws[i % n_buf]), L.lc_dtype(ws[0]), rows, cols, 128, 4, 0, None, None,
                   L.ptr(outs[i % n_buf]), None, L.LC_CODES_NONE, None, None, st)
        us = _time_launches(fake_only)
        nbytes = 2 * rows * cols * esz
        out[name] = {'us': us, 'algorithmic_bytes': nbytes, 'gb_s': nbytes / us / 1e3,
                     'frac_of_measured_hbm': nbytes / us / 1e3 / hbm_peak, 'outputs': 'dequantised weight', 'via': 'C ABI'}
        if rows == 4096:
            codes = [torch.empty((rows, cols // 2), dtype=torch.uint8, device=dev) for _ in range(n_buf)]
            sc = [torch.empty((n_grp, 1), dtype=dt, device=dev) for _ in range(n_buf)]
            zr = [torch.empty((n_grp, 1), dtype=dt, device=dev) for _ in range(n_buf)]

            def all_outputs(i):
                k = i % n_buf
                L.call('lc_rtn_int_quant', L.ptr(ws[k]), L.lc_dtype(ws[0]), rows, cols, 128, 4, 0, None, None,
                       L.ptr(outs[k]), L.ptr(codes[k]), L.LC_CODES_PACK4, L.ptr(sc[k]), L.ptr(zr[k]), st)
            full_bytes = 2 * rows * cols * esz + rows * cols // 2 + 2 * n_grp * esz
            for key, fn, via in (
                    (name + '_all_outputs', all_outputs, 'C ABI'),
                    (name + '_all_outputs_api', lambda i: qz.quant_all_dynamic(ws[i % n_buf], packed=True),
                     'IntegerQuantizer.quant_all_dynamic'),
                    (name + '_fake_api', lambda i: qz.fake_quant_weight_dynamic(ws[i % n_buf]),
                     'IntegerQuantizer.fake_quant_weight_dynamic')):
                us = _time_launches(fn)
                nb = nbytes if key.endswith('_fake_api') else full_bytes
                out[key] = {'us': us, 'algorithmic_bytes': nb, 'gb_s': nb / us / 1e3,
                            'frac_of_measured_hbm': nb / us / 1e3 / hbm_peak, 'via': via,
                            'outputs': ('dequantised weight' if key.endswith('_fake_api') else
                                        'dequantised weight + packed int4 codes + scales + zeros')}
            del codes, sc, zr
        del ws, outs
    return out


def run_secondary(args):
    """`--workload awq`: AWQ scale + clip search of one Llama-2-7B-shape block on 128 x 512 calibration
    tokens in one batch (W4 asym g128, trans_version v2, clip_version v1).  `--workload moe`: FP8 e4m3
    fake quant of a 64-expert MoE layer (per-channel weights once, per-token activations per forward);
    under torch.distributed.run the experts are sharded over the ranks.  Device-resident inputs and an
    end-to-end variant from pinned host memory, CUDA events, one JSON line with the configuration's own
    metric."""
    import torch
    import torch.distributed as dist
    import lightcompress_b200 as lc
    rank = int(os.environ.get('RANK', 0))
    local_rank = int(os.environ.get('LOCAL_RANK', 0))
    world = int(os.environ.get('WORLD_SIZE', 1))
    dev = torch.device('cuda', local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group('nccl', device_id=dev)
    hbm_peak = peaks()[0]
    extra = {}
    if args.workload == 'awq':
        if world > 1:
            raise SystemExit('--workload awq runs on one GPU')
        from lightcompress_b200.awq import Awq
        block_host, kwargs_host = make_block(seq_len=512)
        kwargs = kwargs_to(kwargs_host, dev)
        g = torch.Generator().manual_seed(3001)
        X_host = torch.randn(NS, 512, HID, generator=g)
        X_host[:, :, torch.randperm(HID, generator=g)[:41]] *= 20
        X_host = X_host.to(torch.bfloat16).pin_memory()
        X = X_host.to(dev)
        for p in block_host.parameters():
            p.data = p.data.pin_memory()
        master = copy.deepcopy(block_host).to(dev)
        wq = lc.IntegerQuantizer(4, False, 'per_group', group_size=128)
        awq = Awq(wq, {'trans': True, 'trans_version': 'v2', 'weight_clip': True, 'clip_version': 'v1'},
                  calib_seq_len=512)

        def step():
            return awq.block_transform(copy.deepcopy(master), X, kwargs)

        host_out = {n: torch.empty(p.shape, dtype=p.dtype).pin_memory() for n, p in block_host.named_parameters()}

        def e2e_step():
            blk = copy.deepcopy(block_host).to(dev, non_blocking=True)
            rep = awq.block_transform(blk, X_host.to(dev, non_blocking=True), kwargs)
            for n, p in blk.named_parameters():
                host_out[n].copy_(p.data, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            return rep
        h2d = int(X_host.numel() * 2 + sum(p.numel() * 2 for p in block_host.parameters()))
        d2h = int(sum(p.numel() * 2 for p in block_host.parameters()))
        metric, unit = 'AWQ W4 g128 scale+clip search blocks/sec', 'blocks/s'
        extra['_phases'] = awq.phases
        # FLOPs of the 80 inspect-module forwards (20 candidates x 4 subsets; the block's own bf16 GEMMs, run
        # by cuBLAS): attention module = q, k, v, o projections + attention; MLP = gate, up, down
        tok = NS * 512
        attn = 4 * 2 * tok * HID * HID + 2 * 2 * NS * 512 * 512 * HID
        mlp = 3 * 2 * tok * HID * INTER
        extra["_flops"] = 20 * (attn + 2 * tok * HID * HID + mlp + 2 * tok * HID * INTER)
        workload = ('one Llama-2-7B-shape decoder block, AWQ W4 asym g128, 20-point scale grid on 4 subsets + clip '
                    'search on 5 linears, 128x512 calibration tokens in one batch')
    else:
        from lightcompress_b200.moe_fp8 import Fp8FakeQuantMoE
        g = torch.Generator().manual_seed(5001)
        x_host = torch.randn(16384, 2048, generator=g).to(torch.bfloat16).pin_memory()
        x = x_host.to(dev)
        moe = Fp8FakeQuantMoE(device=dev)
        names = ('w_gate', 'w_up', 'w_down') + (('s_gate', 's_up', 's_down') if moe.has_shared else ())
        pristine = {n: getattr(moe, n).clone() for n in names}
        host_w = {n: t.cpu().pin_memory() for n, t in pristine.items()}
        out_host = torch.empty((16384, 2048), dtype=torch.bfloat16).pin_memory()

        def step():
            for n, t in pristine.items():
                setattr(moe, n, t)
            moe.quantize_weights()
            return moe.forward(x)

        def e2e_step():
            for n, t in host_w.items():
                setattr(moe, n, t.to(dev, non_blocking=True))
            moe.quantize_weights()
            y = moe.forward(x_host.to(dev, non_blocking=True))
            if rank == 0:
                out_host.copy_(y, non_blocking=True)
            torch.cuda.current_stream().synchronize()
        h2d = int(x_host.numel() * 2 * world + sum(t.numel() * 2 for t in host_w.values()) * world)
        d2h = int(out_host.numel() * 2)
        metric, unit = 'FP8 e4m3 fake-quant MoE layer passes/sec (weights quantised + one forward)', 'passes/s'
        workload = ('64 routed experts (1408 x 2048) + shared MLP, top-6, 16384 tokens, e4m3 per-channel weights, '
                    'per-token dynamic activations; experts sharded over the ranks, one all-reduce of the output')
        # algorithmic bytes of the fake-quant passes (weights once, activations per projection input)
        wbytes = 4 * (64 * 3 * 1408 * 2048 + 3 * 2 * 1408 * 2048)
        abytes = 4 * (16384 * 6 * (2048 + 1408) + 16384 * (2048 + 2816))
        extra['algorithmic_bytes'] = {'weights': wbytes, 'activations': abytes}

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
        return float(ms.item()) / steps
    for _ in range(max(3, args.warmup)):
        step()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    phases = extra.pop('_phases', None)
    flops = extra.pop('_flops', None)
    if phases is not None:
        phases.spans, phases.on = [], True
    ms = timed(step, args.steps)
    if phases is not None:
        phases.on = False
        extra['phases_ms'] = {k: v / args.steps for k, v in phases.summary().items()}
        extra['phases_ms']['other (capture forward, block copy)'] = ms - sum(extra['phases_ms'].values())
    for _ in range(2):
        e2e_step()
    e2e_ms = timed(e2e_step, args.steps)
    clocks = sampler.stop() if sampler else None
    if rank == 0:
        line = {'metric': metric, 'value': 1e3 / ms, 'unit': unit, 'n_gpus': world, 'steps': args.steps,
                'warmup': max(3, args.warmup), 'ms_per_step': ms, 'higher_is_better': True, 'scaling': 'strong',
                'vs_baseline': None, 'dtype': 'bf16', 'data': 'synthetic',
                'config': {'workload': workload, 'name': args.workload}, 'hbm_peak_gbs': hbm_peak,
                'e2e': {'value': 1e3 / e2e_ms, 'unit': unit, 'ms_per_step': e2e_ms, 'h2d_bytes_per_step': h2d,
                        'd2h_bytes_per_step': d2h}, 'clocks': clocks}
        line.update(extra)
        if flops:
            tf_peak = peaks()[2]
            line['roofline'] = {'bound': 'tensor', 'kernel': 'bf16 GEMMs of the inspect-module forwards (cuBLAS, library)',
                                'achieved': flops / (ms * 1e-3) / 1e12, 'peak': tf_peak, 'unit': 'TFLOP/s',
                                'frac': flops / (ms * 1e-3) / 1e12 / tf_peak, 'traffic': None,
                                'peak_kind': 'measured sustained cuBLAS bf16 (of measured)',
                                'note': 'FLOPs of the 80 candidate forwards over the whole step, which also holds the '
                                        'clip search and the scale kernels'}
        if args.workload == 'moe':
            tot = extra['algorithmic_bytes']['weights'] + extra['algorithmic_bytes']['activations']
            line['roofline'] = {'bound': 'hbm', 'achieved': tot / world / (ms * 1e-3) / 1e9, 'peak': hbm_peak,
                                'unit': 'GB/s', 'frac': tot / world / (ms * 1e-3) / 1e9 / hbm_peak, 'traffic': None,
                                'note': 'fake-quant bytes of one rank over the whole step; the step also runs the '
                                        "experts' GEMMs (cuBLAS), so this is a lower bound of the kernels' rate"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def n_super(c):
    s = -(-c // 256)
    return s * (s + 1) // 2


# ---- small kernel cases for profiler captures (--workload kernel --case NAME) -----------------------------
def kernel_case(name, n):
    import torch
    import lightcompress_b200 as lc
    from lightcompress_b200 import _lib as L
    wq4 = lc.IntegerQuantizer(4, False, 'per_group', group_size=128)

    def hessian_call(X, T, H, status):
        # the entry point GPTQ.add_batch's replacement uses: only the upper triangle of H is maintained
        import ctypes
        ptrs, toks = (ctypes.c_void_p * 1)(X.data_ptr()), (ctypes.c_int64 * 1)(T)
        L.call('lc_hessian_accum_upper', ptrs, toks, 1, X.shape[1], L.ptr(H), 1.0, 1.0, 0, L.ptr(status), L.stream_of(X))

    def hessian(C, seed):
        T = 16384
        g = torch.Generator().manual_seed(seed)
        X = torch.randn(T, C, generator=g).to(torch.bfloat16).cuda()
        H = torch.zeros(C, C, device='cuda')
        status = torch.zeros(1, dtype=torch.int32, device='cuda')
        for _ in range(n):
            hessian_call(X, T, H, status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        return X, H, status
    if name == 'hessian':
        X, H, status = hessian(4096, 1)
        for _ in range(n):
            hessian_call(X, 2048, H, status)
    elif name == 'hessian_wide':                      # the down_proj width, 16384 tokens per launch
        hessian(11008, 5)
    elif name in ('factor', 'factor_wide', 'factor_cusolver'):   # damp + Cholesky + triangular inverse of one Hessian
        C = 11008 if name == 'factor_wide' else 4096
        g = torch.Generator().manual_seed(6)
        X = torch.randn(2 * C, C, generator=g).cuda()
        H = X.t() @ X
        del X
        solver = lc.GPTQ(wq4, {'actorder': True, 'factorization': 'native' if name == 'factor_cusolver' else FACTORIZATION})
        for _ in range(n):
            solver.factorize(H, 0.5)
        solver.check_status()
    elif name == 'block_ops':                         # RMS norm, rotary embedding, SiLU-gate at Llama-2-7B width
        from lightcompress_b200 import block_ops as B
        g = torch.Generator().manual_seed(7)
        x = torch.randn(8, 2048, 4096, generator=g).to(torch.bfloat16).cuda()
        w = torch.ones(4096, dtype=torch.bfloat16, device='cuda')
        q = x.view(8, 2048, 32, 128).transpose(1, 2)
        cs = torch.randn(8, 2048, 128, generator=g).to(torch.bfloat16).cuda()
        gate = torch.randn(8 * 2048, 11008, generator=g).to(torch.bfloat16).cuda()
        for _ in range(n):
            B._rms_raw(x, w, 1e-5)
            B.rope_apply_one(q, cs, cs)
            B.silu_mul(gate, gate)
    elif name == 'fp8_linear':                        # act_quant + block-scaled FP8 GEMM, M 8192, N 11008, K 4096
        from lightcompress_b200.fp8_linear import act_quant, fp8_gemm
        from lightcompress_b200.quant import weight_cast_to_fp8
        g = torch.Generator().manual_seed(8)
        x = torch.randn(8192, 4096, generator=g).to(torch.bfloat16).cuda()
        w = (torch.randn(11008, 4096, generator=g) * 0.05).to(torch.bfloat16).cuda()
        wq, ws = weight_cast_to_fp8(w)
        for _ in range(n):
            a, a_s = act_quant(x)
            fp8_gemm(a, a_s, wq, ws)
    elif name == 'mse':                               # MSE range search, W4 asym g128, 8192 x 4096 fp32
        g = torch.Generator().manual_seed(9)
        w = (torch.randn(8192, 4096, generator=g) * 0.02).cuda()
        qz = lc.IntegerQuantizer(4, False, 'per_group', group_size=128, calib_algo='mse')
        grouped = qz.reshape_tensor(w)
        for _ in range(n):
            qz.get_tensor_range(grouped)
    elif name == 'awq_clip':                          # clip search of a 4096 x 4096 bf16 linear, 512 tokens
        g = torch.Generator().manual_seed(10)
        w = (torch.randn(4096, 4096, generator=g) * 0.02).to(torch.bfloat16).cuda()
        x = torch.randn(16, 512, 4096, generator=g).to(torch.bfloat16).cuda()
        awq = lc.Awq(wq4, {}, calib_seq_len=512)
        for _ in range(n):
            awq.auto_clip_layer(w, x, apply=False)
    elif name == 'rtn':
        g = torch.Generator().manual_seed(2)
        w = (torch.randn(8192, 4096, generator=g) * 0.02).cuda()
        for _ in range(n):
            wq4.fake_quant_weight_dynamic(w)
        for _ in range(n):
            wq4.quant_all_dynamic(w, packed=True)
        wb = w.to(torch.bfloat16)
        for _ in range(n):
            wq4.fake_quant_weight_dynamic(wb)
        qa = lc.IntegerQuantizer(8, True, 'per_token')
        x = torch.randn(16384, 4096, generator=g).to(torch.bfloat16).cuda()
        for _ in range(n):
            qa.fake_quant_act_dynamic(x)
    elif name == 'fp8':
        g = torch.Generator().manual_seed(3)
        x = torch.randn(65536, 2048, generator=g).to(torch.bfloat16).cuda()
        q = lc.FloatQuantizer('e4m3', True, 'per_token', use_qtorch=True)
        for _ in range(n):
            q.fake_quant_act_dynamic(x)
    elif name in ('gptq', 'gptq_wide'):               # the layer solve (block kernel + trailing updates)
        R, C = (4096, 4096) if name == 'gptq' else (4096, 11008)
        g = torch.Generator().manual_seed(4)
        W = (torch.randn(R, C, generator=g) * 0.02).to(torch.bfloat16).cuda()
        X = torch.randn(max(8192, 2 * C), C, generator=g).to(torch.bfloat16).cuda()
        H = torch.zeros(C, C, device='cuda')
        L.call('lc_hessian_accum', L.ptr(X), X.shape[0], C, L.ptr(H), 1.0, 1.0, 0, None, L.stream_of(X))
        solver = lc.GPTQ(wq4, {'actorder': True})
        fac = solver.factorize(H, 2.0 / 4)
        for _ in range(n):
            solver.solve(W, H, 2.0 / 4, factor=fac)
        solver.check_status()
    elif name == 'spqr':                              # SpQR solve of a 4096 x 4096 layer (groups of 16, outlier detection)
        R, C = 4096, 4096
        g = torch.Generator().manual_seed(11)
        W = torch.randn(R, C, generator=g) * 0.02
        W[torch.rand(R, C, generator=g) < 0.01] *= 8
        W = W.to(torch.bfloat16).cuda()
        X = torch.randn(8192, C, generator=g).to(torch.bfloat16).cuda()
        H = torch.zeros(C, C, device='cuda')
        L.call('lc_hessian_accum', L.ptr(X), X.shape[0], C, L.ptr(H), 1.0, 1.0, 0, None, L.stream_of(X))
        solver = lc.SpQR(lc.IntegerQuantizer(4, False, 'per_group', group_size=16, round_zp=False),
                         {'actorder': True, 'percdamp': 1, 'relative_threshold': 0.2})
        solver.h_upper = False
        fac = solver.factorize(H, 2.0 / 4)
        for _ in range(n):
            solver.solve(W, H, 2.0 / 4, factor=fac)
        solver.check_status()
    elif name == 'act_static':                        # per-tensor ranges of 8 tensors of 64 MB in one launch
        qz = lc.IntegerQuantizer(8, True, 'per_tensor', calib_algo='static_minmax')
        g = torch.Generator(device='cuda').manual_seed(8)
        acts = [torch.randn(4, 2048, 4096, generator=g, device='cuda').to(torch.bfloat16) for _ in range(8)]
        for _ in range(n):
            qz._tensor_ranges(acts)
    elif name == 'quik':
        from lightcompress_b200.quik import QUIK
        g = torch.Generator(device='cuda').manual_seed(9)
        x = torch.randn(65536, 4096, generator=g, device='cuda').to(torch.bfloat16)
        aq = lc.IntegerQuantizer(8, True, 'per_token')
        q = QUIK(lc.IntegerQuantizer(4, True, 'per_channel'), aq,
                 {'fp_relative': False, 'fp_features': 256, 'fp_threshold': 0.0})
        order = torch.randperm(4096, generator=g, device='cuda')
        a = {'int_indices': order[:-256], 'fp_indices': order[-256:]}
        for _ in range(n):
            q.get_tensor_scale('l', x)
            aq.fake_quant_act_dynamic(x[:32768], a)
    elif name == 'w48':
        bit4 = {'symmetric': False, 'granularity': 'per_group', 'group_size': 128, 'scales_bit': 8,
                'scales_symmetric': True, 'zeros_bit': 8, 'zeros_symmetric': True}
        bit8 = {'symmetric': True, 'granularity': 'per_channel', 'int_range': [-120, 120]}
        qz = lc.Weight48IntegerQuantizer(48, bit4, bit8)
        g = torch.Generator(device='cuda').manual_seed(10)
        w = torch.randn(16384, 8192, generator=g, device='cuda').to(torch.bfloat16)
        for _ in range(n):
            qz.fake_quant_weight_dynamic(w)
    else:
        raise SystemExit(f'unknown --case {name}')
    torch.cuda.synchronize()
    print('done', name)


KERNEL_CASES = ['hessian', 'hessian_wide', 'rtn', 'fp8', 'gptq', 'gptq_wide', 'factor', 'factor_wide', 'factor_cusolver', 'block_ops',
                'fp8_linear', 'mse', 'awq_clip', 'act_static', 'quik', 'w48', 'spqr']


# ---- parity of the timed configuration (outside the timed region) --------------------------------------
def parity_of_linear(W, X_list, res_codes_perm, res_perm, deployed, world, dev):
    """Code mismatch and reconstruction error of one quantised linear against the oracle evaluated with
    torch on the same GPU.  W: the linear's original weight; X_list: this rank's input tensors of the
    linear; res_*: the timed run's codes (permuted order) and permutation; deployed: its fake-quant weight.

    Three code figures.  `code_mismatch_perm_pinned`: the same solve repeated with the column order fixed
    to the oracle's -- this isolates the kernels and carries the 0.1 % bar.  `code_mismatch`: the timed
    result as it is.  `oracle_noise_floor`: the oracle against itself with its fp32 Hessian summed in
    another order (sum(x^T x) * 2/n instead of the running mean): with N(0,1) activations the diagonal
    of the Hessian, which is the act-order sort key, is nearly constant, so any change of summation order
    reorders hundreds of columns and moves this many codes of the reference's own result."""
    import torch
    import torch.distributed as dist
    import lightcompress_b200 as lc
    from oracle import gptq_ref
    C = W.shape[1]
    H_sum = torch.zeros(C, C, device=dev)
    n = torch.zeros(1, device=dev)
    for x in X_list:
        x2 = x.reshape(-1, C).float()
        H_sum += x2.t() @ x2
        n += x.shape[0]
    if world > 1:
        dist.all_reduce(H_sum)
        dist.all_reduce(n)
    H_sum *= 2.0 / float(n.item())
    if world == 1:
        st = gptq_ref.hessian_init(C, dev)
        for x in X_list:
            gptq_ref.add_batch(st, x)               # the reference's own running-mean arithmetic
        H = st['H']
    else:
        H = H_sum                                   # sequences are sharded: the summed form is the only one
    ref = gptq_ref.quantize_layer(W, H)
    ref_codes = gptq_ref.codes_permuted(ref).to(torch.int16)

    def orig(codes, perm):
        o = torch.empty(W.shape, dtype=torch.int16, device=dev)
        o[:, perm] = codes.to(torch.int16)
        return o
    b = orig(ref_codes, ref['buf_perm'])
    out = {'code_mismatch': float((orig(res_codes_perm, res_perm) != b).float().mean()),
           'perm_entries_differing': int((res_perm != ref['buf_perm']).sum())}
    if world == 1:
        alt = gptq_ref.quantize_layer(W, H_sum)
        out['oracle_noise_floor'] = float((orig(gptq_ref.codes_permuted(alt), alt['buf_perm']) != b).float().mean())
        out['oracle_noise_floor_perm_entries'] = int((alt['buf_perm'] != ref['buf_perm']).sum())
        del alt
    del H_sum
    # the kernels again, column order pinned to the oracle's
    solver = lc.GPTQ(lc.IntegerQuantizer(4, False, 'per_group', group_size=128), SPECIAL)
    lin = torch.nn.Linear(C, W.shape[0], bias=False, dtype=W.dtype, device=dev)
    lin.weight.data = W
    solver.layer_init(lin, 'p')
    for x in X_list:
        solver.add_batch(lin, 'p', x)
    Hk, hscale = solver._finish_hessian('p')
    fac = solver.factorize(Hk, hscale, perm=ref['buf_perm'])
    pinned = solver.solve(W, Hk, hscale, factor=fac)
    solver.check_status()
    out['code_mismatch_perm_pinned'] = float((pinned['codes_perm'].to(torch.int16) != ref_codes).float().mean())
    Xs = X_list[0].reshape(-1, C)[:4096].double()
    full = Xs @ W.double().t()
    e_got = float((Xs @ (W.double() - deployed.double()).t()).norm() / full.norm())
    e_ref = float((Xs @ (W.double() - gptq_ref.w_qdq(ref, torch.bfloat16).double()).t()).norm() / full.norm())
    out.update({'recon_error': e_got, 'recon_error_oracle': e_ref, 'recon_rel_diff': abs(e_got - e_ref) / e_ref,
                'oracle': 'oracle/gptq_ref.py (pinned to the reference) with torch on the same GPU',
                'bars': {'code_mismatch_perm_pinned': 1e-3, 'recon_rel_diff': 1e-2}})
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=3)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='b200', choices=['b200', 'reference'])
    ap.add_argument('--workload', default='block', choices=['block', 'layer', 'model', 'awq', 'moe', 'kernel'])
    ap.add_argument('--case', default='hessian', choices=KERNEL_CASES, help='--workload kernel: which kernel family')
    ap.add_argument('--launches', type=int, default=3, help='--workload kernel: launches of each kernel')
    ap.add_argument('--layers', type=int, default=32, help='--workload model: decoder layers of the model')
    ap.add_argument('--calib-bs', type=int, default=1,
                    help='sequences per block-forward call (calib.bs of the reference config; block workload)')
    ap.add_argument('--static-groups', action='store_true',
                    help='special.static_groups of the reference (its export configs); a side measurement')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-e2e', action='store_true')
    ap.add_argument('--no-parity', action='store_true')
    args = ap.parse_args()
    if args.static_groups:
        SPECIAL['static_groups'] = True
    rank = int(os.environ.get('RANK', 0))
    local_rank = int(os.environ.get('LOCAL_RANK', 0))
    world = int(os.environ.get('WORLD_SIZE', 1))
    if args.impl == 'reference':
        run_reference(args, rank)
        return
    if args.workload == 'kernel':
        kernel_case(args.case, args.launches)
        return
    if args.workload in ('awq', 'moe'):
        run_secondary(args)
        return

    import torch
    import torch.distributed as dist
    import lightcompress_b200 as lc
    from lightcompress_b200 import block_ops, parallel

    torch.cuda.set_device(local_rank)
    dev = torch.device('cuda', local_rank)
    if world > 1:
        dist.init_process_group('nccl', device_id=dev)
    assert world == args.gpus, f'--gpus {args.gpus} but WORLD_SIZE={world}'
    s0, s1 = parallel.sequence_shard(NS)
    n_seq = s1 - s0
    hbm_peak, tf_burst, tf_sust, peak_kind = peaks()
    wq = lc.IntegerQuantizer(4, False, 'per_group', group_size=128)
    phases = None
    parity_fn = None
    checksum_fn = None
    extra_cfg = {}

    def blocks_per_step_launches(n_calls):
        # Kernels of this library per decoder block (torch's own kernels -- cuBLAS GEMMs of the forward, cuSOLVER
        # potrf of the three 4096-wide Hessians, SDPA, argsort, residual adds -- are not counted).  Per sequence:
        # 2 RMS norms, 2 rotary embeddings, 1 SiLU-gate.  Per Hessian batch and subset: one accumulation launch.
        # The rest is fixed by the shapes (3 Hessians of width 4096, one of 11008; 182 column blocks) and was
        # counted from the ncu launch list of this very workload (profiles/bench_block_workload_launch_list.md):
        # 4 x (diag, damp, permute H, flip, permute W, un-permute), 7 deploy-time dequantisations, 182 in-block
        # kernels, 91 eager FFMA updates, 152 tensor-core GEMMs (triangular inverses + sub-panel / panel updates)
        # with 47 low-part splits and 22 transposes, 3 leaf-inverse launches, and the own Cholesky of the
        # 11008-wide Hessian: 86 leaf + 85 panel + 64 strip launches.
        fixed = 4 * 6 + 7 + 182 + 91 + 152 + 47 + 22 + 3 + 86 + 85 + 64
        return 5 * n_calls + 4 * -(-n_calls // HESSIAN_BATCH) + fixed

    def fresh_host_block(block_host):
        """New module objects over the same (pinned) parameter storage: a step must not see the quantised
        weights an earlier step left on the host copy."""
        return copy.deepcopy(block_host, memo={id(p): torch.nn.Parameter(p.data, requires_grad=False)
                                               for p in block_host.parameters()})

    if args.workload == 'block':
        X_host = make_activations(n_seq, 2001 + rank, pin=not args.no_e2e)
        X = X_host.to(dev)
        block_host, kwargs_host = make_block()
        kwargs = kwargs_to(kwargs_host, dev)
        master = copy.deepcopy(block_host).to(dev)
        runner = lc.GPTQBlockwise(wq, SPECIAL, quant_out=True)
        solver = runner.solver
        phases = runner.phases
        timer = HessianTimer(solver)
        bs = max(1, min(args.calib_bs, n_seq))
        inputs = [X[i:i + bs] for i in range(0, n_seq, bs)]
        last = {}

        def step():
            block = copy.deepcopy(master)          # device copy of the bf16 block (the reference does block.cuda())
            outs = runner.block_opt(block, inputs, kwargs)
            last['block'] = block
            return block, outs

        if not args.no_e2e:
            for p in block_host.parameters():
                p.data = p.data.pin_memory()
            stager = lc.HostStagedGPTQ(runner, dev, chunk=8)
            host_inputs = [X_host[i:i + bs] for i in range(0, n_seq, bs)]
            out_host = {n: torch.empty(rc, dtype=torch.float32).pin_memory()
                        for n, rc in zip(LINEAR_NAMES, LINEAR_SHAPES) if LINEAR_NAMES.index(n) % world == rank}
            e2e_state = {'steps_left': 0, 'next': None}

            def e2e_step():
                # One block from host memory through lightcompress_b200.HostStagedGPTQ: parameters and
                # activations cross PCIe on a copy stream (the first stage waits chunk by chunk), the
                # quantised weights return on another stream while the next stage computes.  Within a
                # sequence of steps the parameters and activations of step s+1 are prefetched while step s
                # computes (a caller that streams a model's blocks through the GPU does the same); the first
                # step copies its own inputs, the last one prefetches nothing and waits for its results on
                # the host, so every copy lies inside the timed region.
                blk = e2e_state['next'] or fresh_host_block(block_host)
                e2e_state['steps_left'] -= 1
                nxt = None
                if e2e_state['steps_left'] > 0:
                    nxt = fresh_host_block(block_host)
                e2e_state['next'] = nxt
                xs = e2e_state.get('xs') or list(host_inputs)
                nxt_xs = list(host_inputs) if nxt is not None else None
                e2e_state['xs'] = nxt_xs
                return stager.block_opt(blk, xs, kwargs, next_block_host=nxt, wait_results=nxt is None,
                                        out_host=out_host, next_inputs=nxt_xs)
            h2d = int(X_host.numel() * 2 * world + sum(p.numel() * 2 for p in block_host.parameters()))   # whole job
            d2h = int(sum(r * c * 4 for r, c in LINEAR_SHAPES))
        launches = blocks_per_step_launches(-(-n_seq // bs))

        def parity_fn():
            blk = last['block']
            q = blk.self_attn.q_proj
            xs = [block_ops.rms_norm(master.input_layernorm, x) for x in inputs]
            return dict(parity_of_linear(master.self_attn.q_proj.weight.data, xs, q._lc_codes[0], q.buf_perm,
                                         q.tmp_weight, world, dev), linear='self_attn.q_proj (4096x4096)')

        def checksum_fn():
            blk = last['block']
            return torch.stack([getattr(p, a).tmp_weight.float().sum() for s in lc.llama_subsets(blk)
                                for p, a in s.values()])
    elif args.workload == 'model':
        from transformers import LlamaConfig
        from transformers.models.llama.modeling_llama import LlamaDecoderLayer
        n_layers = args.layers
        cfg = LlamaConfig(hidden_size=HID, intermediate_size=INTER, num_attention_heads=HEADS,
                          num_key_value_heads=HEADS, num_hidden_layers=n_layers, vocab_size=32000,
                          max_position_embeddings=4096, rms_norm_eps=1e-5)
        cfg._attn_implementation = 'sdpa'
        _, kwargs_host = make_block()
        kwargs = kwargs_to(kwargs_host, dev)
        # random-init weights N(0, 0.02^2) drawn on the GPU (seed per layer, the same on every rank) and
        # kept in pinned host memory like the reference's CPU-resident model; token ids uniform in the vocab
        template = LlamaDecoderLayer(cfg, 0).to(torch.bfloat16)
        blocks_host = []
        for li in range(n_layers):
            gg = torch.Generator(device=dev).manual_seed(7000 + li)
            blk = copy.deepcopy(template)
            for p in blk.parameters():
                d = (torch.randn(p.shape, generator=gg, device=dev) * 0.02).to(torch.bfloat16) if p.dim() == 2 \
                    else torch.ones(p.shape, dtype=torch.bfloat16, device=dev)
                h = torch.empty(p.shape, dtype=torch.bfloat16).pin_memory()
                h.copy_(d)
                p.data = h
            blocks_host.append(blk)
        gg = torch.Generator(device=dev).manual_seed(6999)
        embed_host = (torch.randn(32000, HID, generator=gg, device=dev) * 0.02).to(torch.bfloat16).cpu().pin_memory()
        gi = torch.Generator().manual_seed(4001)
        ids_host = torch.randint(0, 32000, (NS, T), generator=gi)[s0:s1].pin_memory()
        out_pool = [{n: torch.empty(rc, dtype=torch.float32).pin_memory()
                     for n, rc in zip(LINEAR_NAMES, LINEAR_SHAPES) if LINEAR_NAMES.index(n) % world == rank}
                    for _ in range(n_layers)]
        runner = lc.GPTQBlockwise(wq, SPECIAL, quant_out=True)
        solver = runner.solver
        phases = runner.phases
        timer = HessianTimer(solver)
        stager = lc.HostStagedGPTQ(runner, dev, chunk=8)
        per_block = []

        def model_step():
            """Token ids and the embedding table from pinned host memory -> hidden states -> run_block_loop over
            all layers, every block streamed from and back to the host copy (llmc/__main__.py:55-70)."""
            fresh = [fresh_host_block(b) for b in blocks_host]
            emb = embed_host.to(dev, non_blocking=True)
            ids = ids_host.to(dev, non_blocking=True)
            xs = [torch.nn.functional.embedding(ids[i:i + 1], emb) for i in range(n_seq)]
            del emb
            outs, secs = stager.run_block_loop(fresh, xs, kwargs, out_host=out_pool)
            per_block[:] = secs
            return outs
        step = e2e_step = model_step
        h2d = int(ids_host.numel() * 8 * world + embed_host.numel() * 2 * world
                  + n_layers * sum(p.numel() * 2 for p in template.parameters()))
        d2h = int(n_layers * sum(r * c * 4 for r, c in LINEAR_SHAPES))
        launches = n_layers * blocks_per_step_launches(n_seq)
        extra_cfg = {'layers': n_layers, 'inputs': 'token ids + embedding table in pinned host memory'}
        WORKLOADS['model'] = (f'random-init {n_layers}-layer Llama-2-7B-shape model (hidden 4096, 32 heads, MLP 11008, '
                              'vocab 32000, bf16 N(0,0.02^2)) in host memory, GPTQ W4A16 asym g128, act_order, '
                              'true_sequential, quant_out; 128x2048 token ids uniform in the vocab; every block '
                              'streamed through the GPU')
    else:
        X_host = make_activations(n_seq, 2001 + rank, pin=not args.no_e2e)
        X = X_host.to(dev)
        W_host = make_linear_weight().pin_memory() if not args.no_e2e else make_linear_weight()
        W = W_host.to(dev)
        solver = lc.GPTQ(wq, SPECIAL)
        timer = HessianTimer(solver)
        layer = torch.nn.Linear(HID, HID, bias=False, dtype=torch.bfloat16, device=dev)
        r0, r1 = parallel.row_shard(HID)
        last = {}

        def run_layer(x_dev, w):
            layer.weight.data = w
            solver.layer_init(layer, 'l')
            for i in range(n_seq):
                solver.add_batch(layer, 'l', x_dev[i:i + 1])
            res = solver.layer_transform(layer, 'l', rows=None if world == 1 else (r0, r1))
            out = res['weight'] if world == 1 else parallel.gather_rows(res['weight'], HID)
            solver.free('l')
            last['res'] = res
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
                torch.cuda.current_stream().synchronize()      # the step's result is on the host
            h2d = int(X_host.numel() * 2 * world + W_host.numel() * 2 * world)
            d2h = int(HID * HID * 4 + HID * (HID // 128) * 8)
        launches = -(-n_seq // HESSIAN_BATCH) + 1 + 3 + 1 + 2 * (HID // 128) - 1 + 1

        def parity_fn():
            if world > 1:
                return None                      # rows are sharded here; the block workload covers N > 1
            res = last['res']
            lin = torch.nn.Linear(HID, HID, bias=False, dtype=torch.bfloat16, device=dev)
            lin.weight.data = res['weight']
            for k in ('buf_scales', 'buf_zeros', 'buf_perm', 'buf_invperm'):
                lin.register_buffer(k, res[k])
            lin.register_buffer('buf_qmax', wq.qmax.to(dev))
            lin.register_buffer('buf_qmin', wq.qmin.to(dev))
            return dict(parity_of_linear(W, [X[i:i + 1] for i in range(n_seq)], res['codes_perm'], res['buf_perm'],
                                         solver.w_qdq(lin, wq), world, dev), linear='the 4096x4096 layer')

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

    # ---- device-resident throughput (model workload: the same host-staged loop, it has no other form) ----
    for _ in range(args.warmup):
        step()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    timer.on = True
    if phases is not None:
        phases.spans = []
        phases.on = True
    ms_step = timed(step, args.steps) / args.steps
    timer.on = False
    phase_ms = None
    if phases is not None:
        phases.on = False
        phase_ms = {k: v / args.steps for k, v in phases.summary().items()}
        phase_ms['other (host waits, copies of the block, residual)'] = ms_step - sum(phase_ms.values())
    value = (args.layers if args.workload == 'model' else 1) * 1e3 / ms_step
    hess = timer.summary()

    # ---- end to end: host buffers in, host result out ------------------------------------------
    e2e = None
    if args.workload == 'model':
        e2e = {'value': value, 'unit': UNIT, 'ms_per_step': ms_step, 'h2d_bytes_per_step': h2d, 'd2h_bytes_per_step': d2h,
               'overlap': 'the model loop is host-staged by construction: value and e2e are the same measurement',
               'per_block_s': {'first': per_block[0], 'median': sorted(per_block)[len(per_block) // 2],
                               'last': per_block[-1]}}
    elif not args.no_e2e:
        if args.workload == 'block':
            e2e_state['steps_left'] = 2
        for _ in range(2):
            e2e_step()
        if args.workload == 'block':
            e2e_state['steps_left'] = args.steps
        e2e_ms = timed(e2e_step, args.steps) / args.steps
        e2e = {'value': 1e3 / e2e_ms, 'unit': UNIT, 'ms_per_step': e2e_ms, 'h2d_bytes_per_step': h2d,
               'd2h_bytes_per_step': d2h,
               'api': 'lightcompress_b200.HostStagedGPTQ.block_opt' if args.workload == 'block' else 'lightcompress_b200.GPTQ',
               'overlap': ('copies on side streams; the parameters and activations of step s+1 are prefetched into '
                           'a second set of staging buffers while step s computes (not for the first step, none '
                           'after the last, which also waits for its results on the host: all copies lie inside '
                           'the timed region)') if args.workload == 'block' else 'none'}
    clocks = sampler.stop() if sampler else None

    # ---- parity of what was just timed, and agreement of the ranks ---------------------------------
    parity = None
    if not args.no_parity and args.workload in ('block', 'layer'):
        if args.workload == 'block':
            step()
        parity = parity_fn()
        if world > 1 and checksum_fn is not None:
            cs = checksum_fn()
            lo, hi = cs.clone(), cs.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX)
            parity['ranks_agree'] = bool(torch.equal(lo, hi))
            parity['ranks_checksum'] = 'sum of every deployed linear weight, min == max over the ranks'

    # ---- the other two headline kernels, timed alone (HBM-bound family 1) ----------------------
    aux = None
    if rank == 0 and args.workload == 'block':
        aux = rtn_aux(hbm_peak, dev)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel of ours: the Hessian GEMM -------------------------------
    # executed FLOPs = the 256x256 tiles on/above the diagonal that are actually issued (the kernel mirrors
    # them); algorithmic = 2 * tokens * C^2 per launch, the full square the reference computes
    n_l = sum(d[0] for d in hess.values())
    ms_l = sum(d[1] for d in hess.values())
    alg = sum(2.0 * d[2] * c * c for c, d in hess.items())
    exe = sum(2.0 * d[2] * 256 * 256 * n_super(c) for c, d in hess.items())
    achieved = exe / (ms_l * 1e-3) / 1e12
    roofline = {'bound': 'tensor', 'kernel': 'hessian_umma_kernel', 'achieved': achieved, 'peak': tf_sust,
                'unit': 'TFLOP/s', 'frac': achieved / tf_sust,
                'basis': 'executed FLOPs (tiles on and above the diagonal; the rest is mirrored)',
                'peak_kind': f'{peak_kind} sustained cuBLAS bf16 (of measured)',
                'achieved_algorithmic': alg / (ms_l * 1e-3) / 1e12,
                'launch_ms': ms_l / n_l, 'launches_per_step': n_l / args.steps,
                'share_of_step': ms_l / args.steps / ms_step,
                'per_cols': {str(c): {'launches_per_step': d[0] / args.steps, 'launch_ms': d[1] / d[0],
                                      'tokens_per_launch': d[2] / d[0]} for c, d in hess.items()},
                'traffic': None}
    # DRAM bytes per 16384-token launch: static figures from the ncu captures summarised under profiles/
    # (dram__bytes_read.sum + dram__bytes_write.sum of the same launch shapes), not measured in this run
    ncu_traffic = HESSIAN_NCU_TRAFFIC
    if all(c in ncu_traffic and abs(d[2] / d[0] - 16384) < 1 for c, d in hess.items()):
        roofline['traffic'] = sum(d[0] * ncu_traffic[c] for c, d in hess.items()) / n_l
        roofline['traffic_source'] = ('static: profiles/hessian_umma_C4096.md (ncu, per launch), weighted over the '
                                      'launch mix of the step')
        # X read once (bf16) + the 256 x 256 tiles on and above the diagonal of H read and written once (fp32)
        roofline['algorithmic_bytes'] = sum(d[0] * (2.0 * 16384 * c + 8.0 * 65536 * n_super(c))
                                            for c, d in hess.items()) / n_l

    line = {'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': world, 'steps': args.steps,
            'warmup': args.warmup, 'ms_per_step': ms_step, 'higher_is_better': True, 'scaling': 'strong',
            'vs_baseline': None, 'dtype': 'bf16 in / fp32 accumulate', 'data': 'synthetic',
            'config': dict({'workload': WORKLOADS[args.workload], 'name': args.workload,
                            'l2': 'inputs (2.1 GB of activations per step) exceed the 126 MB L2',
                            'sharding': f'{n_seq} sequences per rank; solve units (row ranges of a subset) dealt to the ranks',
                            'hessian_batch': HESSIAN_BATCH, 'calib_bs': args.calib_bs if args.workload == 'block' else 1,
                            'static_groups': bool(SPECIAL['static_groups'])}, **extra_cfg),
            'roofline': roofline, 'gpu_launches': launches * args.steps, 'clocks': clocks}
    if phase_ms:
        line['phases_ms'] = phase_ms
    if e2e:
        line['e2e'] = e2e
    if parity:
        line['parity'] = parity
    if args.workload in ('block', 'model'):
        line['fused_op_rejections'] = block_ops.rejected() + [('stage_plan', c) for c in runner.stage_plan_rejected]
    if aux:
        line['aux_kernels'] = aux
    if not args.no_cpu_baseline and world == 1:
        if args.workload == 'layer':
            v, desc, cores, parts = cpu_port_layer(8)
        else:
            v, desc, cores, parts, _ = cpu_port_block()
        line['cpu_baseline'] = dict({'value': v, 'unit': UNIT, 'cores': cores, 'kind': 'port', 'sample': desc,
                                     'extrapolated': True}, **parts)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    if line.get('fused_op_rejections'):
        raise SystemExit('a fused block op or the staged plan was rejected by its self-check: ' +
                         str(line['fused_op_rejections']))
    if parity and (parity['code_mismatch_perm_pinned'] >= 1e-3 or parity['recon_rel_diff'] >= 1e-2
                   or parity.get('ranks_agree') is False):
        raise SystemExit('parity of the timed configuration is outside its bars: ' + json.dumps(parity))


if __name__ == '__main__':
    main()
