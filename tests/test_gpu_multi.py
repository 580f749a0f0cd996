"""Two-GPU check of the sharded block schedule (NCCL): sequences split over the ranks, one Hessian
all-reduce per subset, solve units dealt to the ranks and broadcast.  Every rank must end with the
same quantised block, and it must match the single-GPU run up to the fp32 summation order of the
Hessian (bar: < 0.1 % differing codes per linear).  Skipped on boxes with one GPU."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, out_dir, extra=None):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE='0')
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    import copy
    from lightcompress_b200 import GPTQBlockwise, IntegerQuantizer, llama_subsets, parallel
    from tests.test_gpu_blockwise import _make_block, _to_cuda
    extra = dict(extra or {})
    block, xs, kwargs = _make_block(**extra.pop('_block', {}))
    b, e = parallel.sequence_shard(len(xs))
    wq = IntegerQuantizer(4, False, 'per_group', group_size=128)
    pins = os.path.join(out_dir, 'pins.pt')
    if os.path.exists(pins):
        # column orders of the single-GPU run: act-order near-ties must not decide the comparison
        extra['pinned_perms'] = {k: v.cuda() for k, v in torch.load(pins).items()}
    runner = GPTQBlockwise(wq, dict({'actorder': True, 'percdamp': 0.01, 'blocksize': 128, 'hessian_batch': 4}, **extra))
    gblock = copy.deepcopy(block).cuda()
    outs = runner.block_opt(gblock, [x.cuda() for x in xs[b:e]], _to_cuda(kwargs))
    torch.cuda.synchronize()
    state = {}
    for subset in llama_subsets(gblock):
        for name, (parent, attr) in subset.items():
            m = getattr(parent, attr)
            state[name] = {'weight': m.weight.cpu(), 'buf_scales': m.buf_scales.cpu(), 'buf_zeros': m.buf_zeros.cpu(),
                           'buf_perm': m.buf_perm.cpu(), 'tmp_weight': m.tmp_weight.cpu()}
    torch.save({'state': state, 'outs': [o.cpu() for o in outs], 'shard': (b, e)}, os.path.join(out_dir, f'r{rank}.pt'))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs two GPUs')
def test_two_rank_block_matches_single_gpu(tmp_path):
    import copy
    import torch.multiprocessing as mp
    from lightcompress_b200 import GPTQBlockwise, IntegerQuantizer, llama_subsets
    from oracle import gptq_ref
    from tests.test_gpu_blockwise import _make_block, _to_cuda
    port = 29700 + (os.getpid() % 200)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0 = torch.load(os.path.join(str(tmp_path), 'r0.pt'))
    r1 = torch.load(os.path.join(str(tmp_path), 'r1.pt'))
    assert r0['shard'] == (0, 8) and r1['shard'] == (8, 16)
    for name in r0['state']:
        for k in r0['state'][name]:
            assert torch.equal(r0['state'][name][k], r1['state'][name][k]), (name, k)   # ranks agree exactly

    block, xs, kwargs = _make_block()
    wq = IntegerQuantizer(4, False, 'per_group', group_size=128)
    runner = GPTQBlockwise(wq, {'actorder': True, 'percdamp': 0.01, 'blocksize': 128, 'hessian_batch': 4})
    gblock = copy.deepcopy(block).cuda()
    outs = runner.block_opt(gblock, [x.cuda() for x in xs], _to_cuda(kwargs))
    for subset in llama_subsets(gblock):
        for name, (parent, attr) in subset.items():
            m = getattr(parent, attr)
            one = {'weight': m.weight.cpu(), 'buf_scales': m.buf_scales.cpu(), 'buf_zeros': m.buf_zeros.cpu(),
                   'buf_perm': m.buf_perm.cpu()}
            two = r0['state'][name]
            R, C = one['weight'].shape
            a, b = torch.empty(R, C), torch.empty(R, C)
            a[:, one['buf_perm']] = gptq_ref.codes_permuted(one)
            b[:, two['buf_perm']] = gptq_ref.codes_permuted(two)
            mism = float((a != b).float().mean())
            print(f'{name}: 1-GPU vs 2-GPU code mismatch {mism:.4%}')
            assert mism < 1e-3, (name, mism)
    full = torch.cat([o.cpu() for o in outs]).float()
    both = torch.cat(r0['outs'] + r1['outs']).float()
    assert float((full - both).norm() / full.norm()) < 1e-2


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs two GPUs')
def test_two_rank_uneven_row_ranges(tmp_path):
    """A block whose stacked subsets hold an odd number of 128-row units (hidden 384: q/k/v 9 units, o 3,
    down 3), so the two ranks solve row ranges of different lengths and the packed gather pads the shorter
    one: the ranks agree exactly, and q/k/v -- same inputs as on one GPU -- match the single-GPU codes."""
    import copy
    import torch.multiprocessing as mp
    from lightcompress_b200 import GPTQBlockwise, IntegerQuantizer, llama_subsets
    from oracle import gptq_ref
    from tests.test_gpu_blockwise import _make_block, _to_cuda
    port = 29300 + (os.getpid() % 100)
    shape = {'hidden': 384, 'inter': 640, 'heads': 3, 'T': 256, 'n_seq': 16}
    block, xs, kwargs = _make_block(**shape)
    wq = IntegerQuantizer(4, False, 'per_group', group_size=128)
    runner = GPTQBlockwise(wq, {'actorder': True, 'percdamp': 0.01, 'blocksize': 128, 'hessian_batch': 4})
    gblock = copy.deepcopy(block).cuda()
    runner.block_opt(gblock, [x.cuda() for x in xs], _to_cuda(kwargs))
    torch.save({k: v.cpu() for k, v in runner.used_perms.items()}, os.path.join(str(tmp_path), 'pins.pt'))
    mp.spawn(_worker, args=(2, port, str(tmp_path), {'_block': shape}), nprocs=2, join=True)
    r0 = torch.load(os.path.join(str(tmp_path), 'r0.pt'))
    r1 = torch.load(os.path.join(str(tmp_path), 'r1.pt'))
    for name in r0['state']:
        for k in r0['state'][name]:
            assert torch.equal(r0['state'][name][k], r1['state'][name][k]), (name, k)
    for subset in llama_subsets(gblock):
        for name, (parent, attr) in subset.items():
            m = getattr(parent, attr)
            one = {'weight': m.weight.cpu(), 'buf_scales': m.buf_scales.cpu(), 'buf_zeros': m.buf_zeros.cpu(),
                   'buf_perm': m.buf_perm.cpu()}
            two = r0['state'][name]
            R, C = one['weight'].shape
            a, b = torch.empty(R, C), torch.empty(R, C)
            a[:, one['buf_perm']] = gptq_ref.codes_permuted(one)
            b[:, two['buf_perm']] = gptq_ref.codes_permuted(two)
            mism = float((a != b).float().mean())
            print(f'uneven {name} ({R} rows): 1-GPU vs 2-GPU code mismatch {mism:.4%}')
            if name in ('self_attn.q_proj', 'self_attn.k_proj', 'self_attn.v_proj'):
                assert mism < 1e-3, (name, mism)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs two GPUs')
def test_two_rank_static_groups_block_matches_single_gpu(tmp_path):
    """static_groups through the row-sharded solve: the ranks agree exactly, the buffers are every
    linear's round-to-nearest ones, and with every subset's column order pinned to the single-GPU run's
    (near-equal Hessian diagonals of this small random block would otherwise sort differently after the
    all-reduce changes the last bits) fewer than 0.1 % of the deployed weights differ, linear by linear, or
    three times what another summation order of the Hessian changes on one GPU."""
    import copy
    import torch.multiprocessing as mp
    from lightcompress_b200 import GPTQBlockwise, IntegerQuantizer
    from tests.test_gpu_blockwise import _make_block, _to_cuda
    port = 29900 + (os.getpid() % 100)
    # 32 sequences of 384 tokens: 24 tokens per column of the widest linear, a well-conditioned Hessian
    shape = {'T': 384, 'n_seq': 32}
    extra = {'static_groups': True}
    block, xs, kwargs = _make_block(**shape)
    wq = IntegerQuantizer(4, False, 'per_group', group_size=128)
    runner = GPTQBlockwise(wq, dict({'actorder': True, 'percdamp': 0.01, 'blocksize': 128, 'hessian_batch': 4}, **extra))
    gblock = copy.deepcopy(block).cuda()
    outs = runner.block_opt(gblock, [x.cuda() for x in xs], _to_cuda(kwargs))
    torch.save({k: v.cpu() for k, v in runner.used_perms.items()}, os.path.join(str(tmp_path), 'pins.pt'))
    # noise floor: the same single-GPU run with the Hessians summed in another order (every launch's tokens
    # accumulated in two parts that meet in fp32 atomics, as two ranks' partial sums meet in the all-reduce)
    # and the same pinned column orders.  o_proj and down_proj see Hessians of nearly rank-deficient
    # activations, where the last bits of H already move some roundings
    runner8 = GPTQBlockwise(wq, dict({'actorder': True, 'percdamp': 0.01, 'blocksize': 128, 'hessian_batch': 4,
                                      'hessian_ksplit': 2}, **extra))
    runner8.pinned_perms = {k: v.clone() for k, v in runner.used_perms.items()}
    gblock8 = copy.deepcopy(block).cuda()
    runner8.block_opt(gblock8, [x.cuda() for x in xs], _to_cuda(kwargs))
    floor = {n: float((m.tmp_weight != dict(gblock.named_modules())[n].tmp_weight).float().mean())
             for n, m in gblock8.named_modules() if hasattr(m, 'tmp_weight')}
    mp.spawn(_worker, args=(2, port, str(tmp_path), dict(extra, _block=shape)), nprocs=2, join=True)
    r0 = torch.load(os.path.join(str(tmp_path), 'r0.pt'))
    r1 = torch.load(os.path.join(str(tmp_path), 'r1.pt'))
    for name in r0['state']:
        for k in r0['state'][name]:
            assert torch.equal(r0['state'][name][k], r1['state'][name][k]), (name, k)
        assert r0['state'][name]['buf_scales'].dtype == torch.bfloat16
    for name, m in gblock.named_modules():
        if name in r0['state']:
            assert torch.equal(m.buf_scales.cpu(), r0['state'][name]['buf_scales']), name
            mism = float((m.tmp_weight.cpu() != r0['state'][name]['tmp_weight']).float().mean())
            print(f'{name}: 1-GPU vs 2-GPU deployed weights differing {mism:.4%} '
                  f'(single GPU, other summation order: {floor[name]:.4%})')
            assert mism < max(1e-3, 3 * floor[name]), (name, mism, floor[name])
    full = torch.cat([o.cpu() for o in outs]).float()
    both = torch.cat(r0['outs'] + r1['outs']).float()
    assert float((full - both).norm() / full.norm()) < 1e-2


def _inverse_worker(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE='0')
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    from lightcompress_b200 import GPTQ, IntegerQuantizer
    wq = IntegerQuantizer(4, False, 'per_group', group_size=128)
    res = {}
    for n in (384, 1152):
        g = torch.Generator().manual_seed(n)
        X = torch.randn(3 * n, n, generator=g)
        H = (X.t() @ X).cuda()
        shared = GPTQ(wq, {'actorder': True, 'percdamp': 0.01, 'shared_inverse': True, 'shared_inverse_min': 256})
        alone = GPTQ(wq, {'actorder': True, 'percdamp': 0.01, 'shared_inverse': False})
        a, b = shared.factorize(H, 2.0 / 3), alone.factorize(H, 2.0 / 3)
        shared.check_status()
        alone.check_status()
        res[n] = (a['U'].cpu(), b['U'].cpu())
    torch.save(res, os.path.join(out_dir, f'inv{rank}.pt'))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs two GPUs')
def test_shared_triangular_inverse_equals_the_single_rank_one(tmp_path):
    """The triangular inverse with its top-level block split over the ranks and exchanged: every rank
    ends with the U it computes alone, bit for bit (skipping zero blocks of a triangular operand and
    slicing the output columns do not change any sum)."""
    import torch.multiprocessing as mp
    port = 29300 + (os.getpid() % 200)
    mp.spawn(_inverse_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0 = torch.load(os.path.join(str(tmp_path), 'inv0.pt'))
    r1 = torch.load(os.path.join(str(tmp_path), 'inv1.pt'))
    for n in r0:
        assert torch.equal(r0[n][0], r0[n][1]), n
        assert torch.equal(r1[n][0], r0[n][0]), n
        assert torch.equal(r0[n][0], torch.triu(r0[n][0]))


def _moe_worker(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE='0')
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    from lightcompress_b200.moe_fp8 import Fp8FakeQuantMoE
    layer = Fp8FakeQuantMoE(hidden=512, inter=256, n_experts=16, n_shared=2, top_k=4, seed=5200,
                            device=torch.device('cuda', rank))
    assert (layer.e0, layer.e1) == (8 * rank, 8 * rank + 8) and layer.has_shared == (rank == 0)
    g = torch.Generator().manual_seed(5201)
    x = torch.randn(1500, 512, generator=g).to(torch.bfloat16).cuda()
    layer.quantize_weights()
    y = layer.forward(x)
    torch.cuda.synchronize()
    torch.save(y.cpu(), os.path.join(out_dir, f'moe{rank}.pt'))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs two GPUs')
def test_two_rank_expert_sharded_moe_matches_the_oracle(tmp_path):
    """The FP8 fake-quantised MoE layer with its experts split over two ranks (8 routed experts each, the
    shared experts on rank 0, one all-reduce of the output): both ranks end with the same output, equal to
    the oracle's on one GPU up to the order of the bf16-rounded expert sums."""
    import torch.multiprocessing as mp
    from lightcompress_b200.moe_fp8 import Fp8FakeQuantMoE
    from oracle import moe_fp8_ref
    port = 29400 + (os.getpid() % 200)
    mp.spawn(_moe_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    y0 = torch.load(os.path.join(str(tmp_path), 'moe0.pt'))
    y1 = torch.load(os.path.join(str(tmp_path), 'moe1.pt'))
    assert torch.equal(y0, y1)
    layer = Fp8FakeQuantMoE(hidden=512, inter=256, n_experts=16, n_shared=2, top_k=4, seed=5200)
    raw = {k: getattr(layer, k).clone() for k in ('gate', 'w_gate', 'w_up', 'w_down', 's_gate', 's_up', 's_down')}
    g = torch.Generator().manual_seed(5201)
    x = torch.randn(1500, 512, generator=g).to(torch.bfloat16).cuda()
    ref = moe_fp8_ref.moe_forward(x, raw['gate'], raw['w_gate'], raw['w_up'], raw['w_down'], raw['s_gate'],
                                  raw['s_up'], raw['s_down'], 4)
    rel = float((y0.float() - ref.cpu().float()).norm() / ref.cpu().float().norm())
    print(f'two-rank MoE vs oracle: rel diff {rel:.2e}')
    assert rel < 3e-3


def _awq_worker(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE='0')
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    import copy
    from lightcompress_b200 import Awq, IntegerQuantizer
    from tests.test_gpu_blockwise import _make_block, _to_cuda
    block, xs, kwargs = _make_block(hidden=512, inter=1024, heads=4, T=128, n_seq=8, seed=11)
    x = torch.cat(xs)                                  # one calibration batch; every rank takes half of it
    half = x.shape[0] // world
    awq = Awq(IntegerQuantizer(4, False, 'per_group', group_size=128),
              {'trans': True, 'trans_version': 'v2', 'weight_clip': True, 'clip_version': 'v1'}, calib_seq_len=128)
    gblock = copy.deepcopy(block).cuda()
    rep = awq.block_transform(gblock, x[rank * half:(rank + 1) * half].cuda(), _to_cuda(kwargs))
    torch.cuda.synchronize()
    torch.save({'params': {n: p.data.cpu() for n, p in gblock.named_parameters()},
                'scales': {k: v.cpu() for k, v in rep['scales'].items()},
                'losses': {k: torch.as_tensor(v).float().cpu() for k, v in rep['losses'].items()}},
               os.path.join(out_dir, f'awq{rank}.pt'))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs two GPUs')
def test_two_rank_awq_matches_single_gpu(tmp_path):
    """AWQ with the calibration batch split over two ranks (summed |x| statistics, summed candidate
    losses, averaged clip thresholds; awq.py:256-273, auto_clip.py:72-76): both ranks end with the same
    block, the chosen scales equal the single-GPU run's on the whole batch up to the rounding of the
    reduced statistics, and the transformed weights differ in fewer than 1 % of their elements (the clip
    thresholds of two half batches are averaged, which is not the threshold of the whole batch)."""
    import copy
    import torch.multiprocessing as mp
    from lightcompress_b200 import Awq, IntegerQuantizer
    from tests.test_gpu_blockwise import _make_block, _to_cuda
    port = 29500 + (os.getpid() % 100)
    mp.spawn(_awq_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0 = torch.load(os.path.join(str(tmp_path), 'awq0.pt'))
    r1 = torch.load(os.path.join(str(tmp_path), 'awq1.pt'))
    for n in r0['params']:
        assert torch.equal(r0['params'][n], r1['params'][n]), n
    block, xs, kwargs = _make_block(hidden=512, inter=1024, heads=4, T=128, n_seq=8, seed=11)
    awq = Awq(IntegerQuantizer(4, False, 'per_group', group_size=128),
              {'trans': True, 'trans_version': 'v2', 'weight_clip': True, 'clip_version': 'v1'}, calib_seq_len=128)
    gblock = copy.deepcopy(block).cuda()
    rep = awq.block_transform(gblock, torch.cat(xs).cuda(), _to_cuda(kwargs))
    same_choice = True
    for k, s in rep['scales'].items():
        l1, l2 = torch.as_tensor(rep['losses'][k]).float().cpu(), r0['losses'][k]
        lrel = float((l1 - l2).abs().max() / l1.abs().max())
        i1, i2 = int(l1.argmin()), int(l2.argmin())
        print(f'awq {k}: candidate losses differ by {lrel:.2e} (relative), chosen grid point {i1} / {i2}')
        # the mean of two half-batch means is the whole batch's mean up to rounding
        assert lrel < 2e-2, (k, lrel)
        if i1 == i2:
            rel = float((s.cpu().float() - r0['scales'][k].float()).abs().max() / s.float().abs().max())
            assert rel < 2e-2, (k, rel)
        else:
            same_choice = False
            assert abs(float(l1[i1] - l1[i2])) <= 2e-2 * float(l1[i1]), (k, i1, i2)      # a near tie
    if same_choice:
        for n, p in gblock.named_parameters():
            rel = float((p.data.cpu().float() - r0['params'][n].float()).norm() / p.data.float().norm())
            print(f'awq {n}: relative difference 1 GPU vs 2 GPUs {rel:.2e}')
            assert rel < 3e-2, (n, rel)
