"""World-size-2 gloo test of the multi-GPU orchestration on CPU: sequence sharding + one Hessian
reduction gives the Hessian the reference accumulates on all sequences, and row-sharded solves
gathered in rank order equal the un-sharded solve.  The solver stand-in is the CPU oracle: this
test covers the host logic only (the kernels need a GPU)."""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import gptq_ref


def _worker(rank, world_size, port, out_dir):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world_size))
    dist.init_process_group('gloo', rank=rank, world_size=world_size)
    torch.set_num_threads(1)
    from lightcompress_b200 import parallel
    g = torch.Generator().manual_seed(4000)
    R, C, ns, T = 48, 256, 6, 96
    W = (torch.randn(R, C, generator=g) * 0.02).to(torch.bfloat16)
    X = torch.randn(ns, T, C, generator=g).to(torch.bfloat16)
    b, e = parallel.sequence_shard(ns)
    H = torch.zeros(C, C)
    for i in range(b, e):
        x = X[i].float()
        H += x.t() @ x
    H, n, code = parallel.reduce_hessian(H, e - b)
    assert code == 0
    assert n == ns
    H = H * (2.0 / n)
    r0, r1 = parallel.row_shard(R)
    res = gptq_ref.quantize_layer(W[r0:r1], H)
    full = parallel.gather_rows(res['weight'], R)
    if rank == 0:
        torch.save({'H': H, 'weight': full, 'shards': [parallel.row_shard(R, r, world_size) for r in range(world_size)]},
                   os.path.join(out_dir, 'out.pt'))
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_hessian_and_row_sharded_solve(tmp_path):
    port = 29500 + (os.getpid() % 400)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    out = torch.load(os.path.join(str(tmp_path), 'out.pt'))
    g = torch.Generator().manual_seed(4000)
    R, C, ns, T = 48, 256, 6, 96
    W = (torch.randn(R, C, generator=g) * 0.02).to(torch.bfloat16)
    X = torch.randn(ns, T, C, generator=g).to(torch.bfloat16)
    st = gptq_ref.hessian_init(C)
    for i in range(ns):
        gptq_ref.add_batch(st, X[i:i + 1])
    assert float((out['H'] - st['H']).abs().max() / st['H'].abs().max()) < 1e-5
    assert out['shards'] == [(0, 32), (32, 48)]
    ref = gptq_ref.quantize_layer(W, out['H'])
    # rows are independent given the same H; the CPU GEMM blocks a 32-row and a 48-row problem
    # differently, so allow fp32 summation-order noise
    assert torch.allclose(out['weight'], ref['weight'], rtol=1e-4, atol=1e-6)


def test_shard_arithmetic():
    from lightcompress_b200 import parallel
    assert [parallel.sequence_shard(128, r, 8) for r in range(8)] == [(16 * r, 16 * r + 16) for r in range(8)]
    assert [parallel.sequence_shard(10, r, 4) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    cover = [parallel.row_shard(11008, r, 8) for r in range(8)]
    assert cover[0][0] == 0 and cover[-1][1] == 11008
    assert all(a[1] == b[0] for a, b in zip(cover, cover[1:]))
    assert all((e - b) % 16 == 0 for b, e in cover)
    assert parallel.row_shard(40, 3, 4) == (40, 40)       # more ranks than row units: empty tail shard


def _status_worker(rank, world_size, port, out_dir):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world_size))
    dist.init_process_group('gloo', rank=rank, world_size=world_size)
    from lightcompress_b200 import parallel
    # rank 1's Hessian kernel "timed out" (status word set on the host): both ranks must learn of it in
    # the same reduction, so that neither goes on into the next collective alone
    H = torch.ones(4, 4) * (rank + 1)
    status = torch.tensor([-7 if rank == 1 else 0], dtype=torch.int32)
    H, n, code = parallel.reduce_hessian(H, 3, status)
    words = parallel.combine_status(torch.tensor([0, -6 if rank == 0 else 0], dtype=torch.int32), 'min')
    # the packed all-gather of the row-sharded solve: slot r filled by rank r
    packed = torch.zeros(world_size, 3, 5)
    packed[rank] = rank + 1
    parallel.all_gather_packed(packed)
    # AWQ over token shards: sums of |x| / of squared errors with their counts; averaged clip thresholds
    sums, cnt = parallel.sum_and_count(torch.tensor([1.0, 2.0, 3.0]) * (rank + 1), 10 * (rank + 1))
    avg = parallel.average_over_ranks(torch.tensor([2.0, 4.0]) * (rank + 1))
    torch.save({'H': H, 'n': n, 'code': code, 'words': words, 'packed': packed, 'sums': sums, 'cnt': cnt, 'avg': avg},
               os.path.join(out_dir, f's{rank}.pt'))
    dist.barrier()
    dist.destroy_process_group()


def test_a_failed_rank_is_seen_by_every_rank(tmp_path):
    from lightcompress_b200 import parallel
    port = 29100 + (os.getpid() % 400)
    mp.spawn(_status_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0 = torch.load(os.path.join(str(tmp_path), 's0.pt'))
    r1 = torch.load(os.path.join(str(tmp_path), 's1.pt'))
    assert r0['n'] == r1['n'] == 6 and torch.equal(r0['H'], torch.full((4, 4), 3.0))
    assert r1['code'] == -7                       # the failing rank reports its own code
    assert r0['code'] == parallel.LC_ERR_PEER     # its peer is told that some rank failed
    assert r0['words'].tolist() == r1['words'].tolist() == [0, -6]
    want = torch.stack([torch.full((3, 5), 1.0), torch.full((3, 5), 2.0)])
    assert torch.equal(r0['packed'], want) and torch.equal(r1['packed'], want)
    for r in (r0, r1):
        assert torch.equal(r['sums'], torch.tensor([3.0, 6.0, 9.0])) and r['cnt'] == 30
        assert torch.equal(r['avg'], torch.tensor([3.0, 6.0]))
