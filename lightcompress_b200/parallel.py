"""Multi-GPU plumbing of the GPTQ path: which sequences and which weight rows a rank owns, the
one-per-layer Hessian reduction, and the gather of row-sharded results.

Device-agnostic torch.distributed code (NCCL on GPUs, gloo in the CPU tests); no kernels here.

The reference shards nothing but the calibration set (base_dataset.py:175-177) and all-reduces the
full Hessian after every add_batch call, dividing by the world size (gptq.py:292-295).  Here every
rank keeps the raw sum of X^T X of its own sequences; one all_reduce(SUM) per layer and the factor
2 / (total number of sequences) give the same matrix up to fp32 summation order.
"""
import torch
import torch.distributed as dist


def world():
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def sequence_shard(n_sequences, rank=None, world_size=None):
    """Contiguous, near-even split of the calibration sequences; returns (begin, end)."""
    r, w = world()
    rank = r if rank is None else rank
    world_size = w if world_size is None else world_size
    base, extra = divmod(n_sequences, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def row_shard(rows, rank=None, world_size=None, multiple=16):
    """Row range of a linear layer solved by this rank.  Rows are independent in the GPTQ solver
    (they share only the inverse-Hessian factor), so any split is valid; ranges are multiples of
    `multiple` rows (the solver's CTA granularity) except possibly the last."""
    r, w = world()
    rank = r if rank is None else rank
    world_size = w if world_size is None else world_size
    units = -(-rows // multiple)
    base, extra = divmod(units, world_size)
    b = (rank * base + min(rank, extra)) * multiple
    e = b + (base + (1 if rank < extra else 0)) * multiple
    return min(b, rows), min(e, rows)


def reduce_hessian(H_raw, n_sequences):
    """Sums the raw Hessians and the sequence counts over the ranks; returns (H_raw, total_n).
    The caller scales by 2 / total_n."""
    _, w = world()
    if w == 1:
        return H_raw, n_sequences
    dist.all_reduce(H_raw, op=dist.ReduceOp.SUM)
    nt = torch.tensor([n_sequences], dtype=torch.int64, device=H_raw.device)
    dist.all_reduce(nt, op=dist.ReduceOp.SUM)
    return H_raw, int(nt.item())


def gather_rows(piece, rows):
    """Concatenates row-sharded (r_i, ...) pieces of every rank in rank order into (rows, ...)."""
    rank, w = world()
    if w == 1:
        return piece
    shards = [row_shard(rows, r, w) for r in range(w)]
    sizes = [e - b for b, e in shards]
    if len(set(sizes)) == 1:
        out = torch.empty((rows,) + tuple(piece.shape[1:]), dtype=piece.dtype, device=piece.device)
        dist.all_gather_into_tensor(out, piece.contiguous())
        return out
    # uneven shards: pad every piece to the largest one (collectives want equal sizes), then trim
    mx = max(sizes)
    padded = torch.zeros((mx,) + tuple(piece.shape[1:]), dtype=piece.dtype, device=piece.device)
    padded[:piece.shape[0]] = piece
    out = torch.empty((w * mx,) + tuple(piece.shape[1:]), dtype=piece.dtype, device=piece.device)
    dist.all_gather_into_tensor(out, padded)
    return torch.cat([out[r * mx: r * mx + sizes[r]] for r in range(w)], dim=0)
