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


def reduce_hessian(H_raw, n_sequences, status=None):
    """Sums the raw Hessians and the sequence counts over the ranks; returns (H_raw, total_n, code).
    The caller scales by 2 / total_n, which is the Hessian of all sequences whatever the split; the
    reference's per-call all-reduce and division by the world size (gptq.py:292-295) equals it when
    every rank holds the same number of sequences (sequence_shard deals them that way when the count
    divides).  status: this rank's int32 device status word of the Hessian kernel (0 = ok, negative =
    error); `code` is the worst one over all ranks, so that every rank can raise together."""
    _, w = world()
    if w == 1:
        return H_raw, n_sequences, (0 if status is None else int(status.item()))
    dist.all_reduce(H_raw, op=dist.ReduceOp.SUM)
    # one small collective carries both: the count in slot 0, the number of failing ranks in slot 1 (formed on
    # the device from the status word: the host waits once, for the reduced pair)
    nt = torch.zeros(2, dtype=torch.int64, device=H_raw.device)
    nt[0] = n_sequences
    if status is not None:
        nt[1] = (status.reshape(-1)[0] != 0).to(torch.int64)
    dist.all_reduce(nt, op=dist.ReduceOp.SUM)
    total, failed = (int(v) for v in nt.tolist())
    if not failed:
        return H_raw, total, 0
    own = 0 if status is None else int(status.item())
    return H_raw, total, (own if own != 0 else LC_ERR_PEER)


LC_ERR_PEER = -8        # LC_ERR_CUDA: "a peer rank reported a device error"


def combine_status(words, how):
    """Element-wise min / max of an integer status vector over the ranks (all ranks pass the same length)."""
    _, w = world()
    if w > 1:
        dist.all_reduce(words, op=dist.ReduceOp.MIN if how == 'min' else dist.ReduceOp.MAX)
    return words


def sum_and_count(vec, count):
    """Sums a per-rank partial-sum vector and its element count over the ranks: (vec, total_count).
    AWQ statistics over token shards: sum |x| per channel with the token count, squared-error sums per
    grid point with the element count (the reference instead lets the rank with the lowest local loss win,
    awq.py:256-273; summing is what its single-rank run over all the data computes)."""
    _, w = world()
    if w == 1:
        return vec, count
    t = torch.cat([vec.reshape(-1).double(), torch.tensor([float(count)], dtype=torch.float64, device=vec.device)])
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return t[:-1].to(vec.dtype).reshape(vec.shape), int(round(float(t[-1].item())))


def average_over_ranks(t):
    """all_reduce(SUM) / world in the tensor's own dtype, in place: the clip thresholds of
    AutoClipper.run (auto_clip.py:72-76)."""
    _, w = world()
    if w > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        t /= w
    return t


def all_gather_packed(packed):
    """packed: (world, ...) contiguous, slot [rank] filled by this rank; on return every slot holds its
    rank's data.  One collective, in place."""
    rank, w = world()
    if w == 1:
        return packed
    assert packed.shape[0] == w and packed.is_contiguous()
    dist.all_gather_into_tensor(packed.view(-1), packed[rank].reshape(-1).clone())
    return packed


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
