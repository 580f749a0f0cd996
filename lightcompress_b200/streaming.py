"""GPTQ over decoder blocks that live in host memory: the block loop with its host <-> device traffic.

The reference keeps the model on the CPU and moves one block at a time to the GPU
(`block.cuda()` ... `block.cpu()` in BaseBlockwiseQuantization.block_opt,
llmc/compression/quantization/base_blockwise_quantization.py:403-432, driven by
BlockwiseOpt.run_block_loop, llmc/compression/blockwise_optimization.py:31-42).  `HostStagedGPTQ`
does the same job with the copies taken off the critical path:

  * parameters of a block cross PCIe once, on a copy stream, into one flat device buffer (two buffers
    alternate); in a process group rank 0 reads the host copy and one broadcast of the flat buffer
    hands it to the other ranks over NVLink;
  * calibration inputs that start on the host (the first block's) are copied chunk by chunk and the
    first stage of the schedule waits only for the chunk it is about to read;
  * while a block computes, the parameters of the next one are already on their way;
  * each subset's quantised weights go back to the host copy on a third stream as soon as the subset is
    solved, while the next stage computes; in a process group the linears are dealt to the ranks for
    this copy (every rank holds the same result).

`run_block_loop` chains the blocks: the outputs of block i stay on the device as the inputs of block
i + 1, exactly the tensors the reference stores in `self.input['data']`.
"""
import copy
import time

import torch
import torch.distributed as dist

from . import parallel
from .blockwise import GPTQBlockwise


def _is_pinned(t):
    return t.device.type == 'cpu' and t.is_pinned()


class HostStagedGPTQ:
    def __init__(self, runner: GPTQBlockwise, device, chunk=8):
        self.runner = runner
        self.dev = torch.device(device)
        self.chunk = chunk
        self.copy_in = torch.cuda.Stream(device=self.dev)
        self.copy_out = torch.cuda.Stream(device=self.dev)
        self.rank, self.world = parallel.world()
        self._flat = [None, None]          # flat parameter staging buffers
        self._slot = 0
        self._pending = None               # (slot, key, param event) of a prefetched block
        self._keep = None                  # device block whose device-to-host copies may still run
        self._pending_x = {}               # id of a prefetched input list -> (staged tensors, events)
        self._xbuf, self._xsig, self._xslot = [None, None], [None, None], 0    # input staging sets

    # ---- parameters ----------------------------------------------------------------------------
    def _layout(self, block_host):
        offs, n = [], 0
        for p in block_host.parameters():
            offs.append((n, p.numel(), p.dtype, tuple(p.shape)))
            n += (p.numel() + 7) // 8 * 8                  # 16-byte aligned views
        return offs, n

    def _start_param_copy(self, block_host, slot):
        """Host -> flat device buffer `slot` on the copy stream (rank 0 only); returns the event."""
        offs, n = self._layout(block_host)
        dt = next(block_host.parameters()).dtype
        if any(o[2] != dt for o in offs):
            raise NotImplementedError('a block with parameters of several dtypes')
        if self._flat[slot] is None or self._flat[slot].numel() < n or self._flat[slot].dtype != dt:
            self._flat[slot] = torch.empty(n, dtype=dt, device=self.dev)
        ev = None
        if self.rank == 0:
            # the buffer's previous readers (an earlier block's kernels on the compute stream) are done
            self.copy_in.wait_stream(torch.cuda.current_stream(self.dev))
            with torch.cuda.stream(self.copy_in):
                for (o, k, _, shape), p in zip(offs, block_host.parameters()):
                    self._flat[slot][o:o + k].view(shape).copy_(p.data, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.copy_in)
        return ev

    def prefetch(self, block_host):
        """Starts the parameter copy of the block that `block_opt` will be given next."""
        slot = 1 - self._slot
        self._pending = (slot, id(block_host), self._start_param_copy(block_host, slot))

    def _device_block(self, block_host):
        """A device copy of `block_host` whose parameters alias the flat staging buffer."""
        if self._pending is not None and self._pending[1] == id(block_host):
            slot, _, ev = self._pending
        else:
            slot = 1 - self._slot
            ev = self._start_param_copy(block_host, slot)
        self._pending = None
        self._slot = slot
        main = torch.cuda.current_stream(self.dev)
        if ev is not None:
            main.wait_event(ev)
        flat = self._flat[slot]
        if self.world > 1:
            dist.broadcast(flat, src=0)
        # structure only: the memo hands deepcopy an empty stand-in for every parameter, so no parameter
        # storage is copied on the host; then the views of the flat buffer are bound
        stand_ins = {id(p): torch.nn.Parameter(torch.empty(0, dtype=p.dtype), requires_grad=False)
                     for p in block_host.parameters()}
        block = copy.deepcopy(block_host, memo=stand_ins)
        offs, _ = self._layout(block_host)
        for (o, k, _, shape), p in zip(offs, block.parameters()):
            p.data = flat[o:o + k].view(shape)
        for name, buf in list(block.named_buffers()):
            if buf.device != self.dev:
                mod = block.get_submodule(name.rpartition('.')[0]) if '.' in name else block
                mod._buffers[name.rpartition('.')[2]] = buf.to(self.dev)
        return block

    # ---- inputs ----------------------------------------------------------------------------------
    def _stage_inputs(self, inputs):
        """inputs: list of tensors.  Host tensors are copied on the copy stream, in groups of `chunk`, into
        one of two persistent sets of staging tensors (allocated on first use, kept until release());
        returns (device tensors, events per tensor index or None)."""
        if all(t.is_cuda for t in inputs):
            return list(inputs), None
        main = torch.cuda.current_stream(self.dev)
        k = self._xslot = 1 - self._xslot
        sig = [(tuple(t.shape), t.dtype) for t in inputs]
        if self._xbuf[k] is None or self._xsig[k] != sig:
            self._xbuf[k] = [torch.empty(sh, dtype=dt, device=self.dev) for sh, dt in sig]
            self._xsig[k] = sig
        # the set's previous readers (the block before last) were enqueued on the compute stream earlier
        self.copy_in.wait_stream(main)
        out, evs = self._xbuf[k], []
        with torch.cuda.stream(self.copy_in):
            for i, t in enumerate(inputs):
                out[i].copy_(t, non_blocking=_is_pinned(t))
                if (i + 1) % self.chunk == 0 or i + 1 == len(inputs):
                    ev = torch.cuda.Event()
                    ev.record(self.copy_in)
                    evs.extend([ev] * (i + 1 - len(evs)))
        return list(out), evs

    def release(self):
        """Frees the staging buffers (inputs and parameters)."""
        self.finish()
        self._xbuf, self._xsig, self._flat = [None, None], [None, None], [None, None]
        self._pending, self._pending_x = None, {}

    def prefetch_inputs(self, inputs):
        """Starts copying host inputs that a later `block_opt` call will be given (the same list object)."""
        self._pending_x[id(inputs)] = (inputs, self._stage_inputs(inputs))

    # ---- one block ---------------------------------------------------------------------------------
    @torch.no_grad()
    def block_opt(self, block_host, inputs, kwargs, next_block_host=None, wait_results=True, out_host=None,
                  next_inputs=None):
        """Quantises `block_host` (a module in host memory; its linears' weights are overwritten with the
        fp32 error-compensated weights and get the buf_* buffers, like the reference's block after
        block.cpu()).  inputs: host or device tensors (this rank's sequences).  Returns the device
        tensors that feed the next block.  next_block_host: its parameters start copying before this
        block computes.  wait_results=False leaves the last device-to-host copies in flight (`finish()`
        waits for them).  out_host: {linear name: pinned fp32 tensor} to receive the compensated weights
        (allocating pinned memory per call is slow; a caller that loops over a model provides them).
        next_inputs: host inputs of the NEXT call (the same list object will be passed then): their copy
        is queued behind this call's own copies and overlaps this block's computation."""
        main = torch.cuda.current_stream(self.dev)
        block = self._device_block(block_host)
        pend = self._pending_x.pop(id(inputs), None)
        xs, evs = pend[1] if pend is not None else self._stage_inputs(inputs)
        if next_block_host is not None:
            self.prefetch(next_block_host)
        if next_inputs is not None:
            self.prefetch_inputs(next_inputs)
        host_mods = dict(block_host.named_modules())
        dev_mods = dict(block.named_modules())
        order = [n for n, m in block_host.named_modules() if isinstance(m, torch.nn.Linear)]

        def on_input(i):
            if evs is not None:
                main.wait_event(evs[i])

        def on_subset_done(names):
            done = torch.cuda.Event()
            done.record(main)
            self.copy_out.wait_event(done)
            with torch.cuda.stream(self.copy_out):
                for n in names:
                    if order.index(n) % self.world != self.rank:
                        continue                       # another rank returns this linear to its host copy
                    src, dst = block.get_submodule(n), host_mods[n]
                    w = src.weight.data
                    if out_host is not None and n in out_host:
                        dst.weight.data = out_host[n]
                    elif dst.weight.data.dtype != w.dtype or not _is_pinned(dst.weight.data):
                        dst.weight.data = torch.empty(w.shape, dtype=w.dtype, pin_memory=True)
                    dst.weight.data.copy_(w, non_blocking=True)
                    for k, b in src.named_buffers(recurse=False):
                        if k.startswith('buf_'):
                            hb = torch.empty(b.shape, dtype=b.dtype, pin_memory=True)
                            hb.copy_(b, non_blocking=True)
                            dst._buffers[k] = hb
        self.runner.on_input, self.runner.on_subset_done = on_input, on_subset_done
        try:
            outs = self.runner.block_opt(block, xs, kwargs)
        finally:
            self.runner.on_input = self.runner.on_subset_done = None
        del dev_mods
        self._keep = block                  # the copies above read from it
        if wait_results:
            self.finish()
        return outs

    def finish(self):
        """Waits (on the host) until every result copy issued so far has reached host memory."""
        self.copy_out.synchronize()
        self._keep = None

    # ---- the model ----------------------------------------------------------------------------------
    @torch.no_grad()
    def run_block_loop(self, blocks_host, first_inputs, kwargs, on_block_done=None, out_host=None):
        """BlockwiseOpt.run_block_loop (blockwise_optimization.py:31-42) for GPTQ: every block of
        `blocks_host` in order, the outputs of one feeding the next.  Returns (device outputs of the last
        block, seconds per block measured on the host after a device synchronisation)."""
        xs = first_inputs
        per_block = []
        for i, blk in enumerate(blocks_host):
            t0 = time.perf_counter()
            nxt = blocks_host[i + 1] if i + 1 < len(blocks_host) else None
            xs = self.block_opt(blk, xs, kwargs, next_block_host=nxt, wait_results=False,
                                out_host=None if out_host is None else out_host[i])
            if on_block_done is not None:
                on_block_done(i)
            torch.cuda.current_stream(self.dev).synchronize()
            per_block.append(time.perf_counter() - t0)
        self.finish()
        return xs, per_block
