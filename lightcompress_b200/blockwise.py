"""Block-level driver of the GPTQ hot path: one decoder block through the reference's schedule.

Mirrors, for the GPTQ algorithm, what BaseBlockwiseQuantization does per block
(llmc/compression/quantization/base_blockwise_quantization.py: block_opt :403-432, run :447-485,
block_transform :487-527, rehook_next_subset :529-549, block_forward :378-401) with the subsets of
the Llama adapter (llmc/models/llama.py:52-91):

    hook the linears -> forward all calibration sequences (Hessians accumulate in the hooks)
    for each subset [q,k,v] -> [o] -> [gate,up] -> [down]:
        quantise its linears (GPTQ.layer_transform)
        true_sequential: swap them for fake-quant linears, hook the next subset, forward again
    quant_out: forward once more through the fully fake-quantised block -> inputs of the next block

Two schedule differences that do not change any result:
  * the linears of a subset read the same tensor, so one Hessian is accumulated per subset and
    shared (the reference accumulates identical copies, gptq.py:247-251, :298-308);
  * with true_sequential the first pass only hooks the first subset: the Hessians of later subsets
    collected in that pass are re-zeroed by subset_init before use (gptq.py:311-315).

For blocks with the Llama layout (pre-norm attention + gated MLP) the same schedule runs as a
staged plan: the tensor each re-forward would recompute up to the next subset's input is kept from
the previous stage (attention context, post-attention residual, MLP product), so the block's GEMMs
and its attention are evaluated once instead of up to five times.  The modules and their order are
those of the block's own forward, so every tensor is bit-identical to the re-forwarded one.

Several ranks: each rank forwards its own sequences; every Hessian is all-reduced once; the
(linear, row-range) solve units of a subset are dealt round-robin to the ranks and the results
broadcast, so every rank continues with identical weights.
"""
import contextlib
from collections import OrderedDict

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from . import block_ops, parallel
from .gptq import GPTQ


class FakeQuantLinear(nn.Module):
    """Replacement linear used for the re-forwards (module_utils.py:679-771): keeps the fp32
    compensated weight and the buf_* buffers, computes the fake-quantised weight once."""

    def __init__(self, module, w_qdq):
        super().__init__()
        self.register_buffer('weight', module.weight.data)
        self.bias = None if getattr(module, 'bias', None) is None else module.bias.data
        for name, buf in module.named_buffers():
            if name.startswith('buf_'):
                self.register_buffer(name, buf.data)
        self.w_qdq = w_qdq
        self.in_features, self.out_features = module.in_features, module.out_features
        # the solver's codes of this very weight tensor (GPTQ._install): the deploy-time weight is then
        # one dequantise + un-permute kernel instead of the gather / fake quant / gather chain
        self._lc_codes = getattr(module, '_lc_codes', None)

    def forward(self, x):
        if not hasattr(self, 'tmp_weight'):
            self.register_buffer('tmp_weight', self.w_qdq(self), persistent=False)
        return F.linear(x, self.tmp_weight, self.bias)


def llama_subsets(block):
    """The four GPTQ subsets of a Llama decoder block (llmc/models/llama.py:52-91), as
    (parent module, attribute name) pairs so that modules can be swapped."""
    a, m = block.self_attn, block.mlp
    return [
        OrderedDict([('self_attn.q_proj', (a, 'q_proj')), ('self_attn.k_proj', (a, 'k_proj')),
                     ('self_attn.v_proj', (a, 'v_proj'))]),
        OrderedDict([('self_attn.o_proj', (a, 'o_proj'))]),
        OrderedDict([('mlp.gate_proj', (m, 'gate_proj')), ('mlp.up_proj', (m, 'up_proj'))]),
        OrderedDict([('mlp.down_proj', (m, 'down_proj'))]),
    ]


def is_llama_layout(block):
    a, m = getattr(block, 'self_attn', None), getattr(block, 'mlp', None)
    return (a is not None and m is not None and hasattr(block, 'input_layernorm')
            and hasattr(block, 'post_attention_layernorm')
            and all(hasattr(a, k) for k in ('q_proj', 'k_proj', 'v_proj', 'o_proj'))
            and all(hasattr(m, k) for k in ('gate_proj', 'up_proj', 'down_proj', 'act_fn')))


class PhaseTimer:
    """Optional split of a block step into its phases, by CUDA events on the launching stream.  A phase's
    time is the span between its first and last kernel on the device timeline, so time the device spends
    waiting for the host between phases shows up as the remainder of the step, not inside a phase."""

    def __init__(self):
        self.on = False
        self.spans = []

    @contextlib.contextmanager
    def __call__(self, name):
        if not self.on:
            yield
            return
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        try:
            yield
        finally:
            e1.record()
            self.spans.append((name, e0, e1))

    def summary(self):
        """{phase: total ms}; call after a device synchronisation.  Clears the record."""
        out = {}
        for name, e0, e1 in self.spans:
            out[name] = out.get(name, 0.0) + e0.elapsed_time(e1)
        self.spans = []
        return out


class _StopForward(Exception):
    """Raised by a Hessian hook once the tensor it needs has been seen (see early_exit)."""


_stage_checked = {}


class GPTQBlockwise:
    def __init__(self, wquantizer, special=None, model_dtype=torch.bfloat16, quant_out=True, solver=None,
                 fake_linear=None):
        """solver: an existing lightcompress_b200.GPTQ to drive (default: a new one from `special`).
        fake_linear: callable(module) -> replacement module for a quantised linear (default:
        FakeQuantLinear of this file); the plugin passes the reference's own FakeQuantLinear.new so that
        the block is left exactly as the reference leaves it."""
        special = dict(special or {})
        self.solver = solver if solver is not None else GPTQ(wquantizer, special, model_dtype)
        self.wquantizer = wquantizer
        self.quant_out = quant_out
        self.fake_linear = fake_linear or (lambda mod: FakeQuantLinear(
            mod, lambda m: self.solver.w_qdq(m, self.wquantizer)))
        # block classes whose staged forward did not reproduce the block's own forward (they run the
        # generic re-forwarding schedule): visible to callers, nothing is skipped silently
        self.stage_plan_rejected = []
        self.phases = PhaseTimer()
        # {first linear of a subset: column order}: fixes the act-order permutation of that subset instead
        # of argsort(diag H), whose order among near-equal entries is implementation-defined (gptq.py:63
        # uses an unstable sort).  For reproducing an earlier run or comparing two implementations.
        self.pinned_perms = dict(special.get('pinned_perms') or {})
        self.used_perms = {}     # {first linear of a subset: the column order its solve used} of the last block
        self.true_sequential = self.solver.true_sequential
        # A re-forward whose only purpose is to feed the hooks of one subset stops as soon as that
        # subset's input has been seen: the rest of the block computes values nobody reads.
        self.early_exit = special.get('early_exit', True)
        self.stage_plan = special.get('stage_plan', True)
        # staged schedule only: RMS norm, rotary embedding and gated activation as one kernel each
        # (bit-identical to the block's stock tensor ops, checked on random data before first use)
        self.fused_block_ops = special.get('fused_block_ops', True)
        self.forward_passes = 0
        # optional callbacks for callers that stream a block through the GPU: on_input(i) runs before
        # the i-th input is first read (e.g. wait for its host-to-device copy), on_subset_done(names)
        # right after a subset's linears were quantised (e.g. start copying them back)
        self.on_input = None
        self.on_subset_done = None

    # ---- forwards ----------------------------------------------------------------------------
    @torch.no_grad()
    def block_forward(self, block, inputs, kwargs, need_output=True):
        self.forward_passes += 1
        outs = []
        for i, x in enumerate(inputs):
            if self.on_input is not None and self.forward_passes == 1:
                self.on_input(i)
            try:
                out = block(x, **(kwargs[i] if isinstance(kwargs, (list, tuple)) else kwargs))
            except _StopForward:
                continue
            if need_output:
                outs.append(out[0] if isinstance(out, tuple) else out)
        return outs

    def _init_subset(self, subset):
        names = list(subset)
        self.solver.layer_init(getattr(*subset[names[0]]), names[0])
        for n in names[1:]:
            self.solver.layers_cache[n] = self.solver.layers_cache[names[0]]
        return names[0], getattr(*subset[names[0]])

    def _hook_subset(self, subset, stop=False):
        """One Hessian per subset: hook the linear of the subset that the block calls first, alias
        the state for the others.  With stop=True the forward of each sequence ends there."""
        names = list(subset)
        first = names[0]
        parent, attr = subset[first]
        layer = getattr(parent, attr)
        self.solver.layer_init(layer, first)
        for n in names[1:]:
            self.solver.layers_cache[n] = self.solver.layers_cache[first]

        if stop:
            # pre-hook: the layer itself (and everything after it) is skipped for this sequence
            def pre_hook(mod, args):
                self.solver.add_batch(mod, first, args[0].data, None)
                raise _StopForward()
            return layer.register_forward_pre_hook(pre_hook)

        def hook(mod, inp, out):
            self.solver.add_batch(mod, first, inp[0].data, None)
        return layer.register_forward_hook(hook)

    # ---- one subset --------------------------------------------------------------------------
    @torch.no_grad()
    def subset_transform(self, subset):
        rank, world = parallel.world()
        names = list(subset)
        layers = [getattr(*subset[n]) for n in names]
        with self.phases('hessian_reduce'):
            H, hscale = self.solver._finish_hessian(names[0])
        # owq: linears with different outlier counts order the columns differently; each count gets its
        # own factor (the reference's n_outs are equal within every Llama subset: one factor as usual)
        by_n_out = OrderedDict()
        for layer, n in zip(layers, names):
            by_n_out.setdefault(self.solver.n_out_of(n), []).append(layer)
        for n_out, group in by_n_out.items():
            fac = self._solve_group(group, H, hscale, n_out, rank, world, self.pinned_perms.get(names[0]))
            self.used_perms[names[0]] = fac['perm']
        for n in names:
            self.solver.layers_cache.pop(n, None)
        if self.on_subset_done is not None:
            self.on_subset_done(names)

    def _solve_group(self, layers, H, hscale, n_out, rank, world, perm=None):
        with self.phases('factorize'):
            fac = self.solver.factorize(H, hscale, perm=perm, n_out=n_out)   # shared by the linears of the group
        # The rows of all linears of a subset are independent given the shared factor: they are solved
        # as one stacked matrix (q/k/v: 12288 rows, gate/up: 22016), which cuts the number of latency-bound
        # 128-column steps by the number of linears; in a process group every rank takes a row range.
        stacked = layers[0].weight.data if len(layers) == 1 else torch.cat([l.weight.data for l in layers], 0)
        static = None
        if self.solver.uses_static():
            # static groups: the layers' own round-to-nearest buffers, stacked like the rows
            parts = [self.solver.static_qparams(l) for l in layers]
            static = (torch.cat([p[0] for p in parts], 0),
                      None if parts[0][1] is None else torch.cat([p[1] for p in parts], 0))
        if world == 1:
            with self.phases('solve'):
                res = self.solver.solve(stacked, H, hscale, factor=fac, static=static)
        else:
            res = self._sharded_solve(stacked, fac, rank, world, static)
        n_groups = res['buf_scales'].shape[0] // stacked.shape[0]      # qparams per row (1 for per_channel)
        r0 = 0
        for layer in layers:
            r1 = r0 + layer.weight.shape[0]
            part = {'weight': res['weight'][r0:r1], 'buf_scales': res['buf_scales'][r0 * n_groups:r1 * n_groups],
                    'buf_zeros': None if res['buf_zeros'] is None else res['buf_zeros'][r0 * n_groups:r1 * n_groups],
                    'buf_perm': res['buf_perm'], 'buf_invperm': res['buf_invperm'],
                    'buf_n_nonout': res.get('buf_n_nonout'), 'static': res.get('static')}
            if res.get('codes_perm') is not None:
                part['codes_perm'] = res['codes_perm'][r0:r1]
            self.solver._install(layer, part)
            r0 = r1
        return fac

    def _sharded_solve(self, stacked, fac, rank, world, static=None):
        """Row range `rank` of the stacked weight solved here, then ONE all-gather per subset: every
        rank packs its rows as [compensated weight | scales | zeros | codes] into one fp32 buffer (row
        ranges are padded to the longest), and unpacks the gathered buffer.  Every rank returns the
        same full result."""
        H = fac['H']
        R, C = stacked.shape
        n_groups = (C + 127) // 128
        dev = H.device
        sym = self.wquantizer.sym
        # row ranges in multiples of 128 rows (whole CTAs of the in-block kernel), as even as possible
        blocks = (R + 127) // 128
        bounds = [min(R, 128 * ((blocks * r) // world)) for r in range(world)] + [R]
        a, b = bounds[rank], bounds[rank + 1]
        with self.phases('solve'):
            mine = self.solver.solve(stacked, H, rows=(a, b), factor=fac, static=static) if b > a else None
        # packed row: C weight floats, then (unless static: the qparams are inputs every rank holds)
        # n_groups scales and n_groups zeros, then the uint8 codes viewed as C / 4 floats
        with_codes = C % 4 == 0 and bool(self.solver.emit_codes)      # the same on every rank
        n_q = 0 if static is not None else n_groups
        off_s, off_z = C, C + n_q
        off_c = off_z + (0 if sym else n_q)
        row_len = off_c + (C // 4 if with_codes else 0)
        max_rows = max(bounds[r + 1] - bounds[r] for r in range(world))
        with self.phases('gather'):
            return self._gather_solved(mine, bounds, rank, world, R, C, n_q, sym, off_s, off_z, off_c, row_len,
                                       max_rows, with_codes, static, fac, dev)

    def _gather_solved(self, mine, bounds, rank, world, R, C, n_q, sym, off_s, off_z, off_c, row_len, max_rows,
                       with_codes, static, fac, dev):
        a, b = bounds[rank], bounds[rank + 1]
        packed = torch.empty((world, max_rows, row_len), dtype=torch.float32, device=dev)
        slot = packed[rank]
        if mine is not None:
            n = b - a
            slot[:n, :C].copy_(mine['weight'])
            if n_q:
                slot[:n, off_s:off_s + n_q].copy_(mine['buf_scales'].view(n, n_q))
                if not sym:
                    slot[:n, off_z:off_z + n_q].copy_(mine['buf_zeros'].view(n, n_q))
            if with_codes:
                slot[:n, off_c:].view(torch.uint8).copy_(mine['codes_perm'])
        parallel.all_gather_packed(packed)
        if world * max_rows == R:
            rows = packed.view(R, row_len)                 # even row ranges: the gathered buffer is the result
        else:
            pieces = [packed[r, :bounds[r + 1] - bounds[r]] for r in range(world) if bounds[r + 1] > bounds[r]]
            rows = pieces[0] if len(pieces) == 1 else torch.cat(pieces, 0)       # (R, row_len)
        full = {'weight': rows[:, :C].contiguous(),
                # every rank computes the same permutation from the same (reduced) Hessian
                'buf_perm': fac['perm'], 'buf_invperm': fac['invperm'], 'buf_zeros': None}
        if n_q:
            full['buf_scales'] = rows[:, off_s:off_s + n_q].reshape(R * n_q, 1)
            if not sym:
                full['buf_zeros'] = rows[:, off_z:off_z + n_q].reshape(R * n_q, 1)
        else:
            full['buf_scales'], full['buf_zeros'], full['static'] = static[0], static[1], True
        if with_codes:
            full['codes_perm'] = rows[:, off_c:].contiguous().view(torch.uint8)
        if fac.get('n_out'):
            full['buf_n_nonout'] = torch.tensor(C - fac['n_out'])
        return full

    # ---- the block -----------------------------------------------------------------------------
    @torch.no_grad()
    def block_opt(self, block, inputs, kwargs, subsets=None):
        """inputs: list of (b, T, C) tensors on the block's device (this rank's share);
        kwargs: dict or list of dicts of extra forward arguments.  Returns the inputs of the next
        block (outputs of the quantised block when quant_out, of the original block otherwise)."""
        if self.solver.owq:
            # n_outs are bound to the block's linears by position (gptq.py:89-93)
            self.solver.set_block_linears([n for sub in (subsets or llama_subsets(block)) for n in sub])
        if (subsets is None and self.stage_plan and self.true_sequential and self.quant_out
                and is_llama_layout(block) and self._staged_forward_matches(block, inputs, kwargs)):
            return self._block_opt_llama_staged(block, inputs, kwargs)
        subsets = subsets or llama_subsets(block)
        outs = None
        if self.true_sequential:
            stop_first = self.early_exit and self.quant_out      # the fp output is only needed without quant_out
            handle = self._hook_subset(subsets[0], stop=stop_first)
            first_out = self.block_forward(block, inputs, kwargs, need_output=not self.quant_out)
            handle.remove()
            if not self.quant_out:
                outs = first_out
            del first_out
            for i, subset in enumerate(subsets):
                self.subset_transform(subset)
                # rehook_next_subset swaps a subset for fake-quant linears only when a re-forward follows
                # (base_blockwise_quantization.py:522-525); the last one is swapped by quant_out below
                if i + 1 < len(subsets) or self.quant_out:
                    self._replace(subset)
                if i + 1 < len(subsets):
                    handle = self._hook_subset(subsets[i + 1], stop=self.early_exit)
                    self.block_forward(block, inputs, kwargs, need_output=False)
                    handle.remove()
        else:
            handles = [self._hook_subset(s) for s in subsets]
            first_out = self.block_forward(block, inputs, kwargs)
            for h in handles:
                h.remove()
            if not self.quant_out:
                outs = first_out
            for subset in subsets:
                self.subset_transform(subset)
                if self.quant_out:
                    self._replace(subset)
        if self.quant_out:
            outs = self.block_forward(block, inputs, kwargs)
        self.solver.check_status()
        return outs

    @torch.no_grad()
    def _staged_forward_matches(self, block, inputs, kwargs):
        """The staged plan hard-codes the data flow of a pre-norm Llama block (x + attn(norm(x)), then
        h + mlp(norm(h))).  Other decoder layers carry the same attribute names and compute something
        else (extra norms around the attention output, residual multipliers, ...), so before a block
        class is first staged one sequence goes through the untouched block and through the staged
        order of operations; only bit-equal outputs admit the plan.  Once per class, device, dtype."""
        if not inputs:
            return False
        x = inputs[0]
        key = (type(block), type(block.self_attn), type(block.mlp), str(x.device), x.dtype, bool(self.fused_block_ops))
        if key not in _stage_checked:
            if self.on_input is not None:
                self.on_input(0)
            kw = kwargs[0] if isinstance(kwargs, (list, tuple)) else kwargs
            a, m = block.self_attn, block.mlp
            norm = block_ops.rms_norm if self.fused_block_ops else (lambda mod, t: mod(t))
            ok = False
            try:
                ref = block(x, **kw)
                ref = ref[0] if isinstance(ref, tuple) else ref
                rotary = (block_ops.fused_rotary(a, x.device, x.dtype) if self.fused_block_ops
                          else contextlib.nullcontext())
                with rotary:
                    att = a(hidden_states=norm(block.input_layernorm, x), **kw)
                att = att[0] if isinstance(att, tuple) else att
                h = x + att
                y = norm(block.post_attention_layernorm, h)
                prod = (block_ops.gated_act(m.act_fn, m.gate_proj(y), m.up_proj(y)) if self.fused_block_ops
                        else m.act_fn(m.gate_proj(y)) * m.up_proj(y))
                out = h + m.down_proj(prod)
                ok = ref.shape == out.shape and torch.equal(ref, out)
            except (TypeError, RuntimeError, ValueError, AttributeError):
                ok = False
            _stage_checked[key] = ok
        if not _stage_checked[key] and type(block).__name__ not in self.stage_plan_rejected:
            self.stage_plan_rejected.append(type(block).__name__)
        return _stage_checked[key]

    @torch.no_grad()
    def _block_opt_llama_staged(self, block, inputs, kwargs):
        """true_sequential + quant_out on a Llama-layout block, one evaluation of every module:
        norm -> [H qkv, solve] -> attention (quantised q,k,v) -> [H o, solve] -> o_proj + residual
        -> norm -> [H gate/up, solve] -> act(gate) * up -> [H down, solve] -> down_proj + residual."""
        a, m = block.self_attn, block.mlp
        subsets = llama_subsets(block)
        kw = (lambda i: kwargs[i]) if isinstance(kwargs, (list, tuple)) else (lambda i: kwargs)
        n = len(inputs)
        self.forward_passes += 1
        norm = block_ops.rms_norm if self.fused_block_ops else (lambda mod, t: mod(t))

        name, layer = self._init_subset(subsets[0])
        normed = []
        with self.phases('forward_hessian'):
            for i, x in enumerate(inputs):
                if self.on_input is not None:
                    self.on_input(i)
                normed.append(norm(block.input_layernorm, x))
                self.solver.add_batch(layer, name, normed[-1], None)
        self.subset_transform(subsets[0])
        self._replace(subsets[0])

        name, layer = self._init_subset(subsets[1])
        seen = {}

        def grab(mod, args):
            seen['x'] = args[0]
            raise _StopForward()
        handle = a.o_proj.register_forward_pre_hook(grab)
        ctx = []
        rotary = (block_ops.fused_rotary(a, normed[0].device, normed[0].dtype) if self.fused_block_ops
                  else contextlib.nullcontext())
        with rotary, self.phases('forward_hessian'):
            for i in range(n):
                try:
                    a(hidden_states=normed[i], **kw(i))
                except _StopForward:
                    pass
                normed[i] = None
                ctx.append(seen.pop('x'))
                self.solver.add_batch(layer, name, ctx[-1], None)
        handle.remove()
        self.subset_transform(subsets[1])
        self._replace(subsets[1])

        name, layer = self._init_subset(subsets[2])
        resid, normed = [], []
        with self.phases('forward_hessian'):
            for i, x in enumerate(inputs):
                h = x + a.o_proj(ctx[i])
                ctx[i] = None
                resid.append(h)
                normed.append(norm(block.post_attention_layernorm, h))
                self.solver.add_batch(layer, name, normed[-1], None)
        self.subset_transform(subsets[2])
        self._replace(subsets[2])

        name, layer = self._init_subset(subsets[3])
        prod = []
        with self.phases('forward_hessian'):
            for i in range(n):
                y = normed[i]
                normed[i] = None
                if self.fused_block_ops:
                    prod.append(block_ops.gated_act(m.act_fn, m.gate_proj(y), m.up_proj(y)))
                else:
                    prod.append(m.act_fn(m.gate_proj(y)) * m.up_proj(y))
                self.solver.add_batch(layer, name, prod[-1], None)
        self.subset_transform(subsets[3])
        self._replace(subsets[3])

        outs = []
        with self.phases('forward_hessian'):
            for i in range(n):
                outs.append(resid[i] + m.down_proj(prod[i]))
                prod[i] = None
                resid[i] = None
        self.solver.check_status()
        return outs

    def _replace(self, subset):
        for n, (parent, attr) in subset.items():
            mod = getattr(parent, attr)
            if isinstance(mod, nn.Linear):
                new = self.fake_linear(mod)
                if getattr(new, '_lc_codes', None) is None:
                    new._lc_codes = getattr(mod, '_lc_codes', None)
                setattr(parent, attr, new)
