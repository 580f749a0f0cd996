"""W8A8 FP8 (e4m3) fake quantisation of a mixture-of-experts MLP layer with expert sharding.

What the reference does for an FP8 RTN recipe (configs/quantization/backend/vllm/fp8/rtn_fp8.yml)
at deploy('fake_quant'): every expert linear becomes an EffcientFakeQuantLinear
(llmc/compression/quantization/module_utils.py:774-852) whose weight is fake-quantised once
(FloatQuantizer per_channel, quant.py:1141-1158) and whose input is fake-quantised on every
forward (FloatQuantizer per_token dynamic, quant.py:1099-1108).  Here the same arithmetic runs in
batched form: all expert weights of a rank in one kernel launch per projection (per-channel = per
row, so stacking experts changes nothing), and the routed tokens of all local experts in one
per-token launch per projection input.  The gate of the router is a plain parameter and stays
unquantised, as in the reference (only nn.Linear modules are collected, base_model.py:361-366).

Expert sharding: rank r owns a contiguous slice of the routed experts, rank 0 also the (small)
shared experts; x is replicated, every rank evaluates its experts on their tokens and the partial
outputs are summed with one all-reduce.
"""
import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import parallel
from .quant import FloatQuantizer


class Fp8FakeQuantMoE:
    def __init__(self, hidden=2048, inter=1408, n_experts=64, n_shared=2, top_k=6, dtype=torch.bfloat16,
                 device='cuda', seed=5000):
        self.hidden, self.inter, self.n_experts, self.top_k = hidden, inter, n_experts, top_k
        self.dtype, self.device = dtype, torch.device(device)
        rank, world = parallel.world()
        self.e0, self.e1 = parallel.sequence_shard(n_experts, rank, world)
        g = torch.Generator().manual_seed(seed)

        def init(*shape):
            return (torch.randn(*shape, generator=g) * 0.02).to(dtype)
        # every rank draws the full set from the same seed and keeps its slice
        self.gate = init(n_experts, hidden).to(self.device)
        w_gate, w_up, w_down = init(n_experts, inter, hidden), init(n_experts, inter, hidden), init(n_experts, hidden, inter)
        sl = slice(self.e0, self.e1)
        self.w_gate, self.w_up, self.w_down = (t[sl].contiguous().to(self.device) for t in (w_gate, w_up, w_down))
        sw = n_shared * inter
        self.has_shared = rank == 0
        s_gate, s_up, s_down = init(sw, hidden), init(sw, hidden), init(hidden, sw)
        if self.has_shared:
            self.s_gate, self.s_up, self.s_down = (t.to(self.device) for t in (s_gate, s_up, s_down))
        self.wq = FloatQuantizer('e4m3', True, 'per_channel', use_qtorch=True)
        self.aq = FloatQuantizer('e4m3', True, 'per_token', use_qtorch=True)
        self.quantized = False

    @torch.no_grad()
    def quantize_weights(self):
        """w_qdq of every local expert linear: one launch per projection (rows of all experts stacked)."""
        def qdq(w):
            shape = w.shape
            return self.wq.fake_quant_weight_dynamic(w.reshape(-1, shape[-1])).reshape(shape)
        self.w_gate, self.w_up, self.w_down = qdq(self.w_gate), qdq(self.w_up), qdq(self.w_down)
        if self.has_shared:
            self.s_gate, self.s_up, self.s_down = qdq(self.s_gate), qdq(self.s_up), qdq(self.s_down)
        self.quantized = True

    @torch.no_grad()
    def route(self, x):
        scores = torch.softmax((x @ self.gate.t()).float(), dim=-1)
        w, idx = torch.topk(scores, self.top_k, dim=-1)
        return w.to(x.dtype), idx

    @torch.no_grad()
    def forward(self, x, a_qdq=True, grouped=True):
        """x: (tokens, hidden).  Returns the layer output (summed over ranks).

        The routed tokens are sorted by expert once; the expert boundaries stay on the device as a
        cumulative offset table, and with grouped=True the three projections of all local experts are one
        grouped GEMM each (torch.nn.functional.grouped_mm over the offset table), so a single-rank forward
        never synchronises with the host.  With several ranks the one host read left is the pair of row
        bounds of this rank's expert slice (it fixes tensor shapes).  grouped=False evaluates expert by
        expert with F.linear (one host read of the 64 counts)."""
        w, idx = self.route(x)
        flat_e = idx.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        tok = (order // self.top_k)
        e_sorted = flat_e[order]
        ends = torch.cumsum(torch.bincount(e_sorted, minlength=self.n_experts), 0)      # device: row ends per expert
        n_rows = flat_e.numel()
        if parallel.world()[1] == 1:
            lo, hi = 0, n_rows
        else:
            b = torch.stack([ends[self.e0 - 1] if self.e0 > 0 else ends.new_zeros(()), ends[self.e1 - 1]]).tolist()
            lo, hi = int(b[0]), int(b[1])
        out = torch.zeros_like(x, dtype=torch.float32)
        if hi > lo:
            xin = x[tok[lo:hi]]
            xq = self.aq.fake_quant_act_dynamic(xin) if a_qdq else xin          # gate_proj / up_proj input
            if grouped:
                offs = (ends[self.e0:self.e1] - lo).to(torch.int32)
                g = F.grouped_mm(xq, self.w_gate.transpose(1, 2), offs=offs)
                u = F.grouped_mm(xq, self.w_up.transpose(1, 2), offs=offs)
                hmid = F.silu(g) * u
                hq = self.aq.fake_quant_act_dynamic(hmid) if a_qdq else hmid     # down_proj input
                y = F.grouped_mm(hq, self.w_down.transpose(1, 2), offs=offs)
            else:
                starts = [0] + ends.tolist()
                hmid = torch.empty((hi - lo, self.inter), dtype=x.dtype, device=x.device)
                for e in range(self.e0, self.e1):
                    a, b = starts[e] - lo, starts[e + 1] - lo
                    if b > a:
                        le = e - self.e0
                        hmid[a:b] = F.silu(F.linear(xq[a:b], self.w_gate[le])) * F.linear(xq[a:b], self.w_up[le])
                hq = self.aq.fake_quant_act_dynamic(hmid) if a_qdq else hmid
                y = torch.empty((hi - lo, self.hidden), dtype=x.dtype, device=x.device)
                for e in range(self.e0, self.e1):
                    a, b = starts[e] - lo, starts[e + 1] - lo
                    if b > a:
                        y[a:b] = F.linear(hq[a:b], self.w_down[e - self.e0])
            wsel = w.reshape(-1)[order][lo:hi].unsqueeze(1)
            out.index_add_(0, tok[lo:hi], (y * wsel).float())
        if self.has_shared:
            xs = self.aq.fake_quant_act_dynamic(x) if a_qdq else x
            hs = F.silu(F.linear(xs, self.s_gate)) * F.linear(xs, self.s_up)
            hs = self.aq.fake_quant_act_dynamic(hs) if a_qdq else hs
            out += F.linear(hs, self.s_down).float()
        if parallel.world()[1] > 1:
            dist.all_reduce(out)
        return out.to(x.dtype)
