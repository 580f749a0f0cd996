"""Host-side mirror of the reference GPTQ algorithm's per-layer hot methods.

Method names, arguments and the buffers left on each layer follow
llmc/compression/quantization/gptq.py: layer_init :298-308, add_batch :254-295,
layer_transform :114-117 (hessian_sorting :58-64, process_hessian_and_weights :128-176,
update_layer_with_transformed_weights :178-196, weight_transform :199-244,
update_model_qparams :398-409), w_qdq :425-452, free :466-471.  `lightcompress_b200.plugin.install()`
re-registers a subclass of the reference's `GPTQ` whose methods of these names forward here; used
stand-alone the class drives one or more `nn.Linear` layers directly.

Differences in schedule, not in result: the Hessian is kept as the raw sum of X^T X and scaled
by 2/nsamples once, and with several ranks it is all-reduced once per layer (in
`layer_transform`) instead of after every `add_batch` call.
"""
import ctypes

import torch

from . import _lib as L
from . import parallel
from .quant import IntegerQuantizer


def _balanced_slices(m1, m2, parts, step=128):
    """Column boundaries (multiples of `step`) of `parts` slices of the m2 x m1 off-diagonal block with
    about equal work: a column c costs (m1 - c) in the first product (the right factor is lower
    triangular) and m2 / 2 in the second."""
    cols = list(range(0, m1, step))
    cost = [(m1 - c) + m2 / 2.0 for c in cols]
    total, acc, bounds = sum(cost), 0.0, [0]
    for i, c in enumerate(cols):
        acc += cost[i]
        while len(bounds) < parts and acc >= total * len(bounds) / parts:
            bounds.append(min(m1, c + step))
    while len(bounds) <= parts:
        bounds.append(m1)
    bounds[parts] = m1
    return bounds


class GPTQ:
    def __init__(self, wquantizer=None, special=None, model_dtype=torch.bfloat16, **wq_kwargs):
        special = dict(special or {})
        self.wquantizer = wquantizer or IntegerQuantizer(4, False, 'per_group', group_size=128, **wq_kwargs)
        self.true_sequential = special.get('true_sequential', True)
        self.static_groups = special.get('static_groups', False)
        self.actorder = special.get('actorder', True)
        self.percdamp = special.get('percdamp', 0.01)
        self.blocksize = special.get('blocksize', 128)
        self.owq = special.get('owq', False)
        self.chunk_num = special.get('chunk_num', 1)
        if self.owq:
            # gptq.py:47-50: one outlier-column count per linear of a block, in get_block_linears order
            self.n_outs = list(special['n_outs'])
            self.static_groups = False
            self.actorder = False
        self.n_out_dict = {}
        self.emit_codes = special.get('emit_codes', True)
        # 'direct': one Cholesky of the index-reversed matrix + one triangular inverse (cuSOLVER / cuBLAS);
        # 'native': the Cholesky by cuSOLVER, the triangular inverse blocked on 128x128 diagonal blocks with
        #           its products on the tensor cores (lc_gptq_invert_factor; C % 128 == 0, else 'direct');
        # 'native_full': the Cholesky blocked the same way too (lc_gptq_factorize): this library's own kernels
        #           from the dampened Hessian to U;
        # 'auto' (default): 'native_full' from `own_cholesky_min` columns on (measured on B200: 13.7 ms against
        #           17.1 ms at C = 11008), 'native' below it (at C = 4096 the own Cholesky's chain of 32
        #           dependent leaf / panel / strip launches takes 3.1 ms against 2.2 ms);
        # 'reference': the reference's three factorisations (gptq.py:172-174).  Same U up to fp32 rounding.
        self.factorization = special.get('factorization', 'auto')
        self.own_cholesky_min = int(special.get('own_cholesky_min', 8192))
        # 'tensor': trailing update batched per 1024-column panel on tcgen05 (3-term tf32 split);
        # 'ffma': the reference's per-block update with the fp32 FFMA kernel
        self.trailing = special.get('trailing', 'tensor')
        # multi-rank runs: the top level of the triangular inverse is computed once per process group and
        # exchanged (every rank factorises the same all-reduced Hessian), for C >= shared_inverse_min
        # Cholesky of matrices at least this wide: blocked over 1024 rows with the panel solves and trailing
        # updates on the tensor cores (cuSOLVER only factorises the diagonal blocks); below it cuSOLVER alone
        self.blocked_cholesky_min = int(special.get('blocked_cholesky_min', 1 << 30))
        self.shared_inverse = special.get('shared_inverse', True)
        self.shared_inverse_min = int(special.get('shared_inverse_min', 1024))
        # forward hooks deliver one sequence per call; up to `hessian_batch` of them (<= 8) are
        # held by reference and accumulated in one launch, so H is updated once per batch
        self.hessian_batch = max(1, min(8, int(special.get('hessian_batch', 8))))
        # token split of the Hessian kernel: 0 = chosen per launch (may combine partial sums with
        # atomics in varying order when the matrix is small), 1 = one work item per tile (deterministic)
        self.hessian_ksplit = int(special.get('hessian_ksplit', 0))
        self.model_dtype = model_dtype
        # the Hessians accumulated by add_batch hold their upper triangle only (see _flush); a caller that
        # hands factorize() / solve() a full symmetric matrix of its own is served by the same read
        self.h_upper = True
        self.layers_cache = {}
        self._pending_status = []       # device status words of tensor-core launches, read lazily
        self._pending_info = []         # cuSOLVER potrf info words (non-zero: not positive definite)
        self._check_config()
        self.need_perm = (self.wquantizer.granularity == 'per_group' and not self.static_groups
                          and self.actorder) or self.owq

    def _check_config(self):
        wq = self.wquantizer
        # per_channel (the reference's w8a8 configs): search_layer_qparams (gptq.py:368-375) fixes one scale per
        # row for every column, i.e. static groups with a single group spanning the row
        self.per_channel = wq.granularity == 'per_channel'
        if self.per_channel and self.owq:
            raise NotImplementedError('owq with per_channel weights is outside the B200 hot path')
        if self.blocksize != 128 or not (self.per_channel or (wq.granularity == 'per_group' and wq.group_size == 128)):
            # gptq.py:216-223 reads group statistics that are only well defined when a group
            # starts at a block boundary; the kernels implement group_size == blocksize == 128.
            raise NotImplementedError('GPTQ kernels need per_channel, or per_group with group_size == blocksize == 128')
        wq._check_supported()

    # ---- Hessian ---------------------------------------------------------------------------
    @torch.no_grad()
    def layer_init(self, layer, name):
        cols = layer.weight.shape[1]
        self.layers_cache[name] = {
            'H': torch.zeros((cols, cols), device=layer.weight.device, dtype=torch.float32),
            'nsamples': 0, 'columns': cols,
            'status': torch.zeros(1, dtype=torch.int32, device=layer.weight.device),
            'pending': [],
        }

    @torch.no_grad()
    def add_batch(self, layer, name, inp, out=None):
        """H_raw += X^T X over the tokens of `inp` ((b, T, C) or (T, C)); nsamples += b."""
        st = self.layers_cache[name]
        if inp.dim() == 2:
            inp = inp.unsqueeze(0)
        b = inp.shape[0]
        x = inp.reshape(-1, inp.shape[-1])
        if x.dtype != torch.bfloat16:
            raise NotImplementedError('the Hessian kernel takes bf16 activations')
        x = x if x.is_contiguous() else x.contiguous()
        L.require_cuda(x)
        # held by reference until the batch is full: remember the tensor's version so that an in-place
        # change made by the caller in between (the reference consumes the tensor inside the hook) is
        # caught instead of silently entering the Hessian
        st['pending'].append(x)
        st.setdefault('versions', []).append(x._version)
        st['nsamples'] += b
        if len(st['pending']) >= self.hessian_batch:
            self._flush(st)

    def _flush(self, st):
        xs = st['pending']
        if not xs:
            return
        n = len(xs)
        for x, v in zip(xs, st.get('versions', [])):
            if x._version != v:
                raise RuntimeError('an activation handed to add_batch was modified in place before its Hessian '
                                   'batch was accumulated; pass a copy or set hessian_batch: 1')
        st['versions'] = []
        ptrs = (ctypes.c_void_p * n)(*[x.data_ptr() for x in xs])
        toks = (ctypes.c_int64 * n)(*[x.shape[0] for x in xs])
        # only the upper triangle of H is kept (half the epilogue's atomic adds); its readers fetch (i, j) from it
        L.call('lc_hessian_accum_upper', ptrs, toks, n, xs[0].shape[1], L.ptr(st['H']), 1.0, 1.0, self.hessian_ksplit,
               L.ptr(st['status']), L.stream_of(xs[0]))
        st['pending'] = []

    def _finish_hessian(self, name):
        """All-reduce once per layer (gptq.py:292-295 does it per call); returns (H_raw, 2/n)."""
        st = self.layers_cache[name]
        self._flush(st)
        if parallel.world()[1] == 1:
            # one rank: no host wait here; the status word is read with the others at check_status()
            n = st['nsamples']
            self._pending_status.append(st['status'])
        else:
            # every rank learns in this reduction whether any rank's kernel failed, and all raise together;
            # the other pending status words are combined over the ranks at the block's check_status()
            _, n, code = parallel.reduce_hessian(st['H'], st['nsamples'], st['status'])
            if code != 0:
                raise L.LcError('lc_hessian_accum', code, L.status_string(code))
        if n == 0:
            raise RuntimeError(f'no calibration samples were accumulated for layer {name}')
        return st['H'], 2.0 / n

    # ---- solver ----------------------------------------------------------------------------
    @staticmethod
    def hessian_full(H_upper):
        """The full symmetric matrix of a Hessian kept as its upper triangle."""
        return torch.triu(H_upper) + torch.triu(H_upper, 1).t()

    @torch.no_grad()
    def layer_transform(self, layer, name, rows=None):
        """Quantises `layer` in place like the reference: weight.data becomes the fp32
        error-compensated weight and buf_scales / buf_zeros / buf_perm / buf_invperm are
        registered.  `rows=(r0, r1)` restricts the solve to a row range (rows are independent);
        the caller then gathers the pieces."""
        H, hscale = self._finish_hessian(name)
        n_out = self.n_out_of(name)
        fac = self.factorize(H, hscale, n_out=n_out) if n_out else None
        static = self.static_qparams(layer) if self.uses_static() else None
        res = self.solve(layer.weight.data, H, hscale, rows=rows, factor=fac, static=static)
        if rows is None:
            self._install(layer, res)
        return res

    @torch.no_grad()
    def uses_static(self):
        """The solver quantises with the layer's own buffers (static_groups, or per_channel weights)."""
        return bool(self.static_groups or self.per_channel)

    @torch.no_grad()
    def static_qparams(self, layer):
        """static_groups: the layer's round-to-nearest buffers (collect_block_qparams,
        base_blockwise_quantization.py:349-376, leaves them before GPTQ runs; computed and registered here
        when the layer does not have them yet).  Returns (buf_scales, buf_zeros or None)."""
        wq = self.wquantizer
        if 'buf_scales' not in layer._buffers:
            _, s, z, qmax, qmin = wq.get_tensor_qparams(layer.weight.data)
            layer.register_buffer('buf_scales', s)
            if not wq.sym:
                layer.register_buffer('buf_zeros', z)
        return layer.buf_scales, (None if wq.sym else layer.buf_zeros)

    def n_out_of(self, name):
        """owq: the number of outlier columns of the linear `name` (gptq.py:122); 0 without owq."""
        if not self.owq:
            return 0
        return int(self.n_out_dict[name])

    def set_block_linears(self, names):
        """owq: binds n_outs to the linears of a block by position (gptq.py:89-93)."""
        if self.owq and not self.n_out_dict:
            self.n_out_dict = {name: self.n_outs[i] for i, name in enumerate(names)}

    def owq_order(self, H, n_out):
        """hessian_sorting with owq (gptq.py:66-83): the n_out columns with the largest Hessian diagonal
        go last, in descending order of it; the others keep their order."""
        C = H.shape[0]
        diag = torch.empty(C, dtype=torch.float32, device=H.device)
        L.call('lc_gptq_diag', L.ptr(H), C, L.ptr(diag), L.stream_of(H))
        top = torch.argsort(diag, descending=True)[:n_out]
        keep = torch.ones(C, dtype=torch.bool, device=H.device)
        keep[top] = False
        perm = torch.cat([torch.arange(C, device=H.device)[keep], top])
        return perm, torch.argsort(perm)

    @torch.no_grad()
    def factorize(self, H, hscale=1.0, perm=None, n_out=0):
        """Everything of process_hessian_and_weights (gptq.py:128-176) that depends on H only:
        act-order permutation, dampening, and U with U^T U = (permuted, damped H)^-1.  Linears that
        read the same input (q/k/v, gate/up) share one result (with owq: if their n_out agree)."""
        L.require_cuda(H)
        C = H.shape[0]
        if n_out:
            if not 0 < n_out < 128 or C % 128 != 0:
                # the reference's own deploy step (gptq.py:425-452) only works while the group count stays
                # C / group_size, i.e. with fewer outlier columns than a group
                raise NotImplementedError('owq needs 0 < n_out < 128 and columns % 128 == 0')
            if perm is None:
                perm, invperm = self.owq_order(H, n_out)
            else:
                perm = perm.to(H.device).contiguous()
                invperm = torch.argsort(perm)
        elif perm is None:
            perm, invperm = self.act_order(H)
        else:
            # caller-supplied column order (argsort leaves the order of equal diagonal entries open)
            perm = perm.to(H.device).contiguous()
            invperm = torch.argsort(perm)
        Hp = torch.empty((C, C), dtype=torch.float32, device=H.device)
        scratch = torch.empty(4, dtype=torch.float32, device=H.device)
        mode = self.factorization
        if mode == 'auto':
            mode = 'native_full' if C >= self.own_cholesky_min else 'native'
        native = mode in ('native', 'native_full') and C % 128 == 0
        direct = native or mode in ('direct', 'native', 'native_full')
        L.call('lc_gptq_permute_damp', None, L.LC_F32, L.ptr(H), L.ptr(perm), 0, C, float(hscale),
               float(self.percdamp), (L.LC_H_REVERSE if direct else 0) | (L.LC_H_UPPER if self.h_upper else 0)
               | getattr(self, 'prep_flags', 0), None,
               L.ptr(Hp), L.ptr(scratch), L.stream_of(H))
        want_lo = self.trailing == 'tensor' and C % 128 == 0 and C > 1024
        fac = {'H': H, 'perm': perm, 'invperm': invperm, 'U': None, 'U_lo': None, 'n_out': int(n_out)}
        if native:
            # blocked Cholesky + triangular inverse with the products on the tensor cores; a matrix that
            # is not positive definite is reported through the status word at the next check_status()
            U = torch.empty((C, C), dtype=torch.float32, device=H.device)
            U_lo = torch.empty_like(U) if want_lo else None
            ws_floats = int(L.lib.lc_gptq_factor_workspace_floats(C))
            ws = self._workspace(ws_floats, H.device)
            status = torch.zeros(1, dtype=torch.int32, device=H.device)
            if mode == 'native_full':
                L.call('lc_gptq_factorize', L.ptr(Hp), C, L.ptr(U), L.ptr(U_lo), L.ptr(ws), ws_floats,
                       L.ptr(status), L.stream_of(H))
            else:
                # cuSOLVER returns the lower factor M column-major: the same bytes are the row-major upper
                # factor G = M^T that the inverse reads
                # no host synchronisation here: potrf's info word joins the status words read at the next
                # check_status(), which raises LinAlgError like torch.linalg.cholesky would have
                if C >= self.blocked_cholesky_min:
                    G = self._blocked_cholesky_upper(Hp, status)
                else:
                    M, info = torch.linalg.cholesky_ex(Hp, check_errors=False)
                    self._pending_info.append(info.reshape(1))
                    G = M.t() if M.stride() == (1, C) else M.t().contiguous()
                world = parallel.world()[1] if self.shared_inverse else 1
                if world > 1 and C >= self.shared_inverse_min:
                    self._shared_inverse(G, C, U, U_lo, ws, ws_floats, status)
                else:
                    L.call('lc_gptq_invert_factor', L.ptr(G), C, L.ptr(U), L.ptr(U_lo), L.ptr(ws), ws_floats,
                           L.ptr(status), L.stream_of(H))
            self._pending_status.append(status)
            fac['U'], fac['U_lo'] = U, U_lo
            return fac
        U = self.inverse_cholesky_upper_reversed(Hp) if direct else self.inverse_cholesky_upper(Hp)
        fac['U'] = U
        if want_lo:
            fac['U_lo'] = torch.empty_like(U)
            L.call('lc_gptq_split_tf32', L.ptr(U), U.numel(), L.ptr(fac['U_lo']), L.stream_of(U))
        return fac

    def _blocked_cholesky_upper(self, A, status, block=1024):
        """Upper Cholesky factor G (A = G^T G, row-major) of a large matrix, right-looking over 1024-row
        blocks: cuSOLVER factorises the diagonal block, everything that scales with C^2 per step -- the
        panel solve X = G_kk^-T A[k, k+1:] (through the inverse of G_kk) and the trailing update
        A[k+1:, k+1:] -= X^T X -- runs on the tensor cores (lc_tf32x3_gemm_tn).  cuSOLVER's own potrf
        spends most of its time in its panel kernels at this size (13.3 ms at C = 11008).
        A (upper triangle valid) is destroyed."""
        n = A.shape[0]
        dev, st = A.device, L.stream_of(A)
        G = torch.zeros((n, n), dtype=torch.float32, device=dev)
        lo = torch.empty((block, n), dtype=torch.float32, device=dev)      # low parts of the current row panel
        ws_floats = int(L.lib.lc_gptq_factor_workspace_floats(block))
        ws = torch.empty(ws_floats, dtype=torch.float32, device=dev)
        Ukk = torch.empty((block, block), dtype=torch.float32, device=dev)
        for k0 in range(0, n, block):
            k1 = min(k0 + block, n)
            b = k1 - k0
            Gkk, info = torch.linalg.cholesky_ex(A[k0:k1, k0:k1], upper=True, check_errors=False)
            self._pending_info.append(info.reshape(1))
            Gkk = torch.triu(Gkk).contiguous()
            G[k0:k1, k0:k1] = Gkk
            if k1 == n:
                break
            # V = G_kk^-1 (upper): lc_gptq_invert_factor returns U = J (G_kk^-1)^T J, so V[i][j] = U[b-1-j][b-1-i]
            u = Ukk[:b, :b] if b == block else torch.empty((b, b), dtype=torch.float32, device=dev)
            L.call('lc_gptq_invert_factor', L.ptr(Gkk), b, L.ptr(u), None, L.ptr(ws), ws_floats, L.ptr(status), st)
            V = u.flip(0, 1).t().contiguous()
            V_lo = torch.empty_like(V)
            L.call('lc_gptq_split_tf32', L.ptr(V), V.numel(), L.ptr(V_lo), st)
            # X = V^T A[k0:k1, k1:] -> G[k0:k1, k1:]; the panel's rows are contiguous, so their low parts are too
            rows_lo = lo[:b]
            L.call('lc_gptq_split_tf32', L.ptr(A[k0:k1]), b * n, L.ptr(rows_lo), st)
            L.call('lc_tf32x3_gemm_tn', L.ptr(G[k0:k1, k1:]), n, L.ptr(V), L.ptr(V_lo), b, L.ptr(A[k0:k1, k1:]),
                   L.ptr(rows_lo[:, k1:]), n, b, n - k1, b, 0, 1.0, L.LC_GEMM_A_UPPER, L.ptr(status), st)
            # A[k1:, k1:] -= X^T X (tiles that reach the diagonal or lie above it)
            L.call('lc_gptq_split_tf32', L.ptr(G[k0:k1]), b * n, L.ptr(rows_lo), st)
            L.call('lc_tf32x3_gemm_tn', L.ptr(A[k1:, k1:]), n, L.ptr(G[k0:k1, k1:]), L.ptr(rows_lo[:, k1:]), n,
                   L.ptr(G[k0:k1, k1:]), L.ptr(rows_lo[:, k1:]), n, n - k1, n - k1, b, 1, -1.0,
                   L.LC_GEMM_UPPER_ONLY, L.ptr(status), st)
        return G

    def _shared_inverse(self, G, C, U, U_lo, ws, ws_floats, status):
        """The triangular inverse with its top-level block (3/4 of the FLOPs) computed once per process
        group instead of once per rank: every rank takes a column slice, the slices are broadcast.  All
        ranks must call this with the same G (they do: the Hessian was all-reduced), and end with
        bit-identical U."""
        import torch.distributed as dist
        rank, world = parallel.world()
        h = int(L.lib.lc_gptq_factor_split(C))
        bounds = _balanced_slices(h, C - h, world)
        c0, c1 = bounds[rank], bounds[rank + 1]
        st = L.stream_of(G)
        L.call('lc_gptq_invert_factor_part', L.ptr(G), C, L.ptr(ws), ws_floats, c0, c1, L.ptr(status), st)
        off = int(L.lib.lc_gptq_factor_vt_offset(C))
        Vt = ws[off:off + C * C].view(C, C)
        for r in range(world):
            a, b = bounds[r], bounds[r + 1]
            if b > a:
                piece = Vt[h:, a:b].contiguous() if r == rank else torch.empty((C - h, b - a), dtype=torch.float32,
                                                                              device=G.device)
                dist.broadcast(piece, src=r)
                if r != rank:
                    Vt[h:, a:b].copy_(piece)
        L.call('lc_gptq_invert_factor_finish', C, L.ptr(ws), ws_floats, L.ptr(U), L.ptr(U_lo), st)

    def _workspace(self, floats, device):
        """Scratch of the native factorisation, kept between calls (2.4 GB at C = 11008)."""
        ws = getattr(self, '_ws', None)
        if ws is None or ws.numel() < floats or ws.device != device:
            self._ws = ws = torch.empty(floats, dtype=torch.float32, device=device)
        return ws

    @torch.no_grad()
    def solve(self, W, H, hscale=1.0, rows=None, factor=None, static=None):
        """static: (buf_scales, buf_zeros or None) of all rows of W, for static_groups."""
        wq = self.wquantizer
        fac = factor or self.factorize(H, hscale)
        H, perm, invperm, U = fac['H'], fac['perm'], fac['invperm'], fac['U']
        L.require_cuda(W, H)
        W = W if W.is_contiguous() else W.contiguous()
        if rows is not None:
            W = W[rows[0]:rows[1]]
        R, C = W.shape
        dev = W.device
        stream = L.stream_of(W)
        n_groups = (C + 127) // 128
        Wp = torch.empty((R, C), dtype=torch.float32, device=dev)
        L.call('lc_gptq_permute_damp', L.ptr(W), L.lc_dtype(W), L.ptr(H), L.ptr(perm), R, C, 1.0, 0.0, 0,
               L.ptr(Wp), None, None, stream)
        err = torch.empty((128, R), dtype=torch.float32, device=dev)
        scales = torch.empty((R * n_groups, 1), dtype=torch.float32, device=dev)
        zeros = torch.empty((R * n_groups, 1), dtype=torch.float32, device=dev)
        codes = torch.empty((R, C), dtype=torch.uint8, device=dev) if self.emit_codes else None
        loss_rows = torch.empty(R, dtype=torch.float32, device=dev)
        # owq: the last n_out (permuted) columns are not quantised; they take the error feedback and stay fp32
        n_quant = C - int(fac.get('n_out', 0))
        if static is not None:
            return self._solve_static(Wp, fac, static, rows, err, codes, loss_rows, stream)
        if fac.get('U_lo') is not None and R % 4 == 0:
            panel = torch.empty((2, 1024, R), dtype=torch.float32, device=dev)
            status = torch.zeros(1, dtype=torch.int32, device=dev)
            L.call('lc_gptq_weight_transform_tc_owq', L.ptr(Wp), L.ptr(U), L.ptr(fac['U_lo']), R, C, n_quant,
                   int(wq.bit), int(wq.sym), L.ptr(err), L.ptr(panel[0]), L.ptr(panel[1]), L.ptr(scales),
                   L.ptr(zeros), L.ptr(codes), L.ptr(loss_rows), L.ptr(status), stream)
            self._pending_status.append(status)
        else:
            L.call('lc_gptq_weight_transform_owq', L.ptr(Wp), L.ptr(U), R, C, n_quant, int(wq.bit), int(wq.sym),
                   L.ptr(err), L.ptr(scales), L.ptr(zeros), L.ptr(codes), L.ptr(loss_rows), stream)
        out = torch.empty((R, C), dtype=torch.float32, device=dev)
        L.call('lc_gptq_unpermute', L.ptr(Wp), L.ptr(perm), R, C, L.ptr(out), L.LC_F32, stream)
        res = {'weight': out, 'buf_scales': scales, 'buf_zeros': None if wq.sym else zeros,
               'buf_perm': perm, 'buf_invperm': invperm, 'codes_perm': codes, 'loss_rows': loss_rows}
        if n_quant < C:
            res['buf_n_nonout'] = torch.tensor(n_quant)
            if codes is not None:
                codes[:, n_quant:] = 0          # the outlier columns have no codes
        return res

    def _solve_static(self, Wp, fac, static, rows, err, codes, loss_rows, stream):
        """weight_transform with static groups (gptq.py:224-227): the layer's own qparams, looked up by the
        group of each column's original position; the buffers are returned unchanged."""
        wq = self.wquantizer
        R, C = Wp.shape
        dev = Wp.device
        perm, invperm, U = fac['perm'], fac['invperm'], fac['U']
        n_groups = (C + 127) // 128
        if C % 128 and not self.per_channel:
            raise NotImplementedError('static_groups needs columns % 128 == 0')
        s_all, z_all = static
        r0, r1 = rows if rows is not None else (0, R)
        # the solver computes in fp32 on the promoted qparams (their values are those of the weight dtype);
        # per_channel: the row's one scale stands in every column group of the kernels' table
        per = 1 if self.per_channel else n_groups

        def table(t):
            t = t.reshape(-1, per)[r0:r1].float()
            return (t.expand(-1, n_groups) if self.per_channel else t).contiguous()
        s32 = table(s_all)
        z32 = None if wq.sym else table(z_all)
        cols = torch.arange(C, device=dev) if perm is None else perm
        col_group = (cols // 128).to(torch.int32).contiguous()
        if fac.get('U_lo') is not None and R % 4 == 0:
            panel = torch.empty((2, 1024, R), dtype=torch.float32, device=dev)
            status = torch.zeros(1, dtype=torch.int32, device=dev)
            L.call('lc_gptq_weight_transform_tc_static', L.ptr(Wp), L.ptr(U), L.ptr(fac['U_lo']), R, C, int(wq.bit),
                   int(wq.sym), L.ptr(err), L.ptr(panel[0]), L.ptr(panel[1]), L.ptr(s32), L.ptr(z32),
                   L.ptr(col_group), L.ptr(codes), L.ptr(loss_rows), L.ptr(status), stream)
            self._pending_status.append(status)
        else:
            L.call('lc_gptq_weight_transform_static', L.ptr(Wp), L.ptr(U), R, C, int(wq.bit), int(wq.sym),
                   L.ptr(err), L.ptr(s32), L.ptr(z32), L.ptr(col_group), L.ptr(codes), L.ptr(loss_rows), stream)
        out = torch.empty((R, C), dtype=torch.float32, device=dev)
        L.call('lc_gptq_unpermute', L.ptr(Wp), L.ptr(perm), R, C, L.ptr(out), L.LC_F32, stream)
        sl = slice(r0 * per, r1 * per)
        return {'weight': out, 'buf_scales': s_all[sl], 'buf_zeros': None if wq.sym else z_all[sl],
                'buf_perm': perm, 'buf_invperm': invperm, 'codes_perm': codes, 'loss_rows': loss_rows,
                'static': True}

    def act_order(self, H):
        """perm = argsort(diag(H), descending) and its inverse (gptq.py:58-64, :158), or (None, None)."""
        if not self.actorder:
            return None, None
        C = H.shape[0]
        diag = torch.empty(C, dtype=torch.float32, device=H.device)
        L.call('lc_gptq_diag', L.ptr(H), C, L.ptr(diag), L.stream_of(H))
        perm = torch.argsort(diag, descending=True)
        return perm, torch.argsort(perm)

    @staticmethod
    def inverse_cholesky_upper(Hp):
        """U with U^T U = Hp^-1 (gptq.py:172-174): cuSOLVER through torch, on the current stream.
        Raises torch.linalg.LinAlgError when Hp is not positive definite, like the reference."""
        Lc = torch.linalg.cholesky(Hp)
        Hinv = torch.cholesky_inverse(Lc)
        del Lc
        # torch returns the upper factor as a transposed view of the lower one; the kernels read
        # row-major memory, so materialise it.
        return torch.linalg.cholesky(Hinv, upper=True).contiguous()

    @staticmethod
    def inverse_cholesky_upper_reversed(Hr):
        """Same U from the index-reversed matrix Hr = J Hp J: Hr = M M^T (one cuSOLVER potrf), then
        U = J M^-1 J (one cuBLAS triangular solve against the identity and a flip)."""
        C = Hr.shape[0]
        M = torch.linalg.cholesky(Hr)
        # explicitly row-major: zeros_like would inherit the column-major strides cuSOLVER results carry
        Minv = torch.zeros(M.shape, dtype=M.dtype, device=M.device)
        GPTQ._lower_inverse(M, Minv)
        del M
        U = torch.empty_like(Minv)
        L.call('lc_gptq_flip', L.ptr(Minv), C, L.ptr(U), L.stream_of(Minv))
        return U

    @staticmethod
    def _lower_inverse(M, out, leaf=1024):
        """out <- M^-1 for lower-triangular M, written into the (pre-zeroed) row-major `out`:
        inv([[A, 0], [B, D]]) = [[A^-1, 0], [-D^-1 B A^-1, D^-1]], recursively; leaves by a cuBLAS
        triangular solve against the identity.  One third of the FLOPs of a full-size solve against
        the identity, almost all of them in large fp32 GEMMs."""
        n = M.shape[0]
        if n <= leaf:
            eye = torch.eye(n, dtype=M.dtype, device=M.device)
            out.copy_(torch.linalg.solve_triangular(M, eye, upper=False))
            return
        h = (n // 2 + 127) // 128 * 128
        GPTQ._lower_inverse(M[:h, :h], out[:h, :h], leaf)
        GPTQ._lower_inverse(M[h:, h:], out[h:, h:], leaf)
        torch.matmul(out[h:, h:], torch.matmul(M[h:, :h], out[:h, :h]), out=out[h:, :h])
        out[h:, :h].neg_()

    def _install(self, layer, res):
        layer.weight.data = res['weight'].reshape(layer.weight.shape)
        wq = self.wquantizer
        for k in ('buf_scales', 'buf_zeros', 'buf_perm', 'buf_invperm', 'buf_n_nonout'):
            v = res.get(k)
            if v is None:
                continue
            if k in layer._buffers:
                layer._buffers[k] = v
            else:
                layer.register_buffer(k, v)
        if 'buf_qmax' not in layer._buffers:
            layer.register_buffer('buf_qmax', wq.qmax.to(layer.weight.device))
            layer.register_buffer('buf_qmin', wq.qmin.to(layer.weight.device))
        # the solver's codes (permuted order), kept for the deploy-time weight; tied to this very weight
        # tensor so that a weight replaced later falls back to re-quantising
        # (not with owq: the outlier columns have no codes, deploy re-quantises like the reference)
        codes = res.get('codes_perm')
        layer._lc_codes = None if codes is None or res.get('buf_n_nonout') is not None or res.get('static') else (
            codes, layer.weight.data.data_ptr())

    @torch.no_grad()
    def w_qdq(self, module, wquantizer):
        """Deploy-time fake quant (gptq.py:425-452).  When the solver's codes of this weight are at hand the
        chain gather -> static fake quant -> gather -> cast is one kernel that dequantises them."""
        weight = module.weight
        kept = getattr(module, '_lc_codes', None)
        if (kept is not None and kept[1] == weight.data.data_ptr() and wquantizer is self.wquantizer
                and wquantizer.granularity == 'per_group' and wquantizer.group_size == 128
                and self.model_dtype in (torch.bfloat16, torch.float16, torch.float32)):
            codes = kept[0]
            R, C = codes.shape
            out = torch.empty((R, C), dtype=self.model_dtype, device=codes.device)
            zeros = None if wquantizer.sym else module.buf_zeros
            L.call('lc_gptq_dequant_unpermute', L.ptr(codes), L.ptr(module.buf_scales), L.ptr(zeros),
                   L.ptr(module.buf_invperm) if self.need_perm else None, R, C, int(wquantizer.bit),
                   int(wquantizer.sym), L.ptr(out), L.lc_dtype(out), L.stream_of(codes))
            return out.reshape(weight.shape)
        if self.need_perm:
            weight = weight[:, module.buf_perm]
        args = {'scales': module.buf_scales, 'zeros': getattr(module, 'buf_zeros', None),
                'qmax': module.buf_qmax, 'qmin': module.buf_qmin}
        fp_weight = weight[:, int(module.buf_n_nonout):] if self.owq else None       # gptq.py:440-447
        weight = wquantizer.fake_quant_weight_static(weight, args).to(self.model_dtype)
        if self.owq:
            weight[:, int(module.buf_n_nonout):] = fp_weight.to(self.model_dtype)
        if self.need_perm:
            weight = weight[:, module.buf_invperm]
        return weight

    def check_status(self):
        """Reads (one sync) the device status words of the tensor-core launches issued so far.  In a
        process group the words are first combined over the ranks (every rank issues the same launches),
        so all ranks raise together."""
        if parallel.world()[1] > 1 and (self._pending_info or self._pending_status):
            if self._pending_info:
                self._pending_info = [parallel.combine_status(torch.cat(self._pending_info).abs(), 'max')]
            if self._pending_status:
                self._pending_status = [parallel.combine_status(torch.cat(self._pending_status), 'min')]
        if self._pending_info:
            infos = torch.cat(self._pending_info).tolist()
            self._pending_info = []
            if any(infos):
                self._pending_status = []
                raise torch.linalg.LinAlgError('cholesky: the dampened Hessian is not positive definite '
                                               f'(potrf info {[i for i in infos if i]})')
        if self._pending_status:
            codes = torch.cat(self._pending_status).tolist()
            self._pending_status = []
            for c in codes:
                if c != 0:
                    if c == L.LC_ERR_NOT_PD:
                        raise torch.linalg.LinAlgError('lc_gptq_factorize: the dampened Hessian is not '
                                                       'positive definite')
                    raise L.LcError('lc_hessian_accum / lc_gptq_factorize / lc_gptq_weight_transform_tc', c, L.status_string(c))

    @torch.no_grad()
    def free(self, name):
        del self.layers_cache[name]
