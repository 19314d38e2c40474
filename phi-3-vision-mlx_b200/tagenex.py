"""Tagenex on B200: a decoder-only language model whose layers put the RMS norm on each sublayer's OUTPUT
(x <- x + N1(mixer(x)), x <- x + N2(ff(x))), with an fp32 residual stream, and whose mixer is grouped-query attention with
per-head query/key RMS norm, no rotation, a logarithmic distance penalty, a sliding window, a sink in the softmax denominator,
value mixing with the first mixing layer's values and a per-head sigmoid output gate. Feed-forwards are a clamped gated-linear
unit with biases, or a top-k mixture of such units without biases.

The model owns weights and launches kernels; it has no cache and no loop of its own. `forward(batch, pool)` runs ONE step of the
engine (engine.py): a ragged batch of new tokens of several sequences against the shared page pool (paged.py), logits only for
the rows the caller wants. Prompt portions and single decoded tokens share the step; only the attention launch differs
(32-row tiles vs one CTA per request and K/V head).

Kernels per layer (csrc/): fused q|k|v|gate projection (one GEMM) -> p3_qkv_post (head norms, value mixing, gate sigmoid, paged
K/V write) -> p3_attn_window_prefill / _decode (window, sink, penalty table, gate in the epilogue) -> output projection ->
p3_postnorm_residual (norm of the sublayer output + residual add + activation copy) -> gate|up GEMM (+bias) -> p3_glu_clamped ->
down GEMM (+bias) -> p3_postnorm_residual; mixture layers: p3_router_topk -> p3_moe_sort -> grouped gate|up GEMM over gathered
rows -> p3_glu_clamped -> grouped down GEMM -> p3_moe_combine.

Precision. dtype=bfloat16 (serving): matrices, activations that feed a matrix product and the cache are bf16, accumulation is
fp32; positions, penalties, scores, softmax, norms, router, gates, value mixing and the residual sum are fp32. dtype=float32:
everything is fp32 on the FMA pipes (no TF32). Dense bf16 products with K % 8 == 0 run on the tcgen05 GEMM (p3_gemm), everything
else on p3_gemm_any.
"""
import os
import torch
from . import _lib
from ._lib import call, call_struct, ptr
from .configs import TagenexConfig
from .paged import PAGE


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _page_slices(pairs, pages, slots=2 * 148):
    """slices of the visible pages per (request, K/V head) for the tensor-core decode attention (two CTAs per SM). Cost model in
    units of the memory latency: a CTA pays one latency to fill its copy ring and half of one per page after that (two pages in
    flight); equal CTAs run in whole rounds of the resident ones."""
    best, best_cost = 1, float('inf')
    for ns in range(1, max(1, min(pages, 32)) + 1):
        per = -(-pages // ns)
        cost = -(-pairs * ns // slots) * (1.0 + per / 2.0)
        if cost < best_cost - 1e-9:
            best, best_cost = ns, cost
    return best


class StepBatch:
    """Device-side description of one engine step (built by engine.Engine.step)."""
    __slots__ = ('T', 'ids', 'tok_slot', 'tok_pos', 'pf_tiles', 'n_pf', 'dec_tiles', 'n_dec', 'want_rows', 'R', 'max_pos', 'flat')


class TagenexB200:
    arch = 'Tagenex'

    def __init__(self, cfg, weights, device='cuda', dtype=torch.bfloat16):
        if not torch.cuda.is_available():
            raise RuntimeError('TagenexB200 needs a CUDA device (sm_100a); there is no CPU fallback')
        _lib.lib()
        if isinstance(cfg, dict):
            cfg = TagenexConfig(cfg)
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError('dtype must be torch.bfloat16 or torch.float32')
        self.cfg, self.dev, self.dtype = cfg, torch.device(device), dtype
        self.f32 = int(dtype == torch.float32)
        self.W, self.V, self.eps = cfg.width, cfg.vocab_size, cfg.eps
        self.use_tc = os.environ.get('P3_LM_TC', '1') != '0'
        self.moe_dense_rows = int(os.environ.get('P3_LM_MOE_DENSE_ROWS', '1024'))   # (token, choice) pairs from which experts run as dense GEMMs
        self.use_skinny = os.environ.get('P3_LM_SKINNY', '1') != '0' and hasattr(_lib.lib(), 'p3_gemm_skinny')
        w = weights
        mat = lambda t: t.to(self.dev, dtype).contiguous()                     # matrices: the compute type
        f32 = lambda t: t.to(self.dev, torch.float32).contiguous()            # everything that enters fp32 arithmetic
        b16 = lambda t: t.to(self.dev, torch.bfloat16).contiguous()
        self.embed = b16(w['embed'])                                           # bf16 values are exact in both modes
        self.final_gain, self.head = f32(w['final.norm']), mat(w['head'])
        self.layers = []
        for i, lc in enumerate(cfg.layers):
            p, m = f'l{i}.', lc.mixer
            L = dict(cfg=lc, norm1=f32(w[p + 'norm1']))
            a = p + 'mix.'
            L['qkvg'] = mat(torch.cat([w[a + 'q'], w[a + 'k'], w[a + 'v'], w[a + 'g']], 0))
            L['q_gain'], L['k_gain'] = f32(w[a + 'q.norm']), f32(w[a + 'k.norm'])
            L['r1'], L['r2'], L['sink'] = f32(w[a + 'r1']), f32(w[a + 'r2']), f32(w[a + 'sink'])
            L['lam'] = float(w[a + 'vmix'].float()) if m.v_role == 'mix' else 0.0
            L['o'] = mat(w[a + 'o'])
            L['pen'] = None
            L['mma'] = bool(_lib.ATTN_WINDOW_MMA and not self.f32 and m.dim % 16 == 0 and m.vdim % 8 == 0 and m.dim <= 128 and m.vdim <= 128)
            f = lc.ff
            if f is not None:
                L['norm2'] = f32(w[p + 'norm2'])
                q = p + 'mlp.'
                if f.kind == 'dense':
                    L['gu'] = mat(torch.cat([w[q + 'gate'], w[q + 'up']], 0))
                    L['down'] = mat(w[q + 'down'])
                    L['gu_b32'], L['down_b32'] = f32(torch.cat([w[q + 'gate.b'], w[q + 'up.b']], 0)), f32(w[q + 'down.b'])
                    L['gu_b16'], L['down_b16'] = b16(torch.cat([w[q + 'gate.b'], w[q + 'up.b']], 0)), b16(w[q + 'down.b'])
                else:
                    L['gu'] = mat(torch.stack([torch.cat([w[f'{q}e{e}.gate'], w[f'{q}e{e}.up']], 0) for e in range(f.experts)], 0))
                    L['down'] = mat(torch.stack([w[f'{q}e{e}.down'] for e in range(f.experts)], 0))
                    L['router'], L['router_b'] = f32(w[q + 'router']), f32(w[q + 'router.b'])
            self.layers.append(L)
        self._pen_len = 0
        # query rows per attention tile the engine cuts prompt portions into: 64 when every layer takes the tensor-core prefill
        # kernel (bf16, key size % 16 == 0, value size % 8 == 0, both <= 128; csrc/attention_window.cu), else 32
        self.q_tile = 64 if all(L['mma'] for L in self.layers) else 32
        self.profile = None      # bench.py: list of (kind, ev0, ev1, flops, bytes) when instrumenting

    def _ev(self, start=None, kind=None, flops=0, nbytes=0):
        if self.profile is None:
            return None
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        if start is not None:
            self.profile.append((kind, start, e, flops, nbytes))
        return e

    # ------------------------------------------------------------------ what the engine asks of a model
    def kv_layout(self):
        return self.cfg.kv_layout()

    def cache_dtype(self):
        return self.dtype

    def prepare(self, max_context):
        """distance-penalty tables r1_h ln(1 + r2_h d) for every distance a query can see: d < window, or < the longest
        sequence the pool can hold when the layer has no window"""
        if max_context <= self._pen_len:
            return
        for L in self.layers:
            m = L['cfg'].mixer
            n = min(m.window, max_context) if m.window > 0 else max_context
            n = max(n, 1)
            if L['pen'] is None or L['pen'].shape[1] < n:
                L['pen'] = torch.empty((m.heads, n), dtype=torch.float32, device=self.dev)
                call('p3_distance_penalty_table', ptr(L['r1']), ptr(L['r2']), ptr(L['pen']), m.heads, n, _stream())
        self._pen_len = max_context

    def graph_safe(self, b):
        """may this step be captured as a CUDA graph? Not when a mixture layer would read its segment offsets back."""
        return all(l.ff is None or l.ff.kind != 'moe' or b.T * l.ff.top < self.moe_dense_rows or self.f32 or not self.use_tc
                   for l in self.cfg.layers)

    # ------------------------------------------------------------------ matrix products
    def linear(self, x, w, out, bias32=None, bias16=None, nxt=None):
        """out[M,N] (fp32 or act type, by out.dtype) = x[M,K] w[N,K]^T (+ bias). Returns the bias (fp32) that is STILL TO ADD: None
        when the product added it, bias32 when the kernel has no bias input (the weight-streaming kernel of small batches); the
        consumer kernel (activation / output norm) then adds it. `nxt`: the matrix of the next product; the weight-streaming
        kernel pulls its first megabytes into L2 so that they arrive while the small kernels in between run."""
        M, K = x.shape
        N = w.shape[0]
        ev = self._ev()
        try:
            return self._linear(x, w, out, bias32, bias16, nxt)
        finally:
            self._ev(ev, 'gemm', 2 * M * N * K, w.numel() * w.element_size() + x.numel() * x.element_size() + out.numel() * out.element_size())

    L2_PREFETCH_CAP = int(os.environ.get('P3_LM_PF_CAP_MB', '16')) << 20

    def _linear(self, x, w, out, bias32=None, bias16=None, nxt=None):
        M, K = x.shape
        N = w.shape[0]
        aligned = (not self.f32 and K % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)
        if (self.use_skinny and aligned and M <= 16 and K % 64 == 0 and N % 16 == 0 and out.dtype == torch.float32
                and w.is_contiguous()):
            # <= 16 tokens: the product is a stream of the weights; the Phi-3 decode kernel does that at HBM speed
            pf = 0 if nxt is None else min(nxt.numel() * nxt.element_size(), self.L2_PREFETCH_CAP)
            call('p3_gemm_skinny', ptr(x), x.stride(0), None, self.eps, ptr(w), ptr(out), out.stride(0), None, M, N, K,
                 _lib.EPI_F32, None, 0, None, ptr(nxt) if pf else None, pf, _stream())
            return bias32
        if self.use_tc and aligned and (bias32 is None or bias16 is not None):
            epi = _lib.EPI_F32 if out.dtype == torch.float32 else _lib.EPI_NONE
            call('p3_gemm', ptr(x), x.stride(0), ptr(w), w.stride(0), ptr(bias16), ptr(out), out.stride(0), None, None,
                 M, N, K, epi, 0, _stream())
            return None
        self.gemm_any(x, w, out, bias32)
        return None

    def gemm_any(self, x, w, out, bias=None, rows=None, row_div=1, seg=None, n_groups=0, M=None):
        a = _lib.GemmAnyArgs()
        a.X, a.ldx, a.x_f32 = ptr(x), x.stride(0), self.f32
        a.x_rows, a.x_row_div = ptr(rows), row_div
        a.W, a.ldw, a.w_f32 = ptr(w), w.stride(-2), self.f32
        a.w_group_stride = w.stride(0) if w.dim() == 3 else 0
        a.bias, a.bias_group_stride = ptr(bias), (bias.stride(0) if bias is not None and bias.dim() == 2 else 0)
        a.out, a.ldo, a.out_f32 = ptr(out), out.stride(0), int(out.dtype == torch.float32)
        a.M, a.N, a.K = (x.shape[0] if M is None else M), w.shape[-2], w.shape[-1]
        a.seg_offsets, a.n_groups = ptr(seg), n_groups
        call_struct('p3_gemm_any', a, _stream())
        return out

    # ------------------------------------------------------------------ one engine step
    def forward(self, b, pool, trace=None):
        """b: StepBatch, pool: paged.PagePool -> fp32 logits [b.R, vocab] (None when no row is wanted).
        `trace` (a list) receives a copy of the residual stream after every layer."""
        st, dev, T, W = _stream(), self.dev, b.T, self.W
        act = self.dtype
        e = lambda *s, dt=torch.float32: torch.empty(s, dtype=dt, device=dev)
        x, xa = e(T, W), e(T, W, dt=act)
        call('p3_embed_rows_f32', ptr(self.embed), ptr(b.ids), ptr(x), ptr(xa), self.f32, T, W, self.V, st)
        v_first = None
        y = e(T, W)
        for li, L in enumerate(self.layers):
            m = L['cfg'].mixer
            H, G, d, dv = m.heads, m.kv_heads, m.dim, m.vdim
            nq, nk, nv = H * d, G * d, G * dv
            proj = e(T, nq + nk + nv + H)
            self.linear(xa, L['qkvg'], proj, nxt=L['o'])
            q, gate, att = e(T, nq, dt=act), e(T, H), e(T, H * dv, dt=act)
            if m.v_role != 'none' and v_first is None:
                v_first = e(T, nv)
            a = _lib.QkvPostArgs()
            a.proj, a.ld_proj, a.q_off, a.k_off, a.v_off, a.g_off = ptr(proj), proj.stride(0), 0, nq, nq + nk, nq + nk + nv
            a.n_heads, a.n_kv, a.dim, a.vdim = H, G, d, dv
            a.q_gain, a.k_gain, a.eps = ptr(L['q_gain']), ptr(L['k_gain']), self.eps
            a.v_mode = {'none': 0, 'source': 1, 'mix': 2}[m.v_role]
            a.v_first, a.v_lambda = (ptr(v_first) if a.v_mode else None), L['lam']
            a.q_out, a.ld_q, a.gate_out = ptr(q), q.stride(0), ptr(gate)
            a.k_pool, a.v_pool = ptr(pool.k[li]), ptr(pool.v[li])
            a.block_table, a.bt_stride = ptr(pool.block_table), pool.block_table.stride(0)
            a.tok_slot, a.tok_pos, a.T, a.act_f32, a.cache_f32 = ptr(b.tok_slot), ptr(b.tok_pos), T, self.f32, self.f32
            call_struct('p3_qkv_post', a, st)
            w = _lib.AttnWindowArgs()
            w.q, w.ld_q, w.k_pool, w.v_pool = ptr(q), q.stride(0), ptr(pool.k[li]), ptr(pool.v[li])
            w.block_table, w.bt_stride = ptr(pool.block_table), pool.block_table.stride(0)
            w.sink, w.penalty, w.n_penalty, w.gate = ptr(L['sink']), ptr(L['pen']), L['pen'].shape[1], ptr(gate)
            w.out, w.ld_out = ptr(att), att.stride(0)
            w.n_heads, w.n_kv, w.dim, w.vdim, w.scale, w.window = H, G, d, dv, m.scale, m.window
            w.act_f32, w.cache_f32 = self.f32, self.f32
            esz = 4 if self.f32 else 2
            if b.n_pf:
                w.tiles, w.n_tiles = ptr(b.pf_tiles), b.n_pf
                ev = self._ev()
                call_struct('p3_attn_window_prefill', w, st)
                span = min(m.window, b.max_pos + 1) if m.window else (b.max_pos + 1) // 2
                self._ev(ev, 'attn_prefill', 2 * (T - b.n_dec) * H * span * (d + dv), 0)
            if b.n_dec:
                w.tiles, w.n_tiles = ptr(b.dec_tiles), b.n_dec
                span = min(m.window, b.max_pos + 1) if m.window else b.max_pos + 1
                if L['mma']:
                    w.n_splits = _page_slices(b.n_dec * G, 2 * -(-span // 128) + 1)
                else:
                    # one key per lane: enough CTAs for eight per SM, at least 128 keys (one pass of a CTA) per slice
                    w.n_splits = max(1, min(-(-8 * 148 // (b.n_dec * G)), -(-span // 128)))
                ws = e(b.n_dec * H * w.n_splits * (dv + 2)) if w.n_splits > 1 else None
                w.ws = ptr(ws)
                ev = self._ev()
                call_struct('p3_attn_window_decode', w, st)
                span = min(m.window, b.max_pos + 1) if m.window else b.max_pos + 1
                self._ev(ev, 'attn_decode', 2 * b.n_dec * H * span * (d + dv), b.n_dec * G * span * (d + dv) * esz)
            f = L['cfg'].ff
            after = self.layers[li + 1]['qkvg'] if li + 1 < len(self.layers) else self.head
            self.linear(att, L['o'], y, nxt=L['gu'] if f is not None and f.kind == 'dense' else (after if f is None else None))
            call('p3_postnorm_residual', ptr(y), y.stride(0), None, ptr(L['norm1']), ptr(x), ptr(xa), self.f32, T, W, self.eps, st)
            f = L['cfg'].ff
            if f is not None:
                if f.kind == 'dense':
                    gu, hid = e(T, 2 * f.ff), e(T, f.ff, dt=act)
                    left = self.linear(xa, L['gu'], gu, L['gu_b32'], L['gu_b16'], nxt=L['down'])
                    call('p3_glu_clamped', ptr(gu), gu.stride(0), ptr(hid), hid.stride(0), self.f32, T, f.ff, f.limit,
                         TagenexConfig.GLU_ALPHA, ptr(left), st)
                    left = self.linear(hid, L['down'], y, L['down_b32'], L['down_b16'], nxt=after)
                else:
                    self._moe(L, f, xa, y, T)
                    left = None
                call('p3_postnorm_residual', ptr(y), y.stride(0), ptr(left), ptr(L['norm2']), ptr(x), ptr(xa), self.f32, T, W,
                     self.eps, st)
            if trace is not None:
                trace.append(x.clone())
        if not b.R:
            return None
        xn = e(b.R, W, dt=act)
        call('p3_rmsnorm_rows_f32', ptr(x), ptr(b.want_rows), ptr(self.final_gain), ptr(xn), self.f32, b.R, W, self.eps, st)
        logits = e(b.R, self.V)
        self.linear(xn, self.head, logits)
        return logits

    def _moe(self, L, f, xa, y, T):
        """top-k mixture: route, sort the (token, choice) pairs by expert, two grouped products over the sorted rows, combine"""
        st, dev, n = _stream(), self.dev, T * f.top
        ids = torch.empty((T, f.top), dtype=torch.int32, device=dev)
        wts = torch.empty((T, f.top), dtype=torch.float32, device=dev)
        call('p3_router_topk', ptr(xa), xa.stride(0), self.f32, ptr(L['router']), ptr(L['router_b']), T, self.W, f.experts, f.top,
             ptr(ids), ptr(wts), st)
        seg = torch.empty(f.experts + 1, dtype=torch.int32, device=dev)
        order = torch.empty(n, dtype=torch.int32, device=dev)
        where = torch.empty(n, dtype=torch.int32, device=dev)
        call('p3_moe_sort', ptr(ids), n, f.experts, ptr(seg), ptr(order), ptr(where), st)
        gu = torch.empty((n, 2 * f.ff), dtype=torch.float32, device=dev)
        hid = torch.empty((n, f.ff), dtype=self.dtype, device=dev)
        dn = torch.empty((n, self.W), dtype=torch.float32, device=dev)
        # Large batches (prompt portions): the segment offsets are read back (one small D2H per mixture layer) and every expert's
        # rows go through the tcgen05 GEMM as a dense product over the gathered, expert-ordered activations. Small batches stay
        # on the device-side grouped kernel, which needs no host knowledge of the counts.
        dense = (self.use_tc and not self.f32 and n >= self.moe_dense_rows and self.W % 8 == 0 and f.ff % 8 == 0)
        ev = self._ev()
        if dense:
            xs = torch.empty((n, self.W), dtype=self.dtype, device=dev)
            call('p3_gather_rows', ptr(xa), xa.stride(0), self.f32, ptr(order), f.top, ptr(xs), n, self.W, st)
            cut = seg.tolist()
            for ex in range(f.experts):
                a0, a1 = cut[ex], cut[ex + 1]
                if a1 > a0:
                    call('p3_gemm', ptr(xs[a0:a1]), xs.stride(0), ptr(L['gu'][ex]), L['gu'].stride(1), None, ptr(gu[a0:a1]), gu.stride(0),
                         None, None, a1 - a0, 2 * f.ff, self.W, _lib.EPI_F32, 0, st)
        else:
            self.gemm_any(xa, L['gu'], gu, rows=order, row_div=f.top, seg=seg, n_groups=f.experts, M=n)
        self._ev(ev, 'moe_gemm', 2 * n * 2 * f.ff * self.W, L['gu'].numel() * L['gu'].element_size())
        call('p3_glu_clamped', ptr(gu), gu.stride(0), ptr(hid), hid.stride(0), self.f32, n, f.ff, f.limit, TagenexConfig.GLU_ALPHA,
             None, st)
        ev = self._ev()
        if dense:
            for ex in range(f.experts):
                a0, a1 = cut[ex], cut[ex + 1]
                if a1 > a0:
                    call('p3_gemm', ptr(hid[a0:a1]), hid.stride(0), ptr(L['down'][ex]), L['down'].stride(1), None, ptr(dn[a0:a1]),
                         dn.stride(0), None, None, a1 - a0, self.W, f.ff, _lib.EPI_F32, 0, st)
        else:
            self.gemm_any(hid, L['down'], dn, seg=seg, n_groups=f.experts, M=n)
        self._ev(ev, 'moe_gemm', 2 * n * f.ff * self.W, L['down'].numel() * L['down'].element_size())
        call('p3_moe_combine', ptr(dn), dn.stride(0), ptr(where), ptr(wts), f.top, ptr(y), T, self.W, st)
