"""Tapalix on B200: a decoder-only language model with parallel layers (one layer norm with weight and bias feeds the mixer AND
the feed-forward, x <- x + mixer(h) + ff(h)), an fp32 residual stream, a block of layers that runs several times with the same
weights (every pass re-enters through x <- W_in [x ; x0], x0 the scaled embedding, and keeps a cache of its own), latent-vector
attention (with rotated positions, or without positions and with a sigmoid output gate), a mixture of experts with sigmoid scores,
a choice correction, expert groups and a shared expert, and soft-capped logits.

The model owns weights and launches kernels; it has no cache and no loop of its own. `forward(batch, pool)` runs ONE step of the
engine (engine.py): a ragged batch of new tokens of several sequences against the shared page pool (paged.py), logits only for
the rows the caller wants.

Latent attention. A token caches ONE row per layer run: its normed latent vector c (kv_rank numbers) followed by the rotated key
part that all heads share (rot_dim numbers). Keys and values of the heads are never materialised: with k_h = U_h c and v_h = V_h c,
    q_h . k_h = (U_h^T q_h) . c          sum_j p_j v_hj = V_h (sum_j p_j c_j)
so the query is taken into the latent space once per token and head, attention runs over the cache rows as ONE shared key/value
head (key = the whole row, value = its leading kv_rank numbers: p3_attn_window_* with v_pool == k_pool), and the value
up-projection is applied to the attention output. Both per-head products are one batched launch of p3_gemm_any.

Kernels per layer run (csrc/): p3_residual_layernorm (adds the previous run's sublayer outputs to x, norms) -> ONE product for
q | latent | output-gate logits | shared expert gate, up | router logits -> p3_latent_post (latent RMS norm, rotation, cache write, plain query
parts, shared expert activation) -> per-head query absorption -> p3_attn_window_prefill / _decode -> per-head value up-projection
(x sigmoid gate) -> ONE product with [W_o | W_down of the shared expert] over [heads | shared hidden] -> routed experts:
p3_router_sigmoid_groups -> p3_moe_sort -> grouped gate|up product -> p3_glu_silu -> grouped down product -> p3_moe_combine.

Precision. dtype=bfloat16 (serving): matrices, activations that feed a matrix product and the cache are bf16, accumulation is fp32;
positions, angles, scores, softmax, norms, router, gates and the residual sum are fp32. dtype=float32: everything is fp32 on the
FMA pipes (no TF32).
"""
import ctypes as C

import torch
from . import _lib
from ._lib import call, call_struct, ptr
from .configs import TapalixConfig, yarn_frequencies
from .lm_base import PagedLM, _page_slices, _stream


class TapalixB200(PagedLM):
    arch = 'Tapalix'

    def __init__(self, cfg, weights, device='cuda', dtype=torch.bfloat16):
        if not torch.cuda.is_available():
            raise RuntimeError('TapalixB200 needs a CUDA device (sm_100a); there is no CPU fallback')
        _lib.lib()
        if isinstance(cfg, dict):
            cfg = TapalixConfig(cfg)
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError('dtype must be torch.bfloat16 or torch.float32')
        self.cfg, self.dev, self.dtype = cfg, torch.device(device), dtype
        self.W, self.V, self.eps = cfg.width, cfg.vocab_size, cfg.eps
        self._init_products()
        w = weights
        mat = lambda t: t.to(self.dev, dtype).contiguous()                     # matrices: the compute type
        f32 = lambda t: t.to(self.dev, torch.float32).contiguous()            # everything that enters fp32 arithmetic
        self.embed = w['embed'].to(self.dev, torch.bfloat16).contiguous()      # bf16 values are exact in both modes
        self.final_gain, self.final_bias, self.head = f32(w['final.norm']), f32(w['final.norm.b']), mat(w['head'])
        self.loop_in = mat(w['loop.in']) if cfg.loop is not None else None
        self.layers = []
        for i, lc in enumerate(cfg.layers):
            p, m, f = f'l{i}.', lc.mixer, lc.ff
            a = p + 'mix.'
            H, d, dr, dv, R = m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank
            L = dict(cfg=lc, norm=f32(w[p + 'norm1']), norm_b=f32(w[p + 'norm1.b']), c_gain=f32(w[a + 'dkv.norm']))
            if R + dr > 4096:
                raise NotImplementedError(f'layer {i}: a cache row of kv_rank + rot_dim = {R + dr} numbers; the attention kernels '
                                          'take at most 4096')
            for name, shape in ((a + 'q', (H * (d + dr), self.W)), (a + 'dkv', (R + dr, self.W)), (a + 'uk', (H * d, R)),
                                (a + 'uv', (H * dv, R)), (a + 'o', (self.W, H * dv))):
                if tuple(w[name].shape) != shape:
                    raise ValueError(f'{name}: shape {tuple(w[name].shape)}, the config gives {shape}')
            # fused input projection: q | latent and shared turning key | gate logits | shared expert gate | shared expert up | router
            parts, off = [w[a + 'q'], w[a + 'dkv']], H * (d + dr) + R + dr
            L['q_off'], L['c_off'] = 0, H * (d + dr)
            L['g_off'] = L['sg_off'] = L['su_off'] = 0
            if m.gated:
                L['g_off'] = off
                parts.append(w[a + 'g'])
                off += H * dv
            sff = f.shared_ff if f is not None else 0
            if sff:
                L['sg_off'], L['su_off'] = off, off + sff
                parts += [w[p + 'mlp.shared.gate'], w[p + 'mlp.shared.up']]
                off += 2 * sff
            if f is not None:
                # the router's rows ride in the same product (fp32 accumulation of exact bf16 products; all-fp32 in the fp32 mode),
                # padded with zero rows to a multiple of 16 so that small batches keep the weight-streaming kernel
                L['r_off'] = off
                pad = -f.experts % 16
                rw = w[p + 'mlp.router']
                parts += [rw] + ([torch.zeros(pad, self.W, dtype=rw.dtype, device=rw.device)] if pad else [])
                off += f.experts + pad
            L['in_w'], L['n_in'] = mat(torch.cat(parts, 0)), off
            # the key up-projection is folded into the query: per head [kv_rank, dim]; the value up-projection stays [vdim, kv_rank]
            L['uk_t'] = mat(w[a + 'uk'].view(H, d, R).transpose(1, 2))
            L['uv'] = mat(w[a + 'uv'])
            # output projection and the shared expert's down projection read one concatenated activation row
            L['out_w'] = mat(torch.cat([w[a + 'o']] + ([w[p + 'mlp.shared.down']] if sff else []), 1))
            if m.rot is not None:
                fr, mag = yarn_frequencies(m.rot)
                L['freq'], L['rot_mag'], L['rot_n'] = torch.tensor(fr, dtype=torch.float64).to(self.dev, torch.float32), float(mag), m.rot.dims
            else:
                L['freq'], L['rot_mag'], L['rot_n'] = None, 1.0, 0
            L['mma'] = self._attention_tile_rows(H, R + dr, R) == 64
            if f is not None:
                q = p + 'mlp.'
                L['gu'] = mat(torch.stack([torch.cat([w[f'{q}e{e}.gate'], w[f'{q}e{e}.up']], 0) for e in range(f.experts)], 0))
                L['down'] = mat(torch.stack([w[f'{q}e{e}.down'] for e in range(f.experts)], 0))
                L['correction'] = f32(w[q + 'correction']) if (q + 'correction') in w else None
            self.layers.append(L)
        # query rows per attention tile the engine cuts prompt portions into: 64 when every layer takes the tensor-core prefill
        # kernel (csrc/attention_window.cu), else 32
        self.q_tile = 64 if all(L['mma'] for L in self.layers) else 32

    def _attention_tile_rows(self, H, key, R):
        """query rows per prefill tile that the attention launch takes for these sizes (64: its tensor-core kernels); asked of the
        library itself so that the engine's tiles and the kernel's choice cannot disagree"""
        a = _lib.AttnWindowArgs()
        a.q = a.out = a.k_pool = a.v_pool = a.block_table = a.tiles = 256              # aligned stand-ins: nothing is launched
        a.ld_q, a.ld_out, a.n_heads, a.n_kv, a.dim, a.vdim, a.v_ld = H * key, H * R, H, 1, key, R, key
        a.act_f32 = a.cache_f32 = self.f32
        return int(_lib.lib().p3_attn_window_tile_rows(C.byref(a)))

    # ------------------------------------------------------------------ what the engine asks of a model
    def kv_layout(self):
        return self.cfg.kv_layout()

    def prepare(self, max_context):
        """nothing depends on the longest context: angles are formed from the positions in the kernels"""

    def graph_safe(self, b):
        """may this step be captured as a CUDA graph? Not when a mixture layer would read its segment offsets back."""
        return not any(l.ff is not None and self.experts_dense(l.ff, b.T) for l in self.cfg.layers)

    # ------------------------------------------------------------------ one engine step
    def _norm(self, x, add1, add2, L, T, xcat=None, rows=None, R=None):
        """x <- x + add1 + add2; -> layer norm of the new x with L's weight and bias in the activation type (None without L);
        xcat: the new x also goes, in the activation type, to the left half of this [T, 2W] buffer (input of the next pass)"""
        n = T if rows is None else R
        h = torch.empty((n, self.W), dtype=self.dtype, device=self.dev) if L is not None else None
        gain, bias = (L['norm'], L['norm_b']) if L is not None else (None, None)
        call('p3_residual_layernorm', ptr(x), ptr(add1), add1.stride(0) if add1 is not None else 0, ptr(add2),
             add2.stride(0) if add2 is not None else 0, ptr(rows), ptr(gain), ptr(bias), ptr(xcat), 2 * self.W, ptr(h), self.W,
             self.f32, n, self.W, self.eps, _stream())
        return h

    def forward(self, b, pool, trace=None):
        """b: StepBatch, pool: paged.PagePool -> fp32 logits [b.R, vocab] (None when no row is wanted).
        `trace` (a list) receives a copy of the residual stream after every layer run."""
        st, dev, T, W, cfg = _stream(), self.dev, b.T, self.W, self.cfg
        act = self.dtype
        e = lambda *s, dt=torch.float32: torch.empty(s, dtype=dt, device=dev)
        x = e(T, W)
        xcat = e(T, 2 * W, dt=act) if cfg.loop is not None else None          # [x | x0] in the activation type
        call('p3_embed_rows_f32', ptr(self.embed), ptr(b.ids), ptr(x), ptr(xcat[:, W:]) if xcat is not None else None, self.f32,
             T, W, self.V, cfg.embed_scale, 2 * W, st)
        y_mix = y_ff = None                                                   # sublayer outputs still to be added to x
        runs = cfg.runs
        for ri, (li, pass_start) in enumerate(runs):
            L = self.layers[li]
            if pass_start:                                                    # finish the run before, then re-enter through W_in
                self._norm(x, y_mix, y_ff, None, T, xcat=xcat)
                if trace is not None and ri > 0:
                    trace.append(x.clone())
                self.linear(xcat, self.loop_in, x, nxt=L['in_w'])
                h = self._norm(x, None, None, L, T)
            else:
                h = self._norm(x, y_mix, y_ff, L, T)
                if trace is not None and ri > 0:
                    trace.append(x.clone())
            y_mix, y_ff = self._layer(L, ri, h, b, pool, runs[ri + 1][0] if ri + 1 < len(runs) else None)
        final = dict(norm=self.final_gain, norm_b=self.final_bias)
        if trace is not None:
            self._norm(x, y_mix, y_ff, None, T)
            trace.append(x.clone())
            y_mix = y_ff = None
        if not b.R:
            return None
        xn = self._norm(x, y_mix, y_ff, final, T, rows=b.want_rows, R=b.R)
        logits = e(b.R, self.V)
        self.linear(xn, self.head, logits)
        if cfg.logit_scale != 1.0 or cfg.logit_softcap > 0:
            call('p3_logit_softcap', ptr(logits), logits.numel(), cfg.logit_scale, cfg.logit_softcap, st)
        return logits

    def _layer(self, L, ri, h, b, pool, next_li):
        """one layer run on the normed input h -> (mixer output + shared expert, routed experts' output or None), both fp32 [T, W]"""
        st, dev, T, W = _stream(), self.dev, b.T, self.W
        act = self.dtype
        e = lambda *s, dt=torch.float32: torch.empty(s, dtype=dt, device=dev)
        m, f = L['cfg'].mixer, L['cfg'].ff
        H, d, dr, dv, R = m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank
        key = R + dr
        sff = f.shared_ff if f is not None else 0
        cache = pool.k[ri]
        proj = e(T, L['n_in'])
        self.linear(h, L['in_w'], proj, nxt=L['out_w'])
        qp, ql, olat = e(T, H * d, dt=act), e(T, H * key, dt=act), e(T, H * R, dt=act)
        hid = e(T, H * dv + sff, dt=act)
        a = _lib.LatentPostArgs()
        a.proj, a.ld_proj, a.q_off, a.c_off, a.gate_off, a.up_off = ptr(proj), proj.stride(0), L['q_off'], L['c_off'], L['sg_off'], L['su_off']
        a.n_heads, a.dim, a.rot_dim, a.kv_rank, a.rot_n, a.n_ff = H, d, dr, R, L['rot_n'], sff
        a.c_gain, a.eps, a.freq, a.rot_mag = ptr(L['c_gain']), self.eps, ptr(L['freq']), L['rot_mag']
        a.q_plain, a.ld_qp, a.q_lat, a.ld_ql = ptr(qp), qp.stride(0), ptr(ql), ql.stride(0)
        a.hid, a.ld_hid, a.hid_off = ptr(hid), hid.stride(0), H * dv
        a.cache, a.block_table, a.bt_stride = ptr(cache), ptr(pool.block_table), pool.block_table.stride(0)
        a.tok_slot, a.tok_pos, a.T, a.act_f32, a.cache_f32 = ptr(b.tok_slot), ptr(b.tok_pos), T, self.f32, self.f32
        call_struct('p3_latent_post', a, st)
        # queries into the latent space: ql[:, h, :R] = U_h^T q_h
        ev = self._ev()
        self.gemm_any(qp, L['uk_t'], ql, N=R, K=d, ldw=d, batch=(H, d, R * d, key))
        self._ev(ev, 'head_gemm', 2 * T * H * R * d, L['uk_t'].numel() * L['uk_t'].element_size())
        w = _lib.AttnWindowArgs()
        w.q, w.ld_q, w.k_pool, w.v_pool, w.v_ld = ptr(ql), ql.stride(0), ptr(cache), ptr(cache), key
        w.block_table, w.bt_stride = ptr(pool.block_table), pool.block_table.stride(0)
        w.out, w.ld_out = ptr(olat), olat.stride(0)
        w.n_heads, w.n_kv, w.dim, w.vdim, w.scale, w.window = H, 1, key, R, m.scale, 0
        w.act_f32, w.cache_f32 = self.f32, self.f32
        esz = 4 if self.f32 else 2
        if b.n_pf:
            w.tiles, w.n_tiles = ptr(b.pf_tiles), b.n_pf
            ev = self._ev()
            call_struct('p3_attn_window_prefill', w, st)
            self._ev(ev, 'attn_prefill', 2 * (T - b.n_dec) * H * ((b.max_pos + 1) // 2) * (key + R), 0)
        if b.n_dec:
            w.tiles, w.n_tiles = ptr(b.dec_tiles), b.n_dec
            span = b.max_pos + 1
            if L['mma']:
                # one shared K/V head: a request is one CTA per slice (two when the values take two column blocks)
                w.n_splits = _page_slices(b.n_dec * (-(-R // 128) if key > 128 else 1), 2 * -(-span // 128) + 1, merge=0.4)
            else:
                w.n_splits = max(1, min(-(-8 * 148 // b.n_dec), -(-span // 128)))
            ws = e(b.n_dec * H * w.n_splits * (R + 2)) if w.n_splits > 1 else None
            w.ws = ptr(ws)
            ev = self._ev()
            call_struct('p3_attn_window_decode', w, st)
            self._ev(ev, 'attn_decode', 2 * b.n_dec * H * span * (key + R), b.n_dec * span * key * esz)
        # values out of the latent space, times the sigmoid gate: hid[:, h, :] = V_h olat[:, h, :] * sigmoid(g)
        ev = self._ev()
        self.gemm_any(olat, L['uv'], hid, N=dv, K=R, ldw=R, batch=(H, R, dv * R, dv),
                      gate=proj[:, L['g_off']:] if m.gated else None)
        self._ev(ev, 'head_gemm', 2 * T * H * R * dv, L['uv'].numel() * L['uv'].element_size())
        y_mix = e(T, W)
        after = self.layers[next_li]['in_w'] if next_li is not None else self.head
        self.linear(hid, L['out_w'], y_mix, nxt=after if f is None else None)
        if f is None:
            return y_mix, None
        y_ff = e(T, W)
        ids = torch.empty((T, f.top), dtype=torch.int32, device=dev)
        wts = torch.empty((T, f.top), dtype=torch.float32, device=dev)
        call('p3_router_sigmoid_groups', None, 0, self.f32, None, ptr(L['correction']), ptr(proj[:, L['r_off']:]), proj.stride(0),
             T, W, f.experts, f.top, f.groups, f.keep, f.scale, ptr(ids), ptr(wts), st)
        glu = lambda gu, hd, n: call('p3_glu_silu', ptr(gu), ptr(gu[:, f.ff:]), gu.stride(0), ptr(hd), hd.stride(0), self.f32, n,
                                     f.ff, st)
        self.experts(L['gu'], L['down'], f, h, y_ff, T, ids, wts, glu)
        return y_mix, y_ff
