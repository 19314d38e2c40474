"""Tagenex on the continuous-batching engine against the plain CPU restatement (oracle/tagenex_oracle.py).

Small random checkpoints of several shapes; the CUDA path (model, page pool, engine, scheduler, public API, trace runner) must
give the oracle's logits whatever the schedule: whole prompts, token-by-token decoding, portions down to two tokens, mixed
batches, reused pages and slots. Attention edges are probed at the kernel level with inputs in which single keys dominate.
"""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F32, B16 = torch.float32, torch.bfloat16
TOL = {F32: 2e-4, B16: 8e-2}


@pytest.fixture(scope='module')
def lib(dev):
    import phi3_b200  # noqa: F401
    from phi3_b200 import _lib
    _lib.lib()
    return _lib


def _mods():
    import phi3_b200  # noqa: F401
    from phi3_b200 import configs, weights, engine, tagenex, paged
    from oracle import tagenex_oracle as O
    return configs, weights, engine, tagenex, paged, O


def row_err(got, ref):
    """per row: rms of the mean-free difference, relative to the spread of the reference"""
    got, ref = got.double().cpu(), ref.double().cpu()
    d = got - ref
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / ref.std()


def rel_err(got, ref):
    return float(row_err(got, ref).max())


def assert_close(got, ref, dtype, what=''):
    """fp32: every row within 2e-4. bf16: rounding may flip a near-tie of the router for a few tokens (random weights have
    such ties) and such a token then differs by its whole feed-forward output, so nine rows in ten must be within the rounding
    bound and the median well inside it"""
    e = row_err(got, ref)
    if dtype == F32:
        assert float(e.max()) < TOL[F32], (what, float(e.max()))
    else:
        q = torch.quantile(e, torch.tensor([0.5, 0.9], dtype=e.dtype))
        assert float(q[0]) < 0.04 and float(q[1]) < TOL[B16], (what, q.tolist(), float(e.max()))


def make(cfg_dict, dtype, seed=0):
    configs, weights, engine, tagenex, paged, O = _mods()
    w = weights.random_tagenex_weights(cfg_dict, seed)
    return tagenex.TagenexB200(cfg_dict, w, dtype=dtype), w


def tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def run_schedule(model, toks, cuts, max_tokens=None, engine=None, rid='r'):
    """feed `toks` in portions of the given sizes (the rest one by one); logits of every position, in order"""
    configs, weights, eng_mod, *_ = _mods()
    eng = engine or eng_mod.Engine(model, max_tokens or len(toks) + 64, 4)
    out, at = [], 0
    sizes = list(cuts)
    while at < len(toks):
        n = sizes.pop(0) if sizes else 1
        n = min(n, len(toks) - at)
        out.append(eng.step([(rid, toks[at:at + n], list(range(n)))]))
        at += n
    eng.finish(rid)
    return torch.cat(out, 0)


# ------------------------------------------------------------------------------------------------ whole model, schedules
@pytest.mark.parametrize('dtype', [F32, B16])
def test_whole_prompt_and_every_layer_match_the_oracle(lib, dtype):
    configs, weights, engine, tagenex, paged, O = _mods()
    cfg = configs.tiny_tagenex()
    model, w = make(cfg, dtype)
    toks = tokens(150, cfg['vocab'], 1)                       # longer than every window (33, 50, 100) and two pages
    ref_trace = []
    ref = O.forward(cfg, w, toks, torch.float64, ref_trace)
    eng = engine.Engine(model, 256, 4)
    trace = []
    got = eng.step([('a', toks, list(range(len(toks))))], ['a'], trace=trace)
    assert_close(got, ref, dtype)
    if dtype == F32:
        for i, (g, r) in enumerate(zip(trace, ref_trace)):
            assert (g.cpu().double() - r).abs().max() < 2e-4, f'residual stream after layer {i}'
    assert eng.pool.free_pages and len(eng.pool.free_pages) == eng.pool.n_pages and len(eng.pool.free_slots) == 4


@pytest.mark.parametrize('dtype', [F32, B16])
def test_prefill_then_token_by_token_decoding(lib, dtype):
    configs, weights, engine, tagenex, paged, O = _mods()
    cfg = configs.tiny_tagenex()
    model, w = make(cfg, dtype, seed=2)
    toks = tokens(140, cfg['vocab'], 3)
    ref = O.forward(cfg, w, toks, torch.float64)
    got = run_schedule(model, toks, [30])                     # 110 decoded tokens: every window and two page borders pass by
    assert_close(got, ref, dtype)
    whole = run_schedule(model, toks, [len(toks)])
    if dtype == F32:
        assert rel_err(got, whole) < 1e-5
    else:
        assert_close(got, whole, dtype)


@pytest.mark.parametrize('cuts', [[2, 2, 3, 31, 33, 2, 64, 1, 2], [63, 2, 63, 2], [1, 1, 64, 65], [100, 2, 2]])
def test_prompt_portions_of_any_size(lib, cuts):
    configs, weights, engine, tagenex, paged, O = _mods()
    cfg = configs.tiny_tagenex()
    model, w = make(cfg, F32, seed=4)
    toks = tokens(sum(cuts) + 5, cfg['vocab'], 5)
    ref = O.forward(cfg, w, toks, torch.float64)
    assert rel_err(run_schedule(model, toks, cuts), ref) < TOL[F32]


@pytest.mark.parametrize('dtype', [F32, B16])
def test_mixed_batch_of_unequal_requests_equals_each_alone(lib, dtype):
    configs, weights, engine, tagenex, paged, O = _mods()
    cfg = configs.tiny_tagenex()
    model, w = make(cfg, dtype, seed=6)
    lens = {'a': 150, 'b': 37, 'c': 2, 'd': 90}
    toks = {k: tokens(n, cfg['vocab'], 10 + i) for i, (k, n) in enumerate(lens.items())}
    alone = {k: run_schedule(model, t, [len(t)]) for k, t in toks.items()}
    eng = engine.Engine(model, 64 * 8, 4)
    plan = {'a': [40, 1, 1, 33, 1, 2, 72], 'b': [1, 30, 1, 1, 1, 3], 'c': [1, 1], 'd': [64, 1, 25]}   # sizes per step; 0-padded
    at = {k: 0 for k in toks}
    got = {k: [] for k in toks}
    for s in range(max(len(v) for v in plan.values())):
        entries = []
        for k in toks:
            if s < len(plan[k]) and at[k] < lens[k]:
                n = min(plan[k][s], lens[k] - at[k])
                entries.append((k, toks[k][at[k]:at[k] + n], list(range(n))))
                at[k] += n
        lg = eng.step(entries)
        o = 0
        for k, t, wnt in entries:
            got[k].append(lg[o:o + len(wnt)])
            o += len(wnt)
    for k in toks:
        assert at[k] == lens[k]
        if dtype == F32:
            assert rel_err(torch.cat(got[k], 0), alone[k]) < 1e-5, k
        else:
            assert_close(torch.cat(got[k], 0), alone[k], dtype, k)
        assert_close(torch.cat(got[k], 0), O.forward(cfg, w, toks[k], torch.float64), dtype, k)


def test_pages_and_slots_are_given_back_and_used_again(lib):
    configs, weights, engine, tagenex, paged, O = _mods()
    cfg = configs.tiny_tagenex()
    model, w = make(cfg, F32, seed=7)
    eng = engine.Engine(model, 64 * 4, 2)                     # four pages, two slots
    for k in eng.pool.k + eng.pool.v:
        k.fill_(300.0)                                        # whatever an earlier owner left must never be read
    seen = []
    for r in range(5):
        n = [130, 200, 70, 256, 129][r]
        toks = tokens(n, cfg['vocab'], 20 + r)
        got = run_schedule(model, toks, [50, 3, 70], engine=eng, rid=f'r{r}')
        assert rel_err(got, O.forward(cfg, w, toks, torch.float64)) < TOL[F32], r
        seen.append(len(eng.pool.free_pages))
    assert seen == [4] * 5 and sorted(eng.pool.free_slots) == [0, 1]
    # two live requests interleaved, one leaves, a third takes its slot and pages while the other goes on
    ta, tb, tc = tokens(100, cfg['vocab'], 31), tokens(60, cfg['vocab'], 32), tokens(120, cfg['vocab'], 33)
    la = [eng.step([('a', ta[:50], list(range(50))), ('b', tb, list(range(60)))], ['b'])]
    la.append(eng.step([('a', ta[50:], list(range(50))), ('c', tc[:64], list(range(64)))]))
    lc = [la[1][50:], eng.step([('c', tc[64:], list(range(56)))], ['a', 'c'])]
    with pytest.raises(paged.PoolExhausted):
        eng.step([('x', tokens(64 * 5, cfg['vocab'], 1), [])])
    assert rel_err(torch.cat([la[0][:50], la[1][:50]], 0), O.forward(cfg, w, ta, torch.float64)) < TOL[F32]
    assert rel_err(torch.cat(lc, 0), O.forward(cfg, w, tc, torch.float64)) < TOL[F32]


def test_first_tokens_and_long_decoding(lib):
    configs, weights, engine, tagenex, paged, O = _mods()
    cfg = configs.tiny_tagenex()
    model, w = make(cfg, F32, seed=8)
    for n in (1, 2, 3):
        toks = tokens(n, cfg['vocab'], 40 + n)
        assert rel_err(run_schedule(model, toks, [n]), O.forward(cfg, w, toks, torch.float64)) < TOL[F32]
    toks = tokens(230, cfg['vocab'], 44)
    assert rel_err(run_schedule(model, toks, [1]), O.forward(cfg, w, toks, torch.float64)) < TOL[F32]   # all decoded one by one


@pytest.mark.parametrize('dtype', [F32, B16])
def test_captured_decode_steps_equal_eager_steps(lib, dtype):
    """decode-only steps replay a CUDA graph from their third occurrence on; the logits must be those of eager launches, bit for
    bit, while requests sit out steps, leave, hand their slot and pages to a newcomer, and the longest context passes a
    128-key bucket"""
    configs, weights, engine, tagenex, paged, O = _mods()
    cfg = configs.tiny_tagenex()
    model, w = make(cfg, dtype, seed=9)
    seqs = {k: tokens(n + 24, cfg['vocab'], 50 + i) for i, (k, n) in enumerate({'a': 120, 'b': 5, 'c': 70, 'd': 66}.items())}
    n_prompt = {'a': 120, 'b': 5, 'c': 70, 'd': 66}

    def run(graphs):
        eng = engine.Engine(model, 64 * 10, 4)
        eng.use_graphs = graphs
        for k in eng.pool.k + eng.pool.v:
            k.fill_(7.0)
        got = {k: [] for k in seqs}
        at = dict(n_prompt)

        def step(names, end=()):
            entries = []
            for k in names:
                n = n_prompt[k] if not got[k] else 1
                lo = 0 if not got[k] else at[k]
                entries.append((k, seqs[k][lo:lo + n], [n - 1]))
                at[k] = lo + n
            lg = eng.step(entries, end)
            for i, k in enumerate(names):
                got[k].append(lg[i:i + 1])

        step(['a', 'b', 'c'])
        for s in range(20):
            live = ['a', 'c'] if 8 <= s < 12 else ['a', 'b', 'c']                  # b sits out four steps
            if s < 15:
                step(live)
            elif s == 15:
                step(live, ['c'])                                                # c leaves ...
                step(['d'])                                                      # ... and d takes its slot and pages
            else:
                step(['a', 'b', 'd'])
        return {k: torch.cat(v, 0) for k, v in got.items()}, eng

    eager, _ = run(False)
    replay, eng = run(True)
    assert any('graph' in g for g in eng._graphs.values()), 'no step was captured'
    for k in seqs:
        assert torch.equal(eager[k], replay[k]), k
        n = eager[k].shape[0]
        ref = O.forward(cfg, w, seqs[k][:n_prompt[k] + n - 1], torch.float64)[n_prompt[k] - 1:]
        assert_close(replay[k], ref, dtype, k)


def _att(heads, kv, dim, vdim, win, mix, scale=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale or dim ** -0.5, v_mix=mix)
    if win:
        m['mask'] = {'size': win}
    return {'type': 'attention', 'mixer': m}


OTHER = {
    'equal_heads_top_all': [dict(_att(4, 4, 32, 32, 40, True), mlp={'kind': 'moe', 'expert': {'ff': 48, 'limit': 1.0},
                                                                        'router': {'experts': 4, 'top': 4}}),
                            dict(_att(4, 4, 32, 32, 40, True), mlp={'kind': 'dense', 'ff': 64, 'limit': 3.0})],
    'top_one_single_head': [dict(_att(1, 1, 20, 12, 1, False), mlp={'kind': 'moe', 'expert': {'ff': 24, 'limit': 2.0},
                                                                       'router': {'experts': 6, 'top': 1}}),
                            dict(_att(2, 1, 20, 12, 2, True), mlp={'kind': 'moe', 'expert': {'ff': 24, 'limit': 2.0},
                                                                   'router': {'experts': 1, 'top': 1}})],
    'wide_heads_many_per_group': [dict(_att(10, 1, 136, 72, 64, False, 0.05), mlp=None),
                                  dict(_att(20, 2, 8, 40, 65, True, 0.3), mlp={'kind': 'dense', 'ff': 30, 'limit': 0.5})],
}


@pytest.mark.parametrize('name', sorted(OTHER))
@pytest.mark.parametrize('width', [64, 100])                 # 100: not a multiple of 8 (no tensor-core route in bf16)
def test_other_sizes(lib, name, width):
    configs, weights, engine, tagenex, paged, O = _mods()
    cfg = configs.tiny_tagenex(width=width, vocab=131, layers=OTHER[name], eps=1e-6)
    toks = tokens(135, cfg['vocab'], 50)
    for dtype in (F32, B16):
        model, w = make(cfg, dtype, seed=9)
        ref = O.forward(cfg, w, toks, torch.float64)
        assert_close(run_schedule(model, toks, [70, 2, 31]), ref, dtype, name)


def test_small_batches_take_the_weight_streaming_products(lib):
    """sizes at which every dense product of a decode step (K % 64 == 0, N % 16 == 0, <= 16 rows) goes to the weight-streaming
    kernel, biases added by the consumer kernels: decoded logits must equal the prompt path's and the oracle's"""
    configs, weights, engine, tagenex, paged, O = _mods()
    layers = [dict(_att(16, 4, 16, 16, 40, True), mlp={'kind': 'dense', 'ff': 192, 'limit': 2.0}),
              dict(_att(16, 4, 16, 16, 0, True), mlp={'kind': 'moe', 'expert': {'ff': 64, 'limit': 2.0}, 'router': {'experts': 4, 'top': 2}})]
    cfg = configs.tiny_tagenex(width=128, vocab=208, layers=layers)
    model, w = make(cfg, B16, seed=15)
    assert model.use_skinny
    toks = tokens(100, cfg['vocab'], 16)
    ref = O.forward(cfg, w, toks, torch.float64)
    dec = run_schedule(model, toks, [20])                     # 80 single-token steps
    assert_close(dec, ref, B16)
    eng = engine.Engine(model, 512, 4)                        # 3 requests decoding together (3 rows per product)
    eng.step([(i, toks[:60], []) for i in range(3)])
    together = [eng.step([(i, [toks[60 + s]], [0]) for i in range(3)]) for s in range(40)]
    for i in range(3):
        assert_close(torch.stack([t[i] for t in together]), ref[60:], B16)
    model.use_skinny = False
    assert_close(run_schedule(model, toks, [20]), dec, B16)


def _random_config(rng):
    """a configuration drawn at random: layer count and order, head counts, group sizes, key / value sizes (with and without the
    tensor-core kernels), windows from 1 to beyond the context, layers with and without value mixing, dense / mixture / no
    feed-forward, top from 1 to all experts"""
    width, vocab = rng.choice([64, 96, 128, 160, 200, 256]), rng.choice([97, 256, 1000])
    gv, vd = rng.choice([1, 2, 4]), rng.choice([16, 24, 40, 64])             # value shape shared by the mixing layers
    layers = []
    for _ in range(rng.randint(2, 6)):
        mix = rng.random() < 0.7
        kv = gv if mix else rng.choice([1, 2, 3])
        dim = rng.choice([16, 24, 48, 80, 128])
        m = dict(heads=kv * rng.choice([1, 2, 5, 8]), kv_heads=kv, dim=dim, vdim=vd if mix else rng.choice([8, 20, 48, 128]),
                 scale=rng.choice([dim ** -0.5, 0.05]), v_mix=mix)
        win = rng.choice([0, 1, 7, 33, 64, 100, 129, 300])
        if win:
            m['mask'] = {'size': win}
        k = rng.random()
        if k < 0.15:
            mlp = None
        elif k < 0.55:
            mlp = {'kind': 'dense', 'ff': rng.choice([64, 100, 136]), 'limit': rng.choice([1.0, 7.0])}
        else:
            e = rng.choice([1, 2, 6, 16])
            mlp = {'kind': 'moe', 'expert': {'ff': rng.choice([32, 56]), 'limit': 3.0}, 'router': {'experts': e, 'top': rng.randint(1, e)}}
        layers.append({'type': 'attention', 'mixer': m, 'mlp': mlp})
    return {'architecture': 'Tagenex', 'vocab': vocab, 'width': width, 'norm': {'eps': rng.choice([1e-5, 1e-6])}, 'layers': layers}


@pytest.mark.parametrize('seed', [11, 12, 13, 14])
def test_random_configurations_under_random_schedules(lib, seed):
    """five requests of unequal length through a four-slot engine whose pool holds less than their sum: random portions (down to
    one token) beside decoded tokens, requests that sit out steps, slots and pages taken over by later requests"""
    import random
    configs, weights, engine, tagenex, paged, O = _mods()
    rng = random.Random(seed)
    cfg = _random_config(rng)
    w = weights.random_tagenex_weights(cfg, seed)
    lens = {'a': rng.randint(130, 330), 'b': rng.randint(2, 90), 'c': rng.randint(60, 200), 'd': rng.randint(1, 40), 'e': rng.randint(65, 130)}
    toks = {k: tokens(n, cfg['vocab'], 100 * seed + i) for i, (k, n) in enumerate(lens.items())}
    ref = {k: O.forward(cfg, w, t, torch.float64) for k, t in toks.items()}
    for dtype in (F32, B16):
        model = tagenex.TagenexB200(cfg, w, dtype=dtype)
        eng = engine.Engine(model, 64 * 12, 4)
        for p in eng.pool.k + eng.pool.v:
            p.fill_(9.0)
        at, got = {k: 0 for k in toks}, {k: [] for k in toks}
        waiting, live, srng = list(toks), [], random.Random(seed)
        while waiting or live:
            while waiting and len(live) < 4 and sum(-(-lens[k] // 64) for k in live + waiting[:1]) <= eng.pool.n_pages:
                live.append(waiting.pop(0))
            entries, end = [], []
            for k in live:
                if srng.random() < 0.15 and len(live) > 1:
                    continue
                n = 1 if at[k] > 0.6 * lens[k] else min(lens[k] - at[k], srng.choice([1, 1, 2, 3, 17, 64, 65, 130]))
                entries.append((k, toks[k][at[k]:at[k] + n], list(range(n))))
                at[k] += n
                if at[k] == lens[k]:
                    end.append(k)
            if not entries:
                continue
            lg = eng.step(entries, end)
            o = 0
            for k, t, wnt in entries:
                got[k].append(lg[o:o + len(wnt)])
                o += len(wnt)
            live = [k for k in live if k not in end]
        for k in toks:
            assert_close(torch.cat(got[k], 0), ref[k], dtype, (seed, k, cfg))
        assert len(eng.pool.free_pages) == eng.pool.n_pages and len(eng.pool.free_slots) == 4


# ------------------------------------------------------------------------------------------------ mechanisms alone
def _attention_case(lib, dtype, H, G, d, dv, window, n_ctx, hot, scale=1.0, seed=0, tile_rows=32, n_splits=1):
    """random q/k/v with a few dominant (query, key) pairs `hot` = [(i, j)]: both rows get a large common component so that
    exp(score) of that pair dwarfs the rest and a wrong mask edge changes the output completely. Returns (kernel out via
    prefill tiles, kernel out via decode tiles, oracle) for all n_ctx queries."""
    configs, weights, engine, tagenex, paged, O = _mods()
    from phi3_b200._lib import AttnWindowArgs, call_struct, call, ptr
    dev = torch.device('cuda')
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(n_ctx, H, d, generator=g) * 0.5
    k = torch.randn(n_ctx, G, d, generator=g) * 0.5
    v = torch.randn(n_ctx, G, dv, generator=g)
    for n, (i, j) in enumerate(hot):
        u = torch.zeros(d)
        u[n % d] = 6.0
        q[i] += u
        k[j] += u
    sink = torch.randn(H, generator=g)
    sink[0] = 3.0
    r1, r2 = torch.rand(H, generator=g) + 0.1, torch.rand(H, generator=g) * 0.5 + 0.01
    gate = torch.rand(n_ctx, H, generator=g)
    if dtype == B16:
        q, k, v = q.bfloat16().float(), k.bfloat16().float(), v.bfloat16().float()
    # oracle
    pos = torch.arange(n_ctx)
    kh, vh = k.double().repeat_interleave(H // G, 1), v.double().repeat_interleave(H // G, 1)
    sc = torch.einsum('thd,shd->hts', q.double(), kh) * scale
    sc = sc - O.distance_penalty(r1.double(), r2.double(), (pos[:, None] - pos[None, :]).double())
    a = O.sink_softmax(sc, O.visible(pos, pos, window or None), sink.double())
    ref = torch.einsum('hts,shd->thd', a, vh) * gate.double()[:, :, None]
    # pool with a scrambled page order, other pages filled with large numbers
    n_pg = -(-n_ctx // 64)
    perm = torch.randperm(n_pg + 3, generator=g)[:n_pg]
    kp = torch.full((n_pg + 3, G, 64, d), 50.0)
    vp = torch.full((n_pg + 3, G, 64, dv), 50.0)
    for p in range(n_pg):
        n = min(64, n_ctx - 64 * p)
        kp[perm[p], :, :n] = k[64 * p:64 * p + n].transpose(0, 1)
        vp[perm[p], :, :n] = v[64 * p:64 * p + n].transpose(0, 1)
    bt = torch.zeros(2, n_pg + 3, dtype=torch.int32)
    bt[1, :n_pg] = perm.int()
    kp, vp, qd = kp.to(dev, dtype), vp.to(dev, dtype), q.reshape(n_ctx, H * d).to(dev, dtype).contiguous()
    bt, sink_d, gate_d = bt.to(dev), sink.to(dev), gate.to(dev).contiguous()
    pen = torch.empty(H, max(window, 1) if window else n_ctx, device=dev)
    r1d, r2d = r1.to(dev), r2.to(dev)                        # named: a temporary would be freed (and reused) before the launch
    call('p3_distance_penalty_table', ptr(r1d), ptr(r2d), ptr(pen), H, pen.shape[1], 0)
    outs = []
    for kind in ('prefill', 'decode'):
        if kind == 'prefill':
            tiles = [(r0, min(tile_rows, n_ctx - r0), 1, r0) for r0 in range(0, n_ctx, tile_rows)]
        else:
            tiles = [(r, 1, 1, r) for r in range(n_ctx)]
        td = torch.tensor(tiles, dtype=torch.int32, device=dev).reshape(-1)
        out = torch.zeros(n_ctx, H * dv, dtype=dtype, device=dev)
        a_ = AttnWindowArgs()
        a_.q, a_.ld_q, a_.k_pool, a_.v_pool, a_.block_table, a_.bt_stride = ptr(qd), H * d, ptr(kp), ptr(vp), ptr(bt), bt.stride(0)
        a_.sink, a_.penalty, a_.n_penalty, a_.gate, a_.out, a_.ld_out = ptr(sink_d), ptr(pen), pen.shape[1], ptr(gate_d), ptr(out), H * dv
        a_.n_heads, a_.n_kv, a_.dim, a_.vdim, a_.scale, a_.window = H, G, d, dv, scale, window
        a_.act_f32 = a_.cache_f32 = int(dtype == F32)
        a_.tiles, a_.n_tiles = ptr(td), len(tiles)
        if kind == 'decode' and n_splits > 1:
            ws = torch.empty(len(tiles) * H * n_splits * (dv + 2), device=dev)
            a_.n_splits, a_.ws = n_splits, ptr(ws)
        call_struct('p3_attn_window_' + kind, a_, 0)
        torch.cuda.synchronize()
        outs.append(out.float().cpu().reshape(n_ctx, H, dv))
    return outs[0], outs[1], ref


@pytest.mark.parametrize('window', [0, 1, 2, 63, 64, 65, 100, 129])
@pytest.mark.parametrize('dtype', [F32, B16])
def test_attention_window_edges_far_keys_and_page_borders(lib, window, dtype):
    n = 300
    probes = [63, 64, 127, 128, 191, 192, 299, 131]
    hot = []
    for i in probes:
        if window:
            hot += [(i, i - window + 1)] if i - window + 1 >= 0 else []       # the last key the window keeps
            hot += [(i + 1, i + 1 - window)] if i + 1 < n and i + 1 - window >= 0 else []   # the first it drops (dominant if seen)
        else:
            hot += [(i, 0), (i, 1)]                                            # far keys, at the very start
    hot = [(i, j) for i, j in hot if 0 <= j <= n - 1][:24]
    pf, dc, ref = _attention_case(lib, dtype, H=4, G=2, d=24, dv=40, window=window, n_ctx=n, hot=hot)
    tol = 1e-4 if dtype == F32 else 3e-2
    assert (pf.double() - ref).abs().max() < tol
    assert (dc.double() - ref).abs().max() < tol


@pytest.mark.parametrize('shape', [(32, 40, 64), (128, 128, 64), (64, 8, 32), (16, 72, 64)])
@pytest.mark.parametrize('window', [0, 65, 200])
def test_attention_on_the_tensor_cores_and_with_key_slices(lib, shape, window):
    """bf16 head sizes that take the mma.sync prefill kernel (64-row tiles), and the decode kernel with 3 and 7 key slices"""
    d, dv, rows = shape
    n = 333
    hot = [(i, i - window + 1) for i in (64, 128, 199, 332) if window and i - window + 1 >= 0]
    hot += [(i + 1, i + 1 - window) for i in (64, 128, 199, 331) if window and i + 1 - window >= 0]
    hot += [(i, 0) for i in (63, 64, 332)] if not window else []
    for splits in (3, 7):
        pf, dc, ref = _attention_case(lib, B16, H=6, G=2, d=d, dv=dv, window=window, n_ctx=n, hot=hot, scale=d ** -0.5,
                                      tile_rows=rows, n_splits=splits)
        assert (pf.double() - ref).abs().max() < 3e-2 and (dc.double() - ref).abs().max() < 3e-2
    pf, dc, ref = _attention_case(lib, F32, H=6, G=2, d=d, dv=dv, window=window, n_ctx=n, hot=hot, scale=d ** -0.5, n_splits=5)
    assert (pf.double() - ref).abs().max() < 1e-4 and (dc.double() - ref).abs().max() < 1e-4


@pytest.mark.parametrize('heads', [(20, 1), (4, 4), (16, 1), (18, 2)])
def test_tensor_core_decode_with_small_and_large_head_groups(lib, heads):
    """the query heads of a K/V head are the rows of a 16-row tile: one head, exactly 16, and more than 16 (two passes)"""
    H, G = heads
    hot = [(i, i - 69) for i in (70, 128, 199)] + [(i, i - 70) for i in (71, 129, 199)]
    for splits in (1, 4):
        pf, dc, ref = _attention_case(lib, B16, H=H, G=G, d=32, dv=48, window=70, n_ctx=200, hot=hot, scale=32 ** -0.5,
                                      tile_rows=64, n_splits=splits)
        assert (pf.double() - ref).abs().max() < 3e-2 and (dc.double() - ref).abs().max() < 3e-2


def test_attention_sink_takes_weight_but_has_no_value(lib):
    pf, dc, ref = _attention_case(lib, F32, H=2, G=1, d=16, dv=8, window=5, n_ctx=70, hot=[], seed=3)
    # position 0 sees one key: with a sink of 3 on head 0 its weight is exp(s) / (exp(s) + exp(3)), far from 1
    assert ref[0, 0].abs().max() < 0.6 * ref[0, 1].abs().max() + 1.0
    assert (pf.double() - ref).abs().max() < 1e-4 and (dc.double() - ref).abs().max() < 1e-4


@pytest.mark.parametrize('shape', [(1, 7, 5), (70, 131, 100), (200, 64, 192), (33, 257, 96)])
def test_gemm_any_against_matmul(lib, shape):
    from phi3_b200._lib import GemmAnyArgs, call_struct, ptr
    M, N, K = shape
    dev = torch.device('cuda')
    g = torch.Generator().manual_seed(M + N)
    for dtype, fma in ((F32, 0), (B16, 0), (B16, 1)):
        x = torch.randn(M, K, generator=g).to(dev, dtype)
        w = torch.randn(N, K, generator=g).to(dev, dtype)
        b = torch.randn(N, generator=g).to(dev)
        out = torch.empty(M, N, device=dev)
        a = GemmAnyArgs()
        a.X, a.ldx, a.x_f32, a.x_row_div, a.W, a.ldw, a.w_f32 = ptr(x), K, int(dtype == F32), 1, ptr(w), K, int(dtype == F32)
        a.bias, a.out, a.ldo, a.out_f32, a.M, a.N, a.K, a.force_fma = ptr(b), ptr(out), N, 1, M, N, K, fma
        call_struct('p3_gemm_any', a, 0)
        ref = x.double() @ w.double().T + b.double()
        assert (out.double() - ref).abs().max() < 1e-3 * K ** 0.5


@pytest.mark.parametrize('dtype', [F32, B16])
def test_router_sort_grouped_products_and_combine(lib, dtype):
    """the mixture path alone: a model of one layer whose attention is switched off by a zero output projection"""
    configs, weights, engine, tagenex, paged, O = _mods()
    layers = [dict(_att(2, 1, 16, 16, 8, False), mlp={'kind': 'moe', 'expert': {'ff': 40, 'limit': 1.0},
                                                       'router': {'experts': 7, 'top': 3}})]
    cfg = configs.tiny_tagenex(width=72, vocab=90, layers=layers)
    w = weights.random_tagenex_weights(cfg, 11)
    w['l0.mix.o'].zero_()
    w['l0.norm1'].zero_()
    model = tagenex.TagenexB200(cfg, w, dtype=dtype)
    toks = tokens(200, cfg['vocab'], 12)
    ref_trace, trace = [], []
    O.forward(cfg, w, toks, torch.float64, ref_trace)
    eng = engine.Engine(model, 256, 1)
    eng.step([('a', toks, [])], ['a'], trace=trace)
    x0 = w['embed'].double()[toks]
    ff = ref_trace[0] - x0                                    # norm2(moe(x)) alone
    assert (trace[0].cpu().double() - x0 - ff).abs().max() < (1e-4 if dtype == F32 else 5e-2)
    # router choices equal the oracle's
    from phi3_b200._lib import call, ptr
    xa = x0.to('cuda', dtype)
    ids = torch.empty(200, 3, dtype=torch.int32, device='cuda')
    wts = torch.empty(200, 3, device='cuda')
    L = model.layers[0]
    call('p3_router_topk', ptr(xa), 72, int(dtype == F32), ptr(L['router']), ptr(L['router_b']), 200, 72, 7, 3, ptr(ids), ptr(wts), 0)
    oi, ow = O.route(x0, {k: v.double() for k, v in w.items()}, 'l0.mlp.', 3)
    assert (ids.cpu().long() == oi).float().mean() > 0.99
    same = (ids.cpu().long() == oi).all(-1)
    assert (wts.cpu().double()[same] - ow[same]).abs().max() < 1e-5


def test_experts_as_dense_products_equal_the_grouped_kernel(lib):
    """large batches run every expert's rows through the tensor-core GEMM over gathered activations (segment offsets read back);
    forced here for a small batch and compared with the device-side grouped kernel and the oracle"""
    configs, weights, engine, tagenex, paged, O = _mods()
    cfg = configs.tiny_tagenex()
    model, w = make(cfg, B16, seed=17)
    toks = tokens(150, cfg['vocab'], 18)
    grouped = run_schedule(model, toks, [150])
    model.moe_dense_rows = 1
    dense = run_schedule(model, toks, [150])
    assert_close(dense, grouped, B16)
    assert_close(dense, O.forward(cfg, w, toks, torch.float64), B16)
    assert float(row_err(dense, grouped).median()) < 5e-3


def test_qkv_post_norms_value_mixing_gate_and_cache_write(lib):
    configs, weights, engine, tagenex, paged, O = _mods()
    from phi3_b200._lib import QkvPostArgs, call_struct, ptr
    dev = torch.device('cuda')
    T, H, G, d, dv = 70, 3, 3, 20, 12
    g = torch.Generator().manual_seed(5)
    proj = torch.randn(T, H * d + G * d + G * dv + H, generator=g)
    qg, kg = torch.rand(d, generator=g) + 0.5, torch.rand(d, generator=g) + 0.5
    vf = torch.randn(T, G * dv, generator=g)
    lam, eps = 0.3, 1e-3
    pos = torch.arange(T) + 60                                # positions 60..129: three pages
    bt = torch.tensor([[0, 0, 0], [2, 0, 1]], dtype=torch.int32)
    kp, vp = torch.zeros(3, G, 64, d, device=dev), torch.zeros(3, G, 64, dv, device=dev)
    q_out, gate = torch.empty(T, H * d, device=dev), torch.empty(T, H, device=dev)
    a = QkvPostArgs()
    pd, vfd = proj.to(dev), vf.to(dev).clone()
    a.proj, a.ld_proj, a.q_off, a.k_off, a.v_off, a.g_off = ptr(pd), proj.shape[1], 0, H * d, H * d + G * d, H * d + G * d + G * dv
    a.n_heads, a.n_kv, a.dim, a.vdim, a.eps = H, G, d, dv, eps
    qgd, kgd, btd = qg.to(dev), kg.to(dev), bt.to(dev)
    slot, posd = torch.ones(T, dtype=torch.int32, device=dev), pos.int().to(dev)
    a.q_gain, a.k_gain, a.v_first, a.v_mode, a.v_lambda = ptr(qgd), ptr(kgd), ptr(vfd), 2, lam
    a.q_out, a.ld_q, a.gate_out, a.k_pool, a.v_pool = ptr(q_out), H * d, ptr(gate), ptr(kp), ptr(vp)
    a.block_table, a.bt_stride, a.tok_slot, a.tok_pos, a.T, a.act_f32, a.cache_f32 = ptr(btd), 3, ptr(slot), ptr(posd), T, 1, 1
    call_struct('p3_qkv_post', a, 0)
    q = O.rms_norm(proj[:, :H * d].view(T, H, d).double(), qg.double(), eps)
    k = O.rms_norm(proj[:, H * d:H * d + G * d].view(T, G, d).double(), kg.double(), eps)
    v = O.mix_values(proj[:, H * d + G * d:H * d + G * d + G * dv].double(), vf.double(), lam).view(T, G, dv)
    assert (q_out.cpu().double().view(T, H, d) - q).abs().max() < 1e-5
    assert (gate.cpu().double() - torch.sigmoid(proj[:, -H:].double())).abs().max() < 1e-6
    for t in range(T):
        p = int(pos[t])
        page = int(bt[1, p // 64])
        assert (kp[page, :, p % 64].cpu().double() - k[t]).abs().max() < 1e-5
        assert (vp[page, :, p % 64].cpu().double() - v[t]).abs().max() < 1e-5


# ------------------------------------------------------------------------------------------------ public entry points
def test_greedy_generation_through_load_generate_and_the_scheduler(lib, tmp_path):
    configs, weights, engine, tagenex, paged, O = _mods()
    from phi3_b200 import api
    from safetensors.torch import save_file
    cfg = configs.tiny_tagenex()
    w = weights.random_tagenex_weights(cfg, 13)
    json.dump(cfg, open(tmp_path / 'config.json', 'w'))
    save_file(w, str(tmp_path / 'model.safetensors'))
    model, proc = api.load(model_path=str(tmp_path), dtype=F32)
    assert type(model).__name__ == 'TagenexB200'
    prompts = [tokens(n, cfg['vocab'], 60 + n) for n in (70, 3, 130, 20, 65)]
    n_new = 12
    # five requests through two slots and a pool of 8 pages: queueing, portions, slot and page reuse
    from phi3_b200.engine import generate_tokens
    outs = generate_tokens(model, prompts, max_new=n_new, max_tokens=64 * 8, n_slots=2, token_budget=96, chunk=40)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for _ in range(n_new):
            seq.append(int(O.forward(cfg, w, seq, torch.float64)[-1].argmax()))
        assert o == seq[len(p):]
    assert api.generate_batch(prompts[:2], preload=(model, proc), max_tokens=n_new, return_tokens=True) == outs[:2]
    text = api.generate('hello there', preload=(model, proc), max_tokens=5, verbose=False)
    assert isinstance(text, str)


def test_trace_runner_replays_steps(lib, tmp_path):
    configs, weights, engine, tagenex, paged, O = _mods()
    from safetensors.torch import save_file
    import numpy as np
    cfg = configs.tiny_tagenex()
    w = weights.random_tagenex_weights(cfg, 14)
    mdir, out = tmp_path / 'm', tmp_path / 'out'
    mdir.mkdir()
    json.dump(cfg, open(mdir / 'config.json', 'w'))
    save_file(w, str(mdir / 'model.safetensors'))
    a, b = tokens(80, cfg['vocab'], 70), tokens(9, cfg['vocab'], 71)
    steps = [{'step': 0, 'entries': [{'id': 'a', 'tokens': a[:70], 'want': [0, 69]}, {'id': 'b', 'tokens': b[:2], 'want': []}], 'end': []},
             {'step': 1, 'entries': [{'id': 'b', 'tokens': b[2:], 'want': [6]}], 'end': ['b']},
             {'step': 2, 'entries': [{'id': 'a', 'tokens': a[70:71], 'want': []}], 'end': []},
             {'step': 3, 'entries': [{'id': 'a', 'tokens': a[71:], 'want': [8]}], 'end': ['a']}]
    r = subprocess.run([os.path.join(ROOT, 'bin', 'trace_run'), '--model', str(mdir), '--dtype', 'float32', '--out', str(out),
                        '--max-tokens', '192'], input='\n'.join(json.dumps(s) for s in steps) + '\n', capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith('done')] == ['done 0', 'done 1', 'done 2', 'done 3']
    ra, rb = O.forward(cfg, w, a, torch.float64), O.forward(cfg, w, b, torch.float64)
    rd = lambda n: torch.from_numpy(np.fromfile(out / f'{n}.f32', dtype='<f4').reshape(-1, cfg['vocab']))
    assert not (out / '2.f32').exists()
    assert rel_err(rd(0), ra[[0, 69]]) < TOL[F32] and rel_err(rd(1), rb[[8]]) < TOL[F32] and rel_err(rd(3), ra[[79]]) < TOL[F32]
