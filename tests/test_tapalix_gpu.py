"""Tapalix on the continuous-batching engine against the plain CPU restatement (oracle/tapalix_oracle.py).

Small random checkpoints of several shapes; the CUDA path (model, page pool, engine, scheduler, public API, trace runner) must
give the oracle's logits whatever the schedule: whole prompts, token-by-token decoding, portions down to two tokens, mixed
batches, reused pages and slots. Each mechanism is also probed alone at the kernel level, with inputs made so that a fault shows
(one dominant key far back or at a page border, choice scores that are all negative, a gate, odd sizes).
"""
import json
import math
import os
import subprocess

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
    from phi3_b200 import configs, weights, engine, tapalix, paged
    from oracle import tapalix_oracle as O
    return configs, weights, engine, tapalix, paged, O


def row_err(got, ref):
    """per row: rms of the mean-free difference, relative to the spread of the reference"""
    got, ref = got.double().cpu(), ref.double().cpu()
    d = got - ref
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / ref.std()


def rel_err(got, ref):
    return float(row_err(got, ref).max())


def assert_close(got, ref, dtype, what=''):
    """fp32: every row within 2e-4. bf16: rounding may flip a near-tie of the router for a few tokens (random weights have such
    ties) and such a token then differs by a whole expert's output, so nine rows in ten must be within the rounding bound and the
    median well inside it"""
    e = row_err(got, ref)
    if dtype == F32:
        assert float(e.max()) < TOL[F32], (what, float(e.max()))
    else:
        q = torch.quantile(e, torch.tensor([0.5, 0.9], dtype=e.dtype))
        assert float(q[0]) < 0.04 and float(q[1]) < TOL[B16], (what, q.tolist(), float(e.max()))


def make(cfg_dict, dtype, seed=0):
    configs, weights, engine, tapalix, paged, O = _mods()
    w = weights.random_tapalix_weights(cfg_dict, seed)
    return tapalix.TapalixB200(cfg_dict, w, dtype=dtype), w


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
def test_whole_prompt_and_every_layer_run_match_the_oracle(lib, dtype):
    configs, weights, engine, tapalix, paged, O = _mods()
    cfg = configs.tiny_tapalix()
    model, w = make(cfg, dtype)
    toks = tokens(150, cfg['vocab'], 1)                       # more than two pages
    ref_trace = []
    ref = O.forward(cfg, w, toks, torch.float64, ref_trace)
    eng = engine.Engine(model, 256, 4)
    trace = []
    got = eng.step([('a', toks, list(range(len(toks))))], ['a'], trace=trace)
    assert_close(got, ref, dtype)
    assert len(trace) == len(ref_trace) == 6                  # layers 1 and 2 run twice
    if dtype == F32:
        for i, (g, r) in enumerate(zip(trace, ref_trace)):
            assert (g.cpu().double() - r).abs().max() < 2e-4, f'residual stream after layer run {i}'
    assert len(eng.pool.free_pages) == eng.pool.n_pages and len(eng.pool.free_slots) == 4
    assert len(eng.pool.k) == 6                               # one cache per layer RUN


@pytest.mark.parametrize('dtype', [F32, B16])
def test_prefill_then_token_by_token_decoding(lib, dtype):
    configs, weights, engine, tapalix, paged, O = _mods()
    cfg = configs.tiny_tapalix()
    model, w = make(cfg, dtype, seed=2)
    toks = tokens(140, cfg['vocab'], 3)
    ref = O.forward(cfg, w, toks, torch.float64)
    got = run_schedule(model, toks, [30])                     # 110 decoded tokens: two page borders pass by
    assert_close(got, ref, dtype)
    whole = run_schedule(model, toks, [len(toks)])
    if dtype == F32:
        assert rel_err(got, whole) < 1e-5
    else:
        assert_close(got, whole, dtype)


@pytest.mark.parametrize('cuts', [[2, 2, 3, 31, 33, 2, 64, 1, 2], [63, 2, 63, 2], [1, 1, 64, 65], [100, 2, 2]])
def test_prompt_portions_of_any_size(lib, cuts):
    configs, weights, engine, tapalix, paged, O = _mods()
    cfg = configs.tiny_tapalix()
    model, w = make(cfg, F32, seed=4)
    toks = tokens(sum(cuts) + 5, cfg['vocab'], 5)
    ref = O.forward(cfg, w, toks, torch.float64)
    assert rel_err(run_schedule(model, toks, cuts), ref) < TOL[F32]


@pytest.mark.parametrize('dtype', [F32, B16])
def test_mixed_batch_of_unequal_requests_equals_each_alone(lib, dtype):
    configs, weights, engine, tapalix, paged, O = _mods()
    cfg = configs.tiny_tapalix()
    model, w = make(cfg, dtype, seed=6)
    lens = {'a': 150, 'b': 37, 'c': 2, 'd': 90}
    toks = {k: tokens(n, cfg['vocab'], 10 + i) for i, (k, n) in enumerate(lens.items())}
    alone = {k: run_schedule(model, t, [len(t)]) for k, t in toks.items()}
    eng = engine.Engine(model, 64 * 8, 4)
    plan = {'a': [40, 1, 1, 33, 1, 2, 72], 'b': [1, 30, 1, 1, 1, 3], 'c': [1, 1], 'd': [64, 1, 25]}   # sizes per step
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
    configs, weights, engine, tapalix, paged, O = _mods()
    cfg = configs.tiny_tapalix()
    model, w = make(cfg, F32, seed=7)
    eng = engine.Engine(model, 64 * 4, 2)                     # four pages, two slots
    for k in eng.pool.k:
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
    configs, weights, engine, tapalix, paged, O = _mods()
    cfg = configs.tiny_tapalix()
    model, w = make(cfg, F32, seed=8)
    for n in (1, 2, 3):
        toks = tokens(n, cfg['vocab'], 40 + n)
        assert rel_err(run_schedule(model, toks, [n]), O.forward(cfg, w, toks, torch.float64)) < TOL[F32]
    toks = tokens(230, cfg['vocab'], 44)
    assert rel_err(run_schedule(model, toks, [1]), O.forward(cfg, w, toks, torch.float64)) < TOL[F32]   # all decoded one by one


@pytest.mark.parametrize('dtype', [F32, B16])
def test_captured_decode_steps_equal_eager_steps(lib, dtype):
    """decode-only steps replay a CUDA graph from their third occurrence on; the logits must be those of eager launches, bit for
    bit, while requests sit out steps, leave and hand their slot and pages to a newcomer"""
    configs, weights, engine, tapalix, paged, O = _mods()
    cfg = configs.tiny_tapalix()
    model, w = make(cfg, dtype, seed=9)
    n_prompt = {'a': 120, 'b': 5, 'c': 70, 'd': 66}
    seqs = {k: tokens(n + 24, cfg['vocab'], 50 + i) for i, (k, n) in enumerate(n_prompt.items())}

    def run(graphs):
        eng = engine.Engine(model, 64 * 10, 4)
        eng.use_graphs = graphs
        for k in eng.pool.k:
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


def _la(heads, dim, rd, vdim, rank, scale=None, scaling=True, base=10000.0, dims=None):
    rot = {'base': base, 'dims': dims or rd}
    if scaling:
        rot['scaling'] = {'factor': 3.0, 'original': 48, 'fast': 8.0, 'slow': 1.0}
    return {'type': 'latent_attention',
            'mixer': dict(heads=heads, dim=dim, rot_dim=rd, vdim=vdim, kv_rank=rank, scale=scale or (dim + rd) ** -0.5, rot=rot)}


def _la2(heads, dim, vdim, rank, scale=None):
    return {'type': 'latent_attention_2', 'mixer': dict(heads=heads, dim=dim, vdim=vdim, kv_rank=rank, scale=scale or dim ** -0.5)}


def _moe(ff, e, top, groups=None, shared=None, scale=1.0):
    return {'kind': 'moe', 'expert': {'ff': ff},
            'router': dict(experts=e, top=top, scale=scale, **({'groups': {'count': groups[0], 'keep': groups[1]}} if groups else {})),
            **({'shared': {'ff': shared}} if shared else {})}


OTHER = {
    # one head, sizes that are no multiple of 8 (every product on the FMA kernels), one group per expert, all groups kept
    'odd': (52, dict(layers=[dict(_la(1, 12, 6, 20, 28), mlp=_moe(20, 4, 2, (4, 4), 12)),
                             dict(_la2(3, 10, 6, 18), mlp=_moe(12, 3, 3, None, None))], loop=(0, 2, 3))),
    # tensor-core sizes: key rows of 64 and 128 numbers; the whole model is the looped block; top == experts
    'tiles': (128, dict(layers=[dict(_la(4, 32, 16, 32, 48), mlp=_moe(64, 8, 8, (2, 2), 64, scale=2.5)),
                                dict(_la2(8, 64, 32, 128), mlp=_moe(32, 16, 4, (8, 3), 128))], loop=(0, 2, 2))),
    # key rows above 128 numbers (fp32 attention kernels also in bf16), no loop at all, no rotation scaling, no shared expert,
    # a rotation over fewer numbers than the turning part holds
    'wide': (96, dict(layers=[dict(_la(2, 24, 40, 24, 152, scaling=False, base=500.0), mlp=_moe(24, 6, 1, (2, 1), None)),
                              dict(_la(3, 16, 16, 40, 56, dims=8), mlp=None),
                              dict(_la2(2, 40, 24, 200), mlp=_moe(16, 4, 2, (2, 1), 40))], loop=None)),
    # nothing is a multiple of 4, let alone 8; cache rows above 256 numbers in the second layer
    'ragged': (50, dict(layers=[dict(_la(3, 7, 6, 5, 9), mlp=_moe(11, 5, 2, None, 13)),
                                dict(_la(2, 9, 10, 11, 290), mlp=_moe(7, 6, 3, (3, 2), 9)),
                                dict(_la2(3, 11, 7, 13), mlp=_moe(9, 4, 1, (2, 1), None))], loop=(1, 3, 2))),
    # a loop of one layer that runs once, in the middle
    'once': (64, dict(layers=[dict(_la2(2, 16, 16, 32), mlp=None), dict(_la(2, 16, 16, 16, 32), mlp=_moe(16, 4, 2, (2, 1), 16)),
                              dict(_la2(2, 16, 16, 32), mlp=_moe(16, 4, 2, None, 16))], loop=(1, 2, 1))),
}


@pytest.mark.parametrize('name', list(OTHER))
@pytest.mark.parametrize('dtype', [F32, B16])
def test_other_sizes(lib, name, dtype):
    configs, weights, engine, tapalix, paged, O = _mods()
    width, kw = OTHER[name]
    cfg = configs.tiny_tapalix(width=width, vocab=211 if name != 'ragged' else 101, **kw)
    if name == 'wide':
        cfg['logit_softcap'], cfg['logit_scale'] = 0.0, 1.0
        del cfg['embedding']
    model, w = make(cfg, dtype, seed=11)
    toks = tokens(150, cfg['vocab'], 12)
    ref = O.forward(cfg, w, toks, torch.float64)
    assert_close(run_schedule(model, toks, [70, 2, 40]), ref, dtype, name)


def test_small_batches_take_the_weight_streaming_products(lib):
    configs, weights, engine, tapalix, paged, O = _mods()
    cfg = configs.tiny_tapalix(width=128, vocab=256, layers=[dict(_la(4, 32, 32, 32, 64), mlp=_moe(64, 4, 2, (2, 1), 64)),
                                                             dict(_la2(4, 32, 32, 64), mlp=_moe(64, 4, 2, None, 64))], loop=(0, 1, 2))
    model, w = make(cfg, B16, seed=15)
    toks = tokens(40, cfg['vocab'], 16)
    ref = O.forward(cfg, w, toks, torch.float64)
    a = run_schedule(model, toks, [20])
    model.use_skinny = False
    b = run_schedule(model, toks, [20])
    assert_close(a, ref, B16)
    assert_close(b, ref, B16)


def _random_config(rng):
    """a configuration drawn at random: layer count and order of the two mixers, head counts, plain / turning / value / latent
    sizes (with and without the tensor-core kernels), rotation constants, feed-forwards with and without groups and shared expert
    or none at all, the looped block anywhere (or nowhere) with 1 to 3 passes, output constants"""
    width, vocab = rng.choice([64, 96, 128, 160, 200, 256]), rng.choice([97, 256, 1000])
    layers = []
    for _ in range(rng.randint(2, 5)):
        heads, vdim = rng.choice([1, 2, 3, 8, 20]), rng.choice([8, 20, 32, 64])
        if rng.random() < 0.5:
            dim, rd = rng.choice([8, 24, 32, 64]), rng.choice([2, 8, 16, 32])
            rank = rng.choice([16, 40, 64, 96, 112, 240 - rd, 128 - rd])
            layer = _la(heads, dim, rd, vdim, rank, scale=rng.choice([None, 0.07]), scaling=rng.random() < 0.7,
                        base=rng.choice([100.0, 10000.0, 1e6]))
        else:
            layer = _la2(heads, rng.choice([8, 24, 32, 64]), vdim, rng.choice([16, 40, 64, 128, 200]), scale=rng.choice([None, 0.07]))
        k = rng.random()
        if k < 0.2:
            mlp = None
        else:
            groups = rng.choice([None, (1, 1), (2, 1), (2, 2), (4, 2), (4, 3)])
            per = rng.choice([1, 2, 4])
            e = per * (groups[0] if groups else rng.choice([1, 3, 5]))
            top = rng.randint(1, e if not groups else groups[1] * per)
            mlp = _moe(rng.choice([16, 24, 56]), e, top, groups, rng.choice([None, 24, 64]), scale=rng.choice([1.0, 2.5]))
        layers.append(dict(layer, mlp=mlp))
    n = len(layers)
    loop = None
    if rng.random() < 0.8:
        lo = rng.randint(0, n - 1)
        loop = (lo, rng.randint(lo + 1, n), rng.randint(1, 3))
    cfg = {'architecture': 'Tapalix', 'vocab': vocab, 'width': width, 'norm': {'eps': rng.choice([1e-5, 1e-6])},
           'embedding': {'scale': rng.choice([1.0, width ** 0.5])}, 'layers': layers, 'logit_scale': rng.choice([1.0, 0.5, 2.0]),
           'logit_softcap': rng.choice([0.0, 10.0, 30.0])}
    if loop:
        cfg['loop'] = {'start': loop[0], 'stop': loop[1], 'times': loop[2]}
    return cfg


@pytest.mark.parametrize('seed', [11, 12, 13, 14, 15, 16])
def test_random_configurations_under_random_schedules(lib, seed):
    """five requests of unequal length through a four-slot engine whose pool holds less than their sum: random portions (down to
    one token) beside decoded tokens, requests that sit out steps, slots and pages taken over by later requests"""
    import random
    configs, weights, engine, tapalix, paged, O = _mods()
    rng = random.Random(seed)
    cfg = _random_config(rng)
    w = weights.random_tapalix_weights(cfg, seed)
    lens = {'a': rng.randint(130, 330), 'b': rng.randint(2, 90), 'c': rng.randint(60, 200), 'd': rng.randint(1, 40), 'e': rng.randint(65, 130)}
    toks = {k: tokens(n, cfg['vocab'], 100 * seed + i) for i, (k, n) in enumerate(lens.items())}
    ref = {k: O.forward(cfg, w, t, torch.float64) for k, t in toks.items()}
    for dtype in (F32, B16):
        model = tapalix.TapalixB200(cfg, w, dtype=dtype)
        eng = engine.Engine(model, 64 * 12, 4)
        for p in eng.pool.k:
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
def test_residual_sum_and_layer_norm(lib):
    configs, weights, engine, tapalix, paged, O = _mods()
    from phi3_b200._lib import call, ptr
    dev = torch.device('cuda')
    g = torch.Generator().manual_seed(0)
    for W, T in ((52, 7), (1500, 3), (9000, 2)):              # the last is longer than the registers of a row's threads hold
        x, a1, a2 = (torch.randn(T, W, generator=g) * 3 + 1.5 for _ in range(3))
        gain, bias = torch.randn(W, generator=g), torch.randn(W, generator=g)
        xd, a1d, a2d = x.to(dev), a1.to(dev), torch.cat([a2, a2], 1).to(dev)          # the second addend has a wider pitch
        gd, bd = gain.to(dev), bias.to(dev)
        h = torch.empty(T, W, device=dev)
        xa = torch.zeros(T, 2 * W, device=dev)
        call('p3_residual_layernorm', ptr(xd), ptr(a1d), W, ptr(a2d), 2 * W, None, ptr(gd), ptr(bd), ptr(xa), 2 * W, ptr(h), W, 1, T, W,
             1e-5, 0)
        s = (x + a1 + a2).double()
        assert (xd.cpu().double() - s).abs().max() < 1e-5 and (xa[:, :W].cpu().double() - s).abs().max() < 1e-5
        assert float(xa[:, W:].abs().max()) == 0.0
        assert (h.cpu().double() - O.layer_norm(s, gain.double(), bias.double(), 1e-5)).abs().max() < 2e-4
        # chosen rows only, bf16 output, x untouched
        rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=dev)
        hb = torch.empty(2, W, dtype=B16, device=dev)
        keep = xd.clone()
        call('p3_residual_layernorm', ptr(xd), ptr(a1d), W, None, 0, ptr(rows), ptr(gd), ptr(bd), None, 0, ptr(hb), W, 0, 2, W, 1e-5, 0)
        ref = O.layer_norm((s + a1.double())[[T - 1, 0]], gain.double(), bias.double(), 1e-5)
        assert torch.equal(xd, keep) and (hb.cpu().double() - ref).abs().max() < 0.05


@pytest.mark.parametrize('dtype', [F32, B16])
def test_latent_post_norm_rotation_cache_write_and_shared_unit(lib, dtype):
    configs, weights, engine, tapalix, paged, O = _mods()
    from phi3_b200._lib import LatentPostArgs, call_struct, ptr
    dev = torch.device('cuda')
    g = torch.Generator().manual_seed(1)
    H, d, dr, R, rot_n, sff, T = 3, 10, 12, 20, 8, 1100, 6
    rot = {'base': 100.0, 'dims': rot_n, 'scaling': {'factor': 5.0, 'original': 32, 'fast': 4.0, 'slow': 0.5}}
    nq = H * (d + dr)
    n_in = nq + R + dr + 2 * sff
    proj = torch.randn(T, n_in + 3, generator=g)
    gain = torch.randn(R, generator=g)
    slot = torch.tensor([1, 1, 1, 0, 0, 1], dtype=torch.int32)
    pos = torch.tensor([62, 63, 64, 0, 1, 700], dtype=torch.int32)
    bt = torch.zeros(2, 12, dtype=torch.int32)
    bt[0, :1] = 5
    bt[1, :11] = torch.tensor([3, 9, 1, 1, 1, 1, 1, 1, 1, 1, 7], dtype=torch.int32)
    cache = torch.full((12, 1, 64, R + dr), 9.0, dtype=dtype)
    fr, mag = configs.yarn_frequencies(configs.TapalixConfig(configs.tiny_tapalix(layers=[dict(
        {'type': 'latent_attention', 'mixer': dict(heads=H, dim=d, rot_dim=dr, vdim=4, kv_rank=R, scale=1.0, rot=rot)}, mlp=None)],
        loop=None)).layers[0].mixer.rot)
    fo, mo = O.yarn_frequencies(rot)
    assert abs(mag - mo) < 1e-12 and max(abs(a - float(b)) for a, b in zip(fr, fo)) < 1e-12
    assert fr[0] == 1.0 and abs(fr[-1] - 100.0 ** (-6 / 8) / 5.0) < 1e-12            # fastest pair untouched, slowest divided
    pd, gd, sd, posd, btd, cd = proj.to(dev), gain.to(dev), slot.to(dev), pos.to(dev), bt.to(dev), cache.to(dev)
    fd = torch.tensor(fr, dtype=torch.float32, device=dev)
    qp, ql = torch.zeros(T, H * d, dtype=dtype, device=dev), torch.zeros(T, H * (R + dr), dtype=dtype, device=dev)
    hid = torch.zeros(T, 5 + sff, dtype=dtype, device=dev)
    a = LatentPostArgs()
    a.proj, a.ld_proj, a.q_off, a.c_off, a.gate_off, a.up_off = ptr(pd), n_in + 3, 0, nq, nq + R + dr, nq + R + dr + sff
    a.n_heads, a.dim, a.rot_dim, a.kv_rank, a.rot_n, a.n_ff = H, d, dr, R, rot_n, sff
    a.c_gain, a.eps, a.freq, a.rot_mag = ptr(gd), 1e-5, ptr(fd), mag
    a.q_plain, a.ld_qp, a.q_lat, a.ld_ql, a.hid, a.ld_hid, a.hid_off = ptr(qp), H * d, ptr(ql), H * (R + dr), ptr(hid), 5 + sff, 5
    a.cache, a.block_table, a.bt_stride = ptr(cd), ptr(btd), 12
    a.tok_slot, a.tok_pos, a.T = ptr(sd), ptr(posd), T
    a.act_f32 = a.cache_f32 = int(dtype == F32)
    call_struct('p3_latent_post', a, 0)
    torch.cuda.synchronize()
    tol = 1e-4 if dtype == F32 else 3e-2
    P = proj.double()
    q = P[:, :nq].view(T, H, d + dr)
    assert (qp.cpu().double().view(T, H, d) - q[..., :d]).abs().max() < tol
    for t in range(T):
        p1 = torch.tensor([int(pos[t])])
        qr = O.rotate_half(q[t, :, None, d:], p1, rot)[:, 0]                      # [H, dr]; numbers rot_n .. dr pass unchanged
        got = ql.cpu().double().view(T, H, R + dr)[t]
        assert (got[:, R:] - qr).abs().max() < tol and float(got[:, :R].abs().max()) == 0.0
        assert (qr[:, rot_n:] - q[t, :, d + rot_n:]).abs().max() == 0
        c = O.rms_norm(P[t, nq:nq + R], gain.double(), 1e-5)
        kr = O.rotate_half(P[t:t + 1, nq + R:nq + R + dr], p1, rot)[0]
        row = cd.cpu().double()[int(bt[int(slot[t]), int(pos[t]) // 64]), 0, int(pos[t]) % 64]
        assert (row[:R] - c).abs().max() < tol and (row[R:] - kr).abs().max() < tol
    want = O.silu(P[:, nq + R + dr:nq + R + dr + sff]) * P[:, nq + R + dr + sff:nq + R + dr + 2 * sff]
    assert (hid.cpu().double()[:, 5:] - want).abs().max() < tol * 4 and float(hid[:, :5].abs().max()) == 0.0
    assert int((cd.cpu().double() != 9.0).any(-1).sum()) == T                     # one cache row per token, nothing else touched


@pytest.mark.parametrize('dtype', [F32, B16])
@pytest.mark.parametrize('shape', [(3, 10, 6, 18), (4, 32, 16, 64), (16, 64, 64, 128)])
def test_products_per_head_with_gate(lib, dtype, shape):
    """H independent products over column blocks of wider matrices in one launch, as the query absorption and the value
    up-projection use them; with and without the sigmoid gate"""
    configs, weights, engine, tapalix, paged, O = _mods()
    dev = torch.device('cuda')
    H, K, N, T = shape[0], shape[1], shape[2], 70
    g = torch.Generator().manual_seed(2)
    x, w, gate = torch.randn(T, H * K + 8, generator=g), torch.randn(H, N, K, generator=g), torch.randn(T, H * N + 8, generator=g)
    m = type('M', (tapalix.TapalixB200,), {'__init__': lambda self: None})()
    m.dev, m.dtype, m.f32 = dev, dtype, int(dtype == F32)
    xd, wd, gd = x.to(dev, dtype), w.to(dev, dtype), gate.to(dev)
    ref = torch.einsum('thk,hnk->thn', xd.double().cpu()[:, :H * K].view(T, H, K), wd.double().cpu())
    for out_dt in (torch.float32, dtype):
        out = torch.zeros(T, H * N + 4, dtype=out_dt, device=dev)
        m.gemm_any(xd, wd, out, N=N, K=K, ldw=K, batch=(H, K, N * K, N))
        exact = out_dt == F32 and dtype == F32                # else: a bf16 result carries 2^-9 of its size
        near = lambda got, want: bool(((got - want).abs() <= (1e-4 if exact else 0.02 + 0.006 * want.abs())).all())
        assert near(out.double().cpu()[:, :H * N].view(T, H, N), ref)
        assert float(out[:, H * N:].abs().max()) == 0.0
        m.gemm_any(xd, wd, out, N=N, K=K, ldw=K, batch=(H, K, N * K, N), gate=gd[:, 4:])
        want = ref * torch.sigmoid(gate.double()[:, 4:4 + H * N].view(T, H, N))
        assert near(out.double().cpu()[:, :H * N].view(T, H, N), want)


@pytest.mark.parametrize('case', ['random', 'negative', 'no_groups', 'single', 'many'])
def test_router_sigmoid_scores_correction_and_groups(lib, case):
    configs, weights, engine, tapalix, paged, O = _mods()
    from phi3_b200._lib import call, ptr
    dev = torch.device('cuda')
    g = torch.Generator().manual_seed(3)
    E, top, groups, keep, W, T = {'random': (12, 3, 4, 2, 40, 50), 'negative': (8, 3, 2, 1, 24, 40), 'no_groups': (7, 7, 1, 1, 33, 9),
                                  'single': (6, 2, 6, 3, 16, 30), 'many': (256, 8, 8, 4, 64, 20)}[case]
    x = torch.randn(T, W, generator=g)
    Wr = torch.randn(E, W, generator=g) * (2.0 / W ** 0.5)
    corr = torch.randn(E, generator=g) * 0.5
    if case == 'negative':
        corr = corr - 3.0                                     # every choice score below zero: a barred expert counted as 0 would win
    w = {'router': Wr.double(), 'correction': corr.double()}
    rc = dict(experts=E, top=top, scale=2.5, **({'groups': {'count': groups, 'keep': keep}} if groups > 1 else {}))
    ids_ref, wts_ref = O.route(x.double(), w, '', rc)
    xd, wd, cd = x.to(dev), Wr.to(dev), corr.to(dev)
    ids = torch.empty(T, top, dtype=torch.int32, device=dev)
    wts = torch.empty(T, top, device=dev)
    ref = {(t, int(e)): float(v) for t in range(T) for e, v in zip(ids_ref[t], wts_ref[t])}
    logits = torch.zeros(T, E + 3, device=dev)
    logits[:, :E] = (x.double() @ Wr.double().T).float().to(dev)
    for from_logits in (False, True):                         # the kernel forms the logits itself, or takes them from a product
        ids.zero_(), wts.zero_()
        if from_logits:
            call('p3_router_sigmoid_groups', None, 0, 1, None, ptr(cd), ptr(logits), E + 3, T, W, E, top, groups, keep, 2.5, ptr(ids), ptr(wts), 0)
        else:
            call('p3_router_sigmoid_groups', ptr(xd), W, 1, ptr(wd), ptr(cd), None, 0, T, W, E, top, groups, keep, 2.5, ptr(ids), ptr(wts), 0)
        got = {(t, int(e)): float(v) for t in range(T) for e, v in zip(ids[t].cpu(), wts[t].cpu())}
        assert got.keys() == ref.keys()
        assert max(abs(got[k] - ref[k]) for k in ref) < 1e-5
    assert abs(float(wts.sum(-1).mean()) - 2.5) < 1e-4        # weights sum to the router scale, not to 1
    if groups > 1:
        assert all(len({int(e) // (E // groups) for e in ids[t].cpu()}) <= keep for t in range(T))


def _latent_attention_case(lib, dtype, H, key, R, n_ctx, hot, scale=1.0, seed=0, tile_rows=32, n_splits=1):
    """random queries and cache rows with a few dominant (query, key) pairs `hot` = [(i, j)]: both rows get a large common
    component so that exp(score) of that pair dwarfs the rest and a lost or wrongly masked key changes the output completely.
    The value of a token is the leading R numbers of its cache row. Returns (prefill tiles, decode tiles, oracle)."""
    from phi3_b200._lib import AttnWindowArgs, call_struct, ptr
    dev = torch.device('cuda')
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(n_ctx, H, key, generator=g) * 0.5
    k = torch.randn(n_ctx, key, generator=g) * 0.5
    for n, (i, j) in enumerate(hot):
        u = torch.zeros(key)
        u[key - 1 - n % 4] = 6.0                              # in the tail of the row: the part that is key only, not value
        q[i] += u
        k[j] += u
    if dtype == B16:
        q, k = q.bfloat16().float(), k.bfloat16().float()
    sc = torch.einsum('thd,sd->hts', q.double(), k.double()) * scale
    mask = torch.ones(n_ctx, n_ctx, dtype=torch.bool).tril()
    ref = torch.einsum('hts,sd->thd', torch.softmax(sc.masked_fill(~mask, float('-inf')), -1), k.double()[:, :R])
    n_pg = -(-n_ctx // 64)
    perm = torch.randperm(n_pg + 3, generator=g)[:n_pg]
    kp = torch.full((n_pg + 3, 1, 64, key), 50.0)
    for p in range(n_pg):
        n = min(64, n_ctx - 64 * p)
        kp[perm[p], 0, :n] = k[64 * p:64 * p + n]
    bt = torch.zeros(2, n_pg + 3, dtype=torch.int32)
    bt[1, :n_pg] = perm.int()
    kp, qd, bt = kp.to(dev, dtype), q.reshape(n_ctx, H * key).to(dev, dtype).contiguous(), bt.to(dev)
    outs = []
    for kind in ('prefill', 'decode'):
        if kind == 'prefill':
            tiles = [(r0, min(tile_rows, n_ctx - r0), 1, r0) for r0 in range(0, n_ctx, tile_rows)]
        else:
            tiles = [(r, 1, 1, r) for r in range(n_ctx)]
        td = torch.tensor(tiles, dtype=torch.int32, device=dev).reshape(-1)
        out = torch.zeros(n_ctx, H * R, dtype=dtype, device=dev)
        a_ = AttnWindowArgs()
        a_.q, a_.ld_q, a_.k_pool, a_.v_pool, a_.v_ld, a_.block_table, a_.bt_stride = ptr(qd), H * key, ptr(kp), ptr(kp), key, ptr(bt), bt.stride(0)
        a_.out, a_.ld_out = ptr(out), H * R
        a_.n_heads, a_.n_kv, a_.dim, a_.vdim, a_.scale, a_.window = H, 1, key, R, scale, 0
        a_.act_f32 = a_.cache_f32 = int(dtype == F32)
        a_.tiles, a_.n_tiles = ptr(td), len(tiles)
        if kind == 'decode' and n_splits > 1:
            ws = torch.empty(len(tiles) * H * n_splits * (R + 2), device=dev)
            a_.n_splits, a_.ws = n_splits, ptr(ws)
        call_struct('p3_attn_window_' + kind, a_, 0)
        torch.cuda.synchronize()
        outs.append(out.float().cpu().reshape(n_ctx, H, R))
    return outs[0], outs[1], ref


@pytest.mark.parametrize('shape', [(3, 28, 20, 32), (4, 64, 48, 64), (20, 128, 96, 64), (2, 200, 152, 32), (9, 112, 96, 32),
                                   (6, 256, 192, 64), (17, 192, 136, 64), (3, 336, 300, 32), (2, 600, 520, 32)])
@pytest.mark.parametrize('dtype', [F32, B16])
@pytest.mark.parametrize('n_splits', [1, 3])
def test_latent_attention_far_keys_page_borders_and_first_tokens(lib, shape, dtype, n_splits):
    """one shared cache row per token serves as key (whole row) and as value (its leading part), for every query head. Probed:
    keys at the very start seen from far away, keys on both sides of page borders, the key at the query's own position, the first
    positions of a sequence. Shapes cover the fp32 kernels and the tensor-core ones (64-, 128- and 256-wide keys, values in one
    or two column blocks, more than 16 heads) and rows above 256 numbers (key chunks and value column blocks of the fp32 kernels)."""
    H, key, R, tile = shape
    n = 300
    hot = [(299, 0), (298, 1), (191, 2), (131, 63), (132, 64), (133, 65), (200, 127), (201, 128), (64, 64), (63, 63), (128, 128),
           (255, 192), (256, 191), (1, 0), (2, 2), (65, 3)]
    tile = tile if dtype == B16 else 32                       # the fp32 kernels take 32 query rows per tile
    pf, dc, ref = _latent_attention_case(lib, dtype, H, key, R, n, hot, scale=0.7, tile_rows=tile, n_splits=n_splits)
    tol = 1e-4 if dtype == F32 else 3e-2
    assert (pf.double() - ref).abs().max() < tol
    assert (dc.double() - ref).abs().max() < tol
    assert (pf[0].double() - pf[0, :1].double()).abs().max() < tol   # position 0 sees itself only: every head returns that row


def test_silu_unit_and_logit_softcap(lib):
    configs, weights, engine, tapalix, paged, O = _mods()
    from phi3_b200._lib import call, ptr
    dev = torch.device('cuda')
    g = torch.Generator().manual_seed(5)
    gu = (torch.randn(9, 2 * 37 + 3, generator=g) * 3).to(dev)
    for dt in (F32, B16):
        out = torch.zeros(9, 40, dtype=dt, device=dev)
        call('p3_glu_silu', ptr(gu), ptr(gu[:, 37:]), gu.stride(0), ptr(out), 40, int(dt == F32), 9, 37, 0)
        want = O.silu(gu[:, :37].double().cpu()) * gu[:, 37:74].double().cpu()
        assert (out.double().cpu()[:, :37] - want).abs().max() < (1e-5 if dt == F32 else 0.1)
        assert float(out[:, 37:].abs().max()) == 0.0
    lg = (torch.randn(5, 300, generator=g) * 20).to(dev)
    a, b = lg.clone(), lg.clone()
    call('p3_logit_softcap', ptr(a), a.numel(), 1.7, 12.0, 0)
    call('p3_logit_softcap', ptr(b), b.numel(), 0.5, 0.0, 0)
    assert (a.cpu().double() - 12.0 * torch.tanh(lg.cpu().double() * 1.7 / 12.0)).abs().max() < 1e-5
    assert (b.cpu().double() - lg.cpu().double() * 0.5).abs().max() < 1e-6


# ------------------------------------------------------------------------------------------------ public entry points
def test_greedy_generation_through_load_generate_and_the_scheduler(lib, tmp_path):
    configs, weights, engine, tapalix, paged, O = _mods()
    from phi3_b200 import api
    from safetensors.torch import save_file
    cfg = configs.tiny_tapalix()
    w = weights.random_tapalix_weights(cfg, 13)
    json.dump(cfg, open(tmp_path / 'config.json', 'w'))
    save_file(w, str(tmp_path / 'model.safetensors'))
    model, proc = api.load(model_path=str(tmp_path), dtype=F32)
    assert type(model).__name__ == 'TapalixB200'
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
    configs, weights, engine, tapalix, paged, O = _mods()
    from safetensors.torch import save_file
    import numpy as np
    cfg = configs.tiny_tapalix()
    w = weights.random_tapalix_weights(cfg, 14)
    mdir, out = tmp_path / 'm', tmp_path / 'out'
    mdir.mkdir()
    json.dump(cfg, open(mdir / 'config.json', 'w'))
    save_file(w, str(mdir / 'model.safetensors'))
    a, b = tokens(80, cfg['vocab'], 70), tokens(9, cfg['vocab'], 71)
    steps = [{'step': 0, 'entries': [{'id': 'a', 'tokens': a[:70], 'want': [0, 69]}, {'id': 'b', 'tokens': b[:2], 'want': []}], 'end': []},
             {'step': 1, 'entries': [{'id': 'b', 'tokens': b[2:], 'want': [6]}], 'end': ['b']},
             {'step': 2, 'entries': [{'id': 'a', 'tokens': a[70:71], 'want': []}], 'end': []},
             {'step': 3, 'entries': [{'id': 'a', 'tokens': a[71:], 'want': [8]}], 'end': ['a']}]
    for dt, tol in (('float32', TOL[F32]), ('bfloat16', TOL[B16])):
        r = subprocess.run([os.path.join(ROOT, 'bin', 'trace_run'), '--model', str(mdir), '--dtype', dt, '--out', str(out),
                            '--max-tokens', '192'], input='\n'.join(json.dumps(s) for s in steps) + '\n', capture_output=True,
                           text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [l for l in r.stdout.splitlines() if l.startswith('done')] == ['done 0', 'done 1', 'done 2', 'done 3']
        ra, rb = O.forward(cfg, w, a, torch.float64), O.forward(cfg, w, b, torch.float64)
        rd = lambda n: torch.from_numpy(np.fromfile(out / f'{n}.f32', dtype='<f4').reshape(-1, cfg['vocab']))
        assert not (out / '2.f32').exists()
        assert rel_err(rd(0), ra[[0, 69]]) < tol and rel_err(rd(1), rb[[8]]) < tol and rel_err(rd(3), ra[[79]]) < tol
        for f in out.iterdir():
            f.unlink()
