"""Host-side parts of the Tapalix integration that need no GPU: config parsing (layer runs of the looped block, one cache per
run), the registry, checkpoint shapes, the rotation frequencies, and the oracle's own mechanisms on hand-made inputs."""
import math

import pytest
import torch

import phi3_b200  # noqa: F401
from phi3_b200 import configs, registry, weights
from phi3_b200.paged import PagePool, PAGE
from oracle import tapalix_oracle as O


def test_config_reads_every_size_and_constant():
    d = configs.tiny_tapalix()
    c = configs.TapalixConfig(d)
    assert c.vocab_size == 300 and c.width == 96 and c.eps == 1e-5 and len(c.layers) == 4
    assert abs(c.embed_scale - 96 ** 0.5) < 1e-12 and c.logit_scale == 1.5 and c.logit_softcap == 20.0
    assert [l.mixer.kind for l in c.layers] == ['latent_attention_2', 'latent_attention', 'latent_attention_2', 'latent_attention']
    assert [l.mixer.rot_dim for l in c.layers] == [0, 8, 0, 24] and [l.mixer.gated for l in c.layers] == [True, False, True, False]
    assert c.layers[2].ff is None and (c.layers[1].ff.experts, c.layers[1].ff.top, c.layers[1].ff.groups, c.layers[1].ff.keep) == (8, 3, 4, 2)
    assert c.layers[3].ff.groups == 1 and c.layers[3].ff.shared_ff == 0 and c.layers[0].ff.shared_ff == 72
    # layers 1 and 2 run twice; every run has a cache row of latent + turning key numbers, one shared head, no value pool
    assert c.runs == [(0, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    assert c.kv_layout() == [(1, 56, 0), (1, 48, 0), (1, 72, 0), (1, 48, 0), (1, 72, 0), (1, 72, 0)]
    assert [r for r in O.layer_runs(d)] == c.runs
    plain = configs.TapalixConfig(configs.tiny_tapalix(loop=None))
    assert plain.loop is None and plain.runs == [(i, False) for i in range(4)]
    whole = configs.TapalixConfig(configs.tiny_tapalix(loop=(0, 4, 3)))
    assert len(whole.runs) == 12 and [r for r in whole.runs if r[1]] == [(0, True)] * 3
    for key, val, err in ((('layers', 0, 'type'), 'recurrent', NotImplementedError), (('loop', 'stop'), 9, ValueError),
                          (('layers', 1, 'mlp', 'router', 'top'), 5, ValueError), (('layers', 1, 'mlp', 'kind'), 'dense', NotImplementedError)):
        bad = configs.tiny_tapalix()
        node = bad
        for k in key[:-1]:
            node = node[k]
        node[key[-1]] = val
        with pytest.raises(err):
            configs.TapalixConfig(bad)


def test_registry_and_checkpoint_shapes():
    assert registry.entry_for({'architecture': 'Tapalix'}).engine == 'paged'
    d = configs.tiny_tapalix()
    shapes = weights.tapalix_tensor_shapes(d)
    w = weights.random_tapalix_weights(d, 0)
    assert set(shapes) == set(w) and all(tuple(w[k].shape) == tuple(v) for k, v in shapes.items())
    assert shapes['loop.in'] == (96, 192) and shapes['l1.mix.q'] == (5 * 24, 96) and shapes['l1.mix.dkv'] == (48, 96)
    assert shapes['l0.mix.g'] == (120, 96) and 'l1.mix.g' not in shapes and 'l2.mlp.router' not in shapes
    assert 'l3.mlp.shared.up' not in shapes and shapes['l0.mlp.shared.down'] == (96, 72) and shapes['l1.mlp.correction'] == (8,)
    assert 'loop.in' not in weights.tapalix_tensor_shapes(configs.tiny_tapalix(loop=None))


def test_page_pool_without_a_value_pool():
    pool = PagePool(configs.TapalixConfig(configs.tiny_tapalix()).kv_layout(), 3 * PAGE, 2, torch.float32, 'cpu')
    assert len(pool.k) == 6 and pool.k[0].shape == (3, 1, PAGE, 56) and pool.v[0].numel() == 0


def test_rotation_frequencies():
    rot = {'base': 10000.0, 'dims': 16, 'scaling': {'factor': 4.0, 'original': 64, 'fast': 16.0, 'slow': 2.0}}
    ns = configs.TapalixConfig(configs.tiny_tapalix(layers=[dict(
        {'type': 'latent_attention', 'mixer': dict(heads=1, dim=8, rot_dim=16, vdim=8, kv_rank=8, scale=1.0, rot=rot)}, mlp=None)],
        loop=None)).layers[0].mixer.rot
    f, mag = configs.yarn_frequencies(ns)
    fo, mo = O.yarn_frequencies(rot)
    assert max(abs(a - float(b)) for a, b in zip(f, fo)) < 1e-15 and abs(mag - mo) < 1e-15 and abs(mag - (0.1 * math.log(4.0) + 1)) < 1e-15
    base = [10000.0 ** (-2 * i / 16) for i in range(8)]
    assert f[0] == base[0] and abs(f[-1] - base[-1] / 4.0) < 1e-15                # fast pairs stay, slow pairs are divided
    assert all(b / 4.0 - 1e-15 <= a <= b + 1e-15 for a, b in zip(f, base))
    ns.scaling = None
    assert configs.yarn_frequencies(ns) == (base, 1.0)


def test_oracle_mechanisms():
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=torch.float64)
    ln = O.layer_norm(x, torch.ones(4, dtype=torch.float64) * 2, torch.ones(4, dtype=torch.float64), 0.0)
    assert torch.allclose(ln, (x - 3.0) / math.sqrt(3.5) * 2 + 1)
    # rotation: pairs (i, i + dims/2); numbers beyond dims pass; position 0 turns nothing but still scales
    rot = {'base': 4.0, 'dims': 4, 'scaling': {'factor': 2.0, 'original': 8, 'fast': 2.0, 'slow': 1.0}}
    v = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0]], [[1.0, 2.0, 3.0, 4.0, 5.0]]], dtype=torch.float64).transpose(0, 1)   # [1, T=2, 5]
    f, mag = O.yarn_frequencies(rot)
    r = O.rotate_half(v, torch.tensor([0, 3]), rot)
    assert torch.allclose(r[0, 0], torch.tensor([mag, 2 * mag, 3 * mag, 4 * mag, 5.0], dtype=torch.float64))
    a0, a1 = 3 * float(f[0]), 3 * float(f[1])
    want = [mag * (1 * math.cos(a0) - 3 * math.sin(a0)), mag * (2 * math.cos(a1) - 4 * math.sin(a1)),
            mag * (3 * math.cos(a0) + 1 * math.sin(a0)), mag * (4 * math.cos(a1) + 2 * math.sin(a1)), 5.0]
    assert torch.allclose(r[0, 1], torch.tensor(want, dtype=torch.float64))
    # router: groups of two; group scores 0.9 + 0.8 < 0.95 + 0.94 although the best single expert sits in group 0; with all choice
    # scores pushed below zero the barred experts still cannot win
    logit = lambda p: math.log(p / (1 - p))
    h = torch.eye(4, dtype=torch.float64)[:1]
    Wr = torch.zeros(4, 4, dtype=torch.float64)
    Wr[:, 0] = torch.tensor([logit(0.96), logit(0.5), logit(0.95), logit(0.94)])
    for shift in (0.0, -5.0):
        w = {'router': Wr, 'correction': torch.tensor([0.0, 0.0, 0.0, 0.0], dtype=torch.float64) + shift}
        idx, wt = O.route(h, w, '', dict(experts=4, top=2, scale=3.0, groups={'count': 2, 'keep': 1}))
        assert sorted(idx[0].tolist()) == [2, 3]
        assert abs(float(wt.sum()) - 3.0) < 1e-12 and abs(float(wt[0, idx[0].tolist().index(2)]) - 3.0 * 0.95 / 1.89) < 1e-7
    # the correction changes the choice but not the weights
    w = {'router': Wr, 'correction': torch.tensor([0.0, 0.6, 0.0, 0.0], dtype=torch.float64)}
    idx, wt = O.route(h, w, '', dict(experts=4, top=2, scale=1.0))
    assert sorted(idx[0].tolist()) == [0, 1] and abs(float(wt[0, idx[0].tolist().index(1)]) - 0.5 / 1.46) < 1e-7
    # latent attention is attention with materialised keys and values: one token alone returns its own value through W_o
    d = configs.tiny_tapalix()
    wts = {k: v.double() for k, v in weights.random_tapalix_weights(d, 3).items()}
    hh = torch.randn(1, 96, dtype=torch.float64)
    mc = d['layers'][1]['mixer']
    c = O.rms_norm((hh @ wts['l1.mix.dkv'].T)[:, :mc['kv_rank']], wts['l1.mix.dkv.norm'], 1e-5)
    assert torch.allclose(O.latent_attention(hh, wts, 'l1.mix.', mc, 1e-5, True), (c @ wts['l1.mix.uv'].T) @ wts['l1.mix.o'].T)
