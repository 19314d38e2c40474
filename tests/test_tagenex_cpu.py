"""Host-side parts of the Tagenex integration that need no GPU: config parsing, the registry, the page pool, the engine's batch
planning and the scheduler (with a stand-in model on the CPU), and the oracle's own mechanisms."""
import math

import pytest
import torch

import phi3_b200  # noqa: F401
from phi3_b200 import configs, registry, weights
from phi3_b200.paged import PagePool, PoolExhausted, PAGE
from oracle import tagenex_oracle as O


def test_config_reads_every_size_and_constant():
    d = configs.tiny_tagenex()
    c = configs.TagenexConfig(d)
    assert c.vocab_size == 300 and c.width == 96 and c.eps == 1e-5 and len(c.layers) == 4
    assert [l.mixer.window for l in c.layers] == [50, 0, 33, 100]
    assert [l.mixer.v_role for l in c.layers] == ['source', 'none', 'mix', 'mix']
    assert c.layers[2].ff is None and c.layers[1].ff.kind == 'moe' and (c.layers[1].ff.experts, c.layers[1].ff.top) == (5, 2)
    assert c.kv_layout() == [(3, 40, 24), (1, 48, 24), (3, 24, 24), (3, 32, 24)]
    bad = configs.tiny_tagenex()
    bad['layers'][0]['mixer']['kv_heads'] = 4
    with pytest.raises(ValueError):
        configs.TagenexConfig(bad)
    bad = configs.tiny_tagenex()
    bad['layers'][0]['type'] = 'recurrent'
    with pytest.raises(NotImplementedError):
        configs.TagenexConfig(bad)


def test_registry_picks_the_class_by_config():
    assert registry.entry_for({'architecture': 'Tagenex'}).engine == 'paged'
    assert registry.entry_for({'architectures': ['Phi3VForCausalLM']}).engine == 'batch'
    with pytest.raises(KeyError):
        registry.entry_for({'architecture': 'nope'})
    shapes = weights.tagenex_tensor_shapes(configs.tiny_tagenex())
    w = weights.random_tagenex_weights(configs.tiny_tagenex(), 0)
    assert set(shapes) == set(w) and all(tuple(w[k].shape) == tuple(v) for k, v in shapes.items())
    assert 'l2.norm2' not in shapes and 'l1.mlp.e4.down' in shapes and 'l1.mlp.e5.down' not in shapes


def test_page_pool_hands_out_and_takes_back():
    pool = PagePool([(1, 4, 4), (2, 8, 2)], max_tokens=5 * PAGE, n_slots=2, dtype=torch.float32, device='cpu')
    assert pool.n_pages == 5 and pool.k[1].shape == (5, 2, PAGE, 8) and pool.v[1].shape == (5, 2, PAGE, 2)
    a, b = pool.admit(), pool.admit()
    with pytest.raises(PoolExhausted):
        pool.admit()
    assert pool.extend(a, 70) == 0 and pool.pages[a] == [0, 1]
    assert pool.extend(b, 1) == 0 and pool.pages[b] == [2]
    assert pool.extend(a, 58) == 70 and pool.pages[a] == [0, 1]           # 128 tokens: still two pages
    assert pool.extend(a, 1) == 128 and pool.pages[a] == [0, 1, 3]
    assert not pool.can_extend(b, 2 * PAGE)
    with pytest.raises(PoolExhausted):
        pool.extend(b, 2 * PAGE)
    pool.sync()
    assert pool.block_table[a, :3].tolist() == [0, 1, 3]
    pool.release(a)
    c = pool.admit()
    assert c == a and pool.extend(c, 3 * PAGE) == 0 and sorted(pool.pages[c]) == [0, 1, 3]   # the freed pages, again
    pool.release(b)
    pool.release(c)
    assert sorted(pool.free_pages) == list(range(5)) and sorted(pool.free_slots) == [0, 1]


class _FakeModel:
    """forward() returns logits that make token (row position + 1) % vocab the argmax"""
    def __init__(self):
        self.dev, self.vocab = torch.device('cpu'), 50
        self.batches = []

    def kv_layout(self):
        return [(1, 4, 4)]

    def cache_dtype(self):
        return torch.float32

    def prepare(self, n):
        self.max_context = n

    def forward(self, b, pool, trace=None):
        self.batches.append(b)
        if not b.R:
            return None
        pos = b.tok_pos[b.want_rows.long()]
        return torch.nn.functional.one_hot((pos.long() + 1) % self.vocab, self.vocab).float()


def test_engine_plans_tiles_positions_and_wanted_rows():
    from phi3_b200.engine import Engine
    m = _FakeModel()
    eng = Engine(m, 4 * PAGE, 3)
    assert m.max_context == 4 * PAGE
    eng.step([('a', list(range(70)), [0, 69]), ('b', [7], [0])])
    b = m.batches[-1]
    assert (b.T, b.n_pf, b.n_dec, b.R) == (71, 3, 1, 3)
    assert b.pf_tiles.view(-1, 4).tolist() == [[0, 32, 0, 0], [32, 32, 0, 32], [64, 6, 0, 64]]
    assert b.dec_tiles.tolist() == [70, 1, 1, 0] and b.want_rows.tolist() == [0, 69, 70]
    assert b.tok_pos[:70].tolist() == list(range(70)) and b.tok_slot[70].item() == 1
    eng.step([('b', [1, 2, 3], [2]), ('a', [5], [])], end=['a'])
    b = m.batches[-1]
    assert b.pf_tiles.tolist() == [0, 3, 1, 1] and b.dec_tiles.tolist() == [3, 1, 0, 70] and b.want_rows.tolist() == [2]
    assert eng.live() == ['b'] and eng.length('b') == 4 and len(eng.pool.free_pages) == 3
    with pytest.raises(PoolExhausted):
        eng.step([('c', [0] * (3 * PAGE + 1), [])])
    assert eng.live() == ['b'] and len(eng.pool.free_slots) == 2          # a refused step takes nothing
    with pytest.raises(IndexError):
        eng.step([('b', [1], [1])])


def test_scheduler_batches_continuously_and_returns_everything(monkeypatch):
    from phi3_b200.engine import Engine, Scheduler
    m = _FakeModel()
    eng = Engine(m, 6 * PAGE, 2)
    sch = Scheduler(eng, token_budget=80, chunk=48)
    monkeypatch.setattr(sch, '_sample', lambda lg: lg.argmax(-1).tolist())
    prompts = [list(range(100)), [1, 2, 3], list(range(130)), [4]]
    seqs = [sch.add(p, 6) for p in prompts]
    done = sch.run()
    assert [s.rid for s in done] == [0, 1, 2, 3]
    for s, p in zip(seqs, prompts):
        assert s.out == [(len(p) + i) % 50 for i in range(6)]              # position of the last fed token + 1
    assert len(eng.pool.free_pages) == 6 and len(eng.pool.free_slots) == 2 and not eng.live()
    assert max(b.T for b in m.batches) <= 80
    assert any(b.n_pf and b.n_dec for b in m.batches)                      # a prompt portion beside a decoded token
    with pytest.raises(PoolExhausted):
        sch.add(list(range(6 * PAGE)), 6)


def test_oracle_mechanisms():
    # window: itself and the size - 1 tokens before it
    pos = torch.arange(6)
    vis = O.visible(pos, pos, 3)
    assert vis[5].tolist() == [False, False, False, True, True, True] and vis[1].tolist() == [True, True] + [False] * 4
    assert O.visible(pos, pos, None)[5].all()
    # sink: counts once, carries no value
    s = torch.zeros(1, 1, 4)
    a = O.sink_softmax(s, torch.ones(1, 4, dtype=torch.bool), torch.tensor([math.log(4.0)]))
    assert torch.allclose(a, torch.full((1, 1, 4), 1 / 8))
    # penalty: zero at distance 0, r1 ln(1 + r2 d) beyond
    p = O.distance_penalty(torch.tensor([2.0]), torch.tensor([0.5]), torch.tensor([[0.0, 4.0]]))
    assert torch.allclose(p, torch.tensor([[[0.0, 2 * math.log(3.0)]]]))
    # activation: gate clamped from above only, up clamped on both sides, (up + 1)
    y = O.clamped_glu(torch.tensor([5.0, -5.0]), torch.tensor([9.0, -9.0]), 2.0)
    assert torch.allclose(y, torch.tensor([2 * torch.sigmoid(torch.tensor(3.404)) * 3.0, -5 * torch.sigmoid(torch.tensor(-8.51)) * -1.0]))
    # router: softmax over the chosen logits only
    w = {'r.router': torch.eye(3), 'r.router.b': torch.tensor([0.0, 0.0, 5.0])}
    idx, wt = O.route(torch.tensor([[1.0, 2.0, -9.0]]), w, 'r.', 2)
    assert idx.tolist() == [[1, 0]] and torch.allclose(wt, torch.softmax(torch.tensor([[2.0, 1.0]]), -1))


def test_decode_attention_slices_fill_the_gpu_without_splitting_pages():
    from phi3_b200.tagenex import _page_slices
    for pairs in (1, 2, 7, 32, 64, 128, 300, 512, 4096):
        for pages in (1, 2, 3, 17, 40):
            ns = _page_slices(pairs, pages)
            assert 1 <= ns <= pages
    assert _page_slices(1, 17) == 17                         # one request, one K/V head: a page per CTA
    assert _page_slices(4096, 17) == 1                       # more pairs than resident CTAs: whole contexts
    assert _page_slices(128, 17) * 128 <= 2 * 148            # a single round when one fits
