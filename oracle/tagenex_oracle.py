"""Plain, slow restatement of the Tagenex decoder (torch on the CPU, float32 or float64), one function per mechanism.

It shares no code with the CUDA path: the tests build small random checkpoints, run both and compare. A sequence is processed
whole (no cache): every position attends to the keys its window allows, computed from scratch.

Notation: x residual stream [T, W]; a layer is  x <- x + N1(mixer(x)),  x <- x + N2(ff(x))  with N = RMS norm applied to the
sublayer OUTPUT; sublayers read x itself. cfg is the parsed config.json (a dict), w the tensor dict of the checkpoint.
"""
import math
import torch


def rms_norm(x, gain, eps):
    """x / sqrt(mean(x^2) + eps) * gain over the last axis"""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * gain


def distance_penalty(r1, r2, dist):
    """what is taken off a score at distance d = i - j >= 0: r1_h * ln(1 + r2_h * d); r1, r2 [H], dist [T, S] -> [H, T, S]"""
    return r1[:, None, None] * torch.log1p(r2[:, None, None] * dist[None].clamp(min=0))


def visible(qpos, kpos, window):
    """[T, S] bool: key j is seen from i when 0 <= i - j < window (window None: every earlier key)"""
    d = qpos[:, None] - kpos[None, :]
    ok = d >= 0
    if window is not None:
        ok &= d < window
    return ok


def sink_softmax(scores, mask, sink):
    """softmax over the visible keys whose denominator also holds exp(sink_h): scores [H, T, S], mask [T, S], sink [H]"""
    s = scores.masked_fill(~mask[None], float('-inf'))
    m = torch.maximum(s.max(-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(s - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink[:, None, None] - m))


def mix_values(v, v_first, lam):
    return (1 - lam) * v + lam * v_first


def attention_mixer(h, w, p, mc, eps, v_first, is_first_mix):
    """h [T, W]; returns (out [T, W], v as cached [T, G, dv])"""
    T = h.shape[0]
    H, G, d, dv = mc['heads'], mc['kv_heads'], mc['dim'], mc['vdim']
    q = (h @ w[p + 'q'].T).view(T, H, d)
    k = (h @ w[p + 'k'].T).view(T, G, d)
    v = (h @ w[p + 'v'].T).view(T, G, dv)
    q = rms_norm(q, w[p + 'q.norm'], eps)
    k = rms_norm(k, w[p + 'k.norm'], eps)
    if mc.get('v_mix') and not is_first_mix:
        v = mix_values(v, v_first, w[p + 'vmix'])
    rep = H // G
    kh = k.repeat_interleave(rep, dim=1)                      # query head a reads key/value head a // (H/G)
    vh = v.repeat_interleave(rep, dim=1)
    pos = torch.arange(T)
    scores = torch.einsum('thd,shd->hts', q, kh) * mc['scale']
    scores = scores - distance_penalty(w[p + 'r1'], w[p + 'r2'], (pos[:, None] - pos[None, :]).to(h.dtype))
    win = (mc.get('mask') or {}).get('size')
    a = sink_softmax(scores, visible(pos, pos, win), w[p + 'sink'])
    o = torch.einsum('hts,shd->thd', a, vh)
    gate = torch.sigmoid(h @ w[p + 'g'].T)                    # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * dv) @ w[p + 'o'].T, v


def clamped_glu(g, u, limit):
    g = g.clamp(max=limit)
    u = u.clamp(min=-limit, max=limit)
    return g * torch.sigmoid(1.702 * g) * (u + 1)


def dense_ff(h, w, p, fc):
    g = h @ w[p + 'gate'].T + w[p + 'gate.b']
    u = h @ w[p + 'up'].T + w[p + 'up.b']
    return clamped_glu(g, u, fc['limit']) @ w[p + 'down'].T + w[p + 'down.b']


def route(h, w, p, top):
    """(expert ids [T, top], weights [T, top]): the `top` largest router logits, softmax over those alone"""
    z = h @ w[p + 'router'].T + w[p + 'router.b']
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def moe_ff(h, w, p, fc):
    idx, wt = route(h, w, p, fc['router']['top'])
    lim = fc['expert']['limit']
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = p + f'e{int(idx[t, j])}.'
            y = clamped_glu(h[t] @ w[e + 'gate'].T, h[t] @ w[e + 'up'].T, lim) @ w[e + 'down'].T
            out[t] += wt[t, j] * y
    return out


def forward(cfg, weights, tokens, dtype=torch.float32, trace=None):
    """tokens: list of ids of ONE sequence -> logits [T, vocab]. `trace` (a list) receives the residual stream after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg['norm']['eps']
    x = w['embed'][torch.as_tensor(tokens, dtype=torch.long)]
    v_first = None
    for i, lc in enumerate(cfg['layers']):
        p = f'l{i}.'
        mc = lc['mixer']
        first = bool(mc.get('v_mix')) and v_first is None
        y, v = attention_mixer(x, w, p + 'mix.', mc, eps, v_first, first)
        if first:
            v_first = v
        x = x + rms_norm(y, w[p + 'norm1'], eps)
        fc = lc.get('mlp')
        if fc is not None:
            y = dense_ff(x, w, p + 'mlp.', fc) if fc['kind'] == 'dense' else moe_ff(x, w, p + 'mlp.', fc)
            x = x + rms_norm(y, w[p + 'norm2'], eps)
        if trace is not None:
            trace.append(x.clone())
    return rms_norm(x, w['final.norm'], eps) @ w['head'].T
