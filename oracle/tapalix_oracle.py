"""Plain, slow restatement of the Tapalix decoder (torch on the CPU, float32 or float64), one function per mechanism.

It shares no code with the CUDA path: the tests build small random checkpoints, run both and compare. A sequence is processed
whole (no cache): keys and values of every head are materialised from the latent vectors, which the product path never does.

Notation: x residual stream [T, W]. A layer is  h = LN(x);  x <- x + mixer(h) + ff(h)  (one layer norm with weight and bias,
both sublayers read it). The layers lo .. hi-1 named by config `loop` run `times` times with the same weights; before the first
layer of every pass (the first too)  x <- W_in [x ; x0]  with x0 the scaled embedding. cfg is the parsed config.json (a dict),
w the tensor dict of the checkpoint.
"""
import math
import torch


def layer_norm(x, gain, bias, eps):
    """(x - mean) / sqrt(mean squared deviation + eps) * gain + bias over the last axis"""
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * gain + bias


def rms_norm(x, gain, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * gain


def silu(z):
    return z * torch.sigmoid(z)


def yarn_frequencies(rot, dtype=torch.float64):
    """-> (angular frequency per pair [dims/2], factor on cos and sin). Pair i has base^(-2i/dims); pairs that turn fewer than
    `slow` times over the original context are divided by `factor`, those with more than `fast` turns stay, linear ramp between."""
    dims, base = int(rot['dims']), float(rot['base'])
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2 * i / dims)
    sc = rot.get('scaling')
    if not sc:
        return f, 1.0
    factor, orig = float(sc['factor']), float(sc['original'])
    where = lambda turns: dims * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))
    lo = max(math.floor(where(float(sc['fast']))), 0)
    hi = min(math.ceil(where(float(sc['slow']))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half(x, pos, rot):
    """x [..., T, n >= dims] (T on axis -2): the first `dims` numbers turn, element i paired with i + dims/2; the rest pass"""
    dims = int(rot['dims'])
    f, mag = yarn_frequencies(rot, x.dtype)
    ang = pos.to(x.dtype)[:, None] * f[None, :]
    c, s = torch.cos(ang) * mag, torch.sin(ang) * mag
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def causal_softmax(scores):
    """scores [H, T, T] of one sequence from its first token: position i sees j <= i"""
    T = scores.shape[-1]
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    return torch.softmax(scores.masked_fill(~mask, float('-inf')), -1)


def latent_attention(h, w, p, mc, eps, rotary):
    """h [T, W]. rotary=True: every head has `dim` plain and `rot_dim` turning query/key numbers, the turning key part is one
    vector shared by the heads; rotary=False: no positions at all and a sigmoid output gate."""
    T = h.shape[0]
    H, d, dv, r = mc['heads'], mc['dim'], mc['vdim'], mc['kv_rank']
    dr = mc['rot_dim'] if rotary else 0
    pos = torch.arange(T)
    q = (h @ w[p + 'q'].T).view(T, H, d + dr)
    ckr = h @ w[p + 'dkv'].T
    c = rms_norm(ckr[:, :r], w[p + 'dkv.norm'], eps)
    k = (c @ w[p + 'uk'].T).view(T, H, d)
    v = (c @ w[p + 'uv'].T).view(T, H, dv)
    scores = torch.einsum('thd,shd->hts', q[..., :d], k)
    if rotary:
        qr = rotate_half(q[..., d:].transpose(0, 1), pos, mc['rot'])        # [H, T, dr]
        kr = rotate_half(ckr[:, r:], pos, mc['rot'])                        # [T, dr]
        scores = scores + torch.einsum('htd,sd->hts', qr, kr)
    a = causal_softmax(scores * mc['scale'])
    o = torch.einsum('hts,shd->thd', a, v).reshape(T, H * dv)
    if not rotary:
        o = o * torch.sigmoid(h @ w[p + 'g'].T)
    return o @ w[p + 'o'].T


def gated_unit(h, w, p):
    return (silu(h @ w[p + 'gate'].T) * (h @ w[p + 'up'].T)) @ w[p + 'down'].T


def route(h, w, p, rc):
    """-> (chosen experts [T, top], weights [T, top]). Sigmoid scores; the choice adds the correction, the weights do not.
    Experts are in `count` groups of neighbours; a group scores the sum of its two best choice scores, only the `keep` best
    groups can be chosen from."""
    E, top = rc['experts'], rc['top']
    s = torch.sigmoid(h @ w[p + 'router'].T)
    choice = s + w[p + 'correction']
    g = rc.get('groups')
    if g:
        n, keep = g['count'], g['keep']
        per = choice.view(-1, n, E // n)
        gs = per.topk(min(2, E // n), -1).values.sum(-1)
        best = gs.topk(keep, -1).indices
        ok = torch.zeros_like(gs, dtype=torch.bool).scatter_(1, best, True)
        choice = choice.masked_fill(~ok[:, :, None].expand_as(per).reshape(-1, E), float('-inf'))
    idx = choice.topk(top, -1).indices
    ws = s.gather(1, idx)
    return idx, ws / (ws.sum(-1, keepdim=True) + 1e-20) * rc['scale']


def moe_ff(h, w, p, fc):
    idx, wt = route(h, w, p, fc['router'])
    out = torch.zeros(h.shape[0], w[p + 'e0.down'].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            out[t] += wt[t, j] * gated_unit(h[t:t + 1], w, f'{p}e{int(idx[t, j])}.')[0]
    if fc.get('shared'):
        out = out + gated_unit(h, w, p + 'shared.')
    return out


def layer_runs(cfg):
    """the order in which layers run: (layer index, does a pass of the loop start here)"""
    n = len(cfg['layers'])
    lp = cfg.get('loop')
    if not lp:
        return [(i, False) for i in range(n)]
    lo, hi, times = lp['start'], lp['stop'], lp['times']
    runs = [(i, False) for i in range(lo)]
    for _ in range(times):
        runs += [(i, i == lo) for i in range(lo, hi)]
    return runs + [(i, False) for i in range(hi, n)]


def forward(cfg, weights, tokens, dtype=torch.float32, trace=None):
    """tokens (one sequence from position 0) -> logits [T, vocab]; trace (a list) gets x after every layer run"""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg['norm']['eps']
    x0 = w['embed'][torch.as_tensor(tokens, dtype=torch.long)] * (cfg.get('embedding') or {}).get('scale', 1.0)
    x = x0
    for i, first in layer_runs(cfg):
        if first:
            x = torch.cat([x, x0], -1) @ w['loop.in'].T
        lc, p = cfg['layers'][i], f'l{i}.'
        h = layer_norm(x, w[p + 'norm1'], w[p + 'norm1.b'], eps)
        y = latent_attention(h, w, p + 'mix.', lc['mixer'], eps, rotary=lc['type'] == 'latent_attention')
        if lc.get('mlp') is not None:
            y = y + moe_ff(h, w, p + 'mlp.', lc['mlp'])
        x = x + y
        if trace is not None:
            trace.append(x.clone())
    h = layer_norm(x, w['final.norm'], w['final.norm.b'], eps)
    logits = (h @ w['head'].T) * cfg.get('logit_scale', 1.0)
    cap = cfg.get('logit_softcap')
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits
