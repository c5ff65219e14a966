"""A plain, slow Pomisun decoder: whole sequences, no cache, float64 by default.

One function per mechanism, written from the design's equations, sharing
nothing with the package (it imports torch and math only).  A model is a
dict `config` (the keys of config.json) and a dict `tensors` (name -> tensor).

Notation: n tokens, D width, H query heads, G key/value heads, d head size,
r rotated dimensions per head, C the chunk of the attention mask, E experts of
which each token takes k.
"""

from __future__ import annotations

import math

import torch


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) along the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_around_zero(x, w, eps):
    """RMS norm whose stored weight is the deviation from one."""
    return rms_unit(x, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def rotary_frequencies(rot: dict, dtype=torch.float64):
    """Per pair i < r/2: base^(-2i/r), blended toward 1/factor of itself for the slow
    pairs, and the magnitude both cosine and sine are multiplied by."""
    r, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(r // 2, dtype=dtype)
    f = base ** (-2.0 * i / r)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def pair_of(turns):          # the pair whose wave makes `turns` turns over the original length
        return r * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(sc["slow"]))), r - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    f = f / factor * ramp + f * (1.0 - ramp)
    return f, 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot: dict):
    """x: [n, heads, d]; the first r dimensions of each head turn, pair (i, i + r/2)."""
    r = int(rot["dims"])
    f, mag = rotary_frequencies(rot, x.dtype)
    a = positions.to(x.dtype)[:, None] * f[None, :]                  # [n, r/2]
    c, s = (torch.cos(a) * mag)[:, None, :], (torch.sin(a) * mag)[:, None, :]
    u, v = x[..., : r // 2], x[..., r // 2: r]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., r:]], dim=-1)


def chunk_visible(n: int, chunk: int | None):
    """[n, n] bool: query i sees key j iff j <= i and both lie in the same chunk."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    vis = j <= i
    if chunk:
        vis = vis & (i // chunk == j // chunk)
    return vis


def attend(q, k, v, scale: float, softcap: float | None = None, chunk: int | None = None):
    """q: [n, H, d], k and v: [n, G, d] of one whole sequence -> [n, H, d].  Query head h reads
    key/value head h // (H / G); scores are capped, then masked, then softmaxed."""
    n, H = q.shape[0], q.shape[1]
    rep = H // k.shape[1]
    kk = k.repeat_interleave(rep, dim=1)
    vv = v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * float(scale)
    if softcap:
        s = float(softcap) * torch.tanh(s / float(softcap))
    s = s.masked_fill(~chunk_visible(n, chunk)[None], float("-inf"))
    return torch.einsum("hij,jhd->ihd", torch.softmax(s, dim=-1), vv)


def attention(h, m: dict, w: dict):
    """h: [n, D]; m: the mixer's sizes and constants; w: 'q', 'k', 'o' matrices [out, in]."""
    n = h.shape[0]
    H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = (h @ w["q"].T).view(n, H, d)
    k = (h @ w["k"].T).view(n, G, d)
    v = k                                                            # values are the unrotated keys
    pos = torch.arange(n)
    if m.get("rot"):
        q, k = rotate(q, pos, m["rot"]), rotate(k, pos, m["rot"])
    o = attend(q, k, v, m["scale"], m.get("softcap"), (m.get("mask") or {}).get("size"))
    return o.reshape(n, H * d) @ w["o"].T


# a test may set this to a list: every routed layer run then appends the smallest distance, in units of the
# logits' spread, between the last chosen and the first rejected expert over the sequence's tokens
ROUTER_MARGINS: list | None = None


def gated(h, w: dict, act):
    return (act(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def routed(h, mlp: dict, w: dict, prefix: str):
    """Each token goes to its k best experts, weighted by the softmax over their k logits; a
    shared expert, if there is one, is added times the sigmoid of one number per token."""
    E, k = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    z = h @ w[prefix + "router"].T                                   # [n, E]
    if ROUTER_MARGINS is not None and k < E:
        ranked = z.sort(dim=-1, descending=True).values
        ROUTER_MARGINS.append(float(((ranked[:, k - 1] - ranked[:, k]) / z.std()).min()))
    top, idx = torch.topk(z, k, dim=-1)
    wt = torch.softmax(top, dim=-1)
    out = torch.zeros_like(h)
    for e in range(E):
        ew = {x: w[f"{prefix}e{e}.{x}"] for x in ("gate", "up", "down")}
        y = gated(h, ew, silu)
        share = (wt * (idx == e)).sum(-1, keepdim=True)
        out = out + share * y
    if mlp.get("shared"):
        sw = {x: w[f"{prefix}shared.{x}"] for x in ("gate", "up", "down")}
        out = out + torch.sigmoid(h @ w[prefix + "shared.sg"].T) * gated(h, sw, silu)
    return out


def feed_forward(h, mlp: dict, w: dict, prefix: str):
    if mlp["kind"] == "dense":
        return gated(h, {x: w[prefix + x] for x in ("gate", "up", "down")}, gelu_tanh)
    if mlp["kind"] == "moe":
        return routed(h, mlp, w, prefix)
    raise ValueError(mlp["kind"])


def layer_order(config: dict):
    """[(layer, first of a repeated pass)] in the order the layers run."""
    L = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, False) for i in range(L)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, False) for i in range(a)]
    for t in range(times):
        order += [(i, t > 0 and i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, L)]


def forward(config: dict, tensors: dict, tokens, dtype=torch.float64, keep_layers: bool = False):
    """Logits [n, vocab] of one whole sequence (and the stream after every layer run)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = float(config["norm"]["eps"])
    x0 = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = x0.clone()
    kept = []
    for i, again in layer_order(config):
        lay, p = config["layers"][i], f"l{i}."
        if again:
            x = x + x0
        if lay["type"] != "attention":
            raise ValueError(lay["type"])
        mw = {k: w[p + "mix." + k] for k in ("q", "k", "o")}
        x = x + attention(norm_around_zero(x, w[p + "norm1"], eps), lay["mixer"], mw)
        if lay.get("mlp"):
            x = x + feed_forward(norm_around_zero(x, w[p + "norm2"], eps), lay["mlp"], w, p + "mlp.")
        if keep_layers:
            kept.append(x.clone())
    logits = norm_around_zero(x, w["final.norm"], eps) @ w["embed"].T
    return (logits, torch.stack(kept)) if keep_layers else logits
