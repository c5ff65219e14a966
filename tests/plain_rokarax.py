"""A plain, slow implementation of the Rokarax decoder: float64, whole sequences, no cache,
one function per mechanism.  It imports nothing from the package; the tests hold the engine
to it.

Notation: T tokens, W the width of the stream, weights `w[name]` stored [out, in].
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def lin(w, x):
    return x @ w.to(F64).T


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def dyt(w, name, x):
    """Dynamic tanh: tanh(alpha x) * weight + bias, no statistics of x."""
    return torch.tanh(w[name + ".alpha"].to(F64) * x) * w[name].to(F64) + w[name + ".b"].to(F64)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def window_mask(T: int, size: int | None):
    """mask[i, j]: query i sees key j, i.e. 0 <= i - j < size (all earlier keys if size is None)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    if size is not None:
        m &= (i - j) < size
    return m


def masked_softmax(scores, mask):
    s = scores.masked_fill(~mask, float("-inf"))
    return torch.softmax(s, dim=-1)


# ---------------------------------------------------------------------------- distance bias

def bucket(n: int, rows: int, far: float) -> int:
    """The row of the bias table for distance n >= 0: one row per distance below rows // 2, then
    rows - rows // 2 rows spaced evenly in log(distance) up to `far`; everything beyond shares the last."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def distance_bias(rel, T: int, far: float):
    """[heads, T, T]: rel[bucket(i - j), head] (zero where j > i; the mask removes those)."""
    rows, heads = rel.shape
    by_distance = torch.tensor([bucket(n, rows, far) for n in range(T)], dtype=torch.long)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    idx = by_distance[(i - j).clamp(min=0)]
    return rel.to(F64)[idx].permute(2, 0, 1)


# ---------------------------------------------------------------------------- rotation

def yarn_frequencies(dims: int, base: float, scaling: dict | None):
    """(frequency of each pair, factor on cosine and sine)."""
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns):
        return dims * math.log(original / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x, positions, dims: int, base: float, scaling):
    """x [..., T, n]: the first `dims` elements of the last axis are rotated, pairs (2i, 2i+1)."""
    f, mag = yarn_frequencies(dims, base, scaling)
    ang = positions.to(F64)[:, None] * f[None, :]              # [T, dims/2]
    c, s = torch.cos(ang) * mag, torch.sin(ang) * mag
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ---------------------------------------------------------------------------- mixers

def gated_attention(w, p, m, h, eps, kv=None):
    """Grouped-query attention with a norm over the whole q and k projections, a learned bias by
    distance, a window, and a sigmoid gate on the heads' outputs.  `kv` = (k, v) of another layer
    replaces this layer's own.  Returns (output, (k, v))."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms(lin(w[p + "q"], h), eps) * w[p + "q.norm"].to(F64)
    if kv is None:
        k = rms(lin(w[p + "k"], h), eps) * w[p + "k.norm"].to(F64)
        v = lin(w[p + "v"], h)
    else:
        k, v = kv
    qh = q.view(T, H, d).transpose(0, 1)
    kh = k.view(T, G, d).transpose(0, 1).repeat_interleave(H // G, dim=0)
    vh = v.view(T, G, dv).transpose(0, 1).repeat_interleave(H // G, dim=0)
    scores = qh @ kh.transpose(1, 2) * m["scale"] + distance_bias(w[p + "rel"], T, m["bias_max"])
    a = masked_softmax(scores, window_mask(T, (m.get("mask") or {}).get("size")))
    o = (a @ vh).transpose(0, 1).reshape(T, H * dv)
    o = o * torch.sigmoid(lin(w[p + "g"], h))
    return lin(w[p + "o"], o), (k, v)


def latent_attention(w, p, m, h, eps):
    """Attention whose queries, keys and values come out of low-rank latents; part of each head's
    query and one key part shared by all heads carry rotary positions."""
    T = h.shape[0]
    H, d, r, dv, kr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m["rot"]
    pos = torch.arange(T)
    cq = rms(lin(w[p + "dq"], h), eps) * w[p + "dq.norm"].to(F64)
    q = lin(w[p + "uq"], cq).view(T, H, d + r)
    ckv = lin(w[p + "dkv"], h)
    c = rms(ckv[:, :kr], eps) * w[p + "dkv.norm"].to(F64)
    k_rot = rotate_interleaved(ckv[:, kr:], pos, rot["dims"], rot["base"], rot.get("scaling"))      # [T, r]
    k_nope = lin(w[p + "uk"], c).view(T, H, d)
    v = lin(w[p + "uv"], c).view(T, H, dv)
    q_nope = q[..., :d]
    q_rot = rotate_interleaved(q[..., d:].transpose(0, 1), pos, rot["dims"], rot["base"], rot.get("scaling"))   # [H, T, r]
    scores = (q_nope.transpose(0, 1) @ k_nope.permute(1, 2, 0) + q_rot @ k_rot.T[None]) * m["scale"]
    a = masked_softmax(scores, window_mask(T, (m.get("mask") or {}).get("size")))
    o = (a @ v.transpose(0, 1)).transpose(0, 1).reshape(T, H * dv)
    return lin(w[p + "o"], o)


def causal_conv(x, weight, bias):
    """x [T, C]; weight [C, taps], the last tap multiplies the current token; zeros before the start."""
    T, C = x.shape
    taps = weight.shape[1]
    xp = torch.cat([torch.zeros(taps - 1, C, dtype=F64), x], dim=0)
    out = bias.to(F64)[None, :].repeat(T, 1)
    for k in range(taps):
        out = out + xp[k:k + T] * weight.to(F64)[:, k][None, :]
    return out


def selective_scan(x, dt, a_log, B, C, D, heads_per_group: int):
    """x [T, H, P], dt [T, H], B and C [T, G, N]: S_t = exp(-exp(a_log) dt_t) S_(t-1) + dt_t B_t x_t^T,
    y_t = S_t^T C_t + D x_t, one token after the other."""
    T, H, P = x.shape
    N = B.shape[-1]
    S = torch.zeros(H, N, P, dtype=F64)
    y = torch.zeros(T, H, P, dtype=F64)
    A = torch.exp(a_log.to(F64))
    group = torch.arange(H) // heads_per_group
    for t in range(T):
        Bt, Ct = B[t, group], C[t, group]                                    # [H, N]
        S = torch.exp(-A * dt[t])[:, None, None] * S + dt[t][:, None, None] * Bt[:, :, None] * x[t][:, None, :]
        y[t] = (S * Ct[:, :, None]).sum(1) + D.to(F64)[:, None] * x[t]
    return y


def mamba2(w, p, m, h, eps):
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    zxbcdt = lin(w[p + "in"], h)
    z = zxbcdt[:, :inner]
    xbc = silu(causal_conv(zxbcdt[:, inner:2 * inner + 2 * G * N], w[p + "conv"], w[p + "conv.b"]))
    dt = softplus(zxbcdt[:, 2 * inner + 2 * G * N:] + w[p + "dt_bias"].to(F64))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    y = selective_scan(x, dt, w[p + "A_log"], B, C, w[p + "D"], H // G).reshape(T, inner)
    y = y * silu(z)
    parts = m["norm_groups"]
    y = rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"].to(F64)
    return lin(w[p + "o"], y)


def dense_mlp(w, p, h):
    return lin(w[p + "down"], silu(lin(w[p + "gate"], h)) * lin(w[p + "up"], h))


# ---------------------------------------------------------------------------- the model

def forward(cfg: dict, w: dict, tokens, collect=None):
    """Logits [T, vocab] in float64.  `collect`, a list, receives the stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = w["embed"].to(F64)[torch.as_tensor(tokens, dtype=torch.long)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    kept = {}
    for i, lay in enumerate(cfg["layers"]):
        pre, m = f"l{i}.", lay["mixer"]
        h = dyt(w, pre + "norm1", x)
        if lay["type"] == "attention":
            src = m.get("kv_from")
            a, kept[i] = gated_attention(w, pre + "mix.", m, h, eps, kept[src] if src is not None else None)
        elif lay["type"] == "latent_attention":
            a = latent_attention(w, pre + "mix.", m, h, eps)
        elif lay["type"] == "mamba2":
            a = mamba2(w, pre + "mix.", m, h, eps)
        else:
            raise ValueError(lay["type"])
        x = x + dyt(w, pre + "norm1b", a)
        if lay.get("mlp") is not None:
            x = x + dyt(w, pre + "norm2b", dense_mlp(w, pre + "mlp.", dyt(w, pre + "norm2", x)))
        if collect is not None:
            collect.append(x.clone())
    return lin(w["head"], dyt(w, "final.norm", x))


def attend(q, k, v, scale: float, window: int | None = None, bias_by_distance=None, first_position: int = 0):
    """Attention of query rows q [nq, H, d] at positions first_position.. over keys k [L, G, d] and values
    v [L, G, dv] at positions 0..L-1 (L = first_position + nq); `bias_by_distance` [H, n] is read at
    min(distance, n - 1).  Returns [nq, H, dv] in float64."""
    nq, H, _ = q.shape
    L, G, _ = k.shape
    kh = k.to(F64).repeat_interleave(H // G, dim=1)
    vh = v.to(F64).repeat_interleave(H // G, dim=1)
    pos = first_position + torch.arange(nq)
    dist = pos[:, None] - torch.arange(L)[None, :]
    scores = torch.einsum("qhd,khd->hqk", q.to(F64), kh) * scale
    if bias_by_distance is not None:
        scores = scores + bias_by_distance.to(F64)[:, dist.clamp(0, bias_by_distance.shape[1] - 1)]
    hidden = dist < 0
    if window is not None:
        hidden |= dist >= window
    a = torch.softmax(scores.masked_fill(hidden[None], float("-inf")), dim=-1)
    return torch.einsum("hqk,khd->qhd", a, vh)
