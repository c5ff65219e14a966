"""The Rokarax decoder on the GPU: each new kernel against a plain formulation, then the engine under every
schedule in both precisions against the plain model."""

from __future__ import annotations

import json
import os
import subprocess
import sys
import types

import numpy as np
import pytest
import torch

from tests import plain_rokarax, schedules
from tests.helpers import assert_bf16_close_to_f32, assert_logits_close, requests_for
from tests.rokarax_cases import (CASE_A, CASE_B, CASE_C, CASES, case_folder, generated_case, make_folder, plain_greedy,
                                 plain_logits)

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = [torch.float32, torch.bfloat16]
F64 = torch.float64


@pytest.fixture(scope="module")
def ops():
    from paged_llm_b200.kernels.ops import CudaOps
    return CudaOps("cuda")


def tol(dtype, scale=1.0):
    return (2e-5 if dtype == torch.float32 else 1.6e-2) * scale


def rand(*shape, seed=0, dtype=torch.float32, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype)


def make_ctx(ops, q_lens, k_lens, plan_keys=(), slots=None):
    """The device metadata of a step whose requests bring q_lens tokens and then hold k_lens."""
    from paged_llm_b200.engine.context import AttentionPlan, HostBatch
    S = len(q_lens)
    host = HostBatch(list(q_lens), [k - q for q, k in zip(q_lens, k_lens)], list(slots) if slots is not None else [-1] * S)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.int32)).cuda()      # noqa: E731
    plans = {}
    for key in plan_keys:
        plan = ops.plan_attention(q_lens, k_lens, *key)
        small, large = plan["small"].reshape(-1, 4), plan["large"].reshape(-1, 4)
        plans[key] = AttentionPlan(dev(small) if len(small) else None, dev(large) if len(large) else None,
                                   dev(plan["splits"]), len(small), len(large), plan["max_splits"], plan["num_small_tokens"])
    pos = np.concatenate([np.arange(k - q, k) for q, k in zip(q_lens, k_lens)])
    tseq = np.concatenate([np.full(q, s) for s, q in enumerate(q_lens)])
    return types.SimpleNamespace(ops=ops, num_tokens=sum(q_lens), num_seqs=S, host=host, cu_seqlens_q=dev(host.cu),
                                 seq_lens_k=dev(k_lens), positions=dev(pos), token_seq=dev(tseq),
                                 state_slots=dev(host.state_slots), attention_plans=plans)


def block_table(k_lens, ps, seed=0, extra=3):
    """Pages assigned by a random permutation: [requests, pages] and the number of pages in the pool."""
    g = torch.Generator().manual_seed(seed)
    n = [-(-L // ps) for L in k_lens]
    total = sum(n) + extra
    perm = torch.randperm(total, generator=g)
    bt = torch.full((len(k_lens), max(n) + 1), -1, dtype=torch.int32)
    o = 0
    for s in range(len(k_lens)):
        bt[s, :n[s]] = perm[o:o + n[s]]
        o += n[s]
    return bt, total


# ---------------------------------------------------------------- dynamic tanh, embedding scale
@pytest.mark.parametrize("dtype", DTYPES)
def test_dynamic_tanh_with_the_sum(ops, dtype):
    ops.set_compute_dtype(dtype)
    rows, H = 37, 200
    x0, br = rand(rows, H, seed=1, std=3.0), rand(rows, H, seed=2, dtype=dtype, std=2.0)
    post = (torch.tensor([0.7]), 1 + rand(H, seed=3, std=0.2), rand(H, seed=4, std=0.1))
    pre = (torch.tensor([0.4]), 1 + rand(H, seed=5, std=0.2), rand(H, seed=6, std=0.1))
    cu = lambda t: tuple(v.cuda() for v in t)      # noqa: E731
    want_x = x0.double() + torch.tanh(0.7 * br.double()) * post[1].double() + post[2].double()
    want_y = torch.tanh(torch.tensor(0.4, dtype=F64) * want_x) * pre[1].double() + pre[2].double()
    x = x0.cuda()
    y = ops.dyt(x, br.cuda(), cu(post), cu(pre))
    assert y.dtype == dtype
    assert (x.cpu().double() - want_x).abs().max() <= 2e-6 * 8      # the stream is float32 in both precisions
    assert (y.cpu().double() - want_y).abs().max() <= tol(dtype, 2.0)
    # the pieces: a plain sum, a norm of the stream alone, a norm of a tensor that is not the stream
    x = x0.cuda()
    assert ops.dyt(x, br.cuda(), None, None) is None
    assert (x.cpu().double() - (x0.double() + br.double())).abs().max() <= 1e-5
    y = ops.dyt(x0.cuda(), None, None, cu(pre))
    assert (y.cpu().double() - (torch.tanh(0.4 * x0.double()) * pre[1].double() + pre[2].double())).abs().max() <= tol(dtype, 2.0)
    y = ops.dyt(None, br.cuda(), None, cu(post))
    assert (y.cpu().double() - (torch.tanh(0.7 * br.double()) * post[1].double() + post[2].double())).abs().max() <= tol(dtype, 2.0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_scale(ops, dtype):
    table = rand(50, 36, seed=1, dtype=dtype)
    ids = torch.tensor([3, 49, 0, 7], dtype=torch.int32)
    out = ops.embedding(table.cuda(), ids.cuda(), 16.0)
    assert out.dtype == torch.float32 and torch.equal(out.cpu(), table[ids.long()].float() * 16.0)
    assert torch.equal(ops.embedding(table.cuda(), ids.cuda()).cpu(), table[ids.long()].float())


# ---------------------------------------------------------------- attention with a bias by distance and a window
def fill_cache(keys, vals, bt, total, ps, D, dtype):
    """keys/vals: per request [L, G, d] / [L, G, dv] -> pool [pages, 2, G, ps, D], padded with zeros, unused slots NaN."""
    G = keys[0].shape[1]
    kv = torch.full((total, 2, G, ps, D), float("nan"))
    for s, (k, v) in enumerate(zip(keys, vals)):
        for n in range(k.shape[0]):
            kv[bt[s, n // ps], :, :, n % ps] = 0.0
            kv[bt[s, n // ps], 0, :, n % ps, :k.shape[2]] = k[n]
            kv[bt[s, n // ps], 1, :, n % ps, :v.shape[2]] = v[n]
    return kv.to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d,window,ps,table_len", [(4, 2, 32, 24, 8, 20), (6, 1, 96, 40, 16, 40), (2, 2, 16, None, 16, 33),
                                                         (8, 4, 64, 100, 16, 7), (3, 3, 128, 17, 32, 17)])
def test_attention_with_bias_by_distance(ops, dtype, nh, nkv, d, window, ps, table_len):
    """Prompt portions, decoded tokens and both in one step; pages behind the window are gone."""
    ops.set_compute_dtype(dtype)
    bias = rand(nh, table_len, seed=7, std=1.5)
    for q_lens, k_lens in (([70, 3, 33], [70, 45, 133]), ([1, 1, 1, 1], [1, 64, 200, 17]), ([1, 40, 1, 2], [90, 121, 33, 2])):
        bt, total = block_table(k_lens, ps, seed=len(q_lens))
        keys = [rand(L, nkv, d, seed=10 + s, dtype=dtype).float() for s, L in enumerate(k_lens)]
        vals = [rand(L, nkv, d, seed=20 + s, dtype=dtype).float() for s, L in enumerate(k_lens)]
        kv = fill_cache(keys, vals, bt, total, ps, d, dtype)
        if window:
            for s, (nq, L) in enumerate(zip(q_lens, k_lens)):
                for j in range(bt.shape[1]):
                    if (j + 1) * ps <= L - nq - window + 1:
                        kv[bt[s, j]] = float("nan")
                        bt[s, j] = -1
        q = rand(sum(q_lens), nh, d, seed=3, dtype=dtype)
        key = (nh // nkv, nkv, window, d)
        ctx = make_ctx(ops, q_lens, k_lens, [key])
        out = ops.paged_attention(q.reshape(-1, nh * d).cuda().contiguous(), nh, nkv, d, kv.cuda(), bt.cuda(), ctx, d ** -0.5,
                                  window, dist_bias=bias.cuda()).float().cpu()
        o = 0
        for s, (nq, L) in enumerate(zip(q_lens, k_lens)):
            want = plain_rokarax.attend(q[o:o + nq].float(), keys[s], vals[s], d ** -0.5, window, bias, L - nq)
            assert (out[o:o + nq].double() - want.reshape(nq, nh * d)).abs().max() <= tol(dtype, 2.0), (q_lens, s)
            o += nq


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decoded", [True, False])
def test_one_key_at_the_edge_of_the_window(ops, dtype, decoded):
    """One key carries a value of its own and a score far above the rest.  The query that has it as the
    last key of its window returns that value; the next query does not see it."""
    ops.set_compute_dtype(dtype)
    nh, nkv, d, ps, window = 2, 1, 32, 16, 48
    L = 200
    for loud in (L - window, L - window - 1, 15, 16, L - 1):     # first inside, first outside, page borders, itself
        keys = rand(L, nkv, d, seed=1, dtype=dtype, std=0.05).float()
        vals = rand(L, nkv, d, seed=2, dtype=dtype, std=0.05).float()
        keys[loud, 0, :] = 0.0
        keys[loud, 0, 0] = 16.0
        vals[loud, 0, :] = 3.0
        nq = 1 if decoded else 60
        bt, total = block_table([L], ps, seed=loud)
        kv = fill_cache([keys], [vals], bt, total, ps, d, dtype)
        q = rand(nq, nh, d, seed=3, dtype=dtype, std=0.05)
        q[:, :, 0] = 4.0
        ctx = make_ctx(ops, [nq], [L], [(2, 1, window, d)])
        out = ops.paged_attention(q.reshape(nq, nh * d).cuda().contiguous(), nh, nkv, d, kv.cuda(), bt.cuda(), ctx, 1.0, window)
        out = out.float().cpu().view(nq, nh, d)
        for i in range(nq):
            pos = L - nq + i
            seen = 0 <= pos - loud < window
            assert (out[i].mean() > 2.9) == seen, f"loud key {loud}, query {pos}: mean {out[i].mean():.3f}"
        want = plain_rokarax.attend(q.float(), keys, vals, 1.0, window, None, L - nq)
        assert (out.double() - want).abs().max() <= tol(dtype, 3.0)


def test_one_far_key_among_hundreds_without_a_window(ops):
    """No window: key 3 of 900 stands out by its score and by the last row of the bias table."""
    ops.set_compute_dtype(torch.bfloat16)
    nh, nkv, d, ps, L = 4, 2, 64, 16, 900
    keys = rand(L, nkv, d, seed=1, dtype=torch.bfloat16, std=0.05).float()
    vals = rand(L, nkv, d, seed=2, dtype=torch.bfloat16, std=0.05).float()
    keys[3, :, :] = 0.0
    keys[3, :, 5] = 8.0
    vals[3] = -2.0
    bias = torch.zeros(nh, 10)
    bias[:, 9] = 4.0                                   # every distance from 9 on
    bt, total = block_table([L], ps)
    kv = fill_cache([keys], [vals], bt, total, ps, d, torch.bfloat16)
    for nq in (1, 130):
        q = rand(nq, nh, d, seed=3, dtype=torch.bfloat16, std=0.05)
        q[:, :, 5] = 2.0
        ctx = make_ctx(ops, [nq], [L], [(2, 2, None, d)])
        out = ops.paged_attention(q.reshape(nq, nh * d).cuda().contiguous(), nh, nkv, d, kv.cuda(), bt.cuda(), ctx, 1.0, None,
                                  dist_bias=bias.cuda()).float().cpu().view(nq, nh, d)
        want = plain_rokarax.attend(q.float(), keys, vals, 1.0, None, bias, L - nq)
        assert want.mean() < -1.9 and (out.double() - want).abs().max() <= tol(torch.bfloat16, 2.0)


# ---------------------------------------------------------------- the mixers alone, through prompts and decoding
def run_mixer(ops, mixer, hs, dtype, ps=8, splits=((1.0,), (0.6, 0.4), None)):
    """Feeds each request's hidden rows through the mixer three ways: whole; in two portions; a portion and then
    token by token.  Returns the outputs per way, each [sum of lengths, width]."""
    from paged_llm_b200.cache.storage import LayerCache
    from paged_llm_b200.parts.base import FixedState, materialize
    ops.set_compute_dtype(dtype)
    req = mixer.cache_requirement()
    lens = [h.shape[0] for h in hs]
    results = []
    for way in splits:
        if isinstance(req, FixedState):
            cache = LayerCache("fixed_state", -1, True, state=torch.zeros((len(hs), *req.shape), device="cuda"))
            bt = None
        else:
            bt, total = block_table(lens, ps, seed=len(results))
            kv = torch.full((total, 2, req.num_kv_heads, ps, req.head_dim), float("nan"), dtype=dtype, device="cuda")
            cache = LayerCache("paged_kv", 0, True, kv=kv)
        outs = [[] for _ in hs]
        done = [0] * len(hs)
        while any(d < n for d, n in zip(done, lens)):
            q_lens = []
            for s, n in enumerate(lens):
                if way is None:
                    q_lens.append(max(1, n // 2) if done[s] == 0 else min(1, n - done[s]))
                else:
                    cut = [round(f * n) for f in way]
                    cut[-1] = n - sum(cut[:-1])
                    k = sum(1 for i in range(len(cut)) if sum(cut[:i + 1]) <= done[s])
                    q_lens.append(cut[k] if k < len(cut) else 0)
            live = [s for s, q in enumerate(q_lens) if q > 0]
            ql = [q_lens[s] for s in live]
            kl = [done[s] + q_lens[s] for s in live]
            keys = [mixer.attention_plan_key()] if hasattr(mixer, "attention_plan_key") else []
            ctx = make_ctx(ops, ql, kl, keys, slots=live)
            if bt is not None:
                ctx.block_tables = [bt[live].cuda().contiguous()]
            h = torch.cat([hs[s][done[s]:done[s] + q_lens[s]] for s in live]).to(dtype).cuda().contiguous()
            out = materialize(mixer.forward(h, ctx, cache), ops).float().cpu()
            o = 0
            for s in live:
                outs[s].append(out[o:o + q_lens[s]])
                o += q_lens[s]
                done[s] += q_lens[s]
        results.append(torch.cat([torch.cat(o) for o in outs]))
    return results


def load_part(cls, params, names, weights, dtype, ops=None, position=None):
    part = cls(weights=names, **params) if position is None else cls(weights=names, position=position, **params)
    part.load({names[k]: (v.to(dtype) if v.dim() == 2 and k not in ("conv", "rel") else v).cuda() for k, v in weights.items()})
    return part


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,P,N,G,taps,parts", [(4, 8, 16, 1, 4, 1), (6, 16, 24, 3, 2, 3), (1, 64, 32, 1, 1, 2), (2, 40, 128, 2, 5, 4),
                                                (3, 20, 4, 1, 3, 5), (3, 5, 6, 1, 2, 1), (2, 64, 200, 2, 4, 2), (1, 8, 72, 1, 2, 1), (1, 16, 256, 1, 3, 1)])
def test_state_space_mixer_alone(ops, dtype, H, P, N, G, taps, parts):
    from paged_llm_b200.parts.ssm import StateSpaceMixer
    W, inner = 48, H * P
    C = inner + 2 * G * N
    names = {k: k for k in ("in_proj", "conv", "conv_bias", "dt_bias", "a_log", "d_skip", "norm", "o_proj")}
    bf = lambda t: t.to(torch.bfloat16).float()      # noqa: E731
    w = {"in_proj": bf(rand(2 * inner + 2 * G * N + H, W, seed=1, std=W ** -0.5)), "conv": bf(rand(C, taps, seed=2, std=0.5)),
         "conv_bias": bf(rand(C, seed=3, std=0.1)), "dt_bias": bf(rand(H, seed=4) - 1.0), "a_log": bf(-2.0 + rand(H, seed=5, std=0.5)),
         "d_skip": bf(1.0 + rand(H, seed=6, std=0.3)), "norm": bf(1.0 + rand(inner, seed=7, std=0.2)),
         "o_proj": bf(rand(W, inner, seed=8, std=inner ** -0.5))}
    mixer = load_part(StateSpaceMixer, dict(hidden_size=W, num_heads=H, head_dim=P, state_size=N, groups=G, conv_taps=taps,
                                            norm_groups=parts, eps=1e-5), names, w, dtype)
    hs = [bf(rand(n, W, seed=30 + n)) for n in (45, 1, 18, 70)]
    pw = {"m.in": w["in_proj"], "m.conv": w["conv"], "m.conv.b": w["conv_bias"], "m.dt_bias": w["dt_bias"], "m.A_log": w["a_log"],
          "m.D": w["d_skip"], "m.norm": w["norm"], "m.o": w["o_proj"]}
    m = {"heads": H, "vdim": P, "state": N, "groups": G, "norm_groups": parts}
    want = torch.cat([plain_rokarax.mamba2(pw, "m.", m, h.double(), 1e-5) for h in hs])
    for got in run_mixer(ops, mixer, hs, dtype):
        assert (got.double() - want).abs().max() <= tol(dtype, 4.0 * max(1.0, float(want.abs().max())))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d,dv,window,rows,far", [(4, 2, 16, 32, 24, 12, 50.0), (6, 1, 32, 16, None, 8, 30.0), (2, 2, 64, 64, 16, 32, 100.0),
                                                         (3, 3, 24, 8, 7, 4, 9.0), (5, 5, 96, 96, 40, 32, 120.5), (2, 1, 10, 6, 11, 5, 7.0), (24, 1, 16, 16, 30, 8, 20.0)])
def test_gated_attention_mixer_alone(ops, dtype, nh, nkv, d, dv, window, rows, far):
    from paged_llm_b200.parts.attention import GatedAttention
    W = 64
    bf = lambda t: t.to(torch.bfloat16).float()      # noqa: E731
    names = {k: k for k in ("q_proj", "k_proj", "v_proj", "g_proj", "o_proj", "q_norm", "k_norm", "rel")}
    w = {"q_proj": bf(rand(nh * d, W, seed=1, std=W ** -0.5)), "k_proj": bf(rand(nkv * d, W, seed=2, std=W ** -0.5)),
         "v_proj": bf(rand(nkv * dv, W, seed=3, std=W ** -0.5)), "g_proj": bf(rand(nh * dv, W, seed=4, std=W ** -0.5)),
         "o_proj": bf(rand(W, nh * dv, seed=5, std=(nh * dv) ** -0.5)), "q_norm": bf(1 + rand(nh * d, seed=6, std=0.2)),
         "k_norm": bf(1 + rand(nkv * d, seed=7, std=0.2)), "rel": bf(rand(rows, nh, seed=8, std=1.5))}
    mixer = load_part(GatedAttention, dict(hidden_size=W, num_heads=nh, num_kv_heads=nkv, head_dim=d, value_dim=dv, scale=0.3,
                                           eps=1e-5, window=window, distance_bias=True, bias_far=far), names, w, dtype)
    hs = [bf(rand(n, W, seed=40 + n)) for n in (61, 2, 33, 100)]
    pw = {"m.q": w["q_proj"], "m.k": w["k_proj"], "m.v": w["v_proj"], "m.g": w["g_proj"], "m.o": w["o_proj"],
          "m.q.norm": w["q_norm"], "m.k.norm": w["k_norm"], "m.rel": w["rel"]}
    m = {"heads": nh, "kv_heads": nkv, "dim": d, "vdim": dv, "scale": 0.3, "bias_max": far, "mask": {"size": window}}
    want = torch.cat([plain_rokarax.gated_attention(pw, "m.", m, h.double(), 1e-5)[0] for h in hs])
    for got in run_mixer(ops, mixer, hs, dtype):
        assert (got.double() - want).abs().max() <= tol(dtype, 3.0 * max(1.0, float(want.abs().max())))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,d,r,dv,qr,kr,window,dims,scaling", [
    (2, 24, 8, 16, 24, 40, 17, 4, None), (3, 16, 16, 24, 32, 48, 100, 16, {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}),
    (4, 32, 32, 32, 64, 96, None, 32, {"factor": 8.0, "original": 64, "fast": 32.0, "slow": 1.0}), (1, 8, 2, 8, 16, 8, 9, 2, None),
    (5, 40, 16, 48, 40, 112, 32, 16, {"factor": 2.0, "original": 16, "fast": 8.0, "slow": 2.0}),
    (3, 6, 6, 5, 10, 7, 20, 4, None), (20, 8, 8, 8, 16, 24, 12, 8, None)])
def test_latent_attention_mixer_alone(ops, dtype, nh, d, r, dv, qr, kr, window, dims, scaling):
    from paged_llm_b200.parts.latent_attention import LatentAttention
    from paged_llm_b200.parts.rope import RotaryEncoding
    W = 64
    bf = lambda t: t.to(torch.bfloat16).float()      # noqa: E731
    position = RotaryEncoding({}, head_dim=r, theta=10000.0, pairing="interleaved", rotary_dim=dims,
                              scaling=dict(scaling, type="yarn") if scaling else None)
    position.prepare(256, torch.device("cuda"), ops)
    names = {k: k for k in ("dq", "dq_norm", "uq", "dkv", "dkv_norm", "uk", "uv", "o_proj")}
    w = {"dq": bf(rand(qr, W, seed=1, std=W ** -0.5)), "dq_norm": bf(1 + rand(qr, seed=2, std=0.2)),
         "uq": bf(rand(nh * (d + r), qr, seed=3, std=qr ** -0.5)), "dkv": bf(rand(kr + r, W, seed=4, std=W ** -0.5)),
         "dkv_norm": bf(1 + rand(kr, seed=5, std=0.2)), "uk": bf(rand(nh * d, kr, seed=6, std=kr ** -0.5)),
         "uv": bf(rand(nh * dv, kr, seed=7, std=kr ** -0.5)), "o_proj": bf(rand(W, nh * dv, seed=8, std=(nh * dv) ** -0.5))}
    mixer = load_part(LatentAttention, dict(hidden_size=W, num_heads=nh, head_dim=d, rot_dim=r, value_dim=dv, q_rank=qr, kv_rank=kr,
                                            scale=0.25, eps=1e-5, window=window), names, w, dtype, position=position)
    hs = [bf(rand(n, W, seed=50 + n)) for n in (61, 2, 33, 120)]
    pw = {"m.dq": w["dq"], "m.dq.norm": w["dq_norm"], "m.uq": w["uq"], "m.dkv": w["dkv"], "m.dkv.norm": w["dkv_norm"],
          "m.uk": w["uk"], "m.uv": w["uv"], "m.o": w["o_proj"]}
    rot = {"dims": dims, "base": 10000.0}
    if scaling:
        rot["scaling"] = scaling
    m = {"heads": nh, "dim": d, "rot_dim": r, "vdim": dv, "kv_rank": kr, "scale": 0.25, "rot": rot, "mask": {"size": window}}
    want = torch.cat([plain_rokarax.latent_attention(pw, "m.", m, h.double(), 1e-5) for h in hs])
    for got in run_mixer(ops, mixer, hs, dtype):
        assert (got.double() - want).abs().max() <= tol(dtype, 3.0 * max(1.0, float(want.abs().max())))


def test_long_recurrence_keeps_a_far_token(ops):
    """A decay close to one: the first token still shows after 3,000 more, in portions and token by token."""
    from paged_llm_b200.parts.ssm import StateSpaceMixer
    W, H, P, N = 32, 2, 8, 16
    names = {k: k for k in ("in_proj", "conv", "conv_bias", "dt_bias", "a_log", "d_skip", "norm", "o_proj")}
    inner, C = H * P, H * P + 2 * N
    w = {"in_proj": rand(2 * inner + 2 * N + H, W, seed=1, std=W ** -0.5), "conv": rand(C, 2, seed=2, std=0.5),
         "conv_bias": torch.zeros(C), "dt_bias": torch.full((H,), -3.0), "a_log": torch.full((H,), -6.0), "d_skip": torch.zeros(H),
         "norm": torch.ones(inner), "o_proj": rand(W, inner, seed=8, std=inner ** -0.5)}
    mixer = load_part(StateSpaceMixer, dict(hidden_size=W, num_heads=H, head_dim=P, state_size=N, groups=1, conv_taps=2,
                                            norm_groups=1, eps=1e-5), names, w, torch.float32)
    h = rand(3001, W, seed=9, std=0.3)
    h[0] *= 30.0
    pw = {"m.in": w["in_proj"], "m.conv": w["conv"], "m.conv.b": w["conv_bias"], "m.dt_bias": w["dt_bias"], "m.A_log": w["a_log"],
          "m.D": w["d_skip"], "m.norm": w["norm"], "m.o": w["o_proj"]}
    m = {"heads": H, "vdim": P, "state": N, "groups": 1, "norm_groups": 1}
    want = plain_rokarax.mamba2(pw, "m.", m, h.double(), 1e-5)
    h2 = h.clone()
    h2[0] /= 30.0
    assert (plain_rokarax.mamba2(pw, "m.", m, h2.double(), 1e-5)[-1] - want[-1]).abs().max() > 1e-2, "the far token must matter"
    for got in run_mixer(ops, mixer, [h], torch.float32, splits=((0.37, 0.63), (0.999, 0.001))):
        assert (got.double() - want).abs().max() <= 1e-4 * max(1.0, float(want.abs().max()))


# ---------------------------------------------------------------- the engine against the plain model
LENGTHS = {"A": (1, 30, 77, 49, 2, 60, 90, 35), "B": (5, 41, 120, 13, 80, 55), "C": (3, 70, 33, 65, 18, 41)}


def replay(folder, dtype, steps, max_tokens, block_size=16, slots=4, **kw):
    from paged_llm_b200.engine.replay import TraceReplayer

    rp = TraceReplayer(folder, dtype, max_tokens, block_size=block_size, poison=float("nan"), max_num_seqs=slots, **kw)
    for lc in rp.storage.layer_caches:
        if lc is not None and lc.state is not None and lc.owner:
            lc.state.fill_(float("nan"))              # a slot that is not zeroed at a request's start shows
    outputs = {}
    for rec in steps:
        out = rp.step(rec)
        if out is not None:
            outputs[rec["step"]] = out
    assert not rp.live, "requests left alive at the end of the trace"
    rp.cm.check_invariants([])
    for g in range(len(rp.cm.pools)):
        assert rp.cm.num_free_in_group(g) == rp.cm.pools[g].num_pages, "pages were lost"
    assert rp.cm.num_free_state_slots == rp.cm.num_state_slots
    return outputs, rp


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: case_folder(tmp_path_factory, name) for name in CASES}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("schedule", ["whole", "tail", "portions", "mixed"])
def test_schedule_matches_plain(folders, name, dtype, schedule):
    hf = CASES[name][0]
    reqs = requests_for(hf["vocab"], LENGTHS[name], seed=ord(name))
    steps, max_tokens = getattr(schedules, schedule)(reqs)
    block = 8 if name == "B" else 16
    outputs, rp = replay(folders[name], dtype, steps, max_tokens, block_size=block)
    got = schedules.collect(steps, outputs)
    for rid, toks in reqs.items():
        assert_logits_close(got[rid], plain_logits(folders[name], toks), dtype, f"{schedule}/{name}/{rid}")
    if schedule == "tail":
        assert rp.runner.num_graph_steps > 0, "decode steps replay graphs: every part of the model can be captured"


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("schedule", ["tail", "portions", "mixed"])
def test_bfloat16_against_the_float32_engine(folders, name, schedule):
    reqs = requests_for(CASES[name][0]["vocab"], LENGTHS[name], seed=ord(name))
    steps, max_tokens = getattr(schedules, schedule)(reqs)
    a, _ = replay(folders[name], "float32", steps, max_tokens)
    b, _ = replay(folders[name], "bfloat16", steps, max_tokens)
    for k in a:
        assert_bf16_close_to_f32(b[k], a[k], f"rokarax {schedule}/{name}/step {k}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_and_eager_decode_agree(folders, dtype):
    reqs = requests_for(CASE_A["vocab"], (66, 90), seed=5)
    steps, max_tokens = schedules.tail(reqs, last=45)                # the decoded tokens pass over both windows
    a, rp_a = replay(folders["A"], dtype, steps, max_tokens)
    b, rp_b = replay(folders["A"], dtype, steps, max_tokens, enforce_eager=True)
    assert rp_a.runner.num_graph_steps > 0 and rp_b.runner.num_graph_steps == 0
    for k in a:
        assert_logits_close(a[k], b[k], dtype, f"graph vs eager step {k}")


@pytest.mark.parametrize("seed", range(8))
def test_generated_configurations(tmp_path, seed):
    hf = generated_case(100 + seed)
    folder = make_folder(tmp_path, hf, seed)
    reqs = requests_for(hf["vocab"], (2, 50, 21, 70, 9, 130), seed=seed)
    steps, max_tokens = schedules.mixed(reqs, live=3, seed=seed)
    for dtype in ("float32", "bfloat16"):
        outputs, _ = replay(folder, dtype, steps, max_tokens, slots=3)
        got = schedules.collect(steps, outputs)
        for rid, toks in reqs.items():
            assert_logits_close(got[rid], plain_logits(folder, toks), dtype, f"generated {seed}/{dtype}/{rid}")


def test_long_decoding(folders):
    """200 tokens one by one behind a short prompt: windows pass over decoded tokens, pages are given back."""
    toks = requests_for(CASE_C["vocab"], (230,), seed=8)["r0"]
    steps, max_tokens = schedules.tail({"a": toks}, last=200)
    for dtype in ("float32", "bfloat16"):
        outputs, _ = replay(folders["C"], dtype, steps, max_tokens)
        got = schedules.collect(steps, outputs)["a"]
        assert_logits_close(got, plain_logits(folders["C"], toks), dtype, f"long decoding {dtype}")


def test_first_tokens(folders):
    a, b = requests_for(CASE_B["vocab"], (1, 2), seed=3).values()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a, "want": [0]}, {"id": "b", "tokens": b, "want": [0, 1]}], "end": ["a", "b"]},
             {"step": 1, "entries": [{"id": "c", "tokens": b[:1], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "c", "tokens": b[1:], "want": [0]}], "end": ["c"]}]
    for dtype in ("float32", "bfloat16"):
        outputs, _ = replay(folders["B"], dtype, steps, 128)
        assert_logits_close(outputs[0][:1], plain_logits(folders["B"], a), dtype, "one token")
        assert_logits_close(outputs[0][1:], plain_logits(folders["B"], b), dtype, "two tokens")
        assert_logits_close(np.concatenate([outputs[1], outputs[2]]), plain_logits(folders["B"], b), dtype, "one by one")


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_engine(folders, name):
    from paged_llm_b200 import LLMEngine, SamplingParams
    hf = CASES[name][0]
    prompts = list(requests_for(hf["vocab"], (3, 22, 47, 9, 31), seed=60).values())
    eng = LLMEngine(folders[name], dtype="float32", block_size=8, num_gpu_blocks=40, max_model_len=96,
                    max_num_batched_tokens=16, max_num_seqs=3)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=30))
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain_greedy(folders[name], p, 30)
    assert eng.block_manager.num_free_state_slots == 3
    assert eng.runner.num_graph_steps > 0 and eng.ops.launches > 0


def test_greedy_generation_in_bfloat16_follows_the_plain_model(folders):
    from paged_llm_b200 import LLMEngine, SamplingParams
    prompts = list(requests_for(CASE_B["vocab"], (4, 35, 62), seed=61).values())
    eng = LLMEngine(folders["B"], dtype="bfloat16", block_size=16, num_gpu_blocks=32, max_model_len=128)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12))
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o.token_ids:
            ref = plain_logits(folders["B"], seq)[-1]
            assert ref.max() - ref[tok] <= 3e-2 * np.abs(ref).max()
            seq.append(tok)


def test_trace_run_program(folders, tmp_path):
    hf = CASE_A
    reqs = requests_for(hf["vocab"], (40, 3, 71, 25, 52), seed=12)
    steps, max_tokens = schedules.mixed(reqs, live=4, seed=2)
    out_dir = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders["A"], "--dtype", "float32",
         "--out", str(out_dir), "--max-tokens", str(max_tokens)],
        input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [ln for ln in proc.stdout.splitlines() if ln.startswith("done ")] == [f"done {s['step']}" for s in steps]
    outputs = {}
    for s in steps:
        n = sum(len(e["want"]) for e in s["entries"])
        if n:
            outputs[s["step"]] = np.fromfile(out_dir / f"{s['step']}.f32", dtype="<f4").reshape(n, hf["vocab"])
    got = schedules.collect(steps, outputs)
    for rid, toks in reqs.items():
        assert_logits_close(got[rid], plain_logits(folders["A"], toks), "float32", f"trace_run/{rid}")
