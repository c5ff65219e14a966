"""The Pomisun decoder on the GPU: each of its mechanisms alone against the plain implementation's
function for it, then the engine (step function, cache, scheduler) on three small configurations
under every schedule, in float32 and bfloat16."""

import json
import math
import os
import subprocess
import sys
import types

import numpy as np
import pytest
import torch

from tests import plain_pomisun, schedules
from tests.helpers import assert_bf16_close_to_f32, assert_logits_close, requests_for
from tests.pomisun_cases import CASES, case_folder, clear_requests, generated_case, make_folder, plain_greedy, plain_logits

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from paged_llm_b200.kernels.ops import CudaOps
    return CudaOps("cuda")


def tol(dtype, scale=1.0):
    return (2e-5 if dtype == torch.float32 else 1.6e-2) * scale


def randn(*shape, seed=0, dtype=torch.float32, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype)


# ---------------------------------------------------------------- helpers: a paged cache and a step's metadata
def paged_case(q_lens, k_lens, nh, nkv, d, ps, dtype, seed=0, values_are_keys=True):
    """Random keys (the values are other random vectors unless `values_are_keys`) in a pool whose pages are
    assigned by a random permutation; unused slots are NaN."""
    g = torch.Generator().manual_seed(seed)
    nblocks = [-(-L // ps) for L in k_lens]
    total = sum(nblocks) + 3
    perm = torch.randperm(total, generator=g)
    bt = torch.full((len(q_lens), max(nblocks) + 2), 10 ** 6, dtype=torch.int32)
    kv = torch.full((total, 2, nkv, ps, d), float("nan"))
    keys, vals, o = [], [], 0
    for s, L in enumerate(k_lens):
        bt[s, :nblocks[s]] = perm[o:o + nblocks[s]]
        o += nblocks[s]
        k = torch.randn(L, nkv, d, generator=g).to(dtype).float()
        v = k.clone() if values_are_keys else torch.randn(L, nkv, d, generator=g).to(dtype).float()
        keys.append(k)
        vals.append(v)
        for n in range(L):
            kv[bt[s, n // ps], 0, :, n % ps] = k[n]
            kv[bt[s, n // ps], 1, :, n % ps] = v[n]
    q = torch.randn(sum(q_lens), nh, d, generator=g).to(dtype)
    return q, kv.to(dtype), bt, keys, vals


def make_ctx(ops, q_lens, k_lens, nh, nkv, d, chunk=None, window=None):
    from paged_llm_b200.engine.context import AttentionPlan, HostBatch
    from paged_llm_b200.kernels.ops import attention_plan_key
    S = len(q_lens)
    host = HostBatch(list(q_lens), [k - q for q, k in zip(q_lens, k_lens)], [-1] * S)
    plan = ops.plan_attention(q_lens, k_lens, nh // nkv, nkv, window, d, chunk)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.int32)).cuda()
    small, large = plan["small"].reshape(-1, 4), plan["large"].reshape(-1, 4)
    ap = AttentionPlan(dev(small) if len(small) else None, dev(large) if len(large) else None, dev(plan["splits"]),
                       len(small), len(large), plan["max_splits"], plan["num_small_tokens"])
    pos = np.concatenate([np.arange(k - q, k) for q, k in zip(q_lens, k_lens)])
    tseq = np.concatenate([np.full(q, s) for s, q in enumerate(q_lens)])
    return types.SimpleNamespace(num_tokens=sum(q_lens), num_seqs=S, host=host, cu_seqlens_q=dev(host.cu),
                                 seq_lens_k=dev(k_lens), positions=dev(pos), token_seq=dev(tseq),
                                 attention_plans={attention_plan_key(nh, nkv, window, d, chunk): ap})


def drop_pages_before_chunks(bt, q_lens, k_lens, chunk, ps):
    """What the cache manager does: pages wholly in front of the chunk of a request's first new token are gone."""
    for s, (nq, L) in enumerate(zip(q_lens, k_lens)):
        first = L - nq
        needed = first - first % chunk
        for j in range(bt.shape[1]):
            if (j + 1) * ps <= needed:
                bt[s, j] = -1


def run_attention(ops, q, kv, bt, q_lens, k_lens, nh, nkv, d, dtype, scale, chunk=None, softcap=None):
    ctx = make_ctx(ops, q_lens, k_lens, nh, nkv, d, chunk)
    qk = torch.cat([q.reshape(-1, nh * d), torch.zeros(q.shape[0], nkv * d, dtype=dtype)], dim=1).cuda().contiguous()
    return ops.paged_attention(qk, nh, nkv, d, kv.cuda(), bt.cuda(), ctx, scale, None, softcap=softcap,
                               chunk=chunk).float().cpu(), ctx


def plain_rows(q_rows, keys, vals, nq, L, scale, softcap, chunk):
    nh, d = q_rows.shape[1], q_rows.shape[2]
    qs = torch.zeros(L, nh, d, dtype=torch.float64)
    qs[L - nq:] = q_rows.double()
    return plain_pomisun.attend(qs, keys.double(), vals.double(), scale, softcap, chunk)[L - nq:].reshape(nq, nh * d).float()


# ---------------------------------------------------------------- the chunked mask
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("softcap", [None, 4.0])
@pytest.mark.parametrize("nh,nkv,d,chunk,ps", [(4, 2, 16, 24, 8), (10, 2, 96, 80, 16), (6, 3, 32, 40, 16), (4, 1, 64, 32, 16),
                                              (2, 2, 128, 50, 32), (32, 1, 48, 7, 16)])
def test_chunked_attention(ops, dtype, softcap, nh, nkv, d, chunk, ps):
    """Prompt portions that start and end anywhere in a chunk beside decoded tokens just before, at and just
    behind a chunk's edge, with the pages of finished chunks taken away."""
    ops.set_compute_dtype(dtype)
    q_lens = [3 * chunk + 5, 1, 1, 1, 2, chunk + 9, 1]
    k_lens = [3 * chunk + 5, 4 * chunk, 4 * chunk + 1, 4 * chunk + 2, 2 * chunk + 1, 5 * chunk + 3, 1]
    q, kv, bt, keys, vals = paged_case(q_lens, k_lens, nh, nkv, d, ps, dtype, seed=chunk)
    drop_pages_before_chunks(bt, q_lens, k_lens, chunk, ps)
    cu = np.concatenate([[0], np.cumsum(q_lens)])
    # the mixed batch, then the decoding requests alone (in bfloat16 they then run as clusters)
    for pick in (list(range(len(q_lens))), [1, 2, 3, 6]):
        ql, kl = [q_lens[s] for s in pick], [k_lens[s] for s in pick]
        rows = torch.cat([torch.arange(cu[s], cu[s + 1]) for s in pick])
        out, _ = run_attention(ops, q[rows], kv, bt[pick].contiguous(), ql, kl, nh, nkv, d, dtype, 0.25, chunk, softcap)
        o = 0
        for s in pick:
            nq, L = q_lens[s], k_lens[s]
            want = plain_rows(q[cu[s]:cu[s + 1]], keys[s], vals[s], nq, L, 0.25, softcap, chunk)
            torch.testing.assert_close(out[o:o + nq], want, atol=tol(dtype), rtol=tol(dtype), msg=f"request {s}")
            o += nq


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decoded", [True, False])
def test_keys_at_the_edge_of_a_chunk(ops, dtype, decoded):
    """Among random scores a wrongly seen or a skipped key hides: one key is made to stand out.  Placed on the
    last position of the chunk in front it must change nothing; on the chunk's first position, at a page's
    border inside it, or at the query itself it must be all the query sees."""
    ops.set_compute_dtype(dtype)
    nh, nkv, d, ps, chunk = 8, 2, 64, 16, 48
    direction = randn(d, seed=1)
    direction = (direction / direction.norm() * 30).to(dtype)
    for L in (chunk * 3 + 1, chunk * 3 + 20, chunk * 4):              # the query is first, in the middle, last of its chunk
        start = (L - 1) - (L - 1) % chunk
        for target in (start - 1, start, min(start + 16, L - 1), L - 1, 0):
            nq = 1 if decoded else 37
            q, kv, bt, keys, vals = paged_case([nq], [L], nh, nkv, d, ps, dtype, seed=L + target, values_are_keys=False)
            q[-1] = direction
            for h in range(nkv):
                keys[0][target, h] = direction.float()
                kv[bt[0, target // ps], 0, h, target % ps] = direction
            if decoded:
                drop_pages_before_chunks(bt, [nq], [L], chunk, ps)
            out, _ = run_attention(ops, q, kv, bt, [nq], [L], nh, nkv, d, dtype, d ** -0.5, chunk)
            want = plain_rows(q, keys[0], vals[0], nq, L, d ** -0.5, None, chunk)
            torch.testing.assert_close(out, want, atol=2e-2, rtol=2e-2, msg=f"context {L}, key {target}")
            seen = vals[0][target].repeat_interleave(nh // nkv, dim=0).reshape(nh * d)
            if start <= target:
                torch.testing.assert_close(out[-1], seen, atol=2e-2, rtol=2e-2, msg=f"context {L}, key {target} is all")
            else:
                assert (out[-1] - seen).abs().max() > 0.5, f"context {L}: key {target} of another chunk was seen"


def test_one_far_chunk_among_many(ops):
    """Decoding far into a long request: of 4,000 keys only those of the last chunk count, whatever the splits."""
    ops.set_compute_dtype(torch.bfloat16)
    nh, nkv, d, ps, chunk = 12, 3, 80, 16, 112
    for L in (4000, 3921, 3920 + 112):
        q, kv, bt, keys, vals = paged_case([1], [L], nh, nkv, d, ps, torch.bfloat16, seed=L)
        out, _ = run_attention(ops, q, kv, bt, [1], [L], nh, nkv, d, torch.bfloat16, d ** -0.5, chunk, 20.0)
        want = plain_rows(q, keys[0], vals[0], 1, L, d ** -0.5, 20.0, chunk)
        torch.testing.assert_close(out, want, atol=1.6e-2, rtol=1.6e-2)


# ---------------------------------------------------------------- rotation, and values that are the unrotated keys
def test_rotary_table_with_yarn(ops):
    from paged_llm_b200.parts.rope import RotaryEncoding
    rot = {"dims": 24, "base": 5000.0, "scaling": {"factor": 3.0, "original": 48, "fast": 8.0, "slow": 1.5}}
    enc = RotaryEncoding({}, head_dim=32, theta=rot["base"], scaling=dict(rot["scaling"], type="yarn"), rotary_dim=24)
    enc.prepare(300, "cuda", ops)
    f, mag = plain_pomisun.rotary_frequencies(rot)
    ang = torch.arange(300, dtype=torch.float64)[:, None] * f[None, :]
    want = torch.stack([ang.cos() * mag, ang.sin() * mag], dim=-1)
    torch.testing.assert_close(enc.table.double().cpu(), want, atol=3e-5, rtol=0)       # float32 angles up to 300 rad
    assert mag > 1.1


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d,rd", [(4, 2, 16, 16), (5, 1, 96, 96), (6, 3, 32, 16), (3, 1, 48, 8), (2, 2, 64, 64)])
def test_rope_write_keeps_the_unrotated_key_as_value(ops, dtype, nh, nkv, d, rd):
    from paged_llm_b200.parts.rope import RotaryEncoding
    ops.set_compute_dtype(dtype)
    ps, q_lens, k_lens = 8, [5, 1, 12], [5, 30, 20]
    rot = {"dims": rd, "base": 100.0, "scaling": {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0}}
    enc = RotaryEncoding({}, head_dim=d, theta=100.0, scaling=dict(rot["scaling"], type="yarn"), rotary_dim=rd)
    enc.prepare(64, "cuda", ops)
    _, kv, bt, _, _ = paged_case(q_lens, k_lens, nh, nkv, d, ps, dtype, seed=rd)
    ctx = make_ctx(ops, q_lens, k_lens, nh, nkv, d)
    T = sum(q_lens)
    qk = randn(T, (nh + nkv) * d, seed=5, dtype=dtype)
    pool = torch.full_like(kv, float("nan")).cuda()
    buf = qk.cuda().clone()
    ops.rope_kv_write(buf, nh, nkv, d, enc, ctx, pool, bt.cuda(), value_from_key=True)
    pos = ctx.positions.cpu().long()
    heads = qk.double().view(T, nh + nkv, d)
    want = plain_pomisun.rotate(heads, pos, rot)
    torch.testing.assert_close(buf.double().cpu().view(T, nh + nkv, d), want, atol=tol(dtype, 4), rtol=tol(dtype))
    seq = ctx.token_seq.cpu().long()
    for t in range(T):
        page, off = int(bt[seq[t], pos[t] // ps]), int(pos[t] % ps)
        torch.testing.assert_close(pool[page, 0, :, off].double().cpu(), want[t, nh:], atol=tol(dtype, 4), rtol=tol(dtype))
        assert torch.equal(pool[page, 1, :, off].cpu(), qk.view(T, nh + nkv, d)[t, nh:]), "the value is the key as projected"


@pytest.mark.parametrize("M", [1, 7, 16])
@pytest.mark.parametrize("nh,nkv,d,K", [(6, 2, 96, 256), (4, 2, 16, 64), (2, 2, 64, 128)])
def test_fused_projection_with_rotation_and_values_from_keys(ops, M, nh, nkv, d, K):
    """Few tokens: projection, rotation and cache write are one kernel; against the separate kernels."""
    from paged_llm_b200.parts.rope import RotaryEncoding
    ops.set_compute_dtype(torch.bfloat16)
    ps = 16
    k_lens = [40 + 3 * i for i in range(M)]
    enc = RotaryEncoding({}, head_dim=d, theta=1000.0, scaling={"type": "yarn", "factor": 2.0, "original": 32,
                                                                "fast": 8.0, "slow": 1.0}, rotary_dim=d)
    enc.prepare(128, "cuda", ops)
    _, kv, bt, _, _ = paged_case([1] * M, k_lens, nh, nkv, d, ps, torch.bfloat16, seed=M)
    ctx = make_ctx(ops, [1] * M, k_lens, nh, nkv, d)
    h = randn(M, K, seed=2, dtype=torch.bfloat16).cuda()
    w = randn((nh + nkv) * d, K, seed=3, dtype=torch.bfloat16, std=K ** -0.5).cuda()
    pool_a, pool_b = kv.cuda().clone(), kv.cuda().clone()
    fused = ops.qkv_rope_write(h, w, nh, nkv, d, enc, ctx, pool_a, bt.cuda(), value_from_key=True)
    ops.use_skinny = False
    try:
        apart = ops.qkv_rope_write(h, w, nh, nkv, d, enc, ctx, pool_b, bt.cuda(), value_from_key=True)
    finally:
        ops.use_skinny = True
    torch.testing.assert_close(fused.float(), apart.float(), atol=2e-2, rtol=2e-2)
    written = ~torch.isnan(pool_b.float())
    assert torch.equal(written, ~torch.isnan(pool_a.float()))
    torch.testing.assert_close(pool_a.float()[written], pool_b.float()[written], atol=2e-2, rtol=2e-2)


# ---------------------------------------------------------------- norm, activation, sums
@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_with_a_weight_around_zero(ops, dtype):
    from paged_llm_b200.parts.norm import RMSNorm
    ops.set_compute_dtype(dtype)
    norm = RMSNorm({"weight": "n"}, dim=96, eps=1e-3, unit_offset=True)
    w = randn(96, seed=1, std=0.3, dtype=torch.bfloat16)
    norm.load({"n": w.to(dtype).cuda()})
    x = randn(9, 96, seed=2, std=2.0).cuda()
    ctx = types.SimpleNamespace(ops=ops)
    want = plain_pomisun.norm_around_zero(x.double().cpu(), w.double(), 1e-3)
    torch.testing.assert_close(norm.forward(x, ctx).double().cpu(), want, atol=tol(dtype, 4), rtol=tol(dtype))
    branch = randn(9, 96, seed=3).to(dtype).cuda()
    x2 = x.clone()
    y = norm.add_forward(x2, branch, ctx)
    want = plain_pomisun.norm_around_zero(x.double().cpu() + branch.double().cpu(), w.double(), 1e-3)
    torch.testing.assert_close(y.double().cpu(), want, atol=tol(dtype, 4), rtol=tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,I", [(7, 172), (33, 256), (1, 5)])
def test_gelu_gate(ops, dtype, rows, I):
    ops.set_compute_dtype(dtype)
    gu = randn(rows, 2 * I, seed=I, std=2.0, dtype=dtype)
    got = ops.act_mul(gu.cuda(), "gelu_tanh").double().cpu()
    want = plain_pomisun.gelu_tanh(gu[:, :I].double()) * gu[:, I:].double()
    torch.testing.assert_close(got, want, atol=tol(dtype, 4), rtol=tol(dtype))


@pytest.mark.parametrize("M", [1, 8, 13])
@pytest.mark.parametrize("I,K", [(224, 288), (100, 96), (7, 32)])
def test_few_token_product_with_the_gelu_gate(ops, M, I, K):
    ops.set_compute_dtype(torch.bfloat16)
    h = randn(M, K, seed=1, dtype=torch.bfloat16)
    w = randn(2 * I, K, seed=2, dtype=torch.bfloat16, std=K ** -0.5)
    got = ops.gated_act_linear(h.cuda(), w.cuda(), "gelu_tanh").double().cpu()
    z = h.double() @ w.double().T
    want = plain_pomisun.gelu_tanh(z[:, :I]) * z[:, I:]
    torch.testing.assert_close(got, want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_sums_into_the_stream(ops, dtype):
    x = randn(11, 70, seed=1).cuda()
    branch, extra = randn(11, 70, seed=2).to(dtype).cuda(), randn(11, 70, seed=3).cuda()
    for b, e in ((branch, extra), (None, extra), (branch, None)):
        y = ops.add_rows(x.clone(), b, e)
        want = x + (b.float() if b is not None else 0) + (e if e is not None else 0)
        torch.testing.assert_close(y, want, atol=1e-6, rtol=1e-6)


# ---------------------------------------------------------------- routed experts
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,D,E,k,F,shared", [(5, 64, 6, 2, 32, 48), (300, 128, 4, 2, 64, 32), (40, 96, 5, 5, 20, None),
                                              (1, 352, 10, 3, 48, 80), (16, 64, 8, 1, 16, None), (130, 72, 3, 2, 24, 8),
                                              (70, 64, 40, 4, 16, None)])
def test_routed_experts(ops, dtype, T, D, E, k, F, shared):
    """Router, top-k, softmax over the chosen logits, experts and the shared expert behind its gate, in every
    form of the grouped product: tiles of 64 pairs, of 16, and the plain one (float32, or sizes that are no
    multiple of 8); experts that get no token; every expert chosen."""
    ops.set_compute_dtype(dtype)
    w = {"m.router": randn(E, D, seed=1, dtype=torch.bfloat16, std=1.0)}
    for e in range(E):
        w[f"m.e{e}.gate"] = randn(F, D, seed=10 + e, dtype=torch.bfloat16, std=D ** -0.5)
        w[f"m.e{e}.up"] = randn(F, D, seed=100 + e, dtype=torch.bfloat16, std=D ** -0.5)
        w[f"m.e{e}.down"] = randn(D, F, seed=1000 + e, dtype=torch.bfloat16, std=F ** -0.5)
    mlp = {"router": {"experts": E, "top": k}}
    if shared:
        mlp["shared"] = {"ff": shared}
        w["m.shared.gate"] = randn(shared, D, seed=5, dtype=torch.bfloat16, std=D ** -0.5)
        w["m.shared.up"] = randn(shared, D, seed=6, dtype=torch.bfloat16, std=D ** -0.5)
        w["m.shared.down"] = randn(D, shared, seed=7, dtype=torch.bfloat16, std=shared ** -0.5)
        w["m.shared.sg"] = randn(1, D, seed=8, dtype=torch.bfloat16, std=0.3)
    h = randn(T, D, seed=9, dtype=torch.bfloat16)
    want = plain_pomisun.routed(h.double(), mlp, {n: t.double() for n, t in w.items()}, "m.")
    from paged_llm_b200.parts.routed_mlp import RoutedMLP
    names = {n[2:]: n for n in w}
    part = RoutedMLP(names, hidden_size=D, expert_size=F, num_experts=E, top_k=k, shared_size=shared)
    assert set(part.tensor_specs()) == set(w)
    part.load({n: t.to(dtype).cuda() for n, t in w.items()})
    got = part.forward(h.to(dtype).cuda(), types.SimpleNamespace(ops=ops))
    assert got.dtype == torch.float32
    scale = float(want.abs().max())
    torch.testing.assert_close(got.double().cpu(), want, atol=tol(dtype, scale), rtol=tol(dtype))


@pytest.mark.parametrize("T,D,E,k,F,shared", [(1100, 128, 4, 2, 64, 32), (700, 192, 6, 3, 128, None), (2048, 256, 16, 1, 64, 64)])
def test_routed_experts_on_the_grouped_tensor_core_product(ops, T, D, E, k, F, shared):
    """Many pairs per expert: the experts' products run on the tcgen05 kernel in its grouped form (rows gathered
    in sorted order, tiles of 256 pairs of one expert, the count of tiles read on the device); one expert gets
    no token at all."""
    ops.set_compute_dtype(torch.bfloat16)
    w = {"m.router": randn(E, D, seed=1, dtype=torch.bfloat16, std=1.0)}
    w["m.router"][E - 1] = 0
    w["m.router"][E - 1, 0] = -100.0                         # never chosen (the inputs' first column is positive)
    for e in range(E):
        w[f"m.e{e}.gate"] = randn(F, D, seed=10 + e, dtype=torch.bfloat16, std=D ** -0.5)
        w[f"m.e{e}.up"] = randn(F, D, seed=100 + e, dtype=torch.bfloat16, std=D ** -0.5)
        w[f"m.e{e}.down"] = randn(D, F, seed=1000 + e, dtype=torch.bfloat16, std=F ** -0.5)
    mlp = {"router": {"experts": E, "top": k}}
    if shared:
        mlp["shared"] = {"ff": shared}
        w["m.shared.gate"] = randn(shared, D, seed=5, dtype=torch.bfloat16, std=D ** -0.5)
        w["m.shared.up"] = randn(shared, D, seed=6, dtype=torch.bfloat16, std=D ** -0.5)
        w["m.shared.down"] = randn(D, shared, seed=7, dtype=torch.bfloat16, std=shared ** -0.5)
        w["m.shared.sg"] = randn(1, D, seed=8, dtype=torch.bfloat16, std=0.3)
    h = randn(T, D, seed=9, dtype=torch.bfloat16)
    h[:, 0] = h[:, 0].abs() + 1
    want = plain_pomisun.routed(h.double(), mlp, {n: t.double() for n, t in w.items()}, "m.")
    from paged_llm_b200.parts.routed_mlp import RoutedMLP
    part = RoutedMLP({n[2:]: n for n in w}, hidden_size=D, expert_size=F, num_experts=E, top_k=k, shared_size=shared)
    part.load({n: t.cuda() for n, t in w.items()})
    old = ops.moe_tc_min_pairs
    try:
        launches = []
        for least in (1024, 1 << 30):                        # the grouped form, then the mma.sync tiles
            ops.moe_tc_min_pairs = least
            before = ops.launches
            got = part.forward(h.cuda(), types.SimpleNamespace(ops=ops))
            launches.append(ops.launches - before)
            ops.check_kernels()
            scale = float(want.abs().max())
            torch.testing.assert_close(got.double().cpu(), want, atol=1.6e-2 * scale, rtol=1.6e-2)
        assert launches[0] == launches[1] + 1, "the grouped form (one more kernel: the gather) was not taken"
    finally:
        ops.moe_tc_min_pairs = old


@pytest.mark.parametrize("M,I,K", [(2048, 256, 128), (2100, 200, 192)])
def test_many_token_product_with_the_gelu_gate(ops, M, I, K):
    """From 2,048 tokens on the gate/up product runs on the tcgen05 kernel with the activation in its epilogue."""
    ops.set_compute_dtype(torch.bfloat16)
    h = randn(M, K, seed=1, dtype=torch.bfloat16)
    w = randn(2 * I, K, seed=2, dtype=torch.bfloat16, std=K ** -0.5)
    got = ops.gated_act_linear(h.cuda(), w.cuda(), "gelu_tanh").double().cpu()
    ops.check_kernels()
    z = (h.double() @ w.double().T).to(torch.bfloat16).double()
    want = plain_pomisun.gelu_tanh(z[:, :I]) * z[:, I:]
    torch.testing.assert_close(got, want, atol=2e-2, rtol=2e-2)


def test_router_weights_are_a_softmax_over_the_chosen(ops):
    """One expert far ahead, the others level: its weight is e^a / (e^a + (k - 1)), not a share of all experts."""
    ops.set_compute_dtype(torch.float32)
    D, E, k, F = 32, 7, 3, 16
    h = torch.zeros(2, D)
    h[:, 0] = 1.0
    router = torch.zeros(E, D)
    router[4, 0] = 2.0                                      # logits: 2 for expert 4, 0 for the rest
    eye_gate = torch.zeros(E, 2 * F, D)
    eye_gate[:, :, 0] = 1.0                                  # gate = up = 1 for every expert
    down = torch.zeros(E, D, F)
    for e in range(E):
        down[e, e, 0] = 1.0                                  # expert e writes silu(1) into column e
    y = ops.routed_experts(h.cuda(), router.cuda(), eye_gate.cuda(), down.cuda(), k).cpu()
    s1 = 1.0 / (1.0 + math.exp(-1.0))
    lead = math.exp(2.0) / (math.exp(2.0) + 2.0)
    assert y[0, 4].item() == pytest.approx(lead * s1, rel=1e-5)
    others = sorted(y[0, :E].tolist(), reverse=True)[1:3]
    assert others == pytest.approx([(1 - lead) / 2 * s1] * 2, rel=1e-5)      # ties go to the lowest indices
    assert y[0, 0].item() > 0 and y[0, 1].item() > 0 and y[0, 5].item() == 0


# ---------------------------------------------------------------- the engine against the plain model
LENGTHS = {"P": (5, 30, 77, 49, 24, 2, 60, 71, 35, 50), "Q": (1, 41, 90, 13, 80, 55, 66, 47),
           "R": (3, 70, 33, 65, 90, 41, 58, 77)}


def replay(folder, dtype, steps, max_tokens, block_size=16, **kw):
    from paged_llm_b200.engine.replay import TraceReplayer

    rp = TraceReplayer(folder, dtype, max_tokens, block_size=block_size, poison=float("nan"), max_num_seqs=4, **kw)
    outputs = {}
    for rec in steps:
        out = rp.step(rec)
        if out is not None:
            outputs[rec["step"]] = out
    assert not rp.live, "requests left alive at the end of the trace"
    rp.cm.check_invariants([])
    assert rp.cm.num_free_blocks == rp.cm.num_blocks, "pages were lost"
    return outputs, rp


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: case_folder(tmp_path_factory, name, dtype="bfloat16") for name in CASES}


@pytest.fixture(scope="module")
def requests(folders):
    return {name: clear_requests(folders[name], CASES[name][0]["vocab"], LENGTHS[name], seed=ord(name)) for name in CASES}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q", "R"])
@pytest.mark.parametrize("schedule", ["whole", "tail", "portions", "mixed"])
def test_schedule_matches_plain(folders, requests, name, dtype, schedule):
    reqs = requests[name]
    steps, max_tokens = getattr(schedules, schedule)(reqs)
    block = 8 if name == "Q" else 16
    outputs, rp = replay(folders[name], dtype, steps, max_tokens, block_size=block)
    got = schedules.collect(steps, outputs)
    for rid, toks in reqs.items():
        assert_logits_close(got[rid], plain_logits(folders[name], toks), dtype, f"{schedule}/{name}/{rid}")
    if schedule == "mixed":
        assert sum(-(-len(t) // block) for t in reqs.values()) > rp.cm.num_blocks, "pages must be used again"
    if schedule == "tail":
        assert rp.runner.num_graph_steps > 0, "decode steps replay graphs: every part of the model can be captured"


@pytest.mark.parametrize("name", ["P", "Q", "R"])
@pytest.mark.parametrize("schedule", ["tail", "portions", "mixed"])
def test_bfloat16_against_the_float32_engine(folders, requests, name, schedule):
    steps, max_tokens = getattr(schedules, schedule)(requests[name])
    a, _ = replay(folders[name], "float32", steps, max_tokens)
    b, _ = replay(folders[name], "bfloat16", steps, max_tokens)
    for k in a:
        assert_bf16_close_to_f32(b[k], a[k], f"{schedule}/{name}/step {k}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_and_eager_decode_agree(folders, requests, dtype):
    reqs = {k: v for k, v in list(requests["P"].items())[2:4]}
    steps, max_tokens = schedules.tail(reqs, last=30)                # the decoded tokens cross a chunk's edge
    a, rp_a = replay(folders["P"], dtype, steps, max_tokens)
    b, rp_b = replay(folders["P"], dtype, steps, max_tokens, enforce_eager=True)
    assert rp_a.runner.num_graph_steps > 0 and rp_b.runner.num_graph_steps == 0
    for k in a:
        assert_logits_close(a[k], b[k], dtype, f"graph vs eager step {k}")


@pytest.mark.parametrize("seed", range(10))
def test_generated_configurations(tmp_path, seed):
    """Other sizes, head counts, layer orders, chunks and constants than the fixed cases: a mixed schedule of four
    requests with reused pages, float32 against the plain model at every position, then bfloat16."""
    hf, init = generated_case(seed)
    folder = make_folder(tmp_path, hf, init, dtype="bfloat16")
    # (bfloat16 on shorter requests, drawn so that no router comes close to a tie)
    for dtype, reqs in (("float32", requests_for(hf["vocab"], (37, 3, 110, 64, 18, 75), seed=seed)),
                        ("bfloat16", clear_requests(folder, hf["vocab"], (30, 3, 48, 17, 40), seed=seed, margin=0.08))):
        steps, max_tokens = schedules.mixed(reqs, live=4, seed=seed)
        outputs, _ = replay(folder, dtype, steps, max_tokens)
        got = schedules.collect(steps, outputs)
        for rid, toks in reqs.items():
            assert_logits_close(got[rid], plain_logits(folder, toks), dtype, f"generated {seed}/{dtype}/{rid}")


def test_long_decoding_over_many_chunks(folders):
    """One token at a time from the third token on, over seven chunks: pages of finished chunks are given back
    while the request runs, and every token still matches."""
    hf = CASES["P"][0]
    toks = requests_for(hf["vocab"], (170,), seed=77)["r0"]
    steps, max_tokens = schedules.tail({"a": toks}, last=168)
    outputs, rp = replay(folders["P"], "float32", steps, max_tokens, block_size=8)
    got = schedules.collect(steps, outputs)["a"]
    assert_logits_close(got, plain_logits(folders["P"], toks), "float32", "long decoding")


def test_first_tokens(folders):
    """Requests of one and two tokens, alone and in one batch: the first positions of a sequence."""
    hf = CASES["Q"][0]
    a, b = requests_for(hf["vocab"], (1, 2), seed=5).values()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a, "want": [0]}, {"id": "b", "tokens": b, "want": [0, 1]}],
              "end": ["a", "b"]},
             {"step": 1, "entries": [{"id": "c", "tokens": b[:1], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "c", "tokens": b[1:], "want": [0]}], "end": ["c"]}]
    for dtype in ("float32", "bfloat16"):
        outputs, _ = replay(folders["Q"], dtype, steps, 128)
        assert_logits_close(outputs[0][:1], plain_logits(folders["Q"], a), dtype, "one token")
        assert_logits_close(outputs[0][1:], plain_logits(folders["Q"], b), dtype, "two tokens")
        assert_logits_close(np.concatenate([outputs[1], outputs[2]]), plain_logits(folders["Q"], b), dtype, "one by one")


@pytest.mark.parametrize("name", ["P", "R"])
def test_greedy_generation_through_the_engine(folders, name):
    from paged_llm_b200 import LLMEngine, SamplingParams
    hf = CASES[name][0]
    prompts = list(requests_for(hf["vocab"], (3, 22, 47, 9, 31), seed=60).values())
    eng = LLMEngine(folders[name], dtype="float32", block_size=8, num_gpu_blocks=24, max_model_len=96,
                    max_num_batched_tokens=16, max_num_seqs=4)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=30))
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain_greedy(folders[name], p, 30)
    assert eng.block_manager.num_free_blocks == 24
    assert eng.runner.num_graph_steps > 0 and eng.ops.launches > 0


def test_greedy_generation_in_bfloat16_follows_the_plain_model(folders):
    from paged_llm_b200 import LLMEngine, SamplingParams
    hf = CASES["Q"][0]
    prompts = list(requests_for(hf["vocab"], (4, 35, 62), seed=61).values())
    eng = LLMEngine(folders["Q"], dtype="bfloat16", block_size=16, num_gpu_blocks=32, max_model_len=128)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12))
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o.token_ids:
            ref = plain_logits(folders["Q"], seq)[-1]
            assert ref.max() - ref[tok] <= 3e-2 * np.abs(ref).max()
            seq.append(tok)


def test_trace_run_program(folders, requests, tmp_path):
    hf = CASES["R"][0]
    reqs = {k: v for k, v in list(requests["R"].items())[:4]}
    steps, max_tokens = schedules.mixed(reqs, live=3, seed=2)
    out_dir = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders["R"], "--dtype", "float32",
         "--out", str(out_dir), "--max-tokens", str(max_tokens), "--max-requests", "4"],
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
        assert_logits_close(got[rid], plain_logits(folders["R"], toks), "float32", f"trace_run/{rid}")
