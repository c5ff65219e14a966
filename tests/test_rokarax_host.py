"""The Rokarax decoder on the host: configuration, the model as data, the cache's needs, and the engine's
host logic (runner, cache manager, state slots, replay, scheduler) with the kernel library replaced by the
tensor-code stand-in, against the plain implementation."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from paged_llm_b200.config.model import ConfigError
from paged_llm_b200.config.registry import parse_model_config
from paged_llm_b200.config.rokarax import RokaraxConfig
from paged_llm_b200.models.causal_lm import build_model
from paged_llm_b200.parts.attention import log_distance_buckets
from paged_llm_b200.parts.base import FixedState, PagedKV
from tests import plain_rokarax, schedules
from tests.helpers import requests_for
from tests.rokarax_cases import (CASE_A, CASE_B, CASES, case_folder, generated_case, make_folder, plain_greedy,
                                 plain_logits)
from tests.torch_ops import TorchOps

F32_TOL = 2e-5


def close(got, want, what):
    assert got.shape == want.shape, what
    assert np.isfinite(got).all(), what
    tol = F32_TOL * max(1.0, float(np.abs(want).max()))
    err = np.abs(got - want)
    assert err.max() <= tol, f"{what}: max |diff| {err.max():.3e} > {tol:.3e}, first bad row {int(np.argmax(err.max(axis=1) > tol))}"


def replay(folder, steps, max_tokens, block_size=8, slots=4):
    from paged_llm_b200.engine.replay import TraceReplayer

    rp = TraceReplayer(folder, "float32", max_tokens, device="cpu", ops=TorchOps(), block_size=block_size, max_num_seqs=slots)
    outputs = {}
    for rec in steps:
        out = rp.step(rec)
        if out is not None:
            outputs[rec["step"]] = out
    assert not rp.live
    rp.cm.check_invariants([])
    for g in range(len(rp.cm.pools)):
        assert rp.cm.num_free_in_group(g) == rp.cm.pools[g].num_pages, "pages were lost"
    assert rp.cm.num_free_state_slots == rp.cm.num_state_slots, "state slots were lost"
    return outputs, rp


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: case_folder(tmp_path_factory, name) for name in CASES}


# ---------------------------------------------------------------- configuration
def test_configuration_round_trip():
    for hf, _ in CASES.values():
        arch, cfg = parse_model_config(hf)
        assert arch.name == "Rokarax"
        again = RokaraxConfig.from_hf_dict(cfg.to_hf_dict())
        assert again == cfg
        assert cfg.num_parameters == sum(int(np.prod(s.draw_shape or s.shape)) for s in build_model(arch.build_spec(cfg)).tensor_specs().values())


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="conv"), "not implemented"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "multiple"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(dim=24), "differ"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=10), "dims"),
    (lambda c: c["layers"][1]["mixer"].update(groups=3), "groups"),
    (lambda c: c["layers"][1]["mixer"].update(norm_groups=5), "norm_groups"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "dense only"),
    (lambda c: c.pop("width"), "width"),
])
def test_configuration_refusals(change, message):
    import copy
    hf = copy.deepcopy(CASE_A)
    change(hf)
    with pytest.raises(ConfigError, match=message):
        parse_model_config(hf)


def test_the_model_as_data():
    arch, cfg = parse_model_config(CASE_A)
    model = build_model(arch.build_spec(cfg))
    names = set(model.tensor_specs())
    assert {"embed", "head", "final.norm", "final.norm.b", "final.norm.alpha", "l0.mix.q.norm", "l0.mix.rel", "l0.mix.g",
            "l1.mix.in", "l1.mix.conv.b", "l1.mix.A_log", "l2.mix.dq.norm", "l2.mix.uk", "l3.norm1b.alpha"} <= names
    # the layer that reads another layer's cache has no key and value tensors, and the layer without a
    # feed-forward no second pair of norms
    assert not {"l3.mix.k", "l3.mix.v", "l3.mix.k.norm", "l3.norm2", "l3.mlp.gate"} & names
    slots = model.cache_slots()
    # the owner keeps what its reader needs: the reader's window of 40, not its own of 24; keys of 16 and values
    # of 32 share a head of 32
    assert slots[0].requirement == PagedKV(2, 32, 40) and slots[3].shares == 0 and slots[3].requirement == slots[0].requirement
    assert slots[2].requirement == PagedKV(1, 48, 17)
    assert slots[1].requirement == FixedState((3 * (32 + 2 * 16) + 4 * 8 * 16,))
    assert model.has_fixed_state and model.capturable
    keys = {b.mixer.attention_plan_key() for b in model.blocks if hasattr(b.mixer, "attention_plan_key")}
    assert keys == {(2, 2, 24, 32), (2, 1, 17, 48), (2, 2, 40, 32)}


def test_bias_rows_follow_the_checkpoint(tmp_path):
    """The number of rows of a bias table is the tensor's, whatever the configuration would draw."""
    import copy
    from tests.rokarax_cases import draw_weights
    hf = copy.deepcopy(CASE_B)
    w = draw_weights(hf, 5)
    g = torch.Generator().manual_seed(1)
    w["l2.mix.rel"] = torch.randn(20, 6, generator=g).to(torch.bfloat16).float()
    folder = make_folder(tmp_path, hf, 5, weights=w)
    reqs = requests_for(hf["vocab"], (45,), seed=3)
    steps, max_tokens = schedules.portions(reqs)
    outputs, _ = replay(folder, steps, max_tokens)
    got = schedules.collect(steps, outputs)
    close(got["r0"], plain_logits(folder, reqs["r0"]), "a table of 20 rows")


# ---------------------------------------------------------------- mechanisms on hand-checked values
def test_distance_buckets_by_hand():
    # 8 rows, farthest 64: distances 0..3 have rows of their own; 4 * 2^k starts row 4 + k
    rows = log_distance_buckets(8, 64.0, 80)
    assert rows[:4] == [0, 1, 2, 3] and rows[4] == 4 and rows[7] == 4 and rows[9] == 5 and rows[17] == 6 and rows[33] == 7
    assert rows[63] == 7 and rows[64] == 7 and rows[79] == 7
    assert rows == [plain_rokarax.bucket(n, 8, 64.0) for n in range(80)]
    for table, far in ((32, 120.0), (12, 50.0), (5, 9.0), (2, 3.0)):
        mine = log_distance_buckets(table, far, 300)
        assert mine == [plain_rokarax.bucket(n, table, far) for n in range(300)]
        assert mine == sorted(mine) and mine[-1] == table - 1 and mine[int(math.ceil(far))] == table - 1


def test_dynamic_tanh_and_the_sum_by_hand():
    ops = TorchOps()
    x = torch.tensor([[1.0, -2.0]])
    branch = torch.tensor([[0.5, 0.25]])
    post = (torch.tensor([2.0]), torch.tensor([1.0, 3.0]), torch.tensor([0.0, 1.0]))
    pre = (torch.tensor([0.5]), torch.tensor([2.0, 2.0]), torch.tensor([-1.0, 0.0]))
    y = ops.dyt(x, branch, post, pre)
    added = torch.tensor([[1.0 + math.tanh(1.0), -2.0 + 3 * math.tanh(0.5) + 1.0]])
    assert torch.allclose(x, added)
    assert torch.allclose(y, torch.tanh(0.5 * added) * 2.0 + torch.tensor([-1.0, 0.0]))


def test_recurrence_by_hand():
    # one head, one state value, head size one: S_t = a_t S + dt_t B_t x_t, y = S C + D x
    x = torch.tensor([[[1.0]], [[2.0]]], dtype=torch.float64)
    dt = torch.tensor([[0.5], [0.25]], dtype=torch.float64)
    B = torch.tensor([[[2.0]], [[1.0]]], dtype=torch.float64)
    C = torch.tensor([[[1.0]], [[3.0]]], dtype=torch.float64)
    y = plain_rokarax.selective_scan(x, dt, torch.tensor([0.0]), B, C, torch.tensor([10.0]), 1)
    s1 = 0.5 * 2.0 * 1.0
    s2 = math.exp(-0.25) * s1 + 0.25 * 1.0 * 2.0
    assert torch.allclose(y.flatten(), torch.tensor([s1 * 1.0 + 10.0, s2 * 3.0 + 20.0], dtype=torch.float64))


# ---------------------------------------------------------------- the engine's host logic against the plain model
LENGTHS = {"A": (1, 30, 77, 49, 2, 60, 90, 35), "B": (5, 41, 120, 13, 80, 55), "C": (3, 70, 33, 65, 18, 41)}


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("schedule", ["whole", "tail", "portions", "mixed"])
def test_schedule_matches_plain(folders, name, schedule):
    hf = CASES[name][0]
    reqs = requests_for(hf["vocab"], LENGTHS[name], seed=ord(name))
    steps, max_tokens = getattr(schedules, schedule)(reqs)
    outputs, rp = replay(folders[name], steps, max_tokens)
    got = schedules.collect(steps, outputs)
    for rid, toks in reqs.items():
        close(got[rid], plain_logits(folders[name], toks), f"{schedule}/{name}/{rid}")
    if schedule == "mixed":
        assert len(reqs) > 4, "state slots must be used again"


def test_pages_behind_the_widest_reader_are_given_back(folders):
    """Case A: the first layer's window is 24 but the layer that reads its cache looks 40 back: pages go when
    position - 40 has passed them, and not before."""
    from paged_llm_b200.engine.replay import TraceReplayer
    rp = TraceReplayer(folders["A"], "float32", 128, device="cpu", ops=TorchOps(), block_size=8, max_num_seqs=2)
    toks = requests_for(CASE_A["vocab"], (100,), seed=9)["r0"]
    rp.step({"step": 0, "entries": [{"id": "a", "tokens": toks[:70], "want": []}], "end": []})
    seq = rp.live["a"]
    shared = [g for g, spec in enumerate(rp.cm.group_specs) if spec.window == 40][0]
    latent = [g for g, spec in enumerate(rp.cm.group_specs) if spec.window == 17][0]
    # next query at 70: needs keys from 31 (window 40) and from 54 (window 17)
    assert [p >= 0 for p in seq.block_tables[shared]] == [False] * 3 + [True] * 6
    assert [p >= 0 for p in seq.block_tables[latent]] == [False] * 6 + [True] * 3
    out = rp.step({"step": 1, "entries": [{"id": "a", "tokens": toks[70:], "want": list(range(30))}], "end": ["a"]})
    close(out, plain_logits(folders["A"], toks)[70:], "behind released pages")


def test_state_does_not_leak_between_requests(folders):
    """A slot that is used again starts from zero: the second request equals itself run alone."""
    reqs = requests_for(CASE_B["vocab"], (40, 37), seed=4)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": reqs["r0"], "want": []}], "end": ["x"]},
             {"step": 1, "entries": [{"id": "y", "tokens": reqs["r1"], "want": list(range(37))}], "end": ["y"]}]
    outputs, rp = replay(folders["B"], steps, 64, slots=1)
    close(outputs[1], plain_logits(folders["B"], reqs["r1"]), "a slot used again")


@pytest.mark.parametrize("seed", range(6))
def test_generated_configurations(tmp_path, seed):
    hf = generated_case(seed)
    folder = make_folder(tmp_path, hf, seed)
    reqs = requests_for(hf["vocab"], (2, 50, 21, 70, 9), seed=seed)
    steps, max_tokens = schedules.mixed(reqs, live=3, seed=seed)
    outputs, _ = replay(folder, steps, max_tokens, block_size=8, slots=3)
    got = schedules.collect(steps, outputs)
    for rid, toks in reqs.items():
        close(got[rid], plain_logits(folder, toks), f"generated {seed}/{rid}")


def test_greedy_generation_through_the_engine(folders):
    from paged_llm_b200 import LLMEngine, SamplingParams
    prompts = list(requests_for(CASE_A["vocab"], (3, 22, 47, 9, 31), seed=60).values())
    eng = LLMEngine(folders["A"], dtype="float32", device="cpu", ops=TorchOps(), block_size=8, num_gpu_blocks=40,
                    max_model_len=96, max_num_batched_tokens=16, max_num_seqs=3)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12))
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain_greedy(folders["A"], p, 12)
    assert eng.block_manager.num_free_state_slots == 3


def test_generation_with_preemption_restarts_the_state(folders):
    """So few pages that running requests are preempted: a request that comes back starts at position 0 with a
    zeroed state slot and ends with the tokens of an undisturbed run."""
    from paged_llm_b200 import LLMEngine, SamplingParams
    prompts = list(requests_for(CASE_B["vocab"], (30, 26, 21, 12), seed=70).values())
    eng = LLMEngine(folders["B"], dtype="float32", device="cpu", ops=TorchOps(), block_size=8, num_gpu_blocks=11,
                    max_model_len=88, max_num_batched_tokens=24, max_num_seqs=4)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=16))
    assert sum(o.num_preemptions for o in outs) > 0, "the pool was meant to run out"
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain_greedy(folders["B"], p, 16)
    assert eng.block_manager.num_free_state_slots == 4
