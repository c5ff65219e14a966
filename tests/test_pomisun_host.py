"""The Pomisun decoder on the host: configuration, the model as data, the cache's handling of chunks,
and the engine's host logic (step function, cache manager, scheduler, replay) with the kernel library
replaced by the tests' stand-in, against the plain implementation."""

import copy
import math

import numpy as np
import pytest
import torch

from paged_llm_b200.cache.manager import CacheManager, GroupSpec
from paged_llm_b200.config import ConfigError, PomisunConfig, parse_model_config
from paged_llm_b200.engine.sequence import NO_PAGE, Sequence
from paged_llm_b200.config.sampling import SamplingParams
from paged_llm_b200.kernels.plan import first_visible_key, plan_attention
from paged_llm_b200.models import build_model, pomisun_spec
from paged_llm_b200.parts.rope import RotaryEncoding
from tests import plain_pomisun, schedules
from tests.helpers import assert_logits_close, requests_for
from tests.pomisun_cases import CASE_P, CASE_Q, CASES, case_folder, generated_case, make_folder, plain_greedy, plain_logits
from tests.torch_ops import TorchOps

LENGTHS = {"P": (5, 30, 77, 49, 24, 2, 60, 71, 35, 50), "Q": (1, 41, 90, 13, 80, 55, 66, 47), "R": (3, 70, 33, 65, 90, 41, 58, 77)}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: case_folder(tmp_path_factory, name) for name in CASES}


# ---------------------------------------------------------------- configuration and spec
def test_config_round_trip_and_registry():
    for hf, _ in CASES.values():
        arch, cfg = parse_model_config(hf)
        assert arch.name == "Pomisun" and isinstance(cfg, PomisunConfig)
        again = PomisunConfig.from_hf_dict(cfg.to_hf_dict())
        assert again == cfg
    cfg = PomisunConfig.from_hf_dict(CASE_Q)
    assert cfg.layers[0].mixer.chunk is None and cfg.layers[1].mixer.chunk == 40 and cfg.layers[1].mixer.softcap is None
    assert cfg.layers[2].mixer.rot is None and cfg.layers[0].mixer.rot.scaling is None
    assert cfg.layers[1].mlp.shared_ff is None and cfg.layers[1].mlp.top == 5


def test_layer_runs_follow_the_loop():
    assert PomisunConfig.from_hf_dict(CASE_P).layer_runs() == [(0, False), (1, False), (0, True), (1, False), (2, False)]
    assert PomisunConfig.from_hf_dict(CASE_Q).layer_runs() == [(0, False), (1, False), (1, True), (1, True), (2, False)]
    once = dict(CASE_P, loop={"start": 1, "stop": 3, "times": 1})
    assert PomisunConfig.from_hf_dict(once).layer_runs() == [(0, False), (1, False), (2, False)]
    assert plain_pomisun.layer_order(CASE_P) == PomisunConfig.from_hf_dict(CASE_P).layer_runs()
    assert plain_pomisun.layer_order(CASE_Q) == PomisunConfig.from_hf_dict(CASE_Q).layer_runs()


@pytest.mark.parametrize("breakage, message", [
    (lambda c: c["layers"][0].update(type="recurrent"), "not implemented"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=8), "values are the keys"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=7), "router.top"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "dims"),
    (lambda c: c.update(loop={"start": 2, "stop": 1, "times": 2}), "loop"),
    (lambda c: c["layers"][0]["mlp"].update(kind="conv"), "not implemented"),
    (lambda c: c.pop("vocab"), "vocab"),
])
def test_config_refuses_what_is_not_computed(breakage, message):
    cfg = copy.deepcopy(CASE_P)
    breakage(cfg)
    with pytest.raises(ConfigError, match=message):
        PomisunConfig.from_hf_dict(cfg)


def test_spec_names_the_checkpoint_tensors_and_caches():
    model = build_model(pomisun_spec(PomisunConfig.from_hf_dict(CASE_P)))
    names = set(model.tensor_specs())
    assert {"embed", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.k", "l0.mix.o", "l0.mlp.gate",
            "l1.mlp.router", "l1.mlp.e5.down", "l1.mlp.shared.sg", "l2.mix.o"} <= names
    assert "l2.norm2" not in names and "l0.mix.v" not in names and not any(n.startswith("l2.mlp") for n in names)
    assert model.tensor_specs()["l1.mlp.shared.sg"].shape == (1, 64)
    slots = model.cache_slots()
    assert len(slots) == 5 and all(s.shares is None for s in slots)            # every run has a cache of its own
    assert slots[0].requirement.chunk == 24 and slots[0].requirement.num_kv_heads == 2
    assert slots[4].requirement.num_kv_heads == 4
    assert len(model.positions) == 1                                            # equal rotations share one table
    model_q = build_model(pomisun_spec(PomisunConfig.from_hf_dict(CASE_Q)))
    assert len(model_q.positions) == 2 and model_q.blocks[2].mixer.position is None


# ---------------------------------------------------------------- mechanisms on the host
def test_yarn_frequencies_and_magnitude():
    for dims, base, sc in ((16, 10000.0, {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}),
                           (32, 500.0, {"factor": 2.0, "original": 64, "fast": 16.0, "slow": 2.0}),
                           (8, 100.0, {"factor": 8.0, "original": 32, "fast": 4.0, "slow": 4.0})):      # lo == hi
        enc = RotaryEncoding({}, head_dim=dims, theta=base, scaling=dict(sc, type="yarn"), rotary_dim=dims)
        f, mag = enc.frequencies()
        want, want_mag = plain_pomisun.rotary_frequencies({"dims": dims, "base": base, "scaling": sc})
        np.testing.assert_allclose(f.double().numpy(), want.numpy(), rtol=1e-6)
        assert mag == pytest.approx(want_mag) and mag == pytest.approx(0.1 * math.log(sc["factor"]) + 1)
    # the fastest pair keeps its frequency, the slowest gets 1/factor of it
    enc = RotaryEncoding({}, head_dim=64, theta=10000.0, scaling={"type": "yarn", "factor": 4.0, "original": 64,
                                                                   "fast": 16.0, "slow": 2.0}, rotary_dim=64)
    f, _ = enc.frequencies()
    plain = 10000.0 ** (-torch.arange(0, 64, 2, dtype=torch.float64) / 64)
    assert f[0].item() == pytest.approx(plain[0].item()) and f[-1].item() == pytest.approx(plain[-1].item() / 4.0)


def test_first_visible_key():
    assert [first_visible_key(p, None, 8) for p in (0, 7, 8, 15, 16, 23)] == [0, 0, 8, 8, 16, 16]
    assert first_visible_key(21, 4, 8) == 18 and first_visible_key(17, 4, 8) == 16 and first_visible_key(5, None, None) == 0


def test_plan_splits_only_the_keys_of_the_chunk():
    # a decoded token at position 1,000 with chunks of 80: 41 keys, one split, whatever the context
    plan = plan_attention([1], [1001], 4, 2, None, chunk=80, small_rows=16, large_rows=64, min_split_keys=64, num_sms=148)
    assert plan["small"].reshape(-1, 4).tolist() == [[0, 0, 0, 1]]
    plan = plan_attention([1], [1001], 4, 2, None, small_rows=16, large_rows=64, min_split_keys=64, num_sms=148)
    assert plan["small"].reshape(-1, 4)[0, 3] > 1


def test_cache_gives_back_the_pages_of_finished_chunks():
    cm = CacheManager([GroupSpec(16, None, 24)], 8, enable_prefix_caching=False)
    seq = Sequence(list(range(70)), SamplingParams())
    assert cm.allocate_slots(seq, 70) is not None
    for done, gone in ((23, 0), (24, 3), (47, 3), (48, 6), (70, 6)):
        seq.num_computed_tokens = done
        cm.release_behind_window(seq)
        table = seq.block_tables[0]
        assert [p == NO_PAGE for p in table].count(True) == gone and all(p == NO_PAGE for p in table[:gone]), (done, table)
    cm.free(seq)
    assert cm.num_free_blocks == 16
    # a chunk that is no multiple of a page: the page that straddles the edge stays
    cm = CacheManager([GroupSpec(16, None, 20)], 8, enable_prefix_caching=False)
    seq = Sequence(list(range(50)), SamplingParams())
    cm.allocate_slots(seq, 50)
    seq.num_computed_tokens = 41
    cm.release_behind_window(seq)
    assert [p == NO_PAGE for p in seq.block_tables[0]] == [True, True, True, True, True, False, False]
    assert not CacheManager([GroupSpec(4, None, 8)], 8, enable_prefix_caching=True).enable_prefix_caching


# ---------------------------------------------------------------- the engine's host logic against the plain model
def replay(folder, steps, max_tokens, block_size=8):
    from paged_llm_b200.engine.replay import TraceReplayer

    rp = TraceReplayer(folder, "float32", max_tokens, device="cpu", ops=TorchOps(), block_size=block_size, max_num_seqs=4)
    outputs = {}
    for rec in steps:
        out = rp.step(rec)
        if out is not None:
            outputs[rec["step"]] = out
    assert not rp.live
    rp.cm.check_invariants([])
    assert rp.cm.num_free_blocks == rp.cm.num_blocks, "pages were lost"
    return outputs, rp


@pytest.mark.parametrize("name", ["P", "Q", "R"])
@pytest.mark.parametrize("schedule", ["whole", "tail", "portions", "mixed"])
def test_replay_schedules_on_the_host(folders, name, schedule):
    hf, _ = CASES[name]
    reqs = requests_for(hf["vocab"], LENGTHS[name], seed=ord(name))
    steps, max_tokens = getattr(schedules, schedule)(reqs)
    outputs, rp = replay(folders[name], steps, max_tokens)
    got = schedules.collect(steps, outputs)
    for rid, toks in reqs.items():
        assert_logits_close(got[rid], plain_logits(folders[name], toks), "float32", f"{schedule}/{name}/{rid}")
    if schedule == "mixed":
        assert sum(-(-len(t) // 8) for t in reqs.values()) > rp.cm.num_blocks, "pages must be used again"


@pytest.mark.parametrize("seed", range(10, 14))
def test_generated_configurations_on_the_host(tmp_path, seed):
    hf, init = generated_case(seed)
    assert PomisunConfig.from_hf_dict(PomisunConfig.from_hf_dict(hf).to_hf_dict()) == PomisunConfig.from_hf_dict(hf)
    folder = make_folder(tmp_path, hf, init)
    reqs = requests_for(hf["vocab"], (21, 2, 70, 45), seed=seed)
    steps, max_tokens = schedules.mixed(reqs, live=3, seed=seed)
    outputs, _ = replay(folder, steps, max_tokens)
    got = schedules.collect(steps, outputs)
    for rid, toks in reqs.items():
        assert_logits_close(got[rid], plain_logits(folder, toks), "float32", f"generated {seed}/{rid}")


def test_greedy_generation_on_the_host(folders):
    from paged_llm_b200 import LLMEngine
    from paged_llm_b200 import SamplingParams as SP
    hf, _ = CASES["P"]
    prompts = [requests_for(hf["vocab"], (n,), seed=40 + n)["r0"] for n in (3, 22, 47)]
    eng = LLMEngine(folders["P"], ops=TorchOps(), dtype="float32", device="cpu", block_size=8, num_gpu_blocks=20,
                    max_model_len=96, max_num_batched_tokens=16, max_num_seqs=4)
    outs = eng.generate(prompts, SP(temperature=0.0, max_tokens=30))       # decoding crosses a chunk's edge
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain_greedy(folders["P"], p, 30)
    assert eng.block_manager.num_free_blocks == 20


def test_plain_model_mechanisms():
    """The plain implementation's own pieces, on values that can be checked by hand."""
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    np.testing.assert_allclose(plain_pomisun.norm_around_zero(x, torch.tensor([0.0, 1.0]), 0.0).numpy(),
                               [[3 / math.sqrt(12.5), 8 / math.sqrt(12.5)]])
    assert plain_pomisun.chunk_visible(5, 2).tolist() == [[True, False, False, False, False], [True, True, False, False, False],
                                                          [False, False, True, False, False], [False, False, True, True, False],
                                                          [False, False, False, False, True]]
    assert plain_pomisun.gelu_tanh(torch.tensor(1.0, dtype=torch.float64)).item() == pytest.approx(0.8411919906082768)
    # one expert of two with all the weight: the routed sum is that expert's output
    h = torch.tensor([[1.0, 0.0]], dtype=torch.float64)
    w = {"m.router": torch.tensor([[5.0, 0.0], [-5.0, 0.0]], dtype=torch.float64)}
    for e in range(2):
        w[f"m.e{e}.gate"] = torch.full((3, 2), 1.0 + e, dtype=torch.float64)
        w[f"m.e{e}.up"] = torch.ones(3, 2, dtype=torch.float64)
        w[f"m.e{e}.down"] = torch.ones(2, 3, dtype=torch.float64)
    y = plain_pomisun.routed(h, {"router": {"experts": 2, "top": 1}}, w, "m.")
    assert y[0, 0].item() == pytest.approx(3 * (1.0 / (1.0 + math.exp(-1.0))))
