"""Small Pomisun configurations for the tests, which differ from each other in every size and
option, and helpers to write their folders with random weights and to ask the plain model."""

from __future__ import annotations

import json
import os

import numpy as np
import torch

from paged_llm_b200.config import PomisunConfig
from paged_llm_b200.weights import write_model_folder
from tests import plain_pomisun


def _attn(heads, kv, dim, scale=None, softcap=None, chunk=None, rot=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": dim ** -0.5 if scale is None else scale}
    if softcap is not None:
        m["softcap"] = softcap
    if chunk is not None:
        m["mask"] = {"size": chunk}
    if rot is not None:
        m["rot"] = rot
    return m


def _layer(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


YARN = {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}

# P: a looped span of two layers (dense, then routed experts with a shared one) run twice, and a
# last layer without a feed-forward; chunks of 24 positions, rotation of the whole head with YaRN.
CASE_P = {
    "architecture": "Pomisun", "vocab": 211, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        _layer(_attn(4, 2, 16, softcap=30.0, chunk=24, rot={"dims": 16, "base": 10000.0, "scaling": YARN}),
               {"kind": "dense", "ff": 96}),
        _layer(_attn(4, 2, 16, softcap=30.0, chunk=24, rot={"dims": 16, "base": 10000.0, "scaling": YARN}),
               {"kind": "moe", "expert": {"ff": 32}, "router": {"experts": 6, "top": 2}, "shared": {"ff": 48}}),
        _layer(_attn(4, 4, 16, scale=0.3, chunk=24, rot={"dims": 16, "base": 10000.0, "scaling": YARN}), None),
    ],
    "loop": {"start": 0, "stop": 2, "times": 2},
}

# Q: layers that differ from each other: one without a mask and with a partial rotation without scaling,
# one with chunks of 40 (no multiple of a page) and no cap; every expert chosen (top = experts), an
# expert size that is no multiple of 8, no shared expert; the middle layer runs three times.
CASE_Q = {
    "architecture": "Pomisun", "vocab": 97, "width": 96, "norm": {"eps": 1e-6},
    "layers": [
        _layer(_attn(6, 3, 32, softcap=8.0, rot={"dims": 16, "base": 500.0}), {"kind": "dense", "ff": 72}),
        _layer(_attn(6, 2, 32, scale=0.2, chunk=40, rot={"dims": 32, "base": 500.0, "scaling": dict(YARN, factor=2.0)}),
               {"kind": "moe", "expert": {"ff": 20}, "router": {"experts": 5, "top": 5}}),
        _layer(_attn(3, 1, 32, softcap=15.0, chunk=7), {"kind": "dense", "ff": 40}),
    ],
    "loop": {"start": 1, "stop": 2, "times": 3},
}

# R: head size 64 without a cap (in bfloat16 the prefill of the layer without a mask runs on the tcgen05
# kernel), one expert per token, no loop.
CASE_R = {
    "architecture": "Pomisun", "vocab": 300, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        _layer(_attn(2, 1, 64, rot={"dims": 64, "base": 250000.0, "scaling": dict(YARN, original=128)}),
               {"kind": "moe", "expert": {"ff": 64}, "router": {"experts": 8, "top": 1}, "shared": {"ff": 32}}),
        _layer(_attn(4, 1, 64, chunk=32, rot={"dims": 64, "base": 250000.0, "scaling": dict(YARN, original=128)}),
               {"kind": "dense", "ff": 160}),
    ],
}

CASES = {"P": (CASE_P, dict(seed=11, std=0.08, norm_std=0.1)),
         "Q": (CASE_Q, dict(seed=12, std=0.1, norm_std=0.2)),
         "R": (CASE_R, dict(seed=13, std=0.06, norm_std=0.05))}


def generated_case(seed: int) -> tuple[dict, dict]:
    """A configuration drawn from a seed: widths, head counts and sizes, rotated dimensions, chunks, caps, kinds of
    feed-forward, the order of layers and the looped span all vary, within what the design allows."""
    import random
    rng = random.Random(seed)
    width = rng.choice([64, 96, 160, 200, 288, 384])
    n_layers = rng.randint(2, 4)
    layers = []
    for _ in range(n_layers):
        dim = rng.choice([16, 32, 48, 64, 80, 96, 128])
        kv = rng.choice([1, 2, 3])
        heads = kv * rng.choice([1, 2, 4, 5])
        rot = None
        if rng.random() < 0.85:
            rot = {"dims": rng.choice([dim, dim, dim // 2, dim - 8 if dim > 16 else dim]), "base": rng.choice([100.0, 10000.0, 500000.0])}
            if rng.random() < 0.7:
                rot["scaling"] = {"factor": rng.choice([1.5, 2.0, 4.0, 8.0]), "original": rng.choice([32, 64, 256]),
                                  "fast": rng.choice([8.0, 16.0, 32.0]), "slow": rng.choice([1.0, 2.0])}
        mixer = _attn(heads, kv, dim, scale=rng.choice([1.0, 0.7, 1.3]) * dim ** -0.5,
                      softcap=rng.choice([None, 5.0, 20.0, 50.0]), chunk=rng.choice([None, 7, 16, 33, 64, 100]), rot=rot)
        kind = rng.choice(["dense", "moe", "moe", None])
        if kind == "dense":
            mlp = {"kind": "dense", "ff": rng.choice([24, 64, 100, 256])}
        elif kind == "moe":
            experts = rng.choice([2, 3, 8, 12, 20])
            mlp = {"kind": "moe", "expert": {"ff": rng.choice([8, 20, 32, 64])},
                   "router": {"experts": experts, "top": rng.randint(1, min(experts, 4))}}
            if rng.random() < 0.6:
                mlp["shared"] = {"ff": rng.choice([16, 40, 96])}
        else:
            mlp = None
        layers.append(_layer(mixer, mlp))
    cfg = {"architecture": "Pomisun", "vocab": rng.choice([50, 131, 300, 777]), "width": width,
           "norm": {"eps": rng.choice([1e-6, 1e-5])}, "layers": layers}
    if rng.random() < 0.7:
        start = rng.randint(0, n_layers - 1)
        stop = rng.randint(start + 1, n_layers)
        cfg["loop"] = {"start": start, "stop": stop, "times": rng.randint(1, 3)}
    return cfg, dict(seed=seed, std=rng.choice([0.05, 0.1]), norm_std=0.1)


def make_folder(path, hf_cfg: dict, init: dict, dtype: str = "float32") -> str:
    return write_model_folder(str(path), PomisunConfig.from_hf_dict(hf_cfg), dtype=dtype, **init)


def case_folder(tmp_path_factory, name: str, dtype: str = "float32") -> str:
    hf, init = CASES[name]
    d = tmp_path_factory.mktemp(f"pomisun{name}_{dtype}")
    return make_folder(d, hf, init, dtype=dtype)


def read_folder(path) -> tuple[dict, dict]:
    from safetensors import safe_open

    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    tensors = {}
    with safe_open(os.path.join(path, "model.safetensors"), framework="pt", device="cpu") as f:
        for k in f.keys():
            tensors[k] = f.get_tensor(k)
    return cfg, tensors


def plain_logits(folder: str, tokens) -> np.ndarray:
    cfg, w = read_folder(folder)
    return plain_pomisun.forward(cfg, w, tokens).to(torch.float32).numpy()


def clear_requests(folder: str, vocab: int, lengths, seed: int = 0, margin: float = 0.02) -> dict[str, list[int]]:
    """Random requests on which no router of the model comes close to a tie (the last chosen expert leads the
    first rejected one by `margin` of the logits' spread at every token): the bfloat16 engine then chooses the
    experts the plain model chooses, and the two differ by rounding only.  A length for which 100 draws find no
    such request is shortened."""
    cfg, w = read_folder(folder)
    out = {}
    for i, n in enumerate(lengths):
        while f"r{i}" not in out:
            for attempt in range(100):
                g = torch.Generator().manual_seed(seed * 100003 + i * 401 + attempt)
                toks = torch.randint(0, vocab, (n,), generator=g).tolist()
                plain_pomisun.ROUTER_MARGINS = []
                try:
                    plain_pomisun.forward(cfg, w, toks)
                    worst = min(plain_pomisun.ROUTER_MARGINS, default=1.0)
                finally:
                    plain_pomisun.ROUTER_MARGINS = None
                if worst >= margin:
                    out[f"r{i}"] = toks
                    break
            else:
                if n <= 2:
                    raise AssertionError("no request without a close call, however short")
                n = max(2, n * 2 // 3)           # (few experts and many routed layers: a shorter request)
    return out


def plain_greedy(folder: str, prompt, n: int) -> list[int]:
    cfg, w = read_folder(folder)
    seq, out = list(prompt), []
    for _ in range(n):
        tok = int(plain_pomisun.forward(cfg, w, seq)[-1].argmax())
        out.append(tok)
        seq.append(tok)
    return out
