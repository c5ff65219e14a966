"""Small Rokarax configurations for the tests, which differ from each other in every size, constant and
order of layers, and helpers to write their folders with random weights and to ask the plain model.

The weights are drawn here, not by the package's random-weights mode, so that the vectors that shape the
recurrence (decays, step sizes, the convolution), the norms' alpha and the bias tables get values that
show a fault: a decay close to one keeps far tokens alive, a bias table of a few units moves the softmax.
"""

from __future__ import annotations

import json
import os
import random

import numpy as np
import torch

from paged_llm_b200.config.registry import parse_model_config
from paged_llm_b200.models.causal_lm import build_model
from tests import plain_rokarax


def attn(heads, kv, dim, vdim, bias_max, window=None, scale=None, kv_from=None, bias_rows=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale,
         "bias_max": bias_max}
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    if bias_rows is not None:
        m["bias_rows"] = bias_rows
    return m


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, window=None, scale=None, dims=None, base=10000.0, scaling=None):
    rot = {"dims": rot_dim if dims is None else dims, "base": base}
    if scaling is not None:
        rot["scaling"] = scaling
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": (dim + rot_dim) ** -0.5 if scale is None else scale, "rot": rot}
    if window is not None:
        m["mask"] = {"size": window}
    return m


def ssm(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


YARN = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}

# A: keys and values of different sizes, a bias table of 12 rows, a layer that reads the first layer's keys
# and values through a LARGER window than the owner's (the cache must keep what the reader needs), a latent
# layer with a partial rotation and no scaling, a state-space layer with one group; the last layer has no
# feed-forward.
CASE_A = {
    "architecture": "Rokarax", "vocab": 131, "width": 64, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
    "layers": [
        layer("attention", attn(4, 2, 16, 32, 50.0, window=24, bias_rows=12), 96),
        layer("mamba2", ssm(4, 8, 16, 1, 4, 1), 48),
        layer("latent_attention", latent(2, 24, 8, 16, 24, 40, window=17, dims=4), 80),
        layer("attention", attn(4, 2, 16, 32, 20.0, window=40, kv_from=0, bias_rows=6), None),
    ],
}

# B: starts with a state-space layer (state 24: no multiple of the lanes of a column; three groups; two taps),
# a latent layer whose cached head is exactly 64 wide with YaRN and a window longer than most requests, attention
# without a window and values shorter than keys, no embedding scale.
CASE_B = {
    "architecture": "Rokarax", "vocab": 77, "width": 96, "norm": {"eps": 1e-6},
    "layers": [
        layer("mamba2", ssm(6, 16, 24, 3, 2, 3), 64),
        layer("latent_attention", latent(3, 16, 16, 24, 32, 48, window=100, base=500.0, scaling=YARN), None),
        layer("attention", attn(6, 1, 32, 16, 30.0, bias_rows=8), 72),
        layer("mamba2", ssm(2, 40, 8, 2, 5, 4), 40),
    ],
}

# C: one kv head per query head, a window of one page, a latent layer without a window, a convolution of one
# tap (no history), a single state-space head.
CASE_C = {
    "architecture": "Rokarax", "vocab": 300, "width": 128, "embedding": {"scale": 0.5}, "norm": {"eps": 1e-5},
    "layers": [
        layer("latent_attention", latent(4, 32, 32, 32, 64, 96, base=1000000.0, scaling=dict(YARN, factor=8.0, original=64)), 160),
        layer("attention", attn(2, 2, 64, 64, 100.0, window=16, scale=0.2, bias_rows=32), 100),
        layer("mamba2", ssm(1, 64, 32, 1, 1, 2), None),
        layer("attention", attn(2, 2, 64, 64, 9.0, window=16, kv_from=1, bias_rows=4), 64),
    ],
}

CASES = {"A": (CASE_A, 21), "B": (CASE_B, 22), "C": (CASE_C, 23)}


def generated_case(seed: int) -> dict:
    """A configuration drawn from a seed: widths, head counts and sizes, ranks, windows, tables, the state-space
    sizes and the order of layers all vary, within what the design allows."""
    rng = random.Random(seed)
    width = rng.choice([48, 64, 96, 160, 200])
    layers = []
    owners = []
    for i in range(rng.randint(2, 5)):
        kind = rng.choice(["attention", "latent_attention", "mamba2"])
        ff = rng.choice([None, 24, 64, 100])
        if kind == "attention":
            if owners and rng.random() < 0.4:
                src = rng.choice(owners)
                m = dict(layers[src]["mixer"])
                m["kv_from"] = src
                m["heads"] = m["kv_heads"] * rng.choice([1, 2, 3])
                m["bias_max"] = rng.choice([9.0, 40.0, 200.0])
                m["bias_rows"] = rng.choice([4, 8, 16])
                w = rng.choice([None, 5, 16, 33, 64])
                m.pop("mask", None)
                if w is not None:
                    m["mask"] = {"size": w}
            else:
                kv = rng.choice([1, 2, 3])
                dim = rng.choice([8, 16, 24, 48, 64, 96])
                m = attn(kv * rng.choice([1, 2, 4]), kv, dim, rng.choice([dim, 8, 16, 40, 80]), rng.choice([12.0, 60.0, 150.0]),
                         window=rng.choice([None, 7, 16, 30, 64]), scale=rng.choice([0.7, 1.0, 1.4]) * dim ** -0.5,
                         bias_rows=rng.choice([4, 10, 16, 32]))
                if m["bias_max"] <= m["bias_rows"] // 2:
                    m["bias_max"] = float(m["bias_rows"])
                owners.append(i)
        elif kind == "latent_attention":
            rot_dim = rng.choice([2, 8, 16, 32])
            scaling = None
            if rng.random() < 0.6:
                scaling = {"factor": rng.choice([2.0, 4.0, 16.0]), "original": rng.choice([16, 64, 256]),
                           "fast": rng.choice([8.0, 32.0]), "slow": rng.choice([1.0, 2.0])}
            m = latent(rng.choice([1, 2, 4, 5]), rng.choice([8, 16, 40, 64]), rot_dim, rng.choice([8, 16, 48]),
                       rng.choice([16, 40, 64]), rng.choice([8, 24, 64, 112]), window=rng.choice([None, 9, 32, 50]),
                       dims=rng.choice([rot_dim, rot_dim, max(2, rot_dim // 2)]), base=rng.choice([100.0, 10000.0, 1e6]),
                       scaling=scaling)
        else:
            groups = rng.choice([1, 2, 3])
            heads = groups * rng.choice([1, 2, 4])
            vdim = rng.choice([8, 16, 24, 64])
            # (a part of a handful of elements makes its norm a steep function of every one of them: bfloat16
            # rounding then says more about the draw than about the engine)
            parts = rng.choice([d for d in (1, 2, 3, 4, 8) if (heads * vdim) % d == 0 and heads * vdim // d >= 16])
            m = ssm(heads, vdim, rng.choice([4, 8, 16, 20, 64, 128]), groups, rng.choice([1, 2, 3, 4]), parts)
        layers.append(layer(kind, m, ff))
    return {"architecture": "Rokarax", "vocab": rng.choice([50, 131, 300, 777]), "width": width,
            "embedding": {"scale": rng.choice([1.0, 2.0, 11.0])}, "norm": {"eps": rng.choice([1e-6, 1e-5])}, "layers": layers}


def draw_weights(hf_cfg: dict, seed: int) -> dict[str, torch.Tensor]:
    """Every tensor the model expects, in float32 with values that bfloat16 holds exactly."""
    arch, cfg = parse_model_config(hf_cfg)
    specs = build_model(arch.build_spec(cfg)).tensor_specs()
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name in sorted(specs):
        shape = specs[name].draw_shape or specs[name].shape
        r = torch.randn(shape, generator=g)
        if name.endswith(".alpha"):
            t = 0.6 + 0.3 * torch.rand(shape, generator=g)
        elif name.endswith(".b"):
            t = 0.1 * r                                            # norm biases and the convolution's bias
        elif ".norm" in name:
            t = 1.0 + 0.2 * r                                      # every norm's weight
        elif name.endswith(".rel"):
            t = 1.5 * r
        elif name.endswith(".conv"):
            t = 0.5 * r
        elif name.endswith(".dt_bias"):
            t = -1.0 + r                                           # steps from 0.1 to 1
        elif name.endswith(".A_log"):
            t = -2.5 + 1.5 * torch.rand(shape, generator=g)       # decays per unit step between 0.7 and 0.92
        elif name.endswith(".D"):
            t = 1.0 + 0.3 * r
        elif name == "embed":
            t = 0.5 * r
        else:
            t = r * (1.2 / np.sqrt(shape[-1]))                     # matrices: outputs of the order of their inputs
        out[name] = t.to(torch.bfloat16).float().contiguous()
    return out


def make_folder(path, hf_cfg: dict, seed: int, dtype: str = "bfloat16", weights=None) -> str:
    from safetensors.torch import save_file

    path = str(path)
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(hf_cfg, f, indent=1)
    w = weights if weights is not None else draw_weights(hf_cfg, seed)
    save_file({k: v.to(torch.bfloat16 if dtype == "bfloat16" else torch.float32).contiguous() for k, v in w.items()},
              os.path.join(path, "model.safetensors"))
    return path


def case_folder(tmp_path_factory, name: str) -> str:
    hf, seed = CASES[name]
    return make_folder(tmp_path_factory.mktemp(f"rokarax{name}"), hf, seed)


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
    with torch.no_grad():
        return plain_rokarax.forward(cfg, w, tokens).to(torch.float32).numpy()


def plain_greedy(folder: str, prompt, n: int) -> list[int]:
    cfg, w = read_folder(folder)
    seq, out = list(prompt), []
    for _ in range(n):
        tok = int(plain_rokarax.forward(cfg, w, seq)[-1].argmax())
        out.append(tok)
        seq.append(tok)
    return out
