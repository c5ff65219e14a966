"""Typed configuration of the Rokarax decoder, read from a checkpoint's config.json.

config.json gives every size and every constant that may differ between models of the design:

    architecture     "Rokarax"
    vocab, width     vocabulary and width of the residual stream
    embedding.scale  factor on the embedding's rows
    norm.eps         epsilon of every RMS norm inside the mixers
    layers           one entry per layer: `type` (the mixer), `mixer` (its sizes and constants) and `mlp`
                     ({"kind": "dense", "ff": n}, or null for none)

Mixers by `type`:

    "attention"         heads, kv_heads, dim (query/key head), vdim (value head), scale, bias_max (the distance
                        at which the bias table ends; the table's rows are the checkpoint tensor's; `bias_rows`,
                        optional, only says how many rows random weights are drawn with), mask.size (window;
                        absent: all earlier keys),
                        kv_from (optional: the layer whose keys and values this one reads)
    "latent_attention"  heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, mask.size,
                        rot {dims, base, scaling {factor, original, fast, slow} (optional)}
    "mamba2"            heads, vdim (head size), state, groups, conv (taps), norm_groups

What the engine does not compute is refused here with a message, never computed wrongly.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any

from .model import ConfigError, ModelConfig

MIXER_TYPES = ("attention", "latent_attention", "mamba2")


def _need(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json: {where} lacks the key {key!r}")
    return d[key]


def _positive_int(d, key: str, where: str) -> int:
    v = int(_need(d, key, where))
    if v < 1:
        raise ConfigError(f"{where}: {key}={v} must be positive")
    return v


def _window(d: dict, where: str) -> int | None:
    size = (d.get("mask") or {}).get("size")
    if size is None:
        return None
    if int(size) < 1:
        raise ConfigError(f"{where}: mask.size={size} must be positive")
    return int(size)


@dataclass(frozen=True)
class RokaraxAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    bias_max: float
    window: int | None = None
    kv_from: int | None = None
    bias_rows: int = 32                 # rows of the bias table that random weights are drawn with (a checkpoint's own count rules)

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "RokaraxAttention":
        heads, kv = _positive_int(d, "heads", where), _positive_int(d, "kv_heads", where)
        if heads % kv:
            raise ConfigError(f"{where}: heads={heads} is not a multiple of kv_heads={kv}")
        dim = _positive_int(d, "dim", where)
        kv_from = d.get("kv_from")
        return cls(heads, kv, dim, int(d.get("vdim", dim)), float(_need(d, "scale", where)),
                   float(_need(d, "bias_max", where)), _window(d, where), int(kv_from) if kv_from is not None else None,
                   int(d.get("bias_rows", 32)))

    def to_dict(self) -> dict:
        d: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                             "scale": self.scale, "bias_max": self.bias_max}
        if self.bias_rows != 32:
            d["bias_rows"] = self.bias_rows
        if self.window is not None:
            d["mask"] = {"size": self.window}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class RokaraxRotary:
    dims: int
    base: float
    scaling: tuple | None = None          # ((name, value), ...) of factor, original, fast, slow

    @classmethod
    def from_dict(cls, d: dict, rot_dim: int, where: str) -> "RokaraxRotary":
        dims, base = int(_need(d, "dims", where)), float(_need(d, "base", where))
        if dims <= 0 or dims % 2 or dims > rot_dim:
            raise ConfigError(f"{where}: dims={dims} must be even and at most rot_dim={rot_dim}")
        if not base > 0:
            raise ConfigError(f"{where}: base={base} must be positive")
        sc = d.get("scaling")
        if sc is not None:
            sc = tuple((k, float(_need(sc, k, where + ".scaling"))) for k in ("factor", "original", "fast", "slow"))
            if not all(v > 0 for _, v in sc):
                raise ConfigError(f"{where}.scaling: factor, original, fast and slow must be positive")
        return cls(dims, base, sc)

    def to_dict(self) -> dict:
        d: dict[str, Any] = {"dims": self.dims, "base": self.base}
        if self.scaling is not None:
            d["scaling"] = dict(self.scaling)
        return d


@dataclass(frozen=True)
class RokaraxLatentAttention:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot: RokaraxRotary
    window: int | None = None

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "RokaraxLatentAttention":
        rot_dim = _positive_int(d, "rot_dim", where)
        if rot_dim % 2:
            raise ConfigError(f"{where}: rot_dim={rot_dim} must be even")
        dim = _positive_int(d, "dim", where)
        return cls(_positive_int(d, "heads", where), dim, rot_dim, int(d.get("vdim", dim)),
                   _positive_int(d, "q_rank", where), _positive_int(d, "kv_rank", where), float(_need(d, "scale", where)),
                   RokaraxRotary.from_dict(_need(d, "rot", where), rot_dim, where + ".rot"), _window(d, where))

    def to_dict(self) -> dict:
        d: dict[str, Any] = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                             "q_rank": self.q_rank, "kv_rank": self.kv_rank, "scale": self.scale, "rot": self.rot.to_dict()}
        if self.window is not None:
            d["mask"] = {"size": self.window}
        return d


@dataclass(frozen=True)
class RokaraxStateSpace:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "RokaraxStateSpace":
        m = cls(*(_positive_int(d, k, where) for k in ("heads", "vdim", "state", "groups", "conv", "norm_groups")))
        if m.heads % m.groups:
            raise ConfigError(f"{where}: heads={m.heads} is not a multiple of groups={m.groups}")
        if (m.heads * m.vdim) % m.norm_groups:
            raise ConfigError(f"{where}: heads * vdim = {m.heads * m.vdim} is not a multiple of norm_groups={m.norm_groups}")
        return m

    def to_dict(self) -> dict:
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups, "conv": self.conv,
                "norm_groups": self.norm_groups}


_MIXERS = {"attention": RokaraxAttention, "latent_attention": RokaraxLatentAttention, "mamba2": RokaraxStateSpace}


@dataclass(frozen=True)
class RokaraxLayer:
    type: str
    mixer: Any
    ff: int | None                      # inner size of the dense feed-forward, None for none


@dataclass(frozen=True)
class RokaraxConfig(ModelConfig):
    norm_eps: float = 1e-5
    embedding_scale: float = 1.0
    layers: tuple = ()
    extra: dict = field(default_factory=dict, compare=False, hash=False)

    @classmethod
    def from_hf_dict(cls, cfg: dict[str, Any], architecture: str = "Rokarax") -> "RokaraxConfig":
        vocab, width = _positive_int(cfg, "vocab", "the top level"), _positive_int(cfg, "width", "the top level")
        eps = float(_need(_need(cfg, "norm", "the top level"), "eps", "norm"))
        if not (eps > 0 and math.isfinite(eps)):
            raise ConfigError(f"norm.eps must be positive, got {eps}")
        scale = float((cfg.get("embedding") or {}).get("scale", 1.0))
        raw = _need(cfg, "layers", "the top level")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, lay in enumerate(raw):
            where = f"layers[{i}]"
            kind = _need(lay, "type", where)
            if kind not in _MIXERS:
                raise ConfigError(f"{where}: type={kind!r} is not implemented ({', '.join(MIXER_TYPES)} only)")
            mixer = _MIXERS[kind].from_dict(_need(lay, "mixer", where), where + ".mixer")
            mlp, ff = lay.get("mlp"), None
            if mlp is not None:
                if _need(mlp, "kind", where + ".mlp") != "dense":
                    raise ConfigError(f"{where}.mlp: kind={mlp['kind']!r} is not implemented (dense only)")
                ff = _positive_int(mlp, "ff", where + ".mlp")
            layers.append(RokaraxLayer(kind, mixer, ff))
        for i, lay in enumerate(layers):
            src = getattr(lay.mixer, "kv_from", None)
            if src is None:
                continue
            where = f"layers[{i}].mixer"
            if not 0 <= src < i or layers[src].type != "attention" or layers[src].mixer.kv_from is not None:
                raise ConfigError(f"{where}: kv_from={src} must name an earlier attention layer with keys and values of its own")
            own, other = lay.mixer, layers[src].mixer
            if (own.kv_heads, own.dim, own.vdim) != (other.kv_heads, other.dim, other.vdim):
                raise ConfigError(f"{where}: kv_from={src}, but that layer's kv heads and head sizes differ")
        return cls(architecture=architecture, vocab_size=vocab, hidden_size=width, num_hidden_layers=len(layers),
                   max_position_embeddings=int(cfg.get("max_positions", 1 << 20)),
                   torch_dtype=str(cfg.get("torch_dtype") or cfg.get("dtype") or "bfloat16"),
                   norm_eps=eps, embedding_scale=scale, layers=tuple(layers))

    def to_hf_dict(self) -> dict:
        return {
            "architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
            "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
            "layers": [{"type": lay.type, "mixer": lay.mixer.to_dict(),
                        "mlp": {"kind": "dense", "ff": lay.ff} if lay.ff is not None else None} for lay in self.layers],
            "torch_dtype": self.torch_dtype,
        }

    def kept_window(self, i: int) -> int | None:
        """What the cache of attention layer i has to keep: the largest window among the layer and the layers
        that read its keys and values; None (everything) if one of them has no window."""
        readers = [lay.mixer for j, lay in enumerate(self.layers)
                   if lay.type == "attention" and (j == i or lay.mixer.kv_from == i)]
        if any(m.window is None for m in readers):
            return None
        return max(m.window for m in readers)

    @property
    def num_parameters(self) -> int:
        """Counted from the tensors the model expects (a bias table with the rows random weights are drawn with)."""
        from ..models.causal_lm import build_model
        from ..models.rokarax import rokarax_spec

        total = 0
        for spec in build_model(rokarax_spec(self)).tensor_specs().values():
            n = 1
            for e in spec.draw_shape or spec.shape:
                n *= e
            total += n
        return total
