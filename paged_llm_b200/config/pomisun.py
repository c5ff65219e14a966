"""Typed configuration of the Pomisun decoder, read from a checkpoint's config.json.

config.json gives every size and every constant that may differ between models of the design:

    architecture  "Pomisun"
    vocab, width  vocabulary and width of the residual stream
    norm.eps      epsilon of every RMS norm
    layers        one entry per layer: `type` (the mixer, "attention"), `mixer` (its sizes and
                  constants) and `mlp` (the feed-forward, or null for none)
    loop          optional: layers start .. stop-1 run `times` times in a row with the same weights

A mixer of type "attention": heads, kv_heads, dim (size of a query/key head), vdim (size of a
value head: the values are the keys, so it equals dim), scale, softcap (optional), mask.size
(optional: the chunk of the mask), rot (optional: dims, base, scaling{factor, original, fast, slow}).
A feed-forward: kind "dense" with ff, or kind "moe" with expert.ff, router.experts, router.top and an
optional shared.ff.

What the engine does not compute is refused here with a message, never computed wrongly.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any

from .model import ConfigError, ModelConfig


def _need(d: dict, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json: {where} lacks the key {key!r}")
    return d[key]


@dataclass(frozen=True)
class PomisunRotary:
    dims: int
    base: float
    scaling: dict | None = None          # factor, original, fast, slow

    @classmethod
    def from_dict(cls, d: dict, head_dim: int, where: str) -> "PomisunRotary":
        dims, base = int(_need(d, "dims", where)), float(_need(d, "base", where))
        if dims <= 0 or dims % 2 or dims > head_dim:
            raise ConfigError(f"{where}: dims={dims} must be even and at most the head size {head_dim}")
        if not base > 0:
            raise ConfigError(f"{where}: base={base} must be positive")
        sc = d.get("scaling")
        if sc is not None:
            sc = {k: float(_need(sc, k, where + ".scaling")) for k in ("factor", "original", "fast", "slow")}
            if not (sc["factor"] > 0 and sc["original"] > 0 and sc["fast"] > 0 and sc["slow"] > 0):
                raise ConfigError(f"{where}.scaling: factor, original, fast and slow must be positive")
        return cls(dims, base, sc)

    def to_dict(self) -> dict:
        d: dict[str, Any] = {"dims": self.dims, "base": self.base}
        if self.scaling is not None:
            d["scaling"] = dict(self.scaling)
        return d


@dataclass(frozen=True)
class PomisunAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float | None = None
    chunk: int | None = None
    rot: PomisunRotary | None = None

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "PomisunAttention":
        heads, kv = int(_need(d, "heads", where)), int(_need(d, "kv_heads", where))
        dim = int(_need(d, "dim", where))
        vdim = int(d.get("vdim", dim))
        if heads < 1 or kv < 1 or heads % kv:
            raise ConfigError(f"{where}: heads={heads} is not a multiple of kv_heads={kv}")
        if dim < 1:
            raise ConfigError(f"{where}: dim={dim}")
        if vdim != dim:
            raise ConfigError(f"{where}: vdim={vdim} differs from dim={dim}, but the values are the keys")
        scale = float(_need(d, "scale", where))
        cap = d.get("softcap")
        if cap is not None and not float(cap) > 0:
            raise ConfigError(f"{where}: softcap={cap} must be positive")
        mask = d.get("mask") or {}
        chunk = mask.get("size")
        if chunk is not None and int(chunk) < 1:
            raise ConfigError(f"{where}: mask.size={chunk} must be positive")
        rot = d.get("rot")
        return cls(heads, kv, dim, vdim, scale, float(cap) if cap is not None else None,
                   int(chunk) if chunk is not None else None,
                   PomisunRotary.from_dict(rot, dim, where + ".rot") if rot is not None else None)

    def to_dict(self) -> dict:
        d: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                             "scale": self.scale}
        if self.softcap is not None:
            d["softcap"] = self.softcap
        if self.chunk is not None:
            d["mask"] = {"size": self.chunk}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass(frozen=True)
class PomisunMLP:
    kind: str                           # "dense" | "moe"
    ff: int                             # dense: the inner size; moe: an expert's
    experts: int = 0
    top: int = 0
    shared_ff: int | None = None

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "PomisunMLP":
        kind = _need(d, "kind", where)
        if kind == "dense":
            ff = int(_need(d, "ff", where))
            if ff < 1:
                raise ConfigError(f"{where}: ff={ff}")
            return cls("dense", ff)
        if kind == "moe":
            ff = int(_need(_need(d, "expert", where), "ff", where + ".expert"))
            router = _need(d, "router", where)
            experts, top = int(_need(router, "experts", where + ".router")), int(_need(router, "top", where + ".router"))
            if ff < 1 or experts < 1 or not 1 <= top <= experts:
                raise ConfigError(f"{where}: expert.ff={ff}, router.experts={experts}, router.top={top}")
            shared = d.get("shared")
            shared_ff = int(_need(shared, "ff", where + ".shared")) if shared is not None else None
            if shared_ff is not None and shared_ff < 1:
                raise ConfigError(f"{where}: shared.ff={shared_ff}")
            return cls("moe", ff, experts, top, shared_ff)
        raise ConfigError(f"{where}: kind={kind!r} is not implemented (dense and moe only)")

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        d: dict[str, Any] = {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff is not None:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass(frozen=True)
class PomisunLayer:
    type: str
    mixer: PomisunAttention
    mlp: PomisunMLP | None


@dataclass(frozen=True)
class PomisunLoop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class PomisunConfig(ModelConfig):
    norm_eps: float = 1e-6
    layers: tuple = ()
    loop: PomisunLoop | None = None
    extra: dict = field(default_factory=dict, compare=False, hash=False)

    @classmethod
    def from_hf_dict(cls, cfg: dict[str, Any], architecture: str = "Pomisun") -> "PomisunConfig":
        vocab, width = int(_need(cfg, "vocab", "the top level")), int(_need(cfg, "width", "the top level"))
        eps = float(_need(_need(cfg, "norm", "the top level"), "eps", "norm"))
        raw_layers = _need(cfg, "layers", "the top level")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, lay in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = _need(lay, "type", where)
            if kind != "attention":
                raise ConfigError(f"{where}: type={kind!r} is not implemented (attention only)")
            mixer = PomisunAttention.from_dict(_need(lay, "mixer", where), where + ".mixer")
            mlp = lay.get("mlp")
            layers.append(PomisunLayer(kind, mixer, PomisunMLP.from_dict(mlp, where + ".mlp") if mlp is not None else None))
        loop = cfg.get("loop")
        if loop is not None:
            loop = PomisunLoop(int(_need(loop, "start", "loop")), int(_need(loop, "stop", "loop")),
                               int(_need(loop, "times", "loop")))
            if not (0 <= loop.start < loop.stop <= len(layers)) or loop.times < 1:
                raise ConfigError(f"loop start={loop.start} stop={loop.stop} times={loop.times} does not fit "
                                  f"{len(layers)} layers")
        if vocab < 1 or width < 1:
            raise ConfigError(f"vocab={vocab}, width={width} must be positive")
        if not (eps > 0 and math.isfinite(eps)):
            raise ConfigError(f"norm.eps must be positive, got {eps}")
        return cls(architecture=architecture, vocab_size=vocab, hidden_size=width, num_hidden_layers=len(layers),
                   max_position_embeddings=int(cfg.get("max_positions", 1 << 20)),
                   torch_dtype=str(cfg.get("torch_dtype") or cfg.get("dtype") or "bfloat16"),
                   norm_eps=eps, layers=tuple(layers), loop=loop)

    def to_hf_dict(self) -> dict:
        d: dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
            "norm": {"eps": self.norm_eps},
            "layers": [{"type": lay.type, "mixer": lay.mixer.to_dict(), "mlp": lay.mlp.to_dict() if lay.mlp else None}
                       for lay in self.layers],
            "torch_dtype": self.torch_dtype,
        }
        if self.loop is not None:
            d["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        return d

    def layer_runs(self) -> list[tuple[int, bool]]:
        """(layer, whether the embedding's output is added in front of it) in the order the layers run: the
        looped span runs `times` times in a row, and every pass but the first begins with that sum."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        a, b, times = self.loop.start, self.loop.stop, self.loop.times
        runs = [(i, False) for i in range(a)]
        for t in range(times):
            runs += [(i, t > 0 and i == a) for i in range(a, b)]
        return runs + [(i, False) for i in range(b, n)]

    @property
    def num_parameters(self) -> int:
        w = self.hidden_size
        total = self.vocab_size * w + w
        for lay in self.layers:
            m = lay.mixer
            total += w + (m.heads + m.kv_heads) * m.dim * w + m.heads * m.vdim * w
            if lay.mlp is None:
                continue
            total += w
            if lay.mlp.kind == "dense":
                total += 3 * lay.mlp.ff * w
            else:
                total += lay.mlp.experts * (3 * lay.mlp.ff * w + w)
                if lay.mlp.shared_ff is not None:
                    total += 3 * lay.mlp.shared_ff * w + w
        return total
