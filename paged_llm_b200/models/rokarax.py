"""The Rokarax decoder as data: `RokaraxConfig` -> `ModelSpec`.

Tensor names: `embed`, `head`, `final.norm{,.b,.alpha}`, and per layer i the four norms `l<i>.norm1`, `norm1b`,
`norm2`, `norm2b` (each with `.b` and `.alpha`), the mixer under `l<i>.mix.` and the feed-forward
`l<i>.mlp.{gate,up,down}`.  Matrices are stored [out, in].

Every layer is a block with a dynamic-tanh norm in front of and behind each part.  The mixer is one of: grouped-query
attention with a norm over the whole q and k projections, a learned bias by distance, a window and an output gate
(`mix.{q,k,v,g,o}`, `q.norm`, `k.norm`, `rel`), optionally reading an earlier layer's keys and values; attention through
latents with a rotated part (`mix.{dq,uq,dkv,uk,uv,o}`, `dq.norm`, `dkv.norm`); a state-space mixer (`mix.{in,conv,
conv.b,dt_bias,A_log,D,norm,o}`).  The feed-forward is SiLU-gated.  The embedding's rows are scaled; the head has a
matrix of its own.
"""

from __future__ import annotations

from ..config.rokarax import RokaraxConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _dyt(name: str, width: int) -> PartSpec:
    return PartSpec("dynamic_tanh", dict(dim=width), {"weight": name, "bias": name + ".b", "alpha": name + ".alpha"})


def rokarax_spec(cfg: RokaraxConfig) -> ModelSpec:
    w, eps = cfg.hidden_size, cfg.norm_eps
    positions: dict[str, PartSpec] = {}
    layers, schedule = [], []
    for i, lay in enumerate(cfg.layers):
        p, m = f"l{i}.", lay.mixer
        cache_from = None
        if lay.type == "attention":
            shares = m.kv_from is not None
            owner = m.kv_from if shares else i
            names = {"q_proj": p + "mix.q", "q_norm": p + "mix.q.norm", "rel": p + "mix.rel", "g_proj": p + "mix.g",
                     "o_proj": p + "mix.o"}
            if shares:
                cache_from = m.kv_from
            else:
                names.update(k_proj=p + "mix.k", v_proj=p + "mix.v", k_norm=p + "mix.k.norm")
            mixer = PartSpec("gated_attention", dict(
                hidden_size=w, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim, scale=m.scale,
                eps=eps, window=m.window, keep_window=cfg.kept_window(owner), distance_bias=True, bias_far=m.bias_max,
                bias_rows=m.bias_rows, gate=True, shares_cache=shares), names)
        elif lay.type == "latent_attention":
            scaling = dict(m.rot.scaling, type="yarn") if m.rot.scaling else None
            rotary = PartSpec("rotary", dict(head_dim=m.rot_dim, theta=m.rot.base, pairing="interleaved",
                                             rotary_dim=m.rot.dims, scaling=scaling))
            position = next((name for name, ps in positions.items() if ps.params == rotary.params), None)
            if position is None:                         # layers with the same rotation share one table
                position = f"rotary{len(positions)}"
                positions[position] = rotary
            mixer = PartSpec("latent_attention", dict(
                hidden_size=w, num_heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim, value_dim=m.vdim, q_rank=m.q_rank,
                kv_rank=m.kv_rank, scale=m.scale, eps=eps, window=m.window, position=position),
                {"dq": p + "mix.dq", "dq_norm": p + "mix.dq.norm", "uq": p + "mix.uq", "dkv": p + "mix.dkv",
                 "dkv_norm": p + "mix.dkv.norm", "uk": p + "mix.uk", "uv": p + "mix.uv", "o_proj": p + "mix.o"})
        else:
            mixer = PartSpec("state_space", dict(
                hidden_size=w, num_heads=m.heads, head_dim=m.vdim, state_size=m.state, groups=m.groups, conv_taps=m.conv,
                norm_groups=m.norm_groups, eps=eps),
                {"in_proj": p + "mix.in", "conv": p + "mix.conv", "conv_bias": p + "mix.conv.b", "dt_bias": p + "mix.dt_bias",
                 "a_log": p + "mix.A_log", "d_skip": p + "mix.D", "norm": p + "mix.norm", "o_proj": p + "mix.o"})
        norms = {"input": _dyt(p + "norm1", w), "behind_mixer": _dyt(p + "norm1b", w)}
        ffn = None
        if lay.ff is not None:
            norms["post_mixer"] = _dyt(p + "norm2", w)
            norms["behind_ffn"] = _dyt(p + "norm2b", w)
            ffn = PartSpec("gated_mlp", dict(hidden_size=w, intermediate_size=lay.ff, activation="silu"),
                           {"gate_proj": p + "mlp.gate", "up_proj": p + "mlp.up", "down_proj": p + "mlp.down"})
        layers.append(LayerSpec("sandwich_norm", mixer, ffn, norms))
        schedule.append(ScheduleEntry(i, cache_from=cache_from))
    return ModelSpec(
        hidden_size=w,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("embedding", dict(vocab_size=cfg.vocab_size, hidden_size=w, scale=cfg.embedding_scale),
                           {"weight": "embed"}),
        layers=layers,
        schedule=schedule,
        final_norm=_dyt("final.norm", w),
        head=PartSpec("lm_head", dict(vocab_size=cfg.vocab_size, hidden_size=w), {"weight": "head"}),
        positions=positions,
    )
