"""The Pomisun decoder as data: `PomisunConfig` -> `ModelSpec`.

Tensor names: `embed`, `final.norm`, and per layer i `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.{q,k,o}`,
and the feed-forward under `l<i>.mlp.`: `gate`, `up`, `down` (dense) or `router`, `e<j>.{gate,up,down}`,
`shared.{gate,up,down,sg}` (routed experts).  Matrices are stored [out, in].

Every layer is a pre-norm block whose norms store their weight around zero.  The mixer is grouped-query
attention without a value projection (the values are the keys before rotation), rotary positions with
YaRN scaling on the first dims of each head, a cap on the scores, and a chunked mask.  The feed-forward is
gated with the tanh form of GELU, or routed experts gated with SiLU plus a shared expert behind a sigmoid
gate.  A span of layers may run several times in a row with the same weights; each run has a cache of its
own, and every pass but the first starts by adding the embedding's output to the stream again.  The head
is the embedding table.
"""

from __future__ import annotations

from ..config.pomisun import PomisunConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def pomisun_spec(cfg: PomisunConfig) -> ModelSpec:
    w, eps = cfg.hidden_size, cfg.norm_eps
    positions: dict[str, PartSpec] = {}
    layers = []
    for i, lay in enumerate(cfg.layers):
        p, m = f"l{i}.", lay.mixer
        position = None
        if m.rot is not None:
            scaling = dict(m.rot.scaling, type="yarn") if m.rot.scaling else None
            rotary = PartSpec("rotary", dict(head_dim=m.dim, theta=m.rot.base, pairing="half", rotary_dim=m.rot.dims,
                                             scaling=scaling))
            # layers with the same rotation share one table
            position = next((name for name, ps in positions.items() if ps.params == rotary.params), None)
            if position is None:
                position = f"rotary{len(positions)}"
                positions[position] = rotary
        mixer = PartSpec(
            "paged_attention",
            dict(hidden_size=w, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, scale=m.scale, window=None,
                 position=position, score_cap=m.softcap, chunk=m.chunk, value_from_key=True),
            {"q_proj": p + "mix.q", "k_proj": p + "mix.k", "o_proj": p + "mix.o"},
        )
        norms = {"input": PartSpec("rms_norm", dict(dim=w, eps=eps, unit_offset=True), {"weight": p + "norm1"})}
        ffn = None
        if lay.mlp is not None:
            norms["post_mixer"] = PartSpec("rms_norm", dict(dim=w, eps=eps, unit_offset=True), {"weight": p + "norm2"})
            if lay.mlp.kind == "dense":
                ffn = PartSpec("gated_mlp", dict(hidden_size=w, intermediate_size=lay.mlp.ff, activation="gelu_tanh"),
                               {"gate_proj": p + "mlp.gate", "up_proj": p + "mlp.up", "down_proj": p + "mlp.down"})
            else:
                names = {"router": p + "mlp.router"}
                for e in range(lay.mlp.experts):
                    for x in ("gate", "up", "down"):
                        names[f"e{e}.{x}"] = f"{p}mlp.e{e}.{x}"
                if lay.mlp.shared_ff is not None:
                    for x in ("gate", "up", "down", "sg"):
                        names[f"shared.{x}"] = f"{p}mlp.shared.{x}"
                ffn = PartSpec("routed_mlp", dict(hidden_size=w, expert_size=lay.mlp.ff, num_experts=lay.mlp.experts,
                                                  top_k=lay.mlp.top, activation="silu", shared_size=lay.mlp.shared_ff),
                               names)
        layers.append(LayerSpec("pre_norm", mixer, ffn, norms))
    return ModelSpec(
        hidden_size=w,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("embedding", dict(vocab_size=cfg.vocab_size, hidden_size=w), {"weight": "embed"}),
        layers=layers,
        schedule=[ScheduleEntry(i, add_embedding=again) for i, again in cfg.layer_runs()],
        final_norm=PartSpec("rms_norm", dict(dim=w, eps=eps, unit_offset=True), {"weight": "final.norm"}),
        head=PartSpec("lm_head", dict(vocab_size=cfg.vocab_size, hidden_size=w, tied_to="embed"), {"weight": "head"}),
        positions=positions,
    )
