"""Silutar as a ModelSpec.  Token table plus a table of learned position vectors; pre-norm layers
whose norm is Dynamic Tanh (tensors `<name>`, `<name>.b`, `<name>.alpha`); per layer one of three
mixers - `gla`, `channel_delta`, or `parallel` = left_scale * chunk attention + right_scale *
generalised delta rule - and a dense gated feed-forward or none; the token table is the output
matrix and the logits are soft-capped.  Layer i's tensors start with `l<i>.`.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.silutar import SilutarConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec


def _norm(width: int, name: str) -> PartSpec:
    return PartSpec("dyt", {"width": width, "weight_name": "", "bias_name": ".b", "alpha_name": ".alpha"}, name)


def _mixer(cfg: SilutarConfig, kind: str, m, prefix: str) -> PartSpec:
    h, eps = cfg.width, cfg.norm_eps
    if kind == "gla":
        return PartSpec("gla", {"hidden": h, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"], "tau": m["tau"],
                                "decay_rank": m["decay_rank"], "eps": eps}, prefix)
    if kind == "channel_delta":
        return PartSpec("channel_delta", {"hidden": h, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"],
                                          "vdim": m["vdim"], "conv": m["conv"], "decay_rank": m["decay_rank"],
                                          "gate_rank": m["gate_rank"], "eps": eps}, prefix)
    left, right = m["left"], m["right"]
    return PartSpec("parallel", {"branches": (
        {"name": "left", "kind": "chunk_attention", "scale": m["left_scale"],
         "params": {"hidden": h, "heads": left["heads"], "kv_heads": left["kv_heads"], "dim": left["dim"], "vdim": left["vdim"],
                    "conv": left["conv"], "chunk": left["mask"]["size"], "scale": left["scale"], "eps": eps}},
        {"name": "right", "kind": "general_delta", "scale": m["right_scale"],
         "params": {"hidden": h, "heads": right["heads"], "dim": right["dim"], "decay_rank": right["decay_rank"], "eps": eps}},
    )}, prefix)


def build_spec(cfg: SilutarConfig) -> ModelSpec:
    h = cfg.width
    layers = []
    ignorable = []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        roles = dict(mixer_norm=_norm(h, p + "norm1"), mixer=_mixer(cfg, l.type, l.mixer, p + "mix."))
        if l.ff is not None:
            roles.update(ffn_norm=_norm(h, p + "norm2"),
                         ffn=PartSpec("swiglu", {"hidden": h, "intermediate": l.ff, "names": ("gate", "up", "down")}, p + "mlp."))
            layers.append(LayerSpec(f"l{i}", block="prenorm", **roles))
        else:
            layers.append(LayerSpec(f"l{i}", block="prenorm_mixer", **roles))
            ignorable += [p + "norm2", p + "norm2.b", p + "norm2.alpha"]      # a norm nobody reads
    return ModelSpec(
        hidden_size=h, vocab_size=cfg.vocab,
        embedding=PartSpec("embedding", {"vocab": cfg.vocab, "hidden": h, "positions": cfg.max_positions,
                                         "table_name": "embed", "positions_name": "pos"}, ""),
        layers=tuple(layers),
        final_norm=_norm(h, "final.norm"),
        lm_head=PartSpec("linear", {"vocab": cfg.vocab, "hidden": h, "tied": True, "softcap": cfg.logit_softcap}, "head."),
        ignorable_tensors=tuple(ignorable))


def register() -> None:
    register_architecture("Silutar", SilutarConfig, build_spec, aliases=("silutar",))
