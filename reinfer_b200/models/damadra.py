"""Damadra as a ModelSpec.  Scaled token embedding; layers whose sublayers read the residual stream itself and
whose RMS norms sit on the sublayers' outputs (block `out_norm`, norm `rms_out` with the residual multiplier);
per layer one of two mixers, both the part `biased_attention` - `attention`: sliding window, q/k norm over the
whole projection, the values are the keys as projected; `attention_2`: causal, q/k norm per head, warmed-up
queries, values of their own, optionally the keys and values of an earlier layer - and a dense gated
feed-forward, a mixture of experts, or none; a final RMS norm and an output matrix of its own.  Layer i's tensors
start with `l<i>.`.
"""
from __future__ import annotations

from ..config.damadra import DamadraConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec


def _mixer(cfg: DamadraConfig, kind: str, m, prefix: str) -> PartSpec:
    params = {"hidden": cfg.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
              "scale": m["scale"], "eps": cfg.norm_eps, "bias_rows": m["bias_rows"], "bias_max": m["bias_max"],
              "own_kv": m["kv_from"] is None}
    if kind == "attention":
        params.update(window=m["window"], qk_norm="whole", values="keys")
    else:
        params.update(qk_norm="head", values="projection", q_temp=m["q_temp"])
    return PartSpec("biased_attention", params, prefix)


def _ffn(cfg: DamadraConfig, mlp, prefix: str) -> PartSpec:
    if mlp["kind"] == "dense":
        return PartSpec("swiglu", {"hidden": cfg.width, "intermediate": mlp["ff"], "names": ("gate", "up", "down")}, prefix)
    return PartSpec("expert_mixture", {"hidden": cfg.width, "experts": mlp["experts"], "identity": mlp["identity"],
                                       "top": mlp["top"], "inner": mlp["ff"]}, prefix)


def build_spec(cfg: DamadraConfig) -> ModelSpec:
    h = cfg.width

    def norm(name: str) -> PartSpec:
        return PartSpec("rms_out", {"width": h, "eps": cfg.norm_eps, "mult": cfg.residual_mult, "weight_name": ""}, name)

    layers, ignorable = [], []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        roles = dict(mixer=_mixer(cfg, l.type, l.mixer, p + "mix."), mixer_norm=norm(p + "norm1"))
        if l.mlp is not None:
            roles.update(ffn=_ffn(cfg, l.mlp, p + "mlp."), ffn_norm=norm(p + "norm2"))
        else:
            ignorable.append(p + "norm2")                      # a norm nobody reads
        src = l.mixer["kv_from"]
        layers.append(LayerSpec(f"l{i}", block="out_norm", cache_from=None if src is None else f"l{src}", **roles))
    return ModelSpec(
        hidden_size=h, vocab_size=cfg.vocab,
        embedding=PartSpec("embedding", {"vocab": cfg.vocab, "hidden": h, "table_name": "embed", "scale": cfg.embedding_scale,
                                         "rounded_copy": True}, ""),
        layers=tuple(layers),
        final_norm=PartSpec("rmsnorm", {"width": h, "eps": cfg.norm_eps, "weight_name": ""}, "final.norm"),
        lm_head=PartSpec("linear", {"vocab": cfg.vocab, "hidden": h, "weight_name": ""}, "head"),
        ignorable_tensors=tuple(ignorable))


def register() -> None:
    register_architecture("Damadra", DamadraConfig, build_spec, aliases=("damadra",))
