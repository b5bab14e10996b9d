"""Typed configuration of the Damadra architecture: a decoder whose layers are listed one by one in
config.json, each with one of two attention mixers and a dense or mixture-of-experts feed-forward (or none).

    {"architecture": "Damadra", "vocab": V, "width": h, "embedding": {"scale": s}, "norm": {"eps": e},
     "residual_mult": m,
     "layers": [{"type": "attention" | "attention_2",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "bias_max",
                           "mask": {"size"}                       (attention: the sliding window)
                           "q_temp": {"coef", "every"}, "kv_from": j   (attention_2, both optional)},
                 "mlp": null | {"kind": "dense", "ff": F}
                             | {"kind": "moe", "expert": {"ff": F}, "router": {"experts", "identity", "top"}}}, ...]}

The number of rows of a layer's distance-bias table is not in config.json: it is read off the shape of the
checkpoint's tensor `l<i>.mix.rel` (`from_dict(raw, shapes)`); a configuration made for random weights states it
as `bias_rows`, which `to_dict()` writes and `from_dict` prefers over the shapes.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .errors import InvalidValue, MissingKey

MIXER_TYPES = ("attention", "attention_2")


def _pos_int(d: Mapping[str, Any], key: str, where: str) -> int:
    v = d.get(key)
    if v is None:
        raise MissingKey(f"{where}.{key}")
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise InvalidValue(f"{where}.{key}", f"expected a positive integer, got {v!r}")
    return int(v)


def _number(d: Mapping[str, Any], key: str, where: str) -> float:
    v = d.get(key)
    if v is None:
        raise MissingKey(f"{where}.{key}")
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v):
        raise InvalidValue(f"{where}.{key}", f"expected a finite number, got {v!r}")
    return float(v)


def _section(d: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = d.get(key)
    if not isinstance(v, Mapping):
        raise MissingKey(f"{where}.{key}")
    return v


@dataclass(frozen=True)
class DamadraLayer:
    type: str
    mixer: Any                       # a plain dict of validated sizes and constants, `bias_rows` included
    mlp: Any                         # None, {"kind": "dense", "ff"} or {"kind": "moe", "ff", "experts", "identity", "top"}


@dataclass(frozen=True)
class DamadraConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    residual_mult: float
    layers: Tuple[DamadraLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Damadra"

    default_eos_ids = ()
    reads_tensor_shapes = True       # load_config hands from_dict the checkpoint's tensor shapes

    # names the serving code asks of any configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], shapes: Optional[Mapping[str, Tuple[int, ...]]] = None) -> "DamadraConfig":
        vocab, width = _pos_int(d, "vocab", "config"), _pos_int(d, "width", "config")
        scale = _number(_section(d, "embedding", "config"), "scale", "embedding")
        eps = _number(_section(d, "norm", "config"), "eps", "norm")
        if eps < 0:
            raise InvalidValue("norm.eps", "must be >= 0")
        mult = _number(d, "residual_mult", "config")
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise MissingKey("layers")
        layers = []
        for i, rl in enumerate(raw_layers):
            where = f"layers[{i}]"
            if not isinstance(rl, Mapping) or rl.get("type") not in MIXER_TYPES:
                raise InvalidValue(where + ".type", f"expected one of {MIXER_TYPES}, got {rl.get('type') if isinstance(rl, Mapping) else rl!r}")
            mixer = _parse_mixer(rl["type"], _section(rl, "mixer", where), shapes, f"l{i}.mix.", where + ".mixer")
            layers.append(DamadraLayer(rl["type"], mixer, _parse_mlp(rl.get("mlp"), where + ".mlp")))
        for i, l in enumerate(layers):
            src = l.mixer.get("kv_from")
            if src is None:
                continue
            where = f"layers[{i}].mixer.kv_from"
            if not 0 <= src < i:
                raise InvalidValue(where, f"layer {i} can read the keys and values of an earlier layer only, got {src}")
            s = layers[src]
            if s.type != l.type or s.mixer.get("kv_from") is not None:
                raise InvalidValue(where, f"layer {src} is no layer of type {l.type} with keys and values of its own")
            for k in ("heads", "kv_heads", "dim", "vdim", "window"):
                if s.mixer.get(k) != l.mixer.get(k):
                    raise InvalidValue(where, f"layers {src} and {i} differ in '{k}'")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else ((int(eos),) if isinstance(eos, int) else tuple(int(e) for e in eos))
        return cls(vocab=vocab, width=width, embedding_scale=scale, norm_eps=eps, residual_mult=mult, layers=tuple(layers),
                   eos_token_ids=eos_ids)

    def to_dict(self) -> dict:
        layers = []
        for l in self.layers:
            m = l.mixer
            mixer: Dict[str, Any] = {k: m[k] for k in ("heads", "kv_heads", "dim", "vdim", "scale", "bias_max", "bias_rows")}
            if m.get("window") is not None:
                mixer["mask"] = {"size": m["window"]}
            if m.get("q_temp") is not None:
                mixer["q_temp"] = {"coef": m["q_temp"][0], "every": m["q_temp"][1]}
            if m.get("kv_from") is not None:
                mixer["kv_from"] = m["kv_from"]
            mlp = l.mlp
            if mlp is not None and mlp["kind"] == "moe":
                mlp = {"kind": "moe", "expert": {"ff": mlp["ff"]},
                       "router": {"experts": mlp["experts"], "identity": mlp["identity"], "top": mlp["top"]}}
            elif mlp is not None:
                mlp = {"kind": "dense", "ff": mlp["ff"]}
            layers.append({"type": l.type, "mixer": mixer, "mlp": mlp})
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
                               "residual_mult": self.residual_mult, "layers": layers}
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out


def _parse_mixer(kind: str, m: Mapping[str, Any], shapes, prefix: str, where: str) -> dict:
    heads, kv = _pos_int(m, "heads", where), _pos_int(m, "kv_heads", where)
    if heads % kv:
        raise InvalidValue(where + ".kv_heads", f"{heads} query heads are no multiple of {kv} key/value heads")
    out: Dict[str, Any] = {"heads": heads, "kv_heads": kv, "dim": _pos_int(m, "dim", where), "vdim": _pos_int(m, "vdim", where),
                           "scale": _number(m, "scale", where), "bias_max": _pos_int(m, "bias_max", where)}
    if m.get("bias_rows") is not None:
        out["bias_rows"] = _pos_int(m, "bias_rows", where)
    elif shapes is not None and prefix + "rel" in shapes and len(shapes[prefix + "rel"]) == 2:
        out["bias_rows"] = int(shapes[prefix + "rel"][0])
    else:
        raise MissingKey(f"{where}.bias_rows (neither stated nor readable from the shape of {prefix}rel)")
    if out["bias_rows"] < 2 or out["bias_max"] <= out["bias_rows"] // 2:
        raise InvalidValue(where + ".bias_max", f"a table of {out['bias_rows']} rows needs a greatest distance beyond "
                                                f"{out['bias_rows'] // 2}, got {out['bias_max']}")
    out["window"] = out["q_temp"] = out["kv_from"] = None
    if kind == "attention":
        out["window"] = _pos_int(_section(m, "mask", where), "size", where + ".mask")
        if out["vdim"] != out["dim"]:
            raise InvalidValue(where + ".vdim", "the values of this mixer are its keys and have their size")
    else:
        qt = m.get("q_temp")
        if qt is not None:
            if not isinstance(qt, Mapping):
                raise InvalidValue(where + ".q_temp", f"expected an object, got {qt!r}")
            out["q_temp"] = (_number(qt, "coef", where + ".q_temp"), _pos_int(qt, "every", where + ".q_temp"))
    src = m.get("kv_from")
    if src is not None:
        if isinstance(src, bool) or not isinstance(src, int):
            raise InvalidValue(where + ".kv_from", f"expected a layer's number, got {src!r}")
        out["kv_from"] = int(src)
    return out


def _parse_mlp(mlp, where: str):
    if mlp is None:
        return None
    if not isinstance(mlp, Mapping) or mlp.get("kind") not in ("dense", "moe"):
        raise InvalidValue(where + ".kind", f"expected 'dense' or 'moe', got {mlp!r}")
    if mlp["kind"] == "dense":
        return {"kind": "dense", "ff": _pos_int(mlp, "ff", where)}
    r = _section(mlp, "router", where)
    experts, top = _pos_int(r, "experts", where + ".router"), _pos_int(r, "top", where + ".router")
    identity = r.get("identity") or 0
    if isinstance(identity, bool) or not isinstance(identity, int) or identity < 0:
        raise InvalidValue(where + ".router.identity", f"expected a count, got {identity!r}")
    if top > experts + identity:
        raise InvalidValue(where + ".router.top", f"{top} of {experts + identity} experts")
    return {"kind": "moe", "ff": _pos_int(_section(mlp, "expert", where), "ff", where + ".expert"), "experts": experts,
            "identity": int(identity), "top": top}
