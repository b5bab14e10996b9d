"""Typed configuration of the Silutar architecture: a decoder whose layers are listed one by one
in config.json, each with one of three mixers and an optional dense feed-forward.

    {"architecture": "Silutar", "vocab": V, "width": h, "max_positions": P, "norm": {"eps": e},
     "logit_softcap": c, "layers": [{"type": "gla" | "parallel" | "channel_delta",
                                     "mixer": {...sizes...}, "mlp": {"kind": "dense", "ff": F} | null}, ...]}

Sizes that config.json does not state - the inner widths of the low-rank maps behind the decays
and gates - are read off the shapes of the checkpoint's tensors (`from_dict(raw, shapes)`); a
configuration made for random weights states them itself under the optional keys `decay_rank`
and `gate_rank`, which `to_dict()` writes and `from_dict` prefers over the shapes.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .errors import InvalidValue, MissingKey

MIXER_TYPES = ("gla", "parallel", "channel_delta")


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


def _rank(m: Mapping[str, Any], key: str, shapes, tensor: str, where: str) -> int:
    """An inner width: the configuration's own key if it is there, else the first dimension of `tensor`."""
    if m.get(key) is not None:
        return _pos_int(m, key, where)
    if shapes is not None and tensor in shapes and len(shapes[tensor]) == 2:
        return int(shapes[tensor][0])
    raise MissingKey(f"{where}.{key} (neither stated nor readable from the shape of {tensor})")


@dataclass(frozen=True)
class SilutarLayer:
    type: str
    mixer: Any                       # a plain dict of validated sizes (nested for 'parallel'), ranks included
    ff: Optional[int]                # the dense feed-forward's inner width; None: the layer has none


@dataclass(frozen=True)
class SilutarConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    logit_softcap: float             # 0: none
    layers: Tuple[SilutarLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Silutar"

    default_eos_ids = ()
    reads_tensor_shapes = True       # load_config hands from_dict the checkpoint's tensor shapes

    # names the serving code asks of any configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def max_position_embeddings(self) -> int:
        return self.max_positions

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], shapes: Optional[Mapping[str, Tuple[int, ...]]] = None) -> "SilutarConfig":
        vocab, width = _pos_int(d, "vocab", "config"), _pos_int(d, "width", "config")
        max_pos = d.get("max_positions")
        if max_pos is None and shapes is not None and "pos" in shapes:
            max_pos = int(shapes["pos"][0])
        if isinstance(max_pos, bool) or not isinstance(max_pos, int) or max_pos <= 0:
            raise InvalidValue("max_positions", f"expected a positive integer, got {max_pos!r}")
        norm = d.get("norm")
        if not isinstance(norm, Mapping):
            raise MissingKey("norm")
        eps = _number(norm, "eps", "norm")
        if eps < 0:
            raise InvalidValue("norm.eps", "must be >= 0")
        cap = d.get("logit_softcap")
        cap = 0.0 if cap is None else _number(d, "logit_softcap", "config")
        if cap < 0:
            raise InvalidValue("logit_softcap", "must be positive (or absent)")
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise MissingKey("layers")
        layers = []
        for i, rl in enumerate(raw_layers):
            where = f"layers[{i}]"
            if not isinstance(rl, Mapping) or rl.get("type") not in MIXER_TYPES:
                raise InvalidValue(where + ".type", f"expected one of {MIXER_TYPES}, got {rl.get('type') if isinstance(rl, Mapping) else rl!r}")
            m = rl.get("mixer")
            if not isinstance(m, Mapping):
                raise MissingKey(where + ".mixer")
            mixer = _MIXER_PARSERS[rl["type"]](m, shapes, f"l{i}.mix.", where + ".mixer")
            mlp = rl.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
                    raise InvalidValue(where + ".mlp.kind", f"only 'dense' feed-forwards exist, got {mlp!r}")
                ff = _pos_int(mlp, "ff", where + ".mlp")
            layers.append(SilutarLayer(rl["type"], mixer, ff))
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else ((int(eos),) if isinstance(eos, int) else tuple(int(e) for e in eos))
        return cls(vocab=vocab, width=width, max_positions=int(max_pos), norm_eps=eps, logit_softcap=cap,
                   layers=tuple(layers), eos_token_ids=eos_ids)

    def to_dict(self) -> dict:
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "max_positions": self.max_positions, "norm": {"eps": self.norm_eps},
                               "layers": [{"type": l.type, "mixer": _plain(l.mixer),
                                           "mlp": None if l.ff is None else {"kind": "dense", "ff": l.ff}} for l in self.layers]}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out


def _plain(x):
    return {k: _plain(v) for k, v in x.items()} if isinstance(x, Mapping) else x


def _parse_gla(m, shapes, prefix, where):
    tau = _number(m, "tau", where)
    if tau <= 0:
        raise InvalidValue(where + ".tau", "must be positive")
    return {"heads": _pos_int(m, "heads", where), "dim": _pos_int(m, "dim", where), "vdim": _pos_int(m, "vdim", where),
            "tau": tau, "decay_rank": _rank(m, "decay_rank", shapes, prefix + "a1", where)}


def _parse_channel_delta(m, shapes, prefix, where):
    heads, kv = _pos_int(m, "heads", where), _pos_int(m, "kv_heads", where)
    if heads % kv:
        raise InvalidValue(where + ".kv_heads", f"{heads} heads are no multiple of {kv} key heads")
    return {"heads": heads, "kv_heads": kv, "dim": _pos_int(m, "dim", where), "vdim": _pos_int(m, "vdim", where),
            "conv": _pos_int(m, "conv", where), "decay_rank": _rank(m, "decay_rank", shapes, prefix + "a1", where),
            "gate_rank": _rank(m, "gate_rank", shapes, prefix + "g1", where)}


def _parse_parallel(m, shapes, prefix, where):
    left, right = m.get("left"), m.get("right")
    if not isinstance(left, Mapping) or not isinstance(right, Mapping):
        raise MissingKey(where + ".left / .right")
    heads, kv = _pos_int(left, "heads", where + ".left"), _pos_int(left, "kv_heads", where + ".left")
    if heads % kv:
        raise InvalidValue(where + ".left.kv_heads", f"{heads} query heads are no multiple of {kv} key/value heads")
    mask = left.get("mask")
    if not isinstance(mask, Mapping):
        raise MissingKey(where + ".left.mask")
    return {"left": {"heads": heads, "kv_heads": kv, "dim": _pos_int(left, "dim", where + ".left"),
                     "vdim": _pos_int(left, "vdim", where + ".left"), "conv": _pos_int(left, "conv", where + ".left"),
                     "mask": {"size": _pos_int(mask, "size", where + ".left.mask")},
                     "scale": _number(left, "scale", where + ".left")},
            "right": {"heads": _pos_int(right, "heads", where + ".right"), "dim": _pos_int(right, "dim", where + ".right"),
                      "decay_rank": _rank(right, "decay_rank", shapes, prefix + "right.w1", where + ".right")},
            "left_scale": _number(m, "left_scale", where), "right_scale": _number(m, "right_scale", where)}


_MIXER_PARSERS = {"gla": _parse_gla, "channel_delta": _parse_channel_delta, "parallel": _parse_parallel}
