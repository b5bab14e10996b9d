"""A plain, slow statement of the Damadra forward pass: one whole sequence at a time, no cache,
no batch, one function per mechanism, torch on the CPU only (float64 unless told otherwise).
It shares no code with `reinfer_b200`; the tests compare the engine with it.

Notation.  x is the residual stream [T, width]; `lin(x, W) = x W^T` with W stored [out, in];
rms(v) = v / sqrt(mean(v^2) + eps).  The sublayers read x itself and the norm sits on their
OUTPUT:   x += m * rms(mixer(x)) * w1;   x += m * rms(ff(x)) * w2.   Two mixers, both softmax
attention without a rotation whose scores get a learned bias by distance:

* `attention`    sliding window; q and k normalised over the whole projection; the values are the
                 keys as projected (before their norm)
* `attention_2`  causal; q and k normalised per head with one weight for all heads; queries
                 warmed up with position; a projection of its own for the values; may read the
                 keys and values of an earlier layer

and two feed-forwards: a dense gated one (silu) and a mixture of small experts (squared relu)
with a softmax router, a correction that only the choice sees, and experts that are the identity.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import numpy as np
import torch


# ---------------------------------------------------------------- file reading
def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    with open(path, "rb") as f:
        raw = f.read()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    data = raw[8 + n:]
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        b, en = e["data_offsets"]
        buf = data[b:en]
        dt = e["dtype"]
        if dt == "F32":
            t = torch.from_numpy(np.frombuffer(buf, dtype="<f4").copy()).double()
        elif dt == "BF16":
            u = np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(u.view(np.float32).copy()).double()
        elif dt in ("I32", "I64"):
            t = torch.from_numpy(np.frombuffer(buf, dtype="<i4" if dt == "I32" else "<i8").copy()).long()
        else:
            raise ValueError(f"{name}: dtype {dt}")
        out[name] = t.reshape(e["shape"])
    return out


def read_model(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# ---------------------------------------------------------------- small pieces
def lin(x, w):
    return x @ w.T


def rms(v, eps):
    """v over its root mean square along the last axis, eps inside the root."""
    return v / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def distance_bucket(n: int, rows: int, far: int) -> int:
    """Row of the bias table for a distance n >= 0: the first half of the rows one distance each, the other half
    spread evenly over the logarithm of the distance up to `far`; the last row takes everything beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def distance_bias(T: int, rel, far: int):
    """[T, T, H]: rel[bucket(i - j), h] for j <= i (zero above the diagonal, where the mask rules)."""
    rows = rel.shape[0]
    idx = torch.zeros((T, T), dtype=torch.long)
    for n in range(T):
        b = distance_bucket(n, rows, far)
        i = torch.arange(n, T)
        idx[i, i - n] = b
    return rel[idx]


def query_warmth(T: int, coef: float, every: int):
    """[T]: 1 + coef ln(floor((p + 1) / every) + 1)."""
    p = torch.arange(T, dtype=torch.float64)
    return 1.0 + coef * torch.log(torch.floor((p + 1.0) / every) + 1.0)


def softmax_attention(q, k, v, scale: float, bias, window: Optional[int]):
    """q [T, H, d], k [T, G, d], v [T, G, dv], bias [T, T, H]; query head h reads key/value head h // (H / G).
    Position i sees j <= i, with a window only those with i - j < window."""
    T, H, _ = q.shape
    G = k.shape[1]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & (i - j < window)
    out = torch.zeros((T, H, v.shape[2]), dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale + bias[:, :, h]
        s = s.masked_fill(~seen, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


# ---------------------------------------------------------------- mixers
def window_attention_kv(h, W, p, m, eps):
    """Keys (after their norm) and values of the mixer `attention`: one norm over all of k's rows at once; the
    values are k as projected."""
    G, d = m["kv_heads"], m["dim"]
    k = lin(h, W[p + "k"])
    v = k.clone()
    k = rms(k, eps) * W[p + "k.norm"]
    return k.reshape(-1, G, d), v.reshape(-1, G, d)


def window_attention(h, W, p, m, eps, kv=None):
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    q = rms(lin(h, W[p + "q"]), eps) * W[p + "q.norm"]
    k, v = kv if kv is not None else window_attention_kv(h, W, p, m, eps)
    bias = distance_bias(T, W[p + "rel"], m["bias_max"])
    o = softmax_attention(q.reshape(T, H, d), k, v, m["scale"], bias, m["mask"]["size"])
    return lin(o.reshape(T, -1), W[p + "o"])


def causal_attention_kv(h, W, p, m, eps):
    """Keys (normalised per head, one weight [d] for all heads) and values of the mixer `attention_2`."""
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = lin(h, W[p + "k"]).reshape(-1, G, d)
    k = rms(k, eps) * W[p + "k.norm"]
    v = lin(h, W[p + "v"]).reshape(-1, G, dv)
    return k, v


def causal_attention(h, W, p, m, eps, kv=None):
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    q = lin(h, W[p + "q"]).reshape(T, H, d)
    q = rms(q, eps) * W[p + "q.norm"]
    if m.get("q_temp"):
        q = q * query_warmth(T, m["q_temp"]["coef"], m["q_temp"]["every"])[:, None, None]
    k, v = kv if kv is not None else causal_attention_kv(h, W, p, m, eps)
    bias = distance_bias(T, W[p + "rel"], m["bias_max"])
    o = softmax_attention(q, k, v, m["scale"], bias, None)
    return lin(o.reshape(T, -1), W[p + "o"])


# ---------------------------------------------------------------- feed-forwards
def dense_ff(h, W, p):
    return lin(silu(lin(h, W[p + "gate"])) * lin(h, W[p + "up"]), W[p + "down"])


def route(h, W, p, r):
    """(chosen [T, top] expert numbers, weights [T, top]): softmax over all router outputs, the choice by
    score + correction, the weights the scores themselves."""
    s = torch.softmax(lin(h, W[p + "router"]), dim=-1)
    chosen = torch.topk(s + W[p + "correction"], r["top"], dim=-1).indices
    return chosen, torch.gather(s, 1, chosen)


def expert_ff(h, W, p):
    return lin(torch.relu(lin(h, W[p + "up"])) ** 2, W[p + "down"])


def moe_ff(h, W, p, r):
    E = r["experts"]
    chosen, weight = route(h, W, p, r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t].tolist(), weight[t]):
            out[t] += w * (expert_ff(h[t:t + 1], W, f"{p}e{e}.")[0] if e < E else h[t])
    return out


# ---------------------------------------------------------------- the model
def forward(cfg, W, tokens: List[int], dtype=torch.float64, layers_out: Optional[list] = None):
    """Logits [T, vocab] of one sequence.  layers_out: a list that receives the residual stream after each layer."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in W.items()}
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    x = W["embed"][torch.as_tensor(tokens)] * cfg["embedding"]["scale"]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        src = m.get("kv_from")
        if layer["type"] == "attention":
            kv = kept[src] if src is not None else window_attention_kv(x, W, p, m, eps)
            y = window_attention(x, W, p, m, eps, kv)
        elif layer["type"] == "attention_2":
            kv = kept[src] if src is not None else causal_attention_kv(x, W, p, m, eps)
            y = causal_attention(x, W, p, m, eps, kv)
        else:
            raise ValueError(layer["type"])
        kept[i] = kv
        x = x + mult * rms(y, eps) * W[f"l{i}.norm1"]
        mlp = layer.get("mlp")
        if mlp is not None:
            y = dense_ff(x, W, f"l{i}.mlp.") if mlp["kind"] == "dense" else moe_ff(x, W, f"l{i}.mlp.", mlp["router"])
            x = x + mult * rms(y, eps) * W[f"l{i}.norm2"]
        if layers_out is not None:
            layers_out.append(x.clone())
    return lin(rms(x, eps) * W["final.norm"], W["head"])
