"""A plain, slow statement of the Silutar forward pass: one whole sequence at a time, no
cache, no batch, one function per mechanism, torch on the CPU only (float64 unless told
otherwise).  It shares no code with `reinfer_b200`; the tests compare the engine with it.

Notation.  x is the residual stream [T, width]; a linear map is `lin(x, W) = x W^T` with W
stored [out, in].  A layer is  x += mixer(dyt(x));  x += ff(dyt(x))  (the second only where
the layer has a feed-forward).  Three mixers:

* `gla`            gated linear attention: S_t = diag(a_t) S_{t-1} + k_t v_t^T, o_t = S_t^T q_t
* `channel_delta`  gated delta rule with a decay per key channel and short convolutions
* `parallel`       the weighted sum of a chunk-masked softmax attention with a logarithmic
                   distance penalty (left) and a generalised delta rule (right)
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List

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
    return x @ w.t()


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def dyt(x, w, b, alpha):
    """Dynamic tanh in place of a normalisation: tanh(alpha x) w + b, no statistics."""
    return torch.tanh(alpha * x) * w + b


def rms_unit(x, eps):
    """x over its root mean square along the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def l2_unit(x):
    """x as a unit vector along the last axis: x / sqrt(sum x^2 + 1e-6)."""
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def short_conv(u, w):
    """Causal convolution over time, each channel alone.  u [T, C], w [C, taps]; the last tap
    multiplies the present token, zeros stand before the sequence."""
    T, C = u.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], 0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + pad[j:j + T] * w[:, j]
    return y


def dense_ff(x, p, W):
    return lin(silu(lin(x, W[p + "gate"])) * lin(x, W[p + "up"]), W[p + "down"])


# ---------------------------------------------------------------- the three recurrences
def scan_gla(q, k, v, a):
    """q, k, a [T, dk], v [T, dv] of one head.  S = diag(a_t) S + k_t v_t^T; o_t = S^T q_t."""
    T, dk = k.shape
    S = torch.zeros(dk, v.shape[1], dtype=q.dtype)
    out = []
    for t in range(T):
        S = a[t][:, None] * S + torch.outer(k[t], v[t])
        out.append(S.t() @ q[t])
    return torch.stack(out)


def scan_general_delta(r, k, v, w, a):
    """One head.  With the unit key u: S = diag(w) S - (a u)(u^T S) + k v^T, both of the first two terms
    from the old state; o = S^T r."""
    T, dk = k.shape
    S = torch.zeros(dk, v.shape[1], dtype=r.dtype)
    u = l2_unit(k)
    out = []
    for t in range(T):
        S = w[t][:, None] * S - torch.outer(a[t] * u[t], u[t] @ S) + torch.outer(k[t], v[t])
        out.append(S.t() @ r[t])
    return torch.stack(out)


def scan_gated_delta(q, k, v, g, beta):
    """One head.  S <- g S (rows); d = beta (v - S^T k); S <- S + k d^T; o = S^T q."""
    T, dk = k.shape
    S = torch.zeros(dk, v.shape[1], dtype=q.dtype)
    out = []
    for t in range(T):
        S = g[t][:, None] * S
        d = beta[t] * (v[t] - S.t() @ k[t])
        S = S + torch.outer(k[t], d)
        out.append(S.t() @ q[t])
    return torch.stack(out)


# ---------------------------------------------------------------- mixers
def mixer_gla(h, p, m, W, eps):
    T = h.shape[0]
    H, dk, dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    q = (lin(h, W[p + "q"]) * dk ** -0.5).view(T, H, dk)
    k = lin(h, W[p + "k"]).view(T, H, dk)
    v = lin(h, W[p + "v"]).view(T, H, dv)
    z = lin(lin(h, W[p + "a1"]), W[p + "a2"]) + W[p + "a2.b"]
    a = (sigmoid(z) ** (1.0 / tau)).view(T, H, dk)
    heads = []
    for i in range(H):
        o = scan_gla(q[:, i], k[:, i], v[:, i], a[:, i])
        heads.append(rms_unit(o, eps) * W[p + "norm"])
    o = torch.cat(heads, -1) * silu(lin(h, W[p + "g"]))
    return lin(o, W[p + "o"])


def chunk_attention(q, k, v, scale, r1, r2, chunk):
    """One query head over its key/value head.  q, k [T, d], v [T, dv].  Position i sees j <= i of its own
    chunk of `chunk` positions (counted from 0); score = q.k * scale - r1 ln(1 + r2 (i - j))."""
    T = q.shape[0]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    s = (q @ k.t()) * scale - r1 * torch.log1p(r2 * (i - j).clamp(min=0).to(q.dtype))
    visible = (j <= i) & (i // chunk == j // chunk)
    s = s.masked_fill(~visible, float("-inf"))
    return torch.softmax(s, -1) @ v


def mixer_parallel_left(h, p, m, W, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv(lin(h, W[p + "q"]), W[p + "q.conv"]).view(T, H, d)
    k = short_conv(lin(h, W[p + "k"]), W[p + "k.conv"]).view(T, G, d)
    v = short_conv(lin(h, W[p + "v"]), W[p + "v.conv"]).view(T, G, dv)
    q, k = rms_unit(q, eps), rms_unit(k, eps)
    heads = []
    for i in range(H):
        kv = i // (H // G)
        heads.append(chunk_attention(q[:, i], k[:, kv], v[:, kv], float(m["scale"]), W[p + "r1"][i], W[p + "r2"][i],
                                     int(m["mask"]["size"])))
    return lin(torch.cat(heads, -1), W[p + "o"])


def mixer_parallel_right(h, p, m, W, eps):
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    r = lin(h, W[p + "r"]).view(T, H, d)
    k = lin(h, W[p + "k"]).view(T, H, d)
    v = lin(h, W[p + "v"]).view(T, H, d)
    w = torch.exp(-math.exp(-0.5) * sigmoid(lin(torch.tanh(lin(h, W[p + "w1"])), W[p + "w2"]) + W[p + "w0"])).view(T, H, d)
    a = sigmoid(lin(h, W[p + "a"]) + W[p + "a.b"]).view(T, H, d)
    heads = [rms_unit(scan_general_delta(r[:, i], k[:, i], v[:, i], w[:, i], a[:, i]), eps) for i in range(H)]
    o = torch.cat(heads, -1) * W[p + "norm"] * sigmoid(lin(h, W[p + "g"]))
    return lin(o, W[p + "o"])


def mixer_parallel(h, p, m, W, eps):
    return float(m["left_scale"]) * mixer_parallel_left(h, p + "left.", m["left"], W, eps) + \
        float(m["right_scale"]) * mixer_parallel_right(h, p + "right.", m["right"], W, eps)


def mixer_channel_delta(h, p, m, W, eps):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(lin(h, W[p + "q"]), W[p + "q.conv"])).view(T, G, dk)
    k = silu(short_conv(lin(h, W[p + "k"]), W[p + "k.conv"])).view(T, G, dk)
    v = silu(short_conv(lin(h, W[p + "v"]), W[p + "v.conv"])).view(T, H, dv)
    q = l2_unit(q) * dk ** -0.5
    k = l2_unit(k)
    beta = sigmoid(lin(h, W[p + "b"]))                                           # [T, H]
    z = lin(lin(h, W[p + "a1"]), W[p + "a2"]) + W[p + "dt_bias"]
    g = torch.exp(-torch.exp(W[p + "A_log"])[None, :, None] * softplus(z).view(T, H, dk))
    gate = sigmoid(lin(lin(h, W[p + "g1"]), W[p + "g2"])).view(T, H, dv)
    heads = []
    for i in range(H):
        kv = i // (H // G)
        o = scan_gated_delta(q[:, kv], k[:, kv], v[:, i], g[:, i], beta[:, i])
        heads.append(rms_unit(o, eps) * W[p + "norm"] * gate[:, i])
    return lin(torch.cat(heads, -1), W[p + "o"])


MIXERS = {"gla": mixer_gla, "parallel": mixer_parallel, "channel_delta": mixer_channel_delta}


# ---------------------------------------------------------------- the model
def norm_of(x, name, W):
    return dyt(x, W[name], W[name + ".b"], W[name + ".alpha"])


def forward(cfg, W, tokens: List[int], dtype=torch.float64, layers_out=None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence.  layers_out: a list that receives the residual stream after every layer."""
    W = {n: (t.to(dtype) if t.is_floating_point() else t) for n, t in W.items()}
    eps = float(cfg["norm"]["eps"])
    T = len(tokens)
    x = W["embed"][torch.tensor(tokens, dtype=torch.long)] + W["pos"][:T]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        x = x + MIXERS[layer["type"]](norm_of(x, p + "norm1", W), p + "mix.", layer["mixer"], W, eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            if mlp["kind"] != "dense":
                raise ValueError(f"feed-forward of kind {mlp['kind']}")
            x = x + dense_ff(norm_of(x, p + "norm2", W), p + "mlp.", W)
        if layers_out is not None:
            layers_out.append(x.clone())
    logits = lin(norm_of(x, "final.norm", W), W["embed"])
    cap = cfg.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    return logits
