"""Plain, slow implementation of the Sisetar decoder: the oracle of its tests.

Whole sequences, no cache, no batching, one function for each mechanism, recurrences as
loops over the tokens.  It shares no code with the package: config.json is read with
``json``, the weights with the ``safetensors`` library, and everything is computed with torch
on the CPU in ``float64`` (or ``float32``).

Notation.  T tokens at positions 0..T-1, x the residual stream [T, width], h the input of a
mixer (the layer-normed stream).  W[name] is stored [out, in] and applied as W h.

* layer_norm:   (x - mean) / sqrt(var + eps) * w, var the mean of the squared deviations.
* rms:          y / sqrt(mean(y^2) + eps).
* gla:          per head, S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T q_t with S [dim, vdim];
                alpha = sigmoid(z)^(1/tau), z = A2 (A1 h) + b.
* softmax attention on chunks: key j is seen from position i if j <= i and i // size == j // size.
* delta rule:   per head, S <- diag(w_t) S - (a_t * u_t)(u_t^T S) + k_t v_t^T (both read the old S),
                o_t = S^T r_t, u the key scaled to unit length.
* polynorm:     a rms(z) + b rms(z^2) + c rms(z^3) + e over the feed-forward's inner vector.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Sequence

import torch


def read_config(folder: str) -> dict:
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)


def read_weights(folder: str, dtype=torch.float64) -> Dict[str, torch.Tensor]:
    from safetensors import safe_open
    out = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            out[name] = f.get_tensor(name).to(dtype)
    return out


# --------------------------------------------------------------------------- small pieces


def layer_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    mean = x.mean(dim=-1, keepdim=True)
    dev = x - mean
    var = (dev * dev).mean(dim=-1, keepdim=True)
    return dev / torch.sqrt(var + eps) * w


def rms(y: torch.Tensor, eps: float) -> torch.Tensor:
    return y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def rotate_part(x: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, d] at positions 0..T-1.  Of each head's first ``dims`` dimensions, i is paired with
    i + dims/2 and the pair is turned by position * base^(-2i/dims); the other dimensions pass."""
    T = x.shape[0]
    half = dims // 2
    out = x.clone()
    if half == 0:
        return out
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    ang = torch.arange(T, dtype=x.dtype)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


# --------------------------------------------------------------------------- mixers


def gla_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, V, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    q = (h @ w[p + "q"].t()).view(T, H, D) * D ** -0.5
    k = (h @ w[p + "k"].t()).view(T, H, D)
    v = (h @ w[p + "v"].t()).view(T, H, V)
    z = (h @ w[p + "a1"].t()) @ w[p + "a2"].t() + w[p + "a2.b"]
    alpha = (torch.sigmoid(z) ** (1.0 / tau)).view(T, H, D)
    S = torch.zeros(H, D, V, dtype=h.dtype)
    o = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms(o, eps) * w[p + "norm"]
    g = silu(h @ w[p + "g"].t())
    return (o.reshape(T, H * V) * g) @ w[p + "o"].t()


def chunk_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].t()).view(T, H, D)
    k = (h @ w[p + "k"].t()).view(T, G, D)
    v = (h @ w[p + "v"].t()).view(T, G, V)
    q = rms(rotate_part(q, m["rot"]["dims"], m["rot"]["base"]), eps)
    k = rms(rotate_part(k, m["rot"]["dims"], m["rot"]["base"]), eps)
    size = m["mask"]["size"]
    pos = torch.arange(T)
    seen = (pos[None, :] <= pos[:, None]) & ((pos[None, :] // size) == (pos[:, None] // size))
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].t()) * m["scale"]
        s = s.masked_fill(~seen, float("-inf"))
        out[:, hh] = torch.softmax(s, dim=-1) @ v[:, g]
    return out.reshape(T, H * V) @ w[p + "o"].t()


def delta_rule_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    r = (h @ w[p + "r"].t()).view(T, H, D)
    k = (h @ w[p + "k"].t()).view(T, H, D)
    v = (h @ w[p + "v"].t()).view(T, H, D)
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ w[p + "w1"].t()) @ w[p + "w2"].t() + w[p + "w0"])).view(T, H, D)
    a = torch.sigmoid(h @ w[p + "a"].t() + w[p + "a.b"]).view(T, H, D)
    u = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    S = torch.zeros(H, D, D, dtype=h.dtype)
    o = torch.zeros(T, H, D, dtype=h.dtype)
    for t in range(T):
        uS = torch.einsum("hd,hdv->hv", u[t], S)
        S = decay[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * uS[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, r[t])
    o = rms(o, eps).reshape(T, H * D) * w[p + "norm"]
    return (o * torch.sigmoid(h @ w[p + "g"].t())) @ w[p + "o"].t()


def parallel_mixer(h, w, p, m, eps):
    left = chunk_attention(h, w, p + "left.", m["left"], eps)
    right = delta_rule_mixer(h, w, p + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


MIXERS = {"gla": gla_mixer, "parallel": parallel_mixer}


# --------------------------------------------------------------------------- feed-forward


def polynorm_mlp(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    z = h @ w[p + "up"].t()
    a, b, c, e = [float(t) for t in w[p + "act"]]
    act = a * rms(z, eps) + b * rms(z * z, eps) + c * rms(z * z * z, eps) + e
    return act @ w[p + "down"].t()


# --------------------------------------------------------------------------- the model


def forward(cfg: dict, w: Dict[str, torch.Tensor], ids: Sequence[int], layers_out: List[torch.Tensor] = None) -> torch.Tensor:
    """Logits [T, vocab] of the whole sequence.  ``layers_out`` collects the stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(list(ids), dtype=torch.long)] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = layer_norm(x, w[p + "norm1"], eps)
        x = x + MIXERS[layer["type"]](h, w, p + "mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"feed-forward kind {layer['mlp']['kind']!r}")
            h = layer_norm(x, w[p + "norm2"], eps)
            x = x + polynorm_mlp(h, w, p + "mlp.", eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = layer_norm(x, w["final.norm"], eps)
    logits = (x @ w["embed"].t()) * cfg["logit_scale"]
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits
