"""Plain, slow implementation of the Vegilix decoder: the oracle of its tests.

Whole sequences, no cache, no batching, one function for each mechanism, the recurrence as a
loop over the tokens.  It shares no code with the package: config.json is read with ``json``,
the weights with the ``safetensors`` library, and everything is computed with torch on the CPU
in ``float64`` (or ``float32``).

Notation.  T tokens at positions 0..T-1, x the residual stream [T, width], h the input of a
sublayer (the normed stream), m the residual multiplier.  W[name] is stored [out, in] and
applied as W h.

* rms(y):            y / sqrt(mean(y^2) + eps).
* norm(y, w):        rms(y) * (1 + w)                              (weights stored around zero)
* layer:             x <- x + m norm_1b(mixer(norm_1(x)));  x <- x + m norm_2b(ff(norm_2(x)))
* differential attention:  every head has two maps of queries and keys over one set of values;
                     a_1, a_2 the two softmax attentions, lam = exp(lq1 . lk1) - exp(lq2 . lk2) + diff,
                     o = rms(a_1 - lam a_2) (1 - diff).  q and k are normed (weight, per map) and then
                     rotated; position i sees j <= i with i - j < size or j < keep_first.
* retention:         per head, S <- decay S + (k_t / sqrt(dim)) v_t^T, o_t = S^T q_t with S [dim, vdim];
                     q and k rotated; o = rms(o) per head, times silu(G h).
* experts:           z = R h; the ``top`` largest z pick the experts, softmax over the picked z weighs them;
                     an expert is D (silu(G h) * (U h)); a shared expert is added for every token.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

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


def rms(y: torch.Tensor, eps: float) -> torch.Tensor:
    return y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps)


def norm(y: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms(y, eps) * (1.0 + w)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def frequencies(rot: dict) -> List[float]:
    """f_i = base^(-2i/dims), i < dims/2; with ``scaling``, long wavelengths are slowed by ``factor``, short ones
    kept, and those between are blended by where original/wavelength lies between ``low`` and ``high``."""
    dims, base = int(rot["dims"]), float(rot["base"])
    out = []
    sc = rot.get("scaling")
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if sc:
            factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
            wavelength = 2.0 * math.pi / f
            if wavelength < orig / high:
                pass
            elif wavelength > orig / low:
                f = f / factor
            else:
                s = (orig / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


def rotate(x: torch.Tensor, rot: dict, positions: Sequence[int]) -> torch.Tensor:
    """x [T, n, d]: the first rot.dims dimensions of every vector are turned, pairs (i, i + dims/2), by
    position * f_i; the others pass."""
    dims = int(rot["dims"])
    if dims == 0:
        return x
    half = dims // 2
    f = torch.tensor(frequencies(rot), dtype=x.dtype)
    pos = torch.tensor(list(positions), dtype=x.dtype)
    angle = pos[:, None] * f[None, :]                       # [T, half]
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def visible(T: int, mask: Optional[dict]) -> torch.Tensor:
    """[T, T] bool: entry (i, j) says whether position i sees position j."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    see = j <= i
    if mask and mask.get("size") is not None:
        see = see & ((i - j < int(mask["size"])) | (j < int(mask.get("keep_first") or 0)))
    return see


# --------------------------------------------------------------------------- mixers


def softmax_map(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, mask: Optional[dict]) -> torch.Tensor:
    """q [T, d], k [T, d], v [T, dv] of one head and map -> [T, dv]: softmax over the visible keys of every row."""
    s = (q @ k.T) * scale
    s = s.masked_fill(~visible(q.shape[0], mask), float("-inf"))
    return torch.softmax(s, dim=-1) @ v


def differential_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, mc: dict, eps: float,
                           positions: Sequence[int]) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = int(mc["heads"]), int(mc["kv_heads"]), int(mc["dim"]), int(mc["vdim"])
    diff = float(mc["diff"])
    q = (h @ W[p + "q"].T).view(T, H * 2, d)
    k = (h @ W[p + "k"].T).view(T, G * 2, d)
    v = (h @ W[p + "v"].T).view(T, G, dv)
    q = rms(q, eps) * W[p + "q.norm"]
    k = rms(k, eps) * W[p + "k.norm"]
    q = rotate(q, mc["rot"], positions)
    k = rotate(k, mc["rot"], positions)
    lam = (math.exp(float((W[p + "lq1"] * W[p + "lk1"]).sum())) - math.exp(float((W[p + "lq2"] * W[p + "lk2"]).sum()))
           + diff)
    heads = []
    for a in range(H):
        g = a // (H // G)
        a1 = softmax_map(q[:, 2 * a], k[:, 2 * g], v[:, g], float(mc["scale"]), mc.get("mask"))
        a2 = softmax_map(q[:, 2 * a + 1], k[:, 2 * g + 1], v[:, g], float(mc["scale"]), mc.get("mask"))
        heads.append(rms(a1 - lam * a2, eps) * (1.0 - diff))
    return torch.cat(heads, dim=1) @ W[p + "o"].T


def retention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, mc: dict, eps: float,
              positions: Sequence[int]) -> torch.Tensor:
    T = h.shape[0]
    H, d, dv = int(mc["heads"]), int(mc["dim"]), int(mc["vdim"])
    q = rotate((h @ W[p + "q"].T).view(T, H, d), mc["rot"], positions)
    k = rotate((h @ W[p + "k"].T).view(T, H, d), mc["rot"], positions) * d ** -0.5
    v = (h @ W[p + "v"].T).view(T, H, dv)
    o = torch.zeros((T, H, dv), dtype=h.dtype)
    for a in range(H):
        S = torch.zeros((d, dv), dtype=h.dtype)
        decay = float(mc["decay"][a])
        for t in range(T):
            S = decay * S + torch.outer(k[t, a], v[t, a])
            o[t, a] = S.T @ q[t, a]
    o = rms(o, eps).reshape(T, H * dv) * silu(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


# --------------------------------------------------------------------------- feed-forward


def expert(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def experts(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, fc: dict, margins: Optional[list] = None) -> torch.Tensor:
    """``margins`` gets, for every token, how far the last chosen logit lies above the first that is not chosen, as a
    part of the largest logit's size (a small margin is a close call that rounding may decide the other way)."""
    n, top = int(fc["router"]["experts"]), int(fc["router"]["top"])
    z = h @ W[p + "router"].T                               # [T, n]
    if margins is not None and top < n:
        ranked = torch.sort(z, dim=1, descending=True).values
        margins.append((ranked[:, top - 1] - ranked[:, top]) / z.abs().max(dim=1).values.clamp_min(1e-9))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        order = sorted(range(n), key=lambda e: (-float(z[t, e]), e))[:top]
        w = torch.softmax(z[t, order], dim=0)
        for e, we in zip(order, w):
            out[t] = out[t] + we * expert(h[t:t + 1], W, f"{p}e{e}.")[0]
    if fc.get("shared"):
        out = out + expert(h, W, p + "shared.")
    return out


# --------------------------------------------------------------------------- the model


def run_order(cfg: dict) -> List[int]:
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: Sequence[int], dtype=torch.float64, streams: Optional[list] = None,
            positions: Optional[Sequence[int]] = None, margins: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence.  ``streams``: a list that gets the residual stream after every layer run;
    ``margins``: a list that gets every router's margins (see ``experts``)."""
    W = {n: t.to(dtype) for n, t in W.items()}
    eps, m = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    pos = list(range(len(tokens))) if positions is None else list(positions)
    x = W["embed"][torch.tensor(list(tokens), dtype=torch.long)]
    for i in run_order(cfg):
        layer, p = cfg["layers"][i], f"l{i}."
        h = norm(x, W[p + "norm1"], eps)
        if layer["type"] == "attention":
            y = differential_attention(h, W, p + "mix.", layer["mixer"], eps, pos)
        elif layer["type"] == "retention":
            y = retention(h, W, p + "mix.", layer["mixer"], eps, pos)
        else:
            raise ValueError(f"layer type {layer['type']!r}")
        x = x + m * norm(y, W[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = norm(x, W[p + "norm2"], eps)
            x = x + m * norm(experts(h, W, p + "mlp.", layer["mlp"], margins), W[p + "norm2b"], eps)
        if streams is not None:
            streams.append(x.clone())
    return norm(x, W["final.norm"], eps) @ W["head"].T
