"""A plain, slow Pezarax: whole sequences at once, no cache, no kernels, one function per
mechanism.  The oracle the engine is compared with; it shares no code with the package.

Notation: x is the residual stream [T, width]; ``tensors`` is a dict name -> torch tensor;
``cfg`` is the raw ``config.json`` dict.  Everything is computed in ``dtype`` (float64 by
default) from the tensors' stored values.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import torch


# ------------------------------------------------------------------------------ reading
def read_folder(folder: str):
    """(cfg, tensors) of a model folder, with a reader of its own for the tensor file: eight
    bytes of header length, the JSON header, then the data."""
    with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as fh:
        cfg = json.load(fh)
    with open(os.path.join(folder, "model.safetensors"), "rb") as fh:
        blob = fh.read()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + n].decode("utf-8"))
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16,
             "I32": torch.int32, "F64": torch.float64}
    tensors = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw = bytearray(blob[8 + n + lo:8 + n + hi])
        t = torch.frombuffer(raw, dtype=kinds[info["dtype"]]) if raw else \
            torch.empty(0, dtype=kinds[info["dtype"]])
        tensors[name] = t.reshape(info["shape"]).clone()
    return cfg, tensors


# ---------------------------------------------------------------------------- mechanisms
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def weighted_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * weight.to(x.dtype)


def embed(tokens: List[int], tensors, cfg: dict, dtype) -> torch.Tensor:
    """Token rows times the embedding's scale."""
    return tensors["embed"].to(dtype)[torch.tensor(tokens)] * float(cfg["embedding"]["scale"])


def rotate_half(v: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """Coordinate i < dims/2 of the last axis pairs with i + dims/2; the pair at position p
    turns by p * base^(-2i/dims); coordinates from ``dims`` on stay.  v: [T, ..., n]."""
    half = dims // 2
    if half == 0:
        return v.clone()
    freq = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(half)], dtype=v.dtype)
    angle = positions.to(v.dtype)[:, None] * freq[None, :]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [half]
    cos, sin = torch.cos(angle).reshape(shape), torch.sin(angle).reshape(shape)
    a, b = v[..., :half], v[..., half:dims]
    out = v.clone()
    out[..., :half] = a * cos - b * sin
    out[..., half:dims] = b * cos + a * sin
    return out


def chunk_mask(t: int, size: int, start: int = 0) -> torch.Tensor:
    """[T, T] True where query i sees key j: j <= i and both lie in the same block of ``size``
    absolute positions (positions start .. start + T - 1)."""
    p = torch.arange(start, start + t)
    return (p[None, :] <= p[:, None]) & ((p[None, :] // size) == (p[:, None] // size))


def differential_attention(h: torch.Tensor, tensors, prefix: str, mx: dict, eps: float,
                           start: int = 0) -> torch.Tensor:
    """Two softmax attentions per head over the same values, subtracted with one learned
    factor, then unit RMS per head and a constant factor; grouped key/value heads; rotation
    on the first coordinates of each map; queries see keys of their own position block."""
    dtype = h.dtype
    w = lambda name: tensors[prefix + "mix." + name].to(dtype)
    t = h.shape[0]
    heads, groups = int(mx["heads"]), int(mx["kv_heads"])
    dim, vdim = int(mx["dim"]), int(mx["vdim"])
    diff = float(mx["diff"])
    pos = torch.arange(start, start + t)
    q = (h @ w("q").T).reshape(t, heads, 2, dim)
    k = (h @ w("k").T).reshape(t, groups, 2, dim)
    v = (h @ w("v").T).reshape(t, groups, vdim)
    q = rotate_half(q, pos, float(mx["rot"]["base"]), int(mx["rot"]["dims"]))
    k = rotate_half(k, pos, float(mx["rot"]["base"]), int(mx["rot"]["dims"]))
    lam = torch.exp((w("lq1") * w("lk1")).sum()) - torch.exp((w("lq2") * w("lk2")).sum()) + diff
    mask = chunk_mask(t, int(mx["mask"]["size"]), start)
    out = torch.zeros((t, heads, vdim), dtype=dtype)
    per = heads // groups
    for hd in range(heads):
        g = hd // per
        maps = []
        for m in range(2):
            s = (q[:, hd, m] @ k[:, g, m].T) * float(mx["scale"])
            s = s.masked_fill(~mask, float("-inf"))
            maps.append(torch.softmax(s, dim=-1) @ v[:, g])
        o = maps[0] - lam * maps[1]
        out[:, hd] = unit_rms(o, eps) * (1.0 - diff)
    return out.reshape(t, heads * vdim) @ w("o").T


def retention(h: torch.Tensor, tensors, prefix: str, mx: dict, eps: float) -> torch.Tensor:
    """Linear attention with one fixed decay per head, token by token:
    S <- decay S + k v^T, o = S^T q; unit RMS per head, a SiLU gate of the input, projection."""
    dtype = h.dtype
    w = lambda name: tensors[prefix + "mix." + name].to(dtype)
    t = h.shape[0]
    heads, dim, vdim = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"])
    pos = torch.arange(t)
    q = (h @ w("q").T).reshape(t, heads, dim)
    k = (h @ w("k").T).reshape(t, heads, dim)
    v = (h @ w("v").T).reshape(t, heads, vdim)
    q = rotate_half(q, pos, float(mx["rot"]["base"]), int(mx["rot"]["dims"]))
    k = rotate_half(k, pos, float(mx["rot"]["base"]), int(mx["rot"]["dims"])) * dim ** -0.5
    out = torch.zeros((t, heads, vdim), dtype=dtype)
    for hd in range(heads):
        decay = float(mx["decay"][hd])
        state = torch.zeros((dim, vdim), dtype=dtype)
        for i in range(t):
            state = decay * state + torch.outer(k[i, hd], v[i, hd])
            out[i, hd] = state.T @ q[i, hd]
    out = unit_rms(out, eps).reshape(t, heads * vdim)
    gate = h @ w("g").T
    return (out * gate * torch.sigmoid(gate)) @ w("o").T


def routed_experts(h: torch.Tensor, tensors, prefix: str, mlp: dict,
                   margins: Optional[list] = None) -> torch.Tensor:
    """Sigmoid scores per expert; the ``top`` largest are chosen and weight the expert's
    INPUT; an expert is down(relu(up(.))^2).  ``margins`` (a list) receives, per token, the gap
    between the last chosen score and the best one left out."""
    dtype = h.dtype
    w = lambda name: tensors[prefix + "mlp." + name].to(dtype)
    n, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    scores = torch.sigmoid(h @ w("router").T)
    order = torch.argsort(scores, dim=-1, descending=True, stable=True)
    out = torch.zeros_like(h)
    for i in range(h.shape[0]):
        if margins is not None:
            ranked = scores[i, order[i]]
            margins.append(float(ranked[top - 1] - ranked[top]) if top < n else float("inf"))
        for e in order[i, :top].tolist():
            u = (scores[i, e] * h[i]) @ w(f"e{e}.up").T
            out[i] += (torch.relu(u) ** 2) @ w(f"e{e}.down").T
    return out


# --------------------------------------------------------------------------------- model
def run_order(cfg: dict) -> List[tuple]:
    """(layer, adds the embedding output first) for every layer run: layers start..stop-1
    run ``times`` times in a row, the others once."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, False) for i in range(a)]
    for rep in range(times):
        order += [(i, rep > 0 and i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def forward(tokens: List[int], tensors, cfg: dict, dtype=torch.float64, taps: Optional[list] = None,
            margins: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  ``taps`` receives the stream after every
    layer run."""
    eps = float(cfg["norm"]["eps"])
    x0 = embed(tokens, tensors, cfg, dtype)
    x = x0.clone()
    for layer, again in run_order(cfg):
        entry, p = cfg["layers"][layer], f"l{layer}."
        if again:
            x = x + x0
        h = weighted_norm(x, tensors[p + "norm1"], eps)
        if entry["type"] == "attention":
            x = x + differential_attention(h, tensors, p, entry["mixer"], eps)
        elif entry["type"] == "retention":
            x = x + retention(h, tensors, p, entry["mixer"], eps)
        else:
            raise ValueError(f"unknown mixer {entry['type']!r}")
        if entry.get("mlp") is not None:
            h = weighted_norm(x, tensors[p + "norm2"], eps)
            x = x + routed_experts(h, tensors, p, entry["mlp"], margins)
        if taps is not None:
            taps.append(x.clone())
    x = weighted_norm(x, tensors["final.norm"], eps)
    return (x @ tensors["head"].to(dtype).T) * float(cfg["logit_scale"])
