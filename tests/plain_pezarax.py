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


def two_map_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor,
                      scale: float, lam: float, eps: float, factor: float) -> torch.Tensor:
    """q [T, heads, 2, dim] (rotated), k [S, groups, 2, dim], v [S, groups, vdim], mask [T, S]
    -> [T, heads, vdim]: a1 - lam a2, unit RMS per head, times ``factor``."""
    t, heads = q.shape[0], q.shape[1]
    per = heads // k.shape[1]
    out = torch.zeros((t, heads, v.shape[-1]), dtype=q.dtype)
    for hd in range(heads):
        g = hd // per
        maps = []
        for m in range(2):
            s = (q[:, hd, m] @ k[:, g, m].T) * scale
            s = s.masked_fill(~mask, float("-inf"))
            maps.append(torch.softmax(s, dim=-1) @ v[:, g])
        out[:, hd] = unit_rms(maps[0] - lam * maps[1], eps) * factor
    return out


def decayed_states(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay, state=None):
    """q, k [T, heads, dim], v [T, heads, vdim] -> (o [T, heads, vdim], last state [heads, dim,
    vdim]) with S <- decay_h S + k v^T and o = S^T q, token by token."""
    t, heads, dim = q.shape
    out = torch.zeros((t, heads, v.shape[-1]), dtype=q.dtype)
    last = torch.zeros((heads, dim, v.shape[-1]), dtype=q.dtype) if state is None else state.clone()
    for hd in range(heads):
        s = last[hd]
        for i in range(t):
            s = float(decay[hd]) * s + torch.outer(k[i, hd], v[i, hd])
            out[i, hd] = s.T @ q[i, hd]
        last[hd] = s
    return out, last


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
    size = int(mx["mask"]["size"]) if mx.get("mask") else start + t
    mask = chunk_mask(t, size, start)
    out = two_map_attention(q, k, v, mask, float(mx["scale"]), float(lam), eps, 1.0 - diff)
    return out.reshape(t, heads * vdim) @ w("o").T


def retention(h: torch.Tensor, tensors, prefix: str, mx: dict, eps: float,
              delicate: Optional[list] = None) -> torch.Tensor:
    """Linear attention with one fixed decay per head, token by token:
    S <- decay S + k v^T, o = S^T q; unit RMS per head, a SiLU gate of the input, projection.
    ``delicate`` (a list) receives a tensor [T]: per token the smallest, over heads, of rms(o)
    over the size o would have if nothing cancelled (|q_t| sqrt(sum_j decay^(2(t-j)) |k_j|^2
    mean(v_j^2))); where that is tiny the unit norm blows rounding up, the sign of o included."""
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
    out, _ = decayed_states(q, k, v, mx["decay"])
    if delicate is not None:
        ratios = torch.zeros((t, heads), dtype=dtype)
        for hd in range(heads):
            acc = 0.0
            for i in range(t):
                acc = float(mx["decay"][hd]) ** 2 * acc + float(k[i, hd].pow(2).sum() * v[i, hd].pow(2).mean())
                size = float(q[i, hd].norm()) * math.sqrt(acc)
                ratios[i, hd] = float(out[i, hd].pow(2).mean().sqrt()) / max(size, 1e-300)
        delicate.append(ratios.min(dim=1).values)
    out = unit_rms(out, eps).reshape(t, heads * vdim)
    gate = h @ w("g").T
    return (out * gate * torch.sigmoid(gate)) @ w("o").T


def routed_experts(h: torch.Tensor, tensors, prefix: str, mlp: dict,
                   margins: Optional[list] = None) -> torch.Tensor:
    """Sigmoid scores per expert; the ``top`` largest are chosen and weight the expert's
    INPUT; an expert is down(relu(up(.))^2).  ``margins`` (a list) receives a tensor [T]: per token the gap
    between the router logits of the last expert chosen and the best one left out."""
    dtype = h.dtype
    w = lambda name: tensors[prefix + "mlp." + name].to(dtype)
    n, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    logits = h @ w("router").T
    scores = torch.sigmoid(logits)
    order = torch.argsort(scores, dim=-1, descending=True, stable=True)
    out = torch.zeros_like(h)
    if margins is not None:
        ranked = torch.gather(logits, 1, order)
        margins.append(ranked[:, top - 1] - ranked[:, top] if top < n
                       else torch.full((h.shape[0],), float("inf"), dtype=dtype))
    for i in range(h.shape[0]):
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
            margins: Optional[list] = None, delicate: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  ``taps`` receives the stream after every
    layer run; ``margins`` and ``delicate``: see ``routed_experts`` and ``retention``."""
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
            x = x + retention(h, tensors, p, entry["mixer"], eps, delicate)
        else:
            raise ValueError(f"unknown mixer {entry['type']!r}")
        if entry.get("mlp") is not None:
            h = weighted_norm(x, tensors[p + "norm2"], eps)
            x = x + routed_experts(h, tensors, p, entry["mlp"], margins)
        if taps is not None:
            taps.append(x.clone())
    x = weighted_norm(x, tensors["final.norm"], eps)
    return (x @ tensors["head"].to(dtype).T) * float(cfg["logit_scale"])


def greedy(prompt: List[int], n_new: int, tensors, cfg: dict, dtype=torch.float64) -> List[int]:
    """The ``n_new`` tokens greedy decoding appends, each from a whole new forward pass."""
    ids, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(forward(ids, tensors, cfg, dtype)[-1].argmax())
        out.append(nxt)
        ids.append(nxt)
    return out
