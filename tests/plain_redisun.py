"""A plain, slow Redisun: whole sequences at once, no cache, no kernels, one function per
mechanism.  The oracle the engine is compared with; it shares no code with the package.

Notation: x is the residual stream [T, width]; tensors are a dict name -> torch tensor;
``cfg`` is the raw ``config.json`` dict.  Everything is computed in ``dtype`` (float64 by
default) from the tensors' stored values.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def scalar_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """Unit RMS times one learned number."""
    return unit_rms(x, eps) * gain.reshape(())


def vector_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """Unit RMS times a learned weight per coordinate."""
    return unit_rms(x, eps) * weight


def embed(tokens: List[int], tensors: Dict[str, torch.Tensor], cfg: dict, dtype) -> torch.Tensor:
    """Token row plus a hashed row for the pair (previous token, token); the first token of a
    sequence takes the table's last row."""
    table = tensors["embed"].to(dtype)
    x = table[torch.tensor(tokens)]
    big = cfg.get("embedding", {}).get("bigram")
    if big:
        pairs = tensors["bigram"].to(dtype)
        n = int(big["buckets"])
        rows = [n]
        for prev, cur in zip(tokens[:-1], tokens[1:]):
            rows.append((prev * int(big["mul_prev"]) + cur * int(big["mul_cur"])) % n)
        x = x + pairs[torch.tensor(rows)]
    return x


def rotate(v: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """Rotary positions in the rotate-half layout on the first ``dims`` coordinates of the
    last axis: coordinate i pairs with i + dims/2 and the pair turns by p * base^(-2i/dims).
    v: [T, ..., n]; positions: [T]."""
    half = dims // 2
    freq = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(half)], dtype=v.dtype)
    angle = positions.to(v.dtype)[:, None] * freq[None, :]              # [T, half]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [half]
    cos, sin = torch.cos(angle).reshape(shape), torch.sin(angle).reshape(shape)
    a, b = v[..., :half], v[..., half:dims]
    out = v.clone()
    out[..., :half] = a * cos - b * sin
    out[..., half:dims] = b * cos + a * sin
    return out


def sink_softmax(scores: torch.Tensor, sink: torch.Tensor) -> torch.Tensor:
    """Softmax over the last axis whose denominator also holds exp(sink): scores [..., n],
    sink broadcastable to scores[..., 0]."""
    m = torch.maximum(scores.max(dim=-1).values, sink)
    e = torch.exp(scores - m[..., None])
    return e / (e.sum(dim=-1) + torch.exp(sink - m))[..., None]


def latent_attention(h: torch.Tensor, tensors, prefix: str, mx: dict, eps: float) -> torch.Tensor:
    """Causal attention whose keys and values are expanded from one low-rank latent per token
    plus one rotated key part shared by the heads; queries pass a latent of their own; a sink
    per head joins the softmax denominator; heads are gated by a sigmoid of the input."""
    dtype = h.dtype
    w = lambda name: tensors[prefix + "mix." + name].to(dtype)
    t = h.shape[0]
    heads, dim, rot_dim = int(mx["heads"]), int(mx["dim"]), int(mx["rot_dim"])
    vdim, rank = int(mx["vdim"]), int(mx["kv_rank"])
    base, rdims = float(mx["rot"]["base"]), int(mx["rot"]["dims"])
    pos = torch.arange(t)
    cq = vector_norm(h @ w("dq").T, w("dq.norm"), eps)
    q = (cq @ w("uq").T).reshape(t, heads, dim + rot_dim)
    q_plain, q_rot = q[..., :dim], rotate(q[..., dim:], pos, base, rdims)
    down = h @ w("dkv").T
    c = vector_norm(down[:, :rank], w("dkv.norm"), eps)
    k_rot = rotate(down[:, rank:], pos, base, rdims)                     # [T, rot_dim]
    k_plain = (c @ w("uk").T).reshape(t, heads, dim)
    v = (c @ w("uv").T).reshape(t, heads, vdim)
    scores = torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)
    scores = scores * float(mx["scale"])
    mask = torch.ones(t, t, dtype=torch.bool).tril()
    scores = scores.masked_fill(~mask, float("-inf"))
    weights = sink_softmax(scores, w("sink")[:, None].expand(heads, t))
    out = torch.einsum("hij,jhd->ihd", weights, v)
    gate = torch.sigmoid(h @ w("g").T)                                   # [T, heads]
    out = out * gate[..., None]
    return out.reshape(t, heads * vdim) @ w("o").T


def dense_ff(h: torch.Tensor, tensors, prefix: str) -> torch.Tensor:
    w = lambda name: tensors[prefix + name].to(h.dtype)
    g = h @ w("gate").T
    return (g * torch.sigmoid(g) * (h @ w("up").T)) @ w("down").T


def clamped_ff(h: torch.Tensor, tensors, prefix: str, limit: float) -> torch.Tensor:
    """An expert: gate capped above, up clamped both ways, g*sigmoid(1.702 g)*(u+1)."""
    w = lambda name: tensors[prefix + name].to(h.dtype)
    g = torch.clamp(h @ w("gate").T, max=limit)
    u = torch.clamp(h @ w("up").T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w("down").T


def route(h: torch.Tensor, tensors, prefix: str, top: int):
    """(chosen experts [T, top], their weights [T, top]): largest logits, softmax over them."""
    z = h @ tensors[prefix + "router"].to(h.dtype).T + tensors[prefix + "router.b"].to(h.dtype)
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1), z


def moe_ff(h: torch.Tensor, tensors, prefix: str, mlp: dict) -> torch.Tensor:
    top = int(mlp["router"]["top"])
    idx, wts, _ = route(h, tensors, prefix, top)
    out = torch.zeros(h.shape[0], tensors[prefix + "e0.down"].shape[0], dtype=h.dtype)
    limit = float(mlp["expert"]["limit"])
    for t in range(h.shape[0]):
        for k in range(top):
            e = int(idx[t, k])
            out[t] += wts[t, k] * clamped_ff(h[t:t + 1], tensors, f"{prefix}e{e}.", limit)[0]
    if mlp.get("shared"):
        out = out + clamped_ff(h, tensors, prefix + "shared.", float(mlp["shared"]["limit"]))
    return out


def feed_forward(h, tensors, prefix: str, mlp: dict) -> torch.Tensor:
    if mlp["kind"] == "dense":
        return dense_ff(h, tensors, prefix + "mlp.")
    if mlp["kind"] == "moe":
        return moe_ff(h, tensors, prefix + "mlp.", mlp)
    raise ValueError(mlp["kind"])


def residual_gate(h, tensors, name: str) -> torch.Tensor:
    return torch.sigmoid(h @ tensors[name].to(h.dtype).T + tensors[name + ".b"].to(h.dtype))


def router_gap(h: torch.Tensor, tensors, prefix: str, mlp: dict) -> torch.Tensor:
    """Per token, how far the last chosen expert's logit lies above the first one left out
    (infinite when all are chosen): a choice with a small gap may fall either way once the
    input is rounded."""
    top = int(mlp["router"]["top"])
    _, _, z = route(h, tensors, prefix, top)
    if top >= z.shape[1]:
        return torch.full((h.shape[0],), float("inf"), dtype=h.dtype)
    ordered = torch.sort(z, dim=-1, descending=True).values
    return ordered[:, top - 1] - ordered[:, top]


def layer(x: torch.Tensor, tensors, i: int, spec: dict, cfg: dict,
          gaps: Optional[list] = None) -> torch.Tensor:
    """Norm after the sum, the branch gated: x <- norm(alpha x + gate(x) * branch(x))."""
    p = f"l{i}."
    eps, alpha = float(cfg["norm"]["eps"]), float(cfg["postln_alpha"])
    if spec["type"] != "latent_attention":
        raise ValueError(spec["type"])
    y = latent_attention(x, tensors, p, spec["mixer"], eps) * residual_gate(x, tensors, p + "rg1")
    x = scalar_norm(alpha * x + y, tensors[p + "norm1"].to(x.dtype), eps)
    if spec.get("mlp"):
        if gaps is not None and spec["mlp"]["kind"] == "moe":
            gaps.append(router_gap(x, tensors, p + "mlp.", spec["mlp"]))
        y = feed_forward(x, tensors, p, spec["mlp"]) * residual_gate(x, tensors, p + "rg2")
        x = scalar_norm(alpha * x + y, tensors[p + "norm2"].to(x.dtype), eps)
    elif p + "norm2" in tensors:               # no feed-forward, yet a second norm in the file
        x = scalar_norm(alpha * x, tensors[p + "norm2"].to(x.dtype), eps)
    return x


def forward(tokens: List[int], tensors, cfg: dict, dtype=torch.float64,
            streams: Optional[list] = None, gaps: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence; ``streams`` collects x after every layer,
    ``gaps`` every routed layer's :func:`router_gap`."""
    x = embed(tokens, tensors, cfg, dtype)
    for i, spec in enumerate(cfg["layers"]):
        x = layer(x, tensors, i, spec, cfg, gaps)
        if streams is not None:
            streams.append(x.clone())
    x = scalar_norm(x, tensors["final.norm"].to(dtype), float(cfg["norm"]["eps"]))
    return x @ tensors["head"].to(dtype).T


# ------------------------------------------------------------------ reading a model folder
def read_folder(folder: str):
    """(config dict, tensors by name as float32 / int32 torch tensors) of a model folder, read
    with nothing but the file format: 8 bytes of header length, a JSON header, the data."""
    import json
    import os
    import struct

    import numpy as np
    with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as fh:
        cfg = json.load(fh)
    with open(os.path.join(folder, "model.safetensors"), "rb") as fh:
        (n,) = struct.unpack("<Q", fh.read(8))
        header = json.loads(fh.read(n))
        data = fh.read()
    tensors = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        lo, hi = entry["data_offsets"]
        raw = data[lo:hi]
        if entry["dtype"] == "BF16":
            bits = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(bits.view(np.float32).copy())
        elif entry["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(raw, dtype="<f4").copy())
        elif entry["dtype"] == "I32":
            t = torch.from_numpy(np.frombuffer(raw, dtype="<i4").copy())
        else:
            raise ValueError(f"{name}: dtype {entry['dtype']}")
        tensors[name] = t.reshape(entry["shape"])
    return cfg, tensors


def greedy(tokens: List[int], n: int, tensors, cfg: dict) -> List[int]:
    """n tokens chosen by largest logit (lowest id among equals), the whole sequence run anew
    for every token."""
    ids, out = list(tokens), []
    for _ in range(n):
        row = forward(ids, tensors, cfg)[-1]
        best = int((row == row.max()).nonzero()[0])
        out.append(best)
        ids.append(best)
    return out
