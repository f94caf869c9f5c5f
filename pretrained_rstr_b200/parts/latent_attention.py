"""Causal attention over one low-rank latent per token (``latent_attention``).

Per token the mixer keeps ONE row that all heads share: the normed latent c (``kv_rank``
numbers) from which a head's keys and values would be expanded, k_h = Uk_h c and
v_h = Uv_h c, and a rotated key part r (``rot_dim`` numbers) common to the heads.  Queries
pass a latent of their own: q = Uq norm(Dq h), per head [``dim`` plain | ``rot_dim`` rotated].
The score of head h is (q_plain . k_h + q_rot . r) * scale; a learned sink per head may join
the softmax's denominator; a head's result may be gated by sigmoid(G h)_h; the output
projection follows.

Nothing is expanded per key.  The query is folded through Uk once per token,
qa_h = [Uk_h^T q_plain | q_rot], so that the score is qa_h . [c | r] and the head's result
Uv_h (sum_j w_j c_j): the attention kernels read one row of ``kv_rank + rot_dim`` numbers per
key for all heads, which is what the cache holds (a group with one pool per layer and one
"head").  Sizes, the rotation's base and reach, the scale, the sink and the gate are
parameters.

The first matrix product carries Dq, Dkv and G in one, and whatever rows an arrangement
asks to ride along (:meth:`fuse_input_rows`); its float32 result feeds the norms unrounded.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..csrc import ops
from .interfaces import KVSpec, LayerCache, Mixer
from .linear import Linear
from .registry import register_part


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


class FusedInput:
    """One matrix product for several consumers of the same input: segments of rows, each
    starting at a multiple of 8 columns of the float32 result.  Segments are added while the
    model is built; the matrix is put together at the first use."""

    def __init__(self, width: int, runtime, key: str):
        self.width, self.runtime, self.key = width, runtime, key
        self._parts: List[Tuple[str, torch.Tensor]] = []
        self.cols: Dict[str, Tuple[int, int]] = {}          # name -> (first column, columns)
        self._linear: Optional[Linear] = None

    def add(self, name: str, weight: torch.Tensor) -> str:
        if self._linear is not None:
            raise RuntimeError("the fused product is built already")
        if weight.dim() != 2 or weight.shape[1] != self.width:
            raise ValueError(f"{name}: expected [rows, {self.width}], found {list(weight.shape)}")
        self._parts.append((name, weight))
        return name

    def linear(self) -> Linear:
        if self._linear is None:
            rows, at = [], 0
            for name, w in self._parts:
                self.cols[name] = (at, w.shape[0])
                rows.append(w.to(self.runtime.dtype))
                pad = _pad8(w.shape[0]) - w.shape[0]
                if pad:
                    rows.append(torch.zeros((pad, self.width), dtype=self.runtime.dtype,
                                            device=w.device))
                at += w.shape[0] + pad
            self._linear = Linear(torch.cat(rows, dim=0), None, self.runtime)
            self._parts = []
        return self._linear

    def run(self, ctx, h) -> torch.Tensor:
        lin = self.linear()
        t = h.shape[0]
        out = ctx.scratch(self.key, (ctx.token_capacity, lin.n_out), torch.float32)[:t]
        lin.forward(ctx, h, out)
        return out

    def view(self, out: torch.Tensor, name: str) -> torch.Tensor:
        at, n = self.cols[name]
        return out[:, at:at + n]


class LatentAttention(Mixer):
    graph_safe = True
    can_overwrite = True

    def __init__(self, p: dict, store, runtime):
        w = p["weights"]
        self.width, self.heads, self.dim = p["width"], p["heads"], p["dim"]
        self.rot_dim, self.vdim = p["rot_dim"], p["vdim"]
        self.rank, self.q_rank = p["kv_rank"], p["q_rank"]
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        self.rot_dims, self.window = int(p.get("rot_dims", self.rot_dim)), p.get("window")
        self.runtime = runtime
        dtype, dev = runtime.dtype, runtime.device
        hd = self.dim + self.rot_dim

        def need(name, shape):
            t = store.get(w[name])
            if tuple(t.shape) != tuple(shape):
                raise ValueError(f"{w[name]}: expected {list(shape)}, found {list(t.shape)}")
            return t

        self.input = FusedInput(self.width, runtime, "latent_in")
        self.input.add("q", need("q_down", (self.q_rank, self.width)))
        self.input.add("kv", need("kv_down", (self.rank + self.rot_dim, self.width)))
        self.head_gate = bool(p.get("head_gate", False))
        if self.head_gate:
            self.input.add("gate", need("gate", (self.heads, self.width)))
        self.q_norm = need("q_norm", (self.q_rank,)).to(torch.float32).contiguous()
        self.kv_norm = need("kv_norm", (self.rank,)).to(torch.float32).contiguous()
        self.q_up = Linear(need("q_up", (self.heads * hd, self.q_rank)), None, runtime)
        self.uk = need("k_up", (self.heads * self.dim, self.rank)).to(dtype).contiguous()
        # the value expansion with the latent axis outermost: a thread per value coordinate
        # then reads neighbouring numbers
        self.uvt = need("v_up", (self.heads * self.vdim, self.rank)).to(dtype) \
            .reshape(self.heads, self.vdim, self.rank).transpose(1, 2).contiguous()
        self.sinks = need("sink", (self.heads,)).to(torch.float32).contiguous() \
            if p.get("sink", False) else None
        self.out = Linear(need("out", (self.width, self.heads * self.vdim)), None, runtime)
        half = self.rot_dims // 2
        base = float(p.get("rot_base", 10000.0))
        self.freq = torch.tensor([base ** (-2.0 * i / self.rot_dims) for i in range(half)] or [0.0],
                                 dtype=torch.float64).to(torch.float32).to(dev)

    # ------------------------------------------------------------------ structure
    def kv_spec(self) -> KVSpec:
        return KVSpec(1, self.rank + self.rot_dim, self.window, values=False)

    def fuse_input_rows(self, name: str, weight: torch.Tensor) -> str:
        """Rows that read the mixer's input and ride along in its first product; their float32
        result is ``fused_rows(name)`` after :meth:`forward`."""
        return self.input.add(name, weight)

    def fused_rows(self, name: str) -> torch.Tensor:
        return self.input.view(self._proj, name)

    # -------------------------------------------------------------------- forward
    def forward(self, ctx, h, x, cache: LayerCache, accumulate: bool = True) -> None:
        t = x.shape[0]
        cap, dtype = ctx.token_capacity, self.runtime.dtype
        group = ctx.groups[cache.group]
        proj = self._proj = self.input.run(ctx, h)
        cols = self.input.cols
        cq = ctx.scratch("latent_cq", (cap, self.q_rank), dtype)[:t]
        ops.latent_prepare(cq, cache.k, proj, cols["q"][0], cols["kv"][0], self.q_norm,
                           self.kv_norm, group.slots if cache.writes else None, ctx.positions,
                           self.freq, self.q_rank, self.rank, self.rot_dim, self.rot_dims,
                           self.eps, ctx.status)
        q = ctx.scratch("latent_q", (cap, self.q_up.n_out), torch.float32)[:t]
        self.q_up.forward(ctx, cq, q)
        qa = ctx.scratch("latent_qa", (cap, self.heads, self.rank + self.rot_dim),
                         torch.float32)[:t]
        ops.latent_fold(qa, q, self.uk, ctx.positions, self.freq, self.heads, self.dim,
                        self.rot_dim, self.rot_dims, self.rank)
        lat = ctx.scratch("latent_sum", (cap, self.heads, self.rank), torch.float32)[:t]
        attend_latent(ctx, lat, qa, cache, group, self.sinks, self.scale, self.window, self.rank)
        o = ctx.scratch("latent_o", (cap, self.heads * self.vdim), dtype)[:t]
        gate = self.input.view(proj, "gate") if self.head_gate else None
        ops.latent_unfold(o, lat, self.uvt, gate, self.heads, self.rank, self.vdim)
        self.out.forward(ctx, o, x, resid=x if accumulate else None)


def attend_latent(ctx, lat, qa, cache: LayerCache, group, sinks, scale: float,
                  window: Optional[int], rank: int) -> None:
    """lat[t, h] = sum_j w_j c_j over the rows token t sees in its request's pages."""
    ops.latent_attention(lat, qa, cache.k, group.block_table, ctx.seq_of_token, ctx.positions,
                         sinks, scale, window, rank, ctx.status)


register_part("mixer", "latent_attention", lambda p, store, rt: LatentAttention(p, store, rt))
