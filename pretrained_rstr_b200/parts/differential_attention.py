"""Differential attention over the paged cache as a mixer.

Every query head carries two "maps" (q of 2 * dim numbers, laid out [map 1 | map 2]; keys
likewise per key/value head); each map is a softmax attention of its own over the SAME
values, and the head's result is

    o = a1 - lambda a2,    o <- o / sqrt(mean(o^2) + eps) * out_scale

with one lambda per layer (computed from the layer's tensors when the model is built).
Query head h uses key/value head h // (heads / kv_heads).  Rotary positions act on the first
``rot_dims`` coordinates of every map of q and k.  With ``block`` a query sees only keys of
its own block of ``block`` absolute positions (and not later ones); without, all earlier keys.

The cache holds ONE row per (token, key/value head): [k map 1 | k map 2 | v], so key sizes
and value sizes need not be equal and one page look-up serves both (a group with one pool
per layer).  Q, K and V are one matrix product whose 32-bit result is rotated unrounded.
Sizes, the scale, lambda's constant, the block, the rotation's base and reach, eps and the
final factor are parameters.
"""
from __future__ import annotations

import math

import torch

from ..csrc import ops
from .interfaces import KVSpec, LayerCache, Mixer
from .latent_attention import FusedInput
from .linear import padded_linear
from .positions_rotary import rotary_frequencies
from .registry import register_part


class DifferentialAttention(Mixer):
    graph_safe = True
    can_overwrite = True
    accepts_lazy_norm = True      # the first matrix product may compute the norm itself

    def __init__(self, p: dict, store, runtime):
        w = p["weights"]
        self.width, self.heads, self.kv_heads = int(p["width"]), int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.rot_dims = int(p.get("rot_dims", 0))
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        self.block = int(p.get("block") or 0)
        self.out_scale = float(p.get("out_scale", 1.0))
        self.runtime = runtime
        if self.heads % self.kv_heads:
            raise ValueError(f"differential_attention: {self.heads} query heads are not a multiple "
                             f"of {self.kv_heads} key/value heads")
        if self.rot_dims % 2 or self.rot_dims > self.dim:
            raise ValueError(f"differential_attention: {self.rot_dims} rotated coordinates of {self.dim}")
        if self.vdim > 512:
            raise ValueError("differential_attention: value heads wider than 512 are not built")

        def need(name, shape):
            t = store.get(w[name])
            if tuple(t.shape) != tuple(shape):
                raise ValueError(f"{w[name]}: expected {list(shape)}, found {list(t.shape)}")
            return t

        self.input = FusedInput(self.width, runtime, "diff_in")
        self.input.add("q", need("q", (self.heads * 2 * self.dim, self.width)))
        self.input.add("k", need("k", (self.kv_heads * 2 * self.dim, self.width)))
        self.input.add("v", need("v", (self.kv_heads * self.vdim, self.width)))
        self.out = padded_linear(need("out", (self.width, self.heads * self.vdim)), runtime)
        # lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + constant: one number, known at load time
        lam = float(p.get("lambda_init", 0.0))
        if w.get("lambda_q1"):
            vec = [need(n, (self.dim,)).to(torch.float64) for n in
                   ("lambda_q1", "lambda_k1", "lambda_q2", "lambda_k2")]
            lam += math.exp(float((vec[0] * vec[1]).sum())) - math.exp(float((vec[2] * vec[3]).sum()))
        self.lam = lam
        self.freq = rotary_frequencies(float(p.get("rot_base", 10000.0)), self.rot_dims,
                                       runtime.device)
        # rows a CTA of the tiled kernel takes (0: the kernel of a CTA per (token, head))
        self.tile_rows = ops.diff_attention_tile_rows(self.heads, self.kv_heads, self.dim, self.vdim) \
            if torch.cuda.is_available() else 0
        self.single_warps = ops.diff_attention_single_warps(self.heads, self.kv_heads, self.dim,
                                                            self.vdim) if torch.cuda.is_available() else 0
        self.sm_count = ops.sm_count() if torch.cuda.is_available() else 148

    def _single_pays(self, tokens: int) -> bool:
        """The single-token kernel where it has all its warps (the keys it stages at once fit
        shared memory eight warps wide), or while its CTAs are few enough to run at once;
        else single tokens go to the tiled kernel, a row a CTA (measured at 64 tokens, heads of
        128 + 128 over 5 key/value heads: 4.9 against 5.6 ms a step)."""
        if self.single_warps <= 0:
            return False
        parts = -(-(self.heads // self.kv_heads) // 4)
        return self.single_warps >= 6 or tokens * self.kv_heads * parts <= 2 * self.sm_count

    def kv_spec(self) -> KVSpec:
        return KVSpec(self.kv_heads, 2 * self.dim + self.vdim, None, values=False)

    def fuse_input_rows(self, name: str, weight) -> str:
        return self.input.add(name, weight)

    def fused_rows(self, name: str):
        return self.input.view(self._proj, name)

    def forward(self, ctx, h, x, cache: LayerCache, accumulate: bool = True) -> None:
        t = x.shape[0]
        cap = ctx.token_capacity
        group = ctx.groups[cache.group]
        proj = self._proj = self.input.run(ctx, h)
        cols = self.input.cols
        q = ctx.scratch("diff_q", (cap, self.heads * 2 * self.dim), torch.float32)[:t]
        ops.diff_prepare(q, cache.k, proj, cols["q"][0], cols["k"][0], cols["v"][0],
                         group.slots if cache.writes else None, ctx.positions, self.freq,
                         self.heads, self.kv_heads, self.dim, self.vdim, self.rot_dims, ctx.status)
        o = ctx.scratch_zero("diff_out", (cap, self.out.n_in), self.runtime.dtype)[:t]
        # a step of single tokens: a CTA per (token, key/value head) whose warps share the keys;
        # portions of prompts: as many consecutive rows as the tiled kernel takes, which share
        # every key they stage
        # (both kernels take any step; a step replayed from a graph keeps the choice of the step
        # that was recorded)
        single = ctx.max_q_len == 1 or ctx.layout.t_cap <= ctx.layout.b_cap
        ops.diff_attention(o, q, cache.k, group.block_table, ctx.seq_of_token, ctx.positions,
                           self.heads, self.dim, self.vdim, self.block, self.scale, self.lam,
                           self.eps, self.out_scale, ctx.status,
                           tile_rows=min(self.tile_rows, 1) if single else self.tile_rows,
                           single=single and self._single_pays(ctx.layout.t_cap))
        self.out.forward(ctx, o, x, resid=x if accumulate else None)


register_part("mixer", "differential_attention",
              lambda p, store, rt: DifferentialAttention(p, store, rt))
