"""Retention as a mixer: linear attention with one fixed decay per head, no softmax and no
denominator, over a running state instead of cached keys.

Per head, with q, k of ``dim`` and v of ``vdim`` numbers per token (rotary positions on the
first ``rot_dims`` coordinates of q and k, k scaled by ``k_scale`` after the rotation):

    S_t = decay_h S_(t-1) + k_t v_t^T          o_t = S_t^T q_t

then each head's o is brought to unit root-mean-square, the heads are gated by silu(G h)
(``gate``: optional) and projected.  The state [heads, vdim, dim] is 32-bit, starts at zero
and is per-request STATE of the cache manager (a slot per live request), so a prompt may be
cut anywhere and decoding is the same kernel with one token; long portions are cut into
segments that run side by side, joined by the states at their starts.  Projections Q, K, V and G are
one matrix product whose 32-bit result feeds the recurrence unrounded.  Sizes, decays, the
rotation's base and reach, the key scale and eps are parameters.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .interfaces import LayerCache, Mixer, StateSpec
from .latent_attention import FusedInput
from .linear import padded_linear
from .positions_rotary import rotary_frequencies
from .registry import register_part


class Retention(Mixer):
    graph_safe = True
    can_overwrite = True
    accepts_lazy_norm = True      # the first matrix product may compute the norm itself

    def __init__(self, p: dict, store, runtime):
        w = p["weights"]
        self.width, self.heads = int(p["width"]), int(p["heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.rot_dims = int(p.get("rot_dims", 0))
        self.eps = float(p["eps"])
        self.k_scale = float(p.get("k_scale", self.dim ** -0.5))
        self.runtime = runtime
        decay = [float(d) for d in p["decay"]]
        if len(decay) != self.heads:
            raise ValueError(f"retention: {len(decay)} decays for {self.heads} heads")
        if self.rot_dims % 2 or self.rot_dims > self.dim:
            raise ValueError(f"retention: {self.rot_dims} rotated coordinates of {self.dim}")
        if torch.cuda.is_available() and ops.retention_lanes(self.dim) == 0:
            raise ValueError(f"retention: a head size of {self.dim} is beyond the scan kernel's 512")

        def need(name, shape):
            t = store.get(w[name])
            if tuple(t.shape) != tuple(shape):
                raise ValueError(f"{w[name]}: expected {list(shape)}, found {list(t.shape)}")
            return t

        self.input = FusedInput(self.width, runtime, "retention_in")
        self.input.add("q", need("q", (self.heads * self.dim, self.width)))
        self.input.add("k", need("k", (self.heads * self.dim, self.width)))
        self.input.add("v", need("v", (self.heads * self.vdim, self.width)))
        self.gated = bool(w.get("gate"))
        if self.gated:
            self.input.add("gate", need("gate", (self.heads * self.vdim, self.width)))
        self.out = padded_linear(need("out", (self.width, self.heads * self.vdim)), runtime)
        dev = runtime.device
        self.decay = torch.tensor(decay, dtype=torch.float64).to(torch.float32).to(dev)
        self.freq = rotary_frequencies(float(p.get("rot_base", 10000.0)), self.rot_dims, dev)
        self.sm_count = ops.sm_count() if torch.cuda.is_available() else 148
        self.one_launch = torch.cuda.is_available() and ops.retention_step_supports(self.dim, self.vdim)

    def state_specs(self):
        return [StateSpec("retention", (self.heads, self.vdim, self.dim), torch.float32)]

    def fuse_input_rows(self, name: str, weight) -> str:
        return self.input.add(name, weight)

    def fused_rows(self, name: str):
        return self.input.view(self._proj, name)

    def _columns_per_cta(self, requests: int) -> int:
        """Value columns a CTA of the scan takes: all of a head's while that fills the GPU
        twice over, else halves down to 8 (a column's result does not depend on the split)."""
        cols = self.vdim
        while cols > 8 and self.heads * requests * -(-self.vdim // cols) < 2 * self.sm_count:
            cols = -(-cols // 2)
        return cols

    def forward(self, ctx, h, x, cache: LayerCache, accumulate: bool = True) -> None:
        t = x.shape[0]
        cap = ctx.token_capacity
        proj = self._proj = self.input.run(ctx, h)
        cols = self.input.cols
        requests = ctx.layout.b_cap
        gated = ctx.scratch_zero("retention_gated", (cap, self.out.n_in), self.runtime.dtype)[:t]
        if ctx.layout.t_cap <= ops.retention_segment() and self.one_launch:
            # a step of few tokens: rotation, recurrence and finish in one launch
            ops.retention_step(gated, proj, cols["q"][0], cols["k"][0], cols["v"][0],
                               cols["gate"][0] if self.gated else -1, cache.state["retention"],
                               ctx.q_start, ctx.state_slot, ctx.positions, self.decay, self.freq,
                               requests, self.heads, self.dim, self.vdim, self.rot_dims,
                               self.k_scale, self.eps, ctx.status)
            self.out.forward(ctx, gated, x, resid=x if accumulate else None)
            return
        raw = ctx.scratch("retention_raw", (cap, self.heads * self.vdim), torch.float32)[:t]
        # a step with room for more tokens than a segment: portions are cut into segments that
        # run side by side (workspaces sized once, for the largest step the runtime takes)
        segments = None
        if ctx.layout.t_cap > ops.retention_segment():
            n = ops.retention_max_segments(max(ctx.runtime.max_batched_tokens, ctx.layout.t_cap),
                                           max(ctx.runtime.max_requests, requests))
            shape = (n, self.heads, self.vdim, self.dim)
            segments = (ctx.scratch("retention_seg_own", shape, torch.float32),
                        ctx.scratch("retention_seg_start", shape, torch.float32))
        lists = n if segments else requests
        ops.retention_scan(raw, proj, cols["q"][0], cols["k"][0], cols["v"][0],
                           cache.state["retention"], ctx.q_start, ctx.state_slot, ctx.positions,
                           self.decay, self.freq, requests, self.heads, self.dim, self.vdim,
                           self.rot_dims, self.k_scale, self._columns_per_cta(lists), ctx.status,
                           segments=segments)
        ops.retention_finish(gated, raw, proj if self.gated else None,
                             cols["gate"][0] if self.gated else 0, ctx.seq_of_token, self.heads,
                             self.vdim, self.eps)
        self.out.forward(ctx, gated, x, resid=x if accumulate else None)


register_part("mixer", "retention", lambda p, store, rt: Retention(p, store, rt))
