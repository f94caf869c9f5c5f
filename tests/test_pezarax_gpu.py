"""Pezarax in the engine against the plain implementation (``plain_pezarax``): every mechanism
alone at the kernels' interface, then whole models of several shapes under every way of
cutting and batching the work, in 32-bit and in bfloat16, and greedy generation through the
package's entry point."""
import math
import random

import pytest
import torch

import plain_pezarax as P
from helpers import Replayer, random_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


# --------------------------------------------------------------------------- configurations
def _ret(heads, dim, vdim, decay, mlp, rot_dims=None, base=10000.0):
    return {"type": "retention",
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay,
                      "rot": {"base": base, "dims": dim if rot_dims is None else rot_dims}},
            "mlp": mlp}


def _att(heads, kv_heads, dim, vdim, block, mlp, rot_dims=None, base=10000.0, diff=0.2, scale=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff,
             "scale": scale if scale is not None else 1.0 / math.sqrt(dim), "mask": {"size": block},
             "rot": {"base": base, "dims": dim if rot_dims is None else rot_dims}}
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def _moe(experts, top, ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def _model(vocab, width, layers, loop=None, scale=5.0, logit_scale=1.0, eps=1e-6):
    out = {"architecture": "Pezarax", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "embedding": {"scale": scale}, "logit_scale": logit_scale, "layers": layers}
    if loop:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


# Every size differs from every other one; key and value sizes that differ; heads that are no
# powers of two; a layer without a feed-forward; one, some and all experts chosen; rotations that
# cover a part, all or nothing of a head; blocks shorter and longer than a page and than the
# kernel's key segment; a loop in the middle, a loop from the first layer on, no loop; a model
# without attention (no pages at all) and one whose first layer is attention; two, three and
# eight query heads a key/value head (eight: two CTAs of the single-token kernel a head).
SHAPE_A = _model(300, 64, [
    _ret(2, 16, 24, [0.9, 0.99], _moe(5, 2, 24), rot_dims=8),
    _att(4, 2, 16, 24, 20, _moe(3, 1, 40), rot_dims=12, diff=0.25),
    _ret(4, 8, 16, [0.5, 0.97, 0.999, 1.0], None),
    _att(8, 1, 24, 8, 70, _moe(4, 4, 16), base=300.0, scale=0.3)], loop=(1, 3, 2), logit_scale=0.6)
SHAPE_B = _model(515, 128, [
    _att(3, 1, 40, 56, 300, _moe(6, 3, 24), rot_dims=0, diff=0.4),
    _ret(3, 80, 40, [0.95, 0.995, 0.9995], _moe(2, 1, 72), rot_dims=32, base=77.0),
    _att(6, 3, 8, 136, 64, None, diff=0.1)], scale=3.0, eps=1e-5)
SHAPE_C = _model(200, 48, [
    _ret(3, 16, 16, [0.8, 0.9, 0.99], _moe(4, 2, 8)),
    _ret(1, 48, 32, [0.98], _moe(3, 2, 16), rot_dims=16)], loop=(0, 2, 3), scale=9.0, logit_scale=2.0)
SHAPES = {"A": (SHAPE_A, 21), "B": (SHAPE_B, 22), "C": (SHAPE_C, 23)}
CASES = [(name, dtype) for name in SHAPES for dtype in ("float32", "bfloat16")]
TOL = {"float32": 2e-4, "bfloat16": 4e-2}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from pretrained_rstr_b200.config.registry import lookup
    from pretrained_rstr_b200.weights import make_random_model
    from pretrained_rstr_b200.weights.safetensors_io import save_file
    out = {}
    for name, (raw, seed) in SHAPES.items():
        cfg = lookup(raw).config_class.from_dict(raw)
        for dtype in ("float32", "bfloat16"):
            path = str(tmp_path_factory.mktemp(f"pezarax{name}_{dtype}"))
            make_random_model(path, cfg, seed, torch.bfloat16 if dtype == "bfloat16" else torch.float32)
            # decisive routers: fewer tokens whose choice hangs on the last bits
            _, tensors = P.read_folder(path)
            for key in tensors:
                if key.endswith(".router"):
                    tensors[key] = tensors[key] * 3.0
            save_file(tensors, path + "/model.safetensors")
            out[(name, dtype)] = path
    return out


# A router's choice between two experts whose logits lie this close may fall either way once
# the stream is rounded to bfloat16 (float32: to its last bits); such a token's row, a
# legitimate other model's, is not compared, and a row after it in its request (which sees it
# through the state or the cache) that misses the tolerance is excused; both kinds together
# stay a small share of all rows, and a row with no close call before it is never excused.
CLOSE = {"float32": 1e-3, "bfloat16": 0.25}
# The same for a retention head whose sum over earlier tokens all but cancels (at a sequence's
# first token it is (q . k) v, whose sign hangs on q . k): the unit norm that follows blows
# rounding up.  Below this share of its uncancelled size the token counts as a close call.
DELICATE = {"float32": 1e-4, "bfloat16": 0.03}


class Oracle(dict):
    pass


def _oracle(folder, prompts, dtype="float32"):
    cfg, tensors = P.read_folder(folder)
    out = Oracle()
    out.close = {}
    for rid, ids in prompts.items():
        gaps, ratios = [], []
        out[rid] = P.forward(list(ids), tensors, cfg, margins=gaps, delicate=ratios).to(torch.float32)
        close = torch.zeros(len(ids), dtype=torch.bool)
        if gaps:
            close |= torch.stack(gaps).min(0).values < CLOSE[dtype]
        if ratios:
            close |= torch.stack(ratios).min(0).values < DELICATE[dtype]
        out.close[rid] = close
    return out


def row_error(row, ref) -> float:
    """Root mean square of the difference (its mean taken off) over that of the reference row."""
    d = row.double() - ref.double()
    d = d - d.mean()
    r = ref.double() - ref.double().mean()
    return float(d.pow(2).mean().sqrt() / r.pow(2).mean().sqrt())


def compare(rows, oracle, tol):
    assert rows
    worst, skipped = 0.0, 0
    for (rid, pos), row in sorted(rows.items()):
        err = row_error(row, oracle[rid][pos])
        assert err == err, f"NaN at request {rid} position {pos}"
        close = oracle.close[rid]
        if bool(close[pos]):
            skipped += 1
            continue
        if err > tol and bool(close[:pos].any()):
            skipped += 1
            continue
        assert err <= tol, (f"request {rid} position {pos} (page offset {pos % 64}): relative "
                            f"difference {err:.3e} > {tol:.1e}")
        worst = max(worst, err)
    assert skipped <= 0.3 * len(rows), "too many close router calls for the test to mean much"
    return worst


def _prompts(name, lengths, salt=0):
    raw, seed = SHAPES[name]
    return {f"r{i}": random_tokens(n, raw["vocab"], 1000 * seed + salt + i) for i, n in enumerate(lengths)}


def _i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


# ------------------------------------------------------------------ mechanisms, one by one
def test_scaled_embedding_kernel():
    from pretrained_rstr_b200.csrc import ops
    g = torch.Generator().manual_seed(1)
    table = torch.randn(40, 24, generator=g)
    ids = random_tokens(11, 40, 2)
    want = P.embed(ids, {"embed": table}, {"embedding": {"scale": 3.5}}, torch.float32)
    for dtype in (torch.float32, torch.bfloat16):
        out, keep = torch.empty(11, 24, device=DEV), torch.empty(16, 24, device=DEV)
        ops.embed_scaled(out, _i32(ids), table.to(dtype).to(DEV), 3.5, keep=keep)
        ref = want if dtype == torch.float32 else table.to(dtype).float()[torch.tensor(ids)] * 3.5
        assert torch.equal(out.cpu(), ref) and torch.equal(keep.cpu()[:11], ref)


def test_router_and_expert_activation_kernels():
    """Scores, the choice of one, some and all experts, weights that are the scores themselves
    (or renormalised), and the activation with the weight inside (or outside)."""
    from pretrained_rstr_b200.csrc import ops
    g = torch.Generator().manual_seed(3)
    t, n_e, ff = 9, 6, 10
    logits = torch.randn(t, n_e + 5, generator=g) * 2
    z = logits[:, 3:3 + n_e]
    for top in (1, 2, 6):
        weights = torch.empty(t, n_e, device=DEV)
        chosen = torch.empty(t, top, dtype=torch.int32, device=DEV)
        chosen_w = torch.empty(t, top, device=DEV)
        ops.route_scores(weights, chosen, chosen_w, logits.to(DEV)[:, 3:3 + n_e], None, top)
        val, idx = torch.topk(torch.sigmoid(z), top, dim=-1)
        assert torch.equal(chosen.cpu().long(), idx)
        assert torch.allclose(chosen_w.cpu(), val, atol=1e-6)
        assert torch.allclose(weights.cpu(), torch.zeros(t, n_e).scatter(1, idx, val), atol=1e-6)
        ops.route_scores(weights, chosen, chosen_w, logits.to(DEV)[:, 3:3 + n_e], None, top,
                         renormalize=True)
        assert torch.allclose(chosen_w.cpu(), val / val.sum(-1, keepdim=True), atol=1e-6)
    # logits so large that their sigmoids all round to 1: the order of the logits decides
    big = torch.tensor([[40.0, 45.0, 30.0, -3.0, 44.0, 20.0]], device=DEV)
    w1, c1, cw1 = torch.empty(1, 6, device=DEV), torch.empty(1, 2, dtype=torch.int32, device=DEV), torch.empty(1, 2, device=DEV)
    ops.route_scores(w1, c1, cw1, big, None, 2)
    assert c1.cpu().tolist() == [[1, 4]] and cw1.cpu().tolist() == [[1.0, 1.0]]
    act = torch.zeros(1, 16, device=DEV)
    ops.route_act(act, torch.cat([torch.ones(1, 12, device=DEV), big], dim=1), 0, 12, 6, 2, 2, weights_out=w1)
    assert w1.cpu().tolist() == [[0.0, 1.0, 0.0, 0.0, 1.0, 0.0]]
    for xt in (torch.float32, torch.bfloat16):                   # the router's own product
        x, w = torch.randn(t, 32, generator=g).to(xt), torch.randn(n_e, 32, generator=g).to(xt)
        ops.route_scores(weights, chosen, chosen_w, x.to(DEV), w.to(DEV), 6, score="identity")
        val, idx = torch.topk(x.double() @ w.double().T, 6, dim=-1)
        assert torch.equal(chosen.cpu().long(), idx)
        assert torch.allclose(chosen_w.cpu().double(), val, atol=1e-4)
    weights = torch.rand(t, n_e, generator=g)
    weights[:, ::2] = 0.0
    for n_cols, col in ((n_e * ff, 4), (n_e * ff, 5)):           # 16-byte and single loads
        inp = torch.randn(t, n_cols + 8, generator=g)
        u = inp[:, col:col + n_cols]
        wide = weights.repeat_interleave(ff, dim=1)
        for act, fn in (("relu_squared", lambda v: torch.relu(v) ** 2), ("silu", lambda v: v * torch.sigmoid(v))):
            for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 2e-2)):
                out = torch.full((t, n_cols + 8), 7.0, dtype=dtype, device=DEV)
                ops.routed_act(out, inp.to(DEV), col, n_cols, weights.to(DEV), ff, act)
                want = torch.where(wide != 0, fn(wide * u), torch.zeros_like(u))
                assert torch.allclose(out.cpu().float()[:, :n_cols], want, atol=tol, rtol=tol)
                ops.routed_act(out, inp.to(DEV), col, n_cols, weights.to(DEV), ff, act, weight_on="output")
                assert torch.allclose(out.cpu().float()[:, :n_cols], wide * fn(u), atol=tol, rtol=tol)


def test_router_and_activation_in_one_launch():
    """The fused kernel against the two it replaces, with and without 16-byte loads."""
    from pretrained_rstr_b200.csrc import ops
    g = torch.Generator().manual_seed(13)
    for t, n_e, ff, top, col in ((9, 6, 12, 2, 8), (5, 3, 10, 1, 4), (40, 16, 24, 16, 4)):
        inp = (torch.randn(t, col + n_e * ff + 8 + n_e, generator=g) * 2).to(DEV)
        rcol = col + n_e * ff + 8
        weights = torch.empty(t, n_e, device=DEV)
        chosen = torch.empty(t, top, dtype=torch.int32, device=DEV)
        chosen_w = torch.empty(t, top, device=DEV)
        ops.route_scores(weights, chosen, chosen_w, inp[:, rcol:rcol + n_e], None, top)
        for dtype in (torch.float32, torch.bfloat16):
            want = torch.full((t, n_e * ff + 8), 3.0, dtype=dtype, device=DEV)
            got = torch.full((t, n_e * ff + 8), 3.0, dtype=dtype, device=DEV)
            w2 = torch.empty(t, n_e, device=DEV)
            ops.routed_act(want, inp, col, n_e * ff, weights, ff)
            ops.route_act(got, inp, col, rcol, n_e, top, ff, weights_out=w2)
            assert torch.equal(got, want) and torch.equal(w2, weights)


class RetentionCase:
    """Hand-made q, k, v (and gate) rows behind a stand-in for the fused projection."""

    def __init__(self, heads, dim, vdim, rot_dims, base, decay, seed=0):
        self.heads, self.dim, self.vdim, self.rot_dims, self.base = heads, dim, vdim, rot_dims, base
        self.decay = decay
        self.g = torch.Generator().manual_seed(seed)
        self.state = torch.full((3, heads, vdim, dim), 9.0, device=DEV)     # what earlier users left
        self.k_scale = dim ** -0.5

    def rows(self, n):
        r = lambda w: torch.randn(n, self.heads, w, generator=self.g)
        return r(self.dim), r(self.dim), r(self.vdim), r(self.vdim)

    def plain(self, q, k, v, gate, eps):
        pos = torch.arange(q.shape[0])
        qr = P.rotate_half(q.double(), pos, self.base, self.rot_dims)
        kr = P.rotate_half(k.double(), pos, self.base, self.rot_dims) * self.k_scale
        o, _ = P.decayed_states(qr, kr, v.double(), self.decay)
        gd = gate.double()
        return P.unit_rms(o, eps) * gd * torch.sigmoid(gd)

    def run(self, parts, eps, cols, out_dtype=torch.float32, segmented=False, one_launch=False):
        """parts: (slot, first position, q, k, v, gate) per request of one step; ``segmented``:
        portions cut into segments that run side by side; ``one_launch``: rotation, recurrence
        and finish in one kernel."""
        from pretrained_rstr_b200.csrc import ops
        from pretrained_rstr_b200.parts.positions_rotary import rotary_frequencies
        h, d, vd = self.heads, self.dim, self.vdim
        proj, pos, seq, qs, slots = [], [], [], [0], []
        for b, (slot, p0, q, k, v, gate) in enumerate(parts):
            n = q.shape[0]
            pad = torch.zeros(n, 4)
            proj.append(torch.cat([pad, q.reshape(n, -1), k.reshape(n, -1), pad, v.reshape(n, -1),
                                   gate.reshape(n, -1)], dim=1))
            pos += list(range(p0, p0 + n))
            seq += [b] * n
            qs.append(qs[-1] + n)
            slots.append(slot)
        proj = torch.cat(proj).to(DEV).contiguous()
        t = proj.shape[0]
        raw = torch.empty(t, h * vd, device=DEV)
        status = torch.zeros(4, dtype=torch.int32, device=DEV)
        decay = torch.tensor(self.decay, dtype=torch.float32, device=DEV)
        freq = rotary_frequencies(self.base, self.rot_dims, DEV)
        if one_launch:
            assert ops.retention_step_supports(d, vd)
            out = torch.zeros(t, h * vd + 8, dtype=out_dtype, device=DEV)
            ops.retention_step(out, proj, 4, 4 + h * d, 8 + 2 * h * d, 8 + 2 * h * d + h * vd, self.state,
                               _i32(qs + [qs[-1]]), _i32(slots + [0]), _i32(pos), decay, freq,
                               len(parts) + 1, h, d, vd, self.rot_dims, self.k_scale, eps, status)
            assert int(status[0]) == 0
            return out.cpu().double()[:, :h * vd].reshape(t, h, vd)
        segments = None
        if segmented:
            n = ops.retention_max_segments(t, len(parts) + 1)
            segments = (torch.full((n, h, vd, d), 7.0, device=DEV), torch.full((n + 2, h, vd, d), 7.0, device=DEV))
        ops.retention_scan(raw, proj, 4, 4 + h * d, 8 + 2 * h * d, self.state, _i32(qs + [qs[-1]]),
                           _i32(slots + [0]), _i32(pos), decay, freq, len(parts) + 1, h, d, vd,
                           self.rot_dims, self.k_scale, cols, status, segments=segments)
        assert int(status[0]) == 0
        out = torch.zeros(t, h * vd + 8, dtype=out_dtype, device=DEV)
        ops.retention_finish(out, raw, proj, 8 + 2 * h * d + h * vd, _i32(seq), h, vd, eps)
        return out.cpu().double()[:, :h * vd].reshape(t, h, vd)


@pytest.mark.parametrize("heads,dim,vdim,rot_dims", [(3, 16, 24, 8), (2, 80, 40, 80), (1, 8, 136, 0),
                                                    (2, 64, 64, 64), (1, 160, 16, 32)])
def test_retention_kernels(heads, dim, vdim, rot_dims):
    """A whole sequence at once, in portions down to one token, beside another request, in any
    split of the value columns over CTAs; a slot's earlier state is not read at position 0."""
    from pretrained_rstr_b200.csrc import ops
    decay = [1.0 - 2.0 ** -(3 + 2 * j) for j in range(heads)]
    case = RetentionCase(heads, dim, vdim, rot_dims, 50.0, decay, seed=heads)
    n = 90
    q, k, v, gate = case.rows(n)
    q2, k2, v2, gate2 = case.rows(37)
    want, want2 = case.plain(q, k, v, gate, 1e-5), case.plain(q2, k2, v2, gate2, 1e-5)
    got = case.run([(1, 0, q, k, v, gate)], 1e-5, cols=vdim)
    assert torch.allclose(got, want, atol=2e-5, rtol=2e-5)
    # segments side by side: a portion of one full segment and a rest, one of exactly two, a
    # short one, and a continuation from a carried state
    q3, k3, v3, gate3 = case.rows(128)
    want3 = case.plain(q3, k3, v3, gate3, 1e-5)
    got = case.run([(1, 0, q[:70], k[:70], v[:70], gate[:70]), (2, 0, q3, k3, v3, gate3),
                    (0, 0, q2[:5], k2[:5], v2[:5], gate2[:5])], 1e-5, cols=7, segmented=True)
    assert torch.allclose(got[:70], want[:70], atol=2e-5, rtol=2e-5)
    assert torch.allclose(got[70:198], want3, atol=2e-5, rtol=2e-5)
    assert torch.allclose(got[198:], want2[:5], atol=2e-5, rtol=2e-5)
    got = case.run([(0, 5, q2[5:], k2[5:], v2[5:], gate2[5:]), (1, 70, q[70:], k[70:], v[70:], gate[70:])],
                   1e-5, cols=vdim, segmented=True)
    assert torch.allclose(got[:32], want2[5:], atol=2e-5, rtol=2e-5)
    assert torch.allclose(got[32:], want[70:], atol=2e-5, rtol=2e-5)
    at, outs = 0, []
    for size in (1, 2, 17, 1, 33, 16, 20):
        # a portion of the request; beside it, before or after, a fresh request in another slot
        part = (1, at, q[at:at + size], k[at:at + size], v[at:at + size], gate[at:at + size])
        m = 1 + at % 7
        other = (2, 0, q2[:m], k2[:m], v2[:m], gate2[:m])
        parts = [other, part] if at % 2 else [part, other]
        got = case.run(parts, 1e-5, cols=8 if size % 2 else 5,
                       one_launch=size in (2, 16, 20) and ops.retention_step_supports(dim, vdim))
        r0 = m if at % 2 else 0
        outs.append(got[r0:r0 + size])
        other_rows = got[:m] if at % 2 else got[size:]
        assert torch.allclose(other_rows, want2[:m], atol=2e-5, rtol=2e-5)
        at += size
    assert at == n
    assert torch.allclose(torch.cat(outs), want, atol=2e-5, rtol=2e-5)
    out16 = case.run([(0, 0, q2, k2, v2, gate2)], 1e-5, cols=16, out_dtype=torch.bfloat16)
    assert torch.allclose(out16, want2, atol=3e-2, rtol=3e-2)


def test_retention_far_token_stands_out():
    """One key far back, made large, among hundreds: with a slow decay it still carries the
    result, through a portion's start and through single tokens, and with a fast decay it is
    gone; a wrong decay, a lost state or a key scaled twice would show."""
    case = RetentionCase(2, 16, 16, 16, 10000.0, [0.999, 0.9], seed=9)
    n, far = 400, 3
    q, k, v, gate = case.rows(n)
    k[far] *= 30.0
    v[far] *= 5.0
    want = case.plain(q, k, v, gate, 1e-6)
    outs, at = [], 0
    for size in [130, 64, 2, 190] + [1] * 14:
        outs.append(case.run([(0, at, q[at:at + size], k[at:at + size], v[at:at + size],
                               gate[at:at + size])], 1e-6, cols=16, segmented=size > 64))
        at += size
    got = torch.cat(outs)
    assert at == n and torch.allclose(got, want, atol=1e-4, rtol=1e-4)
    k[far] /= 30.0
    v[far] /= 5.0
    plain_far = case.plain(q, k, v, gate, 1e-6)
    assert float((want[-1, 0] - plain_far[-1, 0]).abs().max()) > 0.1      # decay 0.999: it counts
    assert float((want[-1, 1] - plain_far[-1, 1]).abs().max()) < 1e-6     # decay 0.9: long gone


class DiffCase:
    """A paged cache of rows [k map 1 | k map 2 | v] filled by hand: requests' rows lie in pages
    taken in a shuffled order from a pool whose other pages hold large numbers."""

    def __init__(self, lengths, kv_heads, dim, vdim, dtype, page=64, seed=0, fill=40.0):
        g = torch.Generator().manual_seed(seed)
        self.kv_heads, self.dim, self.vdim, self.page, self.dtype = kv_heads, dim, vdim, page, dtype
        row = 2 * dim + vdim
        need = sum(-(-n // page) for n in lengths)
        pages = list(range(need + 3))
        random.Random(seed).shuffle(pages)
        self.rows = [(torch.randn(n, kv_heads, row, generator=g) * 0.5).to(dtype).float() for n in lengths]
        self.max_pages = max(-(-n // page) for n in lengths) + 1
        cache = torch.full((need + 3, kv_heads, page, row), fill)
        table = torch.full((len(lengths), self.max_pages), -1, dtype=torch.int32)
        for b, n in enumerate(lengths):
            for li in range(-(-n // page)):
                pg = pages.pop()
                table[b, li] = pg
                m = min(page, n - li * page)
                cache[pg, :, :m] = self.rows[b][li * page:li * page + m].transpose(0, 1)
        self.cache, self.table = cache.to(dtype).to(DEV), table.to(DEV)

    def run(self, queries, heads, block, scale, lam, eps, factor, tile_rows=0):
        """queries: (request, position, q [heads, 2, dim]); returns kernel and plain results.
        ``tile_rows``: 0 the kernel of a CTA per (token, head), -1 the single-token kernel, else
        the tiled kernel."""
        from pretrained_rstr_b200.csrc import ops
        n = len(queries)
        q = torch.stack([x for _, _, x in queries]).reshape(n, -1).to(DEV).contiguous()
        out = torch.full((n, heads * self.vdim + 8), float("nan"), dtype=self.dtype, device=DEV)
        status = torch.zeros(4, dtype=torch.int32, device=DEV)
        ops.diff_attention(out, q, self.cache, self.table, _i32([b for b, _, _ in queries]),
                           _i32([p for _, p, _ in queries]), heads, self.dim, self.vdim, block,
                           scale, lam, eps, factor, status, tile_rows=max(tile_rows, 0),
                           single=tile_rows < 0)
        assert int(status[0]) == 0, status.tolist()
        want = []
        for b, p, x in queries:
            lo = (p // block) * block if block else 0
            rows = self.rows[b][lo:p + 1].double()
            k = rows[:, :, :2 * self.dim].reshape(-1, self.kv_heads, 2, self.dim)
            v = rows[:, :, 2 * self.dim:]
            mask = torch.ones(1, p - lo + 1, dtype=torch.bool)
            want.append(P.two_map_attention(x.double()[None], k, v, mask, scale, lam, eps, factor)[0])
        got = out.cpu().double()[:, :heads * self.vdim].reshape(n, heads, self.vdim)
        return got, torch.stack(want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("block", [0, 20, 64, 300])
@pytest.mark.parametrize("tile_rows", [-1, 0, 1, 5, 10])
def test_differential_attention_kernel(dtype, block, tile_rows):
    """Random rows; queries at the first tokens, at page borders and on both sides of every
    block border; blocks shorter and longer than a page and than the kernel's key segment; a
    CTA per (token, head), and tiles of rows that may hold runs of consecutive positions, single
    tokens and several requests."""
    heads, kv_heads, dim, vdim = 6, 2, 24, 40
    case = DiffCase([1, 65, 200, 700], kv_heads, dim, vdim, dtype, seed=4)
    g = torch.Generator().manual_seed(8)
    places = {0, 1, 63, 64, 65, 127, 128, 199, 255, 256, 257, 511, 512, 513, 699}
    if block:
        places |= {m * block + o for m in range(1, 700 // block + 1) for o in (-1, 0, 1)}
    queries = [(b, p, torch.randn(heads, 2, dim, generator=g))
               for b, n in enumerate([1, 65, 200, 700]) for p in sorted(places) if p < n]
    got, want = case.run(queries, heads, block, 0.3, 0.7, 1e-6, 0.8, tile_rows=tile_rows)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(got, want, atol=tol, rtol=tol)


@pytest.mark.parametrize("tile_rows", [-1, 0, 4])
@pytest.mark.parametrize("block", [0, 50, 300])
def test_differential_attention_edges_stand_out(block, tile_rows):
    """A key made to dominate map 1 at the first position of a block, and one at the last
    position of the block before: the query just after sees the first and not the second; far
    keys among hundreds count when no block hides them."""
    heads, kv_heads, dim, vdim = 2, 1, 16, 8
    n = 650
    case = DiffCase([n], kv_heads, dim, vdim, torch.float32, seed=6)
    g = torch.Generator().manual_seed(2)
    direction = torch.randn(dim, generator=g)
    direction /= direction.norm()
    edge = (n // block - 1) * block if block else 5            # first position of a late block
    rows = case.rows[0]
    for p, mark in ((edge, 3.0), (edge - 1, -3.0)):
        if p >= 0 and (block or p == edge):
            rows[p, 0, :dim] = direction * 6.0                  # stands out in map 1
            rows[p, 0, 2 * dim:] = mark
    pages = case.table[0].tolist()
    for p in (edge, edge - 1):
        if p >= 0 and (block or p == edge):
            case.cache[pages[p // 64], :, p % 64] = rows[p]
    queries = []
    for p in sorted({edge, edge + 1, min(n - 1, edge + block - 1 if block else n - 1), n - 1}):
        x = torch.randn(heads, 2, dim, generator=g) * 0.1
        x[:, 0] = direction * 6.0
        queries.append((0, p, x))
    got, want = case.run(queries, heads, block, 1.0, 0.5, 1e-6, 1.0, tile_rows=tile_rows)
    assert torch.allclose(got, want, atol=2e-5, rtol=2e-5)
    inside = [i for i, (_, p, _) in enumerate(queries) if not block or p // block == edge // block]
    assert inside and all(float(want[i].mean()) > 0.5 for i in inside)     # the edge key carries it


def test_prepare_rotates_and_caches():
    """Rotation of every map of q and k by the token's position, the cache row's layout, rows
    of other tokens untouched, nothing written for a slot of -1."""
    from pretrained_rstr_b200.csrc import ops
    from pretrained_rstr_b200.parts.positions_rotary import rotary_frequencies
    heads, kv_heads, dim, vdim, rot, page = 3, 1, 16, 24, 12, 8
    g = torch.Generator().manual_seed(5)
    t = 5
    proj = torch.randn(t, 8 + heads * 2 * dim + kv_heads * 2 * dim + kv_heads * vdim, generator=g)
    qc, kc = 8, 8 + heads * 2 * dim
    vc = kc + kv_heads * 2 * dim
    pos = [0, 7, 8, 100, 3]
    slots = [3, 2 * page + 1, -1, page, 0]
    cache = torch.full((3, kv_heads, page, 2 * dim + vdim), 5.0, device=DEV)
    q_out = torch.empty(t, heads * 2 * dim, device=DEV)
    ops.diff_prepare(q_out, cache, proj.to(DEV), qc, kc, vc, _i32(slots), _i32(pos),
                     rotary_frequencies(900.0, rot, DEV), heads, kv_heads, dim, vdim, rot)
    p = torch.tensor(pos)
    want_q = P.rotate_half(proj[:, qc:kc].reshape(t, heads, 2, dim).double(), p, 900.0, rot)
    want_k = P.rotate_half(proj[:, kc:vc].reshape(t, kv_heads, 2, dim).double(), p, 900.0, rot)
    assert torch.allclose(q_out.cpu().double().reshape(t, heads, 2, dim), want_q, atol=1e-5)
    flat = cache.cpu().double()
    touched = set()
    for i, s in enumerate(slots):
        if s < 0:
            continue
        row = flat[s // page, 0, s % page]
        touched.add((s // page, s % page))
        assert torch.allclose(row[:2 * dim], want_k[i, 0].reshape(-1), atol=1e-5)
        assert torch.allclose(row[2 * dim:], proj[i, vc:].double(), atol=1e-6)
    for pg in range(3):
        for off in range(page):
            if (pg, off) not in touched:
                assert float((flat[pg, 0, off] - 5.0).abs().max()) == 0.0


# ------------------------------------------------------------------------ whole models
@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_prompts_decode_and_portions(folders, name, dtype):
    """Whole prompts in one step; the last tokens one by one; portions of several sizes, down
    to two tokens, cut inside pages and blocks."""
    folder = folders[(name, dtype)]
    prompts = _prompts(name, [1, 2, 23, 64, 65, 150, 330])
    oracle = _oracle(folder, prompts, dtype)
    rp = Replayer(folder, dtype, max_tokens=512)
    for rid, ids in prompts.items():
        rp.step([(rid, ids, list(range(len(ids))))], end=[rid])
    compare(rp.rows, oracle, TOL[dtype])
    rp.rows.clear()
    for rid, ids in prompts.items():
        head = max(1, len(ids) - 40)
        rp.step([(rid, ids[:head], [head - 1])], end=[rid] if head == len(ids) else [])
        for i in range(head, len(ids)):
            rp.step([(rid, ids[i:i + 1], [0])], end=[rid] if i == len(ids) - 1 else [])
    compare(rp.rows, oracle, TOL[dtype])
    rp.rows.clear()
    sizes = [3, 2, 19, 2, 2, 40, 5, 64, 2, 66, 2, 130]
    for r, (rid, ids) in enumerate(prompts.items()):
        at, k = 0, r
        while at < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - at)
            k += 1
            rp.step([(rid, ids[at:at + n], list(range(n)))], end=[rid] if at + n >= len(ids) else [])
            at += n
    compare(rp.rows, oracle, TOL[dtype])


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16"), ("C", "float32")])
def test_long_decode(folders, name, dtype):
    """Two tokens of prompt and 200 decoded one by one, across page and block borders."""
    folder = folders[(name, dtype)]
    prompts = _prompts(name, [202], salt=50)
    oracle = _oracle(folder, prompts, dtype)
    rp = Replayer(folder, dtype, max_tokens=256)
    ids = prompts["r0"]
    rp.step([("r0", ids[:2], [0, 1])])
    for i in range(2, len(ids)):
        rp.step([("r0", ids[i:i + 1], [0])])
    compare(rp.rows, oracle, TOL[dtype])


@pytest.mark.parametrize("name,dtype", CASES)
def test_mixed_batches_with_reuse(folders, name, dtype):
    """Up to four live requests of unequal lengths, portions of some beside single tokens of
    others, some left out of a step, in a pool so small that pages and state slots of finished
    requests are used again: every row as if its request ran alone."""
    folder = folders[(name, dtype)]
    lengths = [130, 64, 250, 9, 33, 200, 1, 120, 2, 77]
    prompts = _prompts(name, lengths, salt=90)
    oracle = _oracle(folder, prompts, dtype)
    biggest = sorted((-(-n // 64) * 64 for n in lengths), reverse=True)
    rp = Replayer(folder, dtype, max_tokens=sum(biggest[:4]))
    rng = random.Random(5)
    waiting, live, slots_seen = list(prompts), {}, []
    while waiting or live:
        while waiting and len(live) < 4:
            live[waiting.pop(0)] = 0
        entries, end = [], []
        for rid in list(live):
            ids, at = prompts[rid], live[rid]
            left = len(ids) - at
            if rng.random() < 0.25 and len(live) > 1:
                continue                                   # left out of this step
            if left > 20 and at < len(ids) - 12:
                n = min(left - 12, rng.choice([2, 3, 8, 21, 64, 70]))
            else:
                n = 1
            entries.append((rid, ids[at:at + n], list(range(n))))
            live[rid] = at + n
            if live[rid] == len(ids):
                end.append(rid)
                del live[rid]
        if entries:
            rp.step(entries, end=end)
            slots_seen += [rp.lm.cache.slot(r) for r in live if r in rp.pos]
    cache = rp.lm.cache
    if cache.allocators:                                   # (shape C keeps no pages at all)
        assert cache.stats["allocated"] > cache.allocators[0].num_pages
        assert cache.free_pages(0) == cache.allocators[0].num_pages
    assert len(prompts) > 4 >= len(set(slots_seen))          # state slots were used again
    compare(rp.rows, oracle, TOL[dtype])


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("A", "bfloat16"), ("C", "float32")])
def test_greedy_generation_entry_point(folders, name, dtype):
    """``load_lm`` / ``generate_ids`` / ``generate_batch``: the scheduler's portions, batches
    and the steps launched ahead of their token ids choose the plain implementation's tokens."""
    from pretrained_rstr_b200 import generate_batch, generate_ids, load_lm
    folder = folders[(name, dtype)]
    cfg, tensors = P.read_folder(folder)
    m = load_lm(folder, gpu=True, dtype=dtype, max_lanes=3, max_batched_tokens=128,
                prefill_chunk=32, maxpos=256)
    prompts = list(_prompts(name, [1, 9, 33, 70, 130], salt=200).values())
    n_new = 10

    def agree(prompt, got):
        want = P.greedy(prompt, n_new, tensors, cfg)
        for i, (a, b) in enumerate(zip(got, want)):
            if a != b:
                row = P.forward(list(prompt) + want[:i], tensors, cfg)[-1]
                gap = abs(float(row[a] - row[b]))
                assert dtype == "bfloat16" and gap < 0.1, \
                    f"token {i} is {a}, plain says {b} (logit gap {gap:.3g})"
                return
        assert len(got) == len(want)

    agree(prompts[1], generate_ids(m, prompts[1], n_new))
    for p, got in zip(prompts, generate_batch(m, prompts, n_new)):
        agree(p, got)
    cache = m.engine.lm.cache
    assert not cache.requests
    cache.check()


def test_replay_and_generate_as_programs(folders, tmp_path):
    """``bin/trace_run`` and ``python -m pretrained_rstr_b200 generate`` on a Pezarax folder:
    the model class comes from config.json; logits of a replayed trace match the plain ones."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder = folders[("A", "float32")]
    cfg, tensors = P.read_folder(folder)
    ids = random_tokens(40, cfg["vocab"], 77)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": ids[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": ids[30:32], "want": []},
                                     {"id": "b", "tokens": ids[:3], "want": [2]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": ids[32:], "want": [7]}], "end": ["a"]}]
    out = tmp_path / "out"
    proc = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype",
                           "float32", "--out", str(out), "--max-tokens", "128"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", text=True,
                          capture_output=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    want = P.forward(ids, tensors, cfg).to(torch.float32)
    got0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1))
    got1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1))
    got2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(1, -1))
    for row, pos in ((got0[0], 0), (got0[1], 29), (got1[0], 2), (got2[0], 39)):
        assert row_error(row, want[pos]) < TOL["float32"]
    proc = subprocess.run([sys.executable, "-m", "pretrained_rstr_b200", "generate", "--model", folder,
                           "--dtype", "float32", "--ids", ",".join(map(str, ids[:9])), "--n", "5",
                           "--maxpos", "64"], cwd=root, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    rec = json.loads(proc.stdout.strip().splitlines()[-1])
    assert rec["generated"] == P.greedy(ids[:9], 5, tensors, cfg)
