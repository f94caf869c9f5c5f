"""Redisun in the engine against the plain implementation (``plain_redisun``): every mechanism
alone at the kernels' interface, then whole models of several shapes under every way of
cutting and batching the work, in 32-bit and in bfloat16, and greedy generation through the
package's entry point."""
import math
import random

import pytest
import torch

import plain_redisun as P
from helpers import Replayer, random_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


# --------------------------------------------------------------------------- configurations
def _mixer(heads, dim, rot_dim, vdim, kv_rank, q_rank, rot_dims=None, base=10000.0, scale=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
            "q_rank": q_rank, "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims},
            "scale": scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim)}


def _layer(mixer, mlp):
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def _moe(experts, top, ff, limit, shared_ff=0, shared_limit=0.0):
    return {"kind": "moe", "router": {"experts": experts, "top": top},
            "expert": {"ff": ff, "limit": limit},
            "shared": {"ff": shared_ff, "limit": shared_limit} if shared_ff else None}


# Every size differs from every other one; heads, ranks and widths that are no powers of two;
# a layer without a feed-forward; experts with and without a shared one, one of several and all
# of them chosen; a rotation that covers part of the rotated dimensions only.
SHAPE_A = {"architecture": "Redisun", "vocab": 300, "width": 64, "norm": {"eps": 1e-5},
           "postln_alpha": 2.5,
           "embedding": {"bigram": {"buckets": 97, "mul_prev": 1000003, "mul_cur": 11}},
           "layers": [
               _layer(_mixer(3, 16, 8, 24, 40, 24), {"kind": "dense", "ff": 96}),
               _layer(_mixer(3, 16, 8, 24, 40, 24), _moe(5, 2, 16, 0.8, 24, 1.3)),
               _layer(_mixer(2, 24, 16, 8, 56, 32, rot_dims=8, base=500.0, scale=0.3), None),
               _layer(_mixer(3, 16, 8, 24, 40, 24), _moe(4, 1, 24, 2.0)),
               _layer(_mixer(5, 8, 8, 16, 24, 40), {"kind": "dense", "ff": 72})]}
SHAPE_B = {"architecture": "Redisun", "vocab": 515, "width": 128, "norm": {"eps": 1e-6},
           "postln_alpha": 1.0,
           "embedding": {"bigram": {"buckets": 4093, "mul_prev": 3, "mul_cur": 65537}},
           "layers": [
               _layer(_mixer(2, 64, 32, 48, 144, 72, rot_dims=16), _moe(3, 3, 40, 1.0, 64, 1.0)),
               _layer(_mixer(4, 32, 64, 32, 96, 48), {"kind": "dense", "ff": 200})]}
SHAPES = {"A": (SHAPE_A, 11), "B": (SHAPE_B, 12)}
CASES = [(name, dtype) for name in SHAPES for dtype in ("float32", "bfloat16")]
TOL = {"float32": 2e-4, "bfloat16": 3e-2}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from pretrained_rstr_b200.config.registry import lookup
    from pretrained_rstr_b200.weights import make_random_model
    out = {}
    for name, (raw, seed) in SHAPES.items():
        cfg = lookup(raw).config_class.from_dict(raw)
        for dtype in ("float32", "bfloat16"):
            path = str(tmp_path_factory.mktemp(f"redisun{name}_{dtype}"))
            make_random_model(path, cfg, seed, torch.bfloat16 if dtype == "bfloat16" else torch.float32)
            out[(name, dtype)] = path
    return out


# A router's choice between two experts whose logits lie this close may fall either way once the
# stream is rounded to bfloat16 (float32: to its last bits); such a token's row, a legitimate
# other model's, is not compared, and rows after it in its request (which attend to it) get
# ``AFTER`` times the tolerance.
CLOSE = {"float32": 1e-4, "bfloat16": 2e-2}
AFTER = 4.0


class Oracle(dict):
    """request -> plain logits [T, vocab]; ``close[request]``: the first position with a close
    router call, or None."""


def _oracle(folder, prompts, dtype="float32"):
    cfg, tensors = P.read_folder(folder)
    out = Oracle()
    out.close = {}
    for rid, ids in prompts.items():
        gaps = []
        out[rid] = P.forward(list(ids), tensors, cfg, gaps=gaps).to(torch.float32)
        tight = torch.stack(gaps).min(0).values < CLOSE[dtype] if gaps else torch.zeros(len(ids), dtype=torch.bool)
        out.close[rid] = tight
    return out


def row_error(row: torch.Tensor, ref: torch.Tensor) -> float:
    """Root mean square of the difference (its mean taken off: a shift of all logits changes
    no probability) over that of the reference row."""
    d = row.double() - ref.double()
    d = d - d.mean()
    r = ref.double() - ref.double().mean()
    return float(d.pow(2).mean().sqrt() / r.pow(2).mean().sqrt())


def compare(rows, oracle, tol):
    assert rows
    worst = 0.0
    skipped = 0
    for (rid, pos), row in sorted(rows.items()):
        err = row_error(row, oracle[rid][pos])
        assert err == err, f"NaN at request {rid} position {pos}"
        close = oracle.close[rid]
        if bool(close[pos]):
            skipped += 1
            continue
        limit = tol * (AFTER if bool(close[:pos].any()) else 1.0)
        assert err <= limit, (f"request {rid} position {pos} (page offset {pos % 64}): relative "
                              f"difference {err:.3e} > {limit:.1e}")
        worst = max(worst, err)
    assert skipped <= 0.25 * len(rows), "too many close router calls for the test to mean much"
    return worst


def _prompts(name, lengths, salt=0):
    raw, seed = SHAPES[name]
    return {f"r{i}": random_tokens(n, raw["vocab"], 1000 * seed + salt + i) for i, n in enumerate(lengths)}


# ------------------------------------------------------------------ mechanisms, one by one
def test_pair_embedding_kernel():
    """Token row plus hashed pair row; the previous token comes from the step or, at a
    portion's start, from the request's state row; a sequence's first token takes the last
    row whatever the state row held (a slot used again)."""
    from pretrained_rstr_b200.csrc import ops
    vocab, width, buckets, mp, mc = 50, 24, 13, 10 ** 9 + 7, 5
    g = torch.Generator().manual_seed(1)
    table, pairs = torch.randn(vocab, width, generator=g), torch.randn(buckets + 1, width, generator=g)
    tensors = {"embed": table, "bigram": pairs}
    cfg = {"embedding": {"bigram": {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}}}
    seq_a, seq_b = random_tokens(9, vocab, 3), random_tokens(5, vocab, 4)
    want_a = P.embed(seq_a, tensors, cfg, torch.float32)
    want_b = P.embed(seq_b, tensors, cfg, torch.float32)
    state = torch.full((4,), 7, dtype=torch.int32, device=DEV)           # stale values of earlier users

    def step(parts):
        """parts: (slot, tokens, first position)"""
        toks, pos, seq, qs, slots = [], [], [], [0], []
        for b, (slot, ids, p0) in enumerate(parts):
            toks += ids
            pos += list(range(p0, p0 + len(ids)))
            seq += [b] * len(ids)
            qs.append(len(toks))
            slots.append(slot)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        out = torch.empty(len(toks), width, device=DEV)
        status = torch.zeros(4, dtype=torch.int32, device=DEV)
        ops.embed_pair(out, i32(toks), i32(pos), i32(seq), i32(qs), i32(slots), state,
                       table.to(DEV), pairs.to(DEV), buckets, mp, mc, status)
        assert int(status[0]) == 0
        return out.cpu()

    got = step([(2, seq_a[:4], 0), (0, seq_b[:1], 0)])
    assert torch.allclose(got[:4], want_a[:4]) and torch.allclose(got[4:], want_b[:1])
    got = step([(0, seq_b[1:2], 1), (2, seq_a[4:6], 4)])                  # other order, other sizes
    assert torch.allclose(got[:1], want_b[1:2]) and torch.allclose(got[1:], want_a[4:6])
    got = step([(2, seq_a[6:9], 6)])
    assert torch.allclose(got, want_a[6:9])
    got = step([(0, seq_b[2:5], 2)])
    assert torch.allclose(got, want_b[2:5])
    got = step([(2, seq_b[:3], 0)])                                       # slot 2 used again
    assert torch.allclose(got, want_b[:3])


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_rms_norm_kernel(out_dtype):
    from pretrained_rstr_b200.csrc import ops
    g = torch.Generator().manual_seed(2)
    for width in (24, 200, 1030):
        x, y = torch.randn(7, width, generator=g) * 3, torch.randn(7, width, generator=g)
        gate_w = torch.randn(7, width + 8, generator=g)
        bias, weight = torch.randn(width, generator=g), torch.rand(width, generator=g) + 0.5
        gain = torch.tensor([1.7])
        d = lambda t: t.to(DEV)
        # one number, rows gathered
        rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
        out = torch.empty(3, width, dtype=out_dtype, device=DEV)
        ops.rms_norm(d(x), out=out, gain=d(gain), rows=rows, eps=1e-3)
        want = P.scalar_norm(x.double(), gain.double(), 1e-3)[[5, 0, 5]]
        tol = 1e-5 if out_dtype == torch.float32 else 2e-2
        assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol)
        # a weight per coordinate
        out = torch.empty(7, width, dtype=out_dtype, device=DEV)
        ops.rms_norm(d(x), out=out, weight=d(weight), eps=1e-6)
        assert torch.allclose(out.cpu().double(), P.vector_norm(x.double(), weight.double(), 1e-6),
                              atol=tol, rtol=tol)
        # a gated branch joined to the stream, in place, with the typed copy
        xs = d(x).clone()
        ops.rms_norm(xs, out=out, x_out=xs, y=d(y), gate=d(gate_w)[:, 8:], gate_bias=d(bias),
                     gain=d(gain), alpha=2.5, eps=1e-6)
        v = 2.5 * x.double() + torch.sigmoid(gate_w[:, 8:].double() + bias.double()) * y.double()
        want = P.scalar_norm(v, gain.double(), 1e-6)
        assert torch.allclose(xs.cpu().double(), want, atol=1e-5, rtol=1e-5)
        assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol)


def test_gated_pair_and_router_kernels():
    """The experts' activation with its caps, shift and routing weights; the router's choice
    and weights, for one of many, some and all experts."""
    from pretrained_rstr_b200.csrc import ops
    g = torch.Generator().manual_seed(3)
    t, n_e, ff = 9, 6, 10
    for top in (1, 2, 6):
        logits = torch.randn(t, n_e + 3, generator=g)
        bias = torch.randn(n_e, generator=g)
        scale = torch.empty(t, n_e, device=DEV)
        chosen = torch.empty(t, top, dtype=torch.int32, device=DEV)
        chosen_w = torch.empty(t, top, device=DEV)
        ops.route(scale, chosen, chosen_w, logits.to(DEV)[:, 2:2 + n_e], None, bias.to(DEV), top)
        val, idx = torch.topk(logits[:, 2:2 + n_e] + bias, top, dim=-1)
        assert torch.equal(chosen.cpu().long(), idx)
        assert torch.allclose(chosen_w.cpu(), torch.softmax(val, -1), atol=1e-6)
        dense = torch.zeros(t, n_e).scatter(1, idx, torch.softmax(val, -1))
        assert torch.allclose(scale.cpu(), dense, atol=1e-6)
        assert abs(float(scale.sum()) - t) < 1e-4
    x = torch.randn(t, 32, generator=g)
    w = torch.randn(n_e, 32, generator=g)
    ops.route(scale, chosen, chosen_w, x.to(DEV), w.to(DEV), bias.to(DEV), top)
    assert torch.equal(chosen.cpu().long(), torch.topk(x @ w.T + bias, top, dim=-1)[1])
    inp = torch.randn(t, 2 * n_e * ff + 5, generator=g) * 2
    out = torch.zeros(t, n_e * ff + 3, device=DEV)
    ops.gated_pair(out, inp.to(DEV), 5, 5 + n_e * ff, n_e * ff, out_col=3, limit=0.9,
                   act_alpha=1.702, up_shift=1.0, scale=scale, group=ff)
    gg = torch.clamp(inp[:, 5:5 + n_e * ff], max=0.9)
    uu = torch.clamp(inp[:, 5 + n_e * ff:], -0.9, 0.9)
    want = gg * torch.sigmoid(1.702 * gg) * (uu + 1.0) * scale.cpu().repeat_interleave(ff, dim=1)
    assert torch.allclose(out.cpu()[:, 3:], want, atol=1e-5)
    assert float(out[:, :3].abs().max()) == 0.0
    ops.gated_pair(out, inp.to(DEV), 5, 5 + n_e * ff, n_e * ff, out_col=3)      # plain SiLU gate
    g0, u0 = inp[:, 5:5 + n_e * ff], inp[:, 5 + n_e * ff:]
    assert torch.allclose(out.cpu()[:, 3:], g0 * torch.sigmoid(g0) * u0, atol=1e-5)


# --- attention over the shared latent, at the kernels' interface
class LatentCase:
    """A paged cache filled by hand: requests' rows lie in pages taken in a shuffled order from
    a pool whose other pages hold large numbers (what earlier owners left)."""

    def __init__(self, lengths, rank, rot_dim, dtype, page=64, seed=0, fill=50.0):
        g = torch.Generator().manual_seed(seed)
        self.rank, self.rot_dim, self.page, self.dtype = rank, rot_dim, page, dtype
        d = rank + rot_dim
        need = sum(-(-n // page) for n in lengths)
        pages = list(range(need + 3))
        random.Random(seed).shuffle(pages)
        self.rows = [torch.randn(n, d, generator=g) * 0.3 for n in lengths]
        self.max_pages = max(-(-n // page) for n in lengths) + 1
        cache = torch.full((need + 3, 1, page, d), fill)
        table = torch.full((len(lengths), self.max_pages), -1, dtype=torch.int32)
        for b, n in enumerate(lengths):
            for li in range(-(-n // page)):
                pg = pages.pop()
                table[b, li] = pg
                m = min(page, n - li * page)
                cache[pg, 0, :m] = self.rows[b][li * page:li * page + m]
        self.cache_f32, self.table = cache, table

    def to_device(self):
        self.cache = self.cache_f32.to(self.dtype).to(DEV)
        self.rows = [r.to(self.dtype).float() for r in self.rows]        # what the kernel reads
        return self

    def run(self, queries, sinks=None, scale=1.0, window=None, kernel="generic", items=None,
            split_keys=None, rotate=None):
        """queries: list of (request, position, qa [heads, rank + rot_dim]); returns
        [n, heads, rank] and the plain implementation's answer.  ``kernel``: "generic" (32-bit
        arithmetic), or the tensor-core kernel with every query an item of its own whose warps
        split the keys ("single") or not ("tile"), or with ``items`` = [(first query, queries)]
        of consecutive positions of one request."""
        from pretrained_rstr_b200.csrc import ops
        qa = torch.stack([q for _, _, q in queries]).to(DEV).contiguous()
        n, heads, _ = qa.shape
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        out = torch.full((n, heads, self.rank), float("nan"), device=DEV)
        status = torch.zeros(4, dtype=torch.int32, device=DEV)
        seq, pos = i32([b for b, _, _ in queries]), i32([p for _, p, _ in queries])
        sk = None if sinks is None else sinks.to(DEV)
        if kernel == "generic":
            ops.latent_attention(out, qa, self.cache, self.table.to(DEV), seq, pos, sk, scale,
                                 window, self.rank, status)
        else:
            qa = qa.to(torch.bfloat16)
            queries = [(b, p, q.to(torch.bfloat16).float()) for b, p, q in queries]
            kw = ops.latent_mma_single_kw(heads) if kernel == "single" else 1
            items = items or [(i, 1) for i in range(n)]
            ws_rows = heads if kernel == "single" else 128
            longest = max(p for _, p, _ in queries) + 1
            split_keys = split_keys or 128
            splits = -(-longest // split_keys)
            slots = (len(items) + 2) * ws_rows * splits
            ws_o = torch.full((slots * self.rank,), float("nan"), device=DEV)
            ws_ml = torch.full((slots * 2,), float("nan"), device=DEV)
            count = i32([len(items)])
            ops.latent_attention_mma(out, qa, self.cache, self.table.to(DEV), seq, pos,
                                     i32([i for i, _ in items] + [0, 0]),
                                     None if kernel == "single" else i32([k for _, k in items] + [1, 1]),
                                     count, len(items) + 2, sk, ws_o, ws_ml, scale, window, self.rank,
                                     split_keys, splits, kw, ws_rows, status, rotate=rotate)
        assert int(status[0]) == 0, status.tolist()
        want = []
        for b, p, q in queries:
            lo = max(0, p - window + 1) if window else 0
            keys = self.rows[b][lo:p + 1].double()
            s = (q.double() @ keys.T) * scale                                   # [heads, keys]
            sk = sinks.double() if sinks is not None else torch.full((heads,), float("-inf")).double()
            w = P.sink_softmax(s, sk)
            want.append(w @ keys[:, :self.rank])
        return out.cpu().double(), torch.stack(want)


KERNELS = [(torch.float32, "generic"), (torch.bfloat16, "generic"), (torch.bfloat16, "single"),
           (torch.bfloat16, "tile")]
ATOL = {"generic": 2e-5, "single": 4e-3, "tile": 4e-3}


@pytest.mark.parametrize("dtype,kernel", KERNELS)
def test_latent_attention_random(dtype, kernel):
    """Random rows and queries, several requests in one launch, with and without sinks."""
    rank, rot = (40, 8) if kernel == "generic" else (48, 16)
    case = LatentCase([1, 63, 64, 65, 200, 517], rank, rot, dtype, seed=5).to_device()
    g = torch.Generator().manual_seed(6)
    queries = [(b, p, torch.randn(3, rank + rot, generator=g))
               for b, n in enumerate([1, 63, 64, 65, 200, 517]) for p in sorted({0, n // 2, n - 1})]
    for sinks in (None, torch.tensor([-1.0, 0.5, 3.0])):
        got, want = case.run(queries, sinks=sinks, scale=0.4, kernel=kernel)
        assert torch.allclose(got, want, atol=ATOL[kernel], rtol=1e-4)


@pytest.mark.parametrize("heads,rank,rot", [(3, 48, 16), (8, 128, 32), (12, 256, 32), (20, 64, 0),
                                            (40, 32, 16)])
def test_latent_attention_tiles_of_a_portion(heads, rank, rot):
    """A portion of consecutive tokens as the tensor-core kernel's tiles of 128 // heads
    tokens, the keys in ranges of several sizes; and the same tokens one by one."""
    case = LatentCase([700, 90], rank, rot, torch.bfloat16, seed=13).to_device()
    g = torch.Generator().manual_seed(14)
    first, n = 381, 150
    queries = [(0, first + i, torch.randn(heads, rank + rot, generator=g)) for i in range(n)]
    queries += [(1, 20 + i, torch.randn(heads, rank + rot, generator=g)) for i in range(70)]
    tq = 128 // heads
    items = [(r0, min(tq, n - r0)) for r0 in range(0, n, tq)]
    items += [(n + r0, min(tq, 70 - r0)) for r0 in range(0, 70, tq)]
    sinks = torch.randn(heads, generator=g)
    for split_keys in (64, 192, 1024):
        got, want = case.run(queries, sinks=sinks, scale=0.2, kernel="tile", items=items,
                             split_keys=split_keys)
        assert torch.allclose(got, want, atol=4e-3, rtol=1e-3), float((got - want).abs().max())
    got, want = case.run(queries[::7], sinks=sinks, scale=0.2, kernel="single", split_keys=256)
    assert torch.allclose(got, want, atol=4e-3, rtol=1e-3), float((got - want).abs().max())


@pytest.mark.parametrize("dtype,kernel", KERNELS)
@pytest.mark.parametrize("many", [False, True])
def test_latent_attention_needles(dtype, kernel, many):
    """One key is made to stand out (its rotated part is parallel to the query's): the result
    must be that key's latent, wherever it lies: the first rows, both sides of page borders,
    the query's own row, one row among hundreds far back.  A larger number in the row AFTER
    the query (a page's earlier owner) must not be seen.  ``many``: all queries in one
    launch, as a prompt's portion brings them; else one launch per query, as decoding does."""
    n, rank, rot = 900, 32, 16
    case = LatentCase([n, 130], rank, rot, dtype, seed=7)
    needle = torch.zeros(rot)
    needle[3] = 6.0
    spots = [0, 1, 62, 63, 64, 65, 127, 128, 191, 192, 500, 833, 898, 899]
    for j in spots:                                       # needles live in request 0
        pg, off = int(case.table[0, j // 64]), j % 64
        case.cache_f32[pg, 0, off, rank:] = needle
        case.rows[0][j, rank:] = needle
    case.to_device()
    q = torch.zeros(2, rank + rot)
    q[:, rank + 3] = 8.0                                   # score 48 at a needle, ~0 elsewhere
    queries, expect = [], []
    for j in spots:
        later = [s for s in spots if s > j]
        pos = (later[0] - 1) if later else n - 1           # the needle at j is the last one seen...
        for p in sorted({j, pos}):                          # ...as the query's own row and from afar
            queries.append((0, p, q))
            expect.append(j)
    outs = []
    if many:
        outs = case.run(queries, kernel=kernel)[0]
    else:
        outs = torch.cat([case.run([qq], kernel=kernel)[0] for qq in queries])
    for (b, p, _), j, got in zip(queries, expect, outs):
        seen = [s for s in spots if s <= p]
        want = torch.stack([case.rows[0][s, :rank] for s in seen]).double().mean(0)
        assert torch.allclose(got[0], want, atol=4e-3), f"query at {p}: needles {seen} not found"
    # the row after the query's holds a needle too (position p + 1 of the same page): unseen
    got, want = case.run([(0, 61, q), (0, 126, q)], kernel=kernel)
    assert torch.allclose(got, want, atol=ATOL[kernel])
    only = torch.stack([case.rows[0][s, :rank] for s in (0, 1)]).double().mean(0)
    assert torch.allclose(got[0, 0], only, atol=4e-3)


@pytest.mark.parametrize("dtype,kernel", KERNELS)
def test_latent_attention_sink_and_window(dtype, kernel):
    """A sink that dwarfs every score takes all the weight (the result vanishes); one far
    below changes nothing; left out, the result differs from a moderate one's.  A window sees
    the key at its edge and not the one before."""
    rank, rot = 16, 16
    case = LatentCase([300], rank, rot, dtype, seed=9).to_device()
    g = torch.Generator().manual_seed(10)
    q = torch.randn(2, rank + rot, generator=g)
    base, _ = case.run([(0, 299, q)], kernel=kernel)
    got, want = case.run([(0, 299, q)], sinks=torch.tensor([60.0, -60.0]), kernel=kernel)
    assert torch.allclose(got, want, atol=ATOL[kernel])
    assert float(got[0, 0].abs().max()) < 1e-6 and torch.allclose(got[0, 1], base[0, 1], atol=ATOL[kernel])
    got, want = case.run([(0, 299, q)], sinks=torch.tensor([6.0, 5.0]), kernel=kernel)     # about the keys' sum
    assert torch.allclose(got, want, atol=ATOL[kernel]) and float((got - base).abs().max()) > 2e-2
    # window of 70 at position 299: keys 230..299
    case2 = LatentCase([300], rank, rot, dtype, seed=11)
    needle = torch.zeros(rot)
    needle[0] = 6.0
    for j in (229, 230):
        pg, off = int(case2.table[0, j // 64]), j % 64
        case2.cache_f32[pg, 0, off, rank:] = needle * (2.0 if j == 229 else 1.0)
        case2.rows[0][j, rank:] = needle * (2.0 if j == 229 else 1.0)
    case2.to_device()
    qn = torch.zeros(1, rank + rot)
    qn[0, rank] = 8.0
    got, want = case2.run([(0, 299, qn)], window=70, kernel=kernel)
    assert torch.allclose(got, want, atol=ATOL[kernel])
    assert torch.allclose(got[0, 0], case2.rows[0][230, :rank].double(), atol=4e-3)   # 230 in, 229 out
    got, _ = case2.run([(0, 299, qn)], window=71, kernel=kernel)
    assert torch.allclose(got[0, 0], case2.rows[0][229, :rank].double(), atol=4e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_mixer_chain(dtype):
    """prepare -> fold -> attention -> unfold against the plain mixer (its output projection
    the identity), one sequence cut in two steps over shuffled pages."""
    from pretrained_rstr_b200.csrc import ops
    heads, dim, rot_dim, rot_dims, vdim, rank, q_rank, width = 3, 16, 8, 4, 12, 40, 24, 32
    t, cut, page = 100, 37, 64
    g = torch.Generator().manual_seed(12)
    rnd = lambda *s: (torch.randn(*s, generator=g) / math.sqrt(s[-1])).to(dtype).float()
    mx = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
          "q_rank": q_rank, "scale": 0.25, "rot": {"base": 77.0, "dims": rot_dims}}
    tensors = {"l0.mix.dq": rnd(q_rank, width), "l0.mix.dq.norm": torch.rand(q_rank, generator=g) + 0.5,
               "l0.mix.uq": rnd(heads * (dim + rot_dim), q_rank), "l0.mix.dkv": rnd(rank + rot_dim, width),
               "l0.mix.dkv.norm": torch.rand(rank, generator=g) + 0.5, "l0.mix.uk": rnd(heads * dim, rank),
               "l0.mix.uv": rnd(heads * vdim, rank), "l0.mix.sink": torch.randn(heads, generator=g),
               "l0.mix.g": rnd(heads, width), "l0.mix.o": torch.eye(heads * vdim)}
    h = torch.randn(t, width, generator=g)
    want = P.latent_attention(h.double(), tensors, "l0.", mx, 1e-6)
    d = lambda x: x.to(DEV).contiguous()
    cache = torch.full((5, 1, page, rank + rot_dim), 9.0, dtype=dtype, device=DEV)
    table = torch.tensor([[3, 1, -1]], dtype=torch.int32, device=DEV)
    freq = d(torch.tensor([77.0 ** (-2.0 * i / rot_dims) for i in range(rot_dims // 2)]))
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    outs = []
    for lo, hi in ((0, cut), (cut, t)):
        n = hi - lo
        hh = h[lo:hi]
        proj = d(torch.cat([hh @ tensors["l0.mix.dq"].T, hh @ tensors["l0.mix.dkv"].T,
                            hh @ tensors["l0.mix.g"].T], dim=1))
        pos = torch.arange(lo, hi, dtype=torch.int32, device=DEV)
        slots = torch.tensor([int(table[0, p // page]) * page + p % page for p in range(lo, hi)],
                             dtype=torch.int32, device=DEV)
        cq = torch.empty(n, q_rank, device=DEV)
        ops.latent_prepare(cq, cache, proj, 0, q_rank, d(tensors["l0.mix.dq.norm"]),
                           d(tensors["l0.mix.dkv.norm"]), slots, pos, freq, q_rank, rank, rot_dim,
                           rot_dims, 1e-6, status)
        q = (cq @ d(tensors["l0.mix.uq"]).T).contiguous()
        qa = torch.empty(n, heads, rank + rot_dim, device=DEV)
        ops.latent_fold(qa, q, d(tensors["l0.mix.uk"]).to(dtype), pos, freq, heads, dim, rot_dim,
                        rot_dims, rank)
        lat = torch.empty(n, heads, rank, device=DEV)
        ops.latent_attention(lat, qa, cache, table, torch.zeros(n, dtype=torch.int32, device=DEV), pos,
                             d(tensors["l0.mix.sink"]), 0.25, None, rank, status)
        uvt = d(tensors["l0.mix.uv"]).to(dtype).reshape(heads, vdim, rank).transpose(1, 2).contiguous()
        o = torch.empty(n, heads * vdim, device=DEV)
        ops.latent_unfold(o, lat, uvt, proj[:, q_rank + rank + rot_dim:], heads, rank, vdim)
        outs.append(o.cpu())
    assert int(status[0]) == 0
    got = torch.cat(outs).double()
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert torch.allclose(got, want, atol=tol, rtol=tol), float((got - want).abs().max())


@pytest.mark.parametrize("kernel", ["single", "tile"])
def test_latent_attention_rotates_queries(kernel):
    """Given unrotated queries and the rotation's frequencies, the tensor-core kernel rotates
    the last part of every row by the row's position as it loads them: the same result as with
    queries rotated beforehand, for rows of several tokens in one tile and for every key range."""
    heads, rank, rot, rot_dims = 5, 32, 32, 16
    case = LatentCase([400], rank, rot, torch.bfloat16, seed=21).to_device()
    g = torch.Generator().manual_seed(22)
    first, n = 250, 30
    raw = [torch.randn(heads, rank + rot, generator=g).to(torch.bfloat16).float() for _ in range(n)]
    freq = torch.tensor([50.0 ** (-2.0 * i / rot_dims) for i in range(rot_dims // 2)])
    turned = []
    for i, q in enumerate(raw):
        t = q.clone().double()
        t[:, rank:] = P.rotate(t[None, :, rank:], torch.tensor([first + i]), 50.0, rot_dims)[0]
        turned.append(t.float())
    queries = [(0, first + i, q) for i, q in enumerate(raw)]
    items = [(r0, min(25, n - r0)) for r0 in range(0, n, 25)] if kernel == "tile" else None
    _, want = case.run([(0, first + i, q) for i, q in enumerate(turned)], scale=0.3)
    for split_keys in (64, 512):
        got, _ = case.run(queries, scale=0.3, kernel=kernel, items=items, split_keys=split_keys,
                          rotate=(freq.to(DEV), rot_dims))
        assert torch.allclose(got, want, atol=6e-3, rtol=1e-3), float((got - want).abs().max())


# ------------------------------------------------------- whole models through the step function
@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_decode_portions(folders, name, dtype):
    """Each request whole; then most of it at once and the last tokens one by one; then in
    portions of changing size down to two tokens, cut inside pages: the same logits."""
    folder = folders[(name, dtype)]
    prompts = _prompts(name, [1, 2, 23, 64, 65, 150, 260])
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


@pytest.mark.parametrize("name,dtype", CASES)
def test_long_decode(folders, name, dtype):
    """Two tokens of prompt and 200 decoded one by one, across page borders."""
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
    assert rp.lm.cache.stats["allocated"] > rp.lm.cache.allocators[0].num_pages
    assert rp.lm.cache.free_pages(0) == rp.lm.cache.allocators[0].num_pages
    assert len(prompts) > 4 >= len(set(slots_seen))          # state slots were used again
    compare(rp.rows, oracle, TOL[dtype])


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_entry_point(folders, name, dtype):
    """``load_lm`` / ``generate_ids`` / ``generate_batch``: the scheduler's portions, batches
    and the steps launched ahead of their token ids (the previous token lives on the device)
    choose the plain implementation's tokens."""
    from pretrained_rstr_b200 import generate_batch, generate_ids, load_lm
    folder = folders[(name, dtype)]
    cfg, tensors = P.read_folder(folder)
    m = load_lm(folder, gpu=True, dtype=dtype, max_lanes=3, max_batched_tokens=128,
                prefill_chunk=32, maxpos=256)
    prompts = list(_prompts(name, [1, 9, 33, 70, 130], salt=200).values())
    n_new = 12

    def agree(prompt, got):
        want = P.greedy(prompt, n_new, tensors, cfg)
        for i, (a, b) in enumerate(zip(got, want)):
            if a != b:
                row = P.forward(list(prompt) + want[:i], tensors, cfg)[-1]
                gap = abs(float(row[a] - row[b]))
                assert dtype == "bfloat16" and gap < 5e-2, \
                    f"token {i} is {a}, plain says {b} (logit gap {gap:.3g})"
                return
        assert len(got) == len(want)

    agree(prompts[1], generate_ids(m, prompts[1], n_new))
    for p, got in zip(prompts, generate_batch(m, prompts, n_new)):
        agree(p, got)
    cache = m.engine.lm.cache
    assert not cache.requests and cache.free_pages(0) == cache.allocators[0].num_pages
    cache.check()


def test_replay_and_generate_as_programs(folders, tmp_path):
    """``bin/trace_run`` and ``python -m pretrained_rstr_b200 generate`` on a Redisun folder:
    the model class comes from config.json; logits of a replayed trace match the plain ones."""
    import json
    import os
    import subprocess
    import sys
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
    import numpy as np
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


def test_second_norm_without_a_feed_forward(folders, tmp_path):
    """A file that holds the second norm of a layer without a feed-forward: the norm is
    applied to the scaled stream alone."""
    import shutil
    from pretrained_rstr_b200.weights.safetensors_io import save_file
    src = folders[("A", "float32")]
    cfg, tensors = P.read_folder(src)
    assert cfg["layers"][2]["mlp"] is None and "l2.norm2" not in tensors
    tensors["l2.norm2"] = torch.tensor(1.3)
    folder = str(tmp_path / "with_norm2")
    shutil.copytree(src, folder)
    save_file(tensors, folder + "/model.safetensors")
    prompts = {"r0": random_tokens(70, cfg["vocab"], 5)}
    oracle = _oracle(folder, prompts)
    rp = Replayer(folder, "float32", max_tokens=128)
    rp.step([("r0", prompts["r0"][:40], list(range(40)))])
    rp.step([("r0", prompts["r0"][40:], list(range(30)))], end=["r0"])
    compare(rp.rows, oracle, TOL["float32"])
    plain_without = P.forward(prompts["r0"], P.read_folder(src)[1], cfg).to(torch.float32)
    assert row_error(oracle["r0"][69], plain_without[69]) > 1e-3        # the norm matters
