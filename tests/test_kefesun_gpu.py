"""The Kefesun design on the GPU: each mechanism's kernel alone against the plain
restatement, then whole models through the engine under every way of cutting the
work, and greedy generation through the library's own entry point."""
import copy
import math

import numpy as np
import pytest
import torch

import plain_kefesun as pk
from kefesun_models import CONFIGS, model
from helpers import rel_err, run_trace, trace_batches, trace_tail, trace_whole

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = 64


def ops():
    from janas_b200.csrc import ops as o
    return o


def rnd(*shape, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed * 7919 + sum(shape) + len(shape))
    return torch.randn(*shape, generator=g) * scale


def bf(x):
    return x.to(torch.bfloat16).float()


def close(got, want, dtype, what="", bf16_tol=2e-2):
    tol = 2e-5 if dtype == torch.float32 else bf16_tol
    err = (got - want).abs().max() / want.abs().max()
    assert err <= tol, f"{what} {err:.3e}"


def i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


def row_arrays(rows):
    """rows: per sequence (first position, count) -> positions and sequences of all rows."""
    row_pos = torch.tensor([p for (p0, cnt) in rows for p in range(p0, p0 + cnt)], dtype=torch.int32)
    row_seq = torch.tensor([i for i, (p0, cnt) in enumerate(rows) for _ in range(cnt)], dtype=torch.int32)
    return row_pos, row_seq


# ------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("few", [False, True])
@pytest.mark.parametrize("n,dm,S", [(1, 50, 1), (7, 256, 3), (130, 1000, 2), (3, 4100, 1), (8, 352, 4), (40, 2560, 1), (5, 6000, 2)])
def test_norm_on_the_result_alone(few, n, dm, S):
    """x += LN(sum of the partial sums + coefficient * the sublayer's input); x itself is not normed."""
    x = rnd(n, dm, scale=3.0) + 2.0
    y = rnd(S, n, dm, seed=1) + 1.5                     # a mean that matters
    w = 1 + rnd(dm, scale=0.2, seed=2)
    want = x + pk.layer_norm_nobias(y.sum(0), w, 1e-5)
    xd = x.to(DEV).clone()
    ops().norm_residual_(xd, y.to(DEV), w.to(DEV), 1e-5, few_rows=few)
    assert (xd.cpu() - want).abs().max() <= 1e-5
    # the identity experts' share rides along: the input times a coefficient per row
    for sdt in (torch.float32, torch.bfloat16):
        skip = rnd(n, dm, seed=3).to(sdt)
        coef = rnd(n, seed=4).abs()
        want = x + pk.layer_norm_nobias(y.sum(0) + coef[:, None] * skip.float(), w, 1e-5)
        xd = x.to(DEV).clone()
        ops().norm_residual_(xd, y.to(DEV), w.to(DEV), 1e-5, skip=skip.to(DEV), skip_coef=coef.to(DEV),
                             few_rows=few)
        assert (xd.cpu() - want).abs().max() <= 1e-5
    # a result of constant rows has no deviations: nothing is added, whatever its size
    xd = x.to(DEV).clone()
    ops().norm_residual_(xd, torch.full((1, n, dm), 7.0, device=DEV), w.to(DEV), 1e-5, few_rows=few)
    assert (xd.cpu() - x).abs().max() <= 1e-5


class Slots:
    """Sequences in slots that lie in no order."""

    def __init__(self, n_seqs, n_slots, seed):
        perm = torch.randperm(n_slots, generator=torch.Generator().manual_seed(seed))
        self.slot = perm[:n_seqs].to(torch.int32)
        self.n_slots = n_slots


@pytest.mark.parametrize("odt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps,dm,lens", [(4, 352, 0), (2, 50, 0), (5, 136, 0), (3, 1000, 0), (1, 64, 0), (2, 264, 0),
                                          (4, 2048, [700, 1, 901, 3, 299, 507]), (3, 1536, [1203, 2, 2001])])
def test_short_convolution_over_time(odt, taps, dm, lens):
    """Whole prompts, then a portion, then rows one by one, against the convolution of the whole
    sequence: the last inputs are carried in the slots' state.  The long steps run the kernel
    whose threads move along several rows, over the sequences' borders."""
    lens = lens or [1, 9, 2, 70]
    more = ([2, 1, 5, 3] * 2)[:len(lens)] if max(lens) < 100 else [n + 17 for n in lens]
    xs = [rnd(n + m + 8, dm, seed=10 + i) for i, (n, m) in enumerate(zip(lens, more))]
    w = rnd(dm, taps, scale=0.5, seed=5)
    want = [pk.short_conv(x, w) for x in xs]
    sl = Slots(len(lens), 7, 3)
    state = torch.full((sl.n_slots, max(taps - 1, 1), dm), 9.0, device=DEV) if taps > 1 else None   # stale values
    tol = 1e-5 if odt == torch.float32 else 3e-2

    def step(rows, split):
        row_pos, row_seq = row_arrays(rows)
        x = torch.cat([xs[i][p0:p0 + cnt] for i, (p0, cnt) in enumerate(rows)])
        args = (x.to(DEV), w.to(DEV), state, row_pos.to(DEV), row_seq.to(DEV), sl.slot.to(DEV), odt)
        if split:
            got = ops().short_conv(*args, write_h=True, write_state=False)
            if taps > 1:
                ops().short_conv(*args, write_h=False, write_state=True)
        else:
            got = ops().short_conv(*args)
        ref = torch.cat([want[i][p0:p0 + cnt] for i, (p0, cnt) in enumerate(rows)])
        assert (got.float().cpu() - ref).abs().max() <= tol * max(1.0, float(ref.abs().max()))

    step([(0, n) for n in lens], False)                               # prompts from position 0
    step([(n, c) for n, c in zip(lens, more)], True)                  # portions of several sizes
    at = [n + c for n, c in zip(lens, more)]
    for k in range(4):                                                # one row each
        step([(a + k, 1) for a in at], False)
    if taps > 1:
        # the state holds the last taps - 1 inputs of every sequence (a ring over the positions)
        for i, a in enumerate(at):
            have = state[int(sl.slot[i])].cpu()
            for p in range(a + 4 - (taps - 1), a + 4):
                assert torch.equal(have[p % (taps - 1)], xs[i][p])


def test_a_short_sequence_reads_zeros_before_its_start():
    """A slot that another sequence used: a new sequence's first rows see nothing of it."""
    dm, taps = 40, 4
    w = torch.ones(dm, taps)
    state = torch.full((2, taps - 1, dm), 100.0, device=DEV)
    x = torch.ones(2, dm)
    got = ops().short_conv(x.to(DEV), w.to(DEV), state, i32([0, 1]), i32([0, 0]), i32([1]), torch.float32).cpu()
    assert torch.equal(got[0], torch.full((dm,), 2.0)) and torch.equal(got[1], torch.full((dm,), 3.0))


@pytest.mark.parametrize("odt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,S,extra", [(352, 1, 0), (48, 3, 5), (70, 2, 0), (1000, 1, 8)])
def test_mingru_recurrence(odt, width, S, extra):
    """Prompts of unequal length, portions and single rows against the recurrence over the whole
    sequence; the state (float32) is carried per slot."""
    lens = [1, 300, 2, 67]
    more = 9
    ld = 3 * width + extra
    Ps = [rnd(S, n + more, ld, scale=1.5, seed=20 + i) for i, n in enumerate(lens)]
    bias = rnd(3 * width, scale=0.5, seed=7)
    bias[2 * width:] = 0.0
    want = []
    for P in Ps:
        t = P.sum(0)[:, :3 * width] + bias
        want.append(pk.mingru_recurrence(t[:, :width], t[:, width:2 * width], t[:, 2 * width:])[0])
    sl = Slots(len(lens), 6, 5)
    state = torch.full((sl.n_slots, width), 3.0, device=DEV)
    state[sl.slot.long()] = 0.0                                       # a new sequence starts at zero
    tol = 2e-5 if odt == torch.float32 else 2e-2

    def step(rows, decode):
        row_pos, row_seq = row_arrays(rows)
        P = torch.cat([Ps[i][:, p0:p0 + cnt] for i, (p0, cnt) in enumerate(rows)], dim=1)
        got = ops().mingru(P.to(DEV), width, bias.to(DEV), state, row_seq.to(DEV), sl.slot.to(DEV), odt,
                           every_row_starts=decode)
        ref = torch.cat([want[i][p0:p0 + cnt] for i, (p0, cnt) in enumerate(rows)])
        assert (got.float().cpu() - ref).abs().max() <= tol * float(ref.abs().max())

    step([(0, n) for n in lens], False)
    step([(n, c) for n, c in zip(lens, (2, 3, 1, 4))], False)
    at = [n + c for n, c in zip(lens, (2, 3, 1, 4))]
    for k in range(4):
        step([(a + k, 1) for a in at], True)
    assert state.dtype == torch.float32
    # slots of no sequence of the step are left as they were
    others = [s for s in range(sl.n_slots) if s not in sl.slot.tolist()]
    assert all(torch.equal(state[s].cpu(), torch.full((width,), 3.0)) for s in others)


def test_mingru_candidate_and_long_memory():
    """The candidate is u + 1/2 from zero up and sigmoid(u) below; a gate near zero keeps the
    state over hundreds of rows, a gate near one forgets it at once."""
    width, n = 8, 500
    P = torch.zeros(1, n, 3 * width)
    P[0, :, :width] = -30.0                                           # z ~ 0: keep
    P[0, 0, :width] = 30.0                                            # the first row is taken whole
    P[0, 0, width:2 * width] = torch.tensor([-3.0, -1.0, -1e-3, 0.0, 1e-3, 1.0, 3.0, 10.0])
    P[0, :, 2 * width:] = 2.0
    state = torch.zeros(1, width, device=DEV)
    got = ops().mingru(P.to(DEV), width, None, state, i32([0] * n), i32([0]), torch.float32).cpu()
    u = P[0, 0, width:2 * width]
    c = torch.where(u >= 0, u + 0.5, 1 / (1 + torch.exp(-u)))
    silu2 = 2.0 / (1 + math.exp(-2.0))
    assert (got[0] - c * silu2).abs().max() <= 1e-6
    assert (got[-1] - c * silu2).abs().max() <= 1e-5                  # still there 499 rows later
    P[0, -1, :width] = 30.0                                           # z ~ 1 at the last row: replaced
    P[0, -1, width:2 * width] = 4.0
    state.zero_()
    got = ops().mingru(P.to(DEV), width, None, state, i32([0] * n), i32([0]), torch.float32).cpu()
    assert (got[-1] - 4.5 * silu2).abs().max() <= 1e-5


# ------------------------------------------------------------ the router and the weighted activation
def plain_routes(logits, corr, r):
    n, outs = logits.shape
    w = torch.zeros(n, outs)
    for t in range(n):
        chosen, weights = pk.route(logits[t], corr, r)
        for e, wt in zip(chosen, weights):
            w[t, e] = wt
    return w


ROUTERS = [dict(outs=12, ident=3, count=2, keep=1, top=5, scale=2.2),
           dict(outs=8, ident=2, count=4, keep=2, top=3, scale=1.7),
           dict(outs=3, ident=0, count=1, keep=1, top=1, scale=1.0),
           dict(outs=6, ident=3, count=3, keep=2, top=2, scale=1.2),
           dict(outs=64, ident=4, count=8, keep=3, top=6, scale=2.5),
           dict(outs=2, ident=2, count=1, keep=1, top=1, scale=0.5),
           dict(outs=160, ident=0, count=1, keep=1, top=8, scale=1.0)]


@pytest.mark.parametrize("r", ROUTERS)
@pytest.mark.parametrize("with_corr", [True, False])
def test_router(r, with_corr):
    """Softmax over all outputs, the correction for the choice alone, groups, the largest `top`,
    the weights from the scores without the correction, not renormalized."""
    n, S, outs = 97, 2, r["outs"]
    col0, ld = 16, 16 + outs + 3
    P = rnd(S, n, ld, scale=1.2, seed=outs)
    corr = rnd(outs, scale=0.3, seed=outs + 1) if with_corr else None
    rr = {"top": r["top"], "scale": r["scale"], "groups": {"count": r["count"], "keep": r["keep"]}}
    logits = P.sum(0)[:, col0:col0 + outs]
    want = plain_routes(logits, corr if with_corr else torch.zeros(outs), rr)
    first_ident = outs - r["ident"]
    got, skip = ops().moe_route(P.to(DEV), col0, outs, None if corr is None else corr.to(DEV), r["count"],
                                r["keep"], r["top"], first_ident, r["scale"])
    got, skip = got.cpu(), skip.cpu()
    assert ((got > 0).sum(1) == r["top"]).all()
    assert torch.equal(got > 0, want > 0), "another choice"
    assert (got - want).abs().max() <= 1e-6 * r["scale"]
    assert (skip - want[:, first_ident:].sum(1)).abs().max() <= 1e-6 * r["scale"]


def test_router_groups_and_corrections_decide():
    """Scores made by hand: the best single output lies in a group that loses; a negative
    correction keeps an output of a kept group out although its score is the largest; outputs
    of dropped groups are out however negative the kept groups' choice scores are."""
    z = torch.log(torch.tensor([[0.30, 0.02, 0.20, 0.19, 0.05, 0.24]]))       # softmax gives these back (sum 1)
    corr = torch.tensor([-0.5, -0.5, 0.0, 0.0, -0.9, -0.9])
    got, skip = ops().moe_route(z.reshape(1, 1, 6).to(DEV), 0, 6, corr.to(DEV), 3, 1, 2, 5, 3.0)
    # groups (0,1) (2,3) (4,5): choice scores -0.2, -0.48 | 0.20, 0.19 | -0.85, -0.66 -> group 1 alone
    assert torch.allclose(got.cpu(), torch.tensor([[0, 0, 0.60, 0.57, 0, 0]]), atol=1e-6)
    assert float(skip) == 0.0
    # all corrections negative, two groups kept: group 0 and 2 (-0.1 and -0.06); the choice
    # among their outputs goes by the corrected scores, the weights by the plain ones
    corr = torch.tensor([-0.4, -0.35, -0.9, -0.9, -0.6, -0.3])
    got, skip = ops().moe_route(z.reshape(1, 1, 6).to(DEV), 0, 6, corr.to(DEV), 3, 2, 2, 5, 1.0)
    # choice: -0.10, -0.33 | . . | -0.55, -0.06 -> outputs 5 and 0
    assert torch.allclose(got.cpu(), torch.tensor([[0.30, 0, 0, 0, 0, 0.24]]), atol=1e-6)
    assert abs(float(skip) - 0.24) <= 1e-6                   # output 5 is the identity expert


@pytest.mark.parametrize("odt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,E,ff,shared,extra,S", [(5, 6, 40, 24, 11, 1), (70, 3, 30, 0, 5, 2), (9, 0, 0, 40, 3, 1),
                                                   (33, 8, 96, 128, 10, 3), (4, 4, 7, 3, 9, 1)])
def test_weighted_activation(odt, n, E, ff, shared, extra, S):
    """relu(z)^2 times the row's weight for the column's expert; the shared expert's columns bare."""
    width = E * ff + shared
    z = rnd(S, n, width + extra, seed=n)
    wts = rnd(n, E + 2, seed=n + 1).abs()
    wts[:, ::2] = 0.0                                         # experts that were not chosen
    a = torch.relu(z.sum(0)[:, :width]) ** 2
    want = a.clone()
    for e in range(E):
        want[:, e * ff:(e + 1) * ff] *= wts[:, e:e + 1]
    got = ops().activation_weighted(z.to(DEV), width, wts.to(DEV), E, ff, "relu2", odt).float().cpu()
    tol = 1e-6 if odt == torch.float32 else 1e-2
    assert (got - want).abs().max() <= tol * max(1.0, float(want.abs().max()))


# ------------------------------------------------------------ q, k, v: bias, norms, partial rotation, append
class Paged:
    """Rows of several sequences in pages that lie in no order."""

    def __init__(self, lens, seed):
        need = [(n + PAGE - 1) // PAGE for n in lens]
        self.lens = lens
        self.n_pages = sum(need) + 3
        perm = torch.randperm(self.n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
        width = (max(need) + 7) // 8 * 8
        self.table = torch.full((len(lens), width), -1, dtype=torch.int32)
        for i, n in enumerate(need):
            for j in range(n):
                self.table[i, j] = perm.pop()

    def fill(self, per_seq, heads, dim, dtype):
        c = torch.zeros(self.n_pages, heads, PAGE, dim)
        for i, n in enumerate(self.lens):
            for t in range(n):
                c[int(self.table[i, t // PAGE]), :, t % PAGE] = per_seq[i][t]
        return c.to(dtype).to(DEV)

    def read(self, cache, seq, pos):
        return cache[int(self.table[seq, pos // PAGE]), :, pos % PAGE]


def rope_tables(base, dims, n_pos):
    inv = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float32)
    return ops().rope_table(inv.to(DEV), n_pos)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,vd,dims,norms", [(4, 2, 16, 24, 8, True), (3, 3, 10, 6, 0, True),
                                                     (6, 2, 24, 40, 4, False), (2, 2, 128, 128, 128, True),
                                                     (4, 1, 64, 64, 32, True), (4, 2, 128, 64, 32, True)])
def test_bias_norms_partial_rotation_and_append(dtype, nh, nkv, hd, vd, dims, norms):
    lens, rows = [70, 330], [(60, 10), (0, 330)]
    n = sum(c for _, c in rows)
    width = nh * hd + nkv * (hd + vd)
    prod = rnd(2, n, width + 5, seed=5)
    bias = rnd(width, scale=0.5, seed=6)
    qw, kw = (1 + rnd(hd, scale=0.3, seed=7), 1 + rnd(hd, scale=0.3, seed=8)) if norms else (None, None)
    eps = 1e-3
    P = Paged(lens, 9)
    kc, vc = (torch.zeros(P.n_pages, nkv, PAGE, d, dtype=dtype, device=DEV) for d in (hd, vd))
    row_pos, row_seq = row_arrays(rows)
    cos, sin = rope_tables(300.0, dims, 400) if dims else (None, None)
    q = ops().qkv_prepare_append(prod.to(DEV), bias.to(DEV), None if qw is None else qw.to(DEV),
                                 None if kw is None else kw.to(DEV), eps, cos, sin, row_pos.to(DEV),
                                 row_seq.to(DEV), P.table.to(DEV), kc, vc, nh).float().cpu()
    full = prod.sum(0)[:, :width] + bias
    wq = full[:, :nh * hd].reshape(n, nh, hd)
    wk = full[:, nh * hd:nh * hd + nkv * hd].reshape(n, nkv, hd)
    wv = full[:, nh * hd + nkv * hd:].reshape(n, nkv, vd)
    if norms:
        wq, wk = pk.rms(wq, qw, eps), pk.rms(wk, kw, eps)
    wq = pk.rotate_half_partial(wq, row_pos, 300.0, dims)
    wk = pk.rotate_half_partial(wk, row_pos, 300.0, dims)
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    assert (q - wq).abs().max() <= tol * wq.abs().max()
    kc, vc = kc.float().cpu(), vc.float().cpu()
    for r in range(0, n, 7):
        s, p = int(row_seq[r]), int(row_pos[r])
        assert (P.read(kc, s, p) - wk[r]).abs().max() <= tol * wk.abs().max()
        assert (P.read(vc, s, p) - wv[r]).abs().max() <= tol * wv.abs().max()
    if dims and dims < hd:
        # what lies behind the rotated part passes unchanged, at every position
        unrot = pk.rms(full[:, :nh * hd].reshape(n, nh, hd), qw, eps) if norms else full[:, :nh * hd].reshape(n, nh, hd)
        assert (q[..., dims:] - unrot[..., dims:]).abs().max() <= tol * wq.abs().max()
        assert (q[5:, :, :dims] - unrot[5:, :, :dims]).abs().max() > 0.1     # and the first part does turn


# ------------------------------------------------------------ sigmoid attention, window, kept first tokens
def run_sigmoid_attention(dtype, hd, vd, nh, nkv, lens, rows, window=0, keep=0, standout=(), seed=0,
                          decode=False, mode="plain", pb=None, hide=None):
    """rows: per sequence, (first position, count) of the rows that ask.  standout: (sequence, key
    position, query position): that key's score with that query is made large in the LAST head's
    group while all other scores stay far below zero, so that its weight is about one among weights
    near zero.  hide: (sequence, key position): that key's value is made huge; it must not show."""
    P = Paged(lens, seed)
    scale = 0.7 / hd ** 0.5
    ks = [rnd(n, nkv, hd, seed=seed + 10 + i) for i, n in enumerate(lens)]
    vs = [rnd(n, nkv, vd, seed=seed + 50 + i) for i, n in enumerate(lens)]
    qs = [rnd(cnt, nh, hd, seed=seed + 100 + i) for i, (p0, cnt) in enumerate(rows)]
    pb = torch.linspace(-1.0, 0.5, nh) if pb is None else pb
    for (si, kp, qp) in standout:
        p0, cnt = rows[si]
        d = qs[si][qp - p0, nh - 1].clone()
        d = d / d.norm()
        G = nh // nkv
        for a in range(nh - G, nh):
            qs[si][qp - p0, a] = d * 6.0
        ks[si][kp, nkv - 1] = d * (12.0 / scale / 6.0)        # a score of 12 against a bias of -6
        vs[si][kp, nkv - 1] = 5.0
    if dtype == torch.bfloat16:
        qs, ks, vs = [bf(t) for t in qs], [bf(t) for t in ks], [bf(t) for t in vs]
    want = []
    for i, (p0, cnt) in enumerate(rows):
        T = p0 + cnt
        qfull = torch.zeros(T, nh, hd)
        qfull[p0:] = qs[i]
        want.append(pk.sigmoid_attention(qfull, ks[i][:T], vs[i][:T], scale, pb, window or None, keep)[p0:])
    kc, vc = P.fill(ks, nkv, hd, dtype), P.fill(vs, nkv, vd, dtype)
    row_pos, row_seq = row_arrays(rows)
    chunk = ops().attention_chunk()
    max_chunks = int(row_pos.max()) // chunk + 1
    if window:
        # the kept tokens' chunks come first among a row's partial results, always
        max_chunks = min(max_chunks, (window - 1) // chunk + 2) + ops().attention_kept_chunks(window, keep)
    kw = {}
    if mode == "plain":
        kw["force_simt"] = True
    elif not decode:
        per = ops().attention_block_positions(nh, nkv)
        r0, at = [], 0
        for (p0, cnt) in rows:
            r0.append(at)
            at += cnt
        kw["blocks"] = ops().attention_blocks(r0, [p for p, _ in rows], [c for _, c in rows], per,
                                              torch.device(DEV))
    got = ops().attention(torch.cat(qs).to(dtype).to(DEV), kc, vc, row_pos.to(DEV), row_seq.to(DEV),
                          P.table.to(DEV), window, scale, max_chunks, decode=decode,
                          keep_first=keep if window else 0, score_bias=pb.to(DEV), **kw).float().cpu()
    assert ops().attn_tc_error() == 0
    return got, torch.cat(want)


KERNELS = [(torch.float32, "plain", 32, 48), (torch.bfloat16, "plain", 32, 48), (torch.float32, "plain", 128, 64),
           (torch.bfloat16, "tc", 64, 64), (torch.bfloat16, "tc", 128, 128)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd,vd,nh,nkv,window,keep", [(16, 32, 4, 2, 37, 5), (24, 40, 6, 2, 0, 0), (8, 8, 3, 3, 200, 1),
                                                      (64, 64, 4, 1, 130, 64), (128, 128, 2, 2, 64, 130),
                                                      (128, 64, 8, 2, 90, 7), (16, 16, 2, 1, 1, 2)])
def test_sigmoid_attention(dtype, hd, vd, nh, nkv, window, keep):
    lens = [1, 200, 67, 330]
    got, want = run_sigmoid_attention(dtype, hd, vd, nh, nkv, lens, [(0, 1), (0, 200), (60, 7), (329, 1)],
                                      window, keep, seed=3)
    close(got, want, dtype)
    got, want = run_sigmoid_attention(dtype, hd, vd, nh, nkv, lens, [(0, 1), (199, 1), (66, 1), (329, 1)],
                                      window, keep, seed=4, decode=True)
    close(got, want, dtype)


@pytest.mark.parametrize("hd,nh,nkv,window,keep", [(64, 4, 1, 130, 64), (64, 10, 5, 0, 0), (128, 2, 2, 64, 130),
                                                   (128, 8, 2, 1000, 3), (128, 40, 2, 37, 129), (128, 4, 2, 300, 0),
                                                   (128, 6, 2, 100, 9), (64, 12, 2, 260, 5), (128, 24, 2, 140, 4),
                                                   (128, 3, 1, 0, 0)])
def test_sigmoid_attention_on_the_tensor_cores(hd, nh, nkv, window, keep):
    dt = torch.bfloat16
    lens = [1, 300, 131, 1520]
    got, want = run_sigmoid_attention(dt, hd, hd, nh, nkv, lens, [(0, 1), (0, 300), (100, 31), (0, 1520)],
                                      window, keep, seed=4, mode="tc")
    close(got, want, dt, "prompt rows")
    got, want = run_sigmoid_attention(dt, hd, hd, nh, nkv, lens, [(0, 1), (299, 1), (130, 1), (1519, 1)],
                                      window, keep, seed=5, decode=True, mode="tc")
    close(got, want, dt, "decode rows")


def test_the_weights_are_not_normalized():
    """Equal keys and a bias of zero: every visible key weighs one half, so the result grows
    with the number of keys seen; a softmax would give the values' mean."""
    n = 90
    P = Paged([n], 1)
    q = torch.zeros(1, 2, 16)
    k = torch.zeros(n, 1, 16)
    v = torch.ones(n, 1, 16)
    for qp, window, keep, seen in [(89, 0, 0, 90), (89, 30, 0, 30), (89, 30, 7, 37), (20, 30, 7, 21), (33, 30, 7, 34),
                                   (40, 30, 70, 41)]:
        got = ops().attention(q.to(DEV), P.fill([k], 1, 16, torch.float32), P.fill([v], 1, 16, torch.float32),
                              i32([qp]), i32([0]), P.table.to(DEV), window, 1.0,
                              (2 if window else 1) + ops().attention_kept_chunks(window, keep), keep_first=keep,
                              score_bias=torch.tensor([0.0, math.log(3.0)]).to(DEV)).cpu()
        assert abs(float(got[0, 0, 0]) - 0.5 * seen) <= 1e-4, (qp, window, keep)
        assert abs(float(got[0, 1, 0]) - 0.75 * seen) <= 1e-4       # the head's bias: sigmoid(ln 3) = 3/4


@pytest.mark.parametrize("dtype,mode,hd,vd", KERNELS)
@pytest.mark.parametrize("decode", [False, True])
def test_one_key_that_stands_out(dtype, mode, hd, vd, decode):
    """A key far back, at a page's and a chunk's border, and the first one, seen through no window:
    its weight is about one where all others are a few thousandths."""
    n = 900
    pb = torch.full((4,), -6.0)
    for kp, qp in [(3, 899), (0, 700), (63, 899), (64, 640), (127, 128), (128, 899), (767, 768), (512, 513)]:
        rows = [(qp, 1)] if decode else [(max(0, qp - 40), min(41, qp + 1))]
        got, want = run_sigmoid_attention(dtype, hd, vd, 4, 2, [n], rows, 0, 0, standout=[(0, kp, qp)], seed=kp,
                                          decode=decode, mode=mode, pb=pb)
        assert want[-1, 3].mean() > 3.0           # the key does carry its query's result
        close(got, want, dtype, f"key {kp} query {qp}")


@pytest.mark.parametrize("dtype,mode,hd,vd", KERNELS)
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("window,keep", [(1, 2), (37, 5), (64, 64), (128, 1), (200, 130), (96, 6)])
def test_keys_at_the_edges_of_the_window_and_of_the_kept_tokens(dtype, mode, hd, vd, decode, window, keep):
    n = 600
    pb = torch.full((4,), -6.0)
    for qp in (window - 1, window, window + keep, 300, 599):
        rows = [(qp, 1)] if decode else [(max(0, qp - 20), min(21, qp + 1))]
        cases = [(qp + 1 - window, True), (qp - window, qp - window < keep),    # the window's last key, the next
                 (keep - 1, True), (keep, qp - keep < window)]                   # the last kept token, the next
        for kp, seen in cases:
            if kp < 0 or kp > qp:
                continue
            got, want = run_sigmoid_attention(dtype, hd, vd, 4, 2, [n], rows, window, keep,
                                              standout=[(0, kp, qp)], seed=qp, decode=decode, mode=mode, pb=pb)
            if seen:
                assert want[-1, 3].mean() > 3.0, (qp, kp)
            else:
                assert want[-1, 3].mean() < 2.0, (qp, kp)       # just outside: it must not show
            close(got, want, dtype, f"window {window} keep {keep} query {qp} key {kp}")


@pytest.mark.parametrize("window,keep", [(600, 130), (300, 3), (0, 0)])
def test_many_decoded_rows_share_the_device(window, keep):
    """With many rows a block of the tensor-core decode kernel runs over several chunks and
    leaves one partial result for them; the kept tokens' chunks stay partial results of their own."""
    lens = [640 + 3 * i for i in range(40)]
    rows = [(n - 1, 1) for n in lens]
    pb = torch.full((4,), -5.0)
    got, want = run_sigmoid_attention(torch.bfloat16, 128, 128, 4, 2, lens, rows, window, keep, seed=8,
                                      standout=[(7, 2, lens[7] - 1), (9, 131, lens[9] - 1), (11, 300, lens[11] - 1)],
                                      decode=True, mode="tc", pb=pb)
    close(got, want, torch.bfloat16)


# ------------------------------------------------------------------ whole models
LENGTHS = {"KA": [1, 2, 9, 70, 131, 260], "KB": [1, 3, 64, 65, 200, 410], "KC": [2, 17, 128, 129, 300, 520],
           "KD": [1, 5, 33, 64, 190, 330], "KE": [1, 2, 4, 30, 66, 140],
           "KF": [1, 6, 129, 150, 151, 400]}
FP32_TOL = 3e-5
BF16_TOL = 5e-2
_ENGINES = {}


def requests(name):
    rng = np.random.default_rng(900 + len(name) + ord(name[1]))
    return [rng.integers(0, CONFIGS[name]["vocab"], size=n).tolist() for n in LENGTHS[name]]


def engine(name, dtype, max_tokens=2048):
    from janas_b200.engine import Engine
    key = (name, dtype, max_tokens)
    if key not in _ENGINES:
        _ENGINES[key] = Engine.open(model(name)[0], dtype=dtype, max_tokens=max_tokens)
    return _ENGINES[key]


_PLAIN = {}


CLOSE_CALL = 1e-2


def plain_logits(name, toks, rounding=None):
    """The plain model's logits, and for every position how close the closest choice of any of
    its routers was (the gap between the last chosen score and the next)."""
    key = (name, tuple(toks), rounding)
    if key not in _PLAIN:
        _, c, w = model(name)
        margins = []
        logits = pk.forward(c, w, list(toks), rounding, None, margins).numpy()
        m = np.asarray(margins, dtype=np.float64).reshape(-1, len(toks))
        _PLAIN[key] = (logits, m.min(0) if len(m) else np.full(len(toks), np.inf))
    return _PLAIN[key]


def check(name, dtype, got, reqs, ids):
    for rid, toks in zip(ids, reqs):
        have = np.stack([got[rid][p] for p in range(len(toks))])
        if dtype == "float32":
            e = rel_err(have, plain_logits(name, toks)[0])
            assert e <= FP32_TOL, f"{name} {rid} len {len(toks)}: {e:.3e}"
        else:
            # with 16-bit products a router's two scores that are closer than their rounding can
            # change places (rounding moves a choice score by a few thousandths here); such a
            # token takes another expert in either implementation, which is no fault, and the
            # tokens after it see another key, value and state.  So every token before the
            # first such close call is held to the limit, and of the ones from there on a
            # twentieth may be over it (the float32 runs hold every token to theirs).
            want, margin = plain_logits(name, toks, "bfloat16")
            assert np.isfinite(have).all()
            err = np.abs(have - want).max(1) / np.abs(want).max()
            close_calls = np.nonzero(margin < CLOSE_CALL)[0]
            first = int(close_calls[0]) if len(close_calls) else len(toks)
            assert (err[:first] <= BF16_TOL).all(), \
                f"{name} {rid} len {len(toks)}: {err[:first].max():.3e} at {np.nonzero(err[:first] > BF16_TOL)[0].tolist()}"
            over = np.nonzero(err[first:] > BF16_TOL)[0] + first
            assert len(over) <= (len(toks) - first + 19) // 20, f"{name} {rid} len {len(toks)}: over at {over.tolist()}"
            assert np.median(err) <= BF16_TOL / 5 and (err <= 0.5).all(), f"{name} {rid}: {err.max():.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompts(name, dtype):
    reqs = requests(name)
    got = run_trace(engine(name, dtype), trace_whole(reqs))
    check(name, dtype, got, reqs, [f"r{i}" for i in range(len(reqs))])


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_layer_by_layer(name):
    from janas_b200.engine.engine import StepEntry
    toks = requests(name)[3]
    _, c, w = model(name)
    trace = []
    pk.forward(c, w, toks, None, trace)
    e = engine(name, "float32")
    s = e.new_sequence()
    got = e.step_trace([StepEntry(s, toks, [])])
    e.free_sequence(s)
    assert len(got) == len(trace) == len(c["layers"])
    for i, (g, t) in enumerate(zip(got, trace)):
        err = np.abs(np.asarray(g).reshape(t.shape) - t.numpy()).max() / t.abs().max().item()
        assert err <= 1e-5, f"layer {i}: {err:.3e}"


def test_every_part_shows():
    """The plain model with one mechanism changed or left out is far from the engine's logits:
    the comparison tells."""
    name = "KA"
    toks = requests(name)[4]
    _, c, w = model(name)
    have = np.stack([run_trace(engine(name, "float32"), trace_whole([toks]))["r0"][p] for p in range(len(toks))])
    assert rel_err(have, pk.forward(c, w, toks).numpy()) <= FP32_TOL

    def no(key_end):
        def f(d, ww):
            for k in ww:
                if k.endswith(key_end):
                    ww[k] = torch.zeros_like(ww[k])
        return f

    changes = [lambda d, ww: d["layers"][0]["mixer"]["mask"].update(size=36),
               lambda d, ww: d["layers"][0]["mixer"]["mask"].update(keep_first=4),
               lambda d, ww: d["layers"][0]["mixer"]["rot"].update(dims=16),
               lambda d, ww: d["layers"][2]["mixer"]["rot"].update(base=60.0),
               lambda d, ww: d["layers"][0]["mixer"].update(scale=0.25),
               lambda d, ww: d["embedding"].update(scale=7.0),
               lambda d, ww: d["canon"].update(taps=2) or [ww.update({k: v[:, 1:]}) for k, v in list(ww.items()) if "canon" in k],
               lambda d, ww: d["layers"][0]["mlp"]["router"].update(identity=0, experts=8),
               lambda d, ww: d["layers"][0]["mlp"]["router"]["groups"].update(keep=4),
               lambda d, ww: d["layers"][1]["mlp"]["router"].update(top=2),
               lambda d, ww: d["layers"][0]["mlp"]["router"].update(scale=1.0),
               no("mix.pb"), no(".correction"), no("mix.z.b"), no("mix.q.b"), no("canon2"), no("shared.down")]
    for i, change in enumerate(changes):
        d, ww = copy.deepcopy(c), dict(w)
        if i == 7:          # identity experts turned into experts with matrices: they need some
            for L in (0,):
                for e in (6, 7):
                    ww[f"l{L}.mlp.e{e}.up"] = ww[f"l{L}.mlp.e0.up"]
                    ww[f"l{L}.mlp.e{e}.down"] = ww[f"l{L}.mlp.e0.down"]
        change(d, ww)
        assert rel_err(have, pk.forward(d, ww, toks).numpy()) > 1e-3, f"change {i} does not show"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prompt_then_token_by_token(name, dtype):
    reqs = requests(name)
    # long tails: decoding runs over page, chunk and window borders and past the kept tokens
    got = run_trace(engine(name, dtype), trace_tail(reqs, tail=140))
    check(name, dtype, got, reqs, [f"r{i}" for i in range(len(reqs))])


def trace_portions(reqs, sizes):
    """Each request alone, cut into portions whose sizes cycle through ``sizes``."""
    steps, k = [], 0
    for i, toks in enumerate(reqs):
        at, j = 0, i
        while at < len(toks):
            n = min(sizes[j % len(sizes)], len(toks) - at)
            steps.append({"step": k, "entries": [{"id": f"r{i}", "tokens": toks[at:at + n],
                                                  "want": list(range(n))}],
                          "end": [f"r{i}"] if at + n == len(toks) else []})
            at, j, k = at + n, j + 1, k + 1
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["KA", "KB", "KC", "KD", "KF"])
def test_portions(name, dtype):
    """Portions shorter than the convolutions' taps, of a page, over a chunk: the convolutions'
    last inputs and the recurrent state pass from one portion to the next."""
    reqs = requests(name)
    for sizes in ([2], [64, 3, 61, 2, 130], [7, 1, 128]):
        sel = reqs if sizes != [2] else reqs[:4]
        got = run_trace(engine(name, dtype), trace_portions(sel, sizes))
        check(name, dtype, got, sel, [f"r{i}" for i in range(len(sel))])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_batches_of_unequal_requests(name, dtype):
    reqs = requests(name)
    # two batches one after the other in a cache that holds little more than one of them:
    # slots (recurrent state, the convolutions' inputs) and pages are used again by other
    # sequences; the shorter requests end earlier
    b0 = [(reqs[5], len(reqs[5]) - 20), (reqs[0], 1), (reqs[3], len(reqs[3]) - 33), (reqs[2], 2)]
    b1 = [(reqs[4], len(reqs[4]) - 9), (reqs[1], 1), (reqs[3], 40)]
    for b in (b0, b1):
        for i, (t, p) in enumerate(b):
            b[i] = (t, max(1, min(p, len(t))))
    need = max(sum((len(t) + 63) // 64 * 64 for t, _ in b) for b in (b0, b1))
    e = engine(name, dtype, max_tokens=need)
    got = run_trace(e, trace_batches([b0, b1, b0]))
    for b, batch in enumerate([b0, b1, b0]):
        check(name, dtype, got, [t for t, _ in batch], [f"b{b}r{i}" for i in range(len(batch))])
    e.cache.check()
    # in 32-bit a request's logits are the same bits whatever runs beside it
    if dtype == "float32":
        alone = run_trace(e, trace_tail([b0[0][0]], tail=20))
        for p in range(len(b0[0][0])):
            assert np.array_equal(alone["r0"][p], got["b0r0"][p])


def test_state_per_sequence_in_the_cache():
    """The recurrent layers and the convolutions keep their state in the cache manager's slots."""
    e = engine("KA", "bfloat16")
    d = e.cache._op("describe")
    assert any(g.get("window") == 37 and g.get("keep_first") == 5 for g in d["groups"])
    assert len(d["state_entries"]) == 1                         # the one minGRU layer's state
    assert len(d["block_state_entries"]) == 3                   # the convolutions of every layer (both sublayers)


# ------------------------------------------------------------------ generation
@pytest.mark.parametrize("name", ["KA", "KD"])
def test_greedy_generation_through_the_entry_point(name):
    import janas_b200
    folder, c, w = model(name)
    llm = janas_b200.open(folder, janas_b200.LLMParams(n_ctx=512, dtype="float32", max_batch=4, max_tokens=1024))
    prompts = [requests(name)[2], requests(name)[1], requests(name)[3][:50]]
    outs, _ = llm.generate_batch(prompts, [12, 5, 9])
    for p, o, n in zip(prompts, outs, [12, 5, 9]):
        seq = list(p)
        for _ in range(n):
            lg = pk.forward(c, w, seq)[-1]
            top = torch.topk(lg, 2).values
            nxt = int(lg.argmax())
            if (top[0] - top[1]) < 1e-4 * lg.abs().max():
                break                                   # a tie within rounding: stop comparing
            assert o[len(seq) - len(p)] == nxt
            seq.append(nxt)
    llm.close()


def test_long_decoding_with_captured_steps():
    """bfloat16 decode steps are captured and replayed: 300 tokens after a short prompt, a window
    that slides over them past the kept tokens, against the plain model on the whole sequence."""
    name = "KC"
    rng = np.random.default_rng(77)
    toks = rng.integers(0, CONFIGS[name]["vocab"], size=340).tolist()
    got = run_trace(engine(name, "bfloat16"), trace_tail([toks], tail=300))
    check(name, "bfloat16", got, [toks], ["r0"])
