"""The Munisun design on the GPU: each mechanism's kernel alone against the plain
restatement, then whole models through the engine under every way of cutting the
work, and greedy generation through the library's own entry point."""
import copy

import numpy as np
import pytest
import torch

import plain_munisun as pm
from munisun_models import CONFIGS, model
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


def close(got, want, tol, what=""):
    err = (got - want).abs().max() / want.abs().max()
    assert err <= tol, f"{what} {err:.3e}"


def i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


def row_arrays(rows):
    """rows: per sequence (first position, count) -> positions and sequences of all rows."""
    row_pos = torch.tensor([p for (p0, cnt) in rows for p in range(p0, p0 + cnt)], dtype=torch.int32)
    row_seq = torch.tensor([i for i, (p0, cnt) in enumerate(rows) for _ in range(cnt)], dtype=torch.int32)
    return row_pos, row_seq


def cuts(total, sizes):
    """(first, count) pieces of 0 .. total whose sizes cycle through ``sizes``."""
    out, at, j = [], 0, 0
    while at < total:
        n = min(sizes[j % len(sizes)], total - at)
        out.append((at, n))
        at, j = at + n, j + 1
    return out


# ------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("taps,C,col0,ld,S,silu,bias", [(4, 40, 0, 40, 1, False, False), (3, 25, 7, 50, 2, True, True),
                                                        (2, 8, 8, 16, 1, False, True), (5, 130, 3, 140, 3, True, False),
                                                        (1, 12, 0, 12, 1, True, True), (4, 64, 8, 80, 1, True, True),
                                                        (3, 20, 4, 24, 1, False, False), (2, 128, 0, 128, 1, False, True)])
def test_causal_convolution_and_its_state(taps, C, col0, ld, S, silu, bias):
    """Two sequences of unequal length in one step, then in portions down to one and two rows (shorter
    than the taps), in slots that are not in order: the last taps - 1 inputs pass through the state."""
    lens = [37, 9]
    u = [rnd(S, n, ld, seed=3 + i) for i, n in enumerate(lens)]
    w, b = rnd(C, taps, scale=0.5, seed=1), rnd(C, seed=2) if bias else None

    def plain(i):
        y = pm.causal_conv(u[i].sum(0)[:, col0:col0 + C], w) + (b if bias else 0.0)
        return pm.silu(y) if silu else y

    want = [plain(0), plain(1)]
    slots = [3, 1]
    for sizes in ([1000], [1], [2, 5, 1, 3], [8, 2]):
        state = torch.full((5, max(taps - 1, 1), C), 0.0, device=DEV)
        got = [[], []]
        pieces = [cuts(n, sizes) for n in lens]
        for step in range(max(len(p) for p in pieces)):
            live = [i for i in range(2) if step < len(pieces[i])]
            rows = [pieces[i][step] for i in live]
            row_pos, row_seq = row_arrays(rows)
            x = torch.cat([u[i][:, p0:p0 + cnt] for i, (p0, cnt) in zip(live, rows)], dim=1).contiguous().to(DEV)
            starts = all(p0 == 0 for p0, _ in rows)
            ones = all(cnt == 1 for _, cnt in rows)
            args = (x, col0, C, w.to(DEV), b.to(DEV) if bias else None, state if taps > 1 else None, row_pos.to(DEV),
                    row_seq.to(DEV), i32([slots[i] for i in live]), silu, torch.float32)
            if starts or ones:
                out = ops().causal_conv(*args)
            else:
                out = ops().causal_conv(*args, write_out=True, write_state=False)
                ops().causal_conv(*args, write_out=False, write_state=True)
            at = 0
            for i, (p0, cnt) in zip(live, rows):
                got[i].append(out[at:at + cnt].cpu())
                at += cnt
        for i in range(2):
            close(torch.cat(got[i]), want[i], 2e-6, f"sizes {sizes} sequence {i}")
        assert float(state[0].abs().max()) == 0.0 and float(state[4].abs().max()) == 0.0


@pytest.mark.parametrize("taps", [2, 3, 4])
def test_causal_convolution_of_many_rows(taps):
    """Enough rows for the kernel in which a thread moves along eight of them: two sequences that go on
    from states an earlier step left, the border between them inside a thread's rows."""
    C, lens, first = 2048, [1203, 1301], [5, 2]
    u = [rnd(1, n, C + 8, seed=3 + i) for i, n in enumerate(lens)]
    w, b = rnd(C, taps, scale=0.5, seed=1), rnd(C, seed=2)
    want = [pm.silu(pm.causal_conv(x.sum(0)[:, 4:4 + C], w) + b) for x in u]
    state = torch.zeros(3, taps - 1, C, device=DEV)
    got = [[], []]
    for rows in ([(0, f) for f in first], [(f, n - f) for f, n in zip(first, lens)]):
        row_pos, row_seq = row_arrays(rows)
        x = torch.cat([u[i][:, p0:p0 + cnt] for i, (p0, cnt) in enumerate(rows)], dim=1).contiguous().to(DEV)
        args = (x, 4, C, w.to(DEV), b.to(DEV), state, row_pos.to(DEV), row_seq.to(DEV), i32([2, 0]), True, torch.float32)
        if rows[0][0] == 0:
            out = ops().causal_conv(*args)
        else:
            out = ops().causal_conv(*args, write_out=True, write_state=False)
            ops().causal_conv(*args, write_out=False, write_state=True)
        at = 0
        for i, (p0, cnt) in enumerate(rows):
            got[i].append(out[at:at + cnt].cpu())
            at += cnt
    for i in range(2):
        close(torch.cat(got[i]), want[i], 2e-6, f"sequence {i}")


def scan_inputs(kind, n, H, G, N, P, seed):
    """A product's sums [S, n, ld] with v, k, q (and the steps) at uneven places."""
    S = 2
    if kind == "ssm":
        val0, key0, qry0 = 3, 3 + H * P, 3 + H * P + G * N
        ld = qry0 + G * N + 5
        src = rnd(S, n, ld, scale=0.7, seed=seed)
        dt = rnd(S, n, H + 4, seed=seed + 1)
        return src, (val0, key0, qry0), dt
    qry0, key0, val0 = 0, H * N, 2 * H * N
    src = rnd(S, n, val0 + H * P + 3, scale=0.7, seed=seed)
    return src, (val0, key0, qry0), None


def plain_scan(kind, src, cols, dt, H, G, N, P, params, state=None):
    full = src.sum(0)
    n = full.shape[0]
    val0, key0, qry0 = cols
    v = full[:, val0:val0 + H * P].reshape(n, H, P)
    k = full[:, key0:key0 + G * N].reshape(n, G, N)
    q = full[:, qry0:qry0 + G * N].reshape(n, G, N)
    if kind == "ssm":
        d = torch.nn.functional.softplus(dt.sum(0)[:, 2:2 + H] + params["dt_bias"], threshold=1e9)
        y, S = pm.mamba2_scan(v, k, q, d, params["a_log"], params["skip"], state)
    else:
        y, S = pm.decay_scan(pm.silu(q), pm.silu(k), pm.silu(v), params["decay"], state)
    return y.reshape(n, H * P), S


@pytest.mark.parametrize("kind,H,G,N,P", [("ssm", 4, 2, 8, 16), ("ssm", 3, 1, 5, 6), ("ssm", 2, 2, 40, 12), ("ssm", 4, 1, 64, 32),
                                          ("ssm", 1, 1, 130, 3), ("decay", 3, 3, 8, 24), ("decay", 2, 2, 64, 64),
                                          ("decay", 1, 1, 12, 12), ("decay", 2, 2, 128, 40), ("ssm", 1, 1, 600, 2),
                                          ("decay", 1, 1, 1024, 5)])
def test_matrix_state_recurrence(kind, H, G, N, P):
    """Whole sequences against portions and token by token, two unequal sequences in slots that are
    not in order; the state is what the plain recurrence leaves."""
    lens, slots = [45, 11], [2, 0]
    params = {"dt_bias": rnd(H, seed=5) - 1.0, "a_log": rnd(H, scale=0.7, seed=6) - 0.5, "skip": 1 + rnd(H, scale=0.2, seed=7),
              "decay": torch.tensor([0.5, 0.95, 1.0, 0.8][:H])}
    data = [scan_inputs(kind, n, H, G, N, P, 20 + i) for i, n in enumerate(lens)]
    want = [plain_scan(kind, d[0], d[1], d[2], H, G, N, P, params) for d in data]
    cols = data[0][1]
    for sizes in ([1000], [1], [2, 9, 1, 16], [8]):
        state = torch.zeros(3, H, N, P, device=DEV)
        got = [[], []]
        pieces = [cuts(n, sizes) for n in lens]
        for step in range(max(len(p) for p in pieces)):
            live = [i for i in range(2) if step < len(pieces[i])]
            rows = [pieces[i][step] for i in live]
            _, row_seq = row_arrays(rows)
            src = torch.cat([data[i][0][:, p0:p0 + cnt] for i, (p0, cnt) in zip(live, rows)], dim=1).contiguous().to(DEV)
            kw = {}
            if kind == "ssm":
                kw = dict(dt=torch.cat([data[i][2][:, p0:p0 + cnt] for i, (p0, cnt) in zip(live, rows)], dim=1).contiguous().to(DEV),
                          dt_col0=2, dt_bias=params["dt_bias"].to(DEV), a_log=params["a_log"].to(DEV), skip=params["skip"].to(DEV))
            else:
                kw = dict(decay=params["decay"].to(DEV), silu=True)
            out = ops().matrix_state_scan(src, H, G, N, P, cols[0], cols[1], cols[2], state, row_seq.to(DEV),
                                          i32([slots[i] for i in live]), len(live),
                                          every_row_starts=all(cnt == 1 for _, cnt in rows), **kw)
            at = 0
            for i, (p0, cnt) in zip(live, rows):
                got[i].append(out[at:at + cnt].cpu())
                at += cnt
        for i in range(2):
            close(torch.cat(got[i]), want[i][0], 3e-5, f"{kind} sizes {sizes} sequence {i}")
            close(state[slots[i]].cpu(), want[i][1], 3e-5, f"{kind} sizes {sizes} state {i}")
        assert float(state[1].abs().max()) == 0.0


@pytest.mark.parametrize("kind,H,G,N,P", [("ssm", 2, 1, 16, 8), ("decay", 2, 2, 24, 20), ("ssm", 1, 1, 300, 4)])
def test_long_sequences_in_pieces_side_by_side(kind, H, G, N, P):
    """Sequences long enough to be cut into pieces that run side by side (one of them ends in the middle
    of a piece, one is shorter than a piece), from states that an earlier step left."""
    lens, slots = [40, 9, 3], [1, 3, 0]
    more = [517, 384, 50]
    params = {"dt_bias": rnd(H, seed=5) - 1.0, "a_log": rnd(H, scale=0.7, seed=6) - 0.5, "skip": 1 + rnd(H, scale=0.2, seed=7),
              "decay": torch.tensor([0.97, 1.0][:H])}
    data = [scan_inputs(kind, a + b, H, G, N, P, 30 + i) for i, (a, b) in enumerate(zip(lens, more))]
    want = [plain_scan(kind, d[0], d[1], d[2], H, G, N, P, params) for d in data]
    cols = data[0][1]
    state = torch.zeros(4, H, N, P, device=DEV)
    got = [[], [], []]
    for rows in ([(0, n) for n in lens], [(n, m) for n, m in zip(lens, more)]):
        _, row_seq = row_arrays(rows)
        src = torch.cat([data[i][0][:, p0:p0 + cnt] for i, (p0, cnt) in enumerate(rows)], dim=1).contiguous().to(DEV)
        if kind == "ssm":
            kw = dict(dt=torch.cat([data[i][2][:, p0:p0 + cnt] for i, (p0, cnt) in enumerate(rows)], dim=1).contiguous().to(DEV),
                      dt_col0=2, dt_bias=params["dt_bias"].to(DEV), a_log=params["a_log"].to(DEV), skip=params["skip"].to(DEV))
        else:
            kw = dict(decay=params["decay"].to(DEV), silu=True)
        out = ops().matrix_state_scan(src, H, G, N, P, cols[0], cols[1], cols[2], state, row_seq.to(DEV), i32(slots), 3,
                                      max_len=max(c for _, c in rows), **kw)
        at = 0
        for i, (p0, cnt) in enumerate(rows):
            got[i].append(out[at:at + cnt].cpu())
            at += cnt
    assert ops().lib().jb_matrix_state_scratch(3, max(more), H, N, P) > 0
    for i in range(3):
        close(torch.cat(got[i]), want[i][0], 5e-5, f"{kind} sequence {i}")
        close(state[slots[i]].cpu(), want[i][1], 5e-5, f"{kind} state {i}")
    assert float(state[2].abs().max()) == 0.0


@pytest.mark.parametrize("kind", ["ssm", "decay"])
def test_a_sequences_bits_do_not_depend_on_the_batch(kind):
    """A sequence of 200 rows alone (one pass) and beside one of 600 rows (pieces side by side): the
    same bits, in y and in the state it leaves, also when it goes on from an earlier state."""
    H, G, N, P = 2, 1 if kind == "ssm" else 2, 16, 8
    params = {"dt_bias": rnd(H, seed=5) - 1.0, "a_log": rnd(H, scale=0.7, seed=6) - 0.5, "skip": 1 + rnd(H, scale=0.2, seed=7),
              "decay": torch.tensor([0.97, 0.9])}
    a, b = scan_inputs(kind, 205, H, G, N, P, 61), scan_inputs(kind, 600, H, G, N, P, 62)
    cols = a[1]

    def run(parts, state, slots, max_len):
        rows = [(0, x[0].shape[1]) for x in parts]
        _, row_seq = row_arrays(rows)
        src = torch.cat([x[0] for x in parts], dim=1).contiguous().to(DEV)
        if kind == "ssm":
            kw = dict(dt=torch.cat([x[2] for x in parts], dim=1).contiguous().to(DEV), dt_col0=2,
                      dt_bias=params["dt_bias"].to(DEV), a_log=params["a_log"].to(DEV), skip=params["skip"].to(DEV))
        else:
            kw = dict(decay=params["decay"].to(DEV), silu=True)
        return ops().matrix_state_scan(src, H, G, N, P, cols[0], cols[1], cols[2], state, row_seq.to(DEV), i32(slots),
                                       len(parts), max_len=max_len, **kw)

    def cut(x, lo, hi):
        return (x[0][:, lo:hi], x[1], None if x[2] is None else x[2][:, lo:hi])

    for first in (0, 5):                 # from zero, and on from the state five rows left
        alone, both = torch.zeros(2, H, N, P, device=DEV), torch.zeros(2, H, N, P, device=DEV)
        if first:
            run([cut(a, 0, first)], alone, [1], first)
            run([cut(a, 0, first)], both, [1], first)
        y1 = run([cut(a, first, 205)], alone, [1], 205 - first)
        y2 = run([b, cut(a, first, 205)], both, [0, 1], 600)
        assert torch.equal(y1, y2[600:])
        assert torch.equal(alone[1], both[1])


def test_a_key_far_back_in_the_state():
    """A decay of exactly 1 keeps a key for good, a decay of 0.9 loses it: one key is written 700 tokens
    before the query that asks for it, among keys that are orthogonal to it."""
    H, N, P, n = 2, 16, 8, 760
    src = torch.zeros(1, n, 2 * H * N + H * P)
    src[0, :, H * N:2 * H * N] = -30.0                      # silu(-30) = -3e-12: keys that write next to nothing
    src[0, :, 2 * H * N:] = rnd(n, H * P, seed=1)
    src[0, 40, H * N + 3] = 5.0                             # head 0 writes at position 40 into row 3 of its state
    src[0, 40, 2 * H * N + 3] = 5.0                         # head 1 too
    src[0, :, :H * N] = -30.0
    src[0, 741, 3] = 4.0                                    # both heads ask for row 3 at position 741
    src[0, 741, N + 3] = 4.0
    decay = torch.tensor([1.0, 0.9])
    state = torch.zeros(1, H, N, P, device=DEV)
    first = ops().matrix_state_scan(src[:, :700].contiguous().to(DEV), H, H, N, P, 2 * H * N, H * N, 0, state, i32([0] * 700),
                                    i32([0]), 1, decay=decay.to(DEV), silu=True)
    outs = [first.cpu()]
    for t in range(700, n):                                 # the rest token by token
        outs.append(ops().matrix_state_scan(src[:, t:t + 1].contiguous().to(DEV), H, H, N, P, 2 * H * N, H * N, 0, state,
                                            i32([0]), i32([0]), 1, every_row_starts=True, decay=decay.to(DEV),
                                            silu=True).cpu())
    got = torch.cat(outs)
    want, _ = plain_scan("decay", src, (2 * H * N, H * N, 0), None, H, H, N, P, {"decay": decay})
    close(got, want, 1e-5)
    v40 = pm.silu(src[0, 40, 2 * H * N:2 * H * N + P])
    kept = got[741, :P] / (pm.silu(torch.tensor(5.0)) * pm.silu(torch.tensor(4.0)))
    assert (kept - v40).abs().max() <= 1e-4 * v40.abs().max()          # head 0 still has it whole
    assert got[741, P:].abs().max() <= 1e-8                             # 0.9^701: head 1 has lost it
    assert got[740].abs().max() <= 1e-8 and got[742].abs().max() <= 1e-8   # and nobody else asked (silu(-30) is tiny, not 0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,width,parts,pre,post", [(5, 64, 2, True, False), (3, 72, 1, False, True), (70, 300, 4, True, True),
                                                    (2, 50, 5, False, False), (9, 1024, 1, True, False), (2, 12000, 1, True, True), (8, 2560, 1, False, True),
                                                    (8, 4096, 8, True, False), (3, 2052, 4, True, True)])
def test_gate_then_norm_in_parts(dtype, n, width, parts, pre, post):
    y = rnd(n, width, scale=2.0, seed=1)
    z, g = rnd(2, n, width + 9, seed=2), rnd(3, n, width + 4, seed=3)
    w = 1 + rnd(width, scale=0.2, seed=4)
    v = y * pm.silu(z.sum(0)[:, 5:5 + width]) if pre else y
    want = pm.rms(v.view(n, parts, width // parts), 1e-5).reshape(n, width) * w
    if post:
        want = want * torch.sigmoid(g.sum(0)[:, 4:4 + width])
    for few in (False, True):            # few: the kernel for a decode step's rows, where it takes the sizes
        got = ops().gated_part_norm(y.to(DEV), parts, w.to(DEV), 1e-5, dtype, pre=z.to(DEV) if pre else None, pre_col0=5,
                                    post=g.to(DEV) if post else None, post_col0=4, few_rows=few).float().cpu()
        close(got, want, 3e-6 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("n,m,SL,SR,few", [(1, 50, 1, 1, False), (9, 64, 2, 3, True), (130, 300, 1, 4, False),
                                           (8, 2048, 3, 5, True), (1, 517, 1, 2, True), (32, 4100, 2, 2, True)])
def test_two_results_as_one(n, m, SL, SR, few):
    """few: the kernel for a decode step's rows (several blocks to a row)."""
    L, R = rnd(SL, n, m, seed=1), rnd(SR, n, m, scale=3.0, seed=2)
    got = ops().pair_combine(L.to(DEV), R.to(DEV), None, None, 0.7, 1.1, 0.0, few_rows=few).cpu()
    close(got, 0.7 * L.sum(0) + 1.1 * R.sum(0), 2e-6)
    wl, wr = 1 + rnd(m, scale=0.2, seed=3), 1 + rnd(m, scale=0.2, seed=4)
    got = ops().pair_combine(L.to(DEV), R.to(DEV), wl.to(DEV), wr.to(DEV), 0.5, 0.5, 1e-5, few_rows=few).cpu()
    close(got, 0.5 * (pm.rms(L.sum(0), 1e-5) * wl + pm.rms(R.sum(0), 1e-5) * wr), 2e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_tokens_own_input(dtype):
    n, dim, vocab, cols = 37, 6, 50, 20
    P = rnd(2, n, dim + 2, seed=1)
    table = rnd(vocab, cols, seed=2).to(dtype)
    toks = torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(3), dtype=torch.int32)
    got = ops().token_gate(P.to(DEV), table.to(DEV), 12, dim, toks.to(DEV), dtype).float().cpu()
    want = pm.gelu_tanh(P.sum(0)[:, :dim]) * table.float()[toks.long()][:, 12:12 + dim]
    close(got, want, 2e-6 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("E,count,keep,top", [(12, 4, 3, 4), (6, 3, 2, 2), (4, 4, 2, 2), (8, 4, 4, 3), (3, 1, 1, 1), (64, 8, 3, 6)])
def test_router_with_sigmoids_and_group_sums(E, count, keep, top):
    n = 200
    logits = rnd(2, n, E + 5, seed=E)
    corr = rnd(E, scale=0.3, seed=1)
    w, _ = ops().moe_route(logits.to(DEV), 5, E, corr.to(DEV), count, keep, top, E, 1.0, sigmoid_scores=True, group_best=2)
    w = w.cpu()
    r = {"experts": E, "top": top, "groups": {"count": count, "keep": keep}}
    for t in range(n):
        chosen, weights = pm.route(logits.sum(0)[t, 5:], corr, r)
        want = torch.zeros(E)
        want[chosen] = torch.tensor(weights)
        assert torch.equal(w[t] != 0, want != 0), t
        assert (w[t] - want).abs().max() <= 1e-6


def test_a_groups_two_largest_decide():
    """The group with the largest single score loses to the group whose two largest sum to more; a
    correction below zero makes choice scores negative, and the experts outside the kept groups stay out."""
    s = torch.tensor([[0.9, 0.1, 0.1, 0.6, 0.6, 0.1, 0.5, 0.55, 0.1]]).logit()         # groups of three
    w, _ = ops().moe_route(s.to(DEV), 0, 9, None, 3, 1, 2, 9, 1.0, sigmoid_scores=True, group_best=2)
    assert torch.nonzero(w[0]).flatten().tolist() == [3, 4]
    w, _ = ops().moe_route(s.to(DEV), 0, 9, None, 3, 1, 2, 9, 1.0, sigmoid_scores=True, group_best=1)
    assert torch.nonzero(w[0]).flatten().tolist() == [0, 1]
    corr = torch.full((9,), -2.0)
    w, _ = ops().moe_route(s.to(DEV), 0, 9, corr.to(DEV), 3, 1, 3, 9, 1.0, sigmoid_scores=True, group_best=2)
    assert torch.nonzero(w[0]).flatten().tolist() == [3, 4, 5]
    assert (w[0, 3:6].cpu() - torch.tensor([0.6, 0.6, 0.1])).abs().max() <= 1e-6       # the scores without the correction


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_experts_with_a_gate(dtype):
    n, E, ff = 9, 5, 12
    z = rnd(2, n, 2 * E * ff + 8, seed=1)
    w = torch.rand(n, E + 2, generator=torch.Generator().manual_seed(2))
    w[:, 1] = 0.0
    got = ops().gated_weighted(z.to(DEV), w.to(DEV), E, ff, "silu", dtype).float().cpu()
    full = z.sum(0)[:, :2 * E * ff].reshape(n, E, 2, ff)
    want = (pm.silu(full[:, :, 0]) * full[:, :, 1] * w[:, :E, None]).reshape(n, E * ff)
    close(got, want, 2e-6 if dtype == torch.float32 else 1e-2)


class Paged:
    """Pages of several sequences that lie in no order."""

    def __init__(self, lens, seed):
        need = [(n + PAGE - 1) // PAGE for n in lens]
        self.n_pages = sum(need) + 3
        perm = torch.randperm(self.n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
        self.table = torch.full((len(lens), (max(need) + 7) // 8 * 8), -1, dtype=torch.int32)
        for i, n in enumerate(need):
            for j in range(n):
                self.table[i, j] = perm.pop()


def run_prepared_attention(dtype, nh, nkv, hd, vd, rot, lens, rows, unit, cap=0.0, standout=(), seed=0, decode=False,
                           mode="plain"):
    """The products' sums of whole sequences go through the kernel that norms, turns and appends (pages in
    no order), then the rows of ``rows`` (first position, count per sequence) ask.  standout: (sequence,
    key position, query position): that key is made to dominate that query's scores in every head, through
    values that do not turn."""
    P = Paged(lens, seed)
    scale = 14.0 / hd
    width = nh * hd + nkv * (hd + vd)
    prods = [rnd(n, width, seed=seed + 10 + i) for i, n in enumerate(lens)]
    for (si, kp, qp) in standout:
        for g in range(nkv):
            prods[si][:, nh * hd + g * hd + hd - 1] = 0.0   # no other key has anything there
        for a in range(nh):
            prods[si][qp, a * hd + hd - 1] = 40.0           # the last value of a head does not turn (rot < hd)
        for g in range(nkv):
            prods[si][kp, nh * hd + g * hd + hd - 1] = 40.0
            prods[si][kp, nh * hd + nkv * hd + g * vd:nh * hd + nkv * hd + (g + 1) * vd] = 5.0
    qw, kw_ = (None, None) if unit else (1 + rnd(hd, scale=0.2, seed=1), 1 + rnd(hd, scale=0.2, seed=2))
    if not unit:
        qw[-1] = kw_[-1] = 1.0                               # the place the standout key uses keeps its size
    rot_spec = {"base": 300.0, "dims": rot, "scaling": {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 40}} if rot else None
    f = pm.rotation_frequencies(rot_spec) if rot else None
    want, qs = [], []
    kc, vc = (torch.zeros(P.n_pages, nkv, PAGE, d, dtype=dtype, device=DEV) for d in (hd, vd))
    maxpos = max(lens)
    if rot:
        ang = torch.arange(maxpos, dtype=torch.float32)[:, None] * f[None, :]
        cos, sin = torch.cos(ang.double()).float().to(DEV), torch.sin(ang.double()).float().to(DEV)
    for i, n in enumerate(lens):
        pos = torch.arange(n)
        q = prods[i][:, :nh * hd].reshape(n, nh, hd)
        k = prods[i][:, nh * hd:nh * hd + nkv * hd].reshape(n, nkv, hd)
        v = prods[i][:, nh * hd + nkv * hd:].reshape(n, nkv, vd)
        if not unit:
            q, k = pm.rms(q, 1e-5) * qw, pm.rms(k, 1e-5) * kw_
        q, k = pm.rotate_pairs(q, pos, rot_spec), pm.rotate_pairs(k, pos, rot_spec)
        if unit:
            q, k = pm.rms(q, 1e-5), pm.rms(k, 1e-5)
        if dtype == torch.bfloat16:
            q, k, v = bf(q), bf(k), bf(v)
        p0, cnt = rows[i]
        want.append(pm.softmax_attention(q[p0:p0 + cnt], k[:p0 + cnt], v[:p0 + cnt], scale, cap or None, p0))
        # the kernel under test appends every row of the sequence and gives back q
        row_pos, row_seq = row_arrays([(0, 0)] * i + [(0, n)])
        got_q = ops().qkv_prepare_append(prods[i][None].contiguous().to(DEV), None, None if unit else qw.to(DEV),
                                         None if unit else kw_.to(DEV), 1e-5, cos if rot else None, sin if rot else None,
                                         row_pos.to(DEV), row_seq.to(DEV), P.table.to(DEV), kc, vc, nh, pairs=True,
                                         unit_norm=unit)
        close(got_q.float().cpu(), q, 3e-6 if dtype == torch.float32 else 1e-2, "q")
        qs.append(got_q[p0:p0 + cnt])
    row_pos, row_seq = row_arrays(rows)
    chunk = ops().attention_chunk()
    kw = {}
    if mode == "plain":
        kw["force_simt"] = True
    elif not decode:
        per = ops().attention_block_positions(nh, nkv)
        r0, at = [], 0
        for (p0, cnt) in rows:
            r0.append(at)
            at += cnt
        kw["blocks"] = ops().attention_blocks(r0, [p for p, _ in rows], [c for _, c in rows], per, torch.device(DEV))
    got = ops().attention(torch.cat(qs), kc, vc, row_pos.to(DEV), row_seq.to(DEV), P.table.to(DEV), 0, scale,
                          int(row_pos.max()) // chunk + 1, decode=decode, softcap=cap, **kw).float().cpu()
    assert ops().attn_tc_error() == 0
    return got, torch.cat(want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,vd,rot,unit,cap", [(4, 2, 16, 24, 8, False, 15.0), (3, 3, 10, 6, 4, True, 0.0), (2, 1, 32, 16, 30, True, 0.0),
                                                       (4, 1, 64, 64, 32, True, 0.0), (2, 2, 128, 128, 64, False, 30.0),
                                                       (2, 1, 48, 48, 46, False, 20.0), (2, 2, 12, 12, 0, True, 0.0)])
def test_norms_rotation_and_a_key_far_back(dtype, nh, nkv, hd, vd, rot, unit, cap):
    """q and k normed and turned pair by pair (a part of the head, with stretched wavelengths), keys and
    values appended to pages in no order; then one key far back, at a page's first and last place and
    at a chunk's border is made to stand out among hundreds, for rows of a prompt and for decode rows."""
    lens = [700, 70]
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for kp in (0, 63, 64, 127, 128, 383, 384, 640):
        for decode in (False, True):
            rows = [(699, 1), (69, 1)] if decode else [(650, 50), (0, 70)]
            modes = ["plain"] + (["tc"] if dtype == torch.bfloat16 and hd in (64, 128) and vd == hd else [])
            for mode in modes:
                if kp not in (63, 384) and mode == "plain" and dtype == torch.float32 and decode:
                    continue                        # a few places are enough for the slowest combination
                got, want = run_prepared_attention(dtype, nh, nkv, hd, vd, rot, lens, rows, unit, cap,
                                                   standout=[(0, kp, 699)], seed=kp, decode=decode, mode=mode)
                close(got, want, tol, f"key {kp} decode {decode} {mode}")
                # the row that asked got the key's values, almost alone
                assert abs(float(want[-2 if decode else 49].mean()) - 5.0) < 0.5


# ------------------------------------------------------------------ whole models
LENGTHS = {"MA": [1, 2, 9, 70, 131, 260], "MB": [1, 3, 64, 65, 200, 410], "MC": [2, 17, 128, 129, 300, 520],
           "MD": [1, 5, 33, 64, 190, 330], "ME": [1, 2, 4, 30, 66, 140]}
FP32_TOL = 3e-5
BF16_TOL = 5e-2
CLOSE_CALL = 1e-2
_ENGINES = {}
_PLAIN = {}


def requests(name):
    rng = np.random.default_rng(700 + len(name) + ord(name[1]))
    return [rng.integers(0, CONFIGS[name]["vocab"], size=n).tolist() for n in LENGTHS[name]]


def engine(name, dtype, max_tokens=2048):
    from janas_b200.engine import Engine
    key = (name, dtype, max_tokens)
    if key not in _ENGINES:
        _ENGINES[key] = Engine.open(model(name)[0], dtype=dtype, max_tokens=max_tokens)
    return _ENGINES[key]


def plain_logits(name, toks, rounding=None):
    """The plain model's logits, and for every position how close the closest choice of any of its
    routers was."""
    key = (name, tuple(toks), rounding)
    if key not in _PLAIN:
        _, c, w = model(name)
        margins = []
        logits = pm.forward(c, w, list(toks), rounding, None, margins).numpy()
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
            # With 16-bit products a router's two scores that are closer than their rounding can change
            # places; such a token takes another expert in either implementation, which is no fault, and
            # the tokens after it see other keys, values and states.  Every token before the first such
            # close call is held to the limit, of the ones from there on a twentieth may be over it (the
            # float32 runs hold every token to theirs).
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
    pm.forward(c, w, toks, None, trace)
    e = engine(name, "float32")
    s = e.new_sequence()
    got = e.step_trace([StepEntry(s, toks, [])])
    e.free_sequence(s)
    assert len(got) == len(trace) == len(c["layers"])
    for i, (g, t) in enumerate(zip(got, trace)):
        err = np.abs(np.asarray(g).reshape(t.shape) - t.numpy()).max() / t.abs().max().item()
        assert err <= 1e-5, f"layer {i}: {err:.3e}"


def test_every_part_shows():
    """The plain model with one mechanism changed or left out is far from the engine's logits: the
    comparison tells."""
    name = "MA"
    toks = requests(name)[4]
    _, c, w = model(name)
    have = np.stack([run_trace(engine(name, "float32"), trace_whole([toks]))["r0"][p] for p in range(len(toks))])
    assert rel_err(have, pm.forward(c, w, toks).numpy()) <= FP32_TOL

    def no(key_end, value=0.0):
        def f(d, ww):
            hit = [k for k in ww if k.endswith(key_end)]
            assert hit
            for k in hit:
                ww[k] = torch.full_like(ww[k], value)
        return f

    def swap_taps(d, ww):
        for k in [k for k in ww if k.endswith(".conv")]:
            ww[k] = ww[k].flip(1)

    L0, L1 = (lambda d: d["layers"][0]["mixer"]), (lambda d: d["layers"][1]["mixer"])
    changes = [lambda d, ww: L0(d)["left"]["rot"].update(dims=6),
               lambda d, ww: L0(d)["left"]["rot"].pop("scaling"),
               lambda d, ww: L0(d)["left"]["rot"]["scaling"].update(factor=2.0),
               lambda d, ww: L0(d)["left"].update(softcap=3.0),
               lambda d, ww: L0(d)["left"].pop("softcap"),
               lambda d, ww: L0(d)["left"].update(scale=0.25),
               lambda d, ww: L0(d).update(left_scale=1.0),
               lambda d, ww: L0(d).update(right_scale=1.0),
               lambda d, ww: L0(d)["right"].update(norm_groups=1),
               lambda d, ww: L0(d)["right"].update(norm_groups=4),
               lambda d, ww: L1(d)["left"]["rot"].update(base=60.0),
               lambda d, ww: L1(d)["right"].update(decay=[0.5, 0.9, 0.9]),
               lambda d, ww: d["embedding"].update(scale=3.0),
               lambda d, ww: d["norm"].update(eps=1e-2),
               lambda d, ww: d["layers"][1]["mlp"]["router"]["groups"].update(keep=3),
               lambda d, ww: d["layers"][1]["mlp"]["router"].update(top=1),
               lambda d, ww: d.pop("token_side"),
               swap_taps, no("left.q.norm", 1.0), no("left.g"), no("right.g"), no("conv.b"), no("dt_bias"), no("A_log"),
               no("right.D"), no("l0.mix.right.norm", 1.0), no("l1.mix.right.norm", 1.0), no("left.out", 1.0),
               no("right.out", 1.0), no(".correction"), no("norm1b"), no("norm2"), no("side.norm", 1.0), no("final.norm")]
    for i, change in enumerate(changes):
        d, ww = copy.deepcopy(c), dict(w)
        change(d, ww)
        assert rel_err(have, pm.forward(d, ww, toks).numpy()) > 1e-3, f"change {i} does not show"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prompt_then_token_by_token(name, dtype):
    reqs = requests(name)
    got = run_trace(engine(name, dtype), trace_tail(reqs, tail=140))     # over page and chunk borders
    check(name, dtype, got, reqs, [f"r{i}" for i in range(len(reqs))])


def trace_portions(reqs, sizes):
    """Each request alone, cut into portions whose sizes cycle through ``sizes``."""
    steps, k = [], 0
    for i, toks in enumerate(reqs):
        for (at, n) in cuts(len(toks), sizes[i % len(sizes):] + sizes[:i % len(sizes)]):
            steps.append({"step": k, "entries": [{"id": f"r{i}", "tokens": toks[at:at + n], "want": list(range(n))}],
                          "end": [f"r{i}"] if at + n == len(toks) else []})
            k += 1
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_portions(name, dtype):
    """Portions shorter than the convolutions' taps, of a page, over a chunk: the convolutions' last
    inputs and the recurrences' states pass from one portion to the next."""
    reqs = requests(name)
    for sizes in ([2], [64, 3, 61, 2, 130], [7, 1, 128]):
        sel = reqs if sizes != [2] else reqs[:4]
        got = run_trace(engine(name, dtype), trace_portions(sel, sizes))
        check(name, dtype, got, sel, [f"r{i}" for i in range(len(sel))])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_batches_of_unequal_requests(name, dtype):
    reqs = requests(name)
    # two batches one after the other in a cache that holds little more than one of them: slots (the
    # recurrences' states, the convolutions' inputs) and pages are used again by other sequences
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
    """Every layer's mixer keeps the convolutions' inputs and the recurrence's matrix in the cache
    manager's slots, and its attention side keeps pages."""
    e = engine("MA", "bfloat16")
    d = e.cache._op("describe")
    assert len(d["state_entries"]) == 2 and len(d["groups"]) == 2
    c = CONFIGS["MA"]["layers"]
    r0, a1, r1 = c[0]["mixer"]["right"], c[1]["mixer"]["left"], c[1]["mixer"]["right"]
    conv0 = r0["heads"] * r0["vdim"] + 2 * r0["groups"] * r0["state"]
    want0 = (r0["conv"] - 1) * conv0 + r0["heads"] * r0["state"] * r0["vdim"]
    want1 = (a1["conv"] - 1) * (a1["heads"] * a1["dim"] + a1["kv_heads"] * (a1["dim"] + a1["vdim"])) + \
        r1["heads"] * r1["dim"] * r1["vdim"]
    assert sorted(d["state_bytes"]) == sorted([4 * want0, 4 * want1])


# ------------------------------------------------------------------ generation
@pytest.mark.parametrize("name", ["MA", "MD"])
def test_greedy_generation_through_the_entry_point(name):
    import janas_b200
    folder, c, w = model(name)
    llm = janas_b200.open(folder, janas_b200.LLMParams(n_ctx=512, dtype="float32", max_batch=4, max_tokens=1024))
    prompts = [requests(name)[2], requests(name)[1], requests(name)[3][:50]]
    outs, _ = llm.generate_batch(prompts, [12, 5, 9])
    for p, o, n in zip(prompts, outs, [12, 5, 9]):
        seq = list(p)
        for _ in range(n):
            lg = pm.forward(c, w, seq)[-1]
            top = torch.topk(lg, 2).values
            nxt = int(lg.argmax())
            if (top[0] - top[1]) < 1e-4 * lg.abs().max():
                break                                   # a tie within rounding: stop comparing
            assert o[len(seq) - len(p)] == nxt
            seq.append(nxt)
    llm.close()


def test_long_decoding_with_captured_steps():
    """bfloat16 decode steps are captured and replayed: 300 tokens after a short prompt, against the
    plain model on the whole sequence."""
    name = "MC"
    rng = np.random.default_rng(77)
    toks = rng.integers(0, CONFIGS[name]["vocab"], size=340).tolist()
    got = run_trace(engine(name, "bfloat16"), trace_tail([toks], tail=300))
    check(name, "bfloat16", got, [toks], ["r0"])
