"""A plain, slow implementation of the Kefesun decoder, for comparison.

Whole sequences, no cache, one function per mechanism, float32 on the CPU.  It
shares no code with ``janas_b200``: the configuration is a dictionary as
``config.json`` holds it, the weights a dictionary name -> float32 tensor.

The design, in this file's notation.  x is the residual stream [T, W].

    x        = E[token] * embedding.scale
    layer:     x = x + LN_1(mixer(short(x, c1)));  x = x + LN_2(ff(short(x, c2)))   (ff optional)
    LN(v)    = (v - mean v) / sqrt(var v + eps) * w                  no bias
    short(v, c)_t = v_t + sum_{j < taps} c[:, j] * v_{t - taps + 1 + j}   (zeros before the start)

    mixer "attention" (H heads, G key/value heads, head a reads a // (H / G)):
               q = Wq h + bq, k = Wk h + bk, v = Wv h + bv
               q, k <- rms(q) wq, rms(k) wk per head; then the first `dims` values of each
               head turn with the position p: (u_i, u_{i + dims/2}) by the angle p base^(-2i/dims)
               s_ij = (q_i . k_j) scale;  j visible from i: j <= i and (i - j < size or j < keep_first)
               p_ij = sigmoid(s_ij + pb_a)  (no sum to one);  out = Wo concat_heads(sum_j p_ij v_j)

    mixer "mingru":
               z = sigmoid(Wz h + bz);  u = Wx h + bx;  c = u + 1/2 (u >= 0), sigmoid(u) (u < 0)
               S_t = (1 - z_t) S_{t-1} + z_t c_t,  S_{-1} = 0;  out = Wo (S_t * silu(Wg h))

    ff "moe":  s = softmax(R h) over experts and identity experts;  choice = s + correction
               experts in `count` equal groups of neighbours; a group's score is its largest choice
               score; only the `keep` best groups' experts can be chosen; the `top` largest choice
               scores among those are chosen; weight_e = s_e * router.scale (not renormalized)
               expert e: Wd_e relu(Wu_e h)^2; an identity expert gives h itself
               out = sum_chosen weight_e expert_e(h) + shared(h)

    logits   = E LN_final(x)

rms(u) = u / sqrt(mean(u^2) + eps).
``rounding="bfloat16"`` rounds activations where a bfloat16 engine stores them.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def _round(x: torch.Tensor, rounding: Optional[str]) -> torch.Tensor:
    if rounding is None:
        return x
    assert rounding == "bfloat16"
    return x.to(torch.bfloat16).to(torch.float32)


def layer_norm_nobias(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    mu = x.mean(dim=-1, keepdim=True)
    d = x - mu
    var = (d * d).mean(dim=-1, keepdim=True)
    return d / torch.sqrt(var + eps) * w


def rms(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def short_conv(v: torch.Tensor, c: torch.Tensor) -> torch.Tensor:
    """v [T, W], c [W, taps] -> v + causal convolution over time, channel by channel."""
    T, W = v.shape
    taps = c.shape[1]
    out = v.clone()
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += c[:, j] * v[s]
    return out


def rotate_half_partial(x: torch.Tensor, pos: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x [T, heads, D]: the first dims values of every head turn, value i with value i + dims/2."""
    if dims == 0:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=torch.float32)
    f = torch.tensor(base, dtype=torch.float32) ** (-2.0 * i / dims)
    a = pos.to(torch.float32)[:, None] * f[None, :]               # [T, half]
    cos, sin = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


def visible(i: int, j: int, size: Optional[int], keep_first: int) -> bool:
    if j > i:
        return False
    if size is None:
        return True
    return i - j < size or j < keep_first


def sigmoid_attention(q, k, v, scale, pb, size, keep_first):
    """q [T, H, D], k [T, G, D], v [T, G, Dv], pb [H] -> [T, H, Dv]; weights are sigmoids, not normalized."""
    T, H, D = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2])
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = j <= i                                    # the same rule as visible(), for all pairs at once
    if size is not None:
        seen = seen & ((i - j < size) | (j < keep_first))
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * scale + pb[a]
        p = torch.sigmoid(s) * seen
        out[:, a] = p @ v[:, g]
    return out


def attention_mixer(h, w, pre, m, eps, rounding=None, pos0=0):
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(pos0, pos0 + T)
    q = (h @ w[pre + "q"].T + w[pre + "q.b"]).view(T, H, D)
    k = (h @ w[pre + "k"].T + w[pre + "k.b"]).view(T, G, D)
    v = (h @ w[pre + "v"].T + w[pre + "v.b"]).view(T, G, Dv)
    q = rms(q, w[pre + "q.norm"], eps)
    k = rms(k, w[pre + "k.norm"], eps)
    rot = m.get("rot")
    if rot:
        q = rotate_half_partial(q, pos, rot["base"], rot["dims"])
        k = rotate_half_partial(k, pos, rot["base"], rot["dims"])
    q, k, v = _round(q, rounding), _round(k, rounding), _round(v, rounding)
    mask = m.get("mask")
    size = mask["size"] if mask else None
    keep = mask.get("keep_first", 0) if mask else 0
    o = sigmoid_attention(q, k, v, m["scale"], w[pre + "pb"], size, keep)
    o = _round(o.reshape(T, H * Dv), rounding)
    return o @ w[pre + "o"].T


def mingru_candidate(u: torch.Tensor) -> torch.Tensor:
    return torch.where(u >= 0, u + 0.5, torch.sigmoid(u))


def mingru_recurrence(zl, u, g, state=None):
    """zl, u, g [T, W]: the gate's and the candidate's pre-activations and the output gate's;
    -> (S_t * silu(g_t) [T, W], the last state)."""
    T, W = zl.shape
    z, c = torch.sigmoid(zl), mingru_candidate(u)
    S = torch.zeros(W) if state is None else state.clone()
    out = torch.zeros(T, W)
    for t in range(T):
        S = (1 - z[t]) * S + z[t] * c[t]
        out[t] = S * (g[t] * torch.sigmoid(g[t]))
    return out, S


def mingru_mixer(h, w, pre, m, rounding=None, state=None):
    out, S = mingru_recurrence(h @ w[pre + "z"].T + w[pre + "z.b"], h @ w[pre + "x"].T + w[pre + "x.b"],
                               h @ w[pre + "g"].T, state)
    out = _round(out, rounding)
    return out @ w[pre + "o"].T, S


def relu2_expert(h, up, down, rounding=None):
    a = torch.relu(h @ up.T) ** 2
    return _round(a, rounding) @ down.T


def route(logits: torch.Tensor, correction: torch.Tensor, r: dict, margin: Optional[list] = None):
    """One token's router logits -> (chosen indices, weights)."""
    n = logits.shape[0]
    s = torch.softmax(logits, dim=0)
    choice = s + correction
    groups = r.get("groups") or {"count": 1, "keep": 1}
    count, keep = groups["count"], groups["keep"]
    per = n // count
    gscore = [max(choice[g * per:(g + 1) * per].tolist()) for g in range(count)]
    best = sorted(range(count), key=lambda g: (-gscore[g], g))[:keep]
    allowed = [e for e in range(n) if e // per in best]
    ranked = sorted(allowed, key=lambda e: (-float(choice[e]), e))
    chosen = ranked[:r["top"]]
    if margin is not None:
        # how far the choice is from another one: the gap between the last kept group and the
        # next, and between the last chosen output and the next allowed one
        gs = sorted(gscore, reverse=True)
        gaps = [gs[keep - 1] - gs[keep]] if keep < count else []
        if len(ranked) > r["top"]:
            gaps.append(float(choice[ranked[r["top"] - 1]] - choice[ranked[r["top"]]]))
        margin.append(min(gaps) if gaps else float("inf"))
    return chosen, [float(s[e]) * r["scale"] for e in chosen]


def moe(h, w, pre, mlp, rounding=None, margin=None):
    r = mlp["router"]
    E, ident = r["experts"], r.get("identity", 0)
    logits = h @ w[pre + "router"].T                 # [T, E + ident]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen, weights = route(logits[t], w[pre + "correction"], r, margin)
        for e, wt in zip(chosen, weights):
            if e >= E:
                out[t] += wt * h[t]
            else:
                out[t] += wt * relu2_expert(h[t:t + 1], w[pre + "e%d.up" % e], w[pre + "e%d.down" % e], rounding)[0]
    if mlp.get("shared"):
        out = out + relu2_expert(h, w[pre + "shared.up"], w[pre + "shared.down"], rounding)
    return out


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], rounding: Optional[str] = None,
            trace: Optional[list] = None, margins: Optional[list] = None) -> torch.Tensor:
    """All logits [T, vocab] of one sequence; trace gets the residual stream after every layer,
    margins one list per routed feed-forward: for every token, how close its choice was."""
    eps = cfg["norm"]["eps"]
    canon = cfg.get("canon")
    x = w["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        p = "l%d." % i
        h = short_conv(x, w[p + "canon1"]) if canon else x
        h = _round(h, rounding)
        if layer["type"] == "attention":
            y = attention_mixer(h, w, p + "mix.", layer["mixer"], eps, rounding)
        elif layer["type"] == "mingru":
            y, _ = mingru_mixer(h, w, p + "mix.", layer["mixer"], rounding)
        else:
            raise ValueError(layer["type"])
        x = x + layer_norm_nobias(y, w[p + "norm1"], eps)
        if layer.get("mlp"):
            h = short_conv(x, w[p + "canon2"]) if canon else x
            h = _round(h, rounding)
            margin = None
            if margins is not None:
                margin = []
                margins.append(margin)
            x = x + layer_norm_nobias(moe(h, w, p + "mlp.", layer["mlp"], rounding, margin), w[p + "norm2"], eps)
        if trace is not None:
            trace.append(x.clone())
    h = _round(layer_norm_nobias(x, w["final.norm"], eps), rounding)
    return h @ w["embed"].T
