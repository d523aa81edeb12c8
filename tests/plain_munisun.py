"""A plain, slow implementation of the Munisun decoder, for comparison.

Whole sequences, no cache, one function per mechanism, float32 on the CPU.  It
shares no code with ``janas_b200``: the configuration is a dictionary as
``config.json`` holds it, the weights a dictionary name -> float32 tensor.

The design, in this file's notation.  x is the residual stream [T, W]; rms(u) =
u / sqrt(mean(u^2) + eps); N(u, w) = rms(u) (1 + w) is the model's norm.

    x        = E[token] * embedding.scale
    layer i:   x = x + N(mixer(N(x, n1)), n1b);  x = x + N(ff(N(x, n2)), n2b)      (ff optional)
               then the token's own input:  e = Eside[token][i d : (i + 1) d]
               y = P (gelu_tanh(G x) * e);  x = x + rms(y) s
    mixer "parallel":    a softmax attention and a Mamba-2 recurrence read the same h;
               out = left_scale * attention + right_scale * recurrence
      attention: q, k, v = Wq h, Wk h, Wv h;  q, k <- rms per head times a weight of the head's size;
               the first `dims` values of each head turn pair by pair (2i, 2i + 1) by p f_i, f_i =
               base^(-2i/dims), the long wavelengths stretched by rot.scaling;  s = softcap
               tanh((q . k) scale / softcap), causal softmax;  out = Wo (heads * sigmoid(Wg h))
      recurrence: [z | x | B | C | dt] = Win h;  [x | B | C] <- silu(conv(.) + b);  dt <- softplus(dt + dt_bias)
               S_t = exp(-exp(A_log) dt_t) S_{t-1} + dt_t B_t x_t^T;  y_t = S_t^T C_t + D x_t
               out = Wo (rms in norm_groups parts of (y * silu(z)) * w)
    mixer "parallel_2":  a softmax attention and a linear attention with a decay read the same h;
               out = (rms(attention) wl + rms(linear) wr) / 2
      attention: q, k, v = conv(Wq h), conv(Wk h), conv(Wv h);  rotation as above;  q, k <- rms per head,
               no weight;  s = (q . k) scale, causal softmax;  out = Wo heads
      linear:  q, k, v = silu(Wq h), silu(Wk h), silu(Wv h);  S_t = decay_a S_{t-1} + k_t v_t^T;
               o_t = S_t^T q_t;  out = Wo (rms(all heads of o) w * sigmoid(Wg h))
    ff "dense": Wd (silu(Wg h) * (Wu h))
    ff "moe":  s = sigmoid(R h);  choice = s + correction;  experts in `count` equal groups of neighbours,
               a group's score is the sum of its two largest choices, only the `keep` best groups'
               experts can be chosen;  the `top` largest choices among them are;  weight_e = s_e
               out = sum_chosen s_e Wd_e (silu(Wg_e h) * (Wu_e h))
    logits   = Head N(x, final)

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


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_one_plus(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms(x, eps) * (1.0 + w)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def causal_conv(u: torch.Tensor, c: torch.Tensor, history: Optional[torch.Tensor] = None) -> torch.Tensor:
    """u [T, C], c [C, taps] -> sum_j c[:, j] u_{t - taps + 1 + j}; history [taps - 1, C] are the inputs
    before u's first row (zeros when absent)."""
    T, C = u.shape
    taps = c.shape[1]
    past = torch.zeros(taps - 1, C) if history is None else history
    full = torch.cat([past, u], dim=0)
    out = torch.zeros(T, C)
    for j in range(taps):
        out += c[:, j] * full[j:j + T]
    return out


def rotation_frequencies(rot: dict) -> torch.Tensor:
    dims = rot["dims"]
    f = [float(rot["base"]) ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if sc:
        out = []
        for fi in f:
            wavelength = 2.0 * math.pi / fi
            if wavelength < sc["original"] / sc["high"]:
                out.append(fi)
            elif wavelength > sc["original"] / sc["low"]:
                out.append(fi / sc["factor"])
            else:
                s = (sc["original"] / wavelength - sc["low"]) / (sc["high"] - sc["low"])
                out.append((1.0 - s) * fi / sc["factor"] + s * fi)
        f = out
    return torch.tensor(f, dtype=torch.float32)


def rotate_pairs(x: torch.Tensor, pos: torch.Tensor, rot: Optional[dict]) -> torch.Tensor:
    """x [T, heads, D]: values 2i and 2i + 1 of every head turn together, for 2i + 1 < dims."""
    if not rot or not rot.get("dims"):
        return x
    dims = rot["dims"]
    a = pos.to(torch.float32)[:, None] * rotation_frequencies(rot)[None, :]         # [T, dims / 2]
    cos, sin = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def softmax_attention(q, k, v, scale, softcap=None, pos0=0):
    """q [T, H, D] (the last T positions), k [S, G, D], v [S, G, Dv] -> [T, H, Dv]; row t stands at
    position pos0 + t and sees keys 0 .. pos0 + t."""
    T, H, _ = q.shape
    S, G, _ = k.shape
    out = torch.zeros(T, H, v.shape[2])
    i, j = torch.arange(pos0, pos0 + T)[:, None], torch.arange(S)[None, :]
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(j > i, float("-inf"))
        out[:, a] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def gated_attention(h, w, pre, m, eps, rounding=None):
    """The attention of a "parallel" mixer: weighted per-head norms before the rotation, a cap, a gate."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ w[pre + "q"].T).view(T, H, D)
    k = (h @ w[pre + "k"].T).view(T, G, D)
    v = (h @ w[pre + "v"].T).view(T, G, Dv)
    q = rms(q, eps) * w[pre + "q.norm"]
    k = rms(k, eps) * w[pre + "k.norm"]
    q, k = rotate_pairs(q, pos, m.get("rot")), rotate_pairs(k, pos, m.get("rot"))
    q, k, v = _round(q, rounding), _round(k, rounding), _round(v, rounding)
    o = softmax_attention(q, k, v, m["scale"], m.get("softcap")).reshape(T, H * Dv)
    o = _round(_round(o, rounding) * torch.sigmoid(h @ w[pre + "g"].T), rounding)
    return o @ w[pre + "o"].T


def conv_attention(h, w, pre, m, eps, rounding=None):
    """The attention of a "parallel_2" mixer: convolutions after the products, unweighted norms after
    the rotation."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q, k, v = h @ w[pre + "q"].T, h @ w[pre + "k"].T, h @ w[pre + "v"].T
    if m.get("conv"):
        q, k, v = causal_conv(q, w[pre + "q.conv"]), causal_conv(k, w[pre + "k.conv"]), causal_conv(v, w[pre + "v.conv"])
    q, k, v = q.view(T, H, D), k.view(T, G, D), v.view(T, G, Dv)
    q, k = rotate_pairs(q, pos, m.get("rot")), rotate_pairs(k, pos, m.get("rot"))
    q, k = rms(q, eps), rms(k, eps)
    q, k, v = _round(q, rounding), _round(k, rounding), _round(v, rounding)
    o = softmax_attention(q, k, v, m["scale"]).reshape(T, H * Dv)
    return _round(o, rounding) @ w[pre + "o"].T


def mamba2_scan(x, B, C, dt, A_log, D, state=None):
    """x [T, H, P], B and C [T, G, N], dt [T, H] (after the softplus), A_log and D [H] ->
    (y [T, H, P], the last state [H, N, P])."""
    T, H, P = x.shape
    G, N = B.shape[1], B.shape[2]
    S = torch.zeros(H, N, P) if state is None else state.clone()
    y = torch.zeros(T, H, P)
    head_group = torch.arange(H) // (H // G)
    for t in range(T):
        decay = torch.exp(-torch.exp(A_log) * dt[t])                                # [H]
        Bt, Ct = B[t][head_group], C[t][head_group]                                 # [H, N]
        S = decay[:, None, None] * S + dt[t][:, None, None] * Bt[:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnp,hn->hp", S, Ct) + D[:, None] * x[t]
    return y, S


def mamba2_mixer(h, w, pre, m, eps, rounding=None):
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    p = h @ w[pre + "in"].T
    z, xbc, dt = p[:, :inner], p[:, inner:2 * inner + 2 * G * N], p[:, 2 * inner + 2 * G * N:]
    xbc = _round(silu(causal_conv(xbc, w[pre + "conv"]) + w[pre + "conv.b"]), rounding)
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = torch.nn.functional.softplus(dt + w[pre + "dt_bias"], threshold=1e9)
    y, _ = mamba2_scan(x, B, C, dt, w[pre + "A_log"], w[pre + "D"])
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[pre + "norm"]
    return _round(y, rounding) @ w[pre + "o"].T


def decay_scan(q, k, v, decay, state=None):
    """q, k [T, H, D], v [T, H, Dv], decay [H] -> (o [T, H, Dv], the last state [H, D, Dv])."""
    T, H, D = q.shape
    S = torch.zeros(H, D, v.shape[2]) if state is None else state.clone()
    o = torch.zeros(T, H, v.shape[2])
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdp,hd->hp", S, q[t])
    return o, S


def decay_mixer(h, w, pre, m, eps, rounding=None):
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = _round(silu(h @ w[pre + "q"].T), rounding).view(T, H, D)
    k = _round(silu(h @ w[pre + "k"].T), rounding).view(T, H, D)
    v = _round(silu(h @ w[pre + "v"].T), rounding).view(T, H, Dv)
    o, _ = decay_scan(q, k, v, torch.tensor(m["decay"], dtype=torch.float32))
    o = rms(o.reshape(T, H * Dv), eps) * w[pre + "norm"] * torch.sigmoid(h @ w[pre + "g"].T)
    return _round(o, rounding) @ w[pre + "o"].T


def mixer(kind, h, w, pre, m, eps, rounding=None, parts: Optional[dict] = None):
    if kind == "parallel":
        left = gated_attention(h, w, pre + "left.", m["left"], eps, rounding)
        right = mamba2_mixer(h, w, pre + "right.", m["right"], eps, rounding)
        out = m["left_scale"] * left + m["right_scale"] * right
    elif kind == "parallel_2":
        left = conv_attention(h, w, pre + "left.", m["left"], eps, rounding)
        right = decay_mixer(h, w, pre + "right.", m["right"], eps, rounding)
        out = 0.5 * (rms(left, eps) * w[pre + "left.out"] + rms(right, eps) * w[pre + "right.out"])
    else:
        raise ValueError(kind)
    if parts is not None:
        parts["left"], parts["right"] = left, right
    return out


def swiglu(h, gate, up, down, rounding=None):
    return _round(silu(h @ gate.T) * (h @ up.T), rounding) @ down.T


def route(logits: torch.Tensor, correction: torch.Tensor, r: dict, margin: Optional[list] = None):
    """One token's router logits -> (chosen indices, weights)."""
    n = logits.shape[0]
    s = torch.sigmoid(logits)
    choice = s + correction
    groups = r.get("groups") or {"count": 1, "keep": 1}
    count, keep = groups["count"], groups["keep"]
    per = n // count
    gscore = [sum(sorted(choice[g * per:(g + 1) * per].tolist(), reverse=True)[:2]) for g in range(count)]
    best = sorted(range(count), key=lambda g: (-gscore[g], g))[:keep]
    allowed = [e for e in range(n) if e // per in best]
    ranked = sorted(allowed, key=lambda e: (-float(choice[e]), e))
    chosen = ranked[:r["top"]]
    if margin is not None:
        gs = sorted(gscore, reverse=True)
        gaps = [gs[keep - 1] - gs[keep]] if keep < count else []
        if len(ranked) > r["top"]:
            gaps.append(float(choice[ranked[r["top"] - 1]] - choice[ranked[r["top"]]]))
        margin.append(min(gaps) if gaps else float("inf"))
    return chosen, [float(s[e]) for e in chosen]


def moe(h, w, pre, mlp, rounding=None, margin=None):
    r = mlp["router"]
    logits = h @ w[pre + "router"].T
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen, weights = route(logits[t], w[pre + "correction"], r, margin)
        for e, wt in zip(chosen, weights):
            ep = pre + "e%d." % e
            out[t] += wt * swiglu(h[t:t + 1], w[ep + "gate"], w[ep + "up"], w[ep + "down"], rounding)[0]
    return out


def token_side(x, tokens, w, pre, layer_index, dim, eps, rounding=None):
    e = w["side.embed"][torch.tensor(tokens)][:, layer_index * dim:(layer_index + 1) * dim]
    g = gelu_tanh(_round(x, rounding) @ w[pre + "gate"].T) * e
    y = _round(g, rounding) @ w[pre + "proj"].T
    return rms(y, eps) * w[pre + "norm"]


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], rounding: Optional[str] = None,
            trace: Optional[list] = None, margins: Optional[list] = None) -> torch.Tensor:
    """All logits [T, vocab] of one sequence; trace gets the residual stream after every layer,
    margins one list per routed feed-forward: for every token, how close its choice was."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    side = cfg.get("token_side")
    for i, layer in enumerate(cfg["layers"]):
        p = "l%d." % i
        h = _round(norm_one_plus(x, w[p + "norm1"], eps), rounding)
        x = x + norm_one_plus(mixer(layer["type"], h, w, p + "mix.", layer["mixer"], eps, rounding), w[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp:
            h = _round(norm_one_plus(x, w[p + "norm2"], eps), rounding)
            if mlp["kind"] == "dense":
                y = swiglu(h, w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"], rounding)
            else:
                margin = None
                if margins is not None:
                    margin = []
                    margins.append(margin)
                y = moe(h, w, p + "mlp.", mlp, rounding, margin)
            x = x + norm_one_plus(y, w[p + "norm2b"], eps)
        if side:
            x = x + token_side(x, tokens, w, p + "side.", i, side["dim"], eps, rounding)
        if trace is not None:
            trace.append(x.clone())
    h = _round(norm_one_plus(x, w["final.norm"], eps), rounding)
    return h @ w["head"].T
