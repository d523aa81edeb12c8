"""Small Munisun configurations with random weights, written as model folders.

The sizes differ from one configuration to the next in everything: width (a multiple of 8
and not), heads and key/value heads, key and value sizes, rotated dimensions (a part of the
head, the whole head, none) with and without stretched wavelengths, a cap on the scores and
none, taps of the convolutions (1 to 5, none), the recurrences' heads, states, groups and
norm parts (also 1, and as many as heads), decays (also exactly 1), the two factors (also
exactly 1), the order of the mixers, dense and routed feed-forwards and none, routers with
and without groups (groups of one expert, all groups kept), one expert per token, a token
input per layer and none.  The weights are drawn so that every part shows in the logits.
"""
import json
import os
import tempfile

import torch


def attn(heads, kv_heads, dim, vdim, scale, rot=None, scaling=None, softcap=None, conv=None):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": vdim}
    if rot:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
        if scaling:
            m["rot"]["scaling"] = {"factor": scaling[0], "low": scaling[1], "high": scaling[2], "original": scaling[3]}
    if softcap:
        m["softcap"] = softcap
    if conv:
        m["conv"] = conv
    return m


def par(left, heads, vdim, state, groups, conv, norm_groups, left_scale, right_scale, mlp=None):
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": left, "left_scale": left_scale, "right_scale": right_scale,
                      "right": {"conv": conv, "groups": groups, "heads": heads, "norm_groups": norm_groups,
                                "state": state, "vdim": vdim}}}


def par2(left, heads, dim, vdim, decay, mlp=None):
    return {"type": "parallel_2", "mlp": mlp,
            "mixer": {"left": left, "right": {"decay": decay, "dim": dim, "heads": heads, "vdim": vdim}}}


def dense(ff):
    return {"ff": ff, "kind": "dense"}


def moe(experts, ff, top, groups=None):
    r = {"experts": experts, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"expert": {"ff": ff}, "kind": "moe", "router": r}


def config(width, vocab, layers, side=None, eps=1e-5, scale=1.0):
    c = {"architecture": "Munisun", "embedding": {"scale": scale}, "layers": layers, "norm": {"eps": eps},
         "vocab": vocab, "width": width}
    if side:
        c["token_side"] = {"dim": side}
    return c


# a part of the head rotated with stretched wavelengths, a cap, values longer than keys; a
# recurrence with two groups and two norm parts; then the whole head rotated, three taps, a
# linear attention whose values are longer than its keys; groups of which two of three are kept
MA = config(64, 130, [par(attn(4, 2, 16, 24, 0.3, rot=(1000.0, 8), scaling=(4.0, 1.0, 3.0, 24), softcap=6.0),
                          4, 16, 8, 2, 3, 2, 0.7, 1.1, mlp=dense(96)),
                      par2(attn(2, 1, 32, 16, 0.2, rot=(500.0, 32), conv=3), 3, 8, 24, [0.5, 0.9, 0.99],
                           mlp=moe(6, 40, 2, groups=(3, 2)))],
            side=8, eps=1e-6, scale=4.0)
# multiples of nothing (the products leave the tensor cores); the linear attention first, two
# taps, no rotation; a layer without a feed-forward; no cap, no stretching, one group, one norm
# part, one tap on either side (no state of the convolution), factors of exactly 1; one expert per
# token and no groups; no token input
MB = config(50, 101, [par2(attn(3, 3, 10, 6, 0.4, conv=2), 2, 6, 10, [1.0, 0.7]),
                      par(attn(2, 1, 12, 10, 0.35, rot=(77.0, 4)), 3, 6, 5, 1, 1, 1, 1.0, 1.0, mlp=moe(3, 30, 1)),
                      par2(attn(2, 2, 14, 14, 0.3, rot=(50.0, 6), conv=1), 1, 12, 12, [0.95], mlp=dense(70))],
            eps=1e-4, scale=1.0)
# heads of 64 four to a key/value head and heads of 128 (the tensor cores take both in
# bfloat16); four taps; a recurrence whose state is longer than a thread holds alone; every
# group kept; a token input of sixteen values
MC = config(128, 300, [par2(attn(4, 1, 64, 64, 0.11, rot=(100000.0, 32), conv=4), 2, 64, 64, [0.8, 0.999],
                            mlp=moe(8, 24, 3, groups=(4, 4))),
                       par(attn(2, 2, 128, 128, 0.08, rot=(10000.0, 64), scaling=(6.0, 1.0, 5.0, 64), softcap=30.0),
                           4, 32, 64, 1, 4, 4, 0.5, 1.5, mlp=dense(136)),
                       par2(attn(4, 1, 64, 64, 0.12, rot=(100000.0, 64), conv=4), 2, 64, 64, [0.9, 0.97],
                            mlp=moe(4, 72, 2, groups=(2, 1)))],
            side=16, eps=1e-5, scale=11.3)
# five taps; as many norm parts and groups as heads; groups of one expert each (a group's two
# largest are its one); a state of 40 rows; a rotation without a cap, a cap without a rotation
MD = config(96, 211, [par(attn(2, 2, 16, 16, 0.25, rot=(10000.0, 16)), 4, 12, 40, 4, 5, 4, 1.3, 0.4,
                          mlp=moe(4, 40, 2, groups=(4, 2))),
                      par(attn(6, 2, 16, 8, 0.2, softcap=10.0), 2, 24, 16, 1, 2, 1, 0.9, 0.9, mlp=dense(40)),
                      par2(attn(4, 2, 24, 24, 0.2, rot=(3000.0, 12), conv=5), 4, 12, 12, [0.3, 0.6, 0.9, 0.999])],
            side=4, eps=3e-6, scale=5.0)
# the smallest: one layer of each kind, nothing optional
ME = config(32, 77, [par2(attn(2, 1, 8, 8, 0.5), 2, 8, 8, [0.9, 0.5], mlp=dense(16)),
                     par(attn(2, 1, 8, 8, 0.5), 2, 8, 4, 1, 2, 1, 1.0, 0.5)],
            eps=1e-5, scale=3.0)

CONFIGS = {"MA": MA, "MB": MB, "MC": MC, "MD": MD, "ME": ME}
SEEDS = {"MA": 41, "MB": 42, "MC": 43, "MD": 44, "ME": 45}


def tensor_shapes(c):
    W, V = c["width"], c["vocab"]
    side = (c.get("token_side") or {}).get("dim", 0)
    t = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    if side:
        t["side.embed"] = (V, side * len(c["layers"]))
    for i, layer in enumerate(c["layers"]):
        L, m = f"l{i}", layer["mixer"]
        a, r = m["left"], m["right"]
        H, G, D, Dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
        t.update({f"{L}.norm1": (W,), f"{L}.norm1b": (W,), f"{L}.mix.left.q": (H * D, W),
                  f"{L}.mix.left.k": (G * D, W), f"{L}.mix.left.v": (G * Dv, W), f"{L}.mix.left.o": (W, H * Dv)})
        if layer["type"] == "parallel":
            inner, gn = r["heads"] * r["vdim"], r["groups"] * r["state"]
            t.update({f"{L}.mix.left.q.norm": (D,), f"{L}.mix.left.k.norm": (D,), f"{L}.mix.left.g": (H * Dv, W),
                      f"{L}.mix.right.in": (2 * inner + 2 * gn + r["heads"], W),
                      f"{L}.mix.right.conv": (inner + 2 * gn, r["conv"]), f"{L}.mix.right.conv.b": (inner + 2 * gn,),
                      f"{L}.mix.right.dt_bias": (r["heads"],), f"{L}.mix.right.A_log": (r["heads"],),
                      f"{L}.mix.right.D": (r["heads"],), f"{L}.mix.right.norm": (inner,),
                      f"{L}.mix.right.o": (W, inner)})
        else:
            if a.get("conv"):
                t.update({f"{L}.mix.left.q.conv": (H * D, a["conv"]), f"{L}.mix.left.k.conv": (G * D, a["conv"]),
                          f"{L}.mix.left.v.conv": (G * Dv, a["conv"])})
            qk, vv = r["heads"] * r["dim"], r["heads"] * r["vdim"]
            t.update({f"{L}.mix.right.q": (qk, W), f"{L}.mix.right.k": (qk, W), f"{L}.mix.right.v": (vv, W),
                      f"{L}.mix.right.g": (vv, W), f"{L}.mix.right.o": (W, vv), f"{L}.mix.right.norm": (vv,),
                      f"{L}.mix.left.out": (W,), f"{L}.mix.right.out": (W,)})
        f = layer["mlp"]
        if f is not None:
            t[L + ".norm2"] = (W,)
            t[L + ".norm2b"] = (W,)
            if f["kind"] == "dense":
                t.update({f"{L}.mlp.gate": (f["ff"], W), f"{L}.mlp.up": (f["ff"], W), f"{L}.mlp.down": (W, f["ff"])})
            else:
                for e in range(f["router"]["experts"]):
                    ff = f["expert"]["ff"]
                    t.update({f"{L}.mlp.e{e}.gate": (ff, W), f"{L}.mlp.e{e}.up": (ff, W), f"{L}.mlp.e{e}.down": (W, ff)})
                t[L + ".mlp.router"] = (f["router"]["experts"], W)
                t[L + ".mlp.correction"] = (f["router"]["experts"],)
        if side:
            t.update({f"{L}.side.gate": (side, W), f"{L}.side.proj": (W, side), f"{L}.side.norm": (W,)})
    return t


def random_weights(c, seed):
    """bfloat16 weights whose every part shows in the logits."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(c).items():
        r = torch.randn(shape, generator=g)
        parts = name.split(".")
        leaf = parts[-1]
        if leaf in ("norm1", "norm1b", "norm2", "norm2b") or name == "final.norm":
            v = 0.2 * r                                 # stored around zero: the norm multiplies by 1 + w
        elif leaf in ("norm", "out", "D"):
            v = 1.0 + 0.2 * r
        elif leaf == "conv":
            v = 0.4 * r
        elif leaf == "b":
            v = 0.2 * r
        elif leaf == "dt_bias":
            v = -1.0 + 0.5 * r
        elif leaf == "A_log":
            v = -0.5 + 0.7 * r
        elif leaf == "correction":
            v = 0.15 * r                                # as large as the scores' spread: it changes the choice
        elif name == "embed":
            v = 0.3 * r
        elif name == "side.embed":
            v = r
        elif leaf == "router":
            v = r * (0.6 / (shape[1] ** 0.5))
        elif parts[-2:] in (["left", "q"], ["left", "k"]):
            v = r * (2.0 / (shape[1] ** 0.5))           # weights that differ from key to key
        else:
            v = r * (1.0 / (shape[1] ** 0.5))
        out[name] = v.to(torch.bfloat16)
    return out


_FOLDERS = {}


def write_model(c, weights, prefix="munisun_"):
    from safetensors.torch import save_file
    d = tempfile.mkdtemp(prefix=prefix)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(c, f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(d, "model.safetensors"))
    return d


def model(name):
    """(folder, config, float32 weights) of the named configuration, made once."""
    if name not in _FOLDERS:
        c = CONFIGS[name]
        w = random_weights(c, SEEDS[name])
        _FOLDERS[name] = (write_model(c, w, f"munisun_{name}_"), c, {k: v.float() for k, v in w.items()})
    return _FOLDERS[name]
