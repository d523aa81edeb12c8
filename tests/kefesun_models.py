"""Small Kefesun configurations with random weights, written as model folders.

The sizes differ from one configuration to the next in everything: width (a multiple of
8 and not), heads and groups, key and value sizes (multiples of 16 and not), rotated
dimensions (a part of the head, the whole head, none), windows (shorter than a page, a
page, longer than a chunk, none) with kept first tokens (fewer than the window, a whole
page, more than the window, none), taps (1 to 5, none), the order of the mixers, minGRU
widths other than the model's, routers with and without identity experts, groups,
corrections that change the choice, a scale of exactly 1, one expert per token, layers
without a feed-forward.  The weights are drawn so that every part shows in the logits.
"""
import json
import os
import tempfile

import torch


def attn(heads, kv_heads, dim, vdim, scale, window=None, keep=0, rot=None, mlp=None):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": vdim}
    if window:
        m["mask"] = {"keep_first": keep, "size": window}
    if rot:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def gru(width, mlp=None):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": mlp}


def moe(experts, ff, top, identity=0, groups=None, scale=1.0, shared=None):
    r = {"experts": experts, "identity": identity, "scale": scale, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"expert": {"ff": ff}, "kind": "moe", "router": r, "shared": {"ff": shared} if shared else None}


def config(width, vocab, layers, taps, eps=1e-5, scale=1.0):
    c = {"architecture": "Kefesun", "embedding": {"scale": scale}, "layers": layers, "norm": {"eps": eps},
         "vocab": vocab, "width": width}
    if taps:
        c["canon"] = {"taps": taps}
    return c


# a window shorter than a page with a few kept tokens, part of the head rotated; a minGRU
# narrower than the model; groups of which half are kept; the whole head rotated on the last layer
KA = config(64, 130, [attn(4, 2, 16, 24, 0.3, window=37, keep=5, rot=(1000.0, 8),
                           mlp=moe(6, 40, 3, identity=2, groups=(4, 2), scale=1.7, shared=24)),
                      gru(48, mlp=moe(6, 40, 3, identity=2, groups=(4, 2), scale=1.7, shared=24)),
                      attn(4, 4, 16, 16, 0.25, window=70, keep=3, rot=(50.0, 16),
                           mlp=moe(5, 24, 2, identity=1, groups=(2, 1), scale=0.8))],
            3, eps=1e-6, scale=8.0)
# multiples of nothing (the products leave the tensor cores); the minGRU first; no window, no
# rotation; two taps; one expert per token, no identity experts, no groups, no shared expert;
# a layer without a feed-forward
KB = config(50, 101, [gru(70, mlp=moe(3, 30, 1)),
                      attn(3, 3, 10, 6, 0.4, mlp=moe(4, 18, 2, identity=2, scale=2.5, shared=10)),
                      attn(6, 2, 24, 40, 0.2, window=200, keep=1, rot=(77.0, 4)),
                      gru(50)],
            2, eps=1e-4, scale=1.0)
# heads of 64 in one group, a window longer than a chunk with a whole page kept; five taps; a
# router whose groups are all kept and whose scale is exactly 1; as many identity experts as others
KC = config(128, 300, [attn(4, 1, 64, 64, 0.11, window=130, keep=64, rot=(100000.0, 32),
                            mlp=moe(4, 72, 4, identity=4, groups=(2, 2), scale=1.0, shared=136)),
                       gru(160, mlp=moe(8, 16, 2, groups=(4, 1), scale=3.0)),
                       attn(4, 1, 64, 64, 0.13, window=130, keep=64, rot=(100000.0, 32),
                            mlp=moe(2, 200, 1, identity=1, scale=1.5, shared=8))],
            5, eps=1e-5, scale=11.3)
# heads of 128 with as many key/value heads; a window of exactly a page with more kept tokens
# than the window is long (three pages of them); one tap (no state of the convolution);
# identity experts alone beside a shared expert
KD = config(96, 211, [attn(2, 2, 128, 128, 0.08, window=64, keep=130, rot=(10000.0, 128),
                           mlp=moe(3, 40, 1, groups=(3, 1), scale=2.0, shared=72)),
                      gru(96, mlp=moe(0, 0, 1, identity=2, scale=0.5, shared=40)),
                      attn(2, 1, 32, 48, 0.15, mlp=moe(3, 40, 2, identity=3, groups=(3, 2), scale=1.2))],
            1, eps=3e-6, scale=5.0)
# no convolution at all; a window of one position beside kept tokens
KE = config(32, 77, [attn(2, 1, 8, 8, 0.5, window=1, keep=2, rot=(10.0, 2), mlp=moe(2, 16, 1, identity=1, scale=1.0)),
                     gru(24, mlp=moe(2, 16, 2, shared=16))],
            None, eps=1e-5, scale=3.0)

# heads of 128 two to a key/value head, a window that crosses a chunk's border with a few kept
# tokens, half a head rotated (prompts and decoding both on the tensor cores in bfloat16); heads
# of 64 four to a key/value head that see every key; three taps
KF = config(144, 190, [attn(4, 2, 128, 128, 0.09, window=150, keep=7, rot=(5000.0, 64),
                            mlp=moe(5, 48, 2, identity=1, groups=(3, 2), scale=1.4, shared=32)),
                       attn(8, 2, 64, 64, 0.12, rot=(300.0, 64), mlp=moe(4, 32, 2, groups=(2, 1), scale=1.1)),
                       gru(144, mlp=moe(3, 56, 1, identity=1, scale=0.9, shared=24))],
            3, eps=2e-5, scale=6.0)

CONFIGS = {"KA": KA, "KB": KB, "KC": KC, "KD": KD, "KE": KE, "KF": KF}
SEEDS = {"KA": 31, "KB": 32, "KC": 33, "KD": 34, "KE": 35, "KF": 36}


def tensor_shapes(c):
    W, V = c["width"], c["vocab"]
    taps = (c.get("canon") or {}).get("taps", 0)
    t = {"embed": (V, W), "final.norm": (W,)}
    for i, layer in enumerate(c["layers"]):
        L, m = f"l{i}", layer["mixer"]
        t[L + ".norm1"] = (W,)
        if taps:
            t[L + ".canon1"] = (W, taps)
        if layer["type"] == "attention":
            H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            t.update({f"{L}.mix.q": (H * D, W), f"{L}.mix.q.b": (H * D,), f"{L}.mix.k": (G * D, W),
                      f"{L}.mix.k.b": (G * D,), f"{L}.mix.v": (G * Dv, W), f"{L}.mix.v.b": (G * Dv,),
                      f"{L}.mix.q.norm": (D,), f"{L}.mix.k.norm": (D,), f"{L}.mix.pb": (H,),
                      f"{L}.mix.o": (W, H * Dv)})
        else:
            Wg = m["width"]
            t.update({f"{L}.mix.z": (Wg, W), f"{L}.mix.z.b": (Wg,), f"{L}.mix.x": (Wg, W), f"{L}.mix.x.b": (Wg,),
                      f"{L}.mix.g": (Wg, W), f"{L}.mix.o": (W, Wg)})
        f = layer["mlp"]
        if f is not None:
            t[L + ".norm2"] = (W,)
            if taps:
                t[L + ".canon2"] = (W, taps)
            r = f["router"]
            for e in range(r["experts"]):
                t[f"{L}.mlp.e{e}.up"] = (f["expert"]["ff"], W)
                t[f"{L}.mlp.e{e}.down"] = (W, f["expert"]["ff"])
            outs = r["experts"] + r.get("identity", 0)
            t[L + ".mlp.router"] = (outs, W)
            t[L + ".mlp.correction"] = (outs,)
            if f.get("shared"):
                t[L + ".mlp.shared.up"] = (f["shared"]["ff"], W)
                t[L + ".mlp.shared.down"] = (W, f["shared"]["ff"])
    return t


def random_weights(c, seed):
    """bfloat16 weights whose every part shows in the logits."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(c).items():
        r = torch.randn(shape, generator=g)
        parts = name.split(".")
        leaf = parts[-1]
        if leaf == "b":
            v = 0.4 * r
        elif leaf == "norm" or leaf.startswith("norm"):
            v = 1.0 + 0.2 * r
        elif leaf.startswith("canon"):
            v = 0.4 * r
        elif leaf == "pb":
            v = -1.5 + 0.7 * r
        elif leaf == "correction":
            v = 0.15 * r                                # as large as the scores: it changes the choice
        elif name == "embed":
            v = 0.3 * r
        elif leaf == "router":
            v = r * (0.6 / (shape[1] ** 0.5))           # scores that differ from expert to expert
        elif leaf in ("q", "k"):
            v = r * (2.0 / (shape[1] ** 0.5))           # weights that differ from key to key
        else:
            v = r * (1.0 / (shape[1] ** 0.5))
        out[name] = v.to(torch.bfloat16)
    return out


_FOLDERS = {}


def write_model(c, weights, prefix="kefesun_"):
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
        _FOLDERS[name] = (write_model(c, w, f"kefesun_{name}_"), c, {k: v.float() for k, v in w.items()})
    return _FOLDERS[name]
