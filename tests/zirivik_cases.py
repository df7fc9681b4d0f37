"""Small Zirivik configurations and random weights for the tests, made here (names and shapes written out by hand,
so a loader that expects other names or shapes fails).

The configurations differ from one another in every size and option: width, vocabulary, heads, key and value sizes
(equal and unequal), rotated dimensions (all, some, none), decays, windows (shorter and longer than the sequences),
kept first keys (none, a few, more than a page), key/value heads, shared keys and values, experts and choices per
row, layers without a feed-forward, the order of layers, the embedding's scale, eps and the soft cap.
"""
import json
import os

import torch

from plain_llama import write_safetensors


def retention(heads, dim, vdim, decay, rot=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return {"type": "retention", "mixer": m}


def attention(heads, kv_heads, dim, vdim, scale, size=None, keep_first=0, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size is not None:
        m["mask"] = {"size": size, "keep_first": keep_first}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, limit, experts, top):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def config(width, vocab, layers, scale=1.0, eps=1e-5, cap=30.0):
    return {"architecture": "Zirivik", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps},
            "logit_softcap": cap, "layers": [dict(l, mlp=m) for l, m in layers]}


# every mixer and feed-forward once, small everything; head sizes that are no power of two
CASE_A = config(96, 211, [
    (attention(4, 2, 24, 40, 0.3, size=9, keep_first=2), dense(80)),
    (retention(3, 16, 24, [0.9, 0.97, 0.999], rot=(10000.0, 8)), moe(40, 1.5, 5, 2)),
    (attention(4, 2, 24, 40, 0.2, size=17, keep_first=0, kv_from=0), None),
    (retention(2, 32, 16, [0.95, 1.0]), dense(64)),
], scale=3.0, eps=1e-6, cap=12.0)

# windows around a page's edge, kept first keys beyond a page, one key/value head, all dimensions rotated
CASE_B = config(128, 300, [
    (retention(4, 32, 32, [0.99, 0.995, 0.999, 0.9995], rot=(500000.0, 32)), moe(48, 0.7, 3, 1)),
    (attention(6, 1, 48, 48, 0.15, size=64, keep_first=70), dense(96)),
    (attention(6, 1, 48, 48, 0.15, size=200, keep_first=3, kv_from=1), moe(32, 2.0, 4, 3)),
    (attention(2, 2, 16, 16, 0.25), dense(64)),
], scale=8.0, cap=50.0)

# head sizes the tensor-core attention kernels take (a plain window, nothing kept), and a window with kept keys beside it
CASE_C = config(256, 333, [
    (attention(4, 1, 64, 64, 0.125, size=70), dense(128)),
    (retention(4, 64, 64, [0.98, 0.99, 0.995, 0.999], rot=(10000.0, 32)), moe(64, 1.0, 8, 2)),
    (attention(4, 1, 64, 64, 0.125, size=33, keep_first=4, kv_from=0), dense(128)),
    (attention(2, 2, 128, 128, 0.09), None),
], scale=2.0)

CASES = {"a": CASE_A, "b": CASE_B, "c": CASE_C}


def tensor_shapes(cfg):
    E = cfg["width"]
    shapes = {"embed": (cfg["vocab"], E), "final.norm": (E,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = shapes[p + "norm1b"] = (E,)
        if layer["type"] == "retention":
            shapes[p + "mix.q"] = shapes[p + "mix.k"] = (m["heads"] * m["dim"], E)
            shapes[p + "mix.v"] = shapes[p + "mix.g"] = (m["heads"] * m["vdim"], E)
        else:
            shapes[p + "mix.q"] = (m["heads"] * m["dim"], E)
            if "kv_from" not in m:
                shapes[p + "mix.k"] = (m["kv_heads"] * m["dim"], E)
                shapes[p + "mix.v"] = (m["kv_heads"] * m["vdim"], E)
        shapes[p + "mix.o"] = (E, m["heads"] * m["vdim"])
        mlp = layer["mlp"]
        if mlp is None:
            continue
        shapes[p + "norm2"] = shapes[p + "norm2b"] = (E,)
        if mlp["kind"] == "dense":
            shapes[p + "mlp.up"], shapes[p + "mlp.down"] = (mlp["ff"], E), (E, mlp["ff"])
        else:
            F = mlp["expert"]["ff"]
            shapes[p + "mlp.router"] = (mlp["router"]["experts"], E)
            for e in range(mlp["router"]["experts"]):
                shapes[f"{p}mlp.e{e}.gate"] = shapes[f"{p}mlp.e{e}.up"] = (F, E)
                shapes[f"{p}mlp.e{e}.down"] = (E, F)
    return shapes


def random_weights(cfg, seed, sharp=1.0):
    """bfloat16 tensors: matrices ~ N(0, 1/in), norm weights ~ N(0, 0.2), the table ~ N(0, 1).  ``sharp`` multiplies the
    query and key projections of attention layers, so that a few keys carry each softmax and a key that is wrongly
    seen or missed changes the result by much more than bfloat16 rounding does."""
    g = torch.Generator().manual_seed(seed)
    W = {}
    for name, shape in tensor_shapes(cfg).items():
        if len(shape) == 1:
            t = torch.randn(shape, generator=g) * 0.2
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / shape[1] ** 0.5
            layer = cfg["layers"][int(name.split(".")[0][1:])]
            if layer["type"] == "attention" and name.endswith(("mix.q", "mix.k")):
                t = t * sharp
            if name.endswith("router"):
                t = t * 4.0                      # scores away from one another: the choice of experts is no close call
        W[name] = t.to(torch.bfloat16)
    return W


def write_model(path, cfg, W):
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(path, "model.safetensors"), W)
    return str(path)


def make_model(tmp_path, cfg, seed, sharp=1.0):
    """(model folder, float64 weights for the plain implementation)"""
    W = random_weights(cfg, seed, sharp)
    d = write_model(tmp_path, cfg, W)
    return d, {k: v.to(torch.float64) for k, v in W.items()}
