"""Small Salulorn configurations and random weights for the tests, made here (names and shapes written out by hand, so a
loader that expects other names or shapes fails).

The configurations differ from one another in every size and option: width, vocabulary, heads and key/value heads (one,
some, as many as heads), key and value sizes (equal and unequal), rotated dimensions (all, some, none), taps of the short
convolution (none, 2, 4), windows (shorter and longer than the sequences, around a page's edge, none), capped and
uncapped scores, decay temperatures, latent sizes, rotary scaling (with and without), layers without a feed-forward, the
order of layers, and the loop (none; once; three times over a span in the middle; twice over everything).
"""
import json
import os

import torch

from plain_llama import write_safetensors


def gla(heads, dim, vdim, tau, rank):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}, "rank": rank}


def attention(heads, kv_heads, dim, vdim, scale, conv=None, size=None, rot=None, softcap=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if conv is not None:
        m["conv"] = conv
    if size is not None:
        m["mask"] = {"size": size}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    if softcap is not None:
        m["softcap"] = softcap
    return {"type": "attention", "mixer": m}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, scaling=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale, "rot": rot}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def config(width, vocab, layers, loop=None, eps=1e-5):
    """layers: (mixer, mlp) pairs; the rank of a gla mixer's decay pair is a tensor shape, not a key of the file"""
    c = {"architecture": "Salulorn", "vocab": vocab, "width": width, "norm": {"eps": eps},
         "layers": [{"type": l["type"], "mixer": l["mixer"], "mlp": m} for l, m in layers]}
    if loop is not None:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    return c, [l.get("rank") for l, _ in layers]


# every mixer, small everything, head sizes that are no power of two; a span in the middle runs three times
CASE_A = config(96, 211, [
    (gla(3, 16, 24, 4.0, 5), dense(80)),
    (attention(4, 2, 24, 40, 0.3, conv=4, size=9, rot=(10000.0, 8), softcap=20.0), dense(72)),
    (latent(3, 16, 8, 24, 40, 48, 0.2, 10000.0, scaling=(4.0, 64, 8.0, 1.0)), None),
    (gla(2, 32, 16, 1.0, 12), dense(64)),
], loop=(1, 3, 3), eps=1e-6)

# no loop; windows around a page's edge; attention without convolution, cap or window; as many key/value heads as heads
CASE_B = config(128, 300, [
    (attention(6, 1, 48, 48, 0.15, conv=2, size=64, rot=(500000.0, 48)), dense(96)),
    (latent(4, 24, 16, 40, 32, 72, 0.16, 50000.0), dense(64)),
    (attention(2, 2, 16, 16, 0.25), None),
    (gla(4, 32, 32, 16.0, 8), dense(48)),
    (attention(4, 2, 32, 24, 0.2, size=65, softcap=5.0, rot=(100.0, 16)), dense(64)),
])

# head sizes of 64 and 128, everything looped twice, and a loop that runs once
CASE_C = config(256, 333, [
    (latent(4, 64, 32, 128, 96, 64, 0.1, 10000.0, scaling=(16.0, 128, 32.0, 1.0)), dense(128)),
    (gla(2, 64, 128, 8.0, 16), None),
    (attention(4, 1, 128, 64, 0.09, conv=3, size=70, rot=(250000.0, 64), softcap=30.0), dense(192)),
], loop=(0, 3, 2))
CASE_D = config(64, 90, [(gla(2, 16, 16, 2.0, 4), dense(40)), (attention(2, 1, 16, 16, 0.25, conv=3, size=8, rot=(1000.0, 16)), dense(40))],
                loop=(1, 2, 1))

CASES = {"a": CASE_A, "b": CASE_B, "c": CASE_C, "d": CASE_D}


def tensor_shapes(case):
    cfg, ranks = case
    E = cfg["width"]
    shapes = {"embed": (cfg["vocab"], E), "head": (cfg["vocab"], E), "final.norm": (E,)}
    if "loop" in cfg:
        shapes["loop.in"] = (E, 2 * E)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = (E,)
        x = p + "mix."
        if layer["type"] == "gla":
            shapes[x + "q"] = shapes[x + "k"] = (m["heads"] * m["dim"], E)
            shapes[x + "v"] = shapes[x + "g"] = (m["heads"] * m["vdim"], E)
            shapes[x + "o"] = (E, m["heads"] * m["vdim"])
            shapes[x + "norm"] = (m["vdim"],)
            shapes[x + "a1"], shapes[x + "a2"], shapes[x + "a2.b"] = (ranks[i], E), (m["heads"] * m["dim"], ranks[i]), (m["heads"] * m["dim"],)
        elif layer["type"] == "attention":
            rows = {"q": m["heads"] * m["dim"], "k": m["kv_heads"] * m["dim"], "v": m["kv_heads"] * m["vdim"]}
            for n, r in rows.items():
                shapes[x + n], shapes[x + n + ".b"] = (r, E), (r,)
                if "conv" in m:
                    shapes[x + n + ".conv"] = (r, m["conv"])
            shapes[x + "q.norm"], shapes[x + "k.norm"] = (rows["q"],), (rows["k"],)
            shapes[x + "sink"] = (m["heads"],)
            shapes[x + "o"] = (E, m["heads"] * m["vdim"])
        else:
            H = m["heads"]
            shapes[x + "dq"], shapes[x + "dq.norm"] = (m["q_rank"], E), (m["q_rank"],)
            shapes[x + "uq"] = (H * (m["dim"] + m["rot_dim"]), m["q_rank"])
            shapes[x + "dkv"], shapes[x + "dkv.norm"] = (m["kv_rank"] + m["rot_dim"], E), (m["kv_rank"],)
            shapes[x + "uk"], shapes[x + "uv"] = (H * m["dim"], m["kv_rank"]), (H * m["vdim"], m["kv_rank"])
            shapes[x + "sink"] = (H,)
            shapes[x + "g"], shapes[x + "o"] = (H * m["vdim"], E), (E, H * m["vdim"])
        if layer["mlp"] is not None:
            F = layer["mlp"]["ff"]
            shapes[p + "mlp.gate"] = shapes[p + "mlp.up"] = (F, E)
            shapes[p + "mlp.down"] = (E, F)
    return shapes


def random_weights(case, seed, sharp=1.0, sink=1.0):
    """bfloat16 tensors: matrices ~ N(0, 1/in), norm weights ~ 1 + N(0, 0.2), biases ~ N(0, 0.3), taps ~ N(0, 0.5), sinks ~
    N(0, sink), the table ~ N(0, 1).  ``sharp`` multiplies the query and key projections of the two attention mixers, so
    that a few keys carry each softmax and a key that is wrongly seen or missed changes the result by much more than
    bfloat16 rounding does."""
    cfg, _ = case
    g = torch.Generator().manual_seed(seed)
    W = {}
    for name, shape in tensor_shapes(case).items():
        last = name.split(".")[-1]
        if last in ("norm", "norm1"):
            t = 1.0 + torch.randn(shape, generator=g) * 0.2
        elif last == "sink":
            t = torch.randn(shape, generator=g) * sink
        elif last == "b":
            t = torch.randn(shape, generator=g) * (2.0 if name.endswith("a2.b") else 0.3)
        elif last == "conv":
            t = torch.randn(shape, generator=g) * 0.5
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / shape[1] ** 0.5
            if name[0] == "l" and name[1].isdigit():
                layer = cfg["layers"][int(name.split(".")[0][1:])]
                if layer["type"] != "gla" and last in ("q", "k", "uq", "dkv"):
                    t = t * sharp
                if last == "a2":
                    t = t * 3.0                   # decays spread over (0, 1)
        W[name] = t.to(torch.bfloat16)
    return W


def write_model(path, case, W):
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(case[0], f)
    write_safetensors(os.path.join(path, "model.safetensors"), W)
    return str(path)


def make_model(tmp_path, case, seed, sharp=1.0, sink=1.0):
    """(model folder, float64 weights for the plain implementation)"""
    W = random_weights(case, seed, sharp, sink)
    d = write_model(tmp_path, case, W)
    return d, {k: v.to(torch.float64) for k, v in W.items()}
