"""A plain, slow implementation of the Salulorn decoder, one function per mechanism, in float64.

It takes the configuration as the dictionary of config.json and the weights as a dictionary name -> tensor, runs ONE
sequence from its first token, and shares no code with the engine.  The tests compare the engine with it.

Notation: T tokens, E the width, H heads, G key/value heads, d the key size of a head, dv its value size.
"""
import math

import torch

F64 = torch.float64


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def rotary_frequencies(rot):
    """Per pair i: the angle's frequency and the amplitude both cos and sin are multiplied by."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def dim_of(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
    ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(half)], dtype=F64)
    f = f / factor * ramp + f * (1.0 - ramp)
    return f, 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, positions, rot):
    """x [T, heads, size]: the first rot.dims entries of each head, members (2i, 2i + 1) of a pair turned by p * f_i."""
    dims = int(rot["dims"])
    f, amp = rotary_frequencies(rot)
    ang = positions.to(F64)[:, None] * f[None, :]                    # [T, dims / 2]
    c, s = (torch.cos(ang) * amp)[:, None, :], (torch.sin(ang) * amp)[:, None, :]
    out = x.clone()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def short_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros in front of the sequence."""
    T, C = u.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], 0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j][None, :]
    return y


def softmax_with_sink(scores, visible, sink):
    """scores [H, T, T] masked by visible [T, T]; the denominator also holds exp(sink_h).  Returns the weights."""
    scores = scores.masked_fill(~visible[None], float("-inf"))
    m = torch.maximum(scores.max(-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(scores - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink[:, None, None] - m))


def gla_mixer(h, W, pre, m, eps):
    """Linear attention with a decay per key channel that depends on the token; state [H, d, dv] from zero."""
    H, d, dv, tau = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["tau"])
    T = h.shape[0]
    q = (h @ W[pre + "q"].T * d ** -0.5).view(T, H, d)
    k = (h @ W[pre + "k"].T).view(T, H, d)
    v = (h @ W[pre + "v"].T).view(T, H, dv)
    z = (h @ W[pre + "a1"].T) @ W[pre + "a2"].T + W[pre + "a2.b"]
    alpha = (torch.sigmoid(z) ** (1.0 / tau)).view(T, H, d)
    S = torch.zeros(H, d, dv, dtype=F64)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_norm(o, W[pre + "norm"], eps).reshape(T, H * dv)
    return (o * silu(h @ W[pre + "g"].T)) @ W[pre + "o"].T


def attention_mixer(h, W, pre, m, eps):
    """Grouped-query attention: biases, a short convolution over time, a norm over the whole of q and of k, rotation
    of the head's first dimensions, capped scores, a sliding window and a sink in the softmax."""
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    pos = torch.arange(T)

    def project(name):
        u = h @ W[pre + name].T
        if pre + name + ".b" in W:
            u = u + W[pre + name + ".b"]
        if pre + name + ".conv" in W:
            u = short_conv(u, W[pre + name + ".conv"])
        return u

    q, k, v = project("q"), project("k"), project("v")
    if pre + "q.norm" in W:
        q = rms_norm(q, W[pre + "q.norm"], eps)
        k = rms_norm(k, W[pre + "k.norm"], eps)
    q, k, v = q.view(T, H, d), k.view(T, G, d), v.view(T, G, dv)
    if m.get("rot"):
        q, k = rotate_pairs(q, pos, m["rot"]), rotate_pairs(k, pos, m["rot"])
    rep = H // G
    kk, vv = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * float(m["scale"])
    if m.get("softcap"):
        cap = float(m["softcap"])
        s = cap * torch.tanh(s / cap)
    diff = pos[:, None] - pos[None, :]
    visible = diff >= 0
    if m.get("mask"):
        visible = visible & (diff < int(m["mask"]["size"]))
    sink = W.get(pre + "sink")
    if sink is None:
        sink = torch.full((H,), float("-inf"), dtype=F64)
    p = softmax_with_sink(s, visible, sink)
    o = torch.einsum("hij,jhv->ihv", p, vv).reshape(T, H * dv)
    return o @ W[pre + "o"].T


def latent_attention_mixer(h, W, pre, m, eps):
    """Attention whose keys and values are expanded from one small latent per token, plus one rotated key part that
    all heads share; queries through a latent of their own; a sink; a sigmoid gate on the heads' output."""
    H, d, dr, dv, r = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    T = h.shape[0]
    pos = torch.arange(T)
    cq = rms_norm(h @ W[pre + "dq"].T, W[pre + "dq.norm"], eps)
    q = (cq @ W[pre + "uq"].T).view(T, H, d + dr)
    q_plain, q_rot = q[..., :d], q[..., d:]
    kv = h @ W[pre + "dkv"].T
    c = rms_norm(kv[:, :r], W[pre + "dkv.norm"], eps)
    k_rot = kv[:, r:].reshape(T, 1, dr)
    rot = dict(m["rot"])
    rot["dims"] = dr
    q_rot, k_rot = rotate_pairs(q_rot, pos, rot), rotate_pairs(k_rot, pos, rot)
    k_plain = (c @ W[pre + "uk"].T).view(T, H, d)
    v = (c @ W[pre + "uv"].T).view(T, H, dv)
    s = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot[:, 0])) * float(m["scale"])
    visible = pos[:, None] >= pos[None, :]
    sink = W.get(pre + "sink")
    if sink is None:
        sink = torch.full((H,), float("-inf"), dtype=F64)
    p = softmax_with_sink(s, visible, sink)
    o = torch.einsum("hij,jhv->ihv", p, v).reshape(T, H * dv)
    o = o * torch.sigmoid(h @ W[pre + "g"].T)
    return o @ W[pre + "o"].T


def dense_ff(h, W, pre):
    return (silu(h @ W[pre + "gate"].T) * (h @ W[pre + "up"].T)) @ W[pre + "down"].T


MIXERS = {"gla": gla_mixer, "attention": attention_mixer, "latent_attention": latent_attention_mixer}


def layer_order(cfg):
    """The layers in the order they run, and whether the looped span's input map comes in front of each."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, False) for i in range(start)]
    for _ in range(times):
        order += [(i, i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, n)]


def forward(cfg, weights, tokens):
    """Logits [T, vocab] and the residual stream after every layer run [runs, T, E] of one sequence."""
    W = {k: v.to(F64) for k, v in weights.items() if v.is_floating_point()}
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x0 = x
    streams = []
    for i, inject in layer_order(cfg):
        layer = cfg["layers"][i]
        pre = "l%d." % i
        if inject:
            x = torch.cat([x, x0], -1) @ W["loop.in"].T
        h = rms_norm(x, W[pre + "norm1"], eps)
        y = MIXERS[layer["type"]](h, W, pre + "mix.", layer["mixer"], eps)
        if layer.get("mlp"):
            y = y + dense_ff(h, W, pre + "mlp.")
        x = x + y
        streams.append(x)
    logits = rms_norm(x, W["final.norm"], eps) @ W["head"].T
    return logits, torch.stack(streams)
