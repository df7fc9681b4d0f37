"""A plain, slow implementation of the Zirivik decoder: one function per mechanism, written from the
design's equations, CPU only.  It shares no code with ``fastgguf_b200``: it reads config.json and the
safetensors file with its own few lines (the reader of ``plain_llama``) and keeps its own per-sequence memory.

The design, in this file's notation (rows are tokens, ``W`` is stored [out, in] and applied as ``x @ W.T``):

* embedding:  x = embed[token] * embedding.scale
* a layer:    x += norm1b(mixer(norm1(x)));  x += norm2b(ff(norm2(x)))  (the second line only if the layer has a
              feed-forward);  norm(x) = x / sqrt(mean(x^2) + eps) * (1 + w)
* retention:  q, k rotated on the first ``rot.dims`` dimensions of each head (pairs (i, i + dims/2), angle
              pos * base^(-2i/dims)), k * dim^-0.5 after the rotation; per head S <- decay_h S + k v^T, o = S^T q;
              o / rms(o) per head (eps, no weight); (concat o) * silu(W_g h); then W_o
* attention:  no rotation; score = q.k * scale; row i sees key j when j <= i and (i - j < size or j < keep_first);
              softmax; query head h reads key/value head h // (H / G); a layer with ``kv_from: j`` has no key and
              value projections and reads what layer j computed
* dense ff:   W_down relu(W_up h)^2
* experts:    z = W_router h, s = sigmoid(z); the ``top`` largest s are chosen, their s are the weights (not
              renormalised); out = sum_e expert_e(s_e h); expert(x): g = min(W_gate x, limit),
              u = clamp(W_up x, -limit, limit), W_down (g sigmoid(1.702 g) (u + 1))
* output:     logits = cap tanh((norm_final(x) @ embed.T) / cap)

``Memory`` carries what a sequence leaves behind (retention states, keys and values, its length), so the same
functions run a whole prompt, a portion of it, or one token.
"""
import json
import math
import os

import torch

from plain_llama import read_safetensors


def read_model_folder(model_dir, dtype=torch.float64):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    W = {k: (t.to(dtype) if t.dtype.is_floating_point else t)
         for k, t in read_safetensors(os.path.join(model_dir, "model.safetensors")).items()}
    return cfg, W


# ------------------------------------------------------------------------------ small pieces
def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) along the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm whose weight is stored around zero."""
    return unit_rms(x, eps) * (1.0 + w)


def rotate_front(x, positions, dims, base):
    """x: [T, heads, d]; rotates pairs (i, i + dims/2) of the first ``dims`` dimensions by positions * base^(-2i/dims)."""
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(x.dtype)[:, None] * freq[None, :]            # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b, rest = x[..., :half], x[..., half:dims], x[..., dims:]
    return torch.cat([a * c - b * s, b * c + a * s, rest], dim=-1)


def silu(z):
    return z * torch.sigmoid(z)


# ------------------------------------------------------------------------------ mixers
def retention_mixer(h, positions, W, p, mc, eps, state):
    """h: [T, E]; state: [heads, dim, vdim] (updated in place and returned); one token after another."""
    H, dk, dv = mc["heads"], mc["dim"], mc["vdim"]
    T = h.shape[0]
    q = (h @ W[p + "q"].T).reshape(T, H, dk)
    k = (h @ W[p + "k"].T).reshape(T, H, dk)
    v = (h @ W[p + "v"].T).reshape(T, H, dv)
    if mc.get("rot"):                                   # a mixer without "rot" does not rotate
        q = rotate_front(q, positions, mc["rot"]["dims"], mc["rot"]["base"])
        k = rotate_front(k, positions, mc["rot"]["dims"], mc["rot"]["base"])
    k = k * dk ** -0.5
    decay = torch.tensor(mc["decay"], dtype=h.dtype)[:, None, None]
    o = torch.empty(T, H, dv, dtype=h.dtype)
    for t in range(T):
        state.mul_(decay).add_(k[t][:, :, None] * v[t][:, None, :])
        o[t] = torch.einsum("hkv,hk->hv", state, q[t])
    o = unit_rms(o, eps).reshape(T, H * dv)
    return (o * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


def visible(i, j, size, keep_first):
    """May the row at position i read the key at position j?"""
    return j <= i and (i - j < size or j < keep_first)


def attention_mixer(h, positions, W, p, mc, keys, values):
    """h: [T, E]; keys [P, G, dim], values [P, G, vdim]: everything up to and including this portion's tokens."""
    H, G, dk, dv = mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"]
    T, P = h.shape[0], keys.shape[0]
    q = (h @ W[p + "q"].T).reshape(T, H, dk)
    size, keep = (mc["mask"]["size"], mc["mask"]["keep_first"]) if mc.get("mask") else (P + 1, 0)   # no mask: every earlier key
    mask = torch.tensor([[visible(int(i), j, size, keep) for j in range(P)] for i in positions])
    out = torch.empty(T, H, dv, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ keys[:, g].T) * mc["scale"]
        s = s.masked_fill(~mask, -math.inf)
        out[:, head] = torch.softmax(s, dim=-1) @ values[:, g]
    return out.reshape(T, H * dv) @ W[p + "o"].T


# ------------------------------------------------------------------------------ feed-forwards
def dense_ff(h, W, p):
    return torch.relu(h @ W[p + "up"].T) ** 2 @ W[p + "down"].T


def expert(x, W, p, limit):
    g = torch.clamp(x @ W[p + "gate"].T, max=limit)
    u = torch.clamp(x @ W[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def route(h, W, p, top):
    """(indices [T, top], weights [T, top]): the largest sigmoid scores, as they are."""
    s = torch.sigmoid(h @ W[p + "router"].T)
    w, idx = torch.topk(s, top, dim=-1)
    return idx, w


def expert_ff(h, W, p, mlp):
    idx, w = route(h, W, p, mlp["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(idx[t].tolist(), w[t]):
            out[t] += expert(s * h[t:t + 1], W, f"{p}e{e}.", mlp["expert"]["limit"])[0]
    return out


# ------------------------------------------------------------------------------ the model
class Memory:
    """What one sequence has left behind."""

    def __init__(self, cfg, dtype=torch.float64):
        self.length = 0
        self.state, self.keys, self.values = {}, {}, {}
        for i, layer in enumerate(cfg["layers"]):
            mc = layer["mixer"]
            if layer["type"] == "retention":
                self.state[i] = torch.zeros(mc["heads"], mc["dim"], mc["vdim"], dtype=dtype)
            elif "kv_from" not in mc:
                self.keys[i] = torch.zeros(0, mc["kv_heads"], mc["dim"], dtype=dtype)
                self.values[i] = torch.zeros(0, mc["kv_heads"], mc["vdim"], dtype=dtype)


def plain_step(cfg, W, tokens, mem, residuals=None):
    """Runs ``tokens`` as the next portion of the sequence behind ``mem``; logits [T, vocab].
    residuals (a list) receives the residual stream after every layer."""
    dtype = W["embed"].dtype
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    positions = torch.arange(mem.length, mem.length + T)
    x = W["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        p, mc = f"l{i}.", layer["mixer"]
        h = offset_norm(x, W[p + "norm1"], eps)
        if layer["type"] == "retention":
            y = retention_mixer(h, positions, W, p + "mix.", mc, eps, mem.state[i])
        elif layer["type"] == "attention":
            src = mc.get("kv_from", i)
            if src == i:
                G = mc["kv_heads"]
                mem.keys[i] = torch.cat([mem.keys[i], (h @ W[p + "mix.k"].T).reshape(T, G, mc["dim"])])
                mem.values[i] = torch.cat([mem.values[i], (h @ W[p + "mix.v"].T).reshape(T, G, mc["vdim"])])
            y = attention_mixer(h, positions, W, p + "mix.", mc, mem.keys[src], mem.values[src])
        else:
            raise ValueError(f"layer type {layer['type']!r}")
        x = x + offset_norm(y, W[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = offset_norm(x, W[p + "norm2"], eps)
            y = dense_ff(h, W, p + "mlp.") if mlp["kind"] == "dense" else expert_ff(h, W, p + "mlp.", mlp)
            x = x + offset_norm(y, W[p + "norm2b"], eps)
        if residuals is not None:
            residuals.append(x.clone())
    mem.length += T
    cap = cfg["logit_softcap"]
    logits = offset_norm(x, W["final.norm"], eps) @ W["embed"].T
    return (cap * torch.tanh(logits / cap)).to(dtype)


def plain_forward(cfg, W, tokens, residuals=None):
    """A whole sequence from its first token: logits [T, vocab]."""
    return plain_step(cfg, W, tokens, Memory(cfg, W["embed"].dtype), residuals)
