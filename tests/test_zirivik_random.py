"""Seeded random Zirivik configurations, engine against the plain implementation: every size, the order and mix of
layers, rotated dimensions, decays, windows, kept keys, shared keys and values, experts and the constants are drawn;
then a batch of unequal prompts, portions, and decode steps during which sequences leave.  float32 engines are held to
the float32 tolerance everywhere; bfloat16 engines run the same model with its expert layers made dense (a router's close
call may turn the rest of a sequence) and sharpened attention."""
import numpy as np
import pytest

import plain_zirivik as pz
from helpers import rel_err
from test_zirivik import TOL, engine_for, entry, without_experts
from zirivik_cases import attention, config, dense, make_model, moe, retention

pytestmark = pytest.mark.gpu


def draw_config(rng):
    width = int(rng.choice([64, 96, 128, 160, 200, 72, 256]))
    n_layers = int(rng.integers(2, 7))
    layers, owners = [], []
    for i in range(n_layers):
        if rng.random() < 0.5:
            dk = int(rng.choice([16, 32, 64, 128, 24, 48]))
            dv = int(rng.choice([16, 32, 64, 128, 24, 40, 96]))
            if dk * dv > 128 * 128:
                dv = 64
            heads = int(rng.integers(1, 5))
            rot = None if rng.random() < 0.2 else (float(rng.choice([10.0, 1e4, 1e6])), int(rng.choice([d for d in (8, 16, 32, 64, 128) if d <= dk])))
            decay = [float(1.0 - 2.0 ** -rng.uniform(1, 11)) for _ in range(heads)]
            mixer = retention(heads, dk, dv, decay, rot=rot)
        else:
            share = owners and rng.random() < 0.4
            if share:
                j, o = owners[int(rng.integers(len(owners)))]
                kv, dk, dv = o["kv_heads"], o["dim"], o["vdim"]
            else:
                kv, dk = int(rng.choice([1, 2, 3])), int(rng.choice([16, 32, 64, 128, 24, 96]))
                dv = dk if rng.random() < 0.6 else int(rng.choice([16, 40, 64, 96]))
            heads = kv * int(rng.choice([1, 2, 4]))
            size = None if rng.random() < 0.2 else int(rng.choice([1, 5, 17, 63, 64, 65, 100, 300]))
            keep = 0 if size is None or rng.random() < 0.3 else int(rng.choice([1, 3, 6, 64, 70]))
            mixer = attention(heads, kv, dk, dv, float(rng.uniform(0.05, 0.3)), size=size, keep_first=keep, kv_from=j if share else None)
            if not share:
                owners.append((i, mixer["mixer"]))
        r = rng.random()
        if r < 0.15:
            mlp = None
        elif r < 0.55:
            mlp = dense(int(rng.choice([64, 100, 192, 320])))
        else:
            X = int(rng.integers(2, 10))
            mlp = moe(int(rng.choice([32, 48, 64, 136])), float(rng.choice([0.5, 1.0, 7.0])), X, int(rng.integers(1, min(X, 3) + 1)))
        layers.append((mixer, mlp))
    return config(width, int(rng.integers(40, 500)), layers, scale=float(rng.choice([1.0, 4.0, 12.0])),
                  eps=float(rng.choice([1e-5, 1e-6])), cap=float(rng.choice([10.0, 30.0, 1e3])))


@pytest.mark.parametrize("seed", [11, 12, 13, 14, 15, 16, 17, 18, 19, 20, 21, 22])
def test_random_configuration(tmp_path, seed):
    rng = np.random.default_rng(seed)
    cfg = draw_config(rng)
    dtype = "bfloat16" if seed % 3 == 0 else "float32"
    if dtype == "bfloat16":
        cfg = without_experts(cfg)
    d, W = make_model(tmp_path, cfg, seed, sharp=2.0 if dtype == "bfloat16" else 1.0)
    B = int(rng.integers(1, 5))
    lens = [int(rng.choice([1, 2, 17, 63, 64, 65, 130, 200])) for _ in range(B)]
    more = [int(rng.choice([0, 2, 33, 70])) for _ in range(B)]          # a second portion of some sequences
    n_dec = int(rng.integers(2, 7))
    toks = [[int(t) for t in rng.integers(0, cfg["vocab"], size=n + m + n_dec)] for n, m in zip(lens, more)]
    want = [pz.plain_forward(cfg, W, t).numpy() for t in toks]
    eng = engine_for(d, dtype, max_tokens=B * 448, max_batch=B)
    slots = [eng.acquire() for _ in range(B)]
    at = [0] * B

    def run(group, counts):
        got = eng.step_host([entry(slots[b], toks[b][at[b]:at[b] + c]) for b, c in zip(group, counts)])
        row = 0
        for b, c in zip(group, counts):
            for i in range(c):
                assert rel_err(got[row], want[b][at[b] + i]) < TOL[dtype], (seed, dtype, b, at[b] + i, cfg["layers"])
                row += 1
            at[b] += c

    run(list(range(B)), lens)
    second = [b for b in range(B) if more[b]]
    if second:
        run(second, [more[b] for b in second])
    alive = list(range(B))
    for _ in range(n_dec):
        run(alive, [1] * len(alive))
        if len(alive) > 1 and rng.random() < 0.4:
            eng.release(slots[alive.pop(int(rng.integers(len(alive))))])
    for b in alive:
        eng.release(slots[b])
    eng.cache.check()
