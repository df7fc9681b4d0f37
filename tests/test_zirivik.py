"""The Zirivik decoder in the engine against the plain implementation (``plain_zirivik``): each mechanism alone,
whole prompts, portions, decoding, batches, reused slots and pages, and generation through the entry point.

Structure is tested in float32, where any key wrongly seen or missed, any state lost or kept too long is orders of
magnitude above the tolerance; the bfloat16 runs use sharpened attention (see ``zirivik_cases.random_weights``) so that
the same faults stay visible above rounding.  In bfloat16 a router score that nearly ties with the next one may fall the
other way than in the float64 plain implementation, and everything after it in the sequence then differs: the position-by-
position bfloat16 runs therefore use the cases with every expert layer made dense, and the expert layers inside a
bfloat16 model are judged by how many positions agree."""
import numpy as np
import pytest
import torch

import plain_zirivik as pz
from helpers import rel_err
from zirivik_cases import CASES, attention, config, dense, make_model, moe, retention

pytestmark = pytest.mark.gpu

#: max |dlogit| / max |logit| against the float64 plain implementation; about twice the worst any test shows (float32
#: 5.9e-6 among the random configurations, bfloat16 3.7e-2); a key wrongly seen or a lost state is at 1e-3 and above
TOL = {"float32": 1.5e-5, "bfloat16": 6e-2}


def tokens_for(cfg, n, seed):
    rng = np.random.default_rng(seed)
    return [int(t) for t in rng.integers(0, cfg["vocab"], size=n)]


def engine_for(model_dir, dtype, **kw):
    from fastgguf_b200.engine.api import Engine
    args = dict(dtype=dtype, max_tokens=4096, max_batch=8)
    args.update(kw)
    return Engine.from_dir(model_dir, **args)


def entry(slot, toks, want=None):
    from fastgguf_b200.engine.batch import StepEntry
    return StepEntry(slot, toks, list(range(len(toks))) if want is None else want)


def without_experts(cfg):
    layers = [dict(l, mlp=dense(l["mlp"]["expert"]["ff"]) if l["mlp"] and l["mlp"]["kind"] == "moe" else l["mlp"]) for l in cfg["layers"]]
    return dict(cfg, layers=layers)


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """(case, 1.0): the case as it is; (case, 2.0): attention sharpened and expert layers made dense, for bfloat16."""
    out = {}
    for i, (name, cfg) in enumerate(CASES.items()):
        for sharp in (1.0, 2.0):
            c = cfg if sharp == 1.0 else without_experts(cfg)
            d, W = make_model(tmp_path_factory.mktemp(f"z_{name}_{int(sharp)}"), c, 100 + i, sharp)
            out[(name, sharp)] = (d, c, W)
    return out


# ------------------------------------------------------------------------------ mechanisms alone
def test_norm_with_offset():
    from fastgguf_b200.parts import run_part
    g = torch.Generator().manual_seed(1)
    x = torch.randn(7, 52, generator=g, dtype=torch.float64) * 3
    w = (torch.randn(52, generator=g) * 0.3).to(torch.bfloat16)
    got = run_part("norm", "rmsnorm", {"size": 52, "eps": 1e-4, "offset": 1.0}, {"weight": w}, "float32", x=x.numpy())
    assert rel_err(got, pz.offset_norm(x, w.double(), 1e-4)) < 1e-6
    plain = run_part("norm", "rmsnorm", {"size": 52, "eps": 1e-4}, {"weight": w}, "float32", x=x.numpy())
    assert rel_err(plain, pz.unit_rms(x, 1e-4) * w.double()) < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,F,M", [(48, 72, 5), (64, 128, 70), (256, 320, 300), (2048, 128, 200)])
def test_dense_feed_forward(dtype, E, F, M):
    """A few rows, a tile of rows, many rows, and a long reduction over few outputs (which the tensor-core contraction
    splits along k): the squared ReLU sits in a different epilogue each time."""
    from fastgguf_b200.parts import run_part
    g = torch.Generator().manual_seed(2)
    W = {"mlp.up": (torch.randn(F, E, generator=g) / E ** 0.5).to(torch.bfloat16),
         "mlp.down": (torch.randn(E, F, generator=g) / F ** 0.5).to(torch.bfloat16)}
    x = torch.randn(M, E, generator=g).to(torch.bfloat16)
    got = run_part("feed_forward", "mlp", {"hidden_size": E, "d_ff": F, "activation": "relu2"},
                   {"up_proj.weight": W["mlp.up"], "down_proj.weight": W["mlp.down"]}, dtype, x=x.float().numpy(),
                   residual=np.zeros((M, E), np.float32))
    want = pz.dense_ff(x.double(), {k: v.double() for k, v in W.items()}, "mlp.")
    assert rel_err(got, want) < (1e-5 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,F,X,top,M,limit", [(48, 40, 5, 2, 9, 0.5), (64, 32, 3, 1, 3, 4.0), (96, 72, 8, 3, 150, 1.0),
                                                (40, 24, 2, 2, 1, 1.0)])
def test_experts(dtype, E, F, X, top, M, limit):
    """Routing, grouping by expert, the expert's clamps and gate, the weight on the expert's input, the sum - for a few
    rows (a warp per output) and for many (tiles of rows grouped by expert)."""
    from fastgguf_b200.parts import run_part
    g = torch.Generator().manual_seed(3)
    W = {"m.router": (torch.randn(X, E, generator=g) * 4 / E ** 0.5).to(torch.bfloat16)}
    names = {"router.weight": W["m.router"]}
    for e in range(X):
        for n, shape in (("gate", (F, E)), ("up", (F, E)), ("down", (E, F))):
            W[f"m.e{e}.{n}"] = (torch.randn(shape, generator=g) * 2 / shape[1] ** 0.5).to(torch.bfloat16)
            names[f"experts.{e}.{n}_proj.weight"] = W[f"m.e{e}.{n}"]
    x = torch.randn(M, E, generator=g).to(torch.bfloat16)
    params = {"hidden_size": E, "d_ff": F, "n_experts": X, "top_k": top, "limit": limit}
    got = run_part("feed_forward", "moe", params, names, dtype, x=x.float().numpy(), residual=np.zeros((M, E), np.float32))
    mlp = {"expert": {"ff": F, "limit": limit}, "router": {"experts": X, "top": top}}
    want = pz.expert_ff(x.double(), {k: v.double() for k, v in W.items()}, "m.", mlp)
    assert rel_err(got, want) < (1e-5 if dtype == "float32" else 3e-2)


def test_head_soft_cap_and_embedding_scale():
    from fastgguf_b200.parts import run_part
    g = torch.Generator().manual_seed(4)
    table = (torch.randn(77, 40, generator=g) * 2).to(torch.bfloat16)
    x = torch.randn(6, 40, generator=g).to(torch.bfloat16)
    got = run_part("head", "lm_head", {"vocab_size": 77, "hidden_size": 40, "softcap": 5.0}, {"weight": table}, "float32",
                   x=x.float().numpy(), out_cols=77)
    want = 5.0 * torch.tanh(x.double() @ table.double().T / 5.0)
    assert rel_err(got, want) < 1e-6 and np.abs(got).max() > 4.0          # the cap did something
    emb = run_part("embedding", "embedding", {"vocab_size": 77, "hidden_size": 40, "scale": 2.5}, {"weight": table}, "float32",
                   tokens=[3, 76, 0], out_cols=40)
    assert rel_err(emb, table.double()[[3, 76, 0]] * 2.5) < 1e-7


def one_layer(layer, width=80, vocab=50):
    return config(width, vocab, [(layer, None)], scale=1.0, eps=1e-5, cap=1e4)


MIXERS = {
    "retention, some dimensions rotated": retention(3, 16, 24, [0.5, 0.9, 0.999], rot=(100.0, 8)),
    "retention, all rotated, wide values": retention(2, 32, 96, [0.97, 1.0], rot=(10000.0, 32)),
    "retention, none rotated, one head": retention(1, 64, 16, [0.99]),
    "retention, value size that does not divide the block": retention(2, 16, 48, [0.9, 0.8], rot=(10.0, 16)),
    "attention, all keys": attention(4, 2, 24, 40, 0.3),
    "attention, window": attention(6, 1, 16, 16, 0.4, size=5),
    "attention, window and kept keys": attention(3, 3, 32, 8, 0.2, size=7, keep_first=3),
    "attention, more kept keys than window": attention(2, 1, 40, 24, 0.2, size=2, keep_first=11),
    "attention, window of one": attention(2, 2, 16, 16, 0.5, size=1, keep_first=1),
    # head sizes of the tensor-core kernels, sequences of several pages: kept keys on one page and on two, in front of
    # the window's pages and overlapping them
    "long attention, head 64, kept keys on two pages": attention(4, 2, 64, 64, 0.125, size=20, keep_first=70),
    "long attention, head 128, kept keys and a wide window": attention(6, 1, 128, 128, 0.09, size=100, keep_first=5),
    "long attention, head 64, window alone": attention(2, 1, 64, 64, 0.125, size=65),
    "long retention, head 128": retention(2, 128, 128, [0.999, 0.99], rot=(10000.0, 64)),
    "long retention, keys 64 and values 128": retention(2, 64, 128, [0.9, 0.9995], rot=(1000.0, 64)),
    "long retention, keys 128 and values 64": retention(3, 128, 64, [1.0, 0.97, 0.5]),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(MIXERS))
def test_mixer_alone(tmp_path, name, dtype):
    """One layer of a mixer alone (norm, mixer, norm, residual add) on rows given by the test: a portion of 37 rows,
    then one of 2, then single rows, so the second and later calls start from what the first left behind (the long
    cases: 160, 30 and 2 rows, then 38 single ones)."""
    cfg = one_layer(MIXERS[name])
    d, W = make_model(tmp_path, cfg, 7, sharp=2.0)
    eng = engine_for(d, dtype)
    g = torch.Generator().manual_seed(8)
    cuts = [160, 30, 2] + [1] * 38 if name.startswith("long") else [37, 2, 1, 1, 1, 1, 1, 1]
    T = sum(cuts)
    x = torch.randn(T, cfg["width"], generator=g, dtype=torch.float64)
    # the plain layer, whole
    layer, mc = cfg["layers"][0], cfg["layers"][0]["mixer"]
    h = pz.offset_norm(x, W["l0.norm1"], 1e-5)
    pos = torch.arange(T)
    if layer["type"] == "retention":
        y = pz.retention_mixer(h, pos, W, "l0.mix.", mc, 1e-5, torch.zeros(mc["heads"], mc["dim"], mc["vdim"], dtype=torch.float64))
    else:
        full = mc
        keys = (h @ W["l0.mix.k"].T).reshape(T, mc["kv_heads"], mc["dim"])
        values = (h @ W["l0.mix.v"].T).reshape(T, mc["kv_heads"], mc["vdim"])
        y = pz.attention_mixer(h, pos, W, "l0.mix.", full, keys, values)
    want = (x + pz.offset_norm(y, W["l0.norm1b"], 1e-5)).numpy()
    slot = eng.acquire()
    got, at = [], 0
    for n in cuts:
        part = np.ascontiguousarray(x[at:at + n].numpy(), dtype=np.float32)
        got.append(eng.block_forward(0, [(slot, n)], part))
        at += n
    got = np.concatenate(got)
    tol = 5e-6 if dtype == "float32" else 4e-2
    for r in range(T):
        assert rel_err(got[r], want[r]) < tol, (name, r)


# ------------------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype,sharp", [("float32", 1.0), ("bfloat16", 2.0)])
@pytest.mark.parametrize("which", list(CASES))
def test_whole_prompt(models, which, dtype, sharp):
    """Logits at every position of a prompt that passes every window, kept key and page edge of the case."""
    d, cfg, W = models[(which, sharp)]
    toks = tokens_for(cfg, 150, 11)
    res = []
    want = pz.plain_forward(cfg, W, toks, res).numpy()
    eng = engine_for(d, dtype)
    s = eng.acquire()
    got = eng.step_host([entry(s, toks)])
    for p in range(len(toks)):
        assert rel_err(got[p], want[p]) < TOL[dtype], (which, p)
    eng.release(s)
    eng.cache.check()


@pytest.mark.parametrize("which", list(CASES))
def test_residual_stream_layer_by_layer(models, which):
    """Every layer's block on the plain implementation's own input for it: a fault shows in the layer that has it."""
    d, cfg, W = models[(which, 1.0)]
    toks = tokens_for(cfg, 70, 12)
    res = []
    pz.plain_forward(cfg, W, toks, res)
    x0 = W["embed"][torch.tensor(toks)] * cfg["embedding"]["scale"]
    eng = engine_for(d, "float32")
    for i, layer in enumerate(cfg["layers"]):
        if "kv_from" in layer["mixer"]:
            continue                          # reads another layer's keys and values: covered by the whole-model tests
        s = eng.acquire()                     # a fresh sequence for every layer: each starts at position 0
        src = (x0 if i == 0 else res[i - 1]).numpy()
        got = eng.block_forward(i, [(s, 70)], np.ascontiguousarray(src, dtype=np.float32))
        eng.release(s)
        assert rel_err(got, res[i].numpy()) < 1e-5, (which, i)


@pytest.mark.parametrize("dtype,sharp", [("float32", 1.0), ("bfloat16", 2.0)])
@pytest.mark.parametrize("which,cuts", [("a", [2, 2, 3, 17, 33, 64, 65, 2, 31]), ("b", [63, 2, 64, 1, 1, 70, 2, 16]),
                                        ("c", [100, 28, 1, 2, 64, 24])])
def test_portions_and_decoding(models, which, cuts, dtype, sharp):
    """A prompt cut into portions of many sizes, down to two tokens and one, then 40 tokens one by one: the same logits
    as the whole sequence at every position."""
    d, cfg, W = models[(which, sharp)]
    n = sum(cuts) + 40
    toks = tokens_for(cfg, n, 13)
    want = pz.plain_forward(cfg, W, toks).numpy()
    eng = engine_for(d, dtype)
    s = eng.acquire()
    at = 0
    for c in cuts + [1] * 40:
        got = eng.step_host([entry(s, toks[at:at + c])])
        for i in range(c):
            assert rel_err(got[i], want[at + i]) < TOL[dtype], (which, at + i, c)
        at += c
    eng.release(s)
    eng.cache.check()


@pytest.mark.parametrize("dtype,sharp", [("float32", 1.0), ("bfloat16", 2.0)])
@pytest.mark.parametrize("which", list(CASES))
def test_batch_of_unequal_requests(models, which, dtype, sharp):
    """Five requests of 1 to 140 tokens in one step, then decoded together while the shorter ones leave: every
    request's logits equal those it has alone."""
    d, cfg, W = models[(which, sharp)]
    lens, total = [1, 140, 64, 7, 65], [9, 150, 70, 30, 66]
    toks = [tokens_for(cfg, t, 20 + i) for i, t in enumerate(total)]
    want = [pz.plain_forward(cfg, W, t).numpy() for t in toks]
    eng = engine_for(d, dtype)
    slots = [eng.acquire() for _ in toks]
    got = eng.step_host([entry(s, t[:n]) for s, t, n in zip(slots, toks, lens)])
    row = 0
    for b, n in enumerate(lens):
        for p in range(n):
            assert rel_err(got[row], want[b][p]) < TOL[dtype], (which, b, p)
            row += 1
    at = list(lens)
    alive = list(range(len(toks)))
    while alive:
        got = eng.step_host([entry(slots[b], [toks[b][at[b]]]) for b in alive])
        for i, b in enumerate(alive):
            assert rel_err(got[i], want[b][at[b]]) < TOL[dtype], (which, b, at[b])
            at[b] += 1
        for b in [b for b in alive if at[b] == total[b]]:
            eng.release(slots[b])
            alive.remove(b)
    eng.cache.check()
    assert eng.cache.live_slots() == []


def test_slots_and_pages_used_again(models):
    """Sequences come and go in a cache of two slots and few pages: a new sequence starts from nothing (state rows are
    cleared, pages of the one before are not read), also after a sequence that was released halfway."""
    d, cfg, W = models[("b", 1.0)]
    eng = engine_for(d, "float32", max_tokens=512, max_batch=2)
    seqs = [tokens_for(cfg, n, 40 + i) for i, n in enumerate([200, 130, 90, 260, 70, 140])]
    for k, toks in enumerate(seqs):
        s = eng.acquire()
        other = eng.acquire()
        eng.step_host([entry(other, seqs[(k + 1) % len(seqs)][:50], [])])       # a neighbour that is dropped halfway
        want = pz.plain_forward(cfg, W, toks).numpy()
        head = len(toks) - 20
        got = eng.step_host([entry(s, toks[:head], [head - 1])])
        assert rel_err(got[0], want[head - 1]) < TOL["float32"], k
        eng.release(other)
        for p in range(head, len(toks)):
            got = eng.step_host([entry(s, [toks[p]])])
            assert rel_err(got[0], want[p]) < TOL["float32"], (k, p)
        eng.release(s)
        eng.cache.check()


def test_long_decoding_past_windows_and_pages(models):
    """300 tokens one by one after a short prompt: windows slide over decoded tokens, pages leave the windowed groups while
    the kept first keys stay, and the retention state carries the first tokens all along."""
    d, cfg, W = models[("b", 1.0)]
    toks = tokens_for(cfg, 330, 50)
    want = pz.plain_forward(cfg, W, toks).numpy()
    eng = engine_for(d, "float32")
    s = eng.acquire()
    eng.step_host([entry(s, toks[:30], [])])
    for p in range(30, 330):
        got = eng.step_host([entry(s, [toks[p]])])
        assert rel_err(got[0], want[p]) < TOL["float32"], p
    groups = eng.cache.groups
    assert any(g["window"] and g["keep_first"] for g in groups)
    eng.release(s)
    eng.cache.check()


def test_a_far_token_is_remembered(tmp_path):
    """One early token differs between two prompts of 400 tokens: with a slow decay the last logits differ by far more
    than rounding, in the engine exactly as in the plain implementation; with windows alone they would not."""
    cfg = config(64, 90, [(retention(2, 16, 16, [0.9995, 0.999], rot=(10000.0, 16)), dense(48)),
                          (attention(2, 1, 16, 16, 0.25, size=8, keep_first=1), None)], scale=4.0)
    d, W = make_model(tmp_path, cfg, 60)
    a = tokens_for(cfg, 400, 61)
    b = list(a)
    b[3] = (a[3] + 1) % cfg["vocab"]
    eng = engine_for(d, "float32")
    last = []
    for toks in (a, b):
        s = eng.acquire()
        got = eng.step_host([entry(s, toks[:380], [])])
        for p in range(380, 400):
            got = eng.step_host([entry(s, [toks[p]])])
        last.append(got[0])
        eng.release(s)
        assert rel_err(got[0], pz.plain_forward(cfg, W, toks).numpy()[-1]) < TOL["float32"]
    assert np.abs(last[0] - last[1]).max() > 1e-3 * np.abs(last[0]).max()


# ------------------------------------------------------------------------------ generation through the entry point
@pytest.mark.parametrize("use_graphs", [False, True])
@pytest.mark.parametrize("which", ["a", "b"])
def test_greedy_generation(models, which, use_graphs):
    """Greedy decoding through Engine.generate - the scheduler's batches, the recorded decode step, slots that come
    back - follows the plain implementation: each token is the plain logits' best given the tokens before it (where the
    best two are closer than rounding, either counts)."""
    d, cfg, W = models[(which, 1.0)]
    prompts = [tokens_for(cfg, n, 70 + i) for i, n in enumerate([5, 70, 1, 33, 12])]
    eng = engine_for(d, "float32", max_tokens=2048, max_batch=4, use_graphs=use_graphs)
    out = eng.generate(prompts, temp=0, max_tokens=24, ignore_eos=True, batch_size=3)
    for p, c in zip(prompts, out):
        assert len(c.tokens) == 24
        logits = pz.plain_forward(cfg, W, p + c.tokens).numpy()
        for i, t in enumerate(c.tokens):
            row = logits[len(p) + i - 1]
            assert row[t] >= row.max() - 1e-4 * np.abs(row).max(), (which, i)
    eng.cache.check()
    assert eng.cache.live_slots() == []


def test_experts_inside_a_bfloat16_model(models):
    """The cases as they are, expert layers included, in bfloat16: nearly all positions agree with the plain
    implementation (a close call of a router may turn the rest of a sequence)."""
    for which in CASES:
        d, cfg, W = models[(which, 1.0)]
        eng = engine_for(d, "bfloat16")
        good = total = 0
        for k in range(6):
            toks = tokens_for(cfg, 40, 90 + k)
            want = pz.plain_forward(cfg, W, toks).numpy()
            s = eng.acquire()
            got = np.concatenate([eng.step_host([entry(s, toks[:25])])] + [eng.step_host([entry(s, [t])]) for t in toks[25:]])
            eng.release(s)
            good += sum(rel_err(got[p], want[p]) < TOL["bfloat16"] for p in range(40))
            total += 40
        assert good >= 0.8 * total, (which, good, total)


def test_generation_in_bfloat16_runs_the_recorded_step(models):
    d, cfg, W = models[("c", 1.0)]
    prompts = [tokens_for(cfg, n, 80 + i) for i, n in enumerate([9, 40])]
    eng = engine_for(d, "bfloat16", max_tokens=1024, max_batch=2)
    out = eng.generate(prompts, temp=0, max_tokens=70, ignore_eos=True)
    for p, c in zip(prompts, out):
        logits = pz.plain_forward(cfg, W, p + c.tokens).numpy()
        close = sum(logits[len(p) + i - 1][t] >= logits[len(p) + i - 1].max() - 0.05 * np.abs(logits[len(p) + i - 1]).max()
                    for i, t in enumerate(c.tokens))
        assert close >= 0.9 * len(c.tokens)
    eng.cache.check()


def test_command_line_generates(models):
    """``python -m fastgguf_b200 generate`` on a Zirivik folder: the model class comes from config.json, the tokens are
    those of Engine.generate."""
    import json
    import os
    import subprocess
    import sys
    d, cfg, W = models[("a", 1.0)]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, "-m", "fastgguf_b200", "generate", d, "256", "--prompt", "5,17,3,200", "--prompt", "9",
                        "--temp", "0", "--max-tokens", "6", "--ignore-eos", "--dtype", "float32", "--json"],
                       cwd=root, capture_output=True, text=True)
    assert p.returncode == 0, p.stderr
    got = [r["tokens"] for r in json.loads(p.stdout)]
    eng = engine_for(d, "float32", max_tokens=512, max_batch=2)
    want = [c.tokens for c in eng.generate([[5, 17, 3, 200], [9]], temp=0, max_tokens=6, ignore_eos=True)]
    assert got == want
