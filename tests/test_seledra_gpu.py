"""Seledra through the engine against the plain NumPy statement of the design (plain_seledra.py):
each mechanism alone, whole prompts, token-by-token decoding, prompts in portions, unequal batches,
slots, pages and state used again, keys far away and at page borders, the first tokens, long decoding,
odd sizes, and greedy generation through the library's own entry point."""
import functools
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_seledra as plain
import helpers
from helpers import run_batch, run_tail_one_by_one, run_whole
from math_utils_b200 import DecoderModel, LLM, StepEntry
from math_utils_b200.weights.safetensors import write_safetensors

pytestmark = pytest.mark.gpu

# The recurrent layers carry rounding of their inputs from token to token and the whole-projection norms bring
# every query and key to full size, so the rows' noise in bfloat16 is a little above a plain transformer's.
BF16_RMS = {"a": 0.02, "b": 0.04, "c": 0.02}


def check_logits(got, want, dtype, what=""):
    helpers.check_logits(got, want, dtype, what, bf16_rms=BF16_RMS[what.split()[1]])


def attention(heads, kv_heads, dim, vdim, scale, v_mix, ff=None):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                                           "v_mix": v_mix}, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def delta(heads, kv_heads, dim, vdim, conv, ff=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(vocab, width, mult, eps, layers, max_positions=600):
    return {"architecture": "Seledra", "vocab": vocab, "width": width, "max_positions": max_positions,
            "residual_mult": mult, "norm": {"eps": eps}, "layers": layers}


# an attention layer that shares nothing before the sharing ones; a delta layer with and without feed-forward; the
# sharing layers differ in heads and key size
CFG_A = config(300, 64, 0.5, 1e-6, [
    attention(2, 1, 8, 16, 0.3, False, 96), attention(4, 2, 16, 24, 0.25, True, 96), delta(4, 2, 16, 8, 4),
    attention(2, 2, 32, 24, 0.2, True), delta(2, 2, 24, 12, 3, 80), attention(4, 2, 16, 24, 0.25, True, 64)])
# nothing a multiple of 8; as many kv heads as heads and one kv head; one tap (no convolution state) and two; a
# multiplier of one; a large eps; a delta layer first
CFG_B = config(131, 50, 1.0, 1e-3, [
    delta(3, 3, 7, 5, 2, 33), attention(3, 3, 6, 5, 0.4, True, 21), delta(2, 1, 33, 9, 1),
    attention(6, 1, 5, 15, 0.5, False), attention(3, 3, 10, 5, 0.3, True, 21)])
# sizes the tensor-core kernels take; keys of 128 in a delta layer
CFG_C = config(384, 128, 0.35, 2e-5, [
    attention(8, 2, 32, 64, 0.18, True, 256), delta(4, 2, 64, 32, 4), delta(2, 2, 128, 64, 3, 128),
    attention(4, 2, 64, 64, 0.125, True, 256), attention(2, 1, 128, 32, 0.09, False)])
CONFIGS = {"a": CFG_A, "b": CFG_B, "c": CFG_C}


@functools.lru_cache(maxsize=None)
def weights_of(name):
    return plain.random_weights(CONFIGS[name], seed=sum(map(ord, name)) + 41)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, cfg in CONFIGS.items():
        d = str(tmp_path_factory.mktemp(f"seledra_{name}"))
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg, f)
        write_safetensors(os.path.join(d, "model.safetensors"),
                          {k: torch.from_numpy(np.array(v)).to(torch.bfloat16) for k, v in weights_of(name).items()})
        out[name] = d
    return out


_models = {}


def engine(folders, name, dtype):
    key = (name, dtype)
    if key not in _models:
        model = DecoderModel.from_dir(folders[name], dtype=dtype)
        _models[key] = (model, model.new_cache(max_tokens=64 * 24, n_slots=8))
    return _models[key]


def tokens_for(name, n, seed=0):
    return np.random.default_rng(3000 + seed).integers(0, CONFIGS[name]["vocab"], size=n).tolist()


_plain_cache = {}


def plain_logits(name, tokens):
    key = (name, tuple(tokens))
    if key not in _plain_cache:
        _plain_cache[key] = plain.forward(CONFIGS[name], weights_of(name), list(tokens))
    return _plain_cache[key]


CASES = [(n, d) for n in CONFIGS for d in ("float32", "bfloat16")]


# ------------------------------------------------------------------ whole models
@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_prompt_and_every_layer(folders, name, dtype):
    model, cache = engine(folders, name, dtype)
    toks = tokens_for(name, 150)
    layers = []
    want = plain.forward(CONFIGS[name], weights_of(name), toks, layers)
    slot = cache.acquire()
    trace = {}
    got = model.step(cache, [StepEntry(slot, toks, list(range(len(toks))))], trace=trace).cpu().numpy()
    cache.release(slot)
    if dtype == "float32":
        for i, x in enumerate(layers):
            assert np.abs(trace[f"h.{i}.res2"] - x).max() < 1e-4, f"residual stream after layer {i}"
    check_logits(got, want, dtype, f"seledra {name} whole prompt")
    # the same prompt without a trace: the sublayers' additions are then made by the next norm's launch
    check_logits(run_whole(model, cache, toks), want, dtype, f"seledra {name} whole prompt, joins deferred")


@pytest.mark.parametrize("name,dtype", CASES)
def test_prompt_then_token_by_token(folders, name, dtype):
    model, cache = engine(folders, name, dtype)
    toks = tokens_for(name, 150, seed=1)                 # the tail crosses the page border at 128
    got = run_tail_one_by_one(model, cache, toks, tail=120)
    check_logits(got, plain_logits(name, toks), dtype, f"seledra {name} tail one by one")


@pytest.mark.parametrize("name,dtype", CASES)
@pytest.mark.parametrize("portions", [(2, 3, 59, 1, 64, 21), (64, 64, 22), (127, 2, 2, 19), (1, 1, 1, 147), (2,) * 12 + (126,)])
def test_prompt_in_portions(folders, name, dtype, portions):
    model, cache = engine(folders, name, dtype)
    toks = tokens_for(name, sum(portions), seed=2)
    slot = cache.acquire()
    rows, at = [], 0
    for n in portions:
        rows.append(model.step(cache, [StepEntry(slot, toks[at:at + n], list(range(n)))]).cpu().numpy())
        at += n
    cache.release(slot)
    check_logits(np.concatenate(rows), plain_logits(name, toks), dtype, f"seledra {name} portions {portions}")


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_batch_against_each_alone(folders, name, dtype):
    model, cache = engine(folders, name, dtype)
    lens, prompts = (140, 5, 66, 131), (129, 1, 33, 64)
    requests = [tokens_for(name, n, seed=10 + i) for i, n in enumerate(lens)]
    got = run_batch(model, cache, requests, prompts)
    for i, r in enumerate(requests):
        check_logits(got[i], plain_logits(name, r), dtype, f"seledra {name} batch request {i}")
        if dtype == "float32":
            alone = run_tail_one_by_one(model, cache, r, tail=lens[i] - prompts[i])
            assert np.abs(alone - got[i]).max() < 2e-5, "a request's logits depend on its batch"


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("b", "bfloat16"), ("c", "float32")])
def test_slots_pages_and_state_used_again(folders, name, dtype):
    model, cache = engine(folders, name, dtype)
    free = [cache.free_pages(g.index) for g in cache.kv_groups]
    first = tokens_for(name, 200, seed=20)
    second = tokens_for(name, 90, seed=21)
    a = run_whole(model, cache, first)
    slot = cache.acquire()                               # the slot, the pages and the state the first request held
    model.step(cache, [StepEntry(slot, second[:70], [])])
    b = [model.step(cache, [StepEntry(slot, [t], [0])]).cpu().numpy() for t in second[70:]]
    cache.release(slot)
    assert [cache.free_pages(g.index) for g in cache.kv_groups] == free
    check_logits(a, plain_logits(name, first), dtype, f"seledra {name} first holder")
    check_logits(np.concatenate(b), plain_logits(name, second)[70:], dtype, f"seledra {name} second holder of the same slot")


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("b", "float32"), ("c", "bfloat16")])
@pytest.mark.parametrize("n", [1, 2, 3, 4, 5, 63, 64, 65, 127, 128, 129, 193])
def test_first_tokens_and_lengths_around_page_borders(folders, name, dtype, n):
    model, cache = engine(folders, name, dtype)
    toks = tokens_for(name, 193, seed=30)[:n]
    slot = cache.acquire()
    got = model.step(cache, [StepEntry(slot, toks, [0, n - 1])]).cpu().numpy()
    cache.release(slot)
    want = plain_logits(name, tokens_for(name, 193, seed=30))          # causal: a prefix's logits are the long prompt's
    check_logits(got, want[[0, n - 1]], dtype, f"seledra {name} prompt of {n}")


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("b", "float32"), ("c", "bfloat16")])
def test_long_decoding(folders, name, dtype):
    model, cache = engine(folders, name, dtype)
    toks = tokens_for(name, 270, seed=40)
    free = [cache.free_pages(g.index) for g in cache.kv_groups]
    got = run_tail_one_by_one(model, cache, toks, tail=267)            # three tokens, then one by one over four pages
    check_logits(got, plain_logits(name, toks), dtype, f"seledra {name} long decoding")
    assert [cache.free_pages(g.index) for g in cache.kv_groups] == free


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_greedy_generation_through_the_library(folders, name):
    llm = LLM(folders[name], dtype="float32", temperature=0.0, max_tokens=24, context=512)
    assert llm.model.graph_safe                                            # single-token steps replay from a graph
    prompts = [tokens_for(name, n, seed=50 + n) for n in (70, 3, 129)]
    outs = llm.generate(prompts)
    for p, out in zip(prompts, outs):
        assert len(out) == 24
        seq = list(p)
        for tok in out:
            row = plain.forward(CONFIGS[name], weights_of(name), seq)[-1]
            best = int(np.argmax(row))
            assert tok == best or row[best] - row[tok] < 1e-4, f"greedy token {len(seq) - len(p)} of a prompt of {len(p)}"
            seq.append(tok)
    alone = llm.generate([prompts[2]])[0]
    assert alone == outs[2], "a request generates other tokens alone than in a batch"
    from math_utils_b200 import SamplingParams
    from math_utils_b200.engine.generate import generate
    eager = generate(llm.model, [prompts[0]], 24, SamplingParams(0.0, 1, 0), context=512, use_graph=False)[0]
    assert eager == outs[0], "eager steps and replayed steps generate different tokens"


def test_requests_that_end_early_leave_the_others_alone(folders):
    llm = LLM(folders["a"], dtype="float32", temperature=0.0, max_tokens=30, context=512)
    prompts = [tokens_for("a", n, seed=70 + n) for n in (40, 9, 66, 3, 21)]
    free = llm.generate(prompts, stop_ids=[])
    stop = free[0][5]
    want = [out[:out.index(stop)] if stop in out else out for out in free]
    got = llm.generate(prompts, stop_ids=[stop])
    assert got == want
    assert llm.generate(prompts[1:], stop_ids=[stop]) == want[1:]


def test_conversation_on_a_kept_slot(folders):
    """Two turns through ``LLM.prompt``: the slot keeps keys, values, and the recurrence's state."""
    llm = LLM(folders["a"], dtype="float32", temperature=0.0, max_tokens=9, context=512)
    first, second = tokens_for("a", 45, seed=60), tokens_for("a", 30, seed=61)
    out1 = llm.prompt(first)
    out2 = llm.prompt(second)
    seq = list(first) + out1 + list(second)
    assert len(out1) == 9 and len(out2) == 9
    for tok in out2:
        row = plain.forward(CONFIGS["a"], weights_of("a"), seq)[-1]
        best = int(np.argmax(row))
        assert tok == best or row[best] - row[tok] < 1e-4
        seq.append(tok)


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("b", "bfloat16")])
def test_replay_of_steps_through_the_program(folders, name, dtype, tmp_path):
    """``bin/trace_run``: a batch of unequal prompts decoded together, requests that end early, then a second batch
    that takes over the freed slots, pages and states; every position's logits against the plain model."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    lens = {"p": 97, "q": 12, "r": 70, "s": 3, "t": 131}
    reqs = {rid: tokens_for(name, n, seed=70 + i) for i, (rid, n) in enumerate(lens.items())}
    steps, rows = [], {rid: [] for rid in reqs}                   # rows[rid]: (step, index in the step's file) per position
    for ids, cuts in ((("p", "q", "r"), (64, 10, 1)), (("s", "t"), (2, 129))):
        pos = dict(zip(ids, cuts))
        entries = [{"id": i, "tokens": reqs[i][:pos[i]], "want": list(range(pos[i]))} for i in ids]
        live = list(ids)
        while live:
            step, at = len(steps), 0
            for e in entries:
                rows[e["id"]] += [(step, at + k) for k in e["want"]]
                at += len(e["want"])
            ends = [i for i in live if pos[i] >= lens[i]]
            steps.append({"step": step, "entries": entries, "end": ends})
            live = [i for i in live if i not in ends]
            entries = [{"id": i, "tokens": [reqs[i][pos[i]]], "want": [0]} for i in live]
            for i in live:
                pos[i] += 1
    out_dir = str(tmp_path / "out")
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders[name], "--dtype", dtype,
                           "--out", out_dir, "--max-tokens", "320"],
                          input="".join(json.dumps(st) + "\n" for st in steps), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {st['step']}" for st in steps]
    vocab = CONFIGS[name]["vocab"]
    files = {}
    for rid, r in reqs.items():
        got = []
        for step, k in rows[rid]:
            if step not in files:
                files[step] = np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4").reshape(-1, vocab)
            got.append(files[step][k])
        assert len(got) == lens[rid]
        check_logits(np.stack(got), plain_logits(name, r), dtype, f"seledra {name} replayed request {rid}")


# ------------------------------------------------------------------ mechanisms alone
def _ops():
    from math_utils_b200.csrc import ops
    return ops


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device="cuda", dtype=dtype)


def ints(a):
    return dev(np.asarray(a), torch.int32)


def test_join_and_norm_kernel():
    ops, rng = _ops(), np.random.default_rng(1)
    for n in (44, 45, 2600):
        x, y, w = rng.normal(0, 2, (5, n)), rng.normal(0, 1, (5, n)), rng.normal(1, 0.2, n)
        for eps in (1e-6, 0.5):                             # an eps that matters: inside the root
            xs, out = dev(x), torch.zeros((5, n), device="cuda")
            ops.residual_add_norm(xs, dev(y), 0.3, dev(w), eps, out)
            assert np.abs(xs.cpu().numpy() - (x + 0.3 * y)).max() < 1e-6
            assert np.abs(out.cpu().numpy() - plain.rms_norm(x + 0.3 * y, w, eps)).max() < 5e-6
            xs = dev(x)
            ops.residual_add_norm(xs, None, 0.0, dev(w), eps, out)      # nothing to add: the norm alone
            assert np.array_equal(xs.cpu().numpy(), x.astype(np.float32))
            assert np.abs(out.cpu().numpy() - plain.rms_norm(x, w, eps)).max() < 5e-6
            ops.residual_add_norm(xs, dev(y), -1.5, None, 0.0, None)    # the addition alone
            assert np.abs(xs.cpu().numpy() - (x - 1.5 * y)).max() < 1e-6
    out = torch.zeros((5, 2600), device="cuda", dtype=torch.bfloat16)
    ops.residual_add_norm(dev(x), dev(y), 0.3, dev(w), 1e-6, out)
    assert np.abs(out.float().cpu().numpy() - plain.rms_norm(x + 0.3 * y, w, 1e-6)).max() < 3e-2


def test_activation_kernel():
    ops, rng = _ops(), np.random.default_rng(2)
    for shape in ((7, 19), (5, 64)):
        a = rng.normal(0, 3, shape)
        a[0, :3] = (0.0, -1e-3, 1e-3)
        for pair in ((0.3, -0.4), (-2.0, 1.5), (0.0, 0.0)):
            for dtype, tol in ((torch.float32, 3e-6), (torch.bfloat16, 3e-2)):
                ad = dev(a, dtype)
                af = ad.float().cpu().numpy().astype(np.float64)
                out = ops.xielu(ad, dev(np.array(pair))).float().cpu().numpy()
                want = plain.xielu(af, np.array(pair))
                assert np.abs(out - want).max() < tol * max(1.0, np.abs(want).max())


def test_activation_of_bfloat16_rows_is_as_good_as_their_rounding():
    """The form for bfloat16 rows (a series near zero, the fast exponential beyond) against the exact one, entry by
    entry and relative to the entry: tiny and large arguments, and both sides of where the form changes."""
    ops = _ops()
    neg = -np.logspace(-6, 2, 440)
    z = np.concatenate([neg, np.logspace(-6, 2, 120), [-0.25, -0.2500001, -0.2499999, -0.26, -0.24, 0.0, -87.0, -120.0]])
    z = np.concatenate([z, np.zeros(-len(z) % 64)]).reshape(-1, 64)
    for pair in ((0.3, -0.4), (-2.0, 1.5), (3.0, 4.0)):
        zd = dev(z, torch.bfloat16)
        zf = zd.float().cpu().numpy().astype(np.float64)
        out = ops.xielu(zd, dev(np.array(pair))).float().cpu().numpy().astype(np.float64)
        want = plain.xielu(zf, np.array(pair))
        assert np.all(np.abs(out - want) <= 2.0 ** -7 * np.abs(want) + 1e-9)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
# the last two: queries wider than the entries a block keeps in registers, values longer than a warp keeps
@pytest.mark.parametrize("H,G,dim,vdim,mode", [(4, 2, 16, 24, 1), (3, 3, 6, 5, 2), (6, 1, 5, 15, 0), (8, 2, 32, 64, 2),
                                               (10, 10, 128, 8, 1), (2, 1, 8, 300, 2)])
def test_projection_norms_and_shared_values_kernel(dtype, H, G, dim, vdim, mode):
    """Queries and keys normed over the whole projection, values per head, the blend with another layer's values,
    rows written to scattered pages."""
    ops, rng = _ops(), np.random.default_rng(4)
    eps, lam = 1e-2, 0.37
    positions = np.array([0, 63, 64, 130, 5, 40000])
    seq_of = np.array([0, 0, 1, 1, 2, 2])
    table = np.zeros((3, 700), dtype=np.int32)
    table[0, :2], table[1, :3], table[2, 0], table[2, 625] = (4, 1), (2, 6, 5), 3, 0
    T, qw, kw, vw = len(positions), H * dim, G * dim, G * vdim
    pad = -(qw + kw + vw) % 8
    proj = dev(rng.normal(0, 2, (T, qw + kw + vw + pad)), dtype)
    x = proj.float().cpu().numpy().astype(np.float64)
    wq, wk = rng.normal(1, 0.3, qw), rng.normal(1, 0.3, kw)
    first = rng.normal(0, 1, (T, vw))
    want_q = plain.rms_norm(x[:, :qw], wq, eps)
    want_k = plain.rms_norm(x[:, qw:qw + kw], wk, eps)
    want_v = plain.unit_rms(x[:, qw + kw:qw + kw + vw].reshape(T, G, vdim), eps).reshape(T, vw)
    if mode == 2:
        want_v = (1 - lam) * want_v + lam * first
    rows = torch.zeros((7, 64, kw + vw), device="cuda", dtype=dtype)
    shared = dev(first)
    q = proj[:, :qw]
    ops.qkv_norm_rows(q, proj[:, qw:qw + kw], proj[:, qw + kw:qw + kw + vw], dev(wq), dev(wk), eps, G, vdim, True,
                      ints(positions), ints(seq_of), ints(table), 64, rows, shared if mode else None, mode, lam)
    tol = 1e-5 if dtype == torch.float32 else 4e-2
    assert np.abs(q.float().cpu().numpy() - want_q).max() < tol
    got = rows.float().cpu().numpy()
    for t, (p, s) in enumerate(zip(positions, seq_of)):
        row = got[table[s, p // 64], p % 64]
        assert np.abs(row[:kw] - want_k[t]).max() < tol
        assert np.abs(row[kw:] - want_v[t]).max() < tol
    assert np.count_nonzero(got.reshape(-1, kw + vw).any(axis=1)) == T       # no other row was touched
    if mode == 1:                                                            # the source hands on what it caches, in float32
        assert np.abs(shared.cpu().numpy() - want_v).max() < 1e-5
    else:
        assert np.array_equal(shared.cpu().numpy(), first.astype(np.float32))


def _paged(rng, lens, width, page=64):
    """Rows of several sequences in pages handed out in a scrambled order."""
    n_pages = sum(-(-n // page) for n in lens) + 3
    order = rng.permutation(n_pages)
    pages = np.zeros((n_pages, page, width))
    table = np.zeros((len(lens), 24), dtype=np.int32)
    seqs, at = [], 0
    for s, n in enumerate(lens):
        rows = rng.normal(0, 1, (n, width))
        seqs.append(rows)
        for i in range(-(-n // page)):
            table[s, i] = order[at]
            chunk = rows[i * page:(i + 1) * page]
            pages[order[at], :len(chunk)] = chunk
            at += 1
    return seqs, pages, table


def _same_entry_in_every_key(seqs, pages, table, s, value):
    """Entry 0 of kv head 0's keys of sequence ``s`` becomes ``value`` at every position: a query along that entry
    scores the same against all of them."""
    seqs[s][:, 0] = value
    for i in range(-(-len(seqs[s]) // 64)):
        pages[table[s, i], :, 0] = value


def _plain_heads(q, rows, pos, dim, vdim, H, G, scale, temps, gate):
    """One token's heads [H, vdim] from its sequence's rows, through the plain function."""
    n = pos + 1
    k = rows[:n, :G * dim].reshape(n, G, dim)
    v = rows[:n, G * dim:].reshape(n, G, vdim)
    out = np.zeros((H, vdim))
    for a in range(H):
        g = a // (H // G)
        qq = np.zeros((n, dim))
        qq[-1] = q[a]
        out[a] = plain.sink_softmax_attention(qq, k[:, g], v[:, g], scale * temps[a])[-1] * plain.sigmoid(gate[a])
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dim,vdim", [(4, 2, 16, 24), (3, 3, 6, 5), (6, 1, 5, 15), (4, 2, 64, 32), (2, 2, 8, 200)])
def test_attention_with_sink_temperature_and_gate(dtype, H, G, dim, vdim):
    ops, rng = _ops(), np.random.default_rng(5)
    lens = [1, 2, 63, 64, 65, 300, 1400]
    width = G * (dim + vdim)
    seqs, pages, table = _paged(rng, lens, width)
    far = 9
    seqs[6][far, :dim] *= 4.0                                         # a long key: no other key comes near its score
    pages[table[6, far // 64], far % 64, :dim] *= 4.0
    _same_entry_in_every_key(seqs, pages, table, 5, 3.0)
    scale = 0.37
    temps = rng.uniform(0.5, 2.0, H)
    temps[-1] = -0.8                                                  # a temperature may be any number
    if dtype == torch.bfloat16:                                       # the cache holds what bfloat16 can hold
        pages = dev(pages, dtype).float().cpu().numpy().astype(np.float64)
        seqs = [np.concatenate([pages[table[s, i]] for i in range(-(-n // 64))])[:n] for s, n in enumerate(lens)]
    picks = [(s, n - 1) for s, n in enumerate(lens)] + [(5, p) for p in (0, 63, 64, 127, 128, 191, 192, 250)] + [(6, 1100)]
    q = rng.normal(0, 1, (len(picks), H, dim)) / math.sqrt(dim) * 3
    gate = rng.normal(0, 2, (len(picks), H))
    key_of = lambda s, j, g: seqs[s][j, g * dim:(g + 1) * dim]
    # The last query of the longest sequence: head 0 points at a key 1,390 positions back among 1,400, whose value must
    # come through whole.  The last query of the 300: head 0 scores -40 against every key it sees, so the sink takes the
    # softmax and the head's result is nothing; without the sink it would be the mean of the values.
    q[6, 0] = key_of(6, far, 0) * 30.0 / (scale * temps[0]) / (key_of(6, far, 0) ** 2).sum()
    q[5, 0] = 0.0
    q[5, 0, 0] = -40.0 / (3.0 * scale * temps[0])
    if dtype == torch.bfloat16:
        q = dev(q, dtype).float().cpu().numpy().astype(np.float64)
        gate = dev(gate, dtype).float().cpu().numpy().astype(np.float64)
    want = np.stack([_plain_heads(q[i], seqs[s], p, dim, vdim, H, G, scale, temps, gate[i]) for i, (s, p) in enumerate(picks)])
    v_far = seqs[6][far, G * dim:G * dim + vdim] * plain.sigmoid(gate[6, 0])
    assert np.abs(want[6, 0] - v_far).max() < 0.05 * np.abs(v_far).max()                  # the test's own premises
    assert np.abs(want[5, 0]).max() < 1e-6 and np.abs(want[5, 1]).max() > 1e-3
    tol = 3e-5 if dtype == torch.float32 else 4e-2
    for single in (False, True):                                      # the general kernel, and the one of single-token steps
        out = torch.zeros((len(picks), H * vdim), device="cuda", dtype=dtype)
        ops.mapped_attention(dev(q.reshape(len(picks), -1), dtype), dev(pages, dtype), ints(table), 64,
                             ints([p for _, p in picks]), ints([s for s, _ in picks]), H, G, 1, dim, vdim, scale, 0, out,
                             single_tokens=single, head_scale=dev(temps), sink=True, gate=dev(gate, dtype))
        got = out.float().cpu().numpy().reshape(len(picks), H, vdim)
        err = np.abs(got - want).max(axis=(1, 2))
        assert err.max() < tol, f"single {single}: first wrong query {picks[int(np.argmax(err > tol))]}"


@pytest.mark.parametrize("H,G,dim,vdim", [(4, 2, 16, 16), (8, 2, 128, 64), (3, 3, 32, 48), (2, 1, 80, 112)])
def test_attention_with_sink_on_tensor_cores_prompt_tiles(H, G, dim, vdim):
    """Several sequences' tokens in one step as tiles of up to 64; some sequences bring only their last tokens."""
    ops, rng = _ops(), np.random.default_rng(8)
    lens, new = [130, 1, 64, 65, 7, 200], [130, 1, 64, 3, 7, 70]
    width = G * (dim + vdim)
    seqs, pages, table = _paged(rng, lens, width)
    seqs[5][0, :dim] *= 4.0                                           # a long key: no other key comes near its score
    pages[table[5, 0], 0, :dim] *= 4.0
    _same_entry_in_every_key(seqs, pages, table, 0, 3.0)
    scale = 0.21
    temps = rng.uniform(0.5, 2.0, H)
    pages = dev(pages, torch.bfloat16).float().cpu().numpy().astype(np.float64)
    seqs = [np.concatenate([pages[table[s, i]] for i in range(-(-n // 64))])[:n] for s, n in enumerate(lens)]
    tok_seq = np.repeat(np.arange(len(lens)), new)
    tok_pos = np.concatenate([np.arange(n - k, n) for n, k in zip(lens, new)])
    T = len(tok_seq)
    q = rng.normal(0, 1, (T, H, dim)) / math.sqrt(dim) * 4
    gate = rng.normal(0, 2, (T, H))
    # the last token of the longest sequence: head 0 points at the sequence's first key; the last token of the first
    # sequence scores -40 against every key, so the sink takes its softmax
    key0 = seqs[5][0, :dim]
    q[T - 1, 0] = key0 * 30.0 / (scale * temps[0]) / (key0 ** 2).sum()
    q[129, 0] = 0.0
    q[129, 0, 0] = -40.0 / (3.0 * scale * temps[0])
    q = dev(q, torch.bfloat16).float().cpu().numpy().astype(np.float64)
    gate = dev(gate, torch.bfloat16).float().cpu().numpy().astype(np.float64)
    tiles, at = [], 0
    for k in new:
        tiles += [(at + o, min(64, k - o)) for o in range(0, k, 64)]
        at += k
    tiles.sort(key=lambda t: -tok_pos[t[0] + t[1] - 1])
    want = np.stack([_plain_heads(q[t], seqs[tok_seq[t]], tok_pos[t], dim, vdim, H, G, scale, temps, gate[t]) for t in range(T)])
    v_first = seqs[5][0, G * dim:G * dim + vdim] * plain.sigmoid(gate[T - 1, 0])
    assert np.abs(want[T - 1, 0] - v_first).max() < 0.05 * np.abs(v_first).max()          # the test's own premises
    assert np.abs(want[129, 0]).max() < 1e-6 and np.abs(want[129, 1]).max() > 1e-3
    outs = []
    for tc in (True, False):
        out = torch.zeros((T, H * vdim), device="cuda", dtype=torch.bfloat16)
        ops.mapped_attention(dev(q.reshape(T, -1), torch.bfloat16), dev(pages, torch.bfloat16), ints(table), 64, ints(tok_pos),
                             ints(tok_seq), H, G, 1, dim, vdim, scale, 0, out, tiles=ints(np.array(tiles)), tensor_cores=tc,
                             head_scale=dev(temps), sink=True, gate=dev(gate, torch.bfloat16))
        got = out.float().cpu().numpy().reshape(T, H, vdim)
        err = np.abs(got - want).max(axis=(1, 2))
        bad = int(np.argmax(err > 4e-2))
        assert err.max() < 4e-2, f"tensor cores {tc}: first wrong token {bad} (sequence {tok_seq[bad]}, position {tok_pos[bad]})"
        outs.append(got)
    assert np.abs(outs[0] - outs[1]).max() < 3e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv,taps", [(4, 2, 16, 8, 4), (3, 3, 7, 5, 2), (2, 1, 33, 9, 1), (2, 2, 128, 64, 3),
                                            (2, 1, 200, 20, 2), (4, 4, 64, 17, 4), (2, 2, 16, 300, 2)])
def test_delta_rule_kernels(dtype, H, G, dk, dv, taps):
    """Convolution, preparation, recurrence and gated norm against the plain mixer with identity matrices around them:
    a prompt cut into steps of several sizes for two sequences that share the steps."""
    ops, rng = _ops(), np.random.default_rng(6)
    inner, qk = H * dv, G * dk
    ch = 2 * qk + inner
    wide = ch + inner + 2 * H
    eps = 1e-3
    m = {"heads": H, "kv_heads": G, "dim": dk, "vdim": dv, "conv": taps}
    eye = np.eye(wide)
    w = {"q": eye[:qk], "k": eye[qk:2 * qk], "v": eye[2 * qk:ch], "g": eye[ch:ch + inner], "b": eye[ch + inner:ch + inner + H],
         "a": eye[ch + inner + H:], "o": np.eye(inner), "q.conv": rng.normal(0, 0.6, (qk, taps)),
         "k.conv": rng.normal(0, 0.6, (qk, taps)), "v.conv": rng.normal(0, 0.6, (inner, taps)),
         "A_log": rng.uniform(-2, 1, H), "dt_bias": rng.uniform(-3, 1, H), "norm": rng.normal(1, 0.2, dv)}
    lens = [37, 21]
    us = [dev(rng.normal(0, 1.5, (n, wide)), dtype) for n in lens]
    want = [plain.delta_mixer(u.float().cpu().numpy().astype(np.float64), w, "", m, eps) for u in us]
    conv_w = dev(np.concatenate([w["q.conv"], w["k.conv"], w["v.conv"]]))
    tail = (taps - 1) * ch
    state = torch.full((5, tail + inner * dk), 9.0, device="cuda")
    slots = [3, 1]
    state[slots] = 0.0                                                   # what taking a slot does
    cuts = [[(0, 2), (2, 3), (3, 20), (20, 21), (21, 22), (22, 37)], [(0, 1), (1, 3), (3, 20), (20, 21), (21, 21), (21, 21)]]
    got = [[], []]
    for step in range(6):
        live = [s for s in range(2) if cuts[s][step][1] > cuts[s][step][0]]
        u = torch.cat([us[s][cuts[s][step][0]:cuts[s][step][1]] for s in live])
        counts = [cuts[s][step][1] - cuts[s][step][0] for s in live]
        T = sum(counts)
        seq = ints(np.repeat(np.arange(len(live)), counts))
        first, sl = ints(np.cumsum([0] + counts)), ints([slots[s] for s in live])
        qkv = torch.zeros((T, ch), device="cuda")
        ops.ssd_conv(u[:, :ch], conv_w, None, seq, first, sl, state, all(c == 1 for c in counts), qkv)
        kq, beta, decay = (torch.zeros((T, n), device="cuda") for n in (G, H, H))
        ops.delta_prepare(qkv, u[:, ch + inner:ch + inner + H], u[:, ch + inner + H:], dev(w["A_log"]), dev(w["dt_bias"]),
                          H, G, dk, dk ** -0.5, kq, beta, decay)
        o = torch.zeros((T, inner), device="cuda")
        ops.delta_scan(qkv, kq, beta, decay, H, G, dk, dv, first, sl, state, tail, o)
        out = torch.zeros((T, inner), device="cuda", dtype=dtype)
        ops.gated_group_norm(o, u[:, ch:ch + inner], dev(np.tile(w["norm"], H)), H, eps, out, gate_after=True)
        at = 0
        for s, c in zip(live, counts):
            got[s].append(out[at:at + c].float().cpu().numpy())
            at += c
    for s in range(2):
        err = np.abs(np.concatenate(got[s]) - want[s]).max(axis=1)
        tol = 5e-5 if dtype == torch.float32 else 4e-2
        assert err.max() < tol * max(1.0, np.abs(want[s]).max()), f"sequence {s}: first wrong token {int(np.argmax(err > tol))}"
    assert (state[[0, 2, 4]] == 9.0).all()                              # other slots' state is left alone


def test_delta_rule_keeps_a_value_over_hundreds_of_tokens():
    """A state that does not decay gives a value back hundreds of tokens after it was written, and across steps."""
    ops = _ops()
    H = G = 1
    dk, dv, T = 16, 4, 600
    qkv = np.zeros((T, 2 * dk + dv))
    for t in range(T):                                                  # every token its own key among 16; token 5's is asked again
        qkv[t, dk + (t % 15)] = 1.0
    qkv[:, dk:2 * dk][5] = 0.0
    qkv[5, dk + 15] = 1.0
    qkv[5, 2 * dk:] = (1.0, -2.0, 3.0, 0.5)
    qkv[T - 1, 15] = 1.0                                                # the last token's query points at token 5's key
    state = torch.zeros((1, dv * dk), device="cuda")
    outs = []
    for a, b in ((0, 300), (300, 599), (599, 600)):
        n = b - a
        o = torch.zeros((n, dv), device="cuda")
        ops.delta_scan(dev(qkv[a:b]), dev(np.zeros((n, 1))), dev(np.ones((n, 1))), dev(np.ones((n, 1))), H, G, dk, dv,
                       ints([0, n]), ints([0]), state, 0, o)
        outs.append(o.cpu().numpy())
    assert np.abs(outs[-1][0] - np.array([1.0, -2.0, 3.0, 0.5])).max() < 1e-6
