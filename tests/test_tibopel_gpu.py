"""Tibopel through the engine against the plain NumPy statement of the design (plain_tibopel.py):
each mechanism alone, whole prompts, token-by-token decoding, prompts in portions, unequal batches,
slots and pages used again, keys far away, at page borders and just inside and outside the chunks,
the first tokens, long decoding, odd sizes, and greedy generation through the library's own entry point."""
import functools
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_tibopel as plain
import helpers
from helpers import run_batch, run_tail_one_by_one, run_whole
from math_utils_b200 import DecoderModel, LLM, StepEntry
from math_utils_b200.weights.safetensors import write_safetensors

pytestmark = pytest.mark.gpu

check_logits = helpers.check_logits


def attention(heads, kv_heads, dim, vdim, scale, chunk, rot_dims, base=1.0e4, scaling=None, mlp=None, **more):
    rot = {"base": base, "dims": rot_dims}
    if scaling is not None:
        rot["scaling"] = scaling
    return dict({"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                                                "scale": scale, "mask": {"size": chunk}, "rot": rot}, "mlp": mlp}, **more)


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base=1.0e4, mlp=None, **more):
    return dict({"type": "latent_attention",
                 "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                           "scale": scale, "rot": {"base": base, "dims": rot_dim}}, "mlp": mlp}, **more)


def moe(experts, identity, top, ff, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def config(vocab, width, eps, cap, layers):
    out = {"architecture": "Tibopel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if cap is not None:
        out["logit_softcap"] = cap
    return out


BANDS = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
# chunks that are no whole pages (48) and several pages (160); layers that run again with the tensors of an earlier
# one; a layer without a feed-forward; three key/value heads for six; a latent wider than the heads' keys
_A0 = attention(4, 2, 16, 24, 0.25, 48, 8, base=100.0, scaling=BANDS, mlp=moe(5, 2, 2, 48, shared=40))
_A1 = latent(2, 16, 8, 12, 40, 24, 0.2, base=50.0, mlp=moe(4, 0, 2, 32, shared=24))
CFG_A = config(300, 64, 1e-6, 12.0, [
    _A0, _A1, dict(_A0, weights_of=0), attention(6, 3, 8, 16, 0.35, 160, 8, mlp=None), dict(_A1, weights_of=1),
    latent(3, 8, 16, 24, 16, 8, 0.3, mlp=moe(3, 3, 1, 24))])
# nothing a multiple of 8; as many kv heads as heads and one kv head; one head; chunks of 7 and of 1; all experts
# chosen, one chosen, no shared expert, identity experts only beside one expert; nothing rotated; no soft cap;
# a latent layer first and used again
_B0 = latent(1, 5, 2, 3, 9, 5, 0.4, base=30.0, mlp=moe(3, 0, 3, 10))
CFG_B = config(131, 50, 1e-3, None, [
    _B0, attention(3, 3, 6, 5, 0.4, 7, 4, base=20.0, mlp=moe(1, 2, 2, 14, shared=9)),
    attention(6, 1, 5, 15, 0.5, 1, 0, mlp=moe(5, 1, 1, 7)), dict(_B0, weights_of=0),
    latent(5, 3, 6, 7, 11, 13, 0.3, mlp=None)])
# sizes the tensor-core kernels take; a chunk of one page, of half a page and of two pages
CFG_C = config(384, 128, 2e-5, 30.0, [
    attention(8, 2, 32, 64, 0.18, 64, 16, base=1.0e4, scaling=dict(BANDS, original=32, factor=4.0), mlp=moe(8, 4, 2, 64, shared=128)),
    latent(4, 32, 16, 32, 64, 48, 0.15, mlp=moe(8, 2, 3, 64, shared=64)),
    attention(4, 2, 64, 32, 0.125, 32, 64, mlp=moe(4, 0, 2, 128)),
    latent(8, 16, 32, 16, 96, 64, 0.2, mlp=None), attention(4, 4, 128, 64, 0.09, 128, 32, mlp=moe(6, 1, 2, 64, shared=64))])
CONFIGS = {"a": CFG_A, "b": CFG_B, "c": CFG_C}


@functools.lru_cache(maxsize=None)
def weights_of(name, dtype="float32"):
    """Random weights.  The bfloat16 runs get routers that rounding cannot tip: a choice between two experts whose
    scores nearly tie is a matter of noise there, and one flipped choice moves a whole row of logits.  Their
    corrections lie 1.3 apart, more than a softmax score can bridge, so the choice is the same for every token
    while the weights still follow the scores; routing that varies from token to token is what the float32 runs
    and the kernels' own test (exact choices, bfloat16 rows) cover.  For the same reason their queries and keys
    are of ordinary size: where two keys nearly tie at the top of a peaked softmax, rounding decides between them."""
    w = plain.random_weights(CONFIGS[name], seed=sum(map(ord, name)) + 17, sharp=3.0 if dtype == "float32" else 1.0)
    if dtype == "bfloat16":
        rng = np.random.default_rng(5)
        for k in list(w):
            if k.endswith(".correction"):
                w[k] = rng.permutation(len(w[k])) * 1.3125
    return w


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, cfg in CONFIGS.items():
        for dtype in ("float32", "bfloat16"):
            d = str(tmp_path_factory.mktemp(f"tibopel_{name}_{dtype}"))
            with open(os.path.join(d, "config.json"), "w") as f:
                json.dump(cfg, f)
            write_safetensors(os.path.join(d, "model.safetensors"),
                              {k: torch.from_numpy(np.array(v)).to(torch.bfloat16) for k, v in weights_of(name, dtype).items()})
            out[name, dtype] = d
    return out


_models = {}


def engine(folders, name, dtype):
    key = (name, dtype)
    if key not in _models:
        model = DecoderModel.from_dir(folders[key], dtype=dtype)
        _models[key] = (model, model.new_cache(max_tokens=64 * 24, n_slots=8))
    return _models[key]


def tokens_for(name, n, seed=0):
    return np.random.default_rng(7000 + seed).integers(0, CONFIGS[name]["vocab"], size=n).tolist()


_plain_cache = {}


def plain_logits(name, dtype, tokens):
    key = (name, dtype, tuple(tokens))
    if key not in _plain_cache:
        _plain_cache[key] = plain.forward(CONFIGS[name], weights_of(name, dtype), list(tokens))
    return _plain_cache[key]


CASES = [(n, d) for n in CONFIGS for d in ("float32", "bfloat16")]


# ------------------------------------------------------------------ whole models
@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_prompt_and_every_layer(folders, name, dtype):
    model, cache = engine(folders, name, dtype)
    toks = tokens_for(name, 200)
    layers = []
    want = plain.forward(CONFIGS[name], weights_of(name, dtype), toks, layers)
    slot = cache.acquire()
    trace = {}
    got = model.step(cache, [StepEntry(slot, toks, list(range(len(toks))))], trace=trace).cpu().numpy()
    cache.release(slot)
    assert len(layers) == len(CONFIGS[name]["layers"])
    if dtype == "float32":
        for i, x in enumerate(layers):
            assert np.abs(trace[f"h.{i}.res2"] - x).max() < 2e-4, f"residual stream after layer run {i}"
    check_logits(got, want, dtype, f"tibopel {name} whole prompt")
    check_logits(run_whole(model, cache, toks), want, dtype, f"tibopel {name} whole prompt, no trace")


@pytest.mark.parametrize("name,dtype", CASES)
def test_prompt_then_token_by_token(folders, name, dtype):
    model, cache = engine(folders, name, dtype)
    toks = tokens_for(name, 200, seed=1)                 # the tail crosses page borders and the ends of chunks
    got = run_tail_one_by_one(model, cache, toks, tail=170)
    check_logits(got, plain_logits(name, dtype, toks), dtype, f"tibopel {name} tail one by one")


@pytest.mark.parametrize("name,dtype", CASES)
@pytest.mark.parametrize("portions", [(2, 3, 59, 1, 64, 21), (64, 64, 22), (127, 2, 2, 19), (1, 1, 1, 147),
                                      (2,) * 12 + (126,), (47, 2, 47, 49, 5)])
def test_prompt_in_portions(folders, name, dtype, portions):
    model, cache = engine(folders, name, dtype)
    toks = tokens_for(name, sum(portions), seed=2)
    slot = cache.acquire()
    rows, at = [], 0
    for n in portions:
        rows.append(model.step(cache, [StepEntry(slot, toks[at:at + n], list(range(n)))]).cpu().numpy())
        at += n
    cache.release(slot)
    check_logits(np.concatenate(rows), plain_logits(name, dtype, toks), dtype, f"tibopel {name} portions {portions}")


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_batch_against_each_alone(folders, name, dtype):
    model, cache = engine(folders, name, dtype)
    lens, prompts = (140, 5, 66, 200), (129, 1, 33, 64)
    requests = [tokens_for(name, n, seed=10 + i) for i, n in enumerate(lens)]
    got = run_batch(model, cache, requests, prompts)
    for i, r in enumerate(requests):
        check_logits(got[i], plain_logits(name, dtype, r), dtype, f"tibopel {name} batch request {i}")
        if dtype == "float32":
            alone = run_tail_one_by_one(model, cache, r, tail=lens[i] - prompts[i])
            assert np.abs(alone - got[i]).max() < 2e-5, "a request's logits depend on its batch"


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("b", "bfloat16"), ("c", "float32")])
def test_slots_and_pages_used_again(folders, name, dtype):
    model, cache = engine(folders, name, dtype)
    free = [cache.free_pages(g.index) for g in cache.kv_groups]
    first = tokens_for(name, 200, seed=20)
    second = tokens_for(name, 90, seed=21)
    a = run_whole(model, cache, first)
    slot = cache.acquire()                               # the slot and the pages the first request held
    model.step(cache, [StepEntry(slot, second[:70], [])])
    b = [model.step(cache, [StepEntry(slot, [t], [0])]).cpu().numpy() for t in second[70:]]
    cache.release(slot)
    assert [cache.free_pages(g.index) for g in cache.kv_groups] == free
    check_logits(a, plain_logits(name, dtype, first), dtype, f"tibopel {name} first holder")
    check_logits(np.concatenate(b), plain_logits(name, dtype, second)[70:], dtype, f"tibopel {name} second holder of the same slot")


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("b", "float32"), ("c", "bfloat16")])
@pytest.mark.parametrize("n", [1, 2, 3, 4, 5, 47, 48, 49, 63, 64, 65, 127, 128, 129, 193])
def test_first_tokens_and_lengths_around_borders(folders, name, dtype, n):
    model, cache = engine(folders, name, dtype)
    toks = tokens_for(name, 193, seed=30)[:n]
    slot = cache.acquire()
    got = model.step(cache, [StepEntry(slot, toks, [0, n - 1])]).cpu().numpy()
    cache.release(slot)
    want = plain_logits(name, dtype, tokens_for(name, 193, seed=30))   # causal: a prefix's logits are the long prompt's
    check_logits(got, want[[0, n - 1]], dtype, f"tibopel {name} prompt of {n}")


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("b", "float32"), ("c", "bfloat16")])
def test_long_decoding(folders, name, dtype):
    model, cache = engine(folders, name, dtype)
    toks = tokens_for(name, 270, seed=40)
    free = [cache.free_pages(g.index) for g in cache.kv_groups]
    got = run_tail_one_by_one(model, cache, toks, tail=267)            # three tokens, then one by one over four pages
    check_logits(got, plain_logits(name, dtype, toks), dtype, f"tibopel {name} long decoding")
    assert [cache.free_pages(g.index) for g in cache.kv_groups] == free


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_greedy_generation_through_the_library(folders, name):
    llm = LLM(folders[name, "float32"], dtype="float32", temperature=0.0, max_tokens=24, context=512)
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
    llm = LLM(folders["a", "float32"], dtype="float32", temperature=0.0, max_tokens=30, context=512)
    prompts = [tokens_for("a", n, seed=70 + n) for n in (40, 9, 66, 3, 21)]
    free = llm.generate(prompts, stop_ids=[])
    stop = free[0][5]
    want = [out[:out.index(stop)] if stop in out else out for out in free]
    got = llm.generate(prompts, stop_ids=[stop])
    assert got == want
    assert llm.generate(prompts[1:], stop_ids=[stop]) == want[1:]


def test_generation_in_bfloat16_follows_the_plain_model(folders):
    llm = LLM(folders["c", "bfloat16"], dtype="bfloat16", temperature=0.0, max_tokens=12, context=512)
    prompts = [tokens_for("c", n, seed=90 + n) for n in (65, 7)]
    for p, out in zip(prompts, llm.generate(prompts)):
        seq = list(p)
        for tok in out:
            row = plain.forward(CONFIGS["c"], weights_of("c", "bfloat16"), seq)[-1]
            best = int(np.argmax(row))
            assert tok == best or row[best] - row[tok] < helpers.BF16_NEAR_TIE * 2.5 * max(row.std(), 1e-3)
            seq.append(tok)


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("b", "bfloat16")])
def test_replay_of_steps_through_the_program(folders, name, dtype, tmp_path):
    """``bin/trace_run``: a batch of unequal prompts decoded together, requests that end early, then a second batch
    that takes over the freed slots and pages; every position's logits against the plain model."""
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
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders[name, dtype], "--dtype", dtype,
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
        check_logits(np.stack(got), plain_logits(name, dtype, r), dtype, f"tibopel {name} replayed request {rid}")


# ------------------------------------------------------------------ mechanisms alone
def _ops():
    from math_utils_b200.csrc import ops
    return ops


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device="cuda", dtype=dtype)


def ints(a):
    return dev(np.asarray(a), torch.int32)


def held(a, dtype):
    """What the device holds of ``a`` in ``dtype``, as float64."""
    return dev(a, dtype).float().cpu().numpy().astype(np.float64)


def test_frequencies_scaled_by_wavelength_bands():
    from math_utils_b200.parts.position import rotary_frequencies
    for dims, base, sc in ((24, 1.0e6, {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 2048}),
                           (8, 100.0, BANDS), (64, 1.0e4, {"factor": 32.0, "low": 2.0, "high": 3.0, "original": 16}), (6, 50.0, None)):
        got, magnitude = rotary_frequencies(dims, base, sc)
        want = plain.rotary_frequencies(dims, base, sc)
        assert magnitude == 1.0 and np.allclose(got, want, rtol=1e-13)
    kept, stretched = plain.rotary_frequencies(8, 100.0, BANDS)[0], plain.rotary_frequencies(8, 100.0, BANDS)[-1]
    assert kept == 1.0 and stretched == 100.0 ** -0.75 / 8.0              # the test's premise: both ends of the rule occur


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dim,vdim,rot", [(4, 2, 16, 24, 8), (3, 3, 6, 5, 4), (6, 1, 5, 15, 0), (2, 2, 64, 32, 64), (2, 1, 40, 8, 22)])
def test_rotation_in_pairs_without_norms_and_cache_rows(dtype, H, G, dim, vdim, rot):
    """Queries in place, keys and values into scattered cache rows; entry 2i turns with entry 2i + 1; nothing is normed."""
    ops, rng = _ops(), np.random.default_rng(3)
    positions = np.array([0, 1, 63, 64, 130, 5, 40000])
    seq_of = np.array([0, 0, 0, 1, 1, 2, 2])
    table = np.zeros((3, 700), dtype=np.int32)
    table[0, :2], table[1, :3], table[2, 0], table[2, 625] = (4, 1), (2, 6, 5), 3, 0
    T = len(positions)
    freqs = plain.rotary_frequencies(rot, 37.0, BANDS) if rot else np.zeros(0)
    q, k, v = (dev(rng.normal(0, 2, (T, n)), dtype) for n in (H * dim, G * dim, G * vdim))
    want_q = plain.rotate_pairs(held(q.cpu().float().numpy(), dtype).reshape(T, H, dim), positions, freqs).reshape(T, -1)
    want_k = plain.rotate_pairs(held(k.cpu().float().numpy(), dtype).reshape(T, G, dim), positions, freqs).reshape(T, -1)
    rows = torch.zeros((7, 64, G * (dim + vdim)), device="cuda", dtype=dtype)
    ops.qk_prepare(q, k, v, None, None, dev(freqs if rot else np.zeros(1)), 1.0, rot, 1e-5, H, G, 1, dim, vdim, ints(positions),
                   ints(seq_of), ints(table), 64, rows, pairs=True)
    tol = 2e-5 if dtype == torch.float32 else 4e-2
    # (float32 angles at position 40,000 differ from float64 ones by a few 1e-3 of a turn for the fastest pairs)
    err = np.abs(q.float().cpu().numpy() - want_q).max(axis=1)
    assert err[:6].max() < tol and err[6] < 3e-2 + tol
    got = rows.float().cpu().numpy()
    for t, (p, s) in enumerate(zip(positions, seq_of)):
        row = got[table[s, p // 64], p % 64]
        assert np.abs(row[:G * dim] - want_k[t]).max() < (tol if t < 6 else 3e-2 + tol)
        assert np.array_equal(row[G * dim:], v[t].float().cpu().numpy())
    assert np.count_nonzero(got.reshape(-1, got.shape[-1]).any(axis=1)) == T       # no other row was touched


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
            piece = rows[i * page:(i + 1) * page]
            pages[order[at], :len(piece)] = piece
            at += 1
    return seqs, pages, table


def _set_row(seqs, pages, table, s, j, lo, hi, values):
    seqs[s][j, lo:hi] = values
    pages[table[s, j // 64], j % 64, lo:hi] = values


def _chunk_heads(q, rows, pos, dim, vdim, H, G, scale, gate, chunk):
    """One token's heads [H, vdim] from its sequence's rows, through the plain function."""
    n = pos + 1
    k = rows[:n, :G * dim].reshape(n, G, dim)
    v = rows[:n, G * dim:].reshape(n, G, vdim)
    out = np.zeros((H, vdim))
    for a in range(H):
        g = a // (H // G)
        qq = np.zeros((n, dim))
        qq[-1] = q[a]
        out[a] = plain.masked_attention(qq, k[:, g], v[:, g], scale, lambda i: i - i % chunk)[-1] * plain.sigmoid(gate[a])
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dim,vdim,chunk", [(4, 2, 16, 24, 48), (3, 3, 6, 5, 7), (6, 1, 5, 15, 1), (4, 2, 64, 32, 64),
                                                (2, 2, 8, 200, 160), (8, 2, 32, 64, 1000), (34, 2, 16, 16, 48)])
def test_chunked_attention_with_gates(dtype, H, G, dim, vdim, chunk):
    """The general kernel and the one of single-token steps.  In the longest sequence the key just before the query's
    chunk is made enormous along one query's direction (it must not be seen: it would take the whole softmax), and
    the first key of the chunk is made large (it must come through)."""
    ops, rng = _ops(), np.random.default_rng(5)
    lens = [1, 2, 63, 64, 65, 300, 1400]
    width = G * (dim + vdim)
    seqs, pages, table = _paged(rng, lens, width)
    scale = 0.37
    picks = [(s, n - 1) for s, n in enumerate(lens)] + [(5, p) for p in (0, 47, 48, 63, 64, 127, 128, 191, 192, 250)] + [(6, 1100)]
    q = rng.normal(0, 1, (len(picks), H, dim)) / math.sqrt(dim) * 3
    gate = rng.normal(0, 2, (len(picks), H))
    pos = lens[6] - 1
    inside = pos - pos % chunk                                       # the first position the last query sees
    direction = np.zeros(dim); direction[0] = 1.0
    q[6, 0] = direction * 25.0 / scale
    if inside > 0:
        _set_row(seqs, pages, table, 6, inside - 1, 0, dim, direction * 4.0)          # score 100 if it were seen
    if inside < pos:
        _set_row(seqs, pages, table, 6, inside, 0, dim, direction * 2.0)              # score 50: the head's result is its value
    for j in range(inside + 1, pos + 1):
        _set_row(seqs, pages, table, 6, j, 0, 1, 0.0)
    if dtype == torch.bfloat16:                                       # the cache holds what bfloat16 can hold
        pages = held(pages, dtype)
        seqs = [np.concatenate([pages[table[s, i]] for i in range(-(-n // 64))])[:n] for s, n in enumerate(lens)]
        q, gate = held(q, dtype), held(gate, dtype)
    want = np.stack([_chunk_heads(q[i], seqs[s], p, dim, vdim, H, G, scale, gate[i], chunk) for i, (s, p) in enumerate(picks)])
    if inside < pos:                                                  # the test's own premise
        v_in = seqs[6][inside, G * dim:G * dim + vdim] * plain.sigmoid(gate[6, 0])
        assert np.abs(want[6, 0] - v_in).max() < 1e-6 * max(1.0, np.abs(v_in).max())
    tol = 3e-5 if dtype == torch.float32 else 4e-2
    for single in (False, True):
        out = torch.zeros((len(picks), H * vdim), device="cuda", dtype=dtype)
        ops.mapped_attention(dev(q.reshape(len(picks), -1), dtype), dev(pages, dtype), ints(table), 64,
                             ints([p for _, p in picks]), ints([s for s, _ in picks]), H, G, 1, dim, vdim, scale, 0, out,
                             single_tokens=single, gate=dev(gate, dtype), chunk=chunk)
        got = out.float().cpu().numpy().reshape(len(picks), H, vdim)
        err = np.abs(got - want).max(axis=(1, 2))
        assert err.max() < tol, f"single {single}: first wrong query {picks[int(np.argmax(err > tol))]}"


@pytest.mark.parametrize("H,G,dim,vdim,chunk", [(4, 2, 16, 16, 48), (8, 2, 128, 64, 64), (3, 3, 32, 48, 7), (2, 1, 80, 112, 160),
                                                (4, 1, 64, 64, 32)])
def test_chunked_attention_on_tensor_cores_prompt_tiles(H, G, dim, vdim, chunk):
    """Several sequences' tokens in one step as tiles of up to 64; some sequences bring only their last tokens.  For
    EVERY token the key just before its chunk is enormous along the direction that head 0's query has, so a kernel
    that let one such key in anywhere would show it."""
    ops, rng = _ops(), np.random.default_rng(8)
    lens, new = [130, 1, 64, 65, 7, 200], [130, 1, 64, 3, 7, 70]
    width = G * (dim + vdim)
    seqs, pages, table = _paged(rng, lens, width)
    scale = 0.21
    tok_seq = np.repeat(np.arange(len(lens)), new)
    tok_pos = np.concatenate([np.arange(n - k, n) for n, k in zip(lens, new)])
    T = len(tok_seq)
    q = rng.normal(0, 1, (T, H, dim)) / math.sqrt(dim) * 4
    gate = rng.normal(0, 2, (T, H))
    # entry 0 of kv head 0's keys: +6 at the last position of every chunk, 0 elsewhere; head 0's queries: +10 / scale
    # there.  A key at the end of the chunk before would score 60 above everything a token may see, except for the
    # token that is itself the last of its chunk, which sees its own.
    for s, n in enumerate(lens):
        for j in range(n):
            _set_row(seqs, pages, table, s, j, 0, 1, 6.0 if j % chunk == chunk - 1 else 0.0)
    q[:, 0, 0] = 10.0 / scale
    pages = held(pages, torch.bfloat16)
    seqs = [np.concatenate([pages[table[s, i]] for i in range(-(-n // 64))])[:n] for s, n in enumerate(lens)]
    q, gate = held(q, torch.bfloat16), held(gate, torch.bfloat16)
    tiles, at = [], 0
    for k in new:
        tiles += [(at + o, min(64, k - o)) for o in range(0, k, 64)]
        at += k
    tiles.sort(key=lambda t: -tok_pos[t[0] + t[1] - 1])
    want = np.stack([_chunk_heads(q[t], seqs[tok_seq[t]], tok_pos[t], dim, vdim, H, G, scale, gate[t], chunk) for t in range(T)])
    outs = []
    for tc in (True, False):
        out = torch.zeros((T, H * vdim), device="cuda", dtype=torch.bfloat16)
        ops.mapped_attention(dev(q.reshape(T, -1), torch.bfloat16), dev(pages, torch.bfloat16), ints(table), 64, ints(tok_pos),
                             ints(tok_seq), H, G, 1, dim, vdim, scale, 0, out, tiles=ints(np.array(tiles)), tensor_cores=tc,
                             gate=dev(gate, torch.bfloat16), chunk=chunk)
        got = out.float().cpu().numpy().reshape(T, H, vdim)
        err = np.abs(got - want).max(axis=(1, 2))
        bad = int(np.argmax(err > 4e-2))
        assert err.max() < 4e-2, f"tensor cores {tc}: first wrong token {bad} (sequence {tok_seq[bad]}, position {tok_pos[bad]})"
        outs.append(got)
    assert np.abs(outs[0] - outs[1]).max() < 3e-2


def _latent_heads(q, rows, pos, r, H, scale, sinks):
    """One token's weighted sums of latents [H, r] from its sequence's rows: the keys are the whole rows, the values
    their first r entries."""
    n = pos + 1
    out = np.zeros((H, r))
    for a in range(H):
        qq = np.zeros((n, rows.shape[1]))
        qq[-1] = q[a]
        out[a] = plain.masked_attention(qq, rows[:n], rows[:n, :r], scale, lambda i: 0, sink=sinks[a])[-1]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,r,rot", [(2, 40, 8), (1, 9, 2), (5, 11, 6), (4, 64, 16), (8, 96, 32), (40, 64, 16)])
def test_latent_attention_with_learned_sinks(dtype, H, r, rot):
    """Rows far back, at page borders, the first tokens; a sink so large that it takes the whole softmax, one so small
    that it takes nothing, and a query that scores every key far below an ordinary sink."""
    ops, rng = _ops(), np.random.default_rng(9)
    lens = [1, 2, 63, 64, 65, 300, 1400]
    width = r + rot
    seqs, pages, table = _paged(rng, lens, width)
    far = 9
    _set_row(seqs, pages, table, 6, far, 0, width, seqs[6][far] * 4.0)        # a long row: no other row comes near its score
    for j in range(lens[5]):
        _set_row(seqs, pages, table, 5, j, 0, 1, 3.0)
    scale = 0.29
    sinks = rng.normal(0.5, 1.5, H)
    sinks[-1] = 60.0                                                  # takes the whole softmax: the head's result is nothing
    if H > 1:
        sinks[0] = -60.0                                              # takes nothing
    if dtype == torch.bfloat16:
        pages = held(pages, dtype)
        seqs = [np.concatenate([pages[table[s, i]] for i in range(-(-n // 64))])[:n] for s, n in enumerate(lens)]
    picks = [(s, n - 1) for s, n in enumerate(lens)] + [(5, p) for p in (0, 63, 64, 127, 128, 250)] + [(6, 1100)]
    q = rng.normal(0, 1, (len(picks), H, width)) / math.sqrt(width) * 3
    q[6, 0] = seqs[6][far] * 30.0 / scale / (seqs[6][far] ** 2).sum()          # points at the row 1,390 positions back
    if H > 2:
        q[5, 1] = 0.0
        q[5, 1, 0] = -40.0 / (3.0 * scale)                            # every key at -40: the sink takes the softmax
    # (the tensor-core kernel rounds the queries to bfloat16: give it queries that bfloat16 holds)
    q = held(q, torch.bfloat16)
    want = np.stack([_latent_heads(q[i], seqs[s], p, r, H, scale, sinks) for i, (s, p) in enumerate(picks)])
    assert np.abs(want[:, -1]).max() < 1e-9                                                # the test's own premises
    if H > 1:
        assert np.abs(want[6, 0] - seqs[6][far, :r]).max() < 1e-3 * np.abs(seqs[6][far, :r]).max()
    if H > 2:
        assert np.abs(want[5, 1]).max() < 1e-12
    tol = 3e-5 if dtype == torch.float32 else 4e-2
    T = len(picks)
    for splits, single, tc, two in ((1, False, False, False), (3, False, False, False), (1, True, True, False),
                                    (4, True, True, False), (1, True, False, False), (1, True, True, True), (4, True, True, True)):
        out = torch.zeros((T, H * r), device="cuda", dtype=dtype)
        part_o = torch.zeros(T * H * splits * r, device="cuda") if splits > 1 else None
        part_ml = torch.zeros(T * H * splits * 2, device="cuda") if splits > 1 else None
        ops.latent_attention(dev(q.reshape(T, -1)), dev(pages, dtype), ints(table), 64, ints([p for _, p in picks]),
                             ints([s for s, _ in picks]), H, r, scale, out, splits, part_o, part_ml, single_tokens=single,
                             tensor_cores=tc, sink=dev(sinks), two_term_weights=two)
        got = out.float().cpu().numpy().reshape(T, H, r)
        err = np.abs(got - want).max(axis=(1, 2))
        assert err.max() < tol * max(1.0, np.abs(want).max()), \
            f"splits {splits}, single {single}, tensor cores {tc}: first wrong query {picks[int(np.argmax(err > tol))]}"


def test_latent_attention_with_sinks_prompt_tiles_on_tensor_cores():
    ops, rng = _ops(), np.random.default_rng(10)
    H, r, rot, scale = 4, 64, 16, 0.2
    lens, new = [130, 1, 64, 65, 7, 200], [130, 1, 64, 3, 7, 70]
    seqs, pages, table = _paged(rng, lens, r + rot)
    pages = held(pages, torch.bfloat16)
    seqs = [np.concatenate([pages[table[s, i]] for i in range(-(-n // 64))])[:n] for s, n in enumerate(lens)]
    tok_seq = np.repeat(np.arange(len(lens)), new)
    tok_pos = np.concatenate([np.arange(n - k, n) for n, k in zip(lens, new)])
    T = len(tok_seq)
    q = held(rng.normal(0, 1, (T, H, r + rot)) / math.sqrt(r + rot) * 4, torch.bfloat16)
    sinks = np.array([-60.0, 0.3, 2.0, 60.0])
    tiles, at = [], 0
    for k in new:
        tiles += [(at + o, min(64, k - o)) for o in range(0, k, 64)]
        at += k
    tiles.sort(key=lambda t: -tok_pos[t[0] + t[1] - 1])
    want = np.stack([_latent_heads(q[t], seqs[tok_seq[t]], tok_pos[t], r, H, scale, sinks) for t in range(T)])
    rms = {}
    for tc, two in ((True, False), (True, True), (False, False)):
        out = torch.zeros((T, H * r), device="cuda", dtype=torch.bfloat16)
        ops.latent_attention(dev(q.reshape(T, -1)), dev(pages, torch.bfloat16), ints(table), 64, ints(tok_pos), ints(tok_seq), H, r,
                             scale, out, tiles=ints(np.array(tiles)), tensor_cores=tc, sink=dev(sinks), two_term_weights=two)
        diff = out.float().cpu().numpy().reshape(T, H, r) - want
        err = np.abs(diff).max(axis=(1, 2))
        assert err.max() < 4e-2, f"tensor cores {tc}, two terms {two}: first wrong token {int(np.argmax(err > 4e-2))}"
        rms[tc, two] = float(np.sqrt((diff ** 2).mean()))
    # weights in two terms leave little more than the rounding of the result itself, as the float32 weights of the
    # CUDA-core kernel do; weights rounded to eight bits leave visibly more
    assert rms[True, True] < 1.05 * rms[False, False] and rms[True, True] < 0.92 * rms[True, False], rms


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_rows_and_query_parts_rotated_in_pairs(dtype):
    ops, rng = _ops(), np.random.default_rng(11)
    r, rot, H, dim = 12, 6, 3, 5
    positions, seq_of = np.array([0, 1, 63, 64, 300]), np.array([0, 0, 0, 1, 1])
    table = np.zeros((2, 8), dtype=np.int32)
    table[0, 0], table[1, 1], table[1, 4] = 2, 0, 1
    freqs = plain.rotary_frequencies(rot, 30.0)
    T = len(positions)
    down = dev(rng.normal(0, 2, (T, r + rot)), dtype)
    qh = dev(rng.normal(0, 2, (T, H * (dim + rot))), dtype)
    w, eps = rng.normal(1, 0.2, r), 1e-2
    x, qx = held(down.float().cpu().numpy(), dtype), held(qh.float().cpu().numpy(), dtype).reshape(T, H, dim + rot)
    want_row = np.concatenate([plain.rms_norm(x[:, :r], w, eps), plain.rotate_pairs(x[:, r:], positions, freqs)], axis=1)
    want_q = plain.rotate_pairs(qx[..., dim:], positions, freqs)
    rows = torch.zeros((3, 64, r + rot), device="cuda", dtype=dtype)
    qa = torch.zeros((T, H * (r + rot)), device="cuda")
    ops.latent_append(down, dev(w), eps, dev(freqs), 1.0, rot, r, rot, ints(positions), ints(seq_of), ints(table), 64, rows,
                      queries=(qh[:, dim:], dim + rot, qa[:, r:], r + rot, H), pairs=True)
    tol = 3e-5 if dtype == torch.float32 else 4e-2
    got = rows.float().cpu().numpy()
    for t, (p, s) in enumerate(zip(positions, seq_of)):
        assert np.abs(got[table[s, p // 64], p % 64] - want_row[t]).max() < tol
    assert np.abs(qa.cpu().numpy().reshape(T, H, r + rot)[..., r:] - want_q).max() < 3e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D,E,n_id,top,ff,shared", [(64, 5, 2, 2, 48, 40), (50, 3, 0, 3, 10, None), (50, 1, 2, 2, 14, 9),
                                                    (128, 8, 4, 3, 64, 128), (40, 2, 5, 1, 16, 8), (64, 6, 6, 4, 32, None)])
def test_routed_experts_with_identity_and_shared_experts(dtype, D, E, n_id, top, ff, shared):
    """The whole feed-forward part against the plain function, few rows and many (both tile sizes): choices that the
    corrections change, identity experts among the chosen, weights over their sum, the shared expert behind its gate."""
    from math_utils_b200.config.base import PartSpec
    from math_utils_b200.engine.batch import StepContext
    from math_utils_b200.engine.runtime import Runtime
    from math_utils_b200.parts.base import build_part
    rng = np.random.default_rng(12)
    f = moe(E, n_id, top, ff, shared)
    cfg = config(16, D, 1e-5, None, [latent(1, 8, 2, 8, 8, 8, 0.1, mlp=f)])
    w = {k[len("l0.mlp."):]: v for k, v in plain.random_weights(cfg, 5).items() if k.startswith("l0.mlp.")}
    params = {"hidden_size": D, "inner_size": ff, "n_experts": E, "identity": n_id, "top": top, "score": "softmax",
              "renormalize": True, "renorm_eps": 1e-20, "correction": True, "expert_form": "relu2"}
    names = {"router": "router", "correction": "correction", "up": "e{e}.up", "down": "e{e}.down"}
    if shared:
        params["shared"] = {"inner_size": shared, "gate": True}
        names.update(shared_up="shared.up", shared_down="shared.down", shared_gate="shared.sg")
    part = build_part("feed_forward", PartSpec("routed_experts", params, names))
    runtime = Runtime.create("float32" if dtype == torch.float32 else "bfloat16", "cuda:0")
    tensors = {}
    for spec in part.tensor_specs():
        tensors[spec.name] = dev(w[spec.name], torch.float32 if spec.role in ("vector", "matrix32") else dtype)
    part.bind(tensors, runtime)
    for T in (1, 7, 700):
        h = dev(rng.normal(0, 1, (T, D)), dtype)
        hx = held(h.float().cpu().numpy(), dtype)
        chosen, _ = plain.route(hx, w, "", f)
        if n_id and T > 1:
            assert (chosen >= E).any() and (chosen < E).any()            # the test's premise: both kinds are chosen
        want = plain.routed_experts(hx, w, "", f)
        ctx = StepContext(runtime=runtime, position=None, n_tokens=T, n_seqs=1, token_ids=None, tok_pos=None, tok_seq=None,
                          want_rows=None, block_tables=[], seq_slots=None, slots=[0], starts=[0], q_lens=[T], max_q_len=T,
                          max_kv_len=T)
        before = rng.normal(0, 1, (T, D))
        x = dev(before)
        part.forward(h, x, ctx)
        got = x.cpu().numpy() - before.astype(np.float32)
        tol = 2e-5 if dtype == torch.float32 else 3e-2
        err = np.abs(got - want).max(axis=1)
        assert err.max() < tol * max(1.0, np.abs(want).max()), f"{T} rows: first wrong row {int(np.argmax(err > tol))}"
        y = torch.full((T, D), 7.0, device="cuda")
        part.forward(h, y, ctx, accumulate=False)                         # written, not added
        assert np.abs(y.cpu().numpy() - want).max() < tol * max(1.0, np.abs(want).max())


def test_two_norms_of_one_stream_and_soft_cap():
    ops, rng = _ops(), np.random.default_rng(13)
    for n in (50, 64, 320, 4100):
        x, w1, w2 = rng.normal(0, 3, (6, n)), rng.normal(1, 0.2, n), rng.normal(1, 0.2, n)
        for eps in (1e-6, 0.7):
            for dtype, tol in ((torch.float32, 5e-6), (torch.bfloat16, 4e-2)):
                a, b = (torch.zeros((6, n), device="cuda", dtype=dtype) for _ in range(2))
                ops.rms_norm_pair(dev(x), dev(w1), dev(w2), eps, a, b)
                assert np.abs(a.float().cpu().numpy() - plain.rms_norm(x, w1, eps)).max() < tol
                assert np.abs(b.float().cpu().numpy() - plain.rms_norm(x, w2, eps)).max() < tol
    z = rng.normal(0, 40, (5, 77))
    got = ops.softcap(dev(z), 12.5).cpu().numpy()
    assert np.abs(got - 12.5 * np.tanh(z / 12.5)).max() < 1e-5 and np.abs(got).max() < 12.5 + 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [1, 20, 50, 300])
def test_products_with_the_squared_activation(dtype, rows):
    """Every product kernel's epilogue (few rows, some rows, many rows; both dtypes) with max(z, 0)^2."""
    ops, rng = _ops(), np.random.default_rng(14)
    x, w, b = dev(rng.normal(0, 1, (rows, 64)), dtype), dev(rng.normal(0, 0.2, (136, 64)), dtype), dev(rng.normal(0, 0.3, 136))
    want = plain.relu_squared(held(x.float().cpu().numpy(), dtype) @ held(w.float().cpu().numpy(), dtype).T + b.cpu().numpy().astype(np.float64))
    got = ops.linear(x, w, b, act="relu2").float().cpu().numpy()
    assert np.abs(got - want).max() < (2e-5 if dtype == torch.float32 else 3e-2) * max(1.0, np.abs(want).max())
