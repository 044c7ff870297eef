"""Tibopel's configuration and plan, the cache it asks for, and properties of the plain statement itself; no device
needed."""
import json

import numpy as np
import pytest
import torch

import plain_tibopel as plain
from math_utils_b200.cache import SequenceCache
from math_utils_b200.config import ConfigError, TibopelConfig, architecture_for
from math_utils_b200.engine.assemble import assemble, collect_tensor_specs
from math_utils_b200.parts import RowCacheSpec

ATT = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "scale": 0.3, "mask": {"size": 10},
       "rot": {"base": 100.0, "dims": 4, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}}
LAT = {"heads": 3, "dim": 8, "rot_dim": 4, "vdim": 6, "kv_rank": 10, "q_rank": 7, "scale": 0.2, "rot": {"base": 50.0, "dims": 4}}
MOE = {"kind": "moe", "expert": {"ff": 16}, "router": {"experts": 3, "identity": 2, "top": 2}, "shared": {"ff": 8}}
CFG = {"architecture": "Tibopel", "vocab": 90, "width": 32, "norm": {"eps": 1e-5}, "logit_softcap": 20.0,
       "layers": [{"type": "attention", "mixer": ATT, "mlp": MOE},
                  {"type": "latent_attention", "mixer": LAT, "mlp": None},
                  {"type": "attention", "mixer": ATT, "mlp": MOE, "weights_of": 0},
                  {"type": "latent_attention", "mixer": LAT, "mlp": None, "weights_of": 1},
                  {"type": "attention", "mixer": ATT, "mlp": MOE, "weights_of": 2}]}


def test_configuration_and_plan():
    assert architecture_for(CFG).config_class is TibopelConfig
    plan = TibopelConfig.from_json(CFG).plan()
    # two layers with tensors; five runs, each with a cache of its own; a run that borrows from a borrower uses the owner's
    assert len(plan.layers) == 2
    assert [(e.layer, e.cache_of) for e in plan.schedule] == [(0, 0), (1, 1), (0, 2), (1, 3), (0, 4)]
    a, l = plan.layers
    assert a.arrangement == l.arrangement == "parallel_pre_norm"
    assert a.mixer.kind == "mapped_attention" and a.mixer.params["chunk"] == 10 and a.mixer.params["rot_layout"] == "pairs"
    assert a.mixer.params["qk_norm"] is False and a.mixer.params["head_gate"] and a.mixer.params["bias"]
    assert l.mixer.kind == "latent_attention" and l.mixer.params["sink"] and not l.mixer.params["gate"]
    assert l.mixer.params["q_rank"] == 7 and l.feed_forward.kind == "none"
    f = a.feed_forward.params
    assert (f["n_experts"], f["identity"], f["top"], f["score"], f["renormalize"], f["expert_form"]) == (3, 2, 2, "softmax", True, "relu2")
    assert f["shared"] == {"inner_size": 8, "gate": True} and f["renorm_eps"] == 1e-20
    assert plan.head.params["softcap"] == 20.0
    assert TibopelConfig.from_json(TibopelConfig.from_json(CFG).to_json()).plan() == plan
    names = {s.name: tuple(s.shape) for s in collect_tensor_specs(plan) if not s.optional}
    assert names == plain.tensor_shapes(CFG)


def test_tensors_borrowed_from_a_later_layer():
    cfg = json.loads(json.dumps(CFG))
    cfg["layers"][0]["weights_of"] = 4                     # 0 -> 4 -> 2: layer 2 owns the tensors
    cfg["layers"][2].pop("weights_of")
    plan = TibopelConfig.from_json(cfg).plan()
    assert [(e.layer, e.cache_of) for e in plan.schedule] == [(1, 0), (0, 1), (1, 2), (0, 3), (1, 4)]
    names = {s.name for s in collect_tensor_specs(plan)}
    assert "l2.mix.q" in names and "l0.mix.q" not in names and names == set(plain.tensor_shapes(cfg))


def test_optional_keys():
    cfg = json.loads(json.dumps(CFG))
    del cfg["logit_softcap"]
    cfg["layers"][0]["mlp"]["router"].pop("identity")
    cfg["layers"][0]["mlp"].pop("shared")
    cfg["layers"][0]["mixer"]["rot"].pop("scaling")
    for i in (2, 4):
        cfg["layers"][i]["mlp"], cfg["layers"][i]["mixer"] = cfg["layers"][0]["mlp"], cfg["layers"][0]["mixer"]
    plan = TibopelConfig.from_json(cfg).plan()
    f = plan.layers[0].feed_forward.params
    assert plan.head.params["softcap"] == 0.0 and f["identity"] == 0 and "shared" not in f
    names = {s.name: tuple(s.shape) for s in collect_tensor_specs(plan) if not s.optional}
    assert names == plain.tensor_shapes(cfg) and "l0.mlp.shared.sg" not in names and names["l0.mlp.router"] == (3, 32)


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=3), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("high"), "high"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=2), "rot_dim"),
    (lambda c: c["layers"][1]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0].update(type="delta"), "type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "kind"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "top"),
    (lambda c: c["layers"][2].update(weights_of=2), "weights_of"),
    (lambda c: c["layers"][2].update(weights_of=9), "weights_of"),
    (lambda c: (c["layers"][0].update(weights_of=2), c["layers"][2].update(weights_of=0)), "weights_of"),
    (lambda c: c["layers"][3].update(weights_of=0), "type"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.pop("width"), "width"),
])
def test_configuration_errors_name_the_key(change, word):
    bad = json.loads(json.dumps(CFG))
    change(bad)
    with pytest.raises(ConfigError, match=word):
        TibopelConfig.from_json(bad)


def test_cache_of_the_plan():
    plan = TibopelConfig.from_json(CFG).plan()
    layers = assemble(plan).layers
    specs = [layers[e.layer].mixer.cache_spec() for e in plan.schedule]
    assert specs[0] == specs[2] == specs[4] == RowCacheSpec(2 * 8 + 2 * 12, 0) and specs[1] == specs[3] == RowCacheSpec(10 + 4, 0)
    cache = SequenceCache(specs, 64 * 6, 256, torch.float32, "cpu", n_slots=3)
    assert len(cache.kv_groups) == 2 and not cache.has_running_state
    # every run has pages of its own, the runs that share tensors too
    assert len({id(cache.entry(i).pages) if hasattr(cache.entry(i), "pages") else i for i in range(5)}) >= 2
    assert len({cache.entry(i).pages.data_ptr() for i in range(5)}) == 5


def test_plain_statement_chunks_sinks_and_experts():
    """The plain statement itself: a key outside the chunk counts for nothing; a sink far above every score takes the
    softmax; identity experts pass the input; the frequencies' rule keeps the short waves and stretches the long."""
    rng = np.random.default_rng(0)
    k, v = rng.normal(0, 0.1, (9, 4)), rng.normal(0, 1, (9, 3))
    k[2] = (3.0, 0.0, 0.0, 0.0)
    q = np.tile(np.array([20.0, 0.0, 0.0, 0.0]), (9, 1))                       # every query points at key 2
    out = plain.masked_attention(q, k, v, 1.0, lambda i: i - i % 3)
    assert np.abs(out[2] - v[2]).max() < 1e-9                                  # position 2 sees key 2
    assert np.abs(out[3] - v[3]).max() < 1e-12                                 # position 3 starts a chunk: only itself
    assert np.abs(out[4] - v[2]).max() > 1e-3
    out = plain.masked_attention(q, k, v, 1.0, lambda i: 0, sink=1e4)
    assert np.abs(out).max() < 1e-300
    out = plain.masked_attention(q, k, v, 1.0, lambda i: 0, sink=-1e4)
    assert np.abs(out[8] - v[2]).max() < 1e-9
    f = {"router": {"experts": 1, "identity": 2, "top": 2}}
    w = {"router": np.zeros((3, 5)), "correction": np.array([0.0, 1.0, 2.0]), "e0.up": rng.normal(0, 1, (4, 5)),
         "e0.down": rng.normal(0, 1, (5, 4))}
    h = rng.normal(0, 1, (3, 5))
    assert np.allclose(plain.routed_experts(h, w, "", f), h)                   # both chosen are identity experts, weights 1/2 each
    w["correction"] = np.array([2.0, 1.0, 0.0])
    want = 0.5 * h + 0.5 * plain.relu_squared(h @ w["e0.up"].T) @ w["e0.down"].T
    assert np.allclose(plain.routed_experts(h, w, "", f), want)
    fr = plain.rotary_frequencies(8, 100.0, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64})
    assert fr[0] == 1.0 and fr[3] == 100.0 ** -0.75 / 8.0 and 100.0 ** -0.25 / 8.0 < fr[1] < 100.0 ** -0.25
    x = rng.normal(0, 1, (2, 6))
    turned = plain.rotate_pairs(x, [0, 3], np.array([0.5]))
    assert np.array_equal(turned[0], x[0]) and np.array_equal(turned[1, 2:], x[1, 2:])
    assert np.allclose(turned[1, :2], [x[1, 0] * np.cos(1.5) - x[1, 1] * np.sin(1.5), x[1, 1] * np.cos(1.5) + x[1, 0] * np.sin(1.5)])
