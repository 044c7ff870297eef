"""Seledra's configuration and plan, the cache it asks for, and properties of the plain statement itself; no device
needed."""
import json

import numpy as np
import pytest
import torch

import plain_seledra as plain
from math_utils_b200.cache import SequenceCache
from math_utils_b200.config import ConfigError, SeledraConfig, architecture_for
from math_utils_b200.engine.assemble import assemble, collect_tensor_specs
from math_utils_b200.parts import RowCacheSpec, StateCacheSpec

ATT = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "scale": 0.3, "v_mix": True}
DELTA = {"heads": 4, "kv_heads": 2, "dim": 10, "vdim": 6, "conv": 3}
CFG = {"architecture": "Seledra", "vocab": 90, "width": 32, "max_positions": 256, "residual_mult": 0.5,
       "norm": {"eps": 1e-5},
       "layers": [{"type": "attention", "mixer": dict(ATT, v_mix=False), "mlp": {"kind": "dense", "ff": 48}},
                  {"type": "attention", "mixer": ATT, "mlp": {"kind": "dense", "ff": 48}},
                  {"type": "delta", "mixer": DELTA, "mlp": None},
                  {"type": "attention", "mixer": dict(ATT, heads=2, dim=16), "mlp": None}]}


def test_configuration_and_plan():
    assert architecture_for(CFG).config_class is SeledraConfig
    plan = SeledraConfig.from_json(CFG).plan()
    assert [e.cache_of for e in plan.schedule] == [0, 1, 2, 3]
    # the first layer that shares its values hands them on, the later ones blend; a layer that shares nothing does neither
    assert [l.mixer.params.get("value_mix") for l in plan.layers] == ["none", "source", None, "blend"]
    assert plan.layers[2].feed_forward.kind == "none" and plan.layers[2].mixer.kind == "gated_delta"
    assert all(l.arrangement == "scaled_pre_norm" and l.arrangement_params["residual_mult"] == 0.5 for l in plan.layers)
    assert SeledraConfig.from_json(SeledraConfig.from_json(CFG).to_json()).plan() == plan
    names = {s.name: tuple(s.shape) for s in collect_tensor_specs(plan) if not s.optional}
    assert names == plain.tensor_shapes(CFG)


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=8), "share values"),          # shared values of two sizes
    (lambda c: c["layers"][2]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0].update(type="parallel"), "type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "kind"),
    (lambda c: c.pop("residual_mult"), "residual_mult"),
    (lambda c: c.pop("max_positions"), "max_positions"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_configuration_errors_name_the_key(change, word):
    bad = json.loads(json.dumps(CFG))
    change(bad)
    with pytest.raises(ConfigError, match=word):
        SeledraConfig.from_json(bad)


def test_cache_of_the_plan():
    plan = SeledraConfig.from_json(CFG).plan()
    specs = [layer.mixer.cache_spec() for layer in assemble(plan).layers]
    assert specs[0] == specs[1] == RowCacheSpec(2 * 8 + 2 * 12, 0) and specs[3] == RowCacheSpec(2 * 16 + 2 * 12, 0)
    channels = 2 * 2 * 10 + 4 * 6
    assert specs[2] == StateCacheSpec(2 * channels + 4 * 6 * 10)
    cache = SequenceCache(specs, 64 * 6, 256, torch.float32, "cpu", n_slots=3)
    assert len(cache.kv_groups) == 2 and len(cache.state_groups) == 1 and cache.has_running_state
    a = cache.acquire()
    cache.entry(2).values[a] = 3.0
    cache.release(a)
    assert cache.acquire() == a and (cache.entry(2).values[a] == 0.0).all()      # state starts at zero for the next holder


def test_plain_statement_sink_blend_and_state():
    """The plain statement itself: with every score far below zero the sink takes the whole softmax; the blend's
    two ends; the recurrence stores a value under its key and gives it back."""
    rng = np.random.default_rng(0)
    k, v = rng.normal(0, 1, (9, 4)), rng.normal(0, 1, (9, 3))
    q = -40.0 * k[3] / (k[3] ** 2).sum() * np.ones((9, 1))
    out = plain.sink_softmax_attention(q, np.tile(k[3], (9, 1)), v, 1.0)
    assert np.abs(out).max() < 1e-12
    out = plain.sink_softmax_attention(-q, np.tile(k[3], (9, 1)), v, 1.0)
    assert np.abs(out[0] - v[0]).max() < 1e-12                                   # a score of +40: the sink's share is nothing
    w = {"v": rng.normal(0, 1, (6, 5)), "v.b": np.zeros(6), "vmix": np.array(1.0)}
    h = rng.normal(0, 1, (2, 5))
    first = rng.normal(0, 1, (2, 2, 3))
    m = {"kv_heads": 2, "vdim": 3, "v_mix": True}
    assert np.array_equal(plain.attention_values(h, w, "", m, 1e-6, first, False), first)
    own = plain.attention_values(h, w, "", m, 1e-6, first, True)
    assert np.abs((own ** 2).mean(-1) - 1.0).max() < 1e-5
    assert np.array_equal(plain.attention_values(h, dict(w, vmix=np.array(0.0)), "", m, 1e-6, first, False), own)
    key = np.zeros((3, 4)); key[:, 1] = 1.0
    val = rng.normal(0, 1, (3, 2))
    out = plain.delta_recurrence(key, key, val, np.ones(3), np.ones(3))
    assert np.abs(out - val).max() < 1e-12                                       # beta 1: the new value replaces the old one
    out = plain.delta_recurrence(key, key, val, np.zeros(3), np.ones(3))
    assert np.abs(out).max() == 0.0
    z = np.array([-2.0, 0.0, 1.5])
    got = plain.xielu(z, np.array([0.3, -0.4]))
    ap, an = np.log1p(np.exp(0.3)), 0.5 + np.log1p(np.exp(-0.4))
    assert np.allclose(got, [an * (np.exp(-2.0) + 1.0) - 1.0, 0.0, ap * 2.25 + 0.75])
