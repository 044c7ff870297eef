"""Seledra's configuration: its nested config.json, typed, and its plan.

Keys read: ``vocab``, ``width``, ``max_positions`` (rows of the learned position table), ``residual_mult``,
``norm.eps`` and the list ``layers``; an entry of that list has ``type`` (the kind of mixer), ``mixer`` (its sizes)
and ``mlp`` (the feed-forward, or null for a layer that ends after its mixer).
Mixer ``attention``: ``heads, kv_heads, dim, vdim, scale, v_mix``.
Mixer ``delta`` (gated delta rule): ``heads, kv_heads, dim, vdim, conv``.
Feed-forward ``dense``: ``ff``.

The design: x = token row + position row.  Every layer is pre-norm with one multiplier m = ``residual_mult`` on
what its sublayers add: x += m * mixer(norm1(x)); x += m * ff(norm2(x)), the norms x / rms(x) * w.
Attention: projections with biases; queries and keys normed over the whole projection; values normed per head;
scores times ``scale`` and a learned number per head; a softmax with a sink; a sigmoid gate per head; no rotation.
The layers with ``v_mix`` share values: the first of them hands its values on, each later one caches a blend of its
own and those.  Delta layers keep a matrix state per head.  The feed-forward is two matrices around an activation
with two learned numbers.  At the end the same kind of norm and an output matrix.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping

from .base import ConfigError, KeyReader, LayerSpec, ModelPlan, PartSpec, default_schedule

MIXERS = ("attention", "delta")


def _sub(reader: KeyReader, key: str) -> KeyReader:
    value = reader.raw.get(key)
    if not isinstance(value, Mapping):
        raise ConfigError(f"{reader.where}: key '{key}' must be an object")
    return KeyReader(value, f"{reader.where}: {key}")


@dataclass(frozen=True)
class SeledraConfig:
    vocab: int
    width: int
    max_positions: int
    residual_mult: float
    norm_eps: float
    layers: tuple                     # the checked raw entries

    architecture = "Seledra"

    @classmethod
    def from_json(cls, raw: Mapping[str, Any]) -> "SeledraConfig":
        r = KeyReader(raw)
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: key 'layers' must be a list with at least one layer")
        shared = None
        for i, layer in enumerate(layers):
            where = f"config.json: layers[{i}]"
            lr = KeyReader(layer, where)
            kind = lr.string("type", choices=MIXERS)
            m = _sub(lr, "mixer")
            heads, kv = m.integer("heads"), m.integer("kv_heads")
            if heads % kv:
                raise ConfigError(f"{where}: heads {heads} must be a multiple of kv_heads {kv}")
            m.integer("dim"); m.integer("vdim")
            if kind == "attention":
                m.number("scale")
                if m.boolean("v_mix", default=False):
                    sizes = (kv, m.integer("vdim"))
                    if shared is not None and sizes != shared:
                        raise ConfigError(f"{where}: layers that share values agree on kv_heads and vdim")
                    shared = sizes
            else:
                m.integer("conv")
            mlp = layer.get("mlp")
            if mlp is not None:
                f = KeyReader(mlp, where + ": mlp")
                f.string("kind", choices=("dense",))
                f.integer("ff")
        return cls(vocab=r.integer("vocab"), width=r.integer("width"), max_positions=r.integer("max_positions"),
                   residual_mult=r.number("residual_mult", positive=False), norm_eps=_sub(r, "norm").number("eps"),
                   layers=tuple(layers))

    def to_json(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "max_positions": self.max_positions, "residual_mult": self.residual_mult,
                "norm": {"eps": self.norm_eps}, "layers": [dict(layer) for layer in self.layers]}

    def init_distribution(self, rule: str):
        """(mean, standard deviation) of a random-weights rule: matrices N(0, 1/width)."""
        r = 1.0 / math.sqrt(self.width)
        rules = {"normal": (0.0, r), "residual_projection": (0.0, r), "bias": (0.0, 0.1),
                 "norm_weight": (1.0, 0.1), "head_scale": (1.0, 0.2), "mix": (0.4, 0.05), "conv": (0.0, 0.5),
                 "act_params": (0.0, 0.5)}
        if rule not in rules:
            raise ConfigError(f"no random-weights rule '{rule}'")
        return rules[rule]

    # ------------------------------------------------------------------ plan
    def _norm(self, name: str) -> PartSpec:
        return PartSpec("rms_norm", {"size": self.width, "eps": self.norm_eps}, {"weight": name})

    def plan(self) -> ModelPlan:
        D = self.width
        layers = []
        source = None                   # the first layer that shares its values
        for i, layer in enumerate(self.layers):
            p, m = f"l{i}.", layer["mixer"]
            x = p + "mix."
            if layer["type"] == "attention":
                mix = "none"
                if m.get("v_mix"):
                    mix = "source" if source is None else "blend"
                    source = i if source is None else source
                names = {"q": x + "q", "k": x + "k", "v": x + "v", "q_bias": x + "q.b", "k_bias": x + "k.b",
                         "v_bias": x + "v.b", "q_norm": x + "q.norm", "k_norm": x + "k.norm", "head_scale": x + "temp",
                         "gate": x + "g", "out": x + "o", "mix": x + "vmix"}
                mixer = PartSpec("sink_attention",
                                 {"hidden_size": D, "n_heads": int(m["heads"]), "n_kv_heads": int(m["kv_heads"]),
                                  "dim": int(m["dim"]), "vdim": int(m["vdim"]), "softmax_scale": float(m["scale"]),
                                  "eps": self.norm_eps, "window": 0, "bias": True, "value_norm": True, "sink": True,
                                  "head_scale": True, "head_gate": True, "value_mix": mix}, names)
            else:
                names = {"q": x + "q", "k": x + "k", "v": x + "v", "q_conv": x + "q.conv", "k_conv": x + "k.conv",
                         "v_conv": x + "v.conv", "beta": x + "b", "decay": x + "a", "A_log": x + "A_log",
                         "dt_bias": x + "dt_bias", "norm": x + "norm", "gate": x + "g", "out": x + "o"}
                mixer = PartSpec("gated_delta",
                                 {"hidden_size": D, "n_heads": int(m["heads"]), "n_kv_heads": int(m["kv_heads"]),
                                  "dim": int(m["dim"]), "vdim": int(m["vdim"]), "conv": int(m["conv"]),
                                  "eps": self.norm_eps}, names)
            mlp = layer.get("mlp")
            if mlp is None:
                norm2, ffn = PartSpec("identity"), PartSpec("none")
            else:
                norm2 = self._norm(p + "norm2")
                ffn = PartSpec("dense_ffn", {"hidden_size": D, "inner_size": int(mlp["ff"]), "activation": "xielu",
                                             "bias": False},
                               {"up_weight": p + "mlp.up", "down_weight": p + "mlp.down", "act_params": p + "mlp.act"})
            layers.append(LayerSpec("scaled_pre_norm", self._norm(p + "norm1"), mixer, norm2, ffn,
                                    arrangement_params={"residual_mult": self.residual_mult}))
        plan = ModelPlan(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=D, max_positions=self.max_positions,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": D}, {"weight": "embed"}),
            position=PartSpec("learned_absolute", {"max_positions": self.max_positions, "hidden_size": D},
                              {"weight": "pos"}),
            layers=tuple(layers), schedule=default_schedule(len(layers)),
            final_norm=self._norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": D}, {"weight": "head"}))
        plan.validate()
        return plan
