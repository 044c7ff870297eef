"""Tibopel's configuration: its nested config.json, typed, and its plan.

Keys read: ``vocab``, ``width``, ``norm.eps``, ``logit_softcap`` (optional) and the list ``layers``; an entry of
that list has ``type`` (the kind of mixer), ``mixer`` (its sizes), ``mlp`` (the feed-forward, or null) and
optionally ``weights_of`` (an earlier layer whose tensors this layer uses, with a cache of its own).
Mixer ``attention``: ``heads, kv_heads, dim, vdim, scale``, ``mask`` = {``size``} and ``rot`` = {``base, dims``,
optional ``scaling`` = {``factor, low, high, original``}}.
Mixer ``latent_attention``: ``heads, dim, rot_dim, vdim, kv_rank, q_rank, scale`` and ``rot`` = {``base, dims``}.
Feed-forward ``moe``: ``expert.ff``, ``router`` = {``experts, identity, top``} and optionally ``shared`` = {``ff``}.

The design: x = token row.  Every layer is parallel with two norms: x += mixer(N1 x) + ff(N2 x), both of the
same x, N(x) = x / sqrt(mean(x^2) + eps) * w.  Two kinds of mixer in any order.  (1) Grouped-query attention with
biases on its four projections, rotation of the first ``rot.dims`` entries of every query and key head (entry 2i
with entry 2i + 1, frequencies scaled by wavelength bands), scores times ``scale``, a mask of chunks (position p
sees p - p % size .. p, counted from the sequence's start), and a sigmoid gate per head from the mixer's input.
(2) Latent attention: queries through a normed latent, keys and values from one normed latent per position and
one rotated key part shared by the heads, causal, with a learned sink per head in the softmax's denominator.
The feed-forward routes every token to ``top`` of ``experts + identity`` router outputs by softmax score plus a
correction (weights: the chosen scores over their sum + 1e-20); an expert is down(max(up h, 0)^2), the last
``identity`` outputs pass h through; a shared expert of the same form is added behind a sigmoid gate per token.
At the end the same kind of norm, an output matrix and a soft cap c * tanh(logits / c).  Nothing limits the
positions; ``max_positions`` (an optional key of this library's, 131,072 if absent) only sizes the page lists.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping

from .base import ConfigError, KeyReader, LayerSpec, ModelPlan, PartSpec, ScheduleEntry

MIXERS = ("attention", "latent_attention")
DEFAULT_MAX_POSITIONS = 1 << 17
RENORM_EPS = 1e-20                    # added to the chosen scores' sum: the design fixes it


def _sub(reader: KeyReader, key: str) -> KeyReader:
    value = reader.raw.get(key)
    if not isinstance(value, Mapping):
        raise ConfigError(f"{reader.where}: key '{key}' must be an object")
    return KeyReader(value, f"{reader.where}: {key}")


def _check_rot(m: KeyReader, where: str, limit: int, banded: bool) -> None:
    rot = _sub(m, "rot")
    rot.number("base")
    dims = rot.integer("dims", minimum=0)
    if dims % 2 or dims > limit:
        raise ConfigError(f"{where}: rot.dims {dims} must be even and at most {limit}")
    if rot.raw.get("scaling") is not None:
        if not banded:
            raise ConfigError(f"{where}: rot.scaling is not part of this mixer")
        sc = _sub(rot, "scaling")
        for key in ("factor", "low", "high", "original"):
            sc.number(key)
        if not sc.number("high") > sc.number("low"):
            raise ConfigError(f"{where}: rot.scaling.high must exceed rot.scaling.low")


@dataclass(frozen=True)
class TibopelConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_softcap: float              # 0: none
    layers: tuple                     # the checked raw entries
    max_positions: int = DEFAULT_MAX_POSITIONS

    architecture = "Tibopel"

    @classmethod
    def from_json(cls, raw: Mapping[str, Any]) -> "TibopelConfig":
        r = KeyReader(raw)
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: key 'layers' must be a list with at least one layer")
        for i, layer in enumerate(layers):
            cls._check_layer(i, layer, layers)
        cap = raw.get("logit_softcap")
        return cls(vocab=r.integer("vocab"), width=r.integer("width"), norm_eps=_sub(r, "norm").number("eps"),
                   logit_softcap=0.0 if cap is None else r.number("logit_softcap"), layers=tuple(layers),
                   max_positions=r.integer("max_positions", default=DEFAULT_MAX_POSITIONS))

    @staticmethod
    def _check_layer(i: int, layer, layers) -> None:
        where = f"config.json: layers[{i}]"
        lr = KeyReader(layer, where)
        kind = lr.string("type", choices=MIXERS)
        src = layer.get("weights_of")
        if src is not None:
            src = lr.integer("weights_of", minimum=0)
            seen = {i}
            while True:                                    # up to the layer that owns the tensors
                if src >= len(layers) or src in seen or not isinstance(layers[src], Mapping):
                    raise ConfigError(f"{where}: weights_of leads to no layer that has tensors of its own")
                if layers[src].get("weights_of") is None:
                    break
                seen.add(src)
                src = KeyReader(layers[src], f"config.json: layers[{src}]").integer("weights_of", minimum=0)
            if layers[src].get("type") != kind:
                raise ConfigError(f"{where}: a layer that uses layer {src}'s tensors has its type")
        m = _sub(lr, "mixer")
        for key in ("heads", "dim", "vdim"):
            m.integer(key)
        m.number("scale")
        if kind == "attention":
            heads, kv = m.integer("heads"), m.integer("kv_heads")
            if heads % kv:
                raise ConfigError(f"{where}: heads {heads} must be a multiple of kv_heads {kv}")
            if m.raw.get("mask") is not None:
                _sub(m, "mask").integer("size")
            _check_rot(m, where, m.integer("dim"), banded=True)
        else:
            for key in ("kv_rank", "q_rank"):
                m.integer(key)
            rot_dim = m.integer("rot_dim", minimum=0)
            _check_rot(m, where, rot_dim, banded=True)
            if _sub(m, "rot").integer("dims", minimum=0) != rot_dim:
                raise ConfigError(f"{where}: the rotated part is rotated whole: rot.dims equals rot_dim")
        mlp = layer.get("mlp")
        if mlp is None:
            return
        f = KeyReader(mlp, where + ": mlp")
        f.string("kind", default="moe", choices=("moe",))
        _sub(f, "expert").integer("ff")
        router = _sub(f, "router")
        n, top = router.integer("experts"), router.integer("top")
        identity = router.integer("identity", default=0, minimum=0)
        if top > n + identity:
            raise ConfigError(f"{where}: mlp.router.top {top} exceeds its {n + identity} outputs")
        if mlp.get("shared") is not None:
            _sub(f, "shared").integer("ff")

    def to_json(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "layers": [dict(layer) for layer in self.layers]}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out

    def init_distribution(self, rule: str):
        """(mean, standard deviation) of a random-weights rule: matrices N(0, 1/width)."""
        r = 1.0 / math.sqrt(self.width)
        rules = {"normal": (0.0, r), "residual_projection": (0.0, r), "bias": (0.0, 0.1), "norm_weight": (1.0, 0.1)}
        if rule not in rules:
            raise ConfigError(f"no random-weights rule '{rule}'")
        return rules[rule]

    # ------------------------------------------------------------------ plan
    def _norm(self, name: str) -> PartSpec:
        return PartSpec("rms_norm", {"size": self.width, "eps": self.norm_eps}, {"weight": name})

    def _mixer(self, layer, p: str) -> PartSpec:
        D, m, x = self.width, layer["mixer"], p + "mix."
        if layer["type"] == "attention":
            return PartSpec(
                "mapped_attention",
                {"hidden_size": D, "n_heads": int(m["heads"]), "n_kv_heads": int(m["kv_heads"]), "dim": int(m["dim"]),
                 "vdim": int(m["vdim"]), "maps": 1, "softmax_scale": float(m["scale"]), "eps": self.norm_eps,
                 "rot": m["rot"], "bias": True, "qk_norm": False, "rot_layout": "pairs",
                 "chunk": int((m.get("mask") or {}).get("size", 0)), "head_gate": True},
                {"q": x + "q", "k": x + "k", "v": x + "v", "out": x + "o", "q_bias": x + "q.b", "k_bias": x + "k.b",
                 "v_bias": x + "v.b", "out_bias": x + "o.b", "gate": x + "g"})
        return PartSpec(
            "latent_attention",
            {"hidden_size": D, "n_heads": int(m["heads"]), "dim": int(m["dim"]), "rot_dim": int(m["rot_dim"]),
             "vdim": int(m["vdim"]), "kv_rank": int(m["kv_rank"]), "q_rank": int(m["q_rank"]),
             "softmax_scale": float(m["scale"]), "eps": self.norm_eps, "rot": m["rot"], "gate": False, "sink": True,
             "rot_layout": "pairs", "exact_weights": True},
            {"dq": x + "dq", "dq_norm": x + "dq.norm", "uq": x + "uq", "dkv": x + "dkv", "dkv_norm": x + "dkv.norm",
             "uk": x + "uk", "uv": x + "uv", "sink": x + "sink", "out": x + "o"})

    def _mlp(self, mlp, p: str) -> PartSpec:
        router, f = mlp["router"], p + "mlp."
        params = {"hidden_size": self.width, "inner_size": int(mlp["expert"]["ff"]), "n_experts": int(router["experts"]),
                  "identity": int(router.get("identity") or 0), "top": int(router["top"]), "score": "softmax",
                  "renormalize": True, "renorm_eps": RENORM_EPS, "correction": True, "expert_form": "relu2"}
        names = {"router": f + "router", "correction": f + "correction", "up": f + "e{e}.up", "down": f + "e{e}.down"}
        if mlp.get("shared") is not None:
            params["shared"] = {"inner_size": int(mlp["shared"]["ff"]), "gate": True}
            names.update({"shared_up": f + "shared.up", "shared_down": f + "shared.down", "shared_gate": f + "shared.sg"})
        return PartSpec("routed_experts", params, names)

    def plan(self) -> ModelPlan:
        D = self.width
        layers, schedule, own, ignored = [], [], {}, []
        for i, layer in enumerate(self.layers):
            if layer.get("weights_of") is not None:
                continue
            p = f"l{i}."
            mlp = layer.get("mlp")
            if mlp is None:
                norm2, ffn = PartSpec("identity"), PartSpec("none")
                ignored.append(rf"l{i}\.norm2")                 # a file may carry it all the same
            else:
                norm2, ffn = self._norm(p + "norm2"), self._mlp(mlp, p)
            own[i] = len(layers)
            layers.append(LayerSpec("parallel_pre_norm", self._norm(p + "norm1"), self._mixer(layer, p), norm2, ffn))
        for i, layer in enumerate(self.layers):
            # a layer with `weights_of` runs that layer's parts (or, if that one borrows its tensors too, the ones
            # it uses) with a cache of its own
            j = i
            while self.layers[j].get("weights_of") is not None:
                j = int(self.layers[j]["weights_of"])
            schedule.append(ScheduleEntry(layer=own[j], cache_of=i))
        plan = ModelPlan(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=D, max_positions=self.max_positions,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": D}, {"weight": "embed"}),
            position=PartSpec("none"), layers=tuple(layers), schedule=tuple(schedule),
            final_norm=self._norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": D, "softcap": self.logit_softcap},
                          {"weight": "head"}), ignored_tensors=tuple(ignored))
        plan.validate()
        return plan
