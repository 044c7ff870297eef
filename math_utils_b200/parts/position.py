"""Position encodings.

``learned_absolute``: a ``[max_positions, hidden]`` table whose row for a
token's absolute position is added to its embedding
(include/ai/LocalModel.hpp:3694-3697); queries and keys are left as they are.

``rotary_frequencies``: the frequency table of a rotary encoding, plain or
stretched for long contexts; the mixers that rotate their own queries and keys
hand it to ``ops.rotary``.
"""
from __future__ import annotations

from ..config.base import ConfigError, PartSpec
from .base import PositionEncoding, TensorSpec, register_part


class LearnedAbsolutePositions(PositionEncoding):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.max_positions = int(self.param("max_positions"))
        self.hidden_size = int(self.param("hidden_size"))

    def tensor_specs(self):
        return (TensorSpec(self.tensor_name("weight"), (self.max_positions, self.hidden_size), role="table"),)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.weight = tensors[self.tensor_name("weight")]

    def embedding_table(self):
        return self.weight


class NoPositions(PositionEncoding):
    """Nothing is added and nothing is rotated."""


register_part("position", "learned_absolute", LearnedAbsolutePositions, replace=True)
register_part("position", "none", NoPositions, replace=True)


# ------------------------------------------------------------------ rotary frequencies
def rotary_frequencies(dims: int, base: float, scaling=None):
    """(frequencies, magnitude) of a rotary encoding over ``dims`` entries in the rotate-half layout
    (entry i turns with entry i + dims/2): f_i = base^(-2i/dims), i < dims/2, magnitude 1.

    ``scaling`` = {factor, original, fast, slow} stretches the slow dimensions for contexts longer than
    the ``original`` one (the YaRN rule: Peng, Quesnelle, Fan, Shippole, "YaRN: Efficient Context Window
    Extension of Large Language Models"): with turns(t) = dims ln(original / (2 pi t)) / (2 ln base), the
    dimensions below lo = floor(turns(fast)) keep f_i, those above hi = ceil(turns(slow)) get f_i / factor,
    a linear ramp lies between, and cos and sin are multiplied by 0.1 ln(factor) + 1.

    ``scaling`` = {factor, low, high, original} is the rule by wavelength bands (as Llama 3.1 scales its
    frequencies): with l = 2 pi / f, a frequency keeps its value where l < original / high, becomes
    f / factor where l > original / low, and in between is (1 - s) f / factor + s f with
    s = (original / l - low) / (high - low); the magnitude stays 1.  Which rule applies follows from the
    keys.  The order of the frequencies is that of the pairs, whatever the layout of a pair's two entries
    (i with i + dims/2, or 2i with 2i + 1: the kernels take that as a switch).

    Computed in float64 here; the kernels take the table as float32."""
    import math
    if dims < 0 or dims % 2:
        raise ConfigError(f"a rotary encoding turns an even number of entries, got {dims}")
    half = dims // 2
    freqs = [base ** (-2.0 * i / dims) for i in range(half)]
    if not scaling:
        return freqs, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])
    if "low" in scaling or "high" in scaling:
        low, high = float(scaling["low"]), float(scaling["high"])
        if not high > low:
            raise ConfigError("rotary scaling by wavelength bands needs high > low")
        banded = []
        for f in freqs:
            length = 2.0 * math.pi / f
            if length < original / high:
                banded.append(f)
            elif length > original / low:
                banded.append(f / factor)
            else:
                s = (original / length - low) / (high - low)
                banded.append((1.0 - s) * f / factor + s * f)
        return banded, 1.0

    def turns(t):
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turns(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turns(float(scaling["slow"]))), dims - 1)
    out = []
    for i, f in enumerate(freqs):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0
