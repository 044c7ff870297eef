"""A plain, slow statement of the Seledra design in NumPy float64, one function per mechanism.

It shares no code with the package: the tests hold the package's kernels, cache and scheduler to
these functions.  A model is a dict ``config`` (the JSON of config.json) and a dict ``w`` of arrays by
tensor name.  Everything works on one whole sequence (positions 0..T-1); what a cache or a state
would hold is simply recomputed.

Notation: x the residual stream [T, D]; h a sublayer's input (the normed stream); H query heads,
G key/value heads; d the query/key size, d_v the value size; m the residual multiplier.
"""
import math

import numpy as np

F = np.float64


# ------------------------------------------------------------------ elementwise
def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, weight, eps):
    return unit_rms(x, eps) * weight


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def xielu(z, pair):
    """Two branches that meet at zero with slope 1/2: a quadratic one above, an exponential one below;
    ``pair`` holds the two raw parameters, each passed through softplus."""
    a_pos = softplus(float(pair[0]))
    a_neg = 0.5 + softplus(float(pair[1]))
    neg = np.minimum(z, 0.0)
    return np.where(z > 0.0, a_pos * z * z + 0.5 * z, a_neg * (np.exp(neg) - 1.0 - neg) + 0.5 * z)


# ------------------------------------------------------------------ embedding
def embedding(tokens, w):
    tokens = np.asarray(tokens, dtype=np.int64)
    return w["embed"][tokens] + w["pos"][np.arange(len(tokens))]


# ------------------------------------------------------------------ attention with a sink
def sink_softmax_attention(q, k, v, scale):
    """One head: q [T, d], k [T, d], v [T, d_v]; ``scale`` multiplies the scores.  Causal; the denominator
    counts one more key whose score is zero and whose value is nothing."""
    T = q.shape[0]
    out = np.zeros((T, v.shape[1]), dtype=F)
    for i in range(T):
        s = (k[: i + 1] @ q[i]) * scale
        top = max(float(s.max()), 0.0)
        e = np.exp(s - top)
        out[i] = (e @ v[: i + 1]) / (math.exp(-top) + e.sum())
    return out


def attention_values(h, w, p, m, eps, first_values, is_first):
    """The values a layer caches: per head brought to unit rms, then (in a mixing layer that is not the
    first of them) blended with the first mixing layer's values of the same token."""
    G, dv = int(m["kv_heads"]), int(m["vdim"])
    T = h.shape[0]
    v = h @ w[p + "v"].T + w[p + "v.b"]
    v = unit_rms(v.reshape(T, G, dv), eps)
    if m.get("v_mix") and not is_first:
        lam = float(w[p + "vmix"])
        v = (1.0 - lam) * v + lam * first_values
    return v


def attention_mixer(h, w, p, m, eps, first_values=None, is_first=True):
    """Returns (output [T, D], the cached values [T, G, d_v])."""
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    q = rms_norm(h @ w[p + "q"].T + w[p + "q.b"], w[p + "q.norm"], eps).reshape(T, H, d)
    k = rms_norm(h @ w[p + "k"].T + w[p + "k.b"], w[p + "k.norm"], eps).reshape(T, G, d)
    v = attention_values(h, w, p, m, eps, first_values, is_first)
    gate = sigmoid(h @ w[p + "g"].T)                       # [T, H]
    heads = np.zeros((T, H, dv), dtype=F)
    for a in range(H):
        g = a // (H // G)
        heads[:, a] = sink_softmax_attention(q[:, a], k[:, g], v[:, g], float(m["scale"]) * float(w[p + "temp"][a]))
        heads[:, a] *= gate[:, a: a + 1]
    return heads.reshape(T, H * dv) @ w[p + "o"].T, v


# ------------------------------------------------------------------ gated delta rule
def short_convolution(u, taps_weight):
    """Causal convolution per channel: u [T, C], taps_weight [C, taps], the last tap on the current token,
    zeros before the start; then silu."""
    T, C = u.shape
    taps = taps_weight.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C), dtype=F), u], axis=0)
    out = np.zeros((T, C), dtype=F)
    for j in range(taps):
        out += padded[j: j + T] * taps_weight[:, j]
    return silu(out)


def unit_vector(x):
    return x / np.sqrt(np.sum(x * x, axis=-1, keepdims=True) + 1e-6)


def delta_recurrence(q, k, v, beta, decay):
    """One head: q, k [T, d]; v [T, d_v]; beta, decay [T].  S [d, d_v] from zero: decay, write the
    difference between the value and what the key reads, read with the query."""
    T, d = q.shape
    S = np.zeros((d, v.shape[1]), dtype=F)
    out = np.zeros_like(v)
    for t in range(T):
        S = decay[t] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + np.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def delta_mixer(h, w, p, m, eps):
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    q = short_convolution(h @ w[p + "q"].T, w[p + "q.conv"]).reshape(T, G, d)
    k = short_convolution(h @ w[p + "k"].T, w[p + "k.conv"]).reshape(T, G, d)
    v = short_convolution(h @ w[p + "v"].T, w[p + "v.conv"]).reshape(T, H, dv)
    q = unit_vector(q) * d ** -0.5
    k = unit_vector(k)
    beta = sigmoid(h @ w[p + "b"].T)                                           # [T, H]
    decay = np.exp(-np.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    gate = silu(h @ w[p + "g"].T).reshape(T, H, dv)
    heads = np.zeros((T, H, dv), dtype=F)
    for a in range(H):
        g = a // (H // G)
        o = delta_recurrence(q[:, g], k[:, g], v[:, a], beta[:, a], decay[:, a])
        heads[:, a] = unit_rms(o, eps) * w[p + "norm"] * gate[:, a]
    return heads.reshape(T, H * dv) @ w[p + "o"].T


# ------------------------------------------------------------------ feed-forward
def feed_forward(h, w, p):
    return xielu(h @ w[p + "up"].T, w[p + "act"]) @ w[p + "down"].T


# ------------------------------------------------------------------ the model
def forward(config, w, tokens, layers_out=None):
    """Logits [T, vocab] of one whole sequence; ``layers_out`` (a list) receives the stream after every layer."""
    w = {k: np.asarray(v, dtype=F) for k, v in w.items()}
    eps, m = float(config["norm"]["eps"]), float(config["residual_mult"])
    x = embedding(tokens, w)
    first_values = None
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = rms_norm(x, w[p + "norm1"], eps)
        mix = layer["mixer"]
        if layer["type"] == "attention":
            y, values = attention_mixer(h, w, p + "mix.", mix, eps, first_values, first_values is None)
            if mix.get("v_mix") and first_values is None:
                first_values = values
        elif layer["type"] == "delta":
            y = delta_mixer(h, w, p + "mix.", mix, eps)
        else:
            raise ValueError(f"no mixer '{layer['type']}'")
        x = x + m * y
        if layer.get("mlp") is not None:
            x = x + m * feed_forward(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.")
        if layers_out is not None:
            layers_out.append(x.copy())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


# ------------------------------------------------------------------ random weights for tests
def tensor_shapes(config):
    D, V = int(config["width"]), int(config["vocab"])
    shapes = {"embed": (V, D), "pos": (int(config["max_positions"]), D), "final.norm": (D,), "head": (V, D)}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
        shapes[p + "norm1"] = (D,)
        x = p + "mix."
        if layer["type"] == "attention":
            shapes.update({x + "q": (H * d, D), x + "q.b": (H * d,), x + "k": (G * d, D), x + "k.b": (G * d,),
                           x + "v": (G * dv, D), x + "v.b": (G * dv,), x + "q.norm": (H * d,), x + "k.norm": (G * d,),
                           x + "temp": (H,), x + "g": (H, D), x + "o": (D, H * dv)})
            if m.get("v_mix"):
                shapes[x + "vmix"] = ()
        else:
            taps = int(m["conv"])
            shapes.update({x + "q": (G * d, D), x + "q.conv": (G * d, taps), x + "k": (G * d, D),
                           x + "k.conv": (G * d, taps), x + "v": (H * dv, D), x + "v.conv": (H * dv, taps),
                           x + "b": (H, D), x + "a": (H, D), x + "A_log": (H,), x + "dt_bias": (H,), x + "norm": (dv,),
                           x + "g": (H * dv, D), x + "o": (D, H * dv)})
        if layer.get("mlp") is not None:
            ff = int(layer["mlp"]["ff"])
            shapes.update({p + "norm2": (D,), p + "mlp.up": (ff, D), p + "mlp.down": (D, ff), p + "mlp.act": (2,)})
    return shapes


def random_weights(config, seed):
    """Weights that bfloat16 holds exactly (the tests write them to a bfloat16 file), sized so that every mechanism
    matters: temperatures away from one, a blend well inside (0, 1), decays between nothing and everything."""
    rng = np.random.default_rng(seed)
    D = int(config["width"])
    out = {}
    for name, shape in tensor_shapes(config).items():
        last = name.rsplit(".", 1)[-1]
        if name.endswith("norm") or last in ("norm1", "norm2"):
            a = rng.normal(1.0, 0.2, shape)
        elif last == "temp":
            a = rng.uniform(0.5, 2.0, shape)
        elif last == "vmix":
            a = rng.uniform(0.25, 0.6, shape)
        elif last == "conv":
            a = rng.normal(0.0, 0.6, shape)
        elif last == "A_log":
            a = rng.uniform(-2.0, 1.0, shape)
        elif last == "dt_bias":
            a = rng.uniform(-3.0, 1.0, shape)
        elif last == "act":
            a = rng.normal(0.0, 0.7, shape)
        elif last == "b" and len(shape) == 1:
            a = rng.normal(0.0, 0.3, shape)
        elif name in ("embed", "pos"):
            a = rng.normal(0.0, 1.0, shape)
        else:
            a = rng.normal(0.0, 1.0 / math.sqrt(shape[-1]), shape) * (3.0 if last in ("q", "k", "a", "b") else 1.0)
        # to what bfloat16 holds: eight bits of mantissa
        a = np.asarray(a, dtype=np.float32)
        bits = a.view(np.uint32).astype(np.uint64)
        bits = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
        out[name] = bits.astype(np.uint32).view(np.float32).astype(F).reshape(shape)
    return out
