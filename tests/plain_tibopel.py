"""A plain, slow statement of the Tibopel design in NumPy float64, one function per mechanism.

It shares no code with the package: the tests hold the package's kernels, cache and scheduler to
these functions.  A model is a dict ``config`` (the JSON of config.json) and a dict ``w`` of arrays by
tensor name.  Everything works on one whole sequence (positions 0..T-1); what a cache would hold is
simply recomputed.

Notation: x the residual stream [T, D]; h a sublayer's input (a normed stream); H query heads,
G key/value heads; d the query/key size of a head, d_v its value size; r the latent size, d_r the
rotated part of a latent-attention head.
"""
import math

import numpy as np

F = np.float64


# ------------------------------------------------------------------ elementwise
def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * weight


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def relu_squared(z):
    return np.square(np.maximum(z, 0.0))


# ------------------------------------------------------------------ rotation
def rotary_frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims) for i < dims/2.  ``scaling`` = {factor, low, high, original} stretches
    the long wavelengths: with l = 2 pi / f, f stays where l < original/high, becomes f / factor
    where l > original/low, and in between is the mix (1 - s) f / factor + s f with
    s = (original / l - low) / (high - low)."""
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F)
    if not scaling:
        return f
    factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = f.copy()
    for i, fi in enumerate(f):
        l = 2.0 * math.pi / fi
        if l < original / high:
            continue
        if l > original / low:
            out[i] = fi / factor
        else:
            s = (original / l - low) / (high - low)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out


def rotate_pairs(v, positions, freqs):
    """v [T, ..., n]: entry 2i turns with entry 2i+1 by the angle position * freqs[i] for the first
    2 * len(freqs) entries of the last axis; the rest pass."""
    out = np.array(v, dtype=F, copy=True)
    n = 2 * len(freqs)
    if n == 0:
        return out
    ang = np.asarray(positions, dtype=F)[:, None] * freqs[None, :]              # [T, n/2]
    shape = (v.shape[0],) + (1,) * (v.ndim - 2) + (len(freqs),)
    cs, sn = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    a, b = v[..., 0:n:2], v[..., 1:n:2]
    out[..., 0:n:2] = a * cs - b * sn
    out[..., 1:n:2] = b * cs + a * sn
    return out


# ------------------------------------------------------------------ softmax attention of one head
def masked_attention(q, k, v, scale, first_of, sink=None):
    """q [T, d], k [T, d], v [T, d_v]; position i attends to first_of(i) .. i.  With ``sink`` (a number)
    the denominator counts exp(sink) once more, with no value behind it."""
    T = q.shape[0]
    out = np.zeros((T, v.shape[1]), dtype=F)
    for i in range(T):
        lo = first_of(i)
        s = (k[lo: i + 1] @ q[i]) * scale
        top = float(s.max()) if sink is None else max(float(s.max()), float(sink))
        e = np.exp(s - top)
        den = e.sum() + (0.0 if sink is None else math.exp(float(sink) - top))
        out[i] = (e @ v[lo: i + 1]) / den
    return out


# ------------------------------------------------------------------ mixer: chunked grouped-query attention
def chunked_attention(h, w, p, m):
    """Projections with biases, rotation of the first rot.dims entries of every query and key head,
    attention within chunks of mask.size positions counted from position 0, a sigmoid gate per head
    from the mixer's own input, output projection with bias."""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    size = int((m.get("mask") or {}).get("size", 0))               # no mask: every earlier position
    rot = m["rot"]
    freqs = rotary_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
    pos = np.arange(T)
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
    q, k = rotate_pairs(q, pos, freqs), rotate_pairs(k, pos, freqs)
    gate = sigmoid(h @ w[p + "g"].T)                                             # [T, H]
    heads = np.zeros((T, H, dv), dtype=F)
    for a in range(H):
        g = a // (H // G)
        heads[:, a] = masked_attention(q[:, a], k[:, g], v[:, g], float(m["scale"]), lambda i: i - i % size if size else 0)
        heads[:, a] *= gate[:, a: a + 1]
    return heads.reshape(T, H * dv) @ w[p + "o"].T + w[p + "o.b"]


# ------------------------------------------------------------------ mixer: latent attention with a sink
def latent_attention(h, w, p, m, eps):
    """Queries through a normed latent; keys and values from one normed latent per position plus one
    rotated key part that all heads share; causal; every head's softmax has a learned sink."""
    T = h.shape[0]
    H, d, dr, dv, r = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    freqs = rotary_frequencies(dr, float(m["rot"]["base"]), m["rot"].get("scaling"))
    pos = np.arange(T)
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).reshape(T, H, d + dr)
    q_plain, q_rot = q[..., :d], rotate_pairs(q[..., d:], pos, freqs)
    down = h @ w[p + "dkv"].T
    c = rms_norm(down[:, :r], w[p + "dkv.norm"], eps)
    k_rot = rotate_pairs(down[:, r:], pos, freqs)                                # [T, d_r], one for all heads
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, d)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    heads = np.zeros((T, H, dv), dtype=F)
    for a in range(H):
        qa = np.concatenate([q_plain[:, a], q_rot[:, a]], axis=-1)
        ka = np.concatenate([k_plain[:, a], k_rot], axis=-1)
        heads[:, a] = masked_attention(qa, ka, v[:, a], float(m["scale"]), lambda i: 0, sink=float(w[p + "sink"][a]))
    return heads.reshape(T, H * dv) @ w[p + "o"].T


# ------------------------------------------------------------------ feed-forward: routed experts
def route(h, w, p, f):
    """(chosen [T, top], weights [T, top]) over experts + identity outputs: softmax scores, the choice
    by score + correction, the weights the chosen scores over their sum."""
    top = int(f["router"]["top"])
    z = h @ w[p + "router"].T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z)
    s /= s.sum(axis=-1, keepdims=True)
    choice = s + w[p + "correction"]
    chosen = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    weights = np.take_along_axis(s, chosen, axis=-1)
    weights = weights / (weights.sum(axis=-1, keepdims=True) + 1e-20)
    return chosen, weights


def routed_experts(h, w, p, f):
    """Experts down(relu(up h)^2); the last router outputs stand for identity experts (their result
    is h); a shared expert of the same form runs for every token behind a sigmoid gate."""
    T = h.shape[0]
    E = int(f["router"]["experts"])
    chosen, weights = route(h, w, p, f)
    out = np.zeros_like(h)
    for t in range(T):
        for e, g in zip(chosen[t], weights[t]):
            if e >= E:
                out[t] += g * h[t]
            else:
                out[t] += g * (w[f"{p}e{e}.down"] @ relu_squared(w[f"{p}e{e}.up"] @ h[t]))
    if f.get("shared"):
        shared = relu_squared(h @ w[p + "shared.up"].T) @ w[p + "shared.down"].T
        out += sigmoid(h @ w[p + "shared.sg"].T) * shared
    return out


# ------------------------------------------------------------------ the model
def layer_forward(x, w, config, i):
    """x + mixer(norm1 x) + ff(norm2 x), both sublayers reading the same x."""
    layer = config["layers"][i]
    j = i
    while config["layers"][j].get("weights_of") is not None:                    # whose tensors: the owner's
        j = int(config["layers"][j]["weights_of"])
    p = f"l{j}."
    eps = float(config["norm"]["eps"])
    h1 = rms_norm(x, w[p + "norm1"], eps)
    if layer["type"] == "attention":
        y = chunked_attention(h1, w, p + "mix.", layer["mixer"])
    else:
        y = latent_attention(h1, w, p + "mix.", layer["mixer"], eps)
    if layer.get("mlp") is not None:
        y = y + routed_experts(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.", layer["mlp"])
    return x + y


def forward(config, w, tokens, streams=None):
    """Logits [T, vocab] of one whole sequence; ``streams`` (a list) receives the residual stream after
    every layer run."""
    x = w["embed"][np.asarray(tokens, dtype=np.int64)].astype(F)
    for i in range(len(config["layers"])):
        x = layer_forward(x, w, config, i)
        if streams is not None:
            streams.append(x.copy())
    h = rms_norm(x, w["final.norm"], float(config["norm"]["eps"]))
    logits = h @ w["head"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = float(cap) * np.tanh(logits / float(cap))
    return logits


# ------------------------------------------------------------------ files
def read_model(model_dir):
    """(config, weights as float64 arrays) of a folder with config.json and model.safetensors."""
    import json
    import os
    import struct
    with open(os.path.join(model_dir, "config.json")) as f:
        config = json.load(f)
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    w = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw = data[lo:hi]
        if info["dtype"] == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif info["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4")
        elif info["dtype"] == "I32":
            a = np.frombuffer(raw, dtype="<i4")
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
        w[name] = a.reshape(info["shape"]).astype(F)
    return config, w


# ------------------------------------------------------------------ random models for the tests
def tensor_shapes(config):
    """name -> shape of every tensor a model of this configuration has (layers that use another layer's
    tensors have none)."""
    D, V = int(config["width"]), int(config["vocab"])
    out = {"embed": (V, D), "final.norm": (D,), "head": (V, D)}
    for i, layer in enumerate(config["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = (D,)
        x = p + "mix."
        if layer["type"] == "attention":
            H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
            out.update({x + "q": (H * d, D), x + "q.b": (H * d,), x + "k": (G * d, D), x + "k.b": (G * d,),
                        x + "v": (G * dv, D), x + "v.b": (G * dv,), x + "g": (H, D), x + "o": (D, H * dv), x + "o.b": (D,)})
        else:
            H, d, dr, dv = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"])
            r, rq = int(m["kv_rank"]), int(m["q_rank"])
            out.update({x + "dq": (rq, D), x + "dq.norm": (rq,), x + "uq": (H * (d + dr), rq), x + "dkv": (r + dr, D),
                        x + "dkv.norm": (r,), x + "uk": (H * d, r), x + "uv": (H * dv, r), x + "sink": (H,),
                        x + "o": (D, H * dv)})
        f = layer.get("mlp")
        if f is None:
            continue
        out[p + "norm2"] = (D,)
        y = p + "mlp."
        E, n_id, ff = int(f["router"]["experts"]), int(f["router"].get("identity") or 0), int(f["expert"]["ff"])
        out[y + "router"], out[y + "correction"] = (E + n_id, D), (E + n_id,)
        for e in range(E):
            out[f"{y}e{e}.up"], out[f"{y}e{e}.down"] = (ff, D), (D, ff)
        if f.get("shared"):
            s = int(f["shared"]["ff"])
            out.update({y + "shared.up": (s, D), y + "shared.down": (D, s), y + "shared.sg": (1, D)})
    return out


def to_bfloat16(a):
    """The nearest values that bfloat16 holds (eight bits of mantissa, ties to even), as float64."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    bits = a.view(np.uint32).astype(np.uint64)
    bits = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
    return bits.astype(np.uint32).view(np.float32).astype(F).reshape(a.shape)


def random_weights(config, seed, sharp=3.0):
    """Weights that bfloat16 holds exactly (the tests write them to a bfloat16 file), sized so that every
    mechanism matters: sinks that take a visible share, corrections that change choices, gates away from
    one half, queries and keys ``sharp`` times larger than the rest for peaked softmaxes."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("norm", "norm1", "norm2"):
            a = rng.normal(1.0, 0.2, shape)
        elif last == "sink":
            a = rng.normal(0.5, 1.5, shape)
        elif last == "correction":
            a = rng.normal(0.0, 0.08, shape)
        elif last == "b":
            a = rng.normal(0.0, 0.3, shape)
        elif name == "embed":
            a = rng.normal(0.0, 1.0, shape)
        else:
            big = sharp if last in ("q", "k", "uq", "uk", "dkv", "g", "sg", "router") else 1.0
            a = rng.normal(0.0, 1.0 / math.sqrt(shape[-1]), shape) * big
        out[name] = to_bfloat16(a)
    return out
