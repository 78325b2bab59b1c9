"""Plain, slow implementation of the Tomodra decoder: the oracle of the tests.

It shares no code with ``air_b200``: whole sequences, no cache, no batch, numpy on the CPU, one function
per mechanism.  `dtype` is the precision of the arithmetic (float64 for the oracle, float32 to see what
32-bit rounding alone does).

The design, in this file's notation.  x is the stream [T, E].  A layer normalises AFTER each sum:
x = rms(a x + mixer(x)) w1; x = rms(a x + ff(x)) w2, with one constant a for the whole model.  Mixers:

  latent_attention  q = x Wq^T, per head [dim plain | rot rotated]; (c | kr) = x Wdkv^T with c the first `rank`
                    columns, c = rms(c) w_c; kr (rot columns, one for all heads) and q's rotated part are turned by
                    the half-split rotation (element i paired with i + rot/2, angle p base^(-2i/rot)); per head
                    k = c Wuk^T, v = c Wuv^T; score = scale (q_plain . k + q_rot . kr); position i sees
                    i - window < j <= i; softmax; Wo.  A layer that borrows (kv_from j) has no Wdkv and takes c and
                    kr as layer j made them.
  attention         q, k, v = x Wq^T, ...; q and k normalised per head (rms over dim, one weight for all heads);
                    the first `rot` elements of each head of q and k turned in neighbouring pairs (2i, 2i + 1)
                    with frequencies bent by the YaRN rule and cos, sin scaled by 0.1 ln(factor) + 1; query head h
                    reads kv head h // (H / G); score = scale q.k; position i sees j <= i with i // size == j // size;
                    softmax whose denominator also holds exp(sink_h); Wo.

Feed-forward: s = sigmoid(x Wr^T); the `top` experts with the largest s; y = sum_e expert_e(s_e x) (the weight
goes in, not out) + sigmoid(x Wsg^T) shared(x); expert(u) = (silu(u Wg^T) * (u Wu^T)) Wd^T.
Output: rms(x) w_final, then the output matrix.
"""
from __future__ import annotations

import json
import math
import struct

import numpy as np


def read_safetensors(path):
    with open(path, "rb") as f:
        raw = f.read()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n].decode("utf-8"))
    data = memoryview(raw)[8 + n:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        dt = info["dtype"]
        if dt == "BF16":
            a = (np.frombuffer(data[lo:hi], dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif dt == "F32":
            a = np.frombuffer(data[lo:hi], dtype="<f4")
        elif dt == "I32":
            a = np.frombuffer(data[lo:hi], dtype="<i4")
        else:
            raise ValueError(f"dtype {dt} of {name}")
        out[name] = a.reshape(info["shape"]).copy()
    return out


def read_model(folder):
    with open(f"{folder}/config.json") as f:
        config = json.load(f)
    return config, read_safetensors(f"{folder}/model.safetensors")


# ----------------------------------------------------------------------------- small functions
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


def plain_frequencies(dims, base):
    i = np.arange(dims // 2, dtype=np.float64)
    return base ** (-2.0 * i / dims)


def yarn_frequencies(dims, base, scaling):
    """(frequencies, what cos and sin are multiplied by) of the bent rotation."""
    f = plain_frequencies(dims, base)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turns_to_dim(t):
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turns_to_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turns_to_dim(float(scaling["slow"]))), dims - 1)
    i = np.arange(dims // 2, dtype=np.float64)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half_split(x, positions, f, dims):
    """x [T, ..., d]: element i < dims/2 is paired with element i + dims/2; the rest passes."""
    T = x.shape[0]
    a = (positions.astype(np.float64)[:, None] * f[None, :]).reshape((T,) + (1,) * (x.ndim - 2) + (dims // 2,))
    cos, sin = np.cos(a), np.sin(a)
    out = x.copy()
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    out[..., :dims // 2] = u * cos - v * sin
    out[..., dims // 2:dims] = v * cos + u * sin
    return out


def rotate_neighbours(x, positions, f, dims, magnitude=1.0):
    """x [T, ..., d]: element 2i is paired with element 2i + 1, i < dims/2; the rest passes."""
    T = x.shape[0]
    a = (positions.astype(np.float64)[:, None] * f[None, :]).reshape((T,) + (1,) * (x.ndim - 2) + (dims // 2,))
    cos, sin = np.cos(a) * magnitude, np.sin(a) * magnitude
    out = x.copy()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def window_mask(T, size):
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return (j <= i) & (i - j < size)


def chunk_mask(T, size):
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def masked_softmax(scores, mask, sink=None):
    """scores [H, T, T]; sink [H] or None: one more term exp(sink_h) in the denominator, with no value."""
    s = np.where(mask[None], scores, -np.inf)
    m = s.max(axis=-1, keepdims=True)
    if sink is not None:
        m = np.maximum(m, sink[:, None, None])
    e = np.exp(s - m)
    den = e.sum(axis=-1, keepdims=True)
    if sink is not None:
        den = den + np.exp(sink[:, None, None] - m)
    return e / den


# ----------------------------------------------------------------------------- mixers
def latent_kv(x, w, p, m, eps, positions):
    """What a latent layer keeps per token: c [T, rank] and the rotated shared key part [T, rot]."""
    rank, rot = m["kv_rank"], m["rot_dim"]
    ckr = x @ w[p + "dkv"].T
    c = rms_norm(ckr[:, :rank], w[p + "dkv.norm"], eps)
    f = plain_frequencies(rot, float(m["rot"]["base"]))
    return c, rotate_half_split(ckr[:, rank:], positions, f, rot)


def latent_attention(x, w, p, m, eps, positions, kept):
    H, d, rot, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    T = x.shape[0]
    c, kr = kept
    q = (x @ w[p + "q"].T).reshape(T, H, d + rot)
    f = plain_frequencies(rot, float(m["rot"]["base"]))
    q_plain, q_rot = q[..., :d], rotate_half_split(q[..., d:], positions, f, rot)
    k = (c @ w[p + "uk"].T).reshape(T, H, d)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    scores = (np.einsum("thd,shd->hts", q_plain, k) + np.einsum("thr,sr->hts", q_rot, kr)) * float(m["scale"])
    a = masked_softmax(scores, window_mask(T, int(m["mask"]["size"])))
    return np.einsum("hts,shd->thd", a, v).reshape(T, H * dv) @ w[p + "o"].T


def sink_attention(x, w, p, m, eps, positions):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = x.shape[0]
    q = rms_norm((x @ w[p + "q"].T).reshape(T, H, d), w[p + "q.norm"], eps)
    k = rms_norm((x @ w[p + "k"].T).reshape(T, G, d), w[p + "k.norm"], eps)
    v = (x @ w[p + "v"].T).reshape(T, G, dv)
    dims = int(m["rot"]["dims"])
    f, magnitude = yarn_frequencies(dims, float(m["rot"]["base"]), m["rot"].get("scaling"))
    q = rotate_neighbours(q, positions, f, dims, magnitude)
    k = rotate_neighbours(k, positions, f, dims, magnitude)
    k, v = np.repeat(k, H // G, axis=1), np.repeat(v, H // G, axis=1)
    scores = np.einsum("thd,shd->hts", q, k) * float(m["scale"])
    a = masked_softmax(scores, chunk_mask(T, int(m["mask"]["size"])), sink=w[p + "sink"].astype(x.dtype))
    return np.einsum("hts,shd->thd", a, v).reshape(T, H * dv) @ w[p + "o"].T


# ----------------------------------------------------------------------------- feed-forward
def expert(u, w, p):
    return (silu(u @ w[p + "gate"].T) * (u @ w[p + "up"].T)) @ w[p + "down"].T


def mixture(x, w, p, f, margins=None):
    """margins (a list) receives, per token, by how much the last chosen score beats the best one left out."""
    n, top = int(f["router"]["experts"]), int(f["router"]["top"])
    s = sigmoid(x @ w[p + "router"].T)                            # [T, n]
    chosen = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    if margins is not None:
        ranked = -np.sort(-s, axis=-1)
        margins.append(ranked[:, top - 1] - ranked[:, top] if top < n else np.full(len(x), np.inf))
    y = np.zeros_like(x)
    for e in range(n):
        for t in np.nonzero((chosen == e).any(axis=-1))[0]:
            y[t] += expert(s[t, e] * x[t], w, f"{p}e{e}.")
    if f.get("shared"):
        y += sigmoid(x @ w[p + "shared.sg"].T) * expert(x, w, p + "shared.")
    return y


# ----------------------------------------------------------------------------- the model
def forward(config, weights, tokens, dtype=np.float64, layers_out=None, margins=None):
    """Logits [T, vocab] of one sequence; layers_out (a list) receives the stream after every layer, margins (a list)
    the routers' margins per token, one array per layer with a feed-forward."""
    w = {k: (v.astype(dtype) if v.dtype.kind == "f" else v) for k, v in weights.items()}
    eps, alpha = float(config["norm"]["eps"]), float(config["postln_alpha"])
    tokens = np.asarray(tokens)
    positions = np.arange(len(tokens))
    x = w["embed"][tokens]
    kept = {}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        if layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = latent_kv(x, w, p, m, eps, positions)
                src = i
            y = latent_attention(x, w, p, m, eps, positions, kept[src])
        elif layer["type"] == "attention":
            y = sink_attention(x, w, p, m, eps, positions)
        else:
            raise ValueError(layer["type"])
        x = rms_norm(alpha * x + y, w[f"l{i}.norm1"], eps)
        if layer.get("mlp") is not None:
            x = rms_norm(alpha * x + mixture(x, w, f"l{i}.mlp.", layer["mlp"], margins), w[f"l{i}.norm2"], eps)
        elif f"l{i}.norm2" in w:
            x = rms_norm(alpha * x, w[f"l{i}.norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
