"""Plain, slow implementation of the Bivizen decoder: the oracle of the tests.

It shares no code with ``air_b200``: whole sequences, no cache, no batch, numpy on the CPU, one function
per mechanism.  `dtype` is the precision of the arithmetic (float64 for the oracle, float32 to see what
32-bit rounding alone does).

The design, in this file's notation.  x is the stream [T, E].  A layer: h = rms(x) * w_norm1;
x += ls1 * mixer(h) + ls2 * ff(h) (one norm, both sub-layers read it).  Mixers:

  attention  q, k, v = h Wq^T + bq, ...; the first `rot` elements of each head of q and k are rotated, element
             i paired with i + rot/2, angle p * base^(-2i/rot); s = cap * tanh(scale * q.k / cap); causal softmax;
             in layers with v_mix other than the first of them v = (1 - lam) v + lam v_first, v_first the first
             such layer's v of the same token; head h's output times sigmoid(h Wg^T)[h]; Wo.
  delta      q, k (kv_heads x dim), v (heads x vdim): projection, causal depthwise convolution over time
             (taps columns, the last one the current token's), silu; q, k to unit length (q also times
             dim^-0.5); beta = sigmoid(h Wb^T); g = exp(-exp(A_log) * softplus(h Wa^T + dt_bias));
             S = g S; u = beta (v - S^T k); S += k u^T; o = S^T q; o = rms(o) * w * silu(h Wg^T); Wo.
  gla        q = h Wq^T dim^-0.5, k, v; alpha = sigmoid((h Wa1^T) Wa2^T + b)^(1/tau) per key channel;
             S = diag(alpha) S + k v^T; o = S^T q; o = rms(o) * w, times silu(h Wg^T); Wo.

Feed-forward: g = min(h Wgate^T, limit), u = clamp(h Wup^T, -limit, limit), y = g sigmoid(1.702 g) (u + 1); Wdown.
Output: rms(x) * w_final, then the output matrix.
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


def softplus(z):
    return np.logaddexp(0.0, z)


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


def linear(x, w, b=None):
    y = x @ w.T
    return y if b is None else y + b


# ----------------------------------------------------------------------------- mechanisms
def rotate(x, positions, rot, base):
    """x [T, heads, d]: the first `rot` elements of each head, (i, i + rot/2) a pair."""
    if not rot:
        return x
    half = rot // 2
    f = np.asarray(base, dtype=x.dtype) ** (-2.0 * np.arange(half, dtype=x.dtype) / rot)
    a = np.asarray(positions, dtype=x.dtype)[:, None] * f[None, :]
    c, s = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:rot]
    return np.concatenate([u * c - v * s, v * c + u * s, x[..., rot:]], axis=-1)


def capped_attention(q, k, v, scale, softcap):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]; causal, query head h reads kv head h // (H / G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]), dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap:
            s = softcap * np.tanh(s / softcap)
        s = np.where(np.tril(np.ones((T, T), dtype=bool)), s, -np.inf)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        out[:, h] = (p / p.sum(axis=1, keepdims=True)) @ v[:, g]
    return out


def attention_mixer(h, t, pre, m, positions, shared):
    """shared: what the layers of one pass hand to one another (the first v_mix layer's values)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = linear(h, t[pre + "q"], t[pre + "q.b"]).reshape(T, H, d)
    k = linear(h, t[pre + "k"], t[pre + "k.b"]).reshape(T, G, d)
    v = linear(h, t[pre + "v"], t[pre + "v.b"]).reshape(T, G, dv)
    rot = m.get("rot") or {}
    q = rotate(q, positions, rot.get("dims", 0), rot.get("base", 1.0))
    k = rotate(k, positions, rot.get("dims", 0), rot.get("base", 1.0))
    if m.get("v_mix"):
        if "v_first" in shared:
            lam = t[pre + "vmix"].astype(h.dtype)
            v = (1.0 - lam) * v + lam * shared["v_first"]
        else:
            shared["v_first"] = v
    o = capped_attention(q, k, v, m["scale"], m.get("softcap", 0.0))
    gate = sigmoid(linear(h, t[pre + "g"]))                     # [T, H]
    return linear((o * gate[:, :, None]).reshape(T, H * dv), t[pre + "o"])


def short_conv(x, w):
    """x [T, C], w [C, taps]: y[t] = sum_j w[:, j] x[t - (taps - 1 - j)], zeros before the start."""
    T, taps = x.shape[0], w.shape[1]
    y = np.zeros_like(x)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            y[back:] += x[:T - back] * w[:, j]
    return y


def unit(x, eps=1e-6):
    return x / np.sqrt(np.sum(x * x, axis=-1, keepdims=True) + eps)


def delta_rule(q, k, v, g, beta):
    """q, k [T, H, d], v [T, H, dv], g, beta [T, H] -> o [T, H, dv].  One state [d, dv] per head."""
    T, H, d = q.shape
    dv = v.shape[2]
    S = np.zeros((H, d, dv), dtype=q.dtype)
    o = np.zeros((T, H, dv), dtype=q.dtype)
    for t in range(T):
        for h in range(H):
            S[h] *= g[t, h]
            u = beta[t, h] * (v[t, h] - S[h].T @ k[t, h])
            S[h] += np.outer(k[t, h], u)
            o[t, h] = S[h].T @ q[t, h]
    return o


def delta_mixer(h, t, pre, m, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(linear(h, t[pre + "q"]), t[pre + "q.conv"])).reshape(T, G, d)
    k = silu(short_conv(linear(h, t[pre + "k"]), t[pre + "k.conv"])).reshape(T, G, d)
    v = silu(short_conv(linear(h, t[pre + "v"]), t[pre + "v.conv"])).reshape(T, H, dv)
    q = unit(q) * d ** -0.5
    k = unit(k)
    rep = H // G
    q, k = np.repeat(q, rep, axis=1), np.repeat(k, rep, axis=1)      # head h reads q/k head h // rep
    beta = sigmoid(linear(h, t[pre + "b"]))
    g = np.exp(-np.exp(t[pre + "A_log"].astype(h.dtype)) * softplus(linear(h, t[pre + "a"]) + t[pre + "dt_bias"]))
    o = delta_rule(q, k, v, g, beta)
    o = rms_norm(o, t[pre + "norm"], eps) * silu(linear(h, t[pre + "g"])).reshape(T, H, dv)
    return linear(o.reshape(T, H * dv), t[pre + "o"])


def gated_linear_attention(q, k, v, alpha):
    """q, k, alpha [T, H, d], v [T, H, dv] -> [T, H, dv]: S = diag(alpha) S + k v^T, o = S^T q."""
    T, H, d = q.shape
    dv = v.shape[2]
    S = np.zeros((H, d, dv), dtype=q.dtype)
    o = np.zeros((T, H, dv), dtype=q.dtype)
    for t in range(T):
        for h in range(H):
            S[h] = alpha[t, h][:, None] * S[h] + np.outer(k[t, h], v[t, h])
            o[t, h] = S[h].T @ q[t, h]
    return o


def gla_mixer(h, t, pre, m, eps):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (linear(h, t[pre + "q"]) * d ** -0.5).reshape(T, H, d)
    k = linear(h, t[pre + "k"]).reshape(T, H, d)
    v = linear(h, t[pre + "v"]).reshape(T, H, dv)
    z = linear(linear(h, t[pre + "a1"]), t[pre + "a2"], t[pre + "a2.b"])
    alpha = (sigmoid(z) ** (1.0 / m["tau"])).reshape(T, H, d)
    o = gated_linear_attention(q, k, v, alpha)
    o = rms_norm(o, t[pre + "norm"], eps).reshape(T, H * dv) * silu(linear(h, t[pre + "g"]))
    return linear(o, t[pre + "o"])


def clamped_glu(h, t, pre, f):
    lim = f["limit"]
    g = np.minimum(linear(h, t[pre + "gate"]), lim)
    u = np.clip(linear(h, t[pre + "up"]), -lim, lim)
    return linear(g * sigmoid(1.702 * g) * (u + 1.0), t[pre + "down"])


# ----------------------------------------------------------------------------- the model
def forward(config, tensors, tokens, dtype=np.float64, layers_out=None):
    """Logits [T, vocab] of a whole sequence; layers_out (a list) receives the stream after every layer."""
    t = {n: (a.astype(dtype) if a.dtype.kind == "f" else a) for n, a in tensors.items()}
    eps = config["norm"]["eps"]
    x = t["embed"][np.asarray(tokens)]
    positions = np.arange(len(tokens))
    shared = {}
    for i, layer in enumerate(config["layers"]):
        pre = f"l{i}."
        h = rms_norm(x, t[pre + "norm1"], eps)
        kind, m = layer["type"], layer["mixer"]
        if kind == "attention":
            a = attention_mixer(h, t, pre + "mix.", m, positions, shared)
        elif kind == "delta":
            a = delta_mixer(h, t, pre + "mix.", m, eps)
        elif kind == "gla":
            a = gla_mixer(h, t, pre + "mix.", m, eps)
        else:
            raise ValueError(f"mixer {kind}")
        delta = a * t[pre + "ls1"]
        if layer.get("mlp"):
            delta = delta + clamped_glu(h, t, pre + "mlp.", layer["mlp"]) * t[pre + "ls2"]
        x = x + delta
        if layers_out is not None:
            layers_out.append(x.copy())
    return linear(rms_norm(x, t["final.norm"], eps), t["head"])
