"""Set-up of the Tomodra tests: small configurations that differ in every size and option, model folders with weights
drawn so that a fault shows, and the comparison with the plain implementation."""
import functools
import tempfile

import numpy as np

from bivizen_util import bf16


def latent(heads, dim, rot, vdim, rank, window, scale, base=10000.0, kv_from=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot, vdim=vdim, kv_rank=rank, scale=scale, mask=dict(size=window),
             rot=dict(dims=rot, base=base))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="latent_attention", mixer=m)


def attention(heads, kv_heads, dim, vdim, chunk, scale, rot, base=10000.0, scaling=None):
    r = dict(dims=rot, base=base)
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return dict(type="attention", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale,
                                             mask=dict(size=chunk), rot=r))


def with_mlp(layer, experts=None, top=None, ff=None, shared=None):
    if experts is None:
        return dict(layer, mlp=None)
    f = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))
    if shared:
        f["shared"] = dict(ff=shared)
    return dict(layer, mlp=f)


def config(vocab, width, eps, alpha, layers):
    return dict(architecture="Tomodra", vocab=vocab, width=width, norm=dict(eps=eps), postln_alpha=alpha, layers=layers)


# A: two choices of five experts; a layer that reads the latent of layer 0 through a WIDER window than layer 0's own
#    (the pages must live as long as the wider one needs them); part of a head rotated, stretched frequencies; chunks
#    of 40 (no multiple of a page); a layer without feed-forward; a layer without shared expert.
# B: sizes that other models make equal differ and the other way round: one head, kv_heads == heads, dim != vdim, the
#    whole head rotated without stretching, every expert chosen (top == experts), a window wider than any prompt, a
#    chunk of one page, a window of 1 (a token sees itself only).
# C: heads of 64 and 128 with values of the same size, chunks of 64 and 128, a latent of 64 + 32, pages of 64.
CONFIGS = {
    "A": config(211, 64, 1e-5, 2.0, [
        with_mlp(latent(4, 24, 8, 20, 40, 48, 0.2), 5, 2, 48, 40),
        with_mlp(attention(4, 2, 32, 16, 40, 0.17, 16, 5000.0, (4.0, 64, 16.0, 2.0)), 5, 2, 48, 40),
        with_mlp(latent(2, 16, 8, 24, 40, 70, 0.25, kv_from=0)),
        with_mlp(latent(3, 8, 4, 8, 24, 17, 0.3, base=300.0), 3, 1, 32),
        with_mlp(attention(6, 3, 16, 16, 23, 0.3, 8, 1e5, (16.0, 32, 8.0, 1.0)), 5, 2, 48, 40)]),
    "B": config(333, 96, 1e-6, 5.0, [
        with_mlp(attention(1, 1, 48, 20, 16, 0.15, 48, 500.0), 3, 3, 40, 24),
        with_mlp(latent(1, 32, 16, 40, 56, 4096, 0.18, base=1e6), 4, 1, 56, 16),
        with_mlp(latent(5, 8, 2, 8, 16, 1, 0.4, base=50.0), 4, 1, 56, 16),
        with_mlp(attention(3, 3, 24, 40, 1000, 0.2, 12, 1e4, (2.0, 16, 4.0, 1.0)), 2, 1, 64, 64)]),
    "C": config(190, 128, 1e-6, 3.0, [
        with_mlp(attention(4, 2, 64, 64, 64, 0.125, 32, 10000.0, (8.0, 128, 32.0, 1.0)), 6, 2, 64, 128),
        with_mlp(latent(4, 64, 32, 64, 64, 100, 0.1), 6, 2, 64, 128),
        with_mlp(attention(2, 1, 128, 128, 128, 0.09, 128, 1e6), 6, 1, 64, 128),
        with_mlp(latent(2, 32, 32, 32, 64, 64, 0.12, kv_from=1), 6, 2, 64)]),
}
SEEDS = {"A": 21, "B": 22, "C": 23}


def random_config(seed):
    """A configuration drawn at random: 2 to 6 layers in any order, every size and constant from a list that includes
    1, equal and unequal sizes and sizes that are no multiples of 8 or 16; layers that read an earlier layer's latent
    through a window of their own; layers without feed-forward or without shared expert."""
    rng = np.random.default_rng(seed)
    width = int(rng.choice([40, 64, 72, 96, 128, 160, 200]))
    layers, owners = [], []
    for i in range(int(rng.integers(2, 7))):
        if rng.random() < 0.6:
            if owners and rng.random() < 0.4:
                j = int(rng.choice(owners))
                o = layers[j]["mixer"]
                layer = latent(int(rng.choice([1, 2, 3, 5, 8])), int(rng.choice([8, 12, 16, 24, 40])), o["rot_dim"],
                               int(rng.choice([8, 12, 20, 32, 48])), o["kv_rank"], int(rng.choice([1, 7, 33, 64, 100, 5000])),
                               float(rng.choice([0.1, 0.2, 0.3])), base=o["rot"]["base"], kv_from=j)
            else:
                layer = latent(int(rng.choice([1, 2, 4, 6, 16, 20])), int(rng.choice([8, 16, 24, 32, 64])),
                               int(rng.choice([2, 4, 8, 16, 32])), int(rng.choice([8, 16, 24, 40, 64])),
                               int(rng.choice([8, 24, 40, 56, 96, 112])), int(rng.choice([1, 5, 16, 40, 64, 90, 4096])),
                               float(rng.choice([0.1, 0.2, 0.3])), base=float(rng.choice([50.0, 1e4, 5e5])))
                owners.append(i)
        else:
            kv, rep = int(rng.choice([1, 2, 3])), int(rng.choice([1, 2, 4, 5]))
            dim = int(rng.choice([8, 16, 24, 32, 48, 64, 128]))
            rot = int(rng.choice([r for r in (0, 2, 4, 8, 16, 24, 32, 64, dim) if r <= dim and r % 2 == 0]))
            scaling = None if rng.random() < 0.3 or rot == 0 else \
                (float(rng.choice([2.0, 4.0, 8.0, 32.0])), int(rng.choice([16, 64, 1024])), float(rng.choice([4.0, 16.0, 32.0])),
                 float(rng.choice([1.0, 2.0])))
            layer = attention(kv * rep, kv, dim, int(rng.choice([8, 16, 24, 40, 64, 128, dim])),
                              int(rng.choice([1, 6, 16, 33, 64, 100, 5000])), float(rng.choice([0.1, 0.15, 0.25])), rot,
                              float(rng.choice([100.0, 1e4, 1e6])), scaling)
        if rng.random() < 0.15:
            layers.append(with_mlp(layer))
        else:
            n = int(rng.integers(1, 9))
            layers.append(with_mlp(layer, n, int(rng.integers(1, n + 1)), int(rng.choice([16, 24, 40, 64, 100])),
                                   None if rng.random() < 0.25 else int(rng.choice([16, 40, 64, 96]))))
    return config(int(rng.integers(50, 700)), width, float(rng.choice([1e-6, 1e-5, 1e-4])),
                  float(rng.choice([1.0, 2.0, 3.0, 6.0])), layers)


def draw_tensors(cfg, seed):
    """name -> float32 array.  The scales are chosen so that every mechanism matters: attention scores have a standard
    deviation of about 2.5 (a key that is lost or added, or a rotation that is off, moves the logits far beyond
    bfloat16's rounding), sinks are of the order of the scores, and a sub-layer's output is of the order of the stream
    it is added to.

    A router is a discontinuity: with random router weights one token in a hundred has two experts so close that
    bfloat16's rounding picks the other one, and the logits then differ by a whole expert.  So the routers here decide by
    three channels of the stream that only the embedding and the norms touch (the output matrices leave them alone):
    a token carries a sign pattern with magnitudes 1, 0.55, 0.3 there, an expert's router row the pattern of its
    index, and all sums of +-1, +-0.55, +-0.3 are apart.  Which experts a token takes is then a matter of the token,
    clear of rounding; their weights still depend on everything, through the norms and the rest of the router row."""
    rng = np.random.default_rng(seed)
    e, alpha = cfg["width"], cfg["postln_alpha"]
    t = {}

    def mat(out, inp, gain=1.0):
        return rng.normal(0.0, gain / np.sqrt(inp), size=(out, inp))

    def norm_weight(n):
        return 1.0 + rng.normal(0.0, 0.1, size=n)

    t["embed"] = rng.normal(0.0, 1.0, size=(cfg["vocab"], e))
    tokens = np.arange(cfg["vocab"])
    for c in range(3):
        t["embed"][:, c] = np.where((tokens >> c) & 1, 1.0, -1.0) * ROUTE_CHANNELS[c] * 1.5
    t["head"] = mat(cfg["vocab"], e, 2.0)
    t["final.norm"] = norm_weight(e)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        t[p + "norm1"] = norm_weight(e)
        t[p + "norm1"][:3] = 1.4
        if layer["type"] == "attention":
            G = m["kv_heads"]
            t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"] = mat(H * d, e), mat(G * d, e), mat(G * dv, e, 1.5 * alpha)
            gain = (2.5 / (m["scale"] * d ** 0.5)) ** 0.5             # normalised q.k * scale ~ N(0, 2.5^2)
            t[p + "mix.q.norm"], t[p + "mix.k.norm"] = gain * norm_weight(d), gain * norm_weight(d)
            t[p + "mix.sink"] = rng.normal(1.0, 2.0, size=H)
        else:
            rot, R = m["rot_dim"], m["kv_rank"]
            gain = (2.5 / m["scale"]) ** 0.5 / (d + rot) ** 0.25
            t[p + "mix.q"] = mat(H * (d + rot), e, gain)
            if m.get("kv_from") is None:
                t[p + "mix.dkv"] = mat(R + rot, e, gain)
                t[p + "mix.dkv.norm"] = norm_weight(R)
            t[p + "mix.uk"], t[p + "mix.uv"] = mat(H * d, R, gain), mat(H * dv, R, 1.5 * alpha)
        t[p + "mix.o"] = mat(e, H * dv, 1.0)
        t[p + "mix.o"][:3] = 0.0
        f = layer.get("mlp")
        if f:
            t[p + "norm2"] = norm_weight(e)
            t[p + "norm2"][:3] = 1.4
            t[p + "mlp.router"] = mat(f["router"]["experts"], e, 0.02)
            for x in range(f["router"]["experts"]):
                t[p + "mlp.router"][x, :3] = [(1.0 if (x >> c) & 1 else -1.0) * 1.2 for c in range(3)]
                t[f"{p}mlp.e{x}.gate"], t[f"{p}mlp.e{x}.up"] = mat(f["expert"]["ff"], e, 2.0), mat(f["expert"]["ff"], e, 2.0)
                t[f"{p}mlp.e{x}.down"] = mat(e, f["expert"]["ff"], 0.6 * alpha)
                t[f"{p}mlp.e{x}.down"][:3] = 0.0
            if f.get("shared"):
                s = f["shared"]["ff"]
                t[p + "mlp.shared.gate"], t[p + "mlp.shared.up"] = mat(s, e, 1.5), mat(s, e, 1.5)
                t[p + "mlp.shared.down"] = mat(e, s, 0.6 * alpha)
                t[p + "mlp.shared.down"][:3] = 0.0
                t[p + "mlp.shared.sg"] = mat(1, e, 2.0)
    return {n: bf16(a) for n, a in t.items()}


ROUTE_CHANNELS = (1.0, 0.55, 0.3)
_tmp = []


@functools.lru_cache(maxsize=None)
def model_folder(name):
    """config.json and model.safetensors (bfloat16) of a test configuration, in a temporary place."""
    import torch
    from air_b200.weights.loader import write_model_folder
    d = tempfile.TemporaryDirectory(prefix=f"air_b200_tomodra_{name}_")
    _tmp.append(d)
    if name not in CONFIGS:      # "random<seed>": drawn at random
        seed = int(name[len("random"):])
        CONFIGS[name], SEEDS[name] = random_config(seed), seed
    cfg = CONFIGS[name]
    tensors = {n: torch.from_numpy(np.ascontiguousarray(a)).reshape(a.shape).to(torch.bfloat16)
               for n, a in draw_tensors(cfg, SEEDS[name]).items()}
    write_model_folder(d.name, cfg, tensors)
    return d.name


@functools.lru_cache(maxsize=None)
def plain_model(name):
    from plain import tomodra_plain as plain
    return plain.read_model(model_folder(name))


_logits = {}


def plain_run(name, tokens):
    """(logits [T, vocab], the smallest margin by which a router chose)."""
    from plain import tomodra_plain as plain
    key = (name, tuple(tokens))
    if key not in _logits:
        cfg, tensors = plain_model(name)
        margins = []
        logits = plain.forward(cfg, tensors, list(tokens), margins=margins).astype(np.float64)
        _logits[key] = (logits, float(np.min(margins)) if margins else np.inf)
    return _logits[key]


def plain_logits(name, tokens):
    return plain_run(name, tokens)[0]


def tokens_for(name, n, seed):
    return np.random.default_rng(7000 + seed).integers(0, CONFIGS[name]["vocab"], size=n).tolist()


def plain_greedy(name, prompt, n):
    out, toks = [], list(prompt)
    for _ in range(n):
        nxt = int(plain_logits(name, toks)[-1].argmax())
        out.append(nxt)
        toks.append(nxt)
    return out


# float32: sums in another order than the 64-bit oracle.  bfloat16: activations rounded to 8 bits at the inputs of the
# products and in the cache, through five layers of sharp attention (a third of the weight on one key in the mean)
# and experts whose input is scaled: measured over these models, a row's mean difference is 0.4 to 1 % of the largest
# |logit| in the median and up to 4.3 % at single rows, where the largest difference reaches 18 %.  A request's rows
# must all be within the row limits, and their median within the tighter one.  The routers choose with margins of
# 0.02 and more (draw_tensors); check() makes sure of it, since a choice that rounding can tip voids the comparison.
FP32_TOL = 1e-4
BF16_MAX_TOL = 0.3
BF16_MEAN_TOL = 7e-2
BF16_MEDIAN_TOL = 1.8e-2


def check(got, name, streams, dtype):
    """got: {(request, position): logits}; every request of `streams` must have rows, and the rows must agree."""
    for rid, toks in streams.items():
        ref, margin = plain_run(name, toks)
        assert margin > (1e-4 if dtype == "float32" else 0.01), (rid, margin)
        scale = max(1.0, float(np.abs(ref).max()))
        rows = sorted(p for (r, p) in got if r == rid)
        assert rows, f"no logits for request {rid}"
        means = []
        for p in rows:
            out = got[(rid, p)]
            assert np.isfinite(out).all()
            diff = np.abs(out - ref[p])
            if dtype == "float32":
                assert diff.max() <= FP32_TOL * scale, (rid, p, float(diff.max()), scale)
            else:
                assert diff.max() <= BF16_MAX_TOL * scale, (rid, p, float(diff.max()), scale)
                assert diff.mean() <= BF16_MEAN_TOL * scale, (rid, p, float(diff.mean()), scale)
                means.append(diff.mean() / scale)
        if means and len(means) >= 8:
            assert np.median(means) <= BF16_MEDIAN_TOL, (rid, float(np.median(means)))
