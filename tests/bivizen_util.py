"""Set-up of the Bivizen tests: small configurations that differ in every size and option, model folders with
weights drawn so that a fault shows, and the comparison with the plain implementation."""
import functools
import tempfile

import numpy as np


def attention(heads, kv_heads, dim, vdim, scale, softcap=0.0, rot=None, v_mix=False):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, v_mix=v_mix)
    if softcap:
        m["softcap"] = softcap
    if rot:
        m["rot"] = dict(dims=rot[0], base=rot[1])
    return dict(type="attention", mixer=m)


def delta(heads, kv_heads, dim, vdim, conv):
    return dict(type="delta", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv))


def gla(heads, dim, vdim, tau, rank):
    return dict(type="gla", mixer=dict(heads=heads, dim=dim, vdim=vdim, tau=tau, rank=rank))


def with_mlp(layer, ff, limit):
    return dict(layer, mlp=None if ff is None else dict(kind="dense", ff=ff, limit=limit))


def config(vocab, width, eps, layers):
    return dict(architecture="Bivizen", vocab=vocab, width=width, norm=dict(eps=eps), layers=layers)


# P: a recurrent layer first, values mixed between the second and the fourth layer but not the fifth, grouped heads,
#    half of a head rotated, a layer without feed-forward, key sizes that are no powers of two.
# Q: other sizes everywhere; one head, one kv head, an odd value size, two taps, a whole head rotated, no value mixing.
# R: heads of 64 and 128 with values of the same size (what the tensor-core attention kernels take), four taps.
# S: values that the others make equal are different here and the other way round: dim == vdim in the state mixers,
#    kv_heads == heads in attention, one tap (no convolution state), no soft cap, no rotation.
CONFIGS = {
    "P": config(211, 64, 1e-6, [
        with_mlp(delta(4, 2, 24, 20, 3), 96, 1.5),
        with_mlp(attention(4, 2, 32, 16, 0.21, softcap=3.0, rot=(16, 10000.0), v_mix=True), 96, 1.5),
        with_mlp(gla(2, 24, 40, 8.0, 8), None, None),
        with_mlp(attention(4, 2, 32, 16, 0.17, softcap=3.0, rot=(16, 10000.0), v_mix=True), 80, 0.8),
        with_mlp(attention(2, 1, 48, 16, 0.15, softcap=5.0, rot=(48, 500.0), v_mix=False), 96, 1.5)]),
    "Q": config(333, 128, 1e-5, [
        with_mlp(gla(1, 48, 20, 3.0, 4), 160, 3.0),
        with_mlp(delta(2, 2, 40, 33, 2), 160, 3.0),
        with_mlp(attention(6, 3, 16, 32, 0.25, softcap=4.0, rot=(16, 1e6)), 160, 3.0)]),
    "R": config(190, 128, 1e-6, [
        with_mlp(attention(2, 1, 64, 64, 0.125, softcap=4.0, rot=(32, 10000.0), v_mix=True), 128, 2.5),
        with_mlp(delta(2, 1, 64, 64, 4), 128, 2.5),
        with_mlp(attention(2, 1, 64, 64, 0.125, softcap=4.0, rot=(32, 10000.0), v_mix=True), 128, 2.5),
        with_mlp(attention(1, 1, 128, 128, 0.09, softcap=3.0, rot=(128, 1e5)), 128, 2.5)]),
    "S": config(150, 96, 2e-6, [
        with_mlp(attention(3, 3, 24, 24, 0.18, v_mix=True), 64, 1.0),
        with_mlp(delta(3, 3, 32, 32, 1), 64, 1.0),
        with_mlp(gla(3, 16, 16, 1.0, 16), 64, 1.0)]),
}
SEEDS = {"P": 11, "Q": 12, "R": 13, "S": 14}


def random_config(seed, tensor_core_heads=False):
    """A configuration drawn at random: 2 to 7 layers of any order, every size, option and constant from a list that
    includes 1, equal and unequal sizes and sizes that are no powers of two.  tensor_core_heads: attention heads of
    64 or 128 with values of the same size (the heads that the tensor-core attention kernels take in bfloat16)."""
    rng = np.random.default_rng(seed)
    width = int(rng.choice([48, 64, 72, 96, 128, 160, 192, 256, 320]))
    layers, shape = [], None
    for _ in range(int(rng.integers(2, 8))):
        kind = rng.choice(["attention", "delta", "gla"], p=[0.45, 0.3, 0.25])
        if kind == "attention":
            if shape is None or rng.random() < 0.3:
                kv, rep = int(rng.choice([1, 2, 3, 4])), int(rng.choice([1, 2, 4]))
                dim = int(rng.choice([8, 16, 24, 32, 40, 48, 64, 96, 128]))
                vdim = int(rng.choice([8, 16, 24, 32, 48, 64, 128, dim, dim]))
                if tensor_core_heads:
                    dim = vdim = int(rng.choice([64, 128]))
                shape = (kv * rep, kv, dim, vdim)
            H, G, dim, vdim = shape
            rot = None
            if rng.random() < 0.85:
                rot = (int(rng.choice([d for d in (2, 4, 8, 16, 24, 32, 64, dim) if d <= dim and d % 2 == 0])),
                       float(rng.choice([100.0, 10000.0, 250000.0, 1e6])))
            layer = attention(H, G, dim, vdim, float(rng.choice([dim ** -0.5, 0.1, 0.25])),
                              softcap=float(rng.choice([0.0, 3.0, 8.0, 20.0, 50.0])), rot=rot, v_mix=bool(rng.random() < 0.6))
        elif kind == "delta":
            kv, rep = int(rng.choice([1, 2, 3])), int(rng.choice([1, 2, 4]))
            layer = delta(kv * rep, kv, int(rng.choice([8, 16, 24, 32, 48, 64, 128])),
                          int(rng.choice([8, 16, 20, 32, 64, 96, 128])), int(rng.integers(1, 7)))
        else:
            layer = gla(int(rng.choice([1, 2, 3, 4])), int(rng.choice([8, 16, 24, 32, 64])),
                        int(rng.choice([8, 16, 40, 64, 128])), float(rng.choice([1.0, 4.0, 16.0, 32.0])),
                        int(rng.choice([2, 4, 8, 16, 24])))
        if rng.random() < 0.15:
            layers.append(with_mlp(layer, None, None))
        else:
            layers.append(with_mlp(layer, int(rng.choice([64, 96, 100, 128, 160, 200, 256, 384, 512])),
                                   float(rng.choice([0.7, 1.0, 2.0, 5.0]))))
    first = None                 # layers that mix values must agree in the values' shape
    for l in layers:
        if l["type"] == "attention" and l["mixer"].get("v_mix"):
            key = (l["mixer"]["kv_heads"], l["mixer"]["vdim"])
            first = first or key
            if key != first:
                l["mixer"]["v_mix"] = False
    return config(int(rng.integers(50, 700)), width, float(rng.choice([1e-6, 1e-5, 1e-4])), layers)


def bf16(a):
    """Rounded to values that bfloat16 holds (ties to even), as float32."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).reshape(np.shape(a))


def draw_tensors(cfg, seed):
    """name -> float32 array.  The scales are chosen so that every mechanism matters: the stream and the sub-layers'
    outputs are of order one, attention scores have a standard deviation of about 2.5 (a key that is lost or added,
    or a rotation that is off, moves the logits far beyond bfloat16's rounding), decays spread over (0, 1), the
    feed-forward's limits cut a good part of its inputs."""
    rng = np.random.default_rng(seed)
    e = cfg["width"]
    t = {}

    def mat(out, inp, gain=1.0):
        return rng.normal(0.0, gain / np.sqrt(inp), size=(out, inp))

    t["embed"] = rng.normal(0.0, 1.0, size=(cfg["vocab"], e))
    t["head"] = mat(cfg["vocab"], e, 2.0)
    t["final.norm"] = 1.0 + rng.normal(0.0, 0.1, size=e)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        t[p + "norm1"] = 1.0 + rng.normal(0.0, 0.1, size=e)
        t[p + "ls1"] = rng.normal(0.6, 0.15, size=e)
        if layer["type"] == "attention":
            G = m["kv_heads"]
            gain = (2.5 / m["scale"]) ** 0.5 / d ** 0.5          # q.k * scale ~ N(0, 2.5^2)
            t[p + "mix.q"], t[p + "mix.k"] = mat(H * d, e, gain), mat(G * d, e, gain)
            t[p + "mix.v"] = mat(G * dv, e, 3.0)
            for n, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                t[p + f"mix.{n}.b"] = rng.normal(0.0, 0.3, size=rows)
            if m.get("v_mix"):
                t[p + "mix.vmix"] = np.asarray(rng.uniform(0.3, 0.7))
            t[p + "mix.g"] = mat(H, e, 1.5)
            t[p + "mix.o"] = mat(e, H * dv, 3.0)
        elif layer["type"] == "delta":
            G, taps = m["kv_heads"], m["conv"]
            for n, rows in (("q", G * d), ("k", G * d), ("v", H * dv)):
                t[p + f"mix.{n}"] = mat(rows, e, 1.5)
                t[p + f"mix.{n}.conv"] = rng.normal(0.0, 0.6, size=(rows, taps))
            t[p + "mix.b"], t[p + "mix.a"] = mat(H, e, 1.5), mat(H, e, 1.5)
            t[p + "mix.A_log"] = rng.uniform(-2.0, 0.5, size=H)
            t[p + "mix.dt_bias"] = rng.normal(0.0, 1.0, size=H)
            t[p + "mix.norm"] = 1.0 + rng.normal(0.0, 0.1, size=dv)
            t[p + "mix.g"] = mat(H * dv, e, 1.5)
            t[p + "mix.o"] = mat(e, H * dv, 2.0)
        else:
            r = m["rank"]
            t[p + "mix.q"], t[p + "mix.k"] = mat(H * d, e, 1.5), mat(H * d, e, 1.5)
            t[p + "mix.v"], t[p + "mix.g"] = mat(H * dv, e), mat(H * dv, e, 1.5)
            t[p + "mix.o"] = mat(e, H * dv, 2.0)
            t[p + "mix.norm"] = 1.0 + rng.normal(0.0, 0.1, size=dv)
            t[p + "mix.a1"] = mat(r, e)
            t[p + "mix.a2"] = mat(H * d, r, 2.0)
            t[p + "mix.a2.b"] = rng.normal(1.0, 1.5, size=H * d)
        f = layer.get("mlp")
        if f:
            t[p + "mlp.gate"], t[p + "mlp.up"] = mat(f["ff"], e, 1.5 * f["limit"]), mat(f["ff"], e, 1.5 * f["limit"])
            t[p + "mlp.down"] = mat(e, f["ff"], 2.0)
            t[p + "ls2"] = rng.normal(0.6, 0.15, size=e)
    return {n: bf16(a) for n, a in t.items()}


_tmp = []


@functools.lru_cache(maxsize=None)
def model_folder(name):
    """config.json and model.safetensors (bfloat16) of a test configuration, in a temporary place."""
    import torch
    from air_b200.weights.loader import write_model_folder
    d = tempfile.TemporaryDirectory(prefix=f"air_b200_bivizen_{name}_")
    _tmp.append(d)
    if name not in CONFIGS:      # "random<seed>" / "tensorcore<seed>": drawn at random
        seed = int(name.lstrip("randomtensorcore"))
        CONFIGS[name], SEEDS[name] = random_config(seed, tensor_core_heads=name.startswith("tensorcore")), seed
    cfg = CONFIGS[name]
    tensors = {n: torch.from_numpy(np.ascontiguousarray(a)).reshape(a.shape).to(torch.bfloat16)
               for n, a in draw_tensors(cfg, SEEDS[name]).items()}
    write_model_folder(d.name, cfg, tensors)
    return d.name


@functools.lru_cache(maxsize=None)
def plain_model(name):
    from plain import bivizen_plain as plain
    return plain.read_model(model_folder(name))


_logits = {}


def plain_logits(name, tokens):
    from plain import bivizen_plain as plain
    key = (name, tuple(tokens))
    if key not in _logits:
        cfg, tensors = plain_model(name)
        _logits[key] = plain.forward(cfg, tensors, list(tokens)).astype(np.float64)
    return _logits[key]


def tokens_for(name, n, seed):
    return np.random.default_rng(5000 + seed).integers(0, CONFIGS[name]["vocab"], size=n).tolist()


def plain_greedy(name, prompt, n):
    out, toks = [], list(prompt)
    for _ in range(n):
        nxt = int(plain_logits(name, toks)[-1].argmax())
        out.append(nxt)
        toks.append(nxt)
    return out


# float32: sums of a few hundred terms in another order than the 64-bit oracle (measured: 3e-7 of the largest
# |logit| of the request at most).  bfloat16: activations rounded to 8 bits at the inputs of the products and in the
# cache; measured over these models, a row's mean difference is 1.2e-3 of the largest |logit| in the median and up
# to 8e-3 at single positions (a sharp attention whose two best keys are close), where the largest difference of a
# row reaches 5.3e-2; the same for rows of a prompt and for decoded tokens.  A mechanism that is left out moves the logits by 0.1 and more (tests/test_bivizen.py).
FP32_TOL = 5e-5
BF16_MAX_TOL = 8e-2
BF16_MEAN_TOL = 1.5e-2


def check(got, name, streams, dtype):
    """got: {(request, position): logits}; every request of `streams` must have rows, and every row must agree."""
    worst = 0.0
    for rid, toks in streams.items():
        ref = plain_logits(name, toks)
        scale = max(1.0, float(np.abs(ref).max()))
        rows = sorted(p for (r, p) in got if r == rid)
        assert rows, f"no logits for request {rid}"
        for p in rows:
            out = got[(rid, p)]
            assert np.isfinite(out).all()
            diff = np.abs(out - ref[p])
            if dtype == "float32":
                assert diff.max() <= FP32_TOL * scale, (rid, p, float(diff.max()), scale)
            else:
                assert diff.max() <= BF16_MAX_TOL * scale, (rid, p, float(diff.max()), scale)
                assert diff.mean() <= BF16_MEAN_TOL * scale, (rid, p, float(diff.mean()), scale)
            worst = max(worst, float(diff.max()) / scale)
    return worst
