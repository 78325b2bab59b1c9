"""Tomodra on the GPU against the plain implementation (tests/plain/tomodra_plain.py, 64-bit): every mechanism alone
through its kernel, then whole models through Engine.step, the scheduler and the trace runner, in float32 and
bfloat16, for configurations that differ in every size and option (tomodra_util.CONFIGS)."""
import tempfile

import numpy as np
import pytest
import torch

import tomodra_util as tu
import util
from plain import tomodra_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.ascontiguousarray(a)).to(device=DEV, dtype=dtype)


def i32(a):
    return torch.tensor(list(a), dtype=torch.int32, device=DEV)


# ----------------------------------------------------------------------------- mechanisms alone
def test_norm_behind_the_sum():
    from air_b200.csrc import ops
    rng = np.random.default_rng(1)
    T, E = 11, 72
    h, w = rng.normal(size=(T, E)), rng.normal(1, 0.1, size=E)
    a, b, g = rng.normal(size=(3, T, E)), rng.normal(size=(2, T, E)), rng.uniform(size=T)
    want = plain.rms_norm(2.5 * h + a.sum(0) + g[:, None] * b.sum(0), w, 1e-5)
    for out_dtype in (torch.bfloat16, None):
        hd = dev(h)
        out = None if out_dtype is None else torch.empty((T, E), dtype=out_dtype, device=DEV)
        ops.post_norm(hd, 2.5, dev(a), dev(b), dev(g), dev(w), 1e-5, out)
        assert np.abs(hd.cpu().numpy() - want).max() < 1e-5
        if out is not None:
            assert np.abs(out.float().cpu().numpy() - want).max() < 2e-2
    hd = dev(h)
    ops.post_norm(hd, 1.0, dev(a[0]), None, None, dev(w, torch.bfloat16), 1e-5, None)      # one term, a 16-bit weight
    assert np.abs(hd.cpu().numpy() - plain.rms_norm(h + a[0], tu.bf16(w), 1e-5)).max() < 1e-5
    hd = dev(h)
    ops.post_norm(hd, 1.0, None, dev(b[0]), dev(g), None, 0.0, None)                        # the sum alone
    assert np.abs(hd.cpu().numpy() - (h + g[:, None] * b[0])).max() < 1e-5


@pytest.mark.parametrize("H,G,dk,dv,rot,pairing,scaling", [
    (4, 2, 32, 16, 16, "neighbours", (4.0, 64, 16.0, 2.0)), (1, 1, 48, 20, 48, "neighbours", None),
    (3, 3, 24, 40, 12, "half", (2.0, 16, 4.0, 1.0)), (2, 1, 256, 8, 64, "neighbours", (8.0, 1024, 32.0, 1.0)),
    (2, 2, 6, 6, 0, "neighbours", None)])
def test_queries_and_keys_are_normalised_then_rotated(H, G, dk, dv, rot, pairing, scaling):
    """Positions far apart (angles of thousands of turns), pages scattered, two requests: q and the pages against the
    plain functions."""
    from air_b200.csrc import ops
    from air_b200.parts.rope import bent_frequencies
    rng = np.random.default_rng(dk)
    P, base, eps = 16, 5000.0, 1e-5
    sc = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
    positions = np.array([0, 1, 15, 16, 17, 100000, 31, 32])
    slots = np.array([1, 1, 1, 1, 1, 0, 0, 0])
    T = len(positions)
    proj = rng.normal(size=(T, (H + G) * dk + G * dv)) * 3
    qw, kw = rng.normal(1, 0.2, size=dk), rng.normal(1, 0.2, size=dk)
    f, mag = plain.yarn_frequencies(rot, base, sc) if rot else (np.zeros(0), 1.0)
    rotate = plain.rotate_neighbours if pairing == "neighbours" else \
        (lambda x, p, f, d, m: plain.rotate_half_split(x, p, f, d) * 1.0)
    q = plain.rms_norm(proj[:, :H * dk].reshape(T, H, dk), qw, eps)
    k = plain.rms_norm(proj[:, H * dk:(H + G) * dk].reshape(T, G, dk), kw, eps)
    if rot:
        q, k = rotate(q, positions, f, rot, mag), rotate(k, positions, f, rot, mag)
    v = proj[:, (H + G) * dk:].reshape(T, G, dv)
    table = torch.full((2, 8192), -1, dtype=torch.int32, device=DEV)
    table[1, :2] = i32([5, 2])
    table[0, [100000 // P, 1, 2]] = i32([7, 0, 3])
    freq = bent_frequencies(rot, base, sc)[0].to(DEV) if rot else None
    if pairing == "half" and sc:
        mag = 1.0           # (the plain half-split rotation has no magnitude)
    cache = torch.zeros((8, G * P * (dk + dv)), device=DEV)
    qo = torch.empty((T, H, dk), device=DEV)
    ops.qk_normed_prepare(dev(proj), dev(qw), dev(kw), eps, freq, pairing, mag, i32(positions), i32(slots), table, qo,
                          cache, G, dv, P)
    assert np.abs(qo.cpu().numpy() - q).max() < 2e-5
    pages = cache.cpu().numpy()
    for t in range(T):
        page = int(table[slots[t], positions[t] // P])
        keys = pages[page, :G * P * dk].reshape(G, P, dk)[:, positions[t] % P]
        values = pages[page, G * P * dk:].reshape(G, P, dv)[:, positions[t] % P]
        assert np.abs(keys - k[t]).max() < 2e-5 and np.abs(values - v[t]).max() < 1e-6
    if rot == 0:      # and without weights nothing is normalised
        ops.qk_normed_prepare(dev(proj), None, None, eps, None, pairing, 1.0, i32(positions), i32(slots), table, qo,
                              cache, G, dv, P)
        assert np.abs(qo.cpu().numpy() - proj[:, :H * dk].reshape(T, H, dk)).max() < 1e-6


def attend(q, k, v, scale, mask, sink=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv], with the plain softmax."""
    H, G = q.shape[1], k.shape[1]
    k, v = np.repeat(k, H // G, axis=1), np.repeat(v, H // G, axis=1)
    a = plain.masked_softmax(np.einsum("thd,shd->hts", q, k) * scale, mask, sink)
    return np.einsum("hts,shd->thd", a, v)


def pointed(rng, T, H, G, d, dv, pairs, scale):
    """Random queries, keys and values in which query i of each pair (i, j) points at key j so strongly that key j,
    if it is seen, takes nearly all the weight; its value is large."""
    q, k, v = rng.normal(size=(T, H, d)), rng.normal(size=(T, G, d)), rng.normal(size=(T, G, dv))
    for i, j in pairs:
        q[i] = np.repeat(k[j], H // G, axis=0) * (14.0 / scale / d)
        v[j] = 20.0 + j / 20.0
    return q, k, v


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind,size", [("window", 50), ("chunk", 40), ("window", 1), ("chunk", 16), ("all", None)])
def test_attention_sees_the_keys_inside_its_mask_and_no_other(kind, size, dtype):
    """One request of 300 tokens over scattered pages of 16.  Queries are made to point at keys far away, at the first
    key that their window or chunk still holds and at the one just outside it; a sink in the softmax.  As rows of
    prompt portions, and token by token."""
    from air_b200.csrc import ops
    rng = np.random.default_rng(size or 0)
    T, P, H, G, d, dv, scale = 300, 16, 4, 2, 32, 24, 0.2
    n = size or T
    if kind == "chunk":
        mask = plain.chunk_mask(T, n)
        pairs = [(299, 299 - 299 % n), (298, 299 - 299 % n - 1), (2 * n - 1, n), (2 * n, 2 * n - 1), (250, 3)]
    else:
        mask = plain.window_mask(T, n)
        pairs = [(299, 299 - n + 1), (298, max(298 - n, 0)), (min(n + 5, 280), 6), (min(n + 4, 279), 3), (250, 3)]
    q, k, v = pointed(rng, T, H, G, d, dv, pairs, scale)
    sink = rng.normal(1.0, 2.0, size=H)
    if dtype == torch.bfloat16:
        q, k, v = (tu.bf16(x).astype(np.float64) for x in (q, k, v))
    want = attend(q, k, v, scale, mask, sink)
    if size and size > 1:
        other = plain.window_mask(T, n + 1) if kind == "window" else plain.chunk_mask(T, n + 1)
        assert np.abs(attend(q, k, v, scale, other, sink) - want).max() > 5.0        # one key more or less shows
    pages = rng.permutation(40)[:-(-T // P)]
    table = torch.full((2, 64), -1, dtype=torch.int32, device=DEV)
    table[1, :len(pages)] = i32(pages)
    cache = torch.zeros((40, G * P * (d + dv)), dtype=dtype, device=DEV)
    for t in range(T):
        page = cache[pages[t // P]]
        page[:G * P * d].view(G, P, d)[:, t % P] = dev(k[t], dtype)
        page[G * P * d:].view(G, P, dv)[:, t % P] = dev(v[t], dtype)
    for cuts in ([2, 61, T - 63], [T - 3, 1, 1, 1]):
        at = 0
        for m in cuts:
            for kernel, more in ((ops.paged_attention_ref, {}), (ops.grouped_attention, {}),
                                 (ops.grouped_attention, {"splits": 3})):
                out = torch.empty((m, H, dv), dtype=dtype, device=DEV)
                kernel(dev(q[at:at + m], dtype), cache, table, i32([1] * m), i32(range(at, at + m)), out,
                       size if kind == "window" else None, scale, kv_heads=G, page_tokens=P,
                       chunk=size if kind == "chunk" else None, sink=dev(sink), **more)
                tol = 3e-4 if dtype == torch.float32 else 0.3          # (values up to 35: bfloat16 holds them to 0.125)
                assert np.abs(out.float().cpu().numpy() - want[at:at + m]).max() < tol, (at, m, kernel.__name__)
            at += m
    if dtype != torch.bfloat16:
        return
    # the same rows as portions of a batch: long portions through the matrix products over gathered keys (in blocks of
    # 100 queries here, so that blocks begin inside windows and chunks), a short one and single tokens of another
    # request through the pages, in one step
    from types import SimpleNamespace
    from air_b200.parts.base import HostBatch, Runtime
    from air_b200.parts.gathered_attention import PortionAttention

    class Road(PortionAttention):
        BLOCK = 100
        rt = Runtime(device=torch.device(DEV), dtype=torch.bfloat16, page_tokens=P)
        heads, kv_heads, window, chunk, sinks = H, G, size if kind == "window" else None, size if kind == "chunk" else None, dev(sink)

    road = Road()
    road.scale = scale
    table[0, :len(pages)] = i32(pages)                  # a second request that holds the same pages
    for counts, lengths, slots in (([1, 33, 1], [40, 0, 299], [0, 1, 0]), ([2, 261], [37, 39], [0, 1]), ([300], [0], [1])):
        q_start = [0] + np.cumsum(counts).tolist()
        batch = HostBatch(counts=counts, lengths=lengths, slots=slots, q_start=q_start)
        plan = road.plan(batch)
        positions = [p for n, l in zip(counts, lengths) for p in range(l, l + n)]
        seq = [s_ for n, s_ in zip(counts, slots) for _ in range(n)]
        ctx = SimpleNamespace(plans={road.plan_key(): SimpleNamespace(small_seq=i32(plan.arrays["small_seq"]), **plan.values)},
                              token_seq=i32(seq), positions=i32(positions))
        out = torch.empty((len(positions), H, dv), dtype=dtype, device=DEV)
        road.attend(dev(q[positions], dtype), cache, table, ctx, out, kv_heads=G, page_tokens=P)
        assert np.abs(out.float().cpu().numpy() - want[positions]).max() < 0.3, counts


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,d,rot,R,dv,window", [(4, 24, 8, 40, 20, 48), (1, 32, 16, 56, 40, None), (3, 8, 4, 300, 8, 17), (16, 32, 16, 112, 24, 40), (7, 16, 8, 600, 8, None)])
def test_latent_attention_through_its_kernels(H, d, rot, R, dv, window, dtype):
    """From the projection's output to the heads' outputs: the rows in the pages, the queries carried through the key
    expansion, attention over the rows, the value expansion.  Against keys and values expanded per head, as the
    equations have them.  Queries point at the first row inside the window and at the one before it."""
    from air_b200.csrc import ops
    rng = np.random.default_rng(R)
    T, P, scale, base, eps = 150, 16, 0.2, 1000.0, 1e-5
    n = window or T
    proj = rng.normal(size=(T, H * (d + rot) + R + rot))
    cw = rng.normal(1, 0.2, size=R)
    uk, uv = rng.normal(size=(H * d, R)) / R ** 0.5, rng.normal(size=(H * dv, R)) / R ** 0.5
    m = dict(kv_rank=R, rot_dim=rot, rot=dict(base=base))
    f = plain.plain_frequencies(rot, base)
    positions = np.arange(T)
    c = plain.rms_norm(proj[:, H * (d + rot):H * (d + rot) + R], cw, eps)
    kr = plain.rotate_half_split(proj[:, H * (d + rot) + R:], positions, f, rot)
    for i, j in ((T - 1, T - n), (T - 2, max(T - 2 - n, 0)), (100, 3)):
        # the plain part of the query is the key it should find, enlarged
        key = (c[j] @ uk.T).reshape(H, d)
        proj[i, :H * (d + rot)].reshape(H, d + rot)[:, :d] = key * (14.0 / scale / (key ** 2).sum(-1, keepdims=True))
    if dtype == torch.bfloat16:
        uk, uv = tu.bf16(uk), tu.bf16(uv)
    q = proj[:, :H * (d + rot)].reshape(T, H, d + rot)
    q = np.concatenate([q[..., :d], plain.rotate_half_split(q[..., d:], positions, f, rot)], axis=-1)
    keys = np.concatenate([(c @ uk.T).reshape(T, H, d), np.repeat(kr[:, None], H, axis=1)], axis=-1)
    values = (c @ uv.T).reshape(T, H, dv)
    want = attend(q, keys, values, scale, plain.window_mask(T, n))
    if window:
        assert np.abs(attend(q, keys, values, scale, plain.window_mask(T, n + 1)) - want).max() > 0.3
    pages = rng.permutation(20)[:-(-T // P)]
    table = torch.full((3, 64), -1, dtype=torch.int32, device=DEV)
    table[2, :len(pages)] = i32(pages)
    rows = torch.zeros((20, P, R + rot), dtype=dtype, device=DEV)
    uk_t = dev(uk.reshape(H, d, R).transpose(0, 2, 1), dtype)
    uv_d = dev(uv.reshape(H, dv, R), dtype)
    freq = dev(f, torch.float64)
    at = 0
    for cut in (3, 61, T - 67, 1, 1, 1):
        pos, seq = i32(range(at, at + cut)), i32([2] * cut)
        q_plain = torch.empty((cut, H, d), dtype=dtype, device=DEV)
        q_full = torch.empty((cut, H, R + rot), device=DEV)
        ops.latent_prepare(dev(proj[at:at + cut]), dev(cw), eps, freq, pos, seq, table, q_plain, q_full, rows, True)
        ops.grouped_gemm(q_plain, uk_t, q_full, R, d, lda=H * d, ldo=H * (R + rot), groups=H, a_group_stride=d,
                         o_group_stride=R + rot, a_local=True, o_local=True, rows_per_group=cut)
        summed = torch.empty((cut, H, R), dtype=dtype, device=DEV)
        ops.paged_attention_ref(q_full, rows, table, seq, pos, summed, window, scale, latent=True)
        if ops.grouped_attention_ok(dtype, R + rot, R):
            again = torch.empty((cut, H, R), dtype=dtype, device=DEV)
            ops.grouped_attention(q_full, rows, table, seq, pos, again, window, scale, latent=True)
            assert np.abs(again.float().cpu().numpy() - summed.float().cpu().numpy()).max() < (1e-5 if dtype == torch.float32 else 2e-2)
        out = torch.empty((cut, H, dv), dtype=dtype, device=DEV)
        ops.grouped_gemm(summed, uv_d, out, dv, R, lda=H * R, ldo=H * dv, groups=H, a_group_stride=R,
                         o_group_stride=dv, a_local=True, o_local=True, rows_per_group=cut)
        tol = 3e-4 if dtype == torch.float32 else 0.1
        assert np.abs(out.float().cpu().numpy() - want[at:at + cut]).max() < tol, (at, cut)
        at += cut
    kept = rows.float().cpu().numpy()
    for t in (0, 15, 16, T - 1):
        row = kept[pages[t // P], t % P]
        tol = 2e-5 if dtype == torch.float32 else 3e-2
        assert np.abs(row[:R] - c[t]).max() < tol and np.abs(row[R:] - kr[t]).max() < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,top,E,F,T", [(5, 2, 64, 48, 150), (3, 3, 96, 40, 7), (8, 1, 72, 64, 65), (130, 6, 32, 20, 40)])
def test_router_and_experts(n, top, E, F, T, dtype):
    """The chosen experts and their weights against a sort; every (token, choice) once in its expert's slots; the two
    grouped products against the plain expert with the weight on its input."""
    from air_b200.csrc import ops
    rng = np.random.default_rng(n)
    x = rng.normal(size=(T, E))
    z = rng.normal(size=(T, n + 1)) * 2
    z[3, :n] = 0.7                                             # all equal: the lowest indices win
    if n > 2:
        z[5, 1], z[5, 2] = 1.5, 1.5
    expert = torch.empty((T, top), dtype=torch.int32, device=DEV)
    weight = torch.empty((T, top), device=DEV)
    gate = torch.empty((T,), device=DEV)
    ops.moe_route(dev(z), n, top, expert, weight, gate, has_gate=True)
    s = plain.sigmoid(z[:, :n].astype(np.float32).astype(np.float64))
    order = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    assert np.array_equal(expert.cpu().numpy(), order)
    assert np.abs(weight.cpu().numpy() - np.take_along_axis(s, order, -1)).max() < 1e-6
    assert np.abs(gate.cpu().numpy() - plain.sigmoid(z[:, n])).max() < 1e-6
    soft = torch.empty((T, top), device=DEV)
    ops.moe_route(dev(z), n, top, expert, soft, None, score="softmax", renormalize=True)
    p = np.exp(z[:, :n] - z[:, :n].max(-1, keepdims=True))
    p = np.take_along_axis(p / p.sum(-1, keepdims=True), np.argsort(-p, axis=-1, kind="stable")[:, :top], -1)
    assert np.abs(soft.cpu().numpy() - p / p.sum(-1, keepdims=True)).max() < 1e-5
    ops.moe_route(dev(z), n, top, expert, weight, gate, has_gate=True)
    pairs = T * top
    start = torch.empty(n + 1, dtype=torch.int32, device=DEV)
    slots = torch.empty(pairs, dtype=torch.int32, device=DEV)
    tiles = torch.full((pairs // ops.GROUP_TILE + n, 2), -1, dtype=torch.int32, device=DEV)
    count = torch.empty(1, dtype=torch.int32, device=DEV)
    ops.moe_sort(expert, n, start, slots, tiles, count)
    st, sl = start.cpu().numpy(), slots.cpu().numpy()
    assert sorted(sl.tolist()) == list(range(pairs)) and st[0] == 0 and st[-1] == pairs
    for e in range(n):
        assert all(order.reshape(-1)[p] == e for p in sl[st[e]:st[e + 1]])
    listed = tiles.cpu().numpy()[:int(count)]
    assert sum(-(-(st[e + 1] - st[e]) // ops.GROUP_TILE) for e in range(n)) == len(listed)
    w = {}
    for e in range(n):
        w[f"e{e}.gate"], w[f"e{e}.up"] = rng.normal(size=(F, E)) / E ** 0.5, rng.normal(size=(F, E)) / E ** 0.5
        w[f"e{e}.down"] = rng.normal(size=(E, F)) / F ** 0.5
    if dtype == torch.bfloat16:
        w = {k: tu.bf16(a).astype(np.float64) for k, a in w.items()}
        x = tu.bf16(x).astype(np.float64)
    gate_up = dev(np.stack([np.concatenate([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(n)]), dtype)
    down = dev(np.stack([w[f"e{e}.down"] for e in range(n)]), dtype)
    act = torch.empty((pairs, F), dtype=dtype, device=DEV)
    ops.grouped_gemm(dev(x, dtype), gate_up, act, F, E, lda=E, ldo=F, groups=n, a_index=slots, a_div=top,
                     a_scale=weight.view(-1), start=start, tiles=tiles, num_tiles=count, silu_mul=True)
    y = torch.full((top, T, E), 9.0, device=DEV)
    ops.grouped_gemm(act, down, y, E, F, lda=F, ldo=E, groups=n, o_index=slots, o_div=top, o_part_stride=T * E,
                     start=start, tiles=tiles, num_tiles=count)
    want = np.zeros((T, E))
    sw = weight.cpu().numpy().astype(np.float64)
    for t in range(T):
        for j in range(top):
            u = sw[t, j] * x[t]
            want[t] += plain.expert(tu.bf16(u).astype(np.float64) if dtype == torch.bfloat16 else u, w, f"e{order[t, j]}.")
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    assert np.abs(y.sum(0).cpu().numpy() - want).max() < tol * max(1.0, np.abs(want).max())


# ----------------------------------------------------------------------------- whole models
LENGTHS = {"A": (1, 7, 33, 97, 150), "B": (5, 40, 131, 64), "C": (2, 65, 150, 300)}


def streams_for(name, seed=0, lengths=None):
    return {f"{name}{i}": tu.tokens_for(name, n, seed + i) for i, n in enumerate(lengths or LENGTHS[name])}


def replay(name, dtype, steps, page_tokens=16, max_requests=4, peak_page=64):
    return util.replay(tu.model_folder(name), dtype, steps, max_tokens=util.peak_tokens(steps, page=peak_page),
                       page_tokens=page_tokens, max_requests=max_requests)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompts(name, dtype):
    streams = streams_for(name)
    got, _ = replay(name, dtype, util.trace_whole(streams))
    tu.check(got, name, streams, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_prompt_then_token_by_token(name, dtype):
    """The tail is decoded one by one, long enough for windows and chunks to pass over decoded tokens."""
    streams = streams_for(name, 10)
    got, _ = replay(name, dtype, util.trace_bulk_tail(streams, tail=75))
    tu.check(got, name, streams, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_portions_down_to_two_tokens(name, dtype):
    streams = streams_for(name, 20)
    got, _ = replay(name, dtype, util.trace_portions(streams))
    tu.check(got, name, streams, dtype)
    got, _ = replay(name, dtype, util.trace_portions(streams, sizes=(2, 2, 1, 3, 16, 15, 17, 64, 63, 65, 2)), page_tokens=64)
    tu.check(got, name, streams, dtype)


@pytest.mark.parametrize("page", [16, 64])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_unequal_requests_together_with_pages_and_slots_used_again(name, dtype, page):
    """Ten requests through three slots and a pool that holds the peak only: every request must come out as it does
    alone (the oracle runs each alone), whatever shared its batches and whoever had its slot and pages before."""
    lengths = LENGTHS[name] + (120, 2, 77, 101, 64, 129)
    streams = streams_for(name, 50, lengths)
    steps = util.trace_mixed(streams, seed=3, live=3)
    got, engine = replay(name, dtype, steps, page_tokens=page, max_requests=3)
    tu.check(got, name, streams, dtype)
    for group in engine.cache.groups:
        assert group.pool.takes > group.pool.num_pages, "pages were used again"


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_experts_through_the_librarys_grouped_product(name, monkeypatch):
    """The road that steps of many rows per expert take through the experts, forced for short prompts too; experts that
    nobody chose, experts with one row, mixed batches."""
    from air_b200.parts.experts import RoutedExperts
    monkeypatch.setattr(RoutedExperts, "LIBRARY_ROWS", 0)
    streams = streams_for(name, 70, (3, 150, 41))
    got, _ = replay(name, "bfloat16", util.trace_whole(streams), page_tokens=64)
    tu.check(got, name, streams, "bfloat16")
    got, _ = replay(name, "bfloat16", util.trace_mixed(streams, seed=4, live=3), page_tokens=64, max_requests=3)
    tu.check(got, name, streams, "bfloat16")


@pytest.mark.parametrize("name", ["random1", "random2", "random3", "random5", "random8", "random13", "random21", "random34"])
def test_configurations_drawn_at_random(name):
    """Layer orders, sizes and constants that nobody chose (tomodra_util.random_config): whole prompts and a mixed
    schedule through three slots, in float32 within its tolerance; bfloat16 must be finite and agree with the oracle in
    the median (how far single rows lie depends on how a drawn model amplifies rounding)."""
    folder = tu.model_folder(name)
    streams = {f"{name}_{i}": tu.tokens_for(name, n, 80 + i) for i, n in enumerate((150, 3, 70, 1, 97))}
    margin = min(tu.plain_run(name, toks)[1] for toks in streams.values())
    whole = util.trace_whole(streams)
    mixed = util.trace_mixed(streams, seed=5, live=3, tail=20)
    got, _ = replay(name, "float32", whole, page_tokens=64)
    tu.check(got, name, streams, "float32")
    got, _ = replay(name, "float32", mixed, page_tokens=16, max_requests=3)
    tu.check(got, name, streams, "float32")
    for steps, page in ((whole, 16), (mixed, 64)):
        got, _ = replay(name, "bfloat16", steps, page_tokens=page, max_requests=3)
        means = []
        for (rid, p), row in got.items():
            ref = tu.plain_logits(name, streams[rid])[p]
            assert np.isfinite(row).all()
            means.append(np.abs(row - ref).mean() / max(1.0, np.abs(tu.plain_logits(name, streams[rid])).max()))
        if margin > 0.01:
            assert np.median(means) <= 2 * tu.BF16_MEDIAN_TOL, (name, float(np.median(means)))


@pytest.mark.parametrize("name", ["A", "C"])
def test_float32_does_not_depend_on_the_cut_or_the_batch(name):
    streams = streams_for(name, 30, (97, 40, 131))
    whole, _ = replay(name, "float32", util.trace_whole(streams))
    cut, _ = replay(name, "float32", util.trace_portions(streams, sizes=(2, 31, 1, 16, 5)))
    mixed, _ = replay(name, "float32", util.trace_mixed(streams, seed=1, live=3), max_requests=3)
    for key, row in whole.items():
        assert np.abs(cut[key] - row).max() < 2e-5
        assert np.abs(mixed[key] - row).max() < 2e-5


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_bfloat16_agrees_with_itself_across_schedules(name):
    """Rows of whole prompts against the same rows from portions and from mixed batches.  Long portions attend through
    matrix products over gathered keys, short ones and single tokens through the pages, so a row's rounding depends on
    the schedule; the rows must still agree as they agree with the oracle."""
    streams = streams_for(name, 30, (97, 40, 131))
    whole, _ = replay(name, "bfloat16", util.trace_whole(streams), page_tokens=64)
    cut, _ = replay(name, "bfloat16", util.trace_portions(streams, sizes=(2, 31, 1, 16, 5)), page_tokens=64)
    mixed, _ = replay(name, "bfloat16", util.trace_mixed(streams, seed=1, live=3), page_tokens=64, max_requests=3)
    for other in (cut, mixed):
        means = []
        for key, row in whole.items():
            scale = max(1.0, np.abs(row).max())
            diff = np.abs(other[key] - row)
            # (each is within the row limits of the oracle: together twice that)
            assert diff.max() <= 2 * tu.BF16_MAX_TOL * scale and diff.mean() <= 2 * tu.BF16_MEAN_TOL * scale, key
            means.append(diff.mean() / scale)
        assert np.median(means) <= tu.BF16_MEDIAN_TOL


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_page_borders_and_first_tokens(name, dtype):
    """Prompts that end just before, on and just behind a page's last place, then decoded across the border; and
    requests decoded from their very first token."""
    from air_b200.engine.batch import Entry
    from air_b200.engine.engine import Engine, EngineConfig
    engine = Engine.from_folder(tu.model_folder(name), EngineConfig(dtype=dtype, page_tokens=16, max_tokens=1024,
                                                                    max_requests=4))
    for n in (15, 16, 17, 31, 33):
        toks = tu.tokens_for(name, n + 4, n)
        got = [engine.step([Entry("r", toks[:n], range(n))]).cpu().numpy()]
        got += [engine.step([Entry("r", [t], [0])]).cpu().numpy() for t in toks[n:]]
        engine.finish("r")
        tu.check({("r", p): row for p, row in enumerate(np.concatenate(got))}, name, {"r": toks}, dtype)
    toks = tu.tokens_for(name, 6, 99)
    got = np.concatenate([engine.step([Entry("s", [t], [0])]).cpu().numpy() for t in toks])
    tu.check({("s", p): row for p, row in enumerate(got)}, name, {"s": toks}, dtype)
    got = [engine.step([Entry("t", toks[:2], [0, 1])]).cpu().numpy()]
    got += [engine.step([Entry("t", [t], [0])]).cpu().numpy() for t in toks[2:]]
    tu.check({("t", p): row for p, row in enumerate(np.concatenate(got))}, name, {"t": toks}, dtype)
    engine.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding(name, dtype):
    """320 tokens one by one after a prompt of five, across twenty pages, windows and chunks (the decode steps replay
    a CUDA graph); pages that windows and chunks have left are back in the pool."""
    from air_b200.engine.batch import Entry
    from air_b200.engine.engine import Engine, EngineConfig
    toks = tu.tokens_for(name, 325, 7)
    engine = Engine.from_folder(tu.model_folder(name), EngineConfig(dtype=dtype, page_tokens=16, max_tokens=384,
                                                                    max_requests=2))
    got = [engine.step([Entry("r", toks[:5], range(5))]).cpu().numpy()]
    got += [engine.step([Entry("r", [t], [0])]).cpu().numpy() for t in toks[5:]]
    tu.check({("r", p): row for p, row in enumerate(np.concatenate(got))}, name, {"r": toks}, dtype)
    assert engine.graphs, "decode steps ran as a graph"
    held = [sum(p >= 0 for p in pages) for pages in engine.cache.sequences["r"].pages]
    assert min(held) < 21 and max(held) <= 21
    engine.check_status()


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_service(name):
    from air_b200 import GenerationConfig
    from air_b200.engine.engine import Engine, EngineConfig
    from air_b200.engine.service import InferenceService, SchedulerConfig
    engine = Engine.from_folder(tu.model_folder(name), EngineConfig(dtype="float32", page_tokens=16, max_tokens=1024,
                                                                    max_requests=4))
    svc = InferenceService(engine, SchedulerConfig(max_active_requests=4, prefill_quantum_tokens=5,
                                                   token_budget_per_cycle=12))
    prompts = [tu.tokens_for(name, n, 40 + n) for n in (1, 7, 33, 20, 3)]
    want = [tu.plain_greedy(name, p, 12) for p in prompts]
    got = svc.generate_cohort([(p, GenerationConfig(max_new_tokens=12, stop_on_eos=False)) for p in prompts])
    assert [r.tokens for r in got] == want
    assert engine.cache.free_pages() == engine.cache.num_pages
    engine.check_status()


def test_trace_runner_program_and_command_line(capsys):
    """bin/trace_run as a program on a Tomodra folder (the class is chosen by config.json), and the command line."""
    name = "B"
    streams = streams_for(name, 60, (40, 9))
    steps = util.trace_mixed(streams, seed=2, live=2)
    with tempfile.TemporaryDirectory() as out:
        util.run_trace_program(tu.model_folder(name), "float32", steps, util.peak_tokens(steps), out)
        got = util.collect(steps, out, tu.CONFIGS[name]["vocab"])
    tu.check(got, name, streams, "float32")
    from air_b200 import cli
    prompt = tu.tokens_for(name, 9, 70)
    assert cli.main(["cuda", tu.model_folder(name), ",".join(map(str, prompt)), "--tokens", "6", "--dtype", "float32",
                     "--no-stop-on-eos"]) == 0
    assert capsys.readouterr().out.strip() == ",".join(map(str, tu.plain_greedy(name, prompt, 6)))
