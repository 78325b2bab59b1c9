"""Bivizen on the GPU against the plain implementation (tests/plain/bivizen_plain.py, 64-bit): every mechanism
alone through its kernel, then whole models through Engine.step, the scheduler and the trace runner, in float32 and
bfloat16, for configurations that differ in every size and option (bivizen_util.CONFIGS)."""
import json
import tempfile

import numpy as np
import pytest
import torch

import bivizen_util as bu
import util
from plain import bivizen_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.ascontiguousarray(a)).to(device=DEV, dtype=dtype)


def i32(a):
    return torch.tensor(list(a), dtype=torch.int32, device=DEV)


# ----------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("taps,channels", [(4, 70), (2, 33), (1, 16), (7, 130), (13, 40)])
def test_short_convolution_with_state_over_portions(taps, channels):
    """Three requests of unequal length in one batch per step, portions of 1 to 40 tokens (shorter than the taps
    too), one slot used twice: the second request in it must not see the first one's inputs."""
    from air_b200.csrc import ops
    rng = np.random.default_rng(taps)
    w = rng.normal(0, 0.6, size=(channels, taps))
    lengths = {"a": 75, "b": 9, "c": 41}
    xs = {r: rng.normal(size=(n, channels)) for r, n in lengths.items()}
    want = {r: plain.silu(plain.short_conv(x, w)) for r, x in xs.items()}
    state = torch.full((3, channels, max(taps - 1, 1)), 7.0, device=DEV)[:, :, :taps - 1].contiguous()
    slot = {"a": 0, "b": 2, "c": 2}              # c takes b's slot after b has ended
    plan = [[("a", 1), ("b", 2)], [("a", 2), ("b", 1)], [("a", 40), ("b", 6)], [("a", 3), ("c", 1)],
            [("a", 29), ("c", 38)], [("c", 2)]]
    at = {r: 0 for r in lengths}
    for r in ("a", "b"):
        state[slot[r]].zero_()
    for step in plan:
        if any(r == "c" and at["c"] == 0 for r, _ in step):
            state[slot["c"]].zero_()
        rows = np.concatenate([xs[r][at[r]:at[r] + n] for r, n in step])
        wide = np.concatenate([rows, rng.normal(size=(rows.shape[0], 5))], axis=1)      # a band of a wider matrix
        q_start = np.cumsum([0] + [n for _, n in step])
        y = torch.empty((rows.shape[0], channels), device=DEV)
        ops.short_conv_silu(dev(wide)[:, :channels], dev(w), state, y, i32(q_start), i32(slot[r] for r, _ in step),
                            max(n for _, n in step))
        y = y.cpu().numpy()
        for (r, n), lo in zip(step, q_start):
            assert np.abs(y[lo:lo + n] - want[r][at[r]:at[r] + n]).max() < 2e-5, (r, at[r], n)
            at[r] += n
    assert at == lengths


def scan_inputs(rng, T, H, G, d, dv):
    return (rng.normal(size=(T, G * d)), rng.normal(size=(T, G * d)), rng.normal(size=(T, H * dv)))


@pytest.mark.parametrize("H,G,d,dv", [(4, 2, 24, 20), (1, 1, 64, 33), (2, 2, 130, 8), (3, 1, 16, 128), (2, 1, 600, 5)])
def test_delta_rule_scan(H, G, d, dv):
    """Against the plain recurrence: whole, and cut into portions of 1, 2, 17 and the rest (the state is carried), two
    requests in the batch, key sizes that are no powers of two and a value size that fills no block."""
    from air_b200.csrc import ops
    rng = np.random.default_rng(d)
    T = 70
    seqs = {}
    for r in range(2):
        q, k, v = scan_inputs(rng, T, H, G, d, dv)
        a, b = rng.normal(size=(T, H)) * 2, rng.normal(size=(T, H)) * 2
        seqs[r] = (q, k, v, a, b)
    a_log, dt_bias = rng.uniform(-2, 0.5, size=H), rng.normal(size=H)
    want = {}
    for r, (q, k, v, a, b) in seqs.items():
        qq = np.repeat(plain.unit(q.reshape(T, G, d)) * d ** -0.5, H // G, axis=1)
        kk = np.repeat(plain.unit(k.reshape(T, G, d)), H // G, axis=1)
        g = np.exp(-np.exp(a_log) * plain.softplus(a + dt_bias))
        want[r] = plain.delta_rule(qq, kk, v.reshape(T, H, dv), g, plain.sigmoid(b))
    for cuts in ([T], [1, 2, 17, T - 20]):
        state = torch.zeros((2, H, d, dv), device=DEV)
        at = 0
        for n in cuts:
            rows = [np.concatenate([seqs[r][i][at:at + n] for r in (1, 0)]) for i in range(5)]
            out = torch.empty((2 * n, H, dv), device=DEV)
            ops.linear_scan(ops.SCAN_DELTA, dev(rows[0]), dev(rows[1]), dev(rows[2]), dev(rows[3]), state, out,
                            i32([0, n, 2 * n]), i32([1, 0]), i32([1] * n + [0] * n), q_scale=d ** -0.5, beta=dev(rows[4]),
                            a_log=dev(a_log),
                            dt_bias=dev(dt_bias), unit=True)
            out = out.cpu().numpy()
            for j, r in enumerate((1, 0)):
                assert np.abs(out[j * n:(j + 1) * n] - want[r][at:at + n]).max() < 3e-5
            at += n


@pytest.mark.parametrize("H,d,dv,tau", [(2, 24, 40, 8.0), (1, 48, 20, 1.0), (3, 16, 16, 16.0), (1, 200, 70, 4.0)])
def test_gated_linear_attention_scan(H, d, dv, tau):
    from air_b200.csrc import ops
    rng = np.random.default_rng(dv)
    T = 90
    q, k, v = scan_inputs(rng, T, H, H, d, dv)
    z = rng.normal(1.0, 2.0, size=(T, H * d))
    alpha = plain.sigmoid(z) ** (1.0 / tau)
    want = plain.gated_linear_attention((q * d ** -0.5).reshape(T, H, d), k.reshape(T, H, d), v.reshape(T, H, dv),
                                        alpha.reshape(T, H, d))
    for cuts in ([T], [2, 1, 33, 16, T - 52]):
        state = torch.full((4, H, d, dv), 3.0, device=DEV)
        state[3].zero_()
        at = 0
        for n in cuts:
            out = torch.empty((n, H, dv), device=DEV)
            ops.linear_scan(ops.SCAN_GLA, dev(q[at:at + n]), dev(k[at:at + n]), dev(v[at:at + n]), dev(z[at:at + n]),
                            state, out, i32([0, n]), i32([3]), i32([3] * n), q_scale=d ** -0.5, tau=tau)
            assert np.abs(out.cpu().numpy() - want[at:at + n]).max() < 3e-5 * max(1.0, np.abs(want).max())
            at += n
        assert float(state[0].min()) == 3.0              # other requests' states are not touched


def test_gated_norm_feed_forward_activation_and_scaled_sum():
    from air_b200.csrc import ops
    rng = np.random.default_rng(5)
    T, H, dv, E, I = 13, 3, 20, 72, 48
    o, gate, w = rng.normal(size=(T, H, dv)), rng.normal(size=(T, H * dv)), rng.normal(1, 0.1, size=dv)
    out = torch.empty((T, H * dv), device=DEV)
    ops.gated_rmsnorm(dev(o), dev(gate), dev(w), 1e-5, out, i32([0] * T))
    want = plain.rms_norm(o, w, 1e-5).reshape(T, H * dv) * plain.silu(gate)
    assert np.abs(out.cpu().numpy() - want).max() < 1e-5
    g, u = rng.normal(size=(T, I)) * 3, rng.normal(size=(T, I)) * 3
    for block in (I, 16):
        gu = np.stack([g.reshape(T, I // block, block), u.reshape(T, I // block, block)], axis=2).reshape(T, 2 * I)
        act = torch.empty((T, I), device=DEV)
        ops.glu(dev(gu), act, block=block, alpha=1.702, limit=2.5, shift=1.0)
        gg, uu = np.minimum(g, 2.5), np.clip(u, -2.5, 2.5)
        assert np.abs(act.cpu().numpy() - gg * plain.sigmoid(1.702 * gg) * (uu + 1.0)).max() < 1e-5
    h, a, b = rng.normal(size=(T, E)), rng.normal(size=(T, E)), rng.normal(size=(T, E))
    sa, sb, wn = rng.normal(size=E), rng.normal(size=E), rng.normal(1, 0.1, size=E)
    x = h + sa * a + sb * b
    hd, out = dev(h), torch.empty((T, E), device=DEV)
    ops.scaled_norm(hd, [(dev(a), dev(sa)), (dev(b), dev(sb))], dev(wn), 1e-6, out)
    assert np.abs(hd.cpu().numpy() - x).max() < 1e-5 and np.abs(out.cpu().numpy() - plain.rms_norm(x, wn, 1e-6)).max() < 1e-5
    hd, rows = dev(h), i32([4, 0, 12])
    out = torch.empty((3, E), device=DEV)
    ops.scaled_norm(hd, [(dev(a), None)], dev(wn), 1e-6, out, rows=rows)
    assert np.abs(hd.cpu().numpy() - h).max() < 1e-6               # with rows the stream is left alone
    assert np.abs(out.cpu().numpy() - plain.rms_norm(h + a, wn, 1e-6)[[4, 0, 12]]).max() < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv,rot,cap", [(4, 2, 32, 16, 16, 14.0), (2, 1, 48, 80, 48, 0.0), (3, 3, 64, 64, 0, 25.0)])
def test_attention_finds_a_far_key(H, G, dk, dv, rot, cap, dtype):
    """One request of 300 tokens over pages of 16 that are scattered and listed out of order.  The last query is
    made to point at key 3 (its score stands out among 300; the cap, where there is one, is wide enough to let it),
    the one before it at key 250, and the values of those keys are large: a lost, shifted or wrongly rotated key shows at once.  In portions of 2, 61 and the rest, so that
    the last queries are rows of a prompt portion and, in a second pass, single tokens."""
    from air_b200.csrc import ops
    rng = np.random.default_rng(dk)
    T, P, scale, base = 300, 16, 0.2, 1000.0
    W = (H + G) * dk + G * dv + H
    proj = rng.normal(size=(T, W))
    k_cols = slice(H * dk, (H + G) * dk)
    bias = rng.normal(0, 0.1, size=W)
    bias[-H:] = 0.0
    for query, key in ((T - 1, 3), (T - 2, 250)):
        # the query, once rotated to its place, is six times the key as rotated to the key's place
        kk = (proj[key, k_cols] + bias[k_cols]).reshape(1, G, dk)
        qq = plain.rotate(np.repeat(kk, H // G, axis=1) * 6.0, [key - query], rot, base)
        proj[query, :H * dk] = qq.reshape(H * dk) - bias[:H * dk]
        proj[key, (H + G) * dk:(H + G) * dk + G * dv] = 25.0
    full = proj + bias
    q = plain.rotate(full[:, :H * dk].reshape(T, H, dk), np.arange(T), rot, base)
    k = plain.rotate(full[:, k_cols].reshape(T, G, dk), np.arange(T), rot, base)
    v = full[:, (H + G) * dk:(H + G) * dk + G * dv].reshape(T, G, dv)
    if dtype == torch.bfloat16:
        q, k, v = bu.bf16(q).astype(np.float64), bu.bf16(k).astype(np.float64), bu.bf16(v).astype(np.float64)
    gate = plain.sigmoid(full[:, -H:])
    want = plain.capped_attention(q, k, v, scale, cap) * gate[:, :, None]
    lost = plain.capped_attention(np.delete(q, 3, 0), np.delete(k, 3, 0), np.delete(v, 3, 0), scale, cap)
    assert np.abs(lost[-1] * gate[-1, :, None] - want[-1]).max() > 1.0          # the far key carries the answer

    pages = rng.permutation(40)[:-(-T // P)]
    table = torch.full((2, 64), -1, dtype=torch.int32, device=DEV)
    table[1, :len(pages)] = i32(pages)
    inv_freq = dev(base ** (-2.0 * np.arange(rot // 2) / rot)) if rot else None
    for cuts in ([2, 61, T - 63], [T - 2, 1, 1]):
        cache = torch.zeros((40, G * P * (dk + dv)), dtype=dtype, device=DEV)
        at = 0
        for n in cuts:
            pos, seq = i32(range(at, at + n)), i32([1] * n)
            qo = torch.empty((n, H, dk), dtype=dtype, device=DEV)
            go = torch.empty((n, H), device=DEV)
            ops.qkv_prepare(dev(proj[at:at + n]), dev(bias), inv_freq, pos, seq, table, qo, cache, G, dv, P, gate_out=go)
            out = torch.empty((n, H, dv), dtype=dtype, device=DEV)
            ops.paged_attention_ref(qo, cache, table, seq, pos, out, None, scale, softcap=cap, gate=go, kv_heads=G,
                                    page_tokens=P)
            got = out.float().cpu().numpy()
            tol = 2e-4 if dtype == torch.float32 else 0.15
            assert np.abs(got - want[at:at + n]).max() < tol, (at, n)
            at += n


def test_values_are_mixed_with_an_earlier_layers():
    from air_b200.csrc import ops
    rng = np.random.default_rng(8)
    T, H, G, dk, dv, P = 5, 2, 2, 16, 24, 16
    W = (H + G) * dk + G * dv
    table = i32([0, 1]).view(1, 2)
    proj1, proj2 = rng.normal(size=(T, W)), rng.normal(size=(T, W))
    cache = torch.zeros((2, G * P * (dk + dv)), device=DEV)
    first = torch.empty((T, G * dv), device=DEV)
    q = torch.empty((T, H, dk), device=DEV)
    pos, seq = i32(range(T)), i32([0] * T)
    ops.qkv_prepare(dev(proj1), None, None, pos, seq, table, q, cache, G, dv, P, v_first=first, v_mode=1)
    assert np.abs(first.cpu().numpy() - proj1[:, -G * dv:]).max() < 1e-6
    ops.qkv_prepare(dev(proj2), None, None, pos, seq, table, q, cache, G, dv, P, v_first=first, v_mode=2,
                    v_lambda=torch.tensor([0.25], device=DEV))
    values = cache[0, G * P * dk:].view(G, P, dv)[:, :T].permute(1, 0, 2).reshape(T, G * dv).cpu().numpy()
    assert np.abs(values - (0.75 * proj2[:, -G * dv:] + 0.25 * proj1[:, -G * dv:])).max() < 1e-6


# ----------------------------------------------------------------------------- whole models
LENGTHS = {"P": (1, 7, 33, 97, 150), "Q": (5, 40, 131, 64), "R": (2, 65, 150, 300), "S": (3, 50, 140)}


def streams_for(name, seed=0, lengths=None):
    return {f"{name}{i}": bu.tokens_for(name, n, seed + i) for i, n in enumerate(lengths or LENGTHS[name])}


def replay(name, dtype, steps, page_tokens=16, max_requests=4, peak_page=64):
    return util.replay(bu.model_folder(name), dtype, steps, max_tokens=util.peak_tokens(steps, page=peak_page),
                       page_tokens=page_tokens, max_requests=max_requests)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
def test_whole_prompts(name, dtype):
    streams = streams_for(name)
    got, _ = replay(name, dtype, util.trace_whole(streams))
    bu.check(got, name, streams, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
def test_prompt_then_token_by_token(name, dtype):
    streams = streams_for(name, 10)
    got, _ = replay(name, dtype, util.trace_bulk_tail(streams, tail=32))
    bu.check(got, name, streams, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
def test_portions_down_to_two_tokens(name, dtype):
    streams = streams_for(name, 20)
    got, _ = replay(name, dtype, util.trace_portions(streams))
    bu.check(got, name, streams, dtype)
    got, _ = replay(name, dtype, util.trace_portions(streams, sizes=(2, 2, 1, 3, 16, 15, 17, 64, 63, 65, 2)), page_tokens=64)
    bu.check(got, name, streams, dtype)


@pytest.mark.parametrize("page", [16, 64])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
def test_unequal_requests_together_with_pages_and_slots_used_again(name, dtype, page):
    """Ten requests through three state slots and a pool that holds the peak only: every request must come out as it
    does alone (the oracle runs each alone), whatever shared its batches and whoever had its slot and pages before."""
    lengths = LENGTHS[name] + (120, 2, 77, 101, 64, 129)
    streams = streams_for(name, 50, lengths)
    steps = util.trace_mixed(streams, seed=3, live=3)
    got, engine = replay(name, dtype, steps, page_tokens=page, max_requests=3)
    bu.check(got, name, streams, dtype)
    for group in engine.cache.groups:
        assert group.pool.takes > group.pool.num_pages, "pages were used again"


@pytest.mark.parametrize("name", ["random1", "random4", "random9", "random13", "tensorcore5", "tensorcore11"])
def test_configurations_drawn_at_random(name):
    """Layer orders, sizes and constants that nobody chose (bivizen_util.random_config): whole prompts and a mixed
    schedule through three slots, float32 within its tolerance; bfloat16 must agree with itself across schedules (its
    distance from the oracle depends on how a drawn model amplifies rounding)."""
    folder = bu.model_folder(name)
    streams = {f"{name}_{i}": bu.tokens_for(name, n, 80 + i) for i, n in enumerate((150, 3, 70, 1, 97))}
    whole = util.trace_whole(streams)
    mixed = util.trace_mixed(streams, seed=5, live=3, tail=20)
    got, _ = replay(name, "float32", whole, page_tokens=64)
    bu.check(got, name, streams, "float32")
    got, _ = replay(name, "float32", mixed, page_tokens=64, max_requests=3)
    bu.check(got, name, streams, "float32")
    a, _ = replay(name, "bfloat16", whole, page_tokens=64)
    b, _ = replay(name, "bfloat16", mixed, page_tokens=64, max_requests=3)
    for key, row in a.items():
        ref = bu.plain_logits(name, streams[key[0]])[key[1]]
        scale = max(1.0, float(np.abs(bu.plain_logits(name, streams[key[0]])).max()))
        assert np.isfinite(b[key]).all()
        assert np.abs(b[key] - row).max() <= max(2 * np.abs(row - ref).max(), 1e-2 * scale), key


@pytest.mark.parametrize("name", ["P", "R"])
def test_float32_does_not_depend_on_the_cut_or_the_batch(name):
    streams = streams_for(name, 30, (97, 40, 131))
    whole, _ = replay(name, "float32", util.trace_whole(streams))
    cut, _ = replay(name, "float32", util.trace_portions(streams, sizes=(2, 31, 1, 16, 5)))
    mixed, _ = replay(name, "float32", util.trace_mixed(streams, seed=1, live=3), max_requests=3)
    for key, row in whole.items():
        assert np.abs(cut[key] - row).max() < 2e-5
        assert np.abs(mixed[key] - row).max() < 2e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "R"])
def test_page_borders_and_first_tokens(name, dtype):
    """Prompts that end just before, on and just behind a page's last place, then decoded across the border; and
    requests decoded from their very first token."""
    from air_b200.engine.batch import Entry
    from air_b200.engine.engine import Engine, EngineConfig
    engine = Engine.from_folder(bu.model_folder(name), EngineConfig(dtype=dtype, page_tokens=16, max_tokens=1024,
                                                                    max_requests=4))
    tol = bu.FP32_TOL if dtype == "float32" else bu.BF16_MAX_TOL
    for n in (15, 16, 17, 31, 33):
        toks = bu.tokens_for(name, n + 4, n)
        want = bu.plain_logits(name, toks)
        got = [engine.step([Entry("r", toks[:n], range(n))]).cpu().numpy()]
        got += [engine.step([Entry("r", [t], [0])]).cpu().numpy() for t in toks[n:]]
        engine.finish("r")
        assert np.abs(np.concatenate(got) - want).max() < tol * max(1.0, np.abs(want).max()), n
    toks = bu.tokens_for(name, 6, 99)
    want = bu.plain_logits(name, toks)
    got = np.concatenate([engine.step([Entry("s", [t], [0])]).cpu().numpy() for t in toks])
    assert np.abs(got - want).max() < tol * max(1.0, np.abs(want).max())
    got = [engine.step([Entry("t", toks[:2], [0, 1])]).cpu().numpy()]
    got += [engine.step([Entry("t", [t], [0])]).cpu().numpy() for t in toks[2:]]
    assert np.abs(np.concatenate(got) - want).max() < tol * max(1.0, np.abs(want).max())
    engine.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["Q", "R"])
def test_long_decoding(name, dtype):
    """320 tokens one by one after a prompt of five, across twenty pages (the decode steps replay a CUDA graph)."""
    from air_b200.engine.batch import Entry
    from air_b200.engine.engine import Engine, EngineConfig
    toks = bu.tokens_for(name, 325, 7)
    want = bu.plain_logits(name, toks)
    engine = Engine.from_folder(bu.model_folder(name), EngineConfig(dtype=dtype, page_tokens=16, max_tokens=384,
                                                                    max_requests=2))
    got = [engine.step([Entry("r", toks[:5], range(5))]).cpu().numpy()]
    got += [engine.step([Entry("r", [t], [0])]).cpu().numpy() for t in toks[5:]]
    got = np.concatenate(got)
    scale = max(1.0, np.abs(want).max())
    if dtype == "float32":
        assert np.abs(got - want).max() < bu.FP32_TOL * scale
    else:
        assert np.abs(got - want).max() < bu.BF16_MAX_TOL * scale
        assert np.abs(got - want).mean(axis=1).max() < bu.BF16_MEAN_TOL * scale
    assert engine.graphs, "decode steps ran as a graph"
    engine.check_status()


@pytest.mark.parametrize("name", ["P", "S"])
def test_greedy_generation_through_the_service(name):
    from air_b200 import GenerationConfig
    from air_b200.engine.engine import Engine, EngineConfig
    from air_b200.engine.service import InferenceService, SchedulerConfig
    engine = Engine.from_folder(bu.model_folder(name), EngineConfig(dtype="float32", page_tokens=16, max_tokens=1024,
                                                                    max_requests=4))
    svc = InferenceService(engine, SchedulerConfig(max_active_requests=4, prefill_quantum_tokens=5,
                                                   token_budget_per_cycle=12))
    prompts = [bu.tokens_for(name, n, 40 + n) for n in (1, 7, 33, 20, 3)]
    want = [bu.plain_greedy(name, p, 12) for p in prompts]
    got = svc.generate_cohort([(p, GenerationConfig(max_new_tokens=12, stop_on_eos=False)) for p in prompts])
    assert [r.tokens for r in got] == want
    assert engine.cache.free_pages() == engine.cache.num_pages
    engine.check_status()


def test_trace_runner_program_and_command_line():
    """bin/trace_run as a program on a Bivizen folder: the class is chosen by config.json."""
    name = "Q"
    streams = streams_for(name, 60, (40, 9))
    steps = util.trace_mixed(streams, seed=2, live=2)
    with tempfile.TemporaryDirectory() as out:
        util.run_trace_program(bu.model_folder(name), "float32", steps, util.peak_tokens(steps), out)
        got = util.collect(steps, out, bu.CONFIGS[name]["vocab"])
    bu.check(got, name, streams, "float32")


def test_command_line_generates(capsys):
    from air_b200 import cli
    prompt = bu.tokens_for("Q", 9, 70)
    assert cli.main(["cuda", bu.model_folder("Q"), ",".join(map(str, prompt)), "--tokens", "6", "--dtype", "float32",
                     "--no-stop-on-eos"]) == 0
    assert capsys.readouterr().out.strip() == ",".join(map(str, bu.plain_greedy("Q", prompt, 6)))
