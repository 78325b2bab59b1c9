"""Tomodra without a GPU: its configuration and description, the cache manager's handling of chunks and of a latent
that several layers read, and the plain implementation's mechanisms against closed forms written here."""
import json

import numpy as np
import pytest

import tomodra_util as tu
from plain import tomodra_plain as plain


def test_config_round_trip_and_description():
    from air_b200.config import load_config, ConfigError
    from air_b200.parts import registry
    from air_b200.engine.model import Model
    for name, cfg in tu.CONFIGS.items():
        c = load_config(cfg)
        assert c.architecture == "Tomodra" and c.width == cfg["width"] and len(c.layers) == len(cfg["layers"])
        assert load_config(c.to_dict()) == c
        model = Model(registry.architecture(c.architecture).build_spec(c))
        names = {t.name: tuple(t.shape) for t in model.tensor_specs() if not t.optional}
        assert {n: a.shape for n, a in tu.draw_tensors(cfg, 0).items()} == names
    with pytest.raises(ConfigError):
        load_config(dict(tu.CONFIGS["B"], layers=[dict(type="conv", mixer={})]))
    with pytest.raises(ConfigError):
        load_config({k: v for k, v in tu.CONFIGS["B"].items() if k != "postln_alpha"})
    bad = json.loads(json.dumps(tu.CONFIGS["A"]))
    bad["layers"][2]["mixer"]["kv_from"] = 1            # layer 1 is no latent layer
    with pytest.raises(ConfigError):
        load_config(bad)
    bad = json.loads(json.dumps(tu.CONFIGS["A"]))
    bad["layers"][2]["mixer"]["kv_rank"] = 48           # the reader's latent must have the owner's size
    with pytest.raises(ConfigError):
        load_config(bad)
    bad = json.loads(json.dumps(tu.CONFIGS["A"]))
    bad["layers"][0]["mlp"]["router"]["top"] = 6        # of five experts
    with pytest.raises(ConfigError):
        load_config(bad)


def test_runs_that_read_another_layers_latent_and_how_long_pages_live():
    from air_b200.config import load_config
    from air_b200.parts import registry
    from air_b200.engine.model import Model
    from air_b200.parts.base import PagedKV, PagedLatent
    c = load_config(tu.CONFIGS["A"])
    spec = registry.architecture(c.architecture).build_spec(c)
    assert [r.cache_from for r in spec.order] == [None, None, 0, None, None]
    needs = Model(spec).cache_needs()
    # layer 0 looks back 48 tokens, layer 2 reads the same rows through a window of 70: the rows live for 70
    assert needs[0] == (PagedLatent(48, 70),) and needs[2] == ()
    assert needs[1] == (PagedKV(2, 32, None, 16, 40),) and needs[3] == (PagedLatent(28, 17),)
    assert "feed_forward" not in spec.layers[2].parts and "feed_forward_norm" not in spec.layers[2].parts
    assert spec.layers[3].parts["feed_forward"]["shared_intermediate"] == 0
    # a chunk's pages go back once the request has left the chunk; a window's as it passes
    assert PagedKV(2, 32, None, 16, 40).first_live(79) == 40 and PagedKV(2, 32, None, 16, 40).first_live(80) == 80
    assert PagedLatent(48, 70).first_live(100) == 31 and PagedLatent(48, None).first_live(100) == 0


def test_cache_gives_back_the_pages_of_chunks_that_are_over():
    from air_b200.cache.manager import CacheManager
    from air_b200.parts.base import PagedKV, PagedLatent
    m = CacheManager([(PagedKV(1, 16, None, None, 40),), (PagedLatent(24, 20),)], 16, 12, 2, allocate=False)
    m.open("r")
    for n in (30, 9, 1, 45, 3):          # lengths 30, 39, 40, 85, 88
        m.reserve([("r", n)])
        m.commit("r", n)
        length = m.length("r")
        chunk_pages, window_pages = m.sequences["r"].pages
        first_chunk = (length - length % 40) // 16
        assert all((p < 0) == (b < first_chunk) for b, p in enumerate(chunk_pages)), (length, chunk_pages)
        first_window = max(0, length - 19) // 16
        assert all((p < 0) == (b < first_window) for b, p in enumerate(window_pages)), (length, window_pages)
        m.check()
    m.close("r")
    assert m.free_pages() == 12


def test_stretched_frequencies_match_the_plain_rule():
    from air_b200.parts.rope import bent_frequencies
    for dims, base, sc in ((64, 10000.0, (8.0, 1024, 32.0, 1.0)), (16, 5000.0, (4.0, 64, 16.0, 2.0)),
                           (8, 1e5, (16.0, 32, 8.0, 1.0)), (12, 1e4, None), (48, 500.0, (2.0, 4096, 1.0, 1.0))):
        scaling = dict(zip(("factor", "original", "fast", "slow"), sc)) if sc else None
        f, mag = bent_frequencies(dims, base, scaling)
        want, want_mag = plain.yarn_frequencies(dims, base, scaling)
        assert np.abs(f.numpy() - want).max() <= 1e-15 * want.max() and abs(mag - want_mag) < 1e-15
    f, _ = plain.yarn_frequencies(64, 10000.0, dict(factor=8.0, original=1024, fast=32.0, slow=1.0))
    g = plain.plain_frequencies(64, 10000.0)
    assert f[0] == g[0] and abs(f[-1] - g[-1] / 8.0) < 1e-18 and np.all(np.diff(f / g) <= 1e-12)


def test_plain_mechanisms_against_closed_forms():
    rng = np.random.default_rng(0)
    # a rotation by the key's angle and back: q.k depends on the distance only, for both pairings
    x, y = rng.normal(size=(1, 1, 8)), rng.normal(size=(1, 1, 8))
    f = plain.plain_frequencies(6, 100.0)
    for rotate in (plain.rotate_half_split, plain.rotate_neighbours):
        a = (rotate(x, np.array([7]), f, 6) * rotate(y, np.array([3]), f, 6)).sum()
        b = (rotate(x, np.array([104]), f, 6) * rotate(y, np.array([100]), f, 6)).sum()
        assert abs(a - b) < 1e-9
        assert np.array_equal(rotate(x, np.array([5]), f, 6)[..., 6:], x[..., 6:])        # the rest passes
    assert plain.rotate_neighbours(np.array([[[1.0, 0.0]]]), np.array([1]), np.array([np.pi / 2]), 2)[0, 0, 1] == pytest.approx(1.0)
    # masks
    w, c = plain.window_mask(10, 3), plain.chunk_mask(10, 4)
    assert w[5].tolist() == [False] * 3 + [True] * 3 + [False] * 4 and c[5].tolist() == [False] * 4 + [True] * 2 + [False] * 4
    assert c[4].sum() == 1 and c[7].sum() == 4 and w[0].sum() == 1
    # a sink as large as the only score takes half of the weight
    p = plain.masked_softmax(np.full((1, 1, 1), 2.0), np.ones((1, 1), dtype=bool), sink=np.array([2.0]))
    assert p[0, 0, 0] == pytest.approx(0.5)
    # the weight goes into the expert, not behind it
    w = {"e0.gate": rng.normal(size=(5, 4)), "e0.up": rng.normal(size=(5, 4)), "e0.down": rng.normal(size=(4, 5)),
         "router": np.array([[10.0, 0, 0, 0]])}
    u = np.array([[0.05, 1.0, -2.0, 0.5]])
    s = plain.sigmoid(0.5)
    y = plain.mixture(u, w, "", dict(router=dict(experts=1, top=1)))
    assert np.allclose(y, plain.expert(s * u, w, "e0.")) and not np.allclose(y, s * plain.expert(u, w, "e0."))
