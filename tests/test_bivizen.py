"""Bivizen without a GPU: its configuration and description, and the plain implementation's mechanisms against
closed forms written here."""
import json
import os

import numpy as np
import pytest

import bivizen_util as bu
from plain import bivizen_plain as plain


def test_config_round_trip_and_description():
    from air_b200.config import load_config, ConfigError
    from air_b200.parts import registry
    from air_b200.engine.model import Model
    for name, cfg in bu.CONFIGS.items():
        c = load_config(cfg)
        assert c.architecture == "Bivizen" and c.width == cfg["width"] and len(c.layers) == len(cfg["layers"])
        again = load_config(c.to_dict())
        assert again == c
        spec = registry.architecture(c.architecture).build_spec(c)
        model = Model(spec)
        names = {t.name: tuple(t.shape) for t in model.tensor_specs() if not t.optional}
        assert {n: a.shape for n, a in bu.draw_tensors(cfg, 0).items()} == names
    with pytest.raises(ConfigError):
        load_config(dict(bu.CONFIGS["Q"], layers=[dict(type="conv", mixer={})]))
    with pytest.raises(ConfigError):
        load_config({k: v for k, v in bu.CONFIGS["Q"].items() if k != "norm"})
    bad = json.loads(json.dumps(bu.CONFIGS["Q"]))
    bad["layers"][2]["mixer"]["kv_heads"] = 4          # 6 heads over 4
    with pytest.raises(ConfigError):
        load_config(bad)


def test_value_mixing_is_first_then_mix_and_the_feed_forward_may_be_absent():
    from air_b200.config import load_config
    from air_b200.parts import registry
    c = load_config(bu.CONFIGS["P"])
    spec = registry.architecture(c.architecture).build_spec(c)
    kinds = [(b.parts["mixer"].kind, b.parts["mixer"].get("v_mix")) for b in spec.layers]
    assert kinds == [("gated_delta", None), ("capped_attention", "first"), ("gla", None), ("capped_attention", "mix"),
                     ("capped_attention", None)]
    assert "feed_forward" not in spec.layers[2].parts
    from air_b200.engine.model import Model
    idle = [t for t in Model(spec).tensor_specs() if t.optional]
    assert [t.name for t in idle] == ["l2.ls2"]        # a scale for a feed-forward that is not there may be in the file
    assert spec.layers[4].parts["mixer"]["position"].params["rotary_dim"] == 48


def test_rank_of_the_decay_projection_comes_from_the_file(tmp_path):
    """config.json need not name it: the shape of the tensor does."""
    from air_b200.config import load_config, ConfigError
    folder = bu.model_folder("Q")
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    del cfg["layers"][0]["mixer"]["rank"]
    with pytest.raises(ConfigError):
        load_config(cfg)
    other = tmp_path / "m"
    other.mkdir()
    (other / "config.json").write_text(json.dumps(cfg))
    os.symlink(os.path.join(folder, "model.safetensors"), other / "model.safetensors")
    assert load_config(str(other)).layers[0].rank == 4


def test_command_line_inspects_and_writes_a_bivizen_folder(tmp_path, capsys):
    from air_b200 import cli
    assert cli.main(["inspect", bu.model_folder("Q")]) == 0
    shown = json.loads(capsys.readouterr().out)
    assert shown["architecture"] == "Bivizen" and shown["config"]["layers"][1]["mixer"]["conv"] == 2
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(bu.CONFIGS["S"]))
    assert cli.main(["random", str(cfg), str(tmp_path / "model"), "--seed", "3"]) == 0
    capsys.readouterr()
    assert cli.main(["inspect", str(tmp_path / "model"), "--tensors"]) == 0
    assert "l0.mix.vmix\t[]" in capsys.readouterr().out
    config, tensors = plain.read_model(str(tmp_path / "model"))          # the oracle reads what the engine wrote
    assert np.isfinite(plain.forward(config, tensors, [1, 2, 3])).all()


# ----------------------------------------------------------------------------- the oracle's mechanisms
def test_plain_short_conv_is_a_causal_correlation():
    rng = np.random.default_rng(0)
    x, w = rng.normal(size=(9, 3)), rng.normal(size=(3, 4))
    y = plain.short_conv(x, w)
    for c in range(3):
        padded = np.concatenate([np.zeros(3), x[:, c]])
        want = [np.dot(padded[t:t + 4], w[c]) for t in range(9)]
        assert np.allclose(y[:, c], want)


def test_plain_gated_linear_attention_is_its_sum_over_the_past():
    rng = np.random.default_rng(1)
    T, H, d, dv = 7, 2, 3, 4
    q, k, v = rng.normal(size=(T, H, d)), rng.normal(size=(T, H, d)), rng.normal(size=(T, H, dv))
    alpha = rng.uniform(0.2, 1.0, size=(T, H, d))
    o = plain.gated_linear_attention(q, k, v, alpha)
    for t in range(T):
        for h in range(H):
            want = np.zeros(dv)
            for s in range(t + 1):
                decay = np.prod(alpha[s + 1:t + 1, h], axis=0)
                want += np.dot(q[t, h] * decay, k[s, h]) * v[s, h]
            assert np.allclose(o[t, h], want)


def test_plain_delta_rule_stores_and_replaces():
    """With beta = 1, no decay and orthonormal keys the state is a table: a key reads back the value written last."""
    d, dv = 4, 3
    keys = np.eye(d)
    seq = [0, 1, 2, 1, 3, 0]
    rng = np.random.default_rng(2)
    v = rng.normal(size=(len(seq), 1, dv))
    k = keys[seq][:, None, :]
    ones = np.ones((len(seq), 1))
    o = plain.delta_rule(k.copy(), k, v, ones, ones)
    assert np.allclose(o, v)                     # the read-out sees the current token's write
    probe = plain.delta_rule(np.concatenate([k, keys[[1]][:, None, :]]), np.concatenate([k, np.zeros((1, 1, d))]),
                             np.concatenate([v, np.zeros((1, 1, dv))]), np.ones((len(seq) + 1, 1)),
                             np.ones((len(seq) + 1, 1)))
    assert np.allclose(probe[-1, 0], v[3, 0])    # key 1 holds its second value, not the first
    half = plain.delta_rule(k.copy(), k, v, 0.5 * ones, ones)
    assert np.allclose(half[3, 0], v[3, 0])      # a decayed state is still overwritten completely when beta = 1


def test_plain_rotation_and_cap():
    x = np.arange(16, dtype=np.float64).reshape(1, 2, 8)
    y = plain.rotate(np.repeat(x, 3, axis=0), [0, 1, 5], 4, 100.0)
    assert np.allclose(y[0], x[0])                                    # position 0 rotates nothing
    assert np.allclose(y[:, :, 4:], x[:, :, 4:])                      # the rest of the head passes
    a = 5 * 100.0 ** (-2.0 * 1 / 4)
    assert np.allclose(y[2, 0, [1, 3]], [1 * np.cos(a) - 3 * np.sin(a), 3 * np.cos(a) + 1 * np.sin(a)])
    q = np.array([[[40.0, 0.0]], [[40.0, 0.0]]])
    k = np.array([[[1.0, 0.0]], [[-1.0, 0.0]]])
    v = np.array([[[1.0]], [[0.0]]])
    o = plain.capped_attention(q, k, v, 1.0, 2.0)                      # scores +-40 are capped to about +-2
    assert np.allclose(o[1, 0, 0], 1.0 / (1.0 + np.exp(-4.0)), atol=1e-6)


def test_plain_model_depends_on_every_option():
    """Dropping a mechanism from the oracle's input moves the logits far beyond the tests' tolerances: the test
    models are made so that it shows."""
    cfg, tensors = bu.plain_model("P")
    toks = bu.tokens_for("P", 60, 1)
    ref = plain.forward(cfg, tensors, toks)
    scale = np.abs(ref).max()

    def moved(change):
        c, t = json.loads(json.dumps(cfg)), dict(tensors)
        change(c, t)
        return np.abs(plain.forward(c, t, toks) - ref).max() / scale

    # (the float32 tests allow 5e-5 of the scale, the bfloat16 tests 5e-2)
    assert moved(lambda c, t: c["layers"][1]["mixer"].pop("rot")) > 0.05
    assert moved(lambda c, t: c["layers"][1]["mixer"].update(softcap=0.0)) > 0.005
    assert moved(lambda c, t: c["layers"][3]["mixer"].update(v_mix=False)) > 0.1
    assert moved(lambda c, t: t.update({"l0.mix.q.conv": np.roll(t["l0.mix.q.conv"], 1, axis=1)})) > 0.1
    assert moved(lambda c, t: t.update({"l2.mix.a2.b": t["l2.mix.a2.b"] + 3.0})) > 0.1
    assert moved(lambda c, t: t.update({"l1.ls2": np.ones_like(t["l1.ls2"])})) > 0.1
    assert moved(lambda c, t: c["layers"][0]["mlp"].update(limit=50.0)) > 0.1
