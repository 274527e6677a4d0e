"""Supevik without a GPU: the configuration reader, the order of layer runs, the tensors the
specification asks for, and the rotation's frequency table against the plain implementation."""
import json

import pytest
import torch

import plain_supevik as plain
import supevik_util as U


def parse(cfg):
    import moe_b200

    arch, typed = moe_b200.parse_config(cfg)
    return arch, typed, arch.model_spec(typed)


@pytest.mark.parametrize("name", sorted(U.CONFIGS))
def test_the_specification_asks_for_exactly_the_checkpoints_tensors(name):
    from moe_b200.models.decoder import expected_tensors

    cfg = U.config_dict(name)
    arch, typed, spec = parse(cfg)
    assert arch.name == "Supevik"
    want = {n: tuple(t.shape) for n, t in U.draw_weights(cfg, 1).items()}
    got = {n: tuple(ts.shape) for n, ts in expected_tensors(spec).items()}
    assert got == want


@pytest.mark.parametrize("name", sorted(U.CONFIGS))
def test_layers_run_in_the_plain_order_each_run_with_a_cache_of_its_own(name):
    cfg = U.config_dict(name)
    _, typed, spec = parse(cfg)
    order = plain.layer_order(cfg)
    assert [(e.layer, e.join is not None) for e in spec.schedule] == order
    assert [e.cache for e in spec.schedule] == list(range(len(order)))
    assert all(e.writes_cache for e in spec.schedule)
    assert len(spec.joins) == (1 if cfg.get("loop") else 0)


def test_the_order_of_a_loop_in_the_middle():
    cfg = U.config_dict("loop3")
    assert [l for l, _ in plain.layer_order(cfg)] == [0, 1, 2, 1, 2, 1, 2, 3]
    _, typed, _ = parse(cfg)
    assert typed.run_order() == [(0, False), (1, True), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]


def test_config_round_trip_and_what_is_read_from_it():
    cfg = U.config_dict("loop3")
    arch, typed, spec = parse(cfg)
    assert arch.config_dict(typed) == cfg
    assert typed.layers[1].mlp is None and typed.layers[2].mixer.rot_scaling is None
    assert typed.layers[2].mixer.window == 21 and typed.layers[0].mixer.rot_scaling.factor == 4.0
    m = spec.layers[2].mixer.params
    assert (m["num_heads"], m["num_kv_heads"], m["head_dim"], m["value_dim"]) == (2, 2, 48, 16)
    assert m["position"]["kind"] == "rotary" and spec.layers[0].mixer.params["position"]["kind"] == "rotary_yarn"
    assert spec.layers[1].ffn is None and spec.layers[1].post2 is None and spec.layers[0].post2 is not None
    assert spec.embedding.params["scale"] == 5.0
    # a typed configuration built by hand writes the same keys
    from moe_b200.config.supevik import SupevikConfig

    again = SupevikConfig(typed.vocab, typed.width, typed.embedding_scale, typed.norm_eps, typed.layers, typed.loop)
    assert json.loads(json.dumps(again.to_dict())) == cfg


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown mixer type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "unknown kind"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=34), "at most dim"),
    (lambda c: c["loop"].update(stop=9), "delimit"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "vdim"),
])
def test_a_configuration_that_cannot_be_a_model_is_refused_in_words(edit, word):
    from moe_b200 import ConfigError

    cfg = U.config_dict("loop3")
    edit(cfg)
    with pytest.raises(ConfigError, match=word):
        parse(cfg)


@pytest.mark.parametrize("rot", [
    {"dims": 16, "base": 10000.0, "scaling": U.YARN},
    {"dims": 64, "base": 250000.0, "scaling": {"factor": 6.0, "original": 2048, "fast": 24.0, "slow": 1.5}},
    {"dims": 8, "base": 100.0, "scaling": {"factor": 1.5, "original": 64, "fast": 16.0, "slow": 2.0}},
    {"dims": 32, "base": 10000.0, "scaling": {"factor": 2.0, "original": 16, "fast": 1.0, "slow": 1.0}},   # lo == hi
])
def test_yarn_frequencies_and_factor(rot):
    from moe_b200.config.spec import PartSpec
    from moe_b200.parts.base import make_part

    s = rot["scaling"]
    part = make_part("position", PartSpec("rotary_yarn", dict(theta=rot["base"], rotary_dim=rot["dims"], **s)))
    f, m = plain.yarn_frequencies(rot)
    assert torch.allclose(part.frequencies().double(), f, rtol=1e-6, atol=0)
    assert abs(part.cos_sin_scale() - m) < 1e-12
    # the ramp really has both ends in the first two tables
    base = rot["base"] ** (-2.0 * torch.arange(rot["dims"] // 2, dtype=torch.float64) / rot["dims"])
    assert torch.all(f <= base * (1 + 1e-12)) and torch.all(f >= base / s["factor"] * (1 - 1e-12))


def test_record_width():
    from moe_b200.parts.attention import record_width

    assert record_width(80, 72, True) == 128 and record_width(32, 16, True) == 64 and record_width(64, 64, True) == 64
    assert record_width(16, 160, True) == 160 and record_width(40, 24, False) == 48 and record_width(80, 72, False) == 80


def test_the_plain_windowed_attention_sees_exactly_the_window():
    """The oracle's own mask, by hand: with a window of 3, query 5 sees keys 3, 4, 5."""
    T, d = 8, 4
    q = torch.zeros(T, 1, d, dtype=torch.float64)
    k = torch.zeros(T, 1, d, dtype=torch.float64)
    v = torch.eye(T, dtype=torch.float64).reshape(T, 1, T)
    out = plain.windowed_softmax_attention(q, k, v, 1.0, 3)
    assert torch.allclose(out[5, 0], torch.tensor([0, 0, 0, 1, 1, 1, 0, 0], dtype=torch.float64) / 3)
    assert torch.allclose(out[1, 0], torch.tensor([1, 1, 0, 0, 0, 0, 0, 0], dtype=torch.float64) / 2)
    out = plain.windowed_softmax_attention(q, k, v, 1.0, None)
    assert torch.allclose(out[5, 0], torch.tensor([1, 1, 1, 1, 1, 1, 0, 0], dtype=torch.float64) / 6)


def test_info_prints_a_supevik_folder_in_the_words_of_its_parts(tmp_path, capsys):
    from moe_b200 import cli

    d = U.model_folder(tmp_path, "loop3")
    assert cli.main(["info", d, "--dtype", "float32"]) == 0
    out = capsys.readouterr().out
    assert "Supevik" in out and "layers 4  hidden 64  vocab 131" in out
    assert "schedule   0 +1 2 +1[cache 3] 2[cache 4] +1[cache 5] 2[cache 6] 3[cache 7]" in out
    assert "token embedding x 5" in out and "join with the embedding output" in out
    assert "Dynamic Tanh" in out and "sigmoid output gate" in out and "window 21" in out and "YaRN x4 from 64" in out
    assert "dense gated gelu_tanh 96   (2 of 3)" in out and "value heads of 16" in out


def test_bytes_of_a_decode_step_count_every_layer_run_and_every_join(tmp_path):
    import moe_b200
    from moe_b200 import cli

    d = U.model_folder(tmp_path, "loop3")
    m = moe_b200.load_model(d, dtype="float32", device="cpu")
    w = U.draw_weights(U.config_dict("loop3"), 11)
    per_layer = [sum(t.numel() for n, t in w.items() if n.startswith(f"l{i}.")) for i in range(4)]
    runs = [0, 1, 2, 1, 2, 1, 2, 3]
    want = sum(per_layer[l] for l in runs) + 3 * w["loop.in"].numel() + w["head"].numel() + 2 * 64 + 1 + 2 * 64
    got, kv = cli.step_bytes(m, [30, 30])
    assert got == 4 * want
    # windows of 7, 7, 21, 7 bound what the eight runs read: records of 32, 32, 48 and 32 floats for keys and for values
    per_pos = {0: 2 * 2 * 32, 1: 2 * 1 * 32, 2: 2 * 2 * 48, 3: 2 * 2 * 32}
    assert kv == 4 * 2 * sum(per_pos[l] * (21 if l == 2 else 7) for l in runs)
