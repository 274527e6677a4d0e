"""Fogapel without a GPU: the configuration reader, the translation into parts, the tensor names
and shapes against the tests' own checkpoints, and the plain implementation's own consistency (a
whole sequence against the same sequence with the state carried by hand)."""
import json

import pytest
import torch

import fogapel_util as U
import plain_fogapel as plain


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return tmp_path_factory.mktemp("fogapel_cpu")


@pytest.mark.parametrize("name", sorted(U.CONFIGS))
def test_config_parts_and_tensor_names_fit_the_checkpoint(root, name):
    from moe_b200.config import parse_config, read_config_json
    from moe_b200.models.decoder import expected_tensors
    from moe_b200.weights import SafetensorsStore

    d = U.model_folder(root, name)
    arch, typed = parse_config(read_config_json(d))
    assert arch.name == "Fogapel"
    spec = arch.model_spec(typed)
    store = SafetensorsStore(d)
    store.check({n: ts.shape for n, ts in expected_tensors(spec, store).items()}, spec.ignorable)
    assert [l.block for l in spec.layers] == ["parallel"] * len(typed.layers)
    assert typed.to_dict() == json.load(open(d + "/config.json"))
    for L, ls in zip(typed.layers, spec.layers):
        assert ls.mixer.kind == {"attention": "gqa_attention", "wkv": "wkv"}[L.type]
        assert (ls.ffn is None) == (L.mlp is None) and (ls.scale2 is None) == (L.mlp is None)


def test_a_config_written_from_the_typed_form_reads_back_the_same():
    from moe_b200.config.fogapel import FogapelConfig

    for name in U.CONFIGS:
        typed = FogapelConfig.from_dict(U.config_dict(name))
        again = FogapelConfig.from_dict(FogapelConfig(typed.vocab, typed.width, typed.embedding_scale, typed.norm_eps,
                                                      typed.layers).to_dict())
        assert again.layers == typed.layers and again.vocab == typed.vocab


@pytest.mark.parametrize("bad,word", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown mixer type"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "not a multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "exceeds"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "unknown kind"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_config_errors_say_what_is_wrong(bad, word):
    from moe_b200.config import ConfigError, parse_config

    cfg = U.config_dict("mix")
    bad(cfg)
    with pytest.raises(ConfigError) as e:
        parse_config(cfg)
    assert word in str(e.value)


def test_a_decay_projection_of_another_width_is_read_from_the_tensors(root):
    """The width of the recurrent mixer's narrow projection stands in no configuration: 5 here, 3
    and 1 elsewhere; a checkpoint whose two projections disagree is refused by the shape check."""
    from moe_b200.config import parse_config, read_config_json
    from moe_b200.models.decoder import expected_tensors
    from moe_b200.weights import SafetensorsStore, TensorDictStore, WeightError

    d = U.model_folder(root, "mix")
    arch, typed = parse_config(read_config_json(d))
    spec = arch.model_spec(typed)
    store = SafetensorsStore(d)
    assert store.shape("l1.mix.w1") == (5, 64) and store.shape("l1.mix.w2") == (64, 5)
    t = {n: store.raw(n) for n in store.names()}
    t["l1.mix.w2"] = torch.zeros(63, 5)
    with pytest.raises(WeightError):
        bad = TensorDictStore(t)
        bad.check({n: ts.shape for n, ts in expected_tensors(spec, bad).items()}, spec.ignorable)


def test_plain_recurrent_mixer_and_convolution_do_not_depend_on_where_a_sequence_is_cut(root):
    """The plain implementation runs whole sequences only; its recurrences restated with the state
    carried by hand give the same numbers, which is what the library's cuts are compared to."""
    cfg, w = plain.read_model(U.model_folder(root, "mix"))
    g = torch.Generator().manual_seed(3)
    n = torch.randn(30, cfg["width"], generator=g, dtype=torch.float64)
    whole = plain.short_convolution(n, w["l0.mix.q.conv"][:64])
    taps = w["l0.mix.q.conv"].shape[1]
    again = torch.cat([plain.short_convolution(torch.cat([n[max(0, a - taps + 1):a], n[a:b]]), w["l0.mix.q.conv"][:64])[-(b - a):]
                       for a, b in ((0, 1), (1, 3), (3, 30))])
    assert (whole - again).abs().max() < 1e-12
    first = plain.wkv_mixer(w, "l1.mix", cfg["layers"][1]["mixer"], n, 1e-5)
    assert first.shape == (30, cfg["width"]) and torch.isfinite(first).all()
    # a token's output depends on no later token
    shorter = plain.wkv_mixer(w, "l1.mix", cfg["layers"][1]["mixer"], n[:17], 1e-5)
    assert (first[:17] - shorter).abs().max() < 1e-12
