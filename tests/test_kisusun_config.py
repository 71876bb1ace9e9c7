"""Kisusun's configuration reader and what the model asks of the cache manager (no GPU)."""
import copy

import pytest
import torch

import sparseengine_b200.models  # noqa: F401
from sparseengine_b200.config.registry import load_model_spec
from sparseengine_b200.engine.model import Model


def mixer(**kw):
    m = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 8, "scale": 0.2, "softcap": 12.0, "mask": {"size": 10},
         "rot": {"base": 1000.0, "dims": 8, "scaling": {"factor": 2.0}}, "v_mix": True}
    m.update(kw)
    return m


MOE = {"kind": "moe", "expert": {"ff": 24, "limit": 1.5}, "shared": {"ff": 40, "limit": 2.5},
       "router": {"experts": 6, "top": 2, "scale": 1.7, "groups": {"count": 3, "keep": 2}}}
CFG = {
    "architecture": "Kisusun", "vocab": 100, "width": 64, "logit_scale": 0.25, "embedding": {"scale": 4.0}, "norm": {"eps": 1e-4},
    "layers": [
        {"type": "attention", "mixer": mixer(v_mix=False), "mlp": {"kind": "dense", "ff": 128}},
        {"type": "attention", "mixer": mixer(), "mlp": MOE},
        {"type": "attention", "mixer": mixer(mask={"size": 7}), "mlp": None},
    ],
}


def test_the_configuration_becomes_parts_with_its_own_constants():
    _, spec = load_model_spec(copy.deepcopy(CFG))
    assert spec.architecture == "Kisusun" and spec.residual_stream == "float32"
    assert (spec.embed_scale, spec.logit_scale, spec.vocab_size, spec.head_source) == (4.0, 0.25, 100, None)
    a, b, c = (ls.mixer for ls in spec.layers)
    assert (a.kind, a.prep, a.v_head_dim, a.scale, a.score_softcap, a.sink, a.output_gate, a.window) == \
        ("attention", "general", 8, 0.2, 12.0, "zero", True, 10)
    assert (a.qk_norm, a.qk_norm_eps) == ("whole_projection", 1e-4)
    assert (a.position.rotary_dim, a.position.theta, a.position.pairing, dict(a.position.frequency_scaling)["factor"]) == \
        (8, 1000.0, "split_half", 2.0)
    # the first layer that blends keeps its values; the later ones blend with them
    assert (a.value_mix, b.value_mix, c.value_mix, c.window) == (None, "first", "blend", 7)
    d, m, none = (ls.feed_forward for ls in spec.layers)
    assert none is None and spec.layers[2].feed_forward_norm is None
    assert (d.kind, d.intermediate_size, d.activation) == ("dense_mlp", 128, "silu")
    assert (m.num_experts, m.top_k, m.intermediate_size, m.score_fn, m.renormalize, m.routed_scale, m.groups, m.keep_groups) == \
        (6, 2, 24, "sigmoid", False, 1.7, 3, 2)
    assert (m.activation, m.activation_limit, m.activation_alpha) == ("clamped_swiglu", 1.5, 1.702)
    assert (m.shared.intermediate_size, m.shared.activation_limit) == (40, 2.5)
    assert all(ls.arrangement == "sublayer_norm" and ls.mixer_norm.eps == 1e-4 for ls in spec.layers)


def test_cache_needs_and_parameters():
    _, spec = load_model_spec(copy.deepcopy(CFG))
    m = Model(spec, torch.bfloat16)
    reqs = [(r.num_kv_heads, r.head_dim, r.value_dim, n) for r, n in m.layout.groups]
    assert sorted(reqs) == [(2, 16, 8, 1), (2, 16, 8, 2)] or reqs == [(2, 16, 8, 3)]      # windows 10, 10 and 7
    assert not m.layout.states
    names = {s.name for p in m.params() for s in p.sources}
    assert {"embed", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q.norm", "l0.mix.k.norm", "l0.mix.g", "l1.mix.vmix", "l2.mix.vmix",
            "l1.mlp.router", "l1.mlp.e5.down", "l1.mlp.shared.up", "l0.mlp.gate"} <= names
    assert not {"head", "l0.mix.vmix", "l2.norm2"} & names
    shapes = {p.qualified: tuple(p.spec.shape) for p in m.params()}
    assert shapes["layers.0.mixer.qkv"] == (4 * 16 + 2 * 16 + 2 * 8 + 4 * 8, 64)      # queries, keys, values, gate
    assert shapes["layers.0.mixer.o"] == (64, 4 * 8)
    assert shapes["layers.1.feed_forward.w13"] == (6, 48, 64) and shapes["layers.1.feed_forward.shared_w13"] == (1, 80, 64)


def test_defaults_where_the_configuration_is_silent():
    cfg = copy.deepcopy(CFG)
    m = cfg["layers"][1]["mixer"]
    for key in ("kv_heads", "vdim", "softcap", "mask", "rot", "scale"):
        m.pop(key)
    cfg["layers"][1]["mlp"]["router"].pop("groups")
    cfg["layers"][1]["mlp"].pop("shared")
    _, spec = load_model_spec(cfg)
    a, f = spec.layers[1].mixer, spec.layers[1].feed_forward
    assert (a.num_kv_heads, a.v_head_dim, a.score_softcap, a.window, a.position, a.scale) == (4, 16, None, None, None, 0.25)
    assert (f.groups, f.shared) == (1, None)


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][0].update(type="convolution"), "unknown mixer type"),
    (lambda c: c["layers"][0]["mixer"].pop("dim"), "missing mixer keys"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple of 'kv_heads'"),
    (lambda c: c["layers"][0]["mixer"]["rot"].pop("base"), "'rot' needs"),
    (lambda c: c["layers"][0]["mlp"].update(kind="conv"), "kind must be"),
    (lambda c: c["layers"][1]["mlp"]["expert"].pop("limit"), "moe feed-forward needs"),
    (lambda c: c["layers"][1]["mlp"]["shared"].pop("ff"), "shared expert needs"),
    (lambda c: c.pop("width"), "missing key 'width'"),
])
def test_a_configuration_that_cannot_be_used_says_why(change, text):
    cfg = copy.deepcopy(CFG)
    change(cfg)
    with pytest.raises(ValueError, match=text):
        load_model_spec(cfg)


def test_groups_that_cannot_hold_the_chosen_are_refused():
    cfg = copy.deepcopy(CFG)
    cfg["layers"][1]["mlp"]["router"].update(top=5)          # two groups of two experts hold four
    _, spec = load_model_spec(cfg)
    with pytest.raises(ValueError, match="groups"):
        Model(spec, torch.bfloat16)
