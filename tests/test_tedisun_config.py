"""The Tedisun design without a GPU: the plain implementation's own pieces on cases worked by hand, what the
configuration reader accepts, refuses and makes of a configuration, and what the model asks of the cache
manager (pages that hold the kept first tokens are never given back early)."""
import copy
import math

import numpy as np
import pytest
import torch

import plain_tedisun as pt
import sparseengine_b200.models  # noqa: F401
from sparseengine_b200.cache.manager import CacheManager
from sparseengine_b200.config.registry import load_model_spec
from sparseengine_b200.engine.model import CacheLayout, EntryCache, Model
from sparseengine_b200.parts.base import KVRequest
from test_tedisun_gpu import att, config, delta, mem, moe, par

F64 = torch.float64
CFG = config(64, 100, [delta(4, 2, 16, 8, 3, mlp=moe(6, 2, 24, 2)),
                       par(att(4, 2, 16, 8, 10, 3, rot=8, base=1000.0, scaling=(2.0, 1.0, 4.0, 128), scale=0.2), mem(2, 8, 12, 9.0),
                           0.25, 1.5),
                       par(att(2, 2, 8, 8), mem(1, 8, 8), mlp=moe(3, 3, 16, 0))], streams=3, eps=1e-4, softcap=20.0, scale=4.0)


def test_the_plain_mechanisms_are_what_they_claim():
    # rotation: pairs (i, i + dims/2), the rest passes
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0]]], dtype=F64)
    y = pt.rotate_half_pairs(x, torch.tensor([3]), {"dims": 4, "base": 100.0})
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    want = [np.cos(a0) - 3 * np.sin(a0), 2 * np.cos(a1) - 4 * np.sin(a1), 3 * np.cos(a0) + np.sin(a0),
            4 * np.cos(a1) + 2 * np.sin(a1), 5.0]
    assert np.allclose(y[0, 0].numpy(), want)
    # scaled frequencies: short waves kept, long waves slowed, the band between blended
    rot = {"dims": 8, "base": 10000.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 100}}
    f = [10000.0 ** (-2.0 * i / 8) for i in range(4)]
    got = pt.scaled_frequencies(rot).tolist()
    assert got[0] == f[0] and math.isclose(got[3], f[3] / 4.0)          # wavelengths 6.3 and 6283
    s = (100 / (2 * math.pi / f[1]) - 1.0) / 3.0                          # wavelength 63: between 25 and 100
    assert 0 < s < 1 and math.isclose(got[1], (1 - s) * f[1] / 4.0 + s * f[1])
    # convolution: the last tap weighs the current token, zeros before the start
    c = pt.causal_conv(torch.tensor([[1.0], [2.0], [3.0]], dtype=F64), torch.tensor([[10.0, 100.0, 1000.0]], dtype=F64))
    assert c[:, 0].tolist() == [1000.0, 2100.0, 3210.0]
    # a router that chooses every output weighs experts and identity experts by the softmax over all of them
    cfg = config(8, 10, [delta(1, 1, 4, 4, 2, mlp=moe(2, 4, 4, 2))], streams=2)
    w = {k: v.double() for k, v in pt.random_weights(cfg, 1).items()}
    h = torch.randn(5, 8, dtype=F64)
    z = torch.softmax(h @ w["l0.mlp.router"].T, -1)
    each = [(pt.silu(h @ w[f"l0.mlp.e{e}.gate"].T) * (h @ w[f"l0.mlp.e{e}.up"].T)) @ w[f"l0.mlp.e{e}.down"].T for e in range(2)]
    want = sum(z[:, e:e + 1] * each[e] for e in range(2)) + (z[:, 2:3] + z[:, 3:4]) * h
    assert torch.allclose(pt.routed_ff(h, w, "l0.mlp.", cfg["layers"][0]["mlp"]), want)
    # the correction moves the choice, not the weights
    w2 = dict(w)
    w2["l0.mlp.correction"] = torch.tensor([0.0, 0.0, 5.0, -5.0], dtype=F64)
    one = copy.deepcopy(cfg["layers"][0]["mlp"])
    one["router"]["top"] = 1
    assert torch.allclose(pt.routed_ff(h, w2, "l0.mlp.", one), z[:, 2:3] * h)
    # the matrix memory's first token: m = max(f, i) from m = 0; with a closed input gate the denominator is exp(-m)
    m = {"heads": 1, "dim": 2, "vdim": 2, "gate_cap": 10.0}
    ww = {"q": torch.eye(2, dtype=F64), "k": torch.eye(2, dtype=F64), "v": torch.eye(2, dtype=F64), "g": torch.zeros(2, 2, dtype=F64),
          "i": torch.zeros(1, 2, dtype=F64), "i.b": torch.tensor([-9.0], dtype=F64), "f": torch.zeros(1, 2, dtype=F64),
          "f.b": torch.tensor([2.0], dtype=F64), "norm": torch.ones(2, dtype=F64), "o": torch.eye(2, dtype=F64)}
    hh = torch.tensor([[3.0, 4.0]], dtype=F64)
    i = 10 * math.tanh(-0.9)
    f = -math.log1p(math.exp(-10 * math.tanh(0.2)))
    assert f > i                                                            # so m = f and the input weighs exp(i - f)
    raw = math.exp(i - f) * torch.tensor([3.0, 4.0]) * (3 * 3 + 4 * 4) * 2 ** -0.5 / (math.exp(-f) + 1e-6)
    want = raw / math.sqrt(float((raw * raw).mean()) + 1e-5) * 0.5
    assert torch.allclose(pt.matrix_memory(hh, ww, "", m, 1e-5)[0], want.double())


def test_the_configuration_becomes_parts_with_its_own_constants():
    cfg, spec = load_model_spec(copy.deepcopy(CFG))
    assert spec.architecture == "Tedisun" and spec.residual_stream == "float32" and spec.streams == 3
    assert (spec.embed_scale, spec.logit_softcap, spec.vocab_size, spec.head_source) == (4.0, 20.0, 100, "head")
    assert spec.final_norm.offset == 1.0 and spec.final_norm.eps == 1e-4
    d, p, q = (ls.mixer for ls in spec.layers)
    assert (d.kind, d.decay_per, d.gate_activation, d.num_heads, d.num_kv_heads, d.head_dim, d.v_head_dim, d.conv_taps) == \
        ("channel_delta", "head", "silu", 4, 2, 16, 8, 3)
    assert p.kind == "parallel" and p.scales == (0.25, 1.5) and p.names == ("left", "right")
    a, m = p.branches
    assert (a.qk_norm, a.bias, a.sink, a.window, a.keep_first, a.scale, a.v_head_dim, a.qk_norm_eps) == \
        ("per_head", True, "learned", 10, 3, 0.2, 8, 1e-4)
    assert (a.position.rotary_dim, a.position.theta, dict(a.position.frequency_scaling)["rope_type"]) == (8, 1000.0, "llama3")
    assert (m.kind, m.num_heads, m.head_dim, m.v_head_dim, m.gate_cap) == ("matrix_memory", 2, 8, 12, 9.0)
    b = q.branches[0]
    assert (b.window, b.keep_first, b.position, b.v_head_dim) == (None, 0, None, None)
    f0, none, f2 = (ls.feed_forward for ls in spec.layers)
    assert none is None and "feed_forward_streams" not in spec.layers[1].extra
    assert (f0.num_experts, f0.identity_experts, f0.top_k, f0.score_fn, f0.renormalize, f0.selection_bias) == (6, 2, 2, "softmax", False, True)
    assert f2.identity_experts == 0
    s = spec.layers[0].extra["mixer_streams"]
    assert (s.streams, s.gated, s.learned) == (3, True, True) and all(ls.arrangement == "stream_mix" for ls in spec.layers)
    # the scaled frequencies the engine's table holds are the plain implementation's
    from sparseengine_b200.parts.position import scaled_frequencies
    table, amp = scaled_frequencies(8, 1000.0, dict(a.position.frequency_scaling))
    assert amp == 1.0 and np.allclose(table.numpy(), pt.scaled_frequencies(CFG["layers"][1]["mixer"]["left"]["rot"]).numpy(), rtol=1e-6)
    # every tensor of a checkpoint is claimed by one parameter, and nothing else is asked for
    model = Model(spec, torch.float32)
    asked = sorted(src.name for prm in model.params() for src in prm.sources)
    assert asked == sorted(pt.random_weights(CFG, 0))
    # one group of pages per (sizes, window, kept tokens); one state per layer
    assert [(r.num_kv_heads, r.head_dim, r.window, r.keep_first) for r, _ in model.layout.groups] == [(2, 16, 10, 3), (2, 8, None, 0)]
    assert [st.shape for st in model.layout.states] == [(4 * 8 * 16 + 2 * (2 * 2 * 16 + 4 * 8),), (2 * 8 * 13 + 2,), (8 * 9 + 1,)]


def test_what_a_configuration_must_have():
    for breaker, word in ((lambda c: c["layers"][0].__setitem__("type", "attention"), "unknown mixer type"),
                          (lambda c: c["layers"][0]["mixer"].pop("conv"), "conv"),
                          (lambda c: c["layers"][1]["mixer"]["right"].pop("gate_cap"), "right.gate_cap"),
                          (lambda c: c["layers"][1]["mixer"]["left"]["rot"]["scaling"].pop("low"), "rot.scaling"),
                          (lambda c: c["layers"][1]["mixer"]["left"]["mask"].pop("size"), "'mask' needs 'size'"),
                          (lambda c: c["layers"][0]["mlp"]["router"].pop("top"), "router.top"),
                          (lambda c: c.pop("width"), "width")):
        c = copy.deepcopy(CFG)
        breaker(c)
        with pytest.raises(ValueError, match=word):
            load_model_spec(c)
    for breaker, word in ((lambda c: c.__setitem__("streams", 17), "residual streams"),
                          (lambda c: c["layers"][1]["mixer"]["left"]["mask"].__setitem__("keep_first", -1), "keep_first"),
                          (lambda c: c["layers"][1]["mixer"]["right"].__setitem__("dim", 300), "head_dim"),
                          (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 9), "top_k")):
        c = copy.deepcopy(CFG)
        breaker(c)
        _, spec = load_model_spec(c)
        with pytest.raises(ValueError, match=word):
            Model(spec, torch.float32)


def test_pages_of_the_kept_first_tokens_stay_and_the_rest_of_the_past_goes():
    group = (KVRequest(2, 16, window=10, keep_first=6), 1)
    cm = CacheManager(CacheLayout((group,), (), (EntryCache(0, 0, True, None),)), page_size=4, num_pages=12, max_rows=2,
                      max_seq_len=48, allocate=False)
    cm.admit("a")
    for n in (9, 2, 1, 17, 1, 1, 1, 1):
        cm.reserve("a", n)
        cm.commit("a", n)
        cm.check()
        held = sorted(cm._requests["a"].pages[0])
        first_needed = max(0, cm.length("a") - 10 + 1)
        # pages 0 and 1 hold positions 0..5; then every page that still holds a key of the next query's window
        want = sorted(set([0, 1][: -(-min(cm.length("a"), 6) // 4)]) | set(range(first_needed // 4, -(-cm.length("a") // 4))))
        assert held == want, (cm.length("a"), held, want)
    assert cm.free_pages() == 12 - len(held)
    cm.release("a")
    assert cm.free_pages() == 12
    cm.check()
