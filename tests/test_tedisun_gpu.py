"""The Tedisun design in the engine against the plain implementation (tests/plain_tedisun.py): each
mechanism alone, whole prompts against token-by-token decoding, portions down to two tokens, mixed
batches with pages and state slots that are used again, keys at the window's two edges, at the edge
of the kept first tokens and at page borders, the sink, a far token held by a slow decay, the first
tokens, long decoding, other sizes (also values equal to one another or to 1), and greedy
generation through ``LLM``."""
import copy
import json
import os

import numpy as np
import pytest
import torch

import plain_tedisun as pt
import trace_util as tu

pytestmark = pytest.mark.gpu


def moe(experts, top, ff, identity=0):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}


def delta(heads, kv_heads, dim, vdim, conv, mlp=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": mlp}


def att(heads, kv_heads, dim, vdim, window=None, keep=0, rot=None, base=10000.0, scaling=None, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if window is not None:
        m["mask"] = {"size": window, "keep_first": keep}
    if rot:
        m["rot"] = {"dims": rot, "base": base}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return m


def mem(heads, dim, vdim, cap=10.0):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def par(left, right, left_scale=0.7, right_scale=1.2, mlp=None):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": mlp}


def config(width, vocab, layers, streams=3, eps=1e-5, softcap=12.0, scale=None):
    c = {"architecture": "Tedisun", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps},
         "embedding": {"scale": scale if scale is not None else width ** 0.5}, "logit_softcap": softcap}
    if streams is not None:
        c["streams"] = streams
    return c


CONFIGS = {
    # both mixers, layers with and without feed-forward, a rotation over part of a head with scaled frequencies
    "hybrid": config(96, 160, [delta(4, 2, 16, 24, 4, mlp=moe(5, 2, 24, 1)),
                               par(att(6, 3, 16, 12, 11, 3, rot=8, base=300.0, scaling=(4.0, 1.0, 4.0, 64)), mem(3, 12, 20, 8.0),
                                   mlp=moe(4, 2, 32, 2)),
                               delta(2, 2, 8, 8, 2),
                               par(att(2, 1, 16, 16, 20, 0, rot=16), mem(2, 16, 8), 1.0, 0.5)]),
    # sizes that bfloat16 steps give to the tensor-core kernels; the layers start with a parallel one
    "wide": config(128, 200, [par(att(4, 2, 64, 64, 33, 5, rot=32, scaling=(8.0, 1.0, 2.0, 48)), mem(2, 32, 32), mlp=moe(8, 3, 64, 2)),
                              delta(4, 4, 32, 32, 3, mlp=moe(8, 2, 64, 1)),
                              par(att(2, 1, 128, 64, 40, 17, rot=64), mem(4, 16, 48, 15.0), 0.4, 0.9, mlp=moe(8, 2, 64, 0))],
                   streams=4),
    # sizes that are equal or 1: one stream, one head, one expert, a window of one key, one kept token
    "ones": config(32, 48, [par(att(1, 1, 32, 32, 1, 1, rot=32), mem(1, 32, 32), 1.0, 1.0, mlp=moe(1, 1, 32, 1)),
                            delta(1, 1, 32, 32, 2, mlp=moe(1, 1, 32, 0))], streams=1, softcap=None),
    # sizes that are multiples of nothing in particular; more chosen than half of the router's outputs
    "odd": config(52, 77, [delta(3, 1, 10, 5, 3, mlp=moe(7, 5, 9, 2)), par(att(5, 5, 6, 7, 19, 4, rot=6, base=50.0), mem(2, 10, 3, 5.0)),
                           par(att(3, 1, 10, 3, 4, 9, rot=2), mem(3, 5, 7), 1.3, 0.2, mlp=moe(3, 2, 10, 3))], streams=5, eps=1e-6),
}


def write_folder(folder, cfg, seed, w=None):
    from safetensors.torch import save_file
    w = w if w is not None else pt.random_weights(cfg, seed)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in w.items()}, os.path.join(folder, "model.safetensors"))
    return w


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        d = str(tmp_path_factory.mktemp("ted_" + name))
        out[name] = (d, cfg, write_folder(d, cfg, 51 + i))
    return out


_plain_cache = {}


def plain_logits(name, cfg, w, seqs):
    out = {}
    for sid, toks in seqs.items():
        key = (name, json.dumps(cfg, sort_keys=True), tuple(toks))
        if key not in _plain_cache:
            _plain_cache[key] = pt.forward(cfg, w, toks).float().numpy()
        out[sid] = _plain_cache[key]
    return out


def row_errors(got, ref):
    """Difference of every logits row (mean taken off, root mean square) in units of the reference
    rows' root mean square."""
    rows = np.stack([ref[sid][p] for sid, p in got])
    rms = float(np.sqrt((rows.astype(np.float64) ** 2).mean()))
    out = {}
    for (sid, p), row in got.items():
        d = row.astype(np.float64) - ref[sid][p]
        d -= d.mean()
        e = float(np.sqrt((d * d).mean())) / rms
        out[(sid, p)] = e if e == e else float("inf")
    return out


# 32-bit: every row within 5e-5.  bfloat16: rounding alone moves the rows of these small models by a few
# hundredths, and a token whose router scores nearly tie goes to another expert than in the plain
# implementation, which moves its row (and, through the recurrent states, the rows behind it a little) in
# every way of cutting alike.  So nine rows of ten must lie within 0.08, and no more than 2 rows (or 3 %)
# beyond 0.2.  A fault of the cache, the state or a window moves every row behind it by its whole size.
BOUND32 = 5e-5


def assert_close(got, ref, dtype, what, bound=None):
    errs = row_errors(got, ref)
    v = np.array(list(errs.values()))
    where = max(errs, key=errs.get)
    if bound is not None or dtype == "float32":
        limit = bound or BOUND32
        assert v.max() < limit, f"{what} ({dtype}): row error {v.max():.3e} at {where}"
        return
    assert np.quantile(v, 0.9) < 0.08, f"{what} ({dtype}): nine rows of ten within {np.quantile(v, 0.9):.3e}"
    assert int((v > 0.2).sum()) <= max(2, len(v) * 3 // 100), \
        f"{what} ({dtype}): {int((v > 0.2).sum())} of {len(v)} rows beyond 0.2, worst at {where}"


def make_runner(folder, dtype, steps, page_size=16, rows=4, **kw):
    from sparseengine_b200.engine.factory import build_runner
    tokens = tu.max_live_tokens(steps, round_to=page_size)
    return build_runner(folder, dtype=dtype, page_size=page_size, num_pages=max(1, tokens // page_size), max_rows=rows,
                        max_seq_len=max(64, tokens), **kw)


def check_trace(folders, name, dtype, steps, seqs, what, bound=None, **kw):
    folder, cfg, w = folders[name]
    runner = make_runner(folder, dtype, steps, **kw)
    got = tu.run_trace_runner(runner, steps)
    from sparseengine_b200.csrc import ops
    ops.error_check(runner.device)
    runner.cache.check()
    assert runner.cache.free_rows == runner.cache.max_rows
    assert_close(got, plain_logits(name, cfg, w, seqs), dtype, f"{what}, {name}", bound)
    return runner


def prompts(cfg, lengths, seed):
    return {f"s{i}": tu.random_prompt(cfg["vocab"], n, seed + i) for i, n in enumerate(lengths)}


# ---- each mechanism alone ----------------------------------------------------------------------

SINGLE = {
    "delta_rule": dict(layers=[delta(4, 2, 8, 12, 3)]),
    "delta_rule_long_taps": dict(layers=[delta(2, 1, 12, 4, 5)]),
    "attention": dict(layers=[par(att(4, 2, 8, 12, 9, 2, rot=4), mem(1, 4, 4), 1.0, 0.0)]),
    "attention_all_keys": dict(layers=[par(att(2, 2, 8, 8, None, 0, rot=8, scaling=(3.0, 1.0, 2.0, 20)), mem(1, 4, 4), 1.0, 0.0)]),
    "attention_unrotated": dict(layers=[par(att(3, 1, 12, 4, 6, 6), mem(1, 4, 4), 1.0, 0.0)]),
    "matrix_memory": dict(layers=[par(att(1, 1, 4, 4, 1, 0), mem(3, 12, 20, 6.0), 0.0, 1.0)]),
    "both_side_by_side": dict(layers=[par(att(2, 1, 8, 8, 7, 1, rot=8), mem(2, 8, 8), 0.6, 1.1)]),
    "routed_feed_forward": dict(layers=[delta(1, 1, 4, 4, 2, mlp=moe(6, 3, 16, 0))]),
    "identity_experts": dict(layers=[delta(1, 1, 4, 4, 2, mlp=moe(3, 3, 16, 3))]),
    "one_plain_stream": dict(layers=[delta(2, 1, 8, 8, 3, mlp=moe(4, 2, 16, 1))], streams=None),
    "eight_streams": dict(layers=[delta(2, 1, 8, 8, 3, mlp=moe(4, 2, 16, 1))], streams=8),
    "eleven_streams": dict(layers=[delta(2, 1, 8, 8, 3, mlp=moe(4, 2, 16, 1))], streams=11),
    "delta_rule_one_tap": dict(layers=[delta(2, 2, 8, 8, 1)]),
    "a_width_that_is_no_multiple_of_four": dict(layers=[delta(2, 1, 8, 8, 3, mlp=moe(4, 2, 10, 1)),
                                                        par(att(2, 1, 8, 8, 7, 1, rot=8), mem(2, 8, 8), mlp=moe(3, 2, 6, 2))], width=54),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", sorted(SINGLE))
def test_each_mechanism_alone(tmp_path, which, dtype):
    kw = dict(SINGLE[which])
    cfg = config(kw.pop("width", 40), 50, **kw)
    w = write_folder(str(tmp_path), cfg, 5)
    seqs = prompts(cfg, (37, 1, 18), 3)
    for cut in (tu.trace_whole, lambda s: tu.trace_chunks(s, sizes=(2, 3, 1, 5, 2)), lambda s: tu.trace_tail_decode(s, tail=9)):
        check_trace({which: (str(tmp_path), cfg, w)}, which, dtype, cut(seqs), seqs, "alone")


def test_a_checkpoint_without_gates_and_corrections(tmp_path):
    """The reader goes by the tensors a checkpoint holds: no gate on the sublayers' results, no correction
    of the router's choice, the head tied to the embedding."""
    cfg = config(40, 50, [delta(2, 1, 8, 8, 3, mlp=moe(4, 2, 16, 1)), par(att(2, 1, 8, 8, 7, 1, rot=8), mem(2, 8, 8))])
    w = {k: v for k, v in pt.random_weights(cfg, 8).items() if ".rg" not in k and "correction" not in k and k != "head"}
    write_folder(str(tmp_path), cfg, 0, w)
    seqs = prompts(cfg, (23, 6), 5)
    check_trace({"bare": (str(tmp_path), cfg, w)}, "bare", "float32", tu.trace_chunks(seqs, sizes=(5, 2, 9)), seqs, "bare")


# ---- ways of cutting ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_decode_chunks_mixed(folders, name, dtype):
    cfg = CONFIGS[name]
    seqs = prompts(cfg, (70, 33, 1, 18, 49, 2, 26), 20)
    check_trace(folders, name, dtype, tu.trace_whole(seqs), seqs, "whole")
    check_trace(folders, name, dtype, tu.trace_tail_decode(seqs, tail=20), seqs, "decode")
    check_trace(folders, name, dtype, tu.trace_chunks(seqs), seqs, "portions")
    check_trace(folders, name, dtype, tu.trace_chunks(seqs, sizes=(2,)), seqs, "portions of two")
    # three rows for seven requests, and a pool of the live tokens only: rows, state slots and pages are used again
    runner = check_trace(folders, name, dtype, tu.trace_mixed(seqs, live=3, chunk=6, decode_tail=5), seqs, "mixed", rows=3)
    assert all(g.pool.reused_total > 0 for g in runner.cache.groups)
    check_trace(folders, name, dtype, tu.trace_random(seqs, seed=3, live=4), seqs, "random schedule", page_size=8)


def test_a_state_slot_that_is_used_again_starts_from_zero(folders):
    """One row: every request gets the slot and the pages the one before it left; a long request
    first, so that its states and its running maximum are far from zero."""
    seqs = prompts(CONFIGS["hybrid"], (60, 5, 1, 9), 40)
    check_trace(folders, "hybrid", "float32", tu.trace_chunks(seqs, sizes=(7, 2)), seqs, "one slot", rows=1)


# ---- places where a fault would sit --------------------------------------------------------------

def sharp_window_model(window, keep, seed=9, dim=16, vdim=16, heads=4, kv_heads=2):
    """One attention layer (the memory beside it is weighed 0) whose softmax is sharp, so that a query hangs on
    the one or two keys it sees with the highest score: a key that is lost at the window's far edge or among
    the kept first tokens, or one that is let in from between the two, moves the row by much."""
    cfg = config(64, 80, [par(att(heads, kv_heads, dim, vdim, window, keep, rot=dim // 2, scale=2.5), mem(1, 4, 4), 1.0, 0.0,
                              mlp=moe(2, 1, 32, 1))], streams=2)
    w = pt.random_weights(cfg, seed)
    w["l0.mix.left.sink"] = torch.full_like(w["l0.mix.left.sink"], -4.0)
    return cfg, w


@pytest.mark.parametrize("dtype,dim,vdim", [("float32", 16, 16), ("bfloat16", 16, 16), ("bfloat16", 64, 64), ("bfloat16", 128, 32)])
def test_the_windows_edges_the_kept_first_tokens_and_page_borders(tmp_path, dtype, dim, vdim):
    """Window 37 with 21 kept first tokens over pages of 16: the oldest key of the window wanders through every
    place of a page, the kept tokens end inside the second page, in prompts, in portions that start and end
    anywhere, and in tokens decoded alone; pages between the two are given back and used again meanwhile.
    (In bfloat16 the rounding of queries and keys moves such sharp weights by itself, hence the wider bound; a
    lost key moves the row by its whole size.)  Head sizes 64 and 128 take the tensor-core kernels."""
    cfg, w = sharp_window_model(37, 21, dim=dim, vdim=vdim)
    write_folder(str(tmp_path), cfg, 0, w)
    seqs = prompts(cfg, (150, 37, 38, 58, 59, 16, 95, 22), 60)
    fs = {"edge": (str(tmp_path), cfg, w)}
    bound = 0.3 if dtype == "bfloat16" else None
    check_trace(fs, "edge", dtype, tu.trace_whole(seqs), seqs, "window, whole", bound)
    check_trace(fs, "edge", dtype, tu.trace_tail_decode(seqs, tail=60), seqs, "window, decoded", bound)
    check_trace(fs, "edge", dtype, tu.trace_chunks(seqs, sizes=(15, 2, 16, 33, 1, 37, 38)), seqs, "window, portions", bound)
    runner = check_trace(fs, "edge", dtype, tu.trace_mixed(seqs, live=3, chunk=21, decode_tail=40), seqs, "window, mixed", bound, rows=3)
    assert runner.cache.groups[0].pool.reused_total > 0


def test_the_plain_edges_matter_and_the_engine_is_on_the_right_side(tmp_path):
    """The premise of the test above: a window one key longer or shorter, or one kept token more or fewer,
    moves the plain logits far beyond the bound the engine is held to."""
    cfg, w = sharp_window_model(37, 21)
    toks = tu.random_prompt(80, 150, 60)
    ref = pt.forward(cfg, w, toks)
    rms = float(ref.pow(2).mean().sqrt())
    for key, other in (("size", 36), ("size", 38), ("keep_first", 20), ("keep_first", 22)):
        c = copy.deepcopy(cfg)
        c["layers"][0]["mixer"]["left"]["mask"][key] = other
        d = pt.forward(c, w, toks) - ref
        assert float(d[:36].abs().max()) < 1e-9                     # the first tokens see everything either way
        assert float(d[70:].pow(2).mean().sqrt()) / rms > 3e-3, (key, other)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_heavy_sink(tmp_path, dtype):
    """Sinks far above every score take almost all of the weight (outputs near the bias), sinks far
    below take none; both in one model, with windows of two keys and of one."""
    cfg = config(48, 64, [par(att(4, 2, 8, 8, 2, 0, rot=4), mem(1, 4, 4), 1.0, 0.1),
                          par(att(4, 4, 8, 8, 1, 2, rot=8), mem(1, 4, 4), 1.0, 0.1, mlp=moe(2, 1, 16, 1))])
    w = pt.random_weights(cfg, 4)
    w["l0.mix.left.sink"] = torch.tensor([9.0, -30.0, 2.0, 0.0]).to(torch.bfloat16)
    w["l1.mix.left.sink"] = torch.tensor([-2.0, 30.0, 0.5, -9.0]).to(torch.bfloat16)
    write_folder(str(tmp_path), cfg, 0, w)
    seqs = prompts(cfg, (21, 2, 1), 7)
    fs = {"sink": (str(tmp_path), cfg, w)}
    no_sink = dict(w)
    no_sink["l0.mix.left.sink"] = torch.full_like(w["l0.mix.left.sink"], -1e4)
    a, b = pt.forward(cfg, w, seqs["s0"]), pt.forward(cfg, no_sink, seqs["s0"])
    assert float((a - b).pow(2).mean().sqrt() / a.pow(2).mean().sqrt()) > 1e-2           # the premise: the sink matters
    for cut in (tu.trace_whole, lambda s: tu.trace_chunks(s, sizes=(2, 1, 3)), lambda s: tu.trace_tail_decode(s, tail=12)):
        check_trace(fs, "sink", dtype, cut(seqs), seqs, "sink")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["delta", "memory"])
def test_a_far_token_held_by_the_state(tmp_path, dtype, which):
    """A delta rule whose decays are almost 1 and whose writes are small, or a matrix memory whose forget gates are almost open, keeps the
    first tokens for good: the model's only way back is the state (the attention beside the memory sees one key), so a
    changed first token can reach position 400 through the state alone.  A state that is lost at a portion's
    start or copied to the wrong slot shows there."""
    if which == "delta":
        cfg = config(48, 64, [delta(3, 1, 16, 16, 2, mlp=moe(2, 1, 32, 1))])
        w = pt.random_weights(cfg, 12)
        w["l0.mix.A_log"] = torch.tensor([-9.0, -7.0, -1.0]).to(torch.bfloat16)
        # every token writes little (beta near 0), so that what the first ones wrote is not written over: a channel
        # that is the same in every embedding and weighs against beta
        w["embed"][:, 0] = 1.0
        w["l0.hc1.in"] = torch.tensor([0.4, 0.3, 0.3]).to(torch.bfloat16)
        w["l0.mix.b"][:, 0] = -1.0
    else:
        cfg = config(48, 64, [par(att(1, 1, 8, 8, 1, 0), mem(3, 16, 16, 12.0), 0.3, 1.0, mlp=moe(2, 1, 32, 1))])
        w = pt.random_weights(cfg, 12)
        w["l0.mix.right.f.b"] = torch.tensor([9.0, 7.0, 2.0]).to(torch.bfloat16)
        w["l0.mix.right.i"] = w["l0.mix.right.i"] * 0.2
    write_folder(str(tmp_path), cfg, 0, w)
    seqs = prompts(cfg, (420, 130, 3), 70)
    changed = list(seqs["s0"])
    changed[0] = (changed[0] + 1) % 64
    a, b = pt.forward(cfg, w, seqs["s0"]), pt.forward(cfg, w, changed)
    assert float((a[400:] - b[400:]).pow(2).mean().sqrt() / a.pow(2).mean().sqrt()) > 1e-3        # the premise
    fs = {"far": (str(tmp_path), cfg, w)}
    check_trace(fs, "far", dtype, tu.trace_whole(seqs), seqs, "far token, whole")
    check_trace(fs, "far", dtype, tu.trace_chunks(seqs, sizes=(64, 2, 33, 7, 1)), seqs, "far token, portions")
    check_trace(fs, "far", dtype, tu.trace_tail_decode(seqs, tail=40), seqs, "far token, decoded")
    check_trace(fs, "far", dtype, tu.trace_mixed(seqs, live=2, chunk=50, decode_tail=10), seqs, "far token, mixed", rows=2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_first_tokens(folders, dtype):
    """Requests of one to four tokens, whole, in portions of one and two, and side by side."""
    seqs = prompts(CONFIGS["hybrid"], (1, 2, 3, 4, 1), 90)
    check_trace(folders, "hybrid", dtype, tu.trace_whole(seqs), seqs, "first tokens")
    check_trace(folders, "hybrid", dtype, tu.trace_chunks(seqs, sizes=(1, 2, 1)), seqs, "first tokens, portions")
    check_trace(folders, "hybrid", dtype, tu.trace_mixed(seqs, live=4, chunk=2, decode_tail=1), seqs, "first tokens, mixed")


def test_long_decoding_through_replayed_graphs(folders):
    """140 tokens decoded one by one, far past every window, through replayed CUDA graphs."""
    seqs = prompts(CONFIGS["hybrid"], (170, 150), 120)
    steps = tu.trace_tail_decode(seqs, tail=140)
    runner = check_trace(folders, "hybrid", "float32", steps, seqs, "long decoding")
    assert runner.graph_replays > 200
    check_trace(folders, "hybrid", "bfloat16", steps, seqs, "long decoding")
    check_trace(folders, "wide", "bfloat16", steps, {k: [t % 200 for t in v] for k, v in seqs.items()}, "long decoding")


def test_a_batch_does_not_change_a_request(folders):
    """Unequal requests in one step against each alone: equal up to the order of sums in 32-bit."""
    from sparseengine_b200.engine.runner import StepEntry
    folder, cfg, w = folders["hybrid"]
    seqs = prompts(cfg, (29, 3, 11), 140)
    steps = [{"step": 0, "entries": [{"id": sid, "tokens": toks} for sid, toks in seqs.items()], "end": []}]
    runner = make_runner(folder, "float32", steps, rows=4)       # pages for all three at once
    alone = {}
    for sid, toks in seqs.items():
        runner.admit(sid)
        runner.step([StepEntry(sid, toks[:-1], [])])
        alone[sid] = runner.step([StepEntry(sid, toks[-1:], [0])]).clone()
        runner.release(sid)
    for sid in seqs:
        runner.admit(sid)
    runner.step([StepEntry(sid, toks[:-1], []) for sid, toks in seqs.items()])
    together = runner.step([StepEntry(sid, toks[-1:], [0]) for sid, toks in seqs.items()])
    for i, sid in enumerate(seqs):
        assert float((together[i] - alone[sid][0]).abs().max()) < 2e-5 * float(alone[sid][0].abs().max()), sid


def test_the_streams_sum_after_every_layer(folders):
    """The sum of the 32-bit streams after each layer against the plain implementation's."""
    from sparseengine_b200.engine.runner import StepEntry
    folder, cfg, w = folders["hybrid"]
    toks = tu.random_prompt(cfg["vocab"], 45, 8)
    taps = []
    pt.forward(cfg, w, toks, taps)
    assert len(taps) == len(cfg["layers"])
    runner = make_runner(folder, "float32", [{"step": 0, "entries": [{"id": "a", "tokens": toks}], "end": []}])
    runner.model.stream_taps = got = []
    runner.admit("a")
    runner.step([StepEntry("a", toks, [0])])
    assert len(got) == len(taps)
    for i, (a, b) in enumerate(zip(got, taps)):
        assert float((a.cpu().double() - b).abs().max()) < 3e-5 * float(b.abs().max()), i


# ---- kernels against one another -----------------------------------------------------------------

@pytest.mark.parametrize("d,dv,heads,kv_heads,window,keep", [(64, 64, 4, 2, 33, 5), (128, 64, 6, 1, 70, 70), (64, 32, 2, 2, 5, 100),
                                                              (128, 128, 8, 2, 100, 1), (64, 128, 3, 3, None, 0)])
def test_tensor_core_attention_against_the_plain_kernel(d, dv, heads, kv_heads, window, keep):
    """The same queries, pages and block table through the plain kernel, the split-key kernel and the
    prompt-portion kernel: portions that start anywhere beside single tokens, pages in a shuffled order, windows
    and kept first keys that end inside key tiles and pages, learned sinks that take much, little and almost
    none of the weight."""
    from sparseengine_b200.csrc import ops
    dev, page = "cuda:0", 16
    g = torch.Generator(device=dev).manual_seed(d + heads)
    q_lens, kv_lens = [37, 1, 130, 1, 2, 1], [37, 64, 209, 140, 17, 3]
    entries, tokens = len(q_lens), sum(q_lens)
    max_pages = -(-max(kv_lens) // page)
    perm = torch.randperm(entries * max_pages, generator=torch.Generator().manual_seed(1)).to(torch.int32)
    seq_rows = torch.tensor([3, 0, 4, 1, 5, 2], dtype=torch.int32, device=dev)
    table = perm.view(entries, max_pages).to(dev)[torch.argsort(seq_rows.cpu()).to(dev)].contiguous()
    cache = (torch.randn(entries * max_pages, page * kv_heads * (d + dv), generator=g, device=dev) * 0.7).to(torch.bfloat16)
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    positions = torch.cat([torch.arange(k - n, k) for n, k in zip(q_lens, kv_lens)]).to(torch.int32).to(dev)
    token_seq = torch.repeat_interleave(torch.arange(entries), torch.tensor(q_lens)).to(torch.int32).to(dev)
    cu_q = torch.tensor(cu, dtype=torch.int32, device=dev)
    kv_len = torch.tensor(kv_lens, dtype=torch.int32, device=dev)
    q = torch.randn(tokens, heads * d, generator=g, device=dev).to(torch.bfloat16)
    sink = torch.linspace(-6.0, 4.0, heads, device=dev)
    common = dict(num_heads=heads, num_kv_heads=kv_heads, head_dim=d, page_size=page, scale=d ** -0.5 * 2.0, window=window,
                  v_head_dim=dv, sink=sink, keep_first=keep if window else 0)
    plain = torch.empty(tokens, heads * dv, dtype=torch.bfloat16, device=dev)
    ops.paged_attention_plain(q, cache, table, seq_rows, token_seq, positions, plain, **common)
    portions = torch.full_like(plain, float("nan"))
    ops.attn_prefill(q, cache, table, seq_rows, cu_q, kv_len, portions, entries=entries, max_q_len=max(q_lens), **common)
    split = torch.full_like(plain, float("nan"))
    max_keys = max(kv_lens) if window is None else min(max(kv_lens), window + keep)
    ops.attn_decode(q, cache, table, seq_rows, token_seq, positions, split, max_keys=max_keys, **common)
    others = [(portions, "portions"), (split, "split keys")]
    if d == dv and ops.attn_prefill_tc_supported(d, heads, kv_heads):
        tc = torch.full_like(plain, float("nan"))
        ops.attn_prefill_tc(q, cache.view(-1, 2, kv_heads, page, d), table, seq_rows, cu_q, kv_len, tc, entries=entries,
                            max_q_len=max(q_lens), **common)
        others.append((tc, "portions, tensor memory"))
    ops.error_check(dev)
    for other, what in others:
        assert bool(torch.isfinite(other.float()).all()), what
        assert float((other.float() - plain.float()).abs().max()) < 3e-2 * float(plain.float().abs().max()), what


@pytest.mark.parametrize("heads,d,dv", [(3, 12, 20), (2, 64, 64), (1, 256, 31), (4, 130, 33), (2, 128, 128)])
def test_the_matrix_memory_kernels_against_the_recurrence_written_out(heads, d, dv):
    """Gates, recurrence and read-out of the three kernels against the same equations in 64-bit torch, from non-zero
    states and maxima, entries of 1, 31, 32, 33 and 200 tokens in one step; the states they leave."""
    from types import SimpleNamespace
    from sparseengine_b200.csrc import ops
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(d + dv)
    q_lens = [31, 1, 200, 32, 33]
    tokens, entries = sum(q_lens), len(q_lens)
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    rows = [2, 0, 4, 1, 3]
    step = SimpleNamespace(cu_q=torch.tensor(cu, dtype=torch.int32, device=dev), num_seqs=entries, max_q_len=max(q_lens),
                           seq_rows=torch.tensor(rows, dtype=torch.int32, device=dev))
    qk, vv, cap, eps = heads * d, heads * dv, 7.0, 1e-5
    g_off, i_off, f_off, m_off = 2 * qk + vv, 2 * qk + 2 * vv, 2 * qk + 2 * vv + heads, heads * d * (dv + 1)
    proj = torch.randn(tokens, f_off + heads, generator=g, device=dev)
    proj[:, i_off:] *= 3.0
    bias = torch.randn(2 * heads, generator=g, device=dev)
    norm_w = 1.0 + 0.1 * torch.randn(vv, generator=g, device=dev)
    state0 = torch.randn(5, m_off + heads, generator=g, device=dev) * 0.3
    results = []
    # token by token; in chunks of 64 tokens, in one pass and in segments of 64 and of 128 tokens side by side
    for walk, kw in ((ops.memory_scan, {}), (ops.memory_chunk, {"segments": (1, 0)}), (ops.memory_chunk, {"segments": (4, 64)}),
                     (ops.memory_chunk, {"segments": (2, 128)})):
        state = state0.clone()
        gates = torch.empty(tokens, heads, 3, device=dev)
        ops.memory_gates(proj, i_off, f_off, bias, cap, state, m_off, step, gates, heads=heads)
        o = torch.full((tokens, heads, dv + 1), float("nan"), device=dev)
        walk(proj, 0, qk, 2 * qk, gates, d ** -0.5, state, step, o, heads=heads, head_dim=d, v_head_dim=dv, **kw)
        out = torch.full((tokens, vv), float("nan"), device=dev)
        ops.memory_out(o, gates, proj, g_off, norm_w, out, heads=heads, v_head_dim=dv, eps=eps, den_eps=1e-6)
        results.append((out, state))
    P, B, Wn = proj.double().cpu(), bias.double().cpu(), norm_w.double().cpu()
    want = torch.zeros(tokens, vv, dtype=torch.float64)
    left = state0.double().cpu().clone()
    for e in range(entries):
        S = left[rows[e], :m_off].view(heads, d, dv + 1).clone()
        m = left[rows[e], m_off:].clone()
        for t in range(cu[e], cu[e + 1]):
            q = P[t, :qk].view(heads, d) * d ** -0.5
            k = P[t, qk:2 * qk].view(heads, d)
            v1 = torch.cat([P[t, 2 * qk:2 * qk + vv].view(heads, dv), torch.ones(heads, 1, dtype=torch.float64)], 1)
            gi = cap * torch.tanh((P[t, i_off:i_off + heads] + B[:heads]) / cap)
            gf = pt.log_sigmoid(cap * torch.tanh((P[t, f_off:f_off + heads] + B[heads:]) / cap))
            new = torch.maximum(gf + m, gi)
            S = torch.exp(gf + m - new)[:, None, None] * S + torch.exp(gi - new)[:, None, None] * k[:, :, None] * v1[:, None, :]
            m = new
            r = torch.einsum("hdv,hd->hv", S, q)
            u = r[:, :dv] / (torch.maximum(r[:, dv].abs(), torch.exp(-m)) + 1e-6)[:, None]
            u = pt.unit_rms(u, eps).reshape(vv) * Wn * torch.sigmoid(P[t, g_off:g_off + vv])
            want[t] = u
        left[rows[e], :m_off] = S.reshape(-1)
        left[rows[e], m_off:] = m
    for out, state in results:
        assert bool(torch.isfinite(out).all())
        assert float((out.double().cpu() - want).abs().max()) < 5e-5 * float(want.abs().max())
        assert float((state.double().cpu() - left).abs().max()) < 5e-5 * float(left.abs().max())


# ---- the entry point -----------------------------------------------------------------------------

def plain_greedy(cfg, w, prompt, steps):
    toks, out, margins = list(prompt), [], []
    for _ in range(steps):
        logits = pt.forward(cfg, w, toks)[-1]
        top = torch.topk(logits, 2).values
        margins.append(float(top[0] - top[1]))
        out.append(int(logits.argmax()))
        toks.append(out[-1])
    return out, margins


@pytest.mark.parametrize("name", ["hybrid", "odd"])
def test_greedy_generation_through_the_entry_point(folders, name):
    from sparseengine_b200 import LLM, SamplingParams
    folder, cfg, w = folders[name]
    llm = LLM(folder, dtype="float32", page_size=8, num_kvcache_slots=512, max_num_batched_tokens=16, max_model_len=128,
              max_num_seqs_in_gpu=3)
    ps = [tu.random_prompt(cfg["vocab"], n, 200 + n) for n in (5, 21, 9, 2, 14)]
    outs = llm.generate(ps, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    for p, o in zip(ps, outs):
        want, margins = plain_greedy(cfg, w, p, 10)
        if min(margins) > 1e-4:
            assert o["token_ids"] == want
        else:       # a near-tie: the tokens up to it
            k = next(i for i, m in enumerate(margins) if m <= 1e-4)
            assert o["token_ids"][:k] == want[:k]
    assert llm.is_finished() and llm.runner.cache.free_rows == llm.runner.cache.max_rows


def test_trace_program(folders, tmp_path):
    """bin/trace_run as a program on a folder of this design, pages and slots used again."""
    folder, cfg, w = folders["wide"]
    seqs = prompts(cfg, (40, 7, 22, 31, 3), 300)
    steps = tu.trace_mixed(seqs, live=4, chunk=9, decode_tail=4)
    for dtype in ("float32", "bfloat16"):
        out = str(tmp_path / dtype)
        got = tu.run_trace_cli(folder, dtype, steps, out, tu.max_live_tokens(steps))
        assert_close(got, plain_logits("wide", cfg, w, seqs), dtype, "trace program")


def test_command_line(folders, tmp_path):
    import subprocess
    import sys
    folder, cfg, w = folders["hybrid"]
    hyper = json.dumps({"dtype": "bfloat16", "page_size": 8, "num_kvcache_slots": 1024, "max_model_len": 256})
    for extra in ([], ["--tiny_random"]):
        r = subprocess.run([sys.executable, "-m", "sparseengine_b200.cli.bench", "--model_path", folder, "--lengths", "24",
                            "--batch_sizes", "3", "--output_len", "6", "--random_prompts", "--generate", "--hyper_params", hyper,
                            *extra], cwd=tu.ROOT, capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr[-2000:]
        assert r.stdout.strip()


@pytest.mark.parametrize("heads,kv_heads,d,dv", [(3, 1, 12, 20), (2, 2, 64, 64), (1, 1, 256, 31), (4, 2, 130, 33), (4, 2, 128, 128)])
def test_the_chunked_delta_rule_against_the_walk_token_by_token(heads, kv_heads, d, dv):
    """The triangular system per chunk of 64 tokens and the chain of single steps, on the same inputs and from the
    same non-zero states: entries of 1, 63, 64, 65 and 200 tokens in one step, decays from almost 1 down to 0.3, writes of
    every strength; outputs and the states they leave."""
    from types import SimpleNamespace
    from sparseengine_b200.csrc import ops
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(d + dv)
    q_lens = [63, 1, 200, 64, 65]
    tokens, entries = sum(q_lens), len(q_lens)
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    step = SimpleNamespace(cu_q=torch.tensor(cu, dtype=torch.int32, device=dev), num_seqs=entries, max_q_len=max(q_lens),
                           seq_rows=torch.tensor([2, 0, 4, 1, 3], dtype=torch.int32, device=dev))
    qk, vv = kv_heads * d, heads * dv
    qkv = torch.randn(tokens, 2 * qk + vv, generator=g, device=dev)
    unit = qkv[:, :2 * qk].view(tokens, 2 * kv_heads, d)
    unit /= unit.norm(dim=-1, keepdim=True)
    unit[:, :kv_heads] *= d ** -0.5
    log_dec = -torch.rand(tokens, heads, generator=g, device=dev) ** 3 * 1.2
    beta = torch.rand(tokens, heads, generator=g, device=dev)
    dec = log_dec.exp().repeat_interleave(d, 1).contiguous()
    state0 = torch.randn(5, heads * d * dv + 7, generator=g, device=dev) * 0.2
    outs = []
    for chunked in (False, True):
        state = state0.clone()
        o = torch.full((tokens, vv), float("nan"), device=dev)
        if chunked:
            ops.delta_chunk(qkv, log_dec, beta, state, step, o, heads=heads, kv_heads=kv_heads, head_dim=d, v_head_dim=dv)
        else:
            ops.delta_scan(qkv, dec, beta, state, step, o, heads=heads, kv_heads=kv_heads, head_dim=d, v_head_dim=dv)
        outs.append((o, state))
    (o1, s1), (o2, s2) = outs
    assert bool(torch.isfinite(o2).all())
    assert float((o1 - o2).abs().max()) < 3e-5 * float(o1.abs().max())
    assert float((s1 - s2).abs().max()) < 3e-5 * float(s1.abs().max())
