"""Prefill and decode throughput of the hybrid design (Bavutar: attention, state-space and
gated-delta mixers between post-norms) at layer sizes that resemble a real model's, beside
the engine's closest other model (MiniMax M2 layers: the same attention sizes, routed experts
with the same number of active feed-forward weights per token) at equal width, and each of the
hybrid design's own kernels alone against its roofline.

    python -m sparseengine_b200.cli.hybrid_bench [--sizes 2048,4096] [--steps 20] [--warmup 3]

Random weights, bfloat16, one GPU, device-timed with CUDA events; inputs differ from step to step
and the weights of a step exceed the L2 cache.  ``bench.py --design hybrid`` prints the same
record as its one JSON line.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

from .kernel_bench import peaks, timed

PAGE_SIZE = 16
VOCAB = 32768


def hybrid_config(width: int, repeats: int = 1) -> dict:
    """Four layers per repeat: attention, state space, gated delta, attention over the first
    one's cache; head size 128, four query heads per key/value head, state 128."""
    heads = width // 128
    a = {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
         "q_temp": {"coef": 0.1, "every": 1024}}
    ff = {"kind": "dense", "ff": 4 * width}
    layers = []
    for r in range(repeats):
        layers += [
            {"type": "attention", "mixer": dict(a), "mlp": ff},
            {"type": "mamba2", "mixer": {"heads": 2 * width // 64, "vdim": 64, "state": 128, "groups": 8, "conv": 4,
                                         "norm_groups": 8}, "mlp": ff},
            {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": heads, "dim": 128, "vdim": 128, "conv": 4,
                                                "rank": 64}, "mlp": ff},
            {"type": "attention", "mixer": dict(a, kv_from=4 * r), "mlp": ff},
        ]
    return {"architecture": "Bavutar", "vocab": VOCAB, "width": width, "layers": layers, "postln_alpha": 2.0,
            "embedding": {"scale": 8.0}, "logit_softcap": 30.0, "norm": {"eps": 1e-6}, "max_position": 16384}


def closest_config(width: int, layers: int) -> dict:
    """MiniMax M2 layers of the same width and attention sizes; two experts, both active, each a third
    as wide as the hybrid's feed-forward of 4 x width (a gated expert has three matrices), so that a
    layer's feed-forward holds and uses as many weights as the hybrid's."""
    heads = width // 128
    return {"architectures": ["MiniMaxM2ForCausalLM"], "model_type": "minimax_m2", "hidden_size": width,
            "num_attention_heads": heads, "num_key_value_heads": max(1, heads // 4), "head_dim": 128, "rotary_dim": 64,
            "rope_theta": 1e6, "rms_norm_eps": 1e-6, "num_local_experts": 2, "num_experts_per_tok": 2,
            "intermediate_size": (4 * width // 3 + 127) // 128 * 128, "vocab_size": VOCAB, "max_position_embeddings": 16384,
            "num_hidden_layers": layers, "torch_dtype": "bfloat16"}


def _throughput(cfg: dict, points, steps: int, warmup: int) -> dict:
    """Tokens per second of the step function at each point ``(kind, batch, tokens)``: ``prefill``
    runs ``batch`` prompts of ``tokens`` tokens in one step, ``decode`` one token for each of ``batch``
    requests that hold ``tokens`` tokens."""
    from ..engine.factory import build_runner
    from ..engine.runner import StepEntry
    most = max(b * (t + steps + warmup + 8) for _, b, t in points)
    rows = max(b for _, b, _ in points)
    runner = build_runner(cfg, dtype="bfloat16", page_size=PAGE_SIZE, num_pages=-(-most // PAGE_SIZE) + rows,
                          max_rows=rows, max_seq_len=16384, random_weights=True, seed=3, norm_std=0.05, bias_std=0.1)
    vocab = runner.model.spec.vocab_size
    gen = torch.Generator().manual_seed(5)
    out = {}
    for kind, batch, tokens in points:
        ids = [f"{kind}{batch}_{i}" for i in range(batch)]

        def prompts():
            return [torch.randint(0, vocab, (tokens,), generator=gen).tolist() for _ in ids]

        times = []
        if kind == "prefill":
            for it in range(warmup + steps):
                toks = prompts()
                for s in ids:
                    runner.admit(s)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                e0.record()
                runner.step([StepEntry(s, t, [len(t) - 1]) for s, t in zip(ids, toks)])
                e1.record()
                torch.cuda.synchronize()
                if it >= warmup:
                    times.append(e0.elapsed_time(e1))
                for s in ids:
                    runner.release(s)
            per_step = batch * tokens
        else:
            for s in ids:
                runner.admit(s)
            per = max(1, 8192 // tokens)
            toks = prompts()
            for a in range(0, batch, per):
                runner.step([StepEntry(s, t, []) for s, t in zip(ids[a:a + per], toks[a:a + per])])
            nxt = torch.randint(0, vocab, (warmup + steps, batch), generator=gen).tolist()
            for it in range(warmup):
                runner.step([StepEntry(s, [nxt[it][j]], [0]) for j, s in enumerate(ids)])
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for it in range(warmup, warmup + steps):
                runner.step([StepEntry(s, [nxt[it][j]], [0]) for j, s in enumerate(ids)])
            e1.record()
            torch.cuda.synchronize()
            times = [e0.elapsed_time(e1) / steps]
            for s in ids:
                runner.release(s)
            per_step = batch
        ms = sorted(times)[len(times) // 2]
        out[f"{kind}_b{batch}_t{tokens}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(per_step / ms * 1e3, 1)}
    from ..csrc import ops
    ops.error_check(runner.device)
    del runner
    torch.cuda.empty_cache()
    return out


def _parts(cfg: dict, tokens: int, batch: int) -> dict:
    """Milliseconds per part (CUDA events around each) of one prompt step of ``tokens`` tokens and of
    one decode step of ``batch`` requests, launch by launch."""
    from ..engine.factory import build_runner
    from ..engine.runner import StepEntry
    runner = build_runner(cfg, dtype="bfloat16", page_size=PAGE_SIZE, num_pages=-(-(batch + 1) * (tokens + 64) // PAGE_SIZE),
                          max_rows=batch + 1, max_seq_len=16384, random_weights=True, seed=3, norm_std=0.05, bias_std=0.1,
                          decode_graphs=False)
    vocab = runner.model.spec.vocab_size
    gen = torch.Generator().manual_seed(7)
    out = {}

    def collect():
        torch.cuda.synchronize()
        rec = {k: round(sum(a.elapsed_time(b) for a, b in v) / 3, 4) for k, v in runner.model.profile.items()}
        runner.model.profile = None
        return rec

    for it in range(5):          # two untimed, three timed
        if it == 2:
            runner.model.profile = {}
        runner.admit("p")
        runner.step([StepEntry("p", torch.randint(0, vocab, (tokens,), generator=gen).tolist(), [tokens - 1])])
        runner.release("p")
    out[f"prefill_t{tokens}"] = collect()
    ids = [f"d{i}" for i in range(batch)]
    for s in ids:
        runner.admit(s)
        runner.step([StepEntry(s, torch.randint(0, vocab, (tokens,), generator=gen).tolist(), [])])
    for it in range(5):
        if it == 2:
            runner.model.profile = {}
        runner.step([StepEntry(s, [int(torch.randint(0, vocab, (1,), generator=gen))], [0]) for s in ids])
    out[f"decode_b{batch}_t{tokens}"] = collect()
    del runner
    torch.cuda.empty_cache()
    return out


def _kernels(width: int, tokens_list, pk: dict) -> dict:
    """Each kernel of the hybrid design alone: microseconds, the bytes it has to move (inputs read
    once, outputs written once), and the share of the copy bandwidth that is.  The two
    recurrences are chains of dependent steps along the tokens of a request, so their time is
    also given per token of the longest request."""
    from types import SimpleNamespace

    from ..csrc import ops
    dev = torch.device("cuda:0")
    cfg = hybrid_config(width)
    m2, dl = cfg["layers"][1]["mixer"], cfg["layers"][2]["mixer"]
    heads = width // 128
    out = {}
    for tokens, entries in tokens_list:
        per = tokens // entries
        step = SimpleNamespace(token_seq=torch.arange(tokens, device=dev, dtype=torch.int32) // per,
                               cu_q=torch.arange(entries + 1, device=dev, dtype=torch.int32) * per,
                               seq_rows=torch.arange(entries, device=dev, dtype=torch.int32), num_seqs=entries,
                               positions=(torch.arange(tokens, device=dev, dtype=torch.int32) % per) + 2048)
        rec = {}

        def add(name, fn, nbytes, iters=20):
            ms = timed(fn, iters)
            rec[name] = {"us": round(ms * 1e3, 2), "mbytes": round(nbytes / 1e6, 2),
                         "of_hbm_measured": round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 3)}

        bf = torch.bfloat16
        # norm over the stream
        x32 = torch.randn(tokens, width, device=dev)
        y = torch.randn(tokens, width, device=dev, dtype=bf)
        w = torch.ones(width, device=dev, dtype=bf)
        o32, oa = torch.empty_like(x32), torch.empty_like(y)
        add("add_layernorm", lambda: ops.add_layernorm(x32, y, 2.0, w, w, 1e-6, out32=o32, out_act=oa), tokens * width * 12)
        xa, wa, ra, oo, ro = y, w, torch.randn_like(y), torch.empty_like(y), torch.empty_like(y)
        add("closest: add_rmsnorm", lambda: ops.rmsnorm(xa, wa, 1e-6, oo, residual=ra, residual_out=ro), tokens * width * 8)
        # feed-forward activation
        hmid = torch.randn(tokens, 4 * width, device=dev, dtype=bf)
        add("activation", lambda: ops.activation_(hmid, "relu2"), tokens * 4 * width * 4)
        # state space
        H, P, N, G = m2["heads"], m2["vdim"], m2["state"], m2["groups"]
        inner, C = H * P, H * P + 2 * G * N
        proj = torch.randn(tokens, 2 * inner + 2 * G * N + H, device=dev, dtype=bf)
        state = torch.zeros(entries, H * P * N + 3 * C, device=dev)
        cw, cb = torch.randn(C, 4, device=dev) * 0.3, torch.zeros(C, device=dev)
        xbc = torch.empty(tokens, C, device=dev)
        add("causal_conv (state space)", lambda: ops.causal_conv(proj, inner, cw, cb, state, H * P * N, step, xbc), tokens * C * 6)
        dtb, al, dk = torch.zeros(H, device=dev), torch.zeros(H, device=dev), torch.ones(H, device=dev)
        yy = torch.empty(tokens, inner, device=dev)
        scan_bytes = tokens * (C + inner) * 4 + entries * H * P * N * 8
        add("ssm_scan", lambda: ops.ssm_scan(xbc, proj, inner + C, dtb, al, dk, state, step, yy, heads=H, head_dim=P,
                                             state_size=N, groups=G), scan_bytes, iters=5)
        rec["ssm_scan"]["us_per_token_of_a_request"] = round(rec["ssm_scan"]["us"] / per, 3)
        nw, gg = torch.ones(inner, device=dev), torch.empty(tokens, inner, device=dev, dtype=bf)
        add("gated_group_norm", lambda: ops.gated_group_norm(yy, proj, 0, nw, gg, parts=8, eps=1e-6), tokens * inner * 8)
        # gated delta
        H, Gk, d, dv = dl["heads"], dl["kv_heads"], dl["dim"], dl["vdim"]
        C = 2 * Gk * d + H * dv
        proj2 = torch.randn(tokens, C + H + 128, device=dev, dtype=bf)
        state2 = torch.zeros(entries, H * dv * d + 3 * C, device=dev)
        cw2 = torch.randn(C, 4, device=dev) * 0.3
        qkv = torch.empty(tokens, C, device=dev)
        add("causal_conv (gated delta)", lambda: ops.causal_conv(proj2, 0, cw2, None, state2, H * dv * d, step, qkv), tokens * C * 6)
        a = torch.randn(tokens, H * d, device=dev, dtype=bf)
        dec, beta = torch.empty(tokens, H * d, device=dev), torch.empty(tokens, H, device=dev)
        dtb2, al2 = torch.zeros(H * d, device=dev), torch.zeros(H, device=dev)
        add("delta_prep", lambda: ops.delta_prep(qkv, a, proj2, C, dtb2, al2, dec, beta, heads=H, kv_heads=Gk, head_dim=d,
                                                 v_head_dim=dv, unit_eps=1e-6, q_scale=d ** -0.5), tokens * (2 * Gk * d * 8 + H * d * 6))
        oo2 = torch.empty(tokens, H * dv, device=dev)
        add("delta_scan", lambda: ops.delta_scan(qkv, dec, beta, state2, step, oo2, heads=H, kv_heads=Gk, head_dim=d, v_head_dim=dv),
            tokens * (C + H * d + H * dv) * 4 + entries * H * d * dv * 8, iters=5)
        rec["delta_scan"]["us_per_token_of_a_request"] = round(rec["delta_scan"]["us"] / per, 3)
        gate, nw2, out2 = torch.randn(tokens, H * dv, device=dev, dtype=bf), torch.ones(dv, device=dev), torch.empty(tokens, H * dv, device=dev, dtype=bf)
        add("delta_out", lambda: ops.delta_out(oo2, gate, nw2, out2, heads=H, v_head_dim=dv, eps=1e-6), tokens * H * dv * 8)
        # query/key preparation (pages written round-robin)
        kvh = max(1, heads // 4)
        qn, kn = heads * 128, kvh * 128
        pr = torch.randn(tokens, qn + 2 * kn, device=dev, dtype=bf)
        pages = -(-(2048 + per) // PAGE_SIZE)
        table = torch.arange(entries * pages, device=dev, dtype=torch.int32).view(entries, pages)
        cache = torch.zeros(entries * pages, 2, kvh, PAGE_SIZE, 128, device=dev, dtype=bf)
        qw, kw, qo = torch.ones(qn, device=dev, dtype=bf), torch.ones(kn, device=dev, dtype=bf), torch.empty(tokens, qn, device=dev, dtype=bf)
        add("qk_prep_general", lambda: ops.qk_prep_general(pr, qw, kw, step.positions, step.token_seq, step.seq_rows, table, cache, qo,
                                                           num_heads=heads, num_kv_heads=kvh, head_dim=128, v_head_dim=128, eps=1e-6,
                                                           page_size=PAGE_SIZE, temperature=(0.1, 1024)), tokens * (qn + 2 * kn) * 4)
        inv = torch.ones(32, device=dev)
        add("closest: qk_prep (rotary)", lambda: ops.qk_prep(pr, qw, kw, inv, step.positions, step.token_seq, step.seq_rows, table, cache, qo,
                                                             num_heads=heads, num_kv_heads=kvh, head_dim=128, rotary_dim=64, eps=1e-6,
                                                             rope_scale=1.0, page_size=PAGE_SIZE), tokens * (qn + 2 * kn) * 4)
        out[f"tokens{tokens}_requests{entries}"] = rec
        ops.error_check(dev)
    return out


def run(sizes=(2048, 4096), steps: int = 20, warmup: int = 3, kernels: bool = True, parts: bool = True) -> dict:
    torch.cuda.set_device(0)
    pk = peaks()
    points = [("prefill", 1, 2048), ("prefill", 1, 8192), ("prefill", 4, 2048), ("decode", 8, 2048), ("decode", 64, 2048)]
    rec = {"design": "Bavutar (hybrid)", "closest": "MiniMaxM2ForCausalLM", "dtype": "bf16", "data": "synthetic",
           "peaks": pk, "sizes": {}}
    for width in sizes:
        hyb, m2 = hybrid_config(width, repeats=2), closest_config(width, layers=8)
        one = {"layers": 8, "hybrid": _throughput(hyb, points, steps, warmup), "closest": _throughput(m2, points, steps, warmup)}
        if parts:
            one["hybrid_parts_ms"] = _parts(hyb, 2048, 8)
            one["closest_parts_ms"] = _parts(m2, 2048, 8)
        if kernels:
            one["kernels"] = _kernels(width, [(2048, 1), (8192, 4), (64, 64)], pk)
        rec["sizes"][str(width)] = one
    return rec


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--sizes", default="2048,4096")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-kernels", action="store_true")
    ap.add_argument("--no-parts", action="store_true")
    a = ap.parse_args(argv)
    print(json.dumps(run(tuple(int(s) for s in a.sizes.split(",")), a.steps, max(a.warmup, 3), not a.no_kernels, not a.no_parts)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
