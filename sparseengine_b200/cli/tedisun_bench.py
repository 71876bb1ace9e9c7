"""Prefill and decode throughput of the Tedisun design (several residual streams, a gated delta rule
with one decay per head, attention with kept first keys and a learned sink beside a matrix memory,
routed experts with identity experts) at layer sizes that resemble a real model's, beside the
engine's closest other model (Zisevik: pre-norm over a 32-bit stream, windowed attention with a
learned sink, a linear recurrence with a matrix state, routed experts) at equal width and number of
layer visits, and each of the design's own kernels alone against its roofline, with the like kernel
of the closest models beside it.

    python -m sparseengine_b200.cli.tedisun_bench [--sizes 2048,4096] [--steps 20] [--warmup 3]

Random weights, bfloat16, one GPU, device-timed with CUDA events; inputs differ from step to step
and the weights of a step exceed the L2 cache.  ``bench.py --design tedisun`` prints the same
record as its one JSON line.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

from .hybrid_bench import PAGE_SIZE, VOCAB, _parts, _throughput
from .kernel_bench import peaks, timed
from .zisevik_bench import zisevik_config

WINDOW, KEPT, STREAMS = 1024, 4, 4


def tedisun_config(width: int) -> dict:
    """Eight layers, delta rule and parallel mixer in turn.  Delta rule: heads with a 128 x 128 state, two
    value heads per query/key head; attention: head size 128, four query heads per key/value head, a window of
    1,024 with 4 kept first tokens, half of a head rotated; matrix memory: heads with a 128 x 128 state; routed
    experts: 8 of the model's width and 2 identity experts, 2 per token; four residual streams."""
    heads = width // 128
    d = {"heads": heads, "kv_heads": max(1, heads // 2), "dim": 128, "vdim": 128, "conv": 4}
    left = {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
            "mask": {"size": WINDOW, "keep_first": KEPT},
            "rot": {"base": 500000.0, "dims": 64, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    right = {"heads": max(1, heads // 2), "dim": 128, "vdim": 128, "gate_cap": 15.0}
    moe = {"kind": "moe", "expert": {"ff": width}, "router": {"experts": 8, "identity": 2, "top": 2}}
    layers = []
    for _ in range(4):
        layers += [{"type": "delta", "mixer": dict(d), "mlp": moe},
                   {"type": "parallel", "mixer": {"left": dict(left), "right": dict(right), "left_scale": 0.6, "right_scale": 1.1},
                    "mlp": moe}]
    return {"architecture": "Tedisun", "vocab": VOCAB, "width": width, "streams": STREAMS, "layers": layers,
            "embedding": {"scale": width ** 0.5}, "logit_softcap": 30.0, "norm": {"eps": 1e-6}, "max_position": 16384}


def _kernels(width: int, cases, pk: dict) -> dict:
    """Each kernel of the design alone: microseconds, the bytes it has to move (inputs read once, outputs
    written once) or the operations it has to do, and the share of the measured copy bandwidth or bfloat16
    matrix throughput that is; ``like: ...`` are kernels of the closest models on inputs of the same size.
    ``cases``: (tokens, requests, keys each request already holds)."""
    from types import SimpleNamespace

    from ..csrc import ops
    dev = torch.device("cuda:0")
    cfg = tedisun_config(width)
    dl, pm = cfg["layers"][0]["mixer"], cfg["layers"][1]["mixer"]
    bf = torch.bfloat16
    out = {}
    for tokens, entries, held in cases:
        per = tokens // entries
        step = SimpleNamespace(token_seq=torch.arange(tokens, device=dev, dtype=torch.int32) // per,
                               cu_q=torch.arange(entries + 1, device=dev, dtype=torch.int32) * per,
                               seq_rows=torch.arange(entries, device=dev, dtype=torch.int32), num_seqs=entries, max_q_len=per,
                               positions=(torch.arange(tokens, device=dev, dtype=torch.int32) % per) + held)
        kv_len = torch.full((entries,), held + per, device=dev, dtype=torch.int32)
        rec = {}

        def add(name, fn, nbytes=None, flops=None, iters=20):
            ms = timed(fn, iters)
            r = {"us": round(ms * 1e3, 2)}
            if nbytes is not None:
                r.update(mbytes=round(nbytes / 1e6, 2), of_hbm_measured=round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 3))
            if flops is not None:
                r.update(gflop=round(flops / 1e9, 2), of_bf16_measured=round(flops / (ms * 1e-3) / 1e12 / pk["bf16_tflops"], 3))
            rec[name] = r

        # the streams: a sublayer's write and the next one's read in one kernel
        S = STREAMS
        xs = torch.randn(tokens, S, width, device=dev)
        y = torch.randn(tokens, width, device=dev, dtype=bf)
        gl = torch.randn(tokens, width, device=dev, dtype=bf)
        gb, nw = torch.zeros(width, device=dev), torch.ones(width, device=dev)
        mix, ow, iw = torch.eye(S, device=dev), torch.ones(S, device=dev), torch.full((S,), 1.0 / S, device=dev)
        h = torch.empty(tokens, width, device=dev, dtype=bf)
        add("stream_mix (write + read)", lambda: ops.stream_mix(xs, write=(y, gl, gb, mix, ow), read=(iw, nw, 1e-6, h), dtype=bf),
            tokens * width * (8 * S + 6))
        x32, w16, oa = torch.randn(tokens, width, device=dev), torch.ones(width, device=dev, dtype=bf), torch.empty_like(y)
        add("like: add_rmsnorm_stream (one stream)", lambda: ops.add_rmsnorm_stream(x32, y, w16, 1e-6, out32=x32, out_act=oa),
            tokens * width * 12)
        y2, so = torch.randn_like(y), torch.empty_like(y)
        add("scaled_sum", lambda: ops.scaled_sum(y, y2, 0.6, 1.1, so, bias=gb), tokens * width * 6)
        # attention: preparation, then the keys
        a = pm["left"]
        hq, hkv, d = a["heads"], a["kv_heads"], a["dim"]
        pages = -(-(held + per) // PAGE_SIZE)
        table = torch.arange(entries * pages, device=dev, dtype=torch.int32).view(entries, pages)
        cache = (torch.randn(entries * pages, 2, hkv, PAGE_SIZE, d, device=dev) * 0.5).to(bf)
        cols = (hq + 2 * hkv) * d
        proj = torch.randn(tokens, cols, device=dev, dtype=bf)
        inv = (500000.0 ** (-torch.arange(0, 64, 2, dtype=torch.float32) / 64)).to(dev)
        q = torch.empty(tokens, hq * d, device=dev, dtype=bf)
        w_head, w_whole_q, w_whole_k = torch.ones(d, device=dev, dtype=bf), torch.ones(hq * d, device=dev, dtype=bf), \
            torch.ones(hkv * d, device=dev, dtype=bf)
        bias = torch.zeros(cols, device=dev)
        prep = dict(num_heads=hq, num_kv_heads=hkv, head_dim=d, v_head_dim=d, eps=1e-6, page_size=PAGE_SIZE, inv_freq=inv, rotary_dim=64)
        add("qk_prep_general (bias, norm per head)", lambda: ops.qk_prep_general(
            proj, w_head, w_head, step.positions, step.token_seq, step.seq_rows, table, cache, q, bias=bias, per_head=True, **prep),
            tokens * cols * 4)
        add("like: qk_prep_general (norm over the projection)", lambda: ops.qk_prep_general(
            proj, w_whole_q, w_whole_k, step.positions, step.token_seq, step.seq_rows, table, cache, q, **prep), tokens * cols * 4)
        q.normal_()
        o = torch.empty(tokens, hq * d, device=dev, dtype=bf)
        sink = torch.zeros(hq, device=dev)
        att = dict(num_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=PAGE_SIZE, scale=d ** -0.5, window=WINDOW)
        seen = sum(min(WINDOW + KEPT, held + i + 1) for i in range(per)) * entries
        key_rows = entries * min(held + per, WINDOW + KEPT + per - 1)
        if per > 1:
            add("attn_prefill (window, kept first keys, learned sink)", lambda: ops.attn_prefill(
                q, cache, table, step.seq_rows, step.cu_q, kv_len, o, entries=entries, max_q_len=per, sink=sink, keep_first=KEPT, **att),
                flops=4.0 * seen * hq * d)
            add("like: attn_prefill (window, sink of 0)", lambda: ops.attn_prefill(
                q, cache, table, step.seq_rows, step.cu_q, kv_len, o, entries=entries, max_q_len=per, sink=True, **att),
                flops=4.0 * seen * hq * d)
            add("attn_prefill_tc (window, kept first keys, learned sink)", lambda: ops.attn_prefill_tc(
                q, cache, table, step.seq_rows, step.cu_q, kv_len, o, entries=entries, max_q_len=per, sink=sink, keep_first=KEPT, **att),
                flops=4.0 * seen * hq * d)
            add("like: attn_prefill_tc (window, sink of 0)", lambda: ops.attn_prefill_tc(
                q, cache, table, step.seq_rows, step.cu_q, kv_len, o, entries=entries, max_q_len=per, sink=True, **att),
                flops=4.0 * seen * hq * d)
        else:
            nbytes = key_rows * hkv * d * 4 + tokens * hq * d * 4
            add("attn_decode (window, kept first keys, learned sink)", lambda: ops.attn_decode(
                q, cache, table, step.seq_rows, step.token_seq, step.positions, o, sink=sink, keep_first=KEPT,
                max_keys=min(held + 1, WINDOW + KEPT), **att), nbytes)
            add("like: attn_decode (window, sink of 0)", lambda: ops.attn_decode(
                q, cache, table, step.seq_rows, step.token_seq, step.positions, o, sink=True, max_keys=min(held + 1, WINDOW), **att),
                nbytes)
        # matrix memory
        r = pm["right"]
        Hm, dm, dvm = r["heads"], r["dim"], r["vdim"]
        qk, vv = Hm * dm, Hm * dvm
        g_off, i_off, f_off, m_off = 2 * qk + vv, 2 * qk + 2 * vv, 2 * qk + 2 * vv + Hm, Hm * dm * (dvm + 1)
        proj_m = torch.randn(tokens, f_off + Hm, device=dev, dtype=bf) * 0.3
        gbias, nwm = torch.zeros(2 * Hm, device=dev), torch.ones(vv, device=dev)
        state = torch.zeros(entries, m_off + Hm, device=dev)
        gates = torch.empty(tokens, Hm, 3, device=dev)
        add("memory_gates", lambda: ops.memory_gates(proj_m, i_off, f_off, gbias, 15.0, state, m_off, step, gates, heads=Hm),
            tokens * Hm * 16)
        rec["memory_gates"]["us_per_token_of_a_request"] = round(rec["memory_gates"]["us"] / per, 3)
        om = torch.empty(tokens, Hm, dvm + 1, device=dev)
        scan_bytes = tokens * (2 * qk * 2 + vv * 2 + Hm * (dvm + 1) * 4) + entries * Hm * dm * (dvm + 1) * 8
        add("memory_scan", lambda: ops.memory_scan(proj_m, 0, qk, 2 * qk, gates, dm ** -0.5, state, step, om, heads=Hm, head_dim=dm,
                                                   v_head_dim=dvm), scan_bytes, iters=5)
        rec["memory_scan"]["us_per_token_of_a_request"] = round(rec["memory_scan"]["us"] / per, 3)
        if per >= 16:
            add("memory_chunk", lambda: ops.memory_chunk(proj_m, 0, qk, 2 * qk, gates, dm ** -0.5, state, step, om, heads=Hm, head_dim=dm,
                                                         v_head_dim=dvm), scan_bytes, iters=5)
            rec["memory_chunk"]["us_per_token_of_a_request"] = round(rec["memory_chunk"]["us"] / per, 3)
        gm = torch.empty(tokens, vv, device=dev, dtype=bf)
        add("memory_out", lambda: ops.memory_out(om, gates, proj_m, g_off, nwm, gm, heads=Hm, v_head_dim=dvm, eps=1e-6, den_eps=1e-6),
            tokens * vv * 8)
        # like: the retention of the closest model, the same number of heads and state size
        proj_r = torch.randn(tokens, 2 * qk + 2 * vv, device=dev, dtype=bf) * 0.3
        q32, k32 = torch.randn(tokens, qk, device=dev) * 0.1, torch.randn(tokens, qk, device=dev) * 0.1
        decay = torch.full((Hm,), 0.99, device=dev)
        state_r = torch.zeros(entries, Hm * dm * dvm, device=dev)
        o_r = torch.empty(tokens, vv, device=dev)
        add("like: retention_scan", lambda: ops.retention_scan(q32, k32, proj_r, 2 * qk, decay, state_r, step, o_r, heads=Hm, head_dim=dm,
                                                               v_head_dim=dvm), tokens * (2 * qk * 4 + vv * 6) + entries * Hm * dm * dvm * 8, iters=5)
        rec["like: retention_scan"]["us_per_token_of_a_request"] = round(rec["like: retention_scan"]["us"] / per, 3)
        if per >= 16:
            add("like: retention_chunk", lambda: ops.retention_chunk(q32, k32, proj_r, 2 * qk, decay, state_r, step, o_r, heads=Hm, head_dim=dm,
                                                                     v_head_dim=dvm), tokens * (2 * qk * 4 + vv * 6) + entries * Hm * dm * dvm * 8, iters=5)
            rec["like: retention_chunk"]["us_per_token_of_a_request"] = round(rec["like: retention_chunk"]["us"] / per, 3)
        add("like: retention_out", lambda: ops.retention_out(o_r, proj_r, 2 * qk + vv, gm, heads=Hm, v_head_dim=dvm, eps=1e-6), tokens * vv * 8)
        # delta rule: one decay per head (the recurrence is the closest model's own kernel)
        Hd, Gd, dd, dvd = dl["heads"], dl["kv_heads"], dl["dim"], dl["vdim"]
        C = 2 * Gd * dd + Hd * dvd
        proj_d = torch.randn(tokens, C + 2 * Hd + Hd * dvd, device=dev, dtype=bf) * 0.3
        qkv = torch.randn(tokens, C, device=dev) * 0.1
        dec, beta = torch.empty(tokens, Hd * dd, device=dev), torch.empty(tokens, Hd, device=dev)
        dtb, alog, nwd = torch.zeros(Hd, device=dev), torch.zeros(Hd, device=dev), torch.ones(dvd, device=dev)
        add("delta_prep (one decay per head)", lambda: ops.delta_prep(
            qkv, proj_d[:, C + Hd:C + 2 * Hd], proj_d, C, dtb, alog, dec, beta, heads=Hd, kv_heads=Gd, head_dim=dd, v_head_dim=dvd,
            unit_eps=1e-6, q_scale=dd ** -0.5, per_head=True), tokens * (2 * Gd * dd * 8 + Hd * dd * 4))
        state_d = torch.zeros(entries, Hd * dd * dvd + 3 * C, device=dev)
        o_d = torch.empty(tokens, Hd * dvd, device=dev)
        add("delta_scan", lambda: ops.delta_scan(qkv, dec, beta, state_d, step, o_d, heads=Hd, kv_heads=Gd, head_dim=dd, v_head_dim=dvd),
            tokens * (C + Hd * dd + Hd * dvd) * 4 + entries * Hd * dd * dvd * 8, iters=5)
        rec["delta_scan"]["us_per_token_of_a_request"] = round(rec["delta_scan"]["us"] / per, 3)
        if per >= 16:
            log_dec = torch.rand(tokens, Hd, device=dev) * -0.1
            add("delta_chunk", lambda: ops.delta_chunk(qkv, log_dec, beta, state_d, step, o_d, heads=Hd, kv_heads=Gd, head_dim=dd,
                                                       v_head_dim=dvd), tokens * (C + Hd + Hd * dvd) * 4 + entries * Hd * dd * dvd * 8, iters=5)
            rec["delta_chunk"]["us_per_token_of_a_request"] = round(rec["delta_chunk"]["us"] / per, 3)
        out_d = torch.empty(tokens, Hd * dvd, device=dev, dtype=bf)
        add("delta_out (silu gate from the projection)", lambda: ops.delta_out(
            o_d, proj_d[:, C + 2 * Hd:], nwd, out_d, heads=Hd, v_head_dim=dvd, eps=1e-6, silu=True), tokens * Hd * dvd * 8)
        # the sum over the chosen experts' rows, with identity experts
        top = 2
        yk = torch.randn(tokens * top, width, device=dev, dtype=bf)
        inv_pos = torch.arange(tokens * top, device=dev, dtype=torch.int32)
        inv_id = inv_pos.clone()
        inv_id[::5] = -1
        wts = torch.rand(tokens, top, device=dev)
        xo = torch.empty(tokens, width, device=dev, dtype=bf)
        add("moe_combine (a fifth of the slots identity experts)", lambda: ops.moe_combine(yk, inv_id, xo, top, identity=(y, wts)),
            tokens * width * 2 * (top + 1))
        add("like: moe_combine", lambda: ops.moe_combine(yk, inv_pos, xo, top), tokens * width * 2 * (top + 1))
        out[f"tokens{tokens}_requests{entries}_held{held}"] = rec
        ops.error_check(dev)
    return out


def run(sizes=(2048, 4096), steps: int = 20, warmup: int = 3, kernels: bool = True, parts: bool = True) -> dict:
    torch.cuda.set_device(0)
    pk = peaks()
    points = [("prefill", 1, 2048), ("prefill", 1, 8192), ("prefill", 4, 2048), ("decode", 8, 2048), ("decode", 64, 2048)]
    rec = {"design": "Tedisun", "closest": "Zisevik", "dtype": "bf16", "data": "synthetic", "peaks": pk, "sizes": {}}
    for width in sizes:
        ted, zis = tedisun_config(width), zisevik_config(width)
        one = {"layer_visits": 8, "tedisun": _throughput(ted, points, steps, warmup), "closest": _throughput(zis, points, steps, warmup)}
        if parts:
            one["tedisun_parts_ms"] = _parts(ted, 2048, 8)
        if kernels:
            one["kernels"] = _kernels(width, [(2048, 1, 0), (8192, 4, 0), (64, 64, 2048)], pk)
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
