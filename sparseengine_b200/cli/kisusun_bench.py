"""Prefill and decode throughput of the Kisusun design (norms on the sublayers' outputs over a 32-bit
stream; attention with capped scores, a window, a zero sink, an output gate and blended values; a dense
layer and routed layers with grouped selection, clamped gated experts and a shared expert) at layer
sizes that resemble a real model's, beside the engine's closest other model (MiniMax M2 layers: the
same attention sizes, as many active expert weights per token) at equal width and depth, and each of
the design's own kernels alone against its roofline, with the like kernel of the closest model beside it.

    python -m sparseengine_b200.cli.kisusun_bench [--sizes 2048,4096] [--steps 20] [--warmup 3]

Random weights, bfloat16, one GPU, device-timed with CUDA events; inputs differ from step to step
and the weights of a step exceed the L2 cache.  ``bench.py --design kisusun`` prints the same
record as its one JSON line.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

from .hybrid_bench import PAGE_SIZE, VOCAB, _parts, _throughput
from .kernel_bench import peaks, timed

WINDOW = 4096
LAYERS = 8
EXPERTS = 8


def kisusun_config(width: int, layers: int = LAYERS) -> dict:
    """Head size 128 (values as wide), four query heads per key/value head, half of a head rotated, a
    window of 4,096 keys, blended values everywhere; the first layer's feed-forward is dense (3 x width),
    the others route 2 of 8 experts of ``width`` each in 4 groups of which 2 stay open, plus a shared
    expert of ``width``: three experts' worth of active feed-forward weights per token and layer."""
    heads = width // 128
    mixer = {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "softcap": 50.0,
             "mask": {"size": WINDOW}, "rot": {"base": 1e6, "dims": 64, "scaling": {"factor": 8.0}}, "v_mix": True}
    moe = {"kind": "moe", "expert": {"ff": width, "limit": 7.0},
           "router": {"experts": EXPERTS, "top": 2, "scale": 2.0, "groups": {"count": 4, "keep": 2}},
           "shared": {"ff": width, "limit": 7.0}}
    body = [{"type": "attention", "mixer": dict(mixer), "mlp": {"kind": "dense", "ff": 3 * width} if i == 0 else moe}
            for i in range(layers)]
    return {"architecture": "Kisusun", "vocab": VOCAB, "width": width, "layers": body, "logit_scale": 0.5,
            "embedding": {"scale": 8.0}, "norm": {"eps": 1e-6}, "max_position": 16384}


def closest_config(width: int, layers: int = LAYERS) -> dict:
    """MiniMax M2 layers of the same width and attention sizes; 8 experts of ``width`` each, 3 per token."""
    heads = width // 128
    return {"architectures": ["MiniMaxM2ForCausalLM"], "model_type": "minimax_m2", "hidden_size": width,
            "num_attention_heads": heads, "num_key_value_heads": max(1, heads // 4), "head_dim": 128, "rotary_dim": 64,
            "rope_theta": 1e6, "rms_norm_eps": 1e-6, "num_local_experts": EXPERTS, "num_experts_per_tok": 3,
            "intermediate_size": width, "vocab_size": VOCAB, "max_position_embeddings": 16384,
            "num_hidden_layers": layers, "torch_dtype": "bfloat16"}


def _kernels(width: int, cases, pk: dict) -> dict:
    """Each kernel the design adds or extends, alone: microseconds, the bytes it has to move (inputs
    read once, outputs written once) or the operations it has to do, and the share of the measured copy
    bandwidth or bfloat16 matrix throughput that is; ``like: ...`` is the closest model's kernel for the
    same step on inputs of the same size.  ``cases``: (tokens, requests, keys each request already holds)."""
    from types import SimpleNamespace

    from ..csrc import ops
    dev = torch.device("cuda:0")
    bf = torch.bfloat16
    hq, hkv, d = width // 128, max(1, width // 512), 128
    qn, kn = hq * d, hkv * d
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

        # the norm of a sublayer's output into the 32-bit stream
        x32 = torch.randn(tokens, width, device=dev)
        y = torch.randn(tokens, width, device=dev, dtype=bf)
        w = torch.ones(width, device=dev, dtype=bf)
        oa = torch.empty_like(y)
        add("rmsnorm_add_stream", lambda: ops.rmsnorm_add_stream(x32, y, w, 1e-6, out_act=oa), tokens * width * 12)
        ra, oo, ro = torch.randn_like(y), torch.empty_like(y), torch.empty_like(y)
        add("like: rmsnorm with residual", lambda: ops.rmsnorm(y, w, 1e-6, oo, residual=ra, residual_out=ro), tokens * width * 8)
        # query/key preparation: norms, rotation, blended values, page writes (the gate's columns are passed over)
        pages = -(-(held + per) // PAGE_SIZE)
        table = torch.arange(entries * pages, device=dev, dtype=torch.int32).view(entries, pages)
        cache = (torch.randn(entries * pages, 2, hkv, PAGE_SIZE, d, device=dev) * 0.5).to(bf)
        proj = torch.randn(tokens, 2 * qn + 2 * kn, device=dev, dtype=bf)
        v_first = torch.randn(tokens, kn, device=dev, dtype=bf)
        mix = torch.full((), 0.3, device=dev)
        qw, kw = torch.ones(qn, device=dev, dtype=bf), torch.ones(kn, device=dev, dtype=bf)
        inv = (1e6 ** (-torch.arange(0, 64, 2, dtype=torch.float32) / 64) / 8.0).to(dev)
        qo = torch.empty(tokens, qn, device=dev, dtype=bf)
        add("qk_prep_general (rotation, blended values)", lambda: ops.qk_prep_general(
            proj, qw, kw, step.positions, step.token_seq, step.seq_rows, table, cache, qo, num_heads=hq, num_kv_heads=hkv,
            head_dim=d, v_head_dim=d, eps=1e-6, page_size=PAGE_SIZE, inv_freq=inv, rotary_dim=64, v_first=v_first, v_mix=mix),
            tokens * ((qn + 2 * kn) * 4 + kn * 2))
        pr = torch.randn(tokens, qn + 2 * kn, device=dev, dtype=bf)
        add("like: qk_prep", lambda: ops.qk_prep(pr, qw, kw, inv, step.positions, step.token_seq, step.seq_rows, table, cache, qo,
                                                 num_heads=hq, num_kv_heads=hkv, head_dim=d, rotary_dim=64, eps=1e-6, rope_scale=1.0,
                                                 page_size=PAGE_SIZE), tokens * (qn + 2 * kn) * 4)
        # attention: cap, window, sink and gate against the same kernel without them (what the closest model runs)
        q = torch.randn(tokens, qn, device=dev, dtype=bf)
        o = torch.empty(tokens, qn, device=dev, dtype=bf)
        gate = proj[:, qn + 2 * kn:]
        opts = dict(softcap=50.0, sink=True, gate=gate)
        seen = sum(min(WINDOW, held + i + 1) for i in range(per)) * entries
        key_rows = entries * min(held + per, WINDOW + per - 1)
        if per > 1:
            common = dict(entries=entries, max_q_len=per, num_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=PAGE_SIZE,
                          scale=d ** -0.5, window=WINDOW)
            fl = 4.0 * seen * hq * d
            add("attn_prefill_tc (cap, sink, gate)", lambda: ops.attn_prefill_tc(q, cache, table, step.seq_rows, step.cu_q, kv_len, o,
                                                                                 **common, **opts), flops=fl)
            add("like: attn_prefill_tc", lambda: ops.attn_prefill_tc(q, cache, table, step.seq_rows, step.cu_q, kv_len, o, **common),
                flops=fl)
            add("attn_prefill (cap, sink, gate)", lambda: ops.attn_prefill(q, cache, table, step.seq_rows, step.cu_q, kv_len, o,
                                                                           **common, **opts), flops=fl)
            add("like: attn_prefill", lambda: ops.attn_prefill(q, cache, table, step.seq_rows, step.cu_q, kv_len, o, **common), flops=fl)
        else:
            common = dict(num_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=PAGE_SIZE, scale=d ** -0.5, window=WINDOW,
                          max_keys=min(WINDOW, held + 1))
            by = key_rows * hkv * d * 4 + tokens * qn * 4
            add("attn_decode (cap, sink, gate)", lambda: ops.attn_decode(q, cache, table, step.seq_rows, step.token_seq, step.positions,
                                                                         o, **common, **opts), nbytes=by + tokens * qn * 2)
            add("like: attn_decode", lambda: ops.attn_decode(q, cache, table, step.seq_rows, step.token_seq, step.positions, o,
                                                             **common), nbytes=by)
        # values half as wide as keys (query/key heads of 64, values of 32): the m16n8k16 kernels
        h64, g64 = 2 * hq, 2 * hkv
        cache64 = (torch.randn(entries * pages, g64 * PAGE_SIZE * 96, device=dev) * 0.5).to(bf)
        q64 = torch.randn(tokens, h64 * 64, device=dev, dtype=bf)
        o64 = torch.empty(tokens, h64 * 32, device=dev, dtype=bf)
        gate64 = torch.randn(tokens, h64 * 32, device=dev, dtype=bf)
        o6464 = torch.empty(tokens, h64 * 64, device=dev, dtype=bf)
        cache6464 = (torch.randn(entries * pages, g64 * PAGE_SIZE * 128, device=dev) * 0.5).to(bf)
        if per > 1:
            common = dict(entries=entries, max_q_len=per, num_heads=h64, num_kv_heads=g64, head_dim=64, page_size=PAGE_SIZE,
                          scale=0.125, window=WINDOW)
            add("attn_prefill (heads of 64, values of 32; cap, sink, gate)", lambda: ops.attn_prefill(
                q64, cache64, table, step.seq_rows, step.cu_q, kv_len, o64, v_head_dim=32, softcap=50.0, sink=True, gate=gate64, **common),
                flops=2.0 * seen * h64 * 96)
            add("like: attn_prefill (heads of 64)", lambda: ops.attn_prefill(q64, cache6464, table, step.seq_rows, step.cu_q, kv_len,
                                                                            o6464, **common), flops=4.0 * seen * h64 * 64)
        else:
            common = dict(num_heads=h64, num_kv_heads=g64, head_dim=64, page_size=PAGE_SIZE, scale=0.125, window=WINDOW,
                          max_keys=min(WINDOW, held + 1))
            add("attn_decode (heads of 64, values of 32; cap, sink, gate)", lambda: ops.attn_decode(
                q64, cache64, table, step.seq_rows, step.token_seq, step.positions, o64, v_head_dim=32, softcap=50.0, sink=True,
                gate=gate64, **common), nbytes=key_rows * g64 * 96 * 2 + tokens * h64 * (64 + 32 + 32) * 2)
            add("like: attn_decode (heads of 64)", lambda: ops.attn_decode(
                q64, cache6464, table, step.seq_rows, step.token_seq, step.positions, o6464, **common),
                nbytes=key_rows * g64 * 128 * 2 + tokens * h64 * 128 * 2)
        # the router: grouped selection against selection among all experts
        E, top = 64, 6
        gw = torch.randn(E, width, device=dev) * 0.02
        ids, wt = torch.empty(tokens, top, device=dev, dtype=torch.int32), torch.empty(tokens, top, device=dev)
        lg = torch.empty(tokens, E, device=dev)
        rb = tokens * (width * 2 + E * 4 + top * 8) + E * width * 4
        add("router (64 experts, 8 groups, 4 open)", lambda: ops.router(y, gw, None, ids, wt, top_k=top, renormalize=False,
                                                                        routed_scale=2.0, logits_out=lg, groups=8, keep_groups=4), rb)
        add("like: router (64 experts)", lambda: ops.router(y, gw, None, ids, wt, top_k=top, renormalize=True, logits_out=lg), rb)
        out[f"tokens{tokens}_requests{entries}_held{held}"] = rec
        ops.error_check(dev)
    return out


def run(sizes=(2048, 4096), steps: int = 20, warmup: int = 3, kernels: bool = True, parts: bool = True) -> dict:
    torch.cuda.set_device(0)
    pk = peaks()
    points = [("prefill", 1, 2048), ("prefill", 1, 8192), ("prefill", 4, 2048), ("decode", 8, 2048), ("decode", 64, 2048)]
    rec = {"design": "Kisusun", "closest": "MiniMaxM2ForCausalLM", "dtype": "bf16", "data": "synthetic", "peaks": pk, "sizes": {}}
    for width in sizes:
        kis, m2 = kisusun_config(width), closest_config(width)
        one = {"layers": LAYERS, "kisusun": _throughput(kis, points, steps, warmup), "closest": _throughput(m2, points, steps, warmup)}
        if parts:
            one["kisusun_parts_ms"] = _parts(kis, 2048, 8)
            one["closest_parts_ms"] = _parts(m2, 2048, 8)
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
