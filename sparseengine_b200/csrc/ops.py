"""Python bindings of the exported kernel launchers (ctypes, raw device pointers).

Every launcher is ``extern "C" int se_<name>(..., cudaStream_t)``.  A binding checks
device, dtype and contiguity of each tensor, passes ``data_ptr()`` and the current
CUDA stream, and raises on a non-zero return.  There is no other implementation behind
these functions: without the compiled library they raise.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build as _build

_P, _I, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
_SIG = {"p": _P, "i": _I, "f": _F, "l": ctypes.c_longlong}

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}

_ERRORS = {-2: "a size this kernel does not support", -3: "an inconsistent argument"}

_fns: dict = {}

# Kernels launched through these bindings since the process started (a launcher that
# starts two kernels counts two).  Benchmarks read the difference around a timed region.
KERNELS_PER_CALL = {"se_attn_decode": 2, "se_router": 2, "se_causal_conv": 2, "se_ssm_scan": 2}   # upper bounds per call
launch_count = 0
calls: dict = {}     # launcher name -> times called (tests check which kernels a path took)


def library():
    return _build.load()


# Sizes beyond which a kernel refuses (SE_ERR_UNSUPPORTED).  The parts check them when they are
# built, so that a model this library cannot run fails at construction with the limit named,
# not at its first step; the numbers restate the launchers' own (a GPU test compares them with
# what the compiled library reports through `limit`).
LIMITS = {
    "rmsnorm_max_width": 51200,             # a row is kept in shared memory in 32-bit
    "router_max_experts": 12800,            # four floats per expert in shared memory during selection
    "router_max_unaligned_width": 6400,     # widths that are no multiple of 4 keep 8 token rows in shared memory
    "moe_max_experts": 6079,                # the routing build's scans keep two ints per expert in shared memory
    "attention_max_head_dim": 256,          # in steps of 16
    "layernorm_max_width": 51200,           # as the RMS norm: the row is kept in shared memory in 32-bit
    "recurrent_max_state_rows": 512,        # rows of a recurrence's state on the key/state side (16 registers x 32 lanes)
    "latent_max_row": 1024,                 # latent plus shared key part of one position (32 registers x 32 lanes)
    "retention_max_head_dim": 256,          # rows of a retention state (32 registers x 8 warps)
    "stream_mix_max_streams": 16,           # a column's stream values live in registers
    "memory_max_head_dim": 256,
    "delta_chunk_max_head_dim": 256,        # a chunk's transposed q and k tiles in shared memory             # rows of a matrix memory's state (32 registers x 8 warps)
    "grid_dim_yz": 65535,                   # heads, KV heads and a step's entries map to grid dimensions y and z
}


def limit(name: str) -> int:
    """A size limit as the compiled library reports it."""
    f = getattr(library(), "se_" + name)
    f.restype = _I
    f.argtypes = []
    return int(f())


def _fn(name: str, sig: str):
    global launch_count
    launch_count += KERNELS_PER_CALL.get(name, 1)
    calls[name] = calls.get(name, 0) + 1
    f = _fns.get(name)
    if f is None:
        f = getattr(library(), name)
        f.restype = _I
        f.argtypes = [_SIG[c] for c in sig]
        _fns[name] = f
    return f


def _ptr(t: Optional[torch.Tensor], dtype=None, name: str = "tensor") -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    return t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _check(code: int, what: str) -> None:
    if code == 0:
        return
    if code in _ERRORS:
        raise ValueError(f"{what}: {_ERRORS[code]}")
    raise RuntimeError(f"{what}: CUDA error {code}")


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise TypeError(f"activation dtype must be float32 or bfloat16, got {dtype}") from None


# ---- elementwise -------------------------------------------------------------------------

def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    tokens, hidden = out.shape
    _check(_fn("se_embed_gather", "pppiiiip")(
        _ptr(table, out.dtype, "table"), _ptr(ids, torch.int32, "ids"), _ptr(out), tokens, hidden,
        table.shape[0], dtype_code(out.dtype), _stream()), "embed_gather")
    return out


def rmsnorm(x, w, eps: float, out, residual=None, residual_out=None):
    """out = rmsnorm(x [+ residual]) * w; with a residual, residual_out = x + residual."""
    rows, hidden = x.shape
    if (residual is None) != (residual_out is None):
        raise ValueError("residual and residual_out go together")
    if w.shape != (hidden,):
        raise ValueError(f"norm weight shape {tuple(w.shape)} does not match width {hidden}")
    _check(_fn("se_rmsnorm", "pppppiifip")(
        _ptr(x, None, "x"), _ptr(residual, x.dtype, "residual"), _ptr(w, x.dtype, "w"), _ptr(out, x.dtype, "out"),
        _ptr(residual_out, x.dtype, "residual_out"), rows, hidden, float(eps), dtype_code(x.dtype), _stream()),
        "rmsnorm")
    return out


def gather_rows(src, idx, out):
    rows, width = out.shape
    _check(_fn("se_gather_rows", "pppiiip")(
        _ptr(src, out.dtype, "src"), _ptr(idx, torch.int32, "idx"), _ptr(out), rows, width,
        dtype_code(out.dtype), _stream()), "gather_rows")
    return out


def table_update(table, updates, n: int, num_pages: int):
    """Apply ``n`` (row, index, page) triples to a block table of a pool of ``num_pages`` pages."""
    _check(_fn("se_table_update", "piipiipp")(
        _ptr(table, torch.int32, "table"), table.shape[0], table.shape[1], _ptr(updates, torch.int32, "updates"), n,
        num_pages, _ptr(error_word(table.device)), _stream()), "table_update")


def table_update_dyn(table, updates, count, max_n: int, num_pages: int):
    _check(_fn("se_table_update_dyn", "piippiipp")(
        _ptr(table, torch.int32, "table"), table.shape[0], table.shape[1], _ptr(updates, torch.int32, "updates"),
        _ptr(count, torch.int32, "count"), max_n, num_pages, _ptr(error_word(table.device)), _stream()),
        "table_update_dyn")


# ---- attention ---------------------------------------------------------------------------

ROTARY_PAIRING = {"split_half": 0, "interleaved_to_split_half": 1, "interleaved": 3}


def qk_prep(qkv, q_w, k_w, inv_freq, positions, token_seq, seq_rows, table, cache, q_out, *, num_heads,
            num_kv_heads, head_dim, rotary_dim, eps, rope_scale, page_size, write_cache=True,
            pairing: str = "split_half", num_pages=None, step_inputs_settled: bool = False):
    """``num_pages``: the pool the block table's entries must lie in (default: the pages ``cache``
    holds); an entry outside it is not followed and shows in the error word.
    ``step_inputs_settled``: ``positions`` were complete before the kernel launched just before this
    call (the one that writes ``qkv``) began; the rotation angles are then computed while it runs."""
    tokens = qkv.shape[0]
    dt = qkv.dtype
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise ValueError("qkv width does not match the head counts")
    if pairing not in ROTARY_PAIRING:
        raise ValueError(f"rotary pairing {pairing!r} is not known; known: {sorted(ROTARY_PAIRING)}")
    inv_rms = None
    if q_w is not None and tokens > 64:      # many tokens: norm statistics once per token, not once per head
        inv_rms = torch.empty(tokens, 2, dtype=torch.float32, device=qkv.device)
    _check(_fn("se_qk_prep", "pppppppp" "ipp" "iiiii" "ff" "iip" "iip" "iip")(
        _ptr(qkv, None, "qkv"), _ptr(q_w, dt, "q_norm"), _ptr(k_w, dt, "k_norm"),
        _ptr(inv_freq, torch.float32, "inv_freq"), _ptr(positions, torch.int32, "positions"),
        _ptr(token_seq, torch.int32, "token_seq"), _ptr(seq_rows, torch.int32, "seq_rows"),
        _ptr(table, torch.int32, "table"), table.shape[1], _ptr(cache, dt, "cache"), _ptr(q_out, dt, "q_out"),
        tokens, num_heads, num_kv_heads, head_dim, rotary_dim, float(eps), float(rope_scale),
        page_size, int(write_cache), _ptr(inv_rms), ROTARY_PAIRING[pairing],
        cache.shape[0] if num_pages is None else int(num_pages), _ptr(error_word(qkv.device)),
        int(bool(step_inputs_settled)), dtype_code(dt), _stream()), "qk_prep")
    return q_out


def _has_sink(sink) -> int:
    return 1 if isinstance(sink, torch.Tensor) else int(bool(sink))


def _sink_logits(sink, num_heads: int):
    """The pointer of a learned sink's logits (one 32-bit number per query head), or None."""
    if not isinstance(sink, torch.Tensor):
        return None
    if sink.shape != (num_heads,):
        raise ValueError(f"a learned sink has one logit per query head ({num_heads}), got {tuple(sink.shape)}")
    return _ptr(sink, torch.float32, "sink")


def paged_attention_plain(q, cache, table, seq_rows, token_seq, positions, out, *, num_heads, num_kv_heads,
                          head_dim, page_size, scale, window=None, num_pages=None, v_head_dim=None, softcap=None,
                          sink=False, gate=None, keep_first: int = 0):
    """``v_head_dim``: the values' head size where it differs from the queries' and keys'.
    ``softcap`` c: scaled scores become c tanh(s / c).  ``sink``: True: a key of score 0 without a value
    joins the softmax's denominator; a 32-bit tensor [num_heads]: its logit is the head's entry (unscaled).
    ``gate``: a matrix (rows may be a view with a pitch) whose sigmoid multiplies the output,
    [tokens, num_heads * v_head_dim].  ``keep_first`` n (with a window): keys 0..n-1 stay visible."""
    tokens = q.shape[0]
    dt = q.dtype
    if gate is not None and (gate.dim() != 2 or gate.stride(1) != 1 or gate.dtype != dt):
        raise ValueError("gate must be a matrix of q's dtype with contiguous rows")
    sink_logits = _sink_logits(sink, num_heads)
    _check(_fn("se_paged_attention_plain", "pppipppp" "iiiiii" "f" "iip" "fipi" "pi" "ip")(
        _ptr(q, None, "q"), _ptr(cache, dt, "cache"), _ptr(table, torch.int32, "table"), table.shape[1],
        _ptr(seq_rows, torch.int32, "seq_rows"), _ptr(token_seq, torch.int32, "token_seq"),
        _ptr(positions, torch.int32, "positions"), _ptr(out, dt, "out"), tokens, num_heads, num_kv_heads,
        head_dim, int(v_head_dim or head_dim), page_size, float(scale), int(window or 0),
        cache.shape[0] if num_pages is None else int(num_pages), _ptr(error_word(q.device)),
        float(softcap or 0.0), _has_sink(sink), gate.data_ptr() if gate is not None else None,
        gate.stride(0) if gate is not None else 0, sink_logits, int(keep_first or 0), dtype_code(dt), _stream()),
        "paged_attention_plain")
    return out


def qk_prep_general(proj, q_w, k_w, positions, token_seq, seq_rows, table, cache, q_out, *, num_heads, num_kv_heads,
                    head_dim, v_head_dim, eps, page_size, has_kv=True, temperature=None, num_pages=None,
                    inv_freq=None, rotary_dim: int = 0, v_first=None, v_mix=None, bias=None, per_head: bool = False):
    """Query/key preparation in 32-bit, rounded once: whole-projection RMS norms (optional), a rotation
    of the first ``rotary_dim`` dims of every head (split halves, angles ``position * inv_freq``), a query
    temperature ``(coef, every)`` (q times 1 + coef ln(floor((p+1)/every) + 1)), keys and values of
    different head sizes into their page; ``has_kv=False``: the row holds queries only.
    ``v_first`` (a matrix with contiguous rows, [tokens, kv heads * v_head_dim]) and ``v_mix`` (one 32-bit
    number on the device): the values written are ``(1 - v_mix) v + v_mix v_first``.
    ``bias`` (32-bit, one per column of the projection row): added before anything else.  ``per_head``: the
    norms are per head, with weights of ``head_dim`` elements shared by the heads."""
    tokens = proj.shape[0]
    if bias is not None and bias.numel() != num_heads * head_dim + (num_kv_heads * (head_dim + int(v_head_dim)) if has_kv else 0):
        raise ValueError("qk_prep_general: the bias has one entry per column of the projection row")
    dt = proj.dtype
    if proj.dim() != 2 or proj.stride(1) != 1:
        raise ValueError("proj must be a matrix with contiguous rows")
    coef, every = (float(temperature[0]), int(temperature[1])) if temperature else (0.0, 0)
    if v_first is not None and (v_first.dim() != 2 or v_first.stride(1) != 1 or v_first.dtype != dt or v_mix is None):
        raise ValueError("v_first must be a matrix of proj's dtype with contiguous rows, and comes with v_mix")
    _check(_fn("se_qk_prep_general", "pipp" "pipip" "ppp" "pi" "pp" "iiiii" "f" "fi" "iiip" "pi" "ip")(
        proj.data_ptr(), proj.stride(0), _ptr(q_w, dt, "q_norm"), _ptr(k_w, dt, "k_norm"),
        _ptr(inv_freq, torch.float32, "inv_freq"), int(rotary_dim), v_first.data_ptr() if v_first is not None else None,
        v_first.stride(0) if v_first is not None else 0, _ptr(v_mix, torch.float32, "v_mix") if v_first is not None else None,
        _ptr(positions, torch.int32, "positions"), _ptr(token_seq, torch.int32, "token_seq"),
        _ptr(seq_rows, torch.int32, "seq_rows"), _ptr(table, torch.int32, "table"), table.shape[1] if table is not None else 0,
        _ptr(cache, dt, "cache") if has_kv else None, _ptr(q_out, dt, "q_out"), tokens, num_heads, num_kv_heads, head_dim,
        int(v_head_dim), float(eps), coef, every, page_size, int(bool(has_kv)),
        (cache.shape[0] if num_pages is None else int(num_pages)) if has_kv else 0, _ptr(error_word(proj.device)),
        _ptr(bias, torch.float32, "bias"), int(bool(per_head)), dtype_code(dt), _stream()), "qk_prep_general")
    return q_out


# ---- a 32-bit residual stream (csrc/stream32.cu) -------------------------------------------------

ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "silu": 2, "relu": 3}


def embed_stream(table, ids, stream, act=None, scale: float = 1.0):
    """stream[t] = table[ids[t]] * scale in 32-bit; ``act``: the same rounded to the table's type."""
    tokens, hidden = stream.shape
    _check(_fn("se_embed_stream", "pppp" "iii" "f" "ip")(
        _ptr(table, None, "table"), _ptr(ids, torch.int32, "ids"), _ptr(stream, torch.float32, "stream"),
        _ptr(act, table.dtype, "act"), tokens, hidden, table.shape[0], float(scale), dtype_code(table.dtype), _stream()),
        "embed_stream")
    return stream


def add_layernorm(x, y, alpha: float, w, b, eps: float, out32=None, out_act=None):
    """Layer norm (weight ``w``, optional bias ``b``) of ``alpha * x + y``: ``x`` is the 32-bit
    stream, ``y`` (optional) has the weights' type; ``out32`` receives the result in 32-bit,
    ``out_act`` in the weights' type."""
    rows, hidden = x.shape
    dt = w.dtype
    if w.shape != (hidden,):
        raise ValueError(f"norm weight shape {tuple(w.shape)} does not match width {hidden}")
    _check(_fn("se_add_layernorm", "pp" "f" "pppp" "ii" "f" "ip")(
        _ptr(x, torch.float32, "x"), _ptr(y, dt, "y"), float(alpha), _ptr(w), _ptr(b, dt, "b"),
        _ptr(out32, torch.float32, "out32"), _ptr(out_act, dt, "out_act"), rows, hidden, float(eps), dtype_code(dt),
        _stream()), "add_layernorm")


def activation_(x, kind: str):
    """An activation of :data:`ACTIVATIONS` in place (32-bit arithmetic, rounded once)."""
    if kind not in ACTIVATIONS:
        raise ValueError(f"activation {kind!r} is not known; known: {sorted(ACTIVATIONS)}")
    _check(_fn("se_activation", "plii" "p")(_ptr(x, None, "x"), x.numel(), ACTIVATIONS[kind], dtype_code(x.dtype),
                                           _stream()), "activation")
    return x


def softcap_(x, cap: float):
    """x <- cap * tanh(x / cap) in place (32-bit arithmetic, rounded once)."""
    _check(_fn("se_softcap", "pl" "f" "ip")(_ptr(x, None, "x"), x.numel(), float(cap), dtype_code(x.dtype), _stream()),
           "softcap")
    return x


def add_rmsnorm_stream(x, y, w, eps: float, out32=None, out_act=None):
    """A pre-norm model's 32-bit stream: ``v = x + y`` (``y`` optional, activation type) goes to
    ``out32`` (which may be ``x``); ``out_act`` receives ``v / sqrt(mean(v^2) + eps) * w``, or, without
    a weight, ``v`` rounded to the activation type."""
    rows, hidden = x.shape
    dt = out_act.dtype if out_act is not None else (y.dtype if y is not None else torch.float32)
    if w is not None and w.shape != (hidden,):
        raise ValueError(f"norm weight shape {tuple(w.shape)} does not match width {hidden}")
    _check(_fn("se_add_rmsnorm_stream", "ppppp" "ii" "f" "ip")(
        _ptr(x, torch.float32, "x"), _ptr(y, dt, "y"), _ptr(w, dt, "w"), _ptr(out32, torch.float32, "out32"),
        _ptr(out_act, dt, "out_act"), rows, hidden, float(eps), dtype_code(dt), _stream()), "add_rmsnorm_stream")


def rmsnorm_add_stream(stream, y, w, eps: float, out_act=None):
    """A stream whose sublayers are normed on their way out: ``stream += y / sqrt(mean(y^2) + eps) * w``
    in place (32-bit); ``out_act`` receives the new stream rounded to ``y``'s type."""
    rows, hidden = stream.shape
    dt = y.dtype
    if w.shape != (hidden,) or y.shape != stream.shape:
        raise ValueError("rmsnorm_add_stream: y and w must match the stream's shape and width")
    _check(_fn("se_rmsnorm_add_stream", "pppp" "ii" "f" "ip")(
        _ptr(stream, torch.float32, "stream"), _ptr(y, None, "y"), _ptr(w, dt, "w"), _ptr(out_act, dt, "out_act"), rows,
        hidden, float(eps), dtype_code(dt), _stream()), "rmsnorm_add_stream")
    return stream


# ---- attention over a cached latent (csrc/latent_attention.cu) -----------------------------------

def latent_prep(proj, q_w, kv_w, inv_freq, positions, token_seq, seq_rows, table, cache, cq_out, *, q_rank, rank, rot,
                rotary_dim, eps, page_size, write_cache=True, num_pages=None):
    """From a step's rows ``[q latent | kv latent | shared key part]``: the normalised query latent
    (``cq_out``), and into each token's page slot the normalised kv latent and the rotated key part."""
    tokens = proj.shape[0]
    dt = proj.dtype
    if proj.dim() != 2 or proj.stride(1) != 1 or proj.shape[1] != q_rank + rank + rot:
        raise ValueError("proj must be [tokens, q_rank + rank + rot] with contiguous rows")
    _check(_fn("se_latent_prep", "pippp" "ppp" "pi" "pp" "iiiii" "f" "iii" "p" "ip")(
        proj.data_ptr(), proj.stride(0), _ptr(q_w, dt, "q_norm"), _ptr(kv_w, dt, "kv_norm"),
        _ptr(inv_freq, torch.float32, "inv_freq"), _ptr(positions, torch.int32, "positions"),
        _ptr(token_seq, torch.int32, "token_seq"), _ptr(seq_rows, torch.int32, "seq_rows"),
        _ptr(table, torch.int32, "table"), table.shape[1], _ptr(cache, dt, "cache"), _ptr(cq_out, dt, "cq_out"),
        tokens, q_rank, rank, rot, rotary_dim, float(eps), page_size,
        cache.shape[0] if num_pages is None else int(num_pages), int(bool(write_cache)), _ptr(error_word(proj.device)),
        dtype_code(dt), _stream()), "latent_prep")
    return cq_out


def latent_attention_plain(q_lat, q, inv_freq, cache, table, seq_rows, token_seq, positions, sink, out, *, heads,
                           head_dim, rank, rot, rotary_dim, page_size, scale, window=None, num_pages=None):
    """``q_lat`` float32 [heads, tokens, rank] (queries taken into the latent's space), ``q`` [tokens,
    heads * (head_dim + rot)] whose rotated parts are rotated here; ``out`` [tokens, heads, rank]."""
    tokens = q.shape[0]
    dt = q.dtype
    _check(_fn("se_latent_attention_plain", "ppipi" "ppi" "pppp" "p" "iiii" "i" "f" "ii" "p" "ip")(
        _ptr(q_lat, torch.float32, "q_lat"), _ptr(q, None, "q"), head_dim, _ptr(inv_freq, torch.float32, "inv_freq"),
        rotary_dim, _ptr(cache, dt, "cache"), _ptr(table, torch.int32, "table"), table.shape[1],
        _ptr(seq_rows, torch.int32, "seq_rows"), _ptr(token_seq, torch.int32, "token_seq"),
        _ptr(positions, torch.int32, "positions"), _ptr(sink, torch.float32, "sink"), _ptr(out, dt, "out"),
        tokens, heads, rank, rot, page_size, float(scale), int(window or 0),
        cache.shape[0] if num_pages is None else int(num_pages), _ptr(error_word(q.device)), dtype_code(dt), _stream()),
        "latent_attention_plain")
    return out


def latent_attention_tiled_supported(rank: int, rot: int) -> bool:
    """What ``se_latent_attention_tiled_supported`` answers, restated here so that asking does not compile
    the kernel (a GPU test compares the two)."""
    return rank > 0 and rot >= 0 and rank % 16 == 0 and rot % 16 == 0 and rank + rot <= 256


def latent_q_pack(q_lat, q, inv_freq, positions, qfull, *, heads, head_dim, rank, rot, rotary_dim):
    """``qfull[t, h] = [q_lat[h, t] | rotated part of q[t, h]]`` in bfloat16: the query rows of the tiled kernel."""
    tokens = q.shape[0]
    _check(_fn("se_latent_q_pack", "ppipi" "pp" "iiii" "p")(
        _ptr(q_lat, torch.float32, "q_lat"), _ptr(q, torch.bfloat16, "q"), head_dim, _ptr(inv_freq, torch.float32, "inv_freq"),
        rotary_dim, _ptr(positions, torch.int32, "positions"), _ptr(qfull, torch.bfloat16, "qfull"), tokens, heads, rank,
        rot, _stream()), "latent_q_pack")
    return qfull


def latent_tile_keys(max_q_len: int) -> int:
    """Keys per tile of the tiled latent attention: 32 for steps with prompt portions, 64 for steps of single tokens and
    short pieces (measured: 181 against 198 us over a 2,048-token prompt, 30.0 against 27.4 us for 64 decoding requests).
    ``SE_LATENT_TILE_KEYS`` forces one (a tuning aid; results do not depend on it beyond rounding)."""
    forced = os.environ.get("SE_LATENT_TILE_KEYS")
    if forced:
        return int(forced)
    return 32 if max_q_len >= 16 else 64


def latent_split_plan(row_tiles: int, entries: int, max_keys: int, sms: Optional[int] = None, tile_keys: int = 64):
    """How many CTAs share a row tile's keys, and how many 64-key tiles each takes.  Steps whose row
    tiles alone do not fill the device twice over (decode, short portions) over windows of several
    tiles are split along the keys; the merge kernel joins the parts."""
    if sms is None:
        sms = sm_count()
    tiles = -(-max_keys // tile_keys) + 1               # a window may straddle one more tile
    ctas = max(1, row_tiles * entries)
    if ctas >= 2 * sms or tiles < 4:
        return 1, tiles
    splits = min(-(-2 * sms // ctas), tiles // 2)
    per = -(-tiles // splits)
    return -(-tiles // per), per


def latent_attention_tiled(qfull, cache, table, seq_rows, cu_q, kv_len, sink, out, *, entries, max_q_len, heads, rank, rot,
                           page_size, scale, window=None, num_pages=None, max_keys=None, splits=None, tile_keys=None):
    """bfloat16, tensor-core tiles; ``qfull`` [tokens, heads, rank + rot], ``out`` [tokens, heads, rank].
    ``max_keys``: an upper bound of the keys a query of this step sees (window, or the longest
    request); with it, steps of few rows are split along the keys (``splits`` forces a count)."""
    tokens = qfull.shape[0]
    row_tiles = -(-max_q_len * heads // 64)
    if tile_keys is None:
        tile_keys = latent_tile_keys(max_q_len)
    per = 0
    if splits is None:
        splits, per = (latent_split_plan(row_tiles, entries, max_keys, sm_count(qfull.device), tile_keys)
                       if max_keys else (1, 0))
    elif splits > 1:
        per = -(-(-(-(max_keys or 0) // tile_keys) + 1) // splits)
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty(tokens * heads * splits * rank, dtype=torch.float32, device=qfull.device)
        part_ml = torch.empty(tokens * heads * splits * 2, dtype=torch.float32, device=qfull.device)
    global launch_count
    launch_count += 1 if splits > 1 else 0
    _check(_fn("se_latent_attention_tiled", "pppi" "ppp" "pp" "iiiiii" "i" "f" "ii" "p" "iipp" "i" "p")(
        _ptr(qfull, torch.bfloat16, "qfull"), _ptr(cache, torch.bfloat16, "cache"), _ptr(table, torch.int32, "table"),
        table.shape[1], _ptr(seq_rows, torch.int32, "seq_rows"), _ptr(cu_q, torch.int32, "cu_q"),
        _ptr(kv_len, torch.int32, "kv_len"), _ptr(sink, torch.float32, "sink"), _ptr(out, torch.bfloat16, "out"),
        tokens, entries, max_q_len, heads, rank, rot, page_size, float(scale), int(window or 0),
        cache.shape[0] if num_pages is None else int(num_pages), _ptr(error_word(qfull.device)), int(splits), int(per),
        _ptr(part_o), _ptr(part_ml), int(tile_keys), _stream()), "latent_attention_tiled")
    return out


# ---- retention (csrc/retention.cu) ----------------------------------------------------------------

def retention_prep(proj, q_off: int, k_off: int, inv_freq, positions, q32, k32, *, heads, head_dim, rotary_dim, k_scale):
    tokens = proj.shape[0]
    _check(_fn("se_retention_prep", "piii" "pp" "pp" "iiii" "f" "ip")(
        proj.data_ptr(), proj.stride(0), int(q_off), int(k_off), _ptr(inv_freq, torch.float32, "inv_freq"),
        _ptr(positions, torch.int32, "positions"), _ptr(q32, torch.float32, "q32"), _ptr(k32, torch.float32, "k32"),
        tokens, heads, head_dim, rotary_dim, float(k_scale), dtype_code(proj.dtype), _stream()), "retention_prep")


def retention_scan(q32, k32, proj, v_off: int, decay, state, step, o, *, heads, head_dim, v_head_dim):
    _check(_fn("se_retention_scan", "pp" "pii" "p" "pl" "pp" "p" "iiii" "ip")(
        _ptr(q32, torch.float32, "q32"), _ptr(k32, torch.float32, "k32"), proj.data_ptr(), proj.stride(0), int(v_off),
        _ptr(decay, torch.float32, "decay"), _ptr(state, torch.float32, "state"), state.stride(0), _ptr(step.cu_q),
        _ptr(step.seq_rows), _ptr(o, torch.float32, "o"), step.num_seqs, heads, head_dim, v_head_dim,
        dtype_code(proj.dtype), _stream()), "retention_scan")
    return o


def retention_segment_plan(entries: int, heads: int, v_head_dim: int, max_q_len: int, sms: Optional[int] = None):
    """``(segments per entry, tokens per segment)`` for the chunked recurrence.  A step whose (entry, head, 32
    columns) blocks fill less than half of the device runs each entry's tokens in segments side by side (each
    from a zero state; a second kernel joins them by the decay's powers, a third adds what the state at a
    segment's start contributes): a single long prompt is then as parallel as several.  As many segments as
    keep all blocks on the device at once (two per SM), of a multiple of 64 tokens and at least 256.
    Measured, 16 heads of 128 x 128, one 2,048-token prompt: 550 us in one pass, 326 in 4 segments; with 32
    heads (128 blocks) one pass is ahead, 568 against 660 us in 2 segments, hence the half."""
    if sms is None:
        sms = sm_count()
    blocks = entries * heads * (-(-v_head_dim // 32))
    segs = 2 * sms // max(blocks, 1)
    if segs < 4 or max_q_len <= 256:
        return 1, 0
    seg_len = max(256, -(-(-(-max_q_len // segs)) // 64) * 64)
    segs = -(-max_q_len // seg_len)
    return (segs, seg_len) if segs > 1 else (1, 0)


def retention_chunk(q32, k32, proj, v_off: int, decay, state, step, o, *, heads, head_dim, v_head_dim, segments=None):
    """The same recurrence as :func:`retention_scan` in chunks of 64 tokens (closed form per chunk, 32-bit
    FMA arithmetic): for steps that bring prompt portions.  ``segments``: ``(per entry, tokens each)``, default
    by :func:`retention_segment_plan`."""
    global launch_count
    max_seg, seg_len = segments if segments is not None else retention_segment_plan(
        step.num_seqs, heads, v_head_dim, step.max_q_len, sm_count(q32.device))
    seg_state = None
    if max_seg > 1:
        seg_state = torch.empty(step.num_seqs * max_seg * heads * head_dim * v_head_dim, dtype=torch.float32, device=q32.device)
        launch_count += 2
    _check(_fn("se_retention_chunk", "pp" "pii" "p" "pl" "pp" "p" "iiii" "iip" "ip")(
        _ptr(q32, torch.float32, "q32"), _ptr(k32, torch.float32, "k32"), proj.data_ptr(), proj.stride(0), int(v_off),
        _ptr(decay, torch.float32, "decay"), _ptr(state, torch.float32, "state"), state.stride(0), _ptr(step.cu_q),
        _ptr(step.seq_rows), _ptr(o, torch.float32, "o"), step.num_seqs, heads, head_dim, v_head_dim, int(max_seg),
        int(seg_len), _ptr(seg_state), dtype_code(proj.dtype), _stream()), "retention_chunk")
    return o


def retention_out(o, proj, g_off: int, out, *, heads, v_head_dim, eps):
    tokens = proj.shape[0]
    _check(_fn("se_retention_out", "ppii" "p" "iii" "f" "ip")(
        _ptr(o, torch.float32, "o"), proj.data_ptr(), proj.stride(0), int(g_off), _ptr(out, proj.dtype, "out"), tokens,
        heads, v_head_dim, float(eps), dtype_code(proj.dtype), _stream()), "retention_out")
    return out


# ---- mixers with a recurrent state (csrc/recurrent.cu) -------------------------------------------

def causal_conv(x, c0: int, w, bias, state, conv_off: int, step, out):
    """out[t, c] = silu(bias[c] + sum_j w[c, j] x[t - (taps-1-j), c0 + c]) over each request's own
    tokens; what lies before this step's tokens comes from the carried inputs in ``state`` (rows
    ``step.state_rows``, from element ``conv_off`` on, ``[taps-1, C]``), which are brought up to date."""
    tokens = x.shape[0]
    C, taps = w.shape
    _check(_fn("se_causal_conv", "pii" "pp" "pli" "ppp" "p" "iiii" "ip")(
        x.data_ptr(), x.stride(0), int(c0), _ptr(w, torch.float32, "conv weight"), _ptr(bias, torch.float32, "conv bias"),
        _ptr(state, torch.float32, "state"), state.stride(0), int(conv_off), _ptr(step.token_seq), _ptr(step.cu_q),
        _ptr(step.seq_rows), _ptr(out, torch.float32, "out"), tokens, step.num_seqs, C, taps, dtype_code(x.dtype),
        _stream()), "causal_conv")
    return out


def ssm_scan(xbc, proj, dt_off: int, dt_bias, a_log, d_skip, state, step, y, *, heads, head_dim, state_size, groups):
    tokens = xbc.shape[0]
    steps = torch.empty(tokens, heads, 2, dtype=torch.float32, device=xbc.device)     # step sizes and decays
    _check(_fn("se_ssm_scan", "ppii" "ppp" "pl" "pp" "pp" "iiiiii" "ip")(
        _ptr(xbc, torch.float32, "xbc"), proj.data_ptr(), proj.stride(0), int(dt_off), _ptr(dt_bias, torch.float32),
        _ptr(a_log, torch.float32), _ptr(d_skip, torch.float32), _ptr(state, torch.float32, "state"), state.stride(0),
        _ptr(step.cu_q), _ptr(step.seq_rows), _ptr(y, torch.float32, "y"), _ptr(steps), tokens, step.num_seqs, heads,
        head_dim, state_size, groups, dtype_code(proj.dtype), _stream()), "ssm_scan")
    return y


def gated_group_norm(y, proj, z_off: int, w, out, *, parts: int, eps: float):
    tokens, inner = y.shape
    _check(_fn("se_gated_group_norm", "ppii" "pp" "iii" "f" "ip")(
        _ptr(y, torch.float32, "y"), proj.data_ptr(), proj.stride(0), int(z_off), _ptr(w, torch.float32, "w"),
        _ptr(out, proj.dtype, "out"), tokens, inner, parts, float(eps), dtype_code(proj.dtype), _stream()),
        "gated_group_norm")
    return out


def delta_prep(qkv, a, proj, b_off: int, dt_bias, a_log, dec, beta, *, heads, kv_heads, head_dim, v_head_dim,
               unit_eps: float, q_scale: float, per_head: bool = False, log_dec=None):
    """``a``: the decay projection, ``[tokens, heads * head_dim]`` or (``per_head``) ``[tokens, heads]``; it may
    be a view of columns of the input projection (rows ``a.stride(0)`` apart).  ``log_dec`` (with ``per_head``):
    receives the decays' logarithms ``[tokens, heads]``, which the chunked recurrence reads."""
    if a.dtype != proj.dtype or a.stride(-1) != 1:
        raise TypeError("delta_prep: the decay projection must have the projection's type and unit column stride")
    _check(_fn("se_delta_prep", "ppipii" "pp" "pp" "iiiii" "ff" "ipip")(
        _ptr(qkv, torch.float32, "qkv"), a.data_ptr(), a.stride(0), proj.data_ptr(), proj.stride(0), int(b_off),
        _ptr(dt_bias, torch.float32), _ptr(a_log, torch.float32), _ptr(dec, torch.float32), _ptr(beta, torch.float32),
        qkv.shape[0], heads, kv_heads, head_dim, v_head_dim, float(unit_eps), float(q_scale), int(per_head),
        _ptr(log_dec, torch.float32, "log_dec"), dtype_code(proj.dtype), _stream()), "delta_prep")


def delta_scan(qkv, dec, beta, state, step, o, *, heads, kv_heads, head_dim, v_head_dim):
    _check(_fn("se_delta_scan", "ppp" "pl" "pp" "p" "iiiii" "p")(
        _ptr(qkv, torch.float32, "qkv"), _ptr(dec, torch.float32), _ptr(beta, torch.float32),
        _ptr(state, torch.float32, "state"), state.stride(0), _ptr(step.cu_q), _ptr(step.seq_rows),
        _ptr(o, torch.float32, "o"), step.num_seqs, heads, kv_heads, head_dim, v_head_dim, _stream()), "delta_scan")
    return o


def delta_chunk(qkv, log_dec, beta, state, step, o, *, heads, kv_heads, head_dim, v_head_dim):
    """The delta rule with one decay per head in chunks of 64 tokens (a triangular system per chunk, then three small
    matrix products; csrc/delta_chunk.cu): for steps with prompt portions.  ``log_dec`` [tokens, heads]: log decays."""
    _check(_fn("se_delta_chunk", "ppp" "pl" "pp" "p" "iiiii" "p")(
        _ptr(qkv, torch.float32, "qkv"), _ptr(log_dec, torch.float32, "log_dec"), _ptr(beta, torch.float32, "beta"),
        _ptr(state, torch.float32, "state"), state.stride(0), _ptr(step.cu_q), _ptr(step.seq_rows),
        _ptr(o, torch.float32, "o"), step.num_seqs, heads, kv_heads, head_dim, v_head_dim, _stream()), "delta_chunk")
    return o


def delta_out(o, gate, w, out, *, heads: int, v_head_dim: int, eps: float, silu: bool = False):
    """``gate`` [tokens, heads * v_head_dim] may be a view of columns of a projection; ``silu``: the gate is
    ``g * sigmoid(g)`` instead of ``sigmoid(g)``."""
    rows = o.numel() // v_head_dim
    if gate.dtype != out.dtype or gate.stride(-1) != 1:
        raise TypeError("delta_out: the gate must have the output's type and unit column stride")
    _check(_fn("se_delta_out", "ppipp" "iii" "f" "iip")(
        _ptr(o, torch.float32, "o"), gate.data_ptr(), gate.stride(0), _ptr(w, torch.float32, "w"), _ptr(out), rows,
        heads, v_head_dim, float(eps), int(silu), dtype_code(out.dtype), _stream()), "delta_out")
    return out


# ---- matrix memory (csrc/matrix_memory.cu) ---------------------------------------------------

def memory_gates(proj, i_off: int, f_off: int, bias, cap: float, state, m_off: int, step, gates, *, heads: int):
    """The gates of a matrix memory: ``gates[t, h] = (log keep, log take, exp(-m))`` from the log input and forget
    gates (columns ``i_off + h`` and ``f_off + h`` of the projection, plus ``bias`` [2, heads]), each
    ``cap tanh(. / cap)``; the running maximum ``m`` lives at ``state[row, m_off + h]`` and is brought up to date."""
    _check(_fn("se_memory_gates", "piii" "pf" "pli" "pp" "p" "ii" "ip")(
        proj.data_ptr(), proj.stride(0), int(i_off), int(f_off), _ptr(bias, torch.float32, "bias"), float(cap),
        _ptr(state, torch.float32, "state"), state.stride(0), int(m_off), _ptr(step.cu_q), _ptr(step.seq_rows),
        _ptr(gates, torch.float32, "gates"), step.num_seqs, heads, dtype_code(proj.dtype), _stream()), "memory_gates")
    return gates


def memory_scan(proj, q_off: int, k_off: int, v_off: int, gates, q_scale: float, state, step, o, *, heads, head_dim,
                v_head_dim):
    """``S <- keep S + take k [v | 1]^T``, ``o = S^T (q_scale q)`` token by token; ``state[row]`` starts with
    ``[heads, head_dim, v_head_dim + 1]``; ``o`` [tokens, heads, v_head_dim + 1] (the last column is n . q)."""
    _check(_fn("se_memory_scan", "piiii" "pf" "pl" "pp" "p" "iiii" "ip")(
        proj.data_ptr(), proj.stride(0), int(q_off), int(k_off), int(v_off), _ptr(gates, torch.float32, "gates"),
        float(q_scale), _ptr(state, torch.float32, "state"), state.stride(0), _ptr(step.cu_q), _ptr(step.seq_rows),
        _ptr(o, torch.float32, "o"), step.num_seqs, heads, head_dim, v_head_dim, dtype_code(proj.dtype), _stream()),
        "memory_scan")
    return o


def memory_chunk(proj, q_off: int, k_off: int, v_off: int, gates, q_scale: float, state, step, o, *, heads, head_dim,
                 v_head_dim, segments=None):
    """:func:`memory_scan` in chunks of 64 tokens (closed form per chunk): for steps with prompt portions.
    ``segments``: ``(per entry, tokens each)``, default by :func:`retention_segment_plan` (a single long prompt
    runs in segments side by side, joined by the sums of their log keeps)."""
    global launch_count
    max_seg, seg_len = segments if segments is not None else retention_segment_plan(
        step.num_seqs, heads, v_head_dim, step.max_q_len, sm_count(proj.device))
    seg_state = seg_logs = None
    if max_seg > 1:
        seg_state = torch.empty(step.num_seqs * max_seg * heads * head_dim * (v_head_dim + 1), dtype=torch.float32,
                                device=proj.device)
        seg_logs = torch.empty(step.num_seqs * max_seg * heads, dtype=torch.float64, device=proj.device)
        launch_count += 2
    _check(_fn("se_memory_chunk", "piiii" "pf" "pl" "pp" "p" "iiii" "iipp" "ip")(
        proj.data_ptr(), proj.stride(0), int(q_off), int(k_off), int(v_off), _ptr(gates, torch.float32, "gates"),
        float(q_scale), _ptr(state, torch.float32, "state"), state.stride(0), _ptr(step.cu_q), _ptr(step.seq_rows),
        _ptr(o, torch.float32, "o"), step.num_seqs, heads, head_dim, v_head_dim, int(max_seg), int(seg_len),
        _ptr(seg_state), _ptr(seg_logs), dtype_code(proj.dtype), _stream()), "memory_chunk")
    return o


def memory_out(o, gates, proj, g_off: int, w, out, *, heads, v_head_dim, eps: float, den_eps: float,
               out_scale: float = 1.0):
    """The read-out of a matrix memory: ``o / (max(|n . q|, exp(-m)) + den_eps)``, each head over its root mean
    square, times ``w`` [heads * v_head_dim], times sigmoid of the gate's projection (columns from ``g_off``)."""
    tokens = out.shape[0]
    _check(_fn("se_memory_out", "pppiip" "pi" "iii" "fff" "ip")(
        _ptr(o, torch.float32, "o"), _ptr(gates, torch.float32, "gates"), proj.data_ptr(), proj.stride(0), int(g_off),
        _ptr(w, torch.float32, "w"), out.data_ptr(), out.stride(0), tokens, heads, v_head_dim, float(eps),
        float(den_eps), float(out_scale), dtype_code(out.dtype), _stream()), "memory_out")
    return out


# ---- several residual streams (csrc/stream_mix.cu) -----------------------------------------------

def stream_embed(table, ids, streams, scale: float = 1.0):
    """streams[t, s] = table[ids[t]] * scale for every stream s (32-bit)."""
    tokens, S, width = streams.shape
    _check(_fn("se_stream_embed", "ppp" "iiii" "f" "ip")(
        _ptr(table, None, "table"), _ptr(ids, torch.int32, "ids"), _ptr(streams, torch.float32, "streams"), tokens, S,
        width, table.shape[0], float(scale), dtype_code(table.dtype), _stream()), "stream_embed")
    return streams


def stream_mix(streams, *, write=None, read=None, dtype, store: bool = True):
    """One kernel over ``streams`` [tokens, S, width] (32-bit, in place).  ``write = (y, gate, gate_bias, mix,
    out_w)``: ``x_t <- sum_s mix[s, t] x_s + out_w[t] * y'`` with ``y' = y * sigmoid(gate + gate_bias)`` (gate and
    bias optional).  ``read = (in_w, norm_w, eps, h)``: ``h = norm(sum_s in_w[s] x_s) * norm_w`` (``in_w`` None:
    ones), read after the write.  ``store=False``: the streams are left as they were."""
    tokens, S, width = streams.shape
    y = gate = gate_bias = mix = out_w = in_w = norm_w = h = None
    eps = 0.0
    if write is not None:
        y, gate, gate_bias, mix, out_w = write
    if read is not None:
        in_w, norm_w, eps, h = read
    _check(_fn("se_stream_mix", "piii" "pp" "pppp" "pf" "pi" "ip")(
        _ptr(streams, torch.float32, "streams"), tokens, S, width, _ptr(y, dtype, "y"), _ptr(gate, dtype, "gate"),
        _ptr(gate_bias, torch.float32, "gate_bias"), _ptr(mix, torch.float32, "mix"), _ptr(out_w, torch.float32, "out_w"),
        _ptr(in_w, torch.float32, "in_w"), _ptr(norm_w, torch.float32, "norm_w"), float(eps), _ptr(h, dtype, "h"),
        int(bool(store)), dtype_code(dtype), _stream()), "stream_mix")
    return h


def stream_sum(streams, out):
    tokens, S, width = streams.shape
    _check(_fn("se_stream_sum", "pp" "iii" "p")(
        _ptr(streams, torch.float32, "streams"), _ptr(out, torch.float32, "out"), tokens, S, width, _stream()), "stream_sum")
    return out


def scaled_sum(x, y, a: float, b: float, out, bias=None):
    """out = a * x + b * y (+ bias [width], 32-bit), 32-bit arithmetic, rounded once."""
    rows, width = out.shape
    _check(_fn("se_scaled_sum", "pp" "ff" "pp" "ii" "ip")(
        _ptr(x, out.dtype, "x"), _ptr(y, out.dtype, "y"), float(a), float(b), _ptr(bias, torch.float32, "bias"), _ptr(out),
        rows, width, dtype_code(out.dtype), _stream()), "scaled_sum")
    return out


# ---- feed-forward ------------------------------------------------------------------------

# "top_softmax": the bias is part of the logit, the largest logits are chosen and weighed by a softmax
# among themselves
SCORE_FN = {"sigmoid": 0, "softmax": 1, "top_softmax": 2}


def router(x, gate, bias, ids, weights, *, top_k, score_fn="sigmoid", renormalize=True, routed_scale=1.0,
           logits_out=None, groups: int = 1, keep_groups: int = 1):
    """32-bit router logits, scores, top-k and weights.  A token's logits are summed in one
    fixed order whatever the batch, so its experts do not depend on what shares its step.
    ``groups`` > 1: the experts form that many equal groups of neighbours, a group's score is the sum of
    its two largest selection scores, and only experts of the ``keep_groups`` best groups can be chosen."""
    tokens, hidden = x.shape
    experts = gate.shape[0]
    if gate.shape != (experts, hidden):
        raise ValueError("router weight shape does not match the activations")
    if logits_out is None:
        logits_out = torch.empty(tokens, experts, dtype=torch.float32, device=x.device)
    _check(_fn("se_router", "pppppp" "iiiii" "i" "f" "ii" "ip")(
        _ptr(x, None, "x"), _ptr(gate, torch.float32, "gate"), _ptr(bias, torch.float32, "bias"),
        _ptr(ids, torch.int32, "ids"), _ptr(weights, torch.float32, "weights"),
        _ptr(logits_out, torch.float32, "logits_out"), tokens, hidden, experts, top_k, SCORE_FN[score_fn],
        int(renormalize), float(routed_scale), int(groups), int(keep_groups), dtype_code(x.dtype), _stream()), "router")
    return ids, weights


def router_select(logits, bias, ids, weights, *, top_k, score_fn="sigmoid", renormalize=True, routed_scale=1.0,
                  impl="auto", groups: int = 1, keep_groups: int = 1):
    """Selection alone from given 32-bit logits [tokens, experts], or from their parts
    [chunks, tokens, terms, experts], whose sum over chunks and terms (taken in that order inside the
    kernel) is the logit.  ``impl``: "auto", "block" (a block per token, any size and score function)
    or "warp" (a warp per token: sigmoid scores, up to 256 experts)."""
    if logits.dim() == 4:
        chunks, tokens, terms, experts = logits.shape
    else:
        (tokens, experts), chunks, terms = logits.shape, 1, 1
    _check(_fn("se_router_select", "pii" "ppp" "iiiii" "f" "iii" "p")(
        _ptr(logits, torch.float32, "logits"), chunks, terms, _ptr(bias, torch.float32, "bias"),
        _ptr(ids, torch.int32, "ids"), _ptr(weights, torch.float32, "weights"), tokens, experts, top_k,
        SCORE_FN[score_fn], int(renormalize), float(routed_scale), {"auto": 0, "block": 1, "warp": 2}[impl], int(groups),
        int(keep_groups), _stream()), "router_select")
    return ids, weights


def moe_plain_tile_rows() -> int:
    f = library().se_moe_plain_tile_rows
    f.restype = _I
    return int(f())


def moe_route_build(ids, experts: int, tile_rows: int, ws: dict, gather=None, stats=None):
    """ws: int32 tensors counts[E], rank[A], offsets[E+1], sorted[A], inv_pos[A],
    tile_expert[max_tiles], tile_row0[max_tiles], num_tiles[1].
    gather = (x [tokens, width], xs [A, width], top_k): also xs[p] = x[sorted[p] // top_k], the
    activation rows in expert order (in the same launch when there are few assignments).
    stats: optional int64[2] on the device; [0] += experts that got a row, [1] += 1.
    Returns whether the lists were complete before the last kernel of the build began (the
    gather of rows as a launch of its own): a grouped GEMM launched next may then read them
    while that kernel still runs (``lists_settled``)."""
    global launch_count
    assignments = ids.numel()
    x = xs = None
    top_k = row_bytes = 1
    if gather is not None:
        x, xs, top_k = gather
        if x.dtype != xs.dtype or x.shape[1] != xs.shape[1] or xs.shape[0] != assignments:
            raise ValueError("gather: xs must be [assignments, width] of x's dtype")
        row_bytes = x.shape[1] * x.element_size()
    small = bool(library().se_moe_route_is_small(assignments, experts))
    launch_count += (0 if small else 1) + (0 if small or gather is None else 1)
    _check(_fn("se_moe_route_gather", "piiii" "pppppppp" "ppi" "pp")(
        _ptr(ids, torch.int32, "ids"), assignments, experts, tile_rows, top_k,
        *[_ptr(ws[k], torch.int32, k) for k in ("counts", "rank", "offsets", "sorted", "inv_pos", "tile_expert",
                                                 "tile_row0", "num_tiles")],
        _ptr(x, None, "x"), _ptr(xs, None, "xs"), row_bytes, _ptr(stats, torch.int64, "stats"), _stream()),
        "moe_route_build")
    return not small and gather is not None


def moe_max_tiles(assignments: int, experts: int, tile_rows: int) -> int:
    return -(-assignments // tile_rows) + min(experts, assignments)


# Gated activations of the experts' first product: ``silu`` is silu(gate) * up; ``clamped_swiglu`` is
# g sigmoid(alpha g) (u + 1) with g = min(gate, limit) and u = clamp(up, -limit, limit).
GLU_KINDS = {"silu": 0, "clamped_swiglu": 1}


def _glu_args(activation):
    """``activation``: a name of :data:`GLU_KINDS`, or ``(name, limit, alpha)``."""
    if activation is None or isinstance(activation, str):
        name, limit, alpha = activation or "silu", 0.0, 0.0
    else:
        name, limit, alpha = activation
    if name not in GLU_KINDS:
        raise ValueError(f"gated activation {name!r} is not known; known: {sorted(GLU_KINDS)}")
    return GLU_KINDS[name], float(limit), float(alpha)


def moe_grouped_gemm_plain(mode: int, a, w, ws: dict, route_w, out, *, max_tiles, n_out, k_dim, top_k, activation=None):
    dt = a.dtype
    _check(_fn("se_moe_grouped_gemm_plain", "i" "ppppppppp" "iiii" "iff" "ip")(
        mode, _ptr(a, None, "a"), _ptr(w, dt, "w"), _ptr(ws["sorted"]), _ptr(ws["offsets"]),
        _ptr(ws["tile_expert"]), _ptr(ws["tile_row0"]), _ptr(ws["num_tiles"]),
        _ptr(route_w, torch.float32, "route_w"), _ptr(out, dt, "out"), max_tiles, n_out, k_dim, top_k,
        *_glu_args(activation), dtype_code(dt), _stream()), "moe_grouped_gemm_plain")
    return out


def moe_combine(y, inv_pos, out, top_k: int, add=None, identity=None):
    """out[t] = the sum over the slots (32-bit, slot order) and, last, of ``add[t]`` ([tokens, hidden], optional:
    a shared expert's output), rounded once.  ``identity = (x, weights)``: a slot that got no row in the routing
    build (its expert has no weights) adds ``weights[t, slot] * x[t]``."""
    tokens, hidden = out.shape
    x, weights = identity if identity is not None else (None, None)
    _check(_fn("se_moe_combine", "ppppiiippip")(
        _ptr(y, out.dtype, "y"), _ptr(inv_pos, torch.int32, "inv_pos"), _ptr(add, out.dtype, "add"), _ptr(out), tokens,
        hidden, top_k, _ptr(x, out.dtype, "x"), _ptr(weights, torch.float32, "weights"), dtype_code(out.dtype), _stream()),
        "moe_combine")
    return out


# ---- tensor-core GEMMs (bf16; csrc/gemm_tc.cu) ---------------------------------------------

_error_words = {}

# What a code in the error word says (csrc/common.cuh).
_WAIT_ROLES = "a tensor-core kernel timed out waiting on a barrier (role code {code}); its results are not valid"
_INDEX_CODES = {21: "the q/k preparation kernel", 22: "the plain attention kernel", 23: "the split-key decode attention kernel",
                24: "the prompt-portion attention kernel", 25: "the tcgen05 prompt-portion attention kernel",
                26: "the block-table update kernel", 27: "the latent preparation kernel",
                28: "the latent attention kernel", 29: "the tiled latent attention kernel"}


def error_text(code: int) -> str:
    if code in _INDEX_CODES:
        return (f"{_INDEX_CODES[code]} was given a block-table entry outside its page pool (code {code}); "
                "the access was skipped, the step's results are not valid")
    return _WAIT_ROLES.format(code=code)


def error_word(device) -> torch.Tensor:
    """The device word the kernels write when a bounded wait runs out or an index they were
    given points outside what they may touch (0 = all fine; the first code stays).  One per
    device, created on first use."""
    t = _error_words.get(device)
    if t is None:
        key = _device_key(device)
        t = _error_words.get(key)
        if t is None:
            t = torch.zeros(1, dtype=torch.int32, device=key)
            _error_words[key] = t
    return t


def _device_key(device) -> torch.device:
    key = torch.device(device)
    return torch.device(key.type, torch.cuda.current_device()) if key.index is None else key


def error_check(device) -> None:
    """Raise if a kernel reported a failure (reads one word from the device)."""
    t = _error_words.get(_device_key(device))
    if t is not None:
        code = int(t.item())
        if code:
            t.zero_()
            raise RuntimeError(error_text(code))


_error_host = {}


def error_enqueue(device) -> None:
    """Queue a copy of the error word to pinned host memory on the current stream: the step
    function calls this after a forward pass and reads the copy (:func:`error_raise`) once
    it has synchronised for its own results, so the check costs no synchronisation of its own."""
    key = _device_key(device)
    t = _error_words.get(key)
    if t is None:
        return
    h = _error_host.get(key)
    if h is None:
        h = torch.zeros(1, dtype=torch.int32).pin_memory()
        _error_host[key] = h
    h.copy_(t, non_blocking=True)


def error_raise(device) -> None:
    """Raise if the copy queued by :func:`error_enqueue` (and since completed) shows a failure."""
    key = _device_key(device)
    h = _error_host.get(key)
    if h is not None and int(h[0]):
        code = int(h[0])
        h.zero_()
        _error_words[key].zero_()
        raise RuntimeError(error_text(code))


def gemm_tc_supported(k_dim: int, n_out: int, nt: int = 16) -> bool:
    f = library().se_gemm_tc_supported
    f.restype = _I
    f.argtypes = [_I, _I, _I]
    return bool(f(k_dim, n_out, nt))


def moe_tile_rows_tc(assignments: int, experts: int) -> int:
    """Activation rows per tile for the tensor-core grouped GEMM: the power of two in [16, 256]
    that is at least 4/3 of the mean number of rows per expert.  A tile that holds fewer rows
    (an expert's last one) runs MMAs of its own rows only, so a large tile wastes no tensor
    work; what a tile size costs is shared memory per stage, what it saves is that an expert's
    weights cross from L2 to an SM once per tile.  Measured at M2 sizes over 256 experts
    (expert layer, ms, best first): 512 tokens 32 > 64 > 16; 1,024 and 1,536 tokens 64 > 32, 128;
    3,072 tokens 128 > 256 > 64; 4,096 tokens and more 256 > 128."""
    forced = os.environ.get("SE_MOE_TILE_ROWS")          # tuning aid
    if forced:
        return int(forced)
    want = -(-4 * assignments // (3 * max(experts, 1)))
    nt = 16
    while nt < want and nt < 256:
        nt *= 2
    return nt


def moe_grouped_gemm_tc(mode: int, a, w, ws: dict, route_w, out, *, experts, max_tiles, n_out, k_dim, nt,
                        lists_settled: bool = False, activation=None):
    """``lists_settled``: the kernel launched just before this one does not write the lists in ``ws``
    (they were complete before it began).  The GEMM starts as a dependent of that kernel and then
    asks for its first weight tiles while it still runs; otherwise it waits for it first."""
    _check(_fn("se_moe_grouped_gemm_tc", "i" "pppppppppp" "iiiiiii" "iff" "p")(
        mode, _ptr(a, torch.bfloat16, "a"), _ptr(w, torch.bfloat16, "w"), _ptr(ws["sorted"]), _ptr(ws["offsets"]),
        _ptr(ws["tile_expert"]), _ptr(ws["tile_row0"]), _ptr(ws["num_tiles"]),
        _ptr(route_w, torch.float32, "route_w"), _ptr(out, torch.bfloat16, "out"), _ptr(error_word(a.device)),
        a.shape[0], experts, max_tiles, n_out, k_dim, nt, int(bool(lists_settled)), *_glu_args(activation), _stream()),
        "moe_grouped_gemm_tc")
    return out


PAIR_TILE_ROWS = 256      # activation rows per tile of the kernel that runs on pairs of SMs (csrc/gemm_tc_pair.cu)


def moe_grouped_gemm_pair_supported(k_dim: int, n_out: int) -> bool:
    f = library().se_moe_grouped_gemm_pair_supported
    f.restype = _I
    f.argtypes = [_I, _I]
    return bool(f(k_dim, n_out))


def moe_grouped_gemm_pair(mode: int, a, w, ws: dict, route_w, out, *, experts, max_tiles, n_out, k_dim, activation=None):
    """The grouped expert GEMM on pairs of SMs (``tcgen05.mma.cta_group::2``, tiles of 256 x 256); the
    tile list in ``ws`` must have been built with ``PAIR_TILE_ROWS`` rows per tile."""
    _check(_fn("se_moe_grouped_gemm_pair", "i" "pppppppppp" "iiiii" "iff" "p")(
        mode, _ptr(a, torch.bfloat16, "a"), _ptr(w, torch.bfloat16, "w"), _ptr(ws["sorted"]), _ptr(ws["offsets"]),
        _ptr(ws["tile_expert"]), _ptr(ws["tile_row0"]), _ptr(ws["num_tiles"]),
        _ptr(route_w, torch.float32, "route_w"), _ptr(out, torch.bfloat16, "out"), _ptr(error_word(a.device)),
        a.shape[0], experts, max_tiles, n_out, k_dim, *_glu_args(activation), _stream()), "moe_grouped_gemm_pair")
    return out


def gemm_tc_dense(x, w, out, nt: int = 128):
    rows, k_dim = x.shape
    n_out = w.shape[0]
    _check(_fn("se_gemm_tc_dense", "pppp" "iiii" "p")(
        _ptr(x, torch.bfloat16, "x"), _ptr(w, torch.bfloat16, "w"), _ptr(out, torch.bfloat16, "out"),
        _ptr(error_word(x.device)), rows, n_out, k_dim, nt, _stream()), "gemm_tc_dense")
    return out


# ---- decode attention on tensor cores (bf16; csrc/attention_decode.cu) ----------------------

def attn_decode_supported(head_dim: int, num_heads: int, num_kv_heads: int) -> bool:
    """What ``se_attn_decode_supported`` of the library answers, restated here so that asking does not
    compile the kernel for a model that cannot use it (a GPU test compares the two)."""
    return head_dim in (64, 128) and num_kv_heads > 0 and num_heads % num_kv_heads == 0


_sm_counts: dict = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device (asked once per device)."""
    key = torch.cuda.current_device() if device is None or torch.device(device).index is None else torch.device(device).index
    n = _sm_counts.get(key)
    if n is None:
        n = _sm_counts[key] = torch.cuda.get_device_properties(key).multi_processor_count
    return n


def attn_decode_plan(tokens: int, num_heads: int, num_kv_heads: int, max_keys: int, sms: Optional[int] = None,
                     ctas_per_sm: int = 2):
    """How many key splits, and how many keys each.  CTAs = tokens x KV heads x splits run in
    waves of ``sms * ctas_per_sm`` (``sms``: the device's count unless given; two CTAs of the
    kernel fit an SM by shared memory); a CTA costs its 64-key tiles plus about three tiles of
    fixed work.  Pick the split count with the least waves x cost."""
    if sms is None:
        sms = sm_count()
    group = num_heads // num_kv_heads
    base = tokens * num_kv_heads * (-(-group // 16))
    slots = sms * ctas_per_sm
    tiles = -(-max_keys // 64)
    best = None
    for s in range(1, max(1, tiles // 2) + 1):
        per_tiles = -(-tiles // s)
        if s > 1 and -(-tiles // per_tiles) != s:
            continue                                  # the same split size as a smaller count
        waves = -(-base * s // slots)
        cost = waves * (per_tiles + 3)
        if best is None or cost < best[0]:
            best = (cost, s, per_tiles)
    _, splits, per_tiles = best
    return splits, per_tiles * 64


def _softmax_options(q, gate, num_heads, v_head_dim, softcap, sink, keep_first=None):
    """The tail of the tensor-core attention kernels' arguments: cap, sink, gate pointer, gate pitch and, where
    ``keep_first`` is given (a number), the learned sink's logits and the count of first keys that stay visible."""
    if gate is not None and (gate.dim() != 2 or gate.stride(1) != 1 or gate.dtype != q.dtype
                             or gate.shape[1] != num_heads * v_head_dim):
        raise ValueError("gate must be a matrix [tokens, heads * value size] of q's dtype with contiguous rows")
    tail = (float(softcap or 0.0), _has_sink(sink), gate.data_ptr() if gate is not None else None,
            gate.stride(0) if gate is not None else 0)
    if keep_first is None:
        if isinstance(sink, torch.Tensor):
            raise ValueError("this kernel takes no learned sink")
        return tail
    return tail + (_sink_logits(sink, num_heads), int(keep_first))


def attn_decode_value_dim_supported(v_head_dim: int) -> bool:
    """Value head sizes the tensor-core kernels take beside a query/key head size they take."""
    return v_head_dim in (32, 64, 128)


def attn_decode(q, cache, table, seq_rows, token_seq, positions, out, *, num_heads, num_kv_heads, head_dim, page_size,
                scale, window=None, max_keys: int, num_pages=None, step_inputs_settled: bool = False, v_head_dim=None,
                softcap=None, sink=False, gate=None, keep_first: int = 0):
    """``step_inputs_settled``: ``table``, ``seq_rows``, ``token_seq`` and ``positions`` were complete
    before the kernel launched just before this call began (that kernel wrote ``q`` and the step's
    keys).  The attention kernel, launched as its dependent, then finds its place in the block table
    while it still runs; otherwise it waits for it first.  ``v_head_dim``, ``softcap``, ``sink`` and
    ``gate`` as :func:`paged_attention_plain`'s."""
    tokens = q.shape[0]
    dv = int(v_head_dim or head_dim)
    splits, per = attn_decode_plan(tokens, num_heads, num_kv_heads, max_keys, sms=sm_count(q.device))
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty(tokens * num_heads * splits * dv, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(tokens * num_heads * splits * 2, dtype=torch.float32, device=q.device)
    _check(_fn("se_attn_decode", "pppipppppp" "iiiiii" "f" "iii" "ip" "i" "fipi" "pi" "p")(
        _ptr(q, torch.bfloat16, "q"), _ptr(cache, torch.bfloat16, "cache"), _ptr(table, torch.int32, "table"),
        table.shape[1], _ptr(seq_rows, torch.int32, "seq_rows"), _ptr(token_seq, torch.int32, "token_seq"),
        _ptr(positions, torch.int32, "positions"), _ptr(out, torch.bfloat16, "out"), _ptr(part_o), _ptr(part_ml),
        tokens, num_heads, num_kv_heads, head_dim, dv, page_size, float(scale), int(window or 0), splits, per,
        cache.shape[0] if num_pages is None else int(num_pages), _ptr(error_word(q.device)),
        int(bool(step_inputs_settled)), *_softmax_options(q, gate, num_heads, dv, softcap, sink, keep_first or 0),
        _stream()), "attn_decode")
    return out


def attn_prefill(q, cache, table, seq_rows, cu_q, kv_len, out, *, entries, max_q_len, num_heads, num_kv_heads,
                 head_dim, page_size, scale, window=None, num_pages=None, v_head_dim=None, softcap=None,
                 sink=False, gate=None, keep_first: int = 0):
    dv = int(v_head_dim or head_dim)
    _check(_fn("se_attn_prefill", "pppipppp" "iiiiiii" "f" "i" "ip" "fipi" "pi" "p")(
        _ptr(q, torch.bfloat16, "q"), _ptr(cache, torch.bfloat16, "cache"), _ptr(table, torch.int32, "table"),
        table.shape[1], _ptr(seq_rows, torch.int32, "seq_rows"), _ptr(cu_q, torch.int32, "cu_q"),
        _ptr(kv_len, torch.int32, "kv_len"), _ptr(out, torch.bfloat16, "out"), entries, max_q_len, num_heads,
        num_kv_heads, head_dim, dv, page_size, float(scale), int(window or 0),
        cache.shape[0] if num_pages is None else int(num_pages), _ptr(error_word(q.device)),
        *_softmax_options(q, gate, num_heads, dv, softcap, sink, keep_first or 0), _stream()), "attn_prefill")
    return out


def attn_prefill_tc_supported(head_dim: int, num_heads: int, num_kv_heads: int) -> bool:
    """What ``se_attn_prefill_tc_supported`` answers (restated, as :func:`attn_decode_supported`)."""
    return head_dim == 128 and num_kv_heads > 0 and num_heads % num_kv_heads == 0


def attn_prefill_tc(q, cache, table, seq_rows, cu_q, kv_len, out, *, entries, max_q_len, num_heads, num_kv_heads,
                    head_dim, page_size, scale, window=None, num_pages=None, v_head_dim=None, softcap=None,
                    sink: bool = False, gate=None, keep_first: int = 0):
    """Prompt-portion attention on tcgen05 (head size 128, values of the same size)."""
    if int(v_head_dim or head_dim) != head_dim:
        raise ValueError("the tcgen05 prompt kernel takes values of the keys' head size")
    _check(_fn("se_attn_prefill_tc", "pppippppp" "iiiiii" "f" "ii" "fipi" "pi" "p")(
        _ptr(q, torch.bfloat16, "q"), _ptr(cache, torch.bfloat16, "cache"), _ptr(table, torch.int32, "table"),
        table.shape[1], _ptr(seq_rows, torch.int32, "seq_rows"), _ptr(cu_q, torch.int32, "cu_q"),
        _ptr(kv_len, torch.int32, "kv_len"), _ptr(out, torch.bfloat16, "out"), _ptr(error_word(q.device)),
        entries, max_q_len, num_heads, num_kv_heads, head_dim, page_size, float(scale), int(window or 0),
        cache.shape[0] if num_pages is None else int(num_pages),
        *_softmax_options(q, gate, num_heads, head_dim, softcap, sink, keep_first or 0), _stream()),
        "attn_prefill_tc")
    return out


# ---- dense projection for a handful of rows (bf16; csrc/gemv.cu) --------------------------------

def gemv_supported(rows: int, n_out: int, k_dim: int) -> bool:
    return 1 <= rows <= 16 and n_out >= 1 and k_dim >= 32 and k_dim % 32 == 0


def gemv(x, w, out):
    """out[rows <= 16, n] = x · wᵀ, weights streamed once through tensor-core fragments."""
    rows, k_dim = x.shape
    n_out = w.shape[0]
    _check(_fn("se_gemv", "pppiiip")(
        _ptr(x, torch.bfloat16, "x"), _ptr(w, torch.bfloat16, "w"), _ptr(out, torch.bfloat16, "out"), rows, n_out,
        k_dim, _stream()), "gemv")
    return out


# ---- read stream (csrc/read_stream.cu) ---------------------------------------------------------

def read_stream(t: torch.Tensor) -> None:
    """Read a contiguous tensor once with bulk asynchronous copies into shared memory, the way the
    weight-streaming GEMMs read HBM, and drop what arrives (a measuring aid: benchmarks time it)."""
    _check(_fn("se_read_stream", "plpp")(_ptr(t, None, "tensor"), t.numel() * t.element_size(),
                                         _ptr(error_word(t.device)), _stream()), "read_stream")
