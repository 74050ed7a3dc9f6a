"""ctypes binding of the kernel library and thin tensor-level wrappers.

Every wrapper checks dtype, device and contiguity, passes raw pointers and the
current CUDA stream, and raises on a non-zero return.  There is no fallback: without
a CUDA device or without the library these functions raise ``CUDAUnavailableError``.
"""

from __future__ import annotations

import ctypes
import os as _os
from ctypes import c_float, c_int, c_ulonglong, c_void_p

import torch

from ..errors import CUDAUnavailableError, ForgeEngineError, UnsupportedShapeError
from .build import attention_library_path, general_attention_library_path, library_path

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

STATUS_BITS = {
    1: "a token id lies outside the vocabulary",
    2: "a block-table entry is negative or outside the page pool",
    4: "a position lies outside its request's block table",
    8: "a bounded wait inside a kernel ran out",
    16: "logits contain NaN or +inf",
}

_ERRORS = {
    10001: "unsupported dtype combination",
    10002: "unsupported shape",
    10003: "pointer or stride not aligned as the kernel needs",
    10004: "size beyond what the kernel can launch",
}

_lib = None

# Kernel launches issued through this module since import (a claim for benchmarks).
LAUNCHES = 0


def lib() -> ctypes.CDLL:
    """Load (building first if needed) the kernel library exactly once."""
    global _lib
    if _lib is None:
        path = library_path()
        try:
            _lib = ctypes.CDLL(str(path))
        except OSError as error:
            raise CUDAUnavailableError(f"cannot load {path}: {error}") from error
        _declare(_lib)
    return _lib


def _declare(handle: ctypes.CDLL) -> None:
    p, i, f, ll = c_void_p, c_int, c_float, ctypes.c_longlong
    signatures = {
        "fe_embedding": [p, p, i, p, i, i, i, f, i, p, p, i, p, p],
        "fe_stream_mix_norm": [p, i, p, i, f, p, p, p, i, p, f, p, i, p, i, i, i, p],
        "fe_act_mul": [p, i, p, i, i, i, i, i, f, f, p],
        "fe_gated_rmsnorm": [p, p, i, i, p, p, i, i, i, f, p],
        "fe_qkv_prepare": [p, i, i, i, i, i, i, p, i, p, i, i, i, i, i, p, i, p, i, i, i, f, p, i, i, p, ll, ll, i,
                           p, p, i, p, i, i, i, p, p, i, p, p],
        "fe_attention_general": [p, ll, ll, p, i, i, p, i, i, p, ll, ll, i, p, i, i, i, i, i, p, p, p, p, i, i, f,
                                 i, f, f, i, i, ll, i, ll, p, ll, i, p, i, p, p],
        "fe_differential_combine": [p, p, i, ll, i, f, f, f, p],
        "fe_bias_xielu": [p, i, p, p, i, ll, i, f, f, p],
        "fe_bias_act": [p, i, p, p, i, ll, i, i, p],
        "fe_scale_cap": [p, ll, f, f, p],
        "fe_gated_recurrence": [p, ll, i, i, i, p, p, p, f, p, i, p, p, p, i, i, i, i, i, i, i, p, p, p],
        "fe_gated_recurrence_scratch": [i, i, i, i, i],
        "fe_gated_recurrence_long_from": [],
        "fe_add_normed_rmsnorm": [p, p, i, p, p, p, i, p, i, i, f, f, i, p, p, ll, p, i, p],
        "fe_causal_conv_state": [p, p, p, ll, p, p, p, p, i, i, i, i, i, p],
        "fe_moe_route": [p, ll, i, i, i, i, i, p, p, p, p, p, p, p, p, p, i, i, i, p, i, i, f, f, i, p],
        "fe_moe_grouped": [p, i, ll, p, p, i, p, i, i, i, i, i, p, p, p, p, p, i, f, f, i, p],
        "fe_moe_combine": [p, p, p, i, i, p, i, p, ll, p, i, i, p, i, p, i, p],
        "fe_moe_max_tiles": [i, i, i],
        "fe_linear_recurrence": [p, i, i, i, i, i, i, p, p, p, p, p, i, i, i, i, i, p],
        "fe_linear_recurrence_chunked": [p, i, i, i, i, i, i, p, p, p, p, p, p, i, i, i, i, i, i, p],
        "fe_linear_recurrence_chunks": [i, i],
        "fe_gemm_simt_batched": [p, i, p, i, p, i, i, i, i, i, ll, ll, ll, ll, ll, p],
        "fe_add_rmsnorm": [p, p, i, p, p, i, p, p, i, i, f, i, p],
        "fe_silu_mul": [p, p, i, i, i, i, p],
        "fe_qk_rope_cache": [p, i, p, p, f, p, p, i, p, p, p, p, p, i, i, i, i, i, i, i, i, p, p],
        "fe_qk_rope_cache_sums": [p, p, p, p, f, p, p, p, p, p, p, p, i, i, i, i, i, i, i, i, p, p],
        "fe_rope_table": [p, p, i, i, p, p],
        "fe_attention_simt": [p, i, i, p, p, p, i, i, i, p, p, i, f, p, i, i, i, i, p, p],
        "fe_gemm_simt": [p, i, p, i, p, p, i, i, i, i, i, p],
        "fe_sample": [p, i, i, p, p, p, p, p, p, p, p, p],
        "fe_gemm_tc5": [p, p, p, p, i, i, i, i, i, p, p, p, f, f, p],
        "fe_gemm_tc5_grouped": [p, p, p, i, i, i, i, i, i, i, p, p, p, f, f, p, p],
        "fe_moe_gather": [p, i, i, i, i, p, p, p, p],
        "fe_moe_logits": [p, i, p, p, i, i, i, p],
        "fe_gemm_tc5_qkv_rope": [p, p, p, p, i, i, i, p, p, f, p, p, p, p, p, p, i, i, i, i, i, i, p, p],
    }
    for name, argtypes in signatures.items():
        fn = getattr(handle, name)
        fn.argtypes = argtypes
        fn.restype = c_int
    handle.fe_gated_recurrence_scratch.restype = ctypes.c_longlong
    handle.fe_uniform_host.argtypes = [c_ulonglong, c_ulonglong]
    handle.fe_uniform_host.restype = c_float


_attention_libs: dict = {}
_attention_handles: dict = {}


def attention_lib(head_dim: int):
    """The tensor-core attention entry point compiled for ``head_dim`` (built on first use)."""
    fn = _attention_libs.get(head_dim)
    if fn is None:
        path = attention_library_path(head_dim)
        try:
            handle = ctypes.CDLL(str(path))
        except OSError as error:
            raise CUDAUnavailableError(f"cannot load {path}: {error}") from error
        fn = getattr(handle, f"fe_attention_mma_d{head_dim}")
        p, i, f = c_void_p, c_int, c_float
        fn.argtypes = [p, i, p, p, p, p, i, i, i, i, i, p, p, i, i, i, i, f, i, i, p, p, p, p]
        fn.restype = c_int
        _attention_libs[head_dim] = fn
        _attention_handles[head_dim] = handle
    return fn


PREFILL_TC5_ROWS = 128     # rows of a query tile of the tcgen05 prefill attention
PREFILL_TC5_KEYS = 128     # keys of one of its key tiles


def prefill_tc5_takes(dtype, head_dim: int, value_dim: int, groups: int, page_size: int) -> bool:
    """Whether the tcgen05 prefill attention runs for these sizes: bfloat16, keys and values of
    64 or 128, heads per kv head that divide a query tile, pages of 4 to 128 keys that divide a
    key tile."""
    return (dtype == torch.bfloat16 and head_dim == value_dim and head_dim in (64, 128) and groups >= 1
            and PREFILL_TC5_ROWS % groups == 0 and 4 <= page_size <= PREFILL_TC5_KEYS
            and PREFILL_TC5_KEYS % page_size == 0 and _os.environ.get("FORGE_ENGINE_GENERAL_TC5", "1") != "0")


def attention_prefill_tc5(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                          block_table: torch.Tensor, cu_tokens: torch.Tensor, starts: torch.Tensor, n_entries: int,
                          max_new: int, num_q_heads: int, window: int | None, keep_first: int, scale: float,
                          gate: torch.Tensor | None, row_lo: int, status: torch.Tensor,
                          distance_bias: torch.Tensor | None = None, softcap: float | None = None) -> None:
    """The tcgen05 prefill attention for the entries of a step with more than ``row_lo`` rows
    (new tokens x heads per kv head): ``q`` [N, heads * D] and ``out`` [N, heads * D] bfloat16,
    caches [pages, kv_heads, page_size, D].  ``window`` with ``keep_first``: keys below it
    stay visible; ``gate`` (32-bit [N, >= heads]): sigmoid gates per (token, head);
    ``distance_bias`` (32-bit [heads, L]): entry min(query position - key position, L - 1) of the
    head's row is added to the score before the scale, so it holds the bias over the scale;
    ``softcap`` c (not together with the bias): scaled scores become c tanh(score / c)."""
    _dense(q, "q"), _dense(out, "out"), _dense(k_cache, "k_cache"), _dense(v_cache, "v_cache"), _dense(block_table, "block_table")
    num_pages, nkv, page_size, d = k_cache.shape
    n = q.shape[0]
    assert q.dtype == out.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16 and v_cache.shape == k_cache.shape
    assert q.shape == out.shape == (n, num_q_heads * d) and num_q_heads % nkv == 0
    assert gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape[0] == n)
    handle = _attention_handle(d)
    fn = getattr(handle, f"fe_attention_prefill_tc5_d{d}")
    if not getattr(fn, "_declared", False):
        p, i, f, ll = c_void_p, c_int, c_float, ctypes.c_longlong
        fn.argtypes = [p, i, p, p, p, p, i, i, i, i, i, p, p, i, i, i, i, i, f, p, ll, i, p, i, f, p, p]
        fn.restype = c_int
        fn._declared = True
    assert not (softcap and distance_bias is not None)
    assert distance_bias is None or (distance_bias.dtype == torch.float32 and distance_bias.is_contiguous()
                                     and distance_bias.dim() == 2 and distance_bias.shape[0] == num_q_heads)
    gate_stride = 0 if gate is None else (int(gate.stride(0)) if n > 1 else int(gate.shape[1]))
    check(fn(ptr(q), int(q.shape[1]), ptr(out), ptr(k_cache), ptr(v_cache), ptr(block_table), block_table.shape[1],
             page_size, num_pages, nkv, num_q_heads // nkv, ptr(cu_tokens), ptr(starts), int(n_entries), int(max_new), n,
             int(window or 0), int(keep_first or 0), float(scale), ptr(gate), gate_stride, int(row_lo),
             ptr(distance_bias), 0 if distance_bias is None else int(distance_bias.shape[1]), float(softcap or 0.0),
             ptr(status), stream()), "attention_prefill_tc5")


def _attention_handle(head_dim: int):
    """The library compiled for ``head_dim`` (built and loaded on first use)."""
    attention_lib(head_dim)
    return _attention_handles[head_dim]


def has_symbol(name: str) -> bool:
    return hasattr(lib(), name)


def check(code: int, what: str) -> None:
    global LAUNCHES
    if code == 0:
        LAUNCHES += 1
        return
    if code in _ERRORS:
        raise UnsupportedShapeError(f"{what}: {_ERRORS[code]}")
    raise ForgeEngineError(f"{what}: CUDA error {code}")


# ---------------------------------------------------------------------------
# scratch memory with canary words
# ---------------------------------------------------------------------------

CANARY = 0x5AFEC0DE
GUARD_BYTES = 256


class GuardedBuffer:
    """A device buffer with ``GUARD_BYTES`` of a fixed bit pattern before and after it.

    Stands in for a memory checker: a kernel that writes one element before or past its
    scratch (or its cache pool) changes a canary word, which ``damaged()`` reports."""

    def __init__(self, name: str, numel: int, dtype: torch.dtype, device, zero: bool = False) -> None:
        self.name = name
        item = torch.empty((), dtype=dtype).element_size()
        guard = GUARD_BYTES // item
        body = -(-max(1, numel) // guard) * guard          # the rear guard starts 256-byte aligned
        flat = (torch.zeros if zero else torch.empty)(guard + body + guard, dtype=dtype, device=device)
        self._flat = flat
        self.data = flat[guard : guard + numel]
        self._guards = (flat[:guard].view(torch.int32), flat[guard + body :].view(torch.int32))
        for words in self._guards:
            words.fill_(CANARY)

    def numel(self) -> int:
        return self.data.numel()

    def damaged(self) -> torch.Tensor:
        """0-d bool tensor on the device: a canary word was overwritten."""
        return (self._guards[0] != CANARY).any() | (self._guards[1] != CANARY).any()


class _Scratch:
    """Scratch buffers of this module, per (kind, device).  A buffer that turns out too
    small is replaced by a larger one; the old one stays referenced, because a captured CUDA
    graph may still hold its address."""

    def __init__(self) -> None:
        self.current: dict = {}
        self.all: list = []

    def get(self, kind: str, device, numel: int, dtype: torch.dtype, floor: int, zero: bool = False) -> torch.Tensor:
        key = (kind, torch.device(device))
        buffer = self.current.get(key)
        if buffer is None or buffer.numel() < numel:
            buffer = GuardedBuffer(f"{kind} scratch", max(numel, floor), dtype, device, zero)
            self.current[key] = buffer
            self.all.append(buffer)
        return buffer.data


_scratch = _Scratch()


def damaged_canaries(extra=()) -> list:
    """Names of the scratch buffers of this module (and of ``extra`` GuardedBuffers, such as
    the cache pools) whose canary words no longer hold their pattern; synchronises."""
    buffers = list(_scratch.all) + list(extra)
    if not buffers:
        return []
    by_device: dict = {}
    for buffer in buffers:
        by_device.setdefault(buffer.data.device, []).append(buffer)
    bad = []
    for group in by_device.values():
        flags = torch.stack([b.damaged() for b in group]).cpu().tolist()
        bad.extend(b.name for b, flag in zip(group, flags) if flag)
    return bad


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise CUDAUnavailableError("no CUDA device: this engine runs on the GPU only")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream() -> int:
    """Handle of the current CUDA stream of the current device (asked for at every launch: a
    graph capture runs on a stream of its own)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise UnsupportedShapeError(f"dtype {t.dtype} is neither float32 nor bfloat16") from None


def _dense(t: torch.Tensor, name: str) -> torch.Tensor:
    if not t.is_cuda:
        raise CUDAUnavailableError(f"{name} must live on the CUDA device")
    if not t.is_contiguous():
        raise UnsupportedShapeError(f"{name} must be contiguous")
    return t


# ---------------------------------------------------------------------------
# wrappers
# ---------------------------------------------------------------------------


def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, status: torch.Tensor,
              scale: float = 1.0, positions: torch.Tensor | None = None, position_table: torch.Tensor | None = None) -> None:
    """out[n] = float(table[ids[n]]) * scale; out is the 32-bit residual stream [N, H], or
    [N, S, H] for S copies of it (every copy gets the same row).  With ``position_table``
    [places, H] (dtype of ``table``) row ``positions[n]`` of it is added, unscaled."""
    _dense(ids, "ids"), _dense(table, "table"), _dense(out, "out")
    assert ids.dtype == torch.int32 and out.dtype == torch.float32
    n, hidden = out.shape[0], out.shape[-1]
    copies = out.shape[1] if out.dim() == 3 else 1
    assert table.shape[1] == hidden
    places = 0
    if position_table is not None:
        _dense(position_table, "position_table")
        assert position_table.dtype == table.dtype and position_table.shape[1] == hidden
        assert positions is not None and positions.dtype == torch.int32 and positions.numel() == n
        places = position_table.shape[0]
    check(
        lib().fe_embedding(ptr(ids), ptr(table), code(table), ptr(out), n, hidden, table.shape[0],
                           float(scale), int(copies), ptr(positions) if position_table is not None else None,
                           ptr(position_table), int(places), ptr(status), stream()),
        "embedding",
    )


NORM_NONE, NORM_RMS, NORM_LAYER = 0, 1, 2
MAX_STREAMS = 16


def stream_mix_norm(
    streams: torch.Tensor,
    update: torch.Tensor | None,
    update_scale: float,
    mix: torch.Tensor | None,
    out_coef: torch.Tensor | None,
    in_coef: torch.Tensor | None,
    norm_kind: int,
    weight: torch.Tensor | None,
    eps: float,
    out: torch.Tensor | None,
    row_map: torch.Tensor | None = None,
    write_streams: bool = True,
) -> None:
    """One launch over the residual streams [N, S, W] (32-bit; [N, W] is S = 1):
    x'_t = sum_s mix[s, t] x_s + update_scale * out_coef[t] * update (only with ``update``;
    ``mix`` None is the identity, ``out_coef`` None ones), written back unless
    ``write_streams`` is false; u = sum_t in_coef[t] x'_t (None: ones); ``out`` = norm(u) *
    weight (``NORM_RMS``, ``NORM_LAYER`` - mean taken off, variance as the mean squared
    deviation - or ``NORM_NONE``: u itself).  ``out`` None only updates the streams.  With
    ``row_map`` row r of ``out`` comes from token ``row_map[r]``."""
    _dense(streams, "streams")
    assert streams.dtype == torch.float32
    n, width = streams.shape[0], streams.shape[-1]
    count = streams.shape[1] if streams.dim() == 3 else 1
    if update is not None:
        _dense(update, "update")
        assert update.shape == (n, width)
    for name, t, numel in (("mix", mix, count * count), ("out_coef", out_coef, count), ("in_coef", in_coef, count),
                           ("weight", weight, width)):
        assert t is None or (t.dtype == torch.float32 and t.is_cuda and t.is_contiguous() and t.numel() == numel), name
    rows = n if row_map is None else row_map.numel()
    if out is not None:
        _dense(out, "out")
        assert out.shape == (rows, width)
    assert row_map is None or row_map.dtype == torch.int32
    check(
        lib().fe_stream_mix_norm(
            ptr(streams), count, ptr(update), code(update) if update is not None else F32, float(update_scale),
            ptr(mix), ptr(out_coef), ptr(in_coef), int(norm_kind), ptr(weight), float(eps), ptr(out),
            code(out) if out is not None else F32, ptr(row_map), rows, width, 1 if write_streams else 0, stream(),
        ),
        "stream_mix_norm",
    )


ACT_SILU, ACT_GELU_TANH, ACT_CLAMPED_SWISH = 0, 1, 2


def act_mul(gate_up: torch.Tensor, out: torch.Tensor, act: int, block: int = 0, limit: float = 0.0,
            slope: float = 1.0) -> None:
    """out[n, i] = act(gate) * up in 32-bit, rounded on store; for ACT_CLAMPED_SWISH
    g' sigmoid(slope g') (u' + 1) with g' = min(gate, limit), u' = clamp(up, -limit, limit).
    ``block`` 0: a row of ``gate_up`` is all gate features then all up features; ``block`` B:
    it alternates B gate, B up features."""
    _dense(gate_up, "gate_up"), _dense(out, "out")
    rows, inter = out.shape
    assert gate_up.shape == (rows, 2 * inter)
    check(lib().fe_act_mul(ptr(gate_up), code(gate_up), ptr(out), code(out), rows, inter, int(act), int(block),
                           float(limit), float(slope), stream()), "act_mul")


def differential_combine(maps: torch.Tensor, out: torch.Tensor, value_dim: int, lam: float, eps: float, mult: float) -> None:
    """``maps`` 32-bit [N, heads * 2 * value_dim] holds two attention maps per head side by
    side; out[N, heads * value_dim] = (a1 - lam a2) / sqrt(mean((a1 - lam a2)^2) + eps) * mult
    per head, in 32-bit, rounded on store."""
    _dense(maps, "maps"), _dense(out, "out")
    assert maps.dtype == torch.float32 and maps.numel() == 2 * out.numel() and out.numel() % value_dim == 0
    check(lib().fe_differential_combine(ptr(maps), ptr(out), code(out), out.numel() // value_dim, int(value_dim),
                                        float(lam), float(eps), float(mult), stream()), "differential_combine")


def moe_max_tiles(slots: int, experts: int, tile_rows: int = 0) -> int:
    """Row tiles the grouped products are launched with for ``slots`` (token, choice) pairs cut
    into tiles of ``tile_rows`` rows (0: the 64 of the plain grouped kernels)."""
    return int(lib().fe_moe_max_tiles(int(slots), int(experts), int(tile_rows)))


def moe_logits(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[n, r] = x[n] . w[r] for a handful of 32-bit rows ``w`` (a router), in plain 32-bit
    FMAs whatever the dtype of ``x``."""
    _dense(x, "x"), _dense(w, "w"), _dense(out, "out")
    n, k = x.shape
    assert w.dtype == torch.float32 and out.dtype == torch.float32 and w.shape[1] == k and out.shape == (n, w.shape[0])
    check(lib().fe_moe_logits(ptr(x), code(x), ptr(w), ptr(out), n, int(w.shape[0]), int(k), stream()), "moe_logits")


def moe_gather(x: torch.Tensor, plan: dict, top: int, slot_weight: torch.Tensor | None, out: torch.Tensor) -> None:
    """out[row] = x[token of the row's slot] (times the slot's weight), rows sorted by expert."""
    _dense(x, "x"), _dense(out, "out")
    slots, width = out.shape
    assert x.shape[1] == width and out.dtype == x.dtype and slots == x.shape[0] * top
    check(lib().fe_moe_gather(ptr(x), code(x), int(width), int(top), int(slots), ptr(plan["row_slot"]), ptr(slot_weight),
                              ptr(out), stream()), "moe_gather")


def gemm_tc5_grouped(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int, plan: dict, tile_rows: int,
                     max_tiles: int, status: torch.Tensor, limit: float = 0.0, slope: float = 1.0) -> None:
    """The tcgen05 product over rows sorted by expert: ``x`` [slots, k], ``w`` [experts, o, k],
    ``out`` [slots, o] (epilogue 0: bfloat16, 1: 32-bit) or [slots, o / 2] (the gated
    epilogues, for ``w`` whose rows alternate 16 gate and 16 up features).  ``plan`` is what
    ``moe_route`` made with the same ``tile_rows`` and ``max_tiles``."""
    _dense(x, "x"), _dense(w, "w"), _dense(out, "out")
    slots, k = x.shape
    experts, o, _ = w.shape
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[2] == k and k % 8 == 0
    gated = epilogue in (TC5_SILU_MUL, TC5_GELU_MUL, TC5_CLAMP_MUL)
    assert out.shape == (slots, o // 2 if gated else o)
    assert out.dtype == (torch.float32 if epilogue == TC5_STORE_F32 else torch.bfloat16)
    # epilogues 7 and 8 (``TC5_UNARY``) store an activation of one argument of every sum
    check(lib().fe_gemm_tc5_grouped(ptr(x), ptr(w), ptr(out), int(slots), int(experts), int(o), int(k), int(epilogue),
                                    int(tile_rows), int(max_tiles), ptr(plan["tile_expert"]), ptr(plan["tile_row"]),
                                    ptr(plan["offsets"]), float(limit), float(slope), ptr(status), stream()),
          "gemm_tc5_grouped")


def moe_route(logits: torch.Tensor, experts: int, top: int, softmax: bool, renormalise: bool, counts: torch.Tensor,
              ints: torch.Tensor, slot_weight: torch.Tensor, max_tiles: int, tile_rows: int = 0, *,
              identity: int = 0, correction: torch.Tensor | None = None, groups: tuple | None = None,
              renorm_floor: float = 0.0, weight_scale: float = 1.0, group_top2: bool = False) -> dict:
    """Choose ``top`` of ``experts`` per token from 32-bit ``logits`` [N, >= experts] and lay
    the (token, choice) slots out by expert.  ``counts`` int32 [experts + 1] must be zero (it is
    zero again afterwards); ``ints`` is int32 scratch of at least 4 * N * top + experts + 2 +
    2 * max_tiles elements.  Returns views of it by name.

    ``identity``: the router has that many outputs more, for units that hand their input on;
    a slot that chose one gets expert number ``experts`` (rows, but no tiles).  ``correction``
    (32-bit [experts + identity]) is added to the scores for the choice only.  ``groups``
    (count, keep): the outputs form ``count`` equal groups of neighbours and only those of the
    ``keep`` groups with the largest choice score (``group_top2``: with the largest sum of their
    two largest choice scores) can be chosen.  Weights are the chosen scores
    (divided by their sum + ``renorm_floor`` with ``renormalise``) times ``weight_scale``."""
    n = logits.shape[0]
    slots = n * top
    outputs = experts + int(identity)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and logits.shape[1] >= outputs
    assert counts.dtype == torch.int32 and counts.numel() >= experts + 1 and ints.dtype == torch.int32
    assert slot_weight.dtype == torch.float32 and slot_weight.numel() >= slots
    assert ints.numel() >= 4 * slots + experts + 2 + 2 * max_tiles
    assert correction is None or (correction.dtype == torch.float32 and correction.numel() == outputs and correction.is_cuda)
    group_count, group_keep = groups or (0, 0)
    names = (("slot_expert", slots), ("slot_rank", slots), ("slot_row", slots), ("row_slot", slots),
             ("offsets", experts + 2), ("tile_expert", max_tiles), ("tile_row", max_tiles))
    views, at = {}, 0
    for name, count in names:
        views[name] = ints[at : at + count]
        at += count
    check(lib().fe_moe_route(ptr(logits), int(logits.stride(0)) if n > 1 else int(logits.shape[1]), n, int(experts),
                             int(top), 1 if softmax else 0, 1 if renormalise else 0, ptr(counts),
                             ptr(views["slot_expert"]), ptr(slot_weight), ptr(views["slot_rank"]), ptr(views["slot_row"]),
                             ptr(views["row_slot"]), ptr(views["offsets"]), ptr(views["tile_expert"]),
                             ptr(views["tile_row"]), int(max_tiles), int(tile_rows), int(identity), ptr(correction),
                             int(group_count), int(group_keep), float(renorm_floor), float(weight_scale),
                             1 if group_top2 else 0, stream()), "moe_route")
    global LAUNCHES
    LAUNCHES += 1
    return views


def moe_grouped(a: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor | None, out: torch.Tensor, plan: dict, top: int,
                max_tiles: int, *, gather: bool, slot_weight: torch.Tensor | None = None, act: int = 0,
                limit: float = 0.0, slope: float = 1.0) -> None:
    """One product over rows grouped by expert.  ``w1`` (and ``w2``) [experts, n, k];
    ``gather``: ``a`` holds the tokens' activations [N, k] and a sorted row reads its slot's
    token, times ``slot_weight`` when given; else ``a`` holds sorted rows [slots, k].  With
    ``w2``: out = act(a w1^T, a w2^T) (see ``act_mul``), else out = a w1^T, or an activation of
    one argument of it when ``act`` is one of ``MOE_UNARY``'s codes."""
    _dense(a, "a"), _dense(w1, "w1"), _dense(out, "out")
    experts, n, k = w1.shape
    assert a.shape[1] == k and out.shape[1] == n and (w2 is None or (w2.shape == w1.shape and w2.dtype == w1.dtype))
    use_mma = (a.dtype == torch.bfloat16 and w1.dtype == torch.bfloat16 and k % 8 == 0
               and _os.environ.get("FORGE_ENGINE_MOE_MMA", "1") != "0")
    check(lib().fe_moe_grouped(ptr(a), code(a), int(k), ptr(w1), ptr(w2), code(w1), ptr(out), code(out), int(n), int(k),
                               int(top), int(max_tiles), ptr(plan["offsets"]), ptr(plan["tile_expert"]),
                               ptr(plan["tile_row"]), ptr(plan["row_slot"]) if gather else None,
                               ptr(slot_weight) if gather else None, int(act), float(limit), float(slope),
                               1 if use_mma else 0, stream()), "moe_grouped")


def moe_combine(rows: torch.Tensor, plan: dict, top: int, out: torch.Tensor, *, slot_weight: torch.Tensor | None = None,
                shared: torch.Tensor | None = None, shared_logit: torch.Tensor | None = None,
                identity_input: torch.Tensor | None = None, experts: int = 0) -> None:
    """out[token] = sum over the token's slots of rows[slot's row] (times ``slot_weight``) +
    sigmoid(shared_logit[token]) * shared[token] (the gate 1 without a logit); 32-bit sums.
    With ``identity_input`` [N, width] a slot whose expert number is ``experts`` or above
    contributes the token's row of it instead of a row of ``rows``."""
    _dense(rows, "rows"), _dense(out, "out")
    n, width = out.shape
    assert rows.dtype == torch.float32 and rows.shape == (n * top, width)
    assert shared is None or (shared.shape == out.shape and shared.is_contiguous())
    assert shared_logit is None or (shared_logit.dtype == torch.float32 and shared_logit.shape[0] == n)
    assert identity_input is None or (identity_input.shape == out.shape and identity_input.is_contiguous())
    check(lib().fe_moe_combine(ptr(rows), ptr(plan["slot_row"]), ptr(slot_weight), int(top), int(width), ptr(shared),
                               code(shared) if shared is not None else F32, ptr(shared_logit),
                               int(shared_logit.stride(0)) if shared_logit is not None and n > 1 else 1,
                               ptr(out), code(out), n, ptr(plan["slot_expert"]), int(experts), ptr(identity_input),
                               code(identity_input) if identity_input is not None else F32, stream()), "moe_combine")


CONV_MAX_TAPS = 8      # what causal_conv_state takes


def bias_xielu(x: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor, a_pos: float, a_neg: float) -> None:
    """out = act(x + bias), act(z) = a_pos z^2 + z / 2 above zero and a_neg (exp(z) - 1 - z) + z / 2
    at and below it; taken in 32-bit, one rounding on store.  ``bias`` 32-bit [C] or None."""
    _dense(x, "x"), _dense(out, "out")
    rows, width = x.shape
    assert out.shape == x.shape and (bias is None or (bias.dtype == torch.float32 and bias.numel() == width))
    check(lib().fe_bias_xielu(ptr(x), code(x), ptr(bias), ptr(out), code(out), rows, width, float(a_pos), float(a_neg),
                              stream()), "bias_xielu")


UNARY_GELU_TANH, UNARY_RELU2 = 0, 1      # activations of one argument (``bias_act``)
TC5_UNARY = {UNARY_RELU2: 7, UNARY_GELU_TANH: 8}      # -> epilogue of the tcgen05 product that stores act(sum + bias) in bfloat16
MOE_UNARY = {None: 16, UNARY_RELU2: 17, UNARY_GELU_TANH: 18}   # -> what ``moe_grouped`` applies to a single product's sums


def bias_act(x: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor, act: int) -> None:
    """out = act(x + bias) for an activation of one argument (``UNARY_GELU_TANH``: the tanh form
    of GELU; ``UNARY_RELU2``: the square of relu), taken in 32-bit, one rounding on store.
    ``bias`` 32-bit [C] or None."""
    _dense(x, "x"), _dense(out, "out")
    rows, width = x.shape
    assert out.shape == x.shape and (bias is None or (bias.dtype == torch.float32 and bias.numel() == width))
    check(lib().fe_bias_act(ptr(x), code(x), ptr(bias), ptr(out), code(out), rows, width, int(act), stream()), "bias_act")


def scale_cap(x: torch.Tensor, scale: float, cap: float | None) -> None:
    """In place on 32-bit values: x <- x * scale, then with a cap x <- cap * tanh(x / cap)."""
    _dense(x, "x")
    assert x.dtype == torch.float32
    check(lib().fe_scale_cap(ptr(x), x.numel(), float(scale), float(cap or 0.0), stream()), "scale_cap")


def gated_recurrence(proj: torch.Tensor, q_off: int, f_off: int, v_off: int, f_bias: torch.Tensor | None,
                     lower: torch.Tensor, norm_weight: torch.Tensor, eps: float, state: torch.Tensor,
                     slots: torch.Tensor, cu_tokens: torch.Tensor, out: torch.Tensor, n_entries: int,
                     status: torch.Tensor, max_new: int = 1) -> None:
    """The gated linear recurrence over the tokens of every entry, from and to the request's
    state row.  ``proj`` 32-bit [N, C] holds the sums of the q, f and v projections from
    columns ``q_off``, ``f_off`` and ``v_off`` on (heads x dk, heads x dk, heads x dv);
    q = silu(zq), f = lower + (1 - lower) sigmoid(zf + f_bias); ``state`` 32-bit
    [rows, heads, dk, dv]: S <- diag(f) S + (1 - f) v^T, o = S^T q, and ``out`` [N, heads * dv]
    gets o / sqrt(mean_over_dv(o^2) + eps) * norm_weight per head.
    ``max_new``: the most tokens an entry brings.  Entries of gated_recurrence_long_from() tokens
    or more run chunk-parallel (chunks of 64 tokens side by side from a zero state, the chunks'
    start states chained afterwards and added in, all in 32-bit) where the kernels' tiles fit
    shared memory; shorter entries of the same step are walked token by token."""
    _dense(proj, "proj"), _dense(state, "state"), _dense(out, "out")
    rows, heads, dk, dv = state.shape
    assert proj.dtype == torch.float32 and state.dtype == torch.float32
    assert lower.dtype == torch.float32 and lower.numel() == heads * dk and lower.is_contiguous()
    assert f_bias is None or (f_bias.dtype == torch.float32 and f_bias.numel() == heads * dk and f_bias.is_contiguous())
    assert norm_weight.dtype == torch.float32 and norm_weight.numel() == dv
    assert out.shape == (proj.shape[0], heads * dv) and slots.dtype == torch.int32 and cu_tokens.dtype == torch.int32
    assert max(q_off, f_off) + heads * dk <= proj.shape[1] and v_off + heads * dv <= proj.shape[1]
    n = int(proj.shape[0])
    scratch = None
    if max_new >= gated_recurrence_long_from():
        floats = int(lib().fe_gated_recurrence_scratch(n, int(n_entries), int(heads), int(dk), int(dv)))
        if floats > 0:
            scratch = _scratch.get("gated recurrence chunks", proj.device, floats, torch.float32, 1 << 22)
    check(lib().fe_gated_recurrence(ptr(proj), int(proj.shape[1]), int(q_off), int(f_off), int(v_off), ptr(f_bias),
                                    ptr(lower), ptr(norm_weight), float(eps), ptr(state), int(rows), ptr(slots),
                                    ptr(cu_tokens), ptr(out), code(out), int(n_entries), int(heads), int(dk), int(dv),
                                    n, int(max_new), ptr(scratch), ptr(status), stream()), "gated_recurrence")
    if scratch is not None:
        global LAUNCHES
        LAUNCHES += 3


def gated_recurrence_long_from() -> int:
    """Tokens from which on an entry of gated_recurrence runs chunk-parallel."""
    return int(lib().fe_gated_recurrence_long_from())


def add_normed_rmsnorm(residual: torch.Tensor, update: torch.Tensor | None, update_weight: torch.Tensor | None,
                       weight: torch.Tensor, out: torch.Tensor, eps_update: float, eps: float,
                       row_map: torch.Tensor | None = None, write_residual: bool = True,
                       conv: tuple | None = None) -> None:
    """residual (32-bit [N, C]) += update / sqrt(mean(update^2) + eps_update) * update_weight,
    then out = residual / sqrt(mean(residual^2) + eps) * weight; both weights 32-bit as they
    multiply.  Without ``update`` only the second norm runs; without ``weight`` (None) there is no
    second norm and out = residual, rounded to ``out``'s dtype.  With ``row_map`` only those rows
    are produced (``write_residual`` False leaves the stream as it was).
    ``conv`` = (taps_weight, state, slots) as ``causal_conv_state`` takes them, for a step in
    which every entry brings one token (row r is entry r): ``out`` then gets the convolution
    of the normalised rows, bit for bit what the two kernels give one after the other."""
    _dense(residual, "residual"), _dense(out, "out")
    size = residual.shape[-1]
    rows = residual.shape[0] if row_map is None else row_map.numel()
    assert residual.dtype == torch.float32 and (weight is None or (weight.dtype == torch.float32 and weight.numel() == size))
    assert out.shape == (rows, size) and (weight is not None or conv is None)
    if update is not None:
        _dense(update, "update")
        assert update.shape == residual.shape and update_weight is not None
        assert update_weight.dtype == torch.float32 and update_weight.numel() == size
    conv_w = state = slots = None
    taps = stride = 0
    if conv is not None:
        conv_w, state, slots = conv
        _dense(conv_w, "taps_weight")
        taps = int(conv_w.shape[0])
        assert row_map is None and conv_w.dtype == torch.float32 and conv_w.shape[1] == size and slots.dtype == torch.int32
        assert slots.numel() >= rows
        if taps > 1:
            assert state is not None and state.dtype == torch.float32 and state[0].is_contiguous()
            assert state[0].numel() == (taps - 1) * size
            stride = int(state.stride(0))
        else:
            state = None
    check(lib().fe_add_normed_rmsnorm(ptr(residual), ptr(update), code(update) if update is not None else F32,
                                      ptr(update_weight), ptr(weight), ptr(out), code(out), ptr(row_map), int(rows),
                                      int(size), float(eps_update), float(eps), 1 if write_residual else 0,
                                      ptr(conv_w), ptr(state), stride, ptr(slots), taps, stream()),
          "add_normed_rmsnorm")


def causal_conv_state(y: torch.Tensor, taps_weight: torch.Tensor, state: torch.Tensor | None, slots: torch.Tensor,
                      cu_tokens: torch.Tensor, token_entry: torch.Tensor, out: torch.Tensor, n_entries: int) -> None:
    """out_t = y_t + sum_j w[j] * y_(t - taps + 1 + j) per channel over every entry's tokens.
    ``y`` 32-bit [N, C]; ``taps_weight`` 32-bit [taps, C]; ``state`` 32-bit, row ``slot`` (its
    first extent) holds the request's last taps - 1 rows of y, oldest first, read at an
    entry's start and left for the next step."""
    _dense(y, "y"), _dense(out, "out"), _dense(taps_weight, "taps_weight")
    n, width = y.shape
    taps = taps_weight.shape[0]
    assert y.dtype == torch.float32 and taps_weight.dtype == torch.float32 and taps_weight.shape[1] == width
    assert out.shape == y.shape
    stride = 0
    if taps > 1:
        assert state is not None and state.dtype == torch.float32 and state[0].is_contiguous()
        assert state[0].numel() == (taps - 1) * width
        stride = int(state.stride(0))
    check(lib().fe_causal_conv_state(ptr(y), ptr(taps_weight), ptr(state), stride, ptr(slots), ptr(cu_tokens),
                                     ptr(token_entry), ptr(out), code(out), int(n), int(n_entries), int(width), int(taps),
                                     stream()), "causal_conv_state")


def gated_rmsnorm(x: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float) -> None:
    """out = x / sqrt(mean(x^2) + eps) * weight * sigmoid(gate); x is 32-bit [N, C]; ``gate``
    [N, C] may be a column slice of a wider contiguous tensor."""
    _dense(x, "x"), _dense(out, "out")
    rows, size = x.shape
    assert x.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == size
    assert gate.shape == (rows, size) and gate.stride(1) == 1 and out.shape == (rows, size)
    check(lib().fe_gated_rmsnorm(ptr(x), ptr(gate), code(gate), int(gate.stride(0)) if rows > 1 else size, ptr(weight),
                                 ptr(out), code(out), rows, size, float(eps), stream()), "gated_rmsnorm")


PREP_NORM_NONE, PREP_NORM_HEAD, PREP_NORM_WHOLE = 0, 1, 2
PREP_NORM_HEAD_AFTER = 3      # per head like PREP_NORM_HEAD, but of the rotated head: the rotation comes first


def qkv_prepare(
    *,
    q: torch.Tensor | None,
    q_heads: int = 0,
    q_dim: int = 0,
    q_norm: tuple = (PREP_NORM_NONE, 0, None),
    q_rot_off: int = 0,
    q_head_stride: int = 0,
    q_out: torch.Tensor | None = None,
    q_out_strides: tuple = (0, 0),
    q_out_offset: int = 0,
    k: torch.Tensor | None = None,
    k_heads: int = 0,
    k_dim: int = 0,
    k_norm: tuple = (PREP_NORM_NONE, 0, None),
    k_rot_off: int = 0,
    v: torch.Tensor | None = None,
    v_dim: int = 0,
    eps: float = 0.0,
    table: torch.Tensor | None = None,
    rot_dims: int = 0,
    interleaved: bool = False,
    k_cache: torch.Tensor | None = None,
    v_cache: torch.Tensor | None = None,
    block_table: torch.Tensor | None = None,
    positions: torch.Tensor,
    token_entry: torch.Tensor,
    status: torch.Tensor,
) -> None:
    """Normalise, rotate and store one step's queries, keys and values (all optional).

    ``q`` [N, >= q_heads * q_dim] and ``k``, ``v`` may be column slices of one contiguous
    projection output (row stride taken from the tensor).  ``q_norm`` / ``k_norm`` =
    (mode, leading elements of a head that are normalised, 32-bit weight): per head (before the
    rotation, or with ``PREP_NORM_HEAD_AFTER`` after it; the weight may be None) or over
    the whole projection.  ``table`` [N, rot_dims / 2, 2] holds cosine and sine of the
    tokens' angles; elements [rot_off, rot_off + rot_dims) of every head are rotated (a
    negative ``rot_off`` leaves that side as it is), neighbours paired when ``interleaved``,
    else element j with j + rot_dims / 2.  Head h of a query token starts ``q_head_stride``
    elements after head h - 1 (0: ``q_dim``).  Queries
    go to ``q_out`` at token * q_out_strides[0] + head * q_out_strides[1] + q_out_offset,
    keys and values into the pages of ``k_cache`` / ``v_cache``
    [pages, k_heads, page_size, k_dim | v_dim]."""
    n = positions.numel()
    source = q if q is not None else k
    assert source is not None and positions.dtype == torch.int32 and token_entry.dtype == torch.int32
    for t in (q, k, v):
        assert t is None or (t.is_cuda and t.stride(1) == 1 and t.shape[0] == n and t.dtype == source.dtype)
    cache_dtype = q_out if q_out is not None else k_cache
    if k is not None:
        _dense(k_cache, "k_cache"), _dense(block_table, "block_table")
        assert k_cache.shape[1] == k_heads and k_cache.shape[3] == k_dim
        assert v is None or (v_cache is not None and v_cache.shape[3] == v_dim and v_cache.dtype == k_cache.dtype)
    assert table is None or (table.dtype == torch.float32 and table.is_contiguous() and table.shape == (n, rot_dims // 2, 2))
    for mode, dims, w in (q_norm, k_norm):
        assert w is None or (w.dtype == torch.float32 and w.is_cuda and w.is_contiguous())
        assert mode != PREP_NORM_WHOLE or w is not None     # the per-head norms take no weight as a weight of ones
    stride = lambda t: 0 if t is None else int(t.stride(0)) if n > 1 else int(t.shape[1])  # noqa: E731
    pages = 0 if k_cache is None else k_cache.shape[0]
    check(
        lib().fe_qkv_prepare(
            ptr(q), stride(q), int(q_head_stride), int(q_heads), int(q_dim), int(q_norm[0]), int(q_norm[1]), ptr(q_norm[2]), int(q_rot_off),
            ptr(k), stride(k), int(k_heads), int(k_dim), int(k_norm[0]), int(k_norm[1]), ptr(k_norm[2]), int(k_rot_off),
            ptr(v), stride(v), int(v_dim), code(source), float(eps), ptr(table), int(rot_dims if table is not None else 0),
            1 if interleaved else 0, ptr(q_out), int(q_out_strides[0]), int(q_out_strides[1]), int(q_out_offset),
            ptr(k_cache), ptr(v_cache), code(cache_dtype), ptr(block_table),
            0 if block_table is None else block_table.shape[1], 0 if k_cache is None else k_cache.shape[2], pages,
            ptr(positions), ptr(token_entry), n, ptr(status), stream(),
        ),
        "qkv_prepare",
    )


_general_libs: dict = {}
GENERAL_MMA_MAX_VALUE = 512     # two warp groups of a block take 256 columns each
GENERAL_MMA_MAX_KEY = 576
GENERAL_MMA_ROWS = 64           # (token, head) rows of one block


def general_attention_lib(key_dim: int, value_dim: int, value_in_key: bool):
    """(launcher, workspace size function) of the tensor-core general attention compiled for
    one shape (built on first use)."""
    key = (key_dim, value_dim, bool(value_in_key))
    fns = _general_libs.get(key)
    if fns is None:
        path = general_attention_library_path(*key)
        try:
            handle = ctypes.CDLL(str(path))
        except OSError as error:
            raise CUDAUnavailableError(f"cannot load {path}: {error}") from error
        suffix = f"{key_dim}_{value_dim}_{1 if value_in_key else 0}"
        run = getattr(handle, f"fe_attention_gmma_{suffix}")
        p, i, f, ll = c_void_p, c_int, c_float, ctypes.c_longlong
        run.argtypes = [p, ll, ll, p, i, p, i, p, ll, ll, p, i, i, i, i, i, p, p, i, i, p, p, i, i, f, i, p,
                        i, f, f, i, i, ll, i, ll, p, ll, i, i, p, p, p]
        run.restype = c_int
        space = getattr(handle, f"fe_attention_gmma_workspace_{suffix}")
        space.argtypes = [i, i, i, i, i]
        space.restype = ll
        fns = _general_libs[key] = (run, space, handle)
    return fns[0], fns[1]


def general_mma_takes(dtype, key_dim: int, value_dim: int) -> bool:
    """Whether the tensor-core form of the general attention runs for these sizes."""
    return (dtype == torch.bfloat16 and key_dim % 16 == 0 and value_dim % 16 == 0
            and 16 <= key_dim <= GENERAL_MMA_MAX_KEY and 16 <= value_dim <= GENERAL_MMA_MAX_VALUE
            and (value_dim <= 256 or value_dim % 32 == 0)
            and _os.environ.get("FORGE_ENGINE_GENERAL_MMA", "1") != "0")


def general_splits(entries: list, groups: int, kv_heads: int, window: int | None, slots: int = 296,
                   keep_first: int = 0) -> int:
    """How many blocks share the keys of one row tile, for a step of ``entries`` ((slot,
    cached, new) each).  Only steps whose entries all fit one row tile (decoding, short
    portions) are split: enough blocks to fill the GPU once, each with at least two key
    tiles of 64, a power of two up to 32."""
    if not entries or any(count * groups > GENERAL_MMA_ROWS for _, _, count in entries):
        return 1
    longest = max(start + count for _, start, count in entries)
    if window:
        longest = min(longest, window + max(count for _, _, count in entries) + int(keep_first or 0))
    tiles = -(-longest // 64)
    wish = min(slots // max(1, len(entries) * kv_heads), tiles // 2, 32)
    return 1 if wish < 2 else 1 << (wish.bit_length() - 1)


def attention_general(
    q: torch.Tensor,
    q_strides: tuple,
    k_cache: torch.Tensor,
    k_dim: int,
    v_cache: torch.Tensor,
    v_dim: int,
    out: torch.Tensor,
    o_strides: tuple,
    block_table: torch.Tensor,
    positions: torch.Tensor,
    token_entry: torch.Tensor,
    num_q_heads: int,
    slopes: torch.Tensor | None,
    window: int | None,
    scale: float,
    status: torch.Tensor,
    entries: tuple | None = None,
    splits: int = 1,
    keep_first: int = 0,
    softcap: float | None = None,
    query_temperature: tuple | None = None,
    parts: int = 1,
    part_strides: tuple = (0, 0, 0),
    gate: torch.Tensor | None = None,
    row_hi: int = 0,
    distance_bias: torch.Tensor | None = None,
    sinks: torch.Tensor | None = None,
) -> None:
    """Paged causal attention for any key and value size: scores, softmax and sums in 32-bit.

    ``sinks`` (32-bit, per query head): exp(sink) joins the softmax's denominator once - a
    weight that belongs to no key and no value, neither scaled nor capped.

    ``entries = (cu_tokens, starts, number of entries, most new tokens of an entry)`` lets
    bfloat16 calls whose sizes are multiples of 16 run on the tensor-core kernel (``splits``
    blocks per row tile share its keys); everything else runs the plain kernel.

    Row (token, head) of ``q`` starts ``token * q_strides[0] + head * q_strides[1]`` elements
    into it, likewise for ``out``.  ``k_cache`` is [pages, kv_heads, page_size, row]; the key
    is the first ``k_dim`` elements of a row, the value the first ``v_dim`` of ``v_cache``'s
    row (``v_cache`` may be ``k_cache`` itself: one cached vector that is key and value).
    ``slopes`` (per query head, 32-bit) takes slope * (query position - key position) off
    every score; ``distance_bias`` (32-bit [heads, L]) adds entry [head, min(distance, L - 1)] to
    every (scaled, capped) score; ``window`` keeps the query's own and the window - 1 keys before it, and with
    ``keep_first`` the keys at positions below it as well.  ``softcap`` c: scores become
    c tanh(score / c); ``query_temperature`` (coef, every): a query at position p has its
    scores multiplied by 1 + coef ln(floor((p + 1) / every) + 1).  ``parts`` > 1: every head has
    that many score maps over the same values; map m reads its query ``part_strides[0]`` * m
    elements after the head's first, its key ``part_strides[1]`` * m elements into the cached
    row, and writes ``part_strides[2]`` * m elements after the head's first output.  ``gate``
    (32-bit [N, >= heads], a column slice is fine): row (token, head) is multiplied by
    sigmoid(gate[token, head]).  ``out`` may be 32-bit whatever the cache holds.  ``row_hi`` > 0
    (tensor-core kernel only): entries with more rows (new tokens x heads per kv head) are
    skipped - another kernel serves them."""
    num_pages, nkv, page_size, k_row = k_cache.shape
    v_row = v_cache.shape[3]
    n = positions.numel()
    assert q.dtype == k_cache.dtype == v_cache.dtype and out.dtype in (q.dtype, torch.float32)
    assert slopes is None or (slopes.dtype == torch.float32 and slopes.numel() == num_q_heads and slopes.is_cuda)
    assert gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape[0] == n and gate.shape[1] >= num_q_heads)
    assert distance_bias is None or (distance_bias.dtype == torch.float32 and distance_bias.is_cuda and distance_bias.is_contiguous()
                                     and distance_bias.dim() == 2 and distance_bias.shape[0] == num_q_heads)
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.is_cuda and sinks.is_contiguous() and sinks.numel() == num_q_heads)
    dist_len = 0 if distance_bias is None else int(distance_bias.shape[1])
    out_f32 = 1 if out.dtype == torch.float32 and q.dtype != torch.float32 else 0
    coef, every = query_temperature or (0.0, 0)
    gate_stride = 0 if gate is None else (int(gate.stride(0)) if n > 1 else int(gate.shape[1]))
    extras = (int(keep_first or 0), float(softcap or 0.0), float(coef), int(every), int(parts), int(part_strides[0]),
              int(part_strides[1]), int(part_strides[2]), ptr(gate), gate_stride, out_f32)
    value_in_key = v_cache.data_ptr() == k_cache.data_ptr()
    if (entries is not None and general_mma_takes(q.dtype, k_dim, v_dim)
            and (k_dim == k_row if parts == 1 else (not value_in_key and part_strides[1] * (parts - 1) + k_dim <= k_row))
            and (value_in_key or v_dim == v_row)
            and all(s % 8 == 0 for s in (*q_strides, *o_strides, *part_strides))):
        cu_tokens, starts, n_entries, max_new = entries
        run, space = general_attention_lib(k_dim, v_dim, value_in_key)
        groups = num_q_heads // nkv
        floats = int(space(int(n_entries), int(max_new), groups, nkv * int(parts), int(splits)))
        workspace = _attention_workspace(q.device, floats) if floats else None
        check(
            run(ptr(q), int(q_strides[0]), int(q_strides[1]), ptr(k_cache), k_row, ptr(v_cache), v_row, ptr(out),
                int(o_strides[0]), int(o_strides[1]), ptr(block_table), block_table.shape[1], page_size, num_pages, nkv,
                int(num_q_heads), ptr(cu_tokens), ptr(starts), int(n_entries), int(max_new), ptr(slopes),
                ptr(distance_bias), dist_len, int(window or 0), float(scale), int(splits), ptr(workspace), *extras, int(row_hi), ptr(sinks), ptr(status), stream()),
            "attention_general (tensor cores)",
        )
        if splits > 1:
            global LAUNCHES
            LAUNCHES += 1
        return
    assert row_hi == 0, "only the tensor-core kernel leaves entries to another kernel"
    check(
        lib().fe_attention_general(
            ptr(q), int(q_strides[0]), int(q_strides[1]), ptr(k_cache), k_row, int(k_dim), ptr(v_cache), v_row,
            int(v_dim), ptr(out), int(o_strides[0]), int(o_strides[1]), code(q), ptr(block_table),
            block_table.shape[1], page_size, num_pages, nkv, int(num_q_heads), ptr(positions), ptr(token_entry),
            ptr(slopes), ptr(distance_bias), dist_len, int(window or 0), float(scale), *extras, ptr(sinks), n, ptr(status), stream(),
        ),
        "attention_general",
    )


RECURRENCE_SERIAL_TOKENS = 16    # up to here an entry's tokens are walked one by one


def linear_recurrence(
    proj: torch.Tensor,
    q_off: int,
    k_off: int,
    v_off: int,
    act: int,
    state: torch.Tensor,
    slots: torch.Tensor,
    cu_tokens: torch.Tensor,
    decay: torch.Tensor,
    out: torch.Tensor,
    entries: int,
    max_new: int = 1,
) -> None:
    """S = decay_h S + k v^T, o = S^T q token by token for every entry of the step, from and
    to the 32-bit ``state`` [slots, heads, dk, dv] rows named by ``slots``.  q, k, v are
    act(columns of ``proj``) starting at ``q_off``, ``k_off`` (heads x dk each) and ``v_off``
    (heads x dv); ``act`` ACT_SILU or -1 for none.  ``out`` 32-bit [N, heads * dv].
    ``max_new``: the most tokens an entry brings; beyond RECURRENCE_SERIAL_TOKENS the step
    runs chunk-parallel (chunks of 64 tokens side by side, their states chained afterwards)
    where the chunk kernels' tiles fit shared memory."""
    _dense(proj, "proj"), _dense(state, "state"), _dense(out, "out")
    rows, heads, dk, dv = state.shape
    assert state.dtype == torch.float32 and out.dtype == torch.float32 and decay.dtype == torch.float32
    assert decay.numel() == heads and out.shape == (proj.shape[0], heads * dv)
    assert slots.dtype == torch.int32 and cu_tokens.dtype == torch.int32
    n = proj.shape[0]
    fits = 4 * max(64 * dk + dk * 68 + 64 * dv + 64 * 68 + 68, 64 * dk + dk * dv + 68) <= 200 * 1024
    if max_new > RECURRENCE_SERIAL_TOKENS and fits and dv % 4 == 0:
        chunks = int(lib().fe_linear_recurrence_chunks(int(n), int(entries)))
        sums = _scratch.get("recurrence chunk states", proj.device, chunks * heads * dk * dv, torch.float32, 1 << 22)
        check(
            lib().fe_linear_recurrence_chunked(ptr(proj), code(proj), int(proj.shape[1]), int(q_off), int(k_off),
                                               int(v_off), int(act), ptr(state), ptr(slots), ptr(cu_tokens), ptr(decay),
                                               ptr(out), ptr(sums), int(n), int(entries), heads, dk, dv, rows, stream()),
            "linear_recurrence (chunked)",
        )
        global LAUNCHES
        LAUNCHES += 2
        return
    check(
        lib().fe_linear_recurrence(ptr(proj), code(proj), int(proj.shape[1]), int(q_off), int(k_off), int(v_off),
                                   int(act), ptr(state), ptr(slots), ptr(cu_tokens), ptr(decay), ptr(out),
                                   int(entries), heads, dk, dv, rows, stream()),
        "linear_recurrence",
    )


def gemm_simt_batched(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[n, b, :] = x[n, b, :] @ w[b].T with plain 32-bit FMAs, for x [n, batch, k] and out
    [n, batch, o] that may be strided in their first two extents, and w [batch, o, k]
    contiguous."""
    _dense(w, "w")
    n, batch, k = x.shape
    o = w.shape[1]
    assert w.shape == (batch, o, k) and out.shape == (n, batch, o) and x.stride(2) == 1 and out.stride(2) == 1
    check(
        lib().fe_gemm_simt_batched(ptr(x), code(x), ptr(w), code(w), ptr(out), code(out), n, o, k, batch,
                                   int(x.stride(0)), int(out.stride(0)), int(x.stride(1)), o * k, int(out.stride(1)),
                                   stream()),
        "gemm_simt_batched",
    )


def add_rmsnorm(
    residual: torch.Tensor,
    update: torch.Tensor | None,
    weight: torch.Tensor,
    out: torch.Tensor,
    eps: float,
    row_map: torch.Tensor | None = None,
    write_residual: bool = True,
    shift: torch.Tensor | None = None,
) -> None:
    """residual += update (+ ``shift``, one 32-bit vector added to every row) (32-bit, in
    place unless ``write_residual`` is false); out = rmsnorm(residual) * weight.  With
    ``row_map`` row r of ``out`` comes from row ``row_map[r]`` of ``residual`` and ``update``."""
    _dense(residual, "residual"), _dense(weight, "weight"), _dense(out, "out")
    assert residual.dtype == torch.float32 and weight.dtype == torch.float32
    rows, size = out.shape
    assert residual.shape[1] == size and weight.numel() == size
    if update is not None:
        _dense(update, "update")
        assert update.shape == residual.shape
    if row_map is not None:
        assert row_map.dtype == torch.int32 and row_map.numel() == rows
    else:
        assert residual.shape[0] == rows
    assert shift is None or (shift.dtype == torch.float32 and shift.numel() == size and shift.is_contiguous())
    check(
        lib().fe_add_rmsnorm(
            ptr(residual), ptr(update), code(update) if update is not None else code(out),
            ptr(weight), ptr(out), code(out), ptr(row_map), ptr(shift), rows, size, float(eps),
            1 if write_residual else 0, stream(),
        ),
        "add_rmsnorm",
    )


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, block: int = 0) -> None:
    """out[n, i] = silu(gate[n, i]) * up[n, i].  ``block`` 0: a row of ``gate_up`` is all gate
    features then all up features; ``block`` B: it alternates B gate, B up features."""
    _dense(gate_up, "gate_up"), _dense(out, "out")
    rows, inter = out.shape
    assert gate_up.shape == (rows, 2 * inter) and gate_up.dtype == out.dtype
    check(lib().fe_silu_mul(ptr(gate_up), ptr(out), code(out), rows, inter, int(block), stream()), "silu_mul")


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, table: torch.Tensor) -> None:
    """table[t, j] = (cos, sin) of float(positions[t]) * inv_freq[j], in 32-bit."""
    _dense(positions, "positions"), _dense(inv_freq, "inv_freq"), _dense(table, "table")
    n, half = positions.numel(), inv_freq.numel()
    assert positions.dtype == torch.int32 and inv_freq.dtype == torch.float32
    assert table.dtype == torch.float32 and table.shape == (n, half, 2)
    check(lib().fe_rope_table(ptr(positions), ptr(inv_freq), half, n, ptr(table), stream()), "rope_table")


def qk_rope_cache(
    qkv: torch.Tensor,
    q_weight: torch.Tensor | None,
    k_weight: torch.Tensor | None,
    eps: float,
    inv_freq: torch.Tensor | None,
    rotary_dim: int,
    positions: torch.Tensor,
    token_entry: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    num_q_heads: int,
    write_kv: bool,
    status: torch.Tensor,
    table: torch.Tensor | None = None,
) -> None:
    """Normalise and rotate q (in place) and k, and store k, v into their pages.

    qkv is [N, (nq + 2 nkv) * D]; the caches are [pages, nkv, page_size, D].  ``table``:
    ``rope_table`` of these tokens (then the kernel does not take cosine and sine itself)."""
    _dense(qkv, "qkv"), _dense(k_cache, "k_cache"), _dense(v_cache, "v_cache")
    _dense(block_table, "block_table")
    num_pages, nkv, page_size, head_dim = k_cache.shape
    n = qkv.shape[0]
    assert qkv.shape[1] == (num_q_heads + 2 * nkv) * head_dim
    assert k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype
    assert block_table.dtype == torch.int32 and block_table.dim() == 2
    assert positions.dtype == torch.int32 and token_entry.dtype == torch.int32
    for w in (q_weight, k_weight, inv_freq, table):
        assert w is None or (w.dtype == torch.float32 and w.is_cuda and w.is_contiguous())
    assert table is None or (inv_freq is not None and table.shape == (n, rotary_dim // 2, 2))
    check(
        lib().fe_qk_rope_cache(
            ptr(qkv), code(qkv), ptr(q_weight), ptr(k_weight), float(eps), ptr(inv_freq), ptr(table),
            int(rotary_dim), ptr(positions), ptr(token_entry), ptr(k_cache), ptr(v_cache),
            ptr(block_table), block_table.shape[1], page_size, num_pages, num_q_heads, nkv,
            head_dim, n, 1 if write_kv else 0, ptr(status), stream(),
        ),
        "qk_rope_cache",
    )


def qk_rope_cache_sums(
    sums: torch.Tensor,
    q_out: torch.Tensor,
    q_weight: torch.Tensor | None,
    k_weight: torch.Tensor | None,
    eps: float,
    inv_freq: torch.Tensor | None,
    positions: torch.Tensor,
    token_entry: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    num_q_heads: int,
    write_kv: bool,
    status: torch.Tensor,
    table: torch.Tensor | None = None,
) -> None:
    """``qk_rope_cache`` for a projection whose k-splits were added into the 32-bit ``sums``
    [N, (nq + 2 nkv) * D]: reads the sums and leaves zeros behind, stores the finished
    queries as bfloat16 into the q columns of ``q_out`` (same shape) and k, v into their
    bfloat16 pages.  The whole head is rotated (or none of it: inv_freq and table None)."""
    _dense(sums, "sums"), _dense(q_out, "q_out"), _dense(k_cache, "k_cache"), _dense(v_cache, "v_cache")
    _dense(block_table, "block_table")
    num_pages, nkv, page_size, head_dim = k_cache.shape
    n = q_out.shape[0]
    width = (num_q_heads + 2 * nkv) * head_dim
    assert sums.dtype == torch.float32 and sums.numel() >= n * width and q_out.shape == (n, width)
    assert q_out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16
    assert block_table.dtype == torch.int32 and block_table.dim() == 2
    assert positions.dtype == torch.int32 and token_entry.dtype == torch.int32
    for w in (q_weight, k_weight, inv_freq, table):
        assert w is None or (w.dtype == torch.float32 and w.is_cuda and w.is_contiguous())
    assert table is None or table.shape == (n, head_dim // 2, 2)
    check(
        lib().fe_qk_rope_cache_sums(
            ptr(sums), ptr(q_out), ptr(q_weight), ptr(k_weight), float(eps), ptr(inv_freq), ptr(table),
            ptr(positions), ptr(token_entry), ptr(k_cache), ptr(v_cache), ptr(block_table),
            block_table.shape[1], page_size, num_pages, num_q_heads, nkv, head_dim, n,
            1 if write_kv else 0, ptr(status), stream(),
        ),
        "qk_rope_cache_sums",
    )


def projection_sums(device: torch.device, count: int) -> torch.Tensor:
    """A 32-bit buffer of at least ``count`` zeros that lives as long as the process, for
    projections that add their k-splits into it; whoever reads the sums puts zeros back."""
    return _scratch.get("projection sums", device, count, torch.float32, 1 << 20, zero=True)


def attention_simt(
    q: torch.Tensor,
    q_stride: int,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    positions: torch.Tensor,
    token_entry: torch.Tensor,
    window: int | None,
    scale: float,
    out: torch.Tensor,
    num_q_heads: int,
    status: torch.Tensor,
) -> None:
    """General paged causal attention; q row n starts at q + n * q_stride elements."""
    num_pages, nkv, page_size, head_dim = k_cache.shape
    n = out.shape[0]
    assert out.shape[1] == num_q_heads * head_dim and out.dtype == q.dtype == k_cache.dtype
    check(
        lib().fe_attention_simt(
            ptr(q), int(q_stride), code(q), ptr(k_cache), ptr(v_cache), ptr(block_table),
            block_table.shape[1], page_size, num_pages, ptr(positions), ptr(token_entry),
            int(window or 0), float(scale), ptr(out), num_q_heads, nkv, head_dim, n, ptr(status),
            stream(),
        ),
        "attention_simt",
    )


_balanced_blocks: dict = {}


def attention_balanced_blocks(head_dim: int) -> int:
    """Blocks the balanced decode kernel of this head size runs with (0: it cannot run)."""
    blocks = _balanced_blocks.get(head_dim)
    if blocks is None:
        attention_lib(head_dim)
        fn = getattr(_attention_handles[head_dim], f"fe_attn_balanced_blocks_d{head_dim}")
        fn.restype = c_int
        fn.argtypes = []
        blocks = _balanced_blocks[head_dim] = int(fn())
    return blocks


def _attention_counters(device, pairs: int) -> torch.Tensor:
    """Zeroed arrival counters, one per (entry, kv head); launches leave them zeroed."""
    return _scratch.get("attention counters", device, pairs, torch.int32, 8192, zero=True)


def _attention_workspace(device, floats: int) -> torch.Tensor:
    """Partial results of split decode attention.  One buffer per device serves every layer:
    a layer's attention has combined its parts before the next layer's begins."""
    return _scratch.get("attention workspace", device, floats, torch.float32, 1 << 22)


ATTN_DECODE_ROWS = 16  # rows (new tokens x heads per kv head) the split decode kernel takes


def attention_mma(
    q: torch.Tensor,
    q_stride: int,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    cu_tokens: torch.Tensor,
    starts: torch.Tensor,
    entries: int,
    max_new: int,
    window: int | None,
    scale: float,
    out: torch.Tensor,
    num_q_heads: int,
    status: torch.Tensor,
    run_prefill: bool,
    run_decode: bool,
    num_splits: int = 1,
    merge_in_kernel: bool = True,
) -> None:
    """Tensor-core paged attention (bfloat16).  Entries with more than 16 rows (new
    tokens x heads per kv head) go to the prefill kernel, the others to the split
    decode kernel; ``run_prefill`` / ``run_decode`` say which kinds the batch holds.
    ``num_splits`` blocks share a request's keys; 0 spreads the key tiles of all decode
    entries evenly over as many blocks as the GPU holds at once."""
    num_pages, nkv, page_size, head_dim = k_cache.shape
    assert q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    groups = num_q_heads // nkv
    mode = (1 if run_prefill else 0) | (2 if run_decode else 0)
    workspace = counters = None
    if run_decode and num_splits == 0:
        blocks = attention_balanced_blocks(head_dim)
        if blocks <= 0:
            raise UnsupportedShapeError(f"attention_mma: no balanced decode kernel for head size {head_dim}")
        workspace = _attention_workspace(q.device, 2 * blocks * ATTN_DECODE_ROWS * (head_dim + 2))
    elif run_decode and num_splits > 1:
        floats = entries * nkv * num_splits * ATTN_DECODE_ROWS * (head_dim + 2)
        workspace = _attention_workspace(q.device, floats)
        if merge_in_kernel:
            counters = _attention_counters(q.device, entries * nkv)
    check(
        attention_lib(head_dim)(
            ptr(q), int(q_stride), ptr(out), ptr(k_cache), ptr(v_cache), ptr(block_table),
            block_table.shape[1], page_size, num_pages, nkv, groups, ptr(cu_tokens), ptr(starts),
            entries, int(max_new), int(q.shape[0]), int(window or 0), float(scale), mode, int(num_splits),
            ptr(workspace), ptr(counters), ptr(status), stream(),
        ),
        "attention_mma",
    )


def gemm_simt(
    x: torch.Tensor,
    w: torch.Tensor,
    out: torch.Tensor,
    bias: torch.Tensor | None = None,
    accumulate: bool = False,
) -> None:
    """out = x @ w.T (+ bias) (+ out) with plain 32-bit FMAs; w is [out, in]."""
    _dense(x, "x"), _dense(w, "w"), _dense(out, "out")
    n, k = x.shape
    o = w.shape[0]
    assert w.shape[1] == k and out.shape == (n, o)
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == o)
    check(
        lib().fe_gemm_simt(ptr(x), code(x), ptr(w), code(w), ptr(bias), ptr(out), code(out), n, o, k,
                           1 if accumulate else 0, stream()),
        "gemm_simt",
    )


TC5_STORE_BF16, TC5_STORE_F32, TC5_ADD_F32, TC5_SILU_MUL = 0, 1, 2, 3
TC5_GELU_MUL = 5      # the gated epilogue with the tanh form of GELU
TC5_CLAMP_MUL = 6     # the gated epilogue with the clamped unit g' sigmoid(slope g') (u' + 1)
TC5_GATED = {0: 3, 1: 5, 2: 6}      # activation code (ACT_*) -> gated epilogue


def tc5_tile(n: int) -> int:
    return 16 if n <= 16 else 32 if n <= 32 else 64 if n <= 64 else 128 if n <= 128 else 256


def _tc5_workspace(device, tiles: int, ksplit: int, tile_n: int):
    """(partial tiles, arrival counters) for k-splits that do not add up inside a cluster."""
    part = _scratch.get("gemm partial tiles", device, tiles * ksplit * tile_n * 128, torch.float32, 1 << 22)
    count = _scratch.get("gemm tile counters", device, tiles, torch.int32, 16384, zero=True)
    return part, count


def gemm_tc5_set_test_fault(wait_limit: int = 0, skip_kblock: int = -1) -> None:
    """For tests of the bounded waits: later ``gemm_tc5`` launches poll at most ``wait_limit``
    times per wait and leave out the load of k-block ``skip_kblock``, so that a block gives
    up, sets status bit 8 and returns.  ``(0, -1)`` restores the usual behaviour."""
    fn = lib().fe_gemm_tc5_set_test_fault
    fn.argtypes = [ctypes.c_uint, c_int]
    fn.restype = None
    fn(int(wait_limit), int(skip_kblock))


TC5_MAX_ROWS = int(_os.environ.get("FORGE_ENGINE_TC5_MAX_ROWS", "64"))   # up to this many rows the tcgen05 kernel is used instead of the library GEMM


_ADD_TARGET = int(_os.environ.get("FORGE_ENGINE_ADD_BLOCKS", "288"))
_ADD_LIMIT = int(_os.environ.get("FORGE_ENGINE_ADD_SPLITS", "16"))


def tc5_ksplit_add(o: int, k: int) -> int:
    """Blocks per 128-feature tile of a product that adds into the residual stream.  Its
    partial sums meet in memory through atomic adds, so the k-splits need not form a cluster
    and there may be more of them: about 288 blocks, just under the 296 a B200 holds at once
    (measured at the 4B shape, batch 8, per decode step: 2.60 ms with 8 splits, 2.53 with 12,
    2.51 with 14 or 15, 2.72 with 16 - 320 blocks no longer run in one round).  So whatever the
    number of tiles, the splits never make more blocks than are resident at once (two per SM;
    FORGE_ENGINE_RESIDENT_BLOCKS overrides the count).  A block keeps at least four 64-wide
    k-blocks."""
    tiles = -(-o // 128)
    fits = max(1, _resident_blocks() // tiles)          # never more blocks than run at once
    return max(1, min(_ADD_LIMIT, round(_ADD_TARGET / tiles), fits, (k // 64) // 4))


_SUMS_TARGET = int(_os.environ.get("FORGE_ENGINE_SUMS_BLOCKS", "0"))


def tc5_ksplit_sums(o: int, k: int, n: int) -> int:
    """Blocks per 128-feature tile of the q/k/v projection that adds its k-splits into 32-bit
    sums for ``n`` tokens.  Up to 16 tokens it aims at 240 blocks instead of 288: the attention
    kernel that follows finds room on more SMs while the projection still runs and has keys in
    flight earlier (4B shape, 48 tiles, per decode step at batch 1 / 8 / 16: 2.098 / 2.445 /
    2.915 ms with 5 splits against 2.105 / 2.460 / 2.929 with 6; at batch 32 and 64 six are
    better, 3.819 / 5.775 against 3.840 / 5.796 ms).  FORGE_ENGINE_SUMS_BLOCKS names another
    number of blocks to aim at."""
    target = _SUMS_TARGET or (240 if n <= 16 else _ADD_TARGET)
    tiles = -(-o // 128)
    return max(1, min(_ADD_LIMIT, round(target / tiles), max(1, _resident_blocks() // tiles), (k // 64) // 4))


_RESIDENT_BLOCKS = 0


def _resident_blocks() -> int:
    """Blocks of the tcgen05 product for few tokens that the GPU holds at once: two per SM."""
    global _RESIDENT_BLOCKS
    if not _RESIDENT_BLOCKS:
        _RESIDENT_BLOCKS = int(_os.environ.get("FORGE_ENGINE_RESIDENT_BLOCKS", "0")) or \
            2 * torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _RESIDENT_BLOCKS


def tc5_ksplit(o: int, k: int) -> int:
    """Blocks per 128-feature tile for few tokens.  A weight with few tiles is cut along k
    so that about 190 blocks stream it (measured best on a B200: 4 for 48 tiles, 8 for 20);
    up to 8 such blocks form a cluster and add their partial tiles through shared memory.
    A block keeps at least four 64-wide k-blocks."""
    tiles = -(-o // 128)
    return max(1, min(8, round(int(_os.environ.get("FORGE_ENGINE_TC5_BLOCKS", "192")) / tiles), (k // 64) // 4))


def gemm_tc5(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int, status: torch.Tensor,
             bias: torch.Tensor | None = None, ksplit: int = 1, limit: float = 0.0, slope: float = 1.0) -> None:
    """out = x @ w.T on tcgen05 tensor cores (bfloat16 operands, TMA-fed).

    epilogue 0: out bf16 [n, o]; 1: out f32 [n, o]; 2: out f32 [n, o] += product;
    3: out bf16 [n, o/2] = silu(gate) * up for w whose rows alternate 16 gate, 16 up features
    (5: the same with the tanh form of GELU; 6: g' sigmoid(slope g') (u' + 1) with g' = min(gate,
    limit), u' = clamp(up, -limit, limit)); 7, 8 (``TC5_UNARY``): out bf16 [n, o] = the square of
    relu, or the tanh form of GELU, of the 32-bit sum + bias.
    ``ksplit`` blocks share an output tile (deterministic reduction through a workspace)."""
    _dense(x, "x"), _dense(w, "w"), _dense(out, "out")
    n, k = x.shape
    o = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] == k
    if epilogue in (TC5_SILU_MUL, TC5_GELU_MUL, TC5_CLAMP_MUL):
        assert out.shape == (n, o // 2) and out.dtype == torch.bfloat16
    else:
        assert out.shape == (n, o)
        assert out.dtype == (torch.bfloat16 if epilogue == TC5_STORE_BF16 or epilogue in TC5_UNARY.values() else torch.float32)
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == o)
    part = count = None
    ksplit = max(1, min(int(ksplit), -(-k // 64)))
    if ksplit > 1:
        tile_n = tc5_tile(n)
        tiles = -(-o // 128) * -(-n // tile_n)
        part, count = _tc5_workspace(x.device, tiles, ksplit, tile_n)
    check(lib().fe_gemm_tc5(ptr(x), ptr(w), ptr(bias), ptr(out), n, o, k, int(epilogue), ksplit, ptr(part),
                            ptr(count), ptr(status), float(limit), float(slope), stream()),
          "gemm_tc5")


def gemm_tc5_qkv_rope(
    x: torch.Tensor,
    w: torch.Tensor,
    bias: torch.Tensor | None,
    qkv: torch.Tensor,
    q_weight: torch.Tensor | None,
    k_weight: torch.Tensor | None,
    eps: float,
    table: torch.Tensor | None,
    positions: torch.Tensor,
    token_entry: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    num_q_heads: int,
    write_kv: bool,
    status: torch.Tensor,
    ksplit: int = 1,
) -> None:
    """The fused q/k/v projection of up to 64 tokens for heads of 128: x @ w.T on tcgen05,
    then per head the q/k RMS norm, the rotation and - for keys and values - the write into
    the cache pages, all in the product's epilogue.  ``qkv`` [n, (nq + 2 nkv) * 128] receives
    the finished queries (its key and value columns are not written).  ``table`` is the
    ``rope_table`` of these tokens [n, 64, 2], or None for no rotation."""
    _dense(x, "x"), _dense(w, "w"), _dense(qkv, "qkv"), _dense(k_cache, "k_cache"), _dense(v_cache, "v_cache")
    _dense(block_table, "block_table")
    n, k = x.shape
    num_pages, nkv, page_size, head_dim = k_cache.shape
    assert head_dim == 128 and n <= TC5_MAX_ROWS
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and qkv.dtype == torch.bfloat16
    assert k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16
    assert w.shape == ((num_q_heads + 2 * nkv) * 128, k) and qkv.shape == (n, w.shape[0])
    assert block_table.dtype == torch.int32 and block_table.dim() == 2
    assert positions.dtype == torch.int32 and token_entry.dtype == torch.int32
    for name, t in (("q_weight", q_weight), ("k_weight", k_weight), ("table", table), ("bias", bias)):
        assert t is None or (t.dtype == torch.float32 and t.is_cuda and t.is_contiguous()), \
            f"{name}: a contiguous 32-bit tensor on the GPU is needed, got {t.dtype} on {t.device}"
    assert table is None or table.shape == (n, 64, 2)
    check(
        lib().fe_gemm_tc5_qkv_rope(
            ptr(x), ptr(w), ptr(bias), ptr(qkv), n, k, max(1, min(8, int(ksplit))), ptr(q_weight), ptr(k_weight),
            float(eps), ptr(table), ptr(positions), ptr(token_entry), ptr(k_cache), ptr(v_cache), ptr(block_table),
            block_table.shape[1], page_size, num_pages, num_q_heads, nkv, 1 if write_kv else 0, ptr(status), stream(),
        ),
        "gemm_tc5_qkv_rope",
    )


# ---------------------------------------------------------------------------
# several dependent projections of a decode step in one persistent kernel
# ---------------------------------------------------------------------------

CHAIN_SRC_ACTIVATIONS, CHAIN_SRC_NORM = 0, 1
CHAIN_ADD, CHAIN_SILU_MUL = 0, 1
CHAIN_MAX_TOKENS = 16


class _ChainOp(ctypes.Structure):
    _fields_ = [("w", c_void_p), ("x", c_void_p), ("norm_w", c_void_p), ("out", c_void_p),
                ("m", c_int), ("k", c_int), ("src", c_int), ("epi", c_int), ("eps", c_float)]


def _chain_ops(ops: list):
    array = (_ChainOp * len(ops))()
    for slot, op in zip(array, ops):
        w = op["w"]
        slot.w, slot.x, slot.out = ptr(w), ptr(op["x"]), ptr(op["out"])
        slot.norm_w = ptr(op.get("norm_w"))
        slot.m, slot.k = int(w.shape[0]), int(w.shape[1])
        slot.src, slot.epi, slot.eps = int(op["src"]), int(op["epi"]), float(op.get("eps", 0.0))
    return array


def decode_chain_takes(shapes: list, n: int) -> bool:
    """Whether ``decode_chain`` takes projections of these ``(m, k, src, epi)`` for ``n`` tokens."""
    array = (_ChainOp * len(shapes))()
    for slot, (m, k, src, epi) in zip(array, shapes):
        slot.m, slot.k, slot.src, slot.epi = int(m), int(k), int(src), int(epi)
    fn = lib().fe_decode_chain_check
    fn.argtypes = [ctypes.POINTER(_ChainOp), c_int, c_int]
    fn.restype = c_int
    return fn(array, len(shapes), int(n)) == 0


def decode_chain(ops: list, n: int, status: torch.Tensor) -> None:
    """Up to three projections, each reading what the one before wrote, in one launch.

    Every op is a dict: ``w`` bfloat16 [m, k]; ``src`` CHAIN_SRC_ACTIVATIONS with ``x`` bfloat16
    [n, k], or CHAIN_SRC_NORM with ``x`` the 32-bit residual stream [n, k], ``norm_w`` [k] and
    ``eps`` (the operand is then rmsnorm(x) * norm_w); ``epi`` CHAIN_ADD with ``out`` 32-bit
    [n, m] that the product is added to, or CHAIN_SILU_MUL with ``out`` bfloat16 [n, m / 2] for
    a weight whose rows alternate 16 gate and 16 up features.  ``n`` <= 16 tokens."""
    for op in ops:
        w, x, out = _dense(op["w"], "w"), _dense(op["x"], "x"), _dense(op["out"], "out")
        m, k = w.shape
        assert w.dtype == torch.bfloat16 and x.shape == (n, k)
        if op["src"] == CHAIN_SRC_NORM:
            norm_w = _dense(op["norm_w"], "norm_w")
            assert x.dtype == torch.float32 and norm_w.dtype == torch.float32 and norm_w.numel() == k
        else:
            assert x.dtype == torch.bfloat16
        if op["epi"] == CHAIN_ADD:
            assert out.dtype == torch.float32 and out.shape == (n, m)
        else:
            assert out.dtype == torch.bfloat16 and out.shape == (n, m // 2)
    handle = lib()
    handle.fe_decode_chain_counters.restype = c_int
    handle.fe_decode_chain_staging.restype = c_int
    device = ops[0]["w"].device
    counters = _scratch.get("chain counters", device, handle.fe_decode_chain_counters(), torch.int32, 0, zero=True)
    staging = _scratch.get("chain staging", device, handle.fe_decode_chain_staging(), torch.float32, 0, zero=True)
    fn = handle.fe_decode_chain
    fn.argtypes = [ctypes.POINTER(_ChainOp), c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
    fn.restype = c_int
    check(fn(_chain_ops(ops), len(ops), int(n), ptr(counters), ptr(staging), ptr(status), stream()), "decode_chain")


def sample(
    logits: torch.Tensor,
    out: torch.Tensor,
    status: torch.Tensor,
    temperature: torch.Tensor | None = None,
    top_k: torch.Tensor | None = None,
    top_p: torch.Tensor | None = None,
    min_p: torch.Tensor | None = None,
    seeds: torch.Tensor | None = None,
    counters: torch.Tensor | None = None,
) -> None:
    """One token per row of 32-bit logits; all parameter tensors are per row."""
    _dense(logits, "logits")
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and out.numel() >= rows
    for t, dt in ((temperature, torch.float32), (top_k, torch.int32), (top_p, torch.float32),
                  (min_p, torch.float32), (seeds, torch.int64), (counters, torch.int64)):
        assert t is None or (t.dtype == dt and t.is_cuda and t.numel() >= rows)
    check(
        lib().fe_sample(ptr(logits), rows, vocab, ptr(temperature), ptr(top_k), ptr(top_p), ptr(min_p),
                        ptr(seeds), ptr(counters), ptr(out), ptr(status), stream()),
        "sample",
    )
