"""Python face of the compiled kernels: loads the shared library through ctypes and
launches each entry point on torch's current CUDA stream with raw device pointers.

There is no other implementation behind these functions.  If the library cannot
be built or loaded, or a tensor is not on a CUDA device, the call raises.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build as _build

_LIB: ctypes.CDLL | None = None
_LIB_PATH: str | None = None

_P, _I, _F, _L = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong

# entry point -> argument types ('p' pointer, 'i' int, 'f' float, 'l' long long); the stream is appended
_SIGNATURES = {
    "frb_embed_rows": "ppipiii",
    "frb_rmsnorm": "pppppippifiipipi",
    "frb_qkv_prepare": "pippifppipppipppiiiiiiiiii",
    "frb_wait_probe": "lpp",
    "frb_add_rows": "ppl",
    "frb_attention_generic": "pppipipppiiiifi",
    "frb_router_topk": "ppiiiifpp",
    "frb_expert_plan": "piiiippppppp",
    "frb_expert_combine": "pppiiip",
    "frb_expert_gemm_generic": "ppipppppipiiii",
    "frb_sample_rows": "piipppp",
    "frb_argmax_rows": "piippp",
    "frb_sample_floor": "piippppppp",
    "frb_gated_unit": "ppiii",
    "frb_attention_decode_mma": "ppppipppppiiiifiip",
    "frb_attention_prefill_mma": "ppppippipppppiiifi",
    "frb_attention_decode_tma": "pppipipppppiiiifiiip",
    "frb_expert_gemm_mma": "pppppppiipiiiii",
    "frb_weight_stream": "pippppppiipiiiiiiip",
    "frb_route_plan_small": "ppiiiifipppppppp",
    "frb_router_small": "ppipppiiiifipppppppp",
    "frb_router_logits": "ppiiip",
    "frb_expert_gemm_tc": "pipippppiipiiip",
    "frb_gather_rows_bf16": "pppii",
    "frb_attention_prefill_tc": "pippipippipppppiiifip",
}
_CTYPE = {"p": _P, "i": _I, "f": _F, "l": _L}


class KernelError(RuntimeError):
    pass


def library() -> ctypes.CDLL:
    """The compiled kernels; built at the first call."""
    global _LIB, _LIB_PATH
    if _LIB is None:
        path = _build.build()
        lib = ctypes.CDLL(path)
        lib.frb_last_error.restype = ctypes.c_char_p
        lib.frb_last_error.argtypes = []
        for name, spec in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = _I
            fn.argtypes = [_CTYPE[c] for c in spec] + [_P]
        _LIB, _LIB_PATH = lib, path
    return _LIB


def library_file() -> str:
    library()
    assert _LIB_PATH is not None
    return _LIB_PATH


def register(name: str, spec: str) -> None:
    """Declare one more entry point of the library (used by kernels that live in files of their own)."""
    _SIGNATURES[name] = spec
    if _LIB is not None:
        fn = getattr(_LIB, name)
        fn.restype = _I
        fn.argtypes = [_CTYPE[c] for c in spec] + [_P]


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return 0
    if dtype == torch.bfloat16:
        return 1
    raise KernelError(f"the kernels take float32 and bfloat16, not {dtype}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("a CPU tensor was given to a CUDA kernel; fieldrun_b200 has no CPU path")
    if not t.is_contiguous():
        raise KernelError("a kernel was given a tensor that is not contiguous")
    return t.data_ptr()


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle.  The direct call costs a fraction of a microsecond; building a
    ``torch.cuda.Stream`` object for every kernel of a step was a tenth of a short prompt's time on the host."""
    if _RAW_STREAM is not None:
        return _RAW_STREAM(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


_LAUNCHES = 0
_KERNELS_PER_CALL = {"frb_sample_floor": 3, "frb_argmax_rows": 2, "frb_expert_plan": 3, "frb_attention_decode_mma": 2, "frb_attention_decode_tma": 2}


def launches() -> int:
    """How many kernels of this library have been launched by this process."""
    return _LAUNCHES


def count_launches(n: int) -> None:
    """Account for kernels of this library launched by replaying a recorded step."""
    global _LAUNCHES
    _LAUNCHES += n


_TIMINGS: Optional[list] = None


def timing_start() -> None:
    """Start recording a pair of CUDA events around every launch (kernels of this library and the library
    products that go through :func:`timed`); :func:`timing_report` adds them up.  For finding out where a
    step's time goes; it slows the host side down, so never inside a measurement."""
    global _TIMINGS
    _TIMINGS = []


def timing_report() -> dict[str, tuple[int, float]]:
    """name -> (launches, milliseconds) since :func:`timing_start`; stops recording."""
    global _TIMINGS
    torch.cuda.synchronize()
    out: dict[str, tuple[int, float]] = {}
    for name, begin, end in _TIMINGS or []:
        n, ms = out.get(name, (0, 0.0))
        out[name] = (n + 1, ms + begin.elapsed_time(end))
    _TIMINGS = None
    return out


class timed:
    """``with timed("name"):`` records the enclosed launches under ``name`` while timing is on."""

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        if _TIMINGS is not None:
            self.begin = torch.cuda.Event(enable_timing=True)
            self.begin.record()
        return self

    def __exit__(self, *exc):
        if _TIMINGS is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            _TIMINGS.append((self.name, self.begin, end))
        return False


def _call(name: str, *args) -> None:
    global _LAUNCHES
    lib = library()
    if _TIMINGS is not None:
        with timed(name[4:]):
            status = getattr(lib, name)(*args, _stream())
    else:
        status = getattr(lib, name)(*args, _stream())
    _LAUNCHES += _KERNELS_PER_CALL.get(name, 1)
    if status != 0:
        raise KernelError(f"{name}: {lib.frb_last_error().decode(errors='replace')} (status {status})")


def _want(t: torch.Tensor, dtype: torch.dtype, what: str) -> None:
    if t.dtype != dtype:
        raise KernelError(f"{what} must be {dtype}, found {t.dtype}")


# ------------------------------------------------------------------------------------------------

def embed_rows(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = table[tokens[t]] as float32."""
    _want(tokens, torch.int32, "tokens")
    _want(out, torch.float32, "the residual stream")
    vocab, width = table.shape
    _call("frb_embed_rows", _ptr(tokens), _ptr(table), _code(table.dtype), _ptr(out), tokens.numel(), width, vocab)


NORM_MAX_SUMMED_ROWS = 32      # most weighted rows per token that the norm kernel sums itself (NORM_MAX_TOP_K)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, *,
            delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
            out32: Optional[torch.Tensor] = None, write_back: bool = False,
            experts: Optional[tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None) -> None:
    """out[r] = rmsnorm(x[src] + delta[src]) * weight with src = rows[r] (or r); the sum is stored back
    into x when write_back.  ``experts`` = (y [N, width], weights [T, k], row_of_assign [T * k]) adds the
    weighted sum of each token's expert outputs, in rank order, as a further update."""
    _want(x, torch.float32, "the residual stream")
    if delta is not None:
        _want(delta, torch.float32, "the residual update")
    if rows is not None:
        _want(rows, torch.int32, "row indices")
    if out32 is not None:
        _want(out32, torch.float32, "the 32-bit copy")
    num_rows = rows.numel() if rows is not None else x.shape[0]
    width = x.shape[-1]
    y = ew = rowmap = None
    top_k = 0
    if experts is not None:
        y, ew, rowmap = experts
        _want(y, torch.float32, "expert outputs")
        _want(ew, torch.float32, "expert weights")
        _want(rowmap, torch.int32, "rows of the assignments")
        top_k = ew.shape[-1]
    _call("frb_rmsnorm", _ptr(x), _ptr(delta), _ptr(y), _ptr(ew), _ptr(rowmap), top_k, _ptr(rows), _ptr(weight),
          _code(weight.dtype), float(eps), num_rows, width, _ptr(out), _code(out.dtype), _ptr(out32), int(write_back))


def add_rows(x: torch.Tensor, delta: torch.Tensor) -> None:
    _want(x, torch.float32, "the residual stream")
    _want(delta, torch.float32, "the residual update")
    _call("frb_add_rows", _ptr(x), _ptr(delta), x.numel())


def qkv_prepare(qkv: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                cos_table: Optional[torch.Tensor], sin_table: Optional[torch.Tensor], tok_pos: torch.Tensor,
                tok_slot: torch.Tensor, page_table: Optional[torch.Tensor], q_out: torch.Tensor,
                k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], *, num_heads: int,
                num_kv_heads: int, head_dim: int, rotary_dim: int, interleaved: bool, write_cache: bool,
                per_head: bool = False, tables_final: bool = False) -> None:
    """Q/K RMSNorm (when weights are given: over the whole row with weights [heads * head_dim], or with
    ``per_head`` over each head with weights [head_dim]), rotary from the tables, Q out, K/V into their pages.
    ``tables_final``: positions, slots and the page table were complete before the kernel before this one in
    the stream began (a step's tables, with the projection between them and this call); the kernel then reads
    them, and the angles, while that kernel still runs."""
    if (q_weight is None) != (k_weight is None):
        raise KernelError("q and k norm weights come together or not at all")
    wdtype = q_weight.dtype if q_weight is not None else torch.float32
    if k_weight is not None and k_weight.dtype != wdtype:
        raise KernelError("q and k norm weights must have one dtype")
    if write_cache and (k_pages is None or v_pages is None or page_table is None):
        raise KernelError("a cache write needs pages and a page table")
    table_positions = cos_table.shape[0] if cos_table is not None else 0
    max_pages = page_table.shape[1] if page_table is not None else 0
    out_dtype = q_out.dtype
    if k_pages is not None and k_pages.dtype != out_dtype:
        raise KernelError("queries and cache must have one dtype")
    _call("frb_qkv_prepare", _ptr(qkv), _code(qkv.dtype), _ptr(q_weight), _ptr(k_weight), _code(wdtype), float(eps),
          _ptr(cos_table), _ptr(sin_table), table_positions, _ptr(tok_pos), _ptr(tok_slot), _ptr(page_table), max_pages,
          _ptr(q_out), _ptr(k_pages), _ptr(v_pages), _code(out_dtype), qkv.shape[0], num_heads, num_kv_heads, head_dim,
          rotary_dim, int(interleaved), int(write_cache), int(per_head), int(tables_final))


def attention_generic(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, page_table: torch.Tensor,
                      tok_pos: torch.Tensor, tok_slot: torch.Tensor, out: torch.Tensor, *, num_heads: int,
                      num_kv_heads: int, head_dim: int, scale: float, window: Optional[int]) -> None:
    if k_pages.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelError("queries, cache and output must have one dtype")
    _call("frb_attention_generic", _ptr(q), _ptr(k_pages), _ptr(v_pages), _code(q.dtype), _ptr(page_table),
          page_table.shape[1], _ptr(tok_pos), _ptr(tok_slot), _ptr(out), q.shape[0], num_heads, num_kv_heads, head_dim,
          float(scale), int(window or 0))


def router_topk(logits: torch.Tensor, bias: Optional[torch.Tensor], top_k: int, renormalize: bool, routed_scale: float,
                ids: torch.Tensor, weights: torch.Tensor) -> None:
    _want(logits, torch.float32, "router logits")
    if bias is not None:
        _want(bias, torch.float32, "the routing bias")
    _want(ids, torch.int32, "expert ids")
    _want(weights, torch.float32, "expert weights")
    tokens, experts = logits.shape
    _call("frb_router_topk", _ptr(logits), _ptr(bias), tokens, experts, top_k, int(renormalize), float(routed_scale),
          _ptr(ids), _ptr(weights))


def expert_plan(ids: torch.Tensor, num_experts: int, tile_rows: int, counts: torch.Tensor, offsets: torch.Tensor,
                sorted_token: torch.Tensor, row_of_assign: torch.Tensor, tile_expert: torch.Tensor,
                tile_row0: torch.Tensor, num_tiles: torch.Tensor) -> None:
    tokens, top_k = ids.shape
    for t in (ids, counts, offsets, sorted_token, row_of_assign, tile_expert, tile_row0, num_tiles):
        _want(t, torch.int32, "expert plan buffers")
    _call("frb_expert_plan", _ptr(ids), tokens, top_k, num_experts, tile_rows, _ptr(counts), _ptr(offsets),
          _ptr(sorted_token), _ptr(row_of_assign), _ptr(tile_expert), _ptr(tile_row0), _ptr(num_tiles))


def expert_combine(y: torch.Tensor, weights: torch.Tensor, row_of_assign: torch.Tensor, out: torch.Tensor) -> None:
    _want(y, torch.float32, "expert outputs")
    _want(out, torch.float32, "the residual update")
    tokens, top_k = weights.shape
    _call("frb_expert_combine", _ptr(y), _ptr(weights), _ptr(row_of_assign), tokens, top_k, y.shape[-1], _ptr(out))


def expert_gemm_generic(w: torch.Tensor, x: torch.Tensor, x_rows: Optional[torch.Tensor], tile_expert: torch.Tensor,
                        tile_row0: torch.Tensor, num_tiles: torch.Tensor, offsets: torch.Tensor, max_tiles: int,
                        out: torch.Tensor, *, paired: bool) -> None:
    """out[row] = silu(x W1^T) * (x W3^T) (paired; w is [E, 2F, K]) or x W^T (w is [E, F, K]) per sorted row."""
    if w.dtype != x.dtype:
        raise KernelError("expert weights and their input must have one dtype")
    feats = w.shape[1] // 2 if paired else w.shape[1]
    _call("frb_expert_gemm_generic", _ptr(w), _ptr(x), _code(w.dtype), _ptr(x_rows), _ptr(tile_expert), _ptr(tile_row0),
          _ptr(num_tiles), _ptr(offsets), max_tiles, _ptr(out), _code(out.dtype), feats, w.shape[2], int(paired))


def sample_rows(logits: torch.Tensor, temperature: Optional[torch.Tensor], uniform: Optional[torch.Tensor],
                out: torch.Tensor, floor: Optional[torch.Tensor] = None) -> None:
    """out[r] = the largest logit of row r (the last index on ties), or where temperature[r] > 0 a sample of
    softmax(logits[r] / temperature[r]) by inverse CDF with uniform[r]; ``floor[r]`` (from :func:`sample_floor`)
    is the smallest logit that may be sampled."""
    _want(logits, torch.float32, "logits")
    _want(out, torch.int32, "picked tokens")
    rows, vocab = logits.shape
    if temperature is None and vocab >= ARGMAX_SLICED_VOCAB:
        # every row greedy and long: many blocks a row, then a warp among their results
        key = str(logits.device)
        scratch = _ARGMAX_SCRATCH.get(key)
        if scratch is None or scratch[0].numel() < rows * 32:
            count = max(rows, 64) * 32
            scratch = (torch.empty(count, dtype=torch.float32, device=logits.device),
                       torch.empty(count, dtype=torch.int32, device=logits.device))
            _ARGMAX_SCRATCH[key] = scratch
        _call("frb_argmax_rows", _ptr(logits), rows, vocab, _ptr(scratch[0]), _ptr(scratch[1]), _ptr(out))
        return
    _call("frb_sample_rows", _ptr(logits), rows, vocab, _ptr(temperature), _ptr(uniform), _ptr(floor), _ptr(out))


ARGMAX_SLICED_VOCAB = 16384     # from this many logits a row on, a greedy pick takes 32 blocks a row
_ARGMAX_SCRATCH: dict[str, tuple[torch.Tensor, torch.Tensor]] = {}


_FLOOR_SCRATCH: dict[str, tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = {}


def sample_floor(logits: torch.Tensor, temperature: torch.Tensor, top_k: Optional[torch.Tensor], top_p: Optional[torch.Tensor],
                 floor: torch.Tensor) -> None:
    """floor[r] = the smallest logit of row r that stays when only the ``top_k[r]`` largest logits (0: all) and the
    smallest set of them holding ``top_p[r]`` of the probability (1: all) may be sampled; equal logits stay or go
    together.  -inf for greedy rows and rows that cut nothing."""
    _want(logits, torch.float32, "logits")
    _want(floor, torch.float32, "the sampling floor")
    if top_k is not None:
        _want(top_k, torch.int32, "top_k")
    if top_p is not None:
        _want(top_p, torch.float32, "top_p")
    rows, vocab = logits.shape
    scratch = _FLOOR_SCRATCH.get(str(logits.device))
    if scratch is None or scratch[0].numel() < rows:
        # zero before a call, left zero by it: the rows' largest logits (as ordered keys) and first histograms
        held = max(rows, 64)
        scratch = (torch.zeros(held, dtype=torch.int32, device=logits.device),
                   torch.zeros(held * 256, dtype=torch.int32, device=logits.device),
                   torch.zeros(held * 256, dtype=torch.int64, device=logits.device))
        _FLOOR_SCRATCH[str(logits.device)] = scratch
    _call("frb_sample_floor", _ptr(logits), rows, vocab, _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(floor),
          _ptr(scratch[0]), _ptr(scratch[1]), _ptr(scratch[2]))


def gated_unit(both: torch.Tensor, out: torch.Tensor) -> None:
    """out = silu(both[:, :w]) * both[:, w:]."""
    _want(both, torch.float32, "gate and up rows")
    rows, width = out.shape
    _call("frb_gated_unit", _ptr(both), _ptr(out), _code(out.dtype), rows, width)


MMA_HEAD_DIMS = (32, 64, 96, 128)
ATTENTION_CHUNK = 256


def attention_decode_mma(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, page_table: torch.Tensor,
                         seq_pos: torch.Tensor, seq_slot: torch.Tensor, part_o: torch.Tensor, part_ml: torch.Tensor,
                         out: torch.Tensor, *, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                         window: Optional[int], max_chunks: int) -> None:
    """One token per sequence, bfloat16: keys split into chunks of 256 over blocks, merged in chunk order."""
    for t in (q, k_pages, v_pages, out):
        _want(t, torch.bfloat16, "tensor-core attention operands")
    _want(part_o, torch.float32, "partial outputs")
    _call("frb_attention_decode_mma", _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(page_table), page_table.shape[1],
          _ptr(seq_pos), _ptr(seq_slot), _ptr(part_o), _ptr(part_ml), _ptr(out), q.shape[0], num_heads, num_kv_heads,
          head_dim, float(scale), int(window or 0), max_chunks, _ptr(tc_status(q.device)))


_SM_COUNT: dict[int, int] = {}


def sm_count(device=None) -> int:
    """Multiprocessors of the device (asked once per device)."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    if index is None:
        index = torch.cuda.current_device()
    if index not in _SM_COUNT:
        _SM_COUNT[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _SM_COUNT[index]


def decode_chunks_per_block(num_seqs: int, num_kv_heads: int, max_chunks: int, sms: int = 148) -> int:
    """How many chunks of 256 keys one block of :func:`attention_decode_tma` takes.  A block's set-up and its
    combine cost about as much as three pages, so runs of several chunks win as soon as the SMs have a block
    each (measured on a B200: 32 sequences of 4,096 keys 4.7 TB/s with one chunk per block, 5.85 with eight;
    8 sequences of 32,768 keys 4.1 and 6.2).  Not more than eight: the grid is laid out for the longest
    sequence of the step, and with longer runs a step of unequal sequences is left with a few long blocks.
    The run is then shortened as far as the number of blocks per sequence stays the same (9 chunks: 5 + 4,
    not 8 + 1)."""
    most = max(1, min(8, max_chunks, (num_seqs * num_kv_heads * max_chunks) // sms))
    blocks = -(-max_chunks // most)
    return -(-max_chunks // blocks)


def attention_decode_tma(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, page_table: torch.Tensor,
                         seq_pos: torch.Tensor, seq_slot: torch.Tensor, part_o: torch.Tensor, part_ml: torch.Tensor,
                         out: torch.Tensor, *, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                         window: Optional[int], max_chunks: int, chunks_per_block: Optional[int] = None) -> None:
    """As :func:`attention_decode_mma` for head sizes 64 and 128, with the pages copied into shared memory by
    TMA through a ring of stages, which keeps far more bytes in flight; a block takes ``chunks_per_block``
    chunks (default: :func:`decode_chunks_per_block`)."""
    for t in (q, k_pages, v_pages, out):
        _want(t, torch.bfloat16, "tensor-core attention operands")
    _want(part_o, torch.float32, "partial outputs")
    if chunks_per_block is None:
        chunks_per_block = decode_chunks_per_block(q.shape[0], num_kv_heads, max_chunks, sm_count(q.device))
    _call("frb_attention_decode_tma", _ptr(q), _ptr(k_pages), _ptr(v_pages), k_pages.shape[0], _ptr(page_table),
          page_table.shape[1], _ptr(seq_pos), _ptr(seq_slot), _ptr(part_o), _ptr(part_ml), _ptr(out), q.shape[0], num_heads,
          num_kv_heads, head_dim, float(scale), int(window or 0), max_chunks, int(chunks_per_block),
          _ptr(tc_status(q.device)))


def attention_prefill_mma(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, page_table: torch.Tensor,
                          tile_seq: torch.Tensor, tile_q0: torch.Tensor, seq_slot: torch.Tensor, seq_start: torch.Tensor,
                          seq_q_len: torch.Tensor, cu_q_len: torch.Tensor, out: torch.Tensor, *, num_heads: int,
                          num_kv_heads: int, head_dim: int, scale: float, window: Optional[int]) -> None:
    """Many tokens per sequence, bfloat16: tiles of 16 queries, causal, blockwise over the cache pages."""
    for t in (q, k_pages, v_pages, out):
        _want(t, torch.bfloat16, "tensor-core attention operands")
    _call("frb_attention_prefill_mma", _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(page_table), page_table.shape[1],
          _ptr(tile_seq), _ptr(tile_q0), tile_seq.numel(), _ptr(seq_slot), _ptr(seq_start), _ptr(seq_q_len),
          _ptr(cu_q_len), _ptr(out), num_heads, num_kv_heads, head_dim, float(scale), int(window or 0))


def expert_gemm_mma(w: torch.Tensor, x: torch.Tensor, x_rows: Optional[torch.Tensor], tile_expert: torch.Tensor,
                    tile_row0: torch.Tensor, num_tiles: torch.Tensor, offsets: torch.Tensor, max_tiles: int,
                    tile_rows: int, out: torch.Tensor, *, paired: bool, splits: int = 1, groups: int = 4) -> None:
    """The expert products as a stream over bfloat16 weights (tiles of 8, 16 or 32 rows; per block ``groups``
    groups of 16 features and ``splits`` parts of the inner size; see :func:`stream_shape`)."""
    _want(w, torch.bfloat16, "streamed expert weights")
    _want(x, torch.bfloat16, "streamed expert inputs")
    _want(out, torch.bfloat16 if paired else torch.float32, "streamed expert outputs")
    feats = w.shape[1] // 2 if paired else w.shape[1]
    _call("frb_expert_gemm_mma", _ptr(w), _ptr(x), _ptr(x_rows), _ptr(tile_expert), _ptr(tile_row0), _ptr(num_tiles),
          _ptr(offsets), max_tiles, tile_rows, _ptr(out), feats, w.shape[2], int(paired), int(splits), int(groups))


import os as _os
STREAM_RING_KB = int(_os.environ.get("FIELDRUN_B200_STREAM_RING_KB", "144"))   # shared memory of weight_stream's ring of stages
STREAM_PIECES = int(_os.environ.get("FIELDRUN_B200_STREAM_PIECES", "24"))     # most pieces of 64 k in a stage


def weight_stream_takes(features: int, inner: int, paired: bool) -> bool:
    """Whether :func:`weight_stream` takes these sizes."""
    return inner % 64 == 0 and inner > 0 and features > 0 and features % (8 if paired else 16) == 0


def weight_stream(w: torch.Tensor, x: torch.Tensor, x_rows: Optional[torch.Tensor], tile_expert: torch.Tensor,
                  tile_row0: torch.Tensor, num_tiles: torch.Tensor, offsets: torch.Tensor, max_tiles: int,
                  tile_rows: int, out: torch.Tensor, *, paired: bool, lists_final: bool = False,
                  blocks: Optional[int] = None, ring_kb: Optional[int] = None, pieces: int = 0) -> None:
    """Products of a few rows with bfloat16 weights [E, F or 2F, K] as one stream over the weights per SM: TMA into
    a ring of stages, ``mma.sync`` from shared memory (tiles of 8, 16 or 32 rows).  ``lists_final``: the lists of
    tiles were complete before the kernel before this one in the stream began (a dense layer's fixed lists; the
    experts' second product), so the weights may be asked for before that kernel has ended."""
    _want(w, torch.bfloat16, "streamed weights")
    _want(x, torch.bfloat16, "streamed inputs")
    _want(out, torch.bfloat16 if paired else torch.float32, "streamed outputs")
    feats = w.shape[1] // 2 if paired else w.shape[1]
    _call("frb_weight_stream", _ptr(w), w.shape[0], _ptr(x), _ptr(x_rows), _ptr(tile_expert), _ptr(tile_row0),
          _ptr(num_tiles), _ptr(offsets), max_tiles, tile_rows, _ptr(out), feats, w.shape[2], int(paired),
          int(lists_final), int(blocks or sm_count(w.device)), int(ring_kb or STREAM_RING_KB), int(pieces or STREAM_PIECES),
          _ptr(tc_status(w.device)))


SMALL_ROUTE_ASSIGNMENTS = 1024
SMALL_ROUTE_TOKENS = 16       # one token per warp of the one-block kernel: beyond that the separate kernels are faster
ROUTER_SMALL_TOKENS = 8       # most tokens of a step for router_small


ROUTER_LOGITS_TOKENS = 256     # up to this many tokens the router's float32 product is this library's kernel


def router_logits(act32: torch.Tensor, router: torch.Tensor, logits: torch.Tensor) -> None:
    """logits [T, E] = act32 [T, width] x router [E, width]^T in float32, for steps of a few hundred tokens at most
    (each block re-reads its eight tokens' rows: beyond that the library's product is the better one)."""
    _want(act32, torch.float32, "router input")
    _want(router, torch.float32, "router weight")
    _want(logits, torch.float32, "router logits")
    _call("frb_router_logits", _ptr(act32), _ptr(router), act32.shape[1], act32.shape[0], router.shape[0], _ptr(logits))


def route_plan_small(logits: torch.Tensor, bias: Optional[torch.Tensor], top_k: int, renormalize: bool, routed_scale: float,
                     tile_rows: int, ids: torch.Tensor, weights: torch.Tensor, offsets: torch.Tensor,
                     sorted_token: torch.Tensor, row_of_assign: torch.Tensor, tile_expert: torch.Tensor,
                     tile_row0: torch.Tensor, num_tiles: torch.Tensor) -> None:
    """Expert choice and expert-sorted lists in one launch by one block, for steps of at most 1024 (token, expert)
    pairs; the parts use it up to ``SMALL_ROUTE_TOKENS`` tokens, beyond which the separate kernels are faster."""
    _want(logits, torch.float32, "router logits")
    tokens, experts = logits.shape
    _call("frb_route_plan_small", _ptr(logits), _ptr(bias), tokens, experts, top_k, int(renormalize), float(routed_scale),
          tile_rows, _ptr(ids), _ptr(weights), _ptr(offsets), _ptr(sorted_token), _ptr(row_of_assign), _ptr(tile_expert),
          _ptr(tile_row0), _ptr(num_tiles))


def stream_shape(tiles: int, features: int, inner: int, tile_rows: int, paired: bool = False) -> dict:
    """How a block of the streaming kernel is cut.  Measured on a B200 at MiniMax-M2's sizes: one group of 16
    features per block with the inner size cut into parts among the block's warps is never slower than
    several groups over the whole inner size, and it is faster where few tiles leave the device short of
    bytes in flight: about 4096 warps for a plain product (a warp keeps 4 KB in flight), about 1536 for a
    paired one (8 KB), and at least two parts.  Returns the keyword arguments ``splits`` and ``groups``."""
    nb = tile_rows // 8
    total = max(1, tiles * ((features + 15) // 16))
    most = max(1, 16 // nb)
    want = -(-(1536 if paired else 4096) // total)
    splits = max(1, min(most, max(2, want), max(1, inner // 128)))
    return {"splits": splits, "groups": 1}


_TC_STATUS: dict[str, torch.Tensor] = {}
# what each code of the status word means: which wait of which kernel gave up
_WAIT_CODES = {
    1: "expert products: the producer waiting for a free stage",
    2: "expert products: the MMA thread waiting for a loaded stage",
    3: "expert products: the epilogue waiting for the accumulators",
    6: "expert products: the MMA thread waiting for the epilogue to have read the accumulators",
    4: "one-token attention: waiting for a page's copy",
    5: "one-token attention: a sequence has more keys than the launch was sized for (max_chunks); keys were left out",
    21: "weight stream: the producer waiting for a free stage",
    22: "weight stream: a compute warp waiting for a loaded stage",
    11: "prompt attention: the producer waiting for a free key/value stage",
    12: "prompt attention: the query tile's copy",
    13: "prompt attention: the MMA thread waiting for a loaded key/value stage",
    15: "prompt attention: the MMA thread waiting for the probabilities",
    16: "prompt attention: the softmax waiting for the scores",
    18: "prompt attention: the correction waiting for the step before",
    19: "prompt attention: the epilogue waiting for the last steps",
    99: "the wait probe, whose wait is meant to run out",
}


def tc_status(device) -> torch.Tensor:
    """One int on the device that the tensor-core expert kernel sets when one of its waits gives up."""
    key = str(device)
    if key not in _TC_STATUS:
        _TC_STATUS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _TC_STATUS[key]


def tc_status_check(device) -> None:
    """Raise if a kernel reported a wait that gave up since the last check (this reads one int from the
    device, so it waits for the work before it)."""
    key = str(device)
    if key in _TC_STATUS:
        tc_status_raise(device, int(_TC_STATUS[key].item()))


def tc_status_raise(device, code: int) -> None:
    """Raise for a status word that was read from the device (0: nothing happened) and clear the word."""
    if code != 0:
        _TC_STATUS[str(device)].zero_()
        where = _WAIT_CODES.get(code, f"code {code}")
        raise KernelError(f"a kernel gave up instead of finishing ({where}); the step's results are not valid")


def gather_rows(x: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    """out[i] = x[rows[i]] for bfloat16 rows."""
    _want(x, torch.bfloat16, "gathered rows")
    _want(rows, torch.int32, "row indices")
    _call("frb_gather_rows_bf16", _ptr(x), _ptr(rows), _ptr(out), rows.numel(), x.shape[-1])


def expert_gemm_tc(w: torch.Tensor, x: torch.Tensor, tile_expert: torch.Tensor, tile_row0: torch.Tensor,
                   num_tiles: torch.Tensor, offsets: torch.Tensor, max_tiles: int, tile_rows: int, out: torch.Tensor, *,
                   paired: bool) -> None:
    """The expert products on tcgen05 tensor cores; x holds the rows in expert-sorted order (tiles of 32, 64,
    128 or 256 rows; features in steps of 128, inner size in steps of 64)."""
    _want(w, torch.bfloat16, "expert weights")
    _want(x, torch.bfloat16, "expert inputs")
    _want(out, torch.bfloat16 if paired else torch.float32, "expert outputs")
    feats = w.shape[1] // 2 if paired else w.shape[1]
    _call("frb_expert_gemm_tc", _ptr(w), w.shape[0], _ptr(x), x.shape[0], _ptr(tile_expert), _ptr(tile_row0), _ptr(num_tiles),
          _ptr(offsets), max_tiles, tile_rows, _ptr(out), feats, w.shape[2], int(paired), _ptr(tc_status(w.device)))


_ROUTER_TICKETS: dict[str, torch.Tensor] = {}


def router_small(act32: torch.Tensor, router: torch.Tensor, logits: torch.Tensor, bias: Optional[torch.Tensor], top_k: int,
                 renormalize: bool, routed_scale: float, tile_rows: int, ids: torch.Tensor, weights: torch.Tensor,
                 offsets: torch.Tensor, sorted_token: torch.Tensor, row_of_assign: torch.Tensor, tile_expert: torch.Tensor,
                 tile_row0: torch.Tensor, num_tiles: torch.Tensor) -> None:
    """Router logits (float32 rows x float32 weight), expert choice and expert-sorted lists in one launch, for
    steps of at most ``ROUTER_SMALL_TOKENS`` tokens (a decode step of a small batch)."""
    _want(act32, torch.float32, "router input")
    _want(router, torch.float32, "router weight")
    _want(logits, torch.float32, "router logits")
    tokens, width = act32.shape
    key = str(act32.device)
    if key not in _ROUTER_TICKETS:
        _ROUTER_TICKETS[key] = torch.zeros(1, dtype=torch.int32, device=act32.device)
    _call("frb_router_small", _ptr(act32), _ptr(router), width, _ptr(logits), _ptr(_ROUTER_TICKETS[key]), _ptr(bias), tokens,
          router.shape[0], top_k, int(renormalize), float(routed_scale), tile_rows, _ptr(ids), _ptr(weights), _ptr(offsets),
          _ptr(sorted_token), _ptr(row_of_assign), _ptr(tile_expert), _ptr(tile_row0), _ptr(num_tiles))


TC_ATTENTION_HEAD_DIMS = (64, 128)
TC_ATTENTION_QUERIES = 128


def attention_prefill_tc(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, page_table: torch.Tensor,
                         tile_seq: torch.Tensor, tile_q0: torch.Tensor, seq_slot: torch.Tensor, seq_start: torch.Tensor,
                         seq_q_len: torch.Tensor, cu_q_len: torch.Tensor, out: torch.Tensor, *, num_heads: int,
                         num_kv_heads: int, head_dim: int, scale: float, window: Optional[int]) -> None:
    """Many tokens per sequence on tcgen05 tensor cores: tiles of 128 queries of one head (bfloat16, head sizes
    64 and 128)."""
    for t in (q, k_pages, v_pages, out):
        _want(t, torch.bfloat16, "tensor-core attention operands")
    _call("frb_attention_prefill_tc", _ptr(q), q.shape[0], _ptr(k_pages), _ptr(v_pages), k_pages.shape[0], _ptr(page_table),
          page_table.shape[1], _ptr(tile_seq), _ptr(tile_q0), tile_seq.numel(), _ptr(seq_slot), _ptr(seq_start),
          _ptr(seq_q_len), _ptr(cu_q_len), _ptr(out), num_heads, num_kv_heads, head_dim, float(scale), int(window or 0),
          _ptr(tc_status(q.device)))


def wait_probe(device, limit_cycles: int = 100_000) -> int:
    """Launch the one block whose wait is meant to run out after ``limit_cycles`` clock cycles: it leaves code
    99 in the device's status word (see :func:`tc_status_check`).  Returns the cycles it waited.  For testing
    the way from a device-side give-up to the host-side error; nothing faults and nothing is left pending."""
    waited = torch.zeros(1, dtype=torch.int64, device=device)
    with torch.cuda.device(device):
        _call("frb_wait_probe", int(limit_cycles), _ptr(tc_status(device)), _ptr(waited))
    return int(waited.item())
