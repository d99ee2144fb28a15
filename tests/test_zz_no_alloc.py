"""The attention entry point that brings its own scratch memory (csrc/noalloc.h), called through its exported
C symbol as a program without torch's allocator would call it, against the ordinary entry point.

Callers that may not allocate on the device (a loop that owns a fixed share of the memory, a latency-critical
loop that cannot afford cudaMalloc's device-wide synchronisation, code inside a stream capture) use it; the
test makes two calls in a row because every call shares one built-in array that keeps the last call's
contents.  The file sorts last so that a run that stops at the first failure has run everything else."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _symbol():
    from fieldrun_b200.csrc import ops
    lib = ctypes.CDLL(ops.library_file())
    fn = lib.frb_attention_decode_noalloc
    fn.restype = ctypes.c_int
    p, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [p, p, p, p, i, p, p, p, i, i, i, i, f, i, i, p]
    lib.frb_last_error.restype = ctypes.c_char_p
    return lib, fn


def _case(rng, lengths, heads, kv_heads, head_dim):
    pages = sum((n + 63) // 64 for n in lengths) + 3
    order = list(rng.permutation(pages))
    keys = (torch.randn(pages, kv_heads, 64, head_dim, device=DEV) * 0.5).to(torch.bfloat16)
    values = (torch.randn(pages, kv_heads, head_dim, 64, device=DEV) * 0.5).to(torch.bfloat16)
    table = np.full((len(lengths), pages), -1, dtype=np.int32)
    for slot, n in enumerate(lengths):
        for i in range((n + 63) // 64):
            table[slot, i] = order.pop()
    q = torch.randn(len(lengths), heads * head_dim, device=DEV).to(torch.bfloat16)
    positions = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)
    slots = torch.arange(len(lengths), dtype=torch.int32, device=DEV)
    return q, keys, values, torch.from_numpy(table).to(DEV), positions, slots


def test_no_alloc_attention_equals_the_ordinary_entry_point_twice_in_a_row():
    from fieldrun_b200.csrc import ops
    lib, fn = _symbol()
    rng = np.random.default_rng(0)
    torch.manual_seed(0)
    stream = torch.cuda.current_stream().cuda_stream
    # two different problems back to back: the second must not be disturbed by what the first left behind
    for lengths, heads, kv_heads, head_dim, window in (([700, 64, 257, 1], 12, 2, 128, 0), ([300, 900], 8, 8, 64, 200)):
        q, keys, values, table, positions, slots = _case(rng, lengths, heads, kv_heads, head_dim)
        chunks = (max(lengths) + 255) // 256
        scale = head_dim ** -0.5
        want = torch.empty_like(q)
        part_o = torch.empty(len(lengths), heads, chunks, head_dim, dtype=torch.float32, device=DEV)
        part_ml = torch.empty(len(lengths), heads, chunks, 2, dtype=torch.float32, device=DEV)
        ops.attention_decode_mma(q, keys, values, table, positions, slots, part_o, part_ml, want, num_heads=heads,
                                 num_kv_heads=kv_heads, head_dim=head_dim, scale=scale, window=window or None, max_chunks=chunks)
        got = torch.full_like(q, 3.0)
        before = torch.cuda.memory_allocated()
        status = fn(q.data_ptr(), keys.data_ptr(), values.data_ptr(), table.data_ptr(), table.shape[1], positions.data_ptr(),
                    slots.data_ptr(), got.data_ptr(), len(lengths), heads, kv_heads, head_dim, scale, window, chunks, stream)
        assert status == 0, lib.frb_last_error().decode()
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        err = (got.float() - want.float()).abs().max().item() / max(want.float().abs().max().item(), 1e-30)
        assert err <= 1e-2, f"relative error {err:.3e}"            # the tolerance of the other bfloat16 kernel tests
        assert torch.equal(got, want)                               # and in fact the same kernels: the same bits


def test_no_alloc_attention_refuses_what_its_scratch_cannot_hold():
    lib, fn = _symbol()
    q = torch.zeros(64, 48 * 128, dtype=torch.bfloat16, device=DEV)
    kv = torch.zeros(1, 8, 64, 128, dtype=torch.bfloat16, device=DEV)
    table = torch.zeros(64, 64, dtype=torch.int32, device=DEV)
    ints = torch.zeros(64, dtype=torch.int32, device=DEV)
    status = fn(q.data_ptr(), kv.data_ptr(), kv.data_ptr(), table.data_ptr(), 64, ints.data_ptr(), ints.data_ptr(), q.data_ptr(),
                64, 48, 8, 128, 0.1, 0, 16, torch.cuda.current_stream().cuda_stream)
    assert status != 0
    message = lib.frb_last_error().decode()
    assert "the built-in scratch holds" in message and "6389760" in message
