"""The allocation-free attention entry point (b200_attention_decode_static) against the regular one.

Some users of the library cannot allocate device memory on the token path: their memory was budgeted at start-up,
belongs to a pool they do not control, or they cannot accept the device-wide synchronisation that comes with
cudaMalloc / cudaFree.  For them the split partials of the decode attention live in a fixed array inside the library
image.  The test calls both entry points through the C ABI on the same inputs, twice in a row (the built-in array is
shared between calls and keeps the previous call's contents), and expects the same answer; the answer is also held against
the CPU oracle's grouped-query attention (the reference's softmax(q K^T / sqrt(hd)) V restated in C), so the test stands on
its own.  It also checks that a shape beyond the array's size is refused with a message instead of overrunning it.

This file is named to be collected last, so that a run that stops at the first failure has already run every other
test; it must pass alone in a fresh process as well.
"""
import ctypes as C

import numpy as np
import pytest

import ctorch_b200 as B
import oracle
from ctorch_b200 import workloads as W

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

STATIC_BYTES = 8 << 20


def _cache(dtype, sequences, kv_heads, head_dim, capacity):
    handle = C.c_void_p()
    B.kcheck(B.lib().b200_kv_cache_create(0, dtype, sequences, kv_heads, head_dim, capacity, 64, C.byref(handle)))
    return handle


def _fill(cache, k, v, lengths):
    stream = B.lib().dl_b200_stream(B.cuda(0))
    kd, vd = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
    torch.cuda.synchronize()
    B.kcheck(B.lib().b200_kv_cache_append(cache, kd.data_ptr(), vd.data_ptr(), k.shape[2], stream))
    B.synchronize(0)
    arr = np.ascontiguousarray(lengths, dtype=np.int32)
    B.kcheck(B.lib().b200_kv_cache_set_lengths(cache, arr.ctypes.data_as(C.POINTER(C.c_int32)), stream))


@pytest.mark.parametrize("dtype,head_dim,heads,kv_heads", [(B.BF16, 64, 12, 4), (B.F32, 32, 8, 2)])
def test_static_scratch_matches_caller_scratch_twice(dtype, head_dim, heads, kv_heads):
    l = B.lib()
    stream = l.dl_b200_stream(B.cuda(0))
    rng = np.random.default_rng(head_dim)
    sequences, capacity = 6, 1200
    lengths = np.array([1199, 5, 130, 64, 400, 1025], dtype=np.int32)    # several splits, ragged
    cache = _cache(dtype, sequences, kv_heads, head_dim, capacity)
    try:
        k = rng.standard_normal((sequences, kv_heads, capacity, head_dim), dtype=np.float32)
        v = rng.standard_normal((sequences, kv_heads, capacity, head_dim), dtype=np.float32)
        _fill(cache, k, v, lengths)
        need = l.b200_attention_scratch_bytes(sequences, heads, kv_heads, head_dim, capacity, 64)
        assert 256 < need <= STATIC_BYTES          # the case really uses split partials
        scratch = torch.empty((need,), dtype=torch.uint8, device="cuda")
        for attempt in range(2):
            q = torch.from_numpy(rng.standard_normal((sequences, heads, head_dim), dtype=np.float32)).cuda()
            want = torch.zeros((sequences, heads * head_dim), dtype=torch.float32, device="cuda")
            got = torch.zeros_like(want)
            torch.cuda.synchronize()
            B.kcheck(l.b200_attention_decode(q.data_ptr(), sequences, 1, heads, cache, capacity, 1, scratch.data_ptr(), need,
                                             want.data_ptr(), stream))
            B.kcheck(l.b200_attention_decode_static(q.data_ptr(), sequences, 1, heads, cache, capacity, 1, got.data_ptr(), stream))
            B.synchronize(0)
            status = C.c_int32()
            B.kcheck(l.b200_take_device_status(0, stream, C.byref(status)))
            assert status.value == 0
            a, b = got.cpu().numpy(), want.cpu().numpy()
            assert np.isfinite(a).all() and np.abs(b).max() > 0
            assert float(np.abs(a - b).max() / np.abs(b).max()) < 1e-6, attempt
            # against the CPU oracle: with one new token per sequence, row s attends over keys 0 .. lengths[s]
            stored_k, stored_v = (W.bf16_to_f32(W.bf16_bits(k)), W.bf16_to_f32(W.bf16_bits(v))) if dtype == B.BF16 else (k, v)
            queries = q.cpu().numpy()
            for s, length in enumerate(lengths):
                seen = int(length) + 1
                reference = oracle.gqa_attention(queries[s][None, :, None, :], stored_k[s:s + 1, :, :seen], stored_v[s:s + 1, :, :seen])
                error = float(np.abs(a[s].reshape(heads, head_dim) - reference[0, :, 0, :]).max() / np.abs(reference).max())
                assert error < (1e-2 if dtype == B.BF16 else 1e-5), (attempt, s, error)   # the tolerances of the attention kernel tests
    finally:
        l.b200_kv_cache_release(cache)


def test_static_scratch_rejects_oversized_shapes():
    l = B.lib()
    stream = l.dl_b200_stream(B.cuda(0))
    sequences, heads, kv_heads, head_dim, capacity = 64, 32, 8, 128, 8192
    assert l.b200_attention_scratch_bytes(sequences, heads, kv_heads, head_dim, capacity, 64) > STATIC_BYTES
    cache = _cache(B.BF16, sequences, kv_heads, head_dim, capacity)
    try:
        q = torch.zeros((sequences, heads, head_dim), dtype=torch.float32, device="cuda")
        out = torch.zeros((sequences, heads * head_dim), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        status = l.b200_attention_decode_static(q.data_ptr(), sequences, 1, heads, cache, capacity, 1, out.data_ptr(), stream)
        assert status == -1
        message = l.b200_last_error().decode()
        assert "built-in array holds" in message and str(STATIC_BYTES) in message
    finally:
        l.b200_kv_cache_release(cache)
