"""Kernel-level parity: every CUDA kernel is called through the kernel C ABI (b200_*) and compared with the CPU
oracle on the same seeded inputs.  torch is used only to hold device memory.

Tolerances (relative = max|a-b| / max|b|):
  f32 paths           1e-5   (the 1e-4 logits budget of the f32 configuration leaves room for depth)
  bf16 KV / mma path  1e-2   (bf16 storage of K, V, q and the softmax weights; the bf16 logits budget is 2e-2)
"""
import ctypes as C

import numpy as np
import pytest

import ctorch_b200 as B
import oracle
from ctorch_b200 import workloads as W

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def rel(a, b):
    return float(np.abs(a.astype(np.float64) - b.astype(np.float64)).max() / max(1e-30, np.abs(b).max()))


def dev(array, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(array)).cuda()
    torch.cuda.synchronize()
    return t


def bf16_dev(bits):
    return dev(bits.view(np.int16))


def stream():
    return B.lib().dl_b200_stream(B.cuda(0))


def sync():
    B.synchronize(0)


class Cache:
    def __init__(self, dtype, sequences, kv_heads, head_dim, capacity, page_size=64):
        h = C.c_void_p()
        B.kcheck(B.lib().b200_kv_cache_create(0, dtype, sequences, kv_heads, head_dim, capacity, page_size, C.byref(h)))
        self.h, self.shape = h, (sequences, kv_heads, head_dim, capacity)

    def __del__(self):
        B.lib().b200_kv_cache_release(self.h)

    def set_lengths(self, lengths):
        arr = np.ascontiguousarray(lengths, dtype=np.int32)
        B.kcheck(B.lib().b200_kv_cache_set_lengths(self.h, arr.ctypes.data_as(C.POINTER(C.c_int32)), stream()))

    def set_page_table(self, table):
        arr = np.ascontiguousarray(table, dtype=np.int32)
        B.kcheck(B.lib().b200_kv_cache_set_page_table(self.h, arr.ctypes.data_as(C.POINTER(C.c_int32)), stream()))

    def pages_per_sequence(self):
        return B.lib().b200_kv_cache_pages_per_sequence(self.h)

    def append(self, k, v):
        kd, vd = dev(k), dev(v)
        B.kcheck(B.lib().b200_kv_cache_append(self.h, kd.data_ptr(), vd.data_ptr(), k.shape[2], stream()))
        sync()

    def gather(self, which, length):
        s, hk, hd, _ = self.shape
        out = torch.empty((s, hk, length, hd), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        B.kcheck(B.lib().b200_kv_cache_gather(self.h, which, length, out.data_ptr(), stream()))
        sync()
        return out.cpu().numpy()


def run_linear(x, w, epilogue=0, norm=None, eps=1e-5, residual=None, qkv=None, out_cols=None):
    rows, inner = x.shape
    out = w.shape[0]
    xd = dev(x)
    wd = bf16_dev(w) if w.dtype == np.uint16 else dev(w)
    nd = None
    if norm is not None:
        nd = bf16_dev(norm) if norm.dtype == np.uint16 else dev(norm)
    rd = dev(residual) if residual is not None else None
    y = torch.zeros((rows, out_cols or out), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    B.kcheck(B.lib().b200_linear(xd.data_ptr(), rows, inner, wd.data_ptr(), B.BF16 if w.dtype == np.uint16 else B.F32, out,
                                 nd.data_ptr() if nd is not None else None,
                                 (B.BF16 if norm.dtype == np.uint16 else B.F32) if norm is not None else 0, eps, epilogue,
                                 rd.data_ptr() if rd is not None else None, C.byref(qkv) if qkv is not None else None,
                                 y.data_ptr(), stream()))
    sync()
    return y.cpu().numpy()


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("rows,inner,out", [(1, 256, 256), (2, 768, 1280), (3, 64, 97), (5, 2048, 768), (8, 4096, 130),
                                            (11, 768, 514), (16, 768, 2048), (4, 12, 8), (1, 6152, 66), (19, 72, 40)])
def test_linear_store(dtype, rows, inner, out):
    rng = np.random.default_rng(rows * 1000 + inner + out)
    x = rng.standard_normal((rows, inner), dtype=np.float32)
    w = (0.05 * rng.standard_normal((out, inner), dtype=np.float32)).astype(np.float32)
    if dtype == "bf16":
        w = W.bf16_bits(w)
    got = run_linear(x, w)
    want = oracle.linear(x, w)
    assert rel(got, want) < 1e-5


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_linear_fused_norm_residual_swiglu(dtype):
    rng = np.random.default_rng(7)
    rows, inner, hidden = 6, 768, 1024
    cast = W.bf16_bits if dtype == "bf16" else (lambda a: a)
    x = rng.standard_normal((rows, inner), dtype=np.float32) * 3
    norm = cast((1 + 0.1 * rng.standard_normal(inner)).astype(np.float32))
    norm_f = W.bf16_to_f32(norm) if dtype == "bf16" else norm
    gate = cast(0.05 * rng.standard_normal((hidden, inner), dtype=np.float32))
    up = cast(0.05 * rng.standard_normal((hidden, inner), dtype=np.float32))
    xn = oracle.rms_norm(x, norm_f, 1e-5)
    # norm fused into a store
    assert rel(run_linear(x, gate, norm=norm), oracle.linear(xn, gate)) < 1e-5
    # SwiGLU epilogue on interleaved rows
    inter = np.empty((2 * hidden, inner), dtype=gate.dtype)
    inter[0::2], inter[1::2] = gate, up
    got = run_linear(x, inter, epilogue=2, norm=norm, out_cols=hidden)
    want = oracle.silu_mul(oracle.linear(xn, gate), oracle.linear(xn, up))
    assert rel(got, want) < 1e-5
    # residual epilogue
    res = rng.standard_normal((rows, hidden), dtype=np.float32)
    got = run_linear(x, gate, epilogue=1, residual=res)
    assert rel(got, res + oracle.linear(x, gate)) < 1e-5


def test_rms_norm_matches_reference_rounding():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((9, 768), dtype=np.float32) * 5
    w = (1 + 0.1 * rng.standard_normal(768)).astype(np.float32)
    xd, wd = dev(x), dev(w)
    y = torch.empty_like(xd)
    torch.cuda.synchronize()
    B.kcheck(B.lib().b200_rms_norm(xd.data_ptr(), wd.data_ptr(), B.F32, 9, 768, 1e-5, y.data_ptr(), stream()))
    sync()
    want = oracle.rms_norm(x, w, 1e-5)
    got = y.cpu().numpy()
    # f64 accumulation on both sides: at most the last bit differs (summation order of the f64 sum)
    assert np.abs(got.view(np.int32) - want.view(np.int32)).max() <= 1


def test_embedding_and_argmax_rules():
    rng = np.random.default_rng(5)
    table = W.bf16_bits(rng.standard_normal((50, 64), dtype=np.float32))
    ids = rng.integers(0, 50, size=(7,), dtype=np.int64)
    td, idd = bf16_dev(table), dev(ids)
    out = torch.empty((7, 64), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    B.kcheck(B.lib().b200_embedding(td.data_ptr(), B.BF16, idd.data_ptr(), 7, 50, 64, out.data_ptr(), stream()))
    sync()
    assert np.array_equal(out.cpu().numpy(), W.bf16_to_f32(table)[ids])

    x = rng.standard_normal((5, 32000), dtype=np.float32)
    x[0, 17] = x[0, 31999] = 9.0          # tie: the first wins
    x[1, 20000] = np.nan                  # NaN wins
    x[1, 25000] = np.nan
    x[2, :] = -1.0                        # all equal
    x[3, 31999] = 50.0                    # last element
    xd = dev(x)
    idx = torch.empty((5,), dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    B.kcheck(B.lib().b200_argmax(xd.data_ptr(), 5, 32000, idx.data_ptr(), stream()))
    sync()
    assert idx.cpu().numpy().tolist() == oracle.argmax(x).tolist() == [17, 20000, 0, 31999, int(np.argmax(x[4]))]


@pytest.mark.parametrize("cache_dtype", [B.F32, B.BF16])
def test_qkv_epilogue_rope_and_append(cache_dtype):
    """Fused q|k|v projection: RoPE on q and k, append of k and v at positions lengths[s] + t (paged)."""
    rng = np.random.default_rng(11)
    B_, L, H, HK, hd, cap = 3, 4, 6, 2, 32, 100
    D, KV = H * hd, HK * hd
    x = rng.standard_normal((B_ * L, D), dtype=np.float32)
    w = (0.05 * rng.standard_normal((D + 2 * KV, D), dtype=np.float32)).astype(np.float32)
    cos, sin = oracle.rope_tables(hd, cap)
    cache = Cache(cache_dtype, B_, HK, hd, cap)
    lengths = np.array([0, 61, 70], dtype=np.int32)   # crosses the 64-token page boundary
    cache.set_lengths(lengths)
    cd, sd = dev(cos), dev(sin)
    q = torch.zeros((B_ * L, D), dtype=torch.float32, device="cuda")
    args = B.QkvArgs(H, HK, hd, L, cd.data_ptr(), sd.data_ptr(), cap, cache.h.value, q.data_ptr(), 0, 0.0, None, None, None)
    run_linear(x, w, epilogue=3, qkv=args)
    y = oracle.linear(x, w)
    for b in range(B_):
        rows = y[b * L:(b + 1) * L]
        qb = rows[:, :D].reshape(1, L, H, hd).transpose(0, 2, 1, 3)
        kb = rows[:, D:D + KV].reshape(1, L, HK, hd).transpose(0, 2, 1, 3)
        vb = rows[:, D + KV:].reshape(1, L, HK, hd).transpose(0, 2, 1, 3)
        q_want = oracle.rotary(qb, 10000.0, cap, int(lengths[b])).transpose(0, 2, 1, 3).reshape(L, D)
        k_want = oracle.rotary(kb, 10000.0, cap, int(lengths[b]))[0]
        assert rel(q.cpu().numpy()[b * L:(b + 1) * L], q_want) < 1e-5
        end = int(lengths[b]) + L
        got_k = cache.gather(0, end)[b][:, lengths[b]:end]
        got_v = cache.gather(1, end)[b][:, lengths[b]:end]
        tol = 1e-5 if cache_dtype == B.F32 else 5e-3
        assert rel(got_k, k_want) < tol and rel(got_v, vb[0]) < tol


def attention(q, cache, L, heads, max_length, causal=1):
    rows = q.shape[0]
    s, hk, hd, cap = cache.shape
    qd = dev(q)
    need = B.lib().b200_attention_scratch_bytes(rows, heads, hk, hd, max_length, 64)
    scratch = torch.empty((need,), dtype=torch.uint8, device="cuda")
    out = torch.zeros((rows, heads * hd), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    B.kcheck(B.lib().b200_attention_decode(qd.data_ptr(), rows, L, heads, cache.h, max_length, causal, scratch.data_ptr(), need,
                                           out.data_ptr(), stream()))
    sync()
    status = C.c_int32()
    B.kcheck(B.lib().b200_take_device_status(0, stream(), C.byref(status)))
    assert status.value == 0
    return out.cpu().numpy()


@pytest.mark.parametrize("cache_dtype,hd,heads,kv_heads,lengths", [
    (B.F32, 32, 8, 2, [1, 37, 64, 65, 200]),          # generic path, C1 head shape
    (B.F32, 16, 4, 4, [5, 130]),
    (B.BF16, 64, 12, 4, [1, 63, 64, 65, 700]),        # tensor-core path, C2 head shape (G = 3)
    (B.BF16, 128, 32, 8, [17, 128, 1000, 2500]),      # tensor-core path, C3/C5 head shape (G = 4), several splits
    (B.BF16, 128, 8, 8, [300]),                        # G = 1
    (B.BF16, 64, 16, 1, [129, 77]),                    # G = 16
    (B.BF16, 32, 8, 2, [40, 90]),                      # bf16 pool on the generic path
    # more unsplit items than the GPU holds at once: persistent CTAs walk several items each, their producer warp running
    # into the next item's pages while the current one is merged (96 x 8 = 768 items, two CTAs per SM; 200 x 2 = 400, one)
    (B.BF16, 64, 32, 8, [1 + (37 * s) % 700 for s in range(96)]),
    (B.BF16, 128, 8, 2, [1 + (53 * s) % 900 for s in range(200)]),
])
def test_decode_attention_ragged(cache_dtype, hd, heads, kv_heads, lengths):
    """One new token per sequence, per-sequence context lengths, shuffled physical pages."""
    rng = np.random.default_rng(hd + heads + len(lengths))
    n = len(lengths)
    cap = max(lengths)
    cache = Cache(cache_dtype, n, kv_heads, hd, cap)
    pages = cache.pages_per_sequence() * n
    cache.set_page_table(rng.permutation(pages).astype(np.int32))
    k = rng.standard_normal((n, kv_heads, cap, hd), dtype=np.float32)
    v = rng.standard_normal((n, kv_heads, cap, hd), dtype=np.float32)
    cache.set_lengths(np.zeros(n, dtype=np.int32))
    cache.append(k, v)
    # the kernel's rule for L == 1: row s sees keys 0 .. lengths[s] (the new token included)
    cache.set_lengths(np.array(lengths, dtype=np.int32) - 1)
    q = rng.standard_normal((n, heads, hd), dtype=np.float32)
    got = attention(q, cache, 1, heads, cap)
    if cache_dtype == B.BF16:
        k, v = W.bf16_to_f32(W.bf16_bits(k)), W.bf16_to_f32(W.bf16_bits(v))
    for s, length in enumerate(lengths):
        want = oracle.gqa_attention(q[s][None, :, None, :], k[s:s + 1, :, :length], v[s:s + 1, :, :length])
        tol = 1e-5 if cache_dtype == B.F32 else 1e-2
        assert rel(got[s].reshape(heads, hd), want[0, :, 0, :]) < tol, (s, length)


@pytest.mark.parametrize("cache_dtype,hd", [(B.F32, 32), (B.BF16, 64)])
def test_chunk_attention_is_causal(cache_dtype, hd):
    """L new tokens per sequence appended to a prefix: row l sees keys 0 .. prefix + l."""
    rng = np.random.default_rng(23)
    n, L, heads, kv_heads, prefix = 2, 5, 4, 2, 70
    cap = prefix + L
    cache = Cache(cache_dtype, n, kv_heads, hd, cap)
    k = rng.standard_normal((n, kv_heads, cap, hd), dtype=np.float32)
    v = rng.standard_normal((n, kv_heads, cap, hd), dtype=np.float32)
    cache.append(k, v)
    cache.set_lengths(np.full(n, prefix, dtype=np.int32))
    q = rng.standard_normal((n * L, heads, hd), dtype=np.float32)
    got = attention(q, cache, L, heads, cap).reshape(n, L, heads, hd)
    if cache_dtype == B.BF16:
        k, v = W.bf16_to_f32(W.bf16_bits(k)), W.bf16_to_f32(W.bf16_bits(v))
    want = oracle.gqa_attention(q.reshape(n, L, heads, hd).transpose(0, 2, 1, 3), k, v, causal_offset=prefix)
    assert rel(got, want.transpose(0, 2, 1, 3)) < (1e-5 if cache_dtype == B.F32 else 1e-2)


def test_attention_linearity_in_values_at_long_context():
    """Size-independent property at a context the oracle would take minutes for: attention is linear in V, and
    with all keys equal it returns the mean of V."""
    rng = np.random.default_rng(31)
    n, heads, kv_heads, hd, length = 2, 32, 8, 128, 20000
    cache = Cache(B.BF16, n, kv_heads, hd, length)
    k = np.broadcast_to(rng.standard_normal((n, kv_heads, 1, hd), dtype=np.float32), (n, kv_heads, length, hd)).copy()
    v = W.bf16_to_f32(W.bf16_bits(rng.standard_normal((n, kv_heads, length, hd), dtype=np.float32)))
    cache.append(k, v)
    cache.set_lengths(np.full(n, length - 1, dtype=np.int32))
    q = rng.standard_normal((n, heads, hd), dtype=np.float32)
    got = attention(q, cache, 1, heads, length).reshape(n, heads, hd)
    mean = v.mean(axis=2)                                   # [n, kv_heads, hd]
    want = np.repeat(mean, heads // kv_heads, axis=1)
    assert np.abs(got - want).max() < 2e-3


def test_rotary_permute_feedback_helpers():
    rng = np.random.default_rng(41)
    x = rng.standard_normal((3, 2, 4, 16), dtype=np.float32)
    cos, sin = oracle.rope_tables(16, 12)
    xd, cd, sd = dev(x), dev(cos[3:7]), dev(sin[3:7])
    y = torch.empty_like(xd)
    torch.cuda.synchronize()
    B.kcheck(B.lib().b200_rotary(xd.data_ptr(), 6, 4, 16, cd.data_ptr(), sd.data_ptr(), y.data_ptr(), stream()))
    sync()
    assert np.array_equal(y.cpu().numpy(), oracle.rotary(x, 10000.0, 12, 3))
    p = torch.empty((3, 4, 2, 16), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    B.kcheck(B.lib().b200_permute_0213(xd.data_ptr(), 3, 2, 4, 16, p.data_ptr(), stream()))
    sync()
    assert np.array_equal(p.cpu().numpy(), x.transpose(0, 2, 1, 3))


def shadow_to_f32(hi, lo):
    return (hi.float() + lo.float()).cpu().numpy()


@pytest.mark.parametrize("rows,inner,out", [(16, 768, 1280), (5, 2048, 768), (16, 768, 4096), (3, 72, 40)])
def test_shadow_protocol_norm_linear_residual(rows, inner, out):
    """Activations travelling as bf16 hi + lo planes: producer folds the norm weight and leaves row sums of squares,
    the consumer applies 1/sqrt(mean + eps); residual epilogue writes the next shadow and its partial sums."""
    l = B.lib()
    rng = np.random.default_rng(rows + inner + out)
    x = rng.standard_normal((rows, inner), dtype=np.float32) * 2
    norm = W.bf16_bits((1 + 0.1 * rng.standard_normal(inner)).astype(np.float32))
    w = W.bf16_bits(0.05 * rng.standard_normal((out, inner), dtype=np.float32))
    res = rng.standard_normal((rows, out), dtype=np.float32)
    next_norm = W.bf16_bits((1 + 0.1 * rng.standard_normal(out)).astype(np.float32))
    xd, nd, wd, rd, nnd = dev(x), bf16_dev(norm), bf16_dev(w), dev(res), bf16_dev(next_norm)
    hi = torch.zeros((rows, inner), dtype=torch.bfloat16, device="cuda")
    lo = torch.zeros_like(hi)
    sq = torch.zeros((1, rows), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    B.kcheck(l.b200_shadow_from_rows(xd.data_ptr(), rows, inner, nd.data_ptr(), B.BF16, hi.data_ptr(), lo.data_ptr(), sq.data_ptr(), stream()))
    sync()
    assert rel(shadow_to_f32(hi, lo), x * W.bf16_to_f32(norm)) < 2e-5
    assert rel(sq.cpu().numpy()[0], (x.astype(np.float64) ** 2).sum(axis=1)) < 1e-5
    parts = l.b200_linear_shadow_parts(rows, inner, out)
    assert parts > 0
    y = torch.zeros((rows, out), dtype=torch.float32, device="cuda")
    ohi = torch.zeros((rows, out), dtype=torch.bfloat16, device="cuda")
    olo = torch.zeros_like(ohi)
    osq = torch.zeros((parts, rows), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    args = B.ShadowLinearArgs(hi.data_ptr(), lo.data_ptr(), rows, inner, wd.data_ptr(), out, sq.data_ptr(), 1, 1e-5, 1, rd.data_ptr(), None,
                              y.data_ptr(), ohi.data_ptr(), olo.data_ptr(), nnd.data_ptr(), B.BF16, osq.data_ptr())
    B.kcheck(l.b200_linear_shadow(C.byref(args), stream()))
    sync()
    want = res + oracle.linear(oracle.rms_norm(x, W.bf16_to_f32(norm), 1e-5), w)
    assert rel(y.cpu().numpy(), want) < 2e-5
    assert rel(shadow_to_f32(ohi, olo), want * W.bf16_to_f32(next_norm)) < 3e-5
    assert rel(osq.cpu().numpy().sum(axis=0), (want.astype(np.float64) ** 2).sum(axis=1)) < 1e-4


def test_shadow_protocol_swiglu_and_attention_output():
    l = B.lib()
    rng = np.random.default_rng(77)
    rows, inner, hidden = 16, 768, 2048
    x = rng.standard_normal((rows, inner), dtype=np.float32)
    gate = W.bf16_bits(0.05 * rng.standard_normal((hidden, inner), dtype=np.float32))
    up = W.bf16_bits(0.05 * rng.standard_normal((hidden, inner), dtype=np.float32))
    inter = np.empty((2 * hidden, inner), dtype=np.uint16)
    inter[0::2], inter[1::2] = gate, up
    xd, wd = dev(x), bf16_dev(inter)
    hi = torch.zeros((rows, inner), dtype=torch.bfloat16, device="cuda")
    lo = torch.zeros_like(hi)
    sq = torch.zeros((1, rows), dtype=torch.float32, device="cuda")
    ahi = torch.zeros((rows, hidden), dtype=torch.bfloat16, device="cuda")
    alo = torch.zeros_like(ahi)
    torch.cuda.synchronize()
    B.kcheck(l.b200_shadow_from_rows(xd.data_ptr(), rows, inner, None, 0, hi.data_ptr(), lo.data_ptr(), sq.data_ptr(), stream()))
    args = B.ShadowLinearArgs(hi.data_ptr(), lo.data_ptr(), rows, inner, wd.data_ptr(), 2 * hidden, None, 0, 0.0, 2, None, None, None,
                              ahi.data_ptr(), alo.data_ptr(), None, 0, None)
    B.kcheck(l.b200_linear_shadow(C.byref(args), stream()))
    sync()
    want = oracle.silu_mul(oracle.linear(x, gate), oracle.linear(x, up))
    assert rel(shadow_to_f32(ahi, alo), want) < 3e-5
    # attention result as a shadow equals the f32 result
    n, heads, kv_heads, hd, cap = 4, 12, 4, 64, 300
    cache = Cache(B.BF16, n, kv_heads, hd, cap)
    k = rng.standard_normal((n, kv_heads, cap, hd), dtype=np.float32)
    v = rng.standard_normal((n, kv_heads, cap, hd), dtype=np.float32)
    cache.append(k, v)
    cache.set_lengths(np.array([299, 10, 64, 128], dtype=np.int32))
    q = rng.standard_normal((n, heads, hd), dtype=np.float32)
    plain = attention(q, cache, 1, heads, cap)
    qd = dev(q)
    shi = torch.zeros((n, heads * hd), dtype=torch.bfloat16, device="cuda")
    slo = torch.zeros_like(shi)
    scratch = torch.empty((1 << 20,), dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    B.kcheck(l.b200_attention_decode_shadow(qd.data_ptr(), n, 1, heads, cache.h, cap, 1, scratch.data_ptr(), 1 << 20, shi.data_ptr(),
                                            slo.data_ptr(), stream()))
    sync()
    assert rel(shadow_to_f32(shi, slo), plain) < 2e-5


@pytest.mark.parametrize("rows,inner,out,epilogue", [(40, 768, 1280, 0), (130, 2048, 768, 1), (300, 768, 4096, 2), (17, 4096, 200, 1),
                                                     (128, 72, 136, 0), (32, 4096, 1024, 1), (256, 2048, 3072, 2),
                                                     (1000, 512, 2560, 0), (20, 256, 76000, 0), (1100, 2304, 2304, 1), (40, 4096, 32, 0), (300, 768, 24, 0),
                                                     (64, 2048, 16384, 2), (256, 2048, 16384, 2), (200, 8192, 2048, 1), (96, 2048, 2048, 1),
                                                     (32, 2048, 32000, 0), (48, 1032, 1000, 0), (257, 768, 1280, 1),
                                                     (40, 768, 1282, 1), (24, 512, 330, 0), (150, 2048, 1282, 1)])
def test_dense_tensor_core_linear(rows, inner, out, epilogue):
    """More than 16 rows (or a wide input) take the tcgen05 kernels: shadow input, split norm, every epilogue family.
    Up to 256 rows run on the decode-batch kernel (weights as the streamed M operand, tokens as the N side): one, two or four
    weight tiles per CTA ((256, 2048, 16384): two tiles and a K split of two; (32, 2048, 32000): two tiles, no split), K split
    over a thread-block cluster with the partial tiles summed through distributed shared memory ((200, 8192, 2048): eight
    CTAs, a row count that is no multiple of 16), ragged last tiles and K blocks ((48, 1032, 1000), (17, 4096, 200)).  More
    rows run on the prefill kernel: (1000, 512, 2560) on its persistent variant (8 token tiles, short K, more tiles than
    SMs), (1100, 2304, 2304) one tile per CTA with two CTAs per SM, (300, 768, 4096) and (257, 768, 1280) with a K split;
    widths that are no multiple of 4 ((40, 768, 1282), (24, 512, 330), (150, 2048, 1282)) take the epilogue's pair form;
    (40, 4096, 32) and (300, 768, 24) (at most 64 output features, store epilogue: adapter down-projections) on the thin
    CUDA-core kernel."""
    l = B.lib()
    rng = np.random.default_rng(rows + inner + out)
    x = rng.standard_normal((rows, inner), dtype=np.float32) * 2
    norm = W.bf16_bits((1 + 0.1 * rng.standard_normal(inner)).astype(np.float32))
    w = W.bf16_bits(0.05 * rng.standard_normal((out, inner), dtype=np.float32))
    xd, nd, wd = dev(x), bf16_dev(norm), bf16_dev(w)
    hi = torch.zeros((rows, inner), dtype=torch.bfloat16, device="cuda")
    lo = torch.zeros_like(hi)
    sq = torch.zeros((1, rows), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    B.kcheck(l.b200_shadow_from_rows(xd.data_ptr(), rows, inner, nd.data_ptr(), B.BF16, hi.data_ptr(), lo.data_ptr(), sq.data_ptr(), stream()))
    xn = oracle.rms_norm(x, W.bf16_to_f32(norm), 1e-5)
    full = oracle.linear(xn, w)
    parts = l.b200_linear_shadow_parts(rows, inner, out)
    assert parts in ((out + 127) // 128, (out + 255) // 256)   # one partial per feature tile of the dense kernel
    cols = out // 2 if epilogue == 2 else out
    y = torch.zeros((rows, cols), dtype=torch.float32, device="cuda")
    ohi = torch.zeros((rows, cols), dtype=torch.bfloat16, device="cuda")
    olo = torch.zeros_like(ohi)
    osq = torch.zeros((parts, rows), dtype=torch.float32, device="cuda")
    res = rng.standard_normal((rows, out), dtype=np.float32)
    rd = dev(res)
    torch.cuda.synchronize()
    args = B.ShadowLinearArgs(hi.data_ptr(), lo.data_ptr(), rows, inner, wd.data_ptr(), out, sq.data_ptr(), 1, 1e-5, epilogue,
                              rd.data_ptr() if epilogue == 1 else None, None, y.data_ptr(),
                              ohi.data_ptr() if epilogue else None, olo.data_ptr() if epilogue else None, None, 0,
                              osq.data_ptr() if epilogue == 1 else None)
    B.kcheck(l.b200_linear_shadow(C.byref(args), stream()))
    sync()
    status = C.c_int32()
    B.kcheck(l.b200_take_device_status(0, stream(), C.byref(status)))
    assert status.value == 0
    if epilogue == 0:
        want = full
    elif epilogue == 1:
        want = res + full
    else:
        want = oracle.silu_mul(np.ascontiguousarray(full[:, 0::2]), np.ascontiguousarray(full[:, 1::2]))
    assert rel(y.cpu().numpy(), want) < 3e-5
    if epilogue:
        assert rel(shadow_to_f32(ohi, olo), want) < 4e-5
    if epilogue == 1:
        assert rel(osq.cpu().numpy().sum(axis=0), (want.astype(np.float64) ** 2).sum(axis=1)) < 1e-4


@pytest.mark.parametrize("rows,inner,vocab", [(16, 768, 32000), (5, 256, 1000), (40, 512, 5000), (32, 2048, 1024), (200, 256, 777 * 2),
                                              (20, 256, 76000)])
def test_fused_logits_argmax(rows, inner, vocab):
    """Logits + greedy choice without logits in memory: per-tile candidates from the projection's epilogue (streaming kernel
    up to 16 rows, tcgen05 kernel above, K-split clusters when the tiles are few), then the merge.  Duplicated weight
    rows make exact ties: the lowest index must win (src/kernels/cpu/reduction.cpp:128-151 of the reference)."""
    l = B.lib()
    rng = np.random.default_rng(rows * 7 + vocab)
    x = rng.standard_normal((rows, inner), dtype=np.float32)
    norm = W.bf16_bits((1 + 0.1 * rng.standard_normal(inner)).astype(np.float32))
    w = 0.05 * rng.standard_normal((vocab, inner), dtype=np.float32)
    xn = oracle.rms_norm(x, W.bf16_to_f32(norm), 1e-5)
    # make the winning row of every activation row appear three times (same bits -> equal logits)
    first = oracle.linear(xn, W.bf16_bits(w))
    for r in range(rows):
        top = int(first[r].argmax())
        for clone in ((top * 7 + 11) % vocab, (top * 13 + 5) % vocab):
            w[clone] = w[top]
    wb = W.bf16_bits(w)
    logits = oracle.linear(xn, wb)
    want = oracle.argmax(logits)
    xd, nd, wd = dev(x), bf16_dev(norm), bf16_dev(wb)
    hi = torch.zeros((rows, inner), dtype=torch.bfloat16, device="cuda")
    lo = torch.zeros_like(hi)
    sq = torch.zeros((1, rows), dtype=torch.float32, device="cuda")
    B.kcheck(l.b200_shadow_from_rows(xd.data_ptr(), rows, inner, nd.data_ptr(), B.BF16, hi.data_ptr(), lo.data_ptr(), sq.data_ptr(), stream()))
    parts = l.b200_linear_argmax_parts(rows, inner, vocab)
    assert parts > 0
    best_value = torch.zeros((parts, rows), dtype=torch.float32, device="cuda")
    best_index = torch.zeros((parts, rows), dtype=torch.int32, device="cuda")
    next_ids = torch.full((rows,), -1, dtype=torch.int64, device="cuda")
    ids = torch.full((rows,), -1, dtype=torch.int64, device="cuda")
    history = torch.full((3, rows), -1, dtype=torch.int64, device="cuda")
    counter = torch.tensor([1], dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    args = B.ShadowLinearArgs(hi.data_ptr(), lo.data_ptr(), rows, inner, wd.data_ptr(), vocab, sq.data_ptr(), 1, 1e-5, 4, None, None, None,
                              None, None, None, 0, None, best_value.data_ptr(), best_index.data_ptr())
    B.kcheck(l.b200_linear_shadow(C.byref(args), stream()))
    B.kcheck(l.b200_argmax_finish(best_value.data_ptr(), best_index.data_ptr(), parts, rows, next_ids.data_ptr(), ids.data_ptr(),
                                  history.data_ptr(), 3, counter.data_ptr(), None, 0, stream()))
    sync()
    got = next_ids.cpu().numpy()
    # a tie in the oracle's f32 sums may not be a tie in the tensor-core sums (other summation order) only if the clone rows
    # differ, and they do not: equal rows give equal sums on either side
    chosen = logits[np.arange(rows), got]
    assert np.allclose(chosen, logits.max(axis=1), rtol=0, atol=2e-4 * np.abs(logits).max())
    near_tie = np.sort(logits, axis=1)[:, -4] > logits.max(axis=1) - 1e-3 * np.abs(logits).max()   # a fourth contender
    assert np.array_equal(got[~near_tie], want[~near_tie])
    assert np.array_equal(ids.cpu().numpy(), got) and np.array_equal(history.cpu().numpy()[1], got)
    assert int(counter.item()) == 2


@pytest.mark.parametrize("rows,width,temperature", [(16, 32000, 0.8), (3, 517, 1.5), (40, 1000, 0.3)])
def test_temperature_sampling(rows, width, temperature):
    """Draws must equal the oracle's (softmax + running-sum inverse) unless the variate lies within 1e-6 of a boundary of
    the running sums, where the summation order of the two may legitimately disagree."""
    l = B.lib()
    rng = np.random.default_rng(rows + width)
    logits = (rng.standard_normal((rows, width)) * rng.uniform(0.5, 5.0, size=(rows, 1))).astype(np.float32)
    uniforms = rng.uniform(0, 1, rows)
    uniforms[0] = 0.0
    uniforms[-1] = 1.0 - 2.0 ** -53
    xd = dev(logits)
    ud = torch.from_numpy(uniforms).cuda()
    index = torch.full((rows,), -1, dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    B.kcheck(l.b200_sample(xd.data_ptr(), rows, width, temperature, ud.data_ptr(), index.data_ptr(), stream()))
    sync()
    got = index.cpu().numpy()
    want = oracle.sample(logits, temperature, uniforms)
    scaled = logits / np.float32(temperature)
    p = np.exp(scaled - scaled.max(axis=1, keepdims=True)).astype(np.float64)
    running = np.cumsum(p / p.sum(axis=1, keepdims=True), axis=1)
    for r in range(rows):
        if got[r] != want[r]:
            lo, hi = sorted((got[r], want[r]))
            assert hi - lo == 1 and abs(running[r, lo] - uniforms[r]) < 1e-6, (r, got[r], want[r])
    assert (got >= 0).all() and (got < width).all()


def _tp_regions(world, slot_bytes):
    l = B.lib()
    size = l.b200_tp_region_bytes(slot_bytes, world)
    regions = [torch.zeros((size,), dtype=torch.uint8, device="cuda") for _ in range(world)]
    table = (C.c_void_p * world)(*[r.data_ptr() for r in regions])
    return regions, table


def _slot_view(region, slot_bytes, world, slot, sender, rows, width):
    """Where rank `sender` deposits its partial rows of sum `slot` inside one rank's region."""
    at = B.lib().b200_tp_slot(region.data_ptr(), slot_bytes, world, slot, sender) - region.data_ptr()
    assert at == 4096 + (slot * world + sender) * slot_bytes
    return region[at: at + rows * width * 4].view(torch.float32).view(rows, width)


def test_peer_memory_sum_one_gpu():
    """The tensor-parallel sum kernel on one GPU: as a group of one, and as rank 0 of two with the other rank's arrival and
    partial rows put in place by the host beforehand (two kernels that wait on one another never share a GPU).  The rows of
    every sender lie in the summing rank's own region: the projections push them there."""
    l = B.lib()
    rows, width, slot_bytes = 5, 2560, 65536    # 2560 columns: three column chunks per row, the last one partial
    rng = np.random.default_rng(12)
    norm = W.bf16_bits((1 + 0.1 * rng.standard_normal(width)).astype(np.float32))
    nd = bf16_dev(norm)
    out = torch.zeros((rows, width), device="cuda")
    hi = torch.zeros((rows, width), dtype=torch.bfloat16, device="cuda")
    lo = torch.zeros_like(hi)
    sums = torch.zeros((l.b200_tp_reduce_parts(width), rows), device="cuda")
    for world, pull in ((1, 0), (2, 0), (2, 1)):
        regions, table = _tp_regions(world, slot_bytes)
        for call, slot in ((1, 0), (2, 1), (3, 0)):
            parts = [rng.standard_normal((rows, width), dtype=np.float32) for _ in range(world)]
            for r in range(world):
                # pushed: every sender's rows lie in rank 0's own region (the sum reads local memory only); pulled: sender
                # r's rows lie in rank r's region and the sum loads them from there
                _slot_view(regions[r if pull else 0], slot_bytes, world, slot, r, rows, width).copy_(torch.from_numpy(parts[r]))
            if world == 2:   # rank 1 "arrived" for this call
                regions[0][4:8].view(torch.int32)[0] = call
            torch.cuda.synchronize()
            B.kcheck(l.b200_tp_reduce_shadow(table, 0, world, slot, slot_bytes, pull, rows, width, nd.data_ptr(), B.BF16, out.data_ptr(),
                                             hi.data_ptr(), lo.data_ptr(), sums.data_ptr(), stream()))
            sync()
            status = C.c_int32()
            B.kcheck(l.b200_take_device_status(0, stream(), C.byref(status)))
            assert status.value == 0
            want = parts[0] if world == 1 else parts[0] + parts[1]
            assert np.array_equal(out.cpu().numpy(), want)
            assert rel(shadow_to_f32(hi, lo), want * W.bf16_to_f32(norm)) < 2e-5
            assert rel(sums.cpu().numpy().sum(axis=0), (want.astype(np.float64) ** 2).sum(axis=1)) < 1e-5
            control = regions[0][:256].view(torch.int32).cpu().numpy()
            assert control[0] == call and control[32] == call and control[33] == 0      # arrive[0], calls, ticket
            if world == 2:
                assert regions[1][:4].view(torch.int32).item() == call                  # the signal sent to the peer


def test_peer_memory_sum_gives_up_when_a_rank_never_arrives():
    """A flag that nothing sets: the wait ends after its limit, the status word reports it, the context stays usable, and a
    later call does not wait again while the status is set."""
    import time
    l = B.lib()
    rows, width, slot_bytes = 2, 256, 4096
    regions, table = _tp_regions(2, slot_bytes)
    out = torch.zeros((rows, width), device="cuda")
    hi = torch.zeros((rows, width), dtype=torch.bfloat16, device="cuda")
    lo = torch.zeros_like(hi)
    sums = torch.zeros((1, rows), device="cuda")
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    B.kcheck(l.b200_tp_reduce_shadow(table, 0, 2, 0, slot_bytes, 0, rows, width, None, 0, out.data_ptr(), hi.data_ptr(), lo.data_ptr(),
                                     sums.data_ptr(), stream()))
    sync()
    waited = time.perf_counter() - t0
    assert 1.5 < waited < 10.0
    t0 = time.perf_counter()
    B.kcheck(l.b200_tp_reduce_shadow(table, 0, 2, 1, slot_bytes, 1, rows, width, None, 0, out.data_ptr(), hi.data_ptr(), lo.data_ptr(),
                                     sums.data_ptr(), stream()))
    sync()
    assert time.perf_counter() - t0 < 1.0
    status = C.c_int32()
    B.kcheck(l.b200_take_device_status(0, stream(), C.byref(status)))
    assert status.value != 0
    B.kcheck(l.b200_take_device_status(0, stream(), C.byref(status)))
    assert status.value == 0
    x = torch.ones((4,), device="cuda") * 2
    assert float(x.sum()) == 8.0


@pytest.mark.parametrize("rows,inner,out", [(40, 768, 1280), (256, 2048, 3072), (32, 4096, 1024)])
def test_dense_linear_with_single_plane_activations(rows, inner, out):
    """x_lo = NULL: the dense kernel multiplies the hi plane only, i.e. activations rounded to bf16.  The result must equal
    the oracle's linear of the ROUNDED activations to f32 accuracy, and the unrounded one within bf16 resolution."""
    l = B.lib()
    rng = np.random.default_rng(rows + out)
    x = rng.standard_normal((rows, inner), dtype=np.float32)
    w = W.bf16_bits(0.05 * rng.standard_normal((out, inner), dtype=np.float32))
    xd, wd = dev(x), bf16_dev(w)
    hi = torch.zeros((rows, inner), dtype=torch.bfloat16, device="cuda")
    lo = torch.zeros_like(hi)
    sq = torch.zeros((1, rows), dtype=torch.float32, device="cuda")
    y = torch.zeros((rows, out), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    B.kcheck(l.b200_shadow_from_rows(xd.data_ptr(), rows, inner, None, 0, hi.data_ptr(), lo.data_ptr(), sq.data_ptr(), stream()))
    args = B.ShadowLinearArgs(hi.data_ptr(), None, rows, inner, wd.data_ptr(), out, None, 0, 0.0, 0, None, None, y.data_ptr(),
                              None, None, None, 0, None, None, None)
    B.kcheck(l.b200_linear_shadow(C.byref(args), stream()))
    sync()
    rounded = W.bf16_to_f32(W.bf16_bits(x))
    assert rel(y.cpu().numpy(), oracle.linear(rounded, w)) < 3e-5
    assert rel(y.cpu().numpy(), oracle.linear(x, w)) < 1e-2
    # up to 16 rows the streaming kernel serves the call and needs both planes
    args = B.ShadowLinearArgs(hi.data_ptr(), None, 8, 768, wd.data_ptr(), 64, None, 0, 0.0, 0, None, None, y.data_ptr(),
                              None, None, None, 0, None, None, None)
    assert l.b200_linear_shadow(C.byref(args), stream()) != 0


@pytest.mark.parametrize("a_shape,b_shape,axes_a,axes_b", [((3, 4, 5), (5, 6), (2,), (0,)), ((2, 3, 4, 5), (4, 7, 3), (1, 2), (2, 0)),
                                                             ((6, 8), (6, 8), (0, 1), (0, 1)), ((2, 5, 3), (4, 3, 5), (-2, -1), (2, 1))])
def test_tensordot_matches_the_reference_rule(a_shape, b_shape, axes_a, axes_b):
    """dl_tensordot (include/dl/decoder_c_api.h:13-14 of the reference, src/ops/contraction.cpp:9-42): contracted axes paired
    in the given order, the result has a's remaining axes followed by b's; checked against numpy.tensordot in f64."""
    rng = np.random.default_rng(len(a_shape) * 10 + len(b_shape))
    a = rng.standard_normal(a_shape, dtype=np.float32)
    b = rng.standard_normal(b_shape, dtype=np.float32)
    ta, tb = B.Tensor.from_numpy(a, device=B.cuda(0)), B.Tensor.from_numpy(b, device=B.cuda(0))
    xa = (C.c_int64 * len(axes_a))(*axes_a)
    xb = (C.c_int64 * len(axes_b))(*axes_b)
    out = C.c_void_p()
    B.check(B.lib().dl_tensordot(ta.h, tb.h, B.Shape(xa, len(axes_a)), B.Shape(xb, len(axes_b)), C.byref(out)))
    got = B.Tensor(out).numpy()
    want = np.tensordot(a.astype(np.float64), b.astype(np.float64), axes=(list(axes_a), list(axes_b)))
    assert got.shape == want.shape
    assert rel(got, want) < 1e-5
    # mismatching contracted sizes and repeated axes are refused with the reference's messages
    bad = C.c_void_p(1)
    last_a, first_b = (C.c_int64 * 1)(len(a_shape) - 1), (C.c_int64 * 1)(0)
    if a_shape[-1] != b_shape[0]:
        assert B.lib().dl_tensordot(ta.h, tb.h, B.Shape(last_a, 1), B.Shape(first_b, 1), C.byref(bad)) == 1
        assert not bad.value and b"contracted dimensions differ" in B.lib().dl_last_error()
    twice = (C.c_int64 * 2)(0, 0)
    assert B.lib().dl_tensordot(ta.h, tb.h, B.Shape(twice, 2), B.Shape(twice, 2), C.byref(bad)) == 1
    assert b"must be distinct" in B.lib().dl_last_error()


@pytest.mark.parametrize("rows,inner,out,epilogue", [(4, 512, 1024, 1), (40, 1024, 512, 1), (200, 768, 1280, 0), (16, 2048, 768, 0)])
def test_projection_pushes_its_rows_to_extra_destinations(rows, inner, out, epilogue):
    """y_copies of a shadow linear: every extra destination receives exactly the rows written to y - the mechanism by which
    a tensor-parallel rank's projection deposits its partial sums in the peers' memory from its own epilogue (here the
    destinations are buffers of the same GPU).  Streaming kernel (4 and 16 rows), decode-batch kernel (40), prefill kernel (200)."""
    l = B.lib()
    rng = np.random.default_rng(rows + out)
    x = rng.standard_normal((rows, inner), dtype=np.float32)
    w = W.bf16_bits(0.05 * rng.standard_normal((out, inner), dtype=np.float32))
    res = rng.standard_normal((rows, out), dtype=np.float32)
    xd, wd, rd = dev(x), bf16_dev(w), dev(res)
    hi = torch.zeros((rows, inner), dtype=torch.bfloat16, device="cuda")
    lo = torch.zeros_like(hi)
    sq = torch.zeros((1, rows), dtype=torch.float32, device="cuda")
    y = torch.zeros((rows, out), dtype=torch.float32, device="cuda")
    copies = [torch.full((rows, out), -7.0, dtype=torch.float32, device="cuda") for _ in range(3)]
    table = (C.c_void_p * 3)(*[c.data_ptr() for c in copies])
    torch.cuda.synchronize()
    B.kcheck(l.b200_shadow_from_rows(xd.data_ptr(), rows, inner, None, 0, hi.data_ptr(), lo.data_ptr(), sq.data_ptr(), stream()))
    args = B.ShadowLinearArgs(hi.data_ptr(), lo.data_ptr(), rows, inner, wd.data_ptr(), out, None, 0, 0.0, epilogue,
                              rd.data_ptr() if epilogue == 1 else None, None, y.data_ptr(), None, None, None, 0, None, None, None, table, 3)
    B.kcheck(l.b200_linear_shadow(C.byref(args), stream()))
    sync()
    want = oracle.linear(x, w) + (res if epilogue == 1 else 0)
    assert rel(y.cpu().numpy(), want) < 3e-5
    for copy in copies:
        assert torch.equal(copy, y)
    bad = B.ShadowLinearArgs(hi.data_ptr(), lo.data_ptr(), rows, inner, wd.data_ptr(), out, None, 0, 0.0, 2, None, None, y.data_ptr(),
                             None, None, None, 0, None, None, None, table, 3)
    assert l.b200_linear_shadow(C.byref(bad), stream()) != 0      # copies belong to the store and residual epilogues


def test_cross_rank_greedy_choice_one_gpu():
    """The merge of the vocabulary-split greedy choice on one GPU: as a group of one, and as rank 0 of two with the other
    rank's candidates and signal put in place by the host.  Ties between ranks go to the lower global index, NaN wins, and a
    row whose best value sits in the peer's slice takes the peer's index."""
    l = B.lib()
    rows, parts, slot_bytes, first = 6, 5, 4096, 1000
    rng = np.random.default_rng(3)
    values = rng.standard_normal((parts, rows)).astype(np.float32)
    indices = rng.permutation(parts * rows).reshape(parts, rows).astype(np.int32)
    values[2, 1] = values[:, 1].max() + 1          # row 1: this rank wins clearly
    values[:, 2] = -5.0                            # row 2: the peer will win
    values[3, 3] = 9.0                             # row 3: exact tie with the peer, whose global index is lower
    values[1, 4] = np.nan                          # row 4: NaN on this rank
    local_best = []
    for r in range(rows):
        order = sorted(range(parts), key=lambda t: (not np.isnan(values[t, r]), -values[t, r] if not np.isnan(values[t, r]) else 0, indices[t, r]))
        local_best.append((values[order[0], r], int(indices[order[0], r]) + first))
    vd, idd = dev(values), dev(indices)
    for world in (1, 2):
        regions, table = _tp_regions(world, slot_bytes)
        next_ids = torch.full((rows,), -1, dtype=torch.int64, device="cuda")
        ids = torch.zeros((rows,), dtype=torch.int64, device="cuda")
        history = torch.zeros((4, rows), dtype=torch.int64, device="cuda")
        counter = torch.zeros((2,), dtype=torch.int32, device="cuda")
        want = [index for _, index in local_best]
        if world == 2:
            area = 4096 + 2 * world * slot_bytes
            peer_values = np.array([-1.0, -100.0, 3.0, 9.0, 50.0, np.inf], dtype=np.float32)
            peer_index = np.array([7, 8, 9, 10, 11, 12], dtype=np.int32)
            packed = (peer_index.astype(np.uint32).astype(np.uint64) << np.uint64(32)) | peer_values.view(np.uint32).astype(np.uint64)
            regions[0][area + 1024 * 8: area + 1024 * 8 + rows * 8].view(torch.int64).copy_(torch.from_numpy(packed.view(np.int64)))
            regions[0][(34 + 1) * 4:(34 + 2) * 4].view(torch.int32)[0] = 1      # chosen[1] = call 1: the peer's candidates are in place
            want = [local_best[0][1] if local_best[0][0] > -1.0 else 7, want[1], 9, 10, want[4], 12]
        torch.cuda.synchronize()
        B.kcheck(l.b200_tp_argmax_finish(table, 0, world, slot_bytes, first, vd.data_ptr(), idd.data_ptr(), parts, rows, next_ids.data_ptr(),
                                         ids.data_ptr(), history.data_ptr(), 4, counter.data_ptr(), None, 0, stream()))
        sync()
        status = C.c_int32()
        B.kcheck(l.b200_take_device_status(0, stream(), C.byref(status)))
        assert status.value == 0
        assert next_ids.cpu().tolist() == want, (world, next_ids.cpu().tolist(), want)
        assert ids.cpu().tolist() == want and history[0].cpu().tolist() == want and int(counter[0]) == 1
        assert regions[0][50 * 4:51 * 4].view(torch.int32).item() == 1              # the owner's exchange counter
        if world == 2:
            assert regions[1][34 * 4:35 * 4].view(torch.int32).item() == 1          # the signal sent to the peer
            sent = regions[1][4096 + 2 * world * slot_bytes: 4096 + 2 * world * slot_bytes + rows * 8].view(torch.int64).cpu().numpy().view(np.uint64)
            assert [int(v >> np.uint64(32)) for v in sent] == [index for _, index in local_best]
