"""ctypes access to the CPU checkers.  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Two libraries expose the same function set (prefix ``oracle_`` / ``ref_``):

* ``liboracle.so``        -- the plain-C restatement in ``decoder_oracle.c`` ("port"),
* ``_ref/libref_harness.so`` -- the unmodified reference CPU library behind ``ref_harness.cpp`` ("reference").

Only tests, the smoke check and the CPU-baseline leg of the benchmark import this package; the shipped
library never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_PATH = os.path.join(HERE, "liboracle.so")
REF_PATH = os.path.join(HERE, "_ref", "libref_harness.so")

F32, BF16 = 0, 5


class Config(C.Structure):
    _fields_ = [
        ("vocab", C.c_int64), ("d_model", C.c_int64), ("layers", C.c_int64), ("heads", C.c_int64),
        ("kv_heads", C.c_int64), ("hidden", C.c_int64), ("context", C.c_int64),
        ("weight_dtype", C.c_int32), ("tied", C.c_int32),
        ("eps", C.c_double), ("rope_base", C.c_double),
        ("lora_rank", C.c_int64), ("lora_alpha", C.c_double),
    ]


def build(ref: bool = True) -> None:
    """Compile the port and, when the reference tree is present, the reference harness."""
    subprocess.run(["make", "-s", "port"], cwd=HERE, check=True)
    reference = os.environ.get("CTORCH_REFERENCE", "/root/reference")
    if ref and os.path.isdir(reference):
        subprocess.run(["make", "-s", "-j8", "ref", "REF=" + reference], cwd=HERE, check=True)


def have_ref() -> bool:
    return os.path.exists(REF_PATH)


def _ptr(array: np.ndarray, ctype=C.c_float):
    return array.ctypes.data_as(C.POINTER(ctype))


class CpuLib:
    """One of the two checker libraries, with argument types declared."""

    def __init__(self, kind: str = "port"):
        if kind == "port" and not os.path.exists(PORT_PATH):
            build(ref=False)
        self.kind = kind
        self.prefix = "oracle_" if kind == "port" else "ref_"
        self.lib = C.CDLL(PORT_PATH if kind == "port" else REF_PATH)
        f = self._fn
        fp, ip = C.POINTER(C.c_float), C.POINTER(C.c_int64)
        f("last_error", C.c_char_p, [])
        f("decoder_create", C.c_void_p, [C.POINTER(Config), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)])
        f("decoder_release", None, [C.c_void_p])
        f("cache_create", C.c_void_p, [C.c_void_p])
        f("cache_release", None, [C.c_void_p])
        f("cache_length", C.c_int64, [C.c_void_p])
        f("cache_clear", None, [C.c_void_p])
        f("cache_truncate", C.c_int, [C.c_void_p, C.c_int64])
        f("decoder_decode", C.c_int, [C.c_void_p, C.c_void_p, fp, C.c_int64, C.c_int64, fp])
        f("model_decode", C.c_int, [C.c_void_p, C.c_void_p, ip, C.c_int64, C.c_int64, fp])
        f("generate", C.c_int, [C.c_void_p, C.c_void_p, ip, C.c_int64, C.c_int64, C.c_int64, ip, fp])
        f("gqa_attention", C.c_int, [fp, fp, fp] + [C.c_int64] * 7 + [fp])
        f("rms_norm", None if kind == "port" else C.c_int, [fp, fp, C.c_int64, C.c_int64, C.c_double, fp])
        f("silu_mul", None if kind == "port" else C.c_int, [fp, fp, C.c_int64, fp])
        f("argmax", None if kind == "port" else C.c_int, [fp, C.c_int64, C.c_int64, ip])
        if kind == "port":
            f("rope_tables", None, [C.c_int64, C.c_int64, C.c_double, fp, fp])
            f("sample", None, [fp, C.c_int64, C.c_int64, C.c_double, C.POINTER(C.c_double), ip])
            f("linear", None, [fp, fp, C.c_int64, C.c_int64, C.c_int64, fp])
            f("rotary", None, [fp] + [C.c_int64] * 4 + [fp, fp, C.c_int64, fp])
            f("lora_linear", None, [fp, fp, fp, fp] + [C.c_int64] * 4 + [C.c_double, fp])
            f("lora_merge", None, [fp, fp, fp] + [C.c_int64] * 3 + [C.c_double, C.c_int32, fp])
            f("round_bf16", C.c_uint16, [C.c_float])
            f("decoder_cosine", fp, [C.c_void_p])
            f("decoder_sine", fp, [C.c_void_p])
        else:
            f("decoder_rope_tables", C.c_int, [C.c_void_p, fp, fp])
            f("decoder_state_names", C.c_int, [C.c_void_p, C.c_char_p, C.c_int64])
            f("cache_dtype", C.c_int, [C.c_void_p, C.c_int64])
            f("cache_copy", C.c_int, [C.c_void_p, C.c_int64, C.c_int32, fp])
            f("generate_threads", C.c_int, [C.c_void_p, ip] + [C.c_int64] * 4 + [ip])
            f("timed_decode", C.c_int, [C.c_void_p, ip] + [C.c_int64] * 6 + [C.POINTER(C.c_double)])
            f("linear", C.c_int, [fp, C.c_void_p, C.c_int32, C.c_int64, C.c_int64, C.c_int64, fp])
            f("rotary", C.c_int, [fp] + [C.c_int64] * 4 + [C.c_double, C.c_int64, C.c_int64, fp])
            f("lora_linear", C.c_int, [fp, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32] + [C.c_int64] * 4
              + [C.c_double, fp, C.c_void_p])
            f("sample", C.c_int, [fp, C.c_int64, C.c_int64, C.c_double, C.POINTER(C.c_double), ip])
            f("save_state", C.c_int, [C.c_void_p, C.c_char_p])
            f("save_onnx", C.c_int, [C.c_void_p, C.c_char_p, C.c_int])
            f("archive_size", C.c_int64, [C.c_char_p])
            f("archive_entry", C.c_int, [C.c_char_p, C.c_int64, C.c_char_p, C.c_int64, ip, ip, C.POINTER(C.c_int32), C.c_void_p, C.c_int64])

    def _fn(self, name, restype, argtypes):
        fn = getattr(self.lib, self.prefix + name)
        fn.restype, fn.argtypes = restype, argtypes
        setattr(self, name, fn)

    def error(self) -> str:
        return self.last_error().decode()

    def check(self, status: int) -> None:
        if status:
            raise RuntimeError(self.error())


_LIBS: dict[str, CpuLib] = {}


def lib(kind: str = "port") -> CpuLib:
    if kind not in _LIBS:
        _LIBS[kind] = CpuLib(kind)
    return _LIBS[kind]


def reference_archive(path: str) -> list[tuple[str, tuple[int, ...], int, bytes]]:
    """Entries (name, shape, dtype code, element bytes) of a weight archive as the reference's own dl::io::load reads it."""
    l = lib("ref")
    count = l.archive_size(path.encode())
    if count < 0:
        raise RuntimeError(l.error())
    entries = []
    for i in range(count):
        name = C.create_string_buffer(512)
        shape = (C.c_int64 * 8)()
        rank, dtype = C.c_int64(), C.c_int32()
        l.check(l.archive_entry(path.encode(), i, name, 512, shape, C.byref(rank), C.byref(dtype), None, 0))
        dims = tuple(shape[d] for d in range(rank.value))
        size = int(np.prod(dims, dtype=np.int64)) * (4, 8, 8, 1, 2, 2)[dtype.value]
        data = C.create_string_buffer(max(1, size))
        l.check(l.archive_entry(path.encode(), i, name, 512, shape, C.byref(rank), C.byref(dtype), data, size))
        entries.append((name.value.decode(), dims, dtype.value, data.raw[:size]))
    return entries


def make_config(spec: dict) -> Config:
    return Config(spec["vocab"], spec["d_model"], spec["layers"], spec["heads"], spec["kv_heads"], spec["hidden"],
                  spec["context"], BF16 if spec.get("dtype", "f32") == "bf16" else F32, int(spec.get("tied", True)),
                  spec.get("eps", 1e-5), spec.get("rope_base", 10000.0), spec.get("lora_rank", 0),
                  spec.get("lora_alpha", 1.0))


class CpuDecoder:
    """Decoder + caches on the CPU checker of the given kind.

    ``tensors`` is the ordered list documented at ``oracle_decoder_create`` (numpy float32, or uint16 bit
    patterns for bf16 models); ``lora`` the optional 4-per-layer adapter list (port only).
    """

    def __init__(self, spec: dict, tensors: list[np.ndarray], lora: list[np.ndarray] | None = None,
                 kind: str = "port"):
        self.l = lib(kind)
        self.spec = spec
        self.cfg = make_config(spec)
        self._keep = [np.ascontiguousarray(t) for t in tensors]
        table = (C.c_void_p * len(self._keep))(*[t.ctypes.data for t in self._keep])
        lora_table = None
        if lora:
            self._keep_lora = [np.ascontiguousarray(t) for t in lora]
            lora_table = (C.c_void_p * len(self._keep_lora))(*[t.ctypes.data for t in self._keep_lora])
        self.handle = self.l.decoder_create(C.byref(self.cfg), table, lora_table)
        if not self.handle:
            raise RuntimeError(self.l.error())
        self.cache = None

    def save_state(self, path: str) -> None:
        """Reference only: the model's weights written by the reference's dl::io::save."""
        self.l.check(self.l.save_state(self.handle, path.encode()))

    def save_onnx(self, path: str, with_head: bool) -> None:
        """Reference only: the decoder written by the reference's own ONNX exporter (dl::onnx::save_decoder)."""
        self.l.check(self.l.save_onnx(self.handle, path.encode(), int(with_head)))

    def close(self):
        if self.cache:
            self.l.cache_release(self.cache)
            self.cache = None
        if self.handle:
            self.l.decoder_release(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def new_cache(self):
        if self.cache:
            self.l.cache_release(self.cache)
        self.cache = self.l.cache_create(self.handle)
        return self.cache

    def cache_length(self) -> int:
        return self.l.cache_length(self.cache)

    def truncate(self, length: int) -> None:
        self.l.check(self.l.cache_truncate(self.cache, length))

    def clear(self) -> None:
        self.l.cache_clear(self.cache)

    def decode_features(self, x: np.ndarray) -> np.ndarray:
        if self.cache is None:
            self.new_cache()
        x = np.ascontiguousarray(x, dtype=np.float32)
        batch, length, _ = x.shape
        out = np.empty_like(x)
        self.l.check(self.l.decoder_decode(self.handle, self.cache, _ptr(x), batch, length, _ptr(out)))
        return out

    def decode_ids(self, ids: np.ndarray) -> np.ndarray:
        if self.cache is None:
            self.new_cache()
        ids = np.ascontiguousarray(ids, dtype=np.int64)
        batch, length = ids.shape
        logits = np.empty((batch, length, self.spec["vocab"]), dtype=np.float32)
        self.l.check(self.l.model_decode(self.handle, self.cache, _ptr(ids, C.c_int64), batch, length, _ptr(logits)))
        return logits

    def generate(self, prompt: np.ndarray, steps: int, want_logits: bool = True):
        self.new_cache()
        prompt = np.ascontiguousarray(prompt, dtype=np.int64)
        batch, plen = prompt.shape
        tokens = np.empty((batch, steps), dtype=np.int64)
        logits = np.empty((steps, batch, self.spec["vocab"]), dtype=np.float32) if want_logits else None
        self.l.check(self.l.generate(self.handle, self.cache, _ptr(prompt, C.c_int64), batch, plen, steps,
                                     _ptr(tokens, C.c_int64), _ptr(logits) if want_logits else None))
        return tokens, logits

    def generate_threads(self, prompt: np.ndarray, steps: int, threads: int) -> np.ndarray:
        """Reference library only: one worker thread per slice of the batch, own cache each."""
        prompt = np.ascontiguousarray(prompt, dtype=np.int64)
        batch, plen = prompt.shape
        tokens = np.empty((batch, steps), dtype=np.int64)
        self.l.check(self.l.generate_threads(self.handle, _ptr(prompt, C.c_int64), batch, plen, steps, threads,
                                             _ptr(tokens, C.c_int64)))
        return tokens


def timed_decode(model: "CpuDecoder", prompt: np.ndarray, warmup: int, steps: int, threads: int, cached: int = 0) -> float:
    """Seconds the CPU checker needs for `steps` greedy single-token steps of the whole batch after a prefill and
    `warmup` untimed steps, with the batch spread over `threads` workers (each with its own cache).  `cached` (reference
    build only) puts that many positions of pseudo-random K and V into every cache before the prompt, so that the steps
    attend over a long context without a CPU prefill of that length."""
    prompt = np.ascontiguousarray(prompt, dtype=np.int64)
    batch, plen = prompt.shape
    threads = max(1, min(threads, batch))
    if model.l.kind != "port":
        seconds = C.c_double()
        model.l.check(model.l.timed_decode(model.handle, _ptr(prompt, C.c_int64), batch, plen, warmup, steps, threads, cached,
                                           C.byref(seconds)))
        return seconds.value
    if cached:
        raise ValueError("the plain-C restatement has no cache pre-fill; pass cached=0")
    # port: ctypes releases the GIL during calls, so Python threads run the C code in parallel
    import threading
    import time
    share = (batch + threads - 1) // threads
    start, finish = threading.Barrier(threads + 1), threading.Barrier(threads + 1)
    errors = []

    def worker(t):
        rows = prompt[t * share:(t + 1) * share]
        count = rows.shape[0]
        cache = model.l.cache_create(model.handle)
        vocab = model.spec["vocab"]
        logits = np.empty((count, plen, vocab), dtype=np.float32)
        one = np.empty((count, 1, vocab), dtype=np.float32)
        try:
            if count:
                model.l.check(model.l.model_decode(model.handle, cache, _ptr(rows, C.c_int64), count, plen, _ptr(logits)))
                nxt = argmax(logits[:, -1])
                for _ in range(warmup):
                    model.l.check(model.l.model_decode(model.handle, cache, _ptr(nxt, C.c_int64), count, 1, _ptr(one)))
                    nxt = argmax(one[:, 0])
            start.wait()
            for _ in range(steps if count else 0):
                model.l.check(model.l.model_decode(model.handle, cache, _ptr(nxt, C.c_int64), count, 1, _ptr(one)))
                nxt = argmax(one[:, 0])
        except Exception as error:  # noqa: BLE001
            errors.append(error)
            start.abort()
        finally:
            try:
                finish.wait()
            except threading.BrokenBarrierError:
                pass
            model.l.cache_release(cache)

    pool = [threading.Thread(target=worker, args=(t,)) for t in range(threads)]
    for t in pool:
        t.start()
    start.wait()
    begin = time.perf_counter()
    finish.wait()
    elapsed = time.perf_counter() - begin
    for t in pool:
        t.join()
    if errors:
        raise errors[0]
    return elapsed


def gqa_attention(q, k, v, causal_offset: int = -1, kind: str = "port") -> np.ndarray:
    """q [B,Hq,L,hd], k/v [B,Hkv,S,hd] float32 -> [B,Hq,L,hd]."""
    l = lib(kind)
    q, k, v = (np.ascontiguousarray(a, dtype=np.float32) for a in (q, k, v))
    out = np.empty_like(q)
    l.check(l.gqa_attention(_ptr(q), _ptr(k), _ptr(v), q.shape[0], q.shape[1], k.shape[1], q.shape[2], k.shape[2],
                            q.shape[3], causal_offset, _ptr(out)))
    return out


def rms_norm(x, weight, eps: float, kind: str = "port") -> np.ndarray:
    l = lib(kind)
    x = np.ascontiguousarray(x, dtype=np.float32)
    weight = np.ascontiguousarray(weight, dtype=np.float32)
    y = np.empty_like(x)
    status = l.rms_norm(_ptr(x), _ptr(weight), x.size // x.shape[-1], x.shape[-1], eps, _ptr(y))
    if kind != "port":
        l.check(status)
    return y


def silu_mul(gate, up, kind: str = "port") -> np.ndarray:
    l = lib(kind)
    gate = np.ascontiguousarray(gate, dtype=np.float32)
    up = np.ascontiguousarray(up, dtype=np.float32)
    y = np.empty_like(gate)
    status = l.silu_mul(_ptr(gate), _ptr(up), gate.size, _ptr(y))
    if kind != "port":
        l.check(status)
    return y


def argmax(x, kind: str = "port") -> np.ndarray:
    l = lib(kind)
    x = np.ascontiguousarray(x, dtype=np.float32)
    index = np.empty(x.shape[:-1], dtype=np.int64)
    status = l.argmax(_ptr(x), x.size // x.shape[-1], x.shape[-1], _ptr(index, C.c_int64))
    if kind != "port":
        l.check(status)
    return index


def sample(x, temperature: float, uniforms, kind: str = "port") -> np.ndarray:
    """One index per row drawn from softmax(x / temperature) with the given uniform variates (multiples of 2**-53 for
    the reference, whose std::discrete_distribution is fed through a fixed-output generator)."""
    l = lib(kind)
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = np.ascontiguousarray(uniforms, dtype=np.float64)
    index = np.empty(x.shape[0], dtype=np.int64)
    status = l.sample(_ptr(x), x.shape[0], x.shape[1], float(temperature), _ptr(u, C.c_double), _ptr(index, C.c_int64))
    if kind != "port":
        l.check(status)
    return index


def widen_bf16(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def linear(x, w, kind: str = "port") -> np.ndarray:
    """x [rows,in] float32; w [out,in] float32 or uint16 (bf16 bit patterns) -> [rows,out] float32."""
    l = lib(kind)
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w)
    rows, inner = x.shape
    out = w.shape[0]
    y = np.empty((rows, out), dtype=np.float32)
    if kind == "port":
        wf = widen_bf16(w) if w.dtype == np.uint16 else w.astype(np.float32, copy=False)
        wf = np.ascontiguousarray(wf)
        l.linear(_ptr(x), _ptr(wf), rows, inner, out, _ptr(y))
    else:
        l.check(l.linear(_ptr(x), w.ctypes.data, BF16 if w.dtype == np.uint16 else F32, rows, inner, out, _ptr(y)))
    return y


def rotary(x, base: float, capacity: int, offset: int, kind: str = "port") -> np.ndarray:
    """x [B,H,L,hd] float32 -> rotated, positions offset..offset+L-1."""
    l = lib(kind)
    x = np.ascontiguousarray(x, dtype=np.float32)
    b, h, length, hd = x.shape
    y = np.empty_like(x)
    if kind == "port":
        cos = np.empty((capacity, hd // 2), dtype=np.float32)
        sin = np.empty_like(cos)
        l.rope_tables(hd, capacity, base, _ptr(cos), _ptr(sin))
        l.rotary(_ptr(x), b, h, length, hd, _ptr(cos), _ptr(sin), offset, _ptr(y))
    else:
        l.check(l.rotary(_ptr(x), b, h, length, hd, base, capacity, offset, _ptr(y)))
    return y


def rope_tables(head_dim: int, capacity: int, base: float = 10000.0):
    l = lib("port")
    cos = np.empty((capacity, head_dim // 2), dtype=np.float32)
    sin = np.empty_like(cos)
    l.rope_tables(head_dim, capacity, base, _ptr(cos), _ptr(sin))
    return cos, sin


def lora_linear(x, w, down, up, rank: int, alpha: float, kind: str = "port"):
    """Returns (y, merged weight).  w/down/up float32 or uint16 bf16 bit patterns (all the same dtype)."""
    l = lib(kind)
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, inner = x.shape
    out = w.shape[0]
    y = np.empty((rows, out), dtype=np.float32)
    is_bf16 = w.dtype == np.uint16
    if kind == "port":
        wf, df, uf = (np.ascontiguousarray(widen_bf16(a) if is_bf16 else a.astype(np.float32)) for a in (w, down, up))
        l.lora_linear(_ptr(x), _ptr(wf), _ptr(df), _ptr(uf), rows, inner, out, rank, alpha, _ptr(y))
        merged = np.empty((out, inner), dtype=np.float32)
        l.lora_merge(_ptr(wf), _ptr(df), _ptr(uf), inner, out, rank, alpha, int(is_bf16), _ptr(merged))
        return y, merged
    w, down, up = (np.ascontiguousarray(a) for a in (w, down, up))
    merged = np.empty((out, inner), dtype=w.dtype)
    l.check(l.lora_linear(_ptr(x), w.ctypes.data, down.ctypes.data, up.ctypes.data, BF16 if is_bf16 else F32,
                          rows, inner, out, rank, alpha, _ptr(y), merged.ctypes.data))
    return y, (widen_bf16(merged) if is_bf16 else merged)
