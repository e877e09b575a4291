"""Python access to libctorch_b200.so: ctypes declarations of the C ABI plus a thin object layer for tests and
the benchmark.  The library is the product; this module only forwards calls.  Importing it never falls back to
another implementation: a missing library or a failing call raises."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libctorch_b200.so")

F32, F64, I64, BOOL, F16, BF16 = 0, 1, 2, 3, 4, 5
CPU, CUDA = 0, 1
_NP_OF = {F32: np.float32, F64: np.float64, I64: np.int64, BOOL: np.bool_, BF16: np.uint16}
_CODE_OF = {np.dtype(np.float32): F32, np.dtype(np.float64): F64, np.dtype(np.int64): I64, np.dtype(np.bool_): BOOL,
            np.dtype(np.uint16): BF16}


class Device(C.Structure):
    _fields_ = [("type", C.c_int), ("index", C.c_int32)]


class Shape(C.Structure):
    _fields_ = [("data", C.POINTER(C.c_int64)), ("size", C.c_size_t)]


class TensorOptions(C.Structure):
    _fields_ = [("dtype", C.c_int), ("device", Device), ("requires_grad", C.c_int32)]


class TensorInfo(C.Structure):
    _fields_ = [("dtype", C.c_int), ("device", Device), ("numel", C.c_int64), ("contiguous", C.c_int32),
                ("requires_grad", C.c_int32), ("leaf", C.c_int32)]


class QkvArgs(C.Structure):
    _fields_ = [("heads", C.c_int32), ("kv_heads", C.c_int32), ("head_dim", C.c_int32), ("tokens_per_sequence", C.c_int32),
                ("cosine", C.c_void_p), ("sine", C.c_void_p), ("context", C.c_int32), ("cache", C.c_void_p),
                ("q_out", C.c_void_p), ("lora_rank", C.c_int32), ("lora_scale", C.c_float), ("low", C.c_void_p),
                ("q_up", C.c_void_p), ("v_up", C.c_void_p)]


class ShadowLinearArgs(C.Structure):
    _fields_ = [("x_hi", C.c_void_p), ("x_lo", C.c_void_p), ("rows", C.c_int64), ("inner", C.c_int64), ("weight", C.c_void_p),
                ("out", C.c_int64), ("sumsq_in", C.c_void_p), ("parts_in", C.c_int32), ("eps", C.c_double), ("epilogue", C.c_int),
                ("residual", C.c_void_p), ("qkv", C.POINTER(QkvArgs)), ("y", C.c_void_p), ("out_hi", C.c_void_p),
                ("out_lo", C.c_void_p), ("out_norm_weight", C.c_void_p), ("out_norm_dtype", C.c_int32), ("sumsq_out", C.c_void_p),
                ("best_value", C.c_void_p), ("best_index", C.c_void_p), ("y_copies", C.POINTER(C.c_void_p)), ("copies", C.c_int32)]


class B200Error(RuntimeError):
    pass


_lib = None


def lib() -> C.CDLL:
    """The shared library, loaded once.  Raises if it has not been built (python -m ctorch_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise B200Error(f"{LIB_PATH} is missing: build it with `python -m ctorch_b200.build`")
        _lib = C.CDLL(LIB_PATH)
        _declare(_lib)
    return _lib


def _declare(l: C.CDLL) -> None:
    vp, i64, i32, sz = C.c_void_p, C.c_int64, C.c_int32, C.c_size_t
    pp = C.POINTER(vp)
    sig = {
        "dl_version": (C.c_char_p, []), "dl_last_error": (C.c_char_p, []),
        "dl_default_tensor_options": (TensorOptions, []),
        "dl_tensor_release": (None, [vp]), "dl_tensor_retain": (C.c_int, [vp, pp]),
        "dl_tensor_get_info": (TensorInfo, [vp]), "dl_tensor_shape": (Shape, [vp]), "dl_tensor_strides": (Shape, [vp]),
        "dl_tensor_data": (vp, [vp]), "dl_tensor_nbytes": (sz, [vp]), "dl_tensor_copy_to_host": (C.c_int, [vp, vp]),
        "dl_from_host": (C.c_int, [vp, Shape, TensorOptions, pp]), "dl_full": (C.c_int, [Shape, C.c_double, TensorOptions, pp]),
        "dl_zeros": (C.c_int, [Shape, TensorOptions, pp]), "dl_ones": (C.c_int, [Shape, TensorOptions, pp]),
        "dl_clone": (C.c_int, [vp, pp]), "dl_astype": (C.c_int, [vp, C.c_int, pp]), "dl_to": (C.c_int, [vp, Device, pp]),
        "dl_reshape": (C.c_int, [vp, Shape, pp]), "dl_select": (C.c_int, [vp, i64, i64, pp]),
        "dl_narrow": (C.c_int, [vp, i64, i64, i64, pp]),
        "dl_argmax": (C.c_int, [vp, i64, i32, pp]), "dl_linear": (C.c_int, [vp, vp, vp, pp]),
        "dl_embedding": (C.c_int, [vp, vp, pp]), "dl_rms_norm": (C.c_int, [vp, Shape, vp, C.POINTER(C.c_double), pp]),
        "dl_synchronize": (C.c_int, [Device]),
        "dl_tensordot": (C.c_int, [vp, vp, Shape, Shape, pp]),
        "dl_rotary_embedding": (C.c_int, [vp, vp, vp, pp]), "dl_grouped_query_attention": (C.c_int, [vp, vp, vp, vp, pp]),
        "dl_module_release": (None, [vp]), "dl_module_retain": (C.c_int, [vp, pp]),
        "dl_linear_create": (C.c_int, [i64, i64, i32, TensorOptions, pp]), "dl_linear_from_tensors": (C.c_int, [vp, vp, pp]),
        "dl_embedding_create": (C.c_int, [i64, i64, TensorOptions, pp]), "dl_embedding_from_tensor": (C.c_int, [vp, pp]),
        "dl_rms_norm_create": (C.c_int, [Shape, C.POINTER(C.c_double), i32, TensorOptions, pp]),
        "dl_module_forward": (C.c_int, [vp, vp, pp]), "dl_module_train": (C.c_int, [vp, i32]),
        "dl_module_is_training": (i32, [vp]), "dl_module_to": (C.c_int, [vp, Device]),
        "dl_module_state": (C.c_int, [vp, pp]), "dl_module_load_state": (C.c_int, [vp, vp]),
        "dl_state_release": (None, [vp]), "dl_state_size": (sz, [vp]), "dl_state_name": (C.c_char_p, [vp, sz]),
        "dl_state_tensor": (C.c_int, [vp, sz, pp]),
        "dl_state_create": (C.c_int, [C.POINTER(C.c_char_p), pp, sz, pp]),
        "dl_state_save": (C.c_int, [C.c_char_p, vp]), "dl_state_load": (C.c_int, [C.c_char_p, pp]),
        "dl_swiglu_create": (C.c_int, [i64, i64, i32, TensorOptions, pp]),
        "dl_lora_linear_create": (C.c_int, [vp, i64, C.c_double, pp]), "dl_lora_linear_merge": (C.c_int, [vp, pp]),
        "dl_rotary_embedding_create": (C.c_int, [i64, i64, C.c_double, TensorOptions, pp]),
        "dl_rotary_embedding_forward": (C.c_int, [vp, vp, i64, pp]),
        "dl_grouped_query_attention_create": (C.c_int, [i64, i64, i64, i64, TensorOptions, pp]),
        "dl_transformer_decoder_create": (C.c_int, [i64, i64, i64, i64, i64, i64, TensorOptions, pp]),
        "dl_decoder_cache_create": (C.c_int, [vp, pp]), "dl_decoder_cache_release": (None, [vp]),
        "dl_decoder_cache_clear": (C.c_int, [vp]), "dl_decoder_cache_truncate": (C.c_int, [vp, i64]),
        "dl_decoder_cache_length": (C.c_int, [vp, C.POINTER(i64)]),
        "dl_transformer_decoder_decode": (C.c_int, [vp, vp, vp, pp]),
        "dl_transformer_decoder_set_cache_dtype": (C.c_int, [vp, C.c_int]),
        "dl_transformer_decoder_set_activation_dtype": (C.c_int, [vp, C.c_int]),
        "dl_transformer_decoder_set_adapters": (C.c_int, [vp, i64, vp, vp]),
        "dl_generation_create": (C.c_int, [vp, vp, vp, vp, i64, i64, pp]), "dl_generation_release": (None, [vp]),
        "dl_generation_prefill": (C.c_int, [vp, vp]), "dl_generation_step": (C.c_int, [vp, i64]),
        "dl_generation_step_host": (C.c_int, [vp, C.POINTER(i64), C.POINTER(i64)]),
        "dl_generation_run_host": (C.c_int, [vp, C.POINTER(i64), i64, C.POINTER(i64)]),
        "dl_generation_tokens": (C.c_int, [vp, pp]), "dl_generation_logits": (C.c_int, [vp, pp]),
        "dl_generation_launches_per_step": (i64, [vp]),
        "dl_b200_shadow_partial_rows": (i64, [i64, i64]),
        "dl_onnx_save_decoder": (C.c_int, [C.c_char_p, vp, vp, vp]),
        "dl_decoder_generate": (C.c_int, [vp, vp, vp, vp, i64, vp, pp]),
        "dl_generation_profile_step": (C.c_int, [vp, C.POINTER(C.c_double)]),
        "dl_b200_tp_unique_id": (C.c_int, [vp]), "dl_b200_tp_init": (C.c_int, [Device, i32, i32, vp]),
        "dl_b200_tp_finalize": (C.c_int, [Device]), "dl_b200_tp_set_push": (C.c_int, [Device, i32]),
        "dl_b200_tp_symmetric_handle": (C.c_int, [Device, sz, vp]), "dl_b200_tp_symmetric_open": (C.c_int, [Device, vp, i32]), "dl_transformer_decoder_set_tensor_parallel": (C.c_int, [vp, i32, i32]),
        "dl_b200_timer_start": (C.c_int, [Device]), "dl_b200_timer_stop": (C.c_int, [Device, C.POINTER(C.c_double)]),
        "dl_b200_stream": (vp, [Device]),
        # kernel-level ABI
        "b200_last_error": (C.c_char_p, []),
        "b200_kv_cache_create": (C.c_int, [i32, i32, i32, i32, i32, i32, i32, pp]), "b200_kv_cache_release": (None, [vp]),
        "b200_kv_cache_set_lengths": (C.c_int, [vp, C.POINTER(i32), vp]), "b200_kv_cache_fill_lengths": (C.c_int, [vp, i32, vp]),
        "b200_kv_cache_set_page_table": (C.c_int, [vp, C.POINTER(i32), vp]),
        "b200_kv_cache_lengths": (vp, [vp]), "b200_kv_cache_page_table": (vp, [vp]), "b200_kv_cache_pool": (vp, [vp, i32]),
        "b200_kv_cache_pages_per_sequence": (i32, [vp]), "b200_kv_cache_page_size": (i32, [vp]),
        "b200_kv_cache_pool_bytes": (sz, [vp]), "b200_kv_cache_advance": (C.c_int, [pp, i32, i32, vp]),
        "b200_kv_cache_gather": (C.c_int, [vp, i32, i32, vp, vp]), "b200_kv_cache_append": (C.c_int, [vp, vp, vp, i32, vp]),
        "b200_permute": (C.c_int, [vp, C.POINTER(i64), C.POINTER(i64), i32, vp, vp]),
        "b200_embedding": (C.c_int, [vp, i32, vp, i64, i64, i64, vp, vp]),
        "b200_rms_norm": (C.c_int, [vp, vp, i32, i64, i64, C.c_double, vp, vp]),
        "b200_linear": (C.c_int, [vp, i64, i64, vp, i32, i64, vp, i32, C.c_double, C.c_int, vp, C.POINTER(QkvArgs), vp, vp]),
        "b200_attention_scratch_bytes": (sz, [i64, i32, i32, i32, i32, i32]),
        "b200_attention_decode": (C.c_int, [vp, i64, i32, i32, vp, i32, i32, vp, sz, vp, vp]),
        "b200_attention_decode_static": (C.c_int, [vp, i64, i32, i32, vp, i32, i32, vp, vp]),
        "b200_linear_shadow": (C.c_int, [C.POINTER(ShadowLinearArgs), vp]),
        "b200_linear_shadow_parts": (i32, [i64, i64, i64]),
        "b200_embedding_shadow": (C.c_int, [vp, i32, vp, i64, i64, i64, vp, i32, vp, vp, vp, vp, vp]),
        "b200_shadow_from_rows": (C.c_int, [vp, i64, i64, vp, i32, vp, vp, vp, vp]),
        "b200_attention_decode_shadow": (C.c_int, [vp, i64, i32, i32, vp, i32, i32, vp, sz, vp, vp, vp]),
        "b200_argmax": (C.c_int, [vp, i64, i64, vp, vp]), "b200_select_rows": (C.c_int, [vp, i64, i64, i64, i64, vp, vp]),
        "b200_rotary": (C.c_int, [vp, i64, i64, i64, vp, vp, vp, vp]),
        "b200_permute_0213": (C.c_int, [vp, i64, i64, i64, i64, vp, vp]),
        "b200_token_feedback": (C.c_int, [vp, i64, vp, vp, i64, vp, vp]),
        "b200_sample": (C.c_int, [vp, i64, i64, C.c_double, vp, vp, vp]),
        "dl_generation_step_sampled": (C.c_int, [vp, C.c_double, vp, vp]),
        "b200_linear_argmax_parts": (i32, [i64, i64, i64]),
        "b200_linear_shadow_kernel": (C.c_char_p, [i64, i64, i64]),
        "b200_linear_decode_launch_shape": (i32, [i64, i64, i64, i32, C.POINTER(i32)]),
        "b200_tp_argmax_finish": (C.c_int, [pp, i32, i32, sz, i32, vp, vp, i32, i64, vp, vp, vp, i64, vp, pp, i32, vp]),
        "b200_tp_reduce_parts": (i32, [i64]), "b200_tp_region_bytes": (sz, [sz, i32]), "b200_tp_slot": (vp, [vp, sz, i32, i32, i32]),
        "b200_tp_reduce_shadow": (C.c_int, [pp, i32, i32, i32, sz, i32, i64, i64, vp, i32, vp, vp, vp, vp, vp]),
        "b200_argmax_finish": (C.c_int, [vp, vp, i32, i64, vp, vp, vp, i64, vp, pp, i32, vp]),
        "b200_scaled_add": (C.c_int, [vp, vp, C.c_float, i64, vp]),
        "b200_take_device_status": (C.c_int, [i32, vp, C.POINTER(i32)]),
    }
    for name, (restype, argtypes) in sig.items():
        fn = getattr(l, name)
        fn.restype, fn.argtypes = restype, argtypes


def check(status: int) -> None:
    if status != 0:
        raise B200Error(lib().dl_last_error().decode() or "DL_ERROR")


def kcheck(status: int) -> None:
    if status != 0:
        raise B200Error(f"b200 status {status}: {lib().b200_last_error().decode()}")


def _shape(dims) -> tuple[Shape, object]:
    arr = (C.c_int64 * max(1, len(dims)))(*dims)
    return Shape(C.cast(arr, C.POINTER(C.c_int64)), len(dims)), arr


def cuda(index: int = 0) -> Device:
    return Device(CUDA, index)


def cpu() -> Device:
    return Device(CPU, 0)


class Tensor:
    """Owning wrapper of a dl_tensor handle."""

    def __init__(self, handle):
        self.h = C.c_void_p(handle) if not isinstance(handle, C.c_void_p) else handle

    def __del__(self):
        try:
            if self.h:
                lib().dl_tensor_release(self.h)
                self.h = None
        except Exception:
            pass

    @staticmethod
    def from_numpy(array: np.ndarray, device: Device | None = None, dtype: int | None = None) -> "Tensor":
        array = np.ascontiguousarray(array)
        code = dtype if dtype is not None else _CODE_OF[array.dtype]
        shape, keep = _shape(array.shape)
        out = C.c_void_p()
        check(lib().dl_from_host(array.ctypes.data, shape, TensorOptions(code, device or cpu(), 0), C.byref(out)))
        return Tensor(out)

    @property
    def shape(self) -> tuple[int, ...]:
        s = lib().dl_tensor_shape(self.h)
        return tuple(s.data[i] for i in range(s.size))

    @property
    def dtype(self) -> int:
        return lib().dl_tensor_get_info(self.h).dtype

    @property
    def device(self) -> Device:
        return lib().dl_tensor_get_info(self.h).device

    @property
    def data_ptr(self) -> int:
        return lib().dl_tensor_data(self.h) or 0

    def numpy(self) -> np.ndarray:
        out = np.empty(self.shape, dtype=_NP_OF[self.dtype])
        check(lib().dl_tensor_copy_to_host(self.h, out.ctypes.data))
        return out

    def to(self, device: Device) -> "Tensor":
        out = C.c_void_p()
        check(lib().dl_to(self.h, device, C.byref(out)))
        return Tensor(out)

    def select(self, axis: int, index: int) -> "Tensor":
        out = C.c_void_p()
        check(lib().dl_select(self.h, axis, index, C.byref(out)))
        return Tensor(out)

    def narrow(self, axis: int, start: int, length: int) -> "Tensor":
        out = C.c_void_p()
        check(lib().dl_narrow(self.h, axis, start, length, C.byref(out)))
        return Tensor(out)


class Module:
    def __init__(self, handle):
        self.h = handle if isinstance(handle, C.c_void_p) else C.c_void_p(handle)

    def __del__(self):
        try:
            if self.h:
                lib().dl_module_release(self.h)
                self.h = None
        except Exception:
            pass

    def __call__(self, x: Tensor) -> Tensor:
        out = C.c_void_p()
        check(lib().dl_module_forward(self.h, x.h, C.byref(out)))
        return Tensor(out)

    def to(self, device: Device) -> "Module":
        check(lib().dl_module_to(self.h, device))
        return self

    def state_names(self) -> list[str]:
        state = C.c_void_p()
        check(lib().dl_module_state(self.h, C.byref(state)))
        names = [lib().dl_state_name(state, i).decode() for i in range(lib().dl_state_size(state))]
        lib().dl_state_release(state)
        return names

    def state(self) -> dict[str, Tensor]:
        state = C.c_void_p()
        check(lib().dl_module_state(self.h, C.byref(state)))
        out = {}
        for i in range(lib().dl_state_size(state)):
            t = C.c_void_p()
            check(lib().dl_state_tensor(state, i, C.byref(t)))
            out[lib().dl_state_name(state, i).decode()] = Tensor(t)
        lib().dl_state_release(state)
        return out

    def load_state(self, named: dict[str, Tensor]) -> None:
        names = (C.c_char_p * len(named))(*[n.encode() for n in named])
        handles = (C.c_void_p * len(named))(*[t.h for t in named.values()])
        state = C.c_void_p()
        check(lib().dl_state_create(names, handles, len(named), C.byref(state)))
        try:
            check(lib().dl_module_load_state(self.h, state))
        finally:
            lib().dl_state_release(state)


def load_archive(path: str) -> dict[str, Tensor]:
    """Entries of a weight archive (".ct", the reference's dl::io::save layout) as host tensors, in file order."""
    state = C.c_void_p()
    check(lib().dl_state_load(os.fspath(path).encode(), C.byref(state)))
    out = {}
    try:
        for i in range(lib().dl_state_size(state)):
            t = C.c_void_p()
            check(lib().dl_state_tensor(state, i, C.byref(t)))
            out[lib().dl_state_name(state, i).decode()] = Tensor(t)
    finally:
        lib().dl_state_release(state)
    return out


def save_archive(path: str, named: dict[str, Tensor]) -> None:
    names = (C.c_char_p * len(named))(*[n.encode() for n in named])
    handles = (C.c_void_p * len(named))(*[t.h for t in named.values()])
    state = C.c_void_p()
    check(lib().dl_state_create(names, handles, len(named), C.byref(state)))
    try:
        check(lib().dl_state_save(os.fspath(path).encode(), state))
    finally:
        lib().dl_state_release(state)


def options(dtype: int = F32, device: Device | None = None) -> TensorOptions:
    return TensorOptions(dtype, device or cpu(), 0)


class DecoderModel:
    """Embedding + TransformerDecoder + output Linear, the arrangement of the reference's ByteDecoder example, built
    through the C ABI from the canonical ordered tensor list (see ctorch_b200.workloads.tensor_shapes)."""

    def __init__(self, spec: dict, tensors: list[np.ndarray], lora: list[np.ndarray] | None = None, device: int | None = 0,
                 cache_dtype: str | None = None, tensor_parallel: tuple[int, int] | None = None,
                 activation_dtype: str | None = None):
        """`device=None` keeps the modules on the host: enough for state handling and the ONNX export, not for compute."""
        l = lib()
        self.spec = spec
        self.dev = cuda(device) if device is not None else cpu()
        code = BF16 if spec["dtype"] == "bf16" else F32
        D, hd = spec["d_model"], spec["d_model"] // spec["heads"]
        dec = C.c_void_p()
        check(l.dl_transformer_decoder_create(spec["layers"], D, spec["heads"], spec["kv_heads"], spec["hidden"],
                                              spec["context"], options(code, cpu()), C.byref(dec)))
        self.decoder = Module(dec)
        # load weights by state name; rotary buffers keep the values the library computed
        state = self.decoder.state()
        names = [n for n in state if "rotary" not in n]
        order = []
        for i in range(spec["layers"]):
            p = f"layer{i}."
            order += [p + "attention.query.weight", p + "attention.key.weight", p + "attention.value.weight",
                      p + "attention.output.weight", p + "feedforward.gate.weight", p + "feedforward.up.weight",
                      p + "feedforward.down.weight", p + "attention_norm.weight", p + "feedforward_norm.weight"]
        order.append("normalization.weight")
        assert sorted(order) == sorted(names), (sorted(set(order) ^ set(names)))
        for name, array in zip(order, tensors[1:1 + len(order)]):
            state[name] = Tensor.from_numpy(array, dtype=code)
        self.decoder.load_state(state)
        if device is not None:
            self.decoder.to(self.dev)
        if activation_dtype is not None:
            check(l.dl_transformer_decoder_set_activation_dtype(self.decoder.h, BF16 if activation_dtype == "bf16" else F32))
        if cache_dtype is not None:
            check(l.dl_transformer_decoder_set_cache_dtype(self.decoder.h, BF16 if cache_dtype == "bf16" else F32))
        table = Tensor.from_numpy(tensors[0], device=self.dev, dtype=code)
        emb = C.c_void_p()
        check(l.dl_embedding_from_tensor(table.h, C.byref(emb)))
        self.embedding = Module(emb)
        out_weight = table if spec.get("tied", True) else Tensor.from_numpy(tensors[-1], device=self.dev, dtype=code)
        out = C.c_void_p()
        check(l.dl_linear_from_tensors(out_weight.h, None, C.byref(out)))
        self.output = Module(out)
        if lora:
            self._adapters = []
            kvw = spec["kv_heads"] * hd
            for i in range(spec["layers"]):
                pair = []
                for j, (rows, which) in enumerate([(D, "query"), (kvw, "value")]):
                    base_w = Tensor.from_numpy(tensors[1 + 9 * i + (0 if j == 0 else 2)], device=self.dev, dtype=code)
                    base = C.c_void_p()
                    check(l.dl_linear_from_tensors(base_w.h, None, C.byref(base)))
                    base = Module(base)
                    adapter = C.c_void_p()
                    check(l.dl_lora_linear_create(base.h, spec["lora_rank"], spec["lora_alpha"], C.byref(adapter)))
                    adapter = Module(adapter)
                    st = adapter.state()
                    st["down.weight"] = Tensor.from_numpy(lora[4 * i + 2 * j], dtype=code)
                    st["up.weight"] = Tensor.from_numpy(lora[4 * i + 2 * j + 1], dtype=code)
                    adapter.load_state(st)
                    pair.append(adapter)
                check(l.dl_transformer_decoder_set_adapters(self.decoder.h, i, pair[0].h, pair[1].h))
                self._adapters.append(pair)
        if tensor_parallel is not None:
            check(l.dl_transformer_decoder_set_tensor_parallel(self.decoder.h, tensor_parallel[0], tensor_parallel[1]))
        self.cache = None
        self.new_cache()

    def save_onnx(self, path: str, with_head: bool = True) -> None:
        """The decoder as an ONNX file with its KV cache as graph ports: input_ids -> logits with the embedding and output
        layers, features -> hidden states without them."""
        check(lib().dl_onnx_save_decoder(os.fsencode(path), self.decoder.h, self.embedding.h if with_head else None,
                                         self.output.h if with_head else None))

    def load_archive_state(self, state: dict[str, Tensor]) -> None:
        """Weights from an archive of the reference's example model: "tokens.weight" (shared with the output projection
        when tied, "output.weight" otherwise) and the decoder's own state under "decoder."."""
        self.decoder.load_state({n[len("decoder."):]: t for n, t in state.items() if n.startswith("decoder.")})
        self.embedding.load_state({"weight": state["tokens.weight"]})
        if not self.spec.get("tied", True):
            self.output.load_state({"weight": state["output.weight"]})

    def new_cache(self):
        self.release_cache()
        cache = C.c_void_p()
        check(lib().dl_decoder_cache_create(self.decoder.h, C.byref(cache)))
        self.cache = cache

    def release_cache(self):
        if getattr(self, "cache", None):
            lib().dl_decoder_cache_release(self.cache)
            self.cache = None

    def __del__(self):
        try:
            self.release_cache()
        except Exception:
            pass

    def cache_length(self) -> int:
        n = C.c_int64()
        check(lib().dl_decoder_cache_length(self.cache, C.byref(n)))
        return n.value

    def truncate(self, length: int) -> None:
        check(lib().dl_decoder_cache_truncate(self.cache, length))

    def clear(self) -> None:
        check(lib().dl_decoder_cache_clear(self.cache))

    def decode_features(self, x: np.ndarray) -> np.ndarray:
        """TransformerDecoder::decode through dl_transformer_decoder_decode: host features in, host features out."""
        xin = Tensor.from_numpy(np.asarray(x, dtype=np.float32), device=self.dev)
        out = C.c_void_p()
        check(lib().dl_transformer_decoder_decode(self.decoder.h, xin.h, self.cache, C.byref(out)))
        return Tensor(out).numpy()

    def decode_ids(self, ids: np.ndarray) -> np.ndarray:
        """The reference example's decode: embedding -> decoder.decode -> output Linear; logits [B, L, V]."""
        tid = Tensor.from_numpy(np.asarray(ids, dtype=np.int64), device=self.dev)
        x = self.embedding(tid)
        h = C.c_void_p()
        check(lib().dl_transformer_decoder_decode(self.decoder.h, x.h, self.cache, C.byref(h)))
        return self.output(Tensor(h)).numpy()

    def generate(self, prompt: np.ndarray, steps: int, prompt_on_device: bool = False) -> np.ndarray:
        self.new_cache()
        p = Tensor.from_numpy(np.asarray(prompt, dtype=np.int64), device=self.dev if prompt_on_device else cpu())
        out = C.c_void_p()
        check(lib().dl_decoder_generate(self.decoder.h, self.embedding.h, self.output.h, p.h, steps, self.cache, C.byref(out)))
        return Tensor(out).numpy()


class Generation:
    def __init__(self, model: DecoderModel, batch: int, max_steps: int):
        self.model = model
        g = C.c_void_p()
        check(lib().dl_generation_create(model.decoder.h, model.embedding.h, model.output.h, model.cache, batch, max_steps,
                                         C.byref(g)))
        self.h = g
        self.batch = batch

    def __del__(self):
        try:
            if self.h:
                lib().dl_generation_release(self.h)
                self.h = None
        except Exception:
            pass

    def prefill(self, prompt: np.ndarray, on_device: bool = False) -> None:
        p = Tensor.from_numpy(np.asarray(prompt, dtype=np.int64), device=self.model.dev if on_device else cpu())
        check(lib().dl_generation_prefill(self.h, p.h))

    def step(self, steps: int = 1) -> None:
        check(lib().dl_generation_step(self.h, steps))

    def step_host(self, ids_in: np.ndarray | None, ids_out: np.ndarray) -> None:
        ip = C.POINTER(C.c_int64)
        check(lib().dl_generation_step_host(self.h, ids_in.ctypes.data_as(ip) if ids_in is not None else None,
                                            ids_out.ctypes.data_as(ip)))

    def run_host(self, ids_in: np.ndarray | None, steps: int) -> np.ndarray:
        """`steps` host-in-the-loop steps in one library call; returns the chosen ids [steps, batch]."""
        ip = C.POINTER(C.c_int64)
        out = np.empty((steps, self.batch), dtype=np.int64)
        check(lib().dl_generation_run_host(self.h, ids_in.ctypes.data_as(ip) if ids_in is not None else None, steps,
                                           out.ctypes.data_as(ip)))
        return out

    def step_sampled(self, temperature: float, uniforms: np.ndarray) -> np.ndarray:
        u = np.ascontiguousarray(uniforms, dtype=np.float64)
        out = np.empty(u.shape[0], dtype=np.int64)
        check(lib().dl_generation_step_sampled(self.h, float(temperature), u.ctypes.data, out.ctypes.data))
        return out

    def tokens(self) -> np.ndarray:
        out = C.c_void_p()
        check(lib().dl_generation_tokens(self.h, C.byref(out)))
        return Tensor(out).numpy()

    def logits(self) -> np.ndarray:
        out = C.c_void_p()
        check(lib().dl_generation_logits(self.h, C.byref(out)))
        return Tensor(out).numpy()

    def profile_step(self) -> dict:
        ms = (C.c_double * 4)()
        check(lib().dl_generation_profile_step(self.h, ms))
        return {"linear_ms": ms[0], "attention_ms": ms[1], "other_ms": ms[2], "launches": int(ms[3])}

    def launches_per_step(self) -> int:
        return lib().dl_generation_launches_per_step(self.h)


def synchronize(device: int = 0) -> None:
    check(lib().dl_synchronize(cuda(device)))


def timer_start(device: int = 0) -> None:
    check(lib().dl_b200_timer_start(cuda(device)))


def timer_stop(device: int = 0) -> float:
    ms = C.c_double()
    check(lib().dl_b200_timer_stop(cuda(device), C.byref(ms)))
    return ms.value


def tensor_parallel_init(rank: int, world: int, device: int, peer_slot_bytes: int = 8 << 20, push: bool | None = None) -> None:
    """Joins the tensor-parallel group of `world` ranks; the NCCL id travels over torch.distributed (any backend).
    `peer_slot_bytes` > 0 also maps the ranks' symmetric memory (CUDA IPC handles gathered the same way) so that steps of
    up to that many bytes of residual rows sum over NVLink peer memory instead of calling NCCL."""
    import torch
    import torch.distributed as dist
    ident = (C.c_char * 128)()
    if rank == 0:
        check(lib().dl_b200_tp_unique_id(ident))
    payload = torch.tensor(list(ident.raw), dtype=torch.uint8)
    if dist.get_backend() == "nccl":
        payload = payload.cuda(device)
    dist.broadcast(payload, src=0)
    raw = bytes(payload.cpu().tolist())
    check(lib().dl_b200_tp_init(cuda(device), rank, world, raw))
    if peer_slot_bytes > 0 and world <= 8:
        handle = (C.c_char * 64)()
        check(lib().dl_b200_tp_symmetric_handle(cuda(device), peer_slot_bytes, handle))
        mine = torch.tensor(list(handle.raw), dtype=torch.uint8)
        if dist.get_backend() == "nccl":
            mine = mine.cuda(device)
        table = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(table, mine)
        check(lib().dl_b200_tp_symmetric_open(cuda(device), bytes(torch.cat(table).cpu().tolist()), world))
        if push is not None:
            check(lib().dl_b200_tp_set_push(cuda(device), int(push)))
        dist.barrier()   # every rank has mapped every region before the first step


def tensor_parallel_finalize(device: int) -> None:
    check(lib().dl_b200_tp_finalize(cuda(device)))
