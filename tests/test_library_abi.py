"""CPU-side checks of the shipped library: it loads without a GPU or driver, exports every symbol the headers
under include/ declare, and refuses to compute without a CUDA device (no CPU fallback)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import ctorch_b200 as B

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = []
    for header in ("ctorch_b200_c_api.h", "ctorch_b200_kernels.h"):
        text = open(os.path.join(ROOT, "include", header)).read()
        names += [n for n in re.findall(r"(?:DL_API|B200_API)[^;(]*?\b(\w+)\s*\(", text) if n not in ("__attribute__", "defined")]
    return names


def test_library_exports_every_declared_symbol():
    lib = B.lib()
    names = declared_symbols()
    assert len(names) > 90
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    assert lib.dl_version() == b"0.3.0"


def test_python_binding_declares_every_symbol():
    lib = B.lib()
    undeclared = [n for n in declared_symbols() if getattr(lib, n).argtypes is None]
    assert not undeclared, undeclared


def test_host_tensors_are_containers():
    x = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    t = B.Tensor.from_numpy(x)
    assert t.shape == (2, 3, 4) and t.dtype == B.F32 and t.device.type == B.CPU
    assert np.array_equal(t.numpy(), x)
    assert np.array_equal(t.select(1, 2).numpy(), x[:, 2])
    assert np.array_equal(t.narrow(2, 1, 2).numpy(), x[:, :, 1:3])
    assert np.array_equal(t.narrow(0, 1, 1).numpy(), x[1:2])


def test_modules_build_on_the_host_with_reference_state_names():
    dec = C.c_void_p()
    B.check(B.lib().dl_transformer_decoder_create(2, 8, 4, 2, 12, 16, B.options(B.BF16), C.byref(dec)))
    module = B.Module(dec)
    names = module.state_names()
    expected = []
    for i in range(2):
        p = f"layer{i}."
        expected += [p + "attention.query.weight", p + "attention.key.weight", p + "attention.value.weight",
                     p + "attention.output.weight", p + "feedforward.gate.weight", p + "feedforward.up.weight",
                     p + "feedforward.down.weight", p + "attention_norm.weight", p + "feedforward_norm.weight"]
    expected.append("normalization.weight")
    assert [n for n in names if "rotary" not in n] == expected
    assert [n for n in names if "rotary" in n] == ["layer0.attention.rotary.cosine", "layer0.attention.rotary.sine",
                                                   "layer1.attention.rotary.cosine", "layer1.attention.rotary.sine"]
    state = module.state()
    assert state["layer0.attention.key.weight"].shape == (4, 8) and state["layer0.attention.key.weight"].dtype == B.BF16
    assert state["layer0.attention.rotary.cosine"].dtype == B.F32
    # a state with a wrong shape is rejected and names the entry
    state["normalization.weight"] = B.Tensor.from_numpy(np.ones(7, dtype=np.uint16), dtype=B.BF16)
    with pytest.raises(B.B200Error, match="normalization.weight"):
        module.load_state(state)


def test_argument_errors_follow_the_reference_messages():
    dec = C.c_void_p(1)
    assert B.lib().dl_transformer_decoder_create(0, 8, 4, 2, 12, 16, B.options(B.F32), C.byref(dec)) == 1
    assert not dec.value and b"at least one layer" in B.lib().dl_last_error()
    assert B.lib().dl_transformer_decoder_create(1, 8, 3, 2, 12, 16, B.options(B.F32), C.byref(dec)) == 1
    assert b"divide evenly" in B.lib().dl_last_error()
    assert B.lib().dl_transformer_decoder_create(1, 8, 4, 2, 12, 16, B.options(B.F64), C.byref(dec)) == 1
    assert b"f32 or bf16" in B.lib().dl_last_error()


def test_no_cpu_fallback():
    """Operators on host tensors fail loudly instead of computing on the CPU."""
    x = B.Tensor.from_numpy(np.ones((2, 8), dtype=np.float32))
    w = B.Tensor.from_numpy(np.ones((4, 8), dtype=np.float32))
    out = C.c_void_p()
    assert B.lib().dl_linear(x.h, w.h, None, C.byref(out)) == 1
    assert b"no CPU compute path" in B.lib().dl_last_error()


def test_decoder_options_are_validated_on_the_host():
    """Tensor-parallel slicing, activation and cache dtypes are checked when they are set (no GPU involved)."""
    l = B.lib()
    dec = C.c_void_p()
    B.check(l.dl_transformer_decoder_create(1, 64, 8, 4, 96, 16, B.options(B.BF16), C.byref(dec)))
    assert l.dl_transformer_decoder_set_tensor_parallel(dec, 0, 2) == 0          # 4 + 2 heads, 48 features per rank
    assert l.dl_transformer_decoder_set_tensor_parallel(dec, 2, 2) == 1 and b"rank must lie" in l.dl_last_error()
    assert l.dl_transformer_decoder_set_tensor_parallel(dec, 0, 3) == 1 and b"split evenly" in l.dl_last_error()
    assert l.dl_transformer_decoder_set_tensor_parallel(dec, 0, 8) == 1 and b"split evenly" in l.dl_last_error()   # 4 KV heads
    assert l.dl_transformer_decoder_set_tensor_parallel(dec, 0, 1) == 0
    assert l.dl_transformer_decoder_set_activation_dtype(dec, B.BF16) == 0
    assert l.dl_transformer_decoder_set_activation_dtype(dec, 1) == 1 and b"f32 or bf16" in l.dl_last_error()       # f64
    assert l.dl_transformer_decoder_set_cache_dtype(dec, 1) == 1 and b"f32 or bf16" in l.dl_last_error()
    l.dl_module_release(dec)
    plain = C.c_void_p()
    B.check(l.dl_transformer_decoder_create(1, 64, 8, 4, 96, 16, B.options(B.F32), C.byref(plain)))
    assert l.dl_transformer_decoder_set_activation_dtype(plain, B.BF16) == 1 and b"bf16 decoder" in l.dl_last_error()
    l.dl_module_release(plain)
    # the group itself lives on a GPU
    assert l.dl_b200_tp_init(B.cpu(), 0, 1, (C.c_char * 128)()) == 1 and b"CUDA device" in l.dl_last_error()
    assert l.dl_b200_tp_symmetric_open(B.cuda(0), (C.c_char * 64)(), 1) == 1 and b"not initialised" in l.dl_last_error()


def test_partial_sum_buffers_follow_the_kernels_tilings():
    """The [parts, rows] buffers that carry per-row sums of squares between kernels are sized from the producers' own
    tile counts.  With the SwiGLU width below the model width the streaming kernel tiles the down-projection by 8
    features: d 4096 / hidden 2048 writes 512 partials per row, d 3072 / hidden 2048 writes 384 (host arithmetic only)."""
    l = B.lib()
    assert l.dl_b200_shadow_partial_rows(4096, 2048) >= 512
    assert l.dl_b200_shadow_partial_rows(3072, 2048) >= 384
    for d, f in ((768, 2048), (2048, 8192), (4096, 14336), (2304, 2048)):
        need = max(l.b200_linear_shadow_parts(rows, inner, d) for rows in (1, 16, 17, 256) for inner in (d, f))
        assert l.dl_b200_shadow_partial_rows(d, f) >= need >= 1
    assert l.dl_b200_shadow_partial_rows(0, 8) == 0


def test_shadow_linear_dispatch_by_row_count():
    """Which kernel family serves a shadow linear: the streaming kernel up to 16 rows (inner size up to 2048), the
    decode-batch kernel up to 256 rows, the prefill kernel above, the thin kernel for adapter down-projections."""
    name = lambda rows, inner, out: B.lib().b200_linear_shadow_kernel(rows, inner, out).decode()
    assert name(1, 768, 2304) == name(16, 2048, 32000) == "linear_stream_kernel"
    assert name(8, 4096, 6144) == "linear_decode_kernel"          # few rows, but wider than the streaming kernel's ring
    assert name(17, 768, 2304) == name(128, 2048, 16384) == name(256, 8192, 2048) == "linear_decode_kernel"
    assert name(257, 2048, 16384) == name(8192, 2048, 3072) == "linear_gemm_kernel"
    assert name(32, 4096, 32) == "linear_thin_kernel"


def test_decode_launch_shapes_fit_the_sm():
    """The cost-model search of the decode-batch kernel, on the host: for the projection sizes of every BASELINE
    configuration and some odd ones, at every row count it serves, the shape it picks fits an SM (227 KB of shared memory,
    512 tensor-memory columns, a ring of at least two stages unless the CTA has a single K block) and covers the problem."""
    shape = (C.c_int32 * 10)()
    sizes = [(768, 2304), (768, 768), (768, 4096), (2048, 768), (768, 32000), (2048, 3072), (2048, 2048), (2048, 16384), (8192, 2048),
             (2048, 32000), (4096, 6144), (4096, 4096), (4096, 28672), (14336, 4096), (4096, 128256), (2048, 1024), (1024, 7168),
             (7168, 4096), (64, 128), (136, 200), (4096, 50257)]
    for inner, out in sizes:
        for rows in (1, 15, 16, 17, 31, 32, 33, 64, 100, 128, 129, 200, 256):
            for planes in (0, 1):
                assert B.lib().b200_linear_decode_launch_shape(rows, inner, out, planes, shape) == 1, (rows, inner, out)
                tiles, split, groups, stages, stage_bytes, n_pad, tmem, smem, token_tile, token_tiles = list(shape)
                k_blocks = -(-inner // 64)
                per_cta = -(-k_blocks // split)
                assert tiles in (1, 2, 4) and 1 <= split <= 8 and split <= max(1, k_blocks // 2), (rows, inner, out, list(shape))
                assert groups * tiles * 128 >= out and (groups - 1) * tiles * 128 < out
                assert token_tile <= 128 and token_tile * token_tiles >= rows and (token_tiles - 1) * token_tile < rows
                assert n_pad % 16 == 0 and token_tile <= n_pad <= 128
                assert tmem <= 512 and tmem >= tiles * n_pad and tmem & (tmem - 1) == 0
                assert smem <= 232448 and stages * stage_bytes + 1024 <= smem
                assert stage_bytes == tiles * 16384 + (2 if planes else 1) * n_pad * 128
                assert 1 <= stages <= 8 and stages >= min(2, per_cta)
    assert B.lib().b200_linear_decode_launch_shape(257, 2048, 2048, 1, shape) == 0
