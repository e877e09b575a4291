"""Where the reference library has been compiled (oracle/_ref), the oracle port must agree with it bit for bit
on fresh seeded cases beyond the committed golden vectors, and the golden file must be reproducible."""
import numpy as np
import pytest

import oracle
from ctorch_b200 import workloads as W

pytestmark = pytest.mark.skipif(not oracle.have_ref(), reason="reference library not built on this machine")


@pytest.mark.parametrize("dtype,batch,seed", [("f32", 1, 1), ("f32", 3, 2), ("bf16", 2, 3)])
def test_teacher_forced_bit_exact(dtype, batch, seed):
    spec = W.tiny(dtype, batch=batch, d_model=80, heads=10, kv_heads=5, hidden=112, context=20)
    weights = W.make_weights(spec, seed=seed, scale=0.1)
    port, ref = oracle.CpuDecoder(spec, weights, kind="port"), oracle.CpuDecoder(spec, weights, kind="ref")
    ids = np.random.default_rng(seed).integers(0, spec["vocab"], size=(batch, 14), dtype=np.int64)
    port.new_cache(), ref.new_cache()
    for lo, hi in [(0, 6), (6, 7), (7, 8), (8, 12), (12, 14)]:
        a, b = port.decode_ids(ids[:, lo:hi]), ref.decode_ids(ids[:, lo:hi])
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_config1_greedy_bit_exact():
    spec = dict(W.CONFIGS["c1"])
    weights = W.make_weights(spec)
    port, ref = oracle.CpuDecoder(spec, weights, kind="port"), oracle.CpuDecoder(spec, weights, kind="ref")
    prompt = W.make_prompts(spec)
    tp, lp = port.generate(prompt, 24)
    tr, lr = ref.generate(prompt, 24)
    assert np.array_equal(tp, tr) and np.array_equal(lp.view(np.uint32), lr.view(np.uint32))


def test_rope_tables_bit_exact():
    spec = W.tiny("bf16")
    model = oracle.CpuDecoder(spec, W.make_weights(spec), kind="ref")
    hd = spec["d_model"] // spec["heads"]
    cos = np.empty((spec["context"], hd // 2), dtype=np.float32)
    sin = np.empty_like(cos)
    import ctypes as C
    fp = C.POINTER(C.c_float)
    model.l.check(model.l.decoder_rope_tables(model.handle, cos.ctypes.data_as(fp), sin.ctypes.data_as(fp)))
    pc, ps = oracle.rope_tables(hd, spec["context"])
    assert np.array_equal(cos, pc) and np.array_equal(sin, ps)


def test_reference_cache_is_f32_for_bf16_weights():
    spec = W.tiny("bf16")
    model = oracle.CpuDecoder(spec, W.make_weights(spec), kind="ref")
    model.new_cache()
    model.decode_ids(W.make_prompts(spec))
    assert model.l.cache_dtype(model.cache, 0) == oracle.F32


def test_threaded_baseline_matches_serial():
    spec = W.tiny("f32", batch=4)
    model = oracle.CpuDecoder(spec, W.make_weights(spec), kind="ref")
    prompt = W.make_prompts(spec)
    serial, _ = model.generate(prompt, 4)
    assert np.array_equal(model.generate_threads(prompt, 4, 4), serial)


def test_sampling_port_equals_reference_on_fresh_inputs():
    rng = np.random.default_rng(8)
    logits = (rng.standard_normal((40, 1031)) * rng.uniform(0.2, 8.0, size=(40, 1))).astype(np.float32)
    uniforms = np.floor(rng.uniform(0, 1, 40) * 2.0 ** 53) / 2.0 ** 53
    for temperature in (0.5, 1.0, 1.7):
        assert np.array_equal(oracle.sample(logits, temperature, uniforms), oracle.sample(logits, temperature, uniforms, kind="ref"))
