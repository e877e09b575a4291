"""The plain-C oracle must answer the committed golden vectors (produced by the unmodified reference CPU
library, see tests/golden/make_golden.py) bit for bit."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))

import oracle
from cases import attention_cases, attention_inputs, decoder_cases, sampling_case, token_stream
from ctorch_b200 import workloads as W

GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "decoder_golden.npz"))


def same_bits(a, b):
    return a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))


@pytest.mark.parametrize("name", list(decoder_cases()))
def test_decoder_teacher_forced_and_greedy(name):
    spec, seed, scale, chunks = decoder_cases()[name]
    model = oracle.CpuDecoder(spec, W.make_weights(spec, seed=seed, scale=scale), kind="port")
    ids = token_stream(spec, chunks)
    model.new_cache()
    start = 0
    for i, n in enumerate(chunks):
        assert same_bits(model.decode_ids(ids[:, start:start + n]), GOLDEN[f"{name}/logits{i}"]), (name, i)
        start += n
    assert model.cache_length() == sum(chunks)
    tokens, logits = model.generate(W.make_prompts(spec), spec["steps"])
    assert np.array_equal(tokens, GOLDEN[f"{name}/greedy_tokens"])
    assert same_bits(logits, GOLDEN[f"{name}/greedy_logits"])


@pytest.mark.parametrize("name", list(attention_cases()))
def test_attention(name):
    case = attention_cases()[name]
    q, k, v = attention_inputs(case)
    assert same_bits(oracle.gqa_attention(q, k, v, case[6]), GOLDEN[f"attention/{name}"])


def test_small_operators():
    rng = np.random.default_rng(31)
    x = rng.standard_normal((3, 2, 4, 16), dtype=np.float32)
    assert same_bits(oracle.rotary(x, 10000.0, 12, 3), GOLDEN["rotary/offset3"])
    xr = rng.standard_normal((5, 48), dtype=np.float32)
    w = 1 + 0.1 * rng.standard_normal(48).astype(np.float32)
    assert same_bits(oracle.rms_norm(xr, w, 1e-5), GOLDEN["rms_norm/eps1e-5"])


@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_linear_and_lora(dt):
    r2 = np.random.default_rng(41)
    cast = W.bf16_bits if dt == "bf16" else (lambda a: a)
    w = cast(0.1 * r2.standard_normal((24, 40), dtype=np.float32))
    down = cast(0.1 * r2.standard_normal((4, 40), dtype=np.float32))
    up = cast(0.1 * r2.standard_normal((24, 4), dtype=np.float32))
    x = r2.standard_normal((3, 40), dtype=np.float32)
    y, merged = oracle.lora_linear(x, w, down, up, 4, 8.0)
    assert same_bits(y, GOLDEN[f"lora/{dt}/y"])
    assert same_bits(merged, GOLDEN[f"lora/{dt}/merged"])
    assert same_bits(oracle.linear(x, w), GOLDEN[f"linear/{dt}"])


def test_cached_equals_uncached():
    """The property the reference's own state test pins: chunked decode == one full pass."""
    spec = W.tiny("f32")
    model = oracle.CpuDecoder(spec, W.make_weights(spec, seed=3, scale=0.08))
    ids = token_stream(spec, [6])
    model.new_cache()
    full = model.decode_ids(ids)
    model.new_cache()
    parts = np.concatenate([model.decode_ids(ids[:, :2]), model.decode_ids(ids[:, 2:])], axis=1)
    np.testing.assert_allclose(parts, full, rtol=1e-5, atol=1e-6)


def test_cache_errors_and_rollback():
    spec = W.tiny("f32", context=8)
    model = oracle.CpuDecoder(spec, W.make_weights(spec, seed=3))
    ids = token_stream(spec, [9])
    model.new_cache()
    model.decode_ids(ids[:, :6])
    with pytest.raises(RuntimeError, match="exceeds capacity"):
        model.decode_ids(ids[:, 6:9])
    assert model.cache_length() == 6
    with pytest.raises(RuntimeError, match="existing prefix"):
        model.truncate(7)
    model.truncate(2)
    assert model.cache_length() == 2
    model.clear()
    assert model.cache_length() == 0


def test_argmax_rules():
    x = np.array([[1.0, 3.0, 3.0, 2.0], [0.0, np.nan, 5.0, np.nan], [-1.0, -1.0, -1.0, -1.0]], dtype=np.float32)
    assert oracle.argmax(x).tolist() == [1, 1, 0]


def test_temperature_sampling_matches_reference_draws():
    """softmax(logits / T) + std::discrete_distribution of the reference example (examples/text_generate.cpp:38-39), answered
    by the reference library with a generator that yields the given uniform variates."""
    logits, temperature, uniforms = sampling_case()
    assert np.array_equal(oracle.sample(logits, temperature, uniforms), GOLDEN["sample/index"])
