"""The seeded cases behind the golden vectors: shared by make_golden.py (which runs them on the reference
library) and by the tests (which run them on the oracle port and on the CUDA path)."""
import numpy as np

from ctorch_b200 import workloads as W


def decoder_cases():
    """name -> (spec, weight seed, weight scale, chunk lengths of a teacher-forced token stream)."""
    return {
        "tiny_f32": (W.tiny("f32"), 11, 0.08, [5, 1, 1, 3, 1]),
        "tiny_bf16": (W.tiny("bf16"), 12, 0.08, [4, 1, 1, 1, 2]),
        "gqa3_f32": (W.tiny("f32", d_model=96, heads=6, kv_heads=2, hidden=160, vocab=131, layers=3, context=40),
                     13, 0.06, [7, 1, 1, 1, 1, 6]),
        "untied_bf16": (W.tiny("bf16", tied=False, d_model=128, heads=4, kv_heads=4, hidden=192, vocab=211,
                               context=32), 14, 0.05, [9, 1, 1, 1]),
    }


def attention_cases():
    """name -> (batch, heads, kv_heads, length, source, head_dim, causal_offset, seed)."""
    return {
        "decode_g4": (2, 8, 2, 1, 37, 32, -1, 21),
        "decode_hd128": (1, 8, 2, 1, 130, 128, -1, 22),
        "chunk_masked": (2, 4, 2, 5, 12, 16, 7, 23),
        "prefill": (1, 6, 3, 9, 9, 64, 0, 24),
    }


def attention_inputs(case):
    b, h, hk, l, s, hd, _, seed = case
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((b, h, l, hd), dtype=np.float32)
    k = rng.standard_normal((b, hk, s, hd), dtype=np.float32)
    v = rng.standard_normal((b, hk, s, hd), dtype=np.float32)
    return q, k, v


def token_stream(spec, chunks, seed=5):
    rng = np.random.default_rng([seed, sum(chunks)])
    return rng.integers(0, spec["vocab"], size=(spec["batch"], sum(chunks)), dtype=np.int64)


def archive_cases():
    """name -> spec of the decoders whose weights the reference writes to tests/golden/<name>.ct (a few KB each)."""
    micro = dict(vocab=19, d_model=16, layers=2, heads=4, kv_heads=2, hidden=24, batch=2, prompt=3, steps=2, context=8, tied=True,
                 eps=1e-5, rope_base=10000.0)
    return {"micro_f32": dict(micro, dtype="f32"), "micro_bf16": dict(micro, dtype="bf16")}


def sampling_case():
    """(logits [rows, width] f32, temperature, uniforms [rows] as multiples of 2**-53): peaked and flat rows, variates at
    both ends of the unit interval."""
    import numpy as np
    rng = np.random.default_rng(2024)
    rows, width = 24, 517
    logits = (rng.standard_normal((rows, width)) * rng.uniform(0.5, 6.0, size=(rows, 1))).astype(np.float32)
    uniforms = np.floor(rng.uniform(0, 1, rows) * 2.0 ** 53) / 2.0 ** 53
    uniforms[0], uniforms[1], uniforms[2] = 0.0, 1.0 - 2.0 ** -53, 0.5
    return logits, 0.8, uniforms
