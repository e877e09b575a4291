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
