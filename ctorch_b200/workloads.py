"""Seeded synthetic decoder workloads: shapes, weights and prompts.

The five shapes are the benchmark configurations of the decoder token loop.  No dataset or checkpoint is
involved: weights are N(0, 0.02) from a fixed numpy seed (RMSNorm weights 1 + small noise so that the norm
weight product is exercised), prompts are uniform random token ids.  bf16 tensors travel as uint16 bit
patterns (round-to-nearest-even of the f32 draw), which is how every consumer here takes them.
"""
from __future__ import annotations

import numpy as np

CONFIGS = {
    # byte-level decoder the reference can run on a CPU in seconds
    "c1": dict(vocab=256, d_model=256, layers=4, heads=8, kv_heads=2, hidden=688, dtype="f32",
               batch=1, prompt=64, steps=128),
    # small GQA decoder, the single-GPU benchmark workload
    "c2": dict(vocab=32000, d_model=768, layers=12, heads=12, kv_heads=4, hidden=2048, dtype="bf16",
               batch=16, prompt=512, steps=256),
    # decode-attention microbenchmark (attention only)
    "c3": dict(batch=64, heads=32, kv_heads=8, head_dim=128, min_context=1024, max_context=32768, dtype="bf16"),
    # 1B-shape decoder, batch sharded over GPUs by sequence
    "c4": dict(vocab=32000, d_model=2048, layers=16, heads=32, kv_heads=8, hidden=8192, dtype="bf16",
               batch=256, prompt=1024, steps=512),
    # 8B-shape decoder with rank-16 adapters on q and v, KV-head tensor parallel
    "c5": dict(vocab=128256, d_model=4096, layers=32, heads=32, kv_heads=8, hidden=14336, dtype="bf16",
               batch=32, prompt=4096, steps=256, lora_rank=16, lora_alpha=32.0),
}
for _c in CONFIGS.values():
    if "prompt" in _c:
        _c.setdefault("context", _c["prompt"] + _c["steps"])
        _c.setdefault("tied", True)
        _c.setdefault("eps", 1e-5)
        _c.setdefault("rope_base", 10000.0)


def tiny(dtype: str = "f32", **overrides) -> dict:
    """A decoder small enough for exhaustive CPU comparison (the shape of the reference's own state test)."""
    spec = dict(vocab=97, d_model=64, layers=2, heads=4, kv_heads=2, hidden=96, dtype=dtype, batch=2,
                prompt=6, steps=5, context=24, tied=True, eps=1e-5, rope_base=10000.0)
    spec.update(overrides)
    return spec


def bf16_bits(values: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns, round to nearest even."""
    u = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def tensor_shapes(spec: dict) -> list[tuple[str, tuple[int, ...]]]:
    """(state name, shape) in the canonical order every implementation here consumes."""
    D, F = spec["d_model"], spec["hidden"]
    kv = spec["kv_heads"] * (D // spec["heads"])
    out = [("tokens.weight", (spec["vocab"], D))]
    for i in range(spec["layers"]):
        p = f"decoder.layer{i}."
        out += [(p + "attention.query.weight", (D, D)), (p + "attention.key.weight", (kv, D)),
                (p + "attention.value.weight", (kv, D)), (p + "attention.output.weight", (D, D)),
                (p + "feedforward.gate.weight", (F, D)), (p + "feedforward.up.weight", (F, D)),
                (p + "feedforward.down.weight", (D, F)), (p + "attention_norm.weight", (D,)),
                (p + "feedforward_norm.weight", (D,))]
    out.append(("decoder.normalization.weight", (D,)))
    if not spec.get("tied", True):
        out.append(("output.weight", (spec["vocab"], D)))
    return out


def make_weights(spec: dict, seed: int = 1234, scale: float = 0.02, threads: int | None = None) -> list[np.ndarray]:
    """Ordered tensors in the model dtype (float32 arrays, or uint16 bf16 bit patterns).  Every tensor has its own
    generator seeded by (seed, index), so the draws do not depend on how many worker threads make them."""
    def one(item):
        index, (name, shape) = item
        rng = np.random.default_rng([seed, index])
        if name.endswith("norm.weight") or name.endswith("normalization.weight"):
            w = (1.0 + 0.1 * rng.standard_normal(shape)).astype(np.float32)
        else:
            w = rng.standard_normal(shape, dtype=np.float32)
            w *= np.float32(scale)
        return bf16_bits(w) if spec["dtype"] == "bf16" else w

    items = list(enumerate(tensor_shapes(spec)))
    if threads is None:
        import os
        threads = min(16, len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    if threads <= 1 or len(items) < 4:
        return [one(item) for item in items]
    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(max_workers=threads) as pool:   # numpy releases the GIL inside the generators
        return list(pool.map(one, items))


def make_lora(spec: dict, seed: int = 4321) -> list[np.ndarray] | None:
    """Per layer: q.down [r,D], q.up [D,r], v.down [r,D], v.up [kv,r].  `up` is non-zero on purpose (the
    reference initialises it to zero, which would make the adapter a no-op)."""
    r = spec.get("lora_rank", 0)
    if not r:
        return None
    D = spec["d_model"]
    kv = spec["kv_heads"] * (D // spec["heads"])
    out = []
    for i in range(spec["layers"]):
        for j, shape in enumerate([(r, D), (D, r), (r, D), (kv, r)]):
            rng = np.random.default_rng([seed, i, j])
            w = (0.05 * rng.standard_normal(shape, dtype=np.float32)).astype(np.float32)
            out.append(bf16_bits(w) if spec["dtype"] == "bf16" else w)
    return out


def make_prompts(spec: dict, batch: int | None = None, length: int | None = None, seed: int = 99) -> np.ndarray:
    batch = spec["batch"] if batch is None else batch
    length = spec["prompt"] if length is None else length
    rng = np.random.default_rng([seed, batch, length])
    return rng.integers(0, spec["vocab"], size=(batch, length), dtype=np.int64)


def weight_bytes(spec: dict) -> int:
    """Bytes of weights one decode step must read (tied table counted once)."""
    size = 2 if spec["dtype"] == "bf16" else 4
    return sum(int(np.prod(shape)) for _, shape in tensor_shapes(spec)) * size


def kv_bytes_per_token(spec: dict, kv_dtype: str) -> int:
    """Bytes of K and V one cached position holds across all layers, per sequence."""
    hd = spec["d_model"] // spec["heads"]
    return 2 * spec["layers"] * spec["kv_heads"] * hd * (2 if kv_dtype == "bf16" else 4)
