"""Regenerates tests/golden/decoder_golden.npz, the weight archives tests/golden/*.ct and the ONNX files tests/golden/*.onnx by running the seeded cases of cases.py on the UNMODIFIED
reference CPU library (oracle/_ref, built by `make -C oracle ref` where the reference tree is present).

    python tests/golden/make_golden.py

The vectors are what the reference itself answers; tests compare the oracle port (bit-exact) and the CUDA path
(within the stated tolerances) with them on machines where the reference is absent.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import oracle  # noqa: E402
from cases import sampling_case, archive_cases, attention_cases, attention_inputs, decoder_cases, token_stream  # noqa: E402
from ctorch_b200 import workloads as W  # noqa: E402


def main():
    out = {}
    for name, (spec, seed, scale, chunks) in decoder_cases().items():
        weights = W.make_weights(spec, seed=seed, scale=scale)
        model = oracle.CpuDecoder(spec, weights, kind="ref")
        ids = token_stream(spec, chunks)
        model.new_cache()
        start = 0
        for i, n in enumerate(chunks):
            out[f"{name}/logits{i}"] = model.decode_ids(ids[:, start:start + n])
            start += n
        tokens, logits = model.generate(W.make_prompts(spec), spec["steps"])
        out[f"{name}/greedy_tokens"] = tokens
        out[f"{name}/greedy_logits"] = logits
        model.close()
    for name, case in attention_cases().items():
        q, k, v = attention_inputs(case)
        out[f"attention/{name}"] = oracle.gqa_attention(q, k, v, case[6], kind="ref")
    rng = np.random.default_rng(31)
    x = rng.standard_normal((3, 2, 4, 16), dtype=np.float32)
    out["rotary/offset3"] = oracle.rotary(x, 10000.0, 12, 3, kind="ref")
    xr = rng.standard_normal((5, 48), dtype=np.float32)
    out["rms_norm/eps1e-5"] = oracle.rms_norm(xr, 1 + 0.1 * rng.standard_normal(48).astype(np.float32), 1e-5, kind="ref")
    for dt in ("f32", "bf16"):
        r2 = np.random.default_rng(41)
        cast = (lambda a: W.bf16_bits(a)) if dt == "bf16" else (lambda a: a)
        w = cast((0.1 * r2.standard_normal((24, 40), dtype=np.float32)))
        down = cast((0.1 * r2.standard_normal((4, 40), dtype=np.float32)))
        up = cast((0.1 * r2.standard_normal((24, 4), dtype=np.float32)))
        xl = r2.standard_normal((3, 40), dtype=np.float32)
        y, merged = oracle.lora_linear(xl, w, down, up, 4, 8.0, kind="ref")
        out[f"lora/{dt}/y"] = y
        out[f"lora/{dt}/merged"] = merged
        out[f"linear/{dt}"] = oracle.linear(xl, w, kind="ref")
    logits, temperature, uniforms = sampling_case()
    out["sample/index"] = oracle.sample(logits, temperature, uniforms, kind="ref")
    here = os.path.dirname(os.path.abspath(__file__))
    for name, spec in archive_cases().items():   # weight archives written by the reference's dl::io::save
        model = oracle.CpuDecoder(spec, W.make_weights(spec, seed=77), kind="ref")
        model.save_state(os.path.join(here, name + ".ct"))
        # the same decoder written by the reference's ONNX exporter: features -> hidden states, and input_ids -> logits
        model.save_onnx(os.path.join(here, name + "_decoder.onnx"), False)
        model.save_onnx(os.path.join(here, name + "_lm.onnx"), True)
        model.close()
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "decoder_golden.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
