"""One rank of the tensor-parallel parity check; started by test_tensor_parallel_gpu.py through torch.distributed.run.

Every rank holds the same seeded weights and prompts, computes its slice of the heads / SwiGLU features, and must end
with the same logits as a single-GPU run of the same model on its own device (summation order differs, so the bound
is the bf16 tolerance, not bit equality).  Rank 0 also checks against the CPU oracle and prints one JSON line."""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch.distributed as dist

import ctorch_b200 as B
import oracle
from ctorch_b200 import workloads as W


def rel(a, b):
    return float(np.abs(a.astype(np.float64) - b.astype(np.float64)).max() / max(1e-30, np.abs(b).max()))


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dist.init_process_group("gloo")
    # 64 KiB slots: single-token steps (rows * 512 * 4 bytes <= 64 KiB) sum over NVLink peer memory, prefill chunks keep NCCL
    B.tensor_parallel_init(rank, world, local, peer_slot_bytes=64 << 10)
    report = {"rank": rank, "cases": []}
    # streaming kernel with adapters, partial sums pulled by the sum kernel; tensor-core kernel without adapters, partial sums
    # pushed by the projections' epilogues
    for batch, adapters, push in ((4, True, False), (32, False, True), (4, False, True)):
        B.check(B.lib().dl_b200_tp_set_push(B.cuda(local), int(push)))
        spec = dict(vocab=1024, d_model=512, layers=3, heads=8, kv_heads=8 if world > 4 else 4, hidden=1024, dtype="bf16", batch=batch, prompt=40,
                    steps=6, context=64, tied=True, eps=1e-5, rope_base=10000.0)
        if adapters:
            spec.update(lora_rank=8, lora_alpha=16.0)
        weights = W.make_weights(spec, seed=5)
        lora = W.make_lora(spec, seed=6) if adapters else None
        prompt = W.make_prompts(spec, seed=7)
        single = B.DecoderModel(spec, weights, lora=lora, device=local)
        want_prefill = single.decode_ids(prompt)
        want_step = single.decode_ids(prompt[:, :1])
        sharded = B.DecoderModel(spec, weights, lora=lora, device=local, tensor_parallel=(rank, world))
        got_prefill = sharded.decode_ids(prompt)
        got_step = sharded.decode_ids(prompt[:, :1])
        sharded.new_cache()
        tokens = sharded.generate(prompt, spec["steps"])          # graph replay with the all-reduce captured inside
        gathered = [None] * world
        dist.all_gather_object(gathered, tokens.tolist())
        case = {"batch": batch, "push": push, "prefill": rel(got_prefill, want_prefill), "step": rel(got_step, want_step),
                "same_tokens_on_all_ranks": all(g == gathered[0] for g in gathered), "cache_length": sharded.cache_length()}
        if rank == 0:
            cpu = oracle.CpuDecoder(spec, weights, lora=lora)
            case["oracle_prefill"] = rel(got_prefill, cpu.decode_ids(prompt))
        report["cases"].append(case)
        del single, sharded
    B.synchronize(local)
    dist.barrier()
    B.tensor_parallel_finalize(local)
    print(json.dumps(report), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
