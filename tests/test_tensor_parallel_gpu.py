"""KV-head tensor parallelism over two and four GPUs (one process per GPU; sums over NVLink peer memory for single-token
steps, NCCL all-reduce on the library's stream for prefill chunks): each rank computes its share of the heads and SwiGLU
features; logits must match the single-GPU run and the CPU oracle within the bf16 tolerance, and every rank must generate the
same tokens.  Skipped on a box with fewer GPUs."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BF16_TOL = 2e-2


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_matches_single_gpu(world):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr", "127.0.0.1",
           "--master-port", str(29671 + world), os.path.join(ROOT, "tests", "tp_worker.py")]
    result = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert result.returncode == 0, (result.stdout[-1500:], result.stderr[-8000:])
    decoder, reports, at = json.JSONDecoder(), [], result.stdout.find('{"rank"')
    while at >= 0:   # the ranks share one pipe: their lines may arrive without a newline between them
        value, end = decoder.raw_decode(result.stdout, at)
        reports.append(value)
        at = result.stdout.find('{"rank"', end)
    assert sorted(r["rank"] for r in reports) == list(range(world))
    for report in reports:
        for case in report["cases"]:
            assert case["prefill"] < BF16_TOL and case["step"] < BF16_TOL, case
            assert case["same_tokens_on_all_ranks"], case
            assert case["cache_length"] == 40 + 6 - 1
            if report["rank"] == 0:
                assert case["oracle_prefill"] < BF16_TOL, case
