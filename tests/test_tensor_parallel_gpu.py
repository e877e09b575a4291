"""KV-head tensor parallelism over two, four and eight GPUs (one process per GPU; sums over NVLink peer memory for single-token
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


@pytest.mark.parametrize("world", [2, 4, 8])
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


def test_group_init_times_out_when_a_rank_never_joins():
    """Failure made on the host: one process asks to join a group of two and nobody else ever does.  The call must come back
    with an error after the configured deadline instead of blocking for good (ncclCommInitRank runs on a helper thread).  It
    runs in a child process, which is left with that helper thread and simply exits."""
    import subprocess
    import sys
    import textwrap
    script = textwrap.dedent("""
        import ctypes as C, os, sys, time
        sys.path.insert(0, %r)
        os.environ["CTORCH_B200_TP_INIT_TIMEOUT_S"] = "4"
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        import ctorch_b200 as B
        l = B.lib()
        ident = (C.c_char * 128)()
        B.check(l.dl_b200_tp_unique_id(ident))
        begin = time.time()
        status = l.dl_b200_tp_init(B.cuda(0), 0, 2, ident.raw)
        elapsed = time.time() - begin
        message = l.dl_last_error().decode()
        print("status", status, "elapsed", round(elapsed, 1), message)
        ok = status == 1 and "timed out" in message and 3.0 < elapsed < 60.0
        # the device is still usable and outside any group
        x = B.Tensor.from_numpy(__import__("numpy").ones((2, 8), dtype="float32"), device=B.cuda(0))
        ok = ok and float(x.numpy().sum()) == 16.0
        sys.stdout.flush()
        os._exit(0 if ok else 1)
    """ % ROOT)
    result = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=300)
    assert result.returncode == 0, result.stdout + result.stderr
