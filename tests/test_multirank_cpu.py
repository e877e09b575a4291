"""Rank plumbing of the benchmark with two host-only processes (gloo): every rank decodes its own sequences
(different prompt seeds), times are reduced with MAX over ranks, only rank 0 reports, and the reference arm runs
on rank 0 alone while the other ranks exit 0."""
import json
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_ranks(script_args, port):
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), *script_args]
    return subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)


def json_objects(text):
    """Every top-level JSON object in `text`; two ranks may write to the shared pipe without a newline between them."""
    decoder, found, at = json.JSONDecoder(), [], text.find("{")
    while at >= 0:
        try:
            value, end = decoder.raw_decode(text, at)
            found.append(value)
            at = text.find("{", end)
        except json.JSONDecodeError:
            at = text.find("{", at + 1)
    return found


def test_rank_helpers_under_gloo(tmp_path):
    script = tmp_path / "ranks.py"
    script.write_text(textwrap.dedent("""
        import json, sys
        sys.path.insert(0, %r)
        import bench
        from ctorch_b200 import workloads as W
        rank, world, local, dist = bench.distributed()
        assert world == 2 and dist is not None
        bench.barrier(dist, local)
        slowest = bench.max_over_ranks(10.0 + rank, dist, local)
        spec = W.tiny("f32")
        prompt = W.make_prompts(spec, seed=99 + rank)
        print(json.dumps({"rank": rank, "slowest": slowest, "first": int(prompt[0, 0]), "sum": int(prompt.sum())}))
        dist.destroy_process_group()
    """ % ROOT))
    result = run_ranks([str(script)], 29641)
    assert result.returncode == 0, result.stderr[-2000:]
    lines = json_objects(result.stdout)
    assert sorted(l["rank"] for l in lines) == [0, 1]
    assert all(l["slowest"] == 11.0 for l in lines)          # MAX over ranks
    assert lines[0]["sum"] != lines[1]["sum"]                  # independent sequences per rank


def test_reference_arm_prints_on_rank0_only():
    result = run_ranks(["bench.py", "--impl", "reference", "--workload", "c1", "--gpus", "2", "--steps", "3", "--warmup", "3"], 29642)
    assert result.returncode == 0, result.stderr[-2000:]
    lines = json_objects(result.stdout)
    assert len(lines) == 1
    line = lines[0]
    assert line["impl"] == "reference" and line["n_gpus"] == 2 and line["value"] > 0
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["e2e"]["h2d_bytes_per_step"] == 0
