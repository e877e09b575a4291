"""Decode throughput of the B200 decoder token loop.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload c4]

A step is one greedy single-token decode step of the whole batch (embedding ... logits, argmax, token feedback).
Default workload: BASELINE configuration 4, the one the metric is quoted on at 1/2/4/8 GPUs (1B shape: vocab 32000,
d 2048, 16 layers, 32/8 heads, SwiGLU 8192, bf16 weights, 256 independent sequences, prompt 1024 random ids).  Weights
and prompts are seeded synthetic data.  With N > 1 (one process per GPU under torch.distributed.run) the 256 sequences
are divided over the GPUs (256 / N each), weights replicated, no collective on the data path: strong scaling.
`--workload c5` is the 8B shape with adapters, KV-head tensor parallel over the GPUs; `c2` the small decoder (replicas);
`c3` the decode-attention microbenchmark; `linear` one projection in isolation.

The printed JSON line carries the device-resident throughput (`value`: median of 5 timed rounds of K steps), the
host-in-the-loop throughput through the C ABI (`e2e`), the roofline of the kernel class that dominates the step
(`roofline`; the other class in `roofline_second_kernel`), the reference's CPU decoder timed on the host cores
(`cpu_baseline`) and, for the default workload on one GPU, the c3 and c2 figures (`secondary`).  `--impl reference`
times only that CPU decoder: whole for the small configurations, as a full-width slice of 2 and 4 layers extrapolated
linearly in depth for the 1B and 8B shapes (labelled so in the line).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from ctorch_b200 import workloads as W  # noqa: E402

METRIC, UNIT = "decode_tokens_per_s", "tokens/s"
ROUNDS = 5   # timed rounds of `steps` steps each; the line reports the median round


def measured_peaks() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as handle:
            return float(json.load(handle)["hbm_gbs"]), "measured"
    except Exception:  # noqa: BLE001
        return 6650.0, "fallback"


def tensor_peak_tflops() -> float:
    """Measured dense bf16 burst throughput of this pool's B200s (a kernel timed alone), else the stated fallback."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as handle:
            return float(json.load(handle)["bf16_tflops"])
    except Exception:  # noqa: BLE001
        return 1590.0


class ClockSampler:
    """SM clock and throttle reasons of one GPU while the timed region runs: NVML read from a thread every few
    milliseconds (the timed loops last tens of milliseconds), nvidia-smi as a fall-back.  Read-only."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.index, self.rows, self.process = index, [], None
        self.samples, self.thread, self.running, self.nvml, self.first = [], None, False, None, 0

    def mark(self):
        """The timed region starts here: earlier NVML samples (set-up, warm-up) are left out of the summary."""
        self.first = len(self.samples)

    def _visible_index(self) -> int:
        """Index of the CUDA device among the GPUs NVML sees (CUDA_VISIBLE_DEVICES may renumber them)."""
        visible = os.environ.get("CUDA_VISIBLE_DEVICES", "")
        entries = [e for e in visible.split(",") if e.strip()]
        if entries and self.index < len(entries) and entries[self.index].strip().isdigit():
            return int(entries[self.index])
        return self.index

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByIndex(self._visible_index())
            maximum = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            self.nvml, self.running = pynvml, True

            def poll():
                while self.running:
                    try:
                        clock = float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM))
                        reasons = int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle))
                        self.samples.append((clock, maximum, reasons))
                    except Exception:  # noqa: BLE001
                        break
                    time.sleep(0.02)   # the timed host loops run inside one library call, which releases the GIL

            self.thread = threading.Thread(target=poll, daemon=True)
            self.thread.start()
            return
        except Exception:  # noqa: BLE001
            self.nvml = None
        try:
            self.process = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}",
                                             "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                            stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.process = None

    def _read(self):
        for line in self.process.stdout:
            self.rows.append([cell.strip() for cell in line.split(",")])

    def stop(self) -> dict:
        clocks, maxima, reasons = [], [], set()
        if self.nvml is not None:
            self.running = False
            if self.thread:
                self.thread.join(timeout=2)
            for clock, maximum, bits in self.samples[self.first:] or self.samples[-1:]:
                clocks.append(clock)
                maxima.append(maximum)
                reasons.update(name for bit, name in self.REASON_BITS.items() if bits & bit)
            try:
                self.nvml.nvmlShutdown()
            except Exception:  # noqa: BLE001
                pass
        if self.process:
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()
        for row in self.rows:
            try:
                clocks.append(float(row[0]))
                maxima.append(float(row[1]))
            except (ValueError, IndexError):
                continue
            for name, cell in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), row[2:6]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(clocks)) if clocks else None, "sm_max_mhz": max(maxima) if maxima else None,
                "reasons": sorted(reasons), "samples": len(clocks)}


def layer_slice(spec: dict, weights, layers: int):
    """The first `layers` layers of a decoder: (spec, tensors) in the canonical order (table, 9 per layer, final norm)."""
    tail = weights[1 + 9 * spec["layers"]:]
    return dict(spec, layers=layers), [weights[0], *weights[1:1 + 9 * layers], *tail]


def cpu_reference(spec: dict, weights, steps: int, warmup: int, threads: int | None = None, start_context: int | None = None) -> dict:
    """The reference's CPU decoder on this machine's cores, one or more sequences per worker thread, `steps` timed greedy
    steps.  The caches are pre-filled to the benchmark's context (pseudo-random K and V through the reference's own
    KVCache::append, then a short real prompt): a CPU prefill of the full prompt would take minutes.  Models too large to
    run whole (more than 300 M parameters) are timed at two reduced depths, full width, with one sequence per core, and
    extrapolated linearly in the layer count; the result says so."""
    import oracle
    kind = "ref" if oracle.have_ref() else "port"
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    prompt_length = 8
    start_context = start_context or spec["prompt"]
    cached = max(0, start_context - prompt_length) if kind == "ref" else 0

    def timed(run_spec, run_weights, batch, workers):   # reads cached / prompt_length / warmup / steps at call time
        cpu_spec = dict(run_spec, batch=batch, context=cached + prompt_length + warmup + steps + 2)
        model = oracle.CpuDecoder(cpu_spec, run_weights, kind=kind)
        try:
            return oracle.timed_decode(model, W.make_prompts(cpu_spec, batch=batch, length=prompt_length), warmup, steps, workers, cached)
        finally:
            model.close()

    parameters = W.weight_bytes(spec) // (2 if spec["dtype"] == "bf16" else 4)
    context_note = (f"caches pre-filled to {cached + prompt_length} positions ({cached} pseudo-random, {prompt_length}-token prompt decoded)"
                    if cached else f"an {prompt_length}-token prompt")
    if parameters <= 300e6:
        workers = max(1, min(threads or cores, spec["batch"]))
        seconds = timed(spec, weights, spec["batch"], workers)
        return {"value": spec["batch"] * steps / seconds, "unit": UNIT, "cores": workers,
                "kind": "reference" if kind == "ref" else "port", "seconds": seconds, "extrapolated": False,
                "mean_context": cached + prompt_length + warmup + steps / 2.0,
                "sample": f"{steps} greedy steps of batch {spec['batch']} after {context_note} and {warmup} warm-up steps, "
                          f"{workers} threads (own sequences and caches each)"}
    # Reduced slice: one sequence per core, full width, 2 and 4 layers; time(L) = head + L * layer.  A CPU step of this
    # width takes seconds per sequence (the reference widens every bf16 matrix to f32 on each call), so at most four
    # steps are timed after one warm-up step, whatever K and W the GPU arm was given.
    workers = max(1, threads or cores)
    shallow, deep = 2, 4
    steps, warmup, prompt_length = min(steps, 4), min(warmup, 1), 2
    cached = max(0, start_context - prompt_length) if kind == "ref" else 0
    context_note = (f"caches pre-filled to {cached + prompt_length} positions ({cached} pseudo-random, {prompt_length}-token prompt decoded)"
                    if cached else f"a {prompt_length}-token prompt")
    t_shallow = timed(*layer_slice(spec, weights, shallow), workers, workers)
    t_deep = timed(*layer_slice(spec, weights, deep), workers, workers)
    per_layer = max(0.0, (t_deep - t_shallow) / (deep - shallow))
    full = t_shallow + (spec["layers"] - shallow) * per_layer
    return {"value": workers * steps / full, "unit": UNIT, "cores": workers, "kind": "reference" if kind == "ref" else "port",
            "seconds": t_shallow + t_deep, "extrapolated": True, "mean_context": cached + prompt_length + warmup + steps / 2.0,
            "sample": f"EXTRAPOLATED linearly in depth: {steps} greedy steps of {workers} sequences (one per thread, own caches) at full "
                      f"width with {shallow} layers ({t_shallow:.2f} s) and {deep} layers ({t_deep:.2f} s) after {context_note}; "
                      f"{spec['layers']} layers = {full:.2f} s.  The CPU decoder gains nothing from batching, so tokens/s of "
                      f"{workers} sequences on {workers} cores stands for the batch of {spec['batch']}"}


def distributed():
    """(rank, world, local_rank, dist module or None).  torch.distributed is only plumbing: barrier and max-reduce."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world == 1:
        return 0, 1, 0, None
    import torch
    import torch.distributed as dist
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if torch.cuda.is_available():
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:   # host-only processes (tests of the rank plumbing)
        dist.init_process_group("gloo")
    return dist.get_rank(), world, local, dist


def over_ranks(value: float, dist, local: int) -> list[float]:
    """The value of every rank, in rank order."""
    if dist is None:
        return [value]
    import torch
    device = torch.device("cuda", local) if torch.cuda.is_available() else torch.device("cpu")
    mine = torch.tensor([value], dtype=torch.float64, device=device)
    table = [torch.empty_like(mine) for _ in range(dist.get_world_size())]
    dist.all_gather(table, mine)
    return [float(t.item()) for t in table]


def max_over_ranks(value: float, dist, local: int) -> float:
    return max(over_ranks(value, dist, local))


def barrier(dist, local: int):
    if dist is not None:
        import torch
        if torch.cuda.is_available():
            dist.barrier(device_ids=[local])
            torch.cuda.synchronize(local)
        else:
            dist.barrier()


def describe(name: str, spec: dict) -> str:
    """The workload in words: BASELINE configuration and its shape (the JSON line carries no model keys)."""
    return (f"{name}: GQA decoder, vocab {spec['vocab']}, d_model {spec['d_model']}, {spec['layers']} layers, "
            f"{spec['heads']}/{spec['kv_heads']} heads, SwiGLU {spec['hidden']}, {spec['dtype']} weights"
            + (f", rank-{spec['lora_rank']} adapters on q and v" if spec.get("lora_rank") else "")
            + f", batch {spec['batch']}, prompt {spec['prompt']}")


def timed_context(spec: dict, args) -> int:
    """Cache length at which the middle one of the timed rounds starts (prompt, first token, warm-up, two rounds)."""
    return spec["prompt"] + 1 + args.warmup + (ROUNDS // 2) * args.steps


def run_reference(args, spec, weights) -> dict:
    result = cpu_reference(spec, weights, args.steps, args.warmup, start_context=timed_context(spec, args))
    ms = 1000.0 * spec["batch"] / result["value"]   # one step of the whole batch at the measured (or extrapolated) rate
    scaling = "strong" if args.workload in ("c4", "c5") else "weak"
    return {"impl": "reference", "metric": METRIC, "value": result["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": scaling,
            "vs_baseline": None, "dtype": "f32 math on " + spec["dtype"] + " weights (the reference's CPU decoder)", "data": "synthetic",
            "config": {"workload": describe(args.workload, spec), "batch": spec["batch"], "prompt": spec["prompt"],
                       "mean_context": result["mean_context"], "parallelism": f"host threads x{result['cores']}, rank 0 only",
                       "extrapolated": result["extrapolated"]},
            "cpu_baseline": {k: result[k] for k in ("value", "unit", "cores", "kind", "sample", "extrapolated")},
            "e2e": {"value": result["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}


def measure_decoder(args, name, spec, weights, rank, world, local, dist) -> dict:
    """Prefill + timed greedy decode of one decoder workload on this rank's GPU; the numbers of the JSON line."""
    import ctorch_b200 as B
    # Configuration 4 is one batch of 256 independent sequences divided over the GPUs (strong scaling: 256 / N each).
    divided = name == "c4" and world > 1
    whole_batch = spec["batch"]
    if divided:
        spec = dict(spec, batch=spec["batch"] // world)
    batch, prompt_len = spec["batch"], spec["prompt"]
    total_steps = (ROUNDS + 1) * args.steps + 2 * args.warmup + 8
    spec = dict(spec, context=max(spec["context"], prompt_len + total_steps + 1))
    # Configuration 5 on more than one GPU is ONE model sliced over the ranks (KV-head tensor parallel): every rank
    # feeds the same sequences and the job's tokens are counted once.  Every other workload runs independent sequences.
    sliced = name == "c5" and world > 1
    if sliced:
        B.tensor_parallel_init(rank, world, local)
    model = B.DecoderModel(spec, weights, lora=W.make_lora(spec), device=local, tensor_parallel=(rank, world) if sliced else None,
                           activation_dtype=args.activations if spec["dtype"] == "bf16" else None)
    gen = B.Generation(model, batch, total_steps + 1)
    if divided:
        prompt = np.ascontiguousarray(W.make_prompts(spec, batch=whole_batch)[rank * batch:(rank + 1) * batch])
    else:
        prompt = W.make_prompts(spec, seed=99 if sliced else 99 + rank)
    sampler = ClockSampler(local)
    sampler.start()
    B.timer_start(local)
    gen.prefill(prompt)
    prefill_ms = B.timer_stop(local)   # first call: includes weight packing and workspace allocation

    # ---- device-resident loop: ROUNDS x K graph replays, each round timed with CUDA events on the library's stream ----
    gen.step(args.warmup)
    B.synchronize(local)
    rounds = []
    sampler.mark()
    for _ in range(ROUNDS):
        start_length = model.cache_length()
        barrier(dist, local)
        B.timer_start(local)
        gen.step(args.steps)
        elapsed = B.timer_stop(local)
        barrier(dist, local)
        rounds.append((max_over_ranks(elapsed, dist, local), start_length))
    device_ms, start_length = sorted(rounds)[ROUNDS // 2]

    # ---- host in the loop: ids H2D, one step, chosen ids D2H, every step (the reference example's loop), one C call ----
    feed = np.ascontiguousarray(gen.tokens()[:, -1])
    feed = np.ascontiguousarray(gen.run_host(feed, args.warmup)[-1])
    barrier(dist, local)
    B.timer_start(local)
    gen.run_host(feed, args.steps)
    e2e_ranks = over_ranks(B.timer_stop(local), dist, local)
    e2e_ms = max(e2e_ranks)
    clocks = sampler.stop()

    # ---- per-kernel-class device time of one eager step (events after every launch) ----
    profile = gen.profile_step()
    for _ in range(2):
        more = gen.profile_step()
        profile = {k: min(profile[k], more[k]) for k in profile}
    launches = gen.launches_per_step()

    tokens = (1 if sliced else world) * batch * args.steps
    mean_context = start_length + args.steps / 2.0
    kv_dtype = "bf16" if spec["dtype"] == "bf16" else "f32"
    linear_bytes = W.weight_bytes(spec)
    kv_bytes = W.kv_bytes_per_token(spec, kv_dtype) * mean_context * batch
    if sliced:   # per GPU: the slice of the layer weights and of the KV heads, plus the replicated logits table
        table = spec["vocab"] * spec["d_model"] * 2
        linear_bytes = (linear_bytes - table) // world + table
        kv_bytes /= world
    peak, peak_kind = measured_peaks()
    step_ms = device_ms / args.steps
    # Device time of a kernel class inside the timed graph replays: the timed step duration times the class's share of
    # device time in the per-launch event profile (the profile runs the same step eagerly, one event after every launch,
    # without the overlap between consecutive kernels that the replayed graph has).
    profiled = profile["linear_ms"] + profile["attention_ms"] + profile["other_ms"]
    shares = {k: (profile[k + "_ms"] / profiled if profiled > 0 else 0.0) for k in ("linear", "attention", "other")}

    def roofline_of(kind):
        bytes_ = linear_bytes if kind == "linear" else kv_bytes
        ms = step_ms * shares[kind]
        achieved = bytes_ / (ms / 1000.0) / 1e9 if ms > 0 else None
        if kind == "linear":
            # the family the library runs the largest projection (gate/up) of this batch on
            kernel = (B.lib().b200_linear_shadow_kernel(batch, spec["d_model"], 2 * spec["hidden"]).decode()
                      if spec["dtype"] == "bf16" else "linear_small_kernel")
            kernel += " (the %d projection launches of one step: weights streamed once)" % (profile["launches"] - spec["layers"] - 2)
        else:
            kernel = ("attention_mma_kernel" if spec["dtype"] == "bf16" else "attention_generic_kernel") + " (%d launches of one step: K and V streamed once)" % spec["layers"]
        # DRAM traffic per algorithmic byte from the ncu captures of these kernels (dram__bytes_read + dram__bytes_write
        # of one launch / its algorithmic bytes): attention 1.03; projections 1.03 (gate/up) to 1.31 (down, whose
        # activation planes and residual rows weigh most against its weights), 1.1 over the launches of a layer
        ratio = 1.03 if kind == "attention" else 1.1
        return {"bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak if achieved else None, "peak_kind": peak_kind, "traffic": bytes_ * ratio,
                "traffic_source": "ncu capture of one launch of a smaller case, scaled by the units processed (x%.2f algorithmic)" % ratio,
                "algorithmic_bytes": bytes_, "launch_ms": ms, "share_of_step": shares[kind],
                "share_source": "per-launch CUDA events of the same step run eagerly", "eager_profile_ms": profile[kind + "_ms"]}

    dominant = "linear" if shares["linear"] >= shares["attention"] else "attention"
    other = "attention" if dominant == "linear" else "linear"
    line = {
        "metric": METRIC, "value": tokens / (device_ms / 1000.0), "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": step_ms, "higher_is_better": True, "scaling": "strong" if name in ("c4", "c5") else "weak", "vs_baseline": None,
        "dtype": ("bf16 weights and KV, f32 accumulate and activations" if args.activations == "f32" else
                  "bf16 weights and KV, f32 accumulate, bf16 activations in passes over more than 16 rows") if spec["dtype"] == "bf16" else "f32",
        "data": "synthetic",
        "config": {"workload": describe(name, dict(spec, batch=whole_batch)), "batch": whole_batch, "batch_per_gpu": batch, "prompt": prompt_len,
                   "mean_context": mean_context,
                   "parallelism": (f"tp{world} (heads, KV heads and SwiGLU features sliced; 2 sums per layer)" if sliced else
                                   f"{whole_batch} independent sequences divided over {world} GPUs, replicated weights, no collective" if divided else
                                   f"replicas x{world}"),
                   "timing": f"median of {ROUNDS} rounds of {args.steps} CUDA-graph replays, CUDA events on the launching stream, max over ranks",
                   "rounds_ms_per_step": [r[0] / args.steps for r in rounds],
                   "l2": "inputs larger than L2: %.0f MB of weights and KV are streamed per step" % ((linear_bytes + kv_bytes) / 1e6),
                   "step_bytes": linear_bytes + kv_bytes,
                   "step_gbs": (linear_bytes + kv_bytes) / (step_ms / 1000.0) / 1e9,
                   "step_frac_of_peak": (linear_bytes + kv_bytes) / (step_ms / 1000.0) / 1e9 / peak,
                   "step_frac_of_nominal_8tbs": (linear_bytes + kv_bytes) / (step_ms / 1000.0) / 1e9 / 8000.0,
                   "roofline_ms_per_step": (linear_bytes + kv_bytes) / peak / 1e6,
                   "kernel_ms_per_step": profile, "prefill_ms_first_call": prefill_ms,
                   "prefill_tokens_per_s_first_call": batch * prompt_len / (prefill_ms / 1000.0)},
        "clocks": clocks,
        "e2e": {"value": tokens / (e2e_ms / 1000.0), "unit": UNIT, "h2d_bytes_per_step": 8 * batch, "d2h_bytes_per_step": 8 * batch,
                "ms_per_step": e2e_ms / args.steps,
                "ranks_ms_per_step": {"min": min(e2e_ranks) / args.steps, "median": float(np.median(e2e_ranks)) / args.steps,
                                      "max": max(e2e_ranks) / args.steps}},
        "gpu_launches": launches * args.steps,
        "roofline": roofline_of(dominant),
        "roofline_second_kernel": roofline_of(other),
    }
    del gen, model
    if sliced:
        B.tensor_parallel_finalize(local)
    return line


def run_b200(args, spec, weights) -> dict:
    rank, world, local, dist = distributed()
    line = measure_decoder(args, args.workload, spec, weights, rank, world, local, dist)
    if rank == 0 and world == 1 and not args.no_cpu and args.workload != "c5":
        cpu = cpu_reference(spec, weights, args.cpu_steps, 1, start_context=timed_context(spec, args))
        line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample", "extrapolated")}
    if world == 1 and args.workload == "c4" and not args.no_secondary:
        # The cheap companions of the headline, in the same record: the decode-attention microbenchmark and the small decoder.
        secondary = {}
        try:
            c3 = run_c3(args, alone=False)
            secondary["c3"] = {"ms_per_step": c3["ms_per_step"], "tokens_per_s": c3["value"], "attention_gbs": c3["roofline"]["achieved"],
                               "frac_of_peak": c3["roofline"]["frac"], "workload": c3["config"]["workload"]}
        except Exception as error:  # noqa: BLE001
            secondary["c3"] = {"error": str(error)[:200]}
        try:
            small = dict(W.CONFIGS["c2"])
            c2 = measure_decoder(args, "c2", small, W.make_weights(small), rank, world, local, dist)
            secondary["c2"] = {"ms_per_step": c2["ms_per_step"], "tokens_per_s": c2["value"], "e2e_tokens_per_s": c2["e2e"]["value"],
                               "step_frac_of_peak": c2["config"]["step_frac_of_peak"], "launches_per_step": c2["config"]["kernel_ms_per_step"]["launches"],
                               "workload": c2["config"]["workload"]}
        except Exception as error:  # noqa: BLE001
            secondary["c2"] = {"error": str(error)[:200]}
        line["secondary"] = secondary
    if dist is not None:
        dist.destroy_process_group()
    return line if rank == 0 else {}


def run_c3(args, alone: bool = True) -> dict:
    """BASELINE configuration 3: decode attention only (batch 64, 32 query / 8 KV heads, head_dim 128, bf16 cache,
    per-sequence contexts uniform in [1024, 32768], one new token per sequence per step)."""
    import ctypes as C

    import torch

    import ctorch_b200 as B
    rank, world, local, dist = distributed() if alone else (0, 1, 0, None)
    cfg = dict(W.CONFIGS["c3"])
    if args.small:   # profiling-sized case of the same kernel: a few hundred MB of K and V, still far above L2
        cfg.update(batch=16, min_context=1024, max_context=8192)
    n, heads, kv_heads, hd = cfg["batch"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    capacity = cfg["max_context"]
    l = B.lib()
    torch.cuda.set_device(local)
    stream = l.dl_b200_stream(B.cuda(local))
    cache = C.c_void_p()
    B.kcheck(l.b200_kv_cache_create(local, B.BF16, n, kv_heads, hd, capacity, 64, C.byref(cache)))
    generator = torch.Generator(device="cuda").manual_seed(7 + rank)
    chunk = 1024
    handles = (C.c_void_p * 1)(cache)
    for _ in range(capacity // chunk):     # K, V ~ N(0, 1), appended chunk by chunk through the C ABI
        k = torch.randn((n, kv_heads, chunk, hd), device="cuda", generator=generator)
        v = torch.randn((n, kv_heads, chunk, hd), device="cuda", generator=generator)
        torch.cuda.synchronize()
        B.kcheck(l.b200_kv_cache_append(cache, k.data_ptr(), v.data_ptr(), chunk, stream))
        B.kcheck(l.b200_kv_cache_advance(handles, 1, chunk, stream))
        B.synchronize(local)
    lengths = np.random.default_rng(11 + rank).integers(cfg["min_context"], capacity + 1, size=n).astype(np.int32)
    B.kcheck(l.b200_kv_cache_set_lengths(cache, (lengths - 1).ctypes.data_as(C.POINTER(C.c_int32)), stream))
    q = torch.randn((n, heads, hd), device="cuda", generator=generator)
    out = torch.zeros((n, heads * hd), device="cuda")
    need = l.b200_attention_scratch_bytes(n, heads, kv_heads, hd, capacity, 64)
    scratch = torch.empty((need,), dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()

    def step():
        B.kcheck(l.b200_attention_decode(q.data_ptr(), n, 1, heads, cache, capacity, 1, scratch.data_ptr(), need, out.data_ptr(), stream))

    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(args.warmup):
        step()
    B.synchronize(local)
    barrier(dist, local)
    B.timer_start(local)
    for _ in range(args.steps):
        step()
    ms = max_over_ranks(B.timer_stop(local), dist, local)
    # host in the loop: q from pinned host memory every step, result read back
    q_host = q.cpu().pin_memory()
    out_host = torch.empty((n, heads * hd)).pin_memory()
    barrier(dist, local)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        q.copy_(q_host, non_blocking=True)
        torch.cuda.synchronize()
        step()
        B.synchronize(local)
        out_host.copy_(out, non_blocking=True)
        torch.cuda.synchronize()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1000.0, dist, local)
    clocks = sampler.stop()
    status = C.c_int32()
    B.kcheck(l.b200_take_device_status(local, stream, C.byref(status)))
    assert status.value == 0 and bool(torch.isfinite(out).all())
    l.b200_kv_cache_release(cache)
    bytes_per_step = float(lengths.astype(np.int64).sum()) * 2 * kv_heads * hd * 2
    peak, peak_kind = measured_peaks()
    achieved = bytes_per_step / (ms / args.steps / 1000.0) / 1e9
    line = {"metric": METRIC, "value": world * n * args.steps / (ms / 1000.0), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16 KV, f32 accumulate", "data": "synthetic",
            "config": {"workload": "c3 decode-attention microbench" + (" (small)" if args.small else ""), "batch_per_gpu": n, "heads": heads, "kv_heads": kv_heads,
                       "head_dim": hd, "mean_context": float(lengths.mean()), "l2": "inputs larger than L2: %.2f GB of K and V per step" % (bytes_per_step / 1e9)},
            "clocks": clocks,
            "e2e": {"value": world * n * args.steps / (e2e_ms / 1000.0), "unit": UNIT, "h2d_bytes_per_step": n * heads * hd * 4,
                    "d2h_bytes_per_step": n * heads * hd * 4, "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": 2 * args.steps,
            "roofline": {"bound": "hbm", "kernel": "attention_mma_kernel<128> (+ attention_combine_kernel)", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind, "traffic": None,
                         "algorithmic_bytes": bytes_per_step, "launch_ms": ms / args.steps}}
    del k, v, q, out, scratch
    torch.cuda.empty_cache()
    if dist is not None:
        dist.destroy_process_group()
    return line if rank == 0 else {}


def run_linear(args) -> dict:
    """One shadow linear in isolation (`--rows R --inner K --out N --epilogue store|residual|swiglu`): the skinny streaming
    kernel for up to 16 rows, the tcgen05 kernel above.  A step is one launch; the weights rotate through copies that
    together exceed L2, as they do inside a decode step of a model larger than L2."""
    import ctypes as C

    import torch

    import ctorch_b200 as B
    rank, world, local, dist = distributed()
    rows, inner, out = args.rows, args.inner, args.out
    epilogue = {"store": 0, "residual": 1, "swiglu": 2}[args.epilogue]
    l = B.lib()
    torch.cuda.set_device(local)
    stream = l.dl_b200_stream(B.cuda(local))
    generator = torch.Generator(device="cuda").manual_seed(5 + rank)
    copies = max(2, int(300e6 // (inner * out * 2)) + 1)
    weights = [(0.05 * torch.randn((out, inner), device="cuda", generator=generator)).to(torch.bfloat16) for _ in range(copies)]
    x = torch.randn((rows, inner), device="cuda", generator=generator)
    hi = torch.zeros((rows, inner), dtype=torch.bfloat16, device="cuda")
    lo = torch.zeros_like(hi)
    sq = torch.zeros((1, rows), device="cuda")
    torch.cuda.synchronize()   # torch filled these on its own stream; the library works on another
    B.kcheck(l.b200_shadow_from_rows(x.data_ptr(), rows, inner, None, 0, hi.data_ptr(), lo.data_ptr(), sq.data_ptr(), stream))
    columns = out // 2 if epilogue == 2 else out
    y = torch.zeros((rows, columns), device="cuda")
    residual = torch.zeros((rows, out), device="cuda")
    out_hi = torch.zeros((rows, columns), dtype=torch.bfloat16, device="cuda")
    out_lo = torch.zeros_like(out_hi)
    parts = l.b200_linear_shadow_parts(rows, inner, out)
    sums = torch.zeros((max(parts, 1), rows), device="cuda")
    torch.cuda.synchronize()

    def step(i):
        a = B.ShadowLinearArgs(hi.data_ptr(), lo.data_ptr(), rows, inner, weights[i % copies].data_ptr(), out, sq.data_ptr(), 1, 1e-5,
                               epilogue, residual.data_ptr() if epilogue == 1 else None, None, y.data_ptr(),
                               out_hi.data_ptr() if epilogue else None, out_lo.data_ptr() if epilogue else None, None, 0,
                               sums.data_ptr() if epilogue == 1 else None, None, None)
        B.kcheck(l.b200_linear_shadow(C.byref(a), stream))

    # One CUDA graph holds one launch per weight copy (as a decode step holds its launches in a graph: no host work per
    # launch); a timed step is one launch, so K steps are ceil(K / copies) replays.
    for i in range(min(args.warmup, copies)):
        step(i)
    B.synchronize(local)
    side = torch.cuda.ExternalStream(stream, device=torch.device("cuda", local))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for i in range(copies):
            step(i)
    replays = (args.steps + copies - 1) // copies
    launches = replays * copies
    sampler = ClockSampler(local)
    sampler.start()
    with torch.cuda.stream(side):   # replays go to the library's stream, where the timer's events are recorded
        graph.replay()
        B.synchronize(local)
        barrier(dist, local)
        B.timer_start(local)
        for _ in range(replays):
            graph.replay()
        elapsed = B.timer_stop(local)
    ms = max_over_ranks(elapsed, dist, local) * args.steps / launches   # scaled to K launches
    clocks = sampler.stop()
    status = C.c_int32()
    B.kcheck(l.b200_take_device_status(local, stream, C.byref(status)))
    want = x @ weights[copies - 1].float().T * torch.rsqrt((x * x).mean(dim=1, keepdim=True) + 1e-5)
    if epilogue == 2:
        want = torch.nn.functional.silu(want[:, 0::2]) * want[:, 1::2]
    error = float((y - want).abs().max() / want.abs().max())
    assert status.value == 0 and error < 1e-3, (status.value, error, float(y.abs().max()), float(want.abs().max()))
    seconds = ms / args.steps / 1000.0
    weight_bytes = inner * out * 2
    flops = 2.0 * rows * inner * out
    peak, peak_kind = measured_peaks()
    hbm_bound = rows <= 512   # arithmetic intensity rows flop/B against a ridge of ~220: decode batches stream weights
    tensor_peak = tensor_peak_tflops()
    roofline = ({"bound": "hbm", "achieved": weight_bytes / seconds / 1e9, "peak": peak, "unit": "GB/s", "peak_kind": peak_kind,
                 "algorithmic_bytes": weight_bytes}
                if hbm_bound else
                {"bound": "tensor", "achieved": flops / seconds / 1e12, "peak": tensor_peak, "unit": "TFLOP/s", "peak_kind": "measured burst",
                 "algorithmic_flops": flops, "note": "useful flops; the kernel issues twice as many (activation hi + lo planes)"})
    roofline.update(frac=roofline["achieved"] / roofline["peak"], traffic=None,
                    kernel="linear_stream_kernel" if rows <= 16 and inner <= 2048 else "linear_gemm_kernel", launch_ms=ms / args.steps)
    line = {"metric": "linear_rows_per_s", "value": world * rows / seconds, "unit": "rows/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16 weights, f32 activations as bf16 hi+lo, f32 accumulate", "data": "synthetic",
            "config": {"workload": f"linear microbench rows {rows} in {inner} out {out} {args.epilogue}", "copies": copies,
                       "l2": "weights rotate through %d copies (%.0f MB) > L2" % (copies, copies * weight_bytes / 1e6), "max_rel_error": error},
            "clocks": clocks, "gpu_launches": args.steps, "roofline": roofline}
    if dist is not None:
        dist.destroy_process_group()
    return line if rank == 0 else {}


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--workload", default="c4", choices=["c1", "c2", "c3", "c4", "c5", "linear"])
    parser.add_argument("--activations", default="f32", choices=["f32", "bf16"],
                        help="bf16 decoders: precision of the activations between kernels in passes over more than 16 rows")
    parser.add_argument("--batch", type=int, default=0, help="decoder workloads: override the configuration's batch (e.g. c4 with 32 = one GPU's share of the 8-GPU run)")
    parser.add_argument("--rows", type=int, default=16, help="linear only")
    parser.add_argument("--inner", type=int, default=768, help="linear only")
    parser.add_argument("--out", type=int, default=32000, help="linear only")
    parser.add_argument("--epilogue", default="store", choices=["store", "residual", "swiglu"], help="linear only")
    parser.add_argument("--cpu-steps", type=int, default=4, help="timed CPU-baseline steps of the default run")
    parser.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    parser.add_argument("--no-secondary", action="store_true", help="c4 on one GPU: skip the c3 and c2 companions of the record")
    parser.add_argument("--small", action="store_true", help="c3 only: batch 16, contexts up to 8192 (profiler captures)")
    args = parser.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.workload in ("c3", "linear"):
        line = run_c3(args) if args.workload == "c3" else run_linear(args)
        if line:
            print(json.dumps(line))
        return
    spec = dict(W.CONFIGS[args.workload])
    if args.batch > 0:
        spec["batch"] = args.batch
    if args.impl == "reference" and int(os.environ.get("RANK", "0")) != 0:
        return   # the CPU arm runs on rank 0 alone
    weights = W.make_weights(spec)
    line = run_reference(args, spec, weights) if args.impl == "reference" else run_b200(args, spec, weights)
    if line:
        print(json.dumps(line))


if __name__ == "__main__":
    main()
