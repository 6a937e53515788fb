"""Benchmark of the sampling path: rows/s of one decode step's sampling on synthetic logits.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one pass of the sampler over one batch of logits (one call of the library's
leat_sample on resident inputs).  N = 1 runs the batched server decode step (16 rows, 151936
tokens: per-row temperature, top-k 64, min-p, presence/frequency/repetition penalties over a
1024-token history); the logits of successive steps come from a pool of buffers larger than L2, so
every step reads HBM.  N > 1 (under torchrun) runs the vocabulary-sharded configuration (512 rows,
201088 tokens split over the ranks, one all-gather of candidates per step).  The last line printed
by rank 0 is one JSON object; `all_configs` in it holds the device-timed figures of every
configuration at one GPU.

--impl reference times the CPU restatement of leat's exact sampler (oracle/) on the host's cores
for the same workload: leat itself needs tinygrad, which is not installed here, so its own code
cannot be run.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_HBM_GBS = 6650.0  # an earlier measurement on this pool, used when MEASURED_PEAKS.json is absent
NORTH_STAR_HBM_GBS = 8000.0
L2_BYTES = 126 << 20
# DRAM bytes filter_kernel moved per algorithmic byte in the ncu capture summarised in
# profiles/filter_path_c3_160rows.md: (dram__bytes_read.sum + dram__bytes_write.sum) / (B x V x 4)
# = (167.79 + 3.37) MB / 167.77 MB on 160 rows of the large-batch configuration; traffic grows with
# the rows and the vocabulary, so it is scaled to the launch being reported
TRAFFIC_PER_ALGORITHMIC_BYTE = 1.02


def peak_hbm() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except (ValueError, KeyError):
            pass
    return FALLBACK_HBM_GBS, "fallback"


# ---- clocks -------------------------------------------------------------------------------------


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while a timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")  # fmt: skip

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.thread = index, [], None, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)  # fmt: skip
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def keep_busy(self, step, seconds: float = 0.6, wanted: int = 3) -> None:
        """The timed steps last milliseconds and nvidia-smi answers every 100 ms: the same steps go
        on, untimed, until a few samples are in (or `seconds` are over, whichever comes last, at most
        five times that), so that the clocks are seen under the load that was timed."""
        import torch

        start, i = time.perf_counter(), 0
        while True:
            for _ in range(16):
                step(i)
                i += 1
            torch.cuda.synchronize()
            spent = time.perf_counter() - start
            if (spent >= seconds and len(self.rows) >= wanted) or spent >= 5 * seconds:
                return

    def summary(self) -> dict:
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        top = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 9 for n, v in zip(names, r[5:9]) if v.lower().startswith("active")})
        busy = [x for x in sm if x > 0.5 * max(sm)] if sm else []
        return {"sm_mhz": float(np.median(busy)) if busy else None, "sm_max_mhz": max(top) if top else None,
                "reasons": reasons, "samples": len(sm)}  # fmt: skip


# ---- CPU baseline (the oracle on the host's cores) ------------------------------------------------


def cpu_step_seconds(w, mode: str, pool: ThreadPoolExecutor) -> float:
    """Seconds the CPU oracle takes for one pass over the rows of `w`, one row per pool task
    (NumPy releases the GIL in its sorts)."""
    from oracle import sampler_oracle as oracle

    def one(b: int) -> int:
        sel = slice(b, b + 1)
        oracle.sample(w.logits[sel], w.options[sel], w.seed[sel], w.position[sel],
                      history=None if w.history is None else w.history[sel],
                      penalties=None if w.penalties is None else w.penalties[sel],
                      uniform_draws=w.uniform[sel] if mode == "U" else None, survivors=False)  # fmt: skip
        return 1

    start = time.perf_counter()
    sum(pool.map(one, range(w.rows)))
    return time.perf_counter() - start


def cpu_rows_per_second(w, mode: str, seconds: float, threads: int) -> tuple[float, str]:
    """Rows per second of the CPU oracle over whole passes of `w` for about `seconds`."""
    passes, spent = 0, 0.0
    with ThreadPoolExecutor(threads) as pool:
        while spent < seconds:
            spent += cpu_step_seconds(w, mode, pool)
            passes += 1
    return passes * w.rows / spent, f"{passes} passes over {w.rows} rows x {w.vocab} of {w.name} in {spent:.1f} s"


def run_reference(args) -> None:
    from leat_b200 import workloads

    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    config = 2 if int(os.environ.get("WORLD_SIZE", 1)) == 1 else 5
    # a step is one pass over a bounded sample of the workload's rows
    w = workloads.config2() if config == 2 else workloads.config5(rows=32)
    threads = os.cpu_count() or 1
    times = []
    with ThreadPoolExecutor(threads) as pool:
        for step in range(args.warmup + args.steps):
            seconds = cpu_step_seconds(w, "U", pool)
            if step >= args.warmup:
                times.append(seconds)
    value = w.rows / float(np.mean(times))
    sample = f"{args.steps} steps of {w.rows} rows x {w.vocab} of {WORKLOAD_NAMES[config]}, one row per task on {threads} threads"
    line = {
        "impl": "reference", "metric": "sampler rows/s", "value": value, "unit": "rows/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * SHAPES_ROWS[config] / value,
        "higher_is_better": True, "scaling": "weak" if config == 2 else "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD_NAMES[config], "rows": SHAPES_ROWS[config], "vocab": w.vocab, "draw": "supplied uniform"},
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "leat's own sampler needs tinygrad (not installed, no network): this is the NumPy restatement of "
                "its exact path (LEAT_KERNELS=ref) on the host cores",
    }  # fmt: skip
    print(json.dumps(line), flush=True)


WORKLOAD_NAMES = {1: "c1_single_row", 2: "c2_server_step", 3: "c3_large_batch", 4: "c4_draft_verify", 5: "c5_vocab_sharded"}
SHAPES_ROWS = {1: 1, 2: 16, 3: 256, 4: 72, 5: 512}


# ---- the GPU arm ---------------------------------------------------------------------------------


class DeviceWorkload:
    """A workload resident in HBM, its logits replicated into a pool larger than L2."""

    def __init__(self, w, device, min_pool_bytes=2 * L2_BYTES, max_copies=512, dtype=None):
        import torch

        self.w, self.device = w, device
        self.logit_bytes = w.logit_bytes if dtype is None else w.logit_bytes // 2
        copies = int(min(max_copies, max(1, -(-min_pool_bytes // self.logit_bytes))))
        base = torch.as_tensor(w.logits).to(device)
        if dtype is not None:  # the lm_head's own 16-bit output, read as it is
            base = base.to(dtype)
        self.pool = [base] + [base.clone() for _ in range(copies - 1)]
        t = lambda x: None if x is None else torch.as_tensor(x).to(device)  # noqa: E731
        self.options, self.penalties, self.history = t(w.options), t(w.penalties), t(w.history)
        self.uniform, self.position = t(w.uniform), t(w.position)
        self.seed = torch.as_tensor(w.seed.astype(np.int64)).to(device).to(torch.uint32)
        self.out = torch.empty((w.rows, 1), dtype=torch.int32, device=device)
        self.l2_note = ("logits pool of %d buffers (%.0f MB) cycled, larger than L2" % (copies, copies * self.logit_bytes / 1e6)
                        if copies > 1 else "inputs larger than L2")  # fmt: skip

    def step(self, sampler, i: int):
        return sampler.sample_full(self.pool[i % len(self.pool)], self.options, self.seed, self.position,
                                   history=self.history, penalties=self.penalties, uniform=self.uniform, out=self.out)  # fmt: skip


def time_device(step, steps: int, warmup: int) -> float:
    """Mean milliseconds per step over `steps` steps, CUDA events on the launching stream."""
    import torch

    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(steps):
        step(warmup + i)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


def time_graph(step, steps: int, warmup: int, inner: int) -> float:
    """Mean milliseconds per step with `inner` steps captured in one CUDA graph (launch overhead
    of the host taken out, as in leat's engine, which replays captured graphs)."""
    import torch

    for i in range(max(warmup, 3)):
        step(i)
    torch.cuda.synchronize()
    graph, stream = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            for i in range(inner):
                step(i)
    torch.cuda.synchronize()
    replays = max(1, steps // inner)
    graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(replays):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / (replays * inner)


def kernel_milliseconds(sampler, dw, steps: int = 12) -> dict:
    """Median duration of each kernel of a step, from CUDA events the library records on the
    launching stream around its launches (plain launches, one step per pool buffer)."""
    sampler.time_kernels(True)
    rows = []
    for i in range(steps + 3):
        dw.step(sampler, i)
        rows.append(sampler.kernel_times())
    sampler.time_kernels(False)
    floor_ms, filter_ms, finish_ms = np.median(np.array(rows[3:]), axis=0)
    return {"floor_kernel": float(floor_ms), "filter_kernel": float(filter_ms), "sample_kernel": float(finish_ms)}


def run_one(args) -> None:
    """One configuration, a few Python-launched steps: the command ncu captures are taken from."""
    import torch

    from leat_b200 import workloads
    from leat_b200.sampler import Sampler

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    kw = {"rows": args.rows} if args.rows and args.workload != 4 else {}
    w = workloads.CONFIGS[args.workload](**kw)
    sampler = Sampler(max(w.rows, 8), w.vocab, 256, device)
    dw = DeviceWorkload(w, device, min_pool_bytes=0, max_copies=1)
    ms = time_device(lambda i: dw.step(sampler, i), args.steps, args.warmup)
    print(json.dumps({"workload": WORKLOAD_NAMES[args.workload], "rows": w.rows, "vocab": w.vocab, "ms_per_step": ms,
                      "launch": dict(zip(("threads", "slices", "shared_bytes"),
                                         sampler.plan(w.rows, w.vocab, 0 if w.history is None else w.history.shape[1]))),
                      "kernels_per_step": sampler.last_launches}), flush=True)


def run_single(args) -> None:
    import torch

    from leat_b200 import workloads
    from leat_b200.sampler import Sampler

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    peak, peak_kind = peak_hbm()
    sampler = Sampler(512, 262144, 256, device)

    # every configuration, device-timed under graph replay (kernel figures)
    all_configs = {}
    for number, dtype in ((1, None), (2, None), (3, None), (4, None), (5, None), (3, torch.bfloat16)):
        w = workloads.CONFIGS[number]()
        dw = DeviceWorkload(w, device, dtype=dtype)
        ms = time_graph(lambda i, dw=dw: dw.step(sampler, i), steps=max(args.steps, 2 * len(dw.pool)),
                        warmup=args.warmup, inner=len(dw.pool))  # fmt: skip
        gbs = dw.logit_bytes / (ms * 1e-3) / 1e9
        kernels = kernel_milliseconds(sampler, dw)
        filter_gbs = dw.logit_bytes / (kernels["filter_kernel"] * 1e-3) / 1e9 if kernels["filter_kernel"] > 0 else None
        all_configs[WORKLOAD_NAMES[number] + ("" if dtype is None else "_bf16_logits")] = {
            "rows": w.rows, "vocab": w.vocab, "us_per_step": round(ms * 1e3, 2), "rows_per_s": round(w.rows / (ms * 1e-3)),
            "hbm_gbs": round(gbs, 1), "frac_of_measured": round(gbs / peak, 4), "frac_of_8tbs": round(gbs / NORTH_STAR_HBM_GBS, 4),
            "kernel_us": {k: round(v * 1e3, 2) for k, v in kernels.items()},
            "filter_kernel_gbs": None if filter_gbs is None else round(filter_gbs, 1),
            "filter_kernel_frac_of_measured": None if filter_gbs is None else round(filter_gbs / peak, 4),
        }  # fmt: skip
        del dw
        torch.cuda.empty_cache()

    # the headline workload: the batched server decode step
    w = workloads.config2()
    dw = DeviceWorkload(w, device)
    with ClockSampler(0) as clocks:
        inner = len(dw.pool)
        steps = max(inner, args.steps // inner * inner)
        ms = time_graph(lambda i: dw.step(sampler, i), steps, args.warmup, inner)
        launches = sampler.last_launches * steps
        clocks.keep_busy(lambda i: dw.step(sampler, i))
        # end to end: host logits in pinned memory, copied in every step; ids read back every step
        from leat_b200 import sample as public_sample

        host_logits = torch.as_tensor(w.logits).pin_memory()
        host_ids = torch.empty((w.rows, 1), dtype=torch.int32).pin_memory()
        staging = torch.empty_like(dw.pool[0])

        def e2e_step(i):
            staging.copy_(host_logits, non_blocking=True)
            ids = public_sample(staging, dw.options, dw.seed, dw.position, history=dw.history,
                                penalties=dw.penalties, uniform=dw.uniform)  # fmt: skip
            host_ids.copy_(ids, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        ms_e2e = time_device(e2e_step, args.steps, args.warmup)
        kernels = kernel_milliseconds(sampler, dw)
    value = w.rows / (ms * 1e-3)
    # the kernel that moves the bytes is filter_kernel: every logit once
    achieved = w.logit_bytes / (kernels["filter_kernel"] * 1e-3) / 1e9
    step_achieved = w.logit_bytes / (ms * 1e-3) / 1e9
    traffic = None if TRAFFIC_PER_ALGORITHMIC_BYTE is None else TRAFFIC_PER_ALGORITHMIC_BYTE * w.logit_bytes
    large = all_configs[WORKLOAD_NAMES[3]]

    threads = os.cpu_count() or 1
    cpu_value, cpu_sample = cpu_rows_per_second(w, "U", seconds=12.0, threads=threads)
    line = {
        "metric": "sampler rows/s", "value": value, "unit": "rows/s", "n_gpus": 1, "steps": steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD_NAMES[2], "rows": w.rows, "vocab": w.vocab, "draw": "supplied uniform",
                   "l2": dw.l2_note,
                   "timing": "CUDA events around replays of a CUDA graph that holds one step per pool buffer"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic, "peak_kind": peak_kind, "kernel": "filter_kernel",
                     "algorithmic_bytes_per_launch": w.logit_bytes,
                     "launch_us": kernels["filter_kernel"] * 1e3,
                     "kernel_us": {k: v * 1e3 for k, v in kernels.items()},
                     "whole_step": {"achieved": step_achieved, "frac": step_achieved / peak,
                                    "note": "all three launches of a step under graph replay"},
                     "large_batch": {"workload": WORKLOAD_NAMES[3], "rows": large["rows"], "vocab": large["vocab"],
                                     "filter_kernel_gbs": large["filter_kernel_gbs"],
                                     "filter_kernel_frac": large["filter_kernel_frac_of_measured"],
                                     "whole_step_gbs": large["hbm_gbs"], "whole_step_frac": large["frac_of_measured"]}},
        "cpu_baseline": {"value": cpu_value, "unit": "rows/s", "cores": threads, "kind": "port", "sample": cpu_sample},
        "e2e": {"value": w.rows / (ms_e2e * 1e-3), "unit": "rows/s", "h2d_bytes_per_step": w.logit_bytes,
                "d2h_bytes_per_step": w.rows * 4},
        "gpu_launches": launches, "clocks": clocks.summary(), "all_configs": all_configs,
        "us_per_step_b1": all_configs[WORKLOAD_NAMES[1]]["us_per_step"],
    }  # fmt: skip
    print(json.dumps(line), flush=True)


def run_sharded(args) -> None:
    import torch
    import torch.distributed as dist

    from leat_b200 import workloads
    from leat_b200.sharded import ShardedSampler

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", device_id=device)
    peak, peak_kind = peak_hbm()
    w = workloads.config5()
    sharded = ShardedSampler(w.rows, w.vocab, k_max=64, cap=128, device=device)
    start, stop = sharded.start, sharded.stop
    t = lambda x: None if x is None else torch.as_tensor(x).to(device)  # noqa: E731
    copies = max(1, -(-2 * L2_BYTES // ((stop - start) * w.rows * 4)))
    base = torch.as_tensor(np.ascontiguousarray(w.logits[:, start:stop])).to(device)
    pool = [base] + [base.clone() for _ in range(min(copies, 32) - 1)]
    options, penalties, history, uniform, position = t(w.options), t(w.penalties), t(w.history), t(w.uniform), t(w.position)
    seed = torch.as_tensor(w.seed.astype(np.int64)).to(device).to(torch.uint32)
    out = torch.empty((w.rows, 1), dtype=torch.int32, device=device)

    def step(i):
        return sharded.sample(pool[i % len(pool)], options, seed, position, history=history, penalties=penalties,
                              uniform=uniform, out=out)  # fmt: skip

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    # the two device steps are replayed from CUDA graphs (one select graph per pool buffer, one finish
    # graph), as a serving engine that replays captured decode steps would run them; the all-gather
    # between them is issued eagerly
    side = torch.cuda.Stream()
    selects, finish = [], torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        for buffer in pool:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                sharded.select(buffer, options, seed, position, history, None, penalties, uniform)
            selects.append(g)
        with torch.cuda.graph(finish, stream=side):
            sharded.finish(w.rows, options, seed, position, uniform, out=out)
    torch.cuda.synchronize()

    def graph_step(i):
        selects[i % len(selects)].replay()
        sharded.exchange(w.rows)
        finish.replay()

    for i in range(3):
        graph_step(i)
    torch.cuda.synchronize()
    steps = args.steps
    dist.barrier()
    torch.cuda.synchronize()
    with ClockSampler(local) as clocks:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(steps):
            graph_step(i)
        b.record()
        torch.cuda.synchronize()
        ms = torch.tensor([a.elapsed_time(b) / steps], device=device)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        ms = float(ms.item())
        # the timed steps last milliseconds and nvidia-smi answers every 100 ms: the same steps go on,
        # untimed, for about 0.6 s (the same number on every rank: each holds a collective)
        for i in range(min(50000, int(600.0 / max(ms, 1e-3)))):
            graph_step(i)
        torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    # end to end: this rank's slice comes from pinned host memory every step, the ids go back
    host_slice = torch.as_tensor(np.ascontiguousarray(w.logits[:, start:stop])).pin_memory()
    host_ids = torch.empty((w.rows, 1), dtype=torch.int32).pin_memory()

    def e2e_step(i):
        pool[0].copy_(host_slice, non_blocking=True)
        result = sharded.sample(pool[0], options, seed, position, history=history, penalties=penalties, uniform=uniform, out=out)
        host_ids.copy_(result.ids, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for i in range(3):
        e2e_step(i)
    dist.barrier()
    torch.cuda.synchronize()
    a.record()
    for i in range(args.steps):
        e2e_step(i)
    b.record()
    torch.cuda.synchronize()
    ms_e2e = torch.tensor([a.elapsed_time(b) / args.steps], device=device)
    dist.all_reduce(ms_e2e, op=dist.ReduceOp.MAX)
    ms_e2e = float(ms_e2e.item())
    if rank == 0:
        achieved = w.logit_bytes / world / (ms * 1e-3) / 1e9  # per GPU: each reads its slice once
        line = {
            "metric": "sampler rows/s", "value": w.rows / (ms * 1e-3), "unit": "rows/s", "n_gpus": world,
            "steps": steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD_NAMES[5], "rows": w.rows, "vocab": w.vocab, "parallelism": f"vocab{world}",
                       "draw": "supplied uniform", "l2": f"logits pool of {len(pool)} buffers per rank cycled, larger than L2",
                       "exchange": "one NCCL all-gather of packed (score, id, count, greedy) candidate records per step",
                       "timing": "CUDA events around the timed steps; the two device steps replayed from CUDA graphs, the all-gather issued eagerly between them; max over ranks"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_kind": peak_kind, "kernel": "whole step per GPU (floor, filter, candidates, all-gather, finish) over its vocabulary slice",
                         "algorithmic_bytes_per_launch": w.logit_bytes // world},
            "e2e": {"value": w.rows / (ms_e2e * 1e-3), "unit": "rows/s", "h2d_bytes_per_step": int(host_slice.numel() * 4) * world,
                    "d2h_bytes_per_step": w.rows * 4 * world},
            "gpu_launches": 5 * steps, "clocks": clocks.summary(),  # floor, filter, candidates, second pass, finish
        }  # fmt: skip
        print(json.dumps(line), flush=True)
    del selects, finish
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", type=int, default=0, choices=[0, 1, 2, 3, 4, 5],
                        help="profiling aid: time only this configuration, launched from Python, and print a short line")
    parser.add_argument("--rows", type=int, default=0, help="with --workload: fewer rows than the configuration has")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.workload:
        run_one(args)
    elif args.impl == "reference":
        run_reference(args)
    elif int(os.environ.get("WORLD_SIZE", 1)) > 1:
        run_sharded(args)
    else:
        run_single(args)


if __name__ == "__main__":
    main()
