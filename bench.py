"""Benchmark of the paged KV-cache decode path: one step = append one new K/V row per sequence, then
flash-decoding attention of one query per sequence over its whole paged context (one layer) -- ONE kernel launch
(llaisysPagedDecodeStepDev).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload north_star|config2|...]

Prints ONE JSON line (rank 0). With N > 1 it is launched under torch.distributed.run, one rank per GPU; whole
sequences are sharded across ranks, each rank owns its page pool, and there is no data-path collective
(weak scaling: per-GPU work is fixed).

Workloads (synthetic, seeded, N(0,1) bf16; 12 query / 2 kv heads, head_dim 128, 16-token pages, physical pages a
random permutation of a 16384-page pool):
  north_star  64 sequences x 4096-token context -- the shape the target "paged decode attention sustaining
              >= 70 % of HBM peak" is quoted on; uses the whole pool (256 MiB per layer)
  config2     32 sequences, context ~ U{128..4096}
  config3     chunked prefill: 8 sequences, context ~ U{0..8192}, a 512-token chunk appended and attended causally
  config5     one 131072-token sequence, 28 layers, KV range split over the GPUs, partial results exchanged and merged
The default run (north_star) also measures config2 and config3 in the same process (N = 1: sub-records "config2",
"config3") and, with N > 1, the KV-range split of config5 in the same process group (sub-record "kv_split"): the one
mode of this path in which GPUs exchange data.

Numbers:
  value      tokens/s of the step with inputs resident in HBM, device-timed: a CUDA graph of K steps is replayed R >= 30
             times with an event pair around every replay; value uses the MEDIAN replay, min and max are reported;
             max over ranks
  roofline   achieved HBM GB/s of the step kernel = algorithmic bytes / its launch-to-launch period in that graph
             (consecutive launches overlap by programmatic dependent launch); the same kernel launched without overlap
             and the decode-only / append-only kernels are timed beside it
  e2e        same step through the host-buffer C-ABI call with host<->device copies of q, k, v, out in the
             timed region, wall clock bracketed by device synchronisation
  cpu_baseline / --impl reference   the reference's CPU definition of the path (oracle port of its PyTorch
             torch_self_attention) on a bounded sample of the same workload, all host threads; the library's own
             plain-C++ CPU backend of llaisysSelfAttention is timed beside it
Between timed steps the layer rotates over pools that together exceed L2 several times, so K/V always comes
from HBM.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

NH, NKVH, D, PAGE, POOL_PAGES = 12, 2, 128, 16, 16384
METRIC = "decode tokens/s (paged KV append + flash-decoding attention, one layer)"
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the step kernel (mean of two captured launches), from
# `ncu --set full -k regex:paged_decode_tma -s 4 -c 2` over `bench.py --quick --steps 3 --warmup 3 --layers 2
# [--workload config2]`: a profiler reading, taken once per kernel change, not measured by this run.
NCU_TRAFFIC_BYTES = {"north_star": 273_638_912, "config2": 73_196_160}
MIN_REPEATS = 30


def workload_lengths(name: str, seed: int):
    import torch

    g = torch.Generator().manual_seed(seed)
    if name == "north_star":
        return [4096] * 64
    if name == "config2":
        return torch.randint(128, 4097, (32,), generator=g).tolist()
    raise SystemExit(f"unknown workload {name}")


def algorithmic_bytes(ctx: list[int], with_append: bool = False) -> int:
    """Bytes one decode launch must move: K and V read once, q read, out written, block-table entries; the one-launch
    step also reads the new K/V rows and writes them into their pages."""
    b = len(ctx)
    total = sum(ctx) * (2 * NKVH * D * 2) + 2 * b * NH * D * 2 + 4 * sum(-(-c // PAGE) for c in ctx)
    if with_append:
        total += 2 * b * (2 * NKVH * D * 2)
    return total


def decode_config(workload: str, ctx: list[int], world: int, layers: int, overlap: bool) -> dict:
    """The `config` object of the decode workloads; both arms (this library and --impl reference) print the same one."""
    return {"workload": workload, "batch_per_gpu": len(ctx), "context": f"{min(ctx)}..{max(ctx)}",
            "heads": "12q/2kv", "head_dim": D, "page_size": PAGE, "pool_pages": POOL_PAGES,
            "parallelism": f"sequences sharded over {world} GPU(s), no collective",
            "l2": f"inputs larger than L2: layer pool rotates over {layers} x {POOL_PAGES * PAGE * 1024 >> 20} MiB between steps",
            "launch": ("programmatic dependent launch: a kernel's set-up and first K/V copies overlap the previous "
                       "kernel's tail") if overlap else "plain"}


def spread(samples: list[float], scale: float = 1.0) -> dict:
    """median / min / max of a list of timings (already divided by `scale` units each)."""
    xs = [x / scale for x in samples]
    return {"median": statistics.median(xs), "min": min(xs), "max": max(xs), "n": len(xs)}


class ClockSampler:
    """Samples the SM clock and the throttle reasons through NVML (read-only queries) about once a millisecond
    while the timed region runs."""

    REASONS = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, index: int, period_s: float = 0.001):
        self.index, self.period, self.sm, self.bits, self.max_mhz = index, period_s, [], 0, None
        self.stop = threading.Event()
        self.thread = None
        self.error = None

    def __enter__(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            uuid = None
            try:  # CUDA_VISIBLE_DEVICES may renumber devices; match the CUDA device by UUID
                import torch

                uuid = str(torch.cuda.get_device_properties(self.index).uuid)
            except Exception:
                pass
            handle = None
            if uuid:
                for cand in (uuid, "GPU-" + uuid):
                    try:
                        handle = pynvml.nvmlDeviceGetHandleByUUID(cand.encode())
                        break
                    except Exception:
                        continue
            if handle is None:
                handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))

            def loop():
                while not self.stop.is_set():
                    try:
                        self.sm.append(float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)))
                        self.bits |= int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle))
                    except Exception as exc:  # keep the bench alive; report the failure in the JSON
                        self.error = repr(exc)
                        return
                    time.sleep(self.period)

            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
        except Exception as exc:
            self.error = repr(exc)
        return self

    def __exit__(self, *exc):
        self.stop.set()
        if self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        if not self.sm:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [f"no samples: {self.error}"]}
        reasons = sorted(name for name, bit in self.REASONS.items() if self.bits & bit)
        return {"sm_mhz": statistics.median(self.sm), "sm_min_mhz": min(self.sm), "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(self.sm)}


def host_threads() -> int:
    return len(os.sched_getaffinity(0))


def cpu_sample(ctx: list[int], seed: int, max_seqs: int):
    """The bounded CPU sample of a decode workload: the first max_seqs sequences, contiguous bf16 K/V, one query each."""
    import torch

    from oracle import workloads

    g = torch.Generator().manual_seed(seed)
    sample = ctx[:max_seqs]
    qs = [workloads.randn((1, NH, D), torch.bfloat16, g) for _ in sample]
    ks = [workloads.randn((c, NKVH, D), torch.bfloat16, g) for c in sample]
    vs = [workloads.randn((c, NKVH, D), torch.bfloat16, g) for c in sample]
    return sample, qs, ks, vs


def reference_cpu_rate(ctx: list[int], seed: int, min_seconds: float, max_seqs: int):
    """Times the oracle port of the reference's torch_self_attention (reference: test/ops/self_attention.py:11-28),
    one call per sequence on contiguous bf16 K/V, on a bounded sample of the workload. -> tokens/s, seconds, description, threads"""
    import torch

    from oracle import attention

    torch.set_num_threads(host_threads())
    sample, qs, ks, vs = cpu_sample(ctx, seed, max_seqs)
    scale = 1.0 / D ** 0.5
    attention.self_attention(qs[0], ks[0], vs[0], scale)  # warm-up
    done, t0 = 0, time.perf_counter()
    while True:
        for q, k, v in zip(qs, ks, vs):
            attention.self_attention(q, k, v, scale)
        done += len(sample)
        dt = time.perf_counter() - t0
        if dt >= min_seconds:
            break
    desc = (f"{len(sample)} of {len(ctx)} sequences (ctx {sample[0]}..), {done // len(sample)} passes, "
            f"{dt:.1f} s, torch {torch.__version__}")
    return done / dt, dt, desc, torch.get_num_threads()


def cpp_backend_cpu_rate(ctx: list[int], seed: int, min_seconds: float, max_seqs: int) -> dict:
    """The same sample through the library's own CPU backend of llaisysSelfAttention (plain C++ loops, OpenMP over
    query heads): what a CPU-only build of the reference's operator interface runs. -> record for cpu_baseline"""
    import llaisys_b200 as llaisys
    from tests import helpers

    cpu = llaisys.DeviceType.CPU
    sample, qs, ks, vs = cpu_sample(ctx, seed, max_seqs)
    scale = 1.0 / D ** 0.5
    tensors = [tuple(helpers.to_llaisys(t, cpu, "bf16") for t in (q, k, v)) for q, k, v in zip(qs, ks, vs)]
    outs = [llaisys.Tensor((1, NH, D), dtype=llaisys.DataType.BF16, device=cpu) for _ in sample]
    llaisys.Ops.self_attention(outs[0], *tensors[0], scale)
    done, t0 = 0, time.perf_counter()
    while True:
        for o, (q, k, v) in zip(outs, tensors):
            llaisys.Ops.self_attention(o, q, k, v, scale)
        done += len(sample)
        dt = time.perf_counter() - t0
        if dt >= min_seconds:
            break
    threads = int(os.environ.get("OMP_NUM_THREADS") or host_threads())
    return {"value": done / dt, "unit": "tokens/s", "cores": threads, "kind": "llaisys_b200 CPU backend (C++, OpenMP)",
            "sample": f"{len(sample)} of {len(ctx)} sequences, {done // len(sample)} passes, {dt:.1f} s"}


def run_reference_arm(args) -> None:
    """--impl reference: the reference's own CPU definition of the path on the host cores, rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # launchers such as torch.distributed.run export OMP_NUM_THREADS=1; the CPU arm is meant to use the whole host
    os.environ["OMP_NUM_THREADS"] = str(host_threads())
    if args.workload == "config4":
        rate, threads, sample = model_cpu_rate(QWEN2_1P5B, 20.0)
        print(json.dumps({
            "impl": "reference", "metric": "decode tokens/s (Qwen2-1.5B architecture, greedy, paged KV cache)",
            "value": rate, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1e3 / rate, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": {"workload": "config4", "batch": 64},
            "cpu_baseline": {"value": rate, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": rate, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}), flush=True)
        return
    if args.workload not in ("north_star", "config2"):
        print(json.dumps({"impl": "reference", "unavailable":
                          f"the CPU arm covers north_star, config2 and config4; {args.workload} has no bounded CPU sample"}),
              flush=True)
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    ctx = workload_lengths(args.workload, seed=2)
    per_step = max(1, min(4, len(ctx)))
    args.steps = min(args.steps, 200)  # bounded: the CPU arm needs seconds per step, not microseconds
    import torch

    from oracle import attention

    torch.set_num_threads(host_threads())
    sample, qs, ks, vs = cpu_sample(ctx, 2, per_step)
    scale = 1.0 / D ** 0.5
    threads = torch.get_num_threads()
    times = []
    for step in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        for q, k, v in zip(qs, ks, vs):
            attention.self_attention(q, k, v, scale)
        if step >= args.warmup:
            times.append(time.perf_counter() - t0)
    total = sum(times)
    value = per_step * len(times) / total
    desc = (f"each step = the first {per_step} of the workload's {len(ctx)} sequences (ctx {sample}), bf16, contiguous K/V, "
            f"oracle port of torch_self_attention, torch {torch.__version__}; tokens/s does not depend on how many of the "
            "equal-length sequences a step holds")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": decode_config(args.workload, ctx, world, args.layers, not args.no_overlap),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def _init_device():
    """Per-rank device set-up shared by every workload. -> torch, llaisys, rank, local_rank, world, dist"""
    import torch

    import llaisys_b200 as llaisys

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU stand-in")
    torch.cuda.set_device(local_rank)
    llaisys.set_context_runtime(llaisys.DeviceType.NVIDIA, local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    return torch, llaisys, rank, local_rank, world, dist


def _peaks():
    """-> HBM GB/s, bf16 TFLOP/s burst, bf16 TFLOP/s sustained, "measured" | "fallback" """
    peaks_file = ROOT / "MEASURED_PEAKS.json"
    if peaks_file.exists():
        d = json.loads(peaks_file.read_text())
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), float(d["bf16_tflops_sustained"]), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


def replay_times(torch, stream, graph, repeats: int) -> list[float]:
    """Replays a captured graph `repeats` times with an event pair around every replay -> milliseconds per replay."""
    events = [torch.cuda.Event(enable_timing=True) for _ in range(repeats + 1)]
    with torch.cuda.stream(stream):
        graph.replay()  # untimed: the first replay uploads the graph
        events[0].record(stream)
        for r in range(repeats):
            graph.replay()
            events[r + 1].record(stream)
    stream.synchronize()
    return [events[r].elapsed_time(events[r + 1]) for r in range(repeats)]


def reduce_max(torch, dist, values: list[float]) -> list[float]:
    if dist is None:
        return values
    t = torch.tensor(values, device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t]


def measure_decode(env, workload: str, args, *, steps: int, repeats: int, with_e2e: bool, sampler=None) -> dict:
    """One decode workload on this rank's GPU -> record (timings already reduced to the max over ranks).

    The timed loops are CUDA graphs (a step is shorter than the Python time to queue it): `steps` consecutive steps with
    the layer rotating over pools larger than L2, replayed `repeats` times. Graphs: the one-launch step (the product
    path), the same without launch overlap, decode only, append only, and the two-launch step (append, then decode)."""
    torch, llaisys, rank, local_rank, world, dist = env
    dev = llaisys.DeviceType.NVIDIA
    ctx = workload_lengths(workload, seed=2 + rank)
    B, layers = len(ctx), args.layers
    max_pages = max(-(-c // PAGE) for c in ctx)
    cache = llaisys.PagedKVCache(POOL_PAGES, NKVH, D, nlayer=layers, dtype=llaisys.DataType.BF16, device=dev,
                                 device_id=local_rank, max_seqs=B, max_pages_per_seq=max_pages)
    g = torch.Generator().manual_seed(100 + rank)
    perm = torch.randperm(POOL_PAGES, generator=g).tolist()
    seqs, at = [], 0
    for c in ctx:
        s = cache.add_seq()
        n = -(-c // PAGE)
        cache.assign_pages(s, perm[at:at + n])
        at += n
        seqs.append(s)
    cache.flush()
    stream = torch.cuda.Stream()
    cs = stream.cuda_stream
    cg = torch.Generator(device="cuda").manual_seed(200 + rank)
    seq_ids_dev = torch.tensor(seqs, dtype=torch.int32, device="cuda")
    kv_lens_dev = torch.tensor(ctx, dtype=torch.int32, device="cuda")
    last_pos_dev = kv_lens_dev - 1
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        # fill every layer's pages: all rows but the last of each sequence (the timed step appends the last)
        row_seq = torch.repeat_interleave(seq_ids_dev, (kv_lens_dev - 1).long())
        starts = torch.cumsum(kv_lens_dev - 1, 0) - (kv_lens_dev - 1)
        row_pos = (torch.arange(row_seq.numel(), device="cuda", dtype=torch.int32)
                   - torch.repeat_interleave(starts, (kv_lens_dev - 1).long()).int())
        n_rows = row_seq.numel()
        for layer in range(layers):
            k_rows = torch.randn((n_rows, NKVH, D), generator=cg, device="cuda", dtype=torch.float32).bfloat16()
            v_rows = torch.randn((n_rows, NKVH, D), generator=cg, device="cuda", dtype=torch.float32).bfloat16()
            cache.append_dev(layer, k_rows, v_rows, row_seq, row_pos, n_rows, cs)
            stream.synchronize()
            del k_rows, v_rows
        q = torch.randn((B, NH, D), generator=cg, device="cuda", dtype=torch.float32).bfloat16()
        k_new = torch.randn((B, NKVH, D), generator=cg, device="cuda", dtype=torch.float32).bfloat16()
        v_new = torch.randn((B, NKVH, D), generator=cg, device="cuda", dtype=torch.float32).bfloat16()
        out = torch.empty_like(q)
    stream.synchronize()
    cache.check()
    scale, max_kv = 1.0 / D ** 0.5, max(ctx)
    overlap = not args.no_overlap

    def step_one_launch(i):
        cache.decode_step_dev(i % layers, out, q, k_new, v_new, seq_ids_dev, kv_lens_dev, B, max_kv, NH, scale, cs)

    def only_decode(i):
        cache.decode_dev(i % layers, out, q, seq_ids_dev, kv_lens_dev, B, max_kv, NH, scale, cs)

    def only_append(i):
        cache.append_dev(i % layers, k_new, v_new, seq_ids_dev, last_pos_dev, B, cs)

    def step_two_launches(i):
        only_append(i)
        only_decode(i)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    cache.set_launch_overlap(overlap)
    for i in range(max(3, args.warmup)):
        step_one_launch(i)
    stream.synchronize()
    assert cache.last_kernel() == llaisys.Kernel.DECODE_TMA_FUSED, "the step did not run on the TMA decode kernel"
    if args.quick:  # profiler runs: a few eager launches of each kernel of the step, no graphs, no timing
        for i in range(steps):
            step_one_launch(i)
        for i in range(steps):
            step_two_launches(i)
        stream.synchronize()
        cache.check()
        cache.close()
        return {"workload": workload, "quick": True, "launches": {"paged_decode_tma_kernel": max(3, args.warmup) + 2 * steps,
                                                                    "paged_append_kernel": layers + steps}}

    def capture(body, with_overlap):
        cache.set_launch_overlap(with_overlap)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(steps):
                body(i)
        cache.set_launch_overlap(overlap)
        return graph

    g_step = capture(step_one_launch, overlap)
    g_step_plain = capture(step_one_launch, False)
    g_decode = capture(only_decode, overlap)
    g_append = capture(only_append, overlap)
    g_two = capture(step_two_launches, overlap)

    barrier()
    if sampler is not None:
        sampler.__enter__()
    step_ms = replay_times(torch, stream, g_step, repeats)
    barrier()
    plain_ms = replay_times(torch, stream, g_step_plain, repeats)
    decode_ms = replay_times(torch, stream, g_decode, repeats)
    append_ms = replay_times(torch, stream, g_append, repeats)
    two_ms = replay_times(torch, stream, g_two, repeats)
    if sampler is not None:
        sampler.__exit__()
    cache.check()

    # ---- the no-allocation entry point (the caller's pool, static scratch, the cp.async decode kernel): decode only, plain
    #      launches queued back to back, one event pair around the lot (no claim is made for it about graph capture) -------
    no_alloc_ms = None
    if B * NKVH <= 512:
        n_na = max(20, min(steps, 100))

        def no_alloc(i):
            llaisys.decode_no_alloc(out, q, cache.pool_ptr(i % layers), cache.block_table_ptr(), cache.max_pages_per_seq,
                                    POOL_PAGES, seq_ids_dev, kv_lens_dev, B, max_kv, NH, NKVH, scale, device_id=local_rank,
                                    stream=cs)

        for i in range(3):
            no_alloc(i)
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(n_na):
            no_alloc(i)
        e1.record(stream)
        stream.synchronize()
        no_alloc_ms = e0.elapsed_time(e1) / n_na

    # ---- end to end through the host-buffer call: host buffers, copies inside the timed region ---------------------
    e2e = None
    if with_e2e:
        q_h, k_h, v_h = (t.cpu().pin_memory() for t in (q, k_new, v_new))
        out_h = torch.empty_like(q_h).pin_memory()
        seqs_np, ctx_np = np.asarray(seqs, dtype=np.int32), np.asarray(ctx, dtype=np.int32)

        def step_e2e(i: int):
            # the library's host-buffer step: pinned q / new K,V rows in, the step kernel, attention output back, one
            # synchronise -- one call per decode step, as a serving loop without device-resident activations makes it
            cache.decode_step_host(i % layers, out_h, q_h, k_h, v_h, seqs_np, ctx_np, NH, scale)

        e2e_steps = max(10, min(steps * repeats, 1000))
        for i in range(3):
            step_e2e(i)
        barrier()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            step_e2e(i)
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
        cache.check()
        step_e2e(0)  # both legs on the same layer must give the same bits
        step_one_launch(0)
        stream.synchronize()
        same = bool(torch.equal(out_h.view(torch.int16), out.cpu().view(torch.int16)))
        e2e_s = reduce_max(torch, dist, [e2e_s])[0]
        e2e = {"value": B * world * e2e_steps / e2e_s, "unit": "tokens/s",
               "h2d_bytes_per_step": (q_h.numel() + k_h.numel() + v_h.numel()) * 2 + 2 * B * 4,  # + two index arrays
               "d2h_bytes_per_step": out_h.numel() * 2, "steps": e2e_steps, "ms_per_step": 1e3 * e2e_s / e2e_steps,
               "matches_device_path": same,
               "what": "PagedKVCache.decode_step_host(): pinned host q / K,V rows in, attention out, one synchronise"}

    med = [statistics.median(x) for x in (step_ms, plain_ms, decode_ms, append_ms, two_ms)]
    med = reduce_max(torch, dist, med)
    lo_hi = reduce_max(torch, dist, [max(step_ms), -min(step_ms)])
    bytes_step = algorithmic_bytes(ctx, with_append=True)
    hbm, _, _, kind = _peaks()
    period_ms = med[0] / steps
    achieved = bytes_step / (period_ms * 1e-3) / 1e9
    record = {
        "workload": workload,
        "value": B * world * steps / (med[0] * 1e-3), "unit": "tokens/s",
        "ms_per_step": period_ms, "ms_per_step_min": -lo_hi[1] / steps, "ms_per_step_max": lo_hi[0] / steps,
        "steps": steps, "repeats": repeats,
        "config": decode_config(workload, ctx, world, layers, overlap),
        "roofline": {"bound": "hbm", "kernel": "paged_decode_tma_kernel (one launch per step: append + decode)",
                     "achieved": achieved, "peak": hbm, "peak_kind": f"of {kind}", "unit": "GB/s", "frac": achieved / hbm,
                     "frac_of_nominal_8000": achieved / 8000.0, "traffic": NCU_TRAFFIC_BYTES.get(workload),
                     "algorithmic_bytes_per_launch": bytes_step,
                     "kernel_ms": period_ms, "kernel_ms_spread": spread(step_ms, steps),
                     "kernel_ms_without_launch_overlap": med[1] / steps,
                     "frac_without_launch_overlap": bytes_step / (med[1] / steps * 1e-3) / 1e9 / hbm,
                     "decode_only_kernel_ms": med[2] / steps, "append_only_kernel_ms": med[3] / steps,
                     "two_launch_step_ms": med[4] / steps,
                     "no_alloc_entry_decode_only_ms": no_alloc_ms},  # llaisysPagedAttentionDecodeNoAlloc, plain launches
        "e2e": e2e,
        "gpu_launches": steps * repeats,
        "timing": f"CUDA graph of {steps} steps, {repeats} replays, event pair per replay, median (min/max beside it)",
    }
    del g_step, g_step_plain, g_decode, g_append, g_two
    cache.close()
    return record


def measure_prefill(env, args, *, repeats: int) -> dict:
    """Configuration 3: chunked prefill. 8 sequences, existing context ~ U{0..8192}, a 512-token chunk appended and then
    attended causally. A step = append of the chunk rows + the tcgen05 chunk kernel; graphs of `layers` steps."""
    torch, llaisys, rank, local_rank, world, dist = env
    dev = llaisys.DeviceType.NVIDIA
    g = torch.Generator().manual_seed(3 + rank)
    B, chunk, layers = 8, 512, max(2, args.layers)
    context = torch.randint(0, 8193, (B,), generator=g).tolist()
    kv_lens = [c + chunk for c in context]
    cache = llaisys.PagedKVCache(POOL_PAGES, NKVH, D, nlayer=layers, dtype=llaisys.DataType.BF16, device=dev,
                                 device_id=local_rank, max_seqs=B,
                                 max_pages_per_seq=max(-(-k // PAGE) for k in kv_lens))
    perm = torch.randperm(POOL_PAGES, generator=g).tolist()
    seqs, at = [], 0
    for k in kv_lens:
        n = -(-k // PAGE)
        s = cache.add_seq()
        cache.assign_pages(s, perm[at:at + n])
        at += n
        seqs.append(s)
    cache.flush()
    stream = torch.cuda.Stream()
    cs = stream.cuda_stream
    cg = torch.Generator(device="cuda").manual_seed(300 + rank)
    ids = torch.tensor(seqs, dtype=torch.int32, device="cuda")
    lens = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
    starts = torch.tensor([i * chunk for i in range(B + 1)], dtype=torch.int32, device="cuda")
    ctx_t = torch.tensor(context, dtype=torch.int32, device="cuda")
    # rows of the existing contexts (filled once) and of the chunks (appended every step)
    old_seq = torch.repeat_interleave(ids, ctx_t.long())
    old_pos = (torch.arange(old_seq.numel(), device="cuda", dtype=torch.int32)
               - torch.repeat_interleave(torch.cumsum(ctx_t, 0) - ctx_t, ctx_t.long()).int())
    new_seq = torch.repeat_interleave(ids, chunk)
    new_pos = (torch.arange(chunk, device="cuda", dtype=torch.int32).repeat(B) + torch.repeat_interleave(ctx_t, chunk))
    torch.cuda.synchronize()
    n_old = old_seq.numel()
    for layer in range(layers):
        k_rows = torch.randn((n_old, NKVH, D), generator=cg, device="cuda").bfloat16()
        v_rows = torch.randn((n_old, NKVH, D), generator=cg, device="cuda").bfloat16()
        cache.append_dev(layer, k_rows, v_rows, old_seq, old_pos, n_old, cs)
        stream.synchronize()
    q = torch.randn((B * chunk, NH, D), generator=cg, device="cuda").bfloat16()
    k_new = torch.randn((B * chunk, NKVH, D), generator=cg, device="cuda").bfloat16()
    v_new = torch.randn((B * chunk, NKVH, D), generator=cg, device="cuda").bfloat16()
    out = torch.empty_like(q)
    scale, max_kv = 1.0 / D ** 0.5, max(kv_lens)
    torch.cuda.synchronize()

    def do_append(i):
        cache.append_dev(i % layers, k_new, v_new, new_seq, new_pos, B * chunk, cs)

    def do_attend(i):
        cache.prefill_dev(i % layers, out, q, ids, starts, lens, B, B * chunk, chunk, max_kv, NH, scale, cs)

    def do_step(i):
        do_append(i)
        do_attend(i)

    for i in range(max(3, args.warmup)):
        do_step(i)
    stream.synchronize()
    cache.check()
    assert cache.last_kernel() == llaisys.Kernel.PREFILL_TC, "the chunk attention did not run on the tcgen05 kernel"
    steps = 2 * layers  # per graph: a run of launches over the rotating layer pools
    if args.quick:  # profiler runs: eager launches only
        for i in range(steps):
            do_step(i)
        stream.synchronize()
        cache.check()
        cache.close()
        return {"workload": "config3", "quick": True, "launches": {"paged_prefill_tc_kernel": max(3, args.warmup) + steps}}

    overlap = not args.no_overlap

    def capture(body, with_overlap):
        cache.set_launch_overlap(with_overlap)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(steps):
                body(i)
        cache.set_launch_overlap(False)
        return graph

    g_step, g_att, g_app = capture(do_step, overlap), capture(do_attend, overlap), capture(do_append, overlap)
    g_att_plain = capture(do_attend, False)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    step_ms = replay_times(torch, stream, g_step, repeats)
    attend_ms = replay_times(torch, stream, g_att, repeats)
    attend_plain_ms = replay_times(torch, stream, g_att_plain, repeats)
    append_ms = replay_times(torch, stream, g_app, repeats)
    cache.check()

    # end to end: host index arrays, pinned host q / k / v / out, copies and a synchronise per step
    e2e = None
    if not args.no_e2e:
        api, lib_stream = llaisys.RuntimeAPI(dev), llaisys.context_stream()
        q_h, k_h, v_h = (t.cpu().pin_memory() for t in (q, k_new, v_new))
        out_h = torch.empty_like(q_h).pin_memory()
        q_d, k_d, v_d, out_d = (torch.empty_like(t) for t in (q, k_new, v_new, out))
        new_seq_h, new_pos_h = new_seq.cpu().numpy(), new_pos.cpu().numpy()
        H2D, D2H = llaisys.MemcpyKind.H2D, llaisys.MemcpyKind.D2H

        def step_e2e(i):
            for dst, src in ((q_d, q_h), (k_d, k_h), (v_d, v_h)):
                api.memcpy_async(dst, src, src.numel() * 2, H2D, lib_stream)
            cache.append(i % layers, k_d, v_d, new_seq_h, new_pos_h)
            cache.prefill(i % layers, out_d, q_d, seqs, [chunk] * B, kv_lens, NH, scale)
            api.memcpy_async(out_h, out_d, out_h.numel() * 2, D2H, lib_stream)
            api.stream_synchronize(lib_stream)

        n_e2e = 30
        for i in range(2):
            step_e2e(i)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(n_e2e):
            step_e2e(i)
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
        step_e2e(0)
        do_step(0)
        stream.synchronize()
        e2e = {"value": world * B * chunk * n_e2e / e2e_s, "unit": "tokens/s",
               "h2d_bytes_per_step": (q_h.numel() + k_h.numel() + v_h.numel()) * 2,
               "d2h_bytes_per_step": out_h.numel() * 2, "steps": n_e2e,
               "matches_device_path": bool(torch.equal(out_h.view(torch.int16), out.cpu().view(torch.int16)))}

    med = reduce_max(torch, dist, [statistics.median(x) for x in (step_ms, attend_ms, append_ms, attend_plain_ms)])
    _, burst, sustained, kind = _peaks()
    flops = sum(4 * NH * D * (chunk * c + chunk * (chunk + 1) // 2) for c in context)
    kernel_ms = med[1] / steps
    achieved = flops / (kernel_ms * 1e-3) / 1e12
    record = {
        "workload": "config3",
        "metric": "prefill tokens/s (paged KV append of a 512-token chunk + causal chunk attention, one layer)",
        "value": world * B * chunk * steps / (med[0] * 1e-3), "unit": "tokens/s", "ms_per_step": med[0] / steps,
        "steps": steps, "repeats": repeats,
        "config": {"workload": "config3", "batch_per_gpu": B, "context": context, "chunk": chunk,
                   "heads": "12q/2kv", "head_dim": D, "page_size": PAGE, "pool_pages": POOL_PAGES,
                   "parallelism": f"sequences sharded over {world} GPU(s), no collective",
                   "l2": f"layer pool rotates over {layers} x {cache.layer_bytes() >> 20} MiB between steps",
                   "launch": ("programmatic dependent launch: a kernel's set-up overlaps the previous kernel's tail" if overlap
                              else "plain launches")},
        "roofline": {"bound": "tensor", "kernel": "paged_prefill_tc_kernel", "achieved": achieved,
                     "peak": burst, "peak_kind": f"burst bf16 (a kernel timed alone), of {kind}", "unit": "TFLOP/s",
                     "frac": achieved / burst, "frac_of_sustained": achieved / sustained, "peak_sustained": sustained,
                     "frac_of_nominal_2250": achieved / 2250.0, "traffic": None,
                     "algorithmic_flops_per_launch": flops, "kernel_ms": kernel_ms,
                     "kernel_ms_spread": spread(attend_ms, steps), "append_kernel_ms": med[2] / steps,
                     "kernel_ms_without_launch_overlap": med[3] / steps,
                     "frac_without_launch_overlap": flops / (med[3] / steps * 1e-3) / 1e12 / burst},
        "e2e": e2e, "gpu_launches": 2 * steps * repeats,
        "timing": f"CUDA graphs of {steps} steps, {repeats} replays, event pair per replay, median",
    }
    del g_step, g_att, g_app, g_att_plain
    cache.close()
    return record


QWEN2_1P5B = dict(hidden_size=1536, num_hidden_layers=28, num_attention_heads=12, num_key_value_heads=2, head_dim=128,
                  intermediate_size=8960, vocab_size=151936, max_position_embeddings=4096, rms_norm_eps=1e-6,
                  rope_theta=10000.0, eos_token_id=-1, tie_word_embeddings=False)


def qwen2_random_weights(cfg: dict, seed: int, device: str, std: float = 0.02):
    """Yields (Hugging Face parameter name, tensor) of a random-init model: matrices, embeddings and biases N(0, std),
    norm weights 1 (what a freshly initialised checkpoint holds)."""
    import torch

    g = torch.Generator(device=device).manual_seed(seed)
    hs, qd = cfg["hidden_size"], cfg["num_attention_heads"] * cfg["head_dim"]
    kd, di, voc = cfg["num_key_value_heads"] * cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"]

    def normal(*shape):
        return torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * std

    yield "model.embed_tokens.weight", normal(voc, hs)
    yield "lm_head.weight", normal(voc, hs)
    yield "model.norm.weight", torch.ones(hs, device=device)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        yield p + "input_layernorm.weight", torch.ones(hs, device=device)
        yield p + "post_attention_layernorm.weight", torch.ones(hs, device=device)
        for name, rows in (("q", qd), ("k", kd), ("v", kd)):
            yield p + f"self_attn.{name}_proj.weight", normal(rows, hs)
            yield p + f"self_attn.{name}_proj.bias", normal(rows)
        yield p + "self_attn.o_proj.weight", normal(hs, qd)
        yield p + "mlp.gate_proj.weight", normal(di, hs)
        yield p + "mlp.up_proj.weight", normal(di, hs)
        yield p + "mlp.down_proj.weight", normal(hs, di)


def model_cpu_rate(cfg: dict, min_seconds: float):
    """The oracle model (reference operator definitions composed in torch) on the host cores, bf16: one sequence with a
    short prompt, then greedy decode steps until min_seconds have passed. -> decode tokens/s, threads, description"""
    import torch

    from oracle.qwen2 import Qwen2Oracle

    torch.set_num_threads(len(os.sched_getaffinity(0)))
    state = {k: v for k, v in qwen2_random_weights(cfg, 4, "cpu")}
    oracle = Qwen2Oracle(cfg, state, torch.bfloat16)
    del state
    g = torch.Generator().manual_seed(4)
    prompt = torch.randint(0, cfg["vocab_size"], (64,), generator=g).tolist()
    token = int(oracle.forward(prompt).argmax())
    n, t0 = 0, time.perf_counter()
    while n < 3 or time.perf_counter() - t0 < min_seconds:
        token = int(oracle.forward([token]).argmax())
        n += 1
    rate = n / (time.perf_counter() - t0)
    return rate, torch.get_num_threads(), f"1 of the 64 sequences, 64-token prompt (not 2048), {n} greedy decode steps, bf16"


def run_model_workload(args) -> None:
    """--workload config4: greedy decode of a random-init Qwen2-1.5B-architecture model, bf16. 64 sequences (sharded
    over the N GPUs: strong scaling), 2048-token random prompts, then decode steps on the paged cache. One bench step =
    one decode step of the whole batch through all 28 layers (embedding -> ... -> argmax), replayed as a CUDA graph
    with the loop state on the device; device time comes from CUDA events inside the library around the replays."""
    torch, llaisys, rank, local_rank, world, dist = _init_device()
    cfg = QWEN2_1P5B
    total_seqs, prompt_len = 64, 2048
    if total_seqs % world:
        raise SystemExit("config4 shards 64 sequences: --gpus must divide 64")
    tp = bool(args.tp) and world > 1
    if tp and cfg["num_key_value_heads"] % world:
        raise SystemExit("--tp shards by KV head: --gpus must divide 2 for this model")
    # sequence sharding: each GPU runs its share of the 64 sequences on a full weight replica, no collective;
    # --tp: every GPU runs all 64 sequences on its share of the heads and MLP rows, two NCCL all-reduces per layer
    B = total_seqs if tp else total_seqs // world
    steps = args.steps if args.steps != 2000 else 256  # the configuration's 256 greedy steps unless told otherwise
    warm = max(3, min(args.warmup, 8))
    n_e2e = 0 if args.no_e2e else 32
    max_tokens = prompt_len + warm + steps + 1 + n_e2e + 16

    model = llaisys.models.Qwen2(config=cfg, device=llaisys.DeviceType.NVIDIA, device_id=local_rank,
                                 dtype=llaisys.DataType.BF16, max_seq_len=max_tokens,
                                 tp_group=dist.group.WORLD if tp else None)
    weight_bytes = 0
    for name, value in qwen2_random_weights(cfg, 4, "cuda"):  # the same weights on every rank
        model.load_tensor(name, value)
        if "embed_tokens" not in name:
            # every matrix is read once per decode step (the embedding only B rows); per GPU, so a sharded matrix counts
            # with its share
            sharded = tp and ("_proj." in name)
            weight_bytes += value.numel() * 2 // (world if sharded else 1)
    model.configure_cache(B, max_tokens)
    seqs = [model.add_seq() for _ in range(B)]
    g = torch.Generator().manual_seed(100 + (0 if tp else rank))  # tensor-parallel ranks must feed the same tokens
    prompts = torch.randint(0, cfg["vocab_size"], (B, prompt_len), generator=g).tolist()

    # prefill, eight sequences per call (bounds the activation workspace), timed on the host with a synchronise
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    nxt = []
    for i in range(0, B, 8):
        nxt += model.step(seqs[i:i + 8], prompts[i:i + 8])
    prefill_s = time.perf_counter() - t0

    nxt = model.decode_loop(seqs, nxt, warm)[-1].tolist()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    with ClockSampler(local_rank) as clocks:
        log = model.decode_loop(seqs, nxt, steps + 1)  # first step eager and untimed, `steps` timed graph replays
    step_ms = model.last_loop_ms
    nxt = log[-1].tolist()
    assert log.shape == (steps + 1, B) and 0 <= int(log.min()) and int(log.max()) < cfg["vocab_size"]
    ctx_mid = prompt_len + warm + 1 + steps // 2

    e2e = None
    if n_e2e:
        # the public per-step call: host token lists in, host tokens out, index arrays uploaded every step
        cur = model.step(seqs, [[t] for t in nxt])
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(n_e2e - 1):
            cur = model.step(seqs, [[t] for t in cur])
        e2e_s = time.perf_counter() - t0
        e2e = {"value": total_seqs * (n_e2e - 1) / e2e_s, "unit": "tokens/s", "steps": n_e2e - 1,
               "h2d_bytes_per_step": B * (4 * 8 + 5 * 4) + 4, "d2h_bytes_per_step": B * 8,
               "what": "Qwen2.step() once per decode step: host tokens in (index arrays uploaded), the step replayed as a CUDA graph, "
                       "host greedy tokens out, one synchronise per step"}

    stats = torch.tensor([step_ms, prefill_s], device="cuda", dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        step_ms, prefill_s = (float(x) for x in stats)
        if e2e is not None:
            rate = torch.tensor([e2e["value"]], device="cuda", dtype=torch.float64)
            dist.all_reduce(rate, op=dist.ReduceOp.MIN)
            e2e["value"] = float(rate)
    if rank == 0:
        hbm_peak, _, _, kind = _peaks()
        kv_bytes = cfg["num_hidden_layers"] * B * ctx_mid * (2 * (NKVH // world if tp else NKVH) * D * 2)
        achieved = (weight_bytes + kv_bytes) / (step_ms * 1e-3) / 1e9
        # per layer: 2 norms, bias+rope+append, decode attention, activation; per step: embedding, norm, argmax, 2 x advance
        own = cfg["num_hidden_layers"] * 5 + 5
        line = {
            "metric": "decode tokens/s (Qwen2-1.5B architecture, greedy, paged KV cache)",
            "value": total_seqs * 1e3 / step_ms, "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": warm,
            "ms_per_step": step_ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (random-init weights N(0, 0.02), random-token prompts)",
            "config": {"workload": "config4", "batch": total_seqs, "batch_per_gpu": B, "prompt": prompt_len,
                       "layers": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"], "heads": "12q/2kv",
                       "head_dim": D, "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                       "page_size": PAGE, "parallelism": (f"tensor parallel over {world} GPUs (heads and MLP rows), 2 NCCL all-reduces per layer"
                                       if tp else f"sequences sharded over {world} GPU(s), no collective"),
                       "l2": "every step reads all weights and the whole KV cache (several GB): larger than L2"},
            "roofline": {"bound": "hbm", "kernel": "whole decode step (paged decode attention + cuBLAS projections)",
                         "achieved": achieved, "peak": hbm_peak, "peak_kind": f"copy bandwidth, of {kind}",
                         "unit": "GB/s", "frac": achieved / hbm_peak, "traffic": None,
                         "algorithmic_bytes_per_step": {"weights": weight_bytes, "kv_cache_mid_loop": kv_bytes}},
            "prefill": {"tokens_per_s": total_seqs * prompt_len / prefill_s, "seconds": prefill_s,
                        "what": "2048-token prompts, 8 sequences per call, host clock"},
            "e2e": e2e, "gpu_launches": own * steps,
            "library_launches": (cfg["num_hidden_layers"] * 4 + 1) * steps,
            "timing": "CUDA events around the graph replays, max over ranks", "clocks": clocks.summary(),
        }
        if not args.no_cpu_baseline and world == 1:
            rate, threads, sample = model_cpu_rate(cfg, 12.0)
            line["cpu_baseline"] = {"value": rate, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def run_copy_workload(args) -> None:
    """--workload copy: the data-movement kernels of the path alone, at a row count where bandwidth (not launch latency)
    decides: K1 paged append, K1b bias + RoPE + append over a packed q|k|v projection, K5 gather. 65536 rows = 64
    sequences x 1024 tokens into a 16384-page pool (random physical pages); layers rotate so that every launch misses L2.
    Algorithmic bytes: append reads and writes each K and V row once (2 x 1 KiB per row) plus 8 B of indices; the fused
    kernel reads the 4 KiB packed projection row and writes the 3 KiB q row and the 1 KiB of K and V; gather reads and
    writes 1 KiB per token."""
    torch, llaisys, rank, local_rank, world, dist = _init_device()
    dev = llaisys.DeviceType.NVIDIA
    B, ctx, layers = 64, 1024, max(4, args.layers)
    rows = B * ctx
    cache = llaisys.PagedKVCache(POOL_PAGES, NKVH, D, nlayer=layers, dtype=llaisys.DataType.BF16, device=dev,
                                 device_id=local_rank, max_seqs=B, max_pages_per_seq=ctx // PAGE)
    g = torch.Generator().manual_seed(7 + rank)
    perm = torch.randperm(POOL_PAGES, generator=g).tolist()
    seqs = []
    for i in range(B):
        s = cache.add_seq()
        cache.assign_pages(s, perm[i * (ctx // PAGE):(i + 1) * (ctx // PAGE)])
        seqs.append(s)
    cache.flush()
    stream = torch.cuda.Stream()
    cs = stream.cuda_stream
    k_rows = torch.randn((rows, NKVH, D), device="cuda").bfloat16()
    v_rows = torch.randn((rows, NKVH, D), device="cuda").bfloat16()
    qkv = torch.randn((rows, (NH + 2 * NKVH) * D), device="cuda").bfloat16()
    bias = torch.randn(((NH + 2 * NKVH) * D,), device="cuda").bfloat16()
    q_out = torch.empty((rows, NH, D), device="cuda", dtype=torch.bfloat16)
    seq_of_row = torch.repeat_interleave(torch.tensor(seqs, dtype=torch.int32, device="cuda"), ctx)
    pos_of_row = torch.arange(ctx, dtype=torch.int32, device="cuda").repeat(B)
    k_out = torch.empty((ctx, NKVH, D), device="cuda", dtype=torch.bfloat16)
    v_out = torch.empty_like(k_out)
    torch.cuda.synchronize()
    reps = max(5, min(args.steps, 50))

    def timed(body):
        with torch.cuda.stream(stream):
            for i in range(3):
                body(i)
            stream.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for i in range(reps):
                body(i)
            e1.record(stream)
        stream.synchronize()
        return e0.elapsed_time(e1) / reps

    overlap = not args.no_overlap
    with ClockSampler(local_rank) as clocks:
        append_plain_ms = timed(lambda i: cache.append_dev(i % layers, k_rows, v_rows, seq_of_row, pos_of_row, rows, cs))
        cache.set_launch_overlap(overlap)  # programmatic launches: the next append is scheduled under this one's tail
        append_ms = timed(lambda i: cache.append_dev(i % layers, k_rows, v_rows, seq_of_row, pos_of_row, rows, cs))
        cache.set_launch_overlap(False)
    fused_ms = timed(lambda i: cache.rope_append_dev(i % layers, q_out, qkv, bias, seq_of_row, pos_of_row, rows, NH, 10000.0, cs))
    # A plain device-to-device copy that moves the same bytes as the append (K and V rows read once, written once), timed
    # the same way: what a copy of THIS size reaches (the measured peak is taken on a 4 GB copy). Four destinations rotate.
    copy_src = torch.cat([k_rows.view(-1), v_rows.view(-1)])
    copy_dst = [torch.empty_like(copy_src) for _ in range(4)]
    plain_copy_ms = timed(lambda i: copy_dst[i % 4].copy_(copy_src, non_blocking=True))
    del copy_dst

    def gather_all(i):  # the gather entry point takes one sequence: 64 launches move the same 64 MiB back out
        with torch.cuda.stream(stream):
            for s in seqs:
                cache.gather(i % layers, s, ctx, k_out, v_out)
    # gather queues on the library's stream: time it there
    ext = torch.cuda.ExternalStream(llaisys.context_stream())
    for i in range(2):
        gather_all(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(ext)
    for i in range(reps):
        gather_all(i)
    e1.record(ext)
    torch.cuda.synchronize()
    gather_ms = e0.elapsed_time(e1) / reps
    cache.check()
    if rank == 0:
        hbm_peak, _, _, kind = _peaks()
        row_kv = 2 * NKVH * D * 2
        append_bytes = rows * (2 * row_kv + 8)
        fused_bytes = rows * ((NH + 2 * NKVH) * D * 2 + NH * D * 2 + row_kv + 8)
        gather_bytes = rows * 2 * row_kv
        line = {
            "metric": "paged append rows/s (65536 rows of K and V into random pages, one layer)",
            "value": world * rows / (append_ms * 1e-3), "unit": "rows/s", "n_gpus": world, "steps": reps, "warmup": 3,
            "ms_per_step": append_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": "copy", "rows": rows, "heads": "12q/2kv", "head_dim": D, "page_size": PAGE,
                       "pool_pages": POOL_PAGES, "l2": f"layer pool rotates over {layers} x 256 MiB between launches",
                       "launch": "programmatic dependent launch" if overlap else "plain launches"},
            "roofline": {"bound": "hbm", "kernel": "paged_append_kernel", "achieved": append_bytes / (append_ms * 1e-3) / 1e9,
                         "peak": hbm_peak, "peak_kind": f"of {kind}", "unit": "GB/s",
                         "frac": append_bytes / (append_ms * 1e-3) / 1e9 / hbm_peak, "traffic": None,
                         "algorithmic_bytes_per_launch": append_bytes, "kernel_ms_mean": append_ms,
                         "kernel_ms_without_launch_overlap": append_plain_ms,
                         "frac_without_launch_overlap": append_bytes / (append_plain_ms * 1e-3) / 1e9 / hbm_peak,
                         "plain_copy_of_the_same_bytes": {"ms": plain_copy_ms, "GB/s": 2 * rows * row_kv / (plain_copy_ms * 1e-3) / 1e9,
                                                          "append_vs_copy": plain_copy_ms / append_ms}},
            "rope_append": {"kernel": "paged_rope_append_kernel", "ms": fused_ms, "algorithmic_bytes_per_launch": fused_bytes,
                            "GB/s": fused_bytes / (fused_ms * 1e-3) / 1e9,
                            "frac": fused_bytes / (fused_ms * 1e-3) / 1e9 / hbm_peak},
            "gather": {"kernel": "paged_gather_kernel", "ms_for_64_launches": gather_ms,
                       "algorithmic_bytes": gather_bytes, "GB/s": gather_bytes / (gather_ms * 1e-3) / 1e9,
                       "note": "one launch per sequence (1024 tokens, 2 MiB moved each): latency-bound by design, it is "
                               "a test and debugging entry point"},
            "e2e": None, "gpu_launches": reps, "timing": "CUDA events around back-to-back launches", "clocks": clocks.summary(),
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def measure_kv_split(env, args, *, steps: int, one_gpu_reference: bool) -> dict:
    """Configuration 5: ONE 131072-token sequence, 28 layers, KV range split across the N GPUs (strong scaling).

    Each rank holds its page-aligned slice of every layer (28 per-layer "sequences" in one pool). A step is one decode
    token's attention through all 28 layers. Batched mode: the synthetic workload supplies every layer's query up front,
    so it is one partial-decode launch over 28 sequences whose rows the kernel itself stores into every rank's exchange
    slots, and one merge. Per-layer mode: 28 dependent rounds of the same two launches (what a real model needs). Both
    are replayed as CUDA graphs; the NCCL path (partial decode, all_gather_into_tensor, merge, host-driven) is timed
    beside them and must give the same bits. Layer 0 is also checked against the float64 oracle on the full sequence."""
    torch, llaisys, rank, local_rank, world, dist = env
    from llaisys_b200 import sharding

    dev = llaisys.DeviceType.NVIDIA
    total_tokens, n_layers = 131072, 28
    lo, hi = sharding.kv_range(total_tokens, world, rank)
    local = hi - lo
    pages_per = -(-local // PAGE)
    cache = llaisys.PagedKVCache(n_layers * pages_per, NKVH, D, nlayer=1, dtype=llaisys.DataType.BF16, device=dev,
                                 device_id=local_rank, max_seqs=n_layers, max_pages_per_seq=pages_per)
    g = torch.Generator().manual_seed(5 + rank)
    perm = torch.randperm(n_layers * pages_per, generator=g).tolist()
    seqs = []
    for layer in range(n_layers):
        s = cache.add_seq()
        cache.assign_pages(s, perm[layer * pages_per:(layer + 1) * pages_per])
        seqs.append(s)
    cache.flush()
    cs = llaisys.context_stream()
    ext = torch.cuda.ExternalStream(cs)
    api = llaisys.RuntimeAPI(dev)
    cg = torch.Generator(device="cuda").manual_seed(500 + rank)
    pos = torch.arange(local, dtype=torch.int32, device="cuda")
    k0 = v0 = None
    for i, s in enumerate(seqs):  # N(0,1) K/V rows of this rank's slice of each layer
        k_rows = torch.randn((local, NKVH, D), generator=cg, device="cuda").bfloat16()
        v_rows = torch.randn((local, NKVH, D), generator=cg, device="cuda").bfloat16()
        torch.cuda.synchronize()
        cache.append_dev(0, k_rows, v_rows, torch.full((local,), s, dtype=torch.int32, device="cuda"), pos, local, cs)
        api.stream_synchronize(cs)
        if i == 0:
            k0, v0 = k_rows, v_rows  # layer 0's slice, for the oracle check
    qg = torch.Generator(device="cuda").manual_seed(999)  # the same queries on every rank
    q = torch.randn((n_layers, NH, D), generator=qg, device="cuda").bfloat16()
    out = torch.empty_like(q)
    part = torch.empty((n_layers, NH, D + 2), dtype=torch.float32, device="cuda")
    lens = [local] * n_layers
    scale = 1.0 / D ** 0.5
    torch.cuda.synchronize()

    def merge(parts, n_parts, rows, dst):
        llaisys.lse_merge(dst, parts, n_parts, rows, D, dtype=llaisys.DataType.BF16, device=dev, device_id=local_rank)

    def nccl_batched():
        if world > 1:
            sharding.split_decode(cache, 0, out, q, seqs, lens, NH, scale)
        else:
            cache.decode_partial(0, part, q, seqs, lens, NH, scale)
            merge(part, 1, n_layers * NH, out)

    def nccl_per_layer():
        for layer in range(n_layers):
            if world > 1:
                sharding.split_decode(cache, 0, out[layer:layer + 1], q[layer:layer + 1], seqs[layer:layer + 1], [local],
                                      NH, scale)
            else:
                cache.decode_partial(0, part[layer:layer + 1], q[layer:layer + 1], seqs[layer:layer + 1], [local], NH, scale)
                merge(part[layer:layer + 1], 1, NH, out[layer:layer + 1])

    def only_decode():
        cache.decode_partial(0, part, q, seqs, lens, NH, scale)

    def only_decode_one_layer():
        cache.decode_partial(0, part[:1], q[:1], seqs[:1], [local], NH, scale)

    # ---- the same step through peer memory: no collective library, no host work between the kernels ----------------
    peer = sharding.PeerExchange(n_layers * NH, D, device_id=local_rank)
    seq_dev = torch.tensor(seqs, dtype=torch.int32, device="cuda")
    len_dev = torch.full((n_layers,), local, dtype=torch.int32, device="cuda")
    out_p = torch.empty_like(q)

    def peer_batched():
        peer.split_decode(cache, 0, out_p, q, seq_dev, len_dev, n_layers, local, NH, scale, cs)

    def peer_per_layer():
        for layer in range(n_layers):
            peer.split_decode(cache, 0, out_p[layer:layer + 1], q[layer:layer + 1], seq_dev[layer:layer + 1],
                              len_dev[layer:layer + 1], 1, local, NH, scale, cs)

    def sync_all():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def graphed(body):
        body()  # eager once
        peer.check(cs)
        sync_all()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=ext):
            body()

        def replay():
            with torch.cuda.stream(ext):
                graph.replay()
        return replay

    def timed(body, n):
        """-> milliseconds per call, one event pair per call (median taken by the caller)."""
        for _ in range(3):
            body()
        sync_all()
        events = [torch.cuda.Event(enable_timing=True) for _ in range(n + 1)]
        events[0].record(ext)
        for i in range(n):
            body()
            events[i + 1].record(ext)
        torch.cuda.synchronize()
        sync_all()
        return [events[i].elapsed_time(events[i + 1]) for i in range(n)]

    n_rep = max(MIN_REPEATS, min(steps, 200))
    nccl_ms = timed(nccl_batched, n_rep)
    nccl_layer_ms = timed(nccl_per_layer, max(10, n_rep // 5))
    torch.cuda.synchronize()
    expect_layer = out.clone()  # per-layer launches cut the pairs differently from the batched one: their own reference
    decode_ms = timed(only_decode, n_rep)
    decode_layer_ms = timed(only_decode_one_layer, n_rep)
    cache.check()
    nccl_batched()
    torch.cuda.synchronize()
    expect = out.clone()
    peer_ms = timed(graphed(peer_batched), n_rep)
    peer.check(cs)
    # consecutive tokens: four steps per graph, so that a step's launch and set-up overlap the merge of the step before it
    # (programmatic launches), as they do in the per-layer mode and in the headline's graphs of many steps
    steps_per_graph = 4

    def peer_batched_run():
        for _ in range(steps_per_graph):
            peer_batched()

    peer_run_ms = [t / steps_per_graph for t in timed(graphed(peer_batched_run), n_rep)]
    peer.check(cs)
    assert cache.last_kernel() == llaisys.Kernel.DECODE_TMA, "the partial decode did not run on the TMA decode kernel"
    peer_same = bool(torch.equal(out_p.view(torch.int16), expect.view(torch.int16)))  # same partials, same merge order
    peer_layer_ms = timed(graphed(peer_per_layer), max(10, n_rep // 5))
    peer.check(cs)
    peer_layer_same = bool(torch.equal(out_p.view(torch.int16), expect_layer.view(torch.int16)))

    # ---- layer 0 against the float64 oracle on the FULL sequence (rank 0 collects the slices) -----------------------
    if world > 1:
        k_all = torch.empty((world * local, NKVH, D), dtype=torch.bfloat16, device="cuda")
        v_all = torch.empty_like(k_all)
        dist.all_gather_into_tensor(k_all, k0)
        dist.all_gather_into_tensor(v_all, v0)
    else:
        k_all, v_all = k0, v0
    max_abs = None
    if rank == 0:
        from oracle import attention

        f64 = attention.decode_attention_f64_chunked(q[:1].cpu(), k_all.cpu(), v_all.cpu(), scale)
        max_abs = float((out_p[:1].cpu().double() - f64).abs().max())
    del k_all, v_all, k0, v0

    # ---- the whole sequence on ONE GPU, for the speed-up (rank 0 alone; the others wait) -----------------------------
    one_gpu_ms = None
    if one_gpu_reference and world > 1:
        if rank == 0:
            full_pages = total_tokens // PAGE
            big = llaisys.PagedKVCache(n_layers * full_pages, NKVH, D, nlayer=1, dtype=llaisys.DataType.BF16, device=dev,
                                       device_id=local_rank, max_seqs=n_layers, max_pages_per_seq=full_pages)
            bperm = torch.randperm(n_layers * full_pages, generator=g).tolist()
            bseqs = []
            for layer in range(n_layers):
                s = big.add_seq()
                big.assign_pages(s, bperm[layer * full_pages:(layer + 1) * full_pages])
                bseqs.append(s)
            big.flush()
            bpos = torch.arange(total_tokens, dtype=torch.int32, device="cuda")
            for s in bseqs:
                k_rows = torch.randn((total_tokens, NKVH, D), generator=cg, device="cuda").bfloat16()
                v_rows = torch.randn((total_tokens, NKVH, D), generator=cg, device="cuda").bfloat16()
                torch.cuda.synchronize()
                big.append_dev(0, k_rows, v_rows, torch.full((total_tokens,), s, dtype=torch.int32, device="cuda"), bpos,
                               total_tokens, cs)
                api.stream_synchronize(cs)
                del k_rows, v_rows
            blens = [total_tokens] * n_layers

            def one_gpu():
                big.decode(0, out, q, bseqs, blens, NH, scale)

            for _ in range(3):
                one_gpu()
            torch.cuda.synchronize()
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(n_rep + 1)]
            ev[0].record(ext)
            for i in range(n_rep):
                one_gpu()
                ev[i + 1].record(ext)
            torch.cuda.synchronize()
            one_gpu_ms = statistics.median(ev[i].elapsed_time(ev[i + 1]) for i in range(n_rep))
            big.close()
        sync_all()

    med = reduce_max(torch, dist, [statistics.median(x) for x in
                                   (peer_ms, peer_layer_ms, nccl_ms, nccl_layer_ms, decode_ms, decode_layer_ms, peer_run_ms)])
    hbm, _, _, kind = _peaks()
    bytes_per_launch = n_layers * local * (2 * NKVH * D * 2) + 2 * n_layers * NH * D * 2 + 4 * n_layers * pages_per
    achieved = bytes_per_launch / (med[4] * 1e-3) / 1e9
    record = {
        "workload": "config5",
        "metric": "decode tokens/s (one 131072-token sequence, attention of 28 layers, KV range split across GPUs)",
        "value": 1e3 / med[0], "unit": "tokens/s", "n_gpus": world,
        "ms_per_step": med[0], "ms_per_step_spread": spread(peer_ms),
        "ms_per_step_in_a_run": med[6], "steps_per_graph_in_a_run": steps_per_graph,
        "per_layer_ms": med[1], "per_layer_round_ms": med[1] / n_layers,
        "nccl_ms": med[2], "nccl_per_layer_ms": med[3],
        "speedup_vs_1gpu": (one_gpu_ms / med[0]) if one_gpu_ms else None, "one_gpu_ms": one_gpu_ms,
        "max_abs_vs_oracle": max_abs,
        "peer_path_matches_nccl_path": peer_same and peer_layer_same,
        "decode_kernel_ms": med[4], "decode_kernel_ms_one_layer_host_driven": med[5],
        "config": {"workload": "config5", "context": total_tokens, "layers": n_layers, "tokens_per_gpu": local,
                   "heads": "12q/2kv", "head_dim": D, "page_size": PAGE,
                   "mode": "batched: one partial-decode launch that stores its rows into every rank's exchange slots over "
                           "NVLink (peer memory) and stamps the flags, one merge; per-layer: 28 dependent rounds of the "
                           "same two launches; both replayed as CUDA graphs",
                   "parallelism": f"KV range split over {world} GPU(s), (o, m, l) partials exchanged through peer memory",
                   "l2": f"{bytes_per_launch >> 20} MiB of K/V per GPU per step" +
                         (", larger than L2" if bytes_per_launch > 2e8 else " (fits L2 at this GPU count)")},
        "roofline": {"bound": "hbm", "kernel": "paged_decode_tma_kernel", "achieved": achieved, "peak": hbm,
                     "peak_kind": f"of {kind}", "unit": "GB/s", "frac": achieved / hbm,
                     "frac_of_nominal_8000": achieved / 8000.0, "traffic": None,
                     "algorithmic_bytes_per_launch": bytes_per_launch, "kernel_ms": med[4]},
        "oracle": "layer 0 of the batched peer-memory step against the float64 statement of the reference's attention over "
                  "all 131072 tokens (max-abs; one bf16 ulp of the output is 8e-3)",
        "timing": f"CUDA events on the library stream, one pair per step, median of {n_rep}, max over ranks",
        "gpu_launches": 2 * n_rep,
    }
    peer.close()
    cache.close()
    return record


def run_longctx_workload(args) -> None:
    """--workload config5 as its own line."""
    env = _init_device()
    torch, llaisys, rank, local_rank, world, dist = env
    with ClockSampler(local_rank) as clocks:
        rec = measure_kv_split(env, args, steps=args.steps, one_gpu_reference=False)
    if rank == 0:
        line = {"metric": rec["metric"], "value": rec["value"], "unit": "tokens/s", "n_gpus": world, "steps": rec["ms_per_step_spread"]["n"],
                "warmup": 3, "ms_per_step": rec["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": rec["config"],
                "roofline": rec["roofline"],
                "per_layer": {"ms_per_step": rec["per_layer_ms"], "ms_per_round": rec["per_layer_round_ms"],
                              "note": "28 dependent rounds of partial decode (+ exchange in the kernel) + merge",
                              "decode_kernel_ms_one_layer_host_driven": rec["decode_kernel_ms_one_layer_host_driven"]},
                "in_a_run": {"ms_per_step": rec["ms_per_step_in_a_run"], "steps_per_graph": rec["steps_per_graph_in_a_run"]},
                "nccl_all_gather": {"ms_per_step": rec["nccl_ms"], "per_layer_ms_per_step": rec["nccl_per_layer_ms"],
                                    "peer_path_matches": rec["peer_path_matches_nccl_path"]},
                "max_abs_vs_oracle": rec["max_abs_vs_oracle"], "e2e": None, "gpu_launches": rec["gpu_launches"],
                "timing": rec["timing"], "clocks": clocks.summary()}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def run_prefill_workload(args) -> None:
    """--workload config3 as its own line."""
    env = _init_device()
    torch, llaisys, rank, local_rank, world, dist = env
    if args.quick:
        print(json.dumps(measure_prefill(env, args, repeats=1)), flush=True)
        return
    with ClockSampler(local_rank) as clocks:
        rec = measure_prefill(env, args, repeats=max(MIN_REPEATS, min(args.steps, 200)))
    if rank == 0:
        line = {"metric": rec["metric"], "value": rec["value"], "unit": "tokens/s", "n_gpus": world, "steps": rec["steps"],
                "repeats": rec["repeats"], "warmup": max(3, args.warmup), "ms_per_step": rec["ms_per_step"],
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": rec["config"], "roofline": rec["roofline"], "e2e": rec["e2e"], "gpu_launches": rec["gpu_launches"],
                "timing": rec["timing"], "clocks": clocks.summary()}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100, help="steps per timed graph replay (the graph is replayed >= 30 times)")
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="north_star", choices=["north_star", "config2", "config3", "config4", "config5", "copy"])
    ap.add_argument("--layers", type=int, default=4, help="pools to rotate over between steps (L2 flush)")
    ap.add_argument("--repeats", type=int, default=100, help="replays of the timed graph (at least 30)")
    ap.add_argument("--tp", action="store_true", help="config4 on several GPUs: tensor parallelism instead of sequence sharding")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-API leg (profiling runs)")
    ap.add_argument("--no-sub-records", action="store_true",
                    help="north_star only: skip the config2 / config3 (N = 1) and kv_split (N > 1) sub-records")
    ap.add_argument("--quick", action="store_true",
                    help="profiler runs (north_star, config2, config3): warm-up plus --steps eager launches, no graphs or timing")
    ap.add_argument("--no-overlap", action="store_true",
                    help="launch kernels without programmatic stream serialisation (on by default for decode workloads)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3

    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.workload == "config3":
        run_prefill_workload(args)
        return
    if args.workload == "config5":
        run_longctx_workload(args)
        return
    if args.workload == "config4":
        if args.steps == 100:
            args.steps = 2000  # run_model_workload's marker for "the configuration's own 256 steps"
        run_model_workload(args)
        return
    if args.workload == "copy":
        run_copy_workload(args)
        return

    env = _init_device()
    torch, llaisys, rank, local_rank, world, dist = env
    if args.quick:
        print(json.dumps(measure_decode(env, args.workload, args, steps=max(1, min(args.steps, 8)), repeats=1, with_e2e=False)),
              flush=True)
        return
    steps = max(args.layers, min(args.steps, 400) // args.layers * args.layers)  # whole rotations of the layer pools
    repeats = max(MIN_REPEATS, args.repeats)
    clocks = ClockSampler(local_rank)
    rec = measure_decode(env, args.workload, args, steps=steps, repeats=repeats, with_e2e=not args.no_e2e, sampler=clocks)
    subs = {}
    if args.workload == "north_star" and not args.no_sub_records:
        if world == 1:
            sub_args = argparse.Namespace(**vars(args))
            c2 = measure_decode(env, "config2", sub_args, steps=steps, repeats=repeats, with_e2e=False)
            subs["config2"] = {k: c2[k] for k in ("value", "unit", "ms_per_step", "ms_per_step_min", "ms_per_step_max", "steps",
                                                  "repeats", "config", "roofline", "timing")}
            c3 = measure_prefill(env, sub_args, repeats=repeats)
            subs["config3"] = {k: c3[k] for k in ("metric", "value", "unit", "ms_per_step", "steps", "repeats", "config",
                                                  "roofline", "timing")}
        else:
            kv = measure_kv_split(env, args, steps=repeats, one_gpu_reference=True)
            subs["kv_split"] = {k: kv[k] for k in ("metric", "value", "unit", "n_gpus", "ms_per_step", "ms_per_step_spread",
                                                   "ms_per_step_in_a_run", "steps_per_graph_in_a_run",
                                                   "per_layer_ms", "per_layer_round_ms", "speedup_vs_1gpu", "one_gpu_ms",
                                                   "max_abs_vs_oracle", "nccl_ms", "nccl_per_layer_ms",
                                                   "peer_path_matches_nccl_path", "decode_kernel_ms", "config", "oracle",
                                                   "timing")}
    if rank == 0:
        line = {
            "metric": METRIC, "value": rec["value"], "unit": "tokens/s", "n_gpus": world, "steps": steps, "repeats": repeats,
            "warmup": max(3, args.warmup), "ms_per_step": rec["ms_per_step"], "ms_per_step_min": rec["ms_per_step_min"],
            "ms_per_step_max": rec["ms_per_step_max"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": rec["config"], "roofline": rec["roofline"], "e2e": rec["e2e"],
            "gpu_launches": rec["gpu_launches"], "timing": rec["timing"], "clocks": clocks.summary(),
        }
        line.update(subs)
        if world == 1 and not args.no_cpu_baseline:
            ctx = workload_lengths(args.workload, seed=2)
            rate, dt, desc, threads = reference_cpu_rate(ctx, seed=2, min_seconds=10.0, max_seqs=4)
            line["cpu_baseline"] = {"value": rate, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": desc,
                                    "cpp_backend": cpp_backend_cpu_rate(ctx, seed=2, min_seconds=5.0, max_seqs=4)}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
