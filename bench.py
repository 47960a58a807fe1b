"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline workload (N = 1): the Qwen2.5-0.5B-shaped GQA causal prefill forward, B = 1,
14 query heads / 2 KV heads, D = 64, S = 2048, bf16, seeded N(0, 1) inputs. A step is one
forward pass over one batch; with N > 1 every rank runs its own batch (weak scaling, no
collective). The line also carries the forward+backward, decode, SDXL and packed
workloads as `extra` legs (each with its error statistics against the float64 ruler), a
roofline for the dominant kernel, and the reference's CPU path (PyTorch CPU SDPA on the
same bf16 tensors) timed on this box's host cores. With N > 1 the `extra` legs are the
sharded forms of the decode, SDXL and packed workloads and the ring-attention leg.

`--impl reference` times only that CPU path, on the headline workload.
"""

import argparse
import hashlib
import json
import math
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HEADLINE = dict(batch=1, heads=14, kv_heads=2, seq=2048, head_dim=64)
L2_BYTES = 126 * 1024 * 1024
MIN_REGION_MS = 50.0   # the timed graph is replayed until the region is at least this long


def causal_forward_flops(b, h, s, d):
    """2 FLOP per multiply-add, QK^T + PV over visible (query, key) pairs only."""
    return 4.0 * b * h * d * (s * (s + 1) / 2)


def seeded(shapes, seed, device=None, dtype=torch.bfloat16):
    """Seeded N(0, 1) tensors drawn in order on CPU in fp32, then cast (the reference's
    tests draw their inputs this way, tests/hardware/ops/test_flash.py:48-53)."""
    g = torch.Generator().manual_seed(seed)
    out = tuple(torch.randn(*s, generator=g).to(dtype) for s in shapes)
    return out if device is None else tuple(t.to(device) for t in out)


def device_randn(shape, seed, device):
    """Large operands are drawn on the device (seeded)."""
    g = torch.Generator(device=device).manual_seed(seed)
    return torch.randn(shape, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            m = json.load(f)
        return {"bf16": m["bf16_tflops"], "bf16_sustained": m["bf16_tflops_sustained"],
                "hbm": m["hbm_gbs"], "source": "measured"}
    return {"bf16": 1590.0, "bf16_sustained": 1400.0, "hbm": 6650.0, "source": "fallback"}


def git_blob_hash(path):
    """The git blob id of a file's current contents (what `git hash-object` prints)."""
    with open(path, "rb") as f:
        data = f.read()
    return hashlib.sha1(b"blob %d\0" % len(data) + data).hexdigest()


def captured_traffic():
    """DRAM bytes per launch of the headline kernel from the tracked ncu figures beside the
    profile summary; None when the kernel source has changed since the capture."""
    path = os.path.join(ROOT, "profiles", "fwd_row_headline.json")
    try:
        with open(path) as f:
            rec = json.load(f)
        src = os.path.join(ROOT, "kohaku_tt_b200", "csrc", rec["kernel_source"])
        if git_blob_hash(src) != rec["kernel_source_blob"]:
            return None
        return int(rec["dram_bytes_read"]) + int(rec["dram_bytes_write"])
    except (OSError, KeyError, ValueError):
        return None


class ClockSampler:
    """Samples SM clock and clock-event reasons through NVML while a region runs."""

    REASONS = {
        0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
        0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.handle, self.nv.NVML_CLOCK_SM))
                try:
                    bits = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:
                    bits = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for bit, name in self.REASONS.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.01)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def host_threads(world, local):
    """Gives this rank its own share of the host cores (torchrun sets OMP_NUM_THREADS=1 and
    leaves every rank on all CPUs) and returns the thread count."""
    try:
        cpus = sorted(os.sched_getaffinity(0))
    except AttributeError:
        cpus = list(range(os.cpu_count() or 1))
    share = max(1, len(cpus) // max(world, 1))
    if world > 1:
        mine = cpus[local * share:(local + 1) * share] or cpus
        try:
            os.sched_setaffinity(0, mine)
        except (AttributeError, OSError):
            pass
    torch.set_num_threads(share)
    return share


def headline_inputs(seed, device=None):
    c = HEADLINE
    return seeded(
        [(c["batch"], c["heads"], c["seq"], c["head_dim"]),
         (c["batch"], c["kv_heads"], c["seq"], c["head_dim"]),
         (c["batch"], c["kv_heads"], c["seq"], c["head_dim"])], seed, device)


def time_cpu_path(steps, warmup):
    """The reference's CPU path for this op: torch CPU SDPA on the bf16 tensors
    (restated in oracle.attention_oracle.cpu_dense)."""
    from oracle import attention_oracle as ao

    q, k, v = headline_inputs(0)
    for _ in range(warmup):
        ao.cpu_dense(q, k, v, causal=True)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        ao.cpu_dense(q, k, v, causal=True)
        times.append(time.perf_counter() - t0)
    return times


def run_reference(args):
    rank, world, local = dist_env()
    if rank != 0:
        return
    # Rank 0 alone runs the CPU arm: it takes every host core, not torchrun's single thread.
    cores = host_threads(1, 0)
    c = HEADLINE
    flops = causal_forward_flops(c["batch"], c["heads"], c["seq"], c["head_dim"])
    times = time_cpu_path(args.steps, max(args.warmup, 1))
    total = sum(times)
    value = flops * len(times) / total / 1e12
    line = {
        "impl": "reference",
        "metric": "attn_fwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": workload_config(),
        "cpu_baseline": {
            "value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"{len(times)} full forward passes of the headline workload through torch CPU SDPA "
                      f"on bf16 tensors, {cores} threads ({os.cpu_count()} host CPUs visible)",
        },
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def workload_config():
    c = HEADLINE
    return {
        "workload": "GQA causal prefill forward, Qwen2.5-0.5B shape",
        "batch_per_gpu": c["batch"], "heads": c["heads"], "kv_heads": c["kv_heads"],
        "seq_len": c["seq"], "head_dim": c["head_dim"],
        "l2_policy": "each step uses the next of a ring of input sets larger than L2 in total",
        "launch": "the K timed steps are one CUDA graph (K kernel launches back to back); the graph is "
                  "replayed until at least 50 ms of device time are measured (the line's `replays`), each "
                  "replay timed by its own event pair, and the median replay is reported",
        "parallelism": "one batch per GPU, no collective",
    }


def timed_region(fn, steps, warmup, world, graph=False, fork=None, join=None, min_ms=0.0):
    """W untimed calls, then K calls between two events on the current stream, bracketed
    by a barrier and a device synchronize; returns (milliseconds for K steps, replays). With
    `graph` the K calls are captured once into a CUDA graph and the timed region is its
    replay, so the device sees K back-to-back launches without host gaps; the replay is
    repeated (each with its own event pair) until `min_ms` of device time has been measured
    and the median replay is returned, max over ranks. `fork` / `join` make side streams
    start after the start event and finish before the stop event."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    replay = None
    if graph:
        replay = torch.cuda.CUDAGraph()
        with torch.cuda.graph(replay):
            for i in range(steps):
                fn(warmup + i)
        torch.cuda.synchronize()
        replay.replay()   # one untimed replay: first-use costs of the instantiated graph
        torch.cuda.synchronize()
    if world > 1:
        torch.distributed.barrier()

    def once():
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        if fork is not None:
            fork()
        if replay is not None:
            replay.replay()
        else:
            for i in range(steps):
                fn(warmup + i)
        if join is not None:
            join()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop)

    first = once()
    replays = 1
    if replay is not None and min_ms > 0 and first > 0:
        replays = max(1, min(2000, int(math.ceil(min_ms / first))))
    if world > 1:
        t = torch.tensor([replays], dtype=torch.int64, device="cuda")
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        replays = int(t.item())
    samples = [first] + [once() for _ in range(replays - 1)]
    ms = statistics.median(samples)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        torch.distributed.barrier()
        ms = t.item()
    return ms, replays


def stats_of(got, want):
    """The error statistics every leg reports against the float64 ruler."""
    import kohaku_tt_b200 as ktt

    st = ktt.diff_stats(got, want)
    return {k: st[k] for k in ("abs_max", "rel_median", "cosine", "nonfinite")}


def rows_parity(out, lse, q, k, v, pairs, rows, causal=False, shift=0, klen=None):
    """Sampled (batch, head) pairs x sampled query rows of a dense call against float64 rows
    (oracle.ruler_rows): for sizes whose full float64 score matrix does not fit."""
    from oracle import attention_oracle as ao

    group = q.shape[1] // k.shape[1]
    got, want, lse_err = [], [], 0.0
    idx = torch.as_tensor(rows, dtype=torch.long)
    for b, h in pairs:
        o, l = ao.ruler_rows(q[b, h].cpu(), k[b, h // group].cpu(), v[b, h // group].cpu(), rows,
                             shift=shift, causal=causal, klen=None if klen is None else klen[b])
        got.append(out[b, h].cpu()[idx])
        want.append(o)
        if lse is not None:
            lse_err = max(lse_err, float((lse[b, h].cpu()[idx].double() - l).abs().max()))
    st = stats_of(torch.stack(got), torch.stack(want))
    st["lse_abs_max"] = lse_err
    st["sample"] = f"{len(pairs)} (batch, head) pairs x {len(rows)} query rows vs float64"
    return st


def run_ours(args):
    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    threads = host_threads(world, local)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # NCCL keeps its default CTA budget. Measured on two GPUs with the ring leg: capping
        # its send / recv kernels at 4 or 8 CTAs (so that the persistent attention kernels keep
        # more SMs) costs 15-20 % (the exchange then outlasts a step's compute); 16, 32 and no
        # cap are within noise of one another.
        torch.distributed.init_process_group("nccl", device_id=dev)

    import torch.nn.functional as F

    import kohaku_tt_b200 as ktt
    from kohaku_tt_b200 import _lib, ops
    from oracle import attention_oracle as ao

    ktt.build()
    ktt.install()
    peaks = measured_peaks()
    c = HEADLINE
    flops = causal_forward_flops(c["batch"], c["heads"], c["seq"], c["head_dim"])
    steps, warmup = args.steps, max(args.warmup, 3)

    # ---- headline: inputs resident in HBM, a ring of sets larger than L2 -------------
    per_set = 2 * (2 * c["batch"] * c["heads"] + 2 * c["batch"] * c["kv_heads"]) * c["seq"] * c["head_dim"]
    nsets = max(4, int(1.5 * L2_BYTES / per_set) + 1)
    sets = [headline_inputs(1000 * rank + i % 4, dev) for i in range(4)]
    sets = [tuple(t.clone() for t in sets[i % 4]) for i in range(nsets)]

    def step(i):
        q, k, v = sets[i % nsets]
        return ops.sdpa_forward(q, k, v, causal=True, need_lse=True)

    # Parity of the timed path, on this rank's first set, against the float64 ruler.
    q0, k0, v0 = (t.cpu() for t in sets[0])
    out, _ = step(0)
    torch.cuda.synchronize()
    _lib.device_status()
    parity = stats_of(out, ao.ruler_dense(q0, k0, v0, causal=True))

    ktt.reset_counters()
    ms, replays = timed_region(step, steps, warmup, world, graph=not args.eager, min_ms=MIN_REGION_MS)
    launches = steps   # one kernel of this library per step (counted by the library below)
    counted = sum(ktt.counters()[k] for k in ("attention_flash", "attention_mma"))
    _lib.device_status()
    kernel = "tcgen05" if ktt.counters()["attention_flash"] else "warp-mma"
    value = flops * steps * world / (ms * 1e-3) / 1e12
    per_launch_ms = ms / steps

    # Clocks: the same loop repeated for about half a second with the sampler running.
    with ClockSampler(local) as sampler:
        t_end = time.time() + 0.5
        i = 0
        while time.time() < t_end:
            for _ in range(50):
                step(i)
                i += 1
            torch.cuda.synchronize()
    clocks = sampler.summary()

    # ---- end to end: host buffers, H2D and D2H inside the timed region -----------------
    # Steps are independent batches, so they are issued round-robin on a few streams: one
    # step's copies overlap its neighbours' kernel and copies in the other direction, the
    # way a serving loop feeds a GPU. Every step still moves its own inputs in and its
    # result out; the stop event waits for all of them.
    # A step's q, k and v sit back to back in one pinned staging buffer (as a qkv
    # projection's output would) and cross in one copy; the kernel reads the three views.
    shapes = [(c["batch"], c["heads"], c["seq"], c["head_dim"])] + [(c["batch"], c["kv_heads"], c["seq"], c["head_dim"])] * 2
    counts = [math.prod(sh) for sh in shapes]
    host = []
    for i in range(4):
        stage = torch.empty((sum(counts),), dtype=torch.bfloat16).pin_memory()
        for t, off, n in zip(headline_inputs(2000 * rank + i), (0, counts[0], counts[0] + counts[1]), counts):
            stage[off:off + n] = t.reshape(-1)
        host.append(stage)
    lanes = max(0, args.e2e_streams)
    ring = 4
    out_host = [torch.empty((c["batch"], c["heads"], c["seq"], c["head_dim"]), dtype=torch.bfloat16).pin_memory()
                for _ in range(max(lanes, ring))]
    views = lambda flat: tuple(flat[off:off + n].view(sh) for off, n, sh in
                               zip((0, counts[0], counts[0] + counts[1]), counts, shapes))
    if lanes == 0:
        # Three streams with one job each, the classic feed of a GPU: inputs come in on one,
        # the attention call runs on the second, results leave on the third; events hand a
        # step from one to the next and guard the ring of device staging buffers. Copies of
        # one direction never run beside one another (they would only share the link).
        s_in, s_run, s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
        streams = [s_in, s_run, s_out]
        dev_in = [torch.empty((sum(counts),), dtype=torch.bfloat16, device=dev) for _ in range(ring)]
        arrived = [torch.cuda.Event() for _ in range(ring)]
        computed = [torch.cuda.Event() for _ in range(ring)]
        left = [torch.cuda.Event() for _ in range(ring)]
        results = [None] * ring   # a step's output stays referenced until its slot comes round again

        def e2e_step(i):
            r = i % ring
            with torch.cuda.stream(s_in):
                if results[r] is not None:
                    s_in.wait_event(computed[r])   # the kernel that read this buffer last is done
                dev_in[r].copy_(host[i % 4], non_blocking=True)
                arrived[r].record(s_in)
            with torch.cuda.stream(s_run):
                s_run.wait_event(arrived[r])
                if results[r] is not None:
                    # The slot's previous output goes back to this stream's allocator below:
                    # nothing here may reuse it before its copy to the host has finished.
                    s_run.wait_event(left[r])
                q, k, v = views(dev_in[r])
                results[r] = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
                computed[r].record(s_run)
            with torch.cuda.stream(s_out):
                s_out.wait_event(computed[r])
                out_host[r].copy_(results[r], non_blocking=True)
                left[r].record(s_out)
    else:
        streams = [torch.cuda.Stream(device=dev) for _ in range(lanes)]

        def e2e_step(i):
            with torch.cuda.stream(streams[i % lanes]):
                flat = host[i % 4].to(dev, non_blocking=True)
                q, k, v = views(flat)
                o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
                out_host[i % lanes].copy_(o, non_blocking=True)

    def e2e_join():
        main = torch.cuda.current_stream()
        for s_ in streams:
            main.wait_stream(s_)

    def e2e_fork():
        main = torch.cuda.current_stream()
        for s_ in streams:
            s_.wait_stream(main)

    e2e_steps = max(100, steps)
    e2e_ms, _ = timed_region(e2e_step, e2e_steps, warmup, world, fork=e2e_fork, join=e2e_join)
    # Host time to issue one step (copies, views, the attention call, the copy back), measured
    # on a loop short enough not to fill the launch queue, the device idle at the start.
    torch.cuda.synchronize()
    e2e_fork()
    wall0 = time.perf_counter()
    for i in range(50):
        e2e_step(i)
    host_issue_us = (time.perf_counter() - wall0) / 50 * 1e6
    e2e_join()
    torch.cuda.synchronize()
    e2e_value = flops * e2e_steps * world / (e2e_ms * 1e-3) / 1e12
    h2d = host[0].numel() * host[0].element_size()
    d2h = out_host[0].numel() * out_host[0].element_size()

    # What bounds the end-to-end step: the copies alone, on the same three streams.
    def copies_only(i):
        if lanes == 0:
            r = i % ring
            with torch.cuda.stream(s_in):
                dev_in[r].copy_(host[i % 4], non_blocking=True)
                arrived[r].record(s_in)
            with torch.cuda.stream(s_out):
                s_out.wait_event(arrived[r])
                out_host[r].copy_(dev_in[r][:counts[0]].view(shapes[0]), non_blocking=True)
            return
        with torch.cuda.stream(streams[i % lanes]):
            flat = host[i % 4].to(dev, non_blocking=True)
            out_host[i % lanes].copy_(flat[:counts[0]].view(shapes[0]), non_blocking=True)

    copy_ms, _ = timed_region(copies_only, e2e_steps, warmup, world, fork=e2e_fork, join=e2e_join)
    from kohaku_tt_b200 import aten

    e2e_parts = {
        "host_issue_us_per_step": host_issue_us,
        "copies_only_us_per_step": copy_ms / e2e_steps * 1e3, "kernel_us_per_step": per_launch_ms * 1e3,
        "host_threads": threads, "aten_registration": "c++" if aten.using_cpp_registration() else "python",
        "note": "the step time is the largest of the three when they overlap perfectly",
    }
    if world > 1:
        t = torch.tensor([host_issue_us, copy_ms / e2e_steps * 1e3, e2e_ms / e2e_steps * 1e3],
                         dtype=torch.float64, device=dev)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        e2e_parts["max_over_ranks"] = {"host_issue_us_per_step": t[0].item(), "copies_only_us_per_step": t[1].item(),
                                       "e2e_us_per_step": t[2].item()}

    line = {
        "metric": "attn_fwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": per_launch_ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": workload_config(), "replays": replays,
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / e2e_steps, "steps": e2e_steps,
                "api": "torch.nn.functional.scaled_dot_product_attention on CUDA tensors; " + (
                    "a copy-in stream, a compute stream and a copy-out stream chained by events" if lanes == 0
                    else f"steps issued round-robin on {lanes} streams"),
                "parts": e2e_parts},
        "gpu_launches": launches,
        "library_calls_counted": counted,
        "clocks": clocks,
        "kernel": kernel,
        "parity_vs_f64": parity,
    }
    achieved = flops / (per_launch_ms * 1e-3) / 1e12
    line["roofline"] = {
        "bound": "tensor", "achieved": achieved, "peak": peaks["bf16"], "unit": "TFLOP/s",
        "frac": achieved / peaks["bf16"],
        "traffic": captured_traffic() if kernel == "tcgen05" else None,
        "traffic_unit": "DRAM bytes per launch (one ncu capture of this kernel source; null when the source changed since)",
        "algorithmic_bytes": per_set,
        "peak_source": f"{peaks['source']} cuBLAS bf16 burst", "frac_of_nominal_2250": achieved / 2250.0,
    }

    if rank == 0 and world == 1 and not args.headline_only:
        line["extra"] = extra_legs(dev, peaks, warmup)
        times = time_cpu_path(3, 1)
        cpu_tflops = flops / statistics.median(times) / 1e12
        cpu_out = ao.cpu_dense(q0, k0, v0, causal=True)
        line["cpu_baseline"] = {
            "value": cpu_tflops, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": "median of 3 full forward passes of the headline workload through torch CPU SDPA on "
                      "bf16 tensors after one warm-up",
            "parity_vs_f64": stats_of(cpu_out, ao.ruler_dense(q0, k0, v0, causal=True)),
        }
    if world > 1 and not args.headline_only:
        extra = sharded_legs(dev, peaks, rank, world, warmup)
        ring = ring_leg(dev, peaks, rank, world)
        copies = host_copies_leg(dev, rank, world)
        if rank == 0:
            extra["ring_attention"] = ring
            extra["host_copies"] = copies
            line["extra"] = extra
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        from kohaku_tt_b200 import parallel

        parallel._PeerRing.release_all()   # the ring leg's shared slots, before the processes part
        torch.distributed.destroy_process_group()


# ---- multi-GPU legs -------------------------------------------------------------------------

def _max_min_over_ranks(ms, dev):
    t = torch.tensor([ms, -ms], dtype=torch.float64, device=dev)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return t[0].item(), -t[1].item()


def host_copies_leg(dev, rank, world):
    """Where the end-to-end rate of N ranks goes: the headline step's host-to-device and
    device-to-host copies alone (pinned buffers, one stream each way, no kernel), run by all
    ranks at once, by one rank at a time and by subsets. One rank alone shows what a GPU's
    link gives; the growth with the number of active ranks is the host's share (PCIe switches,
    root complex, memory), which no kernel can buy back."""
    import time

    c = HEADLINE
    n_in = c["batch"] * (c["heads"] + 2 * c["kv_heads"]) * c["seq"] * c["head_dim"]
    n_out = c["batch"] * c["heads"] * c["seq"] * c["head_dim"]
    hin, hout = torch.empty((n_in,), dtype=torch.bfloat16).pin_memory(), torch.empty((n_out,), dtype=torch.bfloat16).pin_memory()
    hin.fill_(1)
    hout.fill_(1)
    din, dout = torch.empty((n_in,), dtype=torch.bfloat16, device=dev), torch.empty((n_out,), dtype=torch.bfloat16, device=dev)
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()

    def loop(steps, h2d, d2h):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            if h2d:
                with torch.cuda.stream(s_in):
                    din.copy_(hin, non_blocking=True)
            if d2h:
                with torch.cuda.stream(s_out):
                    hout.copy_(dout, non_blocking=True)
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / steps * 1e6

    def case(active, h2d=True, d2h=True):
        torch.distributed.barrier()
        us = loop(200, h2d, d2h) if rank in active else 0.0
        t = torch.tensor([us], dtype=torch.float64, device=dev)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return round(t.item(), 1)

    loop(20, True, True)
    everyone = set(range(world))
    out = {
        "unit": "us per step on the slowest active rank (4.72 MB in, 3.67 MB out per rank and step)",
        "all_ranks": case(everyone),
        "all_ranks_h2d_only": case(everyone, d2h=False),
        "all_ranks_d2h_only": case(everyone, h2d=False),
        "one_rank_alone": [case({r}) for r in sorted({0, world // 2, world - 1})],
    }
    if world >= 4:
        out["first_two_ranks"] = case({0, 1})
        out["first_half_of_the_ranks"] = case(set(range(world // 2)))
        out["every_other_rank"] = case(set(range(0, world, 2)))
    return out


def sharded_legs(dev, peaks, rank, world, warmup):
    """The other configurations split over the GPUs the way they shard, with no collective
    on the data path: decode by whole sequences (batch 64 / N per GPU), SDXL self-attention
    by (batch, head) pairs (20 pairs over N), the packed batch by whole sequences balanced
    by sum L^2. Each reports the aggregate rate from the slowest rank's time, the fastest
    rank's time beside it, and this rank-0 shard's error statistics."""
    from kohaku_tt_b200 import ops, parallel
    from oracle import attention_oracle as ao

    out = {}
    # decode: B 64 over N GPUs
    g = torch.Generator().manual_seed(0)
    lengths = torch.randint(512, 4097, (64,), generator=g, dtype=torch.int32)
    lo, hi = parallel.shard_range(64, world, rank)
    mine = lengths[lo:hi]
    nb = hi - lo
    caches = [(device_randn((nb, 2, 4096, 128), 10 * rank + i, dev), device_randn((nb, 2, 4096, 128), 10 * rank + 5 + i, dev))
              for i in range(max(2, int(1.5 * L2_BYTES / (nb * 2 * 4096 * 128 * 2 * 2)) + 1))]
    q = seeded([(64, 16, 1, 128)], 3)[0][lo:hi].contiguous().to(dev)
    ln = mine.to(dev)
    ms, _ = timed_region(lambda i: ops.decode(q, *caches[i % len(caches)], key_lengths=ln), 50, warmup, 1, graph=True)
    ms /= 50
    slow, fast = _max_min_over_ranks(ms, dev)
    nbytes = float(lengths.sum()) * 2 * (128 + 128) * 2 + 2 * 64 * 16 * 128 * 2
    o, _ = ops.decode(q, *caches[0], key_lengths=ln)
    out["decode_kv_gbs_sharded"] = {
        "value": nbytes / (slow * 1e-3) / 1e9, "ms_slowest_rank": slow, "ms_fastest_rank": fast,
        "frac_of_measured_hbm_per_gpu": nbytes / (slow * 1e-3) / 1e9 / world / peaks["hbm"],
        "sequences_per_gpu": nb,
        "parity_vs_f64": stats_of(o, ao.ruler_lengths(q.cpu(), caches[0][0].cpu(), caches[0][1].cpu(), mine)),
    }
    del caches

    # SDXL self-attention: 20 (batch, head) pairs over N GPUs
    pairs = parallel.shard_pairs(2, 10, world)[rank]
    npairs = max(len(pairs), 1)
    xs = [tuple(device_randn((1, npairs, 4096, 64), 100 * rank + 3 * i + j, dev) for j in range(3)) for i in range(12)]
    ms, _ = timed_region(lambda i: ops.sdpa_forward(*xs[i % 12]), 30, warmup, 1, graph=True)
    ms /= 30
    slow, fast = _max_min_over_ranks(ms, dev)
    f = 4.0 * 20 * 4096 * 4096 * 64
    o, l = ops.sdpa_forward(*xs[0])
    out["sdxl_self_tflops_sharded"] = {
        "value": f / (slow * 1e-3) / 1e12, "ms_slowest_rank": slow, "ms_fastest_rank": fast,
        "pairs_per_gpu": len(pairs),
        "parity_vs_f64": rows_parity(o, l, *xs[0], [(0, 0), (0, npairs - 1)], [0, 1, 2047, 4095]),
    }
    del xs

    # packed batch: whole sequences balanced by sum L^2
    lens = packed_lengths()
    first, last = parallel.shard_sequences(lens, world)[rank]
    mine = lens[first:last]
    tokens = sum(mine)
    cu = torch.tensor([0] + list(torch.tensor(mine).cumsum(0)), dtype=torch.int32, device=dev)
    q, k, v, do = (device_randn((tokens, 16, 128), 200 * rank + j, dev) for j in range(4))
    ms_f, _ = timed_region(lambda i: ops.varlen_forward(q, k, v, cu, cu, max(mine), max(mine), causal=True), 10, warmup, 1, graph=True)
    ms_f /= 10
    o, l = ops.varlen_forward(q, k, v, cu, cu, max(mine), max(mine), causal=True)
    ms_b, _ = timed_region(lambda i: ops.varlen_backward(do, q, k, v, o, l, cu, cu, max(mine), max(mine), causal=True), 5, warmup, 1, graph=True)
    ms_b /= 5
    slow_f, fast_f = _max_min_over_ranks(ms_f, dev)
    slow_b, fast_b = _max_min_over_ranks(ms_b, dev)
    f = sum(4.0 * 16 * 128 * n * (n + 1) / 2 for n in lens)
    out["varlen_tflops_sharded"] = {
        "forward": {"value": f / (slow_f * 1e-3) / 1e12, "ms_slowest_rank": slow_f, "ms_fastest_rank": fast_f},
        "backward": {"value": 2.5 * f / (slow_b * 1e-3) / 1e12, "ms_slowest_rank": slow_b, "ms_fastest_rank": fast_b},
        "sequences_per_gpu": len(mine), "tokens_this_rank": tokens,
        "parity_vs_f64": packed_parity(o, q, k, v, do, mine, None, heads=(0, 15)),
    }
    return out


def ring_leg(dev, peaks, rank, world):
    """The long-context configuration: one causal sequence of 16,384 x N tokens (131,072 at
    N = 8), 16 heads, D 128, sharded zigzag over the N GPUs, K/V blocks passed around the
    ring by NCCL send/recv. Every rank takes part; times are the max over ranks. Parity:
    sampled query rows of two heads on every rank against float64 rows over the whole
    sequence's keys (gathered for those heads only), and full gradients of a down-scaled
    ring (1,024 tokens per rank, 2 heads) against float64 autograd."""
    from kohaku_tt_b200 import parallel
    from oracle import attention_oracle as ao

    tokens, heads, d = 16384, 16, 128
    q, k, v, do = (device_randn((1, heads, tokens, d), 100 + 7 * rank + j, dev) for j in range(4))
    seq = tokens * world
    fwd_flops = 4.0 * heads * d * (seq * (seq + 1) / 2)

    def timed(fn, steps):
        fn()
        torch.cuda.synchronize()
        torch.distributed.barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            fn()
        stop.record()
        torch.cuda.synchronize()
        t = torch.tensor([start.elapsed_time(stop) / steps], dtype=torch.float64, device=dev)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return t.item()

    ms_f = timed(lambda: parallel.ring_forward(q, k, v), 3)
    out, lse = parallel.ring_forward(q, k, v)
    ms_b = timed(lambda: parallel.ring_backward(do, q, k, v, out, lse), 3)

    # Forward parity on sampled rows: gather two heads' K / V from every rank, put the chunks
    # back in sequence order, evaluate this rank's sampled rows in float64.
    hs = [0, heads - 1]
    c = tokens // 2
    gathered = []
    for t in (k, v):
        mine = t[0, hs].contiguous()
        parts = [torch.empty_like(mine) for _ in range(world)]
        torch.distributed.all_gather(parts, mine)
        gathered.append(parallel.zigzag_merge([p_.cpu() for p_ in parts], dim=1))
    kf, vf = gathered
    local_rows = [0, 1, c - 1, c, c + 1, tokens - 1]
    chunk_a, chunk_b = parallel.zigzag_chunks(world, rank)
    global_rows = [r if r < c else (chunk_b * c + (r - c)) for r in local_rows]
    global_rows = [chunk_a * c + r if r < c else g for r, g in zip(local_rows, global_rows)]
    got, want, lse_err = [], [], 0.0
    for i, h in enumerate(hs):
        qr = q[0, h].cpu()[torch.tensor(local_rows)]
        o, l = ao.ruler_rows(qr, kf[i], vf[i], global_rows, causal=True)
        got.append(out[0, h].cpu()[torch.tensor(local_rows)])
        want.append(o)
        lse_err = max(lse_err, float((lse[0, h].cpu()[torch.tensor(local_rows)].double() - l).abs().max()))
    st = stats_of(torch.stack(got), torch.stack(want))
    worst = torch.tensor([st["abs_max"], st["rel_median"], lse_err, float(st["nonfinite"])], dtype=torch.float64, device=dev)
    torch.distributed.all_reduce(worst, op=torch.distributed.ReduceOp.MAX)

    # Gradients on a down-scaled ring against float64 autograd of the whole sequence.
    small, sh = 1024, 2
    g = torch.Generator().manual_seed(77)
    full = [torch.randn((1, sh, small * world, d), generator=g).to(torch.bfloat16) for _ in range(4)]
    shards = [parallel.zigzag_split(t, world, dim=2)[rank].to(dev) for t in full]
    so, sl = parallel.ring_forward(shards[0], shards[1], shards[2])
    gq, gk, gv = parallel.ring_backward(shards[3], shards[0], shards[1], shards[2], so, sl)
    ruler, dq, dk, dv = ao.grads_dense(full[0], full[1], full[2], full[3], causal=True)
    import kohaku_tt_b200 as ktt

    grad_err = [ktt.rel_rms(got_, parallel.zigzag_split(want_, world, dim=2)[rank])
                for got_, want_ in ((so, ruler), (gq, dq), (gk, dk), (gv, dv))]
    ge = torch.tensor(grad_err, dtype=torch.float64, device=dev)
    torch.distributed.all_reduce(ge, op=torch.distributed.ReduceOp.MAX)

    kv_bytes = 2 * tokens * heads * d * 2
    return {
        "workload": f"one causal sequence of {seq} tokens, 16 heads, D 128, zigzag over {world} GPUs",
        "forward_tflops": fwd_flops / (ms_f * 1e-3) / 1e12, "forward_ms": ms_f,
        "forward_frac_of_measured_bf16_per_gpu": fwd_flops / (ms_f * 1e-3) / 1e12 / world / peaks["bf16"],
        "backward_tflops": 2.5 * fwd_flops / (ms_b * 1e-3) / 1e12, "backward_ms": ms_b,
        "backward_frac_of_measured_bf16_per_gpu": 2.5 * fwd_flops / (ms_b * 1e-3) / 1e12 / world / peaks["bf16"],
        "ring_bytes_per_step_per_gpu": kv_bytes,
        "parity_vs_f64": {
            "abs_max": worst[0].item(), "rel_median": worst[1].item(), "lse_abs_max": worst[2].item(),
            "nonfinite": int(worst[3].item()),
            "sample": f"worst rank; per rank 2 heads x {len(local_rows)} query rows against float64 over all {seq} keys",
        },
        "small_ring_rel_rms_vs_f64": {"out": ge[0].item(), "dq": ge[1].item(), "dk": ge[2].item(), "dv": ge[3].item(),
                                      "workload": f"{small * world} tokens, {sh} heads, full float64 autograd, worst rank"},
    }


# ---- single-GPU legs --------------------------------------------------------------------------

def _time(fn, steps, warmup):
    return timed_region(fn, steps, warmup, 1, graph=True, min_ms=20.0)[0] / steps


def leg_fwd_bwd(dev, peaks, warmup):
    """Forward + backward on the headline shape (3.5 x the forward FLOPs)."""
    from kohaku_tt_b200 import ops
    from oracle import attention_oracle as ao

    c = HEADLINE
    sets = []
    for i in range(8):
        sets.append(seeded(
            [(1, c["heads"], c["seq"], 64), (1, c["kv_heads"], c["seq"], 64),
             (1, c["kv_heads"], c["seq"], 64), (1, c["heads"], c["seq"], 64)], 50 + i, dev))

    def fwd_bwd(i):
        q, k, v, do = sets[i % len(sets)]
        out, lse = ops.sdpa_forward(q, k, v, causal=True)
        ops.sdpa_backward(do, q, k, v, out, lse, causal=True)

    ms = _time(fwd_bwd, 30, warmup)
    f = 3.5 * causal_forward_flops(1, c["heads"], c["seq"], 64)
    # Gradients of one whole GQA group (7 query heads on K/V head 0) against float64 autograd.
    q, k, v, do = sets[0]
    out, lse = ops.sdpa_forward(q, k, v, causal=True)
    gq, gk, gv = ops.sdpa_backward(do, q, k, v, out, lse, causal=True)
    grp = c["heads"] // c["kv_heads"]
    ruler, dq, dk, dv = ao.grads_dense(q[:, :grp].cpu(), k[:, :1].cpu(), v[:, :1].cpu(), do[:, :grp].cpu(), causal=True)
    return {"value": f / (ms * 1e-3) / 1e12, "ms": ms,
            "frac_of_measured_bf16": f / (ms * 1e-3) / 1e12 / peaks["bf16"],
            "workload": "headline shape, forward + backward",
            "parity_vs_f64": {"out": stats_of(out[:, :grp], ruler), "dq": stats_of(gq[:, :grp], dq),
                              "dk": stats_of(gk[:, :1], dk), "dv": stats_of(gv[:, :1], dv),
                              "sample": "GQA group 0: 7 query heads and their K/V head, full float64 autograd"}}


def leg_fwd_b8(dev, peaks, warmup):
    """Headline shape at batch 8 (the whole-box batch on one GPU)."""
    from kohaku_tt_b200 import ops

    c = HEADLINE
    q8 = [seeded([(8, c["heads"], c["seq"], 64), (8, c["kv_heads"], c["seq"], 64), (8, c["kv_heads"], c["seq"], 64)], 60 + i, dev)
          for i in range(4)]
    ms = _time(lambda i: ops.sdpa_forward(*q8[i % 4], causal=True), 50, warmup)
    f = causal_forward_flops(8, c["heads"], c["seq"], 64)
    out, lse = ops.sdpa_forward(*q8[0], causal=True)
    return {"value": f / (ms * 1e-3) / 1e12, "ms": ms,
            "frac_of_measured_bf16": f / (ms * 1e-3) / 1e12 / peaks["bf16"],
            "parity_vs_f64": rows_parity(out, lse, *q8[0], [(0, 0), (3, 6), (7, 13)], [0, 127, 128, 1000, 2047], causal=True)}


def leg_fwd_d128(dev, peaks, warmup):
    """Dense causal forward at head dim 128: B 2, 16 heads, S 4096."""
    from kohaku_tt_b200 import ops

    xs = [tuple(device_randn((2, 16, 4096, 128), 300 + 3 * i + j, dev) for j in range(3)) for i in range(4)]
    ms = _time(lambda i: ops.sdpa_forward(*xs[i % 4], causal=True), 20, warmup)
    f = causal_forward_flops(2, 16, 4096, 128)
    out, lse = ops.sdpa_forward(*xs[0], causal=True)
    return {"value": f / (ms * 1e-3) / 1e12, "ms": ms,
            "frac_of_measured_bf16": f / (ms * 1e-3) / 1e12 / peaks["bf16"],
            "frac_of_measured_bf16_sustained": f / (ms * 1e-3) / 1e12 / peaks["bf16_sustained"],
            "workload": "B 2, 16 heads, S 4096, D 128, causal",
            "parity_vs_f64": rows_parity(out, lse, *xs[0], [(0, 0), (1, 15)], [0, 127, 128, 2047, 4095], causal=True)}


def leg_decode(dev, peaks, warmup):
    """Decode: batch 64, 16 / 2 heads, D 128, lengths uniform in [512, 4096]."""
    from kohaku_tt_b200 import ops
    from oracle import attention_oracle as ao

    g = torch.Generator().manual_seed(0)
    lengths = torch.randint(512, 4097, (64,), generator=g, dtype=torch.int32)
    # two caches, 268 MB each: nothing of a step's reads survives in L2
    caches = [(device_randn((64, 2, 4096, 128), i, dev), device_randn((64, 2, 4096, 128), 9 + i, dev)) for i in range(2)]
    q = seeded([(64, 16, 1, 128)], 3, dev)[0]
    ln = lengths.to(dev)
    ms = _time(lambda i: ops.decode(q, *caches[i % 2], key_lengths=ln), 50, warmup)
    nbytes = float(lengths.sum()) * 2 * (128 + 128) * 2 + 2 * q.numel() * 2
    gbs = nbytes / (ms * 1e-3) / 1e9
    out, _ = ops.decode(q, *caches[0], key_lengths=ln)
    ruler = ao.ruler_lengths(q.cpu(), caches[0][0].cpu(), caches[0][1].cpu(), lengths)
    return {"value": gbs, "ms": ms, "bytes": nbytes,
            "frac_of_measured_hbm": gbs / peaks["hbm"], "frac_of_nominal_8000": gbs / 8000.0,
            "workload": "B 64, 16 q heads / 2 kv heads, D 128, lengths U[512, 4096] seed 0",
            "parity_vs_f64": dict(stats_of(out, ruler), sample="all 64 x 16 (batch, head) pairs, full float64")}


def leg_plain_read(dev, peaks, warmup):
    """For scale beside the decode leg: a kernel that only reads the decode workload's byte
    count (two buffers alternating, so nothing survives in L2) with 16-byte grid-stride
    loads and does nothing else. The decode kernel cannot be faster than this on its bytes."""
    import ctypes

    from kohaku_tt_b200 import _lib

    g = torch.Generator().manual_seed(0)
    lengths = torch.randint(512, 4097, (64,), generator=g, dtype=torch.int32)
    nbytes = int(lengths.sum()) * 2 * (128 + 128) * 2
    bufs = [torch.full((nbytes // 4,), i + 1, dtype=torch.int32, device=dev) for i in range(2)]
    sink = torch.zeros((1,), dtype=torch.int32, device=dev)
    handle = _lib.lib()

    def read(i):
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        _lib.check(handle.ktt_b200_probe_read(ctypes.c_void_p(bufs[i % 2].data_ptr()), nbytes,
                                              ctypes.c_void_p(sink.data_ptr()), stream), "probe_read")

    ms = _time(read, 50, warmup)
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"value": gbs, "ms": ms, "bytes": float(nbytes), "frac_of_measured_hbm": gbs / peaks["hbm"],
            "workload": "read-only kernel over the decode leg's byte count, cold, 16-byte grid-stride loads"}


def leg_decode_step(dev, peaks, warmup):
    """One decode token with its neighbours: rotary on q and the new key, cache append,
    attention. The fused launch beside the same work as separate ops (rotary by torch
    elementwise ops twice, index_copy_ twice, then the decode kernel)."""
    import kohaku_tt_b200 as ktt
    from kohaku_tt_b200 import ops
    from oracle import attention_oracle as ao

    g = torch.Generator().manual_seed(0)
    lengths = torch.randint(512, 4096, (64,), generator=g, dtype=torch.int32)
    caches = [(device_randn((64, 2, 4096, 128), i, dev), device_randn((64, 2, 4096, 128), 9 + i, dev)) for i in range(2)]
    q, k_new, v_new = seeded([(64, 16, 1, 128), (64, 2, 1, 128), (64, 2, 1, 128)], 3, dev)
    pos = torch.arange(4096, dtype=torch.float32, device=dev)[:, None]
    inv = 1.0 / (10000.0 ** (torch.arange(0, 128, 2, dtype=torch.float32, device=dev) / 128))
    ang = torch.cat([pos * inv, pos * inv], dim=-1)
    cos, sin = ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)
    ln = lengths.to(dev)
    ln_next = ln + 1
    idx = ln.long()

    # Parity first, on a copy of cache 0 (the timed loops below overwrite the same rows with
    # the same values every step).
    kc, vc = caches[0][0].clone(), caches[0][1].clone()
    want, k_want, v_want = ao.decode_step(q.cpu(), k_new.cpu(), v_new.cpu(), kc.cpu(), vc.cpu(), lengths.tolist(),
                                          cos[idx].cpu(), sin[idx].cpu())
    got = ktt.decode_step(q, k_new, v_new, kc, vc, ln, cos, sin)
    parity = dict(stats_of(got, want), cache_rows_equal=bool(torch.equal(kc.cpu(), k_want) and torch.equal(vc.cpu(), v_want)),
                  sample="all 64 x 16 pairs, float64 over the updated cache")
    del kc, vc

    def fused(i):
        ktt.decode_step(q, k_new, v_new, *caches[i % 2], ln, cos, sin)

    def rotary(x, c, s_):
        xf = x.float()
        x1, x2 = xf.chunk(2, -1)
        return (xf * c + torch.cat([-x2, x1], -1) * s_).to(x.dtype)

    batch = torch.arange(64, device=dev)

    def separate(i):
        kc, vc = caches[i % 2]
        c, s_ = cos[idx][:, None, None, :].float(), sin[idx][:, None, None, :].float()
        q_rot, k_rot = rotary(q, c, s_), rotary(k_new, c, s_)
        kc[batch, :, idx] = k_rot[:, :, 0]
        vc[batch, :, idx] = v_new[:, :, 0]
        ops.decode(q_rot, kc, vc, key_lengths=ln_next)

    ms = _time(fused, 50, warmup)
    ms_sep = _time(separate, 50, warmup)
    nbytes = float((lengths + 1).sum()) * 2 * (128 + 128) * 2 + 2 * q.numel() * 2
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"value": gbs, "ms": ms, "separate_ops_ms": ms_sep, "bytes": nbytes,
            "frac_of_measured_hbm": gbs / peaks["hbm"],
            "workload": "decode leg's shape; new token at position lengths[b]",
            "parity_vs_f64": parity}


def leg_sdxl_self(dev, peaks, warmup):
    """SDXL self-attention: B 2, 10 heads, S 4096, D 64, head views of [B, S, 640]."""
    from kohaku_tt_b200 import ops

    xs = [seeded([(2, 4096, 3 * 640)], 70 + i, dev)[0].view(2, 4096, 3, 10, 64) for i in range(12)]
    views = lambda x: tuple(x[:, :, j].transpose(1, 2) for j in range(3))
    ms = _time(lambda i: ops.sdpa_forward(*views(xs[i % 12])), 30, warmup)
    f = 4.0 * 2 * 10 * 4096 * 4096 * 64
    out, lse = ops.sdpa_forward(*views(xs[0]))
    return {"value": f / (ms * 1e-3) / 1e12, "ms": ms,
            "frac_of_measured_bf16": f / (ms * 1e-3) / 1e12 / peaks["bf16"],
            "parity_vs_f64": rows_parity(out, lse, *views(xs[0]), [(0, 0), (1, 9)], [0, 1, 2047, 4095])}


def leg_sdxl_cross(dev, peaks, warmup):
    """SDXL cross-attention: 77 keys, the last 20 masked by a bool key-padding mask."""
    from kohaku_tt_b200 import ops
    from oracle import attention_oracle as ao

    q = seeded([(2, 10, 4096, 64)], 80, dev)[0]
    k, v = seeded([(2, 10, 77, 64)] * 2, 81, dev)
    keep = torch.ones(2, 1, 1, 77, dtype=torch.bool, device=dev)
    keep[..., 57:] = False
    ms = _time(lambda i: ops.sdpa_forward(q, k, v, mask=keep), 30, warmup)
    out, _ = ops.sdpa_forward(q, k, v, mask=keep)
    ruler = ao.ruler_dense(q.cpu(), k.cpu(), v.cpu(), mask=keep.cpu())
    return {"ms": ms, "gflop_kept_keys": 4.0 * 2 * 10 * 4096 * 57 * 64 / 1e9,
            "parity_vs_f64": dict(stats_of(out, ruler), sample="all 20 pairs, full float64")}


def packed_lengths():
    """Lengths U[64, 4096] (seed 0) drawn until 65,536 tokens; the last one truncated."""
    g = torch.Generator().manual_seed(0)
    lens, total = [], 0
    while total < 65536:
        n = int(torch.randint(64, 4097, (1,), generator=g))
        n = min(n, 65536 - total)
        lens.append(n)
        total += n
    if lens[-1] < 64 and len(lens) > 1:
        lens[-2] += lens.pop()
    return lens


def packed_parity(out, q, k, v, do, lens, grads, heads=(0, 15)):
    """Whole sequences (the shortest, the longest, the last) of a packed batch, two heads,
    against the float64 per-sequence ruler; with `grads` = (dq, dk, dv) also against its
    float64 autograd."""
    from oracle import attention_oracle as ao

    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    picks = sorted({min(range(len(lens)), key=lambda i: lens[i]), max(range(len(lens)), key=lambda i: lens[i]), len(lens) - 1})
    hs = list(heads)
    res = {"sample": f"sequences {picks} (lengths {[lens[i] for i in picks]}), heads {hs}, float64 per sequence"}
    worst = {}
    for i in picks:
        sl = slice(cu[i], cu[i + 1])
        qs, ks, vs = (t[sl][:, hs].cpu() for t in (q, k, v))
        c = [0, lens[i]]
        if grads is None:
            ruler = ao.ruler_varlen(qs, ks, vs, c, c, causal=True)
            pairs = [("out", out[sl][:, hs], ruler)]
        else:
            ruler, dq, dk, dv = ao.ruler_varlen(qs, ks, vs, c, c, causal=True, dout=do[sl][:, hs].cpu())
            pairs = [("out", out[sl][:, hs], ruler), ("dq", grads[0][sl][:, hs], dq),
                     ("dk", grads[1][sl][:, hs], dk), ("dv", grads[2][sl][:, hs], dv)]
        for name, got, want in pairs:
            st = stats_of(got, want)
            old = worst.get(name)
            if old is None or st["abs_max"] > old["abs_max"]:
                worst[name] = st
    res.update(worst)
    return res


def leg_varlen(dev, peaks, warmup):
    """Packed causal training attention: 16 heads, D 128, 65,536 tokens, lengths
    U[64, 4096] (seed 0), forward and backward."""
    from kohaku_tt_b200 import ops

    lens = packed_lengths()
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
    q, k, v, do = (device_randn((65536, 16, 128), 400 + j, dev) for j in range(4))
    f = sum(4.0 * 16 * 128 * n * (n + 1) / 2 for n in lens)
    ms = _time(lambda i: ops.varlen_forward(q, k, v, cu, cu, max(lens), max(lens), causal=True), 10, warmup)
    fwd = {"value": f / (ms * 1e-3) / 1e12, "ms": ms, "sequences": len(lens),
           "frac_of_measured_bf16": f / (ms * 1e-3) / 1e12 / peaks["bf16"]}
    out, lse = ops.varlen_forward(q, k, v, cu, cu, max(lens), max(lens), causal=True)
    ms = _time(lambda i: ops.varlen_backward(do, q, k, v, out, lse, cu, cu, max(lens), max(lens), causal=True), 5, warmup)
    bwd = {"value": 2.5 * f / (ms * 1e-3) / 1e12, "ms": ms,
           "frac_of_measured_bf16": 2.5 * f / (ms * 1e-3) / 1e12 / peaks["bf16"]}
    grads = ops.varlen_backward(do, q, k, v, out, lse, cu, cu, max(lens), max(lens), causal=True)
    return {"forward": fwd, "backward": bwd, "parity_vs_f64": packed_parity(out, q, k, v, do, lens, grads)}


def leg_masked_training(dev, peaks, warmup):
    """A masked training step: key-padding mask (one row per batch entry), forward +
    backward, B 4, 16 / 4 heads, S 2048, D 128, keys past 0.7 S masked in even batches."""
    from kohaku_tt_b200 import ops
    from oracle import attention_oracle as ao

    b, h, hk, s, d = 4, 16, 4, 2048, 128
    q, k, v, do = seeded([(b, h, s, d), (b, hk, s, d), (b, hk, s, d), (b, h, s, d)], 90, dev)
    keep = torch.ones(b, 1, 1, s, dtype=torch.bool, device=dev)
    keep[::2, ..., int(0.7 * s):] = False

    def stepf(i):
        out, lse = ops.sdpa_forward(q, k, v, mask=keep)
        ops.sdpa_backward(do, q, k, v, out, lse, mask=keep)

    ms = _time(stepf, 10, warmup)
    kept = float(keep.sum()) / b
    f = 3.5 * 4.0 * b * h * s * kept * d
    out, lse = ops.sdpa_forward(q, k, v, mask=keep)
    gq, gk, gv = ops.sdpa_backward(do, q, k, v, out, lse, mask=keep)
    grp = h // hk
    ruler, dq, dk, dv = ao.grads_dense(q[:1, :grp].cpu(), k[:1, :1].cpu(), v[:1, :1].cpu(), do[:1, :grp].cpu(), mask=keep[:1].cpu())
    return {"value": f / (ms * 1e-3) / 1e12, "ms": ms, "frac_of_measured_bf16": f / (ms * 1e-3) / 1e12 / peaks["bf16"],
            "workload": "B 4, 16 / 4 heads, S 2048, D 128, bool key-padding mask, forward + backward; FLOPs over kept keys",
            "parity_vs_f64": {"out": stats_of(out[:1, :grp], ruler), "dq": stats_of(gq[:1, :grp], dq),
                              "dk": stats_of(gk[:1, :1], dk), "dv": stats_of(gv[:1, :1], dv),
                              "sample": "batch 0, GQA group 0, full float64 autograd"}}


LEGS = {
    "fwd_bwd_tflops": leg_fwd_bwd,
    "fwd_b8_tflops": leg_fwd_b8,
    "fwd_d128_tflops": leg_fwd_d128,
    "decode_kv_gbs": leg_decode,
    "decode_step_gbs": leg_decode_step,
    "plain_read_gbs": leg_plain_read,
    "sdxl_self_tflops": leg_sdxl_self,
    "sdxl_cross_ms": leg_sdxl_cross,
    "varlen_tflops": leg_varlen,
    "masked_training_tflops": leg_masked_training,
}


def extra_legs(dev, peaks, warmup):
    """The other configurations of the benchmark plan, each timed the same way."""
    out = {}
    for name, fn in LEGS.items():
        out[name] = fn(dev, peaks, warmup)
        torch.cuda.empty_cache()
    return out


def run_leg(args):
    """`--leg NAME`: one extra leg alone (for profiling a single kernel family)."""
    torch.cuda.set_device(0)
    import kohaku_tt_b200 as ktt

    ktt.build()
    ktt.install()
    print(json.dumps({args.leg: LEGS[args.leg](torch.device("cuda", 0), measured_peaks(), max(args.warmup, 3))}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--eager", action="store_true", help="time eager launches instead of a CUDA graph replay")
    ap.add_argument("--headline-only", action="store_true", help="skip the extra legs and the CPU baseline")
    ap.add_argument("--e2e-streams", type=int, default=0,
                    help="0: copy-in / compute / copy-out streams chained by events; N > 0: whole steps issued round-robin on N streams")
    ap.add_argument("--leg", default=None, choices=sorted(LEGS), help="run one extra leg alone and print it")
    args = ap.parse_args()
    if args.leg:
        run_leg(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
