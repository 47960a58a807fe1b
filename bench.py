"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline workload (N = 1): the Qwen2.5-0.5B-shaped GQA causal prefill forward, B = 1,
14 query heads / 2 KV heads, D = 64, S = 2048, bf16, seeded N(0, 1) inputs. A step is one
forward pass over one batch; with N > 1 every rank runs its own batch (weak scaling, no
collective). The line also carries the forward+backward, decode, SDXL and packed
workloads as `extra` legs, a roofline for the dominant kernel, and the reference's CPU
path (PyTorch CPU SDPA on the same bf16 tensors) timed on this box's host cores.

`--impl reference` times only that CPU path, on the headline workload.
"""

import argparse
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


def causal_forward_flops(b, h, s, d):
    """2 FLOP per multiply-add, QK^T + PV over visible (query, key) pairs only."""
    return 4.0 * b * h * d * (s * (s + 1) / 2)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            m = json.load(f)
        return {"bf16": m["bf16_tflops"], "bf16_sustained": m["bf16_tflops_sustained"],
                "hbm": m["hbm_gbs"], "source": "measured"}
    return {"bf16": 1590.0, "bf16_sustained": 1400.0, "hbm": 6650.0, "source": "fallback"}


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


def headline_inputs(seed, device=None, pin=False):
    from oracle import attention_oracle as ao

    c = HEADLINE
    q, k, v = ao.make_inputs(
        [(c["batch"], c["heads"], c["seq"], c["head_dim"]),
         (c["batch"], c["kv_heads"], c["seq"], c["head_dim"]),
         (c["batch"], c["kv_heads"], c["seq"], c["head_dim"])], seed)
    if device is not None:
        return q.to(device), k.to(device), v.to(device)
    if pin:
        return q.pin_memory(), k.pin_memory(), v.pin_memory()
    return q, k, v


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
    rank, world, _ = dist_env()
    if rank != 0:
        return
    c = HEADLINE
    flops = causal_forward_flops(c["batch"], c["heads"], c["seq"], c["head_dim"])
    times = time_cpu_path(args.steps, max(args.warmup, 1))
    total = sum(times)
    value = flops * len(times) / total / 1e12
    cores = torch.get_num_threads()
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
                      f"on bf16 tensors ({os.cpu_count()} host CPUs visible)",
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
        "launch": "the K timed steps are one CUDA graph replay (K kernel launches back to back)",
        "parallelism": "one batch per GPU, no collective",
    }


def timed_region(fn, steps, warmup, world, graph=False, fork=None, join=None):
    """W untimed calls, then K calls between two events on the current stream, bracketed
    by a barrier and a device synchronize; returns milliseconds (max over ranks). With
    `graph` the K calls are captured once into a CUDA graph and the timed region is its
    replay, so the device sees K back-to-back launches without host gaps. `fork` / `join`
    make side streams start after the start event and finish before the stop event."""
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
    if world > 1:
        torch.distributed.barrier()
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
    ms = start.elapsed_time(stop)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        torch.distributed.barrier()
        ms = t.item()
    return ms


def run_ours(args):
    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
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
    parity = ktt.diff_stats(out, ao.ruler_dense(q0, k0, v0, causal=True))

    ktt.reset_counters()
    ms = timed_region(step, steps, warmup, world, graph=not args.eager)
    launches = sum(ktt.counters()[k] for k in ("attention_flash", "attention_mma")) - warmup
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
    lanes = 3
    streams = [torch.cuda.Stream(device=dev) for _ in range(lanes)]
    out_host = [torch.empty((c["batch"], c["heads"], c["seq"], c["head_dim"]), dtype=torch.bfloat16).pin_memory()
                for _ in range(lanes)]

    def e2e_step(i):
        with torch.cuda.stream(streams[i % lanes]):
            flat = host[i % 4].to(dev, non_blocking=True)
            q, k, v = (flat[off:off + n].view(sh) for off, n, sh in
                       zip((0, counts[0], counts[0] + counts[1]), counts, shapes))
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

    e2e_steps = max(20, steps)
    e2e_ms = timed_region(e2e_step, e2e_steps, warmup, world, fork=e2e_fork, join=e2e_join)
    e2e_value = flops * e2e_steps * world / (e2e_ms * 1e-3) / 1e12
    h2d = host[0].numel() * host[0].element_size()
    d2h = out_host[0].numel() * out_host[0].element_size()

    line = {
        "metric": "attn_fwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": per_launch_ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": workload_config(),
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / e2e_steps,
                "api": "torch.nn.functional.scaled_dot_product_attention on CUDA tensors, steps issued round-robin on 3 streams"},
        "gpu_launches": launches,
        "clocks": clocks,
        "kernel": kernel,
        "parity_vs_f64": {k: parity[k] for k in ("abs_max", "rel_median", "cosine", "nonfinite")},
    }
    achieved = flops / (per_launch_ms * 1e-3) / 1e12
    line["roofline"] = {
        "bound": "tensor", "achieved": achieved, "peak": peaks["bf16"], "unit": "TFLOP/s",
        "frac": achieved / peaks["bf16"],
        # DRAM bytes of one launch from the ncu capture summarised in
        # profiles/fwd_tc5_headline.md (dram__bytes_read.sum + dram__bytes_write.sum; the
        # output stays in L2 at this size). Algorithmic bytes are 8.4 MB: no re-reads.
        "traffic": 4775936 if kernel == "tcgen05" and c["batch"] == 1 else None,
        "traffic_unit": "bytes per launch (ncu)",
        "peak_source": f"{peaks['source']} cuBLAS bf16 burst", "frac_of_nominal_2250": achieved / 2250.0,
    }

    if rank == 0 and world == 1 and not args.headline_only:
        line["extra"] = extra_legs(dev, peaks, warmup)
        times = time_cpu_path(3, 1)
        cpu_tflops = flops / statistics.median(times) / 1e12
        cpu_out = ao.cpu_dense(q0, k0, v0, causal=True)
        cpu_parity = ktt.diff_stats(cpu_out, ao.ruler_dense(q0, k0, v0, causal=True))
        line["cpu_baseline"] = {
            "value": cpu_tflops, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": "median of 3 full forward passes of the headline workload through torch CPU SDPA on "
                      "bf16 tensors after one warm-up",
            "parity_vs_f64": {k: cpu_parity[k] for k in ("abs_max", "rel_median", "cosine")},
        }
    if world > 1 and not args.headline_only:
        ring = ring_leg(dev, peaks, rank, world)
        if rank == 0:
            line.setdefault("extra", {})["ring_attention"] = ring
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()


def ring_leg(dev, peaks, rank, world):
    """The long-context configuration: one causal sequence of 16,384 x N tokens (131,072 at
    N = 8), 16 heads, D 128, sharded zigzag over the N GPUs, K/V blocks passed around the
    ring by NCCL send/recv. Every rank takes part; times are the max over ranks."""
    from kohaku_tt_b200 import parallel

    tokens, heads, d = 16384, 16, 128
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    q, k, v, do = (torch.randn((1, heads, tokens, d), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
                   for _ in range(4))
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
    ms_b = timed(lambda: parallel.ring_backward(do, q, k, v, out, lse), 1)
    kv_bytes = 2 * tokens * heads * d * 2
    return {
        "workload": f"one causal sequence of {seq} tokens, 16 heads, D 128, zigzag over {world} GPUs",
        "forward_tflops": fwd_flops / (ms_f * 1e-3) / 1e12, "forward_ms": ms_f,
        "forward_frac_of_measured_bf16_per_gpu": fwd_flops / (ms_f * 1e-3) / 1e12 / world / peaks["bf16"],
        "backward_tflops": 2.5 * fwd_flops / (ms_b * 1e-3) / 1e12, "backward_ms": ms_b,
        "ring_bytes_per_step_per_gpu": kv_bytes,
    }


def _time(fn, steps, warmup):
    return timed_region(fn, steps, warmup, 1, graph=True) / steps


def leg_fwd_bwd(dev, peaks, warmup):
    """Forward + backward on the headline shape (3.5 x the forward FLOPs)."""
    from kohaku_tt_b200 import ops
    from oracle import attention_oracle as ao

    c = HEADLINE
    sets = []
    for i in range(8):
        q, k, v, do = ao.make_inputs(
            [(1, c["heads"], c["seq"], 64), (1, c["kv_heads"], c["seq"], 64),
             (1, c["kv_heads"], c["seq"], 64), (1, c["heads"], c["seq"], 64)], 50 + i)
        sets.append(tuple(t.to(dev) for t in (q, k, v, do)))

    def fwd_bwd(i):
        q, k, v, do = sets[i % len(sets)]
        out, lse = ops.sdpa_forward(q, k, v, causal=True)
        ops.sdpa_backward(do, q, k, v, out, lse, causal=True)

    ms = _time(fwd_bwd, 30, warmup)
    f = 3.5 * causal_forward_flops(1, c["heads"], c["seq"], 64)
    return {"value": f / (ms * 1e-3) / 1e12, "ms": ms,
            "frac_of_measured_bf16": f / (ms * 1e-3) / 1e12 / peaks["bf16"],
            "workload": "headline shape, forward + backward"}


def leg_fwd_b8(dev, peaks, warmup):
    """Headline shape at batch 8 (the whole-box batch on one GPU)."""
    from kohaku_tt_b200 import ops
    from oracle import attention_oracle as ao

    c = HEADLINE
    q8 = []
    for i in range(4):
        q, k, v = ao.make_inputs(
            [(8, c["heads"], c["seq"], 64), (8, c["kv_heads"], c["seq"], 64), (8, c["kv_heads"], c["seq"], 64)], 60 + i)
        q8.append((q.to(dev), k.to(dev), v.to(dev)))
    ms = _time(lambda i: ops.sdpa_forward(*q8[i % 4], causal=True), 50, warmup)
    f = causal_forward_flops(8, c["heads"], c["seq"], 64)
    return {"value": f / (ms * 1e-3) / 1e12, "ms": ms,
            "frac_of_measured_bf16": f / (ms * 1e-3) / 1e12 / peaks["bf16"]}


def leg_decode(dev, peaks, warmup):
    """Decode: batch 64, 16 / 2 heads, D 128, lengths uniform in [512, 4096]."""
    from kohaku_tt_b200 import ops
    from oracle import attention_oracle as ao

    g = torch.Generator().manual_seed(0)
    lengths = torch.randint(512, 4097, (64,), generator=g, dtype=torch.int32)
    caches = []
    for i in range(2):  # two caches, 268 MB each: nothing of a step's reads survives in L2
        k = torch.randn((64, 2, 4096, 128), generator=torch.Generator(device=dev).manual_seed(i), device=dev, dtype=torch.float32).to(torch.bfloat16)
        v = torch.randn((64, 2, 4096, 128), generator=torch.Generator(device=dev).manual_seed(9 + i), device=dev, dtype=torch.float32).to(torch.bfloat16)
        caches.append((k, v))
    q = ao.make_inputs([(64, 16, 1, 128)], 3)[0].to(dev)
    ln = lengths.to(dev)
    ms = _time(lambda i: ops.decode(q, *caches[i % 2], key_lengths=ln), 50, warmup)
    nbytes = float(lengths.sum()) * 2 * (128 + 128) * 2 + 2 * q.numel() * 2
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"value": gbs, "ms": ms, "bytes": nbytes,
            "frac_of_measured_hbm": gbs / peaks["hbm"], "frac_of_nominal_8000": gbs / 8000.0,
            "workload": "B 64, 16 q heads / 2 kv heads, D 128, lengths U[512, 4096] seed 0"}


def leg_decode_step(dev, peaks, warmup):
    """One decode token with its neighbours: rotary on q and the new key, cache append,
    attention. The fused launch beside the same work as separate ops (rotary by torch
    elementwise ops twice, index_copy_ twice, then the decode kernel)."""
    import kohaku_tt_b200 as ktt
    from kohaku_tt_b200 import ops
    from oracle import attention_oracle as ao

    g = torch.Generator().manual_seed(0)
    lengths = torch.randint(512, 4096, (64,), generator=g, dtype=torch.int32)
    caches = []
    for i in range(2):
        k = torch.randn((64, 2, 4096, 128), generator=torch.Generator(device=dev).manual_seed(i), device=dev, dtype=torch.float32).to(torch.bfloat16)
        v = torch.randn((64, 2, 4096, 128), generator=torch.Generator(device=dev).manual_seed(9 + i), device=dev, dtype=torch.float32).to(torch.bfloat16)
        caches.append((k, v))
    q, k_new, v_new = (t.to(dev) for t in ao.make_inputs([(64, 16, 1, 128), (64, 2, 1, 128), (64, 2, 1, 128)], 3))
    pos = torch.arange(4096, dtype=torch.float32, device=dev)[:, None]
    inv = 1.0 / (10000.0 ** (torch.arange(0, 128, 2, dtype=torch.float32, device=dev) / 128))
    ang = torch.cat([pos * inv, pos * inv], dim=-1)
    cos, sin = ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)
    ln = lengths.to(dev)
    ln_next = ln + 1
    idx = ln.long()

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
            "workload": "decode leg's shape; new token at position lengths[b]"}


def leg_sdxl_self(dev, peaks, warmup):
    """SDXL self-attention: B 2, 10 heads, S 4096, D 64, head views of [B, S, 640]."""
    from kohaku_tt_b200 import ops
    from oracle import attention_oracle as ao

    xs = [ao.make_inputs([(2, 4096, 3 * 640)], 70 + i)[0].to(dev).view(2, 4096, 3, 10, 64) for i in range(12)]
    ms = _time(lambda i: ops.sdpa_forward(*(xs[i % 12][:, :, j].transpose(1, 2) for j in range(3))), 30, warmup)
    f = 4.0 * 2 * 10 * 4096 * 4096 * 64
    return {"value": f / (ms * 1e-3) / 1e12, "ms": ms,
            "frac_of_measured_bf16": f / (ms * 1e-3) / 1e12 / peaks["bf16"]}


def leg_sdxl_cross(dev, peaks, warmup):
    """SDXL cross-attention: 77 keys, the last 20 masked by a bool key-padding mask."""
    from kohaku_tt_b200 import ops
    from oracle import attention_oracle as ao

    q = ao.make_inputs([(2, 10, 4096, 64)], 80)[0].to(dev)
    k, v = (t.to(dev) for t in ao.make_inputs([(2, 10, 77, 64)] * 2, 81))
    keep = torch.ones(2, 1, 1, 77, dtype=torch.bool, device=dev)
    keep[..., 57:] = False
    ms = _time(lambda i: ops.sdpa_forward(q, k, v, mask=keep), 30, warmup)
    return {"ms": ms, "gflop_kept_keys": 4.0 * 2 * 10 * 4096 * 57 * 64 / 1e9}


def leg_varlen(dev, peaks, warmup):
    """Packed causal training attention: 16 heads, D 128, 65,536 tokens, lengths
    U[64, 4096] (seed 0), forward and backward."""
    from kohaku_tt_b200 import ops

    g = torch.Generator().manual_seed(0)
    lens, total = [], 0
    while total < 65536:
        n = int(torch.randint(64, 4097, (1,), generator=g))
        n = min(n, 65536 - total)
        lens.append(n)
        total += n
    if lens[-1] < 64 and len(lens) > 1:
        lens[-2] += lens.pop()
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
    q, k, v, do = (torch.randn((65536, 16, 128), device=dev, dtype=torch.float32).to(torch.bfloat16) for _ in range(4))
    f = sum(4.0 * 16 * 128 * n * (n + 1) / 2 for n in lens)
    ms = _time(lambda i: ops.varlen_forward(q, k, v, cu, cu, max(lens), max(lens), causal=True), 10, warmup)
    fwd = {"value": f / (ms * 1e-3) / 1e12, "ms": ms, "sequences": len(lens),
           "frac_of_measured_bf16": f / (ms * 1e-3) / 1e12 / peaks["bf16"]}
    out, lse = ops.varlen_forward(q, k, v, cu, cu, max(lens), max(lens), causal=True)
    ms = _time(lambda i: ops.varlen_backward(do, q, k, v, out, lse, cu, cu, max(lens), max(lens), causal=True), 5, warmup)
    bwd = {"value": 2.5 * f / (ms * 1e-3) / 1e12, "ms": ms,
           "frac_of_measured_bf16": 2.5 * f / (ms * 1e-3) / 1e12 / peaks["bf16"]}
    return {"forward": fwd, "backward": bwd}


LEGS = {
    "fwd_bwd_tflops": leg_fwd_bwd,
    "fwd_b8_tflops": leg_fwd_b8,
    "decode_kv_gbs": leg_decode,
    "decode_step_gbs": leg_decode_step,
    "sdxl_self_tflops": leg_sdxl_self,
    "sdxl_cross_ms": leg_sdxl_cross,
    "varlen_tflops": leg_varlen,
}


def extra_legs(dev, peaks, warmup):
    """The other configurations of the benchmark plan, each timed the same way."""
    return {name: fn(dev, peaks, warmup) for name, fn in LEGS.items()}


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
