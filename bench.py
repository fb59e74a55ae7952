"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--skip-extras]

One "step" is one forward + backward pass of causal attention at the headline configuration
(batch 2, 16 heads, sequence 2048, head_dim 128, fp16, bottom-right causal mask, seeded N(0,1) inputs).
With N > 1 (launched under torchrun, one rank per GPU) every rank runs the same step on its own batch
(the path partitions by batch x head and needs no communication), so scaling is weak and the reported
value is N x FLOPs / max-over-ranks time.

The single JSON line printed by rank 0 carries
  value      device-resident throughput: algorithmic FLOPs of fwd+bwd / CUDA-event time of the four kernels
  e2e        the same metric through the public API with pinned HOST buffers (H2D of q, k, v, dO and D2H of
             O, dQ, dK, dV inside the timed region)
  roofline   the dominant kernel against the measured tensor-core peak (kernels are timed one by one)
  kernels    every kernel of the step: time, algorithmic work, achieved rate
  decode     secondary headline numbers: split-K and paged decode KV GB/s against the measured HBM peak
  cpu_baseline  the fp32 math-attention oracle on the host cores, on a bounded sample of the same workload

`--impl reference` times that CPU path alone (the reference's kernels cannot run without an AMD GPU; its
CPU-capable path is fp32 math attention, which the oracle restates).
"""
import argparse
import ctypes as C
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "flash-attention-rdna3_b200"))

import torch
import torch.nn.functional as F

METRIC = "fwd/bwd TFLOP/s (% tcgen05 peak) 2x16x2048x128 causal; decode KV GB/s (% HBM)"
B, H, S, D = 2, 16, 2048, 128
FWD_FLOPS = 4 * B * H * S * S * D / 2          # causal: half of 4*B*H*S^2*D
BWD_FLOPS = 2.5 * FWD_FLOPS                    # reference convention (bench/benchmark.py:123 of fa_rdna3)
STEP_FLOPS = FWD_FLOPS + BWD_FLOPS
# Algorithmic share of the backward matmuls: dK/dV kernel = S^T, dP^T, dV, dK (4 of 5), dQ kernel = dQ (1 of 5: with
# the dS scratch it is exactly that GEMM; without it, its recomputed S and dP are not counted).
KERNEL_FLOPS = {"fwd": FWD_FLOPS, "bwd_dkdv": 0.8 * BWD_FLOPS, "bwd_dq": 0.2 * BWD_FLOPS}
DELTA_BYTES = 2 * B * H * S * D * 2 + B * H * S * 4   # reads O and dO, writes delta

# dram__bytes_read.sum + dram__bytes_write.sum per launch of this workload, from ncu captures of these kernels at this
# size (a constant, not measured per run). Reads match the operand sizes (every input once); most of the output is
# still in the write-back L2 when the kernel ends, so the write counter is below the output size.
NCU_TRAFFIC_BYTES = {"fwd": 51.6e6, "bwd_dkdv": 199.0e6, "bwd_dq": 171.8e6}   # with the dS scratch in use


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"tflops": d["bf16_tflops"], "tflops_sustained": d.get("bf16_tflops_sustained"),
                "hbm_gbs": d["hbm_gbs"], "source": "measured"}
    return {"tflops": 1590.0, "tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        clocks, cmax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(float(parts[0]))
                cmax = float(parts[1])
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": cmax,
                "reasons": sorted(reasons), "samples": len(clocks)}


def seeded(seed, *shape, dtype=torch.float16):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32).to(dtype)


# ---------------------------------------------------------------------------------------------------------
# CPU arm: fp32 math attention (the oracle) on the host cores, bounded sample of the headline workload
# ---------------------------------------------------------------------------------------------------------
def cpu_sample_step(heads):
    """One fwd+bwd of batch 1 x `heads` heads x 2048 x 128 causal in fp32; returns (seconds, flops)."""
    from oracle.attention_oracle import attention_grads_ref

    q, k, v, dout = (seeded(1002 + i, 1, heads, S, D).float() for i in range(4))
    t0 = time.perf_counter()
    attention_grads_ref(q, k, v, dout, causal=True, softmax_scale=1.0 / math.sqrt(D))
    dt = time.perf_counter() - t0
    return dt, STEP_FLOPS * heads / (B * H)


def cpu_baseline(steps=3, heads=8):
    torch.set_num_threads(os.cpu_count() or 1)
    cpu_sample_step(1)  # warm-up
    times, flops = [], 0.0
    for _ in range(steps):
        dt, flops = cpu_sample_step(heads)
        times.append(dt)
    t = statistics.median(times)
    return {"value": flops / t / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"fp32 math attention fwd+bwd (autograd) of 1 batch x {heads} heads of the "
                      f"{B}x{H}x{S}x{D} causal workload, median of {steps}; FLOPs counted as for the GPU arm"}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    heads = 2
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_sample_step(1)
    times, flops = [], 0.0
    for _ in range(args.steps):
        dt, flops = cpu_sample_step(heads)
        times.append(dt)
    total = sum(times)
    value = flops * args.steps / total / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"fwd+bwd causal attention {B}x{H}x{S}x{D}, seeded N(0,1); each step is a bounded "
                               f"sample of 1 batch x {heads} heads on the host cores"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"1 batch x {heads} heads per step, fp32 math attention with autograd backward"},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------------
class Flusher:
    """Writes a buffer larger than L2 (126 MB) so the next timed launch starts from a cold cache. The write
    also gives the host time to queue the next launch behind it, so launch latency is not timed."""

    def __init__(self, device, mbytes=512):
        self.buf = torch.empty(mbytes * 1024 * 1024, dtype=torch.uint8, device=device)

    def __call__(self):
        self.buf.zero_()


def timed(fn, flush, stream_events=True):
    flush()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    fn()
    e.record()
    return s, e


def gpu_arm(args):
    import fa_b200
    from fa_b200 import _lib, interface

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    distributed = world > 1
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if distributed:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
    reason = fa_b200.unsupported_reason(device)
    if reason is not None:
        raise RuntimeError(reason)
    lib = _lib.load()
    peaks = load_peaks()
    scale = 1.0 / math.sqrt(D)

    # every rank owns its own batch: weak scaling over batch x heads, no data-path collective
    host = [seeded(1002 + 10 * rank + i, B, H, S, D).pin_memory() for i in range(4)]
    q, k, v, dout = (t.to(device) for t in host)
    flush = Flusher(device)
    stream = torch.cuda.current_stream(device)

    # one parameter block reused by every launch: outputs and scratch are allocated once
    out = torch.empty_like(q)
    lse = torch.empty(B, H, S, dtype=torch.float32, device=device)
    delta = torch.empty_like(lse)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    p = interface._attn_params(q, k, v, out, lse, True, scale, (-1, -1), 0.0, None, None, 0.0, 0)
    interface._fill_backward(p, dout, delta, dq, dk, dv, False)
    # the dS scratch of the dense backward (dQ = dS K as one GEMM), as the public API attaches it
    ds_scratch = interface._ds_workspace(p, device)
    sptr = C.c_void_p(stream.cuda_stream)

    def launch_fwd():
        _lib.check(lib.fa_fwd(C.byref(p), sptr))

    def launch_bwd(parts):
        p.bwd_parts = parts
        _lib.check(lib.fa_bwd(C.byref(p), sptr))

    parts = [("fwd", launch_fwd), ("bwd_delta", lambda: launch_bwd(_lib.FA_BWD_DELTA)),
             ("bwd_dkdv", lambda: launch_bwd(_lib.FA_BWD_DKDV)), ("bwd_dq", lambda: launch_bwd(_lib.FA_BWD_DQ))]

    all_parts = _lib.FA_BWD_DELTA | _lib.FA_BWD_DKDV | _lib.FA_BWD_DQ
    calls = [("fwd", launch_fwd), ("bwd", lambda: launch_bwd(all_parts))]

    def step():
        """One fwd+bwd pass as a caller makes it: one fa_fwd call and one fa_bwd call (delta, dK/dV and dQ
        kernels), each timed on its own behind an L2 flush."""
        return [(name, *timed(fn, flush)) for name, fn in calls]

    def breakdown():
        """The four kernels launched one by one, each behind its own flush (not part of the timed steps)."""
        return [(name, *timed(fn, flush)) for name, fn in parts]

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    if interface.last_kernel_path() != "tcgen05":
        raise RuntimeError("the headline configuration did not run on the tcgen05 kernels")
    if distributed:
        dist.barrier()
    torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    recorded = [step() for _ in range(args.steps)]
    torch.cuda.synchronize()
    if distributed:
        dist.barrier()
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    fa_b200.check_status(device)

    per_call = {name: [] for name, _ in calls}
    step_ms = []
    for evs in recorded:
        total = 0.0
        for name, s, e in evs:
            ms = s.elapsed_time(e)
            per_call[name].append(ms)
            total += ms
        step_ms.append(total)
    # per-kernel times for the roofline and the shares (separate launches, outside the timed steps)
    broken = [breakdown() for _ in range(min(args.steps, 10))]
    torch.cuda.synchronize()
    per_kernel = {name: [s.elapsed_time(e) for evs in broken for n, s, e in evs if n == name] for name, _ in parts}
    fa_b200.check_status(device)

    def graph_us(fn, reps=10):
        """`reps` launches of one kernel replayed from a CUDA graph: device time without launch gaps (warm L2)."""
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            inner = C.c_void_p(torch.cuda.current_stream(device).cuda_stream)
            for _ in range(reps):
                fn(inner)
        graph.replay()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        graph.replay()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / reps * 1e3

    def captured(parts_mask):
        def fn(inner):
            if parts_mask is None:
                _lib.check(lib.fa_fwd(C.byref(p), inner))
            else:
                p.bwd_parts = parts_mask
                _lib.check(lib.fa_bwd(C.byref(p), inner))
        return fn

    graph_replay = {"fwd": graph_us(captured(None)), "bwd_delta": graph_us(captured(_lib.FA_BWD_DELTA)),
                    "bwd_dkdv": graph_us(captured(_lib.FA_BWD_DKDV)), "bwd_dq": graph_us(captured(_lib.FA_BWD_DQ)),
                    "bwd": graph_us(captured(all_parts))}
    total_ms = torch.tensor([sum(step_ms)], dtype=torch.float64, device=device)
    if distributed:
        dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)
    total_ms = float(total_ms.item())
    ms_per_step = total_ms / args.steps
    value = world * STEP_FLOPS / (ms_per_step * 1e-3) / 1e12

    # end to end through the public API: every step copies Q, K, V, dO from pinned host memory, runs
    # flash_attention(...).backward() and copies O, dQ, dK, dV back to pinned host memory. Steps are pipelined the
    # way a loader feeds a device: copies in, compute and copies out run on three streams over two sets of device
    # buffers, so step i+1's upload overlaps step i's download (PCIe is full duplex); an L2 flush precedes every
    # step's compute.
    host_out = [[torch.empty(B, H, S, D, dtype=torch.float16).pin_memory() for _ in range(4)] for _ in range(2)]
    dev_in = [[torch.empty(B, H, S, D, dtype=torch.float16, device=device) for _ in range(4)] for _ in range(2)]
    s_main = torch.cuda.current_stream(device)
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)

    def e2e_run(n_steps):
        """Queues n_steps pipelined steps; returns (start, end) events on the main stream."""
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(s_main)
        s_in.wait_stream(s_main)
        s_out.wait_stream(s_main)
        computed = [None, None]   # event: compute of the step that last used buffer set i is finished
        drained = [None, None]    # event: results of the step that last used host set i are on the host
        keep = []
        for i in range(n_steps):
            b = i & 1
            with torch.cuda.stream(s_in):
                if computed[b] is not None:
                    s_in.wait_event(computed[b])
                for dst, src in zip(dev_in[b], host):
                    dst.copy_(src, non_blocking=True)
                uploaded = torch.cuda.Event()
                uploaded.record(s_in)
            s_main.wait_event(uploaded)
            flush()
            qd, kd, vd = (t.detach().requires_grad_(True) for t in dev_in[b][:3])
            o = fa_b200.flash_attention(qd, kd, vd, causal=True)
            o.backward(dev_in[b][3])
            results = (o.detach(), qd.grad, kd.grad, vd.grad)
            computed[b] = torch.cuda.Event()
            computed[b].record(s_main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(computed[b])
                if drained[b] is not None:
                    s_out.wait_event(drained[b])
                for dst, src in zip(host_out[b], results):
                    dst.copy_(src, non_blocking=True)
                    src.record_stream(s_out)
                drained[b] = torch.cuda.Event()
                drained[b].record(s_out)
            keep.append(results)
        s_main.wait_stream(s_out)
        s_main.wait_stream(s_in)
        end.record(s_main)
        return start, end

    e2e_run(3)
    torch.cuda.synchronize()
    if distributed:
        dist.barrier()
    s, e = e2e_run(args.steps)
    torch.cuda.synchronize()
    e2e_total = torch.tensor([s.elapsed_time(e)], dtype=torch.float64, device=device)
    if distributed:
        dist.all_reduce(e2e_total, op=dist.ReduceOp.MAX)
    e2e_value = world * STEP_FLOPS / (float(e2e_total.item()) / args.steps * 1e-3) / 1e12

    def copies_only(n_steps):
        """The same uploads and downloads with no compute in between (one copy per tensor, the two directions on
        their own streams): the PCIe floor of a step at this number of GPUs."""
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(s_main)
        s_in.wait_stream(s_main)
        s_out.wait_stream(s_main)
        for i in range(n_steps):
            b = i & 1
            with torch.cuda.stream(s_in):
                for dst, src in zip(dev_in[b], host):
                    dst.copy_(src, non_blocking=True)
            with torch.cuda.stream(s_out):
                for dst, src in zip(host_out[b], dev_in[b ^ 1]):
                    dst.copy_(src, non_blocking=True)
        s_main.wait_stream(s_out)
        s_main.wait_stream(s_in)
        end.record(s_main)
        return start, end

    copies_only(2)
    torch.cuda.synchronize()
    if distributed:
        dist.barrier()
    s, e = copies_only(args.steps)
    torch.cuda.synchronize()
    copy_total = torch.tensor([s.elapsed_time(e)], dtype=torch.float64, device=device)
    if distributed:
        dist.all_reduce(copy_total, op=dist.ReduceOp.MAX)
    copy_ms_per_step = float(copy_total.item()) / args.steps
    e2e_ms_per_step = float(e2e_total.item()) / args.steps
    e2e_check = float(host_out[(args.steps - 1) & 1][0].float().abs().sum())  # the results did reach the host
    if not math.isfinite(e2e_check) or e2e_check == 0.0:
        raise RuntimeError("end-to-end outputs did not arrive in host memory")
    tensor_bytes = B * H * S * D * 2

    sharded, sharded_configs = None, None
    if distributed and not args.skip_extras:
        sharded = sharded_decode_extra(device, rank, world)
        sharded_configs = sharded_config_extras(device, rank, world, flush, peaks)
        from fa_b200 import distributed as _fd
        _fd.release_peer_buffers()   # collective: nobody exits while a peer still maps its gather buffers

    if rank != 0:
        if distributed:
            dist.destroy_process_group()
        return

    kernels = {}
    for name, times in per_kernel.items():
        ms = statistics.mean(times)
        entry = {"ms": ms, "share": ms / sum(statistics.mean(t) for t in per_kernel.values())}
        if name in KERNEL_FLOPS:
            entry["algorithmic_flops"] = KERNEL_FLOPS[name]
            entry["tflops"] = KERNEL_FLOPS[name] / (ms * 1e-3) / 1e12
        else:
            entry["algorithmic_bytes"] = DELTA_BYTES
            entry["gbs"] = DELTA_BYTES / (ms * 1e-3) / 1e9
        kernels[name] = entry
    dominant = max(KERNEL_FLOPS, key=lambda n: kernels[n]["ms"])
    achieved = kernels[dominant]["tflops"]
    roofline = {"bound": "tensor", "kernel": dominant, "achieved": achieved, "peak": peaks["tflops"],
                "unit": "TFLOP/s", "frac": achieved / peaks["tflops"], "traffic": NCU_TRAFFIC_BYTES.get(dominant),
                "peak_source": f"{peaks['source']} bf16 burst GEMM", "frac_of_nominal_2250": achieved / 2250.0}

    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"fwd+bwd causal attention {B}x{H}x{S}x{D} fp16 per GPU, seeded N(0,1) "
                               "(the configuration the metric is quoted on)", "l2": "512 MB flush before the fa_fwd call and before the fa_bwd call of every step",
                   "parallelism": f"batch x head partition over {world} GPU(s), no collective"},
        "frac_of_measured_peak": value / world / peaks["tflops"],
        "fwd_tflops": FWD_FLOPS / (statistics.mean(per_call["fwd"]) * 1e-3) / 1e12,
        "bwd_tflops": BWD_FLOPS / (statistics.mean(per_call["bwd"]) * 1e-3) / 1e12,
        "calls_ms": {name: statistics.mean(t) for name, t in per_call.items()},
        "kernels": kernels, "kernels_note": "each kernel launched alone behind its own L2 flush, outside the timed steps",
        "graph_replay_us": graph_replay,
        "graph_replay_note": "ten launches of each kernel (and of the whole fa_bwd call) replayed from one CUDA graph: "
                             "device time without launch gaps, inputs warm in L2", "roofline": roofline, "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": 4 * tensor_bytes,
                "d2h_bytes_per_step": 4 * tensor_bytes,
                "ms_per_step": e2e_ms_per_step, "copies_only_ms_per_step": copy_ms_per_step,
                "pcie_gbs_each_way_all_gpus": world * 4 * tensor_bytes / copy_ms_per_step / 1e6,
                "frac_of_copy_bound": copy_ms_per_step / e2e_ms_per_step,
                "note": "steps pipelined over three streams and two buffer sets; time = first upload to last download; "
                        "copies_only = the same host<->device copies of every rank with no compute (max over ranks): "
                        "the ranks of one node share the host's memory and PCIe paths, which is what bounds e2e"},
        "gpu_launches": 4 * args.steps,
        "bwd_ds_scratch_bytes": int(p.ds_workspace_bytes) if ds_scratch is not None else 0,
    }
    if not args.skip_extras and world == 1:
        line["decode"] = decode_extras(device, flush, peaks)
        line["configs"] = baseline_configs(device, flush, peaks)
        line["other_shapes"] = other_shapes(device)
        line["cpu_baseline"] = cpu_baseline()
    if sharded is not None:
        line["decode_kv_sharded"] = sharded
    if sharded_configs is not None:
        line["configs_sharded"] = sharded_configs
    print(json.dumps(line))
    if distributed:
        dist.destroy_process_group()


def sharded_decode_extra(device, rank, world, iters=20):
    """Long-context paged decode with the KV pages of every sequence sharded block-cyclically over the ranks
    (strong scaling of one fixed problem: 4 sequences x 262144 tokens, 32/8 heads, 16-token pages, 4.3 GB of KV):
    local partial -> every rank stores its (O, LSE) into the peers' gather buffers over NVLink and raises a flag ->
    bounded wait and local merge (no collective; "push"), or one NCCL all-gather in its place ("nccl", also timed).
    Every rank holds the whole pool here but reads only the pages of its own blocks. Time = max over ranks of the
    CUDA-event time of `iters` calls."""
    import torch.distributed as dist

    from fa_b200 import distributed as fd

    Bp, Hq, Hk, Dd, bs, ctx_len = 4, 32, 8, 128, 16, 262144
    maxb = ctx_len // bs
    nblocks = Bp * maxb
    g = torch.Generator().manual_seed(1006)
    q = torch.randn(Bp, Hq, Dd, generator=g).half().to(device)
    table = torch.randperm(nblocks, generator=g).to(torch.int32).reshape(Bp, maxb).to(device)
    ctx = torch.full((Bp,), ctx_len, dtype=torch.int32, device=device)
    # the same pools on every rank (same device-side seed), so that "rank r owns blocks r, r + G, ..." describes one
    # problem and the sharded result can be compared with the one-GPU call
    dg = torch.Generator(device=device).manual_seed(1006)
    pools = [(torch.randn(nblocks, bs, Hk, Dd, device=device, dtype=torch.float16, generator=dg),
              torch.randn(nblocks, bs, Hk, Dd, device=device, dtype=torch.float16, generator=dg)) for _ in range(2)]
    for kc, vc in pools:
        got = fd.paged_decode_kv_sharded(q, kc, vc, table, ctx)    # checks that the ranks agree, warms up NCCL
    # every rank holds the whole pool here, so the sharded result can be held against the one-GPU call before timing
    import fa_b200

    whole = fa_b200.flash_attention_decode_paged(q, pools[-1][0], pools[-1][1], table, ctx, max_context_len=ctx_len)
    max_err = float((got.float() - whole.float()).abs().max())
    if not max_err <= 2e-3:
        raise RuntimeError(f"KV-sharded decode differs from the single-GPU result by {max_err}")
    def timed(transport):
        for kc, vc in pools:   # warm-up of this transport
            fd.paged_decode_kv_sharded(q, kc, vc, table, ctx, check_ranks_agree=False, transport=transport)
        torch.cuda.synchronize()
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for i in range(iters):
            kc, vc = pools[i & 1]
            fd.paged_decode_kv_sharded(q, kc, vc, table, ctx, check_ranks_agree=False, transport=transport)
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / iters], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # the default transport: peer stores where every rank could set them up, else the all-gather
    pushed = len(fd._peer_gathers) > 0
    ms = timed(None)
    ms_nccl = timed("nccl") if pushed else ms
    nbytes = Bp * ctx_len * 2 * Hk * Dd * 2
    return {"us": ms * 1e3, "gbs_all_gpus": nbytes / ms / 1e6, "kv_bytes": nbytes, "n_gpus": world,
            "max_abs_vs_single_gpu": max_err, "transport": "push" if pushed else "nccl",
            "us_with_nccl_all_gather": ms_nccl * 1e3,
            "workload": "paged decode, 4 seqs x 262144 tokens, 32/8 heads, page 16, pages sharded block-cyclically",
            "collective": ("none: the local kernels write this rank's (O, LSE) into its own slot, fa_peer_merge stores "
                           "it into every peer's buffer over NVLink, raises a flag, waits for the peers' flags and "
                           "merges") if pushed else
                          ("the local kernels write into the gather buffer, one in-place all_gather of "
                           "batch*heads*(head_dim+1) floats per rank, local merge"), "scaling": "strong"}


def sharded_config_extras(device, rank, world, flush, peaks, iters=10):
    """The two benchmark configurations that partition with no exchange, as strong scaling of one fixed problem:
    split-K decode 4x32x8192x128 by (batch, head) and the packed causal + window + ALiBi + soft-cap configuration
    (8 sequences, 32/8 heads, bf16, forward + backward) by kv-head group. Every rank builds the whole problem from the
    same seeds and runs its own slice; time = max over ranks (CUDA events behind an L2 flush, median of `iters`)."""
    import torch.distributed as dist

    import fa_b200
    from fa_b200 import distributed as fd

    def median_ms(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        times = []
        for _ in range(iters):
            flush()
            torch.cuda._sleep(600000)   # lets the host queue the launches before the start event fires
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e))
        t = torch.tensor([statistics.median(times)], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def randn(g, *shape, dtype=torch.float16):
        return torch.randn(*shape, generator=g, dtype=torch.float32).to(dtype).to(device)

    res = {}
    # split-K decode: the 128 (batch, head) pairs are dealt to the ranks (MHA: a kv head per query head)
    g = torch.Generator().manual_seed(1004)
    Bd, Hd, Sk = 4, 32, 8192
    q = randn(g, Bd, Hd, 1, 128)
    k, v = randn(g, Bd, Hd, Sk, 128), randn(g, Bd, Hd, Sk, 128)
    lo, hi = fd.partition_batch_heads(Bd, Hd, world, rank)
    qs, ks, vs = (t.reshape(1, Bd * Hd, *t.shape[2:])[:, lo:hi] for t in (q, k, v))
    with torch.no_grad():
        ms = median_ms(lambda: fa_b200.flash_attention_decode(qs, ks, vs))
    nbytes = 2 * Bd * Hd * Sk * 128 * 2
    res["c3a_splitk_4x32x8192x128_by_batch_x_head"] = {
        "us": ms * 1e3, "gbs_all_gpus": nbytes / ms / 1e6, "frac_hbm_per_gpu": nbytes / ms / 1e6 / world / peaks["hbm_gbs"]}
    del q, k, v, qs, ks, vs

    seed = 1007
    while True:
        g = torch.Generator().manual_seed(seed)
        lengths = torch.randint(128, 4097, (8,), generator=g).tolist()
        if sum(lengths) <= 16384:
            break
        seed += 1
    T = sum(lengths)
    q, k, v, dout = (randn(g, T, h, 128, dtype=torch.bfloat16) for h in (32, 8, 8, 32))
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32, device=device)
    slopes = fa_b200.alibi_slopes(32, device=device)
    per = 8 // world                      # kv heads per rank (world is 2, 4 or 8)
    kvs, qsl = slice(rank * per, (rank + 1) * per), slice(rank * per * 4, (rank + 1) * per * 4)
    ql, kl, vl, dl = (t[:, sl].contiguous() for t, sl in ((q, qsl), (k, kvs), (v, kvs), (dout, qsl)))
    ql.requires_grad_(True), kl.requires_grad_(True), vl.requires_grad_(True)
    ms = median_ms(lambda: fa_b200.flash_attention_varlen(ql, kl, vl, cu, cu, max(lengths), max(lengths), causal=True,
                                                          window_size=(1023, 0), softcap=30.0,
                                                          alibi_slopes=slopes[qsl]).backward(dl))
    pairs = sum(L * (L + 1) // 2 if L <= 1024 else 1024 * 1025 // 2 + (L - 1024) * 1024 for L in lengths)
    flops = 3.5 * 4.0 * 32 * 128 * pairs
    res["c5_fwd_bwd_varlen_by_kv_head"] = {"us": ms * 1e3, "tflops_all_gpus": flops / ms / 1e9}
    res["note"] = "strong scaling of one fixed problem; no collective on the data path; time = max over ranks"
    return res


def _splitk_entry(res, device, lib, run, run_graph, entry, sm, nsets, Bd, Hd, Sk, Dd):
    """Split-K decode, MHA 4x32x16384x128, through the C ABI (see decode_extras)."""
    from fa_b200 import _lib, interface

    q = seeded(1004, Bd, Hd, 1, Dd).to(device)
    out = torch.empty_like(q)
    splits = interface._decode_splits_b200(Bd, Hd, 1, Sk, sm, tensor_core=True)
    op = torch.empty(splits, Bd, Hd, 1, Dd, dtype=torch.float32, device=device)
    lp = torch.empty(splits, Bd, Hd, 1, dtype=torch.float32, device=device)
    sets, params = [], []
    for i in range(nsets):
        k, v = (torch.randn(Bd, Hd, Sk, Dd, device=device, dtype=torch.float16) for _ in range(2))
        sets.append((k, v))
        p = _lib.DecodeParams()
        p.dtype = _lib.FA_F16
        p.batch, p.heads_q, p.heads_kv, p.seqlen_q, p.seqlen_k, p.head_dim = Bd, Hd, Hd, 1, Sk, Dd
        p.q, p.k, p.v, p.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
        for f, t in ((p.q_strides, q), (p.k_strides, k), (p.v_strides, v), (p.o_strides, out)):
            for j, st in enumerate(t.stride()):
                f[j] = st
        p.softmax_scale, p.num_splits = 1.0 / math.sqrt(Dd), splits
        p.o_partial, p.lse_partial = op.data_ptr(), lp.data_ptr()
        params.append(p)
    ms = run(lib.fa_decode_splitk, params)
    ms_graph = run_graph(lib.fa_decode_splitk, params)
    nbytes = 2 * Bd * Hd * Sk * Dd * 2
    res["splitk_4x32x16384x128"] = entry(ms, ms_graph, nbytes, splits)



def decode_extras(device, flush, peaks, iters=40, nsets=4, splitk=True):
    """Split-K decode (4x32x16384x128) and paged decode (4 seqs, 32/8 heads, page 16, 16384 tokens each) through the
    C ABI: `iters` launches back to back over `nsets` different K/V sets (each set is larger than L2, so every
    launch streams its K/V from HBM); GB/s counts K and V bytes once (kv heads)."""
    from fa_b200 import _lib, interface

    lib = _lib.load()
    sptr = C.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    sm = torch.cuda.get_device_properties(device).multi_processor_count
    res = {}

    def run(launch, params):
        for p in params:
            _lib.check(launch(C.byref(p), sptr))
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for i in range(iters):
            _lib.check(launch(C.byref(params[i % len(params)]), sptr))
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / iters

    def run_graph(launch, params):
        """The same `iters` launches recorded once by stream capture and replayed: no per-launch host work."""
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            sp = C.c_void_p(torch.cuda.current_stream(device).cuda_stream)
            for i in range(iters):
                _lib.check(launch(C.byref(params[i % len(params)]), sp))
        graph.replay()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        graph.replay()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / iters

    def entry(ms, ms_graph, nbytes, splits):
        return {"us": ms * 1e3, "gbs": nbytes / ms / 1e6, "frac_hbm": nbytes / ms / 1e6 / peaks["hbm_gbs"],
                "frac_hbm_nominal_8000": nbytes / ms / 1e6 / 8000.0, "graph_replay_us": ms_graph * 1e3,
                "num_splits": splits}

    Bd, Hd, Sk, Dd = 4, 32, 16384, 128
    if splitk:
        _splitk_entry(res, device, lib, run, run_graph, entry, sm, nsets, Bd, Hd, Sk, Dd)

    # paged decode, GQA 32/8: full contexts and the ragged contexts of the paged benchmark configuration, through the
    # balanced tensor-core kernel the public entry point uses (one CTA per SM, dealt to the sequences on the device)
    Bp, Hq, Hk, bs, maxb = 4, 32, 8, 16, 1024
    nblocks = Bp * maxb
    qp = seeded(1009, Bp, Hq, Dd).to(device)
    outp = torch.empty_like(qp)
    g = torch.Generator().manual_seed(1006)
    ragged = torch.randint(1, 16385, (Bp,), generator=g).to(torch.int32)
    table = torch.randperm(nblocks, generator=g).to(torch.int32).reshape(Bp, maxb).to(device)
    splits = interface._paged_balanced_slots(Hk, bs, maxb, sm, 16384)
    op = torch.empty(Bp, Hq, splits, Dd, dtype=torch.float32, device=device)
    lp = torch.empty(Bp, Hq, splits, dtype=torch.float32, device=device)
    pools = [tuple(torch.randn(nblocks, bs, Hk, Dd, device=device, dtype=torch.float16) for _ in range(2))
             for _ in range(nsets)]
    for name, lens in (("paged_4x32/8x16384x128", torch.full((Bp,), 16384, dtype=torch.int32)),
                       ("paged_4x32/8_ragged_contexts", ragged)):
        ctx = lens.to(device)
        params = []
        for kc, vc in pools:
            p = _lib.PagedParams()
            p.dtype = _lib.FA_F16
            p.batch, p.heads_q, p.heads_kv, p.head_dim = Bp, Hq, Hk, Dd
            p.num_blocks, p.block_size, p.max_blocks = nblocks, bs, maxb
            p.q, p.k_cache, p.v_cache, p.out = qp.data_ptr(), kc.data_ptr(), vc.data_ptr(), outp.data_ptr()
            p.block_table, p.context_lens = table.data_ptr(), ctx.data_ptr()
            for j, st in enumerate(qp.stride()):
                p.q_strides[j] = st
                p.o_strides[j] = outp.stride(j)
            for j in range(4):
                p.k_strides[j], p.v_strides[j] = kc.stride(j), vc.stride(j)
            p.bt_strides[0], p.bt_strides[1] = table.stride()
            p.cl_stride = 1
            p.softmax_scale, p.num_splits, p.first_block, p.block_step = 1.0 / math.sqrt(Dd), splits, 0, 1
            p.o_partial, p.lse_partial = op.data_ptr(), lp.data_ptr()
            p.balance = 1
            params.append(p)
        ms = run(lib.fa_decode_paged, params)
        ms_graph = run_graph(lib.fa_decode_paged, params)
        res[name] = entry(ms, ms_graph, int(lens.sum()) * 2 * Hk * Dd * 2, splits)
        res[name]["context_lens"] = lens.tolist()
    res["note"] = ("KV bytes read once (kv heads); %d launches back to back over %d K/V sets of 0.27-1.07 GB each "
                   "(larger than L2); frac_hbm = of the measured copy bandwidth, frac_hbm_nominal_8000 = of 8 TB/s; "
                   "graph_replay_us = the same launches replayed from one CUDA graph" % (iters, nsets))
    return res


def _fp32_reference_c5(q, k, v, slopes, window_left, softcap):
    """fp32 math attention of one packed sequence (heads first) with the modifiers of the varlen configuration,
    written out here so that the benchmark does not depend on the test oracle: scale, tanh soft-cap, ALiBi,
    causal + left window, softmax, P V. q (Hq, L, D), k / v (Hkv, L, D) in fp32."""
    Hq, L, Dh = q.shape
    group = Hq // k.shape[0]
    kk, vv = k.repeat_interleave(group, 0), v.repeat_interleave(group, 0)
    s = torch.matmul(q, kk.transpose(1, 2)) / math.sqrt(Dh)
    s = softcap * torch.tanh(s / softcap)
    pos = torch.arange(L, device=q.device)
    dist = (pos[None, :] - pos[:, None]).abs().float()
    s = s - slopes[:, None, None] * dist[None]
    keep = (pos[None, :] <= pos[:, None]) & (pos[None, :] >= pos[:, None] - window_left)
    s = s.masked_fill(~keep[None], float("-inf"))
    return torch.matmul(torch.softmax(s, -1), vv)


def baseline_configs(device, flush, peaks, iters=10):
    """Every other benchmark configuration through the public Python API, each launch behind an L2 flush (median of
    `iters`): time, algorithmic FLOPs or KV bytes, achieved rate and its fraction of the measured peak. Seeds and
    shapes are those of tests/test_baseline_configs_gpu.py, which holds the same calls to the oracle."""
    import fa_b200

    def median_us(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        times = []
        for _ in range(iters):
            flush()
            # The calls below go through Python (validation, allocation of outputs and scratch, ctypes, autograd): a
            # spin of about 1 ms on the device (no memory traffic, the cache stays cold) lets the host queue the
            # launches before the start event fires, so host time is not counted as kernel time.
            torch.cuda._sleep(2000000)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e) * 1e3)
        return statistics.median(times)

    def tensor(us, flops):
        return {"us": us, "algorithmic_flops": flops, "tflops": flops / us / 1e6,
                "frac_of_measured_tensor_peak": flops / us / 1e6 / peaks["tflops"]}

    def hbm(us, nbytes):
        return {"us": us, "kv_bytes": nbytes, "gbs": nbytes / us / 1e3, "frac_hbm": nbytes / us / 1e3 / peaks["hbm_gbs"],
                "frac_hbm_nominal_8000": nbytes / us / 1e3 / 8000.0}

    def randn(g, *shape, dtype=torch.float16):
        return torch.randn(*shape, generator=g, dtype=torch.float32).to(dtype).to(device)

    res = {}
    with torch.no_grad():
        g = torch.Generator().manual_seed(1001)
        q, k, v = (randn(g, 1, 16, 1024, 64) for _ in range(3))
        res["c1_fwd_1x16x1024x64_noncausal_fp16"] = tensor(median_us(lambda: fa_b200.flash_attention(q, k, v)),
                                                            4.0 * 16 * 1024 * 1024 * 64)
        # the ComfyUI tensor layout, (batch, tokens, heads * head_dim), through the model-patch adapter: the shapes
        # of the reference's bench/benchmark.py:43-89 (self-attention and cross-attention over 77 prompt tokens)
        from fa_b200.comfyui import ComfyUIAttentionOverride

        def no_fallback(*args, **kwargs):
            raise RuntimeError("the ComfyUI adapter fell back in the benchmark")

        override = ComfyUIAttentionOverride()
        g = torch.Generator().manual_seed(1002)
        for tokens_k in (77, 4096):
            q, k, v = randn(g, 2, 4096, 8 * 64), randn(g, 2, tokens_k, 8 * 64), randn(g, 2, tokens_k, 8 * 64)
            entry = tensor(median_us(lambda: override(no_fallback, q, k, v, 8)), 4.0 * 2 * 8 * 4096 * tokens_k * 64)

            def heads_of(t):
                return t.view(2, t.shape[1], 8, 64).transpose(1, 2)

            entry["torch_sdpa_us"] = median_us(
                lambda: F.scaled_dot_product_attention(heads_of(q), heads_of(k), heads_of(v)).transpose(1, 2).reshape(
                    2, 4096, 512))
            want = F.scaled_dot_product_attention(heads_of(q).float(), heads_of(k).float(), heads_of(v).float())
            got = override(no_fallback, q, k, v, 8)
            entry["max_abs_err_vs_fp32"] = float((heads_of(got).float() - want).abs().max())
            res["comfyui_layout_2x4096x(8x64)_keys%d_fp16" % tokens_k] = entry
        del q, k, v, want, got
    g = torch.Generator().manual_seed(1003)
    q, k, v, dout = (randn(g, 1, 16, 4096, 64) for _ in range(4))
    flops = 4.0 * 16 * 4096 * 4096 * 64 / 2
    with torch.no_grad():
        res["c2b_fwd_1x16x4096x64_causal_fp16"] = tensor(median_us(lambda: fa_b200.flash_attention(q, k, v, causal=True)),
                                                          flops)
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    res["c2b_fwd_bwd_1x16x4096x64_causal_fp16"] = tensor(
        median_us(lambda: fa_b200.flash_attention(q, k, v, causal=True).backward(dout)), 3.5 * flops)
    del q, k, v, dout

    with torch.no_grad():
        for name, seed, Bd, Hd, Sk in (("c3a_splitk_4x32x8192x128", 1004, 4, 32, 8192),
                                       ("c3b_splitk_1x8x16384x128", 1005, 1, 8, 16384)):
            g = torch.Generator().manual_seed(seed)
            q = randn(g, Bd, Hd, 1, 128)
            k, v = randn(g, Bd, Hd, Sk, 128), randn(g, Bd, Hd, Sk, 128)
            res[name] = hbm(median_us(lambda: fa_b200.flash_attention_decode(q, k, v)), 2 * Bd * Hd * Sk * 128 * 2)
        del q, k, v

        g = torch.Generator().manual_seed(1006)
        ctx = torch.randint(1, 16385, (4,), generator=g).to(torch.int32)
        kc, vc = randn(g, 4096, 16, 8, 128), randn(g, 4096, 16, 8, 128)
        table = torch.randperm(4096, generator=g).to(torch.int32).reshape(4, 1024).to(device)
        q = randn(g, 4, 32, 128)
        ctx_d = ctx.to(device)
        entry = hbm(median_us(lambda: fa_b200.flash_attention_decode_paged(q, kc, vc, table, ctx_d, max_context_len=16384)),
                    int(ctx.sum()) * 2 * 8 * 128 * 2)
        entry["context_lens"] = ctx.tolist()
        res["c4_paged_4x32/8_ragged_contexts_page16"] = entry
        del kc, vc

        g = torch.Generator().manual_seed(7)
        q, k, v = (randn(g, 2, 8, 19, 128, dtype=torch.float32) for _ in range(3))
        res["tiny_fp32_2x8x19x128"] = {"us": median_us(lambda: fa_b200.flash_attention(q, k, v))}

    # packed causal + window 1024 + ALiBi + soft-cap 30, bf16, 32/8 heads
    seed = 1007
    while True:
        g = torch.Generator().manual_seed(seed)
        lengths = torch.randint(128, 4097, (8,), generator=g).tolist()
        if sum(lengths) <= 16384:
            break
        seed += 1
    T = sum(lengths)
    q, k, v, dout = (randn(g, T, h, 128, dtype=torch.bfloat16) for h in (32, 8, 8, 32))
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32, device=device)
    slopes = fa_b200.alibi_slopes(32, device=device)
    pairs = sum(L * (L + 1) // 2 if L <= 1024 else 1024 * 1025 // 2 + (L - 1024) * 1024 for L in lengths)
    flops = 4.0 * 32 * 128 * pairs

    def c5():
        return fa_b200.flash_attention_varlen(q, k, v, cu, cu, max(lengths), max(lengths), causal=True,
                                              window_size=(1023, 0), softcap=30.0, alibi_slopes=slopes)

    with torch.no_grad():
        entry = tensor(median_us(c5), flops)
        # worst absolute error of O against fp32 math attention (true fp32 matmuls), longest sequence
        old_tf32 = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        b = max(range(8), key=lambda i: lengths[i])
        sl = slice(int(cu[b]), int(cu[b]) + lengths[b])
        ref = _fp32_reference_c5(q[sl].float().transpose(0, 1), k[sl].float().transpose(0, 1),
                                 v[sl].float().transpose(0, 1), slopes, 1023, 30.0)
        got = c5()[sl].float().transpose(0, 1)
        entry["max_abs_err_o_vs_fp32_longest_sequence"] = float((got - ref).abs().max())
        entry["max_abs_o"] = float(ref.abs().max())
        torch.backends.cuda.matmul.allow_tf32 = old_tf32
        entry["lengths"] = lengths
        res["c5_fwd_varlen_8seq_32/8x128_window1024_alibi_softcap30_bf16"] = entry
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    res["c5_fwd_bwd_varlen_8seq_32/8x128_window1024_alibi_softcap30_bf16"] = tensor(
        median_us(lambda: c5().backward(dout)), 3.5 * flops)
    res["note"] = ("public Python API, every launch behind a 512 MB L2 flush and a 1 ms device-side spin that hides "
                   "the host's launch work, median of %d; FLOPs count visible "
                   "(query, key) pairs only; KV bytes are read once per kv head" % iters)
    return res


def other_shapes(device, tokens=2048, batch=2, heads=16, repeats=5):
    """Forward and forward+backward times of the shapes beside the headline one, through the Python API: head dims
    the tensor-core kernels take unpadded (32, 80), the wide kernels (160, 256: one query tile per CTA forward, scores
    + products over a scratch buffer backward) and the tiled CUDA-core kernels (fp32, 512). Median of `repeats` calls
    (warm L2), each between CUDA events behind a device-side spin that lets the host queue the call's launches first:
    a forward + backward through autograd is several hundred microseconds of host work, more than the kernels take."""
    import fa_b200

    def timed(fn):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        times = []
        for _ in range(repeats):
            torch.cuda._sleep(2000000)   # about 1 ms; no memory traffic
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3)
        return statistics.median(times)

    out = {}
    for head_dim, dtype in ((32, torch.float16), (80, torch.float16), (160, torch.float16), (256, torch.float16),
                            (512, torch.float16), (128, torch.float32)):
        gen = torch.Generator(device=device).manual_seed(head_dim)
        q, k, v, dout = (torch.randn(batch, heads, tokens, head_dim, device=device, dtype=dtype, generator=gen)
                         for _ in range(4))
        q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
        with torch.no_grad():
            fwd_us = timed(lambda: fa_b200.flash_attention(q, k, v, causal=True))
        both_us = timed(lambda: fa_b200.flash_attention(q, k, v, causal=True).backward(dout))
        flops = 4.0 * batch * heads * tokens * tokens * head_dim / 2
        out[f"{batch}x{heads}x{tokens}x{head_dim}_{str(dtype)[6:]}_causal"] = {
            "fwd_us": fwd_us, "fwd_tflops": flops / fwd_us / 1e6,
            "fwd_bwd_us": both_us, "fwd_bwd_tflops": 3.5 * flops / both_us / 1e6}
    # fp32 inputs with the tensor-core switch on (tf32 scores, fp16 tiles and operands, fp32 results)
    from fa_b200 import interface as _interface
    gen = torch.Generator(device=device).manual_seed(128)
    q, k, v, dout = (torch.randn(batch, heads, tokens, 128, device=device, dtype=torch.float32, generator=gen)
                     for _ in range(4))
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    previous, _interface.FP32_ON_TENSOR_CORES = _interface.FP32_ON_TENSOR_CORES, True
    try:
        with torch.no_grad():
            us = timed(lambda: fa_b200.flash_attention(q, k, v, causal=True))
        both_us = timed(lambda: fa_b200.flash_attention(q, k, v, causal=True).backward(dout))
    finally:
        _interface.FP32_ON_TENSOR_CORES = previous
    flops = 4.0 * batch * heads * tokens * tokens * 128 / 2
    out[f"{batch}x{heads}x{tokens}x128_float32_causal_tf32_switch_on"] = {
        "fwd_us": us, "fwd_tflops": flops / us / 1e6, "fwd_bwd_us": both_us, "fwd_bwd_tflops": 3.5 * flops / both_us / 1e6}
    # one head of 512 channels over a 128 x 128 latent: the attention block of an image autoencoder, which the SDPA
    # hook serves when a whole pipeline runs under it (forward only, non-causal)
    gen = torch.Generator(device=device).manual_seed(512)
    q, k, v = (torch.randn(1, 1, 16384, 512, device=device, dtype=torch.float16, generator=gen) for _ in range(3))
    with torch.no_grad():
        us = timed(lambda: fa_b200.flash_attention(q, k, v))
    out["1x1x16384x512_float16_full"] = {"fwd_us": us, "fwd_tflops": 4.0 * 16384 * 16384 * 512 / us / 1e6}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--skip-extras", action="store_true", help="skip decode numbers and the CPU baseline")
    ap.add_argument("--decode-only", action="store_true", help="only the decode numbers (one GPU), as their own JSON line")
    ap.add_argument("--paged-only", action="store_true",
                    help="with --decode-only: only the paged entries, over one K/V set (a small case for profilers)")
    ap.add_argument("--configs", action="store_true",
                    help="only the other benchmark configurations (one GPU), as their own JSON line")
    ap.add_argument("--other-shapes", action="store_true",
                    help="only the times of other head dims and fp32 inputs (one GPU), as their own JSON line")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.decode_only:
        import fa_b200  # noqa: F401  (fails loudly without the CUDA library)
        device = torch.device("cuda", 0)
        torch.cuda.set_device(0)
        if args.paged_only:
            print(json.dumps({"decode": decode_extras(device, None, load_peaks(), iters=4, nsets=1, splitk=False)}))
        else:
            print(json.dumps({"decode": decode_extras(device, Flusher(device), load_peaks())}))
    elif args.configs:
        import fa_b200  # noqa: F401  (fails loudly without the CUDA library)
        device = torch.device("cuda", 0)
        torch.cuda.set_device(0)
        print(json.dumps({"configs": baseline_configs(device, Flusher(device), load_peaks())}))
    elif args.other_shapes:
        import fa_b200  # noqa: F401  (fails loudly without the CUDA library)
        torch.cuda.set_device(0)
        print(json.dumps({"other_shapes": other_shapes(torch.device("cuda", 0))}))
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
