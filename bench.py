"""Benchmark of the Delta-Matching fp8 attention hot path (forward + backward, quantizers included) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config 3] [--impl reference]

One "step" = `o = dm_attn_func(q, k, v, causal, mode); o.backward(dO)` on one batch of synthetic input (the reference's
own protocol, benchmarks/bench.py:52-55 of the reference: the whole composition, producers included).  The default
workload is BASELINE config 3 (B=4, N=4096, H=32, Hk=8, D=128, causal GQA, matched: the Llama-3-8B-like attention the
metric "causal D=128" is quoted on); --config 1..5 selects another.
Prints ONE JSON line (rank 0).  Keys:
  value        whole-job TFLOP/s over all ranks with inputs resident in HBM (algorithmic FLOPs: 7 matmuls of 2*N*N*D per
               head, halved when causal; pass-0 recomputation and softmax work are not counted).  The K steps are
               repeated until at least two seconds of GPU time have been timed, so `value` is a sustained figure with the
               clocks sampled under it; `burst` keeps the first K steps alone and `eager_ms_per_step` the same step
               launched from Python without the CUDA graph
  e2e          the same metric through the public API with HOST pinned buffers: H2D of q, k, v, dO and D2H of O, dQ, dK,
               dV inside the timed region
  roofline     the dominant kernel's algorithmic TFLOP/s (CUDA events around that kernel, live) against the measured dense
               FP8 GEMM peak of this GPU (torch._scaled_mm, measured in this run) -- the bf16 peak of MEASURED_PEAKS.json and
               the nominal 4500 TFLOP/s are reported beside it
  cpu_baseline the CPU oracle (a PyTorch restatement of the reference numerics) timed on the host cores on a bounded
               sample of the same workload
With --impl reference the CPU oracle itself is the timed arm (the reference's CUDA kernels are Hopper-only and cannot run
here); under torchrun only rank 0 runs it.  Multi-GPU: one process per GPU; by default the configuration's (batch x KV
group) units are partitioned across the ranks with no data-path collective ("scaling": "strong"; --scaling weak gives every
rank a whole configuration of its own instead, --scaling cp splits the sequence round an NCCL ring), time = max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {  # BASELINE.json configs: (B, N, H, Hk, D, causal, mode)
    1: (1, 256, 2, 2, 128, True, "matched"),
    2: (2, 2048, 16, 16, 128, True, "matched"),
    3: (4, 4096, 32, 8, 128, True, "matched"),
    4: (2, 4096, 16, 4, 256, False, "stale"),
    5: (1, 65536, 32, 8, 128, True, "matched"),
}
NOMINAL_FP8_TFLOPS = 4500.0


def ncu_traffic_bytes(config, kernel):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of `kernel` at BASELINE config `config`, read from the table in
    profiles/dram_traffic.md (filled from the committed ncu captures; a bench run does not re-measure it).  None when the
    table has no row for the pair."""
    try:
        for line in open(os.path.join(ROOT, "profiles", "dram_traffic.md")):
            cells = [c.strip() for c in line.strip().strip("|").split("|")]
            if len(cells) >= 4 and cells[0] == str(config) and cells[1] == kernel:
                return float(cells[2]) + float(cells[3])
    except (OSError, ValueError):
        pass
    return None


def algorithmic_flops(B, N, H, D, causal):
    return (7 if causal else 14) * B * H * N * N * D


def make_host_inputs(cfg, seed):
    B, N, H, Hk, D, causal, mode = cfg
    g = torch.Generator("cpu").manual_seed(seed)
    mk = lambda h: torch.randn(B, N, h, D, generator=g).to(torch.bfloat16).pin_memory()
    q, k, v, dO = mk(H), mk(Hk), mk(Hk), mk(H)
    return q, k, v, dO


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz, self._stop = [], set(), None, threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None
        self.t = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                 "hw_power_brake": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                r = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h) if hasattr(self.nv, "nvmlDeviceGetCurrentClocksEventReasons") \
                    else self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for n, bit in names.items():
                    if r & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(0.02)

    def __enter__(self):
        if self.nv:
            self.t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self.nv:
            self.t.join(timeout=1)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"]}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def measure_fp8_peak(dev):
    """Dense e4m3 x e4m3 GEMM 8192^3 through torch._scaled_mm: best of 10 (the denominator of the roofline fraction)."""
    try:
        n = 8192
        a = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn).t()
        one = torch.ones((), device=dev)
        for _ in range(3):
            torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        best = 1e9
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return 2 * n ** 3 / (best * 1e-3) / 1e12
    except Exception:
        return None


def cpu_oracle_time(cfg, budget_s=25.0, total_s=0.0):
    """The CPU oracle on a bounded sample of the workload: whole heads of batch 0 (heads and batches are independent, so the
    full-workload time is sample time x factor).  With total_s > 0 the sample is repeated until about that many seconds of
    CPU work have been timed.  Returns (TFLOP/s of the sample, cores, description, seconds)."""
    from oracle import dm_oracle as O
    B, N, H, Hk, D, causal, mode = cfg
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    rep = H // Hk
    # per-KV-group cost estimate from a small probe, then pick how many KV groups fit the budget
    groups = 1
    n_s = N if N <= 8192 else 8192
    q, k, v, dO = O.make_inputs(1, n_s, rep * groups, groups, D, 77)
    t0 = time.perf_counter()
    O.attention_fwd_bwd(q, k, v, dO, causal, mode)
    dt = time.perf_counter() - t0
    fl = algorithmic_flops(1, n_s, rep * groups, D, causal)
    if dt < budget_s / 4 and Hk > 1 and n_s == N:
        groups = int(min(Hk, max(1, (budget_s / 2) // max(dt, 1e-3))))
        q, k, v, dO = O.make_inputs(1, n_s, rep * groups, groups, D, 78)
        t0 = time.perf_counter()
        O.attention_fwd_bwd(q, k, v, dO, causal, mode)
        dt = time.perf_counter() - t0
        fl = algorithmic_flops(1, n_s, rep * groups, D, causal)
    factor = algorithmic_flops(B, N, H, D, causal) / fl
    runs = 1
    if total_s > dt:
        more = int(min(40, max(0, round(total_s / max(dt, 1e-3)) - 1)))
        t0 = time.perf_counter()
        for _ in range(more):
            O.attention_fwd_bwd(q, k, v, dO, causal, mode)
        dt_more = time.perf_counter() - t0
        dt, fl, runs = dt + dt_more, fl * (1 + more), 1 + more
    desc = (f"oracle fwd+bwd on batch 0, {groups} of {B * Hk} KV groups ({rep * groups} query heads), seqlen {n_s} of {N}; "
            f"full workload = sample x {factor:.1f} by FLOPs" + (f"; sample run {runs} times" if runs > 1 else ""))
    return fl / dt / 1e12, cores, desc, dt


def run_reference_arm(args, cfg, rank, world):
    if rank != 0:
        return
    B, N, H, Hk, D, causal, mode = cfg
    vals, desc, cores = [], "", 1
    for i in range(args.warmup + args.steps):
        tf, cores, desc, dt = cpu_oracle_time(cfg, budget_s=12.0)
        if i >= args.warmup:
            vals.append((tf, dt))
    tf = statistics.mean(v[0] for v in vals)
    ms = statistics.mean(v[1] for v in vals) * 1e3
    line = {"impl": "reference", "metric": "fp8_attn_fwd_bwd_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak" if world == 1 or args.scaling == "weak" else "strong",      # the key of the GPU arm's line
            "vs_baseline": None, "dtype": "e4m3", "data": "synthetic",
            "config": workload_config(args.config, cfg),
            "parallelism": "host (CPU oracle: PyTorch restatement of the reference numerics; the reference's own kernels are "
                           "sm_90a-only and cannot run on this machine)",
            "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc},
            "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def workload_config(idx, cfg):
    """The workload's identity only (the same dict in both arms); how it is spread over ranks and how L2 is treated are
    separate keys of the line."""
    B, N, H, Hk, D, causal, mode = cfg
    return {"workload": f"BASELINE config {idx}: B={B} N={N} H={H} Hk={Hk} D={D} {'causal' if causal else 'full'} {mode}, "
                        f"fwd+bwd incl. quantizers", "B": B, "N": N, "H": H, "Hk": Hk, "D": D, "causal": causal, "mode": mode}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--scaling", default="strong", choices=["weak", "strong", "cp"],
                    help="strong (default): the config's (batch x KV-head) groups are partitioned across the ranks "
                         "(delta_matching_b200.shard), e.g. config 5 sharded over heads; weak: every rank runs a whole config "
                         "(its own seed); cp: the "
                         "sequence is split across the ranks (delta_matching_b200.cp: zig-zag chunks, K / V codes round an NCCL "
                         "ring, dK / dV partials to the key owners), head_dim 128, reported as strong scaling")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="run the timed steps eagerly instead of replaying a CUDA graph of the step")
    ap.add_argument("--min-seconds", type=float, default=2.0, help="repeat the K timed steps until this much GPU time has been timed")
    ap.add_argument("--profile", action="store_true", help="only warm-up and timed steps (for ncu captures): no e2e, no per-kernel "
                    "timing, no peak measurement, no CPU baseline")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup
    cfg = CONFIGS[args.config]
    B, N, H, Hk, D, causal, mode = cfg
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, cfg, rank, world)
        return

    import torch.distributed as dist
    import delta_matching_b200 as dm
    from delta_matching_b200 import _lib
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # NCCL announces its version on stdout at the first communicator unless told otherwise; stdout is for the one JSON line
        # (the WARN level prints it too)
        if os.environ.get("NCCL_DEBUG", "").upper() not in ("INFO", "TRACE"):
            os.environ["NCCL_DEBUG"] = "NONE"
        dist.init_process_group("nccl", device_id=dev)

    # count the library's kernel launches per call (one entry point can launch more than one kernel)
    launches = {"n": 0}
    per_call = {"dm_kmean": 2, "dm_quant": 1, "dm_quant_do": 1, "dm_fwd_fp8": 1, "dm_delta_fp8": 1, "dm_bwd_fp8_pass1": 1,
                "dm_bwd_fp8_pass2": 1, "dm_gqa_fold": 1, "dm_attn_forward": 3 if (N // 64 <= 128 and D == 128) else 4, "dm_quant_qv_kpartials": 1, "dm_kmean_partials": 1, "dm_kmean_fold": 1,
                "dm_fold_f32": 1, "dm_fold_to_owners": 1, "dm_fwd_fp8_cp": 1, "dm_delta_fp8_cp": 1, "dm_bwd_fp8_pass1_cp": 1, "dm_bwd_fp8_pass2_cp": 1,
                "dm_attn_backward": 3 + (1 if mode == "matched" else 0) + (1 if Hk < H else 0)}
    orig_call = _lib._call

    def counting_call(name, *a):
        launches["n"] += per_call.get(name, 0)
        return orig_call(name, *a)
    _lib._call = counting_call

    scaling = args.scaling if world > 1 else "weak"     # one GPU: the whole config either way
    if scaling == "strong":
        from delta_matching_b200.shard import kv_group_range
        first, count = kv_group_range(B, Hk, rank, world)
        rep = H // Hk
        if count >= Hk:
            B = count // Hk
        else:
            B, Hk, H = 1, count, count * rep
        cfg = (B, N, H, Hk, D, causal, mode)          # this rank's shard; generated directly at shard size
    cp_mode = scaling == "cp"
    cp_map = None
    if cp_mode:
        from delta_matching_b200 import cp as dmcp
        cp_map = dmcp.zigzag_map(rank, world, N)      # also checks that the sequence splits
        cfg = (B, N // world, H, Hk, D, causal, mode)  # this rank's two zig-zag chunks, generated directly at that size
        attn = lambda a, b, c: dmcp.dm_attn_func_cp(a, b, c, causal=causal, mode=mode)
    else:
        attn = lambda a, b, c: dm.dm_attn_func(a, b, c, causal=causal, mode=mode)
    hq, hk, hv, hdo = make_host_inputs(cfg, 1000 + args.config + 17 * rank)
    q, k, v, dO = (t.to(dev) for t in (hq, hk, hv, hdo))
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    flush = torch.empty(256 * 2 ** 20, dtype=torch.uint8, device=dev)
    flops = algorithmic_flops(B, N, H, D, causal) / (world if cp_mode else 1)      # per rank

    def step():
        q.grad = k.grad = v.grad = None
        o = attn(q, k, v)
        o.backward(dO)
        return o

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed_steps(fn, n):
        """n steps, each bracketed by its own pair of events (the L2 flush between steps stays outside them); the host does
        not wait for a step before it enqueues the next, so the events measure the device, not the launch path."""
        evs = []
        for _ in range(n):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            evs.append((e0, e1))
        sync_all()
        return sum(a.elapsed_time(b) for a, b in evs)

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for _ in range(args.warmup):
        step()
    sync_all()
    # the same step launched from Python (no graph), timed before the capture: what a caller of the API sees
    eager_ms = None if args.profile else max_over_ranks(timed_steps(step, args.steps)) / args.steps
    # The step (forward + backward through autograd) is captured once into a CUDA graph and replayed: at the small
    # configurations the host's launch path (~0.3 ms of Python per step) is as long as the kernels themselves.  Kernels
    # are counted during the capture.  --no-graph, a sequence split (NCCL inside the step) or a failed capture fall back to
    # eager steps.
    graph, launches_per_step = None, None
    if not args.no_graph and not cp_mode and not args.profile:
        try:
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            launches["n"] = 0
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            launches_per_step = launches["n"]
            for _ in range(2):
                graph.replay()
        except Exception as e:                      # noqa: BLE001
            print(f"bench: CUDA graph capture of the step failed ({type(e).__name__}: {e}); running eager", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()
    run_step = graph.replay if graph is not None else step
    sync_all()
    launches["n"] = 0

    # The timed region: the K steps, repeated (same K steps again) until at least --min-seconds of GPU time have been timed, so
    # that the number is a sustained one and the clock sampler sees the GPU under load.  The first K steps alone are kept as
    # the burst figure.  Every rank runs the same number of repeats (agreed from rank 0's burst time).
    with ClockSampler(local) as clk:
        burst_ms = max_over_ranks(timed_steps(run_step, args.steps))
        repeats = 1 if args.profile else max(1, min(2000, int(-(-args.min_seconds * 1e3 // max(burst_ms, 1e-3)))))
        if world > 1:
            t = torch.tensor([repeats], device=dev, dtype=torch.int64)
            dist.broadcast(t, 0)
            repeats = int(t.item())
        total_ms = burst_ms
        for _ in range(repeats - 1):
            total_ms += max_over_ranks(timed_steps(run_step, args.steps))
    n_timed = args.steps * repeats
    n_launch = launches["n"] if graph is None else launches_per_step * n_timed
    ms_step = total_ms / n_timed
    value = world * flops / (ms_step * 1e-3) / 1e12       # every rank does `flops` (its whole config, or its equal shard)
    burst = {"value": world * flops / (burst_ms / args.steps * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": burst_ms / args.steps,
             "steps": args.steps}
    status = _lib.device_status(local)
    if status != 0:
        raise SystemExit(f"bench: a kernel reported a bounded-wait timeout (device status {status}); the timed numbers are void")

    if args.profile:
        if rank == 0:
            print(json.dumps({"metric": "fp8_attn_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "ms_per_step": ms_step,
                              "profile_only": True, "gpu_launches": n_launch}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- end to end with host buffers: every step copies its q, k, v, dO from pinned host memory and its O, dQ, dK, dV back,
    # all inside the timed region.  The copies dominate (PCIe), so the steps run as a three-stage pipeline on three streams
    # (copy in, compute, copy out) over two sets of buffers: step i + 1's inputs travel while step i computes and step
    # i - 1's results leave, which uses both directions of the link at once.
    hosts = (hq, hk, hv, hdo)
    nbuf = 2
    s_in, s_cmp, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    dev_in = [[torch.empty(t.shape, dtype=t.dtype, device=dev) for t in hosts] for _ in range(nbuf)]
    outs = [[torch.empty_like(t).pin_memory() for t in (hq, hq, hk, hv)] for _ in range(nbuf)]

    def e2e_pipeline(n):
        ev_cmp, ev_out = [None] * nbuf, [None] * nbuf
        for i in range(n):
            b = i % nbuf
            with torch.cuda.stream(s_in):
                if ev_cmp[b] is not None:
                    s_in.wait_event(ev_cmp[b])            # step i - nbuf has finished with this set of input buffers
                for d, h in zip(dev_in[b], hosts):
                    d.copy_(h, non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(ev_in)
                flush.fill_(1)
                qq, kk, vv = (t.detach().requires_grad_(True) for t in dev_in[b][:3])
                o = attn(qq, kk, vv)
                o.backward(dev_in[b][3])
                res = (o.detach(), qq.grad, kk.grad, vv.grad)
                ev_cmp[b] = torch.cuda.Event()
                ev_cmp[b].record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_cmp[b])
                for dst, src in zip(outs[b], res):
                    dst.copy_(src, non_blocking=True)
                    src.record_stream(s_out)
                ev_out[b] = torch.cuda.Event()
                ev_out[b].record(s_out)

    sync_all()
    e2e_pipeline(3)
    sync_all()
    n_e2e = max(4, args.steps // 2)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(s_in)
    e2e_pipeline(n_e2e)
    for st_ in (s_in, s_cmp):
        s_out.wait_stream(st_)
    e1.record(s_out)
    sync_all()
    e2e_ms = e0.elapsed_time(e1) / n_e2e
    e2e_ms = max_over_ranks(e2e_ms)
    nbytes = lambda t: t.numel() * t.element_size()
    e2e = {"value": world * flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": sum(nbytes(t) for t in hosts), "d2h_bytes_per_step": sum(nbytes(t) for t in outs[0]),
           "pipeline": "3 streams (copy in / compute / copy out), 2 buffer sets, every step's copies inside the timed region"}

    torch.cuda.empty_cache()      # blocks cached for the pipeline's streams go back before the default stream allocates
    # ---- per-kernel timing (CUDA events around each library call, same inputs, L2 flushed) and the roofline
    roof, kernels = None, {}
    if rank == 0:
        with torch.no_grad():
            qf, kf, vf = q.detach(), k.detach(), v.detach()
            reps = max(5, min(args.steps, 10))
            acc = {}

            def timed(name, fn):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                r = fn()
                e1.record()
                acc.setdefault(name, []).append((e0, e1))
                return r
            for _ in range(reps + 1):
                flush.fill_(1)
                # keep the GPU busy (~2 ms) while the host enqueues the whole chain, so that the events bracket kernel time
                # only and not the gaps in which the GPU would wait for the host
                torch.cuda._sleep(4_000_000)
                Q8, Q8s = timed("quant_q", lambda: _lib.quant(0, qf))
                km = timed("kmean", lambda: _lib.kmean(kf))
                K8, K8s = timed("quant_k", lambda: _lib.quant(1, kf, km))
                V8, V8s = timed("quant_v", lambda: _lib.quant(2, vf))
                if cp_mode:        # kernel timing only: the other ranks' keys are stood in for by copies of this rank's
                    K8, K8s, V8, V8s = (t.repeat(1, world, 1) if t.dim() == 3 else t.repeat(1, world) for t in (K8, K8s, V8, V8s))
                O_, lse = timed("fwd", lambda: _lib.fwd_fp8(Q8, K8, V8, Q8s, K8s, V8s, B, H, Hk, causal, cp=cp_map))
                dO8, dO8s, dl = timed("quant_do", lambda: _lib.quant_do(dO, None if mode == "matched" else O_))
                if mode == "matched":
                    dl = timed("pass0_delta", lambda: _lib.delta_fp8(Q8, K8, V8, dO8, Q8s, K8s, V8s, dO8s, lse, B, H, Hk, causal,
                                                                     cp=cp_map))
                hp = dm.split._bwd_heads_per_call(B, H, Hk, H // Hk, N)
                if hp >= H or cp_mode:
                    dk_, dv_, ws = timed("pass1", lambda: _lib.bwd_pass1(Q8, K8, V8, dO8, Q8s, K8s, V8s, dO8s, lse, dl, B, H, Hk, causal,
                                                                         cp=cp_map, out_fp32=cp_mode))
                    timed("pass2", lambda: _lib.bwd_pass2(ws, K8, B, H, Hk, N, D, causal, cp=cp_map))
                    del dk_, dv_, ws
            torch.cuda.synchronize()
            # the first repetition also pays for the allocator's first blocks on this stream: leave it out
            kernels = {n: statistics.median(a.elapsed_time(b) for a, b in ev[1:]) for n, ev in acc.items()}
        u = flops / 7.0                      # one matmul's FLOPs (causal halving already inside `flops`)
        alg = {"fwd": 2 * u, "pass1": 4 * u, "pass2": 1 * u}
        fp8_peak = measure_fp8_peak(dev)
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        cand = {n: kernels[n] for n in alg if n in kernels}
        if cand:
            top = max(cand, key=cand.get)
            achieved = alg[top] / (kernels[top] * 1e-3) / 1e12
            peak = fp8_peak or NOMINAL_FP8_TFLOPS
            roof = {"bound": "tensor", "kernel": top, "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                    "peak_source": "torch._scaled_mm e4m3 8192^3 best of 10, measured in this run" if fp8_peak else "nominal dense FP8",
                    "frac_of_nominal_fp8_4500": achieved / NOMINAL_FP8_TFLOPS,
                    "frac_of_measured_bf16": achieved / peaks["bf16_tflops"] if "bf16_tflops" in peaks else None,
                    "traffic": ncu_traffic_bytes(args.config, top), "kernel_ms": kernels,
                    "per_kernel_tflops": {n: alg[n] / (kernels[n] * 1e-3) / 1e12 for n in cand}}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        tf, cores, desc, dt = cpu_oracle_time(cfg, total_s=12.0)      # about 12 s of CPU work in all
        cpu = {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc, "sample_seconds": dt}

    if rank == 0:
        line = {"metric": "fp8_attn_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
                "scaling": "strong" if cp_mode else scaling, "vs_baseline": None,
                "timed_steps": n_timed, "timed_seconds": total_ms * 1e-3, "burst": burst, "eager_ms_per_step": eager_ms,
                "dtype": "e4m3", "data": "synthetic",
                "config": workload_config(args.config, CONFIGS[args.config]),
                "parallelism": (f"cp{world}: sequence split in zig-zag chunks, K / V codes round an NCCL ring, dK / dV partials to the "
                                f"key owners" if cp_mode else f"dp{world} over (batch x KV group), no collective" +
                                ("; the config's KV groups partitioned across the ranks" if scaling == "strong" else
                                 "; every rank runs a whole config of its own")),
                "l2": "flushed between timed iterations (256 MiB write)",
                "tflops_per_gpu": value / world, "frac_of_nominal_fp8_per_gpu": value / world / NOMINAL_FP8_TFLOPS,
                "clocks": clk.summary(), "e2e": e2e, "gpu_launches": n_launch,
                "step_launch": "CUDA graph replay of one captured step" if graph is not None else "eager", "roofline": roof, "cpu_baseline": cpu}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
