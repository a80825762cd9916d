"""Benchmark of the attention-forward hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload: the long-context causal configuration that is defined for 1/2/4/8 GPUs
(fp16 Q/K/V of shape [B=8, H=64, N=32768, d=128], causal, scale 1/sqrt(128)), sharded over the
independent (batch, head) axis: rank r of N owns a contiguous slab of 512/N heads, there is no
collective on the data path (total work is fixed, so this is strong scaling). One "step" is one
forward over the rank's slab. Inputs are synthetic: i.i.d. N(0,1), seeded, generated on the
device; every slab (>= 2 GiB) is larger than L2, so no flush is needed between steps.

Printed (rank 0, one JSON line): the whole-job TFLOP/s with inputs resident in HBM (`value`),
the same through the host-buffer C-ABI call with uploads and download inside the timed region
(`e2e`), the roofline of the kernel, the CPU baseline, SM clocks during the timed region, and
the smaller single-GPU configurations for context (`per_config`, N=1 only).

`--impl reference` times the reference's own CPU attention (compiled from its sources into
oracle/_ref when they were available at build time, else the C restatement) on all host cores,
on a bounded sample of the same workload.
"""
import argparse
import ctypes
import json
import math
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

WORKLOAD = dict(name="C5 long-context causal", B=8, H=64, N=32768, d=128, causal=True, wl=-1, wr=-1)
OTHER_CONFIGS = [
    dict(name="C1", B=1, H=4, N=512, d=64, causal=False, wl=-1, wr=-1),
    dict(name="C2", B=4, H=16, N=2048, d=64, causal=True, wl=-1, wr=-1),
    dict(name="C3", B=2, H=32, N=8192, d=128, causal=True, wl=-1, wr=-1),
    dict(name="C4", B=4, H=16, N=16384, d=128, causal=True, wl=1024, wr=-1),
]
# 12 heads of the workload's own per-head shape (three head groups of 4): the case the DRAM-traffic capture runs on;
# traffic per head carries over to the full workload only while heads are scheduled in groups of the same size there
# (checked at run time: TRAFFIC_HEAD_GROUP).
TRAFFIC_CASE = dict(name="C5s", B=1, H=12, N=32768, d=128, causal=True, wl=-1, wr=-1)
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of TRAFFIC_CASE under ncu (456.3 MB + 84.8 MB for 12
# heads), per head. Algorithmic bytes per head are 33.6 MB.
TRAFFIC_BYTES_PER_HEAD = (456277504 + 84791040) / 12
TRAFFIC_HEAD_GROUP = 4  # heads per scheduling group during that capture
METRIC = "fwd attention TFLOP/s (whole job; FLOPs = 4*B*H*N^2*d, halved for causal)"
FALLBACK_TFLOPS = 1590.0  # earlier measurement on this pool, used only if MEASURED_PEAKS.json is absent


def env_int(name, default):
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            p = json.load(open(path))
            return dict(burst=float(p["bf16_tflops"]), sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                        source="measured")
        except Exception:
            pass
    return dict(burst=FALLBACK_TFLOPS, sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.out,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        rows = []
        for line in open(self.path):
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 9:
                try:
                    rows.append((float(parts[1]), float(parts[2]), float(parts[3]), parts[5], parts[6], parts[7], parts[8]))
                except ValueError:
                    pass
        os.unlink(self.path)
        if not rows:
            return None
        pmax = max(r[2] for r in rows)
        loaded = [r for r in rows if r[2] >= 0.5 * pmax] or rows
        clocks = sorted(r[0] for r in loaded)
        reasons = []
        for name, idx in (("hw_slowdown", 3), ("hw_thermal_slowdown", 4), ("sw_thermal_slowdown", 5), ("sw_power_cap", 6)):
            if any(r[idx].lower().startswith("active") for r in loaded):
                reasons.append(name)
        return dict(sm_mhz=clocks[len(clocks) // 2], sm_max_mhz=rows[0][1], power_w_max=pmax, samples=len(loaded),
                    reasons=reasons)


def shard(rank, world, total_heads):
    """Contiguous slab of the flattened (batch, head) axis owned by `rank`: [begin, end)."""
    base, rem = divmod(total_heads, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def cpu_sample(ob, cfg, cores, seconds_hint=None):
    """One bounded CPU sample of the workload: the causal prefix (first n rows and keys) of `cores`
    heads, one head per host thread. For causal attention the first n rows of a head depend on
    the first n keys only, so this is exactly the work of those rows. Returns (seconds, flops
    by the metric's causal count, description, kind)."""
    import numpy as np

    n = 1024
    d = cfg["d"]
    rng = np.random.default_rng(26)
    q, k, v = (rng.standard_normal((1, cores, n, d), dtype=np.float32).astype(np.float16) for _ in range(3))
    if ob.ref_available():
        kind = "reference"
        t0 = time.perf_counter()
        ob.reference_attention(q, k, v, causal=True, window_size=-1, nthreads=cores)
        dt = time.perf_counter() - t0
    else:
        kind = "port"
        t0 = time.perf_counter()
        ob.attention(q, k, v, causal=True, nthreads=cores)
        dt = time.perf_counter() - t0
    flops = 2.0 * cores * n * n * d
    desc = (f"first {n} query rows (causal prefix) of {cores} heads of the workload, d={d}, one head per thread, "
            f"{'unmodified reference attention_forward_cpu' if kind == 'reference' else 'C restatement of it'}; "
            f"dense-count rate {2 * flops / dt / 1e9:.3f} GFLOP/s")
    return dt, flops, desc, kind


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def run_reference(args):
    rank = env_int("RANK", 0)
    if rank != 0:
        return 0
    ob = entry.load_oracle()
    cores = host_cores()
    for _ in range(args.warmup):
        cpu_sample(ob, WORKLOAD, cores)
    total_t, total_f, desc, kind = 0.0, 0.0, "", "port"
    for _ in range(args.steps):
        dt, fl, desc, kind = cpu_sample(ob, WORKLOAD, cores)
        total_t += dt
        total_f += fl
    value = total_f / total_t / 1e12
    line = dict(impl="reference", metric=METRIC, value=value, unit="TFLOP/s", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=1e3 * total_t / args.steps, higher_is_better=True, scaling="strong",
                vs_baseline=None, dtype="f16", data="synthetic",
                config=dict(workload="B8 H64 N32768 d128 causal fp16, sharded by (batch, head); CPU arm runs a bounded sample",
                            timing="host wall clock around each sample"),
                cpu_baseline=dict(value=value, unit="TFLOP/s", cores=cores, kind=kind, sample=desc),
                e2e=dict(value=value, unit="TFLOP/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)
    print(json.dumps(line))
    return 0


def time_config(pkg, torch, cfg, heads, iters, warmup, stream, kernel=0):
    """Device-resident timing of one configuration on the current GPU (heads = this rank's slab)."""
    N, d = cfg["N"], cfg["d"]
    g = torch.Generator(device="cuda")
    g.manual_seed(26)
    q, k, v = (torch.randn((1, heads, N, d), generator=g, device="cuda", dtype=torch.float16) for _ in range(3))
    o = torch.empty_like(q)
    args = (q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), 1, heads, N, d)
    kw = dict(is_causal=cfg["causal"], window_left=cfg["wl"], window_right=cfg["wr"], stream=stream.cuda_stream,
              kernel=kernel)
    for _ in range(warmup):
        pkg.flash_forward(*args, **kw)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    stream.synchronize()
    e0.record(stream)
    for _ in range(iters):
        pkg.flash_forward(*args, **kw)
    e1.record(stream)
    e1.synchronize()
    pkg.check(stream.cuda_stream)
    ms = e0.elapsed_time(e1) / iters
    fl = pkg.flops(1, heads, N, d, cfg["causal"], cfg["wl"], cfg["wr"])
    return ms, fl, (q, k, v, o)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--heads-per-gpu", type=int, default=0, help="override the slab size (debugging only)")
    ap.add_argument("--case", default="", help="profiling aid: time only this smaller configuration (C1..C4) on one "
                    "GPU, device-resident, and print a short JSON line that is not a benchmark line")
    ap.add_argument("--kernel", type=int, default=0, help="with --case only: 0 default kernel, 2 CTA-pair kernel "
                    "(head_dim 128 cases)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    # stdout carries the JSON line and nothing else: whatever a library prints there on its own (NCCL's version
    # banner, for one) is sent to stderr by pointing descriptor 1 at it; the line is written to the saved descriptor.
    sys.stdout.flush()
    real_stdout = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    sys.stdout = real_stdout
    if args.impl == "reference":
        return run_reference(args)

    import numpy as np
    import torch
    import torch.distributed as dist

    rank, world, local = env_int("RANK", 0), env_int("WORLD_SIZE", 1), env_int("LOCAL_RANK", 0)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU: the attention forward has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = entry.load_package()
    pkg.lib()  # fails loudly if the CUDA library is missing
    stream = torch.cuda.Stream()

    if args.case:
        c = next(x for x in OTHER_CONFIGS + [TRAFFIC_CASE] if x["name"] == args.case)
        ms, fl_c, _ = time_config(pkg, torch, c, c["B"] * c["H"], args.steps, args.warmup, stream, args.kernel)
        print(json.dumps(dict(case=c["name"], kernel=args.kernel, ms=ms, tflops=fl_c / (ms * 1e-3) / 1e12, steps=args.steps,
                              note="profiling aid, not a benchmark line")))
        return 0

    cfg = WORKLOAD
    total_heads = cfg["B"] * cfg["H"]
    h0, h1 = shard(rank, world, total_heads)
    heads = args.heads_per_gpu or (h1 - h0)
    N, d = cfg["N"], cfg["d"]

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput -------------------------------------------------------
    g = torch.Generator(device="cuda")
    g.manual_seed(1000 + h0)
    q, k, v = (torch.randn((1, heads, N, d), generator=g, device="cuda", dtype=torch.float16) for _ in range(3))
    o = torch.empty_like(q)
    ptrs = (q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), 1, heads, N, d)
    kw = dict(is_causal=cfg["causal"], window_left=cfg["wl"], window_right=cfg["wr"], stream=stream.cuda_stream)
    for _ in range(args.warmup):
        pkg.flash_forward(*ptrs, **kw)
    pkg.check(stream.cuda_stream)
    sampler = ClockSampler(local) if rank == 0 else None
    barrier()
    if sampler:
        sampler.start()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    evs[0].record(stream)
    for i in range(args.steps):
        pkg.flash_forward(*ptrs, **kw)
        evs[i + 1].record(stream)
    evs[-1].synchronize()
    barrier()
    clocks = sampler.stop() if sampler else None
    pkg.check(stream.cuda_stream)
    total_ms = evs[0].elapsed_time(evs[-1])
    kernel_ms = sum(evs[i].elapsed_time(evs[i + 1]) for i in range(args.steps)) / args.steps
    t = torch.tensor([total_ms], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    flops_rank = pkg.flops(1, heads, N, d, cfg["causal"], cfg["wl"], cfg["wr"])
    fl = torch.tensor([flops_rank], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(fl, op=dist.ReduceOp.SUM)
    flops_job = float(fl.item())
    ms_per_step = total_ms / args.steps
    value = flops_job / (ms_per_step * 1e-3) / 1e12

    # ---- sanity on EVERY rank: sampled rows of the first, middle and last head of the slab against the CPU
    # oracle (outside every timed region); verdict and worst error are reduced over the ranks
    ob = entry.load_oracle()
    rows = np.unique(np.concatenate([np.arange(0, 130), np.arange(N - 64, N),
                                     np.random.default_rng(5 + rank).integers(0, N, 64)])).astype(np.int32)
    check_heads = sorted({0, heads // 2, heads - 1})
    p_max, p_mean, p_nan = 0.0, 0.0, 0
    for hh in check_heads:
        hq_, hk_, hv_, ho_ = (x[0, hh].cpu().numpy() for x in (q, k, v, o))
        want = ob.attention_rows(hq_, hk_, hv_, rows, causal=cfg["causal"], window_left=cfg["wl"], window_right=cfg["wr"])
        mx, mean, nans = ob.abs_error(ho_[rows], want)
        p_max, p_mean, p_nan = max(p_max, mx), max(p_mean, mean), p_nan + nans
    p_ok = bool(p_nan == 0 and p_max <= 2e-3 and p_mean <= 2e-4)
    pr = torch.tensor([p_max, p_mean, float(p_nan), 0.0 if p_ok else 1.0], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(pr, op=dist.ReduceOp.MAX)
    parity = dict(ranks=world, heads_per_rank=len(check_heads), rows_per_head=int(rows.size), max_abs=float(pr[0]),
                  mean_abs=float(pr[1]), nan=int(pr[2]), ok=bool(pr[3].item() == 0.0))

    # ---- end to end: host buffers through the C ABI, copies inside the timed region ----------
    chunk = min(8, heads)  # heads per upload/kernel/download stage: 8 measured 3 % faster than 32 (shorter fill and drain)
    ws_bytes = pkg.host_workspace_bytes(N, d, chunk)
    hq, hk, hv = (torch.empty((1, heads, N, d), dtype=torch.float16, pin_memory=True) for _ in range(3))
    ho = torch.empty((1, heads, N, d), dtype=torch.float16, pin_memory=True)
    hq.copy_(q); hk.copy_(k); hv.copy_(v)
    o_dev_copy = o[0, check_heads].cpu()  # whole heads of the device-resident result
    del q, k, v, o
    torch.cuda.empty_cache()
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    e2e_steps = max(2, min(args.steps, 8))

    def e2e_step():
        pkg.flash_forward_host(hq.data_ptr(), hk.data_ptr(), hv.data_ptr(), ho.data_ptr(), 1, heads, N, d,
                               ws.data_ptr(), ws_bytes, chunk, is_causal=cfg["causal"], window_left=cfg["wl"],
                               window_right=cfg["wr"])

    def timed(step, n):
        step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(n):
            step()
        torch.cuda.synchronize()
        tt = torch.tensor([time.perf_counter() - t0], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item()) / n

    e2e_s = timed(e2e_step, e2e_steps)
    same = torch.tensor([0.0 if torch.equal(ho[0, check_heads], o_dev_copy) else 1.0], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(same, op=dist.ReduceOp.MAX)
    e2e_ok = bool(same.item() == 0.0)

    # The same bytes through the same pinned buffers, chunking, two-slot workspace and stream structure, without the
    # kernel: the ceiling the host-buffer entry point can reach on this machine at this number of ranks.
    wsv = ws.view(torch.float16).view(2, 4, chunk, N, d)
    up, down = torch.cuda.Stream(), torch.cuda.Stream()
    in_ready = [torch.cuda.Event() for _ in range(2)]
    out_done = [torch.cuda.Event() for _ in range(2)]

    def copy_only_step():
        n = 0
        for c0 in range(0, heads, chunk):
            slot, nh = n & 1, min(chunk, heads - c0)
            if n >= 2:
                up.wait_event(out_done[slot])
            with torch.cuda.stream(up):
                for t_, src in enumerate((hq, hk, hv)):
                    wsv[slot, t_, :nh].copy_(src[0, c0:c0 + nh], non_blocking=True)
                in_ready[slot].record(up)
            down.wait_event(in_ready[slot])
            with torch.cuda.stream(down):
                ho[0, c0:c0 + nh].copy_(wsv[slot, 3, :nh], non_blocking=True)
                out_done[slot].record(down)
            n += 1
        up.synchronize()
        down.synchronize()

    copy_s = timed(copy_only_step, e2e_steps)
    bytes_in = 3 * heads * N * d * 2 * world
    bytes_out = heads * N * d * 2 * world
    e2e = dict(value=flops_job / e2e_s / 1e12, unit="TFLOP/s", h2d_bytes_per_step=bytes_in, d2h_bytes_per_step=bytes_out,
               steps=e2e_steps, ms_per_step=1e3 * e2e_s, matches_device_path=e2e_ok,
               compared="whole heads (first, middle, last of every rank's slab), bitwise",
               copy_only_ms=1e3 * copy_s, copy_only_gbs_per_gpu=(bytes_in + bytes_out) / world / copy_s / 1e9,
               frac_of_copy_ceiling=copy_s / e2e_s,
               api="flash_forward_host (pinned host buffers, chunked upload/kernel/download pipeline)")
    del ws, wsv, hq, hk, hv, ho
    torch.cuda.empty_cache()

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return 0

    # ---- rank 0 only: roofline, other configurations, CPU baseline ---------------------------
    pk = peaks()
    achieved = flops_rank / (kernel_ms * 1e-3) / 1e12
    # each timed step is one ~0.1 s launch inside a seconds-long loop under the power cap
    # the captured traffic per head only carries over while the launch groups its heads as the capture did
    hg = pkg.head_group(heads, N, d, cfg["causal"], cfg["wl"], cfg["wr"], torch.cuda.get_device_properties(local).multi_processor_count)
    traffic_ok = hg == TRAFFIC_HEAD_GROUP
    roofline = dict(bound="tensor", achieved=achieved, peak=pk["sustained"], unit="TFLOP/s", frac=achieved / pk["sustained"],
                    traffic=TRAFFIC_BYTES_PER_HEAD * heads if traffic_ok else None, traffic_unit="bytes per launch",
                    traffic_source=("ncu capture of 12 heads of the same per-head shape, scaled by heads per launch" if traffic_ok else
                                    f"null: this launch schedules heads in groups of {hg}, the capture used {TRAFFIC_HEAD_GROUP}"),
                    algorithmic_bytes=4.0 * heads * N * d * 2, peak_source=f"{pk['source']} bf16 GEMM, sustained figure (kernel timed inside a long loop)",
                    frac_of_burst_peak=achieved / pk["burst"], burst_peak=pk["burst"],
                    kernel="fwd_persistent_kernel<128>", launch_ms=kernel_ms, flops_per_launch=flops_rank)
    per_config = []
    cpu_baseline = None
    if world == 1:
        for c in OTHER_CONFIGS:
            bh = c["B"] * c["H"]
            ms, fl_c, _ = time_config(pkg, torch, c, bh, 20, 5, stream)
            tf = fl_c / (ms * 1e-3) / 1e12
            per_config.append(dict(name=c["name"], shape=f"B{c['B']} H{c['H']} N{c['N']} d{c['d']}", causal=c["causal"],
                                   window_left=c["wl"], ms=ms, tflops=tf, frac_of_burst_peak=tf / pk["burst"]))
            torch.cuda.empty_cache()
        ob = entry.load_oracle()
        cores = host_cores()
        dt_cpu, fl_cpu, desc, kind = cpu_sample(ob, cfg, cores)
        cpu_baseline = dict(value=fl_cpu / dt_cpu / 1e12, unit="TFLOP/s", cores=cores, kind=kind, sample=desc,
                            seconds=dt_cpu)
    line = dict(metric=METRIC, value=value, unit="TFLOP/s", n_gpus=world, steps=args.steps, warmup=args.warmup,
                ms_per_step=ms_per_step, higher_is_better=True, scaling="strong", vs_baseline=None, dtype="f16",
                data="synthetic",
                config=dict(workload="B8 H64 N32768 d128 causal fp16 (long-context config), sharded by (batch, head)",
                            heads_per_gpu=heads, global_heads=total_heads if not args.heads_per_gpu else heads * world,
                            seq_len=N, head_dim=d, parallelism=f"head-shard x{world}, no collective",
                            l2="inputs larger than L2 (>= 2 GiB per tensor per GPU), no flush",
                            timing="CUDA events on the launch stream, max over ranks"),
                roofline=roofline, cpu_baseline=cpu_baseline, e2e=e2e, clocks=clocks, gpu_launches=args.steps * world,
                parity=parity, per_config=per_config, tflops_per_gpu=value / world)
    print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
