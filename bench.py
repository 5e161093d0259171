"""Benchmark of sliding-window causal 2-simplicial attention, forward + backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload C3|C2|C5]
                    [--kernel auto|simt|tcgen05] [--impl ours|reference]

A step is one forward + backward pass of the operator over one batch of
seeded synthetic tensors.  The default workload is the forward+backward
configuration b4 h8 n4096 d64 w1=512 w2=32 bf16 ("C3"); with N GPUs every rank
runs that batch on its own GPU (batch x head sharding, no collective on the
data path), so the global batch is 4*N and scaling is weak.

Prints ONE JSON line:
  value     whole-job TFLOP/s with the inputs resident in HBM, counting only
            algorithmic work: 14*d flop per unmasked (i, j, k) triple
            (4*d forward, 10*d backward); masked cells, the elementwise
            products, the softmax and any recomputation count zero;
  e2e       the same metric through the package's host-buffer call
            (HostPipeline.run) with pinned HOST tensors: host->device copy of
            q, k, k', v, v', dO and device->host copy of out and the five
            gradients inside the timed region, overlapped with the kernels by
            batch chunks (sequence sharding: the autograd API, serial copies);
  roofline  the dominant phase (the backward entry point) against the measured
            dense bf16 tensor peak of this pool's B200s;
  cpu_baseline  the CPU oracle timed on this machine's host cores on a bounded
            sample of the same workload (rank 0, N=1 only).

``--impl reference`` times the reference's CPU path for this operator - the
oracle port of its naive PyTorch implementation, since the reference itself is
a Python package that is not present on the GPU machine - with all host threads.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: b (per GPU), hq, hk, n, d, w1, w2
    "C2": dict(b=2, hq=8, hk=8, n=1024, d=64, w1=512, w2=32),
    "C3": dict(b=4, hq=8, hk=8, n=4096, d=64, w1=512, w2=32),
    "C5": dict(b=8, hq=16, hk=16, n=16384, d=128, w1=512, w2=32),
}
# CPU sample: two batch elements, eight heads, up to 4096 rows of the same head dim and windows (~10 s on 16 cores)
CPU_SAMPLE = dict(b=2, hq=8, hk=8, n=4096)


def valid_pairs(n, w1, w2):
    return sum(min(i + 1, w1) * min(i + 1, w2) for i in range(n))


def work_flops(cfg):
    p = valid_pairs(cfg["n"], cfg["w1"], cfg["w2"]) * cfg["b"] * cfg["hq"]
    return {"fwd": 4 * cfg["d"] * p, "bwd": 10 * cfg["d"] * p, "fwd_bwd": 14 * cfg["d"] * p}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            m = json.load(f)
        return {"tflops": float(m.get("bf16_tflops_sustained") or m["bf16_tflops"]), "hbm_gbs": float(m["hbm_gbs"]),
                "source": "measured (MEASURED_PEAKS.json, sustained cuBLAS bf16)"}
    return {"tflops": 1400.0, "hbm_gbs": 6650.0, "source": "fallback (earlier measurement on this pool, sustained)"}


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML read-only queries from a
    thread every few milliseconds (the timed region of the default run lasts ~55 ms, less than nvidia-smi
    needs to start), nvidia-smi as the fallback."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc, self.nvml, self.stop_flag = index, [], None, None, False

    def _nvml_loop(self):
        n, h = self.nvml
        masks = (n.nvmlClocksEventReasonHwSlowdown if hasattr(n, "nvmlClocksEventReasonHwSlowdown") else 0x8,
                 n.nvmlClocksEventReasonHwThermalSlowdown if hasattr(n, "nvmlClocksEventReasonHwThermalSlowdown") else 0x40,
                 n.nvmlClocksEventReasonSwThermalSlowdown if hasattr(n, "nvmlClocksEventReasonSwThermalSlowdown") else 0x20,
                 n.nvmlClocksEventReasonSwPowerCap if hasattr(n, "nvmlClocksEventReasonSwPowerCap") else 0x4)
        query = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
        mx = n.nvmlDeviceGetMaxClockInfo(h, n.NVML_CLOCK_SM)
        while not self.stop_flag:
            try:
                sm = n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM)
                bits = query(h)
                self.rows.append([str(sm), str(mx)] + ["Active" if bits & m else "Not Active" for m in masks])
            except Exception:
                break
            time.sleep(0.004)

    def start(self):
        try:
            import pynvml as n
            n.nvmlInit()
            # the process may see a subset of the machine's GPUs: map the CUDA index through its UUID
            uuid = str(torch.cuda.get_device_properties(self.index).uuid)
            handle = None
            for k in range(n.nvmlDeviceGetCount()):
                h = n.nvmlDeviceGetHandleByIndex(k)
                u = n.nvmlDeviceGetUUID(h)
                u = u.decode() if isinstance(u, bytes) else u
                if uuid in u:
                    handle = h
            if handle is None:
                handle = n.nvmlDeviceGetHandleByIndex(self.index)
            self.nvml = (n, handle)
            self.thread = threading.Thread(target=self._nvml_loop, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.nvml:
            self.stop_flag = True
            self.thread.join(timeout=2)
        elif self.proc:
            self.proc.terminate()
            self.thread.join(timeout=2)
        else:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(self.NAMES, r[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "source": "nvml" if self.nvml else "nvidia-smi", "reasons": sorted(reasons)}


def make_inputs(cfg, seed, dtype, device, pin=False):
    gen = torch.Generator().manual_seed(seed)
    b, n, hq, hk, d = cfg["b"], cfg["n"], cfg["hq"], cfg["hk"], cfg["d"]
    shapes = [(b, n, hq, d)] + [(b, n, hk, d)] * 4 + [(b, n, hq, d)]
    host = [torch.randn(s, generator=gen, dtype=torch.float32).to(dtype) for s in shapes]
    if pin:
        host = [t.pin_memory() for t in host]
    return host, [t.to(device) for t in host]


def reduce_max(x, world):
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def cpu_oracle_sample(cfg, steps=1, warmup=0):
    """Oracle forward + backward on the bounded CPU sample; returns (TFLOP/s, seconds per pass, description)."""
    from oracle import oracle as O
    s = dict(cfg)
    s.update(CPU_SAMPLE)
    s["n"] = min(s["n"], cfg["n"])
    ins = O.make_inputs(s["b"], s["n"], s["hq"], s["hk"], s["d"], seed=1)
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        O.two_simplicial_fwd_bwd(*ins, s["w1"], s["w2"], chunk=32)
        if it >= warmup:
            times.append(time.perf_counter() - t0)
    sec = statistics.median(times)
    fl = work_flops(s)["fwd_bwd"]
    desc = (f"oracle fwd+bwd (fp32, torch CPU) on b{s['b']} h{s['hq']} n{s['n']} d{s['d']} w1={s['w1']} w2={s['w2']}: "
            f"{fl / 1e9:.1f} GFLOP in {sec:.2f} s")
    return fl / sec / 1e12, sec, desc, s


def run_reference(args, cfg, name):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = torch.get_num_threads()
    tf, sec, desc, s = cpu_oracle_sample(cfg, steps=max(1, args.steps), warmup=min(args.warmup, 1))
    line = {
        "impl": "reference", "metric": "2-simplicial attn fwd+bwd TFLOP/s", "value": tf, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, **cfg, "sample": f"b{s['b']} h{s['hq']} n{s['n']}"},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": desc,
                         "host_cpus": os.cpu_count()},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "tokens_per_s": s["b"] * s["n"] / sec, "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


C4 = dict(dim=512, depth=8, heads=8, key_value_heads=4, dim_head=64, every=2, vocab=256, batch=16, seq_len=1024,
          w1=512, w2=32)


def run_c4(args):
    """Full training step of the 8-layer decoder (every 2nd layer simplicial, byte vocabulary,
    batch 16 x 1024 tokens per GPU, bf16 autocast, Adam): tokens/s.  N > 1: data parallel (DDP)."""
    from simplicial_attention_b200.transformer import TwoSimplicialLM, training_step
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(0)
    c = C4
    model = TwoSimplicialLM(num_tokens=c["vocab"], dim=c["dim"], depth=c["depth"], max_seq_len=c["seq_len"],
                            dim_head=c["dim_head"], heads=c["heads"], two_simplicial_attn_every=c["every"],
                            transformer_kwargs=dict(key_value_heads=c["key_value_heads"],
                                                    two_simplicial_attn_kwargs=dict(w1=c["w1"], w2=c["w2"], qk_rmsnorm=True))).to(dev)
    net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local]) if world > 1 else model
    opt = torch.optim.Adam(net.parameters(), lr=1e-4)
    gen = torch.Generator().manual_seed(100 + rank)
    host = torch.randint(0, c["vocab"], (c["batch"], c["seq_len"] + 1), generator=gen, dtype=torch.uint8).pin_memory()
    resident = host.to(dev).long()

    def step(tokens):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            return training_step(net, opt, tokens)

    for _ in range(max(3, args.warmup)):
        step(resident)
    sampler = ClockSampler(local)
    barrier(world)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step(resident)
    e1.record()
    barrier(world)
    ms = reduce_max(e0.elapsed_time(e1), world) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    # end to end: token ids from pinned host memory every step, loss read back every step
    barrier(world)
    e0.record()
    for _ in range(args.steps):
        loss = step(host.to(dev, non_blocking=True).long())
        loss_host = loss.item()
    e1.record()
    barrier(world)
    e2e_ms = reduce_max(e0.elapsed_time(e1), world) / args.steps
    if rank == 0:
        tokens = c["batch"] * c["seq_len"] * world
        simplicial_layers = c["depth"] // c["every"]
        print(json.dumps({
            "metric": "training tokens/s (8-layer decoder, every 2nd layer 2-simplicial)", "value": tokens / (ms * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "C4", **c, "global_batch": c["batch"] * world, "parallelism": f"dp{world}",
                       "optimizer": "Adam lr 1e-4, grad clip 0.5"},
            "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": host.numel(),
                    "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms, "last_loss": loss_host},
            "gpu_launches": args.steps * simplicial_layers * 5, "clocks": clocks}), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="C3", choices=sorted(WORKLOADS) + ["C4"])
    ap.add_argument("--kernel", default="auto", choices=("auto", "simt", "tcgen05"))
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--sharding", default="batch", choices=("batch", "seq"),
                    help="batch: every rank runs its own batch (no collective); seq: the ranks hold consecutive blocks "
                         "of one sequence of length n * N and exchange the key/value halo over NCCL")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (for profiler captures)")
    args = ap.parse_args()
    if args.workload == "C4":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the decoder training step has no CPU reference arm; "
                              "the operator's arm is --workload C3"}), flush=True)
            return
        run_c4(args)
        return
    cfg = dict(WORKLOADS[args.workload])

    if args.impl == "reference":
        run_reference(args, cfg, args.workload)
        return

    import simplicial_attention_b200 as sa
    from simplicial_attention_b200 import _lib

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    dtype = torch.bfloat16
    host, devt = make_inputs(cfg, seed=1234 + rank, dtype=dtype, device=dev, pin=True)
    q, k1, k2, v1, v2, do = devt
    w1, w2 = cfg["w1"], cfg["w2"]
    fl = work_flops(cfg)
    seq = args.sharding == "seq" and world > 1
    if seq:
        # one sequence of length n * world: per-rank share of its unmasked triples
        whole = dict(cfg, n=cfg["n"] * world)
        fl = {k: v / world for k, v in work_flops(whole).items()}
        from simplicial_attention_b200 import shard
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)   # > 126 MB L2

    def seq_forward(leaves):
        return shard.sequence_parallel_attn(leaves[0], (leaves[1], leaves[2]), (leaves[3], leaves[4]),
                                            w1=w1, w2=w2, kernel=args.kernel)

    def step_resident():
        if seq:
            leaves = [t.detach().requires_grad_() for t in (q, k1, k2, v1, v2)]
            out = seq_forward(leaves)
            out.backward(do)
            return out, [t.grad for t in leaves]
        out, lse = sa.sa2_forward(q, k1, k2, v1, v2, w1, w2, kernel=args.kernel)
        return out, sa.sa2_backward(q, k1, k2, v1, v2, out, lse, do, w1, w2, kernel=args.kernel)

    def timed_resident(steps):
        """Per-step CUDA-event timing on the current stream, L2 flushed between steps."""
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
        for s in range(steps):
            flush.zero_()
            ev[s][0].record()
            if seq:
                leaves = [t.detach().requires_grad_() for t in (q, k1, k2, v1, v2)]
                out = seq_forward(leaves)          # includes the halo exchange
                ev[s][1].record()
                out.backward(do)                   # includes the exchange of the halo gradients
            else:
                out, lse = sa.sa2_forward(q, k1, k2, v1, v2, w1, w2, kernel=args.kernel)
                ev[s][1].record()
                sa.sa2_backward(q, k1, k2, v1, v2, out, lse, do, w1, w2, kernel=args.kernel)
            ev[s][2].record()
        torch.cuda.synchronize()
        fwd = [e[0].elapsed_time(e[1]) for e in ev]
        bwd = [e[1].elapsed_time(e[2]) for e in ev]
        return fwd, bwd

    dq_h = [torch.empty_like(t) for t in host[:5]]
    out_h = torch.empty_like(host[0])
    dq_h = [t.pin_memory() for t in dq_h]
    out_h = out_h.pin_memory()

    pipe = None
    if not seq:
        from simplicial_attention_b200.host import HostPipeline
        pipe = HostPipeline(dev, w1=w1, w2=w2, chunk=max(1, cfg["b"] // 2), kernel=args.kernel)

    def step_e2e():
        if pipe is not None:
            # batch chunks on three streams: copy-in, compute and copy-out overlap, also across steps
            pipe.run(host, [out_h] + dq_h)
            return
        ins = [t.to(dev, non_blocking=True) for t in host]
        leaves = [t.requires_grad_() for t in ins[:5]]
        out = seq_forward(leaves) if seq else sa.sliding_two_simplicial_attn(
            leaves[0], (leaves[1], leaves[2]), (leaves[3], leaves[4]), w1=w1, w2=w2, causal=True, kernel=args.kernel)
        out.backward(ins[5])
        out_h.copy_(out.detach(), non_blocking=True)
        for h_, l_ in zip(dq_h, leaves):
            h_.copy_(l_.grad, non_blocking=True)

    h2d = sum(t.numel() * t.element_size() for t in host)
    d2h = sum(t.numel() * t.element_size() for t in dq_h + [out_h])

    # ---- warm-up
    for _ in range(max(3, args.warmup)):
        step_resident()
    torch.cuda.synchronize()

    # ---- timed, inputs resident in HBM
    sampler = ClockSampler(local)
    barrier(world)
    if rank == 0:
        sampler.start()
    fwd_ms, bwd_ms = timed_resident(args.steps)
    barrier(world)
    total_ms = reduce_max(sum(fwd_ms) + sum(bwd_ms), world)
    clocks = sampler.stop() if rank == 0 else None

    # ---- timed, end to end through the autograd API with host buffers
    e2e_ms = float("nan")
    if not args.no_e2e:
        for _ in range(2):
            step_e2e()
        if pipe is not None:
            pipe.synchronize()
        barrier(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step_e2e()
        if pipe is not None:
            pipe.join()
        e1.record()
        barrier(world)
        e2e_ms = reduce_max(e0.elapsed_time(e1), world)

    if rank != 0:
        if world > 1:
            torch.distributed.destroy_process_group()
        return

    peaks = measured_peaks()
    ms_per_step = total_ms / args.steps
    value = fl["fwd_bwd"] * world / (ms_per_step * 1e-3) / 1e12
    e2e_value = fl["fwd_bwd"] * world / (e2e_ms / args.steps * 1e-3) / 1e12
    shape = _lib.Shape(cfg["b"], cfg["n"], cfg["hq"], cfg["hk"], cfg["d"], w1, w2, 0, 0, _lib.SA2_BF16,
                       _lib.KERNELS[args.kernel], cfg["d"] ** -0.5)
    lib = _lib.lib()
    launches = lib.sa2_kernel_launches(ctypes.byref(shape), 0) + lib.sa2_kernel_launches(ctypes.byref(shape), 1)
    fwd_avg, bwd_avg = statistics.mean(fwd_ms), statistics.mean(bwd_ms)
    fwd_tf = fl["fwd"] / (fwd_avg * 1e-3) / 1e12
    bwd_tf = fl["bwd"] / (bwd_avg * 1e-3) / 1e12
    min_bytes = {"fwd": 6 * cfg["b"] * cfg["n"] * cfg["hq"] * cfg["d"] * 2, "bwd": 12 * cfg["b"] * cfg["n"] * cfg["hq"] * cfg["d"] * 2}

    # DRAM bytes per launch from the ncu captures summarised under profiles/ (C3, tensor-core kernels):
    # backward = dK1/dV1 kernel 115.6 MB + dQ/dK2/dV2 kernel 293.4 MB; forward 91.4 MB
    traffic_bwd = 409.0e6 if (args.workload == "C3" and args.kernel == "auto" and not seq) else None
    traffic_fwd = 91.4e6 if (args.workload == "C3" and args.kernel == "auto" and not seq) else None
    line = {
        "metric": "2-simplicial attn fwd+bwd TFLOP/s", "value": value, "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, **cfg, "global_batch": cfg["b"] * world, "kernel": args.kernel,
                   "sharding": ("sequence blocks, NCCL send/recv of the w1-1 / w2-1 row halo" if seq
                                else "batch x head per rank, no collective"),
                   "l2": "256 MB buffer written between timed steps"},
        "tokens_per_s": cfg["b"] * cfg["n"] * world / (ms_per_step * 1e-3),
        "e2e": None if args.no_e2e else {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms / args.steps},
        "gpu_launches": launches * args.steps,
        "roofline": {"bound": "tensor", "kernel": "sa2_bwd", "achieved": bwd_tf, "peak": peaks["tflops"], "unit": "TFLOP/s",
                     "frac": bwd_tf / peaks["tflops"], "traffic": traffic_bwd, "peak_source": peaks["source"],
                     "ms_per_launch": bwd_avg},
        "roofline_fwd": {"bound": "tensor", "kernel": "sa2_fwd", "achieved": fwd_tf, "peak": peaks["tflops"],
                         "unit": "TFLOP/s", "frac": fwd_tf / peaks["tflops"], "traffic": traffic_fwd, "ms_per_launch": fwd_avg},
        "hbm_min_gbs": {"fwd": min_bytes["fwd"] / (fwd_avg * 1e-3) / 1e9, "bwd": min_bytes["bwd"] / (bwd_avg * 1e-3) / 1e9,
                        "peak": peaks["hbm_gbs"]},
        "clocks": clocks,
    }
    if world == 1 and not args.no_cpu_baseline:
        tf, sec, desc, _ = cpu_oracle_sample(cfg)
        line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                                "sample": desc, "host_cpus": os.cpu_count()}
    print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
