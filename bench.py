"""Benchmark of sliding-window causal 2-simplicial attention, forward + backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload C3|C2|C5|C4]
                    [--kernel auto|simt|tcgen05] [--impl ours|reference]

A step is one forward + backward pass of the operator over one batch of
seeded synthetic tensors.  The default workload is the forward+backward
configuration b4 h8 n4096 d64 w1=512 w2=32 bf16 ("C3"); with N GPUs every rank
runs that batch on its own GPU (batch x head sharding, no collective on the
data path), so the global batch is 4*N and scaling is weak.

Prints ONE JSON line:
  value     whole-job TFLOP/s with the inputs resident in HBM (the timed steps
            replay CUDA graphs of the sa2_fwd and sa2_bwd calls), counting only
            algorithmic work: 14*d flop per unmasked (i, j, k) triple
            (4*d forward, 10*d backward); masked cells, the elementwise
            products, the softmax and any recomputation count zero;
  e2e       the same metric through the package's host-buffer call
            (HostPipeline.run) with pinned HOST tensors: host->device copy of
            q, k, k', v, v', dO and device->host copy of out and the five
            gradients inside the timed region, on three streams so that they
            overlap the kernels of the neighbouring steps (--e2e-chunk cuts a
            call into batch chunks that overlap within the call);
  roofline  the dominant kernel (timed alone, live, with CUDA events) against the
            measured burst bf16 tensor peak of this pool's B200s, the sustained
            figure beside it; `kernels` lists all three tensor-core kernels;
  seq       (N > 1) the same tensors as ONE sequence of length n*N in sequence
            blocks with the NCCL halo exchange; c5: the long-sequence
            configuration (b8 h16 n16384 d128) split over the N ranks;
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
    # two (batch, head) pairs of C5 and one batch element of C3: small cases for profiler captures
    "C5s": dict(b=1, hq=2, hk=2, n=16384, d=128, w1=512, w2=32),
    "C3s": dict(b=1, hq=8, hk=8, n=4096, d=64, w1=512, w2=32),
}
# CPU sample: two batch elements, eight heads, up to 4096 rows of the same head dim and windows (~10 s on 16 cores)
CPU_SAMPLE = dict(b=2, hq=8, hk=8, n=4096)


def valid_pairs(n, w1, w2):
    return sum(min(i + 1, w1) * min(i + 1, w2) for i in range(n))


def work_flops(cfg):
    p = valid_pairs(cfg["n"], cfg["w1"], cfg["w2"]) * cfg["b"] * cfg["hq"]
    return {"fwd": 4 * cfg["d"] * p, "bwd": 10 * cfg["d"] * p, "fwd_bwd": 14 * cfg["d"] * p}


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


def host_threads():
    """Host threads this process may use.  A launcher such as torch.distributed.run exports
    OMP_NUM_THREADS=1; the CPU arm uses every core its affinity mask allows instead."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def cpu_oracle_sample(cfg, steps=1, warmup=0, budget_s=None):
    """Oracle forward + backward on a bounded CPU sample; returns (TFLOP/s, seconds per pass, description,
    sample).  With ``budget_s`` the sample ((batch, head) pairs of up to 4096 rows) is sized from a one-pair
    probe so that warmup + steps passes fit the budget."""
    from oracle import oracle as O
    s = dict(cfg)
    s.update(CPU_SAMPLE)
    s["n"] = min(s["n"], cfg["n"])
    if budget_s is not None:
        probe = dict(s, b=1, hq=1, hk=1)
        ins = O.make_inputs(1, probe["n"], 1, 1, probe["d"], seed=1)
        t0 = time.perf_counter()
        O.two_simplicial_fwd_bwd(*ins, probe["w1"], probe["w2"], chunk=32)
        per_pair = time.perf_counter() - t0
        # the probe itself used every thread; more pairs parallelise better, credit at most 4x (1x on one core)
        gain = float(min(4, torch.get_num_threads()))
        pairs = int(budget_s / max(1, warmup + steps) / max(per_pair / gain, 1e-3))
        pairs = max(1, min(16, pairs))
        s["b"], s["hq"], s["hk"] = 1, pairs, pairs
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
    """The reference arm: the CPU path of the operator (the oracle port of the reference's naive PyTorch
    implementation) on this machine's host cores.  Rank 0 alone runs it; the other ranks exit at once."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = host_threads()
    tf, sec, desc, s = cpu_oracle_sample(cfg, steps=max(1, args.steps), warmup=min(args.warmup, 1), budget_s=150.0)
    line = {
        "impl": "reference", "metric": "2-simplicial attn fwd+bwd TFLOP/s", "value": tf, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": sec * 1e3,
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


def load_traffic():
    """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the tensor-core kernels, taken
    from the ncu captures summarised under profiles/ and scaled to a full launch where the capture was a
    smaller case.  Keyed by "<workload>:<kernel>"."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        with open(path) as f:
            return json.load(f)
    except (OSError, ValueError):
        return {}


def timed_operator(sa, _lib, tensors, w1, w2, kernel, steps, flush):
    """Per-step CUDA-event timing on the current stream, L2 flushed between steps: the forward and the
    backward entry points.  Each is captured once into a CUDA graph (the same sa2_fwd / sa2_bwd calls on the
    capturing stream) and replayed per step, so that a slow or busy host cannot leave the GPU idle between
    the launches of a step; if the capture fails the calls are made directly.  Returns the two lists of
    milliseconds and how the steps were launched."""
    q, k1, k2, v1, v2, do = tensors
    how = "direct calls"
    run_f = run_b = None
    try:
        gf, gb = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        # thread-local capture: what other threads of the process do meanwhile (a collective library's watchdog)
        # neither joins nor breaks the capture
        with torch.cuda.graph(gf, capture_error_mode="thread_local"):
            out, lse = sa.sa2_forward(q, k1, k2, v1, v2, w1, w2, kernel=kernel)
        call = sa.BackwardCall(q, k1, k2, v1, v2, out, lse, do, w1, w2, kernel=kernel)
        with torch.cuda.graph(gb, capture_error_mode="thread_local"):
            call.launch(0)
        gf.replay()
        gb.replay()
        torch.cuda.synchronize()
        run_f, run_b, how = gf.replay, gb.replay, "CUDA graphs of the forward call and of the backward call, replayed per step"
    except Exception as e:      # noqa: BLE001 - any capture problem falls back to plain launches
        sys.stderr.write("bench: graph capture failed (%s); launching directly\n" % (e,))
        torch.cuda.synchronize()
        state = {}

        def run_f():
            state["fwd"] = sa.sa2_forward(q, k1, k2, v1, v2, w1, w2, kernel=kernel)

        def run_b():
            sa.sa2_backward(q, k1, k2, v1, v2, state["fwd"][0], state["fwd"][1], do, w1, w2, kernel=kernel)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
    for s in range(steps):
        flush.zero_()
        ev[s][0].record()
        run_f()
        ev[s][1].record()
        run_b()
        ev[s][2].record()
    torch.cuda.synchronize()
    return [e[0].elapsed_time(e[1]) for e in ev], [e[1].elapsed_time(e[2]) for e in ev], how


def timed_kernels(sa, _lib, tensors, w1, w2, kernel, steps, flush):
    """The backward's kernels timed apart, live, with CUDA events on the launching stream (the phases of
    sa2_bwd are launched one by one; L2 flushed before each): milliseconds per launch of the row sums, the
    dK1/dV1 kernel and the dQ/dK2/dV2 kernel (+ its reduction)."""
    q, k1, k2, v1, v2, do = tensors
    out, lse = sa.sa2_forward(q, k1, k2, v1, v2, w1, w2, kernel=kernel)
    call = sa.BackwardCall(q, k1, k2, v1, v2, out, lse, do, w1, w2, kernel=kernel)
    call.launch(0)
    res = {}
    for name, phase in (("rowsum", _lib.BWD_ROWSUM), ("dk1_dv1", _lib.BWD_K1), ("dq_dk2_dv2", _lib.BWD_Q)):
        ms = []
        for _ in range(steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            call.launch(phase)
            e1.record()
            torch.cuda.synchronize()
            ms.append(e0.elapsed_time(e1))
        res[name] = statistics.mean(ms)
    return res


def seq_record(sa, cfg, kernel, steps, world, rank, dev, flush):
    """The same per-rank tensors as ONE sequence of length n * N split into consecutive blocks, one per
    rank, with the key/value halo exchanged over NCCL (simplicial_attention_b200/shard.py)."""
    from simplicial_attention_b200 import shard
    import torch.distributed as dist
    w1, w2 = cfg["w1"], cfg["w2"]
    _, devt = make_inputs(cfg, seed=4321 + rank, dtype=torch.bfloat16, device=dev)
    q, k1, k2, v1, v2, do = devt

    def step():
        leaves = [t.detach().requires_grad_() for t in (q, k1, k2, v1, v2)]
        out = shard.sequence_parallel_attn(leaves[0], (leaves[1], leaves[2]), (leaves[3], leaves[4]), w1=w1, w2=w2, kernel=kernel)
        out.backward(do)

    for _ in range(3):
        step()
    barrier(world)
    ms = []
    for _ in range(steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step()
        e1.record()
        torch.cuda.synchronize()
        ms.append(e0.elapsed_time(e1))
    barrier(world)
    step_ms = reduce_max(sum(ms), world) / steps
    # the exchange alone (forward halos): events around the batched send/recv of the four tails
    h1, h2, n = w1 - 1, w2 - 1, cfg["n"]
    ex_ms = []
    for _ in range(steps):
        send = [k1[:, n - h1:].contiguous(), v1[:, n - h1:].contiguous(), k2[:, n - h2:].contiguous(), v2[:, n - h2:].contiguous()]
        recv = [torch.empty_like(t) for t in send]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        e0.record()
        ex = shard._Exchange(send if rank < world - 1 else None, rank + 1, recv if rank > 0 else None, rank - 1, None, "forward")
        ex.wait(60.0)
        e1.record()
        torch.cuda.synchronize()
        ex_ms.append(e0.elapsed_time(e1))
    exchange_ms = reduce_max(statistics.median(ex_ms), world)
    whole = dict(cfg, n=cfg["n"] * world)
    fl = work_flops(whole)["fwd_bwd"]
    halo_bytes = 2 * cfg["b"] * cfg["hk"] * cfg["d"] * 2 * (h1 + h2)
    return {"sharding": "sequence blocks, one NCCL send/recv batch of the w1-1 / w2-1 row halo per direction, overlapped with the interior rows",
            "sequence": cfg["n"] * world, "ms_per_step": step_ms, "value": fl / (step_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "tokens_per_s": cfg["b"] * cfg["n"] * world / (step_ms * 1e-3),
            "halo_bytes_per_boundary": halo_bytes, "exchange_ms": exchange_ms}


def c5_record(sa, kernel, world, rank, dev, flush, steps=2):
    """Strong scaling of the long-sequence configuration (b8 h16 n16384 d128, w 512/32): ONE problem split
    over the N ranks by batch (no communication) and, for N > 1, by sequence blocks with the halo exchange."""
    cfg = dict(WORKLOADS["C5"])
    if cfg["b"] % world:
        return {"skipped": f"batch {cfg['b']} does not divide over {world} ranks"}
    fl = work_flops(cfg)["fwd_bwd"]
    w1, w2 = cfg["w1"], cfg["w2"]
    rec = {"config": dict(cfg), "scaling": "strong", "unit": "TFLOP/s"}

    def run(local, fn):
        _, devt = make_inputs(local, seed=555 + rank, dtype=torch.bfloat16, device=dev)
        for _ in range(2):
            fn(devt)
        barrier(world)
        ms = []
        for _ in range(steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn(devt)
            e1.record()
            torch.cuda.synchronize()
            ms.append(e0.elapsed_time(e1))
        barrier(world)
        del devt
        torch.cuda.empty_cache()
        return reduce_max(sum(ms), world) / steps

    def batch_step(t):
        q, k1, k2, v1, v2, do = t
        out, lse = sa.sa2_forward(q, k1, k2, v1, v2, w1, w2, kernel=kernel)
        sa.sa2_backward(q, k1, k2, v1, v2, out, lse, do, w1, w2, kernel=kernel)

    ms = run(dict(cfg, b=cfg["b"] // world), batch_step)
    rec["batch_split"] = {"ms_per_step": ms, "value": fl / (ms * 1e-3) / 1e12, "tokens_per_s": cfg["b"] * cfg["n"] / (ms * 1e-3)}
    if world > 1 and cfg["n"] % world == 0:
        from simplicial_attention_b200 import shard

        def seq_step(t):
            leaves = [x.detach().requires_grad_() for x in t[:5]]
            out = shard.sequence_parallel_attn(leaves[0], (leaves[1], leaves[2]), (leaves[3], leaves[4]), w1=w1, w2=w2, kernel=kernel)
            out.backward(t[5])

        ms = run(dict(cfg, n=cfg["n"] // world), seq_step)
        rec["sequence_split"] = {"ms_per_step": ms, "value": fl / (ms * 1e-3) / 1e12, "tokens_per_s": cfg["b"] * cfg["n"] / (ms * 1e-3),
                                 "halo_bytes_per_boundary": 2 * cfg["b"] * cfg["hk"] * cfg["d"] * 2 * (w1 - 1 + w2 - 1)}
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="C3", choices=sorted(WORKLOADS) + ["C4"])
    ap.add_argument("--kernel", default="auto", choices=("auto", "simt", "tcgen05"))
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (for profiler captures)")
    ap.add_argument("--no-extra", action="store_true", help="skip the sequence-sharded and long-sequence records")
    ap.add_argument("--e2e-chunk", type=int, default=0, help="batch elements per chunk of the host-buffer leg (default: the whole batch; copies then overlap the kernels of the neighbouring steps)")
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
    big = args.workload == "C5"
    if args.workload in ("C5s", "C3s"):
        args.no_extra = args.no_e2e = args.no_cpu_baseline = True
    numa_cpus, all_cpus = None, (os.sched_getaffinity(0) if hasattr(os, "sched_getaffinity") else None)
    if not (args.no_e2e or big):
        from simplicial_attention_b200.host import bind_to_device_cpus
        numa_cpus = bind_to_device_cpus(dev)        # before the pinned buffers are allocated
    host, devt = make_inputs(cfg, seed=1234 + rank, dtype=dtype, device=dev, pin=not (args.no_e2e or big))
    w1, w2 = cfg["w1"], cfg["w2"]
    fl = work_flops(cfg)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)   # > 126 MB L2
    steps = args.steps
    warmup = max(3, args.warmup)

    # ---- warm-up
    for _ in range(warmup):
        out, lse = sa.sa2_forward(*devt[:5], w1, w2, kernel=args.kernel)
        sa.sa2_backward(*devt[:5], out, lse, devt[5], w1, w2, kernel=args.kernel)
    torch.cuda.synchronize()
    sa.check_device()

    # ---- timed, inputs resident in HBM
    sampler = ClockSampler(local)
    barrier(world)
    if rank == 0:
        sampler.start()
    fwd_ms, bwd_ms, launch_how = timed_operator(sa, _lib, devt, w1, w2, args.kernel, steps, flush)
    barrier(world)
    total_ms = reduce_max(sum(fwd_ms) + sum(bwd_ms), world)
    clocks = sampler.stop() if rank == 0 else None
    kern_ms = timed_kernels(sa, _lib, devt, w1, w2, args.kernel, min(steps, 5), flush)

    # ---- timed, end to end from pinned host buffers (copies inside the timed region)
    e2e = None
    if not (args.no_e2e or big):
        from simplicial_attention_b200.host import HostPipeline
        outs_h = [torch.empty_like(t).pin_memory() for t in [host[0]] + host[:5]]
        pipe = HostPipeline(dev, w1=w1, w2=w2, chunk=args.e2e_chunk or cfg["b"], kernel=args.kernel)
        for _ in range(3):
            pipe.run(host, outs_h)
        pipe.synchronize()
        pipe.record_copies()
        barrier(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            pipe.run(host, outs_h)      # three streams: copy-in, compute and copy-out of consecutive steps (and chunks) overlap
        pipe.join()
        e1.record()
        barrier(world)
        e2e_ms = reduce_max(e0.elapsed_time(e1), world) / steps
        pipe.synchronize()
        cs = pipe.copy_stats()
        gbs = torch.tensor([cs["h2d_gbs"] or 0.0, cs["d2h_gbs"] or 0.0], dtype=torch.float64, device=dev)
        if world > 1:
            lo = gbs.clone()
            torch.distributed.all_reduce(lo, op=torch.distributed.ReduceOp.MIN)
            gbs = lo
        e2e = {"value": fl["fwd_bwd"] * world / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in host),
               "d2h_bytes_per_step": sum(t.numel() * t.element_size() for t in outs_h),
               "ms_per_step": e2e_ms, "h2d_gbs_min_rank": gbs[0].item(), "d2h_gbs_min_rank": gbs[1].item(),
               "host_cpus_rank0": (len(numa_cpus) if numa_cpus else "unchanged"),
               "note": "throughput of back-to-back pipelined calls (copies of step s+1 overlap the kernels of step s), "
                       "not the latency of one call; GB/s = bytes / time the copy stream was busy, slowest rank"}
        del pipe, outs_h
    if numa_cpus and all_cpus:
        os.sched_setaffinity(0, all_cpus)           # the CPU baseline below uses every core again

    # ---- extra records: the partitioned multi-GPU paths
    seq = c5 = None
    if not args.no_extra and not big:
        del devt
        torch.cuda.empty_cache()
        if world > 1:
            seq = seq_record(sa, cfg, args.kernel, min(steps, 5), world, rank, dev, flush)
        c5 = c5_record(sa, args.kernel, world, rank, dev, flush)
    status = sa.device_status()

    if rank != 0:
        if world > 1:
            torch.distributed.destroy_process_group()
        return

    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        with open(peaks_path) as f:
            m = json.load(f)
        burst, sustained, hbm, psrc = float(m["bf16_tflops"]), float(m.get("bf16_tflops_sustained") or m["bf16_tflops"]), float(m["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    else:
        burst, sustained, hbm, psrc = 1590.0, 1400.0, 6650.0, "fallback (earlier measurement on this pool)"
    ms_per_step = total_ms / steps
    value = fl["fwd_bwd"] * world / (ms_per_step * 1e-3) / 1e12
    shape = _lib.Shape(cfg["b"], cfg["n"], cfg["hq"], cfg["hk"], cfg["d"], w1, w2, 0, 0, _lib.SA2_BF16,
                       _lib.KERNELS[args.kernel], cfg["d"] ** -0.5)
    lib = _lib.lib()
    launches = lib.sa2_kernel_launches(ctypes.byref(shape), 0) + lib.sa2_kernel_launches(ctypes.byref(shape), 1)
    fwd_avg, bwd_avg = statistics.mean(fwd_ms), statistics.mean(bwd_ms)
    # algorithmic work per kernel: forward 2 GEMM-equivalents (4 d per triple); of the backward's 5, the dK1/dV1
    # kernel owns 2 (4 d) and the dQ/dK2/dV2 kernel 3 (6 d); recomputed products count zero
    kernels = {
        "fwd": {"ms": fwd_avg, "flops": fl["fwd"]},
        "dk1_dv1": {"ms": kern_ms["dk1_dv1"], "flops": fl["bwd"] * 0.4},
        "dq_dk2_dv2": {"ms": kern_ms["dq_dk2_dv2"], "flops": fl["bwd"] * 0.6},
    }
    for k in kernels.values():
        k["tflops"] = k["flops"] / (k["ms"] * 1e-3) / 1e12
        k["frac_of_burst"] = k["tflops"] / burst
    top = max(kernels, key=lambda k: kernels[k]["ms"])
    traffic = load_traffic()
    min_bytes = {"fwd": 6 * cfg["b"] * cfg["n"] * cfg["hq"] * cfg["d"] * 2, "bwd": 12 * cfg["b"] * cfg["n"] * cfg["hq"] * cfg["d"] * 2}
    line = {
        "metric": "2-simplicial attn fwd+bwd TFLOP/s", "value": value, "unit": "TFLOP/s",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, **cfg, "global_batch": cfg["b"] * world, "kernel": args.kernel,
                   "sharding": "batch x head per rank, no collective",
                   "l2": "256 MB buffer written between timed steps", "launch": launch_how},
        "tokens_per_s": cfg["b"] * cfg["n"] * world / (ms_per_step * 1e-3),
        "e2e": e2e,
        "gpu_launches": launches * steps,
        "roofline": {"bound": "tensor", "kernel": top, "achieved": kernels[top]["tflops"], "peak": burst, "unit": "TFLOP/s",
                     "frac": kernels[top]["tflops"] / burst, "frac_of_sustained": kernels[top]["tflops"] / sustained,
                     "peak_sustained": sustained, "traffic": traffic.get(f"{args.workload}:{top}"),
                     "peak_source": psrc + ": cuBLAS bf16 burst; the sustained figure beside it",
                     "ms_per_launch": kernels[top]["ms"]},
        "kernels": {k: {"ms_per_launch": v["ms"], "tflops": v["tflops"], "frac_of_burst": v["frac_of_burst"],
                        "traffic": traffic.get(f"{args.workload}:{k}")} for k, v in kernels.items()},
        "step_frac_of_burst": value / world / burst,
        "rowsum_ms": kern_ms["rowsum"],
        "hbm_min_gbs": {"fwd": min_bytes["fwd"] / (fwd_avg * 1e-3) / 1e9, "bwd": min_bytes["bwd"] / (bwd_avg * 1e-3) / 1e9,
                        "peak": hbm},
        "clocks": clocks, "device_status": status,
    }
    if seq is not None:
        line["seq"] = seq
    if c5 is not None:
        line["c5"] = c5
    if world == 1 and not args.no_cpu_baseline:
        threads = host_threads()
        tf, sec, desc, _ = cpu_oracle_sample(cfg, budget_s=25.0)
        line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                "sample": desc, "host_cpus": os.cpu_count()}
    print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
