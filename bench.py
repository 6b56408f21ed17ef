"""Benchmark of the MoE layer forward+backward hot path (MXFP8, sm_100a).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config C2|C3|C4|C5]

One "step" = one forward + backward of the expert compute on pre-routed inputs
(routing metadata, quantizers, six grouped GEMMs, two combines, weight-gradient
accumulation into an fp32 main_grad) - the region the reference's own benchmark
times.  N=1 runs config C2 (T=8192 H=3072 I=1536 E=8 K=8); N>1 runs the
expert-parallel step (experts sharded over ranks, NCCL all-to-all dispatch and
combine) with a fixed number of tokens per rank (weak scaling); before timing,
every multi-GPU run checks a small expert-parallel step against the single-GPU
layer ("ep_parity"), and after the headline series it also times the skewed
fine-grained config and the large-TK config with the GLOBAL token count fixed
(strong scaling; "ep_c4_strong", "ep_c5_strong").
Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "supersonic-moe_b200"))

import torch  # noqa: E402

CONFIGS = {
    "C1": dict(T=256, H=256, I=128, E=8, K=2, seed=0, skew=False),
    "C2": dict(T=8192, H=3072, I=1536, E=8, K=8, seed=0, skew=False),
    "C3": dict(T=8192, H=4096, I=4096, E=8, K=8, seed=1, skew=False),
    "C4": dict(T=16384, H=2048, I=768, E=128, K=8, seed=2, skew=True),
    "C5": dict(T=65536, H=6144, I=3072, E=64, K=8, seed=3, skew=False),
    # C5's layer on a token count that a 1-GPU smoke run can hold next to the 64 experts' weights
    "C5s": dict(T=8192, H=6144, I=3072, E=64, K=8, seed=3, skew=False),
    # C2's layer at T=2048: small enough for multi-pass ncu captures, weights (453 MB bf16 + 226 MB fp8) >> L2
    "P1": dict(T=2048, H=3072, I=1536, E=8, K=8, seed=0, skew=False),
    # the reference's published sweeps around C2 (README.md:343-347, HANDOFF.md:27-33)
    "T1024": dict(T=1024, H=3072, I=1536, E=8, K=8, seed=0, skew=False),
    "T4096": dict(T=4096, H=3072, I=1536, E=8, K=8, seed=0, skew=False),
    "T16384": dict(T=16384, H=3072, I=1536, E=8, K=8, seed=0, skew=False),
    "E16": dict(T=8192, H=3072, I=1536, E=16, K=8, seed=0, skew=False),
    "E32": dict(T=8192, H=3072, I=1536, E=32, K=8, seed=0, skew=False),
}


def ncu_dram_bytes(cname):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of the six GEMMs of one step, from the ncu capture
    summarised beside this table under profiles/ ({"<op>#<occurrence within a step>": bytes}); None when no capture
    of this workload is kept."""
    path = os.path.join(ROOT, "profiles", f"gemm_dram_traffic_{cname.lower()}.json")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        return json.load(f).get("bytes_per_launch")

# reference README.md:28-38,343-348, HANDOFF.md:27-34 (its own FP8 path, 1x SM100)
PUBLISHED_US = {"C2": 2659.8, "C3": 8521.7, "T1024": 566.0, "P1": 870.1, "T4096": 1459.1, "T16384": 5224.9,
                "E16": 2800.7, "E32": 3187.5}
FP8_PEAK_NOMINAL = 4.5e15
# kernels launched per wrapper call (sonicmoe/ops.py)
LAUNCHES = dict(topk_metadata=3, count_cumsum=3)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16=d["bf16_tflops"], bf16_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


def make_inputs(cfg, device, T=None, weights=True):
    """Seeded synthetic inputs with the shapes and distributions of the named config:
    x, dy ~ N(0,1) bf16; weights ~ N(0,0.02) bf16; router logits ~ N(0,1) (+ log Zipf(1.2) bias over a seeded
    expert permutation when skewed); top-K of the logits, softmax over the K selected."""
    T = T or cfg["T"]
    H, I, E, K = cfg["H"], cfg["I"], cfg["E"], cfg["K"]
    # the largest config (C5: 2.4 G weight elements) is drawn on the device, expert by expert, from a seeded
    # device generator: the host-side draw would need tens of GB of fp32 scratch; everything else is drawn on the
    # host so that the numbers match the CPU oracle's inputs
    big = E * 2 * I * H > (1 << 30)
    gdev = torch.device(device) if big else torch.device("cpu")
    g = torch.Generator(device=gdev).manual_seed(cfg["seed"])
    rn = lambda *shape: torch.randn(*shape, generator=g, device=gdev)
    x = rn(T, H).to(torch.bfloat16)
    dy = rn(T, H).to(torch.bfloat16)
    if not weights:
        w1 = w2 = None
    elif big:
        w1 = torch.stack([(rn(2 * I, H) * 0.02).to(torch.bfloat16) for _ in range(E)])
        w2 = torch.stack([(rn(H, I) * 0.02).to(torch.bfloat16) for _ in range(E)])
    else:
        w1 = (rn(E, 2 * I, H) * 0.02).to(torch.bfloat16)
        w2 = (rn(E, H, I) * 0.02).to(torch.bfloat16)
    logits = rn(T, E)
    if cfg["skew"]:
        p = torch.arange(1, E + 1, dtype=torch.float32, device=gdev) ** -1.2
        logits = logits + torch.log(p / p.sum())[torch.randperm(E, generator=g, device=gdev)]
    vals, idx = logits.topk(K, dim=-1)
    scores = torch.softmax(vals, dim=-1)
    return dict(x=x, dy=dy, w1=w1, w2=w2, idx=idx.to(torch.int32), scores=scores.float())


class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx, self.proc, self.lines = gpu_index, None, []
        self.nvml, self.samples, self.stop_flag = None, [], False

    def _physical_index(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if self.idx < len(ids) and ids[self.idx].isdigit():
                return int(ids[self.idx])
        return self.idx

    def start(self):
        """Read-only NVML polling every ~2 ms in a thread (a timed region lasts tens of ms); nvidia-smi at 100 ms
        is the fallback when the NVML binding is missing."""
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.max_sm = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.idx)], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _poll(self):
        n = self.nvml
        while not self.stop_flag:
            try:
                clk = n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)
                rs = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                pw = n.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
                self.samples.append((clk, rs, pw))
            except Exception:
                pass
            time.sleep(0.002)

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.nvml is not None:
            self.stop_flag = True
            self.thread.join(timeout=1.0)
            n = self.nvml
            names = (("hw_slowdown", "nvmlClocksEventReasonHwSlowdown"),
                     ("hw_thermal_slowdown", "nvmlClocksEventReasonHwThermalSlowdown"),
                     ("sw_thermal_slowdown", "nvmlClocksEventReasonSwThermalSlowdown"),
                     ("sw_power_cap", "nvmlClocksEventReasonSwPowerCap"))
            reasons = set()
            raw = 0
            for _, rs, _ in self.samples:
                raw |= rs
                for name, attr in names:
                    bit = getattr(n, attr, None)
                    if bit is None:
                        bit = getattr(n, attr.replace("ClocksEventReason", "ClocksThrottleReason"), 0)
                    if rs & bit:
                        reasons.add(name)
            sm = [c for c, _, _ in self.samples]
            pw = [p for _, _, p in self.samples]
            return dict(sm_mhz=statistics.median(sm) if sm else None, sm_min_mhz=min(sm) if sm else None,
                        sm_max_mhz=self.max_sm, reasons=sorted(reasons), samples=len(sm),
                        power_w=round(statistics.median(pw), 0) if pw else None, reasons_mask=hex(raw),
                        source="nvml, 2 ms polling")
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [t.strip() for t in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm), source="nvidia-smi -lms 100")


def flops_of(cfg, T=None):
    return 18.0 * (T or cfg["T"]) * cfg["K"] * cfg["H"] * cfg["I"]


# ------------------------------------------------------------------ CPU reference arm
def cpu_reference(cfg, budget_s=20.0, T_job=None):
    """The reference's pure-PyTorch expert path (restated in oracle/moe.py) timed on the host cores with all the
    threads the box offers, on a bounded token sub-sample of the same config and the SAME region as the GPU arm:
    pre-routed inputs, expert compute forward + backward (the router linear / top-k stay outside, as in the
    reference's own benchmark); reported scaled linearly in T to the job's token count."""
    from oracle.moe import TorchMoEBaseline
    try:
        torch.set_num_threads(max(1, os.cpu_count() or 1))     # torchrun pins OMP_NUM_THREADS=1: undo it here
    except Exception:
        pass
    torch.manual_seed(cfg["seed"])
    H, I, E, K = cfg["H"], cfg["I"], cfg["E"], cfg["K"]
    T_job = T_job or cfg["T"]
    cores = torch.get_num_threads()
    Ts = 256
    model = TorchMoEBaseline(E, K, H, I, seed=cfg["seed"])
    x = torch.randn(Ts, H).to(torch.bfloat16).requires_grad_(True)
    dy = torch.randn(Ts, H).to(torch.bfloat16)
    logits = torch.randn(Ts, E)
    vals, idx = logits.topk(K, dim=-1)
    scores = torch.softmax(vals, dim=-1)

    def step():
        model.zero_grad(set_to_none=True)
        out = model.experts_only(x, idx, scores)
        out.backward(dy)

    step()
    t0 = time.perf_counter(); step(); t1 = time.perf_counter() - t0
    iters = max(1, min(5, int(budget_s / max(t1, 1e-3))))
    ts = []
    for _ in range(iters):
        t0 = time.perf_counter(); step(); ts.append(time.perf_counter() - t0)
    med = statistics.median(ts)
    us_full = med * 1e6 * T_job / Ts
    return dict(value=us_full, unit="us/iter", cores=cores, kind="port",
                sample=f"T={Ts} of {T_job} tokens (same H,I,E,K; pre-routed expert compute fwd+bwd, autograd, bf16 "
                       f"params; router outside, as in the GPU arm), median of {iters} iters = {med * 1e3:.1f} ms, "
                       f"scaled linearly in T; torch threads={cores}, os.cpu_count()={os.cpu_count()}")


def config_keys(cname, cfg, world, T_rank, scaling):
    """The `config` object shared by both arms."""
    T, H, I, E, K = cfg["T"], cfg["H"], cfg["I"], cfg["E"], cfg["K"]
    c = {"workload": f"{cname}: T={T_rank}{' per rank' if world > 1 else ''} H={H} I={I} E={E} K={K}, seed "
                     f"{cfg['seed']}" + (f", expert-parallel over {world} ranks ({scaling} scaling)" if world > 1 else ""),
         "l2": "no flush: one step touches ~2.5 GB (> 126 MB L2)",
         "timed_region": "same as the reference's bench (pre-routed expert compute; router linear/top-k outside)"}
    return c


# ------------------------------------------------------------------ same-box library bar (diagnostic, not product)
def fp8_library_bar(cfg, dev):
    """cuBLASLt's MXFP8 block-scaled GEMM (torch._scaled_mm, e4m3 x e4m3, ue8m0 1x32 scales) on dense problems
    with the FLOPs and shapes of the four plain GEMMs of this layer: what a library kernel reaches on this box,
    next to the "2 x measured bf16" estimate of the FP8 peak.  Diagnostic leg only - nothing here is on the
    product path."""
    T, H, I, E, K = cfg["T"], cfg["H"], cfg["I"], cfg["E"], cfg["K"]
    TK = T * K
    shapes = {"down_proj": (TK, H, I), "dgrad_dx": (TK, H, 2 * I), "dw1": (2 * I, H, TK), "dw2": (I, H, TK)}
    out = {}
    ceil = lambda a, b: -(-a // b)
    try:
        for name, (M, N, Kd) in shapes.items():
            a = torch.randint(0, 120, (M, Kd), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
            b = torch.randint(0, 120, (N, Kd), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
            sa = torch.full((ceil(M, 128) * 128 * ceil(Kd // 32, 4) * 4,), 127, dtype=torch.uint8,
                            device=dev).view(torch.float8_e8m0fnu)
            sb = torch.full((ceil(N, 128) * 128 * ceil(Kd // 32, 4) * 4,), 127, dtype=torch.uint8,
                            device=dev).view(torch.float8_e8m0fnu)
            f = lambda: torch._scaled_mm(a, b.t(), sa, sb, out_dtype=torch.bfloat16)
            for _ in range(3):
                f()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            n = 10
            e0.record()
            for _ in range(n):
                f()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) / n * 1e3
            out[name] = {"us": round(us, 1), "tflops": round(2.0 * M * N * Kd / us / 1e6, 1), "dense_shape": [M, N, Kd]}
            del a, b, sa, sb
        out["note"] = ("torch._scaled_mm MXFP8 on ONE dense GEMM of the same FLOPs per call (the layer's calls are "
                       "grouped over E experts), 10 back-to-back launches after 3 warm-ups")
    except Exception as exc:     # this torch build has no block-scaled _scaled_mm: say so, carry on
        out = {"unavailable": repr(exc)[:200]}
    return out


# ------------------------------------------------------------------ GPU arm
def run_ours(args):
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    import sonicmoe
    from sonicmoe import ops

    # One GPU: the reference-shape layer C2.  N GPUs: the same layer per rank (T tokens per rank, its E experts
    # sharded over the ranks), so the per-rank work equals the 1-GPU run and the values form one weak-scaling series.
    # The configs the expert-parallel case is specified on follow with the GLOBAL token count fixed (strong
    # scaling): the skewed fine-grained C4 and the large-TK C5.
    cname = args.config or "C2"
    parity = None
    if world > 1:
        parity = _ep_parity(dist, dev)
    line = _measure(args, cname, world, rank, dev, dist, sonicmoe, ops, strong=False)
    if world > 1 and args.config is None and not args.lean and not args.no_extras:
        for key, extra_cfg in (("ep_c4_strong", "C4"), ("ep_c5_strong", "C5")):
            torch.cuda.empty_cache()
            extra = _measure(args, extra_cfg, world, rank, dev, dist, sonicmoe, ops, strong=True, extra=True)
            if line is not None and extra is not None:
                line[key] = {k: extra[k] for k in ("value", "unit", "config", "scaling", "tokens_per_s", "tflops",
                                                   "per_step_ms", "kernel_us")}
    if line is not None:
        if parity is not None:
            line["ep_parity"] = parity
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def _write_timeline(path, step, d, rank, barrier):
    """The GPU operations of one step (kernels, copies, memsets of every stream) in start order, as text: start,
    duration, idle time since the previous operation ended, stream, name.  torch.profiler, not ncu (ncu is never put
    around a multi-rank command); rank 0 writes the file."""
    from torch.profiler import ProfilerActivity, profile
    barrier()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            step(d["x"], d["dy"], d["idx"], d["scores"])
        torch.cuda.synchronize()
    barrier()
    if rank != 0:
        return
    ops_ = [e for e in prof.events() if e.device_type is not None and "cuda" in str(e.device_type).lower()]
    ops_.sort(key=lambda e: e.time_range.start)
    # the middle step: from the second to the third occurrence of the step's first kernel
    first = ops_[0].name
    marks = [i for i, e in enumerate(ops_) if e.name == first]
    per = len(marks) // 3 if len(marks) >= 3 else 1
    a, b = (marks[per], marks[2 * per]) if len(marks) >= 3 * per and per > 0 else (0, len(ops_))
    t0 = ops_[a].time_range.start
    prev_end = t0
    with open(path, "w") as f:
        f.write(f"step: {ops_[b - 1].time_range.end - t0:.1f} us, {b - a} GPU operations (start us, duration us, "
                "idle us since the previous operation ended, name)\n")
        for e in ops_[a:b]:
            f.write(f"{e.time_range.start - t0:9.1f} {e.time_range.end - e.time_range.start:8.1f} "
                    f"{e.time_range.start - prev_end:7.1f}  {e.name[:100]}\n")
            prev_end = max(prev_end, e.time_range.end)


def _ep_parity(dist, dev):
    """A small expert-parallel step against the single-GPU layer on the same tokens, on every rank, before anything
    is timed: {tensor: [min cosine over ranks, max relative RMS error over ranks]} plus the verdict."""
    from sonicmoe.ep import PARITY_LIMITS, parity_against_single_gpu
    res = parity_against_single_gpu(dist.group.WORLD, dev)
    names = sorted(PARITY_LIMITS)
    t = torch.tensor([[-res[n][0], res[n][1]] for n in names], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    out = {n: [round(-float(t[i, 0]), 6), round(float(t[i, 1]), 6)] for i, n in enumerate(names)}
    out["ok"] = all(out[n][0] > PARITY_LIMITS[n][0] and out[n][1] < PARITY_LIMITS[n][1] for n in names)
    out["against"] = ("run_sonic_moe on one GPU with all experts local, same tokens (T=1024 per rank, H=512, I=256, "
                      "8 experts per rank, K=4); [min cos, max rrmse] over ranks")
    if not out["ok"]:
        raise RuntimeError(f"expert-parallel parity check failed: {out}")
    return out


def _measure(args, cname, world, rank, dev, dist, sonicmoe, ops, strong, extra=False):
    local = dev.index
    cfg = CONFIGS[cname]
    E, K, H, I = cfg["E"], cfg["K"], cfg["H"], cfg["I"]
    T = cfg["T"] // world if strong else cfg["T"]          # tokens of this rank
    big = E * 2 * I * H > (1 << 30)
    if world > 1:
        # every rank draws the experts' weights from the same seeded stream and keeps its own slice; its tokens come
        # from a rank-specific stream (all ranks hold different tokens, as data-parallel ranks do)
        El = E // world
        assert E % world == 0
        gdev = dev if big else torch.device("cpu")
        gw = torch.Generator(device=gdev).manual_seed(cfg["seed"])
        w1l, w2l = [], []
        for e in range(E):
            a = (torch.randn(2 * I, H, generator=gw, device=gdev) * 0.02).to(torch.bfloat16)
            b = (torch.randn(H, I, generator=gw, device=gdev) * 0.02).to(torch.bfloat16)
            if rank * El <= e < (rank + 1) * El:
                w1l.append(a.to(dev)); w2l.append(b.to(dev))
            del a, b
        w1 = torch.nn.Parameter(torch.stack(w1l)); w2 = torch.nn.Parameter(torch.stack(w2l))
        del w1l, w2l
        sub = dict(cfg, seed=cfg["seed"] + 1000 * (rank + 1), E=E)
        inp = make_inputs(sub, dev, T=T, weights=False)
        from sonicmoe.ep import ExpertParallelMoE
        ep = ExpertParallelMoE(E, K, dist.group.WORLD, capacity_tokens=T)
    else:
        El = E
        inp = make_inputs(cfg, dev, T=T)
        w1 = torch.nn.Parameter(inp["w1"].to(dev))
        w2 = torch.nn.Parameter(inp["w2"].to(dev))
    pin = {k: inp[k].cpu().pin_memory() for k in ("x", "dy", "idx", "scores")}
    w1.main_grad = torch.zeros(El, 2 * I, H, dtype=torch.float32, device=dev)
    w2.main_grad = torch.zeros(El, I, H, dtype=torch.float32, device=dev)
    sonicmoe.precompute_weight_fp8(w1, w2)          # once per optimizer step, outside the timed region
    counts = torch.bincount(inp["idx"].flatten().long(), minlength=E).tolist()
    d = {k: inp[k].to(dev) for k in ("x", "dy", "idx", "scores")}

    def step(x, dy, idx, scores):
        x = x.detach().requires_grad_(True)
        if world > 1:
            out = ep(x, idx, scores, w1, w2)
        else:
            out = sonicmoe.run_sonic_moe(x, idx, scores, K, E, w1, w2, fp8=True, tokens_per_expert=counts)
        out.backward(dy)
        return out, x.grad

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    steps = args.steps if not extra else max(4, min(args.steps, 8))
    warmup = args.warmup if not extra else 3
    for _ in range(warmup):
        step(d["x"], d["dy"], d["idx"], d["scores"])
    barrier()
    ops.check_status(dev)

    sampler = ClockSampler(local)
    sampler.start()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    barrier()
    ev[0].record()
    for i in range(steps):
        step(d["x"], d["dy"], d["idx"], d["scores"])
        ev[i + 1].record()
    barrier()
    ops.check_status(dev)
    total_ms = ev[0].elapsed_time(ev[-1])
    per_step = [ev[i].elapsed_time(ev[i + 1]) for i in range(steps)]
    ms = total_ms / steps

    if args.timeline:      # one more step under torch.profiler: every GPU operation with start, duration, gap
        _write_timeline(args.timeline, step, d, rank, barrier)
    if args.lean:      # profiling runs: warm-up + timed steps only, nothing else launches
        sampler.stop()
        if rank == 0:
            print(json.dumps({"metric": "MoE fwd+bwd us/iter", "value": round(ms * 1e3, 1), "unit": "us/iter",
                              "n_gpus": world, "steps": steps, "warmup": warmup, "lean": True,
                              "config": {"workload": cname}}), flush=True)
        return None

    e2e_ms = h2d = d2h = None
    clocks = None
    if not extra:
        # ---- end to end through the public API with host buffers.  Every step copies its inputs from pinned host
        # memory and returns out / dx to pinned host memory; the copies run on their own streams (inputs of step i+1
        # and results of step i-1 move while step i computes, as a data loader would), with two device input buffer
        # sets.
        out_h = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()
        dx_h = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()
        e2e_steps = max(4, min(steps, 8))
        main_s = torch.cuda.current_stream()
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        bufs = [{k: torch.empty_like(d[k]) for k in pin} for _ in range(2)]

        def e2e_run(n):
            in_ready = [torch.cuda.Event() for _ in range(n)]
            used = [torch.cuda.Event() for _ in range(n)]
            for i in range(n + 1):
                if i < n:                                   # inputs of step i -> buffer set i % 2
                    with torch.cuda.stream(s_in):
                        if i >= 2:
                            s_in.wait_event(used[i - 2])    # that buffer set has been consumed
                        for k in pin:
                            bufs[i % 2][k].copy_(pin[k], non_blocking=True)
                        in_ready[i].record(s_in)
                if i >= 1:                                  # step i-1
                    j = i - 1
                    main_s.wait_event(in_ready[j])
                    b = bufs[j % 2]
                    out, dx = step(b["x"], b["dy"], b["idx"], b["scores"])
                    used[j].record(main_s)
                    s_out.wait_event(used[j])
                    with torch.cuda.stream(s_out):
                        out_h.copy_(out, non_blocking=True)
                        dx_h.copy_(dx, non_blocking=True)
                    out.record_stream(s_out)
                    dx.record_stream(s_out)
            main_s.wait_stream(s_out)

        e2e_run(2)
        # three passes of `e2e_steps` steps, the median pass is reported (the host link is shared with other
        # tenants of the machine: single passes moved between 3.2 and 6.5 ms per step from box to box)
        e2e_passes = []
        for _ in range(3):
            barrier()
            e2e_ev0, e2e_ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e2e_ev0.record()
            e2e_run(e2e_steps)
            e2e_ev1.record()
            barrier()
            e2e_passes.append(e2e_ev0.elapsed_time(e2e_ev1) / e2e_steps)
        e2e_ms = sorted(e2e_passes)[1]
        h2d = sum(pin[k].numel() * pin[k].element_size() for k in pin)
        d2h = 2 * T * H * 2
    clocks = sampler.stop()      # sampled over the timed steps (and the end-to-end steps that follow them)

    # ---- per-kernel breakdown with CUDA events on the launching stream (separate pass)
    rec = []
    ops.set_recorder(rec)
    nprof = 3
    for _ in range(nprof):
        step(d["x"], d["dy"], d["idx"], d["scores"])
    torch.cuda.synchronize()
    ops.set_recorder(None)
    agg, order = {}, []
    per = max(1, len(rec) // nprof)
    for i, (name, e0, e1) in enumerate(rec):
        key = f"{name}#{i % per}"
        if key not in agg:
            agg[key] = []
            order.append(key)
        agg[key].append(e0.elapsed_time(e1))
    launches = sum(LAUNCHES.get(k.split("#")[0], 1) for k in order)
    breakdown = {k: round(statistics.median(v) * 1e3, 1) for k, v in agg.items()}

    # max over ranks
    if world > 1:
        t = torch.tensor([ms, e2e_ms if e2e_ms is not None else 0.0], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_max = t.tolist()
        e2e_ms = e2e_max if e2e_ms is not None else None
        n_tok = torch.tensor([float(T)], device=dev, dtype=torch.float64)
        dist.all_reduce(n_tok)
        T_job = int(n_tok.item())
    else:
        T_job = T
    if rank != 0:
        return None

    pk = peaks()
    us = ms * 1e3
    F = 18.0 * T_job * K * H * I
    scaling = "strong" if strong else "weak"
    line = {
        "metric": "MoE fwd+bwd us/iter (FP8 MXFP8 1x32, pre-routed expert compute incl. routing metadata, quant, "
                  "6 GEMMs, combines, wgrad into fp32 main_grad)",
        "value": round(us, 1), "unit": "us/iter", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": False, "scaling": scaling,
        "vs_baseline": round(us / PUBLISHED_US[cname], 4) if (world == 1 and cname in PUBLISHED_US) else None,
        "dtype": "fp8_e4m3 (ue8m0 1x32 scales), f32 accumulate", "data": "synthetic",
        "config": dict(config_keys(cname, cfg, world, T, scaling),
                       **({"ep_return_exchange": {"1": "peer memory, both directions (SONIC_MOE_EP_PEER=1)",
                                                  "fwd": "forward: peer-memory pull fused with the reduction; backward "
                                                         "(dx): nccl all_to_all under the weight gradients",
                                                  "0": "nccl all_to_all"}[os.getenv("SONIC_MOE_EP_PEER", "fwd")],
                           "ep_dispatch": "rows fetched from the sources' mapped memory (pull kernel)"
                           if os.getenv("SONIC_MOE_EP_DISPATCH", "pull") == "pull" else "nccl all_to_all"}
                          if world > 1 else {})),
        "mfu_fp8_of_4.5PF": round(F / (ms * 1e-3) / FP8_PEAK_NOMINAL / world, 4),
        "tflops": round(F / (ms * 1e-3) / 1e12, 1),
        "tokens_per_s": round(T_job / (ms * 1e-3), 1),
        "per_step_ms": [round(v, 3) for v in per_step],
        # the power cap moves the step time inside the timed region: both ends, and time x clock, are reported
        "step_drift": {"first10_median_ms": round(statistics.median(per_step[:10]), 4),
                       "last10_median_ms": round(statistics.median(per_step[-10:]), 4),
                       "ms_x_ghz": round(ms * (clocks.get("sm_mhz") or 0) / 1e3, 4)},
        "clocks": clocks,
        "gpu_launches": launches,
        "kernel_us": breakdown,
    }
    if e2e_ms is not None:
        line["e2e"] = {"value": round(e2e_ms * 1e3, 1), "unit": "us/iter",
                       "passes_us": [round(v * 1e3, 1) for v in e2e_passes] if world == 1 else None,
                       "h2d_bytes_per_step": h2d,
                       "d2h_bytes_per_step": d2h}
    line["roofline"] = _roofline(cname, world, T, K, H, I, order, breakdown, pk)
    if world == 1 and cname in ("C2", "P1") and not extra:
        line["full_layer"] = _full_layer(args, cfg, inp, dev, sonicmoe, ops)
        line["fp8_library_bar"] = fp8_library_bar(cfg, dev)
    if world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_reference(cfg)
    return line


def _roofline(cname, world, T, K, H, I, order, breakdown, pk):
    """The slowest GEMM call of the per-kernel pass: FLOPs / CUDA-event time against the FP8 tensor peak, taken as
    twice the measured bf16 figure.  The per-kernel pass is three steps (~10 ms) right after idle-ish copies, i.e.
    burst clocks: `frac` divides by the BURST peak; the sustained figure is given beside it."""
    gemm_keys = [k for k in order if k.startswith("gemm_")]
    if not gemm_keys:
        return None
    dom = max(gemm_keys, key=lambda k: breakdown[k])
    TKH_I = float(T) * K * H * I          # rows routed to this rank's experts = T*K per rank in both series
    per_gemm_flops, seen = {}, {"gemm_varlen_m": 0, "gemm_wgrad": 0}
    for k in gemm_keys:
        n = k.split("#")[0]
        if n.startswith("gemm_wgrad"):
            n = "gemm_wgrad"
        if k.split("#")[0] == "gemm_wgrad_pair":        # dw1 (4) and dw2 (2) in one launch
            per_gemm_flops[k] = 6 * TKH_I
        elif n == "gemm_gated":
            per_gemm_flops[k] = 4 * TKH_I
        elif n in ("gemm_dgated", "gemm_dgated_fused"):
            per_gemm_flops[k] = 2 * TKH_I
        else:       # gemm_varlen_m: down-proj (2) then dgrad (4); gemm_wgrad: dw2 (2) then dw1 (4)
            per_gemm_flops[k] = (2 if seen[n] == 0 else 4) * TKH_I
            seen[n] += 1
    ach = per_gemm_flops[dom] / (breakdown[dom] * 1e-6) / 1e12
    peak_burst, peak_sus = 2.0 * pk["bf16"], 2.0 * pk["bf16_sustained"]
    traffic = None
    table = ncu_dram_bytes(cname) if world == 1 else None
    if table is not None:
        dn = dom.split("#")[0]
        same = [k for k in gemm_keys if k.split("#")[0] == dn]
        traffic = table.get(f"{dn}#{same.index(dom)}")
        if traffic is None and dn == "gemm_wgrad_pair":
            # the two weight gradients were captured as separate launches; run together they move the same tiles
            parts = [table.get("gemm_wgrad_mn#0"), table.get("gemm_wgrad_mn#1")]
            traffic = sum(parts) if all(p is not None for p in parts) else None
    return {"bound": "tensor", "kernel": dom, "achieved": round(ach, 1), "peak": round(peak_burst, 1),
            "unit": "TFLOP/s", "frac": round(ach / peak_burst, 4),
            "frac_of_sustained_peak": round(ach / peak_sus, 4), "peak_sustained": round(peak_sus, 1),
            "applies": "burst (kernel timed in a 3-step pass, not inside a seconds-long region)",
            "traffic": traffic,
            "traffic_unit": "bytes per launch (ncu dram__bytes_read.sum + dram__bytes_write.sum, "
                            f"profiles/gemm_dram_traffic_{cname.lower()}.json)",
            "peak_source": f"2 x bf16_tflops of MEASURED_PEAKS.json ({pk['source']}); the FP8 tensor rate is taken "
                           "as twice the bf16 rate, see fp8_library_bar for what cuBLASLt reaches on this box"}


def _full_layer(args, cfg, inp, dev, sonicmoe, ops):
    """The same layer through the `MoE` module: router linear, top-k + softmax, the expert compute above, and the
    backward through the scores into the router weight (the region the headline number leaves out, as the
    reference's own benchmark does)."""
    E, K, H, I = cfg["E"], cfg["K"], cfg["H"], cfg["I"]
    moe = sonicmoe.MoE(E, K, H, I, sonicmoe.ActivationType.SWIGLU, add_bias=False, std=0.02).to(dev).to(torch.bfloat16)
    with torch.no_grad():
        moe.c_fc.weight.copy_(inp["w1"])
        moe.c_proj.weight.copy_(inp["w2"])
    moe.c_fc.weight.main_grad = torch.zeros(E, 2 * I, H, dtype=torch.float32, device=dev)
    moe.c_proj.weight.main_grad = torch.zeros(E, I, H, dtype=torch.float32, device=dev)
    x, dy = inp["x"].to(dev), inp["dy"].to(dev)

    def step():
        xg = x.detach().requires_grad_(True)
        out, _ = moe(xg, use_fp8=True)
        out.backward(dy)

    for _ in range(max(3, args.warmup // 2)):
        step()
    torch.cuda.synchronize()
    n = max(3, min(args.steps, 8))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        step()
    e1.record()
    torch.cuda.synchronize()
    ops.check_status(dev)
    return {"value": round(e0.elapsed_time(e1) / n * 1e3, 1), "unit": "us/iter", "steps": n,
            "includes": "router linear + top-k softmax + drouter around the timed region of `value`"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    cname = args.config or "C2"           # same workload as the GPU arm at every N
    cfg = CONFIGS[cname]
    T_job = cfg["T"] * world              # one host runs the whole job's tokens
    cb = cpu_reference(cfg, budget_s=10.0 * max(1, min(args.steps, 6)), T_job=T_job)
    us = cb["value"]
    line = {
        "impl": "reference",
        "metric": "MoE fwd+bwd us/iter (FP8 MXFP8 1x32, pre-routed expert compute incl. routing metadata, quant, "
                  "6 GEMMs, combines, wgrad into fp32 main_grad)",
        "value": round(us, 1), "unit": "us/iter", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(us / 1e3, 3), "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 params, fp32 accumulate (reference CPU path)", "data": "synthetic",
        "config": config_keys(cname, cfg, world, cfg["T"], "weak"),
        "cpu_baseline": cb,
        "e2e": {"value": round(us, 1), "unit": "us/iter", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default=None, choices=list(CONFIGS))
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-extras", action="store_true", help="multi-GPU: skip the strong-scaling C4 / C5 runs")
    ap.add_argument("--lean", action="store_true", help="warm-up and timed steps only (for ncu captures)")
    ap.add_argument("--timeline", default=None, metavar="FILE",
                    help="also write the GPU operations of one step (torch.profiler) to FILE (rank 0)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
