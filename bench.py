#!/usr/bin/env python
"""Block-attention throughput on B200: query tokens/s at 32K tokens of int4 "4c/4" KV per sequence.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config decode|prefill|ragged]

A step is one denoising-step's worth of attention: 20 layers, every sequence's 32-token query block attending its
committed context (packed records) plus its own fresh fp16 K/V, ONE kernel launch per layer (the split-KV merge is
part of the kernel). Workload of the contract line (--config decode) at N=1: 64 independent sequences of 32768
committed tokens, the batched configuration the metric is quoted on; 24.9 GB of records, so every step streams far
more than the L2 holds. With N GPUs each rank holds its own 64 sequences (requests are sharded, no collective on the
step path; one all-gather of the last layer's output after the timed region): weak scaling.

value    = query tokens/s over all ranks with everything resident in HBM, the 20-layer step replayed as a CUDA graph,
           timed with CUDA events on the launch stream, max over ranks.
roofline = the attention kernel: the graph holds nothing but its 20 launches, so its mean launch time is
           ms_per_step / 20 of the SAME timed region (launch gaps included); algorithmic flops per launch / that time
           against the measured bf16 tensor peaks (sustained and burst); the HBM view beside it.
e2e      = the same metric through the host-buffer C-ABI call: every layer's Q / fresh K / fresh V come from pinned
           host memory and its fp16 output goes back to the host inside the timed region (the KV cache is resident, as
           in the reference engine). e2e.act is the same with the int8 activation form as the downloaded output (what
           the reference's call site consumes, engine/engine.cu:432); e2e.copy_only_ms is the time of the same copies
           with no kernel in between (the host link's ceiling for this step).
extras   (N=1 only unless noted): `strong` = 64 sequences IN TOTAL over the N ranks (every N); `sweep` = 64 sequences
           at 128 / 1K / 8K / 16K committed tokens; `reference_kernel` = the reference's own attn_partial +
           attn_combine, compiled for sm_100a, on one layer of the same 64 x 32K workload (one launch pair per sequence
           over 8 streams), when oracle/_ref travelled.
cpu_baseline / --impl reference = the reference's CPU flow for this path (fp32 simulated quantisation + SDPA,
           torch CPU, all host threads this process may use) on a bounded sample: one sequence x one layer per step,
           scaled to the metric.
--config prefill / ragged print their own JSON line (the prefill and the ragged serving workloads): a 16-block prefill pass on 31,744
           committed tokens followed by the commit of the 16 blocks; 256 ragged sequences balanced over the ranks by
           KV bytes.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = "llada2-orin-cuda_b200"
sys.path.insert(0, ROOT)

LAYERS = 20
METRIC = "block-attn query tok/s @32K int4 KV"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="decode", choices=["decode", "prefill", "ragged"])
    ap.add_argument("--nseq", type=int, default=64, help="sequences per GPU (decode), in total (ragged: 256 by default)")
    ap.add_argument("--ctx", type=int, default=32768, help="committed tokens per sequence")
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip strong scaling, context sweep and reference-kernel timing")
    ap.add_argument("--precise", action="store_true", help="time the LLATTN_IO_PRECISE_P path (fp16 P + fp16 remainder) instead of the default")
    ap.add_argument("--dense", action="store_true",
                    help="time the W4.A8 attention-output projection (the consumer of the path) instead; own JSON line")
    return ap.parse_args()


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm=float(d["hbm_gbs"]), tf_burst=float(d["bf16_tflops"]), tf_sustained=float(d["bf16_tflops_sustained"]), src="measured")
    return dict(hbm=6650.0, tf_burst=1590.0, tf_sustained=1400.0, src="fallback")


def ncu_traffic_per_unit():
    """DRAM bytes (read + write) the attention kernel moved per KV unit in the committed ncu capture
    (profiles/attn_tile_kernel_traffic.json); a launch's traffic is this figure times its units."""
    p = os.path.join(ROOT, "profiles", "attn_tile_kernel_traffic.json")
    try:
        d = json.load(open(p))
        return float(d["dram_bytes_read_plus_write"]) / float(d["kv_units"]), os.path.relpath(p, ROOT)
    except (OSError, KeyError, ValueError):
        return None, None


class ClockSampler:
    """SM clock and throttle reasons of one GPU while the timed region runs (read-only queries). NVML in a thread every
    10 ms when the binding is there (the timed region is a fraction of a second), else nvidia-smi every 50 ms."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = ((0x8, "hw_slowdown"), (0x40, "hw_thermal_slowdown"), (0x20, "sw_thermal_slowdown"), (0x4, "sw_power_cap"))

    def __init__(self, index: int, pci_bus_id: str | None = None):
        self.index, self.pci, self.proc, self.lines = index, pci_bus_id, None, []
        self.nvml, self.handle, self.stop_flag, self.samples, self.max_mhz = None, None, False, [], None

    def _nvml_open(self) -> bool:
        try:
            import pynvml
            pynvml.nvmlInit()
            self.handle = (pynvml.nvmlDeviceGetHandleByPciBusId(self.pci.encode()) if self.pci
                           else pynvml.nvmlDeviceGetHandleByIndex(self.index))
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            pynvml.nvmlDeviceGetClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
            self.nvml = pynvml
            return True
        except Exception:
            self.nvml = None
            return False

    def _nvml_loop(self):
        n = self.nvml
        reasons_fn = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(n, "nvmlDeviceGetCurrentClocksThrottleReasons")
        while not self.stop_flag:
            try:
                self.samples.append((float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)), int(reasons_fn(self.handle))))
            except Exception:
                pass
            time.sleep(0.01)

    def start(self):
        if self._nvml_open():
            self.th = threading.Thread(target=self._nvml_loop, daemon=True)
            self.th.start()
            return
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self):
        if self.nvml:
            self.stop_flag = True
            self.th.join(timeout=2)
            sm = [c for c, _ in self.samples]
            bits = 0
            for _, r in self.samples:
                bits |= r
            return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.max_mhz,
                    "reasons": sorted(name for bit, name in self.REASON_BITS if bits & bit), "samples": len(sm), "source": "nvml"}
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi"}


# ------------------------------------------------------------------------------------------------ CPU arm

def host_threads() -> int:
    """Threads this process may use: its CPU affinity, not what a launcher put into OMP_NUM_THREADS (torchrun sets 1)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_sample_seconds(ctx_tokens: int, reps: int):
    """Times the reference's CPU flow on one (sequence, layer) of the workload; returns (seconds each, threads)."""
    import numpy as np
    import torch
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import simquant_torch as sq
    threads = host_threads()
    torch.set_num_threads(threads)
    wl = importlib.import_module(PKG).workload
    nblk = ctx_tokens // 32
    Kc, Vc = wl.context_blocks(nblk, seq=0, layer=0)
    Q, Kf, Vf = wl.query_blocks(1, seq=0, layer=0)
    t = [torch.from_numpy(np.ascontiguousarray(a)) for a in (Q[0], Kf[0], Vf[0], Kc, Vc)]
    sq.block_attention(*t)                       # warm-up (thread pool, allocator)
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        sq.block_attention(*t)
        times.append(time.perf_counter() - t0)
    return times, torch.get_num_threads()


def run_reference(a):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    reps = a.warmup + a.steps
    times, threads = cpu_sample_seconds(a.ctx, reps)
    times = times[a.warmup:]
    sec = sum(times) / len(times)
    # one step here = one (sequence, layer); a query token needs all `layers` of them
    value = 32.0 / (a.layers * sec)
    sample = f"1 sequence x 1 layer at {a.ctx} committed tokens per step (torch CPU fp32 fake-quant + SDPA), scaled by 1/{a.layers} layers"
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "query_tok/s", "n_gpus": a.gpus, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": workload_config(a, 1),
            "cpu_baseline": {"value": value, "unit": "query_tok/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "query_tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def workload_config(a, world):
    return {"workload": f"{a.nseq} sequences/GPU x {a.ctx} committed tokens (int4 4c/4 records) x {a.layers} layers, one 32-token query block each, GQA 16/4, d=128",
            "nseq_per_gpu": a.nseq, "ctx_tokens": a.ctx, "layers": a.layers, "sharding": f"requests over {world} GPU(s), no step-path collective",
            "l2": "inputs larger than L2 (every step streams all layers' records)", "graph": "20-layer step replayed as one CUDA graph"}


# ------------------------------------------------------------------------------------------------ GPU arm: set-up

class Rank:
    def __init__(self):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.pkg = importlib.import_module(PKG)
        self.api = importlib.import_module(PKG + ".api")
        self.api.lib()                               # fails loudly when the CUDA library is missing
        self.wl = self.pkg.workload
        self.stream = torch.cuda.Stream(device=self.dev)
        try:      # NVML numbers GPUs physically; the PCI address names this rank's device whatever CUDA_VISIBLE_DEVICES says
            pr = torch.cuda.get_device_properties(self.local)
            self.pci = "%08X:%02X:%02X.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
        except AttributeError:
            self.pci = None

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, values):
        t = self.torch.tensor(values, device=self.dev, dtype=self.torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(x) for x in t.tolist()]

    def gather(self, value):
        """`value` of every rank, in rank order."""
        t = self.torch.tensor([value], device=self.dev, dtype=self.torch.float64)
        if self.world == 1:
            return [float(value)]
        out = [self.torch.empty_like(t) for _ in range(self.world)]
        self.dist.all_gather(out, t)
        return [float(x.item()) for x in out]

    def finish(self):
        if self.world > 1:
            self.dist.barrier()
            self.dist.destroy_process_group()


def record_pool(R, npool=2048, seed_offset=0):
    """Records of `npool` seeded N(0,1)+outlier blocks, made by the commit kernel: [4][npool][4736]."""
    torch, wl = R.torch, R.wl
    g = torch.Generator(device=R.dev)
    g.manual_seed(wl.BASE_SEED + 1000 * R.rank + seed_offset)
    K = torch.randn((npool, 32, 4, 128), generator=g, device=R.dev, dtype=torch.float32)
    K[..., list(wl.OUTLIER_CHANNELS)] *= wl.OUTLIER_GAIN
    K = K.half()
    V = torch.randn((npool, 32, 4, 128), generator=g, device=R.dev, dtype=torch.float32).half()
    pool = torch.zeros((4, npool, 4736), dtype=torch.uint8, device=R.dev)
    R.api.kv_commit(K, V, pool, npool, 0)
    torch.cuda.synchronize()
    return pool, g


def build_caches(R, lens, layers, spare=1):
    """One flat buffer per layer holding every sequence's cache [4][len + spare][4736] back to back, all layers laid
    out alike (so one plan plus a per-layer byte offset serves the whole step). Each cache is a seeded random draw (with
    repetition) from a pool of committed records: values have the workload's distribution, all memory is distinct, and
    generation runs at memory-copy speed. Returns (buffer [layers][bytes], list of (byte offset, max_blocks))."""
    torch = R.torch
    pool, g = record_pool(R)
    npool = pool.shape[1]
    offs, total = [], 0
    for n in lens:
        offs.append((total, n + spare))
        total += 4 * (n + spare) * 4736
    total = (total + 255) // 256 * 256
    buf = torch.empty((layers, total), dtype=torch.uint8, device=R.dev)
    for l in range(layers):
        for (off, maxb), n in zip(offs, lens):
            if n == 0:
                continue
            view = buf[l, off:off + 4 * maxb * 4736].view(4, maxb, 4736)
            idx = torch.randint(0, npool, (n,), generator=g, device=R.dev)
            for h in range(4):
                view[h, :n] = pool[h].index_select(0, idx)
    torch.cuda.synchronize()
    return buf, offs


def fresh_inputs(R, layers, nq_total, seed=99):
    torch, wl = R.torch, R.wl
    g = torch.Generator(device=R.dev)
    g.manual_seed(seed + R.rank)
    Q = torch.randn((layers, nq_total, 32, 16, 128), generator=g, device=R.dev, dtype=torch.float32).half()
    Kf = torch.randn((layers, nq_total, 32, 4, 128), generator=g, device=R.dev, dtype=torch.float32)
    Kf[..., list(wl.OUTLIER_CHANNELS)] *= wl.OUTLIER_GAIN
    Kf = Kf.half()
    Vf = torch.randn((layers, nq_total, 32, 4, 128), generator=g, device=R.dev, dtype=torch.float32).half()
    return Q, Kf, Vf


def seq_list(R, buf, offs, lens, nq=None, which=None):
    """api.Seq descriptors on layer 0's caches for the sequences `which` (default all), query blocks numbered in order."""
    out, q0 = [], 0
    for i in (range(len(lens)) if which is None else which):
        off, maxb = offs[i]
        k = 1 if nq is None else nq[i]
        out.append(R.api.Seq(cache=buf[0, off:off + 4 * maxb * 4736].view(4, maxb, 4736), nblocks=lens[i], nq=k, q_first=q0))
        q0 += k
    return out


class Step:
    """A 20-layer attention step over one plan, eager or as a CUDA graph, with timing on the launch stream."""

    def __init__(self, R, ctx, plan, layer_bytes, Q, Kf, Vf, O, graph=True, precise=False, extra=None):
        self.R, self.ctx, self.plan = R, ctx, plan
        self.args = (layer_bytes, Q, Kf, Vf, O, precise)
        self.extra = extra                          # optional callable(stream) run after the layers inside the step
        self.graph = None
        torch = R.torch
        with torch.cuda.stream(R.stream):
            self.eager()
            R.stream.synchronize()
            assert ctx.device_status(R.stream) == 0
            if graph:
                self.graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self.graph, stream=R.stream):
                    self.eager()

    def eager(self):
        layer_bytes, Q, Kf, Vf, O, precise = self.args
        for l in range(Q.shape[0]):
            self.ctx.attention(self.plan, Q[l], Kf[l], Vf[l], O16=O[l], stream=self.R.stream, precise=precise, cache_offset=l * layer_bytes)
        if self.extra:
            self.extra(self.R.stream)

    def run(self):
        if self.graph is not None:
            self.graph.replay()
        else:
            self.eager()

    def timed(self, steps, warmup, sampler=None):
        """W warm-up steps, barrier, K timed steps between CUDA events, barrier. Returns ms for the K steps."""
        R, torch = self.R, self.R.torch
        with torch.cuda.stream(R.stream):
            for _ in range(max(warmup, 3)):
                self.run()
        R.barrier()
        if sampler:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(R.stream):
            e0.record(R.stream)
            for _ in range(steps):
                self.run()
            e1.record(R.stream)
        R.barrier()
        return e0.elapsed_time(e1)


def bind_to_nvml_cpu_set(R, node):
    """The CPUs NVML names as closest to this rank's GPU (nvmlDeviceGetCpuAffinity), if that is a proper subset of
    the CPUs this process may use."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByPciBusId(R.pci.encode() if isinstance(R.pci, str) else R.pci)
        ncpu = max(os.sched_getaffinity(0)) + 1
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (ncpu + 63) // 64)
        cpus = {64 * i + b for i, w in enumerate(words) for b in range(64) if (int(w) >> b) & 1}
        mine = set(os.sched_getaffinity(0))
        allowed = cpus & mine
        if not allowed or allowed == mine:
            return {"numa_node": node, "bound": False, "nvml_cpus": len(cpus)}
        os.sched_setaffinity(0, allowed)
        return {"numa_node": node, "bound": True, "cpus": len(allowed), "source": "nvml cpu affinity"}
    except Exception as e:                             # noqa: BLE001 - best effort, reported
        return {"numa_node": node, "bound": False, "nvml": type(e).__name__}


def bind_to_gpu_numa_node(R):
    """Best effort: run this rank's host threads on the CPUs of its GPU's NUMA node before pinned buffers are allocated
    (first touch then places them there). Returns what was done, for the JSON line."""
    if not R.pci:
        return None
    try:
        dom, rest = R.pci.split(":", 1)
        node = int(open(f"/sys/bus/pci/devices/{dom[-4:].lower()}:{rest.lower()}/numa_node").read())
        if node < 0:                                   # no topology in sysfs (virtualised): ask the driver for the GPU's CPUs
            return bind_to_nvml_cpu_set(R, node)
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & set(os.sched_getaffinity(0))
        if not allowed:
            return {"numa_node": node, "bound": False}
        os.sched_setaffinity(0, allowed)
        return {"numa_node": node, "bound": True, "cpus": len(allowed)}
    except (OSError, ValueError):
        return None


# ------------------------------------------------------------------------------------------------ GPU arm: decode (the contract line)

def run_decode(a):
    R = Rank()
    torch, api, wl = R.torch, R.api, R.wl
    nblk, nseq, L = a.ctx // 32, a.nseq, a.layers
    pk = peaks()
    lens = [nblk] * nseq
    buf, offs = build_caches(R, lens, L)
    layer_bytes = buf.shape[1]
    ctx = api.Context(R.local)
    plan = ctx.plan(seq_list(R, buf, offs, lens))
    st = plan.stats
    Q, Kf, Vf = fresh_inputs(R, L, nseq)
    O = torch.zeros((L, nseq * 32, 16, 128), dtype=torch.float16, device=R.dev)
    step = Step(R, ctx, plan, layer_bytes, Q, Kf, Vf, O, graph=not a.no_graph, precise=a.precise)

    sampler = ClockSampler(R.local, R.pci) if R.rank == 0 else None
    ms = step.timed(a.steps, a.warmup, sampler)
    clocks = sampler.stop() if sampler else None
    assert ctx.device_status(R.stream) == 0

    # ---- end to end: host buffers per layer through the host-buffer entry point
    e2e = {}
    if not a.no_e2e:
        numa = bind_to_gpu_numa_node(R)
        hQ, hK, hV = Q.cpu().pin_memory(), Kf.cpu().pin_memory(), Vf.cpu().pin_memory()
        hO = torch.zeros((L, nseq * 32, 16, 128), dtype=torch.float16).pin_memory()
        hq8 = torch.zeros((L, nseq * 32, 2048), dtype=torch.int8).pin_memory()
        hs8 = torch.zeros((L, nseq * 32, 16), dtype=torch.float32).pin_memory()
        hsum = torch.zeros((L, nseq * 32, 16), dtype=torch.int32).pin_memory()
        h2d = L * (hQ[0].numel() + hK[0].numel() + hV[0].numel()) * 2
        d2h = L * hO[0].numel() * 2
        d2h_act = L * (hq8[0].numel() + hs8[0].numel() * 4 + hsum[0].numel() * 4)

        def step_host(act):
            for l in range(L):
                if act:
                    ctx.attention_host(plan, hQ[l], hK[l], hV[l], q8=hq8[l], s8=hs8[l], sum8=hsum[l], stream=R.stream,
                                       precise=a.precise, cache_offset=l * layer_bytes)
                else:
                    ctx.attention_host(plan, hQ[l], hK[l], hV[l], O16=hO[l], stream=R.stream, precise=a.precise, cache_offset=l * layer_bytes)
            ctx.host_flush(R.stream)

        dQ, dK, dV, dO = torch.empty_like(Q[0]), torch.empty_like(Kf[0]), torch.empty_like(Vf[0]), torch.empty_like(O[0])
        s_up, s_dn = torch.cuda.Stream(device=R.dev), torch.cuda.Stream(device=R.dev)

        def step_copies():      # the step's copies alone: uploads and downloads on their own streams, no kernel
            for l in range(L):
                with torch.cuda.stream(s_up):
                    dQ.copy_(hQ[l], non_blocking=True); dK.copy_(hK[l], non_blocking=True); dV.copy_(hV[l], non_blocking=True)
                with torch.cuda.stream(s_dn):
                    hO[l].copy_(dO, non_blocking=True)
            R.stream.wait_stream(s_up); R.stream.wait_stream(s_dn)

        n_e2e = max(2, a.steps // 2)

        def timed_host(fn):
            with torch.cuda.stream(R.stream):
                fn()
            R.barrier()
            t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(R.stream):
                s_up.wait_stream(R.stream); s_dn.wait_stream(R.stream)
                t0.record(R.stream)
                for _ in range(n_e2e):
                    fn()
                t1.record(R.stream)
            R.barrier()
            return t0.elapsed_time(t1) / n_e2e

        e2e_ms = timed_host(lambda: step_host(False))
        assert torch.equal(hO[L - 1].to(R.dev), O[L - 1]), "host-buffer path and resident path disagree"
        act_ms = timed_host(lambda: step_host(True))
        copy_ms = timed_host(step_copies)
        e2e = dict(e2e_ms=e2e_ms, act_ms=act_ms, copy_ms=copy_ms, h2d=h2d, d2h=d2h, d2h_act=d2h_act, numa=numa)
        del hQ, hK, hV, hO, hq8, hs8, hsum

    # ---- strong scaling: the same 64 sequences IN TOTAL, shared out over the ranks
    strong = None
    if not a.no_extras and nseq % R.world == 0:
        mine = nseq // R.world
        plan_s = ctx.plan(seq_list(R, buf, offs, lens, which=range(mine)))
        step_s = Step(R, ctx, plan_s, layer_bytes, Q[:, :mine], Kf[:, :mine], Vf[:, :mine], O[:, :mine * 32], graph=not a.no_graph, precise=a.precise)
        ms_s = R.max_over_ranks([step_s.timed(a.steps, a.warmup)])[0] / a.steps
        strong = {"sequences_total": nseq, "sequences_per_gpu": mine, "ms_per_step": ms_s, "value": nseq * 32 / (ms_s * 1e-3),
                  "unit": "query_tok/s", "scaling": "strong"}
        plan_s.close()

    # ---- shorter contexts on the same caches (N = 1)
    sweep = None
    if not a.no_extras and R.world == 1:
        sweep = []
        for tokens in (128, 1024, 8192, 16384):
            if tokens >= a.ctx:
                continue
            nb = tokens // 32
            plan_c = ctx.plan(seq_list(R, buf, offs, [nb] * nseq))
            step_c = Step(R, ctx, plan_c, layer_bytes, Q, Kf, Vf, O, graph=not a.no_graph, precise=a.precise)
            ms_c = step_c.timed(2 * a.steps, a.warmup) / (2 * a.steps)
            fl = nseq * wl.algorithmic_flops(nb) * L
            by = nseq * wl.algorithmic_bytes(nb) * L
            t_roof = max(fl / (pk["tf_sustained"] * 1e12), by / (pk["hbm"] * 1e9))
            sweep.append({"ctx_tokens": tokens, "ms_per_step": ms_c, "value": nseq * 32 / (ms_c * 1e-3), "frac_of_slower_roofline": t_roof / (ms_c * 1e-3)})
            plan_c.close()

    # ---- the reference's own kernels on one layer of this workload (N = 1, when they travelled)
    refk = None
    if not a.no_extras and R.world == 1:
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        try:
            import refkernel
            if refkernel.available():
                caches0 = buf[0, :nseq * 4 * (nblk + 1) * 4736].view(nseq, 4, nblk + 1, 4736)
                runner = refkernel.BatchRunner(nseq, nblk, R.dev)
                for _ in range(3):
                    runner.launch(Q[0], Kf[0], Vf[0], caches0, nblk + 1)
                torch.cuda.synchronize()
                ts = []
                for _ in range(max(3, a.steps // 2)):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    cur = torch.cuda.current_stream()
                    e0.record(cur)
                    for s_ in runner.streams:
                        s_.wait_event(e0)
                    runner.launch(Q[0], Kf[0], Vf[0], caches0, nblk + 1)
                    for s_ in runner.streams:
                        cur.wait_stream(s_)
                    e1.record(cur)
                    torch.cuda.synchronize()
                    ts.append(e0.elapsed_time(e1))
                ref_ms = statistics.median(ts)
                with torch.cuda.stream(R.stream):        # layer 0 again with the full-length plan (the sweep reused O)
                    ctx.attention(plan, Q[0], Kf[0], Vf[0], O16=O[0], stream=R.stream, precise=a.precise)
                R.stream.synchronize()
                got = O[0].float()
                ref = runner.O.float()
                rel = float(((got - ref).norm() / ref.norm()).item())
                refk = {"ms_per_layer": ref_ms, "launch_pairs": nseq, "streams": len(runner.streams), "chunks_per_head": runner.nch,
                        "ctas": 4 * runner.nch * nseq, "rel_l2_vs_ours": rel}
            else:
                refk = {"unavailable": "oracle/_ref/libattn_ref.so is not built on this machine"}
        except Exception as e:  # noqa: BLE001
            refk = {"unavailable": f"{type(e).__name__}: {e}"}

    # ---- max over ranks, final output gather (outside every timed region)
    vals = R.max_over_ranks([ms] + ([e2e["e2e_ms"], e2e["act_ms"], e2e["copy_ms"]] if e2e else [0.0, 0.0, 0.0]))
    ms, e2e_ms, act_ms, copy_ms = vals
    if R.world > 1:
        gathered = [torch.empty_like(O[L - 1]) for _ in range(R.world)]
        R.dist.all_gather(gathered, O[L - 1])

    if R.rank == 0:
        tokens_step = R.world * nseq * 32
        ms_step = ms / a.steps
        launch_ms = ms_step / L
        value = tokens_step / (ms_step * 1e-3)
        flops_launch = nseq * wl.algorithmic_flops(nblk)
        bytes_launch = nseq * wl.algorithmic_bytes(nblk)
        ach_tf = flops_launch / (launch_ms * 1e-3) / 1e12
        ach_gbs = bytes_launch / (launch_ms * 1e-3) / 1e9
        t_tensor = flops_launch / (pk["tf_sustained"] * 1e12)
        t_hbm = bytes_launch / (pk["hbm"] * 1e9)
        per_unit, traffic_src = ncu_traffic_per_unit()
        line = {
            "metric": METRIC, "value": value, "unit": "query_tok/s", "n_gpus": R.world, "steps": a.steps, "warmup": max(a.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic", "config": workload_config(a, R.world),
            "roofline": {"bound": "tensor", "achieved": ach_tf, "peak": pk["tf_sustained"], "unit": "TFLOP/s",
                         "frac": ach_tf / pk["tf_sustained"], "frac_burst": ach_tf / pk["tf_burst"], "peak_burst": pk["tf_burst"],
                         "traffic": per_unit * st.total_units if per_unit else None,
                         "traffic_note": ("ncu dram read+write per KV unit from %s x the launch's units; algorithmic bytes per launch = %d" % (traffic_src, bytes_launch)) if per_unit else "no ncu capture on file",
                         "kernel": "attn_tile_kernel", "ms_per_launch": launch_ms,
                         "ms_per_launch_note": "ms_per_step / layers: the timed graph holds only this kernel's launches",
                         "peak_source": pk["src"] + " bf16 (frac: sustained, frac_burst: burst)",
                         "hbm_achieved_gbs": ach_gbs, "hbm_peak_gbs": pk["hbm"], "hbm_frac": ach_gbs / pk["hbm"],
                         "slower_bound": "tensor" if t_tensor >= t_hbm else "hbm"},
            "gpu_launches": a.steps * L,
            "plan": {"ctas": st.nctas, "runs": st.nitems, "total_units": st.total_units, "max_cta_units": st.max_cta_units},
            "clocks": clocks,
        }
        if a.precise:
            line["config"]["p_precision"] = "fp16 value + fp16 remainder (LLATTN_IO_PRECISE_P)"
        if e2e:
            line["e2e"] = {"value": tokens_step / (e2e_ms * 1e-3), "unit": "query_tok/s", "h2d_bytes_per_step": e2e["h2d"],
                           "d2h_bytes_per_step": e2e["d2h"], "ms_per_step": e2e_ms, "copy_only_ms": copy_ms,
                           "act": {"value": tokens_step / (act_ms * 1e-3), "ms_per_step": act_ms, "d2h_bytes_per_step": e2e["d2h_act"],
                                   "note": "int8 activation form downloaded instead of fp16 O (engine/engine.cu:432 consumes that form)"},
                           "numa": e2e["numa"]}
        if strong:
            line["strong"] = strong
        if sweep:
            line["sweep"] = sweep
        if refk:
            if "ms_per_layer" in refk:
                refk["ours_ms_per_layer"] = launch_ms
                refk["speedup"] = refk["ms_per_layer"] / launch_ms
            line["reference_kernel"] = refk
        if not a.no_cpu_baseline and R.world == 1:        # a reported baseline of the N = 1 line only (other ranks would be spinning beside it)
            times, threads = cpu_sample_seconds(a.ctx, 3)
            sec = min(times)
            line["cpu_baseline"] = {"value": 32.0 / (L * sec), "unit": "query_tok/s", "cores": threads, "kind": "port",
                                    "sample": f"1 sequence x 1 layer at {a.ctx} tokens (torch CPU fp32 fake-quant + SDPA, best of 3), scaled by 1/{L} layers"}
        print(json.dumps(line), flush=True)
    R.finish()


# ------------------------------------------------------------------------------------------------ prefill pass

def run_prefill(a):
    """A 16-block prefill pass: 512 query tokens appended to 31,744 committed tokens, per layer the commit of the 16 new
    blocks and then block-causal attention (the reference's order, engine/engine.cu:589-599), 20 layers."""
    R = Rank()
    torch, api, wl = R.torch, R.api, R.wl
    L, nq = a.layers, 16
    ctx0 = (a.ctx // 32) - nq - 16 if a.ctx == 32768 else a.ctx // 32          # 992 blocks = 31,744 tokens by default
    pk = peaks()
    buf, offs = build_caches(R, [ctx0], L, spare=nq)
    layer_bytes = buf.shape[1]
    maxb = offs[0][1]
    ctx = api.Context(R.local)
    plan = ctx.plan(seq_list(R, buf, offs, [ctx0], nq=[nq]))
    st = plan.stats
    Q, Kf, Vf = fresh_inputs(R, L, nq)
    O = torch.zeros((L, nq * 32, 16, 128), dtype=torch.float16, device=R.dev)
    cache_l = [buf[l, :4 * maxb * 4736].view(4, maxb, 4736) for l in range(L)]

    class PrefillStep(Step):
        def eager(self):
            for l in range(L):
                api.kv_commit(Kf[l], Vf[l], cache_l[l], maxb, ctx0, stream=R.stream)
                ctx.attention(plan, Q[l], Kf[l], Vf[l], O16=O[l], stream=R.stream, precise=a.precise, cache_offset=l * layer_bytes)

    step = PrefillStep(R, ctx, plan, layer_bytes, Q, Kf, Vf, O, graph=not a.no_graph, precise=a.precise)
    sampler = ClockSampler(R.local, R.pci) if R.rank == 0 else None
    ms = R.max_over_ranks([step.timed(a.steps, a.warmup, sampler)])[0]
    clocks = sampler.stop() if sampler else None
    assert ctx.device_status(R.stream) == 0
    # commit-only time, for the share it has in the step
    with torch.cuda.stream(R.stream):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(R.stream)
        for _ in range(a.steps):
            for l in range(L):
                api.kv_commit(Kf[l], Vf[l], cache_l[l], maxb, ctx0, stream=R.stream)
        e1.record(R.stream)
    R.barrier()
    commit_ms = e0.elapsed_time(e1) / a.steps
    if R.rank == 0:
        ms_step = ms / a.steps
        flops = sum(wl.algorithmic_flops(ctx0 + j) for j in range(nq)) * L
        # records of the context are read once per query block by the kernel's design; algorithmically once per pass
        bytes_alg = (wl.algorithmic_bytes(ctx0 + nq - 1) + (nq - 1) * (131072 + 65536 + 131072)) * L + nq * (65536 + 18944) * L
        ach_tf = flops / (ms_step * 1e-3) / 1e12
        line = {"metric": "prefill tok/s: 16 blocks on 31,744 committed int4 KV tokens, attention + commit", "value": R.world * nq * 32 / (ms_step * 1e-3),
                "unit": "tok/s", "n_gpus": R.world, "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": ms_step,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                "config": {"workload": f"1 sequence/GPU, {nq} query blocks appended to {ctx0 * 32} committed tokens, {L} layers: commit of the {nq} blocks, then block-causal attention",
                           "l2": "388 MB of records per pass, larger than L2", "graph": "whole pass replayed as one CUDA graph"},
                "roofline": {"bound": "tensor", "achieved": ach_tf, "peak": pk["tf_sustained"], "unit": "TFLOP/s", "frac": ach_tf / pk["tf_sustained"],
                             "frac_burst": ach_tf / pk["tf_burst"], "traffic": None, "kernel": "attn_tile_kernel",
                             "hbm_achieved_gbs": bytes_alg / (ms_step * 1e-3) / 1e9, "hbm_peak_gbs": pk["hbm"],
                             "note": "whole pass (commit included) against the tensor roofline of its attention flops"},
                "commit": {"ms_per_step": commit_ms, "share_of_step": commit_ms / ms_step, "bytes_read": nq * 65536 * L, "bytes_written": nq * 18944 * L},
                "gpu_launches": a.steps * L * 2, "plan": {"ctas": st.nctas, "runs": st.nitems, "total_units": st.total_units, "max_cta_units": st.max_cta_units},
                "clocks": clocks}
        print(json.dumps(line), flush=True)
    R.finish()


# ------------------------------------------------------------------------------------------------ ragged serving batch

def run_ragged(a):
    """256 sequences with committed lengths uniform over the multiples of 32 in [128, 32768] tokens, one query block each,
    20 layers; sequences are dealt to the ranks by longest-processing-time on KV units (sharding.shard_lpt)."""
    R = Rank()
    torch, api, wl = R.torch, R.api, R.wl
    sharding = R.pkg.sharding
    L = a.layers
    nseq = 256 if a.nseq == 64 else a.nseq
    lens_all = [int(x) for x in wl.ragged_lengths(nseq, seed=wl.BASE_SEED)]
    shards = sharding.shard_lpt(lens_all, R.world)
    mine = shards[R.rank]
    lens = [lens_all[i] for i in mine]
    pk = peaks()
    buf, offs = build_caches(R, lens, L)
    layer_bytes = buf.shape[1]
    ctx = api.Context(R.local)
    plan = ctx.plan(seq_list(R, buf, offs, lens))
    st = plan.stats
    Q, Kf, Vf = fresh_inputs(R, L, len(lens))
    O = torch.zeros((L, len(lens) * 32, 16, 128), dtype=torch.float16, device=R.dev)
    step = Step(R, ctx, plan, layer_bytes, Q, Kf, Vf, O, graph=not a.no_graph, precise=a.precise)
    sampler = ClockSampler(R.local, R.pci) if R.rank == 0 else None
    ms_mine = step.timed(a.steps, a.warmup, sampler)
    ms = R.max_over_ranks([ms_mine])[0]
    ms_ranks = [x / a.steps for x in R.gather(ms_mine)]
    units_ranks = R.gather(st.total_units)
    clocks = sampler.stop() if sampler else None
    assert ctx.device_status(R.stream) == 0
    if R.rank == 0:
        ms_step = ms / a.steps
        kv_bytes = [sum(4 * 4736 * lens_all[i] for i in s) * L for s in shards]
        flops_rank = [sum(wl.algorithmic_flops(lens_all[i]) for i in s) * L for s in shards]
        bytes_rank = [sum(wl.algorithmic_bytes(lens_all[i]) for i in s) * L for s in shards]
        ach_tf = max(flops_rank) / (ms_step * 1e-3) / 1e12
        line = {"metric": "ragged batch query tok/s: 256 sequences, 128..32768 committed int4 KV tokens", "value": nseq * 32 / (ms_step * 1e-3),
                "unit": "query_tok/s", "n_gpus": R.world, "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": ms_step,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                "config": {"workload": f"{nseq} sequences in total, lengths uniform over multiples of 32 in [128, 32768] tokens (seeded), one 32-token query block each, {L} layers",
                           "sharding": f"longest-processing-time on KV units over {R.world} GPU(s), no step-path collective",
                           "l2": "inputs larger than L2", "graph": "20-layer step replayed as one CUDA graph"},
                "balance": {"kv_bytes_per_gpu_max": max(kv_bytes), "kv_bytes_per_gpu_mean": sum(kv_bytes) / len(kv_bytes),
                            "max_over_mean": max(kv_bytes) / (sum(kv_bytes) / len(kv_bytes)), "sequences_per_gpu": [len(s) for s in shards],
                            "cta_max_over_mean_units_rank0": st.max_cta_units / (st.total_units / st.nctas),
                            "ms_per_step_per_gpu": ms_ranks, "kv_units_per_gpu": units_ranks},
                "roofline": {"bound": "tensor", "achieved": ach_tf, "peak": pk["tf_sustained"], "unit": "TFLOP/s", "frac": ach_tf / pk["tf_sustained"],
                             "frac_burst": ach_tf / pk["tf_burst"], "traffic": None, "kernel": "attn_tile_kernel",
                             "hbm_achieved_gbs": max(bytes_rank) / (ms_step * 1e-3) / 1e9, "hbm_peak_gbs": pk["hbm"],
                             "note": "busiest rank's flops over the step time (max over ranks)"},
                "gpu_launches": a.steps * L, "plan": {"ctas": st.nctas, "runs": st.nitems, "total_units": st.total_units, "max_cta_units": st.max_cta_units},
                "clocks": clocks}
        print(json.dumps(line), flush=True)
    R.finish()


# ------------------------------------------------------------------------------------------------ dense projection (side measurement)

def run_dense(a):
    """Side measurement, not the contract line: the 2048 x 2048 W4.A8 projection that consumes the attention output, on
    the tokens of one step (--nseq x 32), device-resident inputs, CUDA events, a buffer larger than L2 written between
    launches. Also times the reference's own GEMM when its library travelled (oracle/_ref/libgemm_ref.so)."""
    import numpy as np
    import torch
    api = importlib.import_module(PKG + ".api")
    wl = importlib.import_module(PKG).workload
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    rows = K = 2048
    ntok = a.nseq * 32
    strips, _, _, _ = wl.dense_weights(rows, K, 1)
    q, s, qsum = wl.int8_activations(ntok, K, 2)
    d = [torch.from_numpy(x).to(dev) for x in (strips, q, s, qsum)]
    Y = torch.zeros((ntok, rows), dtype=torch.float32, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)

    def timed(fn):
        for _ in range(max(a.warmup, 3)):
            fn()
        ts = []
        for _ in range(a.steps):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts)

    ms = timed(lambda: api.dense_w4a8(d[0], d[1], d[2], d[3], Y, err_word=err))
    assert int(err.item()) == 0
    pk = peaks()
    ktot = K // 128
    bytes_alg = strips.size + ntok * K + 2 * 4 * ntok * ktot + 2 * 4 * ntok * rows      # weights, int8 acts, scales+sums, Y read+write
    ops = 2.0 * ntok * rows * K
    out = {"metric": "W4.A8 attention-output projection tokens/s", "value": ntok / (ms * 1e-3), "unit": "tok/s", "n_gpus": 1,
           "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "dtype": "u8 x s8 -> s32, fp32 scale chain",
           "data": "synthetic", "config": {"workload": f"{ntok} tokens x (2048 x 2048, 4-bit weights, int8 activations), Y += W x", "l2": "256 MB written between launches"},
           "roofline": {"bound": "hbm", "achieved": bytes_alg / (ms * 1e-3) / 1e9, "peak": pk["hbm"], "unit": "GB/s",
                        "frac": bytes_alg / (ms * 1e-3) / 1e9 / pk["hbm"], "traffic": None, "algorithmic_bytes": bytes_alg,
                        "int8_tops": ops / (ms * 1e-3) / 1e12, "peak_source": pk["src"]},
           "gpu_launches": a.steps}
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    try:
        import refkernel
        if refkernel.gemm_available() and ntok % 32 == 0:
            aux = refkernel.dense_aux(ntok, dev)
            out["reference_kernel_ms"] = timed(lambda: refkernel.dense_w4a8(d[0], d[1], d[2], d[3], Y, aux=aux, sync=False))
    except Exception as e:  # noqa: BLE001
        out["reference_kernel_ms"] = f"unavailable: {e}"
    print(json.dumps(out))


if __name__ == "__main__":
    # Libraries (NCCL's version banner, torchrun notices) may write to stdout; the contract is ONE JSON line there. Everything
    # written to fd 1 from here on goes to stderr, and the JSON line is written to the saved stdout.
    _real_stdout = os.fdopen(os.dup(1), "w")
    sys.stdout.flush()
    os.dup2(2, 1)
    _print = print

    def print(*a, **k):  # noqa: A001  (only the JSON lines use print in this file)
        k.pop("flush", None)
        _print(*a, file=_real_stdout, **k)
        _real_stdout.flush()

    args = parse()
    if args.dense:
        run_dense(args)
    elif args.impl == "reference":
        run_reference(args)
    elif args.config == "prefill":
        run_prefill(args)
    elif args.config == "ragged":
        run_ragged(args)
    else:
        run_decode(args)
