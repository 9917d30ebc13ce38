#!/usr/bin/env python
"""Block-attention throughput on B200: query tokens/s at 32K tokens of int4 "4c/4" KV per sequence.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--nseq 64] [--ctx 32768]

A step is one denoising-step's worth of attention: 20 layers, every sequence's 32-token query block attending its
committed context (packed records) plus its own fresh fp16 K/V. Workload at N=1: 64 independent sequences of
32768 committed tokens (the batched configuration the metric is quoted on; 24.9 GB of records, so every step
streams far more than the L2 holds). With N GPUs each rank holds its own 64 sequences (requests are sharded, no
collective on the step path; one all-gather of the last layer's output after the timed region).

value  = query tokens/s over all ranks with everything resident in HBM, 20-layer step replayed as a CUDA graph,
         timed with CUDA events on the launch stream, max over ranks.
e2e    = same metric through the host-buffer C-ABI call: every layer's Q / fresh K / fresh V come from pinned host
         memory and its fp16 output goes back to the host inside the timed region (the KV cache is resident, as
         in the reference engine).
roofline = the tile kernel's algorithmic flops per launch / its mean launch time (CUDA events around that kernel
         alone) against the measured bf16 tensor peak; the HBM view is reported beside it.
cpu_baseline / --impl reference = the reference's CPU flow for this path (fp32 simulated quantisation + SDPA,
         torch CPU, all host threads) on a bounded sample: one sequence x one layer per step, scaled to the metric.
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
# DRAM bytes (read + write) the tile kernel moved per KV unit (one 4736-byte record, or the fresh block) in an ncu capture
# of a 32-sequence, 1-layer launch: 643.3 MB over 131,200 units. Traffic grows in proportion to the units a launch
# processes, so a launch's traffic is this figure times its units.
NCU_TRAFFIC_BYTES_PER_UNIT = 643.3e6 / 131200


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--nseq", type=int, default=64, help="sequences per GPU")
    ap.add_argument("--ctx", type=int, default=32768, help="committed tokens per sequence")
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
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

def cpu_sample_seconds(ctx_tokens: int, reps: int):
    """Times the reference's CPU flow on one (sequence, layer) of the workload; returns (seconds each, threads)."""
    import numpy as np
    import torch
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import simquant_torch as sq
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


# ------------------------------------------------------------------------------------------------ GPU arm

def build_caches(torch, api, wl, nseq, nblk, layers, dev, rank):
    """Per (layer, sequence) record caches [4][nblk+1][4736], all distinct memory. Records come from the commit kernel
    run on a pool of seeded N(0,1)+outlier blocks; each cache is a seeded random draw (with repetition) from the
    pool, so values have the workload's distribution while generation stays at memory-copy speed."""
    import numpy as np
    POOL = 2048
    g = torch.Generator(device=dev)
    g.manual_seed(wl.BASE_SEED + 1000 * rank)
    K = torch.randn((POOL, 32, 4, 128), generator=g, device=dev, dtype=torch.float32)
    K[..., list(wl.OUTLIER_CHANNELS)] *= wl.OUTLIER_GAIN
    K = K.half()
    V = torch.randn((POOL, 32, 4, 128), generator=g, device=dev, dtype=torch.float32).half()
    pool = torch.zeros((4, POOL, 4736), dtype=torch.uint8, device=dev)
    api.kv_commit(K, V, pool, POOL, 0)
    torch.cuda.synchronize()
    del K, V
    maxb = nblk + 1
    caches = torch.empty((layers, nseq, 4, maxb, 4736), dtype=torch.uint8, device=dev)
    for l in range(layers):
        for s in range(nseq):
            idx = torch.randint(0, POOL, (nblk,), generator=g, device=dev)
            for h in range(4):
                caches[l, s, h, :nblk] = pool[h].index_select(0, idx)
    torch.cuda.synchronize()
    return caches, maxb


def run_ours(a):
    import numpy as np
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    pkg = importlib.import_module(PKG)
    api = importlib.import_module(PKG + ".api")
    api.lib()                                        # fails loudly when the CUDA library is missing
    wl = pkg.workload
    nblk, nseq, L = a.ctx // 32, a.nseq, a.layers
    pk = peaks()

    caches, maxb = build_caches(torch, api, wl, nseq, nblk, L, dev, rank)
    ctx = api.Context(local)
    plans = [ctx.plan([api.Seq(cache=caches[l, s], nblocks=nblk, nq=1, q_first=s) for s in range(nseq)]) for l in range(L)]
    st = plans[0].stats
    g = torch.Generator(device=dev)
    g.manual_seed(99 + rank)
    Q = torch.randn((L, nseq, 32, 16, 128), generator=g, device=dev, dtype=torch.float32).half()
    Kf = torch.randn((L, nseq, 32, 4, 128), generator=g, device=dev, dtype=torch.float32)
    Kf[..., list(wl.OUTLIER_CHANNELS)] *= wl.OUTLIER_GAIN
    Kf = Kf.half()
    Vf = torch.randn((L, nseq, 32, 4, 128), generator=g, device=dev, dtype=torch.float32).half()
    O = torch.zeros((L, nseq * 32, 16, 128), dtype=torch.float16, device=dev)
    stream = torch.cuda.Stream(device=dev)

    def step(parts=3):
        for l in range(L):
            ctx.attention(plans[l], Q[l], Kf[l], Vf[l], O16=O[l], stream=stream, parts=parts, precise=a.precise)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    graph = None
    with torch.cuda.stream(stream):
        step()
        stream.synchronize()
        assert ctx.device_status(stream) == 0
        if not a.no_graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                step()
    run = (lambda: graph.replay()) if graph is not None else step

    with torch.cuda.stream(stream):
        for _ in range(max(a.warmup, 3)):
            run()
    barrier()
    try:      # NVML numbers GPUs physically; the PCI address names this rank's device whatever CUDA_VISIBLE_DEVICES says
        pr = torch.cuda.get_device_properties(local)
        pci = "%08X:%02X:%02X.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
    except AttributeError:
        pci = None
    sampler = ClockSampler(local, pci)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(a.steps):
            run()
        e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    assert ctx.device_status(stream) == 0

    # ---- per-kernel time: the 20 tile-kernel launches of a step alone (and the 20 merges alone), each set replayed as
    # its own CUDA graph with events around the replays on the launch stream
    def timed_parts(parts):
        with torch.cuda.stream(stream):
            step(parts=parts)
            stream.synchronize()
            g_ = None
            if not a.no_graph:
                g_ = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g_, stream=stream):
                    step(parts=parts)
            go = (lambda: g_.replay()) if g_ is not None else (lambda: step(parts=parts))
            go()
            k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            k0.record(stream)
            for _ in range(a.steps):
                go()
            k1.record(stream)
        barrier()
        return k0.elapsed_time(k1) / (a.steps * L)

    tile_ms = timed_parts(1)
    merge_ms = timed_parts(2)

    # ---- end to end: host buffers per layer through the host-buffer entry point
    e2e_ms, h2d, d2h = None, 0, 0
    if not a.no_e2e:
        hQ, hK, hV = Q.cpu().pin_memory(), Kf.cpu().pin_memory(), Vf.cpu().pin_memory()
        hO = torch.zeros((L, nseq * 32, 16, 128), dtype=torch.float16).pin_memory()
        h2d = L * (hQ[0].numel() + hK[0].numel() + hV[0].numel()) * 2
        d2h = L * hO[0].numel() * 2

        def step_host():
            for l in range(L):
                ctx.attention_host(plans[l], hQ[l], hK[l], hV[l], O16=hO[l], stream=stream)
            ctx.host_flush(stream)

        with torch.cuda.stream(stream):
            step_host()
        barrier()
        n_e2e = max(2, a.steps // 2)
        t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            t0.record(stream)
            for _ in range(n_e2e):
                step_host()
            t1.record(stream)
        barrier()
        e2e_ms = t0.elapsed_time(t1) / n_e2e
        assert torch.equal(hO[L - 1].to(dev), O[L - 1]), "host-buffer path and resident path disagree"

    # ---- max over ranks, final output gather (outside the timed region)
    vals = torch.tensor([ms, tile_ms, merge_ms, e2e_ms or 0.0], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
        gathered = [torch.empty_like(O[L - 1]) for _ in range(world)]
        dist.all_gather(gathered, O[L - 1])
    ms, tile_ms, merge_ms, e2e_ms_max = (float(x) for x in vals.tolist())

    if rank == 0:
        tokens_step = world * nseq * 32
        ms_step = ms / a.steps
        value = tokens_step / (ms_step * 1e-3)
        flops_launch = nseq * wl.algorithmic_flops(nblk)
        bytes_launch = nseq * wl.algorithmic_bytes(nblk)
        ach_tf = flops_launch / (tile_ms * 1e-3) / 1e12
        ach_gbs = bytes_launch / (tile_ms * 1e-3) / 1e9
        t_tensor = flops_launch / (pk["tf_sustained"] * 1e12)
        t_hbm = bytes_launch / (pk["hbm"] * 1e9)
        line = {
            "metric": METRIC, "value": value, "unit": "query_tok/s", "n_gpus": world, "steps": a.steps, "warmup": max(a.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic", "config": workload_config(a, world),
            "roofline": {"bound": "tensor", "achieved": ach_tf, "peak": pk["tf_sustained"], "unit": "TFLOP/s",
                         "frac": ach_tf / pk["tf_sustained"], "traffic": NCU_TRAFFIC_BYTES_PER_UNIT * st.total_units,
                         "traffic_note": "ncu dram read+write of a 32-sequence launch scaled by units; algorithmic bytes per launch = %d" % bytes_launch,
                         "kernel": "attn_tile_kernel", "ms_per_launch": tile_ms, "peak_source": pk["src"] + " sustained bf16",
                         "hbm_achieved_gbs": ach_gbs, "hbm_peak_gbs": pk["hbm"], "hbm_frac": ach_gbs / pk["hbm"],
                         "slower_bound": "tensor" if t_tensor >= t_hbm else "hbm",
                         "merge_ms_per_launch": merge_ms,
                         "step_frac_of_roofline": (L * max(t_tensor, t_hbm)) / (ms_step * 1e-3)},
            "gpu_launches": a.steps * L * 2,
            "plan": {"ctas": st.nctas, "items": st.nitems, "total_units": st.total_units, "max_cta_units": st.max_cta_units},
            "clocks": clocks,
        }
        if e2e_ms:
            line["e2e"] = {"value": tokens_step / (e2e_ms_max * 1e-3), "unit": "query_tok/s", "h2d_bytes_per_step": h2d,
                           "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms_max}
        if not a.no_cpu_baseline:
            times, threads = cpu_sample_seconds(a.ctx, 3)
            sec = min(times)
            line["cpu_baseline"] = {"value": 32.0 / (L * sec), "unit": "query_tok/s", "cores": threads, "kind": "port",
                                    "sample": f"1 sequence x 1 layer at {a.ctx} tokens (torch CPU fp32 fake-quant + SDPA, best of 3), scaled by 1/{L} layers"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


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
    sys.path.insert(0, os.path.join(ROOT, "tests"))
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
    else:
        run_ours(args)
