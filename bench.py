#!/usr/bin/env python3
"""Benchmark of the block-quantized matvec / matmul path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  The headline workload is the Q4_K decode matvec over an
FFN-shaped triple (gate, up: 2560 -> 9728; down: 9728 -> 2560) at batch 1 with
fp16 activations, repeated over 64 layers that each own a distinct copy of the
weights, so one step streams 2.69 GB of native GGUF blocks and nothing is
served from L2.  `value` is algorithmic bytes (blocks + x + y) per second with
everything resident in HBM, the median of five timed regions of K steps each;
`e2e` is the same pass through the host-buffer operator (QB.matvec twin), x
copied from pinned host memory and y copied back on every call.  A `suite`
object carries the other configurations (Q8_0, ternary, IQ2_XXS trunk sweep at
batch 1 and 4, the verify batches, and the 32 / 128 / 512-token matmuls).

`--impl reference` times the reference's CPU engine on the host cores.  That
engine is Swift and cannot be built here, so it is the C restatement in
oracle/ (kind "port"), row-parallel over all host threads, over the same 64
layers of distinct weights.

Under torchrun (N > 1) every matrix is split by output rows across the ranks and
the kernels themselves store every rank's rows into every rank's copy of the
output over NVLink (okf_gemm_gather: the matvec's final stores, the matmul's
epilogue); an NCCL all-gather after the launch is timed beside it.  Every
exchange completes inside the timed region.  The total work is fixed, so scaling is
"strong".  Before anything is timed, every rank checks its own gathered copy of
each distinct matrix's output against the CPU oracle on sampled rows and the
worst error over all ranks is printed as `parity`.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from chatokf_b200.gguf_types import GGUFType, block_bytes, block_elems, row_byte_count  # noqa: E402

F32, F16, BF16 = 0, 1, 2
L2_BYTES = 126 * 1024 * 1024

# name -> (seed, activation dtype, matrices per layer [(label, type, K, M)], layers)
WORKLOADS = {
    "q8_0_gemv_2048": (0, F32, [("w", GGUFType.Q8_0, 2048, 2048)], 64),
    "q4k_ffn_gemv": (1, F16, [("gate", GGUFType.Q4_K, 2560, 9728), ("up", GGUFType.Q4_K, 2560, 9728),
                               ("down", GGUFType.Q4_K, 9728, 2560)], 64),
    "ternary_ffn": (2, F16, [("gate", GGUFType.Q2_0, 2048, 6144), ("up", GGUFType.Q2_0, 2048, 6144),
                              ("down", GGUFType.Q2_0, 6144, 2048)], 64),
    "q4k_prefill": (3, BF16, [("up", GGUFType.Q4_K, 5120, 17408), ("down", GGUFType.Q4_K, 17408, 5120)], 2),
    "iq2xxs_trunk": (4, F16, [("q", GGUFType.IQ2_XXS, 5120, 5120), ("k", GGUFType.IQ2_XXS, 5120, 1024),
                               ("v", GGUFType.IQ2_XXS, 5120, 1024), ("o", GGUFType.IQ2_XXS, 5120, 5120),
                               ("gate", GGUFType.IQ2_XXS, 5120, 17408), ("up", GGUFType.IQ2_XXS, 5120, 17408),
                               ("down", GGUFType.IQ2_XXS, 17408, 5120)], 64),
    # not a BASELINE configuration: the headline's shapes in the gemma trunks' Q4_0
    "q4_0_ffn_gemv": (5, F16, [("gate", GGUFType.Q4_0, 2560, 9728), ("up", GGUFType.Q4_0, 2560, 9728),
                                ("down", GGUFType.Q4_0, 9728, 2560)], 64),
}
HEADLINE = "q4k_ffn_gemv"


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm": float(d["hbm_gbs"]), "tensor": float(d["bf16_tflops"]),
                "tensor_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "src": "measured"}
    return {"hbm": 6650.0, "tensor": 1590.0, "tensor_sustained": 1400.0, "src": "fallback"}


def dt_size(dt):
    return 4 if dt == F32 else 2


def workload_config(name, batch, layers):
    """What both arms of the benchmark run; the same dict on both JSON lines."""
    seed, xdt, mats, nl = WORKLOADS[name]
    layers = nl if layers is None else layers
    wbytes = sum(row_byte_count(ty, k) * m for _, ty, k, m in mats) * layers
    return {"workload": name, "batch": batch, "activations": {F32: "f32", F16: "f16", BF16: "bf16"}[xdt],
            "layers_per_step": layers,
            "matrices": [[lab, GGUFType(ty).name, k, m] for lab, ty, k, m in mats],
            "weight_bytes_per_step": wbytes,
            "l2": "inputs larger than L2: every layer owns a distinct copy of its weights "
                  f"({wbytes / 1e9:.2f} GB per step vs 126 MB L2)"}


def pool_blocks(ty, seed, n_blocks=1 << 15):
    """A pool of valid blocks quantized on the host from seeded N(0, 0.02)
    weights (ternary: P = 1/4, 1/2, 1/4 with |N(0, 0.05)| scales per 256)."""
    from chatokf_b200 import synth

    rng = np.random.default_rng(seed)
    per = block_elems(ty)
    if ty == GGUFType.Q2_0:
        return synth.ternary_q2_0(rng, n_blocks * per, group=256).reshape(n_blocks, -1)
    w = rng.normal(0.0, 0.02, size=n_blocks * per).astype(np.float32)
    return synth.quantize(ty, w).reshape(n_blocks, -1)


def algorithmic_bytes(mats, xdt, n):
    """Native GGUF block bytes + activations in + fp32 outputs, per layer."""
    total = 0
    for _, ty, k, m in mats:
        total += row_byte_count(ty, k) * m + n * k * dt_size(xdt) + n * m * 4
    return total


class ClockSampler:
    """NVML readings of SM clock, power and throttle reasons every 20 ms."""

    BAD = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20}
    NOTE = {"sw_power_cap": 0x4}

    def __init__(self, index):
        self.samples, self._stop, self._t = [], threading.Event(), None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception as e:  # no NVML: report that instead of clocks
            self.nv, self.err = None, repr(e)

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    rs = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    rs = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                pw = nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0
                self.samples.append((time.perf_counter(), mhz, rs, pw))
            except Exception:
                pass
            self._stop.wait(0.02)

    def start(self):
        if self.nv:
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()

    def stop(self):
        self._stop.set()
        if self._t:
            self._t.join()

    def summary(self, t0, t1, note=""):
        if not self.nv:
            return {"error": self.err}
        inside = [s for s in self.samples if t0 <= s[0] <= t1]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0, "note": note}
        mask = 0
        for s in inside:
            mask |= s[2]
        reasons = [k for k, b in {**self.BAD, **self.NOTE}.items() if mask & b]
        return {"sm_mhz": float(np.median([s[1] for s in inside])), "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "power_w_max": max(s[3] for s in inside), "samples": len(inside),
                "note": note}


# ---------------------------------------------------------------------------
# reference arm: the CPU engine (C restatement) on the host cores
# ---------------------------------------------------------------------------

def cpu_layer_weights(mats, pool, rng, rows_frac=1.0):
    """One layer's matrices assembled from the block pool (a distinct draw per call)."""
    out = []
    for _, ty, k, m in mats:
        mm = max(1, int(m * rows_frac))
        nblk = k // block_elems(ty) * mm
        out.append((mm, pool[ty][rng.integers(0, pool[ty].shape[0], size=nblk)].reshape(-1)))
    return out


def cpu_pass(mats, weights, xs, faithful=False):
    """One pass of the oracle over one layer's matrices; returns (seconds, bytes)."""
    import oracle

    secs, nbytes = 0.0, 0
    for (_, ty, k, _), (mm, w), x in zip(mats, weights, xs):
        t0 = time.perf_counter()
        oracle.matvec(ty, w, k, mm, x, threads=os.cpu_count() or 1, faithful=faithful)
        secs += time.perf_counter() - t0
        nbytes += row_byte_count(ty, k) * mm + k * 4 + mm * 4
    return secs, nbytes


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    seed, xdt, mats, nl = WORKLOADS[args.workload]
    layers = nl if args.layers is None else args.layers
    pool = {ty: pool_blocks(ty, seed, 1 << 12) for ty in {m[1] for m in mats}}
    rng = np.random.default_rng(seed + 100)
    cast = np.float16 if xdt == F16 else np.float32
    xs = [rng.normal(size=k).astype(cast).astype(np.float32) for _, _, k, _ in mats]
    # every layer its own copy of the weights, as on the GPU arm (a few GB of host memory)
    per_layer = [cpu_layer_weights(mats, pool, rng) for _ in range(layers)]

    def step():
        secs = nbytes = 0.0
        for w in per_layer:
            s_, b_ = cpu_pass(mats, w, xs)
            secs += s_
            nbytes += b_
        return secs, nbytes

    for _ in range(min(args.warmup, 3)):
        step()
    secs = nbytes = 0.0
    for _ in range(args.steps):
        s_, b_ = step()
        secs += s_
        nbytes += b_
    val = nbytes / secs / 1e9
    cores = os.cpu_count() or 1
    sample = (f"{args.steps} steps x {layers} layers of distinct weights; C restatement of GQ.matvec (scratch hoisted out "
              f"of the block loop), activations widened to f32 as the CPU engine takes them, {cores} threads")
    print(json.dumps({
        "impl": "reference", "metric": "quant GEMV HBM GB/s at b=1 (%s)" % args.workload, "value": val, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": secs / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.workload, 1, args.layers),
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": "port", "variant": "hoisted", "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------

class Layers:
    """Device-resident weights of a workload: per layer and matrix a distinct
    copy assembled from the block pool, plus activations and output buffers."""

    def __init__(self, ctx, name, n, rank, world, layers=None, gather="fused"):
        import torch

        from chatokf_b200.enc import GGUFTensor

        self.torch = torch
        seed, xdt, mats, nl = WORKLOADS[name]
        self.name, self.xdt, self.n = name, xdt, n
        self.layers = nl if layers is None else layers
        self.mats = [(lab, ty, k, m // world) for lab, ty, k, m in mats]
        self.full_mats = mats
        self.world, self.rank = world, rank
        tdt = {F32: torch.float32, F16: torch.float16, BF16: torch.bfloat16}[xdt]
        gen = torch.Generator(device="cuda").manual_seed(seed * 1000 + rank)
        pools = {ty: torch.from_numpy(pool_blocks(ty, seed)).cuda() for ty in {m[1] for m in mats}}
        self.items = []  # (GGUFTensor, Weights, x, out_local)
        self.bufs = []   # the weight bytes behind every item (this rank's rows)
        xs = {}
        for _, _, k, _ in mats:
            if k not in xs:
                g = torch.Generator(device="cuda").manual_seed(seed * 77 + k)
                xs[k] = torch.randn(n, k, generator=g, device="cuda", dtype=torch.float32).to(tdt)
        self.xs = xs
        for layer in range(self.layers):
            for lab, ty, k, m in self.mats:
                nblk = k // block_elems(ty) * m
                idx = torch.randint(0, pools[ty].shape[0], (nblk,), generator=gen, device="cuda")
                buf = torch.empty(nblk * block_bytes(ty) + 256, dtype=torch.uint8, device="cuda")
                buf[: nblk * block_bytes(ty)] = pools[ty][idx].reshape(-1)
                buf[nblk * block_bytes(ty):] = 0
                w = ctx.wrap(buf, nblk * block_bytes(ty))
                out = torch.empty(n, m, dtype=torch.float32, device="cuda")
                self.items.append((GGUFTensor(f"l{layer}.{lab}", (k, m), ty), w, xs[k], out))
                self.bufs.append(buf)
        self.bytes_per_step = algorithmic_bytes(mats, xdt, n) * self.layers
        self.weight_bytes_per_step = sum(row_byte_count(ty, k) * m for _, ty, k, m in mats) * self.layers
        self.flops_per_step = sum(2 * n * k * m for _, _, k, m in mats) * self.layers
        # how the row shards' outputs reach every rank: "fused" = the kernel stores into every
        # rank's buffer itself (the matvec's final stores, the matmul's epilogue), "nccl" = an
        # all-gather after every launch,
        # "none" = not at all (compute only, for comparison)
        self.gather = gather if world > 1 else "none"
        if world > 1:
            self.gathered = {m: torch.empty(world, n, m, dtype=torch.float32, device="cuda")
                             for m in {mm[3] for mm in self.mats}}
        if self.gather == "fused":
            from chatokf_b200 import tp

            sizes = [(n, t.M * world) for t, _, _, _ in self.items]
            # free-running: no launch waits for the exchange before it (x here never derives from
            # a gathered output) and the step ends with one wait that covers them all; ordered:
            # every launch waits for the exchange launched before it, as a chain of dependent
            # projections has to
            self.peers = tp.PeerOutputs(ctx, sizes, free=True)
            self.peers_ordered = tp.PeerOutputs(ctx, sizes, free=False)

    # Projections the reference's engines wrap in one MetalEnc.parallel region
    # (QwenMetalEngine.swift:464-469 gate || up, :691-696 q || k || v): they read the
    # same activations and have no order among themselves.
    REGIONS = ({"q", "k", "v"}, {"gate", "up"})

    def step(self, enc, ordered=False):
        import torch.distributed as dist

        peers = (self.peers_ordered if ordered else self.peers) if self.gather == "fused" else None

        i, per_layer = 0, len(self.mats)
        while i < len(self.items):
            lab = self.mats[i % per_layer][0]
            region = next((r for r in self.REGIONS if lab in r), None)
            j = i + 1
            while region and j < len(self.items) and j // per_layer == i // per_layer \
                    and self.mats[j % per_layer][0] in region:
                j += 1
            def call(idx):
                t, w, x, out = self.items[idx]
                if self.gather == "fused":
                    enc.gemm_gather(t, x, peers.slot(idx, t.M), w, self.n)
                else:
                    enc.gemm(t, x, out, w, self.n)

            if j - i > 1:
                with enc.parallel():
                    for idx in range(i, j):
                        call(idx)
            else:
                call(i)
            if self.gather == "nccl":
                for t, w, x, out in self.items[i:j]:
                    dist.all_gather_into_tensor(self.gathered[t.M].view(-1), out.view(-1))
            i = j
        if self.gather == "fused":
            enc.gather_wait()  # every launch waited for the exchange before it; this waits for the last

    def gathered_output(self, idx):
        """This rank's copy of the whole output of item idx as a host array [n][M_total]."""
        t, _, _, out = self.items[idx]
        if self.world == 1:
            return out.cpu().numpy()
        if self.gather == "fused":
            return self.peers.read(idx)
        if self.gather == "nccl":
            from chatokf_b200 import tp

            return tp.to_token_major(self.gathered[t.M]).cpu().numpy()
        return None

    def check_parity(self, enc, dist, rows_per_rank=16):
        """Untimed checker leg: one step, then every rank compares its own gathered copy of the
        outputs of the first and the last layer with the CPU oracle on sampled rows of the
        whole matrices (each rank contributes the bytes of its sampled rows).  Returns the
        worst max|y - ref| / max|ref| over matrices; the caller reduces it over the ranks."""
        import oracle

        torch = self.torch
        self.step(enc)
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        if self.world > 1 and self.gather == "none":
            return None
        per_layer, worst = len(self.mats), 0.0
        rng = np.random.default_rng(12345)  # the same rows on every rank
        for idx in list(range(per_layer)) + list(range(len(self.items) - per_layer, len(self.items))):
            t, _, x, _ = self.items[idx]
            m_local, rb = t.M, row_byte_count(t.type, t.K)
            rows = np.unique(np.concatenate([[0, m_local - 1], rng.integers(0, m_local, size=rows_per_rank - 2)]))
            mine = self.bufs[idx][: m_local * rb].view(m_local, rb)[torch.from_numpy(rows).cuda()].contiguous()
            if self.world > 1:
                every = [torch.empty_like(mine) for _ in range(self.world)]
                dist.all_gather(every, mine)
            else:
                every = [mine]
            blocks = torch.cat(every).cpu().numpy().reshape(-1)
            global_rows = np.concatenate([r * m_local + rows for r in range(self.world)])
            X = x.float().cpu().numpy().reshape(self.n, t.K)
            ref = oracle.matmul(int(t.type), blocks, t.K, global_rows.size, X, self.n)
            if self.world > 1 and self.gather == "nccl":
                # the gather buffers are shared by matrices of one size: run this one again
                tt, w, xx, out = self.items[idx]
                enc.gemm(tt, xx, out, w, self.n)
                dist.all_gather_into_tensor(self.gathered[tt.M].view(-1), out.view(-1))
                torch.cuda.synchronize()
            got = self.gathered_output(idx).reshape(self.n, -1)[:, global_rows]
            mag = float(np.abs(ref).max())
            worst = max(worst, float(np.abs(got - ref).max()) / (mag if mag > 0 else 1.0))
        return worst

    def count_launches(self, ctx, enc):
        """Kernel launches of one step, counted by the library while the step runs once."""
        before = ctx.launches
        self.step(enc)
        self.launches_per_step = ctx.launches - before
        return self.launches_per_step


def time_graph(torch, stream, fn, steps, warmup, use_graph=True):
    """Warm up, capture one step in a CUDA graph, replay it `steps` times between
    two events on the launching stream.  Returns (ms per step, graph used?)."""
    with torch.cuda.stream(stream):
        for _ in range(max(warmup, 1)):
            fn()
    stream.synchronize()
    graph = None
    if use_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                fn()
        except Exception as e:  # fall back to plain launches, and say so
            sys.stderr.write(f"bench: graph capture failed ({e!r}); timing plain launches\n")
            graph = None
            torch.cuda.synchronize()
    run = graph.replay if graph is not None else fn
    with torch.cuda.stream(stream):
        for _ in range(max(warmup, 3)):
            run()
    stream.synchronize()
    return run, graph is not None


def timed_region(torch, stream, run, steps, dist=None):
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    with torch.cuda.stream(stream):
        start.record(stream)
        for _ in range(steps):
            run()
        end.record(stream)
    end.synchronize()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    ms = start.elapsed_time(end)
    if dist is not None:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    return ms, t0, t1


def e2e_steps(ctx, L, steps, warmup, torch, dist):
    """The same pass through the host-facing calls: x from pinned host memory, y back to
    host memory, on every call.  One GPU: the host-buffer operator (okf_matmul_host).
    Row shards: per matrix x up, this rank's rows with the exchange fused into the kernel
    (decode) or an all-gather after it (prefill), a wait for the exchange, the whole y down.
    Returns (seconds per step, h2d bytes, d2h bytes, api)."""
    from chatokf_b200.enc import CudaEnc, QB

    qb = QB(ctx)
    enc = CudaEnc(ctx)
    hx = {k: torch.empty(L.n, k, dtype=torch.float32).pin_memory() for k in L.xs}
    for k in hx:
        hx[k].copy_(L.xs[k].float().cpu())
    hy = {m: torch.empty(L.n, m, dtype=torch.float32).pin_memory() for m in {mm[3] for mm in L.mats}}
    full = {m: torch.empty(L.world, L.n, m, dtype=torch.float32).pin_memory() for m in hy} if L.world > 1 else None
    xd = {k: torch.empty(L.n, k, dtype=torch.float32, device="cuda") for k in L.xs}
    h2d = sum(L.n * t.K * 4 for t, _, _, _ in L.items)
    d2h = sum(L.n * t.M * 4 * L.world for t, _, _, _ in L.items)
    host_calls = [(t, w, hx[t.K].data_ptr(), hy[t.M].data_ptr()) for t, w, _, _ in L.items]
    if L.world == 1:
        api = "okf_matmul_host (QB.matvec twin) on page-locked host buffers, one synchronous call per matrix"
    elif L.gather == "fused":
        api = ("per matrix: cudaMemcpyAsync of x, okf_gemm_gather (rows stored into every rank's output by the "
               "kernel), okf_gather_wait, okf_copy_to_host of the whole y")
    else:
        api = "per matrix: copy of x, okf_gemm on this rank's rows, NCCL all-gather, copy of the whole y, stream sync"

    def one():
        if L.world == 1:
            for t, w, x_addr, y_addr in host_calls:
                qb.matmul_at(t, w, x_addr, L.n, y_addr)
            return
        for idx, (t, w, _, out) in enumerate(L.items):
            if L.gather == "fused":
                xd[t.K].copy_(hx[t.K], non_blocking=True)
                enc.gemm_gather(t, xd[t.K], L.peers.slot(idx, t.M), w, L.n)
                enc.gather_wait()
                L.peers.read_into(idx, full[t.M])
            else:
                xd[t.K].copy_(hx[t.K], non_blocking=True)
                enc.gemm(t, xd[t.K], out, w, L.n)
                if L.gather == "nccl":
                    dist.all_gather_into_tensor(L.gathered[t.M].view(-1), out.view(-1))
                    full[t.M].copy_(L.gathered[t.M], non_blocking=True)
                torch.cuda.current_stream().synchronize()

    for _ in range(max(1, min(warmup, 3))):
        one()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        one()
    torch.cuda.synchronize()
    sec = time.perf_counter() - t0
    if dist is not None:
        t = torch.tensor([sec], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec = float(t.item())
    return sec / steps, h2d, d2h, api


def cpu_baseline(name, batch=1, budget_s=10.0):
    """Time the oracle (all host threads) on a slice of the workload sized to about
    `budget_s` seconds: whole layers of distinct weights.  `value` is the variant with the
    decode scratch hoisted out of the block loop; `faithful` allocates the 256-float
    scratch per block as GQ.matvec does (LLM/Gemma/Gemma4Quant.swift:125-136)."""
    seed, xdt, mats, _ = WORKLOADS[name]
    pool = {ty: pool_blocks(ty, seed, 1 << 10) for ty in {m[1] for m in mats}}
    rng = np.random.default_rng(seed + 100)
    xs = [rng.normal(size=k).astype(np.float16).astype(np.float32) for _, _, k, _ in mats]
    probe = cpu_layer_weights(mats, pool, rng, rows_frac=1 / 16)
    s0, _ = cpu_pass(mats, probe, xs)
    reps = int(max(1, min(64, budget_s / max(s0 * 16, 1e-3))))
    layers = [cpu_layer_weights(mats, pool, rng) for _ in range(reps)]
    secs = nbytes = 0.0
    for w in layers:
        s_, b_ = cpu_pass(mats, w, xs)
        secs += s_
        nbytes += b_
    fsecs = fbytes = 0.0
    for w in layers[:max(1, reps // 4)]:
        s_, b_ = cpu_pass(mats, w, xs, faithful=True)
        fsecs += s_
        fbytes += b_
    cores = os.cpu_count() or 1
    if batch > 8:
        # GQ.matmul answers these types as `batch` independent matvecs: same rate per column
        flops = 2.0 * sum(k * m for _, _, k, m in mats) * reps
        return {"value": flops / secs / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port", "variant": "hoisted",
                "sample": f"{reps} single-column pass(es) over one layer, {secs:.1f} s; GQ.matmul runs these "
                          f"types as N independent matvecs, so the per-column rate is the matmul rate"}
    return {"value": nbytes / secs / 1e9, "unit": "GB/s", "cores": cores, "kind": "port", "variant": "hoisted",
            "faithful": {"value": fbytes / fsecs / 1e9, "unit": "GB/s",
                         "note": "256-float scratch allocated per block per row, as the Swift code does"},
            "sample": f"{reps} layer(s) of distinct weights (all rows of every matrix) of the {WORKLOADS[name][3]}, "
                      f"{secs:.1f} s; C restatement of GQ.matvec (the Swift engine does not build on Linux)"}


def median_region(torch, stream, run, steps, dist=None, regions=5):
    """`regions` timed regions of `steps` steps each; returns (median ms per region, all of
    them, host clock around the median one)."""
    got = [timed_region(torch, stream, run, steps, dist) for _ in range(regions)]
    order = sorted(range(regions), key=lambda i: got[i][0])
    mid = got[order[regions // 2]]
    return mid[0], [g[0] for g in got], got[0][1], got[-1][2]


def suite_entry(ctx, torch, stream, name, n, pk, steps=20, layers=None, tile=False, rank=0, world=1, dist=None,
                gather="fused"):
    from chatokf_b200.enc import CudaEnc

    L = Layers(ctx, name, n, rank, world, layers=layers, gather=gather)
    enc = CudaEnc(ctx)
    if tile:
        def fn():
            for t, w, x, out in L.items:
                enc.gemmTile(t, x, out, w, L.n)
    else:
        def fn():
            L.step(enc)
    with torch.cuda.stream(stream):
        parity = L.check_parity(enc, dist) if not tile else None
    stream.synchronize()
    # NCCL calls inside a captured step are left to plain launches
    run, graphed = time_graph(torch, stream, fn, steps, 3, use_graph=not (world > 1 and L.gather == "nccl"))
    ms, _, _ = timed_region(torch, stream, run, steps, dist)
    ms /= steps
    gbs = L.bytes_per_step / ms / 1e6
    tf = L.flops_per_step / ms / 1e9
    if parity is not None and dist is not None:
        t = torch.tensor([parity], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        parity = float(t.item())
    out = {"n": n, "layers": L.layers, "ms_per_step": ms, "GB/s": gbs, "TFLOP/s": tf,
           "frac_hbm": gbs / pk["hbm"], "frac_tensor": tf / pk["tensor"], "frac_tensor_nominal": tf / 2250.0,
           "graph": graphed, "bytes_per_step": L.bytes_per_step, "parity_max_rel": parity}
    if world > 1:
        out["gather"] = L.gather
    if L.gather == "fused" and world > 1:
        run_o, _ = time_graph(torch, stream, lambda: L.step(enc, ordered=True), steps, 3)
        ms_o, _, _ = timed_region(torch, stream, run_o, steps, dist)
        out["ordered_chain"] = {"ms_per_step": ms_o / steps, "GB/s": L.bytes_per_step / (ms_o / steps) / 1e6}
        L.peers.close()
        L.peers_ordered.close()
    del L
    torch.cuda.empty_cache()
    return out


def run_ours(args):
    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        args.gpus = world
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (there is no CPU path to fall back to)")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    import __graft_entry__

    if rank == 0:
        __graft_entry__.build()
    if dist is not None:
        dist.barrier()
    from chatokf_b200.enc import Context, CudaEnc

    pk = peaks()
    ctx = Context(local)
    enc = CudaEnc(ctx)
    stream = torch.cuda.Stream()
    wl, batch = args.workload, args.batch
    L = Layers(ctx, wl, batch, rank, world, layers=args.layers, gather=args.gather)
    tensor_bound = batch > 8
    tol = 1e-2 if tensor_bound else 1e-4

    # ---- untimed checker leg: this rank's gathered outputs against the CPU oracle
    with torch.cuda.stream(stream):
        parity = L.check_parity(enc, dist)
    stream.synchronize()
    status = ctx.device_status()
    if dist is not None:
        t = torch.tensor([parity if parity is not None else -1.0, float(status)], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        parity, status = (float(t[0]) if parity is not None else None), int(t[1])
    parity_rec = {"max_rel": parity, "tol": tol, "status": status, "ranks": world,
                  "what": "first and last layer, every matrix, 16 sampled rows per rank of the whole matrix, "
                          "each rank's own copy of the gathered output vs the CPU oracle"}
    if status != 0 or (parity is not None and not parity <= tol):
        if rank == 0:
            print(json.dumps({"error": "parity check failed before timing", "parity": parity_rec}))
        sys.stdout.flush()
        os._exit(3)

    with torch.cuda.stream(stream):
        L.count_launches(ctx, enc)
    stream.synchronize()
    sampler = ClockSampler(local)
    sampler.start()
    use_graph = not (world > 1 and L.gather == "nccl")  # NCCL calls are not captured here
    run, graphed = time_graph(torch, stream, lambda: L.step(enc), args.steps, args.warmup, use_graph=use_graph)
    for _ in range(args.warmup):
        with torch.cuda.stream(stream):
            run()
    ms, all_ms, t0, t1 = median_region(torch, stream, run, args.steps, dist)
    note = "clocks sampled across the five timed regions"
    if len([s for s in sampler.samples if t0 <= s[0] <= t1]) < 3:
        # timed regions shorter than a few sampler periods: sample an untimed
        # loop of the same graph for about a second instead
        reps = int(max(10, 1000.0 / max(ms / args.steps, 1e-3)))
        t0 = time.perf_counter()
        with torch.cuda.stream(stream):
            for _ in range(reps):
                run()
        stream.synchronize()
        t1 = time.perf_counter()
        note = "timed regions too short to sample; clocks sampled over an untimed loop of the same step right after them"
    sampler.stop()
    clocks = sampler.summary(t0, t1, note)

    ms_step = ms / args.steps
    value = L.bytes_per_step / ms_step / 1e6  # GB/s
    tflops = L.flops_per_step / ms_step / 1e9
    launches = L.launches_per_step * args.steps  # graph replays launch the captured kernels again
    per_launch_bytes = L.bytes_per_step / L.launches_per_step / world
    per_launch_us = ms_step * 1e3 / L.launches_per_step

    ordered = None
    if world > 1 and L.gather == "fused":
        # the same step with every launch waiting for the exchange before it
        run_o, _ = time_graph(torch, stream, lambda: L.step(enc, ordered=True), args.steps, args.warmup)
        ms_o, _, _, _ = median_region(torch, stream, run_o, args.steps, dist, regions=3)
        ordered = {"ms_per_step": ms_o / args.steps,
                   "value": (L.flops_per_step / (ms_o / args.steps) / 1e9) if tensor_bound
                   else L.bytes_per_step / (ms_o / args.steps) / 1e6,
                   "note": "every launch waits, before it reads x, for the exchange launched before it: what a chain "
                           "of dependent projections pays (a few NVLink crossings per launch)"}

    e2e_s, h2d, d2h, api = e2e_steps(ctx, L, max(1, min(args.steps, 10)), args.warmup, torch, dist)
    e2e_val = (L.flops_per_step / e2e_s / 1e12) if tensor_bound else (L.bytes_per_step / e2e_s / 1e9)

    traffic = TRAFFIC.get(wl) if world == 1 else None  # measured on one GPU only
    if tensor_bound:
        roof = {"bound": "tensor", "achieved": tflops / world, "peak": pk["tensor"], "unit": "TFLOP/s",
                "frac": tflops / world / pk["tensor"], "frac_of_nominal_2250": tflops / world / 2250.0,
                "traffic": traffic, "peak_source": pk["src"] + " (burst)",
                "flops_per_launch": L.flops_per_step / L.launches_per_step / world,
                "us_per_launch": per_launch_us, "kernel": "okf gemm_tc (tcgen05)"}
    else:
        roof = {"bound": "hbm", "achieved": per_launch_bytes / per_launch_us / 1e3, "peak": pk["hbm"],
                "unit": "GB/s", "frac": per_launch_bytes / per_launch_us / 1e3 / pk["hbm"],
                "traffic": traffic, "peak_source": pk["src"],
                "bytes_per_launch": per_launch_bytes, "us_per_launch": per_launch_us,
                "kernel": "okf gemv_kernel (decode matvec)"}
    result = {
        "metric": ("prefill GEMM TFLOP/s" if tensor_bound else "quant GEMV HBM GB/s at b=%d" % batch)
                  + " (%s)" % wl,
        "value": tflops if tensor_bound else value, "unit": "TFLOP/s" if tensor_bound else "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16" if tensor_bound else "int8", "data": "synthetic",
        "config": workload_config(wl, batch, args.layers),
        "how": {"arithmetic": ("weights decoded to bf16, tcgen05 MMA, fp32 accumulate" if tensor_bound else
                               "weights as stored bytes x activations as 2 x int8 with one scale per 256, "
                               "s32 accumulate, fp32 scales"),
                "launches_per_step": L.launches_per_step,
                "parallel_regions": "gate || up and q || k || v leave as one launch each, as the "
                                    "reference's engines co-schedule them",
                "parallelism": (f"rows/{world}, outputs to every rank by " +
                                {"fused": "stores from the matvec kernel into peer memory (no collective); free-running: "
                                          "x never derives from a gathered output here, so no launch waits for the "
                                          "exchange before it and the step ends with one wait that covers them all "
                                          "(`ordered_chain` is the same step with every launch waiting)",
                                 "nccl": "an NCCL all-gather after every launch",
                                 "none": "nothing (compute only)"}[L.gather]) if world > 1 else "single GPU",
                "cuda_graph": graphed,
                "regions": {"n": len(all_ms), "steps_each": args.steps, "value_from": "median",
                            "ms_per_step_min": min(all_ms) / args.steps, "ms_per_step_max": max(all_ms) / args.steps}},
        "roofline": roof,
        "ordered_chain": ordered,
        "parity": parity_rec,
        "e2e": {"value": e2e_val, "unit": "TFLOP/s" if tensor_bound else "GB/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_s * 1e3, "api": api},
        "gpu_launches": launches * len(all_ms),
        "fallbacks": ctx.fallbacks,
        "clocks": clocks,
    }
    assert L.launches_per_step > 0
    if not args.no_suite:
        suite = {}
        if world == 1:
            plan = [("q8_0_gemv_2048", 1, {}), ("ternary_ffn", 1, {}), ("iq2xxs_trunk", 1, {}),
                    ("iq2xxs_trunk", 4, {}), ("q4k_ffn_gemv", 4, {}), ("q4k_ffn_gemv", 8, {}),
                    ("q4k_prefill", 32, {"steps": 5}), ("q4k_prefill", 128, {"steps": 5}),
                    ("q4k_prefill", 512, {"steps": 5}), ("ternary_ffn", 512, {"steps": 5, "layers": 4}),
                    ("q4_0_ffn_gemv", 1, {}), ("q4_0_ffn_gemv", 4, {})]
        else:
            # the configurations that are specified as row-sharded: the IQ2_XXS trunk at batch 1 and 4
            # and the 512-token matmul with the stores into every rank's output fused into its
            # epilogue, with an NCCL all-gather after it instead, and without any gather
            plan = [("iq2xxs_trunk", 1, {"layers": 16}), ("iq2xxs_trunk", 4, {"layers": 16}),
                    ("q4k_prefill", 512, {"steps": 5, "gather": "fused"}),
                    ("q4k_prefill", 512, {"steps": 5, "gather": "nccl"}),
                    ("q4k_prefill", 512, {"steps": 5, "gather": "none"})]
        for name, n, kw in plan:
            key = f"{name}_n{n}" + ("_" + kw["gather"] if "gather" in kw else "")
            try:
                suite[key] = suite_entry(ctx, torch, stream, name, n, pk, rank=rank, world=world, dist=dist, **kw)
            except Exception as e:  # one failing entry must not lose the headline
                suite[key] = {"error": repr(e)}
                if dist is not None:
                    raise  # the ranks have to stay in step
        result["suite"] = suite
        result["fallbacks"] = ctx.fallbacks
    if rank == 0 and world == 1 and not args.no_cpu:
        result["cpu_baseline"] = cpu_baseline(wl, batch)
    if rank == 0:
        print(json.dumps(result))
    if dist is not None:
        # Tearing the NCCL communicator down has hung on this software stack; leave
        # it to process exit once every rank is past its last collective.
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel on ONE GPU, from the
# ncu captures summarised under profiles/ (gemv_kernel_q4k_ffn_b1.md: gate || up 28.06 MB and down
# 14.07 MB, the mean of the two; gemm_tc_kernel_q4k_prefill_n512.md).  Not printed for N > 1.
TRAFFIC = {"q4k_ffn_gemv": {"value": 21.07e6, "source": "profiles/gemv_kernel_q4k_ffn_b1.md, one-GPU ncu capture"},
           "q4k_prefill": {"value": 65.4e6, "source": "profiles/gemm_tc_kernel_q4k_prefill_n512.md, one-GPU ncu capture"}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-suite", action="store_true", help="skip the other configurations")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg (profiling runs)")
    ap.add_argument("--workload", default=HEADLINE, choices=sorted(WORKLOADS), help="which configuration is the timed one")
    ap.add_argument("--batch", type=int, default=1, help="activation columns (tokens) per call")
    ap.add_argument("--layers", type=int, default=None, help="layers per step (default: the workload's own count)")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl", "none"],
                    help="N > 1 GPUs: how every rank gets the whole output (fused needs batch <= 8)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
