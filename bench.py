"""Benchmark of the W4G128 / W4A8 matmul path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (benchmark configuration 1, the decode GEMV): y[1,9728] = x[1,2560] * W^T with W a
W4G128 weight, synthetic and seeded.  One step = GEMVs of one activation vector against R
distinct weight copies, walked several times (R * 12.9 MB > the 126 MB L2, so every GEMV
streams its weight from HBM) -- the reference's own microbenchmark does the same on the CPU
(tests/bench_matmul.cpp rotates weight sets under one input).
metric = algorithmic bytes moved per second (weights at 4.125 bit + fp32 x + fp32 y).

ours, N=1      : the walk as ONE persistent kernel (b2w4_chain_*: a list of GEMVs, weights of
                 later GEMVs streaming while earlier ones compute), weights and activations
                 resident in HBM, CUDA-event timing (`value`); the same list through
                 b2w4_chain_run_host with pinned HOST x and every y stored to pinned host
                 memory (`e2e`); the list with every GEMV consuming its predecessor's output,
                 and the one-launch-per-GEMV kernel (`variants`); M in {4,16,64,256} and a
                 Qwen3-4B-shaped decode matmul walk (`sweep`); the reference's own CUDA
                 kernels on this GPU (`gpu_reference`) and its CPU kernel on this box's host
                 cores (`cpu_baseline`).
ours, N>1      : tensor parallel -- every weight is split by output rows across the ranks,
                 each rank streams its shard and the full row is rebuilt on every rank, by the
                 exchange inside the kernels (`value`) and by an NCCL all-gather (strong
                 scaling).
--impl reference: the reference's CPU implementation of the same step (rank 0 only).
Prints ONE JSON line on rank 0.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
from __graft_entry__ import load_package  # noqa: E402

N_OUT, K_IN = 9728, 2560
COPIES = 32   # distinct weight buffers walked by one pass
PASSES = 16   # passes per list: one persistent-kernel launch = PASSES * COPIES GEMVs
RUNS_PER_STEP = 20  # launches of the list per step (a step is about 25 ms of device time)
DEP_RESTART = 16    # a dependent list restarts from x every so many GEMVs (the rows grow by a
                    # factor of up to twenty per GEMV; fp32 carries sixteen of them)
SEED_W, SEED_X = 20261125, 7
METRIC, UNIT = "w4g128_gemv_hbm_gbs", "GB/s"
L2_MB = 126


# dram__bytes_read.sum + dram__bytes_write.sum per GEMV of this workload, from ncu captures of
# the two kernels (persistent list: 410 981 120 B read for 32 GEMVs; one launch per GEMV)
NCU_DRAM_BYTES_PER_GEMV_CHAIN = 410981120 // 32
NCU_DRAM_BYTES_PER_LAUNCH = 12876800


def workload_config(world=1, passes=PASSES, graph=True):
    return {"workload": f"W4G128 W4A8 GEMV M=1 K={K_IN} N={N_OUT} "
                        f"(benchmark configuration 1, decode)",
            "gemvs_per_step": COPIES * passes,
            "l2": f"rotates {COPIES} distinct weight copies "
                  f"({COPIES * 12.84:.0f} MB) > {L2_MB} MB L2",
            "parallelism": (f"tp{world}: output rows split over the ranks, the full row rebuilt "
                            f"on every rank after every GEMV") if world > 1 else "single GPU",
            "act_rule": "int8 per 128 values",
            "launch": ("CUDA graph replay" if graph else "eager")
                      + ", programmatic dependent launch"}


def algorithmic_bytes(n, k, m):
    """int4 weights + one fp16 scale per 128 weights + fp32 x + fp32 y."""
    return n * k // 2 + n * (k // 128) * 2 + m * k * 4 + m * n * 4


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def measured_tensor_peak():
    """Dense bf16 TFLOP/s of a cuBLAS GEMM timed alone on this pool (the tensor roofline the
    many-row matmuls are held against; the int8 path's own peak is twice that)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["bf16_tflops"]), "measured"
    return 1590.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 9
                          for i in range(4) if r[5 + i].lower().startswith("active")})
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def time_steps(torch, fn, steps, warmup, barrier=None):
    for _ in range(warmup):
        fn()
    if barrier:
        barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    if barrier:
        barrier()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps  # ms per step


# --------------------------------------------------------------------------- reference

def reference_lib():
    """oracle/_ref (the unmodified reference CPU library) if it was built, else None."""
    path = os.path.join(ROOT, "oracle", "_ref", "libref_shim.so")
    if not os.path.exists(path):
        return None
    lib = ctypes.CDLL(path)
    lib.ref_time_matmul_bg128.restype = ctypes.c_double
    lib.ref_isa_name.restype = ctypes.c_char_p
    return lib


def cpu_gemv_seconds(pkg, m, copies, repeat, warmup=2):
    """Seconds per GEMV of the reference's CPU kernel (all host threads) on the bench
    workload, rotating `copies` weight buffers; falls back to the scalar oracle port."""
    cores = os.cpu_count() or 1
    x = pkg.synth.activations(SEED_X, 0, m, K_IN)
    one = pkg.synth.bg128_weight(SEED_W, 1, N_OUT, K_IN)
    lib = reference_lib()
    if lib is not None:
        buf = np.concatenate([np.roll(one, 544 * i) for i in range(copies)])
        y = np.zeros((m, N_OUT), dtype=np.float32)
        sec = lib.ref_time_matmul_bg128(
            x.ctypes.data_as(ctypes.c_void_p), m, K_IN, buf.ctypes.data_as(ctypes.c_void_p),
            ctypes.c_size_t(one.nbytes), copies, N_OUT, y.ctypes.data_as(ctypes.c_void_p),
            cores, warmup, repeat)
        return sec, "reference", cores, lib.ref_isa_name().decode()
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol
    t0 = time.perf_counter()
    for _ in range(max(1, repeat // 50)):
        ol.matmul_w4(one, N_OUT, K_IN, x)
    return (time.perf_counter() - t0) / max(1, repeat // 50), "port", 1, "scalar C"


def run_reference(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    pkg = load_package()
    copies = 16
    probe, kind, cores, isa = cpu_gemv_seconds(pkg, 1, copies, 8, warmup=2)
    per_step = max(copies, min(COPIES * 8, int(2.0 / max(probe, 1e-6))))  # ~2 s per step
    times = []
    for i in range(args.warmup + args.steps):
        sec, kind, cores, isa = cpu_gemv_seconds(pkg, 1, copies, per_step, warmup=0)
        if i >= args.warmup:
            times.append(sec)
    sec = sum(times) / len(times)
    gbs = algorithmic_bytes(N_OUT, K_IN, 1) / sec / 1e9
    sample = (f"{per_step} GEMVs per step rotating {copies} weight copies, "
              f"{cores} host threads, isa {isa} (W4A32 arithmetic)")
    line = {"impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT,
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": sec * per_step * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": dict(workload_config(1, 1, False), gemvs_per_step=per_step,
                           l2=f"rotates {copies} weight copies ({copies * 13.2:.0f} MB)",
                           launch=f"{cores} host threads, {isa}",
                           reference="the reference's own CPU kernel (W4A32) on the host cores"),
            "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": cores, "kind": kind,
                             "sample": sample},
            "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def gpu_reference(torch, pkg, args, our_gemv_gbs, our_m256_us):
    """The reference's own CUDA matmul kernels (engine/cuda_matmul.cu, compiled unmodified for
    sm_100 into oracle/_ref/libref_cuda.so) on this GPU and this workload: its one-row GEMV
    (fp32 activations, W4A32) and its many-row path (dequantise the whole weight to fp16,
    cast the activations, cuBLAS), the same rotation of weight copies, CUDA events on the
    legacy default stream the reference launches on.  A comparator, never on the product
    path."""
    path = os.path.join(ROOT, "oracle", "_ref", "libref_cuda.so")
    if not os.path.exists(path):
        return {"unavailable": "oracle/_ref/libref_cuda.so was not built (make -C oracle refcuda)"}
    lib = ctypes.CDLL(path)
    vp = ctypes.c_void_p
    one = pkg.synth.bg128_weight(SEED_W, 1, N_OUT, K_IN)
    copies = [torch.from_numpy(np.roll(one, 544 * i)).cuda() for i in range(COPIES)]
    out = {"kernels": "engine/cuda_matmul.cu of the reference, built for sm_100"}
    with torch.cuda.stream(torch.cuda.default_stream()):
        for m, reps in ((1, 8), (256, 1)):
            x = torch.from_numpy(pkg.synth.activations(SEED_X, 0, m, K_IN)).cuda()
            y = torch.zeros((m, N_OUT), dtype=torch.float32, device="cuda")

            def walk():
                for _ in range(reps):
                    for c in copies:
                        if m == 1:
                            rc = lib.refcuda_gemv_g128(vp(x.data_ptr()), vp(c.data_ptr()),
                                                       vp(y.data_ptr()), N_OUT, K_IN)
                        else:
                            rc = lib.refcuda_gemm_g128(vp(x.data_ptr()), K_IN, vp(c.data_ptr()),
                                                       vp(y.data_ptr()), m, N_OUT, K_IN)
                        if rc != 0:
                            raise RuntimeError(f"reference CUDA kernel failed: {rc}")
            try:
                ms = time_steps(torch, walk, 5, 3)
            except RuntimeError as exc:
                out[f"m{m}"] = {"error": str(exc)[:200]}
                continue
            us = ms * 1e3 / (reps * COPIES)
            if m == 1:
                gbs = algorithmic_bytes(N_OUT, K_IN, 1) / us / 1e3
                out["m1_q4_g128_dense_gemv_cuda"] = {
                    "us_per_gemv": us, "value": gbs, "unit": UNIT,
                    "ours_over_reference": our_gemv_gbs / gbs}
            else:
                out["m256_dequant_then_cublas"] = {
                    "us_per_matmul": us, "tflops": 2.0 * m * N_OUT * K_IN / us / 1e6,
                    "ours_over_reference": us / our_m256_us}
    lib.refcuda_release()
    return out


# --------------------------------------------------------------------------------- ours

def moe_layer(torch, pkg, ctx, args):
    """One Qwen3-30B-A3B-shaped routed-MoE layer (benchmark configuration 4): hidden 2048,
    128 experts, top-8 softmax routing, expert intermediate 768; one decode token and a
    256-token prefill.  Router, routing, compaction, both grouped expert matmuls, SwiGLU and
    the ordered combine are all inside the timed call (b2w4_moe_forward)."""
    h, e, top_k, inter = 2048, 128, 8, 768
    router = torch.from_numpy(pkg.synth.router_weight(SEED_W, 70, e, h).view(np.int16)).cuda()
    gu = ctx.upload_weight(pkg.synth.bg128_weight(SEED_W, 71, e * 2 * inter, h), e * 2 * inter, h)
    dn = ctx.upload_weight(pkg.synth.bg128_weight(SEED_W, 72, e * h, inter), e * h, inter)
    expert_bytes = (2 * inter * h + h * inter) * 4.125 / 8
    out = {}
    for t in (1, 256):
        x = torch.from_numpy(pkg.synth.activations(SEED_X, 80 + t, t, h)).cuda()
        y = torch.zeros((t, h), dtype=torch.float32, device="cuda")
        idx = torch.zeros((t, top_k), dtype=torch.int32, device="cuda")

        def call():
            ctx.moe_forward(x, router, top_k, inter, gu, dn, y, None, idx, None)
        call()  # also grows the context's scratch buffers before the capture
        torch.cuda.synchronize()
        active = len(set(idx.cpu().numpy().ravel().tolist()))
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            ctx.set_stream(side.cuda_stream)
            with torch.cuda.graph(g, stream=side):
                call()
        ctx.set_stream(torch.cuda.current_stream().cuda_stream)
        ms = time_steps(torch, g.replay, 20, 3)
        out[f"tokens{t}"] = {"us_per_layer": ms * 1e3, "active_experts": active,
                             "tokens_per_s_per_layer": t / (ms * 1e-3),
                             "expert_weight_gbs": active * expert_bytes / (ms * 1e-3) / 1e9}
    gu.free()
    dn.free()
    return out


def moe_layer_ep(torch, dist, pkg, ctx, rank, world):
    """The same Qwen3-30B-A3B-shaped MoE layer expert-parallel over `world` ranks: each rank
    holds 128/world experts, computes the routes of its experts, one NCCL all-reduce of the
    [tokens*top_k, H] route buffer, ordered combine on every rank.  Device time, max over
    ranks."""
    h, e, top_k, inter = 2048, 128, 8, 768
    router = torch.from_numpy(pkg.synth.router_weight(SEED_W, 70, e, h).view(np.int16)).cuda()
    gu_blocks = pkg.synth.bg128_weight(SEED_W, 71, e * 2 * inter, h)
    dn_blocks = pkg.synth.bg128_weight(SEED_W, 72, e * h, inter)
    op = pkg.expert_parallel.build_device_moe(ctx, router, gu_blocks, dn_blocks, e, top_k, h,
                                              inter, rank, world,
                                              lambda t: dist.all_reduce(t))
    out = {}
    for t in (1, 256):
        x = torch.from_numpy(pkg.synth.activations(SEED_X, 80 + t, t, h)).cuda()
        y = torch.zeros((t, h), dtype=torch.float32, device="cuda")
        op.forward(x, y)  # grows scratch, warms NCCL
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            ctx.set_stream(side.cuda_stream)
            with torch.cuda.graph(g, stream=side):
                op.forward(x, y)
        ctx.set_stream(torch.cuda.current_stream().cuda_stream)
        ms = time_steps(torch, g.replay, 20, 3, lambda: dist.barrier())
        tm = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        ms = float(tm.item())
        out[f"tokens{t}"] = {"us_per_layer": ms * 1e3,
                             "tokens_per_s_per_layer": t / (ms * 1e-3),
                             "exchange": "NCCL all-reduce of the route buffer",
                             "exchange_bytes": t * top_k * h * 4}
    # decode step with the hand-over inside the kernels (peer stores into staging buffers)
    try:
        import torch.distributed._symmetric_memory as symm
        rows = top_k
        words = pkg.expert_parallel.PeerExchangeMoE.stage_words(rows, h)
        stage = symm.empty((words,), dtype=torch.int64, device=f"cuda:{torch.cuda.current_device()}")
        stage.zero_()
        torch.cuda.synchronize()
        hs = symm.rendezvous(stage, dist.group.WORLD.group_name)
    except Exception as exc:
        print(f"in-kernel MoE hand-over unavailable: {exc}", file=sys.stderr)
        return out
    group = pkg.capi.TpGroup()
    group.rank, group.world = rank, world
    for p_ in range(world):
        group.stage_peers[p_] = hs.buffer_ptrs[p_]
    peer = pkg.expert_parallel.PeerExchangeMoE(op.engine, group, rows)
    x = torch.from_numpy(pkg.synth.activations(SEED_X, 81, 1, h)).cuda()
    y = torch.zeros((1, h), dtype=torch.float32, device="cuda")
    y2 = torch.zeros((1, h), dtype=torch.float32, device="cuda")
    op.forward(x, y)  # the shared kernels' code is loaded before the ranks meet
    torch.cuda.synchronize()
    dist.barrier()
    same = True
    for _ in range(3):  # both halves of the staging buffer; bit for bit the all-reduce result
        op.forward(x, y)
        try:
            peer.forward(x, y2)
            ctx.sync()
        except pkg.capi.B200W4Error as exc:  # e.g. the bounded wait ran out
            print(f"in-kernel MoE hand-over failed: {exc}", file=sys.stderr)
            same = False
        torch.cuda.synchronize()
        same = same and torch.equal(y, y2)
    agree = torch.tensor([1 if same else 0], device="cuda", dtype=torch.int32)
    dist.all_reduce(agree, op=dist.ReduceOp.MIN)
    if not bool(agree.item()):  # never time a path whose result differs
        print("in-kernel MoE hand-over and all-reduce disagree: not timed", file=sys.stderr)
        out["tokens1_peer_exchange"] = {"error": "result differs from the all-reduce path"}
        return out
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        ctx.set_stream(side.cuda_stream)
        with torch.cuda.graph(g, stream=side):
            peer.forward(x, y2)
    ctx.set_stream(torch.cuda.current_stream().cuda_stream)
    ms = time_steps(torch, g.replay, 20, 3, lambda: dist.barrier())
    tm = torch.tensor([ms], device="cuda", dtype=torch.float64)
    dist.all_reduce(tm, op=dist.ReduceOp.MAX)
    ms = float(tm.item())
    out["tokens1_peer_exchange"] = {
        "us_per_layer": ms * 1e3, "tokens_per_s_per_layer": 1 / (ms * 1e-3),
        "exchange": "in the kernels: tagged 8-byte peer stores into every rank's staging buffer",
        "exchange_bytes": top_k * h * 8}
    moe_layer_ep.keep = (stage, hs, group)  # peer mappings outlive the graph replays
    return out


def lm_head_greedy_tp(torch, dist, pkg, ctx, rank, world):
    """Greedy token at a Qwen3-4B lm_head [151936, 2560] sharded by rows over `world` ranks:
    every rank streams its shard, keeps one (maximum, index) pair, the pairs cross as tagged
    words and a small kernel picks the token on every rank.  Device time, max over ranks,
    8 weight copies per rank so that the weight comes from HBM."""
    import torch.distributed._symmetric_memory as symm
    vocab, k, copies = 151936, 2560, 8
    if vocab % (8 * world):
        return {"skipped": f"{vocab} rows do not split into 8-row tiles over {world} ranks"}
    one = pkg.synth.bg128_weight(SEED_W, 60, vocab, k)
    shard, n_local, lo = pkg.shard.shard_blocks(one, vocab, k, rank, world)
    ws = [ctx.upload_weight(np.roll(shard, 544 * i), n_local, k) for i in range(copies)]
    x = torch.from_numpy(pkg.synth.activations(SEED_X, 61, 1, k)).cuda()
    stage = symm.empty((2 + 256,), dtype=torch.int64, device=f"cuda:{torch.cuda.current_device()}")
    stage.zero_()
    torch.cuda.synchronize()
    hs = symm.rendezvous(stage, dist.group.WORLD.group_name)
    group = pkg.capi.TpGroup()
    group.rank, group.world = rank, world
    for p_ in range(world):
        group.stage_peers[p_] = hs.buffer_ptrs[p_]
    tok = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    # Every kernel of the exchange runs once on a private one-rank group BEFORE the ranks meet:
    # the first launch of a kernel loads its code, and a rank still loading while its peers'
    # gathers already spin is host skew the bounded wait would have to absorb.
    solo_stage = torch.zeros((2 + 256,), dtype=torch.int64, device="cuda")
    solo = pkg.capi.TpGroup()
    solo.rank, solo.world = 0, 1
    solo.stage_peers[0] = solo_stage.data_ptr()
    ctx.matmul_argmax_tp(ws[0], x, lo, solo)
    ctx.tp_gather_token(solo, tok)
    ctx.sync()
    torch.cuda.synchronize()
    dist.barrier()

    def eager():
        for w in ws:
            ctx.matmul_argmax_tp(w, x, lo, group)
            ctx.tp_gather_token(group, tok)
    ok = True
    try:
        eager()
        ctx.sync()
    except pkg.capi.B200W4Error as exc:  # e.g. the bounded wait ran out
        print(f"tensor-parallel greedy token failed: {exc}", file=sys.stderr)
        ok = False
    torch.cuda.synchronize()
    # every rank must hold the same token (the weight copies differ, the last one counts)
    toks = [torch.zeros_like(tok) for _ in range(world)]
    dist.all_gather(toks, tok if ok else torch.full_like(tok, -2 - rank))
    same = all(int(t.item()) == int(toks[0].item()) for t in toks)
    if not same:  # the same decision on every rank: nothing is timed
        for w in ws:
            w.free()
        return {"error": "ranks disagree or the exchange failed", "ranks_agree": False}
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        ctx.set_stream(side.cuda_stream)
        with torch.cuda.graph(g, stream=side):
            eager()
    ctx.set_stream(torch.cuda.current_stream().cuda_stream)
    ms = time_steps(torch, g.replay, 10, 3, lambda: dist.barrier())
    tm = torch.tensor([ms], device="cuda", dtype=torch.float64)
    dist.all_reduce(tm, op=dist.ReduceOp.MAX)
    us = float(tm.item()) * 1e3 / copies
    lm_head_greedy_tp.keep = (stage, hs, group)
    for w in ws:
        w.free()
    return {"us_per_token": us, "gbs": algorithmic_bytes(vocab, k, 1) / us / 1e3,
            "ranks_agree": same, "token": int(toks[0].item())}


def decode_walk(torch, pkg, ctx, args):
    """The W4 matmuls of one decode token of a Qwen3-4B-shaped dense decoder (benchmark
    configuration 3): 36 layers of qkv [6144,2560], o [2560,4096], gate_up [19456,2560],
    down [2560,9728], then lm_head [151936,2560]; 2.07 GB of weights per token, every layer
    its own device buffers.  Matmul path only (no attention, norms or sampling)."""
    shapes = [(6144, 2560), (2560, 4096), (19456, 2560), (2560, 9728)]
    layers, vocab = 36, 151936
    host = [pkg.synth.bg128_weight(SEED_W, 50 + i, n, k) for i, (n, k) in enumerate(shapes)]
    ws = []
    for layer in range(layers):
        for (n, k), blk in zip(shapes, host):
            ws.append(ctx.upload_weight(np.roll(blk, 544 * layer), n, k))
    ws.append(ctx.upload_weight(pkg.synth.bg128_weight(SEED_W, 60, vocab, 2560), vocab, 2560))
    xs = {k: torch.from_numpy(pkg.synth.activations(SEED_X, k, 1, k)).cuda()
          for k in (2560, 4096, 9728)}
    ys = {n: torch.zeros((1, n), dtype=torch.float32, device="cuda")
          for n in (6144, 2560, 19456, vocab)}

    def eager():
        for w in ws:
            ctx.matmul(w, xs[w.k], ys[w.n])
    eager()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        ctx.set_stream(side.cuda_stream)
        with torch.cuda.graph(g, stream=side):
            eager()
    ctx.set_stream(torch.cuda.current_stream().cuda_stream)
    ms = time_steps(torch, g.replay, max(5, min(args.steps, 30)), 3)
    total = sum(algorithmic_bytes(w.n, w.k, 1) for w in ws)
    out = {"matmuls_per_token": len(ws), "weight_gb_per_token": total / 1e9,
           "ms_per_token": ms, "tokens_per_s": 1e3 / ms, "gbs": total / (ms * 1e-3) / 1e9}
    # the same walk restricted to one layer shape at a time (36 distinct buffers each)
    per_shape = {}
    for i, (n, k) in enumerate(shapes + [(vocab, 2560)]):
        sel = [w for w in ws if (w.n, w.k) == (n, k)]
        reps = 1 if n == vocab else 1

        def eager_shape():
            for _ in range(reps):
                for w in sel:
                    ctx.matmul(w, xs[w.k], ys[w.n])
        gs = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            ctx.set_stream(side.cuda_stream)
            with torch.cuda.graph(gs, stream=side):
                eager_shape()
        ctx.set_stream(torch.cuda.current_stream().cuda_stream)
        s_ms = time_steps(torch, gs.replay, 10, 3)
        us = s_ms * 1e3 / (len(sel) * reps)
        per_shape[f"n{n}_k{k}"] = {"us": us, "gbs": algorithmic_bytes(n, k, 1) / us / 1e3}
    out["per_shape"] = per_shape
    # greedy step at the lm_head: logits written + a library argmax kernel, against the token
    # picked in the matmul's own epilogue with no logits written (8 graph nodes each so that
    # the weight, 195 MB, is re-read from HBM every time: it exceeds L2)
    lm = ws[-1]
    tok = torch.zeros((1,), dtype=torch.int32, device="cuda")
    tok64 = torch.zeros((1,), dtype=torch.int64, device="cuda")
    greedy = {}
    for name in ("matmul_then_torch_argmax", "matmul_argmax_fused"):
        def eager_greedy():
            for _ in range(8):
                if name == "matmul_argmax_fused":
                    ctx.matmul_argmax(lm, xs[2560], tok)
                else:
                    ctx.matmul(lm, xs[2560], ys[vocab])
                    torch.argmax(ys[vocab], dim=1, out=tok64)
        eager_greedy()
        torch.cuda.synchronize()
        gg = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            ctx.set_stream(side.cuda_stream)
            with torch.cuda.graph(gg, stream=side):
                eager_greedy()
        ctx.set_stream(torch.cuda.current_stream().cuda_stream)
        greedy[name] = {"us": time_steps(torch, gg.replay, 10, 3) * 1e3 / 8}
    greedy["same_token"] = bool(int(tok.item()) == int(tok64.item()))
    out["lm_head_greedy_token"] = greedy
    for w in ws:
        w.free()
    return out


def json_only_stdout():
    """stdout carries the ONE JSON line.  Libraries that log to file descriptor 1 (NCCL with
    NCCL_DEBUG=INFO does) are sent to stderr instead: fd 1 is re-pointed at fd 2 and the
    returned file object, a duplicate of the original stdout, is what the line is printed to."""
    sys.stdout.flush()
    keep = os.dup(1)
    os.dup2(2, 1)
    return os.fdopen(keep, "w")


def decoder_leg(torch, pkg, ctx, cfg, config_text, rules):
    """A whole decoder end to end on one GPU (palm-infra_b200/decoder.py: every operator a
    libb200w4 kernel; synthetic W4G128 weights), a 256-token random prompt and 64 greedy steps.
    The reference's protocol (examples/cli_common.cpp:418-436): prefill_tps = 256 / prefill
    seconds, decode_tps = 64 / decode seconds; wall clock around synchronised regions, the
    greedy token read back every step as a sampler would."""
    dec = pkg.decoder
    prompt = np.random.default_rng(11).integers(0, cfg.vocab, 256).tolist()
    out = {"config": config_text,
           "decode_launch": "one captured CUDA graph per step (position and tokens on the "
                            "device), the token read back by the host after every step"}
    for name, rule in rules:
        weights = dec.synthetic_weights(cfg, seed=SEED_W, distinct_layers=1, lazy=True)
        model = dec.DenseDecoder(ctx, cfg, weights, capacity=384, multi_row_rule=rule)
        del weights
        model.generate(prompt, 3)  # warm every kernel and buffer
        model.generate(prompt, 3, replay=True)
        times = []
        for _ in range(3):
            model.reset()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            model.prefill(prompt)
            ctx.sync()
            t1 = time.perf_counter()
            toks = []
            for _ in range(64):
                model.replay_decode_step()
                toks.append(int(model.token.item()))  # synchronises: a host sampler's read
            t2 = time.perf_counter()
            for _ in range(64):  # the same steps with no host read in between
                model.replay_decode_step()
            torch.cuda.synchronize()
            t3 = time.perf_counter()
            model.reset()
            model.prefill(prompt)
            ctx.sync()
            t4 = time.perf_counter()
            for _ in range(16):  # eager: one host call and one launch per operator
                model.decode_step()
            ctx.sync()
            t5 = time.perf_counter()
            times.append((t1 - t0, t2 - t1, t3 - t2, (t5 - t4) * 4))
        pf, dc, dq, de = (statistics.median(t[i] for t in times) for i in range(4))
        out[name] = {"prefill_tps": 256 / pf, "decode_tps": 64 / dc, "prefill_ms": pf * 1e3,
                     "decode_ms_per_token": dc * 1e3 / 64,
                     "decode_tps_no_host_read": 64 / dq, "decode_tps_eager_launches": 64 / de,
                     "multi_row_rule": "per 32 values (the reference's)" if rule == 32 else
                                       "per 128 values"}
        model.free()
    return out


def dense_decoder(torch, pkg, ctx, args):
    """Benchmark configuration 3: the Qwen3-4B-shaped dense decoder."""
    return decoder_leg(torch, pkg, ctx, pkg.decoder.DecoderConfig.qwen3_4b(),
                       "36 layers, hidden 2560, 32/8 heads x 128, intermediate 9728, vocab 151936",
                       (("reference_rule", pkg.capi.ACT_G32), ("per128_prefill", pkg.capi.ACT_G128)))


def moe_decoder(torch, pkg, ctx, args):
    """Benchmark configuration 4: the Qwen3-30B-A3B-shaped decoder (16 GB of W4G128 weights;
    --moe-decoder, not part of the default run)."""
    return decoder_leg(torch, pkg, ctx, pkg.decoder.DecoderConfig.qwen3_30b_a3b(),
                       "48 layers, hidden 2048, 32/4 heads x 128, 128 experts x 768 top-8, "
                       "vocab 151936", (("reference_rule", pkg.capi.ACT_G32),))


def moe_decoder_235b(torch, pkg, ctx, args):
    """Benchmark configuration 5: the Qwen3-235B-A22B-shaped decoder on ONE GPU (121 GB of
    W4G128 weights in 180 GB of HBM; --moe-decoder-235b, minutes of weight generation)."""
    return decoder_leg(torch, pkg, ctx, pkg.decoder.DecoderConfig.qwen3_235b_a22b(),
                       "94 layers, hidden 4096, 64/4 heads x 128, 128 experts x 1536 top-8, "
                       "vocab 151936", (("reference_rule", pkg.capi.ACT_G32),))


def tp_decoder_leg(torch, dist, pkg, ctx, rank, world):
    """Benchmark configuration 3 over `world` GPUs (--tp-decoder; opt-in: the tensor-parallel
    driver is verified on CPU ranks only so far): 256-token prompt, 64 greedy steps, one
    launch per operator, NCCL all-gathers between the row-split matmuls.  Wall clock around
    synchronised regions, max over ranks."""
    dec = pkg.decoder
    cfg = dec.DecoderConfig.qwen3_4b()
    weights = dec.synthetic_weights(cfg, seed=SEED_W, distinct_layers=1)
    prompt = np.random.default_rng(11).integers(0, cfg.vocab, 256).tolist()
    model = dec.TensorParallelDecoder(ctx, cfg, weights, capacity=384, rank=rank, world=world)
    del weights
    model.generate(prompt, 3)
    times = []
    for _ in range(3):
        model.reset()
        torch.cuda.synchronize()
        dist.barrier()
        t0 = time.perf_counter()
        model.prefill(prompt)
        ctx.sync()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        for _ in range(64):
            model.decode_step()
        ctx.sync()
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        times.append((t1 - t0, t2 - t1))
    pf = statistics.median(t[0] for t in times)
    dc = statistics.median(t[1] for t in times)
    both = torch.tensor([pf, dc], device="cuda", dtype=torch.float64)
    dist.all_reduce(both, op=dist.ReduceOp.MAX)
    pf, dc = float(both[0].item()), float(both[1].item())
    token = int(model.token.item())
    model.free()
    return {"config": "36 layers, hidden 2560, 32/8 heads x 128, intermediate 9728, vocab 151936",
            "parallelism": f"tp{world}: row-split matmuls, attention on the rank's heads, four "
                           "NCCL all-gathers per layer",
            "prefill_tps": 256 / pf, "decode_tps": 64 / dc, "prefill_ms": pf * 1e3,
            "decode_ms_per_token": dc * 1e3 / 64, "last_token": token}


class ExtrasGuard:
    """Bounds the extra legs of a multi-GPU run on every rank: after `seconds` rank 0 prints the
    JSON line as it stands (the headline is complete before the guard starts) with a note, and
    the process ends with status 0 without running any destructor."""

    def __init__(self, rank, line, out, seconds):
        import threading
        self.rank, self.line, self.out, self.seconds = rank, line, out, seconds
        self.lock = threading.Lock()
        self.done = False
        self.timer = threading.Timer(seconds, self._expire)
        self.timer.daemon = True
        self.timer.start()

    def _expire(self):
        with self.lock:
            if self.done:
                return
            self.done = True
            if self.rank == 0:
                snapshot = dict(self.line)
                snapshot["extras_abandoned"] = (
                    f"the legs after the headline did not finish within {self.seconds:.0f} s on "
                    "some rank; this line carries what was measured before")
                self.out.write(json.dumps(snapshot) + "\n")
                self.out.flush()
            sys.stderr.write("bench: extra legs abandoned by the guard timer\n")
            sys.stderr.flush()
            os._exit(0)

    def finish(self):
        """True when the legs ended in time (the caller prints the line)."""
        with self.lock:
            if self.done:
                return False
            self.done = True
        self.timer.cancel()
        return True


def run_ours(args):
    out = json_only_stdout()
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    barrier = (lambda: dist.barrier()) if world > 1 else None

    pkg = load_package()
    ctx = pkg.capi.Context(local)
    ctx.set_stream(torch.cuda.current_stream().cuda_stream)

    # rank r owns output rows [r*N/P, (r+1)*N/P) of every weight copy (8-row tiles kept whole)
    one = pkg.synth.bg128_weight(SEED_W, 1, N_OUT, K_IN)
    shard, n_local, _ = pkg.shard.shard_blocks(one, N_OUT, K_IN, rank, world)
    weights = []
    for i in range(COPIES):  # distinct device buffers; rolling by whole blocks keeps layout
        weights.append(ctx.upload_weight(np.roll(shard, 544 * i), n_local, K_IN))
    stream_bytes = weights[0].stream_bytes

    def make_io(m):
        x = torch.from_numpy(pkg.synth.activations(SEED_X, 0, m, K_IN)).cuda()
        y_local = torch.zeros((m, n_local), dtype=torch.float32, device="cuda")
        y_full = torch.zeros((world, m, n_local), dtype=torch.float32, device="cuda")
        return x, y_local, y_full

    def make_step(m, rule=pkg.capi.ACT_G128, passes=args.passes, graph=not args.no_graph):
        """One step = `passes` walks over the weight copies.  The launches are captured in
        a CUDA graph once (decode loops are launch-bound otherwise) and replayed."""
        x, y_local, y_full = make_io(m)

        def eager():
            for _ in range(passes):
                for w in weights:
                    ctx.matmul(w, x, y_local, rule=rule)
                    if world > 1:
                        dist.all_gather_into_tensor(y_full, y_local)
        if not graph:
            return eager
        eager()  # warm every kernel variant and NCCL before capture
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            ctx.set_stream(side.cuda_stream)
            with torch.cuda.graph(g, stream=side):
                eager()
        ctx.set_stream(torch.cuda.current_stream().cuda_stream)
        return g.replay

    def all_ranks_agree(flag):
        t = torch.tensor([1 if flag else 0], device="cuda", dtype=torch.int32)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item())

    def make_peer_step(passes=args.passes):
        """The same walk with the exchange inside the kernels: the GEMV's epilogue stores
        (value, exchange number) words into every rank's staging buffer over peer mappings
        (symmetric memory) and a small gather kernel waits, bounded, for all of them and
        unpacks the row.  Returns None when symmetric memory is not available."""
        try:
            import torch.distributed._symmetric_memory as symm
            stage = symm.empty((2 + 16 * N_OUT,), dtype=torch.int64, device=f"cuda:{local}")
            stage.zero_()
            torch.cuda.synchronize()
            hs = symm.rendezvous(stage, dist.group.WORLD.group_name)
        except Exception as exc:  # no peer mappings on this box: the NCCL walk stands
            print(f"in-kernel exchange unavailable: {exc}", file=sys.stderr)
            return None
        group = pkg.capi.TpGroup()
        group.rank, group.world = rank, world
        for p_ in range(world):
            group.stage_peers[p_] = hs.buffer_ptrs[p_]
        m = args.rows
        x, y_local, y_full = make_io(m)
        y_row = torch.zeros((m, N_OUT), dtype=torch.float32, device="cuda")
        # both kernels of the exchange once on a private one-rank group before the ranks meet
        # (a first launch loads the kernel's code: host skew the bounded wait should not pay)
        solo_stage = torch.zeros((2 + 16 * n_local,), dtype=torch.int64, device="cuda")
        solo = pkg.capi.TpGroup()
        solo.rank, solo.world = 0, 1
        solo.stage_peers[0] = solo_stage.data_ptr()
        y_solo = torch.zeros((m, n_local), dtype=torch.float32, device="cuda")
        ctx.matmul_tp(weights[0], x, n_local, 0, solo)
        ctx.tp_gather(solo, y_solo, n_local)
        ctx.sync()
        torch.cuda.synchronize()
        dist.barrier()
        # eagerly, twice (both halves of the staging buffer): the gathered row must equal the
        # NCCL all-gather of the shards, bit for bit
        same = True
        for w in weights[:2]:
            ctx.matmul(w, x, y_local)
            dist.all_gather_into_tensor(y_full, y_local)
            try:
                ctx.matmul_tp(w, x, N_OUT, rank * n_local, group)
                ctx.tp_gather(group, y_row, N_OUT)
                ctx.sync()
            except pkg.capi.B200W4Error as exc:  # e.g. the bounded wait ran out
                print(f"in-kernel exchange failed: {exc}", file=sys.stderr)
                same = False
            torch.cuda.synchronize()
            same = same and torch.equal(y_full.permute(1, 0, 2).reshape(m, N_OUT), y_row)
        if not all_ranks_agree(same):  # never time a path whose result differs
            print("in-kernel exchange and all-gather disagree: not used", file=sys.stderr)
            return None

        def eager():
            for _ in range(passes):
                for w in weights:
                    ctx.matmul_tp(w, x, N_OUT, rank * n_local, group)
                    ctx.tp_gather(group, y_row, N_OUT)
        eager()
        torch.cuda.synchronize()
        dist.barrier()
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            ctx.set_stream(side.cuda_stream)
            with torch.cuda.graph(g, stream=side):
                eager()
        ctx.set_stream(torch.cuda.current_stream().cuda_stream)
        keep = (stage, hs, group, y_row)  # peer mappings live as long as the step

        def replay():
            g.replay()
            return keep
        return replay

    def make_list_step_tp(passes=args.passes, dependent=False):
        """The walk as the persistent list kernel on every rank's row shards: each GEMV's
        values go, tagged and as plain fp32, into EVERY rank's buffers over peer mappings
        (symmetric memory) from the kernel's epilogue -- the all-gather is those stores -- so
        every rank ends with the full rows and an op that consumes an earlier op's row polls
        its own scratch.  No collective call, no extra launch.  Checked bit for bit against
        the shards' NCCL all-gather before it is timed.  Returns (step, ops per launch) or
        None."""
        try:
            import torch.distributed._symmetric_memory as symm
            n_ops = COPIES * passes
            rows = symm.empty((COPIES, N_OUT), dtype=torch.float32, device=f"cuda:{local}")
            rows.fill_(-1.0)
            table = pkg.capi.Chain.shard_table(
                [(rank * n_local, N_OUT, None) for _ in range(n_ops)])
            words = pkg.capi.Chain.scratch_words(table)
            scratch = symm.empty((words,), dtype=torch.int64, device=f"cuda:{local}")
            scratch.zero_()
            torch.cuda.synchronize()
            hr = symm.rendezvous(rows, dist.group.WORLD.group_name)
            hs = symm.rendezvous(scratch, dist.group.WORLD.group_name)
        except Exception as exc:  # no peer mappings on this box
            print(f"tensor-parallel list unavailable: {exc}", file=sys.stderr)
            return None
        table = pkg.capi.Chain.shard_table(
            [(rank * n_local, N_OUT,
              [hr.buffer_ptrs[p] + (i % COPIES) * N_OUT * 4 for p in range(world)])
             for i in range(n_ops)])
        group = pkg.capi.TpGroup()
        group.rank, group.world = rank, world
        for p_ in range(world):
            group.stage_peers[p_] = hs.buffer_ptrs[p_]
        x, y_local, y_full = make_io(1)
        if dependent:
            ops = [dict(w=weights[i % COPIES], x=x) if i % DEP_RESTART == 0 else
                   dict(w=weights[i % COPIES], x_from=i - 1) for i in range(n_ops)]
        else:
            ops = [dict(w=weights[i % COPIES], x=x) for i in range(n_ops)]
        chain = pkg.capi.Chain(ctx, ops, table, group)
        dist.barrier()
        ok = True
        try:
            chain.run()
            ctx.sync()
        except pkg.capi.B200W4Error as exc:
            print(f"tensor-parallel list failed: {exc}", file=sys.stderr)
            ok = False
        torch.cuda.synchronize()
        dist.barrier()  # every rank's stores of the run have landed
        if ok:  # full rows on this rank == all-gather of the shards' rows, bit for bit
            cur = x
            for i in range(COPIES if dependent else 2):
                if i % DEP_RESTART == 0:
                    cur = x
                ctx.matmul(weights[i], cur[:, :K_IN].contiguous(), y_local)
                dist.all_gather_into_tensor(y_full, y_local)
                torch.cuda.synchronize()
                want = y_full.permute(1, 0, 2).reshape(1, N_OUT).contiguous()
                ok = ok and torch.equal(rows[i:i + 1].view(torch.int32), want.view(torch.int32))
                if dependent:
                    cur = want.clone()
        if not all_ranks_agree(ok):
            print("tensor-parallel list and all-gather disagree: not used", file=sys.stderr)
            return None
        keep = (rows, scratch, hr, hs, group, table, chain)

        def step():
            for _ in range(RUNS_PER_STEP):
                chain.run()
            return keep
        return step, n_ops

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    if args.moe_only:  # one leg alone (profiling commands)
        if rank == 0:
            out.write(json.dumps({"moe30b_layer": moe_layer(torch, pkg, ctx, args)}) + "\n")
            out.flush()
        ctx.close()
        return

    # ---- headline: M=1, resident inputs -------------------------------------------------
    alg = algorithmic_bytes(N_OUT, K_IN, 1)
    peak, peak_kind = measured_peaks()
    use_list = world == 1 and args.rows == 1 and not args.per_launch
    variants = {}
    if use_list:
        # One step = RUNS_PER_STEP launches of the persistent kernel, each a list of
        # passes * COPIES GEMVs of one activation vector (the list shares its quantisation, as
        # the reference's batch entry point does for identical inputs).
        x, _, _ = make_io(1)
        ys = torch.zeros((COPIES, N_OUT), dtype=torch.float32, device="cuda")
        n_ops = COPIES * args.passes
        ops = [dict(w=weights[i % COPIES], x=x, y=ys[i % COPIES:i % COPIES + 1])
               for i in range(n_ops)]
        chain = pkg.capi.Chain(ctx, ops)
        runs = RUNS_PER_STEP

        def step():
            for _ in range(runs):
                chain.run()
        l0 = ctx.launches
        step()
        launches_per_step = ctx.launches - l0
        ctx.sync()
        # the list's rows against the one-launch-per-GEMV kernel's, bit for bit
        y_one = torch.zeros((1, N_OUT), dtype=torch.float32, device="cuda")
        for i in (0, COPIES - 1):
            ctx.matmul(weights[i], x, y_one)
            ctx.sync()
            assert torch.equal(ys[i:i + 1], y_one), "list kernel and per-launch kernel differ"
        with ClockSampler(local) as clocks:
            ms = time_steps(torch, step, args.steps, args.warmup, barrier)
        gemvs = n_ops * runs
        kernel_name, launch_desc = "gemv_chain_kernel", (
            f"{runs} launches of one persistent cooperative kernel per step, each a list of "
            f"{n_ops} GEMVs on one activation vector")
        alg_per_launch = alg * n_ops
        launch_us = ms * 1e3 / runs
        traffic = NCU_DRAM_BYTES_PER_GEMV_CHAIN * n_ops
        exchange = "none (one GPU)"
        nccl_ms = None
    else:
        l0 = ctx.launches
        make_step(args.rows, rule=args.act_rule, graph=False)()
        launches_per_step = ctx.launches - l0
        step = make_step(args.rows, rule=args.act_rule)
        with ClockSampler(local) as clocks:
            ms = time_steps(torch, step, args.steps, args.warmup, barrier)
        ms = max_over_ranks(ms)
        exchange = "none (one GPU)" if world == 1 else "NCCL all-gather after every GEMV"
        nccl_ms = None
        gemvs = COPIES * args.passes
        kernel_name = "gemv_w4a8_kernel"
        launch_desc = None
        alg_per_launch = algorithmic_bytes(n_local, K_IN, 1)
        launch_us = ms * 1e3 / gemvs
        traffic = NCU_DRAM_BYTES_PER_LAUNCH if world == 1 else None
        if world > 1 and args.rows <= 8 and not args.no_graph and world <= 8:
            nccl_ms = ms
            peer_step = make_peer_step()
            if peer_step is not None:
                p_ms = max_over_ranks(time_steps(torch, peer_step, args.steps, args.warmup,
                                                 barrier))
                variants["one_launch_per_gemv_exchange_in_kernels"] = {
                    "value": gemvs * alg / (p_ms * 1e-3) / 1e9, "unit": UNIT,
                    "us_per_gemv": p_ms * 1e3 / gemvs,
                    "what": "GEMV kernel stores tagged words to every rank, gather kernel after it"}
                ms = p_ms
                launch_us = ms * 1e3 / gemvs
                exchange = ("in the GEMV kernel: tagged 8-byte peer stores into every rank's "
                            "staging buffer, gather kernel with a bounded wait")
            tp_list = make_list_step_tp() if args.rows == 1 else None
            if tp_list is not None:
                tp_step, n_ops = tp_list
                with ClockSampler(local) as clocks:
                    ms = max_over_ranks(time_steps(torch, tp_step, args.steps, args.warmup,
                                                   barrier))
                launches_per_step = RUNS_PER_STEP
                gemvs = n_ops * RUNS_PER_STEP
                kernel_name = "gemv_chain_kernel"
                launch_desc = (f"{RUNS_PER_STEP} launches of one persistent cooperative kernel "
                               f"per step and rank, each a list of {n_ops} GEMVs on this "
                               f"rank's row shards")
                alg_per_launch = algorithmic_bytes(n_local, K_IN, 1) * n_ops
                launch_us = ms * 1e3 / RUNS_PER_STEP
                exchange = ("in the list kernel's epilogue: every value stored, tagged and "
                            "plain, into every rank's buffers over peer mappings")
                dep = make_list_step_tp(dependent=True)
                if dep is not None:
                    d_ms = max_over_ranks(time_steps(torch, dep[0], max(3, min(args.steps, 10)),
                                                     3, barrier))
                    variants["list_with_dependent_gemvs"] = {
                        "value": dep[1] * RUNS_PER_STEP * alg / (d_ms * 1e-3) / 1e9,
                        "unit": UNIT, "us_per_gemv": d_ms * 1e3 / (dep[1] * RUNS_PER_STEP),
                        "what": "each GEMV reads the full row of its predecessor, which every "
                                "rank's epilogue stored into this rank's scratch"}
    value = gemvs * alg / (ms * 1e-3) / 1e9
    achieved = alg_per_launch / (launch_us * 1e-6) / 1e9

    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "s8*s4->s32, f32 scale chain", "data": "synthetic",
            "config": workload_config(world, args.passes, not args.no_graph),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic,
                         "kernel": kernel_name, "peak_kind": peak_kind,
                         "algorithmic_bytes_per_launch": alg_per_launch,
                         "avg_launch_us": launch_us},
            "clocks": clocks.summary(),
            "gpu_launches": launches_per_step * args.steps}
    line["config"]["gemvs_per_step"] = gemvs
    line["config"]["exchange"] = exchange
    if launch_desc:
        line["config"]["launch"] = launch_desc
    if world > 1:
        line["config"]["parallelism"] += f"; timed exchange: {exchange}"
    if nccl_ms is not None:
        line["nccl_allgather_variant"] = {
            "value": COPIES * args.passes * alg / (nccl_ms * 1e-3) / 1e9, "unit": UNIT,
            "ms_per_step": nccl_ms,
            "what": "one launch per GEMV, NCCL all-gather of y after every GEMV"}
    if world > 1 and variants:
        line["variants"] = variants

    if use_list and not args.headline_only:
        # ---- the same GEMVs two other ways ------------------------------------------------
        # (a) every GEMV consumes the first K outputs of its predecessor (a decode step's data
        #     dependency; the chain restarts from x every DEP_RESTART GEMVs to stay inside fp32)
        dep_ops = [dict(w=weights[i % COPIES], x=x) if i % DEP_RESTART == 0 else
                   dict(w=weights[i % COPIES], x_from=i - 1) for i in range(n_ops)]
        dep = pkg.capi.Chain(ctx, dep_ops)
        d_ms = time_steps(torch, dep.run, max(3, min(args.steps, 20)), 3)
        variants["list_with_dependent_gemvs"] = {
            "value": n_ops * alg / (d_ms * 1e-3) / 1e9, "unit": UNIT,
            "us_per_gemv": d_ms * 1e3 / n_ops,
            "what": "each GEMV reads its predecessor's output (tagged words, polled on the device)"}
        dep.free()
        # (b) one kernel launch per GEMV, CUDA graph replay with programmatic dependent launch
        p_ms = time_steps(torch, make_step(1), max(3, min(args.steps, 20)), 3)
        variants["one_launch_per_gemv"] = {
            "value": COPIES * args.passes * alg / (p_ms * 1e-3) / 1e9, "unit": UNIT,
            "us_per_gemv": p_ms * 1e3 / (COPIES * args.passes), "kernel": "gemv_w4a8_kernel"}
        line["variants"] = variants

    if not args.headline_only:
        # ---- e2e: the same step from HOST buffers ------------------------------------------
        xh = torch.from_numpy(pkg.synth.activations(SEED_X, 0, 1, K_IN)).pin_memory()
        if use_list:
            # x from pinned host memory every launch; every GEMV's row is stored by the kernel
            # straight into pinned host memory (its y pointer is the mapped host buffer)
            yh = torch.zeros((n_ops, N_OUT), dtype=torch.float32).pin_memory()
            yh_t = [yh[i:i + 1] for i in range(n_ops)]
            e_ops = [dict(w=weights[i % COPIES], y=yh_t[i]) for i in range(n_ops)]
            e_chain = pkg.capi.Chain(ctx, e_ops)
            none_y = np.zeros(0, dtype=np.float32)
            call = e_chain.bind_run_host(xh.numpy().reshape(-1), none_y)

            def host_step():
                for _ in range(runs):
                    call()
            host_step()
            assert np.array_equal(yh[COPIES - 1].numpy(), ys[COPIES - 1].cpu().numpy()), \
                "host-buffer rows differ from the device-resident run"
            h2d, d2h = runs * K_IN * 4, runs * n_ops * N_OUT * 4
            api = ("b2w4_chain_run_host: pinned host x uploaded per launch, every GEMV's row "
                   "stored into pinned host memory by the kernel, one synchronisation per list")
        else:
            yh = torch.zeros((1, n_local), dtype=torch.float32).pin_memory()
            xn, yn = xh.numpy(), yh.numpy()
            calls = [ctx.bind_matmul_host(w, xn, yn) for w in weights]

            def host_step():
                for _ in range(args.passes):
                    for call in calls:
                        call()
            h2d, d2h = gemvs * K_IN * 4 * world, gemvs * N_OUT * 4
            api = "b2w4_matmul_host (pinned host x and y, synchronous)"
        for _ in range(args.warmup):
            host_step()
        if barrier:
            barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            host_step()
        e2e_s = max_over_ranks((time.perf_counter() - t0) / args.steps)
        line["e2e"] = {"value": gemvs * alg / e2e_s / 1e9, "unit": UNIT,
                       "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                       "ms_per_step": e2e_s * 1e3, "api": api}
        if use_list:
            # one synchronous host call per GEMV, for comparison
            yh1 = torch.zeros((1, N_OUT), dtype=torch.float32).pin_memory()
            calls = [ctx.bind_matmul_host(w, xh.numpy(), yh1.numpy()) for w in weights]
            for c in calls:
                c()
            t0 = time.perf_counter()
            for _ in range(8):
                for c in calls:
                    c()
            per = (time.perf_counter() - t0) / (8 * COPIES)
            line["e2e"]["one_host_call_per_gemv"] = {
                "value": alg / per / 1e9, "unit": UNIT, "us_per_call": per * 1e6,
                "api": "b2w4_matmul_host"}
            e_chain.free()

    if rank == 0 and world == 1 and not args.headline_only:
        # ---- sweep: batched decode and prefill on the same weight -----------------------
        sweep = {}
        for m in (4, 8, 16, 64, 256):
            s_ms = time_steps(torch, make_step(m, passes=1), max(3, min(args.steps, 25)), 3)
            per = s_ms * 1e-3 / COPIES
            tflops = 2.0 * m * N_OUT * K_IN / per / 1e12
            gbs = algorithmic_bytes(N_OUT, K_IN, m) / per / 1e9
            t_peak, t_kind = measured_tensor_peak()
            sweep[f"m{m}"] = {"us_per_matmul": per * 1e6, "gbs": gbs, "tflops": tflops,
                              "tokens_per_s": m / per,
                              # the binding roofline of the shape: weight streaming up to 64
                              # rows, the tensor pipe at 256
                              "roofline": ({"bound": "tensor", "frac": tflops / t_peak,
                                            "peak": t_peak, "unit": "TFLOP/s", "peak_kind": t_kind}
                                           if m >= 256 else
                                           {"bound": "hbm", "frac": gbs / peak, "peak": peak,
                                            "unit": "GB/s", "peak_kind": peak_kind})}
        # the reference's M > 1 rule (one activation scale per 32 values) on the prefill shape
        s_ms = time_steps(torch, make_step(256, rule=pkg.capi.ACT_G32, passes=1),
                          max(3, min(args.steps, 25)), 3)
        per = s_ms * 1e-3 / COPIES
        sweep["m256_per32_rule"] = {"us_per_matmul": per * 1e6,
                                    "tflops": 2.0 * 256 * N_OUT * K_IN / per / 1e12,
                                    "tokens_per_s": 256 / per}
        sweep["dense4b_decode_matmul_walk"] = decode_walk(torch, pkg, ctx, args)
        sweep["moe30b_layer"] = moe_layer(torch, pkg, ctx, args)
        line["sweep"] = sweep
        line["gpu_reference"] = gpu_reference(torch, pkg, args, value,
                                              sweep["m256"]["us_per_matmul"])
        line["dense_decoder_4b"] = dense_decoder(torch, pkg, ctx, args)
        if args.moe_decoder:
            line["moe_decoder_30b_a3b"] = moe_decoder(torch, pkg, ctx, args)
        if args.moe_decoder_235b:
            line["moe_decoder_235b_a22b"] = moe_decoder_235b(torch, pkg, ctx, args)

        # ---- CPU baseline: the reference's own kernel on this box's host cores ----------
        probe, kind, cores, isa = cpu_gemv_seconds(pkg, 1, 16, 8)
        repeat = max(32, min(20000, int(12.0 / max(probe, 1e-6))))
        sec, kind, cores, isa = cpu_gemv_seconds(pkg, 1, 16, repeat)
        line["cpu_baseline"] = {
            "value": alg / sec / 1e9, "unit": UNIT, "cores": cores, "kind": kind,
            "sample": f"{repeat} GEMVs rotating 16 weight copies, isa {isa}, "
                      f"W4A32 arithmetic ({sec * 1e3:.3f} ms per GEMV)"}

    # The legs below are extras of a multi-GPU run; each ends in collectives, and a rank that
    # does not come back from one would hold every other rank in the next collective until the
    # library's own time-out (ten minutes).  A timer on every rank bounds them: when it runs
    # out, rank 0 prints the line with what is measured and every rank leaves.
    guard = None
    if world > 1 and not args.headline_only:
        guard = ExtrasGuard(rank, line, out, seconds=300.0)
    if world > 1 and not args.headline_only and 128 % world == 0:
        ep = moe_layer_ep(torch, dist, pkg, ctx, rank, world)  # every rank takes part
        line["moe30b_layer_ep"] = ep
    if world > 1 and not args.headline_only:
        if world >= 8:
            # At 8 ranks this leg failed in both runs it had: ranks reported the time-out
            # status of the bounded wait, and in the second run one rank never came back from
            # the leg.  The cause is not established; the leg is left out there.
            line["lm_head_greedy_token_tp"] = {
                "skipped": "not run at 8 ranks: it failed there twice (time-out status; one "
                           "rank not returning), cause not established"}
        else:
            try:
                line["lm_head_greedy_token_tp"] = lm_head_greedy_tp(torch, dist, pkg, ctx, rank,
                                                                    world)
            except Exception as exc:  # no symmetric memory on this box
                line["lm_head_greedy_token_tp"] = {"skipped": str(exc)[:200]}

    if world > 1 and args.tp_decoder and not args.headline_only:
        try:
            line["dense_decoder_4b_tp"] = tp_decoder_leg(torch, dist, pkg, ctx, rank, world)
        except Exception as exc:
            line["dense_decoder_4b_tp"] = {"error": str(exc)[:300]}

    if guard is not None and not guard.finish():
        return  # the timer is printing the line and ending the process
    if rank == 0:
        out.write(json.dumps(line) + "\n")
        out.flush()
    if world > 1:
        # Tear-down order matters with NCCL work captured in CUDA graphs: drain the device,
        # meet the other ranks, then leave without running NCCL's destructors (they can wait
        # for ever on a communicator a captured graph still references).
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)
    for w in weights:
        w.free()
    ctx.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--passes", type=int, default=PASSES,
                    help="walks over the weight copies per step")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch eagerly instead of replaying a CUDA graph (profiling)")
    ap.add_argument("--rows", type=int, default=1,
                    help="activation rows of the timed matmul (1 = the headline GEMV; other "
                         "values are for profiling the batched kernels)")
    ap.add_argument("--act-rule", type=int, default=128, choices=[128, 32],
                    help="activation rule of the --rows matmul (32 = the reference's rule for "
                         "several rows; profiling)")
    ap.add_argument("--moe-only", action="store_true",
                    help="run only the MoE layer leg of the sweep (single GPU)")
    ap.add_argument("--per-launch", action="store_true",
                    help="time the one-launch-per-GEMV kernel as the headline instead of the "
                         "persistent list kernel (profiling)")
    ap.add_argument("--moe-decoder", action="store_true",
                    help="also run the 30B-A3B-shaped mixture-of-experts decoder end to end "
                         "(uploads 16 GB of synthetic weights; single GPU)")
    ap.add_argument("--tp-decoder", action="store_true",
                    help="multi-GPU runs: also run the 4B-shaped dense decoder tensor-parallel "
                         "over the ranks (opt-in)")
    ap.add_argument("--moe-decoder-235b", action="store_true",
                    help="also run the 235B-A22B-shaped decoder end to end on one GPU (121 GB "
                         "of synthetic weights, several minutes)")
    ap.add_argument("--headline-only", action="store_true",
                    help="skip the e2e, sweep and CPU-baseline legs (profiling)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
