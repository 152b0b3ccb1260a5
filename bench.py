#!/usr/bin/env python
"""BERT-large S=384 encoder throughput on B200 through the sm_100a plugin kernels.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--dtype int8|fp16] [--impl b200|reference]
    python bench.py --sweep                      # kernel sweep against the rooflines (one GPU), one JSON object

One step = one forward pass of the 24-layer BERT-large encoder (EmbLayerNorm + 24 x [FC(QKV), fused MHA, FC,
SkipLayerNorm, FC+GELU, FC, SkipLayerNorm]) over ONE global batch of 64 synthetic sequences of 384 tokens, split
evenly over the N GPUs (64 / 32 / 16 / 8 sequences per GPU: strong scaling, no collective on the data path; the time
is the max over ranks). Prints ONE JSON line (rank 0). Sub-objects of that line: `weak` (64 sequences per GPU, N > 1
only), `fp16` (the same network in FP16), `config4` (packed variable-length batch of 256 sequences, lengths uniform
in [32, 384], sharded by token count), `plugin_path` (the FP16 network driven through the IPluginV3 enqueue() calls
instead of the C++ layer loop, one GPU only).

`--impl reference` times the CPU restatement of the reference math (oracle/cpu_encoder.py, FP32, all host cores) on a
bounded sample of the same workload: the reference plugins have no CPU implementation and neither TensorRT nor
ONNX-Runtime is installed, so this port is the CPU arm.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYERS, HIDDEN, HEADS, FFN, SEQ, BATCH = 24, 1024, 16, 4096, 384, 64
FLOPS_PER_SEQ_LAYER_FC = 24 * HIDDEN * HIDDEN * SEQ      # 2*S*(3E*E + E*E + 2*E*F), F = 4E
FLOPS_PER_SEQ_LAYER_MHA = 4 * SEQ * SEQ * HIDDEN
L2_BYTES = 126e6
# dram__bytes_read.sum + dram__bytes_write.sum per FC launch at 64 sequences per GPU, mean of the four shapes of a
# layer, from one `ncu --set full` capture of a 2-layer run (a profiler reading: it cannot be measured by the bench)
FC_DRAM_BYTES_PER_LAUNCH_INT8 = 69.4e6


def _peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return dict(hbm=p["hbm_gbs"], tc=p["bf16_tflops"], tc_sustained=p["bf16_tflops_sustained"], source="measured")
    except Exception:
        return dict(hbm=6650.0, tc=1590.0, tc_sustained=1400.0, source="fallback")


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs (read only)."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._halt = threading.Event()

    def run(self):
        try:
            import pynvml as nv

            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}
            while not self._halt.is_set():
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                self.reasons.update(k for k, bit in names.items() if r & bit)
                time.sleep(0.005)
        except Exception as e:  # NVML missing: report that instead of clocks
            self.reasons.add(f"nvml_unavailable:{type(e).__name__}")

    def stop(self):
        self._halt.set()
        self.join(timeout=2)
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def cpu_forward_rate(batch_hint=None, budget_s=15.0, steps=1, warmup=0):
    """Sequences/s of the FP32 torch-CPU port on a bounded sample (full 24 layers, S=384)."""
    import torch

    from oracle import cpu_encoder as ce

    # all the host threads this process may use (torchrun exports OMP_NUM_THREADS=1 to its ranks; only rank 0 runs this)
    torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    p = ce.random_params(LAYERS, HIDDEN, HEADS, FFN, seed=0)
    g = torch.Generator().manual_seed(1)

    def run(b):
        ids = torch.randint(0, 30522, (b, SEQ), generator=g)
        seg = (torch.arange(SEQ)[None] >= torch.randint(1, SEQ, (b, 1), generator=g)).long()
        t0 = time.perf_counter()
        ce.forward(p, ids, seg, b, SEQ)
        return time.perf_counter() - t0

    if batch_hint is None:
        t1 = run(1)
        batch_hint = max(1, min(64, int(budget_s / max(t1, 1e-3))))
    for _ in range(warmup):
        run(batch_hint)
    times = [run(batch_hint) for _ in range(steps)]
    return batch_hint, times, torch.get_num_threads()


def _workload(dtype):
    if dtype == "int8":
        return ("BERT-large encoder, 24 layers, hidden 1024, 16 heads x 64, FFN 4096, seq 384, one global batch of 64 "
                "split evenly over the GPUs (benchmark configuration 3); explicit INT8 with amax/127 scales from one seeded "
                "calibration batch")
    return ("BERT-large encoder, 24 layers, hidden 1024, 16 heads x 64, FFN 4096, seq 384, one global batch of 64 split "
            "evenly over the GPUs, FP16")


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    b = 2
    _, times, cores = cpu_forward_rate(batch_hint=b, steps=args.steps, warmup=args.warmup)
    ms = 1e3 * sum(times) / len(times)
    value = b / (ms / 1e3)
    sample = (f"{b} of the {BATCH} sequences per step (24 layers, S=384), FP32 torch-CPU port of the reference math "
              "(the reference has no CPU implementation of its plugins; the same network in FP32)")
    # same metric / unit / workload as the GPU arm, so that the two lines divide
    line = {
        "impl": "reference", "metric": f"BERT-large s384 {args.dtype.upper()} encoder sequences/s", "value": value, "unit": "seq/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": _workload(args.dtype), "layers": LAYERS, "global_batch": BATCH, "seq_len": SEQ,
                   "cpu_arm": "bounded sample of the workload on the host cores"},
        "cpu_baseline": {"value": value, "unit": "seq/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "seq/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def _events():
    import torch

    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def time_forward(fn, steps, warmup, world, dist):
    """W warm-up calls, then K calls between two CUDA events on the launching stream; barrier + synchronize on both
    sides when several ranks run."""
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = _events()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    return e0.elapsed_time(e1) / steps


def step_latency(fn, n=100):
    """Median and 99th percentile of single steps, each between its own pair of CUDA events (N = 1 only; the
    convention of the reference's own reporting: samples/common/sampleReporting.cpp:232-265)."""
    import torch

    evs = [_events() for _ in range(n)]
    torch.cuda.synchronize()
    for e0, e1 in evs:
        e0.record()
        fn()
        e1.record()
    torch.cuda.synchronize()
    t = sorted(e0.elapsed_time(e1) for e0, e1 in evs)
    return {"median": t[len(t) // 2], "p99": t[min(len(t) - 1, int(0.99 * len(t)))], "min": t[0], "samples": n}


def kernel_breakdown(enc, ids, seg, cu, out, profile_steps=3):
    """`profile_steps` forwards with every kernel bracketed by CUDA events (same inputs, same stream) to split the
    step by kernel kind. The brackets cost the overlap of consecutive kernels (programmatic dependent launch), so the
    per-kind times add up to more than the step; they are not part of the reported step time."""
    import torch

    kind_ms, kind_n = (C.c_float * 5)(), (C.c_int32 * 5)()
    enc.enable_timing(True)
    enc.forward(ids, seg, cu, SEQ, out=out)  # creates the events
    torch.cuda.synchronize()
    for _ in range(profile_steps):
        enc.forward(ids, seg, cu, SEQ, out=out)
        enc.read_timing(kind_ms, kind_n)  # synchronises, then adds this forward's per-kind times
    enc.enable_timing(False)
    return [v / profile_steps for v in kind_ms], [v // profile_steps for v in kind_n]


def time_e2e(enc, ids, seg, cu, steps, warmup, world, dist, out_dev):
    """Same step through the host-buffer entry point of the C ABI (the pipelined form a serving loop uses): every step
    copies ids / segment ids / cu_seqlens from pinned host memory, runs the encoder and copies the FP16 hidden states
    into pinned host memory. The output copy of step i runs on a second stream and overlaps step i + 1 (two
    alternating output buffers); the timed region ends when the last copy has landed."""
    import torch

    ids_h, seg_h, cu_h = ids.cpu().pin_memory(), seg.cpu().pin_memory(), cu.cpu().pin_memory()
    outs_dev = [out_dev, torch.empty_like(out_dev)]
    outs_h = [torch.empty(out_dev.shape, dtype=torch.float16).pin_memory() for _ in range(2)]
    copy_stream = torch.cuda.Stream()
    cur = torch.cuda.current_stream()
    for i in range(warmup):
        enc.forward_host_async(ids_h, seg_h, cu_h, SEQ, outs_dev[i & 1], outs_h[i & 1], copy_stream, i & 1)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = _events()
    e0.record()
    for i in range(steps):
        enc.forward_host_async(ids_h, seg_h, cu_h, SEQ, outs_dev[i & 1], outs_h[i & 1], copy_stream, i & 1)
    cur.wait_stream(copy_stream)  # the timed region includes the last device-to-host copy
    e1.record()
    enc.wait_host(0)
    enc.wait_host(1)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    h2d = ids_h.numel() * 4 + seg_h.numel() * 4 + cu_h.numel() * 4
    d2h = outs_h[0].numel() * 2
    return ms, h2d, d2h


def probe_mma_rate(T, type_id, k_blocks=20000):
    """TOP/s the tensor pipes sustain for the FC kernels' MMA shape with operands resident in shared memory."""
    import torch

    v = C.c_float(0)
    T._lib.check(T._lib.lib.bert_b200_probe_mma_rate(C.c_void_p(torch.cuda.current_stream().cuda_stream), type_id, k_blocks,
                                                     None, C.byref(v)), "probe_mma_rate")
    return float(v.value)


def rotating(make, nbytes_each, min_total=2.5 * L2_BYTES):
    """Enough independent copies of a kernel's operands that consecutive launches never find theirs in the L2."""
    n = max(2, int(min_total // max(nbytes_each, 1)) + 1)
    return [make() for _ in range(min(n, 64))]


def time_rotating(launch, sets, iters=None):
    import torch

    iters = iters or max(20, 2 * len(sets))
    for i in range(len(sets)):
        launch(sets[i])
    torch.cuda.synchronize()
    e0, e1 = _events()
    e0.record()
    for i in range(iters):
        launch(sets[i % len(sets)])
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _product_lib():
    from tensorrt_b200._lib import lib

    return lib


def time_rotating_graph(launch, sets, reps=10):
    """The same rotation captured once into a CUDA graph (one launch per operand set) and replayed: per-launch time
    without the host's share (Python, ctypes, tensor-map encoding), which for launches of 10-30 us is as large as the
    kernel. `launch(set, stream_handle)` must enqueue on the given stream."""
    import torch

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for t in sets:
            launch(t, side.cuda_stream)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for t in sets:
                launch(t, side.cuda_stream)
    torch.cuda.current_stream().wait_stream(side)
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = _events()
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (reps * len(sets))


def isolated_skip_ln(T, dev, tokens, ld, int8, bias=True):
    """SkipLayerNorm (+ bias) alone at `tokens` x `ld`, operands rotated beyond the L2: GB/s of algorithmic traffic."""
    import torch

    g = torch.ones(ld, device=dev).half()
    b = torch.zeros(ld, device=dev).half()
    elem = 1 if int8 else 2

    def make():
        if int8:
            x = torch.randint(-127, 127, (tokens, ld), device=dev, dtype=torch.int8)
            return x, torch.randint(-127, 127, (tokens, ld), device=dev, dtype=torch.int8), torch.empty_like(x)
        x = torch.randn(tokens, ld, device=dev).half()
        return x, torch.randn(tokens, ld, device=dev).half(), torch.empty_like(x)

    sets = rotating(make, 3 * tokens * ld * elem)
    # replayed from a CUDA graph: up to a few hundred thousand tokens the launch is shorter than the host's enqueue
    if int8:
        ms = time_rotating_graph(lambda s, st: T.skip_layer_norm_dqq(s[0], s[1], g, b, b if bias else None, 0.02, 0.02, 40.0, out=s[2]), sets)
    else:
        ms = time_rotating_graph(lambda s, st: T.skip_layer_norm(s[0], s[1], g, b, bias=b if bias else None, out=s[2]), sets)
    return ms, 3 * tokens * ld * elem / (ms * 1e-3) / 1e9


class PluginEncoder:
    """The FP16 network wired from plugin OBJECTS in the fixed [S, B, E] layout, driven through their
    IPluginV3OneRuntime::enqueue (the C harness stands in for TensorRT): per layer FC -> QKVToContext v4 -> FC ->
    SkipLayerNorm v5 -> FC(+GELU) -> FC -> SkipLayerNorm v5, what a TensorRT engine built from these plugins executes."""

    def __init__(self, params, batch, dev):
        import numpy as np
        import torch

        from tensorrt_b200 import plugin_harness as H

        self.H, self.B, self.dev = H, batch, dev
        E, N, F = params.hidden, params.heads, params.ffn
        f32 = lambda t: t.detach().float().cpu().numpy()
        FC, QKV, SKIP = "CustomFCPluginDynamic", "CustomQKVToContextPluginDynamic", "CustomSkipLayerNormPluginDynamic"
        self.layers = []
        for lp in params.layers:
            fc = lambda w, out, extra=(): H.Plugin(FC, "2", [("out_dims", out), ("type_id", 1), ("W", f32(w).ravel())] + list(extra)).attach()
            ln = lambda g, b, bias: H.Plugin(SKIP, "5", [("type_id", 1), ("ld", E), ("beta", f32(b)), ("gamma", f32(g)),
                                                         ("bias", f32(bias))]).attach()
            self.layers.append((
                fc(lp.w_qkv, 3 * E, [("bias", f32(lp.b_qkv))]),
                H.Plugin(QKV, "4", [("type_id", 1), ("hidden_size", E), ("num_heads", N), ("has_mask", 1)]).attach(),
                fc(lp.w_out, E), ln(lp.ln1_gamma, lp.ln1_beta, lp.b_out),
                fc(lp.w_ffn1, F, [("bias", f32(lp.b_ffn1)), ("activation", 1)]), fc(lp.w_ffn2, E),
                ln(lp.ln2_gamma, lp.ln2_beta, lp.b_ffn2)))
            if not all(p.ok for p in self.layers[-1]):
                raise RuntimeError("plugin creation failed")
        d = lambda c: H.make_desc((SEQ, batch, c, 1, 1), H.HALF)
        self.d = {c: d(c) for c in (E, 3 * E, F)}
        self.dmask = H.make_desc((batch, 1), H.INT32)
        buf = lambda c: torch.empty((SEQ, batch, c), dtype=torch.float16, device=dev)
        self.qkv, self.ctx, self.ao, self.h1, self.f1, self.f2 = buf(3 * E), buf(E), buf(E), buf(E), buf(F), buf(E)
        self.x = [buf(E), buf(E)]
        self.mask_idx = torch.full((batch, 1), SEQ, dtype=torch.int32, device=dev)
        self.ws = torch.empty(4096, dtype=torch.uint8, device=dev)
        self.E, self.F = E, F
        self.np = np

    def forward(self, x0):
        import torch

        s = torch.cuda.current_stream().cuda_stream
        E, F, d = self.E, self.F, self.d

        def enq(p, ins, outs, ind, outd, ws=None):
            st = p.enqueue(ind, outd, [t.data_ptr() for t in ins], [t.data_ptr() for t in outs], ws.data_ptr() if ws is not None else None, s)
            if st != 0:
                raise RuntimeError(f"plugin enqueue returned {st}")

        x = x0
        for i, (qkv_p, att_p, out_p, ln1_p, f1_p, f2_p, ln2_p) in enumerate(self.layers):
            y = self.x[i & 1]
            enq(qkv_p, [x], [self.qkv], [d[E]], [d[3 * E]])
            enq(att_p, [self.qkv, self.mask_idx], [self.ctx], [d[3 * E], self.dmask], [d[E]], self.ws)
            enq(out_p, [self.ctx], [self.ao], [d[E]], [d[E]])
            enq(ln1_p, [self.ao, x], [self.h1], [d[E], d[E]], [d[E]])
            enq(f1_p, [self.h1], [self.f1], [d[E]], [d[F]])
            enq(f2_p, [self.f1], [self.f2], [d[F]], [d[E]])
            enq(ln2_p, [self.f2, self.h1], [y], [d[E], d[E]], [d[E]])
            x = y
        return x

    def close(self):
        for layer in self.layers:
            for p in layer:
                p.close()


def run_b200(args):
    import numpy as np
    import torch

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the B200 kernels have no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist = None
    if world > 1:
        import torch.distributed as dist

        # stdout carries the one JSON line only: NCCL's banner / debug text (NCCL_DEBUG=VERSION or INFO) goes to stderr
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=dev)

    import tensorrt_b200 as T
    from tensorrt_b200 import sharding, synthetic

    peaks = _peaks()
    params = synthetic.make_params(LAYERS, HIDDEN, HEADS, FFN, seed=0, device=dev)
    # the global batch (same on every rank) and this rank's contiguous share of it
    g_ids, g_seg, _, _ = synthetic.make_inputs(BATCH, SEQ, seed=100, device=dev)
    mine = sharding.shard_even(BATCH, world, rank)
    my_b = len(mine)

    def slice_batch(lo, n):
        ids = g_ids[lo * SEQ:(lo + n) * SEQ].contiguous()
        seg = g_seg[lo * SEQ:(lo + n) * SEQ].contiguous()
        cu = torch.arange(0, (n + 1) * SEQ, SEQ, dtype=torch.int32, device=dev)
        return ids, seg, cu

    ids, seg, cu = slice_batch(mine.start, my_b)
    w_ids, w_seg, w_cu = slice_batch(0, BATCH)     # 64 sequences per GPU: the weak-scaling side number
    out = torch.empty((BATCH * SEQ, HIDDEN), dtype=torch.float16, device=dev)

    enc16 = T.BertEncoder(params, T.FP16, dev)
    encs = {"fp16": enc16}
    if args.dtype == "int8" or args.both:
        # explicit INT8: per-tensor scales amax/127 from one seeded calibration batch of the same distribution
        cids, cseg, ccu, _ = synthetic.make_inputs(8, SEQ, seed=7, device=dev)
        amax = enc16.calibrate(cids, cseg, ccu, SEQ)
        synthetic.assign_int8_scales(params, amax)
        encs["int8"] = T.BertEncoder(params, T.INT8, dev)
    order = [args.dtype] + (["fp16" if args.dtype == "int8" else "int8"] if args.both else [])

    def reduce_max(*vals):
        if world == 1:
            return list(vals)
        t = torch.tensor(vals, dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    results = {}
    sampler = ClockSampler(local) if rank == 0 else None
    clocks = None
    for name in order:
        enc = encs[name]
        if sampler and name == args.dtype:
            sampler.start()
        my_out = out[:my_b * SEQ]
        ms = time_forward(lambda: enc.forward(ids, seg, cu, SEQ, out=my_out), args.steps, args.warmup, world, dist)
        if sampler and name == args.dtype:
            clocks = sampler.stop()
        status = enc.status_word()
        lat = step_latency(lambda: enc.forward(ids, seg, cu, SEQ, out=my_out)) if world == 1 else None
        if lat is not None:
            # the same forward captured once into a CUDA graph and replayed (170 launches become one): what is left of
            # the step when the host submits nothing
            try:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    enc.forward(ids, seg, cu, SEQ, out=my_out)
                    side.synchronize()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=side):
                        enc.forward(ids, seg, cu, SEQ, out=my_out)
                torch.cuda.current_stream().wait_stream(side)
                lat["cuda_graph_replay_ms"] = time_forward(graph.replay, args.steps, 3, 1, None)
                del graph
            except Exception as e:
                lat["cuda_graph_replay_ms"] = f"unavailable: {type(e).__name__}: {e}"
        kind_ms, kind_n = kernel_breakdown(enc, ids, seg, cu, my_out)
        ms_e2e, h2d, d2h = time_e2e(enc, ids, seg, cu, args.steps, 3, world, dist, my_out)
        ms_weak = None
        if world > 1:
            ms_weak = time_forward(lambda: enc.forward(w_ids, w_seg, w_cu, SEQ, out=out), args.steps, args.warmup, world, dist)
            ms, ms_e2e, ms_weak = reduce_max(ms, ms_e2e, ms_weak)
        results[name] = dict(ms=ms, ms_e2e=ms_e2e, ms_weak=ms_weak, h2d=h2d, d2h=d2h, kind_ms=kind_ms, kind_n=kind_n, status=status, lat=lat,
                             launches=enc.launches_per_forward)

    # ---- config 4: packed variable-length batch, lengths uniform in [32, 384] (seed 1), B = 256, token-balanced shards ----
    lengths_all = np.random.default_rng(1).integers(32, 385, size=256).astype(np.int32)
    shards = sharding.shard_by_tokens(lengths_all, world)
    my_len = torch.from_numpy(lengths_all[shards[rank]])
    c4_cu = torch.zeros(len(my_len) + 1, dtype=torch.int32)
    c4_cu[1:] = torch.cumsum(my_len, 0)
    c4_total = int(c4_cu[-1])
    gen = torch.Generator(device="cpu").manual_seed(4 + rank)
    c4_ids = torch.randint(0, 30522, (c4_total,), generator=gen, dtype=torch.int32).to(dev)
    c4_seg = torch.randint(0, 2, (c4_total,), generator=gen, dtype=torch.int32).to(dev)
    c4_cu = c4_cu.to(dev)
    c4_out = torch.empty((c4_total, HIDDEN), dtype=torch.float16, device=dev)
    c4 = {}
    for name in ([] if args.no_extras else order):
        enc = encs[name]
        c4_ms = time_forward(lambda: enc.forward(c4_ids, c4_seg, c4_cu, SEQ, out=c4_out), max(5, args.steps // 2), 3, world, dist)
        (c4_ms,) = reduce_max(c4_ms)
        c4[name] = c4_ms

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # measured tensor-pipe rates for the FC MMA shape (rank 0, after the timed regions)
    mma_rate = {"int8": probe_mma_rate(T, T.INT8), "fp16": probe_mma_rate(T, T.FP16)}

    def roofline(name):
        r = results[name]
        fc_ms, fc_n = r["kind_ms"][1], r["kind_n"][1]
        flops_per_forward = my_b * LAYERS * FLOPS_PER_SEQ_LAYER_FC
        achieved = flops_per_forward / (fc_ms * 1e-3) / 1e12 if fc_ms > 0 else None
        if name == "int8":
            peak = mma_rate["int8"]
            src = ("measured in this run: tcgen05.mma.cta_group::2.kind::i8 256x256x32 chains on all SM pairs, operands "
                   "resident in shared memory (bert_b200_probe_mma_rate)")
        else:
            peak, src = peaks["tc_sustained"], f"{peaks['source']} bf16 sustained"
        traffic = FC_DRAM_BYTES_PER_LAUNCH_INT8 if (name == "int8" and my_b == 64) else None
        return {"bound": "tensor", "kernel": "fcTcgen05PairKernel (4 FC shapes per layer)", "achieved": achieved, "peak": peak,
                "unit": "TFLOP/s" if name == "fp16" else "TOP/s", "frac": achieved / peak if achieved else None,
                "traffic": traffic, "peak_source": src, "launches_per_step": fc_n,
                "flops_per_launch_avg": flops_per_forward / max(fc_n, 1), "ms_per_launch_avg": fc_ms / max(fc_n, 1),
                "mma_rate_probe": {"int8_tops": mma_rate["int8"], "fp16_tflops": mma_rate["fp16"]}}

    def breakdown(name):
        r = results[name]
        kinds = ("emb_layer_norm", "fc", "mha", "skip_layer_norm", "other")
        d = {k: {"ms_per_step": r["kind_ms"][i], "launches": r["kind_n"][i]} for i, k in enumerate(kinds)}
        d["note"] = ("every launch bracketed by CUDA events in extra forwards: the brackets cost the overlap of consecutive "
                     "kernels, so these times add up to more than ms_per_step")
        mha_flops = my_b * LAYERS * FLOPS_PER_SEQ_LAYER_MHA
        if r["kind_ms"][2] > 0:
            d["mha"]["achieved_tflops"] = mha_flops / (r["kind_ms"][2] * 1e-3) / 1e12
            d["mha"]["frac_of_tensor_peak"] = d["mha"]["achieved_tflops"] / (mma_rate["int8"] if name == "int8" else peaks["tc_sustained"])
        elem = 1 if name == "int8" else 2
        ln_bytes = 2 * LAYERS * my_b * SEQ * 3 * HIDDEN * elem
        if r["kind_ms"][3] > 0:
            d["skip_layer_norm"]["achieved_gbs"] = ln_bytes / (r["kind_ms"][3] * 1e-3) / 1e9
            d["skip_layer_norm"]["frac_of_hbm_peak"] = d["skip_layer_norm"]["achieved_gbs"] / peaks["hbm"]
        # the same kernel alone at the step's shape, operands rotated beyond the L2 (no event between launches)
        iso_ms, iso_gbs = isolated_skip_ln(T, dev, my_b * SEQ, HIDDEN, name == "int8")
        d["skip_layer_norm"]["isolated"] = {"ms_per_launch": iso_ms, "achieved_gbs": iso_gbs, "frac_of_hbm_peak": iso_gbs / peaks["hbm"],
                                            "rows": my_b * SEQ, "l2": "operand sets rotated over more than 2.5 x the 126 MB L2"}
        return d

    main = results[args.dtype]
    n = world
    line = {
        "metric": f"BERT-large s384 {args.dtype.upper()} encoder sequences/s", "value": BATCH / (main["ms"] * 1e-3),
        "unit": "seq/s", "n_gpus": n, "steps": args.steps, "warmup": args.warmup, "ms_per_step": main["ms"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8" if args.dtype == "int8" else "f16",
        "data": "synthetic",
        "config": {"workload": _workload(args.dtype),
                   "layers": LAYERS, "global_batch": BATCH, "per_gpu_batch": my_b, "seq_len": SEQ,
                   "parallelism": f"dp{n} (one batch of {BATCH} split evenly, no collective)",
                   "l2": "working set per step (activations + weights > 300 MB per GPU) exceeds the 126 MB L2"},
        "e2e": {"value": BATCH / (main["ms_e2e"] * 1e-3), "unit": "seq/s", "ms_per_step": main["ms_e2e"],
                "h2d_bytes_per_step": main["h2d"], "d2h_bytes_per_step": main["d2h"]},
        "gpu_launches": main["launches"] * args.steps,
        "launches_per_step": main["launches"],
        "clocks": clocks,
        "roofline": roofline(args.dtype),
        "kernels": breakdown(args.dtype),
        "device_wait_status": main["status"],
    }
    if main["lat"]:
        line["step_latency_ms"] = main["lat"]
    if n > 1:
        line["weak"] = {"value": n * BATCH / (main["ms_weak"] * 1e-3), "unit": "seq/s", "ms_per_step": main["ms_weak"],
                        "per_gpu_batch": BATCH, "scaling": "weak"}
    for name in order[1:]:
        r = results[name]
        line[name] = {"value": BATCH / (r["ms"] * 1e-3), "unit": "seq/s", "ms_per_step": r["ms"],
                      "e2e_value": BATCH / (r["ms_e2e"] * 1e-3), "roofline": roofline(name), "kernels": breakdown(name),
                      "device_wait_status": r["status"]}
        if r["lat"]:
            line[name]["step_latency_ms"] = r["lat"]
        if n > 1:
            line[name]["weak_value"] = n * BATCH / (r["ms_weak"] * 1e-3)
    tokens4 = int(lengths_all.sum())
    line["config4"] = None if args.no_extras else {
        "workload": "BERT-large packed variable-length batch: 256 sequences, lengths uniform in [32, 384] (seed 1), "
                    f"{tokens4} tokens, sequences assigned longest-first to the least-loaded GPU (benchmark configuration 4)",
        "tokens": tokens4, "shard_tokens": [int(lengths_all[s].sum()) for s in shards],
        **{name: {"seq_per_s": 256 / (c4[name] * 1e-3), "tokens_per_s": tokens4 / (c4[name] * 1e-3), "ms_per_step": c4[name]}
           for name in order}}

    if n == 1 and not args.no_extras:
        # the FP16 network through the plugin objects' enqueue() (what a TensorRT engine built from them runs)
        try:
            pe = PluginEncoder(params, BATCH, dev)
            x0 = torch.randn((SEQ, BATCH, HIDDEN), device=dev).half()
            p_ms = time_forward(lambda: pe.forward(x0), max(5, args.steps // 2), 3, 1, None)
            line["plugin_path"] = {"value": BATCH / (p_ms * 1e-3), "unit": "seq/s", "ms_per_step": p_ms, "dtype": "f16",
                                   "enqueues_per_step": 7 * LAYERS,
                                   "path": "IPluginV3OneRuntime::enqueue of FC v2 / QKVToContext v4 / SkipLayerNorm v5 objects, "
                                           "fixed [S, B, E] layout, 24 layers (no embedding plugin in the loop)"}
            pe.close()
        except Exception as e:  # the plugin library needs the TensorRT headers at build time
            line["plugin_path"] = {"unavailable": f"{type(e).__name__}: {e}"}
    if n == 1 and not args.no_cpu:
        b, times, cores = cpu_forward_rate(budget_s=15.0)
        line["cpu_baseline"] = {"value": b / times[0], "unit": "seq/s", "cores": cores, "kind": "port",
                                "sample": f"{b} sequences x 24 layers x S=384 (one forward), FP32 torch-CPU port of the reference math"}
    else:
        line["cpu_baseline"] = None
    emit(line)
    if world > 1:
        dist.destroy_process_group()


def run_sweep(args):
    """Kernel sweep against the rooflines (benchmark configuration 5) on one GPU: fused attention as tensor throughput for
    S in {128, 256, 384, 512}, SkipLayerNorm + bias as HBM GB/s for hidden in {768, 1024, 4096} x tokens 2^10 .. 2^20,
    the embedding gather + LayerNorm (vocab 30522, hidden 1024) as GB/s; beside each the reference's own kernel from
    oracle/_ref when that library has been built (tests' checker, timed here as the same-box bar)."""
    import numpy as np
    import torch

    import tensorrt_b200 as T

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    peaks = _peaks()
    ref = None
    try:
        from oracle import ref_lib

        if ref_lib.available():
            ref = ref_lib.RefLib()
    except Exception:
        ref = None
    vp = C.c_void_p
    res = {"peaks": {"hbm_gbs": peaks["hbm"], "bf16_tflops": peaks["tc"], "bf16_tflops_sustained": peaks["tc_sustained"],
                     "source": peaks["source"],
                     "int8_mma_tops_probe": probe_mma_rate(T, T.INT8), "fp16_mma_tflops_probe": probe_mma_rate(T, T.FP16)},
           "reference_kernels": "oracle/_ref/libref_bert.so" if ref else None}
    N, d = 16, 64
    mha = []
    for S in (128, 256, 384, 512):
        tiles = -(-S // 128)
        B = -(-4 * 148 // (N * tiles))          # smallest batch with B * 16 * ceil(S / 128) >= 4 * 148 query tiles
        flops = 4 * S * S * d * N * B
        cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device=dev)
        x = torch.randn(S * B, 3 * N * d, device=dev)
        amax = float(x.abs().max())
        q16 = lambda: (x.half(), torch.empty(S * B, N * d, device=dev, dtype=torch.float16))
        q8 = lambda: (torch.clamp(torch.round(x * (127 / amax)), -127, 127).to(torch.int8), torch.empty(S * B, N * d, device=dev, dtype=torch.int8))
        s1 = (amax / 127) ** 2 * 0.125
        row = {"S": S, "B": B, "heads": N, "head_size": d}
        sets16, sets8 = rotating(q16, S * B * 4 * N * d * 2), rotating(q8, S * B * 4 * N * d)
        # attention launches are timed as CUDA-graph replays (ours and the reference's alike)
        ms = time_rotating_graph(lambda s, st: T.mha(s[0], B, S, N, cu_seqlens=cu, out=s[1]), sets16)
        row["fp16"] = {"ms": ms, "tflops": flops / ms / 1e9, "frac_of_bf16_sustained": flops / ms / 1e9 / peaks["tc_sustained"],
                       "hbm_cap_tflops": (S / 2) * peaks["hbm"] / 1e3}
        ms = time_rotating_graph(lambda s, st: T.mha(s[0], B, S, N, cu_seqlens=cu, scale_bmm1=s1, scale_softmax=127.0, scale_bmm2=1.0 / 64,
                                                     out=s[1]), sets8)
        row["int8"] = {"ms": ms, "tops": flops / ms / 1e9, "frac_of_int8_probe": flops / ms / 1e9 / res["peaks"]["int8_mma_tops_probe"]}
        if S == 384:
            # the CHW32-interleaved INT8 form of plugin version 6 (same values, other layout)
            tot = S * B
            mk_il = lambda: (torch.randint(-127, 127, (3 * N * d // 32, tot, 32), device=dev, dtype=torch.int8),
                             torch.empty((N * d // 32, tot, 32), device=dev, dtype=torch.int8))
            sets_il = rotating(mk_il, tot * 4 * N * d)
            ms = time_rotating_graph(lambda s, st: T.mha(s[0], B, S, N, cu_seqlens=cu, scale_bmm1=s1, scale_softmax=127.0, scale_bmm2=1.0 / 64,
                                                         interleaved=True, out=s[1]), sets_il)
            row["int8_interleaved"] = {"ms": ms, "tops": flops / ms / 1e9}
            if ref is not None:
                try:
                    ms = time_rotating_graph(lambda s, st: ref.lib.ref_fmha_v2(
                        vp(st), 2, B, S, N, d, tot, vp(s[0].data_ptr()), vp(s[1].data_ptr()), vp(cu.data_ptr()), 1, C.c_float(s1),
                        C.c_float(127.0), C.c_float(1.0 / 64)), sets_il)
                    row["int8_interleaved"]["reference_tops"] = flops / ms / 1e9
                except Exception as e:
                    row["int8_interleaved"]["reference_error"] = str(e)
            del sets_il
        if ref is not None:
            def ref16(s, st):
                ref.lib.ref_fmha_v2(vp(st), 1, B, S, N, d, S * B, vp(s[0].data_ptr()), vp(s[1].data_ptr()), vp(cu.data_ptr()), 0,
                                    C.c_float(0.125), C.c_float(1.0), C.c_float(1.0))

            def ref8(s, st):
                ref.lib.ref_fmha_v2(vp(st), 2, B, S, N, d, S * B, vp(s[0].data_ptr()), vp(s[1].data_ptr()), vp(cu.data_ptr()), 0,
                                    C.c_float(s1), C.c_float(127.0), C.c_float(1.0 / 64))
            try:
                row["fp16"]["reference_tflops"] = flops / time_rotating_graph(ref16, sets16) / 1e9
                row["int8"]["reference_tops"] = flops / time_rotating_graph(ref8, sets8) / 1e9
                if S in (128, 384):
                    # the fixed-length kernels of plugin versions 1-3: the same bytes read as [S, B, N, 3, d], full mask
                    wm, wn = (1, 8) if S == 384 else (2, 2)
                    xm = -(-S // (16 * wm))
                    packed = torch.empty((B, xm, wm * wn * 32), dtype=torch.int32, device=dev)
                    ones = torch.ones((S, B), dtype=torch.int32, device=dev)
                    ref.lib.ref_convert_mask(S, B, wm, wn, 1, vp(ones.data_ptr()), vp(packed.data_ptr()), None)
                    torch.cuda.synchronize()

                    def ref_v1(tid, s, st, a, b, c):
                        ref.lib.ref_fmha_v1(vp(st), tid, B, S, N, d, vp(s[0].data_ptr()), vp(s[1].data_ptr()), vp(packed.data_ptr()),
                                            C.c_float(a), C.c_float(b), C.c_float(c))

                    row["fp16"]["reference_fixed_length_tflops"] = flops / time_rotating_graph(
                        lambda s, st: ref_v1(1, s, st, 0.125, 1.0, 1.0), sets16) / 1e9
                    row["int8"]["reference_fixed_length_tops"] = flops / time_rotating_graph(
                        lambda s, st: ref_v1(2, s, st, s1, 127.0, 1.0 / 64), sets8) / 1e9
            except Exception as e:
                row["reference_error"] = str(e)
        mha.append(row)
        del sets16, sets8
    res["mha"] = mha

    ln = []
    for ld in (768, 1024, 4096):
        for e in range(10, 21, 2):
            tokens = 1 << e
            row = {"hidden": ld, "tokens": tokens}
            ms, gbs = isolated_skip_ln(T, dev, tokens, ld, False)
            row["fp16"] = {"ms": ms, "gbs": gbs, "frac_of_hbm_peak": gbs / peaks["hbm"]}
            ms, gbs = isolated_skip_ln(T, dev, tokens, ld, True)
            row["int8"] = {"ms": ms, "gbs": gbs, "frac_of_hbm_peak": gbs / peaks["hbm"]}
            if ref is not None and tokens == 1 << 16:
                g = torch.ones(ld, device=dev).half()
                sets = rotating(lambda: (torch.randn(tokens, ld, device=dev).half(), torch.randn(tokens, ld, device=dev).half(),
                                         torch.empty(tokens, ld, device=dev).half()), 6 * tokens * ld)
                ms = time_rotating_graph(lambda s, st: ref.lib.ref_skip_layer_norm(vp(st), 1, ld, tokens * ld, vp(s[0].data_ptr()), vp(s[1].data_ptr()),
                                                                                   vp(g.data_ptr()), vp(g.data_ptr()), vp(s[2].data_ptr()), vp(g.data_ptr())), sets)
                row["fp16"]["reference_gbs"] = 6 * tokens * ld / ms / 1e6
                if ld != 4096:  # the reference's INT8 kernel exists for 768 and 1024 only
                    sets = rotating(lambda: (torch.randint(-127, 127, (tokens, ld), device=dev, dtype=torch.int8),
                                             torch.randint(-127, 127, (tokens, ld), device=dev, dtype=torch.int8),
                                             torch.empty(tokens, ld, device=dev, dtype=torch.int8)), 3 * tokens * ld)
                    ms = time_rotating_graph(lambda s, st: ref.lib.ref_skip_layer_norm_dqq(
                        vp(st), ld, tokens * ld, vp(s[0].data_ptr()), vp(s[1].data_ptr()), vp(g.data_ptr()), vp(g.data_ptr()), vp(s[2].data_ptr()),
                        vp(g.data_ptr()), C.c_float(0.02), C.c_float(0.02), C.c_float(40.0)), sets)
                    row["int8"]["reference_gbs"] = 3 * tokens * ld / ms / 1e6
            ln.append(row)
    res["skip_layer_norm_bias"] = ln

    # INT8 SkipLayerNorm on the CHW32-interleaved layout of plugin versions 7 / 8 (no bias), hidden 1024
    il = []
    for tokens in (24576, 262144):
        ld = 1024
        g = torch.ones(ld, device=dev).half()
        sets = rotating(lambda: (torch.randint(-127, 127, (ld // 32, tokens, 32), device=dev, dtype=torch.int8),
                                 torch.randint(-127, 127, (ld // 32, tokens, 32), device=dev, dtype=torch.int8),
                                 torch.empty((ld // 32, tokens, 32), device=dev, dtype=torch.int8)), 3 * tokens * ld)
        nbytes = 3 * tokens * ld
        ms = time_rotating_graph(lambda s, st: _product_lib().bert_b200_skip_layer_norm_interleaved_hface(
            vp(st), ld, tokens, vp(s[0].data_ptr()), vp(s[1].data_ptr()), vp(g.data_ptr()), vp(g.data_ptr()), vp(s[2].data_ptr()),
            C.c_float(0.02), C.c_float(0.02), C.c_float(40.0)), sets)
        row = {"hidden": ld, "tokens": tokens, "ms": ms, "gbs": nbytes / ms / 1e6, "frac_of_hbm_peak": nbytes / ms / 1e6 / peaks["hbm"]}
        if ref is not None:
            ms = time_rotating_graph(lambda s, st: ref.lib.ref_skip_layer_norm_interleaved(
                vp(st), 1, ld, tokens, vp(s[0].data_ptr()), vp(s[1].data_ptr()), vp(g.data_ptr()), vp(g.data_ptr()), vp(s[2].data_ptr()),
                None, C.c_float(0.02), C.c_float(0.02), C.c_float(40.0), C.c_float(1.0)), sets)
            row["reference_gbs"] = nbytes / ms / 1e6
        il.append(row)
    res["skip_layer_norm_interleaved"] = il

    # embedding gather + LayerNorm: vocab 30522, hidden 1024, FP16 tables; bytes = word row in + row out + two ids
    E, vocab = 1024, 30522
    word = (0.02 * torch.randn(vocab, E, device=dev)).half()
    pos = (0.02 * torch.randn(512, E, device=dev)).half()
    tok = (0.02 * torch.randn(2, E, device=dev)).half()
    gam, bet = torch.ones(E, device=dev), torch.zeros(E, device=dev)
    emb = []
    for S, B in ((128, 32), (384, 64), (384, 512)):
        sets = rotating(lambda: (torch.randint(0, vocab, (S, B), device=dev, dtype=torch.int32),
                                 torch.randint(0, 2, (S, B), device=dev, dtype=torch.int32)), S * B * (2 * E * 2 + 8), min_total=0)
        ms = time_rotating_graph(lambda s, st: T.emb_layer_norm(s[0], s[1], word, pos, tok, gam, bet), sets)
        nbytes = S * B * (2 * E * 2 + 8)
        row = {"S": S, "B": B, "tokens": S * B, "ms": ms, "gbs": nbytes / ms / 1e6, "frac_of_hbm_peak": nbytes / ms / 1e6 / peaks["hbm"],
               "note": "62 MB word table, random rows: every launch gathers different rows; the output (2 KB per token) is written once"}
        if ref is not None:
            outr = torch.empty(S, B, E, device=dev, dtype=torch.float16)
            ms = time_rotating_graph(lambda s, st: ref.lib.ref_emb_layer_norm(
                vp(st), 1, E, B, S, vp(s[0].data_ptr()), vp(s[1].data_ptr()), vp(bet.data_ptr()), vp(gam.data_ptr()), vp(word.data_ptr()),
                vp(pos.data_ptr()), vp(tok.data_ptr()), vocab, 2, vp(outr.data_ptr())), sets)
            row["reference_gbs"] = nbytes / ms / 1e6
        emb.append(row)
    res["emb_layer_norm"] = emb

    # the packed (variable-length) embedding kernel on the lengths of benchmark configuration 4
    lens = np.random.default_rng(1).integers(32, 385, size=256).astype(np.int32)
    cu4 = torch.from_numpy(np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)).to(dev)
    tot4 = int(lens.sum())
    sets = rotating(lambda: (torch.randint(0, vocab, (tot4,), device=dev, dtype=torch.int32),
                             torch.randint(0, 2, (tot4,), device=dev, dtype=torch.int32)), 1, min_total=0)
    nbytes = tot4 * (2 * E * 2 + 8)
    ms = time_rotating_graph(lambda s, st: T.emb_layer_norm_var_seqlen(s[0], s[1], cu4, 384, word, pos, tok, gam, bet), sets)
    row = {"sequences": 256, "tokens": tot4, "ms": ms, "gbs": nbytes / ms / 1e6, "frac_of_hbm_peak": nbytes / ms / 1e6 / peaks["hbm"]}
    if ref is not None:
        outr = torch.empty(tot4, E, device=dev, dtype=torch.float16)
        ms = time_rotating_graph(lambda s, st: ref.lib.ref_emb_layer_norm_var_seqlen(
            vp(st), E, 256, 384, vp(s[0].data_ptr()), vp(s[1].data_ptr()), vp(cu4.data_ptr()), vp(bet.data_ptr()), vp(gam.data_ptr()),
            vp(word.data_ptr()), vp(pos.data_ptr()), vp(tok.data_ptr()), vocab, 2, vp(outr.data_ptr()), None), sets)
        row["reference_gbs"] = nbytes / ms / 1e6
    res["emb_layer_norm_var_seqlen"] = row

    # the four FC shapes of a BERT-large layer at 24576 tokens (+ a square one): tera-operations/s per epilogue, operands
    # rotated; torch.matmul (cuBLAS, FP16, no epilogue) on the same operands as the library bar
    fc = []
    for (m, k, n) in ((24576, 1024, 3072), (24576, 1024, 1024), (24576, 1024, 4096), (24576, 4096, 1024), (8192, 8192, 8192)):
        row = {"m": m, "k": k, "n": n}
        ops = 2.0 * m * n * k
        bias = torch.zeros(n, device=dev)
        s16 = rotating(lambda: (torch.randn(m, k, device=dev).half(), (0.02 * torch.randn(n, k, device=dev)).half(),
                                torch.empty(m, n, device=dev, dtype=torch.float16)), 2 * (m * k + n * k + m * n))
        row["fp16"] = ops / time_rotating(lambda t: T.fc(t[0], t[1], out=t[2]), s16) / 1e9
        row["fp16_bias_gelu"] = ops / time_rotating(lambda t: T.fc(t[0], t[1], bias, T.ACT_GELU_ERF, out=t[2]), s16) / 1e9
        row["cublas_fp16_matmul"] = ops / time_rotating(lambda t: torch.matmul(t[0], t[1].t(), out=t[2]), s16) / 1e9
        del s16
        s8 = rotating(lambda: (torch.randint(-127, 128, (m, k), device=dev, dtype=torch.int8),
                               torch.randint(-127, 128, (n, k), device=dev, dtype=torch.int8),
                               torch.empty(m, n, device=dev, dtype=torch.int8)), m * k + n * k + m * n)
        row["int8"] = ops / time_rotating(lambda t: T.fc(t[0], t[1], alpha=1e-4, out_dtype=torch.int8, out_scale=20.0, out=t[2]), s8) / 1e9
        row["int8_bias_gelu"] = ops / time_rotating(lambda t: T.fc(t[0], t[1], bias, T.ACT_GELU_ERF, alpha=1e-4, out_dtype=torch.int8,
                                                                   out_scale=20.0, out=t[2]), s8) / 1e9
        del s8
        fc.append(row)
    res["fc_tera_ops"] = fc
    emit({"sweep": res})


def run_case(name):
    """Profiling captures: ONE kernel launched a few times on inputs larger than the L2 and a few GB at most, so that a
    profiler capture of it (`-k <kernel> -c 1..3`) ends in a minute: mha_f16 / mha_i8 (S=384, 64 sequences, 16 heads x
    64), ln_f16 / ln_i8 (SkipLayerNorm + bias, 131072 rows of 1024), emb (S=384, 256 sequences, vocab 30522, hidden
    1024), fc_f16 / fc_i8 (the four BERT-large FC shapes at 24576 rows, two launches each). Prints no bench value."""
    import torch

    import tensorrt_b200 as T

    dev = torch.device("cuda:0")
    N, d = 16, 64
    if name in ("mha_f16", "mha_i8"):
        S, B = 384, 64
        cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device=dev)
        if name == "mha_f16":
            qkv = torch.randn(S * B, 3 * N * d, device=dev).half()
            for _ in range(4):
                out = T.mha(qkv, B, S, N, cu_seqlens=cu)
        else:
            q8 = torch.randint(-127, 127, (S * B, 3 * N * d), device=dev, dtype=torch.int8)
            for _ in range(4):
                out = T.mha(q8, B, S, N, cu_seqlens=cu, scale_bmm1=1e-4, scale_softmax=127.0, scale_bmm2=0.01)
    elif name in ("ln_f16", "ln_i8"):
        tokens, ld = 131072, 1024
        g = torch.ones(ld, device=dev).half()
        b = torch.zeros(ld, device=dev).half()
        if name == "ln_f16":
            x, s = torch.randn(tokens, ld, device=dev).half(), torch.randn(tokens, ld, device=dev).half()
            out = torch.empty_like(x)
            for _ in range(4):
                T.skip_layer_norm(x, s, g, b, bias=b, out=out)
        else:
            x = torch.randint(-127, 127, (tokens, ld), device=dev, dtype=torch.int8)
            s = torch.randint(-127, 127, (tokens, ld), device=dev, dtype=torch.int8)
            out = torch.empty_like(x)
            for _ in range(4):
                T.skip_layer_norm_dqq(x, s, g, b, b, 0.02, 0.02, 40.0, out=out)
    elif name == "emb":
        E, vocab, S, B = 1024, 30522, 384, 256
        word = (0.02 * torch.randn(vocab, E, device=dev)).half()
        pos = (0.02 * torch.randn(512, E, device=dev)).half()
        tok = (0.02 * torch.randn(2, E, device=dev)).half()
        gam, bet = torch.ones(E, device=dev), torch.zeros(E, device=dev)
        for _ in range(4):
            ids = torch.randint(0, vocab, (S, B), device=dev, dtype=torch.int32)
            seg = torch.randint(0, 2, (S, B), device=dev, dtype=torch.int32)
            out = T.emb_layer_norm(ids, seg, word, pos, tok, gam, bet)
    elif name in ("fc_f16", "fc_i8"):
        for (m, k, n, act) in [(24576, 1024, 3072, 0), (24576, 1024, 1024, 0), (24576, 1024, 4096, 1), (24576, 4096, 1024, 0)]:
            bias = torch.zeros(n, device=dev) if act or n == 3072 else None
            if name == "fc_f16":
                a, w = torch.randn(m, k, device=dev).half(), (0.02 * torch.randn(n, k, device=dev)).half()
                for _ in range(2):
                    out = T.fc(a, w, bias, T.ACT_GELU_ERF if act else T.ACT_NONE)
            else:
                a = torch.randint(-127, 127, (m, k), device=dev, dtype=torch.int8)
                w = torch.randint(-127, 127, (n, k), device=dev, dtype=torch.int8)
                for _ in range(2):
                    out = T.fc(a, w, bias, T.ACT_GELU_ERF if act else T.ACT_NONE, alpha=1e-4, out_dtype=torch.int8, out_scale=20.0)
    else:
        raise SystemExit(f"unknown case {name}")
    torch.cuda.synchronize()
    print("case", name, "ok", float(out.float().abs().mean()), file=sys.stderr)


_JSON_FD = None


def _claim_stdout():
    """Keeps a private handle on stdout for the one JSON line and points file descriptor 1 at stderr, so that text
    printed by libraries (NCCL's version banner, for one) cannot end up next to the result."""
    global _JSON_FD
    if _JSON_FD is None:
        sys.stdout.flush()
        _JSON_FD = os.dup(1)
        os.dup2(2, 1)


def emit(line):
    data = (json.dumps(line) + "\n").encode()
    if _JSON_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_JSON_FD, data)


def main():
    _claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--dtype", choices=["int8", "fp16"], default="int8")
    ap.add_argument("--both", action=argparse.BooleanOptionalAction, default=True,
                    help="also time the other precision and report it in a sub-object")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extras", action="store_true", help="skip the plugin-path and packed variable-length legs")
    ap.add_argument("--sweep", action="store_true", help="kernel sweep against the rooflines instead of the encoder step")
    ap.add_argument("--case", default=None, help="profiling captures only: launch ONE kernel a few times (see run_case)")
    ap.add_argument("--layers", type=int, default=LAYERS, help="profiling captures only: fewer encoder layers")
    ap.add_argument("--batch", type=int, default=BATCH, help="profiling captures only: sequences in the global batch")
    args = ap.parse_args()
    globals().update(LAYERS=args.layers, BATCH=args.batch)
    if args.warmup < 3:
        args.warmup = 3
    if args.case:
        run_case(args.case)
    elif args.sweep:
        run_sweep(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
