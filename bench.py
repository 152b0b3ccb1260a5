#!/usr/bin/env python
"""BERT-large S=384 encoder throughput on B200 through the sm_100a plugin kernels.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--dtype int8|fp16] [--impl b200|reference]

One step = one forward pass of the 24-layer BERT-large encoder (EmbLayerNorm + 24 x [FC(QKV), fused MHA, FC,
SkipLayerNorm, FC+GELU, FC, SkipLayerNorm]) over a batch of 64 synthetic sequences of 384 tokens per GPU.
Prints ONE JSON line (rank 0). With N > 1 (launched by torchrun, one rank per GPU) every rank runs its own
64 sequences (weak scaling, no collective on the data path); the time is the max over ranks.

`--impl reference` times the CPU restatement of the reference math (oracle/cpu_encoder.py, FP32, all host
cores) on a bounded sample of the same workload: the reference plugins have no CPU implementation and neither
TensorRT nor ONNX-Runtime is installed, so this port is the CPU arm.
"""
from __future__ import annotations

import argparse
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
                time.sleep(0.01)
        except Exception as e:  # NVML missing: report that instead of clocks
            self.reasons.add(f"nvml_unavailable:{type(e).__name__}")

    def stop(self):
        self._halt.set()
        self.join(timeout=2)
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


FC_DRAM_BYTES_PER_LAUNCH_INT8 = 69.4e6  # dram__bytes_read.sum + dram__bytes_write.sum, mean of QKV / out / FFN1 / FFN2


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
        batch_hint = max(1, min(16, int(budget_s / max(t1, 1e-3))))
    for _ in range(warmup):
        run(batch_hint)
    times = [run(batch_hint) for _ in range(steps)]
    return batch_hint, times, torch.get_num_threads()


def _workload(dtype):
    if dtype == "int8":
        return ("BERT-large encoder, 24 layers, hidden 1024, 16 heads x 64, FFN 4096, seq 384, batch 64 per GPU "
                "(BASELINE configs[2]); explicit INT8 with amax/127 scales from one seeded calibration batch")
    return "BERT-large encoder, 24 layers, hidden 1024, 16 heads x 64, FFN 4096, seq 384, batch 64 per GPU, FP16"


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
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": _workload(args.dtype), "layers": LAYERS, "per_gpu_batch": BATCH, "seq_len": SEQ,
                   "cpu_arm": "bounded sample of the workload on the host cores"},
        "cpu_baseline": {"value": value, "unit": "seq/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "seq/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def time_encoder(enc, ids, seg, cu, steps, warmup, world, dist, out, profile_steps=3):
    """Device-resident timing: W warm-up forwards, then K forwards between two CUDA events on the launching stream.
    Afterwards `profile_steps` more forwards run with every kernel bracketed by CUDA events (same inputs, same stream)
    to split the step by kernel kind; those instrumented steps are not part of the reported step time."""
    import ctypes as C

    import torch

    for _ in range(warmup):
        enc.forward(ids, seg, cu, SEQ, out=out)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        enc.forward(ids, seg, cu, SEQ, out=out)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        dist.barrier()
    kind_ms, kind_n = (C.c_float * 5)(), (C.c_int32 * 5)()
    enc.enable_timing(True)
    enc.forward(ids, seg, cu, SEQ, out=out)  # creates the events
    torch.cuda.synchronize()
    for _ in range(profile_steps):
        enc.forward(ids, seg, cu, SEQ, out=out)
        enc.read_timing(kind_ms, kind_n)  # synchronises, then adds this forward's per-kind times
    enc.enable_timing(False)
    return ms, [v / profile_steps for v in kind_ms], [v // profile_steps for v in kind_n]


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
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
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


def run_b200(args):
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
    from tensorrt_b200 import synthetic

    peaks = _peaks()
    params = synthetic.make_params(LAYERS, HIDDEN, HEADS, FFN, seed=0, device=dev)
    ids, seg, cu, _ = synthetic.make_inputs(BATCH, SEQ, seed=100 + rank, device=dev)
    total = ids.shape[0]
    out = torch.empty((total, HIDDEN), dtype=torch.float16, device=dev)

    enc16 = T.BertEncoder(params, T.FP16, dev)
    results = {}
    encs = {"fp16": enc16}
    if args.dtype == "int8" or args.both:
        # explicit INT8: per-tensor scales amax/127 from one seeded calibration batch of the same distribution
        cids, cseg, ccu, _ = synthetic.make_inputs(8, SEQ, seed=7, device=dev)
        amax = enc16.calibrate(cids, cseg, ccu, SEQ)
        synthetic.assign_int8_scales(params, amax)
        encs["int8"] = T.BertEncoder(params, T.INT8, dev)
    order = [args.dtype] + (["fp16" if args.dtype == "int8" else "int8"] if args.both else [])

    sampler = ClockSampler(local) if rank == 0 else None
    for name in order:
        enc = encs[name]
        if sampler and name == args.dtype:
            sampler.start()
        ms, kind_ms, kind_n = time_encoder(enc, ids, seg, cu, args.steps, args.warmup, world, dist, out)
        if sampler and name == args.dtype:
            clocks = sampler.stop()
        status = enc.status_word()
        ms_e2e, h2d, d2h = time_e2e(enc, ids, seg, cu, max(3, args.steps // 2), 3, world, dist, out)
        if world > 1:
            t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms, ms_e2e = t.tolist()
        results[name] = dict(ms=ms, ms_e2e=ms_e2e, h2d=h2d, d2h=d2h, kind_ms=kind_ms, kind_n=kind_n, status=status,
                             launches=enc.launches_per_forward)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    def roofline(name):
        r = results[name]
        fc_ms, fc_n = r["kind_ms"][1], r["kind_n"][1]
        flops_per_forward = BATCH * LAYERS * FLOPS_PER_SEQ_LAYER_FC
        achieved = flops_per_forward / (fc_ms * 1e-3) / 1e12 if fc_ms > 0 else None
        if name == "int8":
            peak, src = 2 * peaks["tc_sustained"], f"2 x {peaks['source']} bf16 sustained (no measured INT8 figure)"
        else:
            peak, src = peaks["tc_sustained"], f"{peaks['source']} bf16 sustained"
        # DRAM bytes per FC launch from one `ncu --set full` capture of the four launches of a layer at this batch
        # (profiles/fc_pair_int8_bert_large_layer_fullset.md); no capture exists for FP16 or other batch sizes
        traffic = FC_DRAM_BYTES_PER_LAUNCH_INT8 if (name == "int8" and BATCH == 64) else None
        return {"bound": "tensor", "kernel": "fcTcgen05PairKernel (4 FC shapes per layer)", "achieved": achieved, "peak": peak,
                "unit": "TFLOP/s" if name == "fp16" else "TOP/s", "frac": achieved / peak if achieved else None,
                "traffic": traffic, "peak_source": src, "launches_per_step": fc_n,
                "flops_per_launch_avg": flops_per_forward / max(fc_n, 1), "ms_per_launch_avg": fc_ms / max(fc_n, 1)}

    def breakdown(name):
        r = results[name]
        kinds = ("emb_layer_norm", "fc", "mha", "skip_layer_norm", "other")
        d = {k: {"ms_per_step": r["kind_ms"][i], "launches": r["kind_n"][i]} for i, k in enumerate(kinds)}
        mha_flops = BATCH * LAYERS * FLOPS_PER_SEQ_LAYER_MHA
        if r["kind_ms"][2] > 0:
            d["mha"]["achieved_tflops"] = mha_flops / (r["kind_ms"][2] * 1e-3) / 1e12
        elem = 1 if name == "int8" else 2
        ln_bytes = 2 * LAYERS * BATCH * SEQ * 3 * HIDDEN * elem
        if r["kind_ms"][3] > 0:
            d["skip_layer_norm"]["achieved_gbs"] = ln_bytes / (r["kind_ms"][3] * 1e-3) / 1e9
            d["skip_layer_norm"]["frac_of_hbm_peak"] = d["skip_layer_norm"]["achieved_gbs"] / peaks["hbm"]
        return d

    main = results[args.dtype]
    n = world
    line = {
        "metric": f"BERT-large s384 {args.dtype.upper()} encoder sequences/s", "value": n * BATCH / (main["ms"] * 1e-3),
        "unit": "seq/s", "n_gpus": n, "steps": args.steps, "warmup": args.warmup, "ms_per_step": main["ms"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8" if args.dtype == "int8" else "f16",
        "data": "synthetic",
        "config": {"workload": _workload(args.dtype),
                   "layers": LAYERS, "per_gpu_batch": BATCH, "global_batch": n * BATCH, "seq_len": SEQ, "parallelism": f"dp{n} (batch sharding, no collective)",
                   "l2": "working set per step (activations > 250 MB + weights > 300 MB) exceeds the 126 MB L2"},
        "e2e": {"value": n * BATCH / (main["ms_e2e"] * 1e-3), "unit": "seq/s", "ms_per_step": main["ms_e2e"],
                "h2d_bytes_per_step": main["h2d"], "d2h_bytes_per_step": main["d2h"]},
        "gpu_launches": main["launches"] * args.steps,
        "launches_per_step": main["launches"],
        "clocks": clocks,
        "roofline": roofline(args.dtype),
        "kernels": breakdown(args.dtype),
        "device_wait_status": main["status"],
    }
    for name in order[1:]:
        r = results[name]
        line[name] = {"value": n * BATCH / (r["ms"] * 1e-3), "unit": "seq/s", "ms_per_step": r["ms"],
                      "e2e_value": n * BATCH / (r["ms_e2e"] * 1e-3), "roofline": roofline(name), "kernels": breakdown(name),
                      "device_wait_status": r["status"]}
    if n == 1 and not args.no_cpu:
        b, times, cores = cpu_forward_rate(budget_s=15.0)
        line["cpu_baseline"] = {"value": b / times[0], "unit": "seq/s", "cores": cores, "kind": "port",
                                "sample": f"{b} sequences x 24 layers x S=384 (one forward), FP32 torch-CPU port of the reference math"}
    else:
        line["cpu_baseline"] = None
    emit(line)
    if world > 1:
        dist.destroy_process_group()


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
    ap.add_argument("--layers", type=int, default=LAYERS, help="profiling captures only: fewer encoder layers")
    ap.add_argument("--batch", type=int, default=BATCH, help="profiling captures only: sequences per GPU and step")
    args = ap.parse_args()
    globals().update(LAYERS=args.layers, BATCH=args.batch)
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
