#!/usr/bin/env python
"""Benchmark of the batch SM120 decode path: Ginsn/s on synthetic instruction streams.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--words M]

One step = one pass of the decode kernel over one batch (default 64 Mi words = 1 GiB, forms
Zipf(1.1) over a seeded permutation of the instruction keys; the stream is synthetic because
the reference's own corpus is private).  With N > 1 (torchrun, one rank per GPU) every rank
decodes its own 64 Mi-word range of the same stream: weak scaling, no collective on the data
path.  Rank 0 prints one JSON line.

`value` is timed with CUDA events around K back-to-back launches on device-resident buffers;
`e2e` runs the same batch through the host-buffer entry point (pinned host memory, copies in
and out inside the timed region); `cpu_baseline` / `--impl reference` time the CPU oracle
(a C++ port of the reference's decoder; the Rust original cannot be built here) on host cores.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

UNIT = "Ginsn/s"
# Algorithmic bytes per instruction: decode 16 in + 2 (form) + 32 (8 slots) + 4 (ctrl) out; encode the reverse;
# roundtrip 16 in + 1 status byte out.
WORKLOADS = {
    "decode": {"metric": "decode_throughput", "bytes": 54, "kernel": "decode_kernel", "noise_ppm": 0,
               "text": "cfg1 batch decode: 64 Mi SM120 words per GPU, forms Zipf(1.1) over a seeded permutation of the "
                       "keys, SoA records out"},
    "encode": {"metric": "encode_throughput", "bytes": 54, "kernel": "encode_kernel", "noise_ppm": 0,
               "text": "cfg2 batch encode: the generator's 64 Mi (form, 8 slots, ctrl) records per GPU to words"},
    "roundtrip": {"metric": "roundtrip_throughput", "bytes": 17, "kernel": "roundtrip_kernel", "noise_ppm": 10000,
                  "text": "cfg3 fused roundtrip (decode, encode, compare): 64 Mi words per GPU, Zipf(1.1) forms, 1 % raw "
                          "random words, one status byte out"},
}
METRIC = WORKLOADS["decode"]["metric"]


def run_cubin(args, rank, world, local):
    """cfg4: a synthetic multi-kernel cubin per GPU (kernel lengths lognormal(ln 20000, 1.0) clamped to
    [2000, 200000] words, MMA-heavy family mix), every word of every kernel decoded by ONE launch through
    cubit_decode_elf.  Host buffers in and out, so the number includes the copies over PCIe."""
    import numpy as np
    import torch
    import torch.distributed as dist

    import cubit_b200
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    codec = cubit_b200.Codec(devices=(local,))
    rng = np.random.default_rng(1000 + rank)
    lengths = np.clip(np.exp(rng.normal(np.log(20000.0), 1.0, args.kernels)), 2000, 200000).astype(np.int64)
    total = int(lengths.sum())
    first = rank * (1 << 34)     # ranks draw disjoint ranges of one family-mix stream
    words = codec.synth(cubit_b200.MIX_FAMILY, STREAM_SEED, total, first=first)[0]
    starts = np.concatenate([[0], np.cumsum(lengths)])
    kernels = [(f"k{rank:02d}_{k:05d}", words[starts[k]:starts[k + 1]].tobytes()) for k in range(args.kernels)]
    image = cubit_b200.build_cubin(kernels)
    del kernels
    # Pinned host buffers, allocated once: the image, the records and the raw words.
    lib, ctx = codec._lib, codec._ctx
    n_out = int(((lengths + 7) // 8 * 8).sum())

    def pinned(nbytes, dtype, shape):
        p = C.c_void_p()
        codec._check(lib.cubit_host_alloc(ctx, nbytes, C.byref(p)))
        return p, np.ctypeslib.as_array(C.cast(p, C.POINTER(dtype)), shape=shape)
    p_img, img = pinned(len(image), C.c_uint8, (len(image),))
    img[:] = np.frombuffer(image, np.uint8)
    p_form, form = pinned(n_out * 2, C.c_uint16, (n_out,))
    p_slots, slots = pinned(n_out * 32, C.c_uint32, (8, n_out))
    p_ctrl, ctrl = pinned(n_out * 4, C.c_uint32, (n_out,))
    p_raw, raw = pinned(n_out * 16, C.c_uint8, (n_out, 16))
    word_start = np.zeros(args.kernels + 1, np.uint64)
    counts = cubit_b200._native.Counts()
    times = []
    for it in range(args.warmup + args.steps):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        elf = C.c_void_p()
        codec._check(lib.cubit_elf_parse(p_img, len(image), C.byref(elf)))
        assert lib.cubit_elf_num_text(elf) == args.kernels
        codec._check(lib.cubit_decode_elf(ctx, elf, None, args.kernels, C.c_void_p(word_start.ctypes.data), n_out, p_form, p_slots,
                                          p_ctrl, p_raw if it == 0 else None, C.byref(counts)))
        lib.cubit_elf_free(elf)
        dt = time.perf_counter() - t0
        if it == 0:
            # padding: every section is a multiple of 8 words (NOPs, then one self-branch)
            assert int(word_start[-1]) == n_out
            sample = np.arange(0, n_out, 4099)
            sys.path.insert(0, str(ROOT / "oracle"))
            from oracle_lib import Oracle
            of, os_, oc = Oracle().decode_batch(raw[sample])
            assert (form[sample] == of).all() and (slots[:, sample] == os_).all() and (ctrl[sample] == oc).all()
        if it >= args.warmup:
            times.append(dt)
    counts = counts.as_dict()
    t = torch.tensor([sum(times)], dtype=torch.float64, device=torch.device("cuda", local))
    nw = torch.tensor([float(word_start[-1])], dtype=torch.float64, device=torch.device("cuda", local))
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(nw, op=dist.ReduceOp.SUM)
    if rank == 0:
        sec = float(t.item()) / args.steps
        value = float(nw.item()) / sec / 1e9
        line = {"metric": "decode_kernel_cubin_throughput", "value": value, "unit": UNIT, "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "u32", "data": "synthetic",
                "config": {"workload": "cfg4 multi-kernel cubin: parse + one decode launch per GPU over all kernels; pinned host "
                                       "buffers in and out", "kernels_per_gpu": args.kernels,
                           "words_per_gpu": int(word_start[-1]), "image_bytes": len(image), "sections": 9 + 4 * args.kernels},
                "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": int(word_start[-1]) * 16,
                        "d2h_bytes_per_step": int(word_start[-1]) * 38},
                "gpu_launches": args.steps, "counts": counts}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
DEFAULT_WORDS = 64 * 1024 * 1024    # 1 GiB of 16-byte words
STREAM_SEED = 1
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum per word of one captured launch, from the ncu summaries
# under profiles/ (smaller cases than the bench's, scaled by the word count: the traffic is the
# stream itself, read and written once).  decode: (268.7 MB + 580.7 MB) / 16 Mi words;
# encode: (319.0 MB + 99.8 MB) / 8 Mi; roundtrip: (134.5 MB + 6.2 MB) / 8 Mi.  Part of the last
# writes of a captured launch is still in L2 when it ends, more so in the smaller captures.
NCU_DRAM_BYTES_PER_WORD = {"decode": 50.6, "encode": 49.9, "roundtrip": 16.8}


def env_int(name, default):
    return int(os.environ.get(name, default))


def hbm_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(index), "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def finish(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "note": "nvidia-smi unavailable"}
        time.sleep(0.15)
        self.proc.terminate()
        out, _ = self.proc.communicate(timeout=10)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def oracle_rate(words_np, threads, seconds=15.0):
    """Oracle decode throughput (insn/s) on a bounded prefix of `words_np`."""
    sys.path.insert(0, str(ROOT / "oracle"))
    from oracle_lib import Oracle
    o = Oracle()
    probe = min(len(words_np), 1 << 18)
    t0 = time.perf_counter()
    o.decode_batch(words_np[:probe], threads=threads)
    rate = probe / max(time.perf_counter() - t0, 1e-6)
    n = int(max(probe, min(len(words_np), rate * seconds)))
    t0 = time.perf_counter()
    o.decode_batch(words_np[:n], threads=threads)
    dt = time.perf_counter() - t0
    return n / dt, n, dt


def run_reference(args, rank):
    """`--impl reference`: the reference's CPU algorithm (C++ port) on all host cores, rank 0 only."""
    if rank != 0:
        return
    sys.path.insert(0, str(ROOT / "oracle"))
    from oracle_lib import Oracle
    threads = len(os.sched_getaffinity(0))
    o = Oracle()
    # Bounded sample of the benchmark stream: the first `sample` words, sized from a probe so that
    # warmup + steps stay within a few minutes.
    probe = 1 << 18
    words = o.synth(1, STREAM_SEED, probe, threads=threads, records=False)
    t0 = time.perf_counter()
    o.decode_batch(words, threads=threads)
    rate = probe / max(time.perf_counter() - t0, 1e-6)
    total_steps = args.steps + args.warmup
    sample = int(min(args.words, max(probe, rate * min(20.0, 150.0 / total_steps))))
    words = o.synth(1, STREAM_SEED, sample, threads=threads, records=False)
    for _ in range(args.warmup):
        o.decode_batch(words, threads=threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        o.decode_batch(words, threads=threads)
    dt = time.perf_counter() - t0
    value = sample * args.steps / dt / 1e9
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u32", "data": "synthetic",
            "config": {"workload": "cfg1 batch decode, Zipf(1.1) forms, seed 1", "words_per_step": sample,
                       "words_per_gpu_in_gpu_arm": args.words},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                             "sample": f"first {sample} words of the stream, {args.steps} passes; C++ port of the "
                                       "reference decoder (the Rust crate cannot be built on this box)"},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def run_e2e(args, codec, n, first, form, barrier, rank, world, dev):
    """The batch through the host-buffer entry point: pinned host memory, copies inside the timed
    region.  Also times the CPU oracle on the same host words (rank 0 of a 1-GPU run)."""
    import numpy as np
    import torch
    import torch.distributed as dist

    import cubit_b200
    lib, ctx = codec._lib, codec._ctx
    sizes = {"words": n * 16, "form": n * 2, "slots": n * 32, "ctrl": n * 4}
    host = {}
    for name, b in sizes.items():
        p = C.c_void_p()
        codec._check(lib.cubit_host_alloc(ctx, b, C.byref(p)))
        host[name] = p
    torch.cuda.synchronize()
    codec._check(lib.cubit_synth_batch(ctx, cubit_b200.MIX_ZIPF, STREAM_SEED, 0, first, n, host["words"], None, None, None, 0, None))

    def e2e_step():
        codec._check(lib.cubit_decode_batch(ctx, host["words"], n, host["form"], host["slots"], host["ctrl"], None, 0, None))

    e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    t = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = world * n * args.e2e_steps / float(t.item()) / 1e9
    # The device path and the host path must agree on the result.
    host_form = np.ctypeslib.as_array(C.cast(host["form"], C.POINTER(C.c_uint16)), shape=(n,))
    same = bool((torch.from_numpy(host_form[: 1 << 20].astype(np.int16)) == form[: 1 << 20].cpu()).all())
    e2e = {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": sizes["words"],
           "d2h_bytes_per_step": sizes["form"] + sizes["slots"] + sizes["ctrl"], "steps": args.e2e_steps,
           "matches_device_path": same}
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = len(os.sched_getaffinity(0))
        sample_words = np.ctypeslib.as_array(C.cast(host["words"], C.POINTER(C.c_uint8)), shape=(n, 16))
        rate, used, dt = oracle_rate(sample_words, threads)
        cpu = {"value": rate / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": f"first {used} words of the same stream in {dt:.1f} s; C++ port of the reference decoder "
                         "(the Rust crate cannot be built on this box)"}
    for p in host.values():
        lib.cubit_host_free(ctx, p)
    return e2e, cpu


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--words", type=int, default=DEFAULT_WORDS, help="words per GPU per step")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--kernels", type=int, default=1000, help="cubin workload: kernels per GPU (cfg4 uses 10000 in all)")
    ap.add_argument("--workload", default="decode", choices=sorted(WORKLOADS) + ["cubin"],
                    help="decode is the headline (cfg1); encode / roundtrip report the other two kernels")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (for profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank, world, local = env_int("RANK", 0), env_int("WORLD_SIZE", 1), env_int("LOCAL_RANK", 0)
    if args.impl == "reference":
        run_reference(args, rank)
        return

    if args.workload == "cubin":
        run_cubin(args, rank, world, local)
        return

    import numpy as np
    import torch
    import torch.distributed as dist

    import cubit_b200

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the codec has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    codec = cubit_b200.Codec(devices=(local,))
    n = args.words
    first = rank * n    # every rank owns its own contiguous range of one stream

    wl = WORKLOADS[args.workload]
    words = torch.empty(n * 16, dtype=torch.uint8, device=dev)
    form = torch.empty(n, dtype=torch.int16, device=dev)
    slots = torch.empty(8 * n, dtype=torch.int32, device=dev)
    ctrl = torch.empty(n, dtype=torch.int32, device=dev)
    status = torch.empty(n, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream()
    sptr = stream.cuda_stream
    codec.synth_device(cubit_b200.MIX_ZIPF, STREAM_SEED, n, words_ptr=words.data_ptr(), form_ptr=form.data_ptr(),
                       slots_ptr=slots.data_ptr(), ctrl_ptr=ctrl.data_ptr(), noise_ppm=wl["noise_ppm"], first=first, stream=sptr)
    torch.cuda.synchronize()

    if args.workload == "decode":
        def step():
            codec.decode_device(words.data_ptr(), n, form.data_ptr(), slots.data_ptr(), ctrl.data_ptr(), stream=sptr)
    elif args.workload == "encode":
        def step():
            codec.encode_device(form.data_ptr(), slots.data_ptr(), ctrl.data_ptr(), n, words.data_ptr(), stream=sptr)
    else:
        def step():
            codec.roundtrip_device(words.data_ptr(), n, status.data_ptr(), stream=sptr)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    evs[0].record(stream)
    for k in range(args.steps):
        step()
        evs[k + 1].record(stream)
    barrier()
    clocks = sampler.finish() if sampler else None
    total_ms = evs[0].elapsed_time(evs[-1])
    per_launch_ms = [evs[k].elapsed_time(evs[k + 1]) for k in range(args.steps)]
    t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    value = world * n / (ms_per_step * 1e-3) / 1e9
    if args.workload == "roundtrip":
        counts = codec.roundtrip_device(words.data_ptr(), n, status.data_ptr(), stream=sptr, want_counts=True)
    elif args.workload == "decode":
        counts = codec.decode_device(words.data_ptr(), n, form.data_ptr(), slots.data_ptr(), ctrl.data_ptr(), stream=sptr,
                                     want_counts=True)
    else:
        counts = None

    e2e, cpu = None, None
    if not args.no_e2e and args.workload == "decode":
        e2e, cpu = run_e2e(args, codec, n, first, form, barrier, rank, world, dev)

    if rank == 0:
        peak, peak_kind = hbm_peak()
        kernel_ms = statistics.mean(per_launch_ms)
        achieved = wl["bytes"] * n / (kernel_ms * 1e-3) / 1e9
        line = {"metric": wl["metric"], "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "u32", "data": "synthetic",
                "config": {"workload": wl["text"],
                           "words_per_gpu": n, "seed": STREAM_SEED, "l2": "inputs larger than L2 (1 GiB of words per GPU)",
                           "sharding": "contiguous ranges of one stream, no collective"},
                "e2e": e2e,
                "gpu_launches": args.steps,
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                             "peak_kind": f"of {peak_kind}", "kernel": wl["kernel"], "kernel_ms": kernel_ms,
                             "bytes_per_insn": wl["bytes"],
                             "traffic": NCU_DRAM_BYTES_PER_WORD[args.workload] * n
                             if args.workload in NCU_DRAM_BYTES_PER_WORD else None},
                "counts": counts, "clocks": clocks}
        if cpu:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
