#!/usr/bin/env python
"""Benchmark of the batch SM120 codec: Ginsn/s on synthetic instruction streams.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--words M]

One step = one pass of a kernel over one batch (default 64 Mi words = 1 GiB, forms Zipf(1.1) over a
seeded permutation of the instruction keys; the stream is synthetic because the reference's own
corpus is private).  Rank 0 prints one JSON line:

* headline `value`: cfg1 batch decode, CUDA events around K back-to-back launches on device-resident
  buffers.  With N > 1 (torchrun, one rank per GPU) every rank decodes its own 64 Mi-word range of the
  same stream: weak scaling, no collective on the data path;
* `encode` (cfg2: the generator's records back to words) and `roundtrip` (cfg3's mix, 1 % raw random
  words) timed the same way, each with its own roofline;
* `cfg3_strong`: ONE stream of 256 Mi words range-sharded over the ranks (strong scaling);
* `e2e` / `roundtrip_e2e`: the same batch through the host-buffer entry points (pinned host memory,
  copies in and out inside the timed region) and `copy_only`, the same copies without a kernel;
* `single_process` (N > 1): rank 0 alone drives all N GPUs through one context;
* `cpu_baseline` / `--impl reference`: the CPU oracle (a C++ port of the reference's decoder; the
  Rust original cannot be built here) on the host cores.
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
# dram__bytes_read.sum + dram__bytes_write.sum per word of one captured launch, from the newest ncu summaries
# under profiles/ (8 Mi-word captures, scaled by the word count: the traffic is the stream itself, read
# and written once).  decode: (134.46 MB + 261.45 MB) / 8 Mi words; encode: (319.2 MB + 98.1 MB) / 8 Mi;
# roundtrip: (134.47 MB + 6.85 MB) / 8 Mi.  Part of the last writes of a captured launch is still in L2 when it ends.
NCU_DRAM_BYTES_PER_WORD = {"decode": 47.20, "encode": 49.74, "roundtrip": 16.85}
# The capture each figure comes from (summaries under profiles/).
NCU_CAPTURE = {"decode": "profiles/decode_kernel_zipf.md", "encode": "profiles/encode_kernel_records.md",
               "roundtrip": "profiles/roundtrip_kernel_mix.md"}


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
                                          "-i", str(index), "-lms", "25"], stdout=subprocess.PIPE,
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
    """`--impl reference`: the reference's CPU algorithm (C++ port) on all host cores, rank 0 only, on the same
    workload as the GPU arm: the first `--words` words of the cfg1 stream, every pass."""
    if rank != 0:
        return
    sys.path.insert(0, str(ROOT / "oracle"))
    from oracle_lib import Oracle
    threads = len(os.sched_getaffinity(0))
    o = Oracle()
    words = o.synth(1, STREAM_SEED, args.words, threads=threads, records=False)
    # One untimed pass gives the time of a pass; the timed passes are args.steps unless that would take
    # more than about four minutes, in which case fewer are run and the line says how many.
    t0 = time.perf_counter()
    o.decode_batch(words, threads=threads)
    one = time.perf_counter() - t0
    warm = max(0, min(args.warmup, int(30.0 / max(one, 1e-6))) - 1)
    for _ in range(warm):
        o.decode_batch(words, threads=threads)
    passes = max(1, min(args.steps, int(240.0 / max(one, 1e-6))))
    t0 = time.perf_counter()
    for _ in range(passes):
        o.decode_batch(words, threads=threads)
    dt = time.perf_counter() - t0
    value = args.words * passes / dt / 1e9
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / passes * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u32", "data": "synthetic",
            "config": config_of(args.words),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                             "sample": f"all {args.words} words of the GPU arm's per-GPU batch, {passes} timed passes of "
                                       f"{args.steps} asked for ({warm + 1} untimed before); C++ port of the reference "
                                       "decoder (the Rust crate cannot be built on this box)"},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def config_of(n):
    """The workload description shared by both arms."""
    in_bytes = n * 16
    return {"workload": WORKLOADS["decode"]["text"], "words_per_gpu": n, "seed": STREAM_SEED,
            "l2": (f"inputs larger than L2 ({in_bytes / 2**20:.0f} MiB of words and {n * 38 / 2**20:.0f} MiB of records per GPU "
                   "against 126 MB)") if in_bytes > 126e6 else
                  f"inputs of {in_bytes / 2**20:.0f} MiB fit the 126 MB L2: not a valid bench size",
            "sharding": "contiguous ranges of one stream, no collective"}


class PinnedBuffers:
    """Host buffers from cubit_host_alloc (pinned), freed together."""

    def __init__(self, codec):
        self.codec, self.ptrs = codec, {}

    def add(self, name, nbytes):
        p = C.c_void_p()
        self.codec._check(self.codec._lib.cubit_host_alloc(self.codec._ctx, nbytes, C.byref(p)))
        self.ptrs[name] = p
        return p

    def array(self, name, ctype, shape):
        import numpy as np
        return np.ctypeslib.as_array(C.cast(self.ptrs[name], C.POINTER(ctype)), shape=shape)

    def free(self):
        for p in self.ptrs.values():
            self.codec._lib.cubit_host_free(self.codec._ctx, p)
        self.ptrs = {}


def load_cudart():
    """libcudart of the torch installation, for the copy-only leg (plain cudaMemcpyAsync, no kernel of anyone)."""
    import glob
    import torch
    roots = [Path(torch.__file__).parent / "lib", Path(torch.__file__).parent.parent / "nvidia" / "cuda_runtime" / "lib",
             Path("/usr/local/cuda/lib64")]
    for r in roots:
        for cand in sorted(glob.glob(str(r / "libcudart.so*"))):
            try:
                lib = C.CDLL(cand)
                lib.cudaMemcpyAsync.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]
                lib.cudaMemcpyAsync.restype = C.c_int
                lib.cudaSetDevice.argtypes = [C.c_int]
                lib.cudaSetDevice.restype = C.c_int
                return lib
            except OSError:
                continue
    return None


def run_copy_only(args, n, host, dev, barrier, world):
    """The copies of the host decode path and nothing else: the same pinned buffers, the same 4 Mi-word chunks on two
    streams (16 B in, then ten plane copies of 38 B out per word), no kernel.  Its rate is the roof of `e2e`."""
    import torch
    import torch.distributed as dist
    rt = load_cudart()
    if rt is None or rt.cudaSetDevice(dev.index):
        return None
    chunk = min(1 << 22, n)
    stage = [torch.empty(chunk * 54 + 4096, dtype=torch.uint8, device=dev) for _ in range(2)]
    streams = [torch.cuda.Stream(device=dev) for _ in range(2)]
    H2D, D2H = 1, 2
    words, form, slots, ctrl = (host.ptrs[k].value for k in ("words", "form", "slots", "ctrl"))

    def step():
        for k, at in enumerate(range(0, n, chunk)):
            m = min(chunk, n - at)
            s, st = streams[k & 1].cuda_stream, stage[k & 1].data_ptr()
            rc = rt.cudaMemcpyAsync(st, words + at * 16, m * 16, H2D, s)
            rc |= rt.cudaMemcpyAsync(form + at * 2, st + chunk * 16, m * 2, D2H, s)
            for p in range(8):
                rc |= rt.cudaMemcpyAsync(slots + (p * n + at) * 4, st + chunk * 18 + p * chunk * 4, m * 4, D2H, s)
            rc |= rt.cudaMemcpyAsync(ctrl + at * 4, st + chunk * 50, m * 4, D2H, s)
            if rc:
                raise RuntimeError(f"cudaMemcpyAsync failed ({rc})")
        for s in streams:
            s.synchronize()
    step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        step()
    dt = time.perf_counter() - t0
    t = torch.tensor([dt], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    sec = float(t.item()) / args.e2e_steps
    return {"value": world * n / sec / 1e9, "unit": UNIT, "bytes_per_insn": 54, "gb_per_s": world * n * 54 / sec / 1e9,
            "what": "cudaMemcpyAsync only: the host decode path's pinned buffers, chunks and streams, no kernel"}


def run_e2e(args, codec, n, first, form, status_dev, barrier, rank, world, dev):
    """The batch through the host-buffer entry points: pinned host memory, copies inside the timed region — decode
    (16 B in, 38 B out per word) and fused roundtrip (16 B in, 1 B out).  Also the copy-only leg on the same buffers
    and, on rank 0 of a 1-GPU run, the CPU oracle on the same host words."""
    import numpy as np
    import torch
    import torch.distributed as dist

    import cubit_b200
    lib, ctx = codec._lib, codec._ctx
    sizes = {"words": n * 16, "form": n * 2, "slots": n * 32, "ctrl": n * 4, "status": n}
    host = PinnedBuffers(codec)
    for name, b in sizes.items():
        host.add(name, b)
    torch.cuda.synchronize()
    codec._check(lib.cubit_synth_batch(ctx, cubit_b200.MIX_ZIPF, STREAM_SEED, 0, first, n, host.ptrs["words"], None, None, None, 0, None))

    def timed(fn):
        fn()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            fn()
        torch.cuda.synchronize()
        t = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return world * n * args.e2e_steps / float(t.item()) / 1e9

    e2e_value = timed(lambda: codec._check(lib.cubit_decode_batch(ctx, host.ptrs["words"], n, host.ptrs["form"], host.ptrs["slots"],
                                                                  host.ptrs["ctrl"], None, 0, None)))
    # The device path and the host path must agree on the result.
    host_form = host.array("form", C.c_uint16, (n,))
    k = min(n, 1 << 20)
    same = bool((torch.from_numpy(host_form[:k].astype(np.int16)) == form[:k].cpu()).all())
    assert same, "host-buffer decode and device-buffer decode disagree"
    e2e = {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": sizes["words"],
           "d2h_bytes_per_step": sizes["form"] + sizes["slots"] + sizes["ctrl"], "steps": args.e2e_steps,
           "matches_device_path": same}
    copy_only = run_copy_only(args, n, host, dev, barrier, world)
    if copy_only:
        e2e["link_frac"] = e2e_value / copy_only["value"]
    # Roundtrip of the same host words (no noise words in this stream: the device leg has its own mix).
    rt_value = timed(lambda: codec._check(lib.cubit_roundtrip_batch(ctx, host.ptrs["words"], n, host.ptrs["status"], None, 0, None)))
    e2e_rt = {"value": rt_value, "unit": UNIT, "h2d_bytes_per_step": sizes["words"], "d2h_bytes_per_step": sizes["status"],
              "steps": args.e2e_steps, "h2d_gb_per_s": rt_value * 16}
    del status_dev
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = len(os.sched_getaffinity(0))
        rate, used, dt = oracle_rate(host.array("words", C.c_uint8, (n, 16)), threads)
        cpu = {"value": rate / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": f"first {used} words of the same stream in {dt:.1f} s; C++ port of the reference decoder "
                         "(the Rust crate cannot be built on this box)"}
    host.free()
    return e2e, e2e_rt, copy_only, cpu


def run_single_process(args, n, per_rank_form_sample, rank, world):
    """Rank 0 alone: one context over all `world` GPUs, one host batch through the host-buffer entry points, which
    shard it inside the library (one host thread per GPU).  Checked against the oracle on a strided sample."""
    import numpy as np

    import cubit_b200
    del per_rank_form_sample
    codec = cubit_b200.Codec(devices=tuple(range(world)))
    lib, ctx = codec._lib, codec._ctx
    host = PinnedBuffers(codec)
    for name, b in {"words": n * 16, "form": n * 2, "slots": n * 32, "ctrl": n * 4, "status": n}.items():
        host.add(name, b)
    codec._check(lib.cubit_synth_batch(ctx, cubit_b200.MIX_ZIPF, STREAM_SEED, 10000, 0, n, host.ptrs["words"], None, None, None, 0, None))
    out = {}
    calls = {"decode": lambda: lib.cubit_decode_batch(ctx, host.ptrs["words"], n, host.ptrs["form"], host.ptrs["slots"],
                                                      host.ptrs["ctrl"], None, 0, None),
             "roundtrip": lambda: lib.cubit_roundtrip_batch(ctx, host.ptrs["words"], n, host.ptrs["status"], None, 0, None)}
    for name, fn in calls.items():
        codec._check(fn())
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            codec._check(fn())
        out[name] = {"value": n * args.e2e_steps / (time.perf_counter() - t0) / 1e9, "unit": UNIT}
    sys.path.insert(0, str(ROOT / "oracle"))
    from oracle_lib import Oracle
    o = Oracle()
    sample = np.arange(0, n, max(1, n // 50000))
    words = host.array("words", C.c_uint8, (n, 16))[sample]
    of, os_, oc = o.decode_batch(words)
    ok = bool((host.array("form", C.c_uint16, (n,))[sample] == of).all() and (host.array("slots", C.c_uint32, (8, n))[:, sample] == os_).all()
              and (host.array("ctrl", C.c_uint32, (n,))[sample] == oc).all()
              and (host.array("status", C.c_uint8, (n,))[sample] == o.roundtrip_batch(words)).all())
    assert ok, "in-process sharded results differ from the oracle"
    host.free()
    codec.close()
    return {"devices": world, "words": n, "decode": out["decode"], "roundtrip": out["roundtrip"], "matches": ok,
            "checked_words": int(len(sample)),
            "what": "one process, one context over all GPUs, pinned host buffers sharded inside the library"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--words", type=int, default=DEFAULT_WORDS, help="words per GPU per step")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--kernels", type=int, default=1000, help="cubin workload: kernels per GPU (cfg4 uses 10000 in all)")
    ap.add_argument("--workload", default="all", choices=["all"] + sorted(WORKLOADS) + ["cubin"],
                    help="all (default): cfg1 decode as the headline plus encode, roundtrip and cfg3 strong scaling as "
                         "sub-records; decode / encode / roundtrip: that kernel only (for profiler captures)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer legs (for profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank, world, local = env_int("RANK", 0), env_int("WORLD_SIZE", 1), env_int("LOCAL_RANK", 0)
    if args.impl == "reference":
        run_reference(args, rank)
        return

    if args.workload == "cubin":
        run_cubin(args, rank, world, local)
        return

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
    stream = torch.cuda.current_stream()
    sptr = stream.cuda_stream

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def time_steps(step):
        """W warm-up launches, then K launches between events on the launching stream; max over ranks."""
        for _ in range(args.warmup):
            step()
        barrier()
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
        evs[0].record(stream)
        for k in range(args.steps):
            step()
            evs[k + 1].record(stream)
        barrier()
        total_ms = evs[0].elapsed_time(evs[-1])
        kernel_ms = statistics.mean(evs[k].elapsed_time(evs[k + 1]) for k in range(args.steps))
        t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / args.steps, kernel_ms

    peak, peak_kind = hbm_peak()

    def leg(name, items_all_ranks, items_this_rank, ms_per_step, kernel_ms):
        wl = WORKLOADS[name]
        achieved = wl["bytes"] * items_this_rank / (kernel_ms * 1e-3) / 1e9
        return {"metric": wl["metric"], "value": items_all_ranks / (ms_per_step * 1e-3) / 1e9, "unit": UNIT,
                "ms_per_step": ms_per_step,
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                             "peak_kind": f"of {peak_kind}", "kernel": wl["kernel"], "kernel_ms": kernel_ms,
                             "bytes_per_insn": wl["bytes"],
                             "traffic": NCU_DRAM_BYTES_PER_WORD[name] * items_this_rank,
                             "traffic_from": NCU_CAPTURE[name]}}

    which = sorted(WORKLOADS) if args.workload == "all" else [args.workload]
    words = torch.empty(n * 16, dtype=torch.uint8, device=dev)
    form = torch.empty(n, dtype=torch.int16, device=dev)
    slots = torch.empty(8 * n, dtype=torch.int32, device=dev)
    ctrl = torch.empty(n, dtype=torch.int32, device=dev)
    status = torch.empty(n, dtype=torch.uint8, device=dev)
    out_words = torch.empty(n * 16, dtype=torch.uint8, device=dev) if "encode" in which else None

    def synth(noise_ppm, records):
        codec.synth_device(cubit_b200.MIX_ZIPF, STREAM_SEED, n, words_ptr=words.data_ptr(),
                           form_ptr=form.data_ptr() if records else None, slots_ptr=slots.data_ptr() if records else None,
                           ctrl_ptr=ctrl.data_ptr() if records else None, noise_ppm=noise_ppm, first=first, stream=sptr)
        torch.cuda.synchronize()

    sampler = ClockSampler(local) if rank == 0 else None
    legs, counts, launches = {}, {}, 0
    if "encode" in which:
        # cfg2: the generator's own records of the cfg1 stream, encoded into a separate buffer.
        synth(0, True)
        ms, kms = time_steps(lambda: codec.encode_device(form.data_ptr(), slots.data_ptr(), ctrl.data_ptr(), n, out_words.data_ptr(),
                                                         stream=sptr))
        assert bool((out_words[: 1 << 24] == words[: 1 << 24]).all()), "encode of the generator's records differs from its words"
        legs["encode"] = leg("encode", world * n, n, ms, kms)
        launches += args.steps
    if "roundtrip" in which:
        synth(WORKLOADS["roundtrip"]["noise_ppm"], False)
        ms, kms = time_steps(lambda: codec.roundtrip_device(words.data_ptr(), n, status.data_ptr(), stream=sptr))
        counts["roundtrip"] = codec.roundtrip_device(words.data_ptr(), n, status.data_ptr(), stream=sptr, want_counts=True)
        legs["roundtrip"] = leg("roundtrip", world * n, n, ms, kms)
        launches += args.steps
    if "decode" in which:
        synth(0, False)
        ms, kms = time_steps(lambda: codec.decode_device(words.data_ptr(), n, form.data_ptr(), slots.data_ptr(), ctrl.data_ptr(),
                                                         stream=sptr))
        counts["decode"] = codec.decode_device(words.data_ptr(), n, form.data_ptr(), slots.data_ptr(), ctrl.data_ptr(), stream=sptr,
                                               want_counts=True)
        legs["decode"] = leg("decode", world * n, n, ms, kms)
        launches += args.steps

    cfg3 = None
    if args.workload == "all":
        # cfg3: ONE stream of 4 x --words words (256 Mi by default) with 1 % raw random words, cut into `world`
        # contiguous ranges; every rank runs the fused roundtrip on its own range.  Strong scaling: the total is fixed.
        total = 4 * n
        b, e = cubit_b200.shard_range(total, world, rank)
        mine = e - b
        w3 = torch.empty(mine * 16, dtype=torch.uint8, device=dev)
        s3 = torch.empty(mine, dtype=torch.uint8, device=dev)
        codec.synth_device(cubit_b200.MIX_ZIPF, STREAM_SEED, mine, words_ptr=w3.data_ptr(), noise_ppm=10000, first=b, stream=sptr)
        torch.cuda.synchronize()
        ms, kms = time_steps(lambda: codec.roundtrip_device(w3.data_ptr(), mine, s3.data_ptr(), stream=sptr))
        c3 = codec.roundtrip_device(w3.data_ptr(), mine, s3.data_ptr(), stream=sptr, want_counts=True)
        tot = torch.tensor([float(c3["n_exact"]), float(c3["n_mismatch"]), float(c3["n_rejected"])], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(tot, op=dist.ReduceOp.SUM)
        cfg3 = leg("roundtrip", total, mine, ms, kms)
        cfg3.update({"metric": "roundtrip_throughput_cfg3", "scaling": "strong", "total_words": total, "words_this_rank": mine,
                     "counts": dict(zip(("n_exact", "n_mismatch", "n_rejected"), (int(x) for x in tot.tolist()))),
                     "what": "one 4 x --words stream (256 Mi words by default), 1 % raw random words, range-sharded over the "
                             "ranks; time of K launches per rank, max over ranks"})
        assert sum(cfg3["counts"].values()) == total
        launches += args.steps
        del w3, s3
    clocks = sampler.finish() if sampler else None

    e2e = e2e_rt = copy_only = cpu = None
    if not args.no_e2e and "decode" in which:
        e2e, e2e_rt, copy_only, cpu = run_e2e(args, codec, n, first, form, status, barrier, rank, world, dev)

    single = None
    if world > 1 and args.workload == "all" and not args.no_e2e:
        barrier()
        if rank == 0:
            single = run_single_process(args, n, None, rank, world)
        barrier()

    if rank == 0:
        head = legs["decode"] if "decode" in legs else legs[which[0]]
        line = {"metric": head["metric"], "value": head["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "u32", "data": "synthetic", "config": config_of(n),
                "e2e": e2e, "gpu_launches": launches, "roofline": head["roofline"], "counts": counts.get("decode"),
                "clocks": clocks}
        if "decode" in counts:
            line["decoded_only"] = {"value": head["value"] * counts["decode"]["n_decoded"] / n, "unit": UNIT,
                                    "what": "words per second that decode to a form (the stream also holds words that no form "
                                            "matches; they are rejected on a shorter path)"}
        for name in ("encode", "roundtrip"):
            if name in legs and legs[name] is not head:
                line[name] = legs[name]
                line[name]["config"] = WORKLOADS[name]["text"]
        if "roundtrip" in counts and "roundtrip" in line:
            line["roundtrip"]["counts"] = counts["roundtrip"]
        if cfg3:
            line["cfg3_strong"] = cfg3
        if e2e_rt:
            line["roundtrip_e2e"] = e2e_rt
        if copy_only:
            line["copy_only"] = copy_only
        if single:
            line["single_process"] = single
        if cpu:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
