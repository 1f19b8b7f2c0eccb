"""Range sharding over ranks: pure host logic, exercised with a world of 2 on the gloo backend."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

from cubit_b200 import shard_range, shard_sections

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("n,world", [(0, 1), (1, 3), (10, 3), (47244, 8), (1 << 28, 8), (7, 8)])
def test_shard_ranges_tile_the_stream(n, world):
    ranges = [shard_range(n, world, r) for r in range(world)]
    assert ranges[0][0] == 0 and ranges[-1][1] == n
    assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
    sizes = [e - b for b, e in ranges]
    assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(n, world, world)


def test_shard_sections_balances_kernels_by_words():
    rng = np.random.default_rng(0)
    counts = np.clip(np.exp(rng.normal(np.log(20000), 1.0, 1000)), 2000, 200000).astype(int).tolist()
    world = 8
    total, seen = sum(counts), []
    for r in range(world):
        pieces = shard_sections(counts, world, r)
        words = sum(p[2] for p in pieces)
        assert abs(words - total / world) <= 1
        seen += pieces
    # every word of every kernel exactly once, in order
    rebuilt = {}
    for k, first, n in seen:
        assert rebuilt.get(k, 0) == first
        rebuilt[k] = first + n
    assert [rebuilt[k] for k in range(len(counts))] == counts


def _worker(rank, world, port, out):
    import torch.distributed as dist
    sys.path.insert(0, str(ROOT)); sys.path.insert(0, str(ROOT / "oracle"))
    from oracle_lib import Oracle
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    n = 20001
    oracle = Oracle()
    begin, end = shard_range(n, world, rank)
    # each rank produces and decodes only its own range of the stream; results are gathered on the host
    words = oracle.synth(1, 42, end - begin, noise_ppm=10000, first=begin, records=False)
    form, slots, ctrl = oracle.decode_batch(words)
    gathered = [None] * world
    dist.all_gather_object(gathered, (begin, end, words, form, ctrl))
    dist.barrier()
    if rank == 0:
        whole = oracle.synth(1, 42, n, noise_ppm=10000, records=False)
        wform, _, wctrl = oracle.decode_batch(whole)
        ok = True
        for b, e, w, f, c in gathered:
            ok &= bool((w == whole[b:e]).all() and (f == wform[b:e]).all() and (c == wctrl[b:e]).all())
        out.put(ok and gathered[0][0] == 0 and gathered[-1][1] == n)
    dist.destroy_process_group()


def test_two_ranks_on_gloo_reproduce_the_single_rank_result():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert out.get(timeout=5) is True
