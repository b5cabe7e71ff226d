"""Multi-GPU host logic on CPU: the row partition, chunk-keyed data generation, and the
max-over-ranks reduction, as world-size-2 gloo processes.  The path has no data-path collective,
so what has to hold is that (1) the shards tile the token rows exactly, (2) a rank's rows are
bit-identical to the same rows of the whole matrix, and (3) per-rank results concatenate to the
whole result (checked with the CPU oracle standing in for the kernel)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kernel_pocs_b200 import workloads as W
from oracle import oracle as O


def test_row_shard_tiles_exactly():
    for total in (0, 1, 7, 8, 65536, 68298):
        for world in (1, 2, 3, 4, 8):
            spans = [W.row_shard(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            for (a, b), (c, d) in zip(spans, spans[1:]):
                assert b == c and a <= b
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        W.row_shard(10, 2, 2)


def test_workload_table_matches_the_benchmark_configurations():
    ws = W.workloads()
    assert (ws["c1"].tokens, ws["c1"].width, ws["c1"].dtype) == (256, 1024, torch.float32)
    assert (ws["c2"].tokens, ws["c2"].width, ws["c2"].dtype) == (32768, 14336, torch.bfloat16)
    assert (ws["c5"].tokens, ws["c5"].width) == (65536, 28672)
    lens = W.varlen_lengths()
    assert len(lens) == 16 and all(1 <= n <= 8192 for n in lens) and ws["c3"].tokens == sum(lens)
    assert ws["c3"].width == 11008 and ws["c3"].std == 2.0
    assert ws["c2"].bytes_fwd() == 3 * 32768 * 14336 * 2 and ws["c2"].bytes_bwd() == 5 * 32768 * 14336 * 2


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, tokens: int, width: int):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = W.Workload("t", tokens, width, torch.bfloat16, 5)
        lo, hi = W.row_shard(tokens, world, rank)
        gate, up, dh = W.generate_rows(w, lo, hi, "cpu")
        h = O.fwd(gate, up, 1.0, 1.0, "once")
        dgate, dup = O.bwd(dh, gate, up, 1.0, 1.0, "once")
        # what bench.py reduces: the slowest rank's time, and the total tokens
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        n = torch.tensor([hi - lo])
        dist.all_reduce(n, op=dist.ReduceOp.SUM)
        assert t.item() == world and n.item() == tokens
        parts = [None] * world
        dist.all_gather_object(parts, (lo, hi, h.view(torch.int16), dgate.view(torch.int16), dup.view(torch.int16)))
        if rank == 0:
            parts.sort(key=lambda p: p[0])
            whole_gate, whole_up, whole_dh = W.generate_rows(w, 0, tokens, "cpu")
            want_h = O.fwd(whole_gate, whole_up, 1.0, 1.0, "once").view(torch.int16)
            want_dg, want_du = (x.view(torch.int16) for x in O.bwd(whole_dh, whole_gate, whole_up, 1.0, 1.0, "once"))
            assert torch.equal(torch.cat([p[2] for p in parts]), want_h)
            assert torch.equal(torch.cat([p[3] for p in parts]), want_dg)
            assert torch.equal(torch.cat([p[4] for p in parts]), want_du)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("tokens", [8192 + 37, 3])
def test_two_ranks_reproduce_the_whole(tokens):
    mp.spawn(_worker, args=(2, _free_port(), tokens, 96), nprocs=2, join=True)
