"""World-size-2 CPU test of the multi-GPU host logic: two ranks shard the sessions, each
runs the shared GptDecoder wrapper on its block (CPU checker as the backend), the token rows
are gathered on the host, and the result equals the single-process run."""
import os
import socket
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _greedy_rows(rows_range, steps):
    sys.path.insert(0, ROOT)
    from tests.helpers import cpu_decoder, kv_model
    from tests.workloads import kv_test_tokens
    from tnsr_b200.nn import argmax_last
    model = kv_model(12)
    prompts = kv_test_tokens(5, 4)
    out = []
    start, count = rows_range
    if count == 0:
        return out
    dec = cpu_decoder(model, count)
    rows = [list(p) for p in prompts[start:start + count]]
    logits = dec.decode([t for r in rows for t in r]).reshape(count, 4, 367)
    for _ in range(steps):
        nxt = [argmax_last(logits[b, -1]) for b in range(count)]
        for r, t in zip(rows, nxt):
            r.append(t)
        logits = dec.decode(nxt).reshape(count, 1, 367)
    return rows


def _worker(rank, world, port, queue):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    from tnsr_b200.sharding import gather_token_rows, shard_sessions
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rows = _greedy_rows(shard_sessions(5, world, rank), steps=5)
        everything = gather_token_rows(rows)
        dist.barrier()
        if rank == 0:
            queue.put(everything)
    finally:
        dist.destroy_process_group()


def test_shard_sessions_partitions_exactly():
    from tnsr_b200.sharding import shard_sessions
    for total in (0, 1, 5, 256, 257):
        for world in (1, 2, 4, 8):
            blocks = [shard_sessions(total, world, r) for r in range(world)]
            assert sum(c for _, c in blocks) == total
            assert blocks[0][0] == 0
            for (s0, c0), (s1, _) in zip(blocks, blocks[1:]):
                assert s1 == s0 + c0
            assert max(c for _, c in blocks) - min(c for _, c in blocks) <= 1
    assert shard_sessions(256, 8, 3) == (96, 32)
    with pytest.raises(ValueError):
        shard_sessions(4, 2, 2)


def test_two_ranks_reproduce_the_single_process_tokens():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, queue)) for r in range(2)]
    for p in procs:
        p.start()
    result = queue.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert result == _greedy_rows((0, 5), steps=5)
