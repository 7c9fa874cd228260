"""Frame sharding and the final gather, world_size 2 over gloo on the CPU."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from velox_voice_b200.stack import StackConfig, gather_rows, shard_capacity, shard_rows


def test_shards_cover_all_frames_without_overlap():
    for total in (0, 1, 7, 90000, 89999, 24000, 129):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_rows(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                assert a1 == b0 and a0 <= a1
            assert all(s % 2 == 0 for s, _ in spans if s < total)  # row pairs stay together
            assert all(e - s <= shard_capacity(total, world) for s, e in spans)


def test_cfg5_shards_are_equal():
    assert [shard_rows(90000, 8, r) for r in range(8)] == [(11250 * r, 11250 * (r + 1)) for r in range(8)]


def test_flops_per_frame_matches_hand_count():
    # 12 blocks x 12,582,912 + CTC 2 * 512 * 5538
    assert StackConfig().flops_per_frame() == 156_665_856


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, total, cols, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = torch.arange(total * cols, dtype=torch.float32).reshape(total, cols)
        a, b = shard_rows(total, world, rank)
        got = gather_rows(full[a:b].clone(), total, world, rank)
        ids = gather_rows(full[a:b].argmax(dim=1, keepdim=True).int(), total, world, rank)
        q.put((rank, bool(torch.equal(got, full)), bool(torch.equal(ids[:, 0], full.argmax(dim=1).int()))))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("total", [10, 7, 1])
def test_gather_rows_world2_gloo(total):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, total, 3, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res == [(0, True, True), (1, True, True)]
