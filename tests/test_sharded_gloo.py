"""Host logic of the multi-GPU path on CPU: shard planning, slicing a packed weight by rows, and
the all-gather that reassembles y, with two gloo ranks.  No kernel runs here."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from unifur_b200.sharded import column_shards, gather_columns, shard_packed_rows


def test_column_shards_cover_the_columns_once():
    for d_out, world, gran in ((14336, 8, 1), (11008, 8, 1), (3584, 8, 64), (512, 8, 64), (48, 4, 1),
                               (7, 8, 1), (18944, 8, 64), (100, 3, 64)):
        s = column_shards(d_out, world, gran)
        assert len(s) == world and s[0][0] == 0 and s[-1][1] == d_out
        for (a, b), (c, d) in zip(s[:-1], s[1:]):
            assert b == c and a <= b
        widths = [b - a for a, b in s]
        assert max(widths) - min(w for w in widths) <= max(gran, 1) or d_out < world * gran
        if d_out % (world * gran) == 0:
            assert len(set(widths)) == 1
    assert column_shards(14336, 8) == [(1792 * r, 1792 * (r + 1)) for r in range(8)]
    # the Qwen2-7B-shaped block: per-GPU widths 448 / 64 / 2368 / 448
    assert column_shards(3584, 8)[3] == (1344, 1792)
    assert column_shards(512, 8)[7] == (448, 512)
    assert column_shards(18944, 8)[0] == (0, 2368)


def test_shard_packed_rows_matches_requantizing_the_rows(oracle):
    rng = np.random.default_rng(3)
    d_out, d_in = 24, 128
    w = rng.standard_normal((d_out, d_in)).astype(np.float32)
    packed, absmax = oracle.quantize_packed(w)
    for a, b in column_shards(d_out, 3):
        codes, sc = shard_packed_rows(torch.from_numpy(packed), torch.from_numpy(absmax), d_in, (a, b))
        p2, a2 = oracle.quantize_packed(w[a:b])
        assert np.array_equal(codes.numpy(), p2) and np.array_equal(sc.numpy(), a2)
    with pytest.raises(ValueError):
        shard_packed_rows(torch.from_numpy(packed), torch.from_numpy(absmax), 100, (0, 1))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, d_out, gran, ok):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rows = 5
        shards = column_shards(d_out, world, gran)
        a, b = shards[rank]
        full = (torch.arange(rows).view(-1, 1) * 1000 + torch.arange(d_out).view(1, -1)).float()
        y = gather_columns(full[:, a:b].contiguous(), shards)
        good = torch.equal(y, full)
        out = torch.full((rows, d_out), -1.0)
        gather_columns(full[:, a:b].to(torch.bfloat16).contiguous().float(), shards, out=out)
        good = good and torch.equal(out, full.to(torch.bfloat16).float())
        try:
            gather_columns(full[:, : (b - a) + 1], shards)
            good = False
        except ValueError:
            pass
        ok[rank] = int(good)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("d_out,gran", [(64, 1), (70, 1), (192, 64), (5, 1)])
def test_gather_columns_two_gloo_ranks(d_out, gran):
    world = 2
    ctx = mp.get_context("spawn")
    ok = ctx.Array("i", [0] * world)
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, d_out, gran, ok)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert list(ok) == [1] * world
