"""The multi-process sharding logic on CPU: world_size 2 over gloo, the oracle standing in for the device kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mimir_b200.shard import split_range


def test_split_range_partitions():
    for n in (0, 1, 7, 8, 128, 8192):
        for world in (1, 2, 3, 4, 8):
            spans = [split_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        split_range(4, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle as mo
    from mimir_b200 import shard

    g = torch.Generator().manual_seed(5)           # same global tensors on every rank
    a = torch.rand(12, 20, generator=g) * 2 - 1
    b = torch.rand(9, 20, generator=g) * 2 - 1     # stored [N,K], N = 9 does not divide by 2
    x = torch.randn(7, 16, generator=g)
    q, k, v = (torch.randn(5, 8, 4, generator=g) for _ in range(3))

    gemm = lambda aa, bb: torch.from_numpy(mo.gemm(aa.numpy(), bb.contiguous().numpy(), b_nk=True))
    c_local, (lo, hi) = shard.sharded_product_2d(a, b, gemm)
    assert c_local.shape == (12, hi - lo)
    c = shard.sharded_product_2d(a, b, gemm, gather=True)
    want = torch.from_numpy(mo.gemm(a.numpy(), b.numpy(), b_nk=True))
    assert torch.equal(c, want)

    soft = lambda xx: torch.from_numpy(mo.softmax_rows(xx.contiguous().numpy()))
    y = shard.sharded_rows(x, soft, gather=True)
    assert torch.equal(y, torch.from_numpy(mo.softmax_rows(x.numpy())))

    attn = lambda qq, kk, vv: torch.from_numpy(
        mo.attention(qq.contiguous().numpy(), kk.contiguous().numpy(), vv.contiguous().numpy(), scale=0.5, causal=True))
    o = shard.sharded_heads(q, k, v, attn, gather=True)
    assert torch.equal(o, torch.from_numpy(mo.attention(q.numpy(), k.numpy(), v.numpy(), scale=0.5, causal=True)))

    # max-over-ranks timing reduction as bench.py does it
    t = torch.tensor([float(rank + 1)], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert t.item() == world
    dist.barrier()
    dist.destroy_process_group()
    open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")


def test_two_rank_sharding_over_gloo(tmp_path):
    import oracle
    oracle.build()
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]
