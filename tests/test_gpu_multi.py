"""Multi-GPU parity of the epilogue-fused all-gather (needs >= 2 CUDA devices; skipped otherwise)."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import oracle as mo
    from mimir_b200 import shard
    from mimir_b200 import tensor as T

    def bits(t):
        return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)

    g = torch.Generator().manual_seed(11)        # the same global tensors on every rank
    M, K, F, N = 512, 256, 1024, 512
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w1 = (torch.randn(K, F, generator=g) * 0.05).to(torch.bfloat16).cuda()
    w3 = (torch.randn(K, F, generator=g) * 0.05).to(torch.bfloat16).cuda()
    w2 = (torch.randn(F, N, generator=g) * 0.05).to(torch.bfloat16).cuda()
    fl, nl = F // world, N // world

    # plain contraction, column slabs gathered in the epilogue: every rank ends up with the whole product
    c = shard.GatheredMatrix(M, F)
    shard.gemm_gather(x, w1[:, rank * fl:(rank + 1) * fl].contiguous(), c, rank * fl)
    c.barrier()
    want = mo.gemm_truth(bits(x), bits(w1), bf16=True)
    assert mo.normalised_error(c.local.float().cpu().numpy(), want) <= 2e-2
    assert torch.equal(c.local, T.product_2d(x, w1))           # same kernel, same bits, whichever rank wrote the slab

    # tensor-parallel gated MLP
    h = shard.GatheredMatrix(M, F)
    y = shard.tp_mlp_gated(x, w1[:, rank * fl:(rank + 1) * fl].contiguous(), w3[:, rank * fl:(rank + 1) * fl].contiguous(),
                           w2[:, rank * nl:(rank + 1) * nl].contiguous(), h)
    T.device_status()
    wanty = mo.mlp_gated_truth(bits(x), bits(w1), bits(w3), bits(w2))[:, rank * nl:(rank + 1) * nl]
    assert mo.normalised_error(y.float().cpu().numpy(), wanty) <= 2e-2

    # the same block with W2 split by rows: no gather of H, f32 partials of Y reduce-scattered; rank g ends with rows g M/G ..
    h_loc = torch.empty((M, fl), dtype=torch.bfloat16, device="cuda")
    yr = shard.tp_mlp_gated_rows(x, w1[:, rank * fl:(rank + 1) * fl].contiguous(), w3[:, rank * fl:(rank + 1) * fl].contiguous(),
                                 w2[rank * fl:(rank + 1) * fl, :].contiguous(), h_loc)
    T.device_status()
    per = M // world
    wantr = mo.mlp_gated_truth(bits(x), bits(w1), bits(w3), bits(w2))[rank * per:(rank + 1) * per]
    assert yr.shape == (per, N) and mo.normalised_error(yr.float().cpu().numpy(), wantr) <= 2e-2
    # ... and with the reduce-scatter fused into the second contraction's epilogue (bulk reductions into the owners' row
    # blocks): twice, the accumulators are reused
    acc = shard.GatheredMatrix(per, N, dtype=torch.float32)
    for _ in range(2):
        yf = shard.tp_mlp_gated_rows_fused(x, w1[:, rank * fl:(rank + 1) * fl].contiguous(), w3[:, rank * fl:(rank + 1) * fl].contiguous(),
                                           w2[rank * fl:(rank + 1) * fl, :].contiguous(), h_loc, acc)
        T.device_status()
        assert yf.shape == (per, N) and mo.normalised_error(yf.float().cpu().numpy(), wantr) <= 2e-2
        assert mo.normalised_error(yf.float().cpu().numpy(), yr.float().cpu().numpy()) <= 1e-2

    # a slab large enough for the paired-SM kernel (>= 74 tiles of 256 x 256 per rank): its epilogue sends each piece with
    # one bulk store per destination. The product is checked bit for bit against the one-GPU product of the same operands.
    M, K, fl, nl = 2560, 256, 2048, 256
    F, N = fl * world, nl * world
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w1 = (torch.randn(K, F, generator=g) * 0.05).to(torch.bfloat16).cuda()
    w3 = (torch.randn(K, F, generator=g) * 0.05).to(torch.bfloat16).cuda()
    w2 = (torch.randn(F, N, generator=g) * 0.02).to(torch.bfloat16).cuda()
    c = shard.GatheredMatrix(M, F)
    for _ in range(2):                                         # twice: the second pass overwrites a full buffer
        shard.gemm_gather(x, w1[:, rank * fl:(rank + 1) * fl].contiguous(), c, rank * fl)
        c.barrier()
        assert torch.equal(c.local, T.product_2d(x, w1))
        c.barrier()
    h = shard.GatheredMatrix(M, F)
    y = shard.tp_mlp_gated(x, w1[:, rank * fl:(rank + 1) * fl].contiguous(), w3[:, rank * fl:(rank + 1) * fl].contiguous(),
                           w2[:, rank * nl:(rank + 1) * nl].contiguous(), h)
    T.device_status()
    whole_y = T.mlp_gated(x, w1, w3, w2)
    whole = whole_y[:, rank * nl:(rank + 1) * nl].float().cpu().numpy()
    assert mo.normalised_error(y.float().cpu().numpy(), whole) <= 1e-2
    # W2 by rows, reduce-scatter in the epilogue, at the size where every CTA pair has tiles of several owners
    accl = shard.GatheredMatrix(M // world, N, dtype=torch.float32)
    hl = torch.empty((M, fl), dtype=torch.bfloat16, device="cuda")
    yf = shard.tp_mlp_gated_rows_fused(x, w1[:, rank * fl:(rank + 1) * fl].contiguous(), w3[:, rank * fl:(rank + 1) * fl].contiguous(),
                                       w2[rank * fl:(rank + 1) * fl, :].contiguous(), hl, accl, out_dtype=torch.float32)
    T.device_status()
    assert mo.normalised_error(yf.cpu().numpy(), whole_y[rank * (M // world):(rank + 1) * (M // world)].float().cpu().numpy()) <= 1e-2
    # the output all-gather fused into the second contraction as well: the whole Y on every rank
    yg = shard.GatheredMatrix(M, N)
    for mode in ("fused", "nccl"):
        full = shard.tp_mlp_gated(x, w1[:, rank * fl:(rank + 1) * fl].contiguous(), w3[:, rank * fl:(rank + 1) * fl].contiguous(),
                                  w2[:, rank * nl:(rank + 1) * nl].contiguous(), h, gather=mode, y=yg)
        T.device_status()
        assert full.shape == (M, N)
        assert mo.normalised_error(full.float().cpu().numpy(), whole_y.float().cpu().numpy()) <= 1e-2
        dist.barrier()
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")


def test_fused_all_gather_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    import __graft_entry__ as entry
    entry.build()
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]


def test_fused_all_gather_every_gpu(tmp_path):
    world = torch.cuda.device_count()
    if world < 4:
        pytest.skip("needs four or more GPUs")
    world = 8 if world >= 8 else 4
    import torch.multiprocessing as mp
    import __graft_entry__ as entry
    entry.build()
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == sorted(f"ok{r}" for r in range(world))
