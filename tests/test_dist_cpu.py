"""Host-side logic of the multi-GPU paths on two CPU ranks (gloo): the N-sharded
linear's all-gather reassembly and the expert-parallel dispatch / combine index
arithmetic.  The local compute is a plain torch stand-in, so these tests check
the exchange, not the kernels (those are checked by the GPU tests)."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from garnet_b200.dist import ExpertParallelMoe, ShardedLinear
    ok = True
    # ---- N-sharded linear: every rank holds rows [r*N/G, (r+1)*N/G) of W
    g = torch.Generator().manual_seed(0)
    n, k, m = 12, 8, 3
    w = torch.randn(n, k, generator=g)
    x = torch.randn(m, k, generator=g)
    local = w[rank * n // world:(rank + 1) * n // world]
    lin = ShardedLinear(lambda a: a @ local.T, n)
    ok &= torch.allclose(lin.forward(x), x @ w.T, atol=1e-6)

    # ---- expert-parallel MoE with a toy expert: f_e(row) = row * (e + 1) + e
    experts, topk, hidden = 8, 2, 4
    tokens = 5 + rank                                  # ragged: ranks hold different token counts
    gx = torch.Generator().manual_seed(100 + rank)
    xt = torch.randn(tokens, hidden, generator=gx).bfloat16().float()
    sel = torch.stack([torch.randperm(experts, generator=gx)[:topk] for _ in range(tokens)]).to(torch.int32)
    if rank == 1:
        sel[:] = torch.tensor([0, 1], dtype=torch.int32)     # skew: rank 1 sends everything to rank 0
    probs = torch.rand(tokens, topk, generator=gx)
    per = experts // world

    def experts_on_rows(rows, row_expert):
        assert ((row_expert // per) == rank).all()          # only rows of local experts arrive
        e = row_expert.float()[:, None]
        return (rows * (e + 1) + e).bfloat16().float()

    def combine(vals, p):
        return (vals.reshape(p.shape[0], topk, -1) * p[:, :, None]).sum(1)

    moe = ExpertParallelMoe(lambda a: (sel, probs), experts_on_rows, combine, experts, topk)
    y = moe.forward(xt)
    e = sel.float()[:, :, None]
    expect = ((xt[:, None, :] * (e + 1) + e).bfloat16().float() * probs[:, :, None]).sum(1)
    ok &= torch.allclose(y, expect, atol=1e-6)
    ok &= moe.last_recv_rows >= 0
    results[rank] = bool(ok)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_exchange_logic():
    world = 2
    port = 29500 + os.getpid() % 2000
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert all(results.get(r) for r in range(world)), dict(results)


def test_dispatch_plan_is_stable_and_complete():
    sys.path.insert(0, ROOT)
    from garnet_b200.dist import dispatch_plan
    sel = torch.tensor([[5, 0], [1, 6], [7, 2], [0, 4]], dtype=torch.int32)
    order, counts, dest_expert = dispatch_plan(sel, experts=8, world=4)
    assert counts.tolist() == [3, 1, 2, 2]
    assert order.tolist() == [1, 2, 6, 5, 0, 7, 3, 4]      # by destination rank, slot order kept inside a rank
    assert dest_expert.tolist() == [0, 1, 0, 2, 5, 4, 6, 7]
