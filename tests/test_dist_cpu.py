"""The multi-GPU exchange protocol on two CPU ranks (gloo): the placement rule of the
expert-parallel exchange (garnet_b200_moe_ep_plan_host, the rule the device kernels
follow), its fixed-capacity regions, counts, epoch flags and router-order combine,
restated on the host by garnet_b200.dist.HostExchange; and what happens when a rank
never posts its flag: the bounded wait ends with the device's fault code, nobody hangs.
The kernels themselves are checked by the GPU tests."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _toy_expert(rows, row_expert):
    e = row_expert.float()[:, None]
    return (rows * (e + 1) + e).bfloat16().float()


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from garnet_b200.dist import HostExchange
    ok = True
    experts, topk, hidden = 8, 2, 4
    per = experts // world
    tokens = 5 + rank                                  # ragged: ranks hold different token counts
    gx = torch.Generator().manual_seed(100 + rank)
    xt = torch.randn(tokens, hidden, generator=gx).bfloat16().float()
    sel = torch.stack([torch.randperm(experts, generator=gx)[:topk] for _ in range(tokens)]).to(torch.int32)
    if rank == 1:
        sel[:] = torch.tensor([0, 1], dtype=torch.int32)     # skew: rank 1 sends everything to rank 0
    probs = torch.rand(tokens, topk, generator=gx).bfloat16().float()

    def experts_on_rows(rows, row_expert):
        assert ((row_expert // per) == rank).all()           # only rows of local experts are run
        return _toy_expert(rows, row_expert)

    ex = HostExchange(experts, topk, hidden, tokens_local_max=8, limit_s=0.05)
    e = sel.float()[:, :, None]
    per_slot = (xt[:, None, :] * (e + 1) + e).bfloat16().float()
    expect = torch.zeros(tokens, hidden)
    for j in range(topk):
        expect = expect + per_slot[:, j] * probs[:, j:j + 1]
    for _ in range(2):                                       # two steps: the epoch moves on
        y = ex.step(xt, sel, probs, experts_on_rows)
        ok &= ex.fault == 0 and torch.equal(y, expect.bfloat16())
    # rows received: rank 0 owns experts 0..3 and gets all of rank 1's rows
    sent_to = [(sel.reshape(-1) // per == d).sum().item() for d in range(world)]
    totals = torch.tensor(sent_to)
    dist.all_reduce(totals)
    ok &= ex.rows_received == int(totals[rank])

    # a rank that never posts its flags: the other's wait runs out with code 71, and the
    # silent rank in turn never gets values back (72); both return, nobody hangs
    y = ex.step(xt, sel, probs, experts_on_rows, post_flags=(rank != 1))
    ok &= y is None and ex.fault in (71, 72)
    results[rank] = bool(ok)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_exchange_protocol_and_a_rank_that_never_posts():
    world = 2
    port = 29500 + os.getpid() % 2000
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert all(results.get(r) for r in range(world)), dict(results)


def test_placement_rule_is_stable_and_complete():
    sys.path.insert(0, ROOT)
    from garnet_b200.dist import plan_host
    sel = np.array([[5, 0], [1, 6], [7, 2], [0, 4]], np.int32)
    send_idx, counts = plan_host(sel, experts_per_rank=2, world=4)
    assert counts.tolist() == [3, 1, 2, 2]
    # slot order is kept inside a destination: slots 1, 2, 6 go to rank 0 in that order
    assert send_idx.tolist() == [0, 0, 1, 0, 1, 0, 2, 1]
    dest = sel.reshape(-1) // 2
    for d in range(4):
        assert sorted(send_idx[dest == d].tolist()) == list(range(counts[d]))
