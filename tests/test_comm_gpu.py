"""The library's own collectives and the expert-parallel exchange on GPUs, through the C ABI.

With one rank everything runs on one GPU (a rank's peer stores land in its own arena), which
checks the kernels, the placement rule, the fixed-capacity regions and the combine: the
exchange must reproduce the single-GPU operator bit for bit.  The cross-GPU tests start
one process per GPU and are skipped on a box with a single GPU; a wait whose partner
never shows up is tested with a flag that nothing writes (no GPU is made to hang or
fault: the wait's limit ends it and the status word reports it)."""
import os
import sys

import numpy as np
import pytest
import torch

import garnet_b200
from garnet_b200 import _lib, synth
from garnet_b200.dist import Channel, Comm, ExpertParallel, ep_arena_bytes

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def build_moe(case, **kw):
    moe = garnet_b200.GptOssMoe(case["hidden"], case["inter"], case["experts"], case["topk"], **kw)
    return moe.prepare(*[dev(case[k]) for k in ("router_w", "router_b", "gu_blocks", "gu_scales", "gu_bias",
                                                 "dn_blocks", "dn_scales", "dn_bias")])


def test_single_rank_collectives_and_bounded_wait():
    comm = Comm(1 << 20)
    ch = Channel(comm, 4096)
    x = torch.randn(1000, device="cuda")
    out = torch.zeros(1, 1000, device="cuda")
    for _ in range(3):                               # the regions alternate with the epoch
        ch.all_gather(x, out)
        assert torch.equal(out[0], x)
        red = torch.zeros_like(x)
        ch.all_reduce(x, red)
        assert torch.equal(red, x)
        ch.all_reduce(x, red, wire=torch.bfloat16)
        assert torch.equal(red, x.bfloat16().float())
        xb, rb = x.bfloat16(), torch.zeros(1000, device="cuda", dtype=torch.bfloat16)
        ch.all_reduce_bf16(xb, rb)
        assert torch.equal(rb, xb)
    torch.cuda.synchronize()
    assert comm.fault() == 0
    # a flag that nobody writes: the wait gives up after its limit and says so; the context lives on
    assert comm.selftest_wait(20) == _lib.DEVICE_FAULT
    assert b"gave up" in garnet_b200.lib().garnet_b200_last_error()
    ch.all_gather(x, out)
    torch.cuda.synchronize()
    assert torch.equal(out[0], x) and comm.fault() == 0
    # too large for the channel's slot, and a misaligned source: rejected before any launch
    big = torch.zeros(2048, device="cuda")
    L = garnet_b200.lib()
    assert L.garnet_b200_comm_all_gather(ch._h, big.data_ptr(), 8192, big.data_ptr(), None) == _lib.INVALID_VALUE
    assert L.garnet_b200_comm_all_gather(ch._h, x.data_ptr() + 4, 64, out.data_ptr(), None) == _lib.INVALID_VALUE


@pytest.mark.parametrize("tokens", [5, 64, 300])
def test_single_rank_exchange_equals_the_operator(tokens):
    case = synth.moe_layer(tokens, 96, 64, experts=8, topk=4, seed=tokens, bias_scale=0.1)
    moe = build_moe(case, io_dtype=torch.bfloat16)
    comm = Comm(ep_arena_bytes(moe, 1, 320) + (1 << 16))
    ep = ExpertParallel(moe, comm, 320)
    x = dev(case["x"]).bfloat16()
    expected = moe.run(x)
    for _ in range(2):                               # second step: stale regions from the first
        y = ep.run(x)
        torch.cuda.synchronize()
        assert comm.fault() == 0 and moe.fault() == 0
        assert ep.rows_received() == tokens * 4
        assert torch.equal(y, expected)


def _two_gpu_worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ok = True
    try:
        # ---- collectives
        comm = Comm(256 << 20)
        ch = Channel(comm, 1 << 20)
        g = torch.Generator(device="cuda").manual_seed(10 + rank)
        x = torch.randn(50000, device="cuda", generator=g)
        everyone = [torch.randn(50000, device="cuda", generator=torch.Generator(device="cuda").manual_seed(10 + r))
                    for r in range(world)]
        out = torch.zeros(world, 50000, device="cuda")
        red = torch.zeros(50000, device="cuda")
        for _ in range(4):
            ch.all_gather(x, out)
            ch.all_reduce(x, red)
            torch.cuda.synchronize()
            ok &= all(torch.equal(out[r], everyone[r]) for r in range(world))
            total = everyone[0].clone()
            for r in range(1, world):
                total = total + everyone[r]
            ok &= torch.equal(red, total)
            ch.all_reduce(x, red, wire=torch.bfloat16)
            torch.cuda.synchronize()
            tb = everyone[0].bfloat16().float()
            for r in range(1, world):
                tb = tb + everyone[r].bfloat16().float()
            ok &= torch.equal(red, tb.bfloat16().float())
            # bf16 in, bf16 out: for two ranks exactly bf16(a + b) (tp_peer_math.cuh:10-14)
            rb = torch.zeros(50000, device="cuda", dtype=torch.bfloat16)
            ch.all_reduce_bf16(x.bfloat16(), rb)
            torch.cuda.synchronize()
            ok &= torch.equal(rb, tb.bfloat16())
        ok &= comm.fault() == 0
        # ---- a K-sharded (row-parallel) int4 linear: partial sums added over the ranks by the
        # library's bf16 all-reduce equal the sum of the ranks' own partial results
        n, k, m = 512, 1024, 3
        lc = synth.int4_linear(n, k, m, seed=5)
        nib = dev(lc["nibbles"])
        sc = torch.from_numpy(lc["scales_bits"].view(np.int16)).view(torch.bfloat16).reshape(n, k // 128).cuda()
        xl = torch.from_numpy(lc["x_bits"].view(np.int16)).view(torch.bfloat16).reshape(m, k).cuda()
        kl = k // world
        parts = [garnet_b200.W4A16Linear().prepare(nib, sc, n, k, 128, r, world, shard_axis=1).forward(
            xl[:, r * kl:(r + 1) * kl].contiguous()) for r in range(world)]
        want = parts[0].float()
        for r in range(1, world):
            want = want + parts[r].float()
        got = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
        ch.all_reduce_bf16(parts[rank], got)
        torch.cuda.synchronize()
        ok &= torch.equal(got, want.bfloat16())
        # ---- expert-parallel exchange against the single-GPU operator
        E, K, H, I, T = 8, 4, 96, 64, 48
        case = synth.moe_layer(T * world, H, I, experts=E, topk=K, seed=77, zipf_s=1.1, bias_scale=0.1)
        full = build_moe(case, io_dtype=torch.bfloat16)
        per = E // world
        local = dict(case)
        for k in ("gu_blocks", "gu_scales", "gu_bias", "dn_blocks", "dn_scales", "dn_bias"):
            local[k] = case[k][rank * per:(rank + 1) * per]
        mine = build_moe(local, io_dtype=torch.bfloat16, ep_rank=rank, ep_world=world, expert_weights_sharded=True)
        ep = ExpertParallel(mine, comm, T)
        x_all = dev(case["x"]).bfloat16()
        expected = full.run(x_all)[rank * T:(rank + 1) * T]
        for _ in range(3):
            y = ep.run(x_all[rank * T:(rank + 1) * T])
            torch.cuda.synchronize()
            ok &= comm.fault() == 0 and mine.fault() == 0
            ok &= torch.equal(y, expected)
        rows = torch.tensor([ep.rows_received()], device="cuda")
        dist.all_reduce(rows)
        ok &= int(rows.item()) == T * world * K
        dist.barrier()
    except Exception as e:  # noqa: BLE001
        results[f"error{rank}"] = repr(e)
        ok = False
    results[rank] = bool(ok)
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_collectives_and_exchange():
    import torch.multiprocessing as mp
    world = 2
    port = 29700 + os.getpid() % 1000
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_two_gpu_worker, args=(world, port, results), nprocs=world, join=True)
        assert all(results.get(r) for r in range(world)), dict(results)
