"""The workspace-free MoE entry point (garnet_b200_moe_run_static).

Some hosts cannot hand the operator a workspace because they may not allocate
device memory where they call it - a decode loop that must never hit the CUDA
allocator (allocation and free serialise the whole device), or a process in
which another runtime already owns all of the GPU's memory.  For them the
library carries a 8 MiB scratch array of its own.  This file checks, through the
C ABI, that the entry point gives exactly what the ordinary entry point gives,
twice in a row (the array is shared and keeps its old contents between calls),
and that requests beyond the array's size are refused with a clear message.

The file name sorts last on purpose: if this test fails, a run that stops at the
first failure has already run everything else."""
import ctypes

import numpy as np
import pytest
import torch

import garnet_b200
from garnet_b200 import synth

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def build(case, **kw):
    moe = garnet_b200.GptOssMoe(case["hidden"], case["inter"], case["experts"], case["topk"], **kw)
    return moe.prepare(*[dev(case[k]) for k in ("router_w", "router_b", "gu_blocks", "gu_scales", "gu_bias",
                                                 "dn_blocks", "dn_scales", "dn_bias")])


def test_static_scratch_matches_workspace_entry_point_twice():
    # a layer with the gpt-oss-120b widths but few experts, so that it builds quickly
    case = synth.moe_layer(16, hidden=2880, inter=2880, experts=8, topk=4, seed=11, bias_scale=0.05)
    moe = build(case)
    x_first = dev(case["x"])
    x_second = dev(synth.moe_layer(5, hidden=2880, inter=2880, experts=8, topk=4, seed=12)["x"])
    for x in (x_first, x_second):                 # second call: fewer tokens, stale scratch from the first
        expected = moe.run(x)
        got = moe.run_static(x)
        torch.cuda.synchronize()
        assert moe.fault() == 0
        assert torch.isfinite(got).all()
        # same kernels, same order of operations: the tolerance of the MoE tests is
        # |a - e| <= 0.002 (1 + |e|); here the results are in fact identical
        assert (got - expected).abs().max().item() <= 0.002 * (1 + expected.abs().max().item())
        assert torch.equal(got, expected)


def test_static_scratch_allocates_nothing_and_survives_stale_block_scaled_scratch():
    """Two calls large enough for the block-scaled kernels (more than six rows per expert),
    the second with fewer tokens over the first one's leftovers; device memory in use does
    not change across the calls (neither through torch's allocator nor through the driver)."""
    case = synth.moe_layer(20, hidden=512, inter=512, experts=8, topk=4, seed=21, bias_scale=0.05)
    moe = build(case)
    x_first = dev(case["x"])
    x_second = dev(synth.moe_layer(16, hidden=512, inter=512, experts=8, topk=4, seed=22)["x"])
    expected = [moe.run(x) for x in (x_first, x_second)]
    outs = [torch.empty_like(x) for x in (x_first, x_second)]
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    held_before = torch.cuda.memory_allocated()
    for x, y in zip((x_first, x_second), outs):
        moe.run_static(x, out=y)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == held_before
    assert torch.cuda.mem_get_info()[0] == free_before
    assert moe.fault() == 0
    for y, e in zip(outs, expected):
        assert torch.equal(y, e)


def test_static_scratch_rejects_what_does_not_fit():
    case = synth.moe_layer(1, hidden=2880, inter=2880, experts=8, topk=4, seed=13)
    moe = build(case)
    L = garnet_b200.lib()
    x = torch.zeros(64, 2880, device="cuda")
    y = torch.empty_like(x)
    rc = L.garnet_b200_moe_run_static(moe._h, x.data_ptr(), y.data_ptr(), 64, None)
    assert rc == 1
    message = L.garnet_b200_last_error().decode()
    assert "built-in array" in message and "at most" in message
    assert L.garnet_b200_moe_run_static(None, x.data_ptr(), y.data_ptr(), 1, None) == 1
    assert L.garnet_b200_moe_run_static(moe._h, x.data_ptr(), y.data_ptr(), 0, None) == 1
