"""Multi-GPU paths of the quantized operators: one process per GPU, torch.distributed
for the plumbing (NCCL over NVLink on the GPU box, gloo in the CPU tests).

* `ShardedLinear`: an int4 linear split along N (tensor parallel); every rank
  computes its N/G output columns and the logits are all-gathered - the
  reference's vocab-parallel lm_head (src/backends/tensorrt/trt_builder.cpp:7360-7371,
  plugins/gpt_oss/cuda/tp_collective.cpp:123-148: all-gather + row interleave).
* `ExpertParallelMoe`: experts in contiguous blocks of E/G per rank; each rank
  routes its own tokens, rows are dispatched to the owners of their experts with an
  all-to-all, the owners run the experts, the per-row values come back with a
  second all-to-all and the source rank applies the router weights in router
  order.  The reference only has a 2-way split with replicated tokens and an
  all-reduce (gpt_oss_kernels.cu:771,:818); parity target is the single-GPU result.

The exchange logic is independent of the compute: both classes take the local
compute as a callable, so that the index arithmetic is tested on CPU ranks."""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist


class ShardedLinear:
    """y[M, N] = x[M, K] W^T with W's rows split evenly over the ranks of `group`."""

    def __init__(self, local_forward: Callable[[torch.Tensor], torch.Tensor], n: int, group=None):
        self.local_forward = local_forward
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if n % self.world:
            raise ValueError("output rows must divide evenly over the ranks")
        self.n = n
        self.n_local = n // self.world

    def forward(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        y_local = self.local_forward(x)                       # [M, N/G]
        m = y_local.shape[0]
        gathered = torch.empty(self.world, m, self.n_local, dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(gathered.view(-1), y_local.contiguous().view(-1), group=self.group)
        # rank-major -> row-major: [G, M, N/G] -> [M, G, N/G] -> [M, N]
        y = gathered.permute(1, 0, 2).reshape(m, self.n)
        if out is not None:
            out.copy_(y)
            return out
        return y


def dispatch_plan(selected: torch.Tensor, experts: int, world: int):
    """Slots (token-major, router order) sorted by destination rank, stable.
    Returns (order [slots] int64: slot ids in send order, send_counts [world] int64,
    dest_expert [slots] int32 in send order)."""
    flat = selected.reshape(-1).to(torch.int64)
    per = experts // world
    dest = torch.div(flat, per, rounding_mode="floor")
    order = torch.sort(dest, stable=True).indices
    send_counts = torch.bincount(dest, minlength=world)
    return order, send_counts, flat[order].to(torch.int32)


class ExpertParallelMoe:
    """Expert-parallel MoE over `group`.

    route(x) -> (selected [T, k] int32, probs [T, k] fp32) on the local tokens;
    experts_on_rows(rows [R, H], row_expert [R] int32) -> values [R, H] fp32 for rows
    whose experts this rank owns; combine(vals [T*k, H] fp32, probs) -> y [T, H]."""

    def __init__(self, route, experts_on_rows, combine, experts: int, top_k: int, group=None,
                 wire_dtype: torch.dtype = torch.bfloat16):
        self.route, self.experts_on_rows, self.combine = route, experts_on_rows, combine
        self.experts, self.top_k, self.group = experts, top_k, group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if experts % self.world:
            raise ValueError("experts must divide evenly over the ranks")
        self.wire_dtype = wire_dtype
        self.last_recv_rows = 0

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        tokens, hidden = x.shape
        selected, probs = self.route(x)
        order, send_counts, send_expert = dispatch_plan(selected, self.experts, self.world)
        # 1. sizes (the only host synchronisation: split sizes must be known on the host)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        send_sizes = send_counts.tolist()
        recv_sizes = recv_counts.tolist()
        n_recv = int(sum(recv_sizes))
        self.last_recv_rows = n_recv
        # 2. dispatch rows and their expert ids
        token_of_slot = torch.div(order, self.top_k, rounding_mode="floor")
        send_rows = x[token_of_slot].to(self.wire_dtype).contiguous()
        recv_rows = torch.empty(n_recv, hidden, dtype=self.wire_dtype, device=x.device)
        dist.all_to_all_single(recv_rows, send_rows, recv_sizes, send_sizes, group=self.group)
        recv_expert = torch.empty(n_recv, dtype=torch.int32, device=x.device)
        dist.all_to_all_single(recv_expert, send_expert.contiguous(), recv_sizes, send_sizes, group=self.group)
        # 3. local experts (values are bf16-representable, so the bf16 wire is exact)
        if n_recv:
            vals = self.experts_on_rows(recv_rows.to(x.dtype), recv_expert)
        else:
            vals = torch.empty(0, hidden, dtype=torch.float32, device=x.device)
        # 4. return the per-row values to their sources
        back_send = vals.to(self.wire_dtype).contiguous()
        back_recv = torch.empty(order.numel(), hidden, dtype=self.wire_dtype, device=x.device)
        dist.all_to_all_single(back_recv, back_send, send_sizes, recv_sizes, group=self.group)
        # 5. undo the send order and combine in router order
        slot_vals = torch.empty(order.numel(), hidden, dtype=torch.float32, device=x.device)
        slot_vals[order] = back_recv.float()
        return self.combine(slot_vals, probs)
