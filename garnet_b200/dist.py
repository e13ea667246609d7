"""Multi-GPU paths of the quantized operators: one process per GPU.  The data path is the
library's own (include/garnet_b200.h, "collectives over NVLink" and "expert-parallel
MoE"): peer stores into arenas mapped through CUDA IPC, device-side flags with bounded
waits, no host synchronisation.  torch.distributed is only the host channel that carries
the 128-byte IPC blobs once at set-up.

* `Comm` / `Channel`: garnet_b200_comm_* (all-gather of the N-sharded lm_head's logits,
  all-reduce of expert-sharded partial sums; the reference's GptOssTpAllGather /
  GptOssTpAllReduce / GptOssTpAllReduceBf16, plugins/gpt_oss/cuda/tp_collective.cpp:77-148).
* `ExpertParallel`: garnet_b200_moe_ep_* (tokens split over the ranks, experts in
  contiguous blocks, rows pushed to the owner of their expert and values pushed back).

`HostExchange` restates the expert-parallel exchange on the host with the same placement
rule (garnet_b200_moe_ep_plan_host), fixed-capacity regions, counts, epoch flags and
bounded waits, over any torch.distributed backend: the protocol's arithmetic is tested
with it on CPU ranks (gloo), where no GPU is needed."""
from __future__ import annotations

import ctypes
import time

import numpy as np
import torch
import torch.distributed as dist

from ._lib import BF16, FP32, check, lib

BLOB_BYTES = 128


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


class Comm:
    """A rank's communicator: an arena of `arena_bytes` of device memory that the peers map."""

    def __init__(self, arena_bytes: int, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self._c = ctypes.c_void_p(None)
        check(lib().garnet_b200_comm_create(self.rank, self.world, arena_bytes, ctypes.byref(self._c)))
        blob = (ctypes.c_ubyte * BLOB_BYTES)()
        check(lib().garnet_b200_comm_export(self._c, blob, BLOB_BYTES))
        if self.world > 1:
            mine = torch.tensor(list(blob), dtype=torch.uint8, device="cuda")
            everyone = torch.empty(self.world * BLOB_BYTES, dtype=torch.uint8, device="cuda")
            dist.all_gather_into_tensor(everyone, mine, group=group)
            blobs = (ctypes.c_ubyte * (self.world * BLOB_BYTES))(*everyone.cpu().tolist())
            check(lib().garnet_b200_comm_connect(self._c, blobs))
            dist.barrier(group=group)      # every rank has opened every arena before anyone stores into one
        else:
            check(lib().garnet_b200_comm_connect(self._c, None))

    def fault(self) -> int:
        return lib().garnet_b200_comm_fault(self._c)

    def selftest_wait(self, limit_ms: int = 20) -> int:
        return lib().garnet_b200_comm_selftest_wait(self._c, limit_ms, _stream_ptr())

    def close(self) -> None:
        if self._c:
            lib().garnet_b200_comm_destroy(self._c)
            self._c = ctypes.c_void_p(None)


class Channel:
    """Collectives of up to `slot_bytes` per rank on a communicator."""

    def __init__(self, comm: Comm, slot_bytes: int):
        self.comm = comm
        self._h = ctypes.c_void_p(None)
        check(lib().garnet_b200_comm_channel_create(comm._c, slot_bytes, ctypes.byref(self._h)))

    def all_gather(self, src: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
        """dst[r] = src of rank r (dst: [world, *src.shape], contiguous)."""
        nbytes = src.numel() * src.element_size()
        check(lib().garnet_b200_comm_all_gather(self._h, src.data_ptr(), nbytes, dst.data_ptr(), _stream_ptr()))
        return dst

    def all_reduce(self, src: torch.Tensor, dst: torch.Tensor, wire: torch.dtype = torch.float32) -> torch.Tensor:
        """dst = sum over ranks of src (fp32 tensors); `wire` bf16 sends bf16 and rounds the sum to bf16."""
        check(lib().garnet_b200_comm_all_reduce(self._h, src.data_ptr(), dst.data_ptr(), src.numel(),
                                                BF16 if wire == torch.bfloat16 else FP32, _stream_ptr()))
        return dst


    def all_reduce_bf16(self, src: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
        """dst = bf16(sum over ranks of src), bf16 tensors; for two ranks exactly bf16(a + b)."""
        check(lib().garnet_b200_comm_all_reduce_bf16(self._h, src.data_ptr(), dst.data_ptr(), src.numel(), _stream_ptr()))
        return dst


def ep_arena_bytes(moe, world: int, tokens_local_max: int) -> int:
    out = ctypes.c_size_t(0)
    check(lib().garnet_b200_moe_ep_arena_bytes(ctypes.byref(moe.opt), world, tokens_local_max, ctypes.byref(out)))
    return out.value


class ExpertParallel:
    """Expert-parallel MoE with the exchange on the device (garnet_b200_moe_ep_*).  `moe` holds
    this rank's block of experts (ep_rank / ep_world of the communicator, bf16 io)."""

    def __init__(self, moe, comm: Comm, tokens_local_max: int):
        self.moe, self.comm = moe, comm
        self._e = ctypes.c_void_p(None)
        check(lib().garnet_b200_moe_ep_create(moe._h, comm._c, tokens_local_max, ctypes.byref(self._e)))

    def run(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        x2 = x.reshape(-1, self.moe.opt.hidden).contiguous()
        y = out if out is not None else torch.empty_like(x2)
        check(lib().garnet_b200_moe_ep_run(self._e, x2.data_ptr(), y.data_ptr(), x2.shape[0], _stream_ptr()))
        return y

    def rows_received(self) -> int:
        return lib().garnet_b200_moe_ep_rows_received(self._e)

    def close(self) -> None:
        if self._e:
            lib().garnet_b200_moe_ep_destroy(self._e)
            self._e = ctypes.c_void_p(None)


def plan_host(selected: np.ndarray, experts_per_rank: int, world: int):
    """The exchange's placement rule (garnet_b200_moe_ep_plan_host): position of every routed
    row among the rows this rank sends to its owner, and the rows per owner."""
    sel = np.ascontiguousarray(selected, np.int32).reshape(-1)
    send_idx = np.empty(sel.size, np.int32)
    dest_count = np.empty(world, np.int32)
    ip = ctypes.POINTER(ctypes.c_int)
    check(lib().garnet_b200_moe_ep_plan_host(sel.ctypes.data_as(ip), sel.size, experts_per_rank, world,
                                             send_idx.ctypes.data_as(ip), dest_count.ctypes.data_as(ip)))
    return send_idx, dest_count


class HostExchange:
    """The expert-parallel exchange restated on the host, region for region and flag for
    flag (see moe_ep.cu): receive regions of fixed capacity per source, a count and an
    epoch flag per source, unused rows marked -1, values returned into per-owner regions,
    combine in router order.  "Peer stores" are all-to-alls of the padded regions; a
    flag that never arrives ends the wait after `limit_s` with the device's fault codes
    (71: a source never posted its rows, 72: an owner never returned its values)."""

    def __init__(self, experts: int, top_k: int, hidden: int, tokens_local_max: int, group=None, limit_s: float = 2.0):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.per = experts // self.world
        self.top_k, self.hidden = top_k, hidden
        self.cap = tokens_local_max * top_k
        self.epoch = 0
        self.limit_s = limit_s
        self.fault = 0
        self.rows_received = 0

    def _exchange(self, regions: torch.Tensor) -> torch.Tensor:
        """regions[d] goes to rank d; returns what every rank sent to this one, by source."""
        out = torch.empty_like(regions)
        dist.all_to_all_single(out, regions.contiguous(), group=self.group)
        return out

    def _wait(self, flags: torch.Tensor, code: int) -> bool:
        """Bounded wait for every source's flag to show this epoch."""
        t0 = time.monotonic()
        while True:
            if bool((flags == self.epoch).all()):
                return True
            if time.monotonic() - t0 > self.limit_s:
                self.fault = code
                return False
            time.sleep(0.002)

    def step(self, x: torch.Tensor, selected: torch.Tensor, probs: torch.Tensor, experts_on_rows, post_flags: bool = True):
        self.epoch += 1
        W, cap, H, k = self.world, self.cap, self.hidden, self.top_k
        sel = selected.reshape(-1).to(torch.int32)
        send_idx, dest_count = plan_host(sel.numpy(), self.per, W)
        send_idx_t = torch.from_numpy(send_idx).long()
        dest = (sel // self.per).long()
        # "push": rows, expert ids, count and flag into the region this rank owns at each destination
        rows = torch.zeros(W, cap, H, dtype=torch.bfloat16)
        ids = torch.full((W, cap), -1, dtype=torch.int32)
        token = torch.arange(sel.numel()) // k
        rows[dest, send_idx_t] = x[token].to(torch.bfloat16)
        ids[dest, send_idx_t] = sel
        meta = torch.zeros(W, 2, dtype=torch.int32)
        meta[:, 0] = torch.from_numpy(dest_count)
        meta[:, 1] = self.epoch if post_flags else 0
        got_rows, got_ids, got_meta = self._exchange(rows), self._exchange(ids), self._exchange(meta)
        # owner: wait for every source, mark what nobody sent, run the experts
        vals = torch.zeros(W, cap, H, dtype=torch.bfloat16)
        if self._wait(got_meta[:, 1], 71):
            counts = got_meta[:, 0].clamp(0, cap)
            unused = torch.arange(cap)[None, :] >= counts[:, None]
            got_ids[unused] = -1
            self.rows_received = int(counts.sum())
            flat_ids = got_ids.reshape(-1)
            valid = flat_ids >= 0
            if bool(valid.any()):
                out = experts_on_rows(got_rows.reshape(-1, H)[valid].float(), flat_ids[valid])
                v = vals.reshape(-1, H)
                v[valid] = out.to(torch.bfloat16)
        ret_flag = torch.full((W, 1), self.epoch if self.fault == 0 else 0, dtype=torch.int32)
        back, back_flag = self._exchange(vals), self._exchange(ret_flag)
        if not self._wait(back_flag[:, 0], 72):
            return None
        # source: combine in router order from the per-owner regions
        slot_vals = back[dest, send_idx_t].float().reshape(-1, k, H)
        acc = torch.zeros(slot_vals.shape[0], H)
        for j in range(k):
            acc = acc + slot_vals[:, j] * probs[:, j:j + 1]
        return acc.to(torch.bfloat16)
