"""Host-side mirror of the reference's gpt-oss MoE operator for the CUDA path.

`GptOssMoe` follows Garnet::GptOssMarlin (plugins/gpt_oss/include/gpt_oss_marlin.h:17-30):
construct with the options, query `workspace_bytes(tokens)`, `run(x)`.  Operands
keep the order and original checkpoint layout of the reference operator
`gpt_oss_moe_mxfp4` (src/backends/tensorrt/gpt_oss_lowering.cpp:309-312).  All
compute happens in libgarnet_b200.so through the C ABI."""
from __future__ import annotations

import ctypes

import torch

from ._lib import BF16, FP32, check, lib


class MoeOptions(ctypes.Structure):
    _fields_ = [("abi", ctypes.c_int), ("struct_size", ctypes.c_int), ("hidden", ctypes.c_int),
                ("intermediate", ctypes.c_int), ("experts", ctypes.c_int), ("top_k", ctypes.c_int),
                ("prefill", ctypes.c_int), ("ep_rank", ctypes.c_int), ("ep_world", ctypes.c_int),
                ("ep_interleaved", ctypes.c_int), ("expert_weights_sharded", ctypes.c_int),
                ("io_dtype", ctypes.c_int), ("limit", ctypes.c_float), ("layouts", ctypes.c_int),
                ("tp_rank", ctypes.c_int), ("tp_world", ctypes.c_int), ("tp_weights_sharded", ctypes.c_int)]


LAYOUT_BOTH, LAYOUT_STREAM, LAYOUT_BLOCK = 0, 1, 2


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


class GptOssMoe:
    def __init__(self, hidden: int, intermediate: int, experts: int, top_k: int, limit: float = 7.0,
                 io_dtype: torch.dtype = torch.float32, ep_rank: int = 0, ep_world: int = 1,
                 ep_interleaved: bool = False, expert_weights_sharded: bool = False, prefill: int = 0,
                 layouts: int = LAYOUT_BOTH, tp_rank: int = 0, tp_world: int = 0, tp_weights_sharded: bool = False):
        """`intermediate` is the layer's full width; with tp_world > 1 this handle computes
        intermediate / tp_world channels of it (see garnet_b200_moe_options)."""
        self.opt = MoeOptions(abi=1, struct_size=ctypes.sizeof(MoeOptions), hidden=hidden,
                              intermediate=intermediate, experts=experts, top_k=top_k, prefill=prefill,
                              ep_rank=ep_rank, ep_world=ep_world, ep_interleaved=int(ep_interleaved),
                              expert_weights_sharded=int(expert_weights_sharded),
                              io_dtype=FP32 if io_dtype == torch.float32 else BF16, limit=limit, layouts=layouts,
                              tp_rank=tp_rank, tp_world=tp_world, tp_weights_sharded=int(tp_weights_sharded))
        self.io_dtype = io_dtype
        self.inter_local = intermediate // tp_world if tp_world > 1 else intermediate
        self._h = ctypes.c_void_p(None)
        self._keep = None
        self._ws = None

    # GptOssMarlin::Workspace (gpt_oss_marlin.h:25)
    def workspace_bytes(self, tokens: int) -> int:
        out = ctypes.c_size_t(0)
        check(lib().garnet_b200_moe_workspace(ctypes.byref(self.opt), tokens, ctypes.byref(out)))
        return out.value

    def prepare(self, router_w, router_b, gu_blocks, gu_scales, gu_bias, dn_blocks, dn_scales, dn_bias) -> "GptOssMoe":
        self.close()
        tensors = [router_w.float(), router_b.float(), gu_blocks, gu_scales, gu_bias.float(), dn_blocks, dn_scales,
                   dn_bias.float()]
        tensors = [t.contiguous() for t in tensors]
        if not all(t.is_cuda for t in tensors):
            raise ValueError("prepare needs device-resident operands")
        arr = (ctypes.c_void_p * 8)(*[t.data_ptr() for t in tensors])
        h = ctypes.c_void_p(None)
        check(lib().garnet_b200_moe_create(ctypes.byref(self.opt), arr, _stream_ptr(), ctypes.byref(h)))
        self._h = h
        self._keep = tensors            # router weights and biases are borrowed by the handle
        return self

    def prepare_prepacked(self, router_w, router_b, gu_bias, dn_bias, packed) -> "GptOssMoe":
        """The operator over packed blobs the caller keeps (garnet_b200_moe_create_prepacked):
        `packed` = [gate_up stream, down stream, gate_up block, down block] device uint8 tensors,
        None where options.layouts leaves a layout out."""
        self.close()
        small = [t.float().contiguous() for t in (router_w, router_b, gu_bias, dn_bias)]
        arr = (ctypes.c_void_p * 4)(*[t.data_ptr() for t in small])
        blobs = (ctypes.c_void_p * 4)(*[(t.data_ptr() if t is not None else None) for t in packed])
        h = ctypes.c_void_p(None)
        check(lib().garnet_b200_moe_create_prepacked(ctypes.byref(self.opt), arr, blobs, _stream_ptr(), ctypes.byref(h)))
        self._h = h
        self._keep = small + [t for t in packed if t is not None]
        return self

    def packed_view(self, which: int, layout: int) -> torch.Tensor:
        """A copy of the handle's packed blob of a projection in a layout (device uint8)."""
        ptr, n = ctypes.c_void_p(None), ctypes.c_size_t(0)
        check(lib().garnet_b200_moe_packed_view(self._h, which, layout, ctypes.byref(ptr), ctypes.byref(n)))
        class _View:   # the blob through the CUDA array interface: no copy until clone()
            __cuda_array_interface__ = {"shape": (n.value,), "typestr": "|u1", "data": (ptr.value, False), "version": 2}
        return torch.as_tensor(_View(), device="cuda").clone()

    def packed_bytes(self, which: int, layout: int, experts: int) -> int:
        out = ctypes.c_size_t(0)
        check(lib().garnet_b200_moe_packed_bytes(ctypes.byref(self.opt), which, layout, experts, ctypes.byref(out)))
        return out.value

    def pack_host(self, which: int, layout: int, blocks, scales):
        """Host packer (garnet_b200_moe_pack_host): numpy uint8 blocks [E, rows, K/32, 16] and scales
        [E, rows, K/32] of one projection -> the packed blob as a numpy uint8 array."""
        import numpy as np
        b = np.ascontiguousarray(blocks, np.uint8)
        sc = np.ascontiguousarray(scales, np.uint8)
        experts = b.shape[0]
        out = np.empty(self.packed_bytes(which, layout, experts), np.uint8)
        check(lib().garnet_b200_moe_pack_host(ctypes.byref(self.opt), which, layout, b.ctypes.data, sc.ctypes.data, experts,
                                              out.ctypes.data))
        return out

    def _workspace(self, tokens: int, device) -> torch.Tensor:
        need = self.workspace_bytes(tokens)
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(need, dtype=torch.uint8, device=device)
        return self._ws

    # GptOssMarlin::Run (gpt_oss_marlin.h:28-29)
    def run(self, x: torch.Tensor, out: torch.Tensor | None = None, workspace: torch.Tensor | None = None) -> torch.Tensor:
        if x.dtype != self.io_dtype or not x.is_cuda:
            raise ValueError("run needs a CUDA tensor of the operator's io dtype")
        x2 = x.reshape(-1, self.opt.hidden).contiguous()
        tokens = x2.shape[0]
        y = out if out is not None else torch.empty_like(x2)
        ws = workspace if workspace is not None else self._workspace(tokens, x.device)
        check(lib().garnet_b200_moe_run(self._h, x2.data_ptr(), y.data_ptr(), ws.data_ptr(), ws.numel(), tokens,
                                        _stream_ptr()))
        return y

    def run_static(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """`run` without a workspace: the scratch is the 8 MiB array built into the
        library, for callers that must not allocate device memory (see
        garnet_b200_moe_run_static in include/garnet_b200.h for the limits: small
        token counts only, one call at a time per device)."""
        if x.dtype != self.io_dtype or not x.is_cuda:
            raise ValueError("run_static needs a CUDA tensor of the operator's io dtype")
        x2 = x.reshape(-1, self.opt.hidden).contiguous()
        y = out if out is not None else torch.empty_like(x2)
        check(lib().garnet_b200_moe_run_static(self._h, x2.data_ptr(), y.data_ptr(), x2.shape[0], _stream_ptr()))
        return y

    # RunGptOssMoeRoute (gpt_oss_kernels.h:54-56)
    def route(self, x: torch.Tensor):
        x2 = x.reshape(-1, self.opt.hidden).contiguous()
        tokens = x2.shape[0]
        logits = torch.empty(tokens, self.opt.experts, dtype=torch.float32, device=x.device)
        selected = torch.empty(tokens, self.opt.top_k, dtype=torch.int32, device=x.device)
        probs = torch.empty(tokens, self.opt.top_k, dtype=torch.float32, device=x.device)
        need = ctypes.c_size_t(0)
        check(lib().garnet_b200_moe_route_workspace(ctypes.byref(self.opt), tokens, ctypes.byref(need)))
        ws = torch.empty(need.value, dtype=torch.uint8, device=x.device)
        # the router as `run` evaluates it for this token count
        check(lib().garnet_b200_moe_route_ws(self._h, x2.data_ptr(), selected.data_ptr(), probs.data_ptr(),
                                             logits.data_ptr(), tokens, ws.data_ptr(), ws.numel(), _stream_ptr()))
        return logits, selected, probs

    def route_fp32(self, x: torch.Tensor):
        """Router on the fp32 pipe at every size (garnet_b200_moe_route)."""
        x2 = x.reshape(-1, self.opt.hidden).contiguous()
        tokens = x2.shape[0]
        logits = torch.empty(tokens, self.opt.experts, dtype=torch.float32, device=x.device)
        selected = torch.empty(tokens, self.opt.top_k, dtype=torch.int32, device=x.device)
        probs = torch.empty(tokens, self.opt.top_k, dtype=torch.float32, device=x.device)
        check(lib().garnet_b200_moe_route(self._h, x2.data_ptr(), selected.data_ptr(), probs.data_ptr(),
                                          logits.data_ptr(), tokens, _stream_ptr()))
        return logits, selected, probs

    def rows_workspace_bytes(self, rows: int) -> int:
        out = ctypes.c_size_t(0)
        check(lib().garnet_b200_moe_rows_workspace(ctypes.byref(self.opt), rows, ctypes.byref(out)))
        return out.value

    def run_rows(self, rows_x: torch.Tensor, row_expert: torch.Tensor, out: torch.Tensor | None = None,
                 workspace: torch.Tensor | None = None) -> torch.Tensor:
        """Experts only, on already routed rows: returns unweighted per-row values
        [rows, hidden] fp32 (bf16-valued)."""
        x2 = rows_x.reshape(-1, self.opt.hidden).contiguous()
        rows = x2.shape[0]
        vals = out if out is not None else torch.empty(rows, self.opt.hidden, dtype=torch.float32, device=x2.device)
        need = self.rows_workspace_bytes(rows)
        ws = workspace if workspace is not None else torch.empty(need, dtype=torch.uint8, device=x2.device)
        ex = row_expert.to(torch.int32).contiguous()
        check(lib().garnet_b200_moe_run_rows(self._h, x2.data_ptr(), ex.data_ptr(), rows, vals.data_ptr(),
                                             ws.data_ptr(), ws.numel(), _stream_ptr()))
        return vals

    def run_rows_hidden(self, rows_x: torch.Tensor, row_expert: torch.Tensor) -> torch.Tensor:
        """First half of run_rows: SwiGLU activations [rows, intermediate] fp32 (bf16-valued)."""
        x2 = rows_x.reshape(-1, self.opt.hidden).contiguous()
        rows = x2.shape[0]
        hid = torch.zeros(rows, self.inter_local, dtype=torch.float32, device=x2.device)
        ws = torch.empty(self.rows_workspace_bytes(rows), dtype=torch.uint8, device=x2.device)
        ex = row_expert.to(torch.int32).contiguous()
        check(lib().garnet_b200_moe_run_rows_stage(self._h, 1, x2.data_ptr(), ex.data_ptr(), rows, hid.data_ptr(), None,
                                                   ws.data_ptr(), ws.numel(), _stream_ptr()))
        return hid

    def run_rows_down(self, hidden: torch.Tensor, row_expert: torch.Tensor) -> torch.Tensor:
        """Second half of run_rows: per-row values [rows, hidden] from given activations."""
        h2 = hidden.reshape(-1, self.inter_local).float().contiguous()
        rows = h2.shape[0]
        vals = torch.zeros(rows, self.opt.hidden, dtype=torch.float32, device=h2.device)
        ws = torch.empty(self.rows_workspace_bytes(rows), dtype=torch.uint8, device=h2.device)
        ex = row_expert.to(torch.int32).contiguous()
        check(lib().garnet_b200_moe_run_rows_stage(self._h, 2, None, ex.data_ptr(), rows, h2.data_ptr(), vals.data_ptr(),
                                                   ws.data_ptr(), ws.numel(), _stream_ptr()))
        return vals

    def combine(self, vals: torch.Tensor, probs: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """y[t] = bf(sum_j vals[t*k+j] * probs[t, j]) in router order."""
        tokens = probs.shape[0]
        y = out if out is not None else torch.empty(tokens, self.opt.hidden, dtype=self.io_dtype, device=vals.device)
        v, p = vals.contiguous(), probs.contiguous()
        check(lib().garnet_b200_moe_combine(self._h, v.data_ptr(), p.data_ptr(), y.data_ptr(), tokens, _stream_ptr()))
        return y

    def dequantized(self, which: int, stored_expert: int) -> torch.Tensor:
        rows, cols = (2 * self.inter_local, self.opt.hidden) if which in (0, 2) else (self.opt.hidden, self.inter_local)
        out = torch.empty(rows, cols, dtype=torch.float32, device="cuda")
        check(lib().garnet_b200_moe_dequant(self._h, which, stored_expert, out.data_ptr(), _stream_ptr()))
        return out

    def fault(self) -> int:
        return lib().garnet_b200_moe_fault(self._h)

    def close(self) -> None:
        if self._h:
            lib().garnet_b200_moe_destroy(self._h)
            self._h = ctypes.c_void_p(None)
        self._keep = None
        self._ws = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def mxfp4_decode(blocks: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """rows x 32 MXFP4 values -> fp32 (TestGptOssMxfp4Decode)."""
    rows = scales.numel()
    out = torch.empty(rows, 32, dtype=torch.float32, device=blocks.device)
    check(lib().garnet_b200_mxfp4_decode(blocks.data_ptr(), scales.data_ptr(), out.data_ptr(), rows, _stream_ptr()))
    return out


def gather_intermediate_shard(source, rank: int, world: int, mode: int):
    """Rank-local part of a checkpoint tensor for the intermediate-axis split (numpy in, numpy out):
    garnet_b200_moe_gather_intermediate_shard, the reference's GatherGptOssIntermediateShard
    (src/backends/tensorrt/gpt_oss_weight_shard.h:25-60)."""
    import numpy as np
    a = np.ascontiguousarray(source)
    shape = (ctypes.c_longlong * a.ndim)(*a.shape)
    if mode == 3:
        out = np.empty_like(a)
    else:
        axis = 1 if mode == 1 else 2
        if a.ndim <= axis or a.shape[axis] % world:
            raise ValueError("axis does not divide")
        out_shape = list(a.shape)
        out_shape[axis] //= world
        out = np.empty(out_shape, a.dtype)
    check(lib().garnet_b200_moe_gather_intermediate_shard(a.ctypes.data, a.nbytes, shape, a.ndim, a.itemsize, rank, world, mode,
                                                          out.ctypes.data))
    return out
