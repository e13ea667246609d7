"""Host-side mirror of the reference's int4 linear operator for the CUDA path.

`W4A16Linear` follows the life cycle of Garnet::Q4Q8Linear
(src/backends/cpu/q4q8_linear.h:21-35): `prepare` takes the canonical artifact
(QuantizedWeight: row-major nibbles and one 16-bit scale per (row, K-group),
src/model/weight_quantization.h:14-25), `forward` computes y = x W^T.  All
compute happens in libgarnet_b200.so through the C ABI; torch only provides
device memory and streams."""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import BF16, FP16, FP32, check, lib

_SCALE_KIND = {torch.float16: FP16, torch.bfloat16: BF16}
_SRC_KIND = {torch.float16: FP16, torch.bfloat16: BF16, torch.float32: FP32}


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def quantize_int4(weight: torch.Tensor, group: int = 128, scale_dtype: torch.dtype = torch.bfloat16):
    """Device twin of Garnet::QuantizeSymmetricINT4 (weight_quantization.cpp:188-270).
    Returns (nibbles uint8 [rows*cols/2], scales [rows, cols/group] of scale_dtype)."""
    if weight.dim() != 2 or not weight.is_cuda:
        raise ValueError("quantize_int4 needs a rank-two CUDA tensor")
    w = weight.contiguous()
    rows, cols = w.shape
    nibbles = torch.empty(rows * cols // 2, dtype=torch.uint8, device=w.device)
    scales = torch.empty(rows, cols // group, dtype=scale_dtype, device=w.device)
    check(lib().garnet_b200_int4_quantize(w.data_ptr(), _SRC_KIND[w.dtype], rows, cols, group,
                                          _SCALE_KIND[scale_dtype], nibbles.data_ptr(), scales.data_ptr(),
                                          _stream_ptr()))
    return nibbles, scales


def packed_bytes(n: int, k: int, group: int = 128) -> int:
    out = ctypes.c_size_t(0)
    check(lib().garnet_b200_w4a16_packed_bytes(n, k, group, ctypes.byref(out)))
    return out.value


def pack_host(nibbles, scales, n: int, k: int, group: int = 128) -> torch.Tensor:
    """Host repacker; `nibbles` uint8 CPU tensor, `scales` fp16/bf16 CPU tensor."""
    nb = nibbles.contiguous().cpu()
    sc = scales.contiguous().cpu()
    out = torch.empty(packed_bytes(n, k, group), dtype=torch.uint8)
    check(lib().garnet_b200_w4a16_pack_host(nb.data_ptr(), sc.data_ptr(), _SCALE_KIND[sc.dtype], n, k, group,
                                            out.data_ptr()))
    return out


def forward_group(linears, x: torch.Tensor, outs=None, pdl: bool = True):
    """One launch for up to 4 linears that share the input x (q/k/v, gate/up)."""
    x2 = x.reshape(-1, linears[0].k).contiguous()
    m = x2.shape[0]
    if outs is None:
        outs = [torch.empty(m, lin.n, dtype=torch.bfloat16, device=x.device) for lin in linears]
    hs = (ctypes.c_void_p * len(linears))(*[lin._h for lin in linears])
    ys = (ctypes.c_void_p * len(linears))(*[o.data_ptr() for o in outs])
    check(lib().garnet_b200_w4a16_run_group(hs, len(linears), x2.data_ptr(), ys, m, 1 if pdl else 0, _stream_ptr()))
    return outs


class LinearList:
    """A prepared list of linears run by one persistent launch (garnet_b200_w4a16_list_*).
    `calls` is a sequence of (linear, x, y[, dep]) with device tensors; dep is the index of
    an earlier call whose output x holds, or -1."""

    def __init__(self, calls, m: int = 1):
        self._keep = list(calls)
        n = len(self._keep)
        hs = (ctypes.c_void_p * n)(*[c[0]._h for c in self._keep])
        xs = (ctypes.c_void_p * n)(*[c[1].data_ptr() for c in self._keep])
        ys = (ctypes.c_void_p * n)(*[c[2].data_ptr() for c in self._keep])
        deps = (ctypes.c_int * n)(*[(c[3] if len(c) > 3 else -1) for c in self._keep])
        self._l = ctypes.c_void_p(None)
        check(lib().garnet_b200_w4a16_list_create(hs, xs, ys, deps, n, m, ctypes.byref(self._l)))

    def run(self, pdl: bool = False) -> None:
        check(lib().garnet_b200_w4a16_list_run(self._l, 1 if pdl else 0, _stream_ptr()))

    def fault(self) -> int:
        return lib().garnet_b200_w4a16_list_fault(self._l)

    def close(self) -> None:
        if self._l:
            lib().garnet_b200_w4a16_list_destroy(self._l)
            self._l = ctypes.c_void_p(None)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class ListItem(ctypes.Structure):
    """garnet_b200_w4a16_list_item."""
    _fields_ = [("linear", ctypes.c_void_p), ("d_x", ctypes.c_void_p), ("d_y", ctypes.c_void_p), ("dep", ctypes.c_int),
                ("activation", ctypes.c_int), ("d_norm_weight", ctypes.c_void_p), ("norm_eps", ctypes.c_float),
                ("residual_dep", ctypes.c_int), ("d_residual", ctypes.c_void_p)]


class GlueList(LinearList):
    """A list whose linears carry the glue of a decoder layer (garnet_b200_w4a16_list_create_ex).
    `calls` is a sequence of dicts: linear, x, y, and optionally dep, activation (1 = the input is
    silu(x[:, :K]) * x[:, K:]), norm_weight with norm_eps, residual (a tensor) or residual_dep."""

    def __init__(self, calls, m: int = 1):
        self._keep = list(calls)
        n = len(self._keep)
        items = (ListItem * n)()
        for it, c in zip(items, self._keep):
            it.linear = c["linear"]._h
            it.d_x, it.d_y = c["x"].data_ptr(), c["y"].data_ptr()
            it.dep = c.get("dep", -1)
            it.activation = c.get("activation", 0)
            nw = c.get("norm_weight")
            it.d_norm_weight = nw.data_ptr() if nw is not None else None
            it.norm_eps = c.get("norm_eps", 0.0)
            it.residual_dep = c.get("residual_dep", -1)
            res = c.get("residual")
            it.d_residual = res.data_ptr() if res is not None else None
        self._l = ctypes.c_void_p(None)
        check(lib().garnet_b200_w4a16_list_create_ex(items, n, m, ctypes.byref(self._l)))


class HostBatch:
    """A prepared list of (linear, host x, host y) calls (garnet_b200_w4a16_batch_*); after
    `run` the outputs are complete once the current stream has been synchronised."""

    def __init__(self, calls):
        self._keep = list(calls)
        n = len(self._keep)
        hs = (ctypes.c_void_p * n)(*[lin._h for lin, _, _ in self._keep])
        xs = (ctypes.c_void_p * n)(*[x.data_ptr() for _, x, _ in self._keep])
        ys = (ctypes.c_void_p * n)(*[y.data_ptr() for _, _, y in self._keep])
        ms = (ctypes.c_int * n)(*[x.numel() // lin.k for lin, x, _ in self._keep])
        self._b = ctypes.c_void_p(None)
        check(lib().garnet_b200_w4a16_batch_create(hs, xs, ys, ms, n, ctypes.byref(self._b)))

    def run(self) -> None:
        check(lib().garnet_b200_w4a16_batch_run(self._b, _stream_ptr()))

    def close(self) -> None:
        if self._b:
            lib().garnet_b200_w4a16_batch_destroy(self._b)
            self._b = ctypes.c_void_p(None)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class W4A16Linear:
    """y[M, N] = x[M, K] W^T, W int4 with one scale per (row, `group` columns)."""

    def __init__(self):
        self._h = ctypes.c_void_p(None)
        self.n = self.k = self.group = 0
        self._keep = None
        self._ws = None
        self._host_rows = 0

    def reserve_host(self, max_m: int) -> None:
        """Allocates the device staging of the host-buffer calls for up to max_m rows."""
        if max_m > self._host_rows:
            check(lib().garnet_b200_w4a16_reserve_host(self._h, max_m))
            self._host_rows = max_m

    # Q4Q8Linear::Prepare (q4q8_linear.cpp:227-283)
    def prepare(self, nibbles: torch.Tensor, scales: torch.Tensor, n: int, k: int, group: int = 128,
                shard_rank: int = 0, shard_world: int = 1, shard_axis: int = 0) -> "W4A16Linear":
        """shard_axis 0 splits the rows (N: tp_mode "vocab" / "qkv"), 1 the columns (K: tp_mode "row",
        whose partial sums are then added over the ranks)."""
        self.close()
        if not nibbles.is_cuda or not scales.is_cuda:
            raise ValueError("prepare needs device-resident canonical weights")
        nb, sc = nibbles.contiguous(), scales.contiguous()
        h = ctypes.c_void_p(None)
        create = lib().garnet_b200_w4a16_create if shard_axis == 0 else lib().garnet_b200_w4a16_create_k_shard
        check(create(nb.data_ptr(), sc.data_ptr(), _SCALE_KIND[sc.dtype], n, k, group, shard_rank, shard_world,
                     _stream_ptr(), ctypes.byref(h)))
        self._h, self.group = h, group
        self.n = n // shard_world if shard_axis == 0 else n
        self.k = k // shard_world if shard_axis == 1 else k
        return self

    # Q4Q8Linear::BindPackedView (q4q8_linear.cpp:285-313): borrows packed bytes
    def bind_packed(self, packed: torch.Tensor, scale_dtype: torch.dtype, n: int, k: int,
                    group: int = 128) -> "W4A16Linear":
        self.close()
        h = ctypes.c_void_p(None)
        check(lib().garnet_b200_w4a16_create_prepacked(packed.data_ptr(), _SCALE_KIND[scale_dtype], n, k, group,
                                                       ctypes.byref(h)))
        self._h, self.n, self.k, self.group, self._keep = h, n, k, group, packed
        return self

    def workspace_bytes(self, m: int) -> int:
        out = ctypes.c_size_t(0)
        check(lib().garnet_b200_w4a16_workspace(self._h, m, ctypes.byref(out)))
        return out.value

    def _workspace(self, m: int, device) -> torch.Tensor | None:
        need = self.workspace_bytes(m)
        if need == 0:
            return None
        if self._ws is None or self._ws.numel() < need or self._ws.device != device:
            self._ws = torch.empty(need, dtype=torch.uint8, device=device)
        return self._ws

    # Q4Q8Linear::Forward (q4q8_linear.cpp:315-389)
    def forward(self, x: torch.Tensor, out: torch.Tensor | None = None, workspace: torch.Tensor | None = None,
                pdl: bool = True) -> torch.Tensor:
        if x.dtype != torch.bfloat16 or not x.is_cuda:
            raise ValueError("forward needs a bf16 CUDA tensor")
        x2 = x.reshape(-1, self.k).contiguous()
        m = x2.shape[0]
        y = out if out is not None else torch.empty(m, self.n, dtype=torch.bfloat16, device=x.device)
        ws = workspace if workspace is not None else self._workspace(m, x.device)
        check(lib().garnet_b200_w4a16_run(self._h, x2.data_ptr(), y.data_ptr(), m,
                                          ws.data_ptr() if ws is not None else None,
                                          ws.numel() if ws is not None else 0, 1 if pdl else 0, _stream_ptr()))
        return y

    def forward_host(self, x_host: torch.Tensor, y_host: torch.Tensor) -> torch.Tensor:
        """Host buffers in, host buffers out (copies inside the call)."""
        m = x_host.numel() // self.k
        self.reserve_host(m)
        check(lib().garnet_b200_w4a16_run_host(self._h, x_host.data_ptr(), y_host.data_ptr(), m, _stream_ptr()))
        return y_host

    def forward_host_async(self, x_host: torch.Tensor, y_host: torch.Tensor) -> torch.Tensor:
        """`forward_host` without the final synchronisation: y_host is complete once the
        current stream has been synchronised."""
        m = x_host.numel() // self.k
        self.reserve_host(m)
        check(lib().garnet_b200_w4a16_run_host_async(self._h, x_host.data_ptr(), y_host.data_ptr(), m, _stream_ptr()))
        return y_host

    def dequantized(self) -> torch.Tensor:
        out = torch.empty(self.n, self.k, dtype=torch.float32, device="cuda")
        check(lib().garnet_b200_w4a16_dequant(self._h, out.data_ptr(), _stream_ptr()))
        return out

    def fault(self) -> int:
        return lib().garnet_b200_w4a16_fault(self._h)

    def close(self) -> None:
        if self._h:
            lib().garnet_b200_w4a16_destroy(self._h)
            self._h = ctypes.c_void_p(None)
        self._keep = None
        self._ws = None
        self._host_rows = 0

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
