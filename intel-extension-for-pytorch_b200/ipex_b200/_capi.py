"""ctypes binding of libwoq_b200.so (include/woq_b200.h) for torch CUDA tensors.

This is the thin host layer the tests, the benchmark and the Python modules share.  There is
no fallback: if the shared library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libwoq_b200.so")

# constants of include/woq_b200.h
DTYPE_INT8, DTYPE_INT4, DTYPE_NF4, DTYPE_FP8 = 1, 2, 3, 4
LOWP_NONE, LOWP_FP16, LOWP_BF16, LOWP_INT8 = 0, 1, 2, 3
ACT_NONE, ACT_PER_TENSOR, ACT_PER_M, ACT_PER_TENSOR_SYM, ACT_PER_M_SYM = -1, 0, 2, 4, 6
ACT_PER_K_BLOCK, ACT_PER_M_K_BLOCK, ACT_PER_K_BLOCK_SYM, ACT_PER_M_K_BLOCK_SYM = 1, 3, 5, 7
ROUTE_INT4_BF16, ROUTE_INT8, ROUTE_GENERAL, ROUTE_INT8_BLOCK = 0, 1, 2, 3
FMT_PLAIN, FMT_GPTQ, FMT_AWQ = 0, 1, 2
FUSE_NONE, FUSE_GELU_ERF, FUSE_GELU_TANH, FUSE_RELU, FUSE_SILU = 0, 1, 2, 3, 4
FUSE_ADD, FUSE_ADD_ADD, FUSE_MUL, FUSE_SILU_MUL = 0x10, 0x20, 0x30, 0x100
T_NONE, T_F32, T_F16, T_BF16, T_U8, T_S8, T_I32 = 0, 1, 2, 3, 4, 5, 6
LAYOUT_GATE_UP, LAYOUT_STREAM_ONLY, LAYOUT_TC_ONLY, LAYOUT_SCALES_NK, LAYOUT_DEFER_CHECK = 1, 2, 4, 8, 16
LAYOUT_GENERIC = 32
HINT_AUTO, HINT_TENSOR_CORE, HINT_STREAM, HINT_STREAM_FAST = 0, 1, 2, 3
OPT_DECODE_SPLIT = 1
SPLIT_AUTO, SPLIT_STREAM_K, SPLIT_CLUSTER = 0, 1, 2

EXPORTS = [
    "woq_b200_version",
    "woq_b200_last_error",
    "woq_b200_kernel_launches",
    "woq_b200_set_option",
    "woq_b200_ctx_create",
    "woq_b200_ctx_destroy",
    "woq_b200_ctx_desc",
    "woq_b200_ctx_device_bytes",
    "woq_b200_ctx_unpack",
    "woq_b200_workspace_bytes",
    "woq_b200_workspace_header_bytes",
    "woq_b200_linear",
    "woq_b200_linear_any",
    "woq_b200_dump_dequant_f32",
    "woq_b200_linear_scatter",
    "woq_b200_linear_static_scratch",
    "woq_b200_static_scratch_status",
    "woq_b200_moe_workspace_bytes",
    "woq_b200_moe_expert",
    "woq_b200_dump_dequant",
    "woq_b200_int8_internals",
    "woq_b200_rmsnorm_quant",
    "woq_b200_linear_prequant",
    "woq_b200_int8_block_internals",
    "woq_b200_int8_block_size",
    "woq_b200_ctx_route",
    "woq_b200_int8_zero_points",
    "woq_b200_workspace_status",
    "woq_b200_decode_plan",
    "woq_b200_tc_plan",
    "woq_b200_comm_create",
    "woq_b200_comm_export",
    "woq_b200_comm_connect",
    "woq_b200_comm_gather_ptr",
    "woq_b200_comm_destroy",
    "woq_b200_comm_fence",
    "woq_b200_comm_status",
    "woq_b200_linear_allreduce",
    "woq_b200_linear_allgather",
]


class Desc(ctypes.Structure):
    _fields_ = [
        ("n", ctypes.c_int64),
        ("k", ctypes.c_int64),
        ("weight_dtype", ctypes.c_int32),
        ("group_size", ctypes.c_int32),
        ("lowp_mode", ctypes.c_int32),
        ("act_quant_mode", ctypes.c_int32),
        ("weight_format", ctypes.c_int32),
        ("scale_dtype", ctypes.c_int32),
        ("zp_dtype", ctypes.c_int32),
        ("bias_dtype", ctypes.c_int32),
        ("layout_flags", ctypes.c_int32),
        ("kernel_hint", ctypes.c_int32),
    ]


class WoqError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"libwoq_b200 status {code}: {msg}")
        self.code = code


_lib = None


def lib() -> ctypes.CDLL:
    """Load the shared library once.  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with "
            "`python intel-extension-for-pytorch_b200/build_native.py` (no CPU fallback exists)"
        )
    L = ctypes.CDLL(LIB_PATH)
    vp, i32, i64, sz = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_size_t
    L.woq_b200_version.restype = ctypes.c_int
    L.woq_b200_last_error.restype = ctypes.c_char_p
    L.woq_b200_kernel_launches.restype = i64
    L.woq_b200_set_option.argtypes = [i32, i32]
    L.woq_b200_ctx_create.argtypes = [ctypes.POINTER(Desc), vp, vp, vp, vp, vp, ctypes.POINTER(vp)]
    L.woq_b200_ctx_destroy.argtypes = [vp]
    L.woq_b200_ctx_desc.argtypes = [vp, ctypes.POINTER(Desc)]
    L.woq_b200_ctx_device_bytes.argtypes = [vp]
    L.woq_b200_ctx_device_bytes.restype = sz
    L.woq_b200_ctx_unpack.argtypes = [vp, vp, vp]
    L.woq_b200_workspace_bytes.argtypes = [vp, i64]
    L.woq_b200_workspace_bytes.restype = sz
    L.woq_b200_workspace_header_bytes.restype = sz
    L.woq_b200_linear.argtypes = [vp, vp, i64, i64, i32, ctypes.POINTER(vp), i32, vp, i64, vp, sz, vp]
    L.woq_b200_linear_any.argtypes = [vp, vp, i32, i64, i64, i32, ctypes.POINTER(vp), i32, vp, i64, vp, sz, vp]
    L.woq_b200_dump_dequant_f32.argtypes = [vp, i32, vp, vp]
    L.woq_b200_linear_static_scratch.argtypes = [vp, vp, i64, i64, i32, ctypes.POINTER(vp), i32, vp, i64, vp]
    L.woq_b200_static_scratch_status.argtypes = [vp]
    L.woq_b200_linear_scatter.argtypes = [vp, vp, i64, i64, vp, vp, vp, i64, vp, sz, vp]
    L.woq_b200_moe_workspace_bytes.argtypes = [vp, vp, i64]
    L.woq_b200_moe_workspace_bytes.restype = sz
    L.woq_b200_moe_expert.argtypes = [vp, vp, vp, i64, vp, vp, i64, vp, i64, vp, sz, vp]
    L.woq_b200_dump_dequant.argtypes = [vp, vp, vp]
    L.woq_b200_int8_internals.argtypes = [vp, vp, i64, i64, vp, vp, vp, vp, sz, vp]
    L.woq_b200_rmsnorm_quant.argtypes = [vp, i64, vp, ctypes.c_float, i64, i64, i32, vp, i64, vp, vp, vp, vp]
    L.woq_b200_linear_prequant.argtypes = [vp, vp, vp, vp, i64, i32, ctypes.POINTER(vp), i32, vp, i64, vp, sz, vp]
    L.woq_b200_int8_block_internals.argtypes = [vp, vp, i64, i64, vp, vp, vp, vp, vp, sz, vp]
    L.woq_b200_int8_block_size.argtypes = [vp]
    L.woq_b200_ctx_route.argtypes = [vp]
    L.woq_b200_int8_zero_points.argtypes = [vp, i64, vp, vp, sz, vp]
    L.woq_b200_workspace_status.argtypes = [vp, vp]
    L.woq_b200_decode_plan.argtypes = [vp, i64, ctypes.POINTER(i32)]
    L.woq_b200_tc_plan.argtypes = [i32, ctypes.POINTER(i32)]
    L.woq_b200_comm_create.argtypes = [i32, i32, i64, sz, ctypes.POINTER(vp)]
    L.woq_b200_comm_export.argtypes = [vp, vp]
    L.woq_b200_comm_connect.argtypes = [vp, vp]
    L.woq_b200_comm_gather_ptr.argtypes = [vp]
    L.woq_b200_comm_gather_ptr.restype = vp
    L.woq_b200_comm_destroy.argtypes = [vp]
    L.woq_b200_comm_fence.argtypes = [vp, vp]
    L.woq_b200_comm_status.argtypes = [vp, vp]
    L.woq_b200_linear_allreduce.argtypes = [vp, vp, vp, i64, i64, i32, ctypes.POINTER(vp), i32, vp, vp, i64,
                                            vp, sz, vp]
    L.woq_b200_linear_allgather.argtypes = [vp, vp, vp, i64, i64, i32, ctypes.POINTER(vp), i32, sz, vp, sz, vp]
    _lib = L
    return L


def _check(rc: int):
    if rc != 0:
        raise WoqError(rc, lib().woq_b200_last_error().decode())


def set_option(option: int, value: int):
    """Process-wide tuning switch (woq_b200_set_option)."""
    _check(lib().woq_b200_set_option(option, value))


def _others(others, m: int, n_out: int, out: torch.Tensor):
    """Extra operands as the C ABI wants them: rows as far apart as the output's."""
    oth = [o.reshape(m, n_out) for o in others]
    if out.stride(0) == n_out:
        return [o.contiguous() for o in oth]
    for o in oth:
        if o.stride(-1) != 1 or o.stride(0) != out.stride(0):
            raise ValueError("extra operands must have the output's row stride "
                             f"({out.stride(0)}), got {o.stride(0)}")
    return oth


def tc_plan(n_tok: int) -> dict:
    """Pipeline shape of a tcgen05 INT4 launch with n_tok token columns (woq_b200_tc_plan; no GPU needed)."""
    out = (ctypes.c_int32 * 5)()
    _check(lib().woq_b200_tc_plan(n_tok, out))
    return {"kbs": out[0], "stages": out[1], "w_ring": out[2], "a_col0": out[3], "smem_bytes": out[4]}


def static_scratch_status():
    """woq_b200_static_scratch_status on the current device: raises if a kernel gave up a wait."""
    _check(lib().woq_b200_static_scratch_status(_stream()))


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


_TORCH_T = {
    torch.float32: T_F32,
    torch.float16: T_F16,
    torch.bfloat16: T_BF16,
    torch.uint8: T_U8,
    torch.int8: T_S8,
    torch.int32: T_I32,
}


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


class Workspace:
    """Scratch buffer shared by stream-ordered calls; zeroed once at creation."""

    def __init__(self, nbytes: int, device):
        self.buf = torch.zeros(max(int(nbytes), 1), dtype=torch.uint8, device=device)

    @property
    def nbytes(self) -> int:
        return self.buf.numel()

    def status(self) -> None:
        _check(lib().woq_b200_workspace_status(self.buf.data_ptr(), _stream()))


class _DevicePointer:
    """Wraps a raw device address for torch.as_tensor (CUDA array interface)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None,
        }


class Comm:
    """Peer-mapped buffers of the tensor-parallel ranks of one node (woq_b200_comm).

    `exchange(handle_bytes) -> list of every rank's handle bytes in rank order` is how the 64-byte
    handles travel; by default torch.distributed.all_gather_object of the default group is used.
    All ranks must issue the same sequence of fused calls on a Comm."""

    HANDLE_BYTES = 64

    def __init__(self, rank: int, world: int, max_n: int, gather_bytes: int, device, exchange=None):
        self.rank, self.world = rank, world
        self.device = torch.device(device)
        self.gather_bytes = int(gather_bytes)
        self._h = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _check(lib().woq_b200_comm_create(rank, world, max_n, self.gather_bytes, ctypes.byref(self._h)))
            mine = ctypes.create_string_buffer(self.HANDLE_BYTES)
            _check(lib().woq_b200_comm_export(self._h, mine))
            if world > 1:
                if exchange is None:
                    import torch.distributed as dist

                    def exchange(b):
                        out = [None] * world
                        dist.all_gather_object(out, b)
                        return out

                handles = exchange(mine.raw)
                if len(handles) != world or any(len(h) != self.HANDLE_BYTES for h in handles):
                    raise ValueError("exchange() must return one 64-byte handle per rank")
                _check(lib().woq_b200_comm_connect(self._h, b"".join(handles)))
            else:
                _check(lib().woq_b200_comm_connect(self._h, mine.raw))
            ptr = lib().woq_b200_comm_gather_ptr(self._h)
            self._gather = torch.as_tensor(_DevicePointer(ptr, max(self.gather_bytes, 1)), device=self.device)

    def gathered(self, offset: int, m: int, n_full: int) -> torch.Tensor:
        """View of the [m, n_full] bf16 tensor at byte `offset` of this rank's gather area."""
        nbytes = m * n_full * 2
        return self._gather[offset:offset + nbytes].view(torch.bfloat16).view(m, n_full)

    def fence(self):
        """Completes an outstanding all-gather on this rank (woq_b200_comm_fence): after it the
        whole gathered tensor is in place.  Needed before reading other ranks' columns unless
        another fused call on the comm has run since the gather."""
        with torch.cuda.device(self.device):
            _check(lib().woq_b200_comm_fence(self._h, _stream()))

    def status(self):
        with torch.cuda.device(self.device):
            _check(lib().woq_b200_comm_status(self._h, _stream()))

    def close(self):
        if getattr(self, "_h", None) and self._h.value:
            torch.cuda.synchronize(self.device)
            lib().woq_b200_comm_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class WoqContext:
    """Owns one packed layer (woq_b200_ctx)."""

    def __init__(
        self,
        qweight: torch.Tensor,
        scales: torch.Tensor,
        zero_points: Optional[torch.Tensor],
        bias: Optional[torch.Tensor],
        n: int,
        k: int,
        weight_dtype: int = DTYPE_INT4,
        group_size: int = -1,
        lowp_mode: int = LOWP_BF16,
        act_quant_mode: int = ACT_NONE,
        weight_format: int = FMT_PLAIN,
        layout_flags: int = 0,
        kernel_hint: int = 0,
    ):
        for t in (qweight, scales, zero_points, bias):
            if t is not None and (not t.is_cuda or not t.is_contiguous()):
                raise ValueError("WoqContext wants contiguous CUDA tensors")
        d = Desc(
            n=n, k=k, weight_dtype=weight_dtype, group_size=group_size, lowp_mode=lowp_mode,
            act_quant_mode=act_quant_mode, weight_format=weight_format,
            scale_dtype=_TORCH_T[scales.dtype],
            zp_dtype=T_NONE if zero_points is None else _TORCH_T[zero_points.dtype],
            bias_dtype=T_NONE if bias is None else _TORCH_T[bias.dtype],
            layout_flags=layout_flags, kernel_hint=kernel_hint,
        )
        self.n, self.k = n, k
        self.device = qweight.device
        self.layout_flags = layout_flags
        self.weight_dtype = weight_dtype
        self._h = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _check(
                lib().woq_b200_ctx_create(
                    ctypes.byref(d), _ptr(qweight), _ptr(scales), _ptr(zero_points), _ptr(bias),
                    _stream(), ctypes.byref(self._h),
                )
            )
        self._ws: Optional[Workspace] = None

    # -- lifetime ---------------------------------------------------------------------
    def close(self):
        if getattr(self, "_h", None) and self._h.value:
            lib().woq_b200_ctx_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def handle(self) -> int:
        return self._h.value

    def device_bytes(self) -> int:
        return lib().woq_b200_ctx_device_bytes(self._h)

    def workspace_bytes(self, m: int) -> int:
        return lib().woq_b200_workspace_bytes(self._h, m)

    def decode_plan(self, m: int) -> dict:
        """How the M <= 16 kernel would be launched for this layer (woq_b200_decode_plan)."""
        out = (ctypes.c_int32 * 4)()
        _check(lib().woq_b200_decode_plan(self._h, m, out))
        return {"grid": out[0], "cluster": out[1], "kblocks_per_warp": out[2], "smem_budget": out[3]}

    def workspace(self, m: int) -> Workspace:
        need = self.workspace_bytes(m)
        if self._ws is None or self._ws.nbytes < need:
            self._ws = Workspace(need, self.device)
        return self._ws

    # -- compute ------------------------------------------------------------------------
    def linear(
        self,
        x: torch.Tensor,
        fusion: int = FUSE_NONE,
        others: Sequence[torch.Tensor] = (),
        out: Optional[torch.Tensor] = None,
        workspace: Optional[Workspace] = None,
    ) -> torch.Tensor:
        if x.dtype != torch.bfloat16 or not x.is_cuda:
            raise ValueError("x must be a bf16 CUDA tensor")
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        m = x2.shape[0]
        n_out = self.n // 2 if fusion == FUSE_SILU_MUL else self.n
        if out is None:
            out = torch.empty((m, n_out), dtype=torch.bfloat16, device=x.device)
        ws = workspace or self.workspace(m)
        oth = _others(others, m, n_out, out)
        arr = (ctypes.c_void_p * max(len(oth), 1))(*[o.data_ptr() for o in oth])
        with torch.cuda.device(self.device):
            _check(
                lib().woq_b200_linear(
                    self._h, x2.data_ptr(), m, x2.stride(0), fusion, arr, len(oth),
                    out.data_ptr(), out.stride(0), ws.buf.data_ptr(), ws.nbytes, _stream(),
                )
            )
        return out.reshape(*x.shape[:-1], n_out)

    def linear_any(self, x: torch.Tensor, fusion: int = FUSE_NONE, others: Sequence[torch.Tensor] = (),
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """woq_b200_linear_any: activations, extra tensors and output of x's dtype (bf16, fp16
        or fp32); the compute dtype follows the context's lowp mode."""
        if x.dtype not in (torch.bfloat16, torch.float16, torch.float32) or not x.is_cuda:
            raise ValueError("x must be a bf16, fp16 or fp32 CUDA tensor")
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        m = x2.shape[0]
        if out is None:
            out = torch.empty((m, self.n), dtype=x.dtype, device=x.device)
        oth = [o.to(x.dtype) for o in _others(others, m, self.n, out)]
        arr = (ctypes.c_void_p * max(len(oth), 1))(*[o.data_ptr() for o in oth])
        ws = self.workspace(m)
        with torch.cuda.device(self.device):
            _check(lib().woq_b200_linear_any(
                self._h, x2.data_ptr(), _TORCH_T[x.dtype], m, x2.stride(0), fusion, arr, len(oth),
                out.data_ptr(), out.stride(0), ws.buf.data_ptr(), ws.nbytes, _stream()))
        return out.reshape(*x.shape[:-1], self.n)

    def dump_dequant_f32(self, compute_dtype: torch.dtype) -> torch.Tensor:
        """General-route contexts: the values the kernel multiplies by, as fp32 [n, k]."""
        out = torch.empty((self.n, self.k), dtype=torch.float32, device=self.device)
        with torch.cuda.device(self.device):
            _check(lib().woq_b200_dump_dequant_f32(self._h, _TORCH_T[compute_dtype], out.data_ptr(), _stream()))
        return out

    def linear_allreduce(self, comm: "Comm", x, fusion: int = FUSE_NONE, others: Sequence[torch.Tensor] = (),
                         bias: Optional[torch.Tensor] = None, out=None, workspace=None) -> torch.Tensor:
        """Row-parallel linear (this rank's K shard) fused with the all-reduce; 1..16 tokens."""
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        m = x2.shape[0]
        if out is None:
            out = torch.empty((m, self.n), dtype=torch.bfloat16, device=x.device)
        ws = workspace or self.workspace(m)
        oth = [o.reshape(m, self.n).contiguous() for o in others]
        arr = (ctypes.c_void_p * max(len(oth), 1))(*[o.data_ptr() for o in oth])
        if bias is not None and (bias.dtype != torch.float32 or not bias.is_cuda):
            raise ValueError("bias must be an fp32 CUDA tensor")
        with torch.cuda.device(self.device):
            _check(lib().woq_b200_linear_allreduce(
                self._h, comm._h, x2.data_ptr(), m, x2.stride(0), fusion, arr, len(oth), _ptr(bias),
                out.data_ptr(), out.stride(0), ws.buf.data_ptr(), ws.nbytes, _stream()))
        return out

    def linear_allgather(self, comm: "Comm", x, fusion: int = FUSE_NONE, others: Sequence[torch.Tensor] = (),
                         gather_offset: int = 0, workspace=None) -> torch.Tensor:
        """Column-parallel linear (this rank's N shard) fused with the all-gather; returns the
        gathered [m, world * n_out] view inside the comm's gather area."""
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        m = x2.shape[0]
        n_out = self.n // 2 if fusion == FUSE_SILU_MUL else self.n
        ws = workspace or self.workspace(m)
        oth = [o.reshape(m, n_out).contiguous() for o in others]
        arr = (ctypes.c_void_p * max(len(oth), 1))(*[o.data_ptr() for o in oth])
        with torch.cuda.device(self.device):
            _check(lib().woq_b200_linear_allgather(
                self._h, comm._h, x2.data_ptr(), m, x2.stride(0), fusion, arr, len(oth), gather_offset,
                ws.buf.data_ptr(), ws.nbytes, _stream()))
        return comm.gathered(gather_offset, m, n_out * comm.world)

    def linear_static_scratch(self, x, fusion=FUSE_NONE, others=(), out=None):
        """woq_b200_linear_static_scratch: at most 16 tokens, scratch inside the library, no
        allocation by the library (the output tensor is the caller's)."""
        x2 = x.reshape(-1, x.shape[-1])
        m = x2.shape[0]
        n_out = self.n // 2 if fusion == FUSE_SILU_MUL else self.n
        if out is None:
            out = torch.empty((m, n_out), dtype=torch.bfloat16, device=x.device)
        oth = _others(others, m, n_out, out)
        arr = (ctypes.c_void_p * max(len(oth), 1))(*[o.data_ptr() for o in oth])
        with torch.cuda.device(self.device):
            _check(
                lib().woq_b200_linear_static_scratch(
                    self._h, x2.data_ptr(), m, x2.stride(0), fusion, arr, len(oth),
                    out.data_ptr(), out.stride(0), _stream(),
                )
            )
        return out

    def linear_scatter(self, x, row_idx, row_weight, out, workspace=None):
        x2 = x.reshape(-1, x.shape[-1])
        m = x2.shape[0]
        ws = workspace or self.workspace(m)
        with torch.cuda.device(self.device):
            _check(
                lib().woq_b200_linear_scatter(
                    self._h, x2.data_ptr(), m, x2.stride(0), row_idx.data_ptr(),
                    row_weight.data_ptr(), out.data_ptr(), out.stride(0), ws.buf.data_ptr(),
                    ws.nbytes, _stream(),
                )
            )
        return out

    def unpack(self) -> torch.Tensor:
        if self.weight_dtype in (DTYPE_INT4, DTYPE_NF4):
            out = torch.empty((self.n, (self.k + 1) // 2), dtype=torch.uint8, device=self.device)
        else:
            out = torch.empty((self.n, self.k), dtype=torch.uint8 if self.weight_dtype == DTYPE_FP8 else torch.int8,
                              device=self.device)
        with torch.cuda.device(self.device):
            _check(lib().woq_b200_ctx_unpack(self._h, out.data_ptr(), _stream()))
        return out

    def dump_dequant(self) -> torch.Tensor:
        out = torch.empty((self.n, self.k), dtype=torch.bfloat16, device=self.device)
        with torch.cuda.device(self.device):
            _check(lib().woq_b200_dump_dequant(self._h, out.data_ptr(), _stream()))
        return out

    def route(self) -> int:
        return lib().woq_b200_ctx_route(self._h)

    def int8_block_internals(self, x: torch.Tensor):
        """K-block INT8 route: codes [m, k] (u8 bit patterns), scales and zero points [m, k / block],
        block accumulators [k / block, m, n] (woq_b200_int8_block_internals)."""
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        m = x2.shape[0]
        kb = lib().woq_b200_int8_block_size(self._h)
        kc = self.k // kb
        qa = torch.empty((m, self.k), dtype=torch.uint8, device=self.device)
        sa = torch.empty((m, kc), dtype=torch.float32, device=self.device)
        zpa = torch.empty((m, kc), dtype=torch.int32, device=self.device)
        acc = torch.empty((kc, m, self.n), dtype=torch.int32, device=self.device)
        ws = self.workspace(m)
        with torch.cuda.device(self.device):
            _check(lib().woq_b200_int8_block_internals(
                self._h, x2.data_ptr(), m, x2.stride(0), qa.data_ptr(), sa.data_ptr(), zpa.data_ptr(),
                acc.data_ptr(), ws.buf.data_ptr(), ws.nbytes, _stream()))
        return qa, sa, zpa, acc

    def int8_internals(self, x: torch.Tensor):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        m = x2.shape[0]
        qa = torch.empty((m, self.k), dtype=torch.int8, device=self.device)
        sa = torch.empty((m,), dtype=torch.float32, device=self.device)
        acc = torch.empty((m, self.n), dtype=torch.int32, device=self.device)
        ws = self.workspace(m)
        with torch.cuda.device(self.device):
            _check(
                lib().woq_b200_int8_internals(
                    self._h, x2.data_ptr(), m, x2.stride(0), qa.data_ptr(), sa.data_ptr(),
                    acc.data_ptr(), ws.buf.data_ptr(), ws.nbytes, _stream(),
                )
            )
        return qa, sa, acc

    def linear_prequant(self, qa, sa, zpa=None, fusion: int = FUSE_NONE, others=(), out=None, workspace=None):
        """woq_b200_linear_prequant: the linear on activations quantised beforehand (rmsnorm_quant)."""
        m = qa.shape[0]
        n_out = self.n // 2 if fusion == FUSE_SILU_MUL else self.n
        y = out if out is not None else torch.empty((m, n_out), dtype=torch.bfloat16, device=self.device)
        ws = workspace if workspace is not None else self.workspace(m)
        oth = _others(others, m, n_out, y)
        arr = (ctypes.c_void_p * max(len(oth), 1))(*[o.data_ptr() for o in oth])
        with torch.cuda.device(self.device):
            _check(
                lib().woq_b200_linear_prequant(
                    self._h, qa.data_ptr(), sa.data_ptr(), None if zpa is None else zpa.data_ptr(), m, fusion,
                    arr, len(oth), y.data_ptr(), y.stride(0), ws.buf.data_ptr(), ws.nbytes, _stream(),
                )
            )
        return y

    def int8_zero_points(self, m: int) -> torch.Tensor:
        """Activation zero points the latest INT8 call with m tokens left in this context's workspace."""
        zp = torch.empty((m,), dtype=torch.int32, device=self.device)
        ws = self.workspace(m)
        with torch.cuda.device(self.device):
            _check(lib().woq_b200_int8_zero_points(self._h, m, zp.data_ptr(), ws.buf.data_ptr(), ws.nbytes, _stream()))
        return zp


def rmsnorm_quant(x: torch.Tensor, gamma: torch.Tensor, eps: float, act_quant_mode: int = 6, want_y: bool = False):
    """woq_b200_rmsnorm_quant on torch tensors: x bf16 [m, k], gamma bf16 [k].  Returns
    (qa int8 [m, k], sa f32 [m], zpa int32 [m] or None, y bf16 [m, k] or None)."""
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    m, k = x2.shape
    dev = x.device
    qa = torch.empty((m, k), dtype=torch.int8, device=dev)
    sa = torch.empty((m,), dtype=torch.float32, device=dev)
    zpa = torch.empty((m,), dtype=torch.int32, device=dev) if act_quant_mode == ACT_PER_M else None
    y = torch.empty((m, k), dtype=torch.bfloat16, device=dev) if want_y else None
    g = gamma.to(device=dev, dtype=torch.bfloat16).contiguous()
    with torch.cuda.device(dev):
        _check(
            lib().woq_b200_rmsnorm_quant(
                x2.data_ptr(), x2.stride(0), g.data_ptr(), float(eps), m, k, act_quant_mode,
                None if y is None else y.data_ptr(), k, qa.data_ptr(), sa.data_ptr(),
                None if zpa is None else zpa.data_ptr(), _stream(),
            )
        )
    return qa, sa, zpa, y


def moe_expert(w13: "WoqContext", w2: "WoqContext", hidden, token_idx, token_weight, out, workspace=None):
    """woq_b200_moe_expert on torch tensors; token_idx int32 [t], token_weight bf16 [t]."""
    t = int(token_idx.numel())
    need = lib().woq_b200_moe_workspace_bytes(w13._h, w2._h, t)
    ws = workspace if workspace is not None and workspace.nbytes >= need else Workspace(need, hidden.device)
    with torch.cuda.device(hidden.device):
        _check(
            lib().woq_b200_moe_expert(
                w13._h, w2._h, hidden.data_ptr(), hidden.stride(0), token_idx.data_ptr(),
                token_weight.data_ptr(), t, out.data_ptr(), out.stride(0), ws.buf.data_ptr(), ws.nbytes,
                _stream(),
            )
        )
    return ws


def kernel_launches() -> int:
    return int(lib().woq_b200_kernel_launches())
