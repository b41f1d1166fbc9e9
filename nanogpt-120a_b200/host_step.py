"""ctypes binding of the C++ training-step driver (include/nvfp4_b200_step.hpp behind include/nvfp4_b200_step.h).

The driver owns its quantized operands, scratch, gradient buckets, streams and (multi-GPU) an NCCL
communicator, and enqueues a whole forward + backward pass of the projection set from C++: one call per step
instead of several hundred Python-level launches.  It is the caller side of the C ABI -- the role
crates/gpt2-nvfp4 plays for the reference's kernels -- with no PyTorch on the path; this module only hands it
the device pointers of the input tensors (weights, activations, upstream gradients) that `ProjectionSet`
already holds, and wraps its outputs as torch tensors for the tests and the benchmark.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_int, c_uint8, c_uint32, c_uint64, c_void_p
from typing import Dict, List, Optional

import torch

from . import Nvfp4Error, library

_HERE = os.path.dirname(os.path.abspath(__file__))
STEP_LIB_PATH = os.path.join(_HERE, "libnvfp4_b200_step.so")
_lib = None


class StepConfig(Structure):
    _fields_ = [("n_layer", c_uint32), ("d_model", c_uint32), ("d_mlp", c_uint32), ("vocab", c_uint32),
                ("tokens", c_uint32), ("token_offset", c_uint32), ("total_tokens", c_uint32), ("seed", c_uint64),
                ("fused_mlp", c_int), ("reproducible_sharding", c_int)]


def step_library() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        library()  # the kernel library first: the step library links against it
        if not os.path.exists(STEP_LIB_PATH):
            raise RuntimeError(f"{STEP_LIB_PATH} is missing: build it with `python nanogpt-120a_b200/build.py`")
        lib = ctypes.CDLL(STEP_LIB_PATH)
        PP = POINTER(c_void_p)
        PU = POINTER(c_uint32)
        lib.nvfp4_step_create.restype = c_void_p
        lib.nvfp4_step_create.argtypes = [POINTER(StepConfig), PP, PP, c_uint32, PU, PP, c_uint32, PU, PP, c_uint32]
        lib.nvfp4_step_destroy.restype = None
        lib.nvfp4_step_destroy.argtypes = [c_void_p]
        lib.nvfp4_step_error.restype = c_char_p
        lib.nvfp4_step_error.argtypes = [c_void_p]
        lib.nvfp4_step_run.restype = c_int
        lib.nvfp4_step_run.argtypes = [c_void_p, c_void_p, c_int]
        lib.nvfp4_step_set_inputs.restype = c_int
        lib.nvfp4_step_set_inputs.argtypes = [c_void_p, PU, PP, c_uint32, PU, PP, c_uint32]
        lib.nvfp4_step_bucket.restype = c_int
        lib.nvfp4_step_bucket.argtypes = [c_void_p, c_uint32, POINTER(c_void_p), POINTER(c_uint64)]
        lib.nvfp4_step_dx.restype = c_int
        lib.nvfp4_step_dx.argtypes = [c_void_p, c_uint32, POINTER(c_void_p)]
        lib.nvfp4_step_y.restype = c_int
        lib.nvfp4_step_y.argtypes = [c_void_p, c_uint32, POINTER(c_void_p)]
        lib.nvfp4_step_flops.restype = c_uint64
        lib.nvfp4_step_flops.argtypes = [c_void_p]
        lib.nvfp4_step_nccl_unique_id.restype = c_int
        lib.nvfp4_step_nccl_unique_id.argtypes = [POINTER(c_uint8)]
        lib.nvfp4_step_attach_nccl.restype = c_int
        lib.nvfp4_step_attach_nccl.argtypes = [c_void_p, POINTER(c_uint8), c_int, c_int]
        _lib = lib
    return _lib


def _ptr_array(tensors):
    arr = (c_void_p * len(tensors))()
    for i, t in enumerate(tensors):
        arr[i] = None if t is None else t.data_ptr()
    return arr


def _width_arrays(group: Dict[int, torch.Tensor]):
    widths = sorted(group)
    return (c_uint32 * len(widths))(*widths), _ptr_array([group[w] for w in widths]), len(widths)


def _as_tensor(ptr: int, numel: int, dtype: torch.dtype, device) -> torch.Tensor:
    """A torch view of device memory the C++ driver owns (valid while the driver lives)."""
    nbytes = numel * torch.empty((), dtype=dtype).element_size()

    class _Iface:
        __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}

    return torch.as_tensor(_Iface(), device=device).view(dtype)


class HostStep:
    """The projection set of `ProjectionSet` driven by the C++ step driver: same inputs, same seeds, same
    kernels, same bytes; Python touches it once per step."""

    def __init__(self, ps, process_group=None):
        """`ps`: a `ProjectionSet` that supplies shape, token shard, seed and the input tensors."""
        lib = step_library()
        self._lib, self.ps, self.device = lib, ps, ps.device
        shape = ps.shape
        cfg = StepConfig(shape.n_layer, shape.d_model, shape.d_mlp, shape.vocab, ps.tokens, ps.token_offset,
                         ps.total_tokens, ps.seed, 1 if ps.fused_mlp else 0, 1 if ps.reproducible else 0)
        linears = ps.all_linears()
        self._keep = [_ptr_array([l.weight for l in linears]), _ptr_array([l.bias for l in linears])]
        xw, xp, nx = _width_arrays(ps.x)
        dw, dp, nd = _width_arrays(ps.dy)
        with torch.cuda.device(self.device):
            self.handle = lib.nvfp4_step_create(ctypes.byref(cfg), self._keep[0], self._keep[1], len(linears), xw, xp, nx,
                                                dw, dp, nd)
        if not self.handle:
            raise RuntimeError("nvfp4_step_create failed: " + lib.nvfp4_step_error(None).decode())
        self.buckets: List[torch.Tensor] = []
        for i in range(shape.n_layer + 1):
            p, n = c_void_p(), c_uint64()
            self._check(lib.nvfp4_step_bucket(self.handle, i, ctypes.byref(p), ctypes.byref(n)))
            self.buckets.append(_as_tensor(p.value, n.value, torch.float32, self.device))
        if process_group is not None:
            self._attach(process_group)

    def _check(self, rc: int) -> None:
        if rc != 0:
            raise Nvfp4Error(rc, self._lib.nvfp4_step_error(self.handle).decode())

    def _attach(self, pg) -> None:
        """Creates the driver's own NCCL communicator: rank 0 draws the id, torch.distributed carries its 128
        bytes to the other ranks (plumbing only; the all-reduces of a step are issued from C++)."""
        import torch.distributed as dist

        rank, world = dist.get_rank(pg), dist.get_world_size(pg)
        ident = (c_uint8 * 128)()
        if rank == 0:
            rc = self._lib.nvfp4_step_nccl_unique_id(ident)
            if rc != 0:
                raise RuntimeError("ncclGetUniqueId failed: " + self._lib.nvfp4_step_error(None).decode())
        t = torch.tensor(list(ident), dtype=torch.uint8, device=self.device)
        dist.broadcast(t, src=dist.get_global_rank(pg, 0) if hasattr(dist, "get_global_rank") else 0, group=pg)
        ident = (c_uint8 * 128)(*t.cpu().tolist())
        with torch.cuda.device(self.device):
            self._check(self._lib.nvfp4_step_attach_nccl(self.handle, ident, rank, world))

    def step(self, weights_changed: bool = True) -> None:
        self._check(self._lib.nvfp4_step_run(self.handle, c_void_p(torch.cuda.current_stream().cuda_stream),
                                             1 if weights_changed else 0))

    def set_inputs(self, x: Dict[int, torch.Tensor], dy: Dict[int, torch.Tensor]) -> None:
        xw, xp, nx = _width_arrays(x)
        dw, dp, nd = _width_arrays(dy)
        self._inputs = (x, dy)  # keep the tensors alive
        self._check(self._lib.nvfp4_step_set_inputs(self.handle, xw, xp, nx, dw, dp, nd))

    def dx(self, width: int) -> torch.Tensor:
        p = c_void_p()
        self._check(self._lib.nvfp4_step_dx(self.handle, width, ctypes.byref(p)))
        return _as_tensor(p.value, self.ps.tokens * width, torch.bfloat16, self.device).view(self.ps.tokens, width)

    def y(self, width: int) -> torch.Tensor:
        p = c_void_p()
        self._check(self._lib.nvfp4_step_y(self.handle, width, ctypes.byref(p)))
        return _as_tensor(p.value, self.ps.tokens * width, torch.bfloat16, self.device).view(self.ps.tokens, width)

    def flops_per_step(self) -> int:
        return int(self._lib.nvfp4_step_flops(self.handle))

    def result_digest(self) -> torch.Tensor:
        return torch.stack([b.abs().sum() for b in self.buckets])

    def close(self) -> None:
        if getattr(self, "handle", None):
            torch.cuda.synchronize(self.device)
            self._lib.nvfp4_step_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
