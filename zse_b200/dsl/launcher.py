"""Launch configuration and the launch itself (zse-compiler/zse_compiler/runtime/launcher.py:14-318).

``LaunchConfig`` pads grid and block to three dimensions and checks them against the limits of the target (1024
threads per block, 227 KB of shared memory per block on sm_100, grid limits of the driver API).  ``KernelLauncher``
packs the arguments (tensors as device addresses, numbers by the parameter's declared type) and calls
``cuLaunchKernel`` on torch's current stream, so a launch is ordered with the surrounding torch work and can be
captured in a CUDA graph; it does not synchronise."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Any, List, Optional, Sequence, Tuple

from . import dtypes
from .compiler import CompiledKernel, _check, _driver
from .errors import KernelLaunchError, KernelTypeError

MAX_THREADS_PER_BLOCK = 1024
MAX_BLOCK_DIM = (1024, 1024, 64)
MAX_GRID_DIM = (2**31 - 1, 65535, 65535)
MAX_SHARED_BYTES = 227 * 1024            # opt-in limit of one block on sm_100
DEFAULT_SHARED_BYTES = 48 * 1024         # above this a kernel must opt in (done here before the launch)


def _pad3(v: Sequence[int], what: str) -> Tuple[int, int, int]:
    v = tuple(int(x) for x in (v if isinstance(v, (tuple, list)) else (v,)))
    if not 1 <= len(v) <= 3 or any(x <= 0 for x in v):
        raise KernelLaunchError(f"{what} must have one to three positive dimensions, got {v}")
    return v + (1,) * (3 - len(v))


@dataclass
class LaunchConfig:
    grid: Tuple[int, ...]
    block: Tuple[int, ...]
    shared_mem_bytes: int = 0

    def __post_init__(self):
        self.grid, self.block = _pad3(self.grid, "grid"), _pad3(self.block, "block")
        self.validate()

    @property
    def threads_per_block(self) -> int:
        return self.block[0] * self.block[1] * self.block[2]

    @property
    def total_threads(self) -> int:
        return self.threads_per_block * self.grid[0] * self.grid[1] * self.grid[2]

    def validate(self, static_shared_bytes: int = 0, needs_full_warps: bool = False) -> None:
        if self.threads_per_block > MAX_THREADS_PER_BLOCK:
            raise KernelLaunchError(f"{self.threads_per_block} threads per block exceeds {MAX_THREADS_PER_BLOCK}")
        for i in range(3):
            if self.block[i] > MAX_BLOCK_DIM[i]:
                raise KernelLaunchError(f"block dimension {i} = {self.block[i]} exceeds {MAX_BLOCK_DIM[i]}")
            if self.grid[i] > MAX_GRID_DIM[i]:
                raise KernelLaunchError(f"grid dimension {i} = {self.grid[i]} exceeds {MAX_GRID_DIM[i]}")
        if self.shared_mem_bytes < 0 or self.shared_mem_bytes + static_shared_bytes > MAX_SHARED_BYTES:
            raise KernelLaunchError(f"{self.shared_mem_bytes + static_shared_bytes} bytes of shared memory exceed "
                                    f"the {MAX_SHARED_BYTES} a block can have")
        if needs_full_warps and self.threads_per_block % 32:
            raise KernelLaunchError(f"the kernel uses warp or block collectives: its block size "
                                    f"({self.threads_per_block}) must be a multiple of 32")


def pack_args(param_ctypes: Sequence[str], args: Sequence[Any], elems: Sequence[Any] = ()) -> List[Any]:
    """ctypes values in parameter order.  ``param_ctypes``: C type of each parameter (``float*``, ``int``...);
    ``elems``: expected element type name of each tensor parameter (None for scalars), checked against torch tensors."""
    if len(param_ctypes) != len(args):
        raise KernelTypeError(f"the kernel takes {len(param_ctypes)} arguments, got {len(args)}")
    out = []
    for i, (ct, a) in enumerate(zip(param_ctypes, args)):
        if ct.endswith("*"):
            want = elems[i] if i < len(elems) else None
            a = getattr(a, "data", a) if isinstance(a, dtypes.Tensor) else a
            if hasattr(a, "data_ptr"):
                if hasattr(a, "is_contiguous") and not a.is_contiguous():
                    raise KernelTypeError(f"argument {i} must be contiguous")
                if want and hasattr(a, "dtype") and dtypes.ALL[want].torch_name:
                    have = str(a.dtype).replace("torch.", "")
                    if have != dtypes.ALL[want].torch_name:
                        raise KernelTypeError(f"argument {i} holds {have} but the kernel expects {want}")
                out.append(ctypes.c_void_p(int(a.data_ptr())))
            elif isinstance(a, int):
                out.append(ctypes.c_void_p(a))
            else:
                raise KernelTypeError(f"argument {i} must be a tensor or a device address, not {type(a).__name__}")
        elif ct == "float":
            out.append(ctypes.c_float(float(a)))
        elif ct == "bool":
            out.append(ctypes.c_bool(bool(a)))
        elif ct == "unsigned int":
            out.append(ctypes.c_uint(int(a)))
        else:
            out.append(ctypes.c_int(int(a)))
    return out


class PrepackedArgs:
    """The argument array of a kernel, built once and changed in place (``set``): repeated launches skip the packing,
    and the array keeps its address (zse-compiler/zse_compiler/runtime/launcher.py: ``PrepackedArgs``)."""

    def __init__(self, param_ctypes: Sequence[str], args: Sequence[Any], elems: Sequence[Any] = ()):
        self._ctypes, self._elems = list(param_ctypes), list(elems) or [None] * len(param_ctypes)
        self.values = pack_args(param_ctypes, args, elems)
        self.array = (ctypes.c_void_p * len(self.values))(
            *[ctypes.cast(ctypes.pointer(v), ctypes.c_void_p) for v in self.values])

    def set(self, index: int, value: Any) -> None:
        new = pack_args([self._ctypes[index]], [value], [self._elems[index]])[0]
        self.values[index].value = new.value            # same storage, so ``array`` stays valid

    # ---- the reference's way of building and updating the array (launcher.py:251-318 there) -------------------------
    @classmethod
    def from_args(cls, *args) -> "PrepackedArgs":
        """From values alone: tensors (descriptors, torch tensors) and raw addresses become pointers, ints ``int``,
        floats ``float``.  The typed constructor above additionally checks element types against the kernel."""
        ctypes_of, args = [], list(args)
        for i, a in enumerate(args):
            if isinstance(a, dtypes.Tensor) or hasattr(a, "data_ptr"):
                ctypes_of.append("void*")
                if isinstance(a, dtypes.Tensor) and a.data is None:
                    args[i] = int(a.data_ptr)          # a bare description: its address (0) is filled in by set_ptr
            elif isinstance(a, bool):
                ctypes_of.append("bool")
            elif isinstance(a, int):
                ctypes_of.append("int")
            elif isinstance(a, float):
                ctypes_of.append("float")
            else:
                raise TypeError(f"Unsupported arg type: {type(a)}")
        return cls(ctypes_of, list(args))

    def set_ptr(self, index: int, ptr_value: int) -> None:
        self.values[index].value = int(ptr_value)

    def set_int(self, index: int, value: int) -> None:
        self.values[index].value = int(value)

    def set_float(self, index: int, value: float) -> None:
        self.values[index].value = float(value)

    @property
    def arg_array(self):
        """The ``void**`` array handed to the driver (stable for the life of the object)."""
        return self.array

    def __len__(self) -> int:
        return len(self.values)

    @property
    def address(self) -> int:
        return ctypes.addressof(self.array)


class KernelLauncher:
    def sync(self, compiled: Optional[CompiledKernel] = None) -> None:
        """Waits for everything launched so far (launches are asynchronous).  Without a device there is nothing to
        wait for."""
        import torch
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    def launch_prepacked(self, compiled: CompiledKernel, config: LaunchConfig, prepacked: PrepackedArgs,
                         stream=None) -> None:
        self.launch(compiled, config, prepacked.values, stream)

    def launch(self, compiled: CompiledKernel, config: LaunchConfig, packed: List[Any], stream=None) -> None:
        import torch
        if not torch.cuda.is_available():
            raise KernelLaunchError("no CUDA device: use .emulate(...) to run the kernel on the CPU")
        drv = _driver()
        fn = compiled.function()
        if config.shared_mem_bytes > DEFAULT_SHARED_BYTES:
            err, = drv.cuFuncSetAttribute(fn, drv.CUfunction_attribute.CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES,
                                          int(config.shared_mem_bytes))
            _check(err, "raising the shared-memory limit")
        ptrs = (ctypes.c_void_p * len(packed))(*[ctypes.cast(ctypes.pointer(p), ctypes.c_void_p) for p in packed])
        s = stream if stream is not None else torch.cuda.current_stream()
        handle = drv.CUstream(int(getattr(s, "cuda_stream", s)))
        err, = drv.cuLaunchKernel(fn, *config.grid, *config.block, int(config.shared_mem_bytes), handle,
                                  ctypes.addressof(ptrs), 0)
        _check(err, f"launching '{compiled.name}'")
