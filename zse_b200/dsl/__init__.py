"""Kernel language: write a GPU kernel as a restricted Python function, get CUDA C for sm_100a, a cubin, a launch on
torch's stream - and a CPU emulation of the same launch for development and tests.

    import zse_b200.dsl as zse

    @zse.kernel
    def scale_add(x: zse.Tensor, y: zse.Tensor, out: zse.Tensor, alpha: float, n: int):
        i = zse.global_id(0)
        if i < n:
            out[i] = alpha * x[i] + y[i]

    print(scale_add.source())                                    # CUDA text
    scale_add.emulate((blocks,), (256,), (x, y, out, 2.0, n))    # CPU tensors
    scale_add.launch((blocks,), (256,), (x, y, out, 2.0, n))     # CUDA tensors

This is the counterpart of the reference's ``zse_compiler`` package (zse-compiler/zse_compiler/__init__.py:1-95) with
one target instead of three.  The engine's hot kernels are hand-written CUDA (``csrc/``); this package is for the
surrounding element-wise and reduction work a user wants to add without writing C++."""
from ..runtime.device import DeviceInfo, detect_backend, get_devices
from ..runtime.profiler import AutoTuner, KernelProfile, KernelProfiler, TuneResult
from .compiler import CompiledKernel, RuntimeCompiler
from .dtypes import (DType, Tensor, bfloat16, empty, float16, float32, int4, int8, int16, int32, uint4, uint8, uint16,
                     uint32, zeros)
from .emulate import KernelRaceError, RaceTracker
from .codegen import BaseCodegen, CUDACodegen
from .errors import (KernelCompileError, KernelError, KernelLaunchError, KernelSyntaxError, KernelTypeError,
                     SourceLocation)
from .infer import infer as infer_types
from .parser import validate_kernel

KernelValidationError = KernelSyntaxError          # the reference's name for what its validator raises
from .kernel import KernelFunction, fuse, kernel
from .launcher import KernelLauncher, LaunchConfig, PrepackedArgs
from .memory import GPUMemory
from .primitives import *          # noqa: F401,F403  (thread_id, warp_reduce_sum, ... for use inside kernels)
from .primitives import __all__ as _prims

__all__ = ["kernel", "fuse", "KernelFunction", "DType", "Tensor", "empty", "zeros", "float16", "float32", "bfloat16",
           "int32", "int16", "int8", "uint32", "uint16", "uint8", "int4", "uint4", "detect_backend", "get_devices",
           "DeviceInfo", "GPUMemory", "RuntimeCompiler", "CompiledKernel", "KernelLauncher", "LaunchConfig", "PrepackedArgs",
           "KernelProfiler", "KernelProfile", "AutoTuner", "TuneResult", "SourceLocation", "BaseCodegen", "CUDACodegen",
           "KernelError", "KernelSyntaxError", "KernelTypeError", "KernelCompileError",
           "KernelLaunchError", "KernelRaceError", "RaceTracker"] + list(_prims)
