"""``@kernel``, ``KernelFunction`` and ``fuse`` (zse-compiler/zse_compiler/kernel.py:40-158).

A decorated function is validated and parsed once.  Types are settled per *signature* - the element types of the
tensor arguments - so one Python kernel serves fp32, fp16 and bf16 tensors: ``source()`` shows the text for a
signature (all-fp32 unless told otherwise), ``compile()`` builds its cubin for sm_100a (no GPU needed),
``launch()`` picks the signature from the arguments and launches on torch's current stream, and ``emulate()`` runs
the same launch on the CPU."""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

from . import dtypes, ir
from .codegen import generate_cuda
from .compiler import CompiledKernel, RuntimeCompiler, default_compiler
from .emulate import emulate as _emulate
from .errors import KernelTypeError
from .infer import TypedKernel, infer
from .launcher import KernelLauncher, LaunchConfig, PrepackedArgs, pack_args
from .parser import KernelParser, validate_kernel
from .primitives import COLLECTIVES, WARP_WIDE

Signature = Tuple[Tuple[str, str], ...]


class KernelFunction:
    def __init__(self, func: Optional[Callable], ir_func: Optional[ir.Function] = None,
                 compiler: Optional[RuntimeCompiler] = None):
        self._func = func
        self.warnings: List[str] = []
        if ir_func is None:
            self.warnings = validate_kernel(func)
            ir_func = KernelParser().parse(func)
        self._ir = ir_func
        self._name = ir_func.name
        self._typed: Dict[Signature, TypedKernel] = {}
        self._compiled: Dict[Signature, CompiledKernel] = {}
        self._compiler = compiler
        self._launcher = KernelLauncher()
        self.__doc__ = getattr(func, "__doc__", None)

    # ---- facts --------------------------------------------------------------------------------------------------
    @property
    def name(self) -> str:
        return self._name

    @property
    def ir(self) -> ir.Function:
        return self._ir

    @property
    def params(self) -> List[ir.Param]:
        return list(self._ir.params)

    def _sig(self, dtypes_by_param: Optional[Dict[str, Any]]) -> Signature:
        out = []
        for p in self._ir.params:
            if p.kind != "tensor":
                continue
            d = p.elem or (dtypes_by_param or {}).get(p.name) or "float32"
            d = d.name if isinstance(d, dtypes.DType) else str(d)
            if d not in dtypes.ALL:
                raise KernelTypeError(f"'{d}' is not an element type")
            if p.elem and (dtypes_by_param or {}).get(p.name) not in (None, p.elem, dtypes.ALL[p.elem]):
                raise KernelTypeError(f"parameter '{p.name}' is declared {p.elem}")
            out.append((p.name, d))
        return tuple(out)

    def _sig_of_args(self, args: Sequence[Any]) -> Signature:
        if len(args) != len(self._ir.params):
            raise KernelTypeError(f"{self._name}() takes {len(self._ir.params)} arguments, got {len(args)}")
        by = {}
        for p, a in zip(self._ir.params, args):
            if p.kind != "tensor":
                continue
            if isinstance(a, dtypes.Tensor):
                by[p.name] = a.dtype.name
            elif hasattr(a, "dtype") and hasattr(a, "data_ptr"):
                by[p.name] = dtypes.from_torch(a.dtype).name
            elif hasattr(a, "dtype"):
                by[p.name] = str(a.dtype)
            if p.elem and by.get(p.name, p.elem) != p.elem and dtypes.ALL[p.elem].torch_name:
                raise KernelTypeError(f"argument '{p.name}' holds {by[p.name]} but is declared {p.elem}")
            if p.elem:
                by[p.name] = p.elem
        return self._sig(by)

    def typed(self, dtypes_by_param: Optional[Dict[str, Any]] = None) -> TypedKernel:
        sig = self._sig(dtypes_by_param)
        k = self._typed.get(sig)
        if k is None:
            import copy
            k = self._typed[sig] = infer(copy.deepcopy(self._ir), dict(sig))
        return k

    # ---- text, binary, launch -----------------------------------------------------------------------------------
    def source(self, backend: Optional[str] = "cuda", dtypes: Optional[Dict[str, Any]] = None,
               line_info: bool = False) -> str:
        if backend not in (None, "cuda"):
            raise ValueError(f"Unknown backend: {backend}. Available: ['cuda'] (sm_100a)")
        return generate_cuda(self.typed(dtypes), line_info)

    def compile(self, backend: Optional[str] = "cuda", dtypes: Optional[Dict[str, Any]] = None) -> CompiledKernel:
        if backend not in (None, "cuda"):
            raise ValueError(f"Unknown backend: {backend}. Available: ['cuda'] (sm_100a)")
        sig = self._sig(dtypes)
        ck = self._compiled.get(sig)
        if ck is None:
            comp = self._compiler or default_compiler()
            ck = self._compiled[sig] = comp.compile(self.source("cuda", dict(sig), line_info=True), self._name)
        return ck

    def resources(self, dtypes: Optional[Dict[str, Any]] = None) -> Dict[str, int]:
        """Registers, spills and shared memory of the compiled kernel, as ptxas reports them."""
        comp = self._compiler or default_compiler()
        return comp.resource_usage(self.source("cuda", dtypes, line_info=True), self._name)

    def uses_collectives(self) -> bool:
        return any(isinstance(e, ir.Call) and (e.func in COLLECTIVES or e.func in WARP_WIDE)
                   and e.func not in ("syncthreads",)
                   for e in ir.walk_exprs(self._ir.body))

    def static_shared_bytes(self) -> int:
        n = 0
        for s in ir.walk_stmts(self._ir.body):
            if isinstance(s, ir.ArrayDecl) and s.space == "shared":
                n += int(s.size * dtypes.ALL[s.elem].bits // 8)
        return n

    def _config(self, grid, block, shared_mem_bytes: int) -> LaunchConfig:
        cfg = LaunchConfig(grid, block, shared_mem_bytes)
        cfg.validate(self.static_shared_bytes(), self.uses_collectives())
        return cfg

    def launch(self, grid, block, args: Sequence[Any], backend: Optional[str] = None, shared_mem_bytes: int = 0,
               stream=None) -> None:
        """Compiles for the arguments' element types if needed and launches; returns without waiting."""
        cfg = self._config(grid, block, shared_mem_bytes)
        sig = self._sig_of_args(args)
        k = self.typed(dict(sig))
        ck = self.compile("cuda", dict(sig))
        ctypes_ = [k.param_ctype(p) for p in self._ir.params]
        elems = [k.ptr_elem.get(p.name) if p.kind == "tensor" else None for p in self._ir.params]
        self._launcher.launch(ck, cfg, pack_args(ctypes_, args, elems), stream)

    def prepack(self, args: Sequence[Any]) -> PrepackedArgs:
        """Packs ``args`` once for repeated launches with ``launch_prepacked``; ``set(i, value)`` changes one."""
        k = self.typed(dict(self._sig_of_args(args)))
        return PrepackedArgs([k.param_ctype(p) for p in self._ir.params], args,
                             [k.ptr_elem.get(p.name) if p.kind == "tensor" else None for p in self._ir.params])

    def launch_prepacked(self, grid, block, prepacked: PrepackedArgs, dtypes: Optional[Dict[str, Any]] = None,
                         shared_mem_bytes: int = 0, stream=None) -> None:
        self._launcher.launch_prepacked(self.compile("cuda", dtypes), self._config(grid, block, shared_mem_bytes),
                                        prepacked, stream)

    def emulate(self, grid, block, args: Sequence[Any], shared_mem_bytes: int = 0, check_races: bool = False) -> None:
        """The same launch on the CPU (tensors are CPU tensors or numpy arrays, modified in place).  ``check_races``
        also looks for unordered conflicting accesses to shared and global memory and raises ``KernelRaceError``."""
        cfg = self._config(grid, block, shared_mem_bytes)
        _emulate(self.typed(dict(self._sig_of_args(args))), cfg.grid, cfg.block, list(args), shared_mem_bytes,
                 check_races)

    def profile(self, grid, block, args: Sequence[Any], shared_mem_bytes: int = 0, nbytes: int = 0, flops: int = 0,
                profiler=None):
        """Median device time of the launch (CUDA events, cold L2 between runs): ``runtime.profiler.ProfileResult``."""
        from ..runtime.profiler import KernelProfiler
        prof = profiler or KernelProfiler()
        self.launch(grid, block, args, shared_mem_bytes=shared_mem_bytes)        # compile outside the timed runs
        return prof.time(self._name, lambda: self.launch(grid, block, args, shared_mem_bytes=shared_mem_bytes),
                         nbytes, flops)

    def autotune(self, n: int, args: Sequence[Any], block_sizes: Sequence[int] = (32, 64, 128, 256, 512, 1024),
                 shared_mem_bytes: int = 0, tuner=None) -> dict:
        """Times a one-dimensional launch over ``n`` elements for each block size and returns the fastest
        (``{"best": block, "ms": ..., "all": [...]}``), like the reference's tuner
        (zse-compiler/zse_compiler/runtime/autotune.py:72-170)."""
        from ..runtime.profiler import AutoTuner
        tuner = tuner or AutoTuner()
        return tuner.tune(self._name, lambda b: (lambda: self.launch(((n + b - 1) // b,), (b,), args,
                                                                    shared_mem_bytes=shared_mem_bytes)),
                          [b for b in block_sizes if not (self.uses_collectives() and b % 32)])

    def __call__(self, *args, **kwargs):
        raise RuntimeError(f"Cannot call @kernel '{self._name}' directly. "
                           f"Use {self._name}.launch(grid=..., block=..., args=...) instead.")

    def __repr__(self) -> str:
        built = [",".join(d for _, d in s) or "-" for s in self._compiled] or ["not compiled"]
        return f"KernelFunction('{self._name}', compiled={built})"


def kernel(func: Callable) -> KernelFunction:
    """Marks a Python function as a GPU kernel::

        @kernel
        def vector_add(a: Tensor, b: Tensor, out: Tensor, n: int):
            i = global_id(0)
            if i < n:
                out[i] = a[i] + b[i]

        vector_add.launch(grid=(blocks,), block=(256,), args=(a, b, out, n))
    """
    return KernelFunction(func)


def fuse(kernels: list, name: Optional[str] = None, chain: Optional[list] = None) -> KernelFunction:
    """One kernel that runs element-wise ``kernels`` back to back without the intermediate tensors (see
    ``fusion.FusionPass``)."""
    from .fusion import FusionPass
    return KernelFunction(None, FusionPass().fuse(kernels, name=name, chain=chain))
