"""Typed kernel IR -> CUDA C for sm_100a (the CUDA emitter of the reference is zse-compiler/zse_compiler/codegen/
base.py:36-473 and cuda.py:40-488; its ROCm and Metal emitters have no counterpart: this package has one target).

The text is one ``extern "C" __global__`` function plus the few helpers it uses.  Warp collectives use the full mask,
so a kernel that uses them (or a block reduction, which is built on them) must run with a block size that is a
multiple of 32; ``launcher.LaunchConfig`` checks that.  With ``line_info`` every statement is preceded by a ``#line``
directive naming the Python file and line, so nvcc's messages and profilers' source views point at the kernel's
Python source."""
from __future__ import annotations

import math
from typing import Dict, List

from . import dtypes, ir
from .infer import TypedKernel, widen

_C_SCALAR = {"int": "int", "uint": "unsigned int", "float": "float", "bool": "bool", "half": "__half",
             "bf16": "__nv_bfloat16", "float4": "float4", "half2": "__half2",
             "frag_a": "nvcuda::wmma::fragment<nvcuda::wmma::matrix_a, 16, 16, 16, __half, nvcuda::wmma::row_major>",
             "frag_b": "nvcuda::wmma::fragment<nvcuda::wmma::matrix_b, 16, 16, 16, __half, nvcuda::wmma::row_major>",
             "frag_c": "nvcuda::wmma::fragment<nvcuda::wmma::accumulator, 16, 16, 16, float>"}
_AXIS = "xyz"
_MATH1 = {"exp": "expf", "log": "logf", "sqrt": "sqrtf", "rsqrt": "rsqrtf", "cos": "cosf", "sin": "sinf",
          "tanh": "tanhf"}
_RED_OP = {"sum": "a + b", "max": "a > b ? a : b", "min": "a < b ? a : b"}
_RED_ID = {("sum", "float"): "0.0f", ("sum", "int"): "0", ("sum", "uint"): "0u",
           ("max", "float"): "-INFINITY", ("max", "int"): "INT_MIN", ("max", "uint"): "0u",
           ("min", "float"): "INFINITY", ("min", "int"): "INT_MAX", ("min", "uint"): "UINT_MAX"}

PRELUDE = """#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <climits>
#include <cmath>

__device__ __forceinline__ int zse_tid() {
  return (int)(threadIdx.x + blockDim.x * (threadIdx.y + blockDim.y * threadIdx.z));
}
__device__ __forceinline__ int zse_nthreads() { return (int)(blockDim.x * blockDim.y * blockDim.z); }
"""

_HELPERS = {
    "floordiv": """__device__ __forceinline__ int zse_floordiv(int a, int b) {
  int q = a / b;
  return ((a % b != 0) && ((a < 0) != (b < 0))) ? q - 1 : q;
}
""",
    "mod": """__device__ __forceinline__ int zse_mod(int a, int b) {
  int r = a % b;
  return (r != 0 && ((r < 0) != (b < 0))) ? r + b : r;
}
""",
    "fmod": """__device__ __forceinline__ float zse_fmod(float a, float b) {
  float r = fmodf(a, b);
  return (r != 0.0f && ((r < 0.0f) != (b < 0.0f))) ? r + b : r;
}
""",
}


def _warp_helper(op: str, t: str) -> str:
    c = _C_SCALAR[t]
    return (f"__device__ __forceinline__ {c} zse_warp_{op}_{t}({c} a) {{\n"
            f"#pragma unroll\n  for (int o = 16; o > 0; o >>= 1) {{\n"
            f"    {c} b = __shfl_xor_sync(0xffffffffu, a, o);\n    a = {_RED_OP[op]};\n  }}\n  return a;\n}}\n")


def _block_helper(op: str, t: str) -> str:
    c, ident = _C_SCALAR[t], _RED_ID[(op, t)]
    return (f"__device__ __forceinline__ {c} zse_block_{op}_{t}({c} a) {{\n"
            f"  __shared__ {c} part[32];\n  __shared__ {c} total;\n"
            f"  const int tid = zse_tid(), lane = tid & 31, warp = tid >> 5, nw = (zse_nthreads() + 31) >> 5;\n"
            f"  a = zse_warp_{op}_{t}(a);\n"
            f"  __syncthreads();            // an earlier reduction may still be reading part[] / total\n"
            f"  if (lane == 0) part[warp] = a;\n  __syncthreads();\n"
            f"  if (warp == 0) {{\n    a = lane < nw ? part[lane] : ({c})({ident});\n"
            f"    a = zse_warp_{op}_{t}(a);\n    if (lane == 0) total = a;\n  }}\n"
            f"  __syncthreads();\n  return total;\n}}\n")


def _float_lit(v: float) -> str:
    if math.isnan(v):
        return "NAN"
    if math.isinf(v):
        return "INFINITY" if v > 0 else "-INFINITY"
    s = repr(float(v))
    if "e" in s or "E" in s:
        mant, exp = s.lower().split("e")
        if "." not in mant:
            mant += ".0"
        return f"{mant}e{exp}f"
    return s + "f"


class CudaEmitter:
    def __init__(self, line_info: bool = False):
        self.line_info = line_info

    # ---- entry ------------------------------------------------------------------------------------------------
    def generate(self, k: TypedKernel) -> str:
        self.k = k
        self._helpers: Dict[str, str] = {}
        self._tmp = 0
        f = k.func
        body = self._block(f.body, 1)
        decls: List[str] = []
        for a in k.arrays:
            c = dtypes.ALL[a.elem].c_name
            if a.space == "shared":
                decls.append(f"  __shared__ {c} {a.name}[{a.size}];")
            elif a.space == "local":
                decls.append(f"  {c} {a.name}[{a.size}];")
            else:
                decls.append("  extern __shared__ __align__(16) unsigned char zse_dyn_smem[];")
                decls.append(f"  {c}* {a.name} = reinterpret_cast<{c}*>(zse_dyn_smem);")
        params = {p.name for p in f.params}
        for name, t in sorted(k.var_types.items()):
            if name not in params:
                decls.append(f"  {_C_SCALAR[t]} {name};")
        sig = ", ".join(f"{k.param_ctype(p)} {p.name}" for p in f.params)
        out = [PRELUDE] + list(self._helpers.values())
        out.append(f'extern "C" __global__ void {f.name}({sig}) {{')
        out += decls
        out += body
        out.append("}")
        return "\n".join(out) + "\n"

    def _need(self, key: str, text: str) -> None:
        self._helpers.setdefault(key, text)

    # ---- statements -------------------------------------------------------------------------------------------
    def _block(self, body, depth: int) -> List[str]:
        out: List[str] = []
        for s in body:
            if self.line_info and s.lineno:
                out.append(f'#line {s.lineno} "{self.k.func.filename}"')
            out += self._stmt(s, depth)
        return out

    def _stmt(self, s: ir.Stmt, d: int) -> List[str]:
        pad = "  " * d
        if isinstance(s, ir.Assign):
            t = self.k.var_types[s.name]
            if t.startswith("frag_"):
                return self._wmma_assign(s, pad)
            return [f"{pad}{s.name} = {self._as(s.value, t)};"]
        if isinstance(s, ir.Store):
            elem = self.k.ptr_elem[s.base]
            return [f"{pad}{s.base}[{self._val(s.index)}] = {self._to_elem(s.value, elem)};"]
        if isinstance(s, (ir.ArrayDecl,)):
            return []
        if isinstance(s, ir.PtrCast):
            c = dtypes.ALL[s.elem].c_name
            return [f"{pad}{c}* {s.name} = reinterpret_cast<{c}*>({s.source});"]
        if isinstance(s, ir.ExprStmt):
            return self._call_stmt(s.call, d)
        if isinstance(s, ir.If):
            out = [f"{pad}if ({self._val(s.cond)}) {{"] + self._block(s.then, d + 1)
            if s.orelse:
                out += [f"{pad}}} else {{"] + self._block(s.orelse, d + 1)
            return out + [f"{pad}}}"]
        if isinstance(s, ir.For):
            self._tmp += 1
            n = self._tmp
            stop, step = f"zse_stop{n}", f"zse_step{n}"
            if isinstance(s.step, ir.Const):
                cond = f"{s.var} < {stop}" if s.step.value > 0 else f"{s.var} > {stop}"
            else:
                cond = f"({step} > 0 ? {s.var} < {stop} : {s.var} > {stop})"
            return ([f"{pad}{{", f"{pad}  const int {stop} = {self._as(s.stop, 'int')};",
                     f"{pad}  const int {step} = {self._as(s.step, 'int')};",
                     f"{pad}  for ({s.var} = {self._as(s.start, 'int')}; {cond}; {s.var} += {step}) {{"]
                    + self._block(s.body, d + 2) + [f"{pad}  }}", f"{pad}}}"])
        if isinstance(s, ir.While):
            return [f"{pad}while ({self._val(s.cond)}) {{"] + self._block(s.body, d + 1) + [f"{pad}}}"]
        if isinstance(s, ir.Return):
            return [f"{pad}return;"]
        if isinstance(s, ir.Break):
            return [f"{pad}break;"]
        if isinstance(s, ir.Continue):
            return [f"{pad}continue;"]
        raise NotImplementedError(type(s).__name__)

    # ---- values -----------------------------------------------------------------------------------------------
    def _val(self, e: ir.Expr) -> str:
        """C text of ``e`` with fp16 / bf16 widened to float."""
        raw = self._raw(e)
        if e.type == "half":
            return f"__half2float({raw})"
        if e.type == "bf16":
            return f"__bfloat162float({raw})"
        return raw

    def _as(self, e: ir.Expr, t: str) -> str:
        """``e`` converted to scalar type ``t``."""
        if t in ("float4", "half2"):
            return self._raw(e)
        if t == "half":
            return self._raw(e) if e.type == "half" else f"__float2half((float)({self._val(e)}))"
        if t == "bf16":
            return self._raw(e) if e.type == "bf16" else f"__float2bfloat16((float)({self._val(e)}))"
        v = self._val(e)
        if widen(e.type) == t:
            return v
        if t == "bool":
            return f"(({v}) != 0)"
        return f"({_C_SCALAR[t]})({v})"

    def _to_elem(self, e: ir.Expr, elem: str) -> str:
        if elem == "float16":
            return self._as(e, "half")
        if elem == "bfloat16":
            return self._as(e, "bf16")
        if elem == "float32":
            return self._as(e, "float")
        return f"({dtypes.ALL[elem].c_name})({self._val(e)})"

    def _raw(self, e: ir.Expr) -> str:
        if isinstance(e, ir.Const):
            if isinstance(e.value, bool):
                return "true" if e.value else "false"
            if isinstance(e.value, int):
                return str(e.value) if -2**31 <= e.value < 2**31 else f"{e.value}u"
            return _float_lit(e.value)
        if isinstance(e, ir.Var):
            return e.name
        if isinstance(e, ir.Load):
            return f"{e.base}[{self._val(e.index)}]"
        if isinstance(e, ir.Field):
            v = self._raw(e.value)
            if e.value.type == "float4":
                return f"({v}).{'xyzw'[e.index]}"
            return f"{'__low2float' if e.index == 0 else '__high2float'}({v})"
        if isinstance(e, ir.BinOp):
            return self._binop(e)
        if isinstance(e, ir.UnaryOp):
            v = self._val(e.operand)
            if e.op == "not":
                return f"(!({v}))"
            if widen(e.operand.type) == "bool":
                v = f"(int)({v})"
            return f"({e.op}({v}))"
        if isinstance(e, ir.Compare):
            return f"({self._val(e.left)} {e.op} {self._val(e.right)})"
        if isinstance(e, ir.BoolOp):
            op = " && " if e.op == "and" else " || "
            return "(" + op.join(self._as(v, "bool") for v in e.values) + ")"
        if isinstance(e, ir.Ternary):
            return f"({self._as(e.cond, 'bool')} ? {self._as(e.then, e.type)} : {self._as(e.other, e.type)})"
        if isinstance(e, ir.Cast):
            return self._as(e.value, e.to) if widen(e.value.type) != e.to else self._val(e.value)
        if isinstance(e, ir.Call):
            return self._call(e)
        raise NotImplementedError(type(e).__name__)

    def _binop(self, e: ir.BinOp) -> str:
        t = e.type
        if e.op == "/":
            return f"({self._as(e.left, 'float')} / {self._as(e.right, 'float')})"
        if e.op == "**":
            return f"powf({self._as(e.left, 'float')}, {self._as(e.right, 'float')})"
        a, b = self._as(e.left, t), self._as(e.right, t)
        if e.op == "//":
            if t == "float":
                return f"floorf({a} / {b})"
            if t == "uint":
                return f"({a} / {b})"
            self._need("floordiv", _HELPERS["floordiv"])
            return f"zse_floordiv({a}, {b})"
        if e.op == "%":
            if t == "float":
                self._need("fmod", _HELPERS["fmod"])
                return f"zse_fmod({a}, {b})"
            if t == "uint":
                return f"({a} % {b})"
            self._need("mod", _HELPERS["mod"])
            return f"zse_mod({a}, {b})"
        return f"({a} {e.op} {b})"

    def _reduce(self, scope: str, op: str, e: ir.Call) -> str:
        t = e.type
        self._need(f"warp_{op}_{t}", _warp_helper(op, t))
        if scope == "block":
            self._need(f"block_{op}_{t}", _block_helper(op, t))
        return f"zse_{scope}_{op}_{t}({self._as(e.args[0], t)})"

    def _call(self, e: ir.Call) -> str:
        n, a = e.func, e.args
        if n in ("thread_id", "block_id", "block_dim", "grid_dim"):
            reg = {"thread_id": "threadIdx", "block_id": "blockIdx", "block_dim": "blockDim", "grid_dim": "gridDim"}[n]
            return f"(int){reg}.{_AXIS[a[0].value]}"
        if n == "global_id":
            x = _AXIS[a[0].value]
            return f"(int)(blockIdx.{x} * blockDim.{x} + threadIdx.{x})"
        if n == "lane_id":
            return "(zse_tid() & 31)"
        if n == "warp_id":
            return "(zse_tid() >> 5)"
        if n == "syncthreads":
            return "__syncthreads()"
        if n.startswith("atomic_"):
            tgt = a[0]
            elem = self.k.ptr_elem[tgt.base]
            c = dtypes.ALL[elem].c_name
            addr = f"&{tgt.base}[{self._val(tgt.index)}]"
            fn = {"atomic_add": "atomicAdd", "atomic_max": "atomicMax", "atomic_min": "atomicMin",
                  "atomic_cas": "atomicCAS"}[n]
            rest = ", ".join(f"({c})({self._val(x)})" for x in a[1:])
            return f"{fn}({addr}, {rest})"
        if n in _MATH1:
            return f"{_MATH1[n]}({self._as(a[0], 'float')})"
        if n == "pow":
            return f"powf({self._as(a[0], 'float')}, {self._as(a[1], 'float')})"
        if n == "fma":
            return "fmaf(" + ", ".join(self._as(x, "float") for x in a) + ")"
        if n in ("max_val", "min_val"):
            t = e.type
            fn = ("fmaxf" if n == "max_val" else "fminf") if t == "float" else ("max" if n == "max_val" else "min")
            return f"{fn}({self._as(a[0], t)}, {self._as(a[1], t)})"
        if n == "abs":
            return f"fabsf({self._val(a[0])})" if e.type == "float" else f"abs({self._as(a[0], 'int')})"
        if n in ("half_to_float", "bf16_to_float"):
            return self._as(a[0], "float")
        if n == "float_to_half":
            return self._as(a[0], "half")
        if n == "float_to_bf16":
            return self._as(a[0], "bf16")
        if n.startswith("warp_shuffle"):
            fn = {"warp_shuffle_down": "__shfl_down_sync", "warp_shuffle_up": "__shfl_up_sync",
                  "warp_shuffle_xor": "__shfl_xor_sync", "warp_shuffle": "__shfl_sync"}[n]
            t = "int" if e.type == "bool" else e.type
            width = f", {self._as(a[2], 'int')}" if len(a) > 2 else ""
            v = f"{fn}(0xffffffffu, {self._as(a[0], t)}, {self._as(a[1], 'int')}{width})"
            return f"(({v}) != 0)" if e.type == "bool" else v
        if n == "warp_ballot":
            return f"__ballot_sync(0xffffffffu, {self._as(a[0], 'bool')})"
        if n in ("warp_all", "warp_any"):
            return f"(__{n[5:]}_sync(0xffffffffu, {self._as(a[0], 'bool')}) != 0)"
        if n.startswith("warp_reduce_") or n.startswith("block_reduce_"):
            scope, _, op = n.split("_")
            return self._reduce(scope, op, e)
        if n == "load_float4":
            return f"reinterpret_cast<const float4*>({a[0].name})[{self._val(a[1])}]"
        if n == "load_half2":
            return f"reinterpret_cast<const __half2*>({a[0].name})[{self._val(a[1])}]"
        raise NotImplementedError(f"{n} cannot be used as a value")

    def _wmma_assign(self, s: ir.Assign, pad: str) -> List[str]:
        self._need("wmma", "#include <mma.h>\n")
        v = s.value
        if isinstance(v, ir.Var):
            return [f"{pad}{s.name} = {v.name};"]
        n, a = v.func, v.args
        if n in ("wmma_load_a", "wmma_load_b"):
            ld = self._as(a[3], "int")
            return [f"{pad}nvcuda::wmma::load_matrix_sync({s.name}, {a[0].name} + (long long)({self._as(a[1], 'int')}) * "
                    f"({ld}) + ({self._as(a[2], 'int')}), {ld});"]
        if n == "wmma_fill":
            val = self._as(a[0], "float") if a else "0.0f"
            return [f"{pad}nvcuda::wmma::fill_fragment({s.name}, {val});"]
        return [f"{pad}nvcuda::wmma::mma_sync({s.name}, {a[0].name}, {a[1].name}, {a[2].name});"]

    def _call_stmt(self, e: ir.Call, d: int) -> List[str]:
        pad, n, a = "  " * d, e.func, e.args
        if n == "wmma_store":
            self._need("wmma", "#include <mma.h>\n")
            ld = self._as(a[3], "int")
            return [f"{pad}nvcuda::wmma::store_matrix_sync({a[0].name} + (long long)({self._as(a[1], 'int')}) * ({ld}) + "
                    f"({self._as(a[2], 'int')}), {a[4].name}, {ld}, nvcuda::wmma::mem_row_major);"]
        if n == "store_float4":
            vals = ", ".join(self._as(x, "float") for x in a[2:])
            return [f"{pad}reinterpret_cast<float4*>({a[0].name})[{self._val(a[1])}] = make_float4({vals});"]
        if n == "store_half2":
            return [f"{pad}reinterpret_cast<__half2*>({a[0].name})[{self._val(a[1])}] = "
                    f"__floats2half2_rn({self._as(a[2], 'float')}, {self._as(a[3], 'float')});"]
        if n in ("unpack_int4", "unpack_uint4"):
            c = dtypes.ALL[self.k.ptr_elem[a[1].name]].c_name
            nib = ("((int)(zse_p << (28 - 4 * zse_j))) >> 28" if n == "unpack_int4"
                   else "(zse_p >> (4 * zse_j)) & 0xFu")
            return [f"{pad}{{", f"{pad}  const unsigned int zse_p = (unsigned int)({self._val(a[0])});",
                    f"{pad}  const int zse_b = {self._as(a[2], 'int')};", f"#pragma unroll",
                    f"{pad}  for (int zse_j = 0; zse_j < 8; ++zse_j) {a[1].name}[zse_b + zse_j] = ({c})({nib});",
                    f"{pad}}}"]
        if n in ("tile_load", "tile_store"):
            return self._tile(e, d)
        return [f"{pad}{self._call(e)};"]

    def _tile(self, e: ir.Call, d: int) -> List[str]:
        pad, a = "  " * d, e.args
        load = e.func == "tile_load"
        tensor, smem = (a[0].name, a[4].name) if load else (a[1].name, a[0].name)
        trow, tcol, tsz = (a[1], a[2], a[3]) if load else (a[2], a[3], a[4])
        brow, bcol, ld = a[5], a[6], a[7]
        te, se = self.k.ptr_elem[tensor], self.k.ptr_elem[smem]

        def conv(src: str, src_elem: str, dst_elem: str) -> str:
            if src_elem == dst_elem:
                return src
            if src_elem == "float16":
                src = f"__half2float({src})"
            elif src_elem == "bfloat16":
                src = f"__bfloat162float({src})"
            if dst_elem == "float16":
                return f"__float2half((float)({src}))"
            if dst_elem == "bfloat16":
                return f"__float2bfloat16((float)({src}))"
            return f"({dtypes.ALL[dst_elem].c_name})({src})"

        zero = conv("0.0f", "float32", se)
        lines = [f"{pad}{{", f"{pad}  const int zse_t = {tsz.value};",
                 f"{pad}  const int zse_r0 = {self._as(trow, 'int')} * zse_t, zse_c0 = {self._as(tcol, 'int')} * zse_t;",
                 f"{pad}  const int zse_br = {self._as(brow, 'int')}, zse_bc = {self._as(bcol, 'int')};",
                 f"{pad}  const int zse_ldv = {self._as(ld, 'int')}, zse_ld = zse_ldv >= 0 ? zse_ldv : zse_bc;"]
        if not load:
            lines.append(f"{pad}  __syncthreads();          // the whole tile is written before anyone copies it out")
        lines += [f"{pad}  for (int zse_e = zse_tid(); zse_e < zse_t * zse_t; zse_e += zse_nthreads()) {{",
                  f"{pad}    const int zse_r = zse_r0 + zse_e / zse_t, zse_c = zse_c0 + zse_e % zse_t;",
                  f"{pad}    const bool zse_ok = (zse_br < 0 || zse_r < zse_br) && (zse_bc < 0 || zse_c < zse_bc);"]
        g = f"{tensor}[(long long)zse_r * zse_ld + zse_c]"
        if load:
            lines.append(f"{pad}    {smem}[zse_e] = zse_ok ? {conv(g, te, se)} : {zero};")
        else:
            lines.append(f"{pad}    if (zse_ok) {g} = {conv(f'{smem}[zse_e]', se, te)};")
        lines.append(f"{pad}  }}")
        if load:
            lines.append(f"{pad}  __syncthreads();")
        lines.append(f"{pad}}}")
        return lines


def generate_cuda(k: TypedKernel, line_info: bool = False) -> str:
    return CudaEmitter(line_info).generate(k)


class BaseCodegen:
    """The reference's generator object (zse-compiler/zse_compiler/codegen/base.py:36-60): ``generate(kernel)`` returns
    the source text.  ``kernel`` is a typed kernel, or a ``@kernel`` function (typed with its default element types).
    There is one target here, so the base class already produces CUDA."""
    backend = "cuda"

    def __init__(self, line_info: bool = False):
        self.line_info = line_info

    def generate(self, kernel) -> str:
        typed = kernel.typed(None) if hasattr(kernel, "typed") else kernel
        return generate_cuda(typed, self.line_info)


class CUDACodegen(BaseCodegen):
    """CUDA C for sm_100a (zse-compiler/zse_compiler/codegen/cuda.py:40-488 is the reference's generator)."""

