"""Type pass over the kernel IR (zse-compiler/zse_compiler/ir/type_inference.py:24-134).

Scalars are ``bool`` < ``int`` < ``uint`` < ``float``; fp16 / bf16 elements widen to ``float`` as soon as they take
part in arithmetic and narrow again when stored.  A local takes the widest type ever assigned to it (so ``acc = 0``
followed by ``acc += x[i]`` is a float), unless its first assignment declares one.  ``/`` is true division as in
Python, ``//`` and ``%`` follow Python's sign rules.  The element type of an un-annotated tensor parameter comes from
the ``signature`` (the argument types of a launch), ``float32`` when nothing is known."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

from . import dtypes, ir
from .errors import KernelTypeError
from .primitives import FRAGMENTS, PRIMITIVES

_RANK = {"bool": 0, "int": 1, "uint": 2, "float": 3}
_ELEM_VALUE = {"float32": "float", "float16": "half", "bfloat16": "bf16", "int32": "int", "int16": "int",
               "int8": "int", "uint32": "uint", "uint16": "uint", "uint8": "uint"}


def widen(t: str) -> str:
    return "float" if t in ("half", "bf16") else t


def promote(a: str, b: str) -> str:
    a, b = widen(a), widen(b)
    if a not in _RANK or b not in _RANK:
        raise KernelTypeError(f"cannot combine {a} and {b}")
    return a if _RANK[a] >= _RANK[b] else b


@dataclass
class TypedKernel:
    func: ir.Function
    signature: Dict[str, str]                      # tensor parameter -> element type name
    var_types: Dict[str, str] = field(default_factory=dict)
    ptr_elem: Dict[str, str] = field(default_factory=dict)     # every indexable name -> element type name
    arrays: List[ir.ArrayDecl] = field(default_factory=list)
    uses: set = field(default_factory=set)         # primitives used (the emitter prints helpers for some)

    def param_ctype(self, p: ir.Param) -> str:
        if p.kind == "tensor":
            return dtypes.ALL[self.ptr_elem[p.name]].c_name + "*"
        return {"int": "int", "float": "float", "bool": "bool"}[p.kind]


class TypeInference:
    def run(self, func: ir.Function, signature: Optional[Dict[str, str]] = None) -> TypedKernel:
        sig = {}
        for p in func.params:
            if p.kind == "tensor":
                sig[p.name] = p.elem or (signature or {}).get(p.name) or "float32"
        k = TypedKernel(func, sig)
        self.k, self.f = k, func
        self._declared: Dict[str, str] = {}
        for p in func.params:
            if p.kind == "tensor":
                k.ptr_elem[p.name] = sig[p.name]
            else:
                k.var_types[p.name] = p.kind
                self._declared[p.name] = p.kind
        for s in ir.walk_stmts(func.body):
            if isinstance(s, ir.ArrayDecl):
                self._new_ptr(s.name, s.elem, s)
                k.arrays.append(s)
            elif isinstance(s, ir.Assign) and s.declared and s.name not in self._declared:
                self._declared[s.name] = s.declared
                k.var_types[s.name] = s.declared
        for s in ir.walk_stmts(func.body):                 # pointer casts may refer to arrays declared anywhere above
            if isinstance(s, ir.PtrCast):
                if s.source not in k.ptr_elem:
                    raise self._err(s, f"'{s.source}' is not a tensor or array")
                self._new_ptr(s.name, s.elem, s)
        for _ in range(6):                                 # widen locals until nothing changes
            before = dict(k.var_types)
            self._block(func.body)
            if before == k.var_types:
                break
        else:
            raise KernelTypeError(f"the types of the locals of '{func.name}' do not settle")
        return k

    # ---- helpers ------------------------------------------------------------------------------------------------
    def _err(self, node, msg: str) -> KernelTypeError:
        ln = getattr(node, "lineno", 0) or None
        return KernelTypeError(msg, self.f.filename, ln, self.f.line_text(ln) if ln else None)

    def _new_ptr(self, name: str, elem: str, node) -> None:
        if name in self.k.var_types or (name in self.k.ptr_elem and self.k.ptr_elem[name] != elem):
            raise self._err(node, f"'{name}' is already in use")
        self.k.ptr_elem[name] = elem

    def _elem_value(self, base: str, node) -> str:
        elem = self.k.ptr_elem.get(base)
        if elem is None:
            raise self._err(node, f"'{base}' is not a tensor or array")
        if elem not in _ELEM_VALUE:
            raise self._err(node, f"'{base}' holds packed {elem} values: reinterpret it as uint8 or uint32 and unpack")
        return _ELEM_VALUE[elem]

    def _set_var(self, name: str, t: str, node) -> None:
        if name in self.k.ptr_elem:
            raise self._err(node, f"'{name}' names a tensor or array and cannot be assigned")
        if t in ("float4", "half2", "void") + FRAGMENTS:
            if t == "void":
                raise self._err(node, "this call gives no value")
            old = self.k.var_types.get(name)
            if old not in (None, t):
                raise self._err(node, f"'{name}' is a {old} elsewhere")
            self.k.var_types[name] = t
            return
        if name in self._declared:
            return
        old = self.k.var_types.get(name)
        if old in ("float4", "half2") + FRAGMENTS:
            raise self._err(node, f"'{name}' is a {old} elsewhere")
        self.k.var_types[name] = widen(t) if old is None else promote(old, t)

    # ---- statements -------------------------------------------------------------------------------------------
    def _block(self, body) -> None:
        for s in body:
            if isinstance(s, ir.Assign):
                self._set_var(s.name, self._expr(s.value), s)
            elif isinstance(s, ir.Store):
                self._elem_value(s.base, s)
                self._scalar(s.index, "an index", integer=True)
                self._scalar(s.value, "a stored value")
            elif isinstance(s, ir.ExprStmt):
                self._expr(s.call)
            elif isinstance(s, ir.If):
                self._scalar(s.cond, "a condition")
                self._block(s.then)
                self._block(s.orelse)
            elif isinstance(s, ir.For):
                for e in (s.start, s.stop, s.step):
                    self._scalar(e, "a loop bound", integer=True)
                self.k.var_types.setdefault(s.var, "int")
                self._block(s.body)
            elif isinstance(s, ir.While):
                self._scalar(s.cond, "a condition")
                self._block(s.body)

    def _scalar(self, e: ir.Expr, what: str, integer: bool = False) -> str:
        t = self._expr(e)
        if widen(t) not in _RANK:
            raise self._err(e, f"{what} cannot be a {t}")
        if integer and widen(t) == "float":
            raise self._err(e, f"{what} must be an integer")
        return t

    # ---- expressions ----------------------------------------------------------------------------------------------
    def _expr(self, e: ir.Expr) -> str:
        e.type = self._expr_type(e)
        return e.type

    def _expr_type(self, e: ir.Expr) -> str:
        if isinstance(e, ir.Const):
            return "bool" if isinstance(e.value, bool) else "int" if isinstance(e.value, int) else "float"
        if isinstance(e, ir.Var):
            if e.name in self.k.ptr_elem:
                return "ptr:" + self.k.ptr_elem[e.name]
            t = self.k.var_types.get(e.name)
            if t is None:
                raise self._err(e, f"'{e.name}' is read before it is assigned")
            return t
        if isinstance(e, ir.Load):
            self._scalar(e.index, "an index", integer=True)
            return self._elem_value(e.base, e)
        if isinstance(e, ir.Field):
            t = self._expr(e.value)
            if t not in ("float4", "half2") or not 0 <= e.index < (4 if t == "float4" else 2):
                raise self._err(e, f"component {e.index} of a {t} does not exist")
            return "float"
        if isinstance(e, ir.BinOp):
            a, b = self._scalar(e.left, "an operand"), self._scalar(e.right, "an operand")
            if e.op in ("&", "|", "^", "<<", ">>"):
                if widen(a) == "float" or widen(b) == "float":
                    raise self._err(e, f"'{e.op}' needs integers")
                return "int" if promote(a, b) == "bool" else promote(a, b)
            if e.op in ("/", "**"):
                return "float"
            t = promote(a, b)
            return "int" if t == "bool" else t
        if isinstance(e, ir.UnaryOp):
            t = self._scalar(e.operand, "an operand")
            if e.op == "not":
                return "bool"
            if e.op == "~" and widen(t) == "float":
                raise self._err(e, "'~' needs an integer")
            return "int" if widen(t) == "bool" else widen(t)
        if isinstance(e, ir.Compare):
            self._scalar(e.left, "an operand")
            self._scalar(e.right, "an operand")
            return "bool"
        if isinstance(e, ir.BoolOp):
            for v in e.values:
                self._scalar(v, "an operand")
            return "bool"
        if isinstance(e, ir.Ternary):
            self._scalar(e.cond, "a condition")
            return promote(self._scalar(e.then, "a value"), self._scalar(e.other, "a value"))
        if isinstance(e, ir.Cast):
            self._scalar(e.value, "a converted value")
            return e.to
        if isinstance(e, ir.Call):
            return self._call(e)
        raise self._err(e, f"unknown expression {type(e).__name__}")

    def _ptr_arg(self, e: ir.Expr, what: str) -> str:
        if not isinstance(e, ir.Var) or e.name not in self.k.ptr_elem:
            raise self._err(e, f"{what} must be a tensor or array")
        e.type = "ptr:" + self.k.ptr_elem[e.name]
        return self.k.ptr_elem[e.name]

    def _call(self, e: ir.Call) -> str:
        name, args = e.func, e.args
        self.k.uses.add(name)
        if name == "abs":
            return widen(self._scalar(args[0], "an argument"))
        rule = PRIMITIVES[name][2]
        if name.startswith("atomic_"):
            target = args[0]
            vt = self._expr(target)
            elem = self.k.ptr_elem[target.base]
            if elem not in ("float32", "int32", "uint32") or (name != "atomic_add" and elem == "float32"):
                raise self._err(e, f"{name} works on int32 / uint32 elements" +
                                (" and float32" if name == "atomic_add" else "") + f", not {elem}")
            for a in args[1:]:
                self._scalar(a, "an argument")
            return vt
        if name in ("wmma_load_a", "wmma_load_b", "wmma_store"):
            want = "float32" if name == "wmma_store" else "float16"
            if self._ptr_arg(args[0], "the first argument") != want:
                raise self._err(e, f"{name} works on a {want} tensor or array")
            for a in args[1:4]:
                self._scalar(a, "a tile coordinate", integer=True)
            if name == "wmma_store" and self._expr(args[4]) != "frag_c":
                raise self._err(e, "wmma_store writes an accumulator fragment (from wmma_fill / wmma_mma)")
            return rule
        if name == "wmma_fill":
            for a in args:
                self._scalar(a, "the fill value")
            return rule
        if name == "wmma_mma":
            got = tuple(self._expr(a) for a in args)
            if not all(isinstance(a, ir.Var) for a in args):
                raise self._err(e, "wmma_mma(a, b, c) takes named fragments")
            if got != FRAGMENTS:
                raise self._err(e, f"wmma_mma(a, b, c) takes an A, a B and an accumulator fragment, got {got}")
            return rule
        if name in ("load_float4", "store_float4"):
            if self._ptr_arg(args[0], "the first argument") != "float32":
                raise self._err(e, f"{name} needs a float32 tensor")
        elif name in ("load_half2", "store_half2"):
            if self._ptr_arg(args[0], "the first argument") != "float16":
                raise self._err(e, f"{name} needs a float16 tensor")
        elif name in ("unpack_int4", "unpack_uint4"):
            self._scalar(args[0], "the packed word", integer=True)
            if self._ptr_arg(args[1], "the output") not in ("int32", "uint32", "float32"):
                raise self._err(e, f"{name} writes to an int32, uint32 or float32 array")
            self._scalar(args[2], "the base index", integer=True)
            return "void"
        elif name in ("tile_load", "tile_store"):
            t_i, s_i = (0, 4) if name == "tile_load" else (1, 0)
            te, se = self._ptr_arg(args[t_i], "the tensor"), self._ptr_arg(args[s_i], "the shared tile")
            if te not in _ELEM_VALUE or se not in _ELEM_VALUE:
                raise self._err(e, f"{name} does not move packed types")
            for i, a in enumerate(args):
                if i not in (t_i, s_i):
                    self._scalar(a, "a tile coordinate", integer=True)
            tile = args[3] if name == "tile_load" else args[4]
            if not (isinstance(tile, ir.Const) and isinstance(tile.value, int) and tile.value > 0):
                raise self._err(e, f"{name}: tile_size is a positive integer constant")
            ld = args[7]
            if isinstance(ld, ir.Const) and ld.value == -1 and isinstance(args[6], ir.Const) and args[6].value == -1:
                raise self._err(e, f"{name} needs the row pitch of the matrix: pass ld= or bound_col=")
            return "void"
        types = []
        for i, a in enumerate(args):
            if name in ("load_float4", "store_float4", "load_half2", "store_half2") and i == 0:
                continue
            types.append(self._scalar(a, "an argument"))
        if rule == "arg0":
            t = widen(types[0])
            return "int" if t == "bool" and not name.startswith("warp_shuffle") else t
        if rule == "promote":
            t = types[0]
            for u in types[1:]:
                t = promote(t, u)
            return t
        return rule


def infer(func: ir.Function, signature: Optional[Dict[str, str]] = None) -> TypedKernel:
    return TypeInference().run(func, signature)
