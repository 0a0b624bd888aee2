"""Python function -> kernel IR (zse-compiler/zse_compiler/ast_parser/parser.py:53-728, validator.py:60-125).

The kernel language is a subset of Python: assignments (plain, annotated, augmented), ``if`` / ``for ... in range`` /
``while`` / ``break`` / ``continue`` / bare ``return``, arithmetic, comparisons, ``and`` / ``or`` / ``not``, the
conditional expression, indexing of tensors and arrays, and calls of the primitives.  Module-level numbers that the
function refers to (``BLOCK = 256``) are folded in as constants.  Everything else is refused with the source line."""
from __future__ import annotations

import ast
import inspect
import textwrap
from typing import Callable, Dict, List, Optional, Set

from . import dtypes, ir
from .errors import KernelSyntaxError
from .primitives import BUILTINS, DECLARATIONS, PRIMITIVES

_FORBIDDEN = {
    ast.FunctionDef: "nested functions", ast.AsyncFunctionDef: "async functions", ast.ClassDef: "classes",
    ast.Import: "imports", ast.ImportFrom: "imports", ast.Try: "try/except", ast.With: "with blocks",
    ast.AsyncWith: "with blocks", ast.Yield: "yield", ast.YieldFrom: "yield", ast.Await: "await",
    ast.ListComp: "comprehensions", ast.SetComp: "comprehensions", ast.DictComp: "comprehensions",
    ast.GeneratorExp: "comprehensions", ast.JoinedStr: "f-strings", ast.Global: "global", ast.Nonlocal: "nonlocal",
    ast.Lambda: "lambda", ast.Raise: "raise", ast.Delete: "del", ast.Starred: "star arguments",
}
_BINOPS = {ast.Add: "+", ast.Sub: "-", ast.Mult: "*", ast.Div: "/", ast.FloorDiv: "//", ast.Mod: "%",
           ast.BitAnd: "&", ast.BitOr: "|", ast.BitXor: "^", ast.LShift: "<<", ast.RShift: ">>", ast.Pow: "**"}
_CMPOPS = {ast.Lt: "<", ast.LtE: "<=", ast.Gt: ">", ast.GtE: ">=", ast.Eq: "==", ast.NotEq: "!="}
_FIELDS = {"x": 0, "y": 1, "z": 2, "w": 3}


def _source_of(func: Callable):
    try:
        lines, first = inspect.getsourcelines(func)
    except (OSError, TypeError) as exc:
        raise KernelSyntaxError(f"the source of {getattr(func, '__name__', func)!r} is not available: {exc}") from None
    text = textwrap.dedent("".join(lines))
    filename = inspect.getsourcefile(func) or "<kernel>"
    return text, [l.rstrip("\n") for l in lines], first, filename


def _function_def(tree: ast.Module) -> ast.FunctionDef:
    for node in tree.body:
        if isinstance(node, ast.FunctionDef):
            return node
    raise KernelSyntaxError("no function definition found")


def validate_kernel(func: Callable) -> List[str]:
    """Raises for constructs the language does not have; returns warnings (calls of unknown functions)."""
    text, lines, first, filename = _source_of(func)
    fdef = _function_def(ast.parse(text))
    warnings: List[str] = []

    def fail(node, what):
        ln = first + node.lineno - 1
        raise KernelSyntaxError(f"{what} are not part of the kernel language", filename, ln, lines[node.lineno - 1])

    for node in ast.walk(fdef):
        if node is fdef:
            continue
        for bad, what in _FORBIDDEN.items():
            if isinstance(node, bad):
                fail(node, what)
        if isinstance(node, ast.Call):
            name = _call_name(node.func)
            if name is None or (name not in PRIMITIVES and name not in DECLARATIONS and name not in BUILTINS
                                and name != "range"):
                warnings.append(f"line {first + node.lineno - 1}: call of unknown function "
                                f"{name or ast.dump(node.func)}")
    if fdef.args.vararg or fdef.args.kwarg or fdef.args.kwonlyargs or fdef.args.defaults:
        fail(fdef, "variadic, keyword-only and default arguments")
    return warnings


def _call_name(node: ast.expr) -> Optional[str]:
    if isinstance(node, ast.Name):
        return node.id
    if isinstance(node, ast.Attribute):
        return node.attr
    return None


class KernelParser:
    def parse(self, func: Callable) -> ir.Function:
        text, lines, first, filename = _source_of(func)
        fdef = _function_def(ast.parse(text))
        self._lines, self._first, self._filename = lines, first, filename
        self._globals: Dict[str, object] = dict(getattr(func, "__globals__", {}))
        if getattr(func, "__closure__", None):
            for name, cell in zip(func.__code__.co_freevars, func.__closure__):
                try:
                    self._globals[name] = cell.cell_contents
                except ValueError:
                    pass
        params = [self._param(a) for a in fdef.args.args]
        self._locals: Set[str] = {p.name for p in params}
        for node in ast.walk(fdef):
            if isinstance(node, ast.Name) and isinstance(node.ctx, ast.Store):
                self._locals.add(node.id)
        # locals that hold a float4 / half2: ``v[1]`` on them selects a component rather than loading from memory
        self._vectors: Set[str] = set()
        for node in ast.walk(fdef):
            if (isinstance(node, ast.Assign) and len(node.targets) == 1 and isinstance(node.targets[0], ast.Name)
                    and isinstance(node.value, ast.Call) and _call_name(node.value.func) in ("load_float4", "load_half2")):
                self._vectors.add(node.targets[0].id)
        body = self._block(fdef.body)
        return ir.Function(fdef.name, params, body, filename, first, lines)

    # ---- helpers ------------------------------------------------------------------------------------------------
    def _err(self, node, message: str) -> KernelSyntaxError:
        ln = getattr(node, "lineno", 1)
        text = self._lines[ln - 1] if 0 < ln <= len(self._lines) else ""
        return KernelSyntaxError(message, self._filename, self._first + ln - 1, text)

    def _at(self, out, node):
        out.lineno = self._first + getattr(node, "lineno", 1) - 1
        return out

    def _param(self, arg: ast.arg) -> ir.Param:
        ann = arg.annotation
        if ann is None:
            return ir.Param(arg.arg, "tensor")
        if isinstance(ann, ast.Subscript) and _call_name(ann.value) == "Tensor":
            return ir.Param(arg.arg, "tensor", self._dtype_name(ann.slice))
        name = _call_name(ann) if not isinstance(ann, ast.Constant) else str(ann.value)
        if name == "Tensor":
            return ir.Param(arg.arg, "tensor")
        if name in ("int", "float", "bool"):
            return ir.Param(arg.arg, name)
        if name in dtypes.ALL:                         # ``n: zse.int32`` / ``eps: zse.float32``
            d = dtypes.ALL[name]
            return ir.Param(arg.arg, "float" if d.is_float else "int")
        raise self._err(arg, f"parameter '{arg.arg}' has an annotation the kernel language does not know")

    def _dtype_name(self, node: ast.expr) -> str:
        name = _call_name(node)
        if name is None and isinstance(node, ast.Constant):
            name = str(node.value)
        if name == "float":
            name = "float32"
        if name == "int":
            name = "int32"
        if name not in dtypes.ALL:
            raise self._err(node, f"'{name}' is not an element type")
        return name

    def _const_int(self, node: ast.expr, what: str) -> int:
        e = self._expr(node)
        if isinstance(e, ir.Const) and isinstance(e.value, int) and not isinstance(e.value, bool):
            return int(e.value)
        if isinstance(e, ir.UnaryOp) and e.op == "-" and isinstance(e.operand, ir.Const):
            return -int(e.operand.value)
        raise self._err(node, f"{what} must be an integer constant")

    # ---- statements -------------------------------------------------------------------------------------------
    def _block(self, stmts) -> List[ir.Stmt]:
        out: List[ir.Stmt] = []
        for s in stmts:
            r = self._stmt(s)
            if r is not None:
                out.append(self._at(r, s))
        return out

    def _stmt(self, node: ast.stmt) -> Optional[ir.Stmt]:
        if isinstance(node, ast.Assign):
            if len(node.targets) != 1:
                raise self._err(node, "chained assignment is not part of the kernel language")
            return self._assign(node.targets[0], node.value, None, node)
        if isinstance(node, ast.AnnAssign):
            if node.value is None:
                raise self._err(node, "a declaration needs a value")
            ann = _call_name(node.annotation)
            if ann in dtypes.ALL:
                d = dtypes.ALL[ann]
                ann = {"float16": "half", "bfloat16": "bf16"}.get(ann, "float" if d.is_float else
                                                                  ("uint" if d.kind == "uint" else "int"))
            if ann not in ("int", "float", "bool", "uint", "half", "bf16"):
                raise self._err(node, "a local can be declared int, float, bool or an element type")
            return self._assign(node.target, node.value, ann, node)
        if isinstance(node, ast.AugAssign):
            op = _BINOPS.get(type(node.op))
            if op is None:
                raise self._err(node, "this operator is not part of the kernel language")
            if isinstance(node.target, ast.Name):
                cur = self._at(ir.Var(node.target.id), node)
                return ir.Assign(node.target.id, self._at(ir.BinOp(op, cur, self._expr(node.value)), node))
            if isinstance(node.target, ast.Subscript) and isinstance(node.target.value, ast.Name):
                base, idx = node.target.value.id, self._expr(node.target.slice)
                cur = self._at(ir.Load(base, idx), node)
                return ir.Store(base, idx, self._at(ir.BinOp(op, cur, self._expr(node.value)), node))
            raise self._err(node, "cannot assign to this target")
        if isinstance(node, ast.Expr):
            if isinstance(node.value, ast.Constant):          # a docstring or a stray literal
                return None
            if isinstance(node.value, ast.Call):
                call = self._expr(node.value)
                if not isinstance(call, ir.Call):
                    raise self._err(node, "this call has no effect as a statement")
                return ir.ExprStmt(call)
            raise self._err(node, "an expression statement must be a call")
        if isinstance(node, ast.If):
            return ir.If(self._expr(node.test), self._block(node.body), self._block(node.orelse))
        if isinstance(node, ast.For):
            return self._for(node)
        if isinstance(node, ast.While):
            if node.orelse:
                raise self._err(node, "while/else is not part of the kernel language")
            return ir.While(self._expr(node.test), self._block(node.body))
        if isinstance(node, ast.Return):
            if node.value is not None:
                raise self._err(node, "a kernel returns nothing: write results through a tensor")
            return ir.Return()
        if isinstance(node, ast.Break):
            return ir.Break()
        if isinstance(node, ast.Continue):
            return ir.Continue()
        if isinstance(node, ast.Pass):
            return None
        raise self._err(node, f"{type(node).__name__} statements are not part of the kernel language")

    def _assign(self, target, value, declared, node) -> ir.Stmt:
        if isinstance(target, ast.Subscript):
            if not isinstance(target.value, ast.Name):
                raise self._err(node, "only named tensors and arrays can be indexed on the left")
            return ir.Store(target.value.id, self._expr(target.slice), self._expr(value))
        if not isinstance(target, ast.Name):
            raise self._err(node, "tuple and attribute targets are not part of the kernel language")
        if isinstance(value, ast.Call) and _call_name(value.func) in DECLARATIONS:
            return self._declaration(target.id, value)
        return ir.Assign(target.id, self._expr(value), declared)

    def _declaration(self, name: str, call: ast.Call) -> ir.Stmt:
        kind, args = _call_name(call.func), call.args
        kw = {k.arg: k.value for k in call.keywords}
        if kind == "shared_memory" or kind == "local_array":
            if not args:
                raise self._err(call, f"{kind}(size, dtype) needs a size")
            size_node = args[0]
            if isinstance(size_node, ast.Tuple):            # a shape: the array is flat, row-major
                size = 1
                for el in size_node.elts:
                    size *= self._const_int(el, "a dimension")
            else:
                size = self._const_int(size_node, "the size")
            dt = args[1] if len(args) > 1 else kw.get("dtype")
            elem = self._dtype_name(dt) if dt is not None else "float32"
            if size <= 0:
                raise self._err(call, "the size must be positive")
            return ir.ArrayDecl(name, "shared" if kind == "shared_memory" else "local", elem, size)
        if kind == "dynamic_shared_memory":
            dt = args[0] if args else kw.get("dtype")
            return ir.ArrayDecl(name, "dynamic_shared", self._dtype_name(dt) if dt is not None else "float32", 0)
        # reinterpret(ptr, dtype)
        if not args or not isinstance(args[0], ast.Name):
            raise self._err(call, "reinterpret(ptr, dtype) takes a named tensor or array")
        dt = args[1] if len(args) > 1 else kw.get("dtype")
        if dt is None:
            raise self._err(call, "reinterpret(ptr, dtype) needs the new element type")
        return ir.PtrCast(name, args[0].id, self._dtype_name(dt))

    def _for(self, node: ast.For) -> ir.For:
        if node.orelse:
            raise self._err(node, "for/else is not part of the kernel language")
        it = node.iter
        if not (isinstance(it, ast.Call) and _call_name(it.func) == "range" and 1 <= len(it.args) <= 3
                and isinstance(node.target, ast.Name)):
            raise self._err(node, "loops run over range(...) with a plain loop variable")
        a = [self._expr(x) for x in it.args]
        zero, one = ir.Const(0), ir.Const(1)
        start, stop, step = (zero, a[0], one) if len(a) == 1 else (a[0], a[1], one) if len(a) == 2 else a
        return ir.For(node.target.id, start, stop, step, self._block(node.body))

    # ---- expressions ----------------------------------------------------------------------------------------------
    def _expr(self, node: ast.expr) -> ir.Expr:
        return self._at(self._expr_inner(node), node)

    def _expr_inner(self, node: ast.expr) -> ir.Expr:
        if isinstance(node, ast.Constant):
            if isinstance(node.value, (bool, int, float)):
                return ir.Const(node.value)
            raise self._err(node, f"constants of type {type(node.value).__name__} are not part of the kernel language")
        if isinstance(node, ast.Name):
            if node.id in self._locals:
                return ir.Var(node.id)
            if node.id in ("True", "False"):
                return ir.Const(node.id == "True")
            val = self._globals.get(node.id)
            if isinstance(val, (bool, int, float)):
                return ir.Const(val)
            raise self._err(node, f"'{node.id}' is neither a local, a parameter nor a module-level number")
        if isinstance(node, ast.BinOp):
            op = _BINOPS.get(type(node.op))
            if op is None:
                raise self._err(node, "this operator is not part of the kernel language")
            return ir.BinOp(op, self._expr(node.left), self._expr(node.right))
        if isinstance(node, ast.UnaryOp):
            if isinstance(node.op, ast.UAdd):
                return self._expr_inner(node.operand)
            op = {ast.USub: "-", ast.Not: "not", ast.Invert: "~"}[type(node.op)]
            inner = self._expr(node.operand)
            if op == "-" and isinstance(inner, ir.Const) and not isinstance(inner.value, bool):
                return ir.Const(-inner.value)
            return ir.UnaryOp(op, inner)
        if isinstance(node, ast.Compare):
            parts, left = [], self._expr(node.left)
            for op, right in zip(node.ops, node.comparators):
                sym = _CMPOPS.get(type(op))
                if sym is None:
                    raise self._err(node, "is / in comparisons are not part of the kernel language")
                r = self._expr(right)
                parts.append(self._at(ir.Compare(sym, left, r), node))
                left = r
            return parts[0] if len(parts) == 1 else ir.BoolOp("and", parts)
        if isinstance(node, ast.BoolOp):
            return ir.BoolOp("and" if isinstance(node.op, ast.And) else "or", [self._expr(v) for v in node.values])
        if isinstance(node, ast.IfExp):
            return ir.Ternary(self._expr(node.test), self._expr(node.body), self._expr(node.orelse))
        if isinstance(node, ast.Subscript):
            if (isinstance(node.value, ast.Name) and node.value.id in self._locals
                    and node.value.id not in self._vectors):
                return ir.Load(node.value.id, self._expr(node.slice))
            return ir.Field(self._expr(node.value), self._const_int(node.slice, "a component index"))
        if isinstance(node, ast.Attribute):
            if node.attr in _FIELDS and not (isinstance(node.value, ast.Name) and node.value.id not in self._locals):
                return ir.Field(self._expr(node.value), _FIELDS[node.attr])
            # ``module.CONSTANT``
            try:
                val = getattr(self._globals.get(node.value.id), node.attr) if isinstance(node.value, ast.Name) else None
            except AttributeError:
                val = None
            if isinstance(val, (bool, int, float)):
                return ir.Const(val)
            raise self._err(node, f"attribute '{node.attr}' is not part of the kernel language")
        if isinstance(node, ast.Call):
            return self._call(node)
        if isinstance(node, ast.Tuple):
            raise self._err(node, "tuples are not part of the kernel language")
        raise self._err(node, f"{type(node).__name__} expressions are not part of the kernel language")

    def _call(self, node: ast.Call) -> ir.Expr:
        name = _call_name(node.func)
        if name in DECLARATIONS:
            raise self._err(node, f"{name}(...) declares storage: assign it to a name on a line of its own")
        if name in BUILTINS and isinstance(node.func, ast.Name):
            args = [self._expr(a) for a in node.args]
            target = BUILTINS[name]
            if target in ("float", "int", "bool"):
                if len(args) != 1:
                    raise self._err(node, f"{name}(x) takes one argument")
                return ir.Cast(target, args[0])
            if target == "abs":
                if len(args) != 1:
                    raise self._err(node, "abs(x) takes one argument")
                return ir.Call("abs", args)
            if len(args) < 2:
                raise self._err(node, f"{name}(a, b, ...) takes at least two arguments")
            out = args[0]
            for a in args[1:]:
                out = self._at(ir.Call(target, [out, a]), node)
            return out
        if name not in PRIMITIVES:
            raise self._err(node, f"'{name}' is not a function of the kernel language")
        lo, hi, _ = PRIMITIVES[name]
        args = [self._expr(a) for a in node.args]
        if name in ("tile_load", "tile_store"):
            order = (["tensor", "tile_row", "tile_col", "tile_size", "shared_buf", "bound_row", "bound_col", "ld"]
                     if name == "tile_load" else
                     ["shared_buf", "tensor", "tile_row", "tile_col", "tile_size", "bound_row", "bound_col", "ld"])
            kw = {k.arg: self._expr(k.value) for k in node.keywords}
            full: List[Optional[ir.Expr]] = list(args) + [None] * (len(order) - len(args))
            for k, v in kw.items():
                if k not in order:
                    raise self._err(node, f"{name}() has no argument '{k}'")
                full[order.index(k)] = v
            if any(a is None for a in full[:5]):
                raise self._err(node, f"{name}() needs {', '.join(order[:5])}")
            args = [a if a is not None else ir.Const(-1) for a in full]      # -1: not given
            for i in (0, 4) if name == "tile_load" else (0, 1):
                if not isinstance(args[i], ir.Var):
                    raise self._err(node, f"{name}(): '{order[i]}' must be a named tensor or array")
        elif name == "wmma_store" and len(node.keywords) == 1 and node.keywords[0].arg == "frag":
            args.append(self._expr(node.keywords[0].value))
        elif node.keywords:
            if name.startswith("warp_shuffle") and all(k.arg == "width" for k in node.keywords):
                args.append(self._expr(node.keywords[0].value))
            else:
                raise self._err(node, f"{name}() takes positional arguments")
        if not lo <= len(args) <= hi:
            raise self._err(node, f"{name}() takes {lo if lo == hi else f'{lo} to {hi}'} arguments, got {len(args)}")
        if name in ("thread_id", "block_id", "block_dim", "grid_dim", "global_id"):
            axis = 0
            if args:
                if not (isinstance(args[0], ir.Const) and args[0].value in (0, 1, 2)):
                    raise self._err(node, f"{name}(axis): the axis is the constant 0, 1 or 2")
                axis = int(args[0].value)
            args = [ir.Const(axis)]
        if name.startswith("atomic_") and not isinstance(args[0], ir.Load):
            raise self._err(node, f"{name}(target, ...): the target is an element, e.g. out[0]")
        if name in ("load_float4", "load_half2", "store_float4", "store_half2") and not isinstance(args[0], ir.Var):
            raise self._err(node, f"{name}(): the first argument is a named tensor or array")
        if name in ("wmma_load_a", "wmma_load_b", "wmma_store") and not isinstance(args[0], ir.Var):
            raise self._err(node, f"{name}(): the first argument is a named tensor or array")
        if name == "wmma_store" and not isinstance(args[4], ir.Var):
            raise self._err(node, "wmma_store(tensor, row, col, stride, frag): frag is an accumulator fragment")
        if name in ("unpack_int4", "unpack_uint4") and not isinstance(args[1], ir.Var):
            raise self._err(node, f"{name}(packed, buf, base): buf is a named array")
        return ir.Call(name, args)
