"""Intermediate form of a kernel: a small tree of dataclasses that the parser produces, the type pass annotates, the
fusion pass rewrites, the CUDA emitter prints and the CPU emulator executes
(zse-compiler/zse_compiler/ir/nodes.py:13-502 plays this part in the reference).

Value types are strings: ``int``, ``uint``, ``float``, ``bool``, ``half``, ``bf16``, ``float4``, ``half2`` and
``ptr:<element type name>`` for tensors, shared arrays, local arrays and reinterpreted pointers."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, List, Optional


# ---- expressions --------------------------------------------------------------------------------------------------
@dataclass
class Expr:
    type: Optional[str] = field(default=None, init=False, repr=False)     # filled by the type pass
    lineno: int = field(default=0, init=False, repr=False)


@dataclass
class Const(Expr):
    value: Any = 0


@dataclass
class Var(Expr):
    name: str = ""


@dataclass
class BinOp(Expr):
    op: str = "+"                 # + - * / // % & | ^ << >> **
    left: Expr = None
    right: Expr = None


@dataclass
class UnaryOp(Expr):
    op: str = "-"                 # - not ~
    operand: Expr = None


@dataclass
class Compare(Expr):
    op: str = "<"                 # < <= > >= == !=
    left: Expr = None
    right: Expr = None


@dataclass
class BoolOp(Expr):
    op: str = "and"
    values: List[Expr] = field(default_factory=list)


@dataclass
class Ternary(Expr):
    cond: Expr = None
    then: Expr = None
    other: Expr = None


@dataclass
class Load(Expr):
    base: str = ""                # name of a tensor / shared array / local array / reinterpreted pointer
    index: Expr = None


@dataclass
class Field(Expr):
    value: Expr = None            # a float4 or half2 value
    index: int = 0                # component 0..3


@dataclass
class Call(Expr):
    func: str = ""                # a primitive of the language (see primitives.PRIMITIVES)
    args: List[Expr] = field(default_factory=list)


@dataclass
class Cast(Expr):
    to: str = "float"
    value: Expr = None


# ---- statements ---------------------------------------------------------------------------------------------------
@dataclass
class Stmt:
    lineno: int = field(default=0, init=False, repr=False)


@dataclass
class Assign(Stmt):
    name: str = ""
    value: Expr = None
    declared: Optional[str] = None      # type from an annotation (``acc: float = 0.0``)


@dataclass
class Store(Stmt):
    base: str = ""
    index: Expr = None
    value: Expr = None


@dataclass
class ArrayDecl(Stmt):
    name: str = ""
    space: str = "shared"               # shared | dynamic_shared | local
    elem: str = "float32"               # element type name (dtypes.ALL)
    size: int = 0                       # elements; 0 for dynamic shared memory


@dataclass
class PtrCast(Stmt):
    name: str = ""                      # new pointer name
    source: str = ""                    # existing pointer
    elem: str = "uint32"


@dataclass
class ExprStmt(Stmt):
    call: Call = None                   # syncthreads, atomics, vector stores, unpack, tile moves


@dataclass
class If(Stmt):
    cond: Expr = None
    then: List[Stmt] = field(default_factory=list)
    orelse: List[Stmt] = field(default_factory=list)


@dataclass
class For(Stmt):
    var: str = ""
    start: Expr = None
    stop: Expr = None
    step: Expr = None
    body: List[Stmt] = field(default_factory=list)


@dataclass
class While(Stmt):
    cond: Expr = None
    body: List[Stmt] = field(default_factory=list)


@dataclass
class Return(Stmt):
    pass


@dataclass
class Break(Stmt):
    pass


@dataclass
class Continue(Stmt):
    pass


# ---- function -----------------------------------------------------------------------------------------------------
@dataclass
class Param:
    name: str
    kind: str                           # "tensor" | "int" | "float" | "bool"
    elem: Optional[str] = None          # fixed element type of a tensor parameter (None: taken from the argument)


@dataclass
class Function:
    name: str
    params: List[Param]
    body: List[Stmt]
    filename: str = "<kernel>"
    first_line: int = 1
    source_lines: List[str] = field(default_factory=list)

    def line_text(self, lineno: int) -> str:
        i = lineno - self.first_line
        return self.source_lines[i] if 0 <= i < len(self.source_lines) else ""


def walk_exprs(node):
    """Every expression below ``node`` (a statement, an expression or a list of statements), depth first."""
    if isinstance(node, list):
        for n in node:
            yield from walk_exprs(n)
        return
    if isinstance(node, Expr):
        yield node
    for v in vars(node).values():
        if isinstance(v, (Expr, Stmt)):
            yield from walk_exprs(v)
        elif isinstance(v, list):
            for x in v:
                if isinstance(x, (Expr, Stmt)):
                    yield from walk_exprs(x)


def walk_stmts(body):
    for s in body:
        yield s
        for attr in ("then", "orelse", "body"):
            sub = getattr(s, attr, None)
            if isinstance(sub, list):
                yield from walk_stmts(sub)
