"""Fusing element-wise kernels into one (zse-compiler/zse_compiler/ir/fusion.py:41-268).

``fuse([k1, k2, ...])`` builds one kernel that runs the bodies back to back for the same element: the tensor that
``k_i`` writes never goes to memory - its store becomes a local - and the reads of the chained input of ``k_{i+1}``
read that local.  Which input is chained is clear when the kernel reads a single tensor; otherwise ``chain`` names
it (one entry per kernel after the first).  The pass refuses kernels that are not element-wise in the needed sense:
several written tensors, barriers or collectives, or a store and a chained load that do not address the same element
(judged after replacing single-assignment locals such as ``idx = global_id(0)`` by their definitions).

Parameters of the fused kernel: every remaining parameter of every kernel in order of first appearance; parameters
with the same name and kind are one parameter (``n`` of both kernels is the same ``n``)."""
from __future__ import annotations

import copy
from dataclasses import fields, is_dataclass
from typing import Dict, List, Optional, Sequence, Set

from . import ir
from .errors import KernelSyntaxError
from .primitives import COLLECTIVES


def _map(node, fn):
    """Bottom-up rewrite of an IR tree: ``fn(node)`` may return a replacement."""
    if isinstance(node, list):
        return [_map(n, fn) for n in node]
    if is_dataclass(node) and isinstance(node, (ir.Expr, ir.Stmt)):
        for f in fields(node):
            v = getattr(node, f.name)
            if isinstance(v, (ir.Expr, ir.Stmt, list)):
                setattr(node, f.name, _map(v, fn))
        return fn(node)
    return node


def _written(func: ir.Function) -> List[str]:
    params = {p.name for p in func.params if p.kind == "tensor"}
    out: List[str] = []

    def note(name):
        if name in params and name not in out:
            out.append(name)

    for s in ir.walk_stmts(func.body):
        if isinstance(s, ir.Store):
            note(s.base)
        elif isinstance(s, ir.ExprStmt):
            c = s.call
            if c.func.startswith("atomic_"):
                note(c.args[0].base)
            elif c.func in ("store_float4", "store_half2"):
                note(c.args[0].name)
            elif c.func == "tile_store":
                note(c.args[1].name)
            elif c.func in ("unpack_int4", "unpack_uint4"):
                note(c.args[1].name)
    return out


def _read(func: ir.Function) -> List[str]:
    params = {p.name for p in func.params if p.kind == "tensor"}
    out: List[str] = []
    for e in ir.walk_exprs(func.body):
        name = e.base if isinstance(e, ir.Load) else e.name if isinstance(e, ir.Var) else None
        if name in params and name not in out:
            out.append(name)
    return out


def _single_defs(func: ir.Function) -> Dict[str, ir.Expr]:
    count: Dict[str, int] = {}
    for s in ir.walk_stmts(func.body):
        if isinstance(s, ir.Assign):
            count[s.name] = count.get(s.name, 0) + 1
        elif isinstance(s, ir.For):
            count[s.var] = count.get(s.var, 0) + 2
    return {s.name: s.value for s in func.body if isinstance(s, ir.Assign) and count[s.name] == 1}


def _signature(e: ir.Expr, defs: Dict[str, ir.Expr], depth: int = 0) -> str:
    def sub(n):
        if isinstance(n, ir.Var) and n.name in defs and depth < 8:
            return copy.deepcopy(defs[n.name])
        return n
    resolved = e
    for _ in range(8):
        before = repr(resolved)
        resolved = _map(copy.deepcopy(resolved), sub)
        if repr(resolved) == before:
            break
    return repr(resolved)


class FusionPass:
    def fuse(self, kernels: Sequence, name: Optional[str] = None, chain: Optional[Sequence[str]] = None) -> ir.Function:
        funcs = [copy.deepcopy(getattr(k, "ir", k)) for k in kernels]
        if len(funcs) < 2:
            raise KernelSyntaxError("fuse() needs at least two kernels")
        if chain is not None and len(chain) != len(funcs) - 1:
            raise KernelSyntaxError(f"chain= names the chained input of every kernel after the first "
                                    f"({len(funcs) - 1} names), got {len(chain)}")
        params: List[ir.Param] = []
        body: List[ir.Stmt] = []
        prev_local: Optional[str] = None
        prev_sig: Optional[str] = None
        for i, f in enumerate(funcs):
            last = i == len(funcs) - 1
            for e in ir.walk_exprs(f.body):
                if isinstance(e, ir.Call) and e.func in COLLECTIVES:
                    raise KernelSyntaxError(f"'{f.name}' uses {e.func}(): only element-wise kernels can be fused")
            written = _written(f)
            if len(written) != 1:
                raise KernelSyntaxError(f"'{f.name}' writes {len(written)} tensors ({', '.join(written) or 'none'}): "
                                        f"a kernel in a fusion writes exactly one")
            out_name = written[0]
            chained = None
            if i > 0:
                reads = [r for r in _read(f) if r != out_name]
                if chain is not None:
                    chained = chain[i - 1]
                    if chained not in reads:
                        raise KernelSyntaxError(f"'{f.name}' does not read a tensor named '{chained}'")
                elif len(reads) == 1:
                    chained = reads[0]
                else:
                    raise KernelSyntaxError(f"'{f.name}' reads {len(reads)} tensors ({', '.join(reads)}): say which "
                                            f"one takes the previous kernel's result with chain=[...]")
            defs = _single_defs(f)
            stores = [s for s in ir.walk_stmts(f.body) if isinstance(s, ir.Store) and s.base == out_name]
            sigs = {_signature(s.index, defs) for s in stores}
            if not last:
                if len(stores) == 0 or len(sigs) != 1:
                    raise KernelSyntaxError(f"'{f.name}' must write one element of '{out_name}' per thread to be fused")
            if chained is not None:
                for e in ir.walk_exprs(f.body):
                    if isinstance(e, ir.Load) and e.base == chained and _signature(e.index, defs) != prev_sig:
                        raise KernelSyntaxError(f"'{f.name}' reads '{chained}' at an element other than the one the "
                                                f"previous kernel wrote: the kernels are not element-wise aligned")
                    if isinstance(e, ir.Var) and e.name == chained:
                        raise KernelSyntaxError(f"'{f.name}' passes '{chained}' to a call: it cannot be fused away")
            local = f"_fused_{i}"
            tensor_params = {p.name for p in f.params if p.kind == "tensor"}
            scalar_params = {p.name for p in f.params if p.kind != "tensor"}
            locals_: Set[str] = set()
            for s in ir.walk_stmts(f.body):
                if isinstance(s, (ir.Assign, ir.ArrayDecl, ir.PtrCast)):
                    locals_.add(s.name)
                elif isinstance(s, ir.For):
                    locals_.add(s.var)
            locals_ -= tensor_params | scalar_params
            ren = {n: f"{n}__k{i}" for n in locals_}
            pl, ch, on = prev_local, chained, out_name

            def rewrite(n):
                if isinstance(n, ir.Load):
                    if ch is not None and n.base == ch:
                        v = ir.Var(pl)
                        v.lineno = n.lineno
                        return v
                    n.base = ren.get(n.base, n.base)
                elif isinstance(n, ir.Var):
                    n.name = ren.get(n.name, n.name)
                elif isinstance(n, ir.Store):
                    if not last and n.base == on:
                        a = ir.Assign(local, n.value)
                        a.lineno = n.lineno
                        return a
                    n.base = ren.get(n.base, n.base)
                elif isinstance(n, (ir.Assign, ir.ArrayDecl)):
                    n.name = ren.get(n.name, n.name)
                elif isinstance(n, ir.PtrCast):
                    n.name, n.source = ren.get(n.name, n.name), ren.get(n.source, n.source)
                elif isinstance(n, ir.For):
                    n.var = ren.get(n.var, n.var)
                return n

            body += _map(f.body, rewrite)
            for p in f.params:
                if p.name == chained or (not last and p.name == out_name):
                    continue
                same = next((q for q in params if q.name == p.name), None)
                if same is None:
                    params.append(p)
                elif (same.kind, same.elem) != (p.kind, p.elem):
                    raise KernelSyntaxError(f"parameter '{p.name}' means different things in the fused kernels")
            prev_local = local
            prev_sig = next(iter(sigs)) if sigs else None
        first = funcs[0]
        return ir.Function(name or "_".join(f.name for f in funcs), params, body, first.filename, first.first_line,
                           first.source_lines)
