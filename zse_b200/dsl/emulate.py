"""CPU execution of a kernel's IR: every thread of a launch is a Python generator that runs the statements in order
and pauses at barriers and warp / block collectives, where a small scheduler exchanges the values.  It is the oracle
the generated CUDA is checked against, and lets kernels be developed and tested on a machine without a GPU.  (The
reference has no such path: its kernels can only be checked on a device.)

Arithmetic follows the emitter: floats are fp32, fp16 / bf16 elements widen on load and round on store, ``//`` and
``%`` keep Python's sign rules.  A launch in which some threads of a block wait at a barrier that others never reach
is reported as an error instead of hanging."""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np

from . import dtypes, ir
from .errors import KernelLaunchError, KernelTypeError
from .infer import TypedKernel, widen
from .primitives import COLLECTIVES

_NP = {"float32": np.float32, "float16": np.float16, "int32": np.int32, "int16": np.int16, "int8": np.int8,
       "uint32": np.uint32, "uint16": np.uint16, "uint8": np.uint8, "int4": np.uint8, "uint4": np.uint8}
f32 = np.float32


class _Return(Exception):
    pass


class _Break(Exception):
    pass


class _Continue(Exception):
    pass


def _has_collective(node) -> bool:
    return any(isinstance(e, ir.Call) and e.func in COLLECTIVES for e in ir.walk_exprs(node))


def _to_scalar(v, t: str):
    t = widen(t)
    if t == "float":
        return f32(v)
    if t == "bool":
        return bool(v)
    if t == "uint":
        return int(v) & 0xFFFFFFFF
    return int(v)


class RaceTracker:
    """Data-race detection for an emulated launch.  Two accesses to the same byte race when they come from different
    threads, at least one writes, they are not both atomic, and nothing orders them: inside a block only a barrier
    (``syncthreads``, a block reduction, a tile move) orders shared and global memory; between blocks of one launch
    nothing does.  Every byte remembers its last writer and the readers since, each with the barrier epoch of its
    block.  Races are collected (``races``) with the Python lines of both accesses; the first ``limit`` are kept."""

    def __init__(self, limit: int = 20):
        self.cells: Dict[Tuple[Any, int], list] = {}
        self.races: List[str] = []
        self.limit = limit
        self._seen: set = set()

    def _report(self, kind: str, what: str, idx: int, a, b) -> None:
        key = (kind, what, a[2], b[2])
        if key in self._seen:
            return
        self._seen.add(key)
        if len(self.races) < self.limit:
            self.races.append(f"{kind} race on {what}[{idx}]: block {a[0]} thread {a[1]} (line {a[2]}) and "
                              f"block {b[0]} thread {b[1]} (line {b[2]})")

    @staticmethod
    def _unordered(prev, blk, epoch) -> bool:
        return prev[0] != blk or prev[3] == epoch

    def access(self, root, what: str, idx: int, byte0: int, nbytes: int, blk, tid: int, epoch: int, line: int,
               write: bool, atomic: bool) -> None:
        me = (blk, tid, line, epoch, atomic)
        for byte in range(byte0, byte0 + nbytes):
            cell = self.cells.get((root, byte))
            if cell is None:
                cell = self.cells[(root, byte)] = [None, {}]            # last writer, readers by (blk, tid)
            w, readers = cell
            if w is not None and (w[0], w[1]) != (blk, tid) and self._unordered(w, blk, epoch) \
                    and not (atomic and w[4]):
                self._report("write-write" if write else "read-after-write", what, idx, w, me)
            if write:
                for r in readers.values():
                    if (r[0], r[1]) != (blk, tid) and self._unordered(r, blk, epoch):
                        self._report("write-after-read", what, idx, r, me)
                cell[0] = me
                cell[1] = {}
            else:
                readers[(blk, tid)] = me


class KernelRaceError(KernelLaunchError):
    """``emulate(..., check_races=True)`` found unordered conflicting accesses; ``races`` lists them."""

    def __init__(self, races: List[str]):
        super().__init__(f"{len(races)} data race(s) found:\n  " + "\n  ".join(races))
        self.races = races


class _Block:
    """State shared by the threads of one block."""

    def __init__(self, k: TypedKernel, mem: Dict[str, np.ndarray], scalars: Dict[str, Any], block_idx, block_dim,
                 grid_dim, dyn_smem_bytes: int):
        self.k, self.scalars = k, scalars
        self.block_idx, self.block_dim, self.grid_dim = block_idx, block_dim, grid_dim
        self.mem = dict(mem)
        for a in k.arrays:
            if a.space == "shared":
                self.mem[a.name] = np.zeros(a.size, _NP[a.elem])
            elif a.space == "dynamic_shared":
                esz = np.dtype(_NP[a.elem]).itemsize
                self.mem[a.name] = np.zeros(max(1, dyn_smem_bytes // esz), _NP[a.elem])
        self.nthreads = block_dim[0] * block_dim[1] * block_dim[2]
        self.epoch = 0                       # advanced at every block-wide barrier
        self.tracker: Optional[RaceTracker] = None
        self.shared_names = {a.name for a in k.arrays if a.space in ("shared", "dynamic_shared")}


class _Thread:
    def __init__(self, blk: _Block, tid3: Tuple[int, int, int]):
        self.b, self.tid3 = blk, tid3
        bd = blk.block_dim
        self.tid = tid3[0] + bd[0] * (tid3[1] + bd[1] * tid3[2])
        self.env: Dict[str, Any] = dict(blk.scalars)
        self.mem = dict(blk.mem)
        for a in blk.k.arrays:
            if a.space == "local":
                self.mem[a.name] = np.zeros(a.size, _NP[a.elem])
        self._coll: Dict[int, bool] = {}
        self._local = {a.name for a in blk.k.arrays if a.space == "local"}
        self._root: Dict[str, str] = {}      # reinterpreted pointer -> the array it aliases
        self._quiet = False                  # warp-wide tile calls are one access by the warp, not 32 by its lanes

    def _track(self, name: str, idx: int, node, write: bool, atomic: bool = False) -> None:
        t = self.b.tracker
        if t is None or self._quiet:
            return
        root = self._root.get(name, name)
        if root in self._local:
            return
        size = int(self.mem[name].dtype.itemsize)
        key = (root, self.b.block_idx) if root in self.b.shared_names else root
        t.access(key, name, idx, idx * size, size, self.b.block_idx, self.tid, self.b.epoch,
                 getattr(node, "lineno", 0), write, atomic)

    # ---- memory -------------------------------------------------------------------------------------------------
    def _arr(self, name: str, idx: int, node) -> np.ndarray:
        arr = self.mem[name]
        if not 0 <= idx < arr.shape[0]:
            raise IndexError(f"line {node.lineno}: {name}[{idx}] is outside its {arr.shape[0]} elements "
                             f"(block {self.b.block_idx}, thread {self.tid3})")
        return arr

    def _load(self, name: str, idx: int, node, atomic: bool = False):
        self._track(name, idx, node, False, atomic)
        v = self._arr(name, idx, node)[idx]
        return f32(v) if isinstance(v, np.floating) else int(v)

    def _store(self, name: str, idx: int, value, node, atomic: bool = False) -> None:
        self._track(name, idx, node, True, atomic)
        arr = self._arr(name, idx, node)
        if np.issubdtype(arr.dtype, np.integer):
            info = np.iinfo(arr.dtype)
            v = int(value) & ((1 << (8 * arr.dtype.itemsize)) - 1)
            arr[idx] = v - (1 << (8 * arr.dtype.itemsize)) if v > info.max else v
        else:
            arr[idx] = value

    # ---- expressions ----------------------------------------------------------------------------------------------
    def _is_coll(self, e) -> bool:
        r = self._coll.get(id(e))
        if r is None:
            r = self._coll[id(e)] = _has_collective(e)
        return r

    def pe(self, e: ir.Expr):
        """Plain evaluation (no collective below ``e``)."""
        if isinstance(e, ir.Ternary):
            return _to_scalar(self.pe(e.then) if self.pe(e.cond) else self.pe(e.other), e.type)
        if isinstance(e, ir.BoolOp):
            if e.op == "and":
                return all(bool(self.pe(v)) for v in e.values)
            return any(bool(self.pe(v)) for v in e.values)
        return self._apply(e, [self.pe(c) for c in _children(e)])

    def ge(self, e: ir.Expr):
        """Evaluation that may pause at collectives (a generator; the value is its return value)."""
        if not self._is_coll(e):
            return self.pe(e)
        if isinstance(e, ir.Ternary):
            c = yield from self.ge(e.cond)
            v = yield from self.ge(e.then if c else e.other)
            return _to_scalar(v, e.type)
        if isinstance(e, ir.BoolOp):
            for v in e.values:
                x = bool((yield from self.ge(v)))
                if x != (e.op == "and"):
                    return x
            return e.op == "and"
        vals = []
        for c in _children(e):
            vals.append((yield from self.ge(c)))
        if isinstance(e, ir.Call) and e.func in COLLECTIVES:
            return (yield from self._collective(e, vals))
        return self._apply(e, vals)

    def _apply(self, e: ir.Expr, v: List[Any]):
        if isinstance(e, ir.Const):
            return _to_scalar(e.value, e.type)
        if isinstance(e, ir.Var):
            return e.name if e.name in self.mem else self.env[e.name]
        if isinstance(e, ir.Load):
            return self._load(e.base, int(v[0]), e)
        if isinstance(e, ir.Field):
            return f32(v[0][e.index])
        if isinstance(e, ir.Cast):
            if e.to == "int":
                return int(math.trunc(float(v[0])))        # numpy.float32 has no __trunc__
            return _to_scalar(v[0], e.to)
        if isinstance(e, ir.Compare):
            a, b = v
            return {"<": a < b, "<=": a <= b, ">": a > b, ">=": a >= b, "==": a == b, "!=": a != b}[e.op]
        if isinstance(e, ir.UnaryOp):
            if e.op == "not":
                return not v[0]
            return _to_scalar(-v[0] if e.op == "-" else ~int(v[0]), e.type)
        if isinstance(e, ir.BinOp):
            return self._binop(e, v[0], v[1])
        if isinstance(e, ir.Call):
            return self._call(e, v)
        raise NotImplementedError(type(e).__name__)

    def _binop(self, e: ir.BinOp, a, b):
        t, op = e.type, e.op
        with np.errstate(all="ignore"):
            if op == "/":
                return f32(a) / f32(b)
            if op == "**":
                return f32(np.power(f32(a), f32(b)))
            if t == "float":
                a, b = f32(a), f32(b)
                if op == "//":
                    return f32(np.floor(a / b))
                if op == "%":
                    r = np.fmod(a, b)
                    return f32(r + b) if (r != 0 and ((r < 0) != (b < 0))) else f32(r)
                return f32({"+": a + b, "-": a - b, "*": a * b}[op])
            a, b = int(a), int(b)
            r = {"+": lambda: a + b, "-": lambda: a - b, "*": lambda: a * b, "//": lambda: a // b,
                 "%": lambda: a % b, "&": lambda: a & b, "|": lambda: a | b, "^": lambda: a ^ b,
                 "<<": lambda: a << b, ">>": lambda: a >> b}[op]()
            return _to_scalar(r, t)

    def _call(self, e: ir.Call, v: List[Any]):
        n, b = e.func, self.b
        if n == "thread_id":
            return self.tid3[e.args[0].value]
        if n == "block_id":
            return b.block_idx[e.args[0].value]
        if n == "block_dim":
            return b.block_dim[e.args[0].value]
        if n == "grid_dim":
            return b.grid_dim[e.args[0].value]
        if n == "global_id":
            ax = e.args[0].value
            return b.block_idx[ax] * b.block_dim[ax] + self.tid3[ax]
        if n == "lane_id":
            return self.tid & 31
        if n == "warp_id":
            return self.tid >> 5
        if n.startswith("atomic_"):
            base, idx = e.args[0].base, int(v[0])
            self._quiet = True
            old = self._load(base, idx, e)
            self._quiet = False
            if n == "atomic_add":
                new = old + v[1]
            elif n == "atomic_max":
                new = max(old, int(v[1]))
            elif n == "atomic_min":
                new = min(old, int(v[1]))
            else:
                new = v[2] if old == v[1] else old
            self._store(base, idx, new, e, atomic=True)
            return old
        with np.errstate(all="ignore"):
            if n in ("exp", "log", "sqrt", "cos", "sin", "tanh"):
                return f32(getattr(np, n)(f32(v[0])))
            if n == "rsqrt":
                return f32(1.0) / np.sqrt(f32(v[0]))
            if n == "pow":
                return f32(np.power(f32(v[0]), f32(v[1])))
            if n == "fma":
                return f32(np.float64(v[0]) * np.float64(v[1]) + np.float64(v[2]))
        if n in ("max_val", "min_val"):
            return _to_scalar(max(v) if n == "max_val" else min(v), e.type)
        if n == "abs":
            return _to_scalar(abs(v[0]), e.type)
        if n in ("half_to_float", "bf16_to_float"):
            return f32(v[0])
        if n == "float_to_half":
            return f32(np.float16(v[0]))
        if n == "float_to_bf16":
            return _bf16_round(v[0])
        if n == "load_float4":
            i = int(v[1])
            return tuple(self._load(v[0], 4 * i + j, e) for j in range(4))
        if n == "load_half2":
            i = int(v[1])
            return tuple(self._load(v[0], 2 * i + j, e) for j in range(2))
        if n in ("store_float4", "store_half2"):
            w = 4 if n == "store_float4" else 2
            for j in range(w):
                self._store(v[0], w * int(v[1]) + j, f32(v[2 + j]), e)
            return None
        if n in ("wmma_load_a", "wmma_load_b"):
            r0, c0, ld = int(v[1]), int(v[2]), int(v[3])
            self._quiet = (self.tid & 31) != 0
            try:
                return self._wmma_tile(v[0], r0, c0, ld, e)
            finally:
                self._quiet = False
        if n == "wmma_fill":
            return np.full((16, 16), f32(v[0]) if v else f32(0), f32)
        if n == "wmma_mma":
            return (v[0].astype(np.float64) @ v[1].astype(np.float64) + v[2]).astype(f32)
        if n == "wmma_store":
            r0, c0, ld = int(v[1]), int(v[2]), int(v[3])
            self._quiet = (self.tid & 31) != 0
            try:
                for r in range(16):
                    for c in range(16):
                        self._store(v[0], (r0 + r) * ld + c0 + c, v[4][r, c], e)
            finally:
                self._quiet = False
            return None
        if n in ("unpack_int4", "unpack_uint4"):
            p, base = int(v[0]) & 0xFFFFFFFF, int(v[2])
            for j in range(8):
                nib = (p >> (4 * j)) & 0xF
                if n == "unpack_int4" and nib >= 8:
                    nib -= 16
                self._store(v[1], base + j, nib, e)
            return None
        raise NotImplementedError(n)

    def _wmma_tile(self, name: str, r0: int, c0: int, ld: int, e) -> np.ndarray:
        return np.array([[self._load(name, (r0 + r) * ld + c0 + c, e) for c in range(16)] for r in range(16)], f32)

    def _collective(self, e: ir.Call, v: List[Any]):
        n = e.func
        if n == "syncthreads":
            yield ("block", "sync", None)
            return None
        if n in ("tile_load", "tile_store"):
            load = n == "tile_load"
            tensor, smem = (v[0], v[4]) if load else (v[1], v[0])
            trow, tcol, t = (v[1], v[2], v[3]) if load else (v[2], v[3], v[4])
            br, bc, ld = int(v[5]), int(v[6]), int(v[7])
            ld = ld if ld >= 0 else bc
            if not load:
                yield ("block", "sync", None)
            for el in range(self.tid, t * t, self.b.nthreads):
                r, c = int(trow) * t + el // t, int(tcol) * t + el % t
                ok = (br < 0 or r < br) and (bc < 0 or c < bc)
                if load:
                    self._store(smem, el, self._load(tensor, r * ld + c, e) if ok else 0, e)
                elif ok:
                    self._store(tensor, r * ld + c, self._load(smem, el, e), e)
            if load:
                yield ("block", "sync", None)
            return None
        scope = "block" if n.startswith("block_") else "warp"
        if n.startswith("warp_shuffle"):
            width = int(v[2]) if len(v) > 2 else 32
            res = yield ("warp", n, (v[0], int(v[1]), width))
        else:
            res = yield (scope, n, v[0])
        return res if n in ("warp_ballot", "warp_all", "warp_any") else _to_scalar(res, e.type)

    # ---- statements -------------------------------------------------------------------------------------------
    def run(self):
        try:
            yield from self._block(self.b.k.func.body)
        except _Return:
            pass

    def _block(self, body):
        for s in body:
            yield from self._stmt(s)

    def _stmt(self, s: ir.Stmt):
        if isinstance(s, ir.Assign):
            v = yield from self.ge(s.value)
            t = self.b.k.var_types[s.name]
            self.env[s.name] = (v if t in ("float4", "half2") or t.startswith("frag_")
                                else _to_scalar(_narrow(v, t), t))
        elif isinstance(s, ir.Store):
            idx = yield from self.ge(s.index)
            v = yield from self.ge(s.value)
            self._store(s.base, int(idx), v, s)
        elif isinstance(s, ir.PtrCast):
            src = self.mem[s.source]
            self.mem[s.name] = src.view(np.uint8).view(_NP[s.elem])
            self._root[s.name] = self._root.get(s.source, s.source)
        elif isinstance(s, ir.ExprStmt):
            yield from self.ge(s.call)
        elif isinstance(s, ir.If):
            c = yield from self.ge(s.cond)
            yield from self._block(s.then if c else s.orelse)
        elif isinstance(s, ir.For):
            i = int((yield from self.ge(s.start)))
            stop = int((yield from self.ge(s.stop)))
            step = int((yield from self.ge(s.step)))
            if step == 0:
                raise ZeroDivisionError(f"line {s.lineno}: range() step is zero")
            self.env[s.var] = i
            while (i < stop) if step > 0 else (i > stop):
                try:
                    yield from self._block(s.body)
                except _Break:
                    break
                except _Continue:
                    pass
                i = int(self.env[s.var]) + step
                self.env[s.var] = i
        elif isinstance(s, ir.While):
            while (yield from self.ge(s.cond)):
                try:
                    yield from self._block(s.body)
                except _Break:
                    break
                except _Continue:
                    pass
        elif isinstance(s, ir.Return):
            raise _Return()
        elif isinstance(s, ir.Break):
            raise _Break()
        elif isinstance(s, ir.Continue):
            raise _Continue()
        elif isinstance(s, ir.ArrayDecl):
            pass
        else:
            raise NotImplementedError(type(s).__name__)


def _children(e: ir.Expr) -> List[ir.Expr]:
    if isinstance(e, (ir.Const, ir.Var)):
        return []
    if isinstance(e, ir.Load):
        return [e.index]
    if isinstance(e, (ir.Field, ir.Cast)):
        return [e.value]
    if isinstance(e, ir.UnaryOp):
        return [e.operand]
    if isinstance(e, (ir.BinOp, ir.Compare)):
        return [e.left, e.right]
    if isinstance(e, ir.Call):
        if e.func.startswith("atomic_"):
            return [e.args[0].index] + list(e.args[1:])          # the target element is an address, not a value
        return list(e.args)
    raise NotImplementedError(type(e).__name__)


def _bf16_round(v) -> np.float32:
    bits = np.array([v], np.float32).view(np.uint32)[0]
    if np.isnan(np.float32(v)):
        return f32(np.nan)
    bits = (int(bits) + 0x7FFF + ((int(bits) >> 16) & 1)) & 0xFFFF0000
    return np.array([bits], np.uint32).view(np.float32)[0]


def _narrow(v, t: str):
    if t == "half":
        return f32(np.float16(v))
    if t == "bf16":
        return _bf16_round(v)
    return v


# ---- collectives: what a group of waiting threads gets back -------------------------------------------------------
def _resolve_warp(op: str, reqs: Dict[int, Any]) -> Dict[int, Any]:
    """``reqs``: lane -> payload of every live lane of one warp."""
    lanes = sorted(reqs)
    if op.startswith("warp_shuffle"):
        out = {}
        for lane in lanes:
            val, arg, width = reqs[lane]
            base = lane - lane % width
            if op == "warp_shuffle_down":
                src = lane + arg if (lane % width) + arg < width else lane
            elif op == "warp_shuffle_up":
                src = lane - arg if (lane % width) - arg >= 0 else lane
            elif op == "warp_shuffle_xor":
                src = base + ((lane % width) ^ arg) if ((lane % width) ^ arg) < width else lane
            else:
                src = base + arg % width
            out[lane] = reqs[src][0] if src in reqs else val      # an absent lane: CUDA leaves it undefined
        return out
    if op == "warp_ballot":
        mask = sum(1 << l for l in lanes if reqs[l])
        return {l: mask for l in lanes}
    if op == "warp_all":
        r = all(bool(reqs[l]) for l in lanes)
        return {l: r for l in lanes}
    if op == "warp_any":
        r = any(bool(reqs[l]) for l in lanes)
        return {l: r for l in lanes}
    return {l: _reduce(op, [reqs[x] for x in lanes]) for l in lanes}


def _reduce(op: str, vals: List[Any]):
    kind = op.rsplit("_", 1)[1]
    if kind == "sum":
        if any(isinstance(v, np.floating) for v in vals):
            return f32(np.sum(np.array(vals, np.float64)))
        return sum(int(v) for v in vals)
    return max(vals) if kind == "max" else min(vals)


def _run_block(blk: _Block) -> None:
    bd = blk.block_dim
    threads = [_Thread(blk, (x, y, z)) for z in range(bd[2]) for y in range(bd[1]) for x in range(bd[0])]
    gens = {t.tid: t.run() for t in threads}
    waiting: Dict[int, Tuple[str, str, Any]] = {}
    resume: Dict[int, Any] = {tid: None for tid in gens}           # threads ready to run, with the value they get
    while gens:
        for tid, value in list(resume.items()):
            try:
                req = gens[tid].send(value)
                waiting[tid] = req
            except StopIteration:
                del gens[tid]
        resume = {}
        if not gens:
            break
        # warps whose live lanes all wait at the same warp-level call
        by_warp: Dict[int, List[int]] = {}
        for tid in gens:
            by_warp.setdefault(tid >> 5, []).append(tid)
        for warp, tids in by_warp.items():
            if all(t in waiting and waiting[t][0] == "warp" for t in tids):
                ops = {waiting[t][1] for t in tids}
                if len(ops) != 1:
                    raise KernelLaunchError(f"block {blk.block_idx}, warp {warp}: lanes wait at different warp "
                                            f"calls ({', '.join(sorted(ops))})")
                res = _resolve_warp(ops.pop(), {t & 31: waiting[t][2] for t in tids})
                for t in tids:
                    resume[t] = res[t & 31]
                    del waiting[t]
        if not resume and all(t in waiting and waiting[t][0] == "block" for t in gens):
            if len(gens) != blk.nthreads:
                raise KernelLaunchError(f"block {blk.block_idx}: {blk.nthreads - len(gens)} threads returned while "
                                        f"the others wait at a barrier or block reduction")
            ops = {waiting[t][1] for t in gens}
            if len(ops) != 1:
                raise KernelLaunchError(f"block {blk.block_idx}: threads wait at different block-level calls "
                                        f"({', '.join(sorted(ops))})")
            op = ops.pop()
            value = None if op == "sync" else _reduce(op, [waiting[t][2] for t in sorted(gens)])
            for t in gens:
                resume[t] = value
            waiting.clear()
            blk.epoch += 1
        if not resume:
            raise KernelLaunchError(f"block {blk.block_idx}: the threads wait for one another at different "
                                    f"collectives and none can proceed")


def emulate(k: TypedKernel, grid: Sequence[int], block: Sequence[int], args: Sequence[Any],
            shared_mem_bytes: int = 0, check_races: bool = False) -> None:
    """Runs the launch on the CPU, blocks one after another.  Tensor arguments (torch CPU tensors, numpy arrays or
    ``dsl.Tensor`` objects holding one) are modified in place.  With ``check_races`` every access to global and
    shared memory is checked for unordered conflicts (``RaceTracker``) and ``KernelRaceError`` is raised at the end if
    any was seen."""
    grid = tuple(int(g) for g in grid) + (1,) * (3 - len(grid))
    block = tuple(int(b) for b in block) + (1,) * (3 - len(block))
    f = k.func
    if len(args) != len(f.params):
        raise KernelTypeError(f"{f.name}() takes {len(f.params)} arguments, got {len(args)}")
    mem: Dict[str, np.ndarray] = {}
    scalars: Dict[str, Any] = {}
    write_back = []
    for p, a in zip(f.params, args):
        if p.kind != "tensor":
            scalars[p.name] = _to_scalar(a, p.kind)
            continue
        elem = k.ptr_elem[p.name]
        a = getattr(a, "data", a) if isinstance(a, dtypes.Tensor) else a
        if hasattr(a, "detach"):                      # a torch tensor
            import torch
            if a.device.type != "cpu":
                raise KernelLaunchError("the emulator works on CPU tensors")
            if not a.is_contiguous():
                raise KernelLaunchError(f"argument '{p.name}' must be contiguous")
            if a.dtype == torch.bfloat16:
                arr = a.detach().float().numpy().reshape(-1).copy()
                write_back.append((a, arr))
                if elem != "bfloat16":
                    raise KernelTypeError(f"argument '{p.name}' is bfloat16 but the kernel expects {elem}")
                mem[p.name] = _BF16View(arr)
                continue
            arr = a.detach().numpy().reshape(-1)
        else:
            arr = np.asarray(a).reshape(-1)
        if arr.dtype != np.dtype(_NP[elem]):
            raise KernelTypeError(f"argument '{p.name}' holds {arr.dtype} but the kernel expects {elem}")
        mem[p.name] = arr
    tracker = RaceTracker() if check_races else None
    for bz in range(grid[2]):
        for by in range(grid[1]):
            for bx in range(grid[0]):
                blk = _Block(k, mem, scalars, (bx, by, bz), block, grid, shared_mem_bytes)
                blk.tracker = tracker
                _run_block(blk)
    for t, arr in write_back:
        import torch
        t.copy_(torch.from_numpy(arr.reshape(tuple(t.shape))).to(torch.bfloat16))
    if tracker is not None and tracker.races:
        raise KernelRaceError(tracker.races)


class _BF16View:
    """A float32 array that rounds what is stored into it to bf16 (numpy has no bf16)."""

    def __init__(self, arr: np.ndarray):
        self.arr, self.shape, self.dtype = arr, arr.shape, arr.dtype

    def __getitem__(self, i):
        return self.arr[i]

    def __setitem__(self, i, v):
        self.arr[i] = _bf16_round(v)

    def view(self, *_):
        raise KernelLaunchError("a bfloat16 argument cannot be reinterpreted in the emulator")
