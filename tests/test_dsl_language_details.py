"""More of the kernel language, feature by feature: control flow (while, elif chains, break / continue), integer and bit
arithmetic with Python's floor semantics, the math intrinsics, casts, two-dimensional launches, shared memory with
barriers, block and warp reductions, atomics, packed half2 access.  Every kernel is run on the CPU emulator against
plain torch / numpy and its CUDA text is checked for the constructs it should map to (the reference's compiler tests,
zse-compiler/tests/test_tier*.py, assert on generated source only)."""
import numpy as np
import pytest
import torch

import zse_b200.dsl as zse


@zse.kernel
def collatz(x: zse.Tensor[zse.int32], steps: zse.Tensor[zse.int32], n: int):
    i = zse.global_id(0)
    if i < n:
        v = x[i]
        c = 0
        while v != 1:
            if v % 2 == 0:
                v = v // 2
            else:
                v = 3 * v + 1
            c += 1
        steps[i] = c

@zse.kernel
def classify(x: zse.Tensor, out: zse.Tensor[zse.int32], n: int):
    i = zse.global_id(0)
    if i < n:
        v = x[i]
        if v < -1.0:
            out[i] = 0
        elif v < 0.0:
            out[i] = 1
        elif v < 1.0:
            out[i] = 2
        else:
            out[i] = 3

@zse.kernel
def bits(x: zse.Tensor[zse.int32], out: zse.Tensor[zse.int32], n: int):
    i = zse.global_id(0)
    if i < n:
        v = x[i]
        out[i] = ((v << 3) | (v >> 1)) ^ (v & 0xF)

@zse.kernel
def mathk(x: zse.Tensor, out: zse.Tensor, n: int):
    i = zse.global_id(0)
    if i < n:
        v = x[i]
        a = zse.fma(v, 2.0, 1.0)
        b = zse.tanh(v) + zse.sin(v) * zse.cos(v)
        c = zse.sqrt(zse.max_val(v, 0.0)) + zse.log(zse.min_val(zse.max_val(v, 0.5), 4.0)) + zse.pow(2.0, v)
        out[i] = a + b + c

@zse.kernel
def grid2d(out: zse.Tensor[zse.int32], w: int, h: int):
    x = zse.global_id(0)
    y = zse.global_id(1)
    if x < w and y < h:
        out[y * w + x] = zse.block_id(1) * 1000 + zse.thread_id(1) * 100 + zse.block_dim(1) * 10 + zse.grid_dim(0)

@zse.kernel
def tree_sum(x: zse.Tensor, out: zse.Tensor, n: int):
    buf = zse.shared_memory(64, zse.float32)
    tid = zse.thread_id(0)
    acc = 0.0
    for i in range(tid, n, 64):
        acc += x[zse.block_id(0) * n + i]
    buf[tid] = acc
    zse.syncthreads()
    s = 32
    while s > 0:
        if tid < s:
            buf[tid] = buf[tid] + buf[tid + s]
        zse.syncthreads()
        s = s // 2
    if tid == 0:
        out[zse.block_id(0)] = buf[0]

@zse.kernel
def minmax(x: zse.Tensor, out: zse.Tensor, n: int):
    tid = zse.thread_id(0)
    lo = 1e30
    hi = -1e30
    for i in range(tid, n, zse.block_dim(0)):
        lo = zse.min_val(lo, x[i])
        hi = zse.max_val(hi, x[i])
    a = zse.block_reduce_min(lo)
    b = zse.block_reduce_max(hi)
    c = zse.warp_reduce_min(lo)
    if tid == 0:
        out[0] = a
        out[1] = b
        out[2] = c

@zse.kernel
def atom(x: zse.Tensor[zse.int32], out: zse.Tensor[zse.int32], n: int):
    i = zse.global_id(0)
    if i < n:
        zse.atomic_max(out[0], x[i])
        zse.atomic_min(out[1], x[i])
        zse.atomic_cas(out[2], 0, x[i] + 1)

@zse.kernel
def half2k(x: zse.Tensor[zse.float16], out: zse.Tensor[zse.float16], n: int):
    i = zse.global_id(0)
    if i * 2 < n:
        v = zse.load_half2(x, i)
        zse.store_half2(out, i, v.x * 2.0, v.y + 1.0)

@zse.kernel
def casts(x: zse.Tensor, out: zse.Tensor[zse.int32], n: int):
    i = zse.global_id(0)
    if i < n:
        out[i] = int(x[i] * 10.0) + int(float(i) / 2.0)

@zse.kernel
def skip(x: zse.Tensor, out: zse.Tensor, n: int):
    tid = zse.thread_id(0)
    acc = 0.0
    for i in range(n):
        if x[i] < 0.0:
            continue
        if x[i] > 100.0:
            break
        acc += x[i]
    out[tid] = acc


# ---- control flow -----------------------------------------------------------------------------------------------
def test_while_loop_with_data_dependent_trip_count():
    x = torch.tensor([1, 2, 3, 6, 7, 27], dtype=torch.int32)
    steps = torch.zeros(6, dtype=torch.int32)
    collatz.emulate((1,), (32,), (x, steps, 6))
    assert steps.tolist() == [0, 1, 7, 8, 16, 111]
    text = collatz.source()
    assert "while ((v != 1)) {" in text and "zse_floordiv(v, 2)" in text and "zse_mod(v, 2)" in text


def test_elif_chain_becomes_nested_else_branches():
    x = torch.tensor([-2.0, -0.5, 0.5, 3.0, -1.0, 0.0, 1.0])
    out = torch.full((7,), -1, dtype=torch.int32)
    classify.emulate((1,), (32,), (x, out, 7))
    assert out.tolist() == [0, 1, 2, 3, 1, 2, 3]
    text = classify.source()
    assert text.count("} else {") == 3 and "(v < -1.0f)" in text


def test_break_and_continue_inside_a_counted_loop():
    x = torch.tensor([1.0, -5.0, 2.0, 200.0, 7.0])
    out = torch.zeros(32)
    skip.emulate((1,), (32,), (x, out, 5))
    assert out.tolist() == [3.0] * 32                          # -5 skipped, the loop ends at 200
    text = skip.source()
    assert "continue;" in text and "break;" in text and "for (i = 0; i < zse_stop1; i += zse_step1)" in text


# ---- integer arithmetic -----------------------------------------------------------------------------------------
def test_shifts_and_bitwise_operators():
    x = torch.arange(40, dtype=torch.int32)
    out = torch.zeros(40, dtype=torch.int32)
    bits.emulate((2,), (32,), (x, out, 40))
    v = x.numpy()
    assert (out.numpy() == (((v << 3) | (v >> 1)) ^ (v & 0xF))).all()
    assert "(((v << 3) | (v >> 1)) ^ (v & 15))" in bits.source()


@zse.kernel
def floor_ops(a: zse.Tensor[zse.int32], b: zse.Tensor[zse.int32], q: zse.Tensor[zse.int32], r: zse.Tensor[zse.int32],
              n: int):
    i = zse.global_id(0)
    if i < n:
        q[i] = a[i] // b[i]
        r[i] = a[i] % b[i]


def test_floor_division_and_modulo_follow_python_for_negative_operands():
    a = torch.tensor([7, -7, 7, -7, 0, -1, 6, -6], dtype=torch.int32)
    b = torch.tensor([2, 2, -2, -2, 5, 5, 3, 3], dtype=torch.int32)
    q, r = torch.zeros(8, dtype=torch.int32), torch.zeros(8, dtype=torch.int32)
    floor_ops.emulate((1,), (32,), (a, b, q, r, 8))
    assert q.tolist() == [x // y for x, y in zip(a.tolist(), b.tolist())] == [3, -4, -4, 3, 0, -1, 2, -2]
    assert r.tolist() == [x % y for x, y in zip(a.tolist(), b.tolist())] == [1, 1, -1, -1, 0, 4, 0, 0]
    text = floor_ops.source()
    assert "__device__ __forceinline__ int zse_floordiv(int a, int b)" in text and "zse_mod(a[i], b[i])" in text


def test_casts_truncate_toward_zero():
    x = torch.tensor([0.19, 1.25, -0.31, 2.0])
    out = torch.zeros(4, dtype=torch.int32)
    casts.emulate((1,), (32,), (x, out, 4))
    assert out.tolist() == [1, 12, -3 + 1, 20 + 1]             # int(-3.1) = -3 (not -4); i/2 truncated: 0, 0, 1, 1
    assert "(int)((x[i] * 10.0f))" in casts.source() and "(float)(i) / 2.0f" in casts.source()


# ---- math -------------------------------------------------------------------------------------------------------
def test_math_intrinsics_map_to_the_single_precision_functions():
    x = torch.linspace(-2, 2, 50)
    out = torch.zeros(50)
    mathk.emulate((2,), (32,), (x, out, 50))
    want = (x * 2 + 1 + torch.tanh(x) + torch.sin(x) * torch.cos(x) + torch.sqrt(x.clamp(min=0))
            + torch.log(x.clamp(0.5, 4.0)) + torch.pow(2.0, x))
    torch.testing.assert_close(out, want, atol=1e-5, rtol=1e-5)
    text = mathk.source()
    for fn in ("fmaf(v, 2.0f, 1.0f)", "tanhf(v)", "sinf(v)", "cosf(v)", "sqrtf(", "logf(", "powf(2.0f, v)", "fmaxf(",
               "fminf("):
        assert fn in text


# ---- launches in two dimensions ---------------------------------------------------------------------------------
def test_two_dimensional_ids_and_extents():
    out = torch.full((6 * 5,), -1, dtype=torch.int32)
    grid2d.emulate((2, 3), (4, 2), (out, 6, 5))                # 8 x 6 threads over a 6 x 5 image
    img = out.view(5, 6)
    for y in range(5):
        assert (img[y] == (y // 2) * 1000 + (y % 2) * 100 + 2 * 10 + 2).all()     # block y, thread y, blockDim.y, gridDim.x
    text = grid2d.source()
    assert "blockIdx.y * blockDim.y + threadIdx.y" in text and "(int)gridDim.x" in text and "((x < w) && (y < h))" in text


# ---- shared memory, barriers, reductions ------------------------------------------------------------------------
def test_shared_memory_tree_reduction_with_barriers():
    x = torch.randn(3, 100, generator=torch.Generator().manual_seed(0))
    out = torch.zeros(3)
    tree_sum.emulate((3,), (64,), (x, out, 100))
    torch.testing.assert_close(out, x.sum(-1), atol=1e-4, rtol=1e-4)
    text = tree_sum.source()
    assert "__shared__ float buf[64];" in text and text.count("__syncthreads();") == 2


def test_block_and_warp_min_max_reductions():
    x = torch.randn(500, generator=torch.Generator().manual_seed(1))
    out = torch.zeros(3)
    minmax.emulate((1,), (64,), (x, out, 500))
    assert out[0] == x.min() and out[1] == x.max()
    first_warp = torch.stack([x[i::64] for i in range(32)]).min()                # what lanes 0..31 saw
    assert out[2] == first_warp
    text = minmax.source()
    assert "zse_block_min_float" in text and "zse_block_max_float" in text and "__shfl_xor_sync" in text


# ---- atomics and packed access ----------------------------------------------------------------------------------
def test_atomic_max_min_and_compare_and_swap():
    x = torch.tensor([5, -3, 9, 2], dtype=torch.int32)
    out = torch.tensor([-100, 100, 0], dtype=torch.int32)
    atom.emulate((1,), (32,), (x, out, 4))
    assert out[0] == 9 and out[1] == -3
    assert out[2] == 6                                         # only the first thread finds 0 there: 5 + 1
    text = atom.source()
    assert "atomicMax(&out[0]" in text and "atomicMin(&out[1]" in text and "atomicCAS(&out[2], (int)(0)" in text


def test_half2_loads_and_stores_move_two_values_at_once():
    x = torch.arange(8).half()
    out = torch.zeros(8).half()
    half2k.emulate((1,), (32,), (x, out, 8))
    assert out.tolist() == [0.0, 2.0, 4.0, 4.0, 8.0, 6.0, 12.0, 8.0]              # even lanes doubled, odd lanes + 1
    text = half2k.source()
    assert "reinterpret_cast<const __half2*>(x)[i]" in text and "__floats2half2_rn(" in text
    assert "__low2float(v)" in text and "__high2float(v)" in text


# ---- every kernel of this file is real CUDA ---------------------------------------------------------------------
@pytest.mark.timeout(600)
def test_these_kernels_compile_for_sm_100a(tmp_path, monkeypatch):
    import shutil
    if shutil.which("nvcc") is None:
        pytest.skip("nvcc is not installed")
    monkeypatch.setenv("ZSE_KERNEL_CACHE", str(tmp_path))
    comp = zse.RuntimeCompiler()
    kernels = (collatz, classify, bits, mathk, grid2d, tree_sum, minmax, atom, half2k, casts, skip, floor_ops)
    for k in kernels:
        ck = comp.compile(k.source(line_info=True), k.name)
        assert ck.cubin[:4] == b"\x7fELF" and not ck.from_cache, k.name
    assert comp.stats["compiled"] == len(kernels)


# ---- the type pass and the IR walkers ---------------------------------------------------------------------------------
@zse.kernel
def typed(x: zse.Tensor, y: zse.Tensor[zse.float16], out: zse.Tensor, n: int, s: float):
    i = zse.global_id(0)
    acc = 0
    for j in range(n):
        acc += x[j] * s
    h = y[i]
    b = i < n and acc > 0.0
    if b:
        out[i] = acc + h


def test_scalar_ranks_and_widening():
    from zse_b200.dsl.infer import promote, widen
    assert widen("half") == widen("bf16") == "float" and widen("int") == "int"
    assert promote("bool", "int") == "int" and promote("int", "uint") == "uint" and promote("uint", "float") == "float"
    assert promote("half", "int") == "float" and promote("bool", "bool") == "bool"
    assert promote("float", "int") == promote("int", "float")
    with pytest.raises(zse.KernelTypeError, match="cannot combine"):
        promote("int", "fragment")


def test_a_local_takes_the_widest_type_assigned_to_it():
    t = zse.infer_types(typed.ir, {"x": "float32"})
    assert t.var_types == {"n": "int", "s": "float", "i": "int", "acc": "float", "j": "int", "h": "float", "b": "bool"}
    assert t.ptr_elem == {"x": "float32", "y": "float16", "out": "float32"}       # the annotation wins for y
    assert t.uses == {"global_id"}
    assert [t.param_ctype(p) for p in typed.ir.params] == ["float*", "__half*", "float*", "int", "float"]
    half = zse.infer_types(typed.ir, {"x": "float16", "out": "bfloat16", "y": "float32"})
    assert half.ptr_elem == {"x": "float16", "y": "float16", "out": "bfloat16"}
    assert half.var_types["acc"] == "float"                                        # fp16 elements widen in arithmetic
    assert [half.param_ctype(p) for p in typed.ir.params][:3] == ["__half*", "__half*", "__nv_bfloat16*"]


def test_ir_walkers_visit_nested_bodies():
    from zse_b200.dsl import ir
    stmts = [type(s).__name__ for s in ir.walk_stmts(typed.ir.body)]
    assert stmts == ["Assign", "Assign", "For", "Assign", "Assign", "Assign", "If", "Store"]
    exprs = list(ir.walk_exprs(typed.ir.body))
    kinds = [type(e).__name__ for e in exprs]
    assert kinds.count("Load") == 2 and kinds.count("Call") == 1 and kinds.count("BoolOp") == 1
    assert kinds.count("Compare") == 2 and kinds.count("BinOp") == 3
    assert {e.name for e in exprs if isinstance(e, ir.Var)} >= {"n", "acc", "j", "s", "i", "b", "h"}
    first_if = next(s for s in ir.walk_stmts(typed.ir.body) if isinstance(s, ir.If))
    assert [type(e).__name__ for e in ir.walk_exprs(first_if.cond)] == ["Var"]    # an expression walks itself too


def _uses_helper(x: zse.Tensor, n: int):
    i = zse.global_id(0)
    if i < n:
        x[i] = my_helper(x[i])            # noqa: F821  (not a primitive: a warning, the parser refuses it later)


def _has_default(x: zse.Tensor, n: int = 4):
    x[0] = n


def _has_lambda(x: zse.Tensor):
    f = lambda v: v                       # noqa: E731
    x[0] = 1.0


def test_validation_warns_about_unknown_calls_and_refuses_python_only_constructs():
    warnings = zse.validate_kernel(_uses_helper)
    assert len(warnings) == 1 and "my_helper" in warnings[0] and "line" in warnings[0]
    assert typed.warnings == []
    with pytest.raises(zse.KernelSyntaxError, match="default arguments"):
        zse.validate_kernel(_has_default)
    with pytest.raises(zse.KernelSyntaxError, match="lambda") as exc:
        zse.validate_kernel(_has_lambda)
    assert "f = lambda v: v" in str(exc.value)                                     # the offending line is quoted
