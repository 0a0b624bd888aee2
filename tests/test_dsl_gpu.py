"""The kernel language on a GPU: every kernel of ``zse_b200.dsl.kernels`` is compiled to a cubin, loaded through the
driver API, launched on torch's stream, and compared with its own CPU emulation (argument packing, module loading and
``cuLaunchKernel`` are what is under test).  All shapes are a few KB and every kernel guards its indices."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from zse_b200.dsl import kernels as K
from tests.test_dsl_kernels import cases


def _to(dev, args):
    return tuple(a.clone().to(dev) if isinstance(a, torch.Tensor) else a for a in args)


# Written after the last GPU session of their author: emulated against torch (with the race check) and compiled for
# sm_100a in tests/test_dsl_kernels.py, to be added here once they have been launched on hardware.
EMULATED_AND_COMPILED_ONLY = {"paged_attention", "tiled_dequant_matmul_int4"}


@pytest.mark.parametrize("name", sorted(set(K.ALL) - EMULATED_AND_COMPILED_ONLY))
def test_launch_matches_emulation(name):
    kern, grid, block, args, checks = cases()[name]
    dev_args = _to("cuda", args)
    kern.launch(grid, block, dev_args)
    torch.cuda.synchronize()
    kern.emulate(grid, block, args)
    for host, _, atol in checks:                      # every output tensor: device result against the emulated one
        i = next(j for j, a in enumerate(args) if a is host)
        torch.testing.assert_close(dev_args[i].cpu().float(), host.float(), atol=max(atol, 1e-5), rtol=1e-3)


def test_prepacked_launch_and_graph_capture():
    """A prepacked launch captured in a CUDA graph replays on new data (the packed arguments keep their storage)."""
    a, b = torch.randn(300, device="cuda"), torch.randn(300, device="cuda")
    out = torch.zeros(300, device="cuda")
    pk = K.vector_add.prepack((a, b, out, 300))
    K.vector_add.launch_prepacked((5,), (64,), pk)
    torch.cuda.synchronize()
    torch.testing.assert_close(out, a + b)
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            K.vector_add.launch_prepacked((5,), (64,), pk)
    torch.cuda.current_stream().wait_stream(s)
    a.normal_()
    out.zero_()
    g.replay()
    torch.cuda.synchronize()
    torch.testing.assert_close(out, a + b)


def test_gpu_memory_and_profile():
    import zse_b200.dsl as zse
    mem = zse.GPUMemory()
    t = mem.allocate((64,), zse.float32) if hasattr(mem, "allocate") else None
    x = torch.randn(1 << 16, device="cuda")
    o = torch.zeros_like(x)
    r = K.silu.profile(((1 << 16) // 256,), (256,), (x, o, 1 << 16), nbytes=2 * 4 * (1 << 16))
    assert r.ms > 0 and r.launches > 0
    torch.testing.assert_close(o, torch.nn.functional.silu(x), atol=1e-5, rtol=1e-4)
