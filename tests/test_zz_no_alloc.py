"""bibo_moe_route_noalloc: the routing call for callers that cannot allocate device memory.

Some users of the library only own the buffers they were given -- a serving runtime that reserved
all device memory at start-up, or a loop where cudaMalloc's implicit synchronisation is not
allowed.  For them the library offers one routing call whose intermediates live in a fixed array
inside the library.  This test drives it through the C-ABI and checks it against the regular
routing call (bibo_moe_router_fwd, whose intermediates the caller allocates) on two calls in a
row with different inputs, so contents left in the shared array by the first call cannot leak
into the second.  Collected last on purpose: a failure here stops nothing else.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _call(lib, _lib, x, wr, bias, k, norm, scale):
    n, h = x.shape
    e = wr.shape[0]
    # outputs are allocated by the caller BEFORE the call; the call itself allocates nothing
    idx = torch.full((n, k), -1, dtype=torch.int32, device=DEV)
    w = torch.zeros(n, k, dtype=torch.float32, device=DEV)
    counts = torch.full((e,), -1, dtype=torch.int32, device=DEV)
    dt = _lib.BF16 if x.dtype == torch.bfloat16 else _lib.F32
    rc = lib.bibo_moe_route_noalloc(x.data_ptr(), wr.data_ptr(), bias.data_ptr(), n, h, e, k, norm, scale, dt,
                                    idx.data_ptr(), w.data_ptr(), counts.data_ptr(),
                                    torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "bibo_moe_route_noalloc")
    return idx, w, counts


@pytest.mark.parametrize("dtype,n,h,e,k", [(torch.bfloat16, 5000, 1024, 64, 6), (torch.float32, 777, 96, 22, 2)])
def test_route_noalloc_matches_router_fwd_twice(dtype, n, h, e, k):
    from bibo_b200 import _lib, functional as Fn
    lib = _lib.load()
    for call in range(2):                      # two calls in a row, different inputs and sizes
        g = torch.Generator().manual_seed(100 + call)
        nn = n - 300 * call
        x = torch.randn(nn, h, generator=g).to(dtype).to(DEV)
        wr = (torch.randn(e, h, generator=g) * 0.02).to(dtype).to(DEV)
        bias = ((torch.rand(e, generator=g) * 2 - 1) * 0.01).to(DEV)
        idx, w, counts = _call(lib, _lib, x, wr, bias, k, _lib.NORM_SUM, 1.0)
        ref_idx, ref_w, _, ref_bc, _ = Fn.router_forward(x, wr, bias, k, "sum")
        torch.cuda.synchronize()
        assert torch.equal(idx, ref_idx), "same kernel, same inputs: indices are bit-identical"
        assert torch.equal(w, ref_w), "weights are bit-identical"
        assert torch.equal(counts, ref_bc.sum(0).to(torch.int32))
        assert int(counts.sum()) == nn * k


def test_route_noalloc_refuses_oversized_batches():
    from bibo_b200 import _lib
    lib = _lib.load()
    n = int(lib.bibo_moe_route_noalloc_max_tokens()) + 1
    x = torch.zeros(n, 64, dtype=torch.bfloat16, device=DEV)
    wr = torch.zeros(64, 64, dtype=torch.bfloat16, device=DEV)
    bias = torch.zeros(64, device=DEV)
    idx = torch.zeros(n, 6, dtype=torch.int32, device=DEV)
    w = torch.zeros(n, 6, device=DEV)
    counts = torch.zeros(64, dtype=torch.int32, device=DEV)
    rc = lib.bibo_moe_route_noalloc(x.data_ptr(), wr.data_ptr(), bias.data_ptr(), n, 64, 64, 6, _lib.NORM_SUM, 1.0,
                                    _lib.BF16, idx.data_ptr(), w.data_ptr(), counts.data_ptr(), None)
    assert rc == -4 and b"exceed the fixed scratch" in lib.bibo_moe_last_error_string()


def test_route_noalloc_against_the_cpu_oracle_at_the_largest_layout():
    """The largest call the fixed array must hold (max tokens, 256 experts, top-8; CUDA-core router) against the
    CPU oracle's selection on the kernel's own fp32 logits path: histogram = bincount of the oracle's indices,
    except tokens at a last-bit near-tie; then the status word through its accessor, and an empty call."""
    from bibo_b200 import _lib
    from oracle import moe_oracle as orc
    lib = _lib.load()
    n, h, e, k = int(lib.bibo_moe_route_noalloc_max_tokens()), 64, 256, 8
    g = torch.Generator().manual_seed(9)
    x = torch.randn(n, h, generator=g)
    wr = torch.randn(e, h, generator=g) * 0.02
    bias = (torch.rand(e, generator=g) * 2 - 1) * 0.01
    idx, w, counts = _call(lib, _lib, x.to(DEV), wr.to(DEV), bias.to(DEV), k, _lib.NORM_SUM, 1.0)
    status = torch.full((1,), -1, dtype=torch.int32, device=DEV)
    _lib.check(lib.bibo_moe_route_noalloc_status(status.data_ptr(), torch.cuda.current_stream().cuda_stream), "status")
    torch.cuda.synchronize()
    assert int(status) == 0
    logits = orc.router_logits(x, wr)
    ref_idx, ref_w, ref_counts = orc.router_select(logits, bias, k)
    same = (idx.cpu().long() == ref_idx).all(-1)
    gap = orc.boundary_gap(logits, bias, k)
    assert bool((gap[~same] < 1e-5).all()), "a token may differ from the oracle only at a near-tie of the k-th score"
    assert float(same.float().mean()) > 0.999
    assert int((counts.cpu().long() - ref_counts).abs().sum()) <= 2 * int((~same).sum())
    assert float((w.cpu()[same] - ref_w[same]).abs().max()) < 1e-6
    # an empty call writes an all-zero histogram and touches nothing else
    counts.fill_(7)
    rc = lib.bibo_moe_route_noalloc(None, None, None, 0, h, e, k, _lib.NORM_SUM, 1.0, _lib.F32, None, None,
                                    counts.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(counts.abs().sum()) == 0
