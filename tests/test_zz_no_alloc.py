"""LayerNorm backward without caller-provided scratch (ptj_layernorm_bwd_noalloc).

Some users of the library cannot allocate device memory: their process gave the whole GPU to another allocator up
front, or their step must not touch the driver's allocation path. This entry point keeps its partial sums in a fixed
array inside the library instead. The test calls it through the C ABI twice in a row (the array keeps the previous
call's contents, so the second call checks that stale data does no harm) and compares with the regular entry point.
The file name makes pytest collect it last.
"""
import ctypes

import pytest
import torch

from conftest import pkg

pytestmark = pytest.mark.gpu


def _run(lib, fn_noalloc, dy, x, gamma, dx_add):
    rows, dim = x.shape
    dt = 1 if x.dtype == torch.bfloat16 else 0
    st = torch.cuda.current_stream().cuda_stream
    out = {}
    for name in ("regular", "noalloc"):
        dx = torch.empty_like(x)
        dg = torch.empty(dim, device="cuda")
        db = torch.empty(dim, device="cuda")
        if name == "regular":
            n = lib.ptj_layernorm_bwd_scratch_floats(rows, dim)
            scratch = torch.empty(n, device="cuda")
            rc = lib.ptj_layernorm_bwd(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), dx_add.data_ptr(), dx.data_ptr(),
                                       dg.data_ptr(), db.data_ptr(), scratch.data_ptr(), n, rows, dim, dt, st)
        else:
            rc = fn_noalloc(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), dx_add.data_ptr(), dx.data_ptr(),
                            dg.data_ptr(), db.data_ptr(), rows, dim, dt, st)
        assert rc == 0, lib.ptj_status_string(rc)
        out[name] = (dx, dg, db)
    torch.cuda.synchronize()
    return out


def test_matches_regular_entry_point_twice_in_a_row():
    lib = pkg("_lib").lib()
    fn = lib.ptj_layernorm_bwd_noalloc
    g = torch.Generator().manual_seed(0)
    # two different problems back to back: the second one finds the first one's partial sums in the shared array
    for rows, dim, dtype in ((4096, 768, torch.bfloat16), (300, 1000, torch.float32)):
        x = torch.randn(rows, dim, generator=g).to(dtype).cuda()
        dy = torch.randn(rows, dim, generator=g).to(dtype).cuda()
        res = torch.randn(rows, dim, generator=g).to(dtype).cuda()
        gamma = (1 + 0.1 * torch.randn(dim, generator=g)).cuda()
        out = _run(lib, fn, dy, x, gamma, res)
        for a, b in zip(out["regular"], out["noalloc"]):
            tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
            denom = float(a.float().abs().max())
            assert float((a.float() - b.float()).abs().max()) <= tol * denom
            assert torch.equal(a, b), "same kernels, same grid: the two entry points agree bit for bit"


def test_rejects_sizes_beyond_the_fixed_capacity():
    lib = pkg("_lib").lib()
    cap = lib.ptj_layernorm_bwd_noalloc_max_dim()
    assert cap == 2048
    x = torch.zeros(4, cap + 8, device="cuda")
    g = torch.ones(cap + 8, device="cuda")
    rc = lib.ptj_layernorm_bwd_noalloc(x.data_ptr(), x.data_ptr(), g.data_ptr(), None, x.data_ptr(), g.data_ptr(),
                                       g.data_ptr(), 4, cap + 8, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == -9 and b"capacity" in lib.ptj_status_string(rc)


def test_optional_outputs_empty_input_and_the_capacity_edge():
    """dgamma / dbeta may be left out (no partial sums are needed then), zero rows are legal, and the widest row the
    fixed array is sized for (dim 2048, every block of the grid in use) matches the regular entry point bit for bit."""
    lib = pkg("_lib").lib()
    fn = lib.ptj_layernorm_bwd_noalloc
    st = torch.cuda.current_stream().cuda_stream
    g = torch.Generator().manual_seed(1)
    rows, dim = 600, 768
    x = torch.randn(rows, dim, generator=g).bfloat16().cuda()
    dy = torch.randn(rows, dim, generator=g).bfloat16().cuda()
    gamma = (1 + 0.1 * torch.randn(dim, generator=g)).cuda()
    full = _run(lib, fn, dy, x, gamma, torch.zeros_like(x))["noalloc"][0]
    dx = torch.empty_like(x)
    assert fn(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), None, dx.data_ptr(), None, None, rows, dim, 1, st) == 0
    torch.cuda.synchronize()
    assert torch.equal(dx, full), "leaving out the parameter gradients must not change dx"
    # zero rows: nothing to read, parameter gradients are zero
    dg, db = torch.full((dim,), 3.0, device="cuda"), torch.full((dim,), 3.0, device="cuda")
    assert fn(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), None, dx.data_ptr(), dg.data_ptr(), db.data_ptr(), 0, dim, 1, st) == 0
    torch.cuda.synchronize()
    assert float(dg.abs().max()) == 0.0 and float(db.abs().max()) == 0.0
    # dim at the capacity, enough rows to occupy every block of the grid
    cap = int(lib.ptj_layernorm_bwd_noalloc_max_dim())
    rows = 8 * 148 * 2 + 5
    x = torch.randn(rows, cap, generator=g).bfloat16().cuda()
    dy = torch.randn(rows, cap, generator=g).bfloat16().cuda()
    gamma = (1 + 0.1 * torch.randn(cap, generator=g)).cuda()
    out = _run(lib, fn, dy, x, gamma, torch.zeros_like(x))
    for a, b in zip(out["regular"], out["noalloc"]):
        assert torch.equal(a, b)
