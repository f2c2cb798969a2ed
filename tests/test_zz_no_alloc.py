"""The allocation-free normalisation backward, called through its exported C symbol.

Some callers of the library may not allocate device memory when they call it (for instance a
serving loop inside a host runtime that owns all device memory, or a plugin interface that only
hands over input and output buffers).  For them the library exports ``fm_norm_bwd_static``, which
keeps its partial sums in a scratch array inside the library image instead of a per-call buffer.
This test loads the shared object with ctypes, calls the symbol twice in a row with different
inputs, and checks each result against the regular entry point.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from fluidmoe_b200 import build as b
    lib = ctypes.CDLL(str(b.target_path()))
    fn = lib.fm_norm_bwd_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 9 + [ctypes.c_int] * 3 + [ctypes.c_void_p]
    lib.fm_last_error.restype = ctypes.c_char_p
    return lib, fn


@pytest.mark.parametrize("kind", ["layernorm", "rmsnorm"])
def test_norm_bwd_static_matches_regular_entry_point(kind):
    from fluidmoe_b200.ops import norm

    lib, fn = _lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream().cuda_stream
    for call, (T, H) in enumerate([(777, 4096), (64, 1024), (300, 8192), (5, 8)]):   # calls in a row share the scratch;
        # the largest width with more rows than blocks, and the smallest width
        torch.manual_seed(10 + call)
        x = torch.randn(T, H, device=dev).bfloat16()
        w = (1 + 0.1 * torch.randn(H, device=dev)).bfloat16()
        b = (0.1 * torch.randn(H, device=dev)).bfloat16() if kind == "layernorm" else None
        dy = torch.randn(T, H, device=dev).bfloat16()
        rg = torch.randn(T, H, device=dev).bfloat16()
        _, mean, rstd = norm.norm_fwd(x, w, b, 1e-5, kind)
        ref_dx, ref_dw, ref_db = norm.norm_bwd(dy, x, w, mean, rstd, kind, b is not None, rg)
        dx = torch.empty_like(x)
        dw = torch.empty(H, dtype=torch.float32, device=dev)
        db = torch.empty(H, dtype=torch.float32, device=dev) if b is not None else None
        rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), mean.data_ptr() if mean is not None else None,
                rstd.data_ptr(), rg.data_ptr(), dx.data_ptr(), dw.data_ptr(),
                db.data_ptr() if db is not None else None, T, H, 0 if kind == "layernorm" else 1, stream)
        assert rc == 0, lib.fm_last_error()
        torch.cuda.synchronize()

        def close(a, b_, tol=2e-2):
            err = (a.float() - b_.float()).abs().max().item()
            assert err <= tol * (b_.float().abs().max().item() + 1e-6), err
        close(dx, ref_dx)
        close(dw, ref_dw)
        if db is not None:
            close(db, ref_db)


def test_norm_bwd_static_rejects_sizes_beyond_the_scratch():
    lib, fn = _lib()
    torch.cuda.set_device(0)
    rc = fn(None, None, None, None, None, None, None, None, None, 16, 8192 + 8, 1, None)
    assert rc != 0
    assert b"not supported" in lib.fm_last_error()
    rc = fn(None, None, None, None, None, None, None, None, None, 0, 1024, 1, None)
    assert rc != 0
    assert b"at least one row" in lib.fm_last_error()
