"""The allocation-free RMSNorm backward: called through its exported C symbol, twice in a row,
and compared with the regular entry point (which takes scratch memory from the caller).

Callers that cannot allocate — a frozen memory pool, a host that sizes device memory up front, a
binding without an allocator — use this symbol; the test does the same: ctypes, raw pointers."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_noalloc_matches_regular_entry_point_twice():
    from kareus_b200.kernels import cuda as KC
    lib = ctypes.CDLL(str(KC.LIB_PATH))
    fn = lib.kb_rmsnorm_bwd_noalloc
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    stream = torch.cuda.current_stream().cuda_stream
    for call, (rows, H) in enumerate([(777, 3072), (64, 8192)]):
        x = torch.randn(rows, H, device="cuda").bfloat16()
        w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16()
        dy = torch.randn(rows, H, device="cuda").bfloat16()
        _, rstd = KC.rmsnorm_fwd(x, w, 1e-5)
        dx_ref, dw_ref = KC.rmsnorm_bwd(dy, x, rstd, w)
        dx = torch.empty_like(x)
        dw = torch.empty(H, device="cuda", dtype=torch.float32)
        rc = fn(dy.data_ptr(), x.data_ptr(), rstd.data_ptr(), w.data_ptr(), dx.data_ptr(), dw.data_ptr(), rows, H,
                stream)
        assert rc == 0, f"call {call} returned {rc}"
        torch.cuda.synchronize()
        torch.testing.assert_close(dx, dx_ref)                          # same kernel, same row order
        rel = ((dw - dw_ref).norm() / dw_ref.norm()).item()
        assert rel < 5e-3, rel                                          # partial sums grouped differently
    # sizes beyond the built-in array are refused without launching anything
    assert fn(0, 0, 0, 0, 0, 0, 16, 16384, stream) == 7
    assert fn(0, 0, 0, 0, 0, 0, 16, 256, stream) == 7
