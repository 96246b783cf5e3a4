"""Host-side choices of the native library that need no GPU: the K split of accumulating GEMMs and the
number of copy drivers of the fused all-gather kernels."""
import ctypes

import pytest

from kareus_b200.kernels import build


def _lib():
    if not build.LIB.exists():
        pytest.skip("native library not built")
    L = ctypes.CDLL(str(build.LIB))
    L.kb_gemm_accum_plan.argtypes = [ctypes.c_int] * 4 + [ctypes.POINTER(ctypes.c_int)] * 2
    L.kb_gemm_accum_plan.restype = None
    return L


def _plan(L, n_out, n_in, tokens, sms=148):
    tile, ks = ctypes.c_int(), ctypes.c_int()
    L.kb_gemm_accum_plan(n_out, n_in, tokens, sms, ctypes.byref(tile), ctypes.byref(ks))
    return tile.value, ks.value


def test_weight_gradients_with_few_tiles_split_k():
    L = _lib()
    tokens = 16384
    # TP8 shards of a 3B Llama layer: 36-96 tiles for 148 SMs → more than one CTA per tile
    for n_out, n_in in [(640, 3072), (3072, 384), (2048, 3072), (3072, 1024)]:
        tile, ks = _plan(L, n_out, n_in, tokens)
        assert tile in (128, 256) and 2 <= ks <= 8, (n_out, n_in, tile, ks)
    # the LM head has thousands of tiles: no split
    assert _plan(L, 128256, 3072, tokens) == (256, 1)
    # a split never leaves fewer than eight 64-deep K steps per part
    for k in (512, 1024, 2048):
        _, ks = _plan(L, 640, 3072, k)
        assert ks == 1 or (k // 64) // ks >= 8
    # the choice follows the number of SMs given to the GEMM
    assert _plan(L, 2048, 3072, tokens, sms=32)[1] <= _plan(L, 2048, 3072, tokens, sms=148)[1]


def test_copy_driver_count_scales_with_output_width_and_budget():
    from kareus_b200.ops.fused import FusedAGGemm as F
    assert F.auto_drivers(12, 640) == 36 and F.auto_drivers(12, 1024) == 24 and F.auto_drivers(12, 2048) == 12
    # a kernel confined to 72 SMs keeps two thirds of them for the GEMM
    assert F.auto_drivers(12, 640, 72) == 24 and F.auto_drivers(12, 2048, 72) == 12
    # a plan's own number is never lowered by the cap
    assert F.auto_drivers(40, 4096, 72) == 40
