"""The allocation-free norm backward (``sb200_norm_bwd_noalloc``), called through its exported C symbol.

It is for hosts that cannot give the library a workspace - a server whose device memory was committed at
start-up, or a plain C program without a tensor allocator.  The test calls the symbol with ctypes exactly as such
a host would (raw pointers, a stream handle), twice in a row because all calls share one built-in workspace, and
compares against the regular entry point that takes caller-provided workspaces.
"""

import ctypes
from ctypes import c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbols():
    from scaling_b200.ops import _build

    handle = ctypes.CDLL(str(_build.build()))
    noalloc = handle.sb200_norm_bwd_noalloc
    noalloc.argtypes = [c_void_p] * 8 + [c_int] * 5 + [c_void_p]
    noalloc.restype = c_int
    regular = handle.sb200_norm_bwd
    regular.argtypes = [c_void_p] * 10 + [c_int] * 6 + [c_void_p]
    regular.restype = c_int
    rows = handle.sb200_norm_bwd_partial_rows
    rows.argtypes = [c_int, c_int]
    rows.restype = c_int
    return noalloc, regular, rows


def _problem(M, H, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(M, H, device="cuda", dtype=dtype, generator=g)
    dy = torch.randn(M, H, device="cuda", dtype=dtype, generator=g)
    w = (torch.rand(H, device="cuda", generator=g) + 0.5).to(dtype)
    xf = x.float()
    mean = xf.mean(-1)
    rstd = torch.rsqrt(xf.var(-1, unbiased=False) + 1e-5)
    rstd_rms = torch.rsqrt(xf.pow(2).mean(-1) + 1e-5)
    return x, dy, w, mean.contiguous(), rstd.contiguous(), rstd_rms.contiguous()


@pytest.mark.parametrize("rms", [1, 0])
@pytest.mark.parametrize("dtype,code", [(torch.bfloat16, 1), (torch.float32, 0)])
def test_noalloc_matches_regular_entry_point_twice(rms, dtype, code):
    noalloc, regular, partial_rows = _symbols()
    stream = torch.cuda.current_stream().cuda_stream
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    # two different problems back to back: the second call must not see leftovers of the first in the workspace
    for seed, (M, H) in enumerate([(517, 4096), (64, 768)]):
        x, dy, w, mean, rstd_ln, rstd_rms = _problem(M, H, dtype, seed)
        rstd = rstd_rms if rms else rstd_ln
        out = {}
        for name in ("noalloc", "regular"):
            dx = torch.empty_like(x)
            dw = torch.empty(H, device="cuda", dtype=dtype)
            db = torch.empty(H, device="cuda", dtype=dtype)
            if name == "noalloc":
                rc = noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                             dw.data_ptr(), None if rms else db.data_ptr(), M, H, rms, 0, code, stream)
            else:
                rows = partial_rows(M, sms)
                dwp = torch.empty(rows, H, device="cuda", dtype=torch.float32)
                dbp = torch.empty(rows, H, device="cuda", dtype=torch.float32)
                rc = regular(dy.data_ptr(), x.data_ptr(), w.data_ptr(), mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                             dwp.data_ptr(), None if rms else dbp.data_ptr(), dw.data_ptr(),
                             None if rms else db.data_ptr(), M, H, rms, 0, rows, code, stream)
            assert rc == 0, f"{name} returned {rc}"
            torch.cuda.synchronize()
            out[name] = (dx, dw, None if rms else db)
        tol = 2e-2 if dtype != torch.float32 else 1e-5
        for a, b in zip(out["noalloc"], out["regular"]):
            if a is None:
                continue
            rel = ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()
            assert rel < tol, rel
        # dx does not depend on the partial-row count, only on the order of the per-row sums, which may differ
        # between the block-per-row kernel of this entry point and the kernel the regular entry point picks
        assert torch.allclose(out["noalloc"][0].float(), out["regular"][0].float(), rtol=tol, atol=tol)


def test_noalloc_rejects_oversized_rows():
    noalloc, _, _ = _symbols()
    H = 16384  # beyond SB200_NOALLOC_MAX_H
    x = torch.zeros(4, H, device="cuda", dtype=torch.bfloat16)
    v = torch.zeros(H, device="cuda", dtype=torch.bfloat16)
    r = torch.ones(4, device="cuda")
    rc = noalloc(x.data_ptr(), x.data_ptr(), v.data_ptr(), None, r.data_ptr(), x.data_ptr(), v.data_ptr(), None, 4, H,
                 1, 0, 1, torch.cuda.current_stream().cuda_stream)
    assert rc == 103  # SB_ERR_TOO_LARGE


def test_noalloc_refuses_misaligned_pointers_before_any_launch():
    noalloc, _, _ = _symbols()
    H = 256
    x = torch.zeros(4 * H + 8, device="cuda", dtype=torch.bfloat16)
    v = torch.zeros(H, device="cuda", dtype=torch.bfloat16)
    r = torch.ones(4, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    torch.cuda.synchronize()
    # dx two bytes off a 16-byte boundary: refused on the host (SB_ERR_BAD_ARG), so no kernel ever sees the pointer
    rc = noalloc(x.data_ptr(), x.data_ptr(), v.data_ptr(), None, r.data_ptr(), x.data_ptr() + 2, v.data_ptr(), None, 4,
                 H, 1, 0, 1, stream)
    assert rc == 102
    torch.cuda.synchronize()  # the context is untouched
