"""The allocation-free entry point, called through its exported C symbol, must agree with the regular
add_rmsnorm backward on two consecutive calls (the second with other sizes, so contents left in the library's
internal array by the first call would show up as an error).  Collected last on purpose."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(a, b, atol=1e-3, rtol=3e-2):
    a, b = a.float(), b.float()
    assert ((a - b).abs() <= atol + rtol * b.abs()).all(), f"max err {(a - b).abs().max().item():.4e}"


def _reference(res, w, dout, dres, eps):
    """existing entry point: partial sums in a caller-allocated buffer, reduced by the caller"""
    from state_space_models_neuron_b200.ops import native
    lib = native.lib()
    rows, D = res.shape
    slices = min(rows, 296)
    part = torch.empty(slices, D, dtype=torch.float32, device="cuda")
    dsum = torch.empty_like(res)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    fn = lib.ssm_add_rmsnorm_bwd
    fn.restype = ctypes.c_int
    code = fn(ctypes.c_void_p(res.data_ptr()), ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(dout.data_ptr()),
              ctypes.c_void_p(dres.data_ptr()), ctypes.c_void_p(dsum.data_ptr()), ctypes.c_void_p(part.data_ptr()),
              slices, ctypes.c_longlong(rows), D, ctypes.c_float(eps), int(res.dtype == torch.float32), st)
    assert code == 0
    return dsum, part.sum(0)


def _noalloc(res, w, dout, dres, eps):
    from state_space_models_neuron_b200.ops import native
    lib = native.lib()
    rows, D = res.shape
    dsum = torch.empty_like(res)
    dw = torch.full((D,), float("nan"), dtype=torch.float32, device="cuda")
    fn = lib.ssm_add_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    code = fn(ctypes.c_void_p(res.data_ptr()), ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(dout.data_ptr()),
              ctypes.c_void_p(dres.data_ptr()), ctypes.c_void_p(dsum.data_ptr()), ctypes.c_void_p(dw.data_ptr()),
              ctypes.c_longlong(rows), D, ctypes.c_float(eps), int(res.dtype == torch.float32), st)
    return code, dsum, dw


def _fp32_reference(res, w, dout, dres, eps):
    """plain PyTorch in fp32: gradient of rmsnorm(res) * w with respect to res (plus the incoming residual gradient)
    and to w"""
    x = res.float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * wf
    y.backward(dout.float())
    return x.grad + dres.float(), wf.grad


def test_no_alloc_entry_point_matches_regular_one_twice():
    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda").manual_seed(11)
    for rows, D, dtype in [(1000, 4096, torch.bfloat16), (37, 1024, torch.float32)]:
        res = torch.randn(rows, D, device="cuda", generator=g).to(dtype)
        dres = torch.randn(rows, D, device="cuda", generator=g).to(dtype)
        dout = torch.randn(rows, D, device="cuda", generator=g).bfloat16()
        w = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).bfloat16()
        ref_dsum, ref_dw = _reference(res, w, dout, dres, 1e-5)
        code, dsum, dw = _noalloc(res, w, dout, dres, 1e-5)
        torch.cuda.synchronize()
        assert code == 0
        _close(dsum, ref_dsum)
        _close(dw, ref_dw, atol=1e-3 * max(1.0, ref_dw.abs().max().item()))
        # and against fp32 PyTorch (dsum is rounded to the residual's dtype by the kernel)
        o_dsum, o_dw = _fp32_reference(res, w, dout, dres, 1e-5)
        _close(dsum, o_dsum, atol=2e-2, rtol=2e-2)
        _close(dw, o_dw, atol=2e-3 * max(1.0, o_dw.abs().max().item()), rtol=2e-2)


def test_no_alloc_entry_point_rejects_oversize():
    torch.cuda.set_device(0)
    D = 8192 + 8
    res = torch.zeros(2, D, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(D, device="cuda", dtype=torch.bfloat16)
    code, _, _ = _noalloc(res, w, res, res, 1e-5)
    assert code == -4


def test_no_alloc_entry_point_rejects_misaligned_pointers():
    """A row pointer that is not 16-byte aligned must come back as a bad-argument code; nothing is launched."""
    from state_space_models_neuron_b200.ops import native
    torch.cuda.set_device(0)
    lib = native.lib()
    fn = lib.ssm_add_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    rows, D = 4, 256
    buf = torch.zeros(rows * D + 8, device="cuda", dtype=torch.bfloat16)
    ok = buf[:rows * D]
    odd = buf[1:rows * D + 1]                      # starts 2 bytes past a 16-byte boundary
    w = torch.ones(D, device="cuda", dtype=torch.bfloat16)
    dw = torch.zeros(D, device="cuda", dtype=torch.float32)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def call(res, dout, dsum):
        return fn(ctypes.c_void_p(res.data_ptr()), ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(dout.data_ptr()),
                  ctypes.c_void_p(0), ctypes.c_void_p(dsum.data_ptr()), ctypes.c_void_p(dw.data_ptr()),
                  ctypes.c_longlong(rows), D, ctypes.c_float(1e-5), 0, st)

    out = torch.zeros(rows * D, device="cuda", dtype=torch.bfloat16)
    assert call(odd, ok, out) == -3
    assert call(ok, odd, out) == -3
    assert call(ok, ok, odd) == -3
