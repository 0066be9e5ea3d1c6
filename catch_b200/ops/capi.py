"""ctypes mirror of the device library's C ABI (csrc/device/kernels_api.h).

Used by the kernel-level tests and benchmarks, which call a launcher with raw
device pointers (for example ``torch.cuda`` tensors' ``data_ptr()``) and compare
the result with a plain PyTorch fp32 reference.
"""
from __future__ import annotations

import ctypes as C

import torch

from .._loader import load_device_library

DT = {torch.uint8: 0, torch.int8: 1, torch.int16: 2, torch.int32: 3, torch.int64: 4, torch.float16: 5,
      torch.float32: 6, torch.float64: 7, torch.bool: 11, torch.bfloat16: 15}


class GemmParams(C.Structure):
    _fields_ = [
        ("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("batch", C.c_int),
        ("A", C.c_void_p), ("B", C.c_void_p), ("D", C.c_void_p),
        ("lda", C.c_int64), ("ldb", C.c_int64), ("ldd", C.c_int64),
        ("stride_a", C.c_int64), ("stride_b", C.c_int64), ("stride_d", C.c_int64),
        ("a_mn_major", C.c_int), ("b_mn_major", C.c_int),
        ("ab_dtype", C.c_int), ("d_dtype", C.c_int),
        ("bias", C.c_void_p), ("bias_dtype", C.c_int), ("bias_per_row", C.c_int),
        ("residual", C.c_void_p), ("ldr", C.c_int64), ("stride_r", C.c_int64), ("res_dtype", C.c_int),
        ("alpha", C.c_float), ("beta", C.c_float), ("act", C.c_int), ("tile_n", C.c_int), ("max_ctas", C.c_int),
        ("col_scale", C.c_void_p), ("batch_inner", C.c_int), ("stride_a2", C.c_int64), ("stride_b2", C.c_int64),
        ("stride_d2", C.c_int64), ("stride_r2", C.c_int64), ("accumulate", C.c_int), ("splits", C.c_int),
    ]


def lib() -> C.CDLL:
    l = load_device_library()
    if not getattr(l, "_catch_b200_typed", False):
        l.b200_gemm.argtypes = [C.POINTER(GemmParams), C.c_void_p]
        l.b200_gemm.restype = C.c_int
        l.b200_read_and_clear_error_flag.argtypes = [C.POINTER(C.c_int)]
        l.b200_read_and_clear_error_flag.restype = C.c_int
        l.b200_error_string.argtypes = [C.c_int]
        l.b200_error_string.restype = C.c_char_p
        l._catch_b200_typed = True
    return l


def check(rc: int, what: str = "kernel") -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed: {lib().b200_error_string(rc).decode()} ({rc})")


def read_error_flag() -> int:
    """The code recorded by a kernel whose bounded wait ran out (0 = none), cleared by the read.  Under host
    simulation no kernel runs: always 0."""
    if torch.b200.is_hostsim():
        return 0
    v = C.c_int(0)
    check(lib().b200_read_and_clear_error_flag(C.byref(v)), "read_error_flag")
    return v.value


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn_major=False, b_mn_major=False, bias=None, residual=None,
         alpha=1.0, beta=1.0, act=0, out_dtype=None, tile_n=0, bias_per_row=False, stream: int = 0) -> torch.Tensor:
    """D = act(alpha * A @ B^T + bias + beta * R) on the tcgen05 GEMM kernel.

    ``a`` is [M, K] (K-major) or [K, M] (MN-major) -- optionally with a leading
    batch dimension -- and ``b`` likewise [N, K] or [K, N]; both dense tensors
    of the same 16-bit (or fp32) dtype on a CUDA device.
    """
    batched = a.dim() == 3
    nb = a.shape[0] if batched else 1
    am, bm = a.shape[-2:], b.shape[-2:]
    M, K = (am[1], am[0]) if a_mn_major else (am[0], am[1])
    N, Kb = (bm[1], bm[0]) if b_mn_major else (bm[0], bm[1])
    assert K == Kb, (a.shape, b.shape)
    out_dtype = out_dtype or a.dtype
    d = torch.empty((nb, M, N) if batched else (M, N), dtype=out_dtype, device=a.device)
    p = GemmParams()
    p.M, p.N, p.K, p.batch = M, N, K, nb
    p.A, p.B, p.D = a.data_ptr(), b.data_ptr(), d.data_ptr()
    p.lda, p.ldb, p.ldd = a.stride(-2), b.stride(-2), N
    p.stride_a = a.stride(0) if batched else 0
    p.stride_b = b.stride(0) if batched else 0
    p.stride_d = M * N
    p.a_mn_major, p.b_mn_major = int(a_mn_major), int(b_mn_major)
    p.ab_dtype, p.d_dtype = DT[a.dtype], DT[out_dtype]
    if bias is not None:
        p.bias, p.bias_dtype, p.bias_per_row = bias.data_ptr(), DT[bias.dtype], int(bias_per_row)
    if residual is not None:
        p.residual, p.ldr, p.res_dtype = residual.data_ptr(), residual.stride(-2), DT[residual.dtype]
        p.stride_r = residual.stride(0) if residual.dim() == 3 else 0
    p.alpha, p.beta, p.act, p.tile_n = alpha, beta, act, tile_n
    check(lib().b200_gemm(C.byref(p), C.c_void_p(stream)), "b200_gemm")
    return d
