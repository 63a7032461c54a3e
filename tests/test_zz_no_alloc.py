"""sm_gemm_tc_static: the tensor-core product for callers that cannot allocate device memory
at the moment of the call (a plug-in inside another program's memory budget, a path that
must not meet cudaMalloc's device-wide synchronisation). Its split-K scratch is a fixed array
inside the library instead of a workspace from the caller. The test calls it through its
exported C symbol and compares it with the existing entry point, twice in a row on the same
array, checks that the calls leave the device's free memory as they found it, and that a
shape beyond the array is refused. It is collected last, so that a
run that stops at the first failure has already run every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
SCRATCH_BYTES = 4 << 20


def _rand(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).cuda()


def _ptr(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _static(lib, x, w, bias, out, mode=0, up_offset=0):
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    out_dt = 0 if out.dtype == torch.float32 else 1
    return lib.sm_gemm_tc_static(_ptr(x), _ptr(w), _ptr(bias), 1, _ptr(out), out_dt, x.shape[0], out.shape[1], x.shape[1],
                                 mode, up_offset, ctypes.c_void_p(0), stream)


def test_static_scratch_entry_point_matches_the_allocating_one():
    from smolmoe_c99_b200.kernels import get_ops
    ops = get_ops()
    lib = ops.lib
    lib.sm_gemm_tc_static.restype = ctypes.c_int
    lib.sm_gemm_tc_static_error.restype = ctypes.c_int
    # shapes whose reduction is split over more CTAs than a cluster holds, which exchange their sums through global
    # memory, so that the scratch is really used (a few tokens over a long K and few row tiles; up to 8 splits are the
    # CTAs of a cluster and need none)
    cases = [(16, 896, 4864, 0), (10, 640, 4096, 0), (12, 160, 4096, 2)]
    for round_ in range(2):                       # two calls in a row per shape: the array is shared and never cleared
        for T, N, K, mode in cases:
            need = int(lib.sm_gemm_tc_workspace_bytes(T, N, K, int(mode == 2)))
            assert 0 < need <= SCRATCH_BYTES, (T, N, K, need)
            x = _rand((T, K), 10 * round_ + T)
            w = _rand(((2 if mode == 2 else 1) * N, K), 20 * round_ + N, 0.05)
            bias = None if mode == 2 else _rand((N,), 3)
            want = torch.empty((T, N), dtype=torch.bfloat16 if mode == 2 else torch.float32, device="cuda")
            ops.gemm_tc(x, w, bias, want, mode=mode, up_offset=N if mode == 2 else 0)
            got = torch.full_like(want, float("nan"))
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
            status = _static(lib, x, w, bias, got, mode, N if mode == 2 else 0)
            assert status == 0, lib.sm_last_error().decode()
            torch.cuda.synchronize()
            if round_ == 1:
                # what the entry point is for: after a device's first call, a call takes no memory from the device
                # (the first call of all may load the library's module and with it the array)
                assert torch.cuda.mem_get_info()[0] == free_before, (T, N, K)
            ref = x.float() @ w[:N].float().T
            if mode == 2:
                up = x.float() @ w[N:].float().T
                ref = up * (ref / (1 + torch.exp(-ref)))
            else:
                ref = ref + bias.float()
            tol = 1e-3 * (K ** 0.5) * 0.05 + (0.0 if got.dtype == torch.float32 else 8e-3 * float(ref.abs().max()))
            assert float((got.float() - want.float()).abs().max()) <= tol       # the tolerance of the kernel's own test
            assert float((got.float() - ref).abs().max()) <= tol
    assert lib.sm_gemm_tc_static_error() == 0
    ops.check_error_flag()


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from smolmoe_c99_b200.kernels import get_ops
    lib = get_ops().lib
    lib.sm_gemm_tc_static.restype = ctypes.c_int
    N, K = 512, 4864                                          # a gated product: two accumulators, K split several ways
    sizes = {T: int(lib.sm_gemm_tc_workspace_bytes(T, N, K, 1)) for T in (200, 256, 300)}
    too_big = [T for T, need in sizes.items() if need > SCRATCH_BYTES]
    assert too_big, f"no shape of this family exceeds the array: {sizes}"
    T, need = too_big[0], sizes[too_big[0]]
    x, w = _rand((T, K), 1), _rand((2 * N, K), 2, 0.05)
    out = torch.zeros((T, N), dtype=torch.bfloat16, device="cuda")
    assert _static(lib, x, w, None, out, 2, N) == 1
    message = lib.sm_last_error().decode()
    assert str(need) in message and str(SCRATCH_BYTES) in message
    assert _static(lib, x[:0], w, None, out[:0], 2, N) == 1 and "must be positive" in lib.sm_last_error().decode()
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0                      # nothing ran
    assert _static(lib, x[:8].contiguous(), w, None, out[:8].contiguous(), 2, N) == 0   # the next call still works
