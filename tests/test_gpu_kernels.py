"""Each kernel alone against a plain float32 computation in PyTorch, at sizes other than
the engine's tiny configurations (widths and vocabularies that are no power of two, head
sizes in steps of 16, ragged tiles)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from smolmoe_c99_b200.kernels import get_ops
    return get_ops()


def _rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).cuda()


@pytest.mark.parametrize("T,N,K", [(1, 896, 896), (8, 1152, 896), (64, 896, 4864), (3, 100, 72), (130, 300, 200),
                                   (2048, 896, 896), (500, 1000, 136), (17, 128, 64), (256, 256, 8)])
@pytest.mark.parametrize("mode", ["store_f32", "store_bf16", "accumulate"])
def test_gemm_tc(ops, T, N, K, mode):
    x, w = _rand((T, K), torch.bfloat16, 1), _rand((N, K), torch.bfloat16, 2, 0.05)
    bias = _rand((N,), torch.bfloat16, 3)
    want = x.float() @ w.float().T
    if mode == "accumulate":
        out = _rand((T, N), torch.float32, 4)
        want = want + out
        ops.gemm_tc(x, w, None, out, mode=1)
    else:
        out = torch.empty((T, N), dtype=torch.float32 if mode == "store_f32" else torch.bfloat16, device="cuda")
        want = want + bias.float()
        ops.gemm_tc(x, w, bias, out, mode=0)
    ops.check_error_flag()
    tol = 1e-3 * math.sqrt(K) * 0.05 + (0.0 if out.dtype == torch.float32 else 8e-3 * float(want.abs().max()))
    assert float((out.float() - want).abs().max()) <= tol


@pytest.mark.parametrize("T,H,K", [(1, 4864, 896), (8, 4864, 896), (64, 160, 96), (300, 520, 264), (2048, 1024, 128)])
def test_gemm_tc_gated(ops, T, H, K):
    x, w = _rand((T, K), torch.bfloat16, 5), _rand((2 * H, K), torch.bfloat16, 6, 0.05)
    g, u = x.float() @ w[:H].float().T, x.float() @ w[H:].float().T
    want = u * (g / (1 + torch.exp(-g)))
    out = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")
    ops.gemm_tc(x, w, None, out, mode=2, up_offset=H)
    ops.check_error_flag()
    assert float((out.float() - want).abs().max()) <= 8e-3 * float(want.abs().max()) + 1e-3


def test_gemm_tc_refuses_unaligned_k(ops):
    from smolmoe_c99_b200.kernels import KernelError
    x, w = _rand((4, 100), torch.bfloat16, 1), _rand((16, 100), torch.bfloat16, 2)
    with pytest.raises(KernelError, match="multiple of 8"):
        ops.gemm_tc(x, w, None, torch.empty((4, 16), dtype=torch.float32, device="cuda"))
    # the dispatcher takes the CUDA-core kernel for it instead
    got = ops.linear(x, w, None, out_dtype=torch.float32)
    assert float((got - x.float() @ w.float().T).abs().max()) < 1e-3


@pytest.mark.parametrize("xd,wd,od", [(torch.float32, torch.float32, torch.float32),
                                      (torch.bfloat16, torch.bfloat16, torch.float32),
                                      (torch.bfloat16, torch.float32, torch.bfloat16)])
@pytest.mark.parametrize("T,N,K", [(1, 70, 50), (65, 129, 33), (200, 64, 1000)])
def test_gemm_simt(ops, xd, wd, od, T, N, K):
    x, w, b = _rand((T, K), xd, 1), _rand((N, K), wd, 2, 0.05), _rand((N,), wd, 3)
    want = x.float() @ w.float().T + b.float()
    out = ops.gemm_simt(x, w, b, torch.empty((T, N), dtype=od, device="cuda"))
    tol = 2e-5 if od == torch.float32 else 8e-3 * float(want.abs().max())
    assert float((out.float() - want).abs().max()) <= tol
    # each output is one chain over k: more rows in the batch change no bit
    alone = ops.gemm_simt(x[:1].contiguous(), w, b, torch.empty((1, N), dtype=od, device="cuda"))
    assert torch.equal(alone[0], out[0])
