"""The public kernel callables (`XXT`, `ba_plus_cAA`, `fused_bmm_add`, `ns5_smem`) and the symmetric-output mode of
the GEMM behind the first two, against fp32 PyTorch.  Follows the reference's tests/integration/test_kernels.py:
building blocks at atol = rtol = 1e-2 on unit-scale data, boundary shapes that are not multiples of any tile size,
2-D and 3-D inputs, imported through the reference's module path."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _check(out, ref, atol=1e-2, rtol=1e-2):
    err = (out.float() - ref.float()).abs()
    tol = atol + rtol * ref.float().abs()
    assert bool((err <= tol).all()), f"max err {err.max().item():.4g} (ref max {ref.abs().max().item():.4g})"


def _unit_rows(*shape, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(*shape, generator=g)
    return (x / x.norm(dim=-1, keepdim=True)).cuda().bfloat16()


@pytest.mark.parametrize("shape", [(4, 256, 512), (3, 512, 512), (2, 1024, 256), (2, 384, 128), (640, 320), (1, 1024, 1024),
                                   (4, 100, 70), (2, 50, 130), (3, 200, 100), (2, 520, 264)])
def test_xxt_matches_torch_and_is_exactly_symmetric(shape):
    from himuon.triton_kernels import XXT
    from himuon_b200 import ops

    A = _unit_rows(*shape)
    M = A.shape[-2]
    out = torch.full((*A.shape[:-2], M, M), float("nan"), device="cuda", dtype=torch.bfloat16)
    XXT(A, out)
    torch.cuda.synchronize()
    ops.check_status()
    _check(out, A.float() @ A.float().transpose(-2, -1))
    assert torch.equal(out, out.transpose(-2, -1)), "mirrored tiles differ from the computed ones"


@pytest.mark.parametrize("shape", [(4, 256, 256), (3, 512, 512), (2, 1024, 1024), (384, 384), (2, 130, 130), (3, 200, 200),
                                   (2, 776, 776)])
def test_ba_plus_caa_matches_torch(shape):
    from himuon.triton_kernels import ba_plus_cAA
    from himuon_b200 import ops

    X = _unit_rows(*shape, seed=1)
    A = (X.float() @ X.float().transpose(-2, -1)).bfloat16()
    A = torch.tril(A) + torch.tril(A, -1).transpose(-2, -1)          # exactly symmetric input
    out = torch.full_like(A, float("nan"))
    ba_plus_cAA(A, 2.0315, -4.7750, out)
    torch.cuda.synchronize()
    ops.check_status()
    ref = 2.0315 * (A.float() @ A.float().transpose(-2, -1)) - 4.7750 * A.float()
    _check(out, ref, atol=2e-2, rtol=1e-2)
    assert torch.equal(out, out.transpose(-2, -1))


@pytest.mark.parametrize("shape", [(4, 100, 70), (2, 50, 130), (3, 200, 100), (2, 256, 512), (1, 512, 1024)])
def test_fused_bmm_add_boundaries(shape):
    from himuon.triton_kernels import fused_bmm_add
    from himuon_b200 import ops

    Bt, M, N = shape
    B = _unit_rows(Bt, M, M, seed=2)
    X = _unit_rows(Bt, M, N, seed=3)
    out = fused_bmm_add(B, X, 3.4445)
    out2 = torch.full_like(X, float("nan"))
    assert fused_bmm_add(B, X, 3.4445, out=out2) is out2
    torch.cuda.synchronize()
    ops.check_status()
    ref = torch.bmm(B.float(), X.float()).bfloat16().float() + 3.4445 * X.float()
    _check(out, ref, atol=2e-2, rtol=1e-2)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_fused_bmm_add_other_dtypes_use_the_torch_path(dtype):
    from himuon.triton_kernels import fused_bmm_add

    B = torch.randn(2, 64, 64, device="cuda", dtype=dtype) / 8
    X = torch.randn(2, 64, 96, device="cuda", dtype=dtype)
    out = fused_bmm_add(B, X, 0.5)
    assert out.dtype == dtype
    _check(out, torch.bmm(B.float(), X.float()) + 0.5 * X.float(), atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("shape", [(8, 128, 128), (5, 64, 256), (3, 16, 1024), (4, 32, 512), (6, 16, 16), (128, 128), (2, 64, 64)])
def test_ns5_smem_matches_the_oracle_on_well_conditioned_tiles(shape):
    from himuon.triton_kernels import ns5_smem
    from himuon_b200 import ops
    from himuon_b200.ops import reference as ref

    g = torch.Generator().manual_seed(4)
    x = torch.randn(*shape, generator=g)
    U, _, Vh = torch.linalg.svd(x, full_matrices=False)
    x = ((U * torch.linspace(0.8, 1.2, min(shape[-2:]))) @ Vh).bfloat16()
    out = ns5_smem(x.cuda())
    out_p = ns5_smem(x.cuda(), persistent=True)
    torch.cuda.synchronize()
    ops.check_status()
    assert out.shape == x.shape and out.dtype == torch.bfloat16 and out.data_ptr() != x.data_ptr()
    want = ref.newton_schulz(x if x.dim() == 3 else x.unsqueeze(0), 5).reshape(x.shape)
    _check(out.cpu(), want, atol=4e-2, rtol=4e-2)
    assert torch.equal(out, out_p)


def test_symmetric_gemm_equals_the_full_product_bit_for_bit_below_the_diagonal():
    """The symmetric mode must change which tiles are computed, not their values: the lower triangle (and the tiles
    straddling the diagonal) come out identical to the plain GEMM, and the mirrored part is their exact transpose."""
    from himuon_b200 import ops

    for B, M, K in [(3, 512, 512), (2, 1024, 384), (2, 776, 200), (1, 1280, 128)]:
        X = _unit_rows(B, M, K, seed=5)
        full = ops.gemm(X, X, trans_b=True)
        sym = ops.gemm(X, X, trans_b=True, symmetric=True)
        torch.cuda.synchronize()
        assert torch.equal(torch.tril(full), torch.tril(sym)), (B, M, K)
        assert torch.equal(sym, sym.transpose(-2, -1)), (B, M, K)
        # tall operand (A = X^T X through the MN-major operand path)
        Xt = X.transpose(-2, -1).contiguous()
        full_t = ops.gemm(Xt, Xt, trans_a=True)
        sym_t = ops.gemm(Xt, Xt, trans_a=True, symmetric=True)
        torch.cuda.synchronize()
        assert torch.equal(torch.tril(full_t), torch.tril(sym_t)), (B, M, K)
        assert torch.equal(sym_t, sym_t.transpose(-2, -1)), (B, M, K)
    ops.check_status()
