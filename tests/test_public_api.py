"""The reference's import surface (`src/himuon/...`) resolves to this library, and the public kernel callables keep
the reference's signatures and semantics (checked here on the CPU path; the sm_100a kernels behind them are checked in
the GPU tier)."""

import inspect

import pytest
import torch


def test_reference_import_paths_resolve():
    import himuon
    import himuon_b200
    from himuon.fsdp_bank import (BankScheme, BankSpec, Llama3BankScheme, ParamBank, Qwen3BankScheme,  # noqa: F401
                                  release_pre_shard_refs, unbank_state_dict, wrap_with_banks)
    from himuon.optim import get_optimizer, get_optimizer_kwargs  # noqa: F401
    from himuon.optimizers import SOAP, AdamW, HiMuon, HiMuonLegacy, Muon, MuonFsdp  # noqa: F401
    from himuon.optimizers.himuon import HiMuon as H2
    from himuon.triton_kernels import XXT, ba_plus_cAA, fused_bmm_add, ns5_smem  # noqa: F401
    from himuon.utils import TimeBudget, merge_kv_args, parse_kv_args, seed_everything  # noqa: F401

    assert H2 is HiMuon is himuon_b200.optimizers.HiMuon
    assert himuon.__version__ == himuon_b200.__version__
    import himuon.dataset
    import himuon.logger
    import himuon.model
    assert himuon.dataset.ToyDataset is himuon_b200.dataset.ToyDataset


def test_kernel_callables_have_the_reference_signatures():
    from himuon.triton_kernels import XXT, ba_plus_cAA, fused_bmm_add, ns5_smem

    assert list(inspect.signature(XXT).parameters) == ["A", "out"]
    assert list(inspect.signature(ba_plus_cAA).parameters) == ["A", "alpha", "beta", "out"]
    assert list(inspect.signature(fused_bmm_add).parameters) == ["B", "X", "a", "out"]
    sig = inspect.signature(ns5_smem).parameters
    assert list(sig) == ["X", "persistent", "grid_size"]
    assert sig["persistent"].kind is inspect.Parameter.KEYWORD_ONLY and sig["persistent"].default is False


@pytest.mark.parametrize("shape", [(4, 100, 70), (2, 50, 130), (200, 100)])
def test_kernel_callables_on_cpu_match_torch(shape):
    from himuon.triton_kernels import XXT, ba_plus_cAA, fused_bmm_add

    torch.manual_seed(0)
    A = torch.randn(*shape)
    M = shape[-2]
    out = torch.empty(*shape[:-2], M, M)
    assert XXT(A, out) is out
    assert torch.allclose(out, A @ A.transpose(-2, -1), atol=1e-4)
    S = out.clone()
    out2 = torch.empty_like(S)
    ba_plus_cAA(S, 2.0315, -4.775, out2)
    assert torch.allclose(out2, 2.0315 * (S @ S.transpose(-2, -1)) - 4.775 * S, rtol=1e-4, atol=1e-2)
    if A.ndim == 3:
        got = fused_bmm_add(S, A, 3.4445)
        assert torch.allclose(got, S @ A + 3.4445 * A, rtol=1e-4, atol=1e-3)


def test_ns5_smem_contract_on_cpu():
    from himuon.triton_kernels import ns5_smem
    from himuon_b200.ops import reference as ref

    x = torch.randn(3, 16, 64).bfloat16()
    out = ns5_smem(x)
    assert out.shape == x.shape and out.dtype == torch.bfloat16 and out.data_ptr() != x.data_ptr()
    assert torch.equal(out, ref.newton_schulz(x, 5))
    assert ns5_smem(x[0]).shape == (16, 64)
    with pytest.raises(AssertionError):
        ns5_smem(torch.randn(64, 16).bfloat16())          # tall tiles must be transposed by the caller
    with pytest.raises(AssertionError):
        ns5_smem(torch.randn(16, 64))                      # bf16 only
