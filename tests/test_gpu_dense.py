"""Fused single-token kernels around the attention against the same steps written with PyTorch ops."""

from __future__ import annotations

import pytest
import torch

from sparse_kv_reads_b200._lib import check, lib
from sparse_kv_reads_b200.qwen3 import RMSNorm, apply_rope
from _helpers import DEV

pytestmark = pytest.mark.gpu


def stream():
    return torch.cuda.current_stream().cuda_stream


def test_add_rmsnorm():
    g = torch.Generator().manual_seed(0)
    for B, hidden in ((1, 1024), (3, 2560), (8, 64)):
        h = torch.randn(B, hidden, generator=g).to(torch.bfloat16).to(DEV)
        delta = torch.randn(B, hidden, generator=g).to(torch.bfloat16).to(DEV)
        norm = RMSNorm(hidden, 1e-6).to(DEV).to(torch.bfloat16)
        norm.weight.data = (1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16).to(DEV)
        want_h = h + delta
        want = norm(want_h)
        out = torch.empty_like(h)
        hh = h.clone()
        check(lib().skv_add_rmsnorm(hh.data_ptr(), delta.data_ptr(), norm.weight.data_ptr(), out.data_ptr(), B, hidden,
                                    1e-6, stream()), "skv_add_rmsnorm")
        assert torch.equal(hh, want_h)
        torch.testing.assert_close(out.float(), want.float(), rtol=1e-2, atol=1e-2)
        check(lib().skv_add_rmsnorm(hh.data_ptr(), None, norm.weight.data_ptr(), out.data_ptr(), B, hidden, 1e-6,
                                    stream()), "skv_add_rmsnorm")
        assert torch.equal(hh, want_h)
        torch.testing.assert_close(out.float(), want.float(), rtol=1e-2, atol=1e-2)


def test_qk_norm_rope_and_cache_write():
    g = torch.Generator().manual_seed(1)
    B, H, H_kv, d, L = 2, 4, 2, 128, 64
    qkv = torch.randn(B, (H + 2 * H_kv) * d, generator=g).to(torch.bfloat16).to(DEV)
    qn, kn = RMSNorm(d, 1e-6).to(DEV).to(torch.bfloat16), RMSNorm(d, 1e-6).to(DEV).to(torch.bfloat16)
    qn.weight.data = (1 + 0.1 * torch.randn(d, generator=g)).to(torch.bfloat16).to(DEV)
    kn.weight.data = (1 + 0.1 * torch.randn(d, generator=g)).to(torch.bfloat16).to(DEV)
    ang = torch.outer(torch.arange(L, dtype=torch.float64), 1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float64) / d)))
    ang = torch.cat((ang, ang), -1)
    cos, sin = ang.cos().to(torch.bfloat16).to(DEV), ang.sin().to(torch.bfloat16).to(DEV)
    pos = torch.tensor([37], dtype=torch.long, device=DEV)
    kc = torch.zeros(B, H_kv, L, d, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    q_out = torch.empty(B * H, d, dtype=torch.bfloat16, device=DEV)
    check(lib().skv_qk_rope_cache(qkv.data_ptr(), qn.weight.data_ptr(), kn.weight.data_ptr(), cos.data_ptr(),
                                  sin.data_ptr(), pos.data_ptr(), q_out.data_ptr(), kc.data_ptr(), vc.data_ptr(), B, H,
                                  H_kv, d, kc.stride(0), kc.stride(1), kc.stride(2), 1e-6, stream()), "skv_qk_rope_cache")
    q = qn(qkv[:, :H * d].view(B, 1, H, d)).transpose(1, 2)
    k = kn(qkv[:, H * d:(H + H_kv) * d].view(B, 1, H_kv, d)).transpose(1, 2)
    v = qkv[:, (H + H_kv) * d:].view(B, 1, H_kv, d).transpose(1, 2)
    q, k = apply_rope(q, k, cos[37:38], sin[37:38])
    torch.testing.assert_close(q_out.float(), q.reshape(B * H, d).float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(kc[:, :, 37].float(), k[:, :, 0].float(), rtol=2e-2, atol=2e-2)
    assert torch.equal(vc[:, :, 37], v[:, :, 0])
    assert float(kc[:, :, :37].abs().sum()) == 0 and float(kc[:, :, 38:].abs().sum()) == 0


def test_silu_mul():
    g = torch.Generator().manual_seed(2)
    B, inter = 3, 3072
    gu = (torch.randn(B, 2 * inter, generator=g) * 2).to(torch.bfloat16).to(DEV)
    out = torch.empty(B, inter, dtype=torch.bfloat16, device=DEV)
    check(lib().skv_silu_mul(gu.data_ptr(), out.data_ptr(), B, inter, stream()), "skv_silu_mul")
    want = torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]
    torch.testing.assert_close(out.float(), want.float(), rtol=1e-2, atol=1e-2)

