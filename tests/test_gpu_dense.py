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


@pytest.mark.parametrize("B", [1, 3, 8])
def test_gemv_and_fused_norm_gemv(B):
    g = torch.Generator().manual_seed(3)
    K, N = 1024, 520
    W = (torch.randn(2 * N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    x = torch.randn(B, K, generator=g).to(torch.bfloat16).to(DEV)
    y = torch.empty(B, N, dtype=torch.bfloat16, device=DEV)
    check(lib().skv_gemv(W.data_ptr(), x.data_ptr(), y.data_ptr(), B, N, K, stream()), "skv_gemv")
    torch.testing.assert_close(y.float(), (x.float() @ W[:N].float().T), rtol=2e-2, atol=2e-2)
    # residual add + norm in front; plain and gated
    h = torch.randn(B, K, generator=g).to(torch.bfloat16).to(DEV)
    delta = torch.randn(B, K, generator=g).to(torch.bfloat16).to(DEV)
    norm = RMSNorm(K, 1e-6).to(DEV).to(torch.bfloat16)
    norm.weight.data = (1 + 0.1 * torch.randn(K, generator=g)).to(torch.bfloat16).to(DEV)
    h_new = h + delta
    xn = norm(h_new)
    for dl, want_h in ((delta, h_new), (None, h)):
        xn = norm(want_h)
        h_out = torch.zeros_like(h)
        check(lib().skv_norm_gemv(W.data_ptr(), h.data_ptr(), None if dl is None else dl.data_ptr(),
                                  norm.weight.data_ptr(), h_out.data_ptr(), y.data_ptr(), B, N, K, 1e-6, 0, stream()),
              "skv_norm_gemv")
        assert torch.equal(h_out, want_h)
        torch.testing.assert_close(y.float(), xn.float() @ W[:N].float().T, rtol=2e-2, atol=3e-2)
    check(lib().skv_norm_gemv(W.data_ptr(), h.data_ptr(), delta.data_ptr(), norm.weight.data_ptr(), h_out.data_ptr(),
                              y.data_ptr(), B, N, K, 1e-6, 1, stream()), "skv_norm_gemv")
    xn = norm(h_new)
    gate, up = torch.nn.functional.linear(xn, W[:N]), torch.nn.functional.linear(xn, W[N:])
    torch.testing.assert_close(y.float(), (torch.nn.functional.silu(gate) * up).float(), rtol=3e-2, atol=3e-2)
    assert lib().skv_norm_gemv(W.data_ptr(), h.data_ptr(), None, norm.weight.data_ptr(), h.data_ptr(), y.data_ptr(), B,
                               N, K, 1e-6, 0, stream()) == -5
    assert lib().skv_gemv(W.data_ptr(), x.data_ptr(), y.data_ptr(), 9, N, K, stream()) == -5
