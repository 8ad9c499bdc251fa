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
                                  sin.data_ptr(), pos.data_ptr(), 0, q_out.data_ptr(), kc.data_ptr(), vc.data_ptr(), B, H,
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



@pytest.mark.parametrize("B", [1, 2, 3, 8])
def test_gemv_with_the_three_input_modes(B):
    """y = x W^T against float32 matmul of the same bf16 operands, for the projection shapes of the two models
    and a few awkward ones (rows not a multiple of the CTA count, one row, a long row)."""
    g = torch.Generator().manual_seed(B)
    L = lib()
    for N, K in ((4096, 1024), (1024, 2048), (6144, 1024), (1024, 3072), (1000, 2560), (1, 64)) + (((300, 9728),) if B <= 4 else ()):
        W = (torch.randn(N, K, generator=g) / K ** 0.5).to(torch.bfloat16).to(DEV)
        x = torch.randn(B, K, generator=g).to(torch.bfloat16).to(DEV)
        y = torch.full((B, N), 7.0, dtype=torch.bfloat16, device=DEV)
        check(L.skv_gemv(W.data_ptr(), N, K, y.data_ptr(), B, 0, x.data_ptr(), None, None, None, None, 0.0, stream()),
              "skv_gemv")
        want = x.float() @ W.float().T
        torch.testing.assert_close(y.float(), want, rtol=1e-2, atol=1e-2)
        # mode 1: residual add + RMSNorm feeding the product, h_out out of place
        h = torch.randn(B, K, generator=g).to(torch.bfloat16).to(DEV)
        delta = torch.randn(B, K, generator=g).to(torch.bfloat16).to(DEV)
        gw = (1 + 0.1 * torch.randn(K, generator=g)).to(torch.bfloat16).to(DEV)
        for dl in (delta, None):
            h_out = torch.zeros_like(h)
            check(L.skv_gemv(W.data_ptr(), N, K, y.data_ptr(), B, 1, None, h.data_ptr(),
                             None if dl is None else dl.data_ptr(), gw.data_ptr(), h_out.data_ptr(), 1e-6, stream()),
                  "skv_gemv")
            hs = h + dl if dl is not None else h
            assert torch.equal(h_out, hs)
            xn = torch.empty_like(h)
            check(L.skv_add_rmsnorm(hs.clone().data_ptr(), None, gw.data_ptr(), xn.data_ptr(), B, K, 1e-6, stream()),
                  "skv_add_rmsnorm")
            torch.testing.assert_close(y.float(), xn.float() @ W.float().T, rtol=2e-2, atol=2e-2)
        # mode 2: silu(gate) * up feeding the product
        gu = torch.randn(B, 2 * K, generator=g).to(torch.bfloat16).to(DEV)
        act = torch.empty(B, K, dtype=torch.bfloat16, device=DEV)
        check(L.skv_silu_mul(gu.data_ptr(), act.data_ptr(), B, K, stream()), "skv_silu_mul")
        check(L.skv_gemv(W.data_ptr(), N, K, y.data_ptr(), B, 2, gu.data_ptr(), None, None, None, None, 0.0, stream()),
              "skv_gemv")
        torch.testing.assert_close(y.float(), act.float() @ W.float().T, rtol=1e-2, atol=1e-2)


def _rms(x, g, eps=1e-6):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * g.float()).to(torch.bfloat16)


@pytest.mark.parametrize("world,B,N", [(2, 12, 256), (4, 32, 2560), (8, 3, 64)])
def test_partial_sums_pushed_into_every_buffer_add_up_to_the_same_bits(world, B, N):
    """The exchange for producers that are not this library's products (batches beyond 8): every emulated rank pushes
    its partial results, every rank then reads the same sum; several steps, both slots."""
    from sparse_kv_reads_b200.peer_reduce import PeerExchange
    L = lib()
    g = torch.Generator().manual_seed(7 * world + B)
    ex = PeerExchange.emulated(world, B * N, DEV)
    for use in range(5):
        for e in ex:
            e.tick(stream())
        parts = [torch.randn(B, N, generator=g).to(torch.bfloat16).to(DEV) for _ in range(world)]
        for r in range(world):
            check(L.skv_comm_push(ex[r].ref(), use, parts[r].data_ptr(), B, N, stream()), "skv_comm_push")
        want = torch.stack([x.float() for x in parts]).sum(0)
        got = []
        for r in range(world):
            delta = torch.empty(B, N, dtype=torch.bfloat16, device=DEV)
            check(L.skv_comm_reduce(ex[r].ref(), use, delta.data_ptr(), B, N, stream()), "skv_comm_reduce")
            got.append(delta)
        torch.testing.assert_close(got[0].float(), want, rtol=1e-2, atol=2e-2)
        assert all(torch.equal(got[0], x) for x in got[1:])
    assert all(e.status() == 0 for e in ex)
    y = torch.zeros(B, N, dtype=torch.bfloat16, device=DEV)
    assert L.skv_comm_push(ex[0].ref(), 255, y.data_ptr(), B, N, stream()) == -5       # exchange numbers end at 254
    assert L.skv_comm_push(ex[0].ref(), 0, y.data_ptr(), B + 1, N, stream()) == -5     # more than the buffers hold
    assert L.skv_comm_push(ex[0].ref(), 0, None, B, N, stream()) == -1
    for e in ex:
        e.close()


@pytest.mark.parametrize("B", [1, 4])
def test_row_parallel_product_summed_through_exchange_buffers(B):
    """Two ranks emulated on one device (their kernels run one after the other): each multiplies its half of
    the inputs, the partial sums land in both exchange buffers, and the next product of either rank adds them."""
    import ctypes
    from sparse_kv_reads_b200._lib import ST_WAIT_TIMEOUT
    from sparse_kv_reads_b200.peer_reduce import PeerExchange
    L = lib()
    g = torch.Generator().manual_seed(40 + B)
    world, N, K, N2 = 2, 1024, 2048, 512
    ex = PeerExchange.emulated(world, B * N, DEV)
    W = (torch.randn(N, K, generator=g) / K ** 0.5).to(torch.bfloat16).to(DEV)
    W2 = (torch.randn(N2, N, generator=g) / N ** 0.5).to(torch.bfloat16).to(DEV)
    gw = (1 + 0.1 * torch.randn(N, generator=g)).to(torch.bfloat16).to(DEV)
    Ks = K // world
    Wr = [W[:, r * Ks:(r + 1) * Ks].contiguous() for r in range(world)]
    for use in range(3):                                  # several steps, both slots
        slot = use
        for e in ex:
            e.tick(stream())
        x = torch.randn(B, K, generator=g).to(torch.bfloat16).to(DEV)
        h = torch.randn(B, N, generator=g).to(torch.bfloat16).to(DEV)
        for r in range(world):
            xr = x[:, r * Ks:(r + 1) * Ks].contiguous()
            check(L.skv_gemv_tp(Wr[r].data_ptr(), N, Ks, None, B, 0, xr.data_ptr(), None, None, None, 0.0, None, 0,
                                ex[r].ref(), slot, stream()), "skv_gemv_tp")
        parts = torch.stack([xr.float() @ wr.float().T for xr, wr in
                             ((x[:, r * Ks:(r + 1) * Ks], Wr[r]) for r in range(world))])
        h_new = (h.float() + parts.sum(0)).to(torch.bfloat16)
        want = _rms(h_new, gw).float() @ W2.float().T
        outs = []
        for r in range(world):
            y = torch.empty(B, N2, dtype=torch.bfloat16, device=DEV)
            h_out = torch.empty_like(h)
            check(L.skv_gemv_tp(W2.data_ptr(), N2, N, y.data_ptr(), B, 3, None, h.data_ptr(), gw.data_ptr(),
                                h_out.data_ptr(), 1e-6, ex[r].ref(), slot, None, 0, stream()), "skv_gemv_tp")
            assert (h_out.float() - h_new.float()).abs().max() <= 0.07      # one unit in the last place of a bf16 near 8
            torch.testing.assert_close(y.float(), want, rtol=3e-2, atol=3e-2)
            outs.append((y, h_out))
            delta = torch.empty(B, N, dtype=torch.bfloat16, device=DEV)
            check(L.skv_comm_reduce(ex[r].ref(), slot, delta.data_ptr(), B, N, stream()), "skv_comm_reduce")
            torch.testing.assert_close(delta.float(), parts.sum(0), rtol=1e-2, atol=1e-2)
        assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])   # same bits on every rank
    assert all(e.status() == 0 for e in ex)
    assert L.skv_gemv_tp(W2.data_ptr(), N2, N, None, B, 0, h.data_ptr(), None, None, None, 0.0, None, 0, None, 0,
                         stream()) == -1                 # neither y nor an exchange to write to
    assert L.skv_gemv_tp(W2.data_ptr(), N2, 4096, None, B, 3, None, h.data_ptr(), gw.data_ptr(), None, 0.0,
                         ex[0].ref(), 0, None, 0, stream()) == -1
    for e in ex:
        e.close()


def test_wait_for_a_rank_that_never_delivers_gives_up_and_reports():
    """A bounded wait: rank 0 has produced, rank 1 never does; rank 0's consumer polls rank 1's values for a fraction
    of a second (the limit is set low here), sets the time-out bit in its status word and finishes (nothing hangs, the context stays usable)."""
    from sparse_kv_reads_b200._lib import ST_WAIT_TIMEOUT
    from sparse_kv_reads_b200.peer_reduce import PeerExchange
    L = lib()
    B, N, K = 1, 256, 512
    ex = PeerExchange.emulated(2, B * N, DEV, wait_kpolls=512)      # about a third of a second
    for e in ex:
        e.tick(stream())
    W = torch.randn(N, K, device=DEV).to(torch.bfloat16)
    x = torch.randn(B, K, device=DEV).to(torch.bfloat16)
    check(L.skv_gemv_tp(W.data_ptr(), N, K, None, B, 0, x.data_ptr(), None, None, None, 0.0, None, 0, ex[0].ref(), 0,
                        stream()), "skv_gemv_tp")
    delta = torch.empty(B, N, dtype=torch.bfloat16, device=DEV)
    check(L.skv_comm_reduce(ex[0].ref(), 0, delta.data_ptr(), B, N, stream()), "skv_comm_reduce")
    torch.cuda.synchronize()
    assert ex[0].status() & ST_WAIT_TIMEOUT
    assert ex[1].status() == 0
    assert float(torch.ones(4, device=DEV).sum()) == 4.0      # the device still answers
    # once a wait has given up, later waits on the same GPU look once and move on: a consumer that polls every
    # element of the missing rank (a product with the sum folded in, then another reduce) ends in milliseconds,
    # not in one full limit per polled element
    import time
    gw = torch.ones(N, dtype=torch.bfloat16, device=DEV)
    h = torch.zeros(B, N, dtype=torch.bfloat16, device=DEV)
    y = torch.empty(B, 64, dtype=torch.bfloat16, device=DEV)
    W2 = torch.randn(64, N, device=DEV).to(torch.bfloat16)
    t0 = time.perf_counter()
    check(L.skv_gemv_tp(W2.data_ptr(), 64, N, y.data_ptr(), B, 3, None, h.data_ptr(), gw.data_ptr(), None, 1e-6,
                        ex[0].ref(), 0, None, 0, stream()), "skv_gemv_tp")
    check(L.skv_comm_reduce(ex[0].ref(), 0, delta.data_ptr(), B, N, stream()), "skv_comm_reduce")
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 0.1
    for e in ex:
        e.close()
