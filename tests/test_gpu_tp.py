"""Tensor-parallel decode on two GPUs (skipped on a single-GPU box): the sums after the row-parallel products
taken through the peer-memory exchange against the same model with NCCL all-reduces, at budget 1 where the
clustering cannot matter.  One process per GPU, rendezvous on 127.0.0.1."""

from __future__ import annotations

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu

TINY = dict(vocab_size=1000, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=8,
            num_key_value_heads=4, head_dim=128, max_position_embeddings=4096)


def _rank_main(rank: int, world: int, port: int, out_path: str, batch: int) -> None:
    import torch.distributed as dist
    from sparse_kv_reads_b200 import GraphDecoder, Qwen3Config, Qwen3Model
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    P, T = 300, 24
    ids = torch.randint(0, 1000, (batch, P + T + 1), generator=torch.Generator().manual_seed(3)).to(dev)

    def run(peer: bool):
        os.environ["SKV_PEER_REDUCE"] = "1" if peer else "0"
        with torch.device(dev):
            model = Qwen3Model(Qwen3Config(**TINY), tp_group=dist.group.WORLD, tp_size=world, tp_rank=rank)
        model = model.to(torch.bfloat16).eval().init_random(seed=5, std=0.05)
        cache = model.alloc_cache(336, max_batch=batch)
        with torch.no_grad():
            model.prefill(ids[:, :P], cache, chunk=128)
            dec = GraphDecoder(model, cache, mode="cluster", budget=1.0, C=64, C_init=16, split_factor=2.0, window=4,
                               delta=float("inf"), summary_bits=8)
            dec.prepare(P)
            dec.capture()
            outs = [dec.step(ids[:, t:t + 1], t)[:, -1].float().clone() for t in range(P, P + T)]
        status = dec._peer.status() if dec._peer is not None else 0
        used = dec._peer is not None
        if used:                                      # unmap the other rank's buffer and free this rank's
            torch.cuda.synchronize()
            dist.barrier()
            dec._peer.close()
        return torch.stack(outs, 1), status, used

    a, status, used = run(True)
    b, _, _ = run(False)
    if rank == 0:
        torch.save({"peer": a.cpu(), "nccl": b.cpu(), "status": status, "used": used}, out_path)
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0)                                   # captured graphs hold NCCL work: leave without the teardown


# two sequences run the library's own products with the sums inside them; twelve run library GEMMs with the
# partial results pushed into the exchange buffers and added up by a reduce launch
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("batch", [2, 12])
def test_peer_memory_sums_match_nccl_all_reduce(tmp_path, batch):
    import torch.multiprocessing as mp
    out_path = str(tmp_path / "tp.pt")
    ctx = mp.get_context("spawn")
    with socket.socket() as sock:                 # a port nobody holds right now
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, out_path, batch)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    codes = [p.exitcode for p in procs]
    for p in procs:                               # a rank still running must not outlive the test on a shared box
        if p.exitcode is None:
            p.kill()
            p.join()
    assert all(c == 0 for c in codes), codes
    got = torch.load(out_path)
    assert got["used"] and got["status"] == 0
    torch.testing.assert_close(got["peer"], got["nccl"], rtol=3e-2, atol=6e-2)
    assert (got["peer"].argmax(-1) == got["nccl"].argmax(-1)).float().mean() > 0.9
