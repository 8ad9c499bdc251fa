"""Fidelity of the sparse decode against exact attention over a long generation:
``python -m sparse_kv_reads_b200.long_gen_tvd --prompt 8192 --steps 256 --budgets 0.05 0.2 1.0``.

Both decoders are fed the same (random) token ids; the figure is the total-variation distance between the
next-token distributions, averaged over the steps.  Counterpart of the reference's long-generation check
(ssa/harness/long_gen_tvd.py:119-169), on a random-weight Qwen3 architecture and synthetic ids because no
checkpoint or corpus is available here; with random weights attention is diffuse, so the distances are a
self-consistency measure (budget 1 must give ~0), not a quality claim.
"""

from __future__ import annotations

import argparse
import json

import torch

from .graph_decode import GraphDecoder
from .qwen3 import Qwen3Config, Qwen3Model
from .stamp import stamp


@torch.no_grad()
def decode_logits(model, ids: torch.Tensor, prompt: int, steps: int, capture: bool = True, **kw) -> torch.Tensor:
    """Logits ``[B, steps, vocab]`` of ``steps`` teacher-forced decode steps after a ``prompt``-token prefill."""
    B = ids.shape[0]
    cache = model.alloc_cache(-(-(prompt + steps + 8) // 16) * 16, max_batch=B)
    model.prefill(ids[:, :prompt], cache, chunk=2048)
    dec = GraphDecoder(model, cache, **kw)
    dec.prepare(prompt)
    if capture:
        dec.capture()
    out = []
    for t in range(prompt, prompt + steps):
        out.append(dec.step(ids[:, t:t + 1], t)[:, -1].float().clone())
    return torch.stack(out, 1)


def tvd(a: torch.Tensor, b: torch.Tensor) -> float:
    """Mean total-variation distance between the softmax distributions of two logit tensors."""
    return float(0.5 * (torch.softmax(a, -1) - torch.softmax(b, -1)).abs().sum(-1).mean())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="0.6b", choices=["0.6b", "4b"])
    ap.add_argument("--prompt", type=int, default=8192)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--budgets", type=float, nargs="+", default=[0.05, 0.2, 1.0])
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    cfg = Qwen3Config.qwen3_0_6b() if args.model == "0.6b" else Qwen3Config.qwen3_4b()
    with torch.device(dev):
        model = Qwen3Model(cfg)
    model = model.to(torch.bfloat16).eval().init_random(seed=0)
    ids = torch.randint(0, cfg.vocab_size, (1, args.prompt + args.steps + 1),
                        generator=torch.Generator().manual_seed(1)).to(dev)
    exact = decode_logits(model, ids, args.prompt, args.steps, mode="dense")
    rows = []
    for b in args.budgets:
        got = decode_logits(model, ids, args.prompt, args.steps, mode="cluster", budget=b, C=2048, C_init=256,
                            cap_keys=64.0, window=64)
        rows.append({"budget": b, "tvd": tvd(got, exact),
                     "top1_agreement": float((got.argmax(-1) == exact.argmax(-1)).float().mean())})
        print(json.dumps(rows[-1]), flush=True)
    if args.out:
        with open(args.out, "w") as fh:
            json.dump({"stamp": stamp(), "model": args.model, "prompt": args.prompt, "steps": args.steps, "rows": rows},
                      fh, indent=1)


if __name__ == "__main__":
    main()
