#!/usr/bin/env python
"""The communication patterns of tensor, pipeline, sequence and expert parallelism, each on the
library's primitives through torch.distributed (backend "hxccl"), each checked against the
same computation done on one rank.

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 4 examples/parallel_patterns.py [--cpu]

* tensor parallel: a two-layer MLP with the first weight split by columns and the second by
  rows; the partial outputs are summed with reduce_scatter and re-assembled with all_gather.
* pipeline parallel: activations travel rank to rank with send / recv, one micro-batch after
  another.
* sequence parallel (ring): every rank owns a block of keys; the blocks go round the ring with
  send / recv so that each rank meets all of them (the data movement of ring attention).
* expert parallel: tokens go to the rank that owns their expert with an uneven all_to_all and
  come back with the mirrored one.
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cpu", action="store_true")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    import hxccl_b200.parallel as hp

    hp.register()
    rank, n = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if args.cpu:
        dev = torch.device("cpu")
    else:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("hxccl", rank=rank, world_size=n)
    g = torch.Generator().manual_seed(7)  # the same numbers on every rank
    ok = {}

    # ---- tensor parallel ---------------------------------------------------------------------
    d, h, tokens = 64, 32 * n, 8 * n
    x = torch.randn(tokens, d, generator=g).to(dev)
    w1, w2 = torch.randn(d, h, generator=g).to(dev), torch.randn(h, d, generator=g).to(dev)
    cols = slice(rank * h // n, (rank + 1) * h // n)
    partial = torch.relu(x @ w1[:, cols]) @ w2[cols, :]          # this rank's share of the sum
    mine = torch.empty(tokens // n, d, device=dev)
    dist.reduce_scatter_tensor(mine, partial.contiguous())        # sum, each rank keeps some rows
    full = torch.empty(tokens, d, device=dev)
    dist.all_gather_into_tensor(full, mine)
    ok["tensor"] = torch.allclose(full, torch.relu(x @ w1) @ w2, rtol=1e-4, atol=1e-3)

    # ---- pipeline parallel -------------------------------------------------------------------
    stage = torch.nn.Linear(d, d).to(dev)
    with torch.no_grad():
        stage.weight.copy_(torch.eye(d) * (rank + 2))
        stage.bias.zero_()
    outs = []
    for micro in range(3):
        if rank == 0:
            act = torch.full((4, d), float(micro + 1), device=dev)
        else:
            act = torch.empty(4, d, device=dev)
            dist.recv(act, src=rank - 1)
        with torch.no_grad():
            act = stage(act)
        if rank < n - 1:
            dist.send(act, dst=rank + 1)
        else:
            outs.append(float(act[0, 0]))
    scale = 1.0
    for r in range(n):
        scale *= r + 2
    ok["pipeline"] = rank < n - 1 or outs == [scale * (m + 1) for m in range(3)]

    # ---- sequence parallel: blocks round the ring -------------------------------------------------
    block = torch.full((16,), float(rank), device=dev)
    seen = [float(block[0])]
    batched = dist.distributed_c10d._get_default_group()._get_backend(dev).supports_coalescing
    for _ in range(n - 1):
        incoming = torch.empty_like(block)
        if batched:         # one library group: send and receive move together
            for w in dist.batch_isend_irecv([dist.P2POp(dist.isend, block, (rank + 1) % n),
                                             dist.P2POp(dist.irecv, incoming, (rank - 1) % n)]):
                w.wait()
        elif rank % 2 == 0:  # even ranks send first, odd ranks receive first: no pair waits on itself
            dist.send(block, dst=(rank + 1) % n)
            dist.recv(incoming, src=(rank - 1) % n)
        else:
            dist.recv(incoming, src=(rank - 1) % n)
            dist.send(block, dst=(rank + 1) % n)
        block = incoming
        seen.append(float(block[0]))
    ok["sequence"] = sorted(seen) == [float(r) for r in range(n)]

    # ---- expert parallel: uneven all_to_all there and back ------------------------------------------
    tg = torch.Generator().manual_seed(100 + rank)
    expert_of = torch.randint(0, n, (40,), generator=tg)           # one expert per rank
    order = torch.argsort(expert_of, stable=True)
    toks = (torch.arange(40, dtype=torch.float32) + 1000 * rank)[order].to(dev)
    send_counts = torch.bincount(expert_of, minlength=n)
    counts_in = torch.empty(n, dtype=torch.int64, device=dev)
    dist.all_to_all_single(counts_in, send_counts.to(dev))          # how many tokens each rank sends me
    recv_counts = counts_in.cpu().tolist()
    got = torch.empty(sum(recv_counts), device=dev)
    dist.all_to_all_single(got, toks, output_split_sizes=recv_counts, input_split_sizes=send_counts.tolist())
    processed = got * 2 + rank                                       # the expert's work
    back = torch.empty_like(toks)
    dist.all_to_all_single(back, processed, output_split_sizes=send_counts.tolist(), input_split_sizes=recv_counts)
    want = toks * 2 + expert_of[order].to(dev)
    ok["expert"] = bool(torch.equal(back, want))

    flags = torch.tensor([float(all(ok.values()))], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if rank == 0:
        print({k: bool(v) for k, v in ok.items()}, "all ranks agree:", bool(flags[0] == 1.0), flush=True)
    dist.destroy_process_group()
    return 0 if flags[0] == 1.0 else 1


if __name__ == "__main__":
    sys.exit(main())
