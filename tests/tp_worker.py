"""One rank of a tensor-parallel engine run (launched by the tests, 2 ranks).

    python tests/tp_worker.py cpu|gpu|gpufused <rank> <world> <port> <out.npz>

cpu: the engine on the oracle stand-in, the allreduce over gloo. gpu: the engine on the
library, the allreduce over NCCL (NVLS off, plain peer transport). gpufused: the cross-rank sum
fused with residual add and RMSNorm over peer memory (tp_reduce_norm). Rank 0 writes the prefill
logits, one decode step's logits, the greedy tokens of a short generation and its KV cache
shard; the other ranks write their cache shards.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)


def model():
    from tessel_b200.model import Config, Weights
    cfg = Config(dim=256, layers=2, heads=8, kv_heads=2, head_dim=64, ffn=512, vocab=1000, eps=1e-5,
                 rope_theta=10000.0, max_pos=512, bos=1, eos=-1)
    return cfg, Weights.random(cfg, 13)


def requests(cfg):
    from tessel_b200.sched import Request
    g = np.random.default_rng(2)
    return [Request(g.integers(0, cfg.vocab, n).tolist(), 12) for n in (40, 7, 33)]


def run(gpu, rank, world, out, exchange=None):
    from tessel_b200.engine import Decode, Engine, Limits, Packed
    from tessel_b200.model import argmax
    from tessel_b200.sched import generate_with
    cfg, w = model()
    lim = Limits(page=16, pages=40, max_tokens=128, max_seq_pages=8)
    e = Engine(gpu, w, lim, rank=rank, nranks=world, exchange=exchange)
    g = np.random.default_rng(1)
    p1, p2 = g.integers(0, cfg.vocab, 37).tolist(), g.integers(0, cfg.vocab, 20).tolist()
    toks, pos = p1 + p2, list(range(37)) + list(range(20))
    slots = [16 * 3 + i for i in range(37)] + [16 * 9 + i for i in range(20)]
    pre = e.step(toks, pos, slots, Packed([0] * 37 + [37] * 20), [36, 56]).copy()
    t1, t2 = argmax(pre[0]), argmax(pre[1])
    dec = e.step([t1, t2], [37, 20], [16 * 5 + 5, 16 * 10 + 4], Decode([[3, 4, 5], [9, 10]], [38, 21]), [0, 1]).copy()
    kc, vc = e.read_cache(1)
    e2 = Engine(gpu, w, Limits(page=16, pages=64, max_tokens=128, max_seq_pages=8), rank=rank, nranks=world,
                exchange=exchange)
    outs, _ = generate_with(e2, requests(cfg), 3, True, device_argmax=True)
    np.savez(out, pre=pre, dec=dec, kc=kc, vc=vc, tokens=np.asarray([o.tokens for o in outs]))


def main():
    mode, rank, world, port, out = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), sys.argv[4], sys.argv[5]
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", port
    if world > 1:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    if mode == "cpu":
        from emu import EmuGpu

        def allreduce(a):
            t = torch.from_numpy(a)
            dist.all_reduce(t)
            return t.numpy()

        gpu = EmuGpu(allreduce if world > 1 else None)
    else:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        from tessel_b200.gpu import Gpu
        gpu = Gpu(rank)
        if world > 1:
            ids = [gpu.comm_id() if rank == 0 else None]
            dist.broadcast_object_list(ids, src=0)
            gpu.comm_init(rank, world, ids[0])
    exchange = None
    if mode == "gpufused" and world > 1:
        def exchange(mine):
            everyone = [None] * world
            dist.all_gather_object(everyone, mine)
            return everyone
    run(gpu, rank, world, out, exchange)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
