"""One rank of a tensor-parallel engine run (launched by the tests, 1 to 8 ranks).

    python tests/tp_worker.py cpu|gpu|gpufused <rank> <world> <port> <out.npz>

cpu: the engine on the oracle stand-in, the allreduce over gloo. gpu: the engine on the
library, the allreduce over NCCL (NVLS off, plain peer transport). gpufused: the cross-rank sum
fused with residual add and RMSNorm over peer memory (tp_reduce_norm). Every rank writes what
``tessel_b200.tpcheck.run`` returns: the prefill logits, one decode step's logits, the greedy
tokens of a 32-step generation, its KV cache shard, and its x and h after the decode step.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)


def main():
    mode, rank, world, port, out = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), sys.argv[4], sys.argv[5]
    import torch
    import torch.distributed as dist
    from tessel_b200 import tpcheck
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
    np.savez(out, **tpcheck.run(gpu, rank, world, exchange))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
