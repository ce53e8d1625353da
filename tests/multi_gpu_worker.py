"""One rank of the 2..8-GPU parity check of the gathered decode matvec (run by
tests/test_gpu_multi.py under torch.distributed.run, one process per GPU).

Every rank holds the rows [rank * M / G, (rank + 1) * M / G) of each matrix, runs
okf_gemm_gather, and checks its own copy of the whole output against the oracle
run on the whole matrix."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle  # noqa: E402
from chatokf_b200 import tp  # noqa: E402
from chatokf_b200.enc import Context, CudaEnc, GGUFTensor  # noqa: E402
from chatokf_b200.gguf_types import GGUFType  # noqa: E402
from helpers import lcg_fill, make_weights, rel_err  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = Context(local)
    enc = CudaEnc(ctx)
    cases = [(GGUFType.Q4_K, 2560, 1024, 1), (GGUFType.Q4_K, 2560, 512, 1), (GGUFType.Q4_K, 1024, 256, 3),
             (GGUFType.IQ2_XXS, 5120, 512, 1), (GGUFType.Q8_0, 2048, 384, 2), (GGUFType.Q2_0, 2048, 640, 1),
             (GGUFType.Q4_K, 9728, 640, 1), (GGUFType.IQ2_XXS, 17408, 512, 2),  # long rows, cut into k-chunks
             (GGUFType.Q4_K, 1024, 768, 40), (GGUFType.Q4_K, 8192, 256, 45)]  # more than 8 tokens: the matmul (one with k-ranges)
    # ordered: every launch waits for the exchange before it; free: nobody waits until gather_wait
    all_peers = [tp.PeerOutputs(ctx, [(n, m) for _, _, m, n in cases], free=f) for f in (False, True)]
    worst = worst_tile = 0.0
    shards, refs, xs = [], [], []
    for i, (ty, k, m, n) in enumerate(cases):
        blocks = make_weights(ty, m, k, seed=100 + i)  # the same on every rank
        X = np.stack([lcg_fill(k, 7 + i + c) for c in range(n)])
        refs.append(oracle.matmul(ty, blocks, k, m, X, n))
        lo, hi = tp.shard_bounds(m, rank, world)
        shards.append((GGUFTensor(f"w{i}", (k, hi - lo), ty), ctx.upload(tp.shard_rows(ty, blocks, k, m, rank, world))))
        xs.append(torch.from_numpy(X).cuda())
    for rounds in range(6):  # the counters keep counting from exchange to exchange
        peers = all_peers[rounds // 2 % 2]
        # Matrices 0 and 1 multiply the same x.  Even rounds: one launch, one exchange on
        # matrix 0's counter.  Odd rounds: each alone, so the same counter sees exchanges of
        # another grid size (the count an exchange completes at is a running total).
        if rounds % 2 == 0:
            with enc.parallel():
                for i in (0, 1):
                    enc.gemm_gather(shards[i][0], xs[0], peers.slot(i, shards[i][0].M), shards[i][1], 1)
        else:
            for i in (0, 1):
                enc.gemm_gather(shards[i][0], xs[0], peers.slot(i, shards[i][0].M), shards[i][1], 1)
        for i in range(2, len(cases)):
            enc.gemm_gather(shards[i][0], xs[i], peers.slot(i, shards[i][0].M), shards[i][1], cases[i][3])
        enc.gather_wait()  # every launch waited for the one before it; this waits for the last
        torch.cuda.synchronize()
        dist.barrier()  # nobody starts the next round while a rank may still read this one
        for i in range(len(cases)):
            ref = refs[i] if i != 1 else oracle.matmul(cases[1][0], make_weights(cases[1][0], cases[1][2], cases[1][1], seed=101),
                                                       cases[1][1], cases[1][2], xs[0].cpu().numpy(), 1)
            err = rel_err(peers.read(i), ref)
            if cases[i][3] > 8:  # 16-bit operands on the tensor cores: their own bound
                worst_tile = max(worst_tile, err)
            else:
                worst = max(worst, err)
        dist.barrier()
    status = ctx.device_status()
    ok = worst <= 1e-4 and worst_tile <= 1e-2 and status == 0
    print(f"rank {rank}/{world}: max rel err {worst:.2e} (matmul {worst_tile:.2e}), device status {status}: "
          f"{'OK' if ok else 'FAIL'}", flush=True)
    flag = torch.tensor([0 if ok else 1], device="cuda")
    dist.all_reduce(flag)
    torch.cuda.synchronize()
    for peers in all_peers:
        peers.close()
    # tearing the communicator down has hung on this software stack: leave it to process exit
    os._exit(0 if flag.item() == 0 else 1)


if __name__ == "__main__":
    main()
