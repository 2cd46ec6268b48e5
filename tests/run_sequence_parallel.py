"""torchrun worker of tests/test_sequence_parallel_gpu.py: sequence-parallel prefill over the local GPUs,
compared on rank 0 with the single-GPU pass over the whole sequence.  Also usable by hand:

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 tests/run_sequence_parallel.py
"""

import argparse
import os
import sys
import time

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import mlstm_kernels_b200 as mk  # noqa: E402
from mlstm_kernels_b200 import sharding  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="scan")
    ap.add_argument("--out", default="")
    ap.add_argument("--S", type=int, default=16384)
    ap.add_argument("--NH", type=int, default=8)
    ap.add_argument("--DHQK", type=int, default=256)
    ap.add_argument("--DHHV", type=int, default=512)
    ap.add_argument("--chunk", type=int, default=256)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--no-bw", action="store_true", help="skip the backward chain (forward timing only)")
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    # every rank draws the same full sequence (same seed, same generator type) on its GPU and keeps its own segment;
    # all comparisons below stay on the GPU, so long sequences cost no host time
    g = torch.Generator(device=dev).manual_seed(0)
    shape = (1, args.NH, args.S)
    q = torch.randn(*shape, args.DHQK, generator=g, device=dev).bfloat16()
    k = torch.randn(*shape, args.DHQK, generator=g, device=dev).bfloat16()
    v = torch.randn(*shape, args.DHHV, generator=g, device=dev).bfloat16()
    i = torch.randn(*shape, generator=g, device=dev).bfloat16()
    f = (3 + torch.randn(*shape, generator=g, device=dev)).bfloat16()
    seg = args.S // world
    sl = slice(rank * seg, (rank + 1) * seg)
    loc = [t[:, :, sl].contiguous() for t in (q, k, v, i, f)]

    def rel_err(a, b):   # same definition as inputs.max_rel_err, on the device
        a, b = a.double(), b.double()
        return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))
    ms = None
    for rep in range(args.reps):
        dist.barrier(); torch.cuda.synchronize()
        t0 = time.perf_counter()
        h, last = sharding.mlstm_chunkwise_sequence_parallel(*loc, return_last_states=True, chunk_size=args.chunk,
                                                             mode=args.mode)
        torch.cuda.synchronize(); dist.barrier()
        ms = (time.perf_counter() - t0) * 1e3
    hs = [torch.empty_like(h) for _ in range(world)]
    dist.all_gather(hs, h)
    # backward through the sequence-parallel call: a chain of messages from the last rank to the first
    gathered, dh_full = [], None
    if not args.no_bw:
        dh_full = torch.randn(1, args.NH, args.S, args.DHHV, generator=g, device=dev).bfloat16()
        leaves = [t.detach().clone().requires_grad_(True) for t in loc]
        h_b = sharding.mlstm_chunkwise_sequence_parallel(*leaves, chunk_size=args.chunk, mode=args.mode)
        h_b.backward(dh_full[:, :, sl].contiguous())
        torch.cuda.synchronize()
        for t in leaves:
            parts = [torch.empty_like(t.grad) for _ in range(world)]
            dist.all_gather(parts, t.grad.contiguous())
            gathered.append(torch.cat(parts, 2))
    if rank == 0:
        full = [q, k, v, i, f]
        for rep in range(args.reps):
            torch.cuda.synchronize(); t0 = time.perf_counter()
            h1, last1 = mk.mlstm_chunkwise__b200_xl_chunk(*full, return_last_states=True, chunk_size=args.chunk)
            torch.cuda.synchronize(); ms1 = (time.perf_counter() - t0) * 1e3
        err_g = {}
        if not args.no_bw:
            full_leaves = [t.detach().clone().requires_grad_(True) for t in full]
            mk.mlstm_chunkwise__b200_xl_chunk(*full_leaves, chunk_size=args.chunk).backward(dh_full)
            err_g = {"err_d" + n: rel_err(a, b.grad) for n, a, b in zip("qkvif", gathered, full_leaves)}
        err = dict(err_h=rel_err(torch.cat(hs, 2), h1), err_c=rel_err(last[0], last1[0]),
                   err_n=rel_err(last[1], last1[1]), err_m=rel_err(last[2], last1[2]), **err_g)
        print(f"mode={args.mode} world={world} S={args.S}: sequence-parallel {ms:.3f} ms, single GPU {ms1:.3f} ms, "
              + " ".join(f"{k_}={v_:.2e}" for k_, v_ in err.items()))
        if args.out:
            np.savez(os.path.join(args.out, "result.npz"), ms_sp=ms, ms_single=ms1, **err)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
