"""Multi-GPU worker: bucketed, overlapped reduce-scatter + sharded AdamW against torch.optim.AdamW.

Every rank fills its bf16 gradient buffer with its own random gradients, announces the buckets in
backward order (as the model's layer hooks do) and steps; after three steps the bf16 parameters of
every rank must equal those of a single fp32 torch.optim.AdamW run on the rank-summed gradients
(with the same global-norm clipping).  Launched with torch.distributed.run; plain peer ld/st only.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dcp_b200.parallel.dist_optimizer import FlatBuffers, ShardedAdamW, shard_layout  # noqa: E402


def main():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl")
    group = dist.group.WORLD
    # buckets that do not divide evenly by the world size, one of them tiny
    buckets = [(0, 4096), (4096, 8 * 1001), (4096 + 8 * 1001, 8), (4096 + 8 * 1002, 8 * 3333)]
    n = sum(b[1] for b in buckets)
    bufs = FlatBuffers(n, dev, group)
    g0 = torch.Generator(device=dev).manual_seed(7)
    bufs.params.copy_(torch.randn(n, device=dev, generator=g0).bfloat16())
    clip = 0.5
    opt = ShardedAdamW(bufs, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, clip_grad=clip, group=group,
                       buckets=buckets)
    assert opt.overlap and sum(s.length for s in shard_layout(buckets, world, rank)) == opt.master.numel()
    ref = bufs.params.float().clone().requires_grad_(True)
    ref_opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(3):
        g = torch.Generator(device=dev).manual_seed(100 * step + rank)
        grad = torch.randn(n, device=dev, generator=g).bfloat16()
        bufs.grads.copy_(grad)
        total = grad.float().clone()
        dist.all_reduce(total, group=group)
        # buckets become final in reverse order, the first one only at the end (step() picks it up)
        for b in (3, 2, 1):
            opt.reduce_bucket(b)
        opt.step(1.0)
        coef = min(1.0, clip / (total.norm().item() + 1e-6))
        ref.grad = total * coef
        ref_opt.step()
        torch.cuda.synchronize()
        opt.check_status()
        err = (bufs.params.float() - ref.detach()).abs().max().item()
        gn = abs(opt.grad_norm() - total.norm().item()) / total.norm().item()
        assert err < 2e-2 and gn < 1e-3, (step, err, gn)
    # every rank holds the same parameters
    mine = bufs.params.float().clone()
    other = mine.clone()
    dist.broadcast(other, src=0, group=group)
    assert (mine - other).abs().max().item() == 0
    # resume path: zero the bf16 parameters, rebuild them from the sharded fp32 master weights
    bufs.params.zero_()
    opt.rebuild_params()
    torch.cuda.synchronize()
    assert (bufs.params.float() - mine).abs().max().item() == 0
    # a set status word keeps the weights untouched
    before = bufs.params.clone()
    bufs.arena.status.fill_(2)
    bufs.grads.copy_(torch.ones(n, device=dev).bfloat16())
    opt.step(1.0)
    torch.cuda.synchronize()
    assert (bufs.params == before).all()
    bufs.arena.status.zero_()
    if rank == 0:
        print("OPT_OK", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
