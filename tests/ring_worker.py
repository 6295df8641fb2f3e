"""Worker of test_ring_baselines_match_dense_attention (torch.distributed.run, backend gloo):
plain and zigzag ring attention over packed sequences, forward and backward, against dense causal
attention of the whole batch."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dcp_b200.bench.baselines import HierarchicalA2AP2P, RingAttention  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.set_num_threads(2)
    g = torch.Generator().manual_seed(7)
    seqlens = RingAttention.adjust_seqlens([70, 129, 36, 260], world)
    T, H, Hkv, d = sum(seqlens), 4, 2, 16
    q = torch.randn(T, H, d, generator=g, dtype=torch.float64)
    k = torch.randn(T, Hkv, d, generator=g, dtype=torch.float64)
    v = torch.randn(T, Hkv, d, generator=g, dtype=torch.float64)
    dout = torch.randn(T, H, d, generator=g, dtype=torch.float64)
    # dense reference on every rank (same seed)
    qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
    cu = [0]
    for n in seqlens:
        cu.append(cu[-1] + n)
    outs = []
    gq = H // Hkv
    for a, b in zip(cu[:-1], cu[1:]):
        s = (qr[a:b].transpose(0, 1) @ kr[a:b].transpose(0, 1).repeat_interleave(gq, 0).transpose(1, 2)) * d ** -0.5
        s = s.masked_fill(~torch.ones(b - a, b - a, dtype=torch.bool).tril(), float("-inf"))
        outs.append((torch.softmax(s, -1) @ vr[a:b].transpose(0, 1).repeat_interleave(gq, 0)).transpose(0, 1))
    ref = torch.cat(outs)
    ref.backward(dout)
    ok = True
    variants = [("ring", lambda: RingAttention(dist.group.WORLD, seqlens, head_dim=d, zigzag=False)),
                ("zigzag", lambda: RingAttention(dist.group.WORLD, seqlens, head_dim=d, zigzag=True))]
    if world >= 4:
        variants += [("double ring", lambda: RingAttention(dist.group.WORLD, seqlens, head_dim=d, zigzag=True, window=2)),
                     ("plain double ring", lambda: RingAttention(dist.group.WORLD, seqlens, head_dim=d, zigzag=False, window=2)),
                     ("a2a+p2p", lambda: HierarchicalA2AP2P(dist.group.WORLD, seqlens, H, Hkv, 2, head_dim=d))]
    for zigzag, make in variants:
        ring = make()
        idx = ring.local_indices()
        ql, kl, vl = (t[idx].clone().requires_grad_(True) for t in (q, k, v))
        out = ring(ql, kl, vl)
        out.backward(dout[idx])
        for name, got, want in (("out", out, ref[idx]), ("dq", ql.grad, qr.grad[idx]), ("dk", kl.grad, kr.grad[idx]),
                                ("dv", vl.grad, vr.grad[idx])):
            err = (got - want).abs().max().item()
            if err > 1e-5:
                ok = False
                print(f"rank {rank} zigzag={zigzag} {name} max err {err}", flush=True)
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0 and flag.item() == 1:
        print("RING_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
