"""Two-rank worker: tensor-parallel training step vs the fp32 PyTorch model assembled from the
shards (launched with torch.distributed.run by tests/test_gpu_engine.py)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dcp_b200.data import synth  # noqa: E402
from dcp_b200.models.llama import tiny_config  # noqa: E402
from dcp_b200.models.reference import reference_loss  # noqa: E402
from dcp_b200.train import EngineConfig, TrainEngine, init_distributed  # noqa: E402


def full_param(name, shards, cfg, tp):
    """Assemble the unsharded matrix from the per-rank shards (list indexed by tensor-parallel rank)."""
    d = cfg.head_dim
    hq, hkv = cfg.n_heads // tp, cfg.n_kv_heads // tp
    if name.endswith("wqkv"):
        q = [s[:hq * d] for s in shards]
        k = [s[hq * d:(hq + hkv) * d] for s in shards]
        v = [s[(hq + hkv) * d:] for s in shards]
        return torch.cat(q + k + v, 0)
    if name.endswith("wgu"):
        f = cfg.ffn // tp
        return torch.cat([s[:f] for s in shards] + [s[f:] for s in shards], 0)
    if name.endswith((".wo", ".wd")):
        return torch.cat(shards, 1)
    return shards[0]


def main():
    rank, world, local, group = init_distributed()
    assert world == 2
    dev = torch.device("cuda", local)
    full = tiny_config(n_layers=2, hidden=1024, n_heads=8, n_kv_heads=2, ffn=2048, vocab=2048)
    cfg = EngineConfig(full, tokens_per_step=1536, block_size=256, tp_size=2,
                       length_dist=synth.LengthDist("lognormal", 400.0, 0.6, 64, 1536), planner_workers=0,
                       clip_grad=1.0)
    eng = TrainEngine(cfg, dev, group)
    assert eng.tp_size == 2 and eng.n_cp_ranks == 1 and eng.model.cfg.n_heads == 4
    plan = eng.plans.get(0)
    toks, labels, pos = eng.stage_inputs(plan)
    eng.model.zero_grad()
    loss = eng.model.loss(toks, labels, pos, 1.0 / plan.n_global_tokens)
    loss.backward()
    torch.cuda.synchronize()
    eng.executor.check_status()
    # gather both ranks' parameters and gradients
    params, grads = {}, {}
    for name, t in eng.model.p.items():
        both_p = [torch.empty_like(t) for _ in range(2)]
        both_g = [torch.empty_like(t.grad) for _ in range(2)]
        dist.all_gather(both_p, t.detach().contiguous())
        dist.all_gather(both_g, t.grad.contiguous())
        params[name], grads[name] = both_p, both_g
    ok = True
    if rank == 0:
        p32 = {n: full_param(n, [s.float() for s in sh], full, 2).requires_grad_(True) for n, sh in params.items()}
        ref = reference_loss(full, p32, toks, labels, pos, plan.seqlens, 1.0 / plan.n_global_tokens)
        ref.backward()
        rel_loss = abs(loss.item() - ref.item()) / abs(ref.item())
        print("loss", loss.item(), ref.item(), rel_loss)
        ok &= rel_loss < 2e-2
        for name in ("l0.wqkv", "l1.wo", "l0.wgu", "l1.wd", "l0.norm1", "embed", "lm_head"):
            g = full_param(name, [s.float() for s in grads[name]], full, 2)
            r = p32[name].grad
            err = ((g - r).abs().max() / (r.abs().max() + 1e-6)).item()
            print(name, err)
            ok &= err < 8e-2
        # replicated parameters get the same gradient on both ranks
        ok &= torch.equal(grads["embed"][0], grads["embed"][1])
    # a full step (clipping norm across shards, sharded state) keeps the replicated parameters identical
    eng.optimizer.step(1.0)
    torch.cuda.synchronize()
    both = [torch.empty_like(eng.model.p["norm_f"]) for _ in range(2)]
    dist.all_gather(both, eng.model.p["norm_f"].detach().contiguous())
    ok &= torch.equal(both[0], both[1])
    l2 = eng.train_step(eng.plans.get(1))
    ok &= l2 == l2
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    eng.close()
    if rank == 0 and flag.item() == 1:
        print("TP_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
