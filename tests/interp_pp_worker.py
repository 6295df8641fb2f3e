"""Worker of test_interpreter_pipeline_times_context_parallel (torch.distributed.run, 4 gloo ranks):
2 pipeline stages x 2 context-parallel ranks on the plan interpreter, three planned micro-batches in
one-forward-one-backward order, against the unsplit fp32 model: micro-batch losses and the summed
gradients of every stage's parameters."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dcp_b200.data import synth  # noqa: E402
from dcp_b200.models.llama import LlamaConfig  # noqa: E402
from dcp_b200.models.reference import reference_loss  # noqa: E402
from dcp_b200.train_interp import InterpreterEngine, init_params  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.set_num_threads(1)
    n_pp, n_cp = 2, world // 2
    stage, cp_rank = rank // n_cp, rank % n_cp
    cp_groups = [dist.new_group([s * n_cp + c for c in range(n_cp)]) for s in range(n_pp)]
    pp_groups = [dist.new_group([s * n_cp + c for s in range(n_pp)]) for c in range(n_cp)]
    cfg = LlamaConfig(3, 64, 4, 2, 16, 96, 101)           # 3 layers: stage 0 takes two, stage 1 one
    n_micro = 3
    eng = InterpreterEngine(cfg, 1200, block_size=128, group=cp_groups[stage], seed=5, pp_group=pp_groups[cp_rank],
                            n_micro=n_micro)
    assert eng.stage == stage and eng.rank == cp_rank and list(eng.layers) == ([0, 1] if stage == 0 else [2])
    losses = eng.pipeline_loss_and_grads(0)
    # the unsplit model on the same three batches
    ref_p = init_params(cfg, 5)
    ref_losses = []
    for mb in range(n_micro):
        seed = eng.spec.seed * 1000003 + mb
        seqlens = synth.sample_seqlens(eng.spec.tokens_per_step, eng.spec.length_dist, seed)
        batch = synth.make_token_batch(seqlens, cfg.vocab, seed)
        loss = reference_loss(cfg, ref_p, torch.from_numpy(batch["tokens"]), torch.from_numpy(batch["labels"]),
                              torch.from_numpy(batch["positions"]), seqlens, 1.0 / sum(seqlens))
        loss.backward()
        ref_losses.append(loss.item())
    ok = True
    mine = eng.stage_parameters()
    for name in ref_p:
        if name in mine:
            g, r = eng.p[name].grad, ref_p[name].grad
            err = (g - r).abs().max().item() / (r.abs().max().item() + 1e-12)
            if err > 2e-4:
                print(f"rank {rank} {name}: relative gradient error {err}", flush=True)
                ok = False
        else:
            ok &= eng.p[name].grad is None                 # another stage's parameter is never touched
    if stage == n_pp - 1:
        ok &= len(losses) == n_micro and all(abs(a - b) < 1e-5 * abs(b) for a, b in zip(losses, ref_losses))
    else:
        ok &= losses == []
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0 and flag.item() == 1:
        print("INTERP_PP_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
