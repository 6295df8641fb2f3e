"""Worker of test_pipeline_stage_boundary (torch.distributed.run, backend gloo): a small MLP and the
Llama architecture (fp32 PyTorch model) cut into pipeline stages, variable-length micro-batches in
one-forward-one-backward order; every stage's parameter gradients and the losses must equal those
of the unsplit model."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dcp_b200.parallel.pipeline import PipelineComm, run_stage_1f1b  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(3)
    hidden, n_layers, tokens = 32, 2 * world, [40, 17, 64, 5, 33]
    layers = [torch.nn.Linear(hidden, hidden, dtype=torch.float64) for _ in range(n_layers)]
    xs = [torch.randn(n, hidden, dtype=torch.float64) for n in tokens]
    ys = [torch.randn(n, hidden, dtype=torch.float64) for n in tokens]
    run = lambda ls, x: [x := torch.tanh(l(x)) for l in ls][-1]
    # unsplit reference (every rank computes it: same seed)
    ref_losses = []
    for x, y in zip(xs, ys):
        loss = ((run(layers, x) - y) ** 2).mean()
        loss.backward()
        ref_losses.append(loss.item())
    ref_grads = [l.weight.grad.clone() for l in layers]
    for l in layers:
        l.weight.grad = None
        l.bias.grad = None
    mine = layers[rank * 2:(rank + 1) * 2]
    comm = PipelineComm(dist.group.WORLD, lambda mb: (tokens[mb], hidden), torch.float64, torch.device("cpu"))
    losses = run_stage_1f1b(comm, len(tokens), lambda mb, x: run(mine, xs[mb] if x is None else x),
                            lambda mb, y: ((y - ys[mb]) ** 2).mean())
    ok = all((l.weight.grad - g).abs().max().item() < 1e-10 for l, g in zip(mine, ref_grads[rank * 2:(rank + 1) * 2]))
    if comm.is_last:
        ok = ok and len(losses) == len(tokens) and all(abs(a.item() - b) < 1e-12 for a, b in zip(losses, ref_losses))
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    flag2 = torch.tensor([1 if llama_stages(rank, world) else 0])
    dist.all_reduce(flag2, op=dist.ReduceOp.MIN)
    if rank == 0 and flag.item() == 1 and flag2.item() == 1:
        print("PP_OK", flush=True)
    dist.destroy_process_group()


def llama_stages(rank: int, world: int) -> bool:
    """The Llama architecture (fp32 PyTorch model) cut into ``world`` stages of consecutive layers:
    embedding on the first stage, final norm + LM head + loss on the last, packed variable-length
    micro-batches; losses and every stage's parameter gradients equal the unsplit model's."""
    from dcp_b200.models.llama import LlamaModel, tiny_config
    from dcp_b200.models.reference import (reference_embed, reference_head_loss, reference_layers, reference_loss,
                                           stage_layer_range)
    cfg = tiny_config(n_layers=world + 1, hidden=64, n_heads=4, n_kv_heads=2, ffn=96, vocab=50)
    cfg.head_dim = 16
    g = torch.Generator().manual_seed(5)
    p = {}
    for name, shp in LlamaModel.param_shapes(cfg):
        p[name] = (torch.ones(shp, dtype=torch.float64) if "norm" in name
                   else 0.1 * torch.randn(shp, generator=g, dtype=torch.float64)).requires_grad_(True)
    batches = []
    for seqlens in ([9, 4, 12], [20], [3, 3, 3, 8]):
        n = sum(seqlens)
        toks = torch.randint(0, cfg.vocab, (n,), generator=g)
        pos = torch.cat([torch.arange(s) for s in seqlens])
        batches.append((toks, torch.roll(toks, -1), pos, seqlens))
    ref_losses = []
    for toks, labels, pos, seqlens in batches:
        loss = reference_loss(cfg, p, toks, labels, pos, seqlens, 1.0 / len(toks))
        loss.backward()
        ref_losses.append(loss.item())
    ref_grads = {k: v.grad.clone() for k, v in p.items()}
    for v in p.values():
        v.grad = None
    layers = stage_layer_range(cfg.n_layers, rank, world)
    comm = PipelineComm(dist.group.WORLD, lambda mb: (len(batches[mb][0]), cfg.hidden), torch.float64, torch.device("cpu"))

    def forward_fn(mb, x):
        toks, _, pos, seqlens = batches[mb]
        if x is None:
            x = reference_embed(p, toks)
        return reference_layers(cfg, p, x, pos, seqlens, layers.start, layers.stop)

    losses = run_stage_1f1b(comm, len(batches), forward_fn,
                            lambda mb, y: reference_head_loss(cfg, p, y, batches[mb][1], 1.0 / len(batches[mb][0])))
    mine = [k for k in p if any(k.startswith(f"l{l}.") for l in layers)]
    mine += ["embed"] if comm.is_first else []
    mine += ["norm_f", "lm_head"] if comm.is_last else []
    ok = all(p[k].grad is not None and (p[k].grad - ref_grads[k]).abs().max().item() < 1e-10 for k in mine)
    ok = ok and all(p[k].grad is None for k in p if k not in mine)          # a stage touches only its own parameters
    if comm.is_last:
        ok = ok and all(abs(a.item() - b) < 1e-12 for a, b in zip(losses, ref_losses))
    return ok


if __name__ == "__main__":
    main()
