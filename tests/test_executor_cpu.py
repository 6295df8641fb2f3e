"""Planner + executor correctness on CPU against dense masked attention.

* in-process ranks (threads + mailboxes) for several device counts / masks, forward and backward;
* the two-rank gloo run of the reference configuration: lengths 512/1024/2048/4096, block 256,
  8 Q heads, 2 KV heads, head_dim 64, fp32, outputs/LSE/dQ/dK/dV within 1e-5;
* host-side failure detection: a rank that dies or a message that is dropped turns into an
  exception on the survivors within the timeout instead of a hang.
"""
import os
import subprocess
import sys

import pytest
import torch

from dcp_b200.core.common import get_default_execution_context
from dcp_b200.planner import masks
from dcp_b200.planner.compiler import CompilerConfig, InstrCompiler
from dcp_b200.planner.workload import generate_workload, pad_seqlens
from dcp_b200.runtime.comm import CommTimeout, MailboxHub
from dcp_b200.runtime.simulate import dense_reference, run_plans_in_process

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _compile(n_dev, n_nodes, raw, bs, H, Hkv, d, hbs, mask_name, n_stages=None):
    ctx = get_default_execution_context(n_dev, n_nodes)
    pad = pad_seqlens(raw, bs)
    m = masks.get_mask_fn(mask_name)(raw, pad, torch.int32)
    wl = generate_workload((sum(pad), H, d), (sum(pad), 2, Hkv, d), raw, pad, bs, hbs, ctx.comp_cost_model, m,
                           torch.float32)
    return ctx, pad, m, InstrCompiler(ctx, CompilerConfig(n_stages=n_stages)).compile(wl)


@pytest.mark.parametrize("n_dev,n_nodes,mask,hbs,n_stages", [
    (2, 1, "causal", 4, None), (4, 1, "lambda", 8, 2), (4, 2, "shared_question", 2, None),
    (8, 2, "causal_blockwise", 2, 3), (3, 1, "chunked_first_chunk", 4, 1)])
def test_plans_match_dense_attention(n_dev, n_nodes, mask, hbs, n_stages):
    torch.manual_seed(0)
    raw, bs, H, Hkv, d = [150, 500, 333, 64], 64, 8, 2, 16
    ctx, pad, m, (fw_wl, bw_wl, fw, bw) = _compile(n_dev, n_nodes, raw, bs, H, Hkv, d, hbs, mask, n_stages)
    T = sum(raw)
    q, kv, dout = torch.randn(T, H, d), torch.randn(T, 2, Hkv, d), torch.randn(T, H, d)
    out, lse, dq, dkv = run_plans_in_process(ctx, fw_wl, fw, q, kv, raw, bw_wl, bw, dout, timeout_s=30)
    ro, rl, rdq, rdkv = dense_reference(q, kv, raw, pad, m, d ** -0.5, dout)
    fin = torch.isfinite(rl)
    assert (out - ro).abs().max() < 1e-5
    assert (lse - rl)[fin].abs().max() < 1e-5
    assert (dq - rdq).abs().max() < 2e-5 and (dkv - rdkv).abs().max() < 2e-5


def test_tree_packed_pipeline_on_three_nodes_matches_dense_attention(monkeypatch):
    """The "tree" pipeline algorithm (fan-out transfers relayed along packed multicast trees) on a
    3-node x 2-device cluster: some blocks really travel through a relay node, the plans validate
    and they compute dense attention forward and backward."""
    from dcp_b200.planner import steiner
    from dcp_b200.planner.validate import validate_plans
    relayed = []
    packer = steiner.pack_multicast_trees

    def counting(requests, *a, **k):
        trees = packer(requests, *a, **k)
        owner = {r[0]: r[1] for r in requests}
        relayed.append(sum(1 for b, edges in trees.items() for _, h, _ in edges if h != owner[b]))
        return trees

    monkeypatch.setattr(steiner, "pack_multicast_trees", counting)
    torch.manual_seed(0)
    raw, bs, H, Hkv, d = [2500, 400], 64, 4, 2, 16
    ctx = get_default_execution_context(6, 3)
    pad = pad_seqlens(raw, bs)
    m = masks.get_mask_fn("causal")(raw, pad, torch.int32)
    wl = generate_workload((sum(pad), H, d), (sum(pad), 2, Hkv, d), raw, pad, bs, 1, ctx.comp_cost_model, m, torch.float32)
    fw_wl, bw_wl, fw, bw = InstrCompiler(ctx, CompilerConfig(pipeline_algo="tree", n_stages=4)).compile(wl)
    assert sum(relayed) > 0
    validate_plans(ctx, fw_wl, fw, True)
    validate_plans(ctx, bw_wl, bw, False)
    T = sum(raw)
    q, kv, dout = torch.randn(T, H, d), torch.randn(T, 2, Hkv, d), torch.randn(T, H, d)
    out, lse, dq, dkv = run_plans_in_process(ctx, fw_wl, fw, q, kv, raw, bw_wl, bw, dout, timeout_s=60)
    ro, rl, rdq, rdkv = dense_reference(q, kv, raw, pad, m, d ** -0.5, dout)
    assert (out - ro).abs().max() < 1e-5 and (dq - rdq).abs().max() < 3e-5 and (dkv - rdkv).abs().max() < 3e-5


def test_gloo_world2_reference_config():
    """Two real processes over gloo: the planner/executor correctness configuration."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29611", os.path.join(ROOT, "tests", "gloo_worker.py")]
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="2")
    res = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:]
    assert "GLOO_OK" in res.stdout, res.stdout[-3000:]


@pytest.mark.parametrize("world,mask,dcp_size", [(2, "causal", 2), (3, "causal", 3), (2, "shared_question", 2),
                                                 (2, "causal_blockwise", 2), (4, "causal", 2)])
def test_interpreter_training_matches_unsplit_model(world, mask, dcp_size):
    """End-to-end DCP training without a GPU: synthetic batch -> placement -> plans -> two-layer Llama
    with distributed attention on the plan interpreter over gloo ranks -> gradient sum -> AdamW; loss,
    gradients and the parameters after three steps equal those of the unsplit fp32 model, for causal
    and for structured masks (the unsplit model applies the same per-query key ranges densely), and for
    two context-parallel groups of two ranks each (CP x DP: the batch dealt over the groups)."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29620 + world), os.path.join(ROOT, "tests", "interp_worker.py"), mask,
           str(dcp_size)]
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="2")
    res = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert res.returncode == 0 and "INTERP_OK" in res.stdout, res.stdout[-3000:]


def test_interpreter_pipeline_times_context_parallel():
    """Pipeline parallelism together with DCP: 2 stages x 2 context-parallel ranks (4 gloo ranks), every
    stage of a context-parallel rank plans the same batches, three micro-batches in one-forward-one-
    backward order; losses and every stage's gradients equal the unsplit fp32 model's."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr",
           "127.0.0.1", "--master-port", "29627", os.path.join(ROOT, "tests", "interp_pp_worker.py")]
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="1")
    res = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert res.returncode == 0 and "INTERP_PP_OK" in res.stdout, res.stdout[-3000:]


def test_interpreter_tensor_times_context_parallel():
    """Tensor parallelism together with DCP: heads and FFN channels split over 2 adjacent ranks, 2
    context-parallel ranks per shard (4 gloo ranks); the planner plans for the per-shard head counts;
    loss and every shard's gradients equal the unsplit model's, replicated parameters stay identical."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr",
           "127.0.0.1", "--master-port", "29628", os.path.join(ROOT, "tests", "interp_tp_worker.py")]
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="1")
    res = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert res.returncode == 0 and "INTERP_TP_OK" in res.stdout, res.stdout[-3000:]


def test_rank_failure_surfaces_as_exception():
    torch.manual_seed(0)
    raw = [256, 256]
    ctx, pad, m, (fw_wl, bw_wl, fw, bw) = _compile(2, 1, raw, 64, 4, 2, 16, 2, "causal")
    q, kv = torch.randn(sum(raw), 4, 16), torch.randn(sum(raw), 2, 2, 16)
    with pytest.raises(RuntimeError, match="injected failure"):
        run_plans_in_process(ctx, fw_wl, fw, q, kv, raw, timeout_s=1.0, fail_rank=1)


def test_dropped_message_times_out():
    torch.manual_seed(0)
    raw = [512]
    ctx, pad, m, (fw_wl, bw_wl, fw, bw) = _compile(2, 1, raw, 64, 4, 2, 16, 2, "causal")
    q, kv = torch.randn(sum(raw), 4, 16), torch.randn(sum(raw), 2, 2, 16)
    hub = MailboxHub(2, timeout_s=1.0)
    from dcp_b200.core.instructions import CommLaunchInstr, CommType
    key = next(i.key for i in fw[(0, 0)].instructions if isinstance(i, CommLaunchInstr)
               and any(op.comm_type == CommType.SEND for op in i.comm_ops))
    hub.dropped.add((0, 1, key))
    with pytest.raises(CommTimeout):
        run_plans_in_process(ctx, fw_wl, fw, q, kv, raw, hub=hub)


def test_flag_barrier_protocol_model():
    """The cross-GPU barrier protocol on a host model with real threads: safety and liveness over
    many epochs (including 32-bit wrap-around), and a withheld signal ends in a timeout status on
    the rank that misses it, never in a hang."""
    import random
    import threading
    import time
    from dcp_b200.runtime.symm import FlagBarrierModel
    world, n_epochs, base = 4, 40, 0xFFFFFFF0           # epochs run across the uint32 wrap
    model = FlagBarrierModel(world)
    for r in range(world):                               # as after base earlier barriers
        model.flags[r] = [base & 0xFFFFFFFF] * world
    arrived = [[0.0] * world for _ in range(n_epochs)]
    passed = [[0.0] * world for _ in range(n_epochs)]

    def run(rank):
        rnd = random.Random(rank)
        for e in range(n_epochs):
            time.sleep(rnd.random() * 0.002)
            arrived[e][rank] = time.monotonic()
            assert model.arrive_and_wait(rank, base + 1 + e, timeout_s=5.0) == FlagBarrierModel.STATUS_OK
            passed[e][rank] = time.monotonic()

    threads = [threading.Thread(target=run, args=(r,)) for r in range(world)]
    [t.start() for t in threads]
    [t.join(timeout=60) for t in threads]
    assert not any(t.is_alive() for t in threads)
    for e in range(n_epochs):
        assert min(passed[e]) >= max(arrived[e]) - 1e-6   # nobody left before the last one arrived

    # fault injection: rank 1 never tells rank 0 -> rank 0 times out, the others pass
    model = FlagBarrierModel(3)
    out = {}
    def run2(rank):
        out[rank] = model.arrive_and_wait(rank, 1, timeout_s=0.3, withhold_from=(0,) if rank == 1 else ())
    threads = [threading.Thread(target=run2, args=(r,)) for r in range(3)]
    t0 = time.monotonic()
    [t.start() for t in threads]
    [t.join(timeout=10) for t in threads]
    assert time.monotonic() - t0 < 5 and not any(t.is_alive() for t in threads)
    assert out == {0: FlagBarrierModel.STATUS_SIGNAL_TIMEOUT, 1: 0, 2: 0}
