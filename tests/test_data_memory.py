"""Data pipeline, plan service, memory subsystem, compatibility shims, utilities (CPU only)."""
import io
import os

import numpy as np
import pytest
import torch

from dcp_b200.core.common import ModelSpec, get_default_execution_context
from dcp_b200.data import synth
from dcp_b200.data.dataloader import DCPDataLoader, ExecutionPlanner, TrainingSpec
from dcp_b200.data.datasets import (DummyMultiModelDataset, MockGPTLowLevelDataset, OrderedBatchSampler,
                                    SyntheticLengthDataset)
from dcp_b200.data.kv_store import KVStore, KVTimeout
from dcp_b200.data.plan_service import PlanService, PlanSpec, plan_iteration, split_batch_over_groups
from dcp_b200.memory.allocation_simulator import AllocationSimulator, OutOfArena
from dcp_b200.memory.host_caching_allocator import HostCachingAllocator


def test_length_distributions_are_seeded_and_fill_budget():
    for dist in (synth.LOGNORMAL_8K, synth.LOGNORMAL_16K, synth.MIXTURE):
        a = synth.sample_seqlens(131072, dist, 5)
        assert a == synth.sample_seqlens(131072, dist, 5) and sum(a) == 131072
        assert a != synth.sample_seqlens(131072, dist, 6)
    lens = np.concatenate([synth.sample_seqlens(1 << 22, synth.LOGNORMAL_8K, s)[:-1] for s in range(3)])
    assert 6000 < np.median(lens) < 11000 and lens.min() >= 512
    b = synth.make_token_batch([5, 3], 100, 0)
    assert b["labels"][4] == -100 and b["labels"][7] == -100 and (b["labels"][:4] == b["tokens"][1:5]).all()
    assert b["positions"].tolist() == [0, 1, 2, 3, 4, 0, 1, 2]


def test_sampler_packs_within_budget_and_resumes():
    ds = SyntheticLengthDataset(200, synth.LengthDist("lognormal", 500, 0.9, 32, 4096), vocab=100, seed=1)
    s = OrderedBatchSampler(ds, 8192, shuffle=True, seed=3)
    batches = list(s)
    assert all(sum(min(ds.seqlens[i], 8192) for i in b) <= 8192 for b in batches)
    assert all(sum(ds.seqlens[i] for i in b) >= 0.75 * 8192 for b in batches)
    s2 = OrderedBatchSampler(ds, 8192, shuffle=True, seed=3)
    it = iter(s2)
    first = [next(it), next(it)]
    state = s2.state_dict()
    s3 = OrderedBatchSampler(ds, 8192, shuffle=True, seed=3)
    s3.load_state_dict(state)
    assert first == batches[:2] and list(s3) == batches[2:]


def test_dataloader_yields_local_batches_and_plans():
    ds = SyntheticLengthDataset(30, synth.LengthDist("lognormal", 600, 0.8, 64, 3000), vocab=1000)
    ts = TrainingSpec(get_default_execution_context(2, 1), ModelSpec(128, 8, 2), block_size=256, head_block_size=8,
                      dcp_size=2)
    seen = {0: [], 1: []}
    for rank in (0, 1):
        dl = DCPDataLoader(ts, ds, dcp_rank=rank, batch_sampler=OrderedBatchSampler(ds, 4096, shuffle=False),
                           num_preprocess_workers=0)
        for local, fw, bw, fw_wl, bw_wl, spec in dl:
            assert local["tokens"].shape == local["labels"].shape == local["position_ids"].shape
            assert local["tokens"].shape[1] == local["program"].q_local_rows == fw.local_cu_seqlens[-1]
            assert fw.local_device_id == rank and bw is not None
            seen[rank].append(local["tokens"].shape[1])
    assert [a + b for a, b in zip(seen[0], seen[1])] == [sum(ds.seqlens[i] for i in b)
                                                          for b in OrderedBatchSampler(ds, 4096, shuffle=False)]
    fw, bw, fw_wl, bw_wl, padded = ExecutionPlanner(0, 1, ts).plan([500, 1200, 300])
    assert set(fw) == {(0, 0), (0, 1)} and all(p % ExecutionPlanner(0, 1, ts).block_size == 0 or True for p in padded)


def test_plan_service_matches_direct_planning_and_splits_groups():
    spec = PlanSpec(4, 2, 8192, 8, 2, 128, 256, 0, "causal", synth.LengthDist("lognormal", 700, 0.8, 64, 4096))
    svc = PlanService(spec, rank=3, n_workers=1, lookahead=2)
    try:
        p0, p1 = svc.get(0), svc.get(1)
    finally:
        svc.close()
    d0 = plan_iteration(spec, 0, 3)
    assert torch.equal(p0.tokens, d0.tokens) and p0.program.q_local_rows == d0.program.q_local_rows
    assert p1.iteration == 1 and p0.n_global_tokens == 8192
    # the four ranks (2 groups x 2) cover every token exactly once
    total = sum(plan_iteration(spec, 0, r).tokens.numel() for r in range(4))
    assert total == 8192
    groups = split_batch_over_groups([100, 5000, 300, 4000, 50], 2)
    assert sorted(i for g in groups for i in g) == [0, 1, 2, 3, 4]
    mixed = PlanSpec(2, 2, 16384, 8, 2, 128, 512, 0, "mixed", synth.LengthDist("lognormal", 5000, 0.5, 4096, 16384))
    assert plan_iteration(mixed, 0, 1).program.fwd_flops > 0


def test_allocation_simulator_and_host_arena():
    sim = AllocationSimulator(1 << 20, alignment=256)
    a, b, c = sim.alloc(1000), sim.alloc(5000), sim.alloc(300)
    assert a == 0 and b == 1024 and sim.in_use == 1024 + 5120 + 512
    sim.free(b)
    assert sim.alloc(4000) == 1024            # best fit reuses the hole
    sim.free(a); sim.free(c)
    with pytest.raises(OutOfArena):
        sim.alloc(2 << 20)
    arena = HostCachingAllocator(1 << 16, pin=False)
    batch = {"x": torch.arange(100), "y": [torch.ones(3, 4)], "z": "keep"}
    pinned = arena.pin(batch)
    assert torch.equal(pinned["x"], batch["x"]) and pinned["z"] == "keep"
    assert pinned["x"].untyped_storage().data_ptr() == arena.arena.untyped_storage().data_ptr()
    used = arena.sim.in_use
    del pinned
    import gc; gc.collect()
    assert arena.sim.in_use < used
    big = arena.alloc((1 << 18,), torch.uint8)   # larger than the arena: falls back, never fails
    assert big.numel() == 1 << 18 and arena.n_fallback == 1


def test_kv_store_blocks_with_timeout():
    kv = KVStore(timeout_s=0.2)
    kv.set("a", {"n": 1})
    assert kv.get("a") == {"n": 1} and kv.exists("a") and kv.add("ctr", 2) == 2 and kv.add("ctr") == 3
    with pytest.raises(KVTimeout):
        kv.get("missing")


def test_reference_import_paths_resolve():
    import dcp_cpp
    from dcp.core.block_table import BlockType, WorkloadSpec  # noqa: F401
    from dcp.core.compiler import CompilerConfig, InstrCompiler  # noqa: F401
    from dcp.core.instructions import AttnInstr, ExecutionPlan  # noqa: F401
    from dcp.core.scheduler import convert_forward_to_backward, schedule  # noqa: F401
    from dcp.data.dataloader import DCPDataLoader, ExecutionPlanner, TrainingSpec, _generate_workload  # noqa: F401
    from dcp.data.hf_dataset import OrderedBatchSampler as S  # noqa: F401
    from dcp.graph_partition.graph import HGPSolver, construct_and_partition_graph_multiconstraint  # noqa: F401
    from dcp.ops.fused_ops import flash_attn_update_out_lse, fused_blockwise_sum, warmup_triton_ops  # noqa: F401
    from dcp.runtime.flash_attention import DCPAttention, get_executor, prepare_dcp_distributed_attn_for_test  # noqa: F401
    from dcp.runtime.flash_attention.utils import lambda_mask_fn, shared_question_mask_fn  # noqa: F401
    from dcp.utils.logger import create_logger, read_env_bool  # noqa: F401
    assert callable(dcp_cpp.greedy_selection_per_device)
    o, l = flash_attn_update_out_lse(torch.randn(2, 5, 3, 8), torch.randn(2, 5, 3))
    assert o.shape == (5, 3, 8) and l.shape == (5, 3)


def test_dcp_attention_autograd_single_device():
    """DCPAttention through the plan interpreter on one CPU device equals dense attention."""
    from dcp_b200.runtime.comm import MailboxComm, MailboxHub
    from dcp_b200.runtime.interface import DCPAttention, prepare_dcp_distributed_attn_for_test
    from dcp_b200.runtime.simulate import dense_reference
    ctx = get_default_execution_context(1, 1)
    raw = [200, 120]
    ex, lq, lkv, ldo, q, kv, dout, _, pad = prepare_dcp_distributed_attn_for_test(
        raw, 4, 2, 16, 64, 4, ctx, 0, "causal", torch.float32, comm=MailboxComm(MailboxHub(1), 0))
    lq.requires_grad_(True); lkv.requires_grad_(True)
    out = DCPAttention.apply(ex, False, False, lq, lkv)
    out.backward(ldo)
    ro, _, rdq, rdkv = dense_reference(q, kv, raw, pad, None, 16 ** -0.5, dout)
    assert (out.detach() - ro).abs().max() < 1e-5            # one device, one head block: local order == global
    assert (lq.grad - rdq).abs().max() < 1e-4 and (lkv.grad - rdkv).abs().max() < 1e-4


def test_visualization_and_logger(tmp_path, monkeypatch):
    from dcp_b200.planner.compiler import InstrCompiler
    from dcp_b200.planner.workload import generate_workload, pad_seqlens
    from dcp_b200.utils.common import read_env_int, trepr
    from dcp_b200.utils.logger import create_logger
    from dcp_b200.utils.visualization import visualize_workload_spec_figure, visualize_workload_spec_tty
    ctx = get_default_execution_context(2, 1)
    raw = [300, 200]
    pad = pad_seqlens(raw, 64)
    wl = generate_workload((sum(pad), 4, 16), (sum(pad), 2, 2, 16), raw, pad, 64, 4, ctx.comp_cost_model)
    fw_wl, _, _, _ = InstrCompiler(ctx).compile(wl, generate_backward=False)
    text = visualize_workload_spec_tty(fw_wl, 2)
    assert "seq 0: 5 blocks" in text and "seq 1: 4 blocks" in text
    g = visualize_workload_spec_figure(fw_wl, str(tmp_path / "g.json"), 2)
    assert (tmp_path / "g.json").exists() and len(g["edges"]) == 4 * len(fw_wl.workloads)
    monkeypatch.setenv("DCP_DEBUG", "DEBUG")
    monkeypatch.setenv("DCP_LOGGING_DEBUG_DIR", str(tmp_path))
    lg = create_logger("t", log_file="x/y.log")
    lg.debug("hello")
    for h in lg.handlers:
        h.flush()
    assert "hello" in (tmp_path / "x" / "y.log").read_text()
    monkeypatch.setenv("N", "7")
    assert read_env_int("N") == 7 and read_env_int("NOPE", 3) == 3 and "Tensor(shape=(2,)" in trepr(torch.zeros(2))


def test_plan_cache_reuses_plans_by_batch_signature(tmp_path):
    from dcp_b200.data import synth
    from dcp_b200.data.plan_service import PlanSpec, batch_signature, plan_iteration
    mk = lambda **kw: PlanSpec(world=2, dcp_size=2, tokens_per_step=8192, n_heads=8, n_kv_heads=2, block_size=512,
                               length_dist=synth.LengthDist("lognormal", 2000.0, 0.8, 128, 8192), vocab=1000, **kw)
    spec = mk(cache_dir=str(tmp_path))
    first = plan_iteration(spec, 3, 1)
    files = sorted(p.name for p in tmp_path.iterdir())
    assert len(files) == 1 and files[0].startswith("plan_")
    again = plan_iteration(spec, 3, 1)
    assert len(list(tmp_path.iterdir())) == 1
    assert torch.equal(first.tokens, again.tokens) and torch.equal(first.positions, again.positions)
    for a, b in zip(first.program.q_pulls + first.program.kv_pulls, again.program.q_pulls + again.program.kv_pulls):
        assert (a == b).all()
    uncached = plan_iteration(mk(), 3, 1)
    assert torch.equal(uncached.tokens, first.tokens)
    # another rank, another batch or another block size is another key
    s0 = batch_signature(spec, 0, [100, 200], None, None)
    assert s0 != batch_signature(spec, 1, [100, 200], None, None)
    assert s0 != batch_signature(spec, 0, [100, 201], None, None)
    assert s0 != batch_signature(mk(cache_dir=str(tmp_path), mem_imbalance_epsilon=0.2), 0, [100, 200], None, None)


def test_plan_service_validate_mode(monkeypatch):
    """DCP_B200_VALIDATE=1: every rank's tables are lowered and cross-checked before the rank's own
    program is handed out; the program is the same as without the check."""
    from dcp_b200.data import synth
    from dcp_b200.data.plan_service import PlanSpec, plan_iteration
    spec = PlanSpec(world=4, dcp_size=4, tokens_per_step=8192, n_heads=8, n_kv_heads=2, block_size=512,
                    length_dist=synth.LengthDist("lognormal", 2000.0, 0.8, 128, 8192), vocab=1000)
    plain = plan_iteration(spec, 2, 1)
    monkeypatch.setenv("DCP_B200_VALIDATE", "1")
    checked = plan_iteration(spec, 2, 1)
    assert torch.equal(plain.tokens, checked.tokens)
    assert plain.program.q_rows == checked.program.q_rows and plain.program.part_rows == checked.program.part_rows
    for a, b in zip(plain.program.kv_pulls, checked.program.kv_pulls):
        assert (a == b).all()


def test_every_public_name_of_the_reference_api_resolves():
    """The reference's public API surface, module by module: every name a user of the reference
    imports must resolve under the same path."""
    import importlib
    surface = {
        "dcp_cpp": ["greedy_selection_per_device"],
        "dcp.core.common": ["ExecutionContext", "ModelSpec", "get_default_execution_context"],
        "dcp.core.cost_model": ["CommunicationCostModel", "AttnRooflineCostModel"],
        "dcp.core.block_table": ["BlockType", "DataBlockMeta", "ComputationBlockMeta", "BlockMappings", "BlockManager",
                                 "WorkloadSpec", "serialize_list_of_workloads", "deserialize_list_of_workloads"],
        "dcp.core.instructions": ["MemcpyInstr", "CommLaunchInstr", "BarrierInstr", "CommWaitInstr", "AttnInstr",
                                  "AttnBackwardInstr", "AttnReductionInstr", "SumInstr", "ExecutionPlan", "BufferBlock",
                                  "BufferType", "CommOp", "CommType", "serialize_list_of_execution_plans",
                                  "deserialize_list_of_execution_plans"],
        "dcp.core.serialization": [],
        "dcp.core.compiler": ["CompilerConfig", "InstrCompiler"],
        "dcp.core.scheduler": ["schedule", "convert_forward_to_backward"],
        "dcp.core.executor": ["DCPExecutor"],
        "dcp.core.pipeline": [],
        "dcp.core.steiner_tree_packing": [],
        "dcp.graph_partition.graph": ["HGPSolver", "construct_and_partition_graph_multiconstraint",
                                      "assign_device_by_heuristic", "assign_input_outputs"],
        "dcp.data.dataloader": ["TrainingSpec", "generate_workload", "ExecutionPlanner", "DCPDataLoader"],
        "dcp.data.hf_dataset": ["HuggingFaceDatasetConfig", "HuggingFaceDataset", "DummyMultiModelDataset",
                                "OrderedBatchSampler"],
        "dcp.data.kv_redis": [],
        "dcp.runtime.flash_attention": ["get_executor", "AttentionExecutor", "DCPAttention",
                                        "prepare_dcp_distributed_attn_for_test", "get_local_q_kv"],
        "dcp.runtime.flash_attention.utils": ["lambda_mask_fn", "shared_question_mask_fn", "causal_blockwise_mask_fn",
                                              "get_local_attn_ranges_zigzag", "get_per_step_attn_range",
                                              "reconstruct_attention_forward_output_for_test",
                                              "reconstruct_attention_backward_output_for_test"],
        "dcp.ops.fused_ops": ["flash_attn_update_out_lse", "fused_blockwise_sum", "warmup_triton_ops"],
        "dcp.memory.host_caching_allocator": ["apply_monkey_patch"],
        "dcp.utils.logger": ["create_logger", "read_env_bool", "logger"],
        "dcp.utils.common": ["trepr", "read_env_int"],
    }
    missing = []
    for mod, names in surface.items():
        m = importlib.import_module(mod)
        missing += [f"{mod}.{n}" for n in names if not hasattr(m, n)]
    assert not missing, missing
    ex = importlib.import_module("dcp.core.executor").DCPExecutor
    for method in ("register_handler", "check_all_handlers_registered", "init_buffers", "init_forward_input",
                   "init_backward_input", "deallocate_buffers", "execute"):
        assert hasattr(ex, method), method
    ae = importlib.import_module("dcp.runtime.flash_attention").AttentionExecutor
    for method in ("prepare", "forward", "backward", "switch_to_backward", "capture_cudagraph", "set_local_out_lse",
                   "deallocate_all_buffers", "log_memory_usage"):
        assert hasattr(ae, method), method


def test_planning_is_identical_across_processes():
    """Every rank plans on its own and all ranks must arrive at the same placement: the plan of a
    batch may not depend on the process (hash seeds, set iteration order, thread timing)."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = (
        "import hashlib, numpy as np\n"
        "from dcp_b200.data import synth\n"
        "from dcp_b200.data.plan_service import PlanSpec, plan_iteration\n"
        "spec = PlanSpec(world=8, dcp_size=8, tokens_per_step=65536, n_heads=8, n_kv_heads=2, block_size=1024,\n"
        "                length_dist=synth.MIXTURE, vocab=1000)\n"
        "h = hashlib.sha1()\n"
        "for rank in (0, 5):\n"
        "    p = plan_iteration(spec, 4, rank).program\n"
        "    for a in p.q_pulls + p.kv_pulls + [p.merge_ops, p.merge_src, p.dq_push, p.dkv_push]:\n"
        "        h.update(np.ascontiguousarray(a).tobytes())\n"
        "    for t in p.fwd:\n"
        "        if t is not None:\n"
        "            h.update(t.tiles.numpy().tobytes()); h.update(t.kv_entries.numpy().tobytes())\n"
        "print('PLANHASH', h.hexdigest())\n")
    digests = set()
    for seed in ("0", "1", "12345"):
        res = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, PYTHONPATH=root, PYTHONHASHSEED=seed),
                             stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
        assert res.returncode == 0, res.stdout[-2000:]
        digests.add([l for l in res.stdout.splitlines() if l.startswith("PLANHASH")][0])
    assert len(digests) == 1, digests


def test_optimizer_shard_layout_covers_every_bucket_for_any_world_size():
    """The slicing formula shared by optimizer state, reduce-scatter, all-gather and resume: for
    world sizes that do not divide the buckets (3, 5, 6, 7) the ranks' slices tile every bucket
    exactly, are 8-element aligned, and the state offsets are the running sum of the lengths."""
    from dcp_b200.parallel.dist_optimizer import shard_layout
    buckets = [(0, 4096), (4096, 8 * 1001), (4096 + 8 * 1001, 8), (4096 + 8 * 1002, 8 * 3333)]
    for world in (1, 2, 3, 5, 6, 7, 8):
        per_rank = [shard_layout(buckets, world, r) for r in range(world)]
        for b, (off, length) in enumerate(buckets):
            pos = off
            for r in range(world):
                s = per_rank[r][b]
                assert s.bucket == b and s.length % 8 == 0 and s.flat_off % 8 == 0
                if s.length:
                    assert s.flat_off == pos
                    pos += s.length
            assert pos == off + length
        for shards in per_rank:
            acc = 0
            for s in shards:
                assert s.state_off == acc
                acc += s.length


def test_optimizer_state_is_recut_for_another_world_size():
    """Resume on a different number of ranks: the state of every new rank, cut out of the old ranks'
    state dictionaries, equals the slice of the full state that the new layout gives it."""
    import torch
    from dcp_b200.parallel.dist_optimizer import reshard_state, shard_layout
    buckets = [(0, 4096), (4096, 8 * 1001), (4096 + 8 * 1001, 8), (4096 + 8 * 1002, 8 * 3333)]
    n = sum(b[1] for b in buckets)
    full = {k: torch.randn(n) for k in ("master", "m", "v")}

    def state_of(world, rank):
        parts = {k: torch.cat([full[k][s.flat_off:s.flat_off + s.length] for s in shard_layout(buckets, world, rank)])
                 for k in full}
        return {**parts, "step": 7, "buckets": buckets, "world": world, "rank": rank}

    for old_world, new_world in ((8, 2), (2, 8), (3, 5), (6, 1), (1, 7)):
        for new_rank in range(new_world):
            got = reshard_state((state_of(old_world, r) for r in reversed(range(old_world))), buckets, new_world, new_rank)
            want = state_of(new_world, new_rank)
            assert got["step"] == 7 and got["world"] == new_world and got["rank"] == new_rank
            for k in full:
                assert torch.equal(got[k], want[k]), (old_world, new_world, new_rank, k)
    # a missing old rank is an error, not a silently zero-filled slice
    import pytest
    with pytest.raises(AssertionError):
        reshard_state((state_of(4, r) for r in (0, 1, 3)), buckets, 2, 1)


def test_merge_cross_check_dumps_arguments_on_mismatch(tmp_path):
    """DCP_DEBUG_LOG_REDUCTION_ARGS_ON_ERROR: the table-driven torch recomputation of the merge agrees
    with the dense formula, passes a correct result and, for a wrong one, saves the arguments and raises."""
    import pytest
    import torch
    from dcp_b200.ops import block_ops
    torch.manual_seed(0)
    n_src, t, h, d = 3, 5, 2, 8
    part_out = torch.randn(64, h, d)
    part_lse = torch.randn(h, 64)
    part_lse[:, 20:22] = float("-inf")                       # a source that saw no key for two tokens
    src_rows = torch.tensor([3, 20, 40, 50], dtype=torch.int32)
    ops = torch.tensor([[7, t, 0, n_src], [30, 2, 3, 1]], dtype=torch.int32)
    ref = block_ops.merge_tables_reference(ops, src_rows, part_out, part_lse)
    outs = torch.stack([part_out[r:r + t] for r in (3, 20, 40)])
    lses = torch.stack([part_lse[:, r:r + t].t() for r in (3, 20, 40)])
    o, l = block_ops.merge_out_lse_reference(outs, lses)
    assert ref[0][0] == 7 and torch.allclose(ref[0][1], o) and torch.allclose(ref[0][2], l.t())
    assert torch.allclose(ref[1][1], part_out[50:52])          # a single source is copied
    out, lse = torch.zeros(64, h, d), torch.zeros(h, 64)
    for dst, oo, ll in ref:
        out[dst:dst + oo.shape[0]] = oo
        lse[:, dst:dst + oo.shape[0]] = ll
    block_ops.check_merge_against_reference(ops, src_rows, part_out, part_lse, out, lse, str(tmp_path))
    assert not list(tmp_path.iterdir())
    out[8, 1, 3] += 1.0
    with pytest.raises(RuntimeError, match="disagrees"):
        block_ops.check_merge_against_reference(ops, src_rows, part_out, part_lse, out, lse, str(tmp_path))
    saved = torch.load(next(tmp_path.iterdir()), weights_only=False)
    assert saved["op_index"] == 0 and torch.equal(saved["ops"], ops)


def test_shared_planning_gives_every_rank_the_plan_it_would_compute_itself():
    """One planner (rank 0) plans every batch once in its worker pool and publishes per-rank shares in
    a key-value store; the other ranks only read.  Every rank must receive exactly the plan it would
    have computed alone, entries must be deleted after the last reader (two readers per rank here, as
    with tensor parallelism), and nothing may be planned twice."""
    import threading
    import torch
    from dcp_b200.data import synth
    from dcp_b200.data.kv_store import KVStore
    from dcp_b200.data.plan_service import PlanSpec, SharedPlanService, plan_iteration
    spec = PlanSpec(4, 2, 8192, 8, 2, 128, 512, 0, "causal", synth.LengthDist("lognormal", 1024.0, 0.7, 128, 4096))
    store = KVStore()
    readers = 2
    svcs = {(r, t): SharedPlanService(spec, r, store, (r, t) == (0, 0), n_workers=2, lookahead=2, readers=readers,
                                      timeout_s=120.0) for r in range(4) for t in range(readers)}
    got, errs = {}, []

    def run(key):
        try:
            got[key] = [svcs[key].get(i) for i in range(3)]
        except Exception as e:     # surfaced below; a thread must not die silently
            errs.append((key, repr(e)))

    threads = [threading.Thread(target=run, args=(k,)) for k in svcs]
    [t.start() for t in threads]
    [t.join(300) for t in threads]
    svcs[(0, 0)].close()
    assert not errs, errs
    assert 3 <= svcs[(0, 0)].n_published <= 5      # each batch once; up to two planned ahead may be out already
    for (r, t), plans in got.items():
        for i, p in enumerate(plans):
            ref = plan_iteration(spec, i, r)
            assert torch.equal(ref.tokens, p.tokens) and torch.equal(ref.labels, p.labels)
            assert (ref.program.merge_ops == p.program.merge_ops).all() and ref.program.q_rows == p.program.q_rows
            assert all(torch.equal(a.tiles, b.tiles) for a, b in zip(ref.program.fwd, p.program.fwd) if a is not None)
    # iterations planned ahead of the last get() may still sit in the store; the consumed ones must be gone
    left = [k for k in store._local if int(k.split("/")[1]) < 3]
    assert not left, f"plans left in the store after the last reader: {left}"


def test_kv_store_moves_values_larger_than_the_tcp_store_payload_limit():
    """Plans of long batches pickle to more than the 8 MiB a TCPStore message may carry: such values
    travel in pieces behind a header key, read back whole, and deleting removes the pieces too."""
    import os
    from dcp_b200.data.kv_store import KVServer, KVStore
    port = 29700 + os.getpid() % 200
    srv = KVServer("127.0.0.1", port)
    a, b = KVStore("127.0.0.1", port, 10.0), KVStore("127.0.0.1", port, 10.0)
    big = os.urandom(19 << 20)
    a.set("big", big)
    assert b.get("big") == big
    b.delete("big")
    assert not a.exists("big") and not a.exists("big#0")
    a.set("small", b"x" * 100)
    assert b.get("small") == b"x" * 100 and a.add("n", 2) == 2 and b.add("n", 1) == 3
    del srv


def test_torch_caching_allocator_model():
    """Pools, segment sizes, split thresholds, coalescing and cache release of the allocator model."""
    from dcp_b200.memory.allocation_simulator import OutOfArena, TorchCachingAllocatorSimulator as Sim
    MiB = 1 << 20
    sim = Sim()
    a = sim.alloc(1000)                      # small pool: rounded to 1024, one 2 MiB segment
    assert sim.stats() == {"allocated": 1024, "reserved": 2 * MiB, "peak_allocated": 1024, "peak_reserved": 2 * MiB, "segments": 1}
    b = sim.alloc(MiB)                       # still small (<= 1 MiB): same segment, no new reservation
    assert sim.reserved == 2 * MiB
    c = sim.alloc(3 * MiB)                   # large pool: a 20 MiB segment, split (17 MiB remainder kept)
    assert sim.reserved == 22 * MiB and sim.allocated == 1024 + MiB + 3 * MiB
    d = sim.alloc(16 * MiB + 512 * 1024)     # fits the 17 MiB remainder; its 0.5 MiB tail is not split off
    assert sim.reserved == 22 * MiB and sim.allocated == 1024 + MiB + 20 * MiB
    e = sim.alloc(25 * MiB + 1)              # >= 10 MiB: own segment rounded up to 2 MiB
    assert sim.reserved == 22 * MiB + 26 * MiB
    sim.free(c); sim.free(d)                 # neighbours merge back into one 20 MiB block
    assert sim.empty_cache() == 20 * MiB and sim.reserved == 28 * MiB
    sim.free(a); sim.free(b); sim.free(e)
    assert sim.allocated == 0 and sim.empty_cache() == 28 * MiB and sim.stats()["segments"] == 0
    assert sim.peak_reserved == 48 * MiB
    small = Sim(capacity=4 * MiB)            # a cap on reserved bytes: cached segments are released before giving up
    h = [small.alloc(MiB) for _ in range(4)]
    for x in h:
        small.free(x)
    assert small.reserved == 4 * MiB         # two cached 2 MiB segments
    import pytest
    with pytest.raises(OutOfArena):          # a 20 MiB segment cannot be had even after releasing the cache ...
        small.alloc(3 * MiB + MiB // 2)
    assert small.reserved == 0               # ... but the cache was released in the attempt


def test_text_dataset_tokenises_once_and_loads_its_cache(tmp_path):
    """HuggingFaceDataset on in-memory texts with the byte tokenizer: samples, length filter, x2 length
    scaling, the on-disk cache (second construction does not tokenise) and batching by the sampler."""
    from dcp_b200.data.datasets import HuggingFaceDataset, HuggingFaceDatasetConfig, OrderedBatchSampler, byte_tokenizer
    texts = ["hello world " * k for k in (1, 3, 9, 27, 81)] + ["x"]
    cfg = HuggingFaceDatasetConfig(tokenizer_name="bytes", min_seq_len=8, max_seq_len=400, cache_dir=str(tmp_path))
    ds = HuggingFaceDataset(cfg, texts=texts)
    assert not ds.built_from_cache and len(ds) == 5                      # "x" is filtered out
    assert ds.seqlens == [min(12 * k, 400) for k in (1, 3, 9, 27, 81)]
    s = ds[1]
    assert s["tokens"].tolist() == byte_tokenizer(texts[1])[:-1] and s["labels"].tolist() == byte_tokenizer(texts[1])[1:]
    calls = []
    ds2 = HuggingFaceDataset(cfg, texts=texts, tokenizer=lambda t: calls.append(t) or [0])
    assert ds2.built_from_cache and not calls and ds2.seqlens == ds.seqlens
    assert all((a == b).all() for a, b in zip(ds.ids, ds2.ids))
    scaled = HuggingFaceDataset(HuggingFaceDatasetConfig(tokenizer_name="bytes", min_seq_len=8, seqlen_scale=2.0), texts=texts)
    assert scaled.seqlens[0] == 2 * 13 - 1
    batches = list(OrderedBatchSampler(ds, 512, shuffle=False, min_fill=0.0))
    assert sorted(i for b in batches for i in b) == list(range(5))
