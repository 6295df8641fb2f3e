"""The lowering of placements to fused-executor tables, checked on CPU for world sizes the GPU
tests cannot reach: every rank's program is emulated with torch ops (runtime/emulate_fused.py) and
the gathered result is compared with dense masked attention, forward and backward."""
import pytest
import torch

from dcp_b200.core.common import get_default_execution_context
from dcp_b200.core.instructions import BufferType
from dcp_b200.planner import masks
from dcp_b200.planner.compiler import CompilerConfig, InstrCompiler
from dcp_b200.planner.lowering import lower_all
from dcp_b200.planner.validate import PlanValidationError, validate_programs
from dcp_b200.planner.workload import generate_workload, pad_seqlens
from dcp_b200.runtime.emulate_fused import emulate
from dcp_b200.runtime.layout import LocalLayout, gather_local, scatter_to_global
from dcp_b200.runtime.simulate import dense_reference


@pytest.mark.parametrize("world,raw,bs,H,Hkv,mask_name,n_stages", [
    (2, [1000, 300, 640], 256, 4, 2, "causal", None),
    (4, [1000, 300, 2100, 640], 256, 4, 2, "lambda", 2),
    (4, [3000, 700], 512, 4, 4, "shared_question", 3),
    (8, [2048, 1024, 512, 4000, 130], 256, 8, 2, "causal", None),
    (8, [2048, 3100, 900], 256, 4, 1, "causal_blockwise", 4),
])
def test_emulated_programs_match_dense_attention(world, raw, bs, H, Hkv, mask_name, n_stages):
    _check_emulated_case(world, raw, bs, H, Hkv, mask_name, n_stages, H)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_self_check_cases_are_valid_at_every_world_size(world):
    """The batches that ``bench.py`` runs through the GPU self-check on 2 or more GPUs: at every world
    size the driver uses, their kernel tables validate and the emulated programs equal dense attention."""
    from dcp_b200.runtime.selfcheck import DEFAULT_CASES
    for raw, bs, H, Hkv, mask_name, hbs, n_stages in DEFAULT_CASES:
        # the long batch is only validated statically (its dense fp64 attention takes a minute on a CPU)
        _check_emulated_case(world, list(raw), bs, H, Hkv, mask_name, n_stages, hbs, numerics=sum(raw) < 8000)


def _check_emulated_case(world, raw, bs, H, Hkv, mask_name, n_stages, hbs, numerics=True):
    d = 32
    ctx = get_default_execution_context(world, 1)
    pad = pad_seqlens(raw, bs)
    m = masks.get_mask_fn(mask_name)(raw, pad, torch.int32)
    wl = generate_workload((sum(pad), H, d), (sum(pad), 2, Hkv, d), raw, pad, bs, hbs, ctx.comp_cost_model, m,
                           torch.bfloat16)
    fw_wl, _, _, _ = InstrCompiler(ctx, CompilerConfig(n_stages=n_stages)).compile(wl, generate_backward=False)
    progs = lower_all(ctx, fw_wl)
    counts = validate_programs(progs)                     # static cross-rank consistency of the tables
    assert counts["tiles"] > 0 and counts["items"] > 0
    if not numerics:
        return
    devs = ctx.devices()
    T = sum(raw)
    g = torch.Generator().manual_seed(11)
    q = torch.randn(T, H, d, generator=g, dtype=torch.float64)
    kv = torch.randn(T, 2, Hkv, d, generator=g, dtype=torch.float64)
    dout = torch.randn(T, H, d, generator=g, dtype=torch.float64)
    lays = [LocalLayout(fw_wl, dev) for dev in devs]
    res = emulate([progs[dev] for dev in devs],
                  [gather_local(q, lay, BufferType.LOCAL_Q, raw, 1) for lay in lays],
                  [gather_local(kv, lay, BufferType.LOCAL_KV, raw, 2) for lay in lays],
                  [gather_local(dout, lay, BufferType.LOCAL_OUT, raw, 1) for lay in lays])
    out_g, lse_g = torch.zeros(T, H, d, dtype=torch.float64), torch.zeros(H, T, dtype=torch.float64)
    dq_g, dkv_g = torch.zeros(T, H, d, dtype=torch.float64), torch.zeros(T, 2, Hkv, d, dtype=torch.float64)
    for lay, (out, lse, dq, dkv) in zip(lays, res):
        scatter_to_global(out, out_g, lay, BufferType.LOCAL_OUT, raw, 1)
        scatter_to_global(lse, lse_g, lay, BufferType.LOCAL_LSE, raw, 0, token_axis_local=1)
        scatter_to_global(dq, dq_g, lay, BufferType.LOCAL_Q, raw, 1)
        scatter_to_global(dkv, dkv_g, lay, BufferType.LOCAL_KV, raw, 2)
    ro, rl, rdq, rdkv = dense_reference(q, kv, raw, pad, m, d ** -0.5, dout)
    fin = torch.isfinite(rl)
    assert (out_g - ro).abs().max() < 1e-9
    assert (lse_g - rl)[fin].abs().max() < 1e-9
    assert (dq_g - rdq).abs().max() < 1e-8 and (dkv_g - rdkv).abs().max() < 1e-8
    # something actually moved between ranks (otherwise the case would not test the lowering)
    assert sum(int(x.shape[0]) for p in progs.values() for x in p.q_pulls + p.kv_pulls) > 0


def test_program_validator_catches_corrupted_tables():
    import copy
    world, raw, bs, H, Hkv = 4, [1000, 300, 2100, 640], 256, 4, 2
    ctx = get_default_execution_context(world, 1)
    pad = pad_seqlens(raw, bs)
    m = masks.get_mask_fn("causal")(raw, pad, torch.int32)
    wl = generate_workload((sum(pad), H, 32), (sum(pad), 2, Hkv, 32), raw, pad, bs, H, ctx.comp_cost_model, m,
                           torch.bfloat16)
    fw_wl, _, _, _ = InstrCompiler(ctx, CompilerConfig()).compile(wl, generate_backward=False)
    good = list(lower_all(ctx, fw_wl).values())
    validate_programs(good)
    r = next(i for i, p in enumerate(good) if sum(len(t) for t in p.kv_pulls) > 0 and len(p.merge_ops) > 0)

    def corrupted(fn):
        progs = copy.deepcopy(good)
        fn(progs[r])
        return progs

    def drop_pull(p):
        s = next(i for i, t in enumerate(p.kv_pulls) if len(t))
        p.kv_pulls[s] = p.kv_pulls[s][1:]

    def late_pull(p):       # a block pulled one stage after its first reader
        s = next(i for i, t in enumerate(p.kv_pulls) if len(t))
        if s + 1 < p.n_stages:
            import numpy as np
            p.kv_pulls[s + 1] = np.concatenate([p.kv_pulls[s + 1].reshape(-1, 4), p.kv_pulls[s][:1]])
        p.kv_pulls[s] = p.kv_pulls[s][1:]

    def bad_merge(p):
        p.merge_src = p.merge_src.copy()
        p.merge_src[0] += 8

    def lost_push(p):
        p.dkv_push = p.dkv_push[1:]

    def out_of_arena(p):
        s = next(i for i, t in enumerate(p.fwd) if t is not None)
        p.fwd[s].tiles[0, 0] = p.q_rows + 5

    for fn in (drop_pull, late_pull, bad_merge, lost_push, out_of_arena):
        with pytest.raises(PlanValidationError):
            validate_programs(corrupted(fn))


def _assert_same_programs(a, b, desc):
    import dataclasses
    import numpy as np
    assert a.keys() == b.keys(), desc

    def same(x, y, path):
        if dataclasses.is_dataclass(x):
            for f in dataclasses.fields(x):
                if f.name == "relayed_blocks":      # informational: how often the plan relays through a non-owner
                    continue
                same(getattr(x, f.name), getattr(y, f.name), f"{path}.{f.name}")
        elif isinstance(x, (list, tuple)):
            assert len(x) == len(y), (desc, path)
            for i, (u, v) in enumerate(zip(x, y)):
                same(u, v, f"{path}[{i}]")
        elif isinstance(x, torch.Tensor):
            assert x.shape == y.shape and bool((x == y).all()), (desc, path)
        elif isinstance(x, np.ndarray):
            assert x.shape == y.shape and bool((x == y).all()), (desc, path)
        else:
            assert x == y, (desc, path, x, y)

    for dev in a:
        same(a[dev], b[dev], str(dev))


@pytest.mark.parametrize("seed", [1, 2])
def test_random_configurations(seed):
    """Seeded fuzz over world sizes (odd ones included), block sizes, head-block splits, masks, stage
    counts and batches with sequences shorter than a block: the instruction plans pass the symbolic
    executor, the fused tables pass the static validator, and small cases are emulated against dense
    attention (forward and backward)."""
    import random
    from dcp_b200.planner.validate import validate_plans
    rnd = random.Random(seed)
    for case in range(10):
        world = rnd.choice([2, 3, 4, 5, 6, 8])
        bs = rnd.choice([128, 256, 512])
        H, Hkv = rnd.choice([(4, 4), (4, 2), (8, 2), (4, 1)])
        per_group = H // Hkv
        hbs = rnd.choice([h for h in (1, 2, 4, 8) if h <= H and H % h == 0 and (h % per_group == 0 or per_group % h == 0)])
        mask_name = rnd.choice(["causal", "lambda", "shared_question", "causal_blockwise", "chunked_first_chunk"])
        raw = [rnd.choice([17, 100, 128, 129, 300, 700, 1500]) for _ in range(rnd.randint(1, 4))]
        n_stages = rnd.choice([None, 1, 2, 3])
        desc = f"world={world} bs={bs} H={H}/{Hkv} hbs={hbs} mask={mask_name} raw={raw} stages={n_stages}"
        ctx = get_default_execution_context(world, 1)
        pad = pad_seqlens(raw, bs)
        m = masks.get_mask_fn(mask_name)(raw, pad, torch.int32)
        d = 16
        wl = generate_workload((sum(pad), H, d), (sum(pad), 2, Hkv, d), raw, pad, bs, hbs, ctx.comp_cost_model, m,
                               torch.bfloat16)
        fw_wl, bw_wl, fw, bw = InstrCompiler(ctx, CompilerConfig(n_stages=n_stages)).compile(wl)
        validate_plans(ctx, fw_wl, fw, True)
        validate_plans(ctx, bw_wl, bw, False)
        progs = lower_all(ctx, fw_wl)
        validate_programs(progs)
        # the fused programs derived from the instruction streams (here: plans that went through their
        # byte serialisation) are identical to the ones derived from the placed workload
        from dcp_b200.core.instructions import ExecutionPlan
        from dcp_b200.planner.lowering import lower_plans
        fw_bytes = {dev: ExecutionPlan.deserialize(plan.serialize())[0] for dev, plan in fw.items()}
        _assert_same_programs(lower_plans(ctx, fw_wl, fw_bytes), progs, desc)
        if sum(raw) > 2000:
            continue
        devs, T = ctx.devices(), sum(raw)
        g = torch.Generator().manual_seed(case)
        q = torch.randn(T, H, d, generator=g, dtype=torch.float64)
        kv = torch.randn(T, 2, Hkv, d, generator=g, dtype=torch.float64)
        dout = torch.randn(T, H, d, generator=g, dtype=torch.float64)
        lays = [LocalLayout(fw_wl, dev) for dev in devs]
        res = emulate([progs[dev] for dev in devs],
                      [gather_local(q, lay, BufferType.LOCAL_Q, raw, 1) for lay in lays],
                      [gather_local(kv, lay, BufferType.LOCAL_KV, raw, 2) for lay in lays],
                      [gather_local(dout, lay, BufferType.LOCAL_OUT, raw, 1) for lay in lays])
        out_g, dq_g = torch.zeros(T, H, d, dtype=torch.float64), torch.zeros(T, H, d, dtype=torch.float64)
        dkv_g = torch.zeros(T, 2, Hkv, d, dtype=torch.float64)
        for lay, (out, _lse, dq, dkv) in zip(lays, res):
            scatter_to_global(out, out_g, lay, BufferType.LOCAL_OUT, raw, 1)
            scatter_to_global(dq, dq_g, lay, BufferType.LOCAL_Q, raw, 1)
            scatter_to_global(dkv, dkv_g, lay, BufferType.LOCAL_KV, raw, 2)
        ro, _rl, rdq, rdkv = dense_reference(q, kv, raw, pad, m, d ** -0.5, dout)
        err = max((out_g - ro).abs().max().item(), (dq_g - rdq).abs().max().item(), (dkv_g - rdkv).abs().max().item())
        assert err < 1e-8, (desc, err)


def test_copy_jobs_move_exactly_the_pulled_rows():
    """The copy-job form of the pulls (what the attention kernels' fetch warps execute) moves the same
    bytes as the row pulls it was derived from: emulate the job semantics of copy_jobs.cuh on NumPy
    regions for row data (16-byte units, chunked) and for per-head statistics (4-byte units)."""
    import numpy as np
    from dcp_b200.planner import lowering as L
    rng = np.random.default_rng(0)
    world, hq, rows = 3, 4, 700
    row_units = hq * 16                                   # [rows, hq, 128] bf16 -> 16-byte units per row
    src = [rng.integers(0, 1 << 30, size=(rows * row_units, 4), dtype=np.int64).astype(np.uint32) for _ in range(world)]
    stats = [rng.standard_normal((hq, rows)).astype(np.float32) for _ in range(world)]
    pulls = np.asarray([(1, 10, 300, 257), (2, 0, 560, 33), (1, 400, 600, 1)], dtype=np.int32)
    L_saved = L.JOB_CHUNK_UNITS
    L.JOB_CHUNK_UNITS = 1000                              # force several chunks per pull, with a ragged tail
    try:
        jobs = L.row_copy_jobs(pulls, L.KIND_Q, row_units)
    finally:
        L.JOB_CHUNK_UNITS = L_saved
    assert jobs.shape[0] > pulls.shape[0] and (jobs[:, 2] <= 1000).all()
    dst = np.zeros_like(src[0])
    for s_off, d_off, n, where in jobs.tolist():
        assert (where >> 8) & 0xff == L.KIND_Q and not where & (1 << 16)
        dst[d_off:d_off + n] = src[where & 0xff][s_off:s_off + n]
    ref = np.zeros_like(src[0])
    for peer, s_row, d_row, n in pulls.tolist():
        ref[d_row * row_units:(d_row + n) * row_units] = src[peer][s_row * row_units:(s_row + n) * row_units]
    assert (dst == ref).all()
    sjobs = L.stat_copy_jobs(pulls, L.KIND_LSE, hq)
    assert sjobs.shape[0] == pulls.shape[0] * hq
    dst_s, ref_s = np.zeros((hq, rows), np.float32), np.zeros((hq, rows), np.float32)
    for s_off, d_off, n, where in sjobs.tolist():
        assert where & (1 << 16) and (where >> 8) & 0xff == L.KIND_LSE
        h = (where >> 24) & 0xff
        dst_s[h, d_off:d_off + n] = stats[where & 0xff][h, s_off:s_off + n]
    for peer, s_row, d_row, n in pulls.tolist():
        ref_s[:, d_row:d_row + n] = stats[peer][:, s_row:s_row + n]
    assert (dst_s == ref_s).all()


def test_native_table_builders_equal_their_python_twins():
    """csrc/planner/kernel_tables.cpp against the Python builders on random attention rows (ragged
    blocks, empty and reversed ranges, rows without keys, peer destinations): identical arrays."""
    import numpy as np
    from dcp_b200.ops import attention as A
    rng = np.random.default_rng(7)
    for trial in range(60):
        bs = int(rng.choice([128, 256, 512]))
        hq = int(rng.choice([2, 4]))
        rows, q_row = [], 0
        for _ in range(int(rng.integers(1, 6))):
            n_tok = int(rng.integers(1, bs + 1))
            n_kv = int(rng.integers(0, 5))
            kv = [(int(rng.integers(0, 50)) * bs, int(rng.integers(1, bs + 1))) for _ in range(n_kv)]
            span = max(1, n_kv * bs)
            r = np.sort(rng.integers(0, span + 1, size=(n_tok, 4)), axis=1).astype(np.int32)
            kind = rng.integers(0, 4, size=n_tok)
            r[kind == 0, 2:] = 0                                  # single range
            r[kind == 1] = r[kind == 1][:, [1, 0, 3, 2]]          # reversed (empty) ranges
            if trial % 3 == 0:                                    # causal-like: whole tiles fully visible
                r[:, 0], r[:, 1], r[:, 2], r[:, 3] = 0, span, 0, 0
            rows.append(A.AttnRow(q_row, n_tok, list(range(hq)), kv, r, int(rng.integers(0, 3)), int(rng.integers(0, 9)) * bs,
                                  int(rng.integers(0, 3)), int(rng.integers(0, 9)) * bs,
                                  [(int(rng.integers(0, 3)), int(rng.integers(0, 9)) * bs) for _ in kv] if trial % 2 else []))
            q_row += bs
        for tile_m in (A.TILE_M, A.TILE_M_PAIR):
            a, b = A.build_fwd_tables(rows, bs, "cpu", tile_m), A.build_fwd_tables_py(rows, bs, "cpu", tile_m)
            assert torch.equal(a.tiles, b.tiles) and torch.equal(a.kv_entries, b.kv_entries) and torch.equal(a.masks, b.masks)
            assert (a.n_tiles, a.flops, a.tile_m, a.kv_entries.shape) == (b.n_tiles, b.flops, b.tile_m, b.kv_entries.shape)
        a, b = A.build_bwd_tables(rows, bs, hq, 1, "cpu"), A.build_bwd_tables_py(rows, bs, hq, 1, "cpu")
        assert torch.equal(a.ctas, b.ctas) and torch.equal(a.items, b.items) and torch.equal(a.masks, b.masks)
        assert (a.n_ctas, a.n_items, a.flops) == (b.n_ctas, b.n_items, b.flops)
