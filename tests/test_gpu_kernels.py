"""GPU numerics: every hand-written sm_100a kernel against a plain fp32 PyTorch reference."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from dcp_b200.ops import attention as A
from dcp_b200.ops import block_ops, model_ops


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from dcp_b200.ops import _lib
    assert _lib.available(), "dcp_b200/_kernels.so must be built (python -m dcp_b200.csrc.build)"
    return torch.device("cuda", 0)


def _ranges(kind, nq, off=0):
    r = np.zeros((nq, 4), np.int32)
    i = np.arange(nq)
    if kind == "full":
        r[:, 1] = off
    elif kind == "causal":
        r[:, 1] = i + 1 + off
    elif kind == "two":   # sink + sliding window with a hole between them
        r[:, 1] = 40
        r[:, 2] = np.maximum(40, i + off - 120)
        r[:, 3] = i + 1 + off
    return r


CASES = [
    # nq, kv blocks (tokens per block), block size, hq, hkv, mask kind, key offset
    (128, [128], 128, 1, 1, "full", 128),
    (256, [256, 256, 256], 256, 4, 2, "causal", 512),
    (200, [256, 256, 180], 256, 4, 2, "two", 400),
    (1000, [1024, 1024], 1024, 8, 2, "causal", 1024),
    (77, [512], 512, 2, 1, "two", 300),
]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("variant", [0, 1, 2])   # one tile per CTA with P in TMEM / in smem; two tiles per CTA
def test_attention_forward(dev, case, variant):
    nq, kv_blocks, bs, hq, hkv, kind, off = case
    torch.manual_seed(0)
    nkv = len(kv_blocks) * bs
    q = torch.randn(nq + 128, hq, 128, device=dev).bfloat16()
    kv = torch.randn(nkv + 128, 2, hkv, 128, device=dev).bfloat16()
    out = torch.zeros_like(q)
    lse = torch.zeros(hq, nq + 128, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    rng = _ranges(kind, nq, off)
    row = A.AttnRow(0, nq, list(range(hq)), [(i * bs, n) for i, n in enumerate(kv_blocks)], rng)
    tabs = A.build_fwd_tables([row], bs, dev, tile_m=256 if variant == 2 else 128)
    A.attn_fwd(q, kv, tabs, [out], [lse], 128 ** -0.5, status, variant)
    torch.cuda.synchronize()
    assert status.item() == 0
    valid = torch.zeros(nkv, dtype=torch.bool)
    for i, n in enumerate(kv_blocks):
        valid[i * bs:i * bs + n] = True
    mask = A.ranges_to_dense(rng, nkv) & valid[None]
    ro, rl = A.attention_reference(q[:nq], kv[:nkv, 0], kv[:nkv, 1], mask, 128 ** -0.5)
    fin = torch.isfinite(rl)
    assert (out[:nq].float() - ro).abs().max() < 2e-2
    assert (lse[:, :nq][fin] - rl[fin]).abs().max() < 1e-3
    assert torch.isinf(lse[:, :nq][~fin]).all()


@pytest.mark.parametrize("case", CASES)
def test_attention_backward(dev, case):
    nq, kv_blocks, bs, hq, hkv, kind, off = case
    torch.manual_seed(1)
    nkv = len(kv_blocks) * bs
    q = torch.randn(nq + 128, hq, 128, device=dev).bfloat16()
    kv = torch.randn(nkv + 128, 2, hkv, 128, device=dev).bfloat16()
    dout = torch.randn(nq + 128, hq, 128, device=dev).bfloat16()
    out = torch.zeros_like(q)
    lse = torch.zeros(hq, nq + 128, device=dev)
    delta = torch.zeros_like(lse)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    rng = _ranges(kind, nq, off)
    row = A.AttnRow(0, nq, list(range(hq)), [(i * bs, n) for i, n in enumerate(kv_blocks)], rng)
    scale = 128 ** -0.5
    A.attn_fwd(q, kv, A.build_fwd_tables([row], bs, dev), [out], [lse], scale, status, 0)
    A.attn_delta(out, dout, delta, 0, nq)
    bt = A.build_bwd_tables([row], bs, hq, hkv, dev)
    dq = torch.zeros(nq + 128, hq, 128, device=dev)
    dkv = torch.zeros(nkv + 128, 2, hkv, 128, device=dev)
    A.attn_bwd(q, dout, kv, lse, delta, bt, [dq], [dkv], scale, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    valid = torch.zeros(nkv, dtype=torch.bool)
    for i, n in enumerate(kv_blocks):
        valid[i * bs:i * bs + n] = True
    mask = A.ranges_to_dense(rng, nkv) & valid[None]
    _, _, rdq, rdk, rdv = A.attention_reference_bwd(q[:nq], kv[:nkv, 0], kv[:nkv, 1], mask, scale, dout[:nq])
    rel = lambda a, b: ((a - b).abs().max() / (b.abs().max() + 1e-9)).item()
    assert rel(dq[:nq], rdq) < 2e-2 and rel(dkv[:nkv, 0], rdk) < 2e-2 and rel(dkv[:nkv, 1], rdv) < 2e-2
    assert dq[nq:].abs().max() == 0 and dkv[nkv:].abs().max() == 0     # nothing written past the valid rows


def test_rmsnorm(dev):
    torch.manual_seed(0)
    for hidden in (1024, 4096):
        x = torch.randn(300, hidden, device=dev).bfloat16().requires_grad_(True)
        w = (1 + 0.1 * torch.randn(hidden, device=dev)).bfloat16().requires_grad_(True)
        dy = torch.randn(300, hidden, device=dev).bfloat16()
        y = model_ops.rmsnorm(x, w, 1e-5)
        y.backward(dy)
        xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
        yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
        yr.backward(dy.float())
        assert (y.float() - yr).abs().max() < 3e-2
        assert (x.grad.float() - xr.grad).abs().max() < 5e-2
        assert ((w.grad.float() - wr.grad).abs() / (wr.grad.abs() + 1.0)).max() < 3e-2


def test_swiglu(dev):
    torch.manual_seed(0)
    gu = torch.randn(257, 2 * 1024, device=dev).bfloat16().requires_grad_(True)
    dy = torch.randn(257, 1024, device=dev).bfloat16()
    y = model_ops.swiglu(gu)
    y.backward(dy)
    gr = gu.detach().float().requires_grad_(True)
    g, u = gr.chunk(2, dim=-1)
    yr = torch.nn.functional.silu(g) * u
    yr.backward(dy.float())
    assert ((y.float() - yr).abs() / (yr.abs() + 1.0)).max() < 1e-2
    assert ((gu.grad.float() - gr.grad).abs() / (gr.grad.abs() + 1.0)).max() < 2e-2


def test_cross_entropy(dev):
    torch.manual_seed(0)
    logits = (3 * torch.randn(129, 4096, device=dev)).bfloat16()
    labels = torch.randint(0, 4096, (129,), device=dev)
    labels[5] = -100
    lr = logits.float().requires_grad_(True)
    ref = model_ops.cross_entropy_reference(lr, labels)
    (ref.sum() * 0.25).backward()
    loss = model_ops.cross_entropy_inplace(logits, labels, 0.25)
    assert (loss - ref.detach()).abs().max() < 2e-2
    assert (logits.float() - lr.grad).abs().max() < 2e-3
    assert loss[5] == 0 and logits[5].abs().max() == 0


def test_qkv_rope_split_and_pack(dev):
    torch.manual_seed(0)
    T, hq, hkv = 200, 8, 2
    qkv = torch.randn(T, (hq + 2 * hkv) * 128, device=dev).bfloat16()
    pos = torch.randint(0, 100000, (T,), device=dev)
    cos, sin = model_ops.rope_tables(pos, 500000.0, 128)
    q_arena = torch.zeros(T + 64, hq, 128, device=dev, dtype=torch.bfloat16)
    kv_arena = torch.zeros(T + 64, 2, hkv, 128, device=dev, dtype=torch.bfloat16)
    model_ops.qkv_rope_split(qkv, cos, sin, q_arena, kv_arena, hq, hkv, 32, 16)
    parts = qkv.view(T, hq + 2 * hkv, 128)
    assert (q_arena[32:32 + T].float() - model_ops.rope_reference(parts[:, :hq], cos, sin).float()).abs().max() < 3e-2
    assert (kv_arena[16:16 + T, 0].float() - model_ops.rope_reference(parts[:, hq:hq + hkv], cos, sin).float()).abs().max() < 3e-2
    assert torch.equal(kv_arena[16:16 + T, 1], parts[:, hq + hkv:])
    # the backward kernel applies the transposed rotation: <rope(x), g> == <x, rope^T(g)>
    dq = torch.randn(T + 64, hq, 128, device=dev)
    dkv = torch.randn(T + 64, 2, hkv, 128, device=dev)
    dqkv = model_ops.qkv_rope_pack_bwd(dq, dkv, cos, sin, T, hq, hkv, 32, 16).view(T, hq + 2 * hkv, 128).float()
    x = parts.float()
    lhs = (model_ops.rope_reference(x[:, :hq], cos, sin) * dq[32:32 + T]).sum() + \
          (model_ops.rope_reference(x[:, hq:hq + hkv], cos, sin) * dkv[16:16 + T, 0]).sum() + (x[:, hq + hkv:] * dkv[16:16 + T, 1]).sum()
    rhs = (x * dqkv).sum()
    assert abs(lhs - rhs) / abs(lhs) < 5e-3


def test_merge_out_lse_and_aliases(dev):
    torch.manual_seed(0)
    n, t, h = 3, 150, 4
    outs = torch.randn(n, t, h, 128, device=dev).bfloat16()
    lses = torch.randn(n, t, h, device=dev)
    lses[1, :10] = float("-inf")
    lses[:, 20] = float("-inf")
    o, l = block_ops.flash_attn_update_out_lse(outs, lses)
    ro, rl = block_ops.merge_out_lse_reference(outs, lses)
    fin = torch.isfinite(rl)
    assert (o.float() - ro)[fin].abs().max() < 2e-2
    assert (l - rl)[fin].abs().max() < 1e-4 and torch.isinf(l[~fin]).all()
    assert torch.allclose(block_ops.fused_blockwise_sum(outs).float(), outs.float().sum(0), atol=5e-2)
    block_ops.warmup_triton_ops()


def test_gather_push_cast(dev):
    torch.manual_seed(0)
    src = torch.randn(500, 4, 128, device=dev).bfloat16()
    dst = torch.zeros(300, 4, 128, device=dev, dtype=torch.bfloat16)
    ent = torch.tensor([[0, 10, 5, 100], [0, 400, 150, 77]], dtype=torch.int32, device=dev)
    block_ops.gather_rows(ent, [src], dst, 4 * 128 * 2)
    assert torch.equal(dst[5:105], src[10:110]) and torch.equal(dst[150:227], src[400:477]) and dst[105:150].abs().max() == 0
    stat = torch.randn(4, 500, device=dev)
    sdst = torch.zeros(4, 300, device=dev)
    block_ops.gather_stats(ent, [stat], sdst, 4, 500)
    assert torch.equal(sdst[:, 5:105], stat[:, 10:110])
    acc = torch.ones(300, 4, 128, device=dev)
    g = torch.randn(500, 4, 128, device=dev)
    block_ops.push_add_rows(ent, g, [acc], 4 * 128)     # (peer, src_row, dst_row, n)
    assert torch.allclose(acc[5:105], 1 + g[10:110]) and torch.allclose(acc[150:227], 1 + g[400:477])
    bf = torch.empty(300, 4, 128, device=dev, dtype=torch.bfloat16)
    block_ops.cast_f32_bf16(acc, bf)
    assert torch.equal(bf, acc.bfloat16())


def test_corrupt_tables_are_reported_not_executed(dev):
    """A table entry that points outside its arena makes the kernel set the bad-arguments status
    and skip the work; nothing is stored out of range and the context stays usable."""
    torch.manual_seed(0)
    nq, bs, hq, hkv = 256, 256, 4, 2
    q = torch.randn(nq + 128, hq, 128, device=dev).bfloat16()
    kv = torch.randn(bs + 128, 2, hkv, 128, device=dev).bfloat16()
    dout = torch.randn_like(q)
    out = torch.zeros_like(q)
    lse = torch.zeros(hq, nq + 128, device=dev)
    delta = torch.zeros_like(lse)
    rng = _ranges("causal", nq, 0)
    row = A.AttnRow(0, nq, list(range(hq)), [(0, bs)], rng)
    tabs = A.build_fwd_tables([row], bs, dev)
    tabs.tiles[0, 7] = 1 << 28                       # out_row far past the destination
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    A.attn_fwd(q, kv, tabs, [out], [lse], 128 ** -0.5, status, 0)
    torch.cuda.synchronize()
    assert status.item() == 3
    bt = A.build_bwd_tables([row], bs, hq, hkv, dev)
    bt.items[0, 5] = 1 << 28                         # dq_row far past the accumulator
    status.zero_()
    dq = torch.zeros(nq + 128, hq, 128, device=dev)
    dkv = torch.zeros(bs + 128, 2, hkv, 128, device=dev)
    A.attn_bwd(q, dout, kv, lse, delta, bt, [dq], [dkv], 128 ** -0.5, status)
    torch.cuda.synchronize()
    assert status.item() == 3
    assert torch.isfinite(dq).all() and torch.isfinite(dkv).all()
    assert torch.ones(4, device=dev).sum().item() == 4


def test_barrier_wait_is_bounded(dev):
    """A peer flag nobody sets: the barrier kernel gives up after its deadline and reports it."""
    flags = torch.zeros(64, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    # both "ranks" point at local memory; rank 1 never runs, so flags[1] of rank 0's row stays 0
    block_ops.signal_barrier([flags.data_ptr(), flags[32:].data_ptr()], 0, 2, 1, status, timeout_s=0.2)
    torch.cuda.synchronize()
    assert status.item() == 2
    assert flags[32].item() == 1          # our own arrival was published to the peer's row
    # the context is still usable
    assert torch.ones(4, device=dev).sum().item() == 4


def test_adamw_and_reduce_scatter_single_rank(dev):
    from dcp_b200.parallel.dist_optimizer import FlatBuffers, ShardedAdamW
    torch.manual_seed(0)
    n = 4096
    bufs = FlatBuffers(n, dev)
    bufs.params.copy_(torch.randn(n, device=dev).bfloat16())
    p0 = bufs.params.float().clone()
    opt = ShardedAdamW(bufs, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, clip_grad=None)
    ref_p = p0.clone().requires_grad_(True)
    ref = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for _ in range(3):
        g = torch.randn(n, device=dev).bfloat16()
        bufs.grads.copy_(g)
        opt.step(1.0)
        ref_p.grad = g.float()
        ref.step()
    assert (opt.master - ref_p.detach()).abs().max() < 1e-5
    assert torch.equal(bufs.params, opt.master.bfloat16())
