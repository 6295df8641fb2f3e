"""Python entry points of the block movement / reduction kernels (csrc/kernels/block_ops.cu) and
torch references of the same operations.  Names used by the reference's ``dcp.ops.fused_ops``
(flash_attn_update_out_lse, fused_blockwise_sum, fused_copy_*, warmup_triton_ops) are kept as
thin aliases; the kernels are ahead-of-time compiled, so the warm-up is a no-op.
"""
from __future__ import annotations

import ctypes
from typing import Sequence

import numpy as np
import torch

from . import _lib
from .attention import _ptr_array

_c_int = ctypes.c_int


def _table(rows, device) -> torch.Tensor:
    a = np.asarray(rows, dtype=np.int32).reshape(-1, 4)
    return torch.from_numpy(a).to(device)


def gather_rows(entries: torch.Tensor, src_ptrs: Sequence, dst: torch.Tensor, row_bytes: int) -> None:
    """entries int32 [n,4] = (peer, src_row, dst_row, n_rows); src_ptrs: arena base per peer."""
    if entries.shape[0] == 0:
        return
    lib = _lib.load()
    _lib.check(lib.dcpk_gather_rows(_lib.ptr(entries), _c_int(entries.shape[0]), _ptr_array(src_ptrs),
                                    _c_int(len(src_ptrs)), _lib.ptr(dst), _c_int(row_bytes), _lib.stream_handle()),
               "gather_rows")


def gather_stats(entries: torch.Tensor, src_ptrs: Sequence, dst: torch.Tensor, n_heads: int, src_stride: int) -> None:
    """Per-head fp32 rows ([heads, rows] layout) from peers into ``dst`` [heads, rows]."""
    if entries.shape[0] == 0:
        return
    lib = _lib.load()
    _lib.check(lib.dcpk_gather_stats(_lib.ptr(entries), _c_int(entries.shape[0]), _ptr_array(src_ptrs),
                                     _c_int(len(src_ptrs)), _lib.ptr(dst), _c_int(n_heads), _c_int(src_stride),
                                     _c_int(dst.shape[1]), _lib.stream_handle()), "gather_stats")


def merge_out_lse(ops: torch.Tensor, src_rows: torch.Tensor, part_out: torch.Tensor, part_lse: torch.Tensor,
                  out: torch.Tensor, lse: torch.Tensor) -> None:
    """ops int32 [n,4] = (dst_row, n_tok, src_off, n_src); src_rows int32 = first partial row per source."""
    if ops.shape[0] == 0:
        return
    lib = _lib.load()
    _lib.check(lib.dcpk_merge_out_lse(_lib.ptr(ops), _c_int(ops.shape[0]), _lib.ptr(src_rows), _lib.ptr(part_out),
                                      _lib.ptr(part_lse), _c_int(part_lse.shape[1]), _lib.ptr(out), _lib.ptr(lse),
                                      _c_int(lse.shape[1]), _c_int(out.shape[1]), _lib.stream_handle()),
               "merge_out_lse")


def push_add_rows(entries: torch.Tensor, src: torch.Tensor, dst_ptrs: Sequence, row_floats: int) -> None:
    """entries int32 [n,4] = (peer, src_row, dst_row, n_rows): dst[peer][dst_row..] += src[src_row..] (fp32)."""
    if entries.shape[0] == 0:
        return
    lib = _lib.load()
    _lib.check(lib.dcpk_push_add_rows(_lib.ptr(entries), _c_int(entries.shape[0]), _lib.ptr(src), _ptr_array(dst_ptrs),
                                      _c_int(len(dst_ptrs)), _c_int(row_floats), _lib.stream_handle()),
               "push_add_rows")


def cast_f32_bf16(src: torch.Tensor, dst: torch.Tensor) -> None:
    lib = _lib.load()
    assert src.numel() == dst.numel() and src.dtype == torch.float32 and dst.dtype == torch.bfloat16
    _lib.check(lib.dcpk_cast_f32_bf16(_lib.ptr(src), _lib.ptr(dst), ctypes.c_long(src.numel()), _lib.stream_handle()),
               "cast_f32_bf16")


def signal_barrier(flag_ptrs: Sequence[int], my_rank: int, world: int, epoch: int, status: torch.Tensor,
                   timeout_s: float = 10.0) -> None:
    if world <= 1:
        return
    lib = _lib.load()
    _lib.check(lib.dcpk_signal_barrier(_ptr_array(flag_ptrs), _c_int(my_rank), _c_int(world),
                                       ctypes.c_uint(epoch & 0xFFFFFFFF), ctypes.c_double(timeout_s), _lib.ptr(status),
                                       _lib.stream_handle()), "signal_barrier")


# --------------------------------------------------------------------------- references
def merge_out_lse_reference(outs: torch.Tensor, lses: torch.Tensor):
    """outs [n, t, h, d], lses [n, t, h] -> merged (out [t,h,d] fp32, lse [t,h] fp32)."""
    lses = lses.float()
    lse = torch.logsumexp(lses, dim=0)
    safe = torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)
    w = torch.exp(lses - safe[None])
    w = torch.where(torch.isinf(lses) & (lses < 0), torch.zeros_like(w), w)
    return (outs.float() * w[..., None]).sum(0), lse


def merge_tables_reference(ops: torch.Tensor, src_rows: torch.Tensor, part_out: torch.Tensor, part_lse: torch.Tensor):
    """What the merge kernel must produce for the table ``ops`` / ``src_rows`` (see ``merge_out_lse``), with
    torch ops: a list of (dst_row, out [n_tok, h, d] fp32, lse [h, n_tok] fp32), one entry per table row."""
    res = []
    src = src_rows.tolist()
    for dst_row, n_tok, src_off, n_src in ops.tolist():
        rows = [src[src_off + j] for j in range(n_src)]
        outs = torch.stack([part_out[r:r + n_tok] for r in rows])                 # [n, t, h, d]
        lses = torch.stack([part_lse[:, r:r + n_tok].t() for r in rows])          # [n, t, h]
        o, l = merge_out_lse_reference(outs, lses)
        res.append((dst_row, o, l.t()))
    return res


def check_merge_against_reference(ops, src_rows, part_out, part_lse, out, lse, dump_dir: str, tol: float = 2e-2) -> None:
    """Debug cross-check of the merge kernel (reference switch DCP_DEBUG_LOG_REDUCTION_ARGS_ON_ERROR,
    dcp/runtime/flash_attention/executor.py:1285-1409): recompute every merged row with torch ops
    and, on a mismatch, save the kernel's arguments and both results to ``dump_dir`` and raise."""
    import os
    for i, (dst_row, o_ref, l_ref) in enumerate(merge_tables_reference(ops, src_rows, part_out, part_lse)):
        n_tok = o_ref.shape[0]
        o_got, l_got = out[dst_row:dst_row + n_tok].float(), lse[:, dst_row:dst_row + n_tok]
        fin = torch.isfinite(l_ref)
        bad_o = (o_got - o_ref).abs().max().item() > tol * max(1.0, o_ref.abs().max().item())
        bad_l = bool(fin.any()) and (l_got[fin] - l_ref[fin]).abs().max().item() > tol
        if bad_o or bad_l:
            os.makedirs(dump_dir, exist_ok=True)
            path = os.path.join(dump_dir, f"reduction_args_op{i}_row{dst_row}.pt")
            torch.save({"ops": ops.cpu(), "src_rows": src_rows.cpu(), "op_index": i, "part_out": part_out.cpu(),
                        "part_lse": part_lse.cpu(), "out_kernel": o_got.cpu(), "lse_kernel": l_got.cpu(),
                        "out_reference": o_ref.cpu(), "lse_reference": l_ref.cpu()}, path)
            raise RuntimeError(f"merge kernel disagrees with the torch reference at table row {i}; arguments saved to {path}")


# --------------------------------------------------------------------------- reference-named aliases
def flash_attn_update_out_lse(out_blocks: torch.Tensor, lse_blocks: torch.Tensor):
    """Merge partial (out, lse): out_blocks [n, t, h, d] bf16, lse_blocks [n, t, h] fp32 -> (out, lse).
    CUDA inputs run the merge kernel, CPU inputs the reference."""
    n, t, h, d = out_blocks.shape
    if not out_blocks.is_cuda:
        o, l = merge_out_lse_reference(out_blocks, lse_blocks)
        return o.to(out_blocks.dtype), l
    part_out = out_blocks.reshape(n * t, h, d).contiguous()
    part_lse = lse_blocks.permute(2, 0, 1).reshape(h, n * t).contiguous()
    out = torch.empty(t, h, d, dtype=out_blocks.dtype, device=out_blocks.device)
    lse = torch.empty(h, t, dtype=torch.float32, device=out_blocks.device)
    ops = _table([(0, t, 0, n)], out_blocks.device)
    src_rows = torch.arange(0, n * t, t, dtype=torch.int32, device=out_blocks.device)
    merge_out_lse(ops, src_rows, part_out, part_lse, out, lse)
    return out, lse.t().contiguous()


def fused_blockwise_sum(src_blocks: torch.Tensor) -> torch.Tensor:
    """Sum over the leading axis with fp32 accumulation (the fused path accumulates with red.add in
    fp32 inside the backward kernel; this standalone form serves plan-compatible executors)."""
    return src_blocks.float().sum(0).to(src_blocks.dtype)


def fused_copy(dst: torch.Tensor, src: torch.Tensor) -> None:
    dst.copy_(src)


fused_copy_bf16 = fused_copy_fp16 = fused_copy_fp32 = fused_copy


def warmup_triton_ops(*args, **kwargs) -> None:
    """Nothing to warm up: every kernel is compiled ahead of time for sm_100a."""
    return None
