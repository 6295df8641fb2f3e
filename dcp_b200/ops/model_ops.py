"""Autograd wrappers over the hand-written sm_100a transformer ops (csrc/kernels/model_ops.cu),
each with a plain fp32 PyTorch reference used by the tests.

On a CUDA tensor the kernels always run (a missing library raises); CPU tensors take the
reference path so the model code can be exercised without a GPU.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_c_int, _c_long, _c_float = ctypes.c_int, ctypes.c_long, ctypes.c_float


# --------------------------------------------------------------------------- references (fp32)
def rmsnorm_reference(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


def swiglu_reference(gu: torch.Tensor) -> torch.Tensor:
    g, u = gu.float().chunk(2, dim=-1)
    return (torch.nn.functional.silu(g) * u).to(gu.dtype)


def rope_reference(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [T, H, d], cos/sin [T, d/2]; rotate-half convention.  Computed in fp32, or in fp64 for fp64 input."""
    xf = x.double() if x.dtype == torch.float64 else x.float()
    half = x.shape[-1] // 2
    x1, x2 = xf[..., :half], xf[..., half:]
    c, s = cos[:, None, :].to(xf.dtype), sin[:, None, :].to(xf.dtype)
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


def rope_tables(positions: torch.Tensor, theta: float = 500000.0, dim: int = 128):
    """cos/sin [T, dim/2] in fp32 (computed in fp64 so 131072-token positions stay exact)."""
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float64, device=positions.device) / dim))
    ang = positions.double()[:, None] * inv[None, :]
    return torch.cos(ang).float().contiguous(), torch.sin(ang).float().contiguous()


def cross_entropy_reference(logits: torch.Tensor, labels: torch.Tensor):
    lf = logits.float()
    loss = torch.nn.functional.cross_entropy(lf, labels.clamp(min=0), reduction="none")
    return torch.where(labels >= 0, loss, torch.zeros_like(loss))


# --------------------------------------------------------------------------- RMSNorm
def rmsnorm_fwd_raw(x: torch.Tensor, w: torch.Tensor, eps: float):
    """(y, rstd) for contiguous 2-D bf16 x; no autograd."""
    y = torch.empty_like(x)
    rstd = torch.empty(x.shape[0], dtype=torch.float32, device=x.device)
    _lib.check(_lib.load().dcpk_rmsnorm_fwd(_lib.ptr(x), _lib.ptr(w), _lib.ptr(y), _lib.ptr(rstd), _c_int(x.shape[0]),
                                            _c_int(x.shape[1]), _c_float(eps), _lib.stream_handle()), "rmsnorm_fwd")
    return y, rstd


def rmsnorm_bwd_raw(x: torch.Tensor, w: torch.Tensor, rstd: torch.Tensor, dy: torch.Tensor):
    """(dx bf16, dw fp32) for contiguous 2-D x / dy; no autograd."""
    dx = torch.empty_like(x)
    dw = torch.zeros(x.shape[1], dtype=torch.float32, device=x.device)
    _lib.check(_lib.load().dcpk_rmsnorm_bwd(_lib.ptr(x), _lib.ptr(w), _lib.ptr(dy), _lib.ptr(rstd), _lib.ptr(dx),
                                            _lib.ptr(dw), _c_int(x.shape[0]), _c_int(x.shape[1]), _lib.stream_handle()),
               "rmsnorm_bwd")
    return dx, dw


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        y, rstd = rmsnorm_fwd_raw(x2, w, eps)
        ctx.save_for_backward(x2, w, rstd)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, rstd = ctx.saved_tensors
        dx, dw = rmsnorm_bwd_raw(x2, w, rstd, dy.reshape(x2.shape).contiguous())
        return dx.view(dy.shape), dw.to(w.dtype), None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    if not x.is_cuda:
        return rmsnorm_reference(x, w, eps)
    return _RMSNorm.apply(x, w, eps)


# --------------------------------------------------------------------------- SwiGLU
def swiglu_fwd_raw(gu: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up for contiguous 2-D bf16 [T, 2F] laid out gate | up; no autograd."""
    f = gu.shape[1] // 2
    y = torch.empty(gu.shape[0], f, dtype=gu.dtype, device=gu.device)
    _lib.check(_lib.load().dcpk_swiglu_fwd(_lib.ptr(gu), _lib.ptr(y), _c_long(gu.shape[0]), _c_int(f),
                                           _lib.stream_handle()), "swiglu_fwd")
    return y


def swiglu_bwd_raw(gu: torch.Tensor, dy: torch.Tensor) -> torch.Tensor:
    f = gu.shape[1] // 2
    dgu = torch.empty_like(gu)
    _lib.check(_lib.load().dcpk_swiglu_bwd(_lib.ptr(gu), _lib.ptr(dy), _lib.ptr(dgu), _c_long(gu.shape[0]), _c_int(f),
                                           _lib.stream_handle()), "swiglu_bwd")
    return dgu


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        f = gu.shape[-1] // 2
        g2 = gu.reshape(-1, 2 * f).contiguous()
        ctx.save_for_backward(g2)
        return swiglu_fwd_raw(g2).view(*gu.shape[:-1], f)

    @staticmethod
    def backward(ctx, dy):
        (g2,) = ctx.saved_tensors
        f = g2.shape[1] // 2
        return swiglu_bwd_raw(g2, dy.reshape(-1, f).contiguous()).view(*dy.shape[:-1], 2 * f)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """gate_up [..., 2F] laid out gate | up -> silu(gate) * up [..., F]."""
    if not gate_up.is_cuda:
        return swiglu_reference(gate_up)
    return _SwiGLU.apply(gate_up)


# --------------------------------------------------------------------------- cross entropy
class _CrossEntropy(torch.autograd.Function):
    """Loss per row and dlogits in one pass; the logits tensor is overwritten with its gradient."""

    @staticmethod
    def forward(ctx, logits, labels, grad_scale):
        lib = _lib.load()
        assert logits.is_contiguous() and logits.dim() == 2 and logits.dtype == torch.bfloat16
        loss = torch.empty(logits.shape[0], dtype=torch.float32, device=logits.device)
        _lib.check(lib.dcpk_cross_entropy(_lib.ptr(logits), _lib.ptr(labels), _lib.ptr(loss), _c_int(logits.shape[0]),
                                          _c_int(logits.shape[1]), _c_float(grad_scale), _lib.stream_handle()),
                   "cross_entropy")
        ctx.save_for_backward(logits)  # now holds dlogits * grad_scale
        ctx.mark_dirty(logits)
        return loss

    @staticmethod
    def backward(ctx, dloss):
        (dlogits,) = ctx.saved_tensors
        # the caller folds the loss weighting into grad_scale and sums the loss, so dloss is all ones
        return dlogits, None, None


def cross_entropy_sum(logits: torch.Tensor, labels: torch.Tensor, grad_scale: float = 1.0) -> torch.Tensor:
    """Sum of per-token losses; d(sum * grad_scale)/dlogits is produced in place of ``logits``.
    Rows with a negative label are ignored."""
    if not logits.is_cuda:
        return cross_entropy_reference(logits, labels).sum() * grad_scale
    return _CrossEntropy.apply(logits, labels.contiguous(), grad_scale).sum()


def cross_entropy_inplace(logits: torch.Tensor, labels: torch.Tensor, grad_scale: float):
    """Raw kernel call (no autograd): returns per-row loss, leaves dlogits*grad_scale in ``logits``."""
    lib = _lib.load()
    loss = torch.empty(logits.shape[0], dtype=torch.float32, device=logits.device)
    _lib.check(lib.dcpk_cross_entropy(_lib.ptr(logits), _lib.ptr(labels), _lib.ptr(loss), _c_int(logits.shape[0]),
                                      _c_int(logits.shape[1]), _c_float(grad_scale), _lib.stream_handle()),
               "cross_entropy")
    return loss


# --------------------------------------------------------------------------- QKV split + rotary
def qkv_rope_split(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, q_arena: torch.Tensor,
                   kv_arena: torch.Tensor, hq: int, hkv: int, q_row0: int = 0, kv_row0: int = 0) -> None:
    """qkv bf16 [T, (hq+2hkv)*128] -> rotary(q) into q_arena[q_row0:], rotary(k), v into kv_arena[kv_row0:]."""
    lib = _lib.load()
    n_tok = qkv.shape[0]
    assert qkv.is_contiguous() and qkv.shape[1] == (hq + 2 * hkv) * 128
    _lib.check(lib.dcpk_qkv_rope_split_fwd(_lib.ptr(qkv), _lib.ptr(cos), _lib.ptr(sin), _lib.ptr(q_arena),
                                           _lib.ptr(kv_arena), _c_int(n_tok), _c_int(hq), _c_int(hkv), _c_int(q_row0),
                                           _c_int(kv_row0), _lib.stream_handle()), "qkv_rope_split_fwd")


def qkv_rope_pack_bwd(dq: torch.Tensor, dkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, n_tok: int, hq: int,
                      hkv: int, q_row0: int = 0, kv_row0: int = 0) -> torch.Tensor:
    """fp32 dq [rows, hq, 128], dkv [rows, 2, hkv, 128] -> bf16 dqkv [T, (hq+2hkv)*128] (inverse rotary)."""
    lib = _lib.load()
    out = torch.empty(n_tok, (hq + 2 * hkv) * 128, dtype=torch.bfloat16, device=dq.device)
    _lib.check(lib.dcpk_qkv_rope_pack_bwd(_lib.ptr(dq), _lib.ptr(dkv), _lib.ptr(cos), _lib.ptr(sin), _lib.ptr(out),
                                          _c_int(n_tok), _c_int(hq), _c_int(hkv), _c_int(q_row0), _c_int(kv_row0),
                                          _lib.stream_handle()), "qkv_rope_pack_bwd")
    return out


def adamw_step(master, m, v, grad, param_bf16, lr, beta1, beta2, eps, wd, step, clip_coef=None) -> None:
    lib = _lib.load()
    _lib.check(lib.dcpk_adamw(_lib.ptr(master), _lib.ptr(m), _lib.ptr(v), _lib.ptr(grad), _lib.ptr(param_bf16),
                              _c_long(master.numel()), _c_float(lr), _c_float(beta1), _c_float(beta2), _c_float(eps),
                              _c_float(wd), _c_int(step),
                              _lib.ptr(clip_coef) if clip_coef is not None else ctypes.c_void_p(0),
                              _lib.stream_handle()), "adamw")
