"""Analytic cost models used by the planner.

``CommunicationCostModel`` prices a block transfer between two devices (ms) and
``AttnRooflineCostModel`` prices one attention work unit as (tensor-core time, HBM time) in ms.
Interfaces follow dcp/core/cost_model.py:17-245; the defaults are B200 figures (NVLink 5 through
NVSwitch inside a node, measured bf16 tensor throughput and HBM3e copy bandwidth) instead of the
reference's A100 numbers, and the tile shapes in the memory model are those of the sm_100a
kernels (128-query forward tiles, 128-key backward tiles).
"""
from __future__ import annotations

import struct
from typing import Tuple

import numpy as np
import torch

# Gbps; 770 GB/s per direction measured peer copy, 400 Gb/s NIC class inter-node
B200_INTRA_NODE_GBPS = 6160.0
B200_INTER_NODE_GBPS = 400.0
B200_ATTN_TFLOPS = 800.0      # what the hand-written forward kernel sustains, not the MMA peak
B200_HBM_GBS = 6500.0


class CostModel:
    pass


class CommunicationCostModel(CostModel):
    """Latency in ms, bandwidth in Gbps; ``get_cost`` returns ms for ``size`` bytes."""

    def __init__(self, inter_node_latency: float = 0.0, inter_node_bandwidth: float = B200_INTER_NODE_GBPS,
                 intra_node_latency: float = 0.0, intra_node_bandwidth: float = B200_INTRA_NODE_GBPS):
        self.inter_node_latency = inter_node_latency
        self.inter_node_bandwidth = inter_node_bandwidth
        self.intra_node_latency = intra_node_latency
        self.intra_node_bandwidth = intra_node_bandwidth

    def _fields(self):
        return (self.inter_node_latency, self.inter_node_bandwidth, self.intra_node_latency,
                self.intra_node_bandwidth)

    def __repr__(self):
        return "CommunicationCostModel({},{},{},{})".format(*self._fields())

    def __eq__(self, other):
        return isinstance(other, CommunicationCostModel) and self._fields() == other._fields()

    def get_cost(self, src: Tuple[int, int], dst: Tuple[int, int], size: int) -> float:
        if tuple(src) == tuple(dst):
            return 0.0
        megabits = size * 8 / 1e6
        if src[0] == dst[0]:
            return self.intra_node_latency + megabits / self.intra_node_bandwidth
        return self.inter_node_latency + megabits / self.inter_node_bandwidth

    def serialize(self) -> bytes:
        return struct.pack("<4d", *self._fields())

    @classmethod
    def deserialize(cls, data: bytes):
        vals = struct.unpack("<4d", data[:32])
        return cls(*vals), data[32:]


def mask_allowed_elements(mask: torch.Tensor) -> float:
    """Number of (q, k) pairs allowed by a range mask: [2, n_q] or [2, 2, n_q] (range, bound, q)."""
    m = mask.to(torch.int64)
    if m.dim() == 2:
        return float(torch.clamp(m[1] - m[0], min=0).sum())
    if m.dim() == 3:
        a = torch.clamp(m[0][1] - m[0][0], min=0).sum()
        b = torch.clamp(m[1][1] - m[1][0], min=0).sum()
        both = torch.clamp(torch.minimum(m[0][1], m[1][1]) - torch.maximum(m[0][0], m[1][0]), min=0).sum()
        return float(a + b - both)
    raise ValueError(f"Invalid mask shape: {tuple(mask.shape)}")


class AttnRooflineCostModel(CostModel):
    """Roofline estimate of one attention call; ``get_cost`` returns (flops_ms, mem_ms)."""

    FWD_Q_TILE = 128
    BWD_KV_TILE = 128

    def __init__(self, max_tflops: float = B200_ATTN_TFLOPS, max_mem_bw: float = B200_HBM_GBS):
        self.max_tflops = max_tflops  # TFLOP/s
        self.max_mem_bw = max_mem_bw  # GB/s

    def __repr__(self):
        return "AttnRooflineCostModel({},{})".format(self.max_tflops, self.max_mem_bw)

    def __eq__(self, other):
        return (isinstance(other, AttnRooflineCostModel) and self.max_tflops == other.max_tflops
                and self.max_mem_bw == other.max_mem_bw)

    def _get_flops(self, seqlens_q, seqlens_k, nheads, headdim, mask_sparsity, mode="fwd") -> float:
        assert mode in ("fwd", "bwd")
        f = 4.0 * sum(q * k for q, k in zip(seqlens_q, seqlens_k)) * nheads * headdim * mask_sparsity
        return f if mode == "fwd" else 2.5 * f

    def _get_mem_access(self, seqlens_q, seqlens_k, n_query_groups, headdim, mask_sparsity, mode="fwd") -> float:
        token_bytes = 2 * n_query_groups * headdim
        total = 0.0
        if mode == "fwd":
            # every query tile streams its whole key/value row once
            for q, k in zip(seqlens_q, seqlens_k):
                total += -(-q // self.FWD_Q_TILE) * k * token_bytes
        else:
            total += sum(seqlens_q) * token_bytes  # dO for rowsum(dO * O)
            # every key tile streams q, dO once and adds into dq
            for q, k in zip(seqlens_q, seqlens_k):
                total += 4 * q * -(-k // self.BWD_KV_TILE) * token_bytes
        return total * mask_sparsity

    def get_cost(self, seqlens_q, seqlens_k, mask, n_heads, n_query_groups, headdim, is_forward=True):
        total = float(sum(q * k for q, k in zip(seqlens_q, seqlens_k)))
        sparsity = mask_allowed_elements(mask) / total if total > 0 else 0.0
        mode = "fwd" if is_forward else "bwd"
        flops = self._get_flops(seqlens_q, seqlens_k, n_heads, headdim, sparsity, mode)
        mem = self._get_mem_access(seqlens_q, seqlens_k, n_query_groups if is_forward else n_heads, headdim,
                                   sparsity, mode)
        return flops / self.max_tflops * 1e-9, mem / self.max_mem_bw * 1e-6

    def pair_cost(self, n_q: int, n_k: int, allowed: float, n_heads: int, n_query_groups: int, headdim: int,
                  is_forward: bool = True) -> float:
        """max(flops, mem) ms of one (q block, kv block) unit given its allowed pair count."""
        if n_q * n_k == 0:
            return 0.0
        sp = allowed / (n_q * n_k)
        mode = "fwd" if is_forward else "bwd"
        f = self._get_flops([n_q], [n_k], n_heads, headdim, sp, mode) / self.max_tflops * 1e-9
        m = self._get_mem_access([n_q], [n_k], n_query_groups if is_forward else n_heads, headdim, sp,
                                 mode) / self.max_mem_bw * 1e-6
        return max(f, m)

    def serialize(self) -> bytes:
        return struct.pack("<2d", self.max_tflops, self.max_mem_bw)

    @classmethod
    def deserialize(cls, data: bytes):
        a, b = struct.unpack("<2d", data[:16])
        return cls(a, b), data[16:]
