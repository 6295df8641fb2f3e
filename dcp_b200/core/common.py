"""Cluster and model descriptors shared by planner and runtime (dcp/core/common.py:14-95)."""
from __future__ import annotations

import struct
from dataclasses import dataclass, field

from .cost_model import AttnRooflineCostModel, CommunicationCostModel


@dataclass
class ExecutionContext:
    n_devices_per_node: int
    n_nodes: int
    comm_cost_model: CommunicationCostModel = field(default_factory=CommunicationCostModel)
    comp_cost_model: AttnRooflineCostModel = field(default_factory=AttnRooflineCostModel)

    @property
    def n_devices(self) -> int:
        return self.n_devices_per_node * self.n_nodes

    def devices(self):
        return [(n, d) for n in range(self.n_nodes) for d in range(self.n_devices_per_node)]

    def serialize(self) -> bytes:
        return (struct.pack("<2I", self.n_devices_per_node, self.n_nodes) + self.comm_cost_model.serialize()
                + self.comp_cost_model.serialize())

    @classmethod
    def deserialize(cls, data: bytes):
        ndpn, nn = struct.unpack("<2I", data[:8])
        comm, rest = CommunicationCostModel.deserialize(data[8:])
        comp, rest = AttnRooflineCostModel.deserialize(rest)
        return cls(ndpn, nn, comm, comp), rest


@dataclass
class ModelSpec:
    head_dim: int
    n_heads: int
    n_query_groups: int = 1  # number of KV heads

    def serialize(self) -> bytes:
        return struct.pack("<3I", self.head_dim, self.n_heads, self.n_query_groups)

    @classmethod
    def deserialize(cls, data: bytes):
        return cls(*struct.unpack("<3I", data[:12])), data[12:]


def get_default_execution_context(n_devices: int, n_nodes: int) -> ExecutionContext:
    assert n_devices % n_nodes == 0, "devices must divide evenly over nodes"
    return ExecutionContext(n_devices // n_nodes, n_nodes, CommunicationCostModel(), AttnRooflineCostModel())
