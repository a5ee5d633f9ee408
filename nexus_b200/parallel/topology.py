"""Cluster discovery: launcher environment plus the CUDA peer-access / NVLink picture of this node,
and the recommended all-reduce algorithm.  Behind NVSwitch every GPU reaches every peer at full
bandwidth, so a flat algorithm is recommended inside a node and a hierarchical one across nodes.
Parity: include/nexus/dist/topology.hpp and src/dist/topology.cpp of the reference."""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import List


@dataclass
class ClusterInfo:
    rank: int = 0
    world_size: int = 1
    local_rank: int = 0
    local_world_size: int = 1
    nodes: int = 1
    master_addr: str = "127.0.0.1"
    master_port: int = 29500
    restart_count: int = 0
    gpus: int = 0
    peer_access: List[List[bool]] = field(default_factory=list)
    recommended: str = "ring"


def discover_cluster() -> ClusterInfo:
    e = os.environ
    info = ClusterInfo(rank=int(e.get("RANK", 0)), world_size=int(e.get("WORLD_SIZE", 1)),
                       local_rank=int(e.get("LOCAL_RANK", 0)), local_world_size=int(e.get("LOCAL_WORLD_SIZE", 1)),
                       master_addr=e.get("MASTER_ADDR", "127.0.0.1"), master_port=int(e.get("MASTER_PORT", 29500)),
                       restart_count=int(e.get("NEXUS_RESTART_COUNT", 0)))
    info.nodes = max(1, info.world_size // max(1, info.local_world_size))
    try:
        import torch
        if torch.cuda.is_available():
            n = torch.cuda.device_count()
            info.gpus = n
            info.peer_access = [[i == j or torch.cuda.can_device_access_peer(i, j) for j in range(n)] for i in range(n)]
    except Exception:
        pass
    info.recommended = "hierarchical" if info.nodes > 1 and info.local_world_size > 1 else "ring"
    return info
