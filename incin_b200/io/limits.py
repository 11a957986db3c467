"""Resource limits applied to every file the framework parses (crates/incin-core/src/io/limits.rs:8-139):
a checkpoint or model file is untrusted input, so sizes are bounded before anything is allocated."""
from __future__ import annotations

from dataclasses import dataclass


class LimitError(ValueError):
    pass


@dataclass(frozen=True)
class ResourceLimits:
    max_file_bytes: int = 1 << 40
    max_header_bytes: int = 100 << 20
    max_tensor_count: int = 1 << 20
    max_metadata_entries: int = 1 << 16
    max_name_bytes: int = 4096
    max_rank: int = 8
    max_dimension: int = 1 << 40
    max_tensor_bytes: int = 1 << 38
    max_total_tensor_bytes: int = 1 << 40
    max_graph_nodes: int = 1 << 20

    def check(self, what: str, value: int, limit: int) -> None:
        if value > limit:
            raise LimitError(f"{what} {value} exceeds the limit {limit}")


DEFAULT_LIMITS = ResourceLimits()
