"""Serialisation: safetensors, incin-layout checkpoints with resharding, GGUF / MLX export, inspection."""
from .checkpoint import (GlobalCheckpointManifest, load_checkpoint, load_resharded_checkpoint, load_state_dict,  # noqa: F401
                         save_checkpoint, slice_bytes_for_rank, state_dict)
from .export import export_gguf, export_mlx, inspect_file, read_gguf_index  # noqa: F401
from .limits import DEFAULT_LIMITS, LimitError, ResourceLimits  # noqa: F401
from .safetensors import load_safetensors, save_safetensors  # noqa: F401
