"""Optimisers over flat parameter storage, and learning-rate schedulers."""
from .flat import AdamW, ParamStore, SGD  # noqa: F401
