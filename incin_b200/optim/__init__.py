"""Optimisers over flat parameter storage, and learning-rate schedulers."""
from .flat import SGD, Adam, AdamW, ParamStore, make_store  # noqa: F401
from .scheduler import ConstantLR, CosineAnnealingLR, LinearLR, LRScheduler, StepLR  # noqa: F401
