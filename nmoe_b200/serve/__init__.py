"""Serving side of the curation stack: paged-KV continuous-batching inference for the grading model."""
from .engine import Engine  # noqa: F401
from .kv import BlockPool, Sequence, SeqStatus  # noqa: F401
from .model import ServeConfig, Transformer, pool_hidden  # noqa: F401
