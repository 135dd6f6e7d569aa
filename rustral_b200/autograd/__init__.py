"""Reverse-mode differentiation facade (Tape) and activation checkpointing."""
from .tape import Tape, TensorId, GradientStore, TapeModule, GradExt
from .checkpoint import (CheckpointConfig, checkpoint_segment, CheckpointedTransformerLayer, CheckpointManager, MemoryStats,
                         checkpoint_model)

__all__ = [n for n in dir() if not n.startswith("_")]
