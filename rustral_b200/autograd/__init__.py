"""Reverse-mode differentiation facade (Tape) and activation checkpointing."""
from .tape import Tape, TensorId, GradientStore, TapeModule, GradExt, GradExtFromStore
from .checkpoint import (CheckpointConfig, CheckpointedSegment, checkpoint_segment, CheckpointedTransformerLayer, CheckpointManager, MemoryStats,
                         checkpoint_model)

__all__ = [n for n in dir() if not n.startswith("_")]
