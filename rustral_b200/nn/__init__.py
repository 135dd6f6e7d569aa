"""Layers and models."""
from .linear import Linear, LinearConfig, LinearBuilder, LinearReLU, LinearGELU, LinearSiLU, FusionHelper
from .embedding import Embedding, EmbeddingConfig
from .normalization import LayerNorm, LayerNormConfig, RMSNorm, BatchNorm, BatchNormConfig
from .dropout import Dropout, DropoutConfig
from .loss import MSELoss, CrossEntropyLoss, BCEWithLogitsLoss
from .attention import (SelfAttentionConfig, SelfAttention, MultiHeadAttention, TapeMultiHeadAttention, FlashAttention,
                        FlashAttentionConfig, AttentionMemoryStats, TapeFeedForward, SwiGLUFeedForward,
                        TapeTransformerEncoderConfig, TapeTransformerEncoderLayer, TransformerEncoderBlock, causal_mask,
                        causal_mask_tape, scaled_dot_product_attention)
from .transformer import (PositionalEncoding, TransformerEncoderConfig, TransformerEncoderLayer, TransformerEncoder,
                          TransformerDecoderConfig, TransformerDecoderLayer, TransformerDecoder, TransformerEncoderDecoder,
                          EncoderDecoderConfig)
from .moe import MoEConfig, TopKGating, GatingOutput, Expert, ExpertLayer, MoEOutput, ExpertParallel, MoEStats
from .expert_choice import (ExpertChoiceConfig, ExpertChoiceRouter, ExpertChoiceStats, RoutingComparison, ExpertAssignments,
                            TokenAssignment)
from .shared_expert import (SharedExpertConfig, ExpertMLP, SharedExpertLayer, SharedExpertStats, SharedAndRoutedConfig,
                            HybridRouting)
from .quantization import (QuantizationScheme, QuantConfig, QuantParams, QuantizedLinear, GPTQLinear, DynamicQuantizer,
                           QATTrainer, quantize_model, quantize_model_with_stats, QuantizationStats)
from .conv import Conv2d, Conv2dConfig, max_pool2d, global_max_pool2d
from .lstm import (LstmConfig, GruConfig, LstmState, GruState, BidirectionalOutput, LstmCell, GruCell, RnnCell, StackedLstm,
                   BidirectionalRnn)
from .sequential import Sequential2, Sequential, chain
from .readout import Readout, MultiReadout, BinaryReadout, ReadoutConfig, BinaryPrediction, LabelBinaryPrediction

from ..serve.kv_cache import CacheQuantization, CacheConfig, KVCache, SlidingWindowCache, PagedCache, BatchedCache  # noqa: E402,F401  (the reference keeps these in its nn crate)
__all__ = [n for n in dir() if not n.startswith("_")]
