"""Tensor ops: CUDA tensors run on the hand-written sm_100a kernels, CPU tensors on the reference math.

There is one code path per device class and no third backend: a CUDA tensor never takes an eager
PyTorch route (the native library must be loaded), a CPU tensor takes the fp32 reference route that
also serves as the numerical oracle in the tests.
"""
from .matmul import gemm, linear, act_reference, act_grad_reference
from .norm import layer_norm, rms_norm, norm_forward, norm_backward
from .loss import cross_entropy, cross_entropy_fwd_bwd, softmax, log_softmax
from .attention import flash_attention, attention_reference
from .embed import embedding, embedding_forward, embedding_backward
from .elementwise import (binary, unary, scalar_op, unary_bwd, add_row_vector, sum_dim0, sum_all, transpose2d,
                          gather_rows, scatter_rows, broadcast_to, strided_copy, apply_mask, dropout, argmax_rows,
                          gelu, relu, silu)
from .rotary import rope, rope_, swiglu, swiglu_forward, swiglu_backward
from .optim import adam_step, sgd_step, sumsq, cast_f32_to_bf16

__all__ = [n for n in dir() if not n.startswith("_")]
