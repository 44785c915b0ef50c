"""tritonformer_b200: the tritonformer autograd Functions on hand-written sm_100a CUDA.

Same public names as the reference package (tritonformer/__init__.py:1-8).
"""
from .attention import BiasedCausalAttention as fast_causal_attention_with_bias
from .attention import CausalAttention as fast_causal_attention
from .crossentropy import CrossEntropyLoss as cross_entropy_loss
from .layernorm import LayerNorm as layer_norm
from .linear import LinearBias as linear_bias
from .linear import LinearBiasReLU as linear_fused_bias_relu
from .linear import LinearNoBias as linear_no_bias
from .linear import LinearNoBiasReLU as linear_fused_relu
from .softmax import Softmax as softmax

__all__ = [
    "fast_causal_attention_with_bias", "fast_causal_attention", "cross_entropy_loss", "layer_norm",
    "linear_bias", "linear_fused_bias_relu", "linear_no_bias", "linear_fused_relu", "softmax",
]
