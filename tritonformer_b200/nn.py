"""Parameter-holding modules over the Functions (drop-in for tritonformer/nn.py:14-91).

Same constructor arguments, attribute names and state-dict layout: Linear.weight is
(in_features, out_features); parameters are left uninitialised (the model's init fills them).
"""
import torch
import torch.nn as nn

from . import layer_norm, linear_bias, linear_fused_bias_relu, linear_fused_relu, linear_no_bias


class LayerNorm(nn.Module):
    """LayerNorm over the last dimension with elementwise affine parameters."""

    def __init__(self, normalized_shape: int, eps: float = 1e-5, device=None, dtype=None) -> None:
        super().__init__()
        self.normalized_shape = normalized_shape
        self.eps = eps
        self.weight = nn.Parameter(torch.empty(normalized_shape, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.empty(normalized_shape, device=device, dtype=dtype))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        """Intentionally empty: initialisation is the owning model's job."""

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        return layer_norm.apply(input, self.weight, self.bias, self.eps)

    def extra_repr(self) -> str:
        return f"{self.normalized_shape}, eps={self.eps}, elementwise_affine=True"


class Linear(nn.Module):
    """x @ W (+ b), optionally followed by a fused ReLU."""

    _TABLE = {
        (False, False): linear_no_bias,
        (False, True): linear_fused_relu,
        (True, False): linear_bias,
        (True, True): linear_fused_bias_relu,
    }

    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 fuse_activation: bool = False, device=None, dtype=None) -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.weight = nn.Parameter(torch.empty((in_features, out_features), device=device, dtype=dtype))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features, device=device, dtype=dtype))
        else:
            self.register_parameter("bias", None)
        self.fuse_activation = fuse_activation
        self.reset_parameters()

    def reset_parameters(self) -> None:
        """Intentionally empty: initialisation is the owning model's job."""

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        fn = self._TABLE[(self.bias is not None, bool(self.fuse_activation))]
        if self.bias is None:
            return fn.apply(input, self.weight)
        return fn.apply(input, self.weight, self.bias)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"
