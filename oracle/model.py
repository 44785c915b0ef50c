"""fp32 plain-PyTorch restatement of the reference model (test oracle / CPU baseline).

Follows transformer.py:113-346 of the reference: token (+ learned position) embeddings, L pre-LN
blocks of [LN -> q/k/v projections -> causal attention (+ ALiBi table) -> out projection ->
residual; LN -> relu(x W1 + b1) W2 + b2 -> residual], final LN, untied LM head, loss = mean
cross-entropy of logits[:, :-1] against labels[:, 1:].  Linear weights are (in, out) and applied as
x @ W (tritonformer/nn.py:45-86).  Submodule and parameter names equal the reference's, so
state dicts are interchangeable.
"""
import math
from dataclasses import dataclass

import torch
import torch.nn as nn

from . import ops


@dataclass(frozen=True)
class OracleConfig:
    """The fields of the reference's TransformerConfig (transformer.py:24-34), for callers that must not load
    the product package (the CPU baseline of the benchmark)."""
    vocab_size: int
    hidden_size: int
    max_position_embeddings: int
    num_attention_heads: int
    head_dim: int
    ffn_dim: int
    num_hidden_layers: int
    use_linear_bias: bool
    attn_bias: bool


class _Linear(nn.Module):
    def __init__(self, d_in, d_out, bias, relu=False):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(d_in, d_out))
        self.bias = nn.Parameter(torch.zeros(d_out)) if bias else None
        self.relu = relu
        # Optional boolean mask that replaces the ReLU's own sign test (see `forward`).
        self.forced_mask = None

    def forward(self, x):
        if self.relu and self.forced_mask is not None:
            # ReLU with a prescribed activation pattern: a pre-activation within rounding distance of
            # zero lands on either side in 16-bit arithmetic; evaluating the oracle with the pattern
            # observed in the implementation under test separates arithmetic error from that ambiguity.
            pre = ops.linear(x, self.weight, self.bias, False)
            self.last_pre = pre.detach()
            return pre * self.forced_mask.to(pre.dtype)
        return ops.linear(x, self.weight, self.bias, self.relu)


class _LayerNorm(nn.Module):
    def __init__(self, d, eps=1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d))
        self.bias = nn.Parameter(torch.zeros(d))
        self.eps = eps

    def forward(self, x):
        return ops.layer_norm(x, self.weight, self.bias, self.eps)


class _Attention(nn.Module):
    def __init__(self, d, heads):
        super().__init__()
        self.heads = heads
        self.q_proj = _Linear(d, d, False)
        self.k_proj = _Linear(d, d, False)
        self.v_proj = _Linear(d, d, False)
        self.out_proj = _Linear(d, d, False)

    def forward(self, x, bias):
        b, t, d = x.shape
        split = lambda y: y.view(b, t, self.heads, d // self.heads).transpose(1, 2)
        ctx = ops.attention(split(self.q_proj(x)), split(self.k_proj(x)), split(self.v_proj(x)), bias)
        return self.out_proj(ctx.transpose(1, 2).reshape(b, t, d))


class _MLP(nn.Module):
    def __init__(self, d, ffn, bias):
        super().__init__()
        self.dense_h_to_4h = _Linear(d, ffn, bias, relu=True)
        self.dense_4h_to_h = _Linear(ffn, d, bias)

    def forward(self, x):
        return self.dense_4h_to_h(self.dense_h_to_4h(x))


class _Layer(nn.Module):
    def __init__(self, d, heads, ffn, bias):
        super().__init__()
        self.input_layernorm = _LayerNorm(d)
        self.post_attention_layernorm = _LayerNorm(d)
        self.attention = _Attention(d, heads)
        self.mlp = _MLP(d, ffn, bias)

    def forward(self, x, attn_bias):
        x = x + self.attention(self.input_layernorm(x), attn_bias)
        return x + self.mlp(self.post_attention_layernorm(x))


class OracleTransformer(nn.Module):
    """`config` needs the reference's TransformerConfig fields (any object with those attributes)."""

    def __init__(self, config, bias_dtype=torch.float16):
        super().__init__()
        self.config = config
        d = config.hidden_size
        self.embed_tokens = nn.Embedding(config.vocab_size, d)
        self.embed_positions = None if config.attn_bias else nn.Embedding(config.max_position_embeddings, d)
        self.layer_list = nn.ModuleList(
            [_Layer(d, config.num_attention_heads, config.ffn_dim, config.use_linear_bias)
             for _ in range(config.num_hidden_layers)])
        self.final_layernorm = _LayerNorm(d)
        self.logits_out = _Linear(d, config.vocab_size, False)
        if config.attn_bias:
            # the table carries the reference's rounding (built in `bias_dtype`), then used in fp32
            table = ops.alibi_table(config.max_position_embeddings, config.num_attention_heads, bias_dtype)
            self.register_buffer("attn_bias", table.float())
        else:
            self.attn_bias = None
        init_weights(self, config.num_hidden_layers)

    def forward(self, input_ids, labels=None):
        b, t = input_ids.shape
        x = self.embed_tokens(input_ids)
        if self.embed_positions is not None:
            x = x + self.embed_positions(torch.arange(t, device=x.device))[None]
        for layer in self.layer_list:
            x = layer(x, self.attn_bias)
        logits = self.logits_out(self.final_layernorm(x))
        if labels is None:
            return logits
        rows = ops.cross_entropy_rows(logits[:, :-1].reshape(-1, logits.shape[-1]), labels[:, 1:].reshape(-1))
        return logits, rows.mean()


def init_weights(model, num_layers, lm_head_std=None, generator=None):
    """Reference initialisation (transformer.py:83-105): N(0, 0.02) weights, zero linear biases,
    LayerNorm (1, 0), residual projections N(0, 0.02/sqrt(2L)), LM head zero -- or N(0, lm_head_std)
    when given, because a zero head makes every other gradient vanish."""
    for name, p in model.named_parameters():
        with torch.no_grad():
            if "layernorm" in name:
                p.fill_(1.0) if name.endswith("weight") else p.zero_()
            elif name.endswith("bias"):
                p.zero_()
            elif "out_proj" in name or "dense_4h_to_h" in name:
                p.normal_(0.0, 0.02 / math.sqrt(2 * num_layers), generator=generator)
            elif "logits_out" in name:
                p.normal_(0.0, lm_head_std, generator=generator) if lm_head_std else p.zero_()
            else:
                p.normal_(0.0, 0.02, generator=generator)
