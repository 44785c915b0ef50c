"""GPT-2-style causal transformer over the tritonformer_b200 Functions.

Drop-in for the reference model file (transformer.py:24-346): same `TransformerConfig` fields,
same module tree and state-dict keys (`embed_tokens`, `embed_positions`, `layer_list.{i}.
{input_layernorm, attention.{q,k,v,out}_proj, post_attention_layernorm, mlp.{dense_h_to_4h,
dense_4h_to_h}}`, `final_layernorm`, `logits_out`, buffer `attn_bias`), same initialisation
rule, pre-LN blocks, ReLU MLP, learned positions unless ALiBi is on, untied LM head.

Two deliberate differences, both invisible in the results:
  * the shifted loss is computed on the (B*T, V) logits in place -- the last position of each
    sequence carries an out-of-range label, which the cross-entropy kernel skips -- instead of
    copying logits[:, :-1] first (reference transformer.py:333-334);
  * the mean over the B*(T-1) per-token losses is taken in fp32.
"""
import math
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.nn as nn

from . import fast_causal_attention, fast_causal_attention_with_bias
from . import nn as tnn
from .crossentropy import CrossEntropyLossFP32
from .embedding import Embedding
from .fused import LayerNormFork, LinearResidual, MLPResidual, QKVProjection

# The layer runs on fused Functions (residual adds, ReLU mask and the q/k/v input gradients folded into
# kernel epilogues).  Set to False to run the layer module by module through the plain Functions,
# exactly as the reference composes it; results agree to rounding.
USE_FUSED_BLOCKS = True


@dataclass(frozen=True)
class TransformerConfig:
    vocab_size: int
    hidden_size: int
    max_position_embeddings: int
    num_attention_heads: int
    head_dim: int
    ffn_dim: int
    num_hidden_layers: int
    use_linear_bias: bool
    attn_bias: bool


def get_slopes(n: int) -> List[float]:
    """ALiBi slopes: a geometric sequence for power-of-two head counts, interleaved otherwise."""
    def pow2(m):
        first = 2.0 ** (-(2.0 ** -(math.log2(m) - 3)))
        return [first * first ** i for i in range(m)]

    if math.log2(n).is_integer():
        return pow2(n)
    below = 2 ** math.floor(math.log2(n))
    return pow2(below) + get_slopes(2 * below)[0::2][: n - below]


def generate_alibi_mask(seq_len: int, num_heads: int, device="cuda:0", dtype=torch.float16) -> torch.Tensor:
    """(1, H, P, P) additive bias: -slope_h * (i - j) on and below the diagonal, -inf above.

    Built like the reference table: the (negative) distance and the slopes are rounded to `dtype`
    first and multiplied in `dtype`."""
    pos = torch.arange(seq_len, device=device)
    dist = -torch.tril(pos.view(seq_len, 1) - pos.view(1, seq_len)).to(dtype)
    slopes = torch.tensor(get_slopes(num_heads), device=device, dtype=dtype)
    table = dist * slopes[:, None, None]
    upper = ~torch.ones((seq_len, seq_len), dtype=torch.bool, device=device).tril()
    return table.masked_fill(upper, float("-inf"))[None]


def _weights_init(m, num_layers):
    """N(0, 0.02) for linear and embedding weights, zeros for linear biases, (1, 0) for LayerNorm;
    residual output projections get std 0.02/sqrt(2L); the LM head starts at zero."""
    if isinstance(m, tnn.Linear):
        m.weight.data.normal_(mean=0.0, std=0.02)
        if m.bias is not None:
            nn.init.zeros_(m.bias)
    elif isinstance(m, nn.Embedding):
        m.weight.data.normal_(mean=0.0, std=0.02)
    elif isinstance(m, tnn.LayerNorm):
        nn.init.ones_(m.weight)
        nn.init.zeros_(m.bias)
    resid_std = 0.02 / math.sqrt(2 * num_layers)
    for name, p in m.named_parameters():
        if "weight" not in name:
            continue
        if "out_proj" in name or "dense_4h_to_h" in name:
            p.data.normal_(mean=0.0, std=resid_std)
        elif "logits_out" in name:
            p.data.zero_()


class CausalAttention(nn.Module):
    """Multi-head causal self-attention with separate q/k/v/out projections."""

    def __init__(self, config: TransformerConfig, device=None):
        super().__init__()
        d = config.hidden_size
        self.hidden_size = d
        self.num_attention_heads = config.num_attention_heads
        self.hidden_size_per_attention_head = d // config.num_attention_heads
        for name in ("q_proj", "k_proj", "v_proj", "out_proj"):
            setattr(self, name, tnn.Linear(d, d, bias=False, device=device, dtype=torch.float16))

    def _heads(self, x: torch.Tensor) -> torch.Tensor:
        b, s, _ = x.shape
        # (b, s, nh*hd) -> (b, nh, s, hd) as a strided view, no copy
        return x.view(b, s, self.num_attention_heads, self.hidden_size_per_attention_head).transpose(1, 2)

    def forward(self, hidden_states: torch.Tensor, attn_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        b, s, d = hidden_states.shape
        q = self._heads(self.q_proj(hidden_states))
        k = self._heads(self.k_proj(hidden_states))
        v = self._heads(self.v_proj(hidden_states))
        if attn_bias is None:
            ctx = fast_causal_attention.apply(q, k, v)
        else:
            ctx = fast_causal_attention_with_bias.apply(q, k, v, attn_bias)
        # the output keeps q's layout, so this is a view of a contiguous (b, s, d) buffer
        ctx = ctx.transpose(1, 2).contiguous().view(b, s, d)
        return self.out_proj(ctx)


class MLPBlock(nn.Module):
    """relu(x W1 [+ b1]) W2 [+ b2]"""

    def __init__(self, config: TransformerConfig, device=None):
        super().__init__()
        self.dense_h_to_4h = tnn.Linear(config.hidden_size, config.ffn_dim, bias=config.use_linear_bias,
                                        fuse_activation=True, device=device, dtype=torch.float16)
        self.dense_4h_to_h = tnn.Linear(config.ffn_dim, config.hidden_size, bias=config.use_linear_bias,
                                        device=device, dtype=torch.float16)

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        return self.dense_4h_to_h(self.dense_h_to_4h(hidden_states))


class TransformerLayer(nn.Module):
    """Pre-LayerNorm block: x + attn(ln(x)), then x + mlp(ln(x))."""

    def __init__(self, config: TransformerConfig, device=None):
        super().__init__()
        self.input_layernorm = tnn.LayerNorm(config.hidden_size, device=device, dtype=torch.float16)
        self.post_attention_layernorm = tnn.LayerNorm(config.hidden_size, device=device, dtype=torch.float16)
        self.attention = CausalAttention(config, device=device)
        self.mlp = MLPBlock(config, device=device)

    def forward(self, hidden_states: torch.Tensor, attn_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        if not USE_FUSED_BLOCKS or not hidden_states.is_cuda:
            hidden_states = hidden_states + self.attention(self.input_layernorm(hidden_states), attn_bias)
            return hidden_states + self.mlp(self.post_attention_layernorm(hidden_states))
        att, mlp = self.attention, self.mlp
        ln1, ln2 = self.input_layernorm, self.post_attention_layernorm
        normed, residual = LayerNormFork.apply(hidden_states, ln1.weight, ln1.bias, ln1.eps)
        q, k, v = QKVProjection.apply(normed, att.q_proj.weight, att.k_proj.weight, att.v_proj.weight)
        b, s, d = q.shape
        q, k, v = att._heads(q), att._heads(k), att._heads(v)
        if attn_bias is None:
            ctx = fast_causal_attention.apply(q, k, v)
        else:
            ctx = fast_causal_attention_with_bias.apply(q, k, v, attn_bias)
        ctx = ctx.transpose(1, 2).contiguous().view(b, s, d)
        hidden_states = LinearResidual.apply(ctx, att.out_proj.weight, None, residual)
        normed, residual = LayerNormFork.apply(hidden_states, ln2.weight, ln2.bias, ln2.eps)
        return MLPResidual.apply(normed, mlp.dense_h_to_4h.weight, mlp.dense_h_to_4h.bias,
                                 mlp.dense_4h_to_h.weight, mlp.dense_4h_to_h.bias, residual)


class Transformer(nn.Module):
    def __init__(self, config: TransformerConfig, device=None):
        super().__init__()
        self.config = config
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size, device=device,
                                         dtype=torch.float16)
        self.embed_positions = None
        if not config.attn_bias:
            self.embed_positions = nn.Embedding(config.max_position_embeddings, config.hidden_size,
                                                device=device, dtype=torch.float16)
        self.layer_list = nn.ModuleList(
            [TransformerLayer(config, device=device) for _ in range(config.num_hidden_layers)])
        self.final_layernorm = tnn.LayerNorm(config.hidden_size, device=device, dtype=torch.float16)
        self.logits_out = tnn.Linear(config.hidden_size, config.vocab_size, bias=False, device=device,
                                     dtype=torch.float16, fuse_activation=False)
        self.apply(lambda m: _weights_init(m, config.num_hidden_layers))
        if config.attn_bias:
            table = generate_alibi_mask(config.max_position_embeddings, config.num_attention_heads,
                                        device=device if device is not None else "cuda:0")
            self.register_buffer("attn_bias", table[0])
        else:
            self.attn_bias = None

    def projection_weight_groups(self):
        """The (q, k, v) projection weights of every layer: `GradBuckets(..., column_blocks=...)` lays their
        gradients out as column blocks of one matrix, so the three weight gradients are one product."""
        return [(layer.attention.q_proj.weight, layer.attention.k_proj.weight, layer.attention.v_proj.weight)
                for layer in self.layer_list]

    def fuse_projection_weights(self):
        """Re-homes the q, k and v projection weights of every layer as the column blocks of one (d, 3 d) buffer.
        The three parameters, their names and values stay; the fused projection then reads that buffer directly
        instead of concatenating the weights every step.  Anything that replaces the parameters' storage
        afterwards (`.to()`, `.half()`) undoes this, and the projection goes back to concatenating."""
        with torch.no_grad():
            for layer in self.layer_list:
                att = layer.attention
                ws = (att.q_proj.weight, att.k_proj.weight, att.v_proj.weight)
                if not (ws[0].shape == ws[1].shape == ws[2].shape and ws[0].dtype == ws[1].dtype == ws[2].dtype):
                    continue
                rows, d = ws[0].shape
                buf = torch.cat([w.detach() for w in ws], dim=1)
                for i, lin in enumerate((att.q_proj, att.k_proj, att.v_proj)):
                    lin.weight = nn.Parameter(buf[:, i * d:(i + 1) * d], requires_grad=lin.weight.requires_grad)
        return self

    def forward(self, input_ids: torch.Tensor, labels: Optional[torch.Tensor]
                ) -> Tuple[torch.Tensor, torch.Tensor]:
        batch, seq = input_ids.shape
        hidden_states = Embedding.apply(
            input_ids, self.embed_tokens.weight,
            self.embed_positions.weight if self.embed_positions is not None else None)
        for layer in self.layer_list:
            hidden_states = layer(hidden_states, self.attn_bias)
        hidden_states = self.final_layernorm(hidden_states)
        logits = self.logits_out(hidden_states)
        if labels is None:
            return logits
        # position t predicts token t+1; the last position of each sequence has no target
        shifted = torch.full_like(labels, -1)
        shifted[:, :-1] = labels[:, 1:]
        per_token = CrossEntropyLossFP32.apply(logits.view(-1, logits.size(-1)), shifted.view(-1))
        loss = per_token.sum() / (batch * (seq - 1))
        return logits, loss
