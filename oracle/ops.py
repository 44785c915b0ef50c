"""fp32 plain-PyTorch restatement of each operator on the path (test oracle, not product code).

Each function cites the reference code it restates (paths relative to fattorib/tritonformer).
"""
import math

import torch
import torch.nn.functional as F


def linear(x, weight, bias=None, relu=False):
    """x @ W (+ b) (+ ReLU); W is (in, out).  Restates torch_linear (tritonformer/test_linear.py:19-25)
    and the fused epilogue order bias -> ReLU of kernels/gemm.py:562-567."""
    y = torch.matmul(x, weight)
    if bias is not None:
        y = y + bias
    return torch.relu(y) if relu else y


def layer_norm(x, alpha, beta, eps=1e-5):
    """Restates layer_norm (tritonformer/test_layernorm.py:19-23): biased variance over the last dim."""
    return F.layer_norm(x, (x.shape[-1],), alpha, beta, eps)


def softmax(x):
    """Restates softmax (tritonformer/test_softmax.py:18-20)."""
    return F.softmax(x, dim=-1)


def cross_entropy_rows(logits, labels):
    """Per-row -log softmax(logits)[label]; rows whose label is outside [0, V) give 0.
    Restates the per-row quantity of kernels/crossentropy.py:7-44 / F.cross_entropy(reduction='none')
    used by tritonformer/test_crossentropy.py:38."""
    valid = (labels >= 0) & (labels < logits.shape[-1])
    safe = torch.where(valid, labels, torch.zeros_like(labels))
    loss = F.cross_entropy(logits, safe, reduction="none")
    return torch.where(valid, loss, torch.zeros_like(loss))


def embedding(input_ids, tok, pos=None):
    """Token rows plus, with a learned position table, the row of each position.  Restates the head of
    Transformer.forward (transformer.py:311-321): embed_tokens(x) + embed_positions(arange(T))."""
    x = F.embedding(input_ids, tok)
    if pos is not None:
        x = x + F.embedding(torch.arange(input_ids.shape[1], device=input_ids.device), pos)[None]
    return x


def causal_mask(t, device=None):
    return torch.ones((t, t), dtype=torch.bool, device=device).tril()


def attention(q, k, v, bias=None):
    """softmax(causal(q kᵀ / sqrt(hd) + bias)) v for (B, H, T, hd) inputs.

    Restates torch_ref of tritonformer/test_attention.py:43-62 (scale, mask, softmax, @ v) and of
    tritonformer/test_biased_attention.py:79-102 (bias added after scaling).  `bias` is (H, T, T) or
    broadcastable; entries above the diagonal are masked regardless of the bias content, like the
    kernels do (kernels/biased_attention.py:147-152)."""
    t = q.shape[-2]
    s = torch.matmul(q, k.transpose(-2, -1)) / math.sqrt(q.shape[-1])
    if bias is not None:
        s = s + torch.nan_to_num(bias[..., :t, :t].to(s.dtype), neginf=0.0)
    s = s.masked_fill(~causal_mask(t, q.device), float("-inf"))
    return torch.matmul(F.softmax(s, dim=-1), v)


def get_slopes(n):
    """ALiBi slopes; restates get_slopes (transformer.py:37-52)."""
    def pow2(m):
        start = 2 ** (-(2 ** -(math.log2(m) - 3)))
        return [start * start ** i for i in range(m)]

    if math.log2(n).is_integer():
        return pow2(n)
    c = 2 ** math.floor(math.log2(n))
    return pow2(c) + get_slopes(2 * c)[0::2][: n - c]


def alibi_table(seq_len, num_heads, dtype=torch.float16, device="cpu"):
    """(H, P, P) table; restates generate_alibi_mask (transformer.py:55-75) including its rounding:
    distance and slopes are cast to `dtype` and multiplied in `dtype`; -inf above the diagonal."""
    pos = torch.arange(seq_len, device=device)
    a = -torch.tril(pos.view(seq_len, 1).repeat(1, seq_len) - pos.view(1, seq_len))
    a = a.to(dtype)
    slopes = torch.tensor(get_slopes(num_heads), device=device, dtype=dtype)
    table = a * slopes[..., None, None]
    return table.masked_fill(~causal_mask(seq_len, device), float("-inf"))
