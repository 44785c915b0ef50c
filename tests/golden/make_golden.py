"""Generates the golden vectors under tests/golden/ by importing the reference project and running
its own test oracles and helpers on CPU.

    python tests/golden/make_golden.py /path/to/reference

What is recorded (all small, seeded):
  * get_slopes(n) for several head counts                      (reference transformer.py:37-52)
  * generate_alibi_mask for (seq, heads) = (64, 4), (96, 12)   (reference transformer.py:55-75)
  * the reference model's state-dict keys and shapes            (reference transformer.py:254-303)
  * inputs and outputs of the reference tests' oracle functions: attention torch_ref,
    biased-attention torch_ref, torch_linear, layer_norm, softmax, F.cross_entropy
    (tritonformer/test_*.py)
The reference hard-codes device "cuda:0" in a few helpers; the script maps that name to the CPU
while it runs them.  The reference's Triton kernels are never launched.
"""
import contextlib
import json
import os
import sys

import numpy as np
import torch

OUT = os.path.dirname(os.path.abspath(__file__))


@contextlib.contextmanager
def cuda0_means_cpu():
    """Strip device='cuda:0' from the factory / .to() calls the reference helpers make."""
    real_to, real_ones, real_tensor = torch.Tensor.to, torch.ones, torch.tensor

    def strip(args, kwargs):
        args = tuple(a for a in args if not (isinstance(a, str) and a.startswith("cuda")))
        kwargs = {k: v for k, v in kwargs.items()
                  if not (k == "device" and (str(v).startswith("cuda")))}
        return args, kwargs

    def to(self, *a, **k):
        a, k = strip(a, k)
        return real_to(self, *a, **k) if (a or k) else self

    def ones(*a, **k):
        a, k = strip(a, k)
        return real_ones(*a, **k)

    def tensor(*a, **k):
        a, k = strip(a, k)
        return real_tensor(*a, **k)

    torch.Tensor.to, torch.ones, torch.tensor = to, ones, tensor
    try:
        yield
    finally:
        torch.Tensor.to, torch.ones, torch.tensor = real_to, real_ones, real_tensor


def main(ref_root):
    sys.path.insert(0, ref_root)
    import transformer as ref_model
    import tritonformer.test_attention as t_attn
    import tritonformer.test_biased_attention as t_battn
    import tritonformer.test_crossentropy as t_ce  # noqa: F401  (F.cross_entropy is the oracle there)
    import tritonformer.test_layernorm as t_ln
    import tritonformer.test_linear as t_lin
    import tritonformer.test_softmax as t_sm

    meta = {"slopes": {str(n): ref_model.get_slopes(n) for n in (4, 8, 12, 16, 20, 32)}}

    cfg = ref_model.TransformerConfig(vocab_size=512, hidden_size=64, max_position_embeddings=128,
                                      num_attention_heads=4, head_dim=16, ffn_dim=256,
                                      num_hidden_layers=2, use_linear_bias=True, attn_bias=False)
    model = ref_model.Transformer(cfg, device="cpu")
    meta["state_dict_no_alibi"] = {k: list(v.shape) for k, v in model.state_dict().items()}
    meta["state_dict_dtypes"] = sorted({str(v.dtype) for v in model.state_dict().values()})
    meta["lm_head_is_zero"] = bool((model.logits_out.weight == 0).all())

    arrays = {}
    with cuda0_means_cpu():
        for seq, heads in ((64, 4), (96, 12)):
            arrays[f"alibi_{seq}_{heads}"] = ref_model.generate_alibi_mask(seq, heads)[0].numpy()
        g = torch.Generator().manual_seed(0)
        # attention without bias: (b, nh, sq, hd)
        for tag, (b, nh, sq, hd) in {"a": (1, 4, 128, 32), "b": (2, 3, 64, 64)}.items():
            q, k, v = (torch.randn((b, nh, sq, hd), generator=g).half() for _ in range(3))
            mask = torch.tril(torch.ones((1, 1, sq, sq), dtype=torch.bool))
            out = t_attn.torch_ref(q, k, v, causal_attn=True, attn_mask=mask)
            arrays.update({f"attn_{tag}_q": q.numpy(), f"attn_{tag}_k": k.numpy(),
                           f"attn_{tag}_v": v.numpy(), f"attn_{tag}_out": out.numpy()})
        # attention with the ALiBi table
        for tag, (b, nh, sq, hd) in {"a": (1, 4, 128, 64), "b": (2, 12, 64, 32)}.items():
            q, k, v = (torch.randn((b, nh, sq, hd), generator=g).half() for _ in range(3))
            bias = t_battn.generate_alibi_mask(sq, nh)[0]
            out = t_battn.torch_ref(q, k, v, bias)
            arrays.update({f"battn_{tag}_q": q.numpy(), f"battn_{tag}_k": k.numpy(),
                           f"battn_{tag}_v": v.numpy(), f"battn_{tag}_bias": bias.numpy(),
                           f"battn_{tag}_out": out.numpy()})
    g = torch.Generator().manual_seed(1)
    # linear: (b, m, n) @ (n, k) (+ bias)
    x = torch.randn((3, 70, 129), generator=g).half()
    w = (torch.randn((129, 67), generator=g) / 129 ** 0.5).half()
    bias = torch.randn((67,), generator=g).half()
    arrays.update({"lin_x": x.numpy(), "lin_w": w.numpy(), "lin_b": bias.numpy(),
                   "lin_out": t_lin.torch_linear(x, w).numpy(),
                   "lin_out_bias": t_lin.torch_linear(x, w, bias).numpy()})
    # layernorm, input distribution of the reference test (3.14 + 0.4 randn)
    x = (3.14 + 0.4 * torch.randn((2, 65, 203), generator=g)).half()
    alpha, beta = torch.randn((203,), generator=g).half(), torch.randn((203,), generator=g).half()
    arrays.update({"ln_x": x.numpy(), "ln_alpha": alpha.numpy(), "ln_beta": beta.numpy(),
                   "ln_out": t_ln.layer_norm(x, alpha, beta).numpy()})
    # softmax fp32
    x = torch.randn((2, 33, 301), generator=g)
    arrays.update({"sm_x": x.numpy(), "sm_out": t_sm.softmax(x).numpy()})
    # cross entropy (the reference compares against F.cross_entropy with mean reduction)
    logits = torch.randn((7, 1031), generator=g).half()
    labels = torch.randint(0, 1031, (7,), generator=g)
    arrays.update({"ce_logits": logits.numpy(), "ce_labels": labels.numpy(),
                   "ce_mean": torch.nn.functional.cross_entropy(logits.float(), labels).numpy()})

    np.savez_compressed(os.path.join(OUT, "reference_vectors.npz"), **arrays)
    with open(os.path.join(OUT, "reference_meta.json"), "w") as f:
        json.dump(meta, f, indent=1, sort_keys=True)
    print("wrote", len(arrays), "arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path to a checkout of fattorib/tritonformer>")
    main(sys.argv[1])
