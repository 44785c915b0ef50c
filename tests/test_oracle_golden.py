"""CPU: the oracle against the vectors produced by the reference's own test oracles and helpers."""
import json
import math
import os

import numpy as np
import torch

from oracle import model as omodel
from oracle import ops
from util import GOLDEN, golden_arrays


def _t(a):
    return torch.from_numpy(np.asarray(a))


def test_slopes_match_reference():
    meta = json.load(open(os.path.join(GOLDEN, "reference_meta.json")))
    from tritonformer_b200.transformer import get_slopes
    for n, want in meta["slopes"].items():
        assert np.allclose(ops.get_slopes(int(n)), want, rtol=0, atol=0)
        assert np.allclose(get_slopes(int(n)), want, rtol=1e-15, atol=0)
    # known answers: 16 heads -> 2^-(i+1)/2 ; 12 heads -> 8 powers of two then 4 interleaved
    assert np.allclose(ops.get_slopes(16), [2 ** (-(i + 1) / 2) for i in range(16)])
    assert np.allclose(ops.get_slopes(12)[8:], [2 ** -0.5, 2 ** -1.5, 2 ** -2.5, 2 ** -3.5])


def test_alibi_table_matches_reference_bitwise():
    g = golden_arrays()
    from tritonformer_b200.transformer import generate_alibi_mask
    for seq, heads in ((64, 4), (96, 12)):
        want = _t(g[f"alibi_{seq}_{heads}"])
        got = ops.alibi_table(seq, heads, torch.float16)
        assert torch.equal(got, want)
        assert torch.equal(generate_alibi_mask(seq, heads, device="cpu")[0], want)


def test_attention_oracle_vs_reference_torch_ref():
    g = golden_arrays()
    for tag in ("a", "b"):
        q, k, v = (_t(g[f"attn_{tag}_{n}"]).float() for n in "qkv")
        want = _t(g[f"attn_{tag}_out"]).float()
        got = ops.attention(q, k, v)
        assert (got - want).abs().max().item() < 2e-3  # reference oracle rounds P and out to fp16


def test_biased_attention_oracle_vs_reference_torch_ref():
    g = golden_arrays()
    for tag in ("a", "b"):
        q, k, v = (_t(g[f"battn_{tag}_{n}"]).float() for n in "qkv")
        bias = _t(g[f"battn_{tag}_bias"])
        want = _t(g[f"battn_{tag}_out"]).float()
        got = ops.attention(q, k, v, bias.float())
        assert (got - want).abs().max().item() < 4e-3


def test_linear_layernorm_softmax_ce_oracles():
    g = golden_arrays()
    x, w, b = _t(g["lin_x"]).float(), _t(g["lin_w"]).float(), _t(g["lin_b"]).float()
    assert (ops.linear(x, w) - _t(g["lin_out"]).float()).abs().max().item() < 5e-3
    assert (ops.linear(x, w, b) - _t(g["lin_out_bias"]).float()).abs().max().item() < 5e-3
    x, a, be = _t(g["ln_x"]).float(), _t(g["ln_alpha"]).float(), _t(g["ln_beta"]).float()
    assert (ops.layer_norm(x, a, be) - _t(g["ln_out"]).float()).abs().max().item() < 1e-2
    assert (ops.softmax(_t(g["sm_x"])) - _t(g["sm_out"])).abs().max().item() < 1e-6
    rows = ops.cross_entropy_rows(_t(g["ce_logits"]).float(), _t(g["ce_labels"]))
    assert abs(rows.mean().item() - float(g["ce_mean"])) < 1e-5
    # out-of-range label rows are skipped
    lab = _t(g["ce_labels"]).clone()
    lab[0] = -1
    assert ops.cross_entropy_rows(_t(g["ce_logits"]).float(), lab)[0].item() == 0.0


def _cfg(**kw):
    from tritonformer_b200.transformer import TransformerConfig
    base = dict(vocab_size=512, hidden_size=64, max_position_embeddings=128, num_attention_heads=4,
                head_dim=16, ffn_dim=256, num_hidden_layers=2, use_linear_bias=True, attn_bias=False)
    base.update(kw)
    return TransformerConfig(**base)


def test_state_dict_layout_matches_reference():
    meta = json.load(open(os.path.join(GOLDEN, "reference_meta.json")))
    want = meta["state_dict_no_alibi"]
    from tritonformer_b200.transformer import Transformer
    mine = Transformer(_cfg(), device="cpu")
    got = {k: list(v.shape) for k, v in mine.state_dict().items()}
    assert got == want
    assert {str(v.dtype) for v in mine.state_dict().values()} == set(meta["state_dict_dtypes"])
    assert meta["lm_head_is_zero"] and bool((mine.logits_out.weight == 0).all())
    oracle = omodel.OracleTransformer(_cfg())
    assert {k: list(v.shape) for k, v in oracle.state_dict().items()} == want
    # ALiBi variant: no position table, (H, P, P) buffer
    keys = Transformer(_cfg(attn_bias=True), device="cpu").state_dict()
    assert "embed_positions.weight" not in keys and list(keys["attn_bias"].shape) == [4, 128, 128]
    okeys = omodel.OracleTransformer(_cfg(attn_bias=True)).state_dict()
    assert set(okeys) == set(keys)


def test_oracle_model_known_answer_zero_head():
    torch.manual_seed(0)
    m = omodel.OracleTransformer(_cfg())
    ids = torch.randint(0, 512, (2, 64))
    logits, loss = m(ids, ids)
    assert abs(loss.item() - math.log(512)) < 1e-5 and float(logits.abs().max()) == 0.0
    loss.backward()
    for name, p in m.named_parameters():
        if "logits_out" not in name:
            assert p.grad is None or float(p.grad.abs().max()) == 0.0, name
