"""CPU oracle for the tritonformer forward+backward path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package imports this; only tests/, __graft_entry__.smoke() and the
cpu_baseline / reference legs of bench.py do, and only as the checker or the timed CPU baseline.

Parity status: pinned.  The per-operator functions in oracle/ops.py are checked (tests/
test_oracle_golden.py) against vectors produced by the reference's own test oracles
(`torch_ref`, `torch_linear`, `layer_norm`, `softmax`, `F.cross_entropy` in
tritonformer/test_*.py) and helpers (`get_slopes`, `generate_alibi_mask`, the model's
state-dict layout) imported from the reference tree and run on CPU; the vectors and the script
that made them live in tests/golden/.  The whole-model oracle in oracle/model.py is composed of
those pinned operators following transformer.py:113-346; the reference ships no whole-model
fixture (its `transformer_torch.py` is not in its tree), so that composition is pinned only
through its operators and the known answer loss == ln(vocab) under the reference init.
"""
