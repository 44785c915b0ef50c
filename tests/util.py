"""Shared helpers of the parity tests."""
import os

import numpy as np
import torch

# draws per dimension of the seeded shape lists, as in the reference's tests (tritonformer/test_attention.py:10)
NUM_TEST = int(os.environ.get("NUM_TEST", "5"))
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden_arrays():
    return np.load(os.path.join(GOLDEN, "reference_vectors.npz"))


def norm_rel(a: torch.Tensor, b: torch.Tensor) -> float:
    """||a - b|| / ||b|| in fp64."""
    a, b = a.double(), b.double()
    return (torch.linalg.norm(a - b) / torch.linalg.norm(b).clamp_min(1e-30)).item()


def max_rel(a: torch.Tensor, b: torch.Tensor) -> float:
    """max|a - b| / max|b|."""
    a, b = a.double(), b.double()
    return ((a - b).abs().max() / b.abs().max().clamp_min(1e-30)).item()


def assert_close(got, want, atol, what="", rtol=0.0):
    """|got - want| <= atol + rtol * |want| elementwise.  rtol covers the single rounding of a
    16-bit result whose magnitude is above 1 (half an ulp: 4.9e-4 for fp16, 3.9e-3 for bf16)."""
    got, want = got.double(), want.double()
    excess = ((got - want).abs() - rtol * want.abs()).max().item()
    assert excess <= atol, f"{what}: max abs err beyond rtol {excess:.3e} > {atol}"
