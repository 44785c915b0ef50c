"""Shared helpers of the parity tests."""
import os

import numpy as np
import torch

NUM_TEST = int(os.environ.get("NUM_TEST", "2"))
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


def assert_close(got, want, atol, what=""):
    err = (got.double() - want.double()).abs().max().item()
    assert err <= atol, f"{what}: max abs err {err:.3e} > {atol}"
