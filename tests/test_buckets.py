"""Host logic of the gradient buckets (CPU): flat layout, column-block layout of grouped weights."""
import torch

from tritonformer_b200.dp import GradBuckets


def _params():
    torch.manual_seed(0)
    return [torch.nn.Parameter(torch.randn(s)) for s in [(8, 16), (8, 16), (8, 16), (16, 8), (5,), (3, 7)]]


def test_column_blocks_share_one_matrix():
    ps = _params()
    b = GradBuckets(ps, column_blocks=[(ps[0], ps[1], ps[2])])
    g0, g1, g2 = ps[0].grad, ps[1].grad, ps[2].grad
    assert g0.shape == (8, 16) and g0.stride() == (48, 1) and g1.stride() == (48, 1)
    assert g1.data_ptr() == g0.data_ptr() + 16 * 4 and g2.data_ptr() == g0.data_ptr() + 32 * 4
    whole = torch.as_strided(g0, (8, 48), (48, 1))
    whole.copy_(torch.arange(8 * 48, dtype=torch.float32).view(8, 48))
    assert torch.equal(g1, whole[:, 16:32]) and torch.equal(g2, whole[:, 32:])
    # everything still lives in the flat buckets and nothing overlaps
    b.check_views()
    total = sum(p.grad.numel() for p in ps)
    assert sum(x.numel() for x in b.buckets) >= total
    b.zero()
    for i, p in enumerate(ps):
        p.grad.fill_(float(i + 1))
    for i, p in enumerate(ps):
        assert bool((p.grad == float(i + 1)).all()), i


def test_groups_that_do_not_qualify_fall_back_to_flat_views():
    ps = _params()
    GradBuckets(ps, column_blocks=[(ps[0], ps[3])])  # different shapes
    assert ps[0].grad.is_contiguous() and ps[3].grad.is_contiguous()
    ps = _params()
    GradBuckets(ps, bucket_bytes=8 * 16 * 4, column_blocks=[(ps[0], ps[1], ps[2])])  # one parameter per bucket
    assert all(p.grad.is_contiguous() for p in ps)


def test_partial_clear_skips_what_the_kernels_overwrite():
    """`zero(skip_written=True)` leaves the gradients that were recorded as overwritten and clears the rest:
    other parameters, and the padding between views.  A column-block matrix counts only when ALL of its blocks
    are overwritten."""
    from tritonformer_b200 import linear
    ps = _params()
    b = GradBuckets(ps, column_blocks=[(ps[0], ps[1], ps[2])])
    for x in b.buckets:
        x.fill_(7.0)
    b.zero(skip_written=True)  # nothing recorded yet: everything is cleared
    assert all(bool((x == 0).all()) for x in b.buckets)
    # the block records what kernels would write: the three column blocks and one flat weight
    with b.accumulate(overwrite=True):
        assert linear.accumulating() and linear.overwriting()
        linear.note_written(ps[0].grad, ps[1].grad, ps[2].grad, ps[3].grad)
    assert not linear.accumulating() and not linear.overwriting()
    with b.accumulate():  # the adding mode records nothing
        assert not linear.overwriting()
        linear.note_written(ps[4].grad)
    for x in b.buckets:
        x.fill_(7.0)
    b.zero(skip_written=True)
    for i in (0, 1, 2, 3):
        assert bool((ps[i].grad == 7.0).all()), i      # left alone
    for i in (4, 5):
        assert bool((ps[i].grad == 0.0).all()), i      # cleared
    kept = sum(ps[i].numel() for i in (0, 1, 2, 3))
    assert sum(int((x == 7.0).sum()) for x in b.buckets) == kept  # the padding is cleared too
    # only two of the three column blocks written: the matrix is cleared as a whole
    ps = _params()
    b = GradBuckets(ps, column_blocks=[(ps[0], ps[1], ps[2])])
    with b.accumulate(overwrite=True):
        linear.note_written(ps[0].grad, ps[1].grad)
    for x in b.buckets:
        x.fill_(7.0)
    b.zero(skip_written=True)
    assert all(bool((p.grad == 0.0).all()) for p in ps)


def test_accumulate_blocks_restore_their_switches():
    """The overwrite / deferred-join switches belong to the block that set them, nested or not, and are back to
    their defaults afterwards (also when the block is left by an exception)."""
    from tritonformer_b200 import linear
    assert not linear.accumulating() and not linear.overwriting() and not linear.DEFER_WEIGHT_GRAD_JOIN
    with linear.accumulate_into_grad(overwrite=True, defer_weight_grads=True):
        assert linear.accumulating() and linear.overwriting() and linear.DEFER_WEIGHT_GRAD_JOIN
        with linear.accumulate_into_grad():
            assert linear.accumulating() and not linear.overwriting() and not linear.DEFER_WEIGHT_GRAD_JOIN
        assert linear.overwriting() and linear.DEFER_WEIGHT_GRAD_JOIN
        with linear.accumulate_into_grad(enabled=False):
            assert linear.overwriting()  # a disabled block changes nothing
    assert not linear.accumulating() and not linear.overwriting() and not linear.DEFER_WEIGHT_GRAD_JOIN
    try:
        with linear.accumulate_into_grad(overwrite=True):
            raise ValueError("leave the block")
    except ValueError:
        pass
    assert not linear.accumulating() and not linear.overwriting()
