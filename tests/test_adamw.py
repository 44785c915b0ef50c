"""GPU parity of the optimizer step (no counterpart in the reference): tfb_adamw_step against torch.optim.AdamW
on fp32 CPU tensors, and the loss-scale logic against torch.amp.GradScaler's documented rule (scale backs off and
the step is skipped when a gradient is inf / nan; after `growth_interval` good steps the scale grows)."""
import pytest
import torch

import tritonformer_b200._lib as L

pytestmark = pytest.mark.gpu


def _ulps(a, b):
    """Distance in units of the last place between two fp32 tensors (same sign assumed where it matters)."""
    ia = a.contiguous().view(torch.int32).long()
    ib = b.contiguous().view(torch.int32).long()
    return (ia - ib).abs()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("n", [8 * 1000, 4099])
def test_adamw_step_matches_torch_adamw(dtype, n):
    torch.manual_seed(0)
    lr, betas, eps, wd = 3e-4, (0.9, 0.95), 1e-8, 0.1
    w0 = torch.randn(n).to(dtype)                       # 16-bit parameters; masters start from their values
    ref = torch.nn.Parameter(w0.float().clone())
    opt = torch.optim.AdamW([ref], lr=lr, betas=betas, eps=eps, weight_decay=wd, foreach=False, fused=False)
    param = w0.cuda()
    master = w0.float().cuda()
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    steps = torch.zeros(1, device="cuda")
    inv_scale = torch.tensor([1.0 / 1024.0], device="cuda")
    found = torch.zeros(1, device="cuda", dtype=torch.int32)
    for it in range(5):
        g = (torch.randn(n) * (0.5 + it)).to(dtype)      # what backward leaves in the bucket, times the loss scale
        ref.grad = g.float()
        opt.step()
        L.check(L.lib.tfb_adamw_step(_scaled(g, dtype).data_ptr(), param.data_ptr(), master.data_ptr(), m.data_ptr(),
                                     v.data_ptr(), n, L.dtype_code(dtype), inv_scale.data_ptr(), found.data_ptr(),
                                     steps.data_ptr(), lr, betas[0], betas[1], eps, wd, L.stream_ptr(param.device)))
        steps += 1
        torch.cuda.synchronize()
        st = opt.state[ref]
        # the scaled 16-bit gradient times 1/1024 is exact (a power of two), so both sides see the same g
        um, uv, uw = (_ulps(a.cpu(), b).max().item() for a, b in ((m, st["exp_avg"]), (v, st["exp_avg_sq"]), (master, ref.detach())))
        print(f"step {it}: worst distance in units of the last place: exp_avg {um}, exp_avg_sq {uv}, master weight {uw}")
        import hashlib
        sig = lambda t: hashlib.sha1(t.detach().cpu().contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()[:10]
        note = (f"step {it}: ulps m {um} v {uv} w {uw}; cpu w {sig(ref)} m {sig(st['exp_avg'])} v {sig(st['exp_avg_sq'])}; "
                f"gpu w {sig(master)} m {sig(m)} v {sig(v)}; g {sig(g)}")
        print(note)
        assert um <= 1 and uv <= 1, note
        assert uw <= it + 2, note  # at most one unit per step on top of identical moments
        assert torch.equal(param.float().cpu(), master.cpu().to(dtype).float())


_keep = []


def _scaled(g16, dtype):
    """The bucket's content: the true gradient times the loss scale 1024, in 16 bits (exact for these values)."""
    t = (g16.float() * 1024.0).to(dtype).cuda()
    assert torch.equal(t.float().cpu() / 1024.0, g16.float())
    _keep.append(t)
    return t


def test_skipped_step_changes_nothing_and_loss_scale_follows_gradscaler_rule():
    from tritonformer_b200.optim import LossScaler
    dev = torch.device("cuda", 0)
    n = 4096
    sc = LossScaler(dev, init_scale=1024.0, growth_factor=2.0, backoff_factor=0.5, growth_interval=3)
    param = torch.randn(n, device=dev).half()
    master, m, v = param.float(), torch.rand(n, device=dev), torch.rand(n, device=dev)
    before = [t.clone() for t in (param, master, m, v)]
    g = torch.randn(n, device=dev).half()
    g[1234] = float("inf")

    def one_step(grad):
        L.check(L.lib.tfb_grad_check(grad.data_ptr(), n, 0, sc.found_inf.data_ptr(), L.stream_ptr(dev)))
        L.check(L.lib.tfb_adamw_step(grad.data_ptr(), param.data_ptr(), master.data_ptr(), m.data_ptr(), v.data_ptr(), n, 0,
                                     sc.inv_scale.data_ptr(), sc.found_inf.data_ptr(), sc.steps_taken.data_ptr(),
                                     1e-3, 0.9, 0.999, 1e-8, 0.0, L.stream_ptr(dev)))
        sc.update()
        torch.cuda.synchronize()

    one_step(g)  # inf: skipped bit for bit, the scale halves, the step count stays, the flag is cleared
    for a, b in zip((param, master, m, v), before):
        assert torch.equal(a, b)
    assert sc.state.tolist() == [512.0, 1.0 / 512.0, 0.0, 0.0] and int(sc.found_inf.item()) == 0
    g[1234] = float("nan")
    one_step(g)
    assert sc.state.tolist() == [256.0, 1.0 / 256.0, 0.0, 0.0]
    good = torch.randn(n, device=dev).half()
    for k in range(1, 4):  # three good steps: the third one doubles the scale
        one_step(good)
        want_scale = 256.0 if k < 3 else 512.0
        assert sc.state.tolist() == [want_scale, 1.0 / want_scale, float(k % 3), float(k)]
    assert not torch.equal(master, before[1])


def test_fused_adamw_trains_the_model_like_torch_adamw():
    """The whole path: buckets, re-homed parameters, overlapped scale handling.  Three steps of a small model against
    torch.optim.AdamW on an fp32 copy fed the same (unscaled) gradients."""
    from tritonformer_b200.dp import GradBuckets
    from tritonformer_b200.optim import FusedAdamW, LossScaler
    from tritonformer_b200.transformer import Transformer, TransformerConfig
    cfg = TransformerConfig(vocab_size=512, hidden_size=128, max_position_embeddings=64, num_attention_heads=2,
                            head_dim=64, ffn_dim=512, num_hidden_layers=2, use_linear_bias=True, attn_bias=False)
    torch.manual_seed(0)
    model = Transformer(cfg, device="cuda")
    with torch.no_grad():
        model.logits_out.weight.normal_(0.0, 0.02)
    names = [n for n, _ in model.named_parameters()]
    state = {k: v.clone() for k, v in model.state_dict().items()}
    buckets = GradBuckets(model.parameters(), column_blocks=model.projection_weight_groups())
    scaler = LossScaler("cuda", init_scale=256.0)
    opt = FusedAdamW(buckets, lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01, scaler=scaler)
    assert [n for n, _ in model.named_parameters()] == names
    for k, v in model.state_dict().items():
        assert torch.equal(v, state[k]), k
    shadow = [torch.nn.Parameter(p.detach().float().cpu().clone()) for p in model.parameters()]
    ref = torch.optim.AdamW(shadow, lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01)
    ids = torch.randint(0, 512, (2, 64), device="cuda")
    for _ in range(3):
        buckets.zero()
        with buckets.accumulate():
            with torch.autocast("cuda", dtype=torch.float16):
                _, loss = model(ids, ids)
            (loss * scaler.scale).backward()
        for s, p in zip(shadow, model.parameters()):
            s.grad = p.grad.detach().float().cpu() / 256.0
        opt.step()
        ref.step()
        buckets.check_views()
        for (n, p), s in zip(model.named_parameters(), shadow):
            assert torch.equal(p.detach().float().cpu(), s.detach().half().float()) or \
                (p.detach().float().cpu() - s.detach()).abs().max().item() <= 2e-3 * s.detach().abs().max().item(), n
    assert float(scaler.state[3].item()) == 3.0
