"""Optimizer step on the flat gradient buckets: AdamW with fp32 master weights and a dynamic loss scale, all on
the device.

The reference ships no optimizer (its README trains with one); this is the step that follows forward+backward
in a training loop.  `FusedAdamW` works on `dp.GradBuckets`: every bucket of 16-bit gradients gets a flat
16-bit parameter buffer of the same layout (the model's parameters become views of it, names and values
unchanged), and flat fp32 buffers for the master weights and the two moments.  A step is, per bucket, one pass
that looks for inf / nan and one pass that updates; whether the step is taken, the loss scale and the step
count live in device memory, so nothing synchronises the host and the step can be captured in a CUDA graph
together with forward, backward and the gradient all-reduce.
"""
import torch

from . import _lib


class LossScaler:
    """Dynamic loss scale kept on the device: {scale, 1 / scale, good steps since the scale changed, steps taken}
    and the found-inf flag.  Multiply the loss by `scale` (a 0-d tensor) before backward."""

    def __init__(self, device, init_scale=4096.0, growth_factor=2.0, backoff_factor=0.5, growth_interval=2000):
        self.state = torch.tensor([init_scale, 1.0 / init_scale, 0.0, 0.0], device=device, dtype=torch.float32)
        self.found_inf = torch.zeros(1, device=device, dtype=torch.int32)
        self.growth_factor, self.backoff_factor, self.growth_interval = growth_factor, backoff_factor, growth_interval

    @property
    def scale(self):
        return self.state[0]

    @property
    def inv_scale(self):
        return self.state[1:2]

    @property
    def steps_taken(self):
        return self.state[3:4]

    def update(self):
        """After the optimizer's step kernels: adjusts the scale, advances the step count if the step was taken
        and clears the found-inf flag."""
        _lib.check(_lib.lib.tfb_loss_scale_update(self.state.data_ptr(), self.found_inf.data_ptr(),
                                                  self.growth_factor, self.backoff_factor, self.growth_interval,
                                                  _lib.stream_ptr(self.state.device)))


class FusedAdamW:
    """AdamW over the parameters of `buckets` (a `dp.GradBuckets`).  Hyper-parameters as in torch.optim.AdamW."""

    def __init__(self, buckets, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, scaler=None):
        assert 0.5 < betas[0] < 1.0 and 0.0 <= betas[1] < 1.0
        self.buckets = buckets
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        device = buckets.buckets[0].device
        self.scaler = scaler if scaler is not None else LossScaler(device, init_scale=1.0, growth_factor=1.0,
                                                                   backoff_factor=1.0, growth_interval=1 << 30)
        self.params16, self.master, self.exp_avg, self.exp_avg_sq = [], [], [], []
        with torch.no_grad():
            for flat in buckets.buckets:
                p16 = torch.zeros_like(flat)
                self.params16.append(p16)
            # every parameter becomes a view of its bucket's parameter buffer, laid out like its gradient
            for p, gview in buckets._views:
                flat = next(b for b in buckets.buckets if b.untyped_storage().data_ptr() == gview.untyped_storage().data_ptr())
                p16 = self.params16[[id(b) for b in buckets.buckets].index(id(flat))]
                off = gview.storage_offset() - flat.storage_offset()
                view = p16.as_strided(gview.size(), gview.stride(), p16.storage_offset() + off)
                view.copy_(p.detach())
                p.data = view
            for p16 in self.params16:
                self.master.append(p16.float())
                self.exp_avg.append(torch.zeros_like(p16, dtype=torch.float32))
                self.exp_avg_sq.append(torch.zeros_like(p16, dtype=torch.float32))

    def step(self):
        """One optimizer step over every bucket (after the gradient all-reduce).  Skipped as a whole, on the
        device, if any gradient of any bucket is inf or nan."""
        s = self.scaler
        stream = _lib.stream_ptr(self.buckets.buckets[0].device)
        for g in self.buckets.buckets:
            _lib.check(_lib.lib.tfb_grad_check(g.data_ptr(), g.numel(), _lib.dtype_code(g.dtype),
                                               s.found_inf.data_ptr(), stream))
        for g, p16, w, m, v in zip(self.buckets.buckets, self.params16, self.master, self.exp_avg, self.exp_avg_sq):
            _lib.check(_lib.lib.tfb_adamw_step(g.data_ptr(), p16.data_ptr(), w.data_ptr(), m.data_ptr(), v.data_ptr(),
                                               g.numel(), _lib.dtype_code(g.dtype), s.inv_scale.data_ptr(),
                                               s.found_inf.data_ptr(), s.steps_taken.data_ptr(), self.lr,
                                               self.betas[0], self.betas[1], self.eps, self.weight_decay, stream))
        s.update()

    def bytes_per_step(self):
        """Algorithmic HBM bytes of one step: the check reads the gradients once; the update reads gradient,
        master weight and both moments and writes the three fp32 values and the 16-bit parameter."""
        n = sum(b.numel() for b in self.buckets.buckets)
        e = self.buckets.buckets[0].element_size()
        return n * (e + e + 12 + 12 + e)
