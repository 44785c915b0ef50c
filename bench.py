#!/usr/bin/env python
"""Forward+backward throughput of the transformer on the tritonformer_b200 kernels.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config 410m|840m|1.4b] [--impl b200|reference]

One process per GPU (torchrun sets RANK/LOCAL_RANK/WORLD_SIZE for N > 1).  A step is one
`model(tokens, tokens)` + `loss.backward()` under autocast on synthetic tokens, plus, for N > 1, the
gradient all-reduce; per-GPU batch is fixed (weak scaling).  Rank 0 prints ONE JSON line.

`--impl reference` times the fp32 plain-PyTorch restatement of the reference model (oracle/) on the
host cores, on a bounded sample of the same configuration, and prints the same line shape.
"""
import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    # name: (d_model, layers, heads, ffn, vocab, ctx, batch/GPU, dtype, linear bias, ALiBi)
    "160m": (768, 12, 12, 3072, 50304, 1024, 2, "fp16", False, False),  # the CPU-runnable configuration
    "410m": (1024, 24, 16, 4096, 50304, 2048, 4, "fp16", False, False),
    "840m": (1536, 24, 12, 6144, 50304, 4096, 1, "fp16", False, False),
    "1.4b": (2048, 24, 16, 8192, 50304, 2048, 2, "bf16", True, True),
}
METRIC = "fwd+bwd tokens/s, 410M ctx2048 fp16 AMP"


def make_config(name, config_cls=None):
    """`config_cls`: the class that carries the fields (the product's TransformerConfig by default; the CPU arm
    passes the oracle's own, so that it never loads the product package)."""
    if config_cls is None:
        from tritonformer_b200.transformer import TransformerConfig as config_cls
    d, L, H, ffn, V, T, B, dt, lb, ab = CONFIGS[name]
    cfg = config_cls(vocab_size=V, hidden_size=d, max_position_embeddings=T, num_attention_heads=H,
                     head_dim=d // H, ffn_dim=ffn, num_hidden_layers=L, use_linear_bias=lb, attn_bias=ab)
    return cfg, B, T, (torch.float16 if dt == "fp16" else torch.bfloat16)


def algorithmic_flops(cfg, batch, seq):
    """fwd+bwd FLOPs per step: 6*tok*P_mm (every linear incl. the LM head over all positions) plus
    causal attention at half cost (2 products forward, 5 backward)."""
    d, L, ffn, V = cfg.hidden_size, cfg.num_hidden_layers, cfg.ffn_dim, cfg.vocab_size
    hd = d // cfg.num_attention_heads
    p_mm = L * (4 * d * d + 2 * d * ffn) + d * V
    return 6.0 * batch * seq * p_mm + 7.0 * L * batch * cfg.num_attention_heads * seq * seq * hd


def common_flops(cfg, batch, seq, n_params):
    """The widespread 6*N*tok + 12*L*d*T*tok convention (printed for comparison only)."""
    return 6.0 * n_params * batch * seq + 12.0 * cfg.num_hidden_layers * cfg.hidden_size * seq * batch * seq


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"tflops": p.get("bf16_tflops_sustained", 1400.5), "tflops_burst": p.get("bf16_tflops", 1652.3),
                "hbm_gbs": p.get("hbm_gbs", 6535.4), "source": "measured"}
    return {"tflops": 1400.0, "tflops_burst": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except ValueError:
                continue
            for nm, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------- CPU baseline
CPU_CONFIG = "160m"  # d768, 12 layers, 12 heads, ffn 3072, vocab 50304, ctx 1024, batch 2, fp32: the reference model's
                     # CPU-runnable configuration; one step is 1.65 TFLOP by the count of algorithmic_flops()


def cpu_reference_step_time(steps, warmup):
    """Seconds per fwd+bwd step (median) of the fp32 restatement of the reference model on the host cores, on
    the CPU-runnable configuration at its full batch and context.  Loads nothing of the product package."""
    from oracle.model import OracleConfig, OracleTransformer, init_weights
    cfg, batch, seq, _ = make_config(CPU_CONFIG, OracleConfig)
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    gen = torch.Generator().manual_seed(1234)
    model = OracleTransformer(cfg)
    init_weights(model, cfg.num_hidden_layers, lm_head_std=0.02, generator=gen)
    ids = torch.randint(0, cfg.vocab_size, (batch, seq), generator=gen)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        model.zero_grad(set_to_none=True)
        _, loss = model(ids, ids)
        loss.backward()
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    return statistics.median(times), cores, cfg, batch, seq


def _cpu_sample_text(batch, seq, steps):
    return (f"reference model restated in fp32 PyTorch (oracle/), {CPU_CONFIG} configuration (d768 L12 H12 ffn3072 "
            f"V50304), {batch}x{seq} tokens per step, {steps} timed steps, all host cores")


def run_reference_arm(args):
    """The CPU arm: rank 0 times the restated reference model on the host cores; other ranks leave at once."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    t, cores, cfg, sb, ss = cpu_reference_step_time(steps, warmup)
    tok_s = sb * ss / t
    sample = _cpu_sample_text(sb, ss, steps)
    line = {
        "impl": "reference", "metric": METRIC, "value": tok_s, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{CPU_CONFIG} GPT fwd+bwd on the host cores: d{cfg.hidden_size} "
                               f"L{cfg.num_hidden_layers} H{cfg.num_attention_heads} ffn{cfg.ffn_dim} V{cfg.vocab_size} "
                               f"ctx{ss} batch{sb} (the 410M step of the GPU arm does not finish in minutes on a CPU)",
                   "global_batch": sb, "seq_len": ss, "parallelism": "cpu"},
        "tflops": algorithmic_flops(cfg, sb, ss) / t / 1e12,
        "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------- GPU arm
def build_model(cfg, dtype, device, seed=1234):
    """Random-init weights of the architecture: N(0, 0.02) everywhere incl. the LM head
    (the reference init zeroes the head, which would zero every other gradient)."""
    from tritonformer_b200.transformer import Transformer
    torch.manual_seed(seed)
    model = Transformer(cfg, device=device)
    gen = torch.Generator(device="cpu").manual_seed(seed)
    with torch.no_grad():
        w = model.logits_out.weight
        w.copy_(torch.empty(w.shape).normal_(0.0, 0.02, generator=gen).to(w.dtype))
        if cfg.use_linear_bias:
            for n, p in model.named_parameters():
                if n.endswith("bias") and "layernorm" not in n:
                    p.copy_(torch.empty(p.shape).normal_(0.0, 0.02, generator=gen).to(p.dtype))
    if dtype is torch.bfloat16:
        table = model.attn_bias
        model = model.to(torch.bfloat16)
        if table is not None:
            model.attn_bias = table  # the ALiBi table keeps the reference's fp16 rounding
    return model.fuse_projection_weights()


def run_b200_arm(args):
    import tritonformer_b200._lib as L
    from tritonformer_b200 import linear as tlinear
    from tritonformer_b200.dp import GradBuckets, OverlappedReducer, broadcast_parameters

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device: there is no CPU fallback"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        from datetime import timedelta
        # The overlapped all-reduces share the SMs with the backward kernels, whose persistent CTAs
        # (pairs of SMs for the large GEMMs) are delayed by every SM a collective holds: 16 channels
        # measured best here (2 GPUs: 31.2 ms/step against 32.4 with NCCL's default, 34.3 with 4).
        os.environ.setdefault("NCCL_MAX_CTAS", "16")
        # short timeout: a rank that is missing from a collective ends the run instead of stalling it
        opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=os.environ.get("TFB_COMM_PRIORITY", "1") == "1")
        dist.init_process_group("nccl", device_id=dev, timeout=timedelta(seconds=90), pg_options=opts)

    cfg, B, T, dtype = make_config(args.config)
    model = build_model(cfg, dtype, dev)
    broadcast_parameters(model)
    n_params = sum(p.numel() for p in model.parameters())
    # 32 MB buckets: measured at 2 GPUs, 27.2 ms per step and 0.46 ms of all-reduce left after backward, against
    # 27.6 ms and 1.17 ms with 256 MB (the tail is then the 103 MB token table alone, which is ready last)
    bucket_mb = int(os.environ.get("TFB_BUCKET_MB", "32"))
    buckets = GradBuckets(model.parameters(), bucket_bytes=bucket_mb << 20, column_blocks=model.projection_weight_groups())
    loss_scale = 4096.0 if dtype is torch.float16 else 1.0
    optimizer = scaler = None
    if args.optimizer:
        # the step that follows forward+backward in a training loop: loss scale, inf/nan check, AdamW with fp32
        # master weights on the reduced buckets, all on the device (captured in the graph with the rest)
        from tritonformer_b200.optim import FusedAdamW, LossScaler
        scaler = LossScaler(dev, init_scale=loss_scale)
        optimizer = FusedAdamW(buckets, lr=1e-5, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, scaler=scaler)

    gen = torch.Generator().manual_seed(1234 + rank)
    host_tokens = [torch.randint(0, cfg.vocab_size, (B, T), generator=gen).pin_memory() for _ in range(4)]
    static_ids = torch.empty((B, T), dtype=torch.int64, device=dev)
    static_ids.copy_(host_tokens[0])
    static_loss = torch.zeros((), device=dev, dtype=torch.float32)

    # N > 1: each gradient bucket is all-reduced from a hook as soon as backward has produced it, on a
    # side stream, so the collectives overlap the rest of backward (and are captured with the step)
    # TFB_BENCH_FREE_SMS=k: while collectives are in flight the persistent GEMM grids are sized for k SMs fewer
    # (measured at 2 GPUs: 28.8 ms per step with k = 16 or 20 against 28.9 with 0, i.e. no difference; off)
    # TFB_COMM_PRIORITY=0 puts the collectives on a stream of default priority.  On the high-priority stream their
    # CTAs are placed as soon as an SM frees up instead of after the whole grid of the kernel that is running;
    # measured at 2 GPUs on the 1.4B configuration: 42.1 against 43.3 ms per step.
    free_sms = int(os.environ.get("TFB_BENCH_FREE_SMS", "0"))
    reducer = OverlappedReducer(buckets, list(model.layer_list),
                                on_collectives=(lambda on: L.lib.tfb_debug_set(6, free_sms if on else 0)) if free_sms else None,
                                high_priority=os.environ.get("TFB_COMM_PRIORITY", "1") == "1") \
        if (world > 1 and not args.no_overlap) else None

    zero_stream = torch.cuda.Stream()
    # One micro-batch per step and no shared weights: the linear-weight and LayerNorm gradients are written, not
    # added, so only the rest of the buckets (embedding tables, biases) is cleared (TFB_BENCH_OVERWRITE=0: clear
    # everything and add, the general path).
    overwrite = os.environ.get("TFB_BENCH_OVERWRITE", "1") == "1"
    # the weight-gradient products float on their side stream until a bucket is reduced or the step ends (the fused
    # blocks never write a gradient tensor in place; TFB_BENCH_DEFER=0: joined at the end of each backward function)
    defer = os.environ.get("TFB_BENCH_DEFER", "1") == "1"

    def step(ids, marks=None):
        # the gradient buckets are cleared on a side stream while the forward pass runs (nothing reads them
        # before backward), then the weight-gradient GEMMs add into the bucket views themselves
        main = torch.cuda.current_stream()
        zero_stream.wait_stream(main)
        with torch.cuda.stream(zero_stream):
            buckets.zero(skip_written=overwrite)
        with buckets.accumulate(overwrite=overwrite, defer_weight_grads=defer):
            with torch.autocast("cuda", dtype=dtype):
                _, loss = model(ids, ids)
            main.wait_stream(zero_stream)
            (loss * (scaler.scale if scaler is not None else loss_scale)).backward()
        if marks is not None:  # last backward kernel enqueued ...
            marks[0].record()
        if reducer is not None:
            reducer.finish()
        if marks is not None:  # ... and the stream has joined the collectives
            marks[1].record()
        if optimizer is not None and (reducer is not None or world == 1):
            optimizer.step()
        return loss.detach()

    # eager warm-up (also fills every per-shape cache before graph capture)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            step(static_ids)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    buckets.check_views()

    graph = None
    launches_per_step = None
    if not args.no_graph:
        graph = torch.cuda.CUDAGraph()
        n0 = L.launch_count()
        with torch.cuda.graph(graph):
            static_loss.copy_(step(static_ids))
        launches_per_step = L.launch_count() - n0
    else:
        n0 = L.launch_count()
        step(static_ids)
        launches_per_step = L.launch_count() - n0

    def run_step():
        if graph is not None:
            graph.replay()
        else:
            static_loss.copy_(step(static_ids))
        if reducer is None:
            buckets.all_reduce_mean()
            if optimizer is not None and world > 1:
                optimizer.step()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        run_step()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        run_step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop() if sampler else None
    buckets.check_views()

    # end to end through the public API: pinned host tokens in, loss value out, every step
    barrier()
    t0 = time.perf_counter()
    last = 0.0
    for i in range(args.steps):
        static_ids.copy_(host_tokens[i % len(host_tokens)], non_blocking=True)
        run_step()
        last = float(static_loss.item())
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps

    if world > 1:
        t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = t.tolist()

    # N > 1: how much of the gradient all-reduce is NOT hidden behind backward: an event after the last backward
    # kernel and one after the stream has joined the collectives, on every rank.  The step is captured a second time
    # with the two events in it and replayed, so that the figure belongs to the step that was timed (launched
    # eagerly, the host falls behind at 8 GPUs and the gap measures that instead); eager steps when not replaying.
    exposed_ms = None
    if reducer is not None:
        gaps = []
        if graph is not None:
            marks = [torch.cuda.Event(enable_timing=True, external=True) for _ in range(2)]
            marked = torch.cuda.CUDAGraph()
            with torch.cuda.graph(marked):
                static_loss.copy_(step(static_ids, marks))
        for _ in range(5):
            if graph is not None:
                marked.replay()
            else:
                marks = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
                step(static_ids, marks)
            torch.cuda.synchronize()
            gaps.append(marks[0].elapsed_time(marks[1]))
        t = torch.tensor([statistics.median(gaps[1:])], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        exposed_ms = float(t.item())

    # The two tensor-core kernel families, timed live on the launching stream inside eager steps: a CUDA event
    # before and after every GEMM call and every attention call, on the step's own operands, with the SM clock
    # sampled meanwhile.  Beside it, the GEMM calls recorded (shape, strides, epilogue) and replayed back to back
    # on dense random operands inside a CUDA graph, under its own clock samples.
    roof = roof_attn = None
    if rank == 0 and not args.no_roofline:
        from tritonformer_b200 import attention as tattn
        peaks = measured_peaks()
        recs = []
        tlinear.PROFILE = recs
        if reducer is not None:
            reducer.enabled = False  # these steps run on rank 0 only: no collectives
        # every kernel is timed ALONE here: the weight-gradient products stay on the compute stream for these steps
        # (side by side, as in the timed step, two kernels share the GPU and each one's elapsed time holds the other's)
        fork_was, tlinear.FORK_WEIGHT_GRAD = tlinear.FORK_WEIGHT_GRAD, False
        step(static_ids)
        tlinear.PROFILE = None
        torch.cuda.synchronize()
        gflop = sum(2.0 * r["m"] * r["n"] * r["k"] for r in recs)
        smp = ClockSampler(local)
        smp.start()
        gemm_s, fwd_s, bwd_s, aflop = [], [], [], [0.0, 0.0]
        for _ in range(12):
            tlinear.TIMING, tattn.TIMING = [], []
            step(static_ids)
            gm, am = tlinear.TIMING, tattn.TIMING
            tlinear.TIMING = tattn.TIMING = None
            torch.cuda.synchronize()
            gemm_s.append(sum(a.elapsed_time(b) for a, b, _ in gm) * 1e-3)
            fwd_s.append(sum(a.elapsed_time(b) for a, b, k, _ in am if k == "fwd") * 1e-3)
            bwd_s.append(sum(a.elapsed_time(b) for a, b, k, _ in am if k == "bwd") * 1e-3)
            aflop = [sum(f for _, _, k, f in am if k == "fwd"), sum(f for _, _, k, f in am if k == "bwd")]
            n_attn = len(am)
        clk_step = smp.stop()
        tlinear.FORK_WEIGHT_GRAD = fork_was
        if reducer is not None:
            reducer.enabled = True
        in_step_s, fwd_t, bwd_t = (statistics.median(x[2:]) for x in (gemm_s, fwd_s, bwd_s))
        smp = ClockSampler(local)
        smp.start()
        g_s = _time_cuda(lambda: tlinear.replay(recs, dev), 20, 2)
        clk_replay = smp.stop()
        achieved = gflop / in_step_s / 1e12
        mhz = lambda c: c.get("sm_mhz") if c else None
        # one launch of the dominant kernel under ncu (profiles/ncu_gemm_tc05.md): the forward product of the first
        # MLP linear, M8192 N4096 K1024 fp16.  DRAM read 25.29 MB = X (16.8 MB) + W (8.4 MB) once; 18.76 MB of the
        # 67.1 MB output had been written back when the kernel ended (the rest was still in the L2).
        traffic = {"launch": "gemm_pair_tc05_kernel, forward fc1 M8192 N4096 K1024 fp16 (profiles/ncu_gemm_tc05.md)",
                   "dram_bytes_read": 25.29e6, "dram_bytes_written": 18.76e6,
                   "algorithmic_bytes_read": 2.0 * (8192 * 1024 + 1024 * 4096),
                   "algorithmic_bytes_written": 2.0 * 8192 * 4096}
        roof = {"bound": "tensor",
                "kernel": "gemm_pair_tc05_kernel + gemm_tc05_kernel (all linear fwd/dX/dW products of one step)",
                "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": achieved / peaks["tflops"],
                "traffic": traffic["dram_bytes_read"] + traffic["dram_bytes_written"], "traffic_detail": traffic,
                "launches": len(recs), "tcgen05_launches": sum(1 for r in recs if r["path"] == 1),
                "peak_source": peaks["source"] + " sustained bf16 cuBLAS", "gemm_ms_per_step": in_step_s * 1e3,
                "flops_per_step": gflop, "sm_mhz": mhz(clk_step),
                "ms_x_ghz": in_step_s * 1e3 * (mhz(clk_step) or 0) * 1e-3,
                "how": "CUDA events around every GEMM call of eager steps (median of 10), on the step's own operands, "
                       "one kernel at a time (in the timed step the weight-gradient products run beside the others "
                       "on a side stream)",
                # the same calls back to back on dense random operands inside a CUDA graph: the kernels alone in
                # the power-capped regime; ms_x_ghz (time x median SM clock, i.e. giga-cycles) separates what the
                # lower clock costs from what the operands cost
                "replay": {"gemm_ms_per_step": g_s * 1e3, "achieved": gflop / g_s / 1e12,
                           "frac": gflop / g_s / 1e12 / peaks["tflops"], "sm_mhz": mhz(clk_replay),
                           "ms_x_ghz": g_s * 1e3 * (mhz(clk_replay) or 0) * 1e-3}}
        a_ach = (aflop[0] + aflop[1]) / (fwd_t + bwd_t) / 1e12
        roof_attn = {"bound": "tensor",
                     "kernel": "attn_fwd1_tc05_kernel + attn_bwd_tc05_kernel (+ delta pre-pass, dQ conversion)",
                     "achieved": a_ach, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": a_ach / peaks["tflops"],
                     # DRAM bytes of one forward + one backward launch, from the ncu captures of the B2 H16 T2048
                     # hd64 case scaled by batch*heads (the traffic is q, k, v, dO read once: proportional);
                     # only for the configuration the captures cover
                     "traffic": (2 * (25.23e6 + 50.92e6 + 1.83e6) * (B * cfg.num_attention_heads) / 64.0
                                 if (cfg.head_dim == 64 and T == 2048) else None),
                     "traffic_detail": "profiles/ncu_attention_fwd.md, profiles/ncu_attention_bwd.md",
                     "calls": n_attn, "fwd_ms_per_step": fwd_t * 1e3, "bwd_ms_per_step": bwd_t * 1e3,
                     "fwd_tflops": aflop[0] / fwd_t / 1e12, "bwd_tflops": aflop[1] / bwd_t / 1e12,
                     "flops_per_step": aflop[0] + aflop[1], "sm_mhz": mhz(clk_step),
                     "peak_source": peaks["source"] + " sustained bf16 cuBLAS",
                     "how": "CUDA events around every attention call of eager steps (median of 10); causal FLOPs "
                            "(2 products forward, 5 backward, half of the square)"}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        t_cpu, cores, _, sb, ss = cpu_reference_step_time(3, 1)
        cpu = {"value": sb * ss / t_cpu, "unit": "tokens/s", "cores": cores, "kind": "port",
               "sample": _cpu_sample_text(sb, ss, 3), "ms_per_step": t_cpu * 1e3}

    if rank == 0:
        flops = algorithmic_flops(cfg, B, T)
        tok_s = world * B * T / (ms * 1e-3)
        tflops_gpu = flops / (ms * 1e-3) / 1e12
        line = {
            "metric": METRIC if args.config == "410m" else f"fwd+bwd tokens/s, {args.config}",
            "value": tok_s, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp16" if dtype is torch.float16 else "bf16", "data": "synthetic",
            "config": {"workload": f"{args.config} GPT fwd+bwd: d{cfg.hidden_size} L{cfg.num_hidden_layers} "
                                   f"H{cfg.num_attention_heads} ffn{cfg.ffn_dim} V{cfg.vocab_size} ctx{T} batch{B}/GPU",
                       "global_batch": world * B, "seq_len": T, "parallelism": f"dp{world}",
                       "cuda_graph": graph is not None, "loss_scale": loss_scale,
                       "optimizer": ("fused AdamW, fp32 master weights, dynamic loss scale (in the timed step)"
                                     if optimizer is not None else None),
                       "allreduce": ("overlapped with backward" if reducer is not None else "after backward")
                       if world > 1 else None,
                       "l2": "working set per step (>= 0.8 GB of weights plus activations) exceeds the 126 MB L2"},
            "tflops_per_gpu": tflops_gpu,
            "frac_of_measured_bf16_peak": tflops_gpu / measured_peaks()["tflops"],
            "frac_of_nominal_fp16_peak": tflops_gpu / 2250.0,
            "tflops_per_gpu_6N_convention": common_flops(cfg, B, T, n_params) / (ms * 1e-3) / 1e12,
            "readme_rtx3090_tflops": 50.1719 if args.config == "410m" else None,
            "loss": last,
            "clocks": clocks,
            "e2e": {"value": world * B * T / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": B * T * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches_per_step * args.steps),
            "launches_per_step": int(launches_per_step),
            "roofline": roof,
            "roofline_attention": roof_attn,
            "allreduce_exposed_ms": exposed_ms,
            "cpu_baseline": cpu,
            "device_status": L.device_status(),
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        # Every rank waits for rank 0's extra measurements, then the processes leave without tearing the
        # communicator down: the captured graph still references NCCL kernels, and destroying the
        # process group underneath it has been seen to block at exit.
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        os._exit(0)


# ------------------------------------------------------------------ per-kernel micro-benchmarks
def _time_cuda(fn, iters, warmup):
    """Seconds per call, device time only: the calls are captured into a CUDA graph and replayed so
    that host-side launch work is not part of the measurement."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(warmup):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(iters):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e-3


def run_kernel_bench(args):
    """Isolated kernels through the C ABI on synthetic inputs: one JSON line per case with the achieved
    rate against the measured peak (burst bf16 cuBLAS for tensor kernels, STREAM-style copy for HBM ones).
    HBM-bound cases use inputs larger than the 126 MB L2."""
    import ctypes
    import tritonformer_b200._lib as L
    from tritonformer_b200 import attention as A
    from tritonformer_b200 import crossentropy as CE
    from tritonformer_b200 import layernorm as LN
    from tritonformer_b200 import linear as LIN
    from tritonformer_b200 import softmax as SM
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = measured_peaks()
    iters, warmup = (1, 1) if args.small else (args.steps, max(args.warmup, 3))
    out = []

    def emit(kernel, case, seconds, work, unit, bound):
        peak = peaks["tflops_burst"] if bound == "tensor" else peaks["hbm_gbs"]
        ach = work / seconds / (1e12 if bound == "tensor" else 1e9)
        line = {"kernel": kernel, "case": case, "us": seconds * 1e6,
                "roofline": {"bound": bound, "achieved": ach, "peak": peak, "unit": unit, "frac": ach / peak,
                             "peak_source": peaks["source"]}}
        out.append(line)
        print(json.dumps(line), flush=True)

    torch.manual_seed(0)
    which = args.kernel
    if which in ("gemm", "all"):
        shapes = [("fwd proj", 8192, 1024, 1024, False, True), ("fwd fc1", 8192, 4096, 1024, False, True),
                  ("fwd fc2", 8192, 1024, 4096, False, True), ("fwd head", 8192, 50304, 1024, False, True),
                  ("dX fc1", 8192, 1024, 4096, False, False), ("dX head", 8192, 1024, 50304, False, False),
                  ("dW proj", 1024, 1024, 8192, True, True), ("dW fc1", 1024, 4096, 8192, True, True),
                  ("dW head", 1024, 50304, 8192, True, True)]
        if args.small:
            shapes = shapes[1:2] + shapes[6:7]
        for name, m, n, k, a_mn, b_mn in shapes:
            a = torch.randn((k, m) if a_mn else (m, k), device=dev).half()
            b = torch.randn((k, n) if b_mn else (n, k), device=dev).half()
            c = torch.empty((m, n), device=dev, dtype=torch.float16)
            a_sm, a_sk = (1, m) if a_mn else (k, 1)
            b_sk, b_sn = (n, 1) if b_mn else (1, k)
            fn = lambda: LIN.gemm(a, a_sm, a_sk, b, b_sk, b_sn, m, n, k, out=c)
            # outputs with a 256 x 256 tile for at least every second pair of SMs run on the CTA-pair kernel
            pair = m >= 256 and n >= 256 and -(-m // 256) * -(-n // 256) >= 37
            emit("gemm_pair_tc05_kernel" if pair else "gemm_tc05_kernel", f"{name} M{m} N{n} K{k}",
                 _time_cuda(fn, iters, warmup), 2.0 * m * n * k, "TFLOP/s", "tensor")
    if which in ("attn", "all"):
        cases = [("B4 H16 T2048 hd64 fp16", 4, 16, 2048, 64, torch.float16, False),
                 ("B4 H16 T2048 hd64 fp16 ALiBi", 4, 16, 2048, 64, torch.float16, True),
                 ("B1 H12 T4096 hd128 fp16", 1, 12, 4096, 128, torch.float16, False),
                 ("B2 H16 T2048 hd128 bf16 ALiBi", 2, 16, 2048, 128, torch.bfloat16, True)]
        if args.small:
            # 512 (tile, head) items: enough for every persistent CTA to walk several, small enough for an ncu capture
            cases = [("B2 H16 T2048 hd64 fp16", 2, 16, 2048, 64, torch.float16, False)]
        for name, bsz, h, t, hd, dt, alibi in cases:
            mk = lambda: torch.randn((bsz, t, h * hd), device=dev).to(dt).view(bsz, t, h, hd).transpose(1, 2)
            q, k, v, do = mk(), mk(), mk(), mk()
            slopes = torch.tensor([2.0 ** (-8.0 * (i + 1) / h) for i in range(h)], device=dev) if alibi else None
            bias = A._Bias(slopes=slopes)
            res = {}
            def fwd():
                res["o"], res["lse"], _ = A.attention_forward(q, k, v, bias)
            fl = 2.0 * bsz * h * t * t * hd  # two products, causal half
            emit("attn_fwd1_tc05_kernel", name, _time_cuda(fwd, iters, warmup), fl, "TFLOP/s", "tensor")
            bwd = lambda: A.attention_backward(do, res["o"], q, k, v, res["lse"], bias)
            emit("attn_bwd_tc05_kernel (+delta, dQ convert)", name, _time_cuda(bwd, iters, warmup), 2.5 * fl,
                 "TFLOP/s", "tensor")
    if which in ("layernorm", "all"):
        rows, d = (32768, 1024) if args.small else (131072, 1024)
        x = torch.randn((rows, d), device=dev).half()
        dy = torch.randn((rows, d), device=dev).half()
        al, be = torch.randn(d, device=dev).half(), torch.randn(d, device=dev).half()
        res = {}
        def fwd():
            res["y"], res["st"] = LN.layernorm_forward(x, al, be, 1e-5)
        emit("ln_fwd_vec_kernel", f"rows {rows} d {d} fp16", _time_cuda(fwd, iters, warmup), 4.0 * rows * d, "GB/s", "hbm")
        bwd = lambda: LN.layernorm_backward(dy, x, al, res["st"])
        emit("ln_bwd_split_kernel (+finalize)", f"rows {rows} d {d} fp16", _time_cuda(bwd, iters, warmup), 6.0 * rows * d,
             "GB/s", "hbm")
    if which in ("crossentropy", "all"):
        n, v = (2048, 50304) if args.small else (8188, 50304)
        logits = torch.randn((n, v), device=dev).half()
        labels = torch.randint(0, v, (n,), device=dev)
        loss = torch.empty(n, device=dev, dtype=torch.float16)
        lse = torch.empty(n, device=dev, dtype=torch.float32)
        g = torch.ones(n, device=dev, dtype=torch.float16)
        dl = torch.empty_like(logits)
        st = lambda: L.stream_ptr(dev)  # read at call time: the timing harness replays from its own stream
        fwd = lambda: L.check(L.lib.tfb_cross_entropy_fwd(logits.data_ptr(), labels.data_ptr(), loss.data_ptr(), None,
                                                          lse.data_ptr(), n, v, v, 0, st()))
        emit("ce_fwd_kernel", f"rows {n} vocab {v} fp16", _time_cuda(fwd, iters, warmup), 2.0 * n * v, "GB/s", "hbm")
        bwd = lambda: L.check(L.lib.tfb_cross_entropy_bwd(logits.data_ptr(), labels.data_ptr(), lse.data_ptr(),
                                                          g.data_ptr(), 1, dl.data_ptr(), n, v, v, v, 0, st()))
        emit("ce_bwd_kernel", f"rows {n} vocab {v} fp16", _time_cuda(bwd, iters, warmup), 4.0 * n * v, "GB/s", "hbm")
    if which in ("softmax", "all"):
        rows, cols = (65536, 1024) if args.small else (131072, 1024)
        x = torch.randn((1, rows, cols), device=dev)
        dy = torch.randn((1, rows, cols), device=dev)
        y = torch.empty_like(x)
        dx = torch.empty_like(x)
        st = lambda: L.stream_ptr(dev)  # read at call time: the timing harness replays from its own stream
        fwd = lambda: L.check(L.lib.tfb_softmax_fwd(x.data_ptr(), y.data_ptr(), rows, cols, cols, cols, 2, st()))
        emit("softmax_fwd_vec_kernel", f"rows {rows} cols {cols} fp32", _time_cuda(fwd, iters, warmup), 8.0 * rows * cols,
             "GB/s", "hbm")
        bwd = lambda: L.check(L.lib.tfb_softmax_bwd(dy.data_ptr(), y.data_ptr(), dx.data_ptr(), rows, cols, cols, cols,
                                                    cols, 2, st()))
        emit("softmax_bwd_vec_kernel", f"rows {rows} cols {cols} fp32", _time_cuda(bwd, iters, warmup),
             12.0 * rows * cols, "GB/s", "hbm")
    if which in ("relu", "all"):
        n = 8192 * 4096 * (1 if args.small else 4)
        a, b = torch.randn(n, device=dev).half(), torch.randn(n, device=dev).half()
        emit("relu_bwd_vec_kernel", f"{n} elements fp16", _time_cuda(lambda: LIN.relu_backward(a, b), iters, warmup),
             6.0 * n, "GB/s", "hbm")
    if which in ("embed", "all"):
        from tritonformer_b200 import embedding as EMB
        # batch 4 is the model step's shape (one position in seven shares its token with another); at batch 32
        # three in four do, so most rows go through the fp32 scratch
        for bsz in ((4,) if args.small else (4, 32)):
            t, d, v = 2048, 1024, 50304
            ids = torch.randint(0, v, (bsz, t), device=dev)
            tok, pos = torch.randn((v, d), device=dev).half(), torch.randn((t, d), device=dev).half()
            dout = torch.randn((bsz, t, d), device=dev).half()
            dtok, dpos = torch.zeros_like(tok), torch.zeros_like(pos)
            case = f"B{bsz} T{t} d{d} vocab {v} fp16"
            # forward: every position reads one table row and writes one row
            emit("embed_fwd_kernel", case, _time_cuda(lambda: EMB.embedding_forward(ids, tok, pos), iters, warmup),
                 4.0 * bsz * t * d, "GB/s", "hbm")
            # backward: reads the incoming row, reads and writes the table-gradient row it lands in
            emit("embed_index + embed_clear + embed_bwd_scatter + embed_bwd_fold", case,
                 _time_cuda(lambda: EMB.embedding_backward(ids, dout, dtok, dpos), iters, warmup),
                 6.0 * bsz * t * d, "GB/s", "hbm")
    if which in ("adam", "all"):
        n = (64 if args.small else 256) * (1 << 20)  # elements: 28 B each across the five arrays, far beyond the L2
        g = (torch.randn(n, device=dev) * 64.0).half()
        p16 = torch.randn(n, device=dev).half()
        w, m, v = p16.float(), torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        state = torch.tensor([64.0, 1.0 / 64.0, 0.0, 0.0], device=dev)
        found = torch.zeros(1, device=dev, dtype=torch.int32)
        st = lambda: L.stream_ptr(dev)
        chk = lambda: L.check(L.lib.tfb_grad_check(g.data_ptr(), n, 0, found.data_ptr(), st()))
        emit("grad_check_kernel", f"{n} gradients fp16", _time_cuda(chk, iters, warmup), 2.0 * n, "GB/s", "hbm")
        upd = lambda: L.check(L.lib.tfb_adamw_step(g.data_ptr(), p16.data_ptr(), w.data_ptr(), m.data_ptr(), v.data_ptr(), n,
                                                   0, state[1:2].data_ptr(), found.data_ptr(), state[3:4].data_ptr(), 1e-4,
                                                   0.9, 0.95, 1e-8, 0.1, st()))
        emit("adamw_step_kernel", f"{n} parameters fp16 + fp32 master, m, v", _time_cuda(upd, iters, warmup), 28.0 * n,
             "GB/s", "hbm")
    assert L.device_status() == 0
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", default="410m", choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-overlap", action="store_true",
                    help="N > 1: all-reduce the gradient buckets after the step instead of during backward")
    ap.add_argument("--kernel", default=None,
                    choices=["all", "gemm", "attn", "layernorm", "crossentropy", "softmax", "relu", "embed", "adam"],
                    help="run the isolated-kernel micro-benchmarks instead of the model step")
    ap.add_argument("--optimizer", action="store_true",
                    help="add the fused AdamW step (fp32 master weights, dynamic loss scale) to the timed step")
    ap.add_argument("--no-roofline", action="store_true",
                    help="skip the eager steps that time the GEMM and attention calls (for a short ncu launch list)")
    ap.add_argument("--small", action="store_true", help="with --kernel: one small case, one launch (for ncu captures)")
    args = ap.parse_args()
    if args.kernel:
        run_kernel_bench(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_b200_arm(args)


if __name__ == "__main__":
    main()
