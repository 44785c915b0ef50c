"""CPU, world_size 2 over gloo: gradient buckets alias .grad, all-reduce averages them, shards partition
the batch, and a rank that fails before the collective surfaces as an error on the other rank."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tritonformer_b200.dp import GradBuckets, OverlappedReducer, broadcast_parameters, shard_batch


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, mode, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from datetime import timedelta
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=20))
    except Exception as e:  # noqa: BLE001  (the probed port was taken meanwhile, or the peer was slow to start)
        out.put((rank, "init_error", repr(e)))
        return
    try:
        torch.manual_seed(rank)  # replicas start different on purpose
        model = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 4))
        broadcast_parameters(model, 0)
        buckets = GradBuckets(model.parameters(), bucket_bytes=600 if mode == "overlap" else 1024)
        assert len(buckets.buckets) >= 2
        gen = torch.Generator().manual_seed(7)
        data = torch.randn((8, 16), generator=gen)
        x = shard_batch(data, rank, world)
        reducer = None
        if mode == "overlap":  # buckets are reduced from hooks while backward is still running
            calls = []  # told when the first collective of the step is enqueued and when the step is joined
            reducer = OverlappedReducer(buckets, [model[0], model[2]], on_collectives=calls.append)
            assert reducer.ready_at[0] >= 1 and min(reducer.ready_at) == 0
            model(x).square().mean().backward()
            assert any(reducer.launched), "no bucket was reduced during backward"
            assert calls == [True]
            reducer.finish()
            assert calls == [True, False]
            buckets.check_views()
            flat = torch.cat([p.grad.reshape(-1) for p in model.parameters()])
            out.put((rank, "ok", flat))
            return
        for _ in range(2):  # gradients accumulate in place across steps
            model(x).square().mean().backward()
        buckets.check_views()
        if mode == "fail" and rank == 1:
            raise RuntimeError("injected failure before the collective")
        buckets.all_reduce_mean()
        flat = torch.cat([p.grad.reshape(-1) for p in model.parameters()])
        out.put((rank, "ok", flat))
    except Exception as e:  # noqa: BLE001
        import traceback
        out.put((rank, "error", repr(e) + "\n" + traceback.format_exc()))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def _run(mode):
    ctx = mp.get_context("spawn")
    for attempt in range(3):  # a rendezvous that did not come up is tried again on another port
        out = ctx.Queue()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, 2, port, mode, out)) for r in range(2)]
        for p in procs:
            p.start()
        res = [out.get(timeout=120) for _ in procs]
        for p in procs:
            p.join(timeout=60)
        if attempt < 2 and any(s == "init_error" for _, s, _ in res):
            continue
        return {r: (s, v) for r, s, v in res}


def test_bucketed_allreduce_matches_single_process():
    res = _run("ok")
    assert res[0][0] == "ok" and res[1][0] == "ok", res
    assert torch.allclose(res[0][1], res[1][1])
    # single-process reference: mean over the two shards' accumulated gradients
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 4))
    gen = torch.Generator().manual_seed(7)
    data = torch.randn((8, 16), generator=gen)
    for shard in (data[:4], data[4:]):
        for _ in range(2):
            (model(shard).square().mean() / 2).backward()
    want = torch.cat([p.grad.reshape(-1) for p in model.parameters()])
    assert torch.allclose(res[0][1], want, atol=1e-6)


def test_overlapped_reduction_gives_the_same_mean():
    res = _run("overlap")
    assert res[0][0] == "ok" and res[1][0] == "ok", res
    assert torch.allclose(res[0][1], res[1][1])
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 4))
    gen = torch.Generator().manual_seed(7)
    data = torch.randn((8, 16), generator=gen)
    for shard in (data[:4], data[4:]):
        (model(shard).square().mean() / 2).backward()
    want = torch.cat([p.grad.reshape(-1) for p in model.parameters()])
    assert torch.allclose(res[0][1], want, atol=1e-6)


def test_rank_failure_surfaces_on_the_peer():
    res = _run("fail")
    assert res[1][0] == "error" and "injected" in res[1][1]
    assert res[0][0] == "error"  # the healthy rank's all-reduce ends with an error, not a hang
