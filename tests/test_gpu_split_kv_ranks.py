"""Sequence-split (split-KV) decode across two GPUs over NCCL: every rank holds half of the tokens of each
sequence, attends to its shard with the packed kernels and the ranks fold their (max, sum, out) results
(smartkv_b200.sharding.combine_partials).  Needs two GPUs; skipped otherwise."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_q):
    import torch.distributed as dist

    from smartkv_b200 import sharding
    from smartkv_b200.store import PackedKVStore, bucket_capacities
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    from datetime import timedelta
    # a short collective timeout: if the peer died before its first collective this rank must not spin on the GPU
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=timedelta(seconds=60))
    try:
        B, n, hq, hkv, d = 2, 6000, 32, 8, 128
        g = torch.Generator(device="cpu").manual_seed(3)          # the same data on every rank
        k = torch.randn((B, n, hkv, d), generator=g)
        v = torch.randn((B, n, hkv, d), generator=g)
        bits = torch.tensor([2, 3, 4, 8])[torch.randint(0, 4, (B, n), generator=g)]
        q = torch.randn((B, hq, d), generator=g).half()
        ck = torch.randn((B, hkv, d), generator=g)
        cv = torch.randn((B, hkv, d), generator=g)

        def build(lo, hi):
            s = PackedKVStore(1, B, hkv, d, hq, bucket_capacities(hi - lo, None, d), device=dev, track_importance=False)
            dst = s.plan_bulk(bits[:, lo:hi].contiguous().to(dev))
            s.append(0, k[:, lo:hi].reshape(-1, hkv, d).contiguous().to(dev), v[:, lo:hi].reshape(-1, hkv, d).contiguous().to(dev),
                     dst[0], dst[1], dst[2])
            return s

        # everything that can fail locally (build, kernels, error flag) happens before the first collective
        own = sharding.shard_tokens(n, world, rank)
        shard = build(own.start, own.stop)
        # the current token takes part on the last rank only
        last = rank == world - 1
        o = shard.attention(0, q.to(dev), ck.to(dev) if last else None, cv.to(dev) if last else None).clone()
        shard.check_errors()
        m, l = shard.lse_max.clone(), shard.lse_sum.clone()
        ref = None
        if rank == 0:
            whole = build(0, n)
            ref = whole.attention(0, q.to(dev), ck.to(dev), cv.to(dev)).clone()
            whole.check_errors()
        torch.cuda.synchronize()
        out, M, L = sharding.combine_partials(m, l, o * l[..., None], dist)
        if rank == 0:
            err = (out - ref).abs()
            tol = 2e-3 + 1e-3 * ref.abs()
            assert bool((err <= tol).all()), float(err.max())
            # the running maximum is raised lazily, so only max + log2(sum) is comparable
            assert torch.allclose(M + torch.log2(L), whole.lse_max + torch.log2(whole.lse_sum), atol=1e-3)
        out_q.put((rank, "ok"))
    except BaseException as e:  # reported to the parent; the peer's collective then ends by its timeout
        out_q.put((rank, f"{type(e).__name__}: {e}"))
        raise
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_split_kv_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out_q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out_q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    stuck = [p for p in procs if p.is_alive()]
    for p in stuck:       # never leave a rank behind on the GPU
        p.kill()
        p.join()
    results = []
    while not out_q.empty():
        results.append(out_q.get())
    assert not stuck, f"ranks still running after the limit were killed; reports: {results}"
    assert all(p.exitcode == 0 for p in procs), ([p.exitcode for p in procs], results)
    assert sorted(results) == [(0, "ok"), (1, "ok")]
