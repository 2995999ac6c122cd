"""Host-side logic of the multi-GPU paths, run as two gloo ranks on CPU: the importance exchange of
KV-head shards and the log-sum-exp fold of sequence shards."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import smartkv_oracle as orc
from smartkv_b200 import sharding


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _importance_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(5)
        common = torch.rand((3, 40), generator=g, dtype=torch.float64)     # injected on every rank alike
        local = common.clone()
        synced = common.clone()
        total = common.clone()
        for rnd in range(3):
            adds = [torch.rand((3, 40), generator=torch.Generator().manual_seed(100 * rnd + r), dtype=torch.float64)
                    for r in range(world)]
            local += adds[rank]                     # this rank's heads
            total += sum(adds)                      # all heads
            sharding.sync_importance_delta(local, synced, dist)
            assert torch.allclose(local, total, rtol=0, atol=1e-12)
            assert torch.equal(local, synced)
        gathered = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(gathered, local)
        assert all(torch.equal(gathered[0], t) for t in gathered)      # bit-identical on every rank
        out.put((rank, "ok"))
    finally:
        dist.destroy_process_group()


def _splitkv_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        hq, hkv, d, n = 8, 2, 64, 333
        grp = hq // hkv
        k, v = orc.synth_kv(n, hkv, d, seed=3)
        rng = np.random.default_rng(9)
        bits = rng.choice((2, 3, 4, 8), size=n)
        kq = np.empty(k.shape, np.int8); vq = np.empty(k.shape, np.int8)
        ks = np.empty(k.shape[:2], np.float32); vs = np.empty(k.shape[:2], np.float32)
        for w in (2, 3, 4, 8):
            sel = bits == w
            kq[sel], ks[sel] = orc.quantize_rows(k[sel], w)
            vq[sel], vs[sel] = orc.quantize_rows(v[sel], w)
        q = rng.standard_normal((hq, d)).astype(np.float32)
        # this rank's token slice -> partial (max in log2 units, sum, unnormalised out)
        own = sharding.shard_tokens(n, world, rank)
        sl = slice(own.start, own.stop)
        kd = orc.dequantize_rows(orc.expand_gqa(kq[sl], grp), orc.expand_gqa(ks[sl], grp))   # [m, hq, d]
        vd = orc.dequantize_rows(orc.expand_gqa(vq[sl], grp), orc.expand_gqa(vs[sl], grp))
        logits = np.einsum("hd,mhd->hm", q, kd) / np.sqrt(d) * np.log2(np.e)
        m = logits.max(1)
        p = np.exp2(logits - m[:, None])
        l = p.sum(1)
        o = np.einsum("hm,mhd->hd", p, vd)
        out_t, M, L = sharding.combine_partials(torch.from_numpy(m), torch.from_numpy(l), torch.from_numpy(o), dist)
        # all tokens at once
        ref, _ = orc.dequant_attend(q[None, :, None, :], orc.expand_gqa(kq, grp).transpose(1, 0, 2)[None],
                                    orc.expand_gqa(ks, grp).T[None], orc.expand_gqa(vq, grp).transpose(1, 0, 2)[None],
                                    orc.expand_gqa(vs, grp).T[None])
        assert np.allclose(out_t.numpy(), ref[0, :, 0], atol=2e-5, rtol=1e-5)
        out.put((rank, "ok"))
    finally:
        dist.destroy_process_group()


def _step_exchange_worker(rank, world, port, out):
    """One exchange per decode step: every rank packs (max, sum, unnormalised out) of ALL layers into one tensor, a
    single all_gather_into_tensor carries them, fold_partials folds them.  Rank 1's shard of the last layer is empty
    (max = -inf), which must count for nothing."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        L, B, hq, d, n = 3, 2, 4, 16, 50
        g = torch.Generator().manual_seed(11)
        logits = torch.randn((L, B, hq, n), generator=g, dtype=torch.float64) * 3
        vals = torch.randn((L, B, n, d), generator=g, dtype=torch.float64)
        own = sharding.shard_tokens(n, world, rank)
        lo, hi = own.start, own.stop
        packed = torch.empty((L, B, hq, d + 2), dtype=torch.float64)
        for l in range(L):
            a, b_ = (lo, hi) if not (l == L - 1 and rank == 1) else (hi, hi)     # empty shard
            if l == L - 1 and rank == 0:
                a, b_ = 0, n                                                      # ... whose tokens rank 0 holds
            lg = logits[l, :, :, a:b_]
            if b_ > a:
                m = lg.max(-1).values
                p_ = torch.exp2(lg - m[..., None])
                packed[l, ..., 0], packed[l, ..., 1] = m, p_.sum(-1)
                packed[l, ..., 2:] = torch.einsum("bhn,bnd->bhd", p_, vals[l, :, a:b_])
            else:
                packed[l, ..., 0], packed[l, ..., 1], packed[l, ..., 2:] = float("-inf"), 0.0, 0.0
        flat = torch.empty((world * L,) + tuple(packed.shape[1:]), dtype=torch.float64)    # ranks concatenated along dim 0
        dist.all_gather_into_tensor(flat, packed)
        gathered = flat.view((world,) + tuple(packed.shape))
        folded = sharding.fold_partials(gathered)
        pr = torch.softmax(logits * float(np.log(2.0)), dim=-1)
        ref = torch.einsum("lbhn,lbnd->lbhd", pr, vals)
        assert torch.allclose(folded, ref, atol=1e-10, rtol=1e-10)
        into = torch.zeros_like(ref)
        assert sharding.fold_partials(gathered, out=into) is into and torch.equal(into, folded)
        out.put((rank, "ok"))
    finally:
        dist.destroy_process_group()


def _run(worker, world=2):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    got = sorted(out.get(timeout=5) for _ in range(world))
    assert got == [(r, "ok") for r in range(world)]


def test_importance_sync_two_ranks():
    _run(_importance_worker)


def test_one_exchange_per_step_two_ranks():
    _run(_step_exchange_worker)


def test_split_kv_combine_two_ranks():
    _run(_splitkv_worker)


def test_shard_ranges_cover_everything():
    for world in (1, 2, 4, 8):
        heads = [h for r in range(world) for h in sharding.shard_kv_heads(8, world, r)]
        assert heads == list(range(8))
        toks = [t for r in range(world) for t in sharding.shard_tokens(131072 + 5, world, r)]
        assert toks == list(range(131072 + 5))


def test_combine_partials_single_rank_handles_empty():
    m = torch.tensor([-float("inf"), 0.5])
    l = torch.tensor([0.0, 2.0])
    o = torch.tensor([[0.0, 0.0], [4.0, 6.0]])
    out, M, L = sharding.combine_partials(m, l, o)
    assert torch.equal(out, torch.tensor([[0.0, 0.0], [2.0, 3.0]]))
