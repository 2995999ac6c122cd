"""Multi-GPU sharding of the decode path: one process per GPU, torch.distributed for the exchange.

KV-head shards (batched decode): every rank owns ``num_kv_heads / world`` KV heads with their
query heads for all tokens and layers.  Attention needs no exchange (head outputs are
independent).  Importance is a sum over query heads, so each rank accumulates the mass of its own
heads and the ranks add their contributions up right before every reallocation; the allocator then
runs replicated on identical inputs and produces identical bucket maps on every rank, so storage
order stays the same everywhere without further traffic.

Sequence shards (long context, split-KV): every rank owns a slice of the tokens of each sequence;
the ranks exchange one (max, sum, out[D]) partial per query head and fold them with the same
log-sum-exp rule the combine kernel uses (smartkv/kernels/__init__.py:350-371 is the reference's
cross-bucket form of that rule).

The reference has no multi-GPU path; these are additions around the same kernels.
"""
from __future__ import annotations

from typing import Optional

import torch


def shard_kv_heads(num_kv_heads: int, world: int, rank: int) -> range:
    """KV heads owned by ``rank`` (contiguous blocks; world must divide the head count)."""
    if num_kv_heads % world:
        raise ValueError(f"{num_kv_heads} KV heads cannot be split over {world} ranks")
    per = num_kv_heads // world
    return range(rank * per, (rank + 1) * per)


def shard_tokens(num_tokens: int, world: int, rank: int) -> range:
    """Token range owned by ``rank`` under a sequence split (sizes differ by at most one)."""
    lo = (num_tokens * rank) // world
    hi = (num_tokens * (rank + 1)) // world
    return range(lo, hi)


def sync_importance_delta(local: torch.Tensor, synced: torch.Tensor, dist_module=None, group=None) -> None:
    """``local`` = the value all ranks agreed on at the last sync (``synced``) plus what this rank
    added since.  Adds up the ranks' additions and leaves the agreed total in both tensors."""
    delta = local - synced
    if dist_module is not None and dist_module.is_initialized() and dist_module.get_world_size(group) > 1:
        dist_module.all_reduce(delta, op=dist_module.ReduceOp.SUM, group=group)
    synced.add_(delta)
    local.copy_(synced)


class ImportanceSync:
    """Keeps the cumulative importance of a KV-head-sharded store identical on every rank."""

    def __init__(self, store, dist_module=None, group=None):
        self.store, self.dist, self.group = store, dist_module, group
        self.synced: Optional[torch.Tensor] = None

    def __call__(self) -> None:
        if self.dist is None:
            return
        if self.synced is None:
            # what was injected before the first sync is common to all ranks
            self.synced = self.store.cumulative.clone()
            return
        sync_importance_delta(self.store.cumulative, self.synced, self.dist, self.group)

    def after_repack(self) -> None:
        """Storage order changed (identically on every rank): the agreed copy follows the store."""
        if self.synced is not None:
            self.synced.copy_(self.store.cumulative)


def fold_partials(allp: torch.Tensor, out: Optional[torch.Tensor] = None):
    """allp [world, .., D + 2] = every rank's (max in log2 units, sum, unnormalised out[D]) per query head; returns the
    attention output over all ranks' tokens [.., D] (written into ``out`` if given).  The rule of the combine kernel:
    weights 2^(m_r - M), empty partials (m = -inf) count for nothing."""
    ms, ls, os_ = allp[..., 0], allp[..., 1], allp[..., 2:]
    M = ms.max(dim=0).values
    w = torch.where(torch.isneginf(ms), torch.zeros_like(ms), torch.exp2(ms - M))
    L = (ls * w).sum(0)
    O = (os_ * w.unsqueeze(-1)).sum(0)
    res = torch.where(L.unsqueeze(-1) > 0, O / L.clamp_min(1e-38).unsqueeze(-1), torch.zeros_like(O))
    if out is not None:
        out.copy_(res)
        return out
    return res


def combine_partials(m: torch.Tensor, l: torch.Tensor, o: torch.Tensor, dist_module=None, group=None):
    """Sequence-split attention: m, l [..] and o [.., D] are this rank's running max (log2 units),
    sum and unnormalised output; returns the attention output over all ranks' tokens and the global
    (max, sum).  One all-gather of (D + 2) floats per query head."""
    packed = torch.cat([m.unsqueeze(-1), l.unsqueeze(-1), o], dim=-1).contiguous()
    if dist_module is not None and dist_module.is_initialized() and dist_module.get_world_size(group) > 1:
        world = dist_module.get_world_size(group)
        gathered = [torch.empty_like(packed) for _ in range(world)]
        dist_module.all_gather(gathered, packed, group=group)
        allp = torch.stack(gathered)                     # [world, .., D + 2]
    else:
        allp = packed.unsqueeze(0)
    ms, ls, os_ = allp[..., 0], allp[..., 1], allp[..., 2:]
    M = ms.max(dim=0).values
    w = torch.where(torch.isneginf(ms), torch.zeros_like(ms), torch.exp2(ms - M))
    L = (ls * w).sum(0)
    O = (os_ * w.unsqueeze(-1)).sum(0)
    out = torch.where(L.unsqueeze(-1) > 0, O / L.clamp_min(1e-38).unsqueeze(-1), torch.zeros_like(O))
    return out, M, L
