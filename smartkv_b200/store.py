"""Device-resident bucketed KV store and the decode-step driver over the C ABI.

``PackedKVStore`` owns the HBM arenas (one per layer and sequence, four packed
buckets each), the per-sequence bookkeeping kept in *storage order* and the
scratch buffers of the attention path.  Every compute step is a call into
``libsmartkv_b200.so``; torch is used for device memory, streams and the few
index computations that place tokens into buckets.

What it replaces in the reference: the growable int8 buffers, per-token dicts
and per-bucket tensors of ``SmartKVCache`` (smartkv/core/cache.py:928-1161) and
the clone-everything read path (``retrieve_all_quantized``, cache.py:1441-1491).
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional, Sequence, Tuple

import torch

from . import _lib
from ._lib import BITS_TO_BUCKET, BUCKET_BITS, NUM_BUCKETS, StoreDesc, check, ptr


def round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def bucket_capacities(max_tokens: int, memory_budget: Optional[float] = None, head_dim: int = 128,
                      available_bits: Sequence[int] = (2, 3, 4, 8), slack: int = 128) -> Tuple[int, ...]:
    """Capacity (tokens) of each bucket for sequences of up to ``max_tokens``.

    Without a budget every bucket can hold every token.  With a budget, a
    bucket of width w can never hold more than ``budget*16*N / w`` tokens plus
    the protected ones, because those tokens alone would exhaust the byte
    budget the allocator enforces (smartkv/core/cache.py:374-388, 502-505).
    New tokens enter at 4 bits (cache.py:1214), so that bucket keeps room for
    a reallocation interval's worth of appends.
    """
    caps = []
    for bits in BUCKET_BITS:
        if bits not in available_bits and bits != 4:
            caps.append(0)
            continue
        cap = max_tokens
        if memory_budget is not None and bits > min(available_bits):
            cap = min(max_tokens, int(memory_budget * 16.0 * max_tokens / bits) + 64)
        caps.append(round_up(cap + slack, 128))
    return tuple(caps)


def make_alloc_config(num_kv_heads: int, head_dim: int, memory_budget: float,
                      available_bits: Sequence[int] = (2, 3, 4, 8), utility_alpha: float = 0.5,
                      importance_floor: float = 1e-6, hysteresis_rank_threshold: float = 0.05,
                      hysteresis_intervals: int = 2, high_precision_fraction: float = 0.02,
                      high_precision_boost: float = 1.5, min_high_precision_tokens: int = 0,
                      protected: Sequence[int] = (0, 1, 2), critical_window: int = 4,
                      scale_bits: int = 32) -> "_lib.AllocConfig":
    """SkvAllocConfig with the clamping of SmartKVCache.__init__ (smartkv/core/cache.py:94-97,
    131-144) and of _solve_allocation (alpha to [0.1, 1], :390).  ``num_kv_heads``: KV heads of the
    whole model (accounting only).  bits ** alpha is computed here, with the host's libm."""
    c = _lib.AllocConfig()
    c.num_heads = int(num_kv_heads)
    c.head_dim = int(head_dim)
    bits = sorted(int(b) for b in available_bits)
    if not 1 <= len(bits) <= 4 or any(b not in BITS_TO_BUCKET for b in bits) or len(set(bits)) != len(bits):
        raise ValueError(f"available_bits must be 1 to 4 distinct widths out of 2, 3, 4, 8; got {list(available_bits)}")
    c.num_bits = len(bits)
    alpha = float(utility_alpha) if utility_alpha > 0 else 1.0
    alpha = min(max(alpha, 0.1), 1.0)
    for i, b in enumerate(bits):
        c.bits[i] = b
        c.util[i] = float(b) if alpha == 1.0 else float(math.pow(b, alpha))
    c.memory_budget = float(memory_budget)
    c.importance_floor = float(max(importance_floor, 0.0))
    c.rank_threshold = float(max(hysteresis_rank_threshold, 0.0))
    c.hysteresis_intervals = max(int(hysteresis_intervals), 1)
    c.high_fraction = float(max(0.0, min(high_precision_fraction, 0.5)))
    c.high_boost = float(max(1.0, high_precision_boost))
    c.min_high_tokens = int(max(0, min_high_precision_tokens))
    c.scale_bits = int(scale_bits)
    c.use_packing = 1
    c.critical_window = int(critical_window)
    prot = sorted(set(int(t) for t in protected))
    if len(prot) > _lib.ALLOC_MAX_PROTECTED:
        raise ValueError(f"at most {_lib.ALLOC_MAX_PROTECTED} protected token ids")
    c.num_protected = len(prot)
    for i, t in enumerate(prot):
        c.protected_ids[i] = t
    return c


class PackedKVStore:
    def __init__(self, num_layers: int, num_seqs: int, num_kv_heads: int, head_dim: int, num_q_heads: int,
                 caps: Sequence[int], device="cuda", decay: float = 0.9, head_decay: float = 0.9,
                 track_importance: bool = True):
        self.lib = _lib.lib()
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise _lib.SmartKVLibraryError("PackedKVStore needs a CUDA device; there is no CPU path")
        self.num_layers, self.num_seqs = num_layers, num_seqs
        self.num_kv_heads, self.head_dim, self.num_q_heads = num_kv_heads, head_dim, num_q_heads
        self.group = num_q_heads // num_kv_heads
        self.decay, self.head_decay = float(decay), float(head_decay)
        d = StoreDesc()
        d.num_layers, d.num_seqs, d.num_kv_heads, d.head_dim = num_layers, num_seqs, num_kv_heads, head_dim
        for i, c in enumerate(caps):
            d.cap[i] = int(c)
        check(self.lib.skv_store_layout(ctypes.byref(d)), "skv_store_layout")
        self.desc = d
        self.slots = int(d.slots)
        self.caps = tuple(int(c) for c in d.cap)
        self.bucket_base = tuple(int(c) for c in d.bucket_base)
        dev = self.device
        # zero-filled so that rows never written decode to finite numbers
        self.arena = torch.zeros(int(d.total_bytes), dtype=torch.uint8, device=dev)
        self.counts = torch.zeros((num_seqs, NUM_BUCKETS), dtype=torch.int32, device=dev)
        self.slot_token = torch.full((num_seqs, self.slots), -1, dtype=torch.int32, device=dev)
        self.next_token = torch.zeros(num_seqs, dtype=torch.int32, device=dev)
        self.err = torch.zeros(1, dtype=torch.int32, device=dev)
        self.num_ctas = int(self.lib.skv_attn_num_ctas(dev.index if dev.index is not None else torch.cuda.current_device()))
        pbytes = int(self.lib.skv_attn_partials_bytes(ctypes.byref(d), num_q_heads, self.num_ctas))
        self.partials = torch.empty(pbytes // 4, dtype=torch.float32, device=dev)
        plan_bytes = int(self.lib.skv_attn_plan_bytes(ctypes.byref(d), self.num_ctas))
        self.plan = torch.zeros(plan_bytes // 4, dtype=torch.int32, device=dev)
        self._plan_valid = False
        self.out = torch.empty((num_seqs, num_q_heads, head_dim), dtype=torch.float32, device=dev)
        self.lse_max = torch.empty((num_seqs, num_q_heads), dtype=torch.float32, device=dev)
        self.lse_sum = torch.empty((num_seqs, num_q_heads), dtype=torch.float32, device=dev)
        self.cur_prob = torch.empty((num_seqs, num_q_heads), dtype=torch.float32, device=dev)
        self.track_importance = track_importance
        if track_importance:
            self.logits = torch.empty((num_seqs, num_q_heads, self.slots), dtype=torch.float32, device=dev)
            self.cumulative = torch.zeros((num_seqs, self.slots), dtype=torch.float64, device=dev)
            self.layer_ema = torch.zeros((num_layers, num_seqs, self.slots), dtype=torch.float32, device=dev)
            self.touched = torch.zeros((num_layers, num_seqs, self.slots), dtype=torch.uint8, device=dev)
            self.head_state = torch.ones((num_seqs, 2, num_q_heads), dtype=torch.float32, device=dev)
        else:
            self.logits = self.head_state = None
            self.cumulative = torch.zeros((num_seqs, self.slots), dtype=torch.float64, device=dev)
            self.layer_ema = torch.zeros((num_layers, num_seqs, self.slots), dtype=torch.float32, device=dev)
            self.touched = torch.zeros((num_layers, num_seqs, self.slots), dtype=torch.uint8, device=dev)
        # hysteresis record of the allocator (smartkv/core/cache.py:423-450), storage order; streak -1 = none
        self.rank_pct = torch.zeros((num_seqs, self.slots), dtype=torch.float64, device=dev)
        self.rank_streak = torch.full((num_seqs, self.slots), -1, dtype=torch.int8, device=dev)
        self.appended_total = 0  # rows ever appended over all sequences (host-side upper bound of live tokens)
        self.max_seq_tokens = 0  # upper bound of the cached tokens of any one sequence (host side)
        self._realloc = None
        self.head_parity = 0
        self._bits_lut = torch.full((9,), -1, dtype=torch.int32, device=dev)
        for bits, b in BITS_TO_BUCKET.items():
            self._bits_lut[bits] = b
        self._base_t = torch.tensor(self.bucket_base, dtype=torch.int32, device=dev)
        self._seq_ids = torch.arange(num_seqs, dtype=torch.int32, device=dev)

    # ------------------------------------------------------------------ helpers
    def _stream(self):
        return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    @staticmethod
    def _dtype_code(t: torch.Tensor) -> int:
        if t.dtype == torch.float32:
            return _lib.DTYPE_F32
        if t.dtype == torch.float16:
            return _lib.DTYPE_F16
        raise TypeError(f"expected float32 or float16, got {t.dtype}")

    def algorithmic_bytes(self) -> int:
        """Packed bytes one decode step streams per layer: sum over sequences and
        buckets of n_b * Hkv * 2 * (row_bytes + 4) (reads the live counts: syncs)."""
        c = self.counts.to("cpu", torch.int64)
        per_tok = torch.tensor([self.num_kv_heads * 2 * (int(self.desc.row_bytes[i]) + 4) for i in range(NUM_BUCKETS)])
        return int((c * per_tok).sum())

    # ------------------------------------------------------------------ placement
    def plan_bulk(self, bits: torch.Tensor):
        """Place ``bits.shape[1]`` new tokens per sequence (ids continue each
        sequence's numbering).  bits int [B, n] on the device.  Returns the flat
        (dst_seq, dst_bucket, dst_pos) arrays for skv_quantize_pack_append and
        commits the bookkeeping (counts, storage-order token ids)."""
        B, n = bits.shape
        assert B == self.num_seqs
        bucket = self._bits_lut[bits.long()]                        # [B, n]
        if bool((bucket < 0).any()):
            raise ValueError("bits must be in {2,3,4,8}")
        onehot = torch.nn.functional.one_hot(bucket.long(), NUM_BUCKETS).to(torch.int32)   # [B,n,4]
        rank = torch.cumsum(onehot, dim=1) - onehot                 # tokens of the same bucket before this one
        pos = (rank * onehot).sum(-1).to(torch.int32) + self.counts.gather(1, bucket.long())
        added = onehot.sum(1).to(torch.int32)
        new_counts = self.counts + added
        caps = torch.tensor(self.caps, dtype=torch.int32, device=self.device)
        if bool((new_counts > caps).any()):
            raise _lib.SmartKVLibraryError("bucket capacity exceeded (SKV_ERR_CAPACITY)")
        token_ids = self.next_token[:, None] + torch.arange(n, dtype=torch.int32, device=self.device)[None]
        storage = self._base_t[bucket.long()] + pos
        self.slot_token.scatter_(1, storage.long(), token_ids)
        self.counts.copy_(new_counts)
        self._plan_valid = False
        self.next_token += n
        self.appended_total += B * n
        self.max_seq_tokens += n
        dst_seq = self._seq_ids[:, None].expand(B, n).contiguous().view(-1)
        return dst_seq, bucket.contiguous().view(-1), pos.contiguous().view(-1), storage

    def plan_step(self, bits: Optional[torch.Tensor] = None):
        """Destination of the token each sequence appends this decode step (same bucket position in every
        layer); does not commit.  Returns (dst_seq, dst_bucket, dst_pos, storage), int32 [num_seqs] each,
        in buffers the store reuses every step."""
        if getattr(self, "_step_bufs", None) is None:
            self._step_bufs = tuple(torch.zeros(self.num_seqs, dtype=torch.int32, device=self.device) for _ in range(4))
        seq, bucket, pos, storage = self._step_bufs
        b8 = None if bits is None else bits.to(torch.uint8).contiguous()
        check(self.lib.skv_step_plan(ctypes.byref(self.desc), ptr(self.counts), ptr(b8), ptr(seq), ptr(bucket), ptr(pos),
                                     ptr(storage), ptr(self.err), self._stream()), "skv_step_plan")
        return seq, bucket, pos, storage

    def commit_step(self, plan):
        """End of a decode step: the importance update still owed runs, then the step's token is entered into the
        bookkeeping (counts, storage-order token ids).  A step whose token was committed early (a
        reallocation in the middle of the step needs the token among the candidates) ends with
        end_step() instead."""
        self.end_step()
        _seq, bucket, _pos, storage = plan
        check(self.lib.skv_step_commit(ctypes.byref(self.desc), ptr(self.counts), ptr(self.slot_token),
                                       ptr(self.next_token), ptr(bucket), ptr(storage), self._stream()),
              "skv_step_commit")
        self.appended_total += self.num_seqs
        self.max_seq_tokens += 1
        self._plan_valid = False

    def capture_updates(self) -> int:
        """Importance updates issued under stream capture since the last call (and resets the count); a captured
        graph must hold an even number of them, see end_step."""
        n = getattr(self, "_capture_updates", 0)
        self._capture_updates = 0
        return n

    def end_step(self):
        """The part of commit_step that does not touch the bookkeeping."""
        self.flush_importance()          # reads the counts as they stood during the step
        if getattr(self, "_pipe", None) is not None:
            self._pipe["calls"] = 0      # every step starts on the same buffer set (CUDA graph replays rely on it)
            self._pipe["post_events"] = []
        if torch.cuda.is_current_stream_capturing() and getattr(self, "capture_check", "step") == "caller":
            return      # whoever captures several calls of this into one graph checks the total (capture_updates())
        n = getattr(self, "_capture_updates", 0)
        self._capture_updates = 0
        if torch.cuda.is_current_stream_capturing() and n % 2:
            # The head-importance EMA is double buffered and the half to read is a launch argument: a captured step
            # replays the same arguments, which is only right if the step flips the parity an even number of times.
            # Nothing of the capture has run, so the host's parity goes back to what the device state matches.
            self.head_parity ^= 1
            raise _lib.SmartKVLibraryError(
                f"a CUDA-graph-captured decode step holds {n} importance updates; it must hold an even number "
                "(the head-importance state is double buffered by launch argument): capture two steps per graph "
                "or run this model's steps without a graph")

    # ------------------------------------------------------------------ kernels
    def append(self, layer: int, k: torch.Tensor, v: torch.Tensor, dst_seq, dst_bucket, dst_pos):
        """k, v: [rows, Hkv, D] fp32/fp16 on the device."""
        k = k.contiguous()
        v = v.contiguous()
        rows = k.shape[0]
        assert k.shape == (rows, self.num_kv_heads, self.head_dim) and v.shape == k.shape and k.dtype == v.dtype
        check(self.lib.skv_quantize_pack_append(ctypes.byref(self.desc), ptr(self.arena), layer, ptr(k), ptr(v),
                                                self._dtype_code(k), rows, ptr(dst_seq), ptr(dst_bucket),
                                                ptr(dst_pos), self._stream()), "skv_quantize_pack_append")

    def attention(self, layer: int, query: torch.Tensor, cur_k: Optional[torch.Tensor] = None,
                  cur_v: Optional[torch.Tensor] = None, update_importance: bool = False,
                  cur_storage: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                  kernel_events=None, mask: Optional[torch.Tensor] = None,
                  cur_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One decode-attention call for ``layer``: query [B, Hq, D] (fp32/fp16),
        optional current token cur_k/cur_v [B, Hkv, D].  Returns fp32 [B, Hq, D].
        ``kernel_events`` = (start, end) torch CUDA events recorded around the
        streaming attention kernel alone (for roofline timing).
        ``mask``: additive fp32 [B, n] indexed by token id (natural-log units, as the reference's
        attention_mask); ``cur_mask``: fp32 [B], the mask value of the current token."""
        q = query.contiguous()
        assert q.shape == (self.num_seqs, self.num_q_heads, self.head_dim)
        want_logits = update_importance and self.track_importance
        st = self._stream()
        self.flush_importance()
        if not self._plan_valid:
            self.build_plan()
        if kernel_events is not None:
            kernel_events[0].record()
        if mask is not None:
            mask = mask.to(torch.float32).contiguous()
            assert mask.dim() == 2 and mask.shape[0] == self.num_seqs
        check(self.lib.skv_decode_attention_masked(ctypes.byref(self.desc), ptr(self.arena), layer, ptr(self.plan), ptr(q),
                                                   self._dtype_code(q), self.num_q_heads, ptr(self.partials),
                                                   self.num_ctas, ptr(self.logits) if want_logits else None, ptr(mask),
                                                   0 if mask is None else int(mask.shape[1]),
                                                   ptr(self.slot_token) if mask is not None else None, 0, ptr(self.err), st),
              "skv_decode_attention")
        if kernel_events is not None:
            kernel_events[1].record()
        out = self.out if out is None else out
        if cur_mask is not None:
            cur_mask = cur_mask.to(torch.float32).contiguous()
        kv_code = _lib.DTYPE_F32
        if cur_k is not None:
            cur_k = cur_k.contiguous()
            cur_v = cur_v.contiguous()
            kv_code = self._dtype_code(cur_k)
        check(self.lib.skv_lse_combine_masked(ctypes.byref(self.desc), ptr(self.plan), ptr(q), self._dtype_code(q),
                                              self.num_q_heads, ptr(self.partials), self.num_ctas, ptr(cur_k), ptr(cur_v),
                                              kv_code, ptr(cur_mask), ptr(out), ptr(self.lse_max), ptr(self.lse_sum),
                                              ptr(self.cur_prob), st),
              "skv_lse_combine")
        if want_logits:
            has_cur = cur_k is not None and cur_storage is not None
            check(self.lib.skv_importance_update(ctypes.byref(self.desc), layer, ptr(self.counts), self.num_q_heads,
                                                 ptr(self.logits), ptr(self.lse_max), ptr(self.lse_sum),
                                                 ptr(self.cur_prob) if has_cur else None,
                                                 ptr(cur_storage) if has_cur else None, ptr(self.head_state),
                                                 self.head_parity, ptr(self.cumulative), ptr(self.layer_ema),
                                                 ptr(self.touched), self.decay, self.head_decay, st),
                  "skv_importance_update")
            self.head_parity ^= 1
        return out

    def decode_layer(self, layer: int, query: torch.Tensor, cur_k: torch.Tensor, cur_v: torch.Tensor, step_plan,
                     update_importance: bool = True, out: Optional[torch.Tensor] = None,
                     kernel_events=None, overlap: bool = False, mask: Optional[torch.Tensor] = None,
                     before_post=None) -> torch.Tensor:
        """One layer of a decode step in two launches: the streaming attention kernel, then one kernel
        with this layer's combine, the append of the new token (``step_plan`` from plan_step) and the
        importance update of the PREVIOUS decode_layer call (skv_post_attention).  The last layer's
        importance update is flushed by commit_step / flush_importance.  Same results as
        attention(...) followed by append(...).

        ``overlap``: the second launch goes to a side stream, so that it runs while the NEXT layer's attention
        kernel is already starting (it fills the SMs that kernel's CTAs leave early); the attention kernel of
        call m then only waits for the side work of call m-2 (partials are double, logits triple buffered).
        The outputs of such a call are ready after join() / commit_step().

        ``mask``: additive fp32 [B, n] indexed by token id, natural-log units (see attention()).
        ``before_post``: called between the two launches; a caller that must make the stream wait for something the
        NEXT layer needs (its inputs arriving on a copy stream) does it there, so that the next layer's attention
        kernel directly follows this layer's second launch and can be launched as its dependent."""
        q = query.contiguous()
        assert q.shape == (self.num_seqs, self.num_q_heads, self.head_dim)
        want_logits = update_importance and self.track_importance
        plan_was_valid = self._plan_valid
        if not self._plan_valid:
            self.build_plan()
        pipe = self._pipe_buffers()
        m = pipe["calls"]
        lslot, pslot = m % 3, m % 2
        # The attention kernel of the second and later layers of a step may be launched as a dependent of what runs
        # before it (the previous layer's post-attention kernel, or the model's own kernels between two layers): none of
        # those writes the plan or this layer's rows.  Not so right after a plan rebuild or at the start of a step.
        flags = _lib.ATTN_DEPENDENT_LAUNCH if (m > 0 and plan_was_valid and not overlap and kernel_events is None) else 0
        bufs = pipe["bufs"][lslot]
        partials = pipe["partials"][pslot]
        main = torch.cuda.current_stream(self.device)
        if overlap and len(pipe["post_events"]) >= 2:
            main.wait_event(pipe["post_events"][-2])      # the buffers this call reuses are free again
        st = self._stream()
        if kernel_events is not None:
            kernel_events[0].record()
        if mask is not None:
            assert mask.dtype == torch.float32 and mask.is_contiguous() and mask.shape[0] == self.num_seqs
        check(self.lib.skv_decode_attention_masked(ctypes.byref(self.desc), ptr(self.arena), layer, ptr(self.plan), ptr(q),
                                                   self._dtype_code(q), self.num_q_heads, ptr(partials), self.num_ctas,
                                                   ptr(bufs["logits"]) if want_logits else None, ptr(mask),
                                                   0 if mask is None else int(mask.shape[1]),
                                                   ptr(self.slot_token) if mask is not None else None, flags, ptr(self.err), st),
              "skv_decode_attention")
        if kernel_events is not None:
            kernel_events[1].record()
        out = self.out if out is None else out
        has_cur = cur_k is not None
        if has_cur:
            cur_k = cur_k.contiguous()
            cur_v = cur_v.contiguous()
        dst_seq, dst_bucket, dst_pos, storage = step_plan if has_cur else (None, None, None, None)
        pend = pipe["pending"]
        pb = pipe["bufs"][pend["buf"]] if pend is not None else None
        small = pipe["small"]                         # (max, sum, current-token probability) of every layer of the step
        ps = {k2: v2[pend["layer"]] for k2, v2 in small.items()} if pend is not None else None
        # Under stream capture the host scalars below would be baked into the graph: the importance blocks then
        # cover the store's token capacity (or every storage index, 0 = full grid, if nobody stated one) instead of
        # the capture-time token count, and the
        # head-state parity, which must alternate per update, is refused unless a captured step holds an even
        # number of updates (checked by the caller of commit_step through _capture_updates).
        capturing = torch.cuda.is_current_stream_capturing()
        # token_capacity (set by whoever sized the buckets): the most tokens a sequence can ever hold, a bound that stays
        # valid however often the graph is replayed
        max_tokens_arg = int(getattr(self, "token_capacity", 0) or 0) if capturing else self.max_seq_tokens

        def post(stream_ptr):
            check(self.lib.skv_post_attention(
                ctypes.byref(self.desc), ptr(self.arena), layer, ptr(self.plan), ptr(q), self._dtype_code(q),
                self.num_q_heads, ptr(partials), self.num_ctas, ptr(cur_k), ptr(cur_v),
                self._dtype_code(cur_k) if has_cur else _lib.DTYPE_F32,
                ptr(out), ptr(small["lse_max"][layer]), ptr(small["lse_sum"][layer]), ptr(small["cur_prob"][layer]),
                ptr(self.counts),
                pend["layer"] if pend is not None else 0, ptr(pb["logits"]) if pend is not None else None,
                ptr(ps["lse_max"]) if pend is not None else None, ptr(ps["lse_sum"]) if pend is not None else None,
                ptr(ps["cur_prob"]) if pend is not None else None,
                ptr(pend["storage"]) if pend is not None and pend["storage"] is not None else None,
                ptr(self.head_state), self.head_parity, ptr(self.cumulative), ptr(self.layer_ema), ptr(self.touched),
                self.decay, self.head_decay, ptr(dst_seq), ptr(dst_bucket), ptr(dst_pos), max_tokens_arg,
                ptr(self.err), stream_ptr), "skv_post_attention")

        if overlap:
            side = pipe["side"]
            done = torch.cuda.Event()
            done.record(main)
            side.wait_event(done)
            with torch.cuda.stream(side):
                post(self._stream())
                ev = torch.cuda.Event()
                ev.record(side)
            pipe["post_events"].append(ev)
            pipe["forked"] = True
        else:
            if before_post is not None:
                before_post()
            post(st)
        if pend is not None:
            self.head_parity ^= 1
            if capturing:
                self._capture_updates = getattr(self, "_capture_updates", 0) + 1
        pipe["pending"] = {"layer": layer, "buf": lslot, "storage": storage} if want_logits else None
        pipe["calls"] = m + 1
        self.lse_max, self.lse_sum, self.cur_prob = small["lse_max"][layer], small["lse_sum"][layer], small["cur_prob"][layer]
        return out

    def _pipe_buffers(self):
        """Three sets of (logits, max, sum, current-token probability) and two of partials: the importance
        update of a layer runs one launch after its attention, and with ``overlap`` that launch may still be
        running while the next layer's attention kernel writes the following set."""
        if getattr(self, "_pipe", None) is None:
            dev, B, Hq = self.device, self.num_seqs, self.num_q_heads
            bufs = []
            for i in range(3):
                bufs.append({
                    "logits": (self.logits if i == 0 else torch.empty_like(self.logits)) if self.track_importance else None,
                })
            # the small per-layer results stay addressable for the whole step (a sequence-sharded step exchanges
            # all layers' (max, sum, out) at once)
            small = {k: torch.empty((self.num_layers, B, Hq), dtype=torch.float32, device=dev)
                     for k in ("lse_max", "lse_sum", "cur_prob")}
            self._pipe = {"bufs": bufs, "small": small, "partials": [self.partials, torch.empty_like(self.partials)],
                          "calls": 0, "pending": None, "side": torch.cuda.Stream(device=dev), "post_events": [],
                          "forked": False}
        return self._pipe

    def join(self):
        """Makes the current stream wait for side-stream work of decode_layer(overlap=True) calls."""
        pipe = getattr(self, "_pipe", None)
        if pipe is None or not pipe["forked"]:
            return
        torch.cuda.current_stream(self.device).wait_event(pipe["post_events"][-1])
        pipe["forked"] = False

    def take_pending_logits(self):
        """Cancels the importance update owed by the last decode_layer call and hands its inputs to the caller:
        (logits fp32 [B, Hq, slots] in base-2 units, running max [B, Hq], sum [B, Hq], probability of the current
        token [B, Hq]); the probability of the key at storage index s is exp2(logit - max) / sum.  For callers
        that attribute the attention mass themselves."""
        pipe = getattr(self, "_pipe", None)
        if pipe is None or pipe["pending"] is None:
            return None
        self.join()
        pend = pipe["pending"]
        pipe["pending"] = None
        sm = pipe["small"]
        return (pipe["bufs"][pend["buf"]]["logits"], sm["lse_max"][pend["layer"]], sm["lse_sum"][pend["layer"]],
                sm["cur_prob"][pend["layer"]])

    def flush_importance(self):
        """Runs the importance update still owed by the last decode_layer call (no-op otherwise)."""
        pipe = getattr(self, "_pipe", None)
        if pipe is None:
            return
        self.join()
        pend = pipe["pending"]
        if pend is None:
            return
        pb = pipe["bufs"][pend["buf"]]
        sm = {k: v[pend["layer"]] for k, v in pipe["small"].items()}
        if torch.cuda.is_current_stream_capturing():
            self._capture_updates = getattr(self, "_capture_updates", 0) + 1
        check(self.lib.skv_importance_update(ctypes.byref(self.desc), pend["layer"], ptr(self.counts), self.num_q_heads,
                                             ptr(pb["logits"]), ptr(sm["lse_max"]), ptr(sm["lse_sum"]),
                                             ptr(sm["cur_prob"]) if pend["storage"] is not None else None,
                                             ptr(pend["storage"]) if pend["storage"] is not None else None, ptr(self.head_state),
                                             self.head_parity, ptr(self.cumulative), ptr(self.layer_ema),
                                             ptr(self.touched), self.decay, self.head_decay, self._stream()),
              "skv_importance_update")
        self.head_parity ^= 1
        pipe["pending"] = None

    def build_plan(self):
        """(Re)build the attention work partition from the live bucket counts.  Needed once
        after the counts change (bulk store, a committed decode step, a reallocation); every
        layer of a step shares it."""
        check(self.lib.skv_attn_plan(ctypes.byref(self.desc), ptr(self.counts), self.num_ctas, ptr(self.plan),
                                     self._stream()), "skv_attn_plan")
        self._plan_valid = True

    def autotune_attention(self, query: torch.Tensor, layers: int = 2, iters: int = 3) -> dict:
        """Times the two decode-attention kernels on the cache as it stands (``layers`` launches over different
        layers, ``iters`` repetitions, CUDA events) and selects the faster one for the process
        (skv_set_attention_path).  Only fp16 queries at head_dim 128 have a choice.  The fragment kernel wins
        on mixed-width caches, the tensor-memory kernel once most tokens are 8-bit; which side a cache falls on
        changes with the memory budget, so measure after a reallocation.  Returns the timings in microseconds."""
        q = query.contiguous()
        if self.head_dim != 128 or q.dtype != torch.float16:
            self.lib.skv_set_attention_path(0)
            return {"selected": "fragment", "reason": "only head_dim 128 with fp16 queries has a choice"}
        dev = self.device
        n = max(1, min(layers, self.num_layers))
        times = {}
        for name, path in (("fragment", 1), ("tensor_memory", 2)):
            check(self.lib.skv_set_attention_path(path), "skv_set_attention_path")
            self.build_plan()
            best = float("inf")
            for it in range(iters + 1):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for layer in range(n):
                    check(self.lib.skv_decode_attention(ctypes.byref(self.desc), ptr(self.arena), layer, ptr(self.plan),
                                                        ptr(q), self._dtype_code(q), self.num_q_heads, ptr(self.partials),
                                                        self.num_ctas, None, ptr(self.err), self._stream()),
                          "skv_decode_attention")
                e1.record()
                torch.cuda.synchronize(dev)
                if it > 0:
                    best = min(best, e0.elapsed_time(e1) * 1e3 / n)
            times[name] = round(best, 2)
        sel = "tensor_memory" if times["tensor_memory"] < times["fragment"] else "fragment"
        check(self.lib.skv_set_attention_path(2 if sel == "tensor_memory" else 1), "skv_set_attention_path")
        self._plan_valid = False
        self.check_errors()
        return {"selected": sel, "us_per_launch": times}

    def check_errors(self):
        """Reads the device error flag (synchronises)."""
        val = ctypes.c_int32(0)
        check(self.lib.skv_read_error_flag(ptr(self.err), ctypes.byref(val), self._stream()), "device error flag")


    # ------------------------------------------------------------------ reallocation
    def make_alloc_config(self, memory_budget: float, available_bits: Sequence[int] = (2, 3, 4, 8),
                          total_kv_heads: Optional[int] = None, **kw) -> "_lib.AllocConfig":
        """Allocator parameters for this store (see make_alloc_config at module level).  ``total_kv_heads``:
        KV heads of the whole model when this store holds a shard of them (accounting only)."""
        return make_alloc_config(int(total_kv_heads or self.num_kv_heads), self.head_dim, memory_budget,
                                 available_bits, **kw)

    def _realloc_buffers(self):
        if getattr(self, "_realloc", None) is not None:
            return self._realloc
        dev, B, T = self.device, self.num_seqs, self.slots
        d = ctypes.byref(self.desc)
        r = {
            "alloc_ws": torch.empty(int(self.lib.skv_alloc_workspace_bytes(d)), dtype=torch.uint8, device=dev),
            "plan_ws": torch.empty(int(self.lib.skv_repack_plan_workspace_bytes(d)), dtype=torch.uint8, device=dev),
            "new_bits": torch.zeros((B, T), dtype=torch.uint8, device=dev),
            "new_counts": torch.zeros((B, NUM_BUCKETS), dtype=torch.int32, device=dev),
            "counts_new": torch.zeros((B, NUM_BUCKETS), dtype=torch.int32, device=dev),
            "changed": torch.zeros(B, dtype=torch.int32, device=dev),
            "move_src": torch.zeros((B, T), dtype=torch.int32, device=dev),
            "move_dst": torch.zeros((B, T), dtype=torch.int32, device=dev),
            "n_moves": torch.zeros(B, dtype=torch.int32, device=dev),
            "staging": None,
            "meta_staging": None,
        }
        self._realloc = r
        return r

    def allocate_bits(self, cfg, scores: Optional[torch.Tensor] = None, recency: Optional[torch.Tensor] = None):
        """Runs the allocator on every sequence (skv_alloc_bits).  ``scores``: fp64 [B, slots] in
        storage order, default the cumulative importance.  Returns (new_bits uint8 [B, slots],
        new_counts int32 [B, 4], changed int32 [B]) -- device tensors owned by the store."""
        self.flush_importance()
        r = self._realloc_buffers()
        scores = self.cumulative if scores is None else scores
        check(self.lib.skv_alloc_bits(ctypes.byref(self.desc), ctypes.byref(cfg), ptr(self.counts), ptr(self.slot_token),
                                      ptr(scores), ptr(recency), ptr(self.rank_pct), ptr(self.rank_streak),
                                      ptr(r["new_bits"]), ptr(r["new_counts"]), ptr(r["changed"]), ptr(r["alloc_ws"]),
                                      self._stream()), "skv_alloc_bits")
        return r["new_bits"], r["new_counts"], r["changed"]

    def repack(self, new_bits: torch.Tensor, max_moves: Optional[int] = None, staging_budget: int = 1 << 30):
        """Moves every token to the bucket of its new width (requantising from the stored codes)
        in all layers and permutes the per-token arrays accordingly.  ``max_moves``: upper bound of
        the rows that can move over all sequences (default: every token ever appended)."""
        r = self._realloc_buffers()
        d = ctypes.byref(self.desc)
        st = self._stream()
        check(self.lib.skv_repack_plan(d, ptr(self.counts), ptr(new_bits), ptr(r["move_src"]), ptr(r["move_dst"]),
                                       ptr(r["n_moves"]), ptr(r["counts_new"]), ptr(r["plan_ws"]), ptr(self.err), st),
              "skv_repack_plan")
        if max_moves is None:
            max_moves = self.appended_total
        max_moves = max(int(max_moves), 1)
        per_layer = int(self.lib.skv_requant_staging_bytes(d, max_moves, 1))
        chunk = max(1, min(self.num_layers, staging_budget // max(per_layer, 1)))
        need = per_layer * chunk
        if r["staging"] is None or r["staging"].numel() < need:
            r["staging"] = torch.empty(need, dtype=torch.uint8, device=self.device)
        mneed = int(self.lib.skv_repack_meta_staging_bytes(d, max_moves + 8))
        if r["meta_staging"] is None or r["meta_staging"].numel() < mneed:
            r["meta_staging"] = torch.empty(mneed, dtype=torch.uint8, device=self.device)
        for l0 in range(0, self.num_layers, chunk):
            l1 = min(self.num_layers, l0 + chunk)
            check(self.lib.skv_requant_repack(d, ptr(self.arena), l0, l1, ptr(r["move_src"]), ptr(r["move_dst"]),
                                              ptr(r["n_moves"]), ptr(r["staging"]), r["staging"].numel(), ptr(self.err),
                                              st), "skv_requant_repack")
        check(self.lib.skv_repack_meta(d, ptr(r["move_src"]), ptr(r["move_dst"]), ptr(r["n_moves"]), ptr(self.counts),
                                       ptr(r["counts_new"]), ptr(self.slot_token), ptr(self.cumulative),
                                       ptr(self.rank_pct), ptr(self.rank_streak), ptr(self.layer_ema), ptr(self.touched),
                                       ptr(r["meta_staging"]), r["meta_staging"].numel(), ptr(self.err), st),
              "skv_repack_meta")
        self._plan_valid = False

    def reallocate(self, cfg, max_moves: Optional[int] = None, staging_budget: int = 1 << 30):
        """allocate_bits + repack: one reallocation of the whole store."""
        new_bits, _, _ = self.allocate_bits(cfg)
        self.repack(new_bits, max_moves=max_moves, staging_budget=staging_budget)

    def reallocate_graphed(self, cfg, staging_budget: int = 1 << 30):
        """reallocate() as one CUDA graph launch: a reallocation is about 70 small launches, and issuing them
        one by one costs more than running them once the allocation has settled.  The first call runs eagerly
        (it sizes every buffer for the store's whole capacity, so that the captured launches stay valid as the
        cache grows) and captures the graph; later calls replay it.  ``cfg`` must be the same at every call.
        ``staging_budget`` bytes of staging decide how many layers one pair of row-move launches covers: every
        pair costs tens of microseconds however few rows move, so a larger budget makes a quiet reallocation cheaper."""
        self.flush_importance()
        cap_moves = self.num_seqs * self.slots
        if getattr(self, "_realloc_graph", None) is None:
            self.reallocate(cfg, max_moves=cap_moves, staging_budget=staging_budget)
            self._realloc_cfg = cfg  # the graph's kernels hold a copy of it; keeps the object alive all the same
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self.reallocate(cfg, max_moves=cap_moves, staging_budget=staging_budget)
            self._realloc_graph = graph
            return
        self._realloc_graph.replay()
        self._plan_valid = False

    def token_bits(self, seq: int) -> torch.Tensor:
        """Width of every token of one sequence, indexed by token id (syncs; tests and the API mirror)."""
        counts = self.counts[seq].tolist()
        n = sum(counts)
        out = torch.zeros(max(int(self.next_token[seq]), n), dtype=torch.uint8, device=self.device)
        for i, c in enumerate(counts):
            if c:
                ids = self.slot_token[seq, self.bucket_base[i]: self.bucket_base[i] + c].long()
                out[ids] = BUCKET_BITS[i]
        return out

    # ------------------------------------------------------------------ read back (tests, API mirror)
    def export_sequence(self, layer: int, seq: int):
        """All cached tokens of one sequence in token-id order: (token_ids, bits,
        k_codes int8 [n,Hkv,D], v_codes, k_scale fp32 [n,Hkv], v_scale)."""
        counts = self.counts[seq].tolist()
        seqs, buckets, poss, ids, bits = [], [], [], [], []
        for i, c in enumerate(counts):
            if c == 0:
                continue
            poss.append(torch.arange(c, dtype=torch.int32, device=self.device))
            buckets.append(torch.full((c,), i, dtype=torch.int32, device=self.device))
            ids.append(self.slot_token[seq, self.bucket_base[i]: self.bucket_base[i] + c])
            bits.append(torch.full((c,), BUCKET_BITS[i], dtype=torch.int32, device=self.device))
        n = sum(counts)
        H, D = self.num_kv_heads, self.head_dim
        if n == 0:
            e8 = torch.empty((0, H, D), dtype=torch.int8, device=self.device)
            ef = torch.empty((0, H), dtype=torch.float32, device=self.device)
            ei = torch.empty(0, dtype=torch.int32, device=self.device)
            return ei, ei.clone(), e8, e8.clone(), ef, ef.clone()
        pos, bucket, ids, bits = torch.cat(poss), torch.cat(buckets), torch.cat(ids), torch.cat(bits)
        order = torch.argsort(ids)
        pos, bucket, ids, bits = pos[order].contiguous(), bucket[order].contiguous(), ids[order], bits[order]
        sq = torch.full((n,), seq, dtype=torch.int32, device=self.device)
        kc = torch.empty((n, H, D), dtype=torch.int8, device=self.device)
        vc = torch.empty_like(kc)
        ks = torch.empty((n, H), dtype=torch.float32, device=self.device)
        vs = torch.empty_like(ks)
        check(self.lib.skv_export_rows(ctypes.byref(self.desc), ptr(self.arena), layer, n, ptr(sq), ptr(bucket), ptr(pos),
                                       ptr(kc), ptr(vc), ptr(ks), ptr(vs), self._stream()), "skv_export_rows")
        return ids, bits, kc, vc, ks, vs

    def bucket_rows(self, layer: int, seq: int, bucket: int):
        """Raw packed bytes of one bucket: (K rows uint8 [Hkv, n, row_bytes], V rows, k_scale [Hkv, n], v_scale)."""
        d = self.desc
        n = int(self.counts[seq, bucket])
        base = (layer * self.num_seqs + seq) * int(d.arena_bytes)
        H, cap, rb = self.num_kv_heads, self.caps[bucket], int(d.row_bytes[bucket])

        def region(off, nbytes_row, dtype):
            raw = self.arena[base + off: base + off + H * cap * nbytes_row]
            return raw.view(dtype).view(H, cap, -1)[:, :n]
        k = region(int(d.k_off[bucket]), rb, torch.uint8)
        v = region(int(d.v_off[bucket]), rb, torch.uint8)
        sc = region(int(d.sc_off[bucket]), 8, torch.float32)
        return k, v, sc[..., 0], sc[..., 1]
