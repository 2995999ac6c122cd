"""CPU oracle for the SmartKV quantized-KV decode path.

TEST INFRASTRUCTURE ONLY.  This module is a NumPy restatement of the reference
algorithm (Robbyswimmer/SmartKV, CPU path).  It is imported by the test-suite,
by the smoke check and by the benchmark's CPU-baseline leg, and by nothing
else: the product path (the CUDA library) never calls into it and has no CPU
fallback.

Parity status: PINNED.  Every function below is checked in the CPU test-suite
against golden vectors produced by importing the reference's own Python
modules (see tests/golden/make_golden.py, which records the reference call
that produced each vector), and against the constants the reference's own
tests assert (minimum budgets 0.53125 / 0.515625 / 0.15625 / 0.140625, the
0.2578 packed ratio, code ranges per bit-width, zero-input scale 1.0).

The reference has no CPU bit-packer (its CPU "pack" is a uint8 cast); the
packed byte format is therefore restated from the reference's CUDA pack/unpack
kernels and pinned by round-trip properties plus hand-computed byte vectors.

Each function cites the reference file:line it follows (paths relative to the
reference project root).
"""
from __future__ import annotations

import heapq
import math
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np

SUPPORTED_BITS = (2, 3, 4, 8)


# --------------------------------------------------------------------------
# Quantizer  (smartkv/core/_quant_cpu.py:20-34)
# --------------------------------------------------------------------------
def code_range(bits: int) -> Tuple[int, int]:
    """(min_code, max_code) for a bit-width; bits==1 degenerates to (0, 0).

    smartkv/core/_quant_cpu.py:20-24.
    """
    if bits == 1:
        return 0, 0
    return -(1 << (bits - 1)), (1 << (bits - 1)) - 1


def quantize_rows(x: np.ndarray, bits: int) -> Tuple[np.ndarray, np.ndarray]:
    """Symmetric per-(token, head) quantization of ``x[..., D]``.

    scale = absmax / max(max_code, 1) in fp32, a zero scale becomes 1.0,
    code = clamp(round_half_even(x / scale)).  smartkv/core/_quant_cpu.py:26-29.
    Returns (codes int8 same shape, scale fp32 shape[:-1]).
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    lo, hi = code_range(bits)
    absmax = np.max(np.abs(x), axis=-1, keepdims=True).astype(np.float32)
    scale = (absmax / np.float32(max(hi, 1))).astype(np.float32)
    scale = np.where(scale == 0, np.float32(1.0), scale).astype(np.float32)
    q = np.rint((x / scale).astype(np.float32))
    q = np.clip(q, lo, hi).astype(np.int8)
    return q, scale[..., 0]


def quantize_per_head(k: np.ndarray, v: np.ndarray, bits: int):
    """Mirror of ``quantize_per_head(k, v, bits)`` (smartkv/core/_quant_cpu.py:4-54).

    Returns (k_codes, v_codes, k_scale, v_scale).
    """
    kq, ks = quantize_rows(k, bits)
    vq, vs = quantize_rows(v, bits)
    return kq, vq, ks, vs


def dequantize_rows(codes: np.ndarray, scale: np.ndarray) -> np.ndarray:
    """codes * scale in fp32 (smartkv/core/cache.py:1534-1541)."""
    return codes.astype(np.float32) * scale.astype(np.float32)[..., None]


# --------------------------------------------------------------------------
# Packed byte format  (smartkv/csrc/bit_packing.cu:20-43, 69-95, 128-151;
# unpack helpers smartkv/csrc/quantized_attention.cu:81-113)
# --------------------------------------------------------------------------
def packed_size(num_elements: int, bits: int) -> int:
    """Bytes needed for ``num_elements`` codes (smartkv/kernels/bit_packing.py:102-122)."""
    if bits == 2:
        return (num_elements + 3) // 4
    if bits == 3:
        return ((num_elements + 7) // 8) * 3
    if bits == 4:
        return (num_elements + 1) // 2
    if bits == 8:
        return num_elements
    raise ValueError(f"bits must be 2, 3, 4, or 8, got {bits}")


def pack_codes(codes: np.ndarray, bits: int) -> np.ndarray:
    """Pack a flat int8 code vector.

    Offset-binary (code + 2^(bits-1)), element i of a byte group in the low
    bits first.  2-bit: 4 per byte; 4-bit: even index = low nibble; 3-bit: 8
    codes form a 24-bit little-endian word written as 3 bytes.  8-bit is the
    identity on the two's-complement byte.  A trailing partial group is
    zero-filled.  smartkv/csrc/bit_packing.cu:20-43, 69-95, 128-151, 305-313.
    """
    flat = np.ascontiguousarray(codes, dtype=np.int8).reshape(-1)
    n = flat.size
    if bits == 8:
        return flat.view(np.uint8).copy()
    if bits not in (2, 3, 4):
        raise ValueError(f"bits must be 2, 3, 4, or 8, got {bits}")
    off = 1 << (bits - 1)
    mask = (1 << bits) - 1
    u = ((flat.astype(np.int32) + off) & mask).astype(np.uint32)
    if bits == 2:
        per = 4
    elif bits == 4:
        per = 2
    else:
        per = 8
    groups = (n + per - 1) // per
    padded = np.zeros(groups * per, dtype=np.uint32)
    padded[:n] = u
    padded = padded.reshape(groups, per)
    shifts = (np.arange(per, dtype=np.uint32) * bits)[None, :]
    words = np.bitwise_or.reduce(padded << shifts, axis=1)
    if bits == 3:
        out = np.empty((groups, 3), dtype=np.uint8)
        out[:, 0] = words & 0xFF
        out[:, 1] = (words >> 8) & 0xFF
        out[:, 2] = (words >> 16) & 0xFF
        return out.reshape(-1)
    return words.astype(np.uint8)


def unpack_codes(packed: np.ndarray, bits: int, num_elements: int) -> np.ndarray:
    """Inverse of :func:`pack_codes` (smartkv/csrc/bit_packing.cu:45-62, 97-121, 153-170)."""
    p = np.ascontiguousarray(packed, dtype=np.uint8).reshape(-1)
    if bits == 8:
        return p[:num_elements].view(np.int8).copy()
    off = 1 << (bits - 1)
    mask = (1 << bits) - 1
    idx = np.arange(num_elements, dtype=np.int64)
    bitpos = idx * bits
    byte = bitpos >> 3
    sh = (bitpos & 7).astype(np.uint32)
    lo = p[byte].astype(np.uint32)
    nxt = np.minimum(byte + 1, p.size - 1)
    hi = p[nxt].astype(np.uint32)
    window = lo | (hi << 8)
    u = (window >> sh) & mask
    return (u.astype(np.int32) - off).astype(np.int8)


def pack_rows(codes: np.ndarray, bits: int) -> np.ndarray:
    """Pack ``codes[..., D]`` row by row -> uint8 ``[..., packed_size(D)]``.

    Equals packing the flattened ``[H*D]`` vector and reshaping to ``[H, pd]``
    whenever D % 8 == 0, which is how the reference fills its bucket buffers
    (smartkv/core/cache.py:1067-1072).
    """
    codes = np.ascontiguousarray(codes, dtype=np.int8)
    d = codes.shape[-1]
    if bits != 8 and d % 8 != 0:
        raise ValueError("row packing needs head_dim % 8 == 0")
    pd = packed_size(d, bits)
    return pack_codes(codes.reshape(-1), bits).reshape(codes.shape[:-1] + (pd,))


def unpack_rows(packed: np.ndarray, bits: int, head_dim: int) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    lead = packed.shape[:-1]
    n = int(np.prod(lead, dtype=np.int64)) * head_dim
    return unpack_codes(packed.reshape(-1), bits, n).reshape(lead + (head_dim,))


# --------------------------------------------------------------------------
# Memory accounting  (smartkv/core/allocation.py:401-441, 444-531)
# --------------------------------------------------------------------------
def compute_minimum_budget(num_heads=8, head_dim=128, scale_dtype="fp32", use_packing=False) -> float:
    """smartkv/core/allocation.py:401-441 (counts FOUR scale slots per head)."""
    sbits = 32 if scale_dtype == "fp32" else 16
    per_elem = 2 if use_packing else 8
    payload = 2 * num_heads * head_dim * per_elem
    scales = 4 * num_heads * sbits
    return (payload + scales) / (2 * num_heads * head_dim * 16)


def memory_ratio_true(allocation: Dict[int, int], num_heads: int, head_dim: int,
                      scale_dtype: str = "fp32", use_packing: bool = False) -> float:
    """``memory_ratio_true`` of smartkv/core/allocation.py:444-531 (TWO scale slots per head)."""
    n = len(allocation)
    if n == 0:
        return 0.0
    sbits = 32 if scale_dtype == "fp32" else 16
    elements = 2 * num_heads * head_dim
    payload = sum(b * elements for b in allocation.values()) if use_packing else n * elements * 8
    scales = n * 2 * num_heads * sbits
    return (payload + scales) / (n * elements * 16)


# --------------------------------------------------------------------------
# Attention oracles
# --------------------------------------------------------------------------
def expand_gqa(x: np.ndarray, group: int, axis: int = 1) -> np.ndarray:
    """repeat_interleave(group) along the head axis (smartkv/models/llama_smartkv.py:274-281)."""
    return np.repeat(x, group, axis=axis) if group > 1 else x


def dequant_attend(query, k_codes, k_scale, v_codes, v_scale, mask=None):
    """fp32 dequantise-then-attend (smartkv/kernels/__init__.py:389-416).

    query [B,H,q,D]; codes [B,H,N,D] int8; scales [B,H,N]; mask additive
    broadcastable to [B,H,q,N].  Returns (output [B,H,q,D], probs [B,H,q,N]).
    """
    q = np.asarray(query, dtype=np.float32)
    k = k_codes.astype(np.float32) * np.asarray(k_scale, np.float32)[..., None]
    v = v_codes.astype(np.float32) * np.asarray(v_scale, np.float32)[..., None]
    d = q.shape[-1]
    scores = np.matmul(q, np.swapaxes(k, -1, -2)) / np.float32(d ** 0.5)
    if mask is not None:
        scores = scores + np.asarray(mask, np.float32)
    scores = scores.astype(np.float32)
    m = scores.max(axis=-1, keepdims=True)
    e = np.exp(scores - m, dtype=np.float32)
    p = e / e.sum(axis=-1, keepdims=True, dtype=np.float32)
    return np.matmul(p, v).astype(np.float32), p.astype(np.float32)


def streaming_attention(query, k_codes, k_scale, v_codes, v_scale, *, mask=None,
                        tile_size: Optional[int] = None, current_k=None, current_v=None,
                        current_mask=None, return_attn: bool = True):
    """q_len==1 streaming softmax over int8 tiles plus the current fp token.

    Follows smartkv/core/fused_cpu.py:7-167: per tile dequantise, logits =
    q.k / sqrt(D) (+mask), running (max, sum, out) rescale; the newest token is
    a final one-key tile in full precision; probabilities are rebuilt from the
    saved logits with the final max and sum.

    query [B,H,1,D]; codes [N,H,D] int8 already expanded to the query heads;
    scales [N,H]; current_k/current_v [B,H,D].
    Returns (out [B,H,1,D], probs [B,H,1,N(+1)] or None).
    """
    q = np.asarray(query, dtype=np.float32)
    B, H, qlen, d = q.shape
    assert qlen == 1
    q = q[:, :, 0, :]
    N = k_codes.shape[0]
    if tile_size is None or tile_size <= 0:
        tile_size = max(128, (N + 11) // 12)          # fused_cpu.py:50-53
    out = np.zeros((B, H, d), np.float32)
    run_max = np.full((B, H), -np.inf, np.float32)
    run_sum = np.zeros((B, H), np.float32)
    m = None
    if mask is not None and np.size(mask) > 0:
        m = np.asarray(mask, np.float32).reshape(B, -1, N)
    inv = np.float32(1.0 / (d ** 0.5))
    saved: List[np.ndarray] = []
    for s in range(0, N, tile_size):
        e = min(s + tile_size, N)
        kt = k_codes[s:e].astype(np.float32) * np.asarray(k_scale[s:e], np.float32)[..., None]
        vt = v_codes[s:e].astype(np.float32) * np.asarray(v_scale[s:e], np.float32)[..., None]
        logits = np.einsum("bhd,thd->bht", q, kt, optimize=True).astype(np.float32) * inv
        if m is not None:
            logits = logits + m[..., s:e]
        if return_attn:
            saved.append(logits.copy())
        tmax = logits.max(axis=-1)
        new_max = np.maximum(run_max, tmax)
        with np.errstate(invalid="ignore"):
            resc = np.exp(run_max - new_max, dtype=np.float32)
        run_sum *= resc
        out *= resc[..., None]
        ex = np.exp(logits - new_max[..., None], dtype=np.float32)
        run_sum += ex.sum(axis=-1, dtype=np.float32)
        out += np.einsum("bht,thd->bhd", ex, vt, optimize=True).astype(np.float32)
        run_max = new_max
    cur_logits = None
    if current_k is not None and current_v is not None:
        ck = np.asarray(current_k, np.float32)
        cv = np.asarray(current_v, np.float32)
        lc = np.einsum("bhd,bhd->bh", q, ck).astype(np.float32) * inv
        if current_mask is not None and np.size(current_mask) > 0:
            lc = lc + np.asarray(current_mask, np.float32).reshape(B, -1)
        new_max = np.maximum(run_max, lc)
        with np.errstate(invalid="ignore"):
            resc = np.exp(run_max - new_max, dtype=np.float32)
        run_sum *= resc
        out *= resc[..., None]
        ex = np.exp(lc - new_max, dtype=np.float32)
        run_sum += ex
        out += ex[..., None] * cv
        run_max = new_max
        cur_logits = lc
    out = out / run_sum[..., None]
    probs = None
    if return_attn:
        parts = [np.exp(lg - run_max[..., None], dtype=np.float32) / run_sum[..., None] for lg in saved]
        if cur_logits is not None:
            parts.append((np.exp(cur_logits - run_max, dtype=np.float32) / run_sum)[..., None])
        probs = (np.concatenate(parts, axis=-1) if parts else np.zeros((B, H, 0), np.float32))[:, :, None, :]
    return out[:, :, None, :].astype(np.float32), probs


# --------------------------------------------------------------------------
# Importance  (smartkv/core/cache.py:216-264, smartkv/core/importance.py:44-101)
# --------------------------------------------------------------------------
class ImportanceState:
    """Cumulative + per-layer EMA importance, and the head-weight EMA."""

    def __init__(self, num_layers: int, decay: float = 0.9, head_decay: float = 0.9):
        self.num_layers = num_layers
        self.decay = decay
        self.head_decay = head_decay                       # cache.py:174
        self.head_importance: Optional[np.ndarray] = None  # fp32 [Hq], starts at ones (cache.py:173,233-235)
        self.token_importance: Dict[int, float] = {}       # cumulative, Python double (importance.py:95-99)
        self.layer_importance: Dict[Tuple[int, int], float] = {}  # EMA (importance.py:85-92)
        self.last_seen: Dict[int, int] = {}
        self.global_step = 0

    def head_weights(self, probs: np.ndarray) -> np.ndarray:
        """Update the head EMA with this call's probabilities and return the
        per-head multipliers (cache.py:242-248)."""
        hq = probs.shape[1]
        if self.head_importance is None or self.head_importance.size != hq:
            self.head_importance = np.ones(hq, np.float32)
        head_mean = probs.astype(np.float32).mean(axis=(0, 2, 3), dtype=np.float32)
        self.head_importance = (self.head_importance * np.float32(self.head_decay)
                                + head_mean * np.float32(1.0 - self.head_decay)).astype(np.float32)
        return (self.head_importance / (self.head_importance.mean(dtype=np.float32) + np.float32(1e-6))).astype(np.float32)

    def update(self, layer: int, probs: np.ndarray, key_ids: Sequence[int]) -> np.ndarray:
        """``SmartKVCache.update_attention`` up to (not including) the
        reallocation trigger.  probs [B,Hq,q,Nkeys]; key_ids are the ids OF THE
        KEYS (cache.py:229-230).  Returns the per-key mass that was added."""
        w = self.head_weights(probs)
        weighted = probs.astype(np.float32) * w.reshape(1, -1, 1, 1)
        key_mass = weighted.sum(axis=(0, 1, 2), dtype=np.float32)
        for i, tid in enumerate(key_ids):
            if i >= key_mass.size:
                break
            s = float(key_mass[i])
            lk = (layer, int(tid))
            if lk not in self.layer_importance:
                self.layer_importance[lk] = s
            else:
                self.layer_importance[lk] = self.decay * self.layer_importance[lk] + (1 - self.decay) * s
            if tid not in self.token_importance:
                self.token_importance[int(tid)] = s
            else:
                self.token_importance[int(tid)] += s
        self.global_step += 1
        for tid in key_ids:
            self.last_seen[int(tid)] = self.global_step
        return key_mass


def allocation_scores(tokens: Iterable[int], importance: Dict[int, float], last_seen: Dict[int, int],
                      global_step: int, protected: Iterable[int] = (0, 1, 2), critical_window: int = 4,
                      recency_temperature: float = 512.0) -> Dict[int, float]:
    """Scores fed to the allocator: importance x recency, +inf for protected
    ids and the first ``critical_window`` positions (cache.py:301-311)."""
    prot = set(protected)
    out = {}
    for t in tokens:
        s = importance.get(t, 0.0)
        if recency_temperature > 0:
            age = global_step - last_seen.get(t, global_step)
            s *= math.exp(-age / recency_temperature)
        if t in prot or t < critical_window:
            s = float("inf")
        out[t] = s
    return out


# --------------------------------------------------------------------------
# Budgeted greedy allocator  (smartkv/core/cache.py:353-601)
# --------------------------------------------------------------------------
class AllocatorConfig:
    def __init__(self, num_heads: int, head_dim: int, memory_budget: float,
                 available_bits: Sequence[int] = (2, 3, 4, 8), scale_dtype: str = "fp32",
                 use_packing: bool = True, utility_alpha: float = 0.5, importance_floor: float = 1e-6,
                 hysteresis_rank_threshold: float = 0.05, hysteresis_intervals: int = 2,
                 high_precision_fraction: float = 0.02, high_precision_boost: float = 1.5,
                 min_high_precision_tokens: int = 0, protected: Iterable[int] = (0, 1, 2),
                 critical_window: int = 4):
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.memory_budget = memory_budget
        self.available_bits = sorted(available_bits)
        self.scale_dtype = scale_dtype
        self.use_packing = use_packing
        self.utility_alpha = float(utility_alpha) if utility_alpha > 0 else 1.0      # cache.py:135
        self.importance_floor = float(max(importance_floor, 0.0))
        self.hysteresis_rank_threshold = float(max(hysteresis_rank_threshold, 0.0))
        self.hysteresis_intervals = max(int(hysteresis_intervals), 1)
        self.high_precision_fraction = float(max(0.0, min(high_precision_fraction, 0.5)))
        self.high_precision_boost = float(max(1.0, high_precision_boost))
        self.min_high_precision_tokens = int(max(0, min_high_precision_tokens))
        self.protected = set(protected)
        self.critical_window = critical_window


def solve_allocation(cfg: AllocatorConfig, tokens: Iterable[int], scores: Dict[int, float],
                     rank_state: Optional[Dict[int, Dict[str, float]]] = None) -> Dict[int, int]:
    """Marginal-gain greedy under a byte budget with rank hysteresis and a
    high-priority pass; a literal restatement of cache.py:353-601.

    ``rank_state`` is the allocator's persistent per-token {pct, streak}
    record (mutated in place, as the reference mutates ``_rank_state``).
    Iteration over ``tokens`` is in ascending id order, which is what CPython
    yields for the reference's ``set`` of dense small ints.
    """
    if rank_state is None:
        rank_state = {}
    toks = sorted(set(tokens))
    asc = list(cfg.available_bits)
    lo_bits, hi_bits = asc[0], asc[-1]

    def is_prot(t):
        return t in cfg.protected or t < cfg.critical_window

    alloc = {t: (hi_bits if is_prot(t) else lo_bits) for t in toks}
    n = len(alloc)
    if n == 0:
        return alloc
    sbits = 32 if cfg.scale_dtype == "fp32" else 16
    elements = 2 * cfg.num_heads * cfg.head_dim
    payload = float(sum(b * elements for b in alloc.values())) if cfg.use_packing else float(n * elements * 8)
    scale_total = float(n * 2 * cfg.num_heads * sbits)
    fp16_total = float(n * elements * 16)

    def ratio(p):
        return (p + scale_total) / fp16_total if fp16_total > 0 else 0.0

    alpha = min(max(cfg.utility_alpha, 0.1), 1.0)

    def util(b):
        return float(b) if alpha == 1.0 else float(math.pow(b, alpha))

    # high-priority set (cache.py:397-420)
    high: set = set()
    if cfg.high_precision_fraction > 0.0 or cfg.min_high_precision_tokens > 0:
        scored = [(t, scores.get(t, 0.0)) for t in toks if not is_prot(t)]
        scored = [(t, s) for t, s in scored if math.isfinite(s) and s > 0.0]
        if scored:
            scored.sort(key=lambda it: it[1], reverse=True)
            want = max(cfg.min_high_precision_tokens, int(math.ceil(len(scored) * cfg.high_precision_fraction)))
            want = min(len(scored), want)
            if want > 0 and cfg.use_packing:
                high = {t for t, _ in scored[:want]}

    # rank percentiles + hysteresis streaks (cache.py:423-450)
    ranked = sorted((t for t in toks if not is_prot(t)), key=lambda t: scores.get(t, 0.0), reverse=True)
    pct_of: Dict[int, float] = {}
    if ranked:
        den = max(len(ranked) - 1, 1)
        for i, t in enumerate(ranked):
            pct = 0.0 if len(ranked) == 1 else i / den
            st = rank_state.get(t)
            if st is None:
                rank_state[t] = {"pct": pct, "streak": cfg.hysteresis_intervals}
            else:
                moved = abs(pct - st.get("pct", pct)) >= cfg.hysteresis_rank_threshold
                streak = min(st.get("streak", 0) + 1, cfg.hysteresis_intervals) if moved else 0
                rank_state[t] = {"pct": pct, "streak": streak}
            pct_of[t] = pct
    for t in toks:
        if t not in pct_of and t not in rank_state:
            rank_state[t] = {"pct": 1.0, "streak": cfg.hysteresis_intervals}

    step_index = {b: i for i, b in enumerate(asc)}
    heap: List[Tuple[float, int, int, int]] = []
    state = {"payload": payload}

    def push(t, cur):
        i = step_index.get(cur)
        if i is None or i >= len(asc) - 1:
            return
        nxt = asc[i + 1]
        imp = scores.get(t, 0.0)
        if not math.isfinite(imp):
            imp = cfg.importance_floor if cfg.importance_floor > 0 else 0.0
        if imp <= 0.0:
            if cfg.importance_floor <= 0.0:
                return
            imp = cfg.importance_floor
        if t in high and nxt >= hi_bits:
            imp *= cfg.high_precision_boost
        st = rank_state.get(t)
        if st is not None and t in pct_of:
            gated = ratio(state["payload"]) >= cfg.memory_budget * 0.85
            if gated and st.get("streak", 0) < cfg.hysteresis_intervals:
                return
        gain = util(nxt) - util(cur)
        if gain <= 0.0 or nxt - cur <= 0:
            return
        heapq.heappush(heap, (-((imp * gain) / (nxt - cur)), t, cur, nxt))

    for t in alloc:
        if alloc[t] < hi_bits:
            push(t, alloc[t])

    tol = 1e-6
    while heap:
        _neg, t, expect, nxt = heapq.heappop(heap)
        cur = alloc.get(t, lo_bits)
        if cur != expect:
            continue
        delta = float((nxt - cur) * elements) if cfg.use_packing else 0.0
        cand = ratio(state["payload"] + delta)
        if cand > cfg.memory_budget + tol:
            continue
        alloc[t] = nxt
        state["payload"] += delta
        st = rank_state.get(t)
        if st is not None:
            st["streak"] = 0
            st["pct"] = pct_of.get(t, st.get("pct", 1.0))
        push(t, nxt)
        if cand >= cfg.memory_budget + tol:
            break

    # high-priority post-pass (cache.py:522-591)
    if high and cfg.use_packing:
        for t in sorted(high, key=lambda x: scores.get(x, 0.0), reverse=True):
            cur = alloc.get(t, lo_bits)
            if cur >= hi_bits:
                continue
            delta = float((hi_bits - cur) * elements)
            cand = ratio(state["payload"] + delta)
            if cand > cfg.memory_budget + tol:
                victims = sorted((c for c in alloc if c not in cfg.protected and c not in high and c != t
                                  and alloc.get(c, lo_bits) > lo_bits),
                                 key=lambda c: scores.get(c, float("inf")))
                undone = []
                for c in victims:
                    cb = alloc[c]
                    ci = step_index.get(cb)
                    if ci is None or ci <= 0:
                        continue
                    pb = asc[ci - 1]
                    give = float((cb - pb) * elements)
                    alloc[c] = pb
                    state["payload"] -= give
                    undone.append((c, cb, give))
                    cand = ratio(state["payload"] + delta)
                    if cand <= cfg.memory_budget + tol:
                        break
                if cand > cfg.memory_budget + tol:
                    for c, cb, give in reversed(undone):
                        alloc[c] = cb
                        state["payload"] += give
                    continue
                for c, _cb, _g in undone:
                    st = rank_state.get(c)
                    if st is not None:
                        st["streak"] = 0
                        st["pct"] = pct_of.get(c, st.get("pct", 1.0))
            alloc[t] = hi_bits
            state["payload"] += delta
            st = rank_state.get(t)
            if st is not None:
                st["streak"] = 0
                st["pct"] = pct_of.get(t, st.get("pct", 1.0))
    return alloc


# --------------------------------------------------------------------------
# Requantisation on reallocation  (smartkv/core/cache.py:819-844)
# --------------------------------------------------------------------------
def requantize_rows(codes: np.ndarray, scale: np.ndarray, new_bits: int):
    """Dequantise the stored codes (code*scale, fp32) and quantise the result
    at the new width -- NOT a re-quantisation of the original values."""
    return quantize_rows(dequantize_rows(codes, scale), new_bits)


# --------------------------------------------------------------------------
# Seeded synthetic inputs shared by tests, smoke and bench
# --------------------------------------------------------------------------
def synth_kv(n_tokens: int, num_kv_heads: int, head_dim: int, seed: int, n_outlier: int = 4,
             outlier_scale: float = 8.0) -> Tuple[np.ndarray, np.ndarray]:
    """K, V ~ N(0,1) fp32 [N,Hkv,D] with ``n_outlier`` fixed channels per head scaled up."""
    rng = np.random.default_rng(seed)
    k = rng.standard_normal((n_tokens, num_kv_heads, head_dim), dtype=np.float32)
    v = rng.standard_normal((n_tokens, num_kv_heads, head_dim), dtype=np.float32)
    for h in range(num_kv_heads):
        ch = rng.choice(head_dim, size=n_outlier, replace=False)
        k[:, h, ch] *= np.float32(outlier_scale)
        ch = rng.choice(head_dim, size=n_outlier, replace=False)
        v[:, h, ch] *= np.float32(outlier_scale)
    return k, v


def synth_importance(n_tokens: int, seed: int, zipf_s: float = 1.1, n_sinks: int = 4,
                     n_heavy: int = 0) -> np.ndarray:
    """Zipf(s) mass over positions (rank -> position by a seeded permutation);
    the first ``n_sinks`` positions take the top ranks; ``n_heavy`` extra
    positions get sink-sized mass.  fp32, sums to 1."""
    rng = np.random.default_rng(seed + 7919)
    mass = 1.0 / np.arange(1, n_tokens + 1, dtype=np.float64) ** zipf_s
    order = rng.permutation(n_tokens)
    order = np.concatenate([np.arange(min(n_sinks, n_tokens)), order[order >= n_sinks]])
    imp = np.empty(n_tokens, np.float64)
    imp[order] = mass
    if n_heavy > 0 and n_tokens > n_sinks:
        heavy = rng.choice(np.arange(n_sinks, n_tokens), size=min(n_heavy, n_tokens - n_sinks), replace=False)
        imp[heavy] = mass[min(n_sinks, n_tokens - 1)]
    imp /= imp.sum()
    return imp.astype(np.float32)
