"""Benchmark of the packed-KV decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 1|3|4]

One *step* = one decode step of the Llama-3.1-8B attention shape (32 query heads,
8 KV heads, head_dim 128, fp16 query) over 32 layers, batch 16, KV context 8192:
per layer the fused packed decode attention (+ current fp token, LSE combine),
the importance update and the quantize-pack append of the new token.  K/V are
seeded synthetic N(0,1) with 4 outlier channels per head scaled x8; tokens are stored at
the default 4 bits, a Zipf(1.1) importance is injected and the device allocator +
requantise/repack bring the cache to memory_budget 0.35 (stand-ins for the reference's
benchmark inputs, which are synthetic randn as well).  Every 16th step of the timed
region ends with a full reallocation (allocator, repack of all layers); two untimed
reallocation cycles run first, so that the timed ones see a settled cache.

metric  = packed-KV bytes streamed per second (algorithmic bytes: sum over buckets of
          n_b * Hkv * 2 * (row_bytes + 4) per sequence and layer) over the whole step.
value   = inputs resident in HBM; e2e = the same step driven with HOST buffers
          (queries / new K,V copied in from pinned memory and outputs copied back, layer by
          layer on two copy streams inside the step's CUDA graph).
roofline= the attention kernel alone (CUDA events around one back-to-back launch per layer)
          against the measured HBM copy bandwidth in MEASURED_PEAKS.json.
Under torchrun the configuration is split over the ranks (strong scaling): KV heads for
--config 1 and 4, the tokens of the sequence for --config 3; --replicas keeps the whole
configuration on every rank instead.  Timing is barrier + device events, max over ranks.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# The shapes the metric is quoted on.  1 is the bench line; 3 and 4 are the other GPU-sized shapes (--config).
CONFIGS = {
    1: dict(name="Llama-3.1-8B attention shape", num_layers=32, num_q_heads=32, num_kv_heads=8, head_dim=128, batch=16,
            context=8192, memory_budget=0.35, available_bits=(2, 3, 4, 8), zipf_s=1.1, realloc_every=16, shard="kv_heads"),
    3: dict(name="Llama-3.1-8B attention shape, long context", num_layers=32, num_q_heads=32, num_kv_heads=8, head_dim=128,
            batch=1, context=131072, memory_budget=0.25, available_bits=(2, 3, 4, 8), zipf_s=1.2, heavy_hitters=64,
            realloc_every=16, shard="sequence"),
    4: dict(name="Llama-3.1-70B attention shape", num_layers=80, num_q_heads=64, num_kv_heads=8, head_dim=128, batch=64,
            context=16384, memory_budget=0.35, available_bits=(2, 3, 4, 8), zipf_s=1.1, realloc_every=16, shard="kv_heads"),
}
CFG = CONFIGS[1]
FALLBACK_HBM_GBS = 6650.0
# staging of the graphed reallocation: 4 GiB lets one pair of row-move launches cover 14 of the 32 layers
REALLOC_STAGING_BYTES = 4 << 30


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def zipf_importance(n, seed, s, heavy_hitters=0):
    """Zipf(s) mass over positions, rank -> position by a seeded permutation, first 4 = sinks; optionally
    `heavy_hitters` randomly placed tokens carrying the mass of the top ranks after the sinks."""
    rng = np.random.default_rng(seed + 7919)
    mass = 1.0 / np.arange(1, n + 1, dtype=np.float64) ** s
    order = rng.permutation(n)
    order = np.concatenate([np.arange(4), order[order >= 4]])
    imp = np.empty(n)
    imp[order] = mass
    if heavy_hitters:
        hh = rng.choice(np.arange(4, n), size=heavy_hitters, replace=False)
        imp[hh] = np.maximum(imp[hh], mass[4])
    return (imp / imp.sum()).astype(np.float32)


class ClockSampler:
    """Reads SM clock and throttle reasons through NVML (read-only) every ~2 ms in a thread beside
    the timed region; falls back to one nvidia-smi query if NVML is not importable."""
    REASONS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20),
               ("sw_power_cap", 0x4))

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.samples = []
        self.mask = 0
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None

    def _loop(self):
        nv, h = self._nvml, self._handle
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                self.mask |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(h))
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = self.gpu
            if visible:
                ids = [v for v in visible.split(",") if v.strip()]
                if self.gpu < len(ids) and ids[self.gpu].strip().isdigit():
                    idx = int(ids[self.gpu])
            self._handle = nv.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(self._handle, nv.NVML_CLOCK_SM))
            self._nvml = nv
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        except Exception:
            self._nvml = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self._nvml is not None:
            self._stop.set()
            self._thread.join(timeout=2)
            if self.samples:
                out["sm_mhz"] = float(np.median(self.samples))
                out["sm_max_mhz"] = self.max_mhz
                out["samples"] = len(self.samples)
                out["reasons"] = [nm for nm, bit in self.REASONS if self.mask & bit]
            return out
        try:
            q = "clocks.sm,clocks.max.sm,clocks_event_reasons.active"
            r = subprocess.run(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={q}", "--format=csv,noheader,nounits"],
                               capture_output=True, text=True, timeout=10).stdout.strip().split(",")
            out.update(sm_mhz=float(r[0]), sm_max_mhz=float(r[1]), samples=1)
        except Exception:
            pass
        return out


def workload_string(cfg):
    return (f"{cfg['name']} ({cfg['num_q_heads']} query heads, {cfg['num_kv_heads']} KV heads, head_dim {cfg['head_dim']}), "
            f"{cfg['num_layers']} layers, batch {cfg['batch']}, context {cfg['context']}, budget {cfg['memory_budget']}, "
            "bits [2,3,4,8], fp16 query; one decode step per step")


def algorithmic_bytes_per_layer(counts, cfg):
    """sum_b n_b * Hkv * 2 * (row_bytes + 4); counts int array [B, 4]."""
    D, H = cfg["head_dim"], cfg["num_kv_heads"]
    per_tok = np.array([H * 2 * (D * w // 8 + 4) for w in (2, 3, 4, 8)], np.int64)
    return int((np.asarray(counts, np.int64) * per_tok).sum())


# ----------------------------------------------------------------------------- end-to-end generation (--config 2)
GENERATION = dict(name="random-init TinyLlama-1.1B", num_layers=22, hidden=2048, intermediate=5632, num_q_heads=32,
                  num_kv_heads=4, head_dim=64, vocab=32000, batch=8, prompt=512, decode=256, memory_budget=0.5,
                  available_bits=(2, 3, 4, 8), realloc_freq=16)


def generation_workload_string(g):
    return (f"{g['name']} ({g['num_layers']} layers, hidden {g['hidden']}, {g['num_q_heads']} query / {g['num_kv_heads']} KV "
            f"heads, vocab {g['vocab']}, weights N(0, 0.02)), batch {g['batch']}, prompt {g['prompt']} uniform-random ids, "
            f"{g['decode']} greedy decode tokens, budget {g['memory_budget']}, bits [2,3,4,8]; one step = one decode token "
            "per sequence through the LlamaSmartKV wrapper")


def build_generation_model(g, device, dtype, seed=0):
    import torch
    import transformers
    cfg = transformers.LlamaConfig(vocab_size=g["vocab"], hidden_size=g["hidden"], intermediate_size=g["intermediate"],
                                   num_hidden_layers=g["num_layers"], num_attention_heads=g["num_q_heads"],
                                   num_key_value_heads=g["num_kv_heads"], max_position_embeddings=2048, rms_norm_eps=1e-5,
                                   tie_word_embeddings=False, bos_token_id=1, eos_token_id=2, pad_token_id=None)
    cfg._attn_implementation = "eager"
    with torch.device("meta"):
        model = transformers.LlamaForCausalLM(cfg)
    model = model.to_empty(device=device).to(dtype).eval()
    gen = torch.Generator(device=device).manual_seed(seed)
    with torch.no_grad():
        for _name, p_ in sorted(model.named_parameters(), key=lambda kv: kv[0]):
            if p_.dim() >= 2:
                p_.copy_(torch.empty(p_.shape, dtype=torch.float32, device=device).normal_(0.0, 0.02, generator=gen))
            else:
                p_.fill_(1.0)
        # buffers created on the meta device (rotary inverse frequencies) need their values back
        for m in model.modules():
            if hasattr(m, "inv_freq") and hasattr(m, "rope_init_fn"):
                inv, _ = m.rope_init_fn(m.config, device)
                m.inv_freq = inv
                m.original_inv_freq = inv
    return model


def run_generation(args):
    """End-to-end generation (the TinyLlama-1.1B workload) through the public wrapper: prompt prefill, then greedy decoding with every
    batch row an independent sequence of one multi-sequence cache.  value = decode tokens per second over the
    whole batch (device events around all decode steps; the greedy token of every step is read back to the
    host inside the timed region, as a generation loop does)."""
    import torch
    from smartkv_b200 import LlamaSmartKV, SmartKVConfig
    g = dict(GENERATION)
    if args.batch:
        g["batch"] = args.batch
    if args.layers:
        g["num_layers"] = args.layers
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    model = build_generation_model(g, dev, torch.float16)
    w = LlamaSmartKV(model, SmartKVConfig(enabled=True, memory_budget=g["memory_budget"], realloc_freq=g["realloc_freq"],
                                          available_bits=list(g["available_bits"]), device=str(dev), batched=True,
                                          max_tokens=g["prompt"] + g["decode"] + 8))
    B, n, T = g["batch"], g["prompt"], g["decode"]
    ids = torch.randint(3, g["vocab"], (B, n), generator=torch.Generator().manual_seed(1)).to(dev)
    pos = torch.arange(n, device=dev)[None].expand(B, -1)
    from smartkv_b200.models.graphed_decode import GraphedDecoder
    decoder = None if args.no_graph else GraphedDecoder.for_model(w)
    sampler = ClockSampler(dev.index or 0)
    e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    results = []
    for rep in range(2):                 # the first pass warms every kernel, allocation and graph; the second is timed
        w.reset_cache()
        torch.cuda.synchronize(dev)
        if rep == 1:
            sampler.start()
        with torch.no_grad():
            e[0].record()
            out = w(input_ids=ids, position_ids=pos, use_cache=False)
            tok = out.logits[:, -1].argmax(-1)
            e[1].record()
            toks = []
            if decoder is not None:
                decoder.reset()
            for t in range(T):
                toks.append(tok.tolist())       # the host sees every token, as a generation loop does
                if decoder is not None:
                    tok = decoder.step(tok, n + t).argmax(-1)
                else:
                    out = w(input_ids=tok[:, None], position_ids=torch.full((B, 1), n + t, device=dev), use_cache=False)
                    tok = out.logits[:, -1].argmax(-1)
            e[2].record()
        torch.cuda.synchronize(dev)
        results.append((e[0].elapsed_time(e[1]), e[1].elapsed_time(e[2])))
    clocks = sampler.stop()
    w.smartkv_cache.check_errors()
    stats = w.get_smartkv_stats()
    prefill_ms, decode_ms = results[-1]
    line = {
        "metric": "decode_tokens_per_s", "value": round(B * T / (decode_ms / 1e3), 2), "unit": "tokens/s", "n_gpus": 1,
        "steps": T, "warmup": T, "ms_per_step": round(decode_ms / T, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic (random-init weights, uniform-random prompt ids)",
        "config": {"workload": generation_workload_string(g)},
        "prefill_ms": round(prefill_ms, 2), "prefill_tokens_per_s": round(B * n / (prefill_ms / 1e3), 1),
        "reallocations": stats.get("realloc_count"), "memory_ratio_true_max": round(stats.get("memory_ratio_true_max", 0.0), 4),
        "precision_distribution": stats.get("precision_distribution"), "clocks": clocks,
        "launches_per_layer_per_step": 2,
        "decode_steps_as_cuda_graphs": None if decoder is None else {"graphs_captured": decoder.graphs_captured},
        "generated_tokens_first_sequence": [int(x[0]) for x in toks[:8]],
    }
    print(json.dumps(line))


def run_generation_reference(args):
    """The reference's own wrapper on the host cores (fp32: its CPU path has no fp16 matmul), one sequence, a
    bounded sample: the full prompt, then --decode-sample greedy steps.  Needs the reference package on
    PYTHONPATH; it is not part of this repository."""
    import torch
    g = dict(GENERATION)
    if args.layers:
        g["num_layers"] = args.layers
    try:
        import smartkv.models.llama_smartkv as rl
        from transformers.models.llama.modeling_llama import apply_rotary_pos_emb as hf_rope
    except Exception as ex:                      # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"the reference package is not importable here ({type(ex).__name__}); "
                          "its CPU wrapper can only be timed where a checkout of the reference is on PYTHONPATH"}))
        return
    rl.apply_rotary_pos_emb = lambda q, k, c, s, p=None: hf_rope(q, k, c, s)    # the installed transformers takes 4 arguments
    model = build_generation_model(g, torch.device("cpu"), torch.float32)
    w = rl.LlamaSmartKV(model, rl.SmartKVConfig(enabled=True, memory_budget=g["memory_budget"], realloc_freq=g["realloc_freq"],
                                                device="cpu"))
    w.set_use_fused_cpu(True)
    n, T = g["prompt"], args.decode_sample
    ids = torch.randint(3, g["vocab"], (1, n), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        t0 = time.perf_counter()
        out = w(input_ids=ids, position_ids=torch.arange(n)[None], use_cache=False)
        tok = out.logits[:, -1].argmax(-1)
        t1 = time.perf_counter()
        for t in range(T):
            out = w(input_ids=tok[:, None], position_ids=torch.tensor([[n + t]]),
                    attention_mask=torch.zeros(1, 1, 1, n + t + 1), use_cache=False)
            tok = out.logits[:, -1].argmax(-1)
        t2 = time.perf_counter()
    per_tok = (t2 - t1) / T
    line = {"impl": "reference", "metric": "decode_tokens_per_s", "value": round(1.0 / per_tok, 3), "unit": "tokens/s",
            "n_gpus": 1, "steps": T, "warmup": 0, "ms_per_step": round(per_tok * 1e3, 2), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic (random-init weights, uniform-random prompt ids)",
            "config": {"workload": generation_workload_string(g),
                       "sample": f"one sequence (the reference's cache holds one), prompt {n}, {T} decode steps on {torch.get_num_threads()} threads"},
            "prefill_ms": round((t1 - t0) * 1e3, 1),
            "cpu_baseline": {"value": round(1.0 / per_tok, 3), "unit": "tokens/s", "cores": torch.get_num_threads(),
                             "kind": "reference", "sample": f"prompt {n} + {T} decode steps, one sequence"}}
    print(json.dumps(line))


# ----------------------------------------------------------------------------- our arm
def profile_traffic(kernel_name):
    """DRAM bytes per launch of `kernel_name` on the config-1 shape as the committed ncu summary states them
    (a line `traffic_bytes_per_launch: N`); None if there is no such summary."""
    import glob
    import re
    for path in sorted(glob.glob(os.path.join(ROOT, "profiles", f"{kernel_name}_*.md"))):
        m = re.search(r"traffic_bytes_per_launch:\s*(\d+)", open(path).read())
        if m:
            return int(m.group(1)), os.path.relpath(path, ROOT)
    return None, None


def run_ours(args):
    import torch
    import ctypes

    import torch.distributed as dist

    from smartkv_b200 import _lib as skv_lib
    from smartkv_b200.sharding import ImportanceSync, fold_partials, shard_kv_heads, shard_tokens
    from smartkv_b200.store import PackedKVStore, bucket_capacities

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = dict(CONFIGS[args.config])
    if args.layers:
        cfg["num_layers"] = args.layers      # profiler captures only: fewer layers = less device memory
    # other shapes with the same kernels and settings; not the contract's workload
    if args.batch:
        cfg["batch"] = args.batch
    if args.context:
        cfg["context"] = args.context
    if args.budget:
        cfg["memory_budget"] = args.budget
    shard = "replicas" if args.replicas else cfg["shard"]
    L, Hq, Hkv, D, B, N = (cfg[k] for k in ("num_layers", "num_q_heads", "num_kv_heads", "head_dim", "batch", "context"))
    # ---- what this rank holds ------------------------------------------------------------------------------
    if shard == "kv_heads" and world > 1:
        heads = shard_kv_heads(Hkv, world, rank)            # strong scaling: the same cache split over the GPUs
        Hkv_r, Hq_r, N_r, tok0 = len(heads), Hq // world, N, 0
    elif shard == "sequence" and world > 1:
        own = shard_tokens(N, world, rank)                  # strong scaling: the same sequence split over the GPUs
        Hkv_r, Hq_r, N_r, tok0 = Hkv, Hq, len(own), own.start
    else:
        Hkv_r, Hq_r, N_r, tok0 = Hkv, Hq, N, 0
    seq_mode = shard == "sequence" and world > 1
    steps, warmup = args.steps, args.warmup
    realloc_every = cfg["realloc_every"]
    settle = 0 if (seq_mode or args.no_settle) else 2       # reallocation cycles run before anything is timed
    total_steps = steps * 3 + warmup * 2 + settle * realloc_every + 16 + 32     # + the launch-mode autotune's replays
    caps = bucket_capacities(N_r + total_steps, cfg["memory_budget"], D, cfg["available_bits"])
    store = PackedKVStore(L, B, Hkv_r, D, Hq_r, caps, device=dev, track_importance=not seq_mode)
    store.token_capacity = N_r + total_steps     # what the buckets were sized for: bounds the importance grid under capture

    # ---- populate the cache: seeded synthetic K/V stored at the default 4 bits (cache.py:1214), the
    # Zipf importance injected the way the reference's kernel benchmark does, then one reallocation
    bits0 = torch.full((B, N_r), 4, dtype=torch.int64, device=dev)
    dst = store.plan_bulk(bits0)
    gen = torch.Generator(device=dev)
    chan = torch.Generator(device="cpu").manual_seed(1234)
    out_k = torch.stack([torch.randperm(D, generator=chan)[:4] for _ in range(Hkv_r)]).to(dev)
    out_v = torch.stack([torch.randperm(D, generator=chan)[:4] for _ in range(Hkv_r)]).to(dev)
    hidx = torch.arange(Hkv_r, device=dev)[:, None]
    chunk_b = max(1, min(B, (1 << 21) // max(N_r, 1)))      # bounded staging for the big shapes
    for layer in range(L):
        gen.manual_seed(rank * 100003 + 1000 * layer)
        for b0 in range(0, B, chunk_b):
            nb = min(chunk_b, B - b0)
            k = torch.randn((nb * N_r, Hkv_r, D), generator=gen, device=dev, dtype=torch.float32)
            v = torch.randn((nb * N_r, Hkv_r, D), generator=gen, device=dev, dtype=torch.float32)
            k[:, hidx, out_k] *= 8.0
            v[:, hidx, out_v] *= 8.0
            sl = slice(b0 * N_r, (b0 + nb) * N_r)
            store.append(layer, k, v, dst[0][sl], dst[1][sl], dst[2][sl])
            del k, v
    imp = np.stack([zipf_importance(N, b, cfg["zipf_s"], cfg.get("heavy_hitters", 0)) for b in range(B)])[:, tok0: tok0 + N_r]
    store.cumulative.zero_()
    store.cumulative.scatter_(1, dst[3].view(B, N_r).long(), torch.from_numpy(imp.astype(np.float64)).to(dev))
    alloc_cfg = store.make_alloc_config(cfg["memory_budget"], cfg["available_bits"], total_kv_heads=Hkv)
    importance_sync = ImportanceSync(store, dist if (world > 1 and shard == "kv_heads") else None)
    if world > 1:
        # first use of the communicator (connection set-up) happens here, not inside the timed region
        # (with a buffer of the size the importance sync exchanges: the first all-reduce of a size costs ms)
        warm = torch.zeros_like(store.cumulative)
        dist.all_reduce(warm)
        dist.all_reduce(warm)
        torch.cuda.synchronize()

    sync_events = []

    def reallocate():
        importance_sync()              # KV-head shards: sum the per-shard importance first (no-op on 1 GPU)
        if world > 1 and shard == "kv_heads":      # when the all-reduce was through (it waits for the slowest rank)
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            sync_events.append(e)
        if args.no_graph:
            store.reallocate(alloc_cfg)
        else:
            store.reallocate_graphed(alloc_cfg, staging_budget=REALLOC_STAGING_BYTES)
        importance_sync.after_repack()

    reallocate()
    torch.cuda.synchronize()
    store.check_errors()
    realloc_chunks = -(-L // max(1, min(L, ((1 << 30) if args.no_graph else REALLOC_STAGING_BYTES) // max(1, int(store.lib.skv_requant_staging_bytes(
        ctypes.byref(store.desc), store.appended_total if args.no_graph else store.num_seqs * store.slots, 1))))))
    realloc_launches = 15 + (3 if B > 1 else 0) + 2 * realloc_chunks

    # ---- per-step inputs (resident) -----------------------------------------------------------
    gen.manual_seed(rank + 99)
    n_in = 4  # distinct input sets cycled through (each is small; the cache is what is streamed)
    q_dev = torch.randn((n_in, L, B, Hq_r, D), generator=gen, device=dev, dtype=torch.float32).half()
    k_dev = torch.randn((n_in, L, B, Hkv_r, D), generator=gen, device=dev, dtype=torch.float32).half()
    v_dev = torch.randn((n_in, L, B, Hkv_r, D), generator=gen, device=dev, dtype=torch.float32).half()
    if seq_mode:   # every rank sees the same queries and the same new token
        for t in (q_dev, k_dev, v_dev):
            dist.broadcast(t, 0)
    out_dev = torch.empty((L, B, Hq_r, D), dtype=torch.float32, device=dev)

    # ---- sequence shards check themselves: layer 0 of the populated cache, no new token.  Every rank's (max, sum, out)
    # over its token range is gathered and folded; rank 0 also gets every rank's stored rows of that layer (codes,
    # scales, widths), puts them into ONE store and attends over it; the two must agree at the attention tolerance.
    self_check = None
    if seq_mode:
        from smartkv_b200.store import round_up as _round_up
        qc = q_dev[0, 0].contiguous()
        o = store.attention(0, qc).clone()
        part = torch.cat([store.lse_max[..., None], store.lse_sum[..., None], o * store.lse_sum[..., None]], -1).contiguous()
        parts = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(parts, part)
        folded_chk = fold_partials(torch.stack(parts))
        rows = [store.export_sequence(0, b) for b in range(B)]
        mine = [torch.stack([r[i] for r in rows]).contiguous() for i in range(1, 6)]     # bits, k codes, v codes, k scale, v scale
        everyone = []
        for t in mine:
            g_ = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(g_, t)
            everyone.append(torch.cat(g_, dim=1))                                          # ranks hold consecutive token ranges
        if rank == 0:
            bits_f, kc_f, vc_f, ks_f, vs_f = everyone
            cap = _round_up(N + 1, 128)
            whole = PackedKVStore(1, B, Hkv_r, D, Hq_r, (cap, cap, cap, cap), device=dev, track_importance=False)
            dw = whole.plan_bulk(bits_f.long())
            skv_lib.check(whole.lib.skv_import_rows(ctypes.byref(whole.desc), skv_lib.ptr(whole.arena), 0, B * N, skv_lib.ptr(dw[0]),
                                                    skv_lib.ptr(dw[1]), skv_lib.ptr(dw[2]), skv_lib.ptr(kc_f.reshape(B * N, Hkv_r, D).contiguous()),
                                                    skv_lib.ptr(vc_f.reshape(B * N, Hkv_r, D).contiguous()),
                                                    skv_lib.ptr(ks_f.reshape(B * N, Hkv_r).contiguous()),
                                                    skv_lib.ptr(vs_f.reshape(B * N, Hkv_r).contiguous()), skv_lib.ptr(whole.err),
                                                    whole._stream()), "skv_import_rows")
            ref = whole.attention(0, qc)
            whole.check_errors()
            err = (folded_chk - ref).abs()
            tol = 2e-3 + 1e-3 * ref.abs()
            self_check = {"what": "layer 0: folded partials of the shards against one store holding every shard's rows",
                          "max_abs_err": float(err.max()), "within_tolerance": bool((err <= tol).all())}
            del whole, ref
        del everyone, mine, rows
        torch.cuda.empty_cache()
    q_host = q_dev.cpu().pin_memory()
    k_host = k_dev.cpu().pin_memory()
    v_host = v_dev.cpu().pin_memory()
    out_host = torch.empty((L, B, Hq_r, D), dtype=torch.float32).pin_memory()
    q_stage = torch.empty_like(q_dev[0])
    k_stage = torch.empty_like(k_dev[0])
    v_stage = torch.empty_like(v_dev[0])

    # ---- which attention kernel: both timed on the live cache (the choice depends on the bucket mix) ----------
    tune = None
    if args.attn_kernel == "auto":
        tune = store.autotune_attention(q_dev[0][0], layers=min(L, 4))
        if world > 1:   # all ranks run the same kernel: the slowest rank's preference decides nothing, rank 0's does
            flag = torch.tensor([skv_lib.lib().skv_get_attention_path()], device=dev)
            dist.broadcast(flag, 0)
            skv_lib.lib().skv_set_attention_path(int(flag.item()))
            store._plan_valid = False
    else:
        skv_lib.lib().skv_set_attention_path(2 if args.attn_kernel == "tensor_memory" else 1)
        store._plan_valid = False
    kernel_name = "decode_attn_tc_kernel" if skv_lib.lib().skv_get_attention_path() == 2 else "decode_attn_kernel"

    attn_events = []
    launches = [0]
    last_rank = rank == world - 1

    def decode_step(q, k, v, record=False):
        """One decode step: 2 kernels of this library per layer (attention; combine + append + the
        previous layer's importance update), the attention plan kernel, the last layer's importance update and
        the two kernels that place and commit the new token.  Sequence shards: the new token takes part (and is
        appended) on the last rank only, importance tracking is off."""
        plan = store.plan_step()
        with_cur = last_rank or not seq_mode
        for layer in range(L):
            ev = None
            if record:
                ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                attn_events.append(ev)
            store.decode_layer(layer, q[layer], k[layer] if with_cur else None, v[layer] if with_cur else None, plan,
                               update_importance=not seq_mode, out=out_dev[layer], kernel_events=ev)
        if with_cur:
            store.commit_step(plan)
        else:
            store.flush_importance()
            store._pipe["calls"] = 0

    # sequence shards: one exchange per step for all layers' (max, sum, out) and one fold
    if seq_mode:
        packed = torch.empty((L, B, Hq_r, D + 2), dtype=torch.float32, device=dev)
        gathered = torch.empty((world,) + tuple(packed.shape), dtype=torch.float32, device=dev)
        folded = torch.empty((L, B, Hq_r, D), dtype=torch.float32, device=dev)

        def exchange():
            sm = store._pipe["small"]
            packed[..., 0] = sm["lse_max"]
            packed[..., 1] = sm["lse_sum"]
            torch.mul(out_dev, sm["lse_sum"].unsqueeze(-1), out=packed[..., 2:])
            dist.all_gather_into_tensor(gathered, packed)
            fold_partials(gathered, out=folded)
    else:
        def exchange():
            pass

    per_step_launches = 2 * L + 4
    graph = None
    # Which kernels are launched as programmatic dependents is chosen by measurement, like the attention kernel itself:
    # the attention kernel alone (2) wins on large shards, attention + post-attention (1) on small ones.
    pdl_choice = None
    if not args.no_graph and not args.no_dependent_launch and args.dependent_launch_mode < 0:
        trial = {}
        for mode in (2, 1):
            skv_lib.lib().skv_set_dependent_launch(mode)
            decode_step(q_dev[0], k_dev[0], v_dev[0])
            torch.cuda.synchronize()
            gt = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gt):
                decode_step(q_dev[0], k_dev[0], v_dev[0])
            for _ in range(3):
                gt.replay()
            ea, eb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            ea.record()
            for _ in range(8):
                gt.replay()
            eb.record()
            torch.cuda.synchronize()
            t = torch.tensor([ea.elapsed_time(eb) / 8], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            trial[mode] = float(t.item())
            del gt
        best = min(trial, key=trial.get)
        skv_lib.lib().skv_set_dependent_launch(best)
        pdl_choice = {"selected": {1: "attention and post-attention kernels", 2: "attention kernel only"}[best],
                      "ms_per_step": {("attention+post" if m == 1 else "attention"): round(v, 4) for m, v in trial.items()}}
    if not args.no_graph:
        # the whole step (every layer's launches) as one CUDA graph over static input buffers
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            q_stage.copy_(q_dev[0]); k_stage.copy_(k_dev[0]); v_stage.copy_(v_dev[0])
            decode_step(q_stage, k_stage, v_stage)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            decode_step(q_stage, k_stage, v_stage)
        # resident inputs: one graph per input set reads the set where it lies in HBM
        resident_graphs = []
        for j in range(n_in):
            gj = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gj):
                decode_step(q_dev[j], k_dev[j], v_dev[j])
            resident_graphs.append(gj)

    def run_step():
        if graph is not None:
            graph.replay()
        else:
            decode_step(q_stage, k_stage, v_stage)
        exchange()
        launches[0] += per_step_launches

    def resident_step(i):
        j = i % n_in
        if graph is not None:
            resident_graphs[j].replay()
        else:
            decode_step(q_dev[j], k_dev[j], v_dev[j])
        exchange()
        launches[0] += per_step_launches

    def kernel_timing_step(i):
        j = i % n_in
        decode_step(q_dev[j], k_dev[j], v_dev[j], record=True)

    # end to end: the step's inputs come from pinned host memory and its outputs go back there.  Inside the step
    # the copies are pipelined by layer on two copy streams (layer l+1's inputs arrive while layer l computes,
    # layer l's output leaves while layer l+1 computes); one CUDA graph per input set holds copies and kernels.
    e2e_graphs = []
    if graph is not None and not seq_mode:
        h2d, d2h = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

        def e2e_body(j):
            main = torch.cuda.current_stream(dev)
            h2d.wait_stream(main)
            d2h.wait_stream(main)
            plan = store.plan_step()
            arrived = []
            for layer in range(L):
                with torch.cuda.stream(h2d):
                    q_stage[layer].copy_(q_host[j][layer], non_blocking=True)
                    k_stage[layer].copy_(k_host[j][layer], non_blocking=True)
                    v_stage[layer].copy_(v_host[j][layer], non_blocking=True)
                    ev_in = torch.cuda.Event()
                    ev_in.record(h2d)
                arrived.append(ev_in)
            main.wait_event(arrived[0])
            for layer in range(L):
                # the wait for the NEXT layer's inputs sits between this layer's two launches, so that the next attention
                # kernel directly follows this layer's post-attention kernel (and can be launched as its dependent)
                nxt = (lambda ev=arrived[layer + 1]: main.wait_event(ev)) if layer + 1 < L else None
                store.decode_layer(layer, q_stage[layer], k_stage[layer], v_stage[layer], plan,
                                   update_importance=True, out=out_dev[layer], before_post=nxt)
                ev_out = torch.cuda.Event()
                ev_out.record(main)
                with torch.cuda.stream(d2h):
                    d2h.wait_event(ev_out)
                    out_host[layer].copy_(out_dev[layer], non_blocking=True)
            store.commit_step(plan)
            main.wait_stream(h2d)
            main.wait_stream(d2h)

        for j in range(n_in):
            gj = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gj):
                e2e_body(j)
            e2e_graphs.append(gj)

    def host_step(i):
        j = i % n_in
        if e2e_graphs:
            e2e_graphs[j].replay()
            launches[0] += per_step_launches
            return
        q_stage.copy_(q_host[j], non_blocking=True)
        k_stage.copy_(k_host[j], non_blocking=True)
        v_stage.copy_(v_host[j], non_blocking=True)
        run_step()
        out_host.copy_(folded if seq_mode else out_dev, non_blocking=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with_realloc = not seq_mode
    # Reallocation cycles before anything is timed: the first reallocations of a cache's life move most tokens
    # (the decode attention over random K/V is nearly uniform and swamps the injected importance), later ones a few
    # per cent.  Both timed passes then see the settled cache and do the same work.
    for c in range(settle):
        for i in range(realloc_every):
            resident_step(i)
        reallocate()
    torch.cuda.synchronize()
    store.check_errors()
    counts0 = store.counts.cpu().numpy()
    hist = counts0.sum(0).tolist()

    realloc_events = []
    moved_log = torch.zeros(256, dtype=torch.int64, device=dev)  # tokens moved by every timed reallocation
    rank_ms = {}

    def timed(fn, n_warm, n_steps, first, realloc=True):
        for i in range(n_warm):
            fn(first + i)
        barrier()
        c_before = store.counts.cpu().numpy()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for i in range(n_steps):
            fn(first + n_warm + i)
            if realloc and with_realloc and (i + 1) % realloc_every == 0:
                ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                ev[0].record()
                reallocate()
                ev[1].record()
                if len(realloc_events) < moved_log.numel():
                    moved_log[len(realloc_events)].copy_(store._realloc["n_moves"].sum())
                realloc_events.append(ev)
                launches[0] += realloc_launches
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        clocks = sampler.stop() if rank == 0 else None
        c_after = store.counts.cpu().numpy()
        # bytes streamed: every step reads the cache as it stood at that step
        lcfg = dict(cfg, num_kv_heads=Hkv_r)
        per_layer = [algorithmic_bytes_per_layer(c_before, lcfg), algorithmic_bytes_per_layer(c_after, lcfg)]
        step_bytes = L * (per_layer[0] + per_layer[1]) / 2.0
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            every = [torch.zeros_like(t) for _ in range(world)]
            dist.all_gather(every, t)
            rank_ms[fn.__name__] = [round(float(x.item()) / n_steps, 4) for x in every]
            ms = max(float(x.item()) for x in every)
            bt = torch.tensor([step_bytes], device=dev, dtype=torch.float64)
            dist.all_reduce(bt, op=dist.ReduceOp.SUM)
            step_bytes = float(bt.item())
        return ms, step_bytes, clocks

    launches[0] = 0
    ms, step_bytes, clocks = timed(resident_step, warmup, steps, 0)
    store.check_errors()
    n_launch = launches[0] - warmup * per_step_launches
    realloc_ms = [a.elapsed_time(b) for a, b in realloc_events]
    # the same steps without the reallocations: the steady-state step
    ms_steady, _, _ = timed(resident_step, 1, min(steps, 16), 3, realloc=False)
    steady_ms_per_step = ms_steady / min(steps, 16)

    # ---- the attention kernel alone ---------------------------------------------------------------------
    # (a) back to back: one launch per layer, every layer its own 188 MB, nothing else on the stream -- the kernel's
    #     average launch duration; (b) inside the step: a CUDA event pair around every launch of an un-graphed pass
    #     (includes the gap the host leaves before each launch)
    q0 = q_dev[0]
    store.build_plan()
    bb = []
    for rep in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for layer in range(L):
            skv_lib.check(store.lib.skv_decode_attention(ctypes.byref(store.desc), skv_lib.ptr(store.arena), layer,
                                                         skv_lib.ptr(store.plan), skv_lib.ptr(q0[layer]), skv_lib.DTYPE_F16, Hq_r,
                                                         skv_lib.ptr(store.partials), store.num_ctas,
                                                         skv_lib.ptr(store.logits) if store.track_importance else None,
                                                         skv_lib.ptr(store.err), store._stream()), "skv_decode_attention")
        e1.record()
        torch.cuda.synchronize()
        bb.append(e0.elapsed_time(e1) / L)
    attn_ms = float(np.median(bb[1:])) if len(bb) > 1 else bb[0]
    if world > 1:
        t = torch.tensor([attn_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        attn_ms = float(t.item())
    per_layer_bytes = algorithmic_bytes_per_layer(store.counts.cpu().numpy(), dict(cfg, num_kv_heads=Hkv_r))
    attn_events.clear()
    timed(kernel_timing_step, 1, min(steps, 4), 0, realloc=False)
    timed_events = attn_events[L:]
    attn_ms_in_step = float(np.mean([a.elapsed_time(b) for a, b in timed_events]))
    peak, peak_kind = measured_peak()
    achieved = per_layer_bytes / (attn_ms * 1e-3) / 1e9
    n_before = len(realloc_events)
    if seq_mode:
        ms_e2e, step_bytes_e2e = timed(host_step, warmup, steps, steps + warmup)[:2]
    else:
        ms_e2e, step_bytes_e2e, _ = timed(host_step, warmup, steps, steps + warmup)
    store.check_errors()
    realloc_ms_e2e = [a.elapsed_time(b) for a, b in realloc_events[n_before:]]

    # ---- self-check of the sharded paths: one layer against an unsharded store is the tests' job; here the ranks
    # only make sure they agree (sequence shards: every rank folded the same result)
    agree = None
    if seq_mode:
        chk = folded[0].clone()
        dist.broadcast(chk, 0)
        agree = bool(torch.allclose(chk, folded[0], rtol=0, atol=0))

    value = step_bytes * steps / (ms * 1e-3) / 1e9
    e2e_value = step_bytes_e2e * steps / (ms_e2e * 1e-3) / 1e9
    h2d = (q_stage.numel() * 2 + k_stage.numel() * 2 + v_stage.numel() * 2) * world
    d2h = out_dev.numel() * 4 * world
    traffic, traffic_src = (None, None)
    if args.config == 1 and world == 1 and not (args.batch or args.context or args.budget or args.layers):
        traffic, traffic_src = profile_traffic(kernel_name)
    shard_txt = {"kv_heads": f"KV heads split over the GPUs ({Hkv_r} of {Hkv} per GPU)",
                 "sequence": f"tokens of the sequence split over the GPUs ({N_r} of {N} per GPU), one exchange of all layers' "
                             "(max, sum, out) per step", "replicas": "every GPU holds the whole configuration"}[shard]
    line = {
        "metric": "packed_kv_decode_attention_throughput", "value": round(value, 2), "unit": "GB/s",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": round(ms / steps, 4),
        "higher_is_better": True, "scaling": "weak" if (shard == "replicas" and world > 1) else "strong", "vs_baseline": None,
        "dtype": "int8 tensor-core scores, f16 P.V, f32 accumulate" if kernel_name == "decode_attn_kernel" else "int8 tensor-core scores and P.V (tcgen05), f32 accumulate",
        "data": f"synthetic (seeded N(0,1) K/V, 4 outlier channels x8 per head, Zipf({cfg['zipf_s']}) importance)",
        "config": {"workload": workload_string(cfg),
                   "sharding": shard_txt if world > 1 else "one GPU", "kv_heads_per_gpu": Hkv_r,
                   "l2": "inputs larger than L2 (packed cache per step >> 126 MB)",
                   "bucket_histogram_2_3_4_8": hist,
                   "reallocation": (f"device allocator + requantise/repack of all layers after every {realloc_every}th "
                                    f"step, inside the timed region ({len(realloc_ms)} in {steps} steps); {settle} untimed cycles "
                                    "before, so that timed ones see a settled cache") if with_realloc else
                                   "none inside the timed region (importance tracking is off under sequence shards)",
                   "packed_bytes_per_step": int(step_bytes)},
        "decode_tokens_per_s": round(B * steps / (ms * 1e-3), 1),
        "steady_state_ms_per_step": round(steady_ms_per_step, 4),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "traffic": traffic, "traffic_source": traffic_src,
                     "peak_source": peak_kind, "kernel": kernel_name, "kernel_ms": round(attn_ms, 4),
                     "timing": f"CUDA events around {L} back-to-back launches (one per layer, each over its own cache), median of 2 passes"
                               + ("; max over ranks" if world > 1 else ""),
                     "kernel_ms_inside_step": round(attn_ms_in_step, 4),
                     "algorithmic_bytes_per_launch": int(per_layer_bytes),
                     "whole_step_frac": round(step_bytes / world / (steady_ms_per_step * 1e-3) / 1e9 / peak, 4)},
        "attention_kernel_choice": tune,
        "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h), "ms_per_step": round(ms_e2e / steps, 4),
                "reallocation_ms": round(float(np.mean(realloc_ms_e2e)), 3) if realloc_ms_e2e else None,
                "copies": "per layer on two copy streams inside the step's CUDA graph" if e2e_graphs else "around the step"},
        "reallocation_ms": round(float(np.mean(realloc_ms)), 3) if realloc_ms else None,
        "reallocation_moved_tokens": int(store._realloc["n_moves"].sum()) if realloc_ms else None,   # last one
        "reallocation_detail": [[round(m, 3), int(n)] for m, n in
                                zip(realloc_ms + realloc_ms_e2e, moved_log[:len(realloc_ms) + len(realloc_ms_e2e)].tolist())],
        "ms_per_step_by_rank": rank_ms or None,
        "reallocation_wait_for_ranks_ms": ([round(a[0].elapsed_time(b), 3) for a, b in zip(realloc_events, sync_events[1 + settle:])]
                                           if sync_events else None),
        "ranks_agree": agree,
        "gpu_launches": int(n_launch), "cuda_graph": graph is not None, "dependent_launch": pdl_choice,
        "sharded_self_check": self_check,
        "clocks": clocks,
    }
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(cfg, budget_s=args.cpu_seconds)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ----------------------------------------------------------------------------- CPU baseline
def _reference_modules():
    """The reference's own CPU modules when its package is importable (a checkout on PYTHONPATH); else None."""
    try:
        import torch
        from smartkv.core._quant_cpu import quantize_per_head
        from smartkv.core.cache import SmartKVCache
        from smartkv.core.fused_cpu import quantized_attention_streaming_cpu
        from smartkv.core.importance import ImportanceTracker
        return dict(torch=torch, quantize_per_head=quantize_per_head, SmartKVCache=SmartKVCache,
                    attention=quantized_attention_streaming_cpu, ImportanceTracker=ImportanceTracker)
    except Exception:       # noqa: BLE001
        return None


def cpu_baseline(cfg, budget_s=15.0):
    """The reference CPU path timed on this host: for one (sequence, layer) at the full context the streaming
    attention over int8 codes with the reference's GQA expansion, the importance update and the
    append-quantize; plus, once, the allocator for one sequence and the requantisation of its changed tokens in
    one layer.  The step time is scaled to batch x layers (reallocation amortised over realloc_every steps);
    GB/s counts the same algorithmic packed bytes.  When the reference package is importable its own functions
    are the ones timed (kind "reference": smartkv.core.fused_cpu, smartkv.core.importance, smartkv.core._quant_cpu
    and SmartKVCache._solve_allocation); otherwise the oracle's restatement of them (kind "port")."""
    from oracle import smartkv_oracle as orc
    ref = _reference_modules()
    try:
        from threadpoolctl import threadpool_info
        threads = max([p.get("num_threads", 1) for p in threadpool_info()] + [1])
    except Exception:
        threads = os.cpu_count() or 1
    Hq, Hkv, D, N = cfg["num_q_heads"], cfg["num_kv_heads"], cfg["head_dim"], cfg["context"]
    g = Hq // Hkv
    k, v = orc.synth_kv(N, Hkv, D, seed=0)
    imp0 = zipf_importance(N, 0, cfg["zipf_s"])
    scores = {t: (float("inf") if t < 4 else float(imp0[t])) for t in range(N)}
    if ref is not None:
        import warnings
        torch = ref["torch"]
        threads = torch.get_num_threads()
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            rc = ref["SmartKVCache"](num_layers=1, num_heads=Hkv, head_dim=D, memory_budget=0.9,
                                     available_bits=list(cfg["available_bits"]), device="cpu")
        # packed-byte accounting as on a CUDA device (the CPU constructor turns it off)
        from smartkv.core.allocation import compute_minimum_budget
        rc.use_packing = True
        rc.min_budget = compute_minimum_budget(Hkv, D, rc.scale_dtype, True)
        rc.memory_budget = cfg["memory_budget"]
        t0 = time.perf_counter()
        alloc = rc._solve_allocation(set(range(N)), scores, rc.protected_tokens | rc.special_token_ids)
        alloc_s = time.perf_counter() - t0
    else:
        acfg = orc.AllocatorConfig(Hkv, D, cfg["memory_budget"], cfg["available_bits"])
        t0 = time.perf_counter()
        alloc = orc.solve_allocation(acfg, range(N), scores, {})
        alloc_s = time.perf_counter() - t0
    bits = np.array([alloc[t] for t in range(N)], np.int64)
    # stored at 4 bits, then requantised from the stored codes to the allocated widths (one layer)
    k4, ks4 = orc.quantize_rows(k, 4)
    v4, vs4 = orc.quantize_rows(v, 4)
    kq, vq, ks, vs = k4.copy(), v4.copy(), ks4.copy(), vs4.copy()
    t0 = time.perf_counter()
    for w in (2, 3, 8):
        sel = bits == w
        if not sel.any():
            continue
        if ref is not None:      # cache.py:819-844: dequantise the stored codes, quantise again at the new width
            torch = ref["torch"]
            kd = torch.from_numpy(k4[sel].astype(np.float32) * ks4[sel][..., None])
            vd = torch.from_numpy(v4[sel].astype(np.float32) * vs4[sel][..., None])
            a, b_, c_, d_ = ref["quantize_per_head"](kd, vd, int(w))
            kq[sel], vq[sel], ks[sel], vs[sel] = a.numpy(), b_.numpy(), c_.numpy(), d_.numpy()
        else:
            kq[sel], ks[sel] = orc.requantize_rows(k4[sel], ks4[sel], w)
            vq[sel], vs[sel] = orc.requantize_rows(v4[sel], vs4[sel], w)
    requant_s = time.perf_counter() - t0
    rng = np.random.default_rng(0)
    q = rng.standard_normal((1, Hq, 1, D)).astype(np.float32)
    ck = rng.standard_normal((1, Hkv, D)).astype(np.float32)
    cv = rng.standard_normal((1, Hkv, D)).astype(np.float32)
    counts = np.array([[(bits == w).sum() for w in (2, 3, 4, 8)]])
    nbytes = algorithmic_bytes_per_layer(counts, cfg)
    if ref is not None:
        torch = ref["torch"]
        tq, tkq, tks, tvq, tvs = (torch.from_numpy(x) for x in (q, kq, ks, vq, vs))
        tck, tcv = torch.from_numpy(ck), torch.from_numpy(cv)
        tracker = ref["ImportanceTracker"](1, decay=0.9, device="cpu")
        ids = list(range(N + 1))

        def one():
            # the wrapper expands K/V to the query heads on every call (llama_smartkv.py:274-281)
            o, p = ref["attention"](tq, tkq.repeat_interleave(g, dim=1), tks.repeat_interleave(g, dim=1),
                                    tvq.repeat_interleave(g, dim=1), tvs.repeat_interleave(g, dim=1), tile_size=2048,
                                    current_k=tck.repeat_interleave(g, dim=1), current_v=tcv.repeat_interleave(g, dim=1),
                                    return_attn=True)
            tracker.update_attention(0, p, ids)
            ref["quantize_per_head"](tck, tcv, 4)
    else:
        imp = orc.ImportanceState(1)

        def one():
            # the reference expands K/V to the query heads on every call (llama_smartkv.py:274-281)
            o, p = orc.streaming_attention(q, orc.expand_gqa(kq, g), orc.expand_gqa(ks, g), orc.expand_gqa(vq, g),
                                           orc.expand_gqa(vs, g), tile_size=2048, current_k=orc.expand_gqa(ck, g),
                                           current_v=orc.expand_gqa(cv, g))
            imp.update(0, p, range(N + 1))
            orc.quantize_per_head(ck[0][None], cv[0][None], 4)
    one()
    t0 = time.perf_counter()
    it = 0
    while True:
        one()
        it += 1
        if time.perf_counter() - t0 > budget_s or it >= 200:
            break
    dt = (time.perf_counter() - t0) / it
    B, L, every = cfg["batch"], cfg["num_layers"], cfg["realloc_every"]
    step_s = dt * B * L + (alloc_s * B + requant_s * B * L) / every
    return {"value": round(nbytes * B * L / step_s / 1e9, 4), "unit": "GB/s", "cores": int(threads),
            "kind": "reference" if ref is not None else "port",
            "sample": f"1 sequence x 1 layer at context {N} (attention + importance + append-quantize), {it} iterations, "
                      f"{dt * 1e3:.1f} ms each; allocator for one sequence {alloc_s * 1e3:.0f} ms and requantisation of "
                      f"one (sequence, layer) {requant_s * 1e3:.0f} ms, once; step time scaled to batch {B} x {L} "
                      f"layers with the reallocation amortised over {every} steps",
            "ms_per_sequence_layer": round(dt * 1e3, 3), "ms_per_step": round(step_s * 1e3, 1)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = dict(CONFIGS[args.config])
    t0 = time.perf_counter()
    per_step_budget = max(2.0, min(20.0, 120.0 / max(1, args.steps + args.warmup)))
    vals = []
    base = None
    for i in range(args.warmup + args.steps):
        base = cpu_baseline(cfg, budget_s=per_step_budget)
        if i >= args.warmup:
            vals.append(base["value"])
    value = float(np.mean(vals))
    step_ms = base["ms_per_step"]
    base["value"] = round(value, 4)
    line = {
        "impl": "reference", "metric": "packed_kv_decode_attention_throughput", "value": round(value, 4),
        "unit": "GB/s", "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(step_ms, 2), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic (seeded N(0,1) K/V, 4 outlier channels x8 per head, Zipf(1.1) importance)",
        "config": {"workload": workload_string(cfg),
                   "sample": "each step is a bounded sample of that workload on the host cores: one (sequence, layer) at "
                             "the full context, one allocator call and one requantisation; ms_per_step and value are "
                             "scaled to batch x layers with the reallocation amortised over 16 steps"},
        "cpu_baseline": base,
        "e2e": {"value": round(value, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": round(time.perf_counter() - t0, 1),
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from Python instead of replaying a CUDA graph")
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    ap.add_argument("--batch", type=int, default=0, help="other batch than the contract's 16 (extra measurements only)")
    ap.add_argument("--context", type=int, default=0, help="other context than the contract's 8192 (extra measurements only)")
    ap.add_argument("--budget", type=float, default=0.0, help="other memory budget than the contract's 0.35")
    ap.add_argument("--layers", type=int, default=0,
                    help="override the layer count (profiler captures of a small case only; not a bench line)")
    ap.add_argument("--attn-kernel", default="auto", choices=["auto", "fragment", "tensor_memory"],
                    help="auto: both decode-attention kernels are timed on the populated cache and the faster one runs")
    ap.add_argument("--config", type=int, default=1, choices=sorted(CONFIGS) + [2],
                    help="1 (default, the bench line), 3 (long context, sequence shards), 4 (70B shape, KV-head shards) or "
                         "2 (end-to-end generation through the LlamaSmartKV wrapper; decode tokens/s, one GPU)")
    ap.add_argument("--decode-sample", type=int, default=16, help="--config 2 --impl reference: decode steps to time")
    ap.add_argument("--replicas", action="store_true", help="under torchrun: every rank holds the whole configuration (weak scaling)")
    ap.add_argument("--no-dependent-launch", action="store_true",
                    help="launch the attention / post-attention kernels without programmatic dependent launch (comparison only)")
    ap.add_argument("--dependent-launch-mode", type=int, default=-1, choices=[-1, 0, 1, 2, 3],
                    help="comparison only: 0 off, 1 both kernels, 2 attention kernel only, 3 post-attention kernel only")
    ap.add_argument("--no-settle", action="store_true", help="skip the untimed reallocation cycles before the timed passes")
    args = ap.parse_args()
    if (args.no_dependent_launch or args.dependent_launch_mode >= 0) and args.impl != "reference":
        from smartkv_b200 import _lib as _skv
        _skv.lib().skv_set_dependent_launch(0 if args.no_dependent_launch else args.dependent_launch_mode)
    if args.config == 2:
        if int(os.environ.get("RANK", "0")) == 0:
            (run_generation_reference if args.impl == "reference" else run_generation)(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
