"""CPU-side checks of the C ABI: the library builds for sm_100a, loads without a GPU
and exports every symbol the header declares; host-only entry points behave."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    from smartkv_b200 import _lib, build
    build.build()
    return _lib


def header_functions():
    text = open(os.path.join(ROOT, "include", "smartkv_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(skv_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(L):
    names = header_functions()
    assert len(names) >= 10
    handle = L.lib()
    for n in names:
        assert hasattr(handle, n), f"{n} declared in the header but not exported"
    assert set(names) == set(L.exported_symbols()), "ctypes signature table and header disagree"
    assert handle.skv_build_arch() == 100


def test_status_strings(L):
    assert L.lib().skv_status_string(0) == b"ok"
    assert b"capacity" in L.lib().skv_status_string(-3)
    with pytest.raises(L.SmartKVLibraryError):
        L.check(-1, "x")


def test_store_layout(L):
    d = L.StoreDesc()
    d.num_layers, d.num_seqs, d.num_kv_heads, d.head_dim = 2, 3, 8, 128
    for i, c in enumerate((1024, 512, 256, 128)):
        d.cap[i] = c
    assert L.lib().skv_store_layout(ctypes.byref(d)) == 0
    assert list(d.row_bytes) == [32, 48, 64, 128]
    assert list(d.bucket_base) == [0, 1024, 1536, 1792] and d.slots == 1920
    offs = []
    for i in range(4):
        for arr in (d.k_off, d.v_off, d.sc_off):
            offs.append(arr[i])
            assert arr[i] % 256 == 0          # every region 256-byte aligned (>= the 16 bytes bulk copies need)
    assert offs == sorted(offs) and len(set(offs)) == 12
    assert d.sc_off[3] + 8 * 128 * 8 <= d.arena_bytes and d.arena_bytes % 256 == 0
    assert d.total_bytes == d.arena_bytes * 6
    # packed rows of any bucket start on 16-byte boundaries for every multiple-of-16 key offset
    for i in range(4):
        assert (16 * d.row_bytes[i]) % 16 == 0
    d.head_dim = 96
    assert L.lib().skv_store_layout(ctypes.byref(d)) < 0
    d.head_dim = 64
    d.cap[0] = 100
    assert L.lib().skv_store_layout(ctypes.byref(d)) < 0
    assert L.lib().skv_store_layout(None) < 0


def test_missing_library_fails_loudly(L, monkeypatch):
    import smartkv_b200._lib as mod
    monkeypatch.setattr(mod, "_lib", None)
    monkeypatch.setattr(mod, "LIB_PATH", "/nonexistent/libsmartkv_b200.so")
    with pytest.raises(mod.SmartKVLibraryError, match="no CPU fallback"):
        mod.lib()


def test_bucket_capacities():
    from smartkv_b200.store import bucket_capacities
    caps = bucket_capacities(8192, 0.35)
    assert all(c % 128 == 0 for c in caps)
    assert caps[0] >= 8192 and caps[3] < 8192 and caps[3] >= int(0.35 * 16 * 8192 / 8)


def test_alloc_config_clamps_like_the_reference():
    import math

    from oracle import smartkv_oracle as orc
    from smartkv_b200.store import make_alloc_config
    c = make_alloc_config(8, 128, 0.35, (8, 2, 4, 3), utility_alpha=0.05, importance_floor=-1.0,
                          hysteresis_rank_threshold=-3.0, hysteresis_intervals=0, high_precision_fraction=0.9,
                          high_precision_boost=0.2, min_high_precision_tokens=-4, protected=(2, 0, 1, 1))
    o = orc.AllocatorConfig(8, 128, 0.35, (8, 2, 4, 3), utility_alpha=0.05, importance_floor=-1.0,
                            hysteresis_rank_threshold=-3.0, hysteresis_intervals=0, high_precision_fraction=0.9,
                            high_precision_boost=0.2, min_high_precision_tokens=-4)
    assert list(c.bits)[:c.num_bits] == o.available_bits == [2, 3, 4, 8]
    alpha = min(max(o.utility_alpha, 0.1), 1.0)
    assert [c.util[i] for i in range(4)] == [math.pow(b, alpha) for b in (2, 3, 4, 8)]
    assert (c.importance_floor, c.rank_threshold, c.hysteresis_intervals) == (
        o.importance_floor, o.hysteresis_rank_threshold, o.hysteresis_intervals)
    assert (c.high_fraction, c.high_boost, c.min_high_tokens) == (
        o.high_precision_fraction, o.high_precision_boost, o.min_high_precision_tokens)
    assert c.num_protected == 3 and list(c.protected_ids)[:3] == [0, 1, 2] and c.use_packing == 1
    lin = make_alloc_config(4, 64, 0.5, (2, 4, 8), utility_alpha=0.0)        # alpha <= 0 means linear utility
    assert [lin.util[i] for i in range(3)] == [2.0, 4.0, 8.0]
    import pytest
    with pytest.raises(ValueError):
        make_alloc_config(4, 64, 0.5, (2, 5))
    with pytest.raises(ValueError):
        make_alloc_config(4, 64, 0.5, (2, 4), protected=range(40))


def test_alias_registers_the_reference_import_name():
    """``alias_as_smartkv`` makes ``smartkv...`` imports resolve to this package; it is opt-in."""
    import subprocess
    import sys
    code = ("import sys, smartkv_b200; assert 'smartkv' not in sys.modules; smartkv_b200.alias_as_smartkv(); "
            "from smartkv.models.llama_smartkv import LlamaSmartKV, SmartKVConfig; "
            "from smartkv.core.cache import SmartKVCache; import smartkv.kernels as k; "
            "assert SmartKVCache is smartkv_b200.SmartKVCache and hasattr(k, 'quantized_attention'); "
            "assert SmartKVConfig().device == 'cpu'; print('ok')")
    root = __import__("os").path.dirname(__import__("os").path.dirname(__import__("os").path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=root, timeout=300)
    assert r.returncode == 0 and r.stdout.strip() == "ok", r.stderr
