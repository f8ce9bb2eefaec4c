"""The C-ABI library without a GPU: it loads, exports every symbol the header
declares, and rejects bad arguments on the host before any launch."""
import ctypes as C
import os
import re

import pytest

from vui_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_functions():
    with open(os.path.join(ROOT, "include", "vuib200.h")) as f:
        src = f.read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(vuib_[a-z0-9_]+)\s*\(", src)))


def test_every_declared_symbol_is_exported_and_bound():
    lib = _lib.load()
    names = _header_functions()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/vuib200.h but not exported"
        assert n in _lib.SYMBOLS, f"{n} has no ctypes signature"
    assert sorted(_lib.SYMBOLS) == names


def _cfg(**kw):
    base = dict(d_model=1024, n_layers=24, n_heads=16, n_kv_heads=8, head_dim=64, ffn=3072, n_quantizers=16,
                codebook_size=2048, rq_d_model=512, rq_n_layers=4, rq_n_heads=8, rq_ffn=1408, norm_eps=1e-5,
                rq_norm_eps=1e-6, n_slots=2, max_seq=1024, max_rows=1, max_prefill_rows=256)
    base.update(kw)
    return _lib.VuibConfig(**base)


def test_create_validates_shape_and_ranges():
    lib = _lib.load()
    h = C.c_void_p()
    assert lib.vuib_create(None, C.byref(h)) == -1
    assert lib.vuib_create(C.byref(_cfg(head_dim=96)), C.byref(h)) == -2
    assert lib.vuib_create(C.byref(_cfg(codebook_size=1024)), C.byref(h)) == -2
    assert lib.vuib_create(C.byref(_cfg(rq_ffn=1000)), C.byref(h)) == -2
    assert lib.vuib_create(C.byref(_cfg(max_rows=0)), C.byref(h)) == -3
    assert lib.vuib_create(C.byref(_cfg()), C.byref(h)) == 0 and h.value
    assert lib.vuib_create(C.byref(_cfg(rq_ffn=1536)), C.byref(C.c_void_p())) == 0
    n = C.c_size_t()
    assert lib.vuib_workspace_bytes(h, C.byref(n)) == 0
    assert 1 << 20 < n.value < 1 << 30
    # nothing bound yet: every compute entry refuses on the host
    assert lib.vuib_backbone_step(h, 1, None, None, None, None, None, None, None) == -4
    assert lib.vuib_prefill(h, 1, None, None, None, None, None) == -4
    assert lib.vuib_depth_step(h, 1, None, None, None, None, 0, None, None, None) == -4
    assert lib.vuib_set_sampling(h, C.byref(_lib.VuibSampling(1.0, 1, 1, 1.0, 0, 0, 0)), None) == -4
    assert lib.vuib_bind_workspace(h, C.c_void_p(0x1001), n.value) == -6  # misaligned
    buf = C.create_string_buffer(256)
    assert lib.vuib_last_error(h, buf, 256) == 0 and b"aligned" in buf.value
    with pytest.raises(_lib.VuibError):
        _lib.check(h, -6)
    assert lib.vuib_bind_weights(h, C.byref(_lib.VuibWeights())) == -1
    assert lib.vuib_launch_count(h) == 0
    assert lib.vuib_destroy(h) == 0


def test_struct_sizes_match_header():
    assert C.sizeof(_lib.VuibConfig) == 18 * 4
    assert C.sizeof(_lib.VuibSampling) == 32
    assert C.sizeof(_lib.VuibWeights) == 8 * (5 + 7 * 64 + 5 + 7 * 64)
