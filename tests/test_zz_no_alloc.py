"""The allocation-free attention entry point (vuib_attention_noalloc) against the
handle-based one (vuib_attention) that uses the caller's workspace.

Collected last on purpose: a run that stops at the first failure has then already
run every other test.  Needs a B200; builds its own engine so it also passes when
run alone in a fresh process."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, eng, layer, q, slots, pos, *, n_rows=None, max_seq=None):
    kv = eng.model.decoder.flash_kv_caches[layer]
    q = q.to("cuda", torch.bfloat16).contiguous()
    rs = slots.to("cuda", torch.int32).contiguous()
    rp = pos.to("cuda", torch.int32).contiguous()
    out = torch.zeros_like(q)
    err = C.create_string_buffer(256)
    P = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    rc = lib.vuib_attention_noalloc(
        16, 8, max_seq or eng.max_seq, n_rows if n_rows is not None else q.shape[0], P(q), P(kv.k_cache),
        P(kv.v_cache), P(rs), P(rp), P(out), C.c_void_p(torch.cuda.current_stream().cuda_stream), err, 256)
    return rc, out, err.value.decode()


def test_noalloc_attention_matches_workspace_attention(nano_model):
    """Two calls in a row (different rows, lengths and queries, so the second must not be
    confused by what the first left in the shared scratch) give what vuib_attention gives."""
    from vui_b200 import Engine, _lib

    lib = _lib.load()
    eng = Engine(model=nano_model, max_rows=8, max_seq=640)
    g = torch.Generator().manual_seed(11)
    layer = 3
    kv = eng.model.decoder.flash_kv_caches[layer]
    kv.k_cache.copy_(torch.randn(kv.k_cache.shape, generator=g).to(torch.bfloat16))
    kv.v_cache.copy_(torch.randn(kv.v_cache.shape, generator=g).to(torch.bfloat16))
    cases = [
        (torch.tensor([0, 1, 2, 3, 4, 5, 6, 7]), torch.tensor([639, 0, 127, 128, 400, 255, 256, 31])),
        (torch.tensor([8, 2, 2]), torch.tensor([17, 513, 514])),
    ]
    for slots, pos in cases:
        q = torch.randn(len(slots), 1024, generator=g).to(torch.bfloat16)
        want = eng._attention(layer, q, slots, pos)
        rc, got, msg = _call_noalloc(lib, eng, layer, q, slots, pos)
        assert rc == 0, msg
        torch.cuda.synchronize()
        # same kernel, same split order: the tolerance of the attention parity test is met with zero error
        err = (got.float() - want.float()).abs().max().item()
        assert err <= 2.0 ** -8 * max(1.0, want.float().abs().max().item()), err
        assert torch.equal(got, want)


def test_noalloc_attention_rejects_sizes_beyond_its_scratch(nano_model):
    from vui_b200 import Engine, _lib

    lib = _lib.load()
    eng = Engine(model=nano_model, max_rows=8, max_seq=640)
    q = torch.zeros(8, 1024, dtype=torch.bfloat16)
    slots, pos = torch.zeros(8, dtype=torch.int32), torch.zeros(8, dtype=torch.int32)
    rc, _, msg = _call_noalloc(lib, eng, 0, q, slots, pos, n_rows=9)
    assert rc == -3 and "n_rows" in msg
    rc, _, msg = _call_noalloc(lib, eng, 0, q, slots, pos, max_seq=4096)
    assert rc == -3 and "max_seq" in msg
