"""The allocation-free attention entry point (vuib_attention_noalloc) against the
handle-based one (vuib_attention) that uses the caller's workspace.

Collected last on purpose: a run that stops at the first failure has then already
run every other test.  Needs a B200; builds its own engine so it also passes when
run alone in a fresh process."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, eng, layer, q, slots, pos, *, n_rows=None, max_seq=None, heads=(16, 8)):
    kv = eng.model.decoder.flash_kv_caches[layer]
    q = q.to("cuda", torch.bfloat16).contiguous()
    rs = slots.to("cuda", torch.int32).contiguous()
    rp = pos.to("cuda", torch.int32).contiguous()
    out = torch.zeros_like(q)
    err = C.create_string_buffer(256)
    P = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    rc = lib.vuib_attention_noalloc(
        heads[0], heads[1], max_seq or eng.max_seq, n_rows if n_rows is not None else q.shape[0], P(q), P(kv.k_cache),
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
    for heads in ((32, 16), (16, 4), (16, 5)):  # too many query heads; 4 query heads per kv head; not a multiple
        rc, _, msg = _call_noalloc(lib, eng, 0, q, slots, pos, heads=heads)
        assert rc == -3 and "n_heads" in msg, heads


def test_noalloc_attention_full_scratch_extent_and_equal_heads(nano_model):
    """The largest shape the built-in scratch is sized for (8 rows, 2048 positions = 16 splits per row,
    lengths up to the last position) against vuib_attention, bit for bit; one query head per kv head
    (n_heads == n_kv_heads) on a synthetic cache against fp32 softmax attention; and a position past
    max_seq, which is clamped instead of followed."""
    from vui_b200 import Engine, _lib

    lib = _lib.load()
    eng = Engine(model=nano_model, max_rows=8, max_seq=2048)
    g = torch.Generator().manual_seed(12)
    layer = 1
    kv = eng.model.decoder.flash_kv_caches[layer]
    kv.k_cache.copy_(torch.randn(kv.k_cache.shape, generator=g).to(torch.bfloat16))
    kv.v_cache.copy_(torch.randn(kv.v_cache.shape, generator=g).to(torch.bfloat16))
    slots = torch.tensor([0, 1, 2, 3, 4, 5, 6, 7])
    pos = torch.tensor([2047, 1920, 1919, 1024, 5, 2046, 128, 1500])
    for _ in range(2):
        q = torch.randn(8, 1024, generator=g).to(torch.bfloat16)
        want = eng._attention(layer, q, slots, pos)
        rc, got, msg = _call_noalloc(lib, eng, layer, q, slots, pos)
        assert rc == 0, msg
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    # a position past the cache is clamped to the last one: same result as asking for max_seq - 1
    q1 = torch.randn(1, 1024, generator=g).to(torch.bfloat16)
    rc, a, _ = _call_noalloc(lib, eng, layer, q1, torch.tensor([2]), torch.tensor([10 ** 6]))
    rc2, b, _ = _call_noalloc(lib, eng, layer, q1, torch.tensor([2]), torch.tensor([2047]))
    torch.cuda.synchronize()
    assert rc == 0 and rc2 == 0 and torch.equal(a, b)
    # one query head per kv head: (slots, max_seq, 8, 64) cache, 8 query heads
    kc = torch.randn(3, 300, 8, 64, generator=g).to("cuda", torch.bfloat16)
    vc = torch.randn(3, 300, 8, 64, generator=g).to("cuda", torch.bfloat16)
    q8 = torch.randn(3, 512, generator=g).to("cuda", torch.bfloat16)
    rs = torch.tensor([2, 0, 1], dtype=torch.int32, device="cuda")
    rp = torch.tensor([299, 0, 130], dtype=torch.int32, device="cuda")
    out = torch.zeros_like(q8)
    err = C.create_string_buffer(256)
    P = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    rc = lib.vuib_attention_noalloc(8, 8, 300, 3, P(q8), P(kc), P(vc), P(rs), P(rp), P(out),
                                    C.c_void_p(torch.cuda.current_stream().cuda_stream), err, 256)
    assert rc == 0, err.value.decode()
    torch.cuda.synchronize()
    for r in range(3):
        k = kc[rs[r], : rp[r] + 1].float()
        v = vc[rs[r], : rp[r] + 1].float()
        sc = torch.einsum("hd,thd->ht", q8[r].view(8, 64).float(), k) * 0.125
        ref = torch.einsum("ht,thd->hd", torch.softmax(sc, dim=-1), v).reshape(-1)
        e = (out[r].float() - ref).abs().max().item()
        assert e <= 2.0 ** -8 * max(1.0, ref.abs().max().item()) + 1e-3, (r, e)
