"""The reference-facing Python API (Engine / Row / GenConfig / Segment / RenderRequest) end to
end on the GPU with a stand-in tokenizer (the reference's downloads BPE files) and no codec:
the calls of docs/python-api.md in the reference, checked for shapes, ranges, bookkeeping."""
import zlib

import pytest
import torch

pytestmark = pytest.mark.gpu


class StubTok:
    """Deterministic word-hash tokenizer with the attributes Engine reads."""

    vocab_size = 151936

    def __init__(self):
        self.special_to_id = {"[SC]": 151900}

    def encode(self, text: str):
        ids = [zlib.crc32(w.encode()) % 151000 for w in text.split()]
        return torch.tensor(ids or [1], dtype=torch.long)


@pytest.fixture(scope="module")
def model_tok(nano_sd):
    from vui_b200 import VuiB200, VuiShape

    return VuiB200(VuiShape(), nano_sd, device="cuda", tokenizer=StubTok())


def _prompt_codes(n, seed):
    return torch.randint(0, 2048, (n, 16), generator=torch.Generator().manual_seed(seed))


def test_row_render_and_rewind(model_tok):
    from vui_b200 import Engine, GenConfig, Segment

    eng = Engine(model=model_tok, max_rows=1, max_seq=1024)
    cfg = GenConfig(temperature=0.9, max_secs=4.0, min_secs=0.2, eos_threshold=0.99)
    with eng.new_row() as row:
        off = row.prefill([Segment("A short voice prompt, spoken calmly.", _prompt_codes(20, 1))])
        # [SC] + 6 text tokens + 20 audio positions (no speaker projection in this checkpoint)
        assert off == row.offset == 6 + 1 + 20
        assert abs(row.prompt_wps - 6 / (20 / 12.5)) < 1e-6
        codes, audio = row.render("Hello there, this is a test of the engine. It speaks two sentences.", cfg)
        assert audio is None  # no codec attached
        assert codes.dtype == torch.long and codes.shape[1] == 16 and 1 <= codes.shape[0] <= 50
        assert codes.min() >= 0 and codes.max() < 2048
        assert row.offset > off
        assert row.rewind() == off and row.offset == off
        again, _ = row.render("Hello there, this is a test of the engine. It speaks two sentences.", cfg)
        assert again.shape[1] == 16
        assert row.reset() == 0 and row.offset == 0
    eng.check_device()
    with pytest.raises(RuntimeError):
        eng2 = Engine(model=model_tok, max_rows=1, max_seq=64)
        r = eng2.new_row()
        r.prefill([Segment("one two three", _prompt_codes(80, 2))])  # overflows max_seq


def test_stream_codes_and_cancel(model_tok):
    from vui_b200 import Engine, GenConfig

    eng = Engine(model=model_tok, max_rows=1, max_seq=1024)
    cfg = GenConfig(temperature=0.8, top_k=50, max_secs=3.0, eos_threshold=0.995, n_codebooks=8)
    row = eng.new_row()
    frames = list(eng._stream_codes(row, "Streaming works frame by frame, one chunk after another.", cfg))
    assert 1 <= len(frames) <= int(3.0 * 12.5)
    for f in frames:
        assert f.shape == (16,) and f[:8].max() < 2048 and (f[8:] == 0).all()  # n_codebooks=8 zero-pads

    class Cancel:
        def __init__(self, after):
            self.n, self.after = 0, after

        def is_set(self):
            self.n += 1
            return self.n > self.after

    row.reset()
    few = list(eng._stream_codes(row, "Streaming works frame by frame, one chunk after another.", cfg, Cancel(3)))
    assert len(few) < len(frames) or len(frames) <= 3
    with pytest.raises(RuntimeError):
        next(row.stream("needs a codec"))
    row.close()
    eng.check_device()


def test_render_all_and_continuous_batching(model_tok):
    from vui_b200 import Engine, GenConfig, RenderRequest, Segment

    eng = Engine(model=model_tok, max_rows=3, max_seq=512)
    cfg = GenConfig(temperature=0.9, max_secs=2.0, eos_threshold=0.99)
    rows = [eng.new_row() for _ in range(3)]
    for i, r in enumerate(rows):
        r.prefill([Segment(f"prompt number {i} here", _prompt_codes(10 + i, 10 + i))])
    res = eng._render_rows(rows, ["First row text here.", "Second row says something else entirely.", "Third."], cfg)
    assert set(res) == {0, 1, 2}
    for c in res.values():
        assert c.shape[1] == 16 and 1 <= c.shape[0] <= 25 and c.max() < 2048
    assert eng.render_all(rows, ["a b c.", "d e f.", "g h i."], cfg) == [None, None, None]  # no codec
    for r in rows:
        r.close()
    # five requests over three slots, answered in input order
    reqs = [RenderRequest(segments=[Segment(f"voice {i}", _prompt_codes(8, 30 + i))], text=f"Request {i} speaks now.")
            for i in range(5)]
    out = eng.render_continuous_codes(reqs, cfg)
    assert len(out) == 5
    for c in out:
        assert c.ndim == 2 and c.shape[1] == 16 and 1 <= c.shape[0] <= 25 and c.min() >= 0 and c.max() < 2048
    assert eng.render_continuous_codes([], cfg) == []
    eng.check_device()


def test_cut_short_chunk_is_retried_at_lower_temperature(model_tok):
    """A chunk that ends with fewer than two frames per word is rewound and spoken again at 0.5,
    then 0.3, then accepted (engine.py:953-983).  With an EOS threshold that every frame passes,
    every chunk ends at min_frames, so each of the two chunks is retried exactly twice."""
    from vui_b200 import Engine, GenConfig, Segment

    eng = Engine(model=model_tok, max_rows=1, max_seq=512)
    rewinds, temps = [], []
    orig_rewind, orig_apply = eng._rewind_row, eng._apply_cfg
    eng._rewind_row = lambda row, off: (rewinds.append(off), orig_rewind(row, off))[1]
    eng._apply_cfg = lambda cfg, temperature=None, greedy=False: (temps.append(temperature),
                                                                  orig_apply(cfg, temperature, greedy))[1]
    cfg = GenConfig(temperature=0.9, max_secs=4.0, min_secs=0.16, eos_threshold=-1.0, sentence_only=True)
    row = eng.new_row()
    off0 = row.prefill([Segment("a calm voice prompt", _prompt_codes(12, 5))])
    codes, _ = row.render("The first sentence has seven words here. The second sentence also has seven words.", cfg)
    min_frames = int(0.16 * 12.5)
    assert min_frames == 2
    # two chunks, each accepted after two retries with min_frames + 1 frames kept (frame 0 + 2 steps - the EOS frame)
    assert len(rewinds) == 4 and rewinds[0] == rewinds[1] and rewinds[2] == rewinds[3] and rewinds[0] >= off0
    assert [t for t in temps if t is not None] == [0.5, 0.3, 0.5, 0.3]
    assert codes.shape[1] == 16 and codes.shape[0] == 2 * min_frames
    assert codes.min() >= 0 and codes.max() < 2048
    eng.check_device()


def test_cb0_statistics_and_streaming_entropy_gate(model_tok):
    """The sampler reports entropy and top probability of softmax(cb0 logits / T) (what the reference's
    `_entropy_top1` computes, engine.py:1369-1372); the streaming gate (engine.py:1385-1533) holds the
    first gate_frames frames back, retries the chunk at 0.5 and 0.3 while their mean entropy is above the
    threshold, and otherwise only delays them: a gate that passes yields exactly the ungated frames."""
    from vui_b200 import Engine, GenConfig

    eng = Engine(model=model_tok, max_rows=1, max_seq=512)
    text = "This sentence is long enough for a dozen frames of speech, at the very least."
    base = dict(temperature=0.8, top_k=50, rep_penalty=1.0, max_secs=2.0, min_secs=0.4, eos_threshold=2.0,
                sentence_only=True)

    def stream(cfg):
        eng.reset()
        eng._ws_reset_counters()
        row = eng.new_row()
        out = [f.clone() for f in eng._stream_codes(row, text, cfg)]
        row.close()
        return torch.stack(out)

    plain = stream(GenConfig(**base))
    # statistics of the last frame's cb0 draw against torch on the logits the engine exposes
    p = torch.softmax(eng._g_cb0_out[0].float() / 0.8, dim=-1)
    ent = float(-(p * p.clamp_min(1e-9).log()).sum())
    st = eng._g_cb0_stats[0].cpu()
    assert abs(float(st[0]) - ent) < 2e-3 * max(1.0, ent) and abs(float(st[1]) - float(p.max())) < 1e-4
    assert 0.0 < float(st[0]) <= 7.63  # ln 2048

    passed = stream(GenConfig(**base, gate_frames=4, gate_entropy_max=100.0))
    assert torch.equal(plain, passed)

    rewinds, temps = [], []
    orig_rewind, orig_apply = eng._rewind_row, eng._apply_cfg
    eng._rewind_row = lambda row, off: (rewinds.append(off), orig_rewind(row, off))[1]
    eng._apply_cfg = lambda cfg, temperature=None, greedy=False: (temps.append(temperature),
                                                                  orig_apply(cfg, temperature, greedy))[1]
    gated = stream(GenConfig(**base, gate_frames=4, gate_entropy_max=0.0, gate_retries=2))
    eng._rewind_row, eng._apply_cfg = orig_rewind, orig_apply
    assert len(rewinds) == 2 and rewinds[0] == rewinds[1]           # two retries from the chunk's start
    assert [t for t in temps if t is not None] == [0.5, 0.3]
    assert gated.shape == plain.shape and gated.min() >= 0 and gated.max() < 2048
    eng.check_device()


def test_frame_through_host_memory_equals_replay_and_read(model_tok):
    """vuib_frame_host (host -> device codes, the frame, device -> host codes and EOS, one graph launch inside the
    library) produces the frames that a graph replay followed by the engine's read-back produces, with and
    without the input copy, for one stream and for three (padded to a bucket of four)."""
    from vui_b200 import Engine

    ids = torch.randint(0, 1000, (40,), generator=torch.Generator().manual_seed(3))

    def start(n_rows):
        eng = Engine(model=model_tok, max_rows=4, max_seq=256, seed=11)
        rows = [eng.new_row() for _ in range(n_rows)]
        hid = torch.stack([eng.prefill_ids(r, ids[: 30 + 3 * i]) for i, r in enumerate(rows)])
        eng._apply_cfg(None, greedy=True)
        eng._g_slot_idx[:n_rows] = torch.tensor([r.idx for r in rows], device=eng.device, dtype=torch.int32)
        eng._g_seq_inc[:n_rows].fill_(1)
        eng._g_codes_in[:n_rows] = eng._first_frames(rows, hid)
        return eng

    for n_rows in (1, 3):
        ref = start(n_rows)
        want = []
        for _ in range(5):
            ref._frame_step(n_rows)
            c, e = ref._read_frame(n_rows)
            want.append((c.clone(), e.clone()))
        ref.check_device()

        a = start(n_rows)  # results only
        for c, e in want:
            hc, he = a._frame_host(n_rows)
            assert torch.equal(hc, c) and torch.equal(he, e)
        a.check_device()

        b = start(n_rows)  # the previous frame's codes travel through host memory as well
        h_in = b._g_codes_in[:n_rows].cpu().pin_memory()
        for c, e in want:
            hc, he = b._frame_host(n_rows, h_in)
            assert torch.equal(hc, c) and torch.equal(he, e)
            h_in.copy_(hc)
        b.check_device()
        assert torch.equal(a.seq_lens, ref.seq_lens) and torch.equal(b.seq_lens, ref.seq_lens)


def test_single_row_frames_alternating_between_two_rows(model_tok):
    """The one-stream attention block asks for a row's old keys before it has waited for its predecessor, with the
    (slot, position) it finds in memory, and asks again if they turn out to be another row's.  Two rows of different
    lengths decoded in turn, one frame each, must give exactly the frames each of them gives when decoded alone."""
    from vui_b200 import Engine

    gen = torch.Generator().manual_seed(5)
    ids = [torch.randint(0, 1000, (n,), generator=gen) for n in (31, 57)]

    def first(eng, row, tokens):
        hid = eng.prefill_ids(row, tokens)
        return eng._first_frames([row], hid[None])[0]

    def step(eng, row, codes_in):
        eng._g_slot_idx[0] = row.idx
        eng._g_seq_inc[0] = 1
        eng._g_codes_in[0] = codes_in
        eng._frame_step(1)
        c, _ = eng._read_frame(1)
        return c[0].clone()

    alone = []
    for tokens in ids:
        eng = Engine(model=model_tok, max_rows=2, max_seq=256, seed=3)
        eng._apply_cfg(None, greedy=True)
        row = eng.new_row()
        cur = first(eng, row, tokens)
        out = []
        for _ in range(4):
            cur = step(eng, row, cur.to(eng.device))
            out.append(cur)
        eng.check_device()
        alone.append(out)

    eng = Engine(model=model_tok, max_rows=2, max_seq=256, seed=3)
    eng._apply_cfg(None, greedy=True)
    rows = [eng.new_row(), eng.new_row()]
    cur = [first(eng, rows[i], ids[i]) for i in range(2)]
    for f in range(4):
        for i in range(2):
            cur[i] = step(eng, rows[i], cur[i].to(eng.device))
            assert torch.equal(cur[i], alone[i][f]), (f, i)
    eng.check_device()
