"""The callers either side of the decode step, on the GPU with a stand-in tokenizer and no codec:
KV save / load in the reference's on-disk layouts, the TTSEngine adapter and its command loop, the
older InferenceState / stream_frames API, the conditioning bias and the speaker token."""
import queue
import threading
import zlib

import pytest
import torch

pytestmark = pytest.mark.gpu


class StubTok:
    vocab_size = 151936

    def __init__(self):
        self.special_to_id = {"[SC]": 151900}

    def encode(self, text: str):
        ids = [zlib.crc32(w.encode()) % 151000 for w in text.split()]
        return torch.tensor(ids or [1], dtype=torch.long)


@pytest.fixture(scope="module")
def model_tok(nano_sd):
    """Benchmark-shaped weights plus random conditioning / speaker projections."""
    from vui_b200 import VuiB200, VuiShape

    g = torch.Generator().manual_seed(99)
    sd = dict(nano_sd)
    sd["sq_proj.weight"] = torch.empty(1024, 6).normal_(0, 0.01, generator=g).bfloat16()
    sd["wps_proj.proj.weight"] = torch.empty(1024, 1).normal_(0, 0.01, generator=g).bfloat16()
    sd["spk_proj.weight"] = torch.empty(1024, 1024).normal_(0, 0.01, generator=g).bfloat16()
    return VuiB200(VuiShape(), sd, device="cuda", tokenizer=StubTok())


def _codes(n, seed):
    return torch.randint(0, 2048, (n, 16), generator=torch.Generator().manual_seed(seed))


def _next_frame_logits(tts):
    """cb0 logits and hidden of one greedy decode step from the current position."""
    eng = tts.engine
    eng._apply_cfg(None, greedy=True)
    eng._g_codes_in[0] = _codes(1, 5)[0].cuda()
    off = tts.row.offset
    hidden, cb0, eos = eng._decode_step()
    out = hidden.clone(), cb0.clone(), eos.clone()
    eng._rewind_row(tts.row, off)
    return out


def test_save_kv_load_kv_round_trip(model_tok, tmp_path):
    """save_kv after a prompt prefill, load_kv into a FRESH engine: same position, identical next-frame
    hidden / logits (the K/V bytes are copied, not recomputed); the file has the reference's keys and
    per-layer (slots, T, kv heads, head_dim) tensors.  A file with another codebook count re-prefills."""
    from vui_b200.serving import TTSEngine

    a = TTSEngine(model_tok, max_seq=512).setup()
    a.set_conditioning(wps=1.5, sq=[0.1, 0.2, 0.3, 0.4, 0.5, 0.6])
    a.prefill_prompt([("A calm voice reads a short reference sentence.", _codes(40, 1))],
                     {"wps_score": 1.5, "sq_scores": [0.1, 0.2, 0.3, 0.4, 0.5, 0.6]})
    T = a.T
    assert T == 1 + 8 + 40 and a.prompt_T == T  # text + [SC] + codes
    want = _next_frame_logits(a)
    path = tmp_path / "voice.pt"
    a.save_kv(path, "voice")
    saved = torch.load(path, map_location="cpu", weights_only=False)
    assert set(saved) >= {"name", "codes", "text", "T", "n_q", "d_model", "checkpoint", "kv", "cond_bias", "spk_token_emb"}
    assert len(saved["kv"]) == 24 and saved["kv"][0]["k"].shape == (2, T, 8, 64) and saved["T"] == T
    assert saved["kv"][3]["v"].dtype == torch.bfloat16 and saved["cond_bias"].abs().max() > 0

    b = TTSEngine(model_tok, max_seq=512).setup()
    b.engine._cond_bias.zero_()
    assert b.load_kv(path) == "voice"
    assert b.T == T and b.prompt_T == T and b.row._prompt_offset == T
    assert torch.equal(b.prompt_codes, a.prompt_codes) and b.prompt_text == a.prompt_text
    assert torch.equal(b.engine._cond_bias, a.engine._cond_bias)
    got = _next_frame_logits(b)
    for x, y in zip(got, want):
        assert torch.equal(x, y)
    # stale file (other codebook count): the prompt is prefilled again from its codes, giving the same cache
    saved["n_q"] = 8
    saved["codes"] = saved["codes"][:, :8]
    torch.save(saved, tmp_path / "stale.pt")
    c = TTSEngine(model_tok, max_seq=512).setup()
    c.load_kv(tmp_path / "stale.pt")
    assert c.T == T and c.prompt_codes.shape == (40, 16) and (c.prompt_codes[:, 8:] == 0).all()
    # portable prompt: safetensors, always re-prefilled
    a.save_prompt(tmp_path / "voice.safetensors", "voice2")
    d = TTSEngine(model_tok, max_seq=512).setup()
    assert d.load_kv(tmp_path / "voice.safetensors") == "voice2"
    assert d.T == T
    got = _next_frame_logits(d)
    for x, y in zip(got, want):  # same prefill kernels on the same input: same bits
        assert torch.equal(x, y)
    with pytest.raises(ValueError):
        saved["d_model"] = 768
        torch.save(saved, tmp_path / "other.pt")
        d.load_kv(tmp_path / "other.pt")


def test_tts_process_command_loop(model_tok, tmp_path):
    """The protocol's commands through queues (worker in a thread): prompt upload, user turn, generate
    with its timing / codes / chunk_done / done events, cancel with rewind, save and load, state."""
    from vui_b200.serving import TTSEngine, tts_process

    cmd, out = queue.Queue(), queue.Queue()
    cancel = threading.Event()
    th = threading.Thread(target=tts_process, args=(cmd, out, lambda: TTSEngine(model_tok, max_seq=768).setup(), cancel),
                          daemon=True)
    th.start()

    def get(kind=None, timeout=120):
        while True:
            m = out.get(timeout=timeout)
            if kind is None or m["type"] == kind or m["type"] == "error":
                assert m["type"] != "error" or kind == "error", m
                return m

    assert get()["type"] == "ready"
    cmd.put({"cmd": "allocate_and_prefill", "codes": _codes(30, 2), "text": "This is the voice to clone.", "settings": {}})
    m = get("prompt_loaded")
    T_prompt = m["T"]
    assert T_prompt == 6 + 1 + 30 and m["text"] == "This is the voice to clone."
    cmd.put({"cmd": "prefill_user_turn", "text": "Hello, who is speaking?", "codes": _codes(12, 3)})
    T_user = get("user_prefilled")["T"]
    assert T_user == T_prompt + 4 + 1 + 12
    settings = {"temperature": 0.8, "top_k": 50, "max_duration": 2.0, "eos_threshold": 0.999, "chunk_words": 20}
    cmd.put({"cmd": "generate", "text": "I am a small test of the streaming path.", "settings": settings,
             "new_turn": True, "is_final": True})
    kinds, n_codes = [], 0
    while True:
        m = get()
        kinds.append(m["type"])
        if m["type"] == "codes":
            n_codes += 1
            assert m["data"].shape == (16,) and m["data"].max() < 2048
        if m["type"] == "done":
            done = m
            break
    assert kinds[0] == "timing" and "chunk_done" in kinds and n_codes == done["total_frames"] >= 1
    assert done["T"] > T_user
    cmd.put({"cmd": "get_state"})
    st = get("state")
    assert st["T"] == done["T"] and st["has_prompt"] and st["prompt_text"] == "This is the voice to clone."
    cmd.put({"cmd": "cancel", "rewind_to": T_user})
    cmd.put({"cmd": "get_state"})
    assert get("state")["T"] == T_user
    cmd.put({"cmd": "rewind"})
    assert get("done")["T"] == T_prompt
    cmd.put({"cmd": "save_kv", "name": "clone", "path": str(tmp_path / "clone.pt")})
    assert get("kv_saved")["ok"]
    cmd.put({"cmd": "reset"})
    assert get("done")["T"] == 0
    cmd.put({"cmd": "load_kv", "name": "clone", "path": str(tmp_path / "clone.pt")})
    m = get("kv_loaded")
    assert m["ok"] and m["T"] == T_prompt and m["text"] == "This is the voice to clone."
    cmd.put({"cmd": "prefill_text_sc", "text": "and then"})
    p = get("sc_prob")
    assert 0.0 <= p["prob"] <= 1.0 and p["T"] == T_prompt + 2
    cmd.put({"cmd": "no_such_command"})
    assert get("error")["type"] == "error"
    cmd.put({"cmd": "shutdown"})
    th.join(timeout=30)
    assert not th.is_alive()


def test_inference_state_and_stream_frames(model_tok):
    """The older single-stream API: prefill_prompt + checkpoint / rewind reuse the prompt's K/V; stream_frames
    yields (codes, turn_end) with the chunk info on a turn's last frame; with top_p tiny every cb0 is the
    arg-max of its distribution; the same seed gives the same frames; resume skips the prompt."""
    from vui_b200.inference import InferenceState, stream_frames

    st = InferenceState(model_tok, max_seq=768)
    prompt = [("The reference voice says this.", _codes(25, 4))]
    spk = torch.randn(1024, generator=torch.Generator().manual_seed(6))
    end = st.prefill_prompt(prompt, spk_emb=spk)
    assert end == 1 + 5 + 25 and st.checkpoint() == end  # [spk] text codes
    assert st.rewind(3) == 3 and st.rewind() == end

    def run(**kw):
        frames, ends = [], []
        g = torch.Generator(device="cuda").manual_seed(11)
        st.engine._ws_reset_counters()  # the depth draws are keyed by per-slot frame counters
        for codes, turn_end in stream_frames(st, "This first sentence has six words. Then a second one follows right here.", temperature=0.8,
                                             max_secs=3.0, max_turn_secs=1.2, eos_threshold=0.999, generator=g, **kw):
            assert codes.shape == (16,) and codes.is_cuda and 0 <= int(codes.min()) and int(codes.max()) < 2048
            frames.append(codes.cpu())
            ends.append(turn_end)
        return torch.stack(frames), ends

    st.rewind()
    a, ends = run(resume=True, top_k=50)
    turns = [e for e in ends if e is not None]
    assert len(turns) >= 2 and ends[-1] is not None and sum(t["frames"] for t in turns) == len(a)
    assert all(abs(t["secs"] - t["frames"] / 12.5) < 1e-9 for t in turns)
    assert st.offset > end
    st.rewind()
    b, _ = run(resume=True, top_k=50)
    assert torch.equal(a, b)  # seeded cb0 draws, depth draws keyed by the same frame counters
    # nucleus with a tiny p keeps only the most likely cb0 code: a greedy cb0 stream
    st.rewind()
    c, _ = run(resume=True, top_k=None, top_p=1e-6)
    st.rewind()
    d, _ = run(resume=True, top_k=1)
    assert torch.equal(c, d)
    # not resuming: reset + prompt prefill happen inside
    e, _ = run(prompt_segments=prompt, spk_emb=spk, top_k=50)
    assert e.shape[1] == 16 and len(e) >= 2


def test_conditioning_bias_and_speaker_token(model_tok, nano_sd):
    """set_conditioning (Vui.set_cond_bias, model.py:1258-1274) and the projected speaker token
    (model.py:1276-1278, engine.py:711-714) against the same projections written out in torch, and their
    effect on a prefill: the agent text carries the bias, the prompt text does not, the speaker token is
    one extra position in front of every segment."""
    from vui_b200 import Engine, Segment
    from vui_b200.text import simple_clean

    eng = Engine(model=model_tok, max_rows=1, max_seq=256)
    sd = model_tok.sd
    sq = (0.5, -0.25, 1.0, 0.0, 2.0, -1.0)
    eng.set_conditioning(sq_scores=sq, wps_score=2.5)
    want = torch.nn.functional.linear(torch.tensor([sq], dtype=torch.bfloat16, device="cuda"), sd["sq_proj.weight"])
    want = want.reshape(1, 1, -1).clone()
    want += torch.nn.functional.linear(torch.tensor([[2.5]], dtype=torch.bfloat16, device="cuda"),
                                       sd["wps_proj.proj.weight"]).reshape(1, 1, -1)
    assert torch.equal(eng._cond_bias, want) and eng._cond_bias.abs().max() > 0
    eng.set_conditioning(sq_scores=None, wps_score=0.0)
    assert eng._cond_bias.abs().max() == 0
    eng.set_conditioning(sq_scores=sq, wps_score=0.0)

    spk = torch.randn(1024, generator=torch.Generator().manual_seed(3))
    tok = eng._embed_speaker(spk)
    assert tok.shape == (1, 1, 1024)
    assert torch.equal(tok, torch.nn.functional.linear(spk.to("cuda", torch.bfloat16), sd["spk_proj.weight"]).reshape(1, 1, -1))
    row = eng.new_row()
    off = row.prefill([Segment("Reference text here.", _codes(10, 8))], spk_emb=spk)
    assert off == 1 + 3 + 1 + 10 and torch.equal(row._spk_token, tok)  # [spk] text [SC] codes
    # agent text: [spk] + text with the conditioning bias; compare with a hand-made prefill of the same rows
    h = eng._add_agent_text(row, "hello there")
    assert row.offset == off + 1 + 2
    eng2 = Engine(model=model_tok, max_rows=1, max_seq=256)
    r2 = eng2.new_row()
    ids = model_tok.text_tokenizer
    parts = [tok, model_tok.token_emb(ids.encode(simple_clean("Reference text here."))[None]).to(torch.bfloat16), eng._sc_emb,
             eng2._audio_emb(_codes(10, 8)), tok,
             model_tok.token_emb(ids.encode(simple_clean("hello there"))[None]).to(torch.bfloat16) + eng._cond_bias]
    out = None
    for p in parts:
        out = eng2._prefill_emb(r2, p)
    assert r2.offset == row.offset
    assert torch.equal(out[0, -1], h)
    # and the bias matters: without it the hidden differs
    eng2._rewind_row(r2, off + 1)
    out_nb = eng2._prefill_emb(r2, model_tok.token_emb(ids.encode(simple_clean("hello there"))[None]).to(torch.bfloat16))
    assert not torch.equal(out_nb[0, -1], h)
    # repetition-penalty state is readable the way the serving layer logs it
    eng._set_sampling(1.0, 1, 1, 1.3, 8, 0)
    eng._rep_reset()
    lg = torch.zeros(1, 2048, device="cuda", dtype=torch.bfloat16)
    lg[0, 77] = 3.0
    eng._sample_rows(lg, 3, cb0=True)
    cnt = eng._rep_counts
    assert cnt.shape == (1, 2048) and cnt.sum() == 3 and eng._rep_filled == 3
    eng._rep_reset()
    assert eng._rep_counts.sum() == 0


def test_torch_cuda_standin_computes_the_oracle_step(nano_sd):
    """The bench's many-stream baseline (oracle/torch_cuda_standin.py) is the oracle's algorithm, batched and
    captured in CUDA graphs: one step for three streams at different positions gives the oracle's hidden and
    cb0 logits, and valid codes."""
    from oracle.torch_cuda_standin import TorchGraphDecoder
    from oracle.vui_oracle import Oracle, OracleConfig

    cfg = OracleConfig()
    g = torch.Generator().manual_seed(5)
    o = Oracle(cfg, nano_sd, n_slots=3, max_seq=64, dtype=torch.bfloat16, device="cuda")
    lens = [7, 20, 33]
    for s_, n in enumerate(lens):
        o.prefill_text(s_, torch.randint(0, cfg.vocab, (n,), generator=g))
    dec = TorchGraphDecoder(cfg, nano_sd, 3, 64)
    dec.k_cache.copy_(o.k_cache)
    dec.v_cache.copy_(o.v_cache)
    dec.seq_lens.copy_(torch.tensor(lens))
    codes = torch.randint(0, 2048, (3, 16), generator=g)
    dec.codes.copy_(codes)
    dec.capture()
    dec.step()
    torch.cuda.synchronize()
    h, cb0, _ = o.backbone_step([0, 1, 2], codes)
    rel = lambda a, b: ((a.float() - b.float()).abs().max() / b.float().abs().max()).item()  # noqa: E731
    assert rel(dec.hidden, h) < 2e-2 and rel(dec.cb0, cb0) < 2e-2
    assert dec.seq_lens.tolist() == [n + 1 for n in lens]
    assert dec.codes.min() >= 0 and dec.codes.max() < 2048
