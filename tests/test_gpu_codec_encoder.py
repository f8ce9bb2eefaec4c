"""Codec encoder on the GPU (through the C ABI) against the reference-made fixture and the CPU oracle."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "codec_enc_fp32.pt")


@pytest.fixture(scope="module")
def efx():
    return torch.load(GOLDEN)


@pytest.fixture(scope="module")
def enc():
    from vui_b200.codec_encoder import QwenCodecEncoder

    return QwenCodecEncoder.random_init(0, device="cuda")


def codes_agree_up_to_near_ties(mine, ref, margin, tie=1e-3):
    cut = 0
    for t in range(ref.shape[1]):
        for q in range(ref.shape[0]):
            if int(mine[q, t]) != int(ref[q, t]):
                assert float(margin[q, t]) < tie, (q, t, int(mine[q, t]), int(ref[q, t]), float(margin[q, t]))
                cut += 1
                break
    return cut


def test_full_buffer_codes_and_latents_match_reference_fixture(enc, efx):
    from oracle.codec_enc_oracle import test_audio

    audio = test_audio(240000, seed=0)
    codes = enc(audio.cuda())[0].cpu()
    assert codes.shape == (16, 125) and codes.dtype == torch.int64
    lat = enc.read_latent(125)
    ref_lat = efx["latent"]
    # fp32 throughout: ~40 layers of convolutions and attention, summation order is the only difference
    assert (lat - ref_lat).abs().max().item() <= 2e-4 * ref_lat.abs().max().item()
    ref = efx["codes"].long()
    assert codes_agree_up_to_near_ties(codes, ref, efx["margin"]) <= 2
    assert (codes == ref).float().mean().item() > 0.98
    assert 0 <= codes.min() and codes.max() < 2048


def test_shorter_buffer_fewer_codebooks_and_bad_shapes(enc, efx):
    from oracle.codec_enc_oracle import test_audio

    audio = test_audio(240000, seed=0)
    n = efx["short"].shape[1]
    short = enc(audio[..., : n * 1920].cuda())[0].cpu()
    assert codes_agree_up_to_near_ties(short, efx["short"].long(), efx["margin"][:, :n]) <= 1
    enc.n_q = 4
    try:
        four = enc(audio[..., : n * 1920].cuda())[0].cpu()
        assert four.shape == (4, n) and torch.equal(four, short[:4])
    finally:
        enc.n_q = 16
    with pytest.raises(ValueError):
        enc(torch.zeros(1, 1, 1000).cuda())
    with pytest.raises(ValueError):
        enc(torch.zeros(1, 1, 240000 + 1920).cuda())


def test_streaming_encoder_reproduces_the_reference_trace(enc, efx):
    """Same chunks as the reference's StreamingCodecEncoder run: the same feeds return codes, and the codes are the
    reference's except at near ties (the fixture's margins cover the first 10 s buffer only, so later frames are held
    to the CPU oracle instead)."""
    from oracle.codec_enc_oracle import EncoderOracle, test_audio
    from vui_b200.codec_encoder import StreamingCodecEncoder, random_encoder_state

    st = efx["stream"]
    long_audio = test_audio(240000 + 60000, seed=2)[0, 0]
    for use_graph in (False, True):
        se = StreamingCodecEncoder(enc)
        if use_graph:
            se.setup_graph()
        pos, got = 0, []
        for n, ref in zip(st["sizes"], st["feeds"]):
            r = se.feed(long_audio[pos:pos + n])
            pos += n
            assert (r is None) == (ref is None)
            if r is not None:
                assert r.shape == ref.shape and r.dtype == torch.long
                got.append((r, ref.long()))
        tail = se.flush()
        assert (tail is None) == (st["flush"] is None)
        if tail is not None:
            got.append((tail, st["flush"].long()))
        mine = torch.cat([g[0] for g in got], dim=0)
        ref = torch.cat([g[1] for g in got], dim=0)
        assert mine.shape == ref.shape
        assert (mine == ref).float().mean().item() > 0.97
        if not use_graph:
            eager = mine
        else:
            assert torch.equal(mine, eager)          # graph replays compute the same codes
    # the second buffer (after the 10 s boundary) against the oracle on the same samples
    orc = EncoderOracle(random_encoder_state(0))
    second = torch.zeros(1, 1, 240000)
    second[0, 0, :60000] = long_audio[240000:]
    # the boundary falls where the reference trace reset its buffer: find it from the chunk sizes
    acc = 0
    for n in st["sizes"]:
        if acc + n > 240000:
            break
        acc += n
    second = torch.zeros(1, 1, 240000)
    rest = long_audio[acc:]
    second[0, 0, : rest.numel()] = rest
    want = orc.encode(second)[0]
    have = enc(second.cuda())[0].cpu()
    assert (have == want).float().mean().item() > 0.97


def test_serving_adapter_user_audio_commands(enc, nano_sd):
    """encode_full / stream_start / stream_feed / stream_flush / stream_stop and decode_prompt through the command
    queue, with this package's codec encoder and decoder attached (tts_worker.py:1404-1490, 1804-1878)."""
    import queue
    import threading
    import zlib

    from oracle.codec_enc_oracle import test_audio
    from vui_b200 import VuiB200, VuiShape
    from vui_b200.codec import QwenCodecDecoder
    from vui_b200.serving import TTSEngine, tts_process

    class StubTok:
        vocab_size = 151936

        def __init__(self):
            self.special_to_id = {"[SC]": 151900}

        def encode(self, text):
            return torch.tensor([zlib.crc32(w.encode()) % 151000 for w in text.split()] or [1], dtype=torch.long)

    model = VuiB200(VuiShape(), nano_sd, device="cuda", tokenizer=StubTok())
    dec = QwenCodecDecoder.random_init(0, device="cuda")
    cmd, out = queue.Queue(), queue.Queue()
    th = threading.Thread(target=tts_process, daemon=True,
                          args=(cmd, out, lambda: TTSEngine(model, codec_dec=dec, codec_enc=enc, max_seq=768).setup(),
                                threading.Event()))
    th.start()

    def get(kind, timeout=180):
        while True:
            m = out.get(timeout=timeout)
            assert m["type"] != "error", m
            if m["type"] == kind:
                return m

    get("ready")
    audio = test_audio(24000 * 4, seed=5)[0, 0]
    cmd.put({"cmd": "encode_full", "audio": audio.numpy()})
    full = get("encoded")["codes"]
    assert full.shape == (50, 16) and full.dtype == torch.long and 0 <= full.min() and full.max() < 2048
    cmd.put({"cmd": "stream_start"})
    pos, parts = 0, []
    for n in (9000, 30000, 20000, 37000):
        cmd.put({"cmd": "stream_feed", "audio": audio[pos:pos + n].numpy()})
        pos += n
    cmd.put({"cmd": "stream_flush"})
    cmd.put({"cmd": "stream_stop"})
    while True:
        m = out.get(timeout=180)
        assert m["type"] != "error", m
        if m["type"] == "codes":
            parts.append(m["codes"])
        if m["type"] == "codes_final":
            assert m["n_frames"] == 50
            break
    streamed = torch.cat(parts, dim=0)
    assert streamed.shape == (50, 16)
    assert (streamed == full).float().mean().item() > 0.97     # causal: streamed partials equal the full encode
    cmd.put({"cmd": "allocate_and_prefill", "codes": full[:30], "text": "the user said this", "settings": {}})
    get("prompt_loaded")
    cmd.put({"cmd": "decode_prompt"})
    m = get("prompt_audio")
    assert m["audio"].shape == (30 * 1920,) and m["sample_rate"] == 24000 and m["audio"].abs().max() <= 1
    cmd.put({"cmd": "shutdown"})
    th.join(timeout=60)
