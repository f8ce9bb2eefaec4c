"""Streaming codec decode on the GPU (through the C ABI) against the reference-made fixture and the CPU oracle."""
import os
import zlib

import pytest
import torch

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "codec_fp32.pt")
# fp32 throughout; the reference's own streaming and offline forwards differ by 1.9e-5 on this fixture
TOL = 2e-4


@pytest.fixture(scope="module")
def fx():
    return torch.load(GOLDEN)


@pytest.fixture(scope="module")
def sd():
    from vui_b200.codec import random_codec_state

    return random_codec_state(0)


@pytest.fixture(scope="module")
def dec(sd):
    from vui_b200.codec import QwenCodecDecoder

    return QwenCodecDecoder(sd, device="cuda")


@pytest.fixture(scope="module")
def oracle(sd):
    from oracle.codec_oracle import CodecOracle

    return CodecOracle(sd)


class StubTok:
    """Deterministic word-hash tokenizer with the attributes Engine reads."""

    vocab_size = 151936

    def __init__(self):
        self.special_to_id = {"[SC]": 151900}

    def encode(self, text: str):
        ids = [zlib.crc32(w.encode()) % 151000 for w in text.split()]
        return torch.tensor(ids or [1], dtype=torch.long)


TAPS = {"quantizer": (0, 512, 1), "transformer": (1, 1024, 1), "upsampled": (2, 1024, 4), "decoder0": (3, 1536, 4),
        "block1": (4, 768, 32), "block2": (5, 384, 160), "block3": (6, 192, 640), "block4": (7, 96, 1920)}


def test_streamed_frames_and_taps_match_reference_fixture(dec, fx):
    codes = fx["codes"].cuda()
    got = []
    with dec.streaming(1):
        for t in range(6):
            got.append(dec(codes[:, :, t:t + 1]).cpu())
            if t == 2:
                for name, (which, C, T) in TAPS.items():
                    mine = dec.read_tap(which, C * T).view(C, T)[:, :64]
                    ref = fx["taps"][name]
                    assert mine.shape == ref.shape, name
                    err = (mine - ref).abs().max().item()
                    assert err <= TOL * max(1.0, ref.abs().max().item()), (name, err)
        assert dec.position() == 6
    got = torch.cat(got, dim=-1)
    assert got.shape == (1, 1, 6 * 1920)
    assert (got - fx["stream"]).abs().max().item() <= TOL
    dec.check_device()


def test_offline_forward_and_fewer_codebooks(dec, fx):
    a = dec(fx["codes"].cuda()).cpu()                      # not streaming: starts from zero padding
    assert (a - fx["offline"]).abs().max().item() <= TOL
    with dec.streaming(1):
        q8 = torch.cat([dec(fx["codes"][:, :8, t:t + 1].cuda()).cpu() for t in range(3)], dim=-1)
    assert (q8 - fx["stream_q8"]).abs().max().item() <= TOL
    assert dec.decode is not None and dec.decode_chunked(fx["codes"].cuda(), chunk_size=4, ctx=2).shape[-1] == 6 * 1920


def test_codec_ctx_policy_on_the_gpu_matches_reference_fixture(dec, fx):
    from vui_b200.codec import CodecCtx

    c = fx["ctx"]
    ctx = CodecCtx(dec, max_ctx_secs=0.4)
    ctx.set_prompt(c["prompt"].cuda())
    ctx.prefill()
    assert dec.position() == 2
    got, since = [], []
    for t in range(9):
        got.append(ctx.decode_frame(c["codes"][:, :, t:t + 1].cuda()).cpu())
        since.append(ctx._frames_since_prefill)
    assert since == c["since"]
    assert (torch.cat(got, dim=-1) - c["audio"]).abs().max().item() <= TOL
    ctx.reset()
    assert not dec.is_streaming


def test_long_stream_vs_oracle_and_graph_replay_is_identical(dec, oracle):
    g = torch.Generator().manual_seed(7)
    codes = torch.randint(0, 2048, (1, 16, 40), generator=g)
    oracle.reset()
    ref = torch.cat([oracle.decode(codes[:, :, t:t + 1]) for t in range(40)], dim=-1)
    with dec.streaming(1):
        eager = torch.cat([dec(codes[:, :, t:t + 1].cuda()) for t in range(40)], dim=-1).cpu()
    assert (eager - ref).abs().max().item() <= TOL
    assert (eager.abs() < 1).float().mean() > 0.85
    launches = dec.launch_count()
    dec.setup_streaming_graph()
    try:
        with dec.streaming(1):
            replay = torch.cat([dec(codes[:, :, t:t + 1].cuda()) for t in range(40)], dim=-1).cpu()
        assert torch.equal(replay, eager)                  # same kernels, same order, same bits
        assert dec.launch_count() - launches <= 3 * 100    # the frames themselves were graph replays
    finally:
        dec._use_graph = False


def test_bad_code_is_clamped_and_flagged_and_window_is_enforced(dec):
    from vui_b200 import _lib

    codes = torch.full((1, 16, 1), 5, dtype=torch.long)
    codes[0, 3, 0] = 4096
    with dec.streaming(1):
        a = dec(codes.cuda())
        assert torch.isfinite(a).all()
        with pytest.raises(_lib.VuibError, match="code outside"):
            dec.check_device()
        dec.check_device()                                  # cleared
        with pytest.raises(ValueError, match="positions"):
            dec(torch.zeros(1, 16, 251, dtype=torch.long).cuda())
    with pytest.raises(ValueError):
        dec(torch.zeros(2, 16, 1, dtype=torch.long).cuda())
    with pytest.raises(ValueError):
        dec(torch.zeros(1, 17, 1, dtype=torch.long).cuda())


def test_engine_streams_audio_through_the_codec(dec, nano_sd):
    from vui_b200 import Engine, GenConfig, Segment, VuiB200, VuiShape
    model = VuiB200(VuiShape(), nano_sd, device="cuda", tokenizer=StubTok())
    eng = Engine(model=model, codec=dec, max_rows=1, max_seq=1024)
    cfg = GenConfig(temperature=0.8, top_k=50, max_secs=1.0, eos_threshold=0.999)
    with eng.new_row() as row:
        prompt = torch.randint(0, 2048, (9, 16), generator=torch.Generator().manual_seed(3))
        row.prefill([Segment("A short prompt.", prompt)])
        assert row._codec_ctx is not None and row._codec_ctx.n_frames == 9
        frames = list(row.stream("Hello there, this is streaming audio.", cfg))
        assert 1 <= len(frames) <= 13
        for a in frames:
            assert a.shape == (1, 1, 1920) and a.dtype == torch.float32 and a.abs().max() <= 1
        assert row._codec_ctx.n_frames == 9 + len(frames)
        assert dec.position() == 9 + len(frames)            # 9 seed frames, then one position per frame
        codes, audio = row.render("And this is the offline path.", cfg)
        assert audio is not None and audio.shape[-1] == codes.shape[0] * 1920
    dec.check_device()


def test_codec_on_second_stream_yields_the_same_audio(dec, nano_sd):
    """Row.stream with overlap_codec: frame k's audio is decoded beside the generation of frame k + 1; the frames
    handed out are the same tensors in the same order as without the overlap."""
    from vui_b200 import Engine, GenConfig, Segment, VuiB200, VuiShape

    model = VuiB200(VuiShape(), nano_sd, device="cuda", tokenizer=StubTok())
    cfg = GenConfig(temperature=0.8, top_k=50, max_secs=1.0, eos_threshold=0.999)
    prompt = torch.randint(0, 2048, (9, 16), generator=torch.Generator().manual_seed(3))
    outs = []
    for overlap in (False, True):
        eng = Engine(model=model, codec=dec, max_rows=1, max_seq=1024, seed=11)
        eng.overlap_codec = overlap
        with eng.new_row() as row:
            row.prefill([Segment("A short prompt.", prompt)])
            outs.append(torch.cat([a.cpu() for a in row.stream("Hello there, this is streaming audio.", cfg)], dim=-1))
    assert outs[0].shape == outs[1].shape and outs[0].shape[-1] >= 1920
    assert torch.equal(outs[0], outs[1])
    dec.check_device()
