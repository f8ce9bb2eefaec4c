"""The codec oracle against what the reference's own QwenCodecDecoder / CodecCtx computed
(tests/golden/codec_fp32.pt, made by tests/golden/make_codec_golden.py).  CPU only."""
import os

import pytest
import torch

from oracle.codec_oracle import CodecCtxOracle, CodecOracle
from vui_b200.codec import CodecCtx, codec_param_shapes, random_codec_state

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "codec_fp32.pt")
# the reference's streaming and offline forwards of the same codes differ by 1.9e-5 (fp32 summation order)
TOL = 1e-4


@pytest.fixture(scope="module")
def fx():
    return torch.load(GOLDEN)


@pytest.fixture(scope="module")
def oracle():
    return CodecOracle(random_codec_state(0))


def test_state_dict_names_cover_the_decoder():
    shapes = codec_param_shapes()
    assert len(shapes) == 255 and sum(torch.Size(s).numel() for s in shapes.values()) == 114290369
    sd = random_codec_state(0)
    assert list(sd) == list(shapes) and all(tuple(sd[k].shape) == shapes[k] for k in shapes)
    again = random_codec_state(0)
    assert all(torch.equal(sd[k], again[k]) for k in ("pre_conv.conv.weight", "decoder.6.conv.bias"))


def test_streaming_frames_match_reference(fx, oracle):
    oracle.reset()
    codes = fx["codes"]
    got = []
    for t in range(codes.shape[2]):
        got.append(oracle.decode(codes[:, :, t:t + 1]))
        if t == 2:
            for name, ref in fx["taps"].items():
                mine = oracle.taps[name][0, :, :64]
                assert mine.shape == ref.shape, name
                assert (mine - ref).abs().max() <= TOL * max(1.0, ref.abs().max().item()), name
    got = torch.cat(got, dim=-1)
    assert got.shape == fx["stream"].shape == (1, 1, 6 * 1920)
    assert (got - fx["stream"]).abs().max() <= TOL
    inside = fx["stream"].abs() < 1
    assert inside.float().mean() > 0.9          # the fixture is not a saturated signal


def test_offline_and_fewer_codebooks_match_reference(fx, oracle):
    assert (oracle.decode_offline(fx["codes"]) - fx["offline"]).abs().max() <= TOL
    oracle.reset()
    q8 = torch.cat([oracle.decode(fx["codes"][:, :8, t:t + 1]) for t in range(3)], dim=-1)
    assert (q8 - fx["stream_q8"]).abs().max() <= TOL
    assert (q8 - fx["stream"][..., : 3 * 1920]).abs().max() > 1e-2   # the other 8 codebooks matter


def test_ten_second_policy_matches_reference(fx, oracle):
    c = fx["ctx"]
    ctx = CodecCtxOracle(oracle, max_ctx_secs=0.4)
    ctx.set_prompt(c["prompt"])
    ctx.prefill()
    got, since = [], []
    for t in range(c["codes"].shape[2]):
        got.append(ctx.decode_frame(c["codes"][:, :, t:t + 1]))
        since.append(ctx.since)
    assert since == c["since"] == [3, 4, 5, 1, 2, 3, 4, 5, 1]
    assert (torch.cat(got, dim=-1) - c["audio"]).abs().max() <= TOL


class _CountingDecoder:
    """Stands in for the CUDA decoder: records what the product's CodecCtx asks of it."""

    def __init__(self):
        self.calls, self.resets = [], 0

    class _Ctx:
        def __init__(self, outer):
            self.o = outer

        def __enter__(self):
            self.o.resets += 1
            return self.o

        def __exit__(self, *a):
            return False

    def streaming(self, batch_size=1):
        return self._Ctx(self)

    def __call__(self, codes):
        self.calls.append(tuple(codes.shape))
        return torch.zeros(1, 1, codes.shape[2] * 1920)


def test_product_codec_ctx_follows_the_same_policy(fx):
    """vui_b200.codec.CodecCtx (host logic, no GPU needed) seeds, counts and resets like the reference's trace."""
    c = fx["ctx"]
    dec = _CountingDecoder()
    ctx = CodecCtx(dec, max_ctx_secs=0.4)
    assert ctx.max_ctx == 5
    ctx.set_prompt(c["prompt"])
    assert ctx.n_frames == 7 and ctx._stack is None
    ctx.prefill(n_codebooks=0)
    assert dec.calls == [(1, 16, 2)] and dec.resets == 1          # 7 % 5 = 2 seed frames
    since = []
    for t in range(9):
        a = ctx.decode_frame(c["codes"][:, :, t:t + 1])
        assert a.shape == (1, 1, 1920)
        since.append(ctx._frames_since_prefill)
    assert since == c["since"]
    assert dec.resets == 3                                        # prefill + two window boundaries
    assert ctx.n_frames == 10                                     # 7 + 9 trimmed to 2 * max_ctx, prompt kept
    assert torch.equal(ctx._buf[:, :, :7], c["prompt"])
    # offline rolling decode: context + new frames never exceed the window
    dec2 = _CountingDecoder()
    ctx2 = CodecCtx(dec2, max_ctx_secs=0.4)
    a = ctx2(c["codes"][:, :, :3])
    assert a.shape[-1] == 3 * 1920 and dec2.calls == [(1, 16, 3)]
    a = ctx2(c["codes"][:, :, 3:9])                               # 3 + 6 > 5 -> chunked with half-window context
    assert a.shape[-1] == 6 * 1920 and all(s[2] <= 5 for s in dec2.calls)
    ctx2.reset()
    assert ctx2.n_frames == 0 and ctx2._stack is None


# ---------------------------------------------------------------------------------------------- encoder
ENC_GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "codec_enc_fp32.pt")


@pytest.fixture(scope="module")
def efx():
    return torch.load(ENC_GOLDEN)


def codes_agree_up_to_near_ties(mine, ref, margin, tie=1e-3):
    """Per frame the codes must be identical from codebook 0 up to the first codebook whose two nearest codes are
    closer than `tie` in the reference (after such a flip the residual, hence every later codebook, differs).
    Returns the number of frames that end at a near tie."""
    cut = 0
    for t in range(ref.shape[1]):
        for q in range(ref.shape[0]):
            if int(mine[q, t]) != int(ref[q, t]):
                assert float(margin[q, t]) < tie, (q, t, int(mine[q, t]), int(ref[q, t]), float(margin[q, t]))
                cut += 1
                break
    return cut


def test_encoder_oracle_matches_reference(efx):
    from oracle.codec_enc_oracle import EncoderOracle, test_audio
    from vui_b200.codec_encoder import encoder_param_shapes, random_encoder_state

    shapes = encoder_param_shapes()
    assert len(shapes) == 161 and sum(torch.Size(s).numel() for s in shapes.values()) == 56168736
    orc = EncoderOracle(random_encoder_state(0))
    audio = test_audio(240000, seed=0)
    codes = orc.encode(audio)[0]
    assert codes.shape == (16, 125)
    ref = efx["codes"].long()
    assert (orc.latent - efx["latent"]).abs().max() <= 1e-4 * efx["latent"].abs().max()
    assert codes_agree_up_to_near_ties(codes, ref, efx["margin"]) <= 2
    assert (codes == ref).float().mean() > 0.98
    # causality: a shorter buffer gives the same first frames
    n = efx["short"].shape[1]
    assert codes_agree_up_to_near_ties(orc.encode(audio[..., : n * 1920])[0], efx["short"].long(), efx["margin"][:, :n]) <= 1


class _StubEncoder:
    """Counts frames: code value = frame index, so a trace shows which frames each feed returned."""

    n_q = 16

    def __init__(self):
        self.calls = 0

    def parameters(self):
        return iter([torch.zeros(1)])

    def __call__(self, buf):
        self.calls += 1
        T = buf.shape[-1] // 1920
        return torch.arange(T).view(1, 1, T).expand(1, self.n_q, T).clone()


def test_product_streaming_encoder_follows_the_reference_protocol(efx):
    """vui_b200.codec_encoder.StreamingCodecEncoder (host logic, no GPU): same chunks in, the same feeds return the
    same number of frames at the same frame indices as the reference's trace, across the 10 s boundary."""
    from vui_b200.codec_encoder import StreamingCodecEncoder

    st = efx["stream"]
    se = StreamingCodecEncoder(_StubEncoder())
    assert se.max_samples == 240000 and se.max_frames == 125 and se.min_chunk_samples == 12 * 1920
    first_frame = 0
    for n, ref in zip(st["sizes"], st["feeds"]):
        if se._pos + n > se.max_samples:
            first_frame = 0                       # the buffer restarts at the boundary
        got = se.feed(torch.zeros(n))
        assert (got is None) == (ref is None)
        if got is not None:
            assert got.shape == ref.shape and got.dtype == torch.long
            assert got[:, 0].tolist() == list(range(first_frame, first_frame + got.shape[0]))
            first_frame += got.shape[0]
    tail = se.flush()
    assert (tail is None) == (st["flush"] is None)
    if tail is not None:
        assert tail.shape == st["flush"].shape
    se.reset()
    assert se._pos == 0 and se._emitted == 0 and se.feed(torch.zeros(0)) is None
