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
