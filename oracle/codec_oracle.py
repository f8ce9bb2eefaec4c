"""CPU restatement of the reference's streaming codec decode (codes -> audio), fp32.

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by bench.py's CPU baseline leg;
the product (vui_b200/) never imports it.

Pinned: tests/golden/codec_fp32.pt holds what the reference's own QwenCodecDecoder / CodecCtx classes
(src/vui/qwen_codec.py) compute on CPU for seeded weights and codes (tests/golden/make_codec_golden.py);
tests/test_codec_oracle.py holds this file to those vectors.

Every function names the reference lines it follows.  State is explicit (a dict), layers are plain
torch.nn.functional calls on the reference's state-dict tensors.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor

DOWNSAMPLE_RATE = 1920
FRAME_RATE = 12.5
RATES = (8, 5, 4, 3)
DILATIONS = (1, 3, 9)


def snake_beta(x: Tensor, alpha: Tensor, beta: Tensor) -> Tensor:
    """SnakeBeta.forward, qwen_codec.py:826-829."""
    a = alpha[None, :, None].exp()
    b = beta[None, :, None].exp()
    return x + (1.0 / (b + 1e-9)) * torch.sin(x * a).pow(2)


def rms_norm(x: Tensor, w: Tensor, eps: float = 1e-6) -> Tensor:
    """RMSNorm.forward, qwen_codec.py:813-817."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


class CodecOracle:
    def __init__(self, sd: dict, max_seq: int = 250):
        self.sd = {k: v.detach().float().cpu() for k, v in sd.items()}
        self.max_seq = max_seq
        inv = 1.0 / (10000.0 ** (torch.arange(0, 64, 2, dtype=torch.float32) / 64))   # RoPE, qwen_codec.py:161-171
        fr = torch.outer(torch.arange(max_seq, dtype=torch.float32), inv)
        emb = torch.cat([fr, fr], dim=-1)
        self.cos, self.sin = emb.cos(), emb.sin()
        self.taps: dict[str, Tensor] = {}
        self.reset()

    # -- state: what _init_streaming_state creates (qwen_codec.py:74-90, 122-138, 1011-1032)
    def reset(self) -> None:
        self.prev: dict[str, Tensor] = {}      # CausalConv1d history, created lazily as zeros
        self.partial: dict[str, Tensor] = {}   # CausalTransConv1d trailing partial
        self.k = [torch.zeros(1, 16, self.max_seq, 64) for _ in range(8)]
        self.v = [torch.zeros(1, 16, self.max_seq, 64) for _ in range(8)]
        self.pos = 0

    def _conv(self, name: str, x: Tensor, dilation: int = 1, groups: int = 1) -> Tensor:
        """CausalConv1d.forward, streaming branch, qwen_codec.py:92-102."""
        w, b = self.sd[name + ".conv.weight"], self.sd[name + ".conv.bias"]
        pad = (w.shape[2] - 1) * dilation
        if pad > 0:
            prev = self.prev.get(name)
            if prev is None:
                prev = torch.zeros(x.shape[0], x.shape[1], pad)
            x = torch.cat([prev, x], dim=-1)
            self.prev[name] = x[..., -pad:].clone()
        return F.conv1d(x, w, b, dilation=dilation, groups=groups)

    def _trconv(self, name: str, x: Tensor, stride: int) -> Tensor:
        """CausalTransConv1d.forward, streaming branch, qwen_codec.py:140-158."""
        w, b = self.sd[name + ".conv.weight"], self.sd[name + ".conv.bias"]
        y = F.conv_transpose1d(x, w, b, stride=stride)
        pt = w.shape[2] - stride
        if pt > 0:
            part = self.partial.get(name)
            if part is None:
                part = torch.zeros(y.shape[0], y.shape[1], pt)
            y = y.clone()
            y[..., :pt] = y[..., :pt] + part
            self.partial[name] = y[..., -pt:] - b[:, None]
            y = y[..., :-pt]
        return y

    def _quantizer(self, codes: Tensor) -> Tensor:
        """SplitResidualVQ.decode / ResidualVQ.decode, qwen_codec.py:231-238, 263-271."""
        out = None
        for part, cs in (("semantic", codes[:, :1]), ("acoustic", codes[:, 1:])):
            if cs.shape[1] == 0:
                continue
            q = torch.zeros(1)
            for i in range(cs.shape[1]):
                q = q + F.embedding(cs[:, i], self.sd[f"quantizer.{part}.codebooks.{i}.embed"]).transpose(1, 2)
            y = F.conv1d(q, self.sd[f"quantizer.{part}.output_proj.weight"])
            out = y if out is None else out + y
        return out

    def _transformer(self, x: Tensor) -> Tensor:
        """DecTransformer._forward_streaming + DecTransformerBlock.forward, qwen_codec.py:1048-1076, 940-974."""
        sd, T = self.sd, x.shape[1]
        p = "pre_transformer."
        x = F.linear(x, sd[p + "input_proj.weight"], sd[p + "input_proj.bias"])
        idx = torch.arange(self.pos, self.pos + T)
        cos, sin = self.cos[idx][None, None], self.sin[idx][None, None]
        mask = (torch.arange(self.max_seq)[None, :] <= idx[:, None]).view(1, 1, T, self.max_seq)

        def rot(t):
            a, b = t.chunk(2, dim=-1)
            return torch.cat((-b, a), dim=-1)

        for l in range(8):
            q_ = f"{p}layers.{l}."
            h = rms_norm(x, sd[q_ + "input_layernorm.weight"])
            q = F.linear(h, sd[q_ + "q_proj.weight"]).view(1, T, 16, 64).transpose(1, 2)
            k = F.linear(h, sd[q_ + "k_proj.weight"]).view(1, T, 16, 64).transpose(1, 2)
            v = F.linear(h, sd[q_ + "v_proj.weight"]).view(1, T, 16, 64).transpose(1, 2)
            q, k = q * cos + rot(q) * sin, k * cos + rot(k) * sin
            self.k[l][:, :, idx] = k
            self.v[l][:, :, idx] = v
            a = F.scaled_dot_product_attention(q, self.k[l], self.v[l], attn_mask=mask)
            a = a.transpose(1, 2).reshape(1, T, -1)
            x = x + sd[q_ + "attn_scale"] * F.linear(a, sd[q_ + "o_proj.weight"])
            h = rms_norm(x, sd[q_ + "post_attention_layernorm.weight"])
            x = x + sd[q_ + "mlp_scale"] * F.linear(
                F.silu(F.linear(h, sd[q_ + "gate_proj.weight"])) * F.linear(h, sd[q_ + "up_proj.weight"]),
                sd[q_ + "down_proj.weight"])
        self.pos += T
        return F.linear(rms_norm(x, sd[p + "norm.weight"]), sd[p + "output_proj.weight"], sd[p + "output_proj.bias"])

    def _convnext(self, p: str, x: Tensor) -> Tensor:
        """ConvNeXtBlock.forward, qwen_codec.py:841-848."""
        sd = self.sd
        h = self._conv(p + "dwconv", x, groups=x.shape[1]).transpose(1, 2)
        h = F.layer_norm(h, (h.shape[-1],), sd[p + "norm.weight"], sd[p + "norm.bias"], eps=1e-6)
        h = F.gelu(F.linear(h, sd[p + "pwconv1.weight"], sd[p + "pwconv1.bias"]))
        h = sd[p + "gamma"] * F.linear(h, sd[p + "pwconv2.weight"], sd[p + "pwconv2.bias"])
        return x + h.transpose(1, 2)

    def decode(self, codes: Tensor) -> Tensor:
        """QwenCodecDecoder._streaming_forward_body + _vocoder_chain, qwen_codec.py:1191-1224: (1, n_q, T) codes
        continue the streaming state and give (1, 1, T * 1920) samples."""
        sd = self.sd
        h = self._quantizer(codes)
        self.taps["quantizer"] = h
        h = self._conv("pre_conv", h).transpose(1, 2)
        h = self._transformer(h).transpose(1, 2)
        self.taps["transformer"] = h
        for i in range(2):
            h = self._trconv(f"upsample.{i}.0", h, 2)
            h = self._convnext(f"upsample.{i}.1.", h)
        self.taps["upsampled"] = h
        h = self._conv("decoder.0", h)
        self.taps["decoder0"] = h
        for b, rate in enumerate(RATES):            # DecoderBlock / DecoderResUnit, qwen_codec.py:851-879
            p = f"decoder.{b + 1}.block."
            h = snake_beta(h, sd[p + "0.alpha"], sd[p + "0.beta"])
            h = self._trconv(p + "1", h, rate)
            for r, d in enumerate(DILATIONS):
                q = f"{p}{r + 2}."
                y = self._conv(q + "conv1", snake_beta(h, sd[q + "act1.alpha"], sd[q + "act1.beta"]), dilation=d)
                h = h + self._conv(q + "conv2", snake_beta(y, sd[q + "act2.alpha"], sd[q + "act2.beta"]))
            self.taps[f"block{b + 1}"] = h
        h = snake_beta(h, sd["decoder.5.alpha"], sd["decoder.5.beta"])
        return self._conv("decoder.6", h).clamp(-1, 1)

    def decode_offline(self, codes: Tensor) -> Tensor:
        """QwenCodecDecoder.forward outside a streaming context (qwen_codec.py:1199-1215): zero left padding,
        transposed convolutions trimmed on the right, causal attention — the same function as a fresh stream."""
        self.reset()
        return self.decode(codes)


class CodecCtxOracle:
    """CodecCtx's streaming policy (qwen_codec.py:558-657) over a CodecOracle: seed with n_frames % max_ctx frames,
    start cold every max_ctx frames."""

    def __init__(self, dec: CodecOracle, max_ctx_secs: float = 10.0):
        self.dec, self.max_ctx = dec, int(max_ctx_secs * FRAME_RATE)
        self.buf: Tensor | None = None
        self.prompt_len = 0
        self.active = False
        self.since = 0

    def set_prompt(self, codes: Tensor) -> None:
        self.buf, self.prompt_len, self.active = codes, codes.shape[2], False

    def _append(self, codes: Tensor) -> None:
        self.buf = codes if self.buf is None else torch.cat([self.buf, codes], dim=2)
        limit = 2 * self.max_ctx
        if self.buf.shape[2] > limit:
            if 0 < self.prompt_len < limit:
                self.buf = torch.cat([self.buf[:, :, : self.prompt_len], self.buf[:, :, -(limit - self.prompt_len):]], 2)
            else:
                self.buf = self.buf[:, :, -limit:]

    def prefill(self, n_codebooks: int = 0) -> None:
        self.dec.reset()
        self.active = True
        n = 0 if self.buf is None else self.buf.shape[2] % self.max_ctx
        if n:
            seed = self.buf[:, :, -n:]
            self.dec.decode(seed[:, :n_codebooks] if n_codebooks > 0 else seed)
        self.since = n

    def decode_frame(self, codes: Tensor, store_codes: Tensor | None = None) -> Tensor:
        if not self.active or self.since >= self.max_ctx:
            self.dec.reset()
            self.active, self.since = True, 0
        audio = self.dec.decode(codes)
        self._append(codes if store_codes is None else store_codes)
        self.since += 1
        return audio
