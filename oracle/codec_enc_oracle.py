"""CPU restatement of the reference's codec encoder (audio -> codes), fp32.

TEST INFRASTRUCTURE ONLY: imported by tests/ and by bench.py's CPU baseline leg; the product never imports it.

Pinned: tests/golden/codec_enc_fp32.pt holds what the reference's own QwenCodecEncoder / StreamingCodecEncoder
(src/vui/qwen_codec.py) compute on CPU for seeded weights and audio (tests/golden/make_codec_enc_golden.py);
tests/test_codec_oracle.py holds this file to those vectors.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor

RATIOS = (4, 5, 6, 8)


def test_audio(n_samples: int, seed: int = 0) -> Tensor:
    """Seeded test signal (1, 1, n): two tones plus noise, amplitude about 0.3."""
    g = torch.Generator().manual_seed(seed)
    t = torch.arange(n_samples, dtype=torch.float32) / 24000.0
    x = 0.2 * torch.sin(2 * torch.pi * 220.0 * t) + 0.1 * torch.sin(2 * torch.pi * 1370.0 * t + 0.5)
    return (x + 0.05 * torch.randn(n_samples, generator=g)).view(1, 1, -1)


def causal_conv(x: Tensor, w: Tensor, b: Tensor | None, stride: int = 1) -> Tensor:
    """CausalConv1d.forward outside streaming, qwen_codec.py:92-98: left zero padding of (kernel - stride)."""
    return F.conv1d(F.pad(x, (w.shape[2] - stride, 0)), w, b, stride=stride)


class EncoderOracle:
    def __init__(self, sd: dict):
        self.sd = {k: v.detach().float().cpu() for k, v in sd.items()}
        self.latent: Tensor | None = None

    def conv_encoder(self, x: Tensor) -> Tensor:
        """ConvEncoder.forward / ResBlock.forward, qwen_codec.py:278-311."""
        sd, p = self.sd, "conv_encoder.layers."
        c = lambda name, t, s=1: causal_conv(t, sd[name + ".conv.weight"], sd[name + ".conv.bias"], s)  # noqa: E731
        x = c(p + "0", x)
        idx = 1
        for r in RATIOS:
            x = x + c(f"{p}{idx}.block.3", F.elu(c(f"{p}{idx}.block.1", F.elu(x))))
            x = c(f"{p}{idx + 2}", F.elu(x), r)
            idx += 3
        return c(f"{p}{idx + 1}", F.elu(x))

    def transformer(self, x: Tensor) -> Tensor:
        """EncTransformer.forward / EncTransformerBlock.forward, qwen_codec.py:314-365; x (1, T, 512)."""
        sd, T = self.sd, x.shape[1]
        inv = 1.0 / (10000.0 ** (torch.arange(0, 64, 2, dtype=torch.float32) / 64))
        fr = torch.outer(torch.arange(T, dtype=torch.float32), inv)
        emb = torch.cat([fr, fr], dim=-1)
        cos, sin = emb.cos()[None, None], emb.sin()[None, None]

        def rot(t):
            a, b = t.chunk(2, dim=-1)
            return torch.cat((-b, a), dim=-1)

        for l in range(8):
            q_ = f"transformer.layers.{l}."
            h = F.layer_norm(x, (512,), sd[q_ + "input_layernorm.weight"], sd[q_ + "input_layernorm.bias"], eps=1e-5)
            q, k, v = (F.linear(h, sd[q_ + n + ".weight"]).view(1, T, 8, 64).transpose(1, 2) for n in ("q_proj", "k_proj", "v_proj"))
            q, k = q * cos + rot(q) * sin, k * cos + rot(k) * sin
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(1, T, 512)
            x = x + sd[q_ + "attn_scale"] * F.linear(a, sd[q_ + "o_proj.weight"])
            h = F.layer_norm(x, (512,), sd[q_ + "post_attention_layernorm.weight"], sd[q_ + "post_attention_layernorm.bias"], eps=1e-5)
            x = x + sd[q_ + "mlp_scale"] * F.linear(F.gelu(F.linear(h, sd[q_ + "fc1.weight"])), sd[q_ + "fc2.weight"])
        return x

    def rvq(self, part: str, h: Tensor, n: int) -> Tensor:
        """ResidualVQ.encode / EuclideanCodebook.encode, qwen_codec.py:190-195, 218-229; h (1, 512, T)."""
        sd = self.sd
        res = F.conv1d(h, sd[f"quantizer.{part}.input_proj.weight"]).float()[0].T   # (T, 256)
        out = []
        for i in range(n):
            emb = sd[f"quantizer.{part}.codebooks.{i}.embed"]
            idx = torch.cdist(res.unsqueeze(0), emb.unsqueeze(0)).squeeze(0).argmin(dim=-1)
            res = res - emb[idx]
            out.append(idx)
        return torch.stack(out, dim=0)

    def encode(self, audio: Tensor, n_q: int = 16) -> Tensor:
        """QwenCodecEncoder.forward, qwen_codec.py:385-390: (1, 1, T) -> (1, n_q, T // 1920)."""
        h = self.conv_encoder(audio)
        h = self.transformer(h.transpose(1, 2)).transpose(1, 2)
        h = causal_conv(h, self.sd["downsample.conv.weight"], None, 2)
        self.latent = h[0]
        codes = [self.rvq("semantic", h, 1)]
        if n_q > 1:
            codes.append(self.rvq("acoustic", h, n_q - 1))
        return torch.cat(codes, dim=0).unsqueeze(0)
