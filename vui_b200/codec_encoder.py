"""Codec encoder (24 kHz audio -> codes) on libvuib200's encoder kernels, behind the names the reference uses:
``QwenCodecEncoder`` (src/vui/qwen_codec.py:368-407) and ``StreamingCodecEncoder`` (671-805), which the
serving side uses to turn a user's speech into the codec frames of a user turn.

The encoder keeps the reference module's state-dict keys.  ``StreamingCodecEncoder`` keeps the reference's
protocol: a fixed 10 s buffer that is re-encoded from its start on every ``feed`` that completes enough frames
(all layers are causal, so the zeros behind the write position do not change earlier frames), a hard reset at the
10 s boundary, ``flush`` for the ragged tail.  fp32, one stream, no CPU fallback.
"""

from __future__ import annotations

import ctypes as C
from collections import OrderedDict

import torch
from torch import Tensor

from . import _lib
from .codec import DOWNSAMPLE_RATE, N_CODEBOOKS, SAMPLE_RATE

RATIOS, BASE_DIM, D_MODEL, N_LAYERS, N_HEADS, MLP = (4, 5, 6, 8), 64, 512, 8, 8, 2048


def encoder_param_shapes() -> "OrderedDict[str, tuple]":
    """Names and shapes of the encoder's state dict in the reference module's registration order
    (qwen_codec.py:293-311, 314-365, 368-383)."""
    s: "OrderedDict[str, tuple]" = OrderedDict()
    p = "conv_encoder.layers."
    s[p + "0.conv.weight"], s[p + "0.conv.bias"] = (BASE_DIM, 1, 7), (BASE_DIM,)
    dim, idx = BASE_DIM, 1
    for r in RATIOS:
        s[f"{p}{idx}.block.1.conv.weight"], s[f"{p}{idx}.block.1.conv.bias"] = (dim // 2, dim, 3), (dim // 2,)
        s[f"{p}{idx}.block.3.conv.weight"], s[f"{p}{idx}.block.3.conv.bias"] = (dim, dim // 2, 1), (dim,)
        s[f"{p}{idx + 2}.conv.weight"], s[f"{p}{idx + 2}.conv.bias"] = (2 * dim, dim, 2 * r), (2 * dim,)
        dim, idx = 2 * dim, idx + 3
    s[f"{p}{idx + 1}.conv.weight"], s[f"{p}{idx + 1}.conv.bias"] = (D_MODEL, dim, 3), (D_MODEL,)
    for l in range(N_LAYERS):
        q = f"transformer.layers.{l}."
        s[q + "attn_scale"] = (D_MODEL,)
        s[q + "mlp_scale"] = (D_MODEL,)
        s[q + "input_layernorm.weight"] = (D_MODEL,)
        s[q + "input_layernorm.bias"] = (D_MODEL,)
        for n in ("q_proj", "k_proj", "v_proj", "o_proj"):
            s[q + n + ".weight"] = (D_MODEL, D_MODEL)
        s[q + "post_attention_layernorm.weight"] = (D_MODEL,)
        s[q + "post_attention_layernorm.bias"] = (D_MODEL,)
        s[q + "fc1.weight"] = (MLP, D_MODEL)
        s[q + "fc2.weight"] = (D_MODEL, MLP)
    s["downsample.conv.weight"] = (D_MODEL, D_MODEL, 4)
    for part, n in (("semantic", 1), ("acoustic", 31)):
        s[f"quantizer.{part}.input_proj.weight"] = (256, 512, 1)
        s[f"quantizer.{part}.output_proj.weight"] = (512, 256, 1)
        for i in range(n):
            s[f"quantizer.{part}.codebooks.{i}.embed"] = (2048, 256)
    return s


def random_encoder_state(seed: int = 0) -> "OrderedDict[str, Tensor]":
    """Seeded random weights with every path live (the module's own init leaves layer scales and codebooks at 0):
    matrices ~ N(0, 1/fan_in), layer scales around 0.5, norm weights around 1, codebooks ~ N(0, 1)."""
    g = torch.Generator().manual_seed(seed)
    out: "OrderedDict[str, Tensor]" = OrderedDict()
    for name, shape in encoder_param_shapes().items():
        leaf = name.rsplit(".", 1)[-1]
        if leaf == "embed":
            t = torch.randn(shape, generator=g)
        elif leaf in ("attn_scale", "mlp_scale"):
            t = 0.5 + 0.1 * torch.randn(shape, generator=g)
        elif leaf == "bias":
            t = torch.randn(shape, generator=g) * 0.05
        elif len(shape) == 1:
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        else:
            fan_in = 1
            for d in shape[1:]:
                fan_in *= d
            gain = 4.0 if name.endswith("input_proj.weight") else 1.0   # latents on the codebooks' scale
            t = torch.randn(shape, generator=g) * gain * (1.0 / fan_in) ** 0.5
        out[name] = t
    return out


class QwenCodecEncoder:
    """Audio (1, 1, T) float at 24 kHz -> codes (1, n_q, T // 1920) int64."""

    def __init__(self, state_dict: dict, device="cuda", max_secs: float = 10.0):
        if not torch.cuda.is_available():
            raise RuntimeError("vui_b200.codec_encoder needs a CUDA device: there is no CPU path")
        self.device = torch.device(device)
        self.n_q = N_CODEBOOKS
        self.max_samples = (int(max_secs * SAMPLE_RATE) // DOWNSAMPLE_RATE) * DOWNSAMPLE_RATE
        self._lib = _lib.load()
        shapes = encoder_param_shapes()
        for k, shp in shapes.items():
            if k not in state_dict:
                raise KeyError(f"encoder state dict lacks {k}")
            if tuple(state_dict[k].shape) != shp:
                raise ValueError(f"{k}: expected {shp}, got {tuple(state_dict[k].shape)}")
        sd = {k: state_dict[k].detach().to(self.device, torch.float32).contiguous() for k in shapes}
        self._keep: list[Tensor] = []
        cfg = _lib.VuibCodecEncConfig(BASE_DIM, (C.c_int32 * 4)(*RATIOS), D_MODEL, N_LAYERS, N_HEADS, MLP, self.max_samples)
        self._h = C.c_void_p()
        self._check(self._lib.vuib_codec_enc_create(C.byref(cfg), C.byref(self._h)))
        n = C.c_size_t()
        self._check(self._lib.vuib_codec_enc_workspace_bytes(self._h, C.byref(n)))
        self._ws = torch.zeros(n.value, dtype=torch.uint8, device=self.device)
        self._check(self._lib.vuib_codec_enc_bind_workspace(self._h, self._ws.data_ptr(), n.value))
        self._w = self._pack(sd)
        self._check(self._lib.vuib_codec_enc_bind_weights(self._h, C.byref(self._w)))

    @classmethod
    def random_init(cls, seed: int = 0, device="cuda") -> "QwenCodecEncoder":
        return cls(random_encoder_state(seed), device=device)

    def _check(self, rc: int) -> None:
        if rc != 0:
            buf = C.create_string_buffer(256)
            self._lib.vuib_codec_enc_last_error(self._h, buf, 256)
            raise _lib.VuibError(rc, buf.value.decode(errors="replace") or "(no message)")

    def _p(self, t: Tensor) -> int:
        t = t.contiguous()
        self._keep.append(t)
        return t.data_ptr()

    def _pack(self, sd: dict) -> "_lib.VuibCodecEncWeights":
        w, P = _lib.VuibCodecEncWeights(), self._p
        conv = lambda pre: _lib.VuibConvW(P(sd[pre + ".weight"]), P(sd[pre + ".bias"]))  # noqa: E731
        p = "conv_encoder.layers."
        w.conv_in = conv(p + "0.conv")
        idx = 1
        for i in range(4):
            w.res[i].c3, w.res[i].c1 = conv(f"{p}{idx}.block.1.conv"), conv(f"{p}{idx}.block.3.conv")
            w.down[i] = conv(f"{p}{idx + 2}.conv")
            idx += 3
        w.conv_out = conv(f"{p}{idx + 1}.conv")
        for l in range(N_LAYERS):
            q, lw = f"transformer.layers.{l}.", w.layer[l]
            lw.ln1_w, lw.ln1_b = P(sd[q + "input_layernorm.weight"]), P(sd[q + "input_layernorm.bias"])
            lw.wqkv = P(torch.cat([sd[q + n + ".weight"] for n in ("q_proj", "k_proj", "v_proj")], dim=0))
            lw.wo = P(sd[q + "o_proj.weight"])
            lw.attn_scale, lw.mlp_scale = P(sd[q + "attn_scale"]), P(sd[q + "mlp_scale"])
            lw.ln2_w, lw.ln2_b = P(sd[q + "post_attention_layernorm.weight"]), P(sd[q + "post_attention_layernorm.bias"])
            lw.fc1, lw.fc2 = P(sd[q + "fc1.weight"]), P(sd[q + "fc2.weight"])
        # RoPE.forward (qwen_codec.py:161-171) for every 25 Hz frame of the buffer
        inv = 1.0 / (10000.0 ** (torch.arange(0, 64, 2, dtype=torch.float32, device=self.device) / 64))
        fr = torch.outer(torch.arange(self.max_samples // 960, device=self.device, dtype=torch.float32), inv)
        emb = torch.cat([fr, fr], dim=-1)
        w.rope_cos, w.rope_sin = P(emb.cos()), P(emb.sin())
        w.downsample = P(sd["downsample.conv.weight"])
        w.sem_in = P(sd["quantizer.semantic.input_proj.weight"].reshape(256, 512))
        w.acq_in = P(sd["quantizer.acoustic.input_proj.weight"].reshape(256, 512))
        books = [sd["quantizer.semantic.codebooks.0.embed"]] + [sd[f"quantizer.acoustic.codebooks.{i}.embed"] for i in range(15)]
        for i, e in enumerate(books):
            w.codebook[i] = P(e)
            w.codebook_norm2[i] = P((e * e).sum(dim=1))
        return w

    def forward(self, x: Tensor) -> Tensor:
        if x.dim() != 3 or x.shape[0] != 1 or x.shape[1] != 1:
            raise ValueError(f"audio must be (1, 1, T), got {tuple(x.shape)}")
        T = x.shape[2]
        if T % DOWNSAMPLE_RATE or not 0 < T <= self.max_samples:
            raise ValueError(f"T = {T}: need a multiple of {DOWNSAMPLE_RATE} up to {self.max_samples}")
        audio = x.to(self.device, torch.float32).contiguous()
        codes = torch.empty(self.n_q, T // DOWNSAMPLE_RATE, dtype=torch.int64, device=self.device)
        self._check(self._lib.vuib_codec_enc_encode(self._h, audio.data_ptr(), T, self.n_q, codes.data_ptr(),
                                                    torch.cuda.current_stream(self.device).cuda_stream))
        return codes.unsqueeze(0)

    __call__ = forward
    encode = forward

    def read_latent(self, n_frames: int) -> Tensor:
        """(512, n_frames) latents before quantisation of the last call, for parity tests."""
        buf = (C.c_float * (512 * n_frames))()
        self._check(self._lib.vuib_codec_enc_read_latent(self._h, buf, 512 * n_frames,
                                                         torch.cuda.current_stream(self.device).cuda_stream))
        return torch.tensor(list(buf), dtype=torch.float32).view(512, n_frames)

    def launch_count(self) -> int:
        return int(self._lib.vuib_codec_enc_launch_count(self._h))

    def parameters(self):
        return iter(self._keep)

    def eval(self):
        return self

    def __del__(self):
        try:
            if getattr(self, "_h", None) and self._h.value:
                self._lib.vuib_codec_enc_destroy(self._h)
                self._h = C.c_void_p()
        except Exception:
            pass


class StreamingCodecEncoder:
    """feed(audio chunk) -> new code frames or None; flush() for the tail; reset().  The buffer restarts empty at
    the 10 s boundary because training audio was encoded in independent 10 s chunks (qwen_codec.py:714-723)."""

    def __init__(self, encoder, n_quantizers: int = N_CODEBOOKS, max_secs: float = 10, min_chunk_frames: int = 12):
        self.encoder = encoder
        self.encoder.n_q = n_quantizers
        self.device = next(iter(encoder.parameters())).device
        self.n_q = n_quantizers
        self.max_samples = (int(max_secs * SAMPLE_RATE) // DOWNSAMPLE_RATE) * DOWNSAMPLE_RATE
        self.max_frames = self.max_samples // DOWNSAMPLE_RATE
        self.min_chunk_samples = min_chunk_frames * DOWNSAMPLE_RATE
        self.dtype = torch.float32
        self._audio_buf = torch.zeros(1, 1, self.max_samples, device=self.device, dtype=self.dtype)
        self._pos = 0
        self._emitted = 0
        self._graph = None
        self._codes_out = None

    def _slide(self) -> None:
        self._audio_buf.zero_()
        self._pos = 0
        self._emitted = 0

    def setup_graph(self) -> None:
        """Capture the whole-buffer encode once; feed()/flush() then replay it (qwen_codec.py:725-736)."""
        with torch.inference_mode():
            self.encoder(self._audio_buf)
            torch.cuda.synchronize()
            self._graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph):
                self._codes_out = self.encoder(self._audio_buf)

    def _encode(self) -> Tensor:
        if self._graph is not None:
            self._graph.replay()
            return self._codes_out
        return self.encoder(self._audio_buf)

    @torch.inference_mode()
    def feed(self, audio: Tensor):
        audio = audio.detach().flatten()
        n = len(audio)
        if n == 0:
            return None
        space = self.max_samples - self._pos
        if n > space:
            self._slide()
            n = min(n, self.max_samples)
        if n == 0:
            return None
        self._audio_buf[0, 0, self._pos: self._pos + n].copy_(audio[:n].to(device=self.device, dtype=self.dtype))
        self._pos += n
        n_frames = self._pos // DOWNSAMPLE_RATE
        if n_frames <= self._emitted or (self._pos - self._emitted * DOWNSAMPLE_RATE) < self.min_chunk_samples:
            return None
        new = self._encode()[0, :, self._emitted: n_frames].T.long().cpu()
        self._emitted = n_frames
        return new

    @torch.inference_mode()
    def flush(self):
        rem = self._pos % DOWNSAMPLE_RATE
        if rem > 0:
            self._pos += DOWNSAMPLE_RATE - rem   # the buffer is already zero beyond the write position
        n_frames = self._pos // DOWNSAMPLE_RATE
        if n_frames <= self._emitted:
            return None
        new = self._encode()[0, :, self._emitted: n_frames].T.long().cpu()
        self._emitted = n_frames
        return new

    def reset(self) -> None:
        self._slide()
