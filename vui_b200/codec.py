"""Streaming codec decode (codes -> 24 kHz audio) on libvuib200's codec kernels, behind the names the
reference uses: ``QwenCodecDecoder`` (src/vui/qwen_codec.py:1079-1276) and ``CodecCtx`` (410-668).

The decoder keeps the reference module's state-dict keys, so a state dict saved from the reference's
``QwenCodecDecoder`` loads unchanged.  One frame (16 codes -> 1920 samples) is one call of
``vuib_codec_decode_frame``; longer inputs are fed frame by frame, which for a causal model is the same
function as the reference's batched forward.  fp32 only (the reference's default, engine.py:302), one stream.
There is no CPU fallback.
"""

from __future__ import annotations

import ctypes as C
from collections import OrderedDict
from contextlib import contextmanager

import torch
from torch import Tensor

from . import _lib

SAMPLE_RATE = 24000
DOWNSAMPLE_RATE = 1920
FRAME_RATE = SAMPLE_RATE / DOWNSAMPLE_RATE  # 12.5
N_CODEBOOKS = 16

LATENT, D_MODEL, N_LAYERS, N_HEADS, HEAD_DIM, MLP = 1024, 512, 8, 16, 64, 1024
DEC_DIM, RATES, DILATIONS = 1536, (8, 5, 4, 3), (1, 3, 9)


def codec_param_shapes() -> "OrderedDict[str, tuple]":
    """Names and shapes of the decoder's state dict, in the reference module's registration order
    (qwen_codec.py:1080-1125 and the classes it instantiates)."""
    s: "OrderedDict[str, tuple]" = OrderedDict()
    for part, n in (("semantic", 1), ("acoustic", 15)):
        s[f"quantizer.{part}.input_proj.weight"] = (256, 512, 1)
        s[f"quantizer.{part}.output_proj.weight"] = (512, 256, 1)
        for i in range(n):
            s[f"quantizer.{part}.codebooks.{i}.embed"] = (2048, 256)
    s["pre_conv.conv.weight"] = (LATENT, 512, 3)
    s["pre_conv.conv.bias"] = (LATENT,)
    s["pre_transformer.input_proj.weight"] = (D_MODEL, LATENT)
    s["pre_transformer.input_proj.bias"] = (D_MODEL,)
    for l in range(N_LAYERS):
        p = f"pre_transformer.layers.{l}."
        s[p + "attn_scale"] = (D_MODEL,)
        s[p + "mlp_scale"] = (D_MODEL,)
        s[p + "input_layernorm.weight"] = (D_MODEL,)
        for n in ("q_proj", "k_proj", "v_proj"):
            s[p + n + ".weight"] = (N_HEADS * HEAD_DIM, D_MODEL)
        s[p + "o_proj.weight"] = (D_MODEL, N_HEADS * HEAD_DIM)
        s[p + "post_attention_layernorm.weight"] = (D_MODEL,)
        s[p + "gate_proj.weight"] = (MLP, D_MODEL)
        s[p + "up_proj.weight"] = (MLP, D_MODEL)
        s[p + "down_proj.weight"] = (D_MODEL, MLP)
    s["pre_transformer.norm.weight"] = (D_MODEL,)
    s["pre_transformer.output_proj.weight"] = (LATENT, D_MODEL)
    s["pre_transformer.output_proj.bias"] = (LATENT,)
    for i in range(2):
        p = f"upsample.{i}."
        s[p + "0.conv.weight"] = (LATENT, LATENT, 2)
        s[p + "0.conv.bias"] = (LATENT,)
        s[p + "1.gamma"] = (LATENT,)
        s[p + "1.dwconv.conv.weight"] = (LATENT, 1, 7)
        s[p + "1.dwconv.conv.bias"] = (LATENT,)
        s[p + "1.norm.weight"] = (LATENT,)
        s[p + "1.norm.bias"] = (LATENT,)
        s[p + "1.pwconv1.weight"] = (4 * LATENT, LATENT)
        s[p + "1.pwconv1.bias"] = (4 * LATENT,)
        s[p + "1.pwconv2.weight"] = (LATENT, 4 * LATENT)
        s[p + "1.pwconv2.bias"] = (LATENT,)
    s["decoder.0.conv.weight"] = (DEC_DIM, LATENT, 7)
    s["decoder.0.conv.bias"] = (DEC_DIM,)
    dim = DEC_DIM
    for b, rate in enumerate(RATES):
        out, p = dim // 2, f"decoder.{b + 1}.block."
        s[p + "0.alpha"] = (dim,)
        s[p + "0.beta"] = (dim,)
        s[p + "1.conv.weight"] = (dim, out, 2 * rate)
        s[p + "1.conv.bias"] = (out,)
        for r in range(3):
            q = f"{p}{r + 2}."
            s[q + "act1.alpha"] = (out,)
            s[q + "act1.beta"] = (out,)
            s[q + "conv1.conv.weight"] = (out, out, 7)
            s[q + "conv1.conv.bias"] = (out,)
            s[q + "act2.alpha"] = (out,)
            s[q + "act2.beta"] = (out,)
            s[q + "conv2.conv.weight"] = (out, out, 1)
            s[q + "conv2.conv.bias"] = (out,)
        dim = out
    s["decoder.5.alpha"] = (dim,)
    s["decoder.5.beta"] = (dim,)
    s["decoder.6.conv.weight"] = (1, dim, 7)
    s["decoder.6.conv.bias"] = (1,)
    return s


def random_codec_state(seed: int = 0) -> "OrderedDict[str, Tensor]":
    """Seeded random weights with every path live (the module's own init leaves the transformer's layer
    scales at 0, the ConvNeXt gammas at 1e-6 and the codebooks at 0, so its output would not depend on most
    weights): matrices ~ N(0, 1/fan_in) (a quarter of that deviation for the residual branches' last
    convolution and the output convolution, so that the audio stays inside the clamp), layer scales and gammas around 0.5, SnakeBeta logs ~ N(0, 0.3),
    codebooks ~ N(0, 1).  Used for parity tests and benchmarks; no released checkpoint is involved."""
    g = torch.Generator().manual_seed(seed)
    out: "OrderedDict[str, Tensor]" = OrderedDict()
    for name, shape in codec_param_shapes().items():
        leaf = name.rsplit(".", 1)[-1]
        if leaf == "embed":
            t = torch.randn(shape, generator=g)
        elif leaf in ("alpha", "beta"):
            t = torch.randn(shape, generator=g) * 0.3
        elif leaf in ("attn_scale", "mlp_scale", "gamma"):
            t = 0.5 + 0.1 * torch.randn(shape, generator=g)
        elif leaf == "bias":
            t = torch.randn(shape, generator=g) * 0.05
        elif len(shape) == 1:  # norm weights
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        else:
            if ".block.1.conv.weight" in name or "upsample" in name and name.endswith("0.conv.weight"):
                fan_in = shape[0] * (2 if ".block.1." in name else 1)  # transposed: (in, out, k), two taps overlap
            else:
                fan_in = 1
                for d in shape[1:]:
                    fan_in *= d
            gain = 0.25 if ("conv2.conv.weight" in name or name == "decoder.6.conv.weight") else 1.0
            t = torch.randn(shape, generator=g) * gain * (1.0 / fan_in) ** 0.5
        out[name] = t
    return out


class QwenCodecDecoder:
    """Codes (1, n_q, T) int64 -> audio (1, 1, T * 1920) fp32 in [-1, 1]."""

    def __init__(self, state_dict: dict, device="cuda", max_seq: int = 250):
        if not torch.cuda.is_available():
            raise RuntimeError("vui_b200.codec needs a CUDA device: there is no CPU path")
        self.device = torch.device(device)
        self.max_seq = int(max_seq)
        self._lib = _lib.load()
        shapes = codec_param_shapes()
        missing = [k for k in shapes if k not in state_dict]
        if missing:
            raise KeyError(f"codec state dict lacks {len(missing)} tensors, e.g. {missing[:3]}")
        for k, shp in shapes.items():
            if tuple(state_dict[k].shape) != shp:
                raise ValueError(f"{k}: expected {shp}, got {tuple(state_dict[k].shape)}")
        sd = {k: state_dict[k].detach().to(self.device, torch.float32).contiguous() for k in shapes}
        self._keep: list[Tensor] = []
        cfg = _lib.VuibCodecConfig(16, 2048, 256, 512, LATENT, D_MODEL, N_LAYERS, N_HEADS, MLP, self.max_seq, DEC_DIM,
                                   (C.c_int32 * 4)(*RATES), 1e-6)
        self._h = C.c_void_p()
        self._check(self._lib.vuib_codec_create(C.byref(cfg), C.byref(self._h)))
        n = C.c_size_t()
        self._check(self._lib.vuib_codec_workspace_bytes(self._h, C.byref(n)))
        self._ws = torch.zeros(n.value, dtype=torch.uint8, device=self.device)
        self._check(self._lib.vuib_codec_bind_workspace(self._h, self._ws.data_ptr(), n.value))
        self._w = self._pack(sd)
        self._check(self._lib.vuib_codec_bind_weights(self._h, C.byref(self._w)))
        self._codes_in = torch.zeros(N_CODEBOOKS, dtype=torch.int64, device=self.device)
        self._audio = torch.zeros(DOWNSAMPLE_RATE, dtype=torch.float32, device=self.device)
        self._graphs: dict[int, torch.cuda.CUDAGraph] = {}
        self._streaming = False
        self._use_graph = False
        self.reset_streaming()

    # ------------------------------------------------------------------ construction helpers
    @classmethod
    def from_state_dict(cls, state_dict: dict, device="cuda", max_seq: int = 250) -> "QwenCodecDecoder":
        return cls(state_dict, device=device, max_seq=max_seq)

    @classmethod
    def random_init(cls, seed: int = 0, device="cuda") -> "QwenCodecDecoder":
        return cls(random_codec_state(seed), device=device)

    @classmethod
    def from_pretrained(cls, path: str, device="cuda") -> "QwenCodecDecoder":
        """Load a state dict saved from the reference's ``QwenCodecDecoder`` (``.pt`` or ``.safetensors``).
        The reference's own ``from_pretrained`` downloads the tokenizer weights; there is no network here."""
        if path.endswith(".safetensors"):
            from safetensors.torch import load_file

            sd = load_file(path)
        else:
            sd = torch.load(path, map_location="cpu")
        return cls(sd, device=device)

    def _check(self, rc: int) -> None:
        if rc != 0:
            buf = C.create_string_buffer(256)
            self._lib.vuib_codec_last_error(self._h, buf, 256)
            raise _lib.VuibError(rc, buf.value.decode(errors="replace") or "(no message)")

    def _p(self, t: Tensor) -> int:
        t = t.contiguous()
        self._keep.append(t)
        return t.data_ptr()

    def _pack(self, sd: dict) -> "_lib.VuibCodecWeights":
        w = _lib.VuibCodecWeights()
        P = self._p

        def conv(prefix: str, reshape=None) -> "_lib.VuibConvW":
            wt = sd[prefix + ".weight"]
            return _lib.VuibConvW(P(wt if reshape is None else reshape(wt)), P(sd[prefix + ".bias"]))

        def snake(prefix: str) -> "_lib.VuibSnakeW":
            # SnakeBeta.forward (qwen_codec.py:826-829): a = exp(alpha), 1 / (exp(beta) + 1e-9)
            return _lib.VuibSnakeW(P(sd[prefix + ".alpha"].exp()), P(1.0 / (sd[prefix + ".beta"].exp() + 1e-9)))

        def rows_of_transposed(wt: Tensor) -> Tensor:   # (Cin, Cout, K) -> rows (co, k) over ci
            return wt.permute(1, 2, 0).reshape(wt.shape[1] * wt.shape[2], wt.shape[0])

        def tiles_of_rows(wt: Tensor) -> Tensor:        # (rows, Cin, taps) -> [rows / 96][Cin][taps][96]
            rows, cin, taps = wt.shape
            return wt.reshape(rows // 96, 96, cin, taps).permute(0, 2, 3, 1)

        w.codebook[0] = P(sd["quantizer.semantic.codebooks.0.embed"])
        for i in range(15):
            w.codebook[1 + i] = P(sd[f"quantizer.acoustic.codebooks.{i}.embed"])
        w.sem_proj = P(sd["quantizer.semantic.output_proj.weight"].reshape(512, 256))
        w.acq_proj = P(sd["quantizer.acoustic.output_proj.weight"].reshape(512, 256))
        w.pre_conv = conv("pre_conv.conv")
        w.in_proj = conv("pre_transformer.input_proj")
        for l in range(N_LAYERS):
            p = f"pre_transformer.layers.{l}."
            lw = w.layer[l]
            lw.ln1 = P(sd[p + "input_layernorm.weight"])
            lw.wqkv = P(torch.cat([sd[p + "q_proj.weight"], sd[p + "k_proj.weight"], sd[p + "v_proj.weight"]], 0))
            lw.wo = P(sd[p + "o_proj.weight"])
            lw.attn_scale = P(sd[p + "attn_scale"])
            lw.ln2 = P(sd[p + "post_attention_layernorm.weight"])
            lw.gate, lw.up, lw.down = P(sd[p + "gate_proj.weight"]), P(sd[p + "up_proj.weight"]), P(sd[p + "down_proj.weight"])
            lw.mlp_scale = P(sd[p + "mlp_scale"])
        w.norm = P(sd["pre_transformer.norm.weight"])
        w.out_proj = conv("pre_transformer.output_proj")
        # RoPE.forward (qwen_codec.py:161-171), fp32 tables for every position of the fixed cache
        inv = 1.0 / (10000.0 ** (torch.arange(0, HEAD_DIM, 2, dtype=torch.float32, device=self.device) / HEAD_DIM))
        fr = torch.outer(torch.arange(self.max_seq, device=self.device, dtype=torch.float32), inv)
        emb = torch.cat([fr, fr], dim=-1)
        w.rope_cos, w.rope_sin = P(emb.cos()), P(emb.sin())
        for i in range(2):
            p, st = f"upsample.{i}.", w.stage[i]
            st.up = conv(p + "0.conv", rows_of_transposed)
            st.dw = conv(p + "1.dwconv.conv", lambda t: t.reshape(LATENT, 7))
            st.ln_w, st.ln_b = P(sd[p + "1.norm.weight"]), P(sd[p + "1.norm.bias"])
            st.pw1, st.pw2 = conv(p + "1.pwconv1"), conv(p + "1.pwconv2")
            st.gamma = P(sd[p + "1.gamma"])
        w.dec_in = conv("decoder.0.conv")
        for b in range(4):
            p, bw = f"decoder.{b + 1}.block.", w.block[b]
            bw.act = snake(p + "0")
            # block 0 runs on the row kernel (rows (co, k) over ci); the others on the tiled kernel
            bw.up = conv(p + "1.conv", rows_of_transposed if b == 0 else
                         (lambda t: tiles_of_rows(rows_of_transposed(t).unsqueeze(-1))))
            for r in range(3):
                q, rw = f"{p}{r + 2}.", bw.res[r]
                rw.act1, rw.conv1 = snake(q + "act1"), conv(q + "conv1.conv", tiles_of_rows)
                rw.act2, rw.conv2 = snake(q + "act2"), conv(q + "conv2.conv", tiles_of_rows)
        w.final_act = snake("decoder.5")
        w.final_conv = conv("decoder.6.conv", lambda t: t.reshape(t.shape[1], 7))
        return w

    # ------------------------------------------------------------------ streaming state
    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def reset_streaming(self) -> None:
        """Fresh state for every causal layer (zero histories and partials, transformer position 0)."""
        self._check(self._lib.vuib_codec_reset(self._h, self._stream()))

    @contextmanager
    def streaming(self, batch_size: int = 1):
        """``with decoder.streaming(1):`` — state starts fresh and then carries over between calls
        (StreamingModule.streaming, src/vui/streaming.py:72-83)."""
        if batch_size != 1:
            raise ValueError("the streaming codec decodes one stream")
        self.reset_streaming()
        self._streaming = True
        try:
            yield self
        finally:
            self._streaming = False

    @property
    def is_streaming(self) -> bool:
        return self._streaming

    def position(self) -> int:
        pos = C.c_int32()
        self._check(self._lib.vuib_codec_position(self._h, C.byref(pos), self._stream()))
        return pos.value

    def check_device(self) -> None:
        self._check(self._lib.vuib_codec_check_flag(self._h, self._stream()))

    def setup_streaming_graph(self, batch_size: int = 1, device=None, dtype=None, pool=None) -> None:
        """From now on single frames replay a captured CUDA graph (one per codebook count), as
        QwenCodecDecoder.setup_streaming_graph arranges (qwen_codec.py:1138-1189)."""
        if batch_size != 1:
            raise ValueError("the streaming codec decodes one stream")
        if dtype not in (None, torch.float32):
            raise ValueError("the codec kernels are fp32")
        self._use_graph = True
        self._graph_for(N_CODEBOOKS)
        self.reset_streaming()

    def _graph_for(self, n_q: int) -> "torch.cuda.CUDAGraph":
        g = self._graphs.get(n_q)
        if g is None:
            s = torch.cuda.Stream(self.device)
            s.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(s):   # a first plain call sets the kernels' attributes outside the capture
                self._check(self._lib.vuib_codec_decode_frame(self._h, self._codes_in.data_ptr(), n_q,
                                                              self._audio.data_ptr(), s.cuda_stream))
            torch.cuda.current_stream(self.device).wait_stream(s)
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._check(self._lib.vuib_codec_decode_frame(self._h, self._codes_in.data_ptr(), n_q,
                                                              self._audio.data_ptr(), self._stream()))
            self._graphs[n_q] = g
        return g

    # ------------------------------------------------------------------ decode
    def _frame(self, codes_q: Tensor, out: Tensor) -> None:
        n_q = codes_q.shape[0]
        self._codes_in[:n_q].copy_(codes_q)
        if self._use_graph:
            self._graph_for(n_q).replay()
            out.copy_(self._audio)
        else:
            self._check(self._lib.vuib_codec_decode_frame(self._h, self._codes_in.data_ptr(), n_q, out.data_ptr(),
                                                          self._stream()))

    def forward(self, codes: Tensor) -> Tensor:
        if codes.dim() == 2:
            codes = codes.unsqueeze(0)
        if codes.dim() != 3 or codes.shape[0] != 1:
            raise ValueError(f"codes must be (1, n_q, T), got {tuple(codes.shape)}")
        n_q, T = codes.shape[1], codes.shape[2]
        if not 1 <= n_q <= N_CODEBOOKS:
            raise ValueError(f"n_q = {n_q} outside [1, {N_CODEBOOKS}]")
        codes = codes.to(self.device, torch.int64)
        if not self._streaming:
            self.reset_streaming()   # an offline forward starts from zero padding (qwen_codec.py:92-102)
            start = 0
        else:
            start = self.position() if T > 1 else None
        if start is not None and start + T > self.max_seq:
            raise ValueError(f"{start} + {T} frames exceed the codec transformer's {self.max_seq} positions; "
                             "decode in windows (CodecCtx does)")
        audio = torch.empty(1, 1, T * DOWNSAMPLE_RATE, dtype=torch.float32, device=self.device)
        for t in range(T):
            self._frame(codes[0, :, t], audio[0, 0, t * DOWNSAMPLE_RATE:(t + 1) * DOWNSAMPLE_RATE])
        return audio

    __call__ = forward
    decode = forward

    def decode_chunked(self, codes: Tensor, chunk_size: int = 300, ctx: int = 25) -> Tensor:
        """Long offline decode in windows with `ctx` frames of left context (qwen_codec.py:1229-1261 decodes
        chunks of 300 frames; here a window may not exceed the transformer's fixed cache)."""
        if codes.dim() == 2:
            codes = codes.unsqueeze(0)
        T = codes.shape[2]
        step = max(1, min(chunk_size, self.max_seq - ctx))
        outs, pos = [], 0
        while pos < T:
            lo = max(0, pos - ctx)
            end = min(T, pos + step)
            a = self.forward(codes[:, :, lo:end])
            outs.append(a[..., (pos - lo) * DOWNSAMPLE_RATE:])
            pos = end
        return torch.cat(outs, dim=-1) if outs else torch.zeros(1, 1, 0, device=self.device)

    def read_tap(self, which: int, n: int) -> Tensor:
        buf = (C.c_float * n)()
        self._check(self._lib.vuib_codec_read_tap(self._h, which, buf, n, self._stream()))
        return torch.tensor(list(buf), dtype=torch.float32)

    def launch_count(self) -> int:
        return int(self._lib.vuib_codec_launch_count(self._h))

    def new_ctx(self, max_ctx_secs: float = 10.0) -> "CodecCtx":
        return CodecCtx(self, max_ctx_secs)

    def parameters(self):
        return iter(self._keep)

    def eval(self):
        return self

    def __del__(self):
        try:
            if getattr(self, "_h", None) and self._h.value:
                self._lib.vuib_codec_destroy(self._h)
                self._h = C.c_void_p()
        except Exception:
            pass


class CodecCtx:
    """Rolling code buffer plus the 10-second policy of the streaming decode (qwen_codec.py:410-668): codes are
    kept for context, the decoder is seeded with ``n_frames % max_ctx`` frames when a session starts and starts
    cold again every ``max_ctx`` frames, because training audio was encoded in independent 10 s chunks."""

    def __init__(self, decoder: QwenCodecDecoder, max_ctx_secs: float = 10.0):
        self.decoder = decoder
        self.max_ctx = int(max_ctx_secs * FRAME_RATE)
        self._prompt_len = 0
        self._buf: Tensor | None = None
        self._stack = None                 # the open streaming context, None while no session is active
        self._frames_since_prefill = 0
        self._prefill_n_codebooks = 0

    # ---- buffer
    def set_prompt(self, codes: Tensor) -> None:
        if codes.dim() == 2:
            codes = codes.unsqueeze(0)
        self._prompt_len = codes.shape[2]
        self._buf = codes
        self._close_stack()

    def add(self, codes: Tensor) -> None:
        if codes.dim() == 2:
            codes = codes.unsqueeze(0)
        self._append(codes)

    @property
    def n_frames(self) -> int:
        return 0 if self._buf is None else self._buf.shape[2]

    def _window(self, buf: Tensor, limit: int) -> Tensor:
        """At most `limit` frames: the prompt first, then the newest frames."""
        if buf.shape[2] <= limit:
            return buf
        if 0 < self._prompt_len < limit:
            return torch.cat([buf[:, :, : self._prompt_len], buf[:, :, -(limit - self._prompt_len):]], dim=2)
        return buf[:, :, -limit:]

    def get_context(self, max_frames: int | None = None) -> Tensor | None:
        if self._buf is None:
            return None
        return self._window(self._buf, max_frames or self.max_ctx)

    def _append(self, codes: Tensor) -> None:
        if self._buf is None:
            self._buf = codes
        else:
            if codes.shape[1] != self._buf.shape[1]:   # a stale prompt with another codebook count
                q = min(codes.shape[1], self._buf.shape[1])
                self._buf, codes = self._buf[:, :q].contiguous(), codes[:, :q].contiguous()
            self._buf = torch.cat([self._buf, codes.to(self._buf.device)], dim=2)
        self._buf = self._window(self._buf, 2 * self.max_ctx)

    # ---- offline decode with rolling context
    @torch.inference_mode()
    def __call__(self, codes: Tensor) -> Tensor:
        if codes.dim() == 2:
            codes = codes.unsqueeze(0)
        ctx = self.get_context()
        n_ctx = 0 if ctx is None else ctx.shape[2]
        if n_ctx + codes.shape[2] > self.max_ctx:
            return self._decode_chunked(codes)
        inp = codes if ctx is None else torch.cat([ctx.to(codes.device), codes], dim=2)
        audio = self.decoder(inp)
        self._append(codes)
        return audio[..., n_ctx * DOWNSAMPLE_RATE:]

    def _decode_chunked(self, codes: Tensor) -> Tensor:
        ctx = self.get_context(self.max_ctx // 2)
        T, pos, wavs = codes.shape[2], 0, []
        while pos < T:
            n_ctx = 0 if ctx is None else ctx.shape[2]
            end = min(pos + self.max_ctx - n_ctx, T)
            chunk = codes[:, :, pos:end]
            inp = chunk if ctx is None else torch.cat([ctx.to(chunk.device), chunk], dim=2)
            wavs.append(self.decoder(inp)[..., n_ctx * DOWNSAMPLE_RATE:])
            keep = min(self.max_ctx // 2, end)
            ctx = codes[:, :, end - keep:end]
            pos = end
        self._append(codes)
        return torch.cat(wavs, dim=-1)

    # ---- streaming
    def _open(self) -> None:
        self._close_stack()
        self._stack = self.decoder.streaming(1)
        self._stack.__enter__()

    def prefill(self, n_codebooks: int = 0, device="cuda") -> None:
        self._prefill_n_codebooks = n_codebooks
        self._open()
        self._reseed(device)

    def _reseed(self, device="cuda") -> None:
        n = 0 if self._buf is None else self._buf.shape[2] % self.max_ctx
        if n:
            seed = self._buf[:, :, -n:]
            if self._prefill_n_codebooks > 0:
                seed = seed[:, : self._prefill_n_codebooks]
            self.decoder(seed)
        self._frames_since_prefill = n

    def _hard_reset(self, device="cuda") -> None:
        self._open()
        self._frames_since_prefill = 0

    def decode_frame(self, codes: Tensor, vocoder_ctx: int | None = None, store_codes: Tensor | None = None) -> Tensor:
        if codes.dim() == 2:
            codes = codes.unsqueeze(0)
        if self._stack is None or self._frames_since_prefill >= self.max_ctx:
            self._hard_reset()
        audio = self.decoder(codes)
        self._append(codes if store_codes is None else store_codes)
        self._frames_since_prefill += 1
        return audio

    def _close_stack(self) -> None:
        if self._stack is not None:
            self._stack.__exit__(None, None, None)
            self._stack = None

    def reset(self) -> None:
        self._prompt_len = 0
        self._buf = None
        self._frames_since_prefill = 0
        self._close_stack()
