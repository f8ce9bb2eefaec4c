"""Engine / Row / GenConfig / Segment / RenderRequest: the reference's public
inference API (src/vui/engine.py in fluxions-ai/vui) over libvuib200.

Same names, arguments and error behaviour as ``vui.engine`` so callers
(serving/stream/tts_worker.py, demo.py, docs/python-api.md) can switch engines.
What differs is underneath: one decode frame - backbone step, cb0 sampling, the
15 depth-transformer codebooks and the gather-sum that feeds the next frame - is
one captured CUDA graph of hand-written sm_100a kernels, with no host round trip
inside the frame and one device->host read (codes + EOS probability) after it.

The codec that turns codes into audio is ``vui_b200.codec.QwenCodecDecoder`` (the streaming decode on
this library's own kernels); pass it, or any object with ``decode(codes_bqt)`` and ``new_ctx()``, as
``codec=``, or work with codes only.
"""

from __future__ import annotations

import ctypes as C
from collections import deque
from collections.abc import Iterator
from dataclasses import dataclass
from types import SimpleNamespace

import torch
from torch import Tensor

from . import _lib
from .model import VuiB200
from .text import chunk_text, simple_clean

FRAME_RATE = 12.5  # codec frames per second (src/vui/qwen_codec.py:27-29)
MIN_FPW = 2.0              # frames per word below which a finished chunk counts as cut short (engine.py:909)
RETRY_TEMPS = (0.5, 0.3)   # temperatures of the retries (engine.py:910)
GATE_RETRY_TEMPS = (0.5, 0.3)  # and of the streaming gate's retries (engine.py:1367)
SAMPLE_RATE = 24000
DEFAULT_WPS = 3.0
RQ_TOP_K = 100  # the reference captures its depth graphs with top_k=100 (engine.py:395-397)


@dataclass(frozen=True)
class Segment:
    """One voice-reference unit: a transcript and its codec codes (T, Q) long."""

    text: str = ""
    codes: Tensor | None = None


@dataclass(frozen=True)
class GenConfig:
    """Sampling + generation settings (src/vui/engine.py:60-103)."""

    temperature: float = 0.9
    top_k: int | None = 100
    top_p: float | None = None  # carried for signature parity; the reference engine never reads it
    rep_penalty: float = 1.1
    rep_window: int = 24
    eos_threshold: float = 0.45
    min_secs: float = 0.5
    max_turn_secs: float = 15.0
    max_secs: float = 30.0
    chunk_words: int = 5
    first_chunk_words: int = 0
    n_codebooks: int = 0
    max_turn_wps: float = 0.0
    sentence_only: bool = False
    gate_frames: int = 0
    gate_entropy_max: float = 1.9
    gate_retries: int = 2

    def max_turn_frames(self, n_words: int, prompt_wps: float = 0.0) -> int:
        ceil = int(self.max_turn_secs * FRAME_RATE)
        wps = self.max_turn_wps if self.max_turn_wps > 0 else prompt_wps
        if wps <= 0:
            wps = DEFAULT_WPS
        if n_words <= 0:
            return ceil
        return min(int((n_words / wps * 1.6 + 0.6) * FRAME_RATE), ceil)


@dataclass(frozen=True)
class RenderRequest:
    """One TTS request for continuous batching."""

    segments: list[Segment]
    spk_emb: Tensor | None = None
    text: str = ""
    user_text: str | None = None
    user_codes: Tensor | None = None
    segments_2: list[Segment] | None = None
    spk_emb_2: Tensor | None = None


@dataclass
class _ActiveSlot:
    row: "Row"
    request_idx: int
    chunks: list[dict]
    chunk_idx: int = 0
    frame_count: int = 0
    turn_count: int = 0
    max_turn_frames: int = 0
    seq_offset: int = 0


def _make_buckets(max_bs: int) -> list[int]:
    out, b = [], 1
    while b < max_bs:
        out.append(b)
        b *= 2
    if not out or out[-1] != max_bs:
        out.append(max_bs)
    return out


def _get_bucket(n: int, buckets: list[int]) -> int:
    for b in buckets:
        if n <= b:
            return b
    return buckets[-1]


class Row:
    """A single conversation slot: index into the shared KV cache, the
    end-of-prompt offset for rewind, and the speaker token(s) from prefill."""

    def __init__(self, engine: "Engine", idx: int):
        self._engine = engine
        self._idx = idx
        self._prompt_offset = 0
        self._spk_token: Tensor | None = None
        self._spk_token_2: Tensor | None = None
        self._active_speaker = 0
        self._codec_ctx = engine._new_codec_ctx()
        self._closed = False
        self.prompt_wps: float = 0.0

    @property
    def idx(self) -> int:
        return self._idx

    @property
    def offset(self) -> int:
        return int(self._engine.seq_lens[self._idx].item())

    def prefill(self, segments, spk_emb=None, segments_2=None, spk_emb_2=None) -> int:
        return self._engine._prefill_row(self, segments, spk_emb, segments_2, spk_emb_2)

    def add_user(self, text: str = "", codes: Tensor | None = None, *, final: bool = True) -> int:
        return self._engine._add_user(self, text, codes, final=final)

    def stream(self, text: str, cfg: GenConfig = GenConfig(), cancel=None, *, reset_rep: bool = True,
               final_turn: bool = False) -> Iterator[Tensor]:
        if self._engine.max_rows != 1:
            raise RuntimeError(f"stream() requires Engine(max_rows=1), got {self._engine.max_rows}")
        yield from self._engine._stream_row(self, text, cfg, cancel, reset_rep=reset_rep,
                                            final_turn=final_turn)

    def render(self, text: str, cfg: GenConfig = GenConfig()):
        codes = self._engine._render_row(self, text, cfg)
        return codes, self._engine._decode_full(codes)

    def rewind(self) -> int:
        return self._engine._rewind_row(self, self._prompt_offset)

    def reset(self) -> int:
        return self._engine._rewind_row(self, 0)

    def close(self) -> None:
        if not self._closed:
            self._engine._release_row(self)
            self._closed = True

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class Engine:
    """Streaming (max_rows=1) and batched (max_rows=N) inference over one model."""

    NAMES = {"vui-nano": "vui-nano.safetensors"}

    def __init__(self, name: str = "vui-nano", *, model: VuiB200 | None = None, codec=None,
                 max_rows: int = 1, max_seq: int | None = None, codec_dtype: torch.dtype = torch.float32,
                 vocoder_ctx: int = 25, max_prefill_rows: int = 256, seed: int = 0):
        if not torch.cuda.is_available():
            raise RuntimeError("vui_b200.Engine needs a CUDA device (sm_100a); there is no CPU path")
        if model is None:
            model = VuiB200.from_checkpoint(self.NAMES.get(name, name))
        self.model = model
        self.codec = codec
        self.overlap_codec = False   # True: Row.stream decodes frame k's audio beside the generation of frame k + 1
        self._codec_stream = None
        self.max_rows = max_rows
        self.vocoder_ctx = vocoder_ctx
        self.device = model.device
        self.dtype = model.dtype
        s = model.shape
        self.Q, self.CS, self.D = s.n_quantizers, s.codebook_size, s.d_model
        self.tok = model.text_tokenizer
        self.seed = seed
        trained = model.decoder.max_seqlen
        self.max_seq = max_seq or trained
        if self.max_seq > trained:
            raise ValueError(f"max_seq={self.max_seq} exceeds trained ceiling {trained}")
        self.max_prefill_rows = max_prefill_rows
        if model._cond_bias is None:
            model._cond_bias = torch.zeros(1, 1, self.D, device=self.device, dtype=self.dtype)
        self._cond_bias = model._cond_bias
        self._sc_emb = None
        if self.tok is not None:
            sc_id = self.tok.special_to_id["[SC]"]
            self._sc_emb = model.token_emb(torch.tensor([[sc_id]], device=self.device)).to(self.dtype)
        self._lib = _lib.load()
        self._handle = C.c_void_p()
        self._graphs: dict[int, torch.cuda.CUDAGraph] = {}
        self._host_frames: set[tuple[int, bool]] = set()   # (rows, with input copy) captured inside the library
        self._capture_stream = None
        self._sampling_key = None
        self._setup_native()
        self._free: set[int] = set(range(max_rows))
        self._rows: dict[int, Row] = {}
        self._rep_window_cur = 0

    # ------------------------------------------------------------------ setup
    def _ck(self, code: int) -> None:
        _lib.check(self._handle, code)

    @property
    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def _setup_native(self) -> None:
        s, dev = self.model.shape, self.device
        n_slots = self.max_rows + 1  # spare slot: target of padded rows (engine.py:380-387)
        self._pad_slot = self.max_rows
        cfg = _lib.VuibConfig(
            s.d_model, s.n_layers, s.n_heads, s.n_kv_heads, s.head_dim, s.intermediate_size,
            s.n_quantizers, s.codebook_size, s.rq_d_model, s.rq_n_layers, s.rq_n_heads, s.rq_ffn,
            s.norm_eps, s.rq_norm_eps, n_slots, self.max_seq, self.max_rows, self.max_prefill_rows,
        )
        _lib.check(None, self._lib.vuib_create(C.byref(cfg), C.byref(self._handle)))
        # KV: one allocation, per-layer views in the reference's FlashKVCache layout
        self._kv = torch.zeros(s.n_layers, 2, n_slots, self.max_seq, s.n_kv_heads, s.head_dim,
                               device=dev, dtype=torch.bfloat16)
        self.seq_lens = torch.zeros(n_slots, device=dev, dtype=torch.int32)
        # this engine's caches; model.decoder.flash_kv_caches (where the reference keeps them, model.py:473-495)
        # points at the caches of the engine built last on the model
        self.flash_kv_caches = [
            SimpleNamespace(k_cache=self._kv[i, 0], v_cache=self._kv[i, 1], seq_lens=self.seq_lens)
            for i in range(s.n_layers)
        ]
        self.model.decoder.flash_kv_caches = self.flash_kv_caches
        nbytes = C.c_size_t()
        self._ck(self._lib.vuib_workspace_bytes(self._handle, C.byref(nbytes)))
        self._ws = torch.zeros(nbytes.value + 256, device=dev, dtype=torch.uint8)
        ws_ptr = (self._ws.data_ptr() + 255) & ~255
        self._ck(self._lib.vuib_bind_workspace(self._handle, C.c_void_p(ws_ptr), nbytes.value))
        sd = self.model.sd
        w = _lib.VuibWeights()
        P = lambda name: sd[name].data_ptr()  # noqa: E731
        w.audio_emb, w.codec_head = P("audio_emb.embedding.weight"), P("codec_head.weight")
        w.eos_w, w.eos_b, w.final_norm = P("eos_head.weight"), P("eos_head.bias"), P("decoder.norm.weight")
        for i in range(s.n_layers):
            p = f"decoder.blocks.{i}."
            w.attn_norm[i], w.wqkv[i] = P(p + "attn_norm.weight"), P(p + "attn.Wqkv.weight")
            w.out_proj[i], w.mlp_norm[i] = P(p + "attn.out_proj.weight"), P(p + "mlp_norm.weight")
            w.w1[i], w.w3[i], w.w2[i] = P(p + "mlp.w1.weight"), P(p + "mlp.w3.weight"), P(p + "mlp.w2.weight")
        r = "rq_transformer."
        w.rq_backbone_proj, w.rq_code_emb = P(r + "backbone_proj.weight"), P(r + "code_emb.embedding.weight")
        w.rq_pos_emb, w.rq_head, w.rq_norm = P(r + "pos_emb.weight"), P(r + "head_W"), P(r + "norm.weight")
        for i in range(s.rq_n_layers):
            p = f"{r}blocks.{i}."
            w.rq_attn_norm[i], w.rq_wqkv[i] = P(p + "attn_norm.weight"), P(p + "Wqkv.weight")
            w.rq_out_proj[i], w.rq_mlp_norm[i] = P(p + "out_proj.weight"), P(p + "mlp_norm.weight")
            w.rq_w1[i], w.rq_w3[i], w.rq_w2[i] = P(p + "w1.weight"), P(p + "w3.weight"), P(p + "w2.weight")
        self._ck(self._lib.vuib_bind_weights(self._handle, C.byref(w)))
        karr = (C.c_void_p * s.n_layers)(*[self._kv[i, 0].data_ptr() for i in range(s.n_layers)])
        varr = (C.c_void_p * s.n_layers)(*[self._kv[i, 1].data_ptr() for i in range(s.n_layers)])
        self._ck(self._lib.vuib_bind_kv(self._handle, karr, varr, C.c_void_p(self.seq_lens.data_ptr())))
        if self.model.decoder.freqs_cis.shape[0] < self.max_seq:
            raise ValueError("RoPE table shorter than max_seq")
        self._ck(self._lib.vuib_bind_rope(self._handle, C.c_void_p(self.model.decoder.freqs_cis.data_ptr())))
        # static I/O of the captured frame graphs
        N = self.max_rows
        self._g_codes_in = torch.zeros(N, self.Q, device=dev, dtype=torch.long)
        self._g_hidden_out = torch.zeros(N, self.D, device=dev, dtype=self.dtype)
        self._g_cb0_out = torch.zeros(N, self.CS, device=dev, dtype=self.dtype)
        self._g_eos_out = torch.zeros(N, 1, device=dev, dtype=self.dtype)
        self._g_eos_prob = torch.zeros(N, device=dev, dtype=torch.float32)
        self._g_cb0_stats = torch.zeros(N, 2, device=dev, dtype=torch.float32)  # entropy, top probability of the cb0 draw
        self._ck(self._lib.vuib_set_stats(self._handle, C.c_void_p(self._g_cb0_stats.data_ptr())))
        self._g_slot_idx = torch.arange(N, device=dev, dtype=torch.int32)
        self._g_seq_inc = torch.ones(N, device=dev, dtype=torch.int32)
        self._buckets = _make_buckets(N)
        # pinned landing zone for the one read-back per frame
        self._h_codes = torch.zeros(N, self.Q, dtype=torch.long).pin_memory()
        self._h_eos = torch.zeros(N, dtype=torch.float32).pin_memory()
        self._h_codes_in = torch.zeros(N, self.Q, dtype=torch.long).pin_memory()
        self._done = torch.cuda.Event()
        self._set_sampling(1.0, 1, 1, 1.0, 0, 0)

    def __del__(self):
        try:
            if self._handle:
                self._lib.vuib_destroy(self._handle)
                self._handle = C.c_void_p()
        except Exception:
            pass

    @classmethod
    def from_checkpoint(cls, checkpoint_path: str, *, max_rows: int = 1, max_seq: int | None = None,
                        codec_dtype: torch.dtype = torch.float32, vocoder_ctx: int = 25) -> "Engine":
        return cls(checkpoint_path, max_rows=max_rows, max_seq=max_seq, codec_dtype=codec_dtype,
                   vocoder_ctx=vocoder_ctx)

    def launch_count(self) -> int:
        return int(self._lib.vuib_launch_count(self._handle))

    def check_device(self) -> None:
        """Raise if a kernel saw a slot, position or code out of range."""
        self._ck(self._lib.vuib_check_device_flag(self._handle, self._stream))

    # --------------------------------------------------------------- sampling
    def _set_sampling(self, temperature, top_k_cb0, top_k_rq, rep_penalty, rep_window, n_codebooks) -> None:
        key = (float(temperature), int(top_k_cb0 or 0), int(top_k_rq or 0), float(rep_penalty),
               int(rep_window), int(n_codebooks), int(self.seed))
        if key == self._sampling_key:
            return
        old_ncb = self._sampling_key[5] if self._sampling_key else None
        sp = _lib.VuibSampling(key[0], key[1], key[2], key[3], key[4], key[5], key[6])
        self._ck(self._lib.vuib_set_sampling(self._handle, C.byref(sp), self._stream))
        self._sampling_key = key
        if old_ncb is not None and old_ncb != key[5]:
            self._graphs = {}  # the codebook count is baked into captured graphs
            self._host_frames = set()

    def _apply_cfg(self, cfg: GenConfig | None, temperature: float | None = None, greedy: bool = False) -> None:
        cfg = cfg or GenConfig()
        if greedy:
            self._set_sampling(1.0, 1, 1, 1.0, 0, cfg.n_codebooks)
        else:
            self._set_sampling(temperature or cfg.temperature, cfg.top_k or 0, RQ_TOP_K, cfg.rep_penalty,
                               min(cfg.rep_window, 64), cfg.n_codebooks)

    def _rep_reset(self, penalty: float = 1.0, window: int = 0, slot: int = -1) -> None:
        self._ck(self._lib.vuib_rep_reset(self._handle, slot, self._stream))
        self._rep_window_cur = window

    @property
    def _rep_counts(self) -> Tensor:
        """(max_rows, CS) fp32: how often each cb0 code sits in a row's repetition window
        (the tensor of the same name in the reference, engine.py:555-569)."""
        out = torch.zeros(self.max_rows, self.CS, device=self.device, dtype=torch.float32)
        for r in range(self.max_rows):
            self._ck(self._lib.vuib_rep_state(self._handle, r, C.c_void_p(out[r].data_ptr()), None, self._stream))
        return out

    @property
    def _rep_filled(self) -> int:
        """Codes currently held by row 0's rolling repetition window."""
        cnt = torch.zeros(self.CS, device=self.device, dtype=torch.float32)
        filled = torch.zeros(1, device=self.device, dtype=torch.int32)
        self._ck(self._lib.vuib_rep_state(self._handle, 0, C.c_void_p(cnt.data_ptr()), C.c_void_p(filled.data_ptr()),
                                          self._stream))
        return int(filled.item())

    # ----------------------------------------------------------------- graphs
    def _frame_call(self, B: int) -> None:
        P = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
        self._ck(self._lib.vuib_decode_frame(
            self._handle, B, P(self._g_slot_idx), P(self._g_seq_inc), P(self._g_codes_in),
            P(self._g_hidden_out), P(self._g_cb0_out), P(self._g_eos_out), P(self._g_eos_prob), self._stream))

    def _frame_graph(self, B: int) -> torch.cuda.CUDAGraph:
        g = self._graphs.get(B)
        if g is not None:
            return g
        # One warm-up outside capture loads the kernels; it runs on the spare slot
        # with the length frozen, and the sampler state it touched is put back.
        saved = (self._g_slot_idx.clone(), self._g_seq_inc.clone(), self._g_codes_in.clone(),
                 self.seq_lens.clone(), self._ws.clone())
        self._g_slot_idx.fill_(self._pad_slot)
        self._g_seq_inc.zero_()
        self._g_codes_in.zero_()
        self.seq_lens[self._pad_slot] = 0
        torch.cuda.synchronize(self.device)
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            self._frame_call(B)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._frame_call(B)
        torch.cuda.synchronize(self.device)
        self._g_slot_idx.copy_(saved[0])
        self._g_seq_inc.copy_(saved[1])
        self._g_codes_in.copy_(saved[2])
        self.seq_lens.copy_(saved[3])
        self._ws.copy_(saved[4])
        self._graphs[B] = g
        return g

    def _frame_step(self, B_active: int):
        """Replay one whole frame for the first B_active rows of the static
        buffers (padded to the bucket with rows aimed at the spare slot)."""
        B = _get_bucket(B_active, self._buckets)
        g = self._frame_graph(B)
        if B_active < B:
            self._g_slot_idx[B_active:B].fill_(self._pad_slot)
            self._g_seq_inc[B_active:B].zero_()
        g.replay()

    def _frame_host(self, B_active: int, h_codes_in: Tensor | None = None):
        """One whole frame through host memory in ONE library call (vuib_frame_host): optional host -> device
        copy of the previous frame's codes, the frame's kernels, device -> host copy of the new codes and EOS
        probabilities, all one CUDA-graph launch.  Returns views of the engine's pinned result buffers.
        The per-frame body of `_stream_row` (engine.py:1450-1546)."""
        B = _get_bucket(B_active, self._buckets)
        with_in = h_codes_in is not None
        if (B, with_in) not in self._host_frames:
            self._frame_graph(B)  # runs the frame once outside any capture (kernel loading) and restores the state
            if self._capture_stream is None:
                self._capture_stream = torch.cuda.Stream(self.device)
            torch.cuda.synchronize(self.device)
            P = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
            self._ck(self._lib.vuib_frame_host_capture(
                self._handle, B, int(with_in), P(self._g_slot_idx), P(self._g_seq_inc), P(self._g_codes_in),
                P(self._g_hidden_out), P(self._g_cb0_out), P(self._g_eos_out), P(self._g_eos_prob),
                C.c_void_p(self._capture_stream.cuda_stream)))
            self._host_frames.add((B, with_in))
        if B_active < B:
            self._g_slot_idx[B_active:B].fill_(self._pad_slot)
            self._g_seq_inc[B_active:B].zero_()
        src = None
        if with_in:
            if h_codes_in.dtype != torch.long or not h_codes_in.is_contiguous() or h_codes_in.is_cuda:
                raise ValueError("h_codes_in must be a contiguous int64 host tensor")
            if h_codes_in.shape[0] < B:  # the library reads B rows: pad rows come from the engine's own buffer
                self._h_codes_in[: h_codes_in.shape[0]].copy_(h_codes_in)
                h_codes_in = self._h_codes_in
            src = C.c_void_p(h_codes_in.data_ptr())
        self._ck(self._lib.vuib_frame_host(self._handle, B, int(with_in), src, C.c_void_p(self._h_codes.data_ptr()),
                                           C.c_void_p(self._h_eos.data_ptr()), self._stream))
        return self._h_codes[:B_active], self._h_eos[:B_active]

    def _read_frame(self, B: int):
        """The frame's one device->host read: codes (B, Q) and EOS probabilities."""
        self._h_codes[:B].copy_(self._g_codes_in[:B], non_blocking=True)
        self._h_eos[:B].copy_(self._g_eos_prob[:B], non_blocking=True)
        self._done.record()
        self._done.synchronize()
        return self._h_codes[:B], self._h_eos[:B]

    def _decode_step(self):
        """Backbone-only step over all max_rows slots (engine.py:850-853)."""
        P = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
        self._g_slot_idx.copy_(torch.arange(self.max_rows, device=self.device, dtype=torch.int32))
        self._ck(self._lib.vuib_backbone_step(
            self._handle, self.max_rows, P(self._g_slot_idx), None, P(self._g_codes_in),
            P(self._g_hidden_out), P(self._g_cb0_out), P(self._g_eos_out), self._stream))
        return self._g_hidden_out, self._g_cb0_out, self._g_eos_out

    def _set_codes_in(self, row_idx: int, codes: Tensor) -> None:
        n = codes.shape[0]
        if n < self.Q:
            self._g_codes_in[row_idx].zero_()
            self._g_codes_in[row_idx, :n] = codes
        else:
            self._g_codes_in[row_idx] = codes

    # ---------------------------------------------------------- row lifecycle
    def _new_codec_ctx(self):
        mk = getattr(self.codec, "new_ctx", None)
        return mk() if mk else None

    def new_row(self) -> Row:
        if not self._free:
            raise RuntimeError(f"No free rows (max_rows={self.max_rows} all in use)")
        idx = min(self._free)
        self._free.remove(idx)
        row = Row(self, idx)
        self._rows[idx] = row
        self.seq_lens[idx] = 0
        return row

    def _release_row(self, row: Row) -> None:
        self._rows.pop(row.idx, None)
        self._free.add(row.idx)
        if row._codec_ctx is not None:
            row._codec_ctx.reset()

    def reset(self) -> None:
        for row in list(self._rows.values()):
            row.close()
        self.seq_lens.zero_()

    def _rewind_row(self, row: Row, offset: int) -> int:
        self.seq_lens[row.idx] = offset
        return offset

    def set_conditioning(self, *, sq_scores=None, wps_score: float = 0.0) -> None:
        """SQ / WPS conditioning bias added to text embeddings (Vui.set_cond_bias,
        model.py:1258-1274).  Needs the projection weights in the checkpoint."""
        self._cond_bias.zero_()
        sd = self.model.sd
        if sq_scores is not None and "sq_proj.weight" in sd:
            v = torch.tensor([sq_scores], device=self.device, dtype=torch.bfloat16)
            self._cond_bias.add_(torch.nn.functional.linear(v, sd["sq_proj.weight"]).reshape(1, 1, -1))
        if wps_score > 0 and "wps_proj.proj.weight" in sd:
            v = torch.tensor([[wps_score]], device=self.device, dtype=torch.bfloat16)
            self._cond_bias.add_(torch.nn.functional.linear(v, sd["wps_proj.proj.weight"]).reshape(1, 1, -1))

    # ---------------------------------------------------------------- prefill
    def _prefill_many(self, items: list[tuple[Row, Tensor]]) -> list[Tensor]:
        """Prefill several (row, emb (T_i, d)) pairs in as few calls as fit
        max_prefill_rows.  Returns each row's final-norm output (T_i, d)."""
        outs = []
        pend: list[tuple[int, int, Tensor]] = []  # slot, offset, emb

        def flush():
            if not pend:
                return
            emb = torch.cat([e for _, _, e in pend], dim=0).to(self.dtype).contiguous()
            slot = torch.cat([torch.full((e.shape[0],), s_, dtype=torch.int32) for s_, _, e in pend])
            pos = torch.cat([torch.arange(o, o + e.shape[0], dtype=torch.int32) for _, o, e in pend])
            slot, pos = slot.to(self.device), pos.to(self.device)
            out = torch.empty_like(emb)
            P = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
            self._ck(self._lib.vuib_prefill(self._handle, emb.shape[0], P(slot), P(pos), P(emb), P(out),
                                            self._stream))
            i = 0
            for s_, _, e in pend:
                outs.append(out[i:i + e.shape[0]])
                self.seq_lens[s_] += e.shape[0]
                i += e.shape[0]
            pend.clear()

        offsets = {}
        for row, emb in items:
            emb = emb.reshape(-1, self.D)
            off = offsets.get(row.idx, row.offset)
            if off + emb.shape[0] > self.max_seq:
                raise RuntimeError(f"prefill of {emb.shape[0]} positions overflows max_seq={self.max_seq}")
            # a segment longer than one call is cut; a slot may appear several times in a call (its rows
            # carry consecutive positions, and every row's K/V is in the cache before any row attends)
            start = 0
            while start < emb.shape[0]:
                room = self.max_prefill_rows - sum(e.shape[0] for _, _, e in pend)
                if room == 0:
                    flush()
                    room = self.max_prefill_rows
                n = min(room, emb.shape[0] - start)
                pend.append((row.idx, off + start, emb[start:start + n]))
                start += n
            offsets[row.idx] = off + emb.shape[0]
        flush()
        # stitch cut segments back together per input item
        res, k = [], 0
        for row, emb in items:
            T, parts = emb.reshape(-1, self.D).shape[0], []
            while sum(p.shape[0] for p in parts) < T:
                parts.append(outs[k])
                k += 1
            res.append(torch.cat(parts, dim=0) if len(parts) > 1 else parts[0])
        return res

    def _prefill_emb(self, row: Row, emb: Tensor) -> Tensor:
        """Write (1, T, d) embeddings into the row's slot at its current offset;
        returns the decoder's final-norm output (1, T, d) (engine.py:674-694)."""
        return self._prefill_many([(row, emb)])[0].unsqueeze(0)

    def prefill_ids(self, row: Row, ids: Tensor) -> Tensor:
        """Tokenizer-free prefill of text token ids; returns the last position's hidden (d,)."""
        return self._prefill_emb(row, self.model.token_emb(ids.reshape(1, -1)))[0, -1]

    def _need_tok(self):
        if self.tok is None:
            raise RuntimeError("this model was built without a text tokenizer; use prefill_ids / token ids")

    def _text_emb(self, text: str, with_cond_bias: bool, noisy: bool = False) -> Tensor:
        self._need_tok()
        ids = self.tok.encode(simple_clean(text)).to(self.device)
        emb = self.model.token_emb(ids[None]).to(self.dtype)
        if with_cond_bias:
            emb = emb + self._cond_bias
        if noisy and "noisy_emb" in self.model.sd:
            emb = emb + self.model.sd["noisy_emb"].to(self.dtype)
        return emb

    def _embed_codes_kernel(self, codes: Tensor) -> Tensor:
        """codes (n, Q') long -> (n, d) bf16 gather-sum by the library's kernel;
        fewer than Q codebooks are zero-padded as the reference does (engine.py:473-479)."""
        codes = codes.to(self.device, torch.long)
        if codes.shape[-1] < self.Q:
            codes = torch.nn.functional.pad(codes, (0, self.Q - codes.shape[-1]))
        codes = codes.contiguous()
        out = torch.empty(codes.shape[0], self.D, device=self.device, dtype=self.dtype)
        self._ck(self._lib.vuib_embed_codes(self._handle, codes.shape[0], C.c_void_p(codes.data_ptr()),
                                            C.c_void_p(out.data_ptr()), self._stream))
        return out

    def _audio_emb(self, codes: Tensor) -> Tensor:
        pc = codes.to(self.device)
        if pc.dim() == 3:
            pc = pc[0]
        if pc.shape[-1] < self.Q:  # a prompt with fewer codebooks sums only those tables
            return self.model.embed_audio(pc.unsqueeze(0)).to(self.dtype)
        return self._embed_codes_kernel(pc).unsqueeze(0)

    # ------------------------------------------------- test / debug helpers
    def _set_taps(self, layer_hidden: Tensor | None, rq_logits: Tensor | None) -> None:
        self._graphs = {}
        self._host_frames = set()
        self._tap_refs = (layer_hidden, rq_logits)
        P = lambda t: C.c_void_p(t.data_ptr()) if t is not None else None  # noqa: E731
        self._ck(self._lib.vuib_set_taps(self._handle, P(layer_hidden), P(rq_logits)))

    def _attention(self, layer: int, q: Tensor, row_slot: Tensor, row_pos: Tensor) -> Tensor:
        """Decode attention of one layer over the engine's KV cache: q (n, H*hd) bf16 with RoPE
        applied, row r attends keys [0, row_pos[r]] of slot row_slot[r]."""
        q = q.to(self.device, self.dtype).contiguous()
        rs = row_slot.to(self.device, torch.int32).contiguous()
        rp = row_pos.to(self.device, torch.int32).contiguous()
        out = torch.empty_like(q)
        P = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
        self._ck(self._lib.vuib_attention(self._handle, layer, q.shape[0], P(q), P(rs), P(rp), P(out), self._stream))
        return out

    def _sample_rows(self, logits: Tensor, n_draws: int, cb0: bool = False) -> Tensor:
        """Draw n_draws times per row from logits (B, CS); returns (n_draws, B) on the host."""
        B = logits.shape[0]
        logits = logits.to(self.device, self.dtype).contiguous()
        slots = torch.arange(B, device=self.device, dtype=torch.int32)
        out = torch.zeros(n_draws, B, device=self.device, dtype=torch.long)
        for i in range(n_draws):
            self._ck(self._lib.vuib_sample_rows(self._handle, B, C.c_void_p(slots.data_ptr()),
                                                C.c_void_p(logits.data_ptr()), 0 if cb0 else 1,
                                                C.c_void_p(out[i].data_ptr()), self._stream))
        return out.cpu()

    def _debug_norm_linear(self, x: Tensor, norm_w: Tensor, w: Tensor, tensor_cores: bool = False) -> Tensor:
        """bf16(W . RMSNorm(x) * norm_w) through the GEMV (or tcgen05) kernels: x (n, d), W (n_out, d)."""
        x, norm_w, w = (t.to(self.device, self.dtype).contiguous() for t in (x, norm_w, w))
        out = torch.empty(x.shape[0], w.shape[0], device=self.device, dtype=self.dtype)
        P = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
        self._ck(self._lib.vuib_debug_norm_linear(self._handle, x.shape[0], P(x), P(norm_w), P(w), w.shape[0], P(out),
                                                  int(tensor_cores), self._stream))
        return out

    def _debug_linear_rope(self, x: Tensor, w: Tensor, pos: Tensor, tensor_cores: bool = False) -> Tensor:
        """RoPE(bf16(W . x)) at positions pos (n,), every 64 columns one head: x (n, d), W (d, d)."""
        x, w = (t.to(self.device, self.dtype).contiguous() for t in (x, w))
        pos = pos.to(self.device, torch.int32).contiguous()
        out = torch.empty(x.shape[0], w.shape[0], device=self.device, dtype=self.dtype)
        P = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
        self._ck(self._lib.vuib_debug_linear_rope(self._handle, x.shape[0], P(x), P(w), P(pos), P(out),
                                                  int(tensor_cores), self._stream))
        return out

    def _sample_first_frame(self, cb0_logits: Tensor, n_draws: int) -> Tensor:
        """cb0 draws of a chunk's first frame (no top-k, engine.py:936-937) for rows of logits (B, CS),
        through the depth step the frame-0 path uses; returns (n_draws, B) on the host."""
        B = cb0_logits.shape[0]
        lg = cb0_logits.to(self.device, self.dtype).contiguous()
        hid = torch.zeros(B, self.D, device=self.device, dtype=self.dtype)
        slots = torch.arange(B, device=self.device, dtype=torch.int32)
        codes = torch.zeros(B, self.Q, device=self.device, dtype=torch.long)
        out = torch.zeros(n_draws, B, dtype=torch.long, device=self.device)
        P = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
        for i in range(n_draws):
            self._ck(self._lib.vuib_depth_step(self._handle, B, P(slots), P(hid), P(lg), None, 1, P(codes), None,
                                               self._stream))
            out[i] = codes[:, 0]
        return out.cpu()

    def _ws_reset_counters(self) -> None:
        """Zero the sampler state (draw counters, penalty state, error flag)."""
        self._ck(self._lib.vuib_reset_state(self._handle, self._stream))

    def _embed_speaker(self, spk_emb):
        if spk_emb is None or "spk_proj.weight" not in self.model.sd:
            return None
        return self.model.embed_speaker(spk_emb).to(self.dtype)

    def _prefill_speaker_segments(self, row, segments, spk_token, *, final=False) -> None:
        last = len(segments) - 1
        for i, seg in enumerate(segments):
            if spk_token is not None:
                self._prefill_emb(row, spk_token)
            if seg.text:
                self._prefill_emb(row, self._text_emb(seg.text, with_cond_bias=False))
            if final and i == last and self._sc_emb is not None:
                self._prefill_emb(row, self._sc_emb)
            if seg.codes is not None:
                self._prefill_emb(row, self._audio_emb(seg.codes))

    def _prefill_row(self, row, segments, spk_emb, segments_2=None, spk_emb_2=None) -> int:
        row._spk_token = self._embed_speaker(spk_emb)
        row._spk_token_2 = self._embed_speaker(spk_emb_2)
        row._active_speaker = 0
        all_codes = [s.codes for s in list(segments) + list(segments_2 or []) if s.codes is not None]
        if all_codes and row._codec_ctx is not None:
            row._codec_ctx.set_prompt(torch.cat([c.to(self.device) for c in all_codes], dim=0).T.unsqueeze(0))
        self._prefill_speaker_segments(row, segments, row._spk_token, final=True)
        if segments_2 is not None:
            self._prefill_speaker_segments(row, segments_2, row._spk_token_2, final=True)
        row._prompt_offset = row.offset
        segs = list(segments) + list(segments_2 or [])
        words = sum(len(s.text.split()) for s in segs if s.text)
        frames = sum(s.codes.shape[0] for s in segs if s.codes is not None)
        if frames > 0 and words > 0:
            row.prompt_wps = words / (frames / FRAME_RATE)
        return row._prompt_offset

    def _add_user(self, row, text, codes, *, final=True) -> int:
        if text:
            self._prefill_emb(row, self._text_emb(text, with_cond_bias=False, noisy=True))
        if final and self._sc_emb is not None:
            self._prefill_emb(row, self._sc_emb)
        if codes is not None:
            self._prefill_emb(row, self._audio_emb(codes))
            if row._codec_ctx is not None:
                row._codec_ctx.add(codes.T.unsqueeze(0).to(self.device))
        return row.offset

    def _active_spk_token(self, row):
        if row._active_speaker == 1 and row._spk_token_2 is not None:
            return row._spk_token_2
        return row._spk_token

    def _add_agent_text(self, row, text, *, final=False) -> Tensor:
        spk = self._active_spk_token(row)
        if spk is not None:
            self._prefill_emb(row, spk)
        out = self._prefill_emb(row, self._text_emb(text, with_cond_bias=True))
        if final and self._sc_emb is not None:
            out = self._prefill_emb(row, self._sc_emb)
        return out[0, -1]

    # ------------------------------------------------------------ first frame
    def _first_frames(self, rows: list[Row], hidden: Tensor) -> Tensor:
        """Frame 0 of a chunk for B rows from the prefill's last hidden (B, d):
        codec_head -> cb0 from the whole distribution -> depth loop
        (engine.py:928-951).  Returns codes (B, Q) on the device (a fresh tensor)."""
        B = len(rows)
        P = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
        hid = hidden.reshape(B, self.D).to(self.dtype).contiguous()
        slots = torch.tensor([r.idx for r in rows], device=self.device, dtype=torch.int32)
        cb0 = torch.empty(B, self.CS, device=self.device, dtype=self.dtype)
        eos = torch.empty(B, 1, device=self.device, dtype=self.dtype)
        codes = torch.zeros(B, self.Q, device=self.device, dtype=torch.long)
        self._ck(self._lib.vuib_heads(self._handle, B, P(hid), P(cb0), P(eos), self._stream))
        self._ck(self._lib.vuib_depth_step(self._handle, B, P(slots), P(hid), P(cb0), P(eos), 1, P(codes),
                                           None, self._stream))
        self._last_first = (hid, cb0, eos)
        return codes

    # --------------------------------------------- tokenizer-free generation
    @torch.inference_mode()
    def generate_frames(self, rows: list[Row], first_hidden: Tensor, n_frames: int,
                        cfg: GenConfig = GenConfig(), *, greedy: bool = False, read_back: bool = False,
                        on_frame=None) -> Tensor:
        """Emit ``n_frames`` frames for every row (EOS ignored): frame 0 from
        ``first_hidden`` (B, d), frame k from one replay of the frame graph on
        frame k-1.  Returns codes (B, n_frames, Q) on the device.  ``read_back``
        copies each frame to pinned host memory as a streaming caller would."""
        B = len(rows)
        if B > self.max_rows:
            raise RuntimeError("more rows than max_rows")
        self._apply_cfg(cfg, greedy=greedy)
        out = torch.zeros(n_frames, B, self.Q, device=self.device, dtype=torch.long)
        self._g_slot_idx[:B] = torch.tensor([r.idx for r in rows], device=self.device, dtype=torch.int32)
        self._g_seq_inc[:B].fill_(1)
        codes0 = self._first_frames(rows, first_hidden)
        self._g_codes_in[:B] = codes0
        out[0] = codes0
        for f in range(1, n_frames):
            self._frame_step(B)
            out[f].copy_(self._g_codes_in[:B], non_blocking=True)
            if read_back:
                h_codes, h_eos = self._read_frame(B)
                if on_frame is not None:
                    on_frame(f, h_codes, h_eos)
        return out.transpose(0, 1)

    # ------------------------------------------------------------ render loops
    @torch.inference_mode()
    def _render_rows(self, rows: list[Row], texts: list[str], cfg: GenConfig) -> dict[int, Tensor]:
        """Batched non-streaming decode; returns {row.idx: (T, Q) codes on CPU}
        (engine.py:865-1087: per-chunk text prefill, frame 0 from the prefill's
        hidden, EOS after min_frames, per-chunk frame cap)."""
        max_frames = int(cfg.max_secs * FRAME_RATE)
        min_frames = int(cfg.min_secs * FRAME_RATE)
        max_seq = self.max_seq - 10
        chunks = {r.idx: chunk_text(t, min_words=cfg.chunk_words, sentence_only=cfg.sentence_only,
                                    single_speaker=(r._spk_token_2 is None)) for r, t in zip(rows, texts)}
        ci = {r.idx: 0 for r in rows}
        count = {r.idx: 0 for r in rows}
        turn = {r.idx: 0 for r in rows}
        cap = {r.idx: cfg.max_turn_frames(0, r.prompt_wps) for r in rows}
        frames: dict[int, list[Tensor]] = {r.idx: [] for r in rows}
        active = {r.idx: True for r in rows}
        self._apply_cfg(cfg)
        self._rep_reset(cfg.rep_penalty, cfg.rep_window)
        qi = {r.idx: i for i, r in enumerate(rows)}  # static-buffer row of each Row
        B = len(rows)
        self._g_slot_idx[:B] = torch.tensor([r.idx for r in rows], device=self.device, dtype=torch.int32)

        chunk_start = {r.idx: r.offset for r in rows}  # KV length before the current chunk's text
        retry_idx = {r.idx: 0 for r in rows}

        def advance(row: Row, temp: float | None = None, flip: bool = True) -> bool:
            c = chunks[row.idx]
            if ci[row.idx] >= len(c):
                return False
            ch = c[ci[row.idx]]
            if flip and ch["sc"] and row._spk_token_2 is not None:
                row._active_speaker = 1 - row._active_speaker
            cap[row.idx] = cfg.max_turn_frames(len(ch["text"].split()), row.prompt_wps)
            chunk_start[row.idx] = row.offset
            hidden = self._add_agent_text(row, ch["text"])
            if temp is not None:  # a retry draws the chunk's first frame at the lower temperature
                self._apply_cfg(cfg, temperature=temp)
            codes = self._first_frames([row], hidden[None])[0]
            if temp is not None:
                self._apply_cfg(cfg)
            self._set_codes_in(qi[row.idx], codes)
            frames[row.idx].append(codes.cpu())
            count[row.idx] += 1
            turn[row.idx] = 1
            return True

        def retry_chunk(row: Row) -> bool:
            """A chunk that ended after fewer than MIN_FPW frames per word was cut short: rewind
            the KV to the chunk's start and speak it again at a lower temperature
            (engine.py:953-983).  False when the chunk is long enough or the temperatures are used up."""
            words = len(chunks[row.idx][ci[row.idx]]["text"].split())
            fpw = turn[row.idx] / words if words > 0 else 999.0
            ri = retry_idx[row.idx]
            if fpw >= MIN_FPW or ri >= len(RETRY_TEMPS):
                retry_idx[row.idx] = 0
                return False
            retry_idx[row.idx] = ri + 1
            self._rewind_row(row, chunk_start[row.idx])
            del frames[row.idx][len(frames[row.idx]) - turn[row.idx]:]
            count[row.idx] -= turn[row.idx]
            self._rep_reset(cfg.rep_penalty, cfg.rep_window)
            return advance(row, temp=RETRY_TEMPS[ri], flip=False)

        def next_chunk(row: Row) -> bool:
            if retry_chunk(row):
                return True
            ci[row.idx] += 1
            return advance(row)

        for r in rows:
            if not advance(r):
                active[r.idx] = False
        steps = 0
        while any(active.values()) and steps < max_frames:
            for r in rows:
                if active[r.idx] and turn[r.idx] >= cap[r.idx]:
                    if not next_chunk(r):
                        active[r.idx] = False
            if not any(active.values()):
                break
            for r in rows:
                self._g_seq_inc[qi[r.idx]] = 1 if active[r.idx] else 0
            self._frame_step(B)
            steps += 1
            h_codes, h_eos = self._read_frame(B)
            h_codes = h_codes.clone()
            for r in rows:
                if not active[r.idx]:
                    continue
                if r.offset >= max_seq or count[r.idx] >= max_frames:
                    active[r.idx] = False
                    continue
                if turn[r.idx] >= min_frames and float(h_eos[qi[r.idx]]) > cfg.eos_threshold:
                    if not next_chunk(r):
                        active[r.idx] = False
                    continue
                frames[r.idx].append(h_codes[qi[r.idx]])
                count[r.idx] += 1
                turn[r.idx] += 1
        return {i: torch.stack(f) for i, f in frames.items() if f}

    def _render_row(self, row: Row, text: str, cfg: GenConfig) -> Tensor:
        return self._render_rows([row], [text], cfg).get(row.idx, torch.zeros(0, self.Q, dtype=torch.long))

    def render_all(self, rows: list[Row], texts: list[str], cfg: GenConfig = GenConfig()) -> list:
        res = self._render_rows(rows, texts, cfg)
        return [self._decode_full(res.get(r.idx, torch.zeros(0, self.Q, dtype=torch.long))) for r in rows]

    @torch.inference_mode()
    def render_continuous(self, requests: list[RenderRequest], cfg: GenConfig = GenConfig()) -> list:
        """Continuous batching (engine.py:1112-1302): more requests than slots
        are accepted; a finished slot is refilled from the queue; results come
        back in input order."""
        codes = self.render_continuous_codes(requests, cfg)
        return [self._decode_full(c) for c in codes]

    @torch.inference_mode()
    def render_continuous_codes(self, requests: list[RenderRequest], cfg: GenConfig = GenConfig()) -> list[Tensor]:
        if not requests:
            return []
        max_frames = int(cfg.max_secs * FRAME_RATE)
        min_frames = int(cfg.min_secs * FRAME_RATE)
        max_seq = self.max_seq - 10
        bufs: list[list[Tensor]] = [[] for _ in requests]
        pending: deque[int] = deque(range(len(requests)))
        active: dict[int, _ActiveSlot] = {}
        free_slots = set(range(self.max_rows))
        last_codes: dict[int, Tensor] = {}
        self._apply_cfg(cfg)
        # continuous batching keeps penalty counts without a window (engine.py:606-616)
        self._set_sampling(cfg.temperature, cfg.top_k or 0, RQ_TOP_K, cfg.rep_penalty, 0, cfg.n_codebooks)

        def advance(info: _ActiveSlot) -> bool:
            if info.chunk_idx >= len(info.chunks):
                return False
            ch = info.chunks[info.chunk_idx]
            row = info.row
            if ch["sc"] and row._spk_token_2 is not None:
                row._active_speaker = 1 - row._active_speaker
            info.max_turn_frames = cfg.max_turn_frames(len(ch["text"].split()), row.prompt_wps)
            hidden = self._add_agent_text(row, ch["text"])
            codes = self._first_frames([row], hidden[None])[0]
            last_codes[row.idx] = codes
            bufs[info.request_idx].append(codes.cpu()[None])
            info.frame_count += 1
            info.turn_count = 1
            info.seq_offset = row.offset
            return True

        def backfill() -> None:
            while pending and free_slots:
                ri = pending.popleft()
                req = requests[ri]
                slot = min(free_slots)
                free_slots.remove(slot)
                self.seq_lens[slot] = 0
                self._rep_reset(slot=slot)
                row = Row(self, slot)
                self._rows[slot] = row
                row.prefill(req.segments, spk_emb=req.spk_emb, segments_2=req.segments_2, spk_emb_2=req.spk_emb_2)
                if req.user_text or req.user_codes is not None:
                    row.add_user(req.user_text or "", req.user_codes)
                chunks = chunk_text(req.text, min_words=cfg.chunk_words, sentence_only=cfg.sentence_only,
                                    single_speaker=(row._spk_token_2 is None))
                info = _ActiveSlot(row=row, request_idx=ri, chunks=chunks)
                if not chunks or not advance(info):
                    self._rows.pop(slot, None)
                    free_slots.add(slot)
                    continue
                active[slot] = info

        backfill()
        while active:
            slots = sorted(active)
            B = len(slots)
            for qi, s_ in enumerate(slots):
                self._set_codes_in(qi, last_codes[s_])
            self._g_slot_idx[:B] = torch.tensor(slots, device=self.device, dtype=torch.int32)
            self._g_seq_inc[:B].fill_(1)
            self._frame_step(B)
            h_codes, h_eos = self._read_frame(B)
            h_codes = h_codes.clone()
            done = []
            for qi, s_ in enumerate(slots):
                info = active[s_]
                info.seq_offset += 1
                if info.frame_count >= max_frames or info.seq_offset >= max_seq:
                    done.append(s_)
                    continue
                hit_eos = info.turn_count >= min_frames and float(h_eos[qi]) > cfg.eos_threshold
                if hit_eos or info.turn_count >= info.max_turn_frames:
                    info.chunk_idx += 1
                    if not advance(info):
                        done.append(s_)
                    continue
                last_codes[s_] = self._g_codes_in[qi].clone()
                bufs[info.request_idx].append(h_codes[qi][None])
                info.frame_count += 1
                info.turn_count += 1
            for s_ in done:
                info = active.pop(s_)
                self._rows.pop(s_, None)
                free_slots.add(s_)
            backfill()
        return [torch.cat(b, dim=0) if b else torch.zeros(0, self.Q, dtype=torch.long) for b in bufs]

    # -------------------------------------------------------------- streaming
    @torch.inference_mode()
    def _stream_codes(self, row: Row, text: str, cfg: GenConfig, cancel=None, *, reset_rep: bool = True,
                      final_turn: bool = False) -> Iterator[Tensor]:
        """Per-frame streaming for max_rows=1: yields (Q,) code tensors on the
        host (engine.py:1308-1535, entropy gate included)."""
        max_frames = int(cfg.max_secs * FRAME_RATE)
        min_frames = int(cfg.min_secs * FRAME_RATE)
        max_seq = self.max_seq - 10
        single = row._spk_token_2 is None
        chunks = chunk_text(text, min_words=cfg.chunk_words, sentence_only=cfg.sentence_only, single_speaker=single)
        if not chunks:
            return
        if 0 < cfg.first_chunk_words < cfg.chunk_words:
            words = chunks[0]["text"].split()
            if len(words) > cfg.first_chunk_words:
                head = " ".join(words[: cfg.first_chunk_words])
                rest = chunk_text(" ".join(words[cfg.first_chunk_words:]), min_words=cfg.chunk_words,
                                  sentence_only=cfg.sentence_only, single_speaker=single)
                chunks = [{"text": head, "sc": chunks[0]["sc"]}] + rest + chunks[1:]
        self._apply_cfg(cfg)
        if reset_rep:
            self._rep_reset(cfg.rep_penalty, cfg.rep_window)
        self._g_slot_idx[0] = row.idx
        self._g_seq_inc[0] = 1
        total = 0
        last = len(chunks) - 1
        for ci, ch in enumerate(chunks):
            if total >= max_frames or row.offset >= max_seq or (cancel is not None and cancel.is_set()):
                return
            if ch["sc"] and row._spk_token_2 is not None:
                row._active_speaker = 1 - row._active_speaker
            cap = cfg.max_turn_frames(len(ch["text"].split()), row.prompt_wps)
            # Hallucination gate (engine.py:1385-1533): the first gate_frames frames of the first
            # chunk are held back; if the mean entropy of their cb0 distributions is above
            # gate_entropy_max the chunk is rewound and spoken again at 0.5, then 0.3.
            use_gate = cfg.gate_frames > 0 and ci == 0 and reset_rep
            chunk_start = row.offset
            retry = 0
            while True:
                if retry > 0:
                    self._apply_cfg(cfg, temperature=GATE_RETRY_TEMPS[min(retry - 1, len(GATE_RETRY_TEMPS) - 1)])
                    self._rewind_row(row, chunk_start)
                    self._rep_reset(cfg.rep_penalty, cfg.rep_window)
                held: list[Tensor] = []
                entropies: list[float] = []
                hidden = self._add_agent_text(row, ch["text"], final=(final_turn and ci == last))
                codes = self._first_frames([row], hidden[None])[0]
                self._set_codes_in(0, codes)
                if use_gate:
                    entropies.append(float(self._g_cb0_stats[0, 0]))
                    held.append(codes.cpu())
                else:
                    yield codes.cpu()
                    total += 1
                offset = row.offset
                retry_triggered = False
                for step in range(1, cap):
                    if total >= max_frames or offset >= max_seq or (cancel is not None and cancel.is_set()):
                        if cancel is None or not cancel.is_set():
                            for hc in held:
                                yield hc
                                total += 1
                        self._apply_cfg(cfg)
                        return
                    h_codes, h_eos = self._frame_host(1)
                    offset += 1
                    gathering = use_gate and len(held) < cfg.gate_frames
                    if gathering:
                        entropies.append(float(self._g_cb0_stats[0, 0]))
                    if step >= min_frames and float(h_eos[0]) > cfg.eos_threshold:
                        for hc in held:  # a chunk shorter than the gate: flushed without a decision
                            yield hc
                            total += 1
                        held = []
                        break
                    if gathering:
                        held.append(h_codes[0].clone())
                        if len(held) == cfg.gate_frames:
                            if sum(entropies) / len(entropies) > cfg.gate_entropy_max and retry < cfg.gate_retries:
                                retry_triggered = True
                                break
                            for hc in held:
                                yield hc
                                total += 1
                            held = []
                            use_gate = False
                    else:
                        yield h_codes[0].clone()
                        total += 1
                if retry_triggered:
                    retry += 1
                    continue
                for hc in held:
                    yield hc
                    total += 1
                break
            if retry > 0:
                self._apply_cfg(cfg)

    def _stream_row(self, row, text, cfg, cancel=None, *, reset_rep=True, final_turn=False):
        # seed the codec once per session from the buffered prompt codes (engine.py:1349-1356); later calls
        # keep the streaming state and start cold at the 10 s boundary inside decode_frame
        ctx = row._codec_ctx
        if ctx is not None and hasattr(ctx, "prefill") and getattr(ctx, "_stack", True) is None:
            ctx.prefill(n_codebooks=cfg.n_codebooks)
        if not self.overlap_codec:
            for codes in self._stream_codes(row, text, cfg, cancel, reset_rep=reset_rep, final_turn=final_turn):
                yield self._stream_decode_frame(codes.to(self.device), cfg.n_codebooks)
            return
        # frame k's audio is decoded on a second stream while frame k + 1 is generated on the first: the same
        # audio in the same order, each frame handed out one generation step later
        main = torch.cuda.current_stream(self.device)
        if self._codec_stream is None:
            self._codec_stream = torch.cuda.Stream(self.device)
        side, pending = self._codec_stream, None
        for codes in self._stream_codes(row, text, cfg, cancel, reset_rep=reset_rep, final_turn=final_turn):
            dev_codes = codes.to(self.device)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                audio = self._stream_decode_frame(dev_codes, cfg.n_codebooks)
                done = torch.cuda.Event()
                done.record(side)
            audio.record_stream(side)
            if pending is not None:
                pending[0].synchronize()
                yield pending[1]
            pending = (done, audio)
        if pending is not None:
            pending[0].synchronize()
            yield pending[1]
        main.wait_stream(side)

    def _stream_decode_frame(self, frame_codes: Tensor, n_codebooks: int) -> Tensor:
        if 0 not in self._rows or self._rows[0]._codec_ctx is None:
            raise RuntimeError("streaming audio needs a codec with a streaming context; "
                               "iterate Engine._stream_codes for codes only")
        if frame_codes.shape[0] < self.Q:
            pad = torch.zeros(self.Q, device=self.device, dtype=frame_codes.dtype)
            pad[: frame_codes.shape[0]] = frame_codes
            frame_codes = pad
        codes_t = frame_codes.unsqueeze(0).unsqueeze(-1)
        dec = codes_t[:, :n_codebooks] if n_codebooks > 0 else codes_t
        return self._rows[0]._codec_ctx.decode_frame(dec, store_codes=codes_t)

    def _decode_full(self, codes: Tensor):
        """codes (T, Q) -> audio (1, 1, S) through the codec, if one was given."""
        if self.codec is None:
            return None
        if codes.shape[0] == 0:
            return torch.zeros(1, 1, 0, device=self.device)
        with torch.inference_mode(), torch.autocast("cuda", enabled=False):
            return self.codec.decode(codes.T.unsqueeze(0).to(self.device))

    def sample_rate(self) -> int:
        return SAMPLE_RATE
