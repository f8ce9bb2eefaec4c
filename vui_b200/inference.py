"""The reference's older single-stream API over the B200 engine: ``InferenceState`` and
``stream_frames`` (src/vui/inference.py:140-367, 507-734 in fluxions-ai/vui; used by demo/cli.py).

Same names, arguments and yield protocol.  Underneath, the state is one slot of a
``vui_b200.Engine``: prefill goes through ``vuib_prefill``, a decode frame is one backbone
step plus one depth step of libvuib200.  ``top_p``, which only this older loop honours
(src/vui/sampling.py:23-43), is applied to the cb0 distribution on the device with torch ops;
the chosen code is then handed to the depth step.
"""

from __future__ import annotations

import ctypes as C
from collections import deque

import torch
import torch.nn.functional as F
from torch import Tensor

from .engine import FRAME_RATE, RQ_TOP_K, Engine
from .text import chunk_text, simple_clean

CODEC_HZ = FRAME_RATE


class InferenceState:
    """One stream's KV position, prompt checkpoint and cached speaker tokens
    (src/vui/inference.py:140-367).  ``codec`` is carried for callers that decode audio
    themselves; nothing here runs it."""

    def __init__(self, model, codec=None, chunk_frames: int = 7, ctx_frames: int = 3,
                 sq_scores: tuple[float, ...] | None = None, wps_score: float = 1.0,
                 codec_graphs: bool = True, compile_rq: bool = False, max_seq: int | None = None):
        self.model = model
        self.codec = codec
        self.chunk_frames = chunk_frames
        self.ctx_frames = ctx_frames
        self.device = model.device
        self.dtype = model.dtype
        self.engine = Engine(model=model, codec=codec, max_rows=1, max_seq=max_seq)
        self.row = self.engine.new_row()
        self.offset = 0
        self._ckpt_offset = 0
        self._ckpt_spk_token: Tensor | None = None
        self._ckpt_spk_token_2: Tensor | None = None
        self.engine.set_conditioning(sq_scores=sq_scores, wps_score=wps_score)

    # -- position only: K/V data is never zeroed or copied (inference.py:222-232, 322-345)
    def reset(self) -> None:
        self.rewind(0)

    def teardown(self) -> None:
        self.row.close()

    def checkpoint(self) -> int:
        self._ckpt_offset = self.offset
        return self.offset

    def rewind(self, offset: int | None = None) -> int:
        target = offset if offset is not None else self._ckpt_offset
        self.engine._rewind_row(self.row, target)
        self.offset = target
        return target

    def _forward_emb(self, emb: Tensor) -> Tensor:
        """Write (1, T, d) embeddings at the current offset; returns the final-norm output."""
        out = self.engine._prefill_emb(self.row, emb)
        self.offset += emb.reshape(-1, emb.shape[-1]).shape[0]
        return out

    def _tok(self):
        tok = self.model.text_tokenizer
        if tok is None:
            raise RuntimeError("this model was built without a text tokenizer")
        return tok

    @torch.inference_mode()
    def prefill(self, segments: list[tuple[str, str | Tensor]], cond_last: bool = True) -> int:
        """Interleaved ("text", str) / ("audio", codes (T, Q)) segments; the conditioning bias goes on
        the last segment only unless ``cond_last`` is False (inference.py:234-264)."""
        bias = self.engine._cond_bias
        for i, (kind, data) in enumerate(segments):
            use_bias = (not cond_last) or i == len(segments) - 1
            if kind == "text":
                ids = self._tok().encode(data).to(self.device)
                emb = self.model.token_emb(ids[None]).to(self.dtype)
            else:
                emb = self.engine._audio_emb(data)
            self._forward_emb(emb + bias if use_bias else emb)
        return self.offset

    @torch.inference_mode()
    def prefill_prompt(self, prompt_segments=None, prompt_segments_2=None, spk_emb=None, spk_emb_2=None) -> int:
        """[spk] text codes for every segment of one or two speakers, from position 0
        (inference.py:270-317).  Use with checkpoint() + rewind() to reuse the prompt across turns."""
        self.reset()
        self._ckpt_spk_token = self.engine._embed_speaker(spk_emb)
        self._ckpt_spk_token_2 = self.engine._embed_speaker(spk_emb_2)
        for segs, spk in ((prompt_segments, self._ckpt_spk_token), (prompt_segments_2, self._ckpt_spk_token_2)):
            for text, codes in segs or []:
                if spk is not None:
                    self._forward_emb(spk)
                if text:
                    ids = self._tok().encode(simple_clean(text)).to(self.device)
                    self._forward_emb(self.model.token_emb(ids[None]).to(self.dtype))
                self._forward_emb(self.engine._audio_emb(codes))
        return self.offset


def _sample_cb0(logits: Tensor, temperature: float, top_k: int | None, top_p: float | None,
                generator: torch.Generator | None) -> Tensor:
    """_sample_codes of the older loop (inference.py:491-504) with the filters of
    src/vui/sampling.py:13-43: softmax(l / T), nucleus and/or top-k on the probabilities, draw."""
    probs = F.softmax(logits.float() / temperature, dim=-1)
    if top_p is not None and top_p > 0:
        srt, idx = torch.sort(probs, dim=-1, descending=True)
        csum = torch.cumsum(srt, dim=-1)
        srt = srt * (~(csum - srt > top_p)).float()
        srt = srt / srt.sum(dim=-1, keepdim=True)
        if top_k is not None and top_k > 0:
            kth = torch.topk(srt, min(top_k, srt.shape[-1]), dim=-1).values[..., -1:]
            srt = srt * (srt >= kth).float()
            srt = srt / srt.sum(dim=-1, keepdim=True)
        pick = torch.multinomial(srt, 1, generator=generator)
        return torch.gather(idx, -1, pick).squeeze(-1)
    if top_k is not None and top_k > 0:
        kth = torch.topk(probs, min(top_k, probs.shape[-1]), dim=-1).values[..., -1:]
        probs = probs * (probs >= kth).float()
        probs = probs / probs.sum(dim=-1, keepdim=True)
    return torch.multinomial(probs, 1, generator=generator).squeeze(-1)


@torch.inference_mode()
def stream_frames(state: InferenceState, text: str, *, prompt_segments=None, prompt_segments_2=None,
                  spk_emb=None, spk_emb_2=None, temperature: float = 0.9, top_k: int | None = 100,
                  top_p: float | None = None, rep_penalty: float = 1.0, rep_window: int = 0,
                  sq_scores=None, wps_score: float = 0.0, chunk_words: int = 5, max_secs: float = 120.0,
                  max_turn_secs: float = 15.0, eos_threshold: float = 0.45, min_turn_secs: float = 0.5,
                  resume: bool = False, generator: torch.Generator | None = None):
    """Per-frame code generator: yields ``(code_frame (Q,) long on the GPU, turn_end)`` where
    ``turn_end`` is None inside a turn and the chunk's info dict (with 'frames' and 'secs') on its
    last frame (inference.py:507-734).  ``resume`` skips the reset and the prompt prefill: the
    caller has run ``state.prefill_prompt`` and rewound to its checkpoint.

    cb0 is drawn here (repetition penalty over a rolling window, top-k and/or nucleus), codebooks
    1..Q-1 by the depth step at the same temperature with its fixed top-k of 100.  ``generator``
    (an addition) seeds the cb0 draws."""
    eng, model, dev = state.engine, state.model, state.device
    tok = state._tok()
    sc_id = tok.special_to_id["[SC]"]
    # the older loop disables the words-per-second conditioning at inference (inference.py:556-557)
    eng.set_conditioning(sq_scores=sq_scores, wps_score=0.0)
    cond_bias = eng._cond_bias
    spk_token = eng._embed_speaker(spk_emb)
    spk_token_2 = eng._embed_speaker(spk_emb_2)
    if resume:
        spk_token = spk_token if spk_token is not None else state._ckpt_spk_token
        spk_token_2 = spk_token_2 if spk_token_2 is not None else state._ckpt_spk_token_2
    chunks = chunk_text(text, min_words=chunk_words)
    if not chunks:
        return
    Q, CS = eng.Q, eng.CS
    window: deque[int] = deque(maxlen=rep_window if rep_window > 0 else None)
    counts: dict[int, int] = {}
    # cb0 is chosen on this side: the device sampler takes the arg-max of a one-hot row for cb0 and draws
    # codebooks 1..Q-1 at `temperature` with the depth top-k
    eng._set_sampling(temperature, 1, RQ_TOP_K, 1.0, 0, 0)
    P = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    onehot = torch.zeros(1, CS, device=dev, dtype=eng.dtype)
    codes_buf = torch.zeros(1, Q, device=dev, dtype=torch.long)
    slot = torch.tensor([state.row.idx], device=dev, dtype=torch.int32)

    def depth(cb0_logits: Tensor, hidden: Tensor) -> Tensor:
        lg = cb0_logits.reshape(1, CS).float()
        if rep_penalty > 1.0 and counts:
            ids = torch.tensor(list(counts), device=dev)
            f = torch.tensor([rep_penalty ** counts[i] for i in counts], device=dev)
            v = lg[0, ids]
            lg = lg.clone()
            lg[0, ids] = torch.where(v > 0, v / f, v * f)
        code0 = int(_sample_cb0(lg, temperature, top_k, top_p, generator).item())
        if window.maxlen is not None and len(window) == window.maxlen:
            old = window[0]
            counts[old] -= 1
            if counts[old] == 0:
                del counts[old]
        window.append(code0)
        counts[code0] = counts.get(code0, 0) + 1
        onehot.zero_()
        onehot[0, code0] = 1.0
        hid = hidden.reshape(1, -1).to(eng.dtype).contiguous()
        eng._ck(eng._lib.vuib_depth_step(eng._handle, 1, P(slot), P(hid), P(onehot), None, 0, P(codes_buf), None,
                                         eng._stream))
        return codes_buf[0].clone()

    max_frames, max_per_turn = int(max_secs * CODEC_HZ), int(max_turn_secs * CODEC_HZ)
    min_frames = int(min_turn_secs * CODEC_HZ)
    max_seq = eng.max_seq - 10
    if not resume:
        state.reset()
        if prompt_segments is not None or prompt_segments_2 is not None:
            first_sc = chunks[0]["sc"]
            for segs, spk, last_speaker in ((prompt_segments, spk_token, False), (prompt_segments_2, spk_token_2, True)):
                for i, (seg_text, seg_codes) in enumerate(segs or []):
                    if spk is not None:
                        state._forward_emb(spk)
                    if seg_text:
                        ids = tok.encode(simple_clean(seg_text)).to(dev)
                        if i == len(segs) - 1 and first_sc and (last_speaker or prompt_segments_2 is None):
                            ids = torch.cat([ids, torch.tensor([sc_id], device=dev)])
                        state._forward_emb(model.token_emb(ids[None]).to(eng.dtype))
                    state._forward_emb(eng._audio_emb(seg_codes))
    total = 0
    speaker = 1 if prompt_segments_2 is not None else 0
    for turn, chunk in enumerate(chunks):
        if state.offset >= max_seq or total >= max_frames:
            break
        if chunk["sc"]:
            speaker = 1 - speaker
        spk = spk_token_2 if (speaker == 1 and spk_token_2 is not None) else spk_token
        if spk is not None:
            state._forward_emb(spk)
        ids = tok.encode(chunk["text"]).to(dev)
        if turn + 1 < len(chunks) and chunks[turn + 1]["sc"]:
            ids = torch.cat([ids, torch.tensor([sc_id], device=dev)])
        emb = model.token_emb(ids[None]).to(eng.dtype) + cond_bias
        if state.offset + emb.shape[1] >= max_seq:
            break
        hidden = state._forward_emb(emb)[0, -1]
        cb0 = torch.empty(1, CS, device=dev, dtype=eng.dtype)
        eos = torch.empty(1, 1, device=dev, dtype=eng.dtype)
        hid = hidden.reshape(1, -1).contiguous()
        eng._ck(eng._lib.vuib_heads(eng._handle, 1, P(hid), P(cb0), P(eos), eng._stream))
        pending = depth(cb0, hidden)
        n_turn, codes_in = 1, pending
        total += 1
        for step in range(1, max_per_turn):
            if state.offset >= max_seq or total >= max_frames:
                break
            hid_n, cb0_n, eos_n = model_decode_step(state, codes_in)
            nxt = depth(cb0_n, hid_n)
            if step >= min_frames and torch.sigmoid(eos_n.float()).item() > eos_threshold:
                break
            yield pending, None
            pending, codes_in = nxt, nxt
            n_turn += 1
            total += 1
        chunk["frames"] = n_turn
        chunk["secs"] = n_turn / CODEC_HZ
        yield pending, chunk


def model_decode_step(state: InferenceState, codes: Tensor):
    """One backbone step at ``state.offset`` on the state's own slot (Vui.decode_step, model.py:1289-1300)."""
    eng = state.engine
    eng._g_codes_in[0].copy_(codes.to(eng.device))
    eng._rewind_row(state.row, state.offset)
    hidden, cb0, eos = eng._decode_step()
    state.offset += 1
    return hidden[:1].clone(), cb0[:1].clone(), eos[:1].clone()
