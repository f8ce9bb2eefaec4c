"""Server-side adapter over a single-row ``vui_b200.Engine``: the reference's ``TTSEngine`` and its
``tts_process`` command loop (src/vui/serving/stream/tts_worker.py:109-834, 885-1056, 1498-1919;
message schema src/vui/serving/stream/protocol.py:1-51 in fluxions-ai/vui), reduced to what sits
either side of the decode step: prompt ingest, user-turn prefill, generation events, rewind, and the
KV on-disk formats.

* ``save_kv`` / ``load_kv`` write and read the reference's ``.pt`` layout: per layer
  ``{"k": k_cache[:, :T], "v": v_cache[:, :T]}`` of the FlashKVCache tensors, the prompt codes and text,
  ``T``, ``n_q``, ``d_model``, the checkpoint name, the conditioning bias and the projected speaker
  token.  A file whose codebook count or checkpoint differs is re-prefilled from its codes; a
  ``.safetensors`` prompt (codes + cond_bias [+ spk_token_emb], text and name in the metadata) always is.
* ``tts_process`` serves the command dicts of the reference's protocol from a queue and answers on
  another; it runs in a thread or a process.

The codec decoder and encoder are ``vui_b200.codec.QwenCodecDecoder`` and
``vui_b200.codec_encoder.QwenCodecEncoder`` (or any objects with the same methods); with an encoder attached the
user-audio commands ``encode_full`` / ``stream_start`` / ``stream_feed`` / ``stream_flush`` / ``stream_stop``
work as in the reference (tts_worker.py:1404-1490, 1804-1878).  VAD and ASR alignment are outside this
package.  Without a codec with a streaming context, ``generate`` emits ``{"type": "codes"}`` events in place
of ``{"type": "audio"}``.
"""

from __future__ import annotations

import json
import re
import time
import traceback
from collections import deque
from pathlib import Path

import torch
import torch.nn.functional as F
from torch import Tensor

from .engine import DEFAULT_WPS, FRAME_RATE, Engine, GenConfig, Segment
from .text import simple_clean

CODEC_HZ = FRAME_RATE
PROMPTS_DIR = Path("prompts")
FADE_SAMPLES = 4800  # 200 ms at 24 kHz: linear ramp over the tail of an utterance's audio


class TTSEngine:
    """One persistent ``Row`` for the lifetime of a worker, plus the prompt state that KV save / load
    and context resets need (tts_worker.py:109-155)."""

    def __init__(self, model, codec_dec=None, codec_enc=None, spk_enc=None, *, max_seq: int | None = None):
        self.model = model
        self.tok = model.text_tokenizer
        self.codec_dec, self.codec_enc, self.spk_enc = codec_dec, codec_enc, spk_enc
        self.device = model.device
        self.n_q = model.config.model.n_quantizers
        self.max_seqlen = max_seq or model.decoder.max_seqlen
        self.sc_id = self.tok.special_to_id["[SC]"] if self.tok is not None else None
        self.prompt_segments: list[tuple[str, Tensor]] | None = None
        self.prompt_codes: Tensor | None = None
        self.prompt_text: str | None = None
        self.prompt_T = 0
        self.spk_token_emb: Tensor | None = None
        self._user_spk_token: Tensor | None = None
        self.checkpoint_path: str | None = None
        self.engine: Engine | None = None
        self.row = None
        self.stream_enc = None
        self._prompt_rms = 0.0
        self._reset_user_prefill()
        self._stream_samples_fed = 0
        self._stream_frames_emitted = 0

    @property
    def T(self) -> int:
        return self.row.offset if self.row is not None else 0

    @T.setter
    def T(self, value: int) -> None:
        if self.row is not None:
            self.engine._rewind_row(self.row, value)

    def setup(self) -> "TTSEngine":
        self.engine = Engine(model=self.model, codec=self.codec_dec, max_rows=1, max_seq=self.max_seqlen)
        self.row = self.engine.new_row()
        if self.codec_enc is not None:   # tts_worker.py:231-238
            from .codec_encoder import StreamingCodecEncoder

            self.stream_enc = StreamingCodecEncoder(self.codec_enc, n_quantizers=self.n_q, max_secs=10, min_chunk_frames=12)
            self.stream_enc.setup_graph()
        return self

    # ----------------------------------------------------------- user audio -> codes (tts_worker.py:1404-1490)
    def _reset_user_prefill(self) -> None:
        self._user_codes_parts: list[Tensor] = []
        self._user_codes_consumed = 0
        self._user_text_prefilled: list[str] = []
        self._segment_start_idx = 0

    def _normalize_audio(self, audio: Tensor) -> Tensor:
        """Bring the user's level to the prompt's (gain within [0.25, 4]), tts_worker.py:369-376."""
        if self._prompt_rms < 1e-6:
            return audio
        rms = audio.float().pow(2).mean().sqrt().item()
        if rms < 1e-6:
            return audio
        return audio * max(0.25, min(4.0, self._prompt_rms / rms))

    def _need_enc(self):
        if self.codec_enc is None or self.stream_enc is None:
            raise RuntimeError("no codec encoder is attached")

    def encode_full(self, audio) -> Tensor:
        self._need_enc()
        a = torch.as_tensor(audio).float().reshape(1, 1, -1)
        a = a[..., : a.shape[-1] // 1920 * 1920].to(self.device)
        return self.codec_enc.encode(a)[0, : self.n_q].T.long().cpu()

    def stream_start(self, *, continuation: bool = False) -> None:
        self._need_enc()
        self.stream_enc.reset()
        if not continuation:
            self._reset_user_prefill()
        self._segment_start_idx = len(self._user_codes_parts)
        self._stream_samples_fed = 0
        self._stream_frames_emitted = 0

    def _took(self, codes):
        if codes is None:
            return None
        codes = codes.cpu()
        self._user_codes_parts.append(codes)
        self._stream_frames_emitted += codes.shape[0]
        return codes

    def stream_feed(self, audio):
        self._need_enc()
        a = self._normalize_audio(torch.as_tensor(audio).float())
        self._stream_samples_fed += a.numel()
        return self._took(self.stream_enc.feed(a))

    def stream_flush(self):
        self._need_enc()
        return self._took(self.stream_enc.flush())

    def stream_stop(self):
        """Re-encode the whole buffered segment once more: more accurate than the streamed partials."""
        self._need_enc()
        self.stream_enc.flush()
        total = self.stream_enc._emitted
        if total == 0:
            return None
        return self.stream_enc._encode()[0, :, :total].T.long().cpu()

    # ----------------------------------------------------------- KV position, conditioning
    def reset(self) -> None:
        self.row.reset()
        self._user_spk_token = None

    def rewind(self) -> int:
        if self.prompt_T > 0:
            self.row.rewind()
        else:
            self.row.reset()
        ctx = self.row._codec_ctx
        if ctx is not None:
            if self.prompt_codes is not None:
                ctx.set_prompt(self.prompt_codes.to(self.device).T.unsqueeze(0))
            else:
                ctx.reset()
        return self.row.offset

    def set_conditioning(self, wps: float = 0.0, sq: list | None = None) -> None:
        self.engine.set_conditioning(sq_scores=tuple(sq) if sq else None, wps_score=wps)

    # ----------------------------------------------------------------------------- prefill
    def prefill_prompt(self, segments: list[tuple[str, Tensor]], settings: dict, prompt_audio_24k=None,
                       cond_bias_override=None) -> None:
        """[spk] text_i codes_i per segment from position 0 (tts_worker.py:293-367)."""
        if cond_bias_override is not None:
            self.engine._cond_bias.copy_(cond_bias_override.to(self.engine._cond_bias.device))
        else:
            self.set_conditioning(wps=settings.get("wps_score", 0.0), sq=settings.get("sq_scores"))
        spk_emb = None
        if self.spk_enc is not None and prompt_audio_24k is not None and "spk_proj.weight" in self.model.sd:
            spk_emb = self.spk_enc.embed(prompt_audio_24k[: 30 * 24000], sr=24000)
        self.row.reset()
        self.row.prefill([Segment(text=t, codes=c) for t, c in segments], spk_emb=spk_emb)
        # a context reset passes no audio: keep speaking with the speaker token of the first upload
        if self.row._spk_token is None and self.spk_token_emb is not None:
            self.row._spk_token = self.spk_token_emb.to(self.device, self.engine.dtype)
        self.prompt_segments = segments
        self.prompt_codes = torch.cat([c for _, c in segments], dim=0)
        self.prompt_text = " ".join(t for t, _ in segments if t)
        self.prompt_T = self.row.offset
        if spk_emb is not None and self.row._spk_token is not None:
            self.spk_token_emb = self.row._spk_token

    def prefill_user_turn(self, text: str = "", codes=None, audio_16k=None, settings: dict | None = None) -> None:
        """[user_spk] text [SC] codes (tts_worker.py:511-547); VAD trimming needs the caller's audio stack."""
        if self._user_spk_token is not None:
            self.engine._prefill_emb(self.row, self._user_spk_token)
        self.row.add_user(text=text or "", codes=codes)

    def prefill_text(self, text: str) -> None:
        ids = self.tok.encode(simple_clean(text)).to(self.device)
        emb = self.model.token_emb(ids[None]).to(self.engine.dtype)
        self.engine._prefill_emb(self.row, emb + self.engine._cond_bias)

    def prefill_text_sc(self, text: str) -> float:
        """Feed text and return P([SC]) under the tied text head: learned end-pointing
        (tts_worker.py:558-573)."""
        ids = self.tok.encode(simple_clean(text)).to(self.device)
        out = self.engine._prefill_emb(self.row, self.model.token_emb(ids[None]).to(self.engine.dtype))
        logits = F.linear(out[:, -1].float(), self.model.sd["token_emb.weight"].float())
        return float(torch.softmax(logits[0], dim=-1)[self.sc_id].item())

    # -------------------------------------------------------------------------- generation
    def generate(self, text: str, settings: dict, cancel_event, audio_queue=None, *, is_new_turn: bool = True,
                 is_final_chunk: bool = False, context: str = "") -> dict:
        """Stream one chunk of agent text: timing, audio (or codes) and chunk_done events go to
        ``audio_queue``; returns totals and the generated codes (tts_worker.py:577-843)."""
        max_seq = self.max_seqlen - 10
        if self.row.offset >= max_seq - 200:  # context nearly full: start over from the prompt
            self.row.reset()
            if self.prompt_segments is not None:
                self.prefill_prompt(self.prompt_segments, settings)
            if context:
                self.prefill_text(context)
            if audio_queue:
                audio_queue.put({"type": "context_reset", "T": self.row.offset})
        wps = self.row.prompt_wps if self.row.prompt_wps > 0 else DEFAULT_WPS
        max_duration = min(settings.get("max_duration", 120), len(text.split()) / wps * 1.5 + 1.0)
        cfg = GenConfig(
            temperature=settings.get("temperature", 0.9), top_k=int(settings.get("top_k", 300)),
            top_p=settings.get("top_p"), rep_penalty=settings.get("rep_penalty", 1.1),
            rep_window=int(settings.get("rep_window", 0)), eos_threshold=settings.get("eos_threshold", 0.4),
            max_secs=max_duration, chunk_words=int(settings.get("chunk_words", 20)),
            first_chunk_words=int(settings.get("first_chunk_words", 0)) if is_new_turn else 0,
            n_codebooks=int(settings.get("n_codebooks", 0)), gate_frames=int(settings.get("gate_frames", 0)),
            gate_entropy_max=float(settings.get("gate_entropy_max", 1.9)), gate_retries=int(settings.get("gate_retries", 2)),
        )
        t0 = time.perf_counter()
        with_audio = self.row._codec_ctx is not None
        frames: list[Tensor] = []
        total_secs, cancelled, first = 0.0, False, True
        hold = deque(maxlen=3 if is_final_chunk else 1)  # look-ahead so the tail can be faded out

        def emit(item, T):
            if not audio_queue:
                return
            if with_audio:
                audio_queue.put({"type": "audio", "data": item, "T": T, "secs": item.numel() / 24000})
            else:
                audio_queue.put({"type": "codes", "data": item, "T": T, "secs": 1 / CODEC_HZ})

        codes_iter = self.engine._stream_codes(self.row, text, cfg, cancel_event, reset_rep=is_new_turn,
                                               final_turn=is_final_chunk)
        for codes in codes_iter:
            if first:
                torch.cuda.synchronize()
                ms = (time.perf_counter() - t0) * 1e3
                if audio_queue:
                    audio_queue.put({"type": "timing", "prefill_ms": 0.0, "prefill_tokens": 0, "first_frame_ms": ms,
                                     "ttfb_ms": ms})
                first = False
            frames.append(codes)
            total_secs += 1 / CODEC_HZ
            item = codes
            if with_audio:
                item = self.engine._stream_decode_frame(codes.to(self.device), cfg.n_codebooks)[0, 0].detach().float().cpu()
            if len(hold) == hold.maxlen:
                emit(*hold.popleft())
            hold.append((item, self.row.offset))
            if cancel_event is not None and cancel_event.is_set():
                cancelled = True
                break
        if hold and with_audio and (is_final_chunk or cancelled):
            tail = torch.cat([w for w, _ in hold]).clone()
            n = min(FADE_SAMPLES, tail.numel())
            tail[-n:] *= torch.linspace(1.0, 0.0, n, dtype=tail.dtype)
            emit(tail, hold[-1][1])
        else:
            for item, T in hold:
                emit(item, T)
        gen_time = time.perf_counter() - t0
        if audio_queue and not cancelled:
            audio_queue.put({"type": "chunk_done", "chunk_idx": 1, "text": text, "secs": total_secs, "frames": len(frames),
                             "gen_time": gen_time, "T": self.row.offset})
        return {"total_secs": total_secs, "total_frames": len(frames), "total_gen_time": gen_time, "cancelled": cancelled,
                "codes": torch.stack(frames) if frames else None}

    # ------------------------------------------------------------------- KV save / load
    def save_kv(self, path, name: str) -> None:
        """The reference's ``.pt`` layout (tts_worker.py:885-913)."""
        T = self.row.offset
        kv = [{"k": c.k_cache[:, :T].cpu().clone(), "v": c.v_cache[:, :T].cpu().clone()}
              for c in self.engine.flash_kv_caches]
        torch.save({
            "name": name, "codes": self.prompt_codes, "text": self.prompt_text, "T": T, "n_q": self.n_q,
            "d_model": self.model.config.model.d_model, "checkpoint": self.checkpoint_path, "kv": kv,
            "cond_bias": self.engine._cond_bias.cpu().clone(),
            "spk_token_emb": self.spk_token_emb.cpu().clone() if self.spk_token_emb is not None else None,
        }, path)

    def save_prompt(self, path, name: str) -> None:
        """The portable prompt: codes, conditioning bias and speaker token as safetensors, text and name
        in the metadata; loading it re-prefills (tts_worker.py:1030-1056 reads this format)."""
        from safetensors.torch import save_file

        t = {"codes": self.prompt_codes.contiguous(), "cond_bias": self.engine._cond_bias.cpu().contiguous()}
        if self.spk_token_emb is not None:
            t["spk_token_emb"] = self.spk_token_emb.cpu().contiguous()
        cfg = {"name": name, "text": self.prompt_text or "", "d_model": self.model.config.model.d_model, "n_q": self.n_q}
        save_file(t, str(path), metadata={"config": json.dumps(cfg)})

    def _match_n_q(self, codes: Tensor) -> Tensor:
        q = codes.shape[-1]
        if q == self.n_q:
            return codes
        return codes[..., : self.n_q].contiguous() if q > self.n_q else F.pad(codes, (0, self.n_q - q)).contiguous()

    def _reprefill_from_saved(self, saved: dict) -> None:
        spk = saved.get("spk_token_emb")
        self.spk_token_emb = spk.to(self.device) if spk is not None else None
        self.row._spk_token = self.spk_token_emb
        self.prefill_prompt([(saved.get("text", ""), self._match_n_q(saved["codes"]))], {},
                            cond_bias_override=saved["cond_bias"])

    def load_kv(self, path) -> str:
        """Restore a saved prompt: K/V copied straight into the cache when the file matches this model and
        codebook count, re-prefilled from its codes otherwise (tts_worker.py:941-1028)."""
        path = Path(path)
        if path.suffix == ".safetensors":
            return self._load_safetensors_prompt(path)
        saved = torch.load(path, map_location="cpu", weights_only=False)
        d = self.model.config.model.d_model
        if saved.get("d_model", 0) and saved["d_model"] != d:
            raise ValueError(f"KV cache d_model mismatch: saved={saved['d_model']}, model={d}")
        saved_nq = saved.get("n_q") or int(saved["codes"].shape[-1])
        ck_saved, ck_cur = saved.get("checkpoint"), self.checkpoint_path
        if (saved_nq and saved_nq != self.n_q) or (ck_saved and ck_cur and ck_saved != ck_cur):
            self._reprefill_from_saved(saved)
            return saved.get("name", path.stem)
        caches = self.engine.flash_kv_caches
        if saved["kv"][0]["k"].shape[-1] != caches[0].k_cache.shape[-1]:
            raise ValueError("KV cache head_dim mismatch")
        self.row.reset()
        self.engine._cond_bias.copy_(saved["cond_bias"].to(self.engine._cond_bias.device))
        T = saved["T"]
        for c, s in zip(caches, saved["kv"]):
            k, v = s["k"].to(self.device), s["v"].to(self.device)
            if k.dim() == 4 and k.shape[1] == c.k_cache.shape[2] and k.shape[2] == T:  # older (slots, H, T, hd) files
                k, v = k.transpose(1, 2), v.transpose(1, 2)
            n = min(k.shape[0], c.k_cache.shape[0])
            c.k_cache[:n, :T].copy_(k[:n])
            c.v_cache[:n, :T].copy_(v[:n])
        caches[0].seq_lens.fill_(T)
        self.row._prompt_offset = T
        self.prompt_T = T
        self.prompt_codes = self._match_n_q(saved["codes"])
        self.prompt_text = saved.get("text", "")
        self.prompt_segments = [(self.prompt_text, self.prompt_codes)]
        spk = saved.get("spk_token_emb")
        self.row._spk_token = spk.to(self.device) if spk is not None else None
        self.spk_token_emb = self.row._spk_token
        if self.row._codec_ctx is not None:
            self.row._codec_ctx.set_prompt(self.prompt_codes.to(self.device).T.unsqueeze(0))
        return saved.get("name", path.stem)

    def _load_safetensors_prompt(self, path: Path) -> str:
        from safetensors import safe_open

        with safe_open(str(path), framework="pt") as f:
            cfg = json.loads((f.metadata() or {}).get("config", "{}"))
            t = {k: f.get_tensor(k) for k in f.keys()}
        d = self.model.config.model.d_model
        if int(cfg.get("d_model", 0)) and int(cfg["d_model"]) != d:
            raise ValueError(f"Prompt d_model mismatch: saved={cfg['d_model']}, model={d}")
        self._reprefill_from_saved({"codes": t["codes"], "text": cfg.get("text", ""), "cond_bias": t["cond_bias"],
                                    "spk_token_emb": t.get("spk_token_emb")})
        return cfg.get("name", path.stem)

    def _kv_path_for(self, name: str) -> Path:
        return PROMPTS_DIR / f"{name}.pt"


def tts_process(cmd_queue, audio_queue, engine_or_factory, cancel_event=None) -> None:
    """Serve the protocol's command dicts until ``{"cmd": "shutdown"}`` (tts_worker.py:1498-1919).
    ``engine_or_factory`` is a set-up ``TTSEngine`` or a callable that builds one (in the reference the
    worker loads a checkpoint by path; weights reach this package as tensors)."""
    import threading

    if cancel_event is None:
        cancel_event = threading.Event()
    engine = engine_or_factory() if callable(engine_or_factory) else engine_or_factory
    ctx = torch.inference_mode()
    ctx.__enter__()
    audio_queue.put({"type": "ready"})
    try:
        while True:
            msg = cmd_queue.get()
            cmd = msg.get("cmd")
            try:
                if cmd == "shutdown":
                    break
                elif cmd == "reset":
                    engine.reset()
                    audio_queue.put({"type": "done", "T": 0, "total_secs": 0})
                elif cmd == "rewind":
                    audio_queue.put({"type": "done", "T": engine.rewind(), "total_secs": 0})
                elif cmd == "reprefill":
                    if engine.prompt_segments is not None:
                        engine.prefill_prompt(engine.prompt_segments, msg.get("settings", {}))
                    audio_queue.put({"type": "prompt_loaded", "T": engine.T, "text": engine.prompt_text or ""})
                elif cmd == "set_cond":
                    engine.set_conditioning(wps=msg.get("wps", 0), sq=msg.get("sq"))
                elif cmd == "allocate_and_prefill":
                    codes = msg.get("codes")
                    if codes is None:
                        if engine.codec_enc is None:
                            raise RuntimeError("allocate_and_prefill needs 'codes' (T, Q): no codec encoder is attached")
                        codes = engine.codec_enc.encode(msg["audio_16k"])
                    audio = msg.get("audio_24k")
                    engine.prefill_prompt([(msg.get("text") or "", codes)], msg.get("settings", {}),
                                          prompt_audio_24k=torch.as_tensor(audio).float() if audio is not None else None)
                    audio_queue.put({"type": "prompt_loaded", "T": engine.T, "text": engine.prompt_text or ""})
                elif cmd == "generate":
                    if cancel_event.is_set():
                        continue
                    res = engine.generate(msg["text"], msg.get("settings", {}), cancel_event, audio_queue=audio_queue,
                                          is_new_turn=msg.get("new_turn", True), is_final_chunk=msg.get("is_final", False),
                                          context=msg.get("context", ""))
                    if res["cancelled"]:
                        audio_queue.put({"type": "cancelled", "T": engine.T})
                    else:
                        audio_queue.put({"type": "done", "T": engine.T, "total_secs": res["total_secs"],
                                         "total_frames": res["total_frames"], "total_gen_time": res["total_gen_time"]})
                elif cmd == "prefill_user_turn":
                    engine.prefill_user_turn(text=msg.get("text", ""), codes=msg.get("codes"),
                                             audio_16k=msg.get("audio_16k"), settings=msg.get("settings"))
                    audio_queue.put({"type": "user_prefilled", "T": engine.T})
                elif cmd == "prefill_text":
                    engine.prefill_text(msg["text"])
                    audio_queue.put({"type": "text_prefilled", "T": engine.T})
                elif cmd == "prefill_text_sc":
                    p = engine.prefill_text_sc(msg["text"])
                    audio_queue.put({"type": "sc_prob", "prob": p, "text": msg["text"], "T": engine.T})
                elif cmd == "save_kv":
                    try:
                        name = msg["name"]
                        path = Path(msg["path"]) if msg.get("path") else engine._kv_path_for(re.sub(r"[^\w\-]", "_", name))
                        path.parent.mkdir(parents=True, exist_ok=True)
                        engine.save_kv(path, name)
                        audio_queue.put({"type": "kv_saved", "name": name, "ok": True})
                    except Exception as e:  # noqa: BLE001
                        audio_queue.put({"type": "kv_saved", "name": msg.get("name", ""), "ok": False, "msg": str(e)})
                elif cmd == "load_kv":
                    try:
                        path = Path(msg["path"]) if msg.get("path") else engine._kv_path_for(msg.get("name") or msg["file"])
                        name = engine.load_kv(path)
                        audio_queue.put({"type": "kv_loaded", "name": name, "ok": True, "T": engine.T,
                                         "text": engine.prompt_text})
                    except Exception:  # noqa: BLE001
                        traceback.print_exc()
                        audio_queue.put({"type": "kv_loaded", "name": msg.get("name", ""), "ok": False, "T": 0, "text": ""})
                elif cmd == "cancel":
                    rewind_to = msg.get("rewind_to")
                    if rewind_to is not None and rewind_to < engine.T:
                        engine.T = rewind_to
                    cancel_event.clear()
                elif cmd == "encode_full":
                    try:
                        audio_queue.put({"type": "encoded", "codes": engine.encode_full(msg["audio"])})
                    except Exception:  # noqa: BLE001 - the reference answers None and keeps serving
                        traceback.print_exc()
                        audio_queue.put({"type": "encoded", "codes": None})
                elif cmd == "stream_start":
                    engine.stream_start(continuation=bool(msg.get("continuation", False)))
                elif cmd in ("stream_feed", "stream_flush"):
                    codes = engine.stream_feed(msg["audio"]) if cmd == "stream_feed" else engine.stream_flush()
                    if codes is not None:
                        audio_queue.put({"type": "codes", "codes": codes})
                elif cmd == "stream_stop":
                    try:
                        codes = engine.stream_stop()
                        if codes is not None:   # the re-encoded segment replaces its streamed partials
                            engine._user_codes_parts = engine._user_codes_parts[: engine._segment_start_idx] + [codes]
                        audio_queue.put({"type": "codes_final", "n_frames": 0 if codes is None else codes.shape[0]})
                    except Exception:  # noqa: BLE001
                        traceback.print_exc()
                        audio_queue.put({"type": "codes_final", "n_frames": 0})
                elif cmd == "decode_prompt":
                    if engine.prompt_codes is not None and engine.codec_dec is not None:
                        codes = engine.prompt_codes.long().to(engine.device).T.unsqueeze(0)
                        wav = engine.codec_dec.decode_chunked(codes, chunk_size=200)[0, 0].cpu().float()
                        audio_queue.put({"type": "prompt_audio", "audio": wav, "sample_rate": 24000,
                                         "codes_shape": list(engine.prompt_codes.shape)})
                    else:
                        audio_queue.put({"type": "prompt_audio", "audio": None})
                elif cmd == "get_state":
                    audio_queue.put({"type": "state", "T": engine.T, "max_T": engine.max_seqlen,
                                     "has_prompt": engine.prompt_codes is not None, "prompt_text": engine.prompt_text or ""})
                else:
                    audio_queue.put({"type": "error", "msg": f"unknown or unsupported command '{cmd}'"})
            except Exception as e:  # noqa: BLE001
                traceback.print_exc()
                audio_queue.put({"type": "error", "msg": str(e)})
    finally:
        ctx.__exit__(None, None, None)
