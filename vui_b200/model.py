"""Weights and shape of a Vui model as the B200 engine consumes them.

This is the host-side counterpart of ``vui.model.Vui`` (src/vui/model.py:1054-1311
in fluxions-ai/vui) reduced to what the decode path needs: the bf16 parameter
tensors under the reference's state-dict names, the RoPE table, and the few
embedding helpers the engine's prefill uses.  All arithmetic of the decode step
itself happens in libvuib200; torch is used here for device memory and for the
embedding lookups that feed a prefill.
"""

from __future__ import annotations

import json
import math
from dataclasses import asdict, dataclass
from types import SimpleNamespace

import torch
import torch.nn.functional as F
from torch import Tensor


@dataclass(frozen=True)
class VuiShape:
    """Architecture fields of vui.config.VuiConfig (src/vui/config.py:16-54) that
    the decode path reads, with the Vui-Nano benchmark shape as defaults."""

    d_model: int = 1024
    n_layers: int = 24
    n_heads: int = 16
    n_kv_heads: int = 8
    intermediate_size: int = 3072
    rope_theta: float = 1e6
    vocab_size: int = 151936
    n_quantizers: int = 16
    codebook_size: int = 2048
    rq_d_model: int = 512
    rq_n_layers: int = 4
    rq_n_heads: int = 8
    norm_eps: float = 1e-5
    rq_norm_eps: float = 1e-6
    max_secs: float = 60.0
    codec_hz: float = 12.5

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_heads

    @property
    def rq_ffn(self) -> int:
        # RQBlock sizes its MLP itself (model.py:587-588)
        h = int(self.rq_d_model * 8 / 3)
        return 64 * ((h + 63) // 64)

    @property
    def max_seq_len(self) -> int:
        # Config.max_seq_len (config.py:71-76) + n_quantizers (model.py:1127)
        audio = int(self.max_secs * self.codec_hz)
        total = audio + int(audio * 2.5)
        return 64 * ((total + 63) // 64) + self.n_quantizers


def state_dict_shapes(s: VuiShape) -> dict[str, tuple[int, ...]]:
    """Parameter names and shapes of the reference state dict (the key list is in
    src/vui/mlx/tts/weights.py:121-192; shapes from src/vui/model.py)."""
    d, hd = s.d_model, s.head_dim
    qkv = (s.n_heads + 2 * s.n_kv_heads) * hd
    rd, rf, Q, CS = s.rq_d_model, s.rq_ffn, s.n_quantizers, s.codebook_size
    out: dict[str, tuple[int, ...]] = {
        "token_emb.weight": (s.vocab_size, d),
        "audio_emb.embedding.weight": (Q * CS, d),
        "codec_head.weight": (CS, d),
        "eos_head.weight": (1, d),
        "eos_head.bias": (1,),
        "decoder.norm.weight": (d,),
    }
    for i in range(s.n_layers):
        p = f"decoder.blocks.{i}."
        out[p + "attn_norm.weight"] = (d,)
        out[p + "attn.Wqkv.weight"] = (qkv, d)
        out[p + "attn.out_proj.weight"] = (d, d)
        out[p + "mlp_norm.weight"] = (d,)
        out[p + "mlp.w1.weight"] = (s.intermediate_size, d)
        out[p + "mlp.w3.weight"] = (s.intermediate_size, d)
        out[p + "mlp.w2.weight"] = (d, s.intermediate_size)
    r = "rq_transformer."
    out[r + "backbone_proj.weight"] = (rd, d)
    out[r + "code_emb.embedding.weight"] = ((Q - 1) * CS, rd)
    out[r + "pos_emb.weight"] = (Q, rd)
    out[r + "head_W"] = (Q - 1, CS, rd)
    out[r + "norm.weight"] = (rd,)
    for i in range(s.rq_n_layers):
        p = f"{r}blocks.{i}."
        out[p + "attn_norm.weight"] = (rd,)
        out[p + "Wqkv.weight"] = (3 * rd, rd)
        out[p + "out_proj.weight"] = (rd, rd)
        out[p + "mlp_norm.weight"] = (rd,)
        out[p + "w1.weight"] = (rf, rd)
        out[p + "w3.weight"] = (rf, rd)
        out[p + "w2.weight"] = (rd, rf)
    return out


def freqs_cis_table(head_dim: int, max_seqlen: int, theta: float) -> Tensor:
    """[cos, sin] table (max_seqlen, head_dim, 2), fp32: angle = pos * theta^(-2j/dim),
    each angle repeated for both members of an interleaved pair
    (precompute_freqs_cis, src/vui/rope.py:60-77)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    ang = torch.outer(torch.arange(max_seqlen, dtype=torch.float32), inv)
    ang = torch.repeat_interleave(ang, 2, dim=-1)
    return torch.stack((torch.cos(ang), torch.sin(ang)), dim=-1)


class VuiB200(torch.nn.Module):
    """Parameter container.  ``sd`` maps reference state-dict names to tensors;
    they are moved to ``device`` as bf16 and kept contiguous."""

    def __init__(self, shape: VuiShape, sd: dict[str, Tensor], device="cuda", tokenizer=None):
        super().__init__()
        self.shape = shape
        self.device_ = torch.device(device)
        want = state_dict_shapes(shape)
        self.sd: dict[str, Tensor] = {}
        for name, shp in want.items():
            if name not in sd:
                raise KeyError(f"state dict lacks '{name}'")
            t = sd[name]
            if tuple(t.shape) != shp:
                raise ValueError(f"'{name}' has shape {tuple(t.shape)}, expected {shp}")
            self.sd[name] = t.to(self.device_, torch.bfloat16).contiguous()
        for opt in ("spk_proj.weight", "noisy_emb", "sq_proj.weight", "wps_proj.proj.weight"):
            if opt in sd:
                self.sd[opt] = sd[opt].to(self.device_, torch.bfloat16).contiguous()
        self.text_tokenizer = tokenizer
        max_seqlen = shape.max_seq_len
        self.decoder = SimpleNamespace(
            max_seqlen=max_seqlen,
            # built in fp32 on the host, then cast, as Vui(...).bfloat16() does (model.py:1226)
            freqs_cis=freqs_cis_table(shape.head_dim, max_seqlen, shape.rope_theta)
            .to(torch.bfloat16).to(self.device_).contiguous(),
            flash_kv_caches=None,
            n_kv_heads=shape.n_kv_heads,
            head_dim=shape.head_dim,
        )
        # reference-style view of the config (engine.py:318-320 reads model.config.model.*)
        self.config = SimpleNamespace(model=SimpleNamespace(**asdict(shape)))
        self._cond_bias = None

    # -- constructors ---------------------------------------------------------
    @classmethod
    def random_init(cls, shape: VuiShape = VuiShape(), seed: int = 0, device="cuda", tokenizer=None):
        """Seeded random-init weights: every matrix N(0, 0.02), norm gains 1, eos
        bias 0, drawn in fp32 on the CPU in state-dict order from one generator."""
        g = torch.Generator(device="cpu").manual_seed(seed)
        sd = {}
        for name, shp in state_dict_shapes(shape).items():
            if name.endswith("norm.weight"):
                t = torch.ones(shp)
            elif name == "eos_head.bias":
                t = torch.zeros(shp)
            else:
                t = torch.empty(shp).normal_(0.0, 0.02, generator=g)
            sd[name] = t.to(torch.bfloat16)
        return cls(shape, sd, device=device, tokenizer=tokenizer)

    @classmethod
    def from_checkpoint(cls, path: str, device="cuda", tokenizer=None, **overrides):
        """Load a reference checkpoint: safetensors with a JSON ``config`` in its
        metadata, or a ``.pt`` dict {config, model} (Vui.from_pretrained,
        model.py:1155-1219)."""
        if path.endswith(".safetensors"):
            from safetensors.torch import load_file, safe_open

            with safe_open(path, framework="pt") as f:
                config = json.loads(f.metadata()["config"])
            sd = load_file(path)
        else:
            ck = torch.load(path, map_location="cpu", weights_only=True)
            config, sd = ck["config"], ck["model"]
        sd = {k.replace("module.", "").replace("text_embedding.", "token_emb."): v for k, v in sd.items()}
        m = dict(config.get("model", {}))
        if not m.get("use_rq_transformer", False):
            raise ValueError("only checkpoints with the RQ depth transformer are supported")
        n_heads = m["n_heads"]
        shape = VuiShape(
            d_model=m["d_model"], n_layers=m["n_layers"], n_heads=n_heads,
            n_kv_heads=m.get("n_kv_heads") or n_heads,
            intermediate_size=m.get("intermediate_size") or sd["decoder.blocks.0.mlp.w1.weight"].shape[0],
            rope_theta=m.get("rope_theta", 10000.0), vocab_size=sd["token_emb.weight"].shape[0],
            n_quantizers=m["n_quantizers"], codebook_size=m["codebook_size"],
            rq_d_model=m["rq_d_model"], rq_n_layers=m["rq_n_layers"], rq_n_heads=m["rq_n_heads"],
            max_secs=config.get("data", {}).get("max_secs", 360), codec_hz=m.get("codec_hz", 12.5),
            **overrides,
        )
        for k in ("rope_dim", "window_size", "global_every"):
            if m.get(k):
                raise ValueError(f"checkpoint uses {k}, which this engine does not implement")
        return cls(shape, sd, device=device, tokenizer=tokenizer)

    # -- helpers the engine's prefill uses ------------------------------------
    @property
    def device(self):
        return self.device_

    @property
    def dtype(self):
        return torch.bfloat16

    def token_emb(self, ids: Tensor) -> Tensor:
        return F.embedding(ids.to(self.device_), self.sd["token_emb.weight"])

    def embed_audio(self, codes: Tensor) -> Tensor:
        """codes (..., Q') long -> (..., d): sum of per-codebook rows (model.py:559-563)."""
        codes = codes.to(self.device_)
        off = torch.arange(codes.shape[-1], device=self.device_) * self.shape.codebook_size
        return F.embedding(codes + off, self.sd["audio_emb.embedding.weight"]).sum(dim=-2)

    def embed_speaker(self, spk_emb: Tensor) -> Tensor:
        if "spk_proj.weight" not in self.sd:
            raise RuntimeError("this checkpoint has no spk_proj")
        return F.linear(spk_emb.to(self.device_, torch.bfloat16), self.sd["spk_proj.weight"]).reshape(1, 1, -1)

    # ---- the reference's older single-stream API (Vui.setup_decode_graph / decode_step,
    #      model.py:1228-1300; used by demo/cli.py and inference.py) --------------------------
    def setup_decode_graph(self, pool=None, max_seq: int | None = None) -> None:
        """One slot, static I/O buffers and one captured backbone step.  ``pool`` is accepted
        for signature compatibility (the library works in a caller-provided workspace)."""
        from .engine import Engine  # the engine owns the native handle; imported late to avoid a cycle

        self._decode_engine = Engine(model=self, max_rows=1, max_seq=max_seq)
        self._decode_row = self._decode_engine.new_row()
        self._decode_graph = None

    @torch.inference_mode()
    def decode_step(self, codes: Tensor, pos: int) -> tuple[Tensor, Tensor, Tensor]:
        """Feed one frame of codes (Q,) at position ``pos``: returns the static buffers
        (hidden (1, d), codec logits (1, CS), eos logit (1, 1)); the KV length becomes pos + 1."""
        eng = getattr(self, "_decode_engine", None)
        if eng is None:
            raise RuntimeError("call setup_decode_graph() first")
        eng._g_codes_in[0].copy_(codes.to(eng.device))
        eng._rewind_row(self._decode_row, int(pos))
        if self._decode_graph is None:
            eng._decode_step()  # warm-up outside capture (it advances the position: put it back)
            eng._rewind_row(self._decode_row, int(pos))
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                eng._decode_step()
            eng._rewind_row(self._decode_row, int(pos))
            self._decode_graph = g
        self._decode_graph.replay()
        return eng._g_hidden_out[:1], eng._g_cb0_out[:1], eng._g_eos_out[:1].reshape(1, 1)

    def weight_bytes_per_step(self) -> int:
        """Distinct weight bytes one decode step reads: every backbone, head and
        depth-transformer matrix once (embedding tables are gathered, not streamed)."""
        skip = ("token_emb.weight", "audio_emb.embedding.weight", "rq_transformer.code_emb.embedding.weight",
                "spk_proj.weight", "noisy_emb")
        return sum(t.numel() * 2 for k, t in self.sd.items() if k not in skip)
