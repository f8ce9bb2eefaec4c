"""CPU/torch restatement of Vui Nano's per-codec-frame decode path.

TEST INFRASTRUCTURE ONLY.  This module is the checker for the CUDA path in
``vui_b200``: it may be imported by ``tests/``, by ``__graft_entry__.smoke()``
and by ``bench.py``'s CPU-baseline / ``--impl reference`` legs, and by nothing
that ships.  The product never routes through it.

It restates, op by op, the algorithm of the reference PyTorch engine
(fluxions-ai/vui, paths below are relative to that project):

* ``src/vui/model.py``   - RMSNorm 286-297, MHA.forward_flash 204-258,
  LlamaMLP 261-283, Block.forward_flash 359-375, Decoder.forward_flash 534-549,
  AudioEmbedding 552-563, RQBlock 577-635, RQTransformer.generate 686-728 and
  ``_generate_graph_body_kv`` 908-986, ``Vui._decode_step_inner`` 1280-1287.
* ``src/vui/rope.py``    - rotate_half 16-20, apply_rotary_emb 23-57,
  precompute_freqs_cis 60-77.
* ``src/vui/engine.py``  - ``_backbone_decode_body`` 434-449, ``_prefill_emb``
  674-694, ``_sample_cb0`` 855-863, ``_rep_apply`` 571-576, frame protocol of
  ``_render_rows`` 914-951 / 1023-1079.

Two arithmetic modes:

* ``dtype=torch.float32`` - the reference's CPU path (benchmark configuration 1).
* ``dtype=torch.bfloat16`` - the reference's inference precision: every tensor
  the reference materialises in bf16 is rounded to bf16 here at the same point
  (embedding sum, both RMSNorm roundings, each Linear output, the three RoPE
  roundings, attention output, SiLU, gate product, residual adds, logits).
  GEMMs accumulate in fp32 (``F.linear`` on bf16 does, on CPU and through
  cuBLAS); attention is computed in fp32 from bf16 q/k/v with one rounding of
  the output, which is what flash-attn's fp32 softmax and torch's SDPA math
  backend (which upcasts bf16 operands) both amount to up to summation order.

Parity pin: ``tests/golden/make_golden.py`` runs the reference's own classes
(imported from a checkout, CPU) on the same seeded weights and stores their
outputs as fixtures; ``tests/test_oracle_golden.py`` checks this restatement
against them.  The reference itself ships no golden vectors for this path.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F
from torch import Tensor


# ---------------------------------------------------------------------------
# Shapes
# ---------------------------------------------------------------------------


@dataclass(frozen=True)
class OracleConfig:
    """Model shape.  Defaults are the Vui-Nano shape the benchmark is quoted on."""

    d_model: int = 1024
    n_layers: int = 24
    n_heads: int = 16
    n_kv_heads: int = 8
    ffn: int = 3072
    rope_theta: float = 1e6
    vocab: int = 151936
    n_quantizers: int = 16
    codebook_size: int = 2048
    rq_d_model: int = 512
    rq_n_layers: int = 4
    rq_n_heads: int = 8
    norm_eps: float = 1e-5  # Block / Decoder.norm (model.py:310,391,436)
    rq_norm_eps: float = 1e-6  # RMSNorm default used by RQBlock (model.py:287)

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_heads

    @property
    def rq_head_dim(self) -> int:
        return self.rq_d_model // self.rq_n_heads

    @property
    def rq_ffn(self) -> int:
        # model.py:587-588: int(d*8/3) rounded up to a multiple of 64
        h = int(self.rq_d_model * 8 / 3)
        return 64 * ((h + 63) // 64)


TINY = OracleConfig(
    d_model=256, n_layers=2, n_heads=4, n_kv_heads=2, ffn=512, vocab=1000,
    n_quantizers=16, codebook_size=2048, rq_d_model=512, rq_n_layers=1, rq_n_heads=8,
)


# ---------------------------------------------------------------------------
# Weights: seeded N(0, 0.02), norm gains 1, eos bias 0; reference key names
# (src/vui/mlx/tts/weights.py:121-192 lists them; model.py defines them).
# ---------------------------------------------------------------------------


def weight_shapes(cfg: OracleConfig) -> dict[str, tuple[int, ...]]:
    d, hd = cfg.d_model, cfg.head_dim
    qkv = (cfg.n_heads + 2 * cfg.n_kv_heads) * hd
    rd, rf = cfg.rq_d_model, cfg.rq_ffn
    Q, CS = cfg.n_quantizers, cfg.codebook_size
    s: dict[str, tuple[int, ...]] = {
        "token_emb.weight": (cfg.vocab, d),
        "audio_emb.embedding.weight": (Q * CS, d),
        "codec_head.weight": (CS, d),
        "eos_head.weight": (1, d),
        "eos_head.bias": (1,),
        "decoder.norm.weight": (d,),
    }
    for i in range(cfg.n_layers):
        p = f"decoder.blocks.{i}."
        s[p + "attn_norm.weight"] = (d,)
        s[p + "attn.Wqkv.weight"] = (qkv, d)
        s[p + "attn.out_proj.weight"] = (d, d)
        s[p + "mlp_norm.weight"] = (d,)
        s[p + "mlp.w1.weight"] = (cfg.ffn, d)
        s[p + "mlp.w3.weight"] = (cfg.ffn, d)
        s[p + "mlp.w2.weight"] = (d, cfg.ffn)
    r = "rq_transformer."
    s[r + "backbone_proj.weight"] = (rd, d)
    s[r + "code_emb.embedding.weight"] = ((Q - 1) * CS, rd)
    s[r + "pos_emb.weight"] = (Q, rd)
    s[r + "head_W"] = (Q - 1, CS, rd)
    s[r + "norm.weight"] = (rd,)
    for i in range(cfg.rq_n_layers):
        p = f"{r}blocks.{i}."
        s[p + "attn_norm.weight"] = (rd,)
        s[p + "Wqkv.weight"] = (3 * rd, rd)
        s[p + "out_proj.weight"] = (rd, rd)
        s[p + "mlp_norm.weight"] = (rd,)
        s[p + "w1.weight"] = (rf, rd)
        s[p + "w3.weight"] = (rf, rd)
        s[p + "w2.weight"] = (rd, rf)
    return s


def init_weights(cfg: OracleConfig, seed: int = 0, dtype=torch.bfloat16) -> dict[str, Tensor]:
    """Seeded random-init state dict: every matrix ~ N(0, 0.02), every RMSNorm
    gain 1, eos bias 0.  Values are drawn in fp32 from one CPU generator in the
    (sorted-by-insertion) order of ``weight_shapes`` and then cast to ``dtype``,
    so any two hosts with the same torch build get the same tensors."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    sd: dict[str, Tensor] = {}
    for name, shape in weight_shapes(cfg).items():
        if name.endswith("norm.weight"):
            t = torch.ones(shape, dtype=torch.float32)
        elif name == "eos_head.bias":
            t = torch.zeros(shape, dtype=torch.float32)
        else:
            t = torch.empty(shape, dtype=torch.float32).normal_(0.0, 0.02, generator=g)
        sd[name] = t.to(dtype)
    return sd


def rope_table(head_dim: int, max_seq: int, theta: float, dtype=torch.float32) -> Tensor:
    """(max_seq, head_dim, 2) table of [cos, sin], each frequency repeated for
    the two members of an interleaved pair (rope.py:60-77).  The reference
    builds it in fp32 and ``.bfloat16()`` on the module casts it, so for bf16
    parity pass ``dtype=torch.bfloat16``."""
    pos = torch.arange(max_seq, dtype=torch.float32)
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    ang = pos[:, None] * inv[None, :]
    ang = ang.repeat_interleave(2, dim=-1)
    return torch.stack((ang.cos(), ang.sin()), dim=-1).to(dtype)


# ---------------------------------------------------------------------------
# Ops
# ---------------------------------------------------------------------------


def rmsnorm(x: Tensor, w: Tensor, eps: float) -> Tensor:
    # model.py:292-297 - fp32 normalise, round to x.dtype, then scale by w
    xf = x.float()
    y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).type_as(x)
    return y * w


def apply_rope(freqs: Tensor, t: Tensor) -> Tensor:
    """freqs: (R, hd, 2) already gathered per row; t: (R, H, hd).
    rope.py:50 - ``t*cos*1.0 + rotate_half(t)*sin*1.0`` in t's dtype, each
    product and the sum being separate roundings."""
    cos = freqs[:, None, :, 0]
    sin = freqs[:, None, :, 1]
    x1 = t[..., ::2]
    x2 = t[..., 1::2]
    rot = torch.stack((-x2, x1), dim=-1).flatten(-2)
    return ((t * cos * 1.0) + (rot * sin * 1.0)).to(t.dtype)


def audio_embed(table: Tensor, codes: Tensor, codebook_size: int) -> Tensor:
    # model.py:559-563 - row = q*CS + code_q, sum over q
    Q = codes.shape[-1]
    off = torch.arange(Q, device=codes.device) * codebook_size
    return F.embedding(codes + off, table).sum(dim=-2)


def _attend(q: Tensor, k: Tensor, v: Tensor, scale: float) -> Tensor:
    """q: (H, hd); k, v: (T, H, hd) (kv heads already repeated).  fp32 softmax
    attention with one rounding of the output to q's dtype."""
    s = torch.einsum("hd,thd->ht", q.float(), k.float()) * scale
    p = torch.softmax(s, dim=-1)
    return torch.einsum("ht,thd->hd", p, v.float()).to(q.dtype)


# ---------------------------------------------------------------------------
# Backbone with a slot-indexed KV cache (model.py:71-99 layout)
# ---------------------------------------------------------------------------


class Oracle:
    def __init__(
        self,
        cfg: OracleConfig,
        sd: dict[str, Tensor],
        *,
        n_slots: int = 1,
        max_seq: int = 1024,
        dtype=torch.float32,
        device="cpu",
    ):
        self.cfg = cfg
        self.dtype = dtype
        self.device = torch.device(device)
        self.w = {k: v.to(self.device, dtype) for k, v in sd.items()}
        self.max_seq = max_seq
        self.n_slots = n_slots
        self.freqs = rope_table(cfg.head_dim, max_seq, cfg.rope_theta).to(self.device, dtype)
        L, Hk, hd = cfg.n_layers, cfg.n_kv_heads, cfg.head_dim
        self.k_cache = torch.zeros(L, n_slots, max_seq, Hk, hd, dtype=dtype, device=self.device)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.seq_lens = [0] * n_slots
        self.taps: dict[str, Tensor] | None = None  # filled when a dict is set

    # -- one transformer block over R rows, each row r = (slot, position) ----
    def _block(self, li: int, x: Tensor, slots: list[int], pos: list[int]) -> Tensor:
        cfg, w = self.cfg, self.w
        p = f"decoder.blocks.{li}."
        H, Hk, hd = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        R = x.shape[0]
        h = rmsnorm(x, w[p + "attn_norm.weight"], cfg.norm_eps)
        qkv = F.linear(h, w[p + "attn.Wqkv.weight"])
        q, k, v = torch.split(qkv, [H * hd, Hk * hd, Hk * hd], dim=-1)
        q = q.reshape(R, H, hd)
        k = k.reshape(R, Hk, hd)
        v = v.reshape(R, Hk, hd)
        fr = self.freqs[torch.tensor(pos, device=self.device)]
        q = apply_rope(fr, q)
        k = apply_rope(fr, k)
        # append first, then attend over [0, pos] (flash_attn_with_kvcache
        # semantics, model.py:247-257; causal, so a row sees itself)
        for r in range(R):
            self.k_cache[li, slots[r], pos[r]] = k[r]
            self.v_cache[li, slots[r], pos[r]] = v[r]
        out = torch.empty(R, H, hd, dtype=x.dtype, device=self.device)
        rep = H // Hk
        scale = 1.0 / math.sqrt(hd)
        for r in range(R):
            kk = self.k_cache[li, slots[r], : pos[r] + 1].repeat_interleave(rep, dim=1)
            vv = self.v_cache[li, slots[r], : pos[r] + 1].repeat_interleave(rep, dim=1)
            out[r] = _attend(q[r], kk, vv, scale)
        x = x + F.linear(out.reshape(R, H * hd), w[p + "attn.out_proj.weight"])
        h2 = rmsnorm(x, w[p + "mlp_norm.weight"], cfg.norm_eps)
        a = F.silu(F.linear(h2, w[p + "mlp.w1.weight"])) * F.linear(h2, w[p + "mlp.w3.weight"])
        x = x + F.linear(a, w[p + "mlp.w2.weight"])
        return x

    def _stack(self, x: Tensor, slots: list[int], pos: list[int]) -> Tensor:
        for li in range(self.cfg.n_layers):
            x = self._block(li, x, slots, pos)
            if self.taps is not None:
                self.taps[f"layer{li}"] = x.clone()
        return rmsnorm(x, self.w["decoder.norm.weight"], self.cfg.norm_eps)

    # -- engine.py:674-694: write T embeddings into one slot -----------------
    def prefill_emb(self, slot: int, emb: Tensor) -> Tensor:
        T = emb.shape[0]
        off = self.seq_lens[slot]
        assert off + T <= self.max_seq
        out = self._stack(emb.to(self.device, self.dtype), [slot] * T, list(range(off, off + T)))
        self.seq_lens[slot] = off + T
        return out  # (T, d) final-norm output

    def prefill_text(self, slot: int, ids: Tensor) -> Tensor:
        return self.prefill_emb(slot, F.embedding(ids.to(self.device), self.w["token_emb.weight"]))

    def prefill_codes(self, slot: int, codes: Tensor) -> Tensor:
        return self.prefill_emb(
            slot, audio_embed(self.w["audio_emb.embedding.weight"], codes.to(self.device), self.cfg.codebook_size)
        )

    # -- engine.py:434-449 / 485-502: one decode step for the given slots ----
    def backbone_step(self, slots: list[int], codes: Tensor):
        """codes: (B, Q) previous frame per slot.  Returns hidden (B,d),
        cb0 logits (B,CS), eos logit (B,1) and advances seq_lens."""
        emb = audio_embed(self.w["audio_emb.embedding.weight"], codes.to(self.device), self.cfg.codebook_size)
        emb = emb.to(self.dtype)
        if self.taps is not None:
            self.taps["emb"] = emb.clone()
        pos = [self.seq_lens[s] for s in slots]
        hidden = self._stack(emb, slots, pos)
        for s in slots:
            self.seq_lens[s] += 1
        cb0 = F.linear(hidden, self.w["codec_head.weight"])
        eos = F.linear(hidden, self.w["eos_head.weight"], self.w["eos_head.bias"])
        return hidden, cb0, eos

    # -- RQ depth transformer, KV form (model.py:908-986) --------------------
    def _rq_block(self, li: int, x: Tensor, kc: Tensor, vc: Tensor, pos: list[int]) -> Tensor:
        """x: (B, P, rd) tokens at depth positions ``pos`` (len P); kc/vc:
        (B, Q, H, hd) caches for this layer."""
        cfg, w = self.cfg, self.w
        p = f"rq_transformer.blocks.{li}."
        H, hd = cfg.rq_n_heads, cfg.rq_head_dim
        B, P, D = x.shape
        h = rmsnorm(x, w[p + "attn_norm.weight"], cfg.rq_norm_eps)
        qkv = F.linear(h, w[p + "Wqkv.weight"]).reshape(B, P, 3, H, hd)
        q, k, v = qkv.unbind(2)
        for j, ps in enumerate(pos):
            kc[:, ps] = k[:, j]
            vc[:, ps] = v[:, j]
        out = torch.empty(B, P, H, hd, dtype=x.dtype, device=x.device)
        scale = hd ** -0.5
        for b in range(B):
            for j, ps in enumerate(pos):
                out[b, j] = _attend(q[b, j], kc[b, : ps + 1], vc[b, : ps + 1], scale)
        x = x + F.linear(out.reshape(B, P, D), w[p + "out_proj.weight"])
        h2 = rmsnorm(x, w[p + "mlp_norm.weight"], cfg.rq_norm_eps)
        x = x + F.linear(F.silu(F.linear(h2, w[p + "w1.weight"])) * F.linear(h2, w[p + "w3.weight"]), w[p + "w2.weight"])
        return x

    def rq_generate(
        self,
        hidden: Tensor,
        code0: Tensor,
        *,
        temperature: float = 1.0,
        top_k: int = 1,
        generator: torch.Generator | None = None,
        n_quantizers: int = 0,
        return_logits: bool = False,
        forced: Tensor | None = None,
    ):
        """hidden: (B, d) final-norm backbone output; code0: (B,) long.
        ``top_k=1`` is greedy (first index on ties, like ``torch.argmax``).
        ``forced`` (B, Q') teacher-forces those codes as the inputs of later
        positions (the returned codes are still this model's own choices).
        Returns codes (B, Q') long [, logits (B, Q'-1, CS) in model dtype]."""
        cfg, w = self.cfg, self.w
        r = "rq_transformer."
        Q = n_quantizers if n_quantizers > 0 else cfg.n_quantizers
        CS = cfg.codebook_size
        B = hidden.shape[0]
        H, hd, nl = cfg.rq_n_heads, cfg.rq_head_dim, cfg.rq_n_layers
        kc = torch.zeros(nl, B, cfg.n_quantizers, H, hd, dtype=self.dtype, device=self.device)
        vc = torch.zeros_like(kc)
        pe = w[r + "pos_emb.weight"]
        ce = w[r + "code_emb.embedding.weight"]
        tok0 = F.linear(hidden, w[r + "backbone_proj.weight"]) + pe[0]
        tok1 = F.embedding(code0, ce) + pe[1]
        seq = torch.stack([tok0, tok1], dim=1)
        for li in range(nl):
            seq = self._rq_block(li, seq, kc[li], vc[li], [0, 1])
        codes = [code0]
        all_logits = []
        x = seq[:, 1:2]
        for i in range(Q - 1):
            if i > 0:
                prev = codes[-1] if forced is None else forced[:, i].to(self.device)
                x = (F.embedding(prev + i * CS, ce) + pe[i + 1]).unsqueeze(1)
                for li in range(nl):
                    x = self._rq_block(li, x, kc[li], vc[li], [i + 1])
            h_out = rmsnorm(x[:, 0], w[r + "norm.weight"], cfg.rq_norm_eps)
            logits = F.linear(h_out, w[r + "head_W"][i])
            all_logits.append(logits)
            codes.append(self._choose(logits, temperature, top_k, generator))
        out = torch.stack(codes, dim=1)
        if return_logits:
            return out, torch.stack(all_logits, dim=1)
        return out

    @staticmethod
    def _choose(logits: Tensor, temperature: float, top_k: int, generator) -> Tensor:
        # model.py:955-962: (+bias) / temp, keep entries >= k-th value, softmax, multinomial
        if top_k == 1:
            return torch.argmax(logits, dim=-1)
        lg = logits.float() / temperature
        if top_k and top_k > 0:
            v, _ = lg.topk(top_k)
            lg = lg.masked_fill(lg < v[:, -1:], float("-inf"))
        probs = F.softmax(lg, dim=-1)
        return torch.multinomial(probs, 1, generator=generator).squeeze(-1)

    @staticmethod
    def sample_cb0(logits: Tensor, temperature: float, top_k: int | None, generator=None) -> Tensor:
        # engine.py:855-863: softmax first, top-k over probabilities, renormalise
        if top_k == 1:
            return torch.argmax(logits, dim=-1)
        probs = F.softmax(logits.float() / temperature, dim=-1)
        if top_k is not None and top_k > 0:
            topv, topi = probs.topk(top_k, dim=-1)
            mask = torch.zeros_like(probs).scatter_(1, topi, topv)
            probs = mask / mask.sum(dim=-1, keepdim=True).clamp_min(1e-9)
        return torch.multinomial(probs, 1, generator=generator).squeeze(-1)

    @staticmethod
    def rep_apply(logits: Tensor, counts: Tensor, penalty: float) -> Tensor:
        # engine.py:571-576
        if penalty <= 1.0:
            return logits
        factor = torch.pow(torch.tensor(penalty, dtype=torch.float32, device=logits.device), counts)
        return torch.where(logits > 0, logits / factor, logits * factor)

    # -- frame protocol (engine.py:914-951 then 1023-1079), greedy -----------
    def generate_greedy(self, slot: int, ids: Tensor, n_frames: int, record=None) -> Tensor:
        """Prefill ``ids`` as text into ``slot`` then emit ``n_frames`` frames:
        frame 0 from the prefill's last hidden, frame k>=1 from a decode step on
        frame k-1.  EOS ignored, no rep penalty.  Returns (n_frames, Q) long."""
        h = self.prefill_text(slot, ids)[-1:]
        frames = []
        for f in range(n_frames):
            if f > 0:
                h, cb0, eos = self.backbone_step([slot], frames[-1][None])
            else:
                cb0 = F.linear(h, self.w["codec_head.weight"])
                eos = F.linear(h, self.w["eos_head.weight"], self.w["eos_head.bias"])
            code0 = torch.argmax(cb0, dim=-1)
            codes, rql = self.rq_generate(h, code0, top_k=1, return_logits=True)
            frames.append(codes[0])
            if record is not None:
                record(f, h, cb0, eos, rql, codes)
        return torch.stack(frames, dim=0)


@dataclass
class FrameTrace:
    """Per-frame tensors kept by ``Oracle.generate_greedy(record=...)``."""

    hidden: list = field(default_factory=list)
    cb0: list = field(default_factory=list)
    eos: list = field(default_factory=list)
    rq_logits: list = field(default_factory=list)

    def __call__(self, f, h, cb0, eos, rql, codes):
        self.hidden.append(h[0].float().cpu())
        self.cb0.append(cb0[0].float().cpu())
        self.eos.append(eos[0].float().cpu())
        self.rq_logits.append(rql[0].float().cpu())
