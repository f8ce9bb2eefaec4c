"""Stand-in for the reference's CUDA path on the benchmark box: the oracle's algorithm, batched over
streams, in torch bf16 on cuBLAS, captured in CUDA graphs the way the reference captures its backbone
step and its depth loop (src/vui/engine.py:375-432, 525-534; src/vui/model.py:814-881, 988-1016).

TEST / BENCHMARK INFRASTRUCTURE ONLY (see oracle/vui_oracle.py).  The reference itself cannot run on
the GPU box (its package and flash-attn build are not there), so the "how many times faster than the
reference's CUDA path" figure is taken against this: same operators, same launch structure (one graph
for the backbone step, one for the 15-codebook loop, sampling on the device), torch SDPA with a
length mask in place of flash_attn_with_kvcache (which reads only the valid keys: this stand-in reads
max_seq keys per stream, ~0.3 ms per step at 64 streams x 640 positions, and is that much slower than
the real thing would be).
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from .vui_oracle import OracleConfig, apply_rope, audio_embed, rmsnorm, rope_table


class TorchGraphDecoder:
    def __init__(self, cfg: OracleConfig, sd: dict, n_streams: int, max_seq: int, device="cuda",
                 temperature: float = 0.8, top_k: int = 50):
        self.cfg, self.B, self.S = cfg, n_streams, max_seq
        self.dev = torch.device(device)
        self.w = {k: v.to(self.dev, torch.bfloat16) for k, v in sd.items()}
        self.freqs = rope_table(cfg.head_dim, max_seq, cfg.rope_theta).to(self.dev, torch.bfloat16)
        L, Hk, hd = cfg.n_layers, cfg.n_kv_heads, cfg.head_dim
        self.k_cache = torch.zeros(L, n_streams, max_seq, Hk, hd, device=self.dev, dtype=torch.bfloat16)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.seq_lens = torch.zeros(n_streams, device=self.dev, dtype=torch.long)
        self.codes = torch.zeros(n_streams, cfg.n_quantizers, device=self.dev, dtype=torch.long)
        self.hidden = torch.zeros(n_streams, cfg.d_model, device=self.dev, dtype=torch.bfloat16)
        self.cb0 = torch.zeros(n_streams, cfg.codebook_size, device=self.dev, dtype=torch.bfloat16)
        self.T, self.top_k = temperature, top_k
        self.rows = torch.arange(n_streams, device=self.dev)
        self.key_idx = torch.arange(max_seq, device=self.dev)
        self.g_backbone = self.g_depth = None

    # -- one backbone step for all streams at their own positions (engine.py:434-449)
    def _backbone(self):
        cfg, w = self.cfg, self.w
        H, Hk, hd, B = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, self.B
        x = audio_embed(w["audio_emb.embedding.weight"], self.codes, cfg.codebook_size)
        pos = self.seq_lens
        fr = self.freqs[pos]
        mask = (self.key_idx[None, :] <= pos[:, None])[:, None, None, :]
        for li in range(cfg.n_layers):
            p = f"decoder.blocks.{li}."
            h = rmsnorm(x, w[p + "attn_norm.weight"], cfg.norm_eps)
            q, k, v = torch.split(F.linear(h, w[p + "attn.Wqkv.weight"]), [H * hd, Hk * hd, Hk * hd], dim=-1)
            q = apply_rope(fr, q.reshape(B, H, hd))
            k = apply_rope(fr, k.reshape(B, Hk, hd))
            self.k_cache[li].index_put_((self.rows, pos), k)
            self.v_cache[li].index_put_((self.rows, pos), v.reshape(B, Hk, hd))
            o = F.scaled_dot_product_attention(q[:, :, None, :], self.k_cache[li].permute(0, 2, 1, 3),
                                               self.v_cache[li].permute(0, 2, 1, 3), attn_mask=mask,
                                               scale=1.0 / math.sqrt(hd), enable_gqa=True)
            x = x + F.linear(o.reshape(B, H * hd), w[p + "attn.out_proj.weight"])
            h2 = rmsnorm(x, w[p + "mlp_norm.weight"], cfg.norm_eps)
            x = x + F.linear(F.silu(F.linear(h2, w[p + "mlp.w1.weight"])) * F.linear(h2, w[p + "mlp.w3.weight"]),
                             w[p + "mlp.w2.weight"])
        hid = rmsnorm(x, w["decoder.norm.weight"], cfg.norm_eps)
        self.hidden.copy_(hid)
        self.cb0.copy_(F.linear(hid, w["codec_head.weight"]))
        self.seq_lens.add_(1)

    def _pick(self, logits):
        # model.py:955-962: logits / T, keep entries >= the k-th value, softmax, multinomial
        lg = logits.float() / self.T
        kth = lg.topk(self.top_k).values[:, -1:]
        probs = F.softmax(lg.masked_fill(lg < kth, float("-inf")), dim=-1)
        return torch.multinomial(probs, 1).squeeze(-1)

    # -- cb0 draw + the 15-codebook loop with its own small KV (model.py:908-986)
    def _depth(self):
        cfg, w, B = self.cfg, self.w, self.B
        r = "rq_transformer."
        H, hd, nl, Q, CS = cfg.rq_n_heads, cfg.rq_head_dim, cfg.rq_n_layers, cfg.n_quantizers, cfg.codebook_size
        kc = torch.zeros(nl, B, Q, H, hd, device=self.dev, dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        pe, ce = w[r + "pos_emb.weight"], w[r + "code_emb.embedding.weight"]
        code0 = self._pick(self.cb0)
        self.codes[:, 0] = code0

        def block(li, x, positions):
            p = f"{r}blocks.{li}."
            P = x.shape[1]
            h = rmsnorm(x, w[p + "attn_norm.weight"], cfg.rq_norm_eps)
            q, k, v = F.linear(h, w[p + "Wqkv.weight"]).reshape(B, P, 3, H, hd).unbind(2)
            lo, hi = positions[0], positions[-1] + 1
            kc[li][:, lo:hi] = k
            vc[li][:, lo:hi] = v
            o = F.scaled_dot_product_attention(q.transpose(1, 2), kc[li][:, :hi].transpose(1, 2), vc[li][:, :hi].transpose(1, 2),
                                               is_causal=(P > 1), scale=hd ** -0.5)
            x = x + F.linear(o.transpose(1, 2).reshape(B, P, H * hd), w[p + "out_proj.weight"])
            h2 = rmsnorm(x, w[p + "mlp_norm.weight"], cfg.rq_norm_eps)
            return x + F.linear(F.silu(F.linear(h2, w[p + "w1.weight"])) * F.linear(h2, w[p + "w3.weight"]), w[p + "w2.weight"])

        seq = torch.stack([F.linear(self.hidden, w[r + "backbone_proj.weight"]) + pe[0], F.embedding(code0, ce) + pe[1]], dim=1)
        for li in range(nl):
            seq = block(li, seq, [0, 1])
        x = seq[:, 1:2]
        prev = code0
        for i in range(Q - 1):
            if i > 0:
                x = (F.embedding(prev + i * CS, ce) + pe[i + 1]).unsqueeze(1)
                for li in range(nl):
                    x = block(li, x, [i + 1])
            logits = F.linear(rmsnorm(x[:, 0], w[r + "norm.weight"], cfg.rq_norm_eps), w[r + "head_W"][i])
            prev = self._pick(logits)
            self.codes[:, i + 1] = prev

    def capture(self):
        """Warm up on a side stream, then capture the two graphs (position and codes are rewound after)."""
        seq0, codes0 = self.seq_lens.clone(), self.codes.clone()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s), torch.inference_mode():
            for _ in range(2):
                self._backbone()
                self._depth()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        self.g_backbone, self.g_depth = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with torch.inference_mode():
            with torch.cuda.graph(self.g_backbone):
                self._backbone()
            with torch.cuda.graph(self.g_depth):
                self._depth()
        torch.cuda.synchronize()
        self.seq_lens.copy_(seq0)
        self.codes.copy_(codes0)

    def step(self):
        self.g_backbone.replay()
        self.g_depth.replay()
