"""Generate the golden fixtures in this folder from the REFERENCE's own code.

Run once, in a container that has a checkout of fluxions-ai/vui:

    python tests/golden/make_golden.py --reference /path/to/vui

It imports the reference's classes (``vui.model``, ``vui.rope``, ``vui.engine``
helpers) on CPU with a stub tokenizer (the real one downloads BPE files), loads
the seeded random-init weights of ``oracle.vui_oracle.init_weights`` into them,
and stores what the reference computes:

* ``ops_bf16.pt``   - per-op input/output pairs in bf16 (RMSNorm, RoPE,
  AudioEmbedding gather-sum, LlamaMLP, Wqkv, one RQ block, cb0 top-k
  probabilities) produced by the reference modules.
* ``cfg1_fp32.pt``  - benchmark configuration 1: 64 seeded text ids -> 50 greedy frames,
  CPU fp32, through ``Decoder.forward`` + ``KVCache`` + causal mask and
  ``RQTransformer.generate(top_k=1)``; codes, and hidden / cb0 logits / RQ
  logits of a few frames.
* ``cfg_bf16_cpu.pt`` - the same protocol in bf16 on CPU for 8 frames
  (teacher-forced on its own codes): hidden / cb0 / RQ logits per frame, used
  as a tolerance check (CPU SDPA's bf16 arithmetic differs from flash-attn's).
* ``tiny_fp32.pt``  - the small shape ``oracle.vui_oracle.TINY`` end to end.
* ``text_cases.json`` - ``simple_clean`` / ``chunk_text`` (src/vui/inference.py) on sample strings.

The fixtures travel with the repo; the reference does not.
"""

from __future__ import annotations

import argparse
import os
import sys
import time

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle.vui_oracle import TINY, OracleConfig, init_weights  # noqa: E402


class _StubTok:
    """Stands in for vui.tokenizer.VuiTokenizer (which needs the network)."""

    def __init__(self, vocab):
        self.vocab_size = vocab
        self.special_to_id = {"[SC]": vocab - 4}

    def __call__(self, *_a, **_k):
        return self


def build_reference(ref_root: str, cfg: OracleConfig, sd, dtype):
    sys.path.insert(0, os.path.join(ref_root, "src"))
    import vui.model as vm
    from vui.config import Config, DataConfig, VuiConfig

    vm.VuiTokenizer = lambda *_a, **_k: _StubTok(cfg.vocab)
    mc = VuiConfig(
        d_model=cfg.d_model, n_layers=cfg.n_layers, n_heads=cfg.n_heads, n_kv_heads=cfg.n_kv_heads,
        intermediate_size=cfg.ffn, rope_theta=cfg.rope_theta, use_rq_transformer=True,
        rq_d_model=cfg.rq_d_model, rq_n_layers=cfg.rq_n_layers, rq_n_heads=cfg.rq_n_heads,
        n_quantizers=cfg.n_quantizers, codebook_size=cfg.codebook_size,
    )
    model = vm.Vui(Config(model=mc, data=DataConfig(max_secs=30)))
    missing = model.load_state_dict({k: v.float() for k, v in sd.items()}, strict=False)
    # noisy_emb (unused on this path) is the only parameter we do not set
    assert set(missing.missing_keys) <= {"noisy_emb"}, missing
    assert not missing.unexpected_keys, missing
    model = model.to(dtype).eval()
    return vm, model


@torch.inference_mode()
def reference_greedy(vm, model, cfg, ids, n_frames, dtype, S=256):
    """Reference CPU path: Decoder.forward with KVCache + mask (model.py:42-68,
    146-202, 511-532), frame protocol of engine.py:914-951 / 1023-1079."""
    dec = model.decoder
    for blk in dec.blocks:
        blk.attn.kv_cache = vm.KVCache(1, S, cfg.n_kv_heads, cfg.head_dim, dtype)
    dec.attn_mask = torch.tril(torch.ones(S, S))
    T = ids.numel()
    h = dec(model.token_emb(ids[None]).to(dtype), torch.arange(T))[:, -1]
    pos = T
    out = {"codes": [], "hidden": [], "cb0": [], "eos": [], "rq_logits": []}
    rq = model.rq_transformer
    for f in range(n_frames):
        if f > 0:
            emb = model.audio_emb(out["codes"][-1][None]).unsqueeze(1).to(dtype)
            h = dec(emb, torch.tensor([pos]))[:, 0]
            pos += 1
        cb0 = model.codec_head(h)
        eos = model.eos_head(h)
        code0 = torch.argmax(cb0, dim=-1)
        codes = rq.generate(h, code0, temperature=1.0, top_k=1)
        # teacher-forced logits of the RQ head for the codes it chose (forward(), model.py:665-684)
        rql = rq(h, codes)
        out["codes"].append(codes[0].clone())
        out["hidden"].append(h[0].float().clone())
        out["cb0"].append(cb0[0].float().clone())
        out["eos"].append(eos[0].float().clone())
        out["rq_logits"].append(rql[0].float().clone())
    dec.deallocate_kv_cache()
    return {k: torch.stack(v) for k, v in out.items()}


@torch.inference_mode()
def ops_fixture(vm, model, cfg):
    """Per-op pairs from the reference's modules in bf16 (CPU)."""
    from vui.rope import apply_rotary_emb

    g = torch.Generator().manual_seed(1234)
    d = cfg.d_model
    fx = {}
    blk = model.decoder.blocks[0]
    x = (torch.randn(5, d, generator=g) * 0.7).bfloat16()
    blk.attn_norm.weight.copy_((1.0 + 0.1 * torch.randn(d, generator=g)).bfloat16())
    fx["norm_w"] = blk.attn_norm.weight.clone()
    fx["norm_x"] = x
    fx["norm_y"] = blk.attn_norm(x)
    fx["rq_norm_y"] = model.rq_transformer.norm(x[:, : cfg.rq_d_model])
    # RoPE, per-sample positions (model.py:235-237)
    pos = torch.tensor([0, 1, 17, 511, 1023])
    fr = model.decoder.freqs_cis[pos]
    q = torch.randn(5, cfg.n_heads, cfg.head_dim, generator=g).bfloat16()
    fx["rope_pos"], fx["rope_q"] = pos, q
    fx["rope_table_rows"] = fr.clone()
    fx["rope_out"] = apply_rotary_emb(fr, q)
    # gather-sum
    codes = torch.randint(0, cfg.codebook_size, (4, cfg.n_quantizers), generator=g)
    fx["emb_codes"] = codes
    fx["emb_out"] = model.audio_emb(codes)
    # MLP and Wqkv of layer 0
    h = (torch.randn(3, d, generator=g)).bfloat16()
    fx["mlp_x"] = h
    fx["mlp_y"] = blk.mlp(h)
    fx["qkv_y"] = blk.attn.Wqkv(h)
    # cb0 sampling distribution (engine.py:857-862) for logits row
    lg = (torch.randn(2, cfg.codebook_size, generator=g) * 0.45).bfloat16()
    probs = torch.softmax(lg.float() / 0.8, dim=-1)
    topv, topi = probs.topk(50, dim=-1)
    mask = torch.zeros_like(probs).scatter_(1, topi, topv)
    fx["cb0_logits"] = lg
    fx["cb0_probs_t0.8_k50"] = mask / mask.sum(-1, keepdim=True).clamp_min(1e-9)
    # RQ: greedy generate + teacher-forced logits from a random hidden
    hid = (torch.randn(2, d, generator=g)).bfloat16()
    c0 = torch.tensor([5, 2000])
    rq = model.rq_transformer
    fx["rq_hidden"], fx["rq_code0"] = hid, c0
    fx["rq_codes"] = rq.generate(hid, c0, temperature=1.0, top_k=1)
    fx["rq_logits"] = rq(hid, fx["rq_codes"])
    return fx


def text_fixture(ref_root: str):
    """Outputs of the reference's text cleaning / chunking on a few strings."""
    import json

    sys.path.insert(0, os.path.join(ref_root, "src"))
    from vui.inference import chunk_text, simple_clean

    clean_in = ["Hello there", "It's 5pm \u2014 let's go (now)!",
                "Costs 50% more: really; \"quoted\" 'single' well-known -dash",
                "wait[laugh]what [unknown] ok", "a vs b vs. c\u2026", "line one\n\n\nline two  ",
                "He said 'don't' at 9am?", "tags [breath][sigh] end"]
    chunk_in = [
        ("Hello there, my friend. How are you doing today? I am fine, thanks for asking, really.", {}),
        ("Short. Tiny. Ok.", {}),
        ("First speaker line here okay.\nSecond speaker answers now indeed.", {}),
        ("First speaker line here okay.\nSecond speaker answers now indeed.", {"single_speaker": True}),
        ("One two three four five six seven eight nine ten eleven twelve thirteen. And more words here to go.",
         {"sentence_only": True, "min_words": 6}),
        ("A start [SC] other speaker talks here now. [laugh] And then continues, with a clause, and more.",
         {"min_words": 3}),
        ("", {}),
    ]
    out = {"clean": [{"in": s, "out": simple_clean(s)} for s in clean_in],
           "chunk": [{"in": s, "kw": kw, "out": chunk_text(s, **kw)} for s, kw in chunk_in]}
    with open(os.path.join(HERE, "text_cases.json"), "w") as f:
        json.dump(out, f, indent=1, ensure_ascii=False)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of the reference project")
    ap.add_argument("--skip-full", action="store_true")
    args = ap.parse_args()
    torch.manual_seed(0)
    torch.set_num_threads(os.cpu_count() or 1)

    # the stub tokenizer must be in place before vui.inference pulls in vui.model
    sys.path.insert(0, os.path.join(args.reference, "src"))
    import vui.model as _vm

    _vm.VuiTokenizer = lambda *_a, **_k: _StubTok(1000)
    text_fixture(args.reference)

    # tiny shape, fp32
    sd = init_weights(TINY, seed=0, dtype=torch.float32)
    vm, model = build_reference(args.reference, TINY, sd, torch.float32)
    ids = torch.randint(0, TINY.vocab, (12,), generator=torch.Generator().manual_seed(0))
    ref = reference_greedy(vm, model, TINY, ids, 6, torch.float32, S=64)
    ref["ids"] = ids
    torch.save(ref, os.path.join(HERE, "tiny_fp32.pt"))
    print("tiny_fp32 codes[0]:", ref["codes"][0].tolist())
    if args.skip_full:
        return

    cfg = OracleConfig()
    sd = init_weights(cfg, seed=0, dtype=torch.bfloat16)  # bf16-representable weights for both precisions
    # config 1: fp32
    t0 = time.time()
    vm, model = build_reference(args.reference, cfg, sd, torch.float32)
    ids = torch.randint(0, cfg.vocab, (64,), generator=torch.Generator().manual_seed(0))
    ref = reference_greedy(vm, model, cfg, ids, 50, torch.float32, S=128)
    keep = [0, 1, 2, 31, 49]
    fx = {"ids": ids, "codes": ref["codes"], "frames_kept": torch.tensor(keep)}
    for k in ("hidden", "cb0", "eos", "rq_logits"):
        fx[k] = ref[k][keep].clone()
    torch.save(fx, os.path.join(HERE, "cfg1_fp32.pt"))
    print(f"cfg1_fp32 done in {time.time()-t0:.1f}s; frame0 {ref['codes'][0].tolist()}")

    # bf16 on CPU
    model = model.bfloat16()
    fxo = ops_fixture(vm, model, cfg)
    torch.save(fxo, os.path.join(HERE, "ops_bf16.pt"))
    with torch.no_grad():
        model.decoder.blocks[0].attn_norm.weight.fill_(1.0)
    ref = reference_greedy(vm, model, cfg, ids, 8, torch.bfloat16, S=128)
    ref["ids"] = ids
    torch.save({k: (v if k in ("codes", "ids") else v.bfloat16()) for k, v in ref.items()},
               os.path.join(HERE, "cfg_bf16_cpu.pt"))
    print("cfg_bf16_cpu frame0", ref["codes"][0].tolist())


if __name__ == "__main__":
    main()
