"""Generate ``codec_fp32.pt`` from the REFERENCE's own codec classes.

Run once, in a container that has a checkout of fluxions-ai/vui:

    python tests/golden/make_codec_golden.py --reference /path/to/vui

Imports ``vui.qwen_codec`` on CPU, loads the seeded random weights of ``vui_b200.codec.random_codec_state(0)``
into the reference's ``QwenCodecDecoder`` (no released codec weights are available offline) and stores what
the reference computes in fp32:

* ``stream``   - six frames decoded one at a time inside ``decoder.streaming(1)``;
* ``offline``  - the same six frames through the non-streaming forward;
* ``stream_q8`` - three frames with only the first 8 codebooks;
* ``taps``     - intermediate activations of streamed frame 2 (first 64 columns of each);
* ``ctx``      - ``CodecCtx`` with a 5-frame window (max_ctx_secs = 0.4): a 7-frame prompt, ``prefill()``, then
  nine ``decode_frame`` calls, which crosses the window boundary twice.

The fixture travels with the repo; the reference does not.
"""

from __future__ import annotations

import argparse
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from vui_b200.codec import codec_param_shapes, random_codec_state  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "src"))
    import vui.qwen_codec as qc

    torch.manual_seed(0)
    dec = qc.QwenCodecDecoder().eval()
    ref_shapes = {k: tuple(v.shape) for k, v in dec.state_dict().items()}
    assert list(ref_shapes.items()) == list(codec_param_shapes().items()), "state-dict names or shapes differ"
    dec.load_state_dict(random_codec_state(0))

    g = torch.Generator().manual_seed(123)
    codes = torch.randint(0, 2048, (1, 16, 6), generator=g)
    out: dict = {"codes": codes}
    taps: dict = {}

    def tap(name):
        def hook(_m, _i, o):
            if hook.on:
                taps[name] = o.detach().clone()
        hook.on = False
        return hook

    hooks = {"transformer": tap("transformer"), "upsampled": tap("upsampled"), "decoder0": tap("decoder0")}
    dec.pre_transformer.register_forward_hook(hooks["transformer"])
    dec.upsample[1][1].register_forward_hook(hooks["upsampled"])
    dec.decoder[0].register_forward_hook(hooks["decoder0"])
    for b in range(4):
        hooks[f"block{b + 1}"] = tap(f"block{b + 1}")
        dec.decoder[b + 1].register_forward_hook(hooks[f"block{b + 1}"])

    with torch.inference_mode():
        with dec.streaming(1):
            frames = []
            for t in range(6):
                for h in hooks.values():
                    h.on = t == 2
                frames.append(dec(codes[:, :, t:t + 1]).clone())
            for h in hooks.values():
                h.on = False
        out["stream"] = torch.cat(frames, dim=-1)
        out["offline"] = dec(codes).clone()
        with dec.streaming(1):
            out["stream_q8"] = torch.cat([dec(codes[:, :8, t:t + 1]).clone() for t in range(3)], dim=-1)
        taps["quantizer"] = dec.quantizer.decode(codes[:, :, 2:3])   # stateless; decode() is not a module forward
        t_ = taps["transformer"]
        taps["transformer"] = t_.transpose(1, 2)        # (1, T, 1024) -> channel-major like the others
        out["taps"] = {k: v[0, :, :64].contiguous() for k, v in taps.items()}

        prompt = torch.randint(0, 2048, (1, 16, 7), generator=g)
        new = torch.randint(0, 2048, (1, 16, 9), generator=g)
        ctx = qc.CodecCtx(dec, max_ctx_secs=0.4)
        assert ctx.max_ctx == 5
        ctx.set_prompt(prompt)
        ctx.prefill(device="cpu")
        trace, since = [], []
        for t in range(9):
            trace.append(ctx.decode_frame(new[:, :, t:t + 1]).clone())
            since.append(ctx._frames_since_prefill)
        ctx.reset()
        out["ctx"] = {"prompt": prompt, "codes": new, "audio": torch.cat(trace, dim=-1), "since": since}

    path = os.path.join(HERE, "codec_fp32.pt")
    torch.save(out, path)
    d = (out["stream"] - out["offline"]).abs().max().item()
    print(f"wrote {path} ({os.path.getsize(path) / 1e3:.0f} kB); streaming vs offline max diff {d:.2e}; "
          f"clamped fraction {(out['stream'].abs() >= 1).float().mean().item():.3f}; since = {since}")


if __name__ == "__main__":
    main()
