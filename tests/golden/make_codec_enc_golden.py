"""Generate ``codec_enc_fp32.pt`` from the REFERENCE's own encoder classes.

    python tests/golden/make_codec_enc_golden.py --reference /path/to/vui

Imports ``vui.qwen_codec`` on CPU, loads ``vui_b200.codec_encoder.random_encoder_state(0)`` into the reference's
``QwenCodecEncoder`` and stores what it computes in fp32 for the seeded signal ``oracle.codec_enc_oracle.test_audio``:

* ``codes``    - the 16 x 125 codes of a full 10 s buffer, ``latent`` the (512, 125) latents before quantisation
  and ``margin`` the gap between the nearest and the second nearest code of every (codebook, frame);
* ``short``    - codes of the first 3 s alone (causality: equal to the first frames of ``codes``);
* ``stream``   - ``StreamingCodecEncoder``: chunk sizes fed, what each ``feed`` returned, the ``flush`` tail, across
  the 10 s boundary.
"""

from __future__ import annotations

import argparse
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle.codec_enc_oracle import test_audio  # noqa: E402
from vui_b200.codec_encoder import encoder_param_shapes, random_encoder_state  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "src"))
    import vui.qwen_codec as qc

    enc = qc.QwenCodecEncoder().eval()
    ref_shapes = {k: tuple(v.shape) for k, v in enc.state_dict().items()}
    assert list(ref_shapes.items()) == list(encoder_param_shapes().items()), "state-dict names or shapes differ"
    enc.load_state_dict(random_encoder_state(0))
    audio = test_audio(240000, seed=0)
    out: dict = {}
    with torch.inference_mode():
        lat = {}
        hook = enc.downsample.register_forward_hook(lambda _m, _i, o: lat.__setitem__("h", o.detach().clone()))
        out["codes"] = enc(audio)[0].to(torch.int16)
        hook.remove()
        out["latent"] = lat["h"][0]
        # margins: how far the winner is from the runner-up, per codebook and frame
        margins = []
        for part, n in (("semantic", 1), ("acoustic", 15)):
            q = getattr(enc.quantizer, part)
            res = q.input_proj(lat["h"]).float()[0].T
            for cb in q.codebooks[:n]:
                d = torch.cdist(res.unsqueeze(0), cb.embed.unsqueeze(0)).squeeze(0)
                two = d.topk(2, dim=-1, largest=False).values
                margins.append(two[:, 1] - two[:, 0])
                res = res - cb.embed[d.argmin(dim=-1)]
        out["margin"] = torch.stack(margins, dim=0)
        out["short"] = enc(audio[..., : 3 * 24000 // 1920 * 1920])[0].to(torch.int16)
        se = qc.StreamingCodecEncoder(enc)
        g = torch.Generator().manual_seed(1)
        sizes, got, pos = [], [], 0
        long_audio = test_audio(240000 + 60000, seed=2)[0, 0]
        while pos < long_audio.numel():
            n = int(torch.randint(4000, 40000, (1,), generator=g))
            n = min(n, long_audio.numel() - pos)
            r = se.feed(long_audio[pos:pos + n])
            sizes.append(n)
            got.append(None if r is None else r.to(torch.int16))
            pos += n
        tail = se.flush()
        out["stream"] = {"sizes": sizes, "feeds": got, "flush": None if tail is None else tail.to(torch.int16)}
    path = os.path.join(HERE, "codec_enc_fp32.pt")
    torch.save(out, path)
    print(f"wrote {path} ({os.path.getsize(path) / 1e3:.0f} kB); codes {tuple(out['codes'].shape)}, "
          f"distinct {out['codes'].unique().numel()}, latent std {out['latent'].std():.3f}, "
          f"smallest margin {out['margin'].min():.2e}, median {out['margin'].median():.3f}; "
          f"{sum(x is not None for x in got)} of {len(got)} feeds returned codes")


if __name__ == "__main__":
    main()
