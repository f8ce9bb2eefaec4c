"""Benchmark of the Vui-Nano decode step: codec frames/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--streams B] [--impl b200|reference]

A step is one decode frame for every stream of the batch (backbone step, cb0
sampling, 15 depth-transformer codebooks, gather-sum into the next frame's
input), i.e. one replay of the captured frame graph.  The headline workload is
benchmark configuration 2: one stream, 256 seeded text ids, greedy decode, KV up to
1024 positions; weights are seeded random-init (no checkpoint is available offline).
The K-step timed block is repeated (the stream is rewound in between, so every block
covers the same KV lengths) and the median block is reported.

Beside the headline the same line carries
  streams64   configuration 3: 64 streams, prompts U[64,512], T=0.8 top-k 50;
  cfg4        configuration 4: 16 streams x (128 text ids + 125 codec frames): prefill
              tokens/s, time to first frame, 375 greedy frames;
  streams256  configuration 5's per-GPU shape: 256 streams, 512-id prompts, 2048-position KV;
  codec       the step after the path: streaming codec decode of one stream's frames (16 codes ->
              1920 samples, fp32), ms per frame, x realtime, HBM roofline on its 423 MB of weights; and the
              codec encoder's whole-buffer encode (10 s of audio -> codes) used for user turns.

Under torchrun (N > 1) every rank is an independent replica with its own streams
on its own GPU; there is no data-path collective, the process group only aligns
the timed window and takes the max time over ranks.

`--impl reference` times the CPU restatement of the reference's PyTorch path
(oracle/, fp32, all host threads) on the same metric.  `--profile-frames N` runs N
frames kernel by kernel (no graph) and exits: the command the ncu summaries under
profiles/ are taken with; `--profile-codec N` does the same for N streamed codec frames, `--profile-encoder N`
for N codec-encoder calls.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FRAME_RATE = 12.5
FALLBACK_HBM_GBS = 6650.0
KV_BYTES_PER_POS = 24 * 2 * 8 * 64 * 2  # layers x (K,V) x kv heads x head_dim x bf16 = 49152
GATHER_BYTES_PER_STREAM = 16 * 2048 + 15 * 1024  # audio_emb rows + code_emb rows read per frame


def _dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


class ClockSampler:
    """nvidia-smi clocks / throttle reasons during the timed region."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = sorted(float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit())
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 9 for n, v in zip(names, r[5:9]) if v.lower() == "active"})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def measured_hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


def cpu_oracle_frame_times(prompt_len: int, n_frames: int, threads: int):
    """Reference path on the host cores: the fp32 restatement in oracle/, greedy."""
    import torch
    from oracle.vui_oracle import Oracle, OracleConfig, init_weights

    torch.set_num_threads(threads)
    cfg = OracleConfig()
    sd = init_weights(cfg, 0, torch.bfloat16)
    o = Oracle(cfg, sd, n_slots=1, max_seq=prompt_len + n_frames + 8, dtype=torch.float32)
    ids = torch.randint(0, cfg.vocab, (prompt_len,), generator=torch.Generator().manual_seed(0))
    with torch.inference_mode():
        h = o.prefill_text(0, ids)[-1:]
        F = torch.nn.functional
        code0 = torch.argmax(F.linear(h, o.w["codec_head.weight"]), dim=-1)
        frame = o.rq_generate(h, code0, top_k=1)
        times = []
        for _ in range(n_frames):
            t0 = time.perf_counter()
            h, cb0, _ = o.backbone_step([0], frame)
            frame = o.rq_generate(h, torch.argmax(cb0, dim=-1), top_k=1)
            times.append(time.perf_counter() - t0)
    return times


def run_reference(args):
    rank, _, world = _dist_env()
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    times = cpu_oracle_frame_times(args.prompt_len, args.warmup + args.steps, threads)[args.warmup:]
    total = sum(times)
    fps = len(times) / total
    line = {
        "impl": "reference", "metric": "codec frames/s", "value": fps, "unit": "frames/s",
        "n_gpus": args.gpus, "steps": len(times), "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "x_realtime": fps / FRAME_RATE,
        "config": {"workload": f"cfg2-shaped: B=1, {args.prompt_len} random text ids, greedy decode, CPU fp32",
                   "streams_per_gpu": 1},
        "cpu_baseline": {"value": fps, "unit": "frames/s", "cores": threads, "kind": "port",
                         "sample": f"{len(times)} greedy frames after a {args.prompt_len}-token prefill, "
                                   "oracle/vui_oracle.py fp32 (torch CPU)"},
        "e2e": {"value": fps, "unit": "frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def reference_cuda_standin(n_streams, lens, K, W, max_seq):
    """The baseline leg for the many-stream figure: the oracle's algorithm batched in torch bf16 on this GPU,
    one CUDA graph for the backbone step and one for the depth loop, as the reference captures them
    (oracle/torch_cuda_standin.py says what it is and is not).  Returns ms per step."""
    import torch
    from oracle.torch_cuda_standin import TorchGraphDecoder
    from oracle.vui_oracle import OracleConfig, init_weights

    cfg = OracleConfig()
    dec = TorchGraphDecoder(cfg, init_weights(cfg, 0, torch.bfloat16), n_streams, max_seq)
    g = torch.Generator().manual_seed(7)
    dec.k_cache.copy_((torch.randn(dec.k_cache.shape[1:], generator=g) * 0.5).to(torch.bfloat16))
    dec.v_cache.copy_((torch.randn(dec.v_cache.shape[1:], generator=g) * 0.5).to(torch.bfloat16))
    dec.seq_lens.copy_(torch.tensor(lens))
    dec.codes.copy_(torch.randint(0, cfg.codebook_size, tuple(dec.codes.shape), generator=g))
    dec.capture()
    for _ in range(W):
        dec.step()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(K):
        dec.step()
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / K
    del dec
    torch.cuda.empty_cache()
    return ms


class Bench:
    def __init__(self, model, dev, rank, world):
        self.model, self.dev, self.rank, self.world = model, dev, rank, world

    def barrier(self):
        import torch
        import torch.distributed as dist

        torch.cuda.synchronize(self.dev)
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize(self.dev)

    def aggregate(self, units, ms):
        from vui_b200.replicas import aggregate_rate

        return aggregate_rate(units, ms, self.dev)

    # ------------------------------------------------------------------ decode
    def decode(self, B, K, W, reps, prompt_lens, sample, max_seq, clocks=False, e2e=True, phases=False):
        """Prefill B streams, then time `reps` blocks of K frames device-resident (median block) and
        K frames end to end through host buffers."""
        import torch

        from vui_b200 import Engine, GenConfig

        model, dev = self.model, self.dev
        shape = model.shape
        eng = Engine(model=model, max_rows=B, max_seq=max_seq, max_prefill_rows=1024, seed=1234 + self.rank)
        gen = torch.Generator().manual_seed(100 + self.rank)
        rows = [eng.new_row() for _ in range(B)]
        embs = [(r, model.token_emb(torch.randint(0, shape.vocab_size, (1, n), generator=gen)))
                for r, n in zip(rows, prompt_lens)]
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        hs = eng._prefill_many(embs)
        torch.cuda.synchronize(dev)
        prefill_first_s = time.perf_counter() - t0
        hidden = torch.stack([h[-1] for h in hs])
        cfg = GenConfig(temperature=0.8, top_k=50, rep_penalty=1.0)
        eng._apply_cfg(cfg, greedy=not sample)
        eng._g_slot_idx[:B] = torch.tensor([r.idx for r in rows], device=dev, dtype=torch.int32)
        eng._g_seq_inc[:B].fill_(1)
        eng._g_codes_in[:B] = eng._first_frames(rows, hidden)
        launches0 = eng.launch_count()
        graph = eng._frame_graph(B)
        launches_per_frame = (eng.launch_count() - launches0) // 2  # one warm-up + one captured call

        for _ in range(W):
            graph.replay()
        seq0 = eng.seq_lens.clone()
        codes0 = eng._g_codes_in.clone()
        sampler = ClockSampler(dev.index or 0) if clocks else None
        if sampler:
            sampler.start()
        block_ms = []
        for _ in range(reps):
            eng.seq_lens.copy_(seq0)
            eng._g_codes_in.copy_(codes0)
            self.barrier()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            for _ in range(K):
                graph.replay()
            ev1.record()
            self.barrier()
            block_ms.append(ev0.elapsed_time(ev1))
        clk = sampler.stop() if sampler else None
        eng.check_device()
        ms = statistics.median(block_ms)
        mean_T = float(sum(prompt_lens)) / B + W + K / 2.0

        # end to end: host-driven loop, codes H2D + replay + codes/EOS D2H every frame
        lat, e2e_ms = [], None
        if e2e:
            # the library captures its host-to-host frame graph on first use: outside the timed region
            eng._frame_host(B, eng._g_codes_in[:B].cpu().pin_memory())
            e2e_blocks = []
            for _ in range(max(1, min(reps, 5))):
                eng.seq_lens.copy_(seq0)
                eng._g_codes_in.copy_(codes0)
                h_in = eng._g_codes_in[:B].cpu().pin_memory()
                self.barrier()
                t0 = time.perf_counter()
                for _ in range(K):  # one library call per frame: H2D codes, the frame, D2H codes + EOS, one graph launch
                    t1 = time.perf_counter()
                    h_codes, h_eos = eng._frame_host(B, h_in)
                    h_in.copy_(h_codes)
                    lat.append(time.perf_counter() - t1)
                torch.cuda.synchronize(dev)
                e2e_blocks.append((time.perf_counter() - t0) * 1e3)
            e2e_ms = statistics.median(e2e_blocks)
            lat.sort()

        phase = {}
        if phases and self.rank == 0:
            import ctypes as C

            P = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
            eng.seq_lens.copy_(seq0)
            e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            tb = td = 0.0
            n = 10
            for _ in range(n):
                e0.record()
                eng._ck(eng._lib.vuib_backbone_step(eng._handle, B, P(eng._g_slot_idx), P(eng._g_seq_inc),
                                                    P(eng._g_codes_in), P(eng._g_hidden_out), P(eng._g_cb0_out),
                                                    P(eng._g_eos_out), eng._stream))
                e1.record()
                eng._ck(eng._lib.vuib_depth_step(eng._handle, B, P(eng._g_slot_idx), P(eng._g_hidden_out),
                                                 P(eng._g_cb0_out), P(eng._g_eos_out), 0, P(eng._g_codes_in),
                                                 P(eng._g_eos_prob), eng._stream))
                e2.record()
                torch.cuda.synchronize(dev)
                tb += e0.elapsed_time(e1)
                td += e1.elapsed_time(e2)
            phase = {"backbone_ms_eager": tb / n, "depth_ms_eager": td / n}

        fps, ms_max = self.aggregate(B * K, ms)
        e2e_fps = self.aggregate(B * K, e2e_ms)[0] if e2e_ms else None
        w_bytes = model.weight_bytes_per_step()
        step_bytes = w_bytes + B * (GATHER_BYTES_PER_STREAM + KV_BYTES_PER_POS * (mean_T + 1))
        res = {
            "B": B, "K": K, "reps": reps, "fps": fps, "e2e_fps": e2e_fps, "ms_per_step": ms_max / K,
            "block_ms_min": min(block_ms), "block_ms_max": max(block_ms), "lat": lat, "mean_T": mean_T,
            "max_seq": eng.max_seq, "prefill_first_s": prefill_first_s, "prefill_tokens": int(sum(prompt_lens)),
            "launches_per_frame": launches_per_frame, "step_bytes": step_bytes, "phase": phase, "clocks": clk,
            "greedy": not sample,
        }
        del graph, eng
        torch.cuda.empty_cache()
        return res

    # ------------------------------------------------------------------- cfg 4
    def voice_clone(self, n_streams=16, n_text=128, n_frames_prompt=125, n_decode=375):
        """Configuration 4: every prompt is 128 text ids followed by 125 codec frames; batched prefill
        (tcgen05 GEMMs), then greedy frames.  Reports prefill tokens/s (first call and warm) and the
        time to the first frame on the host."""
        import torch

        from vui_b200 import Engine

        model, dev = self.model, self.dev
        eng = Engine(model=model, max_rows=n_streams, max_seq=640, max_prefill_rows=4096, seed=77 + self.rank)
        g = torch.Generator().manual_seed(400 + self.rank)
        ids = [torch.randint(0, model.shape.vocab_size, (1, n_text), generator=g) for _ in range(n_streams)]
        codes = [torch.randint(0, model.shape.codebook_size, (n_frames_prompt, model.shape.n_quantizers), generator=g)
                 for _ in range(n_streams)]
        h_ids = [t.pin_memory() for t in ids]
        h_codes = [t.pin_memory() for t in codes]
        eng._apply_cfg(None, greedy=True)

        def prefill_and_first_frame():
            """From host buffers to the first frame's codes back on the host."""
            rows = list(eng._rows.values())
            t0 = time.perf_counter()
            items = []
            for r, i_, c_ in zip(rows, h_ids, h_codes):
                items.append((r, model.token_emb(i_.to(dev, non_blocking=True))))
                items.append((r, eng._audio_emb(c_.to(dev, non_blocking=True))))
            outs = eng._prefill_many(items)
            torch.cuda.synchronize(dev)
            t_prefill = time.perf_counter() - t0
            hidden = torch.stack([outs[2 * i + 1][-1] for i in range(n_streams)])
            first = eng._first_frames(rows, hidden)
            first_host = first.cpu()
            return t_prefill, time.perf_counter() - t0, hidden, first, first_host

        for _ in range(n_streams):
            eng.new_row()
        t_first, ttff_first, *_ = prefill_and_first_frame()
        warm_p, warm_t = [], []
        for _ in range(5):
            for r in eng._rows.values():
                eng._rewind_row(r, 0)
            self.barrier()
            tp, tt, hidden, first, _ = prefill_and_first_frame()
            warm_p.append(tp)
            warm_t.append(tt)
        tokens = n_streams * (n_text + n_frames_prompt)
        t_warm, ttff = statistics.median(warm_p), statistics.median(warm_t)
        # decode
        B = n_streams
        rows = list(eng._rows.values())
        eng._g_slot_idx[:B] = torch.tensor([r.idx for r in rows], device=dev, dtype=torch.int32)
        eng._g_seq_inc[:B].fill_(1)
        eng._g_codes_in[:B] = first
        graph = eng._frame_graph(B)
        for _ in range(3):
            graph.replay()
        self.barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(n_decode - 4):
            graph.replay()
        ev1.record()
        self.barrier()
        ms = ev0.elapsed_time(ev1)
        eng.check_device()
        fps, ms_max = self.aggregate(B * (n_decode - 4), ms)
        tok_s, _ = self.aggregate(tokens, t_warm * 1e3)
        res = {
            "workload": f"cfg4: {n_streams} streams x ({n_text} text ids + {n_frames_prompt} codec frames), batched prefill, "
                        f"{n_decode} greedy frames",
            "prefill_tokens_per_s": tok_s, "prefill_ms_warm": t_warm * 1e3, "prefill_tokens": tokens,
            "prefill_tokens_per_s_first_call": tokens / t_first, "time_to_first_frame_ms": ttff * 1e3,
            "time_to_first_frame_ms_first_call": ttff_first * 1e3,
            "decode_frames_per_s": fps, "decode_ms_per_step": ms_max / (n_decode - 4),
            "prefill_flops_frac_of_bf16_peak": None,
        }
        # 0.61 GFLOP per position (2 x 302 M backbone parameters + heads); peak from MEASURED_PEAKS.json when present
        p = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.exists(p):
            with open(p) as f:
                peak = float(json.load(f).get("bf16_tflops_sustained", 0) or 0)
            if peak > 0:
                res["prefill_flops_frac_of_bf16_peak"] = tokens * 0.61e9 / t_warm / (peak * 1e12)
        del graph, eng
        torch.cuda.empty_cache()
        return res


def codec_weight_bytes() -> int:
    """Bytes of codec weights one frame touches: every decoder tensor once, except the quantizer's encoder-side
    input projections (unused when decoding) and the codebooks, of which one 1 KiB row each is gathered."""
    from vui_b200.codec import codec_param_shapes

    n = 0
    for name, shape in codec_param_shapes().items():
        if name.endswith("input_proj.weight") and name.startswith("quantizer."):
            continue
        if name.endswith(".embed"):
            n += 256
            continue
        k = 1
        for d in shape:
            k *= d
        n += k
    return 4 * n


def codec_block(dev, cpu_baseline: bool, frames: int = 100, reps: int = 5, model=None):
    """Streaming codec decode of one stream: `frames` consecutive frames per block (transformer positions
    10..10+frames), median block; device-resident codes for `ms_per_frame`, pinned host codes in and audio out
    every frame for `e2e`."""
    import torch

    from vui_b200.codec import QwenCodecDecoder

    dec = QwenCodecDecoder.random_init(0, device=dev)
    dec.setup_streaming_graph()
    g = dec._graph_for(16)
    codes = torch.randint(0, 2048, (16, 10 + frames), generator=torch.Generator().manual_seed(5)).to(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    blocks = []
    for _ in range(reps):
        with dec.streaming(1):
            for t in range(10):
                dec._codes_in.copy_(codes[:, t])
                g.replay()
            torch.cuda.synchronize(dev)
            e0.record()
            for t in range(10, 10 + frames):
                dec._codes_in.copy_(codes[:, t])
                g.replay()
            e1.record()
            torch.cuda.synchronize(dev)
            blocks.append(e0.elapsed_time(e1))
    ms = statistics.median(blocks) / frames
    # end to end: host codes -> device, replay, audio -> host, every frame
    h_codes = codes.cpu().pin_memory()
    h_audio = torch.empty(1920, dtype=torch.float32).pin_memory()
    with dec.streaming(1):
        t0 = None
        for t in range(10 + frames):
            if t == 10:
                torch.cuda.synchronize(dev)
                t0 = time.perf_counter()
            dec._codes_in.copy_(h_codes[:, t], non_blocking=True)
            g.replay()
            h_audio.copy_(dec._audio, non_blocking=True)
            torch.cuda.current_stream(dev).synchronize()
        e2e_ms = 1e3 * (time.perf_counter() - t0) / frames
    dec.check_device()
    stream_ms = frame_graph = None
    if model is not None:
        from vui_b200 import Engine, GenConfig

        eng = Engine(model=model, max_rows=1, max_seq=1024)
        row = eng.new_row()
        hid = eng.prefill_ids(row, torch.randint(0, model.shape.vocab_size, (64,), generator=torch.Generator().manual_seed(0)))
        eng._apply_cfg(GenConfig(), greedy=True)
        eng._g_slot_idx[:1] = row.idx
        eng._g_seq_inc[:1].fill_(1)
        eng._g_codes_in[:1] = eng._first_frames([row], hid[None])
        frame_graph = eng._frame_graph(1)
    if frame_graph is not None:
        # what Row.stream costs per frame of audio: one generation step + one codec frame, on one stream, and with
        # the codec frame of step k on a second stream beside the generation of step k + 1
        stream_ms = {}
        main, side = torch.cuda.current_stream(dev), torch.cuda.Stream(dev)
        for mode in ("one_stream", "codec_on_second_stream"):
            with dec.streaming(1):
                for t in range(8 + frames):
                    if t == 8:
                        torch.cuda.synchronize(dev)
                        e0.record()
                    frame_graph.replay()
                    dec._codes_in.copy_(codes[:, t % codes.shape[1]])
                    if mode == "one_stream":
                        g.replay()
                    else:
                        side.wait_stream(main)
                        with torch.cuda.stream(side):
                            g.replay()
                        if t + 1 == 8 + frames:
                            main.wait_stream(side)
                e1.record()
                torch.cuda.synchronize(dev)
            stream_ms[mode] = e0.elapsed_time(e1) / frames
    wbytes = codec_weight_bytes()
    kv = 8 * 16 * 64 * 4 * 2 * (10 + frames / 2)
    peak, _ = measured_hbm_peak()
    res = {
        "workload": "streaming codec decode, one stream, 16 codebooks, fp32, seeded random weights; "
                    f"{frames} consecutive frames per block, median of {reps} blocks",
        "ms_per_frame": ms, "frames_per_s": 1e3 / ms, "x_realtime": 1e3 / ms / FRAME_RATE,
        "e2e_ms_per_frame": e2e_ms, "h2d_bytes_per_frame": 128, "d2h_bytes_per_frame": 7680,
        "launches_per_frame": 87, "weight_bytes_per_frame": wbytes,
        "roofline_frac": (wbytes + kv) / (ms * 1e-3) / 1e9 / peak,
    }
    if stream_ms is not None:
        res["generation_plus_codec_ms_per_frame"] = stream_ms
    if cpu_baseline:
        from oracle.codec_oracle import CodecOracle
        from vui_b200.codec import random_codec_state

        torch.set_num_threads(os.cpu_count() or 1)
        orc = CodecOracle(random_codec_state(0))
        cc = codes.cpu()
        for t in range(2):
            orc.decode(cc[None, :, t:t + 1])
        t0 = time.perf_counter()
        for t in range(2, 12):
            orc.decode(cc[None, :, t:t + 1])
        cpu_ms = 1e3 * (time.perf_counter() - t0) / 10
        res["cpu_baseline"] = {"value": 1e3 / cpu_ms, "unit": "frames/s", "cores": os.cpu_count() or 1, "kind": "port",
                               "sample": "10 streamed frames, oracle/codec_oracle.py fp32 on torch CPU"}
    del dec
    torch.cuda.empty_cache()
    return res


def codec_encoder_block(dev, cpu_baseline: bool, reps: int = 5):
    """Codec encoder: one call of StreamingCodecEncoder's whole-buffer encode (10 s of audio -> 16 x 125 codes)."""
    import torch

    from oracle.codec_enc_oracle import test_audio
    from vui_b200.codec_encoder import QwenCodecEncoder, StreamingCodecEncoder

    enc = QwenCodecEncoder.random_init(0, device=dev)
    se = StreamingCodecEncoder(enc)
    se.setup_graph()
    se._audio_buf.copy_(test_audio(240000, seed=0).to(dev))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for _ in range(reps):
        torch.cuda.synchronize(dev)
        e0.record()
        se._graph.replay()
        e1.record()
        torch.cuda.synchronize(dev)
        times.append(e0.elapsed_time(e1))
    ms = statistics.median(times)
    res = {"workload": "codec encoder, 10 s buffer (240000 samples -> 16 x 125 codes), fp32, seeded random weights; "
                       f"median of {reps} graph replays",
           "ms_per_buffer": ms, "x_realtime": 10e3 / ms, "launches": 75, "gflop": 40.0, "tflops": 40.0 / ms}
    if cpu_baseline:
        from oracle.codec_enc_oracle import EncoderOracle
        from vui_b200.codec_encoder import random_encoder_state

        torch.set_num_threads(os.cpu_count() or 1)
        orc = EncoderOracle(random_encoder_state(0))
        a = test_audio(240000, seed=0)
        orc.encode(a)
        t0 = time.perf_counter()
        for _ in range(3):
            orc.encode(a)
        res["cpu_baseline"] = {"value": 1e3 * (time.perf_counter() - t0) / 3, "unit": "ms per buffer", "cores": os.cpu_count() or 1,
                               "kind": "port", "sample": "3 encodes of the same buffer, oracle/codec_enc_oracle.py fp32 on torch CPU"}
    del se, enc
    torch.cuda.empty_cache()
    return res


def profile_codec(dev, n):
    """`n` streamed codec frames kernel by kernel (no graph) after 3 warm-up frames: for ncu."""
    import torch

    from vui_b200.codec import QwenCodecDecoder

    dec = QwenCodecDecoder.random_init(0, device=dev)
    codes = torch.randint(0, 2048, (1, 16, 3 + n), generator=torch.Generator().manual_seed(5)).to(dev)
    with dec.streaming(1):
        for t in range(3):
            dec(codes[:, :, t:t + 1])
        torch.cuda.synchronize(dev)
        before = dec.launch_count()
        for t in range(3, 3 + n):
            dec(codes[:, :, t:t + 1])
        torch.cuda.synchronize(dev)
    dec.check_device()
    print(json.dumps({"profile_codec": n, "launches_before_frames": before,
                      "launches_per_frame": (dec.launch_count() - before) // max(n, 1)}), flush=True)


def profile_encoder(dev, n):
    """`n` whole-buffer encodes of the codec encoder kernel by kernel after one warm-up call: for ncu."""
    import torch

    from oracle.codec_enc_oracle import test_audio
    from vui_b200.codec_encoder import QwenCodecEncoder

    enc = QwenCodecEncoder.random_init(0, device=dev)
    a = test_audio(240000, seed=0).to(dev)
    enc(a)
    torch.cuda.synchronize(dev)
    before = enc.launch_count()
    for _ in range(n):
        enc(a)
    torch.cuda.synchronize(dev)
    print(json.dumps({"profile_encoder": n, "launches_before": before,
                      "launches_per_encode": (enc.launch_count() - before) // max(n, 1)}), flush=True)


def profile_frames(model, dev, n, B, prompt_len):
    """Prefill B streams of `prompt_len` ids, then `n` frames kernel by kernel (no graph): the command the
    `ncu` launch lists and captures under profiles/ are taken with."""
    import torch

    from vui_b200 import Engine, GenConfig

    eng = Engine(model=model, max_rows=B, max_seq=1024, max_prefill_rows=4096)
    rows = [eng.new_row() for _ in range(B)]
    g = torch.Generator().manual_seed(0)
    hs = eng._prefill_many([(r, model.token_emb(torch.randint(0, model.shape.vocab_size, (1, prompt_len), generator=g)))
                            for r in rows])
    h = torch.stack([x[-1] for x in hs])
    eng._apply_cfg(GenConfig(temperature=0.8, top_k=50, rep_penalty=1.0), greedy=(B == 1))
    eng._g_slot_idx[:B] = torch.tensor([r.idx for r in rows], device=dev, dtype=torch.int32)
    eng._g_seq_inc[:B].fill_(1)
    eng._g_codes_in[:B] = eng._first_frames(rows, h)
    torch.cuda.synchronize(dev)
    before = eng.launch_count()
    for _ in range(n):
        eng._frame_call(B)
    torch.cuda.synchronize(dev)
    eng.check_device()
    print(json.dumps({"profile_frames": n, "streams": B, "launches_before_frames": before,
                      "launches_per_frame": (eng.launch_count() - before) // max(n, 1)}), flush=True)


def run_b200(args):
    import torch
    import torch.distributed as dist

    rank, local_rank, world = _dist_env()
    if world > 1:
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = torch.device("cuda", local_rank if world > 1 else 0)
    torch.cuda.set_device(dev)

    from vui_b200 import VuiB200, VuiShape

    if args.profile_codec:
        profile_codec(dev, args.profile_codec)
        return
    if args.profile_encoder:
        profile_encoder(dev, args.profile_encoder)
        return
    model = VuiB200.random_init(VuiShape(), seed=0, device=dev)
    if args.profile_frames:
        profile_frames(model, dev, args.profile_frames, args.streams, args.prompt_len)
        return
    b = Bench(model, dev, rank, world)
    B, W, K = args.streams, args.warmup, args.steps
    ceiling = model.shape.max_seq_len
    if B == 1 and not args.ragged:
        lens, max_seq = [args.prompt_len], max(1024, 64 * ((args.prompt_len + K + W + 80) // 64))
    elif args.ragged:
        lens = torch.randint(64, 513, (B,), generator=torch.Generator().manual_seed(1)).tolist()
        max_seq = 64 * ((512 + K + W + 80) // 64)
    else:
        lens, max_seq = [args.prompt_len] * B, 64 * ((args.prompt_len + K + W + 80) // 64)
    K = min(K, ceiling - max(lens) - W - 40)
    max_seq = min(max_seq, ceiling)
    m = b.decode(B, K, W, args.reps, lens, args.sample, max_seq, clocks=True, phases=True)
    extra = cfg4 = wide = standin_ms = codec = None
    if B == 1 and not args.no_batched and rank == 0:
        try:
            codec = codec_block(dev, world == 1 and not args.no_cpu_baseline, model=model)
            codec["encoder"] = codec_encoder_block(dev, world == 1 and not args.no_cpu_baseline)
        except Exception as exc:  # noqa: BLE001 - an extra block must never take the bench line down
            print(f"codec block failed: {exc}", file=sys.stderr)
    if B == 1 and not args.no_batched:
        lens64 = torch.randint(64, 513, (64,), generator=torch.Generator().manual_seed(1)).tolist()
        k64 = min(K, 100)
        extra = b.decode(64, k64, W, min(args.reps, 5), lens64, True, 64 * ((512 + k64 + W + 80) // 64))
        if rank == 0 and world == 1 and not args.no_cpu_baseline:
            try:
                standin_ms = reference_cuda_standin(64, lens64, min(k64, 30), 3, 64 * ((512 + k64 + W + 80) // 64))
            except Exception as exc:  # noqa: BLE001 - the stand-in must never take the bench line down
                print(f"reference_cuda_standin failed: {exc}", file=sys.stderr)
        cfg4 = b.voice_clone()
        k256 = min(K, 50)
        wide = b.decode(256, k256, W, 3, [512] * 256, True, 2048, e2e=False)
    if rank == 0:
        peak, peak_kind = measured_hbm_peak()
        K, lat = m["K"], m["lat"]
        achieved = m["step_bytes"] / (m["ms_per_step"] * 1e-3) / 1e9
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            ct = cpu_oracle_frame_times(args.prompt_len, 24, threads)[4:]
            cpu = {"value": len(ct) / sum(ct), "unit": "frames/s", "cores": threads, "kind": "port",
                   "sample": f"20 greedy frames after a {args.prompt_len}-token prefill (the headline's shape), "
                             "oracle/vui_oracle.py fp32 on torch CPU"}
        line = {
            "metric": "codec frames/s", "value": m["fps"], "unit": "frames/s", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": m["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "x_realtime": m["fps"] / FRAME_RATE,
            "config": {
                "workload": (f"cfg2: B=1, {args.prompt_len} random text ids, greedy, KV<=1024" if B == 1 and m["greedy"]
                             else f"{B} streams/GPU, prompts {'U[64,512]' if args.ragged else args.prompt_len}, "
                                  f"{'greedy' if m['greedy'] else 'T=0.8 top-k 50'}"),
                "streams_per_gpu": B, "max_seq": m["max_seq"], "mean_kv_len": m["mean_T"],
                "l2": "inputs larger than L2: 666 MB of weights are streamed every step",
                "replicas": world,
                "timing": f"median of {m['reps']} blocks of {K} steps (stream rewound between blocks); "
                          f"block min/max {m['block_ms_min']:.3f}/{m['block_ms_max']:.3f} ms",
                "prefill_first_call_s": m["prefill_first_s"],
            },
            "e2e": {"value": m["e2e_fps"], "unit": "frames/s", "h2d_bytes_per_step": B * 16 * 8,
                    "d2h_bytes_per_step": B * 16 * 8 + B * 4,
                    "p50_frame_latency_ms": 1e3 * lat[len(lat) // 2], "p95_frame_latency_ms": 1e3 * lat[int(len(lat) * 0.95)]},
            "gpu_launches": m["launches_per_frame"] * K * m["reps"],
            "launches_per_frame": m["launches_per_frame"],
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": None,
                         "traffic_note": "per-kernel DRAM bytes of the dominant kernels are in profiles/ (ncu captures of a few "
                                         "launches each); no whole-frame figure is quoted here",
                         "peak_source": peak_kind,
                         "kernel": f"frame graph ({m['launches_per_frame']} launches)",
                         "bytes_per_step": m["step_bytes"], **m["phase"]},
            "cpu_baseline": cpu,
            "clocks": m["clocks"],
        }
        if extra is not None:
            ach = extra["step_bytes"] / (extra["ms_per_step"] * 1e-3) / 1e9
            line["streams64"] = {
                "workload": "cfg3: 64 streams/GPU, prompts U[64,512], T=0.8 top-k 50 (tcgen05 GEMM path)",
                "value": extra["fps"], "unit": "frames/s (aggregate)", "x_realtime": extra["fps"] / FRAME_RATE,
                "ms_per_step": extra["ms_per_step"], "steps": extra["K"], "reps": extra["reps"], "e2e": extra["e2e_fps"],
                "p50_frame_latency_ms": 1e3 * extra["lat"][len(extra["lat"]) // 2],
                "launches_per_frame": extra["launches_per_frame"], "mean_kv_len": extra["mean_T"],
                "prefill_tokens_per_s_first_call": extra["prefill_tokens"] / extra["prefill_first_s"],
                "roofline_frac": ach / peak, "bytes_per_step": extra["step_bytes"],
            }
            if standin_ms:
                line["streams64"]["reference_cuda_standin"] = {
                    "what": "torch bf16 (cuBLAS, SDPA with a length mask) restatement of the reference's CUDA path on this "
                            "GPU, backbone step and depth loop as two CUDA graphs; stands in for the reference, which "
                            "cannot run on this box",
                    "ms_per_step": standin_ms, "value": 64 / (standin_ms * 1e-3), "unit": "frames/s (aggregate)",
                    "speedup": standin_ms / extra["ms_per_step"],
                }
        if cfg4 is not None:
            line["cfg4"] = cfg4
        if codec is not None:
            line["codec"] = codec
        if wide is not None:
            ach = wide["step_bytes"] / (wide["ms_per_step"] * 1e-3) / 1e9
            line["streams256"] = {
                "workload": "cfg5 per-GPU shape: 256 streams/GPU, 512-id prompts, 2048-position KV, T=0.8 top-k 50; "
                            "aggregate over all replicas",
                "value": wide["fps"], "unit": "frames/s (aggregate)", "x_realtime": wide["fps"] / FRAME_RATE,
                "ms_per_step": wide["ms_per_step"], "steps": wide["K"], "reps": wide["reps"],
                "launches_per_frame": wide["launches_per_frame"], "mean_kv_len": wide["mean_T"],
                "prefill_tokens_per_s_first_call": wide["prefill_tokens"] / wide["prefill_first_s"],
                "roofline_frac": ach / peak, "bytes_per_step": wide["step_bytes"],
            }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--reps", type=int, default=25, help="timed blocks of --steps frames; the median is reported")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--streams", type=int, default=1, help="concurrent streams per GPU")
    ap.add_argument("--prompt-len", type=int, default=256)
    ap.add_argument("--ragged", action="store_true", help="prompt lengths U[64,512] (config 3)")
    ap.add_argument("--sample", action="store_true", help="T=0.8 top-k 50 instead of greedy")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-batched", action="store_true", help="skip the 64-stream, cfg4 and 256-stream blocks")
    ap.add_argument("--profile-frames", type=int, default=0, help="run N frames without a graph and exit (for ncu)")
    ap.add_argument("--profile-codec", type=int, default=0, help="run N streamed codec frames without a graph and exit")
    ap.add_argument("--profile-encoder", type=int, default=0, help="run N codec-encoder calls on a 10 s buffer and exit")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        if args.steps > 200:
            args.steps = 200  # bounded sample: ~30 ms per CPU frame
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
