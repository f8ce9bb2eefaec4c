"""Benchmark of the Vui-Nano decode step: codec frames/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--streams B] [--impl b200|reference]

A step is one decode frame for every stream of the batch (backbone step, cb0
sampling, 15 depth-transformer codebooks, gather-sum into the next frame's
input), i.e. one replay of the captured frame graph.  Default workload is
benchmark configuration 2: one stream, 256 seeded text ids, greedy decode, KV up to 1024
positions; weights are seeded random-init (no checkpoint is available offline).

Under torchrun (N > 1) every rank is an independent replica with its own streams
on its own GPU; there is no data-path collective, the process group only aligns
the timed window and takes the max time over ranks.

`--impl reference` times the CPU restatement of the reference's PyTorch path
(oracle/, fp32, all host threads) on the same metric.
"""

from __future__ import annotations

import argparse
import json
import os
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
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
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


# DRAM bytes per frame (dram__bytes_read.sum + dram__bytes_write.sum over the launches of one frame)
# from the ncu capture summarised in profiles/frame_graph_b1_dram_traffic.md.
NCU_TRAFFIC_BYTES_PER_FRAME = {1: 945989120}


def ncu_traffic():
    return {f"B{b}": v for b, v in NCU_TRAFFIC_BYTES_PER_FRAME.items()}


def cpu_oracle_frames_per_s(prompt_len: int, n_frames: int, threads: int):
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
    import torch

    threads = os.cpu_count() or 1
    times = cpu_oracle_frames_per_s(args.prompt_len, args.warmup + args.steps, threads)[args.warmup:]
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


def measure(model, dev, rank, world, B, K, W, prompt_len, ragged, sample, max_seq_arg, phases=True):
    """Prefill B streams, then time K frames device-resident and K frames end to end."""
    import torch
    import torch.distributed as dist

    from vui_b200 import Engine, GenConfig

    shape = model.shape
    ceiling = shape.max_seq_len
    K = min(K, (ceiling - 513 - 2 * W - 40) // 2)  # both timed loops must fit the trained context
    plen = 512 if ragged else prompt_len
    max_seq = max_seq_arg or 64 * ((plen + 2 * (K + W) + 16 + 63) // 64 + 1)
    max_seq = max(max_seq, 1024) if B == 1 else max_seq
    eng = Engine(model=model, max_rows=B, max_seq=min(max_seq, model.decoder.max_seqlen), seed=1234 + rank)
    gen = torch.Generator().manual_seed(100 + rank)
    if ragged:
        lens = torch.randint(64, 513, (B,), generator=torch.Generator().manual_seed(1)).tolist()
    else:
        lens = [prompt_len] * B
    rows = [eng.new_row() for _ in range(B)]
    embs = [(r, model.token_emb(torch.randint(0, shape.vocab_size, (1, n), generator=gen))) for r, n in zip(rows, lens)]
    torch.cuda.synchronize(dev)
    t_pref0 = time.perf_counter()
    hs = eng._prefill_many(embs)
    torch.cuda.synchronize(dev)
    prefill_s = time.perf_counter() - t_pref0
    hidden = torch.stack([h[-1] for h in hs])
    cfg = GenConfig(temperature=0.8, top_k=50, rep_penalty=1.0)
    greedy = not sample
    eng._apply_cfg(cfg, greedy=greedy)
    eng._g_slot_idx[:B] = torch.tensor([r.idx for r in rows], device=dev, dtype=torch.int32)
    eng._g_seq_inc[:B].fill_(1)
    eng._g_codes_in[:B] = eng._first_frames(rows, hidden)
    launches0 = eng.launch_count()
    graph = eng._frame_graph(B)
    launches_per_frame = (eng.launch_count() - launches0) // 2  # one warm-up + one captured call

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- device-resident timing: K replays between CUDA events ------------------
    for _ in range(W):
        graph.replay()
    seq_after_warm = eng.seq_lens.clone()
    codes_after_warm = eng._g_codes_in.clone()
    sampler = ClockSampler(dev.index or 0)
    barrier()
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(K):
        graph.replay()
    ev1.record()
    barrier()
    clocks = sampler.stop()
    ms = ev0.elapsed_time(ev1)
    eng.check_device()
    mean_T = float(sum(lens)) / B + W + K / 2.0

    # ---- end to end: host-driven loop, codes H2D + replay + codes/EOS D2H per frame ----
    eng.seq_lens.copy_(seq_after_warm)
    eng._g_codes_in.copy_(codes_after_warm)
    h_in = eng._g_codes_in[:B].cpu().pin_memory()
    lat = []
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        t1 = time.perf_counter()
        eng._g_codes_in[:B].copy_(h_in, non_blocking=True)
        graph.replay()
        h_codes, h_eos = eng._read_frame(B)
        h_in.copy_(h_codes)
        lat.append(time.perf_counter() - t1)
    torch.cuda.synchronize(dev)
    e2e_s = time.perf_counter() - t0
    lat.sort()

    # ---- phase split (eager, events): backbone step vs depth step ---------------
    eng.seq_lens.copy_(seq_after_warm)
    phase = {}
    if rank == 0 and phases:
        P = lambda t: __import__("ctypes").c_void_p(t.data_ptr())  # noqa: E731
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        reps = 10
        tb = td = 0.0
        for _ in range(reps):
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
        phase = {"backbone_ms_eager": tb / reps, "depth_ms_eager": td / reps}

    from vui_b200.replicas import aggregate_rate

    fps, ms_max = aggregate_rate(B * K, ms, dev)
    e2e_fps, _ = aggregate_rate(B * K, e2e_s * 1e3, dev)
    w_bytes = model.weight_bytes_per_step()
    step_bytes = w_bytes + B * (GATHER_BYTES_PER_STREAM + KV_BYTES_PER_POS * (mean_T + 1))
    res = {
        "B": B, "K": K, "fps": fps, "e2e_fps": e2e_fps, "ms_per_step": ms_max / K, "lat": lat, "lens": lens,
        "mean_T": mean_T, "max_seq": eng.max_seq, "prefill_s": prefill_s, "prefill_tokens": int(sum(lens)),
        "launches_per_frame": launches_per_frame, "step_bytes": step_bytes, "phase": phase, "clocks": clocks,
        "greedy": greedy,
    }
    del graph, eng
    torch.cuda.empty_cache()
    return res


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

    model = VuiB200.random_init(VuiShape(), seed=0, device=dev)
    B, W = args.streams, args.warmup
    m = measure(model, dev, rank, world, B, args.steps, W, args.prompt_len, args.ragged, args.sample, args.max_seq)
    extra = None
    if B == 1 and not args.no_batched:
        # benchmark configuration 3's shape beside the headline: 64 streams, prompts U[64,512], T=0.8 top-k 50
        extra = measure(model, dev, rank, world, 64, min(args.steps, 100), W, 0, True, True, 0, phases=False)
    if rank == 0:
        peak, peak_kind = measured_hbm_peak()
        K, lat = m["K"], m["lat"]
        achieved = m["step_bytes"] / (m["ms_per_step"] * 1e-3) / 1e9
        traffic = ncu_traffic().get(f"B{B}")
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            ct = cpu_oracle_frames_per_s(64, 24, threads)[4:]
            cpu = {"value": len(ct) / sum(ct), "unit": "frames/s", "cores": threads, "kind": "port",
                   "sample": "20 greedy frames after a 64-token prefill (benchmark configuration 1 shape), "
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
                "replicas": world, "prefill_s": m["prefill_s"],
                "prefill_tokens_per_s": m["prefill_tokens"] / m["prefill_s"],
            },
            "e2e": {"value": m["e2e_fps"], "unit": "frames/s", "h2d_bytes_per_step": B * 16 * 8,
                    "d2h_bytes_per_step": B * 16 * 8 + B * 4,
                    "p50_frame_latency_ms": 1e3 * lat[len(lat) // 2], "p95_frame_latency_ms": 1e3 * lat[int(len(lat) * 0.95)]},
            "gpu_launches": m["launches_per_frame"] * K,
            "launches_per_frame": m["launches_per_frame"],
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic, "peak_source": peak_kind,
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
                "ms_per_step": extra["ms_per_step"], "steps": extra["K"], "e2e": extra["e2e_fps"],
                "p50_frame_latency_ms": 1e3 * extra["lat"][len(extra["lat"]) // 2],
                "launches_per_frame": extra["launches_per_frame"], "mean_kv_len": extra["mean_T"],
                "prefill_tokens_per_s": extra["prefill_tokens"] / extra["prefill_s"],
                "roofline_frac": ach / peak, "bytes_per_step": extra["step_bytes"],
            }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--streams", type=int, default=1, help="concurrent streams per GPU")
    ap.add_argument("--prompt-len", type=int, default=256)
    ap.add_argument("--max-seq", type=int, default=0)
    ap.add_argument("--ragged", action="store_true", help="prompt lengths U[64,512] (config 3)")
    ap.add_argument("--sample", action="store_true", help="T=0.8 top-k 50 instead of greedy")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-batched", action="store_true", help="skip the extra 64-stream measurement")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        if args.steps > 200:
            args.steps = 200  # bounded sample: ~0.2 s per CPU frame
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
