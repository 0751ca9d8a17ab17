#!/usr/bin/env python
"""Decode throughput of the B200 backend on the Llama-3-8B-shape config (BASELINE configs[4]):
32 layers, hidden 4096, 32 q / 8 kv heads x 128, MLP 14336, vocab 128256, bf16, batch 32,
KV context 7680..8191, greedy decode.  Weights and the KV context are synthetic (seeded
generator; there is no checkpoint or dataset on this path).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line on stdout (rank 0).  A step is one decode step: one new token for each of the 32
sequences.  `value` = tokens/s with tokens resident on the device (CUDA-graph replay, CUDA
events); `e2e` = the same through lmb200_decode_step with pinned host buffers (H2D of the token
ids and D2H of the next ids inside every timed step).  N > 1 shards heads and MLP columns
tensor-parallel, one process per GPU (launch with torch.distributed.run).
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

CFG = dict(n_layers=32, hidden=4096, n_heads=32, n_kv_heads=8, intermediate=14336, vocab=128256,
           eps=1e-5, rope_base=500000.0)
BATCH = 32
MAX_CTX = 8192
WORKLOAD = "llama3-8b-shape decode, bf16, batch 32, KV context ending at 8192"
METRIC = "decode_tokens_per_sec"


def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.thread.join(timeout=2)
        clk = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = set()
        for r in self.rows:
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": clk[len(clk) // 2] if clk else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(clk)}


# -------------------------------------------------------------------------------------------------
# CPU baseline: the oracle (reference semantics, float32, per-op materialisation, one BLAS call
# per batch slice as src/Execution.jl:21-29 does) on the host cores, bounded sample.
# -------------------------------------------------------------------------------------------------
def cpu_baseline(layers=2, steps=2, ctx=256):
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import luminal_oracle as O
    cfg = dict(CFG, n_layers=layers)
    rng = np.random.default_rng(0)
    H, KV, hid, inter = cfg["n_heads"], cfg["n_kv_heads"], cfg["hidden"], cfg["intermediate"]
    D = hid // H

    def rnd(*shape):
        return (rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02))

    w = {}
    for i in range(layers):
        n = O.layer_names(i)
        w[n["attn_norm"]] = np.ones(hid, np.float32); w[n["ffn_norm"]] = np.ones(hid, np.float32)
        w[n["q"]] = rnd(H * D, hid); w[n["k"]] = rnd(KV * D, hid); w[n["v"]] = rnd(KV * D, hid)
        w[n["o"]] = rnd(hid, H * D); w[n["gate"]] = rnd(inter, hid); w[n["up"]] = rnd(inter, hid)
        w[n["down"]] = rnd(hid, inter)
    # the head and the embedding are timed on a 1/8 slice of the vocabulary and scaled
    vslice = cfg["vocab"] // 8
    w["model.embed_tokens.weight"] = rnd(vslice, hid)
    w["model.norm.weight"] = np.ones(hid, np.float32)
    w["lm_head.weight"] = rnd(vslice, hid)
    cfg_s = dict(cfg, vocab=vslice)
    model = O.CachedLlama(w, cfg_s, BATCH, ctx + steps + 1)
    model.k[:, :, :, :ctx] = rng.standard_normal(model.k[:, :, :, :ctx].shape, dtype=np.float32)
    model.v[:, :, :, :ctx] = rng.standard_normal(model.v[:, :, :, :ctx].shape, dtype=np.float32)
    model.pos = ctx
    toks = rng.integers(0, vslice, size=(BATCH, 1))
    model.forward(toks)                      # warm-up (BLAS threads, page faults)
    # time the head alone to separate it from the layers
    x = rnd(BATCH, 1, hid)
    t0 = time.perf_counter()
    O.linear(O.rms_norm(x, w["model.norm.weight"], cfg["eps"]), w["lm_head.weight"])
    t_head_slice = time.perf_counter() - t0
    t0 = time.perf_counter()
    for _ in range(steps):
        model.forward(toks)
    t_step = (time.perf_counter() - t0) / steps
    t_layer = max(t_step - t_head_slice, 1e-9) / layers
    # linear extrapolation: 32 layers + the full-vocabulary head (attention cost at ctx, not 8192)
    t_full = t_layer * CFG["n_layers"] + t_head_slice * 8
    return {"value": BATCH / t_full, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
            "sample": (f"oracle, float32, batch {BATCH}, {layers} full-width layers x {steps} decode steps at "
                       f"context {ctx} + 1/8 of the head; extrapolated linearly to 32 layers and the full "
                       f"head (attention cost at context {ctx}, not 8192: favours the CPU)"),
            "ms_per_step_extrapolated": t_full * 1e3}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t_all = []
    base = None
    for _ in range(max(1, min(args.steps, 3))):
        base = cpu_baseline(layers=2, steps=1, ctx=256)
        t_all.append(base["ms_per_step_extrapolated"])
    ms = sorted(t_all)[len(t_all) // 2]
    val = BATCH / (ms / 1e3)
    base = dict(base, value=val)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "batch": BATCH, "note": "CPU oracle port of the reference path"},
        "cpu_baseline": base,
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    global BATCH
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--layers", type=int, default=CFG["n_layers"], help="debug only: fewer layers (invalid as a result)")
    ap.add_argument("--batch", type=int, default=BATCH, help="debug only: another batch size (invalid as a result)")
    args = ap.parse_args()
    BATCH = args.batch
    if args.impl == "reference":
        run_reference(args)
        return

    import numpy as np
    import torch
    import luminal_jl_b200 as L

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    warm = max(args.warmup, 3)
    steps = args.steps
    if steps + warm > MAX_CTX - 1:
        raise SystemExit("steps + warmup exceed the 8192-token context")
    ctx_start = MAX_CTX - steps - warm           # the timed steps end exactly at 8192

    stream = torch.cuda.Stream()
    dev = L.B200Device(local, stream=stream.cuda_stream)
    if world > 1:
        uid = [L.B200Device.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        dev.comm_init(world, rank, uid[0])
    cfg = dict(CFG, n_layers=args.layers)
    model = L.Model(dev, dtype="bf16", tp_size=world, tp_rank=rank, **cfg)
    model.init_random(1234, 0.02)
    sess = L.Session(model, BATCH, MAX_CTX)
    sess.fill_kv_random(ctx_start, seed=1234)

    first = torch.randint(0, CFG["vocab"], (BATCH,), dtype=torch.int32, device="cuda")
    out_dev = torch.empty((steps, BATCH), dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident loop -------------------------------------------------------------------
    with torch.cuda.stream(stream):
        sess.decode_n_device(first.data_ptr(), warm, None)
        barrier()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        launches0 = dev.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        sess.decode_n_device(None, steps, out_dev.data_ptr())
        e1.record(stream)
        barrier()
        launches = dev.launch_count() - launches0
        clocks = sampler.stop() if rank == 0 else None
    ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    if dist is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total = float(ms.item())

    # ---- end to end through the host-buffer call ------------------------------------------------
    sess.set_position(ctx_start)
    tok_in = torch.randint(0, CFG["vocab"], (BATCH,), dtype=torch.int32).pin_memory()
    tok_out = torch.empty(BATCH, dtype=torch.int32).pin_memory()
    e2e_steps = steps
    with torch.cuda.stream(stream):
        for _ in range(warm):
            sess.decode_step_raw(tok_in.data_ptr(), tok_out.data_ptr())
            tok_in.copy_(tok_out)
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record(stream)
        for _ in range(e2e_steps):
            sess.decode_step_raw(tok_in.data_ptr(), tok_out.data_ptr())
            tok_in.copy_(tok_out)                      # the result feeds the next step, on the host
        f1.record(stream)
        barrier()
    ms2 = torch.tensor([f0.elapsed_time(f1)], device="cuda")
    if dist is not None:
        dist.all_reduce(ms2, op=dist.ReduceOp.MAX)
    e2e_ms = float(ms2.item())

    # ---- dominant kernel alone: split-KV decode attention, one launch per layer ------------------
    peak, peak_kind = load_peaks()
    T_mid = MAX_CTX - steps // 2
    Hl = CFG["n_heads"] // world
    KVl = CFG["n_kv_heads"] // world
    D = CFG["hidden"] // CFG["n_heads"]
    q = torch.randn(BATCH, Hl * D, device="cuda").to(torch.bfloat16)
    o = torch.empty_like(q)
    attn_bytes = BATCH * KVl * T_mid * D * 2 * 2 + 2 * q.numel() * 2     # K and V read once, q in, out
    with torch.cuda.stream(stream):
        for l in range(min(3, cfg["n_layers"])):
            sess.decode_attention(l, q.data_ptr(), o.data_ptr(), T_mid)
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record(stream)
        for l in range(cfg["n_layers"]):
            sess.decode_attention(l, q.data_ptr(), o.data_ptr(), T_mid)
        g1.record(stream)
        barrier()
    attn_ms = g0.elapsed_time(g1) / cfg["n_layers"]

    if rank == 0:
        tokens = BATCH * steps
        T_avg = MAX_CTX - (steps + 1) / 2.0
        step_bytes = sess.step_bytes(int(round(T_avg)))
        step_gbs = step_bytes / (ms_total / steps * 1e-3) / 1e9
        attn_gbs = attn_bytes / (attn_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": tokens / (ms_total * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": steps, "warmup": warm, "ms_per_step": ms_total / steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "batch": BATCH, "context": [ctx_start + warm, MAX_CTX],
                       "layers": cfg["n_layers"], "parallelism": f"tp{world}",
                       "l2": "inputs larger than L2: every step streams this rank's weights and KV cache "
                             f"({step_bytes / 1e9:.1f} GB) once"},
            "e2e": {"value": BATCH * e2e_steps / (e2e_ms * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": BATCH * 4, "d2h_bytes_per_step": BATCH * 4, "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": {"kernel": "attn_decode_bf16_kernel<128> (per layer; the last CTA of each sequence and kv head merges the splits)", "bound": "hbm",
                         "achieved": attn_gbs, "peak": peak, "unit": "GB/s", "frac": attn_gbs / peak,
                         "peak_kind": peak_kind,
                         # dram__bytes_read + write of one launch from the ncu capture in
                         # profiles/attn_decode_bf16_llama3_8b_b32_ctx8190.md, scaled by keys x local kv heads
                         "traffic": int(1.0793e9 * (KVl * T_mid) / (8 * 8190.0)) if cfg["n_heads"] == 32 else None,
                         "bytes_per_launch": attn_bytes,
                         "ms_per_launch": attn_ms},
            "step_hbm": {"bytes_per_step_per_gpu": step_bytes, "achieved": step_gbs, "peak": peak, "unit": "GB/s",
                         "frac": step_gbs / peak},
        }
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline()
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line))
    sess.close()
    model.close()
    if dist is not None:
        dist.barrier()
        dev.comm_destroy()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
