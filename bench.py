#!/usr/bin/env python
"""Throughput of the B200 backend on the reference's benchmark configurations.

    python bench.py [--config llama3_8b|phi3_mini|whisper_base|small_llama|flash]
                    [--gpus N] [--steps K] [--warmup W] [--repeats R] [--impl ours|reference]

Default: the Llama-3-8B-shape decode (32 layers, hidden 4096, 32 q / 8 kv heads x 128, MLP 14336,
vocab 128256, bf16, batch 32, KV context ending at 8192, greedy).  Weights and the KV context are
synthetic (seeded generator; there is no checkpoint or dataset on this path).

One JSON line on stdout (rank 0).  A step is one decode step: one new token for every sequence of
the batch.  The timed region is exactly K steps bracketed by a barrier and a device synchronise; it
is repeated R times from the same cache position and the MEDIAN region gives `value` (`repeats`
holds min and max).  `value` = tokens/s with the tokens resident on the device (CUDA-graph replay,
CUDA events); `e2e` = the same through lmb200_decode_step with pinned host buffers (H2D of the
token ids and D2H of the next ids inside every timed step).  N > 1 shards heads and MLP columns
tensor-parallel, one process per GPU (launch with torch.distributed.run); before the timed region
such a run checks a small model against the CPU oracle across the N ranks (`tp_parity`) and exits
non-zero when that fails.
"""
from __future__ import annotations

import os

# torch.distributed.run exports OMP_NUM_THREADS=1; the CPU legs (the baseline beside the GPU number
# and --impl reference) must use the host's cores whoever launches them, so the BLAS thread count
# is fixed here, before NumPy or torch load their BLAS.
N_CORES = os.cpu_count() or 1
for _v in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
    os.environ[_v] = str(N_CORES)

import argparse  # noqa: E402
import json  # noqa: E402
import subprocess  # noqa: E402
import sys  # noqa: E402
import threading  # noqa: E402
import time  # noqa: E402

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA3_8B = dict(n_layers=32, hidden=4096, n_heads=32, n_kv_heads=8, intermediate=14336, vocab=128256,
                 eps=1e-5, rope_base=500000.0)
PHI3_MINI = dict(n_layers=32, hidden=3072, n_heads=32, n_kv_heads=8, intermediate=8192, vocab=32064,
                 eps=1e-5, rope_base=10000.0)
SMALL_LLAMA = dict(n_layers=4, hidden=256, n_heads=8, n_kv_heads=8, intermediate=688, vocab=1024,
                   eps=1e-5, rope_base=10000.0)
WHISPER_BASE = dict(d_model=512, heads=8, enc_layers=6, dec_layers=6, ffn=2048, vocab=51865, n_mels=80,
                    max_positions=448)
# decode workloads: the timed steps of llama3_8b END at the cache capacity (positions 8192-K .. 8191);
# those of phi3_mini START after its 2048-token prompt
DECODE = {
    "llama3_8b": dict(cfg=LLAMA3_8B, batch=32, max_ctx=8192, start=None, max_gpus=8,
                      workload="llama3-8b-shape decode, bf16, batch 32, KV context ending at 8192"),
    "phi3_mini": dict(cfg=PHI3_MINI, batch=16, max_ctx=4096, start=2048, max_gpus=2,
                      workload="phi3-mini-shape decode, bf16, batch 16, 2048-token context then K steps (cache 4096)"),
}
METRIC = "decode_tokens_per_sec"


def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return dict(hbm=float(p["hbm_gbs"]), tf_burst=float(p["bf16_tflops"]),
                    tf_sustained=float(p["bf16_tflops_sustained"]), kind="measured")
    except Exception:
        return dict(hbm=6650.0, tf_burst=1590.0, tf_sustained=1400.0, kind="fallback")


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


class Dist:
    """torch.distributed plumbing of one bench process (a no-op at N = 1)."""

    def __init__(self, gpus):
        import torch
        self.torch = torch
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != gpus:
            raise SystemExit(f"--gpus {gpus} but WORLD_SIZE={self.world}: launch with torch.distributed.run")
        torch.cuda.set_device(self.local)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
            self.dist = dist

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.dist is not None:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, value):
        t = self.torch.tensor([float(value)], device="cuda")
        if self.dist is not None:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def close(self):
        if self.dist is not None:
            self.dist.barrier()
            self.dist.destroy_process_group()


def timed_regions(D, stream, repeats, prepare, run):
    """`repeats` regions, each bracketed by barrier + synchronise on both sides and timed with CUDA
    events on the launching stream; the time of a region is the maximum over ranks.  Returns the
    sorted list of region times in ms."""
    torch = D.torch
    out = []
    for r in range(repeats):
        prepare(r)
        D.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        run()
        e1.record(stream)
        D.barrier()
        out.append(D.max_over_ranks(e0.elapsed_time(e1)))
    return sorted(out)


def median(xs):
    return xs[len(xs) // 2]


# -------------------------------------------------------------------------------------------------
# CPU baseline: the oracle (reference semantics, float32, per-op materialisation, one BLAS call
# per batch slice as src/Execution.jl:21-29 does) on the host cores, bounded sample.  Test
# infrastructure used as the checker / the baseline leg only: nothing of it is on the GPU path.
# -------------------------------------------------------------------------------------------------
def blas_threads():
    try:
        from threadpoolctl import threadpool_info
        return max([int(i.get("num_threads", 1)) for i in threadpool_info() if i.get("user_api") == "blas"] or [1])
    except Exception:
        return None


def cpu_baseline(name="llama3_8b", layers=2, steps=1, ctx=None):
    """Decode steps of `layers` full-width layers at the workload's real context length (the KV cache of
    two float32 layers fits in host memory) plus 1/8 of the head; the step time of the whole model is
    that extrapolated linearly over layers and vocabulary -- nothing else is scaled."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import luminal_oracle as O
    try:
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=N_CORES)
    except Exception:
        pass
    wl = DECODE[name]
    full, batch = wl["cfg"], wl["batch"]
    if ctx is None:
        ctx = wl["max_ctx"] - 256 if wl["start"] is None else wl["start"] + 128       # the mean context of the timed steps
    cfg = dict(full, n_layers=layers)
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
    vslice = cfg["vocab"] // 8
    w["model.embed_tokens.weight"] = rnd(vslice, hid)
    w["model.norm.weight"] = np.ones(hid, np.float32)
    w["lm_head.weight"] = rnd(vslice, hid)
    cfg_s = dict(cfg, vocab=vslice)
    model = O.CachedLlama(w, cfg_s, batch, ctx + steps + 2)
    block = rng.standard_normal((1, 1, 1, 64, D), dtype=np.float32)      # the values do not change the timing
    model.k[:, :, :, :ctx] = np.tile(block, (1, 1, 1, (ctx + 63) // 64, 1))[:, :, :, :ctx]
    model.v[:, :, :, :ctx] = np.tile(block, (1, 1, 1, (ctx + 63) // 64, 1))[:, :, :, :ctx]
    model.pos = ctx
    toks = rng.integers(0, vslice, size=(batch, 1))
    model.forward(toks)                      # warm-up (BLAS threads, page faults)
    x = rnd(batch, 1, hid)
    t0 = time.perf_counter()
    O.linear(O.rms_norm(x, w["model.norm.weight"], cfg["eps"]), w["lm_head.weight"])
    t_head_slice = time.perf_counter() - t0
    t0 = time.perf_counter()
    for _ in range(steps):
        model.forward(toks)
    t_sample = time.perf_counter() - t0
    t_step = t_sample / steps
    t_layer = max(t_step - t_head_slice, 1e-9) / layers
    t_full = t_layer * full["n_layers"] + t_head_slice * 8
    return {"value": batch / t_full, "unit": "tokens/s", "cores": N_CORES, "blas_threads": blas_threads(), "kind": "port",
            "sample": (f"oracle, float32, batch {batch}, {layers} full-width layers x {steps} decode step(s) at context {ctx} "
                       f"+ 1/8 of the head; extrapolated linearly over layers ({layers} -> {full['n_layers']}) and "
                       f"vocabulary (1/8 -> 1) only"),
            "sample_seconds": t_sample, "ms_per_step_extrapolated": t_full * 1e3}


def run_reference_small_llama(args):
    """configs[0], the reference's own CPU-runnable case, with nothing extrapolated: the oracle runs the whole job the
    way the reference's generation loop does -- no KV cache for Llama, the whole prefix re-run for every token
    (examples/llama.jl:39-99) -- and, beside it, the cached form of the same function the GPU session is compared with."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import luminal_oracle as O
    try:
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=N_CORES)
    except Exception:
        pass
    cfg = O.CONFIGS["small_llama"]
    w = O.synth_llama_weights(cfg, seed=1234)
    gold = np.load(os.path.join(ROOT, "tests", "golden", "small_llama_golden.npz"))
    prompt, steps = gold["prompt"], 64
    recompute, cached, toks = [], [], None
    for r in range(1 + max(1, min(args.steps, 3))):            # the first pass warms BLAS up and is not counted
        t0 = time.perf_counter()
        toks, _ = O.greedy_generate_recompute(prompt, w, cfg, steps)
        t1 = time.perf_counter()
        toks_c, _ = O.CachedLlama(w, cfg, 1, 128).greedy(prompt, steps)
        t2 = time.perf_counter()
        if r:
            recompute.append((t1 - t0) * 1e3)
            cached.append((t2 - t1) * 1e3)
    ms, ms_c = median(sorted(recompute)), median(sorted(cached))
    identical = bool(np.array_equal(toks, gold["tokens"]) and np.array_equal(toks_c, gold["tokens"]))
    val = steps / (ms * 1e-3)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "tokens/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": 1, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "small llama (4 layers, hidden 256, 8 heads x 32, MLP 688, vocab 1024), float32, batch 1, "
                               "32-token prompt + 64 greedy steps; the time includes the prompt", "name": "small_llama",
                   "note": "CPU oracle port run as the reference generates: the whole prefix re-run per token, no KV cache"},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": N_CORES, "kind": "port",
                         "sample": "the whole job, nothing extrapolated", "sample_seconds": ms * 1e-3,
                         "with_kv_cache_tokens_per_s": steps / (ms_c * 1e-3)},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "parity": {"tokens_identical_to_golden": identical},
    }))
    if not identical:
        raise SystemExit(3)


def run_reference(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    if args.config == "small_llama":
        return run_reference_small_llama(args)
    name = args.config if args.config in DECODE else "llama3_8b"
    wl = DECODE[name]
    samples, base = [], None
    for _ in range(max(1, min(args.steps, 3))):
        base = cpu_baseline(name, layers=2, steps=1)
        samples.append(base["ms_per_step_extrapolated"])
    ms = median(sorted(samples))
    val = wl["batch"] / (ms / 1e3)
    base = dict(base, value=val)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl["workload"], "batch": wl["batch"],
                   "note": "CPU oracle port of the reference path; ms_per_step is the extrapolated whole-model step, "
                           "cpu_baseline.sample_seconds what was actually timed"},
        "cpu_baseline": base,
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# -------------------------------------------------------------------------------------------------
# tensor-parallel parity, outside the timed region: a small model across the N ranks against the oracle
# -------------------------------------------------------------------------------------------------
def tp_parity(L, dev, D):
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import luminal_oracle as O
    name = "mid_gqa_kv8"
    cfg = O.CONFIGS[name]
    w = O.synth_llama_weights(cfg, seed=31)
    B, P, steps = 3, 6, 5
    prompt = O.synth_tokens(31, 1000, (B, P), cfg["vocab"])
    ref_tok, ref_log = O.CachedLlama(w, cfg, B, 32).greedy(prompt, steps)
    _, ref_hidden = O.CachedLlama(w, cfg, B, 32).forward(prompt, return_hidden=True)
    out = {"config": name, "ranks": D.world}
    blobs = []
    for dtype in ("f32", "bf16"):
        model = L.Model(dev, n_layers=cfg["n_layers"], hidden=cfg["hidden"], n_heads=cfg["n_heads"],
                        n_kv_heads=cfg["n_kv_heads"], intermediate=cfg["intermediate"], vocab=cfg["vocab"],
                        eps=cfg["eps"], rope_base=cfg["rope_base"], dtype=dtype, tp_size=D.world, tp_rank=D.rank)
        model.set_weights(w)
        sess = L.Session(model, B, 32)
        if dtype == "f32":
            tok, log = L.greedy_generate(sess, prompt, steps, want_logits=True)
            out["tokens_identical"] = bool(np.array_equal(tok, ref_tok))
            out["logits_max_abs_err"] = float(np.abs(log - ref_log).max())
            blobs.append(tok.tobytes() + log.tobytes())
        else:
            sess.set_capture(True)
            sess.prefill(prompt)
            err = 0.0
            for l in range(cfg["n_layers"]):
                got, ref = sess.layer_output(l).astype(np.float64), ref_hidden[l][:, -1, :].astype(np.float64)
                err = max(err, float(np.linalg.norm(got - ref) / np.linalg.norm(ref)))
                blobs.append(got.tobytes())
            out["bf16_layer_rel_err"] = err
        sess.close(); model.close()
    gathered = [None] * D.world
    D.dist.all_gather_object(gathered, b"".join(blobs))
    out["ranks_agree"] = all(g == gathered[0] for g in gathered)
    out["ok"] = bool(out["tokens_identical"] and out["logits_max_abs_err"] <= 1e-3 and out["bf16_layer_rel_err"] <= 2e-2
                     and out["ranks_agree"])
    return out


# -------------------------------------------------------------------------------------------------
# decode workloads (llama3_8b, phi3_mini)
# -------------------------------------------------------------------------------------------------
def attention_traffic(KVl, T, batch, D):
    """dram bytes of one decode-attention launch, from the tracked ncu capture scaled by the keys and
    kv heads of this launch (DRAM traffic of this kernel grows in proportion to the cache it reads)."""
    try:
        with open(os.path.join(ROOT, "profiles", "attn_decode_bf16_traffic.json")) as f:
            cap = json.load(f)
        units = cap["batch"] * cap["kv_heads"] * cap["keys"] * cap["head_dim"]
        return int(cap["dram_bytes_per_launch"] * (batch * KVl * T * D) / units), cap["source"]
    except Exception:
        return None, None


def run_decode(args):
    import torch
    import luminal_jl_b200 as L
    wl = DECODE[args.config]
    CFG, BATCH, MAX_CTX = wl["cfg"], args.batch or wl["batch"], wl["max_ctx"]
    if args.gpus > wl["max_gpus"]:
        raise SystemExit(f"--config {args.config} shards over at most {wl['max_gpus']} GPUs")
    D = Dist(args.gpus)
    world, rank, local = D.world, D.rank, D.local
    steps = args.steps
    warm = max(args.warmup, 3, 20 if world > 1 else 3)       # after comm_init the first replays are slower
    if wl["start"] is None:
        if steps + warm > MAX_CTX - 1:
            raise SystemExit(f"steps + warmup exceed the {MAX_CTX}-token context")
        ctx_start = MAX_CTX - steps            # the timed steps end exactly at the capacity
        warm_start = ctx_start - warm
    else:
        if wl["start"] + steps > MAX_CTX:
            raise SystemExit(f"{wl['start']} + steps exceed the {MAX_CTX}-token cache")
        ctx_start = wl["start"]
        warm_start = ctx_start - warm

    stream = torch.cuda.Stream()
    dev = L.B200Device(local, stream=stream.cuda_stream)
    parity = None
    if world > 1:
        uid = [L.B200Device.comm_unique_id() if rank == 0 else None]
        D.dist.broadcast_object_list(uid, src=0)
        dev.comm_init(world, rank, uid[0])
        parity = tp_parity(L, dev, D)
        if not parity["ok"]:
            if rank == 0:
                print(json.dumps({"error": "tensor-parallel parity check failed", "tp_parity": parity}))
            raise SystemExit(3)
    cfg = dict(CFG, n_layers=args.layers or CFG["n_layers"])
    tp_size = world
    if args.solo_shard > 1 and world == 1:
        os.environ["LMB200_TP_SOLO"] = "1"
        tp_size = args.solo_shard
    model = L.Model(dev, dtype="bf16", tp_size=tp_size, tp_rank=rank, **cfg)
    model.init_random(1234, 0.02)
    sess = L.Session(model, BATCH, MAX_CTX)
    sess.fill_kv_random(warm_start, seed=1234)

    first = torch.randint(0, CFG["vocab"], (BATCH,), dtype=torch.int32, device="cuda",
                          generator=torch.Generator(device="cuda").manual_seed(1234))
    out_dev = torch.empty((max(steps, warm), BATCH), dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()

    # ---- device-resident loop -------------------------------------------------------------------
    with torch.cuda.stream(stream):
        sess.decode_n_device(first.data_ptr(), warm, out_dev.data_ptr())
        D.barrier()
        if world > 1:
            # every rank must have produced the same greedy tokens in the full-size warm-up steps
            mine = out_dev[:warm].clone()
            every = [torch.empty_like(mine) for _ in range(world)]
            D.dist.all_gather(every, mine)
            parity["full_size_ranks_agree"] = all(bool(torch.equal(e, every[0])) for e in every)
            if not parity["full_size_ranks_agree"]:
                if rank == 0:
                    print(json.dumps({"error": "ranks produced different tokens at full size", "tp_parity": parity}))
                raise SystemExit(3)
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        launches0 = [0]

        def prep(_r):
            sess.set_position(ctx_start)
            launches0[0] = dev.launch_count()

        regions = timed_regions(D, stream, args.repeats, prep,
                                lambda: sess.decode_n_device(first.data_ptr(), steps, out_dev.data_ptr()))
        launches = dev.launch_count() - launches0[0]
        clocks = sampler.stop() if rank == 0 else None
    ms_total = median(regions)

    # ---- end to end through the host-buffer call ------------------------------------------------
    tok_in = torch.randint(0, CFG["vocab"], (BATCH,), dtype=torch.int32,
                           generator=torch.Generator().manual_seed(1234)).pin_memory()      # the same ids on every rank
    tok_out = torch.empty(BATCH, dtype=torch.int32).pin_memory()

    def e2e_run():
        for _ in range(steps):
            sess.decode_step_raw(tok_in.data_ptr(), tok_out.data_ptr())
            tok_in.copy_(tok_out)                      # the result feeds the next step, on the host

    def e2e_prep(_r):
        sess.set_position(ctx_start - 3)
        for _ in range(3):
            sess.decode_step_raw(tok_in.data_ptr(), tok_out.data_ptr())
            tok_in.copy_(tok_out)

    with torch.cuda.stream(stream):
        e2e_regions = timed_regions(D, stream, min(args.repeats, 3), e2e_prep, e2e_run)
    e2e_ms = median(e2e_regions)

    # ---- dominant kernel alone: split-KV decode attention, one launch per layer ------------------
    peaks = load_peaks()
    T_mid = ctx_start + steps // 2
    Hl = CFG["n_heads"] // tp_size
    KVl = CFG["n_kv_heads"] // tp_size
    Dh = CFG["hidden"] // CFG["n_heads"]
    q = torch.randn(BATCH, Hl * Dh, device="cuda").to(torch.bfloat16)
    o = torch.empty_like(q)
    attn_bytes = BATCH * KVl * T_mid * Dh * 2 * 2 + 2 * q.numel() * 2     # K and V read once, q in, out
    with torch.cuda.stream(stream):
        for l in range(min(3, cfg["n_layers"])):
            sess.decode_attention(l, q.data_ptr(), o.data_ptr(), T_mid)

        def attn_run():
            for l in range(cfg["n_layers"]):
                sess.decode_attention(l, q.data_ptr(), o.data_ptr(), T_mid)
        attn_regions = timed_regions(D, stream, 3, lambda _r: None, attn_run)
    attn_ms = median(attn_regions) / cfg["n_layers"]

    if rank == 0:
        tokens = BATCH * steps
        T_avg = ctx_start + (steps - 1) / 2.0 + 1
        step_bytes = sess.step_bytes(int(round(T_avg)))
        step_gbs = step_bytes / (ms_total / steps * 1e-3) / 1e9
        attn_gbs = attn_bytes / (attn_ms * 1e-3) / 1e9
        traffic, traffic_src = attention_traffic(KVl, T_mid, BATCH, Dh)
        line = {
            "metric": METRIC, "value": tokens / (ms_total * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": steps, "warmup": warm, "ms_per_step": ms_total / steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "repeats": {"n": len(regions), "statistic": "median", "min_ms_per_step": regions[0] / steps,
                        "max_ms_per_step": regions[-1] / steps},
            "config": {"workload": wl["workload"], "name": args.config, "batch": BATCH,
                       "context": [ctx_start, ctx_start + steps],
                       "layers": cfg["n_layers"], "parallelism": f"tp{world}" if tp_size == world else f"rank 0 of tp{tp_size} alone (profiling)",
                       "l2": "inputs larger than L2: every step streams this rank's weights and KV cache "
                             f"({step_bytes / 1e9:.1f} GB) once"},
            "e2e": {"value": BATCH * steps / (e2e_ms * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": BATCH * 4, "d2h_bytes_per_step": BATCH * 4, "ms_per_step": e2e_ms / steps},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": {"kernel": f"attn_decode_bf16_kernel<{Dh}> (per layer; the last CTA of each sequence and kv head merges the splits)",
                         "bound": "hbm", "achieved": attn_gbs, "peak": peaks["hbm"], "unit": "GB/s",
                         "frac": attn_gbs / peaks["hbm"], "peak_kind": peaks["kind"],
                         "traffic": traffic, "traffic_source": traffic_src,
                         "bytes_per_launch": attn_bytes, "ms_per_launch": attn_ms},
            "step_hbm": {"bytes_per_step_per_gpu": step_bytes, "achieved": step_gbs, "peak": peaks["hbm"], "unit": "GB/s",
                         "frac": step_gbs / peaks["hbm"]},
        }
        if parity is not None:
            line["tp_parity"] = parity
            # what the 2 x layers reductions of a step move over NVLink, per GPU and direction.  Fused step: every rank
            # stores its bf16 partial [hidden][32] into each of the N - 1 peers' regions; separate norm kernels
            # (LMB200_FUSED_STEP=0): every rank loads the N - 1 peers' float32 partials [32][hidden]
            fused = os.environ.get("LMB200_FUSED_STEP", "1") != "0"
            line["nvlink"] = {"reductions_per_step": 2 * cfg["n_layers"],
                              "bytes_per_step_per_gpu": 2 * cfg["n_layers"] * (world - 1) * CFG["hidden"] * 32 * (2 if fused else 4),
                              "protocol": ("peer stores of bf16 partials + data polling inside the o_proj / down_proj kernels" if fused
                                           else "flag + peer loads of float32 partials inside the norm kernels")}
        if args.prefill:
            line["prefill"] = None
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline(args.config)
        else:
            line["cpu_baseline"] = None
    if args.prefill and wl["start"] is not None:
        # the prompt phase of this configuration, timed separately: batch x start tokens through the GEMM path
        P = wl["start"]
        prompt = torch.randint(0, CFG["vocab"], (BATCH, P), dtype=torch.int32).numpy()
        sess.reset()
        sess.prefill(prompt, want_logits=False)
        times = []
        for _ in range(3):
            sess.reset()
            D.barrier()
            t0 = time.perf_counter()
            sess.prefill(prompt, want_logits=False)
            D.barrier()
            times.append(D.max_over_ranks(time.perf_counter() - t0))
        if rank == 0:
            t = median(sorted(times))
            per_tok = 2 * (model_params(cfg) - cfg["vocab"] * cfg["hidden"] * 2) + 4 * cfg["n_layers"] * cfg["hidden"] * (P / 2.0)
            flop = per_tok * BATCH * P
            line["prefill"] = {"tokens": BATCH * P, "seconds": t, "tokens_per_sec": BATCH * P / t,
                               "tflops": flop / t / 1e12, "frac_of_sustained_bf16": flop / t / 1e12 / peaks["tf_sustained"] / world,
                               "timing": "wall clock around lmb200_prefill (host token upload and the last position's head included)"}
    if rank == 0:
        print(json.dumps(line))
    sess.close()
    model.close()
    if world > 1:
        D.dist.barrier()
        dev.comm_destroy()
    D.close()


def model_params(cfg):
    hid, inter, H, KV = cfg["hidden"], cfg["intermediate"], cfg["n_heads"], cfg["n_kv_heads"]
    Dh = hid // H
    per_layer = hid * hid + 2 * KV * Dh * hid + hid * hid + 3 * inter * hid
    return per_layer * cfg["n_layers"] + 2 * cfg["vocab"] * hid


# -------------------------------------------------------------------------------------------------
# small_llama: BASELINE configs[0], float32, batch 1, 32-token prompt + 64 greedy steps
# -------------------------------------------------------------------------------------------------
def run_small_llama(args):
    import numpy as np
    import torch
    import luminal_jl_b200 as L
    D = Dist(1)
    stream = torch.cuda.Stream()
    dev = L.B200Device(0, stream=stream.cuda_stream)
    cfg = SMALL_LLAMA
    model = L.Model(dev, dtype="f32", **cfg)
    model.init_random(1234, 0.02)
    sess = L.Session(model, 1, 128)
    gold = np.load(os.path.join(ROOT, "tests", "golden", "small_llama_golden.npz"))
    prompt = gold["prompt"].astype(np.int32)
    steps = 64

    def run():
        logits = sess.prefill(prompt)
        first = logits.argmax(-1).astype(np.int32)
        rest = sess.decode_n(first, steps - 1)
        return np.concatenate([first[None, :], rest], 0).T

    with torch.cuda.stream(stream):
        for _ in range(3):
            sess.reset()
            toks = run()
        launches0 = [0]

        def prep(_r):
            sess.reset()
            launches0[0] = dev.launch_count()
        regions = timed_regions(D, stream, args.repeats, prep, run)
        launches = dev.launch_count() - launches0[0]
    ms = median(regions)
    identical = bool(np.array_equal(toks, gold["tokens"]))
    print(json.dumps({
        "metric": METRIC, "value": steps / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": 3,
        "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "repeats": {"n": len(regions), "statistic": "median", "min_ms": regions[0], "max_ms": regions[-1]},
        "config": {"workload": "small llama (4 layers, hidden 256, 8 heads x 32, MLP 688, vocab 1024), float32, batch 1, "
                               "32-token prompt + 64 greedy steps; the time includes the prompt", "name": "small_llama",
                   "l2": "the model (13.7 MB) is L2-resident by nature of the configuration: launch-bound"},
        "e2e": {"value": steps / (ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4,
                "note": "the timed call takes the prompt from host memory and returns the tokens to it"},
        "gpu_launches": int(launches),
        "parity": {"tokens_identical_to_golden": identical},
        "roofline": None, "cpu_baseline": None,
    }))
    sess.close(); model.close()
    if not identical:
        raise SystemExit(3)


# -------------------------------------------------------------------------------------------------
# flash: FlashAttentionOp on [4, 32, 4096, 128], causal and non-causal, bf16 and float32 inputs
# -------------------------------------------------------------------------------------------------
def run_flash(args):
    import ctypes as C
    import torch
    import luminal_jl_b200 as L
    from importlib import import_module
    _lib = import_module("luminal_jl_b200._lib")
    D = Dist(1)
    stream = torch.cuda.Stream()
    dev = L.B200Device(0, stream=stream.cuda_stream)
    B, H, S, Dh = 4, 32, 4096, 128
    peaks = load_peaks()
    gen = torch.Generator(device="cuda").manual_seed(7)
    variants = {}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")      # larger than L2
    for dtype, tdt, code in (("bf16", torch.bfloat16, _lib.BF16), ("f32", torch.float32, _lib.F32)):
        q, k, v = (torch.randn((B, H, S, Dh), device="cuda", generator=gen).to(tdt) for _ in range(3))
        out = torch.empty_like(q)
        for causal in (False, True):
            def run():
                _lib.call("lmb200_flash_attention", dev.handle, C.c_void_p(out.data_ptr()), C.c_void_p(q.data_ptr()),
                          C.c_void_p(k.data_ptr()), C.c_void_p(v.data_ptr()), code, B, H, S, Dh, 1.0 / Dh ** 0.5, int(causal))
            with torch.cuda.stream(stream):
                for _ in range(3):
                    run()
                regions = timed_regions(D, stream, max(args.repeats, 5), lambda _r: flush.fill_(1), run)
            ms = median(regions)
            flop = 4.0 * B * H * Dh * (S * (S + 1) / 2 if causal else S * S)
            variants[f"{dtype}_{'causal' if causal else 'full'}"] = {
                "ms": ms, "tflops": flop / ms / 1e9, "frac_of_burst_bf16": flop / ms / 1e9 / peaks["tf_burst"],
                "min_ms": regions[0], "max_ms": regions[-1]}
    head = variants["bf16_full"]
    print(json.dumps({
        "metric": "flash_attention_tflops", "value": head["tflops"], "unit": "TFLOP/s", "n_gpus": 1, "steps": 1, "warmup": 3,
        "ms_per_step": head["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": "FlashAttentionOp, Q/K/V [4, 32, 4096, 128] ~N(0,1), scale 1/sqrt(128); value = bf16 non-causal",
                   "name": "flash", "l2": "a 256 MB buffer is written between timed launches"},
        "variants": variants,
        "roofline": {"kernel": "flash_tc_kernel<128>", "bound": "tensor", "achieved": head["tflops"], "peak": peaks["tf_burst"],
                     "unit": "TFLOP/s", "frac": head["tflops"] / peaks["tf_burst"], "peak_kind": peaks["kind"] + " (burst)",
                     "traffic": None},
        "e2e": None, "gpu_launches": 1, "cpu_baseline": None,
    }))


# -------------------------------------------------------------------------------------------------
# whisper_base: encoder + cross K/V + 128 greedy steps, batch 8, bf16, random weights
# -------------------------------------------------------------------------------------------------
def run_whisper(args):
    import numpy as np
    import torch
    import luminal_jl_b200 as L
    D = Dist(1)
    stream = torch.cuda.Stream()
    dev = L.B200Device(0, stream=stream.cuda_stream)
    cfg, batch, frames, steps = WHISPER_BASE, 8, 3000, 128
    rng = np.random.default_rng(17)
    w = {}
    for name, shape in sorted(L.whisper.registry_shapes(**cfg).items()):
        a = rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)
        w[name] = a + np.float32(1.0) if name.endswith("layer_norm.weight") else a
    mel = rng.standard_normal((batch, cfg["n_mels"], frames), dtype=np.float32)
    enc = L.whisper.FusedEncoder(dev, d_model=cfg["d_model"], heads=cfg["heads"], enc_layers=cfg["enc_layers"],
                                 dec_layers=cfg["dec_layers"], ffn=cfg["ffn"], n_mels=cfg["n_mels"])
    enc.set_weights(w)
    T = (frames - 1) // 2 + 1
    model = L.WhisperDecoderModel(dev, d_model=cfg["d_model"], heads=cfg["heads"], layers=cfg["dec_layers"], ffn=cfg["ffn"],
                                  vocab=cfg["vocab"], max_positions=cfg["max_positions"], cross_len=T, dtype="bf16")
    for name, a in w.items():
        if name.startswith("model.decoder."):
            model.set_weight(name, a)
    sess = L.Session(model, batch, cfg["max_positions"])
    first = np.full(batch, 50258, dtype=np.int32)          # a start-of-transcript id (sot_sequence, src/Decoding.jl:86)

    def pipeline():
        enc.run(mel, want_output=False)
        enc.cross_kv_into(sess)
        sess.reset()
        return sess.decode_n(first, steps)

    def decode_only():
        sess.reset()
        return sess.decode_n(first, steps)

    with torch.cuda.stream(stream):
        for _ in range(3):
            toks = pipeline()
        launches0 = [0]

        def prep(_r):
            launches0[0] = dev.launch_count()
        whole = timed_regions(D, stream, args.repeats, prep, pipeline)
        launches = dev.launch_count() - launches0[0]
        dec = timed_regions(D, stream, args.repeats, lambda _r: None, decode_only)
    ms_whole, ms_dec = median(whole), median(dec)
    distinct = int(len(np.unique(toks)))
    print(json.dumps({
        "metric": METRIC, "value": batch * steps / (ms_dec * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": 3,
        "ms_per_step": ms_dec / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "repeats": {"n": len(dec), "statistic": "median", "min_ms_per_step": dec[0] / steps, "max_ms_per_step": dec[-1] / steps},
        "config": {"workload": "whisper-base shape (d_model 512, 8 heads, 6 + 6 layers, FFN 2048, vocab 51865), bf16, random "
                               "weights ~N(0, 0.02), mel [8, 80, 3000] ~N(0,1): encoder + cross K/V projection + 128 greedy steps",
                   "name": "whisper_base", "batch": batch,
                   "l2": "decoder weights (97 MB) and cross K/V (147 MB) exceed L2 together; the step is launch-bound"},
        "e2e": {"value": batch * steps / (ms_whole * 1e-3), "unit": "tokens/s", "ms_whole_pipeline": ms_whole,
                "ms_encoder_and_cross_kv": ms_whole - ms_dec, "h2d_bytes_per_step": int(mel.nbytes / steps),
                "d2h_bytes_per_step": batch * 4,
                "note": "one call chain mel (host) -> encoder -> cross K/V -> 128 greedy steps -> tokens (host)"},
        "gpu_launches": int(launches), "distinct_tokens": distinct,
        "roofline": None, "cpu_baseline": None,
    }))
    sess.close(); model.close(); enc.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="llama3_8b", choices=["llama3_8b", "phi3_mini", "whisper_base", "small_llama", "flash"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--repeats", type=int, default=5, help="timed regions of --steps steps; the median is reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--prefill", action="store_true", help="phi3_mini: also time the 2048-token prompt phase")
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers (invalid as a result)")
    ap.add_argument("--batch", type=int, default=0, help="debug only: another batch size (invalid as a result)")
    ap.add_argument("--solo-shard", type=int, default=0,
                    help="profiling only: run rank 0's shard of an N-way tensor-parallel model alone on one GPU, without the "
                         "exchange (kernel sizes are the rank's, the results are not the model's; invalid as a result)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.config in DECODE:
        run_decode(args)
    elif args.config == "small_llama":
        run_small_llama(args)
    elif args.config == "flash":
        run_flash(args)
    else:
        run_whisper(args)


if __name__ == "__main__":
    main()
