"""Benchmark of the quantised scoring hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python bench.py --case NAME      # one small, self-terminating workload of a hot kernel, for an ncu capture

Workload (N = 1): the Llama-style scoring configuration - 12 layers, d_model 768, 12 query / 4 KV
heads, SwiGLU 2048, vocab 32000, Q4_0 weights drawn from N(0, 0.02) - scoring 256 sequences of 1024
uniform-random token ids for their total log-probability (fp16 tensor-core path, f32 accumulation). One step = one pass
over the 256 sequences of a rank. With N > 1 every rank holds a replica and scores its own 256
sequences (no data-path collective); the per-sequence NLL sums are all-gathered at the end of each step
(`value`, weak scaling). The same line then carries `strong` (the 256 sequences of the configuration shared
out over the N ranks) and `c5` (the GPT-2-124M configuration, 512 x 1024, through the multi-GPU group of the
C ABI with the head split over 2 and 4 vocabulary shards, beside the replicated head on the same sequences).
At N = 1 it also carries `decode` (batch-1 greedy decode of the GPT-2-style configuration), `decode64` (the
64-stream Qwen2-style decode) and `sweep` (the isolated quantised product over the whole shape grid).
Everything is synthetic: there is no dataset and no checkpoint.

Prints ONE JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_SEQS, SEQ_LEN = 256, 1024
METRIC, UNIT = "scoring tok/s", "scored tokens/s"


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the largest product (gate/up with the
# SwiGLU epilogue, M = 131072 rows, K = 768, N = 4096) from an ncu capture of a quarter-size launch
# (32 x 1024 rows: 52.2 MB read + 80.3 MB written), scaled by 4; see profiles/.
NCU_TRAFFIC_BYTES = 4 * (52.16e6 + 80.28e6)
NCU_TRAFFIC_NOTE = ("gate/up product, per launch; algorithmic bytes are 740 MB (201 MB f16 rows in, 537 MB f16 out, "
                    "1.8 MB weights) - part of the output is still in L2 when the launch ends")

def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], d.get("bf16_tflops_sustained", d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "200"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])), mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def c3_flops_per_token(cfg) -> float:
    """2 * matrix parameters + causal attention (4 * heads * head_dim * (t + 1) / 2 per layer)."""
    mats = cfg.layers * (cfg.dim * (cfg.q_dim + 2 * cfg.kv_dim) + cfg.q_dim * cfg.dim + 3 * cfg.dim * cfg.hidden)
    mats += cfg.dim * cfg.vocab
    return 2.0 * mats, 4.0 * cfg.heads * cfg.head_dim * (SEQ_LEN / 2.0) * cfg.layers


def run_reference(args, rank: int):
    """The reference's own CPU path for this workload, restated (no Rust toolchain exists here): the f32 oracle
    over the dequantised weights on the reference's tuned kernel (`matmul_tuned`, ferrum_ref/src/kernels/tuned.rs:
    cache panels, a 4 x 8 register tile, rows split over all host threads - "the speed baseline for GPU gates",
    bit-identical to the simple kernel), on a bounded sample per step."""
    if rank != 0:
        return
    from ferrum_gpu_b200 import _ffi
    from ferrum_gpu_b200.hostmodel import config_c3, random_llama, random_tokens
    from oracle import oracle as orc
    cores = os.cpu_count() or 1
    cfg = config_c3()
    model = random_llama(cfg, seed=1)
    ref = orc.dequantised_llama(model, _ffi.FC_Q4_0, snap_embedding=False)
    orc.set_tuned(True)
    oracle = orc.OracleLlama(ref, threads=cores)
    sample_len = 257
    ids = random_tokens(100, sample_len, cfg.vocab)
    for _ in range(min(args.warmup, 1)):
        oracle.score(ids)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.score(ids)
    dt = (time.perf_counter() - t0) / args.steps
    value = (sample_len - 1) / dt
    sample = f"1 sequence x {sample_len} tokens per step (of 256 x 1024), f32 oracle on the tuned kernel, {cores} threads"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": min(args.warmup, 1), "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "c3-llama-12L-d768-q4_0-scoring-256x1024", "sample": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--seqs", type=int, default=N_SEQS, help="sequences per rank (256 = the benchmark workload)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sweep", action="store_true", help="skip the isolated-product shape grid (about a minute)")
    ap.add_argument("--no-c5", action="store_true", help="skip the split-head GPT-2-124M leg of a multi-GPU run")
    ap.add_argument("--case", default=None, help="run one profiling case and exit: " + ", ".join(sorted(CASES)))
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--decode64", action="store_true", help="(default now; kept so that older command lines still parse)")
    ap.add_argument("--no-decode64", action="store_true",
                    help="skip the 64-stream Qwen2-style decode configuration (about 15 s of set-up and prefill)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.case:
        run_case(args.case)
        return

    import torch
    import torch.distributed as dist
    from ferrum_gpu_b200 import CudaGpt2, CudaLlama, Device, Mode, QKind
    from ferrum_gpu_b200.hostmodel import config_c1, config_c3, random_gpt2, random_llama, random_tokens

    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = Device.open(local)
    stream = torch.cuda.ExternalStream(dev.stream(), device=local)
    hbm, tf_burst, tf_sust, peak_src = peaks()

    cfg = config_c3()
    model = random_llama(cfg, seed=1)          # every rank holds the same replica
    g = CudaLlama(dev, model, QKind.Q4_0)
    n_seqs = args.seqs
    ids_host = np.stack([random_tokens(1000 + rank * 100000 + i, SEQ_LEN, cfg.vocab) for i in range(n_seqs)])
    rows = n_seqs * (SEQ_LEN - 1)

    with torch.cuda.stream(stream):
        ids_dev = torch.from_numpy(ids_host).to(f"cuda:{local}", non_blocking=False)
        nll_dev = torch.zeros(n_seqs, dtype=torch.float64, device=f"cuda:{local}")
        gathered = torch.zeros(world * n_seqs, dtype=torch.float64, device=f"cuda:{local}") if world > 1 else None

        def step():
            g.score_dev(ids_dev.data_ptr(), n_seqs, SEQ_LEN, Mode.TENSOR_F16, 0, 0, nll_dev.data_ptr())
            if world > 1:
                dist.all_gather_into_tensor(gathered, nll_dev)

        for _ in range(max(args.warmup, 3)):
            step()
        stream.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        l0 = dev.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            step()
        e1.record(stream)
        stream.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ms = e0.elapsed_time(e1)
        launches = dev.launch_count() - l0
        clocks = sampler.stop() if rank == 0 else None
        tms = torch.tensor([ms], dtype=torch.float64, device=f"cuda:{local}")
        if world > 1:
            dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms_step = float(tms.item()) / args.steps
        nll_total = float(nll_dev.sum().item())

    # end to end through the public API with host buffers: ids go up, log-probs / flags / sums come back
    # (fc_model_score, the call `score_batch` makes), from and to pinned host memory
    from ferrum_gpu_b200 import _ffi
    lib = _ffi.load()
    ids_pin = torch.from_numpy(ids_host).pin_memory()
    lp = torch.empty(n_seqs, SEQ_LEN - 1, dtype=torch.float32).pin_memory()
    gr = torch.empty(n_seqs, SEQ_LEN - 1, dtype=torch.uint8).pin_memory()
    nll = torch.empty(n_seqs, dtype=torch.float64).pin_memory()

    def e2e_step():
        dev.check(lib.fc_model_score(g._h, ids_pin.data_ptr(), n_seqs, SEQ_LEN, int(Mode.TENSOR_F16), lp.data_ptr(),
                                     gr.data_ptr(), nll.data_ptr()))

    for _ in range(2):  # the first calls size the library's workspace and pinned staging
        e2e_step()
    e2e_steps = max(1, args.steps)
    step_s = []
    for _ in range(e2e_steps):  # each call returns after its results are in host memory
        t0 = time.perf_counter()
        e2e_step()
        step_s.append(time.perf_counter() - t0)
    e2e_s = sorted(step_s)[len(step_s) // 2]  # the median: one host hiccup in five calls is not the rate
    assert abs(float(nll.sum()) - nll_total) <= 1e-6 * abs(nll_total), "the host path and the device path disagree"
    te = torch.tensor([e2e_s], dtype=torch.float64, device=f"cuda:{local}")
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_s = float(te.item())

    strong = c5 = None
    if world > 1:
        strong = bench_strong(dev, g, stream, ids_host, world, rank, local, args)
        if not args.no_c5:
            c5 = bench_c5(world, rank, args)

    out = None
    if rank == 0:
        # per-kernel device time of one step (event pairs around every launch), for the roofline
        dev.profile(True)
        g.score_dev(ids_dev.data_ptr(), n_seqs, SEQ_LEN, Mode.TENSOR_F16, 0, 0, nll_dev.data_ptr())
        prof = dev.profile_report()
        dev.profile(False)
        total_ms = sum(v["ms"] for v in prof.values()) or 1.0
        gemm = {"launches": sum(v["launches"] for k, v in prof.items() if k.startswith("qgemm_tc")),
                "ms": sum(v["ms"] for k, v in prof.items() if k.startswith("qgemm_tc"))}
        lin_flops, attn_flops = c3_flops_per_token(cfg)
        gemm_flops_step = lin_flops * rows          # algorithmic: 2 * M * N * K summed over the products
        achieved = gemm_flops_step / (gemm["ms"] * 1e-3) / 1e12 if gemm["ms"] else 0.0
        # the same per role of the product (its epilogue names it): flops of that role / its device time
        role_flops = {"qgemm_tc_qkv": 2.0 * cfg.layers * cfg.dim * (cfg.q_dim + 2 * cfg.kv_dim),
                      "qgemm_tc_resid": 2.0 * cfg.layers * (cfg.q_dim * cfg.dim + cfg.hidden * cfg.dim),
                      "qgemm_tc_swiglu": 2.0 * cfg.layers * cfg.dim * 2 * cfg.hidden,
                      "qgemm_tc_lse": 2.0 * cfg.dim * cfg.vocab}
        by_role = {k: round(f * rows / (prof[k]["ms"] * 1e-3) / 1e12, 1) for k, f in role_flops.items()
                   if k in prof and prof[k]["ms"] > 0}
        attn_ms = sum(prof[k]["ms"] for k in ("attn_causal_tmem", "attn_causal_f16") if k in prof)
        attn_tf = attn_flops * rows / (attn_ms * 1e-3) / 1e12 if attn_ms > 0 else None
        shares = {k: round(v["ms"] / total_ms, 4) for k, v in sorted(prof.items(), key=lambda kv: -kv[1]["ms"])}
        out = {
            "metric": METRIC, "value": world * rows / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "c3-llama-12L-d768-q4_0-scoring-256x1024", "seqs_per_gpu": n_seqs, "seq_len": SEQ_LEN,
                       "weights": "Q4_0", "arithmetic": "fp16 operands on tcgen05 (kind::f16), f32 accumulate",
                       "l2": "inputs larger than L2 (activations of one chunk exceed 126 MB)", "parallelism": f"replica x{world}"},
            "e2e": {"value": world * rows / e2e_s, "unit": UNIT, "timing": "median of the per-step wall times", "h2d_bytes_per_step": int(ids_host.nbytes),
                    "d2h_bytes_per_step": int(lp.nbytes + rows + nll.nbytes)},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": {"bound": "tensor", "kernel": "qgemm_ts_kernel + qgemm_tc_kernel (the products of one step)", "achieved": achieved, "peak": tf_sust,
                         "unit": "TFLOP/s", "frac": achieved / tf_sust, "peak_source": f"{peak_src} (sustained bf16)",
                         "frac_of_burst": achieved / tf_burst, "traffic": NCU_TRAFFIC_BYTES,
                         "traffic_note": NCU_TRAFFIC_NOTE,
                         "launches_per_step": gemm["launches"], "ms_per_step": gemm["ms"], "kernel_shares": shares,
                         "tflops_by_role": by_role, "attention_tflops": attn_tf},
            "model_flops_per_step": (lin_flops + attn_flops) * rows,
            "mfu_of_sustained": (lin_flops + attn_flops) * rows / (ms_step * 1e-3) / 1e12 / tf_sust,
            "nll_checksum": nll_total,
        }
        if strong:
            out["strong"] = strong
        if c5:
            out["c5"] = c5
        if not args.no_decode and world == 1:
            time.sleep(3.0)  # a separate, latency-bound workload: let the clocks recover from the power-capped scoring steps
            dsamp = ClockSampler(local)
            dsamp.start()
            out["decode"] = bench_decode(dev, hbm)
            out["decode"]["clocks"] = dsamp.stop()
            if not args.no_decode64:
                out["decode64"] = bench_decode64(dev, hbm)
        if not args.no_sweep and world == 1:
            out["sweep"] = bench_sweep(dev, hbm, tf_burst)
        if not args.no_cpu_baseline and world == 1:
            out["cpu_baseline"] = cpu_baseline(cfg, model)
    g.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    dev.close()
    if rank == 0:
        print(json.dumps(out))


def bench_decode(dev, hbm_gbs):
    """KV-cached greedy decode, batch 1: the GPT-2-style configuration (6 layers, d_model 384, Q8_0),
    a 16-token prompt then 128 decoded tokens, timed as the reference does (the decoded tokens as a whole)."""
    from ferrum_gpu_b200 import CudaGpt2, QKind
    from ferrum_gpu_b200.hostmodel import config_c1, random_gpt2, random_tokens
    cfg = config_c1()
    m = CudaGpt2(dev, random_gpt2(cfg, seed=1), QKind.Q8_0)
    prompt = random_tokens(2, 16, cfg.vocab)
    best = None
    for _ in range(5):
        m.reset()
        tok = 0
        for t in prompt:
            tok = m.feed_greedy(int(t))
        t0 = time.perf_counter()
        m.decode_greedy([tok], 127)  # 127 chained greedy steps, one call (what `generate` does after the prompt)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    wbytes = m.weight_bytes()
    m.close()
    tok_s = 127 / best
    bytes_per_tok = wbytes + 2 * cfg.dim * 4 * 80 * cfg.layers  # weights + K/V read at mid-run length
    return {"workload": "c1-gpt2-6L-d384-q8_0-b1-16+128", "tok_s": tok_s, "ms_per_token": best / 127 * 1e3,
            "hbm_frac": bytes_per_tok * tok_s / 1e9 / hbm_gbs,
            "note": "weights (11 MB) live in L2; the limiter is launch/dependency latency, not HBM"}


def bench_decode64(dev, hbm_gbs, streams=64, prefill=1536, steps=512):
    """Batched KV-cached decode: the Qwen2-style configuration (24 layers, d_model 1024, 16 q / 2 kv heads,
    SwiGLU 2816, vocab 151936, tied head, q/k/v biases, Q8_0, f32 KV cache), 64 streams each with a
    1536-token prefill, then the configuration's 512 greedy steps of all streams together, chained on the
    device in one call (the cache grows from 1536 to 2048 positions, the step cost with it; the first and
    the last 32 steps are also timed on their own)."""
    from ferrum_gpu_b200 import CudaLlama, QKind
    from ferrum_gpu_b200.hostmodel import config_c4, random_llama, random_tokens
    cfg = config_c4()
    model = random_llama(cfg, seed=2, biases=True, tied=True)
    g = CudaLlama(dev, model, QKind.Q8_0, max_streams=streams)
    toks = random_tokens(7, streams, cfg.vocab)
    for _ in range(3):  # eager step, graph capture, first replay - on throw-away positions
        g.feed_batch(toks)
    for s in range(streams):
        g.reset(s)
    t0 = time.perf_counter()
    for s in range(streams):
        g.prefill(random_tokens(500 + s, prefill, cfg.vocab), stream=s)
    prefill_s = time.perf_counter() - t0
    dev.sync()
    head_n = min(32, steps // 2)
    t0 = time.perf_counter()
    toks = g.decode_greedy(toks, head_n)[-1]
    first_ms = (time.perf_counter() - t0) / head_n * 1e3
    mid = steps - 2 * head_n
    t1 = time.perf_counter()
    if mid > 0:
        toks = g.decode_greedy(toks, mid)[-1]
    t2 = time.perf_counter()
    toks = g.decode_greedy(toks, head_n)[-1]
    t3 = time.perf_counter()
    last_ms = (t3 - t2) / head_n * 1e3
    dt = (t3 - t0) / steps
    for s in range(streams):
        g.reset(s)
    g.prefill(random_tokens(500, prefill, cfg.vocab), stream=0)  # (a step at the initial cache length, per kernel)
    for s in range(1, streams):
        g.prefill(random_tokens(500 + s, 8, cfg.vocab), stream=s)
    dev.profile(True)
    g.feed_batch(toks)
    prof = dev.profile_report()
    dev.profile(False)
    # the same prompt through the scoring kernels into the cache (second of two runs: the first grows the workspace)
    from ferrum_gpu_b200 import Mode
    tc_s = None
    for _ in range(2):
        g.reset(0)
        t0 = time.perf_counter()
        g.prefill(random_tokens(500, prefill, cfg.vocab), stream=0, mode=Mode.TENSOR_F16)
        tc_s = time.perf_counter() - t0
    wbytes = g.weight_bytes()
    mean_len = prefill + steps / 2
    kv_bytes = 2 * cfg.kv_dim * 4 * mean_len * cfg.layers * streams
    g.close()
    total = sum(v["ms"] for v in prof.values()) or 1.0
    return {"workload": f"c4-qwen2-24L-d1024-q8_0-{streams}streams-{prefill}+{steps}", "tok_s": streams / dt,
            "ms_per_step": dt * 1e3, "ms_per_step_first32": first_ms, "ms_per_step_last32": last_ms, "prefill_s": prefill_s,
            "prefill_tok_s": {"exact_f32": streams * prefill / prefill_s, "tensor_f16": prefill / tc_s},
            "bytes_per_step": wbytes + kv_bytes,
            "hbm_frac": (wbytes + kv_bytes) / dt / 1e9 / hbm_gbs,
            "launches_of_a_step": {k: v["launches"] for k, v in sorted(prof.items(), key=lambda kv: -kv[1]["ms"])[:8]}}


def bench_sweep(dev, hbm_gbs, tf_burst):
    """The isolated quantised product Y[M,N] = X[M,K] W[N,K]^T over the configuration's grid: K in {768, 2048,
    4096} x N in {768, 2816, 11008, 32000} x M in {1, 8, 64, 512, 4096}, Q4_0 and Q8_0; X ~ N(0, 1) f32 and
    W ~ N(0, 0.02) on the device. M <= 64 runs the exact decode kernels and is reported as packed weight bytes
    per second against the measured copy bandwidth; M >= 512 runs the tcgen05 product and is reported as
    2 M N K flop per second against the measured burst bf16 peak. Timing: CUDA events around batches of
    back-to-back launches that rotate over several copies of the weight (together above 256 MB where a copy is
    small enough to make eight of them, else the entry says `l2`), best of three batches."""
    import ctypes as C
    import torch
    from ferrum_gpu_b200 import Mode, QKind, upload_quantised, _ffi
    lib = _ffi.load()
    st = torch.cuda.ExternalStream(dev.stream())
    rng = np.random.default_rng(11)
    rows = []
    for k in (768, 2048, 4096):
        for n in (768, 2816, 11008, 32000):
            wt = (rng.standard_normal(k * n, dtype=np.float32) * np.float32(0.02)).astype(np.float32)
            for kind in (QKind.Q4_0, QKind.Q8_0):
                wbytes = k * n * (18 if kind == QKind.Q4_0 else 34) / 32
                copies = int(min(8, max(1, -(-256e6 // wbytes))))
                qws = [upload_quantised(dev, kind, wt, k, n) for _ in range(copies)]
                cold = copies * wbytes >= 256e6
                for m in (1, 8, 64, 512, 4096):
                    x = torch.randn(m, k, device="cuda")
                    y = torch.empty(m, n, device="cuda")
                    mode = int(Mode.EXACT_F32 if m <= 64 else Mode.TENSOR_F16)
                    reps = 3 if m >= 512 else 4
                    for q in qws:
                        dev.check(lib.fc_qmatmul_dev(q.handle, x.data_ptr(), m, y.data_ptr(), mode))
                    dev.sync()
                    best = None
                    for _ in range(3):
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record(st)
                        for _ in range(reps):
                            for q in qws:
                                dev.check(lib.fc_qmatmul_dev(q.handle, x.data_ptr(), m, y.data_ptr(), mode))
                        e1.record(st)
                        e1.synchronize()
                        us = e0.elapsed_time(e1) * 1e3 / (reps * copies)
                        best = us if best is None else min(best, us)
                    dev.sync()
                    if m <= 64:
                        rate = wbytes / best / 1e3  # GB/s
                        rows.append([k, n, m, kind.label(), round(best, 1), round(rate), round(rate / hbm_gbs, 3),
                                     "hbm" if cold else "l2"])
                    else:
                        rate = 2.0 * m * n * k / best / 1e6  # TFLOP/s
                        rows.append([k, n, m, kind.label(), round(best, 1), round(rate, 1), round(rate / tf_burst, 3), "tensor"])
                    del x, y
                for q in qws:
                    q.close()
    return {"columns": ["K", "N", "M", "kind", "us", "GB/s | TFLOP/s", "frac of measured peak", "bound"], "rows": rows}


def bench_strong(dev, g, stream, ids_host, world, rank, local, args):
    """Strong scaling of the scoring configuration: its 256 sequences shared out over the ranks (256 / N each),
    the per-sequence NLL sums all-gathered at the end of every step; same timing protocol as the weak number."""
    import torch
    import torch.distributed as dist
    from ferrum_gpu_b200 import Mode
    per = N_SEQS // world
    ids = np.ascontiguousarray(ids_host[:per])
    with torch.cuda.stream(stream):
        ids_dev = torch.from_numpy(ids).to(f"cuda:{local}")
        nll = torch.zeros(per, dtype=torch.float64, device=f"cuda:{local}")
        gathered = torch.zeros(world * per, dtype=torch.float64, device=f"cuda:{local}")

        def step():
            g.score_dev(ids_dev.data_ptr(), per, SEQ_LEN, Mode.TENSOR_F16, 0, 0, nll.data_ptr())
            dist.all_gather_into_tensor(gathered, nll)

        for _ in range(max(args.warmup, 3)):
            step()
        stream.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            step()
        e1.record(stream)
        stream.synchronize()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=f"cuda:{local}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / args.steps
    return {"scaling": "strong", "seqs_total": per * world, "seqs_per_gpu": per, "ms_per_step": ms,
            "value": per * world * (SEQ_LEN - 1) / (ms * 1e-3), "unit": UNIT}


def bench_c5(world, rank, args):
    """The GPT-2-124M configuration (12 layers, d_model 768, vocab 50257 tied, Q4_0), 512 sequences x 1024, through
    the multi-GPU group of the C ABI (fc_group_score: host ids in, NLL sums out on every rank, NCCL inside the
    library): the replicated head, then the head split over 2 and 4 vocabulary shards. Per layout: tokens/s from
    the slowest rank's wall time per call, the device time of the exchanges, and the largest difference of a
    sequence's NLL from the replicated head's on the same sequences."""
    import torch
    import torch.distributed as dist
    from ferrum_gpu_b200 import Mode, QKind
    from ferrum_gpu_b200.group import GroupScorer
    from ferrum_gpu_b200.hostmodel import config_c5, random_gpt2, random_tokens
    cfg = config_c5()
    model = random_gpt2(cfg, seed=3, tied=True)
    n_seqs = 512
    ids = np.stack([random_tokens(7000 + i, SEQ_LEN, cfg.vocab) for i in range(n_seqs)])
    res, base = {}, None
    for shards in (1, 2, 4):
        if world % shards:
            continue
        gs = GroupScorer(model, QKind.Q4_0, vocab_shards=shards, mode=Mode.TENSOR_F16)
        nll = None
        for _ in range(2):
            nll = gs.score(ids)
        dist.barrier()
        times = []
        for _ in range(max(2, min(args.steps, 3))):
            t0 = time.perf_counter()
            nll = gs.score(ids)
            times.append(time.perf_counter() - t0)
        ex = gs.exchange_ms()
        gs.close()
        t = torch.tensor([min(times)], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if shards == 1:
            base = nll
        res[f"vocab_shards_{shards}"] = {
            "tok_s": n_seqs * (SEQ_LEN - 1) / float(t.item()), "ms_per_call": float(t.item()) * 1e3,
            "exchange_ms": {"hidden_all_gather": ex[0], "partials_all_gather": ex[1], "nll_all_reduce": ex[2]},
            "max_abs_nll_diff_vs_replicated": float(np.abs(nll - base).max()), "nll_checksum": float(nll.sum())}
    return {"workload": "c5-gpt2-124M-q4_0-scoring-512x1024", "entry": "fc_group_score (host ids, NCCL inside the library)",
            "layouts": res} if rank == 0 else None


def cpu_baseline(cfg, model):
    """The f32 oracle (a port of the reference's CPU path) on one host thread, bounded sample."""
    from ferrum_gpu_b200 import _ffi
    from ferrum_gpu_b200.hostmodel import random_tokens
    from oracle import oracle as orc
    ref = orc.dequantised_llama(model, _ffi.FC_Q4_0, snap_embedding=False)
    oracle = orc.OracleLlama(ref, threads=1)
    n = 49
    ids = random_tokens(100, n, cfg.vocab)
    t0 = time.perf_counter()
    oracle.score(ids)
    dt = time.perf_counter() - t0
    return {"value": (n - 1) / dt, "unit": UNIT, "cores": 1, "kind": "port",
            "sample": f"1 sequence x {n} tokens (of 256 x 1024), single thread as `--device cpu` runs scoring"}


# ---- small, self-terminating workloads of the hot kernels, sized for an `ncu` capture (inputs above the 126 MB
# L2 where DRAM figures matter, a few launches, well under a GB on the device): python bench.py --case NAME

def _weights(k, n, seed=1):
    return (np.random.default_rng(seed).standard_normal(k * n, dtype=np.float32) * np.float32(0.02)).astype(np.float32)


def case_gemm(dev):
    """tensor-core product, Q4_0, M=16384 K=768 N=1280"""
    from ferrum_gpu_b200 import Mode, QKind, linear_q, upload_quantised
    k, n, m = 768, 1280, 16384
    qw = upload_quantised(dev, QKind.Q4_0, _weights(k, n), k, n)
    x = np.random.default_rng(2).standard_normal(m * k, dtype=np.float32)
    for _ in range(3):
        linear_q(dev, x, qw, m, Mode.TENSOR_F16)
    qw.close()


def _case_matvec(dev, m):
    from ferrum_gpu_b200 import QKind, linear_q, upload_quantised
    k, n = 4096, 32000
    x = np.random.default_rng(2).standard_normal(m * k, dtype=np.float32)
    for kind in (QKind.Q4_0, QKind.Q8_0):
        qw = upload_quantised(dev, kind, _weights(k, n), k, n)
        for _ in range(3):
            linear_q(dev, x, qw, m)
        qw.close()


def case_matvec(dev):
    """decode product of one row, Q4_0 and Q8_0, K=4096 N=32000"""
    _case_matvec(dev, 1)


def case_matvec8(dev):
    """tensor-core decode product, 8 rows, K=4096 N=32000"""
    _case_matvec(dev, 8)


def _c3_model(dev, layers=None, max_streams=1):
    from ferrum_gpu_b200 import CudaLlama, QKind
    from ferrum_gpu_b200.hostmodel import config_c3, random_llama
    cfg = config_c3()
    if layers:
        cfg.layers = layers
    return cfg, CudaLlama(dev, random_llama(cfg, seed=1), QKind.Q4_0, max_streams=max_streams)


def case_score(dev):
    """8 sequences x 1024 of the Llama scoring configuration, 2 layers"""
    from ferrum_gpu_b200 import Mode
    from ferrum_gpu_b200.hostmodel import random_tokens
    cfg, g = _c3_model(dev, layers=2)
    ids = np.stack([random_tokens(10 + i, 1024, cfg.vocab) for i in range(8)])
    for _ in range(2):
        g.score_batch(ids, Mode.TENSOR_F16)
    g.close()


def case_chunk(dev):
    """32 sequences x 1024, one layer (a quarter of one bench chunk: per-launch DRAM traffic scales with the rows)"""
    from ferrum_gpu_b200 import Mode
    from ferrum_gpu_b200.hostmodel import random_tokens
    cfg, g = _c3_model(dev, layers=1)
    ids = np.stack([random_tokens(10 + i, 1024, cfg.vocab) for i in range(32)])
    for _ in range(2):
        g.score_batch(ids, Mode.TENSOR_F16)
    g.close()


def case_attention(dev):
    """the causal attention kernels alone, 16 x 1024 x 12 heads"""
    n_seqs, t, heads, kv = 16, 1024, 12, 4
    qkv = np.random.default_rng(0).standard_normal((n_seqs * t, (heads + 2 * kv) * 64)).astype(np.float16)
    for variant in (1, 3):
        dev.attention_f16(qkv, n_seqs, t, heads, kv, variant=variant, iters=1)


def _case_decode(dev, streams, layers, vocab, tied):
    from ferrum_gpu_b200 import CudaLlama, QKind
    from ferrum_gpu_b200.hostmodel import LlamaConfig, random_llama, random_tokens
    cfg = LlamaConfig(vocab=vocab, ctx=2048, dim=1024, heads=16, kv_heads=2, head_dim=64, layers=layers, hidden=2816,
                      rope_dim=64, rope_base=1e6, rope_type=1, eps=1e-6)
    g = CudaLlama(dev, random_llama(cfg, seed=1, biases=True, tied=tied), QKind.Q8_0, max_streams=streams)
    for s in range(streams):
        g.prefill(random_tokens(s, 1500, cfg.vocab), stream=s)
    toks = random_tokens(99, streams, cfg.vocab)
    for _ in range(3):
        g.feed_batch(toks)
    g.close()


def case_decode(dev):
    """batched decode step: 16 streams at cache length ~1500, 2 layers"""
    _case_decode(dev, 16, 2, 32000, False)


def case_decode64(dev):
    """four layers and the 151936-row head of the 64-stream decode configuration at 1500 cached positions"""
    _case_decode(dev, 64, 4, 151936, True)


def case_head64(dev):
    """the vocabulary-head product of the 64-stream decode configuration: 64 rows against 151936 x 1024 Q8_0"""
    from ferrum_gpu_b200 import QKind, linear_q, upload_quantised
    k, n, m = 1024, 151936, 64
    qw = upload_quantised(dev, QKind.Q8_0, _weights(k, n), k, n)
    x = np.random.default_rng(2).standard_normal(m * k, dtype=np.float32)
    for _ in range(3):
        linear_q(dev, x, qw, m)
    qw.close()


def case_decode1(dev):
    """batch-1 greedy decode of the GPT-2-style configuration: 16 prompt tokens, then 64 chained steps"""
    from ferrum_gpu_b200 import CudaGpt2, QKind
    from ferrum_gpu_b200.hostmodel import config_c1, random_gpt2, random_tokens
    cfg = config_c1()
    m = CudaGpt2(dev, random_gpt2(cfg, seed=1), QKind.Q8_0)
    tok = 0
    for t in random_tokens(2, 16, cfg.vocab):
        tok = m.feed_greedy(int(t))
    m.decode_greedy([tok], 64)
    m.close()


CASES = {"gemm": case_gemm, "matvec": case_matvec, "matvec8": case_matvec8, "decode": case_decode, "decode64": case_decode64,
         "head64": case_head64, "score": case_score, "head": case_score, "chunk": case_chunk, "attention": case_attention,
         "decode1": case_decode1}


def run_case(name):
    from ferrum_gpu_b200 import Device
    d = Device.open(0)
    try:
        CASES[name](d)
        d.sync()
        print("case", name, "done;", d.launch_count(), "launches")
    finally:
        d.close()


if __name__ == "__main__":
    main()
