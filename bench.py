"""Benchmark of the quantised scoring hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N = 1): the Llama-style scoring configuration - 12 layers, d_model 768, 12 query / 4 KV
heads, SwiGLU 2048, vocab 32000, Q4_0 weights drawn from N(0, 0.02) - scoring 256 sequences of 1024
uniform-random token ids for their total log-probability (fp16 tensor-core path, f32 accumulation). One step = one pass
over the 256 sequences of a rank. With N > 1 every rank holds a replica and scores its own 256
sequences (no data-path collective); the per-sequence NLL sums are all-gathered at the end of each step.
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
# (32 x 1024 rows: 52.1 MB read + 76.5 MB written), scaled by 4; see profiles/.
NCU_TRAFFIC_BYTES = 4 * (52.11e6 + 76.48e6)
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
    """The reference's own CPU path for this workload, restated (no Rust toolchain exists here): the
    f32 oracle over the dequantised weights, all host threads, on a bounded sample per step."""
    if rank != 0:
        return
    from ferrum_gpu_b200 import _ffi
    from ferrum_gpu_b200.hostmodel import config_c3, random_llama, random_tokens
    from oracle import oracle as orc
    cores = os.cpu_count() or 1
    cfg = config_c3()
    model = random_llama(cfg, seed=1)
    ref = orc.dequantised_llama(model, _ffi.FC_Q4_0, snap_embedding=False)
    oracle = orc.OracleLlama(ref, threads=cores)
    sample_len = 129
    ids = random_tokens(100, sample_len, cfg.vocab)
    for _ in range(min(args.warmup, 1)):
        oracle.score(ids)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.score(ids)
    dt = (time.perf_counter() - t0) / args.steps
    value = (sample_len - 1) / dt
    sample = f"1 sequence x {sample_len} tokens per step (of 256 x 1024), f32 oracle, {cores} threads"
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
            "roofline": {"bound": "tensor", "kernel": "qgemm_tc_kernel", "achieved": achieved, "peak": tf_sust,
                         "unit": "TFLOP/s", "frac": achieved / tf_sust, "peak_source": f"{peak_src} (sustained bf16)",
                         "frac_of_burst": achieved / tf_burst, "traffic": NCU_TRAFFIC_BYTES,
                         "traffic_note": NCU_TRAFFIC_NOTE,
                         "launches_per_step": gemm["launches"], "ms_per_step": gemm["ms"], "kernel_shares": shares,
                         "tflops_by_role": by_role, "attention_tflops": attn_tf},
            "model_flops_per_step": (lin_flops + attn_flops) * rows,
            "mfu_of_sustained": (lin_flops + attn_flops) * rows / (ms_step * 1e-3) / 1e12 / tf_sust,
            "nll_checksum": nll_total,
        }
        if not args.no_decode and world == 1:
            time.sleep(3.0)  # a separate, latency-bound workload: let the clocks recover from the power-capped scoring steps
            dsamp = ClockSampler(local)
            dsamp.start()
            out["decode"] = bench_decode(dev, hbm)
            out["decode"]["clocks"] = dsamp.stop()
            if not args.no_decode64:
                out["decode64"] = bench_decode64(dev, hbm)
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


def bench_decode64(dev, hbm_gbs, streams=64, prefill=1536, steps=32):
    """Batched KV-cached decode: the Qwen2-style configuration (24 layers, d_model 1024, 16 q / 2 kv heads,
    SwiGLU 2816, vocab 151936, tied head, q/k/v biases, Q8_0, f32 KV cache), 64 streams each with a
    1536-token prefill, then `steps` greedy steps of all streams together (of the configuration's 512;
    the cache length grows from 1536, the step cost with it)."""
    from ferrum_gpu_b200 import CudaLlama, QKind
    from ferrum_gpu_b200.hostmodel import config_c4, random_llama, random_tokens
    cfg = config_c4()
    model = random_llama(cfg, seed=2, biases=True, tied=True)
    g = CudaLlama(dev, model, QKind.Q8_0, max_streams=streams)
    t0 = time.perf_counter()
    for s in range(streams):
        g.prefill(random_tokens(500 + s, prefill, cfg.vocab), stream=s)
    prefill_s = time.perf_counter() - t0
    toks = random_tokens(7, streams, cfg.vocab)
    for _ in range(3):  # eager step, graph capture, first replay
        toks, _ = g.feed_batch(toks)
    dev.sync()
    t0 = time.perf_counter()
    toks = g.decode_greedy(toks, steps)[-1]  # the steps chained on the device, one call
    dt = (time.perf_counter() - t0) / steps
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
    mean_len = prefill + 3 + steps / 2
    kv_bytes = 2 * cfg.kv_dim * 4 * mean_len * cfg.layers * streams
    g.close()
    total = sum(v["ms"] for v in prof.values()) or 1.0
    return {"workload": f"c4-qwen2-24L-d1024-q8_0-{streams}streams-{prefill}+{steps}", "tok_s": streams / dt,
            "ms_per_step": dt * 1e3, "prefill_s": prefill_s,
            "prefill_tok_s": {"exact_f32": streams * prefill / prefill_s, "tensor_f16": prefill / tc_s},
            "bytes_per_step": wbytes + kv_bytes,
            "hbm_frac": (wbytes + kv_bytes) / dt / 1e9 / hbm_gbs,
            "kernel_shares": {k: round(v["ms"] / total, 3) for k, v in sorted(prof.items(), key=lambda kv: -kv[1]["ms"])[:6]},
            "profiled_step_ms": total}


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


if __name__ == "__main__":
    main()
