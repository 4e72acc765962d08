#!/usr/bin/env python
"""Decode benchmark: tokens/s of the per-token transformer forward over GGUF K-quant weights.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl b200|reference]

A step is one decode step (one new token for every sequence of the batch). The default workload is
the Llama-2-7B-shaped Q4_K_M-style model at batch 1 with a 1024-token prompt and an INT8 KV cache.
Weights are synthetic (seeded N(0, 0.02), quantized by the package's writer); prompts are seeded
uniform token ids. One JSON line is printed by rank 0.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__  # noqa: E402

WORKLOADS = {
    # name: (shape, scheme, batch, prompt_len, kv)
    "c1-tinyllama-q8_0-bs1": ("tinyllama-1.1b", 0, 1, 128, "f32"),
    "c2-tinyllama-q4km-bs1": ("tinyllama-1.1b", 1, 1, 512, "i8"),
    "c3-llama2-7b-q4km-bs1": ("llama2-7b", 1, 1, 1024, "i8"),
    "c3-llama2-7b-q4km-bs16": ("llama2-7b", 1, 16, 1024, "i8"),
    # ragged contexts: prompt lengths uniform in [256, 4096] from PCG64(99)
    "c4-llama3-8b-q6k-bs64": ("llama3-8b", 2, 64, (256, 4096), "i8"),
    # 70B shape: the reference caps the context at 8192 positions (model_config.cpp:171-177), so the
    # "8192-token context + 128 steps" of the configuration is run as an 8064-token prompt + 128 steps
    "c5-llama2-70b-q4km-bs1": ("llama2-70b", 1, 1, 8064, "i8"),
    "c5-llama2-70b-q4km-bs32": ("llama2-70b", 1, 32, 8064, "i8"),
    "tiny": ("tiny", 1, 1, 16, "i8"),
}
# golden case of tests/golden/full_models.npz that belongs to a (shape, scheme): used by the in-run parity check
GOLDEN_CASE = {("tinyllama-1.1b", 0): "c1", ("tinyllama-1.1b", 1): "c2", ("llama2-7b", 1): "c3"}
DEFAULT_WORKLOAD = "c3-llama2-7b-q4km-bs1"
METRIC = "decode tokens/s (Llama-2-7B Q4_K_M, bs=1) and % of HBM roofline at 1/2/4/8 B200"


def peaks():
    """(HBM GB/s, dense bf16 TFLOP/s burst, source): the driver-measured figures when present, else the pool's fallback."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
        except Exception:
            pass
    return 6650.0, 1590.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons while the run lasts (read-only): through NVML every 5 ms when the
    Python binding is there, else through nvidia-smi every 200 ms."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.rows, self._stop_evt = index, [], threading.Event()
        self.nvml = self.handle = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml, self.handle = pynvml, pynvml.nvmlDeviceGetHandleByIndex(index)
        except Exception:
            self.nvml = None

    def _sample_nvml(self):
        n, h = self.nvml, self.handle
        sm = float(n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM))
        mx = float(n.nvmlDeviceGetMaxClockInfo(h, n.NVML_CLOCK_SM))
        try:
            mask = int(n.nvmlDeviceGetCurrentClocksEventReasons(h))
        except Exception:
            mask = int(n.nvmlDeviceGetCurrentClocksThrottleReasons(h))
        self.rows.append((sm, mx, [name for name, bit in self.BITS.items() if mask & bit]))

    def _sample_smi(self):
        out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits"],
                             capture_output=True, text=True, timeout=5).stdout
        parts = [x.strip() for x in out.strip().split(",")]
        if len(parts) >= 7:
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            self.rows.append((float(parts[0]), float(parts[1]), [n for i, n in enumerate(names) if parts[3 + i].lower().startswith("active")]))

    def run(self):
        while not self._stop_evt.is_set():
            try:
                if self.nvml:
                    self._sample_nvml()
                else:
                    self._sample_smi()
            except Exception:
                pass
            self._stop_evt.wait(0.005 if self.nvml else 0.2)

    def finish(self):
        self._stop_evt.set()
        self.join(timeout=6)
        sm = [r[0] for r in self.rows]
        reasons = sorted({n for r in self.rows for n in r[2]})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max((r[1] for r in self.rows), default=None),
                "reasons": reasons, "samples": len(self.rows), "source": "nvml" if self.nvml else "nvidia-smi"}


_T0 = time.perf_counter()


def progress(msg):
    """Phase marks on stderr (stdout carries the one JSON line only)."""
    print(f"[bench {time.perf_counter() - _T0:7.1f} s] {msg}", file=sys.stderr, flush=True)


def model_path(pkg, shape, scheme):
    base = "/dev/shm" if os.path.isdir("/dev/shm") and os.access("/dev/shm", os.W_OK) else "/tmp"
    path = os.path.join(base, f"b200_synth_{shape}_s{scheme}.gguf")
    if not os.path.exists(path):
        tmp = path + f".{os.getpid()}.tmp"
        pkg.synth.write_gguf(tmp, shape, scheme=scheme)
        os.replace(tmp, path)
    return path


def prompt_lengths(batch, prompt_len):
    """One length per sequence: a fixed length, or (lo, hi) = ragged lengths uniform in [lo, hi] from PCG64(99)."""
    if isinstance(prompt_len, tuple):
        lo, hi = prompt_len
        return [int(v) for v in np.random.Generator(np.random.PCG64(99)).integers(lo, hi + 1, batch)]
    return [int(prompt_len)] * batch


def prompts(batch, n, vocab):
    lens = prompt_lengths(batch, n)
    return [np.random.Generator(np.random.PCG64(4321 + s)).integers(0, vocab, lens[s]).astype(np.int32) for s in range(batch)]


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def cpu_reference_tokens_per_s(path, budget_s, max_tokens, prompt=None):
    """Times the reference's own CPU forward (oracle/_ref) on the same model file: after ingesting `prompt`
    through its batch path (untimed; None = empty context), greedy decode steps, as many as fit the time
    budget (at least one). Returns (tokens/s, threads, steps, seconds, start context)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    os.environ.setdefault("OMP_NUM_THREADS", str(cores))
    if hasattr(ol.ref(), "ref_set_threads"):
        ol.ref().ref_set_threads(cores)  # a launcher may have pinned OMP_NUM_THREADS to 1
    m = ol.RefModel(path)
    tok, start = 5, 0
    if prompt is not None and len(prompt):
        tok, start = int(m.prefill(prompt).argmax()), len(prompt)
    n, t0 = 0, time.perf_counter()
    while n < max_tokens:
        tok = int(m.decode(tok, start + n).argmax())
        n += 1
        if time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    return n / dt, cores, n, dt, start


def run_reference(args, shape, scheme, batch, prompt_len, kv):
    """The reference arm: the reference's own CPU path (oracle/_ref) on the workload's model file, batch 1, all host
    threads. Greedy decode steps from an EMPTY context for at most 120 s; `steps` in the line is what really ran (the
    first step also pays the reference's lazy dequantisation, so it is the one warm-up step and is timed with the
    rest). The reference's batch prompt path is not used here: it needs ~15 minutes of CPU time for 32 tokens of the 7B
    shape. A CPU token is weight-bound (every weight is dequantised and multiplied once per token), so the
    1024-token context of the GPU arm would change its time per token by well under 1 %."""
    rank, _, world = dist_env()
    if rank != 0:
        return
    pkg = __graft_entry__.load_package()
    path = model_path(pkg, shape, scheme)
    tps, cores, n, dt, start = cpu_reference_tokens_per_s(path, budget_s=120.0, max_tokens=max(1, args.steps), prompt=None)
    sample = (f"{n} greedy decode steps of the full model from an empty context (batch 1, FP32 KV: the reference has no CPU "
              f"INT8 cache), {dt:.1f} s")
    line = {"impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": n, "warmup": 0, "ms_per_step": 1000.0 / tps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": {"workload": args.workload, "batch": 1, "prompt_len": prompt_len if not isinstance(prompt_len, tuple) else list(prompt_len),
                       "kv_cache": kv, "context_during_timing": [start, start + n],
                       "reference_protocol": "greedy decode from an empty context on the host cores; batch 1; FP32 KV; time per token is "
                                             "weight-bound and independent of the context to well under 1 %",
                       "requested_steps": args.steps, "requested_warmup": args.warmup},
            "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "reference", "sample": sample},
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def parity_in_run(eng, shape, scheme, kv):
    """Replays the committed golden case of this model (ids and logits from the reference's CPU path, or from the
    restated oracle for an INT8 cache; tests/golden/make_golden_full.py) on the engine that was just timed: the
    golden prompt token by token, then the greedy steps. Returns a dict for the JSON line, or None."""
    case = GOLDEN_CASE.get((shape, scheme))
    gpath = os.path.join(ROOT, "tests", "golden", "full_models.npz")
    if case is None or not os.path.exists(gpath):
        return None
    g = np.load(gpath)
    tag = f"{case}_{'i8' if kv == 'i8' and case != 'c1' else 'f32'}"
    if f"{tag}_ids" not in g or (kv == "i8") != tag.endswith("i8"):
        return None
    prompt, ids = g[f"{case}_prompt"], g[f"{tag}_ids"]
    eng.kv_reset(0)
    logits = None
    for i, t in enumerate(prompt):
        logits, _ = eng.decode([int(t)], [i])
    err = float(np.abs(logits[0] - g[f"{tag}_prefill_logits"]).max())
    got, tok = [int(logits[0].argmax())], int(ids[0])
    keep = {int(k): j for j, k in enumerate(g[f"{tag}_step_index"])}
    for i in range(len(ids) - 1):
        logits, amax = eng.decode([tok], [len(prompt) + i])
        if i in keep:
            err = max(err, float(np.abs(logits[0] - g[f"{tag}_step_logits"][keep[i]]).max()))
        got.append(int(amax[0]))
        tok = int(ids[i + 1])
    return {"case": tag, "source": "tests/golden/full_models.npz: " + ("restated oracle (INT8 KV)" if tag.endswith("i8") else "reference CPU path"),
            "ids_checked": len(ids), "ids_match": got == [int(v) for v in ids], "max_abs_logit_err": round(err, 6),
            "logit_gate": 2e-2 if not tag.endswith("i8") else round(max(2e-2, 0.25 * float(np.abs(g[f"{tag}_prefill_logits"] - g[f"{case}_f32_prefill_logits"]).max())), 4),
            "logit_gate_note": None if not tag.endswith("i8") else "INT8 cache: 2e-2 or a quarter of the oracle's own INT8-vs-FP32 drift (rounding flips of cached values)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="timed decode steps (default 256; 96 for the 70B workloads, whose context ends at the reference's 8192-position cap)")
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--planes", type=int, default=3, choices=[2, 3])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-check", action="store_true", help="skip the in-run parity check against the golden fixtures")
    args = ap.parse_args()
    shape, scheme, batch, prompt_len, kv = WORKLOADS[args.workload]
    if args.steps is None:
        args.steps = 96 if shape == "llama2-70b" else 256
    if args.impl == "reference":
        return run_reference(args, shape, scheme, batch, prompt_len, kv)

    rank, local_rank, world = dist_env()
    # stdout carries the one JSON line only: whatever a library prints while the run lasts (NCCL's version banner,
    # for one) goes to stderr, and the line is written to the saved descriptor at the end
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    warmup = max(args.warmup, 3)
    pkg = __graft_entry__.load_package()
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    # model file: written once per box (rank 0), then shared
    if rank == 0:
        path = model_path(pkg, shape, scheme)
        progress("model file ready")
    if dist:
        dist.barrier()
    path = model_path(pkg, shape, scheme)
    t_load = time.perf_counter()
    nccl_id = None
    if dist:  # tensor parallel over the ranks of this node: rank 0 makes the NCCL id, everyone gets it
        import torch
        idt = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            idt.copy_(torch.tensor(list(pkg.api.nccl_unique_id()), dtype=torch.uint8))
        dist.broadcast(idt, src=0)
        nccl_id = bytes(idt.cpu().tolist())
    max_pos = pkg.synth.SHAPES[shape]["max_pos"]
    longest = max(prompt_lengths(batch, prompt_len))
    e2e_steps = max(1, min(args.steps, 64, max_pos - longest - warmup - args.steps - 2))
    if longest + warmup + args.steps + 1 + e2e_steps > max_pos:
        raise SystemExit(f"{args.workload}: prompt {longest} + {warmup} + {args.steps} steps exceed the model's {max_pos} positions")
    eng = pkg.Engine.from_gguf(path, kv_dtype=pkg.KV_I8 if kv == "i8" else pkg.KV_F32, max_seqs=batch,
                               max_ctx=min(max_pos, longest + args.steps + warmup + e2e_steps + 8), act_planes=args.planes, device=local_rank,
                               tp_rank=rank, tp_size=world, nccl_id=nccl_id)
    t_load = time.perf_counter() - t_load
    if rank == 0:
        progress(f"engine loaded in {t_load:.1f} s")
    vocab = eng.vocab
    pr = prompts(batch, prompt_len, vocab)
    t_prefill = time.perf_counter()
    if batch > 1:  # all prompts in one sequence-aware call (shared 512-token chunks)
        first = [int(v.argmax()) for v in eng.prefill_batch(pr)]
    else:
        first = [int(eng.prefill(pr[0], slot=0).argmax())]
    t_prefill = time.perf_counter() - t_prefill
    if rank == 0:
        progress(f"prompts ingested in {t_prefill:.1f} s")
    lens = prompt_lengths(batch, prompt_len)
    pos = 0  # steps decoded so far; sequence s is at position lens[s] + pos

    def at(p):
        return [n + p for n in lens]

    # ---- warm-up, then the timed device-resident loop ----
    sampler = ClockSampler(local_rank)  # runs across warm-up, the timed loop, the end-to-end leg and the per-kind timings
    sampler.start()
    out, _ = eng.generate_greedy(first, at(pos), warmup)
    pos += warmup
    nxt = out[-1].copy()
    if dist:
        dist.barrier()
    out, ms = eng.generate_greedy(nxt, at(pos), args.steps)
    pos += args.steps
    if dist:
        import torch
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    tokens_per_s = batch * args.steps / (ms / 1000.0)  # one tensor-parallel group: the ranks share the same sequences
    if rank == 0:
        progress(f"timed loop done: {ms / args.steps:.3f} ms per step")

    # ---- end to end through the C ABI with host buffers: token ids in, logits out, host argmax ----
    toks = out[-1].copy()
    eng.decode(toks, at(pos))  # graph already warm; one untimed call
    pos += 1
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        logits, _ = eng.decode(toks, at(pos + i), want_logits=True, want_argmax=False)
        toks = logits.argmax(axis=1).astype(np.int32)
    e2e_dt = time.perf_counter() - t0
    e2e_tps = batch * e2e_steps / e2e_dt

    # ---- roofline of the dominant kernel (the fused dequant-GEMV), each kind timed by itself ----
    st = eng.stats()
    L = eng.desc.num_hidden_layers
    kinds = {"gate_up_swiglu": (0, L), "qkv_rope": (1, L), "o_proj": (2, L), "down_proj": (3, L), "lm_head": (4, 1)}
    peak, peak_tf, peak_src = peaks()
    ksum_b = ksum_t = ksum_f = 0.0
    kern = {}
    on_tc = batch >= 16  # the step's linear layers run on the tensor-core matmul: time that path, for the whole batch
    d = eng.desc
    hd = d.hidden_size // d.num_attention_heads
    rows_of = {"gate_up_swiglu": 2 * d.intermediate_size // world, "qkv_rope": (d.num_attention_heads + 2 * d.num_key_value_heads) * hd // world,
               "o_proj": d.hidden_size, "down_proj": d.hidden_size, "lm_head": d.vocab_size // world}
    k_of = {"gate_up_swiglu": d.hidden_size, "qkv_rope": d.hidden_size, "o_proj": d.hidden_size // world,
            "down_proj": d.intermediate_size // world, "lm_head": d.hidden_size}
    for name, (which, per_step) in kinds.items():
        us, nbytes = eng.time_kernel(which + (16 if on_tc else 0), max(2 * L, 32))
        flops = 2.0 * rows_of[name] * k_of[name] * batch
        kern[name] = {"us": round(us, 3), "bytes": nbytes, "GBps": round(nbytes / us / 1e3, 1), "launches_per_step": per_step}
        if on_tc:
            kern[name]["TFLOPs"] = round(flops / us / 1e6, 1)
        ksum_b += nbytes * per_step
        ksum_t += us * per_step
        ksum_f += flops * per_step
    gemv_launches = sum(v[1] for v in kinds.values())
    # DRAM bytes (read + write) per launch from one ncu capture of this workload's four per-layer kinds
    # (profiles/gemv_kernel_7b_q4km_bs1.txt); the lm_head launch was not captured and is scaled from its
    # algorithmic bytes by the mean ratio of the others. Other workloads: no capture, null.
    traffic = traffic_source = None
    if args.workload == "c3-llama2-7b-q4km-bs1" and world == 1:
        traffic_source = "profiles/gemv_kernel_7b_q4km_bs1.txt (one ncu capture of the same launches; not measured in this run)"
        ncu_mb = {"gate_up_swiglu": 51.530, "qkv_rope": 32.998, "down_proj": 38.268, "o_proj": 9.667}
        ratio = sum(ncu_mb.values()) * 1e6 / sum(kern[k]["bytes"] for k in ncu_mb)
        tot = sum(ncu_mb[k] * 1e6 * kinds[k][1] for k in ncu_mb) + ratio * kern["lm_head"]["bytes"]
        traffic = int(tot / gemv_launches)
    achieved = ksum_b / ksum_t / 1e3  # GB/s
    ctx_sum_mid = sum(lens) + batch * (warmup + args.steps / 2.0)  # context positions read per step, over all sequences, mid-run
    # per-rank shares add up to the whole model over the ranks (norm vectors are replicated: negligible)
    step_bytes = world * (st["weight_bytes"] + ctx_sum_mid * st["kv_bytes_per_position"]) + batch * 4 * eng.hidden
    step_gbps = step_bytes / (ms / args.steps / 1e3) / 1e9 / world  # per GPU
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
                "traffic": traffic, "traffic_source": traffic_source, "peak_source": peak_src, "kernel": f"gemv_kernel<{args.planes}>",
                "timed": "each kind alone, stream-ordered launches without programmatic overlap, a different layer's weights per launch",
                "bytes_per_launch": int(ksum_b / gemv_launches), "us_per_launch": round(ksum_t / gemv_launches, 3),
                "kinds": kern, "step_bytes": int(step_bytes), "step_GBps": round(step_gbps, 1),
                "step_frac_of_measured_peak": round(step_gbps / peak, 4), "step_frac_of_8TBps": round(step_gbps / 8000.0, 4)}

    clocks = sampler.finish()
    if on_tc:
        # batch >= 16: the linear layers run on the tcgen05 matmul (with its fp16 conversion and split-K reduction). Below
        # ~128 tokens the matmul is still bound by the packed weight bytes (2 * batch / 0.5625 FLOP per byte against a
        # machine balance of ~250), so the roofline stays the HBM one; the tensor throughput is reported beside it.
        tf = ksum_f / ksum_t / 1e6
        roofline.update({"kernel": "gemm_tc_kernel (+ to_half_kernel, splitk_reduce_kernel)", "traffic": None, "traffic_source": None,
                         "tensor_TFLOPs": round(tf, 1), "tensor_peak_TFLOPs": peak_tf, "tensor_frac": round(tf / peak_tf, 4)})
        if batch >= 128:
            roofline.update({"bound": "tensor", "achieved": round(tf, 1), "peak": peak_tf, "unit": "TFLOP/s", "frac": round(tf / peak_tf, 4)})
    line = {"metric": METRIC, "value": tokens_per_s, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak" if world == 1 else "strong",
            "vs_baseline": None, "dtype": f"i{8 * args.planes} activations x packed int weights, f32 accumulate",
            "data": "synthetic",
            "config": {"workload": args.workload, "batch": batch, "prompt_len": list(prompt_len) if isinstance(prompt_len, tuple) else prompt_len,
                       "kv_cache": kv, "context_during_timing": [min(lens) + warmup, max(lens) + warmup + args.steps],
                       "parallelism": "single GPU" if world == 1 else f"tp{world} (column-split QKV/gate/up/head, row-split O/down, " +
                                      ("one-shot all-reduce over peer memory inside the matvec kernels" if st["launches_per_step"] <= 3 + 5 * L
                                       else "NCCL all-reduce") + ", NCCL all-gather of logits)",
                       "l2": "weights read per step (GBs) exceed the 126 MB L2; no flush needed",
                       "act_planes": args.planes, "load_s": round(t_load, 2), "prefill_s": round(t_prefill, 2)},
            "e2e": {"value": e2e_tps, "unit": "tokens/s", "h2d_bytes_per_step": 12 * batch,
                    "d2h_bytes_per_step": 4 * vocab * batch, "steps": e2e_steps},
            "gpu_launches": st["launches_per_step"] * args.steps, "clocks": clocks, "roofline": roofline}

    if rank == 0 and world == 1 and batch == 1 and not args.no_check:
        chk = parity_in_run(eng, shape, scheme, kv)
        if chk is not None:
            line["parity_in_run"] = chk
    if rank == 0 and world == 1 and not args.no_cpu_baseline and os.path.exists(os.path.join(ROOT, "oracle", "_ref", "libref_cpu.so")):
        eng.close()
        tps, cores, n, dt, _ = cpu_reference_tokens_per_s(path, budget_s=20.0, max_tokens=4)
        line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "reference",
                                "sample": f"{n} decode steps of the same model file from an empty context, {dt:.1f} s"}
    if rank == 0:
        os.write(json_fd, (json.dumps(line) + "\n").encode())
    if dist:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
