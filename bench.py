"""Benchmark of the attention hot path: batched paged decode attention over the block-table KV cache.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one batched paged decode call (one launch of the split-KV kernel, which plans for itself and merges cut sequences) over one batch of
synthetic sequences whose K/V pages already live in HBM.  Workload at N = 1: 64 sequences, context
lengths uniform in [1024, 32768], page 16, shuffled block table, Hq 32 / Hkv 8 / D 128, fp16 K/V,
fp32 Q and output.  At N > 1 every rank owns its own batch of that shape (sequences are
independent: sharded by sequence, no collective inside attention); every step the per-rank outputs
are gathered on every rank by the decode kernel itself, which stores each final row into every rank's buffer
(peer stores over NVLink into symmetric memory; NCCL all-gather as the fall-back).  Prints ONE JSON line (rank 0).

Every run (every N, N = 1 included) also carries `secondary.long_context_b256`: ONE fixed problem - 256
sequences, context lengths log-uniform in [4096, 131072], Hq 64 - split over the N ranks (strong scaling),
by sequence and, when the KV heads divide among the ranks, by KV head; its `ms_per_step` at N = 1, 2, 4, 8
gives the scaling efficiency T(1) / (N T(N)) on the identical problem.

--impl reference times Granite's CPU attention arithmetic on a bounded sample of the same workload, on
the host cores: pages fetched by the rule of metal_compute.h:853-861 into the contiguous cache layout,
then the reference's own statements - the cache widening of src/llm/transformer.mm:1753-1765 and the
loop of :1779-1840 with its thread policy - compiled from the checkout into oracle/_ref when that was
built (kind "reference"), else their restatement in oracle/ (kind "port").
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOAD = "paged_decode_b64"
METRIC = "paged decode attention GB/s"
UNIT = "GB/s"
kT_ROWS = 128  # rows and keys per tile of the tensor-core kernel


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs
    (read-only queries; nothing is set)."""

    def __init__(self, index: int, period_s: float = 0.003):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self.period = period_s
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80): "hw_power_brake_slowdown",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def cpu_arm():
    """(kind, ref): the reference's own compiled statements (oracle/_ref) when present, else the port."""
    from oracle import pyoracle
    if pyoracle.ref_available():
        try:
            return "reference", pyoracle.Ref()
        except Exception as exc:  # noqa: BLE001 - a stale or unloadable build: fall back to the port
            print(f"[bench] oracle/_ref not usable ({exc!r}); timing the port", file=sys.stderr)
    return "port", None


def cpu_threads(ref) -> int:
    from oracle import pyoracle
    return ref.num_threads() if ref is not None else pyoracle.num_threads()


def gather_caches(case_np):
    """The contiguous fp16 caches [Hkv, len, D] that the reference's CPU path reads (its KVCache, src/llm/kv_cache.cpp),
    filled once from the paged pool by the addressing rule of metal_compute.h:853-861.  Cache state, built outside
    every timed region."""
    from granite_b200 import synth
    caches = []
    for b, n in enumerate(int(x) for x in case_np["seq_lens"]):
        pos = np.arange(n)
        rows = case_np["tables"][b, pos // synth.PAGE].astype(np.int64) * synth.PAGE + pos % synth.PAGE
        caches.append((np.ascontiguousarray(case_np["k_pool"][rows].transpose(1, 0, 2)),
                       np.ascontiguousarray(case_np["v_pool"][rows].transpose(1, 0, 2))))
    return caches


def cpu_decode_sample(case_np, caches, ref, repeats: int = 1):
    """Times Granite's CPU decode path on every sequence of `case_np` (caches from gather_caches): the
    whole-cache fp16 -> fp32 widening (transformer.mm:1753-1765) and the attention loop (:1779-1840, seq_q = 1),
    as its attention() does on every call.  Returns (bytes, seconds of widening + loop, seconds of the loop
    alone, sequences): best of `repeats`."""
    from oracle import pyoracle
    from granite_b200 import synth
    lens = case_np["seq_lens"]
    hkv, d, hq = case_np["num_kv_heads"], case_np["head_dim"], case_np["num_heads"]
    pages = int(((lens + synth.PAGE - 1) // synth.PAGE).sum())
    nbytes = int(lens.sum()) * hkv * d * 2 * 2 + pages * 4 + len(lens) * 4 + len(lens) * hq * d * 4 * 2
    scale = float(np.float32(1.0) / np.sqrt(np.float32(d)))
    best_all, best_loop = None, None
    for _ in range(repeats):
        t_all = t_loop = 0.0
        for b, n in enumerate(int(x) for x in lens):
            if n == 0:
                continue
            ck, cv = caches[b]
            t0 = time.perf_counter()
            if ref is not None:
                kf, vf = ref.attention_cache_widen(ck, cv, n)
            else:
                kf, vf = pyoracle.cache_to_fp32(ck, n), pyoracle.cache_to_fp32(cv, n)
            t1 = time.perf_counter()
            q = case_np["q"][b][None, None]
            if ref is not None:
                ref.attention_loop(q, kf, vf, n - 1, scale)
            else:
                pyoracle.attention(q, kf, vf, start_pos=n - 1, scale=scale)
            t2 = time.perf_counter()
            t_all += t2 - t0
            t_loop += t2 - t1
        best_all = t_all if best_all is None else min(best_all, t_all)
        best_loop = t_loop if best_loop is None else min(best_loop, t_loop)
    return nbytes, best_all, best_loop, len(lens)


def host_case_for_cpu(seed: int, cfg: dict, sel):
    """The sequences `sel` of the workload, rebuilt on the host with a compact pool that holds only
    their pages (the CPU arm never needs the other sequences' K/V)."""
    from granite_b200 import synth
    rng = np.random.default_rng(seed)
    lens_all = synth.draw_lengths(rng, cfg["batch"], cfg["len_lo"], cfg["len_hi"], cfg["dist"])
    lens = lens_all[np.asarray(sel)]
    case = synth.paged_case(seed, len(lens), 0, 0, cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"],
                            seq_lens=lens)
    return dict(q=case.q, k_pool=case.k_pool.view(np.uint16), v_pool=case.v_pool.view(np.uint16),
                tables=np.where(case.tables < 0, 0, case.tables), seq_lens=case.seq_lens,
                num_heads=case.num_heads, num_kv_heads=case.num_kv_heads, head_dim=case.head_dim)


def workload_lengths(cfg: dict) -> np.ndarray:
    from granite_b200 import synth
    return synth.draw_lengths(np.random.default_rng(cfg["seed"]), cfg["batch"], cfg["len_lo"], cfg["len_hi"],
                              cfg["dist"])


def run_reference(args):
    """Reference arm: CPU attention on the host cores.  Each step is a bounded sample of the
    workload - whole sequences taken from every 16th position - sized from a calibration run so
    that all steps together take about two minutes."""
    from granite_b200 import synth
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    kind, ref = cpu_arm()
    cfg = dict(synth.CONFIGS[WORKLOAD])
    lens_all = workload_lengths(cfg)
    shortest = int(np.argmin(lens_all))
    calib = host_case_for_cpu(cfg["seed"], cfg, [shortest])
    _, secs, _, _ = cpu_decode_sample(calib, gather_caches(calib), ref)
    tok_per_s = float(lens_all[shortest]) / secs
    budget_tokens = tok_per_s * 120.0 / max(args.steps + args.warmup, 1)
    sel, tokens = [], 0
    for b in range(0, cfg["batch"], 16):
        if tokens + int(lens_all[b]) <= budget_tokens:
            sel.append(b)
            tokens += int(lens_all[b])
    if not sel:
        sel = [shortest]
    hc = host_case_for_cpu(cfg["seed"], cfg, sel)
    caches = gather_caches(hc)  # cache state, like the K/V pages resident in HBM on the GPU side
    for _ in range(args.warmup):
        cpu_decode_sample(hc, caches, ref)
    t0 = time.perf_counter()
    nbytes, loop_s = 0, 0.0
    for _ in range(args.steps):
        b, _, t_loop, _ = cpu_decode_sample(hc, caches, ref)
        nbytes += b
        loop_s += t_loop
    dt = time.perf_counter() - t0
    value = nbytes / dt / 1e9
    cores = cpu_threads(ref)
    sample = (f"sequences {sel} of the workload's {cfg['batch']} ({int(hc['seq_lens'].sum())} tokens) per step")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample, "page": 16, "num_heads": cfg["num_heads"],
                   "num_kv_heads": cfg["num_kv_heads"], "head_dim": cfg["head_dim"]},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample,
                         "value_loop_only": nbytes / loop_s / 1e9,
                         "note": "value: the reference's serial whole-cache fp16->fp32 widening + the attention loop on all "
                                 "host threads, as its CPU path runs each call; value_loop_only: the loop alone"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)
    return 0


def cpu_prefill_sample(ref, kind: str, seq: int, d: int, heads: int = 4):
    """The reference loop (transformer.mm:1779-1840, causal from position 0) on `heads` query heads of one KV head
    of the prefill configuration; returns a cpu_baseline object in TFLOP/s."""
    from oracle import pyoracle
    rng = np.random.default_rng(1002)
    q = rng.standard_normal((1, seq, heads, d), dtype=np.float32).astype(np.float16).astype(np.float32)
    k = rng.standard_normal((seq, 1, d), dtype=np.float32).astype(np.float16).astype(np.float32)
    v = rng.standard_normal((seq, 1, d), dtype=np.float32).astype(np.float16).astype(np.float32)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(d)))
    best = None
    for _ in range(3):
        t0 = time.perf_counter()
        if ref is not None:
            ref.attention_loop(q, k, v, 0, scale)
        else:
            pyoracle.attention(q, k, v, start_pos=0, scale=scale)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    flops = 4 * d * heads * seq * (seq + 1) // 2
    return {"value": flops / best / 1e12, "unit": "TFLOP/s", "cores": cpu_threads(ref), "kind": kind,
            "sample": f"{heads} query heads of one KV head, all {seq} tokens, best of 3, {best:.2f} s each; "
                      "the loop computes the masked half too (it tests k_pos > abs_pos inside), credited flops are the unmasked half"}


def cpu_tree_sample(ref, kind: str, n: int, prefix: int, d: int, parents, heads: int = 8, hkv: int = 2):
    """The reference tree loop (transformer.mm:2044-2126) on one sequence of the tree configuration with
    `heads` query heads over `hkv` KV heads."""
    from oracle import pyoracle
    rng = np.random.default_rng(1004)
    q = rng.standard_normal((1, n, heads, d), dtype=np.float32).astype(np.float16).astype(np.float32)
    kp = rng.standard_normal((prefix, hkv, d), dtype=np.float32).astype(np.float16).astype(np.float32)
    vp = rng.standard_normal((prefix, hkv, d), dtype=np.float32).astype(np.float16).astype(np.float32)
    kt = rng.standard_normal((1, n, hkv, d), dtype=np.float32).astype(np.float16).astype(np.float32)
    vt = rng.standard_normal((1, n, hkv, d), dtype=np.float32).astype(np.float16).astype(np.float32)
    scale = float(np.float32(1.0) / np.sqrt(np.float32(d)))
    best = None
    for _ in range(3):
        t0 = time.perf_counter()
        if ref is not None:
            ref.attention_tree_loop(q, kp, vp, kt, vt, parents, scale)
        else:
            pyoracle.attention_tree(q, kp, vp, kt, vt, parents, scale=scale)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    visible = 0
    for i in range(n):
        c, depth = parents[i], 1
        while c >= 0:
            depth += 1
            c = parents[c]
        visible += depth
    flops = 4 * d * heads * (n * prefix + visible)
    return {"value": flops / best / 1e12, "unit": "TFLOP/s", "cores": cpu_threads(ref), "kind": kind,
            "sample": f"one sequence ({prefix}-token prefix + {n}-node tree), {heads} query heads over {hkv} KV heads, "
                      f"best of 3, {best:.2f} s each"}


def tensor_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return 1590.0, 1400.0, "fallback"


def hold_queue(dev, ms: float = 8.0):
    """Keeps the GPU busy for a few milliseconds so that the launches enqueued next pile up behind
    it: short kernels are then timed back to back, without the idle-queue launch latency that a
    host-bound enqueue loop would add to every event pair."""
    import torch
    torch.cuda._sleep(int(ms * 1.9e6))


def region_ms_per_launch(dev, step, reps: int, clocks: dict | None = None) -> float:
    """Average duration of `reps` launches issued back to back behind a queue-holding kernel, one
    CUDA event pair around the whole region on the launching stream (an event pair around every
    single launch adds the front-end's gap between dependent operations to each of them).  With
    `clocks` given, SM clock and throttle reasons are sampled during the region and stored there."""
    import torch
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    sampler = ClockSampler(dev.index if dev.index is not None else 0, 0.001) if clocks is not None else None
    hold_queue(dev)
    if sampler:
        sampler.start()
    e0.record()
    for i in range(reps):
        step(i)
    e1.record()
    e1.synchronize()
    if sampler:
        clocks.update(sampler.stop())
    return e0.elapsed_time(e1) / reps


def measure_prefill_by_length(compute, dev, reps: int = 0):
    """The prefill kernel at 2048 ... 16384 tokens (Hq 32, Hkv 8, D 128, fp16 in/out): the benchmark's 2048-token
    launch spends a third of its 50 microseconds on start-up, drain and item boundaries (3.5 work items per CTA);
    longer prompts show the pipeline's own rate.  Every length is timed as a burst of 10-30 ms (a loop of half a
    second settles under the power cap: 764 TFLOP/s at 1462 MHz for 16384 tokens, 0.56 of the sustained peak)."""
    import torch
    hq, hkv, d = 32, 8, 128
    gen = torch.Generator(device=dev)
    gen.manual_seed(2002)
    burst, sustained, kind = tensor_peak()
    rows = []
    for seq in (2048, 4096, 8192, 16384):
        q = torch.randn((seq, hq, d), device=dev, generator=gen).half()
        k = torch.randn((hkv, seq, d), device=dev, generator=gen).half()
        v = torch.randn((hkv, seq, d), device=dev, generator=gen).half()
        out = torch.zeros((seq, hq, d), device=dev, dtype=torch.float16)

        def step(i):
            compute.multihead_attention(q, k, v, out, hq, hkv, seq, seq, d, 1.0 / float(np.sqrt(d)), seq, q_dtype=1, out_dtype=1)

        for i in range(3):
            step(i)
        compute.sync()
        n = max(10, min(200, int(200 * (2048 / seq) ** 2)))  # about 10-30 ms per length: bursts, like the 2048-token figure
        clocks = {}
        ms = region_ms_per_launch(dev, step, n, clocks)
        flops = 4 * d * hq * seq * (seq + 1) // 2
        tf = flops / ms / 1e9
        nb = seq // kT_ROWS
        rows.append({"seq": seq, "kernel_ms": ms, "launches": n, "tflops": tf, "frac": tf / burst, "frac_of_sustained": tf / sustained,
                     "kv_steps_per_cta": hq * nb * (nb + 1) / 2 / compute.sm_count, "items_per_cta": hq * nb / compute.sm_count,
                     "sm_mhz": clocks.get("sm_mhz"), "reasons": clocks.get("reasons")})
        del q, k, v, out
    return {"workload": "prefill_causal_by_length", "kernel": "prefill_causal_fa", "bound": "tensor", "peak_tflops": burst,
            "peak_tflops_sustained": sustained, "peak_kind": kind, "lengths": rows}


def e2e_ms_per_call(dev, call, reps: int = 30) -> float:
    """Average duration of `call` (host buffers in, result out, sync inside) over `reps` calls, CUDA events."""
    import torch
    for _ in range(3):
        call()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    e0.record()
    for _ in range(reps):
        call()
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) / reps


def measure_prefill(compute, dev, reps: int = 200, with_cpu: bool = True):
    """Causal prefill, seq 2048, Hq 32, Hkv 8, D 128, fp16 in/out (the prefill benchmark configuration); the
    kernel's own event-timed duration, rotating over 4 input sets."""
    import torch
    from granite_b200 import synth
    cfg = synth.CONFIGS["prefill_causal_s2048"]
    seq, hq, hkv, d = cfg["seq"], cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"]
    gen = torch.Generator(device=dev)
    gen.manual_seed(cfg["seed"])
    sets = [(torch.randn((seq, hq, d), device=dev, generator=gen).half(),
             torch.randn((hkv, seq, d), device=dev, generator=gen).half(),
             torch.randn((hkv, seq, d), device=dev, generator=gen).half()) for _ in range(4)]
    out = torch.zeros((seq, hq, d), device=dev, dtype=torch.float16)

    def step(i):
        q, k, v = sets[i % 4]
        compute.multihead_attention(q, k, v, out, hq, hkv, seq, seq, d, 1.0 / float(np.sqrt(d)), seq,
                                    q_dtype=1, out_dtype=1)

    for i in range(5):
        step(i)
    compute.sync()
    compute.enable_kernel_timing(True)
    compute.reset_kernel_timing()
    hold_queue(dev)
    for i in range(reps):
        step(i)
    st = compute.get_kernel_timing_stats()
    compute.enable_kernel_timing(False)
    ms_each = st["prefill_causal_fa"][0] / st["prefill_causal_fa"][1]
    clocks = {}
    ms = region_ms_per_launch(dev, step, reps, clocks)
    flops = 4 * d * hq * seq * (seq + 1) // 2
    burst, sustained, kind = tensor_peak()
    tf = flops / ms / 1e9
    # end to end through the C ABI: host Q/K/V (pinned, fp16) copied in, output copied out, sync per call
    q_h, k_h, v_h = (t.cpu().pin_memory() for t in sets[0])
    out_h = torch.empty((seq, hq, d), dtype=torch.float16).pin_memory()
    q_d, k_d, v_d = (torch.empty_like(t) for t in sets[0])

    def e2e_call():
        compute.write_buffer(q_d, q_h, q_h.numel() * 2)
        compute.write_buffer(k_d, k_h, k_h.numel() * 2)
        compute.write_buffer(v_d, v_h, v_h.numel() * 2)
        compute.multihead_attention(q_d, k_d, v_d, out, hq, hkv, seq, seq, d, 1.0 / float(np.sqrt(d)), seq,
                                    q_dtype=1, out_dtype=1)
        compute.read_buffer(out_h, out, out_h.numel() * 2)
        compute.sync()

    e2e_ms = e2e_ms_per_call(dev, e2e_call)
    # the pipe executes more than is credited: P as hi + lo (1.5x) and the diagonal tile in full (+6 %)
    executed = 1.5 * (1.0 + (kT_ROWS - 1) / (seq + 1))
    res = {"workload": "prefill_causal_s2048", "kernel": "prefill_causal_fa", "kernel_ms": ms,
           "kernel_ms_timed_singly": ms_each, "launches": reps, "clocks": clocks,
           "algorithmic_flops": flops, "tflops": tf, "bound": "tensor", "peak_tflops": burst,
           "frac": tf / burst, "frac_of_sustained": tf / sustained, "peak_kind": kind,
           "frac_executed": tf * executed / burst,
           "e2e": {"value": flops / e2e_ms / 1e9, "unit": "TFLOP/s", "ms_per_call": e2e_ms,
                   "h2d_bytes_per_step": (q_h.numel() + k_h.numel() + v_h.numel()) * 2, "d2h_bytes_per_step": out_h.numel() * 2},
           "note": "unmasked half of the causal square counted only; P enters the PV product as fp16 hi+lo "
                   "(two MMAs) to keep the CPU path's precision, which `frac` does not credit; `frac_executed` counts "
                   "what the tensor pipe runs (hi + lo, and the whole diagonal tile)"}
    if with_cpu:
        ckind, ref = cpu_arm()
        res["cpu_baseline"] = cpu_prefill_sample(ref, ckind, seq, d)
    return res


def measure_tree(compute, dev, reps: int = 200, nodes: int = 0, with_cpu: bool = True):
    """Tree verification: 16 sequences x (4096-token paged prefix + 64-node tree), Hq 32, Hkv 8
    (the tree-verification benchmark configuration); rotates over 3 pools (268 MB of prefix K/V each, larger than L2)."""
    import torch
    from granite_b200 import synth
    cfg = synth.CONFIGS["tree_verify_b16"]
    batch, n, hq, hkv, L, d = cfg["batch"], nodes or cfg["nodes"], cfg["num_heads"], cfg["num_kv_heads"], cfg["prefix"], 128
    cases = [synth.paged_case(cfg["seed"] + i, batch, 0, 0, hq, hkv, seq_lens=np.full(batch, L, np.int32), device=dev)
             for i in range(3)]
    tables = [torch.from_numpy(c.tables).to(dev) for c in cases]
    gen = torch.Generator(device=dev)
    gen.manual_seed(cfg["seed"] + 500)
    q = torch.randn((batch, hq, n, d), device=dev, generator=gen).half()
    kt = torch.randn((batch, hkv, n, d), device=dev, generator=gen).half()
    vt = torch.randn((batch, hkv, n, d), device=dev, generator=gen).half()
    parents_np = np.stack([synth.tree_parents(cfg["seed"] + 500 + b, n, cfg["max_children"], cfg["max_depth"])
                           for b in range(batch)])
    parents = torch.from_numpy(parents_np).to(dev)
    out = torch.zeros((batch, hq, n, d), device=dev)

    def step(i):
        c = cases[i % 3]
        compute.attention_tree(q, c.k_pool, c.v_pool, kt, vt, parents, out, hq, hkv, n, L, d,
                               1.0 / float(np.sqrt(d)), batch_size=batch, block_tables=tables[i % 3],
                               max_blocks_per_seq=c.max_blocks, num_blocks=c.num_blocks, q_dtype=1)

    for i in range(4):
        step(i)
    compute.sync()
    compute.enable_kernel_timing(True)
    compute.reset_kernel_timing()
    hold_queue(dev)
    for i in range(reps):
        step(i)
    st = compute.get_kernel_timing_stats()
    compute.enable_kernel_timing(False)
    ms_each = st["tree_verify"][0] / st["tree_verify"][1]
    clocks = {}
    ms = region_ms_per_launch(dev, step, reps, clocks)
    visible = 0
    for b in range(batch):  # self + ancestors of every node
        for i in range(n):
            c, depth = parents_np[b, i], 1
            while c >= 0:
                depth += 1
                c = parents_np[b, c]
            visible += depth
    flops = 4 * d * hq * (batch * n * L + visible)
    nbytes = batch * L * hkv * d * 4 + batch * (L // 16) * 4 + 2 * batch * hkv * n * d * 2 + batch * hq * n * d * (2 + 4)
    burst, sustained, kind = tensor_peak()
    hbm, hkind = measured_peaks()
    tf = flops / ms / 1e9
    gbs = nbytes / ms / 1e6
    # end to end through the C ABI: host queries, tree K/V and parents in, output out, sync per call; the
    # committed prefix is cache state and stays in the paged pool
    q_h, kt_h, vt_h, par_h = q.cpu().pin_memory(), kt.cpu().pin_memory(), vt.cpu().pin_memory(), parents.cpu().pin_memory()
    out_h = torch.empty((batch, hq, n, d), dtype=torch.float32).pin_memory()
    q_e, kt_e, vt_e, par_e = torch.empty_like(q), torch.empty_like(kt), torch.empty_like(vt), torch.empty_like(parents)

    def e2e_call():
        compute.write_buffer(q_e, q_h, q_h.numel() * 2)
        compute.write_buffer(kt_e, kt_h, kt_h.numel() * 2)
        compute.write_buffer(vt_e, vt_h, vt_h.numel() * 2)
        compute.write_buffer(par_e, par_h, par_h.numel() * 4)
        c = cases[0]
        compute.attention_tree(q_e, c.k_pool, c.v_pool, kt_e, vt_e, par_e, out, hq, hkv, n, L, d,
                               1.0 / float(np.sqrt(d)), batch_size=batch, block_tables=tables[0],
                               max_blocks_per_seq=c.max_blocks, num_blocks=c.num_blocks, q_dtype=1)
        compute.read_buffer(out_h, out, out_h.numel() * 4)
        compute.sync()

    e2e_ms = e2e_ms_per_call(dev, e2e_call)
    res = {"workload": "tree_verify_b16" if n == cfg["nodes"] else f"tree_verify_b16_n{n}", "kernel": "tree_verify", "kernel_ms": ms,
           "kernel_ms_timed_singly": ms_each, "launches": reps, "clocks": clocks,
           "algorithmic_flops": flops, "algorithmic_bytes": nbytes, "tflops": tf, "gbs": gbs,
           "bound": "ridge (256 flop/B): both fractions reported", "frac_tensor": tf / burst,
           "frac_hbm": gbs / hbm, "peak_tflops": burst, "peak_gbs": hbm, "peak_kind": kind,
           "e2e": {"value": flops / e2e_ms / 1e9, "unit": "TFLOP/s", "ms_per_call": e2e_ms,
                   "h2d_bytes_per_step": (q_h.numel() + kt_h.numel() + vt_h.numel()) * 2 + par_h.numel() * 4,
                   "d2h_bytes_per_step": out_h.numel() * 4}}
    if with_cpu and n == cfg["nodes"]:
        ckind, ref = cpu_arm()
        res["cpu_baseline"] = cpu_tree_sample(ref, ckind, n, L, d, parents_np[0])
    return res


def measure_decode_step_write(compute, dev, reps: int = 200):
    """The cache write of one decode step for 64 sequences (Hq 32, Hkv 8, D 128): RoPE on Q and K plus
    the paged K/V store, as one fused launch and as the reference's two calls
    (rope_multihead, then paged_kv_cache_append; src/llm/transformer.mm:2975-2986)."""
    import torch
    from granite_b200 import synth
    batch, hq, hkv, d = 64, 32, 8, 128
    case = synth.paged_case(2024, batch, 1024, 8192, hq, hkv, d, device=dev, spare_blocks=batch)
    tables = torch.from_numpy(np.where(case.tables < 0, 0, case.tables).astype(np.int32)).to(dev)
    positions = torch.from_numpy((case.seq_lens - 1).astype(np.int32)).to(dev)
    max_seq = 8192
    cos_p, sin_p = compute.rope_table_create(max_seq, d)
    gen = torch.Generator(device=dev)
    gen.manual_seed(7)
    q = torch.randn((batch, 1, hq, d), device=dev, generator=gen)
    k = torch.randn((batch, 1, hkv, d), device=dev, generator=gen)
    v = torch.randn((batch, 1, hkv, d), device=dev, generator=gen)

    def fused(i):
        compute.rope_paged_kv_cache_append(q, k, v, cos_p, sin_p, case.k_pool, case.v_pool, tables, positions, batch, 1,
                                           hq, hkv, d, synth.PAGE, case.max_blocks, case.num_blocks, max_seq)

    def unfused(i):
        # positions differ per sequence, so the unfused pair rotates at one common position; the
        # bytes moved are the same, which is what is timed
        compute.rope_multihead(q, k, hq, hkv, batch, d, 1000, cos_p, sin_p, max_seq)
        compute.paged_kv_cache_append(k, v, case.k_pool, case.v_pool, tables, hkv, d, 0, 0, synth.PAGE,
                                      num_blocks=case.num_blocks, table_len=case.max_blocks, positions=positions,
                                      batch_size=batch)

    for i in range(5):
        fused(i)
        unfused(i)
    compute.sync()
    ms_fused = region_ms_per_launch(dev, fused, reps)
    ms_unfused = region_ms_per_launch(dev, unfused, reps)
    compute.destroy_buffer(cos_p)
    compute.destroy_buffer(sin_p)
    nbytes = batch * (hq * d * 4 * 2 + 2 * hkv * d * 4 + 2 * hkv * d * 2) + batch * 8
    return {"workload": "decode_step_cache_write_b64", "kernel": "rope_paged_kv_append", "kernel_ms": ms_fused,
            "unfused_two_launch_ms": ms_unfused, "launches": reps, "algorithmic_bytes": nbytes,
            "bound": "launch latency (2.9 MB moved)", "gbs": nbytes / ms_fused / 1e6}


def measure_paged_prefill(compute, dev, reps: int = 200):
    """The prefill configuration (2048 tokens, Hq 32, Hkv 8) with K/V read through the block table
    instead of a contiguous cache: what paging costs the tensor-bound kernel."""
    import torch
    from granite_b200 import synth
    seq, hq, hkv, d = 2048, 32, 8, 128
    cases = [synth.paged_case(4000 + i, 1, 0, 0, hq, hkv, d, seq_lens=np.array([seq], np.int32), device=dev, spare_blocks=512)
             for i in range(4)]
    tables = [torch.from_numpy(np.where(c.tables[0] < 0, 0, c.tables[0]).astype(np.int32)).to(dev) for c in cases]
    gen = torch.Generator(device=dev)
    gen.manual_seed(11)
    qs = [torch.randn((seq, hq, d), device=dev, generator=gen).half() for _ in range(4)]
    out = torch.zeros((seq, hq, d), device=dev, dtype=torch.float16)

    def step(i):
        c = cases[i % 4]
        compute.paged_prefill_attention(qs[i % 4], c.k_pool, c.v_pool, tables[i % 4], out, hq, hkv, seq, 0, d, synth.PAGE,
                                        c.max_blocks, c.num_blocks, 1.0 / float(np.sqrt(d)), q_dtype=1, out_dtype=1)

    for i in range(5):
        step(i)
    compute.sync()
    ms = region_ms_per_launch(dev, step, reps)
    flops = 4 * d * hq * seq * (seq + 1) // 2
    burst, sustained, kind = tensor_peak()
    tf = flops / ms / 1e9
    return {"workload": "paged_prefill_s2048", "kernel": "paged_prefill_fa", "kernel_ms": ms, "launches": reps,
            "algorithmic_flops": flops, "tflops": tf, "bound": "tensor", "peak_tflops": burst, "frac": tf / burst,
            "frac_of_sustained": tf / sustained, "peak_kind": kind}


def measure_single_decode(compute, dev, reps: int = 200):
    """One sequence, one new token, 512 tokens of contiguous fp16 cache (Hq 32, Hkv 8, D 128): the
    reference's own CPU-runnable case, and what single-user decoding looks like.  2 MB of traffic: the figure is
    launch latency, not bandwidth."""
    import torch
    hq, hkv, d, ctx = 32, 8, 128, 512
    gen = torch.Generator(device=dev)
    gen.manual_seed(1001)
    q = torch.randn((hq, d), device=dev, generator=gen)
    k = torch.randn((hkv, ctx, d), device=dev, generator=gen).half()
    v = torch.randn((hkv, ctx, d), device=dev, generator=gen).half()
    out = torch.zeros((hq, d), device=dev)

    def step(i):
        compute.multihead_attention(q, k, v, out, hq, hkv, 1, ctx, d, 1.0 / float(np.sqrt(d)), ctx)

    for i in range(5):
        step(i)
    compute.sync()
    ms = region_ms_per_launch(dev, step, reps)
    # the same call captured once into a CUDA graph and replayed (what a serving loop would do)
    import granite_b200 as g
    side = torch.cuda.Stream(device=dev)
    side_compute = g.CudaCompute(dev.index, side.cuda_stream)

    def side_step():
        side_compute.multihead_attention(q, k, v, out, hq, hkv, 1, ctx, d, 1.0 / float(np.sqrt(d)), ctx)

    torch.cuda.synchronize(dev)
    with torch.cuda.stream(side):
        side_step()
    side_compute.sync()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        side_step()
    torch.cuda.synchronize(dev)
    ms_graph = region_ms_per_launch(dev, lambda i: graph.replay(), reps)
    side_compute.shutdown()
    nbytes = 2 * hkv * ctx * d * 2 + hq * d * 4 * 2
    return {"workload": "decode_contiguous_ctx512", "kernels": "contiguous_decode_direct (one launch: a few CTAs per KV head share the pages, the last to finish combines their partials)",
            "call_ms": ms, "graph_replay_ms": ms_graph, "launches": reps, "algorithmic_bytes": nbytes,
            "bound": "launch latency (2 MB moved)"}


def measure_tree16(compute, dev, reps: int = 200):
    """The tree configuration with 16-node trees: four query heads share a 128-row tile."""
    return measure_tree(compute, dev, reps, nodes=16, with_cpu=False)


def measure_generic(compute, dev, reps: int = 50):
    """What the plain fp32 kernel (shapes outside the tuned kernels' tiling) costs against the tuned kernels on
    the nearest tuned shape, and the operator-form kernel on a mid-sized tensor.  Side measurement."""
    import ctypes as C
    import torch
    import granite_b200 as g
    from granite_b200 import synth
    out = {}
    # decode: 16 sequences, lengths uniform [1024, 8192], Hq 32, Hkv 8: head_dim 128 (tuned) against 96 (plain)
    for d in (128, 96):
        case = synth.paged_case(3003, 16, 1024, 8192, 32, 8, d, device=dev)
        tables = torch.from_numpy(case.tables).to(dev)
        lens = torch.from_numpy(case.seq_lens).to(dev)
        o = torch.zeros((16, 32, d), device=dev)

        def step(i):
            compute.batched_paged_attention_decode(case.q, case.k_pool, case.v_pool, tables, lens, o, 16, 32, 8, d, synth.PAGE,
                                                   case.max_blocks, 1.0 / float(np.sqrt(d)), num_blocks=case.num_blocks)
        for i in range(3):
            step(i)
        compute.sync()
        ms = region_ms_per_launch(dev, step, reps)
        out[f"decode_head_dim_{d}"] = {"ms": ms, "gbs": case.algorithmic_bytes() / ms / 1e6,
                                       "kernel": "paged_decode_splitkv" if d == 128 else "generic_attention"}
    out["decode_slowdown_of_plain_kernel"] = out["decode_head_dim_128"]["gbs"] / out["decode_head_dim_96"]["gbs"]
    # prefill: 1024 tokens, Hq 8, Hkv 2, fp16 in/out
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    for d in (128, 96):
        seq, hq, hkv = 1024, 8, 2
        q = torch.randn((seq, hq, d), device=dev, generator=gen).half()
        k = torch.randn((hkv, seq, d), device=dev, generator=gen).half()
        v = torch.randn((hkv, seq, d), device=dev, generator=gen).half()
        o = torch.zeros((seq, hq, d), device=dev, dtype=torch.float16)

        def step(i):
            compute.multihead_attention(q, k, v, o, hq, hkv, seq, seq, d, 1.0 / float(np.sqrt(d)), seq, q_dtype=1, out_dtype=1)
        for i in range(3):
            step(i)
        compute.sync()
        ms = region_ms_per_launch(dev, step, reps)
        flops = 4 * d * hq * seq * (seq + 1) // 2
        out[f"prefill_head_dim_{d}"] = {"ms": ms, "tflops": flops / ms / 1e9,
                                        "kernel": "prefill_causal_fa" if d == 128 else "generic_attention"}
    out["prefill_slowdown_of_plain_kernel"] = out["prefill_head_dim_128"]["tflops"] / out["prefill_head_dim_96"]["tflops"]
    # operator form (one head): fp16 [T, D] layout with the causal limit, 256 queries over 4096 keys, D 128
    from granite_b200 import capi

    class SdpaArgs(C.Structure):
        _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("output", C.c_void_p), ("seq_q", C.c_uint32),
                    ("seq_kv", C.c_uint32), ("head_dim", C.c_uint32), ("dtype", C.c_uint32), ("k_transposed", C.c_uint32),
                    ("causal", C.c_uint32), ("start_pos", C.c_uint32), ("scale", C.c_float)]
    sq, skv, d = 256, 4096, 128
    q = torch.randn((sq, d), device=dev, generator=gen).half()
    k = torch.randn((skv, d), device=dev, generator=gen).half()
    v = torch.randn((skv, d), device=dev, generator=gen).half()
    o = torch.zeros((sq, d), device=dev, dtype=torch.float16)
    a = SdpaArgs(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), sq, skv, d, 1, 0, 1, skv - sq, 1.0 / float(np.sqrt(d)))
    g.lib.granite_cuda_sdpa.argtypes = [C.c_void_p, C.POINTER(SdpaArgs)]

    def step(i):
        capi.check(g.lib.granite_cuda_sdpa(compute.handle, C.byref(a)))
    for i in range(3):
        step(i)
    compute.sync()
    ms = region_ms_per_launch(dev, step, reps)
    out["sdpa_operator_256x4096x128"] = {"ms": ms, "tflops": 4 * d * sq * skv / ms / 1e9, "kernel": "sdpa_operator"}
    return out


class Gather:
    """Buffers every rank's output rows are gathered into: symmetric memory whose peer addresses the
    decode kernel stores to directly, or - where that cannot be set up on every rank - plain buffers
    filled by an NCCL all-gather after each step."""

    def __init__(self, dist, dev, world: int, shape):
        import torch
        self.dist, self.world = dist, world
        self.bufs, self.peer_ptrs = None, None
        self.mode = "none"
        if world == 1:
            return
        try:
            import torch.distributed._symmetric_memory as symm
            self.bufs = [symm.empty(shape, dtype=torch.float32, device=dev) for _ in range(2)]
            for t in self.bufs:
                t.zero_()  # padding rows (ranks own different numbers of sequences) compare equal
            handles = [symm.rendezvous(t, dist.group.WORLD) for t in self.bufs]
            self.peer_ptrs = [[int(p) for p in h.buffer_ptrs] for h in handles]
            self.mode = "rows stored to every rank by the decode kernel (peer stores over NVLink, symmetric memory)"
        except Exception as exc:  # noqa: BLE001 - any failure means: use the collective library
            print(f"[bench] symmetric memory unavailable ({exc!r}); gathering with NCCL", file=sys.stderr)
            self.peer_ptrs = None
        flags = torch.tensor([1 if self.peer_ptrs else 0], device=dev)
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)  # all ranks take the same route
        if int(flags.item()) == 0:
            self.bufs = [torch.zeros(shape, device=dev) for _ in range(2)]
            self.peer_ptrs, self.mode = None, "NCCL all-gather per step"


def timed_regions(dev, dist, world: int, step, steps: int, min_regions: int = 5, min_total_s: float = 0.5,
                  max_regions: int = 40, clock_index=None):
    """Times regions of exactly `steps` calls of step(i), each bracketed by a barrier and a device
    synchronize on both sides, CUDA events on the current stream, maximum over the ranks per region;
    regions are repeated until there are `min_regions` of them and they cover `min_total_s`.
    Returns (median ms per step, best ms per step, regions, clock record)."""
    import torch

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    sampler = ClockSampler(clock_index, 0.002) if clock_index is not None else None
    per_step, total = [], 0.0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    if sampler:
        sampler.start()
    while len(per_step) < max_regions and (len(per_step) < min_regions or total < min_total_s):
        barrier()
        e0.record()
        for i in range(steps):
            step(i)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            # every rank must take the same number of regions: the decision uses the maximum
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        per_step.append(ms / steps)
        total += ms * 1e-3
    clocks = sampler.stop() if sampler else None
    return float(np.median(per_step)), float(min(per_step)), len(per_step), clocks


def measure_long_context(compute, dev, dist, world: int, rank: int, steps: int = 8):
    """The long-context configuration as ONE fixed problem split over the ranks (strong scaling): 256
    sequences, lengths log-uniform in [4096, 131072], Hq 64, Hkv 8, D 128, 38.4 GB of K/V in all.
    Split by sequence (longest first onto the least loaded rank) and, when the KV heads divide among the
    ranks, by KV head (every rank holds all sequences and Hkv / ranks heads; perfectly balanced); both are
    timed with the output gather fused into the decode kernel, and the one the plan predicts faster is
    the figure.  T(1) / (N T(N)) over runs at N = 1, 2, 4, 8 is the scaling efficiency on the identical problem."""
    import torch
    from granite_b200 import sharding, synth
    cfg = dict(synth.CONFIGS["paged_decode_long_b256"])
    lens_all = workload_lengths(cfg)
    B, Hq, Hkv, D = cfg["batch"], cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"]
    scale = 1.0 / float(np.sqrt(D))
    pages_all = int(((lens_all.astype(np.int64) + synth.PAGE - 1) // synth.PAGE).sum())
    total_bytes = int(lens_all.astype(np.int64).sum()) * Hkv * D * 4 + pages_all * 4 + B * 4 + B * Hq * D * 8
    res = {"workload": "paged_decode_long_b256", "scaling": "strong", "n_gpus": world, "sequences": B,
           "tokens": int(lens_all.astype(np.int64).sum()), "algorithmic_bytes": total_bytes, "steps_per_region": steps,
           "predicted_split": sharding.choose_split(lens_all, Hkv, world)}

    def run(split: str):
        if split == "sequence":
            plan = sharding.lpt_assign(lens_all, world)
            mine = plan[rank]
            case = synth.paged_case(cfg["seed"] + 7919 * rank, len(mine), 0, 0, Hq, Hkv, D, seq_lens=lens_all[mine], device=dev)
            rows = sharding.padded_rows(plan)
            n_q, n_kv, q0, gshape = Hq, Hkv, 0, (world * rows, Hq, D)
            row0, extra = rank * rows, {"lpt_imbalance": sharding.imbalance(lens_all, plan)}
        else:
            kv0, n_kv, q0, n_q = sharding.head_split(Hq, Hkv, world)[rank]
            # every rank: all sequences, the same seeded tables, its own heads' K/V and queries
            case = synth.paged_case(cfg["seed"], B, 0, 0, n_q, n_kv, D, seq_lens=lens_all, device=dev)
            rows, gshape, row0, extra = B, (B, Hq, D), 0, {"kv_heads_per_gpu": n_kv}
        nb = case.batch
        tables = torch.from_numpy(case.tables).to(dev)
        lens = torch.from_numpy(case.seq_lens).to(dev)
        outs = [torch.zeros((rows, n_q, D), device=dev) for _ in range(2)]
        g = Gather(dist, dev, world, gshape)

        def step(i):
            kw = {}
            if g.peer_ptrs is not None:
                kw = dict(gather_ptrs=g.peer_ptrs[i & 1], gather_row_offset=row0)
                if split == "kv_head":
                    kw.update(gather_num_heads=Hq, gather_head_offset=q0)
            compute.batched_paged_attention_decode(case.q, case.k_pool, case.v_pool, tables, lens, outs[i & 1], nb, n_q,
                                                   n_kv, D, synth.PAGE, case.max_blocks, scale, num_blocks=case.num_blocks, **kw)
            if world > 1 and g.peer_ptrs is None:
                dist.all_gather_into_tensor(g.bufs[i & 1].view(world, -1), outs[i & 1].view(1, -1), async_op=True).wait()

        for i in range(3):
            step(i)
        med, best, regions, _ = timed_regions(dev, dist, world, step, steps, min_regions=5, min_total_s=0.25, max_regions=12)
        ok = None
        if world > 1 and g.peer_ptrs is not None:
            last = (steps - 1) & 1
            parts = torch.empty((world,) + tuple(outs[last].shape), device=dev)
            dist.all_gather_into_tensor(parts.view(world, -1), outs[last].view(1, -1))
            expect = parts.view(world * rows, Hq, D) if split == "sequence" else \
                parts.permute(1, 0, 2, 3).reshape(B, Hq, D)
            ok = bool(torch.equal(expect, g.bufs[last]))
        out = {"ms_per_step": med, "ms_per_step_best": best, "regions": regions, "gbs": total_bytes / med / 1e6,
               "gather": g.mode, **({"gather_verified": ok} if ok is not None else {}), **extra,
               "kv_bytes_this_gpu": int(case.total_tokens) * n_kv * D * 4}
        del case, tables, lens, outs, g
        torch.cuda.empty_cache()
        return out

    res["by_sequence"] = run("sequence")
    if world > 1 and sharding.head_split(Hq, Hkv, world) is not None:
        res["by_kv_head"] = run("kv_head")
    chosen = "by_kv_head" if res["predicted_split"] == "kv_head" and "by_kv_head" in res else "by_sequence"
    res["split"] = chosen
    res["ms_per_step"] = res[chosen]["ms_per_step"]
    res["value"] = res[chosen]["gbs"]
    res["unit"] = UNIT
    hbm, _ = measured_peaks()
    res["hbm_frac_of_measured_peak"] = res["value"] / world / hbm
    return res


SECONDARY = {"prefill_lengths": measure_prefill_by_length, "generic": measure_generic, "single_decode": measure_single_decode, "tree16": measure_tree16, "prefill": measure_prefill, "tree": measure_tree, "step_write": measure_decode_step_write,
             "paged_prefill": measure_paged_prefill}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="granite_b200")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default=WORKLOAD, choices=[WORKLOAD, "paged_decode_long_b256"],
                    help="paged_decode_long_b256: 256 sequences, log-uniform [4096, 131072], Hq 64, sharded "
                         "across the ranks by sequence (strong scaling); not the default benchmark line")
    ap.add_argument("--only", default="", choices=["", "prefill", "prefill_lengths", "tree", "tree16", "step_write", "paged_prefill", "single_decode", "generic"],
                    help="run just one of the secondary workloads (profiling captures)")
    ap.add_argument("--no-secondary", action="store_true", help="skip the secondary workloads (profiling captures)")
    ap.add_argument("--head-dim", type=int, default=0, choices=[0, 64, 128],
                    help="64: the same sequence lengths with head_dim 64 (the second build of the decode kernel; "
                         "profiling captures and side measurements, not the benchmark line)")
    ap.add_argument("--sequences", type=int, default=0,
                    help="shrink the batch (profiling captures only; the benchmark uses the full workload)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    args.warmup = max(args.warmup, 3)

    import torch
    import granite_b200 as g
    from granite_b200 import synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    else:
        torch.cuda.set_device(0)
    dev = torch.device("cuda", local_rank if world > 1 else 0)
    n_gpus = world

    if args.only:
        compute = g.CudaCompute(dev.index, torch.cuda.current_stream().cuda_stream)
        fn = SECONDARY[args.only]
        print(json.dumps(fn(compute, dev, max(args.steps, 1))), flush=True)
        compute.shutdown()
        return 0

    cfg = dict(synth.CONFIGS[args.workload])
    if args.sequences > 0:
        cfg["batch"] = args.sequences
    if args.head_dim:
        cfg["head_dim"] = args.head_dim
    strong = args.workload != WORKLOAD
    if strong:
        # one fixed problem, sequences dealt to the ranks longest-first (granite_b200/sharding.py)
        from granite_b200 import sharding
        lens_all = synth.draw_lengths(np.random.default_rng(cfg["seed"]), cfg["batch"], cfg["len_lo"],
                                      cfg["len_hi"], cfg["dist"])
        plan = sharding.lpt_assign(lens_all, world)
        case = synth.paged_case(cfg["seed"] + 7919 * rank, len(plan[rank]), 0, 0, cfg["num_heads"],
                                cfg["num_kv_heads"], cfg["head_dim"], seq_lens=lens_all[plan[rank]], device=dev)
    else:
        # every rank owns its own batch of the workload's shape: the same seeded context lengths
        # (per-GPU work is fixed, as weak scaling requires), its own page permutation and K/V/Q values
        lens = synth.draw_lengths(np.random.default_rng(cfg["seed"]), cfg["batch"], cfg["len_lo"], cfg["len_hi"],
                                  cfg["dist"])
        case = synth.paged_case(cfg["seed"] + 7919 * rank, cfg["batch"], 0, 0, cfg["num_heads"],
                                cfg["num_kv_heads"], cfg["head_dim"], seq_lens=lens, device=dev)
    B, Hq, Hkv, D = case.batch, case.num_heads, case.num_kv_heads, case.head_dim
    tokens_local = case.total_tokens
    scale = 1.0 / float(np.sqrt(D))
    stream = torch.cuda.current_stream()
    compute = g.CudaCompute(dev.index, stream.cuda_stream)

    tables_h = torch.from_numpy(case.tables).pin_memory()
    lens_h = torch.from_numpy(case.seq_lens).pin_memory()
    q_h = case.q.cpu().pin_memory()
    tables_d = tables_h.to(dev)
    lens_d = lens_h.to(dev)
    q_d = case.q
    rows = B
    if strong and world > 1:
        rows = sharding.padded_rows(plan)  # ranks own different numbers of sequences
    outs = [torch.zeros((rows, Hq, D), device=dev) for _ in range(2)]
    # Output gather across the ranks: the decode kernel itself stores every final row into every rank's
    # gathered buffer (peer-mapped symmetric memory, plain stores over NVLink) - no extra launch.  NCCL's
    # all-gather is the fall-back where symmetric memory cannot be set up, and the verifier.
    gat = Gather(dist, dev, world, (world * rows, Hq, D))
    gathered, peer_ptrs, gather_mode = gat.bufs, gat.peer_ptrs, gat.mode

    def decode(q, tables, lens, out, gather_ptrs=None):
        compute.batched_paged_attention_decode(q, case.k_pool, case.v_pool, tables, lens, out, B, Hq, Hkv,
                                               D, synth.PAGE, case.max_blocks, scale,
                                               num_blocks=case.num_blocks, gather_ptrs=gather_ptrs,
                                               gather_row_offset=rank * rows)

    def step_with(q, tables, lens, i):
        out = outs[i & 1]
        if world > 1 and peer_ptrs is not None:
            decode(q, tables, lens, out, peer_ptrs[i & 1])
        else:
            decode(q, tables, lens, out)
            if world > 1:
                # the gather is ordered after this step's kernels and before the next step's: a
                # persistent one-CTA-per-SM decode kernel must not share SMs with an NCCL kernel
                dist.all_gather_into_tensor(gathered[i & 1], out, async_op=True).wait()

    def step(i):
        step_with(q_d, tables_d, lens_d, i)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- resident-input throughput ("value"): regions of exactly --steps steps, each bracketed by a barrier
    # and a synchronize, repeated until they cover half a second; the median region is the figure
    for i in range(args.warmup):
        step(i)
    barrier()
    # kernels one step launches, counted by the library (a batch of this size needs no plan kernel: one launch)
    d0 = compute.get_profiling_stats()[0]
    step(0)
    launches_per_step = compute.get_profiling_stats()[0] - d0
    barrier()
    compute.enable_kernel_timing(True)
    compute.reset_kernel_timing()
    ms_per_step, ms_best, regions, clocks = timed_regions(dev, dist, world, step, args.steps, clock_index=dev.index)
    compute.sync()
    kstats = compute.get_kernel_timing_stats()
    compute.enable_kernel_timing(False)
    # the same steps without the output gather (max over ranks), to show what the gather costs
    ms_no_gather = None
    if world > 1:
        ms_no_gather, _, _, _ = timed_regions(dev, dist, world, lambda i: decode(q_d, tables_d, lens_d, outs[i & 1]),
                                              args.steps, min_regions=3, min_total_s=0.1)
    gather_ok = None
    if world > 1 and peer_ptrs is not None:
        # outside the timed region: what the peers stored here must be what NCCL would have gathered
        step(0)
        barrier()
        expect = torch.empty_like(gathered[0])
        dist.all_gather_into_tensor(expect, outs[0])
        gather_ok = bool(torch.equal(expect, gathered[0]))
    local_bytes = case.algorithmic_bytes()
    if world > 1:
        tb = torch.tensor([local_bytes], device=dev, dtype=torch.float64)
        dist.all_reduce(tb)
        total_bytes = float(tb.item())
    else:
        total_bytes = float(local_bytes)
    value = total_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- end to end through the C ABI with host buffers (the gather to the other ranks included)
    # the step's inputs travel as one pinned staging block [Q | block tables | lengths] and one copy
    q_bytes, t_bytes, l_bytes = q_h.numel() * 4, tables_h.numel() * 4, lens_h.numel() * 4
    pad = lambda n: (n + 255) // 256 * 256  # noqa: E731
    stage_h = torch.empty(pad(q_bytes) + pad(t_bytes) + pad(l_bytes), dtype=torch.uint8).pin_memory()
    stage_d = torch.empty_like(stage_h, device=dev)
    o_t, o_l = pad(q_bytes), pad(q_bytes) + pad(t_bytes)
    stage_h[:q_bytes].copy_(q_h.view(torch.uint8).reshape(-1))
    stage_h[o_t:o_t + t_bytes].copy_(tables_h.view(torch.uint8).reshape(-1))
    stage_h[o_l:o_l + l_bytes].copy_(lens_h.view(torch.uint8).reshape(-1))
    q_e = stage_d[:q_bytes].view(torch.float32).view(B, Hq, D)
    tables_e = stage_d[o_t:o_t + t_bytes].view(torch.int32).view(B, -1)
    lens_e = stage_d[o_l:o_l + l_bytes].view(torch.int32)

    # The result goes home without a copy of its own: the pinned host buffer is one more destination of the decode
    # kernel's fused row gather (a kernel can store to pinned host memory through its own address), so the rows
    # cross PCIe while the kernel still runs.  Laid out like the gathered buffer: this rank's rows at rank * rows.
    out_host = torch.zeros((world * rows, Hq, D), dtype=torch.float32).pin_memory()
    host_dst = [out_host.data_ptr()]

    def e2e_step(i):
        compute.write_buffer(stage_d, stage_h, stage_h.numel())
        out = outs[i & 1]
        if world > 1 and peer_ptrs is not None:
            decode(q_e, tables_e, lens_e, out, list(peer_ptrs[i & 1]) + host_dst)
        else:
            decode(q_e, tables_e, lens_e, out, host_dst)
            if world > 1:
                dist.all_gather_into_tensor(gathered[i & 1], out, async_op=True).wait()
        compute.sync()

    e2e_step(0)
    if not torch.equal(out_host[rank * rows:rank * rows + B], outs[0][:B].cpu()):
        raise RuntimeError("end-to-end step: the rows in the pinned host buffer differ from the device output")

    for i in range(3):
        e2e_step(i)
    e2e_steps = max(3, min(args.steps, 200))
    e2e_ms, e2e_best, e2e_regions, _ = timed_regions(dev, dist, world, e2e_step, e2e_steps)
    e2e_value = total_bytes / (e2e_ms * 1e-3) / 1e9
    h2d = stage_h.numel()
    d2h = B * Hq * D * 4  # the output rows, stored into pinned host memory by the decode kernel

    # ---- roofline of the dominant kernel (rank 0's launches)
    peak, peak_kind = measured_peaks()
    main_ms, main_n = kstats.get("paged_decode_splitkv", (0.0, 0))
    kernel_ms = main_ms / max(main_n, 1)
    achieved = local_bytes / (kernel_ms * 1e-3) / 1e9 if kernel_ms > 0 else None
    roofline = {
        "bound": "hbm", "kernel": "paged_decode_splitkv", "achieved": achieved, "peak": peak, "unit": "GB/s",
        "frac": (achieved / peak) if achieved else None, "peak_kind": peak_kind,
        "kernel_ms": kernel_ms, "launches_timed": main_n, "algorithmic_bytes_per_launch": local_bytes,
        "traffic": int(local_bytes * TRAFFIC_PER_ALGORITHMIC_BYTE),
        "other_kernels_ms": {k: v[0] / max(v[1], 1) for k, v in kstats.items() if k != "paged_decode_splitkv"},
    }

    # ---- CPU baseline (rank 0, N = 1 only): bounded sample
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and not strong:
        ckind, ref = cpu_arm()
        sel = list(range(0, cfg["batch"], 4))  # about 10-20 s of CPU work
        hc = host_case_for_cpu(cfg["seed"], cfg, sel)
        nb, secs, loop_secs, nseq = cpu_decode_sample(hc, gather_caches(hc), ref, repeats=1)
        cpu = {"value": nb / secs / 1e9, "unit": UNIT, "cores": cpu_threads(ref), "kind": ckind,
               "value_loop_only": nb / loop_secs / 1e9,
               "sample": f"every 4th sequence ({nseq} of {cfg['batch']}, {int(hc['seq_lens'].sum())} tokens), {secs:.2f} s",
               "note": "value: the reference's serial whole-cache fp16->fp32 widening (transformer.mm:1753-1765) + the attention "
                       "loop on all host threads, as its CPU path runs each call; value_loop_only: the loop alone on K/V "
                       "already widened"}

    secondary = None
    if not strong and args.sequences == 0 and not args.no_secondary:
        secondary = {}
        if world == 1:
            with_cpu = not args.no_cpu_baseline
            secondary = {"prefill": measure_prefill(compute, dev, with_cpu=with_cpu),
                         "prefill_by_length": measure_prefill_by_length(compute, dev),
                         "tree_verify": measure_tree(compute, dev, with_cpu=with_cpu),
                         "decode_step_cache_write": measure_decode_step_write(compute, dev),
                         "paged_prefill": measure_paged_prefill(compute, dev),
                         "single_sequence_decode": measure_single_decode(compute, dev)}
        # the headline workload's buffers are released first: the long-context problem holds 38.4 GB on one GPU
        del case, outs, gat, gathered, stage_d, q_d, q_e, tables_e, lens_e
        torch.cuda.empty_cache()
        secondary["long_context_b256"] = measure_long_context(compute, dev, dist, world, rank)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": n_gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if strong else "weak",
            "vs_baseline": None, "dtype": "f16 storage, f32 accumulate", "data": "synthetic",
            "timing": {"regions": regions, "steps_per_region": args.steps, "ms_per_step_median": ms_per_step,
                       "ms_per_step_best": ms_best,
                       "rule": "regions of exactly --steps steps, each between a barrier + synchronize, repeated until they "
                               "cover 0.5 s; ms_per_step is the median region, maximum over ranks"},
            "config": {"workload": args.workload + (f" (head_dim {D} variant)" if D != synth.CONFIGS[args.workload]["head_dim"] else ""),
                       "sequences_per_gpu": B,
                       "context": f"{cfg['dist']}[{cfg['len_lo']},{cfg['len_hi']}]",
                       "page": synth.PAGE, "num_heads": Hq, "num_kv_heads": Hkv, "head_dim": D,
                       "tokens_per_gpu": tokens_local, "kv_bytes_per_gpu": tokens_local * Hkv * D * 4,
                       "l2": f"inputs larger than L2 ({tokens_local * Hkv * D * 4 / 1e9:.1f} GB of K/V per GPU per step, no reuse)",
                       "sharding": f"by sequence; output gather: {gather_mode}" if world > 1 else "single GPU",
                       **({"gather_verified": gather_ok} if gather_ok is not None else {}),
                       **({"ms_per_step_without_gather": ms_no_gather} if ms_no_gather is not None else {})},
            "hbm_frac_of_measured_peak": value / n_gpus / peak,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms, "ms_per_step_best": e2e_best, "steps": e2e_steps, "regions": e2e_regions,
                    "note": "host Q, block tables and lengths copied in (one pinned staging block), output rows stored into a pinned host buffer by the decode kernel itself (one more destination of its fused gather), sync per step; "
                            "K/V pages are cache state resident in HBM" + ("; the rows also go to every other rank (fused gather)" if world > 1 else "")},
            # per rank: the library's own launch count of one step (paged_decode_splitkv, which plans for itself,
            # merges cut sequences and stores the rows to the other ranks) x the steps of a timed region
            "gpu_launches": launches_per_step * args.steps,
            "roofline": roofline, "cpu_baseline": cpu, "clocks": clocks,
            "secondary": secondary,
        }
        print(json.dumps(line), flush=True)
    compute.shutdown()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


# (dram__bytes_read.sum + dram__bytes_write.sum) / algorithmic bytes of one paged_decode_splitkv
# launch, from an ncu capture of a 16-sequence case of the same kernel (ncu --set full
# --clock-control none, one launch); DRAM traffic grows in proportion to the tokens read.
TRAFFIC_PER_ALGORITHMIC_BYTE = 1.0045

if __name__ == "__main__":
    sys.exit(main())
