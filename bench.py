#!/usr/bin/env python
"""Benchmark of the quantised-GEMV hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-extra]

One "step" is one decode GEMV of the headline workload: Q4_0 weights [262144, 1152] (the Gemma-3
vocabulary head, 170 MB — larger than L2, so every step streams from HBM) times one f32 activation
row. The printed value is algorithmic GB/s = (N*K/32*18 + 4K + 4N) bytes / step time. At N > 1 GPUs
the output rows are split evenly across ranks and each step ends with an all-gather of the outputs
(strong scaling: the total work is fixed).

`--impl reference` times the CPU restatement of zig-nn's own path for the same workload on the
host cores (zig-nn is Zig and cannot be built here; see oracle/).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

WORKLOAD = dict(qtype="q4_0", out_dim=262144, in_dim=1152, m_rows=1)
BPB = {"q4_0": 18, "q4_1": 20, "q8_0": 34}
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the headline kernel, from an ncu capture of
# this workload (172 002 304 bytes read + 4 768 000 written); a shard's launch is scaled by its rows.
NCU_TRAFFIC_BYTES = 176257536
WORKLOAD_NAME = "configs[1]: Q4_0 GEMV 1152->262144, M=1, f32 activations"


def config_dict():
    """The `config` object: identical in both arms (ours and --impl reference), field by field."""
    return dict(workload=WORKLOAD_NAME, qtype=WORKLOAD["qtype"], out_dim=WORKLOAD["out_dim"], in_dim=WORKLOAD["in_dim"],
                m_rows=WORKLOAD["m_rows"], weights="N(0,0.02) seed 42 quantised q4_0", activations="f32 N(0,1) seed 43")


def algorithmic_bytes(qtype, n, k, m=1):
    return n * (k // 32) * BPB[qtype] + 4 * m * k + 4 * m * n


def measured_peak():
    p = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.idx), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
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
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                for name, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                continue
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def load_oracle(native=True):
    """The CPU checker / baseline. Tries a host-tuned build first (same sources, -march=native)."""
    sys.path.insert(0, os.path.join(REPO, "oracle"))
    import oracle
    if native:
        try:
            out = os.path.join(REPO, "oracle", "_build", "libzq_oracle_native.so")
            oracle.build(arch="native", out=out)
            oracle.lib(out)
            return oracle, "native"
        except Exception:
            pass
    oracle.lib()
    return oracle, "x86-64-v3"


def make_weight_bytes(qtype_name, n, k, seed, device):
    import torch
    from zignn_b200 import ggml
    g = torch.Generator(device=device).manual_seed(seed)
    chunks = []
    step = max(1, min(n, (1 << 26) // k))  # <= 64 Mi weights (256 MB f32) at a time
    for r0 in range(0, n, step):
        w = torch.randn(min(step, n - r0), k, generator=g, device=device) * 0.02
        chunks.append(ggml.quantize(ggml.TYPE_IDS[qtype_name], w))
    return torch.cat(chunks)


def _time_calls(fn, target_seconds, max_calls=5000):
    fn()  # warm
    calls, t0 = 0, time.perf_counter()
    while True:
        fn()
        calls += 1
        el = time.perf_counter() - t0
        if el > target_seconds or calls >= max_calls:
            return calls, el


def openblas_leg(oracle, t, raw, x, n, k, qtype_name, target_seconds=4.0):
    """zig-nn's dense CPU path for the same product (src/backend/cpu.zig:148-209: cblas_sgemm): the weight is
    dequantised to f32 once, untimed, then y = x . W^T through the BLAS that numpy is linked against."""
    import numpy as np
    info = "unknown"
    try:
        cfg = np.show_config(mode="dicts")
        b = cfg.get("Build Dependencies", {}).get("blas", {})
        info = "%s %s" % (b.get("name", "?"), b.get("version", "?"))
    except Exception:
        pass
    w = oracle.dequantize(t, raw, n * k).reshape(n, k)
    y = np.empty(n, np.float32)
    calls, el = _time_calls(lambda: np.dot(w, x, out=y), target_seconds, 200)
    threads = int(os.environ.get("OPENBLAS_NUM_THREADS", 0)) or host_threads()
    return {"value": algorithmic_bytes(qtype_name, n, k) * calls / el / 1e9, "unit": "GB/s", "cores": threads,
            "ms_per_call": el / calls * 1e3, "f32_gbs": (4.0 * n * k + 4 * k + 4 * n) * calls / el / 1e9,
            "blas": info, "sample": "%d sgemv calls on the dequantised f32 weight in %.1f s" % (calls, el)}


def cpu_baseline(qtype_name, n, k, target_seconds=10.0):
    """Times the oracle's f32-activation matmul (zig-nn dequant.zig:170-309) on the same [n, k] weight: with
    all host threads (`value`), on one thread — the way gpt2.zig:632-686 calls it — and zig-nn's dense BLAS
    path on the dequantised weight. Bounded to about 20 s of CPU work."""
    import numpy as np
    from zignn_b200 import ggml
    oracle, build = load_oracle()
    threads = host_threads()
    raw = make_weight_bytes(qtype_name, n, k, 42, "cpu").numpy()
    x = np.random.default_rng(43).standard_normal(k).astype(np.float32)
    t = ggml.TYPE_IDS[qtype_name]
    nbytes = algorithmic_bytes(qtype_name, n, k)
    calls, el = _time_calls(lambda: oracle.matmul_f32(t, raw, x, n, k, threads), target_seconds)
    c1, e1 = _time_calls(lambda: oracle.matmul_f32(t, raw, x, n, k, 1), 3.0)
    out = {"value": nbytes * calls / el / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
           "sample": "%d GEMV calls of %s [%d,%d] x f32[1,%d] in %.1f s (oracle build: %s)"
                     % (calls, qtype_name, n, k, k, el, build),
           "reference_threads": {"value": nbytes * c1 / e1 / 1e9, "unit": "GB/s", "cores": 1,
                                 "note": "linear_forward_q of gpt2.zig:632-686 runs matmul_q4_0_f32 on the calling thread",
                                 "sample": "%d calls in %.1f s" % (c1, e1)}}
    try:
        out["openblas_sgemm"] = openblas_leg(oracle, t, raw, x, n, k, qtype_name)
    except Exception as e:
        out["openblas_sgemm"] = {"value": None, "error": repr(e)}
    return out


def run_reference(args):
    rank, _, world = dist_env()
    if rank != 0:
        return
    import numpy as np
    from zignn_b200 import ggml
    oracle, build = load_oracle()
    q, n, k = WORKLOAD["qtype"], WORKLOAD["out_dim"], WORKLOAD["in_dim"]
    threads = host_threads()
    raw = make_weight_bytes(q, n, k, 42, "cpu").numpy()
    x = np.random.default_rng(43).standard_normal(k).astype(np.float32)
    t = ggml.TYPE_IDS[q]
    for _ in range(args.warmup):
        oracle.matmul_f32(t, raw, x, n, k, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.matmul_f32(t, raw, x, n, k, threads)
    el = time.perf_counter() - t0
    ms = el / args.steps * 1e3
    gbs = algorithmic_bytes(q, n, k) / (ms * 1e-3) / 1e9
    line = {
        "impl": "reference", "metric": "q4_0_gemv_algorithmic_gbs", "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_dict(),
        "run": dict(l2="host memory (the 170 MB matrix exceeds the host caches)",
                    sharding="rows split over %d host thread(s): CPU restatement of zig-nn matmul_q4_0_f32 "
                             "(dequant.zig:170-182)" % threads,
                    launch="plain calls"),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": "%d timed GEMV calls (oracle build: %s)" % (args.steps, build)},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def time_region(torch, fn, steps, sync, flush=None):
    """K calls bracketed by sync + CUDA events on the current stream; returns total ms. With `flush`
    (a callable that evicts L2) every call gets its own event pair and the flush runs between the
    pairs, outside the timed intervals; the result is the sum of the K intervals."""
    sync()
    if flush is None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        sync()
        return e0.elapsed_time(e1)
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for e0, e1 in pairs:
        flush()
        e0.record()
        fn()
        e1.record()
    sync()
    return sum(e0.elapsed_time(e1) for e0, e1 in pairs)


def graph_time_us(torch, fns, reps=20):
    """Average device time of one call: the calls are captured once into a CUDA graph (so host launch
    overhead is out of the picture) and the graph is replayed `reps` times."""
    for f in fns:
        f()  # outside capture first: one-time function attributes are set here
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for f in fns:
            f()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * len(fns))


def sweep_extra(torch, zq, ggml, m_list=(1,)):
    """configs[1] shapes x types, HBM-cold: each timed call uses a different weight copy and the copies
    together exceed L2 (126 MB). Times are per call inside a CUDA graph."""
    out = []
    shapes = [(768, 2304), (768, 3072), (3072, 768), (1152, 6912), (6912, 1152), (1152, 262144)]
    for qname in ("q4_0", "q4_1", "q8_0"):
        for k, n in shapes:
            raw = make_weight_bytes(qname, n, k, 42, "cuda")
            wbytes = n * (k // 32) * BPB[qname]
            copies = max(2, min(48, int(400e6 // wbytes) + 1))
            ws = [zq.QuantWeight(raw, ggml.TYPE_IDS[qname], n, k) for _ in range(copies)]
            for m in m_list:
                nbytes = algorithmic_bytes(qname, n, k, m)
                x = torch.randn(m, k, device="cuda")
                y = torch.empty(m, n, device="cuda")
                for mode, mname in ((zq.ACT_F32, "f32"), (zq.ACT_Q8, "q8")):
                    need = _lib_ws(zq, ws[0], m, mode)
                    wsb = torch.empty(max(need, 256), dtype=torch.uint8, device="cuda")
                    fns = [(lambda w=w: zq.quant_matmul_no_grad(x, w, mode, out=y, workspace=wsb)) for w in ws]
                    us = graph_time_us(torch, fns)
                    out.append({"type": qname, "k": k, "n": n, "m": m, "act": mname, "us": round(us, 2),
                                "gbs": round(nbytes / us / 1e3, 1), "copies": copies})
            del ws, raw
    return out


def sweep_stream(torch, zq, ggml):
    """The weight-streaming tensor-core form: 32 / 64 / 128 f32 activation rows against the vocabulary head and the
    4096 -> 14336 projection, HBM-cold (every timed call on another weight copy), per call inside a CUDA graph.
    `gbs` counts the algorithmic bytes (weights once, activations, outputs)."""
    out = []
    for qname in ("q4_0", "q8_0"):
        for k, n in ((1152, 262144), (4096, 14336)):
            raw = make_weight_bytes(qname, n, k, 42, "cuda")
            wbytes = n * (k // 32) * BPB[qname]
            copies = max(2, min(8, int(400e6 // wbytes) + 1))
            ws = [zq.QuantWeight(raw, ggml.TYPE_IDS[qname], n, k) for _ in range(copies)]
            for m in (32, 64, 128):
                x = torch.randn(m, k, device="cuda")
                y = torch.empty(m, n, device="cuda")
                need = _lib_ws(zq, ws[0], m, zq.ACT_F32)
                wsb = torch.empty(max(need, 256), dtype=torch.uint8, device="cuda")
                fns = [(lambda w=w: zq.quant_matmul_no_grad(x, w, zq.ACT_F32, out=y, workspace=wsb)) for w in ws]
                us = graph_time_us(torch, fns)
                nbytes = algorithmic_bytes(qname, n, k, m)
                out.append({"type": qname, "k": k, "n": n, "m": m, "act": "f32", "us": round(us, 2),
                            "gbs": round(nbytes / us / 1e3, 1), "weights_gbs": round(wbytes / us / 1e3, 1),
                            "copies": copies})
            del ws, raw
    return out


def sweep_many_rows(torch, zq, ggml):
    """The tensor-core GEMM at 512 / 2048 / 4096 f32 activation rows (pairs of CTAs, tcgen05 cta_group::2, where the
    library takes that form): TFLOP/s = 2 M N K / time by CUDA events, activation-conversion launch included,
    median of 5 after 3 warm-up calls. `of_peak` is against the measured cuBLAS bf16 burst."""
    peak = 1590.0  # fallback: an earlier measurement on this pool
    try:
        peak = float(json.load(open(os.path.join(REPO, "MEASURED_PEAKS.json")))["bf16_tflops"])
    except Exception:
        pass
    out = []
    for qname, k, n in (("q4_0", 4096, 14336), ("q4_0", 14336, 4096), ("q8_0", 4096, 14336), ("q4_0", 1152, 262144)):
        raw = make_weight_bytes(qname, n, k, 42, "cuda")
        w = zq.QuantWeight(raw, ggml.TYPE_IDS[qname], n, k)
        for m in (512, 2048, 4096):
            if m * n > 600e6:
                continue
            x = torch.randn(m, k, device="cuda")
            y = torch.empty(m, n, device="cuda")
            wsb = torch.empty(max(_lib_ws(zq, w, m, zq.ACT_F32), 256), dtype=torch.uint8, device="cuda")
            for _ in range(3):
                zq.quant_matmul_no_grad(x, w, zq.ACT_F32, out=y, workspace=wsb)
            times = []
            for _ in range(5):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                zq.quant_matmul_no_grad(x, w, zq.ACT_F32, out=y, workspace=wsb)
                e1.record()
                torch.cuda.synchronize()
                times.append(e0.elapsed_time(e1) * 1e3)
            us = sorted(times)[2]
            tf = 2.0 * m * n * k / us / 1e6
            out.append({"type": qname, "k": k, "n": n, "m": m, "us": round(us, 1), "tflops": round(tf, 1),
                        "of_peak": round(tf / peak, 3)})
            del x, y, wsb
        del w, raw
    return out


def decode_bytes_per_token(name, cfg, ctx_mid):
    """Algorithmic HBM bytes of one decoded token: every quantised block once (plus GPT-2's f32 embedding
    matrix as the logits head) and the key / value rows the attention reads at context `ctx_mid`."""
    if name.startswith("gpt2"):
        E, F, L, V = cfg["embed"], cfg["ffn"], cfg["layer"], cfg["vocab"]
        weights = L * (3 * E * E + E * E + 2 * E * F)
        return weights // 32 * BPB["q4_0"] + 4 * V * E + L * 2 * ctx_mid * E * 4
    E, F, L, V, D = cfg["embed"], cfg["ffn"], cfg["layer"], cfg["vocab"], cfg["head_dim"]
    qd, kd = cfg["head"] * D, cfg["head_kv"] * D
    weights = L * ((qd + 2 * kd) * E + E * qd + 3 * E * F) + V * E
    n_global = L // cfg["global_every"]
    kv_rows = (L - n_global) * min(ctx_mid, cfg["sliding_window"]) + n_global * ctx_mid
    return weights // 32 * BPB["q8_0"] + kv_rows * 2 * kd * 4


def decode_extra(torch, zq, ggml):
    """Batch-1 greedy decode rates of the two model shapes (configs[0] and configs[2]) through the engines,
    as a rate and as a fraction of the HBM roofline, next to the CPU checker on the same synthetic weights at
    the same context: with the thread count zig-nn itself uses (GPT-2: the calling thread, gpt2.zig:632-686;
    Gemma-3: min(cores, 8), gemma3.zig:285-286) and, from a short context, with all host threads. The CPU legs
    are bounded samples: one prefill of the prompt and 6 decode steps."""
    import numpy as np
    from zignn_b200 import hostmodel
    oracle, build = load_oracle()
    threads = host_threads()
    peak, peak_kind = measured_peak()
    out = []
    cases = (("gpt2_small_q4_0", hostmodel.Gpt2Host, hostmodel.GPT2_SMALL, ggml.Q4_0, zq.Gpt2, oracle.Gpt2, 32, 128, 1),
             ("gemma3_1b_q8_0", hostmodel.Gemma3Host, hostmodel.GEMMA3_1B, ggml.Q8_0, zq.Gemma3, oracle.Gemma3, 512, 256,
              min(threads, 8)))
    for name, Host, cfg, qt, Eng, Ora, n_prompt, n_decode, ref_threads in cases:
        host = Host.synthetic(cfg, qtype=qt, seed=42, device="cuda")
        prompt = np.random.default_rng(44).integers(0, cfg["vocab"], size=n_prompt)
        rates = {}
        modes = [("persistent_kernel", zq.DECODE_AUTO), ("launch_sequence", zq.DECODE_LAUNCH_SEQUENCE)]
        for label, mode in modes:
            eng = Eng(host)
            if mode is not None:
                eng.set_decode_mode(mode)
                if mode == zq.DECODE_AUTO and eng.decode_mode != zq.DECODE_PERSISTENT:
                    eng.close()
                    continue
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            first = int(eng.prefill(prompt).argmax().item())
            t1 = time.perf_counter()
            eng.decode_greedy(first, 8)  # the first steps set up the replayed launch sequence
            eng.reset_cache()
            first = int(eng.prefill(prompt).argmax().item())
            torch.cuda.synchronize()
            t2 = time.perf_counter()
            toks = eng.decode_greedy(first, n_decode)  # returns after the tokens are on the host
            t3 = time.perf_counter()
            rates[label] = dict(tok_s=n_decode / (t3 - t2), prefill_ms=(t1 - t0) * 1e3, last_token=int(toks[-1]))
            eng.close()
        best = max(rates, key=lambda k: rates[k]["tok_s"])
        gpu_tps = rates[best]["tok_s"]
        ref = Ora(host, ref_threads)
        c0 = time.perf_counter()
        tok = int(np.argmax(ref.prefill(prompt)))
        c1 = time.perf_counter()
        n_cpu = 6
        for _ in range(n_cpu):
            tok = int(np.argmax(ref.decode_next(tok)))
        c2 = time.perf_counter()
        cpu_tps = n_cpu / (c2 - c1)
        del ref
        allt = Ora(host, threads)
        tok = int(np.argmax(allt.prefill(prompt[:4])))
        a1 = time.perf_counter()
        for _ in range(n_cpu):
            tok = int(np.argmax(allt.decode_next(tok)))
        a2 = time.perf_counter()
        del allt
        nbytes = decode_bytes_per_token(name, cfg, n_prompt + n_decode // 2)
        out.append({"model": name, "prompt": n_prompt, "decode_steps": n_decode,
                    "gpu_decode_tok_s": round(gpu_tps, 1), "gpu_path": best,
                    "gpu_paths": {k: round(v["tok_s"], 1) for k, v in rates.items()},
                    "gpu_prefill_ms": round(rates[best]["prefill_ms"], 1),
                    "bytes_per_token": nbytes, "achieved_gbs": round(nbytes * gpu_tps / 1e9, 1),
                    "frac_of_hbm_peak": round(nbytes * gpu_tps / 1e9 / peak, 4), "peak_kind": peak_kind,
                    "cpu_decode_tok_s": round(cpu_tps, 2), "cpu_threads": ref_threads,
                    "cpu_prefill_tok_s": round(n_prompt / (c1 - c0), 2),
                    "cpu_note": "thread count of the reference; same prompt and context as the GPU leg",
                    "cpu_all_threads_short_context_tok_s": round(n_cpu / (a2 - a1), 2), "cpu_all_threads": threads,
                    "cpu_build": build, "gpu_over_cpu": round(gpu_tps / cpu_tps, 1),
                    "last_token": rates[best]["last_token"]})
        del host
    return out


def run_case(args):
    """One quantised matmul, --steps timed calls on fresh weight copies (HBM-cold), one JSON line."""
    import torch
    import zignn_b200
    from zignn_b200 import api as zq
    from zignn_b200 import ggml
    if args.case.startswith("batch:"):
        # batch:<gemma3_1b_q4_1|gemma3_1b_q8_0>,<sequences>,<prompt tokens>,<decode steps>
        import numpy as np
        from zignn_b200 import hostmodel
        name, n_seq, n_prompt, n_steps = args.case[6:].split(",")
        n_seq, n_prompt, n_steps = int(n_seq), int(n_prompt), int(n_steps)
        qt = ggml.Q4_1 if name.endswith("q4_1") else ggml.Q8_0
        host = hostmodel.Gemma3Host.synthetic(hostmodel.GEMMA3_1B, qtype=qt, seed=42, device="cuda")
        eng = zq.Gemma3Batch(host, n_seq)
        rng = np.random.default_rng(44)
        toks = []
        t0 = time.perf_counter()
        for i in range(n_seq):
            if n_prompt == 0:  # no prefill: every sequence starts from an empty cache with a random token
                toks.append(int(rng.integers(0, hostmodel.GEMMA3_1B["vocab"])))
                continue
            toks.append(int(eng.prefill(i, rng.integers(0, hostmodel.GEMMA3_1B["vocab"], size=n_prompt)).argmax().item()))
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        toks = eng.decode_next(toks).argmax(dim=1).cpu().numpy()  # first call: one-time set-up
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        for _ in range(n_steps):
            toks = eng.decode_next(toks).argmax(dim=1).cpu().numpy()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t2
        print(json.dumps({"case": args.case, "tok_s_all_sequences": n_seq * n_steps / dt, "ms_per_step": dt / n_steps * 1e3,
                          "prefill_ms_per_sequence": (t1 - t0) / n_seq * 1e3}), flush=True)
        return
    if args.case.startswith("decode:"):
        # decode:<gpt2_small_q4_0|gemma3_1b_q8_0>,<prompt tokens>,<greedy steps>
        import numpy as np
        from zignn_b200 import hostmodel
        name, n_prompt, n_steps = args.case[7:].split(",")
        if name.startswith("gemma"):
            host = hostmodel.Gemma3Host.synthetic(hostmodel.GEMMA3_1B, qtype=ggml.Q8_0, seed=42, device="cuda")
            eng, vocab = zq.Gemma3(host), hostmodel.GEMMA3_1B["vocab"]
        else:
            host = hostmodel.Gpt2Host.synthetic(hostmodel.GPT2_SMALL, qtype=ggml.Q4_0, seed=42, device="cuda")
            eng, vocab = zq.Gpt2(host), hostmodel.GPT2_SMALL["vocab"]
        prompt = np.random.default_rng(44).integers(0, vocab, size=int(n_prompt))
        first = int(eng.prefill(prompt).argmax().item())
        if int(n_steps) > 16:
            eng.decode_greedy(first, 8)  # the first steps set up the replayed launch sequence
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        toks = eng.decode_greedy(first, int(n_steps))
        dt = time.perf_counter() - t0
        print(json.dumps({"case": args.case, "tok_s": int(n_steps) / dt, "last_token": int(toks[-1])}), flush=True)
        return
    if args.case.startswith("shard:"):
        # shard:<type>,<in_dim K>,<out_dim N>,<rows M>: the product with the weight's rows split over the ranks this
        # process was started with (torchrun; one rank without it), every rank ending up with the whole [M][N]
        # result: M = 1 by the GEMV with the exchange inside, more rows by the local product and the exchange of
        # column slices. Time by CUDA events over --steps calls, max over ranks; `alone` is this rank's product
        # without the exchange.
        import torch.distributed as dist
        from zignn_b200 import sharding
        qname, k, n, m = args.case[6:].split(",")
        k, n, m = int(k), int(n), int(m)
        rank, local_rank, world = dist_env()
        torch.cuda.set_device(local_rank)
        if world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        raw = make_weight_bytes(qname, n, k, 42, "cuda")
        x = torch.randn(m, k, device="cuda", generator=torch.Generator(device="cuda").manual_seed(43))
        qt = ggml.TYPE_IDS[qname]
        if world > 1:
            lin = sharding.cuda_sharded_linear(raw, qt, n, k, zq.ACT_F32, gather="peer", m_rows=m)
            w_local, rows = lin.weight, lin.rows
            call = lambda: lin.forward(x)
        else:
            w_local, rows = zq.QuantWeight(raw, qt, n, k), n
            y = torch.empty(m, n, device="cuda")
            wsb = torch.empty(max(_lib_ws(zq, w_local, m, zq.ACT_F32), 256), dtype=torch.uint8, device="cuda")
            call = lambda: zq.quant_matmul_no_grad(x, w_local, zq.ACT_F32, out=y, workspace=wsb)
        del raw
        y_alone = torch.empty(m, rows, device="cuda")
        ws_alone = torch.empty(max(_lib_ws(zq, w_local, m, zq.ACT_F32), 256), dtype=torch.uint8, device="cuda")
        alone = lambda: zq.quant_matmul_no_grad(x, w_local, zq.ACT_F32, out=y_alone, workspace=ws_alone)

        def sync():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        def timed(fn, steps):
            for _ in range(4):
                fn()
            ms = time_region(torch, fn, steps, sync)
            if world > 1:
                t = torch.tensor([ms], device="cuda")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            return ms / steps * 1e3
        steps = max(2, args.steps - args.steps % 2)
        us = timed(call, steps)
        us_alone = timed(alone, steps)
        if world > 1:
            from zignn_b200 import _lib as zlib
            zlib.check(zlib.load().zq_device_check(1), "peer exchange")
        if rank == 0:
            print(json.dumps({"case": args.case, "n_gpus": world, "us_per_step": round(us, 1), "us_product_alone": round(us_alone, 1),
                              "exchange_share": round(max(0.0, 1.0 - us_alone / us), 3),
                              "tflops_whole_job": round(2.0 * m * n * k / us / 1e6, 1),
                              "gbs_whole_job": round(algorithmic_bytes(qname, n, k, m) / us / 1e3, 1)}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return
    if args.case.startswith("trans:"):
        # trans:<type>,<in_dim K>,<out_dim N>,<rows M>: grad_x[M][K] = grad_out[M][N] . W[N][K]
        qname, k, n, m = args.case[6:].split(",")
        k, n, m = int(k), int(n), int(m)
        raw = make_weight_bytes(qname, n, k, 42, "cuda")
        w = zq.QuantWeight(raw, ggml.TYPE_IDS[qname], n, k)
        go = torch.randn(m, n, device="cuda") * 1e-3
        gx = torch.empty(m, k, device="cuda")
        from zignn_b200 import _lib
        wsb = torch.empty(_lib.load().zq_matmul_transposed_workspace_bytes(w.handle, m), dtype=torch.uint8, device="cuda")
        for _ in range(max(1, args.warmup)):
            zq.quant_matmul_transposed(go, w, grad_x=gx, workspace=wsb)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            zq.quant_matmul_transposed(go, w, grad_x=gx, workspace=wsb)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / args.steps
        print(json.dumps({"case": args.case, "us_per_call": us, "tflops": 2.0 * m * n * k / us / 1e6,
                          "steps": args.steps}), flush=True)
        return
    parts = args.case.split(",")
    qname, k, n, m = parts[0], int(parts[1]), int(parts[2]), int(parts[3])
    mode = zq.ACT_Q8 if len(parts) > 4 and parts[4] == "q8" else zq.ACT_F32
    raw = make_weight_bytes(qname, n, k, 42, "cuda")
    wbytes = n * (k // 32) * BPB[qname]
    copies = max(2, min(16, int(300e6 // wbytes) + 1))
    ws = [zq.QuantWeight(raw, ggml.TYPE_IDS[qname], n, k) for _ in range(copies)]
    x = torch.randn(m, k, device="cuda")
    y = torch.empty(m, n, device="cuda")
    wsb = torch.empty(max(_lib_ws(zq, ws[0], m, mode), 256), dtype=torch.uint8, device="cuda")
    for i in range(max(1, args.warmup)):
        zq.quant_matmul_no_grad(x, ws[i % copies], mode, out=y, workspace=wsb)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        zq.quant_matmul_no_grad(x, ws[i % copies], mode, out=y, workspace=wsb)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / args.steps
    print(json.dumps({"case": args.case, "us_per_call": us, "tflops": 2.0 * m * n * k / us / 1e6,
                      "gbs": algorithmic_bytes(qname, n, k, m) / us / 1e3, "steps": args.steps}), flush=True)


def _lib_ws(zq, w, m, mode):
    from zignn_b200 import _lib
    return _lib.load().zq_matmul_workspace_bytes(w.handle, m, mode)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the sweep / cpu baseline side measurements")
    ap.add_argument("--gather", default="peer", choices=["peer", "nccl"], help="N > 1: how output slices are exchanged")
    ap.add_argument("--case", default=None, metavar="TYPE,K,N,M[,ACT]",
                    help="time one quantised matmul (e.g. q4_0,4096,14336,512 or q8_0,1152,6912,1,q8), or one "
                         "engine run (decode:gemma3_1b_q8_0,300,3 = prompt tokens, greedy steps), and exit; for "
                         "profiling kernels other than the headline one")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.case:
        return run_case(args)

    import torch
    import zignn_b200
    from zignn_b200 import api as zq
    from zignn_b200 import ggml

    rank, local_rank, world = dist_env()
    torch.cuda.set_device(local_rank)
    use_dist = world > 1
    if use_dist:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    q, n, k = WORKLOAD["qtype"], WORKLOAD["out_dim"], WORKLOAD["in_dim"]
    from zignn_b200 import sharding
    # every rank draws the same full-weight stream and keeps its row slice (sharding.row_range)
    raw_full = make_weight_bytes(q, n, k, 42, "cuda")
    # N > 1: the slices are exchanged by the library's peer-store kernel; --gather nccl (or a failed
    # symmetric-memory set-up) uses all_gather_into_tensor instead
    gather_mode = args.gather if use_dist else "none"
    lin = None
    if gather_mode == "peer":
        try:
            lin = sharding.cuda_sharded_linear(raw_full, ggml.TYPE_IDS[q], n, k, zq.ACT_F32, gather="peer", m_rows=1)
        except Exception as e:
            gather_mode = "nccl (peer set-up failed: %r)" % (e,)
    if lin is None:
        lin = sharding.cuda_sharded_linear(raw_full, ggml.TYPE_IDS[q], n, k, zq.ACT_F32)
    qw, n_local = lin.weight, lin.rows
    x = torch.randn(1, k, device="cuda", generator=torch.Generator(device="cuda").manual_seed(43))
    y_local = torch.zeros(1, lin.per, device="cuda")

    # Correctness of what is about to be timed (N > 1): the gathered row against the unsharded product on this
    # rank's GPU, and against the CPU checker on 256 sampled rows. A mismatch ends the run with a non-zero status.
    parity = None
    if use_dist:
        full = zq.QuantWeight(raw_full, ggml.TYPE_IDS[q], n, k)
        want = zq.quant_matmul_no_grad(x, full, zq.ACT_F32)
        if gather_mode == "peer":
            got = lin.forward(x).clone()
            lin.forward(x)  # an even number of exchanges: the two result buffers alternate
        else:
            zq.quant_matmul_no_grad(x, qw, zq.ACT_F32, out=y_local)
            got = lin.gather(y_local).clone()
        torch.cuda.synchronize()
        diff = float((got.double() - want.double()).norm() / want.double().norm())
        parity = {"gathered_vs_unsharded_rel_l2": diff, "bit_equal": bool(torch.equal(got, want)), "tolerance": 2e-6}
        if rank == 0:
            import numpy as np
            oracle, _ = load_oracle()
            rows = np.sort(np.random.default_rng(5).choice(n, size=256, replace=False))
            row_bytes = k // 32 * BPB[q]
            sub = raw_full.view(n, row_bytes)[torch.from_numpy(rows).cuda()].cpu().numpy().reshape(-1)
            ref = oracle.matmul_f32(ggml.TYPE_IDS[q], sub, x.cpu().numpy().reshape(-1), len(rows), k, 4)
            g = got[0, torch.from_numpy(rows).cuda()].cpu().numpy()
            parity["vs_cpu_oracle_rel_l2_256_rows"] = float(np.linalg.norm(g - ref) / np.linalg.norm(ref))
            parity["cpu_tolerance"] = 1e-5  # the path's bar is 1e-3; f32 summation orders differ by about 1e-6
            parity["ok"] = diff <= 2e-6 and parity["vs_cpu_oracle_rel_l2_256_rows"] <= 1e-5
        else:
            parity["ok"] = diff <= 2e-6
        flag = torch.tensor([0 if parity["ok"] else 1], device="cuda")
        dist.all_reduce(flag)
        if int(flag.item()):
            if rank == 0:
                print(json.dumps({"error": "sharded result differs from the unsharded product", "parity": parity}), flush=True)
            dist.destroy_process_group()
            sys.exit(3)
        del full, want, got
    del raw_full

    # One rank's shard is smaller than L2 (126 MB) from 2 ranks up. Consecutive steps therefore use
    # different copies of the shard, enough of them to exceed L2, so every step streams from HBM.
    local_weight_bytes = max(1, n_local * (k // 32) * BPB[q])
    copies = 1
    if use_dist:
        copies = max(2, int(-(-170e6 // local_weight_bytes)))
        copies += copies % 2  # the peer exchange alternates two buffers: keep sequences even
    weights = [qw]
    for _ in range(copies - 1):
        weights.append(zq.QuantWeight(qw.raw_bytes(), ggml.TYPE_IDS[q], n_local, k) if n_local else None)
    counter = [0]

    def step():
        w = weights[counter[0] % copies]
        counter[0] += 1
        if gather_mode == "peer":
            return lin.forward(x, weight=w)  # GEMV with the exchange fused in (or GEMV + exchange kernel)
        if w is not None:
            zq.quant_matmul_no_grad(x, w, zq.ACT_F32, out=y_local)
        return lin.gather(y_local) if use_dist else y_local

    def sync():
        if use_dist:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(3, args.warmup) + (copies - max(3, args.warmup) % copies) % copies):
        step()  # a whole number of passes over the copies: the next step uses copy 0 again
    # Steps are replayed from a captured launch sequence (one pass over the copies): the host-side call
    # overhead of the Python binding would otherwise be a large part of a 10-35 us step. NCCL's collective
    # stays outside capture; the end-to-end leg below always uses plain calls.
    # (one rank: the 170 MB matrix is HBM-cold by size; ten steps per recording, so that consecutive steps
    # follow each other on the device as the kernels of a decode step do)
    seq_len = copies if use_dist else 10
    graph = None
    if gather_mode in ("none", "peer"):
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(seq_len):
                step()
        graph.replay()  # one untimed replay
    sync()

    def timed_region():
        """Exactly args.steps steps: whole replays of the captured sequence, then the rest as plain calls."""
        if graph is None:
            for _ in range(args.steps):
                step()
            return
        for _ in range(args.steps // seq_len):
            graph.replay()
        for _ in range(args.steps % seq_len):
            step()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    total_ms = time_region(torch, timed_region, 1, sync)
    if gather_mode == "peer" and (args.steps % seq_len) % 2:
        step()  # untimed: back to an even number of exchanges
    clocks = sampler.stop() if sampler else None
    if use_dist:
        tmax = torch.tensor([total_ms], device="cuda")
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        total_ms = float(tmax.item())
    ms = total_ms / args.steps
    bytes_step = algorithmic_bytes(q, n, k)
    value = bytes_step / (ms * 1e-3) / 1e9

    # end to end through the public call with host buffers: pinned x -> device, GEMV, y -> pinned host
    hx = torch.randn(1, k).pin_memory()
    hy = torch.empty(tuple(step().shape), dtype=torch.float32).pin_memory()  # the full logits row on every rank

    host_call = zq.HostLinear(qw, 1, zq.ACT_F32) if not use_dist else None
    from zignn_b200 import _lib as zlib
    import ctypes as C

    def copy_f32(dst_ptr, src_ptr, count):
        zlib.check(zlib.load().zq_copy_f32(C.c_void_p(dst_ptr), C.c_void_p(src_ptr), count,
                                           C.c_void_p(torch.cuda.current_stream().cuda_stream)), "zq_copy_f32")

    direct_host = [False]

    def e2e_device_part():
        # pinned x -> device by a copy kernel, the sharded product with its exchange, the full row -> pinned y: the
        # fused kernel writes this rank's rows and the rows it unpacks from its inbox straight into the pinned
        # buffer (as the one-GPU host call does); the other routes copy the gathered row out afterwards
        copy_f32(x.data_ptr(), hx.data_ptr(), k)
        if gather_mode == "peer" and getattr(lin, "fused", False) and lin.peer.tagged and hy.numel() == lin.world * lin.per:
            w = weights[counter[0] % copies]
            counter[0] += 1
            lin.forward(x, weight=w, out=hy)
            direct_host[0] = True
            return
        y = step()
        copy_f32(hy.data_ptr(), y.data_ptr(), hy.numel())

    # N > 1: one recording per weight copy (an even number: the exchange alternates two result buffers, and a
    # recording's copy-out reads the buffer of its own round), replayed in turn; one replay = one call.
    e2e_graphs = []
    if use_dist and gather_mode == "peer":
        for _ in range(copies):
            e2e_device_part()
        torch.cuda.synchronize()
        for _ in range(copies):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                e2e_device_part()
            e2e_graphs.append(g)
    e2e_calls = [0]

    def e2e_step():
        if host_call is not None:
            # the host-buffer call of the public API: x staged to the device, the kernel writes the logits
            # straight into the pinned result buffer (PCIe traffic: 4K bytes in, 4N bytes out per step)
            host_call(hx, hy)
            return
        if e2e_graphs:
            e2e_graphs[e2e_calls[0] % copies].replay()
            e2e_calls[0] += 1
        else:
            x.copy_(hx, non_blocking=True)
            hy.copy_(step(), non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the caller reads hy

    for _ in range(copies if e2e_graphs else 3):
        e2e_step()
    e2e_ms = time_region(torch, e2e_step, args.steps, sync)
    if e2e_graphs and e2e_calls[0] % 2:
        e2e_step()  # untimed: back to an even number of exchanges
    if use_dist:
        tmax = torch.tensor([e2e_ms], device="cuda")
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        e2e_ms = float(tmax.item())
    e2e_value = bytes_step / (e2e_ms / args.steps * 1e-3) / 1e9
    if use_dist and parity is not None:
        # what the end-to-end leg left in the pinned buffer is the gathered row
        torch.cuda.synchronize()
        ref_row = step().clone()
        step()  # an even number of exchanges of the two result buffers
        torch.cuda.synchronize()
        parity["e2e_host_row_equals_gathered_row"] = bool(torch.equal(hy.reshape(-1)[:n], ref_row.reshape(-1)[:n].cpu()))
        parity["e2e_row_written_to_pinned_memory_by_the_kernel"] = bool(direct_host[0])
        if not parity["e2e_host_row_equals_gathered_row"]:
            parity["ok"] = False

    # Greedy decoding over the sharded head (N > 1): the same product with only the index of the first largest
    # logit exchanged (16 bytes per peer instead of the row). Checked against the full gathered row, then timed the
    # same way as the main leg. Reported beside it; the headline stays the gathered row.
    greedy = None
    if use_dist and gather_mode == "peer" and graph is not None and hasattr(lin, "greedy"):
        try:
            full_row = step().clone()
            step()  # an even number of exchanges of the two result buffers
            idx, val = lin.greedy(x, weight=weights[0])
            torch.cuda.synchronize()
            want_idx = int(torch.nonzero(full_row[0] == full_row[0].max())[0, 0].item())
            gc = [0]

            def gstep():
                w = weights[gc[0] % copies]
                gc[0] += 1
                lin.greedy(x, weight=w)
            for _ in range(copies):
                gstep()
            torch.cuda.synchronize()
            gg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gg):
                for _ in range(seq_len):
                    gstep()
            gg.replay()
            sync()
            reps = max(1, args.steps // seq_len)
            g_ms = time_region(torch, lambda: [gg.replay() for _ in range(reps)], 1, sync)
            tg = torch.tensor([g_ms], device="cuda")
            dist.all_reduce(tg, op=dist.ReduceOp.MAX)
            greedy = {"us_per_step": round(float(tg.item()) * 1e3 / (reps * seq_len), 2), "index": int(idx.item()),
                      "matches_first_largest_of_the_gathered_row": int(idx.item()) == want_idx,
                      "exchange_bytes_per_peer": 16}
            if int(idx.item()) != want_idx:
                raise RuntimeError("arg-max exchange: index %d, gathered row says %d" % (int(idx.item()), want_idx))
        except Exception as e:
            greedy = {"error": repr(e)}
            if "arg-max exchange" in repr(e):
                raise

    if rank == 0:
        peak, peak_kind = measured_peak()
        kernel_ms = ms
        if use_dist:  # the GEMV alone, for the roofline of the dominant kernel
            kc = [0]

            def kernel_only():
                w = weights[kc[0] % copies]
                kc[0] += 1
                if w is not None:
                    zq.quant_matmul_no_grad(x, w, zq.ACT_F32, out=y_local)
            kernel_ms = graph_time_us(torch, [kernel_only] * copies) * 1e-3
        local_bytes = algorithmic_bytes(q, n_local, k)
        achieved = local_bytes / (kernel_ms * 1e-3) / 1e9
        line = {
            "metric": "q4_0_gemv_algorithmic_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_dict(),
            "run": dict(
                l2=("weights (170 MB) larger than L2 (126 MB)" if copies == 1 else
                    "%d copies of the %.0f MB shard used in turn (together larger than L2)"
                    % (copies, local_weight_bytes / 1e6)),
                sharding="rows split over %d rank(s)%s" % (
                    world, ", all-gather of outputs: " + gather_mode +
                    (" stores fused into the GEMV epilogue" if getattr(lin, "fused", False) else "")
                    if use_dist else ""),
                launch=("CUDA graph replay, %d steps per recording" % seq_len) if graph is not None else "plain calls",
                **({"greedy_argmax_exchange": greedy} if greedy is not None else {})),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         # ncu capture of the full matrix; a shard's launch is scaled by its rows
                         "traffic": int(NCU_TRAFFIC_BYTES * local_bytes / algorithmic_bytes(q, n, k)),
                         "peak_kind": peak_kind,
                         "algorithmic_bytes_per_launch": local_bytes, "kernel": "gemv_mma1_kernel<q4_0>"},
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": 4 * k, "d2h_bytes_per_step": hy.numel() * 4},
            "gpu_launches": args.steps * (1 if gather_mode != "peer" or getattr(lin, "fused", False) else 3),
            "clocks": clocks,
        }
        if parity is not None:
            line["parity"] = parity
        if not args.no_extra and world == 1:
            try:
                line["cpu_baseline"] = cpu_baseline(q, n, k)
            except Exception as e:  # the baseline is informational; never lose the GPU line
                line["cpu_baseline"] = {"value": None, "unit": "GB/s", "cores": host_threads(), "kind": "port",
                                        "sample": "failed: %r" % (e,)}
            # the second half of the metric: decode tok/s of the two model shapes, with their HBM roofline
            try:
                line["roofline"]["decode"] = decode_extra(torch, zq, ggml)
            except Exception as e:
                line["roofline"]["decode"] = {"error": repr(e)}
            line["decode"] = line["roofline"]["decode"]
            line["extra"] = {}
            try:
                line["extra"]["sweep_hbm_cold"] = sweep_extra(torch, zq, ggml, m_list=(1, 4, 16))
            except Exception as e:
                line["extra"]["sweep_hbm_cold"] = {"error": repr(e)}
            try:
                line["extra"]["sweep_streaming_gemm"] = sweep_stream(torch, zq, ggml)
            except Exception as e:  # noqa: BLE001
                line["extra"]["sweep_streaming_gemm"] = {"error": repr(e)}
            try:
                line["extra"]["sweep_many_rows_gemm"] = sweep_many_rows(torch, zq, ggml)
            except Exception as e:
                line["extra"]["sweep_many_rows_gemm"] = {"error": repr(e)}
        print(json.dumps(line), flush=True)
    if use_dist:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
