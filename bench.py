"""Benchmark of the Qwen3 token loop on B200: batch-1 greedy decode of the Qwen3-4B architecture in Q4.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the configuration the metric is quoted on): 36 layers, hidden 2560, FFN 9728, 32 query / 8 KV
heads, head_dim 128, vocab 151936, tied embeddings; weights N(0, 0.02) from a seed, norms 1, quantised to
the `.brasa` layout (q4_0 linears, q6_0 embedding/lm_head); a seeded 512-token prompt, then 256 greedy
tokens with an f16 KV cache, ctx 2048. One step = the 255 decode forwards that follow the first token
(decode tok/s = (generated - 1) / decode time, the reference's GenStats::decode_tok_s).

`value`   device-resident: the chosen token is fed back on the device, timed with CUDA events.
`e2e`     through Session.generate with host buffers: prompt upload, prefill, and one token id read
          back per step, timed by the session itself (host clock around the decode loop).
`roofline` the dominant kernel, the one-launch-per-token decode kernel: algorithmic bytes of a token over its
          event-timed duration, against the measured HBM copy peak (`gemv_roofline`: the q4_0 GEMV of the
          kernel-per-operation path alone over 36 layers of gate/up weights, 1 GB).
`prefill_16k` a 16 384-token prompt through chunked prefill, f16 and q8_0 caches, and decode over that cache.
`serving` 64 sequences per replica (shared 2048-token prefix + 1024 own tokens each, paged f16 KV), 512 sampled
          tokens per sequence (temperature 0.7, top-p 0.95, one PCG32 stream per sequence).
`cpu_baseline` the oracle's C port of the reference CPU path on the host cores: 32 teacher-forced decode tokens over the
          GPU's own prefill cache, which doubles as the full-size parity check (logit error, tie rule, smallest top-2 gap).
          The keys `gemv_roofline`, `prefill_16k.q8_0` and `serving` carry a CPU baseline of their own configuration.
`tp32b`   the Qwen3-32B architecture decoded tensor-parallel over all ranks of the job (batch 1 and batch 16), with a
          split-versus-unsplit parity check on a reduced model; at one rank the whole model runs on one GPU.

With --gpus N > 1 (launched by torch.distributed.run) every rank serves its own replica: the path has
no exchange step at batch 1, so the ranks share nothing and the aggregate is the sum ("replicas only").
--impl reference times the reference's CPU path alone (rank 0 only): tools/qwen3_ref.py from oracle/_ref/ when that was
made (oracle/make_ref.py), else the oracle's C port.
"""

from __future__ import annotations

import argparse
import json
import os
import pathlib
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PROMPT, GENERATE, CTX = 512, 256, 2048
SEED = 20251
# dram__bytes_read + dram__bytes_write of one gate/up + SwiGLU GEMV launch under ncu (algorithmic bytes: 28 065 792)
GATE_UP_TRAFFIC_BYTES = 28_130_000
# dram__bytes_read + dram__bytes_write of one decode_token_kernel launch at position 512 under ncu (algorithmic bytes at
# that position: 2 436 050 976)
TOKEN_KERNEL_TRAFFIC_BYTES = 2_452_740_000
# dram__bytes_read + dram__bytes_write of one serving decode step of 64 sequences (all its kernels, summed) under ncu,
# captured at the first steps of the leg, where a step's algorithmic bytes are the second figure; the leg scales the
# traffic to its own mean position by its algorithmic bytes (the KV share grows in proportion, the weights do not move).
# ncu empties the caches before every kernel, so the GEMMs' partial tiles (about 1.0 GB of this) come back from DRAM
# there and out of L2 in the timed run: an upper bound.
SERVING_STEP_TRAFFIC_BYTES = 15_283_000_000
SERVING_STEP_TRAFFIC_AT_ALGORITHMIC_BYTES = 12_387_561_504
METRIC = "qwen3_4b_q4_bs1_decode_tok_s"
WORKLOAD = "qwen3-4b-arch q4_0/q6_0 .brasa, bs1, 512-token seeded prompt + 256 greedy tokens, KV f16, ctx 2048"


def measured_peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = max(mx, float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        # samples under load: drop the idle tail below half of the top clock seen
        busy = [v for v in sm if v >= 0.5 * max(sm)] if sm else []
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


def tensor_peak() -> float | None:
    """Measured dense bf16 TFLOP/s (sustained figure: the prefill runs for about a second)."""
    p = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(p.read_text())["bf16_tflops_sustained"])
    except Exception:
        return None


def workload_config(world: int) -> dict:
    """The `config` of the JSON line: the same for the GPU arm and for the reference arm."""
    return {"workload": WORKLOAD, "l2": "inputs larger than L2: 2.36 GB of weights are read per token",
            "parallelism": f"replicas x{world}" if world > 1 else "single GPU"}


def prompt_ids(vocab: int) -> np.ndarray:
    return np.random.default_rng(SEED).integers(0, vocab, size=PROMPT).astype(np.uint32)


def model_path(tag: str) -> pathlib.Path:
    d = pathlib.Path(os.environ.get("BRASA_BENCH_DIR", "/tmp/brasa_bench"))
    d.mkdir(parents=True, exist_ok=True)
    return d / f"{tag}-seed{SEED}.brasa"


# ---- the CPU arm ------------------------------------------------------------------------------------

def cpu_decode_sample(brasa_path, kv_rows, first_ids, pos0: int, tokens: int):
    """Decodes `tokens` tokens with the oracle's C port starting at pos0 over a given KV cache
    (kv_rows: per layer (k, v) float arrays [pos0, kv_dim]) or a zero cache. Returns (seconds per token, logits)."""
    import oracle
    from oracle import brasa_format
    f = brasa_format.BrasaFile(brasa_path)
    orc = oracle.Qwen3Oracle(f, kv="f16", ctx=pos0 + tokens + 1)
    if kv_rows is not None:
        for li, (k, v) in enumerate(kv_rows):
            orc.k[li, :pos0] = k
            orc.v[li, :pos0] = v
    orc.pos = pos0
    times, logits = [], []
    for t in range(tokens):
        t0 = time.perf_counter()
        lg = orc.forward([int(first_ids[t])])
        times.append(time.perf_counter() - t0)
        logits.append(lg[0])
    return times, logits


def write_model_cpu(path, cfg: dict):
    """The workload's `.brasa` file made on the host alone (the reference arm runs without a GPU): seeded N(0, 0.02)
    matrices, norm vectors of ones, quantised with the oracle's restatement of the reference quantisers, tensors
    drawn and quantised in parallel. Same layout, shapes and distribution as brasa_b200.synth.write_synthetic_model."""
    import concurrent.futures
    import hashlib

    import oracle
    from brasa_b200 import synth
    shapes = synth.tensor_shapes(cfg)
    names = sorted(shapes)

    def make(i: int):
        name = names[i]
        dt = synth.dtype_for(name, len(shapes[name]))
        n = int(np.prod(shapes[name]))
        if dt == "f32":
            data = np.ones(n, "<f4").tobytes()
        else:
            w = np.random.Generator(np.random.SFC64([SEED, i])).standard_normal(n, dtype=np.float32)
            w *= np.float32(0.02)
            data = oracle.quantize(oracle.QTYPE[dt], w).tobytes()
        return name, dt, data, hashlib.sha256(data).hexdigest()

    tensors = [{"name": nm, "dtype": synth.dtype_for(nm, len(shapes[nm])), "shape": shapes[nm], "nbytes": 0, "offset": 0, "sha256": "0" * 64}
               for nm in names]
    for t in tensors:
        t["nbytes"] = synth._nbytes(t["dtype"], t["shape"])
    meta = {"format": "brasa", "version": 1, "converter": "bench.py host generator",
            "model": {"family": "qwen3", "source_repo": "synthetic", "source_commit": f"seed-{SEED}", "config": cfg},
            "quant": {"block": 32, "scheme": "q4_0 linears, q6_0 embeddings/lm_head, f32 norms"}, "page": 16384, "tensors": tensors,
            "data_sha256": "0" * 64}
    off = 16384 * 12
    for t in tensors:
        t["offset"] = off
        off = (off + t["nbytes"] + 16383) // 16384 * 16384
    tmp = pathlib.Path(str(path) + f".{os.getpid()}.tmp")
    with open(tmp, "wb") as f:
        f.truncate(off)
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 1)) as ex:
            for i, (name, dt, data, sha) in enumerate(ex.map(make, range(len(names)))):
                tensors[i]["sha256"] = sha
                f.seek(tensors[i]["offset"])
                f.write(data)
        meta["data_sha256"] = hashlib.sha256("".join(t["sha256"] for t in tensors).encode()).hexdigest()
        hdr = synth._header(meta)
        assert len(hdr) <= 16384 * 12
        f.seek(0)
        f.write(hdr)
    os.replace(tmp, path)


def time_qwen3_ref(path, cfg: dict, ids: np.ndarray, warmup: int, steps: int):
    """The reference's own CPU forward (tools/qwen3_ref.py, staged under oracle/_ref/): prefill of the prompt, then
    single-token decode steps over its f16-rounded cache, dequantised layers kept in RAM so that a step is matmuls and
    not re-dequantisation. Returns (seconds per timed token, threads used, greedy token ids)."""
    import concurrent.futures
    import tempfile

    import torch

    import oracle
    sys.path.insert(0, str(ROOT / "oracle" / "_ref"))
    import brasa_file
    import qwen3_ref
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    # Dequantised tensors are kept in RAM (the tool re-reads and dequantises every layer on every call otherwise), and
    # they are filled by the oracle's C dequantiser, several tensors at a time: bit-identical to the tool's numpy
    # dequantiser (the golden tests hold both to the same bytes) and minutes faster for 4e9 weights. The forward itself,
    # prefill and decode steps, is the tool's own code.
    bf = brasa_file.BrasaFile(path)
    cache: dict = {}

    def fill(name):
        t = bf.tensors[name]
        data = np.asarray(bf.map[t["offset"]:t["offset"] + t["nbytes"]])
        if t["dtype"] == "f32":
            arr = data.view("<f4").astype(np.float32).reshape(t["shape"])
        else:
            arr = oracle.dequantize(oracle.QTYPE[t["dtype"]], data, int(np.prod(t["shape"]))).reshape(t["shape"])
        return name, torch.from_numpy(arr)
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(16, threads)) as ex:
        for name, ten in ex.map(fill, list(bf.tensors)):
            cache[name] = ten
    qwen3_ref.BrasaWeights.get = lambda self, name: cache[name]
    with tempfile.TemporaryDirectory() as td:
        (pathlib.Path(td) / "config.json").write_text(json.dumps(cfg))
        m = qwen3_ref.Qwen3Ref(td, brasa=path, kv_dtype=torch.float16)
    with torch.no_grad():
        caches = [m.new_cache()]
        logits = m.forward_many([torch.from_numpy(ids.astype(np.int64))], caches)[0]
        tok = int(logits[-1].argmax())
        times, toks = [], []
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            lg = m.forward_many([torch.tensor([tok])], caches)[0]
            nxt = int(lg[0].argmax())
            times.append(time.perf_counter() - t0)
            toks.append(tok)
            tok = nxt
    timed = times[warmup:]
    return sum(timed) / len(timed), threads, toks


def run_reference(args, rank: int):
    if rank != 0:
        return
    import oracle
    from brasa_b200 import synth
    oracle.build()
    cfg = synth.QWEN3_4B
    path = model_path("qwen3-4b")
    if not path.exists():
        write_model_cpu(path, cfg)
    cores = use_all_host_cores()
    ids = prompt_ids(cfg["vocab_size"])
    if (ROOT / "oracle" / "_ref" / "qwen3_ref.py").exists():
        sec, cores, _ = time_qwen3_ref(path, cfg, ids, args.warmup, args.steps)
        kind = "reference"
        sample = (f"{args.steps} greedy decode tokens at positions {PROMPT}.. of this workload after a CPU prefill of its {PROMPT}-token prompt: the "
                  f"reference's tools/qwen3_ref.py (torch CPU, {cores} threads, KV rounded to f16, dequantised layers kept in RAM), same model file "
                  f"as the GPU arm when that file is already on the machine")
    else:
        total = args.warmup + args.steps
        times, _ = cpu_decode_sample(path, None, ids[:total], PROMPT, total)
        timed = times[args.warmup:]
        sec = sum(timed) / len(timed)
        kind = "port"
        sample = (f"{args.steps} decode tokens at positions {PROMPT}.. of this workload, oracle C port (dequantise a row, f64 dot; OpenMP over rows), "
                  f"KV cache of {PROMPT} zero rows (no CPU prefill: the reference's own Python forward was not staged on this machine)")
    value = 1.0 / sec
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 activations and accumulation, q4_0/q6_0 weights, f16 KV", "data": "synthetic", "config": workload_config(args.gpus),
            "cpu_baseline": {"value": value, "unit": "tok/s", "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def use_all_host_cores() -> int:
    """OpenMP threads for the CPU legs: every host core, also under torchrun (which exports OMP_NUM_THREADS=1)."""
    import ctypes
    cores = os.cpu_count() or 1
    try:
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(cores)
    except OSError:
        pass
    return cores


# ---- the GPU arm ------------------------------------------------------------------------------------

def profiler_range(on: bool):
    """Marks the timed decode region for a profiler started with --profile-from-start off (no effect otherwise)."""
    try:
        from cuda.bindings import runtime as rt
    except ImportError:
        try:
            from cuda import cudart as rt
        except ImportError:
            return
    (rt.cudaProfilerStart if on else rt.cudaProfilerStop)()


def prefill_16k(B, ctx, path, cfg, kv_name: str, cpu_steps: int = 0):
    """The second half of the headline metric: a 16 384-token seeded prompt through chunked causal prefill, then the
    configuration's 128 greedy decode tokens over the long cache. The chunk is the reference's tunable `max_tokens`
    (default 1024 there, qwen3.rs:175-185); 3 584 tokens = 7 token tiles of 512 fill 140 of the 148 SMs in one wave of the
    2 560-row GEMMs (measured: 512 -> 19.4k, 1024 -> 21.5k, 2048 -> 24.6k, 3584 -> 27.9k, 4096 -> 27.0k tok/s).
    cpu_steps > 0: that many decode steps at position 16 384 on the host cores with the oracle's C port over the GPU's
    own cache (read back and dequantised), compared with the GPU's logits for the same steps. Returns a dict."""
    kvt = {"f16": B.KvType.F16, "q8_0": B.KvType.Q8_0}[kv_name]
    n_prompt, chunk, ntok = 16384, 3584, 128
    ids = np.random.default_rng(SEED + 16).integers(0, cfg["vocab_size"], size=n_prompt).astype(np.uint32)
    m = B.Qwen3.load(ctx, path, B.Limits(ctx=n_prompt + 256, max_tokens=chunk, max_logit_rows=1, kv=kvt))
    try:
        # the prompt goes through twice over the same positions and the faster pass is reported: one pass alone carries what
        # a process pays once (kernels loaded on first use, workspaces grown) or a moment of another clock
        passes = []
        lg = None
        for _ in range(2):
            secs = 0.0
            for off in range(0, n_prompt, chunk):
                lg, s = m.forward(ids[off:off + chunk], off, want_logits=off + chunk >= n_prompt)
                secs += s
            passes.append(secs)
        secs = min(passes)
        first = int(np.argmax(lg[0]))
        m.decode_greedy(first, n_prompt, 4)
        toks, dsecs = m.decode_greedy(first, n_prompt, ntok)
        # FLOPs of the prompt: 2 x weights per token (layers + one lm_head row set) + causal attention
        L, H, F, hq, hkv, D, V = (cfg[k] for k in ("num_hidden_layers", "hidden_size", "intermediate_size", "num_attention_heads",
                                                    "num_key_value_heads", "head_dim", "vocab_size"))
        w_layer = H * (hq + 2 * hkv) * D + hq * D * H + 3 * H * F
        flops = 2.0 * n_prompt * L * w_layer + 2.0 * V * H + 4.0 * hq * D * (n_prompt * (n_prompt + 1) / 2) * L
        from brasa_b200 import synth
        per_token = synth.weight_bytes_per_token(cfg) + synth.kv_bytes_per_position(cfg, kv_name) * (n_prompt + 1 + (ntok - 1) / 2.0)
        hbm, _ = measured_peaks()
        out = {"prompt_tokens": n_prompt, "chunk": chunk, "kv": kv_name, "prefill_tok_s": n_prompt / secs, "prefill_s": secs,
               "prefill_s_passes": passes, "tflops": flops / secs / 1e12, "decode_steps": ntok, "decode_tok_s_at_16k": ntok / dsecs,
               "decode_bytes_per_token": per_token, "decode_frac_of_measured_hbm": per_token * ntok / dsecs / 1e9 / hbm}
        if cpu_steps > 0:
            try:
                out["cpu_baseline"] = cpu_decode_over_gpu_cache(B, m, path, cfg, kv_name, n_prompt, [first] + [int(t) for t in toks[:cpu_steps - 1]])
            except Exception as e:  # reported, never required
                out["cpu_baseline"] = {"value": None, "sample": f"failed: {e}"}
        return out
    finally:
        m.free()


def cpu_decode_over_gpu_cache(B, m, path, cfg, kv_name: str, pos0: int, feed: list[int]):
    """Teacher-forced decode steps at position pos0 with the oracle's C port over the cache the GPU model `m` holds for
    positions [0, pos0), against the GPU's logits for the same tokens. Returns a cpu_baseline dict with the parity figures."""
    import oracle
    from oracle import brasa_format
    oracle.build()
    cores = use_all_host_cores()
    kvd = cfg["num_key_value_heads"] * cfg["head_dim"]
    orc = oracle.Qwen3Oracle(brasa_format.BrasaFile(path), kv=kv_name, ctx=pos0 + len(feed) + 1)
    for li in range(cfg["num_hidden_layers"]):
        for which, dst in (("k", orc.k), ("v", orc.v)):
            raw = m.read_kv(li, which, 0, pos0)
            vals = oracle.dequantize_kv_q8(raw) if kv_name == "q8_0" else raw.view(np.float16).astype(np.float32)
            dst[li, :pos0] = vals.reshape(pos0, kvd)
    orc.pos = pos0
    times, worst, same, gap = [], 0.0, True, float("inf")
    for i, tok in enumerate(feed):
        t0 = time.perf_counter()
        want = orc.forward([tok])[0]
        times.append(time.perf_counter() - t0)
        got, _ = m.forward([tok], pos0 + i)
        worst = max(worst, float(np.abs(got[0] - want).max() / np.abs(want).max()))
        top2 = np.sort(want)[-2:]
        gap = min(gap, float(top2[1] - top2[0]))
        same = same and int(np.argmax(got[0])) == int(np.argmax(want))
    sec = statistics.median(times)
    return {"value": 1.0 / sec, "unit": "tok/s", "cores": cores, "kind": "port",
            "sample": f"{len(feed)} teacher-forced decode tokens at positions {pos0}.. over the GPU's own {kv_name} cache, oracle C port with OpenMP",
            "parity_max_rel_logit_err": worst, "parity_same_greedy_tokens": same, "parity_min_top2_gap": gap}


def serving_leg(B, ctx, path, cfg, rank: int, seqs: int = 64, prefix: int = 2048, suffix: int = 1024, steps: int = 512):
    """Batched serving on one replica: `seqs` sequences that share a `prefix`-token prompt head (computed once, its KV pages
    attached to every sequence) and each carry `suffix` tokens of their own, then `steps` sampled tokens per sequence
    (temperature 0.7, top-p 0.95, one PCG32 stream per sequence) over f16 KV in 16-token pages. Returns a dict."""
    V = cfg["vocab_size"]
    page, warm = B.Batch.PAGE, 4
    positions = (prefix + suffix + warm + steps + 1 + page - 1) // page * page  # the most one sequence ever holds
    m = B.Qwen3.load(ctx, path, B.Limits(ctx=positions, max_tokens=suffix, max_logit_rows=1, kv=B.KvType.F16))  # a sequence's own prompt is one chunk
    own_pages = (positions - prefix) // page
    batch = B.Batch(m, seqs, prefix // page + seqs * own_pages + 8, positions)
    try:
        params = B.SamplingParams(temperature=0.7, top_k=0, top_p=0.95, seed=SEED + 1000 * rank)
        shared = np.random.default_rng(SEED + 4).integers(0, V, size=prefix).astype(np.uint32)
        t0 = time.perf_counter()
        batch.set_prefix(shared)
        t_prefix = time.perf_counter() - t0
        ttft = []
        for i in range(seqs):
            own = np.random.default_rng(SEED + 5 + i + 1000 * rank).integers(0, V, size=suffix).astype(np.uint32)
            t1 = time.perf_counter()
            batch.add_sequence(own, params)
            ttft.append(time.perf_counter() - t1)
        t_admit = time.perf_counter() - t0
        batch.decode(warm, params)  # warm-up steps (they advance the sequences by `warm` positions)
        profiler_range(True)
        ids, secs = batch.decode(steps, params)
        profiler_range(False)
        kvb = synth_kv_bytes(cfg)
        mean_pos = prefix + suffix + warm + 1 + (steps - 1) / 2.0
        step_bytes = weight_bytes(cfg) + seqs * kvb * mean_pos
        # the shared prefix is read once per group of four sequences, not once per sequence: what must cross HBM
        own_pos = mean_pos - prefix
        min_bytes = weight_bytes(cfg) + kvb * (prefix + seqs * own_pos)
        hbm, hbm_kind = measured_peaks()
        t_step = secs / steps
        roof = {"bound": "hbm", "kernel": "one decode step of 64 sequences (paged attention + 64-token GEMMs + sampler)",
                "achieved": min_bytes / t_step / 1e9, "peak": hbm, "unit": "GB/s", "frac": min_bytes / t_step / 1e9 / hbm, "peak_source": hbm_kind,
                "algorithmic_bytes_per_step": min_bytes,
                "traffic": SERVING_STEP_TRAFFIC_BYTES * min_bytes / SERVING_STEP_TRAFFIC_AT_ALGORITHMIC_BYTES,
                "note": "numerator: weights once + the shared prefix's KV once + every sequence's own KV; `achieved_gbs` below counts the "
                        "prefix once per sequence, as the configuration's 33.77 GB per step does"}
        return {"sequences": seqs, "roofline": roof, "shared_prefix_tokens": prefix, "own_prompt_tokens": suffix, "decode_steps": steps,
                "sampling": "temperature 0.7, top-p 0.95, top-k 0, PCG32 per sequence", "kv": "f16, pages of 16 positions",
                "decode_tok_s": seqs * steps / secs, "ms_per_step": secs / steps * 1e3,
                "prefix_prefill_s": t_prefix, "admit_all_s": t_admit, "ttft_s_median": statistics.median(ttft), "ttft_s_max": max(ttft),
                "prefix_cache": batch.prefix_cache_stats(), "pages_in_use": batch.pages_in_use,
                "kv_resident_gib": batch.pages_in_use * page * kvb / 2**30,
                "algorithmic_bytes_per_step": step_bytes, "achieved_gbs": step_bytes / (secs / steps) / 1e9,
                "distinct_tokens": int(np.unique(ids).size)}
    finally:
        batch.free()
        m.free()


def weight_bytes(cfg) -> int:
    from brasa_b200 import synth
    return synth.weight_bytes_per_token(cfg)


def synth_kv_bytes(cfg) -> int:
    from brasa_b200 import synth
    return synth.kv_bytes_per_position(cfg, "f16")


def tp_leg(B, ctx, rep, steps: int = 3, prompt: int = 1024, generate: int = 256):
    """Qwen3-32B-architecture batch-1 decode, tensor-parallel over the ranks of this job: every rank holds its share of the
    heads, FFN rows and lm_head rows (random init, q4_0; the q6_0 embedding table replicated), a 1024-token prompt is
    prefilled in 512-token chunks, then `generate` greedy tokens run device-resident with the two sums over ranks of every
    layer and the argmax exchange done by the ranks' own kernels through peer memory. Returns a dict (every rank calls)."""
    from brasa_b200 import synth
    from brasa_b200 import tp as TP
    rank, world = rep.rank, rep.world
    cfg = TP.shard_config(synth.QWEN3_32B, rank, world)
    path = model_path(f"qwen3-32b-tp{world}-rank{rank}")
    if not path.exists():
        tmp = path.with_suffix(".tmp")
        synth.write_synthetic_model(ctx, tmp, cfg, seed=SEED)
        os.replace(tmp, path)
    limits = B.Limits(ctx=2048, max_tokens=512, max_logit_rows=1, kv=B.KvType.F16)
    m = B.Qwen3.load(ctx, path, limits)
    load = m.load_stats()
    tp = TP.TensorParallel(ctx, rank, world, limits.max_tokens * cfg["hidden_size"])
    m.set_tp(tp)
    try:
        ids = np.random.default_rng(SEED + 32).integers(0, cfg["vocab_size"], size=prompt).astype(np.uint32)
        rep.barrier()
        pre_s, lg = 0.0, None
        for off in range(0, prompt, 512):
            lg, s = m.forward(ids[off:off + 512], off, want_logits=off + 512 >= prompt)
            pre_s += s
        # the first generated token: the best logit over every rank's rows (ties to the lower index)
        best = float(np.nanmax(lg[0]))
        cand = int(np.flatnonzero(lg[0] == best)[0]) + m.cfg["head_row0"]
        top = rep.max(best)
        first = int(-rep.max(-(cand if best == top else 2**31)))
        rep.barrier()
        m.decode_greedy(first, prompt, 16)
        secs, toks = [], None
        for _ in range(steps):
            rep.barrier()
            toks, s = m.decode_greedy(first, prompt, generate)
            secs.append(s)
        total = rep.max(float(sum(secs)))
        agree = rep.max(float(int(toks[-1]))) == -rep.max(-float(int(toks[-1])))
        shard_bytes = synth.weight_bytes_per_token(cfg)
        kvb = synth.kv_bytes_per_position(cfg, "f16")
        per_token = shard_bytes + kvb * (prompt + 1 + (generate - 1) / 2.0)
        t_tok = total / (steps * generate)
        # batch 16: sixteen sequences with their own 1024-token prompts decoded together over paged KV, greedy
        nb, warm = 16, 4
        page = B.Batch.PAGE
        per_seq = (prompt + generate + page) // page
        bt = B.Batch(m, nb, nb * per_seq + 8, per_seq * page)
        try:
            for i in range(nb):
                own = np.random.default_rng(SEED + 64 + i).integers(0, cfg["vocab_size"], size=prompt).astype(np.uint32)
                rep.barrier()
                bt.add_sequence(own)
            rep.barrier()
            bt.decode(warm)
            rep.barrier()
            bids, bsecs = bt.decode(generate - warm - 1)
            bsecs = rep.max(bsecs)
            b_agree = rep.max(float(int(bids[:, -1].sum()))) == -rep.max(-float(int(bids[:, -1].sum())))
            batch16 = {"sequences": nb, "decode_steps": generate - warm - 1, "decode_tok_s": nb * (generate - warm - 1) / bsecs,
                       "ms_per_step": bsecs / (generate - warm - 1) * 1e3, "ranks_agree_on_tokens": bool(b_agree)}
        finally:
            bt.free()
        return {"batch16": batch16, "model": "Qwen3-32B architecture, q4_0, random init", "tp": world, "prompt_tokens": prompt, "generated": generate,
                "decode_tok_s": 1.0 / t_tok, "ms_per_token": t_tok * 1e3, "prefill_tok_s": prompt / rep.max(pre_s),
                "bytes_per_token_per_gpu": per_token, "achieved_gbs_per_gpu": per_token / t_tok / 1e9,
                "exchanges_per_token": 2 * cfg["num_hidden_layers"] + 1, "ranks_agree_on_tokens": bool(agree),
                "batch": 1, "shard_load": load}
    finally:
        m.free()
        tp.free()


def tp_parity(B, ctx, rep):
    """Split against unsplit on a reduced untied model (3 layers, hidden 512, 16 query / 8 KV heads, FFN 2048, vocabulary
    1024): rank 0 writes the model and its `world` shards, every rank runs its shard through the exchange (a 40-token
    prefill, one decode forward, 12 device-resident greedy tokens), and rank 0 compares the concatenated logits rows and
    the tokens with the unsplit model on its own GPU. Bounds as in the two-process test: 2e-3 of max |logit| (f16 prefill
    inputs; the split only changes the order of the sums over o_proj's and down_proj's columns). Every rank calls."""
    from brasa_b200 import tp as TP
    rank, world = rep.rank, rep.world
    d = model_path("x").parent / f"tp_parity_w{world}"
    full = d / "full.brasa"
    n_prompt, steps = 40, 12
    if rank == 0:
        import oracle
        from oracle import brasa_format as BF
        oracle.build()
        d.mkdir(parents=True, exist_ok=True)
        cfg = BF.tiny_config(layers=3, hidden=512, heads=16, kv_heads=8, ffn=2048, vocab=1024)
        cfg["tie_word_embeddings"] = False
        BF.write_brasa(full, cfg, BF.synth_weights(cfg, seed=29, std=0.04, norm_jitter=0.1))
        TP.split_model(full, [d / f"shard{r}.brasa" for r in range(world)])
    rep.barrier()
    limits = B.Limits(ctx=256, max_tokens=64, max_logit_rows=1, kv=B.KvType.F16)
    m = B.Qwen3.load(ctx, d / f"shard{rank}.brasa", limits)
    tp = TP.TensorParallel(ctx, rank, world, limits.max_tokens * m.cfg["hidden"])
    m.set_tp(tp)
    try:
        ids = np.random.default_rng(5).integers(0, 1024, size=n_prompt).astype(np.uint32)
        rep.barrier()
        logits, _ = m.forward(ids, 0)
        one, _ = m.forward(ids[:1], n_prompt)
        rep.barrier()
        toks, _ = m.decode_greedy(int(ids[0]), n_prompt, steps)
        np.savez(d / f"rank{rank}.npz", logits=logits, one=one, toks=toks, row0=m.cfg["head_row0"])
        rep.barrier()
    finally:
        m.free()
        tp.free()
    if rank != 0:
        return None
    ranks = [np.load(d / f"rank{r}.npz") for r in range(world)]
    plain = B.Qwen3.load(ctx, full, limits)
    try:
        want, _ = plain.forward(ids, 0)
        want1, _ = plain.forward(ids[:1], n_prompt)
        want_t, _ = plain.decode_greedy(int(ids[0]), n_prompt, steps)
    finally:
        plain.free()
    got = np.concatenate([r["logits"] for r in ranks], axis=1)
    got1 = np.concatenate([r["one"] for r in ranks], axis=1)
    e_pre = float(np.abs(got - want).max() / np.abs(want).max())
    e_dec = float(np.abs(got1 - want1).max() / np.abs(want1).max())
    agree = all(list(r["toks"]) == list(ranks[0]["toks"]) for r in ranks)
    same = list(ranks[0]["toks"]) == list(want_t)
    return {"model": "3 layers, hidden 512, 16 query / 8 KV heads, FFN 2048, vocabulary 1024, untied lm_head", "world": world,
            "max_rel_logit_err_prefill": e_pre, "max_rel_logit_err_decode": e_dec, "bound": 2e-3, "within_bound": e_pre <= 2e-3 and e_dec <= 2e-3,
            "ranks_agree_on_tokens": bool(agree), "greedy_tokens_match_unsplit": bool(same), "greedy_tokens": steps}


def two_device_check(B) -> str:
    """Two contexts on two devices inside this one process (rank 0): a small model prefilled, decoded by the whole-token
    kernel and stepped as a paged batch on each device must give the same tokens on both, and the allocation-free
    decode attention must equal the allocating one on the second device too."""
    import tempfile

    import torch
    if torch.cuda.device_count() < 2:
        return "one GPU visible"
    from oracle import brasa_format as BF
    results = []
    with tempfile.TemporaryDirectory() as td:
        path = pathlib.Path(td) / "model.brasa"
        cfg = BF.tiny_config(layers=2, hidden=256, heads=4, kv_heads=2, ffn=512, vocab=512)
        BF.write_brasa(path, cfg, BF.synth_weights(cfg, seed=3, std=0.05, norm_jitter=0.1))
        for dev in (1, 0):
            c = B.Context(dev)
            try:
                K = B.Kernels(c)
                m = B.Qwen3.load(c, path, B.Limits(ctx=512, max_tokens=256, max_logit_rows=1, kv=B.KvType.F16))
                prompt = np.arange(200, dtype=np.uint32) % 512
                lg, _ = m.forward(prompt, 0)  # 200 tokens: the tensor-core GEMM and attention kernels
                first = int(np.argmax(lg[0]))
                toks, _ = m.decode_greedy(first, 200, 6)
                bt = B.Batch(m, max_seqs=3, num_pages=48, max_positions=256)
                bt.set_prefix(prompt[:192])
                for _ in range(3):
                    bt.add_sequence(prompt[192:])
                ids, _ = bt.decode(6)
                bt.free()
                m.free()
                g = np.random.default_rng(dev)
                hq, hkv, dim, lk = 8, 2, 128, 300
                q = c.buffer_from(g.standard_normal(hq * dim).astype(np.float32))
                k = c.buffer_from(g.standard_normal(lk * hkv * dim).astype(np.float16))
                v = c.buffer_from(g.standard_normal(lk * hkv * dim).astype(np.float16))
                o1, o2 = c.buffer(hq * dim * 4), c.buffer(hq * dim * 4)
                part = c.buffer(B.decode_partials_len(hq, lk) * 4)
                sh = B.AttnShape(1, hq, hkv, dim, lk - 1, B.KvType.F16)
                cmd = c.command()
                K.decode_attention(cmd, q, k, v, part, o1, sh)
                K.decode_attention_static(cmd, q, k, v, o2, sh)
                cmd.wait()
                if not np.array_equal(o1.download(np.float32), o2.download(np.float32)):
                    return f"static decode attention differs on device {dev}"
                results.append(([first] + [int(t) for t in toks], ids.tolist()))
            finally:
                c.close()
    if results[0] != results[1]:
        return "devices 0 and 1 disagree"
    if any(row != results[0][0] for row in results[0][1]):
        return "batch and single-sequence tokens disagree"
    return "ok"


def serving_cpu_baseline(B, ctx, K, path, cfg):
    """Configuration 4 on the host cores: four sequences decoded one token each at position 3 072 with the oracle's C
    port (zero KV rows: CPU speed does not depend on the values), and the reference's sampler (temperature 0.7, top-p
    0.95) restated in C on vocabulary-sized logits. Also the device sampler's identity rate against that sampler on
    the same logits and PCG32 streams at the real vocabulary."""
    import oracle
    oracle.build()
    cores = use_all_host_cores()
    V = cfg["vocab_size"]
    feed = np.random.default_rng(SEED + 77).integers(0, V, size=4)
    times, logits = cpu_decode_sample(path, None, feed, 3072, 4)
    rng = np.random.default_rng(SEED + 78)
    rows, draws = 16, 8
    refs = [oracle.Sampler(temperature=0.7, top_k=0, top_p=0.95, seed=500 + r) for r in range(rows)]
    states = ctx.buffer_from(np.concatenate([B.pcg32_state(500 + r) for r in range(rows)]))
    scratch, out = ctx.buffer(rows * V * 8), ctx.buffer(rows * 4)
    agree = total = 0
    t_sample = []
    for _ in range(draws):
        lg = (rng.standard_normal((rows, V)) * 3.0).astype(np.float32)
        g = ctx.buffer_from(lg)
        cmd = ctx.command()
        K.sample_rows(cmd, g, V, rows, 0.7, 0, 0.95, states, scratch, out)
        cmd.wait()
        got = out.download(np.uint32, rows)
        for r in range(rows):
            t0 = time.perf_counter()
            want = refs[r].sample(lg[r])
            t_sample.append(time.perf_counter() - t0)
            total += 1
            agree += int(got[r]) == want
        g.free()
    sec = statistics.median(times) + statistics.median(t_sample)
    return {"value": 1.0 / sec, "unit": "tok/s per sequence", "cores": cores, "kind": "port",
            "sample": "4 sequences, one decode token each at position 3072 (zero KV rows) with the oracle C port + the C restatement of "
                      "sampler.rs on 151 936 logits; not scaled to 64 sequences",
            "cpu_sampler_ms": statistics.median(t_sample) * 1e3,
            "device_sampler_identity_rate_at_vocab": agree / total, "device_sampler_draws_compared": total}


def gemv_cpu_baseline(cfg):
    """Configuration 1 on the host: W [9728 x 2560] ~ N(0, 0.02) quantised to q4_0, x ~ N(0, 1) rounded to f16; the
    oracle's restatement of reference::matmul (dequantise a row, f64 dot) on one thread and on all cores, and numpy
    (dequantise the matrix, then W @ x in f32). Microseconds per GEMV."""
    import ctypes

    import oracle
    oracle.build()
    rows, cols = cfg["intermediate_size"], cfg["hidden_size"]
    g = np.random.default_rng(SEED + 1)
    w = (g.standard_normal(rows * cols, dtype=np.float32) * np.float32(0.02))
    raw = oracle.quantize(oracle.Q4_0, w)
    x = g.standard_normal(cols).astype(np.float16).astype(np.float32)
    cores = os.cpu_count() or 1
    omp = None
    try:
        omp = ctypes.CDLL("libgomp.so.1")
    except OSError:
        pass

    def timed(fn, reps):
        fn()
        ts = []
        for _ in range(reps):
            t0 = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t0)
        return statistics.median(ts)
    if omp:
        omp.omp_set_num_threads(1)
    t1 = timed(lambda: oracle.matmul(oracle.Q4_0, raw, rows, cols, x), 3)
    if omp:
        omp.omp_set_num_threads(cores)
    tn = timed(lambda: oracle.matmul(oracle.Q4_0, raw, rows, cols, x), 5)
    wf = oracle.dequantize(oracle.Q4_0, raw, rows * cols).reshape(rows, cols)
    t_np = timed(lambda: wf @ x, 5)
    t_np_deq = timed(lambda: oracle.dequantize(oracle.Q4_0, raw, rows * cols).reshape(rows, cols) @ x, 2)
    return {"unit": "us per GEMV", "cores": cores, "kind": "port", "c_single_thread_us": t1 * 1e6, "c_all_cores_us": tn * 1e6,
            "numpy_matvec_on_dequantised_us": t_np * 1e6, "numpy_dequantise_then_matvec_us": t_np_deq * 1e6,
            "value": 1.0 / tn, "sample": "one gate-projection GEMV [9728 x 2560] q4_0, N(0, 0.02) weights, f16-rounded N(0, 1) input"}


def kernel_roofline(B, ctx, K, cfg, peak, peak_kind, profile=False):
    """The dominant kernel alone: gate/up GEMV + SwiGLU over 36 distinct weight pairs (1 GB) in one CUDA graph."""
    roof = None
    try:
        rows, cols = cfg["intermediate_size"], cfg["hidden_size"]
        nlayers = cfg["num_hidden_layers"]
        per = B.qtype_nbytes(B.WeightType.Q4_0, rows * cols)
        # distinct random matrices: generate once, quantise, tile; 72 buffers of 14 MB
        f32buf, filebuf = ctx.buffer(rows * cols * 4), ctx.buffer(per)
        mats = []
        for i in range(2 * nlayers):
            dst = ctx.buffer(per)
            cmd = ctx.command()
            K.randn(cmd, f32buf, rows * cols, SEED + 7, i * rows * cols, 0.02)
            K.quantize(cmd, B.WeightType.Q4_0, f32buf, filebuf, rows * cols)
            K.repack(cmd, B.WeightType.Q4_0, filebuf, dst, rows, cols)
            cmd.wait()
            mats.append(B.QMatrix(dst, B.WeightType.Q4_0, rows, cols, B.Layout.TILED))
        x = np.random.default_rng(1).standard_normal(cols).astype(np.float16).astype(np.float32)
        gx, gw = ctx.buffer_from(x), ctx.buffer_from(np.ones(cols, np.float32))
        gxw, gss, gy = ctx.buffer(cols * 4), ctx.buffer(B.norm_partials(cols) * 4), ctx.buffer(rows * 4)
        cmd = ctx.command()
        K.add_norm_prep(cmd, gx, None, gw, gxw, gss, cols)
        cmd.wait()
        graph = ctx.capture(lambda c: [K.gemv_scaled_swiglu(c, mats[2 * i], mats[2 * i + 1], gxw, gss, 1e-6, gy) for i in range(nlayers)])
        best = []
        for i in range(8):
            if profile and i == 7:
                profiler_range(True)
            cmd = ctx.command()
            graph.launch(cmd)
            best.append(cmd.wait())
        if profile:
            profiler_range(False)
        t_launch = statistics.median(best[3:]) / nlayers
        algo = 2 * per + cols * 4 + rows * 4
        ach = algo / t_launch / 1e9
        roof = {"bound": "hbm", "kernel": "gemv_rows_kernel<q4_0> gate+up+SwiGLU [2x9728x2560]", "achieved": ach, "peak": peak, "unit": "GB/s",
                "frac": ach / peak, "peak_source": peak_kind, "us_per_launch": t_launch * 1e6, "algorithmic_bytes_per_launch": algo,
                "traffic": GATE_UP_TRAFFIC_BYTES}
    except B.BrasaError as e:  # out of memory on a shared device: report the token-level figure only
        roof = {"bound": "hbm", "error": str(e), "achieved": None, "peak": peak, "unit": "GB/s", "frac": None, "traffic": None}
    return roof


def run_ours(args, rank: int, world: int, local_rank: int):
    import brasa_b200 as B
    from brasa_b200 import synth
    from brasa_b200.replicas import Replicas
    rep = Replicas("nccl" if world > 1 else None)  # replicas only: the ranks share a barrier and a few scalars
    dist = rep.dist
    ctx = B.Context(local_rank)
    cfg = synth.QWEN3_4B
    if args.only_kernel:
        if rank == 0:
            peak, peak_kind = measured_peaks()
            print(json.dumps({"roofline": kernel_roofline(B, ctx, B.Kernels(ctx), cfg, peak, peak_kind, profile=True),
                              "note": "dominant kernel alone (profiling run)"}))
        return
    if args.only_attention:
        # the prefill attention kernel alone at long context: 512 queries of 32 heads at positions 15 872.. over a
        # 16 384-position f16 cache of 8 KV heads (67 MB; inputs seeded normal), small enough for profiler captures
        if rank == 0:
            K = B.Kernels(ctx)
            g = np.random.default_rng(SEED + 9)
            hq, hkv, dim, tokens, pos0 = 32, 8, 128, 512, 15872
            kc = ctx.buffer_from(g.standard_normal((pos0 + tokens) * hkv * dim).astype(np.float16))
            vc = ctx.buffer_from(g.standard_normal((pos0 + tokens) * hkv * dim).astype(np.float16))
            q = ctx.buffer_from(g.standard_normal(tokens * hq * dim).astype(np.float32))
            o = ctx.buffer(tokens * hq * dim * 2)
            shape = B.AttnShape(tokens, hq, hkv, dim, pos0, B.KvType.F16)
            for _ in range(3):
                cmd = ctx.command()
                K.flash_attention(cmd, q, kc, vc, o, shape)
                cmd.wait()
            profiler_range(True)
            cmd = ctx.command()
            K.flash_attention(cmd, q, kc, vc, o, shape)
            secs = cmd.wait()
            profiler_range(False)
            flops = 4.0 * hq * dim * sum(pos0 + t + 1 for t in range(tokens))
            print(json.dumps({"metric": "prefill_attention_tflops", "value": flops / secs / 1e12, "unit": "TFLOP/s", "us": secs * 1e6,
                              "config": {"queries": tokens, "first_position": pos0, "heads": hq, "kv_heads": hkv, "kv": "f16"},
                              "note": "prefill attention kernel alone (profiling run)"}))
        return
    if args.only_tp:
        res = tp_leg(B, ctx, rep, steps=args.steps)
        if rank == 0:
            peak, peak_kind = measured_peaks()
            res["frac_of_measured_hbm_per_gpu"] = res["achieved_gbs_per_gpu"] / peak
            print(json.dumps({"metric": "qwen3_32b_tp_decode_tok_s", "value": res["decode_tok_s"], "unit": "tok/s", "n_gpus": world,
                              "scaling": "strong", "tp": res, "note": "tensor-parallel 32B decode leg (run on its own)"}))
        if dist:
            dist.barrier()
        rep.close()
        return
    path = model_path("qwen3-4b")
    if rank == 0 and not path.exists():
        tmp = path.with_suffix(".tmp")
        synth.write_synthetic_model(ctx, tmp, cfg, seed=SEED)
        os.replace(tmp, path)
    if dist:
        dist.barrier()
    ids = prompt_ids(cfg["vocab_size"])
    sess = B.Session(ctx, path, B.Limits(ctx=CTX, max_tokens=512, max_logit_rows=1, kv=B.KvType.F16))
    model = sess.model
    load_stats = model.load_stats()
    K = B.Kernels(ctx)

    if args.only_serving:
        sess.free()
        res = serving_leg(B, ctx, path, cfg, rank, seqs=args.serving_seqs, steps=args.serving_steps)
        if rank == 0:
            print(json.dumps({"metric": "serving_decode_tok_s", "value": res["decode_tok_s"], "unit": "tok/s", "serving": res,
                              "note": "batched serving leg only (profiling run)"}))
        return

    if args.only_prefill:
        model.forward(ids, 0, want_logits=False)
        profiler_range(True)
        _, secs = model.forward(ids, 0)
        ctx.sync()
        profiler_range(False)
        if rank == 0:
            print(json.dumps({"metric": "prefill_tok_s", "value": PROMPT / secs, "unit": "tok/s", "ms": secs * 1e3,
                              "config": {"workload": WORKLOAD, "tokens": PROMPT}, "note": "one prefill forward (profiling run)"}))
        return

    # ---- device-resident decode (value) ----
    logits, _ = model.forward(ids, 0)
    first = int(np.argmax(logits[0]))
    steps_tokens = args.decode_tokens
    for _ in range(args.warmup):
        model.decode_greedy(first, PROMPT, steps_tokens)
    if dist:
        dist.barrier()
    ctx.sync()
    launches0 = ctx.launch_count()
    dev_s, out_ids = [], None
    profiler_range(True)
    with ClockSampler(local_rank) as clocks:
        for _ in range(args.steps):
            out_ids, s = model.decode_greedy(first, PROMPT, steps_tokens)
            dev_s.append(s)
        ctx.sync()
    profiler_range(False)
    launches = ctx.launch_count() - launches0
    if dist:
        dist.barrier()
    total_s = rep.max(float(sum(dev_s)))  # the job is as slow as its slowest replica
    value = rep.sum(args.steps * steps_tokens) / total_s
    if args.only_decode:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                              "ms_per_step": total_s / args.steps * 1e3, "config": {"workload": WORKLOAD, "tokens_per_step": steps_tokens},
                              "gpu_launches": int(launches), "model_load": load_stats, "note": "decode loop only (profiling run)"}))
        return

    # ---- end to end through Session.generate (host buffers) ----
    e2e_vals, prefill_vals = [], []
    for i in range(args.warmup + args.steps):
        sess.reset()
        gen, st = sess.generate(ids, GENERATE)
        if i >= args.warmup:
            e2e_vals.append(st.decode_tok_s())
            prefill_vals.append(st.prefill_tok_s())
    e2e = statistics.median(e2e_vals)
    same_tokens = bool(out_ids is not None and list(gen[1:]) == list(out_ids))
    e2e = rep.sum(e2e)

    # ---- batched serving: every replica decodes its own 64 sequences (shared 2048-token prefix, paged f16 KV) ----
    try:
        serving = serving_leg(B, ctx, path, cfg, rank)
        serving["aggregate_tok_s"] = rep.sum(serving["decode_tok_s"])
        serving["replicas"] = world
    except B.BrasaError as e:
        serving = {"error": str(e)}
        rep.sum(0.0)

    # ---- Qwen3-32B architecture, tensor-parallel over all ranks of the job (one rank: the whole model on one GPU) ----
    tp32b = None
    if not args.skip_tp:
        try:
            tp32b = tp_leg(B, ctx, rep, steps=1)
            tp32b["parity"] = tp_parity(B, ctx, rep)
            if rank == 0:
                hbm, _ = measured_peaks()
                tp32b["frac_of_measured_hbm_per_gpu"] = tp32b["achieved_gbs_per_gpu"] / hbm
                tp32b["two_devices_one_process"] = two_device_check(B) if world > 1 else "one GPU in this job"
        except B.BrasaError as e:
            tp32b = {"error": str(e)}
    if rank != 0:
        return

    peak, peak_kind = measured_peaks()
    wbytes = synth.weight_bytes_per_token(cfg)
    kvb = synth.kv_bytes_per_position(cfg, "f16")
    mean_pos = PROMPT + 1 + (steps_tokens - 1) / 2.0  # keys seen by step s: PROMPT + 1 + s
    bytes_per_token = wbytes + kvb * mean_pos
    per_gpu_tok_s = value / world
    token_frac = per_gpu_tok_s * bytes_per_token / 1e9 / peak

    # ---- dominant kernel: the whole-token decode kernel, one launch per token (timed above with CUDA events) ----
    t_token = total_s / (args.steps * steps_tokens)
    ach = bytes_per_token / t_token / 1e9
    roof = {"bound": "hbm", "kernel": "decode_token_kernel<kv f16>: one launch = one token (36 layers, lm_head, argmax)",
            "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "peak_source": peak_kind, "us_per_launch": t_token * 1e6,
            "algorithmic_bytes_per_launch": bytes_per_token, "traffic": TOKEN_KERNEL_TRAFFIC_BYTES,
            "note": "weights 2 360 553 504 B + 147 456 B per cached position, mean position of the timed steps"}
    if launches != args.steps * steps_tokens:  # the kernel-per-operation path ran (BRASA_TOKEN_KERNEL=0 or unsupported shapes)
        roof = None
    gemv_roof = kernel_roofline(B, ctx, K, cfg, peak, peak_kind)
    if roof is None:
        roof = gemv_roof
    try:
        gemv_roof["cpu_baseline"] = gemv_cpu_baseline(cfg)
    except Exception as e:  # reported, never required
        gemv_roof["cpu_baseline"] = {"value": None, "sample": f"failed: {e}"}
    if "error" not in serving:
        try:
            serving["cpu_baseline"] = serving_cpu_baseline(B, ctx, K, path, cfg)
        except Exception as e:
            serving["cpu_baseline"] = {"value": None, "sample": f"failed: {e}"}

    # ---- CPU baseline: the oracle's port on the host cores, over the GPU's own prefill state ----
    cpu = None
    try:
        import oracle
        oracle.build()
        use_all_host_cores()
        model.forward(ids, 0, want_logits=False)
        kvd = cfg["num_key_value_heads"] * cfg["head_dim"]
        kv_rows = []
        for li in range(cfg["num_hidden_layers"]):
            k = model.read_kv(li, "k", 0, PROMPT).view(np.float16).astype(np.float32).reshape(PROMPT, kvd)
            v = model.read_kv(li, "v", 0, PROMPT).view(np.float16).astype(np.float32).reshape(PROMPT, kvd)
            kv_rows.append((k, v))
        ntok = 32
        feed = [first] + [int(t) for t in out_ids[:ntok - 1]]
        times, cpu_logits = cpu_decode_sample(path, kv_rows, feed, PROMPT, ntok)
        # teacher-forced with the GPU's greedy tokens (crates/models/tests/forward.rs:131-138): the logits of every step are
        # compared; a different top-1 counts as a tie when the CPU's two best logits are closer than the f16-cache bound
        worst, ties, flips, gap = 0.0, 0, 0, float("inf")
        model.forward(ids, 0, want_logits=False)
        for i, tok in enumerate(feed):
            lg, _ = model.forward([tok], PROMPT + i)
            scale = float(np.abs(cpu_logits[i]).max())
            worst = max(worst, float(np.abs(lg[0] - cpu_logits[i]).max() / scale))
            top2 = np.sort(cpu_logits[i])[-2:]
            gap = min(gap, float(top2[1] - top2[0]) / scale)
            if int(np.argmax(lg[0])) != int(np.argmax(cpu_logits[i])):
                if float(top2[1] - top2[0]) <= 1e-3 * scale:
                    ties += 1
                else:
                    flips += 1
        sec = statistics.median(times)
        cpu = {"value": 1.0 / sec, "unit": "tok/s", "cores": os.cpu_count() or 1, "kind": "port",
               "sample": f"{ntok} teacher-forced decode tokens at positions {PROMPT}..{PROMPT + ntok - 1} of this workload over the GPU's prefill KV cache, "
                         f"oracle C port with OpenMP on all host cores",
               "parity_max_rel_logit_err": worst, "parity_same_greedy_tokens": flips == 0 and ties == 0, "parity_top1_flips": flips,
               "parity_top1_ties": ties, "parity_min_top2_gap_rel": gap, "parity_tokens_compared": ntok}
    except Exception as e:  # the baseline is reported, never required for the GPU figure
        cpu = {"value": None, "unit": "tok/s", "cores": os.cpu_count() or 1, "kind": "port", "sample": f"failed: {e}"}

    # ---- prefill at 16k context (f16 cache: tensor-core attention; q8_0 cache: the f32 attention kernel) ----
    long_prefill = {}
    sess.free()
    for kv_name in ("f16", "q8_0"):
        try:
            long_prefill[kv_name] = prefill_16k(B, ctx, path, cfg, kv_name, cpu_steps=3 if kv_name == "q8_0" else 0)
        except B.BrasaError as e:
            long_prefill[kv_name] = {"error": str(e)}
    tc_peak = tensor_peak()
    for v in long_prefill.values():
        if "tflops" in v and tc_peak:
            v["frac_of_measured_bf16_peak"] = v["tflops"] / tc_peak

    line = {"metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": total_s / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 activations and accumulation, q4_0/q6_0 weights, f16 KV", "data": "synthetic",
            "config": workload_config(world), "tokens_per_step": steps_tokens,
            "clocks": clocks.summary(),
            "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": 4 * PROMPT + 4 * steps_tokens, "d2h_bytes_per_step": 4 * GENERATE,
                    "prefill_tok_s": statistics.median(prefill_vals), "same_tokens_as_device_resident": same_tokens},
            "gpu_launches": int(launches), "model_load": load_stats,
            "roofline": roof,
            "gemv_roofline": gemv_roof,
            "prefill_16k": long_prefill,
            "serving": serving,
            "tp32b": tp32b,
            "token_roofline": {"bytes_per_token": bytes_per_token, "achieved_gbs": per_gpu_tok_s * bytes_per_token / 1e9, "peak": peak,
                               "frac_of_measured": token_frac, "frac_of_8tbs": per_gpu_tok_s * bytes_per_token / 8e12,
                               "roofline_tok_s_at_8tbs": 8e12 / bytes_per_token},
            "cpu_baseline": cpu}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--decode-tokens", type=int, default=GENERATE - 1,
                    help="decode forwards per step (default: the workload's 255); smaller values are for profiler captures")
    ap.add_argument("--only-prefill", action="store_true",
                    help="run only one prefill forward of the workload's prompt (profiler captures)")
    ap.add_argument("--only-kernel", action="store_true",
                    help="run only the dominant kernel's own timing leg (profiler captures)")
    ap.add_argument("--only-attention", action="store_true", help="run only the prefill attention kernel at 16k context (profiling)")
    ap.add_argument("--only-tp", action="store_true", help="run only the tensor-parallel Qwen3-32B decode over the job's ranks")
    ap.add_argument("--only-serving", action="store_true", help="run only the batched serving leg (profiling)")
    ap.add_argument("--skip-tp", action="store_true", help="leave out the Qwen3-32B tensor-parallel leg (18.6 GB of weights over the job's ranks)")
    ap.add_argument("--serving-seqs", type=int, default=64)
    ap.add_argument("--serving-steps", type=int, default=512)
    ap.add_argument("--only-decode", action="store_true",
                    help="run only the device-resident decode loop (profiler captures): no end-to-end, kernel or CPU legs")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
    else:
        run_ours(args, rank, world, local_rank)
        if world > 1:
            import torch.distributed as dist
            if dist.is_initialized():
                dist.destroy_process_group()


if __name__ == "__main__":
    main()
