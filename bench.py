#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at the Llama-3.2-1B shape with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--shape 1b|3b|8b] [--layers L]
    python bench.py --scenario mixed|prefix [--shape ...] [--dtype bfloat16|float32]
                                        (continuous batching / shared prefixes through the scheduler, see run_scenario)
    python bench.py --scenario sizes [--shape ...]   (decode steps at a grid of batch sizes and contexts, see run_sizes)
    python bench.py --scenario nipadra               (the Nipadra design beside Llama at equal layer sizes, see run_nipadra)
    python bench.py --scenario gekupel               (the Gekupel design beside Llama at equal layer sizes, see run_gekupel)
    python bench.py --scenario pinorax               (the Pinorax design beside Gekupel and Llama at equal layer sizes, see run_pinorax)
    python bench.py --scenario fovezen               (the Fovezen design beside Nipadra and Llama at equal layer sizes, see run_fovezen)

Prints ONE JSON line. ``value`` is decoded tokens per second at batch 8 and context 8192, timed on
the device over exactly K decode steps (one step = one token for every request of the batch);
``e2e`` is the same through the Python entry point (``Engine.step``: token ids from the host in,
sampled ids back to the host, every step). ``prefill`` is one 2,048-token prompt in one step (its
``frac`` is of the cuBLAS burst figure, ``frac_of_sustained`` of the sustained one); ``roofline``
relates the decode step's bytes (every weight once plus the cache of the live requests) to the
measured copy bandwidth, and ``rooflines`` gives the same fraction for every decode point;
``points`` holds decode at batch 1 and 64, at context 128, the prefill in four portions, and
``short_requests_b*``: requests of 16 prompt + 64 generated tokens through ``Engine.generate``.

``--impl reference`` runs the unmodified reference: its own ``gi_serve_bench`` with its CUDA
backend, built with its CMake files into baseline/_ref/build when it is not there yet, on the same
random model folder, at 8 concurrent requests of 16 prompt + 64 generated tokens (the workload that
finishes; the line says ``same_config: false`` and names ``points.short_requests_b8`` as the figure
to compare with). When it cannot be built or gives no result, the line says ``unavailable`` and why.

This engine runs on one GPU: for --gpus > 1 it prints one line saying so and exits with 2.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# BASELINE.json configs[2]: the Llama-3.2-1B shape.
LLAMA_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu",
    "hidden_size": 2048, "intermediate_size": 8192, "num_hidden_layers": 16, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 64, "vocab_size": 128256, "max_position_embeddings": 131072,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
}
# The other two shapes the baseline names (not the default run): --shape 3b | 8b, usually with --layers.
LLAMA_3B = dict(LLAMA_1B, hidden_size=3072, num_hidden_layers=28, num_attention_heads=24, head_dim=128)
LLAMA_8B = dict(LLAMA_1B, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
                head_dim=128, tie_word_embeddings=False,
                rope_scaling=dict(LLAMA_1B["rope_scaling"], factor=8.0))
SHAPES = {"1b": ("Llama-3.2-1B", LLAMA_1B), "3b": ("Llama-3.2-3B", LLAMA_3B), "8b": ("Llama-3.1-8B", LLAMA_8B)}
CONTEXT = 8192
PAGE = 16
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            out = dict(FALLBACK_PEAKS)
            out.update({k: float(v) for k, v in p.items() if k in out and isinstance(v, (int, float))})
            out["source"] = "measured"
            return out
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def model_folder(config, seed=1):
    """The random-weights model folder (made once per box under the temporary directory)."""
    from geneinfer_b200.weights import write_random_model
    tag = (f"geneinfer_bench_{config['num_hidden_layers']}x{config['hidden_size']}x{config['intermediate_size']}_"
           f"{int(config['tie_word_embeddings'])}_{seed}_{os.getuid()}")
    path = os.path.join(tempfile.gettempdir(), tag)
    if not (os.path.isfile(os.path.join(path, "model.safetensors")) and os.path.isfile(os.path.join(path, "done"))):
        t0 = time.time()
        print(f"[bench] writing random bf16 weights to {path}", file=sys.stderr, flush=True)
        write_random_model(config, seed, path, "bfloat16", std=0.02, norm_mean=1.0, norm_std=0.02)
        open(os.path.join(path, "done"), "w").close()
        print(f"[bench] wrote them in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
    return path


def step_bytes(model, cfg, batch, context):
    """Bytes a decode step has to read: every weight it uses once, and the cache of the live requests."""
    elt = 2
    kv_per_token = 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * elt * cfg["num_hidden_layers"]
    return model.weight_bytes() + batch * context * kv_per_token


def prefill_flops(cfg, T):
    D, I, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    A = cfg["num_attention_heads"] * cfg["head_dim"]
    K = cfg["num_key_value_heads"] * cfg["head_dim"]
    gemm = 2 * T * (D * (A + 2 * K) + A * D + 2 * D * I + I * D) * L
    attention = 2 * T * T * cfg["head_dim"] * cfg["num_attention_heads"] * L      # causal: half of 2 products
    head = 2 * D * cfg["vocab_size"]
    return gemm + attention + head


def fill_cache(engine, keys, length):
    """Gives each request ``length`` cached positions of random keys and values (setup, untimed):
    decoding reads them exactly as it would read real ones."""
    for t in list(engine.group_pages) + [v for v in getattr(engine, "group_value_pages", []) if v is not None]:
        t.normal_(0.0, 1.0)
    for key in keys:
        rc = engine.open(key)
        engine.cache.reserve(rc, length)
        engine.cache.advance(rc, length)


def time_decode_device(engine, batch, context, steps, warmup, vocab):
    """K decode steps of the step function with greedy sampling on the device, timed with CUDA events."""
    import torch
    from geneinfer_b200.engine.step import StepEntry
    from geneinfer_b200.ops import kernels
    keys = [f"b{i}" for i in range(batch)]
    fill_cache(engine, keys, context - steps - warmup)
    ids = torch.zeros(batch, dtype=torch.int32, device=engine.device)
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, vocab, (steps + warmup, batch), generator=g).tolist()

    def one(i):
        logits = engine.step([StepEntry(k, [toks[i][j]], [0]) for j, k in enumerate(keys)])
        kernels.argmax(logits, ids)

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = kernels.launch_count()
    start.record()
    for i in range(warmup, warmup + steps):
        one(i)
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end)
    launches = kernels.launch_count() - launches0
    for k in keys:
        engine.close(k)
    return ms / steps, launches


def time_decode_e2e(llm, batch, context, steps, warmup, vocab):
    """The same decode steps through Engine.step(): host token ids in, sampled ids out, every step."""
    import torch
    from geneinfer_b200 import SamplingParams
    import numpy as np
    rng = np.random.default_rng(5)
    sched = llm.scheduler
    prefill = context - steps - warmup - 1
    for t in llm.steps.group_pages:
        t.normal_(0.0, 1.0)
    rids = []
    for i in range(batch):
        prompt = [int(t) for t in rng.integers(0, vocab, prefill + 1)]
        rids.append(llm.submit(prompt, 0, SamplingParams(0.0)))
    sched._admit()
    for job in sched.running:                     # setup, untimed: the prompt's cache is filled with random values
        llm.steps.cache.reserve(job.cache, prefill)
        llm.steps.cache.advance(job.cache, prefill)
        job.fed = prefill
    for _ in range(warmup):
        llm.step()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    start.record()
    for _ in range(steps):
        llm.step()
    end.record()
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - t0) * 1e3
    assert all(len(llm.result(r).generated_tokens) == warmup + steps for r in rids)
    h2d = llm.steps._desc_size * 4
    d2h = batch * 4
    for job in list(sched.running):
        sched._finish(job)
    return wall_ms / steps, h2d, d2h


def time_prefill(engine, tokens, warmup, vocab, portions=1):
    """One prompt of ``tokens`` ids in ``portions`` equal steps; the median of three, in ms."""
    import torch
    from geneinfer_b200.engine.step import StepEntry
    g = torch.Generator().manual_seed(7)
    times = []
    n = tokens // portions
    for i in range(warmup + 3):
        prompt = torch.randint(0, vocab, (tokens,), generator=g).tolist()
        engine.open("p")
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for c in range(portions):
            engine.step([StepEntry("p", prompt[c * n:(c + 1) * n], [n - 1] if c == portions - 1 else [])])
        end.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(start.elapsed_time(end))
        engine.close("p")
    return sorted(times)[len(times) // 2]


SHORT_PROMPT, SHORT_NEW = 16, 64      # the reference arm's workload (its serve bench's own defaults)


def time_short_requests(llm, batch, vocab, runs=3):
    """``batch`` requests of 16 random prompt ids and 64 greedy tokens each through ``Engine.generate``
    (host token ids in, generated ids out), all submitted together: generated tokens per second of
    wall time, prompts included; the median of ``runs`` after one warm-up run."""
    import numpy as np
    import torch
    rng = np.random.default_rng(7)
    prompts = [[int(t) for t in rng.integers(0, vocab, SHORT_PROMPT)] for _ in range(batch)]
    walls = []
    for run in range(-1, runs):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = llm.generate(prompts, max_new_tokens=SHORT_NEW, temperature=0.0)
        torch.cuda.synchronize()
        if run >= 0:
            walls.append(time.perf_counter() - t0)
        assert all(len(o) == SHORT_NEW for o in out)
    return round(batch * SHORT_NEW / sorted(walls)[len(walls) // 2], 1)


def run_ours(args):
    import torch
    from geneinfer_b200 import Engine
    shape_name, shape = SHAPES[args.shape]
    cfg = dict(shape)
    layers_full = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    pk = peaks()
    folder = model_folder(cfg)
    vocab = cfg["vocab_size"]
    batch = 8
    pages_per_request = CONTEXT // PAGE

    def make(b):
        return Engine(folder, dtype="bfloat16", max_seq_len=CONTEXT, page_size=PAGE, kv_pages=b * pages_per_request,
                      max_running=b, step_tokens=PREFILL_TOKENS, prefix_cache=False)

    llm = make(batch)
    model = llm.model
    clocks = ClockSampler()
    clocks.start()
    ms_step, launches = time_decode_device(llm.steps, batch, CONTEXT, args.steps, args.warmup, vocab)
    ms_e2e, h2d, d2h = time_decode_e2e(llm, batch, CONTEXT, args.steps, args.warmup, vocab)
    ms_prefill = time_prefill(llm.steps, PREFILL_TOKENS, max(1, args.warmup), vocab)
    ms_prefill_4 = time_prefill(llm.steps, PREFILL_TOKENS, 1, vocab, portions=4)
    ms_short, _ = time_decode_device(llm.steps, batch, 128, args.steps, args.warmup, vocab)
    short = {f"short_requests_b{batch}": time_short_requests(llm, batch, vocab)}
    clock_record = clocks.stop()          # sampled through the timed regions above, which follow one another under load
    flops = prefill_flops(cfg, PREFILL_TOKENS)

    def roofline(b, context, ms):
        achieved = step_bytes(model, cfg, b, context) / (ms * 1e-3) / 1e9
        return {"achieved": round(achieved, 1), "frac": round(achieved / pk["hbm_gbs"], 4)}

    rooflines = {"decode_b8": roofline(batch, CONTEXT, ms_step), "decode_b8_context128": roofline(batch, 128, ms_short)}
    del llm
    torch.cuda.empty_cache()

    points = {"decode_b8_context128": round(batch / (ms_short * 1e-3), 1),
              "prefill_2048_in_4_portions": round(PREFILL_TOKENS / (ms_prefill_4 * 1e-3), 1)}
    for b in (1, 64):
        e = make(b)
        ms_b, _ = time_decode_device(e.steps, b, CONTEXT, args.steps, args.warmup, vocab)
        points[f"decode_b{b}"] = round(b / (ms_b * 1e-3), 1)
        rooflines[f"decode_b{b}"] = roofline(b, CONTEXT, ms_b)
        short[f"short_requests_b{b}"] = time_short_requests(e, b, vocab)
        del e
        torch.cuda.empty_cache()
    points.update(short)

    value = batch / (ms_step * 1e-3)
    line = {
        "metric": f"decode tok/s at batch 8, context 8192 ({shape_name} shape, random bf16 weights)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights N(0,0.02), random token ids, random cache contents",
        "impl": "ours",
        "config": {
            "model": f"{shape_name} shape", "global_batch": batch, "seq_len": CONTEXT, "parallelism": "single GPU",
            "layers": cfg["num_hidden_layers"], "layers_of_named_config": layers_full, "hidden": cfg["hidden_size"],
            "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": vocab, "tied_head": cfg["tie_word_embeddings"], "page_size": PAGE,
            "rope": f"theta 500000, llama3 {cfg['rope_scaling']['factor']:g}/1/4/8192", "rms_norm_eps": cfg["rms_norm_eps"],
            "decode_weight_copy": True,
            "l2": "step inputs (weights + cache) are larger than L2", "peaks": pk["source"],
        },
        "e2e": {"value": round(batch / (ms_e2e * 1e-3), 1), "unit": "tok/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": round(ms_e2e, 4)},
        "gpu_launches": launches,
        "prefill": {"value": round(PREFILL_TOKENS / (ms_prefill * 1e-3), 1), "tokens": PREFILL_TOKENS,
                    "ms": round(ms_prefill, 3), "frac": round(flops / (ms_prefill * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                    "peak": pk["bf16_tflops"], "peak_kind": "cuBLAS bf16 burst, TFLOP/s",
                    "frac_of_sustained": round(flops / (ms_prefill * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)},
        "roofline": dict(rooflines["decode_b8"], bound="hbm", peak=pk["hbm_gbs"], unit="GB/s"),
        "rooflines": rooflines,
        "points": points,
        "short_requests": "points.short_requests_b*: generated tok/s of b requests of 16 prompt + 64 generated tokens through "
                          "Engine.generate, wall time with the prompts (the workload of the reference arm)",
        "clocks": clock_record,
    }
    print(json.dumps(line), flush=True)
    return 0


def run_sizes(args):
    """Decode steps of the step function at a grid of batch sizes and context lengths (device time per step with CUDA
    events, the same timing as the default run's), each with its fraction of the HBM roofline. Prints one JSON line."""
    import torch
    from geneinfer_b200 import Engine
    shape_name, shape = SHAPES[args.shape]
    cfg = dict(shape)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    pk = peaks()
    folder = model_folder(cfg)
    vocab = cfg["vocab_size"]
    contexts = (128, 2048, CONTEXT, 4 * CONTEXT)
    points = []
    for batch in (1, 4, 8, 16, 32, 64):
        longest = max(c for c in contexts if batch * c <= 64 * CONTEXT)             # at most 512 Ki cached positions
        llm = Engine(folder, dtype="bfloat16", max_seq_len=longest, page_size=PAGE, kv_pages=batch * ((longest + PAGE - 1) // PAGE),
                     max_running=batch, step_tokens=max(batch, 16), prefix_cache=False)
        for context in contexts:
            if context > longest:
                continue
            ms, _ = time_decode_device(llm.steps, batch, context, args.steps, args.warmup, vocab)
            achieved = step_bytes(llm.model, cfg, batch, context) / (ms * 1e-3) / 1e9
            points.append({"batch": batch, "context": context, "ms_per_step": round(ms, 4), "tok_s": round(batch / ms * 1e3, 1),
                           "gb_s": round(achieved, 1), "frac": round(achieved / pk["hbm_gbs"], 4)})
        llm.steps.check_status()
        del llm
        torch.cuda.empty_cache()
    print(json.dumps({"metric": f"decode steps at a grid of sizes ({shape_name} shape, random bf16 weights)", "impl": "ours", "n_gpus": 1,
                      "dtype": "bf16", "steps": args.steps, "warmup": args.warmup, "peak_gb_s": pk["hbm_gbs"],
                      "peaks": pk["source"], "points": points}))
    return 0


# ---------------------------------------------------------------------------------------------- Nipadra beside Llama
def nipadra_config(width, ff, layers, vocab, heads, head_dim, kv_heads, window):
    """A Nipadra model with the layer sizes of a Llama shape: every layer has the same feed-forward, three of four
    mixers are lightning attention (heads of 128), every fourth is the windowed attention beside the state-space mixer."""
    lh = width // 128
    decay = [1.0 - 2.0 ** (-5 - 3 * i / max(1, lh - 1)) for i in range(lh)]
    light = {"type": "lightning", "mixer": {"heads": lh, "dim": 128, "vdim": 128, "decay": decay}, "mlp": {"ff": ff, "kind": "dense"}}
    par = {"type": "parallel", "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "mask": {"size": window},
                 "rot": {"base": 500000.0, "dims": head_dim}, "scale": head_dim ** -0.5},
        "right": {"heads": width // 64, "vdim": 64, "state": 128, "groups": 1, "conv": 4, "norm_groups": 1},
        "left_scale": 0.5, "right_scale": 0.5}, "mlp": {"ff": ff, "kind": "dense"}}
    return {"architecture": "Nipadra", "width": width, "vocab": vocab, "norm": {"eps": 1e-6}, "postln_alpha": 2.0,
            "layers": [par if i % 4 == 2 else light for i in range(layers)]}


def time_calls(fn, iters=8, flush=None):
    """Median device time of ``fn()`` in ms (CUDA events), the L2 cache swept between calls."""
    import torch
    for _ in range(3):
        fn()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    return sorted(times)[len(times) // 2]


def nipadra_kernel_table(width, heads, kv_heads, head_dim, window, T, pk):
    """Each kernel of the new design alone, and the like kernel of the Llama path, at the sizes of one layer:
    a prompt portion of ``T`` tokens of one request and a decode step of 8 requests. ``frac`` is the time the
    kernel's algorithmic bytes (or, where larger, its multiply-adds on the tensor cores) need at the measured peaks,
    divided by the time it took."""
    import torch
    from geneinfer_b200.ops import kernels as K
    dev = torch.device("cuda:0")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []

    props = torch.cuda.get_device_properties(dev)
    # 32-bit multiply-adds a second on the CUDA cores (128 lanes an SM): the bound of what must stay 32-bit
    simt_ops = props.multi_processor_count * 128 * 1.965e9

    def add(name, like, fn, nbytes, flops=0.0, simt=0.0):
        ms = time_calls(fn, flush=flush)
        ideal = max(nbytes / (pk["hbm_gbs"] * 1e9), flops / (pk["bf16_tflops"] * 1e12)) * 1e3
        row = {"kernel": name, "like": like, "us": round(ms * 1e3, 1), "frac": round(ideal / ms, 3)}
        if simt:
            row["frac_of_32bit_issue"] = round(simt / simt_ops * 1e3 / ms, 3)
        rows.append(row)

    def seg(R, n):
        i32 = dict(dtype=torch.int32, device=dev)
        return (torch.arange(R, **i32) * n, torch.full((R,), n, **i32), torch.arange(R, **i32),
                torch.arange(R, **i32).repeat_interleave(n))

    D = width
    for what, R, n in (("prefill", 1, T), ("decode", 8, 1)):
        rows_n = R * n
        x = torch.randn(rows_n, D, device=dev)
        acc, xo = torch.empty_like(x), torch.empty_like(x)
        xn = torch.empty(rows_n, D, dtype=torch.bfloat16, device=dev)
        w = torch.ones(D, device=dev)
        add(f"residual_norm ({what})", "rmsnorm", lambda: K.residual_norm(x, w, xo, 1e-6, 2.0, acc_out=acc, xn_out=xn), rows_n * D * 14)
        add(f"rmsnorm, Llama ({what})", "", lambda: K.rmsnorm(x, w, xn, 1e-6), rows_n * D * 6)
        # lightning attention: heads of 128 x 128
        H = D // 128
        proj = torch.randn(rows_n, 4 * D, device=dev) * 0.5
        out = torch.empty(rows_n, D, device=dev)
        state = torch.zeros(R, H * 128 * 128, device=dev)
        s0, sl, slots, rr = seg(R, n)
        decay = torch.full((H,), 0.99, device=dev)
        scan_bytes = rows_n * D * 4 * 4 + 2 * R * H * 128 * 128 * 4
        parts = {}
        if rows_n > K.SCAN_PART:        # as the mixers do: long segments are cut into parts that run side by side
            parts = {"part_len": K.SCAN_PART, "ws_state": torch.empty(K.scan_parts(rows_n, R), D * 128, device=dev),
                     "ws_decay": torch.empty(rows_n, max(H, D // 64), device=dev)}
        add(f"linear_scan, constant decay ({what})", "attention", lambda: K.linear_scan(
            proj, 0, proj, D, proj, 2 * D, H, 1, 128, 128, True, state, 0, s0, sl, slots, out, decay=decay, **parts), scan_bytes,
            simt=rows_n * H * 128 * 128 * (4.0 if parts else 3.0))
        y = torch.empty(rows_n, D, dtype=torch.bfloat16, device=dev)
        add(f"gated_group_norm ({what})", "rmsnorm", lambda: K.gated_group_norm(out, proj, 3 * D, w, y, 1, 1e-6, False), rows_n * D * 10)
        # state space: heads of 64, state 128
        Hs, N = D // 64, 128
        C = D + 2 * N
        proj2 = torch.randn(rows_n, 2 * D + 2 * N + Hs, device=dev) * 0.5
        conv_w, conv_b = torch.randn(C, 4, device=dev) * 0.3, torch.zeros(C, device=dev)
        st2 = torch.zeros(R, Hs * N * 64 + 3 * C, device=dev)
        xbc = torch.empty(rows_n, C, device=dev)
        add(f"causal_conv ({what})", "rope_store", lambda: K.causal_conv(proj2, D, conv_w, conv_b, st2, Hs * N * 64, rr, s0, sl, slots, xbc),
            rows_n * C * 8)
        dtb, alog, skip = torch.zeros(Hs, device=dev), torch.zeros(Hs, device=dev), torch.ones(Hs, device=dev)
        add(f"linear_scan, step sizes ({what})", "attention", lambda: K.linear_scan(
            xbc, D + N, xbc, D, xbc, 0, Hs, Hs, N, 64, False, st2, 0, s0, sl, slots, out, dt=proj2, dt_offset=D + C, dt_bias=dtb,
            a_log=alog, skip=skip, **parts), rows_n * (D * 8 + 2 * N * 4) + 2 * R * Hs * N * 64 * 4,
            simt=rows_n * Hs * N * 64 * (4.0 if parts else 3.0))
        # windowed attention: norm + rotation + store, then attention over a context of T
        page = 16
        ctx_len = T
        n_pages = R * ((ctx_len + page - 1) // page)
        kc = torch.randn(n_pages, kv_heads, page, head_dim, device=dev).to(torch.bfloat16)
        vc = torch.randn(n_pages, kv_heads, page, head_dim, device=dev).to(torch.bfloat16)
        tables = torch.arange(n_pages, dtype=torch.int32, device=dev).view(R, -1)
        pos = (torch.arange(n, dtype=torch.int32, device=dev) + (ctx_len - n)).repeat(R)
        qkw = (heads + kv_heads) * head_dim
        proj3 = torch.randn(rows_n, qkw + heads, device=dev)
        q = torch.empty(rows_n, heads * head_dim, dtype=torch.bfloat16, device=dev)
        nw = torch.ones(head_dim, device=dev)
        freq = torch.rand(head_dim // 2, device=dev)
        add(f"norm_rope_store ({what})", "rope_store", lambda: K.norm_rope_store(
            proj3, 0, heads * head_dim, heads * head_dim, nw, nw, 1e-6, freq, True, pos, rr, tables, q, kc, vc, heads, kv_heads,
            head_dim, page), rows_n * (qkw * 4 + (heads + 2 * kv_heads) * head_dim * 2))
        qkv = torch.randn(rows_n, (heads + 2 * kv_heads) * head_dim, device=dev)
        cs = torch.rand(ctx_len, head_dim // 2, device=dev)
        add(f"rope_store, Llama ({what})", "", lambda: K.rope_store(qkv, pos, rr, tables, cs, cs, False, q, kc, vc, heads, kv_heads,
                                                                   head_dim, page), rows_n * (heads + 2 * kv_heads) * head_dim * 6)
        att = torch.empty_like(q)
        keys_seen = sum(min(window, p + 1) for p in range(ctx_len - n, ctx_len))
        att_flops = 4.0 * R * keys_seen * heads * head_dim
        att_bytes = R * min(ctx_len, window + n) * kv_heads * head_dim * 4 + rows_n * heads * head_dim * 4
        rows_dec = torch.arange(R, dtype=torch.int32, device=dev)
        per_tile = 128 // (heads // kv_heads)
        work = torch.tensor([(t, min(per_tile, n - t), 0) for t in range(0, n, per_tile)][::-1], dtype=torch.int32, device=dev)
        chunk = K.attention_chunk_keys()
        n_chunks = (ctx_len + chunk - 1) // chunk
        part_o = torch.empty(R, heads * n_chunks * head_dim, device=dev)
        part_ml = torch.empty(R, heads * n_chunks * 2, device=dev)

        def attend(win, **ep):
            if n == 1:
                K.attention_decode(q, kc, vc, att, rows_dec, rr, pos, tables, heads, kv_heads, head_dim, page, head_dim ** -0.5,
                                   win, part_o, part_ml, n_chunks, n_chunks, **ep)
            else:
                K.attention_prefill_tc(q, kc, vc, att, work, pos, tables, heads, kv_heads, head_dim, page, head_dim ** -0.5, win, **ep)

        add(f"window attention with sink and gate ({what})", "attention",
            lambda: attend(window, sink=True, gate=proj3, gate_offset=qkw), att_bytes, att_flops)
        full_flops = 4.0 * R * sum(p + 1 for p in range(ctx_len - n, ctx_len)) * heads * head_dim
        full_bytes = R * ctx_len * kv_heads * head_dim * 4 + rows_n * heads * head_dim * 4
        add(f"attention, Llama ({what})", "", lambda: attend(None), full_bytes, full_flops)
        gu = torch.randn(rows_n, 4 * D, device=dev)
        hmid = torch.empty(rows_n, 2 * D, dtype=torch.bfloat16, device=dev)
        add(f"gated_act relu ({what})", "swiglu", lambda: K.gated_act(gu, hmid, "relu"), rows_n * 2 * D * 10)
        add(f"swiglu, Llama ({what})", "", lambda: K.swiglu(gu, hmid), rows_n * 2 * D * 10)
    return rows


def run_nipadra(args):
    """Prefill (one 2,048-token prompt in one step) and decode (batch 8 at context 2,048) throughput of Nipadra models
    whose layers have the sizes of the Llama-3.2-1B and Llama-3.1-8B shapes (four layers each, random bf16 weights),
    beside Llama models of the same sizes; then every kernel of the new design alone beside the like kernel of the
    Llama path. Prints one JSON line."""
    import torch
    from geneinfer_b200 import Engine
    pk = peaks()
    layers = args.layers or 4
    context, batch, T = 2048, 8, PREFILL_TOKENS
    models = []
    for name, base in (("1b", LLAMA_1B), ("8b", LLAMA_8B)):
        llama = dict(base, num_hidden_layers=layers, tie_word_embeddings=True)
        nip = nipadra_config(base["hidden_size"], base["intermediate_size"], layers, base["vocab_size"],
                             base["num_attention_heads"], base["head_dim"], base["num_key_value_heads"], 1024)
        for arch, cfg in (("Llama", llama), ("Nipadra", nip)):
            if arch == "Llama":
                folder = model_folder(cfg)
            else:
                from geneinfer_b200.weights import write_random_model
                folder = os.path.join(tempfile.gettempdir(), f"geneinfer_bench_nipadra_{name}_{layers}_{os.getuid()}")
                if not os.path.isfile(os.path.join(folder, "done")):
                    write_random_model(cfg, 1, folder, "bfloat16", std=0.02)
                    open(os.path.join(folder, "done"), "w").close()
            llm = Engine(folder, dtype="bfloat16", max_seq_len=context, page_size=PAGE, kv_pages=batch * (context // PAGE),
                         max_running=batch, step_tokens=T, prefix_cache=False)
            vocab = base["vocab_size"]
            ms_prefill = time_prefill(llm.steps, T, 2, vocab)
            ms_decode, _ = time_decode_device(llm.steps, batch, context, args.steps, args.warmup, vocab)
            llm.steps.check_status()
            models.append({"model": f"{arch} at the {SHAPES[name][0]} layer sizes, {layers} layers",
                           "prefill_2048_tok_s": round(T / ms_prefill * 1e3, 1), "prefill_ms": round(ms_prefill, 3),
                           "decode_b8_ctx2048_tok_s": round(batch / ms_decode * 1e3, 1), "decode_ms_per_step": round(ms_decode, 4),
                           "weight_gb": round(llm.model.weight_bytes() / 1e9, 3)})
            del llm
            torch.cuda.empty_cache()
    table = nipadra_kernel_table(2048, 32, 8, 64, 1024, T, pk)
    print(json.dumps({"metric": "Nipadra beside Llama at equal layer sizes (random bf16 weights)", "impl": "ours", "n_gpus": 1,
                      "dtype": "bf16", "steps": args.steps, "warmup": args.warmup, "peaks": pk["source"],
                      "peak_gb_s": pk["hbm_gbs"], "peak_tflops": pk["bf16_tflops"], "models": models, "kernels": table}))
    return 0


# ---------------------------------------------------------------------------------------------- Gekupel beside Llama
def gekupel_config(width, ff, layers, vocab, heads, head_dim, kv_heads, span):
    """A Gekupel model with the layer sizes of a Llama shape: the attention layers have Llama's heads, the latent ones
    half as many heads with a rotated part of half a head and latents of 3/8 (queries) and 1/4 (keys, values; at most
    512) of the width; the mixture has 8 experts of half the dense width of which a token uses 2 (the dense layer's
    multiply-adds). Layers in turn: latent (scaled rotation, sink) with a dense feed-forward, attention with experts,
    latent with experts, attention with experts."""
    lh = max(heads // 2, 1)
    rot = {"base": 500000.0, "dims": head_dim // 2}
    lat = {"dim": head_dim, "heads": lh, "kv_rank": min(512, width // 4), "mask": {"size": span}, "q_rank": 3 * width // 8, "rot": rot,
           "rot_dim": head_dim // 2, "scale": (head_dim + head_dim // 2) ** -0.5, "vdim": head_dim}
    lat2 = dict(lat, rot=dict(rot, scaling={"factor": 4.0, "fast": 32.0, "original": 8192, "slow": 1.0}))
    att = {"dim": head_dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": span}, "scale": head_dim ** -0.5, "vdim": head_dim}
    moe = {"expert": {"ff": ff // 2}, "kind": "moe", "router": {"experts": 8, "top": 2}}
    kinds = [{"mixer": lat2, "mlp": {"ff": ff, "kind": "dense"}, "type": "latent_attention_2"},
             {"mixer": att, "mlp": moe, "type": "attention"},
             {"mixer": lat, "mlp": moe, "type": "latent_attention"},
             {"mixer": att, "mlp": moe, "type": "attention"}]
    return {"architecture": "Gekupel", "embedding": {"scale": 1.0}, "layers": [kinds[i % 4] for i in range(layers)],
            "norm": {"eps": 1e-6}, "vocab": vocab, "width": width}


def gekupel_kernel_table(width, heads, kv_heads, head_dim, span, ff, T, pk):
    """Each kernel of the new design alone, and the like kernel of the Llama path, at the sizes of one layer: a prompt
    portion of ``T`` tokens of one request and a decode step of 8 requests at a context of ``T``. ``frac`` is the time
    the kernel's algorithmic bytes (or, where larger, its multiply-adds at the tensor cores' measured rate) need,
    divided by the time it took; ``frac_of_32bit_issue`` the same against the CUDA cores' 32-bit rate, for kernels
    whose arithmetic has to stay 32-bit."""
    import torch
    from geneinfer_b200.ops import kernels as K
    dev = torch.device("cuda:0")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []
    props = torch.cuda.get_device_properties(dev)
    simt_ops = props.multi_processor_count * 128 * 1.965e9
    bf = torch.bfloat16

    def add(name, like, fn, nbytes, flops=0.0, simt=0.0):
        ms = time_calls(fn, flush=flush)
        ideal = max(nbytes / (pk["hbm_gbs"] * 1e9), flops / (pk["bf16_tflops"] * 1e12)) * 1e3
        row = {"kernel": name, "like": like, "us": round(ms * 1e3, 1), "frac": round(ideal / ms, 3)}
        if simt:
            row["frac_of_32bit_issue"] = round(simt / simt_ops * 1e3 / ms, 3)
        rows.append(row)

    D, page = width, 16
    lh, rot, kr, qr = max(heads // 2, 1), head_dim // 2, min(512, width // 4), 3 * width // 8
    E, top, I = 8, 2, ff // 2
    for what, R, n in (("prefill", 1, T), ("decode", 8, 1)):
        N = R * n
        i32 = dict(dtype=torch.int32, device=dev)
        rr = torch.arange(R, **i32).repeat_interleave(n)
        n_pages = R * ((T + page - 1) // page)
        tables = torch.arange(n_pages, **i32).view(R, -1)
        pos = (torch.arange(n, **i32) + (T - n)).repeat(R)
        x, y = torch.randn(N, D, device=dev), torch.randn(N, D, device=dev)
        xn = torch.empty(N, D, dtype=bf, device=dev)
        w = torch.ones(D, device=dev)
        add(f"add_normed ({what})", "rmsnorm", lambda: K.add_normed(y, w, x, 1e-6, xn_out=xn, clear_y=True), N * D * 18)
        add(f"rmsnorm, Llama ({what})", "", lambda: K.rmsnorm(x, w, xn, 1e-6), N * D * 6)
        # latent attention: store, queries through the heads' key matrices, attention over the latent rows, values
        down = torch.randn(N, qr + kr + rot, device=dev)
        cq = torch.empty(N, qr, dtype=bf, device=dev)
        cache = torch.randn(n_pages, 1, page, kr + rot, device=dev).to(bf)
        freq = torch.rand(rot // 2, device=dev)
        wq, wc = torch.ones(qr, device=dev), torch.ones(kr, device=dev)
        add(f"latent_store ({what})", "rope_store", lambda: K.latent_store(down, 0, wq, cq, qr, wc, qr + kr, freq, 1.1, 1e-6, pos, rr,
                                                                          tables, cache, page), N * ((qr + kr + rot) * 6))
        q = torch.randn(N, lh * (head_dim + rot), device=dev)
        wuk = (torch.randn(lh, kr, head_dim, device=dev) * 0.05).to(bf)
        qa = torch.empty(N, lh * (kr + rot), device=dev)
        add(f"head_product, queries ({what})", "product", lambda: K.head_product(q, 0, head_dim + rot, wuk, qa, 0, kr + rot, tail=rot,
                                                                                 freq=freq, amplitude=1.1, positions=pos),
            lh * kr * head_dim * 2 + N * lh * (head_dim + kr + 2 * rot) * 4, flops=2.0 * N * lh * kr * head_dim,
            simt=N * lh * kr * head_dim)
        ol = torch.empty(N, lh * kr, device=dev)
        seen = sum(min(span, p + 1) for p in range(T - n, T))
        lat_bytes = R * min(T, span + n) * (kr + rot) * 2 + N * lh * (2 * kr + rot) * 4
        def listed(Hq, Hk, hd_, vd_, alias):
            """The rows as the mixers hand them over: tiles of a prompt portion, or single tokens; few tiles in ranges of keys."""
            pt = K.attention_rows_tile_tokens(Hq, Hk, hd_, vd_, alias)
            if n == 1:
                kw = {"rows": torch.arange(R, **i32)}
                count = R
            else:
                kw = {"tiles": torch.tensor([(t, min(pt, n - t), 0) for t in range(0, n, pt)][::-1], **i32)}
                count = kw["tiles"].shape[0]
            sp = K.attention_rows_splits(count, Hq, Hk, span)
            if sp > 1:
                kw.update(splits=sp, workspace=torch.empty(K.attention_rows_workspace_rows(count, Hq, Hk, sp), vd_ + 2, device=dev))
            return kw

        lat_kw = listed(lh, 1, kr + rot, kr, True)
        add(f"attention_rows over the latent, window {span} ({what})", "attention",
            lambda: K.attention_rows(qa, cache, None, ol, rr, pos, tables, lh, 1, kr + rot, kr, page, 0.1, window=span, **lat_kw),
            lat_bytes, flops=2.0 * R * seen * lh * (2 * kr + rot))
        wuv = (torch.randn(lh, head_dim, kr, device=dev) * 0.05).to(bf)
        att = torch.empty(N, lh * head_dim, dtype=bf, device=dev)
        add(f"head_product, values ({what})", "product", lambda: K.head_product(ol, 0, kr, wuv, att, 0, head_dim),
            lh * kr * head_dim * 2 + N * lh * (kr * 4 + head_dim * 2), flops=2.0 * N * lh * kr * head_dim, simt=N * lh * kr * head_dim)
        # attention in blocks with a distance bias and sinks, beside Llama's attention over the same context
        kc = torch.randn(n_pages, kv_heads, page, head_dim, device=dev).to(bf)
        vc = torch.randn(n_pages, kv_heads, page, head_dim, device=dev).to(bf)
        q2 = torch.randn(N, heads * head_dim, device=dev).to(bf)
        o2 = torch.empty_like(q2)
        slopes, sinks = torch.rand(heads, device=dev) * 0.1, torch.randn(heads, device=dev)
        seen_c = sum(p % span + 1 for p in range(T - n, T))
        att_kw = listed(heads, kv_heads, head_dim, head_dim, False)
        add(f"attention_rows in blocks of {span} with bias and sinks ({what})", "attention",
            lambda: K.attention_rows(q2, kc, vc, o2, rr, pos, tables, heads, kv_heads, head_dim, head_dim, page, head_dim ** -0.5,
                                     chunk=span, slopes=slopes, sinks=sinks, **att_kw),
            R * min(T, span) * kv_heads * head_dim * 4 + N * heads * head_dim * 4, flops=4.0 * R * seen_c * heads * head_dim)
        rows_dec = torch.arange(R, **i32)
        per_tile = 128 // (heads // kv_heads)
        work = torch.tensor([(t, min(per_tile, n - t), 0) for t in range(0, n, per_tile)][::-1], **i32)
        chunk = K.attention_chunk_keys()
        n_chunks = (T + chunk - 1) // chunk
        part_o = torch.empty(R, heads * n_chunks * head_dim, device=dev)
        part_ml = torch.empty(R, heads * n_chunks * 2, device=dev)

        def llama_attention():
            if n == 1:
                K.attention_decode(q2, kc, vc, o2, rows_dec, rr, pos, tables, heads, kv_heads, head_dim, page, head_dim ** -0.5,
                                   span, part_o, part_ml, n_chunks, n_chunks)
            else:
                K.attention_prefill_tc(q2, kc, vc, o2, work, pos, tables, heads, kv_heads, head_dim, page, head_dim ** -0.5, span)

        seen_w = sum(min(span, p + 1) for p in range(T - n, T))
        add(f"attention, Llama kernels, window {span} ({what})", "", llama_attention,
            R * min(T, span + n) * kv_heads * head_dim * 4 + N * heads * head_dim * 4, flops=4.0 * R * seen_w * heads * head_dim)
        # routed experts beside the dense products of the same multiply-adds
        router, corr = torch.randn(E, D, device=dev) * 0.1, torch.zeros(E, device=dev)
        wgu = (torch.randn(E, 2 * I, D, device=dev) * 0.02).to(bf)
        wd = (torch.randn(E, D, I, device=dev) * 0.02).to(bf)
        xb = torch.randn(N, D, device=dev).to(bf)
        ids, wts = torch.empty(N, top, **i32), torch.empty(N, top, device=dev)
        cnt = torch.empty(1, **i32)
        tc = N * top >= 256
        tm = K.TC_TILE_ROWS if tc else K.grouped_tile_rows()
        tiles = K.route_tiles(N, top, E, tm)
        srt, grp, prow = torch.empty(tiles * tm, **i32), torch.empty(tiles, **i32), torch.empty(N * top, **i32)
        add(f"route + bucket ({what})", "", lambda: K.route(xb, router, corr, top, ids, wts, srt, grp, cnt, tile_rows=tm, pair_row=prow),
            N * D * 2 + E * D * 4)
        used = int(cnt.item())
        experts_hit = len(set(ids.view(-1).tolist()))
        if tc:
            rows_x = torch.empty(tiles * tm, D, dtype=bf, device=dev)
            hid = torch.empty(tiles * tm, I, dtype=bf, device=dev)
            part = torch.empty(tiles * tm, D, device=dev)
            add(f"gather_rows ({what})", "", lambda: K.gather_rows(xb, top, srt, cnt, tm, rows_x), used * tm * D * 4)
            add(f"experts [gate; up] on the tensor cores, {used} tiles ({what})", "product",
                lambda: K.expert_product_tc(rows_x, wgu, hid, grp, cnt, gated="silu"),
                experts_hit * 2 * I * D * 2 + used * tm * (D + I) * 2, flops=2.0 * N * top * 2 * I * D)
            add(f"experts down on the tensor cores ({what})", "product", lambda: K.expert_product_tc(hid, wd, part, grp, cnt),
                experts_hit * I * D * 2 + used * tm * (I * 2 + D * 4), flops=2.0 * N * top * I * D)
            yy = torch.zeros(N, D, device=dev)
            add(f"route_combine ({what})", "", lambda: K.route_combine(part, wts, yy, pair_row=prow), N * D * (8 + 4 * top))
        else:
            hid = torch.empty(N * top, I, device=dev)
            part = torch.empty(N * top, D, device=dev)
            add(f"experts [gate; up], tiles of 16 rows, {experts_hit} experts hit ({what})", "product",
                lambda: K.expert_product(xb, top, wgu, hid, srt, grp, cnt, gated="silu"), experts_hit * 2 * I * D * 2,
                simt=used * 16 * 2 * I * D)
            add(f"experts down, tiles of 16 rows ({what})", "product", lambda: K.expert_product(hid, 1, wd, part, srt, grp, cnt),
                experts_hit * I * D * 2, simt=used * 16 * I * D)
        # the dense products of a Llama layer with as many multiply-adds per token (2 experts of ff / 2 = one dense ff)
        wg = (torch.randn(2 * ff, D, device=dev) * 0.02).to(bf)
        wdn = (torch.randn(D, ff, device=dev) * 0.02).to(bf)
        gu = torch.empty(N, 2 * ff, device=dev)
        hd_ = torch.empty(N, ff, dtype=bf, device=dev)
        out = torch.zeros(N, D, device=dev)
        if K.gemm_swiglu_supported(N, ff, D):
            add(f"[gate; up] product with activation, Llama ({what})", "", lambda: K.gemm_swiglu(xb, wg, hd_), 2 * ff * D * 2 + N * (D + ff) * 2,
                flops=2.0 * N * 2 * ff * D)
        else:
            wgt = K.tile_weight(wg)
            add(f"[gate; up] product, Llama ({what})", "", lambda: K.gemm_tc(xb, wg, gu, w_tiles=wgt), 2 * ff * D * 2, flops=2.0 * N * 2 * ff * D)
        wdt = K.tile_weight(wdn)
        add(f"down product, Llama ({what})", "", lambda: K.gemm_tc(hd_, wdn, out, True, w_tiles=wdt), ff * D * 2 + N * (ff * 2 + D * 8),
            flops=2.0 * N * ff * D)
        del wg, wdn, wgu, wd
    return rows


def run_gekupel(args):
    """Prefill (one 2,048-token prompt in one step) and decode (batch 8 at context 2,048) throughput of Gekupel models
    whose layers have the sizes of the Llama-3.2-1B and Llama-3.1-8B shapes (four layers each, random bf16 weights),
    beside Llama models of the same sizes; then every kernel of the new design alone beside the like kernel of the
    Llama path. Prints one JSON line."""
    import torch
    from geneinfer_b200 import Engine
    from geneinfer_b200.weights import write_random_model
    pk = peaks()
    layers = args.layers or 4
    context, batch, T = 2048, 8, PREFILL_TOKENS
    models = []
    for name, base in (("1b", LLAMA_1B), ("8b", LLAMA_8B)):
        llama = dict(base, num_hidden_layers=layers, tie_word_embeddings=True)
        gek = gekupel_config(base["hidden_size"], base["intermediate_size"], layers, base["vocab_size"], base["num_attention_heads"],
                             base["head_dim"], base["num_key_value_heads"], 1024)
        for arch, cfg in (("Llama", llama), ("Gekupel", gek)):
            if arch == "Llama":
                folder = model_folder(cfg)
            else:
                folder = os.path.join(tempfile.gettempdir(), f"geneinfer_bench_gekupel_{name}_{layers}_{os.getuid()}")
                if not os.path.isfile(os.path.join(folder, "done")):
                    write_random_model(cfg, 1, folder, "bfloat16", std=0.02)
                    open(os.path.join(folder, "done"), "w").close()
            llm = Engine(folder, dtype="bfloat16", max_seq_len=context, page_size=PAGE, kv_pages=batch * (context // PAGE),
                         max_running=batch, step_tokens=T, prefix_cache=False)
            vocab = base["vocab_size"]
            ms_prefill = time_prefill(llm.steps, T, 2, vocab)
            ms_decode, _ = time_decode_device(llm.steps, batch, context, args.steps, args.warmup, vocab)
            llm.steps.check_status()
            models.append({"model": f"{arch} at the {SHAPES[name][0]} layer sizes, {layers} layers",
                           "prefill_2048_tok_s": round(T / ms_prefill * 1e3, 1), "prefill_ms": round(ms_prefill, 3),
                           "decode_b8_ctx2048_tok_s": round(batch / ms_decode * 1e3, 1), "decode_ms_per_step": round(ms_decode, 4),
                           "weight_gb": round(llm.model.weight_bytes() / 1e9, 3)})
            del llm
            torch.cuda.empty_cache()
    table = gekupel_kernel_table(2048, 32, 8, 64, 1024, 8192, T, pk)
    print(json.dumps({"metric": "Gekupel beside Llama at equal layer sizes (random bf16 weights)", "impl": "ours", "n_gpus": 1,
                      "dtype": "bf16", "steps": args.steps, "warmup": args.warmup, "peaks": pk["source"],
                      "peak_gb_s": pk["hbm_gbs"], "peak_tflops": pk["bf16_tflops"], "models": models, "kernels": table}))
    return 0


# ---------------------------------------------------------------------------------------------- Pinorax beside Gekupel
def pinorax_config(width, ff, layers, vocab, heads, head_dim, positions):
    """A Pinorax model with the layer sizes of a Llama shape, made like the latent layers of ``gekupel_config``: half of
    Llama's heads, a latent of 1/4 of the width (at most 512). The first layer has a dense feed-forward, the others a
    mixture of 8 experts of 3/8 of the dense width of which a token uses 2, with a shared expert of 1/4 of it (together
    the dense layer's multiply-adds per token)."""
    mixer = {"dim": head_dim, "heads": max(heads // 2, 1), "kv_rank": min(512, width // 4), "scale": head_dim ** -0.5, "vdim": head_dim}
    moe = {"expert": {"ff": 3 * ff // 8, "limit": 7.0}, "kind": "moe", "router": {"experts": 8, "top": 2},
           "shared": {"ff": ff // 4, "limit": 7.0}}
    kinds = [{"mixer": mixer, "mlp": {"ff": ff, "kind": "dense"}, "type": "latent_attention"}] + \
        [{"mixer": mixer, "mlp": moe, "type": "latent_attention"}] * 3
    return {"architecture": "Pinorax", "layers": [kinds[i % 4] for i in range(layers)], "logit_softcap": 30.0,
            "max_positions": positions, "norm": {"eps": 1e-6}, "residual_mult": 0.5, "vocab": vocab, "width": width}


def pinorax_kernel_table(width, heads, head_dim, ff, vocab, layers, T, pk):
    """Each kernel that the Pinorax design added or changed, alone, beside the like kernel of the Gekupel path (the
    closest existing design), at the sizes of one layer: a prompt portion of ``T`` tokens of one request and a decode
    step of 8 requests at a context of ``T``. ``frac`` is the time the kernel's algorithmic bytes (or, where larger, its
    multiply-adds at the tensor cores' measured rate) need, divided by the time it took; ``frac_of_32bit_issue`` the
    same against the CUDA cores' 32-bit rate, for kernels whose arithmetic has to stay 32-bit."""
    import torch
    from geneinfer_b200.ops import kernels as K
    dev = torch.device("cuda:0")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []
    props = torch.cuda.get_device_properties(dev)
    simt_ops = props.multi_processor_count * 128 * 1.965e9
    bf = torch.bfloat16

    def add(name, like, fn, nbytes, flops=0.0, simt=0.0):
        ms = time_calls(fn, flush=flush)
        ideal = max(nbytes / (pk["hbm_gbs"] * 1e9), flops / (pk["bf16_tflops"] * 1e12)) * 1e3
        row = {"kernel": name, "like": like, "us": round(ms * 1e3, 1), "frac": round(ideal / ms, 3)}
        if simt:
            row["frac_of_32bit_issue"] = round(simt / simt_ops * 1e3 / ms, 3)
        rows.append(row)

    D, page = width, 16
    lh, kr = max(heads // 2, 1), min(512, width // 4)
    E, top, I, Is = 8, 2, 3 * ff // 8, ff // 4
    slots, slot = layers + 1, max(layers // 2, 1)
    for what, R, n in (("prefill", 1, T), ("decode", 8, 1)):
        N = R * n
        i32 = dict(dtype=torch.int32, device=dev)
        rr = torch.arange(R, **i32).repeat_interleave(n)
        n_pages = R * ((T + page - 1) // page)
        tables = torch.arange(n_pages, **i32).view(R, -1)
        pos = (torch.arange(n, **i32) + (T - n)).repeat(R)
        x, y = torch.randn(N, D, device=dev), torch.randn(N, D, device=dev)
        xn = torch.empty(N, D, dtype=bf, device=dev)
        w, one = torch.ones(D, device=dev), torch.ones(1, device=dev)
        hist = torch.randn(N, slots, D, device=dev)
        dw, bias = torch.rand(slot + 1, device=dev), torch.randn(D, device=dev)
        add(f"depth_mix, {slot + 1} terms, bias, next norm ({what})", "add_normed",
            lambda: K.depth_mix(x, y, 0.5, hist, slot, dw, next_weight=one, eps=1e-6, xn_out=xn, y_bias=bias), N * D * (4 * slot + 22))
        add(f"add_normed, Gekupel ({what})", "", lambda: K.add_normed(y, w, x, 1e-6, xn_out=xn, clear_y=True), N * D * 18)
        ptab = torch.randn(T, D, device=dev).to(bf)
        add(f"add_rows_at, learned positions ({what})", "embed", lambda: K.add_rows_at(x, ptab, pos), N * D * 10)
        etab = torch.randn(vocab, D, device=dev).to(bf)
        toks = torch.randint(0, vocab, (N,), **i32)
        add(f"embed, Gekupel ({what})", "", lambda: K.embed(etab, toks, x), N * D * 6)
        # latent attention: store, queries through the heads' key matrices, attention over all latent rows, values and gate
        cols = lh * head_dim + kr + lh * head_dim
        down = torch.randn(N, cols, device=dev)
        cache = torch.randn(n_pages, 1, page, kr, device=dev).to(bf)
        wc = torch.ones(kr, device=dev)
        add(f"latent_store, no query latent ({what})", "latent_store",
            lambda: K.latent_store(down, 0, None, None, lh * head_dim, wc, lh * head_dim + kr, None, 1.0, 1e-6, pos, rr, tables, cache, page),
            N * kr * 6)
        wuk = (torch.randn(lh, kr, head_dim, device=dev) * 0.05).to(bf)
        qa = torch.empty(N, lh * kr, device=dev)
        add(f"head_product, queries from the first product ({what})", "head_product",
            lambda: K.head_product(down, 0, head_dim, wuk, qa, 0, kr), lh * kr * head_dim * 2 + N * lh * (head_dim + kr) * 4,
            flops=2.0 * N * lh * kr * head_dim, simt=N * lh * kr * head_dim)
        ol = torch.empty(N, lh * kr, device=dev)
        sinks = torch.randn(lh, device=dev)
        pt = K.attention_rows_tile_tokens(lh, 1, kr, kr, True)

        def listed(span):
            if n == 1:
                kw = {"rows": torch.arange(R, **i32)}
                count = R
            else:
                kw = {"tiles": torch.tensor([(t, min(pt, n - t), 0) for t in range(0, n, pt)][::-1], **i32)}
                count = kw["tiles"].shape[0]
            sp = K.attention_rows_splits(count, lh, 1, span)
            if sp > 1:
                kw.update(splits=sp, workspace=torch.empty(K.attention_rows_workspace_rows(count, lh, 1, sp), kr + 2, device=dev))
            return kw

        for name, like, window in ((f"attention_rows over the latent, all {T} positions, sink ({what})", "attention_rows", None),
                                   (f"attention_rows over the latent, window {T // 2}, Gekupel ({what})", "", T // 2)):
            kw = listed(window or T)
            seen = sum(min(window or T, p + 1) for p in range(T - n, T))
            add(name, like, lambda: K.attention_rows(qa, cache, None, ol, rr, pos, tables, lh, 1, kr, kr, page, 0.1, window=window,
                                                     sinks=sinks, **kw),
                R * min(T, (window or T) + n) * kr * 2 + N * lh * 2 * kr * 4, flops=2.0 * R * seen * lh * 2 * kr)
        wuv = (torch.randn(lh, head_dim, kr, device=dev) * 0.05).to(bf)
        att = torch.empty(N, lh * head_dim, dtype=bf, device=dev)
        for name, like, gate in ((f"head_product, values with the output gate ({what})", "head_product", down),
                                 (f"head_product, values, Gekupel ({what})", "", None)):
            add(name, like, lambda: K.head_product(ol, 0, kr, wuv, att, 0, head_dim, gate=gate, gate_offset=lh * head_dim + kr),
                lh * kr * head_dim * 2 + N * lh * (kr * 4 + head_dim * (6 if gate is not None else 2)), flops=2.0 * N * lh * kr * head_dim,
                simt=N * lh * kr * head_dim)
        # experts chosen by a table beside experts chosen by scores; the capped activation beside SiLU
        router, corr = torch.randn(E, D, device=dev) * 0.1, torch.zeros(E, device=dev)
        table = torch.rand(vocab, E, device=dev).argsort(1)[:, :top].to(torch.int32).contiguous()
        wgu = (torch.randn(E, 2 * I, D, device=dev) * 0.02).to(bf)
        wd = (torch.randn(E, D, I, device=dev) * 0.02).to(bf)
        xb = torch.randn(N, D, device=dev).to(bf)
        ids, wts = torch.empty(N, top, **i32), torch.empty(N, top, device=dev)
        cnt = torch.empty(1, **i32)
        tc = N * top >= 256
        tm = K.TC_TILE_ROWS if tc else K.grouped_tile_rows()
        tiles = K.route_tiles(N, top, E, tm)
        srt, grp, prow = torch.empty(tiles * tm, **i32), torch.empty(tiles, **i32), torch.empty(N * top, **i32)
        add(f"route + bucket, Gekupel ({what})", "", lambda: K.route(xb, router, corr, top, ids, wts, srt, grp, cnt, tile_rows=tm, pair_row=prow),
            N * D * 2 + E * D * 4)
        add(f"route_table + bucket ({what})", "route", lambda: K.route_table(toks, None, table, E, ids, wts, srt, grp, cnt, tile_rows=tm, pair_row=prow),
            N * (4 + 12 * top))
        used = int(cnt.item())
        hit = len(set(ids.view(-1).tolist()))
        for act, like, limit in (("capped_swish", "experts", 7.0), ("silu", "", 0.0)):
            who = "" if like else ", Gekupel"
            if tc:
                rows_x = torch.randn(tiles * tm, D, device=dev).to(bf)
                hid = torch.empty(tiles * tm, I, dtype=bf, device=dev)
                add(f"experts [gate; up] on the tensor cores, {act}{who} ({what})", like,
                    lambda: K.expert_product_tc(rows_x, wgu, hid, grp, cnt, gated=act, limit=limit),
                    hit * 2 * I * D * 2 + used * tm * (D + I) * 2, flops=2.0 * N * top * 2 * I * D)
            else:
                hid = torch.empty(N * top, I, device=dev)
                add(f"experts [gate; up], tiles of 16 rows, {act}{who} ({what})", like,
                    lambda: K.expert_product(xb, top, wgu, hid, srt, grp, cnt, gated=act, limit=limit), hit * 2 * I * D * 2,
                    simt=used * 16 * 2 * I * D)
        # the dense feed-forward with biases (and the shared expert's capped activation) beside the plain one
        wg = (torch.randn(2 * ff, D, device=dev) * 0.02).to(bf)
        b2 = torch.randn(2 * ff, device=dev)
        hd_ = torch.empty(N, ff, dtype=bf, device=dev)
        if K.gemm_swiglu_supported(N, ff, D):
            for name, like, kw in ((f"[gate; up] product with biases and SiLU ({what})", "gemm_swiglu", dict(bias=b2)),
                                   (f"[gate; up] product with the capped activation ({what})", "gemm_swiglu", dict(activation="capped_swish", limit=7.0)),
                                   (f"[gate; up] product with SiLU, Gekupel ({what})", "", {})):
                add(name, like, lambda: K.gemm_swiglu(xb, wg, hd_, **kw), 2 * ff * D * 2 + N * (D + ff) * 2, flops=2.0 * N * 2 * ff * D)
        else:
            gu = torch.randn(N, 2 * ff, device=dev)
            add(f"gated_act with biases ({what})", "swiglu", lambda: K.gated_act(gu, hd_, "silu", 0.0, b2), N * ff * 10 + ff * 8)
            add(f"gated_act, capped ({what})", "swiglu", lambda: K.gated_act(gu, hd_, "capped_swish", 7.0), N * ff * 10)
            add(f"swiglu, Gekupel ({what})", "", lambda: K.swiglu(gu, hd_), N * ff * 10)
        logits = torch.randn(R, vocab, device=dev)
        add(f"softcap of {R} rows of logits ({what})", "", lambda: K.softcap(logits, 30.0), R * vocab * 8)
        del wg, wgu, wd
    return rows


def run_pinorax(args):
    """Prefill (one 2,048-token prompt in one step) and decode (batch 8 at context 2,048) throughput of Pinorax models
    whose layers have the sizes of the Llama-3.2-1B and Llama-3.1-8B shapes (four layers each, random bf16 weights),
    beside Gekupel models (the closest existing design: latent attention and routed experts; their windows and blocks
    set to the whole context, so that both see as many keys) and Llama models of the same sizes; then every kernel
    that the design added or changed alone beside the like kernel of the Gekupel path. Prints one JSON line."""
    import torch
    from geneinfer_b200 import Engine
    from geneinfer_b200.weights import write_random_model
    pk = peaks()
    layers = args.layers or 4
    context, batch, T = 2048, 8, PREFILL_TOKENS
    models = []
    for name, base in (("1b", LLAMA_1B), ("8b", LLAMA_8B)):
        llama = dict(base, num_hidden_layers=layers, tie_word_embeddings=True)
        gek = gekupel_config(base["hidden_size"], base["intermediate_size"], layers, base["vocab_size"], base["num_attention_heads"],
                             base["head_dim"], base["num_key_value_heads"], context)
        pin = pinorax_config(base["hidden_size"], base["intermediate_size"], layers, base["vocab_size"], base["num_attention_heads"],
                             base["head_dim"], context)
        for arch, cfg in (("Llama", llama), ("Gekupel", gek), ("Pinorax", pin)):
            if arch == "Llama":
                folder = model_folder(cfg)
            else:
                folder = os.path.join(tempfile.gettempdir(), f"geneinfer_bench_{arch.lower()}_{name}_{layers}_{context}_{os.getuid()}")
                if not os.path.isfile(os.path.join(folder, "done")):
                    write_random_model(cfg, 1, folder, "bfloat16", std=0.02)
                    open(os.path.join(folder, "done"), "w").close()
            llm = Engine(folder, dtype="bfloat16", max_seq_len=context, page_size=PAGE, kv_pages=batch * (context // PAGE),
                         max_running=batch, step_tokens=T, prefix_cache=False)
            vocab = base["vocab_size"]
            ms_prefill = time_prefill(llm.steps, T, 2, vocab)
            ms_decode, _ = time_decode_device(llm.steps, batch, context, args.steps, args.warmup, vocab)
            llm.steps.check_status()
            models.append({"model": f"{arch} at the {SHAPES[name][0]} layer sizes, {layers} layers",
                           "prefill_2048_tok_s": round(T / ms_prefill * 1e3, 1), "prefill_ms": round(ms_prefill, 3),
                           "decode_b8_ctx2048_tok_s": round(batch / ms_decode * 1e3, 1), "decode_ms_per_step": round(ms_decode, 4),
                           "weight_gb": round(llm.model.weight_bytes() / 1e9, 3)})
            del llm
            torch.cuda.empty_cache()
    table = pinorax_kernel_table(2048, 32, 64, 8192, 128256, layers, T, pk)
    print(json.dumps({"metric": "Pinorax beside Gekupel and Llama at equal layer sizes (random bf16 weights)", "impl": "ours", "n_gpus": 1,
                      "dtype": "bf16", "steps": args.steps, "warmup": args.warmup, "peaks": pk["source"],
                      "peak_gb_s": pk["hbm_gbs"], "peak_tflops": pk["bf16_tflops"], "models": models, "kernels": table}))
    return 0


# ---------------------------------------------------------------------------------------------- Fovezen beside Nipadra
def fovezen_config(width, ff, layers, vocab, heads, head_dim, kv_heads, window):
    """A Fovezen model with the layer sizes of a Llama shape, two copies of the stream, every layer with the same
    feed-forward. Layers in turn: the parallel pair (windowed attention with Llama's heads, three taps and soft-capped
    scores, beside gated linear attention with heads of 64 x 128), attention over all keys with half a head rotated,
    the state-space mixer (heads of 64, state 128), the parallel pair again."""
    par = {"type": "parallel", "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "mask": {"size": window}, "conv": 3,
                 "softcap": 30.0, "scale": head_dim ** -0.5},
        "right": {"heads": width // 128, "dim": 64, "vdim": 128, "tau": 16.0, "rank": 16}}}
    att = {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "scale": head_dim ** -0.5,
                                          "rot": {"base": 500000.0, "dims": head_dim // 2,
                                                  "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}}
    ssm = {"type": "mamba2", "mixer": {"heads": width // 64, "vdim": 64, "state": 128, "groups": 1, "conv": 4, "norm_groups": 1}}
    kinds = [par, att, ssm, par]
    return {"architecture": "Fovezen", "width": width, "vocab": vocab, "norm": {"eps": 1e-6}, "streams": 2, "logit_scale": 0.5,
            "layers": [dict(kinds[i % 4], mlp={"ff": ff, "kind": "dense", "limit": 7.0}) for i in range(layers)]}


def fovezen_kernel_table(width, heads, kv_heads, head_dim, window, T, pk):
    """Each kernel that the design added or changed, alone, beside the like kernel of the Nipadra or Llama path, at the
    sizes of one layer: a prompt portion of ``T`` tokens of one request and a decode step of 8 requests at a context of
    ``T``. ``frac`` is the time the kernel's algorithmic bytes (or, where larger, its multiply-adds on the tensor cores) need
    at the measured peaks, divided by the time it took; ``frac_of_32bit_issue`` the same against the CUDA cores' 32-bit
    rate, for kernels whose arithmetic has to stay 32-bit."""
    import torch
    from geneinfer_b200.ops import kernels as K
    dev = torch.device("cuda:0")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []
    props = torch.cuda.get_device_properties(dev)
    simt_ops = props.multi_processor_count * 128 * 1.965e9
    bf = torch.bfloat16

    def add(name, like, fn, nbytes, flops=0.0, simt=0.0):
        ms = time_calls(fn, flush=flush)
        ideal = max(nbytes / (pk["hbm_gbs"] * 1e9), flops / (pk["bf16_tflops"] * 1e12)) * 1e3
        row = {"kernel": name, "like": like, "us": round(ms * 1e3, 1), "frac": round(ideal / ms, 3)}
        if simt:
            row["frac_of_32bit_issue"] = round(simt / simt_ops * 1e3 / ms, 3)
        rows.append(row)

    D, page, S = width, 16, 2
    for what, R, n in (("prefill", 1, T), ("decode", 8, 1)):
        N = R * n
        i32 = dict(dtype=torch.int32, device=dev)
        s0, sl, slots = torch.arange(R, **i32) * n, torch.full((R,), n, **i32), torch.arange(R, **i32)
        rr = torch.arange(R, **i32).repeat_interleave(n)
        # the copies of the stream: rewrite + next read in one pass, beside the norm kernels of the other designs
        X, y = torch.randn(N, S, D, device=dev), torch.randn(N, D, device=dev)
        xn = torch.empty(N, D, dtype=bf, device=dev)
        w = torch.ones(D, device=dev)
        mix, ow, iw = torch.eye(S, device=dev), torch.ones(S, device=dev), torch.full((S,), 0.5, device=dev)
        add(f"streams: rewrite of 2 copies + next read ({what})", "residual_norm",
            lambda: K.streams(X, y=y, clear_y=True, mix=mix, out_w=ow, in_w=iw, norm_weight=w, eps=1e-6, xn_out=xn), N * D * (S * 8 + 8 + 2))
        acc, xo = torch.empty(N, D, device=dev), torch.empty(N, D, device=dev)
        add(f"residual_norm, Nipadra ({what})", "", lambda: K.residual_norm(y, w, xo, 1e-6, 2.0, acc_out=acc, xn_out=xn), N * D * 14)
        add(f"rmsnorm, Llama ({what})", "", lambda: K.rmsnorm(y, w, xn, 1e-6), N * D * 6)
        add(f"add_normed, a branch's output into the sum ({what})", "rmsnorm", lambda: K.add_normed(y, w, xo, 1e-6, clear_y=True), N * D * 16)
        # gated linear attention: heads of 64 x 128
        H, dk, dv = D // 128, 64, 128
        proj = torch.randn(N, 2 * H * dk + 2 * H * dv, device=dev) * 0.5
        z = torch.randn(N, H * dk, device=dev) + 3.0
        zb = torch.zeros(H * dk, device=dev)
        out = torch.empty(N, H * dv, device=dev)
        state = torch.zeros(R, H * dk * dv, device=dev)
        parts, parts_c = {}, {}
        if N > K.SCAN_PART:
            ws = torch.empty(K.scan_parts(N, R), H * dk * dv, device=dev)
            parts = {"part_len": K.SCAN_PART, "ws_state": ws, "ws_decay": torch.empty(N, H * dk, device=dev)}
            parts_c = {"part_len": K.SCAN_PART, "ws_state": ws, "ws_decay": torch.empty(N, H, device=dev)}
        scan_bytes = N * (2 * H * dk + 2 * H * dv) * 4 + 2 * R * H * dk * dv * 4
        macs = N * H * dk * dv * (4.0 if parts else 3.0)
        add(f"linear_scan, a decay per row ({what})", "linear_scan", lambda: K.linear_scan(
            proj, 0, proj, H * dk, proj, 2 * H * dk, H, 1, dk, dv, False, state, 0, s0, sl, slots, out, row_gate=z, row_gate_bias=zb,
            tau=16.0, q_scale=0.125, **parts), scan_bytes + N * H * dk * 4, simt=macs)
        decay = torch.full((H,), 0.99, device=dev)
        add(f"linear_scan, constant decay, Nipadra ({what})", "", lambda: K.linear_scan(
            proj, 0, proj, H * dk, proj, 2 * H * dk, H, 1, dk, dv, True, state, 0, s0, sl, slots, out, decay=decay, **parts_c), scan_bytes,
            simt=macs)
        yb = torch.empty(N, H * dv, dtype=bf, device=dev)
        nw = torch.ones(H * dv, device=dev)
        add(f"gated_group_norm per head, SiLU gate after ({what})", "gated_group_norm",
            lambda: K.gated_group_norm(out, proj, 2 * H * dk + H * dv, nw, yb, H, 1e-6, False, gate_act="silu"), N * H * dv * 10)
        add(f"gated_group_norm, Nipadra ({what})", "", lambda: K.gated_group_norm(out, proj, 2 * H * dk + H * dv, nw, yb, 1, 1e-6, False),
            N * H * dv * 10)
        # windowed attention: convolution of [q; k; v], norm + store, attention with soft-capped scores
        C = (heads + 2 * kv_heads) * head_dim
        qkv = torch.randn(N, C, device=dev)
        cw = torch.randn(C, 3, device=dev) * 0.3
        st = torch.zeros(R, 2 * C, device=dev)
        mixed = torch.empty(N, C, device=dev)
        add(f"causal_conv of [q; k; v], no bias or activation ({what})", "causal_conv",
            lambda: K.causal_conv(qkv, 0, cw, None, st, 0, rr, s0, sl, slots, mixed, activate=False), N * C * 8)
        cb = torch.zeros(C, device=dev)
        add(f"causal_conv with bias and SiLU, Nipadra ({what})", "", lambda: K.causal_conv(qkv, 0, cw, cb, st, 0, rr, s0, sl, slots, mixed), N * C * 8)
        n_pages = R * ((T + page - 1) // page)
        kc = torch.randn(n_pages, kv_heads, page, head_dim, device=dev).to(bf)
        vc = torch.randn(n_pages, kv_heads, page, head_dim, device=dev).to(bf)
        tables = torch.arange(n_pages, **i32).view(R, -1)
        pos = (torch.arange(n, **i32) + (T - n)).repeat(R)
        q = torch.empty(N, heads * head_dim, dtype=bf, device=dev)
        hw = torch.ones(head_dim, device=dev)
        freq = torch.rand(head_dim // 4, device=dev)
        store_bytes = N * (C * 4 + C * 2)
        add(f"norm_rope_store, norm per head, no rotation ({what})", "norm_rope_store", lambda: K.norm_rope_store(
            qkv, 0, heads * head_dim, (heads + kv_heads) * head_dim, hw, hw, 1e-6, None, False, pos, rr, tables, q, kc, vc, heads, kv_heads,
            head_dim, page), store_bytes)
        wq, wk = torch.ones(heads * head_dim, device=dev), torch.ones(kv_heads * head_dim, device=dev)
        add(f"norm_rope_store, one norm over all heads, half a head rotated ({what})", "norm_rope_store", lambda: K.norm_rope_store(
            qkv, 0, heads * head_dim, (heads + kv_heads) * head_dim, wq, wk, 1e-6, freq, False, pos, rr, tables, q, kc, vc, heads, kv_heads,
            head_dim, page, wide_norm=True), store_bytes)
        fr = torch.rand(head_dim // 2, device=dev)
        add(f"norm_rope_store, Nipadra ({what})", "", lambda: K.norm_rope_store(
            qkv, 0, heads * head_dim, heads * head_dim, hw, hw, 1e-6, fr, True, pos, rr, tables, q, kc, vc, heads, kv_heads, head_dim, page),
            store_bytes)
        att = torch.empty_like(q)
        seen = sum(min(window, p + 1) for p in range(T - n, T))
        att_flops = 4.0 * R * seen * heads * head_dim
        att_bytes = R * min(T, window + n) * kv_heads * head_dim * 4 + N * heads * head_dim * 4

        class Ctx:                      # what attention_rows_of_step reads of a step
            row_req, positions, page_size, max_position = rr, pos, page, T

            @staticmethod
            def scratch(name, shape, dtype, capacity=None):
                key = (name, tuple(shape), dtype)
                if key not in Ctx.kept:
                    Ctx.kept[key] = torch.empty(shape, dtype=dtype, device=dev)
                return Ctx.kept[key]

            @staticmethod
            def attention_work(per_tile):
                if n == 1:
                    return torch.arange(R, **i32), torch.zeros((0, 3), **i32), T
                tiles = [(t, min(per_tile, n - t), 0) for t in range(0, n, per_tile)]
                return torch.zeros(0, **i32), torch.tensor(tiles, **i32), 0
        Ctx.kept = {}
        add(f"attention_rows, window {window}, soft-capped scores ({what})", "attention", lambda: K.attention_rows_of_step(
            Ctx, q, kc, vc, att, tables, heads, kv_heads, head_dim, head_dim, head_dim ** -0.5, window, None, None, None, softcap=30.0),
            att_bytes, att_flops)
        rows_dec = torch.arange(R, **i32)
        per_tile = 128 // (heads // kv_heads)
        work = torch.tensor([(t, min(per_tile, n - t), 0) for t in range(0, n, per_tile)][::-1], **i32)
        chunk = K.attention_chunk_keys()
        n_chunks = (T + chunk - 1) // chunk
        part_o = torch.empty(R, heads * n_chunks * head_dim, device=dev)
        part_ml = torch.empty(R, heads * n_chunks * 2, device=dev)
        gate = torch.randn(N, heads, device=dev)

        def attend(win, **ep):
            if n == 1:
                K.attention_decode(q, kc, vc, att, rows_dec, rr, pos, tables, heads, kv_heads, head_dim, page, head_dim ** -0.5, win,
                                   part_o, part_ml, n_chunks, n_chunks, **ep)
            else:
                K.attention_prefill_tc(q, kc, vc, att, work, pos, tables, heads, kv_heads, head_dim, page, head_dim ** -0.5, win, **ep)
        # where the design's attention runs at these sizes: the tensor-core kernels of plain attention, with the cap in their softmax pass
        add(f"attention on the tensor cores, window {window}, soft-capped scores ({what})", "attention", lambda: attend(window, softcap=30.0),
            att_bytes, att_flops)
        add(f"window attention with sink and gate, Nipadra ({what})", "", lambda: attend(window, sink=True, gate=gate, gate_offset=0),
            att_bytes, att_flops)
    return rows


def run_fovezen(args):
    """Prefill (one 2,048-token prompt in one step) and decode (batch 8 at context 2,048) throughput of Fovezen models whose
    layers have the sizes of the Llama-3.2-1B and Llama-3.1-8B shapes (four layers each, random bf16 weights), beside Nipadra
    (the closest existing design: a windowed attention beside a recurrence, a state-space mixer, linear attention) and Llama
    models of the same sizes; then every kernel that the design added or changed alone beside its like kernel. One JSON line."""
    import torch
    from geneinfer_b200 import Engine
    from geneinfer_b200.weights import write_random_model
    pk = peaks()
    layers = args.layers or 4
    context, batch, T = 2048, 8, PREFILL_TOKENS
    models = []
    for name, base in (("1b", LLAMA_1B), ("8b", LLAMA_8B)):
        llama = dict(base, num_hidden_layers=layers, tie_word_embeddings=True)
        shape = (base["hidden_size"], base["intermediate_size"], layers, base["vocab_size"], base["num_attention_heads"], base["head_dim"],
                 base["num_key_value_heads"], 1024)
        for arch, cfg in (("Llama", llama), ("Nipadra", nipadra_config(*shape)), ("Fovezen", fovezen_config(*shape))):
            if arch == "Llama":
                folder = model_folder(cfg)
            else:
                folder = os.path.join(tempfile.gettempdir(), f"geneinfer_bench_{arch.lower()}_{name}_{layers}_{os.getuid()}")
                if not os.path.isfile(os.path.join(folder, "done")):
                    write_random_model(cfg, 1, folder, "bfloat16", std=0.02)
                    open(os.path.join(folder, "done"), "w").close()
            llm = Engine(folder, dtype="bfloat16", max_seq_len=context, page_size=PAGE, kv_pages=batch * (context // PAGE),
                         max_running=batch, step_tokens=T, prefix_cache=False)
            vocab = base["vocab_size"]
            ms_prefill = time_prefill(llm.steps, T, 2, vocab)
            ms_decode, _ = time_decode_device(llm.steps, batch, context, args.steps, args.warmup, vocab)
            llm.steps.check_status()
            models.append({"model": f"{arch} at the {SHAPES[name][0]} layer sizes, {layers} layers",
                           "prefill_2048_tok_s": round(T / ms_prefill * 1e3, 1), "prefill_ms": round(ms_prefill, 3),
                           "decode_b8_ctx2048_tok_s": round(batch / ms_decode * 1e3, 1), "decode_ms_per_step": round(ms_decode, 4),
                           "weight_gb": round(llm.model.weight_bytes() / 1e9, 3)})
            del llm
            torch.cuda.empty_cache()
    table = fovezen_kernel_table(2048, 32, 8, 64, 1024, T, pk)
    print(json.dumps({"metric": "Fovezen beside Nipadra and Llama at equal layer sizes (random bf16 weights)", "impl": "ours", "n_gpus": 1,
                      "dtype": "bf16", "steps": args.steps, "warmup": args.warmup, "peaks": pk["source"],
                      "peak_gb_s": pk["hbm_gbs"], "peak_tflops": pk["bf16_tflops"], "models": models, "kernels": table}))
    return 0


def run_scenario(args):
    """Two workloads through the entry point, beside the default run: ``mixed`` (32 requests with
    prompts of 128 to 4096 random ids and 256 generated tokens each, admitted together, prompts cut
    into portions beside decoding requests) and ``prefix`` (64 requests with 2,048-token prompts of
    which the first 1,024 are one of four shared prefixes, 512 generated tokens each, with the
    prefix cache on and off). Prints one JSON line."""
    import numpy as np
    import torch
    from geneinfer_b200 import Engine, SamplingParams
    shape_name, shape = SHAPES[args.shape]
    cfg = dict(shape)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    folder = model_folder(cfg)
    vocab = cfg["vocab_size"]
    rng = np.random.default_rng(11)

    def ids(n):
        return [int(t) for t in rng.integers(0, vocab, n)]

    if args.scenario == "mixed":
        n_req, new, running = 32, 256, 32
        prompts = [ids(int(n)) for n in rng.integers(128, 4097, n_req)]
        variants = [("prefix_cache_on", True)]
    else:
        n_req, new, running = 64, 512, 64
        prefixes = [ids(1024) for _ in range(4)]
        prompts = [prefixes[i % 4] + ids(1024) for i in range(n_req)]
        variants = [("prefix_cache_on", True), ("prefix_cache_off", False)]
    longest = max(len(p) for p in prompts) + new
    pages = sum((len(p) + new + PAGE - 1) // PAGE + 1 for p in prompts)
    out = {"metric": f"{args.scenario} workload, generated tok/s ({shape_name} shape, random bf16 weights)", "impl": "ours",
           "n_gpus": 1, "dtype": "bf16", "data": "synthetic: seeded random weights and token ids",
           "config": {"model": f"{shape_name} shape", "layers": cfg["num_hidden_layers"], "requests": n_req,
                      "prompt_tokens": sum(len(p) for p in prompts), "generated_per_request": new, "max_running": running,
                      "step_tokens": 2048, "page_size": PAGE}}
    dtype = "float32" if args.dtype == "float32" else "bfloat16"
    out["dtype"] = "fp32" if dtype == "float32" else "bf16"
    results = {}
    for name, cache_on in variants:
        llm = Engine(folder, dtype=dtype, max_seq_len=longest, page_size=PAGE, kv_pages=pages, max_running=running,
                     step_tokens=2048, prefix_cache=cache_on)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        if args.scenario == "prefix":
            # the first request of each prefix arrives first; the others once its prompt is in the cache
            rids = [llm.submit(p, len(p) + new - 1, SamplingParams(0.0)) for p in prompts[:4]]
            while any(llm.result(r).first_token_step < 0 for r in rids):
                llm.step()
            rids += [llm.submit(p, len(p) + new - 1, SamplingParams(0.0)) for p in prompts[4:]]
        else:
            rids = [llm.submit(p, len(p) + new - 1, SamplingParams(0.0)) for p in prompts]
        llm.run_until_idle()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        res = [llm.result(r) for r in rids]
        bad = [r.error or len(r.generated_tokens) for r in res if r.error or len(r.generated_tokens) != new]
        if bad:
            raise RuntimeError(f"scenario {args.scenario}: requests did not finish as expected: {bad[:4]}")
        results[name] = [list(r.generated_tokens) for r in res]
        st = llm.stats
        out[name] = {"seconds": round(dt, 3), "generated_tok_s": round(n_req * new / dt, 1),
                     "all_tok_s": round((sum(len(p) for p in prompts) + n_req * new) / dt, 1), "steps": st.steps,
                     "preemptions": st.preemptions, "prefix_hits": st.prefix_hits, "cached_positions": st.prefix_tokens,
                     "evicted_pages": st.evicted_pages, "max_tokens_in_step": st.max_tokens_in_step}
        llm.clear_prefix_cache()
        llm.steps.cache.check_invariants()
        if llm.steps.cache.free_pages() != pages:
            raise RuntimeError("scenario: pages were lost")
        del llm
        torch.cuda.empty_cache()
    # a sampled subset again, each request alone (the reference's serve bench compares every request with its run
    # alone, bench/serve_bench_main.cpp:18,202). In 32-bit every output is one fixed chain of operations, so the tokens
    # must be identical; in bfloat16 a product of 1 token and one of 2,048 round differently, and the nearly flat logits
    # of random weights let a near-tie fall either way: there the count is reported, with the first place that differs.
    order = sorted(range(n_req), key=lambda i: len(prompts[i]))
    subset = sorted({order[0], order[n_req // 2], order[-1]})
    alone = Engine(folder, dtype=dtype, max_seq_len=longest, page_size=PAGE, kv_pages=(longest + PAGE - 1) // PAGE + 1,
                   max_running=1, step_tokens=2048, prefix_cache=False)
    same, first_diff = 0, None
    for i in subset:
        got = alone.generate([prompts[i]], max_new_tokens=new, temperature=0.0)[0]
        batched = results[variants[0][0]][i]
        if got == batched:
            same += 1
        elif first_diff is None:
            k = next(k for k in range(new) if got[k] != batched[k])
            # how close the two candidates were: the logits at that place once more (the request alone, fed in portions of 2,048)
            from geneinfer_b200.engine.step import StepEntry
            fed = list(prompts[i]) + batched[:k]
            alone.steps.open("gap")
            for c in range(0, len(fed), 2048):
                part = fed[c:c + 2048]
                logits = alone.steps.step([StepEntry("gap", part, [len(part) - 1] if c + 2048 >= len(fed) else [])])
            row = logits[0].float().cpu()
            alone.steps.close("gap")
            first_diff = {"request": i, "token": k, "logit_gap": round(abs(float(row[got[k]] - row[batched[k]])), 5),
                          "logit_spread": round(float(row.max() - row.median()), 3)}
    out["alone"] = {"requests_checked": len(subset), "identical_to_running_alone": same, "first_difference": first_diff}
    if dtype == "float32" and same != len(subset):
        raise RuntimeError(f"scenario {args.scenario}: in 32-bit a request generated other tokens than alone: {first_diff}")
    out["value"] = out[variants[0][0]]["generated_tok_s"]
    out["unit"] = "tok/s"
    print(json.dumps(out), flush=True)
    return 0


REF_DIR = os.path.join(ROOT, "baseline", "_ref")
REF_RUNS = 3


def reference_binary():
    """Path of the reference's own serve bench built with its CUDA backend, or (None, why). The
    reference is a CMake project (pip has nothing to install); its stock ``gi_serve_bench`` is built
    from the unmodified source tree into baseline/_ref/build when it is not there yet."""
    exe = os.path.join(REF_DIR, "build", "gi_serve_bench")
    if os.path.isfile(exe) and os.access(exe, os.X_OK):
        return exe, None
    src = os.environ.get("GI_REFERENCE_SRC") or os.path.join(os.path.dirname(ROOT), "reference")
    if not os.path.isfile(os.path.join(src, "CMakeLists.txt")):
        return None, f"the reference's source tree is not at {src} and no built gi_serve_bench is under baseline/_ref/build"
    os.makedirs(REF_DIR, exist_ok=True)
    steps = (["cmake", "-S", src, "-B", os.path.join(REF_DIR, "build"), "-DCMAKE_BUILD_TYPE=Release", "-DGI_CUDA=ON",
              "-DCMAKE_CUDA_ARCHITECTURES=100"],
             ["cmake", "--build", os.path.join(REF_DIR, "build"), "--target", "gi_serve_bench", "-j", "8"])
    env = dict(os.environ)
    if os.path.isfile("/usr/local/cuda/bin/nvcc"):
        env.setdefault("CUDACXX", "/usr/local/cuda/bin/nvcc")
    for cmd in steps:
        try:
            p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=1200, env=env)
        except (OSError, subprocess.TimeoutExpired) as e:
            return None, f"building the reference failed: {e}"
        if p.returncode != 0:
            tail = [l for l in p.stdout.splitlines() if l.strip()][-3:]
            return None, "building the reference with its CMake files failed: " + " | ".join(tail)[:400]
    return (exe, None) if os.path.isfile(exe) else (None, "the reference's build produced no gi_serve_bench")


def run_reference(args):
    """The unmodified reference through its own serve bench and CUDA backend, on the random model
    folder this bench writes: 8 requests of 16 prompt + 64 generated tokens run together, the
    workload that finishes (at context 8192 its run printed nothing within 15 minutes and is not
    run again). Nothing of this repository's models, kernels or engine is on this path."""
    if args.gpus != 1:
        print(json.dumps({"impl": "reference", "unavailable": "the reference's device backend runs on one GPU"}), flush=True)
        return 0
    exe, why = reference_binary()
    if exe is None:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
        return 0
    shape_name, shape = SHAPES["1b"]
    cfg = dict(shape)
    folder = model_folder(cfg)
    batch = 8
    cmd = [exe, "--model", folder, "--device", "cuda", "--concurrency", str(batch), "--prompt-tokens", str(SHORT_PROMPT),
           "--decode-tokens", str(SHORT_NEW), "--runs", str(REF_RUNS), "--max-seq-len", "256"]
    clocks = ClockSampler()
    clocks.start()
    try:
        p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=1500)
    except (OSError, subprocess.TimeoutExpired) as e:
        clocks.stop()
        print(json.dumps({"impl": "reference", "unavailable": f"gi_serve_bench did not finish: {e}"}), flush=True)
        return 0
    clock_record = clocks.stop()
    row = None
    for l in p.stdout.splitlines():
        f = l.split()
        if len(f) >= 8 and f[0] == str(batch):
            try:
                row = (float(f[1]), float(f[2]), float(f[4]), " ".join(f[7:]))
            except ValueError:
                pass
    if row is None:
        tail = " | ".join([l for l in p.stdout.splitlines() if l.strip()][-3:])[:400]
        print(json.dumps({"impl": "reference", "unavailable": f"gi_serve_bench gave no result line (exit {p.returncode}): {tail}"}),
              flush=True)
        return 0
    wall, tps, rows_per_pass, outputs = row
    line = {
        "metric": f"generated tok/s, {batch} concurrent requests of {SHORT_PROMPT} prompt + {SHORT_NEW} generated tokens "
                  f"({shape_name} shape, random bf16 weights), wall time with the prompts",
        "value": tps, "unit": "tok/s", "n_gpus": 1, "impl": "reference", "same_config": False,
        "steps": REF_RUNS * SHORT_NEW, "warmup": SHORT_NEW, "ms_per_step": round(wall / SHORT_NEW * 1e3, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 weights; 32-bit activations and cache (the reference's device backend)",
        "data": "synthetic: the same random model folder as the other arm, the tool's own random token ids",
        "config": {"model": f"{shape_name} shape", "global_batch": batch, "seq_len": SHORT_PROMPT + SHORT_NEW,
                   "parallelism": "single GPU", "tool": "gi_serve_bench --device cuda", "runs": REF_RUNS,
                   "rows_per_pass": rows_per_pass, "outputs": outputs,
                   "compare_with": "points.short_requests_b8 of the other arm (the same workload through Engine.generate)",
                   "why_not_context_8192": "the reference's run at context 8192 printed no result within 15 minutes"},
        "e2e": {"value": tps, "unit": "tok/s", "note": "the tool's own wall clock: token ids from the host in, generated ids out"},
        "clocks": clock_record,
    }
    print(json.dumps(line), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the named configuration (0 = all)")
    ap.add_argument("--shape", choices=sorted(SHAPES), default="1b", help="layer sizes (the default is the baseline's third configuration)")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16",
                    help="precision of a --scenario run (float32: the requests run alone must give identical tokens)")
    ap.add_argument("--scenario", choices=["mixed", "prefix", "sizes", "nipadra", "gekupel", "pinorax", "fovezen"], default="",
                    help="a workload through the scheduler (mixed, prefix) or decode steps at a grid of sizes, instead of the default run")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(3, args.warmup)
    if args.scenario == "sizes":
        return run_sizes(args)
    if args.scenario == "nipadra":
        return run_nipadra(args)
    if args.scenario == "gekupel":
        return run_gekupel(args)
    if args.scenario == "fovezen":
        return run_fovezen(args)
    if args.scenario == "pinorax":
        return run_pinorax(args)
    if args.scenario:
        return run_scenario(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
