#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Cerebras-GPT-1.3B shapes (random weights).

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L]

One "step" is one decode step of the whole batch.  The default run has the layer sizes of
the 1.3B configuration, bfloat16, a batch of 8 requests with 1,024-token prompts decoded
towards the context length 2,048.  It prints ONE JSON line:

* ``value``: decoded tokens per second, timed on the device with CUDA events around K replays
  of the captured decode step (model, argmax and the move to the next position all on the
  device);
* ``e2e``: the same through the Python entry point (``Engine.step``: scheduler, packed inputs
  copied from pinned host memory, sampled tokens read back every step);
* ``prefill``: one 2,048-token prompt in one step, tokens per second and the fraction of the
  bf16 matrix peak its flops reach;
* ``roofline``: bytes a decode step has to read (every weight once and the cache of the live
  requests) over its time, against the measured copy bandwidth;
* ``points``: decode at batch 1 and 64.

Peaks come from MEASURED_PEAKS.json beside this file when it exists.  This engine runs on one
GPU: with --gpus N > 1 it says so and exits with status 2.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Cerebras-GPT-1.3B layer sizes (GPT2LMHeadModel)
CONFIG_1_3B = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=24, n_embd=2048, n_head=16,
                   n_inner=8192, vocab_size=50257, n_positions=2048, activation_function="gelu",
                   layer_norm_epsilon=1e-5, tie_word_embeddings=True)
# Cerebras-GPT-6.7B and GPT-2 XL layer sizes (further configurations of the benchmark set)
CONFIG_6_7B = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=32, n_embd=4096, n_head=32,
                   n_inner=16384, vocab_size=50257, n_positions=2048, activation_function="gelu",
                   layer_norm_epsilon=1e-5, tie_word_embeddings=True)
CONFIG_XL = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=48, n_embd=1600, n_head=25,
                 n_inner=6400, vocab_size=50257, n_positions=1024, activation_function="gelu_new",
                 layer_norm_epsilon=1e-5, tie_word_embeddings=True)
# the reference's one fixed model (include/config.hpp:5-21) for its own workload (--config batching)
CONFIG_REFERENCE = dict(architectures=["TinyGPT"], n_layer=4, n_embd=256, n_head=8, n_inner=1024, vocab_size=1000,
                        n_positions=2048, activation_function="gelu", layer_norm_epsilon=1e-5, tie_word_embeddings=False)
REFERENCE_BUILD = os.path.join(ROOT, "baseline", "_ref")     # the unmodified reference, built with its own CMakeLists
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out = {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
            if "bf16_tflops_sustained" in d:
                out["bf16_tflops_sustained"] = float(d["bf16_tflops_sustained"])
            return out
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", default="1.3b", choices=["1.3b", "6.7b", "xl", "batching", "vekedra", "figotar", "vatevik", "divitar"],
                    help="1.3b: the default measurement; 6.7b: batch-64 decode at context 2,048; "
                         "xl: 64 mixed requests through the scheduler (prompts 32-768, 256 outputs each); "
                         "batching: the reference's own workload at the reference's own sizes (both --impl arms); "
                         "vekedra: prefill and decode of the Vekedra design at two layer sizes beside the GPT-2 style model "
                         "of equal width and depth, and its own kernels one by one against their bytes; "
                         "figotar: the same for the Figotar design, beside Vekedra and the GPT-2 style model; "
                         "vatevik: the same for the Vatevik design, beside Figotar and the GPT-2 style model; "
                         "divitar: the same for the Divitar design, beside Figotar, Vekedra and the GPT-2 style model")
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--prompt-len", type=int, default=None)
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1/64, prefill and e2e")
    ap.add_argument("--prefill-only", action="store_true", help="time only the 2,048-token prefill (for profilers)")
    ap.add_argument("--prefill-portion", type=int, default=None, help="with --prefill-only: the prompt in steps of this many tokens")
    args = ap.parse_args()

    if args.config == "batching":
        return reference_workload(args)
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference cannot run this configuration: its model sizes are compile-time constants "
                          "(include/config.hpp:5-21: 4 layers, width 256, vocabulary 1000) and it computes in fp32 only; "
                          "built unmodified with its own CMakeLists it runs its own workload here: "
                          "bench.py --config batching --impl reference"}))
        return 0
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print(f"bench.py: this engine runs on ONE GPU; --gpus {args.gpus} is not supported (single-GPU tier)")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import cbis_b200 as cb
    from cbis_b200.engine import StepEntry
    from cbis_b200.kernels import ops

    torch.cuda.set_device(0)
    if args.config == "xl":
        return mixed_workload(args, cb, torch)
    if args.config == "vekedra":
        return vekedra_workload(args, cb, torch)
    if args.config == "figotar":
        return figotar_workload(args, cb, torch)
    if args.config == "vatevik":
        return vatevik_workload(args, cb, torch)
    if args.config == "divitar":
        return divitar_workload(args, cb, torch)
    if args.config == "6.7b":
        args.skip_points = True
        args.batch = args.batch or 64
        args.steps = min(args.steps, 64)
        args.prompt_len = args.prompt_len or (CONFIG_6_7B["n_positions"] - args.warmup - args.steps - 24)
    args.batch = args.batch or 8
    args.prompt_len = args.prompt_len or 1024
    cfgd = dict(CONFIG_6_7B if args.config == "6.7b" else CONFIG_1_3B)
    n_layer_config = cfgd["n_layer"]
    if args.layers:
        cfgd["n_layer"] = args.layers
    P = cfgd["n_positions"]
    K, W, B, PL = args.steps, args.warmup, args.batch, args.prompt_len
    K = max(1, min(K, P - PL - W - 20))
    pk = peaks()
    max_b = B if args.skip_points else max(B, 64)
    if args.prefill_only:
        max_b = 1
    eng = cb.Engine.from_random(cfgd, seed=1234, dtype="bfloat16", page_size=args.page_size,
                                max_tokens=max_b * P, max_num_seqs=max_b, max_batched_tokens=2048,
                                prefill_chunk=2048)
    model, runner, mgr = eng.model, eng.runner, eng.pool.manager
    V = cfgd["vocab_size"]
    gen = torch.Generator().manual_seed(0)

    def prompts(n, length):
        return torch.randint(0, V, (n, length), generator=gen).tolist()

    def prefill_slots(ps):
        """Prefills prompts through the step function (two per step); returns their slots."""
        slots = [eng.open_request(i) for i in range(len(ps))]
        per = max(1, 2048 // len(ps[0]))
        for i in range(0, len(ps), per):
            eng.forward_step([StepEntry(slots[j], 0, ps[j], []) for j in range(i, min(i + per, len(ps)))])
        return slots

    def decode_device(batch, steps, warm, prompt_len=None):
        """tokens/s of `steps` captured decode steps after `warm` untimed ones; also ms/step, launches/step."""
        PL = prompt_len or args.prompt_len
        ps = prompts(batch, PL)
        slots = prefill_slots(ps)
        for s in slots:
            assert mgr.append(s, warm + steps + 2)
        ops.reset_launch_count()
        loop = runner.decode_loop([StepEntry(s, PL, [1], [0]) for s in slots])
        per_step = ops.launch_count() // 2          # the loop ran its step twice: warm-up and capture
        loop.run(warm)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        loop.run(steps)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        for s in slots:
            eng.close_request(s)
        del loop
        return batch * steps / (ms / 1e3), ms / steps, per_step

    def prefill_once(T, portion=None):
        """Median milliseconds of one T-token prompt run as ONE step, or in steps of ``portion`` tokens
        (3 warm-ups, 5 timed)."""
        toks = prompts(1, T)[0]
        portion = portion or T
        times = []
        for it in range(3 + 5):
            slot = eng.open_request(1000 + it)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for at in range(0, T, portion):
                part = toks[at:at + portion]
                eng.forward_step([StepEntry(slot, at, part, [len(part) - 1] if at + portion >= T else [])])
            e1.record()
            torch.cuda.synchronize()
            if it >= 3:
                times.append(e0.elapsed_time(e1))
            eng.close_request(slot)
        return statistics.median(times)

    if args.prefill_only:
        ms = prefill_once(2048, args.prefill_portion)
        print(json.dumps({"prefill_ms": round(ms, 3), "tokens": 2048, "portion": args.prefill_portion or 2048,
                          "n_layer": cfgd["n_layer"]}))
        return 0

    # ---- main measurement: decode at the default batch, clocks sampled meanwhile -------------
    sampler = ClockSampler()
    sampler.start()
    value, ms_per_step, launches_per_step = decode_device(B, K, W)
    clocks = sampler.stop()
    ctx_mean = PL + 1 + W + K / 2.0
    step_bytes = model.weight_bytes() + B * ctx_mean * eng.pool.bytes_per_token()
    achieved = step_bytes / (ms_per_step / 1e3) / 1e9
    result = {
        "metric": f"decode tokens/s (Cerebras-GPT-{args.config.upper()} shapes, batch {B}, context {PL}->{P})",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights N(0,0.02), uniform random token ids)",
        "impl": "b200",
        "config": {"model": f"Cerebras-GPT-{args.config.upper()} shapes (GPT2LMHeadModel)", "n_layer": cfgd["n_layer"],
                   "n_layer_config": n_layer_config, "n_embd": cfgd["n_embd"], "n_head": cfgd["n_head"],
                   "n_inner": cfgd["n_inner"], "vocab_size": V, "n_positions": P, "activation": "gelu",
                   "tied_head": True, "global_batch": B, "prompt_len": PL, "seq_len": P,
                   "page_size": args.page_size, "parallelism": "single GPU",
                   "l2": "inputs larger than L2: every step reads all weights and the live cache"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk["source"],
                     "bytes_per_step": int(step_bytes)},
        "clocks": clocks,
        "gpu_launches": int(launches_per_step * K),
    }

    if not args.skip_points:
        # ---- prefill of 2,048 tokens in one step ------------------------------------------------
        T = 2048
        ms = prefill_once(T)
        d, F, L = cfgd["n_embd"], cfgd["n_inner"], cfgd["n_layer"]
        flops = L * (2 * T * (3 * d * d + d * d + 2 * d * F) + 2 * T * T * d) + 2 * d * V
        result["prefill"] = {"value": round(T / (ms / 1e3), 1), "tokens": T, "ms": round(ms, 3),
                             "frac": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                             "flops": int(flops), "peak_tflops": pk["bf16_tflops"], "of": pk["source"]}
        ms512 = prefill_once(T, 512)     # the same prompt in four steps of 512 tokens, as a scheduler would cut it
        result["prefill"]["in_portions_of_512"] = {"value": round(T / (ms512 / 1e3), 1), "ms": round(ms512, 3)}
        # ---- decode at batch 1 and 64 -----------------------------------------------------------
        pts = {}
        for b in (1, 64):
            v, _, _ = decode_device(b, min(K, 256), W)
            pts[f"decode_b{b}"] = round(v, 1)
        # the default batch at the two ends of the context range: 32 steps from context 1,024 and 32 steps up to the last position
        v, _, _ = decode_device(B, 32, 3, prompt_len=PL)
        pts[f"decode_b{B}_ctx{PL}"] = round(v, 1)
        v, _, _ = decode_device(B, 32, 3, prompt_len=P - 40)
        pts[f"decode_b{B}_ctx{P}"] = round(v, 1)
        result["points"] = pts
        # ---- end to end through the Python entry point -------------------------------------------
        ps = prompts(B, PL)
        n_new = W + K + 16                      # no request ends inside the timed region
        for p in ps:
            eng.add_request(p, cb.SamplingParams(max_new_tokens=n_new))
        while not all_decoding(eng, B):
            eng.step()
        for _ in range(W):
            eng.step()
        torch.cuda.synchronize()
        tokens_before = eng.tokens_run
        t0 = time.perf_counter()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            eng.step()
        e1.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        steps_e2e, tokens_e2e = K, eng.tokens_run - tokens_before
        while eng.has_unfinished():
            eng.step()
        result["e2e"] = {"value": round(tokens_e2e / wall, 1), "unit": "tokens/s", "steps": steps_e2e,
                         "ms_per_step": round(wall * 1e3 / steps_e2e, 4),
                         "h2d_bytes_per_step": int(runner.bytes_per_step_h2d()), "d2h_bytes_per_step": 4 * B,
                         "device_ms_per_step": round(e0.elapsed_time(e1) / steps_e2e, 4)}
    print(json.dumps(result))
    return 0


def reference_workload(args) -> int:
    """The reference's own workload (src/bench_batching.cpp:26-33: 240 requests, Poisson arrivals 6 ms apart, prompts of
    4-16 and outputs of 8-32 tokens, 16 slots) at the reference's own model sizes.  --impl reference runs the unmodified
    reference's bench_batching (built with its own CMakeLists into baseline/_ref; its sm_89 PTX is compiled for the GPU
    at load) on its committed weights; the default arm runs this engine (bin/bench_batching) on random weights of the
    same sizes.  The throughput of both is set by the arrival rate; the latencies are what the engines decide."""
    import re
    import tempfile
    line = {"metric": "the reference's continuous-batching workload: tokens/s (prompt + output) and request latency",
            "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True, "data": "synthetic (uniform random token ids)",
            "config": {"model": "TinyGPT, the reference's sizes", "n_layer": 4, "n_embd": 256, "n_head": 8, "n_inner": 1024,
                       "vocab_size": 1000, "requests": 240, "mean_interarrival_ms": 6.0, "max_live": 16}}
    if args.impl == "reference":
        exe, weights = os.path.join(REFERENCE_BUILD, "build", "bench_batching"), os.path.join(REFERENCE_BUILD, "weights.bin")
        if not (os.path.isfile(exe) and os.path.isfile(weights)):
            print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref holds no build of the reference "
                              "(cmake -S <reference> -B baseline/_ref/build && cmake --build baseline/_ref/build; "
                              "its python/weights.bin copied to baseline/_ref/weights.bin)"}))
            return 0
        r = subprocess.run([exe, weights], capture_output=True, text=True, timeout=600)
        part = r.stdout.split("== static")[0]
        m = re.search(r"wall clock\s*:\s*([\d.]+) ms.*?token throughput\s*:\s*([\d.]+) tok/s.*?p50/p95/p99\s*:\s*([\d.]+) / "
                      r"([\d.]+) / ([\d.]+) ms", part, re.S)
        if r.returncode != 0 or not m:
            print(json.dumps({"impl": "reference", "unavailable": f"the reference's bench_batching ended with {r.returncode}"}))
            return 0
        line.update(impl="reference", dtype="fp32", value=float(m.group(2)), wall_ms=float(m.group(1)),
                    latency_ms={"p50": float(m.group(3)), "p95": float(m.group(4)), "p99": float(m.group(5))})
        print(json.dumps(line))
        return 0
    with tempfile.TemporaryDirectory() as d:
        cfg = os.path.join(d, "config.json")
        with open(cfg, "w") as f:
            json.dump(CONFIG_REFERENCE, f)
        r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "bench_batching"), "--random", cfg, "--json"],
                           capture_output=True, text=True, timeout=900)
    out = [l for l in r.stdout.splitlines() if l.startswith("{")]
    if r.returncode != 0 or not out:
        print(r.stdout[-2000:], r.stderr[-2000:], file=sys.stderr)
        return 1
    mine = json.loads(out[-1])
    line.update(impl="b200", dtype="bf16", value=mine["tokens_per_s"], wall_ms=mine["wall_ms"], latency_ms=mine["latency_ms"])
    print(json.dumps(line))
    return 0


def mixed_workload(args, cb, torch) -> int:
    """GPT-2 XL layer sizes: 64 requests, prompt lengths uniform in 32..768, 256 outputs each, all submitted at
    t = 0 and run by the scheduler (token budget 2,048, prompt portions of 512)."""
    import random
    cfgd = dict(CONFIG_XL)
    if args.layers:
        cfgd["n_layer"] = args.layers
    n_req, n_out = 64, 256
    eng = cb.Engine.from_random(cfgd, seed=1234, dtype="bfloat16", page_size=args.page_size,
                                max_tokens=n_req * cfgd["n_positions"], max_num_seqs=n_req, max_batched_tokens=2048,
                                prefill_chunk=512)
    rng = random.Random(0)
    prompts = [[rng.randrange(cfgd["vocab_size"]) for _ in range(rng.randint(32, 768))] for _ in range(n_req)]
    eng.generate(prompts[:8], cb.SamplingParams(max_new_tokens=4))       # warm-up: kernels
    eng.warm_up()                                                        # the decode graphs of every batch bucket
    torch.cuda.synchronize()
    steps0 = eng.steps
    step_ms, step_tokens = [], []
    ids = [eng.add_request(p, cb.SamplingParams(max_new_tokens=n_out)) for p in prompts]
    done = {}
    t0 = time.perf_counter()
    last = t0
    while eng.has_unfinished():          # what generate() does, with the wall time of every step noted
        for o in eng.step():
            done[o.request_id] = o.tokens
        now = time.perf_counter()        # the step's sampled tokens have been read back: the device has finished it
        step_ms.append((now - last) * 1e3)
        step_tokens.append(eng.last_step_tokens)
        last = now
    wall = last - t0
    outs = [done[i] for i in ids]
    n_prompt, n_gen = sum(map(len, prompts)), sum(map(len, outs))
    edges = [0.5, 1, 2, 3, 4, 6, 8, 12, 16, 24, 32]
    hist, lo = {}, 0.0
    for e in edges + [float("inf")]:
        hist[f"<={e:g}ms" if e != float("inf") else f">{edges[-1]:g}ms"] = sum(1 for t in step_ms if lo < t <= e)
        lo = e
    decode_only = [t for t, n in zip(step_ms, step_tokens) if n <= n_req]
    print(json.dumps({
        "metric": "mixed continuous-batching workload, tokens/s (GPT-2 XL shapes, 64 requests, prompts 32-768, 256 outputs)",
        "value": round((n_prompt + n_gen) / wall, 1), "unit": "tokens/s", "n_gpus": 1, "impl": "b200", "dtype": "bf16",
        "decode_tokens_per_s": round(n_gen / wall, 1), "wall_s": round(wall, 3), "steps": eng.steps - steps0,
        "prompt_tokens": n_prompt, "output_tokens": n_gen, "preemptions": eng.scheduler.preemptions(),
        "graph_replays": eng.runner.graph_replays, "step_shapes_captured": eng.runner.shape_captures,
        "step_ms": {"median": round(statistics.median(step_ms), 3), "p95": round(sorted(step_ms)[int(0.95 * len(step_ms))], 3),
                    "max": round(max(step_ms), 3),
                    "decode_only_median": round(statistics.median(decode_only), 3) if decode_only else None},
        "step_ms_histogram": hist,
        "higher_is_better": True, "data": "synthetic (random weights, uniform random token ids)",
        "config": {"model": "GPT-2 XL shapes (GPT2LMHeadModel)", "n_layer": cfgd["n_layer"], "n_layer_config": 48,
                   "n_embd": 1600, "n_head": 25, "n_inner": 6400, "vocab_size": 50257, "n_positions": 1024,
                   "requests": n_req, "max_batched_tokens": 2048, "prefill_chunk": 512, "page_size": args.page_size}}))
    return 0


def vekedra_sizes(width, layers):
    """A Vekedra configuration with layers of the sizes a model of this width would have: of every four layers one
    latent attention that keeps its latents, two state-space layers and one latent attention that reads the first
    one's; dense and routed feed-forwards in turn."""
    big = width >= 2048
    lat = {"dim": 128 if big else 64, "heads": 16, "kv_rank": 128, "mask": {"size": 1024 if big else 512},
           "scale": (128 if big else 64) ** -0.5, "vdim": 128 if big else 64}
    ssm = {"conv": 4, "groups": 8 if big else 1, "heads": 2 * width // 64, "norm_groups": 1, "state": 128 if big else 64,
           "vdim": 64}
    dense = {"kind": "dense", "ff": 11 * width // 4}
    moe = {"kind": "moe", "expert": {"ff": 11 * width // 16}, "router": {"experts": 16 if big else 8, "top": 2}}
    out = []
    for i in range(layers):
        kind = ("latent_attention", "mamba2", "mamba2", "latent_attention")[i % 4]
        mixer = dict(ssm if kind == "mamba2" else lat)
        if i % 4 == 3:
            mixer["kv_from"] = i - 3
        out.append({"type": kind, "mixer": mixer, "mlp": dict(dense if i % 2 == 0 else moe)})
    return {"architecture": "Vekedra", "embedding": {"scale": 1.0}, "layers": out, "norm": {"eps": 1e-5},
            "vocab": 32000, "width": width}


def measure_model(args, cb, torch, pk, cfgd, vocab, B, P, T, steps, warm, gen):
    """One model: the median time of a T-token prompt in one step (five runs after three), and decode steps of batch B
    from context 1,024 as one captured graph with the argmax on the device."""
    from cbis_b200.engine import StepEntry
    from cbis_b200.kernels import ops
    eng = cb.Engine.from_random(cfgd, seed=1234, dtype="bfloat16", page_size=args.page_size, max_tokens=B * P,
                                max_num_seqs=B, max_batched_tokens=T, prefill_chunk=T, max_model_len=P)
    mgr = eng.pool.manager
    toks = torch.randint(0, vocab, (B, T), generator=gen).tolist()
    times = []
    for it in range(3 + 5):
        slot = eng.open_request(it)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.forward_step([StepEntry(slot, 0, toks[0], [T - 1])])
        e1.record()
        torch.cuda.synchronize()
        if it >= 3:
            times.append(e0.elapsed_time(e1))
        eng.close_request(slot)
    prefill_ms = statistics.median(times)
    slots = [eng.open_request(100 + i) for i in range(B)]
    for i, s in enumerate(slots):
        eng.forward_step([StepEntry(s, 0, toks[i][:1024], [])])
        assert mgr.append(s, warm + steps + 2)
    ops.reset_launch_count()
    loop = eng.runner.decode_loop([StepEntry(s, 1024, [1], [0]) for s in slots])
    launches = ops.launch_count() // 2
    loop.run(warm)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    loop.run(steps)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    weights = eng.model.weight_bytes()
    del loop
    for s in slots:
        eng.close_request(s)
    del eng
    torch.cuda.empty_cache()
    return {"prefill_tokens_per_s": round(T / prefill_ms * 1e3, 1), "prefill_ms": round(prefill_ms, 3),
            "decode_tokens_per_s": round(B / ms * 1e3, 1), "decode_ms_per_step": round(ms, 4),
            "decode_launches_per_step": launches, "weight_bytes": int(weights),
            "decode_weight_stream_frac": round(weights / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4)}


def vekedra_workload(args, cb, torch) -> int:
    """Prefill (one 2,048-token prompt in one step) and decode (batch 8 from context 1,024, the captured step with
    argmax on the device) of the Vekedra design at two layer sizes, each beside the GPT-2 style model of equal width
    and depth; then the design's own kernels alone, at the larger size, against the bytes they have to move."""
    from cbis_b200.engine import StepEntry
    from cbis_b200.kernels import ops
    pk = peaks()
    P, T, B = 2048, 2048, args.batch or 8
    steps, warm = min(args.steps, 128), max(3, min(args.warmup, 8))
    layers = args.layers or 8
    gen = torch.Generator().manual_seed(0)

    def measure(cfgd, vocab):
        return measure_model(args, cb, torch, pk, cfgd, vocab, B, P, T, steps, warm, gen)

    sampler = ClockSampler()
    sampler.start()
    sizes = {}
    for width in (1024, 2048):
        vek = vekedra_sizes(width, layers)
        gpt = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=layers, n_embd=width, n_head=16,
                   n_inner=4 * width, vocab_size=32000, n_positions=P, activation_function="gelu",
                   layer_norm_epsilon=1e-5, tie_word_embeddings=False)
        sizes[f"width_{width}"] = {"vekedra": measure(vek, 32000), "gpt2_style": measure(gpt, 32000)}
    clocks = sampler.stop()
    line = {"metric": f"Vekedra prefill and decode tokens/s beside the GPT-2 style model of equal width and depth "
                      f"({layers} layers, batch {B}, prompt {T})", "unit": "tokens/s", "n_gpus": 1, "impl": "b200",
            "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids)", "higher_is_better": True,
            "value": sizes["width_2048"]["vekedra"]["decode_tokens_per_s"], "sizes": sizes,
            "kernels": vekedra_kernels(torch, ops, pk), "clocks": clocks, "peaks": pk}
    print(json.dumps(line))
    return 0


def vekedra_kernels(torch, ops, pk):
    """Microseconds of the design's own kernels alone (each replayed from a CUDA graph over buffers that rotate, so that
    inputs come from memory) at the layer sizes of width 2,048, with the bytes each has to move over its time as a
    fraction of the measured copy bandwidth; and the closest model's like kernel (LayerNorm over the same rows)."""
    W, H, Pd, N, G, K = 2048, 64, 64, 128, 8, 4
    inner, C = H * Pd, H * Pd + 2 * G * N
    d_proj = 2 * inner + 2 * G * N + H
    bf = torch.bfloat16
    out = {}

    def timed(make, nbytes, name, reps=20, copies=4):
        fns = [make() for _ in range(copies)]
        for f in fns:
            f()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for f in fns:
                f()
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) / reps / copies * 1e3
        out[name] = {"us": round(us, 2), "bytes": int(nbytes), "frac_of_copy_bandwidth": round(nbytes / us / 1e3 / pk["hbm_gbs"], 4)}

    for rows, segs, tag in ((2048, 1, "prefill_2048"), (8, 8, "decode_8")):
        per = rows // segs
        seg_slot = torch.arange(segs, dtype=torch.int32, device="cuda")
        cu = torch.arange(0, rows + 1, per, dtype=torch.int32, device="cuda")

        def conv():
            proj = torch.randn(rows, d_proj, device="cuda").to(bf)
            w, b = torch.randn(C, K, device="cuda"), torch.randn(C, device="cuda")
            st = torch.zeros(segs, (K - 1) * C, device="cuda")
            o = torch.empty(rows, C, dtype=bf, device="cuda")
            return lambda: ops.causal_conv_act(proj, inner, C, w, b, st, seg_slot, cu, segs, per, "silu", o)
        timed(conv, rows * C * 4 + segs * (K - 1) * C * 4, f"causal_conv_act_{tag}")

        def scan():
            xbc = (torch.randn(rows, C, device="cuda") * 0.5).to(bf)
            proj = torch.randn(rows, d_proj, device="cuda").to(bf)
            v = [torch.zeros(H, device="cuda") for _ in range(3)]
            st = torch.zeros(segs, inner * N, device="cuda")
            y = torch.empty(rows, inner, device="cuda")
            return lambda: ops.ssm_scan(xbc, proj, d_proj - H, v[0], v[1], v[2], st, seg_slot, cu, segs, H, Pd, N, G, y)
        timed(scan, rows * (C * 2 + inner * 4) + 2 * segs * inner * N * 4, f"ssm_scan_{tag}")

        def gnorm():
            y = torch.randn(rows, inner, device="cuda")
            z = torch.randn(rows, d_proj, device="cuda").to(bf)
            w = torch.ones(inner, device="cuda")
            o = torch.empty(rows, inner, dtype=bf, device="cuda")
            return lambda: ops.rms_norm(y, w, 1e-5, o, parts=1, gate=z[:, :inner])
        timed(gnorm, rows * inner * (4 + 2 + 2), f"gated_rms_norm_{tag}")

        def lnorm():
            x = torch.randn(rows, inner, device="cuda")
            d = torch.randn(rows, inner, device="cuda")
            w, b = torch.ones(inner, device="cuda"), torch.zeros(inner, device="cuda")
            o = torch.empty(rows, inner, dtype=bf, device="cuda")
            return lambda: ops.add_layernorm(x, d, None, w, b, 1e-5, o)
        timed(lnorm, rows * inner * (4 + 4 + 4 + 2), f"closest_model_add_layernorm_{tag}")

        E, F, top = 16, 1408, 2

        def experts():
            h = torch.randn(rows, W, device="cuda").to(bf)
            router = torch.randn(E, W, device="cuda").to(bf)
            gu = (torch.randn(E, 2 * F, W, device="cuda") * 0.02).to(bf)
            dn = (torch.randn(E, W, F, device="cuda") * 0.02).to(bf)
            ids = torch.empty(rows, top, dtype=torch.int32, device="cuda")
            wt = torch.empty(rows, top, device="cuda")
            hid = torch.empty(rows * top, F, dtype=bf, device="cuda")
            o = torch.empty(rows, W, device="cuda")

            def run():
                ops.route_topk(h, router, top, "sigmoid", False, ids, wt)
                if ops.routed_tiles_takes(h, gu, dn):          # as the part chooses
                    ops.routed_tiles(h, gu, dn, ids, wt, "silu", True, o)
                else:
                    ops.routed_gate_up(h, gu, ids, wt, "silu", True, hid)
                    ops.routed_down(hid, dn, ids, wt, True, o)
            return run
        touched = min(E, rows * top)
        timed(experts, touched * 3 * F * W * 2 + rows * W * 6, f"routed_feed_forward_{tag}", copies=2)
        if rows > 64:
            flops = 2.0 * rows * top * 3 * F * W
            us = out[f"routed_feed_forward_{tag}"]["us"]
            out[f"routed_feed_forward_{tag}"]["frac_of_bf16_peak"] = round(flops / us / 1e6 / pk["bf16_tflops"], 4)
    return out


def vatevik_sizes(width, layers):
    """A Vatevik configuration with layers of the sizes a model of this width would have: attention (grouped
    key/value heads, stretched rotation, blended values) and retention (half as many heads, values twice as wide as
    keys, decays 1 - 2^-(5 + h)) in turn; every layer with a gated feed-forward."""
    big = width >= 2048
    hd = 128 if big else 64
    heads = width // hd
    att = {"dim": hd, "heads": heads, "kv_heads": max(1, heads // 4),
           "rot": {"base": 500000.0, "dims": hd, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}},
           "scale": hd ** -0.5, "v_mix": True, "vdim": hd}
    ret = {"decay": [1.0 - 2.0 ** (-5 - h) for h in range(heads // 2)], "dim": hd, "heads": heads // 2,
           "rot": {"base": 10000.0, "dims": hd}, "vdim": 2 * hd}
    mlp = {"kind": "dense", "ff": 8 * width // 3 // 64 * 64}
    out = []
    for i in range(layers):
        kind = ("attention", "retention")[i % 2]
        out.append({"type": kind, "mixer": dict(att if kind == "attention" else ret), "mlp": dict(mlp)})
    return {"architecture": "Vatevik", "embedding": {"scale": 8.0}, "layers": out, "logit_scale": 0.25, "logit_softcap": 30.0,
            "norm": {"eps": 1e-6}, "vocab": 32000, "width": width}


def vatevik_workload(args, cb, torch) -> int:
    """Prefill (one 2,048-token prompt in one step) and decode (batch 8 from context 1,024, the captured step with
    argmax on the device) of the Vatevik design at two layer sizes, each beside Figotar (the closest model: norms on
    the parts' results, a matrix recurrence walked row by row, attention with a sink) and the GPT-2 style model of
    equal width and depth; then the design's own kernels alone, at the larger size, beside the like kernels of
    those models."""
    from cbis_b200.kernels import ops
    pk = peaks()
    P, T, B = 2048, 2048, args.batch or 8
    steps, warm = min(args.steps, 128), max(3, min(args.warmup, 8))
    layers = args.layers or 8
    gen = torch.Generator().manual_seed(0)
    sampler = ClockSampler()
    sampler.start()
    sizes = {}
    for width in (1024, 2048):
        gpt = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=layers, n_embd=width, n_head=16,
                   n_inner=4 * width, vocab_size=32000, n_positions=P, activation_function="gelu",
                   layer_norm_epsilon=1e-5, tie_word_embeddings=False)
        sizes[f"width_{width}"] = {name: measure_model(args, cb, torch, pk, cfgd, 32000, B, P, T, steps, warm, gen)
                                   for name, cfgd in (("vatevik", vatevik_sizes(width, layers)),
                                                      ("figotar", figotar_sizes(width, layers)), ("gpt2_style", gpt))}
    clocks = sampler.stop()
    line = {"metric": f"Vatevik prefill and decode tokens/s beside Figotar and the GPT-2 style model of equal width and "
                      f"depth ({layers} layers, batch {B}, prompt {T})", "unit": "tokens/s", "n_gpus": 1, "impl": "b200",
            "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids)", "higher_is_better": True,
            "value": sizes["width_2048"]["vatevik"]["decode_tokens_per_s"], "sizes": sizes,
            "kernels": vatevik_kernels(torch, ops, pk), "clocks": clocks, "peaks": pk}
    print(json.dumps(line))
    return 0


def divitar_sizes(width, layers):
    """A Divitar configuration with layers of the sizes a model of this width would have: of every four layers a latent
    attention that keeps its latents, an attention inside blocks of positions (grouped key/value heads), a latent
    attention that reads the first one's latents, and another block attention; dense and routed feed-forwards (with an
    expert for all) in turn; a second token table of 64 columns a layer."""
    big = width >= 2048
    hd = 128 if big else 64
    heads = width // hd
    att = {"dim": hd, "heads": heads, "kv_heads": max(1, heads // 4), "mask": {"size": 1024 if big else 512},
           "rot": {"base": 10000.0, "dims": hd, "scaling": {"factor": 4.0}}, "scale": hd ** -0.5, "vdim": hd}
    lat = {"dim": 64, "heads": 16, "kv_rank": 64, "mask": {"size": 1024 if big else 512}, "rot_dim": 64,
           "rot": {"base": 500000.0, "dims": 64, "scaling": {"factor": 4.0, "original": 4096, "fast": 16.0, "slow": 2.0}},
           "scale": 128 ** -0.5, "vdim": 64}
    dense = {"kind": "dense", "ff": 4 * width}
    moe = {"kind": "moe", "expert": {"ff": 11 * width // 16}, "router": {"experts": 16 if big else 8, "scale": 2.5, "top": 2},
           "shared": {"ff": 11 * width // 16}}
    out = []
    for i in range(layers):
        kind = ("latent_attention", "attention")[i % 2]
        mixer = dict(lat if kind == "latent_attention" else att)
        if i % 4 == 2:
            mixer["kv_from"] = i - 2
        out.append({"type": kind, "mixer": mixer, "mlp": dict(dense if i % 4 == 0 else moe)})
    return {"architecture": "Divitar", "layers": out, "logit_scale": 0.5, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
            "token_side": {"dim": 64}, "vocab": 32000, "width": width}


def divitar_workload(args, cb, torch) -> int:
    """Prefill (one 2,048-token prompt in one step) and decode (batch 8 from context 1,024, the captured step with
    argmax on the device) of the Divitar design at two layer sizes, each beside Figotar (the closest model in its
    mixers: gated attention over grouped heads, attention over a latent with a rotated key part and a sink), Vekedra
    (the closest in its feed-forwards: routed experts) and the GPT-2 style model of equal width and depth; then the
    design's own kernels alone, at the larger size, beside the like kernels of those models."""
    from cbis_b200.kernels import ops
    pk = peaks()
    P, T, B = 2048, 2048, args.batch or 8
    steps, warm = min(args.steps, 128), max(3, min(args.warmup, 8))
    layers = args.layers or 8
    gen = torch.Generator().manual_seed(0)
    sampler = ClockSampler()
    sampler.start()
    sizes = {}
    for width in (1024, 2048):
        gpt = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=layers, n_embd=width, n_head=16,
                   n_inner=4 * width, vocab_size=32000, n_positions=P, activation_function="gelu",
                   layer_norm_epsilon=1e-5, tie_word_embeddings=False)
        sizes[f"width_{width}"] = {name: measure_model(args, cb, torch, pk, cfgd, 32000, B, P, T, steps, warm, gen)
                                   for name, cfgd in (("divitar", divitar_sizes(width, layers)),
                                                      ("figotar", figotar_sizes(width, layers)),
                                                      ("vekedra", vekedra_sizes(width, layers)), ("gpt2_style", gpt))}
    clocks = sampler.stop()
    line = {"metric": f"Divitar prefill and decode tokens/s beside Figotar, Vekedra and the GPT-2 style model of equal "
                      f"width and depth ({layers} layers, batch {B}, prompt {T})", "unit": "tokens/s", "n_gpus": 1,
            "impl": "b200", "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids)",
            "higher_is_better": True, "value": sizes["width_2048"]["divitar"]["decode_tokens_per_s"], "sizes": sizes,
            "kernels": divitar_kernels(torch, ops, pk), "clocks": clocks, "peaks": pk}
    print(json.dumps(line))
    return 0


def divitar_kernels(torch, ops, pk):
    """Microseconds of the kernels the design added or changed, alone, at the layer sizes of width 2,048, with the bytes
    each has to move over its time as a fraction of the measured copy bandwidth (attention over prompts: its
    arithmetic as a fraction of the measured bf16 peak), each beside the like kernel of the closest model at equal
    sizes."""
    bf = torch.bfloat16
    out = {}
    timed = graph_timer(torch, pk, out)
    W, nh, nkv, hd = 2048, 16, 4, 128              # block attention of width 2,048
    lh, rank, rot = 16, 64, 64                     # latent attention: 16 heads over cached rows of 64 + 64
    E, top, side = 16, 2, 64
    freqs = (10000.0 ** (-2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)).float().cuda()
    for rows, segs, tag in ((2048, 1, "prefill_2048"), (8, 8, "decode_8")):
        per = rows // segs
        pos = (torch.arange(rows, dtype=torch.int32, device="cuda") % per) + (1024 if segs > 1 else 0)
        dq, dk = nh * hd, nkv * hd

        def rope_keep():        # q | k | gate -> q and k rotated, the keys once more as the values
            src = torch.randn(rows, dq + dk + nh, device="cuda").to(bf)
            dst = torch.empty(rows, dq + 2 * dk, dtype=bf, device="cuda")
            return lambda: ops.rope_rows(src, 0, hd, dst, 0, hd, pos, nh + nkv, hd, hd, freqs, keep_col0=dq + dk, keep_head0=nh)
        timed(rope_keep, rows * (2 * (dq + dk) + dk) * 2, f"rope_rows_keys_kept_as_values_{tag}")

        def rope_alone():
            buf = torch.randn(rows, dq + dk, device="cuda").to(bf)
            return lambda: ops.rope_rows(buf, 0, hd, buf, 0, hd, pos, nh + nkv, hd, hd, freqs)
        timed(rope_alone, rows * 2 * (dq + dk) * 2, f"closest_model_rope_rows_{tag}")

        def rope_neighbours():  # the rotated query parts of the latent attention, moved behind the latent-space queries
            q = torch.randn(rows, lh * (64 + rot), device="cuda").to(bf)
            qc = torch.empty(rows, lh * (rank + rot), dtype=bf, device="cuda")
            return lambda: ops.rope_rows(q, 64, 64 + rot, qc, rank, rank + rot, pos, lh, rot, rot, freqs, neighbours=True, length=1.14)
        timed(rope_neighbours, rows * 2 * lh * rot * 2, f"rope_rows_neighbours_{tag}")

        def rope_half():
            q = torch.randn(rows, lh * (64 + rot), device="cuda").to(bf)
            qc = torch.empty(rows, lh * (rank + rot), dtype=bf, device="cuda")
            return lambda: ops.rope_rows(q, 64, 64 + rot, qc, rank, rank + rot, pos, lh, rot, rot, freqs)
        timed(rope_half, rows * 2 * lh * rot * 2, f"closest_model_rope_rows_half_{tag}")

        def scaled_add():
            x, d = torch.randn(rows, W, device="cuda"), torch.randn(rows, W, device="cuda")
            w = torch.ones(W, device="cuda")
            o = torch.empty(rows, W, dtype=bf, device="cuda")
            return lambda: ops.add_rmsnorm(x, d, None, None, w, 1e-6, 0.0, o, delta_scale=0.5)
        timed(scaled_add, rows * W * (4 + 4 + 4 + 2), f"add_rmsnorm_scaled_{tag}")

        def side_add():         # the token input's result through its own norm, scaled, the rows handed on for the next norm
            x, d = torch.randn(rows, W, device="cuda"), torch.randn(rows, W, device="cuda")
            w, wp = torch.ones(W, device="cuda"), torch.ones(W, device="cuda")
            o = torch.empty(rows, W, dtype=bf, device="cuda")
            return lambda: ops.add_rmsnorm(x, d, None, (wp, 1e-6, 0.0), w, 1e-6, 0.0, o, delta_scale=0.5)
        timed(side_add, rows * W * (4 + 4 + 4 + 2), f"add_rmsnorm_scaled_with_the_result_normalised_{tag}")

        def sandwich():
            x, d = torch.randn(rows, W, device="cuda"), torch.randn(rows, W, device="cuda")
            w, wb = torch.zeros(W, device="cuda"), torch.zeros(W, device="cuda")
            o = torch.empty(rows, W, dtype=bf, device="cuda")
            return lambda: ops.add_rmsnorm(x, d, None, (wb, 1e-6, 1.0), w, 1e-6, 1.0, o)
        timed(sandwich, rows * W * (4 + 4 + 4 + 2), f"closest_model_add_rmsnorm_{tag}")

        def table_gate():
            a = torch.randn(rows, side, device="cuda").to(bf)
            table = torch.randn(32000, side, device="cuda").to(bf)
            tok = torch.randint(0, 32000, (rows,), device="cuda").int()
            return lambda: ops.gate_mul(a, table, "gelu_tanh", a, b_rows=tok)
        timed(table_gate, rows * side * 3 * 2, f"gate_mul_table_rows_{tag}")

        def plain_gate():
            a, b = torch.randn(rows, side, device="cuda").to(bf), torch.randn(rows, side, device="cuda").to(bf)
            return lambda: ops.gate_mul(a, b, "gelu_tanh", a)
        timed(plain_gate, rows * side * 3 * 2, f"closest_model_gate_mul_{tag}")

        def route(scale, eps):
            def make():
                h = torch.randn(rows, W, device="cuda").to(bf)
                r = torch.randn(E, W, device="cuda").to(bf)
                ids = torch.empty(rows, top, dtype=torch.int32, device="cuda")
                wt = torch.empty(rows, top, dtype=torch.float32, device="cuda")
                return lambda: ops.route_topk(h, r, top, "sigmoid", scale != 1.0, ids, wt, eps, scale)
            return make
        timed(route(2.5, 1e-20), rows * W * 2 + E * W * 2, f"route_topk_renormalised_scaled_{tag}")
        timed(route(1.0, 0.0), rows * W * 2 + E * W * 2, f"closest_model_route_topk_{tag}")

        def product(act):
            def make():
                x = torch.randn(rows, W, device="cuda").to(bf)
                w = (torch.randn(4 * W, W, device="cuda") * W ** -0.5).to(bf)
                return lambda: ops.linear(x, w, None, act)
            return make
        flops = 2.0 * rows * W * 4 * W
        timed(product("relu2"), (rows * W + 4 * W * W + rows * 4 * W) * 2, f"up_product_relu_squared_{tag}", flops=flops)
        timed(product("gelu_tanh"), (rows * W + 4 * W * W + rows * 4 * W) * 2, f"closest_model_up_product_gelu_{tag}", flops=flops)

    # attention of 16 query heads over 4 key/value heads of 128 inside blocks of 1,024 positions, beside the same
    # kernels with a sliding window of 1,024 and with every key; pages of 16
    ps, ctx_len, size = 16, 2048, 1024
    pages = ctx_len // ps
    bt1 = torch.arange(pages, dtype=torch.int32, device="cuda").view(1, pages)
    cu1 = torch.tensor([0, ctx_len], dtype=torch.int32, device="cuda")
    zero1 = torch.zeros(1, dtype=torch.int32, device="cuda")

    def seen(mask):
        def first(p):
            return max(0, p - mask + 1) if mask > 0 else (p - p % -mask if mask < 0 else 0)
        return sum(p - first(p) + 1 for p in range(ctx_len))
    for name, mask in (("attention_prefill_2048_blocks_of_1024", -size), ("closest_model_attention_prefill_2048_window_1024", size),
                       ("attention_prefill_2048_every_key", 0)):
        def prefill():
            q = torch.randn(ctx_len, nh * hd, device="cuda").to(bf)
            k, v = (torch.randn(pages, nkv, ps, hd, device="cuda").to(bf) for _ in range(2))
            o = torch.empty(ctx_len, nh * hd, dtype=bf, device="cuda")
            return lambda: ops.paged_prefill_tc5(q, k, v, bt1, cu1, zero1, o, 0, 1, ctx_len, nh, nkv, hd, ps, hd ** -0.5, mask)
        timed(prefill, ctx_len * (2 * nh + 2 * nkv) * hd * 2, name, flops=4.0 * seen(mask) * nh * hd)
    B = 8
    btB = torch.arange(B * pages, dtype=torch.int32, device="cuda").view(B, pages)
    row_seq = torch.arange(B, dtype=torch.int32, device="cuda")
    posB = torch.full((B,), ctx_len - 1, dtype=torch.int32, device="cuda")
    slot_map = (btB[:, -1] * ps + ps - 1).contiguous()
    for name, mask in (("attention_decode_8_blocks_of_1024", -size), ("closest_model_attention_decode_8_window_1024", size)):
        def decode():
            qkv = torch.randn(B, (nh + 2 * nkv) * hd, device="cuda").to(bf)
            k, v = (torch.randn(B * pages, nkv, ps, hd, device="cuda").to(bf) for _ in range(2))
            o = torch.empty(B, nh * hd, dtype=bf, device="cuda")
            ns = ops.decode_splits(B, nh, ctx_len)
            scratch = torch.empty(max(1, ops.decode_scratch_floats(B, nh, hd, ns)), device="cuda")
            counters = torch.zeros(B * nh, dtype=torch.int32, device="cuda")
            return lambda: ops.paged_decode_bf16(qkv, nh * hd, (nh + nkv) * hd, k, v, btB, row_seq, posB, slot_map, o, scratch,
                                                 counters, nh, nkv, hd, ps, hd ** -0.5, mask, ns)
        timed(decode, B * size * 2 * nkv * hd * 2, name)
    return out


def graph_timer(torch, pk, out):
    """``timed(make, nbytes, name, flops)``: microseconds of a kernel alone, replayed from a CUDA graph over buffers that
    rotate, with its bytes over its time as a fraction of the measured copy bandwidth."""
    def timed(make, nbytes, name, flops=0.0, reps=20, copies=4):
        fns = [make() for _ in range(copies)]
        for f in fns:
            f()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for f in fns:
                f()
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) / reps / copies * 1e3
        out[name] = {"us": round(us, 2), "bytes": int(nbytes), "frac_of_copy_bandwidth": round(nbytes / us / 1e3 / pk["hbm_gbs"], 4)}
        if flops:
            out[name]["frac_of_bf16_peak"] = round(flops / us / 1e6 / pk["bf16_tflops"], 4)
    return timed


def vatevik_kernels(torch, ops, pk):
    """Microseconds of the design's own kernels alone at the layer sizes of width 2,048, with the bytes each has to move
    over its time as a fraction of the measured copy bandwidth, each beside the like kernel of the closest model at
    equal sizes."""
    bf = torch.bfloat16
    out = {}
    timed = graph_timer(torch, pk, out)
    W, H, D, V = 2048, 8, 128, 256                 # retention of width 2,048: 8 heads of 128 x 256 (the closest model's memory too)
    nh, nkv, hd = 16, 4, 128                       # attention of that width
    freqs = (10000.0 ** (-2.0 * torch.arange(D // 2, dtype=torch.float64) / D)).float().cuda()
    for rows, segs, tag in ((2048, 1, "prefill_2048"), (8, 8, "decode_8")):
        per = rows // segs
        seg_slot = torch.arange(segs, dtype=torch.int32, device="cuda")
        cu = torch.arange(0, rows + 1, per, dtype=torch.int32, device="cuda")
        pos = (torch.arange(rows, dtype=torch.int32, device="cuda") % per) + (1024 if segs > 1 else 0)

        def retention():
            qkv = (torch.randn(rows, 2 * H * D + 2 * H * V, device="cuda") * 0.5).to(bf)
            om = torch.tensor([2.0 ** (-5 - h) for h in range(H)], device="cuda")
            st = torch.zeros(segs, H * D * V, device="cuda")
            y = torch.empty(rows, H * V, device="cuda")
            dp = ops.retention_piece_decays((1.0 - om.double()).tolist()).cuda()
            return lambda: ops.retention(qkv, 0, H * D, 2 * H * D, pos, freqs, D, D ** -0.5, om, st, seg_slot, cu, segs, H, D, V, y,
                                         max_seg_rows=per, piece_decays=dp, piece_rows=None if pieces else 0)
        for pieces in ((True, False) if segs == 1 else (True,)):        # as the engine calls it; the long segment walked in one piece
            timed(retention, rows * ((2 * H * D + H * V) * 2 + H * V * 4) + 2 * segs * H * D * V * 4,
                  f"retention_{tag}" if pieces else f"retention_in_one_piece_{tag}")

        def memory():
            qkv = (torch.randn(rows, 2 * H * D + 2 * H * V, device="cuda") * 0.5).to(bf)
            gates = torch.randn(rows, 2 * H, device="cuda")
            ib, fb = torch.zeros(H, device="cuda"), torch.full((H,), 3.0, device="cuda")
            st = torch.zeros(segs, ops.matrix_memory_state_floats(H, D, V), device="cuda")
            y = torch.empty(rows, H * V, device="cuda")
            return lambda: ops.matrix_memory(qkv, 0, H * D, 2 * H * D, gates, ib, fb, 15.0, D ** -0.5, 1e-6, st, seg_slot, cu,
                                             segs, H, D, V, y, max_seg_rows=per)
        timed(memory, rows * ((2 * H * D + H * V) * 2 + H * V * 4) + 2 * segs * H * D * V * 4, f"closest_model_matrix_memory_{tag}")

        def result_norm():
            x, d = torch.randn(rows, W, device="cuda"), torch.randn(rows, W, device="cuda")
            wb = torch.ones(W, device="cuda")
            o = torch.empty(rows, W, dtype=bf, device="cuda")
            return lambda: ops.add_rmsnorm(x, d, None, (wb, 1e-6, 0.0), None, 0.0, 0.0, o)
        timed(result_norm, rows * W * (4 + 4 + 4 + 2), f"add_rmsnorm_no_norm_before_{tag}")

        def sandwich():
            x, d = torch.randn(rows, W, device="cuda"), torch.randn(rows, W, device="cuda")
            w, wb = torch.zeros(W, device="cuda"), torch.zeros(W, device="cuda")
            o = torch.empty(rows, W, dtype=bf, device="cuda")
            return lambda: ops.add_rmsnorm(x, d, None, (wb, 1e-6, 1.0), w, 1e-6, 1.0, o)
        timed(sandwich, rows * W * (4 + 4 + 4 + 2), f"closest_model_add_rmsnorm_{tag}")

        dq, dk = nh * hd, nkv * hd

        def prepare():
            buf = torch.randn(rows, dq + 2 * dk, device="cuda").to(bf)
            other = torch.randn(rows, dk, device="cuda").to(bf)
            qw, kw = torch.ones(dq, device="cuda"), torch.ones(dk, device="cuda")
            return lambda: ops.qk_prepare(buf, 0, nh, dq, nkv, hd, qw, kw, 1e-6, pos, freqs, hd, dq + dk, dk, other, 0.5)
        timed(prepare, rows * (2 * (dq + 2 * dk) + dk) * 2, f"qk_prepare_{tag}")

        def prepare_in_steps():
            buf = torch.randn(rows, dq + 2 * dk, device="cuda").to(bf)
            other = torch.randn(rows, dk, device="cuda").to(bf)
            qw, kw = torch.ones(dq, device="cuda"), torch.ones(dk, device="cuda")
            q, k, v = buf[:, :dq], buf[:, dq:dq + dk], buf[:, dq + dk:]

            def run():
                ops.rms_norm(q, qw, 1e-6, q)
                ops.rms_norm(k, kw, 1e-6, k)
                ops.rope_rows(buf, 0, hd, buf, 0, hd, pos, nh, hd, hd, freqs)
                ops.rope_rows(buf, dq, hd, buf, dq, hd, pos, nkv, hd, hd, freqs)
                ops.blend_rows(v, other, 0.5, v)
            return run
        timed(prepare_in_steps, rows * (2 * (dq + 2 * dk) + dk) * 2, f"the_same_in_five_kernels_{tag}")

        def rope_alone():       # the closest model's rotation: one array of rotated key parts
            buf = torch.randn(rows, dq + dk, device="cuda").to(bf)
            return lambda: ops.rope_rows(buf, 0, hd, buf, 0, hd, pos, nh + nkv, hd, hd, freqs)
        timed(rope_alone, rows * 2 * (dq + dk) * 2, f"closest_model_rope_rows_{tag}")

        def gated_norm():
            y = torch.randn(rows, H * V, device="cuda")
            z = torch.randn(rows, H * V, device="cuda").to(bf)
            o = torch.empty(rows, H * V, dtype=bf, device="cuda")
            return lambda: ops.rms_norm(y, None, 1e-6, o, parts=H, gate=z, gate_act="silu", gate_after=True)
        timed(gated_norm, rows * H * V * (4 + 2 + 2), f"head_norm_with_gate_{tag}")

    # attention: 16 query heads over 4 key/value heads of 128, all keys, pages of 16, 1 in the denominator
    ps, ctx_len = 16, 2048
    pages = ctx_len // ps
    bt1 = torch.arange(pages, dtype=torch.int32, device="cuda").view(1, pages)
    cu1 = torch.tensor([0, ctx_len], dtype=torch.int32, device="cuda")
    zero1 = torch.zeros(1, dtype=torch.int32, device="cuda")
    sinks = torch.zeros(nh, device="cuda")
    keys = ctx_len * (ctx_len + 1) // 2
    for name, extra in (("attention_prefill_2048_sink", dict(v_head_dim=hd, sinks=sinks)),
                        ("closest_model_attention_prefill_2048_same_kernel_plain", {})):
        def prefill():
            q = torch.randn(ctx_len, nh * hd, device="cuda").to(bf)
            k, v = (torch.randn(pages, nkv, ps, hd, device="cuda").to(bf) for _ in range(2))
            o = torch.empty(ctx_len, nh * hd, dtype=bf, device="cuda")
            return lambda: ops.paged_prefill_bf16(q, k, v, bt1, cu1, zero1, o, 0, 1, ctx_len, nh, nkv, hd, ps, hd ** -0.5, 0, **extra)
        timed(prefill, ctx_len * (2 * nh + 2 * nkv) * hd * 2, name, flops=4.0 * keys * nh * hd)
    B = 8
    btB = torch.arange(B * pages, dtype=torch.int32, device="cuda").view(B, pages)
    row_seq = torch.arange(B, dtype=torch.int32, device="cuda")
    posB = torch.full((B,), ctx_len - 1, dtype=torch.int32, device="cuda")
    slot_map = (btB[:, -1] * ps + ps - 1).contiguous()
    for name, extra in (("attention_decode_8_sink", dict(v_head_dim=hd, sinks=sinks)),
                        ("closest_model_attention_decode_8_tensor_core_form_plain", {})):
        def decode():
            qkv = torch.randn(B, (nh + 2 * nkv) * hd, device="cuda").to(bf)
            k, v = (torch.randn(B * pages, nkv, ps, hd, device="cuda").to(bf) for _ in range(2))
            o = torch.empty(B, nh * hd, dtype=bf, device="cuda")
            ns = ops.decode_splits(B, nh, ctx_len)
            scratch = torch.empty(max(1, ops.decode_scratch_floats(B, nh, hd, ns)), device="cuda")
            counters = torch.zeros(B * nh, dtype=torch.int32, device="cuda")
            return lambda: ops.paged_decode_bf16(qkv, nh * hd, (nh + nkv) * hd, k, v, btB, row_seq, posB, slot_map, o, scratch,
                                                 counters, nh, nkv, hd, ps, hd ** -0.5, 0, ns, **extra)
        timed(decode, B * ctx_len * 2 * nkv * hd * 2, name)
    return out


def figotar_sizes(width, layers):
    """A Figotar configuration with layers of the sizes a model of this width would have: of every four layers one
    windowed attention (grouped key/value heads, values as wide as keys), one attention over a cached latent with a
    rotated key part, and two matrix memories; every layer with a gated feed-forward."""
    big = width >= 2048
    hd = 128 if big else 64
    heads = width // hd
    att = {"dim": hd, "heads": heads, "kv_heads": max(1, heads // 4), "mask": {"size": 1024 if big else 512},
           "q_temp": {"coef": 0.1, "every": 512}, "scale": hd ** -0.5, "vdim": hd}
    lat = {"dim": 64, "heads": 16, "kv_rank": 64, "q_rank": width // 4, "rot": {"base": 10000.0, "dims": 64},
           "rot_dim": 64, "scale": 128 ** -0.5, "vdim": 64}
    mem = {"dim": hd, "gate_cap": 15.0, "heads": heads // 2, "vdim": 2 * hd}
    mlp = {"kind": "dense", "ff": 8 * width // 3 // 64 * 64}
    out = []
    for i in range(layers):
        kind = ("attention", "mlstm", "latent_attention", "mlstm")[i % 4]
        out.append({"type": kind, "mixer": dict({"attention": att, "latent_attention": lat, "mlstm": mem}[kind]), "mlp": dict(mlp)})
    return {"architecture": "Figotar", "layers": out, "norm": {"eps": 1e-6}, "vocab": 32000, "width": width}


def figotar_workload(args, cb, torch) -> int:
    """Prefill (one 2,048-token prompt in one step) and decode (batch 8 from context 1,024, the captured step with
    argmax on the device) of the Figotar design at two layer sizes, each beside Vekedra (the closest model: unlike
    layers, a recurrent state, attention over a latent) and the GPT-2 style model of equal width and depth; then the
    design's own kernels alone, at the larger size, beside the like kernels of those models."""
    from cbis_b200.kernels import ops
    pk = peaks()
    P, T, B = 2048, 2048, args.batch or 8
    steps, warm = min(args.steps, 128), max(3, min(args.warmup, 8))
    layers = args.layers or 8
    gen = torch.Generator().manual_seed(0)
    sampler = ClockSampler()
    sampler.start()
    sizes = {}
    for width in (1024, 2048):
        gpt = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=layers, n_embd=width, n_head=16,
                   n_inner=4 * width, vocab_size=32000, n_positions=P, activation_function="gelu",
                   layer_norm_epsilon=1e-5, tie_word_embeddings=False)
        sizes[f"width_{width}"] = {name: measure_model(args, cb, torch, pk, cfgd, 32000, B, P, T, steps, warm, gen)
                                   for name, cfgd in (("figotar", figotar_sizes(width, layers)),
                                                      ("vekedra", vekedra_sizes(width, layers)), ("gpt2_style", gpt))}
    clocks = sampler.stop()
    line = {"metric": f"Figotar prefill and decode tokens/s beside Vekedra and the GPT-2 style model of equal width and "
                      f"depth ({layers} layers, batch {B}, prompt {T})", "unit": "tokens/s", "n_gpus": 1, "impl": "b200",
            "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids)", "higher_is_better": True,
            "value": sizes["width_2048"]["figotar"]["decode_tokens_per_s"], "sizes": sizes,
            "kernels": figotar_kernels(torch, ops, pk), "clocks": clocks, "peaks": pk}
    print(json.dumps(line))
    return 0


def figotar_kernels(torch, ops, pk):
    """Microseconds of the design's own kernels alone (each replayed from a CUDA graph over buffers that rotate) at the
    layer sizes of width 2,048, with the bytes each has to move over its time as a fraction of the measured copy
    bandwidth (attention over prompts: its arithmetic as a fraction of the measured bf16 peak), each beside the like
    kernel of the closest model at equal sizes."""
    bf = torch.bfloat16
    out = {}

    def timed(make, nbytes, name, flops=0.0, reps=20, copies=4):
        fns = [make() for _ in range(copies)]
        for f in fns:
            f()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for f in fns:
                f()
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) / reps / copies * 1e3
        out[name] = {"us": round(us, 2), "bytes": int(nbytes), "frac_of_copy_bandwidth": round(nbytes / us / 1e3 / pk["hbm_gbs"], 4)}
        if flops:
            out[name]["frac_of_bf16_peak"] = round(flops / us / 1e6 / pk["bf16_tflops"], 4)

    W, H, D, V = 2048, 8, 128, 256                 # the matrix memory of width 2,048: 8 heads of 128 x 256
    sH, sP, sN, sG = 64, 64, 128, 8                # the state-space layer of that width: 64 heads of 64 x 128
    for rows, segs, tag in ((2048, 1, "prefill_2048"), (8, 8, "decode_8")):
        per = rows // segs
        seg_slot = torch.arange(segs, dtype=torch.int32, device="cuda")
        cu = torch.arange(0, rows + 1, per, dtype=torch.int32, device="cuda")

        def memory():
            qkv = (torch.randn(rows, 2 * H * D + 2 * H * V, device="cuda") * 0.5).to(bf)
            gates = torch.randn(rows, 2 * H, device="cuda")
            ib, fb = torch.zeros(H, device="cuda"), torch.full((H,), 3.0, device="cuda")
            st = torch.zeros(segs, ops.matrix_memory_state_floats(H, D, V), device="cuda")
            y = torch.empty(rows, H * V, device="cuda")
            return lambda: ops.matrix_memory(qkv, 0, H * D, 2 * H * D, gates, ib, fb, 15.0, D ** -0.5, 1e-6, st, seg_slot, cu,
                                             segs, H, D, V, y, max_seg_rows=per)
        timed(memory, rows * ((2 * H * D + H * V) * 2 + H * V * 4) + 2 * segs * H * D * V * 4, f"matrix_memory_{tag}")

        def scan():
            inner, C = sH * sP, sH * sP + 2 * sG * sN
            xbc = (torch.randn(rows, C, device="cuda") * 0.5).to(bf)
            proj = torch.randn(rows, 2 * inner + 2 * sG * sN + sH, device="cuda").to(bf)
            v = [torch.zeros(sH, device="cuda") for _ in range(3)]
            st = torch.zeros(segs, inner * sN, device="cuda")
            y = torch.empty(rows, inner, device="cuda")
            return lambda: ops.ssm_scan(xbc, proj, proj.shape[1] - sH, v[0], v[1], v[2], st, seg_slot, cu, segs, sH, sP, sN, sG, y)
        timed(scan, rows * ((sH * sP + 2 * sG * sN) * 2 + sH * sP * 4) + 2 * segs * sH * sP * sN * 4, f"closest_model_ssm_scan_{tag}")

        def sandwich():
            x, d = torch.randn(rows, W, device="cuda"), torch.randn(rows, W, device="cuda")
            w, wb = torch.zeros(W, device="cuda"), torch.zeros(W, device="cuda")
            o = torch.empty(rows, W, dtype=bf, device="cuda")
            return lambda: ops.add_rmsnorm(x, d, None, (wb, 1e-6, 1.0), w, 1e-6, 1.0, o)
        timed(sandwich, rows * W * (4 + 4 + 4 + 2), f"add_rmsnorm_{tag}")

        def lnorm():
            x, d = torch.randn(rows, W, device="cuda"), torch.randn(rows, W, device="cuda")
            w, b = torch.ones(W, device="cuda"), torch.zeros(W, device="cuda")
            o = torch.empty(rows, W, dtype=bf, device="cuda")
            return lambda: ops.add_layernorm(x, d, None, w, b, 1e-5, o)
        timed(lnorm, rows * W * (4 + 4 + 4 + 2), f"closest_model_add_layernorm_{tag}")

        def gated_norm():
            y = torch.randn(rows, H * V, device="cuda")
            z = torch.randn(rows, H * V, device="cuda").to(bf)
            w = torch.ones(H * V, device="cuda")
            o = torch.empty(rows, H * V, dtype=bf, device="cuda")
            return lambda: ops.rms_norm(y, w, 1e-6, o, parts=H, gate=z, gate_act="sigmoid", gate_after=True)
        timed(gated_norm, rows * H * V * (4 + 2 + 2), f"head_norm_with_gate_{tag}")

    # attention: 16 query heads over 4 key/value heads of 128, a window of 1,024, pages of 16
    nh, nkv, hd, ps, ctx_len = 16, 4, 128, 16, 2048
    pages = ctx_len // ps
    bt1 = torch.arange(pages, dtype=torch.int32, device="cuda").view(1, pages)
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / nh) for h in range(nh)], device="cuda")
    cu1 = torch.tensor([0, ctx_len], dtype=torch.int32, device="cuda")
    zero1 = torch.zeros(1, dtype=torch.int32, device="cuda")
    keys = sum(min(i + 1, 1024) for i in range(ctx_len))
    for name, extra in (("attention_prefill_2048_bias_temperature", dict(v_head_dim=hd, slopes=slopes, q_temp=(0.1, 512))),
                        ("closest_model_attention_prefill_2048_same_kernel_plain", {})):
        def prefill():
            q = torch.randn(ctx_len, nh * hd, device="cuda").to(bf)
            k, v = (torch.randn(pages, nkv, ps, hd, device="cuda").to(bf) for _ in range(2))
            o = torch.empty(ctx_len, nh * hd, dtype=bf, device="cuda")
            return lambda: ops.paged_prefill_bf16(q, k, v, bt1, cu1, zero1, o, 0, 1, ctx_len, nh, nkv, hd, ps, hd ** -0.5, 1024, **extra)
        timed(prefill, ctx_len * (2 * nh + 2 * nkv) * hd * 2, name, flops=4.0 * keys * nh * hd)
    B = 8
    btB = torch.arange(B * pages, dtype=torch.int32, device="cuda").view(B, pages)
    row_seq = torch.arange(B, dtype=torch.int32, device="cuda")
    pos = torch.full((B,), ctx_len - 1, dtype=torch.int32, device="cuda")
    slot_map = (btB[:, -1] * ps + ps - 1).contiguous()

    def decode_general():
        q = torch.randn(B, nh * hd, device="cuda").to(bf)
        k, v = (torch.randn(B * pages, nkv, ps, hd, device="cuda").to(bf) for _ in range(2))
        o = torch.empty(B, nh * hd, dtype=bf, device="cuda")
        chunks = ops.generic_key_chunks(B, nh, ctx_len, hd)
        part = torch.empty(B * nh * max(1, chunks[0]) * (hd + 4), device="cuda")
        return lambda: ops.paged_attention_generic(q, k, v, btB, row_seq, pos, o, nh, nkv, hd, ps, hd ** -0.5, 1024, chunks, part,
                                                   v_head_dim=hd, slopes=slopes, q_temp=(0.1, 512))
    timed(decode_general, B * 1024 * 2 * nkv * hd * 2, "attention_decode_8_bias_temperature_general_kernel")

    def decode_lanes():          # what the engine runs: the decode kernel's lane-group form, keys split over blocks
        qkv = torch.randn(B, (nh + 2 * nkv) * hd, device="cuda").to(bf)
        k, v = (torch.randn(B * pages, nkv, ps, hd, device="cuda").to(bf) for _ in range(2))
        o = torch.empty(B, nh * hd, dtype=bf, device="cuda")
        ns = ops.decode_splits(B, nh, ctx_len)
        scratch = torch.empty(max(1, ops.decode_scratch_floats(B, nh, hd, ns)), device="cuda")
        counters = torch.zeros(B * nh, dtype=torch.int32, device="cuda")
        return lambda: ops.paged_decode_bf16(qkv, nh * hd, (nh + nkv) * hd, k, v, btB, row_seq, pos, slot_map, o, scratch, counters,
                                             nh, nkv, hd, ps, hd ** -0.5, 1024, ns, v_head_dim=hd, slopes=slopes, q_temp=(0.1, 512))
    timed(decode_lanes, B * 1024 * 2 * nkv * hd * 2, "attention_decode_8_bias_temperature")

    def decode_plain():
        qkv = torch.randn(B, (nh + 2 * nkv) * hd, device="cuda").to(bf)
        k, v = (torch.randn(B * pages, nkv, ps, hd, device="cuda").to(bf) for _ in range(2))
        o = torch.empty(B, nh * hd, dtype=bf, device="cuda")
        ns = ops.decode_splits(B, nh, ctx_len)
        scratch = torch.empty(max(1, ops.decode_scratch_floats(B, nh, hd, ns)), device="cuda")
        counters = torch.zeros(B * nh, dtype=torch.int32, device="cuda")
        return lambda: ops.paged_decode_bf16(qkv, nh * hd, (nh + nkv) * hd, k, v, btB, row_seq, pos, slot_map, o, scratch, counters,
                                             nh, nkv, hd, ps, hd ** -0.5, 1024, ns)
    timed(decode_plain, B * 1024 * 2 * nkv * hd * 2, "closest_model_attention_decode_8")
    return out


def all_decoding(eng, batch):
    """True once every request of the batch has had its prompt run (each step then feeds one token each)."""
    return eng.scheduler.num_running() == batch and eng.last_step_tokens == batch


if __name__ == "__main__":
    sys.exit(main())
