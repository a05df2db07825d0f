#!/usr/bin/env python3
"""Decode and prefill throughput of the family's three benchmark shapes with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--shape smollm2-1.7b|llama3.2-1b|llama3.1-8b] [--dtype bfloat16|float32]
                    [--batch B] [--context C] [--prompts uniform:LO-HI] [--layers L]

A step is one decode step of a batch of 8 sequences; the K timed steps end at the benchmark
context length (prompts of context - W - K tokens are prefilled first). `value` is decoded tokens
per second, timed on the device with the sampled ids fed to the next step on the device; `e2e` is
the same through the Python entry point (`llm.generate`) with host token ids in and out every
step; `prefill` is one 2,048-token prompt; `roofline` relates the bytes a decode step has to read
(every weight once, the cache of the live requests) to the measured copy bandwidth; `points` holds
decoding at batch 1 and 64. The default run adds `f32`, the same measurements on the true 32-bit
path (its prompt step against a float fused-multiply-add rate measured here), and `shapes`: the
Llama-3.2-1B sizes on a batch of unequal prompts (lengths uniform in 128..2048, seeded; one packed
prompt step, then decoding) and the Llama-3.1-8B sizes at batch 1, 8 and 64. One JSON line on stdout.
`--kernel attn_decode|gemm_small_m` times one decode kernel alone instead (a line per case).

Weights are drawn on the device (`random:<config.json>:seed`), nothing is written but a config.json.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# the benchmark's primary configuration: the SmolLM2-1.7B layer sizes
SHAPE = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 24, "hidden_size": 2048,
    "num_attention_heads": 32, "num_key_value_heads": 32, "head_dim": 64, "intermediate_size": 8192,
    "vocab_size": 49152, "rope_theta": 130000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
    "max_position_embeddings": 8192, "hidden_act": "silu",
}
# further sizes of the family (Llama-3.2-1B and Llama-3.1-8B layer sizes); the default run's headline uses SHAPE
OTHER_SHAPES = {
    "llama3.2-1b": dict(SHAPE, num_hidden_layers=16, num_key_value_heads=8, vocab_size=128256, rope_theta=500000.0,
                        rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                      "original_max_position_embeddings": 8192}),
    "llama3.1-8b": dict(SHAPE, num_hidden_layers=32, hidden_size=4096, num_key_value_heads=8, head_dim=128,
                        intermediate_size=14336, vocab_size=128256, rope_theta=500000.0, tie_word_embeddings=False,
                        rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                      "original_max_position_embeddings": 8192}),
}
CONTEXT = 4096
PREFILL_TOKENS = 2048
UNEQUAL = "uniform:128-2048"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
WIDTH = {"bfloat16": 2, "float32": 4}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            raw = json.load(open(path))
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]), "source": "measured"}
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def mark(self):
        return len(self.rows)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, lo=0, hi=None):
        rows = [r for r in self.rows[lo:hi] if len(r) == 6 and r[0].isdigit()]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": statistics.median(int(r[0]) for r in rows), "sm_max_mhz": int(rows[0][1]), "reasons": reasons,
                "samples": len(rows)}


def model_numbers(cfg, n_layers):
    d, H, G, hd, F, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                         cfg["intermediate_size"], cfg["vocab_size"])
    per_layer = d * (H + 2 * G) * hd + H * hd * d + 3 * d * F          # matrix weights of one layer
    head = V * d
    norms = (2 * n_layers + 1) * d
    return {"layer_params": per_layer, "head_params": head, "norm_params": norms}


def decode_bytes(eng, contexts, width):
    """Bytes one decode step must read at `width` bytes an element, as the engine's own parts and
    cache state them: every weight a step uses once (the output head once, tied or not; of the
    embedding only rows), and the cached keys and values of every live sequence."""
    weights = eng.model.elements_read_per_step()
    kv_per_token = sum(2 * len(g.units) * g.need.kv_heads * g.need.head_dim for g in eng.cache.groups)
    return width * (weights + kv_per_token * sum(contexts))


def prefill_flops(cfg, n_layers, lengths, logit_rows=None):
    """Products of a prompt step over sequences of `lengths` tokens: 2 per weight and token, the head
    on `logit_rows` rows (default one per sequence), and causal attention (Q K^T and P V, half the
    square each) within each sequence."""
    nums = model_numbers(cfg, n_layers)
    T = sum(lengths)
    rows = len(lengths) if logit_rows is None else logit_rows
    linear = 2 * T * nums["layer_params"] * n_layers + 2 * rows * nums["head_params"]
    attn = sum(2 * n * n * cfg["num_attention_heads"] * cfg["head_dim"] * n_layers for n in lengths)
    return linear + attn


def flush_l2(buf):
    buf.add_(1)       # 512 MB read + written: more than the 126 MB L2


def parse_prompts(text):
    """'uniform:LO-HI' -> (LO, HI)."""
    kind, _, rng = text.partition(":")
    lo, _, hi = rng.partition("-")
    if kind != "uniform" or not lo.isdigit() or not hi.isdigit() or int(lo) < 1 or int(hi) < int(lo):
        raise SystemExit(f"--prompts {text!r}: expected uniform:LO-HI with 1 <= LO <= HI")
    return int(lo), int(hi)


class Bench:
    def __init__(self, args, pk, tmp):
        import numpy as np
        import torch
        from scriptling_llm_lib_b200 import llm
        from scriptling_llm_lib_b200.csrc import bindings
        self.np, self.torch, self.llm, self.bindings = np, torch, llm, bindings
        self.args, self.pk, self.tmp = args, pk, tmp
        self.l2 = None
        self._fma = None

    # ------------------------------------------------------------------ models
    def config(self, shape_name, layers=None):
        shape = SHAPE if shape_name == "smollm2-1.7b" else OTHER_SHAPES[shape_name]
        n_layers = layers or shape["num_hidden_layers"]
        raw = dict(shape, num_hidden_layers=n_layers,
                   max_position_embeddings=max(shape["max_position_embeddings"], self.args.context + 64,
                                               self.args.prefill_tokens))
        path = os.path.join(self.tmp, f"{shape_name}-{n_layers}.json")
        if not os.path.isfile(path):
            with open(path, "w") as f:
                json.dump(raw, f)
        return raw, n_layers, f"random:{path}:0"

    def load(self, spec, dtype, max_tokens, max_seqs):
        import gc
        self.llm.unload()
        self.l2 = None
        gc.collect()                 # an engine and its captured steps refer to each other
        self.torch.cuda.empty_cache()
        eng, sampler = self.llm.load(spec, dtype, "cuda:0", max_tokens=max_tokens, max_seqs=max_seqs)
        self.l2 = self.torch.zeros(128 * 1024 * 1024, dtype=self.torch.float32, device="cuda:0")
        return eng, sampler

    def fma_peak(self):
        if self._fma is None:
            self._fma = self.bindings.ProbeKernels().fma_tflops()
        return self._fma

    # ------------------------------------------------------------------ prompt steps
    def time_prompt_step(self, eng, lengths, seed, repeats=5, warm=3):
        """Median device time of one packed prompt step over sequences of `lengths` tokens, L2 flushed
        between runs; the logits of each sequence's last place are computed."""
        from scriptling_llm_lib_b200.engine.step import StepEntry
        torch = self.torch
        rng = self.np.random.default_rng(seed)
        V = eng.layout.vocab_size
        times = []
        for i in range(warm + repeats):
            flush_l2(self.l2)
            seqs = [eng.open() for _ in lengths]
            ids = [rng.integers(0, V, n).tolist() for n in lengths]
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            eng.step([StepEntry(s, t) for s, t in zip(seqs, ids)])
            e1.record()
            torch.cuda.synchronize()
            for s in seqs:
                s.close()
            if i >= warm:
                times.append(e0.elapsed_time(e1))
        return statistics.median(times)

    def prefill_record(self, eng, cfg, n_layers, lengths, dtype, seed=1):
        ms = self.time_prompt_step(eng, lengths, seed)
        flops = prefill_flops(cfg, n_layers, lengths)
        T = sum(lengths)
        if dtype == "bfloat16":
            peak, name = self.pk["bf16_tflops"], f"bf16 tensor ({self.pk['source']})"
        else:
            peak, name = self.fma_peak(), "float FMA (measured here)"
        return {"value": round(T / ms * 1e3, 1), "tokens": T, "ms": round(ms, 3),
                "frac": round(flops / (ms * 1e-3) / (peak * 1e12), 4), "tflops": round(flops / (ms * 1e-3) / 1e12, 1),
                "peak_tflops": round(peak, 1), "peak": name}

    # ------------------------------------------------------------------ decode steps
    def time_decode(self, eng, sampler, prompt_lens, steps, warmup, seed):
        """Prefill one prompt per entry of `prompt_lens`, then warmup + steps decode steps with the
        sampled ids fed back on the device; returns (ms per step, mean keys read per sequence and
        timed step, launches per step)."""
        from scriptling_llm_lib_b200.engine.step import StepEntry
        from scriptling_llm_lib_b200.sampling.sampler import SamplingOptions
        torch, np = self.torch, self.np
        V = eng.layout.vocab_size
        batch = len(prompt_lens)
        rng = np.random.default_rng(seed)
        seqs = [eng.open() for _ in range(batch)]
        greedy = SamplingOptions()
        try:
            # prompts go in a few sequences at a time to bound the activations of one step
            last, i = [], 0
            while i < batch:
                j, tok = i, 0
                while j < batch and (j == i or tok + prompt_lens[j] <= 16384):
                    tok += prompt_lens[j]
                    j += 1
                logits = eng.step([StepEntry(s, rng.integers(0, V, n).tolist()) for s, n in zip(seqs[i:j], prompt_lens[i:j])])
                last.extend(sampler.sample(logits, greedy, [0] * (j - i), [0] * (j - i)).tolist())
                i = j
            ids_dev = torch.tensor(last, dtype=torch.int32, device=eng.device)

            def one():
                nonlocal ids_dev
                logits = eng.decode_step_device(seqs, ids_dev)
                ids_dev = sampler.sample(logits, greedy, [0] * batch, [0] * batch)
            for _ in range(warmup):
                one()
            torch.cuda.synchronize()
            l0 = self.bindings.LAUNCHES[0]
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                one()
            e1.record()
            torch.cuda.synchronize()
            eng.check_errors()
            ms = e0.elapsed_time(e1) / steps
            launches = (self.bindings.LAUNCHES[0] - l0) / steps
            # the first timed step reads prompt + warmup + 1 keys of each sequence, each later step one more
            contexts = [n + warmup + 1 + (steps - 1) / 2 for n in prompt_lens]
            return ms, contexts, launches
        finally:
            for s in seqs:
                s.close()

    def decode_record(self, eng, sampler, cfg, n_layers, prompt_lens, steps, warmup, seed, dtype):
        ms, contexts, launches = self.time_decode(eng, sampler, prompt_lens, steps, warmup, seed)
        achieved = decode_bytes(eng, contexts, WIDTH[dtype]) / (ms * 1e-3) / 1e9
        return {"value": round(len(prompt_lens) / ms * 1e3, 1), "ms": round(ms, 4), "gbs": round(achieved, 1),
                "frac": round(achieved / self.pk["hbm_gbs"], 4)}, launches

    def equal_prompts(self, batch, steps, warmup):
        return [self.args.context - steps - warmup] * batch


def run(args):
    import numpy as np
    import torch
    pk = peaks()
    tmp = tempfile.mkdtemp(prefix="sllm_bench_")
    clocks = ClockSampler()
    b = Bench(args, pk, tmp)
    llm = b.llm
    dtype = args.dtype
    line = None
    try:
        cfg, n_layers, spec = b.config(args.shape, args.layers)
        full_layers = (SHAPE if args.shape == "smollm2-1.7b" else OTHER_SHAPES[args.shape])["num_hidden_layers"]
        want_points = not args.no_points and args.only == "all" and args.prompts is None
        # the batch-64 point needs 64 contexts of cache: at long contexts that is more than the GPU has
        kv_token = 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * n_layers * WIDTH[dtype]
        weights = WIDTH[dtype] * (model_numbers(cfg, n_layers)["layer_params"] * n_layers + 2 * model_numbers(cfg, n_layers)["head_params"])
        free = torch.cuda.mem_get_info()[0]
        point_batches = [bb for bb in (1, 64) if weights + bb * args.context * kv_token < 0.85 * free] if want_points else []
        biggest = max(point_batches + [args.batch])
        eng, sampler = b.load(spec, dtype, max(biggest * args.context, args.prefill_tokens + 64), biggest)
        V = cfg["vocab_size"]

        # ---- the prompt step: 2,048 tokens, or a batch of unequal prompts in one packed step
        if args.prompts is not None:
            lo, hi = parse_prompts(args.prompts)
            lengths = np.random.default_rng(7).integers(lo, hi + 1, args.batch).tolist()
        else:
            lengths = [args.prefill_tokens]
        prefill = b.prefill_record(eng, cfg, n_layers, lengths, dtype) if args.only != "decode" else None
        if args.prompts is not None and prefill is not None:
            prefill["prompts"] = {"dist": args.prompts, "seed": 7, "n": len(lengths), "min": min(lengths), "max": max(lengths)}
        if args.only == "prefill":
            print(json.dumps({"only": "prefill", "shape": args.shape, "dtype": dtype, "layers_run": n_layers, "prefill": prefill}))
            return 0

        # ---- the decode step at the headline batch, clocks sampled meanwhile
        clocks.start()
        time.sleep(0.5)
        c0 = clocks.mark()
        prompt_lens = lengths if args.prompts is not None else b.equal_prompts(args.batch, args.steps, args.warmup)
        head, launches = b.decode_record(eng, sampler, cfg, n_layers, prompt_lens, args.steps, args.warmup, 2, dtype)
        c1 = clocks.mark()
        ms, value = head["ms"], head["value"]
        roofline = {"bound": "hbm", "achieved": head["gbs"], "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": head["frac"],
                    "peaks": pk["source"]}
        if args.only == "decode":
            print(json.dumps({"only": "decode", "shape": args.shape, "dtype": dtype, "layers_run": n_layers, "batch": args.batch,
                              "ms_per_step": ms, "value": value, "roofline": roofline}))
            return 0

        # ---- end to end through the Python entry point: host ids in, host ids out, every step
        e2e = None
        if not args.no_e2e:
            rng = np.random.default_rng(1)
            n_gen = args.steps + args.warmup + 2          # the prompt's token, warm-up + 1 untimed decode steps, the timed ones
            e2e_lens = prompt_lens if args.prompts is not None else [args.context - n_gen] * args.batch
            prompts = [rng.integers(0, V, n).tolist() for n in e2e_lens]
            marks = {}

            def on_step(i, toks):
                # called when token i of every sequence has reached the host; the loop has already queued
                # decode step i + 1 by then, and the synchronize lets it finish before the clock starts
                if i == args.warmup:
                    torch.cuda.synchronize()
                    marks["t0"] = time.perf_counter()
                return False
            # a first call with the same lengths: the cache is sized and the step's graph captured before the timed call
            llm.generate(spec, prompts, n_gen, "greedy", temperature=0.0, stop_ids=[], dtype=dtype)
            out = llm.generate(spec, prompts, n_gen, "greedy", temperature=0.0, stop_ids=[], dtype=dtype, on_step=on_step)
            torch.cuda.synchronize()
            dt = time.perf_counter() - marks["t0"]
            assert all(len(o) == n_gen for o in out)
            graph = llm.load(spec, dtype)[0].decode_graphs.last_graph      # the captured step the run ended on
            e2e = {"value": round(args.batch * args.steps / dt, 1), "unit": "tokens/s",
                   "h2d_bytes_per_step": graph.h2d_bytes, "d2h_bytes_per_step": 4 * args.batch,
                   "window": f"decode steps {args.warmup + 2}..{n_gen - 1} of a generation of {n_gen} tokens: {args.steps} steps "
                             f"after {args.warmup + 1} untimed ones, wall clock, to the last token on the host"}
        c1 = clocks.mark()          # the clock samples cover the device-timed steps and the end-to-end run

        points = {}
        if want_points:
            for bb in point_batches:
                k = max(8, args.steps // 4) if bb == 64 else args.steps
                rec, _ = b.decode_record(eng, sampler, cfg, n_layers, b.equal_prompts(bb, k, args.warmup), k, args.warmup, 3 + bb, dtype)
                points[f"decode_b{bb}"] = rec["value"]
                points[f"decode_b{bb}_frac"] = rec["frac"]
        clk = clocks.summary(c0, c1)

        line = {
            "metric": f"decode tokens/s ({args.shape} shape, random weights, batch {args.batch}, context {args.context})",
            "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16" if dtype == "bfloat16" else "f32",
            "data": "synthetic: uniform random token ids, random-init weights N(0,0.02) drawn on the device",
            "impl": "ours",
            "config": {"model": f"{args.shape} shape", "layers_run": n_layers, "layers_full": full_layers,
                       "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                       "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                       "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                       "rope_theta": cfg["rope_theta"], "rms_eps": cfg["rms_norm_eps"], "tied": cfg["tie_word_embeddings"],
                       "global_batch": args.batch, "seq_len": args.context,
                       "prompt_len": args.prompts or (args.context - args.steps - args.warmup),
                       "parallelism": "1gpu", "l2": "step inputs (weights+cache) exceed L2; prefill flushes L2",
                       "sampling": "greedy"},
            "prefill": prefill, "roofline": roofline, "points": points, "e2e": e2e,
            "gpu_launches": int(round(launches * args.steps)), "clocks": clk,
        }

        # ---- the same model on the true 32-bit path
        if args.f32 and dtype == "bfloat16" and args.prompts is None:
            eng = sampler = None     # the bfloat16 engine's weights and cache go before the next one comes
            eng, sampler = b.load(spec, "float32", 64 * args.context, 64)
            f32 = {"prefill": b.prefill_record(eng, cfg, n_layers, [PREFILL_TOKENS], "float32"), "fma_peak_tflops": round(b.fma_peak(), 1)}
            for bb in (1, 8, 64):
                k = max(8, args.steps // 4) if bb == 64 else args.steps
                rec, _ = b.decode_record(eng, sampler, cfg, n_layers, b.equal_prompts(bb, k, args.warmup), k, args.warmup, 40 + bb, "float32")
                f32[f"decode_b{bb}"] = rec
            line["f32"] = f32

        # ---- the two further shapes of the family
        if args.shapes and dtype == "bfloat16" and args.prompts is None and args.shape == "smollm2-1.7b" and args.layers is None:
            shapes = {}
            lo, hi = parse_prompts(UNEQUAL)
            cfg2, L2, spec2 = b.config("llama3.2-1b")
            lengths = np.random.default_rng(7).integers(lo, hi + 1, 8).tolist()
            eng = sampler = None
            eng, sampler = b.load(spec2, "bfloat16", 8 * args.context, 8)
            rec = {"prompts": UNEQUAL, "batch": 8, "prefill": b.prefill_record(eng, cfg2, L2, lengths, "bfloat16")}
            rec["decode"], _ = b.decode_record(eng, sampler, cfg2, L2, lengths, args.steps, args.warmup, 50, "bfloat16")
            shapes["llama3.2-1b"] = rec
            cfg3, L3, spec3 = b.config("llama3.1-8b")
            eng = sampler = None
            eng, sampler = b.load(spec3, "bfloat16", 64 * args.context, 64)
            rec = {"context": args.context, "prefill": b.prefill_record(eng, cfg3, L3, [PREFILL_TOKENS], "bfloat16")}
            for bb in (1, 8, 64):
                k = max(8, args.steps // 4) if bb == 64 else args.steps
                rec[f"decode_b{bb}"], _ = b.decode_record(eng, sampler, cfg3, L3, b.equal_prompts(bb, k, args.warmup), k,
                                                          args.warmup, 60 + bb, "bfloat16")
            shapes["llama3.1-8b"] = rec
            line["shapes"] = shapes
    finally:
        clocks.stop()
        try:
            llm.unload()
            import shutil
            shutil.rmtree(tmp, ignore_errors=True)
        except Exception:
            pass
    print(json.dumps(line))
    return 0


# ------------------------------------------------------------------ another design beside its closest model
# Layer sizes that resemble a real model's, for the Sozilix decoder (windowed attention beside a gated delta
# rule, then two gated linear recurrences, repeated) and for the Llama decoder of the same width, depth, heads,
# feed-forward and window. `left` widths: keys/values of 128 go through the library's attention kernels, the
# third size (keys 64, values 128) through the kernel that takes values of another width.
DESIGN_SIZES = {
    "w1024": dict(width=1024, heads=8, kv_heads=2, dim=128, vdim=128, window=512, ff=4096, lru=1280, blocks=5, groups=2),
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, window=1024, ff=8192, lru=2560, blocks=10, groups=2),
    "w2048-k64": dict(width=2048, heads=16, kv_heads=4, dim=64, vdim=128, window=1024, ff=8192, lru=2560, blocks=10, groups=2),
}
DESIGN_VOCAB = 32000


def sozilix_config(z):
    par = {"type": "parallel", "mlp": {"ff": z["ff"], "kind": "dense"}, "mixer": {
        "left": {"dim": z["dim"], "heads": z["heads"], "kv_heads": z["kv_heads"], "mask": {"size": z["window"]},
                 "rot": {"base": 10000.0, "dims": z["dim"] // 2}, "scale": z["dim"] ** -0.5, "vdim": z["vdim"]},
        "left_scale": 1.0, "right_scale": 1.0,
        "right": {"conv": 4, "dim": 128, "heads": z["heads"], "kv_heads": z["heads"] // 2, "vdim": 128}}}
    lru = {"type": "rglru", "mlp": None, "mixer": {"width": z["lru"], "blocks": z["blocks"], "conv": 4}}
    return {"architecture": "Sozilix", "canon": {"taps": 4}, "layers": [par, lru, lru] * z["groups"], "norm": {"eps": 1e-5},
            "residual_mult": 1.0, "vocab": DESIGN_VOCAB, "width": z["width"]}


# The Muvorax decoder (latent attention, the selective scan and decayed linear attention, each with routed experts
# but for a dense first layer) at layer sizes that resemble real models of its kinds: a latent of 512 (256) with 128 + 64
# query/key dims a head, scan channels of twice the width with 16 states, linear-attention heads of 128 x 128,
# 64 (32) experts of which 6 (4) are used. The Llama decoder beside it has the same width, depth, heads and the
# dense layer's feed-forward in every layer.
MUVORAX_SIZES = {
    "w1024": dict(width=1024, heads=8, kv_heads=2, dim=128, vdim=128, rot_dim=64, rank=256, ff=4096, experts=32, top=4, n_groups=4,
                  keep=2, expert_ff=704, groups=1),
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, rot_dim=64, rank=512, ff=8192, experts=64, top=6, n_groups=8,
                  keep=3, expert_ff=1408, groups=1),
}


def muvorax_config(z):
    W, H = z["width"], z["heads"]
    rot = {"base": 10000.0, "dims": z["rot_dim"], "scaling": {"factor": 40.0, "fast": 32.0, "original": 4096, "slow": 1.0}}
    moe = {"expert": {"ff": z["expert_ff"]}, "kind": "moe", "router": {
        "experts": z["experts"], "groups": {"count": z["n_groups"], "keep": z["keep"]}, "scale": 2.5, "top": z["top"]}}

    def latent(src=None):
        m = {"dim": z["dim"], "heads": H, "kv_rank": z["rank"], "rot": rot, "rot_dim": z["rot_dim"],
             "scale": (z["dim"] + z["rot_dim"]) ** -0.5, "vdim": z["vdim"]}
        if src is not None:
            m["kv_from"] = src
        return m
    scan = {"conv": 4, "dt_rank": W // 16, "inner": 2 * W, "state": 16}
    lin = {"decay": [1.0 - 2.0 ** (-5 - 3 * h / max(1, H - 1)) for h in range(H)], "dim": 128, "heads": W // 128, "vdim": 128}
    lin["decay"] = lin["decay"][:lin["heads"]] + [0.99] * max(0, lin["heads"] - H)
    layers = []
    for g in range(z["groups"]):
        first = 6 * g
        layers += [{"type": "latent_attention", "mixer": latent(), "mlp": {"ff": z["ff"], "kind": "dense"} if g == 0 else moe},
                   {"type": "mamba1", "mixer": scan, "mlp": moe}, {"type": "lightning", "mixer": lin, "mlp": moe},
                   {"type": "latent_attention", "mixer": latent(first), "mlp": moe}, {"type": "lightning", "mixer": lin, "mlp": moe},
                   {"type": "mamba1", "mixer": scan, "mlp": moe}]
    return {"architecture": "Muvorax", "layers": layers, "norm": {"eps": 1e-6}, "vocab": DESIGN_VOCAB, "width": W}


# The Belasun decoder (chunked grouped-query attention behind short convolutions, a whole-projection query/key norm
# and a gate per head; routed experts with a clamped gate in every layer; a per-layer input from the token) at
# layer sizes that resemble real models of its kinds: heads of 128 of which the first 64 dims turn, chunks of 1024
# (2048) positions, 32 (64) experts of which 4 (6) are used. The Llama decoder beside it has the same width, depth
# and heads, a sliding window as long as a chunk, and a dense feed-forward as wide as a token's experts together.
BELASUN_SIZES = {
    "w1024": dict(width=1024, heads=8, kv_heads=2, dim=128, vdim=128, rot_dims=64, chunk=1024, conv=4, experts=32, top=4,
                  expert_ff=704, side=128, layers=4),
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, rot_dims=64, chunk=2048, conv=4, experts=64, top=6,
                  expert_ff=1408, side=256, layers=4),
}
for _z in BELASUN_SIZES.values():
    _z.update(window=_z["chunk"], ff=_z["top"] * _z["expert_ff"], groups=1)


def belasun_config(z):
    mixer = {"conv": z["conv"], "dim": z["dim"], "heads": z["heads"], "kv_heads": z["kv_heads"], "mask": {"size": z["chunk"]},
             "rot": {"base": 10000.0, "dims": z["rot_dims"], "scaling": {"factor": 8.0, "high": 4.0, "low": 1.0, "original": 8192}},
             "scale": z["dim"] ** -0.5, "vdim": z["vdim"]}
    moe = {"expert": {"ff": z["expert_ff"], "limit": 7.0}, "kind": "moe", "router": {"experts": z["experts"], "top": z["top"]}}
    return {"architecture": "Belasun", "layers": [{"type": "attention", "mixer": mixer, "mlp": moe}] * z["layers"],
            "logit_softcap": 25.0, "norm": {"eps": 1e-6}, "token_side": {"dim": z["side"]}, "vocab": DESIGN_VOCAB, "width": z["width"]}


# The Tufazen decoder (attention whose values are its keys with capped scores, sinks and an elementwise gate, with a dense
# clamped-gate feed-forward; latent attention with queries through a latent and a gate per head, with routed experts in
# groups beside a shared expert; one norm for both sublayers; a pair-table embedding; a per-layer input from the token)
# at layer sizes that resemble real models of its kinds: heads of 128 of which 64 dims turn, a latent of 512 (256) with
# 128 + 64 query/key dims a head and a query latent of 1536 (768), 64 (32) experts of which 6 (4) are used. Four layers of
# which the first two are gone through twice: six layer runs, as many as the Llama decoder beside it has layers (same
# width, heads and dense feed-forward).
TUFAZEN_SIZES = {
    "w1024": dict(width=1024, heads=8, kv_heads=2, dim=128, vdim=128, rot_dim=64, rank=256, q_rank=768, ff=4096, experts=32, top=4,
                  n_groups=4, keep=2, expert_ff=704, shared_ff=1408, side=128, groups=1),
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, rot_dim=64, rank=512, q_rank=1536, ff=8192, experts=64, top=6,
                  n_groups=8, keep=3, expert_ff=1408, shared_ff=2816, side=256, groups=1),
}


def tufazen_config(z):
    att = {"type": "attention", "mlp": {"ff": z["ff"], "kind": "dense", "limit": 7.0}, "mixer": {
        "dim": z["dim"], "heads": z["heads"], "kv_heads": z["kv_heads"], "scale": z["dim"] ** -0.5, "softcap": 30.0, "vdim": z["dim"],
        "rot": {"base": 10000.0, "dims": z["dim"] // 2, "scaling": {"factor": 4.0, "fast": 16.0, "original": 8192, "slow": 2.0}}}}
    lat = {"type": "latent_attention", "mixer": {
        "dim": z["dim"], "heads": z["heads"], "kv_rank": z["rank"], "q_rank": z["q_rank"], "rot_dim": z["rot_dim"],
        "rot": {"base": 10000.0, "dims": z["rot_dim"]}, "scale": (z["dim"] + z["rot_dim"]) ** -0.5, "vdim": z["vdim"]},
        "mlp": {"expert": {"ff": z["expert_ff"]}, "kind": "moe", "shared": {"ff": z["shared_ff"]}, "router": {
            "experts": z["experts"], "groups": {"count": z["n_groups"], "keep": z["keep"]}, "top": z["top"]}}}
    return {"architecture": "Tufazen", "embedding": {"bigram": {"buckets": 100003, "mul_cur": 31, "mul_prev": 1009}},
            "layers": [att, lat, att, lat], "logit_scale": 0.25, "loop": {"start": 0, "stop": 2, "times": 2}, "norm": {"eps": 1e-6},
            "token_side": {"dim": z["side"]}, "vocab": DESIGN_VOCAB, "width": z["width"]}


DESIGNS = {"sozilix": (DESIGN_SIZES, sozilix_config, 3), "muvorax": (MUVORAX_SIZES, muvorax_config, 6),
           "belasun": (BELASUN_SIZES, belasun_config, 4), "tufazen": (TUFAZEN_SIZES, tufazen_config, 6)}


def llama_like(z, max_positions, layers_per_group=3):
    return {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": layers_per_group * z["groups"],
            "hidden_size": z["width"], "num_attention_heads": z["heads"], "num_key_value_heads": z["kv_heads"],
            "head_dim": max(z["dim"], z["vdim"]), "intermediate_size": z["ff"], "vocab_size": DESIGN_VOCAB, "rope_theta": 10000.0,
            "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": max_positions,
            "sliding_window": z.get("window"), "hidden_act": "silu"}


def design_compare(args):
    """Prompt-step and decode throughput of the design named by --design at its sizes beside the Llama decoder
    of equal size (random weights, bfloat16 unless --dtype says otherwise); one JSON line."""
    sizes, make_config, per_group = DESIGNS[args.design]
    pk = peaks()
    tmp = tempfile.mkdtemp(prefix="sllm_bench_")
    b = Bench(args, pk, tmp)
    out = {"metric": "design_compare", "design": args.design, "dtype": args.dtype, "data": "synthetic, random weights",
           "prefill_tokens": args.prefill_tokens, "decode": {"batch": args.batch, "context": args.context, "steps": args.steps,
                                                             "warmup": args.warmup}, "sizes": {}}
    for name in (args.design_sizes.split(",") if args.design_sizes else sizes):
        z = sizes[name]
        rec = {}
        for which, raw in ((args.design, make_config(z)), ("llama", llama_like(z, args.context + args.prefill_tokens + 64, per_group))):
            path = os.path.join(tmp, f"{name}-{which}.json")
            with open(path, "w") as f:
                json.dump(raw, f)
            eng, sampler = b.load(f"random:{path}:0", args.dtype, max(args.batch * (args.context + 64), args.prefill_tokens + 64),
                                  args.batch)
            n_params = sum(p.elements_read_per_step() for e in eng.layout.schedule for p in eng.model.blocks[e.layer].parts())
            r = {"layer_params": n_params}
            if args.only != "decode":
                ms = b.time_prompt_step(eng, [args.prefill_tokens], 1)
                r["prefill"] = {"ms": round(ms, 3), "tok_s": round(args.prefill_tokens / ms * 1e3, 1),
                                "matrix_tflops": round(2 * n_params * args.prefill_tokens / (ms * 1e-3) / 1e12, 1)}
            if args.only != "prefill":
                lens = b.equal_prompts(args.batch, args.steps, args.warmup)
                ms, _, launches = b.time_decode(eng, sampler, lens, args.steps, args.warmup, 3)
                r["decode"] = {"ms": round(ms, 4), "tok_s": round(args.batch / ms * 1e3, 1), "launches_per_step": launches,
                               "weights_gbs": round(WIDTH[args.dtype] * (n_params + DESIGN_VOCAB * z["width"]) / (ms * 1e-3) / 1e9, 1)}
            rec[which] = r
        out["sizes"][name] = rec
    import shutil
    shutil.rmtree(tmp, ignore_errors=True)
    print(json.dumps(out))
    return 0


def sequence_kernels_alone(args):
    """The kernels of the mixers with state, each alone at the sizes of DESIGN_SIZES[--design-sizes or w2048]: a prompt
    of --prefill-tokens rows and a decode step of --batch rows; a JSON line each with the time (CUDA events around a
    captured run of launches whose inputs rotate through more than L2 holds) and what it is of the HBM copy rate or
    of the float FMA rate."""
    import torch
    from scriptling_llm_lib_b200.csrc.bindings import KernelSet, ProbeKernels
    pk = peaks()
    z = DESIGN_SIZES[(args.design_sizes or "w2048").split(",")[0]]
    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[args.dtype]
    k = KernelSet(dt).seq
    fma = ProbeKernels().fma_tflops()
    dev = "cuda"
    W, H, G, dk, dv, LW, bs = z["width"], z["heads"], z["heads"] // 2, 128, 128, z["lru"], z["lru"] // z["blocks"]
    AH, AG, hd, vd, window = z["heads"], z["kv_heads"], z["dim"], z["vdim"], z["window"]
    esz = 2 if dt == torch.bfloat16 else 4

    class Ctx:
        pass

    def timed(launch, n_sets, reps=8):
        torch.cuda.synchronize()          # the inputs were filled on the current stream; the launches run on another
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            for i in range(2):
                launch(i % n_sets)
            torch.cuda.synchronize()
            with torch.cuda.graph(graph, stream=side):
                for i in range(reps):
                    launch(i % n_sets)
        for _ in range(2):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(3):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (3 * reps) * 1e3

    def report(name, rows, us, nbytes=None, flops=None):
        rec = {"kernel": name, "rows": rows, "us": round(us, 1)}
        if nbytes is not None:
            rec.update(gbs=round(nbytes / us / 1e3, 1), of_hbm=round(nbytes / us / 1e3 / pk["hbm_gbs"], 3))
        if flops is not None:
            rec.update(tflops=round(flops / us / 1e6, 2), of_fma=round(flops / us / 1e6 / fma, 3))
        print(json.dumps(rec), flush=True)

    for label, lens in (("prompt", [args.prefill_tokens]), ("decode", [1] * args.batch)):
        T, B = sum(lens), len(lens)
        c = Ctx()
        start = [0]
        for n in lens:
            start.append(start[-1] + n)
        c.seq_start = torch.tensor(start, dtype=torch.int32, device=dev)
        c.tok_seq = torch.repeat_interleave(torch.arange(B, dtype=torch.int32, device=dev), torch.tensor(lens, device=dev)).int()
        c.slots = torch.arange(B, dtype=torch.int32, device=dev)
        c.n_seqs, c.max_new = B, max(lens)
        n_sets = 4 if T > 64 else 24
        # ---- residual sum + layer norm
        xs = [torch.randn(T, W, device=dev) for _ in range(n_sets)]
        ad = [torch.randn(T, W, device=dev).to(dt) for _ in range(n_sets)]
        wn = torch.ones(W, device=dev).to(dt)
        y = torch.empty(T, W, dtype=torch.float32, device=dev)
        us = timed(lambda i: k.add_norm(xs[i], [(ad[i], 0.5)], None, wn, y, 1e-5, True), n_sets)
        report(f"add_norm ({label})", T, us, nbytes=T * W * (4 + 4 + esz + 4))
        # ---- short convolution in front of the mixer (float in, element type out), state update included
        wc = torch.randn(W, 4, device=dev).to(dt)
        st = torch.zeros(B + 1, 3, W, device=dev)
        yo = torch.empty(T, W, dtype=dt, device=dev)
        us = timed(lambda i: k.causal_conv(xs[i], wc, st, c, yo, 4, add_input=True), n_sets)
        report(f"causal_conv width {W} ({label})", T, us, nbytes=T * W * (4 + esz) + (2 * B * 3 * W * 4 if T == B else 0))
        # ---- gated delta rule
        qk = [torch.randn(T, 2 * G * dk, device=dev) for _ in range(n_sets)]
        vv = [torch.randn(T, H * dv, device=dev) for _ in range(n_sets)]
        ba = torch.randn(T, 2 * H, device=dev)
        al, db = torch.zeros(H, device=dev).to(dt), torch.zeros(H, device=dev).to(dt)
        bd = torch.empty(T, 2 * H + G, device=dev)
        n_st = 1 if T > 64 else n_sets
        S = [torch.zeros(B + 1, H, dk, dv, device=dev) for _ in range(n_st)]
        o = torch.empty(T, H * dv, device=dev)
        us = timed(lambda i: k.delta_prepare(qk[i], ba, al, db, bd, H, G, dk), n_sets)
        report(f"delta_prepare ({label})", T, us, nbytes=T * (4 * G * dk * 4))
        k.delta_prepare(qk[0], ba, al, db, bd, H, G, dk)
        us = timed(lambda i: k.delta_rule(qk[i], vv[i], bd, S[i % n_st], c, o, H, G, dk, dv), n_sets)
        report(f"delta_rule heads {H} x {dk} x {dv} ({label})", T, us,
               nbytes=(T * (2 * G * dk + 2 * H * dv) * 4 + 2 * B * H * dk * dv * 4), flops=7 * T * H * dk * dv)
        # ---- gated linear recurrence
        gates = [torch.randn(z["blocks"], T, 2 * bs, device=dev) for _ in range(n_sets)]
        u = [torch.randn(T, LW, device=dev) for _ in range(n_sets)]
        yraw = torch.randn(T, LW, device=dev).to(dt)
        zb = torch.zeros(LW, device=dev).to(dt)
        Ls = torch.zeros(B + 1, LW, device=dev)
        out = torch.empty(T, LW, dtype=dt, device=dev)
        us = timed(lambda i: k.rglru_scan(gates[i], u[i], yraw, zb, zb, zb, zb, Ls, c, out, bs), n_sets)
        report(f"rglru_scan width {LW} ({label})", T, us, nbytes=T * LW * (8 + 4 + esz + esz))
        # ---- attention: cache write with value norm, then the kernel for values of another width than keys
        if dt == torch.bfloat16 or T <= 64:
            ctxlen = args.context if T == B else T
            pages = -(-ctxlen // 64)
            kp = torch.randn(B * pages + 1, AG, 64, hd, device=dev).to(dt)
            vp = torch.randn(B * pages + 1, AG, 64, vd, device=dev).to(dt)
            table = torch.arange(B * pages, dtype=torch.int32, device=dev).view(B, pages).contiguous()
            pos = (torch.arange(T, dtype=torch.int32, device=dev) if T != B else
                   torch.full((B,), ctxlen - 1, dtype=torch.int32, device=dev))
            qkv = torch.randn(T, AH * hd + AG * hd + AG * vd, device=dev).to(dt)
            cs = torch.zeros(ctxlen + 1, hd // 4, 2, device=dev)
            cs[..., 0] = 1.0
            us = timed(lambda i: k.kv_store(qkv, pos, c.tok_seq, table, cs, kp, vp, AH, AG, hd, vd, hd // 2, True, 1e-5), 1)
            report(f"kv_store ({label})", T, us, nbytes=T * (AH * hd + 2 * AG * (hd + vd)) * esz)
            ao = torch.empty(T, AH * vd, dtype=dt, device=dev)
            us = timed(lambda i: k.attn_wide_value(qkv, ao, pos, c.tok_seq, table, kp, vp, AH, AG, hd, vd, window, 0.1), 1)
            keys = sum(min(int(p) + 1, window) for p in pos.tolist())
            report(f"attn_wide_value keys {hd} values {vd} window {window} ({label})", T, us,
                   nbytes=(keys * AG * (hd + vd) * esz if T == B else None), flops=2 * keys * AH * (hd + vd))
    return 0


def mix_kernels_alone(args):
    """The kernels of the Muvorax decoder's mixers and feed-forwards, each alone at MUVORAX_SIZES[--design-sizes or w2048]:
    a prompt of --prefill-tokens rows and a decode step of --batch rows at --context; a JSON line each with the time
    (CUDA events around a captured run of launches whose inputs rotate through more than L2 holds where they are small)
    and what it is of the HBM copy rate or of the float FMA rate (bf16 tensor rate for the grouped products)."""
    import torch
    from types import SimpleNamespace
    from scriptling_llm_lib_b200.csrc.bindings import KernelSet, ProbeKernels
    pk = peaks()
    z = MUVORAX_SIZES[(args.design_sizes or "w2048").split(",")[0]]
    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[args.dtype]
    ks = KernelSet(dt)
    k = ks.mix
    fma = ProbeKernels().fma_tflops()
    dev = "cuda"
    esz = 2 if dt == torch.bfloat16 else 4
    W, H, D, P, V, R = z["width"], z["heads"], z["dim"], z["rot_dim"], z["vdim"], z["rank"]
    LH, LD, LV = W // 128, 128, 128
    I, N, K = 2 * W, 16, W // 16
    E, top, F = z["experts"], z["top"], z["expert_ff"]

    def timed(launch, n_sets, reps=8):
        torch.cuda.synchronize()          # the inputs were filled on the current stream; the launches run on another
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            for i in range(2):
                launch(i % n_sets)
            torch.cuda.synchronize()
            with torch.cuda.graph(graph, stream=side):
                for i in range(reps):
                    launch(i % n_sets)
        for _ in range(2):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(3):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (3 * reps) * 1e3

    def report(name, rows, us, nbytes=None, flops=None, tensor=False):
        rec = {"kernel": name, "rows": rows, "us": round(us, 1)}
        if nbytes is not None:
            rec.update(gbs=round(nbytes / us / 1e3, 1), of_hbm=round(nbytes / us / 1e3 / pk["hbm_gbs"], 3))
        if flops is not None and tensor:
            rec.update(tflops=round(flops / us / 1e6, 1), of_bf16=round(flops / us / 1e6 / pk["bf16_tflops"], 3))
        elif flops is not None:
            rec.update(tflops=round(flops / us / 1e6, 2), of_fma=round(flops / us / 1e6 / fma, 3))
        print(json.dumps(rec), flush=True)

    for label, lens, ctxlen in (("prompt", [args.prefill_tokens], args.prefill_tokens), ("decode", [1] * args.batch, args.context)):
        T, B = sum(lens), len(lens)
        start = [0]
        for n in lens:
            start.append(start[-1] + n)
        pages = -(-ctxlen // 64)
        c = SimpleNamespace(
            seq_start=torch.tensor(start, dtype=torch.int32, device=dev),
            tok_seq=torch.repeat_interleave(torch.arange(B, dtype=torch.int32, device=dev), torch.tensor(lens, device=dev)).int(),
            slots=torch.arange(B, dtype=torch.int32, device=dev), n_seqs=B, max_new=max(lens), engine=SimpleNamespace(sm_count=148),
            tok_pos=(torch.arange(T, dtype=torch.int32, device=dev) if T != B else
                     torch.full((B,), ctxlen - 1, dtype=torch.int32, device=dev)))
        n_sets = 4 if T > 64 else 24
        # ---- residual sum with a normed addend + norm
        xs = [torch.randn(T, W, device=dev) for _ in range(n_sets)]
        ad = [torch.randn(T, W, device=dev).to(dt) for _ in range(n_sets)]
        wn, bn = torch.ones(W, device=dev), torch.zeros(W, device=dev)
        y = torch.empty(T, W, dtype=dt, device=dev)
        us = timed(lambda i: k.dyt_add_norm(xs[i], ad[i], (wn, bn, 0.9), None, wn, bn, 1.1, y), n_sets)
        report(f"dyt_add_norm ({label})", T, us, nbytes=T * W * (4 + 4 + esz + esz))
        # ---- linear attention with a decay per head, and its gated read-out norm
        proj = [(torch.randn(T, 2 * LH * LD + 2 * LH * LV, device=dev) * 0.5).to(dt) for _ in range(n_sets)]
        decay = torch.full((LH,), 0.99, device=dev)
        n_st = 1 if T > 64 else n_sets
        S = [torch.zeros(B + 1, LH, LD, LV, device=dev) for _ in range(n_st)]
        o = torch.empty(T, LH * LV, device=dev)
        us = timed(lambda i: k.lin_attn_decay(proj[i], 0, LH * LD, 2 * LH * LD, decay, S[i % n_st], c, o, LH, LD, LV), n_sets)
        report(f"lin_attn_decay heads {LH} x {LD} x {LV} ({label})", T, us, nbytes=(2 * B * LH * LD * LV * 4 if T == B else None),
               flops=2 * T * LH * (2 * LD * LV + 16 * (LD + LV)))
        yo = torch.empty(T, LH * LV, dtype=dt, device=dev)
        us = timed(lambda i: k.gated_row_rms(o, proj[i][:, 2 * LH * LD + LH * LV:], wn[:1].expand(LH * LV).contiguous(), yo, 1e-6, "sigmoid"), n_sets)
        report(f"gated_row_rms ({label})", T, us, nbytes=T * LH * LV * (4 + esz + esz))
        # ---- the selective scan
        xz = [(torch.randn(T, 2 * I, device=dev) * 0.5).to(dt) for _ in range(n_sets)]
        dtr = torch.randn(T, I, device=dev)
        bc = torch.randn(T, K + 2 * N, device=dev).to(dt)
        zero_i, a_log = torch.zeros(I, device=dev), torch.zeros(I, N, device=dev)
        Ss = [torch.zeros(B + 1, I, N, device=dev) for _ in range(n_st)]
        ys = torch.empty(T, I, dtype=dt, device=dev)
        us = timed(lambda i: k.selective_scan(xz[i][:, :I], dtr, zero_i, a_log, zero_i + 1, bc, K, K + N, xz[i][:, I:], Ss[i % n_st], c, ys, I, N), n_sets)
        report(f"selective_scan inner {I} states {N} ({label})", T, us,
               nbytes=T * I * (4 + 3 * esz) + (2 * B * I * N * 4 if T == B else 0), flops=6 * T * I * N)
        # ---- attention over the cached latent
        Wl = R + P
        lat = torch.randn(B * pages + 1, 1, 64, Wl, device=dev).to(dt)
        table = torch.arange(B * pages, dtype=torch.int32, device=dev).view(B, pages).contiguous()
        q = (torch.randn(T, H * (D + P), device=dev) * 0.3).to(dt)
        wuk, wuv = (torch.randn(H * D, R, device=dev) * 0.05).to(dt), (torch.randn(H * V, R, device=dev) * 0.05).to(dt)
        qa = torch.empty(T, H, Wl, device=dev)
        us = timed(lambda i: k.latent_absorb(q, wuk, qa, H, D, P, R, 0.07), 1)
        report(f"latent_absorb ({label})", T, us, nbytes=(H * D * R * esz if T == B else None), flops=2 * T * H * D * R)
        if T == B:
            n_split = max(1, min(-(-2 * 148 // (B * -(-H // 8))), pages * 2, 64))
            part = torch.empty(T, H, n_split, R + 2, device=dev)
            us = timed(lambda i: k.latent_attn(qa, lat, c, table, part, H, R, P, n_split), 1)
            report(f"latent_attn rank {R} + {P}, {n_split} splits ({label})", T, us, nbytes=B * ctxlen * Wl * esz,
                   flops=2 * B * H * ctxlen * (2 * R + P))
            olat = torch.empty(T, H, R, device=dev)
            ao = torch.empty(T, H * V, dtype=dt, device=dev)
            us = timed(lambda i: k.latent_expand(part, olat, wuv, ao, H, V, R, n_split), 1)
            report(f"latent_expand ({label})", T, us, nbytes=H * V * R * esz + T * H * n_split * R * 4)
        else:
            hd = D + P
            kt = torch.randn(pages, H, 64, hd, device=dev).to(dt)
            qt = torch.randn(T, H * hd, device=dev).to(dt)
            ot = torch.empty(T, H * hd, dtype=dt, device=dev)
            zero_b = torch.zeros(B, dtype=torch.int32, device=dev)
            us = timed(lambda i: ks.attn_paged(qt, ot, c.seq_start, zero_b, table, kt, kt, B, T, H, H, hd, None, 0.07), 1)
            report(f"attn_paged per head, width {hd} ({label}, keys and values made from the latent)", T, us, flops=2 * H * T * T * hd)
        # ---- routed experts
        h = (torch.randn(T, W, device=dev) * 0.5).to(dt)
        zl = torch.randn(T, E, device=dev)
        corr = torch.zeros(E, device=dev)
        idx = torch.empty(T, top, dtype=torch.int32, device=dev)
        wgt = torch.empty(T, top, device=dev)
        us = timed(lambda i: k.moe_route(zl, corr, idx, wgt, z["n_groups"], z["keep"], top, 2.5), 1)
        report(f"moe_route {E} experts ({label})", T, us)
        w_up = (torch.randn(E, F, W, device=dev) * 0.02).to(dt)
        w_down = (torch.randn(E, W, F, device=dev) * 0.02).to(dt)
        pairs = T * top
        if pairs <= 64:
            hid = torch.empty(pairs, F, dtype=dt, device=dev)
            out = torch.empty(top, T, W, device=dev)
            us = timed(lambda i: k.moe_pairs(h, w_up, w_down, idx, wgt, hid, out), 1)
            report(f"moe_pairs {pairs} pairs, experts {W} x {F} ({label})", T, us, nbytes=pairs * 2 * F * W * esz)
        elif dt == torch.bfloat16:
            rows = -(-(pairs + E * 127) // 128) * 128
            counts = torch.zeros(E, dtype=torch.int32, device=dev)
            offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
            por = torch.empty(rows, dtype=torch.int32, device=dev)
            rop = torch.empty(pairs, dtype=torch.int32, device=dev)
            tg = torch.empty(rows // 128, dtype=torch.int32, device=dev)
            xs2 = torch.empty(rows, W, dtype=dt, device=dev)
            hid = torch.empty(rows, F, dtype=dt, device=dev)
            ys2 = torch.empty(rows, W, device=dev)
            out = torch.empty(T, W, device=dev)
            err = torch.zeros(1, dtype=torch.int32, device=dev)
            tc = ks.tensor_core
            us = timed(lambda i: (k.moe_group_rows(idx, counts, offsets, por, rop, tg, pad=128), k.moe_gather_rows(h, por, top, xs2)), 1)
            report(f"moe_group_rows + moe_gather_rows ({label})", T, us, nbytes=rows * W * esz * 2)
            us = timed(lambda i: tc.gemm_grouped(xs2, w_up, hid, tg, err, act="relu_squared", rows_used=offsets[E:]), 1)
            report(f"gemm_grouped up, {rows} rows for {pairs} pairs ({label})", T, us, flops=2 * pairs * F * W, tensor=True)
            us = timed(lambda i: tc.gemm_grouped(hid, w_down, ys2, tg, err, rows_used=offsets[E:]), 1)
            report(f"gemm_grouped down ({label})", T, us, flops=2 * pairs * F * W, tensor=True)
            us = timed(lambda i: k.moe_combine(ys2, rop, wgt, out), 1)
            report(f"moe_combine ({label})", T, us, nbytes=(pairs + T) * W * 4)
    return 0


def gate_kernels_alone(args):
    """The kernels of the Belasun decoder's layers, each alone at BELASUN_SIZES[--design-sizes or w2048] and, where
    another decoder has a kernel of the same kind, that one beside it on the same rows: a prompt of --prefill-tokens
    rows and a decode step of --batch rows at --context; a JSON line each with the time (CUDA events around a captured
    run of launches whose inputs rotate through more than L2 holds where they are small) and what it is of the HBM copy
    rate (bf16 tensor rate for the grouped products and the prompt's attention)."""
    import torch
    from types import SimpleNamespace
    from scriptling_llm_lib_b200.csrc.bindings import KernelSet
    pk = peaks()
    z = BELASUN_SIZES[(args.design_sizes or "w2048").split(",")[0]]
    dt = torch.bfloat16
    ks = KernelSet(dt)
    dev = "cuda"
    esz = 2
    W, H, G, D, V, rot, chunk, taps = z["width"], z["heads"], z["kv_heads"], z["dim"], z["vdim"], z["rot_dims"], z["chunk"], z["conv"]
    E, top, F, side = z["experts"], z["top"], z["expert_ff"], z["side"]
    qw, kw, vw = H * D, G * D, G * V
    Cw = qw + kw + vw
    sms = torch.cuda.get_device_properties(0).multi_processor_count

    def timed(launch, n_sets, reps=8):
        torch.cuda.synchronize()          # the inputs were filled on the current stream; the launches run on another
        side_stream = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side_stream):
            for i in range(2):
                launch(i % n_sets)
            torch.cuda.synchronize()
            with torch.cuda.graph(graph, stream=side_stream):
                for i in range(reps):
                    launch(i % n_sets)
        for _ in range(2):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(3):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (3 * reps) * 1e3

    def report(name, rows, us, nbytes=None, flops=None, like=None):
        rec = {"kernel": name, "rows": rows, "us": round(us, 1)}
        if like is not None:
            rec["like"] = like
        if nbytes is not None:
            rec.update(gbs=round(nbytes / us / 1e3, 1), of_hbm=round(nbytes / us / 1e3 / pk["hbm_gbs"], 3))
        if flops is not None:
            rec.update(tflops=round(flops / us / 1e6, 1), of_bf16=round(flops / us / 1e6 / pk["bf16_tflops"], 3))
        print(json.dumps(rec), flush=True)

    err = torch.zeros(1, dtype=torch.int32, device=dev)
    for label, lens, ctxlen in (("prompt", [args.prefill_tokens], args.prefill_tokens), ("decode", [1] * args.batch, args.context)):
        T, B = sum(lens), len(lens)
        start = [0]
        for n in lens:
            start.append(start[-1] + n)
        pages = -(-ctxlen // 64)
        pos0 = torch.zeros(B, dtype=torch.int32, device=dev) if T != B else torch.full((B,), ctxlen - 1, dtype=torch.int32, device=dev)
        c = SimpleNamespace(
            seq_start=torch.tensor(start, dtype=torch.int32, device=dev),
            tok_seq=torch.repeat_interleave(torch.arange(B, dtype=torch.int32, device=dev), torch.tensor(lens, device=dev)).int(),
            slots=torch.arange(B, dtype=torch.int32, device=dev), n_seqs=B, max_new=max(lens), engine=SimpleNamespace(sm_count=sms),
            seq_pos0=pos0, is_decode=T == B,
            tok_pos=(torch.arange(T, dtype=torch.int32, device=dev) if T != B else pos0.clone()))
        n_sets = 4 if T > 64 else 24
        table = torch.arange(B * pages, dtype=torch.int32, device=dev).view(B, pages).contiguous()
        kp = torch.randn(B * pages + 1, G, 64, D, device=dev).to(dt)
        vp = torch.randn(B * pages + 1, G, 64, V, device=dev).to(dt)
        cs = torch.randn(ctxlen + 1, rot // 2, 2, device=dev)
        # ---- the short convolution behind the projections: element type in, float32 out, the state kept
        ys = [(torch.randn(T, Cw + H, device=dev) * 0.5).to(dt) for _ in range(n_sets)]
        wc = torch.randn(Cw, taps, device=dev).to(dt)
        st = torch.zeros(B + 1, taps - 1, Cw, device=dev)
        cf = [torch.empty(T, Cw, device=dev) for _ in range(n_sets)]
        us = timed(lambda i: ks.seq.causal_conv(ys[i][:, :Cw], wc, st, c, cf[i], taps), n_sets)
        report(f"causal_conv {taps} taps, width {Cw} ({label})", T, us, nbytes=T * Cw * (esz + 4) + (2 * B * (taps - 1) * Cw * 4 if T == B else 0))
        # ---- norm over the whole projection + rotation + cache write, beside the rotation + cache write of a plain layer
        qn, kn = torch.ones(qw, device=dev), torch.ones(kw, device=dev)
        q = torch.empty(T, qw, dtype=dt, device=dev)
        us = timed(lambda i: ks.gate.qk_norm_store(cf[i], q, c.tok_pos, c.tok_seq, table, cs, kp, vp, H, G, D, V, rot, False, qn, kn, 1e-6), n_sets)
        report(f"qk_norm_store ({label})", T, us, nbytes=T * Cw * (4 + esz))
        us = timed(lambda i: ks.gate.conv_qk_norm_store(ys[i][:, :Cw], wc, taps, st, c, q, table, cs, kp, vp, H, G, D, V, rot, False,
                                                        qn, kn, 1e-6), n_sets)
        report(f"conv_qk_norm_store: the two above in one kernel ({label})", T, us, nbytes=2 * T * Cw * esz)
        cs_full = torch.randn(ctxlen + 1, D // 2, 2, device=dev)
        if D == V:
            us = timed(lambda i: ks.rope_kv_write(ys[i], c.tok_pos, c.tok_seq, table, cs_full, kp, vp, H, G, D, D, False), n_sets)
            report(f"rope_kv_write ({label})", T, us, nbytes=T * (2 * (qw + kw) + 2 * vw) * esz, like="conv_qk_norm_store")
        # ---- the gate per head, beside the gated read-out norm of a linear-attention layer
        o = torch.empty(T, H * V, dtype=dt, device=dev)
        us = timed(lambda i: ks.gate.head_gate(o, ys[i][:, Cw:], H, V), n_sets)
        report(f"head_gate ({label})", T, us, nbytes=2 * T * H * V * esz)
        # ---- attention over the keys of the query's chunk, beside a sliding window of the same length
        if T != B:
            if D in ks.prefill_attention_tc.HEAD_DIMS and D == V:
                for span, name, like in ((-chunk, f"chunks of {chunk}", None), (chunk, f"window of {chunk}", "chunks")):
                    seen = sum((p % chunk if span < 0 else min(p, chunk - 1)) + 1 for p in range(T))
                    us = timed(lambda i: ks.prefill_attention_tc.attn(q, o, c.seq_start, c.seq_pos0, table, kp, vp, B, T, H, G, D, span,
                                                                      D ** -0.5, err), 1)
                    report(f"attn_prefill {H}/{G} heads of {D}, {name} ({label})", T, us, flops=4 * H * D * seen, like=like)
        elif D in ks.decode.HEAD_DIMS and D == V:
            n_split = ks.decode.attention_splits(B, H, G, D, pages, sms)
            scratch = torch.empty(B * H * n_split * (D + 2), dtype=torch.float32, device=dev)
            tickets = torch.zeros(B * G, dtype=torch.int32, device=dev)
            for span, name, like in ((-chunk, f"chunks of {chunk}", None), (chunk, f"window of {chunk}", "chunks")):
                seen = ((ctxlen - 1) % chunk if span < 0 else min(ctxlen - 1, chunk - 1)) + 1
                us = timed(lambda i: ks.decode.attn_decode(q, o, c.seq_pos0, table, kp, vp, scratch, B, H, G, D, span, D ** -0.5,
                                                           n_split, tickets=tickets), 1)
                report(f"attn_decode {H}/{G} heads of {D}, {name}, {n_split} splits ({label})", T, us, nbytes=B * seen * G * (D + V) * esz, like=like)
        # ---- the router, beside the router with runs of experts
        zl = torch.randn(T, E, device=dev)
        corr = torch.zeros(E, device=dev)
        idx = torch.empty(T, top, dtype=torch.int32, device=dev)
        wgt = torch.empty(T, top, device=dev)
        us = timed(lambda i: ks.mix.moe_route(zl, corr, idx, wgt, 1, 1, top, 1.0, top_softmax=True), 1)
        report(f"moe_route top_softmax, {top} of {E} ({label})", T, us)
        us = timed(lambda i: ks.mix.moe_route(zl, corr, idx, wgt, 1, 1, top, 1.0), 1)
        report(f"moe_route grouped_sigmoid, {top} of {E} ({label})", T, us, like="moe_route top_softmax")
        ks.mix.moe_route(zl, corr, idx, wgt, 1, 1, top, 1.0, top_softmax=True)
        # ---- the experts: gate and up rows in tiles of 16 with the clamped gate, beside up rows with the square of relu
        h = (torch.randn(T, W, device=dev) * 0.5).to(dt)
        w_gu = (torch.randn(E, 2 * F, W, device=dev) * 0.02).to(dt)
        w_down = (torch.randn(E, W, F, device=dev) * 0.02).to(dt)
        pairs = T * top
        if pairs <= 64:
            hid = torch.empty(pairs, F, dtype=dt, device=dev)
            out = torch.empty(top, T, W, device=dev)
            us = timed(lambda i: ks.mix.moe_pairs(h, w_gu, w_down, idx, wgt, hid, out, glu=(7.0, 1.702), tiled=True), 1)
            report(f"moe_pairs clamped gate, {pairs} pairs, experts {W} x {F} ({label})", T, us, nbytes=pairs * 3 * F * W * esz)
            w_u1 = w_gu[:, :F].contiguous()
            us = timed(lambda i: ks.mix.moe_pairs(h, w_u1, w_down, idx, wgt, hid, out), 1)
            report(f"moe_pairs relu^2 ({label})", T, us, nbytes=pairs * 2 * F * W * esz, like="moe_pairs clamped gate")
        else:
            rows = -(-(pairs + E * 127) // 128) * 128
            counts = torch.zeros(E, dtype=torch.int32, device=dev)
            offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
            por = torch.empty(rows, dtype=torch.int32, device=dev)
            rop = torch.empty(pairs, dtype=torch.int32, device=dev)
            tg = torch.empty(rows // 128, dtype=torch.int32, device=dev)
            xs2 = torch.empty(rows, W, dtype=dt, device=dev)
            hid = torch.empty(rows, F, dtype=dt, device=dev)
            raw = torch.empty(rows, 2 * F, dtype=dt, device=dev)
            ys2 = torch.empty(rows, W, device=dev)
            out = torch.empty(T, W, device=dev)
            tc = ks.tensor_core
            ks.mix.moe_group_rows(idx, counts, offsets, por, rop, tg, pad=128)
            ks.mix.moe_gather_rows(h, por, top, xs2)
            us = timed(lambda i: tc.gemm_grouped(xs2, w_gu, hid, tg, err, rows_used=offsets[E:], glu=(7.0, 1.702)), 1)
            report(f"gemm_grouped gate|up with the clamped gate, {rows} rows for {pairs} pairs ({label})", T, us, flops=4 * pairs * F * W)
            us = timed(lambda i: (tc.gemm_grouped(xs2, w_gu, raw, tg, err, rows_used=offsets[E:]),
                                  ks.mix.glu_clamp(raw, hid, 7.0, 1.702, rows_used=offsets[E:], tiled=True)), 1)
            report(f"gemm_grouped gate|up, then glu_clamp in a pass of its own ({label})", T, us, flops=4 * pairs * F * W)
            w_u2 = w_gu.view(E * 2, F, W)
            us = timed(lambda i: tc.gemm_grouped(xs2, w_u2, hid, tg, err, act="relu_squared", rows_used=offsets[E:]), 1)
            report(f"gemm_grouped up with relu^2 ({label})", T, us, flops=2 * pairs * F * W, like="gemm_grouped gate|up")
            us = timed(lambda i: tc.gemm_grouped(hid, w_down, ys2, tg, err, rows_used=offsets[E:]), 1)
            report(f"gemm_grouped down ({label})", T, us, flops=2 * pairs * F * W)
        # ---- the input from the token: the stream takes the sublayer, gelu(a) * e, the normed addend; beside the sum + norm of every layer
        x32 = [torch.randn(T, W, device=dev) for _ in range(n_sets)]
        d32 = [torch.randn(T, W, device=dev) for _ in range(n_sets)]
        xb = torch.empty(T, W, dtype=dt, device=dev)
        us = timed(lambda i: ks.gate.add_cast(x32[i], d32[i], xb), n_sets)
        report(f"add_cast ({label})", T, us, nbytes=T * W * (4 + 4 + 4 + esz))
        a = (torch.randn(T, side, device=dev)).to(dt)
        tbl = torch.randn(DESIGN_VOCAB, z["layers"] * side, device=dev).to(dt)
        ids = torch.randint(0, DESIGN_VOCAB, (T,), dtype=torch.int32, device=dev)
        g = torch.empty(T, side, dtype=dt, device=dev)
        us = timed(lambda i: ks.gate.gelu_mul_rows(a, ids, tbl, side, g), 1)
        report(f"gelu_mul_rows width {side} ({label})", T, us, nbytes=3 * T * side * esz)
        wn = torch.ones(W, device=dev)
        us = timed(lambda i: ks.gate.add_rms_normed(x32[i], d32[i], wn, 1e-6), n_sets)
        report(f"add_rms_normed ({label})", T, us, nbytes=T * W * (4 + 4 + 4))
        wnb = torch.ones(W, device=dev).to(dt)
        us = timed(lambda i: ks.gate.add_rms_normed(x32[i], d32[i], wn, 1e-6, norm=(wnb, 1e-6, xb)), n_sets)
        report(f"add_rms_normed with the next norm's output ({label})", T, us, nbytes=T * W * (4 + 4 + 4 + esz))
        ad = (torch.randn(T, W, device=dev) * 0.5).to(dt)
        us = timed(lambda i: ks.add_rmsnorm(x32[i], ad, None, wnb, xb, 1e-6), n_sets)
        report(f"add_rmsnorm ({label})", T, us, nbytes=T * W * (4 + 4 + esz + esz), like="add_rms_normed, add_cast")
        lg = torch.randn(max(B, 1), DESIGN_VOCAB, device=dev)
        us = timed(lambda i: ks.gate.softcap(lg, 25.0), 1)
        report(f"softcap {lg.shape[0]} x {DESIGN_VOCAB} ({label})", T, us, nbytes=2 * lg.numel() * 4)
    return 0


def tufazen_kernels_alone(args):
    """What the Tufazen decoder added to the kernels, each alone at TUFAZEN_SIZES[--design-sizes or w2048] beside its like on
    the same rows: attention with a cap and sinks beside the same kernel without, the sum of several addends beside the sum of
    one, the normed addend followed by the norm without statistics beside the one followed by an RMS norm, the embedding with
    a pair table beside the plain one, the gate per element beside the gate per head, the router over all experts beside the
    one over the picked, the dense clamped gate in the grouped product's epilogue beside the SiLU gate. A prompt of
    --prefill-tokens rows and a decode step of --batch rows at --context; a JSON line each (CUDA events around a captured run
    of launches; inputs rotate through more than L2 holds where they are small)."""
    import torch
    from types import SimpleNamespace
    from scriptling_llm_lib_b200.csrc.bindings import KernelSet
    pk = peaks()
    z = TUFAZEN_SIZES[(args.design_sizes or "w2048").split(",")[0]]
    dt, dev, esz = torch.bfloat16, "cuda", 2
    ks = KernelSet(dt)
    W, H, G, D, E, top, F = z["width"], z["heads"], z["kv_heads"], z["dim"], z["experts"], z["top"], z["ff"]
    sms = torch.cuda.get_device_properties(0).multi_processor_count

    def timed(launch, n_sets, reps=8):
        torch.cuda.synchronize()
        side_stream = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side_stream):
            for i in range(2):
                launch(i % n_sets)
            torch.cuda.synchronize()
            with torch.cuda.graph(graph, stream=side_stream):
                for i in range(reps):
                    launch(i % n_sets)
        for _ in range(2):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(3):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (3 * reps) * 1e3

    def report(name, rows, us, nbytes=None, flops=None, like=None):
        rec = {"kernel": name, "rows": rows, "us": round(us, 1)}
        if like is not None:
            rec["like"] = like
        if nbytes is not None:
            rec.update(gbs=round(nbytes / us / 1e3, 1), of_hbm=round(nbytes / us / 1e3 / pk["hbm_gbs"], 3))
        if flops is not None:
            rec.update(tflops=round(flops / us / 1e6, 1), of_bf16=round(flops / us / 1e6 / pk["bf16_tflops"], 3))
        print(json.dumps(rec), flush=True)

    err = torch.zeros(1, dtype=torch.int32, device=dev)
    for label, lens, ctxlen in (("prompt", [args.prefill_tokens], args.prefill_tokens), ("decode", [1] * args.batch, args.context)):
        T, B = sum(lens), len(lens)
        start = [0]
        for n in lens:
            start.append(start[-1] + n)
        pages = -(-ctxlen // 64)
        pos0 = torch.zeros(B, dtype=torch.int32, device=dev) if T != B else torch.full((B,), ctxlen - 1, dtype=torch.int32, device=dev)
        c = SimpleNamespace(
            seq_start=torch.tensor(start, dtype=torch.int32, device=dev),
            tok_seq=torch.repeat_interleave(torch.arange(B, dtype=torch.int32, device=dev), torch.tensor(lens, device=dev)).int(),
            slots=torch.arange(B, dtype=torch.int32, device=dev), n_seqs=B, max_new=max(lens), seq_pos0=pos0, is_decode=T == B,
            tok_pos=(torch.arange(T, dtype=torch.int32, device=dev) if T != B else pos0.clone()))
        n_sets = 4 if T > 64 else 24
        table = torch.arange(B * pages, dtype=torch.int32, device=dev).view(B, pages).contiguous()
        kp = torch.randn(B * pages + 1, G, 64, D, device=dev).to(dt)
        vp = torch.randn(B * pages + 1, G, 64, D, device=dev).to(dt)
        q = torch.randn(T, H * D, device=dev).to(dt)
        o = torch.empty(T, H * D, dtype=dt, device=dev)
        sink = torch.zeros(H, device=dev)
        # ---- attention with capped scores and a sink per head, beside the same kernel without either
        if T != B:
            seen = T * (T + 1) // 2
            for cap, sk, name, like in ((30.0, sink, "cap and sinks", None), (None, None, "plain", "cap and sinks")):
                us = timed(lambda i: ks.prefill_attention_tc.attn(q, o, c.seq_start, c.seq_pos0, table, kp, vp, B, T, H, G, D, 0, D ** -0.5,
                                                                  err, cap, sk), 1)
                report(f"attn_prefill {H}/{G} heads of {D}, {name} ({label})", T, us, flops=4 * H * D * seen, like=like)
        else:
            n_split = ks.decode.attention_splits(B, H, G, D, pages, sms)
            scratch = torch.empty(B * H * n_split * (D + 2), dtype=torch.float32, device=dev)
            tickets = torch.zeros(B * G, dtype=torch.int32, device=dev)
            us = timed(lambda i: ks.decode.attn_decode_capped(q, o, c.seq_pos0, table, kp, vp, scratch, tickets, B, H, G, D, 0, D ** -0.5,
                                                              n_split, 30.0, sink), 1)
            report(f"attn_decode {H}/{G} heads of {D}, cap and sinks, {n_split} splits ({label})", T, us, nbytes=B * ctxlen * G * 2 * D * esz)
            us = timed(lambda i: ks.decode.attn_decode(q, o, c.seq_pos0, table, kp, vp, scratch, B, H, G, D, 0, D ** -0.5, n_split,
                                                       tickets=tickets), 1)
            report(f"attn_decode {H}/{G} heads of {D}, plain, {n_split} splits ({label})", T, us, nbytes=B * ctxlen * G * 2 * D * esz,
                   like="cap and sinks")
        # ---- a latent layer's prompt from position 0, keys and values formed per head (192 and 128 wide): the mma.sync kernel for
        # unequal widths beside the float32 tiled kernel on the same rows
        if T != B:
            hw = z["dim"] + z["rot_dim"]
            widths = ks.prefill_attention_mma.widths_for(hw, z["vdim"])
            if widths is not None:
                hd = max(widths)
                kt = torch.randn(B * pages + 1, H, 64, hd, device=dev).to(dt)
                qt = torch.randn(T, H * hd, device=dev).to(dt)
                ot = torch.empty(T, H * hd, dtype=dt, device=dev)
                flops = 2 * H * (hw + z["vdim"]) * (T * (T + 1) // 2)
                us = timed(lambda i: ks.prefill_attention_mma.attn(qt, hd, ot, hd, c.seq_start, c.seq_pos0, table, kt, kt, B, T, H, H,
                                                                   widths[0], widths[1], 0, hw ** -0.5), 1)
                report(f"attn_prefill_mma {H} heads, keys {widths[0]}, values {widths[1]} ({label})", T, us, flops=flops)
                us = timed(lambda i: ks.attn_paged(qt, ot, c.seq_start, c.seq_pos0, table, kt, kt, B, T, H, H, hd, None, hw ** -0.5), 1)
                report(f"attn_paged {H} heads of {hd}, float32 tiles ({label})", T, us, flops=flops, like="attn_prefill_mma")
        # ---- the stream takes three addends at once, beside one addend
        xs = [torch.randn(T, W, device=dev) for _ in range(n_sets)]
        ad = [[torch.randn(2, T, W, device=dev), torch.randn(T, W, device=dev).to(dt), torch.randn(T, W, device=dev)] for _ in range(n_sets)]
        xb = torch.empty(T, W, dtype=dt, device=dev)
        us = timed(lambda i: ks.gate.add_list_cast(xs[i], ad[i], xb), n_sets)
        report(f"add_list_cast, three addends ({label})", T, us, nbytes=T * W * (8 + 8 + esz + 4 + esz))
        us = timed(lambda i: ks.gate.add_cast(xs[i], ad[i][0], xb), n_sets)
        report(f"add_cast, one addend in two parts ({label})", T, us, nbytes=T * W * (8 + 8 + esz), like="add_list_cast")
        # ---- x += y / rms(y) w (+ a row vector), then the norm without statistics; beside the same followed by an RMS norm
        w1, w2, b2, vec = (torch.randn(W, device=dev) for _ in range(4))
        out = torch.empty(T, W, dtype=dt, device=dev)
        us = timed(lambda i: ks.gate.add_rms_normed(xs[i], ad[i][0], w1, 1e-6, vec=vec, dyt=(w2, b2, 0.8, out)), n_sets)
        report(f"add_rms_normed + row vector + tanh norm ({label})", T, us, nbytes=T * W * (8 + 8 + esz))
        us = timed(lambda i: ks.gate.add_rms_normed(xs[i], ad[i][0], w1, 1e-6, norm=(w2, 1e-6, out)), n_sets)
        report(f"add_rms_normed + RMS norm ({label})", T, us, nbytes=T * W * (8 + 8 + esz), like="add_rms_normed + tanh norm")
        # ---- the embedding with a pair table, beside the plain one
        tab, ptab = torch.randn(DESIGN_VOCAB, W, device=dev).to(dt), torch.randn(100004, W, device=dev).to(dt)
        tok = torch.randint(0, DESIGN_VOCAB, (T,), dtype=torch.int32, device=dev)
        last = torch.zeros(B + 1, dtype=torch.int32, device=dev)
        us = timed(lambda i: ks.embed_pair_rows(tok, c, tab, ptab, 100003, 1009, 31, last, xs[i], err), n_sets)
        report(f"embed_pair_rows ({label})", T, us, nbytes=T * W * (2 * esz + 4))
        us = timed(lambda i: ks.embed_rows(tok, tab, xs[i], err), n_sets)
        report(f"embed_rows ({label})", T, us, nbytes=T * W * (esz + 4), like="embed_pair_rows")
        # ---- the gate per element, beside the gate per head
        gl = [torch.randn(T, H * D, device=dev).to(dt) for _ in range(n_sets)]
        us = timed(lambda i: ks.gate.head_gate(o, gl[i], H * D, 1), n_sets)
        report(f"head_gate per element ({label})", T, us, nbytes=3 * T * H * D * esz)
        us = timed(lambda i: ks.gate.head_gate(o, gl[i][:, :H], H, D), n_sets)
        report(f"head_gate per head ({label})", T, us, nbytes=2 * T * H * D * esz, like="per element")
        # ---- the router: softmax over all experts and groups rated by their best, beside the softmax over the picked
        zl = torch.randn(T, E, device=dev)
        idx = torch.empty(T, top, dtype=torch.int32, device=dev)
        wgt = torch.empty(T, top, device=dev)
        us = timed(lambda i: ks.mix.moe_route(zl, None, idx, wgt, z["n_groups"], z["keep"], top, 1.0, router="grouped_softmax"), 1)
        report(f"moe_route grouped_softmax, {top} of {E} in {z['n_groups']} groups ({label})", T, us)
        us = timed(lambda i: ks.mix.moe_route(zl, None, idx, wgt, 1, 1, top, 1.0, router="top_softmax"), 1)
        report(f"moe_route top_softmax, {top} of {E} ({label})", T, us, like="grouped_softmax")
        # ---- the dense feed-forward's first product with the clamped gate in its epilogue, beside the SiLU gate of the plain product
        if T > 128:
            xin = torch.randn(T, W, device=dev).to(dt)
            wgu = (torch.randn(2 * F, W, device=dev) * 0.02).to(dt)
            hid = torch.empty(T, F, dtype=dt, device=dev)
            group = torch.zeros(-(-T // 128), dtype=torch.int32, device=dev)
            us = timed(lambda i: ks.tensor_core.gemm_grouped(xin, wgu.unsqueeze(0), hid, group, err, glu=(7.0, 1.702)), 1)
            report(f"gate|up product with the clamped gate, {2 * F} x {W} ({label})", T, us, flops=4 * T * F * W)
            us = timed(lambda i: ks.tensor_core.gemm(xin, wgu, hid, err, swiglu=True), 1)
            report(f"gate|up product with the SiLU gate, {2 * F} x {W} ({label})", T, us, flops=4 * T * F * W, like="clamped gate")
    return 0


def kernel_alone(args):
    """One decode kernel by itself, as profiles/ quotes it: launched back to back in a CUDA graph over
    inputs that rotate through more bytes than L2 holds, timed with CUDA events; one JSON line per case.
    attn_decode: the decode attention of --shape for --batch sequences of --context keys, once per split
    count. gemm_small_m: the four products of a layer of --shape (and the head) with --batch rows."""
    import math
    import torch
    from scriptling_llm_lib_b200.csrc.bindings import DecodeKernels
    dk = DecodeKernels()
    cfg = dict(SHAPE if args.shape == "smollm2-1.7b" else OTHER_SHAPES[args.shape])
    H, G = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // H
    D, F, V, B = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], args.batch
    sms = torch.cuda.get_device_properties(0).multi_processor_count

    def timed(launch, n_sets, reps=24):
        torch.cuda.synchronize()          # the inputs were filled on the current stream; the launches run on another
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            for i in range(3):
                launch(i % n_sets)
            torch.cuda.synchronize()
            with torch.cuda.graph(graph, stream=side):
                for i in range(reps):
                    launch(i % n_sets)
        for _ in range(3):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(5):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (5 * reps) * 1e3

    if args.kernel == "attn_decode":
        pages = -(-args.context // 64)
        layer_bytes = B * pages * G * 64 * hd * 4
        n_sets = max(2, min(16, int(1.5e9 // layer_bytes)))
        ks = [torch.randn(B * pages, G, 64, hd, device="cuda").bfloat16() for _ in range(n_sets)]
        vs = [torch.randn(B * pages, G, 64, hd, device="cuda").bfloat16() for _ in range(n_sets)]
        table = torch.randperm(B * pages, device="cuda").int().view(B, pages).contiguous()
        pos0 = torch.full((B,), args.context - 1, dtype=torch.int32, device="cuda")
        q = torch.randn(B, H * hd, device="cuda").bfloat16()
        out = torch.empty(B, H * hd, dtype=torch.bfloat16, device="cuda")
        tickets = torch.zeros(B * G, dtype=torch.int32, device="cuda")
        chosen = dk.attention_splits(B, H, G, hd, pages, sms)
        for n in sorted({1, 2, 3, 4, 5, 6, 8, 12, 16, chosen}):
            if n > pages:
                continue
            scratch = torch.empty(B * H * n * (hd + 2), dtype=torch.float32, device="cuda")
            us = timed(lambda i: dk.attn_decode(q, out, pos0, table, ks[i], vs[i], scratch, B, H, G, hd, None,
                                                1.0 / math.sqrt(hd), n, tickets=tickets), n_sets)
            print(json.dumps({"kernel": "attn_decode", "shape": args.shape, "batch": B, "context": args.context, "splits": n,
                              "chosen": n == chosen, "blocks": n * G * B, "us": round(us, 1),
                              "tb_per_s": round(B * args.context * G * hd * 4 / us / 1e6, 2)}))
        return 0
    products = [("qkv", (H + 2 * G) * hd, D, False), ("o", D, H * hd, False), ("gate_up", 2 * F, D, True), ("down", D, F, False),
                ("head", V, D, False)]
    for name, N, K, gated in products:
        n_sets = max(2, int(600e6 // (N * K * 2)) + 1)
        ws = [torch.randn(N, K, device="cuda").bfloat16() for _ in range(n_sets)]
        x = torch.randn(B, K, device="cuda").bfloat16()
        if name in ("o", "down") and B <= dk.FOLD_MAX_M:
            # as the step runs them: the product adds to the residual stream and prepares the next norm
            resid = torch.zeros(B, N, dtype=torch.float32, device="cuda")
            fold = (torch.ones(N, dtype=torch.float32, device="cuda"), torch.empty(B, N, dtype=torch.bfloat16, device="cuda"),
                    torch.empty(-(-N // 16), B, dtype=torch.float32, device="cuda"))
            us = timed(lambda i: dk.gemm_small_m(x, ws[i], resid, fold=fold), n_sets)
            name += " (residual epilogue)"
        else:
            y = torch.empty(B, N // 2 if gated else N, dtype=torch.bfloat16, device="cuda")
            us = timed(lambda i: dk.gemm_small_m(x, ws[i], y, swiglu=gated), n_sets)
        print(json.dumps({"kernel": "gemm_small_m", "shape": args.shape, "product": name, "rows": B, "n": N, "k": K,
                          "blocks": -(-N // 16), "us": round(us, 1), "tb_per_s": round(N * K * 2 / us / 1e6, 2)}))
        del ws
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="smollm2-1.7b", choices=["smollm2-1.7b"] + sorted(OTHER_SHAPES),
                    help="layer sizes of the headline run (default: the SmolLM2-1.7B shape of the headline metric)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="precision of the headline run; float32 is the true 32-bit path")
    ap.add_argument("--layers", type=int, default=None,
                    help="run fewer layers of the same sizes (named in config as layers_run / layers_full)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--prefill-tokens", dest="prefill_tokens", type=int, default=PREFILL_TOKENS,
                    help="length of the one prompt of the prompt step (the headline metric's is 2,048)")
    ap.add_argument("--prompts", default=None, metavar="uniform:LO-HI",
                    help="a batch of unequal prompts, lengths uniform in LO..HI (seeded): one packed prompt step, then "
                         "decoding from there (instead of equal prompts that end at --context)")
    ap.add_argument("--no-points", action="store_true", help="skip decoding at batch 1 and 64")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-f32", dest="f32", action="store_false", help="skip the 32-bit path's measurements")
    ap.add_argument("--no-shapes", dest="shapes", action="store_false", help="skip the Llama-3.2-1B and Llama-3.1-8B sizes")
    ap.add_argument("--only", default="all", choices=["all", "prefill", "decode"],
                    help="run one part only (a small case to profile); the JSON line then holds that part alone")
    ap.add_argument("--kernel", default=None, choices=["attn_decode", "gemm_small_m", "sequence", "mix", "gate", "tufazen"],
                    help="time one decode kernel alone at --shape, --batch (and --context) instead of the model; 'sequence': "
                         "the kernels of the mixers with state at --design-sizes, for a prompt and for a decode step; 'mix': "
                         "the same for the kernels of latent attention, decayed linear attention, the selective scan and "
                         "routed experts; 'gate': the same for the kernels of the Belasun decoder's layers (convolution behind "
                         "the projections, whole-projection norm, gate per head, chunked attention, gated experts, token input); 'tufazen': "
                         "what the Tufazen decoder added (capped attention with sinks, sums of several addends, the normed addend "
                         "before a tanh norm, the pair-table embedding, the gate per element, the router over groups, the dense "
                         "clamped gate), each beside its like")
    ap.add_argument("--design", default=None, choices=sorted(DESIGNS),
                    help="measure this design's prompt step and decoding at a few real layer sizes beside the Llama decoder "
                         "of equal size (--prefill-tokens, --batch, --context, --steps, --dtype, --only apply) instead of the "
                         "headline run")
    ap.add_argument("--design-sizes", dest="design_sizes", default=None, help="comma-separated names out of DESIGN_SIZES")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference is a Go package (go.mod) with CPU-only code; "
                          "pip cannot install it and no Go toolchain is in the image"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": "this library runs on one GPU; bench.py measures N=1 only", "n_gpus": args.gpus}))
        return 2
    args.warmup = max(3, args.warmup)
    if args.kernel == "sequence":
        return sequence_kernels_alone(args)
    if args.kernel == "gate":
        return gate_kernels_alone(args)
    if args.kernel == "mix":
        return mix_kernels_alone(args)
    if args.kernel == "tufazen":
        return tufazen_kernels_alone(args)
    if args.kernel is not None:
        return kernel_alone(args)
    if args.design is not None:
        return design_compare(args)
    return run(args)


if __name__ == "__main__":
    sys.exit(main())
