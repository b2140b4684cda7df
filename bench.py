"""Serving benchmark on one B200: decode tokens per second of a Qwen3-8B-shaped model.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]

The default run has the layer sizes of the Qwen3-8B configuration (36 layers, hidden 4096, 32 query
and 8 key/value heads of 128, intermediate 12288, vocabulary 151936) with random bfloat16 weights,
a batch of 8 requests and 2,048 tokens of context each. A "step" is one decode step: one new token
for every request of the batch, from the embedding to the sampled token id. It prints one JSON line:
``value`` is decoded tokens per second timed on the device with CUDA events; ``e2e`` is the same
through the Python entry point (``GenerationEngine.step``: host token lists in, host token ids out,
the index arrays copied from pinned memory every step); ``prefill`` is one 2,048-token prompt in one
step; ``roofline`` is the decode step against the bytes it must read; ``points`` are decode at batch
1 and 64, at batch 8 with pages of 32 tokens, and two further sizes at their full depth (the Qwen3-0.6B shape under a
continuous-batching mix of 64 requests, decode at batch 8 at the Qwen3-32B shape). ``breakdown`` gives, for one decode step of the batch
and for the prefill step, the device time of every kernel class (CUDA events around every launch of
an eager step that is queued behind a sleeping kernel, so that launches do not wait for the host) with
the achieved GB/s of the weight-streaming products and the decode attention and the TFLOP/s of the
prefill products and attention, each over the measured peak (burst figure: kernels alone).
``baselines.plain_pytorch`` is this repository's plain PyTorch implementation (``tests/plain_qwen3.py``:
whole sequences, no cache) on the same GPU in bfloat16 at batch 1. ``selfcheck`` compares, outside any
timed region, the greedy tokens of steps of 8 and 64 requests on a two-layer model of the same widths
with the plain implementation. All weights and token ids are synthetic (seeded); the inputs are far
larger than L2, so no flush is needed between iterations.

``--compare zupilorn [--size 1k|2k]`` leaves the headline aside and puts the Zupilorn hybrid decoder (recurrent and
latent-attention mixers, dense and routed-expert feed-forwards) at real layer sizes beside a Qwen3 dense decoder of the
same width, depth and vocabulary: a 2,048-token prompt, decode at ``--batch`` requests of 2,048 tokens, and the device
time of every kernel class of both, in one JSON line of its own shape.

``--compare razelorn [--size 1k|2k]`` does the same for the Razelorn decoder (differential attention under a sliding
window beside a dense or routed-expert feed-forward on one layer norm).

``--compare tupidra [--size 1k|2k]`` does the same for the Tupidra decoder (a selective scan, capped window attention with
kept first tokens, latent attention with query latents, sinks, gates and shared rows, each beside a gated GELU
feed-forward behind norms and input filters of its own).
``--compare nufolix [--size 1k|2k]`` does the same for the Nufolix decoder (a state-space mixer; sigmoid attention with
mixed heads side by side with a gated delta rule; dense xIELU feed-forwards).

``--impl reference`` runs DavidAkinpelu/llm-pipeline's own ``Qwen3ForCausalLM`` from
``baseline/_ref`` (installed offline with pip --no-deps --target) with its ``past_key_values``
loop at the same sizes and prints the same line with ``"impl": "reference"``.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 36, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "attention_bias": False,
    "max_position_embeddings": 4096, "hidden_act": "silu",
}
QWEN3_0_6B = {**QWEN3_8B, "num_hidden_layers": 28, "hidden_size": 1024, "num_attention_heads": 16, "num_key_value_heads": 8,
              "intermediate_size": 3072, "tie_word_embeddings": True}
QWEN3_32B = {**QWEN3_8B, "num_hidden_layers": 64, "hidden_size": 5120, "num_attention_heads": 64, "num_key_value_heads": 8,
             "intermediate_size": 25600}
SHAPES = {"8b": ("Qwen3-8B shape", QWEN3_8B), "0.6b": ("Qwen3-0.6B shape", QWEN3_0_6B), "32b": ("Qwen3-32B shape", QWEN3_32B)}
CONTEXT = 2048
PREFILL_TOKENS = 2048
PAGE_SIZE = 16           # tokens per page of the key/value cache (--page-size)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                data = json.load(f)
            return {"hbm_gbs": float(data["hbm_gbs"]),
                    "bf16_tflops": float(data.get("bf16_tflops_sustained") or data["bf16_tflops"]),
                    "bf16_tflops_burst": float(data["bf16_tflops"]), "source": "measured"}
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_burst": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        clocks, reasons, max_clock = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.samples:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(int(float(parts[0])))
                max_clock = int(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None, "sm_max_mhz": max_clock,
                "reasons": sorted(reasons), "samples": len(clocks)}


def weight_bytes(cfg, layers, element=2):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    d, nq, nkv = cfg["head_dim"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    per_layer = H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I + 2 * H + 2 * d
    return (layers * per_layer + V * H + H) * element          # the layers, the output head and the final norm


def kv_bytes_per_token(engine):
    """Bytes the caches of all layers hold per token, from what the mixers ask of the cache manager."""
    return sum(pages.bytes_per_token(engine.dtype) for pages, _state in engine.model.cache_specs() if pages is not None)


def prefill_flops(cfg, layers, T):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    d, nq, nkv = cfg["head_dim"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    per_token = 2 * (H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I)
    attention = 4 * nq * d * T * (T + 1) / 2           # causal QK^T and PV
    return layers * (per_token * T + attention) + 2 * V * H


def build_ours(cfg, layers, batch_cap, dtype, tokens_per_request=CONTEXT + 256, pages=None, page_size=None, model=None):
    import torch

    from llm_pipeline_b200.config import resolve_config
    from llm_pipeline_b200.engine.generate import GenerationEngine
    from llm_pipeline_b200.models import build_model
    from llm_pipeline_b200.ops import build_library
    from llm_pipeline_b200.weights import random_tensors

    build_library()
    page_size = page_size or PAGE_SIZE
    config = resolve_config({**cfg, "num_hidden_layers": layers})
    if model is None:
        model = build_model(config)
        model.load(random_tensors(config, seed=0, dtype=dtype, device="cuda:0"), torch.device("cuda:0"), dtype)
    if pages is None:
        pages = batch_cap * (-(-tokens_per_request // page_size))
    engine = GenerationEngine(model, config, page_size=page_size, num_pages=pages, max_num_seqs=batch_cap,
                              max_num_batched_tokens=PREFILL_TOKENS, max_model_len=tokens_per_request)
    return engine


def random_prompts(vocab, count, length, seed):
    import torch

    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (count, length), generator=gen).tolist()


def time_decode(engine, batch, steps, warmup, seed, e2e=True, contexts=None):
    """Device-timed decode steps through the step function, and wall-clock steps through
    ``GenerationEngine.step`` (host lists in and out). Returns a dict of figures. ``contexts``: the
    requests' context lengths when they are not all CONTEXT (device-timed part only)."""
    import torch

    from llm_pipeline_b200.engine import StepEntry
    from llm_pipeline_b200.ops import kernels
    from llm_pipeline_b200.sampling import SamplingConfig

    vocab = engine.model.spec.vocab_size
    if contexts is None:
        prompts = random_prompts(vocab, batch, CONTEXT - 1, seed)
    else:
        prompts = [random_prompts(vocab, 1, n - 1, seed + i)[0] for i, n in enumerate(contexts)]
    runner = engine.runner
    ids = [f"bench{seed}_{i}" for i in range(batch)]
    # fill the cache: every request gets its context less one token, in portions of up to 2,048 tokens
    for rid, prompt in zip(ids, prompts):
        for at in range(0, len(prompt), PREFILL_TOKENS):
            runner.step([StepEntry(rid, prompt[at:at + PREFILL_TOKENS], [])])
    last = [p[-1] for p in prompts]
    outs = [torch.empty(batch, dtype=torch.int32, device=engine.device) for _ in range(2)]

    # As the engine steps: the ids a step samples stay on the device, where the next step takes them from
    # (``StepEntry.device_token``); the host reads them a step late (the end-to-end figure below has that read in it).
    def one_step(k, before):
        if before is None:
            entries = [StepEntry(rid, [t], [0]) for rid, t in zip(ids, last)]
        else:
            entries = [StepEntry(rid, [0], [0], None, (before, i)) for i, rid in enumerate(ids)]
        return kernels.argmax(runner.step(entries), outs[k & 1])

    tokens = None
    for k in range(warmup):
        tokens = one_step(k, tokens)
    torch.cuda.synchronize()
    launches_before = kernels.launch_count
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for k in range(warmup, warmup + steps):
        tokens = one_step(k, tokens)
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / steps
    launches = kernels.launch_count - launches_before
    h2d = runner.last_h2d_bytes
    for rid in ids:
        runner.release(rid)
    if not e2e:
        return {"ms": ms, "tok_s": batch * 1e3 / ms, "launches": launches, "h2d": h2d}

    # end to end: the public entry point, requests in as host token lists, tokens out as host ints
    greedy = SamplingConfig(temperature=0.0)
    e2e_prompts = random_prompts(vocab, batch, CONTEXT - 1, seed + 1)
    for p in e2e_prompts:
        engine.add_request(p, max_tokens=warmup + steps + 2 * batch + 16, sampling=greedy, ignore_eos=True)
    while any(r.num_pending > 1 or not r.output for r in engine.scheduler.running) or engine.scheduler.waiting:
        engine.step()                            # prompts, portion by portion
    for _ in range(8):
        engine.step()                            # set-up: the first decode steps of a shape run eagerly, then are captured
    for _ in range(warmup):
        engine.step()                            # the untimed warm-up steps
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / steps
    e2e_h2d = runner.last_h2d_bytes
    while engine.has_unfinished():
        engine.step()
    return {"ms": ms, "tok_s": batch * 1e3 / ms, "launches": launches, "h2d": h2d,
            "e2e_ms": e2e_ms, "e2e_tok_s": batch * 1e3 / e2e_ms, "e2e_h2d": e2e_h2d, "e2e_d2h": batch * 4}


def time_prefill(engine, tokens, repeats, warmup):
    import torch

    from llm_pipeline_b200.engine import StepEntry

    vocab = engine.model.spec.vocab_size
    runner = engine.runner
    times = []
    for i in range(warmup + repeats):
        prompt = random_prompts(vocab, 1, tokens, 500 + i)[0]
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        runner.step([StepEntry("prefill", prompt, [tokens - 1])])
        stop.record()
        torch.cuda.synchronize()
        runner.release("prefill")
        if i >= warmup:
            times.append(start.elapsed_time(stop))
    times.sort()
    return times[len(times) // 2]


def product_labels(cfg):
    """Names the matrix products of a step after what they are in this model (for ``ops.timing.KernelTimes``)."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    qkv = q + 2 * cfg["num_key_value_heads"] * cfg["head_dim"]

    def label(name, work):
        if work is None:
            return name
        _M, N, K = work
        kind = ("product_head" if N == V else "product_gate_up" if N == 2 * I else "product_qkv" if N == qkv and K == H
                else "product_down" if N == H and K == I else "product_o" if N == H and K == q else "product_other")
        return (kind + ("+swiglu" if name.endswith("+swiglu") else "") + (" (library)" if name == "mm" else "") +
                (" (library, into the residual)" if name == "mm+residual" else ""))
    return label


def breakdown_summary(table, peak, attention_bytes=0.0, attention_flops=0.0):
    """Per class: launches, microseconds, and for the products and the attention kernels what they achieved over the
    measured peak (GB/s of the bytes they must read when the rows are few, TFLOP/s otherwise)."""
    out = {}
    total = sum(e["us"] for e in table.values())
    for label, e in table.items():
        row = {"launches": e["launches"], "us": round(e["us"], 1), "share": round(e["us"] / total, 3)}
        seconds = e["us"] * 1e-6
        if label == "decode_attention" and attention_bytes:
            e["bytes"], e["rows"] = attention_bytes, 1
        if label == "paged_attention" and attention_flops:
            e["flops"], e["rows"] = attention_flops, 1 << 20
        if e["bytes"] and e["rows"] <= 64:
            row["gbs"] = round(e["bytes"] / seconds / 1e9, 1)
            row["frac_hbm"] = round(e["bytes"] / seconds / 1e9 / peak["hbm_gbs"], 3)
        elif e["flops"]:
            row["tflops"] = round(e["flops"] / seconds / 1e12, 1)
            row["frac_bf16_burst"] = round(e["flops"] / seconds / 1e12 / peak["bf16_tflops_burst"], 3)
        out[label] = row
    return {"kernel_us": round(total, 1), "classes": out}


def breakdown_of_a_step(engine, cfg, peak, entries_of, attention_bytes=0.0, attention_flops=0.0, release=()):
    """One eager step (no graph) with events around every launch, queued behind a sleeping kernel."""
    import torch

    runner = engine.runner
    graphs, runner.use_graphs = runner.use_graphs, False
    try:
        runner.step(entries_of(0))                      # untimed: first-call set-up of every kernel of the shape
        torch.cuda.synchronize()
        from llm_pipeline_b200.ops.timing import KernelTimes
        times = KernelTimes(product_labels(cfg))
        torch.cuda._sleep(int(1.5e8))                   # some 80 ms at the SM clock: the whole step queues up behind it
        with times:
            runner.step(entries_of(1))
        torch.cuda.synchronize()
    finally:
        runner.use_graphs = graphs
        for rid in release:
            runner.release(rid)
    return breakdown_summary(times.table(), peak, attention_bytes, attention_flops)


def decode_breakdown(engine, cfg, peak, batch):
    import torch

    from llm_pipeline_b200.engine import StepEntry

    vocab = engine.model.spec.vocab_size
    prompts = random_prompts(vocab, batch, CONTEXT - 2, 77)
    ids = [f"breakdown{i}" for i in range(batch)]
    for rid, prompt in zip(ids, prompts):
        engine.runner.step([StepEntry(rid, prompt, [])])
    layers = len(engine.model.schedule)
    kv_bytes = batch * CONTEXT * kv_bytes_per_token(engine)
    out = breakdown_of_a_step(engine, cfg, peak, lambda k: [StepEntry(rid, [p[k]], [0]) for rid, p in zip(ids, prompts)],
                              attention_bytes=kv_bytes, release=ids)
    out["launches_per_step"] = sum(c["launches"] for c in out["classes"].values())
    out["layers"] = layers
    return out


def prefill_breakdown(engine, cfg, peak, tokens):
    from llm_pipeline_b200.engine import StepEntry

    vocab = engine.model.spec.vocab_size
    prompts = random_prompts(vocab, 2, tokens, 88)
    layers = len(engine.model.schedule)
    flops = layers * 4.0 * cfg["num_attention_heads"] * cfg["head_dim"] * tokens * (tokens + 1) / 2
    runner = engine.runner

    def entries(k):
        if k:
            runner.release("prefill_breakdown")
        return [StepEntry("prefill_breakdown", prompts[k], [tokens - 1])]

    return breakdown_of_a_step(engine, cfg, peak, entries, attention_flops=flops, release=["prefill_breakdown"])


def plain_baseline(cfg, layers, tokens):
    """This repository's plain PyTorch implementation (tests/plain_qwen3.py: whole sequences, no cache, library
    products) in bfloat16 on the GPU with the same seeded weights: the time of one forward over ``tokens`` tokens, which
    is its prefill and, having no cache, also what one more decoded token costs it at that context."""
    import torch

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import plain_qwen3 as plain

    from llm_pipeline_b200.config import resolve_config
    from llm_pipeline_b200.weights import random_tensors

    config_json = {**cfg, "num_hidden_layers": layers}
    source = random_tensors(resolve_config(config_json), seed=0, dtype=torch.bfloat16, device="cuda:0")
    weights = {name: source.get(name) for name in source.names()}
    ids = random_prompts(cfg["vocab_size"], 1, tokens, 99)[0]
    times = []
    with torch.no_grad():
        for i in range(5):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            logits = plain.forward_logits(config_json, weights, ids, dtype=torch.bfloat16, rows=[tokens - 1])
            token = int(logits[0].argmax())
            stop.record()
            torch.cuda.synchronize()
            if i >= 2:
                times.append(start.elapsed_time(stop))
    del weights, logits
    torch.cuda.empty_cache()
    ms = sorted(times)[len(times) // 2]
    return {"what": "tests/plain_qwen3.py, bfloat16, whole sequence per token (no cache)", "context": tokens, "layers": layers,
            "ms_per_forward": round(ms, 3), "decode_b1": round(1e3 / ms, 2), "prefill": round(tokens * 1e3 / ms, 1), "last_token": token}


def selfcheck(cfg, batches=(8, 64), prompt_tokens=48, new_tokens=4):
    """Outside every timed region: a two-layer model of the benchmark's widths generates greedily through the Python
    entry point in steps of 8 and of 64 requests (the fused streaming products, the library products and both decode
    attention streams), and every generated token must be the plain implementation's greedy choice at its place, or
    lose to it by less than the bfloat16 rounding noise of these logits (0.25 on logits that reach 7)."""
    import torch

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import plain_qwen3 as plain

    from llm_pipeline_b200.weights import random_tensors

    torch.backends.cuda.matmul.allow_tf32 = False
    engine = build_ours(cfg, 2, max(batches), torch.bfloat16, tokens_per_request=256)
    config_json = {**cfg, "num_hidden_layers": 2}
    source = random_tensors(engine.config, seed=0, dtype=torch.bfloat16, device="cuda:0")
    weights = {name: source.get(name).float() for name in source.names()}
    report = {}
    for batch in batches:
        prompts = random_prompts(cfg["vocab_size"], batch, prompt_tokens, 4000 + batch)
        results = engine.generate(prompts, max_tokens=new_tokens, temperature=0.0, ignore_eos=True)
        equal = close = wrong = 0
        for prompt, result in zip(prompts, results):
            ids = list(prompt) + list(result.token_ids)
            rows = list(range(len(prompt) - 1, len(ids) - 1))
            logits = plain.forward_logits(config_json, weights, ids, rows=rows)
            for row, token in zip(logits, result.token_ids):
                best = int(row.argmax())
                if best == token:
                    equal += 1
                elif float(row[best] - row[token]) < 0.25:
                    close += 1
                else:
                    wrong += 1
        report[f"batch_{batch}"] = {"tokens": batch * new_tokens, "equal": equal, "within_rounding": close, "wrong": wrong}
    del engine, weights
    torch.cuda.empty_cache()
    report["ok"] = all(r["wrong"] == 0 and r["equal"] >= 0.9 * r["tokens"] for r in report.values() if isinstance(r, dict))
    return report


def mix_workload(cfg, layers):
    """A continuous-batching mix through the Python entry point: 64 requests with prompt lengths uniform in
    [16, 2048] and 128 decoded tokens each (seeded), context up to 4,096; returns its figures."""
    import torch

    from llm_pipeline_b200.sampling import SamplingConfig

    engine = build_ours(cfg, layers, 64, torch.bfloat16, tokens_per_request=2048 + 128 + 16)
    gen = torch.Generator().manual_seed(7)
    lengths = torch.randint(16, 2049, (64,), generator=gen).tolist()
    prompts = [random_prompts(cfg["vocab_size"], 1, n, 1000 + i)[0] for i, n in enumerate(lengths)]
    greedy = SamplingConfig(temperature=0.0)
    warm = engine.generate([prompts[0][:64]], max_tokens=4, temperature=0.0)      # builds kernels' first-call state
    del warm
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for p in prompts:
        engine.add_request(p, max_tokens=128, sampling=greedy, ignore_eos=True)
    steps = 0
    while engine.has_unfinished():
        engine.step()
        steps += 1
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    total = sum(lengths) + 64 * 128
    stats = engine.stats()
    del engine
    torch.cuda.empty_cache()
    return {"requests": 64, "prompt_tokens": sum(lengths), "decoded_tokens": 64 * 128, "seconds": round(seconds, 3),
            "tokens_per_s": round(total / seconds, 1), "decoded_tokens_per_s": round(64 * 128 / seconds, 1), "steps": steps,
            "mean_step_ms": round(seconds * 1e3 / steps, 3), "preemptions": stats["preemptions"]}


def run_mix(args):
    name, cfg = SHAPES[args.shape]
    layers = args.layers or cfg["num_hidden_layers"]
    print(json.dumps({"workload": "mix", "model": name, "layers": layers, **mix_workload(cfg, layers)}))
    return 0


def further_points(args):
    """Other sizes through the same engine, each at its full depth: the Qwen3-0.6B shape under the continuous-batching
    mix (total tokens per second through the Python entry point), and decode at batch 8 and 2,048 tokens of context
    at the Qwen3-32B shape (65 GB of weights)."""
    import torch

    out = {}
    _name, small = SHAPES["0.6b"]
    out["qwen3_0.6b_mix_64_requests"] = mix_workload(small, small["num_hidden_layers"])["tokens_per_s"]
    _name, large = SHAPES["32b"]
    engine = build_ours(large, large["num_hidden_layers"], 8, torch.bfloat16)
    r = time_decode(engine, 8, 8, args.warmup, seed=40, e2e=False)
    out["qwen3_32b_decode_b8"] = round(r["tok_s"], 1)
    step_bytes = weight_bytes(large, large["num_hidden_layers"]) + 8 * (CONTEXT + args.warmup + 4) * kv_bytes_per_token(engine)
    out["qwen3_32b_decode_b8_gbs"] = round(step_bytes / (r["ms"] * 1e-3) / 1e9, 1)
    del engine
    torch.cuda.empty_cache()
    return out


def run_ours(args):
    import torch

    if args.workload == "mix":
        return run_mix(args)
    name, cfg = SHAPES[args.shape]
    layers = args.layers or cfg["num_hidden_layers"]
    peak = peaks()
    dtype = torch.bfloat16
    # room per request: the context, the set-up, warm-up and timed decode steps, in whole pages
    room = -(-(CONTEXT + 64 + args.warmup + args.steps) // 256) * 256
    contexts = [int(n) for n in args.contexts.split(",")] if args.contexts else None
    if contexts:
        if args.only != "decode":
            print("--contexts goes with --only decode")
            return 2
        args.batch = len(contexts)
        longest = -(-(max(contexts) + 64 + args.warmup + args.steps) // 256) * 256
        pages = sum(-(-(n + 64 + args.warmup + args.steps) // PAGE_SIZE) for n in contexts)
        engine = build_ours(cfg, layers, args.batch, dtype, tokens_per_request=longest, pages=pages)
    else:
        engine = build_ours(cfg, layers, max(64, args.batch), dtype, tokens_per_request=max(CONTEXT + 256, room))
    clocks = ClockSampler()
    clocks.start()
    if args.only == "prefill":
        clocks.stop()
        prefill_ms = time_prefill(engine, PREFILL_TOKENS, repeats=2, warmup=3)
        print(json.dumps({"only": "prefill", "layers": layers, "prefill_ms": round(prefill_ms, 3)}))
        return 0
    main = time_decode(engine, args.batch, args.steps, args.warmup, seed=1, e2e=args.only == "all", contexts=contexts)
    clock_info = clocks.stop()
    if args.only == "decode":
        line = {"only": "decode", "layers": layers, "batch": args.batch, "ms_per_step": round(main["ms"], 4)}
        if contexts:
            line["contexts"] = args.contexts
        print(json.dumps(line))
        return 0
    points = {}
    for b in (1, 64):
        r = time_decode(engine, b, max(5, args.steps // 2), args.warmup, seed=10 + b, e2e=False)
        points[f"decode_b{b}"] = round(r["tok_s"], 1)
    prefill_ms = time_prefill(engine, PREFILL_TOKENS, repeats=5, warmup=3)
    flops = prefill_flops(cfg, layers, PREFILL_TOKENS)
    kv_per_token = kv_bytes_per_token(engine)
    breakdown = baselines = check = None
    if not args.lean:
        breakdown = {f"decode_b{args.batch}": decode_breakdown(engine, cfg, peak, args.batch),
                     f"prefill_{PREFILL_TOKENS}": prefill_breakdown(engine, cfg, peak, PREFILL_TOKENS)}
        # the same batch with pages of 32 tokens (half as many TMA boxes in the decode attention stream)
        other_page = 32 if PAGE_SIZE != 32 else 16
        wide = build_ours(cfg, layers, max(64, args.batch), dtype, tokens_per_request=max(CONTEXT + 256, room), page_size=other_page,
                          model=engine.model)
        r = time_decode(wide, args.batch, max(5, args.steps // 2), args.warmup, seed=30, e2e=False)
        points[f"decode_b{args.batch}_page{other_page}"] = round(r["tok_s"], 1)
        del wide
        del engine
        torch.cuda.empty_cache()
        baselines = {"plain_pytorch": plain_baseline(cfg, layers, CONTEXT)}
        check = selfcheck(cfg)
        if args.shape == "8b" and not args.layers:
            points.update(further_points(args))
    step_bytes = weight_bytes(cfg, layers) + args.batch * (CONTEXT + args.warmup + args.steps // 2) * kv_per_token
    achieved = step_bytes / (main["ms"] * 1e-3) / 1e9
    line = {
        "metric": f"decode tok/s at batch {args.batch}, 2,048-token context ({name.split()[0]} bf16)",
        "value": round(main["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (seeded random weights and token ids)", "impl": "ours",
        "config": {"model": name, "layers": layers, "layers_of_model": cfg["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": args.batch,
                   "seq_len": CONTEXT, "page_size": PAGE_SIZE, "parallelism": "single GPU",
                   "l2": "inputs larger than L2, no flush", "peaks": peak["source"]},
        "e2e": {"value": round(main["e2e_tok_s"], 1), "unit": "tokens/s", "ms_per_step": round(main["e2e_ms"], 4),
                "h2d_bytes_per_step": main["e2e_h2d"], "d2h_bytes_per_step": main["e2e_d2h"]},
        "gpu_launches": main["launches"],
        "prefill": {"value": round(PREFILL_TOKENS * 1e3 / prefill_ms, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4),
                    "frac_burst": round(flops / (prefill_ms * 1e-3) / (peak["bf16_tflops_burst"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4)},
        "points": points,
        "clocks": clock_info,
    }
    if breakdown is not None:
        line["breakdown"] = breakdown
        line["baselines"] = baselines
        line["selfcheck"] = check
    print(json.dumps(line))
    return 0 if check is None or check["ok"] else 1


# ---- another design beside the closest existing one ------------------------------------------------------------------
# ``--compare zupilorn``: prefill (one 2,048-token prompt) and decode (batch 8, 2,048 tokens of context) of the Zupilorn
# hybrid decoder (recurrent and latent-attention mixers, PolyNorm and routed-expert feed-forwards) at layer sizes of real
# models, beside a Qwen3 dense decoder of the same width, depth and vocabulary on the same GPU, with the device time of
# every kernel class and, where the work of a class is known in closed form, what it achieved over the measured peak.
ZUPILORN_SIZES = {
    "1k": {"width": 1024, "gru": 2048, "ff": 4096, "heads": 8, "dim": 64, "rot": 32, "vdim": 64, "rank": 256,
           "experts": 16, "top": 2, "expert_ff": 1024, "layers": 4, "vocab": 32000, "qwen_heads": (8, 4)},
    "2k": {"width": 2048, "gru": 4096, "ff": 8192, "heads": 16, "dim": 128, "rot": 64, "vdim": 128, "rank": 512,
           "experts": 32, "top": 4, "expert_ff": 1408, "layers": 4, "vocab": 32000, "qwen_heads": (16, 8)},
}


def zupilorn_config(z):
    layers = []
    for i in range(z["layers"]):
        if i % 2 == 0:
            layers.append({"type": "mingru", "mixer": {"width": z["gru"]}, "mlp": {"kind": "dense", "ff": z["ff"]}})
        else:
            layers.append({"type": "latent_attention",
                           "mixer": {"heads": z["heads"], "dim": z["dim"], "rot_dim": z["rot"], "vdim": z["vdim"], "kv_rank": z["rank"],
                                     "scale": (z["dim"] + z["rot"]) ** -0.5, "rot": {"base": 10000.0, "dims": z["rot"]}},
                           "mlp": {"kind": "moe", "expert": {"ff": z["expert_ff"], "limit": 7.0},
                                   "router": {"experts": z["experts"], "top": z["top"]}}})
    return {"architecture": "Zupilorn", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5}, "logit_softcap": 30.0,
            "layers": layers}


def qwen_config_like(z):
    heads, kv = z["qwen_heads"]
    return {**QWEN3_8B, "num_hidden_layers": z["layers"], "hidden_size": z["width"], "num_attention_heads": heads,
            "num_key_value_heads": kv, "head_dim": 128, "intermediate_size": z["ff"], "vocab_size": z["vocab"]}


def zupilorn_work(z, tokens, keys_per_token, decode):
    """Closed-form work of the design's own kernel classes for one step: label -> (bytes, flops). ``tokens`` rows in the
    step, each seeing ``keys_per_token`` keys on average."""
    D, L = z["width"], z["layers"]
    gru_layers, att_layers = (L + 1) // 2, L // 2
    dk = z["rank"] + z["rot"]
    work = {}
    # per layer three folds of the stream (before the mixer, between, and with the depth mix at the next reader)
    mix_reads = sum(i + 1 for i in range(L))
    work["add_norm_mix"] = (tokens * D * (3 * L * (4 + 4 + 4 + 2) + 4 * mix_reads + 4 * L), 0.0)
    work["min_gru"] = (gru_layers * tokens * z["gru"] * ((12 if decode else 24) + 2), 0.0)
    work["poly_norm"] = (gru_layers * tokens * z["ff"] * (4 + 4 + 2), 0.0)
    if decode:
        work["latent_attention_mma"] = (att_layers * tokens * keys_per_token * dk * 2, 0.0)
    else:
        work["latent_attention_mma"] = (0.0, att_layers * 2.0 * tokens * keys_per_token * z["heads"] * (dk + z["rank"]))
    pairs = tokens * z["top"]
    expert_weights = 3 * z["expert_ff"] * D * 2
    if decode:
        work["expert_rows"] = (att_layers * pairs * expert_weights, 0.0)
    else:
        work["expert_rows"] = (0.0, att_layers * 2.0 * pairs * 3 * z["expert_ff"] * D)
    work["expert_grouped"] = work["expert_rows"]
    return work


def qwen_work(cfg, tokens, keys_per_token, decode):
    D, L, I = cfg["hidden_size"], cfg["num_hidden_layers"], cfg["intermediate_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    work = {"add_rmsnorm": (tokens * D * (2 * L + 1) * (4 + 4 + 2 + 2), 0.0), "swiglu": (L * tokens * I * 6, 0.0),
            "qkv_post": (L * tokens * (nq + 2 * nkv) * d * 6, 0.0)}
    if decode:
        work["decode_attention"] = (L * tokens * keys_per_token * 2 * nkv * d * 2, 0.0)
    else:
        work["paged_attention"] = (0.0, L * 4.0 * tokens * keys_per_token * nq * d)
    return work


def compare_one(cfg_json, work_of, peak, args, label=None):
    import torch

    from llm_pipeline_b200.config import resolve_config
    from llm_pipeline_b200.engine import StepEntry
    from llm_pipeline_b200.engine.generate import GenerationEngine
    from llm_pipeline_b200.models import build_model
    from llm_pipeline_b200.ops import build_library
    from llm_pipeline_b200.ops.timing import KernelTimes
    from llm_pipeline_b200.weights import random_tensors

    build_library()
    config = resolve_config(cfg_json)
    model = build_model(config)
    model.load(random_tensors(config, seed=0, dtype=torch.bfloat16, device="cuda:0"), torch.device("cuda:0"), torch.bfloat16)
    room = -(-(CONTEXT + 64 + args.warmup + args.steps) // 256) * 256
    engine = GenerationEngine(model, config, page_size=PAGE_SIZE, num_pages=(args.batch + 1) * (room // PAGE_SIZE),
                              max_num_seqs=args.batch + 1, max_num_batched_tokens=PREFILL_TOKENS, max_model_len=room)
    out = {}
    prefill_ms = time_prefill(engine, PREFILL_TOKENS, repeats=3, warmup=3)
    out["prefill"] = {"tokens": PREFILL_TOKENS, "ms": round(prefill_ms, 3), "tok_s": round(PREFILL_TOKENS * 1e3 / prefill_ms, 1)}
    dec = time_decode(engine, args.batch, args.steps, args.warmup, seed=7, e2e=False)
    out["decode"] = {"batch": args.batch, "context": CONTEXT, "ms_per_step": round(dec["ms"], 4), "tok_s": round(dec["tok_s"], 1)}

    def kernel_table(entries_of, work, release):
        runner = engine.runner
        graphs, runner.use_graphs = runner.use_graphs, False
        try:
            runner.step(entries_of(0))
            torch.cuda.synchronize()
            times = KernelTimes(label)
            torch.cuda._sleep(int(1.5e8))
            with times:
                runner.step(entries_of(1))
            torch.cuda.synchronize()
        finally:
            runner.use_graphs = graphs
            for rid in release:
                runner.release(rid)
        table = times.table()
        total = sum(e["us"] for e in table.values())
        rows = {}
        for name, e in table.items():
            row = {"launches": e["launches"], "us": round(e["us"], 1), "share": round(e["us"] / total, 3)}
            nbytes, flops = work.get(name, (e["bytes"] if e["rows"] and e["rows"] <= 64 else 0.0, e["flops"] if e["rows"] > 64 else 0.0))
            seconds = e["us"] * 1e-6
            if nbytes:
                row["gbs"] = round(nbytes / seconds / 1e9, 1)
                row["frac_hbm"] = round(nbytes / seconds / 1e9 / peak["hbm_gbs"], 3)
            elif flops:
                row["tflops"] = round(flops / seconds / 1e12, 1)
                row["frac_bf16_burst"] = round(flops / seconds / 1e12 / peak["bf16_tflops_burst"], 3)
            rows[name] = row
        return {"kernel_us": round(total, 1), "classes": rows}

    vocab = model.spec.vocab_size
    prompts = random_prompts(vocab, 2, PREFILL_TOKENS, 900)
    if not args.lean:
        out["prefill"]["kernels"] = kernel_table(lambda k: [StepEntry(f"p{k}", prompts[k], [PREFILL_TOKENS - 1])],
                                                 work_of(PREFILL_TOKENS, (PREFILL_TOKENS + 1) / 2, False), ("p0", "p1"))
        ids = [f"d{i}" for i in range(args.batch)]
        contexts = random_prompts(vocab, args.batch, CONTEXT - 2, 901)
        for rid, prompt in zip(ids, contexts):
            engine.runner.step([StepEntry(rid, prompt, [])])
        out["decode"]["kernels"] = kernel_table(lambda k: [StepEntry(rid, [5 + k], [0]) for rid in ids],
                                                work_of(args.batch, CONTEXT, True), ids)
    del engine, model
    torch.cuda.empty_cache()
    return out


# ``--compare razelorn``: the same two measurements for the Razelorn decoder: four layers (differential attention under a
# sliding window beside a squared-ReLU feed-forward, then beside routed experts with identity experts and a shared expert,
# then that layer's tensors once more, then a layer of its own again) beside a Qwen3 dense decoder of the same width, depth
# and vocabulary whose heads hold as many query and key entries.
RAZELORN_SIZES = {
    "1k": {"width": 1024, "heads": 8, "kv_heads": 2, "dim": 64, "vdim": 128, "window": 2048, "rot": 32, "ff": 4096,
           "experts": 16, "top": 2, "identity": 2, "expert_ff": 1024, "shared_ff": 1024, "layers": 4, "vocab": 32000, "qwen_heads": (8, 4)},
    "2k": {"width": 2048, "heads": 16, "kv_heads": 4, "dim": 64, "vdim": 128, "window": 2048, "rot": 64, "ff": 8192,
           "experts": 32, "top": 4, "identity": 2, "expert_ff": 1408, "shared_ff": 2048, "layers": 4, "vocab": 32000, "qwen_heads": (16, 8)},
}


def razelorn_config(z):
    mixer = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"], "scale": z["dim"] ** -0.5, "diff": 0.5,
             "mask": {"size": z["window"]},
             "rot": {"base": 10000.0, "dims": z["rot"], "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "router": {"experts": z["experts"], "top": z["top"], "identity": z["identity"]},
           "shared": {"ff": z["shared_ff"]}}
    layers = [{"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": z["ff"]}},
              {"type": "attention", "mixer": mixer, "mlp": moe}]
    while len(layers) < z["layers"]:
        own = len(layers) % 2 == 1
        layers.append({"type": "attention", "mixer": mixer, "mlp": moe, **({} if own else {"weights_of": 1})})
    return {"architecture": "Razelorn", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "layers": layers}


def razelorn_work(z, tokens, keys_per_token, decode):
    """Closed-form work of the design's own kernel classes for one step: label -> (bytes, flops)."""
    D, L = z["width"], z["layers"]
    H, G, d, dv = z["heads"], z["kv_heads"], z["dim"], z["vdim"]
    moe_layers, dense_layers = L - 1, 1
    keys = min(keys_per_token, z["window"])
    work = {}
    # per layer: residual read and written, two float32 addends read, the normed row written; the head's rows beside
    work["add_layernorm"] = (tokens * D * L * (4 + 4 + 4 + 4 + 2), 0.0)
    work["diff_qkv_post"] = (L * tokens * (2 * d * (H + G) + G * dv) * (2 + 2), 0.0)
    work["relu_squared"] = (dense_layers * tokens * z["ff"] * 4, 0.0)
    work["swiglu"] = (moe_layers * tokens * z["shared_ff"] * 6, 0.0)
    if decode:
        work["diff_attention_mma"] = (L * tokens * keys * G * (2 * d + dv) * 2, 0.0)
    else:
        work["diff_attention_mma"] = (0.0, L * 2.0 * tokens * keys * H * (2 * d + 2 * dv))
    pairs = tokens * z["top"] * z["experts"] / (z["experts"] + z["identity"])      # pairs that name an expert with matrices
    expert_weights = 3 * z["expert_ff"] * D * 2
    if decode:
        work["expert_rows"] = (moe_layers * pairs * expert_weights, 0.0)
    else:
        work["expert_rows"] = (0.0, moe_layers * 2.0 * pairs * 3 * z["expert_ff"] * D)
    work["expert_grouped"] = work["expert_rows"]
    return work


# ``--compare nufolix``: the same two measurements for the Nufolix decoder: four layers (a state-space mixer alone, then
# sigmoid attention with mixed heads side by side with a gated delta rule and a dense xIELU feed-forward, twice) beside a
# Qwen3 dense decoder of the same width, depth and vocabulary.
NUFOLIX_SIZES = {
    "1k": {"width": 1024, "ssd_heads": 16, "ssd_vdim": 128, "state": 64, "groups": 1, "norm_groups": 1, "conv": 4,
           "heads": 8, "kv_heads": 4, "dim": 128, "vdim": 128, "rot": 64, "delta_heads": 8, "delta_qk_heads": 8, "delta_dim": 64,
           "delta_vdim": 128, "ff": 4096, "layers": 4, "vocab": 32000, "qwen_heads": (8, 4)},
    "2k": {"width": 2048, "ssd_heads": 32, "ssd_vdim": 128, "state": 128, "groups": 1, "norm_groups": 1, "conv": 4,
           "heads": 16, "kv_heads": 4, "dim": 128, "vdim": 128, "rot": 64, "delta_heads": 16, "delta_qk_heads": 16, "delta_dim": 128,
           "delta_vdim": 128, "ff": 8192, "layers": 4, "vocab": 32000, "qwen_heads": (16, 8)},
}


def nufolix_config(z):
    ssd = {"heads": z["ssd_heads"], "vdim": z["ssd_vdim"], "state": z["state"], "groups": z["groups"], "conv": z["conv"],
           "norm_groups": z["norm_groups"]}
    side = {"left": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"], "scale": z["dim"] ** -0.5,
                     "softcap": 30.0, "rot": {"base": 10000.0, "dims": z["rot"]}},
            "right": {"heads": z["delta_heads"], "kv_heads": z["delta_qk_heads"], "dim": z["delta_dim"], "vdim": z["delta_vdim"],
                      "conv": z["conv"]},
            "left_scale": 1.0, "right_scale": 1.0}
    layers = []
    for i in range(z["layers"]):
        if i % 2 == 0:
            layers.append({"type": "mamba2", "mixer": ssd, "mlp": None})
        else:
            layers.append({"type": "parallel", "mixer": side, "mlp": {"kind": "dense", "ff": z["ff"]}})
    return {"architecture": "Nufolix", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5}, "residual_mult": 1.0,
            "embedding": {"scale": 1.0}, "layers": layers}


def nufolix_work(z, tokens, keys_per_token, decode, requests=1):
    """Closed-form work of the design's own kernel classes for one step: label -> (bytes, flops)."""
    L = z["layers"]
    ssd_layers, side_layers = (L + 1) // 2, L // 2
    Hs, P, Ns, Gs = z["ssd_heads"], z["ssd_vdim"], z["state"], z["groups"]
    H, G, d, dv = z["heads"], z["kv_heads"], z["dim"], z["vdim"]
    Hd, Gd, dd, ddv = z["delta_heads"], z["delta_qk_heads"], z["delta_dim"], z["delta_vdim"]
    ssd_channels = Hs * P + 2 * Gs * Ns
    delta_channels = 2 * Gd * dd + Hd * ddv
    work = {}
    # rows in and out in float32; the state of every request read and written once a step
    work["short_conv"] = ((ssd_layers * ssd_channels + side_layers * delta_channels) * tokens * 8, 0.0)
    work["ssd_scan"] = (ssd_layers * (tokens * (ssd_channels + Hs + Hs * P) * 4 + requests * Hs * Ns * P * 8), 0.0)
    work["delta_scan"] = (side_layers * (tokens * (delta_channels + Hd * dd + Hd + Hd * ddv) * 4 + requests * Hd * dd * ddv * 8), 0.0)
    work["delta_prep"] = (side_layers * tokens * (2 * Gd * dd + Hd * dd + Hd) * 8, 0.0)
    work["gated_group_norm"] = ((ssd_layers * Hs * P + side_layers * Hd * ddv) * tokens * (4 + 4 + 2), 0.0)
    work["sig_qkv_post"] = (side_layers * tokens * ((H + G) * d + G * dv) * (4 + 2), 0.0)
    work["xielu"] = (side_layers * tokens * z["ff"] * (4 + 2), 0.0)
    if decode:
        work["sigmoid_attention"] = (side_layers * tokens * keys_per_token * G * (d + dv) * 2, 0.0)
    else:
        work["sigmoid_attention"] = (0.0, side_layers * 2.0 * tokens * keys_per_token * H * (d + dv))
    work["sigmoid_attention_mma"] = work["sigmoid_attention"]
    return work


# ``--compare tupidra``: the same two measurements for the Tupidra decoder: four layers (a selective scan; capped window
# attention with kept first tokens; latent attention with query latents, sinks and gates; a latent attention layer that
# reads the third layer's rows), each beside a gated GELU feed-forward behind norms and input filters of its own, beside a
# Qwen3 dense decoder of the same width, depth and vocabulary.
TUPIDRA_SIZES = {
    "1k": {"width": 1024, "inner": 2048, "state": 16, "dt_rank": 64, "conv": 4, "taps": 4, "heads": 8, "kv_heads": 4, "dim": 128,
           "vdim": 128, "window": 1024, "keep": 8, "lat_heads": 8, "lat_dim": 64, "rot": 32, "lat_vdim": 64, "rank": 256, "q_rank": 384,
           "ff": 4096, "layers": 4, "vocab": 32000, "qwen_heads": (8, 4)},
    "2k": {"width": 2048, "inner": 4096, "state": 16, "dt_rank": 128, "conv": 4, "taps": 4, "heads": 16, "kv_heads": 4, "dim": 128,
           "vdim": 128, "window": 1024, "keep": 8, "lat_heads": 16, "lat_dim": 128, "rot": 64, "lat_vdim": 128, "rank": 512, "q_rank": 768,
           "ff": 8192, "layers": 4, "vocab": 32000, "qwen_heads": (16, 8)},
}


def tupidra_config(z):
    mlp = {"kind": "dense", "ff": z["ff"]}
    latent = {"heads": z["lat_heads"], "dim": z["lat_dim"], "rot_dim": z["rot"], "vdim": z["lat_vdim"], "kv_rank": z["rank"],
              "q_rank": z["q_rank"], "scale": (z["lat_dim"] + z["rot"]) ** -0.5,
              "rot": {"base": 10000.0, "dims": z["rot"], "scaling": {"factor": 8.0, "original": 4096, "fast": 16.0, "slow": 2.0}}}
    kinds = [{"type": "mamba1", "mixer": {"inner": z["inner"], "state": z["state"], "dt_rank": z["dt_rank"], "conv": z["conv"]}, "mlp": mlp},
             {"type": "attention", "mixer": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"],
                                             "scale": z["dim"] ** -0.5, "softcap": 30.0, "mask": {"size": z["window"], "keep_first": z["keep"]}},
              "mlp": mlp},
             {"type": "latent_attention", "mixer": latent, "mlp": mlp},
             {"type": "latent_attention", "mixer": {**latent, "kv_from": 2}, "mlp": mlp}]
    layers = [kinds[i % 4] if i % 4 != 3 else {**kinds[3], "mixer": {**latent, "kv_from": i - 1}} for i in range(z["layers"])]
    return {"architecture": "Tupidra", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5}, "canon": {"taps": z["taps"]},
            "layers": layers}


def tupidra_work(z, tokens, keys_per_token, decode, requests=1):
    """Closed-form work of the design's own kernel classes for one step: label -> (bytes, flops)."""
    D, L = z["width"], z["layers"]
    scan_layers, win_layers, lat_layers = (L + 3) // 4, (L + 2) // 4, (L + 1) // 4 + L // 4
    I, N, R = z["inner"], z["state"], z["dt_rank"]
    H, G, d, dv = z["heads"], z["kv_heads"], z["dim"], z["vdim"]
    dk = z["rank"] + z["rot"]
    work = {}
    # residual and two addends in and out in float32, two normed rows out in float32; the last norm reads a few rows only
    work["add_rmsnorm_multi"] = (L * tokens * D * (4 + 4 + 4 + 4 + 8), 0.0)
    # the layers' input filters (two float32 inputs in, two typed rows out) and the scan's own convolution (float32 in, float32 and typed out)
    work["short_conv"] = (L * tokens * 2 * D * (4 + 2) + scan_layers * tokens * I * (4 + 4 + 2), 0.0)
    work["selective_scan"] = (scan_layers * (tokens * (3 * I * 4 + 2 * N * 4 + I * 2) + requests * I * N * 8), 0.0)
    work["gated_act"] = (L * tokens * z["ff"] * (8 + 2), 0.0)
    work["capped_qkv_post"] = (win_layers * tokens * ((H + G) * d + G * dv) * (4 + 2), 0.0)
    work["latent_rows_post"] = (lat_layers * tokens * (z["lat_heads"] * (z["lat_dim"] + z["rot"]) + dk) * (4 + 2), 0.0)
    work["sigmoid_gate"] = (lat_layers * tokens * z["lat_heads"] * z["lat_vdim"] * (2 + 4 + 2), 0.0)
    seen = min(keys_per_token, z["window"] + z["keep"])
    if decode:
        work["capped_attention"] = (win_layers * tokens * seen * G * (d + dv) * 2, 0.0)
        work["latent_attention_mma"] = (lat_layers * tokens * keys_per_token * dk * 2, 0.0)
    else:
        work["capped_attention"] = (0.0, win_layers * 2.0 * tokens * seen * H * (d + dv))
        work["latent_attention_mma"] = (0.0, lat_layers * 2.0 * tokens * keys_per_token * z["lat_heads"] * (dk + z["rank"]))
    work["capped_attention_mma"] = work["capped_attention"]
    return work


def run_compare(args):
    peak = peaks()
    sizes, config_of, work_of = {"zupilorn": (ZUPILORN_SIZES, zupilorn_config, zupilorn_work),
                                 "razelorn": (RAZELORN_SIZES, razelorn_config, razelorn_work),
                                 "nufolix": (NUFOLIX_SIZES, nufolix_config, lambda z, n, k, d: nufolix_work(z, n, k, d, args.batch if d else 1)),
                                 "tupidra": (TUPIDRA_SIZES, tupidra_config, lambda z, n, k, d: tupidra_work(z, n, k, d, args.batch if d else 1))}[args.compare]
    z = sizes[args.size]
    clocks = ClockSampler()
    clocks.start()
    ours = compare_one(config_of(z), lambda n, k, d: work_of(z, n, k, d), peak, args)
    qcfg = qwen_config_like(z)
    beside = compare_one(qcfg, lambda n, k, d: qwen_work(qcfg, n, k, d), peak, args, product_labels(qcfg))
    print(json.dumps({"compare": args.compare, "size": args.size, "dtype": "bf16", "data": "synthetic (seeded random weights and token ids)",
                      "sizes": z, args.compare: ours, "qwen3_same_width_and_depth": beside, "peaks": peak, "clocks": clocks.stop()}))
    return 0


def run_reference(args):
    """The reference's own model class and cache loop, unmodified, from baseline/_ref."""
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "llm_pipeline")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed (pip --no-deps --target)"}))
        return 0
    sys.path.insert(0, ref_root)
    try:
        import torch
        from llm_pipeline.models.qwen3.custom_builder import Qwen3Config as RefConfig, Qwen3ForCausalLM
    except Exception as e:      # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"import failed: {type(e).__name__}: {e}"[:200]}))
        return 0
    cfg = dict(QWEN3_8B)
    layers = args.layers or cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = layers
    torch.manual_seed(0)
    with torch.device("cuda:0"):
        torch.set_default_dtype(torch.bfloat16)
        model = Qwen3ForCausalLM(RefConfig(**cfg)).eval()
        torch.set_default_dtype(torch.float32)
    for p in model.parameters():
        p.data.normal_(0, 0.02)
    batch = args.batch
    ids = torch.tensor(random_prompts(cfg["vocab_size"], batch, CONTEXT - 1, 1), device="cuda:0")
    clocks = ClockSampler()
    with torch.no_grad():
        out = model(input_ids=ids, use_cache=True)
        past = out.past_key_values
        token = out.logits[:, -1, :].argmax(-1, keepdim=True)

        def one_step(token, past):
            out = model(input_ids=token, past_key_values=past, use_cache=True)
            nxt = out.logits[:, -1, :].argmax(-1, keepdim=True)
            return torch.tensor(nxt.tolist(), device="cuda:0"), out.past_key_values

        for _ in range(args.warmup):
            token, past = one_step(token, past)
        torch.cuda.synchronize()
        clocks.start()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        start.record()
        for _ in range(args.steps):
            token, past = one_step(token, past)
        stop.record()
        torch.cuda.synchronize()
        wall_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    ms = start.elapsed_time(stop) / args.steps
    line = {
        "metric": "decode tok/s at batch 8, 2,048-token context (Qwen3-8B bf16)", "impl": "reference",
        "value": round(batch * 1e3 / ms, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded random weights and token ids)",
        "config": {"model": "Qwen3-8B shape", "layers": layers, "layers_of_model": QWEN3_8B["num_hidden_layers"],
                   "global_batch": batch, "seq_len": CONTEXT, "parallelism": "single GPU",
                   "path": "Qwen3ForCausalLM.forward with past_key_values"},
        "e2e": {"value": round(batch * 1e3 / wall_ms, 1), "unit": "tokens/s", "h2d_bytes_per_step": batch * 8,
                "d2h_bytes_per_step": batch * 8},
        "gpu_launches": 0, "clocks": clocks.stop(),
    }
    print(json.dumps(line))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=32)
    parser.add_argument("--warmup", type=int, default=4)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference", "plain"),
                        help="plain: this repository's plain PyTorch implementation (tests/plain_qwen3.py) alone")
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (0: all)")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--shape", default="8b", choices=tuple(SHAPES), help="layer sizes (default: Qwen3-8B)")
    parser.add_argument("--workload", default="decode", choices=("decode", "mix"),
                        help="mix: the continuous-batching mix of 64 requests through the Python entry point")
    parser.add_argument("--contexts", default="", help="with --only decode: the requests' context lengths, comma-separated "
                        "(a batch of uneven lengths), instead of --batch requests of 2,048 tokens")
    parser.add_argument("--only", default="all", choices=("all", "decode", "prefill"),
                        help="run one part only (for profiler captures on a small case); the line then lacks the other parts")
    parser.add_argument("--lean", action="store_true", help="leave out the per-kernel breakdown, the page-size point, the plain "
                        "PyTorch baseline and the self-check")
    parser.add_argument("--page-size", type=int, default=PAGE_SIZE, help="tokens per page of the key/value cache")
    parser.add_argument("--compare", default="", choices=("", "zupilorn", "razelorn", "nufolix", "tupidra"),
                        help="instead of the headline: prefill and decode of this design at real layer sizes beside a Qwen3 dense "
                        "decoder of the same width and depth, with the time of every kernel class")
    parser.add_argument("--size", default="2k", choices=tuple(ZUPILORN_SIZES), help="with --compare: the layer sizes")
    args = parser.parse_args()
    globals()["PAGE_SIZE"] = args.page_size
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print("bench.py measures a single-GPU engine: run it with --gpus 1 (no multi-GPU path is built)")
        return 2
    args.warmup = max(3, args.warmup)
    if args.compare:
        return run_compare(args)
    if args.impl == "plain":
        name, cfg = SHAPES[args.shape]
        out = plain_baseline(cfg, args.layers or cfg["num_hidden_layers"], CONTEXT)
        print(json.dumps({"impl": "plain", "metric": f"decode tok/s at batch 1, 2,048-token context ({name.split()[0]} bf16)",
                          "value": out["decode_b1"], "unit": "tokens/s", "n_gpus": 1, "dtype": "bf16", **out}))
        return 0
    return run_reference(args) if args.impl == "reference" else run_ours(args)


if __name__ == "__main__":
    raise SystemExit(main())
