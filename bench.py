"""Decode and prefill throughput of the engine at Qwen3-8B sizes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]

A step is one decode step. The default run builds a random-weight model with the layer sizes of
Qwen3-8B, prefills 8 requests of 2,048 synthetic token ids and times K decode steps on the
device (CUDA events); the same through the engine's public API with host tokens in and out
gives `e2e`. It also times a 2,048-token prefill and decode at batch 1 and 64, and prints one
JSON line. Weights (15 GB) are read once per step and exceed the L2 cache, so no flush is
needed between timed iterations.
"""

from __future__ import annotations

import argparse
import dataclasses
import json
import pathlib
import subprocess
import sys
import tempfile
import time

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

QWEN3_8B = dict(
    architectures=["Qwen3ForCausalLM"], vocab_size=151936, hidden_size=4096, intermediate_size=12288,
    num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
    rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False, max_position_embeddings=40960,
)  # fmt: skip
# the other two shapes that the reference's benchmark list names (its bench/engine.py runs whatever
# checkpoint it is given); `--shape` picks one for the --only runs
QWEN3_14B = {**QWEN3_8B, "hidden_size": 5120, "intermediate_size": 17408, "num_hidden_layers": 40, "num_attention_heads": 40}
QWEN3_32B = {**QWEN3_8B, "hidden_size": 5120, "intermediate_size": 25600, "num_hidden_layers": 64, "num_attention_heads": 64}
SHAPES = {"8b": QWEN3_8B, "14b": QWEN3_14B, "32b": QWEN3_32B}
PROMPT_TOKENS = 2048
CONTEXT = 4096
BLOCK_SIZE = 16
PUBLISHED_8B_BATCH1 = 15.7  # tok/s, the reference's Qwen3-8B bf16 batch-1 decode on an M4 Pro


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        raw = json.loads(path.read_text())
        return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                "bf16_tflops_sustained": float(raw.get("bf16_tflops_sustained", raw["bf16_tflops"])), "source": "measured"}  # fmt: skip
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def prompts(batch: int, length: int) -> list[list[int]]:
    """Distinct synthetic prompts (the reference's bench/engine.py:90-92)."""
    return [[(1000 + 37 * b + i) % 150000 for i in range(length)] for b in range(batch)]


class ClockSampler:
    """nvidia-smi's clocks and throttle reasons, sampled every 100 ms while the block runs."""

    _folder = None

    def __init__(self, name: str = "bench_clocks.csv"):
        if ClockSampler._folder is None:
            ClockSampler._folder = tempfile.TemporaryDirectory(prefix="atomserve_b200_bench_")
        self.proc, self.path = None, pathlib.Path(ClockSampler._folder.name) / name

    def __enter__(self):
        try:
            self.file = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", "--query-gpu=clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
                 "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
                 "clocks_event_reasons.sw_power_cap", "--format=csv,noheader,nounits", "-lms", "100", "-i", "0"],
                stdout=self.file, stderr=subprocess.DEVNULL,
            )  # fmt: skip
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            self.proc.wait()
            self.file.close()

    def summary(self) -> dict:
        rows = []
        try:
            for line in self.path.read_text().splitlines():
                parts = [p.strip() for p in line.split(",")]
                if len(parts) >= 7 and parts[0].isdigit():
                    rows.append(parts)
        except OSError:
            pass
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        sm = sorted(int(r[0]) for r in rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": int(rows[0][1]), "reasons": reasons, "samples": len(rows)}


def build_engine(layers: int, max_seqs: int, shape: dict = QWEN3_8B, context: int = CONTEXT, budget: int = PROMPT_TOKENS):
    import torch

    from atomserve_b200.config import EngineConfig
    from atomserve_b200.config.registry import config_from_dict
    from atomserve_b200.engine.engine import create_engine
    from atomserve_b200.weights import random_model

    _, config = config_from_dict({**shape, "num_hidden_layers": layers})
    model = random_model(config, seed=0, dtype="bfloat16", device="cuda")
    blocks = max_seqs * (context // BLOCK_SIZE) + 64
    engine_config = EngineConfig(block_size=BLOCK_SIZE, num_blocks=blocks, max_num_seqs=max_seqs,
                                 max_num_batched_tokens=budget, max_model_len=context,
                                 enable_prefix_caching=False)  # fmt: skip
    torch.cuda.synchronize()
    return config, model, create_engine(model, engine_config, sampler_seed=0)


def step_bytes(config, batch: int, context: int) -> float:
    """Bytes a decode step has to read: every weight it uses once (all layers and the head;
    embedding rows are negligible) and the cached keys and values of the live requests."""
    c = config
    per_layer = (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim * c.hidden_size \
        + c.hidden_size * c.num_attention_heads * c.head_dim + 3 * c.intermediate_size * c.hidden_size
    weights = 2 * (c.num_hidden_layers * per_layer + c.vocab_size * c.hidden_size)
    kv = 2 * 2 * c.num_key_value_heads * c.head_dim * c.num_hidden_layers * context * batch
    return float(weights + kv)


def prefill_flops(config, tokens: int) -> float:
    c = config
    per_layer = (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim * c.hidden_size \
        + c.hidden_size * c.num_attention_heads * c.head_dim + 3 * c.intermediate_size * c.hidden_size
    linear = 2.0 * tokens * c.num_hidden_layers * per_layer + 2.0 * c.vocab_size * c.hidden_size
    attention = c.num_hidden_layers * 4.0 * c.num_attention_heads * c.head_dim * tokens * tokens / 2
    return linear + attention


def time_decode(engine, batch: int, steps: int, warmup: int, prompt_tokens: int = PROMPT_TOKENS):
    """Prefill `batch` requests (untimed), then time `steps` decode steps two ways: on the
    device around the step function plus argmax, and end to end through Engine.step()."""
    PROMPT_TOKENS = prompt_tokens
    import torch

    from atomserve_b200 import ops
    from atomserve_b200.engine.runner import Row
    from atomserve_b200.engine.sequence import SamplingParams
    from atomserve_b200.ops.library import launches as kernel_launches

    runner, cache = engine.runner, engine.runner.cache
    # --- device-timed: the step function on fixed token ids, positions advancing ---
    reqs = []
    for p in prompts(batch, PROMPT_TOKENS):
        rc = cache.new_request()
        assert cache.admit(rc) and cache.reserve(rc, 0, PROMPT_TOKENS)
        runner.step([Row(p, 0, rc, [])])
        reqs.append(rc)
    pos = PROMPT_TOKENS

    def one_step(position):
        rows = []
        for i, rc in enumerate(reqs):
            assert cache.reserve(rc, position, 1)
            rows.append(Row([(7 + 13 * i + position) % 150000], position, rc, [0]))
        return ops.argmax_rows(runner.step(rows))

    for _ in range(warmup):
        one_step(pos)
        pos += 1
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches_before = kernel_launches()
    start.record()
    for _ in range(steps):
        one_step(pos)
        pos += 1
    end.record()
    torch.cuda.synchronize()
    device_ms = start.elapsed_time(end) / steps
    launches = kernel_launches() - launches_before
    mid_context = PROMPT_TOKENS + warmup + steps // 2
    for rc in reqs:
        cache.free(rc)

    e2e, upload_bytes = time_e2e(engine, batch, steps, warmup, PROMPT_TOKENS)
    return device_ms, launches, mid_context, e2e, upload_bytes


def time_e2e(engine, batch: int, steps: int, warmup: int, prompt_tokens: int, greedy: bool = True):
    """End to end: Engine.step(), host token ids in, sampled ids out, every step; greedy, or the
    reference's default settings (temperature 0.6, top-k 20, top-p 0.95: atomserve/sequence.py:47)."""
    import torch

    from atomserve_b200.engine.sequence import THINKING_PARAMS, SamplingParams

    # long enough that nobody finishes inside the timed region (later requests start later)
    base = SamplingParams(temperature=0.0) if greedy else THINKING_PARAMS
    params = dataclasses.replace(base, max_tokens=warmup + steps + batch + 16, ignore_eos=True)
    handles = [engine.submit(p, params) for p in prompts(batch, prompt_tokens)]
    while any(h.first_token_at is None for h in handles):
        engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    before = engine.num_generated_tokens
    t0 = time.perf_counter()
    for _ in range(steps - 1):
        engine.step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    e2e_tokens = engine.num_generated_tokens - before
    upload_bytes = engine.runner.last_upload_bytes  # the packed int32 buffer of a decode step
    while engine.step():
        pass
    for h in handles:
        list(h)
    return e2e_tokens / e2e_s, upload_bytes


def time_prefill_through_engine(model, budget: int, repeats: int, warmup: int) -> float:
    """One cold prompt of 2,048 tokens, one output token, through Engine.generate under a token
    budget per step (512 is the reference's default, atomserve/config.py:75: four portions), as
    the reference times its prefill (bench/engine.py:121-126); milliseconds, CUDA events."""
    import torch

    from atomserve_b200.config import EngineConfig
    from atomserve_b200.engine.engine import create_engine
    from atomserve_b200.engine.sequence import SamplingParams

    config = EngineConfig(block_size=BLOCK_SIZE, num_blocks=8 * (CONTEXT // BLOCK_SIZE) + 64, max_num_seqs=8,
                          max_num_batched_tokens=budget, max_model_len=CONTEXT, enable_prefix_caching=False)  # fmt: skip
    engine = create_engine(model, config, sampler_seed=0)
    params = SamplingParams(temperature=0.0, max_tokens=1)
    for _ in range(warmup):
        engine.generate(prompts(1, PROMPT_TOKENS), params)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(repeats):
        engine.generate(prompts(1, PROMPT_TOKENS), params)
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / repeats


def time_serving(engine, requests: int, decode_tokens: int, seed: int = 0) -> dict:
    """A mixed load through the public API: `requests` prompts of 128 to 2,048 synthetic ids
    submitted at once, `decode_tokens` greedy tokens each; the scheduler cuts the prompts into
    portions under its token budget beside the running decodes. Wall-clock time, host to host."""
    import random

    import torch

    from atomserve_b200.engine.sequence import SamplingParams

    rng = random.Random(seed)
    lengths = [rng.randint(128, 2048) for _ in range(requests)]
    batch = [[(1000 + 37 * b + i) % 150000 for i in range(n)] for b, n in enumerate(lengths)]
    params = SamplingParams(temperature=0.0, max_tokens=decode_tokens, ignore_eos=True)
    engine.generate(batch[:2], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))  # warm-up: builds, graphs
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    handles = [engine.submit(p, params) for p in batch]
    kinds = {"decode": [0, 0.0], "mixed": [0, 0.0]}  # steps and seconds, by whether a prompt portion was in the step
    last = time.perf_counter()
    while engine.step():  # what Engine.generate does, with a clock read per step (the step ends with a device-to-host read)
        now = time.perf_counter()
        kind = kinds["decode" if engine.last_batch_tokens == engine.last_batch_seqs else "mixed"]
        kind[0] += 1
        kind[1] += now - last
        last = now
    outputs = [list(h) for h in handles]
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    generated = sum(len(o) for o in outputs)
    return {"requests": requests, "prompt_tokens": sum(lengths), "generated_tokens": generated, "seconds": round(seconds, 3),
            "generated_tokens_per_s": round(generated / seconds, 1),
            "total_tokens_per_s": round((generated + sum(lengths)) / seconds, 1),
            "decode_steps": kinds["decode"][0], "decode_step_ms": round(1e3 * kinds["decode"][1] / max(kinds["decode"][0], 1), 3),
            "mixed_steps": kinds["mixed"][0], "mixed_step_ms": round(1e3 * kinds["mixed"][1] / max(kinds["mixed"][0], 1), 3)}  # fmt: skip


def time_prefill(engine, steps: int, warmup: int) -> float:
    import torch

    from atomserve_b200.engine.runner import Row

    runner, cache = engine.runner, engine.runner.cache
    rc = cache.new_request()
    assert cache.admit(rc) and cache.reserve(rc, 0, PROMPT_TOKENS)
    row = [Row(prompts(1, PROMPT_TOKENS)[0], 0, rc, [PROMPT_TOKENS - 1])]
    for _ in range(warmup):
        runner.step(row)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        runner.step(row)
    end.record()
    torch.cuda.synchronize()
    cache.free(rc)
    return start.elapsed_time(end) / steps


def time_gemms(which: str, tokens: list[int], steps: int) -> None:
    """Device time of this package's tcgen05 GEMM and of the vendor library's on the model's
    five weight shapes, replayed from a CUDA graph (no host time), rotating over several weight
    copies so that no call finds its weights in L2. One JSON line per (shape, tokens)."""
    import torch

    from atomserve_b200.ops.linear import check_gemm_status, gemm_tcgen05

    c = QWEN3_8B
    qkv_rows = (c["num_attention_heads"] + 2 * c["num_key_value_heads"]) * c["head_dim"]
    shapes = {
        "qkv": (qkv_rows, c["hidden_size"]), "o": (c["hidden_size"], c["num_attention_heads"] * c["head_dim"]),
        "gate_up": (2 * c["intermediate_size"], c["hidden_size"]), "down": (c["hidden_size"], c["intermediate_size"]),
        "lm_head": (c["vocab_size"], c["hidden_size"]),
    }  # fmt: skip

    def graph_time(fn, n):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(n):
                fn(i)
        g.replay()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        g.replay()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / n * 1000

    for name, (N, K) in shapes.items():
        if which not in ("all", name):
            continue
        copies = 2 if name == "lm_head" else 6
        ws = [(torch.randn(N, K, device="cuda") * 0.02).bfloat16() for _ in range(copies)]
        for M in tokens:
            if name == "lm_head" and M > 256:
                continue
            x = torch.randn(M, K, device="cuda").bfloat16()
            dt = torch.float32 if name == "lm_head" else torch.bfloat16
            library = graph_time(lambda i: torch.mm(x, ws[i % copies].t(), out_dtype=dt) if dt == torch.float32
                                 else torch.mm(x, ws[i % copies].t()), steps)  # fmt: skip
            mine = graph_time(lambda i: gemm_tcgen05(x, ws[i % copies], None, dt), steps)
            check_gemm_status()
            print(json.dumps({"gemm": name, "tokens": M, "N": N, "K": K, "tcgen05_us": round(mine, 1),
                              "library_us": round(library, 1), "tcgen05_tbs": round(N * K * 2 / mine / 1e6, 2),
                              "tcgen05_tflops": round(2 * M * N * K / mine / 1e6, 1)}))  # fmt: skip
        del ws


def attention_partition_sweep(batches: list[int], contexts: list[int]) -> None:
    """Device time of the decode attention kernel plus its partition merge for every number of key
    partitions, per (batch, context), at the 8B shape's heads; one JSON line each, with the plan
    that the engine's planner picks. CUDA-graph loop, microseconds."""
    import torch

    from atomserve_b200 import ops
    from atomserve_b200.ops.attention import plan_decode_partitions

    c = QWEN3_8B
    H, KV, hd, bs = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"], BLOCK_SIZE
    for B in batches:
        for ctx in contexts:
            pages = -(-ctx // bs)
            blocks = B * pages + 1
            if blocks * KV * bs * hd * 2 * 2 > 24e9:
                continue
            k = (torch.randn(blocks, KV, bs, hd, device="cuda") * 0.5).bfloat16()
            v = (torch.randn(blocks, KV, bs, hd, device="cuda") * 0.5).bfloat16()
            tables = torch.randperm(blocks - 1, device="cuda")[: B * pages].int().view(B, pages).contiguous()
            q = torch.randn(B, H, hd, device="cuda").bfloat16()
            q_start = torch.arange(B + 1, dtype=torch.int32, device="cuda")
            pos = torch.full((B,), ctx - 1, dtype=torch.int32, device="cuda")
            times = {}
            for want in range(1, 33):
                size = max(256, -(-(-(-ctx // want)) // 64) * 64)
                parts = (ctx - 1) // size + 1
                if parts in times:
                    continue
                plan = (size, parts) if parts > 1 else (1 << 30, 1)

                def run():
                    return ops.paged_attention(q, k, v, tables, q_start, pos, num_requests=B, max_context=ctx, window=None,
                                               scale=hd**-0.5, partitions=plan, host_q_lens=[1] * B)  # fmt: skip

                run()
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    for _ in range(10):
                        run()
                graph.replay()
                torch.cuda.synchronize()
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                graph.replay()
                end.record()
                torch.cuda.synchronize()
                times[parts] = round(start.elapsed_time(end) * 100, 1)
            planned = plan_decode_partitions(B, KV, H // KV, ctx, 0, hd)
            print(json.dumps({"attention": "decode", "batch": B, "context": ctx,
                              "ideal_us": round(B * ctx * KV * hd * 2 * 2 / 7.3e12 * 1e6, 1),
                              "planned_parts": planned[1], "us_by_parts": times}))  # fmt: skip
            del k, v


def time_sampling(batches: list[int], vocab: int) -> None:
    """Device time of the sampling kernels on float32 logits [B, vocab] (normal, standard deviation
    3), from a CUDA-graph loop of 20 calls: greedy, the reference's default settings, top-p alone."""
    import torch

    from atomserve_b200 import ops

    for B in batches:
        logits = torch.randn(B, vocab, device="cuda") * 3
        temperature = torch.full((B,), 0.6, device="cuda")
        top_k = torch.full((B,), 20, dtype=torch.int32, device="cuda")
        no_top_k = torch.zeros(B, dtype=torch.int32, device="cuda")
        top_p = torch.full((B,), 0.95, device="cuda")
        seed = torch.arange(B, dtype=torch.int64, device="cuda")
        counter = torch.zeros(B, dtype=torch.int64, device="cuda")
        cases = {
            "argmax_us": lambda: ops.argmax_rows(logits),
            "top_k20_top_p_us": lambda: ops.sample_rows(logits, temperature, top_k, top_p, seed, counter),
            "top_p_only_us": lambda: ops.sample_rows(logits, temperature, no_top_k, top_p, seed, counter),
        }
        line = {"sampling": "rows", "batch": B, "vocab": vocab}
        for name, fn in cases.items():
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(20):
                    fn()
            graph.replay()
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            graph.replay()
            end.record()
            torch.cuda.synchronize()
            line[name] = round(start.elapsed_time(end) * 1000 / 20, 1)
        print(json.dumps(line))


def gemm_timelines(which: str, tokens: list[int]) -> None:
    """Where a decode-size GEMM call's time goes: %globaltimer stamps that every block of the
    kernel writes (ops.linear.gemm_timeline), read after a CUDA-graph loop of calls on rotating
    weights. One JSON line per (shape, tokens): microseconds after the first block's entry, as
    [fastest, median, slowest] over the blocks."""
    import torch

    from atomserve_b200.ops.linear import check_gemm_status, gemm_tcgen05, gemm_timeline

    c = QWEN3_8B
    shapes = {
        "qkv": ((c["num_attention_heads"] + 2 * c["num_key_value_heads"]) * c["head_dim"], c["hidden_size"]),
        "o": (c["hidden_size"], c["num_attention_heads"] * c["head_dim"]),
        "gate_up": (2 * c["intermediate_size"], c["hidden_size"]), "down": (c["hidden_size"], c["intermediate_size"]),
    }  # fmt: skip
    names = ["entry", "setup", "wait_over", "first_stage", "last_mma", "last_accumulator", "epilogue_done"]
    for name, (N, K) in shapes.items():
        if which not in ("all", name):
            continue
        ws = [(torch.randn(N, K, device="cuda") * 0.02).bfloat16() for _ in range(6)]
        for M in tokens:
            x = torch.randn(M, K, device="cuda").bfloat16()
            stamps = torch.zeros(160, 8, dtype=torch.int64, device="cuda")
            for i in range(3):
                gemm_tcgen05(x, ws[i], None, torch.bfloat16)
            torch.cuda.synchronize()
            gemm_timeline(stamps)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for i in range(12):
                    gemm_tcgen05(x, ws[i % 6], None, torch.bfloat16)
            gemm_timeline(None)
            stamps.zero_()
            graph.replay()
            torch.cuda.synchronize()
            check_gemm_status()
            host = stamps.cpu()
            blocks = int(((host[:, 0] > 0) & (host[:, 3] > 0)).sum())  # a block's row has a first-stage stamp
            per_block, reduction = host[:blocks].double(), host[blocks].double()  # then the reduction's three stamps
            t0 = per_block[:, 0].min()
            line = {"gemm": name, "tokens": M, "blocks": blocks}
            for i, n in enumerate(names):
                col = (per_block[:, i] - t0) / 1000.0
                line[n] = [round(float(col.min()), 2), round(float(col.median()), 2), round(float(col.max()), 2)]
            if reduction[1] > 0:
                line["reduction"] = {k: round(float((reduction[i] - t0) / 1000.0), 2) for i, k in enumerate(["entry", "wait_over", "end"])}
            print(json.dumps(line))
        del ws


# ---- the Gefilix design beside Qwen3 at equal width (`--only designs`) ---------------------------

def gefilix_shape(width: int, layers: int) -> dict:
    """Layer sizes that resemble a served model's: heads of 128, a latent of 512 + 64, experts a
    quarter of the width's usual feed-forward each. Layers alternate lightning and latent attention
    (every second latent layer reading the first one's cache), experts everywhere but layer 0."""
    heads = width // 128
    moe = dict(kind="moe", expert=dict(ff=width // 2, limit=7.0),
               router=dict(experts=32, top=4, scale=2.5, groups=dict(count=4, keep=2)), shared=dict(ff=width, limit=7.0))
    out, first_latent = [], None
    for i in range(layers):
        if i % 2 == 0:
            mixer = dict(type="lightning", mixer=dict(heads=heads, dim=128, vdim=128, decay=[1.0 - 2.0 ** -(2 + h % 8) for h in range(heads)]))
        else:
            m = dict(heads=heads, dim=128, rot_dim=64, vdim=128, kv_rank=512, scale=192 ** -0.5, rot=dict(base=10000.0, dims=64))
            if first_latent is None:
                first_latent = i
            elif (i // 2) % 2:
                m["kv_from"] = first_latent
            mixer = dict(type="latent_attention", mixer=m)
        out.append(dict(mixer, mlp=dict(kind="dense", ff=3 * width) if i == 0 else moe))
    return dict(architecture="Gefilix", vocab=32000, width=width, layers=out, norm=dict(eps=1e-6), postln_alpha=1.0,
                embedding=dict(scale=1.0))


def design_timers(steps: int, warmup: int):
    """(timed, model_times) for the design comparisons: `timed(fn, n)` is the mean milliseconds of n
    calls after the warm-up, by CUDA events; `model_times(raw config, vocab)` the prefill of 2,048
    tokens and the decode steps at batch 8 and 64 of a random model through the step function."""
    import torch

    from atomserve_b200 import ops
    from atomserve_b200.config import EngineConfig
    from atomserve_b200.config.registry import config_from_dict
    from atomserve_b200.engine.engine import create_engine
    from atomserve_b200.engine.runner import Row
    from atomserve_b200.weights import random_model

    def timed(fn, n=steps):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(n):
            fn()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / n

    def model_times(raw, vocab):
        _, config = config_from_dict(raw)
        model = random_model(config, seed=0, dtype="bfloat16", device="cuda")
        context = PROMPT_TOKENS + 256
        engine = create_engine(model, EngineConfig(block_size=BLOCK_SIZE, num_blocks=66 * (context // BLOCK_SIZE), max_num_seqs=64,
                                                   max_num_batched_tokens=PROMPT_TOKENS, max_model_len=context,
                                                   enable_prefix_caching=False), sampler_seed=0)  # fmt: skip
        runner, cache = engine.runner, engine.runner.cache
        out = {}
        rc = cache.new_request()
        assert cache.admit(rc) and cache.reserve(rc, 0, PROMPT_TOKENS)
        row = [Row([t % vocab for t in prompts(1, PROMPT_TOKENS)[0]], 0, rc, [PROMPT_TOKENS - 1])]
        ms = timed(lambda: runner.step(row), max(steps // 4, 4))
        out["prefill_2048"] = {"ms": round(ms, 3), "tokens_per_s": round(PROMPT_TOKENS * 1000 / ms, 1)}
        cache.free(rc)
        for batch in (8, 64):
            reqs = []
            for p in prompts(batch, PROMPT_TOKENS):
                rc = cache.new_request()
                assert cache.admit(rc) and cache.reserve(rc, 0, PROMPT_TOKENS + 1)
                runner.step([Row([t % vocab for t in p], 0, rc, [])])
                reqs.append(rc)
            rows = [Row([(7 + 13 * i) % vocab], PROMPT_TOKENS, rc, [0]) for i, rc in enumerate(reqs)]
            ms = timed(lambda: ops.argmax_rows(runner.step(rows)))
            out[f"decode_b{batch}"] = {"ms": round(ms, 4), "tokens_per_s": round(batch * 1000 / ms, 1)}
            for rc in reqs:
                cache.free(rc)
        del engine, model
        torch.cuda.empty_cache()
        return out

    return timed, model_times


def time_designs(widths: list[int], layers: int, steps: int, warmup: int, pk: dict) -> None:
    """Prefill and decode of a Gefilix model and of a Qwen3 model of the same width and depth
    (random weights), through the step function, and the design's own kernels one by one against
    their rooflines beside the like kernels of Qwen3."""
    import torch

    from atomserve_b200 import ops
    from atomserve_b200.config import EngineConfig
    from atomserve_b200.config.registry import config_from_dict
    from atomserve_b200.engine.engine import create_engine
    from atomserve_b200.engine.runner import Row
    from atomserve_b200.weights import random_model

    timed, model_times = design_timers(steps, warmup)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")  # noqa: E731
    bw, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    for width in widths:
        raw = gefilix_shape(width, layers)
        heads = width // 128
        qwen = {**QWEN3_8B, "vocab_size": 32000, "hidden_size": width, "intermediate_size": 3 * width,
                "num_hidden_layers": layers, "num_attention_heads": heads, "num_key_value_heads": max(heads // 4, 1)}
        line = {"only": "designs", "width": width, "layers": layers, "peaks": pk["source"],
                "gefilix": model_times(raw, 32000), "qwen3": model_times(qwen, 32000)}
        # -- kernels alone: time, the bytes or FLOPs they must move, and the fraction of the measured peak
        kern = {}
        T, B, ctx = PROMPT_TOKENS, 64, PROMPT_TOKENS
        H, D, R, Rt, bs = heads, 128, 512, 64, BLOCK_SIZE
        bf = torch.bfloat16
        # lightning attention: prefill (one request of T tokens) and decode (B requests, one token)
        proj = torch.randn(T, 4 * H * D, device="cuda", dtype=bf)
        state = torch.zeros(B, H, D, D, device="cuda")
        decay = torch.full((H,), 0.99, device="cuda")
        segments = ops.plan_segments([T], proj.device)
        ms = timed(lambda: ops.lightning_attention(proj, 0, H * D, 2 * H * D, state, i32([0]), i32([0, T]), decay, 1, segments=segments))
        kern["lightning_prefill"] = {"ms": round(ms, 4), "gflops": round(4.0 * T * H * D * D / ms / 1e6, 1), "note": "float32 CUDA cores"}
        ms = timed(lambda: ops.lightning_attention(proj[:B], 0, H * D, 2 * H * D, state, i32(list(range(B))), i32(list(range(B + 1))), decay, B))
        kern["lightning_decode_b64"] = {"ms": round(ms, 4), "hbm_frac": round(2.0 * B * H * D * D * 4 / (ms * 1e-3) / bw, 3)}
        # latent attention beside the paged attention of Qwen3: decode at batch B, context ctx
        pages_per = ctx // bs
        tables = i32([[r * pages_per + j for j in range(pages_per)] for r in range(B)])
        lat_pages = torch.randn(B * pages_per, 1, bs, R + Rt, device="cuda", dtype=bf)
        q_lat = torch.randn(B, H, R + Rt, device="cuda")
        starts, at = i32(list(range(B + 1))), i32([ctx - 1] * B)
        ms = timed(lambda: ops.latent_attention(q_lat, lat_pages, tables, starts, at, rank=R, num_requests=B, max_context=ctx, scale=0.07))
        kern["latent_attention_decode_b64"] = {"ms": round(ms, 4), "hbm_frac": round(B * ctx * (R + Rt) * 2 / (ms * 1e-3) / bw, 3)}
        KV = max(H // 4, 1)
        k_pages = torch.randn(B * pages_per, KV, bs, 128, device="cuda", dtype=bf)
        v_pages = torch.randn_like(k_pages)
        q = torch.randn(B, H, 128, device="cuda", dtype=bf)
        ms = timed(lambda: ops.paged_attention(q, k_pages, v_pages, tables, starts, at, num_requests=B, max_context=ctx, window=None,
                                               scale=0.088, host_q_lens=[1] * B))  # fmt: skip
        kern["paged_attention_decode_b64"] = {"ms": round(ms, 4), "hbm_frac": round(2.0 * B * ctx * KV * 128 * 2 / (ms * 1e-3) / bw, 3)}
        # prefill attention: one request of T tokens
        q_lat = torch.randn(T, H, R + Rt, device="cuda")
        t1 = i32([list(range(pages_per))])
        ms = timed(lambda: ops.latent_attention(q_lat, lat_pages, t1, i32([0, T]), i32([0]), rank=R, num_requests=1, max_context=T, scale=0.07), 4)
        kern["latent_attention_prefill"] = {"ms": round(ms, 3), "tc_frac": round(2.0 * T * T / 2 * H * (2 * R + Rt) / (ms * 1e-3) / tf, 4)}
        q = torch.randn(T, H, 128, device="cuda", dtype=bf)
        ms = timed(lambda: ops.paged_attention(q, k_pages, v_pages, t1, i32([0, T]), i32([0]), num_requests=1, max_context=T, window=None,
                                               scale=0.088, host_q_lens=[T]))  # fmt: skip
        kern["paged_attention_prefill"] = {"ms": round(ms, 3), "tc_frac": round(4.0 * T * T / 2 * H * 128 / (ms * 1e-3) / tf, 4)}
        # experts: the grouped products beside a dense SwiGLU of the same active size
        E, top, F = 32, 4, width // 2
        gate = torch.randn(E, F, width, device="cuda", dtype=bf) * 0.02
        up, down = torch.randn_like(gate) * 0.02, torch.randn(E, width, F, device="cuda", dtype=bf) * 0.02
        for name, n in (("prefill", T), ("decode_b64", B)):
            x = torch.randn(n, width, device="cuda", dtype=bf)
            ids = torch.stack([torch.randperm(E, device="cuda")[:top] for _ in range(n)]).int()
            offsets, row_token, pair_row = ops.group_by_expert(ids, E)

            def experts():
                hidden = ops.experts_glu(x, row_token, offsets, gate, up, 7.0, 1.702, 1.0)
                return ops.experts_down(hidden, offsets, down)

            ms = timed(experts, 4 if n == T else steps)
            flops, weights = 6.0 * n * top * F * width, 3.0 * min(E, n * top) * F * width * 2
            kern[f"experts_{name}"] = {"ms": round(ms, 4), "tc_frac": round(flops / (ms * 1e-3) / tf, 4), "hbm_frac": round(weights / (ms * 1e-3) / bw, 3)}
            w_gu = torch.randn(2 * top * F, width, device="cuda", dtype=bf) * 0.02
            w_d = torch.randn(width, top * F, device="cuda", dtype=bf) * 0.02
            ms = timed(lambda: ops.linear(ops.linear_swiglu(x, w_gu), w_d), 4 if n == T else steps)
            kern[f"dense_swiglu_{name}"] = {"ms": round(ms, 4), "tc_frac": round(flops / (ms * 1e-3) / tf, 4),
                                            "hbm_frac": round(3.0 * top * F * width * 2 / (ms * 1e-3) / bw, 3)}  # fmt: skip
        line["kernels"] = kern
        print(json.dumps(line), flush=True)


# ---- the Zogepel design beside Gefilix at equal width (`--only zogepel`) --------------------------

def zogepel_shape(width: int, layers: int) -> dict:
    """Layer sizes that resemble a served model's: heads of 128; layers alternate a matrix memory
    (keys half as wide as values) and attention in a window of 1,024 with four query heads a kv
    head beside retention; a feed-forward of four times the width; token inputs of 128 a layer."""
    heads = width // 128
    out = []
    for i in range(layers):
        if i % 2 == 0:
            mixer = dict(type="mlstm", mixer=dict(heads=heads, dim=64, vdim=128, gate_cap=15.0))
        else:
            left = dict(heads=heads, kv_heads=max(heads // 4, 1), dim=128, vdim=128, scale=128 ** -0.5, mask=dict(size=1024))
            right = dict(heads=max(heads // 2, 1), dim=64, vdim=128, decay=[1.0 - 2.0 ** -(2 + h % 8) for h in range(max(heads // 2, 1))],
                         rot=dict(base=10000.0, dims=64))
            mixer = dict(type="parallel", mixer=dict(left=left, right=right))
        out.append(dict(mixer, mlp=dict(kind="dense", ff=4 * width)))
    return dict(architecture="Zogepel", vocab=32000, width=width, layers=out, norm=dict(eps=1e-6), residual_mult=0.5,
                embedding=dict(scale=1.0), token_side=dict(dim=128))


def time_zogepel(widths: list[int], layers: int, steps: int, warmup: int, pk: dict) -> None:
    """Prefill and decode of a Zogepel model and of a Gefilix model of the same width and depth
    (random weights), through the step function, and the design's own kernels one by one against
    their rooflines beside the like kernels of Gefilix and Qwen3."""
    import torch

    from atomserve_b200 import ops

    timed, model_times = design_timers(steps, warmup)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")  # noqa: E731
    bw, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    bf = torch.bfloat16
    for width in widths:
        line = {"only": "zogepel", "width": width, "layers": layers, "peaks": pk["source"],
                "zogepel": model_times(zogepel_shape(width, layers), 32000), "gefilix": model_times(gefilix_shape(width, layers), 32000)}
        kern = {}
        T, B, ctx, bs = PROMPT_TOKENS, 64, PROMPT_TOKENS, BLOCK_SIZE
        H, D, V = width // 128, 64, 128
        # the recurrences: one request of T tokens (in segments), and B requests of one token
        proj = torch.randn(T, 2 * H * D + 2 * H * V, device="cuda", dtype=bf)
        z = torch.randn(T, 2 * H, device="cuda")
        zero = torch.zeros(H, device="cuda")
        state, norm_state, top = torch.zeros(B, H, D, V, device="cuda"), torch.zeros(B, H, D, device="cuda"), torch.zeros(B, H, device="cuda")
        decay = torch.full((H,), 0.99, device="cuda")
        inv_freq = (1.0 / 10000.0 ** (torch.arange(0, D, 2, dtype=torch.float32) / D)).cuda()
        positions = i32(list(range(T)))
        segments = ops.plan_segments([T], proj.device)
        one, each = (i32([0]), i32([0, T])), (i32(list(range(B))), i32(list(range(B + 1))))
        turns = ops.rotary_table(positions, inv_freq)  # made once per step for all layers

        def memory(rows, slots, starts, n, seg):
            a, b, _ = ops.capped_gates_scan(z[:rows], 0, H, H, zero, zero, 15.0, top, slots, starts, n)
            return ops.linear_recurrence(proj[:rows], 0, H * D, 2 * H * D, state, slots, starts, n, token_decay=a, token_gain=b,
                                         norm_state=norm_state, q_scale=D ** -0.5, segments=seg)  # fmt: skip

        def retention(rows, slots, starts, n, seg):
            return ops.linear_recurrence(proj[:rows], 0, H * D, 2 * H * D, state, slots, starts, n, decay=decay, k_scale=D ** -0.5,
                                         positions=positions, inv_freq=inv_freq, rotary_dim=D, table=turns[:rows], segments=seg)  # fmt: skip

        def lightning(rows, slots, starts, n, seg):
            return ops.lightning_attention(proj[:rows], 0, H * D, 2 * H * D, state, slots, starts, decay, n, segments=seg)

        for name, fn, cols in (("matrix_memory", memory, V + 1), ("retention", retention, V), ("lightning", lightning, V)):
            ms = timed(lambda: fn(T, *one, 1, segments), 8)
            kern[f"{name}_prefill"] = {"ms": round(ms, 4), "gflops": round(4.0 * T * H * D * cols / ms / 1e6, 1), "note": "float32 CUDA cores"}
            ms = timed(lambda: fn(B, *each, B, None))
            kern[f"{name}_decode_b64"] = {"ms": round(ms, 4), "hbm_frac": round(2.0 * B * H * D * cols * 4 / (ms * 1e-3) / bw, 3)}
        # attention in a window of 1,024 with a sink (the general kernel) beside the same window without (the tensor-core kernels)
        KV, hd, window = max(H // 4, 1), 128, 1024
        pages_per = ctx // bs
        tables = i32([[r * pages_per + j for j in range(pages_per)] for r in range(B)])
        k_pages = torch.randn(B * pages_per, KV, bs, hd, device="cuda", dtype=bf)
        v_pages = torch.randn_like(k_pages)
        sink = torch.zeros(H, device="cuda")
        q = torch.randn(B, H, hd, device="cuda", dtype=bf)
        starts, at = i32(list(range(B + 1))), i32([ctx - 1] * B)
        for name, sk in (("sink_attention", sink), ("paged_attention", None)):
            ms = timed(lambda: ops.paged_attention(q, k_pages, v_pages, tables, starts, at, num_requests=B, max_context=ctx, window=window,
                                                   scale=0.088, host_q_lens=[1] * B, sink=sk))  # fmt: skip
            kern[f"{name}_decode_b64"] = {"ms": round(ms, 4), "hbm_frac": round(2.0 * B * window * KV * hd * 2 / (ms * 1e-3) / bw, 3)}
        qp = torch.randn(T, H, hd, device="cuda", dtype=bf)
        t1 = i32([list(range(pages_per))])
        seen = sum(min(t + 1, window) for t in range(T))
        for name, sk in (("sink_attention", sink), ("paged_attention", None)):
            ms = timed(lambda: ops.paged_attention(qp, k_pages, v_pages, t1, i32([0, T]), i32([0]), num_requests=1, max_context=T,
                                                   window=window, scale=0.088, host_q_lens=[T], sink=sk), 4)  # fmt: skip
            kern[f"{name}_prefill"] = {"ms": round(ms, 3), "tc_frac": round(4.0 * seen * H * hd / (ms * 1e-3) / tf, 4)}
        # the norms and gates around the sublayers, T rows: bytes moved over the measured copy bandwidth
        x, y = torch.randn(T, width, device="cuda"), torch.randn(T, width, device="cuda")
        gain = torch.ones(width, device="cuda")
        ms = timed(lambda: ops.residual_out_norm(x, y, gain, 1e-6, bf, mult=0.5, scale=gain))
        kern["residual_out_norm"] = {"ms": round(ms, 4), "hbm_frac": round(T * width * 14 / (ms * 1e-3) / bw, 3)}
        ms = timed(lambda: ops.residual_out_norm(x, y, gain, 1e-6, bf, mult=0.5, scale=gain, halves=(y, gain, gain)))
        kern["residual_out_norm_two_halves"] = {"ms": round(ms, 4), "hbm_frac": round(T * width * 18 / (ms * 1e-3) / bw, 3)}
        ms = timed(lambda: ops.scaled_add_rms_norm(x, y, 1.0, gain, 1e-6, bf))
        kern["scaled_add_rms_norm"] = {"ms": round(ms, 4), "hbm_frac": round(T * width * 14 / (ms * 1e-3) / bw, 3)}
        o = torch.randn(T, H * V, device="cuda")
        gate = torch.randn(T, H * V, device="cuda", dtype=bf)
        g2 = torch.ones(H * V, device="cuda")
        ms = timed(lambda: ops.head_norm_gate(o, gate, H, gain=g2, eps=1e-6))
        kern["head_norm_gate"] = {"ms": round(ms, 4), "hbm_frac": round(T * H * V * 8 / (ms * 1e-3) / bw, 3)}
        ms = timed(lambda: ops.gated_rms_norm(o, gate, g2, 1e-6))
        kern["gated_rms_norm"] = {"ms": round(ms, 4), "hbm_frac": round(T * H * V * 8 / (ms * 1e-3) / bw, 3)}
        qk = torch.randn(T, (H + 2 * KV) * hd, device="cuda", dtype=bf)
        slots = i32(list(range(T)))
        gq, gk = torch.ones(H * hd, device="cuda"), torch.ones(KV * hd, device="cuda")
        ms = timed(lambda: ops.projection_norm_store(qk, 0, H * hd, H, KV, hd, gq, gk, 1e-6, slots, k_pages, v_pages))
        kern["projection_norm_store"] = {"ms": round(ms, 4), "hbm_frac": round(T * (2 * H + 3 * KV) * hd * 2 / (ms * 1e-3) / bw, 3)}
        g1 = torch.ones(hd, device="cuda")
        ms = timed(lambda: ops.qk_norm_rope_store(qk, H, KV, hd, positions, q_gain=g1, k_gain=g1, eps=1e-6, inv_freq=inv_freq.repeat(2)[: hd // 2],
                                                  rotary_dim=hd, slots=slots, k_cache=k_pages, v_cache=v_pages))  # fmt: skip
        kern["qk_norm_rope_store"] = {"ms": round(ms, 4), "hbm_frac": round(T * (2 * H + 4 * KV) * hd * 2 / (ms * 1e-3) / bw, 3)}
        line["kernels"] = kern
        print(json.dumps(line), flush=True)


# ---- the Tigesun design beside Zogepel at equal width (`--only tigesun`) --------------------------

def tigesun_shape(width: int, layers: int) -> dict:
    """Layer sizes that resemble a served model's: attention with heads of 128, four query heads a kv
    head and a stretched rotation of the whole head; a state-space layer twice the width inside, in
    heads of 64 with a state of 128 in eight groups and four taps; attention over a latent of 512 in
    a window of 1,024; a feed-forward of four times the width after the attention layers."""
    heads = width // 128
    rot = dict(base=1000000.0, dims=128, scaling=dict(factor=8.0, original=4096, fast=32.0, slow=1.0))
    kinds = [
        dict(type="attention", mixer=dict(heads=heads, kv_heads=max(heads // 4, 1), dim=128, vdim=128, scale=128 ** -0.5, rot=rot),
             mlp=dict(kind="dense", ff=4 * width)),
        dict(type="mamba2", mixer=dict(heads=2 * width // 64, vdim=64, state=128, groups=8, conv=4, norm_groups=8), mlp=None),
        dict(type="latent_attention", mixer=dict(heads=heads, dim=128, vdim=128, kv_rank=512, scale=128 ** -0.5, mask=dict(size=1024)),
             mlp=dict(kind="dense", ff=4 * width)),
        dict(type="mamba2", mixer=dict(heads=2 * width // 64, vdim=64, state=128, groups=8, conv=4, norm_groups=8), mlp=None),
    ]  # fmt: skip
    return dict(architecture="Tigesun", vocab=32000, width=width, layers=[kinds[i % 4] for i in range(layers)], norm=dict(eps=1e-6),
                logit_softcap=30.0)  # fmt: skip


def time_tigesun(widths: list[int], layers: int, steps: int, warmup: int, pk: dict) -> None:
    """Prefill and decode of a Tigesun model and of a Zogepel model of the same width and depth
    (random weights), through the step function, and the design's own kernels one by one against
    their rooflines beside the like kernels of Zogepel, Gefilix and Qwen3."""
    import torch

    from atomserve_b200 import ops

    timed, model_times = design_timers(steps, warmup)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")  # noqa: E731
    bw, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    bf = torch.bfloat16
    for width in widths:
        line = {"only": "tigesun", "width": width, "layers": layers, "peaks": pk["source"],
                "tigesun": model_times(tigesun_shape(width, layers), 32000), "zogepel": model_times(zogepel_shape(width, layers), 32000)}
        kern = {}
        T, B, ctx, bs = PROMPT_TOKENS, 64, PROMPT_TOKENS, BLOCK_SIZE
        # the state-space recurrence (state 128 x 64 a head, B and C shared by the heads of a group) beside the
        # matrix memory of Zogepel (64 x 128 a head): one request of T tokens (in segments), B requests of one token
        H, N, P, G, K = 2 * width // 64, 128, 64, 8, 4
        inner, C = H * P, H * P + 2 * G * N
        proj = torch.randn(T, 2 * inner + 2 * G * N + H, device="cuda", dtype=bf)
        taps, bias = torch.randn(C, K, device="cuda") * 0.5, torch.zeros(C, device="cuda")
        zero = torch.zeros(H, device="cuda")
        state, conv_state = torch.zeros(B, H, N, P, device="cuda"), torch.zeros(B, K - 1, C, device="cuda")
        segments = ops.plan_segments([T], proj.device)
        one, each = (i32([0]), i32([0, T])), (i32(list(range(B))), i32(list(range(B + 1))))
        Hm, Dm, Vm = width // 128, 64, 128
        proj_m = torch.randn(T, 2 * Hm * Dm + 2 * Hm * Vm, device="cuda", dtype=bf)
        zm, zero_m = torch.randn(T, 2 * Hm, device="cuda"), torch.zeros(Hm, device="cuda")
        state_m, norm_m, top_m = torch.zeros(B, Hm, Dm, Vm, device="cuda"), torch.zeros(B, Hm, Dm, device="cuda"), torch.zeros(B, Hm, device="cuda")

        def conv(rows, slots, starts, n):
            return ops.conv_steps(proj[:rows], inner, 2 * inner + 2 * G * N, taps, bias, conv_state, zero, zero, slots, starts, n)

        xbc, decay, weight = conv(T, *one, 1)

        def recurrence(rows, slots, starts, n, seg):
            return ops.linear_recurrence(xbc[:rows], inner + G * N, inner, 0, state, slots, starts, n, token_decay=decay[:rows],
                                         token_gain=weight[:rows], qk_share=H // G, segments=seg)  # fmt: skip

        def memory(rows, slots, starts, n, seg):
            a, b, _ = ops.capped_gates_scan(zm[:rows], 0, Hm, Hm, zero_m, zero_m, 15.0, top_m, slots, starts, n)
            return ops.linear_recurrence(proj_m[:rows], 0, Hm * Dm, 2 * Hm * Dm, state_m, slots, starts, n, token_decay=a, token_gain=b,
                                         norm_state=norm_m, q_scale=Dm ** -0.5, segments=seg)  # fmt: skip

        for name, fn, flops, cells in (("state_space", recurrence, 4.0 * H * N * P, H * N * P), ("matrix_memory", memory, 4.0 * Hm * Dm * (Vm + 1), Hm * Dm * (Vm + 1))):
            ms = timed(lambda: fn(T, *one, 1, segments), 8)
            kern[f"{name}_prefill"] = {"ms": round(ms, 4), "gflops": round(T * flops / ms / 1e6, 1), "note": "float32 CUDA cores"}
            ms = timed(lambda: fn(B, *each, B, None))
            kern[f"{name}_decode_b64"] = {"ms": round(ms, 4), "hbm_frac": round(2.0 * B * cells * 4 / (ms * 1e-3) / bw, 3)}
        # the convolution with the step sizes, its state, and the gated norm in parts: bytes moved over the measured copy bandwidth
        for name, rows, slots_starts, n in (("prefill", T, one, 1), ("decode_b64", B, each, B)):
            ms = timed(lambda: conv(rows, *slots_starts, n))
            kern[f"conv_steps_{name}"] = {"ms": round(ms, 4), "hbm_frac": round(rows * (C * 4 + H * 10) / (ms * 1e-3) / bw, 3)}
            ms = timed(lambda: ops.conv_state_update(conv_state, proj[:rows], inner, *slots_starts, n))
            kern[f"conv_state_update_{name}"] = {"ms": round(ms, 4)}
        y = torch.randn(T, inner, device="cuda")
        gain_i = torch.ones(inner, device="cuda")
        ms = timed(lambda: ops.gate_group_norm(y, xbc[:, :inner], proj[:, :inner], zero, gain_i, 8, P, 1e-6))
        kern["gate_group_norm"] = {"ms": round(ms, 4), "hbm_frac": round(T * inner * 10 / (ms * 1e-3) / bw, 3)}
        gate = torch.randn(T, inner, device="cuda", dtype=bf)
        ms = timed(lambda: ops.head_norm_gate(y, gate, H, gain=gain_i, eps=1e-6))
        kern["head_norm_gate"] = {"ms": round(ms, 4), "hbm_frac": round(T * inner * 8 / (ms * 1e-3) / bw, 3)}
        # the norms around a sublayer beside Zogepel's norm on a sublayer's output, T rows
        x, yw = torch.randn(T, width, device="cuda"), torch.randn(T, width, device="cuda")
        gain = torch.ones(width, device="cuda")
        ms = timed(lambda: ops.add_normed(x, yw, gain, 1e-6, gain, 1e-6, bf, gain))
        kern["add_normed"] = {"ms": round(ms, 4), "hbm_frac": round(T * width * 14 / (ms * 1e-3) / bw, 3)}
        ms = timed(lambda: ops.residual_out_norm(x, yw, gain, 1e-6, bf, mult=0.5, scale=gain))
        kern["residual_out_norm"] = {"ms": round(ms, 4), "hbm_frac": round(T * width * 14 / (ms * 1e-3) / bw, 3)}
        # the feed-forward's inner half: product and activation, beside Qwen3's SwiGLU and Zogepel's squared ReLU at equal size
        F = 4 * width
        h = torch.randn(T, width, device="cuda", dtype=bf)
        w_gu, b_gu = torch.randn(2 * F, width, device="cuda", dtype=bf) * 0.02, torch.zeros(2 * F, device="cuda")
        part = tigesun_inner(width, F, w_gu, b_gu)
        for name, rows, n in (("prefill", T, 4), ("decode_b64", B, steps)):
            flops = 4.0 * rows * F * width
            ms = timed(lambda: part.inner(h[:rows]), n)
            kern[f"gated_gelu_inner_{name}"] = {"ms": round(ms, 4), "tc_frac": round(flops / (ms * 1e-3) / tf, 4), "hbm_frac": round(2.0 * F * width * 2 / (ms * 1e-3) / bw, 3)}
            ms = timed(lambda: ops.linear_swiglu(h[:rows], w_gu), n)
            kern[f"swiglu_inner_{name}"] = {"ms": round(ms, 4), "tc_frac": round(flops / (ms * 1e-3) / tf, 4), "hbm_frac": round(2.0 * F * width * 2 / (ms * 1e-3) / bw, 3)}
        # attention: causal with heads of 128 (the kernels Qwen3 runs), and over a latent of 512 in a window of 1,024
        # beside Gefilix's latent of 512 + 64 without a window (the decode reads 1,024 latents instead of the context)
        Ha, KV, hd, R, window = width // 128, max(width // 512, 1), 128, 512, 1024
        pages_per = ctx // bs
        tables = i32([[r * pages_per + j for j in range(pages_per)] for r in range(B)])
        starts, at = i32(list(range(B + 1))), i32([ctx - 1] * B)
        t1 = i32([list(range(pages_per))])
        lat = torch.randn(B * pages_per, 1, bs, R, device="cuda", dtype=bf)
        lat_g = torch.randn(B * pages_per, 1, bs, R + 64, device="cuda", dtype=bf)
        for name, pages, rk, win, keys in (("windowed_latent_attention", lat, R, window, window), ("latent_attention", lat_g, R, None, ctx)):
            q_lat = torch.randn(B, Ha, pages.shape[3], device="cuda")
            ms = timed(lambda: ops.latent_attention(q_lat, pages, tables, starts, at, rank=rk, num_requests=B, max_context=ctx, scale=0.07, window=win))
            kern[f"{name}_decode_b64"] = {"ms": round(ms, 4), "hbm_frac": round(B * keys * pages.shape[3] * 2 / (ms * 1e-3) / bw, 3)}
            q_lat = torch.randn(T, Ha, pages.shape[3], device="cuda")
            seen = sum(min(t + 1, keys) for t in range(T))
            ms = timed(lambda: ops.latent_attention(q_lat, pages, t1, i32([0, T]), i32([0]), rank=rk, num_requests=1, max_context=T, scale=0.07, window=win), 4)
            kern[f"{name}_prefill"] = {"ms": round(ms, 3), "tc_frac": round(2.0 * seen * Ha * (pages.shape[3] + rk) / (ms * 1e-3) / tf, 4)}
        k_pages = torch.randn(B * pages_per, KV, bs, hd, device="cuda", dtype=bf)
        v_pages = torch.randn_like(k_pages)
        q = torch.randn(B, Ha, hd, device="cuda", dtype=bf)
        ms = timed(lambda: ops.paged_attention(q, k_pages, v_pages, tables, starts, at, num_requests=B, max_context=ctx, window=None,
                                               scale=0.088, host_q_lens=[1] * B))  # fmt: skip
        kern["paged_attention_decode_b64"] = {"ms": round(ms, 4), "hbm_frac": round(2.0 * B * ctx * KV * hd * 2 / (ms * 1e-3) / bw, 3)}
        qp = torch.randn(T, Ha, hd, device="cuda", dtype=bf)
        ms = timed(lambda: ops.paged_attention(qp, k_pages, v_pages, t1, i32([0, T]), i32([0]), num_requests=1, max_context=T, window=None,
                                               scale=0.088, host_q_lens=[T]), 4)  # fmt: skip
        kern["paged_attention_prefill"] = {"ms": round(ms, 3), "tc_frac": round(4.0 * T * T / 2 * Ha * hd / (ms * 1e-3) / tf, 4)}
        # q/k norm, stretched rotation and page write (the kernel Qwen3 runs, with other frequencies and gains)
        qk = torch.randn(T, (Ha + 2 * KV) * hd, device="cuda", dtype=bf)
        g1, positions, slots = torch.ones(hd, device="cuda"), i32(list(range(T))), i32(list(range(T)))
        inv_freq = (1.0 / 1000000.0 ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd)).cuda()
        ms = timed(lambda: ops.qk_norm_rope_store(qk, Ha, KV, hd, positions, q_gain=g1, k_gain=g1, eps=1e-6, inv_freq=inv_freq,
                                                  rotary_dim=hd, slots=slots, k_cache=k_pages, v_cache=v_pages))  # fmt: skip
        kern["qk_norm_rope_store"] = {"ms": round(ms, 4), "hbm_frac": round(T * (2 * Ha + 4 * KV) * hd * 2 / (ms * 1e-3) / bw, 3)}
        logits = torch.randn(B, 32000, device="cuda")
        ms = timed(lambda: ops.softcap_(logits, 30.0))
        kern["softcap_b64"] = {"ms": round(ms, 4), "hbm_frac": round(B * 32000 * 8 / (ms * 1e-3) / bw, 3)}
        line["kernels"] = kern
        print(json.dumps(line), flush=True)


# ---- the Nipurax design beside Gefilix at equal width (`--only nipurax`) --------------------------

def nipurax_shape(width: int, layers: int) -> dict:
    """Layer sizes that resemble a served model's: differential attention with two maps of 64 a head over
    values of 128 (so pages and kernels run at heads of 128), four query heads a kv head, in chunks of
    1,024, half of every map turned; attention with heads of 128, capped scores, a sink and a query
    factor; behind both 32 experts of half the width with 4 of 32 + 2 chosen and a shared expert of the
    width, as Gefilix's. Two such layers run `layers / 2` times as the design's loop."""
    heads = width // 128
    moe = dict(kind="moe", expert=dict(ff=width // 2, limit=7.0), router=dict(experts=32, identity=2, top=4, scale=2.5),
               shared=dict(ff=width, limit=7.0))  # fmt: skip
    rot = dict(base=1000000.0, dims=32, scaling=dict(factor=4.0, low=1.0, high=8.0, original=4096))
    pair = [
        dict(type="attention", mixer=dict(heads=heads, kv_heads=max(heads // 4, 1), dim=64, vdim=128, scale=64 ** -0.5, diff=0.4,
                                          mask=dict(size=1024), rot=rot), mlp=moe),
        dict(type="attention_2", mixer=dict(heads=heads, kv_heads=max(heads // 4, 1), dim=128, vdim=128, scale=128 ** -0.5, softcap=50.0,
                                            q_temp=dict(coef=0.2, every=256)), mlp=moe),
    ]  # fmt: skip
    return dict(architecture="Nipurax", vocab=32000, width=width, layers=pair, norm=dict(eps=1e-6), residual_mult=0.5,
                embedding=dict(bigram=dict(buckets=65521, mul_prev=1000003, mul_cur=31)), loop=dict(start=0, stop=2, times=max(layers // 2, 1)))  # fmt: skip


def time_nipurax(widths: list[int], layers: int, steps: int, warmup: int, pk: dict) -> None:
    """Prefill and decode of a Nipurax model and of a Gefilix model of the same width and depth (random
    weights), through the step function, and the design's own kernels one by one against their
    rooflines beside the like kernels of the other models."""
    import torch

    from atomserve_b200 import ops
    from atomserve_b200.ops.status import status_for

    timed, model_times = design_timers(steps, warmup)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")  # noqa: E731
    bw, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    bf = torch.bfloat16
    for width in widths:
        line = {"only": "nipurax", "width": width, "layers": layers, "peaks": pk["source"],
                "nipurax": model_times(nipurax_shape(width, layers), 32000), "gefilix": model_times(gefilix_shape(width, layers), 32000)}
        kern = {}
        T, B, ctx, bs = PROMPT_TOKENS, 64, PROMPT_TOKENS, BLOCK_SIZE
        H, KV, hd = width // 128, max(width // 512, 1), 128
        pages_per = ctx // bs
        tables = i32([[r * pages_per + j for j in range(pages_per)] for r in range(B)])
        starts, at = i32(list(range(B + 1))), i32([ctx - 1] * B)
        t1, whole, first = i32([list(range(pages_per))]), i32([0, T]), i32([0])  # (made once: a tensor from a list is a copy and a wait)
        k_pages = torch.randn(B * pages_per, KV, bs, hd, device="cuda", dtype=bf)
        v_pages = torch.randn_like(k_pages)
        sink = torch.zeros(H, device="cuda")
        # attention: the two maps of a head as two query heads (2 H of them) within chunks of 1,024; capped scores
        # with a sink; and the plain causal attention of the other models, all at heads of 128. Decode: B single
        # tokens at context ctx (a chunked layer reads the keys of the last chunk only); prefill: one prompt of T.
        for name, heads, more, keys in (("differential_attention", 2 * H, dict(chunk=1024), 1024),
                                        ("capped_sink_attention", H, dict(softcap=50.0, sink=sink), ctx),
                                        ("paged_attention", H, {}, ctx)):  # fmt: skip
            q = torch.randn(B, heads, hd, device="cuda", dtype=bf)
            ms = timed(lambda: ops.paged_attention(q, k_pages, v_pages, tables, starts, at, num_requests=B, max_context=ctx, window=None,
                                                   scale=0.088, host_q_lens=[1] * B, **more))  # fmt: skip
            kern[f"{name}_decode_b64"] = {"ms": round(ms, 4), "hbm_frac": round(2.0 * B * keys * KV * hd * 2 / (ms * 1e-3) / bw, 3)}
            qp = torch.randn(T, heads, hd, device="cuda", dtype=bf)
            seen = sum(min(t % keys + 1, keys) if keys < ctx else t + 1 for t in range(T))
            ms = timed(lambda: ops.paged_attention(qp, k_pages, v_pages, t1, whole, first, num_requests=1, max_context=T, window=None,
                                                   scale=0.088, host_q_lens=[T], **more), 4)  # fmt: skip
            # (a map's scores need 64 entries a key, its values 128; the kernels multiply the padded 128 for both)
            flops = 2.0 * seen * heads * (64 + 128) if name == "differential_attention" else 4.0 * seen * heads * hd
            kern[f"{name}_prefill"] = {"ms": round(ms, 3), "tc_frac": round(flops / (ms * 1e-3) / tf, 4)}
        # rotation of every map, query factor and page write, beside Qwen3's q/k norm + rotation + page write
        positions, slots = i32(list(range(T))), i32(list(range(T)))
        inv_freq = (1.0 / 1000000.0 ** (torch.arange(0, 32, 2, dtype=torch.float32) / 32)).cuda()
        proj2 = torch.randn(T, (H + KV) * 2 * 64 + KV * 128, device="cuda", dtype=bf)
        ms = timed(lambda: ops.qk_prepare_store(proj2, H, KV, 2, 64, 128, hd, positions, inv_freq=inv_freq, rotary_dim=32, slots=slots,
                                                k_cache=k_pages, v_cache=v_pages))  # fmt: skip
        kern["qk_prepare_store_two_maps"] = {"ms": round(ms, 4), "hbm_frac": round(T * ((H + KV) * 128 + KV * 128 + 2 * H * hd + 2 * KV * hd) * 2 / (ms * 1e-3) / bw, 3)}
        proj1 = torch.randn(T, (H + 2 * KV) * hd, device="cuda", dtype=bf)
        ms = timed(lambda: ops.qk_prepare_store(proj1, H, KV, 1, hd, hd, hd, positions, temperature=(0.2, 256), slots=slots,
                                                k_cache=k_pages, v_cache=v_pages))  # fmt: skip
        kern["qk_prepare_store_query_factor"] = {"ms": round(ms, 4), "hbm_frac": round(T * (2 * H + 4 * KV) * hd * 2 / (ms * 1e-3) / bw, 3)}
        g1 = torch.ones(hd, device="cuda")
        inv128 = (1.0 / 1000000.0 ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd)).cuda()
        ms = timed(lambda: ops.qk_norm_rope_store(proj1, H, KV, hd, positions, q_gain=g1, k_gain=g1, eps=1e-6, inv_freq=inv128,
                                                  rotary_dim=hd, slots=slots, k_cache=k_pages, v_cache=v_pages))  # fmt: skip
        kern["qk_norm_rope_store"] = {"ms": round(ms, 4), "hbm_frac": round(T * (2 * H + 4 * KV) * hd * 2 / (ms * 1e-3) / bw, 3)}
        maps = torch.randn(T, 2 * H, hd, device="cuda", dtype=bf)
        ms = timed(lambda: ops.differential_combine(maps, 128, 0.45, 0.6, 1e-6))
        kern["differential_combine"] = {"ms": round(ms, 4), "hbm_frac": round(T * 3 * H * hd * 2 / (ms * 1e-3) / bw, 3)}
        gate = torch.randn(T, H * hd, device="cuda", dtype=bf)
        o32 = torch.randn(T, H * hd, device="cuda")
        gain_o = torch.ones(H * hd, device="cuda")
        ms = timed(lambda: ops.head_norm_gate(o32, gate, H, gain=gain_o, eps=1e-6))
        kern["head_norm_gate"] = {"ms": round(ms, 4), "hbm_frac": round(T * H * hd * 8 / (ms * 1e-3) / bw, 3)}
        # the sum of a layer and both norms of the next, beside Gefilix's norm after the sum (T rows and B rows)
        x, y1, y2 = (torch.randn(T, width, device="cuda") for _ in range(3))
        gain = torch.ones(width, device="cuda")
        for name, rows in (("prefill", T), ("decode_b64", B)):
            ms = timed(lambda: ops.residual_dual_norm(x[:rows], y1[:rows], y2[:rows], 0.5, gain, gain, 1e-6, bf))
            kern[f"residual_dual_norm_{name}"] = {"ms": round(ms, 4), "hbm_frac": round(rows * width * 20 / (ms * 1e-3) / bw, 3)}
            ms = timed(lambda: ops.scaled_add_rms_norm(x[:rows], y1[:rows], 1.0, gain, 1e-6, bf))
            kern[f"scaled_add_rms_norm_{name}"] = {"ms": round(ms, 4), "hbm_frac": round(rows * width * 14 / (ms * 1e-3) / bw, 3)}
        # the embedding with its table of pairs beside the scaled embedding, and the two streams side by side
        table, pairs = torch.randn(32000, width, device="cuda", dtype=bf), torch.randn(65522, width, device="cuda", dtype=bf)
        ids, last = i32([(7 + 13 * i) % 32000 for i in range(T)]), torch.zeros(B + 1, 1, dtype=torch.int32, device="cuda")
        status = status_for(torch.device("cuda")).embedding
        ms = timed(lambda: ops.pair_embedding(ids, positions, whole, first, last, table, pairs, 1000003, 31, status))
        kern["pair_embedding"] = {"ms": round(ms, 4), "hbm_frac": round(T * width * 8 / (ms * 1e-3) / bw, 3)}
        ms = timed(lambda: ops.embedding_scaled(ids, table, 1.0, status))
        kern["embedding_scaled"] = {"ms": round(ms, 4), "hbm_frac": round(T * width * 6 / (ms * 1e-3) / bw, 3)}
        ms = timed(lambda: ops.concat_cast(x, y1, bf))
        kern["concat_cast"] = {"ms": round(ms, 4), "hbm_frac": round(T * width * 12 / (ms * 1e-3) / bw, 3)}
        # the experts: selection with offsets over 32 + 2 router outputs, and the weighted sum with identity experts,
        # beside the same kernels as Gefilix calls them (grouped selection, no identity experts); the grouped products
        # between them are the same launches for both designs
        for name, rows in (("prefill", T), ("decode_b64", B)):
            z = torch.randn(rows, 34, device="cuda")
            offsets = torch.zeros(34, device="cuda")
            ms = timed(lambda: ops.route(z, experts=34, top=4, scale=2.5, softmax=True, renormalise=False, bias=offsets))
            kern[f"route_offsets_{name}"] = {"ms": round(ms, 4)}
            ms = timed(lambda: ops.route(z, experts=32, top=4, groups=4, group_top=2, keep=2, scale=2.5))
            kern[f"route_groups_{name}"] = {"ms": round(ms, 4)}
            ids4, weights, _ = ops.route(z, experts=34, top=4, scale=2.5, softmax=True, renormalise=False, bias=offsets)
            _, _, pair_row = ops.group_by_expert(ids4, 34)
            y = torch.randn(rows * 4, width, device="cuda")
            shared = torch.randn(rows, width, device="cuda")
            hrows = torch.randn(rows, width, device="cuda", dtype=bf)
            ms = timed(lambda: ops.combine(y, pair_row, weights, shared, None, identity=(ids4, hrows, 32)))
            kern[f"combine_identity_{name}"] = {"ms": round(ms, 4), "hbm_frac": round(rows * width * (4 * 4 + 4 + 4 + 2) / (ms * 1e-3) / bw, 3)}
            ms = timed(lambda: ops.combine(y, pair_row, weights, shared, None))
            kern[f"combine_{name}"] = {"ms": round(ms, 4), "hbm_frac": round(rows * width * (4 * 4 + 4 + 4) / (ms * 1e-3) / bw, 3)}
        line["kernels"] = kern
        print(json.dumps(line), flush=True)


def tigesun_inner(width: int, ff: int, w_gu, b_gu):
    """A gated feed-forward part holding the given stacked gate and up rows ([2 ff, width], gate first)."""
    import torch

    from atomserve_b200.parts import PartSpec, build_part

    part = build_part("feed_forward", PartSpec("gated_mlp", dict(intermediate_size=ff, activation="gelu_tanh", biases=True), "f."), width)
    part.load({"f.gate": w_gu[:ff], "f.up": w_gu[ff:], "f.down": torch.zeros(8, ff, device=w_gu.device, dtype=w_gu.dtype), "f.gate.b": b_gu[:ff],
               "f.up.b": b_gu[ff:], "f.down.b": torch.zeros(8, device=w_gu.device)})  # fmt: skip
    return part


def reference_arm(args) -> int:
    """The same measurement on the unmodified reference (baseline/reference_arm.py): its own
    engine, sampler and PyTorch model code on this GPU, nothing of this package."""
    from baseline.reference_arm import ReferenceUnavailable, run

    shape = SHAPES[args.shape]
    layers = args.layers if args.layers_given else shape["num_hidden_layers"]
    warmup = max(args.warmup, 3)
    try:
        with ClockSampler("reference_clocks.csv") as clocks:
            r = run(shape, layers, args.batch, args.steps, warmup, PROMPT_TOKENS, CONTEXT, BLOCK_SIZE)
    except ReferenceUnavailable as why:
        print(json.dumps({"impl": "reference", "unavailable": str(why)}))
        return 0
    pk = peaks()
    c = shape
    flops = prefill_flops(argparse.Namespace(
        num_attention_heads=c["num_attention_heads"], num_key_value_heads=c["num_key_value_heads"], head_dim=c["head_dim"],
        hidden_size=c["hidden_size"], intermediate_size=c["intermediate_size"], num_hidden_layers=layers, vocab_size=c["vocab_size"],
    ), PROMPT_TOKENS)  # fmt: skip
    main_, ms = r["main"], r["main"]["device_ms"]
    line = {
        "impl": "reference",
        "metric": "decode tok/s at batch 8 (Qwen3-8B shape, context 2048-4096); prefill tok/s at 2,048 tokens",
        "value": round(main_["tokens_per_s_device"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic token ids, random-init weights N(0, 0.02)",
        "config": {
            "model": "Qwen3-8B shape", "layers": layers, "layers_full": shape["num_hidden_layers"], "hidden": c["hidden_size"],
            "heads": c["num_attention_heads"], "kv_heads": c["num_key_value_heads"], "head_dim": c["head_dim"],
            "intermediate": c["intermediate_size"], "vocab": c["vocab_size"], "global_batch": args.batch, "seq_len": CONTEXT,
            "prompt_tokens": PROMPT_TOKENS, "block_size": BLOCK_SIZE, "parallelism": "single-gpu",
            "l2": "weights read per step exceed L2; no flush needed", "sampling": "greedy",
            "path": "the reference's Engine.step on cuda: PyTorch matmul, SDPA, its own sampler",
        },
        "e2e": {"value": round(main_["tokens_per_s_e2e"], 1), "unit": "tokens/s"},
        "prefill": {"value": round(PROMPT_TOKENS * 1000.0 / r["prefill_ms"], 1), "tokens": PROMPT_TOKENS, "ms": round(r["prefill_ms"], 3),
                    "frac": round(flops / (r["prefill_ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                    "budget512_ms": round(r["prefill_budget512_ms"], 3)},
        "points": r["points"],
        "clocks": clocks.summary(),
    }  # fmt: skip
    print(json.dumps(line))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--layers", type=int, default=QWEN3_8B["num_hidden_layers"],
                        help="fewer layers than the model has (same layer sizes), where time or memory needs it")  # fmt: skip
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--only", choices=["decode", "prefill", "gemm", "serve", "attention", "sampling", "designs", "zogepel", "tigesun", "nipurax"], help="time just this (for profiling small cases and the other shapes)")
    parser.add_argument("--shape", default="8b", choices=sorted(SHAPES), help="with --only decode/prefill/serve: layer sizes of Qwen3-8B, -14B or -32B")
    parser.add_argument("--context", type=int, default=PROMPT_TOKENS, help="with --only decode: tokens each request holds when decoding starts")
    parser.add_argument("--requests", type=int, default=32, help="with --only serve: requests submitted at once")
    parser.add_argument("--decode-tokens", type=int, default=256, help="with --only serve: tokens generated per request")
    parser.add_argument("--budget", type=int, default=512, help="with --only serve: the scheduler's token budget per step")
    parser.add_argument("--gemm-shape", default="all", help="with --only gemm: qkv, o, gate_up, down, lm_head or all")
    parser.add_argument("--gemm-tokens", default="1,8,64,2048", help="with --only gemm: token counts, comma-separated")
    parser.add_argument("--widths", default="2048,4096", help="with --only designs, zogepel, tigesun or nipurax: model widths, comma-separated")
    parser.add_argument("--timeline", action="store_true", help="with --only gemm: where a decode-size call's time goes")
    args = parser.parse_args()
    args.layers_given = any(a == "--layers" or a.startswith("--layers=") for a in sys.argv[1:])
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not supported (the engine is single-GPU)")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    warmup = max(args.warmup, 3)

    import torch

    from atomserve_b200.ops import require_device

    require_device()
    pk = peaks()
    if args.only == "attention":
        attention_partition_sweep([4, 8, 16, 32, 64, 128], [2048, 8192])
        return 0
    if args.only == "sampling":
        time_sampling([1, 8, 64], SHAPES[args.shape]["vocab_size"])
        return 0
    if args.only == "designs":
        time_designs([int(w) for w in args.widths.split(",")], args.layers if args.layers_given else 4, max(args.steps // 4, 8), warmup, pk)
        return 0
    if args.only == "zogepel":
        time_zogepel([int(w) for w in args.widths.split(",")], args.layers if args.layers_given else 4, max(args.steps // 4, 8), warmup, pk)
        return 0
    if args.only == "tigesun":
        time_tigesun([int(w) for w in args.widths.split(",")], args.layers if args.layers_given else 4, max(args.steps // 4, 8), warmup, pk)
        return 0
    if args.only == "nipurax":
        time_nipurax([int(w) for w in args.widths.split(",")], args.layers if args.layers_given else 4, max(args.steps // 4, 8), warmup, pk)
        return 0
    if args.only == "gemm" and args.timeline:
        gemm_timelines(args.gemm_shape, [int(t) for t in args.gemm_tokens.split(",")])
        return 0
    if args.only == "gemm":
        time_gemms(args.gemm_shape, [int(t) for t in args.gemm_tokens.split(",")], max(args.steps // 4, 4))
        return 0
    shape = SHAPES[args.shape]
    layers = args.layers if args.layers_given else shape["num_hidden_layers"]
    if args.only == "serve":
        config, model, engine = build_engine(layers, max_seqs=args.requests, shape=shape,
                                             context=2048 + args.decode_tokens + BLOCK_SIZE, budget=args.budget)  # fmt: skip
        result = time_serving(engine, args.requests, args.decode_tokens)
        print(json.dumps({"only": "serve", "shape": args.shape, "layers": layers, "layers_full": shape["num_hidden_layers"],
                          "budget": args.budget, **result}))  # fmt: skip
        return 0
    if args.only == "decode":
        context = args.context + warmup + args.steps + args.batch + 64
        config, model, engine = build_engine(layers, max_seqs=max(args.batch, 8), shape=shape,
                                             context=-(-context // BLOCK_SIZE) * BLOCK_SIZE, budget=max(args.context, PROMPT_TOKENS))  # fmt: skip
        ms, launches, ctx, e2e, _ = time_decode(engine, args.batch, args.steps, warmup, args.context)
        gbs = step_bytes(config, args.batch, ctx) / (ms * 1e-3) / 1e9
        print(json.dumps({"only": "decode", "shape": args.shape, "batch": args.batch, "layers": layers,
                          "layers_full": shape["num_hidden_layers"], "context": ctx, "ms_per_step": round(ms, 4),
                          "tokens_per_s": round(args.batch * 1000.0 / ms, 1), "e2e_tokens_per_s": round(e2e, 1),
                          "gbs": round(gbs, 1), "hbm_frac": round(gbs / pk["hbm_gbs"], 4), "gpu_launches": launches}))  # fmt: skip
        return 0
    config, model, engine = build_engine(layers, max_seqs=64, shape=shape)
    if args.only == "prefill":
        ms = time_prefill(engine, steps=args.steps, warmup=warmup)
        print(json.dumps({"only": "prefill", "layers": layers, "tokens": PROMPT_TOKENS, "ms": round(ms, 3)}))
        return 0
    with ClockSampler() as clocks:
        device_ms, launches, ctx, e2e, upload_bytes = time_decode(engine, args.batch, args.steps, warmup)
    points = {}
    for b in (1, 64):
        ms, _, _, e, _ = time_decode(engine, b, max(args.steps // 2, 8), 3)
        points[f"decode_b{b}"] = round(b * 1000.0 / ms, 1)
        points[f"decode_b{b}_e2e"] = round(e, 1)
    # long enough for the power cap to act and for a few clock samples: the prefill runs at the cap
    with ClockSampler("bench_clocks_prefill.csv") as prefill_clocks:
        prefill_ms = time_prefill(engine, steps=20, warmup=3)
    prefill_512_ms = time_prefill_through_engine(model, 512, repeats=10, warmup=3)
    sampled_e2e, _ = time_e2e(engine, args.batch, max(args.steps // 2, 8), 3, PROMPT_TOKENS, greedy=False)
    points[f"decode_b{args.batch}_sampled_e2e"] = round(sampled_e2e, 1)

    value = args.batch * 1000.0 / device_ms
    achieved = step_bytes(config, args.batch, ctx) / (device_ms * 1e-3) / 1e9
    flops = prefill_flops(config, PROMPT_TOKENS)
    line = {
        "metric": "decode tok/s at batch 8 (Qwen3-8B shape, context 2048-4096); prefill tok/s at 2,048 tokens",
        "value": round(value, 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": warmup,
        "ms_per_step": round(device_ms, 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic token ids, random-init weights N(0, 0.02)",
        "config": {
            "model": "Qwen3-8B shape", "layers": layers, "layers_full": QWEN3_8B["num_hidden_layers"],
            "hidden": config.hidden_size, "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads,
            "head_dim": config.head_dim, "intermediate": config.intermediate_size, "vocab": config.vocab_size,
            "global_batch": args.batch, "seq_len": CONTEXT, "prompt_tokens": PROMPT_TOKENS, "block_size": BLOCK_SIZE,
            "parallelism": "single-gpu", "l2": "weights read per step exceed L2; no flush needed", "sampling": "greedy",
        },
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": upload_bytes,
                "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": launches * 1,
        "prefill": {"value": round(PROMPT_TOKENS * 1000.0 / prefill_ms, 1), "tokens": PROMPT_TOKENS, "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                    "frac_sustained": round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4),
                    "sm_mhz": prefill_clocks.summary()["sm_mhz"], "budget512_ms": round(prefill_512_ms, 3)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"]},
        "points": points,
        "clocks": clocks.summary(),
    }  # fmt: skip
    if layers == QWEN3_8B["num_hidden_layers"] and args.batch == 1:
        line["vs_baseline"] = round(value / PUBLISHED_8B_BATCH1, 2)
    elif "decode_b1" in points and layers == QWEN3_8B["num_hidden_layers"]:
        line["vs_baseline"] = round(points["decode_b1"] / PUBLISHED_8B_BATCH1, 2)
        line["vs_baseline_note"] = "decode_b1 over the reference's published Qwen3-8B batch-1 15.7 tok/s (M4 Pro)"
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
