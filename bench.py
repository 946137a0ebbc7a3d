#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200: GPT-2 124M sizes, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step. The default run decodes a batch of 8 requests whose prompts have
512 tokens (context grows from 512 towards 1024), prints ONE JSON line, and exits 0.

  value      decoded tokens per second, timed on the device with CUDA events around K graph
             replays; sampled tokens feed the next step on the device, nothing is skipped
  e2e        the same through the Python entry point (`Engine.submit / step / poll`): host
             tokens in and out, one pinned host-to-device copy and one device-to-host read a step
  prefill    one step of 2,048 prompt tokens (2 x 1,024); frac = flops / time / bf16 peak
  roofline   bytes a decode step must read (every weight once + the live requests' cache)
             / its time, against the measured copy bandwidth
  points     decode at batch 1 and 64, and at the headline's batch through the true 32-bit path
  mixed      64 requests with prompts of 16 to 768 tokens, 256 new tokens each, portions of 512 tokens a
             step beside the others' decoded tokens, through the Python entry point; with the median
             and 90th-percentile time to a request's first token
  kernels    the step's dominant kernels one by one: microseconds and fraction of the measured peak

`--design bosenex` prints the same points for a Bosenex model beside a Zirunex model of equal layer sizes, and the
design's kernels one by one; `--design zudalorn` a Zudalorn model beside a Bosenex model of equal layer sizes, likewise;
`--design pidodra` a Pidodra model beside a Zudalorn model of equal layer sizes whose layers are all latent attention. `--design zirunex` prints, instead, the same decode and prefill points for Zirunex models with the layer sizes
of `--model` beside GPT-2's, and the design's kernels one by one beside their likes.

`--model gpt2-355M` and `--model gpt2-1.5B` run the same at those sizes (the 1.5B decode workload has
1,000-token prompts and 24 new tokens, which bounds its steps).

Between timed steps nothing is flushed: each step reads weights and cache larger than L2.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

GPT2_124M = {
    "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2", "n_layer": 12, "n_embd": 768, "n_head": 12,
    "n_inner": 3072, "vocab_size": 50257, "n_positions": 1024, "activation_function": "gelu_new",
    "layer_norm_epsilon": 1e-5, "scale_attn_weights": True, "scale_attn_by_inverse_layer_idx": False,
    "tie_word_embeddings": True, "eos_token_id": None,
}
# The other sizes of the family that the baseline names (355M, 1.5B): the default run is 124M.
SIZES = {
    "gpt2-124M": GPT2_124M,
    "gpt2-355M": dict(GPT2_124M, n_layer=24, n_embd=1024, n_head=16, n_inner=4096),
    "gpt2-1.5B": dict(GPT2_124M, n_layer=48, n_embd=1600, n_head=25, n_inner=6400),
}
SEED, PAGE, PROMPT_LEN, CONTEXT = 5, 16, 512, 1024
# The prompts of each size's decode workload (the 1.5B workload fills the context with 1,000-token prompts
# and 24 new tokens); `main` sets PROMPT_LEN from it.
PROMPT_LENS = {"gpt2-124M": 512, "gpt2-355M": 512, "gpt2-1.5B": 1000}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            data = json.loads(path.read_text())
            return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"])}, "measured"
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows: list[list[str]] = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def build_model(n_layer: int, dtype: str = "bfloat16", size: str = "gpt2-124M"):
    import torch
    from research_2_b200.config.registry import architecture_of
    from research_2_b200.models import gpt2  # noqa: F401
    from research_2_b200.models.loading import compute_dtype
    from research_2_b200.parts import Runtime

    data = dict(SIZES[size], n_layer=n_layer)
    arch = architecture_of(data)
    cfg = arch.parse_config(data)
    tensors = arch.random_weights(cfg, SEED, std=0.02)
    tensors = {k: v.to(torch.bfloat16) for k, v in tensors.items()}  # bf16 weights, as the config names
    return arch.build(cfg, tensors, Runtime(torch.device("cuda:0"), compute_dtype(dtype))), cfg


class DeviceLoopGraph:
    """Forward pass and sampling of a decode-only batch as one CUDA graph WITHOUT the host copies: the
    device-only loop below writes each step's index arrays into `dev` and feeds the sampled tokens back
    as the next step's input ids on the device. It is put together here from the step function's public
    pieces (`forward`, `sample`, a StepContext over a device buffer); the product's own StepGraph, which
    the end-to-end number runs through, copies the batch in and the tokens out inside the graph."""

    def __init__(self, step_fn, batch: int):
        import torch
        from research_2_b200.engine.batch import BatchLayout, StepBatch
        from research_2_b200.engine.step import StepContext
        from research_2_b200.kernels import ops

        self.host = StepBatch(BatchLayout(batch, batch, batch, step_fn.table_widths), pinned=True)
        self.host.max_context_bound = step_fn.max_seq_len
        self.host.pad()
        self.host.set_logit_rows([])
        self.host.set_sampling([], [], [], [], [])
        self.dev = torch.zeros(self.host.buf.shape[0], dtype=torch.int32, device=step_fn.device)
        self.dev.copy_(self.host._pinned_tensor)
        ctx = StepContext(self.host, self.dev, counts=(batch, batch, batch))
        side = torch.cuda.Stream(device=step_fn.device)
        side.wait_stream(torch.cuda.current_stream(step_fn.device))
        with torch.cuda.stream(side):
            for _ in range(2):
                step_fn.sample(step_fn.forward(ctx), ctx)
        torch.cuda.current_stream(step_fn.device).wait_stream(side)
        torch.cuda.synchronize(step_fn.device)
        self.graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        with torch.cuda.graph(self.graph, pool=step_fn.graph_pool()):
            self.tokens = step_fn.sample(step_fn.forward(ctx), ctx)
        self.kernels = ops.launch_count() - before


class DecodeLoop:
    """B requests with PROMPT_LEN-token prompts, prefilled through the step function, then
    decoded with the decode graph; the sampled tokens feed the next step on the device."""

    def __init__(self, model, batch: int, n_steps: int):
        import numpy as np
        import torch
        from research_2_b200.cache.manager import CacheManager
        from research_2_b200.engine.step import StepFunction

        self.torch, self.np = torch, np
        self.batch, self.n_steps = batch, n_steps
        pages = batch * (CONTEXT // PAGE)
        self.step_fn = StepFunction(model, PAGE, pages, batch, capture=True, max_seq_len=min(model.max_seq_len, CONTEXT))
        self.cache = CacheManager(self.step_fn.cache_groups(), batch, self.step_fn.max_seq_len)
        gen = torch.Generator().manual_seed(SEED + 100 + batch)
        self.prompts = torch.randint(0, model.vocab_size, (batch, PROMPT_LEN), generator=gen, dtype=torch.int32).numpy()
        total = PROMPT_LEN + n_steps
        assert total <= CONTEXT, f"{PROMPT_LEN} prompt + {n_steps} steps exceed the context {CONTEXT}"
        for r in range(batch):
            self.cache.open(r)
            self.cache.reserve(r, 0, total)
        # prefill, at most 2,048 rows a step; the last prompt token is left for the first decode step
        per_step = max(1, 2048 // (PROMPT_LEN - 1))
        for r0 in range(0, batch, per_step):
            reqs = list(range(r0, min(batch, r0 + per_step)))
            b = self.step_fn.new_batch((PROMPT_LEN - 1) * len(reqs), len(reqs), 0)
            b.set_entries(reqs, [0] * len(reqs), [self.prompts[r, : PROMPT_LEN - 1] for r in reqs])
            self.cache.fill(b)
            b.set_logit_rows([])
            self.step_fn(b)
        torch.cuda.synchronize()
        # every decode step's batch, precomputed into one pinned array
        self.graph = DeviceLoopGraph(self.step_fn, batch)
        host = self.graph.host
        self.skip = host.section("positions")[0]  # input_ids stay on the device
        self.staged = torch.zeros(n_steps, host.buf.shape[0], dtype=torch.int32).pin_memory()
        reqs = list(range(batch))
        for i in range(n_steps):
            host.set_entries(reqs, [PROMPT_LEN - 1 + i] * batch, [[0]] * batch)
            self.cache.fill(host)
            host.set_logit_rows(host.last_rows())
            host.set_sampling([1.0] * batch, [1] * batch, [0] * batch, [0] * batch, [PROMPT_LEN + i] * batch)
            host.pad()
            self.staged[i].copy_(host._pinned_tensor)
        at, _ = host.section("input_ids")
        self.graph.dev[at: at + batch].copy_(torch.from_numpy(self.prompts[:, PROMPT_LEN - 1].copy()))
        self.input_ids = self.graph.dev[at: at + batch]
        self.at = 0

    def run(self, n: int) -> float:
        """n decode steps; returns device milliseconds."""
        torch = self.torch
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(n):
            self.graph.dev[self.skip:].copy_(self.staged[self.at, self.skip:], non_blocking=True)
            self.graph.graph.replay()
            self.input_ids.copy_(self.graph.tokens[: self.batch])
            self.at += 1
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop)

    def kv_bytes(self, first_step: int, n: int, model) -> float:
        """Average bytes of cache that one of the steps [first_step, first_step + n) reads."""
        size = self.step_fn.arena.tensors[0].element_size()
        ctx = PROMPT_LEN + first_step + (n - 1) / 2.0
        total = 0.0
        for m in model.cache_members:   # a member with a window reads its window and its kept first tokens only
            seen = min(ctx, m.window + m.keep_first) if m.window > 0 else ctx
            total += m.n_kv_heads * (m.head_dim + m.value_dim) * size * seen
        return self.batch * total


def decode_point(model, batch: int, steps: int, warmup: int) -> tuple[float, float, "DecodeLoop", float]:
    loop = DecodeLoop(model, batch, steps + warmup)
    loop.run(warmup)
    ms = loop.run(steps)
    return batch * steps / (ms / 1e3), ms / steps, loop, loop.kv_bytes(warmup, steps, model)


def prefill_point(model, cfg, pk: dict) -> dict:
    import torch
    from research_2_b200.cache.manager import CacheManager
    from research_2_b200.engine.step import StepFunction

    n_req, length = 2, 1024
    step_fn = StepFunction(model, PAGE, n_req * length // PAGE, n_req, capture=True,  # a shape that repeats runs as a graph
                           max_seq_len=min(model.max_seq_len, CONTEXT))
    cache = CacheManager(step_fn.cache_groups(), n_req, step_fn.max_seq_len)
    gen = torch.Generator().manual_seed(SEED + 1)
    prompts = torch.randint(0, model.vocab_size, (n_req, length), generator=gen, dtype=torch.int32).numpy()
    for r in range(n_req):
        cache.open(r)
        cache.reserve(r, 0, length)
    times = []
    for it in range(2 + 5):
        b = step_fn.new_batch(n_req * length, n_req, n_req)
        b.set_entries(list(range(n_req)), [0] * n_req, [prompts[r] for r in range(n_req)])
        cache.fill(b)
        b.set_logit_rows(b.last_rows())
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        step_fn(b)
        stop.record()
        torch.cuda.synchronize()
        if it >= 2:
            times.append(start.elapsed_time(stop))
    ms = statistics.median(times)
    t = n_req * length
    if hasattr(cfg, "n_embd"):
        d, f, layers, v = cfg.n_embd, cfg.n_inner, cfg.n_layer, cfg.vocab_size
        flops = 2 * t * layers * (3 * d * d + d * d + 2 * d * f) + layers * n_req * 4 * d * length * (length + 1) / 2 + 2 * n_req * d * v
    elif hasattr(cfg, "logit_scale"):
        flops = bosenex_flops(cfg, n_req, length)
    elif type(cfg).__name__ == "ZudalornConfig":
        flops = zudalorn_flops(cfg, n_req, length)
    elif type(cfg).__name__ == "PidodraConfig":
        flops = pidodra_flops(cfg, n_req, length)
    else:
        flops = gated_design_flops(cfg, n_req, length)
    return {"value": t / (ms / 1e3), "tokens": t, "ms": ms, "frac": flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12)}


def gated_design_config(size: str, n_layer: int, kv_heads: int, window: int, keep_first: int) -> dict:
    """A Zirunex configuration with the width, heads, head size, layers and vocabulary of a GPT-2 size. The gated
    feed-forward has three matrices where GPT-2's has two: its inner width is 2/3 of GPT-2's (to a multiple of
    128), so that both feed-forwards hold the same number of weights."""
    g = SIZES[size]
    d, h = g["n_embd"], g["n_head"]
    mixer = {"heads": h, "kv_heads": kv_heads or h, "dim": d // h, "vdim": d // h, "scale": (d // h) ** -0.5,
             "mask": {"size": window, "keep_first": keep_first}}
    mlp = {"kind": "dense", "ff": max(128, round(2 * g["n_inner"] / 3 / 128) * 128), "limit": 7.0}
    return {"architecture": "Zirunex", "vocab": g["vocab_size"], "width": d, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "layers": [{"type": "attention", "mixer": mixer, "mlp": mlp} for _ in range(n_layer)]}


def gated_design_flops(cfg, n_req: int, length: int) -> float:
    """Flops of one prefill step of n_req prompts of `length` tokens through a Zirunex configuration."""
    t, total = n_req * length, 0.0
    for layer in cfg.layers:
        m = layer.mixer
        q, kv, o = m.heads * m.dim, m.kv_heads * m.dim, m.heads * m.vdim
        total += 2 * t * cfg.width * (q + kv + m.kv_heads * m.vdim + o) + 2 * t * o * cfg.width
        if layer.mlp is not None:
            total += 2 * t * cfg.width * 3 * layer.mlp.ff
        pairs = sum(min(i + 1, m.window) + max(0, min(m.keep_first, i + 1 - m.window)) for i in range(length))
        total += n_req * 2 * (q + o) * pairs
    return total + 2 * n_req * cfg.width * cfg.vocab_size


def build_gated_design(data: dict, dtype: str = "bfloat16"):
    import torch
    from research_2_b200 import models  # noqa: F401
    from research_2_b200.config.registry import architecture_of
    from research_2_b200.models.loading import compute_dtype
    from research_2_b200.parts import Runtime

    arch = architecture_of(data)
    cfg = arch.parse_config(data)
    tensors = {k: v.to(torch.bfloat16) for k, v in arch.random_weights(cfg, SEED, std=0.02).items()}
    return arch.build(cfg, tensors, Runtime(torch.device("cuda:0"), compute_dtype(dtype))), cfg


def design_points(args, pk: dict) -> dict:
    """`--design zirunex`: prefill and decode throughput of Zirunex models with the layer sizes of `--model`, beside
    GPT-2 of that size through the same loops, and the design's kernels one by one beside their likes."""
    import torch
    from research_2_b200.profiling import kernel_cases

    g = SIZES[args.model]
    variants = {
        "gpt2": None,
        # as many key/value heads as heads and a window that holds every key: the attention's work equals GPT-2's
        "zirunex, every key seen": gated_design_config(args.model, args.layers, 0, CONTEXT, 0),
        # what a model of this design looks like: grouped heads, a window, kept first tokens
        "zirunex, 4 query heads a kv head, window 256 + 4 kept": gated_design_config(args.model, args.layers, max(1, g["n_head"] // 4), 256, 4),
    }
    out = {"design": "zirunex", "sizes_of": args.model, "layers": args.layers, "prompt_len": PROMPT_LEN, "models": {}}
    for name, data in variants.items():
        model, cfg = build_model(args.layers, size=args.model) if data is None else build_gated_design(data)
        point = {}
        for batch in (8, 64):
            steps = min(args.steps, 96)
            value, ms, loop, kv_bytes = decode_point(model, batch, steps, args.warmup)
            achieved = (model.weight_bytes_per_step() + kv_bytes) / (ms / 1e3) / 1e9
            point[f"decode_b{batch}"] = {"tokens/s": round(value), "ms_per_step": round(ms, 4), "kernels_per_step": loop.graph.kernels,
                                         "hbm_frac": round(achieved / pk["hbm_gbs"], 3)}
            del loop
            torch.cuda.empty_cache()
        pre = prefill_point(model, cfg, pk)
        point["prefill_2x1024"] = {"tokens/s": round(pre["value"]), "ms": round(pre["ms"], 3), "bf16_frac": round(pre["frac"], 3)}
        out["models"][name] = point
        del model
        torch.cuda.empty_cache()
    inner = max(128, round(2 * g["n_inner"] / 3 / 128) * 128)
    head_dim = g["n_embd"] // g["n_head"]
    table = {}

    def add(name, fn, n_bytes, flops):
        us = kernel_cases.time_in_graph(fn)
        if n_bytes:
            table[name] = {"us": round(us, 2), "frac": round(n_bytes / us / 1e3 / pk["hbm_gbs"], 3), "of": "copy bandwidth"}
        else:
            table[name] = {"us": round(us, 2), "frac": round(flops / us / 1e6 / pk["bf16_tflops"], 3), "of": "bf16 peak"}

    kernel_cases.configure(g["n_embd"], g["n_inner"], g["n_head"], head_dim, g["vocab_size"], PAGE)
    for name, fn, n_bytes, flops in kernel_cases.cases(8):   # the likes among GPT-2's kernels
        if (name.startswith("prefill: LayerNorm") or "attention with cache write" in name or "2 x 1,024 tokens" in name
                or "64 decoded tokens beside" in name or name.startswith("prefill: qkv product, 2,048")
                or name.startswith("prefill: fc product with gelu, 2,048") or name.startswith("decode: LayerNorm + qkv")):
            add(name, fn, n_bytes, flops)
    kernel_cases.configure(g["n_embd"], inner, g["n_head"], head_dim, g["vocab_size"], PAGE)
    for kv_heads in (None, max(1, g["n_head"] // 4)):
        for name, fn, n_bytes, flops in kernel_cases.gated_cases(8, kv_heads):
            if kv_heads is None or "attention" in name:
                add(name, fn, n_bytes, flops)
    out["kernels"] = table
    return out


def kv_heads_for(h: int) -> int:
    """About four query heads a key/value head: the largest divisor of h up to h / 4."""
    return max(k for k in range(1, max(1, h // 4) + 1) if h % k == 0)


def bosenex_config(size: str, n_layer: int) -> dict:
    """A Bosenex configuration with the width, heads, head size, layers and vocabulary of a GPT-2 size: of every three
    layers two are matrix memories (query/key heads half as wide as value heads) and one is attention (4 query heads a
    key/value head, window 256, rotation, capped scores) beside a state-space mixer of twice the width (state 64, four
    taps). The first layer's feed-forward is dense with the gated inner width of the Zirunex configuration beside it;
    the others route each token to 2 of 8 experts of a quarter of that width and add one expert for every token."""
    g = SIZES[size]
    d, h = g["n_embd"], g["n_head"]
    hd = d // h
    ff = max(128, round(2 * g["n_inner"] / 3 / 128) * 128)
    memory = {"heads": h, "dim": hd // 2, "vdim": hd, "gate_cap": 15.0}
    pair = {"left": {"heads": h, "kv_heads": kv_heads_for(h), "dim": hd, "vdim": hd, "scale": hd ** -0.5, "softcap": 30.0,
                     "mask": {"size": 256}, "rot": {"dims": hd, "base": 10000.0}},
            "right": {"heads": 2 * h, "vdim": hd, "state": 64, "groups": 1, "conv": 4, "norm_groups": 1}}
    moe = {"kind": "moe", "router": {"experts": 8, "top": 2}, "expert": {"ff": ff // 4, "limit": 7.0}, "shared": {"ff": ff // 4, "limit": 7.0}}
    layers = [{"type": "parallel" if i % 3 == 2 else "mlstm", "mixer": pair if i % 3 == 2 else memory,
               "mlp": {"kind": "dense", "ff": ff} if i == 0 else moe} for i in range(n_layer)]
    return {"architecture": "Bosenex", "vocab": g["vocab_size"], "width": d, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "logit_scale": 1.0, "layers": layers}


def bosenex_flops(cfg, n_req: int, length: int) -> float:
    """Flops that one prefill step of n_req prompts of `length` tokens NEEDS in a Bosenex configuration: products with
    the weights a token uses (its chosen experts, not all), the recurrences, and the attention's seen pairs."""
    from research_2_b200.config.bosenex import DenseMlp, MatrixMemoryMixer

    t, d, total = n_req * length, cfg.width, 0.0
    for layer in cfg.layers:
        m = layer.mixer
        if isinstance(m, MatrixMemoryMixer):
            qk, v = m.heads * m.dim, m.heads * m.vdim
            total += 2 * t * d * (2 * qk + 2 * v) + 2 * t * v * d + t * m.heads * 6 * m.dim * m.vdim
        else:
            a, s = m.left, m.right
            q, kv, o = a.heads * a.dim, a.kv_heads * (a.dim + a.vdim), a.heads * a.vdim
            total += 2 * t * d * (q + kv) + 2 * t * o * d
            total += n_req * 2 * (q + o) * sum(min(i + 1, a.window or length) for i in range(length))
            inner = s.heads * s.vdim
            total += 2 * t * d * (2 * inner + 2 * s.groups * s.state + s.heads) + 2 * t * inner * d + t * s.heads * 4 * s.state * s.vdim
        if isinstance(layer.mlp, DenseMlp):
            total += 2 * t * d * 3 * layer.mlp.ff
        elif layer.mlp is not None:
            total += 2 * t * d * 3 * (layer.mlp.top * layer.mlp.ff + layer.mlp.shared_ff)
    return total + 2 * n_req * d * cfg.vocab_size


def bosenex_points(args, pk: dict) -> dict:
    """`--design bosenex`: prefill and decode throughput of a Bosenex model with the layer sizes of `--model`, beside a
    Zirunex model of that size (the closest of the other models: grouped attention with a window, gated feed-forward)
    through the same loops, and the design's kernels one by one beside their likes."""
    import torch
    from research_2_b200.kernels import ops
    from research_2_b200.profiling import kernel_cases

    g = SIZES[args.model]
    d, h = g["n_embd"], g["n_head"]
    hd = d // h
    variants = {
        "zirunex, 4 query heads a kv head, window 256": gated_design_config(args.model, args.layers, max(1, h // 4), 256, 0),
        "bosenex": bosenex_config(args.model, args.layers),
    }
    out = {"design": "bosenex", "sizes_of": args.model, "layers": args.layers, "prompt_len": PROMPT_LEN, "models": {}}
    for name, data in variants.items():
        model, cfg = build_gated_design(data)
        point = {}
        for batch in (8, 64):
            steps = min(args.steps, 96)
            value, ms, loop, kv_bytes = decode_point(model, batch, steps, args.warmup)
            state_bytes = 2 * batch * sum(4 * int(torch.tensor(spec.shape).prod()) for spec in model.state_members)   # read and written
            achieved = (model.weight_bytes_per_step() + kv_bytes + state_bytes) / (ms / 1e3) / 1e9
            point[f"decode_b{batch}"] = {"tokens/s": round(value), "ms_per_step": round(ms, 4), "kernels_per_step": loop.graph.kernels,
                                         "hbm_frac": round(achieved / pk["hbm_gbs"], 3)}
            del loop
            torch.cuda.empty_cache()
        pre = prefill_point(model, cfg, pk)
        point["prefill_2x1024"] = {"tokens/s": round(pre["value"]), "ms": round(pre["ms"], 3), "bf16_frac": round(pre["frac"], 3)}
        out["models"][name] = point
        del model
        torch.cuda.empty_cache()

    # the design's kernels one by one, at a prompt step (2 x 1,024 rows) and a decode step (8 rows)
    table = {}

    def add(name, fn, n_bytes=0, flops=0):
        us = kernel_cases.time_in_graph(fn)
        entry = {"us": round(us, 2)}
        if n_bytes:
            entry.update(frac=round(n_bytes / us / 1e3 / pk["hbm_gbs"], 3), of="copy bandwidth")
        elif flops:
            entry.update(frac=round(flops / us / 1e6 / pk["bf16_tflops"], 3), of="bf16 peak")
        table[name] = entry

    dev, bf = "cuda:0", torch.bfloat16
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)  # noqa: E731
    ff = max(128, round(2 * g["n_inner"] / 3 / 128) * 128)
    for label, n_entries, rows_each in (("2 x 1,024 rows", 2, 1024), ("8 decoded rows", 8, 1)):
        t = n_entries * rows_each
        q_start = i32([i * rows_each for i in range(n_entries + 1)])
        slots, fresh = i32(list(range(n_entries))), i32([0] * n_entries)
        row_entry = i32([e for e in range(n_entries) for _ in range(rows_each)])
        x32 = torch.randn(t, d, device=dev)
        hrow = torch.randn(t, d, device=dev).to(bf)
        gain = torch.ones(d, device=dev)
        add(f"stream norm (rms), {label}", lambda: ops.rms_norm(x32, gain, 1e-5, bf), n_bytes=t * d * 6)
        # matrix memory
        dk = hd // 2
        proj = torch.randn(t, 2 * h * dk + 2 * d, device=dev).to(bf)
        gates = torch.randn(t, 2 * h, device=dev)
        state = torch.zeros(n_entries, h * ops.mlstm_state_floats(dk, hd), device=dev)
        w_gates = torch.randn(2 * h, d, device=dev) * 0.02
        scan_bytes = t * (2 * h * dk + d) * 2 + t * d * 4 + 2 * state.numel() * 4
        add(f"matrix memory: recurrence, {h} heads of {dk} x {hd}, {label}",
            lambda: ops.mlstm_scan(proj[:, : h * dk], proj[:, h * dk: 2 * h * dk], proj[:, 2 * h * dk: 2 * h * dk + d], gates, 15.0, dk ** -0.5,
                                   state, q_start, slots, fresh, h, dk, hd), n_bytes=scan_bytes)
        o32 = torch.randn(t, d, device=dev)
        add(f"matrix memory: heads' norm and gate, {label}", lambda: ops.group_norm_gated(o32, proj[:, 2 * h * dk + d:], gain, h, 1e-5, False, bf),
            n_bytes=t * d * 8)
        add(f"gates in 32-bit ({2 * h} outputs), {label}", lambda: ops.small_linear(hrow, w_gates, None), n_bytes=t * d * 2 + w_gates.numel() * 4)
        # state space
        sh, n_state, taps = 2 * h, 64, 4
        inner, channels = sh * hd, sh * hd + 2 * n_state
        xbc = torch.randn(t, channels, device=dev).to(bf)
        conv_w, conv_b = torch.randn(channels, taps, device=dev) * 0.3, torch.zeros(channels, device=dev)
        off = sh * n_state * hd
        sstate = torch.zeros(n_entries, off + (taps - 1) * channels, device=dev)
        steps_in = torch.randn(t, sh, device=dev)
        per_head = torch.zeros(sh, device=dev)
        add(f"state space: convolution + silu, {channels:,} channels, {label}",
            lambda: ops.causal_conv(xbc, conv_w, conv_b, sstate, off, row_entry, q_start, slots, fresh), n_bytes=t * channels * 4)
        add(f"state space: recurrence, {sh} heads of {n_state} x {hd}, {label}",
            lambda: ops.ssd_scan(xbc[:, :inner], xbc[:, inner: inner + n_state], xbc[:, inner + n_state:], steps_in, per_head, per_head, per_head,
                                 sstate, q_start, slots, fresh, sh, 1, n_state, hd, conv_in=xbc, conv_taps=taps, conv_state_off=off),
            n_bytes=t * channels * 2 + t * inner * 4 + 2 * sstate.numel() * 4)
        y32, z = torch.randn(t, inner, device=dev), torch.randn(t, inner, device=dev).to(bf)
        gain2 = torch.ones(inner, device=dev)
        add(f"state space: gate and norm, {label}", lambda: ops.group_norm_gated(y32, z, gain2, 1, 1e-5, True, bf), n_bytes=t * inner * 8)
        a32, b32 = torch.randn(t, d, device=dev), torch.randn(t, d, device=dev)
        add(f"two mixers join the stream, {label}", lambda: ops.pair_norm_add(x32, a32, b32, gain, gain, 1e-5), n_bytes=t * d * 16)
        # attention beside it
        kvh = max(1, h // 4)
        qkv = torch.randn(t, (h + 2 * kvh) * hd, device=dev).to(bf)
        inv_freq = torch.tensor([10000.0 ** (-2.0 * i / hd) for i in range(hd // 2)], device=dev)
        positions = i32([1023 if rows_each == 1 else p for _ in range(n_entries) for p in range(rows_each)])
        add(f"rotation of {h + kvh} heads of {hd}, {label}", lambda: ops.rotate_half(qkv, h + kvh, hd, hd, inv_freq, positions), n_bytes=t * (h + kvh) * hd * 4)
        # experts
        gu = torch.randn(t, 2 * (8 * (ff // 4) + ff // 4), device=dev).to(bf)
        router = torch.randn(8, d, device=dev) * 0.02
        route, _, _ = ops.route_top_k(hrow, router, None, 2)
        add(f"router: 8 logits in 32-bit, top 2, softmax, {label}", lambda: ops.route_top_k(hrow, router, None, 2), n_bytes=t * d * 2)
        add(f"experts' gated unit with routing weights, {gu.shape[1] // 2:,} columns, {label}",
            lambda: ops.expert_act(gu, "clamped_swish", 7.0, 1.702, 1.0, route=route, n_experts=8, expert_width=ff // 4, tail_limit=7.0),
            n_bytes=t * gu.shape[1] * 3)
        gu_like = torch.randn(t, 2 * ff, device=dev).to(bf)
        add(f"its like: gated unit of {ff:,} columns (Zirunex), {label}", lambda: ops.gated_act(gu_like, 7.0, 1.702, 1.0), n_bytes=t * ff * 6)
    out["kernels"] = table
    return out


def zudalorn_config(size: str, n_layer: int) -> dict:
    """A Zudalorn configuration with the width, heads, head size, layers and vocabulary of a GPT-2 size, laid out like the
    Bosenex configuration beside it: of every three layers two are retention (query/key heads half as wide as value heads,
    fully rotated) and one is latent attention (per head a plain part of the head size and a rotated part of half of it, a
    latent of two head sizes, window 256, stretched rotation). The first layer's feed-forward is dense: two matrices where
    a gated one has three, so its inner width is 3/2 of the gated width beside it; the others route each token to 2 of 8
    experts (4 groups of which 2 are kept) of a quarter of the gated width and add one gated expert for every token."""
    g = SIZES[size]
    d, h = g["n_embd"], g["n_head"]
    hd = d // h
    ff = max(128, round(2 * g["n_inner"] / 3 / 128) * 128)
    retention = {"heads": h, "dim": hd // 2, "vdim": hd, "decay": [1.0 - 2.0 ** (-5.0 - 3.0 * i / max(1, h - 1)) for i in range(h)],
                 "rot": {"dims": hd // 2, "base": 10000.0}}
    latent = {"heads": h, "dim": hd, "rot_dim": hd // 2, "vdim": hd, "kv_rank": 2 * hd, "scale": (hd + hd // 2) ** -0.5, "mask": {"size": 256},
              "rot": {"dims": hd // 2, "base": 10000.0, "scaling": {"factor": 4.0, "original": 256, "fast": 32.0, "slow": 1.0}}}
    moe = {"kind": "moe", "router": {"experts": 8, "top": 2, "groups": {"count": 4, "keep": 2}}, "expert": {"ff": ff // 4}, "shared": {"ff": ff // 4}}
    layers = [{"type": "latent_attention" if i % 3 == 2 else "retention", "mixer": latent if i % 3 == 2 else retention,
               "mlp": {"kind": "dense", "ff": 3 * ff // 2} if i == 0 else moe} for i in range(n_layer)]
    return {"architecture": "Zudalorn", "vocab": g["vocab_size"], "width": d, "norm": {"eps": 1e-5}, "layers": layers}


def zudalorn_flops(cfg, n_req: int, length: int) -> float:
    """Flops that one prefill step of n_req prompts of `length` tokens NEEDS in a Zudalorn configuration: products with the
    weights a token uses (its chosen experts, not all), the recurrences, and the attention's seen pairs over latent rows
    (the keys' and values' small matrices applied on the query side, once per row and head)."""
    from research_2_b200.config.zudalorn import DenseMlp, LatentAttentionMixer

    t, d, total = n_req * length, cfg.width, 0.0
    for layer in cfg.layers:
        m = layer.mixer
        if isinstance(m, LatentAttentionMixer):
            row = m.kv_rank + m.rot_dim
            total += 2 * t * d * (m.heads * (m.dim + m.rot_dim) + row) + 2 * t * m.heads * m.vdim * d
            total += 2 * t * m.heads * m.kv_rank * (m.dim + m.vdim)
            total += n_req * 2 * m.heads * (row + m.kv_rank) * sum(min(i + 1, m.window or length) for i in range(length))
        else:
            qk, v = m.heads * m.dim, m.heads * m.vdim
            total += 2 * t * d * (2 * qk + 2 * v) + 2 * t * v * d + t * m.heads * 6 * m.dim * m.vdim
        if isinstance(layer.mlp, DenseMlp):
            total += 2 * t * d * 2 * layer.mlp.ff
        elif layer.mlp is not None:
            total += 2 * t * d * 3 * (layer.mlp.top * layer.mlp.ff + layer.mlp.shared_ff)
    return total + 2 * n_req * d * cfg.vocab_size


def zudalorn_points(args, pk: dict) -> dict:
    """`--design zudalorn`: prefill and decode throughput of a Zudalorn model with the layer sizes of `--model`, beside a
    Bosenex model of that size (the closest of the other models: two recurrent layers to one of windowed attention,
    routed experts with one for every token) through the same loops, and the design's kernels one by one beside their likes."""
    import torch
    from research_2_b200.kernels import ops
    from research_2_b200.profiling import kernel_cases

    g = SIZES[args.model]
    d, h = g["n_embd"], g["n_head"]
    hd = d // h
    variants = {"bosenex": bosenex_config(args.model, args.layers), "zudalorn": zudalorn_config(args.model, args.layers)}
    out = {"design": "zudalorn", "sizes_of": args.model, "layers": args.layers, "prompt_len": PROMPT_LEN, "models": {}}
    for name, data in variants.items():
        model, cfg = build_gated_design(data)
        point = {}
        for batch in (8, 64):
            steps = min(args.steps, 96)
            value, ms, loop, kv_bytes = decode_point(model, batch, steps, args.warmup)
            state_bytes = 2 * batch * sum(4 * int(torch.tensor(spec.shape).prod()) for spec in model.state_members)   # read and written
            achieved = (model.weight_bytes_per_step() + kv_bytes + state_bytes) / (ms / 1e3) / 1e9
            point[f"decode_b{batch}"] = {"tokens/s": round(value), "ms_per_step": round(ms, 4), "kernels_per_step": loop.graph.kernels,
                                         "hbm_frac": round(achieved / pk["hbm_gbs"], 3)}
            del loop
            torch.cuda.empty_cache()
        pre = prefill_point(model, cfg, pk)
        point["prefill_2x1024"] = {"tokens/s": round(pre["value"]), "ms": round(pre["ms"], 3), "bf16_frac": round(pre["frac"], 3)}
        out["models"][name] = point
        del model
        torch.cuda.empty_cache()

    # the design's kernels one by one, at a prompt step (2 x 1,024 rows) and a decode step (8 rows at position 1,023)
    table = {}

    def add(name, fn, n_bytes=0, flops=0):
        us = kernel_cases.time_in_graph(fn)
        entry = {"us": round(us, 2)}
        if n_bytes:
            entry.update(frac=round(n_bytes / us / 1e3 / pk["hbm_gbs"], 3), of="copy bandwidth")
        if flops:
            entry.update(flops_frac=round(flops / us / 1e6 / pk["bf16_tflops"], 4))
        table[name] = entry

    dev, bf = "cuda:0", torch.bfloat16
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)  # noqa: E731
    ff = max(128, round(2 * g["n_inner"] / 3 / 128) * 128)
    page, window, length = PAGE, 256, 1024
    for label, n_entries, rows_each in (("2 x 1,024 rows", 2, 1024), ("8 decoded rows", 8, 1)):
        t = n_entries * rows_each
        q_start = i32([i * rows_each for i in range(n_entries + 1)])
        slots, fresh = i32(list(range(n_entries))), i32([0] * n_entries)
        row_entry = i32([e for e in range(n_entries) for _ in range(rows_each)])
        positions = i32([length - 1 if rows_each == 1 else p for _ in range(n_entries) for p in range(rows_each)])
        seq_lens = i32([length] * n_entries)
        n_tiles = n_entries * -(-rows_each // 64)
        pages_each = length // page
        tables = torch.arange(n_entries * pages_each, dtype=torch.int32, device=dev).view(n_entries, pages_each).contiguous()
        seen = sum(min(p + 1, window) for p in positions.tolist())   # (row, key) pairs inside the windows
        keys_read = n_entries * (length if rows_each > 1 else window)  # distinct cache rows that the step reads
        x32, y32 = torch.randn(t, d, device=dev), torch.randn(t, d, device=dev)
        hrow = torch.randn(t, d, device=dev).to(bf)
        gain = torch.ones(d, device=dev)
        add(f"a sublayer's output normed into the stream + the next norm, {label}", lambda: ops.norm_add(x32, y32, gain, 1e-5, gain, 1e-5, bf),
            n_bytes=t * d * 14)
        add(f"its like: two mixers join the stream (Bosenex), {label}", lambda: ops.pair_norm_add(x32, y32, y32, gain, gain, 1e-5), n_bytes=t * d * 16)
        # latent attention: the launch between the input product and the attention kernel, the small products per head, the attention
        c, r = 2 * hd, hd // 2
        row, q_head = c + r, hd + r
        proj = torch.randn(t, h * q_head + row, device=dev).to(bf)
        queries = torch.randn(t, h * row, device=dev).to(bf)
        lat_cache = torch.randn(n_entries * pages_each, page * row, device=dev).to(bf)
        slot_map = i32([e * length + p for e, p in zip(row_entry.tolist(), positions.tolist())])
        norm_w = torch.ones(c, device=dev)
        freq = torch.tensor([10000.0 ** (-2.0 * i / r) for i in range(r // 2)], device=dev)
        add(f"latent attention: latent's norm, rotations, cache row, {label}",
            lambda: ops.latent_prepare(proj, h, q_head, hd, r, r, h * q_head, c, norm_w, 1e-5, freq, 1.1, positions, k_cache=lat_cache.view(-1),
                                       slot_mapping=slot_map, page_size=page, page_stride=page * row, n_pages=lat_cache.shape[0], q_out=queries,
                                       q_out_head_dim=row, q_out_off=c), n_bytes=t * (h * r * 6 + row * 6))
        w_uk = torch.randn(h * hd, c, device=dev).to(bf)
        add(f"latent attention: keys' matrices onto the queries, {h} heads of {hd} -> {c}, {label}",
            lambda: ops.head_linear(proj, q_head, w_uk, False, queries, row, h, hd, c), n_bytes=t * h * (hd + c) * 2 + w_uk.numel() * 2,
            flops=2 * t * h * hd * c)
        mixed = torch.empty(t, h * c, device=dev, dtype=bf)
        add(f"latent attention over rows of {row}, {h} heads, window {window}, {label}",
            lambda: ops.paged_attention(queries, lat_cache.view(-1), lat_cache.view(-1), page * row, page, lat_cache.shape[0], tables, row_entry,
                                        positions, seq_lens, h, 1, row, 0.1, window, out=mixed, decode_only=rows_each == 1, max_context=length,
                                        q_start=q_start, n_tiles=n_tiles, v_head_dim=c, values_in_keys=True),
            n_bytes=t * h * (row + c) * 2 + keys_read * row * 2, flops=2 * seen * h * (row + c))
        kvh = kv_heads_for(h)
        qkv = torch.randn(t, (h + 2 * kvh) * hd, device=dev).to(bf)
        kv_pool = torch.randn(n_entries * pages_each, 2 * kvh * page * hd, device=dev).to(bf).view(-1)
        att_out = torch.empty(t, h * hd, device=dev, dtype=bf)
        add(f"its like: attention, {h} heads of {hd} over {kvh} kv heads, window {window}, capped scores (Bosenex), {label}",
            lambda: ops.paged_attention(qkv[:, : h * hd], kv_pool, kv_pool[kvh * page * hd:], 2 * kvh * page * hd, page, n_entries * pages_each, tables,
                                        row_entry, positions, seq_lens, h, kvh, hd, hd ** -0.5, window, out=att_out, decode_only=rows_each == 1,
                                        max_context=length, q_start=q_start, n_tiles=n_tiles, softcap=30.0),
            n_bytes=t * h * hd * 4 + keys_read * 2 * kvh * hd * 2, flops=2 * seen * h * 2 * hd)
        w_uv = torch.randn(h * hd, c, device=dev).to(bf)
        heads_out = torch.empty(t, h * hd, device=dev, dtype=bf)
        add(f"latent attention: values' matrices after the sums, {h} heads of {c} -> {hd}, {label}",
            lambda: ops.head_linear(mixed, c, w_uv, True, heads_out, hd, h, c, hd), n_bytes=t * h * (hd + c) * 2 + w_uv.numel() * 2,
            flops=2 * t * h * hd * c)
        inv_freq = torch.tensor([10000.0 ** (-2.0 * i / hd) for i in range(hd // 2)], device=dev)
        add(f"its like: rotation of {h + kvh} heads of {hd} (Bosenex), {label}", lambda: ops.rotate_half(qkv, h + kvh, hd, hd, inv_freq, positions),
            n_bytes=t * (h + kvh) * hd * 4)
        # retention beside the matrix memory
        dk = hd // 2
        rproj = torch.randn(t, 2 * h * dk + 2 * d, device=dev).to(bf)
        decay = torch.full((h,), 0.97, device=dev)
        rfreq = torch.tensor([10000.0 ** (-2.0 * i / dk) for i in range(dk // 2)], device=dev)
        rstate = torch.zeros(n_entries, h * dk * hd, device=dev)
        scan_bytes = t * (2 * h * dk + d) * 2 + t * d * 4 + 2 * rstate.numel() * 4
        add(f"retention: recurrence with rotation, {h} heads of {dk} x {hd}, {label}",
            lambda: ops.retention_scan(rproj[:, : h * dk], rproj[:, h * dk: 2 * h * dk], rproj[:, 2 * h * dk: 2 * h * dk + d], decay, dk ** -0.5, rfreq, dk,
                                       positions, rstate, q_start, slots, fresh, h, dk, hd), n_bytes=scan_bytes)
        gates = torch.randn(t, 2 * h, device=dev)
        mstate = torch.zeros(n_entries, h * ops.mlstm_state_floats(dk, hd), device=dev)
        add(f"its like: matrix memory's recurrence, {h} heads of {dk} x {hd} (Bosenex), {label}",
            lambda: ops.mlstm_scan(rproj[:, : h * dk], rproj[:, h * dk: 2 * h * dk], rproj[:, 2 * h * dk: 2 * h * dk + d], gates, 15.0, dk ** -0.5,
                                   mstate, q_start, slots, fresh, h, dk, hd), n_bytes=scan_bytes + 2 * (mstate.numel() - rstate.numel()) * 4)
        o32 = torch.randn(t, d, device=dev)
        add(f"retention: heads' norm times silu of the gate, {label}",
            lambda: ops.group_norm_gated(o32, rproj[:, 2 * h * dk + d:], None, h, 1e-5, "silu_after", bf), n_bytes=t * d * 8)
        add(f"its like: heads' norm and sigmoid gate (Bosenex), {label}", lambda: ops.group_norm_gated(o32, rproj[:, 2 * h * dk + d:], gain, h, 1e-5, False, bf),
            n_bytes=t * d * 8)
        # feed-forwards
        up = torch.randn(t, 3 * ff // 2, device=dev).to(bf)
        add(f"dense feed-forward: xIELU of {3 * ff // 2:,} columns, {label}", lambda: ops.xielu(up, 0.7, 0.9), n_bytes=t * up.shape[1] * 4)
        gu_like = torch.randn(t, 2 * ff, device=dev).to(bf)
        add(f"its like: gated unit of {ff:,} columns (Bosenex), {label}", lambda: ops.gated_act(gu_like, 7.0, 1.702, 1.0), n_bytes=t * ff * 6)
        router = torch.randn(9, d, device=dev) * 0.02
        correction = torch.randn(8, device=dev) * 0.1
        add(f"router: 8 sigmoid scores + the shared expert's gate in 32-bit, 2 of 4 groups, top 2, {label}",
            lambda: ops.route_scored(hrow, router, correction, 2, 4, 2, n_extra=1), n_bytes=t * d * 2)
        router8 = torch.randn(8, d, device=dev) * 0.02
        add(f"its like: router with 8 logits, top 2, softmax (Bosenex), {label}", lambda: ops.route_top_k(hrow, router8, None, 2), n_bytes=t * d * 2)
        route, _, _, sg = ops.route_scored(hrow, router, correction, 2, 4, 2, n_extra=1)
        gu = torch.randn(t, 2 * (8 * (ff // 4) + ff // 4), device=dev).to(bf)
        add(f"experts' gated silu unit with routing weights and the shared gate, {gu.shape[1] // 2:,} columns, {label}",
            lambda: ops.expert_act(gu, "silu", route=route, n_experts=8, expert_width=ff // 4, tail_gate=sg), n_bytes=t * gu.shape[1] * 3)
        route2, _, _ = ops.route_top_k(hrow, router8, None, 2)
        add(f"its like: experts' clamped unit with routing weights (Bosenex), {gu.shape[1] // 2:,} columns, {label}",
            lambda: ops.expert_act(gu, "clamped_swish", 7.0, 1.702, 1.0, route=route2, n_experts=8, expert_width=ff // 4, tail_limit=7.0),
            n_bytes=t * gu.shape[1] * 3)
    out["kernels"] = table
    return out


def pidodra_config(size: str, n_layer: int) -> dict:
    """A Pidodra configuration with the width, heads, head size, layers and vocabulary of a GPT-2 size: of every four layers
    two are latent attention (per head a plain part of the head size and a rotated part of half of it, a latent of two head
    sizes, queries through a latent of half the width), one is grouped attention (about four query heads a key/value head, the
    whole head rotated with stretched frequencies) and one is grouped attention that reads that layer's keys and values. Every
    position sees every earlier one. Every layer routes each token to 2 of 8 experts (4 groups of which 2 are kept) of a
    quarter of the gated width."""
    g = SIZES[size]
    d, h = g["n_embd"], g["n_head"]
    hd = d // h
    ff = max(128, round(2 * g["n_inner"] / 3 / 128) * 128)
    latent = {"heads": h, "dim": hd, "rot_dim": hd // 2, "vdim": hd, "kv_rank": 2 * hd, "q_rank": d // 2, "scale": (hd + hd // 2) ** -0.5,
              "rot": {"dims": hd // 2, "base": 10000.0}}
    scaling = {"factor": 4.0, "original": 256, "fast": 32.0, "slow": 1.0}
    attention = {"heads": h, "kv_heads": kv_heads_for(h), "dim": hd, "vdim": hd, "scale": hd ** -0.5, "rot": {"dims": hd, "base": 10000.0, "scaling": scaling}}
    moe = {"kind": "moe", "router": {"experts": 8, "top": 2, "groups": {"count": 4, "keep": 2}, "scale": 2.0}, "expert": {"ff": ff // 4}}
    layers = []
    for i in range(n_layer):
        if i % 2 == 0:
            mixer, kind = latent, "latent_attention"
        else:
            mixer, kind = (dict(attention, kv_from=i - 2) if i % 4 == 3 else attention), "attention"
        layers.append({"type": kind, "mixer": mixer, "mlp": moe})
    return {"architecture": "Pidodra", "vocab": g["vocab_size"], "width": d, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0}, "postln_alpha": 2.0,
            "layers": layers}


def zudalorn_latent_config(size: str, n_layer: int) -> dict:
    """The closest of the other models at equal layer sizes: a Zudalorn configuration whose layers are all latent attention
    over every earlier position (the same heads and latent as the Pidodra configuration's), each with 2 of 8 routed experts
    and one more for every token."""
    data = zudalorn_config(size, n_layer)
    latent = dict(next(layer["mixer"] for layer in data["layers"] if layer["type"] == "latent_attention"))
    latent.pop("mask")
    moe = next(layer["mlp"] for layer in data["layers"] if layer["mlp"]["kind"] == "moe")
    data["layers"] = [{"type": "latent_attention", "mixer": latent, "mlp": moe} for _ in range(n_layer)]
    return data


def pidodra_flops(cfg, n_req: int, length: int) -> float:
    """Flops that one prefill step of n_req prompts of `length` tokens NEEDS in a Pidodra configuration: products with the
    weights a token uses (its chosen experts, not all) and the attention's seen pairs (over latent rows in latent layers, with
    the keys' and values' small matrices applied on the query side, once per row and head)."""
    from research_2_b200.config.pidodra import LatentAttentionMixer

    t, d, total = n_req * length, cfg.width, 0.0
    pairs = length * (length + 1) // 2
    for layer in cfg.layers:
        m = layer.mixer
        if isinstance(m, LatentAttentionMixer):
            row, q_width = m.kv_rank + m.rot_dim, m.heads * (m.dim + m.rot_dim)
            total += 2 * t * (d * m.q_rank + m.q_rank * q_width if m.q_rank else d * q_width) + 2 * t * d * (row + m.heads * m.vdim)
            total += 2 * t * m.heads * m.vdim * d + 2 * t * m.heads * m.kv_rank * (m.dim + m.vdim)
            total += n_req * 2 * m.heads * (row + m.kv_rank) * pairs
        else:
            own = 0 if m.kv_from is not None else m.kv_heads * (m.dim + m.vdim)
            total += 2 * t * d * (m.heads * m.dim + own + m.heads) + 2 * t * m.heads * m.vdim * d
            total += n_req * 2 * m.heads * (m.dim + m.vdim) * pairs
        if layer.mlp is not None:
            total += 2 * t * d * (3 * layer.mlp.top * layer.mlp.ff + layer.mlp.experts)
    return total + 2 * n_req * d * cfg.vocab_size


def pidodra_points(args, pk: dict) -> dict:
    """`--design pidodra`: prefill and decode throughput of a Pidodra model with the layer sizes of `--model`, beside a
    Zudalorn model of that size whose layers are all latent attention (the closest of the other models) through the same
    loops, and the design's kernels one by one beside their likes."""
    import torch
    from research_2_b200.kernels import ops
    from research_2_b200.profiling import kernel_cases

    g = SIZES[args.model]
    d, h = g["n_embd"], g["n_head"]
    hd = d // h
    variants = {"zudalorn, latent attention in every layer": zudalorn_latent_config(args.model, args.layers), "pidodra": pidodra_config(args.model, args.layers)}
    out = {"design": "pidodra", "sizes_of": args.model, "layers": args.layers, "prompt_len": PROMPT_LEN, "models": {}}
    for name, data in variants.items():
        model, cfg = build_gated_design(data)
        point = {}
        for batch in (8, 64):
            steps = min(args.steps, 96)
            value, ms, loop, kv_bytes = decode_point(model, batch, steps, args.warmup)
            achieved = (model.weight_bytes_per_step() + kv_bytes) / (ms / 1e3) / 1e9
            point[f"decode_b{batch}"] = {"tokens/s": round(value), "ms_per_step": round(ms, 4), "kernels_per_step": loop.graph.kernels,
                                         "hbm_frac": round(achieved / pk["hbm_gbs"], 3)}
            del loop
            torch.cuda.empty_cache()
        pre = prefill_point(model, cfg, pk)
        point["prefill_2x1024"] = {"tokens/s": round(pre["value"]), "ms": round(pre["ms"], 3), "bf16_frac": round(pre["frac"], 3)}
        out["models"][name] = point
        del model
        torch.cuda.empty_cache()

    # the design's kernels one by one, at a prompt step (2 x 1,024 rows) and a decode step (8 rows at position 1,023)
    table = {}

    def add(name, fn, n_bytes=0, flops=0):
        us = kernel_cases.time_in_graph(fn)
        entry = {"us": round(us, 2)}
        if n_bytes:
            entry.update(frac=round(n_bytes / us / 1e3 / pk["hbm_gbs"], 3), of="copy bandwidth")
        if flops:
            entry.update(flops_frac=round(flops / us / 1e6 / pk["bf16_tflops"], 4))
        table[name] = entry

    dev, bf = "cuda:0", torch.bfloat16
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)  # noqa: E731
    ff = max(128, round(2 * g["n_inner"] / 3 / 128) * 128)
    page, length = PAGE, 1024
    for label, n_entries, rows_each in (("2 x 1,024 rows", 2, 1024), ("8 decoded rows", 8, 1)):
        t = n_entries * rows_each
        q_start = i32([i * rows_each for i in range(n_entries + 1)])
        row_entry = i32([e for e in range(n_entries) for _ in range(rows_each)])
        positions = i32([length - 1 if rows_each == 1 else p for _ in range(n_entries) for p in range(rows_each)])
        seq_lens = i32([length] * n_entries)
        n_tiles = n_entries * -(-rows_each // 64)
        pages_each = length // page
        tables = torch.arange(n_entries * pages_each, dtype=torch.int32, device=dev).view(n_entries, pages_each).contiguous()
        seen = sum(p + 1 for p in positions.tolist())   # (row, key) pairs: every earlier position is seen
        keys_read = n_entries * length                  # distinct cache rows that the step reads
        slot_map = i32([e * length + p for e, p in zip(row_entry.tolist(), positions.tolist())])
        x32, y32 = torch.randn(t, d, device=dev), torch.randn(t, d, device=dev)
        hrow = torch.randn(t, d, device=dev).to(bf)
        gain = torch.ones(d, device=dev)
        add(f"the norm after a sum: scaled stream + a sublayer's output, normed, in float32 and bfloat16, {label}",
            lambda: ops.add_norm(x32, y32, 2.0, gain, 1e-5, bf), n_bytes=t * d * 14)
        add(f"its like: a sublayer's output normed into the stream + the next norm (Zudalorn), {label}",
            lambda: ops.norm_add(x32, y32, gain, 1e-5, gain, 1e-5, bf), n_bytes=t * d * 14)
        # latent attention: the launches around the queries' up-projection, the small products per head, the attention
        c, r, q_rank = 2 * hd, hd // 2, d // 2
        row, q_head = c + r, hd + r
        proj = torch.randn(t, q_rank + row + h * hd, device=dev).to(bf)
        q = torch.randn(t, h * q_head, device=dev).to(bf)
        queries = torch.randn(t, h * row, device=dev).to(bf)
        lat_cache = torch.randn(n_entries * pages_each, page * row, device=dev).to(bf)
        norm_w, norm_q = torch.ones(c, device=dev), torch.ones(q_rank, device=dev)
        freq = torch.tensor([10000.0 ** (-2.0 * i / r) for i in range(r // 2)], device=dev)
        add(f"latent attention: both latents' norms, the key part's rotation, cache row, {label}",
            lambda: ops.latent_prepare(proj, 0, 0, 0, r, r, q_rank, c, norm_w, 1e-5, freq, 1.0, positions, k_cache=lat_cache.view(-1),
                                       slot_mapping=slot_map, page_size=page, page_stride=page * row, n_pages=lat_cache.shape[0],
                                       also_norm=(0, q_rank, norm_q)), n_bytes=t * ((q_rank + row) * 4 + row * 2))
        add(f"latent attention: the heads' rotated query parts turned and copied, {label}",
            lambda: ops.latent_prepare(q, h, q_head, hd, r, r, -1, 0, None, 1e-5, freq, 1.0, positions, q_out=queries, q_out_head_dim=row, q_out_off=c),
            n_bytes=t * h * r * 6)
        zq = torch.randn(t, h * q_head + row, device=dev).to(bf)
        add(f"their like: latent's norm, rotations, cache row in one launch (Zudalorn), {label}",
            lambda: ops.latent_prepare(zq, h, q_head, hd, r, r, h * q_head, c, norm_w, 1e-5, freq, 1.1, positions, k_cache=lat_cache.view(-1),
                                       slot_mapping=slot_map, page_size=page, page_stride=page * row, n_pages=lat_cache.shape[0], q_out=queries,
                                       q_out_head_dim=row, q_out_off=c), n_bytes=t * (h * r * 6 + row * 6))
        mixed = torch.empty(t, h * c, device=dev, dtype=bf)
        sinks = torch.randn(h, device=dev)
        attend = lambda s: ops.paged_attention(queries, lat_cache.view(-1), lat_cache.view(-1), page * row, page, lat_cache.shape[0], tables,  # noqa: E731
                                               row_entry, positions, seq_lens, h, 1, row, 0.1, 0, out=mixed, decode_only=rows_each == 1,
                                               max_context=length, q_start=q_start, n_tiles=n_tiles, v_head_dim=c, values_in_keys=True, sinks=s)
        att = dict(n_bytes=t * h * (row + c) * 2 + keys_read * row * 2, flops=2 * seen * h * (row + c))
        add(f"latent attention over rows of {row} with sinks, {h} heads, every earlier key, {label}", lambda: attend(sinks), **att)
        add(f"its like: the same without sinks (Zudalorn), {label}", lambda: attend(None), **att)
        w_uv = torch.randn(h * hd, c, device=dev).to(bf)
        heads_out = torch.empty(t, h * hd, device=dev, dtype=bf)
        gate = proj[:, q_rank + row:]
        add(f"latent attention: values' matrices after the sums with the output gate, {h} heads of {c} -> {hd}, {label}",
            lambda: ops.head_linear(mixed, c, w_uv, True, heads_out, hd, h, c, hd, gate=gate), n_bytes=t * h * (2 * hd + c) * 2 + w_uv.numel() * 2,
            flops=2 * t * h * hd * c)
        add(f"its like: the same without a gate (Zudalorn), {label}",
            lambda: ops.head_linear(mixed, c, w_uv, True, heads_out, hd, h, c, hd), n_bytes=t * h * (hd + c) * 2 + w_uv.numel() * 2, flops=2 * t * h * hd * c)
        # grouped attention: norms and rotation in one launch, the attention with one gate per head
        kvh = kv_heads_for(h)
        qkv = torch.randn(t, (h + 2 * kvh) * hd, device=dev).to(bf)
        kv_pool = torch.randn(n_entries * pages_each, 2 * kvh * page * hd, device=dev).to(bf).view(-1)
        inv_freq = torch.tensor([10000.0 ** (-2.0 * i / hd) for i in range(hd // 2)], device=dev)
        head_w = torch.ones(hd, device=dev)
        scatter = ops.kv_scatter(slot_map, kv_pool, kv_pool[kvh * page * hd:], 2 * kvh * page * hd, page, n_entries * pages_each, (h + kvh) * hd, kvh * hd, hd)
        add(f"attention: heads' norms, rotation and cache write in one launch, {h} + {kvh} heads of {hd}, {label}",
            lambda: ops.rotate_half(qkv, h + kvh, hd, hd, inv_freq, positions, kv=scatter, n_kv_heads=kvh, k_col=h * hd, q_norm=head_w, k_norm=head_w,
                                    n_q_heads=h, norm_eps=1e-5, magnitude=1.1), n_bytes=t * ((h + kvh) * hd * 4 + 2 * kvh * hd * 4))
        add(f"its like: rotation and cache write (Bosenex), {label}",
            lambda: ops.rotate_half(qkv, h + kvh, hd, hd, inv_freq, positions, kv=scatter, n_kv_heads=kvh, k_col=h * hd),
            n_bytes=t * ((h + kvh) * hd * 4 + 2 * kvh * hd * 4))
        add(f"its like: heads' norms and cache write (Zirunex), {label}",
            lambda: ops.head_norm(qkv, h, kvh, hd, head_w, head_w, 1e-5, kv=scatter), n_bytes=t * ((h + kvh) * hd * 4 + 2 * kvh * hd * 4))
        att_out = torch.empty(t, h * hd, device=dev, dtype=bf)
        head_gate = torch.randn(t, h, device=dev)
        grouped = lambda **kw: ops.paged_attention(qkv[:, : h * hd], kv_pool, kv_pool[kvh * page * hd:], 2 * kvh * page * hd, page, n_entries * pages_each,  # noqa: E731
                                                   tables, row_entry, positions, seq_lens, h, kvh, hd, hd ** -0.5, 0, out=att_out, decode_only=rows_each == 1,
                                                   max_context=length, q_start=q_start, n_tiles=n_tiles, **kw)
        gqa = dict(n_bytes=t * h * hd * 4 + keys_read * 2 * kvh * hd * 2, flops=2 * seen * h * 2 * hd)
        if rows_each > 1:
            add(f"attention, {h} heads of {hd} over {kvh} kv heads, one gate per head, every earlier key, {label}", lambda: grouped(head_gate=head_gate), **gqa)
            add(f"its like: the same with capped scores and sinks (Bosenex), {label}", lambda: grouped(softcap=30.0, sinks=sinks), **gqa)
        else:
            fused = lambda **kw: ops.decode_attention_fused(  # noqa: E731
                qkv[:, : h * hd], qkv[:, h * hd: (h + kvh) * hd], qkv[:, (h + kvh) * hd:], slot_map, kv_pool, kv_pool[kvh * page * hd:], 2 * kvh * page * hd, page,
                n_entries * pages_each, tables, row_entry, positions, seq_lens, h, kvh, hd, hd ** -0.5, 0, length, exact_weights=ops.exact_weights(), **kw)
            add(f"attention with the new key's cache write in the kernel, one gate per head, {label}", lambda: fused(head_gate=head_gate), **gqa)
            add(f"its like: the same with capped scores and sinks (Bosenex), {label}", lambda: fused(softcap=30.0, sinks=sinks), **gqa)
            add(f"attention of a layer that reads another's keys (nothing to write), one gate per head, {label}",
                lambda: ops.decode_attention_fused(qkv[:, : h * hd], None, None, None, kv_pool, kv_pool[kvh * page * hd:], 2 * kvh * page * hd, page,
                                                   n_entries * pages_each, tables, row_entry, positions, seq_lens, h, kvh, hd, hd ** -0.5, 0, length,
                                                   exact_weights=ops.exact_weights(), head_gate=head_gate), **gqa)
        w_gate = torch.randn(h, d, device=dev) * 0.02
        add(f"attention: one gate per head in 32-bit, {h} outputs, {label}", lambda: ops.small_linear(hrow, w_gate, None), n_bytes=t * d * 2)
        # the mixture
        router8 = torch.randn(8, d, device=dev) * 0.02
        add(f"router: softmax over 8 experts in 32-bit, 2 of 4 groups by their best, top 2, scaled, {label}",
            lambda: ops.route_scored(hrow, router8, None, 2, 4, 2, scoring="softmax", group_mark="best", normalise=False, weight_scale=2.0), n_bytes=t * d * 2)
        router9 = torch.randn(9, d, device=dev) * 0.02
        correction = torch.randn(8, device=dev) * 0.1
        add(f"its like: 8 sigmoid scores + the shared expert's gate, 2 of 4 groups, top 2 (Zudalorn), {label}",
            lambda: ops.route_scored(hrow, router9, correction, 2, 4, 2, n_extra=1), n_bytes=t * d * 2)
        route, _, _, _ = ops.route_scored(hrow, router8, None, 2, 4, 2, scoring="softmax", group_mark="best", normalise=False, weight_scale=2.0)
        gu = torch.randn(t, 2 * 8 * (ff // 4), device=dev).to(bf)
        add(f"experts' gated silu unit with routing weights, {gu.shape[1] // 2:,} columns, {label}",
            lambda: ops.expert_act(gu, "silu", route=route, n_experts=8, expert_width=ff // 4), n_bytes=t * gu.shape[1] * 3)
        route2, _, _, sg = ops.route_scored(hrow, router9, correction, 2, 4, 2, n_extra=1)
        gu2 = torch.randn(t, 2 * 9 * (ff // 4), device=dev).to(bf)
        add(f"its like: the same with the shared expert's columns and gate (Zudalorn), {gu2.shape[1] // 2:,} columns, {label}",
            lambda: ops.expert_act(gu2, "silu", route=route2, n_experts=8, expert_width=ff // 4, tail_gate=sg), n_bytes=t * gu2.shape[1] * 3)
    out["kernels"] = table
    return out


def e2e_point(model, batch: int, steps: int, warmup: int) -> dict:
    """Through the Python entry point: submit prompts (host token lists), step, poll tokens."""
    import torch
    from research_2_b200.config.engine_options import EngineOptions
    from research_2_b200.engine.engine import Engine

    opts = EngineOptions(dtype="bfloat16", max_requests=batch, block_size=PAGE, max_batch_tokens=2048, capture=True)
    engine = Engine.for_model(model, opts)
    gen = torch.Generator().manual_seed(SEED + 200)
    prompts = torch.randint(0, model.vocab_size, (batch, PROMPT_LEN), generator=gen).tolist()
    room = CONTEXT - PROMPT_LEN   # tokens a request can still generate
    steps = max(1, min(steps, room - warmup - 6))   # (requests must stay alive through the timed steps)
    rids = [engine.submit(p, max_new_tokens=min(steps + warmup + 8, room)) for p in prompts]
    while True:  # prefill until every request decodes
        engine.step()
        if all(engine.scheduler.request_info(r)["n_tokens"] > PROMPT_LEN for r in rids):
            break
    for _ in range(warmup):
        engine.step()
    for r in rids:
        engine.poll(r)
    h0 = engine.step_fn.h2d_bytes
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n_tokens = 0
    for _ in range(steps):
        engine.step(wait=False)   # launched; the polls below run while the GPU works and see the step before
        for r in rids:
            n_tokens += len(engine.poll(r).new_tokens)
    engine.finish()
    for r in rids:
        n_tokens += len(engine.poll(r).new_tokens)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    h2d = (engine.step_fn.h2d_bytes - h0) / steps
    engine.close()
    return {"value": batch * steps / dt, "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
            "d2h_bytes_per_step": 4 * batch, "polled_tokens": n_tokens}


def mixed_point(model, n_requests: int = 64, new_tokens: int = 256) -> dict:
    """A continuous batch through the Python entry point: prompts of 16 to 768 tokens, portions
    of 512 tokens a step beside the decoded tokens of the others (the workload that the baseline
    names for the 355M size, here at the benchmark's own). The first pass captures the graphs of
    the shapes that come; the second is timed by the host's clock."""
    import random

    import torch
    from research_2_b200.config.engine_options import EngineOptions
    from research_2_b200.engine.api import generate_with
    from research_2_b200.engine.engine import Engine

    opts = EngineOptions(dtype="bfloat16", max_requests=n_requests, block_size=PAGE, max_batch_tokens=512 + n_requests, chunk_size=512,
                         capture=True)
    engine = Engine.for_model(model, opts)
    rng = random.Random(SEED + 300)
    gen = torch.Generator().manual_seed(SEED + 300)
    prompts = [torch.randint(0, model.vocab_size, (rng.randint(16, 768),), generator=gen).tolist() for _ in range(n_requests)]
    generate_with(engine, prompts, new_tokens, wait=False)
    engine.request_events()  # (the first pass's records)
    engine.keep_events = True
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    out = generate_with(engine, prompts, new_tokens, wait=False)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    steps = len(engine.events)
    records = engine.request_events()
    preempted = sum(e.n_preempted for e in engine.events)
    engine.close()
    n_out, n_in = sum(len(o) for o in out), sum(len(p) for p in prompts)
    ttft = sorted(r.time_to_first_token_ms for r in records if r.time_to_first_token_ms is not None)
    return {"generated_per_s": n_out / dt, "tokens_per_s": (n_in + n_out) / dt, "requests": n_requests,
            "prompt_tokens": n_in, "generated_tokens": n_out, "steps": steps, "ms": dt * 1e3, "preemptions": preempted,
            "ttft_ms_median": statistics.median(ttft) if ttft else None, "ttft_ms_p90": ttft[int(0.9 * (len(ttft) - 1))] if ttft else None}


def kernel_points(cfg, batch: int, pk: dict) -> dict:
    """The step's dominant kernels one by one at this configuration's sizes, each timed in a CUDA graph of
    20 launches: microseconds, and the fraction of the measured peak that its bytes (decode: the weights or
    the cache it must read) or its flops (prefill at 2,048 tokens) make of that time."""
    import torch
    from research_2_b200.profiling import kernel_cases

    kernel_cases.configure(cfg.n_embd, cfg.n_inner, cfg.n_head, cfg.head_dim, cfg.vocab_size, PAGE)
    out = {}
    for name, fn, n_bytes, flops in kernel_cases.cases(batch):
        wanted = (name.startswith("decode: ") and "sampling at" not in name and f"{batch} rows x {cfg.n_head} heads" in name or
                  name.startswith("decode: ") and " x " in name and "rows" not in name or
                  name.startswith(f"logits, {batch} rows") or name.startswith("decode: greedy") or
                  name.startswith("prefill") and "2,048" in name or "2 x 1,024" in name and "tcgen05" in name)
        if not wanted:
            continue
        us = kernel_cases.time_in_graph(fn)
        if n_bytes:
            out[name] = {"us": round(us, 2), "GB/s": round(n_bytes / us / 1e3, 1), "frac": round(n_bytes / us / 1e3 / pk["hbm_gbs"], 3)}
        else:
            out[name] = {"us": round(us, 2), "TFLOP/s": round(flops / us / 1e6, 1), "frac": round(flops / us / 1e6 / pk["bf16_tflops"], 3)}
    torch.cuda.empty_cache()
    return out


def resident_phases(model, batch: int) -> dict:
    """Where a layer's time goes inside the resident decode kernel (up to 64 rows): the kernel's own clock at
    the end of every phase and at the exit of every grid barrier (`ResidentLayers.stamps`), taken as the latest
    CTA's time minus the latest CTA's at the point before, mean over the middle layers, in microseconds."""
    import torch
    from research_2_b200.engine.step import StepContext
    from research_2_b200.kernels import ops

    before = ops.set_resident_decode_rows(64)
    try:
        loop = DecodeLoop(model, batch, 40)
        resident = getattr(model, "_resident", None)
        if resident is None:
            return {"unavailable": "the model's layers are not of the kind that the resident kernel runs"}
        n_layers = len(resident.schedule)
        n = 1 + 10 * n_layers
        ctx = StepContext(loop.graph.host, loop.graph.dev, counts=(batch, batch, batch))
        loop.run(3)
        for _ in range(3):
            stamps = torch.zeros(3 * n, dtype=torch.int64, device="cuda:0")
            stamps[n: 2 * n] = 1 << 62
            resident.stamps = stamps
            loop.step_fn.sample(loop.step_fn.forward(ctx), ctx)
            torch.cuda.synchronize()
        resident.stamps = None
        early, late = stamps[n: 2 * n].cpu().tolist(), stamps[2 * n:].cpu().tolist()
        names = ["A norm + q/k/v", "barrier", "B attention", "barrier", "C output + residual", "barrier", "D norm + feed-forward in", "barrier",
                 "E feed-forward out + residual", "barrier"]
        layers = range(min(3, n_layers - 1), max(min(3, n_layers - 1) + 1, n_layers - 1))
        out = {"rows": batch, "kernel_us": (late[-1] - early[0]) / 1e3, "phases_us": []}
        for i, name in enumerate(names):
            spans = [(late[1 + 10 * layer + i] - late[10 * layer + i]) / 1e3 for layer in layers]
            out["phases_us"].append([name, round(sum(spans) / len(spans), 2)])
        return out
    finally:
        ops.set_resident_decode_rows(before)


def logits_ctas(model, batch: int) -> dict:
    """How the CTAs of a decode step's last product (the logits) share the GPU: every CTA's own times
    (`ops.gemm_cta_stamps`), in microseconds from the first CTA's start."""
    import torch
    from research_2_b200.kernels import ops

    stamps = torch.zeros(2048, 6, dtype=torch.int64, device="cuda:0")
    ops.gemm_cta_stamps(stamps)
    try:
        loop = DecodeLoop(model, batch, 40)   # (the graph is captured with the buffer in the kernels' arguments)
        loop.run(6)
        torch.cuda.synchronize()
        n = min(ops.gemm_cta_stamps(None), stamps.shape[0])
    finally:
        ops.gemm_cta_stamps(None)
    from research_2_b200.profiling.kernel_cases import summarise_cta_stamps

    return {"rows": batch, **summarise_cta_stamps(stamps, n)}


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--model", default="gpt2-124M", choices=sorted(SIZES), help="layer sizes (the default is the baseline's benchmark configuration)")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has, if memory or time needs it")
    ap.add_argument("--no-points", action="store_true", help="skip prefill, e2e and the batch 1 / 64 points")
    ap.add_argument("--phases", action="store_true", help="print where a layer's time goes inside the resident decode kernel at --batch rows, and stop")
    ap.add_argument("--logits-ctas", action="store_true", help="print when each CTA of a decode step's logits product starts and ends (its waves), and stop")
    ap.add_argument("--prefill", action="store_true", help="print the prefill point (2 x 1,024 tokens in one step) alone, and stop")
    ap.add_argument("--design", default=None, choices=("zirunex", "bosenex", "zudalorn", "pidodra"),
                    help="print prefill and decode throughput of that design at the layer sizes of --model beside GPT-2's, "
                         "and its kernels beside their likes, and stop (the default workload is GPT-2's)")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.layers is None:
        args.layers = SIZES[args.model]["n_layer"]
    global PROMPT_LEN
    PROMPT_LEN = PROMPT_LENS[args.model]
    steps = min(args.steps, CONTEXT - PROMPT_LEN - args.warmup)
    if args.impl == "reference":
        from baseline import reference_arm

        cfg_data = SIZES[args.model]
        skeleton = {
            "metric": f"decode tokens/s (GPT-2 {args.model[5:]}, batch {args.batch}, {PROMPT_LEN}-token prompts)", "value": None, "unit": "tokens/s",
            "n_gpus": 1, "steps": steps, "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic tokens, random weights (seed 5)", "impl": "reference",
            "config": {"model": args.model, "n_layer": cfg_data["n_layer"], "n_layer_model": cfg_data["n_layer"], "n_embd": cfg_data["n_embd"],
                       "n_head": cfg_data["n_head"], "head_dim": cfg_data["n_embd"] // cfg_data["n_head"], "n_inner": cfg_data["n_inner"],
                       "vocab_size": cfg_data["vocab_size"], "n_positions": cfg_data["n_positions"], "global_batch": args.batch,
                       "seq_len": CONTEXT, "prompt_len": PROMPT_LEN, "page_size": PAGE, "parallelism": "none",
                       "l2": "inputs larger than L2, no flush"},
        }
        return reference_arm.main(args, cfg_data, SEED, PAGE, PROMPT_LEN, CONTEXT, skeleton)

    import torch
    from research_2_b200.kernels import ops

    pk, pk_source = peaks()
    if args.design:
        points = {"bosenex": bosenex_points, "zudalorn": zudalorn_points, "pidodra": pidodra_points}.get(args.design, design_points)
        print(json.dumps(points(args, pk)))
        return 0
    model, cfg = build_model(args.layers, size=args.model)
    if args.phases:
        print(json.dumps(resident_phases(model, args.batch)))
        return 0
    if args.prefill:
        print(json.dumps(prefill_point(model, cfg, pk)))
        return 0
    if args.logits_ctas:
        print(json.dumps(logits_ctas(model, args.batch)))
        return 0
    sampler = ClockSampler()
    sampler.start()
    before = ops.launch_count()
    value, ms_per_step, loop, kv_bytes = decode_point(model, args.batch, steps, args.warmup)
    launches = loop.graph.kernels * steps
    clocks = sampler.stop()
    del before
    weight_bytes = model.weight_bytes_per_step()
    achieved = (weight_bytes + kv_bytes) / (ms_per_step / 1e3) / 1e9
    del loop
    torch.cuda.empty_cache()

    line = {
        "metric": f"decode tokens/s (GPT-2 {args.model[5:]}, batch {args.batch}, {PROMPT_LEN}-token prompts)", "value": value, "unit": "tokens/s",
        "n_gpus": 1, "steps": steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic tokens, random weights (seed 5)",
        "impl": "ours",
        "config": {
            "model": args.model, "n_layer": args.layers, "n_layer_model": SIZES[args.model]["n_layer"], "n_embd": cfg.n_embd,
            "n_head": cfg.n_head, "head_dim": cfg.head_dim, "n_inner": cfg.n_inner, "vocab_size": cfg.vocab_size,
            "n_positions": cfg.n_positions, "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN,
            "page_size": PAGE, "parallelism": "none", "l2": "inputs larger than L2, no flush", "peaks": pk_source,
        },
        "clocks": clocks, "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"]},
    }
    if not args.no_points:
        line["prefill"] = prefill_point(model, cfg, pk)
        torch.cuda.empty_cache()
        line["e2e"] = e2e_point(model, args.batch, min(steps, 128), args.warmup)
        torch.cuda.empty_cache()
        points = {}
        for b in (1, 64):
            v, _, lp, _ = decode_point(model, b, min(steps, 96), args.warmup)
            points[f"decode_b{b}"] = v
            del lp
            torch.cuda.empty_cache()
        line["points"] = points
        line["mixed"] = mixed_point(model)
        torch.cuda.empty_cache()
        line["kernels"] = kernel_points(cfg, args.batch, pk)
        # the true 32-bit path of the same model (CUDA-core products and attention, no tensor cores)
        del model
        torch.cuda.empty_cache()
        model32, _ = build_model(args.layers, dtype="float32", size=args.model)
        v32, ms32, lp, _ = decode_point(model32, args.batch, min(steps, 24), args.warmup)
        points[f"decode_b{args.batch}_float32"] = v32
        del lp
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
