"""Measurement: decode tokens a second at a batch size, prefill tokens a second, the same
end to end through the Python entry point, and the fractions of the roofline.

Shapes are those of the benchmark configurations (Llama 3.2 1B, 3.2 3B, 3.1 8B) with random
weights drawn on the device; prompts are seeded uniform token ids. The reference's own
bench loads a model once and times generate runs (src/main.rs:4152-4274); its decode rate
leaves out the first token (src/main.rs:4229-4235), as the decode numbers here do.

Timing: CUDA events on the launching stream around exactly K decode steps after W warm-up
steps; every step reads all weights (gigabytes, far more than the 126 MB of L2), so the
inputs themselves are larger than L2. Clocks are sampled with nvidia-smi meanwhile.
"""
from __future__ import annotations

import copy
import json
import os
import statistics
import subprocess
import threading
import time

import numpy as np
import torch

_ROPE_32 = {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
            "original_max_position_embeddings": 8192}
SHAPES = {
    2: dict(name="llama-3.2-1b", num_hidden_layers=16, hidden_size=2048, num_attention_heads=32, num_key_value_heads=8,
            head_dim=64, intermediate_size=8192, vocab_size=128256, rope_theta=500000.0, rope_scaling=_ROPE_32,
            rms_norm_eps=1e-5, tie_word_embeddings=True, seed=2, context=4096),
    3: dict(name="llama-3.2-3b", num_hidden_layers=28, hidden_size=3072, num_attention_heads=24, num_key_value_heads=8,
            head_dim=128, intermediate_size=8192, vocab_size=128256, rope_theta=500000.0, rope_scaling=_ROPE_32,
            rms_norm_eps=1e-5, tie_word_embeddings=True, seed=3, context=4096),
    4: dict(name="llama-3.1-8b", num_hidden_layers=32, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
            head_dim=128, intermediate_size=14336, vocab_size=128256, rope_theta=500000.0,
            rope_scaling={**_ROPE_32, "factor": 8.0}, rms_norm_eps=1e-5, tie_word_embeddings=False, seed=4, context=8192),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def config_for(index: int, layers: int | None = None) -> dict:
    s = dict(SHAPES[index])
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "max_position_embeddings": 131072,
           **{k: v for k, v in s.items() if k not in ("name", "seed", "context")}}
    if layers:
        cfg["num_hidden_layers"] = layers
    return cfg


def peaks(repo_root: str | None = None) -> dict:
    root = repo_root or os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                if isinstance(d.get(k), (int, float)) and d[k] > 0:
                    out[k] = float(d[k])
            out["source"] = "measured"
            return out
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int = 0):
        self.samples: list = []
        self.proc = None
        self.thread = None
        self.device_index = device_index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.device_index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        for p in self.samples:
            try:
                sm.append(float(p[0]))
                mx.append(float(p[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def _prompts(rng, n: int, length, vocab: int) -> list:
    """``n`` prompts of seeded uniform ids; ``length`` is one number or (lowest, highest) for
    lengths drawn uniformly between the two."""
    if isinstance(length, (tuple, list)):
        lengths = rng.integers(int(length[0]), int(length[1]) + 1, size=n).tolist()
    else:
        lengths = [int(length)] * n
    return [rng.integers(0, vocab, size=t).tolist() for t in lengths]


def linear_params(cfg: dict) -> int:
    h, i, l = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    return l * (h * (q + 2 * kv) + q * h + 3 * h * i)


def prefill_flops(cfg: dict, tokens: int, wanted: int = 1) -> float:
    attn = 2.0 * tokens * tokens * cfg["num_attention_heads"] * cfg["head_dim"] * cfg["num_hidden_layers"]   # causal: half of 4 T^2
    return 2.0 * tokens * linear_params(cfg) + attn + 2.0 * wanted * cfg["hidden_size"] * cfg["vocab_size"]


def decode_bytes(cfg: dict, batch: int, context: float, elem: int) -> float:
    """Bytes a decode step has to read: every weight it uses once, and the cache of the live requests."""
    weights = (linear_params(cfg) + cfg["hidden_size"] * cfg["vocab_size"]
               + (2 * cfg["num_hidden_layers"] + 1) * cfg["hidden_size"]) * elem
    kv = 2 * cfg["num_hidden_layers"] * cfg["num_key_value_heads"] * cfg["head_dim"] * elem * context * batch
    return weights + kv


def measure_prefill(lm, cfg, tokens: int, rng, reps: int = 5, warmup: int = 3) -> dict:
    from .engine.model import StepEntry
    cache = lm.new_cache(((tokens + 63) // 64) * 64, max_slots=1)
    prompt = _prompts(rng, 1, tokens, cfg["vocab_size"])[0]
    times = []
    for r in range(warmup + reps):
        slot = cache.alloc_slot()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        lm.step(cache, [StepEntry(slot, prompt, [tokens - 1])])
        b.record()
        torch.cuda.synchronize()
        cache.free_slot(slot)
        if r >= warmup:
            times.append(a.elapsed_time(b))
    ms = statistics.median(times)
    del cache
    return {"ms": ms, "tokens": tokens, "value": tokens / (ms / 1e3)}


def measure_prefill_batch(lm, cfg, prompts, reps: int = 3, warmup: int = 2) -> dict:
    """All prompts of a batch, of unequal lengths, in one step."""
    from .engine.model import StepEntry
    cache = lm.new_cache(sum(((len(p) + 63) // 64) * 64 for p in prompts), max_slots=len(prompts))
    times = []
    for r in range(warmup + reps):
        slots = [cache.alloc_slot() for _ in prompts]
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        lm.step(cache, [StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        b.record()
        torch.cuda.synchronize()
        for s in slots:
            cache.free_slot(s)
        if r >= warmup:
            times.append(a.elapsed_time(b))
    ms = statistics.median(times)
    del cache
    tokens = sum(len(p) for p in prompts)
    return {"ms": ms, "tokens": tokens, "value": tokens / (ms / 1e3), "prompts": len(prompts),
            "shortest": min(len(p) for p in prompts), "longest": max(len(p) for p in prompts),
            "flops": sum(prefill_flops(cfg, len(p)) for p in prompts)}


def _prefill_batch(lm, cache, prompts, chunk: int = 8):
    """Prefill all prompts (a few per step, to bound the workspace); returns slots and the
    greedy first token of each."""
    from .engine.model import StepEntry
    slots, firsts = [], []
    for i in range(0, len(prompts), chunk):
        part = prompts[i:i + chunk]
        s = [cache.alloc_slot() for _ in part]
        logits = lm.step(cache, [StepEntry(sl, p, [len(p) - 1]) for sl, p in zip(s, part)])
        firsts += logits.argmax(dim=-1).to(torch.int32).tolist()
        slots += s
    return slots, firsts


def measure_decode_device(lm, cfg, batch: int, prompt_tokens, steps: int, warmup: int, rng, prompts=None,
                          sampling=None) -> dict:
    """K decode steps timed on the device, in the loop that ``generate`` runs
    (``DecoderModel.decode_fed``): the captured step graph picks each token and feeds it back on the
    device; per step the host sends the positions from pinned memory and reads the chosen tokens.
    CUDA events bracket exactly the K steps. ``prompt_tokens`` is one length or (lowest, highest);
    ``prompts`` given wins over it. ``sampling`` (``SamplingOptions``): None is greedy; with penalties
    the prompts and what is generated are the histories."""
    from .csrc import ops
    if prompts is None:
        prompts = _prompts(rng, batch, prompt_tokens, cfg["vocab_size"])
    cache = lm.new_cache(sum(((len(p) + steps + warmup + 1 + 63) // 64) * 64 for p in prompts), max_slots=batch)
    slots, firsts = _prefill_batch(lm, cache, prompts)
    model = lm.model
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    adjusts = sampling is not None and sampling.adjusts
    with ClockSampler() as clocks:
        hist = [list(p) + [int(f)] for p, f in zip(prompts, firsts)] if adjusts else None
        warm = model.decode_fed(cache, slots, firsts, warmup, sampling, histories=hist)
        if adjusts:
            hist = [h + [int(t) for t in warm[:, j]] for j, h in enumerate(hist)]
        torch.cuda.synchronize()
        launches0 = ops.launch_count()
        ev0.record()
        model.decode_fed(cache, slots, warm[-1].tolist(), steps, sampling, histories=hist)
        ev1.record()
        torch.cuda.synchronize()
    launches = ops.launch_count() - launches0
    model.check_device_errors()
    ms = ev0.elapsed_time(ev1)
    h2d = model.last_h2d_bytes
    model.drop_graphs(cache)
    for s in slots:
        cache.free_slot(s)
    return {"ms_total": ms, "ms_per_step": ms / steps, "value": batch * steps / (ms / 1e3), "launches": launches,
            "h2d_bytes_per_step": h2d, "clocks": clocks.summary(),
            "context": sum(len(p) for p in prompts) / float(batch) + warmup + steps / 2.0}


def measure_decode_e2e(lm, cfg, batch: int, prompt_tokens, steps: int, warmup: int, rng, prompts=None) -> dict:
    """The same through ``LanguageModel.generate``, the call a user makes: every step sends its
    tokens and positions from pinned host memory and reads the sampled tokens back. Two calls
    on the same prompts, one that stops after the warm-up steps and one that goes on for
    ``steps`` more; the difference of their wall-clock times is the time of exactly those steps."""
    if prompts is None:
        prompts = _prompts(rng, batch, prompt_tokens, cfg["vocab_size"])

    def timed(n_tokens):
        best = None
        for _ in range(2):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            out = lm.generate(prompts, max_tokens=n_tokens, stop_token_ids=())
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            assert all(len(o) == n_tokens for o in out)
            best = dt if best is None else min(best, dt)
        return best

    lm.generate(prompts, max_tokens=warmup + steps + 1, stop_token_ids=())        # graphs captured, buffers made
    short, long = timed(warmup + 1), timed(warmup + steps + 1)
    dt = long - short
    return {"value": batch * steps / dt, "ms_per_step": dt / steps * 1e3, "h2d_bytes_per_step": lm.model.last_h2d_bytes,
            "d2h_bytes_per_step": batch * 4}


FP32_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12        # plain FMA on every lane of 148 SMs at 1,965 MHz: nominal, 74.4


SAMPLED = "temperature 0.8, top-k 40, top-p 0.9, repeat 1.1, presence 0.1"


def _sampled_options(cfg):
    from .sampling import SamplingOptions
    return SamplingOptions(temperature=0.8, top_k=40, top_p=0.9, seed=1, repeat_penalty=1.1,
                           presence_penalty=0.1).validate(cfg["vocab_size"])


def _roofline(cfg, batch, dec, elem, pk) -> dict:
    bytes_step = decode_bytes(cfg, batch, dec["context"], elem)
    achieved = bytes_step / (dec["ms_per_step"] / 1e3) / 1e9
    return {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
            "bytes": bytes_step}


def run(batch: int = 8, prompt_tokens: int = 2048, decode_steps: int = 256, warmup: int = 8, dtype: str = "bfloat16",
        layers: int | None = None, config_index: int = 2, points: bool = True, e2e: bool = True,
        prefill_tokens: int = 2048, prefill: bool = True, decode: bool = True, prompt_range=None,
        fp32: bool = False, fp32_steps: int = 32, sampled: bool = False) -> dict:
    """``prompt_range`` (lowest, highest): prompts of unequal lengths drawn uniformly between the
    two instead of ``prompt_tokens`` each; the record then also times their one prefill step.
    ``fp32``: the same decode step and prefill again with a float32 model, as an ``fp32`` object.
    ``sampled``: the timed decode steps pick their tokens with the stochastic sampler and its
    adjustments (``SAMPLED``) instead of the argmax; the record says so in ``config``."""
    from . import api
    shape = SHAPES[config_index]
    cfg = config_for(config_index, layers)
    pk = peaks()
    lm = api.from_random(cfg, seed=shape["seed"], dtype=dtype)
    rng = np.random.default_rng(shape["seed"])
    elem = 2 if dtype == "bfloat16" else 4
    flop_peak = (pk["bf16_tflops"] if dtype == "bfloat16" else FP32_TFLOPS) * 1e12
    def timed_prefill():
        if not prefill:
            return {"value": None, "tokens": prefill_tokens, "ms": None, "frac": None}
        pre = measure_prefill(lm, cfg, prefill_tokens, rng)
        pre["frac"] = prefill_flops(cfg, prefill_tokens) / (pre["ms"] / 1e3) / flop_peak
        return pre
    if not decode:
        return {"prefill": timed_prefill(), "dtype": dtype,
                "config": {"model": shape["name"], "layers": cfg["num_hidden_layers"]}}
    # The decode steps are timed first: seconds of dense prefill products put the GPU under its power cap,
    # and the steps right behind them would be timed at the clocks that leaves.
    prompts = _prompts(rng, batch, prompt_range, cfg["vocab_size"]) if prompt_range else None
    dec = measure_decode_device(lm, cfg, batch, prompt_tokens, decode_steps, warmup, rng, prompts=prompts,
                                sampling=_sampled_options(cfg) if sampled else None)
    pre = timed_prefill()
    pre_batch = None
    if prompts is not None and prefill:
        pre_batch = measure_prefill_batch(lm, cfg, prompts)
        pre_batch["frac"] = pre_batch.pop("flops") / (pre_batch["ms"] / 1e3) / flop_peak
    roof = _roofline(cfg, batch, dec, elem, pk)
    e2e_steps = max(decode_steps, 128)
    rec = {
        "metric": "decode tokens/s, Llama 3.2 1B shape, batch 8 (2048-token prompts)" if (config_index, batch) == (2, 8)
                  else f"decode tokens/s, {shape['name']} shape, batch {batch}",
        "value": dec["value"], "unit": "tokens/s", "n_gpus": 1, "steps": decode_steps, "warmup": warmup,
        "ms_per_step": dec["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if dtype == "bfloat16" else "fp32", "data": "synthetic (seeded uniform token ids, random weights)",
        "config": {"model": shape["name"], "global_batch": batch, "seq_len": shape["context"],
                   "prompt_tokens": prompt_tokens if prompts is None else f"uniform in {list(prompt_range)}",
                   "decode_steps": decode_steps, "parallelism": "single-gpu",
                   "layers": cfg["num_hidden_layers"], "layers_of_model": shape["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "tied": cfg["tie_word_embeddings"], "weights": f"random, seed {shape['seed']}",
                   "l2": "inputs larger than L2 (every step reads all weights)", "peaks": pk["source"],
                   "e2e_steps": e2e_steps, "fp32_steps": fp32_steps if fp32 else 0,
                   **({"sampling": SAMPLED} if sampled else {})},
        "prefill": {"value": pre["value"], "tokens": pre["tokens"], "ms": pre["ms"], "frac": pre["frac"]},
        "roofline": {k: roof[k] for k in ("bound", "achieved", "peak", "unit", "frac")},
        "clocks": dec["clocks"], "gpu_launches": dec["launches"],
    }
    if pre_batch is not None:
        rec["prefill_batch"] = pre_batch
    if e2e:
        e = measure_decode_e2e(lm, cfg, batch, prompt_tokens, e2e_steps, warmup, rng, prompts=prompts)
        rec["e2e"] = {"value": e["value"], "unit": "tokens/s", "h2d_bytes_per_step": e["h2d_bytes_per_step"],
                      "d2h_bytes_per_step": e["d2h_bytes_per_step"], "ms_per_step": e["ms_per_step"], "steps": e2e_steps}
    if points:
        pts, detail = {}, {}
        for b in (1, 64):
            d = dec if b == batch else measure_decode_device(lm, cfg, b, prompt_tokens, min(decode_steps, 64),
                                                             min(warmup, 4), rng)
            r = _roofline(cfg, b, d, elem, pk)
            pts[f"decode_b{b}"] = d["value"]
            detail[f"decode_b{b}"] = {"value": d["value"], "ms_per_step": d["ms_per_step"], "bytes": r["bytes"],
                                      "frac": r["frac"]}
        # the same steps with the stochastic sampler and its adjustments in the graph (not a key of `points`:
        # those are the two batch sizes the bench line promises)
        d = measure_decode_device(lm, cfg, batch, prompt_tokens, min(decode_steps, 64), min(warmup, 4), rng,
                                  sampling=_sampled_options(cfg))
        detail[f"decode_b{batch}_sampled"] = {"value": d["value"], "ms_per_step": d["ms_per_step"], "sampling": SAMPLED}
        rec["points"] = pts
        rec["points_detail"] = detail
    if fp32 and dtype == "bfloat16":
        del lm
        torch.cuda.empty_cache()
        lm32 = api.from_random(cfg, seed=shape["seed"], dtype="float32")
        d = measure_decode_device(lm32, cfg, batch, prompt_tokens, fp32_steps, 3, rng)
        r = _roofline(cfg, batch, d, 4, pk)
        p32 = measure_prefill(lm32, cfg, prefill_tokens, rng, reps=3, warmup=3)
        rec["fp32"] = {"value": d["value"], "ms_per_step": d["ms_per_step"], "bytes": r["bytes"], "frac": r["frac"],
                       "steps": fp32_steps,
                       "prefill": {"value": p32["value"], "tokens": p32["tokens"], "ms": p32["ms"],
                                   "frac": prefill_flops(cfg, prefill_tokens) / (p32["ms"] / 1e3) / (FP32_TFLOPS * 1e12),
                                   "peak_tflops": FP32_TFLOPS}}
    return rec


# ---------------------------------------------------------------------------------------
# Fomatar beside the dense Llama decoder at equal width, depth and feed-forward size

FOMATAR_SIZES = {
    # width, layers (channel_delta and parallel in turn; every parallel layer has the feed-forward),
    # heads of `head` channels, window of the attention branch
    "small": dict(width=1024, layers=8, ff=4096, heads=8, kv_heads=2, head=128, window=512, vocab=32768),
    "medium": dict(width=2048, layers=16, ff=8192, heads=16, kv_heads=4, head=128, window=1024, vocab=32768),
    "wide": dict(width=4096, layers=8, ff=14336, heads=32, kv_heads=8, head=128, window=1024, vocab=32768),
}


def fomatar_config_for(size: str) -> dict:
    s = FOMATAR_SIZES[size]
    heads, head = s["heads"], s["head"]
    layers = []
    for i in range(s["layers"]):
        if i % 2 == 0:
            layers.append({"type": "channel_delta", "mlp": None,
                           "mixer": {"conv": 4, "dim": head, "vdim": head, "heads": heads, "kv_heads": heads, "rank": 64}})
        else:
            layers.append({"type": "parallel", "mlp": {"kind": "dense", "ff": s["ff"]},
                           "mixer": {"left": {"dim": head, "vdim": head, "heads": heads, "kv_heads": s["kv_heads"],
                                              "mask": {"size": s["window"]}, "scale": head ** -0.5},
                                     "right": {"dim": head, "vdim": head, "heads": heads // 2, "gate_cap": 15.0}}})
    return {"architecture": "Fomatar", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6},
            "logit_softcap": 30.0, "embedding": {"bigram": {"buckets": 65521, "mul_prev": 1000003, "mul_cur": 31}},
            "layers": layers}


def llama_config_like(size: str) -> dict:
    """The dense Llama decoder of the same width, depth, feed-forward size, heads and vocabulary."""
    s = FOMATAR_SIZES[size]
    return {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "max_position_embeddings": 131072,
            "num_hidden_layers": s["layers"], "hidden_size": s["width"], "num_attention_heads": s["heads"],
            "num_key_value_heads": s["kv_heads"], "head_dim": s["head"], "intermediate_size": s["ff"],
            "vocab_size": s["vocab"], "rope_theta": 500000.0, "rope_scaling": None, "rms_norm_eps": 1e-6,
            "tie_word_embeddings": False}


def model_step_bytes(lm, batch: int, context: float) -> dict:
    """Bytes a decode step of ``batch`` sequences at ``context`` positions must move: every matrix and vector once
    (of an embedding table only the rows it reads), the keys and values a query can see, every state read and written."""
    from .cache.book import KVSpec, StateSpec, flatten_specs
    from .cache.sequence_cache import _STATE_DTYPES
    m = lm.model
    elem = 2 if m.dtype == torch.bfloat16 else 4
    tables = set(m.embedding.tensor_specs())
    weights = sum(int(np.prod(sp.shape)) * elem for n, sp in m.tensor_specs().items() if n not in tables)
    kv = state = 0
    for needs, src in zip(m.entry_cache_specs(), m.entry_cache_sources()):
        for sp in flatten_specs(needs):
            if isinstance(sp, KVSpec):
                seen = min(context, sp.window) if sp.window else context
                kv += (0 if src is not None else 0) + batch * seen * sp.n_kv_heads * (sp.head_dim + sp.value_dim) * elem
            elif isinstance(sp, StateSpec) and src is None:
                state += 2 * batch * int(np.prod(sp.shape)) * torch.empty((), dtype=_STATE_DTYPES[sp.dtype]).element_size()
    return {"weights": weights, "kv": int(kv), "state": state, "total": int(weights + kv + state)}


def model_prefill_flops(lm, tokens: int) -> float:
    """2 x tokens x (elements of every matrix a token passes) plus the mixers' own work: attention over the visible
    keys, and per token and head of a recurrent mixer the update and the read-out of its matrix state."""
    from .cache.book import KVSpec, StateSpec, flatten_specs
    m = lm.model
    tables = set(m.embedding.tensor_specs())
    per_layer = {}
    for n, sp in m.tensor_specs().items():
        if n not in tables and len(sp.shape) == 2 and "conv" not in n and not n.startswith(("loop.", "head", "lm_head")):
            per_layer[n] = int(np.prod(sp.shape))
    runs = {}
    for e in m.schedule:
        runs[e.layer] = runs.get(e.layer, 0) + 1
    total = 0.0
    names = {i: [n for n in per_layer if n in m.blocks[i].tensor_specs()] for i in range(len(m.blocks))}
    for i, r in runs.items():
        total += 2.0 * tokens * r * sum(per_layer[n] for n in names[i])
    for needs in m.entry_cache_specs():
        for sp in flatten_specs(needs):
            if isinstance(sp, KVSpec):
                seen = min(tokens, sp.window) if sp.window else tokens / 2.0
                heads = getattr(sp, "n_kv_heads")
                total += 2.0 * tokens * seen * heads * (sp.head_dim + sp.value_dim)      # per kv head; query groups below
            elif isinstance(sp, StateSpec) and sp.name == "memory":
                total += 6.0 * tokens * int(np.prod(sp.shape))
    return total


def _prefill_together(lm, prompts, reps: int = 3, warmup: int = 2) -> dict:
    """All prompts in one step (the recurrent mixers walk the sequences side by side)."""
    from .engine.model import StepEntry
    cache = lm.new_cache(sum(((len(p) + 63) // 64) * 64 for p in prompts), max_slots=len(prompts))
    times = []
    for r in range(warmup + reps):
        slots = [cache.alloc_slot() for _ in prompts]
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        lm.step(cache, [StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        b.record()
        torch.cuda.synchronize()
        for s in slots:
            cache.free_slot(s)
        if r >= warmup:
            times.append(a.elapsed_time(b))
    ms = statistics.median(times)
    lm.model.drop_graphs(cache)
    return {"ms": ms, "tokens": sum(len(p) for p in prompts), "value": sum(len(p) for p in prompts) / (ms / 1e3)}


def run_fomatar(sizes=("small", "medium"), batch: int = 8, prompt_tokens: int = 512, steps: int = 64, warmup: int = 4,
                prefill_tokens: int = 2048, dtype: str = "bfloat16") -> dict:
    """Decode steps (timed on the device in the loop ``generate`` runs) and one prefill step of the Fomatar decoder
    and of the dense Llama decoder of equal width, depth, feed-forward size and vocabulary, random weights."""
    from . import api
    pk = peaks()
    out = {"metric": "decode and prefill tokens/s, Fomatar beside the dense decoder of equal size", "dtype": dtype,
           "batch": batch, "prompt_tokens": prompt_tokens, "steps": steps, "warmup": warmup,
           "prefill_tokens": prefill_tokens, "peaks": pk["source"], "data": "synthetic (seeded uniform token ids, random weights)",
           "sizes": {}}
    for size in sizes:
        rec = {"shape": FOMATAR_SIZES[size]}
        for label, cfg in (("fomatar", fomatar_config_for(size)), ("llama", llama_config_like(size))):
            lm = api.from_random(cfg, seed=7, dtype=dtype)
            vocab = {"vocab_size": FOMATAR_SIZES[size]["vocab"]}
            rng = np.random.default_rng(7)
            dec = measure_decode_device(lm, vocab, batch, prompt_tokens, steps, warmup, rng)
            bytes_step = model_step_bytes(lm, batch, dec["context"])
            pre = measure_prefill(lm, vocab, prefill_tokens, rng)
            flops = model_prefill_flops(lm, prefill_tokens) if label == "fomatar" else prefill_flops(cfg, prefill_tokens)
            together = _prefill_together(lm, _prompts(rng, batch, prompt_tokens, vocab["vocab_size"]))
            rec[label] = {
                "decode_tokens_per_s": dec["value"], "decode_ms_per_step": dec["ms_per_step"], "launches_per_step": dec["launches"] / steps,
                "decode_bytes": bytes_step, "decode_frac_of_copy": bytes_step["total"] / (dec["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"],
                "prefill_tokens_per_s": pre["value"], "prefill_ms": pre["ms"],
                "prefill_batch_tokens_per_s": together["value"], "prefill_batch_ms": together["ms"],
                "prefill_frac_of_gemm": flops / (pre["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12) if dtype == "bfloat16" else None,
                "clocks": dec["clocks"]}
            del lm
            torch.cuda.empty_cache()
        out["sizes"][size] = rec
    return out


ZULOZEN_SIZES = {
    # width, layers (dense and routed feed-forwards in turn), feed-forward size of the dense layers, heads of `head`
    # channels, block of positions a query sees, experts / choices / expert size / shared expert size of the routed
    # layers (choices * expert + shared = ff: a token passes as many feed-forward elements as in a dense layer)
    "small": dict(width=1024, layers=8, ff=4096, heads=8, kv_heads=2, head=128, block=512, experts=16, top=2, expert_ff=1024,
                  shared_ff=2048, vocab=32768),
    "medium": dict(width=2048, layers=16, ff=8192, heads=16, kv_heads=4, head=128, block=1024, experts=32, top=4, expert_ff=1536,
                   shared_ff=2048, vocab=32768),
    "wide": dict(width=4096, layers=8, ff=14336, heads=32, kv_heads=8, head=128, block=1024, experts=32, top=4, expert_ff=2560,
                 shared_ff=4096, vocab=32768),
}


def zulozen_config_for(size: str) -> dict:
    s = ZULOZEN_SIZES[size]
    mixer = {"dim": s["head"], "vdim": s["head"], "heads": s["heads"], "kv_heads": s["kv_heads"], "mask": {"size": s["block"]},
             "rot": {"dims": s["head"] // 2, "base": 10000.0}, "scale": s["head"] ** -0.5}
    layers = []
    for i in range(s["layers"]):
        mlp = ({"kind": "dense", "ff": s["ff"]} if i % 2 == 0 else
               {"kind": "moe", "expert": {"ff": s["expert_ff"]}, "router": {"experts": s["experts"], "top": s["top"]},
                "shared": {"ff": s["shared_ff"]}})
        layers.append({"type": "attention", "mixer": dict(mixer), "mlp": mlp})
    return {"architecture": "Zulozen", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6}, "residual_mult": 0.5,
            "layers": layers}


def llama_config_like_zulozen(size: str) -> dict:
    """The dense Llama decoder of the same width, depth, heads, feed-forward size and vocabulary."""
    s = ZULOZEN_SIZES[size]
    return {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "max_position_embeddings": 131072,
            "num_hidden_layers": s["layers"], "hidden_size": s["width"], "num_attention_heads": s["heads"],
            "num_key_value_heads": s["kv_heads"], "head_dim": s["head"], "intermediate_size": s["ff"],
            "vocab_size": s["vocab"], "rope_theta": 500000.0, "rope_scaling": None, "rms_norm_eps": 1e-6,
            "tie_word_embeddings": False}


def zulozen_step_bytes(cfg: dict, batch: int, context: float, elem: int) -> dict:
    """Bytes a decode step must move: every matrix a row passes once (of the routed experts as many as ``batch`` rows
    with ``top`` choices each reach on average when the choices are uniform, E (1 - (1 - top / E)^batch); the output
    head, no embedding table), and the keys and values of each sequence's running block of positions."""
    W = cfg["width"]
    weights = kv = 0
    for L in cfg["layers"]:
        m, f = L["mixer"], L["mlp"]
        weights += W * (m["heads"] * m["dim"] + m["kv_heads"] * (m["dim"] + m["vdim"]) + m["heads"]) + m["heads"] * m["vdim"] * W
        if f and f["kind"] == "dense":
            weights += 2 * W * f["ff"]
        elif f:
            reach = f["router"]["experts"] * (1.0 - (1.0 - f["router"]["top"] / f["router"]["experts"]) ** batch)
            weights += W * f["router"]["experts"] + 3 * W * (reach * f["expert"]["ff"] + (f.get("shared") or {"ff": 0})["ff"])
        seen = min(context, (context % m["mask"]["size"]) + 1) if m.get("mask") else context
        kv += batch * seen * m["kv_heads"] * (m["dim"] + m["vdim"])
    weights += cfg["vocab"] * W
    return {"weights": int(weights * elem), "kv": int(kv * elem), "state": 0, "total": int((weights + kv) * elem)}


def zulozen_prefill_flops(cfg: dict, tokens: int) -> float:
    """2 x tokens x (elements of every matrix a token passes: of the routed experts its ``top`` choices and the shared
    one) plus the attention over the keys of each query's own block of positions."""
    W = cfg["width"]
    total = 0.0
    for L in cfg["layers"]:
        m, f = L["mixer"], L["mlp"]
        per = W * (m["heads"] * m["dim"] + m["kv_heads"] * (m["dim"] + m["vdim"]) + m["heads"]) + m["heads"] * m["vdim"] * W
        if f and f["kind"] == "dense":
            per += 2 * W * f["ff"]
        elif f:
            per += W * f["router"]["experts"] + 3 * W * (f["router"]["top"] * f["expert"]["ff"] + (f.get("shared") or {"ff": 0})["ff"])
        total += 2.0 * tokens * per
        block = m["mask"]["size"] if m.get("mask") else tokens
        seen = sum((i % block) + 1 for i in range(tokens))
        total += 2.0 * seen * m["heads"] * (m["dim"] + m["vdim"])
    return total + 2.0 * W * cfg["vocab"]


def run_zulozen(sizes=("small", "medium"), batch: int = 8, prompt_tokens: int = 512, steps: int = 64, warmup: int = 4,
                prefill_tokens: int = 2048, dtype: str = "bfloat16") -> dict:
    """Decode steps (timed on the device in the loop ``generate`` runs) and prefill steps of the Zulozen decoder and of
    the dense Llama decoder of equal width, depth, heads, feed-forward size and vocabulary, random weights."""
    from . import api
    pk = peaks()
    elem = 2 if dtype == "bfloat16" else 4
    out = {"metric": "decode and prefill tokens/s, Zulozen beside the dense decoder of equal size", "dtype": dtype,
           "batch": batch, "prompt_tokens": prompt_tokens, "steps": steps, "warmup": warmup,
           "prefill_tokens": prefill_tokens, "peaks": pk["source"], "data": "synthetic (seeded uniform token ids, random weights)",
           "sizes": {}}
    for size in sizes:
        rec = {"shape": ZULOZEN_SIZES[size]}
        for label, cfg in (("zulozen", zulozen_config_for(size)), ("llama", llama_config_like_zulozen(size))):
            lm = api.from_random(cfg, seed=7, dtype=dtype)
            vocab = {"vocab_size": ZULOZEN_SIZES[size]["vocab"]}
            rng = np.random.default_rng(7)
            dec = measure_decode_device(lm, vocab, batch, prompt_tokens, steps, warmup, rng)
            bytes_step = (zulozen_step_bytes(cfg, batch, dec["context"], elem) if label == "zulozen"
                          else model_step_bytes(lm, batch, dec["context"]))
            pre = measure_prefill(lm, vocab, prefill_tokens, rng)
            flops = zulozen_prefill_flops(cfg, prefill_tokens) if label == "zulozen" else prefill_flops(cfg, prefill_tokens)
            together = _prefill_together(lm, _prompts(rng, batch, prompt_tokens, vocab["vocab_size"]))
            rec[label] = {
                "decode_tokens_per_s": dec["value"], "decode_ms_per_step": dec["ms_per_step"], "launches_per_step": dec["launches"] / steps,
                "decode_bytes": bytes_step, "decode_frac_of_copy": bytes_step["total"] / (dec["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"],
                "prefill_tokens_per_s": pre["value"], "prefill_ms": pre["ms"], "prefill_flops": flops,
                "prefill_batch_tokens_per_s": together["value"], "prefill_batch_ms": together["ms"],
                "prefill_frac_of_gemm": flops / (pre["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12) if dtype == "bfloat16" else None,
                "clocks": dec["clocks"]}
            del lm
            torch.cuda.empty_cache()
        out["sizes"][size] = rec
    return out


NUDUSUN_SIZES = {
    # width, layers (one differential attention, then three delta layers, in turn), query heads of two maps of `head` / 2
    # channels and values of `head` channels, window, delta heads with keys and values of `head` channels (half as many
    # q/k heads), experts / identity experts / choices / expert size / shared expert size of every layer's feed-forward
    "small": dict(width=1024, layers=8, heads=8, kv_heads=2, head=128, window=512, experts=16, identity=2, top=2, groups=(6, 3),
                  expert_ff=1024, shared_ff=2048, side=64, vocab=32768),
    "medium": dict(width=2048, layers=16, heads=16, kv_heads=4, head=128, window=1024, experts=32, identity=4, top=4, groups=(6, 3),
                   expert_ff=1536, shared_ff=2048, side=64, vocab=32768),
    "wide": dict(width=4096, layers=8, heads=32, kv_heads=8, head=128, window=1024, experts=32, identity=4, top=4, groups=(6, 3),
                 expert_ff=2560, shared_ff=4096, side=128, vocab=32768),
}


def nudusun_config_for(size: str) -> dict:
    s = NUDUSUN_SIZES[size]
    head = s["head"]
    mlp = {"kind": "moe", "expert": {"ff": s["expert_ff"], "limit": 7.0},
           "router": {"experts": s["experts"], "identity": s["identity"], "top": s["top"], "scale": 2.5,
                      "groups": {"count": s["groups"][0], "keep": s["groups"][1]}},
           "shared": {"ff": s["shared_ff"], "limit": 7.0}}
    layers = []
    for i in range(s["layers"]):
        if i % 4 == 0:
            layers.append({"type": "attention", "mlp": copy.deepcopy(mlp),
                           "mixer": {"dim": head // 2, "vdim": head, "heads": s["heads"], "kv_heads": s["kv_heads"],
                                     "mask": {"size": s["window"]}, "scale": (head // 2) ** -0.5, "softcap": 50.0, "diff": 0.3}})
        else:
            layers.append({"type": "delta", "mlp": copy.deepcopy(mlp),
                           "mixer": {"dim": head, "vdim": head, "heads": s["heads"], "kv_heads": s["heads"] // 2, "conv": 4}})
    return {"architecture": "Nudusun", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6}, "postln_alpha": 2.0,
            "embedding": {"scale": s["width"] ** 0.5}, "max_positions": 4096, "token_side": {"dim": s["side"]}, "layers": layers}


def zulozen_config_like_nudusun(size: str) -> dict:
    """The closest decoder the library had: windowed softmax attention with as many heads of `head` channels and a routed
    feed-forward of the same experts, choices and sizes in every layer, equal width, depth and vocabulary."""
    s = NUDUSUN_SIZES[size]
    mixer = {"dim": s["head"], "vdim": s["head"], "heads": s["heads"], "kv_heads": s["kv_heads"], "mask": {"size": s["window"]},
             "rot": {"dims": s["head"] // 2, "base": 10000.0}, "scale": s["head"] ** -0.5}
    mlp = {"kind": "moe", "expert": {"ff": s["expert_ff"]}, "router": {"experts": s["experts"], "top": s["top"]},
           "shared": {"ff": s["shared_ff"]}}
    return {"architecture": "Zulozen", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6}, "residual_mult": 0.5,
            "layers": [{"type": "attention", "mixer": dict(mixer), "mlp": copy.deepcopy(mlp)} for _ in range(s["layers"])]}


def _nudusun_matrices(cfg: dict, experts_reached) -> float:
    """Elements of the matrices a step passes, with ``experts_reached(router)`` real experts per routed feed-forward."""
    W, side = cfg["width"], (cfg.get("token_side") or {}).get("dim", 0)
    total = 0.0
    for L in cfg["layers"]:
        m, f = L["mixer"], L["mlp"]
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        if L["type"] == "attention":
            total += W * (2 * D * (H + G) + G * Dv) + H * Dv * W
        else:
            total += W * (2 * G * D + 2 * H * Dv + 2 * H) + H * Dv * W
        if f:
            r = f["router"]
            total += W * (r["experts"] + r.get("identity", 0)) + 3 * W * (experts_reached(r) * f["expert"]["ff"] + (f.get("shared") or {"ff": 0})["ff"])
        total += 2 * W * side
    return total + cfg["vocab"] * W


def nudusun_step_bytes(cfg: dict, batch: int, context: float, elem: int) -> dict:
    """Bytes a decode step must move: every matrix a row passes once (of the real experts as many as ``batch`` rows with
    ``top`` choices among real and identity experts reach on average when the choices are uniform; the output head, of
    the two embedding tables only the rows read), the keys and values inside each window, every delta state read and
    written in float32."""
    def reached(r):
        total = r["experts"] + r.get("identity", 0)
        return r["experts"] * (1.0 - (1.0 - r["top"] / total) ** batch)
    weights = _nudusun_matrices(cfg, reached) * elem
    kv = state = 0.0
    for L in cfg["layers"]:
        m = L["mixer"]
        if L["type"] == "attention":
            seen = min(context, m["mask"]["size"]) if m.get("mask") else context
            kv += batch * seen * m["kv_heads"] * (2 * m["dim"] + m["vdim"]) * elem
        else:
            channels = 2 * m["kv_heads"] * m["dim"] + m["heads"] * m["vdim"]
            state += 2 * batch * (m["heads"] * m["dim"] * m["vdim"] + (m["conv"] - 1) * channels) * 4
    return {"weights": int(weights), "kv": int(kv), "state": int(state), "total": int(weights + kv + state)}


def nudusun_prefill_flops(cfg: dict, tokens: int) -> float:
    """2 x tokens x (elements of every matrix a token passes: of the routed experts ``top`` x real / (real + identity)
    on average and the shared one), the two score maps and their two weighted sums of values over each query's window,
    and per token and delta head six operations per element of its state (the prediction, the write, the read-out)."""
    total = 2.0 * tokens * (_nudusun_matrices(cfg, lambda r: r["top"] * r["experts"] / (r["experts"] + r.get("identity", 0))) - cfg["vocab"] * cfg["width"])
    for L in cfg["layers"]:
        m = L["mixer"]
        if L["type"] == "attention":
            window = m["mask"]["size"] if m.get("mask") else tokens
            seen = sum(min(i + 1, window) for i in range(tokens))
            total += 2.0 * seen * m["heads"] * (2 * m["dim"] + 2 * m["vdim"])
        else:
            total += 6.0 * tokens * m["heads"] * m["dim"] * m["vdim"]
    return total + 2.0 * cfg["width"] * cfg["vocab"]


def run_nudusun(sizes=("small", "medium"), batch: int = 8, prompt_tokens: int = 512, steps: int = 64, warmup: int = 4,
                prefill_tokens: int = 2048, dtype: str = "bfloat16") -> dict:
    """Decode steps (timed on the device in the loop ``generate`` runs) and prefill steps of the Nudusun decoder and of
    the Zulozen decoder of equal width, depth, heads, experts and vocabulary, random weights."""
    from . import api
    pk = peaks()
    elem = 2 if dtype == "bfloat16" else 4
    out = {"metric": "decode and prefill tokens/s, Nudusun beside the Zulozen decoder of equal size", "dtype": dtype,
           "batch": batch, "prompt_tokens": prompt_tokens, "steps": steps, "warmup": warmup,
           "prefill_tokens": prefill_tokens, "peaks": pk["source"], "data": "synthetic (seeded uniform token ids, random weights)",
           "sizes": {}}
    for size in sizes:
        rec = {"shape": NUDUSUN_SIZES[size]}
        for label, cfg in (("nudusun", nudusun_config_for(size)), ("zulozen", zulozen_config_like_nudusun(size))):
            lm = api.from_random(cfg, seed=7, dtype=dtype)
            vocab = {"vocab_size": NUDUSUN_SIZES[size]["vocab"]}
            rng = np.random.default_rng(7)
            dec = measure_decode_device(lm, vocab, batch, prompt_tokens, steps, warmup, rng)
            bytes_step = (nudusun_step_bytes if label == "nudusun" else zulozen_step_bytes)(cfg, batch, dec["context"], elem)
            pre = measure_prefill(lm, vocab, prefill_tokens, rng)
            flops = (nudusun_prefill_flops if label == "nudusun" else zulozen_prefill_flops)(cfg, prefill_tokens)
            together = _prefill_together(lm, _prompts(rng, batch, prompt_tokens, vocab["vocab_size"]))
            rec[label] = {
                "decode_tokens_per_s": dec["value"], "decode_ms_per_step": dec["ms_per_step"], "launches_per_step": dec["launches"] / steps,
                "decode_bytes": bytes_step, "decode_frac_of_copy": bytes_step["total"] / (dec["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"],
                "prefill_tokens_per_s": pre["value"], "prefill_ms": pre["ms"], "prefill_flops": flops,
                "prefill_batch_tokens_per_s": together["value"], "prefill_batch_ms": together["ms"],
                "prefill_frac_of_gemm": flops / (pre["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12) if dtype == "bfloat16" else None,
                "clocks": dec["clocks"]}
            del lm
            torch.cuda.empty_cache()
        out["sizes"][size] = rec
    return out


KIZEZEN_SIZES = {
    # width, layers (retention, windowed attention, latent attention, windowed attention, in turn), feed-forward size,
    # query heads of `head` channels (a quarter as many kv heads in the windowed attention), window and kept first keys,
    # the latent's channels and the turned part's
    "small": dict(width=1024, layers=8, ff=4096, heads=8, kv_heads=2, head=128, window=512, keep_first=64, rank=512, rot=64,
                  vocab=32768),
    "medium": dict(width=2048, layers=16, ff=8192, heads=16, kv_heads=4, head=128, window=1024, keep_first=64, rank=512, rot=64,
                   vocab=32768),
    "wide": dict(width=4096, layers=8, ff=14336, heads=32, kv_heads=8, head=128, window=1024, keep_first=64, rank=512, rot=64,
                 vocab=32768),
}


def kizezen_config_for(size: str) -> dict:
    s = KIZEZEN_SIZES[size]
    H, D = s["heads"], s["head"]
    attention = {"dim": D, "vdim": D, "heads": H, "kv_heads": s["kv_heads"], "scale": D ** -0.5,
                 "mask": {"size": s["window"], "keep_first": s["keep_first"]},
                 "rot": {"dims": D, "base": 500000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    latent = {"dim": D, "rot_dim": s["rot"], "vdim": D, "heads": H, "kv_rank": s["rank"], "scale": (D + s["rot"]) ** -0.5,
              "rot": {"dims": s["rot"], "base": 10000.0, "scaling": {"factor": 40.0, "fast": 32.0, "slow": 1.0, "original": 4096}}}
    retention = {"dim": D, "vdim": D, "heads": H, "decay": [1.0 - 2.0 ** (-5.0 - 3.0 * i / max(H - 1, 1)) for i in range(H)],
                 "rot": {"dims": D, "base": 10000.0}}
    kinds = (("retention", retention), ("attention", attention), ("latent_attention", latent), ("attention", attention))
    layers = [{"type": kinds[i % 4][0], "mixer": dict(kinds[i % 4][1]), "mlp": {"kind": "dense", "ff": s["ff"]}}
              for i in range(s["layers"])]
    return {"architecture": "Kizezen", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "logit_scale": 1.0, "layers": layers}


def zulozen_config_like_kizezen(size: str) -> dict:
    """The Zulozen decoder of the same width, depth, heads, feed-forward size and vocabulary, every feed-forward dense and
    blocks of positions as long as the window: the library's closest model (attention with a limited view, q/k norm over
    the whole projection, sink and gate per head, a dense feed-forward)."""
    s = KIZEZEN_SIZES[size]
    mixer = {"dim": s["head"], "vdim": s["head"], "heads": s["heads"], "kv_heads": s["kv_heads"], "mask": {"size": s["window"]},
             "rot": {"dims": s["head"] // 2, "base": 10000.0}, "scale": s["head"] ** -0.5}
    return {"architecture": "Zulozen", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6}, "residual_mult": 0.5,
            "layers": [{"type": "attention", "mixer": dict(mixer), "mlp": {"kind": "dense", "ff": s["ff"]}} for _ in range(s["layers"])]}


def _kizezen_matrices(L: dict, W: int) -> float:
    """Elements of the matrices a row passes in one layer."""
    m, f = L["mixer"], L["mlp"]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    if L["type"] == "attention":
        n = W * (H * D + m["kv_heads"] * (D + Dv) + H) + H * Dv * W
    elif L["type"] == "latent_attention":
        n = W * (H * (D + m["rot_dim"]) + m["kv_rank"] + m["rot_dim"] + H) + H * (D + Dv) * m["kv_rank"] + H * Dv * W
    else:
        n = W * (2 * H * D + 2 * H * Dv) + H * Dv * W
    return n + (2 * W * f["ff"] if f else 0)


def kizezen_step_bytes(cfg: dict, batch: int, context: float, elem: int) -> dict:
    """Bytes a decode step must move: every matrix once (the output head, no embedding table), the keys and values a
    query sees (the window and the kept first keys; of a latent attention one row of latent and turned part per position,
    once), every retention state read and written in float32."""
    W = cfg["width"]
    weights = kv = state = 0.0
    for L in cfg["layers"]:
        m = L["mixer"]
        weights += _kizezen_matrices(L, W)
        if L["type"] == "attention":
            seen = min(context, m["mask"]["size"] + m["mask"].get("keep_first", 0)) if m.get("mask") else context
            kv += batch * seen * m["kv_heads"] * (m["dim"] + m["vdim"])
        elif L["type"] == "latent_attention":
            kv += batch * context * (m["kv_rank"] + m["rot_dim"])
        else:
            state += 2.0 * batch * m["heads"] * m["dim"] * m["vdim"] * 4
    weights += cfg["vocab"] * W
    return {"weights": int(weights * elem), "kv": int(kv * elem), "state": int(state), "total": int((weights + kv) * elem + state)}


def kizezen_prefill_flops(cfg: dict, tokens: int) -> float:
    """2 x tokens x (elements of every matrix a token passes, the latent's maps to keys and values among them) plus
    the attention over the visible keys (per head and pair of positions the key's and the value's channels) and 4 flops
    per element of a retention state and token."""
    W = cfg["width"]
    total = 0.0
    for L in cfg["layers"]:
        m = L["mixer"]
        total += 2.0 * tokens * _kizezen_matrices(L, W)
        if L["type"] == "attention":
            win, kept = (m["mask"]["size"], m["mask"].get("keep_first", 0)) if m.get("mask") else (tokens, 0)
            seen = sum(min(i + 1, win + min(kept, max(i + 1 - win, 0))) for i in range(tokens))
            total += 2.0 * seen * m["heads"] * (m["dim"] + m["vdim"])
        elif L["type"] == "latent_attention":
            total += 2.0 * (tokens * (tokens + 1) / 2.0) * m["heads"] * (m["dim"] + m["rot_dim"] + m["vdim"])
        else:
            total += 4.0 * tokens * m["heads"] * m["dim"] * m["vdim"]
    return total + 2.0 * W * cfg["vocab"]


def run_kizezen(sizes=("small", "medium"), batch: int = 8, prompt_tokens: int = 512, steps: int = 64, warmup: int = 4,
                prefill_tokens: int = 2048, dtype: str = "bfloat16") -> dict:
    """Decode steps (timed on the device in the loop ``generate`` runs) and prefill steps of the Kizezen decoder and of
    the Zulozen decoder of equal width, depth, heads, window, feed-forward size and vocabulary, random weights."""
    from . import api
    pk = peaks()
    elem = 2 if dtype == "bfloat16" else 4
    out = {"metric": "decode and prefill tokens/s, Kizezen beside the Zulozen decoder of equal size", "dtype": dtype,
           "batch": batch, "prompt_tokens": prompt_tokens, "steps": steps, "warmup": warmup,
           "prefill_tokens": prefill_tokens, "peaks": pk["source"], "data": "synthetic (seeded uniform token ids, random weights)",
           "sizes": {}}
    for size in sizes:
        rec = {"shape": KIZEZEN_SIZES[size]}
        for label, cfg in (("kizezen", kizezen_config_for(size)), ("zulozen", zulozen_config_like_kizezen(size))):
            lm = api.from_random(cfg, seed=7, dtype=dtype)
            vocab = {"vocab_size": KIZEZEN_SIZES[size]["vocab"]}
            rng = np.random.default_rng(7)
            dec = measure_decode_device(lm, vocab, batch, prompt_tokens, steps, warmup, rng)
            bytes_step = (kizezen_step_bytes if label == "kizezen" else zulozen_step_bytes)(cfg, batch, dec["context"], elem)
            pre = measure_prefill(lm, vocab, prefill_tokens, rng)
            flops = (kizezen_prefill_flops if label == "kizezen" else zulozen_prefill_flops)(cfg, prefill_tokens)
            together = _prefill_together(lm, _prompts(rng, batch, prompt_tokens, vocab["vocab_size"]))
            rec[label] = {
                "decode_tokens_per_s": dec["value"], "decode_ms_per_step": dec["ms_per_step"], "launches_per_step": dec["launches"] / steps,
                "decode_bytes": bytes_step, "decode_frac_of_copy": bytes_step["total"] / (dec["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"],
                "prefill_tokens_per_s": pre["value"], "prefill_ms": pre["ms"], "prefill_flops": flops,
                "prefill_batch_tokens_per_s": together["value"], "prefill_batch_ms": together["ms"],
                "prefill_frac_of_gemm": flops / (pre["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12) if dtype == "bfloat16" else None,
                "clocks": dec["clocks"]}
            del lm
            torch.cuda.empty_cache()
        out["sizes"][size] = rec
    return out


def ablate_decode(batch: int = 8, prompt_tokens: int = 2048, dtype: str = "bfloat16", layers: int | None = None,
                  config_index: int = 2, reps: int = 50) -> dict:
    """Where a decode step's time goes: the captured step graph is timed whole, and again with
    one kind of kernel switched off at a time (the results are then wrong, only the time is
    read). The difference is what that kernel costs in place, inside the chain of dependent
    launches, which no profiler that serialises kernels can show."""
    from . import api
    from .csrc import ops
    from .engine.graphs import DecodeGraph, bucket_width
    shape = SHAPES[config_index]
    cfg = config_for(config_index, layers)
    lm = api.from_random(cfg, seed=shape["seed"], dtype=dtype)
    rng = np.random.default_rng(0)
    cache = lm.new_cache(batch * (((prompt_tokens + 256 + 63) // 64) * 64), max_slots=batch)
    slots, firsts = _prefill_batch(lm, cache, _prompts(rng, batch, prompt_tokens, cfg["vocab_size"]))
    book = cache.book
    book.check_extend([(s, 128) for s in slots])
    starts = np.array([book.extend(s, 128) for s in slots], dtype=np.int32)

    def time_graph():
        widths = [bucket_width(max(len(book.pages[g][s]) for s in slots)) for g in range(len(book.kv_specs))]
        g = DecodeGraph(lm.model, cache, batch, widths, feed=True)
        i = g.fill(slots, starts, firsts)
        g.send(i, True)
        g.capture()
        for _ in range(5):
            g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        return {"us_per_step": a.elapsed_time(b) / reps * 1e3, "launches": g.launches}

    def noop(*_a, **_k):
        return None

    real_gemm = ops.gemm_tc

    def gemm_without(pred):
        def f(a, b, c, epi, bn, splits, err):
            return None if pred(a, epi) else real_gemm(a, b, c, epi, bn, splits, err)
        return f

    hidden, inter = cfg["hidden_size"], cfg["intermediate_size"]
    qkv = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]
    out = {"full": time_graph()}
    for name in ("attn_decode_fused", "attn_paged_mma", "attn_paged_simt", "rope_kv_from_partials", "rope_kv_write", "rmsnorm",
                 "argmax_rows", "gemm_tn_simt"):
        real = getattr(ops, name)
        setattr(ops, name, noop)
        out["without " + name] = time_graph()
        setattr(ops, name, real)
    for label, pred in (("qkv product", lambda a, e: a.shape[0] == qkv and e == ops.TC_T_PARTIAL),
                        ("output product", lambda a, e: tuple(a.shape) == (hidden, cfg["num_attention_heads"] * cfg["head_dim"])),
                        ("gate-up product", lambda a, e: e == ops.TC_T_SWIGLU),
                        ("down product", lambda a, e: tuple(a.shape) == (hidden, inter)),
                        ("output head", lambda a, e: a.shape[0] == cfg["vocab_size"]),
                        ("any product", lambda a, e: True)):
        ops.gemm_tc = gemm_without(pred)
        out["without " + label] = time_graph()
    ops.gemm_tc = real_gemm
    full = out["full"]["us_per_step"]
    for k, v in out.items():
        v["cost_us"] = round(full - v["us_per_step"], 1)
        v["us_per_step"] = round(v["us_per_step"], 1)
    return {"batch": batch, "prompt_tokens": prompt_tokens, "dtype": dtype, "model": shape["name"],
            "layers": cfg["num_hidden_layers"], "steps": out}


def ablate_prefill(tokens: int = 2048, dtype: str = "bfloat16", layers: int | None = None, config_index: int = 2) -> dict:
    """Where a prefill step's time goes: the step of one prompt is timed whole (as
    ``measure_prefill`` does) and again with one kind of kernel switched off at a time; the
    results are then wrong, only the time is read. The difference is that kernel's cost in
    place, with programmatic dependent launch overlapping its neighbours."""
    from . import api
    from .csrc import ops
    from .options import KernelOptions
    shape = SHAPES[config_index]
    cfg = config_for(config_index, layers)
    # every step launched eagerly: a captured step would replay the kernels it was captured with
    lm = api.from_random(cfg, seed=shape["seed"], dtype=dtype, options=KernelOptions(capture_repeated_steps=False))
    rng = np.random.default_rng(0)

    def timed():
        return {"us_per_step": measure_prefill(lm, cfg, tokens, rng)["ms"] * 1e3}

    def noop(*_a, **_k):
        return None

    out = {"full": timed()}
    for name in ("attn_prefill_tc", "attn_paged_mma", "attn_paged_simt", "gemm_tn_simt", "rope_kv_write", "rmsnorm",
                 "embed_gather"):
        real = getattr(ops, name)
        setattr(ops, name, noop)
        out["without " + name] = timed()
        setattr(ops, name, real)
    real_pair, real_add_norm, real_gemm = ops.gemm_tc_pair, ops.gemm_tc_pair_add_norm, ops.gemm_tc
    hidden, inter = cfg["hidden_size"], cfg["intermediate_size"]
    qkv = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]

    def pair_without(pred):
        def f(a, b, c, epi, err, row_scale=None):
            return None if pred(b, epi) else real_pair(a, b, c, epi, err, row_scale)
        return f

    def add_norm_without(pred):
        def f(a, b, h, err, norm_w, eps, x_out, sumsq):
            if pred(b):
                return ops.RowScale(sumsq, b.shape[0], eps)
            return real_add_norm(a, b, h, err, norm_w, eps, x_out, sumsq)
        return f

    ops.gemm_tc_pair = pair_without(lambda b, e: b.shape[0] == qkv and e == ops.TC_STORE)
    out["without qkv product"] = timed()
    ops.gemm_tc_pair = pair_without(lambda b, e: e == ops.TC_SWIGLU)
    out["without gate-up product"] = timed()
    ops.gemm_tc_pair = real_pair
    o_shape = (hidden, cfg["num_attention_heads"] * cfg["head_dim"])
    ops.gemm_tc_pair_add_norm = add_norm_without(lambda b: tuple(b.shape) == o_shape)
    out["without output product (+ norm)"] = timed()
    ops.gemm_tc_pair_add_norm = add_norm_without(lambda b: tuple(b.shape) == (hidden, inter))
    out["without down product (+ norm)"] = timed()
    ops.gemm_tc_pair_add_norm = real_add_norm
    ops.gemm_tc = lambda *a, **k: None
    out["without output head"] = timed()
    ops.gemm_tc_pair, ops.gemm_tc_pair_add_norm = pair_without(lambda b, e: True), add_norm_without(lambda b: True)
    out["without any product"] = timed()
    ops.gemm_tc_pair, ops.gemm_tc_pair_add_norm, ops.gemm_tc = real_pair, real_add_norm, real_gemm
    full = out["full"]["us_per_step"]
    for v in out.values():
        v["cost_us"] = round(full - v["us_per_step"], 1)
        v["us_per_step"] = round(v["us_per_step"], 1)
    return {"tokens": tokens, "dtype": dtype, "model": shape["name"], "layers": cfg["num_hidden_layers"], "steps": out}
