#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode tokens per second and prefill tokens per
second on the Qwen2.5-1.5B shape with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of the whole batch.  The default run decodes a batch of 8
requests, each with 2,048 tokens of history, and reports on ONE JSON line:

  value      decoded tokens per second, timed on the device (CUDA events around K steps of
             the engine's step function and its device sampler; token ids come from pinned
             host buffers, nothing is read back)
  e2e        the same through the public entry point ``Engine.step()``: scheduling, the
             host-to-device copy of the step's inputs and the device-to-host read of the
             sampled tokens included
  prefill    one prompt of 2,048 tokens: tokens per second, milliseconds, and the fraction
             of the bfloat16 tensor-core peak that its flops amount to
  roofline   bytes the decode step has to read (every weight once, the cache of the live
             requests) over its time, against the measured HBM copy bandwidth
  points     decode tokens per second at batch 1 and batch 64; prefill tokens per second for prompts
             of 128 and 512 tokens; milliseconds of a step of 8 decode tokens beside a 64-token portion
  mixed_7b   the Qwen2.5-7B shape under a mixed continuous batch through ``Engine.step()``
  shape_32b  the Qwen2.5-32B shape: decode at batch 1, 8 and the largest batch that fits, one prefill,
             and what the memory plan says about a batch of 64

Peaks come from MEASURED_PEAKS.json beside this file when it exists, else from the
figures measured earlier on the same pool (6.65 TB/s, 1.59 PFLOP/s).  Data are synthetic:
seeded random weights of the architecture's shapes and uniform random token ids.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN25_1P5B = {
    "architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 28, "hidden_size": 1536,
    "num_attention_heads": 12, "num_key_value_heads": 2, "intermediate_size": 8960, "vocab_size": 151936,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 32768, "use_sliding_window": False, "sliding_window": 32768,
    "max_window_layers": 21,
}
QWEN25_0P5B = {   # head size 64
    "architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 24, "hidden_size": 896,
    "num_attention_heads": 14, "num_key_value_heads": 2, "intermediate_size": 4864, "vocab_size": 151936,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 32768, "use_sliding_window": False,
}
QWEN25_7B = {
    "architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 28, "hidden_size": 3584,
    "num_attention_heads": 28, "num_key_value_heads": 4, "intermediate_size": 18944, "vocab_size": 152064,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 32768, "use_sliding_window": False,
}
QWEN25_32B = {
    "architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 64, "hidden_size": 5120,
    "num_attention_heads": 40, "num_key_value_heads": 8, "intermediate_size": 27648, "vocab_size": 152064,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "max_position_embeddings": 32768, "use_sliding_window": False,
}
SHAPES = {"0.5b": ("Qwen2.5-0.5B shape", QWEN25_0P5B), "1.5b": ("Qwen2.5-1.5B shape", QWEN25_1P5B),
          "7b": ("Qwen2.5-7B shape", QWEN25_7B), "32b": ("Qwen2.5-32B shape", QWEN25_32B)}
FULL_LAYERS = 28
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as handle:
                data = json.load(handle)
            peaks = dict(FALLBACK_PEAKS)
            for key in peaks:
                if isinstance(data.get(key), (int, float)) and data[key] > 0:
                    peaks[key] = float(data[key])
            return peaks, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed work runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self.process = None
        self.thread = None

    def start(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.process = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.process.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        clocks, maxima, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for parts in self.samples:
            try:
                clocks.append(float(parts[0]))
                maxima.append(float(parts[1]))
            except ValueError:
                continue
            for name, value in zip(names, parts[2:6]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None,
                "sm_max_mhz": max(maxima) if maxima else None, "reasons": sorted(reasons),
                "samples": len(clocks)}


def decode_bytes(config, layers, batch, history, element=2):
    """Bytes one decode step has to read: every weight it uses once (the embedding matrix only
    where it is also the output matrix), and the cache of the live requests at the mean history
    of the timed steps."""
    h, d = config["hidden_size"], config["hidden_size"] // config["num_attention_heads"]
    q, kv = config["num_attention_heads"] * d, config["num_key_value_heads"] * d
    per_layer = h * (q + 2 * kv) + q * h + 3 * h * config["intermediate_size"]
    weights = (layers * per_layer + config["vocab_size"] * h) * element
    cache = batch * history * 2 * layers * kv * element
    return weights + cache


def prefill_flops(config, layers, tokens):
    h, d = config["hidden_size"], config["hidden_size"] // config["num_attention_heads"]
    q, kv = config["num_attention_heads"] * d, config["num_key_value_heads"] * d
    per_layer = h * (q + 2 * kv) + q * h + 3 * h * config["intermediate_size"]
    gemm = 2.0 * tokens * layers * per_layer + 2.0 * config["vocab_size"] * h
    attention = 2.0 * tokens * tokens * d * config["num_attention_heads"] * layers  # causal half of 4*T^2*d*heads
    return gemm + attention


class DecodeHarness:
    """`batch` requests with `history` tokens already in the cache (random keys and values,
    placed without running a prefill), decoded one token per step through the engine's
    runner and device sampler."""

    def __init__(self, model, batch, history, steps, page_size=16):
        import numpy as np
        import torch

        from vipera_rs_b200.cache import CachePools
        from vipera_rs_b200.engine import ModelRunner
        from vipera_rs_b200.sampling import DeviceSampler

        self.np, self.torch = np, torch
        self.model, self.batch, self.history = model, batch, history
        per_request = -(-(history + steps + 2) // page_size)
        self.pools = CachePools(model.cache_requests, page_size=page_size, num_pages=batch * per_request + 1,
                                num_state_slots=batch, dtype=model.dtype, device=model.device)
        for pool in self.pools.pool_tensors:
            pool.normal_(0.0, 0.5)
        self.runner = ModelRunner(model, self.pools, max_model_len=model.spec.max_position_embeddings)
        self.sampler_tokens = torch.empty(batch, dtype=torch.int32, device=model.device)
        self.manager = self.pools.manager
        self.requests = list(range(batch))
        for r in self.requests:
            self.manager.open(r)
            self.manager.reserve(r, history)
            self.manager.commit(r, history)
        self.position = history
        rng = np.random.default_rng(batch)
        self.token_stream = rng.integers(0, model.spec.vocab_size, size=(4096, batch), dtype=np.int32)
        self.cursor = 0

    def step(self):
        from vipera_rs_b200.engine import StepInput
        from vipera_rs_b200.kernels import ops

        np = self.np
        for r in self.requests:
            self.manager.reserve(r, self.position + 1)
        tokens = self.token_stream[self.cursor % 4096]
        self.cursor += 1
        step = StepInput(requests=self.requests, tokens=tokens, counts=[1] * self.batch,
                         pos0=[self.position] * self.batch, fresh=[0] * self.batch,
                         logit_rows=np.arange(self.batch, dtype=np.int32))
        logits = self.runner.run(step)
        ops.argmax(logits, self.sampler_tokens)
        for r in self.requests:
            self.manager.commit(r, self.position + 1)
        self.position += 1

    def timed(self, steps, warmup):
        torch = self.torch
        for _ in range(warmup):
            self.step()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        first_position = self.position
        start.record()
        for _ in range(steps):
            self.step()
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / steps
        mean_history = (first_position + self.position - 1) / 2.0 + 1
        return ms, mean_history

    def close(self):
        for r in self.requests:
            self.manager.close(r)


def measure_mixed_step(model, decodes, history, portion, repeats, warmup, page_size=16):
    """One step that carries `decodes` single tokens (each with `history` tokens behind it) and
    one prompt portion of `portion` tokens, as continuous batching makes them: milliseconds,
    median of `repeats`, device time of the step function and the device's greedy draw."""
    import numpy as np
    import torch

    from vipera_rs_b200.cache import CachePools
    from vipera_rs_b200.engine import ModelRunner, StepInput
    from vipera_rs_b200.kernels import ops

    per_request = -(-(history + warmup + repeats + 2) // page_size)
    pools = CachePools(model.cache_requests, page_size=page_size,
                       num_pages=decodes * per_request + -(-portion // page_size) + 1, num_state_slots=decodes + 1,
                       dtype=model.dtype, device=model.device)
    for pool in pools.pool_tensors:
        pool.normal_(0.0, 0.5)
    runner = ModelRunner(model, pools, max_model_len=model.spec.max_position_embeddings)
    manager = pools.manager
    for r in range(decodes):
        manager.open(r)
        manager.reserve(r, history)
        manager.commit(r, history)
    rng = np.random.default_rng(3)
    drawn = torch.empty(decodes + 1, dtype=torch.int32, device=model.device)
    times = []
    for index in range(warmup + repeats):
        position = history + index
        for r in range(decodes):
            manager.reserve(r, position + 1)
        manager.open(decodes)
        manager.reserve(decodes, portion)
        tokens = rng.integers(0, model.spec.vocab_size, size=decodes + portion, dtype=np.int32)
        step = StepInput(requests=list(range(decodes + 1)), tokens=tokens, counts=[1] * decodes + [portion],
                         pos0=[position] * decodes + [0], fresh=[0] * decodes + [1],
                         logit_rows=np.asarray(list(range(decodes)) + [decodes + portion - 1], dtype=np.int32))
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        logits = runner.run(step)
        ops.argmax(logits, drawn)
        stop.record()
        torch.cuda.synchronize()
        for r in range(decodes):
            manager.commit(r, position + 1)
        manager.close(decodes)
        if index >= warmup:
            times.append(start.elapsed_time(stop))
    times.sort()
    return times[len(times) // 2]


def measure_prefill(model, tokens, repeats, warmup, page_size=16):
    import numpy as np
    import torch

    from vipera_rs_b200.cache import CachePools
    from vipera_rs_b200.engine import ModelRunner, StepInput

    pools = CachePools(model.cache_requests, page_size=page_size, num_pages=-(-tokens // page_size) + 1,
                       num_state_slots=1, dtype=model.dtype, device=model.device)
    runner = ModelRunner(model, pools, max_model_len=model.spec.max_position_embeddings)
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, model.spec.vocab_size, size=tokens, dtype=np.int32)
    times = []
    for index in range(warmup + repeats):
        pools.manager.open(0)
        pools.manager.reserve(0, tokens)
        step = StepInput(requests=[0], tokens=prompt, counts=[tokens], pos0=[0], fresh=[1],
                         logit_rows=np.asarray([tokens - 1], dtype=np.int32))
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.run(step)
        stop.record()
        torch.cuda.synchronize()
        pools.manager.close(0)
        if index >= warmup:
            times.append(start.elapsed_time(stop))
    times.sort()
    return times[len(times) // 2]


def measure_e2e(model, batch, history, steps, warmup, page_size=16):
    """Through the public entry point: requests with `history`-token prompts are added and
    prefilled by the engine itself; then decode steps are timed on the host clock, each one
    scheduling, copying its inputs from pinned host memory, running, sampling and reading
    the sampled tokens back."""
    import numpy as np
    import torch

    from vipera_rs_b200 import Engine, SamplingParams

    per_request = -(-(history + steps + warmup + 8) // page_size)
    engine = Engine(model, page_size=page_size, num_pages=batch * per_request + 1, max_num_seqs=batch,
                    max_tokens_per_step=4096, max_portion=2048)
    rng = np.random.default_rng(1)
    params = SamplingParams(max_new_tokens=steps + warmup + 4, eos_ids=[])
    for _ in range(batch):
        engine.add_request(rng.integers(0, model.spec.vocab_size, size=history).tolist(), params)
    while True:  # prefill until every request decodes
        report = engine.step()
        if report.num_entries == batch and report.num_tokens == batch:
            break
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    started = time.perf_counter()
    produced = 0
    for _ in range(steps):
        produced += len(engine.step().tokens)
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - started
    h2d = 4 * (8 * batch + 1 + batch * 256)  # packed int32 inputs of a decode step (tables 256 wide at most)
    d2h = 4 * (8 + 2 * batch)                 # token ids, row states and the kernels' status word, one copy
    return produced / elapsed, h2d, d2h


def release_memory():
    """Give back what finished harnesses held (runners and their captured graphs refer to one
    another, so the collector has to run before the allocator can let go)."""
    import gc

    import torch

    gc.collect()
    torch.cuda.empty_cache()


def measure_mixed(model, requests, prompt_range, new_tokens, max_portion, token_budget, passes=3, page_size=16):
    """The engine's normal mode: `requests` requests with prompt lengths uniform in
    `prompt_range`, all offered at once, prompts cut into portions of `max_portion` under a
    budget of `token_budget` tokens a step beside the running decodes, `new_tokens` tokens each,
    through ``Engine.step()`` on the host clock.  The first passes capture the graphs of the
    step sizes that occur (a buffer that grows in the first pass makes the graphs captured before
    it stale, so the second pass still captures some); the last pass is the one reported, with
    the number of graphs it still had to capture."""
    import numpy as np
    import torch

    from vipera_rs_b200 import Engine, SamplingParams

    rng = np.random.default_rng(7)
    lengths = rng.integers(prompt_range[0], prompt_range[1] + 1, size=requests)
    prompts = [rng.integers(0, model.spec.vocab_size, size=int(n)).tolist() for n in lengths]
    per_request = -(-(int(lengths.max()) + new_tokens + 1) // page_size)
    engine = Engine(model, page_size=page_size, num_pages=requests * per_request + 1, max_num_seqs=requests,
                    max_tokens_per_step=token_budget, max_portion=max_portion, prefix_cache=False)
    params = SamplingParams(max_new_tokens=new_tokens, eos_ids=[])
    report = {}
    for index in range(passes):
        before = dict(engine.totals, stage_micros=dict(engine.totals["stage_micros"]))
        captures_before = engine.runner.graph_captures
        for prompt in prompts:
            engine.add_request(prompt, params)
        torch.cuda.synchronize()
        started = time.perf_counter()
        generated = 0
        while engine.has_work():
            generated += len(engine.step().tokens)
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - started
        totals = engine.totals
        steps = totals["steps"] - before["steps"]
        host = {stage: totals["stage_micros"][stage] - before["stage_micros"][stage] for stage in totals["stage_micros"]}
        prompt_tokens = int(lengths.sum())
        report = {
            "requests": requests, "prompt_tokens": prompt_tokens, "generated_tokens": generated,
            "prompt_min": int(prompt_range[0]), "prompt_max": int(prompt_range[1]), "new_tokens_each": new_tokens,
            "max_portion": max_portion, "token_budget": token_budget, "seconds": round(elapsed, 4),
            "tokens_per_s": round((prompt_tokens + generated) / elapsed, 1),
            "generated_tokens_per_s": round(generated / elapsed, 1),
            "steps": steps, "steps_with_portions": totals["steps_with_portions"] - before["steps_with_portions"],
            "tokens_per_step": round((totals["tokens"] - before["tokens"]) / max(steps, 1), 1),
            "ms_per_step": round(elapsed * 1e3 / max(steps, 1), 4),
            # the host's own work a step: scheduling, building and launching, bookkeeping (the
            # sample stage is mostly the wait for the device and is left out)
            "host_us_per_step": round((host["allocate"] + host["compute"] + host["complete"]) / max(steps, 1), 1),
            "host_us_allocate": round(host["allocate"] / max(steps, 1), 1),
            "host_us_compute": round(host["compute"] / max(steps, 1), 1),
            "host_us_complete": round(host["complete"] / max(steps, 1), 1),
            "wait_us_sample": round(host["sample"] / max(steps, 1), 1),
            "graph_step_share": round((totals["graph_steps"] - before["graph_steps"]) / max(steps, 1), 4),
            "graphs_captured_in_pass": engine.runner.graph_captures - captures_before,
            "timing": "host clock around Engine.step() until every request has ended",
        }
    del engine
    release_memory()
    return report


def measure_shape(name, config, layers, peaks, history, batches, steps, warmup, page_size=16, prefill_tokens=2048):
    """Decode at `batches` with `history` tokens of history and one prefill, for another shape."""
    import torch

    from vipera_rs_b200.engine import random_model

    full_layers = config["num_hidden_layers"]
    config = dict(config, num_hidden_layers=layers)
    model = random_model(config, seed=0, dtype="bfloat16", device="cuda:0")
    out = {"model": name, "layers": layers, "layers_full": full_layers, "seq_len": history, "dtype": "bf16"}
    for batch in batches:
        harness = DecodeHarness(model, batch, history, steps + warmup + 2, page_size=page_size)
        ms, mean_history = harness.timed(steps, warmup)
        harness.close()
        del harness
        release_memory()
        gbs = decode_bytes(config, layers, batch, mean_history) / (ms * 1e-3) / 1e9
        out[f"decode_b{batch}"] = round(batch * 1000.0 / ms, 1)
        out[f"decode_b{batch}_ms"] = round(ms, 4)
        out[f"decode_b{batch}_hbm_frac"] = round(gbs / peaks["hbm_gbs"], 4)
    ms = measure_prefill(model, prefill_tokens, repeats=3, warmup=2, page_size=page_size)
    out["prefill_tokens"] = prefill_tokens
    out["prefill_ms"] = round(ms, 3)
    out["prefill_tok_s"] = round(prefill_tokens * 1000.0 / ms, 1)
    out["prefill_frac"] = round(prefill_flops(config, layers, prefill_tokens) / (ms * 1e-3)
                                / (peaks["bf16_tflops_sustained"] * 1e12), 4)
    return out, model


def measure_32b(peaks, warmup, page_size):
    """The 32B shape: what the memory plan says about a batch of 64 at 8,192 tokens (it does not
    fit), decode at batch 1, 8 and the largest batch that fits, and one 2,048-token prefill."""
    import torch

    history = 8192
    refused = plan_report(QWEN25_32B, history + 256, 64)
    # the largest batch for the measurement is planned against what this device really has, less a
    # margin for the allocator
    usable = int(torch.cuda.get_device_properties(0).total_memory * 0.9)
    largest = 8
    for batch in range(8, 65, 8):
        if plan_report(QWEN25_32B, history + 256, batch, usable)["feasible"]:
            largest = batch
    out, model = measure_shape(SHAPES["32b"][0], QWEN25_32B, QWEN25_32B["num_hidden_layers"], peaks, history,
                               sorted({1, 8, largest}), steps=16, warmup=max(3, min(warmup, 4)), page_size=page_size)
    del model
    release_memory()
    out["largest_batch_that_fits"] = largest
    out["plan_b64_feasible"] = bool(refused["feasible"])
    out["plan_b64_needs_gb"] = round(refused["predicted_device_bytes"] / 1e9, 1)
    out["plan_device_gb"] = round(refused["device_bytes"] / 1e9, 1)
    return out


# ---------------------------------------------------------------------------------------
# --design nobupel: the Nobupel design beside the Qwen2 decoder at equal sizes
# ---------------------------------------------------------------------------------------
def nobupel_config(width, heads, kv_heads, ff, layers, vocab, cell_heads, cell_dim, cell_vdim, window=1024):
    """`layers` layers in the design's usual proportion: three cells without a feed-forward, then
    an attention layer with one; heads of 128 of which 64 values turn, a window that keeps 4 keys."""
    cell = {"type": "mlstm", "mixer": {"heads": cell_heads, "dim": cell_dim, "vdim": cell_vdim, "gate_cap": 15.0},
            "mlp": None}
    attention = {"type": "attention", "mlp": {"kind": "dense", "ff": ff},
                 "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                           "mask": {"size": window, "keep_first": 4},
                           "rot": {"dims": 64, "base": 1000000.0,
                                   "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}}
    return {"architecture": "Nobupel", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
            "layers": [attention if index % 4 == 3 else cell for index in range(layers)], "loop": None}


def qwen_like(width, heads, kv_heads, ff, layers, vocab):
    return {"architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": layers, "hidden_size": width,
            "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": 128, "intermediate_size": ff,
            "vocab_size": vocab, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
            "max_position_embeddings": 32768}


DESIGN_SIZES = {
    # name: width, heads, kv heads, inner size, layers, vocabulary, then the cell's heads, q/k size, value size
    "1.5b-like": (1536, 12, 2, 8960, 8, 32000, 6, 128, 256),
    "7b-like": (4096, 32, 8, 14336, 8, 32000, 8, 256, 512),
}


def nobupel_work(config, tokens, chunk=32):
    """Floating-point operations of a prompt of `tokens` tokens by class of kernel (products of the
    mixers, feed-forwards and output matrix; the cells' recurrence as the chunked form computes
    it; attention within its window), and the bytes one decode step must move per class."""
    width = config["width"]
    flops = {"proj": 2.0 * config["vocab"] * width, "recurrence": 0.0, "attention": 0.0}
    for layer in config["layers"]:
        m = layer["mixer"]
        if layer["type"] == "mlstm":
            h, d, dv = m["heads"], m["dim"], m["vdim"]
            flops["proj"] += 2.0 * tokens * width * (2 * h * d + 3 * h * dv + 2 * h)
            # per token: scores and weighted values within the chunk (half of it masked), the read of S and its update
            flops["recurrence"] += 2.0 * tokens * h * (chunk * (d + dv) / 2 + 2 * d * dv)
        else:
            h, g, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            flops["proj"] += 2.0 * tokens * width * (h * d + g * (d + dv) + h * dv)
            seen = min(tokens, m["mask"]["size"]) if m.get("mask") else tokens
            flops["attention"] += 2.0 * tokens * h * (d + dv) * (seen / 2 if seen == tokens else seen)
        if layer.get("mlp"):
            flops["proj"] += 2.0 * tokens * 3 * width * layer["mlp"]["ff"]
    return flops


def nobupel_decode_bytes(config, batch, history, element=2):
    width = config["width"]
    weights = config["vocab"] * width
    state = cache = 0
    for layer in config["layers"]:
        m = layer["mixer"]
        if layer["type"] == "mlstm":
            h, d, dv = m["heads"], m["dim"], m["vdim"]
            weights += width * (2 * h * d + 3 * h * dv + 2 * h)
            state += 2 * batch * h * d * dv * 4            # the state is read and written, in 32-bit
        else:
            h, g, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            weights += width * (h * d + g * (d + dv) + h * dv)
            seen = min(history, m["mask"]["size"] + m["mask"]["keep_first"]) if m.get("mask") else history
            cache += batch * seen * g * (d + dv) * element
        if layer.get("mlp"):
            weights += 3 * width * layer["mlp"]["ff"]
    return {"weights": weights * element, "state": state, "cache": cache}


# ---------------------------------------------------------------------------------------
# --design gusolix: the Gusolix design beside the Qwen2 decoder at equal sizes
# ---------------------------------------------------------------------------------------
def gusolix_config(width, heads, kv_heads, ff, layers, vocab, *_unused, chunk=1024):
    """`layers` layers in the order attention, Mamba, and two layers of softmax attention with
    mixed head weights beside gated linear attention; every layer with a feed-forward; heads of 128,
    chunks of 1,024 keys, Mamba with twice the width in channels and 16 states."""
    attention = {"type": "attention", "mlp": {"kind": "dense", "ff": ff},
                 "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                           "mask": {"size": chunk},
                           "rot": {"dims": 64, "base": 500000.0,
                                   "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}}
    mamba = {"type": "mamba1", "mlp": {"kind": "dense", "ff": ff},
             "mixer": {"inner": 2 * width, "state": 16, "dt_rank": width // 16, "conv": 4}}
    pair = {"type": "parallel", "mlp": {"kind": "dense", "ff": ff},
            "mixer": {"left": {"heads": heads // 2, "kv_heads": max(kv_heads // 2, 1), "dim": 128, "vdim": 128,
                               "scale": 128 ** -0.5},
                      "right": {"heads": heads // 4, "dim": 128, "vdim": 256, "tau": 16.0, "rank": 16},
                      "left_scale": 0.8, "right_scale": 0.9}}
    order = (attention, mamba, pair, pair)
    return {"architecture": "Gusolix", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "embedding": {"scale": float(width) ** 0.5}, "canon": {"taps": 4},
            "layers": [order[index % 4] for index in range(layers)]}


def gusolix_work(config, tokens):
    """Floating-point operations of a prompt of `tokens` tokens by class of kernel: products,
    attention within its mask (the mixed-weights form computes its scores twice), the
    recurrences as their token-by-token forms compute them."""
    width = config["width"]
    flops = {"proj": 2.0 * config["vocab"] * width, "recurrence": 0.0, "attention": 0.0}

    def softmax_heads(m, seen, passes):
        flops["proj"] += 2.0 * tokens * width * (m["heads"] * m["dim"] + m["kv_heads"] * m["dim"] + m["heads"] * m["vdim"])
        flops["attention"] += 2.0 * tokens * m["heads"] * (passes * m["dim"] + m["vdim"]) * seen

    for layer in config["layers"]:
        m = layer["mixer"]
        if layer["type"] == "attention":
            size = (m.get("mask") or {}).get("size") or tokens
            softmax_heads(m, min(tokens, size) / 2, 1)
        elif layer["type"] == "mamba1":
            flops["proj"] += 2.0 * tokens * (width * 2 * m["inner"] + m["inner"] * (m["dt_rank"] + 2 * m["state"])
                                             + m["dt_rank"] * m["inner"] + m["inner"] * width)
            flops["recurrence"] += tokens * m["inner"] * m["state"] * 5.0
        else:
            left, right = m["left"], m["right"]
            softmax_heads(left, tokens / 2, 2)
            flops["proj"] += 2.0 * tokens * width * left["kv_heads"] * left["vdim"]
            flops["attention"] += 2.0 * tokens * left["heads"] * left["heads"] * tokens / 2      # the mix of the weights
            h, d, dv = right["heads"], right["dim"], right["vdim"]
            flops["proj"] += 2.0 * tokens * (width * h * (2 * d + 3 * dv) + width * right["rank"] + right["rank"] * h * d)
            flops["recurrence"] += tokens * h * d * dv * 4.0
        if layer.get("mlp"):
            flops["proj"] += 2.0 * tokens * 3 * width * layer["mlp"]["ff"]
    return flops


def gusolix_prefill_bytes(config, tokens):
    """Bytes the recurrences of a prompt must move at least (their inputs once, their outputs once; the
    state stays on the chip): the bound of kernels that do a handful of operations per value."""
    moved = 0
    for layer in config["layers"]:
        m = layer["mixer"]
        if layer["type"] == "mamba1":
            moved += tokens * (m["inner"] * (4 + 4 + 4 + 2) + 2 * m["state"] * 4)       # x, dt, gate in 32-bit, out
        elif layer["type"] == "parallel":
            r = m["right"]
            moved += tokens * r["heads"] * ((3 * r["dim"] + 2 * r["vdim"]) * 4 + r["vdim"] * 2)
    return moved


def gusolix_decode_bytes(config, batch, history, element=2):
    width = config["width"]
    weights = config["vocab"] * width
    state = cache = 0
    taps = config["canon"]["taps"]
    for layer in config["layers"]:
        m = layer["mixer"]
        state += 2 * batch * 2 * (taps - 1) * width * 4
        if layer["type"] == "attention":
            weights += width * (m["heads"] * m["dim"] + m["kv_heads"] * m["dim"] + m["heads"] * m["vdim"])
            size = (m.get("mask") or {}).get("size") or history
            cache += batch * min(history, size / 2) * m["kv_heads"] * (m["dim"] + m["vdim"]) * element
        elif layer["type"] == "mamba1":
            weights += width * 2 * m["inner"] + m["inner"] * (m["dt_rank"] + 2 * m["state"]) + m["dt_rank"] * m["inner"] \
                + m["inner"] * width
            state += 2 * batch * m["inner"] * (m["state"] + m["conv"] - 1) * 4
        else:
            left, right = m["left"], m["right"]
            weights += width * (left["heads"] * left["dim"] + left["kv_heads"] * (left["dim"] + left["vdim"])
                                + left["heads"] * left["vdim"])
            cache += batch * history * left["kv_heads"] * (left["dim"] + left["vdim"]) * element
            h, d, dv = right["heads"], right["dim"], right["vdim"]
            weights += width * h * (2 * d + 3 * dv) + width * right["rank"] + right["rank"] * h * d
            state += 2 * batch * h * d * dv * 4
        if layer.get("mlp"):
            weights += 3 * width * layer["mlp"]["ff"]
    return {"weights": weights * element, "state": state, "cache": int(cache)}


# ---------------------------------------------------------------------------------------
# --design pugovik: the Pugovik design beside the Qwen2 decoder at equal sizes
# ---------------------------------------------------------------------------------------
def pugovik_config(width, heads, kv_heads, ff, layers, vocab, cell_heads, cell_dim, cell_vdim, experts=16, top=4):
    """`layers` layers in the proportion three of linear attention to one of attention over a cached
    latent (every second of those reading the pages of the one before it); every layer with a mixture
    of `experts` gated units of which a token uses `top`, sized so that a token's experts together have
    the dense inner size; heads of 128 + 64 turning values over a latent of 512."""
    mlp = {"kind": "moe", "expert": {"ff": ff // top},
           "router": {"experts": experts, "top": top, "groups": {"count": 4, "keep": 2}}}
    decay = [1.0 - 2.0 ** (-5.0 - 5.0 * index / max(cell_heads - 1, 1)) for index in range(cell_heads)]
    lightning = {"type": "lightning", "mlp": mlp,
                 "mixer": {"heads": cell_heads, "dim": cell_dim, "vdim": cell_vdim, "decay": decay}}

    def latent(source=None):
        mixer = {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "scale": 192 ** -0.5,
                 "rot": {"dims": 64, "base": 10000.0,
                         "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
        if source is not None:
            mixer["kv_from"] = source
        return {"type": "latent_attention", "mlp": mlp, "mixer": mixer}

    order, first = [], None
    for index in range(layers):
        if index % 4 != 3:
            order.append(lightning)
        elif first is None:
            order.append(latent())
            first = index
        else:
            order.append(latent(first))
            first = None
    return {"architecture": "Pugovik", "vocab": vocab, "width": width, "norm": {"eps": 1e-6, "groups": 4},
            "residual_mult": 0.5, "layers": order}


def pugovik_work(config, tokens, chunk=64):
    """Floating-point operations of a prompt of `tokens` tokens by class of kernel: products (mixers,
    gates of the stream, the chosen experts, the output matrix), the linear attention as its chunked
    form computes it, attention over the latents (scores against rank + rot_dim values, weighted sums
    of rank values, and the two absorbed matrices per query)."""
    width = config["width"]
    flops = {"proj": 2.0 * config["vocab"] * width, "recurrence": 0.0, "attention": 0.0, "experts": 0.0}
    for layer in config["layers"]:
        m = layer["mixer"]
        if layer["type"] == "lightning":
            h, d, dv = m["heads"], m["dim"], m["vdim"]
            flops["proj"] += 2.0 * tokens * width * (2 * h * d + 3 * h * dv)
            flops["recurrence"] += 2.0 * tokens * h * (chunk * (d + dv) / 2 + 2 * d * dv)
        else:
            h, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            own = 0 if "kv_from" in m else rank + r
            flops["proj"] += 2.0 * tokens * width * (h * (d + r) + own + 2 * h * dv)
            flops["attention"] += 2.0 * tokens * h * ((2 * rank + r) * tokens / 2 + rank * (d + dv))
        flops["proj"] += 2.0 * tokens * width * width            # the gate of what joins the stream
        if layer.get("mlp"):
            router = layer["mlp"]["router"]
            flops["proj"] += 2.0 * tokens * width * width
            flops["experts"] += 2.0 * tokens * (router["top"] * 3 * width * layer["mlp"]["expert"]["ff"] + router["experts"] * width)
    return flops


def pugovik_decode_bytes(config, batch, history, element=2):
    """What one decode step must move: every matrix a token of the batch can use (all experts once the
    batch's choices cover them: min(experts, batch * top)), states read and written, latents read."""
    width = config["width"]
    weights = config["vocab"] * width
    state = cache = 0
    for layer in config["layers"]:
        m = layer["mixer"]
        if layer["type"] == "lightning":
            h, d, dv = m["heads"], m["dim"], m["vdim"]
            weights += width * (2 * h * d + 3 * h * dv)
            state += 2 * batch * h * d * dv * 4
        else:
            h, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            own = 0 if "kv_from" in m else rank + r
            weights += width * (h * (d + r) + own + 2 * h * dv) + h * rank * (d + dv)
            cache += batch * history * (rank + r) * element
        weights += width * width
        if layer.get("mlp"):
            router = layer["mlp"]["router"]
            used = min(router["experts"], batch * router["top"])
            weights += width * width + used * 3 * width * layer["mlp"]["expert"]["ff"] + router["experts"] * width
    return {"weights": weights * element, "state": state, "cache": int(cache)}


# ---------------------------------------------------------------------------------------
# --design fasolorn: the Fasolorn design beside the Qwen2 decoder at equal sizes
# ---------------------------------------------------------------------------------------
def fasolorn_config(width, heads, kv_heads, ff, layers, vocab, *_unused, experts=16, identity=2, top=4, window=1024):
    """`layers` layers in the proportion three of grouped-query attention (heads of 128, a learned sink,
    an output gate, values blended with the first layer's, a window) to one of attention over a cached
    latent of 512 (heads of 128 + 64 turning values, the same window); feed-forwards by turns a gated
    unit of the dense inner size and a mixture of `experts` units without a gate plus `identity` outputs
    that return their input, of which a token uses `top`, beside a shared unit; a token's experts and
    the shared unit together have two thirds of the dense inner size (units without a gate have two
    matrices where a gated one has three)."""
    attention = {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                 "mask": {"size": window}, "rot": {"dims": 128, "base": 500000.0}, "v_mix": True}
    latent = {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "scale": 192 ** -0.5,
              "mask": {"size": window}, "rot": {"dims": 64, "base": 10000.0}}
    piece = ff // (top + 1) // 16 * 16
    moe = {"kind": "moe", "expert": {"ff": piece}, "shared": {"ff": piece},
           "router": {"experts": experts, "identity": identity, "top": top, "scale": 2.5}}
    dense = {"kind": "dense", "ff": ff}
    order = []
    for index in range(layers):
        mixer = ("latent_attention", latent) if index % 4 == 3 else ("attention", attention)
        order.append({"type": mixer[0], "mixer": mixer[1], "mlp": moe if index % 2 else dense})
    return {"architecture": "Fasolorn", "vocab": vocab, "width": width, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-6}, "layers": order}


def fasolorn_work(config, tokens):
    """Floating-point operations of a prompt of `tokens` tokens by class of kernel: products (the mixers'
    matrices, the dense feed-forwards, the output matrix), the chosen experts with the shared unit and
    the router, and attention within the windows (over keys and values, or over the latents: scores
    against rank + rot_dim values, weighted sums of rank values, the two absorbed matrices per query)."""
    width = config["width"]
    flops = {"proj": 2.0 * config["vocab"] * width, "attention": 0.0, "experts": 0.0}
    for layer in config["layers"]:
        m = layer["mixer"]
        window = m["mask"]["size"] if m.get("mask") else tokens
        seen = sum(min(position + 1, window) for position in range(tokens))     # (query, key) pairs
        if layer["type"] == "attention":
            h, g, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            flops["proj"] += 2.0 * tokens * width * (h * d + g * (d + dv) + 2 * h * dv)
            flops["attention"] += 2.0 * seen * h * (d + dv)
        else:
            h, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            flops["proj"] += 2.0 * tokens * width * (h * (d + r) + rank + r + h * dv)
            flops["attention"] += 2.0 * h * (seen * (2 * rank + r) + tokens * rank * (d + dv))
        mlp = layer.get("mlp")
        if mlp and mlp["kind"] == "dense":
            flops["proj"] += 2.0 * tokens * 3 * width * mlp["ff"]
        elif mlp:
            router = mlp["router"]
            inner = router["top"] * mlp["expert"]["ff"] + (mlp.get("shared") or {"ff": 0})["ff"]
            flops["experts"] += 2.0 * tokens * (2 * width * inner + (router["experts"] + router.get("identity", 0)) * width)
    return flops


def fasolorn_decode_bytes(config, batch, history, element=2):
    """What one decode step must move: every matrix a token of the batch can use (all experts once the
    batch's choices cover them: min(experts, batch * top)), and the keys, values and latents within the
    windows."""
    width = config["width"]
    weights = config["vocab"] * width
    cache = 0
    for layer in config["layers"]:
        m = layer["mixer"]
        keys = min(history, m["mask"]["size"]) if m.get("mask") else history
        if layer["type"] == "attention":
            h, g, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            weights += width * (h * d + g * (d + dv) + 2 * h * dv)
            cache += batch * keys * g * (d + dv) * element
        else:
            h, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            weights += width * (h * (d + r) + rank + r + h * dv) + h * rank * (d + dv)
            cache += batch * keys * (rank + r) * element
        mlp = layer.get("mlp")
        if mlp and mlp["kind"] == "dense":
            weights += 3 * width * mlp["ff"]
        elif mlp:
            router = mlp["router"]
            used = min(router["experts"], batch * router["top"])
            weights += 2 * width * (used * mlp["expert"]["ff"] + (mlp.get("shared") or {"ff": 0})["ff"])
            weights += (router["experts"] + router.get("identity", 0)) * width * 2     # the router's matrix is 32-bit
    return {"weights": weights * element, "state": 0, "cache": int(cache)}


DESIGNS = {
    "nobupel": (lambda *sizes: nobupel_config(*sizes), lambda config, tokens: nobupel_work(config, tokens),
                lambda config, batch, history: nobupel_decode_bytes(config, batch, history)),
    "gusolix": (lambda *sizes: gusolix_config(*sizes), lambda config, tokens: gusolix_work(config, tokens),
                lambda config, batch, history: gusolix_decode_bytes(config, batch, history)),
    "pugovik": (lambda *sizes: pugovik_config(*sizes), lambda config, tokens: pugovik_work(config, tokens),
                lambda config, batch, history: pugovik_decode_bytes(config, batch, history)),
    "fasolorn": (lambda *sizes: fasolorn_config(*sizes), lambda config, tokens: fasolorn_work(config, tokens),
                 lambda config, batch, history: fasolorn_decode_bytes(config, batch, history)),
}


def profiled_prefill(model, tokens, page_size):
    """One prompt launched kernel by kernel with an event behind every launch: milliseconds by class of kernel."""
    from vipera_rs_b200.kernels import ops

    ops.profile = ops.KernelProfile()
    try:
        measure_prefill(model, tokens, repeats=1, warmup=2, page_size=page_size)   # sizes seen, kernels loaded
        ops.profile.totals.clear()
        import numpy as np
        import torch

        from vipera_rs_b200.cache import CachePools
        from vipera_rs_b200.engine import ModelRunner, StepInput

        pools = CachePools(model.cache_requests, page_size=page_size, num_pages=-(-tokens // page_size) + 1,
                           num_state_slots=1, dtype=model.dtype, device=model.device)
        runner = ModelRunner(model, pools, max_model_len=model.spec.max_position_embeddings)
        runner.step_graphs = runner.decode_graphs = False
        prompt = np.random.default_rng(0).integers(0, model.spec.vocab_size, size=tokens, dtype=np.int32)
        for _ in range(3):
            pools.manager.open(0)
            pools.manager.reserve(0, tokens)
            step = StepInput(requests=[0], tokens=prompt, counts=[tokens], pos0=[0], fresh=[1],
                             logit_rows=np.asarray([tokens - 1], dtype=np.int32))
            torch.cuda.synchronize()
            ops.profile.begin()
            runner.run(step)
            totals = ops.profile.end("prefill")
            pools.manager.close(0)
        return {name: round(value / totals["steps"], 4) for name, value in totals.items() if name != "steps"}
    finally:
        ops.profile = None


def measure_design(args, peaks, peak_source):
    """Prefill and decode of the design at sizes that resemble real layers, beside the Qwen2 decoder of
    the same width, heads, inner size and layer count; random weights, bfloat16."""
    import torch  # noqa: F401

    from vipera_rs_b200.engine import random_model

    warmup = max(args.warmup, 3)
    tokens = args.prefill_tokens
    sampler = ClockSampler()
    sampler.start()
    sizes = {}
    for name, (width, heads, kv_heads, ff, layers, vocab, cell_heads, cell_dim, cell_vdim) in DESIGN_SIZES.items():
        if args.design_size and name != args.design_size:
            continue
        row = {}
        make_config, work_of, decode_bytes_of = DESIGNS[args.design]
        for label, config in ((args.design, make_config(width, heads, kv_heads, ff, layers, vocab, cell_heads, cell_dim,
                                                        cell_vdim)),
                              ("qwen2", qwen_like(width, heads, kv_heads, ff, layers, vocab))):
            model = random_model(config, seed=0, dtype="bfloat16", device="cuda:0")
            out = {"layers": layers}
            ms = measure_prefill(model, tokens, repeats=5, warmup=3, page_size=args.page_size)
            out["prefill_ms"], out["prefill_tok_s"] = round(ms, 3), round(tokens * 1000.0 / ms, 1)
            out["prefill_ms_by_class"] = profiled_prefill(model, tokens, args.page_size)
            if label == args.design:
                work = work_of(config, tokens)
                out["prefill_flops_by_class"] = {k: round(v / 1e9, 2) for k, v in work.items()}
                out["prefill_frac_by_class"] = {
                    k: round(v / (out["prefill_ms_by_class"][k] * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)
                    for k, v in work.items() if out["prefill_ms_by_class"].get(k)}
                if args.design == "gusolix" and out["prefill_ms_by_class"].get("recurrence"):
                    moved = gusolix_prefill_bytes(config, tokens)
                    out["prefill_recurrence_hbm_frac"] = round(
                        moved / (out["prefill_ms_by_class"]["recurrence"] * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
            else:
                qc = dict(config, hidden_size=width)
                out["prefill_frac"] = round(prefill_flops_head(qc, layers, tokens) / (ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)
            for batch in (1, 8, 64):
                harness = DecodeHarness(model, batch, args.history, args.steps + warmup + 2, page_size=args.page_size)
                step_ms, mean_history = harness.timed(args.steps, warmup)
                harness.close()
                del harness
                release_memory()
                out[f"decode_b{batch}_tok_s"], out[f"decode_b{batch}_ms"] = round(batch * 1000.0 / step_ms, 1), round(step_ms, 4)
                if label == args.design:
                    moved = decode_bytes_of(config, batch, mean_history)
                    out[f"decode_b{batch}_hbm_frac"] = round(sum(moved.values()) / (step_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
                else:
                    out[f"decode_b{batch}_hbm_frac"] = round(
                        decode_bytes_head(config, layers, batch, mean_history) / (step_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
            row[label] = out
            del model
            release_memory()
        sizes[name] = row
    print(json.dumps({"design": args.design, "beside": "qwen2 at equal width, heads, inner size and layers",
                      "dtype": "bf16", "data": "synthetic: seeded random weights, uniform random token ids",
                      "prefill_tokens": tokens, "history": args.history, "steps": args.steps, "warmup": warmup,
                      "peaks": peak_source, "sizes": sizes, "clocks": sampler.stop()}))
    return 0


def prefill_flops_head(config, layers, tokens):
    """prefill_flops for a configuration that names its head size."""
    h, d = config["hidden_size"], config.get("head_dim") or config["hidden_size"] // config["num_attention_heads"]
    q, kv = config["num_attention_heads"] * d, config["num_key_value_heads"] * d
    per_layer = h * (q + 2 * kv) + q * h + 3 * h * config["intermediate_size"]
    return (2.0 * tokens * layers * per_layer + 2.0 * config["vocab_size"] * h
            + 2.0 * tokens * tokens * d * config["num_attention_heads"] * layers)


def decode_bytes_head(config, layers, batch, history, element=2):
    h, d = config["hidden_size"], config.get("head_dim") or config["hidden_size"] // config["num_attention_heads"]
    q, kv = config["num_attention_heads"] * d, config["num_key_value_heads"] * d
    per_layer = h * (q + 2 * kv) + q * h + 3 * h * config["intermediate_size"]
    return (layers * per_layer + config["vocab_size"] * h) * element + batch * history * 2 * layers * kv * element


def plan_report(config, ctx, batch, device_bytes=180 * 10**9):
    """What `vipera plan` says about the shape at this context and batch (on one 180 GB device
    where nothing else is said)."""
    from vipera_rs_b200.config import architecture_of
    from vipera_rs_b200.engine import planner

    arch = architecture_of(config)
    return planner.plan_memory(arch.model_spec(arch.config_from_dict(config)), ctx, batch, "bfloat16", device_bytes)


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--history", type=int, default=2048)
    parser.add_argument("--layers", type=int, default=FULL_LAYERS)
    parser.add_argument("--skip-points", action="store_true")
    parser.add_argument("--page-size", type=int, default=16, help="keys per cache page (the engine's default is 16)")
    parser.add_argument("--only", choices=["decode", "prefill", "mixed", "32b"], default=None,
                        help="run one part only and print a short line (for profiling a small case)")
    parser.add_argument("--config", choices=sorted(SHAPES), default="1.5b",
                        help="the shape the headline line is measured on (default: the 1.5B shape)")
    parser.add_argument("--prefill-tokens", type=int, default=2048)
    parser.add_argument("--skip-workloads", action="store_true",
                        help="leave out the 7B mixed workload and the 32B shape")
    parser.add_argument("--design", choices=sorted(DESIGNS), default=None,
                        help="instead of the headline: prefill and decode of that design at sizes that resemble "
                             "real layers, beside the Qwen2 decoder at equal sizes")
    parser.add_argument("--design-size", choices=sorted(DESIGN_SIZES), default=None, help="one of the sizes only")
    args = parser.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust workspace that loads GGUF files; no cargo/rustc and no "
                          "GGUF model exist here, and pip cannot install it"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": "this engine runs on one GPU; bench.py measures --gpus 1 only",
                          "n_gpus": args.gpus}))
        return 2
    warmup = max(args.warmup, 3)

    import torch

    import vipera_rs_b200  # noqa: F401
    from vipera_rs_b200.engine import random_model

    peaks, peak_source = read_peaks()
    if args.design:
        return measure_design(args, peaks, peak_source)
    shape_name, shape = SHAPES[args.config]
    full_layers = shape["num_hidden_layers"]
    config = dict(shape)
    if args.layers == FULL_LAYERS and args.config != "1.5b":
        args.layers = full_layers
    config["num_hidden_layers"] = args.layers
    from vipera_rs_b200.kernels import ops

    model = random_model(config, seed=0, dtype="bfloat16", device="cuda:0")
    if args.only == "prefill":
        ms = measure_prefill(model, args.prefill_tokens, repeats=2, warmup=warmup, page_size=args.page_size)
        print(json.dumps({"only": "prefill", "layers": args.layers, "tokens": args.prefill_tokens, "ms": round(ms, 3),
                          "tok_s": round(args.prefill_tokens * 1000.0 / ms, 1)}))
        return 0
    if args.only == "mixed":
        print(json.dumps({"only": "mixed", "model": shape_name, "layers": args.layers,
                          **measure_mixed(model, 64, (128, 4096), 256, 512, 2048, page_size=args.page_size)}))
        return 0
    if args.only == "32b":
        del model
        release_memory()
        print(json.dumps({"only": "32b", **measure_32b(peaks, warmup, args.page_size)}))
        return 0
    if args.only == "decode":
        harness = DecodeHarness(model, args.batch, args.history, args.steps + 2 * warmup + 2, page_size=args.page_size)
        ms, _ = harness.timed(args.steps, warmup)
        print(json.dumps({"only": "decode", "layers": args.layers, "batch": args.batch, "ms_per_step": round(ms, 4)}))
        return 0
    sampler = ClockSampler()
    sampler.start()

    # pages for the pass that captures the graphs (2 steps and its warm-up) and the timed pass
    harness = DecodeHarness(model, args.batch, args.history, args.steps + 2 * warmup + 2, page_size=args.page_size)
    harness.timed(2, warmup)  # graphs captured, buffers sized
    launches_before = ops.launches
    ms_per_step, mean_history = harness.timed(args.steps, warmup)
    timed_launches = ops.launches - launches_before
    harness.close()
    value = args.batch * 1000.0 / ms_per_step
    step_bytes = decode_bytes(config, args.layers, args.batch, mean_history)
    achieved_gbs = step_bytes / (ms_per_step * 1e-3) / 1e9

    points = {}
    if not args.skip_points:
        for batch in (1, 64):
            other = DecodeHarness(model, batch, args.history, 32 + warmup, page_size=args.page_size)
            ms, _ = other.timed(32, warmup)
            other.close()
            points[f"decode_b{batch}"] = round(batch * 1000.0 / ms, 1)
            del other
            release_memory()
        # steps as continuous batching makes them: short prompts whole, and a portion beside decodes
        for tokens in (128, 512):
            ms = measure_prefill(model, tokens, repeats=5, warmup=3, page_size=args.page_size)
            points[f"prefill_{tokens}"] = round(tokens * 1000.0 / ms, 1)
        points["step_8_decodes_and_64_token_portion_ms"] = round(
            measure_mixed_step(model, 8, args.history, 64, repeats=9, warmup=4, page_size=args.page_size), 4)
        release_memory()

    prefill_tokens = args.prefill_tokens
    prefill_ms = measure_prefill(model, prefill_tokens, repeats=5, warmup=3, page_size=args.page_size)
    flops = prefill_flops(config, args.layers, prefill_tokens)
    prefill_frac = flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12)

    e2e_value, h2d, d2h = measure_e2e(model, args.batch, args.history, args.steps, warmup, page_size=args.page_size)
    clocks = sampler.stop()

    # The engine's normal mode on the 7B shape and the 32B shape's decode and prefill: numbers of
    # their own beside the headline, each with the sizes it ran at.
    workloads = {}
    if args.config == "1.5b" and not args.skip_workloads:
        del model, harness
        release_memory()
        try:
            big = random_model(dict(QWEN25_7B), seed=1, dtype="bfloat16", device="cuda:0")
            workloads["mixed_7b"] = {"model": SHAPES["7b"][0], "layers": 28, "layers_full": 28,
                                     **measure_mixed(big, 64, (128, 4096), 256, 512, 2048, page_size=args.page_size)}
            del big
            release_memory()
            workloads["shape_32b"] = measure_32b(peaks, warmup, args.page_size)
        except Exception as error:  # the headline stands even where a larger shape does not fit
            workloads["error"] = f"{type(error).__name__}: {error}"

    line = {
        "metric": f"decode tok/s at batch {args.batch}, {args.history} tokens of history ({shape_name}); "
                  f"prefill tok/s at {prefill_tokens} tokens",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights, uniform random token ids",
        "impl": "ours",
        "config": {
            "model": shape_name, "layers": args.layers, "layers_full": full_layers,
            "hidden": config["hidden_size"], "heads": config["num_attention_heads"],
            "kv_heads": config["num_key_value_heads"],
            "head_dim": config["hidden_size"] // config["num_attention_heads"],
            "intermediate": config["intermediate_size"], "vocab": config["vocab_size"],
            "tied_head": bool(config["tie_word_embeddings"]), "global_batch": args.batch, "seq_len": args.history,
            "new_tokens": args.steps, "page_size": args.page_size, "parallelism": "single GPU",
            "l2": "inputs larger than L2: every step reads all weights (GBs) against 126 MB",
            "peaks": peak_source,
        },
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h,
                "overlap": "Engine.step() launches the step after while a step runs; both copies happen every step"},
        "gpu_launches": timed_launches,
        "prefill": {"value": round(prefill_tokens * 1000.0 / prefill_ms, 1), "tokens": prefill_tokens,
                    "ms": round(prefill_ms, 3), "frac": round(prefill_frac, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved_gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved_gbs / peaks["hbm_gbs"], 4)},
        "points": points,
        "clocks": clocks,
    }
    line.update(workloads)
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
