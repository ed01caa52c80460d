"""Measurement: decoded tokens a second of a Llama-3.1-8B-shaped model with random
bfloat16 weights on one B200, with prefill throughput, the decode step's fraction of the
HBM roofline, decode at batch 1 and 64, and the other workloads that the baseline names
(the Llama-3.2-3B and -1B shapes, the two tiny configurations on the CPU's plain implementation).

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line.  A "step" is one decode step of the whole batch.  The timed
region is K steps bracketed by CUDA events after W untimed steps; every step reads all
layer weights (about 15 GB, far more than the 126 MB L2), so no L2 flush is needed.

How generation is timed follows the reference's own benchmark (cmd/benchmark_json/main.go:80-86,
108-115): the prompt step up to the first token is the prefill, tokens a second are counted over the
tokens after the first.
"""
from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))


def llama(hidden, layers, heads, kv_heads, head_dim, inter, factor, tied):
    return dict(architectures=["LlamaForCausalLM"], hidden_size=hidden, num_hidden_layers=layers,
                num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim, intermediate_size=inter,
                vocab_size=128256, rope_theta=500000.0,
                rope_scaling=dict(rope_type="llama3", factor=factor, low_freq_factor=1.0, high_freq_factor=4.0,
                                  original_max_position_embeddings=8192),
                rms_norm_eps=1e-5, tie_word_embeddings=tied, max_position_embeddings=131072)


MODEL = llama(4096, 32, 32, 8, 128, 14336, 8.0, False)           # Llama 3.1 8B layer sizes: the headline
MODEL_3B = llama(3072, 28, 24, 8, 128, 8192, 32.0, True)         # Llama 3.2 3B
MODEL_1B = llama(2048, 16, 32, 8, 64, 8192, 32.0, True)          # Llama 3.2 1B
CONTEXT = 4096
BATCH = 8
PREFILL_TOKENS = 2048
E2E_WARM = 48          # decode steps after a prompt step before a decode figure is timed (device-timed or end to end)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

REFERENCE_UNAVAILABLE = ("the reference is a Go program for Apple Metal with no Python package: pip reports "
                         "\"Directory is not installable. Neither 'setup.py' nor 'pyproject.toml' found\", "
                         "and no Go toolchain or Metal exists here")


def load_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            data = json.loads(path.read_text())
            peaks = {k: float(data[k]) for k in FALLBACK_PEAKS if k in data}
            if "hbm_gbs" in peaks and "bf16_tflops" in peaks:
                peaks.setdefault("bf16_tflops_sustained", peaks["bf16_tflops"])
                return peaks, "measured"
        except (ValueError, KeyError, TypeError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    FIELDS = ["clocks.sm", "clocks.max.sm", "clocks_event_reasons.hw_slowdown",
              "clocks_event_reasons.hw_thermal_slowdown", "clocks_event_reasons.sw_thermal_slowdown",
              "clocks_event_reasons.sw_power_cap"]

    def __init__(self):
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={','.join(self.FIELDS)}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
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
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != len(self.FIELDS):
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[2:]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


class FastClocks:
    """SM clock read through NVML every few milliseconds (reading only), to set the duration of single
    decode steps against the clock they ran at."""

    def __init__(self, period_s: float = 0.004):
        self.period, self.samples, self._stop, self._thread, self._nvml = period_s, [], threading.Event(), None, None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml, self._handle = pynvml, pynvml.nvmlDeviceGetHandleByIndex(0)
        except Exception:
            self._nvml = None

    def start(self):
        if self._nvml is None:
            return
        def run():
            nv = self._nvml
            while not self._stop.is_set():
                try:
                    self.samples.append((time.perf_counter(), nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM)))
                except Exception:
                    return
                self._stop.wait(self.period)
        self._thread = threading.Thread(target=run, daemon=True)
        self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)

    def median_between(self, t0: float, t1: float):
        mhz = [m for t, m in self.samples if t0 <= t <= t1]
        return statistics.median(mhz) if mhz else None


def linear_params(cfg) -> int:
    D, H, Hkv, hd, F = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                        cfg["intermediate_size"])
    return (H + 2 * Hkv) * hd * D + H * hd * D + 3 * F * D


def decode_bytes(cfg, layers: int, batch: int, context: float) -> float:
    """Bytes a decode step has to read: every weight it uses once, and the cache of the live requests."""
    weights = 2.0 * (layers * linear_params(cfg) + cfg["vocab_size"] * cfg["hidden_size"])
    weights += 4.0 * (2 * layers + 1) * cfg["hidden_size"]            # norm gains (float32)
    kv = batch * context * layers * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2.0
    return weights + kv


def prefill_flops(cfg, layers: int, lengths, logit_rows: int) -> float:
    tokens = sum(lengths)
    matmul = 2.0 * tokens * layers * linear_params(cfg) + 2.0 * logit_rows * cfg["vocab_size"] * cfg["hidden_size"]
    attn = sum(layers * 4.0 * cfg["num_attention_heads"] * cfg["head_dim"] * n * (n + 1) / 2.0 for n in lengths)
    return matmul + attn


def events(torch):
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def decode_run(torch, engine, rng, V, batch: int, steps: int, warm: int, prompt_len: int, params, sampler=None,
               settle: int = 0):
    """One prompt step, then decode steps fed with token ids that were drawn beforehand (no host read in the
    loop), each followed by the sampler on its logits: what the device does in a step, timed on the device.
    settle: untimed decode steps before the `warm` warm-up steps, for the clocks to come back from the prompt
    step (a long prompt step runs at the power cap, and the steps right after it at about half the clock)."""
    from longbow_quarrel_b200.kernels import ops
    from longbow_quarrel_b200.sampling import sample
    slots = [engine.new_sequence() for _ in range(batch)]
    prompts = [rng.integers(0, V, prompt_len).tolist() for _ in range(batch)]
    logits = engine.step(list(zip(slots, prompts)))
    warm += settle
    feed = rng.integers(0, V, (warm + steps, batch))
    scratch = torch.empty_like(logits)
    seq_ids = torch.arange(batch, dtype=torch.int32, device=logits.device)
    step_ids = torch.zeros(batch, dtype=torch.int32, device=logits.device)

    def one(i):
        out = engine.step([(s, [int(t)]) for s, t in zip(slots, feed[i])])
        sample(out, params, 1, seq_ids, step_ids, scratch=scratch)
    for i in range(warm):
        one(i)
    before = ops.launch_count()
    a, b = events(torch)
    torch.cuda.synchronize()
    if sampler:
        sampler.start()
    a.record()
    for i in range(warm, warm + steps):
        one(i)
    b.record()
    torch.cuda.synchronize()
    clocks = sampler.stop() if sampler else None
    ms = a.elapsed_time(b)
    for s in slots:
        engine.end_sequence(s)
    mean_ctx = prompt_len + warm + (steps - 1) / 2.0 + 1
    return ms, mean_ctx, ops.launch_count() - before, clocks


def timed_generate(engine, prompts, n_new, params, batch):
    """engine.generate with the arrival time of every step's tokens on the host: [t_prompt_done, t_1, ...]."""
    times, calls = [], [0]
    t0 = time.perf_counter()

    def on_token(i, tok):
        if calls[0] % batch == 0:
            times.append(time.perf_counter())
        calls[0] += 1
    out = engine.generate(prompts, max_new_tokens=n_new, sampling=params, stop_ids=[], callback=on_token)
    return out, t0, times


def other_workload(torch, np, peaks, name, cfg, prompt_lengths, n_steps, params, device_steps):
    """A workload of the baseline through the public entry point: one batch of prompts, then n_steps decode
    steps, host tokens in and out.  Returns flat figures for `points`."""
    from longbow_quarrel_b200.engine import Engine
    rng = np.random.default_rng(1)
    V, L, B = cfg["vocab_size"], cfg["num_hidden_layers"], len(prompt_lengths)
    longest = max(prompt_lengths) + n_steps + 1
    tokens = sum(-(-(n + n_steps + 1) // 64) * 64 for n in prompt_lengths)
    engine = Engine.from_config(cfg, seed=0, dtype="bfloat16", max_tokens=tokens, max_batch=B, max_context=longest,
                                gain_std=0.0)
    prompts = [rng.integers(0, V, n).tolist() for n in prompt_lengths]
    engine.generate(prompts, max_new_tokens=4, sampling=params, stop_ids=[])           # warm-up: kernels, graphs
    torch.cuda.synchronize()
    _, t0, times = timed_generate(engine, prompts, n_steps + 1, params, B)
    prefill_s = times[0] - t0
    decode_s = times[-1] - times[0]
    steps = len(times) - 1
    ms_step = decode_s / steps * 1e3
    mean_ctx = sum(prompt_lengths) / B + (steps + 1) / 2.0
    achieved = decode_bytes(cfg, L, B, mean_ctx) / (ms_step / 1e3) / 1e9
    out = {f"{name}_decode": B * steps / decode_s, f"{name}_ms_per_step": ms_step, f"{name}_decode_frac": achieved / peaks["hbm_gbs"],
           f"{name}_prefill": sum(prompt_lengths) / prefill_s,
           f"{name}_prefill_frac": prefill_flops(cfg, L, prompt_lengths, B) / prefill_s / (peaks["bf16_tflops"] * 1e12)}
    if device_steps:
        # The same decode steps without the host in the loop (tokens drawn beforehand, nothing read back): what is
        # left of a step when the host costs nothing.  1 - device / end-to-end is the host's share of a step.
        # (at the same mean context as the steps above: the prompt is as much longer as those steps are more)
        start = max(1, int(mean_ctx - E2E_WARM - 8 - device_steps / 2.0))
        ms, _, _, _ = decode_run(torch, engine, rng, V, B, device_steps, 8, start, params, settle=E2E_WARM)
        out[f"{name}_device_ms_per_step"] = ms / device_steps
        out[f"{name}_host_share"] = max(0.0, 1.0 - (ms / device_steps) / ms_step)
    engine.close()
    del engine
    torch.cuda.empty_cache()
    return out


def tiny_workloads(torch) -> dict:
    """The two tiny configurations of the baseline (float32): seconds of the plain CPU implementation (the
    oracle of the tests, whole sequences re-run for every token) and of the engine's 32-bit path on the GPU for
    the same greedy generation, and whether they chose the same tokens."""
    import tempfile

    sys.path.insert(0, str(ROOT / "tests"))
    import plain_llama
    from helpers import TINY, make_model_folder, random_tokens
    from longbow_quarrel_b200.engine import Engine
    from longbow_quarrel_b200.sampling import SamplingParams
    out = {}
    for name, lengths, n_new in (("a", [7, 3, 12, 1], 8), ("b", [20, 5, 33], 16)):
        with tempfile.TemporaryDirectory() as tmp:
            folder = make_model_folder(tmp, name.upper(), seed=7)
            vocab = TINY[name.upper()]["vocab_size"]
            prompts = [random_tokens(n, vocab, 300 + i) for i, n in enumerate(lengths)]
            cfg, weights = plain_llama.load_folder(folder)
            t0 = time.perf_counter()
            want = [plain_llama.greedy(cfg, weights, p, n_new) for p in prompts]
            out[f"tiny_{name}_plain_cpu_s"] = time.perf_counter() - t0
            engine = Engine.from_pretrained(folder, dtype="float32", max_tokens=1024)
            engine.generate(prompts, max_new_tokens=2, sampling=SamplingParams(), stop_ids=[])
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            got = engine.generate(prompts, max_new_tokens=n_new, sampling=SamplingParams(), stop_ids=[])
            out[f"tiny_{name}_engine_fp32_s"] = time.perf_counter() - t0
            out[f"tiny_{name}_same_tokens"] = got == want
            engine.close()
    return out


# ------------------------------------------------------------------ --design fetorax: the design beside Llama at equal layer sizes
DESIGN_SIZES = {   # width, heads, kv heads, head size, feed-forward width: the layer sizes of the 1B and 8B Llama shapes
    "1b": (2048, 32, 8, 64, 8192),
    "8b": (4096, 32, 8, 128, 14336),
}
DESIGN_VOCAB = 32000


def fetorax_config(width, heads, kv_heads, dim, ff, groups: int = 1) -> dict:
    """`groups` times four layers: attention, retention, mlstm, attention on the first one's keys and values."""
    rot = {"dims": dim // 2, "base": 1e6, "scaling": {"factor": 2.0}}
    mlp = {"kind": "dense", "ff": ff}
    layers = []
    for g in range(groups):
        att = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "rot": rot}
        layers += [
            {"type": "attention", "mixer": dict(att), "mlp": mlp},
            {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": dim, "rot": {"dims": dim, "base": 1e4},
                                            "decay": [1.0 - 2.0 ** (-5 - 3 * h / heads) for h in range(heads)]}, "mlp": mlp},
            {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": dim, "gate_cap": 15.0}, "mlp": mlp},
            {"type": "attention", "mixer": dict(att, kv_from=4 * g), "mlp": mlp},
        ]
    return {"architecture": "Fetorax", "vocab": DESIGN_VOCAB, "width": width, "norm": {"eps": 1e-5}, "layers": layers,
            "logit_softcap": 30.0, "max_positions": 8192}


ZOPORAX_SIZES = {   # width, heads, unrotated / rotated / value size of a head, query and latent ranks, dense ff, experts, top, expert ff, shared ff
    "1b": (2048, 16, 128, 64, 128, 768, 512, 8192, 64, 6, 1408, 2816),
    "8b": (4096, 32, 128, 64, 128, 1536, 512, 14336, 64, 6, 2048, 4096),
}


def zoporax_config(size: str, window: int, groups: int = 1) -> dict:
    """`groups` times four layers: latent attention and lightning by turns, a dense feed-forward behind the first
    and routed experts (eight groups of which three are kept, a shared expert) behind the others."""
    width, heads, dn, dr, dv, rq, rkv, ff, experts, top, eff, sff = ZOPORAX_SIZES[size]
    lat = {"heads": heads, "dim": dn, "rot_dim": dr, "vdim": dv, "q_rank": rq, "kv_rank": rkv, "scale": (dn + dr) ** -0.5,
           "mask": {"size": window},
           "rot": {"dims": dr, "base": 1e4, "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    lk = DESIGN_SIZES[size][3]
    lig = {"heads": DESIGN_SIZES[size][1], "dim": lk, "vdim": lk,
           "decay": [1.0 - 2.0 ** (-5 - 3 * h / DESIGN_SIZES[size][1]) for h in range(DESIGN_SIZES[size][1])]}
    moe = {"kind": "moe", "expert": {"ff": eff}, "shared": {"ff": sff},
           "router": {"experts": experts, "top": top, "scale": 2.5, "groups": {"count": 8, "keep": 3}}}
    layers = []
    for _ in range(groups):
        layers += [{"type": "latent_attention", "mixer": dict(lat), "mlp": {"kind": "dense", "ff": ff}},
                   {"type": "lightning", "mixer": dict(lig), "mlp": moe},
                   {"type": "latent_attention", "mixer": dict(lat), "mlp": moe},
                   {"type": "lightning", "mixer": dict(lig), "mlp": moe}]
    return {"architecture": "Zoporax", "vocab": DESIGN_VOCAB, "width": width, "norm": {"eps": 1e-5}, "layers": layers,
            "max_positions": 8192}


def raritar_config(size: str, window: int) -> dict:
    """Four layers of attention (capped scores, a window with kept first positions, rotation of half of each head with
    rescaled frequencies, normed values; the last layer on the first one's keys and values) behind a causal convolution,
    each with routed gated experts (62 and two identity outputs in eight groups of which three are kept, six per token) and
    a shared expert; pair-hash embedding; branch multiplier."""
    width, heads, kv, dim, _ = DESIGN_SIZES[size]
    experts, top, eff, sff = ZOPORAX_SIZES[size][8:12]
    att = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "softcap": 50.0,
           "mask": {"size": window, "keep_first": 4},
           "rot": {"dims": dim // 2, "base": 5e5, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    moe = {"kind": "moe", "expert": {"ff": eff}, "shared": {"ff": sff},
           "router": {"experts": experts - 2, "identity": 2, "top": top, "groups": {"count": 8, "keep": 3}}}
    layers = [{"type": "attention", "mixer": dict(att, **({"kv_from": 0} if i == 3 else {})), "mlp": moe} for i in range(4)]
    return {"architecture": "Raritar", "vocab": DESIGN_VOCAB, "width": width, "norm": {"eps": 1e-5}, "residual_mult": 0.5,
            "canon": {"taps": 4}, "embedding": {"bigram": {"buckets": 65521, "mul_prev": 131, "mul_cur": 71}},
            "layers": layers, "max_positions": 8192}


def _kernel_times(torch, run, warm: int = 2) -> tuple[dict, float]:
    """What every kind of kernel adds to the device time of one call of run(): {kind: (launches, total us)}, and the span."""
    import re

    from torch.profiler import ProfilerActivity, profile
    for _ in range(warm):
        run()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        run()
        torch.cuda.synchronize()
    ev = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA
          and not re.search("[Mm]emcpy|[Mm]emset", e.name)]
    # Kernels are launched ahead and wait for the one before them, so a kernel's own span overlaps its
    # predecessor's: what counts is by how much it ends after the kernel before it.
    ev.sort(key=lambda e: e.time_range.start)
    kinds: dict = {}
    prev_end = ev[0].time_range.start if ev else 0.0
    for e in ev:
        m = re.search(r"(\w+)_kernel", e.name)
        k = kinds.setdefault(m.group(1) if m else e.name[:40], [0, 0.0])
        k[0] += 1
        k[1] += max(0.0, e.time_range.end - prev_end)
        prev_end = max(prev_end, e.time_range.end)
    span = max(e.time_range.end for e in ev) - min(e.time_range.start for e in ev) if ev else 0.0
    return {k: (n, round(us, 1)) for k, (n, us) in sorted(kinds.items(), key=lambda kv: -kv[1][1])}, round(span, 1)


def design_bench(args) -> int:
    if args.design == "zoporax":
        return zoporax_bench(args)
    if args.design == "raritar":
        return raritar_bench(args)
    if args.design == "lavutar":
        return lavutar_bench(args)
    return fetorax_bench(args)


def _design_run(torch, np, Engine, cfg, name, T, B, ctx, K, W, rng) -> dict:
    """One model's prompt step and decode step: ms, tokens a second, and what every kind of kernel adds to each."""
    eng = Engine.from_config(cfg, seed=0, dtype="bfloat16", max_tokens=B * (ctx + 256) + T + 64, max_batch=B + 1,
                             max_context=ctx + 256, gain_std=0.0 if name == "llama" else 0.1)
    prompt = rng.integers(0, DESIGN_VOCAB, T).tolist()

    def prefill():
        s = eng.new_sequence()
        eng.step([(s, prompt)])
        eng.end_sequence(s)
    for _ in range(W):
        prefill()
    a, b = events(torch)
    fast = FastClocks()              # the SM clock inside the two timed regions (the run's median also holds the idle set-up)
    fast.start()
    torch.cuda.synchronize()
    t_pre = [time.perf_counter()]
    a.record()
    for _ in range(max(3, K // 4)):
        prefill()
    b.record()
    torch.cuda.synchronize()
    t_pre.append(time.perf_counter())
    prefill_ms = a.elapsed_time(b) / max(3, K // 4)
    prefill_kinds, _ = _kernel_times(torch, prefill)
    slots = [eng.new_sequence() for _ in range(B)]
    eng.step([(s, rng.integers(0, DESIGN_VOCAB, ctx).tolist()) for s in slots])
    feed = rng.integers(0, DESIGN_VOCAB, (W + K + 8, B))
    at = [0]

    def decode():
        eng.step([(s, [int(t)]) for s, t in zip(slots, feed[at[0]])])
        at[0] += 1
    for _ in range(W):
        decode()
    torch.cuda.synchronize()
    t_dec = [time.perf_counter()]
    a.record()
    for _ in range(K):
        decode()
    b.record()
    torch.cuda.synchronize()
    t_dec.append(time.perf_counter())
    fast.stop()
    decode_ms = a.elapsed_time(b) / K
    decode_kinds, _ = _kernel_times(torch, decode)
    res = {"sm_mhz_timed": {"prefill": fast.median_between(*t_pre), "decode": fast.median_between(*t_dec)},
           "prefill_tokens_per_s": round(T / prefill_ms * 1e3), "prefill_ms": round(prefill_ms, 3),
           "decode_tokens_per_s": round(B / decode_ms * 1e3), "decode_ms_per_step": round(decode_ms, 4),
           "prefill_kernels_us": prefill_kinds, "decode_kernels_us": decode_kinds, "weight_bytes": eng.model.weight_bytes()}
    eng.close()
    del eng
    torch.cuda.empty_cache()
    return res


def zoporax_bench(args) -> int:
    """Prefill and decode of a Zoporax model of realistic layer sizes beside the closest model the library has, a
    Fetorax model of attention and retention layers of the same width, depth and dense feed-forward (random weights,
    vocabulary 32,000): tokens a second, what every kind of kernel adds to a prompt step and to a decode step, and
    for the kernels that the design added how many times their roofline they take, beside the like kernel of
    the other model (attention for latent attention; the scan is the same kernel in both)."""
    import numpy as np
    import torch

    from longbow_quarrel_b200.engine import Engine
    peaks, peaks_from = load_peaks()
    K, W = args.steps, max(3, args.warmup)
    T, B, ctx = PREFILL_TOKENS, BATCH, 2048
    hbm, tensor = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    rng = np.random.default_rng(0)
    sampler = ClockSampler()
    sampler.start()
    out = {}
    for size in args.sizes.split(","):
        width, heads, kv, dim, ff = DESIGN_SIZES[size]
        _, zh, dn, dr, dv, rq, rkv, _, experts, top, eff, sff = ZOPORAX_SIZES[size]
        beside = fetorax_config(width, heads, kv, dim, ff)
        for i, layer in enumerate(beside["layers"]):       # attention and retention by turns, each with keys of its own
            if i % 2:
                layer["type"], layer["mixer"] = "retention", dict(beside["layers"][1]["mixer"])
            else:
                layer["type"], layer["mixer"] = "attention", {k: v for k, v in beside["layers"][0]["mixer"].items() if k != "kv_from"}
        configs = {"zoporax": zoporax_config(size, ctx + 256), "fetorax": beside}
        res = {name: _design_run(torch, np, Engine, cfg, name, T, B, ctx, K, W, rng) for name, cfg in configs.items()}

        def per_launch(kinds, *names):
            n = sum(kinds[k][0] for k in names if k in kinds)
            return sum(kinds[k][1] for k in names if k in kinds) / n if n else None

        def times(us, nbytes, flops):
            return round(us / (max(nbytes / hbm, flops / tensor) * 1e6), 2) if us else None
        z, f = res["zoporax"], res["fetorax"]
        Dk = rkv + dr
        pairs = T * (T + 1) / 2
        roof = {
            "prefill": {
                "fetorax attention": times(per_launch(f["prefill_kernels_us"], "attn_prefill_two", "attn_prefill_tc", "attn_prefill"),
                                           T * heads * 3 * dim * 2.0, 4.0 * heads * dim * pairs),
                "zoporax latent attention": times(per_launch(z["prefill_kernels_us"], "latent_attention", "latent_attention_tc"),
                                                  T * zh * (Dk + rkv) * 4.0 + T * Dk * 2.0, 2.0 * zh * (Dk + rkv) * pairs),
                "zoporax per-head matrices": times(per_launch(z["prefill_kernels_us"], "head_matmul", "grouped_gemm"),
                                                   T * zh * (dn + rkv + dv) * 3.0, 2.0 * T * zh * rkv * (dn + dv) / 2),
                "fetorax recurrent scan": times(per_launch(f["prefill_kernels_us"], "linear_scan"),
                                                T * heads * 3 * dim * 2.0 + T * heads * dim * 4.0, 4.0 * T * heads * dim * dim),
                "zoporax recurrent scan": times(per_launch(z["prefill_kernels_us"], "linear_scan"),
                                                T * heads * 3 * dim * 2.0 + T * heads * dim * 4.0, 4.0 * T * heads * dim * dim),
                # The experts' six products of a prompt step are launches of gemm_tc, which also served two small
                # products of the step: their time rides in the sum (an upper bound).
                "zoporax experts, either product": times(sum(z["prefill_kernels_us"].get(k, (0, 0.0))[1] for k in ("gemm_tc",)) / 6 or None,
                                                         experts * eff * width * 2.0, 2.0 * T * top * eff * width),
            },
            "decode": {
                "fetorax attention": times(per_launch(f["decode_kernels_us"], "attn_decode"), B * ctx * 2 * kv * dim * 2.0, 0.0),
                "zoporax latent attention": times(per_launch(z["decode_kernels_us"], "latent_attention", "latent_attention_tc"),
                                                  B * ctx * Dk * 2.0, 0.0),
                "fetorax recurrent scan": times(per_launch(f["decode_kernels_us"], "linear_scan_single"), B * heads * dim * dim * 8.0, 0.0),
                "zoporax recurrent scan": times(per_launch(z["decode_kernels_us"], "linear_scan_single"), B * heads * dim * dim * 8.0, 0.0),
                "zoporax experts, first product": times(per_launch(z["decode_kernels_us"], "moe_up"), min(B * top, experts) * eff * width * 2.0, 0.0),
                "zoporax experts, second product": times(per_launch(z["decode_kernels_us"], "moe_down"), min(B * top, experts) * eff * width * 2.0, 0.0),
            },
        }
        out[size] = {"zoporax": z, "fetorax": f, "times_the_roofline": roof,
                     "zoporax_over_fetorax": {"prefill": round(z["prefill_tokens_per_s"] / f["prefill_tokens_per_s"], 3),
                                              "decode": round(z["decode_tokens_per_s"] / f["decode_tokens_per_s"], 3)}}
    clocks = sampler.stop()
    print(json.dumps({"design": "zoporax", "beside": "fetorax", "dtype": "bf16", "data": "synthetic", "layers": 4,
                      "layer_order": "latent attention + dense, lightning + experts, latent attention + experts, lightning + experts; "
                                     "beside attention, retention, attention, retention, each + dense",
                      "vocab": DESIGN_VOCAB, "prefill_tokens": T, "decode_batch": B, "decode_context": ctx, "steps": K,
                      "warmup": W, "peaks": peaks, "peaks_from": peaks_from, "clocks": clocks, "sizes": out}))
    return 0


def _expert_products_us(torch, T, B, width, experts, identity, top, eff, gated, K) -> dict:
    """Device time of the experts' products alone at one layer's sizes, random routing: the prompt's two row-tiled tcgen05
    products (with the gather ahead of them, the activation between them and the combination behind them) for T tokens,
    and the two streaming kernels for B single tokens.  Every launch reads other weights than fit in L2 beside the one
    before it (several hundred MB of experts), so nothing is flushed."""
    from longbow_quarrel_b200.kernels import ops
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(1)
    n_up = 2 * eff if gated else eff
    w_up = torch.randn((experts, n_up, width), device=dev, dtype=torch.bfloat16, generator=g) * width ** -0.5     # gated: gate and up rows by turns
    w_down = torch.randn((experts, width, eff), device=dev, dtype=torch.bfloat16, generator=g) * eff ** -0.5
    act = "silu"

    def case(rows):
        h = torch.randn((rows, width), device=dev, dtype=torch.bfloat16, generator=g)
        ids = torch.stack([torch.randperm(experts + identity, device=dev, generator=g)[:top] for _ in range(rows)]).to(torch.int32)
        weights = torch.rand((rows, top), device=dev, generator=g)
        return h, ids.contiguous(), weights, torch.zeros((rows, width), device=dev, dtype=torch.float32)

    def timed(fn):
        for _ in range(3):
            fn()
        a, b = events(torch)
        torch.cuda.synchronize()
        a.record()
        for _ in range(K):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / K * 1e3
    out = {}
    h, ids, weights, x = case(T)
    more = dict(ids=ids, E=experts, h=h) if identity else {}
    src, dst, tile_group = ops.group_rows_padded(ids.view(-1), experts)
    rows = ops.gather_rows(h, src, top)
    out["prompt_first_product"] = timed(lambda: ops.gemm_tc_grouped(rows, w_up, tile_group, h.dtype, swiglu=gated))
    u = ops.gemm_tc_grouped(rows, w_up, tile_group, h.dtype, swiglu=gated)
    if not gated:
        ops.activation(u, act, out=u)
    out["prompt_second_product"] = timed(lambda: ops.gemm_tc_grouped(u, w_down, tile_group, torch.float32))
    y = ops.gemm_tc_grouped(u, w_down, tile_group, torch.float32)

    def around():
        s2, d2, _ = ops.group_rows_padded(ids.view(-1), experts)
        r2 = ops.gather_rows(h, s2, top)
        if not gated:
            ops.activation(torch.empty((r2.shape[0], n_up), device=dev, dtype=h.dtype), act)
        ops.moe_combine(y, weights, x, accumulate=True, place=d2, **more)
    out["prompt_order_gather_activation_combination"] = timed(around)
    h, ids, weights, x = case(B)
    out["single_tokens_first_product"] = timed(lambda: ops.moe_up(h, w_up, ids, act, gated=gated, block=8 if gated else 0))
    u = ops.moe_up(h, w_up, ids, act, gated=gated, block=8 if gated else 0)
    out["single_tokens_second_product"] = timed(lambda: ops.moe_down(u, w_down, ids, weights, x, accumulate=True,
                                                                     h=h if identity else None))
    del w_up, w_down
    torch.cuda.empty_cache()
    return {k: round(v, 1) for k, v in out.items()}


def raritar_bench(args) -> int:
    """Prefill and decode of a Raritar model of realistic layer sizes beside the closest model the library has, a Llama
    model of the same width, depth, heads and head size (random weights, vocabulary 32,000, the window longer than the
    context so that both attend to every key): tokens a second, what every kind of kernel adds to a prompt step and to a
    decode step, and how many times their roofline the design's kernels take beside the like kernels: attention beside
    Llama's attention, and the gated experts' products beside the ungated ones of equal sizes as the Zoporax design runs them."""
    import numpy as np
    import torch

    from longbow_quarrel_b200.engine import Engine
    peaks, peaks_from = load_peaks()
    K, W = args.steps, max(3, args.warmup)
    T, B, ctx = PREFILL_TOKENS, BATCH, 2048
    hbm, tensor = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    rng = np.random.default_rng(0)
    sampler = ClockSampler()
    sampler.start()
    out = {}
    for size in args.sizes.split(","):
        width, heads, kv, dim, ff = DESIGN_SIZES[size]
        experts, top, eff, sff = ZOPORAX_SIZES[size][8:12]
        configs = {"raritar": raritar_config(size, ctx + 256),
                   "llama": dict(llama(width, 4, heads, kv, dim, ff, 8.0, False), vocab_size=DESIGN_VOCAB, max_position_embeddings=8192)}
        res = {name: _design_run(torch, np, Engine, cfg, name, T, B, ctx, K, W, rng) for name, cfg in configs.items()}
        gated = _expert_products_us(torch, T, B, width, experts - 2, 2, top, eff, True, max(5, K // 4))
        plain = _expert_products_us(torch, T, B, width, experts, 0, top, eff, False, max(5, K // 4))

        def per_launch(kinds, *names):
            n = sum(kinds[k][0] for k in names if k in kinds)
            return sum(kinds[k][1] for k in names if k in kinds) / n if n else None

        def times(us, nbytes, flops):
            return round(us / (max(nbytes / hbm, flops / tensor) * 1e6), 2) if us else None
        r, l = res["raritar"], res["llama"]
        qkv_bytes = T * heads * 3 * dim * 2.0
        att_flops = 4.0 * heads * dim * T * (T + 1) / 2
        kv_read = B * ctx * 2 * kv * dim * 2.0
        real = top * (experts - 2) / experts                       # of a token's choices, those with matrices of their own

        def expert_rows(us, n_up, share, hit):
            """times the roofline: first product, second product of a prompt; first, second of single tokens."""
            w1, w2 = n_up * width * 2.0, eff * width * 2.0
            return {"prompt, first product": times(us["prompt_first_product"], hit * w1 + T * share * (width + n_up) * 2.0,
                                                   2.0 * T * share * n_up * width),
                    "prompt, second product": times(us["prompt_second_product"], hit * w2 + T * share * (eff * 2.0 + width * 4.0),
                                                    2.0 * T * share * eff * width),
                    "single tokens, first product": times(us["single_tokens_first_product"], min(B * share, hit) * w1, 0.0),
                    "single tokens, second product": times(us["single_tokens_second_product"], min(B * share, hit) * w2, 0.0)}
        roof = {
            "prefill": {
                "llama attention": times(per_launch(l["prefill_kernels_us"], "attn_prefill_two", "attn_prefill_tc", "attn_prefill"),
                                         qkv_bytes, att_flops),
                "raritar attention (capped, window, kept first)": times(
                    per_launch(r["prefill_kernels_us"], "attn_prefill_two", "attn_prefill_tc", "attn_prefill"), qkv_bytes, att_flops),
            },
            "decode": {
                "llama attention": times(per_launch(l["decode_kernels_us"], "attn_decode"), kv_read, 0.0),
                "raritar attention (capped, window, kept first)": times(per_launch(r["decode_kernels_us"], "attn_decode"), kv_read, 0.0),
            },
            "raritar gated experts": expert_rows(gated, 2 * eff, real, experts - 2),
            "ungated experts of equal sizes": expert_rows(plain, eff, top, experts),
        }
        out[size] = {"raritar": r, "llama": l, "expert_products_us": {"raritar gated": gated, "ungated": plain},
                     "times_the_roofline": roof,
                     "raritar_over_llama": {"prefill": round(r["prefill_tokens_per_s"] / l["prefill_tokens_per_s"], 3),
                                            "decode": round(r["decode_tokens_per_s"] / l["decode_tokens_per_s"], 3)}}
    clocks = sampler.stop()
    print(json.dumps({"design": "raritar", "beside": "llama", "dtype": "bf16", "data": "synthetic", "layers": 4,
                      "layer_order": "attention + routed gated experts four times, the last on the first layer's keys and values; "
                                     "beside attention + gated feed-forward four times",
                      "vocab": DESIGN_VOCAB, "prefill_tokens": T, "decode_batch": B, "decode_context": ctx, "steps": K,
                      "warmup": W, "peaks": peaks, "peaks_from": peaks_from, "clocks": clocks, "sizes": out}))
    return 0


def lavutar_config(size: str, block: int, window: int) -> dict:
    """Four layers: attention over blocks of positions with whole-projection norms, capped scores and a gate per head,
    behind a gated feed-forward; two sides side by side (softmax attention with per-head norms and a query temperature,
    linear attention with a decay for every key channel) behind routed gated experts; windowed attention with a
    YaRN-blended rotation behind a gated feed-forward; the two sides again behind a gated feed-forward.  The middle two
    layers are a stretch that is entered through the product over the stream and the embedding's rows."""
    width, heads, kv, dim, ff = DESIGN_SIZES[size]
    experts, top, eff = ZOPORAX_SIZES[size][8:11]
    dense = {"kind": "dense", "ff": ff}
    soft = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": dim ** -0.5}
    two = {"left": dict(soft, q_temp={"coef": 0.1, "every": 256}), "left_scale": 0.8, "right_scale": 0.5,
           "right": {"heads": heads, "dim": dim, "vdim": dim, "tau": 16.0, "rank": 64}}
    layers = [
        {"type": "attention_2", "mixer": dict(soft, softcap=50.0, mask={"size": block}), "mlp": dense},
        {"type": "parallel", "mixer": two, "mlp": {"kind": "moe", "expert": {"ff": eff}, "router": {"experts": experts, "top": top}}},
        {"type": "attention", "mixer": dict(soft, mask={"size": window}, rot={"dims": dim, "base": 1e5, "scaling": {
            "factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}), "mlp": dense},
        {"type": "parallel", "mixer": two, "mlp": dense}]
    return {"architecture": "Lavutar", "vocab": DESIGN_VOCAB, "width": width, "norm": {"eps": 1e-5}, "layers": layers,
            "loop": {"start": 1, "stop": 3, "times": 1}, "max_positions": 8192}


def lavutar_bench(args) -> int:
    """Prefill and decode of a Lavutar model of realistic layer sizes beside the closest model the library has, a
    Fetorax model of attention (sink and gate) and retention layers of the same width, depth and feed-forward width
    (random weights, vocabulary 32,000): tokens a second, what every kind of kernel adds to a prompt step and to a decode
    step, and for the design's kernels how many times their roofline they take, beside the like kernel of the other model."""
    import numpy as np
    import torch

    from longbow_quarrel_b200.engine import Engine
    peaks, peaks_from = load_peaks()
    K, W = args.steps, max(3, args.warmup)
    T, B, ctx = PREFILL_TOKENS, BATCH, 2048
    hbm, tensor = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    rng = np.random.default_rng(0)
    sampler = ClockSampler()
    sampler.start()
    out = {}
    for size in args.sizes.split(","):
        width, heads, kv, dim, ff = DESIGN_SIZES[size]
        experts, top, eff = ZOPORAX_SIZES[size][8:11]
        beside = fetorax_config(width, heads, kv, dim, ff)
        for i, layer in enumerate(beside["layers"]):       # attention and retention by turns, each with keys of its own
            if i % 2:
                layer["type"], layer["mixer"] = "retention", dict(beside["layers"][1]["mixer"])
            else:
                layer["type"], layer["mixer"] = "attention", {k: v for k, v in beside["layers"][0]["mixer"].items() if k != "kv_from"}
        block, window = 1024, 1024
        configs = {"lavutar": lavutar_config(size, block, window), "fetorax": beside}
        res = {name: _design_run(torch, np, Engine, cfg, name, T, B, ctx, K, W, rng) for name, cfg in configs.items()}

        def per_launch(kinds, *names):
            n = sum(kinds[k][0] for k in names if k in kinds)
            return sum(kinds[k][1] for k in names if k in kinds) / n if n else None

        def times(us, nbytes, flops):
            return round(us / (max(nbytes / hbm, flops / tensor) * 1e6), 2) if us else None

        def us(kinds, *names):
            v = per_launch(kinds, *names)
            return round(v, 1) if v is not None else None
        v, f = res["lavutar"], res["fetorax"]
        vp, vd, fp, fd = v["prefill_kernels_us"], v["decode_kernels_us"], f["prefill_kernels_us"], f["decode_kernels_us"]
        qkv_bytes = T * heads * 3 * dim * 2.0
        # Visible (query, key) pairs of a prompt: all earlier positions; a window or blocks of 1,024 positions see about
        # three quarters of them at 2,048 tokens.  The design's three attentions share one kernel: their mean is taken.
        full = T * (T + 1) / 2
        seen = (full + (full - (T - window) * (T - window + 1) / 2) + 2 * (block * (block + 1) / 2) + full) / 4 if T > window else full
        scan_bytes = qkv_bytes + T * heads * dim * 4.0
        scan_flops = 4.0 * T * heads * dim * dim
        state = B * heads * dim * dim * 4.0 * 2
        kv_read = B * ctx * 2 * kv * dim * 2.0
        kv_seen = B * (ctx + min(ctx, window) + (ctx % block + 1) + ctx) / 4 * 2 * kv * dim * 2.0
        roof = {
            "prefill": {
                "fetorax attention (sink, gate)": times(per_launch(fp, "attn_prefill_two", "attn_prefill_tc", "attn_prefill"),
                                                        qkv_bytes, 4.0 * heads * dim * full),
                "lavutar attention (blocks / window / all, sink)": times(per_launch(vp, "attn_prefill_two", "attn_prefill_tc", "attn_prefill"),
                                                                         qkv_bytes, 4.0 * heads * dim * seen),
                "fetorax recurrent scan": times(per_launch(fp, "linear_scan"), scan_bytes, scan_flops),
                "lavutar recurrent scan (channel decays)": times(per_launch(vp, "linear_scan"), scan_bytes + T * heads * dim * 4.0, scan_flops),
                "fetorax norm": times(per_launch(fp, "rmsnorm_add", "rmsnorm", "rmsnorm_vec"), T * width * 10.0, 0.0),
                # Seven of its nine launches norm the stream alone (4 bytes in, 2 out a number); two also add both sides'
                # branches into it (8 for the stream, 8 for the branches, 2 out).
                "lavutar layer norm": times(per_launch(vp, "layernorm", "layernorm_vec"), T * width * (7 * 6.0 + 2 * 18.0) / 9, 0.0),
                "fetorax rotation + cache write": times(per_launch(fp, "rope_partial"), T * (heads + 2 * kv) * dim * 6.0, 0.0),
                "lavutar unit norms + rotation + cache write": times(per_launch(vp, "rope_partial"), T * (heads + 2 * kv) * dim * 6.0, 0.0),
                "lavutar experts, either product": times(sum(vp.get(k, (0, 0.0))[1] for k in ("gemm_tc_grouped", "gemm_tc")) / 2 or None,
                                                         experts * eff * width * 2.0 * 1.5, 2.0 * T * top * eff * width * 1.5),
            },
            "decode": {
                "fetorax attention (sink, gate)": times(per_launch(fd, "attn_decode"), kv_read, 0.0),
                "lavutar attention (blocks / window / all, sink)": times(per_launch(vd, "attn_decode"), kv_seen, 0.0),
                "fetorax recurrent scan": times(per_launch(fd, "linear_scan_single"), state, 0.0),
                "lavutar recurrent scan (channel decays)": times(per_launch(vd, "linear_scan_single"), state, 0.0),
                "lavutar experts, first product": times(per_launch(vd, "moe_up", "moe_up_rows"), min(B * top, experts) * eff * width * 4.0, 0.0),
                "lavutar experts, second product": times(per_launch(vd, "moe_down"), min(B * top, experts) * eff * width * 2.0, 0.0),
            },
        }
        small = {"prefill_us_per_launch": {k: us(vp, *names) for k, names in {
                     "layer norm": ("layernorm", "layernorm_vec"), "unit norms + rotation + cache write": ("rope_partial",),
                     "stream and embedding side by side": ("side_by_side", "side_by_side_vec"), "gate after attention": ("gate_mul",),
                     "gelu(gate) * up": ("gated_act", "gated_act_vec"), "decays' second product (32-bit)": ("gemm_plain",), "unit norm per head + gate": ("head_norm_gate", "head_norm_gate_wide"),
                     "router's 32-bit product": ("small_proj",), "router choice": ("moe_route",)}.items()},
                 "decode_us_per_launch": {k: us(vd, *names) for k, names in {
                     "layer norm": ("layernorm", "layernorm_vec"), "unit norms + rotation + cache write": ("rope_partial",),
                     "gate after attention": ("gate_mul",), "gelu(gate) * up": ("gated_act", "gated_act_vec"),
                     "decays' second product (32-bit)": ("gemm_plain",),
                     "unit norm per head + gate": ("head_norm_gate", "head_norm_gate_wide"),
                     "router's 32-bit product": ("small_proj",)}.items()},
                 "fetorax_prefill_us_per_launch": {k: us(fp, *names) for k, names in {
                     "branch norm + add + next norm": ("rmsnorm_add",), "biases + rotation + cache write": ("rope_partial",),
                     "gate after attention": ("gate_mul",), "unit norm per head + gate": ("head_norm_gate",)}.items()}}
        out[size] = {"lavutar": v, "fetorax": f, "times_the_roofline": roof, "small_kernels": small,
                     "lavutar_over_fetorax": {"prefill": round(v["prefill_tokens_per_s"] / f["prefill_tokens_per_s"], 3),
                                              "decode": round(v["decode_tokens_per_s"] / f["decode_tokens_per_s"], 3)}}
    clocks = sampler.stop()
    print(json.dumps({"design": "lavutar", "beside": "fetorax", "dtype": "bf16", "data": "synthetic", "layers": 4,
                      "layer_order": "attention over blocks + gated ff, two sides + experts, windowed attention + gated ff, two sides + gated ff "
                                     "(the middle two behind the stream's product); beside attention, retention, attention, retention, each + ff",
                      "vocab": DESIGN_VOCAB, "prefill_tokens": T, "decode_batch": B, "decode_context": ctx, "steps": K,
                      "warmup": W, "peaks": peaks, "peaks_from": peaks_from, "clocks": clocks, "sizes": out}))
    return 0


def fetorax_bench(args) -> int:
    """Prefill and decode of a Fetorax model of the 1B and 8B layer sizes beside a Llama model of the same sizes
    (random weights, vocabulary cut to 32,000): tokens a second, the device time of every kind of kernel in one
    prompt step and one decode step, and for the kernels that the design added how many times their roofline
    they take, beside the like kernel of the Llama model (attention)."""
    import numpy as np
    import torch

    from longbow_quarrel_b200.engine import Engine
    peaks, peaks_from = load_peaks()
    K, W = args.steps, max(3, args.warmup)
    T, B, ctx = PREFILL_TOKENS, BATCH, 2048
    hbm, tensor = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    rng = np.random.default_rng(0)
    sampler = ClockSampler()
    sampler.start()
    out = {}
    for size in args.sizes.split(","):
        width, heads, kv, dim, ff = DESIGN_SIZES[size]
        configs = {"fetorax": fetorax_config(width, heads, kv, dim, ff),
                   "llama": dict(llama(width, 4, heads, kv, dim, ff, 8.0, False), vocab_size=DESIGN_VOCAB, max_position_embeddings=8192)}
        res = {}
        for name, cfg in configs.items():
            eng = Engine.from_config(cfg, seed=0, dtype="bfloat16", max_tokens=B * (ctx + 256) + T + 64, max_batch=B + 1,
                                     max_context=ctx + 256, gain_std=0.0 if name == "llama" else 0.1)
            prompt = rng.integers(0, DESIGN_VOCAB, T).tolist()

            def prefill():
                s = eng.new_sequence()
                eng.step([(s, prompt)])
                eng.end_sequence(s)
            for _ in range(W):
                prefill()
            a, b = events(torch)
            torch.cuda.synchronize()
            a.record()
            for _ in range(max(3, K // 4)):
                prefill()
            b.record()
            torch.cuda.synchronize()
            prefill_ms = a.elapsed_time(b) / max(3, K // 4)
            prefill_kinds, prefill_span = _kernel_times(torch, prefill)
            slots = [eng.new_sequence() for _ in range(B)]
            eng.step([(s, rng.integers(0, DESIGN_VOCAB, ctx).tolist()) for s in slots])
            feed = rng.integers(0, DESIGN_VOCAB, (W + K + 8, B))
            at = [0]

            def decode():
                eng.step([(s, [int(t)]) for s, t in zip(slots, feed[at[0]])])
                at[0] += 1
            for _ in range(W):
                decode()
            torch.cuda.synchronize()
            a.record()
            for _ in range(K):
                decode()
            b.record()
            torch.cuda.synchronize()
            decode_ms = a.elapsed_time(b) / K
            decode_kinds, decode_span = _kernel_times(torch, decode)
            res[name] = {"prefill_tokens_per_s": round(T / prefill_ms * 1e3), "prefill_ms": round(prefill_ms, 3),
                         "decode_tokens_per_s": round(B / decode_ms * 1e3), "decode_ms_per_step": round(decode_ms, 4),
                         "prefill_kernels_us": prefill_kinds, "decode_kernels_us": decode_kinds,
                         "weight_bytes": eng.model.weight_bytes()}
            eng.close()
            del eng
            torch.cuda.empty_cache()

        # ---- distance from the roofline, kernel by kernel (us per launch over the us that its bytes or FLOPs take)
        def per_launch(kinds, *names):
            n = sum(kinds[k][0] for k in names if k in kinds)
            return sum(kinds[k][1] for k in names if k in kinds) / n if n else None

        def times(us, nbytes, flops):
            return round(us / (max(nbytes / hbm, flops / tensor) * 1e6), 2) if us else None
        f, l = res["fetorax"], res["llama"]
        qkv_bytes = lambda rows: rows * heads * 3 * dim * 2.0
        att_flops = 4.0 * heads * dim * T * (T + 1) / 2
        scan_flops = 4.0 * T * heads * dim * dim
        state = B * heads * dim * dim * 4.0 * 2
        kv_read = B * ctx * 2 * kv * dim * 2.0
        roof = {
            "prefill": {
                "llama attention": times(per_launch(l["prefill_kernels_us"], "attn_prefill_two", "attn_prefill_tc", "attn_prefill"),
                                         qkv_bytes(T), att_flops),
                "fetorax attention (with sink)": times(per_launch(f["prefill_kernels_us"], "attn_prefill_two", "attn_prefill_tc", "attn_prefill"),
                                                       qkv_bytes(T), att_flops),
                "fetorax recurrent scan": times(per_launch(f["prefill_kernels_us"], "linear_scan"),
                                                qkv_bytes(T) + T * heads * dim * 4.0, scan_flops),
            },
            "decode": {
                "llama attention": times(per_launch(l["decode_kernels_us"], "attn_decode"), kv_read, 0.0),
                "fetorax attention (with sink)": times(per_launch(f["decode_kernels_us"], "attn_decode"), kv_read, 0.0),
                "fetorax recurrent scan": times(per_launch(f["decode_kernels_us"], "linear_scan_single", "linear_scan"), state, 0.0),
            },
        }
        out[size] = {"fetorax": f, "llama": l, "times_the_roofline": roof,
                     "fetorax_over_llama": {"prefill": round(f["prefill_tokens_per_s"] / l["prefill_tokens_per_s"], 3),
                                            "decode": round(f["decode_tokens_per_s"] / l["decode_tokens_per_s"], 3)}}
    clocks = sampler.stop()
    print(json.dumps({"design": "fetorax", "beside": "llama", "dtype": "bf16", "data": "synthetic", "layers": 4,
                      "layer_order": "attention, retention, mlstm, attention on the first layer's keys and values",
                      "vocab": DESIGN_VOCAB, "prefill_tokens": T, "decode_batch": B, "decode_context": ctx, "steps": K,
                      "warmup": W, "peaks": peaks, "peaks_from": peaks_from, "clocks": clocks, "sizes": out}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--design", default="", choices=["", "fetorax", "zoporax", "raritar", "lavutar"],
                    help="instead of the default workload: this design beside the closest model the library has, at equal layer "
                         "sizes (prefill, decode, kernel by kernel): fetorax beside Llama, zoporax beside Fetorax, raritar beside Llama, lavutar beside Fetorax")
    ap.add_argument("--sizes", default="1b,8b", help="--design: layer sizes to run, of " + ", ".join(DESIGN_SIZES))
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=MODEL["num_hidden_layers"],
                    help="fewer layers than the model has (reported in config)")
    ap.add_argument("--no-points", action="store_true", help="only the headline: no other batches, models or tiny runs")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    if args.design:
        return design_bench(args)
    if args.gpus != 1:
        print(f"bench.py measures a one-GPU library: --gpus {args.gpus} is not supported, run it with --gpus 1")
        return 2
    K, W = args.steps, max(3, args.warmup)

    import numpy as np
    import torch

    from longbow_quarrel_b200.engine import Engine
    from longbow_quarrel_b200.sampling import SamplingParams

    peaks, peaks_from = load_peaks()
    cfg = dict(MODEL, num_hidden_layers=args.layers)
    L = args.layers
    max_batch = BATCH if args.no_points else 64
    engine = Engine.from_config(cfg, seed=0, dtype="bfloat16", max_tokens=max_batch * CONTEXT, max_batch=max_batch,
                                max_context=CONTEXT, gain_std=0.0)
    rng = np.random.default_rng(0)
    V = cfg["vocab_size"]
    greedy = SamplingParams(temperature=0.0)

    # ------------------------------------------------------------------ prefill of 2,048 tokens
    def prefill_once():
        slot = engine.new_sequence()
        toks = rng.integers(0, V, PREFILL_TOKENS).tolist()
        a, b = events(torch)
        torch.cuda.synchronize()
        a.record()
        engine.step([(slot, toks)])
        b.record()
        torch.cuda.synchronize()
        engine.end_sequence(slot)
        return a.elapsed_time(b)
    for _ in range(3):
        prefill_once()
    prefill_ms = statistics.median(prefill_once() for _ in range(5))
    pf_flops = prefill_flops(cfg, L, [PREFILL_TOKENS], 1)
    prefill = {"value": PREFILL_TOKENS / (prefill_ms / 1e3), "tokens": PREFILL_TOKENS, "ms": prefill_ms,
               "frac": pf_flops / (prefill_ms / 1e3) / (peaks["bf16_tflops"] * 1e12)}

    # ------------------------------------------------------------------ decode, timed on the device
    ms, mean_ctx, launches, clocks = decode_run(torch, engine, rng, V, BATCH, K, W, CONTEXT - (W + K + E2E_WARM), greedy,
                                                ClockSampler(), settle=E2E_WARM)
    ms_per_step = ms / K
    value = BATCH * K / (ms / 1e3)
    bytes_step = decode_bytes(cfg, L, BATCH, mean_ctx)
    achieved = bytes_step / (ms_per_step / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "peaks": peaks_from}

    # ------------------------------------------------------------------ end to end through generate()
    # K steps through the public entry point: host token ids in, one copy of the step's integers to the device and
    # one read of the sampled ids a step.  Timed on the host from the arrival of one step's tokens to that of the
    # K-th step after it.  The decode steps right after a long prompt step run at the reduced clocks that the
    # prompt step under the power cap leaves behind (about a dozen steps; reported below with the clock they ran
    # at), so this figure, like the device-timed one above, begins E2E_WARM + W steps after the prompt.
    W_dev, W = W, W + E2E_WARM
    prompt_len = CONTEXT - (W + K) - 1
    prompts = [rng.integers(0, V, prompt_len).tolist() for _ in range(BATCH)]
    engine.generate(prompts[:BATCH], max_new_tokens=3, sampling=greedy, stop_ids=[])       # warm-up
    fast = FastClocks()
    fast.start()
    _, t0, times = timed_generate(engine, prompts, W + K + 1, greedy, BATCH)
    fast.stop()
    from longbow_quarrel_b200.engine.step import pack_step
    flat_bytes = pack_step([(i, [0]) for i in range(BATCH)], None, [0] * BATCH, engine.stepper.needs)[0].nbytes   # a step's integers
    e2e_s = times[W + K] - times[W]
    # The first steps after a prompt step against the steady ones, each with the clock it ran at: if duration x
    # clock is the same, the longer first steps are the device's clocks coming back up, not the host.
    head = min(10, W)
    head_ms = (times[head] - times[0]) / head * 1e3
    steady_ms = e2e_s / K * 1e3
    head_mhz, steady_mhz = fast.median_between(times[0], times[head]), fast.median_between(times[W], times[W + K])
    e2e = {"value": BATCH * K / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": flat_bytes, "d2h_bytes_per_step": 4 * BATCH,
           "steps": K, "after_warmup_steps": W, "ms_per_step": steady_ms, "sm_mhz": steady_mhz,
           "first_steps_after_prompt": {"steps": head, "ms_per_step": head_ms, "sm_mhz": head_mhz},
           "from_first_token": {"value": BATCH * (W + K) / (times[W + K] - times[0]), "steps": W + K}}

    W = W_dev
    points = {}
    if not args.no_points:
        for b in (1, 64):
            k = max(16, K // 2)
            ms_b, ctx_b, _, _ = decode_run(torch, engine, rng, V, b, k, W, CONTEXT - (W + k + E2E_WARM), greedy, settle=E2E_WARM)
            points[f"decode_b{b}"] = b * k / (ms_b / 1e3)
            points[f"decode_b{b}_frac"] = decode_bytes(cfg, L, b, ctx_b) / (ms_b / k / 1e3) / 1e9 / peaks["hbm_gbs"]
    engine.close()
    del engine
    torch.cuda.empty_cache()
    if not args.no_points:
        # Llama-3.2-3B shape: 16 unequal prompts U[1, 2048], then 256 decode steps (greedy).
        lengths = [int(n) for n in np.random.default_rng(2).integers(1, 2049, 16)]
        points.update(other_workload(torch, np, peaks, "llama32_3b", MODEL_3B, lengths, 256, greedy, 0))
        # Llama-3.2-1B shape: batch 64, prompts of 128, 1,024 decode steps at temperature 1.
        points.update(other_workload(torch, np, peaks, "llama32_1b", MODEL_1B, [128] * 64, 1024,
                                     SamplingParams(temperature=1.0, seed=5), 256))
        points.update(tiny_workloads(torch))

    line = {
        "metric": "decode tokens/s, Llama-3.1-8B shape, batch 8, context 4096", "value": value, "unit": "tokens/s",
        "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random bf16 weights N(0, 0.02), uniform random token ids",
        "config": {"model": "Llama-3.1-8B shape", "global_batch": BATCH, "seq_len": CONTEXT, "parallelism": "single GPU",
                   "layers": L, "layers_of_model": MODEL["num_hidden_layers"], "hidden_size": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate_size": cfg["intermediate_size"],
                   "vocab_size": V, "rope_theta": cfg["rope_theta"], "rope_scaling": "llama3 factor 8 low 1 high 4 orig 8192",
                   "rms_norm_eps": cfg["rms_norm_eps"], "tied_embeddings": False,
                   "decode_context_mean": mean_ctx, "prefill_tokens": PREFILL_TOKENS, "settle_steps_after_prompt": E2E_WARM,
                   "l2": "every step reads 15 GB of weights, far more than L2; no flush"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "prefill": prefill, "roofline": roofline,
        "points": points, "impl": "ours",
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
