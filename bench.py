"""Throughput of the engine at Gemma 2 sizes with random weights, on one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--size 2b|9b|27b] [--layers L] [--impl reference]
    python bench.py --design fusitar|kofutar|teluzen|lokedra [--design-sizes s,m]      (another line: see `design_line`)

A "step" is one decode step. The default run has the layer sizes of the 2B configuration
(26 layers, hidden 2304, 8 heads over 4 kv heads of 256, intermediate 9216, vocabulary 256000,
window 4096 on even layers, page 16), a batch of 8 sequences that each hold 6,144 tokens of
history, bfloat16. It prints ONE JSON line:

  value        decoded tokens a second, timed on the device with CUDA events over K steps
  e2e          the same through the Python entry point (`Model.scheduler().step()`): every step
               copies its token ids and block tables from pinned host memory and reads the
               sampled tokens back
  prefill      one step of 2,048 prompt tokens: tokens a second, and flops / time / peak
  roofline     the decode step against the bytes it has to read (every weight once, and the
               cached keys and values the live requests see) at the measured copy bandwidth
  points       decode at batch 1 and 64; and, in the default run, the same figures at the 9B
               and 27B sizes ("9b_decode_b8", "27b_prefill", ...) and the 9B mixed workload
  sizes        the details behind the other sizes' points (ms, fractions of the peaks)
  logits       after the timed steps, one more decode step's logits for one request against
               the engine's own 32-bit path over the same weights and the same tokens: they must
               be finite and within the bfloat16 bound, or the run fails
  clocks       SM clocks sampled with nvidia-smi during the timed regions

The 9B mixed workload (`--size 9b --workload mixed`, and "9b_mixed" in the default run) is the
one Kapel's bench example runs (crates/kapel-cli/examples/bench.rs:125-203 with
crates/kapel-infer/src/batch.rs:20-88): prompts of seeded lengths uniform in 64..4096, 256
tokens decoded for each, through the scheduler with 2,048 tokens a pass.

Weights (5.2 GB and more) are larger than L2, so consecutive timed steps cannot reuse them from cache.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# size -> (the configuration's file under kapel_b200/config/presets, tokens of history a sequence holds)
SIZES = {"2b": ("gemma2-2b", 6144), "9b": ("gemma2-9b", 6144), "27b": ("gemma2-27b", 2048)}
CONTEXT = 8192
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
LOGITS_TOL = 2e-2              # bfloat16 against 32-bit through a whole model (the tests see 1e-2 at 26 layers)


def preset(size):
    with open(os.path.join(ROOT, "kapel_b200", "config", "presets", SIZES[size][0] + ".json")) as f:
        return json.load(f)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            raw = json.load(open(path))
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                    "bf16_tflops_sustained": float(raw.get("bf16_tflops_sustained", raw["bf16_tflops"])), "source": "measured"}
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons while `active`: one nvidia-smi process that prints a
    line every 50 ms, read by a thread."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index=0):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.active = False
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-i", str(index), "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _run(self):
        for line in self.proc.stdout:
            out = line.strip().split(",")
            if not self.active or len(out) < 6:
                continue
            try:
                self.samples.append(float(out[0]))
                self.max_mhz = float(out[1])
            except ValueError:
                continue
            for name, v in zip(self.NAMES, out[2:6]):
                if v.strip().lower().startswith("active"):
                    self.reasons.add(name)

    def close(self):
        if self.proc is not None:
            self.proc.terminate()                     # this object's own child, by its handle
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self._thread.join(timeout=2)

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def layer_windows(cfg, layers):
    """The window of each of the first `layers` layers (None: every key), as config.json says it:
    `layer_types` where given, else the even layers slide."""
    w, types = cfg.get("sliding_window"), cfg.get("layer_types")
    out = []
    for l in range(layers):
        slides = (types[l] == "sliding_attention") if types else (l % 2 == 0)
        out.append(w if (w and slides) else None)
    return out


def weight_bytes(cfg, layers):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    hq, hkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (hq + 2 * hkv) * d * h + hq * d * h + 3 * i * h + 4 * h
    return 2 * (layers * per_layer + v * h + h)


def kv_bytes_seen(cfg, layers, context):
    """Bytes of keys and values one sequence's decode step reads at `context` positions."""
    hkv, d = cfg["num_key_value_heads"], cfg["head_dim"]
    return sum((min(context, w) if w else context) * hkv * d * 2 * 2 for w in layer_windows(cfg, layers))


def prefill_flops(cfg, layers, tokens):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    hq, hkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (hq + 2 * hkv) * d * h + hq * d * h + 3 * i * h
    gemm = 2 * tokens * layers * per_layer + 2 * v * h            # the head runs on one row
    att = 0
    for win in layer_windows(cfg, layers):
        pairs = sum(min(c, win) if win else c for c in range(1, tokens + 1))
        att += 4 * pairs * hq * d
    return gemm + att


def breakdown(model, batch, tokens, history) -> int:
    """Where a step's time goes: each kernel entry point timed with CUDA events (every call
    synchronises, so the sums are device times, not a step time)."""
    import torch

    from kapel_b200 import kernels as K
    from kapel_b200.engine import StepEntry

    engine = model.engine
    engine.graphs = None                                  # eager steps only
    ids = [f"s{i}" for i in range(batch)]
    for s in ids:                                         # history in portions of 2,048
        for at in range(0, history, PREFILL_TOKENS):
            engine.step([StepEntry(s, tokens(min(PREFILL_TOKENS, history - at)), [])])
    engine.step([StepEntry("p", tokens(PREFILL_TOKENS), [PREFILL_TOKENS - 1])])
    engine.end("p")
    engine.step([StepEntry(s, tokens(1), [0]) for s in ids])
    torch.cuda.synchronize()
    K.enable_timing()
    engine.step([StepEntry("p", tokens(PREFILL_TOKENS), [PREFILL_TOKENS - 1])])
    engine.end("p")
    rows = K.timing_report()
    print(f"prefill of {PREFILL_TOKENS} tokens: {sum(r[3] for r in rows):.3f} ms in kernels")
    for name, shape, calls, ms in rows:
        print(f"  {ms:9.3f} ms  {calls:4d} x {name} {shape}")
    engine.step([StepEntry(s, tokens(1), [0]) for s in ids])
    rows = K.timing_report()
    print(f"decode step, batch {batch}, {history} tokens of history: {sum(r[3] for r in rows):.3f} ms in kernels")
    for name, shape, calls, ms in rows:
        print(f"  {ms:9.3f} ms  {calls:4d} x {name} {shape}")
    K.disable_timing()
    return 0


class Bench:
    """One model of one size and what is measured on it."""

    def __init__(self, size, layers, batches, steps, warmup, clocks, pk, seed=0):
        import numpy as np
        import torch

        from kapel_b200.model import Model

        self.torch = torch
        self.size = size
        base = preset(size)
        self.history = SIZES[size][1]
        self.full_layers = base["num_hidden_layers"]
        self.layers = layers or self.full_layers
        self.cfg = dict(base, num_hidden_layers=self.layers)
        self.batches, self.steps, self.warmup, self.clocks, self.pk, self.seed = batches, steps, warmup, clocks, pk, seed
        room = max(batches) * (-(-(self.history + 4 * (warmup + steps) + 64) // 64) * 64) + PREFILL_TOKENS + 64
        self.model = Model.random(self.cfg, seed=seed, dtype="bf16", max_tokens_cached=room, max_sequences=max(batches) + 1)
        self.engine = self.model.engine
        self.rng = np.random.default_rng(0)
        self.vocab = self.cfg["vocab_size"]

    def tokens(self, n):
        return [int(t) for t in self.rng.integers(1000, self.vocab - 1000, size=n)]

    def timed(self, fn, n):
        torch = self.torch
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.clocks.active = True
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        self.clocks.active = False
        return a.elapsed_time(b) / n

    def prefill(self):
        from kapel_b200.engine import StepEntry

        def once():
            self.engine.step([StepEntry("p", self.tokens(PREFILL_TOKENS), [PREFILL_TOKENS - 1])])
            self.engine.end("p")

        for _ in range(2):
            once()
        ms = min(self.timed(once, 1) for _ in range(3))
        flops = prefill_flops(self.cfg, self.layers, PREFILL_TOKENS)
        pg = getattr(self.engine, "prompt_graphs", None)
        return {"value": PREFILL_TOKENS / ms * 1e3, "tokens": PREFILL_TOKENS, "ms": ms,
                "frac": flops / (ms * 1e-3) / (self.pk["bf16_tflops"] * 1e12),
                "recorded": bool(pg is not None and pg.replays > 0)}      # the pass's shape was seen before: the engine replays its recording

    def decode_point(self, batch, check_logits=False):
        """dict: device ms a step, e2e ms a step, launches a step, h2d and d2h bytes a step, hbm fraction."""
        from kapel_b200 import kernels as K
        from kapel_b200.engine import StepEntry
        from kapel_b200.engine.scheduler import Request
        from kapel_b200.sampling import Sampling

        torch, engine, steps = self.torch, self.engine, self.steps
        sched = self.model.scheduler(max_pass_tokens=PREFILL_TOKENS, max_sequences=batch)
        rids = [sched.add(Request(prompt=self.tokens(self.history), sampling=Sampling(), max_tokens=10 ** 6, ignore_eos=True))
                for _ in range(batch)]
        while any(sched._pending(r) > 1 for r in rids):       # prompts in portions until every request decodes
            sched.step()
        for _ in range(self.warmup):
            sched.step()
        torch.cuda.synchronize()
        self.clocks.active = True
        t0 = time.perf_counter()
        for _ in range(steps):
            events = sched.step()
            assert len(events) == batch
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) / steps * 1e3
        self.clocks.active = False
        h2d = engine.last_h2d_bytes
        sched.settle()              # the pass enqueued ahead of the host is read: the cache is one token behind each sequence again
        # The same step on the device clock, fed from the step function directly. Nothing is waited
        # for between steps: the staging buffers of a recorded step are guarded by events, so each
        # step runs on its own inputs and the host is at most two steps ahead.
        fed = {r: list(sched.entries[r].sequence) for r in rids}          # fed[r][:-1] is in the cache; the last is fed next

        def one():
            engine.step([StepEntry(r, [fed[r][-1]], [0]) for r in rids])
            for r in rids:
                fed[r].append(fed[r][-1])

        one()
        launches_before = K.launch_count() + (engine.graphs.replayed_kernels if engine.graphs else 0)
        dev_ms = self.timed(one, steps)
        launches = K.launch_count() + (engine.graphs.replayed_kernels if engine.graphs else 0) - launches_before
        context = len(fed[rids[0]]) - 1
        step_bytes = weight_bytes(self.cfg, self.layers) + batch * kv_bytes_seen(self.cfg, self.layers, context)
        achieved = step_bytes / (dev_ms * 1e-3) / 1e9
        out = {"ms": dev_ms, "e2e_ms": e2e_ms, "launches": launches / steps, "h2d": h2d, "d2h": batch * 4, "tok_s": batch / dev_ms * 1e3,
               "bytes": step_bytes, "gbs": achieved, "frac": achieved / self.pk["hbm_gbs"], "context": context}
        if check_logits:
            logits = engine.step([StepEntry(r, [fed[r][-1]], [0]) for r in rids]).clone()
            torch.cuda.synchronize()
            out["logits_row"] = logits[0].cpu()
            out["logits_tokens"] = list(fed[rids[0]])          # the tokens fed to request 0, the last one at the checked place
            out["logits_finite"] = bool(torch.isfinite(logits).all())
        for r in rids:
            sched.cancel(r)
        K.check_async_errors()
        return out

    def check_against_32_bit(self, tokens_fed, row):
        """The bfloat16 logits `row` (of the last of `tokens_fed`) against the engine's 32-bit path over
        the same weights (the same seed gives the same values; the 32-bit path widens them)."""
        from kapel_b200.engine import Engine, StepEntry

        torch = self.torch
        engine = Engine.random(self.cfg, seed=self.seed, dtype="float32", max_tokens=len(tokens_fed) + 64, max_sequences=2)
        logits = None
        for at in range(0, len(tokens_fed), PREFILL_TOKENS):
            part = tokens_fed[at : at + PREFILL_TOKENS]
            last = at + len(part) == len(tokens_fed)
            logits = engine.step([StepEntry("check", part, [len(part) - 1] if last else [])])
        want = logits[0].cpu().double()
        engine.end("check")
        del engine
        gc.collect()
        torch.cuda.empty_cache()
        got = row.double()
        err = float((got - want).abs().max() / want.abs().max())
        return {"rel_err": err, "tol": LOGITS_TOL, "finite": bool(torch.isfinite(got).all()), "positions": len(tokens_fed),
                "same_argmax": bool(int(got.argmax()) == int(want.argmax())), "against": "the engine's float32 path, same weights and tokens"}

    def mixed(self, running, requests, decode=256, lo=64, hi=4096):
        """Kapel's mixed workload: `requests` prompts of seeded lengths uniform in lo..hi, `decode` tokens
        each, at most `running` at once, 2,048 tokens a pass, through the scheduler, host tokens in and out."""
        import numpy as np

        from kapel_b200.engine.scheduler import Request
        from kapel_b200.sampling import Sampling

        torch = self.torch
        rng = np.random.default_rng(7)
        lengths = [int(n) for n in rng.integers(lo, hi + 1, size=requests)]
        sched = self.model.scheduler(max_pass_tokens=PREFILL_TOKENS, max_sequences=running)
        for n in lengths:
            sched.add(Request(prompt=self.tokens(n), sampling=Sampling(), max_tokens=decode, ignore_eos=True))
        weights = weight_bytes(self.cfg, self.layers)
        torch.cuda.synchronize()
        self.clocks.active = True
        t0 = time.perf_counter()
        generated = passes = 0
        must_read = 0
        while sched.has_work():
            events = sched.step()
            passes += 1
            generated += sum(1 for e in events if e.token is not None)
            assert not any(e.finish == "error" for e in events), [e.error for e in events if e.finish == "error"]
            # what the pass had to read: every weight once, and the keys and values each running request sees
            must_read += weights + sum(kv_bytes_seen(self.cfg, self.layers, sched._cached(r)) for r in sched.running)
        torch.cuda.synchronize()
        seconds = time.perf_counter() - t0
        self.clocks.active = False
        st = sched.stats()
        return {"tok_s": generated / seconds, "all_tok_s": (generated + sum(lengths)) / seconds, "seconds": seconds, "requests": requests,
                "running": running, "prompt_tokens": sum(lengths), "generated": generated, "passes": passes, "preemptions": st.preemptions,
                "recorded_passes": st.recorded_passes, "gbs": must_read / seconds / 1e9, "frac": must_read / seconds / 1e9 / self.pk["hbm_gbs"]}

    def close(self):
        self.model = self.engine = None
        gc.collect()
        self.torch.cuda.empty_cache()


# ---------------------------------------------------------------------------------------------
# --design fusitar: the Fusitar design (attention with kept first keys and a gate, mLSTM, mixture
# of experts) beside Gemma 2 at equal sizes: the same width, heads, head size, window, vocabulary,
# as many layers, and as much feed-forward a token (top x expert size = Gemma's intermediate size).
DESIGN_SIZES = {
    # name: width, heads, kv heads, head size, window, first keys kept, experts, top, groups, kept groups, expert size, vocab, layers
    "s": dict(width=2048, heads=16, kv_heads=4, dim=128, window=1024, keep=4, experts=16, top=4, groups=4, keep_groups=2, ff=1024, vocab=32768, layers=4),
    "m": dict(width=4096, heads=32, kv_heads=8, dim=128, window=2048, keep=4, experts=32, top=4, groups=8, keep_groups=4, ff=2048, vocab=32768, layers=4),
}
DESIGN_HISTORY = 3072
DESIGN_BATCH = 8


def fusitar_config(z):
    moe = {"kind": "moe", "expert": {"ff": z["ff"]},
           "router": {"experts": z["experts"], "top": z["top"], "groups": {"count": z["groups"], "keep": z["keep_groups"]}}}
    att = {"type": "attention", "mlp": moe, "mixer": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"],
                                                        "scale": z["dim"] ** -0.5, "mask": {"size": z["window"], "keep_first": z["keep"]}}}
    rec = {"type": "mlstm", "mlp": moe, "mixer": {"heads": z["heads"], "dim": z["dim"], "vdim": z["dim"], "gate_cap": 15.0}}
    return {"architecture": "Fusitar", "vocab": z["vocab"], "width": z["width"], "embedding": {"scale": z["width"] ** 0.5},
            "norm": {"eps": 1e-6}, "layers": [att if i % 2 == 0 else rec for i in range(z["layers"])]}


# --design kofutar: the Kofutar design (attention with per-head norms, attention through latents with a sink,
# the gated delta rule, a dense gated feed-forward, layer norms) beside Fusitar, the engine's other design with
# recurrent and attending layers, and Gemma 2, whose dense feed-forward it shares, at equal sizes: the same width,
# heads, head size, vocabulary, as many layers, Gemma's intermediate size. Its layers take turns: attention, delta,
# latent attention, delta; the loop covers them all once (so the input mix runs). The latents have the sizes usual
# for such layers: three quarters of the width for the queries, 512 + 64 rotated for keys and values.
def kofutar_config(z):
    mlp = {"kind": "dense", "ff": z["top"] * z["ff"]}
    att = {"type": "attention", "mlp": mlp, "mixer": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"],
                                                        "scale": z["dim"] ** -0.5, "rot": {"base": 10000.0, "dims": z["dim"]}}}
    lat = {"type": "latent_attention", "mlp": mlp,
           "mixer": {"heads": z["heads"], "dim": z["dim"], "rot_dim": 64, "vdim": z["dim"], "q_rank": z["width"] * 3 // 4, "kv_rank": KOFUTAR_KV_RANK,
                     "scale": (z["dim"] + 64) ** -0.5, "rot": {"base": 10000.0, "dims": 64}}}
    rec = {"type": "delta", "mlp": mlp, "mixer": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"], "conv": 4}}
    return {"architecture": "Kofutar", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5},
            "loop": {"start": 0, "stop": z["layers"], "times": 1}, "layers": [(att, rec, lat, rec)[i % 4] for i in range(z["layers"])]}


KOFUTAR_KV_RANK = 512


# --design teluzen: the Teluzen design (attention over a window plus pooled blocks below it, biases, norms over the
# whole projections, scaled rotation of neighbours, a number a head, mixed heads' weights, values mixed with the first
# layer's; a plain feed-forward in the first layer and gated experts with a shared expert in the others; learned
# positions) beside Fusitar, the engine's other design with windowed attention and experts, and Gemma 2, at equal
# sizes: the same width, heads, head size, window, vocabulary, as many layers, and as much feed-forward a token
# (top - 1 chosen experts and the shared one of the expert's size; the first layer's plain one of Gemma's size).
TELUZEN_POOL = 16
TELUZEN_POSITIONS = 8192


def teluzen_config(z):
    rot = {"base": 10000.0, "dims": z["dim"] // 2, "scaling": {"factor": 8.0, "original": 1024, "fast": 32.0, "slow": 1.0}}
    mixer = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"], "scale": z["dim"] ** -0.5,
             "mask": {"size": z["window"], "pool": TELUZEN_POOL}, "rot": rot, "v_mix": True}
    moe = {"kind": "moe", "expert": {"ff": z["ff"]}, "router": {"experts": z["experts"], "top": z["top"] - 1}, "shared": {"ff": z["ff"]}}
    dense = {"kind": "dense", "ff": z["top"] * z["ff"]}
    return {"architecture": "Teluzen", "vocab": z["vocab"], "width": z["width"], "max_positions": TELUZEN_POSITIONS, "norm": {"eps": 1e-6},
            "layers": [{"type": "attention", "mixer": mixer, "mlp": dense if i == 0 else moe} for i in range(z["layers"])]}


# --design lokedra: the Lokedra design (parallel blocks with a token shift; the generalized delta rule; chunked attention
# behind short convolutions whose values are its keys, with 1 in the denominator, beside linear attention behind a forget
# gate; attention through latents with stretched rotation; bounded gated experts) beside Kofutar, the engine's other design
# with a delta rule and latent attention, and Fusitar, its other design with masked attention on the same kernels and
# experts, at equal sizes: the same width, heads, head size, vocabulary, as many layers, experts of the same size. Its
# layers take turns: parallel, delta, latent attention, delta; chunks as long as the others' window; latents as Kofutar's.
LOKEDRA_LORA = 64


def lokedra_config(z):
    moe = {"kind": "moe", "expert": {"ff": z["ff"], "limit": 7.0}, "router": {"experts": z["experts"], "top": z["top"]}}
    par = {"type": "parallel", "mlp": moe, "mixer": {
        "left": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"], "conv": 4, "scale": z["dim"] ** -0.5,
                 "mask": {"size": z["window"]}},
        "right": {"heads": z["heads"], "dim": z["dim"], "vdim": z["dim"]}, "left_scale": 1.0, "right_scale": 1.0}}
    rec = {"type": "general_delta", "mlp": moe, "mixer": {"heads": z["heads"], "dim": z["dim"], "lora": LOKEDRA_LORA}}
    lat = {"type": "latent_attention", "mlp": moe,
           "mixer": {"heads": z["heads"], "dim": z["dim"], "rot_dim": 64, "vdim": z["dim"], "q_rank": z["width"] * 3 // 4, "kv_rank": KOFUTAR_KV_RANK,
                     "scale": (z["dim"] + 64) ** -0.5,
                     "rot": {"base": 10000.0, "dims": 64, "scaling": {"factor": 8.0, "original": 1024, "fast": 32.0, "slow": 1.0}}}}
    return {"architecture": "Lokedra", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6}, "embedding": {"scale": z["width"] ** 0.5},
            "layers": [(par, rec, lat, rec)[i % 4] for i in range(z["layers"])]}


def gemma_config(z):
    return {"architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2", "num_hidden_layers": z["layers"], "hidden_size": z["width"],
            "num_attention_heads": z["heads"], "num_key_value_heads": z["kv_heads"], "head_dim": z["dim"],
            "intermediate_size": z["top"] * z["ff"], "vocab_size": z["vocab"], "sliding_window": z["window"],
            "layer_types": ["sliding_attention"] * z["layers"], "query_pre_attn_scalar": z["dim"], "attn_logit_softcapping": 50.0,
            "final_logit_softcapping": 30.0, "rms_norm_eps": 1e-6, "hidden_activation": "gelu_pytorch_tanh", "tie_word_embeddings": True}


def design_kernel_rooflines(which, z, kind, rows, context, batch, pk):
    """{kernel entry point: (what it must do, in flops or bytes)} for one pass: `kind` "prefill" (rows
    tokens of one request from position 0) or "decode" (batch requests of `context` positions)."""
    w, hq, hkv, d, win = z["width"], z["heads"], z["kv_heads"], z["dim"], z["window"]
    layers = z["layers"]
    if which == "teluzen":
        # a query that has seen c positions reads min(c, window) tokens and the blocks wholly below its window; scores,
        # the mix of the heads' weights (hq x hq a key) and the values; the blocks' means are 32-bit in the state
        seen = lambda c: min(c, win) + (max(0, c - win) // TELUZEN_POOL)
        moe_layers = layers - 1
        if kind == "prefill":
            pairs = sum(seen(c) for c in range(1, rows + 1))
            return {"attention": ("flops", layers * 2.0 * pairs * hq * (2 * d + hq)),
                    "feed_forward": ("flops", 2.0 * rows * 2 * z["top"] * z["ff"] * w + moe_layers * 2.0 * rows * 3 * z["top"] * z["ff"] * w)}
        experts_read = min(z["experts"], batch * (z["top"] - 1)) + 1
        return {"attention": ("bytes", layers * batch * (min(context, win) * hkv * 2 * d * 2.0 + (max(0, context - win) // TELUZEN_POOL) * hkv * 2 * d * 4.0)),
                "feed_forward": ("bytes", 2.0 * z["top"] * z["ff"] * w * 2 + moe_layers * experts_read * 3.0 * z["ff"] * w * 2)}
    if which == "lokedra":
        par_layers, lat_layers, rec_layers = (layers + 3) // 4, (layers + 1) // 4, layers // 2
        r, kv = 64, KOFUTAR_KV_RANK
        in_chunk = lambda c: (c - 1) % win + 1              # keys a query that has seen c positions reads: its chunk's so far
        if kind == "prefill":
            pairs = rows * (rows + 1) // 2
            # the memories a row and head: the generalized delta rule decays, removes along the unit key and writes (5 a value of
            # the [d, d] memory) and reads twice (4); the forget gate's memory decays and writes (3) and reads once (2)
            return {"attention": ("flops", par_layers * 4.0 * sum(in_chunk(c) for c in range(1, rows + 1)) * hq * d),
                    "latent_attention": ("flops", lat_layers * 2.0 * pairs * hq * (2 * d + r)),
                    "feed_forward": ("flops", layers * 2.0 * rows * 3 * z["top"] * z["ff"] * w),
                    "decay_scan": ("flops", (rec_layers * 9.0 + par_layers * 5.0) * rows * hq * d * d)}
        experts_read = min(z["experts"], batch * z["top"])
        return {"attention": ("bytes", par_layers * batch * in_chunk(context) * hkv * d * 2.0),          # a key is also the value: one line a position
                "latent_attention": ("bytes", lat_layers * batch * context * (kv + r) * 2.0),
                "feed_forward": ("bytes", layers * experts_read * 3.0 * z["ff"] * w * 2),
                "decay_scan": ("bytes", (rec_layers + par_layers) * batch * hq * d * d * 4 * 2.0)}
    if which == "kofutar":
        att_layers, lat_layers, rec_layers = (layers + 3) // 4, (layers + 1) // 4, layers // 2
        r, kv, ff = 64, KOFUTAR_KV_RANK, z["top"] * z["ff"]
        if kind == "prefill":
            pairs = rows * (rows + 1) // 2
            # the latent layers by what the design asks for (a head's own keys of d + r and values of d), not by the
            # longer lines the kernel walks; the delta rule: decay, two read-outs and the update of a [d, d] memory a row and head
            return {"attention": ("flops", att_layers * 4.0 * pairs * hq * d), "latent_attention": ("flops", lat_layers * 2.0 * pairs * hq * (2 * d + r)),
                    "feed_forward": ("flops", layers * 2.0 * rows * 3 * ff * w), "delta_scan": ("flops", rec_layers * 7.0 * rows * hq * d * d)}
        return {"attention": ("bytes", att_layers * batch * context * hkv * d * 2 * 2.0), "latent_attention": ("bytes", lat_layers * batch * context * (kv + r) * 2.0),
                "feed_forward": ("bytes", layers * 3.0 * ff * w * 2), "delta_scan": ("bytes", rec_layers * batch * hq * d * d * 4 * 2.0)}
    att_layers = layers if which == "gemma2" else (layers + 1) // 2
    rec_layers = 0 if which == "gemma2" else layers // 2
    out = {}
    if kind == "prefill":
        pairs = sum(min(c, win) for c in range(1, rows + 1))
        out["attention"] = ("flops", att_layers * 4.0 * pairs * hq * d)
        out["feed_forward"] = ("flops", layers * 2.0 * rows * 3 * z["top"] * z["ff"] * w if which == "gemma2" else layers * 2.0 * rows * 2 * z["top"] * z["ff"] * w)
        out["mlstm_scan"] = ("flops", rec_layers * 4.0 * rows * hq * d * d)
    else:
        out["attention"] = ("bytes", att_layers * batch * min(context, win) * hkv * d * 2 * 2.0)
        experts_read = min(z["experts"], batch * z["top"])
        out["feed_forward"] = ("bytes", layers * 3.0 * z["top"] * z["ff"] * w * 2 if which == "gemma2" else layers * experts_read * 2.0 * z["ff"] * w * 2)
        out["mlstm_scan"] = ("bytes", rec_layers * batch * hq * d * d * 4 * 2.0)
    return out


# Which timed entry points make up a like kernel of the two designs.
KERNEL_CLASSES = {
    "attention": ("paged_attention_rows", "paged_attention_mma", "paged_attention_decode_fused"),
    "feed_forward": ("moe_grouped", "gemm_glu_fused", "glu", "gemm:ffn"),
    "mlstm_scan": ("mlstm_scan",),
}
# Kofutar's attention layers run the tensor-core kernels; the row-wise kernel is its latent layers', with the products a head around it.
KOFUTAR_KERNEL_CLASSES = {
    "attention": ("paged_attention_mma", "paged_attention_decode_fused"),
    "latent_attention": ("paged_attention_rows", "latent_attention_mma", "head_linear"),
    "feed_forward": ("gemm_glu_fused", "glu"),
    "delta_scan": ("delta_scan",),
}
# Teluzen's attention is the kernel over window and blocks (the means of the blocks a step completes included); its
# feed-forwards are the grouped products with the gated unit between them, the shared expert's fused product, the plain
# layer's activation, and the plain products whose inner width is an expert's or the plain layer's size.
TELUZEN_KERNEL_CLASSES = {
    "attention": ("pooled_attention", "pooled_attention_mma", "pool_blocks"),
    "feed_forward": ("moe_grouped", "gemm_glu_fused", "glu", "act"),
}


# Lokedra's chunked attention runs the row-wise kernel (single tokens) and the mma.sync prompt kernel with the block mask, as
# Fusitar's attention does; its latent layers the kernel over shared lines with the products a head around it; its experts
# the grouped products with the bounded gated unit between them; its two memories the decay scan behind their own inputs' kernels.
LOKEDRA_KERNEL_CLASSES = {
    "attention": ("paged_attention_rows", "paged_attention_mma"),
    "latent_attention": ("latent_attention_mma", "head_linear"),
    "feed_forward": ("moe_grouped", "glu_clamped"),
    "decay_scan": ("gdelta_scan", "gate_scan"),
}


def design_point(which, z, steps, warmup, clocks, pk):
    """Prefill of 2,048 tokens and decode at batch 8 for one design at one size: tokens a second through
    the engine (recorded passes), and the device time of each kernel entry point in one eager pass."""
    import numpy as np
    import torch

    from kapel_b200 import kernels as K
    from kapel_b200.engine import Engine, StepEntry

    cfg = {"fusitar": fusitar_config, "kofutar": kofutar_config, "gemma2": gemma_config, "teluzen": teluzen_config, "lokedra": lokedra_config}[which](z)
    room = (DESIGN_BATCH + 1) * (DESIGN_HISTORY + 4 * (steps + warmup) + 128) + PREFILL_TOKENS
    engine = Engine.random(cfg, seed=0, dtype="bfloat16", max_tokens=room, max_sequences=DESIGN_BATCH + 2)
    rng = np.random.default_rng(0)
    tokens = lambda n: [int(t) for t in rng.integers(0, z["vocab"], size=n)]

    def timed(fn, n):
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        clocks.active = True
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        clocks.active = False
        return a.elapsed_time(b) / n

    def prefill_once():
        engine.step([StepEntry("p", tokens(PREFILL_TOKENS), [PREFILL_TOKENS - 1])])
        engine.end("p")

    for _ in range(3):
        prefill_once()
    prefill_ms = min(timed(prefill_once, 1) for _ in range(3))
    ids = [f"s{i}" for i in range(DESIGN_BATCH)]
    for sid in ids:
        for at in range(0, DESIGN_HISTORY, PREFILL_TOKENS):
            engine.step([StepEntry(sid, tokens(min(PREFILL_TOKENS, DESIGN_HISTORY - at)), [])])
    decode_once = lambda: engine.step([StepEntry(sid, tokens(1), [0]) for sid in ids])
    for _ in range(warmup):
        decode_once()
    decode_ms = timed(decode_once, steps)
    # one eager pass of each kind with every entry point between two events
    engine.graphs = engine.prompt_graphs = None
    K.enable_timing()
    per_kernel = {}
    for kind, fn in (("prefill", prefill_once), ("decode", decode_once)):
        fn()
        K.timing_report()
        fn()
        rows = K.timing_report()
        must = design_kernel_rooflines(which, z, kind, PREFILL_TOKENS, DESIGN_HISTORY, DESIGN_BATCH, pk)
        classes = {}
        for name, shape, calls, ms in rows:
            for cls, members in {"kofutar": KOFUTAR_KERNEL_CLASSES, "teluzen": TELUZEN_KERNEL_CLASSES, "lokedra": LOKEDRA_KERNEL_CLASSES}.get(which, KERNEL_CLASSES).items():
                if name in members:
                    classes[cls] = classes.get(cls, 0.0) + ms
        if which in ("gemma2", "kofutar"):   # the dense way down is a plain product: count the products whose inner width is the intermediate size
            # (Kofutar's input mix has the same shape where the intermediate size is twice the width: one call more than the layers', taken off by its share)
            classes["feed_forward"] = classes.get("feed_forward", 0.0) + sum(
                ms * (z["layers"] / calls if (which == "kofutar" and calls == z["layers"] + 1) else 1.0)
                for name, shape, calls, ms in rows if name == "gemm" and len(shape) == 2 and shape[0] == z["width"] and shape[1] == z["top"] * z["ff"])
        if which == "teluzen":             # the ways down of the plain layer and of the shared expert
            classes["feed_forward"] = classes.get("feed_forward", 0.0) + sum(
                ms for name, shape, calls, ms in rows if name == "gemm" and len(shape) == 2 and shape[0] == z["width"] and shape[1] in (z["ff"], z["top"] * z["ff"]))
        rec = {"kernels": [{"name": n, "shape": list(sh), "calls": c, "ms": round(ms, 4)} for n, sh, c, ms in rows][:14], "classes": {}}
        for cls, ms in classes.items():
            unit, amount = must[cls]
            if amount <= 0 or ms <= 0:
                continue
            peak = pk["bf16_tflops"] * 1e12 if unit == "flops" else pk["hbm_gbs"] * 1e9
            rec["classes"][cls] = {"ms": round(ms, 4), "bound": unit, "frac_of_measured_peak": amount / (ms * 1e-3) / peak}
        per_kernel[kind] = rec
    K.disable_timing()
    K.check_async_errors()
    out = {"prefill_tok_s": PREFILL_TOKENS / prefill_ms * 1e3, "prefill_ms": prefill_ms, "decode_tok_s": DESIGN_BATCH / decode_ms * 1e3,
           "decode_ms": decode_ms, "batch": DESIGN_BATCH, "history": DESIGN_HISTORY, "by_kernel": per_kernel}
    del engine
    gc.collect()
    torch.cuda.empty_cache()
    return out


def design_line(args) -> int:
    import torch

    torch.cuda.set_device(0)
    pk = peaks()
    clocks = ClockSampler()
    sizes = {}
    for name in args.design_sizes.split(","):
        z = DESIGN_SIZES[name]
        beside = ("gemma2",) if args.design == "fusitar" else (("kofutar", "fusitar") if args.design == "lokedra" else ("fusitar", "gemma2"))
        if args.design_beside is not None:
            beside = tuple(b for b in args.design_beside.split(",") if b)
        sizes[name] = {"shape": z}
        for which in (args.design,) + beside:
            sizes[name][which] = design_point(which, z, min(args.steps, 50), max(3, args.warmup), clocks, pk)
    clocks.close()
    first = sizes[args.design_sizes.split(",")[0]]
    print(json.dumps({
        "metric": f"decode tok/s at batch {DESIGN_BATCH} ({args.design.capitalize()}, size {args.design_sizes.split(',')[0]}, bf16, {DESIGN_HISTORY} tokens of history per sequence)",
        "value": first[args.design]["decode_tok_s"], "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True, "dtype": "bf16",
        "data": "synthetic: seeded random weights and uniform-random token ids", "design": args.design, "beside": " and ".join(beside) + " at equal sizes",
        "config": {"peaks": pk["source"], "prefill_tokens": PREFILL_TOKENS}, "sizes": sizes, "clocks": clocks.summary(), "impl": "ours"}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", default="2b", choices=sorted(SIZES), help="layer sizes: Gemma 2 2B (the default and the contract's line), 9B or 27B")
    ap.add_argument("--workload", default="fixed", choices=["fixed", "mixed"],
                    help="fixed: decode at a fixed history and a 2,048-token prefill; mixed: prompts of 64..4096 and 256 decoded tokens each through the scheduler")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--skip-points", action="store_true", help="leave out decode at batch 1 and 64 and the other sizes")
    ap.add_argument("--skip-sizes", action="store_true", help="leave out the 9B and 27B points of the default run")
    ap.add_argument("--skip-check", action="store_true", help="leave out the check of the timed logits against the 32-bit path")
    ap.add_argument("--breakdown", action="store_true",
                    help="instead of the JSON line: device time by kernel for one prefill step and one eager decode step")
    ap.add_argument("--design", default=None, choices=["fusitar", "kofutar", "teluzen", "lokedra"],
                    help="instead of the default line: this design beside Gemma 2 (kofutar and teluzen: beside Fusitar and Gemma 2; lokedra: beside Kofutar and Fusitar) at equal sizes, prefill and decode, with each like kernel's roofline fraction")
    ap.add_argument("--design-beside", default=None, help="which other designs run beside it (comma separated; empty: none); default: the closest ones")
    ap.add_argument("--design-sizes", default="s,m", help="which of the design sizes (s, m), comma separated")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "smallbard/kapel is a Rust workspace; this image has no cargo/rustc and no network, so it cannot be built or installed offline"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.design is not None:
        return design_line(args)
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)

    import torch

    torch.cuda.set_device(0)
    pk = peaks()
    clocks = ClockSampler()
    batches = [args.batch] if args.skip_points else sorted({1, args.batch, 64})
    bench = Bench(args.size, args.layers, batches, steps, warmup, clocks, pk)
    cfg, history = bench.cfg, bench.history

    if args.breakdown:
        return breakdown(bench.model, args.batch, bench.tokens, history)

    if args.workload == "mixed":
        res = {f"running_{r}": bench.mixed(r, n) for r, n in ((8, 16), (64, 96))}
        clocks.close()
        main_res = res["running_64"]
        print(json.dumps({
            "metric": f"generated tok/s, mixed workload (Gemma 2 {args.size.upper()} sizes, bf16, prompts 64..4096, 256 decoded each, 64 running)",
            "value": main_res["tok_s"], "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic: seeded random weights, seeded prompt lengths and uniform-random token ids",
            "config": {"model": f"gemma2-{args.size}-shape", "layers": bench.layers, "layers_of_config": bench.full_layers, "max_pass_tokens": PREFILL_TOKENS,
                       "requests": main_res["requests"], "running": 64, "decode": 256, "peaks": pk["source"]},
            "mixed": res, "clocks": clocks.summary(), "impl": "ours"}))
        return 0

    prefill = bench.prefill()
    results = {b: bench.decode_point(b, check_logits=(b == args.batch and not args.skip_check)) for b in batches}
    main_res = results[args.batch]
    check = None
    if not args.skip_check:
        row, fed = main_res.pop("logits_row"), main_res.pop("logits_tokens")
        bench.close()                                        # the 32-bit weights need the room at the larger sizes
        check = bench.check_against_32_bit(fed, row)
    else:
        bench.close()

    points = {f"decode_b{b}": results[b]["tok_s"] for b in batches if b != args.batch}
    sizes = {}
    if args.size == "2b" and not args.skip_points and not args.skip_sizes:
        for other in ("9b", "27b"):
            try:
                ob = Bench(other, 0, [1, 8, 64], min(steps, 30), warmup, clocks, pk)
                rec = {"layers": ob.layers, "history": ob.history, "prefill": ob.prefill()}
                for b in (1, 8, 64):
                    r = ob.decode_point(b)
                    rec[f"decode_b{b}"] = {k: r[k] for k in ("tok_s", "ms", "e2e_ms", "frac", "gbs")}
                    points[f"{other}_decode_b{b}"] = r["tok_s"]
                points[f"{other}_prefill"] = rec["prefill"]["value"]
                if other == "9b":
                    rec["mixed"] = ob.mixed(64, 96)
                    points["9b_mixed"] = rec["mixed"]["tok_s"]
                sizes[other] = rec
                ob.close()
            except Exception as e:                          # the contract's line must not be lost to another size
                sizes[other] = {"error": f"{type(e).__name__}: {e}"}
    clocks.close()

    line = {
        "metric": f"decode tok/s at batch {args.batch} (Gemma 2 {args.size.upper()} sizes, bf16, {history} tokens of history per sequence)",
        "value": main_res["tok_s"],
        "unit": "tokens/s",
        "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": main_res["ms"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights and uniform-random token ids",
        "config": {
            "model": f"gemma2-{args.size}-shape", "global_batch": args.batch, "seq_len": CONTEXT, "history": history, "parallelism": "single-gpu",
            "layers": bench.layers, "layers_of_config": bench.full_layers, "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
            "vocab": cfg["vocab_size"], "window": cfg["sliding_window"], "page": 16,
            "l2": f"inputs larger than L2 ({weight_bytes(cfg, bench.layers) / 1e9:.1f} GB of weights a step)", "peaks": pk["source"],
        },
        "e2e": {"value": args.batch / main_res["e2e_ms"] * 1e3, "unit": "tokens/s", "ms_per_step": main_res["e2e_ms"],
                "h2d_bytes_per_step": main_res["h2d"], "d2h_bytes_per_step": main_res["d2h"]},
        "gpu_launches": int(round(main_res["launches"] * steps)),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": main_res["gbs"], "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": main_res["frac"],
                     "bytes": main_res["bytes"]},
        "points": points,
        "logits": check,
        "sizes": sizes,
        "clocks": clocks.summary(),
        "impl": "ours",
    }
    print(json.dumps(line))
    if check is not None and not (check["finite"] and check["rel_err"] <= check["tol"]):
        print(f"bench.py: the timed logits differ from the 32-bit path by {check['rel_err']:.3e} (bound {check['tol']}): the figures above are not valid",
              file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
