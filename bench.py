#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode throughput at the layer sizes of
Qwen2.5-1.5B (random bfloat16 weights, batch 8, context 4,096), plus prefill of a
2,048-token prompt, decode at batch 1 and 64, and the achieved fraction of the roofline.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of the whole batch.  ``value`` is decoded tokens per second
from CUDA events around K back-to-back decode steps (inputs of every step copied from
pinned host memory, no host synchronisation inside the timed region).  ``e2e`` is the
same workload through ``Engine.step()``, the call a user makes: host token ids in, host
token ids out, every step.

The cache of the timed requests is filled with random keys and values (their prompts are
not run); weights and caches are far larger than the 126 MB L2, so every step streams
them from HBM.  One JSON line is printed.

``--workload serving-7b`` and ``--workload long-14b`` run the two further workloads that the
baseline names instead (their own JSON line, through ``Engine.generate``): continuous
batching of 64 requests at the 7B layer sizes (prompts uniform in [128, 2048], 256 output
tokens each, context 8,192, pages of 16), and a 16,384-token context at the 14B layer sizes
whose prefix 8 requests share (prefill in 2,048-token portions, prefix pages reused), then
decoding at batch 8.  ``--workload chat-1.5b`` is this repository's own: 256 short requests at the
1.5B layer sizes (prompts uniform in [16, 256], 16 to 128 output tokens each, at most 32 running), so
that requests end and begin all the time and many steps carry a new prompt beside decoded tokens,
which no graph replays: it measures what such steps cost the host.  ``--workload kapudra`` measures the Kapudra design
(matrix-memory layers and attention beside a gated delta rule) at two layer sizes beside Qwen2 at equal sizes: prefill and
decode through the step function, and the mixers' kernels alone.  ``--workload tutunex`` does the same for the Tutunex
design (differential attention over chunks, attention with a sink beside a gated delta rule, norms before and after each
sub-layer), its kernels beside the like kernels of the other models.  ``--workload zegelix`` does the same for the Zegelix
design (gated linear recurrences, window attention over positions and block means, routed experts with a shared expert, a
repeated span of layers).  ``--workload guvusun`` does the same for the Guvusun
design (latent attention with a learned sink and head gates, routed experts, norms after the sum) beside Qwen2 with a dense
feed-forward of the experts' active size.
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

# The headline configuration: Qwen2.5-1.5B layer sizes.
SIZES = dict(vocab_size=151936, hidden_size=1536, intermediate_size=8960, num_hidden_layers=28,
             num_attention_heads=12, num_key_value_heads=2, head_dim=128,
             max_position_embeddings=32768, rms_norm_eps=1e-6, rope_theta=1e6,
             tie_word_embeddings=True)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
# The two further workloads: Qwen2.5-7B and 14B layer sizes.
SIZES_7B = dict(vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_hidden_layers=28,
                num_attention_heads=28, num_key_value_heads=4, head_dim=128, max_position_embeddings=32768,
                rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)
SIZES_14B = dict(vocab_size=152064, hidden_size=5120, intermediate_size=13824, num_hidden_layers=48,
                 num_attention_heads=40, num_key_value_heads=8, head_dim=128, max_position_embeddings=32768,
                 rms_norm_eps=1e-5, rope_theta=1e6, tie_word_embeddings=False)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    src = "fallback"
    p = dict(FALLBACK_PEAKS)
    if os.path.isfile(path):
        try:
            obj = json.load(open(path))
            flat = {}

            def walk(o):
                if isinstance(o, dict):
                    for k, v in o.items():
                        if isinstance(v, (int, float)) and not isinstance(v, bool):
                            flat.setdefault(k, float(v))
                        else:
                            walk(v)
            walk(obj)
            if "hbm_gbs" in flat:
                p["hbm_gbs"] = flat["hbm_gbs"]
            if "bf16_tflops" in flat:
                p["bf16_tflops"] = flat["bf16_tflops"]
            if "bf16_tflops_sustained" in flat:
                p["bf16_tflops_sustained"] = flat["bf16_tflops_sustained"]
            src = "measured"
        except Exception:
            pass
    p["source"] = src
    return p


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def window(self, t0, t1):
        rows = [l.split(", ") for t, l in self.lines if t0 <= t <= t1 + 0.15 and l]
        if not rows:
            rows = [l.split(", ") for _, l in self.lines[-3:] if l]
        return rows

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=3)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    @staticmethod
    def summary(rows):
        mhz, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                mhz.append(int(r[0])); mx = max(mx, int(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[2:6]):
                if v.strip().lower().startswith("active"):
                    reasons.add(name)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def other_workload(args) -> int:
    """configs[3] (serving-7b) or configs[4] (long-14b) of the baseline through Engine.generate, or the
    short-request workload of this repository (chat-1.5b) through Engine.add_request / step."""
    import numpy as np
    import torch

    from coheryn_ai_studio_b200.config import Qwen2Config
    from coheryn_ai_studio_b200.engine import Engine, random_model_on_device
    serving = args.workload == "serving-7b"
    chat = args.workload == "chat-1.5b"
    sizes = dict(SIZES if chat else SIZES_7B if serving else SIZES_14B)
    full_layers = sizes["num_hidden_layers"]
    if args.layers != SIZES["num_hidden_layers"]:
        sizes["num_hidden_layers"] = args.layers
    cfg = Qwen2Config(**sizes)
    model = random_model_on_device(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    rng = np.random.default_rng(0)
    V = cfg.vocab_size
    if chat:
        eng = Engine(model, context=1024, max_num_seqs=32, max_num_batched_tokens=2048, page_size=16,
                     kv_cache_tokens=32 * 448, prefix_reuse=False, use_graphs=not args.no_graphs)
        prompts = [rng.integers(0, V, int(n)).tolist() for n in rng.integers(16, 257, 256)]
        outs = [int(n) for n in rng.integers(16, 129, 256)]

        def run_all():
            ids = [eng.add_request(p, n) for p, n in zip(prompts, outs)]
            steps = 0
            while eng.scheduler.has_work():
                eng.step()
                steps += 1
            return [eng.result(rid) for rid in ids], steps
        run_all()                                          # untimed: compilation, a graph per batch width met
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        res, steps = run_all()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        out_tokens = sum(r.completion_tokens for r in res)
        line = {"metric": "serving_output_tokens_per_s", "value": round(out_tokens / dt, 1), "unit": "tok/s",
                "seconds": round(dt, 3), "prompt_tokens": sum(len(p) for p in prompts), "output_tokens": out_tokens,
                "steps": steps, "ms_per_step": round(dt / steps * 1e3, 3),
                "preemptions": eng.scheduler.stats["preemptions"]}
        what = "Qwen2.5-1.5B layer sizes, 256 requests, prompts uniform[16,256], 16..128 outputs, 32 running, page 16"
    elif serving:
        eng = Engine(model, context=8192, max_num_seqs=64, max_num_batched_tokens=2048, page_size=16,
                     kv_cache_tokens=64 * 2400, prefix_reuse=False, use_graphs=not args.no_graphs)
        prompts = [rng.integers(0, V, int(n)).tolist() for n in rng.integers(128, 2049, 64)]
        outs = 256
        eng.generate(prompts, max_tokens=outs)             # untimed: compilation, a graph per batch width met
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        res = eng.generate(prompts, max_tokens=outs)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        out_tokens = sum(r.completion_tokens for r in res)
        line = {"metric": "serving_output_tokens_per_s", "value": round(out_tokens / dt, 1), "unit": "tok/s",
                "seconds": round(dt, 3), "prompt_tokens": sum(len(p) for p in prompts), "output_tokens": out_tokens,
                "total_tokens_per_s": round((sum(len(p) for p in prompts) + out_tokens) / dt, 1),
                "preemptions": eng.scheduler.stats["preemptions"]}
        what = "Qwen2.5-7B layer sizes, 64 requests, prompts uniform[128,2048], 256 outputs, context 8192, page 16"
    else:
        ctx, outs = 16384, 64
        eng = Engine(model, context=ctx + outs + 16, max_num_seqs=8, max_num_batched_tokens=2048, page_size=16,
                     kv_cache_tokens=3 * ctx, prefix_reuse=True, use_graphs=not args.no_graphs)
        warm = rng.integers(0, V, 2100).tolist()
        eng.generate([warm], max_tokens=4)                  # first-use compilation and graph capture
        shared = rng.integers(0, V, ctx - 256).tolist()
        prompts = [shared + rng.integers(0, V, 256).tolist() for _ in range(8)]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        eng.generate(prompts[:1], max_tokens=1)             # the shared prefix is computed once
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        res = eng.generate(prompts, max_tokens=outs)
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        decode_s = max(r.decode_ms for r in res) / 1e3
        line = {"metric": "long_context_decode_tokens_per_s", "value": round(8 * (outs - 1) / decode_s, 1), "unit": "tok/s",
                "prefill_tokens_per_s": round(ctx / (t1 - t0), 1), "prefill_seconds": round(t1 - t0, 3),
                "shared_prefix_seconds": round(t2 - t1, 3),
                "reused_prompt_tokens": [r.reused_prompt_tokens for r in res]}
        what = "Qwen2.5-14B layer sizes, 16384-token context, prefix shared by 8 requests, decode at batch 8"
    eng.cache.check()
    line.update({"n_gpus": 1, "higher_is_better": True, "dtype": "bf16", "data": "synthetic", "impl": "ours",
                 "config": {"model": what, "layers": cfg.num_hidden_layers, "layers_of_config": full_layers}})
    print(json.dumps(line))
    return 0


# Kapudra at layer sizes that resemble a real model's (random weights), beside Qwen2 at the same width, feed-forward
# size, head counts and number of layers.  Eight layers each: matrix memory, matrix memory, and twice attention beside
# a gated delta rule, repeated.
KAPUDRA_SIZES = {
    "1.5b-like": dict(width=1536, ff=4096, heads=12, kv_heads=2, head_dim=128, window=1024, state_heads=12, state_dim=128,
                      memory_heads=8, memory_vdim=256, vocab=32000, layers=8),
    "3b-like": dict(width=2560, ff=6912, heads=20, kv_heads=4, head_dim=128, window=2048, state_heads=16, state_dim=128,
                    memory_heads=8, memory_vdim=256, vocab=32000, layers=8),
}


def kapudra_config(z):
    left = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["head_dim"], "vdim": z["head_dim"],
            "scale": z["head_dim"] ** -0.5, "mask": {"size": z["window"]}}
    right = {"heads": z["state_heads"], "kv_heads": z["state_heads"], "dim": z["state_dim"], "vdim": z["state_dim"], "conv": 4,
             "a_rank": 64, "g_rank": 64}
    par = {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": 1.0, "right_scale": 1.0},
           "mlp": {"kind": "dense", "ff": z["ff"]}}
    mem = {"type": "mlstm", "mixer": {"heads": z["memory_heads"], "dim": z["state_dim"], "vdim": z["memory_vdim"], "gate_cap": 15.0},
           "mlp": {"kind": "dense", "ff": z["ff"]}}
    kinds = [mem, mem, par, par]
    return {"architecture": "Kapudra", "vocab": z["vocab"], "width": z["width"], "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
            "logit_scale": 1.0, "logit_softcap": 30.0, "layers": [kinds[i % 4] for i in range(z["layers"])]}


def model_bench_tools(args):
    """What the per-design workloads share: peaks, a timer of single kernels with L2 flushed before each run, prefill and
    decode of a model through the step function (CUDA events around the steps, inputs from pinned host memory as every step
    has them), and a step description for kernels that are run alone."""
    import types
    import numpy as np
    import torch

    from coheryn_ai_studio_b200 import ops
    from coheryn_ai_studio_b200.cache import CacheManager
    from coheryn_ai_studio_b200.engine import StepEntry, StepRunner, random_model_on_device

    pk = peaks()
    hbm = pk["hbm_gbs"] * 1e9
    flops_peak = pk.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]) * 1e12
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    tokens, batch, context, steps = args.prefill_tokens, args.batch, min(args.context, 2048), max(8, min(args.steps, 32))
    rng = np.random.default_rng(0)

    def timed(fn, repeats=5):
        """Median of CUDA-event times of fn() with L2 flushed before each."""
        out = []
        for r in range(repeats + 2):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize()
            if r >= 2:
                out.append(e0.elapsed_time(e1))
        return float(np.median(out))

    def run_model(model, vocab):
        need = batch * (context + steps + 16) + tokens + 64
        cache = CacheManager(model.cache_requirements(), [e.cache_from for e in model.spec.schedule], torch.bfloat16, dev,
                             page_size=args.page_size, num_pages=-(-need // args.page_size) + batch + 1, max_requests=batch + 1,
                             prefix_reuse=False)
        runner = StepRunner(model, cache, use_graphs=not args.no_graphs, graph_max_kv_len=context + steps + 16)
        best = None
        for r in range(3):
            cache.admit("p")
            prompt = rng.integers(0, vocab, size=tokens).tolist()
            torch.cuda.synchronize(); flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); runner.step([StepEntry("p", prompt, [tokens - 1])]); e1.record()
            torch.cuda.synchronize()
            runner.check_status()
            cache.free("p")
            if r:
                best = e0.elapsed_time(e1) if best is None else min(best, e0.elapsed_time(e1))
        ids = [f"d{i}" for i in range(batch)]
        for rid in ids:                      # the contexts are really computed: a recurrent state cannot be made up
            cache.admit(rid)
            runner.step([StepEntry(rid, rng.integers(0, vocab, size=context).tolist(), [])])
        nxt = lambda: [StepEntry(rid, [int(rng.integers(0, vocab))], [0]) for rid in ids]
        for _ in range(max(3, args.warmup)):
            runner.step(nxt())
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            runner.step(nxt())
        e1.record()
        torch.cuda.synchronize()
        runner.check_status()
        ms = e0.elapsed_time(e1) / steps
        return {"prefill_tokens_per_s": round(tokens / (best / 1e3)), "prefill_ms": round(best, 3),
                "decode_tokens_per_s": round(batch / (ms / 1e3)), "decode_ms_per_step": round(ms, 4)}

    def step_like(lengths, starts, tables=None):
        import types
        cu = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
        t = lambda a: torch.as_tensor(np.asarray(a, dtype=np.int32)).to(dev)
        st = types.SimpleNamespace(
            num_requests=len(lengths), num_tokens=int(cu[-1]), cu_q=t(cu), token_req=t(np.repeat(np.arange(len(lengths)), lengths)),
            positions=t(np.concatenate([np.arange(s, s + n) for s, n in zip(starts, lengths)])), state_slots=t(np.arange(len(lengths))),
            q_lens=list(lengths), kv_lens=t([s + n for s, n in zip(starts, lengths)]), max_q_len=max(lengths),
            max_kv_len=max(s + n for s, n in zip(starts, lengths)), prior_positions_settled=True, block_tables=[tables])
        return st

    return types.SimpleNamespace(pk=pk, hbm=hbm, flops_peak=flops_peak, dev=dev, tokens=tokens, batch=batch, context=context,
                                 steps=steps, rng=rng, timed=timed, run_model=run_model, step_like=step_like)


def kapudra_workload(args) -> int:
    """Prefill and decode throughput of Kapudra and of Qwen2 at equal sizes through the step function (CUDA events around
    the steps, inputs from pinned host memory as every step has them), and the mixers' kernels alone with their share of
    the roofline.  One JSON line."""
    import numpy as np
    import torch

    from coheryn_ai_studio_b200 import ops
    from coheryn_ai_studio_b200.config import Qwen2Config
    from coheryn_ai_studio_b200.config.kapudra import KapudraConfig
    from coheryn_ai_studio_b200.engine import random_model_on_device

    tools = model_bench_tools(args)
    pk, hbm, flops_peak, dev = tools.pk, tools.hbm, tools.flops_peak, tools.dev
    tokens, batch, context, steps = tools.tokens, tools.batch, tools.context, tools.steps
    timed, run_model, step_like = tools.timed, tools.run_model, tools.step_like

    def kernels(z):
        """The mixers' kernels alone, prompt (one request of ``tokens``) and decode (``batch`` requests at ``context``)."""
        out = {}
        H, G, hd, W, page = z["heads"], z["kv_heads"], z["head_dim"], z["window"], args.page_size
        pages_per = -(-(context + 1) // page)
        for name, lengths, starts in (("prefill", [tokens], [0]), ("decode", [1] * batch, [context] * batch)):
            B, T = len(lengths), sum(lengths)
            per = -(-max(s + n for s, n in zip(starts, lengths)) // page)
            tables = torch.arange(B * per, dtype=torch.int32, device=dev).view(B, per)
            st = step_like(lengths, starts, tables)
            kc = torch.randn((B * per + 1, G, page, hd), device=dev).to(torch.bfloat16)
            vc = torch.randn_like(kc)
            q = torch.randn((T, H * hd), device=dev).to(torch.bfloat16)
            o = torch.empty_like(q)
            slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=torch.float32, device=dev)
            seen = lambda w: sum(min(w, p + 1) for s, n in zip(starts, lengths) for p in range(s, s + n))       # keys read per head
            for label, window, sl in (("attention_bias_window", W, slopes), ("attention_window", W, None), ("attention_full", None, None)):
                fn = lambda: ops.attention_biased(q, o, kc, vc, st, 0, H, G, hd, hd, page, window, hd ** -0.5, sl) if sl is not None else \
                    ops.attention_rows(q, o, kc, vc, tables, st.token_req, st.positions, H, G, hd, page, window, hd ** -0.5, cu_q=st.cu_q,
                                       kv_lens=st.kv_lens, q_lens=st.q_lens, max_kv_len=st.max_kv_len)
                ms = timed(fn)
                keys = seen(window if window else 1 << 30)
                fl = 4.0 * H * hd * keys
                by = 2.0 * 2 * G * hd * sum(min(window or 1 << 30, s + n) for s, n in zip(starts, lengths)) + 4.0 * T * H * hd
                out[f"{name}.{label}"] = {"ms": round(ms, 4), "tflops": round(fl / ms / 1e9, 1), "of_bf16_peak": round(fl / (ms / 1e3) / flops_peak, 4),
                                          "of_hbm": round(by / (ms / 1e3) / hbm, 4)}
            # the two scans: float32 inputs as the projections leave them
            for label, heads, dk, dv in (("gated_delta_scan", z["state_heads"], z["state_dim"], z["state_dim"]),
                                         ("matrix_memory_scan", z["memory_heads"], z["state_dim"], z["memory_vdim"])):
                f = lambda *shape: torch.randn(shape, device=dev)
                qkv = f(T, 2 * heads * dk + heads * dv)
                gate, outb = f(T, heads * dv), torch.empty((T, heads * dv), dtype=torch.bfloat16, device=dev)
                if label == "gated_delta_scan":
                    state = torch.zeros((B, heads * dk * dv), device=dev)
                    beta, pre, bias, rate, w = f(T, heads), f(T, heads * dk), f(heads * dk), f(heads) * 0.1, f(dv)
                    fn = lambda: ops.gated_delta_scan(qkv[:, :heads * dk], qkv[:, heads * dk:2 * heads * dk], qkv[:, 2 * heads * dk:], beta, pre,
                                                      bias, rate, state, st, heads, heads, dk, dv, outb, w, gate, 1e-6)
                    fl = 8.0 * heads * dk * dv * T
                else:
                    state = torch.zeros((B, heads * (dk * dv + dk + 1)), device=dev)
                    gates, bi, w = f(T, 2 * heads), f(heads), f(heads * dv)
                    fn = lambda: ops.matrix_memory_scan(qkv[:, :heads * dk], qkv[:, heads * dk:2 * heads * dk], qkv[:, 2 * heads * dk:],
                                                        gates[:, :heads], gates[:, heads:], bi, bi, 15.0, state, st, heads, dk, dv, outb, w, gate, 1e-6)
                    fl = 6.0 * heads * dk * dv * T
                ms = timed(fn)
                by = 2.0 * state.numel() * 4 + qkv.numel() * 4 + gate.numel() * 4 + outb.numel() * 2
                out[f"{name}.{label}"] = {"ms": round(ms, 4), "tflops": round(fl / ms / 1e9, 2), "of_hbm": round(by / (ms / 1e3) / hbm, 4),
                                          "of_fp32_fma_peak": round(fl / (ms / 1e3) / 75e12, 4)}
        return out

    sampler = ClockSampler()
    sampler.start()
    t0 = time.time()
    results = {}
    chosen = [n for n in KAPUDRA_SIZES if not args.sizes or n in args.sizes.split(",")]
    for name in chosen:
        z = KAPUDRA_SIZES[name]
        entry = {}
        model = random_model_on_device(KapudraConfig.from_dict(kapudra_config(z)), seed=0, dtype="bfloat16", device="cuda:0")
        entry["kapudra"] = run_model(model, z["vocab"])
        del model
        torch.cuda.empty_cache()
        qcfg = Qwen2Config(vocab_size=z["vocab"], hidden_size=z["width"], intermediate_size=z["ff"], num_hidden_layers=z["layers"],
                           num_attention_heads=z["heads"], num_key_value_heads=z["kv_heads"], head_dim=z["head_dim"],
                           max_position_embeddings=32768, rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)
        model = random_model_on_device(qcfg, seed=0, dtype="bfloat16", device="cuda:0")
        entry["qwen2_equal_size"] = run_model(model, z["vocab"])
        del model
        torch.cuda.empty_cache()
        entry["kernels"] = kernels(z)
        results[name] = entry
    clocks = ClockSampler.summary(sampler.window(t0, time.time()))
    sampler.stop()
    print(json.dumps({"workload": "kapudra", "dtype": "bf16", "data": "synthetic", "prefill_tokens": tokens, "decode_batch": batch,
                      "decode_context": context, "decode_steps": steps, "peaks": pk, "clocks": clocks, "l2": "flushed before each timed kernel",
                      "gpu_launches": ops.total_launch_count(), "sizes": results}))
    return 0


# Tutunex at layer sizes that resemble a real model's (random weights), beside Qwen2 at the same width, feed-forward
# size, head counts and number of layers.  Eight layers: differential attention over chunks, attention with a sink beside
# a gated delta rule, differential attention on the first layer's keys and values, differential attention; twice.
TUTUNEX_SIZES = {
    "1.5b-like": dict(width=1536, ff=4096, heads=12, kv_heads=2, map_dim=64, vdim=128, chunk=1024, side_dim=128, state_heads=12,
                      state_dim=128, vocab=32000, layers=8),
    "3b-like": dict(width=2560, ff=6912, heads=20, kv_heads=4, map_dim=64, vdim=128, chunk=2048, side_dim=128, state_heads=16,
                    state_dim=128, vocab=32000, layers=8),
}


def tutunex_config(z):
    rot = {"dims": z["map_dim"], "base": 500000.0, "scaling": {"factor": 8.0, "original": 8192, "fast": 32.0, "slow": 1.0}}

    def attention(kv_from=None):
        m = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["map_dim"], "vdim": z["vdim"], "scale": z["map_dim"] ** -0.5,
             "diff": 0.5, "rot": rot, "mask": {"size": z["chunk"]}}
        if kv_from is not None:
            m["kv_from"] = kv_from
        return {"type": "attention", "mixer": m, "mlp": {"kind": "dense", "ff": z["ff"], "limit": 7.0}}
    left = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["side_dim"], "vdim": z["side_dim"], "scale": z["side_dim"] ** -0.5}
    right = {"heads": z["state_heads"], "kv_heads": z["state_heads"], "dim": z["state_dim"], "vdim": z["state_dim"], "conv": 4}
    par = {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": {"kind": "dense", "ff": z["ff"], "limit": 7.0}}
    layers = []
    for i in range(z["layers"]):
        k = i % 4
        layers.append(par if k == 1 else attention(kv_from=i - 2 if k == 2 else None))
    return {"architecture": "Tutunex", "vocab": z["vocab"], "width": z["width"], "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
            "layers": layers}


def tutunex_workload(args) -> int:
    """Prefill and decode throughput of Tutunex and of Qwen2 at equal sizes through the step function, and the design's own
    kernels alone beside the like kernels of the other models, each with its share of the roofline.  One JSON line."""
    import numpy as np
    import torch

    from coheryn_ai_studio_b200 import ops
    from coheryn_ai_studio_b200.config import Qwen2Config
    from coheryn_ai_studio_b200.config.tutunex import TutunexConfig
    from coheryn_ai_studio_b200.engine import random_model_on_device
    from coheryn_ai_studio_b200.parts.base import Runtime
    from coheryn_ai_studio_b200.parts.position import ComputedRope, RotateHalfRope

    tools = model_bench_tools(args)
    pk, hbm, flops_peak, dev = tools.pk, tools.hbm, tools.flops_peak, tools.dev
    tokens, batch, context = tools.tokens, tools.batch, tools.context
    timed, step_like = tools.timed, tools.step_like

    def kernels(z):
        out = {}
        H, G, dm, dv, chunk, page, W = z["heads"], z["kv_heads"], z["map_dim"], z["vdim"], z["chunk"], args.page_size, z["width"]
        ds = z["side_dim"]
        f = lambda *shape: torch.randn(shape, device=dev)
        b16 = lambda *shape: f(*shape).to(torch.bfloat16)
        for name, lengths, starts in (("prefill", [tokens], [0]), ("decode", [1] * batch, [context] * batch)):
            B, T = len(lengths), sum(lengths)
            per = -(-max(s + n for s, n in zip(starts, lengths)) // page)
            tables = torch.arange(B * per, dtype=torch.int32, device=dev).view(B, per)
            st = step_like(lengths, starts, tables)
            st.slots = [(tables[st.token_req.long(), (st.positions // page).long()] * page + st.positions % page).to(torch.int32)]
            rows = [p for s, n in zip(starts, lengths) for p in range(s, s + n)]

            def report(label, fn, keys, qk, vd, kv_row_bytes, kv_positions):
                ms = timed(fn)
                fl = 2.0 * H * (qk + vd) * keys
                by = kv_row_bytes * G * kv_positions + 2.0 * T * H * (qk + vd)
                out[f"{name}.{label}"] = {"ms": round(ms, 4), "tflops": round(fl / ms / 1e9, 1), "of_bf16_peak": round(fl / (ms / 1e3) / flops_peak, 4),
                                          "of_hbm": round(by / (ms / 1e3) / hbm, 4)}
            # differential attention over chunks, and Qwen2's attention with a window of the chunk's size at the same head size
            kc, vc = b16(B * per + 1, G, page, 2 * dm), b16(B * per + 1, G, page, dv)
            q, o = b16(T, H * 2 * dm), torch.empty((T, H * dv), dtype=torch.bfloat16, device=dev)
            seen_chunk = sum(p % chunk + 1 for p in rows)
            held_chunk = sum(min(chunk, s + n) if n > 1 else (s + n - 1) % chunk + 1 for s, n in zip(starts, lengths))
            report("attention_two_maps_chunk", lambda: ops.attention_maps(q, o, kc, vc, st, 0, H, G, dm, dv, 2, page, None, chunk, False,
                                                                          dm ** -0.5, 0.6, True, 1e-6, 0.5),
                   seen_chunk, 2 * dm, dv, 2.0 * (2 * dm + dv), held_chunk)
            hd = 2 * dm
            kq, vq = b16(B * per + 1, G, page, hd), b16(B * per + 1, G, page, hd)
            qq, oq = b16(T, H * hd), torch.empty((T, H * hd), dtype=torch.bfloat16, device=dev)
            seen_window = sum(min(chunk, p + 1) for p in rows)
            report("qwen2_attention_window", lambda: ops.attention_rows(qq, oq, kq, vq, tables, st.token_req, st.positions, H, G, hd, page, chunk,
                                                                        hd ** -0.5, cu_q=st.cu_q, kv_lens=st.kv_lens, q_lens=st.q_lens,
                                                                        max_kv_len=st.max_kv_len),
                   seen_window, hd, hd, 4.0 * hd, sum(min(chunk, s + n) for s, n in zip(starts, lengths)))
            # causal attention with a sink, and Qwen2's causal attention
            ks, vs = b16(B * per + 1, G, page, ds), b16(B * per + 1, G, page, ds)
            qs, os_ = b16(T, H * ds), torch.empty((T, H * ds), dtype=torch.bfloat16, device=dev)
            seen_all = sum(p + 1 for p in rows)
            held_all = sum(s + n for s, n in zip(starts, lengths))
            report("attention_sink_causal", lambda: ops.attention_maps(qs, os_, ks, vs, st, 0, H, G, ds, ds, 1, page, None, None, True,
                                                                       ds ** -0.5, 0.0, False, 1e-6, 1.0), seen_all, ds, ds, 4.0 * ds, held_all)
            report("qwen2_attention_causal", lambda: ops.attention_rows(qs, os_, ks, vs, tables, st.token_req, st.positions, H, G, ds, page, None,
                                                                        ds ** -0.5, cu_q=st.cu_q, kv_lens=st.kv_lens, q_lens=st.q_lens,
                                                                        max_kv_len=st.max_kv_len), seen_all, ds, ds, 4.0 * ds, held_all)

            def elementwise(label, fn, by):
                ms = timed(fn)
                out[f"{name}.{label}"] = {"ms": round(ms, 4), "of_hbm": round(by / (ms / 1e3) / hbm, 4)}
            # queries and keys rotated by computed angles into the cache, and Qwen2's rotation by table
            proj = f(T, (H * 2 * dm) + (G * 2 * dm) + G * dv)
            nq, nk = H * 2 * dm, G * 2 * dm
            rope = ComputedRope(Runtime(torch.bfloat16, dev), dm, 500000.0, {"factor": 8.0, "original": 8192, "fast": 32.0, "slow": 1.0})
            pairs, amp = rope.frequency_pairs(), rope.amplitude
            elementwise("rotate_computed_and_cache_write",
                        lambda: ops.unit_norm_rope_kv_write(proj[:, :nq], proj[:, nq:nq + nk], proj[:, nq + nk:], None, None, 1e-6, st.positions, pairs,
                                                            dm, amp, st.slots[0], kc, vc, 2 * H, 2 * G, G, dm, dv, page, torch.bfloat16),
                        proj.numel() * 4.0 + proj.numel() * 2.0)
            table = RotateHalfRope(Runtime(torch.bfloat16, dev), hd, hd, 1e6, context + tokens + 8).cos_sin()
            qkv = b16(T, (H + 2 * G) * hd)
            elementwise("qwen2_rotate_by_table_and_cache_write",
                        lambda: ops.rope_kv_write(qkv, st.positions, table, st.slots[0], kq, vq, H, G, hd, hd, page),
                        qkv.numel() * 2.0 + (H + 2 * G) * hd * T * 2.0)
            # the residual add of a normalised summand with the next norm, and the plain add with the norm
            resid, y2, w1, w2 = f(T, W), f(2, T, W), f(W), f(W)
            wi, h = f(2, W), torch.empty((T, W), dtype=torch.bfloat16, device=dev)
            elementwise("add_normalised_and_norm", lambda: ops.add_normed_rmsnorm(resid, y2[0], None, 1.0, w1, w2, 1e-6, h), T * W * (4 + 8 + 2.0))
            elementwise("add_two_normalised_and_norm", lambda: ops.add_normed_rmsnorm(resid, y2, wi, 0.5, w1, w2, 1e-6, h), T * W * (8 + 8 + 2.0))
            yb = b16(T, W)
            elementwise("qwen2_add_and_norm", lambda: ops.add_rmsnorm(resid, yb, w2, 1e-6, h), T * W * (2 + 8 + 2.0))
            # the delta rule with one decay per head and a SiLU gate, and Kapudra's with a decay per head and key channel
            heads, dk = z["state_heads"], z["state_dim"]
            qkvs = f(T, 3 * heads * dk)
            gate, outb = f(T, heads * dk), torch.empty((T, heads * dk), dtype=torch.bfloat16, device=dev)
            state = torch.zeros((B, heads * dk * dk), device=dev)
            beta, pre1, preC, bias1, biasC, rate, wn = f(T, heads), f(T, heads), f(T, heads * dk), f(heads), f(heads * dk), f(heads) * 0.1, f(dk)
            for label, pre, bias, per_channel, act in (("delta_rule_decay_per_head", pre1, bias1, False, "silu"),
                                                       ("kapudra_delta_rule_decay_per_channel", preC, biasC, True, "sigmoid")):
                fn = lambda: ops.gated_delta_scan(qkvs[:, :heads * dk], qkvs[:, heads * dk:2 * heads * dk], qkvs[:, 2 * heads * dk:], beta, pre, bias,
                                                  rate, state, st, heads, heads, dk, dk, outb, wn, gate, 1e-6, decay_per_channel=per_channel,
                                                  gate_activation=act)
                ms = timed(fn)
                by = 2.0 * state.numel() * 4 + qkvs.numel() * 4 + gate.numel() * 4 + outb.numel() * 2
                fl = 8.0 * heads * dk * dk * T
                out[f"{name}.{label}"] = {"ms": round(ms, 4), "of_hbm": round(by / (ms / 1e3) / hbm, 4),
                                          "of_fp32_fma_peak": round(fl / (ms / 1e3) / 75e12, 4)}
        return out

    sampler = ClockSampler()
    sampler.start()
    t0 = time.time()
    results = {}
    chosen = [n for n in TUTUNEX_SIZES if not args.sizes or n in args.sizes.split(",")]
    for name in chosen:
        z = TUTUNEX_SIZES[name]
        entry = {}
        model = random_model_on_device(TutunexConfig.from_dict(tutunex_config(z)), seed=0, dtype="bfloat16", device="cuda:0")
        entry["tutunex"] = tools.run_model(model, z["vocab"])
        del model
        torch.cuda.empty_cache()
        qcfg = Qwen2Config(vocab_size=z["vocab"], hidden_size=z["width"], intermediate_size=z["ff"], num_hidden_layers=z["layers"],
                           num_attention_heads=z["heads"], num_key_value_heads=z["kv_heads"], head_dim=2 * z["map_dim"],
                           max_position_embeddings=32768, rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)
        model = random_model_on_device(qcfg, seed=0, dtype="bfloat16", device="cuda:0")
        entry["qwen2_equal_size"] = tools.run_model(model, z["vocab"])
        del model
        torch.cuda.empty_cache()
        entry["kernels"] = kernels(z)
        results[name] = entry
    clocks = ClockSampler.summary(sampler.window(t0, time.time()))
    sampler.stop()
    print(json.dumps({"workload": "tutunex", "dtype": "bf16", "data": "synthetic", "prefill_tokens": tokens, "decode_batch": batch,
                      "decode_context": context, "decode_steps": tools.steps, "peaks": pk, "clocks": clocks,
                      "l2": "flushed before each timed kernel", "gpu_launches": ops.total_launch_count(), "sizes": results}))
    return 0


# Sizes of --workload guvusun.  Eight layers of latent attention with routed experts; layers 3 and 7 read the cached rows of
# layers 2 and 6.  `small-latent`: cached rows of 256 channels (what the tensor-core attention is compiled for);
# `wide-latent`: rows of 576 channels, the proportions of the large published models with latent attention.  Qwen2 beside
# each at equal width, layers, head count, head size dim + rot_dim, two key/value heads (a cache of about the same bytes per
# token) and a dense feed-forward of top x expert size (the same active matrix rows per token).
GUVUSUN_SIZES = {
    "small-latent": dict(width=2048, heads=16, dim=96, rot_dim=32, vdim=128, kv_rank=224, experts=30, identity=2, top=4,
                         groups=(4, 2), ff=1024, side_dim=64, buckets=100003, vocab=32000, layers=8),
    "wide-latent": dict(width=2048, heads=16, dim=128, rot_dim=64, vdim=128, kv_rank=512, experts=62, identity=2, top=6,
                        groups=(8, 4), ff=1408, side_dim=64, buckets=100003, vocab=32000, layers=8),
}


def guvusun_config(z):
    rot = {"dims": z["rot_dim"], "base": 10000.0, "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}}
    layers = []
    for i in range(z["layers"]):
        m = {"heads": z["heads"], "dim": z["dim"], "rot_dim": z["rot_dim"], "vdim": z["vdim"], "kv_rank": z["kv_rank"],
             "scale": (z["dim"] + z["rot_dim"]) ** -0.5, "rot": rot}
        if i % 4 == 3:
            m["kv_from"] = i - 1
        router = {"experts": z["experts"], "top": z["top"], "identity": z["identity"], "scale": 2.5,
                  "groups": {"count": z["groups"][0], "keep": z["groups"][1]}}
        layers.append({"type": "latent_attention", "mixer": m, "mlp": {"kind": "moe", "expert": {"ff": z["ff"]}, "router": router}})
    return {"architecture": "Guvusun", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6}, "postln_alpha": 2.0,
            "embedding": {"bigram": {"buckets": z["buckets"], "mul_prev": 131, "mul_cur": 11}}, "token_side": {"dim": z["side_dim"]},
            "layers": layers}


def guvusun_workload(args) -> int:
    """Prefill and decode throughput of Guvusun and of Qwen2 at equal sizes through the step function, and the design's own
    kernels alone beside the like kernels of Qwen2, each with its share of the roofline.  One JSON line."""
    import numpy as np
    import torch

    from coheryn_ai_studio_b200 import ops
    from coheryn_ai_studio_b200.config import Qwen2Config
    from coheryn_ai_studio_b200.config.guvusun import GuvusunConfig
    from coheryn_ai_studio_b200.engine import random_model_on_device
    from coheryn_ai_studio_b200.parts.base import Runtime
    from coheryn_ai_studio_b200.parts.position import ComputedRope, RotateHalfRope

    tools = model_bench_tools(args)
    pk, hbm, flops_peak, dev = tools.pk, tools.hbm, tools.flops_peak, tools.dev
    tokens, batch, context = tools.tokens, tools.batch, tools.context
    timed, step_like = tools.timed, tools.step_like

    def kernels(z):
        out = {}
        H, dim, rd, dv, rank, page, W = z["heads"], z["dim"], z["rot_dim"], z["vdim"], z["kv_rank"], args.page_size, z["width"]
        row, hd = rank + rd, dim + rd
        E, top, F, outputs = z["experts"], z["top"], z["ff"], z["experts"] + z["identity"]
        f = lambda *shape: torch.randn(shape, device=dev)
        b16 = lambda *shape: f(*shape).to(torch.bfloat16)
        for name, lengths, starts in (("prefill", [tokens], [0]), ("decode", [1] * batch, [context] * batch)):
            B, T = len(lengths), sum(lengths)
            per = -(-max(s + n for s, n in zip(starts, lengths)) // page)
            tables = torch.arange(B * per, dtype=torch.int32, device=dev).view(B, per)
            st = step_like(lengths, starts, tables)
            st.slots = [(tables[st.token_req.long(), (st.positions // page).long()] * page + st.positions % page).to(torch.int32)]
            st.token_ids = torch.randint(0, z["vocab"], (T,), dtype=torch.int32, device=dev)
            seen = sum(p + 1 for s, n in zip(starts, lengths) for p in range(s, s + n))
            held = sum(s + n for s, n in zip(starts, lengths))

            def attention(label, fn, issued_per_score, needed_per_score, cache_bytes, io_bytes):
                ms = timed(fn)
                out[f"{name}.{label}"] = {
                    "ms": round(ms, 4), "tflops_issued": round(2.0 * H * issued_per_score * seen / ms / 1e9, 1),
                    "of_bf16_peak_issued": round(2.0 * H * issued_per_score * seen / (ms / 1e3) / flops_peak, 4),
                    "of_bf16_peak_needed": round(2.0 * H * needed_per_score * seen / (ms / 1e3) / flops_peak, 4),
                    "of_hbm": round((cache_bytes + io_bytes) / (ms / 1e3) / hbm, 4)}
            # the heads over ONE cached row per position whose first `rank` channels are also the values (queries carried
            # into the latent space), and Qwen2's causal attention over two key/value heads at head size dim + rot_dim
            kc = b16(B * per + 1, 1, page, row)
            q, o = b16(T, H * row), torch.empty((T, H * rank), dtype=torch.bfloat16, device=dev)
            sinks = f(H)
            attention("latent_attention_sink", lambda: ops.attention_maps(
                q, o, kc, None, st, 0, H, 1, row, rank, 1, page, None, None, True, hd ** -0.5, 0.0, False, 1e-6, 1.0,
                sink_scores=sinks, values_in_keys=True), row + rank, min(row + rank, hd + dv), 2.0 * row * held, 2.0 * T * H * (row + rank))
            if name == "prefill" and hd % 16 == 0 and dv % 16 == 0 and hd <= 256 and dv <= 256:
                # what a whole prompt runs instead: its rows expanded per head (keys uk_h c | rotated key, values uv_h c), then the
                # same kernel with a key head per query head and the gates in its epilogue
                rows_c, ukr, uvr = b16(T, row), b16(H, dim, rank), b16(H, dv, rank)
                ke, ve = torch.empty((T, H * hd), dtype=torch.bfloat16, device=dev), torch.empty((T, H * dv), dtype=torch.bfloat16, device=dev)

                def expand():
                    got = ops.gather_rows(kc.view(-1, row), st.slots[0])
                    ops.grouped_linear(got, ukr, ke, a_col=0, c_col=hd)
                    ops.copy_head_columns(got, 0, rank, ke, hd, dim, rd, H)
                    ops.grouped_linear(got, uvr, ve, a_col=0, c_col=dv)
                ms = timed(expand)
                fl = 2.0 * T * H * rank * (dim + dv)
                out[f"{name}.latent_rows_expanded_per_head"] = {"ms": round(ms, 4), "tflops": round(fl / ms / 1e9, 1),
                                                                 "of_bf16_peak": round(fl / (ms / 1e3) / flops_peak, 4)}
                import types
                dense = types.SimpleNamespace(block_tables=[torch.arange(T, dtype=torch.int32, device=dev).view(1, T)], token_req=st.token_req,
                                              positions=st.positions, cu_q=st.cu_q, kv_lens=st.kv_lens, q_lens=st.q_lens, max_kv_len=st.max_kv_len)
                qe, oe, gl = b16(T, H * hd), torch.empty((T, H * dv), dtype=torch.bfloat16, device=dev), f(T, H)
                attention("attention_sink_expanded_rows", lambda: ops.attention_maps(
                    qe, oe, ke.view(T, H, 1, hd), ve.view(T, H, 1, dv), dense, 0, H, H, hd, dv, 1, 1, None, None, True, hd ** -0.5, 0.0, False,
                    1e-6, 1.0, sink_scores=sinks, head_gates=gl), hd + dv, hd + dv, 2.0 * T * H * (hd + dv), 2.0 * T * H * (hd + dv))
            G = 2
            kq, vq = b16(B * per + 1, G, page, hd), b16(B * per + 1, G, page, hd)
            qq, oq = b16(T, H * hd), torch.empty((T, H * hd), dtype=torch.bfloat16, device=dev)
            attention("qwen2_attention_causal", lambda: ops.attention_rows(
                qq, oq, kq, vq, tables, st.token_req, st.positions, H, G, hd, page, None, hd ** -0.5, cu_q=st.cu_q, kv_lens=st.kv_lens,
                q_lens=st.q_lens, max_kv_len=st.max_kv_len), 2 * hd, 2 * hd, 4.0 * hd * G * held, 4.0 * T * H * hd)

            def by_bytes(label, fn, by, flops=None):
                ms = timed(fn)
                out[f"{name}.{label}"] = {"ms": round(ms, 4), "of_hbm": round(by / (ms / 1e3) / hbm, 4)}
                if flops is not None:
                    out[f"{name}.{label}"].update({"tflops": round(flops / ms / 1e9, 1), "of_bf16_peak": round(flops / (ms / 1e3) / flops_peak, 4)})
            # in front of the scores: latent normalised, both rotated parts turned by computed angles, the cache row written,
            # the queries cast; Qwen2's rotation by table with its cache write
            cols = H * hd + row + H
            proj = f(T, cols)
            wn = f(rank)
            rope = ComputedRope(Runtime(torch.bfloat16, dev), rd, 10000.0, {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0})
            by_bytes("latent_prepare_and_cache_write", lambda: ops.latent_prepare(
                proj, H, dim, rd, rank, H * hd, wn, 1e-6, st.positions, rope.frequency_pairs(), rd, rope.amplitude, st.slots[0], kc, page,
                torch.bfloat16), T * (H * hd + row) * 4.0 + T * (H * dim + H * rd + row) * 2.0)
            table = RotateHalfRope(Runtime(torch.bfloat16, dev), hd, hd, 1e6, context + tokens + 8).cos_sin()
            qkv = b16(T, (H + 2 * G) * hd)
            by_bytes("qwen2_rotate_by_table_and_cache_write",
                     lambda: ops.rope_kv_write(qkv, st.positions, table, st.slots[0], kq, vq, H, G, hd, hd, page), 4.0 * T * (H + 2 * G) * hd)
            # the products per head on both sides of the attention
            qp, uk = b16(T, H * dim), b16(H, rank, dim)
            by_bytes("queries_into_latent_space", lambda: ops.grouped_linear(qp, uk, q, a_col=dim, c_col=row),
                     2.0 * (T * H * (dim + rank) + H * rank * dim), 2.0 * T * H * rank * dim)
            uv, gates, og = b16(H, dv, rank), f(T, H), torch.empty((T, H * dv), dtype=torch.bfloat16, device=dev)
            by_bytes("values_out_of_latent_space_gated", lambda: ops.grouped_linear(o, uv, og, a_col=rank, c_col=dv, factor=gates, factor_sigmoid=True),
                     2.0 * (T * H * (dv + rank) + H * rank * dv), 2.0 * T * H * rank * dv)
            # the stream: norm after the sum, and Qwen2's add with the next norm
            x, d, w1 = f(T, W), f(T, W), f(W)
            h = torch.empty((T, W), dtype=torch.bfloat16, device=dev)
            by_bytes("scaled_add_then_norm", lambda: ops.scaled_add_norm(x, d, 2.0, w1, 1e-6, h), T * W * (4 + 4 + 4 + 2.0))
            by_bytes("add_normalised_summand", lambda: ops.scaled_add_norm(x, d, 1.0, w1, 1e-6, h, normed_summand=True), T * W * (4 + 4 + 4 + 2.0))
            resid, yb = f(T, W), b16(T, W)
            by_bytes("qwen2_add_and_norm", lambda: ops.add_rmsnorm(resid, yb, w1, 1e-6, h), T * W * (2 + 8 + 2.0))
            # the router and the experts, and a dense gated feed-forward of top x expert size
            logits, corr = f(T, outputs), f(outputs) * 0.01
            by_bytes("route_select", lambda: ops.route_select(logits, corr, z["groups"][0], z["groups"][1], top, 2.5), T * (outputs * 4.0 + top * 8.0))
            ids, weights = ops.route_select(logits, corr, z["groups"][0], z["groups"][1], top, 2.5)
            by_bytes("route_sort", lambda: ops.route_sort(ids, E), T * top * 12.0)
            rows = ops.route_sort(ids, E)
            real = int((ids < E).sum())
            xb, wgu, wd = b16(T, W), b16(E, 2 * F, W), b16(E, W, F)
            act, y = torch.empty((rows.n, F), dtype=torch.bfloat16, device=dev), torch.empty((rows.n, W), device=dev)
            used = min(E, real)
            by_bytes("experts_gate_up", lambda: ops.grouped_linear(xb, wgu, act, rows=rows, gather=True, epilogue=ops.gated_epilogue_word("silu", None)),
                     2.0 * (used * 2 * F * W + real * (W + F)), 4.0 * real * F * W)
            by_bytes("experts_down", lambda: ops.grouped_linear(act, wd, y, rows=rows), 2.0 * (used * F * W + real * F) + 4.0 * real * W,
                     2.0 * real * F * W)
            if ops.grouped_tc_suits(xb, T * top, E, wgu, wd):      # many rows per expert: the TMA + tcgen05 kernel over 128-row tiles
                wide = ops.route_sort(ids, E, wide_tiles=True)
                by_bytes("experts_rows_in_sorted_order", lambda: ops.gather_rows(xb, wide.token_of), 4.0 * wide.n * W)
                xs = ops.gather_rows(xb, wide.token_of)
                by_bytes("experts_gate_up_tcgen05", lambda: ops.gemm_bf16_tc_grouped(xs, wgu, act, wide, ops.gated_epilogue_word("silu", None)),
                         2.0 * (used * 2 * F * W + real * (W + F)), 4.0 * real * F * W)
                by_bytes("experts_down_tcgen05", lambda: ops.gemm_bf16_tc_grouped(act, wd, y, wide), 2.0 * (used * F * W + real * F) + 4.0 * real * W,
                         2.0 * real * F * W)
            comb = torch.empty((T, W), device=dev)
            by_bytes("route_combine", lambda: ops.route_combine(y, xb, ids, weights, rows, comb), 4.0 * real * W + T * W * 6.0)
            Fd = top * F
            wgu_d, wd_d = b16(2 * Fd, W), b16(W, Fd)
            by_bytes("qwen2_dense_gate_up", lambda: ops.gated_linear(xb, wgu_d, "silu"), 2.0 * (2 * Fd * W + T * (W + Fd)), 4.0 * T * Fd * W)
            actd = b16(T, Fd)
            by_bytes("qwen2_dense_down", lambda: ops.linear(actd, wd_d, out_dtype=torch.float32), 2.0 * (Fd * W + T * Fd) + 4.0 * T * W, 2.0 * T * Fd * W)
            # the token input of a layer: the gate's activation times the token's table columns
            sd = z["side_dim"]
            zt, tab, g = f(T, sd), b16(z["vocab"], z["layers"] * sd), torch.empty((T, sd), dtype=torch.bfloat16, device=dev)
            by_bytes("token_table_gate", lambda: ops.gated_table_mul(zt, tab, sd, st.token_ids, g), T * sd * (4 + 2 + 2.0))
        return out

    sampler = ClockSampler()
    sampler.start()
    t0 = time.time()
    results = {}
    chosen = [n for n in GUVUSUN_SIZES if not args.sizes or n in args.sizes.split(",")]
    for name in chosen:
        z = GUVUSUN_SIZES[name]
        entry = {}
        model = random_model_on_device(GuvusunConfig.from_dict(guvusun_config(z)), seed=0, dtype="bfloat16", device="cuda:0")
        entry["guvusun"] = tools.run_model(model, z["vocab"])
        del model
        torch.cuda.empty_cache()
        qcfg = Qwen2Config(vocab_size=z["vocab"], hidden_size=z["width"], intermediate_size=z["top"] * z["ff"],
                           num_hidden_layers=z["layers"], num_attention_heads=z["heads"], num_key_value_heads=2,
                           head_dim=z["dim"] + z["rot_dim"], max_position_embeddings=32768, rms_norm_eps=1e-6, rope_theta=1e6,
                           tie_word_embeddings=False)
        model = random_model_on_device(qcfg, seed=0, dtype="bfloat16", device="cuda:0")
        entry["qwen2_equal_size"] = tools.run_model(model, z["vocab"])
        del model
        torch.cuda.empty_cache()
        if not args.no_kernels:
            entry["kernels"] = kernels(z)
        results[name] = entry
    clocks = ClockSampler.summary(sampler.window(t0, time.time()))
    sampler.stop()
    print(json.dumps({"workload": "guvusun", "dtype": "bf16", "data": "synthetic", "prefill_tokens": tokens, "decode_batch": batch,
                      "decode_context": context, "decode_steps": tools.steps, "peaks": pk, "clocks": clocks,
                      "l2": "flushed before each timed kernel", "gpu_launches": ops.total_launch_count(), "sizes": results}))
    return 0


# Sizes of --workload zegelix.  Layers in the proportion two recurrences : one window attention, a span of the stack run
# twice, routed experts with a shared expert in every layer.  Qwen2 beside each at equal width, as many layers as the design
# has layer RUNS, the same heads and head size, and a dense feed-forward of (top + shared) x expert size (the same active
# matrix rows per token).
ZEGELIX_SIZES = {
    "w2048": dict(width=2048, rwidth=2560, blocks=16, conv=4, heads=16, kv_heads=4, dim=128, window=1024, pool=32, experts=32, top=4,
                  ff=1024, shared=1024, vocab=32000, kinds="rra" "rra", loop=(0, 3, 2)),
    "w4096": dict(width=4096, rwidth=4096, blocks=16, conv=4, heads=32, kv_heads=8, dim=128, window=2048, pool=64, experts=64, top=6,
                  ff=1408, shared=2816, vocab=32000, kinds="rar", loop=(0, 3, 2)),
}


def zegelix_config(z):
    mlp = {"kind": "moe", "expert": {"ff": z["ff"], "limit": 7.0}, "router": {"experts": z["experts"], "top": z["top"]},
           "shared": {"ff": z["shared"], "limit": 7.0}}
    rec = {"type": "rglru", "mixer": {"width": z["rwidth"], "blocks": z["blocks"], "conv": z["conv"]}, "mlp": mlp}
    att = {"type": "attention", "mlp": mlp,
           "mixer": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"], "scale": z["dim"] ** -0.5,
                     "softcap": 50.0, "rot": {"dims": z["dim"], "base": 10000.0}, "mask": {"size": z["window"], "pool": z["pool"]}}}
    return {"architecture": "Zegelix", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "logit_scale": 1.0, "loop": {"start": z["loop"][0], "stop": z["loop"][1], "times": z["loop"][2]},
            "layers": [rec if c == "r" else att for c in z["kinds"]]}


def zegelix_workload(args) -> int:
    """Prefill and decode throughput of Zegelix and of Qwen2 at equal sizes through the step function, and the design's own
    kernels alone beside the like kernels of the other models, each with its share of the roofline.  One JSON line."""
    import numpy as np
    import torch

    from coheryn_ai_studio_b200 import ops
    from coheryn_ai_studio_b200.config import Qwen2Config
    from coheryn_ai_studio_b200.config.zegelix import ZegelixConfig
    from coheryn_ai_studio_b200.engine import random_model_on_device

    tools = model_bench_tools(args)
    pk, hbm, flops_peak, dev = tools.pk, tools.hbm, tools.flops_peak, tools.dev
    tokens, batch, context = tools.tokens, tools.batch, tools.context
    timed, step_like = tools.timed, tools.step_like
    fma_peak = 148 * 128 * 2 * 1.965e9        # float32 FMA lanes x 2 x the SM clock: what float32 arithmetic is bound by

    def kernels(z):
        out = {}
        H, G, d, W, C, page = z["heads"], z["kv_heads"], z["dim"], z["width"], z["rwidth"], args.page_size
        size, pool, bs, taps = z["window"], z["pool"], z["rwidth"] // z["blocks"], z["conv"]
        f = lambda *shape: torch.randn(shape, device=dev)
        b16 = lambda *shape: f(*shape).to(torch.bfloat16)
        for name, lengths, starts in (("prefill", [tokens], [0]), ("decode", [1] * batch, [context] * batch)):
            B, T = len(lengths), sum(lengths)
            per = -(-max(s + n for s, n in zip(starts, lengths)) // page)
            tables = torch.arange(B * per, dtype=torch.int32, device=dev).view(B, per)
            st = step_like(lengths, starts, tables)
            st.block_tables = [tables, tables]
            st.slots = [(tables[st.token_req.long(), (st.positions // page).long()] * page + st.positions % page).to(torch.int32)]
            rows = -(-page // pool)
            kc, vc = b16(B * per + 1, G, page, d), b16(B * per + 1, G, page, d)
            pkc, pvc = b16(B * per + 1, G, rows, d), b16(B * per + 1, G, rows, d)
            # keys a row meets: its window and the blocks behind it
            met = sum(min(p + 1, size) + max(0, (p - size + 1) // pool) for s, n in zip(starts, lengths) for p in range(s, s + n))
            met_window = sum(min(p + 1, size) for s, n in zip(starts, lengths) for p in range(s, s + n))
            held = sum(min(s + n, size + n) + (s + n) // pool for s, n in zip(starts, lengths))      # cached rows that are read

            def attention(label, fn, keys, rows_read):
                ms = timed(fn)
                fl = 2.0 * H * 2 * d * keys
                by = 4.0 * d * G * rows_read + 4.0 * T * H * d
                out[f"{name}.{label}"] = {"ms": round(ms, 4), "tflops": round(fl / ms / 1e9, 1),
                                          "of_bf16_peak": round(fl / (ms / 1e3) / flops_peak, 4), "of_hbm": round(by / (ms / 1e3) / hbm, 4)}
            q, o = b16(T, H * d), torch.empty((T, H * d), dtype=torch.bfloat16, device=dev)
            temps, sinks, gates = f(H).abs() + 0.5, f(H), f(T, H * d)
            fv = torch.stack([torch.pow(torch.tensor(10000.0), -2.0 * torch.arange(d // 2) / d), torch.zeros(d // 2)], dim=1).to(dev).contiguous()
            attention("window_and_blocks_attention", lambda: ops.pooled_attention(
                q, o, kc, vc, pkc, pvc, st, 0, 1, H, G, d, d, page, size, pool, d ** -0.5, 50.0, temps, sinks, gates, fv), met, held)
            attention("qwen2_attention_same_window", lambda: ops.attention_rows(
                q, o, kc, vc, tables, st.token_req, st.positions, H, G, d, page, size, d ** -0.5, cu_q=st.cu_q, kv_lens=st.kv_lens,
                q_lens=st.q_lens, max_kv_len=st.max_kv_len), met_window, sum(min(s + n, size + n) for s, n in zip(starts, lengths)))

            def by_bytes(label, fn, by, flops=None, peak=None):
                ms = timed(fn)
                out[f"{name}.{label}"] = {"ms": round(ms, 4), "of_hbm": round(by / (ms / 1e3) / hbm, 4)}
                if flops is not None:
                    out[f"{name}.{label}"]["of_flop_peak"] = round(flops / (ms / 1e3) / peak, 4)
            proj = f(T, (H + 2 * G) * d + H * d)
            fk = fv
            by_bytes("rotate_q_k_v_and_write_cache", lambda: ops.pooled_prepare(
                proj, st.positions, fk, d, fv, st.slots[0], kc, vc, H, G, d, d, page, torch.bfloat16), T * (H + 2 * G) * d * 6.0)
            from coheryn_ai_studio_b200.parts.base import Runtime
            from coheryn_ai_studio_b200.parts.position import RotateHalfRope
            rope = RotateHalfRope(Runtime(torch.bfloat16, dev), head_dim=d, rotary_dim=d, theta=10000.0, max_positions=context + tokens + 64)
            qkv = b16(T, (H + 2 * G) * d)
            by_bytes("qwen2_rotate_and_write_cache", lambda: ops.rope_kv_write(
                qkv, st.positions, rope.cos_sin(), st.slots[0], kc, vc, H, G, d, d, page), T * (H + 2 * G) * d * 4.0)
            by_bytes("block_means", lambda: ops.pooled_means(kc, vc, pkc, pvc, st, 0, 1, G, d, d, page, pool),
                     (T // pool + B) * pool * 2 * G * d * 2.0)
            # the recurrence: convolution, the gates' block-diagonal products (float32 FMA), the scan
            state = torch.zeros((B, C * taps), dtype=torch.float32, device=dev)
            x, u, y = f(T, C), f(T, C), f(T, C)
            conv_w, conv_b = f(C, taps), f(C)
            by_bytes("conv_with_bias", lambda: ops.conv_bias(x, conv_w, conv_b, state[:, C:], st), T * C * 8.0)
            from coheryn_ai_studio_b200 import ops as _ops
            by_bytes("tutunex_conv_silu", lambda: _ops.short_conv_silu(x, conv_w, state[:, C:], st), T * C * 8.0)
            wg, gts = f(z["blocks"], 2 * bs, bs), torch.empty((T, 2 * C), dtype=torch.float32, device=dev)
            by_bytes("gates_float32_fma", lambda: ops.grouped_linear(u, wg, gts, a_col=bs, c_col=2 * bs),
                     T * C * 12.0 + wg.numel() * 4.0, flops=2.0 * T * 2 * C * bs, peak=fma_peak)
            lam, br, bi = f(C) - 4.0, f(C), f(C)
            so = torch.empty((T, C), dtype=torch.bfloat16, device=dev)
            by_bytes("gated_scan", lambda: ops.gated_scan(gts, br, bi, u, y, lam, 8.0, bs, state[:, :C], st, so),
                     T * C * (2 * 12.0 + 4.0 + 2.0))
            xs, table = f(T, W), b16(z["vocab"], W)
            st.token_ids = torch.randint(0, z["vocab"], (T,), dtype=torch.int32, device=dev)
            by_bytes("stream_beside_embedding", lambda: ops.stream_join(xs, None, table, st.token_ids, 1.0, torch.bfloat16), T * W * 10.0)
        return out

    sampler = ClockSampler()
    sampler.start()
    t0 = time.time()
    results = {}
    chosen = [n for n in ZEGELIX_SIZES if not args.sizes or n in args.sizes.split(",")]
    for name in chosen:
        z = ZEGELIX_SIZES[name]
        entry = {}
        cfg = ZegelixConfig.from_dict(zegelix_config(z))
        model = random_model_on_device(cfg, seed=0, dtype="bfloat16", device="cuda:0")
        runs = len(model.spec.schedule)
        entry["zegelix"] = tools.run_model(model, z["vocab"])
        del model
        torch.cuda.empty_cache()
        qcfg = Qwen2Config(vocab_size=z["vocab"], hidden_size=z["width"], intermediate_size=z["top"] * z["ff"] + z["shared"],
                           num_hidden_layers=runs, num_attention_heads=z["heads"], num_key_value_heads=z["kv_heads"],
                           head_dim=z["dim"], max_position_embeddings=32768, rms_norm_eps=1e-6, rope_theta=1e6,
                           tie_word_embeddings=False)
        model = random_model_on_device(qcfg, seed=0, dtype="bfloat16", device="cuda:0")
        entry["qwen2_equal_size"] = tools.run_model(model, z["vocab"])
        entry["layer_runs"] = runs
        del model
        torch.cuda.empty_cache()
        if not args.no_kernels:
            entry["kernels"] = kernels(z)
        results[name] = entry
    clocks = ClockSampler.summary(sampler.window(t0, time.time()))
    sampler.stop()
    print(json.dumps({"workload": "zegelix", "dtype": "bf16", "data": "synthetic", "prefill_tokens": tokens, "decode_batch": batch,
                      "decode_context": context, "decode_steps": tools.steps, "peaks": pk, "clocks": clocks,
                      "l2": "flushed before each timed kernel", "gpu_launches": ops.total_launch_count(), "sizes": results}))
    return 0


def timeline(args, make_engine, StepEntry, ops, torch) -> int:
    """Where a decode step's time goes, kernel by kernel, measured inside graph-replayed steps (the
    kernels overlap through programmatic dependent launch, so a kernel's own duration says little):
    ``advance`` is how far a kernel's end lies behind the end of everything before it; the advances
    add up to the step."""
    import collections
    from torch.profiler import ProfilerActivity, profile
    eng, lens, rng = make_engine(args.batch)
    ids = [f"t{i}" for i in range(args.batch)]
    for rid, n in zip(ids, lens):
        assert eng.cache.admit(rid) is not None and eng.cache.reserve(rid, [0] * n)
        eng.cache.commit(rid)
    out = torch.empty(args.batch, dtype=torch.int32, device="cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")

    def one():
        logits = eng.runner.step([StepEntry(rid, [5], [0]) for rid in ids])
        ops.argmax(logits, out, status)
    for _ in range(max(args.warmup, 4)):
        one()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(4):
            one()
        torch.cuda.synchronize()
    events = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA
              and "emcpy" not in e.name and "emset" not in e.name]
    events.sort(key=lambda e: e.time_range.start)
    first = [i for i, e in enumerate(events) if "embed_gather" in e.name][-1]
    step = events[first:]
    t0 = prev_end = step[0].time_range.start
    rows = collections.OrderedDict()
    for e in step:
        start, end = e.time_range.start, e.time_range.end
        name = e.name.replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0]
        r = rows.setdefault(name, [0, 0.0, 0.0])
        r[0] += 1
        r[1] += end - start
        r[2] += max(0.0, end - prev_end)
        prev_end = max(prev_end, end)
    print(f"decode step, batch {args.batch}, {args.layers} layers: {prev_end - t0:.1f} us from the first kernel's start to the last one's end")
    print(f"{'launches':>8} {'duration us':>12} {'advance us':>11} {'step share':>10}  kernel")
    for name, (n, dur, adv) in rows.items():
        print(f"{n:8d} {dur / n:12.2f} {adv / n:11.2f} {adv / (prev_end - t0):10.3f}  {name}")
    if args.timeline_raw:
        # every kernel of the step with its own start and end, relative to the step's start
        print(f"{'start us':>9} {'end us':>9}  kernel")
        for e in step:
            name = e.name.replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0]
            print(f"{e.time_range.start - t0:9.1f} {e.time_range.end - t0:9.1f}  {name}")
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=SIZES["num_hidden_layers"],
                    help="fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--skip-points", action="store_true", help="skip the batch 1 / 64 points")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--workload", default="decode", choices=["decode", "serving-7b", "long-14b", "chat-1.5b", "kapudra", "tutunex", "guvusun", "zegelix"],
                    help="decode: the contract's line (default); the others: see the header")
    ap.add_argument("--sizes", default="", help="--workload kapudra / tutunex / guvusun / zegelix: which of its sizes (comma separated; default all)")
    ap.add_argument("--no-kernels", action="store_true", help="--workload guvusun / zegelix: the models only, not the kernels alone")
    ap.add_argument("--timeline-raw", action="store_true", help="with --timeline: also every kernel's start and end")
    ap.add_argument("--timeline", action="store_true",
                    help="instead of the benchmark: the kernels of one graph-replayed decode step with their times "
                         "inside the step (CUPTI through torch.profiler), one text line per kernel")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust workspace (no setup.py/pyproject.toml, pip reports "
                          "'not installable') and this image has no cargo/rustc; it is CPU-only"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.workload == "kapudra":
        return kapudra_workload(args)
    if args.workload == "tutunex":
        return tutunex_workload(args)
    if args.workload == "guvusun":
        return guvusun_workload(args)
    if args.workload == "zegelix":
        return zegelix_workload(args)
    if args.workload != "decode":
        return other_workload(args)

    import numpy as np
    import torch

    from coheryn_ai_studio_b200 import ops
    from coheryn_ai_studio_b200.config import Qwen2Config
    from coheryn_ai_studio_b200.engine import Engine, StepEntry, random_model_on_device
    from coheryn_ai_studio_b200.engine.scheduler import Request
    from coheryn_ai_studio_b200.sampling import RequestSampler, SamplingParams

    pk = peaks()
    sizes = dict(SIZES, num_hidden_layers=args.layers)
    cfg = Qwen2Config(**sizes)
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    model = random_model_on_device(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    V, H, I, L = cfg.vocab_size, cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers
    nh, nkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    layer_params = (nh + 2 * nkv) * hd * H + H * nh * hd + 3 * H * I
    weight_bytes = 2 * (L * layer_params + V * H) + 2 * L * ((nh + 2 * nkv) * hd + 2 * H) + 4 * H
    kv_bytes_per_token = 2 * L * nkv * hd * 2
    total_steps = args.warmup + args.steps

    sampler = ClockSampler()
    sampler.start()

    def make_engine(batch, context=None):
        margin = 2 * total_steps + 8
        context = context or args.context
        eng = Engine(model, dtype="bfloat16", context=context, max_num_seqs=batch,
                     max_num_batched_tokens=max(2048, args.prefill_tokens), page_size=args.page_size,
                     kv_cache_tokens=batch * (context + 64), prefix_reuse=False,
                     use_graphs=not args.no_graphs)
        for g in eng.cache.groups:
            g.tensor.normal_(0.0, 1.0)
        rng = np.random.default_rng(1234 + batch)
        lens = np.minimum(rng.integers(512, args.context + 1, size=batch), args.context - margin)
        return eng, [int(x) for x in lens], rng

    def inject(eng, lens, rng):
        """Requests that have 'run' their prompts: pages reserved and committed, contents
        random.  Returns the Request objects (already in the scheduler's running list)."""
        reqs = []
        for i, n in enumerate(lens):
            prompt = rng.integers(0, V, size=n).tolist()
            req = Request(f"bench-{i}", prompt, max_tokens=min(4 * total_steps + 64, args.context - n), params=SamplingParams())
            req.sampler = RequestSampler(req.params)
            req.arrival = i
            assert eng.cache.admit(req.request_id) is not None
            assert eng.cache.reserve(req.request_id, prompt[:-1])
            eng.cache.commit(req.request_id)
            eng.scheduler.adopt_running(req, n - 1)
            eng._requests[req.request_id] = req
            from coheryn_ai_studio_b200.engine.engine import _Timing
            eng._timing[req.request_id] = _Timing(time.perf_counter())
            reqs.append(req)
        return reqs

    def decode_device_timed(batch, steps, warmup):
        """K decode steps back to back, timed on the device."""
        eng, lens, rng = make_engine(batch)
        ids = [f"d{i}" for i in range(batch)]
        for rid, n in zip(ids, lens):
            assert eng.cache.admit(rid) is not None
            assert eng.cache.reserve(rid, [0] * n)
            eng.cache.commit(rid)
        out = torch.empty(batch, dtype=torch.int32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        toks = rng.integers(0, V, size=(warmup + steps, batch))

        def one(k):
            logits = eng.runner.step([StepEntry(rid, [int(toks[k, b])], [0]) for b, rid in enumerate(ids)])
            ops.argmax(logits, out, status)
        for k in range(warmup):
            one(k)
        torch.cuda.synchronize()
        l0 = ops.total_launch_count() + eng.runner.graph_launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        e0.record()
        for k in range(warmup, warmup + steps):
            one(k)
        e1.record()
        torch.cuda.synchronize()
        t1 = time.time()
        ms = e0.elapsed_time(e1)
        eng.runner.check_status()          # a kernel that gave up a wait would have timed garbage
        launches = ops.total_launch_count() + eng.runner.graph_launches - l0
        mean_ctx = float(np.mean(lens)) + warmup + steps / 2
        step_bytes = weight_bytes + batch * mean_ctx * kv_bytes_per_token
        del eng
        torch.cuda.empty_cache()
        return {"tok_s": batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "launches": launches,
                "bytes_per_step": step_bytes, "window": (t0, t1), "mean_ctx": mean_ctx}

    def decode_end_to_end(batch, steps, warmup):
        eng, lens, rng = make_engine(batch)
        inject(eng, lens, rng)
        for _ in range(warmup):
            eng.step()
        torch.cuda.synchronize()
        h2d = d2h = 0
        t0 = time.perf_counter()
        for _ in range(steps):
            events = eng.step()
            h2d += eng.runner.h2d_bytes
            d2h += 4 * len(events) + 8        # sampled ids and the two status words
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        del eng
        torch.cuda.empty_cache()
        return {"value": batch * steps / dt, "unit": "tok/s", "h2d_bytes_per_step": h2d // steps,
                "d2h_bytes_per_step": d2h // steps, "ms_per_step": dt / steps * 1e3}

    def prefill_timed(tokens, repeats=3):
        eng, _, rng = make_engine(1, max(args.context, tokens + 64))   # a context shorter than the prompt: room for it
        best = None
        for r in range(repeats + 1):            # the first run is the warm-up
            rid = f"p{r}"
            prompt = rng.integers(0, V, size=tokens).tolist()
            eng.cache.admit(rid)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            eng.runner.step([StepEntry(rid, prompt, [tokens - 1])])
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            eng.runner.check_status()
            eng.cache.free(rid)
            if r > 0:
                best = ms if best is None else min(best, ms)
        # What the step computes: every layer in full but the last, which projects q/k/v for all
        # tokens (their keys and values go to the cache) and runs the rest for the one wanted row.
        full = 2.0 * tokens * layer_params + 4.0 * nh * hd * tokens * (tokens + 1) / 2
        last = (2.0 * tokens * (nh + 2 * nkv) * hd * H + 2.0 * (H * nh * hd + 3 * H * I) + 4.0 * nh * hd * tokens
                if eng.runner.tail_shortcut else full)
        flops = (L - 1) * full + last + 2.0 * V * H
        peak = pk.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]) * 1e12
        del eng
        torch.cuda.empty_cache()
        return {"value": tokens / (best / 1e3), "tokens": tokens, "ms": best, "frac": flops / (best / 1e3) / peak,
                "tflops": flops / (best / 1e3) / 1e12}

    if args.timeline:
        sampler.stop()
        return timeline(args, make_engine, StepEntry, ops, torch)

    main_run = decode_device_timed(args.batch, args.steps, args.warmup)
    clocks = ClockSampler.summary(sampler.window(*main_run["window"]))
    e2e = decode_end_to_end(args.batch, args.steps, args.warmup)
    prefill = prefill_timed(args.prefill_tokens)
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            r = decode_device_timed(b, max(16, args.steps // 2), args.warmup)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
            points[f"decode_b{b}_hbm_frac"] = round(r["bytes_per_step"] / (r["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"], 4)
    sampler.stop()

    achieved = main_run["bytes_per_step"] / (main_run["ms_per_step"] / 1e3) / 1e9
    line = {
        "metric": "decode_tokens_per_s", "value": round(main_run["tok_s"], 1), "unit": "tok/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {
            "model": "Qwen2.5-1.5B layer sizes, random weights", "global_batch": args.batch,
            "seq_len": args.context, "parallelism": "single-gpu", "layers": L,
            "layers_of_config": SIZES["num_hidden_layers"], "hidden": H, "heads": nh, "kv_heads": nkv,
            "head_dim": hd, "intermediate": I, "vocab": V, "tied_embeddings": True,
            "context_per_request": f"uniform[512,{args.context}]", "mean_context": round(main_run["mean_ctx"], 1),
            "page_size": args.page_size, "cuda_graphs": not args.no_graphs,
            "l2": "weights+cache per step exceed L2 (126 MB)", "peaks": pk["source"],
        },
        "e2e": {k: (round(v, 2) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": int(main_run["launches"]),
        "clocks": clocks,
        "prefill": {"value": round(prefill["value"], 1), "tokens": prefill["tokens"], "ms": round(prefill["ms"], 3),
                    "frac": round(prefill["frac"], 4), "tflops": round(prefill["tflops"], 1)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
