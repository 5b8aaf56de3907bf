#!/usr/bin/env python3
"""Decode and prefill speed of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--model a2.7b|57b] [--layers L] [--batch B]
                    [--impl reference]

The model has the layer sizes of Qwen1.5-MoE-A2.7B (default) or of Qwen2-57B-A14B (--model 57b) with seeded
random weights in bfloat16; token ids are synthetic (uniform).  A "step" is one decode step of a batch of 8
sequences that start from 2,048-token prompts (cache for 4,096 each).  One JSON line is printed:
  value     decoded tokens per second, timed on the device with CUDA events over exactly K steps
            (every step reads far more weight and cache bytes than the L2 holds, so no flush)
  e2e       the same through the Python entry point (Model.generate_batch): host token ids in,
            host token ids out, every step's host-to-device and device-to-host copies included
  prefill   one 2,048-token prompt: tokens per second, milliseconds, fraction of the bf16 peak
  roofline  bytes the decode step has to read (each weight it uses once, and the cache of the live
            requests) / its time, against the measured copy bandwidth
  points    decode tokens per second at batch 1 and batch 64 from 2,048-token prompts, and at batch 1, 8 and 64
            with the context at 4,096 by the last timed step; points_frac: each point's fraction of the roofline
  vs_baseline  against the reference's own CPU forward, timed once on this architecture's sizes (`baseline` says how):
            the reference has no GPU path, no batch and no prompt step for it, so this is context, not a race
Only one GPU is supported: for --gpus N > 1 a line says so and the exit code is 2.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Layer sizes of the benchmark model (Qwen1.5-MoE-A2.7B); weights are random.
A27B = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "num_hidden_layers": 24, "hidden_size": 2048, "num_attention_heads": 16, "num_key_value_heads": 16,
    "num_experts": 60, "num_experts_per_tok": 4, "moe_intermediate_size": 1408, "norm_topk_prob": False,
    "shared_expert_intermediate_size": 5632, "intermediate_size": 5632, "vocab_size": 151936,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 8192, "use_sliding_window": False,
    "sliding_window": 0, "max_window_layers": 24, "tie_word_embeddings": False, "decoder_sparse_step": 1,
    "mlp_only_layers": [], "hidden_act": "silu", "torch_dtype": "bfloat16",
}
# Layer sizes of Qwen2-57B-A14B.
B57 = dict(A27B, num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, num_experts=64,
           num_experts_per_tok=8, moe_intermediate_size=2560, shared_expert_intermediate_size=20480,
           intermediate_size=20480, max_position_embeddings=32768, max_window_layers=28)
MODELS = {"a2.7b": ("Qwen1.5-MoE-A2.7B sizes", A27B), "57b": ("Qwen2-57B-A14B sizes", B57)}
PROMPT, CONTEXT = 2048, 4096


def reference_cpu_rate(layers):
    """Tokens per second of the reference's own CPU forward at Qwen1.5-MoE-A2.7B sizes with `layers` layers, from
    the committed record of one timed run on 1 and 2 layers (tests/golden/reference_cpu_timing.txt, made by
    tests/golden/time_reference.sh): head and embedding once, the layer's cost times the number of layers."""
    try:
        ms = {}
        for line in open(os.path.join(ROOT, "tests", "golden", "reference_cpu_timing.txt")):
            f = line.split()
            if f and f[0] == "layers":
                ms[int(f[1])] = float(f[5])
        layer = ms[2] - ms[1]
        return 1e3 / (ms[1] - layer + layers * layer), ms
    except (OSError, KeyError, ValueError, IndexError):
        return None, {}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            d = json.load(open(p))
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d.get("bf16_tflops", 1590.0)), "source": "measured"}
        except Exception:  # noqa: BLE001 - fall through to the stated fallback
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "--id=0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = max((int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()), default=0)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i].lower() == "active" for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else 0, "sm_max_mhz": mx, "reasons": reasons, "samples": len(sm)}


def model_numbers(cfg, layers):
    """Parameter and flop counts from the configuration."""
    H, nh, nkv = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = H // nh
    E, k, I, S, V = (cfg["num_experts"], cfg["num_experts_per_tok"], cfg["moe_intermediate_size"],
                     cfg["shared_expert_intermediate_size"], cfg["vocab_size"])
    attn = H * (nh + 2 * nkv) * hd + (nh + 2 * nkv) * hd + nh * hd * H
    expert = 3 * H * I
    shared = 3 * H * S + H
    router = E * H
    return dict(attn=attn, expert=expert, shared=shared, router=router, norms=2 * H, head=V * H, embed=V * H,
                layers=layers, kv_per_token=layers * 2 * nkv * hd, H=H, E=E, k=k, V=V, nh=nh, hd=hd)


def decode_bytes(n, distinct_experts_per_layer, batch, context_tokens_total, el=2):
    """Bytes one decode step has to read: every weight it uses once and the live requests' cache."""
    per_layer = n["attn"] + n["shared"] + n["router"] + n["norms"]
    w = n["layers"] * per_layer + sum(distinct_experts_per_layer) * n["expert"] + n["head"] + batch * n["H"] + n["H"]
    return w * el + context_tokens_total * n["kv_per_token"] * el


def prefill_flops(n, T):
    per_tok = 2 * (n["attn"] + n["k"] * n["expert"] + n["shared"] + n["router"])
    attn = 4 * n["nh"] * n["hd"] * T * (T + 1) / 2
    return n["layers"] * (T * per_tok + attn) + 2 * n["head"]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--model", choices=sorted(MODELS), default="a2.7b")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16",
                    help="float32: the true 32-bit path of the whole model (exact kernels, SGEMM without TF32)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the prefill")
    ap.add_argument("--kernel-table", default="", help="write a per-kernel time table of a few decode steps and of a "
                    "prefill to this file (torch profiler; not part of any timed number)")
    ap.add_argument("--design", choices=["nuforax", "lumevik", "sisepel", "tasadra"], default="", help="instead of the default workload: prompt "
                    "and decode speed of this design at layer sizes of a real model (random weights), beside the closest other "
                    "decoder of equal width, depth and heads")
    ap.add_argument("--sizes", default="w1024,w2048", help="with --design: which of the sizes to run")
    args = ap.parse_args()
    if args.design and args.impl != "reference":
        return design_compare(args)
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a C project without setup.py/pyproject.toml at its root (pip install fails), "
                          "and its engine runs this architecture from GGUF on the CPU only: no safetensors MoE, no "
                          "random-weights mode, no CUDA forward"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": f"this library runs on one GPU; --gpus {args.gpus} is not supported", "n_gpus": args.gpus}))
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import numpy as np
    import torch
    import turboquant_cpp_b200 as tq
    from turboquant_cpp_b200.kernels import _call

    pk = peaks()
    model_name, cfg = MODELS[args.model]
    cfg = dict(cfg)
    FULL_LAYERS = cfg["num_hidden_layers"]
    args.layers = args.layers or FULL_LAYERS
    cfg["num_hidden_layers"] = args.layers
    cfg["max_window_layers"] = args.layers
    n = model_numbers(cfg, args.layers)
    torch.cuda.set_device(0)
    t_load = time.time()
    EL = 2 if args.dtype == "bfloat16" else 4                 # bytes per weight and per cached value
    model = tq.random_model(cfg, seed=0, dtype=args.dtype, device="cuda:0")
    torch.cuda.synchronize()
    print(f"[bench] model with {args.layers} layers ready in {time.time() - t_load:.1f} s", file=sys.stderr, flush=True)
    rng = np.random.default_rng(0)
    V = cfg["vocab_size"]

    def run_decode(batch, steps, warmup, want_experts=False, prompt=PROMPT):
        """Prefill `batch` prompts of `prompt` tokens, then time `steps` decode steps on the device."""
        eng = tq.Engine(model, max_tokens=batch * CONTEXT, max_slots=batch)
        seqs = [eng.open() for _ in range(batch)]
        group = 8
        for g0 in range(0, batch, group):
            eng.step([tq.StepEntry(s, rng.integers(0, V, size=prompt).tolist(), []) for s in seqs[g0:g0 + group]])
        smp = tq.Sampler(0.0)
        toks = rng.integers(0, V, size=(warmup + steps + 1, batch))

        def one(i):
            logits = eng.step([tq.StepEntry(s, [int(toks[i, j])], [0]) for j, s in enumerate(seqs)])
            return smp.sample(logits, list(range(batch)), [i] * batch)

        distinct = None
        if want_experts:
            eng.debug = {}
            one(0)
            distinct = [int(torch.unique(a).numel()) for a in eng.debug["router_ids"]]
            eng.debug = None
        else:
            one(0)
        for i in range(1, warmup):
            one(i)
        ctx_tokens = sum(s.length for s in seqs)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = _call.LAUNCHES
        torch.cuda.synchronize()
        a.record()
        for i in range(warmup, warmup + steps):
            one(i)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        launches = _call.LAUNCHES - launches0
        ctx_mid = ctx_tokens + batch * steps // 2
        for s in seqs:
            eng.close(s)
        eng.release()             # the engine's graphs point back at it: without this its cache would stay until a collection
        del eng
        gc.collect()
        torch.cuda.empty_cache()
        return dict(ms_per_step=ms / steps, tok_s=batch * steps / ms * 1e3, launches=launches, distinct=distinct,
                    ctx_tokens=ctx_mid)

    # ---- the headline: decode at the default batch ------------------------------------------------
    clocks = ClockSampler()
    clocks.start()
    main_run = run_decode(args.batch, args.steps, args.warmup, want_experts=True)
    clock_rec = clocks.stop()
    dbytes = decode_bytes(n, main_run["distinct"], args.batch, main_run["ctx_tokens"], EL)
    achieved = dbytes / (main_run["ms_per_step"] * 1e-3) / 1e9

    # ---- end to end through the Python entry point ---------------------------------------------------
    m = tq.Model.from_model(model, temperature=0.0, max_tokens=args.steps + 1, context_length=CONTEXT, max_batch=args.batch)
    prompts = [rng.integers(0, V, size=PROMPT).tolist() for _ in range(args.batch)]
    m.generate_batch([p[:64] for p in prompts], max_tokens=4)          # warm-up
    m.generate_batch(prompts)
    st = m.last_stats
    e2e_tok_s = (st.generated_tokens - args.batch) / st.decode_seconds if st.decode_seconds > 0 else 0.0
    h2d = 4 * (7 * args.batch + 1 + args.batch * (CONTEXT // 64))       # packed int32 metadata of a decode step
    d2h = 4 * args.batch
    m.close()

    ref_rate, ref_ms = reference_cpu_rate(args.layers) if args.model == "a2.7b" else (None, {})
    out = {
        "metric": f"decode tok/s @ batch {args.batch} ({model_name}, random weights)", "value": round(main_run["tok_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(main_run["tok_s"] / ref_rate, 1) if ref_rate else None,
        "baseline": ({"value": round(ref_rate, 4), "unit": "tokens/s", "what": "the reference's own forward (tq_forward) on a CPU, "
                      "float32, one token of one sequence at a time: it has no GPU path, no batch and no prompt step for "
                      "this architecture; timed on 1 and 2 layers of these sizes and scaled to this run's layers "
                      "(tests/golden/reference_cpu_timing.txt); other hardware, so context, not a race",
                      "ms_per_token_1_layer": ref_ms.get(1), "ms_per_token_2_layers": ref_ms.get(2)} if ref_rate else None),
        "dtype": "bf16" if args.dtype == "bfloat16" else "fp32", "data": "synthetic token ids, seeded random weights", "impl": "ours",
        "config": {"model": model_name, "layers": args.layers, "layers_of_model": FULL_LAYERS,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["hidden_size"] // cfg["num_attention_heads"], "experts": cfg["num_experts"],
                   "top_k": cfg["num_experts_per_tok"], "moe_inter": cfg["moe_intermediate_size"],
                   "shared_inter": cfg["shared_expert_intermediate_size"], "vocab": V, "global_batch": args.batch,
                   "seq_len": CONTEXT, "prompt_len": PROMPT, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (weights and cache read per step)"},
        "clocks": clock_rec,
        "e2e": {"value": round(e2e_tok_s, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": main_run["launches"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peak_source": pk["source"],
                     "bytes_per_step": int(dbytes)},
    }
    if not args.no_points:
        # ---- prefill of one 2,048-token prompt --------------------------------------------------------
        eng = tq.Engine(model, max_tokens=PROMPT, max_slots=1)
        toks = rng.integers(0, V, size=PROMPT).tolist()
        best = float("inf")
        for i in range(4):
            s = eng.open()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            eng.step([tq.StepEntry(s, toks, [PROMPT - 1])])
            b.record()
            torch.cuda.synchronize()
            if i > 0:
                best = min(best, a.elapsed_time(b))
            eng.close(s)
        eng.release()
        del eng
        gc.collect()
        torch.cuda.empty_cache()
        fl = prefill_flops(n, PROMPT)
        out["prefill"] = {"value": round(PROMPT / best * 1e3, 1), "tokens": PROMPT, "ms": round(best, 3),
                          # (no measured peak for float32 products without TF32: no fraction there)
                          "frac": round(fl / (best * 1e-3) / (pk["bf16_tflops"] * 1e12), 4) if EL == 2 else None}
        k_pts = max(8, min(args.steps, 32))
        out["points"], out["points_frac"] = {}, {}
        # from 2,048-token prompts, and with the context at 4,096 by the last timed step
        for name, batch, prompt in (("decode_b1", 1, PROMPT), ("decode_b64", 64, PROMPT),
                                    ("decode_b1_ctx4096", 1, CONTEXT - k_pts - 3), ("decode_b8_ctx4096", 8, CONTEXT - k_pts - 3),
                                    ("decode_b64_ctx4096", 64, CONTEXT - k_pts - 3)):
            r = run_decode(batch, k_pts, 3, want_experts=True, prompt=prompt)
            by = decode_bytes(n, r["distinct"], batch, r["ctx_tokens"], EL)
            out["points"][name] = round(r["tok_s"], 1)
            out["points_frac"][name] = round(by / (r["ms_per_step"] * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
    if args.kernel_table:
        kernel_table(tq, model, rng, V, args.batch, args.kernel_table)
    print(json.dumps(out))
    return 0


# ---- another design beside the closest existing model ------------------------------------------------------------
def nuforax_config(width, layers, heads, dim, rot, vdim, rank, window, ff, m_heads, m_vdim, m_state, m_groups, vocab):
    """Layers in threes: latent attention, latent attention reading the first one's rows, state-space mixer."""
    rot_cfg = {"base": 1000000.0, "dims": rot, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}
    att = lambda src: {"type": "latent_attention", "mlp": {"kind": "dense", "ff": ff}, "mixer": dict(
        {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank, "scale": (dim + rot) ** -0.5,
         "mask": {"size": window}, "rot": rot_cfg}, **({} if src is None else {"kv_from": src}))}
    ssm = {"type": "mamba2", "mlp": None, "mixer": {"heads": m_heads, "vdim": m_vdim, "state": m_state, "groups": m_groups,
                                                    "conv": 4, "norm_groups": m_groups}}
    out = []
    for i in range(layers):
        out.append(att(None) if i % 3 == 0 else att(i - 1) if i % 3 == 1 else ssm)
    return {"architecture": "Nuforax", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "embedding": {"scale": 1.0, "bigram": {"buckets": 65521, "mul_prev": 31, "mul_cur": 7}}, "layers": out}


def dense_qwen2_config(width, layers, heads, window, inter, vocab):
    return dict(A27B, num_hidden_layers=layers, hidden_size=width, num_attention_heads=heads, num_key_value_heads=max(1, heads // 4),
                head_dim=128, num_experts=0, num_experts_per_tok=0, moe_intermediate_size=0, shared_expert_intermediate_size=0,
                intermediate_size=inter, vocab_size=vocab, use_sliding_window=True, sliding_window=window, max_window_layers=0,
                max_position_embeddings=8192, tie_word_embeddings=True)


def lumevik_config(width, layers, heads, kv_heads, dim, window, keep_first, rank, q_rank, ff, experts, top, e_ff, s_ff, vocab):
    """Layers in pairs: latent attention with a dense feed-forward, then windowed attention with routed experts."""
    lat = {"type": "latent_attention", "mlp": {"kind": "dense", "ff": ff, "limit": 7.0},
           "mixer": {"heads": heads, "dim": dim, "vdim": dim, "kv_rank": rank, "q_rank": q_rank, "scale": dim ** -0.5}}
    att = {"type": "attention",
           "mlp": {"kind": "moe", "expert": {"ff": e_ff, "limit": 7.0}, "shared": {"ff": s_ff, "limit": 7.0},
                   "router": {"experts": experts, "top": top, "groups": {"count": 4, "keep": 2}}},
           "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "bias_max": 2048,
                     "bias_rows": 32, "mask": {"size": window, "keep_first": keep_first}, "v_mix": True}}
    return {"architecture": "Lumevik", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "layers": [lat if i % 2 == 0 else att for i in range(layers)]}


def sparse_qwen2_config(width, layers, heads, kv_heads, dim, window, ff, experts, top, e_ff, s_ff, vocab):
    """The Qwen2 MoE decoder with the same widths: dense feed-forwards on the even layers, experts on the odd ones,
    a window on every layer."""
    return dict(A27B, num_hidden_layers=layers, hidden_size=width, num_attention_heads=heads, num_key_value_heads=kv_heads,
                head_dim=dim, num_experts=experts, num_experts_per_tok=top, moe_intermediate_size=e_ff,
                shared_expert_intermediate_size=s_ff, intermediate_size=ff, vocab_size=vocab, use_sliding_window=True,
                sliding_window=window, max_window_layers=0, max_position_embeddings=8192, tie_word_embeddings=False,
                decoder_sparse_step=1, mlp_only_layers=list(range(0, layers, 2)), norm_topk_prob=True)


LUMEVIK_SIZES = {
    # name: (width, layers, heads, kv heads, head size, window, kept first, kv_rank, q_rank, dense ff, experts, top, expert ff,
    #        shared ff, vocab)
    "w1024": (1024, 4, 8, 2, 128, 1024, 4, 256, 384, 2816, 32, 4, 704, 2816, 32768),
    "w2048": (2048, 4, 16, 4, 128, 1024, 4, 512, 768, 5632, 60, 4, 1408, 5632, 32768),
}

def sisepel_config(width, layers, heads, kv_heads, dim, window, r_heads, r_dim, r_vdim, ff, experts, top, e_ff, s_ff, side, vocab):
    """Layers in pairs: a dense feed-forward, then routed experts; every layer has windowed attention and retention
    side by side and a token input of its own."""
    mixer = {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "softcap": 50.0,
                      "mask": {"size": window},
                      "rot": {"base": 500000.0, "dims": dim // 2, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}},
             "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "rot": {"base": 10000.0, "dims": r_dim},
                       "decay": [1.0 - 2.0 ** (-4.0 - 5.0 * i / max(1, r_heads - 1)) for i in range(r_heads)]}}
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "expert": {"ff": e_ff}, "shared": {"ff": s_ff}, "router": {"experts": experts, "top": top}}
    return {"architecture": "Sisepel", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "logit_scale": 0.25,
            "token_side": {"dim": side},
            "layers": [{"type": "parallel", "mixer": mixer, "mlp": dense if i % 2 == 0 else moe} for i in range(layers)]}


SISEPEL_SIZES = {
    # name: Lumevik's sizes of that name (width, layers, heads, kv heads, head size, window, experts and feed-forwards, vocab)
    # and, for the parts Lumevik does not have: (retention heads, key size, value size, width of a layer's token input)
    "w1024": (8, 64, 128, 64),
    "w2048": (16, 128, 128, 128),
}

DESIGN_SIZES = {
    # name: (width, layers, heads, dim, rot, vdim, rank, window, ff, ssm heads, ssm vdim, ssm state, ssm groups, vocab)
    "w1024": (1024, 6, 8, 64, 64, 64, 256, 1024, 4096, 32, 64, 64, 1, 32768),
    "w2048": (2048, 6, 16, 128, 64, 128, 512, 1024, 8192, 64, 64, 128, 8, 32768),
}


def design_compare(args) -> int:
    """Prompt and decode speed of the Nuforax decoder and of the dense Qwen2 decoder of equal width, depth, heads and
    window (its feed-forward sized to the same number of weights), timed on the device with CUDA events."""
    import numpy as np
    import torch
    import turboquant_cpp_b200 as tq
    from turboquant_cpp_b200.kernels import _call
    if args.gpus != 1:
        print(json.dumps({"error": "one GPU only", "n_gpus": args.gpus}))
        return 2
    pk = peaks()
    rng = np.random.default_rng(0)
    steps, warmup = max(8, min(args.steps, 32)), max(3, args.warmup)
    prompt = 2048

    def weights_bytes(model):
        seen, total = set(), 0
        for spec in model.weight_specs():
            if spec.name not in seen:
                seen.add(spec.name)
                n = 1
                for d in spec.shape:
                    n *= d
                total += 2 * n
        return total

    def measure(model, V):
        out = {"weights_gb": round(weights_bytes(model) / 1e9, 3)}
        eng = tq.Engine(model, max_tokens=prompt + 64, max_slots=1)
        toks = rng.integers(0, V, size=prompt).tolist()
        best = float("inf")
        for i in range(4):
            s = eng.open()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            eng.step([tq.StepEntry(s, toks, [prompt - 1])])
            b.record()
            torch.cuda.synchronize()
            if i > 0:
                best = min(best, a.elapsed_time(b))
            eng.close(s)
        eng.release()
        out["prefill_2048"] = {"ms": round(best, 3), "tokens_per_s": round(prompt / best * 1e3, 1)}
        for batch in (1, 8, 64):
            eng = tq.Engine(model, max_tokens=batch * (prompt + 128), max_slots=batch)
            seqs = [eng.open() for _ in range(batch)]
            for g0 in range(0, batch, 8):
                eng.step([tq.StepEntry(s, rng.integers(0, V, size=prompt).tolist(), []) for s in seqs[g0:g0 + 8]])
            toks = rng.integers(0, V, size=(warmup + steps, batch))
            one = lambda i: eng.step([tq.StepEntry(s, [int(toks[i, j])], [0]) for j, s in enumerate(seqs)])
            for i in range(warmup):
                one(i)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            l0 = _call.LAUNCHES
            torch.cuda.synchronize()
            a.record()
            for i in range(warmup, warmup + steps):
                one(i)
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / steps
            out[f"decode_b{batch}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(batch / ms * 1e3, 1),
                                       "launches_per_step": (_call.LAUNCHES - l0) // steps,
                                       # every weight once per step against the measured copy bandwidth
                                       "weights_frac_of_copy_peak": round(weights_bytes(model) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)}
            for s in seqs:
                eng.close(s)
            eng.release()
            del eng
            gc.collect()
            torch.cuda.empty_cache()
        return out

    if args.design == "lumevik":
        return lumevik_compare(args, tq, measure, weights_bytes, pk, rng, prompt, steps, warmup)
    if args.design == "sisepel":
        return sisepel_compare(args, tq, measure, weights_bytes, pk, rng, prompt, steps, warmup)
    if args.design == "tasadra":
        return tasadra_compare(args, tq, measure, weights_bytes, pk, rng, prompt, steps, warmup)
    result = {"metric": "prompt and decode speed, Nuforax beside the dense Qwen2 decoder of equal width", "unit": "tokens/s",
              "n_gpus": 1, "steps": steps, "warmup": warmup, "dtype": "bf16", "data": "synthetic token ids, seeded random weights",
              "peaks": pk, "sizes": {}}
    clocks = ClockSampler()
    clocks.start()
    for name in args.sizes.split(","):
        if name not in DESIGN_SIZES:
            print(json.dumps({"error": f"unknown size '{name}'; known: {sorted(DESIGN_SIZES)}"}))
            return 2
        (W, L, H, dim, rot, vdim, rank, window, ff, mh, mv, mn, mg, V) = DESIGN_SIZES[name]
        cfg = nuforax_config(W, L, H, dim, rot, vdim, rank, window, ff, mh, mv, mn, mg, V)
        model = tq.random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
        entry = {"nuforax": dict(measure(model, V), config={"width": W, "layers": L, "heads": H, "dim": dim, "rot_dim": rot,
                                                             "vdim": vdim, "kv_rank": rank, "window": window, "ff": ff,
                                                             "ssm": {"heads": mh, "vdim": mv, "state": mn, "groups": mg}})}
        if args.kernel_table:
            kernel_table(tq, model, rng, V, 8, args.kernel_table + f".nuforax_{name}.txt", prompt=prompt, context=prompt + 128)
        nbytes = weights_bytes(model)
        del model
        gc.collect()
        torch.cuda.empty_cache()
        # the sibling's feed-forward takes up the weights the other design spends elsewhere, so both stream equal bytes
        qcfg = dense_qwen2_config(W, L, H, window, 64, V)
        base = weights_bytes(tq.build_model(qcfg, "bfloat16"))
        inter = max(64, int(round((nbytes - base) / 2 / (3 * W * L) / 64.0)) * 64 + 64)
        qcfg = dense_qwen2_config(W, L, H, window, inter, V)
        model = tq.random_model(qcfg, seed=0, dtype="bfloat16", device="cuda:0")
        entry["qwen2_dense"] = dict(measure(model, V), config={"width": W, "layers": L, "heads": H, "kv_heads": max(1, H // 4),
                                                               "head_dim": 128, "window": window, "intermediate": inter})
        if args.kernel_table:
            kernel_table(tq, model, rng, V, 8, args.kernel_table + f".qwen2_{name}.txt", prompt=prompt, context=prompt + 128)
        del model
        gc.collect()
        torch.cuda.empty_cache()
        result["sizes"][name] = entry
    result["clocks"] = clocks.stop()
    print(json.dumps(result))
    return 0


def lumevik_compare(args, tq, measure, weights_bytes, pk, rng, prompt, steps, warmup) -> int:
    """The Lumevik decoder beside the Qwen2 MoE decoder of the same widths, heads, window, experts and feed-forward
    sizes (which has attention with rotation on every layer where Lumevik alternates latent and windowed attention)."""
    import torch
    result = {"metric": "prompt and decode speed, Lumevik beside the Qwen2 MoE decoder of equal sizes", "unit": "tokens/s",
              "n_gpus": 1, "steps": steps, "warmup": warmup, "dtype": "bf16", "data": "synthetic token ids, seeded random weights",
              "peaks": pk, "sizes": {}}
    clocks = ClockSampler()
    clocks.start()
    for name in args.sizes.split(","):
        if name not in LUMEVIK_SIZES:
            print(json.dumps({"error": f"unknown size '{name}'; known: {sorted(LUMEVIK_SIZES)}"}))
            return 2
        (W, L, H, G, D, window, keep, rank, q_rank, ff, E, top, e_ff, s_ff, V) = LUMEVIK_SIZES[name]
        entry = {}
        for who, cfg in (("lumevik", lumevik_config(W, L, H, G, D, window, keep, rank, q_rank, ff, E, top, e_ff, s_ff, V)),
                         ("qwen2_moe", sparse_qwen2_config(W, L, H, G, D, window, ff, E, top, e_ff, s_ff, V))):
            model = tq.random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
            entry[who] = dict(measure(model, V), config={"width": W, "layers": L, "heads": H, "kv_heads": G, "head_size": D,
                                                         "window": window, "dense_ff": ff, "experts": E, "top": top,
                                                         "expert_ff": e_ff, "shared_ff": s_ff})
            if args.kernel_table:
                kernel_table(tq, model, rng, V, args.batch, args.kernel_table + f".{who}_{name}.txt", prompt=prompt, context=prompt + 128)
            del model
            gc.collect()
            torch.cuda.empty_cache()
        result["sizes"][name] = entry
    result["clocks"] = clocks.stop()
    print(json.dumps(result))
    return 0


def sisepel_compare(args, tq, measure, weights_bytes, pk, rng, prompt, steps, warmup) -> int:
    """The Sisepel decoder beside the Lumevik decoder of the same width, depth, heads, window, experts and feed-forward
    sizes: both run windowed attention with a sink on the same kernels and the same expert products; Sisepel adds a
    retention branch and a token input to every layer and has no latent attention."""
    import torch
    result = {"metric": "prompt and decode speed, Sisepel beside the Lumevik decoder of equal sizes", "unit": "tokens/s",
              "n_gpus": 1, "steps": steps, "warmup": warmup, "dtype": "bf16", "data": "synthetic token ids, seeded random weights",
              "peaks": pk, "sizes": {}}
    clocks = ClockSampler()
    clocks.start()
    for name in args.sizes.split(","):
        if name not in SISEPEL_SIZES:
            print(json.dumps({"error": f"unknown size '{name}'; known: {sorted(SISEPEL_SIZES)}"}))
            return 2
        (W, L, H, G, D, window, keep, rank, q_rank, ff, E, top, e_ff, s_ff, V) = LUMEVIK_SIZES[name]
        (rh, rd, rv, side) = SISEPEL_SIZES[name]
        entry = {}
        for who, cfg in (("sisepel", sisepel_config(W, L, H, G, D, window, rh, rd, rv, ff, E, top, e_ff, s_ff, side, V)),
                         ("lumevik", lumevik_config(W, L, H, G, D, window, keep, rank, q_rank, ff, E, top, e_ff, s_ff, V))):
            model = tq.random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
            conf = {"width": W, "layers": L, "heads": H, "kv_heads": G, "head_size": D, "window": window, "dense_ff": ff,
                    "experts": E, "top": top, "expert_ff": e_ff, "shared_ff": s_ff}
            if who == "sisepel":
                conf.update(retention={"heads": rh, "dim": rd, "vdim": rv}, token_input=side)
            entry[who] = dict(measure(model, V), config=conf)
            if args.kernel_table:
                kernel_table(tq, model, rng, V, args.batch, args.kernel_table + f".{who}_{name}.txt", prompt=prompt, context=prompt + 128)
            del model
            gc.collect()
            torch.cuda.empty_cache()
        result["sizes"][name] = entry
    result["clocks"] = clocks.stop()
    print(json.dumps(result))
    return 0


def tasadra_config(width, heads, kv_heads, dim, d_dim, cell, ff, vocab, ranks=(64, 64)):
    """Six layers: delta rule, attention, differential attention in cells, differential attention reading that one's
    rows, attention, delta rule; a dense feed-forward on every layer."""
    att = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "softcap": 50.0,
           "rot": {"base": 500000.0, "dims": dim, "scaling": {"factor": 8.0, "original": 8192, "fast": 32.0, "slow": 1.0}}}
    rule = {"heads": heads, "kv_heads": heads, "dim": dim, "vdim": dim, "conv": 4, "decay_rank": ranks[0], "gate_rank": ranks[1]}
    dif = lambda src: dict({"heads": heads, "kv_heads": kv_heads, "dim": d_dim, "vdim": dim, "scale": d_dim ** -0.5, "diff": 0.2,
                            "mask": {"size": cell}}, **({} if src is None else {"kv_from": src}))
    mlp = {"kind": "dense", "ff": ff}
    kinds = [("channel_delta", rule), ("attention", att), ("attention_2", dif(None)), ("attention_2", dif(2)),
             ("attention", att), ("channel_delta", rule)]
    return {"architecture": "Tasadra", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "residual_mult": 0.5,
            "layers": [{"type": k, "mixer": m, "mlp": mlp} for k, m in kinds]}


def sisepel_dense_config(width, layers, heads, kv_heads, dim, window, r_heads, r_dim, r_vdim, ff, vocab):
    """The Sisepel decoder with a dense feed-forward on every layer and no token input."""
    cfg = sisepel_config(width, layers, heads, kv_heads, dim, window, r_heads, r_dim, r_vdim, ff, 1, 1, 1, 1, 1, vocab)
    cfg.pop("token_side")
    for l in cfg["layers"]:
        l["mlp"] = {"kind": "dense", "ff": ff}
    return cfg


TASADRA_SIZES = {
    # name: (width, heads, kv heads, head size, key size of the differential layers, cells, feed-forward, vocab,
    #        the sibling's retention heads, key size, value size)
    "w1024": (1024, 8, 2, 128, 64, 1024, 4096, 32768, 8, 64, 128),
    "w2048": (2048, 16, 4, 128, 64, 1024, 8192, 32768, 16, 128, 128),
}


def tasadra_compare(args, tq, measure, weights_bytes, pk, rng, prompt, steps, warmup) -> int:
    """The Tasadra decoder beside the Sisepel decoder of the same width, depth, heads, head size and dense feed-forward:
    both run softmax attention over rows of keys and values on the same kernels and a recurrence with a state per
    head; Sisepel has both on every layer, Tasadra one of them a layer."""
    import torch
    result = {"metric": "prompt and decode speed, Tasadra beside the Sisepel decoder of equal sizes", "unit": "tokens/s",
              "n_gpus": 1, "steps": steps, "warmup": warmup, "dtype": "bf16", "data": "synthetic token ids, seeded random weights",
              "peaks": pk, "sizes": {}}
    clocks = ClockSampler()
    clocks.start()
    for name in args.sizes.split(","):
        if name not in TASADRA_SIZES:
            print(json.dumps({"error": f"unknown size '{name}'; known: {sorted(TASADRA_SIZES)}"}))
            return 2
        (W, H, G, D, DD, cell, ff, V, rh, rd, rv) = TASADRA_SIZES[name]
        entry = {}
        for who, cfg in (("tasadra", tasadra_config(W, H, G, D, DD, cell, ff, V)),
                         ("sisepel", sisepel_dense_config(W, 6, H, G, D, cell, rh, rd, rv, ff, V))):
            model = tq.random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
            conf = {"width": W, "layers": 6, "heads": H, "kv_heads": G, "head_size": D, "dense_ff": ff}
            if who == "tasadra":
                conf.update(differential={"dim": DD, "cells": cell}, delta={"heads": H, "dim": D, "vdim": D, "conv": 4})
            else:
                conf.update(window=cell, retention={"heads": rh, "dim": rd, "vdim": rv})
            entry[who] = dict(measure(model, V), config=conf)
            if args.kernel_table:
                kernel_table(tq, model, rng, V, args.batch, args.kernel_table + f".{who}_{name}.txt", prompt=prompt, context=prompt + 128)
            del model
            gc.collect()
            torch.cuda.empty_cache()
        result["sizes"][name] = entry
    result["clocks"] = clocks.stop()
    print(json.dumps(result))
    return 0


def kernel_table(tq, model, rng, V, batch, path, prompt=None, context=None):
    """Per-kernel device time of 4 decode steps at context 2,048 and of one 2,048-token prefill."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    PROMPT, CONTEXT = prompt or globals()["PROMPT"], context or globals()["CONTEXT"]
    eng = tq.Engine(model, max_tokens=batch * CONTEXT, max_slots=batch)
    seqs = [eng.open() for _ in range(batch)]
    for g0 in range(0, batch, 8):
        eng.step([tq.StepEntry(s, rng.integers(0, V, size=PROMPT).tolist(), []) for s in seqs[g0:g0 + 8]])
    step = lambda: eng.step([tq.StepEntry(s, [1], [0]) for s in seqs])
    step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(4):
            step()
        torch.cuda.synchronize()
    text = "== 4 decode steps, batch %d, context %d ==\n" % (batch, PROMPT)
    text += prof.key_averages().table(sort_by="cuda_time_total", row_limit=25, max_name_column_width=70)
    for s in seqs:
        eng.close(s)
    s = eng.open()
    toks = rng.integers(0, V, size=PROMPT).tolist()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        eng.step([tq.StepEntry(s, toks, [PROMPT - 1])])
        torch.cuda.synchronize()
    text += "\n== prefill of one %d-token prompt ==\n" % PROMPT
    text += prof.key_averages().table(sort_by="cuda_time_total", row_limit=25, max_name_column_width=70)
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    open(path, "w").write(text)


if __name__ == "__main__":
    sys.exit(main())
