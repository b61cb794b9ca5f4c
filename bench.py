"""Benchmark of mynah_slm_b200 on one B200: decode tokens per second at the
Qwen3-0.6B shape with random weights (batch 8 by default, 2,048-token prompts,
4,096-token context), prefill of one 2,048-token prompt, and decode at batch 1
and 64.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --workload 4b|8b      (the two larger workloads, a JSON line of their own each)

One JSON line on stdout. A step is one decode step of the batch.
  value     decoded tokens per second, timed on the device with CUDA events
            around exactly K steps that run from a captured graph with the
            sampled token fed back on the device
  e2e       the same through the Python entry point (LLM.generate): every
            step copies its inputs from pinned host memory to the device and
            reads the sampled tokens back to the host
  prefill   one 2,048-token prompt in one step; frac = flops / time / peak
  roofline  bytes a decode step has to read (every weight once, the cache of
            the live requests) / its time, against the HBM peak
  points    decode at batch 1 and 64 behind the 2,048-token prompts, and all three
            batch sizes again in the middle and at the end of the range the
            configuration names (2,048 generated tokens behind the prompt): after
            untimed steps up to 3,072 and 4,096 positions, 64 timed steps each;
            point_fracs gives each point's share of the HBM peak for its bytes
Peaks come from MEASURED_PEAKS.json beside this file when it exists, else from
the stated fallback. The weights are made on the device from the seed; no file is
written.

--workload 4b: 16 prompts of lengths uniform in [16, 2048], 256 generated tokens
each, greedy and at temperature 0.7, at the Qwen3-4B layer sizes, through
LLM.generate. --workload 8b: 64 prompts of 2,048 tokens and 2,048 generated tokens
each at the Qwen3-8B layer sizes (bf16 cache of 38.65 GB), through LLM.generate.
"""
from __future__ import annotations

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

# Qwen3-0.6B layer sizes (the benchmark configuration; random weights, seed 2)
QWEN3_0_6B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=28, hidden_size=1024,
                  num_attention_heads=16, num_key_value_heads=8, head_dim=128, intermediate_size=3072,
                  vocab_size=151936, rope_theta=1000000, rms_norm_eps=1e-6, tie_word_embeddings=True,
                  max_position_embeddings=40960, hidden_act="silu", attention_bias=False, rope_scaling=None,
                  use_sliding_window=False, sliding_window=None, eos_token_id=151645)
# Other layer sizes, for the short single-phase runs (--only) that check and profile the kernels at further sizes
SHAPES = {
    "0.6b": {},
    "4b": dict(num_hidden_layers=36, hidden_size=2560, num_attention_heads=32, num_key_value_heads=8, intermediate_size=9728),
    "8b": dict(num_hidden_layers=36, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, intermediate_size=12288,
               tie_word_embeddings=False),
}
PROMPT_LEN, CTX_LEN, PREFILL_TOKENS = 2048, 4096, 2048
FAR_STEPS = 64            # timed steps of the points in the middle and at the end of the context range
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            out = {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"])}
            if "bf16_tflops_sustained" in p:                        # the library's product back to back for seconds, under the power cap
                out["bf16_tflops_sustained"] = float(p["bf16_tflops_sustained"])
            return out, "measured"
        except (OSError, ValueError, KeyError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.proc = None
        self.lines: list[str] = []
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def model_flops_prefill(c: dict, T: int, layers: int) -> float:
    D, H, KV, HD, F, V = (c["hidden_size"], c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"],
                          c["intermediate_size"], c["vocab_size"])
    linear = 2.0 * T * (D * (H + 2 * KV) * HD + H * HD * D + D * 2 * F + F * D)
    attn = 2.0 * 2.0 * H * HD * (T * (T + 1) / 2.0)          # QK^T and PV, causal
    return layers * (linear + attn) + 2.0 * D * V            # the head runs on the last row only


def decode_bytes(c: dict, layers: int, batch: int, ctx: float) -> float:
    D, H, KV, HD, F, V = (c["hidden_size"], c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"],
                          c["intermediate_size"], c["vocab_size"])
    per_layer = 2 * (D * (H + 2 * KV) * HD + H * HD * D + D * 2 * F + F * D) + 2 * (2 * D + 2 * HD)
    head = 2 * D * V if c["tie_word_embeddings"] else 2 * D * V      # read once as the head (the gather reads B rows)
    kv = batch * ctx * layers * 2 * KV * HD * 2
    return layers * per_layer + head + 2 * D + kv


def run_workload(which: str, layers_override: int = 0) -> int:
    """The two larger workloads, end to end through LLM.generate (host token ids in and out every step)."""
    import numpy as np
    import torch

    from mynah_slm_b200 import LLM

    cfg = dict(QWEN3_0_6B)
    cfg.update(SHAPES[which])
    layers_model = cfg["num_hidden_layers"]
    layers = layers_override or layers_model
    cfg["num_hidden_layers"] = layers
    pk, pk_src = peaks()
    rng = np.random.default_rng(3 if which == "4b" else 4)
    V = cfg["vocab_size"]
    if which == "4b":
        lens = rng.integers(16, 2049, size=16).tolist()
        n_new, runs = 256, [("greedy", 0.0), ("temp_0.7", 0.7)]
        max_tokens = sum(-(-(n + n_new) // 64) * 64 for n in lens)
    else:
        lens = [PROMPT_LEN] * 64
        n_new, runs = CTX_LEN - PROMPT_LEN, [("greedy", 0.0)]
        max_tokens = 64 * CTX_LEN
    prompts = [rng.integers(0, V, size=n).tolist() for n in lens]
    llm = LLM.random(cfg, seed=3 if which == "4b" else 4, dtype="bfloat16", max_tokens=max_tokens, max_seqs=len(lens))
    llm.generate([p[:64] for p in prompts], max_new=4, temp=0.0, ignore_eos=True, max_batch=len(lens))    # warm-up
    out = {"workload": which, "model": f"Qwen3-{which.upper()} shape", "layers": layers, "layers_of_model": layers_model,
           "batch": len(lens), "prompt_tokens": int(sum(lens)), "new_tokens_each": n_new, "dtype": "bf16",
           "data": f"synthetic: random weights (seed {3 if which == '4b' else 4}), uniform random token ids",
           "cache_gb": round(max_tokens * layers * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2 / 1e9, 2),
           "peaks": f"{pk_src}: {pk['hbm_gbs']:.0f} GB/s, {pk['bf16_tflops']:.0f} TFLOP/s", "runs": {}}
    clocks = ClockSampler()
    clocks.start()
    for name, temp in runs:
        res = llm.generate(prompts, max_new=n_new, temp=temp, top_k=0, top_p=1.0, seed=1, ignore_eos=True, max_batch=len(lens))
        t = llm.last_timing
        assert all(len(r.tokens) == n_new for r in res)
        steps = n_new - 1                                   # the first token of each request comes from the prompt step
        mean_ctx = sum(lens) / len(lens) + n_new / 2.0
        step_s = t.decode_s / steps
        gbs = decode_bytes(cfg, layers, len(lens), mean_ctx) / step_s / 1e9
        flops = sum(model_flops_prefill(cfg, n, layers) for n in lens)
        out["runs"][name] = {"decode_tokens_per_s": round(len(lens) * steps / t.decode_s, 1), "ms_per_step": round(step_s * 1e3, 3),
                             "GBps": round(gbs, 1), "hbm_frac": round(gbs / pk["hbm_gbs"], 4),
                             "prefill_tokens_per_s": round(sum(lens) / t.prefill_s, 1), "prefill_ms": round(t.prefill_s * 1e3, 1),
                             "prefill_frac": round(flops / t.prefill_s / (pk["bf16_tflops"] * 1e12), 4)}
        if "bf16_tflops_sustained" in pk and t.prefill_s > 0.5:      # a prompt step of seconds runs under the power cap
            out["runs"][name]["prefill_frac_of_sustained"] = round(flops / t.prefill_s / (pk["bf16_tflops_sustained"] * 1e12), 4)
    out["clocks"] = clocks.stop()
    print(json.dumps(out))
    return 0


def time_products(shape: str, rows: int) -> int:
    """The four matrix products of a decode step of `rows` rows at a shape's layer sizes, each alone: the weights
    through registers, through the ring of asynchronous copies, and the library's product. Enough different
    matrices are cycled through that none is found in L2; the launches replay from a graph; CUDA events."""
    import torch

    from mynah_slm_b200.ops import kernels as k

    cfg = dict(QWEN3_0_6B)
    cfg.update(SHAPES[shape])
    D, H, KV, HD, F = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["intermediate_size"]
    dev = "cuda:0"

    def timed(fn, n):
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        for _ in range(2):
            g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 10 / n * 1e3

    out = {"only": "products", "shape": shape, "rows": rows, "unit": "us (GB/s of weights)" if rows <= 16 else "us (TFLOP/s)", "products": {}}
    for name, N, K, swiglu in (("qkv", (H + 2 * KV) * HD, D, False), ("o", D, H * HD, False), ("gate_up", F, D, True), ("down", D, F, False)):
        n_rows = N * (2 if swiglu else 1)
        n = max(2, int(400e6 / (n_rows * K * 2)) + 1)
        if rows > 16:
            n = min(n, 4)                                           # (the rows and the results are the larger part here)
        ws = [torch.randn(n_rows, K, device=dev).bfloat16() for _ in range(n)]
        x = torch.randn(rows, K, device=dev).bfloat16()
        mb = n_rows * K * 2 / 1e6
        res = {}
        f = (lambda: [k.linear_swiglu(x, w) for w in ws]) if swiglu else (lambda: [k.linear(x, w) for w in ws])
        if rows > 16:
            # a prompt step's product: the package's route (the tensor-core kernel from 129 rows on) against the library
            tf = 2.0 * rows * n_rows * K / 1e6                      # flop / 1e6: with us, TFLOP/s
            t = timed(f, n)
            res["own"] = f"{t:.1f} ({tf / t:.0f} TFLOP/s)"
            t = timed(lambda: [torch.mm(x, w.t()) for w in ws], n)
            res["library" + (" (no activation)" if swiglu else "")] = f"{t:.1f} ({tf / t:.0f} TFLOP/s)"
            out["products"][f"{name} {N}x{K}"] = res
            del ws
            continue
        for label, mode in (("registers", 0), ("ring", 1)):
            k.gemv_decode_mode(mode)
            t = timed(f, n)
            res[label] = f"{t:.1f} ({mb / t * 1e3:.0f})"
        k.gemv_decode_mode(2)
        t = timed(lambda: [torch.mm(x, w.t()) for w in ws], n)
        res["library" + (" (no activation)" if swiglu else "")] = f"{t:.1f} ({mb / t * 1e3:.0f})"
        out["products"][f"{name} {N}x{K}"] = res
        del ws
    print(json.dumps(out))
    return 0


def time_reader() -> int:
    """What the device gives a plain reader of shuffled 16 KB pieces (2 GB, nothing done with them) for a given
    number of bytes in flight an SM: the yardstick for the kernels that stream the cache and the weights."""
    import numpy as np
    import torch

    from mynah_slm_b200.ops.lib import call, ptr, stream_ptr

    dev = "cuda:0"
    n = (2 << 30) // 16384
    buf = torch.ones((n * 16384,), dtype=torch.uint8, device=dev)
    order = torch.from_numpy(np.random.default_rng(1).permutation(n).astype(np.int32)).to(dev)
    sink = torch.zeros((1,), dtype=torch.int64, device=dev)
    status = torch.zeros((1,), dtype=torch.int32, device=dev)
    out = {"only": "reader", "bytes": n * 16384, "unit": "GB/s", "rates": {}}
    for ctas, stages in ((1, 4), (2, 4), (1, 12), (2, 6), (3, 4), (4, 3)):
        call("mynah_read_probe", ptr(buf), ptr(order), n, ctas, stages, ptr(sink), ptr(status), stream_ptr())
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            call("mynah_read_probe", ptr(buf), ptr(order), n, ctas, stages, ptr(sink), ptr(status), stream_ptr())
        e1.record()
        torch.cuda.synchronize()
        out["rates"][f"{ctas * stages * 16} KB in flight an SM ({ctas} CTAs x {stages} copies)"] = round(n * 16384 * 5 / (e0.elapsed_time(e1) / 1e3) / 1e9)
    assert status.item() == 0, "a wait in the reader ran out"
    print(json.dumps(out))
    return 0


def run_reference(args) -> int:
    """The unmodified reference on the same metric: 8 requests with 2,048-token prompts, one after another (it has
    no batch), token by token (prompts too), on the host's CPU cores (it has no GPU path). See baseline/reference_arm.py."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import reference_arm
    except ImportError as e:
        print(json.dumps({"impl": "reference", "unavailable": f"baseline/reference_arm.py cannot be imported: {e}"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"impl": "reference", "unavailable": "the reference runs on the host's CPU cores; there is nothing to run on several GPUs"}))
        return 0
    B, K, W = args.batch, max(1, min(args.steps, 32)), max(3, min(args.warmup, 4))
    try:
        r = reference_arm.run(dict(QWEN3_0_6B), B, PROMPT_LEN, W, K, budget_s=float(os.environ.get("MYNAH_REFERENCE_BUDGET_S", "900")))
    except reference_arm.Unavailable as e:
        print(json.dumps({"impl": "reference", "unavailable": " ".join(str(e).split())}))
        return 0
    except Exception as e:                                    # noqa: BLE001 - the arm must end with a line, not a trace
        print(json.dumps({"impl": "reference", "unavailable": f"the reference arm failed: {type(e).__name__}: {' '.join(str(e).split())[:300]}"}))
        return 0
    value = r["decode_tokens"] / r["decode_s"]
    c = QWEN3_0_6B
    print(json.dumps({
        "metric": "decode tok/s at batch 8, 2,048-token prompts, 4,096 context (Qwen3-0.6B shape)", "value": round(value, 2),
        "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": round(r["decode_s"] / K * 1e3, 2),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32 arithmetic on fp16 weights",
        "data": "synthetic: random weights (seed 2), uniform random token ids", "impl": "reference", "device": "cpu",
        "config": {"model": "Qwen3-0.6B shape", "layers": c["num_hidden_layers"], "hidden": c["hidden_size"], "heads": c["num_attention_heads"],
                   "kv_heads": c["num_key_value_heads"], "head_dim": c["head_dim"], "ffn": c["intermediate_size"], "vocab": c["vocab_size"],
                   "global_batch": B, "prompt_len": PROMPT_LEN, "seq_len": CTX_LEN, "sampling": "greedy",
                   "parallelism": f"{r['threads']} CPU threads, the {B} requests one after another (the reference has no batch)"},
        "e2e": {"value": round(value, 2), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "prefill": {"value": round(r["prompt_tokens"] / r["prompt_s"], 2), "tokens": PROMPT_LEN, "ms": round(r["prompt_s"] / B * 1e3, 1)},
    }))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (0: all)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch-1 and batch-64 points")
    ap.add_argument("--only", default="", choices=["", "decode", "prefill", "products", "reader"],
                    help="run one small phase and print a short line (for profiling a kernel on a small case)")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN, help="prompt length of the decode phases")
    ap.add_argument("--shape", default="0.6b", choices=sorted(SHAPES), help="layer sizes, for --only runs (the full line is always 0.6b)")
    ap.add_argument("--workload", default="", choices=["", "4b", "8b"], help="run one of the two larger workloads instead")
    args = ap.parse_args()

    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print(f"bench.py measures one GPU only (this library does not use several); --gpus {args.gpus} is not run")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import numpy as np
    import torch

    from mynah_slm_b200 import LLM, parse_config
    from mynah_slm_b200.engine.engine import StepEntry
    from mynah_slm_b200.ops import gemm_bf16, lib
    from mynah_slm_b200.sampling.sampler import SamplingParams

    if args.workload:
        return run_workload(args.workload, args.layers)
    if args.only == "products":
        return time_products(args.shape, args.batch)
    if args.only == "reader":
        return time_reader()

    cfg = dict(QWEN3_0_6B)
    if args.only:
        cfg.update(SHAPES[args.shape])
    layers_model = cfg["num_hidden_layers"]
    layers = args.layers or layers_model
    cfg["num_hidden_layers"] = layers
    pk, pk_src = peaks()
    K, W, B = args.steps, args.warmup, args.batch
    max_batch = B if (args.no_points or args.only) else max(B, 64)
    prompt_len = args.prompt_len
    rng = np.random.default_rng(2)
    V = cfg["vocab_size"]

    # the cache: the benchmark's context length a sequence, or more where a longer prompt is asked for
    ctx_tokens = max(CTX_LEN, -(-(prompt_len + 2 * (W + K) + 8 + 64) // 64) * 64)
    llm = LLM.random(cfg, seed=2, dtype="bfloat16", max_tokens=max_batch * ctx_tokens, max_seqs=max_batch)
    eng = llm.engine
    eng.sampler.set_params(SamplingParams.greedy())

    def device_decode(batch: int, steps: int, warmup: int, far: tuple = ()):
        """Prompts of PROMPT_LEN, then `warmup` untimed and `steps` timed decode steps on the device. For every
        length in `far` the sequences then go on untimed until FAR_STEPS steps before that length and those
        steps are timed: far_ms[length] = (ms, mean context)."""
        prompts = [rng.integers(0, V, size=prompt_len).tolist() for _ in range(batch)]
        slots = [eng.open_sequence() for _ in range(batch)]
        eng.sampler.start_sequences(slots, list(range(1, batch + 1)), prompts)
        logits = eng.step([StepEntry(s, p, (prompt_len - 1,)) for s, p in zip(slots, prompts)])
        first = eng.sampler.sample(logits, torch.tensor(slots, dtype=torch.int32, device=eng.device)).cpu().tolist()
        last = eng.decode_loop(slots, first, warmup)
        toks = last[:batch].cpu().tolist()
        torch.cuda.synchronize()
        n0 = lib.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        last = eng.decode_loop(slots, toks, steps)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        launches = lib.launch_count() - n0
        eng.check_status()
        mean_ctx = prompt_len + 1 + warmup + steps / 2.0
        far_ms = {}
        length = prompt_len + warmup + steps
        for target in far:
            gap = target - FAR_STEPS - length
            if gap < 0:
                continue
            if gap:
                last = eng.decode_loop(slots, last[:batch].cpu().tolist(), gap)
            toks = last[:batch].cpu().tolist()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            last = eng.decode_loop(slots, toks, FAR_STEPS)
            e1.record()
            torch.cuda.synchronize()
            far_ms[target] = (e0.elapsed_time(e1), target - FAR_STEPS / 2.0 + 0.5)
            length = target
            eng.check_status()
        for s in slots:
            eng.close_sequence(s)
        return ms, launches, mean_ctx, far_ms

    def time_prefill(n_timed: int = 5):
        p = rng.integers(0, V, size=PREFILL_TOKENS).tolist()
        times = []
        for i in range(3 + n_timed):
            s = eng.open_sequence()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            eng.step([StepEntry(s, p, (PREFILL_TOKENS - 1,))])
            e1.record()
            torch.cuda.synchronize()
            eng.close_sequence(s)
            if i >= 3:
                times.append(e0.elapsed_time(e1))
        return statistics.median(times)

    if args.only == "decode":
        device_decode(B, 4, W)                      # a first batch captures the steps; the figure is the second batch's (see main)
        ms, launches, mean_ctx, _ = device_decode(B, K, W)
        gbs = decode_bytes(cfg, layers, B, mean_ctx) / (ms / K / 1e3) / 1e9
        print(json.dumps({"only": "decode", "shape": args.shape, "batch": B, "layers": layers, "prompt_len": prompt_len, "steps": K,
                          "ms_per_step": round(ms / K, 4), "tokens_per_s": round(B * K / (ms / 1e3), 1),
                          "GBps": round(gbs, 1), "launches": launches}))
        return 0
    if args.only == "prefill":
        pre_ms = time_prefill(max(1, K))
        fl = model_flops_prefill(cfg, PREFILL_TOKENS, layers)
        print(json.dumps({"only": "prefill", "shape": args.shape, "layers": layers, "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3),
                          "tokens_per_s": round(PREFILL_TOKENS / (pre_ms / 1e3), 1),
                          "TFLOPs": round(fl / (pre_ms / 1e3) / 1e12, 1)}))
        return 0

    # Warm the engine as a serving process is warm: one generation through the public entry point (prompt step, eager
    # sampling of the first tokens, the captured decode steps), and one short batch through the loop that is timed
    # below, so that every graph the timed region replays was captured before it. A captured step replays 6 to 7%
    # faster while nothing but that graph has been launched since its capture (1.33 against 1.42 ms at batch 8;
    # re-capturing, cudaGraphUpload or a stream of its own do not bring that back once other kernels have run), and a
    # serving process is never in that state; so no figure here is taken in it.
    prompts = [rng.integers(0, V, size=prompt_len).tolist() for _ in range(B)]
    llm.generate(prompts, max_new=W + 1, temp=0.0, ignore_eos=True, max_batch=B)
    device_decode(B, 4, W)

    clocks = ClockSampler()
    clocks.start()
    far = () if (args.no_points or prompt_len + W + K + FAR_STEPS > 3072) else (3072, CTX_LEN)
    ms, launches, mean_ctx, far_ms = device_decode(B, K, W, far)
    clock_info = clocks.stop()
    value = B * K / (ms / 1e3)
    bytes_step = decode_bytes(cfg, layers, B, mean_ctx)
    achieved = bytes_step / (ms / K / 1e3) / 1e9

    # end to end through the public entry point: host token ids in, host token ids out, every step
    # (the median of three whole generations: one run's host-side jitter moves the figure by several percent)
    e2e_runs = []
    for _ in range(3):
        llm.generate(prompts, max_new=K + 1, temp=0.0, ignore_eos=True, max_batch=B)
        t = llm.last_timing
        e2e_runs.append(B * K / t.decode_s if t.decode_s > 0 else 0.0)
    e2e_value = statistics.median(e2e_runs)
    bucket = eng._bucket(B)
    graph = eng._graphs[max(k for k in eng._graphs if k[0] == bucket)]
    e2e = {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": graph.layout.size * 4,
           "d2h_bytes_per_step": B * 4, "runs": [round(v, 1) for v in e2e_runs]}

    # prefill of one prompt of 2,048 tokens (logits of the last position)
    pre_ms = time_prefill()
    flops = model_flops_prefill(cfg, PREFILL_TOKENS, layers)
    prefill = {"value": round(PREFILL_TOKENS / (pre_ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3),
               "frac": round(flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}

    points, point_fracs = {}, {}

    def add_far(b: int, far_ms: dict) -> None:
        for target, (fms, fctx) in far_ms.items():
            name = f"decode_b{b}_ctx{target if target != CTX_LEN else CTX_LEN - 1}"
            points[name] = round(b * FAR_STEPS / (fms / 1e3), 1)
            point_fracs[name] = round(decode_bytes(cfg, layers, b, fctx) / (fms / FAR_STEPS / 1e3) / 1e9 / pk["hbm_gbs"], 4)

    add_far(B, far_ms)
    if not args.no_points:
        for b, steps in ((1, max(64, K)), (64, min(K, 64))):
            device_decode(b, 4, W)                   # captures this batch size's steps before they are timed
            pms, _, pctx, pfar = device_decode(b, steps, W, far)
            points[f"decode_b{b}"] = round(b * steps / (pms / 1e3), 1)
            point_fracs[f"decode_b{b}"] = round(decode_bytes(cfg, layers, b, pctx) / (pms / steps / 1e3) / 1e9 / pk["hbm_gbs"], 4)
            add_far(b, pfar)

    out = {
        "metric": "decode tok/s at batch 8, 2,048-token prompts, 4,096 context (Qwen3-0.6B shape)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms / K, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights (seed 2), uniform random token ids",
        "impl": "ours",
        "config": {"model": "Qwen3-0.6B shape", "layers": layers, "layers_of_model": layers_model,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "ffn": cfg["intermediate_size"], "vocab": V, "tied_head": True, "global_batch": B,
                   "prompt_len": prompt_len, "seq_len": CTX_LEN, "sampling": "greedy", "cache_dtype": "bf16",
                   "parallelism": "1 GPU", "l2": "inputs larger than L2 (weights 1.2 GB + cache)",
                   "peaks": f"{pk_src}: {pk['hbm_gbs']:.0f} GB/s, {pk['bf16_tflops']:.0f} TFLOP/s"},
        "e2e": e2e, "gpu_launches": int(launches),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points, "point_fracs": point_fracs, "clocks": clock_info,
        "matmul_calls": dict(gemm_bf16.counters),
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
