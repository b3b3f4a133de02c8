#!/usr/bin/env python3
"""Decode and prefill throughput of the SmolLM2-135M shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--shape 135m|360m|1.7b] [--batch B] [--context C] [--layers L] [--skip-points]
                    [--skip-e2e]

A step is one decode step of a batch of 8 sequences whose context ends at 4,096
tokens (prompt 2,048 + 2,048 decoded); ``value`` is decoded tokens per second,
timed with CUDA events over K graph launches: the median of five such regions over
the same range of contexts, as NNIS's own benchmarks take the median of five
(crates/nnis-bench/src/lib.rs:362-428).  ``e2e`` is the same through the Python
entry point with every step's tokens coming from and going back to the host, over
256 steps whatever K is.  The line also carries a 2,048-token prefill, the decode
step's HBM roofline, decoding at batch 1 and 64, and ``kernels``: per kernel of one
more decode step, taken outside every timed region with the kernels' own readings of
the GPU's timer, its launches and the microseconds from its last CTA getting past the
wait for the kernel before to its end, summed over the launches.  Weights are random (seeded),
token ids are uniform random: no checkpoint or dataset is read.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# The shape of SmolLM2-135M; nothing below the configuration knows these numbers.
SMOLLM2_135M = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=49152, hidden_size=576,
    intermediate_size=1536, num_hidden_layers=30, num_attention_heads=9, num_key_value_heads=3,
    max_position_embeddings=8192, rms_norm_eps=1e-5, rope_theta=100000.0, hidden_act="silu",
    tie_word_embeddings=True, attention_bias=False, torch_dtype="bfloat16")
# The two larger shapes of the same family: what differs from the above.
SHAPES = {
    "135m": ("SmolLM2-135M", {}),
    "360m": ("SmolLM2-360M", dict(num_hidden_layers=32, hidden_size=960, intermediate_size=2560,
                                  num_attention_heads=15, num_key_value_heads=5)),
    "1.7b": ("SmolLM2-1.7B", dict(num_hidden_layers=24, hidden_size=2048, intermediate_size=8192,
                                  num_attention_heads=32, num_key_value_heads=32, rope_theta=130000.0)),
}
CONTEXT = 4096
PROMPT = 2048
BATCH = 8
REPEATS = 5     # timed regions per point; the median is reported
E2E_STEPS = 256  # decode steps of the end-to-end run
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
                  "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            raw = json.load(f)
        return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                "bf16_tflops_sustained": float(raw.get("bf16_tflops_sustained", raw["bf16_tflops"])),
                "source": "measured"}
    except (OSError, KeyError, ValueError, TypeError):
        return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_id: str = "0"):
        """``gpu_id``: what ``nvidia-smi -i`` takes for the GPU that the run is on (its
        UUID: index 0 of this process need not be index 0 of the machine)."""
        self.samples, self.proc, self.gpu_id = [], None, gpu_id

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", self.gpu_id, f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), [x.strip() for x in line.split(",")]))

    def mark(self):
        return time.time()

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()

    def summary(self, windows):
        rows = [s for t, s in self.samples if any(a <= t <= b for a, b in windows)] or \
               [s for _, s in self.samples]
        sm = sorted(int(r[0]) for r in rows if r[0].isdigit())
        mx = [int(r[1]) for r in rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active"
                                                         for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(rows), "gpu": self.gpu_id}


def gpu_identity(torch) -> str:
    """The UUID of this process's device 0 in nvidia-smi's spelling; "0" if it cannot be had."""
    try:
        uuid = str(torch.cuda.get_device_properties(0).uuid)
        return uuid if uuid.startswith("GPU-") else "GPU-" + uuid
    except Exception:
        return "0"


def median(values):
    values = sorted(values)
    return values[len(values) // 2]


def write_timeline(path, title, names, rows, marks):
    """The table of one traced step: per launch its begin, first and last CTA past the wait
    for the kernel before, two inner marks, end and duration, relative to the step's first
    begin; then sums per kernel."""
    t0 = min(r[0] for r in rows)
    by_name = {}
    big = 1 << 62
    with open(path, "w") as f:
        f.write(f"# {title}; ns after the step's first CTA\n# launch kernel begin past_wait_first past_wait_last "
                f"mark1_first mark1_last mark2_first mark2_last end duration\n# marks: {marks}\n")
        for i, (name, r) in enumerate(zip(names, rows)):
            rel = [(v - t0 if 0 < v < big else -1) for v in r]
            b, e, w1 = rel[0], rel[1], rel[3]
            f.write(f"{i} {name.replace(' ', '_')} {b} {rel[2]} {w1} {rel[4]} {rel[5]} {rel[6]} {rel[7]} {e} {e - b}\n")
            total = by_name.setdefault(name, [0, 0, 0])
            total[0] += 1
            total[1] += e - b
            total[2] += e - (w1 if w1 >= 0 else b)
        f.write(f"# step: {max(r[1] for r in rows) - t0} ns\n")
        for name, (count, dur, after) in sorted(by_name.items()):
            f.write(f"# {name}: {count} launches, mean begin-to-end {dur / count:.0f} ns, "
                    f"mean last-wait-to-end {after / count:.0f} ns, sum of the latter {after / 1000:.0f} us\n")
    print(open(path).read()[-1800:])


def kernel_times(names, rows):
    """Per kernel of one traced step: launches, and microseconds from the moment its last
    CTA got past the wait for the kernel before to its end (its link in the step's chain),
    summed over the launches; and the step from its first CTA to its last."""
    big = 1 << 62
    out = {}
    for name, r in zip(names, rows):
        begin, end, last_wait = r[0], r[1], r[3]
        start = last_wait if 0 < last_wait < big else begin
        entry = out.setdefault(name, {"launches": 0, "us": 0.0})
        entry["launches"] += 1
        entry["us"] += (end - start) / 1000.0
    for entry in out.values():
        entry["us"] = round(entry["us"], 1)
    out["step"] = {"launches": len(rows), "us": round((max(r[1] for r in rows) - min(r[0] for r in rows)) / 1000.0, 1)}
    return out


def prefill_timeline(engine, path, rng, vocab):
    """One prompt step of 2,048 tokens as the GPU's own timer saw it (the instrumented
    kernels: tcgen05 products, prompt attention, the norms of many rows)."""
    import torch

    from nnis_b200.csrc import ops
    from nnis_b200.engine import SequenceStep
    prompt = [rng.randrange(vocab) for _ in range(PROMPT)]

    def once():
        slot = engine.acquire_slot()
        engine.step([SequenceStep(slot, prompt, [PROMPT - 1])])
        engine.release_slot(slot)
    once()                      # seen once
    buf = ops.trace_begin(4096)
    once()                      # run into its own buffers and captured: both take slots
    names = ops.trace_end()
    for _ in range(3):
        once()
    torch.cuda.synchronize()
    ops.trace_clear()
    once()
    torch.cuda.synchronize()
    half = len(names) // 2
    write_timeline(path, f"one prompt step of {PROMPT} tokens", names[half:], buf[half:2 * half].cpu().tolist(),
                   "products: first operands arrived / all products complete")


def timeline(engine, batch, path, rng, vocab):
    """One decode step at context 4,096 as the GPU's own timer saw it: per launch of the
    decode kernels its begin and end, and when its first and last CTA got past the wait
    for the kernel before, relative to the step's first begin; then sums per kernel."""
    import torch

    from nnis_b200.csrc import ops
    from nnis_b200.engine import SequenceStep
    from nnis_b200.engine.decode import GraphDecoder
    begin = CONTEXT - 16
    slots = [engine.acquire_slot() for _ in range(batch)]
    fed = 0
    while fed < begin:
        n = min(PROMPT, begin - fed)
        per_step = max(1, 16384 // n)
        for i in range(0, batch, per_step):
            engine.step([SequenceStep(s, [rng.randrange(vocab) for _ in range(n)], [])
                         for s in slots[i:i + per_step]])
        fed += n
    dec = GraphDecoder(engine, batch, CONTEXT)
    engine.cache.reserve(slots, [CONTEXT] * batch)
    for r, s in enumerate(slots):
        dec.set_row(r, s, rng.randrange(vocab), begin)
    buf = ops.trace_begin(4096)
    dec.capture()  # the warm-up run takes slots as well; the captured launches take the later half
    names = ops.trace_end()
    for _ in range(4):
        dec.launch()
    torch.cuda.synchronize()
    ops.trace_clear()
    dec.launch()
    torch.cuda.synchronize()
    half = len(names) // 2
    write_timeline(path, f"one decode step, batch {batch}, context {CONTEXT}, {len(dec.chains)} chain(s)",
                   names[half:], buf[half:2 * half].cpu().tolist(),
                   "projections x staged / products done; attention pages done / ticket taken")


def main() -> int:
    global CONTEXT
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has")
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 and 64")
    ap.add_argument("--skip-e2e", action="store_true", help="leave out the end-to-end run")
    ap.add_argument("--batch", type=int, default=BATCH, help="sequences of the main decode point")
    ap.add_argument("--context", type=int, default=CONTEXT,
                    help="tokens at which the decoded contexts end (the metric's: 4096)")
    ap.add_argument("--timeline", metavar="FILE", default=None,
                    help="instead of the benchmark: write the timeline of one decode step of the main "
                         "point (begin, end and wait of every launch of the decode kernels) to FILE; "
                         "with --batch 0, of the 2,048-token prompt step")
    ap.add_argument("--shape", default="135m", choices=sorted(SHAPES),
                    help="layer sizes: the SmolLM2-135M shape (the benchmark) or a larger one of the family")
    args = ap.parse_args()
    CONTEXT = max(args.context, 64)
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "Memorithm/NNIS is a Rust workspace (cargo, NVRTC); pip cannot install it "
                          "and no Rust toolchain is present"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch

    from nnis_b200 import LLM
    from nnis_b200.csrc import ops
    from nnis_b200.engine import SequenceStep
    from nnis_b200.engine.decode import GraphDecoder
    from nnis_b200.weights import write_random_model

    pk = peaks()
    cfg = dict(SMOLLM2_135M)
    shape_name, shape_sizes = SHAPES[args.shape]
    cfg.update(shape_sizes)
    cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], CONTEXT)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    rng = random.Random(0)
    vocab = cfg["vocab_size"]
    K, W = args.steps, args.warmup
    clocks = ClockSampler(gpu_identity(torch))
    windows = []

    with tempfile.TemporaryDirectory() as tmp:
        write_random_model(cfg, seed=0, out_dir=tmp, std=1.0, norm_std=0.1, std_by_fan_in=True)
        most_rows = max(args.batch, 1, 1 if args.skip_points or args.timeline else 64)  # the cache holds the largest point
        llm = LLM(tmp, dtype="bfloat16", device_ordinal=0, max_tokens=max(most_rows * (CONTEXT + 64), 4 * (PROMPT + 64)),
                  max_batch=max(most_rows, 1), pipeline_decode=False)
        engine = llm.engine
        spec = engine.spec
        kv_bytes_per_token = engine.cache.kv_bytes_per_token()
        weight_bytes = engine.model.parameter_bytes()
        clocks.start()

        def timed(fn, n):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            t0 = clocks.mark()
            start.record()
            for _ in range(n):
                fn()
            end.record()
            torch.cuda.synchronize()
            windows.append((t0, clocks.mark()))
            return start.elapsed_time(end)

        def decode_point(batch, steps, warmup, traced=False):
            """Device-timed decode: the contexts end at CONTEXT after the timed steps.
            ``traced``: afterwards one more step with the kernels' own clock readings
            (outside every timed region), summed per kernel."""
            begin = CONTEXT - steps - warmup
            slots = [engine.acquire_slot() for _ in range(batch)]
            fed = 0
            while fed < begin:  # fill the cache in chunks of at most 2,048 tokens per sequence
                n = min(PROMPT, begin - fed)
                per_step = max(1, 16384 // n)
                for i in range(0, batch, per_step):
                    engine.step([SequenceStep(s, [rng.randrange(vocab) for _ in range(n)], [])
                                 for s in slots[i:i + per_step]])
                fed += n
            dec = GraphDecoder(engine, batch, CONTEXT)
            engine.cache.reserve(slots, [CONTEXT] * batch)
            regions = []
            for rep in range(REPEATS):  # every region decodes the same positions again
                for r, s in enumerate(slots):
                    dec.set_row(r, s, rng.randrange(vocab), begin)
                dec.capture()
                for _ in range(warmup):
                    dec.launch()
                before = ops.launch_count()
                regions.append(timed(dec.launch, steps))
                launches = dec.launches_per_step * steps + (ops.launch_count() - before)
            ms = median(regions)
            kernels = None
            if traced:
                seen = GraphDecoder(engine, batch, CONTEXT)  # (its launches get slots of the trace at capture)
                for r, s in enumerate(slots):
                    seen.set_row(r, s, rng.randrange(vocab), begin)
                buf = ops.trace_begin(4096)
                seen.capture()  # the warm-up run takes slots as well; the captured launches the later half
                names = ops.trace_end()
                for _ in range(3):
                    seen.launch()
                torch.cuda.synchronize()
                ops.trace_clear()
                seen.launch()
                torch.cuda.synchronize()
                half = len(names) // 2
                kernels = kernel_times(names[half:], buf[half:2 * half].cpu().tolist())
            for s in slots:
                engine.release_slot(s)
            mean_context = CONTEXT - (steps + 1) / 2.0
            step_bytes = weight_bytes + batch * mean_context * kv_bytes_per_token
            return {"tok_s": batch * steps / (ms * 1e-3), "ms_per_step": ms / steps,
                    "launches": launches, "bytes_per_step": step_bytes,
                    "gbs": step_bytes / (ms / steps * 1e-3) / 1e9,
                    "spread": (max(regions) - min(regions)) / ms, "kernels": kernels}

        if args.timeline:
            if args.batch == 0:
                prefill_timeline(engine, args.timeline, rng, vocab)
            else:
                timeline(engine, args.batch, args.timeline, rng, vocab)
            clocks.stop()
            return 0
        main_point = decode_point(args.batch, K, W, traced=True)

        # -- prefill of 2,048 tokens ------------------------------------------------
        prompt = [rng.randrange(vocab) for _ in range(PROMPT)]

        def prefill_once():
            slot = engine.acquire_slot()
            engine.step([SequenceStep(slot, prompt, [PROMPT - 1])])
            engine.release_slot(slot)

        for _ in range(3):
            prefill_once()
        # regions of four prompts one after another: the host's preparation of the next
        # step runs under the GPU's work on this one, as in a server that has prompts waiting
        prefill_ms = median([timed(prefill_once, 4) for _ in range(REPEATS)]) / 4
        prefill_flops = engine.model.step_flops([PROMPT], [0], 1)  # what the parts say they compute
        prefill_rate = prefill_flops / (prefill_ms * 1e-3)
        prefill = {"value": PROMPT / (prefill_ms * 1e-3), "tokens": PROMPT, "ms": prefill_ms,
                   "frac": prefill_rate / (pk["bf16_tflops"] * 1e12),
                   "frac_of_sustained": prefill_rate / (pk["bf16_tflops_sustained"] * 1e12),
                   "tflops": prefill_rate / 1e12}

        # -- end to end: host tokens in and out every step -----------------------------
        e2e = None
        if not args.skip_e2e:
            e2e_new = E2E_STEPS + 1
            prompts = [[rng.randrange(vocab) for _ in range(CONTEXT - e2e_new)] for _ in range(args.batch)]
            llm.generate([p[:64] for p in prompts], max_new_tokens=4, stop_token_ids=())
            llm.backend._decoder(args.batch, CONTEXT, False).capture()  # the graph the timed run will launch
            stamps = []
            h2d0, d2h0 = llm.backend.h2d_bytes + engine.h2d_bytes, llm.backend.d2h_bytes
            first_done = {}

            def on_token(i, t):
                if i not in first_done:
                    first_done[i] = True
                    if len(first_done) == args.batch:
                        torch.cuda.synchronize()
                        stamps.append((time.perf_counter(), llm.backend.h2d_bytes + engine.h2d_bytes,
                                       llm.backend.d2h_bytes))
            t0 = clocks.mark()
            results = llm.generate(prompts, max_new_tokens=e2e_new, stop_token_ids=(), on_token=on_token)
            torch.cuda.synchronize()
            t_end = time.perf_counter()
            windows.append((t0, clocks.mark()))
            assert all(r.ok and len(r.token_ids) == e2e_new for r in results), \
                [r.error for r in results if not r.ok]
            t_first, h2d1, d2h1 = stamps[0]
            e2e_steps = e2e_new - 1
            e2e = {"value": args.batch * e2e_steps / (t_end - t_first), "unit": "tokens/s",
                   "h2d_bytes_per_step": (llm.backend.h2d_bytes + engine.h2d_bytes - h2d1) // e2e_steps,
                   "d2h_bytes_per_step": (llm.backend.d2h_bytes - d2h1) // e2e_steps,
                   "steps": e2e_steps}

        points = {}
        if not args.skip_points:
            p1 = decode_point(1, min(K, 256), W)
            p64 = decode_point(64, min(K, 64), W)
            points = {"decode_b1": p1["tok_s"], "decode_b64": p64["tok_s"],
                      "decode_b1_hbm_frac": p1["gbs"] / pk["hbm_gbs"],
                      "decode_b64_hbm_frac": p64["gbs"] / pk["hbm_gbs"]}
            # the regime of the reference's own published runs: one 3-token prompt, 32
            # greedy tokens, wall clock around generate() (median of 5 after 2 warm-ups)
            short = [rng.randrange(vocab) for _ in range(3)]
            walls = []
            for i in range(7):
                torch.cuda.synchronize()
                t_a = time.perf_counter()
                out = llm.generate([short], max_new_tokens=32, stop_token_ids=())
                torch.cuda.synchronize()
                if i >= 2:
                    walls.append(time.perf_counter() - t_a)
                assert out[0].ok and len(out[0].token_ids) == 32
            points["generate_3_plus_32_ms"] = sorted(walls)[len(walls) // 2] * 1e3
            points["generate_3_plus_32_tok_s"] = 32 / sorted(walls)[len(walls) // 2]
        clocks.stop()

    line = {
        "metric": f"decode tok/s @ batch {args.batch}, context {CONTEXT} ({shape_name} bf16)",
        "value": main_point["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": main_point["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded random weights and token ids)",
        "impl": "ours",
        "config": {"model": f"{shape_name} shape", "global_batch": args.batch, "seq_len": CONTEXT,
                   "parallelism": "single GPU", "prompt_len": PROMPT, "layers": cfg["num_hidden_layers"],
                   "layers_of_shape": full_layers, "hidden_size": cfg["hidden_size"],
                   "intermediate_size": cfg["intermediate_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"],
                   "vocab_size": vocab, "rope_theta": cfg["rope_theta"],
                   "rms_norm_eps": cfg["rms_norm_eps"], "tied_embeddings": True,
                   "cache_page_tokens": 64, "l2": "inputs larger than L2 (weights + KV per step)",
                   "peaks": pk["source"], "timing": f"median of {REPEATS} regions of K steps"},
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": main_point["gbs"], "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": main_point["gbs"] / pk["hbm_gbs"]},
        "points": points,
        "spread": main_point["spread"],
        "e2e": e2e,
        "gpu_launches": main_point["launches"],
        "kernels": main_point["kernels"],
        "clocks": clocks.summary(windows),
    }
    try:  # where the numbers were taken (NNIS's benchmarks carry such a record too)
        line["environment"] = {"gpu": torch.cuda.get_device_name(0), "cuda": torch.version.cuda,
                               "torch": torch.__version__, "python": sys.version.split()[0]}
    except Exception:  # the record is a courtesy; the measurement stands without it
        pass
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
