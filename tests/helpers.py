"""Shared by the tests: the tiny configurations, model folders made in a
temporary place, trace building and the comparison rules."""
from __future__ import annotations

import json
import os
import random
from typing import Dict, List, Sequence

import numpy as np
import torch

# Two tiny Llama configurations that differ in every size and option.
TINY_A = dict(architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=256,
              hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, max_position_embeddings=512, rms_norm_eps=1e-5,
              rope_theta=10000.0, hidden_act="silu", tie_word_embeddings=True,
              attention_bias=False, torch_dtype="float32", eos_token_id=7)
TINY_B = dict(architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=515,
              hidden_size=96, intermediate_size=272, num_hidden_layers=3, num_attention_heads=3,
              num_key_value_heads=1, head_dim=32, max_position_embeddings=384, rms_norm_eps=1e-6,
              rope_theta=500000.0, hidden_act="silu", tie_word_embeddings=False,
              attention_bias=True, mlp_bias=True, torch_dtype="bfloat16", eos_token_id=[3, 11])
# A third one whose hidden size is not heads * head_dim and no power of two anywhere.
TINY_C = dict(architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=1000,
              hidden_size=120, intermediate_size=200, num_hidden_layers=2, num_attention_heads=6,
              num_key_value_heads=3, head_dim=48, max_position_embeddings=640, rms_norm_eps=1e-5,
              rope_theta=100000.0, hidden_act="silu", tie_word_embeddings=True,
              attention_bias=False, torch_dtype="bfloat16")
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C}

# Rules of comparison, fixed once, both measured against the largest logit of
# the compared rows (at least 1).  float32: the plain implementation is float64,
# so what is left is the engine's float32 rounding, 1e-4 of the scale (the bound
# NNIS uses against its own oracle: crates/nnis-model/examples/compare_tiny_llama.rs:49-50).
# bfloat16: the engine and the plain implementation round at the same tensor
# boundaries; what is left is accumulation order and one-ulp flips of bfloat16
# roundings (2^-8 relative) carried through the layers.
F32_REL_TO_MAX = 1e-4
BF16_REL_TO_MAX = 0.03


def make_model(tmp_dir: str, config: dict, seed: int, healthy: bool = True) -> str:
    """A model folder with random weights.  ``healthy`` scales projections by
    their fan-in so that activations, scores and logits are of order one; with
    N(0, 0.02) everywhere attention is nearly uniform and hides faults."""
    from nnis_b200.weights import write_random_model
    if healthy:
        return write_random_model(config, seed, tmp_dir, std=1.0, norm_std=0.1, std_by_fan_in=True)
    return write_random_model(config, seed, tmp_dir)


def load_plain_weights(model_dir: str, as_bf16: bool) -> Dict[str, torch.Tensor]:
    """Through the safetensors package, not the framework's reader."""
    from safetensors.torch import load_file
    w = load_file(os.path.join(model_dir, "model.safetensors"))
    if as_bf16:
        return {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    return {k: v.float() for k, v in w.items()}


def read_config_json(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def random_tokens(rng: random.Random, n: int, vocab: int) -> List[int]:
    return [rng.randrange(vocab) for _ in range(n)]


def check_logits(got: np.ndarray, want: torch.Tensor, dtype: str, what: str = "") -> None:
    want = want.detach().float().numpy()
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    diff = np.abs(got - want)
    rel = F32_REL_TO_MAX if dtype == "float32" else BF16_REL_TO_MAX
    bad = diff > rel * max(float(np.abs(want).max()), 1.0)
    if bad.any():
        i = np.argwhere(bad)[0]
        raise AssertionError(f"{what}: {int(bad.sum())} of {bad.size} logits differ; first at row "
                             f"{i[0]}, col {i[1]}: got {got[tuple(i)]!r}, want {want[tuple(i)]!r}; "
                             f"max abs diff {diff.max():.3e}, max |want| {np.abs(want).max():.3e}")


def read_step(out_dir: str, step, vocab: int) -> np.ndarray:
    return np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4").reshape(-1, vocab)


class TraceBuilder:
    """Builds the JSON lines of a replay and remembers which (request,
    position) each written row belongs to."""

    def __init__(self):
        self.lines: List[str] = []
        self.rows: Dict[int, List] = {}  # step -> [(request id, position in its sequence)]
        self._step = 0
        self._fed: Dict[str, int] = {}

    def step(self, entries: Sequence, end: Sequence[str] = ()):
        """entries: (id, tokens, want places among these tokens)."""
        rec = {"step": self._step, "entries": [], "end": list(end)}
        rows = []
        for rid, tokens, want in entries:
            start = self._fed.get(rid, 0)
            rec["entries"].append({"id": rid, "tokens": list(tokens), "want": list(want)})
            rows.extend((rid, start + w) for w in want)
            self._fed[rid] = start + len(tokens)
        for rid in end:
            self._fed.pop(rid, None)
        if rows:
            self.rows[self._step] = rows
        self.lines.append(json.dumps(rec))
        self._step += 1
        return self._step - 1


def ragged_batches(rng, vocab, trace, sequences, batches):
    """Each batch: prompts of unequal lengths in one step, then one token each;
    a request ends when its tokens are used up, so shorter ones end earlier.
    ``batches``: per batch a list of (prompt length, total length)."""
    for b, shape in enumerate(batches):
        reqs = {}
        for j, (prompt_len, total) in enumerate(shape):
            rid = f"b{b}r{j}"
            sequences[rid] = random_tokens(rng, total, vocab)
            reqs[rid] = prompt_len
        fed = dict(reqs)
        ends = [rid for rid in reqs if fed[rid] == len(sequences[rid])]
        trace.step([(rid, sequences[rid][:n], [n - 1]) for rid, n in reqs.items()], end=ends)
        live = [rid for rid in reqs if rid not in ends]
        while live:
            entries = [(rid, sequences[rid][fed[rid]:fed[rid] + 1], [0]) for rid in live]
            for rid in live:
                fed[rid] += 1
            ends = [rid for rid in live if fed[rid] == len(sequences[rid])]
            trace.step(entries, end=ends)
            live = [rid for rid in live if rid not in ends]


def three_cuts(rng, vocab, whole=(1, 2, 33, 64, 65, 150), last32=(33, 70, 129),
               batches=([(5, 13), (9, 12), (17, 40)], [(1, 13), (7, 8), (20, 32), (33, 45)],
                        [(70, 75), (3, 3), (64, 66), (2, 80), (31, 33)])):
    """One trace with the three ways of cutting work that every configuration is
    held to: each request alone and whole (all positions wanted); a request with
    its last 32 tokens one by one; batches of unequal lengths one after another,
    whose shorter requests end earlier, so that slots and pages are used again.
    Returns (trace, sequences by request id)."""
    sequences, trace = {}, TraceBuilder()
    for i, n in enumerate(whole):
        rid = f"w{i}"
        sequences[rid] = random_tokens(rng, n, vocab)
        trace.step([(rid, sequences[rid], range(n))], end=[rid])
    for i, n in enumerate(last32):
        rid = f"l{i}"
        toks = sequences[rid] = random_tokens(rng, n, vocab)
        head = n - 32
        trace.step([(rid, toks[:head], [head - 1])])
        for t in range(head, n):
            trace.step([(rid, toks[t:t + 1], [0])], end=[rid] if t == n - 1 else [])
    ragged_batches(rng, vocab, trace, sequences, batches)
    return trace, sequences


def replay_against_plain(engine, model_dir: str, dtype: str, trace: "TraceBuilder", sequences,
                         out_dir: str, what: str) -> None:
    """Replay ``trace`` through ``engine`` and hold every written row to the plain
    implementation's logits of the same request and position; afterwards the cache
    must hold nothing."""
    import plain_llama
    from nnis_b200.engine.replay import replay
    replay(engine, trace.lines, out_dir)
    usage = engine.cache.usage()
    assert usage["slots_held"] == 0 and not any(usage["pages_held"]), usage
    engine.cache.check()
    cfg = read_config_json(model_dir)
    bf = dtype == "bfloat16"
    w = load_plain_weights(model_dir, as_bf16=bf)
    plain = {}
    for step, rows in trace.rows.items():
        got = read_step(out_dir, step, cfg["vocab_size"])
        for rid, _ in rows:
            if rid not in plain:
                plain[rid] = plain_llama.forward(cfg, w, sequences[rid], emulate_bf16=bf)
        want = torch.stack([plain[rid][pos] for rid, pos in rows])
        check_logits(got, want, dtype, f"{what} {dtype} step {step}")
