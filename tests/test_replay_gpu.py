"""Replay through the engine against the plain implementation, in float32 and
in bfloat16: requests whole, with the last 32 tokens one by one, in batches of
unequal lengths one after another (slots used again), long decoding, the first
tokens of a sequence, and once through bin/trace_run as a program."""
import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_llama as P
from helpers import (CONFIGS, TraceBuilder, check_logits, load_plain_weights, make_model,
                     ragged_batches, random_tokens, read_config_json, read_step)

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        d = make_model(str(tmp_path_factory.mktemp(f"model{name}")), cfg, seed=100 + i)
        out[name] = d
    return out


_engines = {}
_plain = {}


def engine_for(models, name, dtype, max_tokens=64 * 64):
    from nnis_b200.engine import Engine
    key = (name, dtype)
    if key not in _engines:
        _engines[key] = Engine.from_dir(models[name], dtype=dtype, max_tokens=max_tokens)
    return _engines[key]


def plain_logits(models, name, dtype, tokens):
    """All-position logits of one sequence, cached per (model, dtype, tokens)."""
    key = (name, dtype, tuple(tokens))
    if key not in _plain:
        bf = dtype == "bfloat16"
        w = load_plain_weights(models[name], as_bf16=bf)
        _plain[key] = P.forward(read_config_json(models[name]), w, tokens, emulate_bf16=bf)
    return _plain[key]


def run_and_check(models, name, dtype, trace: TraceBuilder, sequences, tmp_path, what):
    from nnis_b200.engine.replay import replay
    engine = engine_for(models, name, dtype)
    out = str(tmp_path / f"out_{name}_{dtype}")
    replay(engine, trace.lines, out)
    assert engine.cache.usage()["slots_held"] == 0 and engine.cache.usage()["pages_held"] == [0]
    engine.cache.check()
    vocab = CONFIGS[name]["vocab_size"]
    for step, rows in trace.rows.items():
        got = read_step(out, step, vocab)
        want = torch.stack([plain_logits(models, name, dtype, sequences[rid])[pos]
                            for rid, pos in rows])
        check_logits(got, want, dtype, f"{what} {name} {dtype} step {step}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_each_request_alone_and_whole(models, name, dtype, tmp_path):
    rng = random.Random(1)
    vocab = CONFIGS[name]["vocab_size"]
    sequences = {f"r{i}": random_tokens(rng, n, vocab) for i, n in enumerate((1, 2, 33, 64, 65, 150))}
    trace = TraceBuilder()
    for rid, toks in sequences.items():
        trace.step([(rid, toks, range(len(toks)))], end=[rid])
    run_and_check(models, name, dtype, trace, sequences, tmp_path, "whole")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_last_32_tokens_one_by_one(models, name, dtype, tmp_path):
    rng = random.Random(2)
    vocab = CONFIGS[name]["vocab_size"]
    sequences = {f"r{i}": random_tokens(rng, n, vocab) for i, n in enumerate((33, 70, 129))}
    trace = TraceBuilder()
    for rid, toks in sequences.items():
        head = len(toks) - 32
        trace.step([(rid, toks[:head], [head - 1])])
        for t in range(head, len(toks)):
            trace.step([(rid, toks[t:t + 1], [0])], end=[rid] if t == len(toks) - 1 else [])
    run_and_check(models, name, dtype, trace, sequences, tmp_path, "last32")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_unequal_batches_one_after_another(models, name, dtype, tmp_path):
    rng = random.Random(3)
    vocab = CONFIGS[name]["vocab_size"]
    sequences, trace = {}, TraceBuilder()
    ragged_batches(rng, vocab, trace, sequences, [
        [(5, 13), (9, 12), (17, 40)],
        [(1, 13), (7, 8), (20, 32), (33, 45)],
        [(70, 75), (3, 3), (64, 66), (2, 80), (31, 33)],
    ])
    run_and_check(models, name, dtype, trace, sequences, tmp_path, "ragged")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_crosses_pages(models, dtype, tmp_path):
    name = "A"
    rng = random.Random(4)
    toks = random_tokens(rng, 300, CONFIGS[name]["vocab_size"])
    sequences = {"long": toks}
    trace = TraceBuilder()
    trace.step([("long", toks[:3], [0, 1, 2])])
    for t in range(3, len(toks)):
        trace.step([("long", toks[t:t + 1], [0])], end=["long"] if t == len(toks) - 1 else [])
    run_and_check(models, name, dtype, trace, sequences, tmp_path, "long")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_first_tokens_of_a_sequence(models, name, dtype, tmp_path):
    """A prompt of one token, then single tokens: the first decoded positions."""
    rng = random.Random(5)
    vocab = CONFIGS[name]["vocab_size"]
    sequences = {"x": random_tokens(rng, 6, vocab), "y": random_tokens(rng, 5, vocab)}
    trace = TraceBuilder()
    trace.step([("x", sequences["x"][:1], [0]), ("y", sequences["y"][:1], [0])])
    for t in range(1, 6):
        entries = [("x", sequences["x"][t:t + 1], [0])]
        if t < 5:
            entries.append(("y", sequences["y"][t:t + 1], [0]))
        trace.step(entries, end=(["y"] if t == 4 else []) + (["x"] if t == 5 else []))
    run_and_check(models, name, dtype, trace, sequences, tmp_path, "first")


def test_steps_that_want_nothing_write_nothing(models, tmp_path):
    from nnis_b200.engine.replay import replay
    engine = engine_for(models, "A", "float32")
    trace = TraceBuilder()
    toks = list(range(10))
    trace.step([("q", toks[:6], [])])
    trace.step([("q", toks[6:7], [0])], end=["q"])
    out = str(tmp_path / "o")
    replay(engine, trace.lines, out)
    assert sorted(os.listdir(out)) == ["1.f32"]
    got = read_step(out, 1, 256)
    check_logits(got, plain_logits(models, "A", "float32", toks[:7])[6:7], "float32", "silent prefill")


def test_bad_requests_are_refused_before_anything_runs(models):
    from nnis_b200.cache import CacheFull, SlotError
    from nnis_b200.engine import SequenceStep, StepError
    engine = engine_for(models, "A", "float32")
    slot = engine.acquire_slot()
    try:
        with pytest.raises(StepError, match="vocabulary"):
            engine.step([SequenceStep(slot, [1, 256], [0])])
        with pytest.raises(StepError, match="wanted place"):
            engine.step([SequenceStep(slot, [1, 2], [2])])
        with pytest.raises(StepError, match="at least one token"):
            engine.step([SequenceStep(slot, [], [])])
        with pytest.raises(SlotError):
            engine.step([SequenceStep(slot, [1], [0]), SequenceStep(slot, [2], [0])])
        with pytest.raises(CacheFull):
            engine.step([SequenceStep(slot, [1] * 513, [0])])  # beyond max_position_embeddings
        assert engine.cache.length(slot) == 0
    finally:
        engine.release_slot(slot)


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_run_as_a_program(models, dtype, tmp_path):
    name = "B"
    rng = random.Random(6)
    vocab = CONFIGS[name]["vocab_size"]
    sequences, trace = {}, TraceBuilder()
    ragged_batches(rng, vocab, trace, sequences, [[(4, 9), (11, 12)], [(6, 8)]])
    out = str(tmp_path / "out")
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", models[name], "--dtype",
         dtype, "--out", out, "--max-tokens", "256"],
        input="\n".join(trace.lines) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split("\n")[:-1] == [f"done {i}" for i in range(len(trace.lines))]
    for step, rows in trace.rows.items():
        got = read_step(out, step, vocab)
        want = torch.stack([plain_logits(models, name, dtype, sequences[rid])[pos]
                            for rid, pos in rows])
        check_logits(got, want, dtype, f"program {dtype} step {step}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_recurring_prompt_shapes_are_replayed_from_a_graph(models, dtype, tmp_path):
    """A large prompt step whose shape comes again is captured and then replayed:
    other tokens, other slots and pages each time, same rules."""
    name = "A"
    rng = random.Random(9)
    vocab = CONFIGS[name]["vocab_size"]
    sequences, trace = {}, TraceBuilder()
    hold = random_tokens(rng, 70, vocab)  # keeps a slot and two pages busy so pages differ per run
    sequences["hold"] = hold
    trace.step([("hold", hold, [69])])
    for i in range(4):
        a, b = random_tokens(rng, 300, vocab), random_tokens(rng, 41, vocab)
        sequences[f"a{i}"], sequences[f"b{i}"] = a, b
        trace.step([(f"a{i}", a[:290], [0, 150, 289]), (f"b{i}", b[:40], [39])])
        trace.step([(f"a{i}", a[290:291], [0]), (f"b{i}", b[40:41], [0])], end=[f"b{i}"])
        trace.step([(f"a{i}", a[291:300], range(9))], end=[f"a{i}"])
    trace.step([("hold", [1], [])], end=["hold"])
    sequences["hold"] = hold + [1]
    engine = engine_for(models, name, dtype)
    before = len(engine._step_graphs)
    run_and_check(models, name, dtype, trace, sequences, tmp_path, "graph replay")
    assert len(engine._step_graphs) > before
    assert any(e["graph"] is not None for e in engine._step_graphs.values())


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompts_in_portions_give_the_logits_of_one_step(models, dtype):
    """Long batches of prompts are run as several steps of a bounded number of tokens;
    the cuts fall inside sequences, pages and tiles and change nothing."""
    from nnis_b200.engine import SequenceStep
    name = "B"
    rng = random.Random(12)
    vocab = CONFIGS[name]["vocab_size"]
    engine = engine_for(models, name, dtype)
    seqs = [random_tokens(rng, n, vocab) for n in (70, 5, 131, 64)]
    wants = [[69, 0, 33], [4], [0, 64, 130, 65], []]
    for limit in (48, 64, 1000):
        slots = [engine.acquire_slot() for _ in seqs]
        got = engine.step_in_portions([SequenceStep(s, t, w) for s, t, w in zip(slots, seqs, wants)], limit)
        want = torch.stack([plain_logits(models, name, dtype, t)[w] for t, ws in zip(seqs, wants) for w in ws])
        check_logits(got.cpu().numpy(), want, dtype, f"portions of {limit}")
        assert [engine.cache.length(s) for s in slots] == [len(t) for t in seqs]
        for s in slots:
            engine.release_slot(s)
    assert engine.cache.usage()["pages_held"] == [0]
