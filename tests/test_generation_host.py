"""The generation loop's decisions with a scripted backend, the host sampler,
and the command line's rules (no GPU)."""
import os

import numpy as np
import pytest

import plain_llama as P
from nnis_b200.cli.main import UsageError, parse_args
from nnis_b200.engine.generate import (GenerationConfig, GenerationRequest, Generator,
                                       pages_needed, plan_batches)
from nnis_b200.sampling import HostLogitSampler, SamplingConfig, SamplingError, SplitMix64

VOCAB = 50


class ScriptedBackend:
    """The next token of a sequence is (sum of its tokens) % VOCAB, so every
    sequence has a known continuation; slots and steps are recorded."""

    def __init__(self, n_slots=8, fail_on_step=None):
        self.free = list(range(n_slots))
        self.held = {}
        self.steps = []
        self.fail_on_step = fail_on_step
        self.max_held = 0

    def acquire_slot(self):
        slot = min(self.free)
        self.free.remove(slot)
        self.held[slot] = []
        self.max_held = max(self.max_held, len(self.held))
        return slot

    def release_slot(self, slot):
        assert slot in self.held, "slot freed twice or never held"
        del self.held[slot]
        self.free.append(slot)

    def step(self, batch, need_logits=True):
        if self.fail_on_step is not None and len(self.steps) == self.fail_on_step:
            self.steps.append("boom")
            raise RuntimeError("boom")
        self.steps.append([(s.slot, len(s.tokens)) for s in batch])
        rows = []
        for s in batch:
            assert s.slot in self.held
            self.held[s.slot].extend(s.tokens)
            row = np.full(VOCAB, -1.0, dtype=np.float32)
            row[sum(self.held[s.slot]) % VOCAB] = 5.0
            rows.append(row)
        return np.stack(rows)

    def greedy(self, logits):
        return [int(np.argmax(r)) for r in logits]

    def host_rows(self, logits, rows):
        return logits[list(rows)]


def expected(prompt, n, stops=()):
    seq, out = list(prompt), []
    for _ in range(n):
        t = sum(seq) % VOCAB
        out.append(t)
        seq.append(t)
        if t in stops:
            break
    return out


def gen(backend, max_batch=4, max_tokens=64 * 64, max_positions=1000):
    return Generator(backend, VOCAB, max_positions, max_batch, max_tokens)


def test_unequal_prompts_stop_tokens_and_early_ends():
    b = ScriptedBackend()
    reqs = [GenerationRequest([1, 2, 3], GenerationConfig(6)),
            GenerationRequest([7], GenerationConfig(2)),
            GenerationRequest([4, 4], GenerationConfig(9, stop_token_ids=(expected([4, 4], 3)[2],)))]
    res = gen(b).generate(reqs)
    assert res[0].token_ids == expected([1, 2, 3], 6) and res[0].finish_reason == "length"
    assert res[1].token_ids == expected([7], 2) and res[1].finish_reason == "length"
    assert res[2].token_ids == expected([4, 4], 3) and res[2].finish_reason == "stop"
    # one prompt step with all three, then the batch shrinks as sequences end;
    # the last token of a sequence is never run
    assert [len(s) for s in b.steps] == [3, 3, 2, 1, 1, 1]
    assert b.steps[0] == [(0, 3), (1, 1), (2, 2)]
    assert not b.held and sorted(b.free) == list(range(8))


def test_batches_follow_one_another_and_reuse_slots():
    b = ScriptedBackend(n_slots=2)
    reqs = [GenerationRequest([i + 1], GenerationConfig(3)) for i in range(5)]
    res = gen(b, max_batch=2).generate(reqs)
    assert [r.token_ids for r in res] == [expected([i + 1], 3) for i in range(5)]
    assert b.max_held == 2 and not b.held
    assert [len(s) for s in b.steps] == [2, 2, 2, 2, 2, 2, 1, 1, 1]


def test_plan_respects_pages():
    reqs = [GenerationRequest([0] * 60, GenerationConfig(5)),   # 64 positions -> 1 page
            GenerationRequest([0] * 60, GenerationConfig(6)),   # 65 -> 2 pages
            GenerationRequest([0] * 10, GenerationConfig(5))]
    assert [pages_needed(r) for r in reqs] == [1, 2, 1]
    assert plan_batches(reqs, [True] * 3, 8, 3) == [[0, 1], [2]]
    assert plan_batches(reqs, [True, False, True], 8, 3) == [[0, 2]]
    assert plan_batches(reqs, [True] * 3, 1, 100) == [[0], [1], [2]]


def test_bad_requests_fail_alone():
    b = ScriptedBackend()
    reqs = [GenerationRequest([], GenerationConfig(2)),
            GenerationRequest([1, VOCAB], GenerationConfig(2)),
            GenerationRequest([1], GenerationConfig(2000)),
            GenerationRequest([1], GenerationConfig(2), SamplingConfig(seed=1, temperature=0.0)),
            GenerationRequest([1], GenerationConfig(0)),
            GenerationRequest([5], GenerationConfig(2))]
    res = gen(b).generate(reqs)
    assert [r.ok for r in res] == [False] * 5 + [True]
    assert "empty" in res[0].error and "vocabulary" in res[1].error and "positions" in res[2].error
    assert "temperature" in res[3].error and "max_new_tokens" in res[4].error
    assert res[5].token_ids == expected([5], 2)
    assert b.steps[0] == [(0, 1)]


def test_a_failing_step_is_met_by_running_its_requests_alone():
    """Each request is a failure domain of its own (crates/nnis-model/src/session_batch.rs:82-111):
    when a step of a batch fails, its unfinished requests run again one by one; the one
    that fails alone gets the error, the others their tokens, and no slot is lost."""
    b = ScriptedBackend(n_slots=2, fail_on_step=1)  # fails once: both requests succeed alone
    reqs = [GenerationRequest([i + 1], GenerationConfig(3)) for i in range(3)]
    res = gen(b, max_batch=2).generate(reqs)
    assert [r.token_ids for r in res] == [expected([i + 1], 3) for i in range(3)]
    assert all(r.ok and r.finish_reason == "length" for r in res) and not b.held
    assert b.steps[:3] == [[(0, 1), (1, 1)], "boom", [(0, 1)]]

    class Poisoned(ScriptedBackend):  # every step that holds token 13 fails
        def step(self, batch, need_logits=True):
            if any(13 in list(s.tokens) + self.held.get(s.slot, []) for s in batch):
                raise RuntimeError("poison")
            return super().step(batch, need_logits)
    b = Poisoned(n_slots=4)
    reqs = [GenerationRequest([1], GenerationConfig(3)), GenerationRequest([13], GenerationConfig(3)),
            GenerationRequest([2, 2], GenerationConfig(4))]
    seen = []
    res = gen(b).generate(reqs, on_token=lambda i, t: seen.append((i, t)))
    assert res[0].token_ids == expected([1], 3) and res[2].token_ids == expected([2, 2], 4)
    assert not res[1].ok and "poison" in res[1].error and res[1].finish_reason == "error"
    assert not b.held and sorted(b.free) == list(range(4))
    # the callback saw every token of the good requests once, in order
    assert [t for i, t in seen if i == 0] == expected([1], 3)
    assert [t for i, t in seen if i == 2] == expected([2, 2], 4)

    # a failure in the middle of decoding: tokens already shown are not shown again
    b = ScriptedBackend(n_slots=2, fail_on_step=2)
    seen = []
    reqs = [GenerationRequest([3], GenerationConfig(4)), GenerationRequest([4], GenerationConfig(4))]
    res = gen(b).generate(reqs, on_token=lambda i, t: seen.append((i, t)))
    assert [r.token_ids for r in res] == [expected([3], 4), expected([4], 4)]
    assert [t for i, t in seen if i == 0] == expected([3], 4)
    assert [t for i, t in seen if i == 1] == expected([4], 4)


def test_the_callback_can_stop_one_request_of_a_batch():
    """crates/nnis-model/src/streaming.rs:5-12,59-70: Stop ends that request cleanly
    after the token it was called for; the slot goes back and the others go on."""
    from nnis_b200.engine.generate import StreamControl
    b = ScriptedBackend()
    reqs = [GenerationRequest([1, 2, 3], GenerationConfig(6)), GenerationRequest([7], GenerationConfig(6))]

    def on_token(i, t, seen={0: 0, 1: 0}):
        seen[i] += 1
        return StreamControl.STOP if (i == 1 and seen[i] == 2) else None
    res = gen(b).generate(reqs, on_token)
    assert res[0].token_ids == expected([1, 2, 3], 6) and res[0].finish_reason == "length"
    assert res[1].token_ids == expected([7], 2) and res[1].finish_reason == "stop"
    assert not b.held
    # stopping at the very first token
    b = ScriptedBackend()
    res = gen(b).generate(reqs[:1], lambda i, t: StreamControl.STOP)
    assert res[0].token_ids == expected([1, 2, 3], 1) and res[0].finish_reason == "stop" and not b.held


def test_a_request_on_its_callers_slot_executes_every_token_and_keeps_the_slot():
    """crates/nnis-model/src/runtime.rs:814-846,1264-1268: after generation the
    session holds prompt + emitted tokens, the last one and a stop token included."""
    from nnis_b200.engine.generate import StreamControl
    for stops, n, reason in (((), 4, "length"), ((expected([5, 6], 2)[1],), 2, "stop")):
        b = ScriptedBackend()
        slot = b.acquire_slot()
        req = GenerationRequest([5, 6], GenerationConfig(4, stop_token_ids=stops), slot=slot)
        res = gen(b).generate([req])[0]
        assert res.token_ids == expected([5, 6], n, stops) and res.finish_reason == reason
        assert b.held[slot] == [5, 6] + res.token_ids  # everything emitted was executed
        assert list(b.held) == [slot]                  # and the slot is still the caller's
    # stopped by the callback: the token it was shown has been executed already
    b = ScriptedBackend()
    slot = b.acquire_slot()
    held_when_called = []

    def on_token(i, t):
        held_when_called.append(list(b.held[slot]))
        return StreamControl.STOP if len(held_when_called) == 3 else StreamControl.CONTINUE
    res = gen(b).generate([GenerationRequest([5, 6], GenerationConfig(9), slot=slot)], on_token)[0]
    assert res.token_ids == expected([5, 6], 3) and res.finish_reason == "stop"
    assert b.held[slot] == [5, 6] + res.token_ids
    assert [h[-1] for h in held_when_called] == res.token_ids
    # it goes on after what the slot holds already (start positions count for the capacity)
    b = ScriptedBackend()
    slot = b.acquire_slot()
    b.held[slot] = [9, 9]
    res = gen(b).generate([GenerationRequest([1], GenerationConfig(2), slot=slot, start=2)])[0]
    assert res.token_ids == [19, 38] and b.held[slot] == [9, 9, 1, 19, 38]
    res = gen(b, max_positions=8).generate([GenerationRequest([1], GenerationConfig(2), slot=slot, start=6)])[0]
    assert not res.ok and "positions" in res.error


def test_a_sampler_that_refuses_its_logits_ends_that_request_only():
    class NaNForSlot(ScriptedBackend):
        def step(self, batch, need_logits=True):
            out = super().step(batch, need_logits)
            for r, s in enumerate(batch):
                if 42 in self.held[s.slot]:
                    out[r, :] = np.nan
            return out
    b = NaNForSlot()
    reqs = [GenerationRequest([42], GenerationConfig(3), SamplingConfig(seed=1).with_top_k(1)),
            GenerationRequest([3], GenerationConfig(3), SamplingConfig(seed=2).with_top_k(1))]
    res = gen(b).generate(reqs)
    assert not res[0].ok and "Sampling" in res[0].error and res[0].token_ids == []
    assert res[1].ok and res[1].token_ids == expected([3], 3) and not b.held


def test_sampled_requests_use_their_own_seeded_sampler():
    b = ScriptedBackend()
    reqs = [GenerationRequest([3], GenerationConfig(4), SamplingConfig(seed=9).with_top_k(1)),
            GenerationRequest([3], GenerationConfig(4))]
    res = gen(b).generate(reqs)
    assert res[0].token_ids == res[1].token_ids == expected([3], 4)  # top-k 1 is greedy
    seen = []
    gen(ScriptedBackend()).generate(reqs, on_token=lambda i, t: seen.append((i, t)))
    assert [t for i, t in seen if i == 0] == expected([3], 4)


# ---------------------------------------------------------------------------
def test_splitmix_and_frozen_sequence():
    # crates/nnis-model/src/sampling.rs:326-333
    s = HostLogitSampler(SamplingConfig.seeded(42), 4)
    assert [s.sample([0.0] * 4) for _ in range(10)] == [2, 0, 1, 1, 0, 3, 0, 3, 1, 2]
    a, b = SplitMix64(7), P.PlainSplitMix64(7)
    assert [a.next_u64() for _ in range(5)] == [b.next_u64() for _ in range(5)]


def test_sampler_rules_of_the_reference():
    assert HostLogitSampler(SamplingConfig.seeded(7).with_top_k(1), 4).sample([1, 4, 4, -2]) == 1
    s = HostLogitSampler(SamplingConfig.seeded(9).with_top_p(0.1), 3)
    assert all(s.sample([3.0, 2.0, 1.0]) == 0 for _ in range(32))
    s = HostLogitSampler(SamplingConfig.seeded(123).with_top_k(2), 4)
    assert all(s.sample([4.0, 3.0, 2.0, 1.0]) <= 1 for _ in range(64))
    s = HostLogitSampler(SamplingConfig.seeded(1), 2)
    for bad in ([1.0], [1.0, float("nan")], [1.0, float("inf")]):
        with pytest.raises(SamplingError):
            s.sample(bad)
    for cfg, vocab in ((SamplingConfig.seeded(1), 0),
                       (SamplingConfig.seeded(1).with_temperature(0.0), 4),
                       (SamplingConfig.seeded(1).with_temperature(float("nan")), 4),
                       (SamplingConfig.seeded(1).with_top_k(0), 4),
                       (SamplingConfig.seeded(1).with_top_k(5), 4),
                       (SamplingConfig.seeded(1).with_top_p(0.0), 4),
                       (SamplingConfig.seeded(1).with_top_p(1.1), 4),
                       (SamplingConfig.seeded(-1), 4)):
        with pytest.raises(SamplingError):
            cfg.validate(vocab)


def test_host_sampler_equals_the_plain_sampler():
    rng = np.random.default_rng(0)
    for seed, t, k, p in ((1, 1.0, None, None), (2, 0.7, 5, None), (3, 1.3, None, 0.8),
                          (4, 0.5, 12, 0.6), (5, 2.0, 40, 0.99)):
        cfg = SamplingConfig(seed=seed, temperature=t, top_k=k, top_p=p)
        ours, theirs = HostLogitSampler(cfg, 40), P.PlainSplitMix64(seed)
        for _ in range(50):
            logits = rng.normal(size=40).astype(np.float32)
            logits[rng.integers(40)] = logits[rng.integers(40)]  # a tie now and then
            assert ours.sample(logits) == P.plain_sample(logits, theirs, t, k, p)


# ---------------------------------------------------------------------------
def test_cli_rules():
    a = parse_args(["generate", "--model", "m", "--tokenizer", "t", "--prompt", "hi"])
    assert (a.device_ordinal, a.max_new_tokens, a.sample) == (0, 16, False)
    a = parse_args(["generate", "--model", "m", "--prompt-ids", "1,2,3", "--sample", "--seed", "5",
                    "--temperature", "0.5", "--top-k", "3", "--top-p", "0.9", "--stream",
                    "--max-new-tokens", "4", "--device", "1", "--dtype", "float32"])
    assert a.prompt_ids == [[1, 2, 3]] and a.seeds == [5] and a.stream and a.dtype == "float32"
    assert parse_args(["--help"]) is None
    bad = [
        ["generate", "--model", "m", "--prompt-ids", "1", "--seed", "5"],          # needs --sample
        ["generate", "--model", "m", "--prompt-ids", "1", "--temperature", "1"],
        ["generate", "--model", "m", "--prompt-ids", "1", "--stream"],
        ["generate", "--model", "m", "--prompt-ids", "1", "--sample"],               # needs --seed
        ["generate", "--model", "m", "--prompt", "hi"],                              # tokenizer
        ["generate", "--prompt-ids", "1"],                                           # model
        ["generate", "--model", "m"],                                                # prompt
        ["generate", "--model", "m", "--prompt-ids", "1", "--max-new-tokens", "0"],
        ["generate", "--model", "m", "--prompt-ids", "1", "--device", "-1"],
        ["generate", "--model", "m", "--prompt-ids", "1", "--sample", "--seed", "1", "--top-p", "1.5"],
        ["generate", "--model", "m", "--prompt-ids", "1", "--sample", "--seed", "1", "--temperature", "0"],
        ["generate", "--model", "m", "--prompt-ids", "1", "--bogus", "1"],
        ["generate", "--model", "m", "--prompt-ids", "1", "--model", "n"],
        ["generate-batch", "--model", "m", "--prompt-ids", "1", "--prompt-ids", "2", "--seed", "1"],
        ["generate-batch", "--model", "m", "--prompt-ids", "1", "--seed", "1", "--sample"],
        ["frobnicate"],
    ]
    for argv in bad:
        with pytest.raises(UsageError):
            parse_args(argv)
    a = parse_args(["generate-batch", "--model", "m", "--prompt-ids", "1", "--prompt-ids", "2,3",
                    "--seed", "1", "--seed", "2", "--json"])
    assert a.seeds == [1, 2] and a.json and a.sample and len(a.prompt_ids) == 2


def test_cli_validate_checks_a_folder_without_a_gpu(tmp_path):
    """`nnis validate`: flag rules of NNIS's `nnis-hf validate`, a ready report for a good
    folder, and the loader's one error as the blocker of a bad one."""
    import io
    import json
    import os

    from helpers import TINY_A, make_model
    from nnis_b200.cli.main import main, validate
    from nnis_b200.weights import SafetensorsFile, write_safetensors
    with pytest.raises(UsageError, match="--model is required"):
        parse_args(["validate"])
    with pytest.raises(UsageError, match="--output requires --json"):
        parse_args(["validate", "--model", "m", "--output", "r.json"])
    with pytest.raises(UsageError, match="unknown validate argument"):
        parse_args(["validate", "--model", "m", "--prompt", "x"])
    good = make_model(str(tmp_path / "good"), TINY_A, seed=1)
    args = parse_args(["validate", "--model", good, "--json"])
    out = io.StringIO()
    assert validate(args, out) == 0
    report = json.loads(out.getvalue())
    assert report["ready"] and report["blocker"] is None and report["vocab_size"] == TINY_A["vocab_size"]
    assert report["weights"]["weight_files"] == ["model.safetensors"]
    assert report["weights"]["recognized_tensors"] > 0 and report["layers"] == TINY_A["num_hidden_layers"]
    # the report goes to a file whole, and never over an existing one
    target = str(tmp_path / "report.json")
    assert main(["validate", "--model", good, "--json", "--output", target]) == 0
    assert json.load(open(target))["ready"]
    assert main(["validate", "--model", good, "--json", "--output", target]) == 1
    assert not [n for n in os.listdir(tmp_path) if ".tmp-" in n]
    # a folder whose weights do not fit: one tensor gone, one of another shape
    bad = make_model(str(tmp_path / "bad"), TINY_A, seed=1)
    path = os.path.join(bad, "model.safetensors")
    with SafetensorsFile(path) as f:
        tensors = {n: f.tensor(n) for n in f.names()}
    gone = sorted(n for n in tensors if n.endswith("down_proj.weight"))[0]
    del tensors[gone]
    tensors["model.norm.weight"] = tensors["model.norm.weight"][:-1].clone()
    write_safetensors(path, tensors)
    out = io.StringIO()
    assert validate(parse_args(["validate", "--model", bad]), out) == 1
    text = out.getvalue()
    assert text.startswith("NNIS_PREFLIGHT_BLOCKED") and gone in text and "model.norm.weight" in text
    # no config.json at all
    assert main(["validate", "--model", str(tmp_path / "nothing")]) == 1


def test_process_entry_point_checks_bounds_and_records(tmp_path):
    """`nnis_b200.execute`: the request rules of NNIS's process wrapper, a child that is
    ended at its deadline, output kept whole, and a record that never replaces a file."""
    import json
    import os
    import stat
    import time

    from nnis_b200 import ProcessContractError, execute
    model = tmp_path / "model"
    model.mkdir()
    tok = tmp_path / "tokenizer.json"
    tok.write_text("{}")
    ok = dict(model_dir=str(model), tokenizer_file=str(tok), prompt="Gravity is")
    for change, word in (({"model_dir": str(tmp_path / "none")}, "regular directory"),
                         ({"prompt": ""}, "UTF-8 bytes"), ({"prompt": "a\0b"}, "NUL"),
                         ({"prompt": "x" * (1024 * 1024 + 1)}, "UTF-8 bytes"),
                         ({"tokenizer_file": None}, "needs a tokenizer"),
                         ({"tokenizer_file": str(tmp_path / "gone.json")}, "regular file"),
                         ({"device_ordinal": -1}, "device ordinal"), ({"device_ordinal": True}, "device ordinal"),
                         ({"max_new_tokens": 0}, "max-new-tokens"), ({"max_new_tokens": 65537}, "max-new-tokens"),
                         ({"timeout_seconds": 0}, "timeout"), ({"prompt_ids": [1, 2]}, "not both"),
                         ({"dtype": "float16"}, "dtype")):
        with pytest.raises(ProcessContractError, match=word):
            execute(**{**ok, **change})
    link = tmp_path / "link"
    os.symlink(model, link)
    with pytest.raises(ProcessContractError, match="symlink"):
        execute(**{**ok, "model_dir": str(link)})

    def script(name, body):
        path = tmp_path / name
        path.write_text("#!/usr/bin/env python3\nimport sys, time\n" + body)
        path.chmod(path.stat().st_mode | stat.S_IXUSR)
        return str(path)

    echo = script("echo", "print(' '.join(sys.argv[1:]))\nprint('note', file=sys.stderr)\n")
    target = str(tmp_path / "result.json")
    result = execute(**ok, max_new_tokens=5, result_path=target, nnis_bin=echo)
    said = result["output"]["stdout_utf8"]
    assert said.startswith("generate --model") and "--max-new-tokens 5" in said and "--prompt Gravity is" in said
    assert result["output"]["stderr_utf8"] == "note\n" and result["sampling"] == "greedy"
    assert result["inputs"]["max_new_tokens"] == 5 and result["contract"].startswith("nnis_b200.generation@")
    assert json.load(open(target)) == result
    with pytest.raises(ProcessContractError, match="exists already"):
        execute(**ok, result_path=target, nnis_bin=echo)
    ids = execute(model_dir=str(model), prompt_ids=[3, 1, 4], nnis_bin=echo)
    assert "--prompt-ids 3,1,4" in ids["output"]["stdout_utf8"] and "--tokenizer" not in ids["output"]["stdout_utf8"]
    with pytest.raises(RuntimeError, match="exit code 3"):
        execute(**ok, nnis_bin=script("fail", "print('broken', file=sys.stderr)\nsys.exit(3)\n"))
    t0 = time.monotonic()
    with pytest.raises(TimeoutError):
        execute(**ok, nnis_bin=script("hang", "time.sleep(60)\n"), timeout_seconds=0.5)
    assert time.monotonic() - t0 < 20
    assert not [n for n in os.listdir(tmp_path) if ".tmp-" in n]


def test_replay_drives_the_step_function_and_keeps_slots(tmp_path, monkeypatch):
    """The replay loop on a scripted engine: a slot per request from its first step to its
    `end`, slots used again, logits written in the order of entries and of `want`, a report
    for every step, and an error for a request that ends without having started."""
    import json

    import torch

    from nnis_b200.engine import replay as R

    class Stream:
        def synchronize(self):
            pass
    monkeypatch.setattr(torch.cuda, "current_stream", lambda *a, **k: Stream())

    class ScriptedEngine:
        vocab = 5

        def __init__(self):
            self.free, self.held, self.calls, self.lengths = [1, 0], set(), [], {}

        def acquire_slot(self):
            slot = self.free.pop()
            self.held.add(slot)
            self.lengths[slot] = 0
            return slot

        def release_slot(self, slot):
            self.held.remove(slot)
            self.free.append(slot)

        def step(self, batch):
            rows = []
            for s in batch:
                assert s.slot in self.held
                for w in s.want:  # a row says which slot, position and token it is for
                    rows.append([s.slot, self.lengths[s.slot] + w, s.tokens[w], 0, 0])
                self.lengths[s.slot] += len(s.tokens)
            self.calls.append([(s.slot, list(s.tokens)) for s in batch])
            return torch.tensor(rows, dtype=torch.float32).reshape(len(rows), self.vocab)

        def check_status(self):
            pass

    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]},
                                {"id": "b", "tokens": [9], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": [4], "want": [0]}, {"id": "b", "tokens": [8], "want": [0]}],
         "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": [6], "want": []}], "end": ["a"]},
        {"step": 7, "entries": [{"id": "c", "tokens": [1, 2], "want": [1]}], "end": ["c"]},
    ]
    engine, done = ScriptedEngine(), []
    out = str(tmp_path / "out")
    assert R.replay(engine, [json.dumps(s) for s in steps] + ["", "  "], out, done.append) == 4
    assert done == [0, 1, 2, 7] and not engine.held
    read = lambda n: np.fromfile(f"{out}/{n}.f32", dtype="<f4").reshape(-1, 5)[:, :3].tolist()
    a, b = engine.calls[0][0][0], engine.calls[0][1][0]
    assert a != b
    assert read(0) == [[a, 0, 5], [a, 2, 3]]
    assert read(1) == [[a, 3, 4], [b, 1, 8]]
    assert sorted(os.listdir(out)) == ["0.f32", "1.f32", "7.f32"]  # step 2 wanted nothing
    c = engine.calls[3][0][0]
    assert c in (a, b) and read(7) == [[c, 1, 2]]  # a slot given back is used again, from length 0
    with pytest.raises(R.StepError, match="never started"):
        R.replay(ScriptedEngine(), [json.dumps({"step": 0, "entries": [], "end": ["x"]})], out)


def test_cli_random_model_writes_folders_that_validate(tmp_path):
    import json

    from helpers import TINY_A, TINY_B
    from nnis_b200.cli.main import main
    cfg = tmp_path / "a.json"
    cfg.write_text(json.dumps(TINY_A))
    for fmt in ("hf", "nnis"):
        out = str(tmp_path / fmt)
        assert main(["random-model", "--config", str(cfg), "--seed", "7", "--out", out, "--format", fmt]) == 0
        assert main(["validate", "--model", out]) == 0
        assert main(["random-model", "--config", str(cfg), "--seed", "7", "--out", out]) == 1  # not empty
    assert sorted(os.listdir(tmp_path / "hf")) == ["config.json", "model.safetensors"]
    assert "model.json" in os.listdir(tmp_path / "nnis")
    # the same seed gives the same tensors in both forms
    from nnis_b200.config import read_config
    from nnis_b200.engine.model import DecoderModel
    from nnis_b200.weights import load_weights
    import torch
    both = []
    for fmt in ("hf", "nnis"):
        d = str(tmp_path / fmt)
        wanted = DecoderModel.weight_specs_of(read_config(d).to_spec())
        both.append(load_weights(d, wanted, torch.float32, torch.device("cpu")))
    for name, t in both[0].items():
        assert torch.equal(t, both[1][name]), name
    b = tmp_path / "b.json"
    b.write_text(json.dumps(TINY_B))  # biases: no place in NNIS's own folder
    assert main(["random-model", "--config", str(b), "--seed", "1", "--out", str(tmp_path / "b"), "--format", "nnis"]) == 1
    for bad in (["random-model", "--seed", "1", "--out", "x"], ["random-model", "--config", "c", "--out", "x"],
                ["random-model", "--config", "c", "--seed", "1", "--out", "x", "--format", "gguf"]):
        with pytest.raises(UsageError):
            parse_args(bad)


def test_the_graph_decoders_copy_of_a_page_table_follows_a_truncation(monkeypatch):
    """GraphDecoder.upload keeps a pinned copy of every row's page table and rewrites
    only what changed; a table that was truncated and grew back to the same length with
    other pages must be rewritten (the slot's version says so)."""
    import types

    import torch

    from nnis_b200.cache import CacheManager, KVRequest
    from nnis_b200.engine import decode as D
    cache = CacheManager([KVRequest(1, 16)], torch.float32, torch.device("cpu"), 64 * 6, 2, 1000)
    dec = D.GraphDecoder.__new__(D.GraphDecoder)
    dec.engine = types.SimpleNamespace(cache=cache)
    dec.rows, dec.cols = 2, 4
    dec.tables = [None]
    dec.state_ints = 2 * (3 + 4)
    dec.state = torch.zeros(dec.state_ints, dtype=torch.int32)
    dec.host_state = torch.zeros(dec.state_ints, dtype=torch.int32)
    dec._host_np = dec.host_state.numpy()
    dec._host_state_free = types.SimpleNamespace(synchronize=lambda: None, record=lambda: None)
    dec._mirror = None
    dec.host_tables = [[[-1] * 4 for _ in range(2)]]
    dec._host_tables_unknown = False
    monkeypatch.setattr(D.ops, "copy_async", lambda dst, src: dst.copy_(src))
    a, b = cache.acquire(), cache.acquire()
    cache.reserve([a], [130])
    cache.commit([a], [130])
    line = lambda row: dec.state[6 + 4 * row:10 + 4 * row].tolist()
    dec.upload([5], [129], [a])
    assert line(0)[:3] == cache.page_table(0, a) and line(0)[3] == -1
    cache.truncate(a, 64)
    cache.reserve([b], [64])
    cache.commit([b], [64])
    cache.reserve([a], [130])
    cache.commit([a], [130])
    dec.upload([5], [129], [a])
    assert line(0)[:3] == cache.page_table(0, a)


def test_prompt_steps_are_cut_into_portions_in_order():
    """Engine.step_in_portions on a scripted step: sequences in order, one that does not
    fit is cut, wanted places follow their tokens, rows come back in the order asked for."""
    import torch

    from nnis_b200.engine.engine import Engine, SequenceStep
    calls = []

    class Scripted:
        step_in_portions = Engine.step_in_portions

        def step(self, batch):
            calls.append([(s.slot, list(s.tokens), list(s.want)) for s in batch])
            rows = [[s.slot, s.tokens[w]] for s in batch for w in s.want]
            return torch.tensor(rows, dtype=torch.float32).reshape(len(rows), 2)
    e = Scripted()
    batch = [SequenceStep(0, list(range(100, 107)), [6, 0]), SequenceStep(1, list(range(200, 203)), [2]),
             SequenceStep(2, list(range(300, 312)), [11, 3, 4])]
    got = e.step_in_portions(batch, 5)
    assert [sum(len(t) for _, t, _ in c) for c in calls] == [5, 5, 5, 5, 2]
    assert calls[0] == [(0, [100, 101, 102, 103, 104], [0])]
    assert calls[1] == [(0, [105, 106], [1]), (1, [200, 201, 202], [2])]
    assert got.tolist() == [[0, 106], [0, 100], [1, 202], [2, 311], [2, 303], [2, 304]]
    calls.clear()
    assert e.step_in_portions(batch, 100).shape[0] == 6 and len(calls) == 1
