"""Generation through the Python entry point and the command line on the GPU."""
import json
import os
import subprocess
import sys

import pytest

import plain_llama as P
from helpers import CONFIGS, load_plain_weights, make_model, read_config_json

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    return {n: make_model(str(tmp_path_factory.mktemp(f"gen{n}")), c, seed=40 + i)
            for i, (n, c) in enumerate(CONFIGS.items())}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_matches_the_plain_loop(model_dirs, name, dtype):
    from nnis_b200 import LLM
    d = model_dirs[name]
    cfg = read_config_json(d)
    bf = dtype == "bfloat16"
    w = load_plain_weights(d, as_bf16=bf)
    llm = LLM(d, dtype=dtype, max_tokens=64 * 32, max_batch=3)
    prompts = [[5, 9, 1, 200, 33], [7], [100, 101, 102, 103, 104, 105, 106, 107, 108], [250, 3],
               [9] * 70]
    results = llm.generate(prompts, max_new_tokens=12, stop_token_ids=())
    for p, r in zip(prompts, results):
        assert r.ok and r.finish_reason == "length"
        assert r.token_ids == P.greedy_generate(cfg, w, p, 12, None, bf), (name, dtype, p)
    # a stop token ends its sequence early; the others go on
    stop = results[0].token_ids[3]
    again = llm.generate(prompts[:2], max_new_tokens=12, stop_token_ids=[stop])
    cut = results[0].token_ids[:results[0].token_ids.index(stop) + 1]
    assert again[0].token_ids == cut and again[0].finish_reason == "stop"
    want1 = results[1].token_ids
    if stop in want1:
        want1 = want1[:want1.index(stop) + 1]
    assert again[1].token_ids == want1
    assert llm.engine.cache.usage()["slots_held"] == 0


def test_sampled_generation_is_seeded_and_sessions_work(model_dirs):
    from nnis_b200 import LLM, GenerationConfig, SamplingConfig
    from nnis_b200.sampling import HostLogitSampler
    d = model_dirs["B"]  # its head is not tied, so its logits are of order one
    llm = LLM(d, dtype="float32", max_tokens=64 * 16, max_batch=4)
    policy = SamplingConfig(seed=11, temperature=0.8, top_k=20, top_p=0.9)
    a = llm.generate([[1, 2, 3], [4, 5]], max_new_tokens=8, sampling=policy, stop_token_ids=())
    b = llm.generate([[1, 2, 3], [4, 5]], max_new_tokens=8, sampling=policy, stop_token_ids=())
    c = llm.generate([[1, 2, 3]], max_new_tokens=8, sampling=SamplingConfig(seed=12), stop_token_ids=())
    assert [r.token_ids for r in a] == [r.token_ids for r in b]
    assert a[0].token_ids != c[0].token_ids
    # the session surface: prefill + decode_one with the host sampler gives the same tokens
    session = llm.new_session()
    sampler = HostLogitSampler(policy, 515)
    logits = session.prefill([1, 2, 3])
    tokens = []
    for _ in range(8):
        tokens.append(sampler.sample(logits))
        logits = session.decode_one(tokens[-1])
    assert tokens == a[0].token_ids and session.position() == 3 + 8
    assert session.generate_sampled([1, 2, 3], GenerationConfig(8), policy) == a[0].token_ids
    session.close()
    assert llm.engine.cache.usage()["slots_held"] == 0


def test_command_line_generates(model_dirs):
    d = model_dirs["A"]
    cfg = read_config_json(d)
    w = load_plain_weights(d, as_bf16=False)
    run = lambda *args: subprocess.run([sys.executable, os.path.join(ROOT, "bin", "nnis"), *args],
                                       capture_output=True, text=True, timeout=600)
    r = run("generate", "--model", d, "--prompt-ids", "5,9,1", "--max-new-tokens", "6", "--dtype",
            "float32")
    assert r.returncode == 0, r.stderr[-2000:]
    want = P.greedy_generate(cfg, w, [5, 9, 1], 6, 7)
    assert r.stdout.split() == [str(t) for t in want]
    r = run("generate-batch", "--model", d, "--prompt-ids", "5,9,1", "--prompt-ids", "3,999",
            "--seed", "1", "--seed", "2", "--json", "--dtype", "float32", "--max-new-tokens", "4")
    assert r.returncode == 1
    out = json.loads(r.stdout)
    assert out["schema_version"] == 1 and out["session_count"] == 2
    assert out["results"][0]["ok"] and not out["results"][1]["ok"]
    assert "vocabulary" in out["results"][1]["error"]
    assert run("generate", "--model", d, "--prompt-ids", "1", "--seed", "3").returncode == 2
    assert run("validate", "--model", d).returncode == 0


def test_process_entry_point_generates(model_dirs, tmp_path):
    """`nnis_b200.execute` runs the command line as a bounded child and records its output."""
    from nnis_b200 import execute
    d = model_dirs["B"]
    cfg = read_config_json(d)
    w = load_plain_weights(d, as_bf16=False)
    target = str(tmp_path / "result.json")
    result = execute(d, prompt_ids=[5, 9, 1, 77], max_new_tokens=5, dtype="float32", result_path=target,
                     timeout_seconds=600.0)
    want = P.greedy_generate(cfg, w, [5, 9, 1, 77], 5, cfg.get("eos_token_id"))
    assert result["output"]["stdout_utf8"].split() == [str(t) for t in want]
    assert json.load(open(target)) == result


@pytest.mark.parametrize("pipeline", [True, False])
def test_both_decode_paths_agree_with_the_plain_loop(model_dirs, pipeline):
    """Tokens kept on the device with picks read one step late, and tokens sent
    from the host every step: same results, stops included, slots all free."""
    from nnis_b200 import LLM
    d = model_dirs["C"]
    cfg = read_config_json(d)
    w = load_plain_weights(d, as_bf16=False)
    llm = LLM(d, dtype="float32", max_tokens=64 * 40, max_batch=8, pipeline_decode=pipeline)
    prompts = [[i + 1, 2 * i + 3, 900 - i] * (1 + i % 3) for i in range(11)] + [[4] * 63, [5] * 64]
    plain = [P.greedy_generate(cfg, w, p, 20, None) for p in prompts]
    stop = plain[2][6]
    want = [t[:t.index(stop) + 1] if stop in t else t for t in plain]
    got = llm.generate(prompts, max_new_tokens=20, stop_token_ids=[stop])
    assert [r.token_ids for r in got] == want
    assert got[2].finish_reason == "stop"
    assert llm.engine.cache.usage()["slots_held"] == 0 and llm.engine.cache.usage()["pages_held"] == [0]
    llm.engine.cache.check()
    # a second call reuses decoders, graphs and slots
    again = llm.generate(prompts[:3], max_new_tokens=5, stop_token_ids=())
    assert [r.token_ids for r in again] == [t[:5] for t in plain[:3]]


def test_temperature_sampling_on_the_device_follows_the_seeded_draws(model_dirs):
    """With device_sampling the draws come from the sampling kernel: same seeds,
    same tokens on every run, and the tokens the plain inverse CDF (token-id order,
    float64) picks from the engine's own logits."""
    import numpy as np
    from nnis_b200 import LLM, SamplingConfig
    d = model_dirs["B"]
    llm = LLM(d, dtype="float32", max_tokens=64 * 16, max_batch=4, device_sampling=True)
    policies = [SamplingConfig(seed=5, temperature=0.9), SamplingConfig(seed=6, temperature=1.4)]
    prompts = [[1, 2, 3], [9, 8]]
    a = llm.generate(prompts, max_new_tokens=10, sampling=policies, stop_token_ids=())
    b = llm.generate(prompts, max_new_tokens=10, sampling=policies, stop_token_ids=())
    assert [r.token_ids for r in a] == [r.token_ids for r in b] and all(r.ok for r in a)
    # replay request 0 by hand: its logits through a session, its draws through the plain generator
    session = llm.new_session()
    rng = P.PlainSplitMix64(5)
    logits = session.prefill(prompts[0])
    for t in a[0].token_ids:
        w = np.exp((logits.astype(np.float64) - logits.max()) / float(np.float32(0.9)))
        cdf = np.cumsum(w)
        u = rng.next_unit() * cdf[-1]
        want = int(np.searchsorted(cdf, u, side="right"))
        assert t == want or abs(cdf[t] - u) < 1e-9 * cdf[-1]
        logits = session.decode_one(t)
    session.close()


def test_nnis_model_folder_generates_like_its_hugging_face_twin(model_dirs, tmp_path):
    """A model.json + raw-files folder (NNIS's own format) loads and generates the same tokens."""
    from nnis_b200 import LLM
    from nnis_b200.weights import SafetensorsFile, write_nnis_directory
    d = model_dirs["A"]  # no biases: the format has no place for them
    with SafetensorsFile(os.path.join(d, "model.safetensors")) as f:
        tensors = {n: f.tensor(n) for n in f.names()}
    twin = write_nnis_directory(read_config_json(d), tensors, str(tmp_path / "nnis"))
    prompts = [[5, 9, 1, 200, 33], [7]]
    for dtype in ("float32", "bfloat16"):
        want = LLM(d, dtype=dtype, max_tokens=64 * 8, max_batch=2).generate(prompts, max_new_tokens=8,
                                                                          stop_token_ids=())
        got = LLM(twin, dtype=dtype, max_tokens=64 * 8, max_batch=2).generate(prompts, max_new_tokens=8,
                                                                            stop_token_ids=())
        assert [r.token_ids for r in got] == [r.token_ids for r in want]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_session_truncates_and_goes_on(model_dirs, dtype):
    """Back to an earlier length, then other tokens: the logits are those of the new
    sequence as a whole, across a page boundary of the cache and within a page."""
    import numpy as np
    import torch

    from helpers import check_logits
    from nnis_b200 import LLM
    d = model_dirs["B"]
    cfg = read_config_json(d)
    bf = dtype == "bfloat16"
    w = load_plain_weights(d, as_bf16=bf)
    llm = LLM(d, dtype=dtype, max_tokens=64 * 8, max_batch=2)
    session = llm.new_session()
    first = [(7 * i + 3) % cfg["vocab_size"] for i in range(70)]
    session.prefill(first)
    for t in (11, 12, 13):
        session.decode_one(t)
    for back_to, tail in ((60, [21, 22, 23, 24, 25, 26]), (65, [31]), (3, [41, 42])):
        session.truncate(back_to)
        assert session.position() == back_to
        got = [session.decode_one(t) for t in tail]
        want = P.forward(cfg, w, first[:back_to] + tail, bf)[back_to:]
        check_logits(np.stack(got), want, dtype, f"after truncating to {back_to}")
        first = first[:back_to] + tail
    session.close()
    llm.engine.cache.check()
    assert llm.engine.cache.usage()["pages_held"] == [0]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("pipeline", [True, False])
def test_a_session_goes_on_after_generate(model_dirs, dtype, pipeline):
    """crates/nnis-model/src/runtime.rs:814-846,1264-1274: after ``generate`` the session
    holds prompt + emitted tokens, every one of them executed, and a further
    ``decode_one`` gives the logits of the whole sequence; with a stop token, with a
    callback that stops, with sampling, and after what the session held before."""
    import numpy as np

    from helpers import check_logits
    from nnis_b200 import LLM, GenerationConfig, SamplingConfig, StreamControl
    d = model_dirs["A"]
    cfg = read_config_json(d)
    bf = dtype == "bfloat16"
    w = load_plain_weights(d, as_bf16=bf)
    llm = LLM(d, dtype=dtype, max_tokens=64 * 16, max_batch=2, pipeline_decode=pipeline)
    session = llm.new_session()
    prompt = [5, 9, 1, 200, 33]

    def goes_on(tokens, what):
        """The session holds ``tokens``; one more token's logits are the whole sequence's."""
        assert session.position() == len(tokens), what
        got = session.decode_one(17)
        want = P.forward(cfg, w, list(tokens) + [17], bf)[-1:]
        check_logits(got[None, :], want, dtype, what)

    plain = P.greedy_generate(cfg, w, prompt, 9, None, bf)
    out = session.generate(prompt, GenerationConfig(9))
    assert out == plain
    goes_on(prompt + out, "after a fixed length")
    # a stop token is emitted, executed, and ends the generation
    stop = plain[4]
    out = session.generate(prompt, GenerationConfig(9, stop_token_ids=(stop,)))
    assert out == plain[:plain.index(stop) + 1]
    goes_on(prompt + out, "after a stop token")
    # one token only
    out = session.generate(prompt, GenerationConfig(1))
    assert out == plain[:1]
    goes_on(prompt + out, "after one token")
    # the callback stops after the third token
    seen = []
    out = session.generate(prompt, GenerationConfig(9),
                           on_token=lambda t: (seen.append(t), StreamControl.STOP if len(seen) == 3 else None)[1])
    assert out == plain[:3] == seen
    goes_on(prompt + out, "after the callback's stop")
    # the next generation follows what the session holds
    held = prompt + out + [17]
    more = session.generate([40, 41], GenerationConfig(4), keep_context=True)
    assert more == P.greedy_generate(cfg, w, held + [40, 41], 4, None, bf)
    goes_on(held + [40, 41] + more, "after a generation that kept its context")
    # sampled, streamed, stopped by the caller
    policy = SamplingConfig(seed=3, temperature=0.9, top_k=30)
    full = session.generate_sampled(prompt, GenerationConfig(6), policy)
    assert session.position() == len(prompt) + 6
    seen = []
    out = session.generate_sampled_streaming(
        prompt, GenerationConfig(6), policy,
        lambda t: (seen.append(t), StreamControl.STOP if len(seen) == 2 else StreamControl.CONTINUE)[1])
    assert out == full[:2] == seen
    goes_on(prompt + out, "after a sampled stream that its caller stopped")
    session.close()
    assert llm.engine.cache.usage()["slots_held"] == 0


def test_the_callback_stops_one_prompt_of_a_batch(model_dirs):
    from nnis_b200 import LLM, StreamControl
    d = model_dirs["C"]
    cfg = read_config_json(d)
    w = load_plain_weights(d, as_bf16=False)
    prompts = [[3, 4, 5], [100, 200], [7]]
    plain = [P.greedy_generate(cfg, w, p, 10, None) for p in prompts]
    for pipeline in (True, False):
        llm = LLM(d, dtype="float32", max_tokens=64 * 8, max_batch=4, pipeline_decode=pipeline)
        count = {}

        def on_token(i, t):
            count[i] = count.get(i, 0) + 1
            return StreamControl.STOP if (i == 1 and count[i] == 4) else None
        got = llm.generate(prompts, max_new_tokens=10, stop_token_ids=(), on_token=on_token)
        assert got[0].token_ids == plain[0] and got[2].token_ids == plain[2]
        assert got[1].token_ids == plain[1][:4] and got[1].finish_reason == "stop"
        assert llm.engine.cache.usage()["slots_held"] == 0
