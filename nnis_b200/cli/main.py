"""``nnis generate`` and ``nnis generate-batch`` with NNIS's options and rules
(crates/nnis-cli/src/main.rs:21-23 usage and defaults, :179-365 and :367-498
flag rules, :117-132 the JSON of generate-batch, :1348-1390 exit codes), and
``nnis validate``, the check of a model folder on the CPU that NNIS has as
``nnis-hf validate`` (crates/nnis-cli/src/bin/nnis-hf.rs:17 usage, :86-130 flag
rules, :279-299 tokenizer ids against the vocabulary, :345-478 the report).

Additions: ``--model`` is a Hugging Face folder; ``--prompt-ids 1,2,3`` gives a
prompt as token ids, and then ``--tokenizer`` may be left out (ids are printed);
``--dtype bfloat16|float32``.
"""
from __future__ import annotations

import json
import math
import sys
from dataclasses import dataclass, field
from typing import List, Optional

DEFAULT_DEVICE_ORDINAL = 0
DEFAULT_MAX_NEW_TOKENS = 16
GENERATE_BATCH_JSON_SCHEMA_VERSION = 1
USAGE = """Usage:
  nnis generate --model DIR [--tokenizer FILE] --prompt TEXT | --prompt-ids IDS [--device N] [--max-new-tokens N] [--dtype bfloat16|float32] [--sample --seed U64] [--temperature F] [--top-k N] [--top-p F] [--stream]
  nnis generate-batch --model DIR [--tokenizer FILE] --prompt TEXT [--prompt TEXT ...] | --prompt-ids IDS [--prompt-ids IDS ...] --seed U64 [--seed U64 ...] [--device N] [--max-new-tokens N] [--dtype bfloat16|float32] [--temperature F] [--top-k N] [--top-p F] [--json]
  nnis validate --model DIR [--tokenizer FILE] [--json] [--output FILE]
  nnis random-model --config FILE --seed U64 --out DIR [--format hf|nnis]

`validate` checks config.json, the safetensors files (tensor names, shapes and dtypes against the model that config.json names) and, when a tokenizer is given or DIR/tokenizer.json exists, that its ids fit the vocabulary; it needs no GPU and reads no tensor. `--output FILE` requires `--json` and writes the report there, never over an existing file.
`random-model` writes a model folder with seeded random weights from a config.json (`hf`: config.json + model.safetensors; `nnis`: model.json + raw tensor files); it needs no GPU.

Default decoding on `generate` is greedy. Opt-in `--sample` requires `--seed`. Optional `--temperature`, `--top-k`, and `--top-p` apply only with `--sample`. `--stream` is valid only with `--sample` and prints each token as it is emitted. `generate-batch` requires one `--seed` per prompt and always samples; `--json` emits versioned JSON. CUDA device ordinal defaults to 0."""


class UsageError(Exception):
    pass


@dataclass
class GenerateArgs:
    model_dir: str = ""
    tokenizer_file: Optional[str] = None
    prompts: List[str] = field(default_factory=list)
    prompt_ids: List[List[int]] = field(default_factory=list)
    device_ordinal: int = DEFAULT_DEVICE_ORDINAL
    max_new_tokens: int = DEFAULT_MAX_NEW_TOKENS
    dtype: str = "bfloat16"
    sample: bool = False
    stream: bool = False
    json: bool = False
    seeds: List[int] = field(default_factory=list)
    temperature: Optional[float] = None
    top_k: Optional[int] = None
    top_p: Optional[float] = None
    command: str = "generate"
    output: Optional[str] = None
    config_file: Optional[str] = None
    folder_format: str = "hf"


def _positive_float(flag: str, raw: str) -> float:
    try:
        value = float(raw)
    except ValueError:
        raise UsageError(f"invalid {flag} {raw!r}") from None
    if not math.isfinite(value) or value <= 0:
        raise UsageError(f"{flag} must be finite and positive; got {raw}")
    return value


def _unsigned(flag: str, raw: str, positive: bool = False, limit: int = (1 << 64) - 1) -> int:
    try:
        value = int(raw)
    except ValueError:
        raise UsageError(f"invalid {flag} {raw!r}") from None
    if value < 0 or value > limit or (positive and value == 0):
        raise UsageError(f"{flag} must be {'positive' if positive else 'non-negative'}; got {raw}")
    return value


def _ids(raw: str) -> List[int]:
    try:
        ids = [int(x) for x in raw.replace(" ", "").split(",") if x != ""]
    except ValueError:
        raise UsageError(f"invalid --prompt-ids {raw!r}") from None
    if not ids or any(i < 0 for i in ids):
        raise UsageError(f"--prompt-ids needs non-negative integers; got {raw!r}")
    return ids


def parse_args(argv: List[str]) -> Optional[GenerateArgs]:
    """None for help.  Raises UsageError with NNIS's rules."""
    if not argv or argv[0] in ("-h", "--help", "help"):
        return None
    command = argv[0]
    if command == "validate":
        return _parse_validate(argv[1:])
    if command == "random-model":
        return _parse_random_model(argv[1:])
    if command not in ("generate", "generate-batch"):
        raise UsageError(f"unknown command {command!r}")
    a = GenerateArgs(command=command)
    batch = command == "generate-batch"
    seen = set()
    it = iter(argv[1:])
    for flag in it:
        if flag in ("-h", "--help"):
            return None
        if flag in ("--sample", "--stream", "--json"):
            if (flag == "--json") != batch and flag == "--json":
                raise UsageError("--json belongs to generate-batch")
            if batch and flag != "--json":
                raise UsageError(f"{flag} does not apply to generate-batch (it always samples)")
            setattr(a, flag[2:], True)
            continue
        try:
            value = next(it)
        except StopIteration:
            raise UsageError(f"{flag} needs a value") from None
        repeatable = batch and flag in ("--prompt", "--prompt-ids", "--seed")
        if flag in seen and not repeatable:
            raise UsageError(f"{flag} given twice")
        seen.add(flag)
        if flag == "--model":
            a.model_dir = value
        elif flag == "--tokenizer":
            a.tokenizer_file = value
        elif flag == "--prompt":
            a.prompts.append(value)
        elif flag == "--prompt-ids":
            a.prompt_ids.append(_ids(value))
        elif flag == "--device":
            a.device_ordinal = _unsigned(flag, value, limit=(1 << 31) - 1)
        elif flag == "--max-new-tokens":
            a.max_new_tokens = _unsigned(flag, value, positive=True, limit=65536)
        elif flag == "--dtype":
            if value not in ("bfloat16", "float32"):
                raise UsageError(f"--dtype must be bfloat16 or float32; got {value!r}")
            a.dtype = value
        elif flag == "--seed":
            a.seeds.append(_unsigned(flag, value))
        elif flag == "--temperature":
            a.temperature = _positive_float(flag, value)
        elif flag == "--top-k":
            a.top_k = _unsigned(flag, value, positive=True)
        elif flag == "--top-p":
            a.top_p = _positive_float(flag, value)
            if a.top_p > 1:
                raise UsageError(f"--top-p must be in (0, 1]; got {value}")
        else:
            raise UsageError(f"unknown flag {flag!r}")
    if not a.model_dir:
        raise UsageError("--model is required")
    if a.prompts and a.prompt_ids:
        raise UsageError("give --prompt or --prompt-ids, not both")
    n_prompts = len(a.prompts) + len(a.prompt_ids)
    if n_prompts == 0:
        raise UsageError("--prompt is required")
    if a.prompts and not a.tokenizer_file:
        raise UsageError("--tokenizer is required with --prompt")
    if batch:
        if len(a.seeds) != n_prompts:
            raise UsageError(f"generate-batch needs one --seed per prompt: {n_prompts} prompts, "
                             f"{len(a.seeds)} seeds")
        a.sample = True
    else:
        if n_prompts != 1:
            raise UsageError("generate takes one prompt")
        if not a.sample:
            for name, given in (("--seed", a.seeds), ("--temperature", a.temperature),
                                ("--top-k", a.top_k), ("--top-p", a.top_p), ("--stream", a.stream)):
                if given:
                    raise UsageError(f"{name} requires --sample")
        elif len(a.seeds) != 1:
            raise UsageError("--sample requires --seed")
    return a


def _parse_validate(rest: List[str]) -> Optional[GenerateArgs]:
    a = GenerateArgs(command="validate")
    seen = set()
    it = iter(rest)
    for flag in it:
        if flag in ("-h", "--help"):
            return None
        if flag == "--json":
            a.json = True
            continue
        if flag not in ("--model", "--tokenizer", "--output"):
            raise UsageError(f"unknown validate argument {flag!r}")
        try:
            value = next(it)
        except StopIteration:
            raise UsageError(f"{flag} needs a value") from None
        if flag in seen:
            raise UsageError(f"{flag} given twice")
        seen.add(flag)
        if flag == "--model":
            a.model_dir = value
        elif flag == "--tokenizer":
            a.tokenizer_file = value
        else:
            a.output = value
    if not a.model_dir:
        raise UsageError("--model is required")
    if a.output is not None and not a.json:
        raise UsageError("--output requires --json")
    return a


def _parse_random_model(rest: List[str]) -> Optional[GenerateArgs]:
    a = GenerateArgs(command="random-model")
    seen = set()
    it = iter(rest)
    for flag in it:
        if flag in ("-h", "--help"):
            return None
        if flag not in ("--config", "--seed", "--out", "--format"):
            raise UsageError(f"unknown random-model argument {flag!r}")
        try:
            value = next(it)
        except StopIteration:
            raise UsageError(f"{flag} needs a value") from None
        if flag in seen:
            raise UsageError(f"{flag} given twice")
        seen.add(flag)
        if flag == "--config":
            a.config_file = value
        elif flag == "--seed":
            a.seeds = [_unsigned("--seed", value)]
        elif flag == "--out":
            a.output = value
        elif value in ("hf", "nnis"):
            a.folder_format = value
        else:
            raise UsageError(f"--format must be hf or nnis; got {value!r}")
    for flag, given in (("--config", a.config_file), ("--seed", a.seeds), ("--out", a.output)):
        if not given:
            raise UsageError(f"{flag} is required")
    return a


def random_model(a: GenerateArgs, out=sys.stdout) -> int:
    """A model folder with seeded random weights from the configuration in ``--config``."""
    import os

    from ..weights import SafetensorsFile, write_nnis_directory, write_random_model
    with open(a.config_file, "r", encoding="utf-8") as f:
        config = json.load(f)
    if os.path.lexists(a.output) and (not os.path.isdir(a.output) or os.listdir(a.output)):
        raise ValueError(f"{a.output} exists and is not an empty folder")
    if a.folder_format == "hf":
        write_random_model(config, a.seeds[0], a.output)
    else:
        import tempfile
        with tempfile.TemporaryDirectory() as tmp:
            write_random_model(config, a.seeds[0], tmp)
            with SafetensorsFile(os.path.join(tmp, "model.safetensors")) as f:
                tensors = {n: f.tensor(n) for n in f.names()}
            with open(os.path.join(tmp, "config.json"), "r", encoding="utf-8") as f:
                written = json.load(f)
        write_nnis_directory(written, tensors, a.output)
    out.write(f"{a.output}\n")
    return 0


VALIDATE_SCHEMA = "nnis_b200.model-preflight@1"


def validate(a: GenerateArgs, out=sys.stdout) -> int:
    """0 when the folder can be loaded and run; 1 with the reason otherwise."""
    import os

    from ..config import read_config
    from ..engine.model import DecoderModel
    from ..weights import check_weights
    report = {"schema": VALIDATE_SCHEMA, "model_directory": a.model_dir, "ready": False, "blocker": None}
    try:
        config = read_config(a.model_dir)
        spec = config.to_spec()
        raw = config.to_dict()
        report["architecture"] = (raw.get("architectures") or [None])[0]
        report["model_type"] = raw.get("model_type")
        report["vocab_size"] = spec.vocab_size
        report["layers"] = len(spec.schedule)
        report["weights"] = check_weights(a.model_dir, DecoderModel.weight_specs_of(spec))
        tokenizer_file = a.tokenizer_file
        if tokenizer_file is None and os.path.isfile(os.path.join(a.model_dir, "tokenizer.json")):
            tokenizer_file = os.path.join(a.model_dir, "tokenizer.json")
        report["tokenizer_file"] = tokenizer_file
        if tokenizer_file is not None:
            from ..engine.api import load_tokenizer
            vocab = load_tokenizer(tokenizer_file).get_vocab(True)
            if not vocab:
                raise ValueError("tokenizer vocabulary is empty")
            top = max(vocab.values())
            report["tokenizer"] = {"vocabulary_size": len(vocab), "maximum_token_id": top}
            if top >= spec.vocab_size:
                raise ValueError(f"tokenizer maximum token id {top} is out of range for model "
                                 f"vocabulary {spec.vocab_size}")
        report["ready"] = True
    except Exception as e:  # every fault of the folder is the report's blocker
        report["blocker"] = f"{type(e).__name__}: {e}"
    if a.json:
        text = json.dumps(report, indent=1) + "\n"
        if a.output is not None:
            # never over an existing file, and whole or not at all
            tmp = f"{a.output}.tmp-{os.getpid()}"
            with open(tmp, "x", encoding="utf-8") as f:
                f.write(text)
            try:
                os.link(tmp, a.output)
            finally:
                os.unlink(tmp)
        else:
            out.write(text)
    else:
        out.write("NNIS_PREFLIGHT_" + ("READY" if report["ready"] else "BLOCKED") + "\n")
        for key, value in report.items():
            if key not in ("ready",):
                out.write(f"{key}={json.dumps(value) if isinstance(value, (dict, list)) else value}\n")
    return 0 if report["ready"] else 1


def _policy(a: GenerateArgs, seed: int):
    from ..sampling import SamplingConfig
    return SamplingConfig(seed=seed, temperature=a.temperature if a.temperature is not None else 1.0,
                          top_k=a.top_k, top_p=a.top_p)


def run(a: GenerateArgs, out=sys.stdout) -> int:
    if a.command == "validate":
        return validate(a, out)
    if a.command == "random-model":
        return random_model(a, out)
    from ..engine.api import LLM
    from ..sampling import SAMPLING_POLICY_VERSION
    prompts = a.prompts if a.prompts else a.prompt_ids
    llm = LLM(a.model_dir, dtype=a.dtype, device_ordinal=a.device_ordinal,
              tokenizer_file=a.tokenizer_file, max_batch=max(1, len(prompts)),
              max_tokens=max(4096, sum(len(p) for p in prompts) + len(prompts) * (a.max_new_tokens + 64)))

    def text_of(ids):
        return llm.decode(ids) if llm.tokenizer is not None else " ".join(str(i) for i in ids)

    sampling = [_policy(a, s) for s in a.seeds] if a.sample else None
    emitted = {}

    def on_token(index, token):
        # print only what the new token adds to the decoded text
        ids = emitted.setdefault(index, [])
        before = text_of(ids)
        ids.append(token)
        after = text_of(ids)
        out.write(after[len(before):] if after.startswith(before) else after)
        out.flush()

    results = llm.generate(prompts, max_new_tokens=a.max_new_tokens, sampling=sampling,
                           on_token=on_token if a.stream else None)
    failed = any(not r.ok for r in results)
    if a.command == "generate":
        r = results[0]
        if not r.ok:
            print(f"error: {r.error}", file=sys.stderr)
            return 1
        out.write("\n" if a.stream else text_of(r.token_ids) + "\n")
        return 0
    if a.json:
        json.dump({"schema_version": GENERATE_BATCH_JSON_SCHEMA_VERSION,
                   "sampling_policy_version": SAMPLING_POLICY_VERSION,
                   "session_count": len(results),
                   "results": [{"batch_index": r.index, "seed": a.seeds[r.index], "ok": r.ok,
                                "text": text_of(r.token_ids) if r.ok else None,
                                "error": r.error} for r in results]}, out)
        out.write("\n")
    else:
        for r in results:
            if r.ok:
                out.write(f"[{r.index}] seed={a.seeds[r.index]}: {text_of(r.token_ids)}\n")
            else:
                out.write(f"[{r.index}] seed={a.seeds[r.index]}: error: {r.error}\n")
    return 1 if failed else 0


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    try:
        args = parse_args(argv)
    except UsageError as e:
        print(f"error: {e}\n\n{USAGE}", file=sys.stderr)
        return 2
    if args is None:
        print(USAGE)
        return 0
    try:
        return run(args)
    except Exception as e:  # a run failure, not a usage error
        print(f"error: {type(e).__name__}: {e}", file=sys.stderr)
        return 1
