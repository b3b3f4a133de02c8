"""Generation as a bounded child process with a JSON record of what ran.

NNIS's Python entry point is of this kind: ``execute(nnis_hf_bin, model_dir,
tokenizer_file, prompt, device_ordinal, max_new_tokens, result_path,
timeout_seconds)`` checks the request, runs ``nnis-hf generate`` without a
shell, caps what it keeps of stdout and stderr, ends the child at a deadline
and writes one JSON result that never replaces a file
(tools/nnis_hub_hf_generate.py:25-34 limits, :51-76 request rules, :189-231
the record, :266-306 the call).  This is the same for ``bin/nnis generate``;
``nnis_b200.LLM`` is the in-process entry point.

Additions: ``prompt_ids`` instead of ``prompt`` (then no tokenizer is needed and
ids are printed), and ``dtype``.
"""
from __future__ import annotations

import hashlib
import json
import os
import signal
import subprocess
import sys
import threading
import time
from typing import Any, Dict, List, Optional, Sequence

SCHEMA_VERSION = 1
CONTRACT = "nnis_b200.generation@1"
MAX_PROMPT_BYTES = 1024 * 1024
MAX_NEW_TOKENS = 65_536
MAX_CAPTURE_BYTES = 16 * 1024 * 1024
MAX_DEVICE_ORDINAL = 2_147_483_647
DEFAULT_TIMEOUT_SECONDS = 3600.0


class ProcessContractError(ValueError):
    """The request breaks a rule; nothing was run."""


def default_binary() -> str:
    here = os.path.dirname(os.path.abspath(__file__))
    return os.path.join(os.path.dirname(os.path.dirname(here)), "bin", "nnis")


def check_request(model_dir: str, tokenizer_file: Optional[str], prompt: Optional[str],
                  prompt_ids: Optional[Sequence[int]], device_ordinal: int, max_new_tokens: int,
                  timeout_seconds: float) -> None:
    if os.path.islink(model_dir) or not os.path.isdir(model_dir):
        raise ProcessContractError(f"model path must be a regular directory, not a symlink: {model_dir}")
    if (prompt is None) == (prompt_ids is None):
        raise ProcessContractError("give a prompt or prompt_ids, not both")
    if prompt is not None:
        if tokenizer_file is None:
            raise ProcessContractError("a text prompt needs a tokenizer file")
        if not isinstance(prompt, str) or "\0" in prompt:
            raise ProcessContractError("prompt must be a string without NUL bytes")
        try:
            size = len(prompt.encode("utf-8"))
        except UnicodeEncodeError:
            raise ProcessContractError("prompt must be valid UTF-8") from None
        if not 1 <= size <= MAX_PROMPT_BYTES:
            raise ProcessContractError(f"prompt must encode to 1..={MAX_PROMPT_BYTES} UTF-8 bytes; got {size}")
    else:
        ids = list(prompt_ids)
        if not ids or any(type(i) is not int or i < 0 for i in ids):
            raise ProcessContractError("prompt_ids must be a non-empty list of non-negative integers")
    if tokenizer_file is not None and (os.path.islink(tokenizer_file) or not os.path.isfile(tokenizer_file)):
        raise ProcessContractError(f"tokenizer path must be a regular file, not a symlink: {tokenizer_file}")
    if type(device_ordinal) is not int or not 0 <= device_ordinal <= MAX_DEVICE_ORDINAL:
        raise ProcessContractError(f"device ordinal must be an integer in [0, {MAX_DEVICE_ORDINAL}]")
    if type(max_new_tokens) is not int or not 1 <= max_new_tokens <= MAX_NEW_TOKENS:
        raise ProcessContractError(f"max-new-tokens must be an integer in [1, {MAX_NEW_TOKENS}]; "
                                   f"got {max_new_tokens}")
    if not (isinstance(timeout_seconds, (int, float)) and 0 < float(timeout_seconds) < float("inf")):
        raise ProcessContractError("timeout must be a positive finite number of seconds")


class _Capture(threading.Thread):
    """Reads a pipe to its end, keeping at most MAX_CAPTURE_BYTES."""

    def __init__(self, pipe):
        super().__init__(daemon=True)
        self.pipe, self.kept, self.total = pipe, bytearray(), 0

    def run(self):
        while True:
            chunk = self.pipe.read(64 * 1024)
            if not chunk:
                return
            self.total += len(chunk)
            room = MAX_CAPTURE_BYTES - len(self.kept)
            if room > 0:
                self.kept += chunk[:room]


def run_bounded(command: List[str], timeout_seconds: float):
    """(exit code, stdout, stderr) of ``command`` run without a shell in a process
    group of its own.  Past the deadline exactly that group is ended (SIGTERM,
    then SIGKILL) and TimeoutError is raised; output beyond the cap is an error."""
    child = subprocess.Popen(command, stdin=subprocess.DEVNULL, stdout=subprocess.PIPE,
                             stderr=subprocess.PIPE, start_new_session=True)
    readers = [_Capture(child.stdout), _Capture(child.stderr)]
    for r in readers:
        r.start()
    deadline = time.monotonic() + float(timeout_seconds)
    timed_out = False
    try:
        child.wait(timeout=max(0.0, deadline - time.monotonic()))
    except subprocess.TimeoutExpired:
        timed_out = True
        for sig, grace in ((signal.SIGTERM, 5.0), (signal.SIGKILL, 5.0)):
            try:
                os.killpg(child.pid, sig)  # the group this call started, nothing else
            except ProcessLookupError:
                break
            try:
                child.wait(timeout=grace)
                break
            except subprocess.TimeoutExpired:
                continue
    for r in readers:
        r.join(timeout=5.0)
    if timed_out:
        raise TimeoutError(f"generation exceeded {timeout_seconds} s and was ended")
    for r, label in zip(readers, ("stdout", "stderr")):
        if r.total > MAX_CAPTURE_BYTES:
            raise RuntimeError(f"{label} exceeded {MAX_CAPTURE_BYTES} bytes")
    return child.returncode, bytes(readers[0].kept), bytes(readers[1].kept)


def _text(raw: bytes, label: str) -> str:
    try:
        return raw.decode("utf-8")
    except UnicodeDecodeError as e:
        raise RuntimeError(f"{label} of the generation is not valid UTF-8: {e}") from None


def build_result(inputs: Dict[str, Any], stdout: bytes, stderr: bytes) -> Dict[str, Any]:
    return {
        "schema_version": SCHEMA_VERSION,
        "contract": CONTRACT,
        "status": "generated",
        "inputs": inputs,
        "output": {
            "stdout_utf8": _text(stdout, "stdout"), "stdout_bytes": len(stdout),
            "stdout_sha256": hashlib.sha256(stdout).hexdigest(),
            "stderr_utf8": _text(stderr, "stderr"), "stderr_bytes": len(stderr),
            "stderr_sha256": hashlib.sha256(stderr).hexdigest(),
        },
        "sampling": "greedy",
        "network_access": False,
    }


def write_new_json(path: str, value: Dict[str, Any]) -> None:
    """The whole file or none, and never in place of an existing one."""
    tmp = f"{path}.tmp-{os.getpid()}"
    with open(tmp, "x", encoding="utf-8") as f:
        json.dump(value, f, indent=1, sort_keys=True)
        f.write("\n")
        f.flush()
        os.fsync(f.fileno())
    try:
        os.link(tmp, path)  # fails if `path` exists
    finally:
        os.unlink(tmp)


def execute(model_dir: str, tokenizer_file: Optional[str] = None, prompt: Optional[str] = None,
            device_ordinal: int = 0, max_new_tokens: int = 16, result_path: Optional[str] = None,
            timeout_seconds: float = DEFAULT_TIMEOUT_SECONDS, nnis_bin: Optional[str] = None,
            prompt_ids: Optional[Sequence[int]] = None, dtype: str = "bfloat16") -> Dict[str, Any]:
    """Greedy generation in a child process; the record is returned and, with
    ``result_path``, written there.  Raises ProcessContractError before anything
    runs, TimeoutError at the deadline, RuntimeError when the child fails."""
    check_request(model_dir, tokenizer_file, prompt, prompt_ids, device_ordinal, max_new_tokens,
                  timeout_seconds)
    if dtype not in ("bfloat16", "float32"):
        raise ProcessContractError(f"dtype must be bfloat16 or float32; got {dtype!r}")
    if result_path is not None and os.path.lexists(result_path):
        raise ProcessContractError(f"result path exists already: {result_path}")
    binary = nnis_bin if nnis_bin is not None else default_binary()
    command = [binary] if os.access(binary, os.X_OK) else [sys.executable, binary]
    command += ["generate", "--model", model_dir, "--device", str(device_ordinal),
                "--max-new-tokens", str(max_new_tokens), "--dtype", dtype]
    if tokenizer_file is not None:
        command += ["--tokenizer", tokenizer_file]
    if prompt is not None:
        command += ["--prompt", prompt]
    else:
        command += ["--prompt-ids", ",".join(str(int(i)) for i in prompt_ids)]
    code, stdout, stderr = run_bounded(command, timeout_seconds)
    if code != 0:
        tail = stderr[-4096:].decode("utf-8", "replace")
        raise RuntimeError(f"generation failed with exit code {code}: {tail}")
    inputs = {"model_directory": model_dir, "tokenizer_file": tokenizer_file, "prompt": prompt,
              "prompt_ids": list(prompt_ids) if prompt_ids is not None else None,
              "device_ordinal": device_ordinal, "max_new_tokens": max_new_tokens, "dtype": dtype}
    result = build_result(inputs, stdout, stderr)
    if result_path is not None:
        write_new_json(result_path, result)
    return result
