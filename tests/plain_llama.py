"""Plain, slow Llama decoder used as the oracle of every test.

Whole sequences, no cache, one function per part, float64 on the CPU (so that
what a comparison shows is the engine's rounding, not the oracle's).  It is
written from the formulas of Memorithm/NNIS (each function cites the file and
lines of that project it follows) and shares no code with ``nnis_b200``: it
reads ``config.json`` keys and Hugging Face tensor names by itself.

NNIS's own model code is Rust with NVRTC kernel strings; neither a Rust
toolchain nor a GPU is present where the tests are written, so this file rests
on the formulas alone and was not compared with a run of NNIS.

``emulate_bf16=True`` rounds to bfloat16 at the tensor boundaries where the
bfloat16 engine stores bfloat16 (norm outputs, q/k/v, rotated q/k, attention
output, the gated activation); everything between is unrounded.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch

Tensor = torch.Tensor


F = torch.float64


def _round(x: Tensor, emulate_bf16: bool) -> Tensor:
    return x.to(torch.bfloat16).to(F) if emulate_bf16 else x


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------
def embed(table: Tensor, tokens: Sequence[int]) -> Tensor:
    """hidden = E[token, :] (crates/nnis-kernels/src/gather.rs:17-33,
    crates/nnis-model/src/runtime.rs:933-940)."""
    return table.to(F)[torch.tensor(list(tokens), dtype=torch.long)]


def rms_norm(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    """y = (x * rsqrt(mean(x^2) + eps)) * w
    (crates/nnis-model/src/kernels.rs:15-48)."""
    x = x.to(F)
    ss = (x * x).sum(dim=-1, keepdim=True)
    s = 1.0 / torch.sqrt(ss * (1.0 / x.shape[-1]) + eps)
    return (x * s) * weight.to(F)


def linear(x: Tensor, weight: Tensor, bias: Optional[Tensor] = None) -> Tensor:
    """y = x . W^T (+ b); W is [out, in] as Hugging Face stores it
    (crates/nnis-model/src/runtime.rs:959-985; layout
    crates/nnis-model/src/safetensors_loader.rs:482-502)."""
    y = x.to(F) @ weight.to(F).t()
    if bias is not None:
        y = y + bias.to(F)
    return y


def rope_tables(positions: int, head_dim: int, theta: float):
    """cos/sin [positions, head_dim/2] in float32:
    inv_f = 1 / theta^(2j/d), angle = pos * inv_f
    (crates/nnis-model/src/runtime.rs:1166-1184)."""
    half = head_dim // 2
    expo = (2 * torch.arange(half, dtype=torch.float32)) / float(head_dim)
    inv_f = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32), expo)
    ang = torch.arange(positions, dtype=torch.float32)[:, None] * inv_f[None, :]
    return torch.cos(ang).to(F), torch.sin(ang).to(F)


def rope_rotate_half(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """x [T, heads, d]; pairs (j, j + d/2): a' = a c - b s, b' = b c + a s
    (crates/nnis-model/src/runtime_kernels.rs:38-66)."""
    x = x.to(F)
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1)


def causal_attention(q: Tensor, k: Tensor, v: Tensor, window: int = 0) -> Tensor:
    """q [T, nq, d], k/v [T, nkv, d] -> [T, nq, d].

    score = (q . k) / sqrt(d); query head hq reads kv head hq // (nq/nkv); key t
    is visible to query p when t <= p (and p - t < window when a window is set);
    softmax unrounded (crates/nnis-model/src/kernels.rs:66-125; the causal rule
    crates/nnis-kernels/src/attention.rs:97-108)."""
    q, k, v = q.to(F), k.to(F), v.to(F)
    T, nq, d = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    scale = 1.0 / math.sqrt(float(d))
    out = torch.empty_like(q)
    pos = torch.arange(T)
    visible = pos[None, :] <= pos[:, None]
    if window > 0:
        visible &= (pos[:, None] - pos[None, :]) < window
    for hq in range(nq):
        hk = hq // group
        s = (q[:, hq, :] @ k[:, hk, :].t()) * scale
        s = s.masked_fill(~visible, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, hq, :] = p @ v[:, hk, :]
    return out


def swiglu(g: Tensor, u: Tensor) -> Tensor:
    """silu(g) * u with silu(g) = g / (1 + exp(-g))
    (crates/nnis-model/src/fused_swiglu.rs:14-27)."""
    g, u = g.to(F), u.to(F)
    return (g / (1.0 + torch.exp(-g))) * u


# --------------------------------------------------------------------------
# whole model
# --------------------------------------------------------------------------
def _cfg_sizes(cfg: dict):
    H = cfg["hidden_size"]
    nq = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nq)
    d = cfg.get("head_dim") or H // nq
    return H, nq, nkv, d


def attention_layer(cfg: dict, w: Dict[str, Tensor], prefix: str, n: Tensor, cos: Tensor,
                    sin: Tensor, emulate_bf16: bool, window: int = 0) -> Tensor:
    """Steps 4-10 of one token pass (crates/nnis-model/src/runtime.rs:959-1029)."""
    H, nq, nkv, d = _cfg_sizes(cfg)
    T = n.shape[0]
    bias = cfg.get("attention_bias", False)

    def b(name):
        return w[prefix + name + ".bias"] if bias else None

    q = _round(linear(n, w[prefix + "q_proj.weight"], b("q_proj")), emulate_bf16).view(T, nq, d)
    k = _round(linear(n, w[prefix + "k_proj.weight"], b("k_proj")), emulate_bf16).view(T, nkv, d)
    v = _round(linear(n, w[prefix + "v_proj.weight"], b("v_proj")), emulate_bf16).view(T, nkv, d)
    q = _round(rope_rotate_half(q, cos[:T], sin[:T]), emulate_bf16)
    k = _round(rope_rotate_half(k, cos[:T], sin[:T]), emulate_bf16)
    a = _round(causal_attention(q, k, v, window), emulate_bf16).reshape(T, nq * d)
    return linear(a, w[prefix + "o_proj.weight"], b("o_proj"))


def mlp_layer(cfg: dict, w: Dict[str, Tensor], prefix: str, n: Tensor,
              emulate_bf16: bool) -> Tensor:
    """Steps 14-17 (crates/nnis-model/src/runtime.rs:1054-1087)."""
    bias = cfg.get("mlp_bias", False)

    def b(name):
        return w[prefix + name + ".bias"] if bias else None

    g = linear(n, w[prefix + "gate_proj.weight"], b("gate_proj"))
    u = linear(n, w[prefix + "up_proj.weight"], b("up_proj"))
    return linear(_round(swiglu(g, u), emulate_bf16), w[prefix + "down_proj.weight"],
                  b("down_proj"))


def forward(cfg: dict, w: Dict[str, Tensor], tokens: Sequence[int],
            emulate_bf16: bool = False) -> Tensor:
    """Logits [T, vocab] of one whole sequence
    (crates/nnis-model/src/runtime.rs:918-1120)."""
    H, nq, nkv, d = _cfg_sizes(cfg)
    eps = cfg["rms_norm_eps"]
    T = len(tokens)
    cos, sin = rope_tables(T, d, float(cfg["rope_theta"]))
    h = embed(w["model.embed_tokens.weight"], tokens)
    for layer in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        n = _round(rms_norm(h, w[p + "input_layernorm.weight"], eps), emulate_bf16)
        h = h + attention_layer(cfg, w, p + "self_attn.", n, cos, sin, emulate_bf16)
        n = _round(rms_norm(h, w[p + "post_attention_layernorm.weight"], eps), emulate_bf16)
        h = h + mlp_layer(cfg, w, p + "mlp.", n, emulate_bf16)
    n = _round(rms_norm(h, w["model.norm.weight"], eps), emulate_bf16)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) \
        else w["lm_head.weight"]
    return linear(n, head)


def argmax_lowest(logits: Tensor) -> int:
    """Larger wins, ties go to the lower index
    (crates/nnis-kernels/src/top_k.rs:57-70)."""
    best, idx = None, 0
    for i, v in enumerate(logits.tolist()):
        if best is None or v > best:
            best, idx = v, i
    return idx


def greedy_generate(cfg: dict, w: Dict[str, Tensor], prompt: Sequence[int], max_new_tokens: int,
                    eos_token_id: Optional[int] = None, emulate_bf16: bool = False) -> List[int]:
    """Greedy loop: the stop token is emitted and ends the sequence
    (crates/nnis-model/src/runtime.rs:848-899)."""
    tokens = list(prompt)
    out: List[int] = []
    for _ in range(max_new_tokens):
        logits = forward(cfg, w, tokens, emulate_bf16)[-1]
        t = argmax_lowest(logits)
        out.append(t)
        tokens.append(t)
        if eos_token_id is not None and t == eos_token_id:
            break
    return out


# --------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------
class PlainSplitMix64:
    """crates/nnis-model/src/sampling.rs:261-284."""
    MASK = (1 << 64) - 1

    def __init__(self, seed: int):
        self.state = seed & self.MASK

    def next_u64(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & self.MASK
        v = self.state
        v = ((v ^ (v >> 30)) * 0xBF58476D1CE4E5B9) & self.MASK
        v = ((v ^ (v >> 27)) * 0x94D049BB133111EB) & self.MASK
        return v ^ (v >> 31)

    def next_unit(self) -> float:
        return (self.next_u64() >> 11) * (1.0 / float(1 << 53))


def plain_sample(logits: Sequence[float], rng: PlainSplitMix64, temperature: float = 1.0,
                 top_k: Optional[int] = None, top_p: Optional[float] = None) -> int:
    """Sort (logit descending, id ascending) -> top-k -> temperature softmax in
    float64 -> top-p -> one draw (crates/nnis-model/src/sampling.rs:113-202)."""
    cand = sorted(range(len(logits)), key=lambda i: (-float(logits[i]), i))
    if top_k is not None:
        cand = cand[:top_k]
    inv_t = 1.0 / float(torch.tensor(temperature, dtype=torch.float32))
    mx = float(logits[cand[0]]) * inv_t
    weights = [math.exp(float(logits[i]) * inv_t - mx) for i in cand]
    total = sum(weights)
    if top_p is not None:
        threshold = float(torch.tensor(top_p, dtype=torch.float32)) * total
        cum, keep = 0.0, len(cand)
        for j, wt in enumerate(weights):
            cum += wt
            if cum >= threshold:
                keep = j + 1
                break
        keep = max(keep, 1)
        cand, weights = cand[:keep], weights[:keep]
        total = sum(weights)
    draw = rng.next_unit() * total
    cum = 0.0
    for i, wt in zip(cand, weights):
        cum += wt
        if draw < cum:
            return i
    return cand[-1]
