"""Each part alone against its plain function, and toy parts defined here (a
mixer with state of its own, a feed-forward that routes tokens to experts, another
position encoding), registered, built and stepped without touching the
framework's files."""
import math

import numpy as np
import pytest
import torch

import plain_llama as P
from helpers import check_logits
from nnis_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def prenorm_layer(prefix, mixer_norm, mixer, ffn_norm, ffn):
    return LayerSpec(prefix, "prenorm", {"mixer_norm": mixer_norm, "mixer": mixer,
                                         "ffn_norm": ffn_norm, "ffn": ffn})


def close(got, want, dtype, what=""):
    got, want = got.double().cpu(), want.double().cpu()
    t = dict(rtol=2e-5, atol=2e-5) if dtype == "float32" else dict(rtol=2e-2, atol=2e-2)
    ok = torch.isclose(got, want, **t)
    assert ok.all(), f"{what}: {int((~ok).sum())} of {ok.numel()} differ, max {float((got-want).abs().max()):.3e}"


def make_ctx(cache, slots, counts, workspace):
    """A StepContext for packed tokens, built by hand."""
    from nnis_b200.engine.context import StepContext
    starts = [cache.length(s) for s in slots]
    new = [a + b for a, b in zip(starts, counts)]
    cache.reserve(slots, new)
    pos, seq = [], []
    for i, (a, b) in enumerate(zip(starts, new)):
        pos += list(range(a, b))
        seq += [i] * (b - a)
    cols = max(-(-L // 64) for L in new)
    tables = []
    for g in range(len(cache.groups)):
        rows = [(cache.page_table(g, s) + [-1] * cols)[:cols] for s in slots]
        tables.append(torch.tensor(rows, dtype=torch.int32, device=DEV))
    n = len(pos)
    ctx = StepContext(
        n_tokens=n, n_seqs=len(slots), tokens=torch.zeros(n, dtype=torch.int32, device=DEV),
        token_pos=torch.tensor(pos, dtype=torch.int32, device=DEV),
        token_seq=torch.tensor(seq, dtype=torch.int32, device=DEV),
        seq_slots=torch.tensor(slots, dtype=torch.int32, device=DEV), page_tables=tables,
        workspace=workspace, decode=all(c == 1 for c in counts), max_context=max(new),
        host_slots=slots, host_counts=counts, host_starts=starts)
    return ctx, new


@pytest.mark.parametrize("dtype", list(DT))
def test_norm_part(dtype):
    from nnis_b200.parts import NORMS
    part = NORMS.build("rmsnorm", {"size": 72, "eps": 1e-6, "name": "ln"}, "blk", DT[dtype], DEV)
    assert list(part.weight_specs()) == ["blk.ln.weight"]
    w = 1 + 0.2 * torch.randn(72)
    part.load({"blk.ln.weight": w.to(DEV)})
    x = torch.randn(5, 72) * 2
    out = torch.empty(5, 72, dtype=DT[dtype], device=DEV)
    part.forward(x.to(DEV), out)
    close(out, P.rms_norm(x, w, 1e-6), dtype, "norm part")


def test_position_part_builds_the_reference_table():
    from nnis_b200.parts import POSITIONS
    part = POSITIONS.build("rope_half", {"head_dim": 48, "theta": 500000.0, "max_positions": 300},
                           "", torch.float32, DEV)
    cos, sin = part.rotary_tables()
    pc, ps = P.rope_tables(300, 48, 500000.0)
    assert torch.equal(cos.cpu().double(), pc) and torch.equal(sin.cpu().double(), ps)
    assert POSITIONS.build("none", {}, "", torch.float32, DEV).rotary_tables() is None


@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("dtype", list(DT))
def test_feed_forward_part(dtype, decode):
    from nnis_b200.engine.workspace import Workspace
    from nnis_b200.parts import FEED_FORWARDS
    H, I = 40, 88
    params = {"hidden_size": H, "intermediate_size": I, "activation": "silu", "bias": True,
              "names": {"gate": "g", "up": "u", "down": "d"}}
    part = FEED_FORWARDS.build("gated_mlp", params, "L", DT[dtype], DEV)
    specs = part.weight_specs()
    assert specs["L.g.weight"].shape == (I, H) and specs["L.d.bias"].shape == (H,)
    g = torch.Generator().manual_seed(0)
    w = {n: (torch.randn(s.shape, generator=g) / math.sqrt(s.shape[-1])) for n, s in specs.items()}
    w = {n: (t.to(DT[dtype]) if specs[n].role == "matrix" else t) for n, t in w.items()}
    part.load({n: t.to(DEV) for n, t in w.items()})
    x = torch.randn(6, H).to(DT[dtype])
    residual = torch.randn(6, H)
    res = residual.to(DEV).clone()

    class Ctx:  # decode steps take the fused kernels in bfloat16
        workspace = Workspace(DEV)
    Ctx.decode = decode
    part.forward(x.to(DEV), Ctx, res)
    bf = dtype == "bfloat16"
    gate = P.linear(x, w["L.g.weight"], w["L.g.bias"])
    up = P.linear(x, w["L.u.weight"], w["L.u.bias"])
    want = residual.double() + P.linear(P._round(P.swiglu(gate, up), bf), w["L.d.weight"],
                                        w["L.d.bias"])
    close(res, want, dtype, "feed-forward part")


def attention_params(H, nq, nkv, d, window=0, bias=False, position="rope_half", kv="own"):
    pos = PartSpec(position, {"head_dim": d, "theta": 10000.0, "max_positions": 512})
    return {"hidden_size": H, "heads": nq, "kv_heads": nkv, "head_dim": d, "bias": bias,
            "window": window, "position": pos, "kv": kv,
            "names": {"q": "q", "k": "k", "v": "v", "o": "o"}}


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("window,position", [(0, "rope_half"), (50, "rope_half"), (0, "none")])
def test_attention_part_prompt_then_tokens(dtype, window, position):
    """The mixer alone: a prompt in one step, then single tokens, two sequences
    of unequal length, against the plain functions on the whole sequences."""
    from nnis_b200.cache import CacheManager
    from nnis_b200.engine.workspace import Workspace
    from nnis_b200.parts import MIXERS
    H, nq, nkv, d = 56, 6, 3, 32
    part = MIXERS.build("attention", attention_params(H, nq, nkv, d, window, True, position), "L",
                        DT[dtype], DEV)
    specs = part.weight_specs()
    g = torch.Generator().manual_seed(1)
    w = {n: torch.randn(s.shape, generator=g) / math.sqrt(s.shape[-1]) for n, s in specs.items()}
    w = {n: (t.to(DT[dtype]) if specs[n].role == "matrix" else t) for n, t in w.items()}
    part.load({n: t.to(DEV) for n, t in w.items()})
    cache = CacheManager([part.cache_request()], DT[dtype], DEV, 64 * 16, 4, 512)
    view, ws = cache.view(0), Workspace(DEV)
    lengths = [150, 90]
    x = [torch.randn(L, H, generator=g).to(DT[dtype]) for L in lengths]
    bf = dtype == "bfloat16"
    cfg = {"hidden_size": H, "num_attention_heads": nq, "num_key_value_heads": nkv, "head_dim": d,
           "attention_bias": True}
    pw = {"q_proj.weight": w["L.q.weight"], "k_proj.weight": w["L.k.weight"],
          "v_proj.weight": w["L.v.weight"], "o_proj.weight": w["L.o.weight"],
          "q_proj.bias": w["L.q.bias"], "k_proj.bias": w["L.k.bias"], "v_proj.bias": w["L.v.bias"],
          "o_proj.bias": w["L.o.bias"]}
    cos, sin = P.rope_tables(512, d, 10000.0)
    if position == "none":
        cos, sin = torch.ones_like(cos), torch.zeros_like(sin)
    want = [P.attention_layer(cfg, pw, "", xi.double(), cos, sin, bf, window) for xi in x]
    slots = [cache.acquire(), cache.acquire()]
    fed = [0, 0]
    for counts in ([120, 70], [1, 1], [1, 1], [28, 18]):
        ctx, new = make_ctx(cache, slots, counts, ws)
        xin = torch.cat([x[i][fed[i]:fed[i] + c] for i, c in enumerate(counts)]).to(DEV)
        res = torch.zeros(sum(counts), H, device=DEV)
        part.forward(xin, ctx, res, view)
        cache.commit(slots, new)
        o = 0
        for i, c in enumerate(counts):
            close(res[o:o + c], want[i][fed[i]:fed[i] + c], dtype,
                  f"attention part seq {i} at {fed[i]}")
            o += c
            fed[i] += c


# ---------------------------------------------------------------------------
# A toy mixer with state of its own: a per-channel running mean of its inputs.
# It is no model's part; it shows that the registries, the cache's state area
# and the step function need no change for a mixer that keeps no keys.
# ---------------------------------------------------------------------------
def _register_toy():
    from nnis_b200.cache import StateRequest
    from nnis_b200.parts import MIXERS, Part
    from nnis_b200.weights import WeightSpec

    class RunningMean(Part):
        def __init__(self, params, prefix, dtype, device):
            super().__init__(params, prefix, dtype, device)
            self.width = params["width"]
            self.name = self.tensor_name("mix")

        def weight_specs(self):
            return {self.name: WeightSpec((self.width,), "vector")}

        def load(self, tensors):
            self.gain = tensors[self.name]

        def cache_request(self):
            return StateRequest((self.width + 1,))  # running sum and count

        def forward(self, x, ctx, residual, cache):
            o = 0
            for slot, count in zip(ctx.host_slots, ctx.host_counts):
                state = cache.state[slot]
                for t in range(count):
                    state[:self.width] += x[o + t].float()
                    state[self.width] += 1.0
                    residual[o + t] += self.gain * state[:self.width] / state[self.width]
                o += count

    MIXERS.register("toy_running_mean", RunningMean)


def _toy_plain(tokens, embed, gains, norm_w, head, eps, mlp):
    """The same model, whole sequence, float64."""
    h = embed.double()[torch.tensor(tokens)]
    for gain, (n1, n2, wg, wu, wd) in zip(gains, mlp):
        n = P.rms_norm(h, n1, eps)
        mean = torch.cumsum(n, 0) / torch.arange(1, len(tokens) + 1, dtype=torch.float64)[:, None]
        h = h + gain.double() * mean
        n = P.rms_norm(h, n2, eps)
        h = h + P.linear(P.swiglu(P.linear(n, wg), P.linear(n, wu)), wd)
    return P.linear(P.rms_norm(h, norm_w, eps), head)


def test_a_toy_mixer_with_its_own_state_is_registered_built_and_stepped():
    from nnis_b200.engine import Engine, SequenceStep
    from nnis_b200.engine.model import DecoderModel
    from nnis_b200.weights import random_tensors
    _register_toy()
    H, V, I, eps = 24, 50, 40, 1e-5
    norm = lambda name: PartSpec("rmsnorm", {"size": H, "eps": eps, "name": name})
    layers = tuple(prenorm_layer(
        f"blocks.{i}", norm("n1"), PartSpec("toy_running_mean", {"width": H}), norm("n2"),
        PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": I, "activation": "silu",
                               "bias": False, "names": {"gate": "g", "up": "u", "down": "d"}}))
        for i in range(2))
    spec = ModelSpec(architecture="ToyRunningMean", hidden_size=H, vocab_size=V, max_positions=256,
                     embedding=PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H,
                                                            "name": "emb"}),
                     layers=layers, schedule=(ScheduleEntry(0), ScheduleEntry(1)),
                     final_norm=norm("final"),
                     head=PartSpec("linear_head", {"vocab_size": V, "hidden_size": H, "name": "head",
                                                   "tied_to": None}))
    wanted = DecoderModel.weight_specs_of(spec)
    assert "blocks.1.mix.weight" in wanted
    tensors = random_tensors(wanted, seed=3, std=1.0, norm_std=0.1, std_by_fan_in=True)
    engine = Engine.from_spec(spec, tensors, dtype="float32", max_tokens=64 * 8, max_slots=3)
    assert engine.cache.groups == [] and engine.cache.view(0).state.shape == (3, H + 1)
    seqs = {"a": [3, 1, 4, 1, 5, 9, 2, 6], "b": [2, 7, 1, 8]}
    mlp = [(tensors[f"blocks.{i}.n1.weight"], tensors[f"blocks.{i}.n2.weight"],
            tensors[f"blocks.{i}.g.weight"], tensors[f"blocks.{i}.u.weight"],
            tensors[f"blocks.{i}.d.weight"]) for i in range(2)]
    gains = [tensors[f"blocks.{i}.mix.weight"] for i in range(2)]
    want = {k: _toy_plain(v, tensors["emb.weight"], gains, tensors["final.weight"],
                          tensors["head.weight"], eps, mlp) for k, v in seqs.items()}
    for round_ in range(2):  # the second round reuses the slots: state must start from zero
        sa, sb = engine.acquire_slot(), engine.acquire_slot()
        got = engine.step([SequenceStep(sa, seqs["a"][:5], [0, 4]), SequenceStep(sb, seqs["b"][:2], [1])])
        check_logits(got.cpu().numpy(), torch.stack([want["a"][0], want["a"][4], want["b"][1]]),
                     "float32", f"toy prompt round {round_}")
        for t in range(2):
            got = engine.step([SequenceStep(sa, [seqs["a"][5 + t]], [0]),
                               SequenceStep(sb, [seqs["b"][2 + t]], [0])])
            check_logits(got.cpu().numpy(), torch.stack([want["a"][5 + t], want["b"][2 + t]]),
                         "float32", f"toy token {t} round {round_}")
        engine.release_slot(sb)
        # the way back for a model with state: a snapshot before tokens that are taken back
        with pytest.raises(Exception, match="snapshot"):
            engine.truncate(sa, 3)
        snap = engine.snapshot(sa)
        engine.step([SequenceStep(sa, [11, 12, 13], [])])
        engine.restore(snap)
        assert engine.cache.length(sa) == 7
        got = engine.step([SequenceStep(sa, [seqs["a"][7]], [0])])
        check_logits(got.cpu().numpy(), want["a"][7:8], "float32", "toy tail")
        engine.release_slot(sa)


def test_schedule_runs_a_layer_twice_and_lets_a_layer_read_anothers_cache():
    """Run order as data: layer 0, layer 1 reading entry 0's cache, layer 0 again."""
    from nnis_b200.engine import Engine, SequenceStep
    from nnis_b200.engine.model import DecoderModel
    from nnis_b200.weights import random_tensors
    H, V, I, nq, nkv, d, eps = 32, 40, 48, 2, 1, 16, 1e-5
    norm = lambda name: PartSpec("rmsnorm", {"size": H, "eps": eps, "name": name})
    ffn = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": I, "activation": "silu",
                                 "bias": False, "names": {"gate": "g", "up": "u", "down": "d"}})
    layers = (prenorm_layer("l0", norm("n1"), PartSpec("attention", attention_params(H, nq, nkv, d)),
                            norm("n2"), ffn),
              prenorm_layer("l1", norm("n1"),
                            PartSpec("attention", attention_params(H, nq, nkv, d, kv="shared")),
                            norm("n2"), ffn))
    spec = ModelSpec(architecture="ToySchedule", hidden_size=H, vocab_size=V, max_positions=512,
                     embedding=PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H, "name": "emb"}),
                     layers=layers,
                     schedule=(ScheduleEntry(0), ScheduleEntry(1, cache_of=0), ScheduleEntry(0)),
                     final_norm=norm("final"),
                     head=PartSpec("linear_head", {"vocab_size": V, "hidden_size": H, "name": "head",
                                                   "tied_to": "emb"}))
    wanted = DecoderModel.weight_specs_of(spec)
    assert "l1.k.weight" not in wanted and "l1.q.weight" in wanted and "head.weight" not in wanted
    w = random_tensors(wanted, seed=8, std=1.0, norm_std=0.1, std_by_fan_in=True)
    engine = Engine.from_spec(spec, w, dtype="float32", max_tokens=64 * 8, max_slots=2)
    assert len(engine.cache.groups) == 1 and len(engine.cache.groups[0].entries) == 2
    tokens = [5, 17, 3, 39, 0, 22, 8, 8, 1]
    T = len(tokens)
    cos, sin = P.rope_tables(T, d, 10000.0)

    def attn(prefix, n, kv_from=None):
        q = P.rope_rotate_half(P.linear(n, w[prefix + ".q.weight"]).view(T, nq, d), cos, sin)
        if kv_from is None:
            k = P.rope_rotate_half(P.linear(n, w[prefix + ".k.weight"]).view(T, nkv, d), cos, sin)
            v = P.linear(n, w[prefix + ".v.weight"]).view(T, nkv, d)
        else:
            k, v = kv_from
        out = P.causal_attention(q, k, v).reshape(T, nq * d)
        return P.linear(out, w[prefix + ".o.weight"]), (k, v)

    h = w["emb.weight"].double()[torch.tensor(tokens)]
    kv0 = None
    for prefix, shared in (("l0", False), ("l1", True), ("l0", False)):
        n = P.rms_norm(h, w[prefix + ".n1.weight"], eps)
        a, kv = attn(prefix, n, kv0 if shared else None)
        if kv0 is None:
            kv0 = kv
        h = h + a
        n = P.rms_norm(h, w[prefix + ".n2.weight"], eps)
        h = h + P.linear(P.swiglu(P.linear(n, w[prefix + ".g.weight"]), P.linear(n, w[prefix + ".u.weight"])),
                         w[prefix + ".d.weight"])
    want = P.linear(P.rms_norm(h, w["final.weight"], eps), w["emb.weight"])
    slot = engine.acquire_slot()
    got = engine.step([SequenceStep(slot, tokens[:6], range(6))])
    check_logits(got.cpu().numpy(), want[:6], "float32", "schedule prompt")
    for t in range(6, T):
        got = engine.step([SequenceStep(slot, [tokens[t]], [0])])
        check_logits(got.cpu().numpy(), want[t:t + 1], "float32", f"schedule token {t}")
    engine.release_slot(slot)


# ---------------------------------------------------------------------------
# Two more toys, defined here and registered without a change to the framework:
# a feed-forward that routes every token to one of a few small experts, and a
# position encoding whose angles are those of RoPE at a fraction of the position.
# They are no model's parts; they show what the FEED_FORWARDS and POSITIONS
# registries ask of a new kind.
# ---------------------------------------------------------------------------
def _register_routed_and_interpolated():
    from nnis_b200.parts import FEED_FORWARDS, POSITIONS, Part
    from nnis_b200.parts.linear import STORE, linear
    from nnis_b200.weights import WeightSpec

    class TopOneExperts(Part):
        device_only = False  # the routing decision is read on the host

        def __init__(self, params, prefix, dtype, device):
            super().__init__(params, prefix, dtype, device)
            self.h, self.i, self.e = params["hidden_size"], params["expert_size"], params["experts"]

        def weight_specs(self):
            specs = {self.tensor_name("router"): WeightSpec((self.e, self.h), "matrix", fan_in=self.h)}
            for e in range(self.e):
                specs[self.tensor_name(f"expert{e}.up")] = WeightSpec((self.i, self.h), "matrix", fan_in=self.h)
                specs[self.tensor_name(f"expert{e}.down")] = WeightSpec((self.h, self.i), "matrix", fan_in=self.i)
            return specs

        def load(self, tensors):
            self.router = tensors[self.tensor_name("router")].float()
            self.up = [tensors[self.tensor_name(f"expert{e}.up")] for e in range(self.e)]
            self.down = [tensors[self.tensor_name(f"expert{e}.down")] for e in range(self.e)]

        def forward(self, x, ctx, residual):
            logits = x.float() @ self.router.t()                 # router logits in float32
            prob = torch.softmax(logits, dim=-1)
            choice = torch.argmax(logits, dim=-1)                # ties go to the lower expert
            for e in range(self.e):
                rows = torch.nonzero(choice == e).flatten()
                if rows.numel() == 0:
                    continue
                xe = x[rows].contiguous()
                mid = torch.empty(rows.numel(), self.i, dtype=x.dtype, device=x.device)
                linear(xe, self.up[e], None, mid, STORE)         # the framework's own product kernels
                mid = torch.relu(mid)
                out = torch.empty(rows.numel(), self.h, dtype=x.dtype, device=x.device)
                linear(mid, self.down[e], None, out, STORE)
                residual[rows] += prob[rows, e, None] * out.float()

    class InterpolatedRope(Part):
        def __init__(self, params, prefix, dtype, device):
            super().__init__(params, prefix, dtype, device)
            d, factor = int(params["head_dim"]), float(params["factor"])
            inv = 1.0 / torch.pow(torch.tensor(float(params["theta"])), 2 * torch.arange(d // 2).float() / d)
            angle = (torch.arange(int(params["max_positions"])).float() / factor)[:, None] * inv[None, :]
            self.cos, self.sin = torch.cos(angle).to(device), torch.sin(angle).to(device)

        def rotary_tables(self):
            return self.cos, self.sin

    FEED_FORWARDS.register("toy_top1_experts", TopOneExperts)
    POSITIONS.register("toy_interpolated_rope", InterpolatedRope)


def test_a_toy_routed_feed_forward_and_a_toy_position_encoding_run_in_a_model():
    from nnis_b200.engine import Engine, SequenceStep
    from nnis_b200.engine.model import DecoderModel
    from nnis_b200.weights import random_tensors
    _register_routed_and_interpolated()
    H, V, I, E, nq, nkv, d, eps, factor = 40, 60, 24, 3, 4, 2, 16, 1e-5, 4.0
    norm = lambda name: PartSpec("rmsnorm", {"size": H, "eps": eps, "name": name})
    toy_pos = PartSpec("toy_interpolated_rope", {"head_dim": d, "theta": 10000.0, "max_positions": 512,
                                                 "factor": factor})
    attn0 = dict(attention_params(H, nq, nkv, d), position=toy_pos)
    layers = (prenorm_layer("l0", norm("n1"), PartSpec("attention", attn0), norm("n2"),
                            PartSpec("toy_top1_experts", {"hidden_size": H, "expert_size": I, "experts": E})),
              prenorm_layer("l1", norm("n1"), PartSpec("attention", attention_params(H, nq, nkv, d)),
                            norm("n2"),
                            PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": I, "activation": "silu",
                                                   "bias": False, "names": {"gate": "g", "up": "u", "down": "d"}})))
    spec = ModelSpec(architecture="ToyRouted", hidden_size=H, vocab_size=V, max_positions=512,
                     embedding=PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H, "name": "emb"}),
                     layers=layers, schedule=(ScheduleEntry(0), ScheduleEntry(1)), final_norm=norm("final"),
                     head=PartSpec("linear_head", {"vocab_size": V, "hidden_size": H, "name": "head",
                                                   "tied_to": "emb"}))
    wanted = DecoderModel.weight_specs_of(spec)
    assert "l0.expert2.down.weight" in wanted and "l0.router.weight" in wanted
    w = random_tensors(wanted, seed=21, std=1.0, norm_std=0.1, std_by_fan_in=True)
    w["l0.router.weight"] = w["l0.router.weight"] * 4  # choices well apart from ties
    engine = Engine.from_spec(spec, w, dtype="float32", max_tokens=64 * 8, max_slots=2)

    def plain(tokens):
        T = len(tokens)
        h = w["emb.weight"].double()[torch.tensor(tokens)]
        inv = 1.0 / torch.pow(torch.tensor(10000.0, dtype=torch.float64), 2 * torch.arange(d // 2).double() / d)
        for prefix, f in (("l0", factor), ("l1", 1.0)):
            angle = (torch.arange(T).double() / f)[:, None] * inv[None, :]
            cos, sin = torch.cos(angle), torch.sin(angle)
            n = P.rms_norm(h, w[prefix + ".n1.weight"], eps)
            q = P.rope_rotate_half(P.linear(n, w[prefix + ".q.weight"]).view(T, nq, d), cos, sin)
            k = P.rope_rotate_half(P.linear(n, w[prefix + ".k.weight"]).view(T, nkv, d), cos, sin)
            v = P.linear(n, w[prefix + ".v.weight"]).view(T, nkv, d)
            h = h + P.linear(P.causal_attention(q, k, v).reshape(T, nq * d), w[prefix + ".o.weight"])
            n = P.rms_norm(h, w[prefix + ".n2.weight"], eps)
            if prefix == "l0":
                logits = P.linear(n, w["l0.router.weight"])
                prob, choice = torch.softmax(logits, -1), torch.argmax(logits, -1)
                used.update(choice.tolist())
                for t in range(T):
                    e = int(choice[t])
                    mid = torch.relu(P.linear(n[t:t + 1], w[f"l0.expert{e}.up.weight"]))
                    h[t] = h[t] + prob[t, e] * P.linear(mid, w[f"l0.expert{e}.down.weight"])[0]
            else:
                h = h + P.linear(P.swiglu(P.linear(n, w["l1.g.weight"]), P.linear(n, w["l1.u.weight"])),
                                 w["l1.d.weight"])
        return P.linear(P.rms_norm(h, w["final.weight"], eps), w["emb.weight"])

    used = set()
    seqs = {"a": [3, 14, 15, 9, 26, 5, 35, 8, 9, 7, 9, 32], "b": [38, 4, 6, 26, 43]}
    want = {k: plain(v) for k, v in seqs.items()}
    assert len(used) > 1, "the toy router sent every token to one expert"
    sa, sb = engine.acquire_slot(), engine.acquire_slot()
    got = engine.step([SequenceStep(sa, seqs["a"][:9], range(9)), SequenceStep(sb, seqs["b"][:3], [2])])
    check_logits(got.cpu().numpy(), torch.cat([want["a"][:9], want["b"][2:3]]), "float32", "routed prompt")
    for t in range(2):
        got = engine.step([SequenceStep(sa, [seqs["a"][9 + t]], [0]), SequenceStep(sb, [seqs["b"][3 + t]], [0])])
        check_logits(got.cpu().numpy(), torch.stack([want["a"][9 + t], want["b"][3 + t]]), "float32",
                     f"routed token {t}")
    engine.release_slot(sb)
    got = engine.step([SequenceStep(sa, [seqs["a"][11]], [0])])
    check_logits(got.cpu().numpy(), want["a"][11:12], "float32", "routed tail")
    engine.release_slot(sa)


# ---------------------------------------------------------------------------
# Toys for the remaining seams, again registered from here: a block arrangement with
# other sub-layers than the pre-norm one (a norm after the mixer, a third sub-layer),
# position encodings with arithmetic of their own (pairs of neighbours; half of the
# head), an embedding with a scale and a head with a soft cap.  No model's parts.
# ---------------------------------------------------------------------------
def _register_seam_toys():
    from nnis_b200.csrc import ops
    from nnis_b200.parts import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS,
                                 Block, LinearHead, PositionEncoding, TokenEmbedding)

    class SandwichBlock(Block):
        """h += post(mixer(pre(h))); h += ffn(n2(h)); h += extra(n3(h))."""

        def __init__(self, layer_spec, dtype, device):
            super().__init__(layer_spec, dtype, device)
            self.pre, self.post = self.build(NORMS, "pre"), self.build(NORMS, "post")
            self.mixer = self.build(MIXERS, "mixer")
            self.n2, self.ffn = self.build(NORMS, "n2"), self.build(FEED_FORWARDS, "ffn")
            self.n3, self.extra = self.build(NORMS, "n3"), self.build(FEED_FORWARDS, "extra")

        def parts(self):
            return (self.pre, self.post, self.mixer, self.n2, self.ffn, self.n3, self.extra)

        def forward(self, hidden, ctx, cache):
            n, width = hidden.shape
            normed = ctx.workspace.get("normed", (n, width), self.dtype)
            branch = ctx.workspace.get("toy_branch", (n, width), torch.float32)
            self.pre.forward(hidden, normed)
            branch.zero_()
            self.mixer.forward(normed, ctx, branch, cache)   # the mixer adds into what it is given
            post = ctx.workspace.get("toy_post", (n, width), torch.float32)
            self.post.forward(branch, post)
            hidden += post
            for norm, ffn in ((self.n2, self.ffn), (self.n3, self.extra)):
                norm.forward(hidden, normed)
                ffn.forward(normed, ctx, hidden)

    def rotate(x, pos, pairs_a, pairs_b, inv_freq):
        """x [n, heads, d] in place: (a, b) -> (a c - b s, b c + a s) at each row's position."""
        angle = pos.clamp(min=0).float()[:, None] * inv_freq[None, :]
        c, s_ = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
        live = (pos >= 0)[:, None, None]
        a, b = x[..., pairs_a].float(), x[..., pairs_b].float()
        x[..., pairs_a] = torch.where(live, a * c - b * s_, a).to(x.dtype)
        x[..., pairs_b] = torch.where(live, b * c + a * s_, b).to(x.dtype)

    class PairRope(PositionEncoding):
        """``interleaved``: pairs (2j, 2j + 1) over the whole head; else rotate-half
        pairs over the first ``rotary_dim`` elements only."""
        in_kernel = False

        def __init__(self, params, prefix, dtype, device):
            super().__init__(params, prefix, dtype, device)
            d, r = int(params["head_dim"]), int(params.get("rotary_dim", params["head_dim"]))
            self.inv = (1.0 / torch.pow(torch.tensor(float(params["theta"])),
                                        2 * torch.arange(r // 2).float() / r)).to(device)
            j = torch.arange(r // 2, device=device)
            self.a, self.b = (2 * j, 2 * j + 1) if params.get("interleaved") else (j, j + r // 2)

        def apply(self, qkv, ctx, heads, kv_heads, head_dim):
            n = qkv.shape[0]
            x = qkv[:, :(heads + kv_heads) * head_dim].view(n, heads + kv_heads, head_dim)
            rotate(x, ctx.token_pos[:n], self.a, self.b, self.inv)

    class ScaledEmbedding(TokenEmbedding):
        def forward(self, tokens, hidden, status):
            super().forward(tokens, hidden, status)
            hidden *= float(self.params["scale"])

    class CappedHead(LinearHead):
        """logits = cap * tanh(x W^T / cap); no fused pick."""
        forward_pick = None
        forward_normed = None

        def forward(self, x, logits):
            super().forward(x, logits)
            cap = float(self.params["cap"])
            logits.copy_(cap * torch.tanh(logits / cap))

    BLOCKS.register("toy_sandwich", SandwichBlock)
    POSITIONS.register("toy_pair_rope", PairRope)
    EMBEDDINGS.register("toy_scaled_embedding", ScaledEmbedding)
    HEADS.register("toy_capped_head", CappedHead)


def test_toy_arrangement_positions_embedding_and_head_need_no_change_to_the_framework():
    from nnis_b200.engine import Engine, SequenceStep
    from nnis_b200.engine.model import DecoderModel
    from nnis_b200.weights import random_tensors
    _register_seam_toys()
    H, V, I, nq, nkv, d, eps, theta, scale, cap = 48, 70, 40, 3, 1, 16, 1e-5, 10000.0, 3.0, 2.5
    norm = lambda name: PartSpec("rmsnorm", {"size": H, "eps": eps, "name": name})
    mlp = lambda g, u, dn: PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": I, "activation": "silu",
                                                  "bias": False, "names": {"gate": g, "up": u, "down": dn}})
    pos0 = PartSpec("toy_pair_rope", {"head_dim": d, "theta": theta, "interleaved": True})
    pos1 = PartSpec("toy_pair_rope", {"head_dim": d, "theta": theta, "rotary_dim": d // 2})
    layers = (LayerSpec("l0", "toy_sandwich", {
                  "pre": norm("pre"), "post": norm("post"),
                  "mixer": PartSpec("attention", dict(attention_params(H, nq, nkv, d), position=pos0)),
                  "n2": norm("n2"), "ffn": mlp("g", "u", "d"), "n3": norm("n3"), "extra": mlp("g2", "u2", "d2")}),
              prenorm_layer("l1", norm("n1"),
                            PartSpec("attention", dict(attention_params(H, nq, nkv, d), position=pos1)),
                            norm("n2"), mlp("g", "u", "d")))
    spec = ModelSpec(architecture="ToySeams", hidden_size=H, vocab_size=V, max_positions=512,
                     embedding=PartSpec("toy_scaled_embedding", {"vocab_size": V, "hidden_size": H,
                                                                 "name": "emb", "scale": scale}),
                     layers=layers, schedule=(ScheduleEntry(0), ScheduleEntry(1)), final_norm=norm("final"),
                     head=PartSpec("toy_capped_head", {"vocab_size": V, "hidden_size": H, "name": "head",
                                                       "tied_to": None, "cap": cap}))
    wanted = DecoderModel.weight_specs_of(spec)
    assert {"l0.post.weight", "l0.n3.weight", "l0.d2.weight", "head.weight"} <= set(wanted)
    w = random_tensors(wanted, seed=33, std=1.0, norm_std=0.1, std_by_fan_in=True)

    def plain_rotate(x, interleaved, rotary):
        T = x.shape[0]
        inv = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32), 2 * torch.arange(rotary // 2).float() / rotary)
        ang = (torch.arange(T, dtype=torch.float32)[:, None] * inv[None, :]).double()
        c, s_ = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        out = x.clone()
        j = torch.arange(rotary // 2)
        a, b = (2 * j, 2 * j + 1) if interleaved else (j, j + rotary // 2)
        out[..., a] = x[..., a] * c - x[..., b] * s_
        out[..., b] = x[..., b] * c + x[..., a] * s_
        return out

    def plain(tokens):
        T = len(tokens)
        h = w["emb.weight"].double()[torch.tensor(tokens)] * scale

        def attn(prefix, n, interleaved, rotary):
            q = plain_rotate(P.linear(n, w[prefix + ".q.weight"]).view(T, nq, d), interleaved, rotary)
            k = plain_rotate(P.linear(n, w[prefix + ".k.weight"]).view(T, nkv, d), interleaved, rotary)
            v = P.linear(n, w[prefix + ".v.weight"]).view(T, nkv, d)
            return P.linear(P.causal_attention(q, k, v).reshape(T, nq * d), w[prefix + ".o.weight"])

        def ffn(prefix, n, g, u, dn):
            return P.linear(P.swiglu(P.linear(n, w[f"{prefix}.{g}.weight"]), P.linear(n, w[f"{prefix}.{u}.weight"])),
                            w[f"{prefix}.{dn}.weight"])
        h = h + P.rms_norm(attn("l0", P.rms_norm(h, w["l0.pre.weight"], eps), True, d), w["l0.post.weight"], eps)
        h = h + ffn("l0", P.rms_norm(h, w["l0.n2.weight"], eps), "g", "u", "d")
        h = h + ffn("l0", P.rms_norm(h, w["l0.n3.weight"], eps), "g2", "u2", "d2")
        h = h + attn("l1", P.rms_norm(h, w["l1.n1.weight"], eps), False, d // 2)
        h = h + ffn("l1", P.rms_norm(h, w["l1.n2.weight"], eps), "g", "u", "d")
        return cap * torch.tanh(P.linear(P.rms_norm(h, w["final.weight"], eps), w["head.weight"]) / cap)

    seqs = {"a": [3, 14, 15, 9, 26, 5, 35, 8, 9, 7, 9, 32, 38, 46], "b": [62, 64, 3, 38, 32]}
    want = {k: plain(v) for k, v in seqs.items()}
    for dtype_engine in ("float32",):
        engine = Engine.from_spec(spec, w, dtype=dtype_engine, max_tokens=64 * 8, max_slots=2)
        sa, sb = engine.acquire_slot(), engine.acquire_slot()
        got = engine.step([SequenceStep(sa, seqs["a"][:9], range(9)), SequenceStep(sb, seqs["b"][:3], [2])])
        check_logits(got.cpu().numpy(), torch.cat([want["a"][:9], want["b"][2:3]]), "float32", "seams prompt")
        for t in range(2):
            got = engine.step([SequenceStep(sa, [seqs["a"][9 + t]], [0]), SequenceStep(sb, [seqs["b"][3 + t]], [0])])
            check_logits(got.cpu().numpy(), torch.stack([want["a"][9 + t], want["b"][3 + t]]), "float32",
                         f"seams token {t}")
        engine.release_slot(sb)
        got = engine.step([SequenceStep(sa, seqs["a"][11:], range(3))])
        check_logits(got.cpu().numpy(), want["a"][11:], "float32", "seams tail chunk")
        engine.release_slot(sa)
    # the same model generates through the entry point's loop (no fused pick: the head has none)
    from nnis_b200.engine.api import EngineBackend
    from nnis_b200.engine.generate import GenerationConfig, GenerationRequest, Generator
    gen = Generator(EngineBackend(engine, 2), V, 512, 2, 64 * 8)
    res = gen.generate([GenerationRequest(seqs["a"][:4], GenerationConfig(5))])[0]
    toks = list(seqs["a"][:4])
    for _ in range(5):
        toks.append(P.argmax_lowest(plain(toks)[-1]))
    assert res.ok and res.token_ids == toks[4:]


# ---------------------------------------------------------------------------
# A norm shared out between the projections on either side of it (decode steps)
# ---------------------------------------------------------------------------
def test_norms_are_shared_between_projections_where_both_sides_take_them(tmp_path, monkeypatch):
    """Three layers: in a decode step every norm but the first and the last is begun by the
    projection before it (five of them), the logits match the plain implementation as they
    do with the norms run whole, and a mixer that knows nothing of it is left alone."""
    from helpers import TINY_B, load_plain_weights, make_model, read_config_json
    from nnis_b200 import LLM
    from nnis_b200.csrc import ops
    d = make_model(str(tmp_path), TINY_B, seed=77)
    cfg, w = read_config_json(d), load_plain_weights(d, as_bf16=True)
    ids = [5, 9, 1, 200, 33, 17, 4, 4, 250, 3, 99]
    want = P.forward(cfg, w, ids, True)
    seen = {"emit": 0, "shares": 0}
    real = ops.gemv_bf16

    def counting(*args, **kwargs):
        seen["emit"] += kwargs.get("emit") is not None
        seen["shares"] += kwargs.get("shares") is not None
        return real(*args, **kwargs)

    monkeypatch.setattr(ops, "gemv_bf16", counting)
    got = {}
    for shared in (3, 0):
        monkeypatch.setattr(ops, "SHARED_NORM", shared)
        seen.update(emit=0, shares=0)
        llm = LLM(d, dtype="bfloat16", max_tokens=64 * 4, max_batch=2)
        session = llm.new_session()
        rows = [session.prefill(ids[:6])]
        assert seen == {"emit": 0, "shares": 0}  # a prompt step shares nothing
        rows += [session.decode_one(t) for t in ids[6:]]
        steps = len(ids) - 6
        layers = cfg["num_hidden_layers"]
        assert seen == ({"emit": steps * (2 * layers - 1), "shares": steps * (2 * layers - 1)} if shared
                        else {"emit": 0, "shares": 0})
        got[shared] = np.stack(rows)
        check_logits(got[shared], want[5:], "bfloat16", f"shared norms {shared}")
        session.close()
    # the two ways differ by roundings only
    assert np.abs(got[3] - got[0]).max() <= 0.03 * max(1.0, float(np.abs(got[0]).max()))


# ---------------------------------------------------------------------------
# A toy norm (mean and variance, weight and bias), registered from here: the parts around
# it may fold or share an RMSNorm but must leave any other norm to itself.
# ---------------------------------------------------------------------------
def _register_toy_norm():
    from nnis_b200.parts import NORMS
    from nnis_b200.parts.base import Part
    from nnis_b200.weights.loader import WeightSpec

    class CenteredNorm(Part):
        kind = "toy_centered_norm"

        def __init__(self, params, prefix, dtype, device):
            super().__init__(params, prefix, dtype, device)
            self.size, self.eps = int(params["size"]), float(params["eps"])
            self.stem = params["name"]
            self.weight = self.bias = None

        def weight_specs(self):
            return {self.tensor_name(self.stem): WeightSpec((self.size,), "vector", init="ones"),
                    self.tensor_name(self.stem, "bias"): WeightSpec((self.size,), "vector")}

        def load(self, tensors):
            self.weight = tensors[self.tensor_name(self.stem)]
            self.bias = tensors[self.tensor_name(self.stem, "bias")]

        def forward(self, x, out, rows=None):
            x = x if rows is None else x[rows.long()]
            centered = x - x.mean(-1, keepdim=True)
            out.copy_(centered / torch.sqrt(centered.square().mean(-1, keepdim=True) + self.eps)
                      * self.weight + self.bias)

    NORMS.register("toy_centered_norm", CenteredNorm)


@pytest.mark.parametrize("dtype", list(DT))
def test_a_toy_norm_runs_beside_norms_that_are_folded_and_shared(dtype, monkeypatch):
    """Layer 0 has the toy norm twice, layer 1 RMSNorms.  In a bfloat16 decode step the toy
    norms run as they are (no projection folds or shares them), the first RMSNorm of layer 1 is
    begun by layer 0's down projection and the second by layer 1's O projection: two norms
    change hands a step.  Prompts of unequal length, then single tokens, against the plain
    functions."""
    from nnis_b200.csrc import ops
    from nnis_b200.engine import Engine, SequenceStep
    from nnis_b200.engine.model import DecoderModel
    from nnis_b200.weights import random_tensors
    _register_toy_norm()
    H, V, I, nq, nkv, d, eps = 64, 96, 112, 4, 2, 16, 1e-5
    rms = lambda name: PartSpec("rmsnorm", {"size": H, "eps": eps, "name": name})
    toy = lambda name: PartSpec("toy_centered_norm", {"size": H, "eps": eps, "name": name})
    names = {"q": "self_attn.q_proj", "k": "self_attn.k_proj", "v": "self_attn.v_proj", "o": "self_attn.o_proj"}
    attn = PartSpec("attention", dict(attention_params(H, nq, nkv, d), names=names))
    mlp = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": I, "activation": "silu", "bias": False,
                                 "names": {"gate": "mlp.gate_proj", "up": "mlp.up_proj", "down": "mlp.down_proj"}})
    layers = (prenorm_layer("l0", toy("n1"), attn, toy("n2"), mlp),
              prenorm_layer("l1", rms("n1"), attn, rms("n2"), mlp))
    spec = ModelSpec(architecture="ToyNorm", hidden_size=H, vocab_size=V, max_positions=512,
                     embedding=PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H, "name": "emb"}),
                     layers=layers, schedule=(ScheduleEntry(0), ScheduleEntry(1)), final_norm=rms("final"),
                     head=PartSpec("linear_head", {"vocab_size": V, "hidden_size": H, "name": "head",
                                                   "tied_to": "emb"}))
    wanted = DecoderModel.weight_specs_of(spec)
    assert "l0.n1.bias" in wanted and "l1.n1.bias" not in wanted
    w = random_tensors(wanted, seed=31, std=1.0, norm_std=0.1, std_by_fan_in=True)
    bf = dtype == "bfloat16"
    engine = Engine.from_spec(spec, w, dtype=dtype, max_tokens=64 * 8, max_slots=2)
    pw = {k: (v.bfloat16().double() if bf and v.dim() == 2 else v.double()) for k, v in w.items()}
    cfg = {"hidden_size": H, "num_attention_heads": nq, "num_key_value_heads": nkv, "head_dim": d}
    cos, sin = P.rope_tables(512, d, 10000.0)

    def plain(tokens):
        h = pw["emb.weight"][torch.tensor(tokens)]
        for prefix in ("l0", "l1"):
            for norm_name, part in (("n1", "attention"), ("n2", "mlp")):
                if prefix == "l0":
                    c = h - h.mean(-1, keepdim=True)
                    n = c / torch.sqrt(c.square().mean(-1, keepdim=True) + eps)
                    n = n * pw[f"l0.{norm_name}.weight"] + pw[f"l0.{norm_name}.bias"]
                else:
                    n = P.rms_norm(h, pw[f"l1.{norm_name}.weight"], eps)
                n = P._round(n, bf)
                if part == "attention":
                    h = h + P.attention_layer(cfg, pw, prefix + ".self_attn.", n, cos, sin, bf)
                else:
                    h = h + P.mlp_layer(cfg, pw, prefix + ".mlp.", n, bf)
        return P.linear(P._round(P.rms_norm(h, pw["final.weight"], eps), bf), pw["emb.weight"])

    seen = {"emit": 0, "shares": 0}
    real = ops.gemv_bf16

    def counting(*args, **kwargs):
        seen["emit"] += kwargs.get("emit") is not None
        seen["shares"] += kwargs.get("shares") is not None
        return real(*args, **kwargs)

    monkeypatch.setattr(ops, "gemv_bf16", counting)
    g = torch.Generator().manual_seed(3)
    seqs = {"a": torch.randint(0, V, (30,), generator=g).tolist(), "b": torch.randint(0, V, (11,), generator=g).tolist()}
    want = {k: plain(v) for k, v in seqs.items()}
    sa, sb = engine.acquire_slot(), engine.acquire_slot()
    got = engine.step([SequenceStep(sa, seqs["a"][:25], [0, 24]), SequenceStep(sb, seqs["b"][:6], [5])])
    check_logits(got.cpu().numpy(), torch.stack([want["a"][0], want["a"][24], want["b"][5]]), dtype, "toy norm prompt")
    assert seen == {"emit": 0, "shares": 0}
    for t in range(5):
        got = engine.step([SequenceStep(sa, [seqs["a"][25 + t]], [0]), SequenceStep(sb, [seqs["b"][6 + t]], [0])])
        check_logits(got.cpu().numpy(), torch.stack([want["a"][25 + t], want["b"][6 + t]]), dtype,
                     f"toy norm token {t}")
    assert seen == ({"emit": 10, "shares": 10} if bf else {"emit": 0, "shares": 0})
    engine.release_slot(sa)
    engine.release_slot(sb)
