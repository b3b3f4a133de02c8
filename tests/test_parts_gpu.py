"""Each part alone against its plain function, and toy parts defined here (a
mixer with state of its own, a feed-forward that routes tokens to experts, another
position encoding), registered, built and stepped without touching the
framework's files."""
import math

import pytest
import torch

import plain_llama as P
from helpers import check_logits
from nnis_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


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
    layers = tuple(LayerSpec(
        prefix=f"blocks.{i}", block="prenorm", mixer_norm=norm("n1"),
        mixer=PartSpec("toy_running_mean", {"width": H}), ffn_norm=norm("n2"),
        ffn=PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": I, "activation": "silu",
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
    layers = (LayerSpec("l0", "prenorm", norm("n1"), PartSpec("attention", attention_params(H, nq, nkv, d)),
                        norm("n2"), ffn),
              LayerSpec("l1", "prenorm", norm("n1"),
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
    layers = (LayerSpec("l0", "prenorm", norm("n1"), PartSpec("attention", attn0), norm("n2"),
                        PartSpec("toy_top1_experts", {"hidden_size": H, "expert_size": I, "experts": E})),
              LayerSpec("l1", "prenorm", norm("n1"), PartSpec("attention", attention_params(H, nq, nkv, d)),
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
