"""Generality of the parts, shown with toy parts that exist only in this test: a mixer
with a fixed-size state of its own, a model whose layers differ (window attention, the
stateful mixer, full attention), a schedule that names a layer twice and lets a run
read the cache another run wrote; and a second toy model with a routed feed-forward and a
position encoding of another formula.  Everything is registered, built and stepped through
the framework's public interfaces, with no change to its files, and compared with a
plain whole-sequence computation written here."""
from dataclasses import asdict, dataclass

import numpy as np
import pytest
import torch

import plain_qwen3 as P
import replay_util as ru

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


# ----------------------------------------------------------------- the toy mixer
def _make_ema_mixer(on_device: bool = False):
    from zinfer_b200.parts import Mixer, StateNeed, TensorSpec

    class EmaMixer(Mixer):
        """s_t = decay * s_{t-1} + W_in x_t ; y_t = W_out s_t.  Its only memory is s, one
        vector per request, kept in the cache manager's per-request state slots.
        ``on_device``: steps in which every request brings one token touch the state with device
        operations alone (gather by ``state_slots``, update, scatter), so they can be captured."""

        graph_safe = on_device

        def __init__(self, params, ctx):
            super().__init__(params, ctx)
            self.hidden = int(params["hidden_size"])
            self.decay = float(params["decay"])

        def tensor_specs(self):
            return {"in_proj.weight": TensorSpec((self.hidden, self.hidden)),
                    "out_proj.weight": TensorSpec((self.hidden, self.hidden))}

        def bind(self, tensors):
            self.w_in = tensors["in_proj.weight"].float()
            self.w_out = tensors["out_proj.weight"].float()

        def cache_need(self):
            return StateNeed((self.hidden,), torch.float32)

        def forward(self, x, step, cache):
            u = x.float() @ self.w_in.T
            if on_device and step.n_pf_tiles == 0 and step.n_dec == step.n_seqs:
                slots = step.state_slots.long()              # rows that pad a captured batch name the spare slot
                s = self.decay * cache.state.index_select(0, slots) + u
                cache.state.index_copy_(0, slots, s)
                return (s @ self.w_out.T).to(x.dtype)
            y = torch.empty_like(u)
            slots = step.state_slots.tolist()
            start = 0
            for i, n in enumerate(step.q_lens):        # a request's tokens are scanned in order
                s = cache.state[slots[i]]
                for t in range(start, start + n):
                    s = self.decay * s + u[t]
                    y[t] = s
                cache.state[slots[i]] = s
                start += n
            return (y @ self.w_out.T).to(x.dtype)

    return EmaMixer


@dataclass(frozen=True)
class ToyConfig:
    vocab_size: int = 211
    hidden_size: int = 80
    intermediate_size: int = 112
    num_heads: int = 5
    num_kv_heads: int = 1
    head_dim: int = 32
    window: int = 9
    decay: float = 0.7
    eps: float = 2e-6
    theta: float = 3000.0
    max_positions: int = 256
    model_type: str = "toy_hybrid"

    @classmethod
    def from_dict(cls, d):
        return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})

    def to_dict(self):
        return {**asdict(self), "architectures": ["ToyHybridForCausalLM"]}


def toy_model_spec(cfg: ToyConfig):
    from zinfer_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

    norm = PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.eps})
    rope = PartSpec("rope", {"head_dim": cfg.head_dim, "theta": cfg.theta, "max_positions": cfg.max_positions})
    ffn = PartSpec("swiglu_mlp", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size})

    def attn(window, qk_norm):
        return PartSpec("gqa_attention", {"hidden_size": cfg.hidden_size, "num_heads": cfg.num_heads,
                                          "num_kv_heads": cfg.num_kv_heads, "head_dim": cfg.head_dim,
                                          "qk_norm_eps": cfg.eps if qk_norm else None, "window": window, "position": rope})

    def block(mixer):
        return PartSpec("prenorm_block", {"mixer": mixer, "mixer_norm": norm, "feed_forward": ffn, "ffn_norm": norm})

    mixers = [attn(cfg.window, True), PartSpec("toy_ema_mixer", {"hidden_size": cfg.hidden_size, "decay": cfg.decay}),
              attn(None, False)]
    layers = tuple(LayerSpec(block(m), prefix=f"layers.{i}.") for i, m in enumerate(mixers))
    # layer 1 runs twice (each run with a state of its own); the last run of layer 2 reads the keys
    # and values that its first run wrote
    schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2, cache="shared"), ScheduleEntry(1),
                ScheduleEntry(2, cache="shared"))
    return ModelSpec(
        architecture="ToyHybridForCausalLM", vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
        max_positions=cfg.max_positions,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size, "name": "embed"}),
        layers=layers, schedule=schedule, final_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.eps, "name": "norm"}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size, "name": "head", "tied_to": None}))


# -------------------------------------------------------- the plain computation
def plain_toy_forward(cfg: ToyConfig, w, tokens):
    S = len(tokens)
    cos, sin = P.rope_tables(S, cfg.head_dim, cfg.theta)
    h = w["embed.weight"][torch.as_tensor(tokens)]
    shared_kv = {}

    def attention_layer(x, i, window, qk_norm, reuse):
        p = f"layers.{i}.mixer."
        q = (x @ w[p + "q_proj.weight"].T).reshape(S, cfg.num_heads, cfg.head_dim)
        if qk_norm:
            q = P.rmsnorm(q, w[p + "q_norm.weight"], cfg.eps)
        q = P.apply_rope(q, cos, sin)
        if reuse and "kv" in shared_kv:
            k, v = shared_kv["kv"]
        else:
            k = (x @ w[p + "k_proj.weight"].T).reshape(S, cfg.num_kv_heads, cfg.head_dim)
            v = (x @ w[p + "v_proj.weight"].T).reshape(S, cfg.num_kv_heads, cfg.head_dim)
            if qk_norm:
                k = P.rmsnorm(k, w[p + "k_norm.weight"], cfg.eps)
            k = P.apply_rope(k, cos, sin)
            if reuse:
                shared_kv["kv"] = (k, v)
        o = P.attention(q, k, v, window=window).reshape(S, -1)
        return o @ w[p + "o_proj.weight"].T

    def ema_layer(x, i):
        p = f"layers.{i}.mixer."
        u = x @ w[p + "in_proj.weight"].T
        s = torch.zeros(cfg.hidden_size, dtype=F64)
        ys = []
        for t in range(S):
            s = cfg.decay * s + u[t]
            ys.append(s)
        return torch.stack(ys) @ w[p + "out_proj.weight"].T

    def run(h, i):
        p = f"layers.{i}."
        x = P.rmsnorm(h, w[p + "mixer_norm.weight"], cfg.eps)
        if i == 0:
            a = attention_layer(x, 0, cfg.window, True, False)
        elif i == 1:
            a = ema_layer(x, 1)
        else:
            a = attention_layer(x, 2, None, False, True)
        h = h + a
        x = P.rmsnorm(h, w[p + "ffn_norm.weight"], cfg.eps)
        g = x @ w[p + "feed_forward.gate_proj.weight"].T
        u = x @ w[p + "feed_forward.up_proj.weight"].T
        return h + P.swiglu(g, u) @ w[p + "feed_forward.down_proj.weight"].T

    for i in (0, 1, 2, 1, 2):
        h = run(h, i)
    return (P.rmsnorm(h, w["norm.weight"], cfg.eps) @ w["head.weight"].T).numpy()


@pytest.fixture
def toy_registered():
    from zinfer_b200.config import Family, register_family, unregister_family
    from zinfer_b200.parts import register_part, unregister_part

    register_part("toy_ema_mixer", _make_ema_mixer())
    register_family(Family("ToyHybridForCausalLM", "toy_hybrid", ToyConfig, toy_model_spec))
    yield
    unregister_family("ToyHybridForCausalLM")
    unregister_part("toy_ema_mixer")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_hybrid_model_is_built_and_stepped(toy_registered, dtype):
    from zinfer_b200.config import family_for
    from zinfer_b200.engine import DecoderModel, ModelRunner
    from zinfer_b200.weights import random_tensors

    cfg = ToyConfig()
    fam = family_for(cfg.to_dict())                       # found through the one registry
    assert fam.name == "ToyHybridForCausalLM"
    model = DecoderModel(fam.model_spec(cfg), dtype, DEV)
    tensors = random_tensors(model.tensor_specs(), 77, dtype, DEV)
    model.bind(tensors)
    kv, state = model.cache_needs()
    assert set(state) == {"run1", "run3"} and set(kv) == {"run0", "shared"}   # two states, two key caches
    runner = ModelRunner(model, page_size=4, max_tokens=192, max_requests=3)
    assert runner.graphs is None                           # a mixer that loops on the host is not captured
    assert len(runner.manager.groups) == 2                 # windowed and full caches have pages of their own

    w = {k: v.detach().cpu().to(F64) for k, v in tensors.items()}
    reqs = ru.make_requests(cfg.vocab_size, [41, 7, 64, 30], seed=5)
    plain = {rid: plain_toy_forward(cfg, w, toks) for rid, toks in reqs.items()}
    tol = dict(rtol=5e-5, atol=1e-6) if dtype == torch.float32 else dict(rtol=3e-2, atol=1e-3)
    for mode, trace in (("whole", ru.trace_whole(reqs)), ("tail", ru.trace_tail_decode(reqs, 20)),
                        ("portions", ru.trace_portions(reqs, 4)), ("mixed", ru.trace_mixed(reqs, 9, max_live=3))):
        got = ru.run_in_process(runner, trace)
        ru.assert_close(got, plain, what=f"toy/{mode}", argmax_frac=0.0, **tol)
        assert not runner.manager.requests
    # the window gave pages back while requests were still running
    runner.add_request("w")
    from zinfer_b200.engine import StepEntry
    runner.step([StepEntry("w", reqs["r2"][:40], [])])
    windowed = next(i for i, g in enumerate(runner.manager.groups) if g.window is not None)
    table = runner.manager.block_table("w", windowed)
    assert table[:7] == [-1] * 7 and all(p >= 0 for p in table[8:])
    runner.end_request("w")
    runner.manager.check()


@pytest.fixture
def toy_on_device_registered():
    from zinfer_b200.config import Family, register_family, unregister_family
    from zinfer_b200.parts import register_part, unregister_part

    register_part("toy_ema_mixer", _make_ema_mixer(on_device=True))
    register_family(Family("ToyHybridForCausalLM", "toy_hybrid", ToyConfig, toy_model_spec))
    yield
    unregister_family("ToyHybridForCausalLM")
    unregister_part("toy_ema_mixer")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_mixer_with_state_decodes_from_a_graph(toy_on_device_registered, dtype):
    """The same toy model with a mixer whose decode steps use device operations only: the runner
    captures them, three live requests fill a bucket of four (the row that pads it names the spare
    state slot, so nobody's state is touched), and the logits are the plain model's."""
    from zinfer_b200.config import family_for
    from zinfer_b200.engine import DecoderModel, ModelRunner
    from zinfer_b200.weights import random_tensors

    cfg = ToyConfig()
    model = DecoderModel(family_for(cfg.to_dict()).model_spec(cfg), dtype, DEV)
    tensors = random_tensors(model.tensor_specs(), 77, dtype, DEV)
    model.bind(tensors)
    runner = ModelRunner(model, page_size=4, max_tokens=192, max_requests=3)
    assert runner.graphs is not None
    w = {k: v.detach().cpu().to(F64) for k, v in tensors.items()}
    reqs = ru.make_requests(cfg.vocab_size, [41, 30, 52], seed=8)
    plain = {rid: plain_toy_forward(cfg, w, toks) for rid, toks in reqs.items()}
    tol = dict(rtol=5e-5, atol=1e-6) if dtype == torch.float32 else dict(rtol=3e-2, atol=1e-3)
    # prompts without their last 16 tokens in one step, then 16 steps of one token for all three together
    ids = list(reqs)
    trace = [{"step": 0, "end": [], "entries": [{"id": r, "tokens": reqs[r][:-16], "want": []} for r in ids]}]
    for k in range(16, 0, -1):
        trace.append({"step": len(trace), "end": ids if k == 1 else [],
                      "entries": [{"id": r, "tokens": reqs[r][len(reqs[r]) - k:len(reqs[r]) - k + 1], "want": [0]} for r in ids]})
    got = ru.run_in_process(runner, trace)
    assert runner.graphs.replays >= 10 and len(got) == 3 * 16
    ru.assert_close(got, plain, what="toy/graph", argmax_frac=0.0, **tol)
    for name, t in runner.storage.state.items():
        assert t.shape[0] == 4, "three request slots and the spare one"
    runner.manager.check()


# ---------------------------------------------- a routed feed-forward and another position encoding
def _make_routed_ffn():
    from zinfer_b200.parts import FeedForward, TensorSpec

    class RoutedFFN(FeedForward):
        """Top-2 of E experts per token: router logits and the softmax over the two chosen in 32-bit,
        each expert down(relu(up x)^2).  Written densely (every expert on every token, times a gate
        that is zero for the others), which is fine for a toy and needs no host-side loop."""

        def __init__(self, params, ctx):
            super().__init__(params, ctx)
            self.hidden, self.inter, self.experts = (int(params[k]) for k in ("hidden_size", "intermediate_size", "experts"))

        def tensor_specs(self):
            return {"router.weight": TensorSpec((self.experts, self.hidden)),
                    "experts.up": TensorSpec((self.experts, self.inter, self.hidden)),
                    "experts.down": TensorSpec((self.experts, self.hidden, self.inter))}

        def bind(self, tensors):
            self.router = tensors["router.weight"].float() * 40.0     # spread the logits: clear choices
            self.up, self.down = tensors["experts.up"].float(), tensors["experts.down"].float()

        def forward(self, x):
            xf = x.float()
            logits = xf @ self.router.T
            top, idx = torch.topk(logits, 2, dim=-1)
            gate = torch.zeros_like(logits).scatter_(1, idx, torch.softmax(top, dim=-1))
            mid = torch.relu(torch.einsum("th,eih->tei", xf, self.up)) ** 2
            return torch.einsum("tei,ehi,te->th", mid, self.down, gate).to(x.dtype)

    return RoutedFFN


def _make_scaled_rotary():
    from zinfer_b200.parts import PositionEncoding

    class ScaledRotary(PositionEncoding):
        """Rotary angles of position / factor with a phase per frequency: another position encoding
        that the attention's kernels take, because all they ask for is ``tables()``."""

        def __init__(self, params, ctx):
            super().__init__(params, ctx)
            self.d, self.theta, self.factor = int(params["head_dim"]), float(params["theta"]), float(params["factor"])
            self.n_positions = min(int(params["max_positions"]), ctx.max_positions)
            self._tables = None

        def tables(self):
            if self._tables is None:
                ang = scaled_rotary_angles(self.n_positions, self.d, self.theta, self.factor)
                self._tables = (torch.cos(ang).float().to(self.ctx.device), torch.sin(ang).float().to(self.ctx.device))
            return self._tables

    return ScaledRotary


def scaled_rotary_angles(n, d, theta, factor):
    i = torch.arange(d // 2, dtype=F64)
    inv = theta ** (-2.0 * i / d)
    pos = torch.arange(n, dtype=F64) / factor
    return pos[:, None] * inv[None, :] + 0.1 * i[None, :]


@dataclass(frozen=True)
class RoutedConfig:
    vocab_size: int = 173
    hidden_size: int = 96
    intermediate_size: int = 48
    dense_intermediate_size: int = 144
    experts: int = 5
    num_heads: int = 4
    num_kv_heads: int = 2
    head_dim: int = 48
    eps: float = 1e-5
    theta: float = 700.0
    factor: float = 2.5
    max_positions: int = 256
    model_type: str = "toy_routed"

    @classmethod
    def from_dict(cls, d):
        return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})

    def to_dict(self):
        return {**asdict(self), "architectures": ["ToyRoutedForCausalLM"]}


def routed_model_spec(cfg: RoutedConfig):
    from zinfer_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

    H = cfg.hidden_size
    norm = PartSpec("rmsnorm", {"size": H, "eps": cfg.eps})
    positions = [PartSpec("toy_scaled_rotary", {"head_dim": cfg.head_dim, "theta": cfg.theta, "factor": cfg.factor,
                                                "max_positions": cfg.max_positions}),
                 None,
                 PartSpec("rope", {"head_dim": cfg.head_dim, "theta": cfg.theta, "max_positions": cfg.max_positions})]
    routed = PartSpec("toy_routed_ffn", {"hidden_size": H, "intermediate_size": cfg.intermediate_size, "experts": cfg.experts})
    dense = PartSpec("swiglu_mlp", {"hidden_size": H, "intermediate_size": cfg.dense_intermediate_size})

    def block(position, ffn):
        mixer = PartSpec("gqa_attention", {"hidden_size": H, "num_heads": cfg.num_heads, "num_kv_heads": cfg.num_kv_heads,
                                           "head_dim": cfg.head_dim, "qk_norm_eps": cfg.eps, "window": None,
                                           "position": position})
        return PartSpec("prenorm_block", {"mixer": mixer, "mixer_norm": norm, "feed_forward": ffn, "ffn_norm": norm})

    layers = tuple(LayerSpec(block(p, f), prefix=f"layers.{i}.") for i, (p, f) in enumerate(zip(positions, (routed, dense, routed))))
    return ModelSpec(
        architecture="ToyRoutedForCausalLM", vocab_size=cfg.vocab_size, hidden_size=H, max_positions=cfg.max_positions,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": H, "name": "embed"}),
        layers=layers, schedule=tuple(ScheduleEntry(i) for i in range(3)),
        final_norm=PartSpec("rmsnorm", {"size": H, "eps": cfg.eps, "name": "norm"}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": H, "name": "head", "tied_to": None}))


def plain_routed_forward(cfg: RoutedConfig, w, tokens):
    """Logits [S, V] and, per position, the smallest gap between the second and the third router
    logit in any layer (how safely its experts were chosen)."""
    S = len(tokens)
    ang = scaled_rotary_angles(S, cfg.head_dim, cfg.theta, cfg.factor)
    tables = [(torch.cos(ang), torch.sin(ang)), None, P.rope_tables(S, cfg.head_dim, cfg.theta)]
    h = w["embed.weight"][torch.as_tensor(tokens)]
    margin = torch.full((S,), float("inf"), dtype=F64)
    for i in range(3):
        p = f"layers.{i}."
        x = P.rmsnorm(h, w[p + "mixer_norm.weight"], cfg.eps)
        q = P.rmsnorm((x @ w[p + "mixer.q_proj.weight"].T).reshape(S, cfg.num_heads, cfg.head_dim), w[p + "mixer.q_norm.weight"], cfg.eps)
        k = P.rmsnorm((x @ w[p + "mixer.k_proj.weight"].T).reshape(S, cfg.num_kv_heads, cfg.head_dim), w[p + "mixer.k_norm.weight"], cfg.eps)
        v = (x @ w[p + "mixer.v_proj.weight"].T).reshape(S, cfg.num_kv_heads, cfg.head_dim)
        if tables[i] is not None:
            q, k = P.apply_rope(q, *tables[i]), P.apply_rope(k, *tables[i])
        h = h + P.attention(q, k, v).reshape(S, -1) @ w[p + "mixer.o_proj.weight"].T
        x = P.rmsnorm(h, w[p + "ffn_norm.weight"], cfg.eps)
        if i == 1:
            f = P.swiglu(x @ w[p + "feed_forward.gate_proj.weight"].T, x @ w[p + "feed_forward.up_proj.weight"].T) \
                @ w[p + "feed_forward.down_proj.weight"].T
        else:
            logits = x @ (w[p + "feed_forward.router.weight"] * 40.0).T
            top, idx = torch.topk(logits, 3, dim=-1)
            margin = torch.minimum(margin, top[:, 1] - top[:, 2])
            share = torch.softmax(top[:, :2], dim=-1)
            f = torch.zeros_like(h)
            for t in range(S):
                for j in range(2):
                    e = int(idx[t, j])
                    mid = torch.relu(w[p + "feed_forward.experts.up"][e] @ x[t]) ** 2
                    f[t] += share[t, j] * (w[p + "feed_forward.experts.down"][e] @ mid)
        h = h + f
    return (P.rmsnorm(h, w["norm.weight"], cfg.eps) @ w["head.weight"].T).numpy(), margin.numpy()


@pytest.fixture
def routed_registered():
    from zinfer_b200.config import Family, register_family, unregister_family
    from zinfer_b200.parts import register_part, unregister_part

    register_part("toy_routed_ffn", _make_routed_ffn())
    register_part("toy_scaled_rotary", _make_scaled_rotary())
    register_family(Family("ToyRoutedForCausalLM", "toy_routed", RoutedConfig, routed_model_spec))
    yield
    unregister_family("ToyRoutedForCausalLM")
    unregister_part("toy_scaled_rotary")
    unregister_part("toy_routed_ffn")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_routed_model_with_another_position_encoding(routed_registered, dtype):
    """A feed-forward with routing and a position encoding of another formula, both defined here,
    beside layers without positions and with the dense feed-forward.  A token whose second and third
    router logits lie closer than bfloat16 can tell apart might choose other experts than the plain
    computation does, which would be no fault; so the requests are made token by token from random
    candidates whose choice of experts is clear (a gap of 0.5 between logits that spread over 8)."""
    import random

    from zinfer_b200.config import family_for
    from zinfer_b200.engine import DecoderModel, ModelRunner
    from zinfer_b200.weights import random_tensors

    cfg = RoutedConfig()
    fam = family_for(cfg.to_dict())
    model = DecoderModel(fam.model_spec(cfg), dtype, DEV)
    tensors = random_tensors(model.tensor_specs(), 123, dtype, DEV)
    model.bind(tensors)
    runner = ModelRunner(model, page_size=8, max_tokens=320, max_requests=4)
    assert runner.graphs is not None          # attention everywhere: decode steps are replayed from graphs

    w = {k: v.detach().cpu().to(F64) for k, v in tensors.items()}
    rng = random.Random(11)
    reqs = {}
    for r, n in enumerate((37, 9, 58, 26)):
        toks = []
        for _ in range(n):
            for _ in range(100):
                cand = rng.randrange(cfg.vocab_size)
                if plain_routed_forward(cfg, w, toks + [cand])[1][-1] >= 0.5:
                    toks.append(cand)
                    break
            else:
                raise AssertionError("no candidate token with a clear choice of experts")
        reqs[f"r{r}"] = toks
    plain = {}
    for rid, toks in reqs.items():
        plain[rid], margin = plain_routed_forward(cfg, w, toks)
        assert margin.min() >= 0.5
    tol = dict(rtol=5e-5, atol=1e-6) if dtype == torch.float32 else dict(rtol=3e-2, atol=1e-3)
    for mode, trace in (("whole", ru.trace_whole(reqs)), ("tail", ru.trace_tail_decode(reqs, 20)),
                        ("portions", ru.trace_portions(reqs, 5)), ("mixed", ru.trace_mixed(reqs, 11, max_live=3))):
        got = ru.run_in_process(runner, trace)
        ru.assert_close(got, plain, what=f"routed/{mode}", argmax_frac=0.0, **tol)
        assert not runner.manager.requests
    runner.manager.check()
