"""The kernel that runs whole layers of a decode step in one launch (ops.decode_layers):
against the plain model through the engine, against the chain of kernels it replaces at
every token padding (16, 32, 64 columns), with a sliding window and two cache groups, and in
a model where only some layers are of the kinds it knows (the others go through their parts)."""
import random

import pytest
import torch

import plain_qwen3
import replay_util as ru

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = dict(rtol=3e-2, atol=1e-3)   # bfloat16, as in the replay tests


@pytest.fixture
def whole_layers(monkeypatch):
    """Switches the kernel on for runners built inside the test and counts its launches."""
    from zinfer_b200 import ops

    calls = {"n": 0}
    real = ops.decode_layers

    def counted(*a, **k):
        calls["n"] += 1
        return real(*a, **k)

    monkeypatch.setattr(ops, "DECODE_LAYERS", True)
    monkeypatch.setattr(ops, "decode_layers", counted)
    return calls


def _runner(model_dir, name, fused, **kw):
    from conftest import PAGE_SIZE
    from zinfer_b200 import ops
    from zinfer_b200.engine import ModelRunner

    before = ops.DECODE_LAYERS
    ops.DECODE_LAYERS = fused
    try:
        return ModelRunner.from_model_dir(model_dir, dtype=torch.bfloat16, device=DEV, page_size=PAGE_SIZE[name], **kw)
    finally:
        ops.DECODE_LAYERS = before


@pytest.mark.parametrize("name", ["D", "E"])
def test_whole_layer_kernel_against_the_plain_model(model_dirs, whole_layers, name):
    from zinfer_b200 import ops

    model_dir = model_dirs[(name, "bfloat16")]
    cfg, w = plain_qwen3.load_model(model_dir)
    reqs = ru.make_requests(cfg["vocab_size"], [70, 33, 129, 48], seed=31)
    plain = ru.plain_logits(cfg, w, reqs)
    for mode, trace in (("tail", ru.trace_tail_decode(reqs, 40)), ("mixed", ru.trace_mixed(reqs, 17, tail=30))):
        runner = _runner(model_dir, name, True, max_tokens=ru.max_live_tokens(trace), max_requests=4)
        assert any(p is not None for _, _, p in runner.model._spans), "the model's layers were not prepared for the kernel"
        before = whole_layers["n"]
        got = ru.run_in_process(runner, trace)
        assert whole_layers["n"] > before, "no decode step went through the kernel"
        ru.assert_close(got, plain, what=f"{name}/{mode}", argmax_frac=0.0, **TOL)
        assert ops.kernel_status() == 0


@pytest.mark.parametrize("name,batch", [("D", 1), ("D", 7), ("D", 24), ("E", 3), ("E", 40), ("E", 64)])
def test_whole_layer_kernel_equals_the_chain_of_kernels(model_dirs, whole_layers, name, batch):
    """The same decode steps through both paths: logits agree to bfloat16 rounding, and the
    caches they leave give the same continuation."""
    from zinfer_b200 import ops
    from zinfer_b200.engine import StepEntry

    model_dir = model_dirs[(name, "bfloat16")]
    cfg, _ = plain_qwen3.load_model(model_dir)
    outs = []
    for fused in (False, True):
        runner = _runner(model_dir, name, fused, max_tokens=batch * 192 + 256, max_requests=64)
        rng = random.Random(9)
        ids = [f"q{i}" for i in range(batch)]
        for i, rid in enumerate(ids):
            runner.add_request(rid)
            n = 1 + (i * 37 + 11) % 120
            runner.step([StepEntry(rid, [rng.randrange(cfg["vocab_size"]) for _ in range(n)], [])])
        rows = []
        for _ in range(10):
            toks = [rng.randrange(cfg["vocab_size"]) for _ in ids]
            rows.append(runner.step([StepEntry(r, [t], [0]) for r, t in zip(ids, toks)]).float().cpu())
        outs.append(torch.stack(rows))
        assert ops.kernel_status() == 0
    assert whole_layers["n"] >= 2   # the first step and the capture; the other steps replay the graph
    chain, whole = outs
    assert torch.isfinite(whole).all()
    scale = chain.abs().amax(dim=-1, keepdim=True)
    assert ((whole - chain).abs() <= 2e-2 * scale + 1e-3).all(), \
        f"largest difference {(whole - chain).abs().max().item():.4g} of {scale.max().item():.3g}"


def _make_relu_ffn():
    from zinfer_b200.parts import FeedForward, TensorSpec

    class ReluFFN(FeedForward):
        """down(relu(up(x))): a feed-forward the whole-layer kernel does not know."""

        def __init__(self, params, ctx):
            super().__init__(params, ctx)
            self.hidden, self.inter = int(params["hidden_size"]), int(params["intermediate_size"])

        def tensor_specs(self):
            return {"up.weight": TensorSpec((self.inter, self.hidden)), "down.weight": TensorSpec((self.hidden, self.inter))}

        def bind(self, tensors):
            self.up, self.down = tensors["up.weight"].float(), tensors["down.weight"].float()

        def forward(self, x):
            return (torch.relu(x.float() @ self.up.T) @ self.down.T).to(x.dtype)

    return ReluFFN


def test_layers_of_other_kinds_go_through_their_parts(whole_layers):
    """Three layers: window attention with q/k norm, a layer with a toy feed-forward, full
    attention without q/k norm.  The first and the last run in the kernel (one launch each: the
    toy layer stands between them), the toy layer through its parts; two cache groups."""
    from zinfer_b200 import ops
    from zinfer_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from zinfer_b200.engine import DecoderModel, ModelRunner, StepEntry
    from zinfer_b200.parts import register_part, unregister_part
    from zinfer_b200.weights import random_tensors

    H, I, NQ, NKV, D, V, EPS = 192, 320, 6, 2, 64, 331, 3e-6
    norm = PartSpec("rmsnorm", {"size": H, "eps": EPS})
    rope = PartSpec("rope", {"head_dim": D, "theta": 5000.0, "max_positions": 512})

    def attn(window, qk):
        return PartSpec("gqa_attention", {"hidden_size": H, "num_heads": NQ, "num_kv_heads": NKV, "head_dim": D,
                                          "qk_norm_eps": EPS if qk else None, "window": window, "position": rope})

    swiglu = PartSpec("swiglu_mlp", {"hidden_size": H, "intermediate_size": I})
    relu = PartSpec("toy_relu_ffn", {"hidden_size": H, "intermediate_size": I})

    def block(mixer, ffn):
        return PartSpec("prenorm_block", {"mixer": mixer, "mixer_norm": norm, "feed_forward": ffn, "ffn_norm": norm})

    layers = (LayerSpec(block(attn(21, True), swiglu), prefix="layers.0."),
              LayerSpec(block(attn(None, True), relu), prefix="layers.1."),
              LayerSpec(block(attn(None, False), swiglu), prefix="layers.2."))
    spec = ModelSpec(
        architecture="ToyMixed", vocab_size=V, hidden_size=H, max_positions=512,
        embedding=PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H, "name": "embed"}),
        layers=layers, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2)),
        final_norm=PartSpec("rmsnorm", {"size": H, "eps": EPS, "name": "norm"}),
        head=PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "name": "head", "tied_to": None}))
    register_part("toy_relu_ffn", _make_relu_ffn())
    try:
        outs = []
        for fused in (False, True):
            ops.DECODE_LAYERS = fused
            model = DecoderModel(spec, torch.bfloat16, DEV)
            model.bind(random_tensors(model.tensor_specs(), 5, torch.bfloat16, DEV))
            runner = ModelRunner(model, page_size=16, max_tokens=1024, max_requests=8, cuda_graphs=False)
            kinds = [p is not None for _, _, p in model._spans]
            assert kinds == ([True, False, True] if fused else [False, False, False])
            assert len(runner.manager.groups) == 2
            rng = random.Random(2)
            ids = ["a", "b", "c"]
            for rid, n in zip(ids, (60, 5, 33)):
                runner.add_request(rid)
                runner.step([StepEntry(rid, [rng.randrange(V) for _ in range(n)], [])])
            rows = []
            for _ in range(30):   # long enough for the window to pass pages
                toks = [rng.randrange(V) for _ in ids]
                rows.append(runner.step([StepEntry(r, [t], [0]) for r, t in zip(ids, toks)]).float().cpu())
            outs.append(torch.stack(rows))
            runner.manager.check()
        assert whole_layers["n"] == 60   # two launches a step
        chain, whole = outs
        scale = chain.abs().amax(dim=-1, keepdim=True)
        assert torch.isfinite(whole).all() and ((whole - chain).abs() <= 2e-2 * scale + 1e-3).all()
        assert ops.kernel_status() == 0
    finally:
        unregister_part("toy_relu_ffn")


def test_unsupported_sizes_are_left_to_the_parts(model_dirs, whole_layers):
    """Head sizes the kernel does not take (16, 32, 48) are never prepared for it."""
    for name in ("A", "B", "C"):
        runner = _runner(model_dirs[(name, "bfloat16")], name, True, max_tokens=256, max_requests=2)
        assert all(p is None for _, _, p in runner.model._spans)
