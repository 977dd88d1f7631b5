import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Two tiny configurations of Qwen3 that differ in every size and option.
TINY_A = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=256, hidden_size=64, intermediate_size=128,
    num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16, max_position_embeddings=128,
    rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=True, torch_dtype="bfloat16")
TINY_B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=384, hidden_size=96, intermediate_size=160,
    num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=1, head_dim=32, max_position_embeddings=256,
    rms_norm_eps=1e-5, rope_theta=1000000.0, tie_word_embeddings=False, torch_dtype="bfloat16")
# a third one with sizes that are no powers of two anywhere: width 72, heads of 48, vocabulary 301
TINY_C = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=301, hidden_size=72, intermediate_size=200,
    num_hidden_layers=2, num_attention_heads=3, num_key_value_heads=3, head_dim=48, max_position_embeddings=512,
    rms_norm_eps=3e-6, rope_theta=50000.0, tie_word_embeddings=False, torch_dtype="bfloat16")
# two with the head sizes the tensor-core kernels take (64 and 128), grouped and not, with a
# feed-forward width that is a multiple of 64 (D) and one that is not (E)
TINY_D = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=1000, hidden_size=256, intermediate_size=512,
    num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2, head_dim=64, max_position_embeddings=1024,
    rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False, torch_dtype="bfloat16")
TINY_E = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=777, hidden_size=320, intermediate_size=456,
    num_hidden_layers=2, num_attention_heads=3, num_key_value_heads=3, head_dim=128, max_position_embeddings=640,
    rms_norm_eps=2e-5, rope_theta=20000.0, tie_word_embeddings=True, torch_dtype="bfloat16")
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}
PAGE_SIZE = {"A": 16, "B": 8, "C": 32, "D": 16, "E": 64}


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders with random weights, written once per session into a
    temporary folder: {(name, 'bfloat16'|'float32'): path}."""
    from zinfer_b200.config import Qwen3Config
    from zinfer_b200.weights import write_model_dir

    out = {}
    root = tmp_path_factory.mktemp("models")
    for name, raw in TINY.items():
        cfg = Qwen3Config.from_dict(raw)
        for dt, tdt in (("bfloat16", torch.bfloat16), ("float32", torch.float32)):
            out[(name, dt)] = write_model_dir(str(root / f"{name}_{dt}"), cfg, seed=1234 + ord(name), dtype=tdt)
    return out


@pytest.fixture
def cpu_kernels(monkeypatch):
    """Puts the plain PyTorch references in the kernels' place so that the engine's
    host logic (batching, cache, scheduler) can run without a GPU.  Test-only."""
    import kernel_refs
    from zinfer_b200 import ops
    from zinfer_b200.engine import runner

    for name in ("embed_gather", "add_rmsnorm", "residual_add", "swiglu", "rope_table", "qk_norm_rope_store",
                 "linear", "attention_tile_rows", "attention_prefill_tile_rows", "paged_attention", "attention", "argmax", "linear_argmax", "patch_tokens", "linear_swiglu", "interleave_gate_up", "decode_fused_ok", "sample", "count_tokens"):
        monkeypatch.setattr(ops, name, getattr(kernel_refs, name))
    monkeypatch.setattr(ops, "lib", lambda: None)
    monkeypatch.setattr(runner, "_require_cuda", lambda device: None)
    return kernel_refs
