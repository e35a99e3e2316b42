import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

# Two tiny configurations of the architecture that differ in every size and option: layers, width,
# heads and groups (group 2 vs 3), head size, feed-forward width (176 is no multiple of 32), vocabulary,
# rope base, frequency scaling (none vs llama3 with all three bands in use), eps, tied or not.
TINY_A = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 176, "vocab_size": 256,
    "max_position_embeddings": 128, "rope_theta": 10000.0, "rope_scaling": None, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "eos_token_id": 7,
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 96, "num_hidden_layers": 3, "num_attention_heads": 3,
    "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 256, "vocab_size": 384,
    "max_position_embeddings": 256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 32},
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "eos_token_id": [3, 5],
}
# A third one for odd sizes: width and vocabulary that are no power of two nor multiples of 32,
# head size 48 (a step of 16 that is no power of two), five heads in one group.
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 80, "num_hidden_layers": 2, "num_attention_heads": 5,
    "num_key_value_heads": 1, "head_dim": 48, "intermediate_size": 136, "vocab_size": 301,
    "max_position_embeddings": 512, "rope_theta": 20000.0, "rope_scaling": None, "rms_norm_eps": 3e-6,
    "tie_word_embeddings": False,
}
# Two more with the head sizes the tensor-core attention kernels take (64 and 128), so that the engine tests run
# those kernels inside a whole model: groups of 2 and 3 heads, widths that are no power of two.
TINY_D = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 192, "num_hidden_layers": 2, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 328, "vocab_size": 520,
    "max_position_embeddings": 1024, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
}
TINY_E = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 264, "num_hidden_layers": 2, "num_attention_heads": 3,
    "num_key_value_heads": 1, "head_dim": 128, "intermediate_size": 400, "vocab_size": 333,
    "max_position_embeddings": 1024, "rope_theta": 10000.0, "rope_scaling": None, "rms_norm_eps": 2e-6,
    "tie_word_embeddings": False,
}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


def _has_cuda():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_cuda():
        return
    skip = pytest.mark.skip(reason="no CUDA device here")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def tiny_configs():
    return {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders for the tiny configurations, written once per session into a temporary place.
    Keys: (config name, stored dtype).  Weights are wider than N(0, 0.02) and norm weights are spread
    around 1, so that logits are of order 1 and a forgotten norm weight shows."""
    from ghost_infer_b200.weights import write_random_model
    made = {}

    def get(name, stored):
        key = (name, stored)
        if key not in made:
            cfg = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}[name]
            d = tmp_path_factory.mktemp(f"tiny_{name}_{stored}")
            seed = {"A": 0, "B": 1, "C": 2, "D": 3, "E": 4}[name]
            write_random_model(str(d), cfg, seed=seed, dtype=stored, std=0.05, norm_jitter=0.1)
            made[key] = str(d)
        return made[key]

    return get
