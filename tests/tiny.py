"""Tiny configurations for the tests: they differ in every size and option."""
import json
import os
import tempfile

import torch

TINY_A = dict(
    architectures=["LlamaForCausalLM"], model_type="llama",
    num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
    intermediate_size=176, vocab_size=256, rope_theta=10000.0, rope_scaling=None, rms_norm_eps=1e-5,
    tie_word_embeddings=False, max_position_embeddings=128, rope_layout="interleaved")

TINY_B = dict(
    architectures=["LlamaForCausalLM"], model_type="llama",
    num_hidden_layers=3, hidden_size=96, num_attention_heads=3, num_key_value_heads=1, head_dim=32,
    intermediate_size=256, vocab_size=384, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=64),
    rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=256)

# hidden width, heads and vocabulary that are no power of two; head size 48; heads*head_dim != hidden
TINY_C = dict(
    architectures=["LlamaForCausalLM"], model_type="llama",
    num_hidden_layers=2, hidden_size=120, num_attention_heads=6, num_key_value_heads=3, head_dim=48,
    intermediate_size=200, vocab_size=331, rope_theta=50000.0, rope_scaling=None, rms_norm_eps=3e-6,
    tie_word_embeddings=False, max_position_embeddings=512)


def make_model(cfg: dict, seed: int, dtype=torch.float32, root=None, std_scale: float = 1.0):
    """Write a model folder into a fresh temporary directory; returns (dir, config dict, tensors)."""
    from mdma_b200.weights import write_random_model
    from mdma_b200.weights.safetensors_io import SafetensorsFile
    d = tempfile.mkdtemp(prefix="mdma_tiny_", dir=root)
    write_random_model(d, cfg, seed, dtype)
    sf = SafetensorsFile(os.path.join(d, "model.safetensors"))
    tensors = {n: sf.tensor(n).clone() for n in sf.entries}
    return d, json.load(open(os.path.join(d, "config.json"))), tensors
