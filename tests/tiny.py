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


# Matrices N(0, 0.02 * SHARP): the tiny models' logits then have a standard deviation of 0.6-0.9 and
# their attention is far from uniform, so that a wrong or missing cache row moves the logits by much
# more than bfloat16 rounding does.  Measured on a B200 over these four shapes (97 tokens, all places):
# at 0.02 the bfloat16 engine's largest error is 0.003-0.004 and the least influential single token
# moves some later logit by 0.012-0.030 (3.6-11 times the error); at 0.08 the error is 0.023-0.033 and
# that token's effect 0.31-0.47 (9-16 times); at 0.12 attention is so sharp that some tokens hardly
# matter (4-10 times).  So the tests run at 0.08.
SHARP = 4.0

# a fourth shape: context beyond 2,048 (decoding crosses the 1,024-position bucket of the decode graphs
# and the attention kernel's change of variant there) and 8 kv heads
TINY_D = dict(
    architectures=["LlamaForCausalLM"], model_type="llama",
    num_hidden_layers=2, hidden_size=128, num_attention_heads=16, num_key_value_heads=8, head_dim=16,
    intermediate_size=144, vocab_size=200, rope_theta=100000.0,
    rope_scaling=dict(rope_type="llama3", factor=4.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=512),
    rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=2304)


# heads wider than the tensor-core attention kernels take (128): the plain attention kernel serves them
TINY_E = dict(
    architectures=["LlamaForCausalLM"], model_type="llama",
    num_hidden_layers=2, hidden_size=104, num_attention_heads=2, num_key_value_heads=1, head_dim=160,
    intermediate_size=136, vocab_size=211, rope_theta=10000.0, rope_scaling=None, rms_norm_eps=1e-5,
    tie_word_embeddings=True, max_position_embeddings=192)


def jitter_norm_weights(model_dir: str, seed: int, amount: float = 0.25) -> dict:
    """Rewrite the folder's norm weights (the vectors that the random mode writes as 1.0) as 1 + amount * N(0, 1),
    different in every vector; returns all tensors of the folder as they now are."""
    from mdma_b200.weights import write_safetensors
    from mdma_b200.weights.safetensors_io import SafetensorsFile
    path = os.path.join(model_dir, "model.safetensors")
    sf = SafetensorsFile(path)
    tensors = {n: sf.tensor(n).clone() for n in sf.entries}
    del sf
    g = torch.Generator().manual_seed(1000 + seed)
    for name in sorted(tensors):
        t = tensors[name]
        if t.dim() == 1 and t.is_floating_point() and bool((t == 1).all()):
            tensors[name] = (1.0 + amount * torch.randn(t.shape, generator=g)).to(t.dtype)
    write_safetensors(path, tensors)
    return tensors


def make_model(cfg: dict, seed: int, dtype=torch.float32, root=None, std_scale: float = 1.0, norm_jitter: float = 0.25):
    """Write a model folder into a fresh temporary directory; returns (dir, config dict, tensors).
    Matrices are N(0, 0.02 * std_scale).  The random mode writes every norm weight as 1.0, which would hide
    a norm that reads another layer's weight (or none): the folder is rewritten with norm weights
    1 + norm_jitter * N(0, 1), different in every vector."""
    from mdma_b200.weights import write_random_model
    from mdma_b200.weights.safetensors_io import SafetensorsFile
    d = tempfile.mkdtemp(prefix="mdma_tiny_", dir=root)
    write_random_model(d, cfg, seed, dtype, std=0.02 * std_scale)
    if norm_jitter:
        tensors = jitter_norm_weights(d, seed, norm_jitter)
    else:
        sf = SafetensorsFile(os.path.join(d, "model.safetensors"))
        tensors = {n: sf.tensor(n).clone() for n in sf.entries}
    return d, json.load(open(os.path.join(d, "config.json"))), tensors
