"""The tiny configurations of the tests, and helpers around random model folders.

A and B differ in every size and option: layers, widths, head counts, group
size, head size tied to the width or not, vocabulary, rope base, norm epsilon,
tied or separate head, weight scales, page size.
"""
import os

import torch

from prelude_b200.weights.random_init import write_random_model

TINY_A = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=256, hidden_size=64,
              intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
              max_position_embeddings=128, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
              attention_bias=False, use_sliding_window=False, sliding_window=None, max_window_layers=2,
              hidden_act="silu")
TINY_B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=384, hidden_size=96,
              intermediate_size=160, num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=2, head_dim=32,
              max_position_embeddings=256, rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
              attention_bias=False, use_sliding_window=False, hidden_act="silu", eos_token_id=[7, 9])
# not a power of two anywhere, one key/value head, longer context; used for long decoding and replay
TINY_C = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=331, hidden_size=72,
              intermediate_size=200, num_hidden_layers=2, num_attention_heads=5, num_key_value_heads=1, head_dim=48,
              max_position_embeddings=1024, rope_theta=50000.0, rms_norm_eps=3e-6, tie_word_embeddings=True,
              attention_bias=True)

# the sizes at which the fast kernels take their special paths: head size 128 (permuted pages, bulk copies, the
# vector rope kernel), a feed-forward so wide that the down projection of a decode step cuts K into parts
TINY_D = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=500, hidden_size=192,
              intermediate_size=8192, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2, head_dim=128,
              max_position_embeddings=512, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
              attention_bias=False, use_sliding_window=False, hidden_act="silu")

# sizes that the tcgen05 prompt-attention kernel takes (head size 64, four query heads per key/value head, pages of
# 8 tokens): in the engine tests the long portions then run on it, the short ones and the single tokens beside them
# on the other two attention kernels
TINY_E = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=700, hidden_size=160,
              intermediate_size=416, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2, head_dim=64,
              max_position_embeddings=1024, rope_theta=500000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
              attention_bias=False, use_sliding_window=False, hidden_act="silu")

PARAMS = {"A": (TINY_A, dict(seed=0, std=0.02, norm_jitter=0.1), 4),
          "D": (TINY_D, dict(seed=3, std=0.02, norm_jitter=0.1), 16),
          "E": (TINY_E, dict(seed=4, std=0.04, norm_jitter=0.2), 8),
          "B": (TINY_B, dict(seed=1, std=0.03, norm_jitter=0.2), 8),
          "C": (TINY_C, dict(seed=2, std=0.05, norm_jitter=0.3), 16)}


def make_folder(tmp_path, which: str, dtype=torch.float32, **overrides):
    cfg, init, _ = PARAMS[which]
    init = dict(init, **overrides)
    d = os.path.join(str(tmp_path), f"tiny_{which}_{str(dtype).split('.')[-1]}")
    return write_random_model(d, cfg, dtype=dtype, **init)


def read_weights(model_dir):
    """Tensors by name, read with the safetensors package (not with the engine's reader)."""
    from safetensors import safe_open
    out = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            out[name] = f.get_tensor(name)
    return out


def random_ids(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
