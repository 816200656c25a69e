"""The tiny Qwen3 configurations the tests use, and their seeded weights.

They differ in every size and option: layer count, hidden size, head counts and
group size, head_dim (A: heads*head_dim == hidden; B: != hidden), intermediate size,
vocabulary (no power of two for B), rope_theta, rms_norm_eps, tied or separate
output head, page size.  Weights come from numpy's legacy RandomState so that the
committed golden logits stay valid: matrices N(0, 0.02), norm weights 1 + N(0, 0.01).
This file does not import the engine.
"""
from __future__ import annotations

import numpy as np
import torch

TINY_A = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=1,
    head_dim=16, intermediate_size=128, vocab_size=256, rope_theta=10000.0,
    rms_norm_eps=1e-6, max_position_embeddings=128, tie_word_embeddings=True,
    torch_dtype="float32",
)
TINY_A_PAGE, TINY_A_SEED = 4, 0

TINY_B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=3, hidden_size=96, num_attention_heads=6, num_key_value_heads=3,
    head_dim=32, intermediate_size=224, vocab_size=384, rope_theta=1000000.0,
    rms_norm_eps=1e-5, max_position_embeddings=256, tie_word_embeddings=False,
    torch_dtype="float32",
)
TINY_B_PAGE, TINY_B_SEED = 8, 1

# A third shape for longer sequences (hundreds of keys, many pages): sizes that are
# no power of two, a group of 3, head_dim 48 (a multiple of 16 that is no power of two).
TINY_C = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=80, num_attention_heads=6, num_key_value_heads=2,
    head_dim=48, intermediate_size=176, vocab_size=331, rope_theta=50000.0,
    rms_norm_eps=3e-6, max_position_embeddings=2048, tie_word_embeddings=False,
    torch_dtype="float32",
)
TINY_C_PAGE, TINY_C_SEED = 16, 7


# Head size 64, which the tuned bfloat16 attention kernels take (the others run the generic one).
TINY_D = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=96, num_attention_heads=4, num_key_value_heads=2,
    head_dim=64, intermediate_size=160, vocab_size=211, rope_theta=1000000.0,
    rms_norm_eps=1e-6, max_position_embeddings=4096, tie_word_embeddings=True,
    torch_dtype="bfloat16",
)
TINY_D_PAGE, TINY_D_SEED = 16, 11


# Head size 128: prompt portions run the tcgen05 kernel.  E has groups of two query heads
# (two heads share a key/value tile in one CTA), F a group of three (one head per CTA).
TINY_E = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=160, num_attention_heads=4, num_key_value_heads=2,
    head_dim=128, intermediate_size=192, vocab_size=307, rope_theta=1000000.0,
    rms_norm_eps=1e-6, max_position_embeddings=4096, tie_word_embeddings=False,
    torch_dtype="bfloat16",
)
TINY_E_PAGE, TINY_E_SEED = 16, 13

TINY_F = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=3, hidden_size=112, num_attention_heads=3, num_key_value_heads=1,
    head_dim=128, intermediate_size=144, vocab_size=199, rope_theta=10000.0,
    rms_norm_eps=2e-6, max_position_embeddings=2048, tie_word_embeddings=True,
    torch_dtype="bfloat16",
)
TINY_F_PAGE, TINY_F_SEED = 32, 17


# One layer at the widths of a real 8B model (a small vocabulary keeps it quick): the products'
# k-splits, tiled weight copies and the attention kernels' grids at the sizes they are tuned for.
WIDE_G = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=1, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
    head_dim=128, intermediate_size=12288, vocab_size=1031, rope_theta=1000000.0,
    rms_norm_eps=1e-6, max_position_embeddings=4096, tie_word_embeddings=False,
    torch_dtype="bfloat16",
)
WIDE_G_PAGE, WIDE_G_SEED = 16, 19


def tensor_shapes(cfg: dict) -> dict:
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    shapes = {"model.embed_tokens.weight": (V, H), "model.norm.weight": (H,)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}"
        shapes[f"{p}.input_layernorm.weight"] = (H,)
        shapes[f"{p}.post_attention_layernorm.weight"] = (H,)
        shapes[f"{p}.self_attn.q_proj.weight"] = (nq * d, H)
        shapes[f"{p}.self_attn.k_proj.weight"] = (nkv * d, H)
        shapes[f"{p}.self_attn.v_proj.weight"] = (nkv * d, H)
        shapes[f"{p}.self_attn.o_proj.weight"] = (H, nq * d)
        shapes[f"{p}.self_attn.q_norm.weight"] = (d,)
        shapes[f"{p}.self_attn.k_norm.weight"] = (d,)
        shapes[f"{p}.mlp.gate_proj.weight"] = (I, H)
        shapes[f"{p}.mlp.up_proj.weight"] = (I, H)
        shapes[f"{p}.mlp.down_proj.weight"] = (H, I)
    if not cfg["tie_word_embeddings"]:
        shapes["lm_head.weight"] = (V, H)
    return shapes


def make_weights(cfg: dict, seed: int, bf16_exact: bool = False, matrix_std: float = 0.02) -> dict:
    """Float32 tensors by checkpoint name.  With `bf16_exact` every value is rounded
    to the nearest bfloat16 first, so that a bfloat16 engine and the plain float32
    implementation hold identical weights."""
    rs = np.random.RandomState(seed)
    out = {}
    for name, shape in sorted(tensor_shapes(cfg).items()):
        x = rs.standard_normal(shape).astype(np.float32)
        if len(shape) == 1:
            x = np.float32(1.0) + np.float32(0.01) * x
        else:
            x = np.float32(matrix_std) * x
        t = torch.from_numpy(x)
        if bf16_exact:
            t = t.to(torch.bfloat16).to(torch.float32)
        out[name] = t
    return out


def random_tokens(cfg: dict, n: int, seed: int) -> list:
    rs = np.random.RandomState(10_000 + seed)
    return [int(x) for x in rs.randint(0, cfg["vocab_size"], size=n)]
