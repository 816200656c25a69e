"""A plain, slow implementation of the Qwen3 dense decoder for the tests.

Whole sequences, no cache, one function per part, float32 with plain tensor
arithmetic, on the CPU unless the weights it is given lie on another device (the
tests of wide layers hand it tensors on the GPU, where the same formulas run through
the tensor library's own float32 and float64 products).  It shares no code with `litellmengine_b200` (it does not
import it) and is written from the reference's formulas; each function cites the
reference file and lines it restates.  `tests/golden/` compares it once against
the reference's own C++ code compiled for the CPU.

A "model" here is a dict of hyper-parameters (`cfg`) plus a dict of float32
tensors keyed by checkpoint tensor names (`w`).  `act` (default: identity) is applied
wherever a bfloat16 engine stores an activation as an operand of a matrix product or
in the cache: passing `to_bf16` makes this code round at those places too, which turns
the comparison with a bfloat16 run from "within bfloat16's error" into "the same
numbers up to summation order".  Everything else stays float32 either way.
`forward_logits(..., wd=torch.float64)` runs the same formulas in double precision
(the rotation angle stays the float32 product the reference defines), which makes it
an oracle whose own rounding is negligible beside a float32 engine's.  `window` (None for Qwen3) and a
per-layer hook exist so that tests of the engine's generality can reuse the same
part functions with other wirings.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import numpy as np
import torch


def identity(t: torch.Tensor) -> torch.Tensor:
    return t


def to_bf16(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(torch.float32)


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """h[t,:] = E[ids[t],:]; ids outside [0,V) are an error.  src/layers/embedding.cu:62-89"""
    if ids.numel() and (int(ids.min()) < 0 or int(ids.max()) >= table.shape[0]):
        raise IndexError("token id out of range")
    return table[ids.long()].to(torch.float32)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """out = x * (1/sqrt(mean(x^2) + eps)) * w over the last dim, in float32.
    src/layers/rms_norm.cu:64-93 (mean = sum/size; product order (x*inv)*w)."""
    if not x.dtype.is_floating_point or x.dtype in (torch.bfloat16, torch.float16):
        x = x.to(torch.float32)
    mean_sq = (x * x).sum(dim=-1, keepdim=True) / float(x.shape[-1])
    inv = 1.0 / torch.sqrt(mean_sq + torch.tensor(eps, dtype=torch.float32).to(x.dtype))
    return x * inv * weight.to(x.dtype)


def rope_inv_freq(head_dim: int, theta: float) -> torch.Tensor:
    """inv_freq_i = powf(theta, -(2i)/head_dim): theta and the exponent are float32, the
    exponent is the float32 quotient.  src/layers/rotary.cu:81-83.  The C library's powf is
    correctly rounded in all but rare cases, so it is restated as the double-precision power
    of the float32 operands, rounded to float32 (numpy's float32 power is sometimes one unit
    in the last place off, which shows as an angle error of position * 6e-8)."""
    i = np.arange(head_dim // 2, dtype=np.float32)
    expo = (-(2.0 * i).astype(np.float32) / np.float32(head_dim)).astype(np.float32)
    inv = np.power(np.float64(np.float32(theta)), expo.astype(np.float64)).astype(np.float32)
    return torch.from_numpy(inv)


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Half-split rotation on [T, heads, d]: pairs (i, i+d/2); angle = float(pos) *
    inv_freq_i in float32; o[i] = x[i]*cos - x[i+d/2]*sin; o[i+d/2] = x[i+d/2]*cos + x[i]*sin.
    src/layers/rotary.cu:85-117"""
    T, H, d = x.shape
    half = d // 2
    ang = positions.to(torch.float32)[:, None] * rope_inv_freq(d, theta).to(x.device)[None, :]   # float32 product
    ang = ang.to(x.dtype)
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                     window: Optional[int] = None, scale: Optional[float] = None, act=None) -> torch.Tensor:
    """q [T,nq,d], k/v [T,nkv,d] -> [T,nq,d].  kv_head = q_head // (nq/nkv); score =
    (q.k) / sqrt(d); key j visible to query i iff j <= i (and i-j < window if a window
    is given); softmax in float32; out = sum p_j v_j.  `act` rounds the weights
    exp(score - row max) on their way into the second product, as a bfloat16 engine does
    (the row sum is taken before the rounding).
    src/ops/attention.cu:188-250 (the reference computes the same sum with a running
    max; the two-pass form here is its CPU paged variant, src/ops/paged_attention.cpp:159-217)."""
    T, nq, d = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    if scale is None:
        scale = 1.0 / math.sqrt(float(d))
    out = torch.empty_like(q)
    idx = torch.arange(T, device=q.device)
    visible = idx[None, :] <= idx[:, None]
    if window is not None:
        visible &= (idx[:, None] - idx[None, :]) < window
    for h in range(nq):
        kh = h // group
        s = (q[:, h, :] @ k[:, kh, :].T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        e = torch.exp(s - s.max(dim=-1, keepdim=True).values)          # 0 where masked
        total = e.sum(dim=-1, keepdim=True)
        out[:, h, :] = ((e if act is None else act(e)) @ v[:, kh, :]) / total
    return out


def attention_qkv(x: torch.Tensor, positions: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, cfg: dict,
                  act=identity, with_kv: bool = True):
    """q/k/v projections without bias, per-head RMSNorm of q and k with one [d] weight each
    (same eps), rotation of q and k; v stays as projected.  src/model/qwen3.cpp:357-449"""
    T = x.shape[0]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    q = (x @ w[f"{prefix}.q_proj.weight"].T).view(T, nq, d)
    q = act(rope(rms_norm(q, w[f"{prefix}.q_norm.weight"], cfg["rms_norm_eps"]), positions, cfg["rope_theta"]))
    if not with_kv:
        return q, None, None
    k = (x @ w[f"{prefix}.k_proj.weight"].T).view(T, nkv, d)
    v = (x @ w[f"{prefix}.v_proj.weight"].T).view(T, nkv, d)
    k = act(rope(rms_norm(k, w[f"{prefix}.k_norm.weight"], cfg["rms_norm_eps"]), positions, cfg["rope_theta"]))
    return q, k, act(v)


def attention_block(x: torch.Tensor, positions: torch.Tensor, w: Dict[str, torch.Tensor],
                    prefix: str, cfg: dict, window: Optional[int] = None, act=identity, kv=None,
                    attn_act=None) -> torch.Tensor:
    """Attention over this layer's own keys and values, or over `kv` = (k, v) of another layer
    when given; then the output projection.  `attn_act` rounds the attention weights (see
    `causal_attention`).  src/model/qwen3.cpp:550-567"""
    T = x.shape[0]
    q, k, v = attention_qkv(x, positions, w, prefix, cfg, act, with_kv=kv is None)
    if kv is not None:
        k, v = kv
    a = act(causal_attention(q, k, v, window=window, act=attn_act))
    return a.reshape(T, -1) @ w[f"{prefix}.o_proj.weight"].T


def silu_and_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """(g / (1 + exp(-g))) * u.  src/ops/silu_and_mul.cu:44-46"""
    return gate / (1.0 + torch.exp(-gate)) * up


def swiglu(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, act=identity) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)), no biases.  src/model/qwen3.cpp:143-152"""
    g = act(x @ w[f"{prefix}.gate_proj.weight"].T)
    u = act(x @ w[f"{prefix}.up_proj.weight"].T)
    return act(silu_and_mul(g, u)) @ w[f"{prefix}.down_proj.weight"].T


def decoder_layer(h: torch.Tensor, positions: torch.Tensor, w: Dict[str, torch.Tensor],
                  layer: int, cfg: dict, window: Optional[int] = None, act=identity, attn_act=None) -> torch.Tensor:
    """h += attn(norm_in(h)); h += mlp(norm_post(h)).  src/model/qwen3.cpp:948-968"""
    p = f"model.layers.{layer}"
    a = attention_block(act(rms_norm(h, w[f"{p}.input_layernorm.weight"], cfg["rms_norm_eps"])),
                        positions, w, f"{p}.self_attn", cfg, window, act, attn_act=attn_act)
    h = h + a
    f = swiglu(act(rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], cfg["rms_norm_eps"])), w, f"{p}.mlp", act)
    return h + f


def forward_logits(ids, w: Dict[str, torch.Tensor], cfg: dict,
                   layer_order: Optional[List[int]] = None, act=identity, wd=torch.float32,
                   attn_act=None) -> torch.Tensor:
    """Logits [T, V] for a whole sequence starting at position 0: embedding, the
    layers in order, final RMSNorm, output head (the embedding table when tied and
    `lm_head.weight` is absent).  src/model/qwen3.cpp:1242-1278,1501"""
    dev = w["model.embed_tokens.weight"].device
    ids = torch.as_tensor(ids, dtype=torch.int64, device=dev)
    w = {k: t.to(wd) for k, t in w.items()}
    positions = torch.arange(ids.shape[0], dtype=torch.int32, device=dev)
    h = embedding(ids, w["model.embed_tokens.weight"]).to(wd)
    order = layer_order if layer_order is not None else list(range(cfg["num_hidden_layers"]))
    for layer in order:
        h = decoder_layer(h, positions, w, layer, cfg, act=act, attn_act=attn_act)
    hn = act(rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"]))
    head = w.get("lm_head.weight")
    if head is None:
        if not cfg.get("tie_word_embeddings", False):
            raise KeyError("lm_head.weight")
        head = w["model.embed_tokens.weight"]
    return (hn @ head.T).to(torch.float32)


def argmax_token(logits_row: torch.Tensor) -> int:
    """Largest logit; ties go to the lowest index.  src/ops/argmax.cu:41-62"""
    best, best_v = 0, float(logits_row[0])
    for i in range(1, logits_row.shape[0]):
        v = float(logits_row[i])
        if v > best_v:
            best, best_v = i, v
    return best


def greedy_generate(prompt: List[int], w, cfg, max_new_tokens: int, eos_token_id: int = -1) -> List[int]:
    """Re-forward the whole sequence for every new token; stop after `max_new_tokens`
    or when eos is produced (eos is kept).  src/runtime/generation.cpp:72-155 for the
    loop, src/engine/request_manager.cpp:122-159 for the stopping rule."""
    ids = list(prompt)
    new: List[int] = []
    for _ in range(max_new_tokens):
        t = argmax_token(forward_logits(ids, w, cfg)[-1])
        ids.append(t)
        new.append(t)
        if eos_token_id >= 0 and t == eos_token_id:
            break
    return new


def temperature_probs(logits_row: torch.Tensor, temperature: float) -> torch.Tensor:
    """softmax(logits / T) in float32 (the reference parses --temperature but never
    samples, src/main.cpp:175-178; this is the engine's own rule)."""
    z = logits_row.to(torch.float32) / float(temperature)
    z = z - z.max()
    e = torch.exp(z)
    return e / e.sum()
