"""Plain, slow Qwen3 dense decoder: whole sequences, no cache, one function per part.

Written from the formulas of michaelasper/kir-ai (paths below are relative to
that project); it rests on the formulas alone, because the reference is a Rust
workspace and no Rust toolchain exists where these tests run, so its model code
cannot be compiled or imported for a one-time comparison.  The closed-form
values of the reference's own unit tests are reproduced in
``test_plain_reference.py`` instead.

It shares no code with the engine: it has its own safetensors reader, works on
CPU with ``torch`` tensor arithmetic only, and recomputes every position of a
sequence from scratch.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


# --------------------------------------------------------------------------- files
def read_model_folder(model_dir: str, dtype=torch.float32):
    """config.json as a dict and every tensor of model.safetensors widened to ``dtype``.

    Container format: crates/llm-backend/src/core/safetensors.rs:187-203 (8-byte
    little-endian header length, JSON header, payload).
    """
    with open(os.path.join(model_dir, "config.json")) as handle:
        config = json.load(handle)
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as handle:
        (header_len,) = struct.unpack("<Q", handle.read(8))
        header = json.loads(handle.read(header_len))
        payload = handle.read()
    weights: Dict[str, torch.Tensor] = {}
    for name, item in header.items():
        if name == "__metadata__":
            continue
        begin, end = item["data_offsets"]
        raw = np.frombuffer(payload[begin:end], dtype=np.uint8).copy()
        if item["dtype"] == "BF16":
            # bf16 is the upper half of an f32 (crates/llm-backend/src/core/math.rs:570-572)
            as_u32 = raw.view(np.uint16).astype(np.uint32) << 16
            tensor = torch.from_numpy(as_u32.view(np.float32).copy())
        elif item["dtype"] == "F32":
            tensor = torch.from_numpy(raw.view(np.float32).copy())
        else:
            raise ValueError(f"plain reader: dtype {item['dtype']} of {name}")
        weights[name] = tensor.reshape(item["shape"]).to(dtype)
    return config, weights


# --------------------------------------------------------------------------- parts
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * 1/sqrt(mean(x^2) + eps) * w over the last axis; scale 0 when mean+eps == 0.

    crates/llm-backend/src/core/math.rs:73-113 (plain weight, offset 0, for the dense
    model: crates/llm-backend/src/core/qwen/ops/norm.rs:119-133).
    """
    mean_square = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    variance = mean_square + eps
    scale = torch.where(variance == 0, torch.zeros_like(variance), 1.0 / torch.sqrt(variance))
    return x * scale * weight


def rope(x: torch.Tensor, positions: Sequence[int], theta: float, rotary_dim: Optional[int] = None) -> torch.Tensor:
    """Half-split rotary embedding of ``x`` [T, heads, d] at absolute ``positions``.

    crates/llm-backend/src/core/math.rs:515-529: inv_freq_i = theta^(-2i/rotary_dim) and the
    angle position*inv_freq are formed in 32-bit; pairs are (i, i + rotary_dim/2).
    """
    d = x.shape[-1]
    rotary_dim = d if rotary_dim is None else rotary_dim
    half = rotary_dim // 2
    exponent = -(2.0 * torch.arange(half, dtype=torch.float32)) / float(rotary_dim)
    inv_freq = torch.pow(torch.tensor(theta, dtype=torch.float32), exponent)
    pos = torch.tensor(list(positions), dtype=torch.float32)
    angle = (pos[:, None] * inv_freq[None, :]).to(torch.float64)
    cos = torch.cos(angle).to(x.dtype)[:, None, :]
    sin = torch.sin(angle).to(x.dtype)[:, None, :]
    first, second = x[..., :half], x[..., half:rotary_dim]
    out = x.clone()
    out[..., :half] = first * cos - second * sin
    out[..., half:rotary_dim] = second * cos + first * sin
    return out


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: Optional[int]) -> torch.Tensor:
    """Causal grouped-query attention over a whole sequence.

    q [T, nq, d], k and v [T, nkv, d].  Query head h reads kv head h // (nq/nkv)
    (crates/llm-backend/src/core/native_attention.rs:732); scores are q.k * d^-1/2
    (:827-841) over rows j <= i (a token attends to itself, :409-415); with a window W
    the cache keeps the last W rows, so j >= i - W + 1
    (crates/llm-backend/src/core/qwen/ops/cache.rs:116-121,
    crates/llm-kv-cache/src/layer.rs:765-805); softmax subtracts the maximum
    (crates/llm-backend/src/core/math.rs:476-505).
    """
    T, nq, d = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    scale = d ** -0.5
    rows = torch.arange(T)[:, None]
    cols = torch.arange(T)[None, :]
    visible = cols <= rows
    if window is not None:
        visible = visible & (cols >= rows - window + 1)
    out = torch.zeros_like(q)
    for h in range(nq):
        kv_head = h // group
        scores = (q[:, h, :] @ k[:, kv_head, :].T) * scale
        scores = scores.masked_fill(~visible, float("-inf"))
        weights = torch.exp(scores - scores.max(dim=-1, keepdim=True).values)
        weights = weights / weights.sum(dim=-1, keepdim=True)
        out[:, h, :] = weights @ v[:, kv_head, :]
    return out


def silu(x: torch.Tensor) -> torch.Tensor:
    """x / (1 + e^-x): crates/llm-backend/src/core/math.rs:223-225."""
    return x / (1.0 + torch.exp(-x))


def swiglu_mlp(x: torch.Tensor, gate_w: torch.Tensor, up_w: torch.Tensor, down_w: torch.Tensor) -> torch.Tensor:
    """down(silu(gate x) * (up x)): crates/llm-backend/src/core/math.rs:196-221,
    crates/llm-backend/src/core/qwen/ops/moe.rs:31-88."""
    return (silu(x @ gate_w.T) * (x @ up_w.T)) @ down_w.T


def attention_block(x, weights, prefix, cfg, positions, window):
    """q/k/v projections, per-head q/k RMSNorm before RoPE, attention, output projection.

    crates/llm-backend/src/core/qwen/ops/attention_full.rs:197-309 (order: project, norm
    q and k per head with the shared [d] weight :252-287, rotate at the absolute
    position :249,371-384, attend, o_proj); v is neither normed nor rotated.
    """
    T = x.shape[0]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps, theta = cfg["rms_norm_eps"], cfg["rope_theta"]
    q = (x @ weights[prefix + "q_proj.weight"].T).reshape(T, nq, d)
    k = (x @ weights[prefix + "k_proj.weight"].T).reshape(T, nkv, d)
    v = (x @ weights[prefix + "v_proj.weight"].T).reshape(T, nkv, d)
    q = rms_norm(q, weights[prefix + "q_norm.weight"], eps)
    k = rms_norm(k, weights[prefix + "k_norm.weight"], eps)
    q = rope(q, positions, theta)
    k = rope(k, positions, theta)
    mixed = causal_attention(q, k, v, window)
    return mixed.reshape(T, nq * d) @ weights[prefix + "o_proj.weight"].T


def decoder_layer(h, weights, layer, cfg, positions, window):
    """n1 = norm(h); a = attn(n1); n2 = norm(h + a); m = mlp(n2); out = h + a + m.

    crates/llm-backend/src/core/qwen/ops/decoder.rs:210-314.
    """
    base = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    n1 = rms_norm(h, weights[base + "input_layernorm.weight"], eps)
    a = attention_block(n1, weights, base + "self_attn.", cfg, positions, window)
    r = h + a
    n2 = rms_norm(r, weights[base + "post_attention_layernorm.weight"], eps)
    m = swiglu_mlp(
        n2,
        weights[base + "mlp.gate_proj.weight"],
        weights[base + "mlp.up_proj.weight"],
        weights[base + "mlp.down_proj.weight"],
    )
    return r + m


def layer_window(cfg, layer: int) -> Optional[int]:
    """Window of a layer: the reference windows every layer when enabled
    (crates/llm-backend/src/core/qwen/ops/cache.rs:116-121); ``max_window_layers`` (default 0)
    leaves the layers below it unwindowed."""
    if cfg.get("use_sliding_window") and layer >= cfg.get("max_window_layers", 0):
        return cfg["sliding_window"]
    return None


def normalise_config(config: dict) -> dict:
    cfg = dict(config)
    cfg.setdefault("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])
    return cfg


def forward_logits(config: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    """Logits [T, V] at every position of ``tokens`` (positions 0..T-1).

    Embedding row gather without scaling (crates/llm-backend/src/core/qwen/ops/embedding.rs:26-36),
    the layers in order, final RMSNorm and lm_head, which is the embedding table when
    ``tie_word_embeddings`` (crates/llm-backend/src/core/qwen/ops/lm_head.rs:68-86,
    crates/llm-models/src/qwen.rs:282-288).
    """
    cfg = normalise_config(config)
    table = weights["model.embed_tokens.weight"]
    for token in tokens:
        if not 0 <= token < cfg["vocab_size"]:
            raise ValueError(f"token id {token} outside vocab size {cfg['vocab_size']}")
    h = table[torch.tensor(list(tokens), dtype=torch.long)]
    positions = list(range(len(tokens)))
    for layer in range(cfg["num_hidden_layers"]):
        h = decoder_layer(h, weights, layer, cfg, positions, layer_window(cfg, layer))
    h = rms_norm(h, weights["model.norm.weight"], cfg["rms_norm_eps"])
    head = table if cfg.get("tie_word_embeddings", False) else weights["lm_head.weight"]
    return h @ head.T


# --------------------------------------------------------------------------- sampling
def argmax_first(logits: torch.Tensor) -> int:
    """Greatest logit, lowest index on ties: crates/llm-sampler/src/lib.rs:160-179."""
    best, best_value = 0, float(logits[0])
    for index in range(1, logits.shape[0]):
        if float(logits[index]) > best_value:
            best, best_value = index, float(logits[index])
    return best


def sample_top_p(logits: torch.Tensor, temperature: float, top_p: float, draw: float) -> int:
    """Nucleus sampling with a caller-supplied draw in [0, 1).

    crates/llm-sampler/src/lib.rs:39-108: p = softmax(logits / temperature) in 32-bit; sort
    by probability descending, ties to the lower index (:153-158); the nucleus is the
    shortest prefix whose sum reaches top_p (:110-151); threshold = draw * nucleus_total;
    the first entry whose running sum reaches the threshold is returned.
    """
    scaled = (logits.to(torch.float32) / np.float32(temperature))
    probs = torch.exp(scaled - scaled.max())
    probs = (probs / probs.sum()).numpy()
    order = sorted(range(len(probs)), key=lambda i: (-probs[i], i))
    total = np.float32(0.0)
    nucleus = len(order)
    for offset, index in enumerate(order):
        total = np.float32(total + probs[index])
        if total >= np.float32(top_p):
            nucleus = offset + 1
            break
    threshold = np.float32(draw) * total
    running = np.float32(0.0)
    for index in order[:nucleus]:
        running = np.float32(running + probs[index])
        if threshold <= running:
            return index
    return order[nucleus - 1]


def greedy_generate(config, weights, prompt: Sequence[int], new_tokens: int) -> List[int]:
    """Greedy continuation, every step recomputed from the whole sequence
    (loop shape: crates/llm-native-runtime/src/native_text/driver.rs:439-477)."""
    tokens = list(prompt)
    out: List[int] = []
    for _ in range(new_tokens):
        logits = forward_logits(config, weights, tokens)
        token = argmax_first(logits[-1])
        out.append(token)
        tokens.append(token)
    return out
