"""Plain Qwen3 dense decoder: whole sequences, no cache, one function per part.

This file rests on the formulas of the reference's files only (its code cannot
be compiled here: it needs a Rust toolchain and crates that are not present),
so every function cites the lines it restates.  All arithmetic is float64 on
the CPU except the rotation angle, which the reference defines in float32
(``src/model.rs:5992-5997``) and which is reproduced bit for bit here.

Inputs are a dict ``name -> torch.Tensor`` with the checkpoint's tensor names
and the raw ``config.json`` dict.
"""
from __future__ import annotations

import math

import numpy as np
import torch

DT = torch.float64


def embed(table: torch.Tensor, ids) -> torch.Tensor:
    """x[t, :] = E[ids[t], :], no scaling (src/training.rs:278-282)."""
    ids = torch.as_tensor(ids, dtype=torch.long)
    if ids.numel() and (int(ids.min()) < 0 or int(ids.max()) >= table.shape[0]):
        raise ValueError("token outside vocabulary")  # src/training.rs:267-270
    return table.to(DT)[ids]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x / sqrt(mean(x^2) + eps) * w over the last axis; the weight multiplies
    as it is (no +1), no bias, no mean-centring (src/training.rs:233-238,
    src/kernels.rs:316-341)."""
    x = x.to(DT)
    scale = torch.sqrt((x * x).mean(dim=-1, keepdim=True) + float(eps))
    return x / scale * w.to(DT)


def rope_inv_freq(head_dim: int, theta: float) -> np.ndarray:
    """inv_freq[j] = 1 / theta^(2j/D) in float32, computed on the host
    (src/model.rs:5992-5997: p = i/D for even i, inv = 1/powf(theta, p))."""
    i = np.arange(0, head_dim, 2, dtype=np.float32)
    p = i / np.float32(head_dim)
    return (np.float32(1.0) / np.power(np.float32(theta), p, dtype=np.float32)).astype(np.float32)


def rope_cos_sin(positions, head_dim: int, theta: float):
    """angle = float32(pos) * inv_freq[j], a float32 product (src/kernels.rs:3640-3648);
    its cosine and sine are then taken exactly (float64) here."""
    inv = rope_inv_freq(head_dim, theta)
    pos = np.asarray(positions, dtype=np.float32)[:, None]
    angle = (pos * inv[None, :]).astype(np.float32)  # one float32 rounding
    a64 = torch.from_numpy(angle.astype(np.float64))
    return torch.cos(a64), torch.sin(a64)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Half-split pairing: lo = x[..., :D/2], hi = x[..., D/2:];
    y_lo = lo*cos - hi*sin, y_hi = hi*cos + lo*sin (src/training.rs:240-252).
    ``x`` is [T, heads, D]; cos and sin are [T, D/2]."""
    half = x.shape[-1] // 2
    lo, hi = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([lo * c - hi * s, hi * c + lo * s], dim=-1)


def causal_attention(q, k, v, window=None) -> torch.Tensor:
    """q [T, nq, D], k and v [T, nkv, D] of one sequence starting at position 0.
    Query head h reads kv head h // (nq/nkv) (src/training.rs:296-300); scores are
    q.k / sqrt(D) (src/training.rs:334-335); key j is visible to query i when
    j <= i (src/kernels.rs:1190-1191 masks the rest), and, with a window W, when
    also j > i - W; softmax over the visible keys; o = P.V (src/training.rs:336-341)."""
    T, nq, D = q.shape
    nkv = k.shape[1]
    g = nq // nkv
    out = torch.empty(T, nq, D, dtype=DT)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    visible = j <= i
    if window is not None:
        visible = visible & (j > i - int(window))
    for h in range(nq):
        kh, vh = k[:, h // g, :], v[:, h // g, :]
        s = (q[:, h, :] @ kh.T) / math.sqrt(D)
        s = s.masked_fill(~visible, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ vh
    return out


def attention_block(x, w, prefix, cfg, positions, window=None) -> torch.Tensor:
    """Steps 2-12 of the attention half of a layer (src/training.rs:303-342):
    q, k, v projections without bias, per-head RMSNorm over head_dim with one
    weight vector shared by all heads, applied before the rotation, then rotation
    of q and k, causal GQA attention, concatenation of heads and o_proj."""
    nq, nkv, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    T = x.shape[0]
    q = (x @ w[prefix + "self_attn.q_proj.weight"].to(DT).T).reshape(T, nq, D)
    k = (x @ w[prefix + "self_attn.k_proj.weight"].to(DT).T).reshape(T, nkv, D)
    v = (x @ w[prefix + "self_attn.v_proj.weight"].to(DT).T).reshape(T, nkv, D)
    q = rms_norm(q, w[prefix + "self_attn.q_norm.weight"], cfg["rms_norm_eps"])
    k = rms_norm(k, w[prefix + "self_attn.k_norm.weight"], cfg["rms_norm_eps"])
    cos, sin = rope_cos_sin(positions, D, rope_theta(cfg))
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    o = causal_attention(q, k, v, window).reshape(T, nq * D)
    return o @ w[prefix + "self_attn.o_proj.weight"].to(DT).T


def swiglu(x, w_gate, w_up, w_down) -> torch.Tensor:
    """f = silu(x Wg^T) * (x Wu^T), silu(g) = g / (1 + exp(-g)); d = f Wd^T
    (src/training.rs:344-349, src/kernels.rs:285-295)."""
    g = x @ w_gate.to(DT).T
    u = x @ w_up.to(DT).T
    return ((g / (1.0 + torch.exp(-g))) * u) @ w_down.to(DT).T


def rope_theta(cfg: dict) -> float:
    """The rotation base stands in the ``rope_parameters`` object when the file
    has one, else at the top level (src/quantized_config.rs:66-70, 79-82)."""
    block = cfg.get("rope_parameters")
    if isinstance(block, dict) and "rope_theta" in block:
        return float(block["rope_theta"])
    return float(cfg["rope_theta"])


def layer_window(cfg: dict, layer: int):
    """Which layers look through a window: ``layer_types[layer]`` when the file
    names the kind of every layer (src/quantized_config.rs:116-125 reads that
    list), else ``use_sliding_window``, ``sliding_window`` and
    ``max_window_layers``: layers with index >= max_window_layers see only the
    last ``sliding_window`` keys.  The reference refuses windowed layers
    (src/model.rs:1323-1326); the rule is the documented meaning of those keys."""
    kinds = cfg.get("layer_types")
    if kinds:
        return int(cfg["sliding_window"]) if kinds[layer] == "sliding_attention" else None
    if not cfg.get("use_sliding_window", False):
        return None
    if layer < int(cfg.get("max_window_layers", cfg["num_hidden_layers"])):
        return None
    return int(cfg["sliding_window"])


def decoder_layer(x, w, layer: int, cfg, positions) -> torch.Tensor:
    """Pre-norm residual block: x += Attn(RMSNorm(x)); x += MLP(RMSNorm(x))
    (src/training.rs:303-349)."""
    p = f"model.layers.{layer}."
    n = rms_norm(x, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
    x = x + attention_block(n, w, p, cfg, positions, layer_window(cfg, layer))
    m = rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
    return x + swiglu(m, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                      w[p + "mlp.down_proj.weight"])


def hidden_states(w, cfg, tokens) -> torch.Tensor:
    """Embedding and all layers for one whole sequence at positions 0..T-1."""
    x = embed(w["model.embed_tokens.weight"], tokens)
    positions = list(range(len(tokens)))
    for layer in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, layer, cfg, positions)
    return x


def logits(w, cfg, tokens, rows=None) -> torch.Tensor:
    """Final RMSNorm and the output head at the wanted rows; the head is the
    embedding table when ``tie_word_embeddings`` (src/training.rs:350-362)."""
    x = hidden_states(w, cfg, tokens)
    if rows is not None:
        x = x[torch.as_tensor(rows, dtype=torch.long)]
    h = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return h @ head.to(DT).T


def greedy_generate(w, cfg, prompt, max_new_tokens: int, stop_ids=()):
    """Recomputes the whole prefix for every token.  The stop token is checked
    before it is pushed, so it is neither returned nor fed back
    (src/model.rs:2063, 2086-2089).  Ties go to the lowest index
    (src/model.rs:6075-6086)."""
    seq = list(prompt)
    out = []
    for _ in range(max_new_tokens):
        row = logits(w, cfg, seq, rows=[len(seq) - 1])[0]
        tok = int(torch.argmax(row))  # first maximum
        if tok in stop_ids:
            break
        out.append(tok)
        seq.append(tok)
    return out
