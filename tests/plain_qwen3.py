"""A plain, slow implementation of Qwen3 dense on the CPU, written from the reference's
formulas (ROCm/ATOM, paths within that project).  Whole sequences, no cache, no batching,
one function for each part.  It shares no code with ``atom_b200``: it reads config.json and
model.safetensors itself.

It rests on the formulas: the reference's own model code cannot be imported on this
platform (every arithmetic op is a call into the AMD-only ``aiter`` package).  The two
functions of the reference that are plain torch -- ``apply_rotary_emb``
(atom/model_ops/rotary_embedding.py:14-24) and ``SiluAndMul.forward_native``
(atom/model_ops/activation.py:78-82) -- are compared with this file once, see
tests/golden/make_golden.py.

Arithmetic is float64 by default, on the values stored in the checkpoint (bfloat16
weights widen exactly); rotation angles are formed in float32 as the reference forms them.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


# ----------------------------------------------------------------------------- loading


def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def read_tensors(model_dir: str, dtype=torch.float64) -> Dict[str, torch.Tensor]:
    from safetensors import safe_open

    out = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt", device="cpu") as f:
        for k in f.keys():
            out[k] = f.get_tensor(k).to(dtype)
    return out


# ----------------------------------------------------------------------------- parts


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w over the last dim.
    atom/model_ops/layernorm.py:57-63 (rmsnorm2d_fwd after reshape(-1, dim))."""
    var = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * w


def rope_cos_sin(positions: torch.Tensor, rotary_dim: int, theta: float):
    """inv_freq_j = 1 / theta^(2j/d); angle = pos * inv_freq_j, in float32.
    atom/model_ops/rotary_embedding.py:58-80 (_compute_inv_freq, _compute_cos_sin_cache)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))
    freqs = torch.einsum("i,j -> ij", positions.to(torch.float32), inv_freq)
    return freqs.cos(), freqs.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [T, heads, d].  Half-split pairing: y1 = x1 cos - x2 sin, y2 = x2 cos + x1 sin.
    atom/model_ops/rotary_embedding.py:14-24 (apply_rotary_emb)."""
    cos = cos.unsqueeze(-2).to(x.dtype)
    sin = sin.unsqueeze(-2).to(x.dtype)
    x1, x2 = torch.chunk(x, 2, dim=-1)
    return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     window: Optional[int] = None) -> torch.Tensor:
    """q: [T, nh, d], k, v: [T, nkv, d].  Query head h reads kv head h // (nh / nkv); query
    t sees keys j <= t (and j > t - window).  scale = d^-0.5 (atom/models/qwen3.py:88);
    causal softmax attention (atom/model_ops/attention_mha.py:751-765); window of W keys
    including the query's own (atom/model_ops/attention_mha.py:499-500)."""
    T, nh, d = q.shape
    nkv = k.shape[1]
    rep = nh // nkv
    out = torch.empty_like(q)
    idx = torch.arange(T)
    mask = idx[None, :] <= idx[:, None]
    if window is not None:
        mask &= idx[None, :] > idx[:, None] - window
    for h in range(nh):
        g = h // rep
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, g, :]
    return out


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    """silu(x[:, :I]) * x[:, I:].  atom/model_ops/activation.py:78-82 (forward_native)."""
    d = x.shape[-1] // 2
    g, u = x[..., :d], x[..., d:]
    return g * torch.sigmoid(g) * u


def attention_block(x, w, p: str, cfg: dict, positions, window) -> torch.Tensor:
    """atom/models/qwen3.py:140-163: qkv projection, split, per-head q/k norm, rotary,
    attention, output projection."""
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // nh      # atom/models/qwen3.py:85
    eps = cfg["rms_norm_eps"]
    T = x.shape[0]
    q = x @ w[f"{p}.q_proj.weight"].T
    k = x @ w[f"{p}.k_proj.weight"].T
    v = x @ w[f"{p}.v_proj.weight"].T
    if cfg.get("attention_bias"):
        q = q + w[f"{p}.q_proj.bias"]
        k = k + w[f"{p}.k_proj.bias"]
        v = v + w[f"{p}.v_proj.bias"]
    q = rms_norm(q.view(T, nh, hd), w[f"{p}.q_norm.weight"], eps)      # :159
    k = rms_norm(k.view(T, nkv, hd), w[f"{p}.k_norm.weight"], eps)     # :160
    cos, sin = rope_cos_sin(positions, hd, rope_theta(cfg))
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    o = causal_attention(q, k, v.view(T, nkv, hd), hd ** -0.5, window)
    return o.reshape(T, nh * hd) @ w[f"{p}.o_proj.weight"].T          # :162


def mlp_block(x, w, p: str) -> torch.Tensor:
    """atom/models/qwen3.py:194-198: gate_up, SiluAndMul, down."""
    gu = torch.cat((x @ w[f"{p}.gate_proj.weight"].T, x @ w[f"{p}.up_proj.weight"].T), dim=-1)
    return silu_and_mul(gu) @ w[f"{p}.down_proj.weight"].T


def rope_theta(cfg: dict) -> float:
    rp = cfg.get("rope_parameters")
    if isinstance(rp, dict) and "rope_theta" in rp:
        return float(rp["rope_theta"])
    return float(cfg["rope_theta"])


def layer_window(cfg: dict, i: int) -> Optional[int]:
    """atom/models/llama.py:187-200: a layer typed "sliding_attention" uses sliding_window."""
    lt = cfg.get("layer_types")
    if lt and lt[i] == "sliding_attention" and cfg.get("use_sliding_window", True):
        return cfg["sliding_window"]
    return None


def forward(cfg: dict, w: Dict[str, torch.Tensor], token_ids: Sequence[int]) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  atom/models/qwen3.py:289-313 (model),
    :248-258 (residual pattern: r = h + r; a = norm(r)), :355-360 (logits)."""
    dt = w["model.embed_tokens.weight"].dtype
    ids = torch.as_tensor(list(token_ids), dtype=torch.long)
    positions = torch.arange(len(ids))
    eps = cfg["rms_norm_eps"]
    r = w["model.embed_tokens.weight"][ids]                              # :297
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}"
        a = rms_norm(r, w[f"{p}.input_layernorm.weight"], eps)           # :248-252
        r = r + attention_block(a, w, f"{p}.self_attn", cfg, positions, layer_window(cfg, i))
        b = rms_norm(r, w[f"{p}.post_attention_layernorm.weight"], eps)  # :256
        r = r + mlp_block(b, w, f"{p}.mlp")
    y = rms_norm(r, w["model.norm.weight"], eps)                         # :310
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    return (y @ head.T).to(dt)                                            # :355-360, :339-340


# ----------------------------------------------------------------------------- sampling


def greedy(logits_row: torch.Tensor) -> int:
    """argmax, lowest index on ties (atom/model_ops/embed_head.py:272-275)."""
    return int(torch.argmax(logits_row))


def generate_greedy(cfg: dict, w, prompt: Sequence[int], n_new: int) -> List[int]:
    ids = list(prompt)
    out = []
    for _ in range(n_new):
        nxt = greedy(forward(cfg, w, ids)[-1])
        out.append(nxt)
        ids.append(nxt)
    return out


def _mix32(x: np.ndarray) -> np.ndarray:
    """The 32-bit finaliser used by the engine's sampling noise (written out here again)."""
    x = x.astype(np.uint64)
    x ^= x >> np.uint64(16)
    x = (x * np.uint64(0x7FEB352D)) & np.uint64(0xFFFFFFFF)
    x ^= x >> np.uint64(15)
    x = (x * np.uint64(0x846CA68B)) & np.uint64(0xFFFFFFFF)
    x ^= x >> np.uint64(16)
    return x


def exponential_noise(seed: int, index: int, vocab: int) -> np.ndarray:
    """E_v ~ Exp(1) for every vocabulary entry, a pure function of (seed, index, v)."""
    v = np.arange(vocab, dtype=np.uint64)
    k = _mix32(np.uint64(seed & 0xFFFFFFFF) ^ _mix32(np.uint64(index & 0xFFFFFFFF) + np.uint64(0x9E3779B9)))
    bits = _mix32((v + np.uint64(1)) * np.uint64(0x9E3779B1) & np.uint64(0xFFFFFFFF) ^ k)
    u = ((bits >> np.uint64(8)).astype(np.float64) + 0.5) / 16777216.0
    return -np.log(u)


def sample_temperature(logits_row: torch.Tensor, temperature: float, seed: int, index: int,
                       top_k: int = -1, top_p: float = 1.0) -> int:
    """argmax_v softmax(logits / T)_v / E_v, the exponential race of
    atom/model_ops/sampler.py:104-132 and :304-310; top-k / top-p keep, in descending order of
    probability, the first k entries and those before the cumulative mass passes p
    (atom/model_ops/sampler.py:262-283), and the race runs among the kept."""
    if temperature == 0.0:
        return greedy(logits_row)
    x = logits_row.double().numpy() / temperature
    x = x - x.max()
    p = np.exp(x) / np.exp(x).sum()
    keep = np.ones_like(p, dtype=bool)
    if top_k != -1 or top_p < 1.0:
        order = np.argsort(-p, kind="stable")
        sp = p[order]
        csum = np.cumsum(sp)
        kmask = np.ones_like(sp, dtype=bool)
        if top_p < 1.0:
            kmask &= (csum - sp) <= top_p
        if top_k != -1:
            kmask &= np.arange(len(sp)) < top_k
        kmask[0] = True
        keep = np.zeros_like(keep)
        keep[order[kmask]] = True
    e = exponential_noise(seed, index, len(p))
    score = np.where(keep, np.log(np.maximum(p, 1e-300)) - np.log(e), -np.inf)
    return int(np.argmax(score))
