"""Plain, slow, whole-sequence implementation of the dense GQA decoder.

This file is the oracle of the test-suite.  It shares no code with
``helios_b200``: it reads the raw ``config.json`` dictionary and a dictionary of
checkpoint tensors (HF names), runs every sequence whole, keeps no cache, and
has one function per part.  Each function cites the place in the reference
project (paths inside anish41338/helios) whose formula it restates.

Two formulas have no counterpart in the reference and rest on the published
definition of the configuration keys only: the ``llama3`` rope scaling and the
sliding window (``use_sliding_window`` / ``max_window_layers``).  A comparison of
this file with the reference's own model code, run once on the CPU, lives in
``tests/golden/``.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """python/helios/exec/model.py:109-114 -- mean of squares over the last
    dimension, rsqrt(var + eps), then the weight; no mean subtraction, no bias."""
    var = x.pow(2).mean(-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * weight


def rope_inv_freq(head_dim: int, theta: float, scaling: Optional[dict],
                  dtype=torch.float64) -> torch.Tensor:
    """python/helios/exec/model.py:127-129 -- inv_freq[j] = theta^(-2j/head_dim).

    With ``rope_scaling`` of type ``llama3`` (absent from the reference; the
    definition of the keys factor / low_freq_factor / high_freq_factor /
    original_max_position_embeddings): wavelengths shorter than P/high keep their
    frequency, longer than P/low are divided by factor, and those between are
    interpolated linearly in (P/wavelength - low)/(high - low)."""
    j = torch.arange(0, head_dim, 2, dtype=torch.float64)
    inv = 1.0 / (float(theta) ** (j / head_dim))
    kind = None
    if scaling:
        kind = scaling.get("rope_type", scaling.get("type"))
    if kind in (None, "default"):
        return inv.to(dtype)
    assert kind == "llama3", kind
    f = float(scaling["factor"])
    lo = float(scaling["low_freq_factor"])
    hi = float(scaling["high_freq_factor"])
    P = float(scaling["original_max_position_embeddings"])
    out = inv.clone()
    for i in range(inv.numel()):
        wavelen = 2.0 * math.pi / float(inv[i])
        if wavelen < P / hi:
            continue
        if wavelen > P / lo:
            out[i] = inv[i] / f
        else:
            s = (P / wavelen - lo) / (hi - lo)
            out[i] = (1.0 - s) * inv[i] / f + s * inv[i]
    return out.to(dtype)


def apply_rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """python/helios/exec/model.py:130-132,148-153 -- angle = position * inv_freq;
    rotate-half convention: the two halves of the head dimension form the pairs.
    x: [n, heads, head_dim]."""
    ang = positions.to(inv_freq.dtype)[:, None] * inv_freq[None, :]
    c = ang.cos()[:, None, :].to(x.dtype)
    s = ang.sin()[:, None, :].to(x.dtype)
    x1, x2 = x.chunk(2, dim=-1)
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                     scale: float, window: Optional[int]) -> torch.Tensor:
    """python/helios/exec/paged_attn.py:248-261 (each KV head serves
    n_heads/n_kv_heads consecutive query heads) and :391-408 (scores = q.k^T *
    scale, key position > query position masked to -inf, softmax, times V).
    With a window W a query at position i also does not see keys at positions
    <= i - W (not in the reference).  q: [n, nh, hd]; k, v: [n, nkv, hd]."""
    n, nh, hd = q.shape
    nkv = k.shape[1]
    rep = nh // nkv
    k = k[:, :, None, :].expand(n, nkv, rep, hd).reshape(n, nh, hd)
    v = v[:, :, None, :].expand(n, nkv, rep, hd).reshape(n, nh, hd)
    scores = torch.einsum("qhd,khd->hqk", q, k) * scale
    qi = torch.arange(n)[:, None]
    kj = torch.arange(n)[None, :]
    mask = kj > qi
    if window is not None:
        mask = mask | (kj <= qi - window)
    scores = scores.masked_fill(mask[None], float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    return torch.einsum("hqk,khd->qhd", probs, v)


def swiglu(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor,
           w_down: torch.Tensor) -> torch.Tensor:
    """python/helios/exec/model.py:336-337 -- down(silu(gate(x)) * up(x)), no biases."""
    g = x @ w_gate.T
    u = x @ w_up.T
    return (g * torch.sigmoid(g) * u) @ w_down.T


def layer_windows(cfg: dict) -> List[Optional[int]]:
    """Which layers see only a window of keys.  Not in the reference; by the
    meaning of the configuration keys: with ``use_sliding_window`` the layers
    from ``max_window_layers`` on use ``sliding_window``; an explicit
    ``layer_types`` list wins."""
    L = cfg["num_hidden_layers"]
    W = cfg.get("sliding_window")
    if cfg.get("layer_types") is not None:
        return [W if t == "sliding_attention" else None for t in cfg["layer_types"]]
    if not cfg.get("use_sliding_window", False) or W is None:
        return [None] * L
    first = cfg.get("max_window_layers", L)
    return [W if i >= first else None for i in range(L)]


def has_qkv_bias(cfg: dict) -> bool:
    """python/helios/exec/model.py:79-92 -- ``attention_bias`` if given, else true
    for the qwen2 family."""
    if "attention_bias" in cfg:
        return bool(cfg["attention_bias"])
    mt = str(cfg.get("model_type", "")).lower()
    archs = " ".join(cfg.get("architectures", [])).lower()
    return mt.startswith("qwen2") or "qwen2" in archs


def decoder_layer(cfg: dict, w: Dict[str, torch.Tensor], i: int, h: torch.Tensor,
                  positions: torch.Tensor, inv_freq: torch.Tensor,
                  window: Optional[int]) -> torch.Tensor:
    """python/helios/exec/model.py:373-392 -- pre-norm block: x + attn(norm(x)),
    then x + mlp(norm(x)); projections of :236-251."""
    p = f"model.layers.{i}."
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nh)
    hd = cfg.get("head_dim") or cfg["hidden_size"] // nh
    eps = cfg.get("rms_norm_eps", 1e-5)
    n = h.shape[0]

    x = rms_norm(h, w[p + "input_layernorm.weight"], eps)
    q = x @ w[p + "self_attn.q_proj.weight"].T
    k = x @ w[p + "self_attn.k_proj.weight"].T
    v = x @ w[p + "self_attn.v_proj.weight"].T
    if has_qkv_bias(cfg):
        q = q + w[p + "self_attn.q_proj.bias"]
        k = k + w[p + "self_attn.k_proj.bias"]
        v = v + w[p + "self_attn.v_proj.bias"]
    q = apply_rope(q.view(n, nh, hd), positions, inv_freq)
    k = apply_rope(k.view(n, nkv, hd), positions, inv_freq)
    v = v.view(n, nkv, hd)
    a = causal_attention(q, k, v, 1.0 / math.sqrt(hd), window)
    h = h + a.reshape(n, nh * hd) @ w[p + "self_attn.o_proj.weight"].T

    x = rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
    h = h + swiglu(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                   w[p + "mlp.down_proj.weight"])
    return h


def forward_logits(cfg: dict, weights: Dict[str, torch.Tensor], token_ids: List[int],
                   dtype=torch.float64) -> torch.Tensor:
    """python/helios/exec/model.py:498-521 -- embedding, every layer, final norm,
    output head at every position; tied head per python/helios/exec/loader.py:126-130.
    Returns [len(token_ids), vocab] in ``dtype``."""
    w = {k: t.to(dtype) for k, t in weights.items()}
    nh = cfg["num_attention_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // nh
    inv_freq = rope_inv_freq(hd, cfg.get("rope_theta", 10000.0), cfg.get("rope_scaling"), dtype)
    tokens = torch.tensor(token_ids, dtype=torch.long)
    positions = torch.arange(len(token_ids))
    h = w["model.embed_tokens.weight"][tokens]
    windows = layer_windows(cfg)
    for i in range(cfg["num_hidden_layers"]):
        h = decoder_layer(cfg, w, i, h, positions, inv_freq, windows[i])
    h = rms_norm(h, w["model.norm.weight"], cfg.get("rms_norm_eps", 1e-5))
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    assert "lm_head.weight" in w or cfg.get("tie_word_embeddings", False)
    return h @ head.T


def greedy_generate(cfg: dict, weights: Dict[str, torch.Tensor], prompt: List[int],
                    n_new: int, dtype=torch.float64) -> List[int]:
    """python/helios/exec/sampler.py:51-52 -- argmax of the last position's logits,
    the whole sequence run again for every new token."""
    toks = list(prompt)
    out = []
    for _ in range(n_new):
        t = int(torch.argmax(forward_logits(cfg, weights, toks, dtype)[-1]))
        out.append(t)
        toks.append(t)
    return out


def sample_reference(logits: torch.Tensor, temperature: float, top_k: int, top_p: float,
                     u: float) -> int:
    """python/helios/exec/sampler.py:54-81 -- logits/T; top-k keeps logits >= the
    k-th largest; top-p sorts descending and drops the tokens after the one whose
    cumulative probability crosses top_p; then softmax.  The draw itself is made
    here by inverse CDF over token ids from a given uniform ``u`` (the reference
    draws with torch.multinomial from a CPU generator)."""
    l = logits.double() / temperature
    if top_k > 0:
        k = min(top_k, l.numel())
        kth = torch.topk(l, k).values[-1]
        l = torch.where(l < kth, torch.full_like(l, float("-inf")), l)
    if top_p < 1.0:
        sl, si = torch.sort(l, descending=True)
        cum = torch.cumsum(torch.softmax(sl, -1), -1)
        cut = cum > top_p
        cut = torch.cat([torch.zeros(1, dtype=torch.bool), cut[:-1]])
        sl = sl.masked_fill(cut, float("-inf"))
        l = torch.full_like(l, float("-inf")).scatter(0, si, sl)
    probs = torch.softmax(l, -1)
    cdf = torch.cumsum(probs, -1)
    idx = int(torch.searchsorted(cdf, torch.tensor(u * float(cdf[-1]), dtype=cdf.dtype), right=True))
    return min(idx, l.numel() - 1)
