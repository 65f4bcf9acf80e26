"""Independent restatement of the model forward (logits only) in NumPy float64.

The V1 stage needs an oracle that shares no code with ``model.forward``: the reference keeps a
plain-PyTorch copy of its JAX forward for that (``prometheus/verify/_torch_forward.py:427-476``).
The model here already is PyTorch, so the second statement is written against NumPy instead, in
the most literal form of each definition:

* the delta rule is the per-token recurrence ``S <- (I - b k k^T) S + b k v^T``, ``o = q S``
  (no chunking, no WY transform);
* softmax attention loops over heads and masks by index comparison;
* the MoE loops over tokens and applies each chosen expert to that one token (no sort, no
  grouping), with the same stable tie-break (lower expert index first) and rack limit;
* RoPE rotates interleaved (even, odd) pairs with explicit angles.

Nothing is imported from the package except the config accessors that say which kind a layer is.
"""
from __future__ import annotations

import math

import numpy as np

from .. import model as _m


def _np(t) -> np.ndarray:
    return np.asarray(t.detach().cpu().numpy() if hasattr(t, "detach") else t, dtype=np.float64)


def _rms(x, w, eps=1e-6):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


def _silu(x):
    return x / (1.0 + np.exp(-x))


def _sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def _rotate(x, positions, n_rot, base):
    """x: (S, D); the first ``n_rot`` interleaved pairs are rotated by position * base^(-2i/(2 n_rot))."""
    out = x.copy()
    for i in range(n_rot):
        freq = float(base) ** (-2.0 * i / (2.0 * n_rot))
        c, s = np.cos(positions * freq), np.sin(positions * freq)
        e, o = x[:, 2 * i], x[:, 2 * i + 1]
        out[:, 2 * i], out[:, 2 * i + 1] = e * c - o * s, e * s + o * c
    return out


def _causal_softmax_attention(q, k, v):
    """q: (S, D), k: (S, D), v: (S, Dv) for one head."""
    s = q.shape[0]
    scores = q @ k.T / math.sqrt(q.shape[1])
    scores[np.triu_indices(s, 1)] = -1e9
    scores -= scores.max(axis=-1, keepdims=True)
    p = np.exp(scores)
    return (p / p.sum(axis=-1, keepdims=True)) @ v


def _delta_layer(x, layer):
    wq, wk, wv, wo = (_np(layer[n]) for n in ("W_q", "W_k", "W_v", "W_o"))
    wb = _np(layer["W_beta"]) if "W_beta" in layer else None
    s_len, heads, d = x.shape[0], wq.shape[1], wq.shape[2]
    y = np.zeros_like(x)
    for h in range(heads):
        q, k, v = x @ wq[:, h], x @ wk[:, h], x @ wv[:, h]
        q = q / np.maximum(np.sqrt((q * q).sum(-1, keepdims=True)), 1e-6)
        k = k / np.maximum(np.sqrt((k * k).sum(-1, keepdims=True)), 1e-6)
        beta = _sigmoid(x @ wb[:, h]) if wb is not None else np.ones(s_len)
        state = np.zeros((d, d))
        o = np.zeros((s_len, d))
        for t in range(s_len):
            state = state - beta[t] * np.outer(k[t], k[t] @ state) + beta[t] * np.outer(k[t], v[t])
            o[t] = q[t] @ state
        y += o @ wo[h]
    return y


def _gqa_layer(x, layer, positions, base):
    wq, wk, wv, wo = (_np(layer[n]) for n in ("W_q", "W_k", "W_v", "W_o"))
    hq, hkv, d = wq.shape[1], wk.shape[1], wq.shape[2]
    y = np.zeros_like(x)
    for h in range(hq):
        g = h // (hq // hkv)
        q = _rotate(x @ wq[:, h], positions, d // 2, base)
        k = _rotate(x @ wk[:, g], positions, d // 2, base)
        y += _causal_softmax_attention(q, k, x @ wv[:, g]) @ wo[h]
    return y


def _mla_layer(x, layer, positions, base):
    wq, wo = _np(layer["W_q"]), _np(layer["W_o"])
    ckv = x @ _np(layer["W_kv_compress"])
    k_up = _np(layer["W_kv_up"])
    rk = x @ _np(layer["W_rope_k"])
    rk = _rotate(rk, positions, rk.shape[1] // 2, base)
    y = np.zeros_like(x)
    for h in range(wq.shape[1]):
        k_nope = ckv @ k_up[:, h]
        d_nope = k_nope.shape[1]
        q = x @ wq[:, h]
        q = np.concatenate([q[:, :d_nope], _rotate(q[:, d_nope:], positions, (q.shape[1] - d_nope) // 2, base)], axis=1)
        k = np.concatenate([k_nope, rk], axis=1)
        ones = np.ones(q.shape[1])
        y += _causal_softmax_attention(_rms(q, ones), _rms(k, ones), k_nope) @ wo[h]
    return y


def _choose_experts(scores, top_k, max_racks):
    n_exp = scores.shape[0]
    order = sorted(range(n_exp), key=lambda e: (-scores[e], e))
    n_racks = max(min(max_racks, n_exp), 1)
    if n_racks <= max_racks:
        return order[:top_k]
    rack = [min(e * n_racks // n_exp, n_racks - 1) for e in range(n_exp)]
    used, chosen = set(), []
    for e in order:
        if len(chosen) < top_k and (rack[e] in used or len(used) < max_racks):
            chosen.append(e)
            used.add(rack[e])
    for e in order:
        if len(chosen) >= top_k:
            break
        if e not in chosen:
            chosen.append(e)
    return chosen[:top_k]


def _swiglu(x, wg, wu, wd):
    return (_silu(x @ wg) * (x @ wu)) @ wd


def _moe_layer(x, layer, cfg):
    router = _np(layer["router"])
    bias = _np(layer["router_bias"]) if layer.get("router_bias") is not None else None
    rg, ru, rd = (_np(layer[n]) for n in ("routed_gate", "routed_up", "routed_down"))
    sg, su, sd = (_np(layer[n]) for n in ("shared_gate", "shared_up", "shared_down"))
    y = np.zeros_like(x)
    for t in range(x.shape[0]):
        probs = _sigmoid(x[t] @ router)
        # selection happens on float32 scores in the model; rounding the scores the same way keeps
        # near-ties on the same side
        sel = (probs if bias is None else probs + bias).astype(np.float32)
        ids = _choose_experts(sel, cfg.top_k, cfg.max_racks)
        total = max(sum(probs[e] for e in ids), 1e-9)
        for e in ids:
            y[t] += probs[e] / total * _swiglu(x[t], rg[e], ru[e], rd[e])
        for j in range(sg.shape[0]):
            y[t] += _swiglu(x[t], sg[j], su[j], sd[j])
    return y


def _block(h, layer, cfg, index, positions):
    n = _rms(h, _np(layer["pre_attn_norm"]))
    kind = _m.attention_kind(index, cfg)
    if kind is _m.AttentionKind.LINEAR:
        h = h + _delta_layer(n, layer)
    elif kind is _m.AttentionKind.GQA:
        h = h + _gqa_layer(n, layer, positions, cfg.rope_base)
    else:
        h = h + _mla_layer(n, layer, positions, cfg.rope_base)
    n = _rms(h, _np(layer["pre_ffn_norm"]))
    if _m.ffn_kind(index, cfg) is _m.FfnKind.DENSE:
        return h + _swiglu(n, _np(layer["ffn_gate"]), _np(layer["ffn_up"]), _np(layer["ffn_down"]))
    return h + _moe_layer(n, layer, cfg)


def forward_logits(tokens, params, cfg, r: int = 1) -> np.ndarray:
    """(batch, seq, vocab) float64 logits for ``r`` iterations of the core block."""
    tokens = np.asarray(tokens.cpu().numpy() if hasattr(tokens, "cpu") else tokens)
    prelude, core, coda = _m._recurrent_split(cfg)
    embed, unembed = _np(params["embed"]), _np(params["unembed"])
    layers = params["layers"]
    out = np.zeros((tokens.shape[0], tokens.shape[1], unembed.shape[0]))
    positions = np.arange(tokens.shape[1], dtype=np.float64)
    for b in range(tokens.shape[0]):
        h = embed[tokens[b]]
        for i in range(prelude):
            h = _block(h, layers[i], cfg, i, positions)
        injected = h
        for it in range(r):
            if it:
                h = h + injected
            for i in range(prelude, prelude + core):
                h = _block(h, layers[i], cfg, i, positions)
        for i in range(prelude + core, prelude + core + coda):
            h = _block(h, layers[i], cfg, i, positions)
        out[b] = _rms(h, _np(params["final_norm"])) @ unembed.T
    return out
