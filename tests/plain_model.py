"""A plain, slow implementation of MiniMax-M2 for whole sequences, without a cache.

It rests on the formulas of the reference's Rust source (each function cites
file:line); the reference's own model code is Rust and cannot be compiled here
(no cargo/rustc, no crates), so there is no golden output of the reference to
compare with.  One function per part; numpy only; it shares no code with the
package under test and reads model folders with the small reader below.

Arithmetic is done in ``dtype`` (float64 by default, so that it is the more
exact side of every comparison; float32 repeats the reference's precision).
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np


# --------------------------------------------------------------------------- files

def read_safetensors(path):
    """name -> numpy array (bfloat16 widened to float32).  Format: u64 header length, JSON header, data."""
    with open(path, "rb") as handle:
        (n,) = struct.unpack("<Q", handle.read(8))
        header = json.loads(handle.read(n).decode("utf-8"))
        data = handle.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        begin, end = info["data_offsets"]
        raw = data[begin:end]
        tag = info["dtype"]
        if tag == "BF16":
            bits = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            arr = bits.view(np.float32)
        elif tag == "F32":
            arr = np.frombuffer(raw, dtype="<f4")
        elif tag == "F16":
            arr = np.frombuffer(raw, dtype="<f2").astype(np.float32)
        elif tag == "I32":
            arr = np.frombuffer(raw, dtype="<i4")
        else:
            raise ValueError(f"{path}: dtype {tag} of {name}")
        out[name] = arr.reshape(info["shape"]).copy()
    return out


def read_model_folder(folder):
    with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as handle:
        config = json.load(handle)
    return config, read_safetensors(os.path.join(folder, "model.safetensors"))


def sizes_from_config(c):
    """The sizes with the reference's defaults (src/convert.rs:1209-1219, 610-615)."""
    nh = c["num_attention_heads"]
    d = c["hidden_size"]
    hd = c.get("head_dim") or d // nh
    nested = c.get("rope_parameters") or {}
    # the rotated share of a head: a count, or a factor at the top level or beside theta under rope_parameters
    # (src/convert.rs:965-966 turns a factor into int(head_dim * factor); :610-615 looks under rope_parameters)
    if c.get("rotary_dim") is not None:
        rotary = c["rotary_dim"]
    elif c.get("partial_rotary_factor") is not None:
        rotary = int(hd * c["partial_rotary_factor"])
    elif nested.get("partial_rotary_factor") is not None:
        rotary = int(hd * nested["partial_rotary_factor"])
    else:
        rotary = hd
    theta = c.get("rope_theta")
    if theta is None:
        theta = nested.get("rope_theta", 10000.0)
    return dict(
        layers=c["num_hidden_layers"], d=d, nh=nh, nkv=c.get("num_key_value_heads") or nh, hd=hd, rotary=rotary,
        theta=float(theta), eps=float(c.get("rms_norm_eps", 1e-6)), qk_norm=bool(c.get("use_qk_norm", True)),
        experts=c.get("num_local_experts") or c["num_experts"], top_k=c["num_experts_per_tok"],
        width=c["intermediate_size"], vocab=c["vocab_size"], tied=bool(c.get("tie_word_embeddings", False)),
        routing_bias=bool(c.get("use_routing_bias", True)),
    )


# --------------------------------------------------------------------------- parts

def rms_norm(x, weight, eps):
    """x * rsqrt(mean(x^2) + eps) * w per row; the weight is used as it is (src/minimax.rs:56-66)."""
    ms = np.mean(x * x, axis=-1, keepdims=True)
    return x * (1.0 / np.sqrt(ms + eps)) * weight


def rotary_inverse_frequencies(theta, rotary_dim, dtype):
    """inv[j] = 1 / theta^(2j / rotary_dim), j < rotary_dim/2 (src/minimax.rs:50; partial: src/qwen35moe.rs:81)."""
    j = np.arange(rotary_dim // 2, dtype=dtype)
    return (1.0 / np.power(dtype(theta), 2.0 * j / dtype(rotary_dim))).astype(dtype)


def rotary(x, num_heads, head_dim, rotary_dim, theta, positions):
    """Rotate pairs (j, j + rotary_dim/2) of the first rotary_dim dims of every head by pos * inv[j];
    the other dims pass through (src/minimax.rs:69-84 with rotary_dim = head_dim; src/qwen35moe.rs:121-138)."""
    dtype = x.dtype.type
    out = x.copy()
    half = rotary_dim // 2
    if half == 0:
        return out
    inv = rotary_inverse_frequencies(theta, rotary_dim, dtype)
    angle = positions.astype(dtype)[:, None] * inv[None, :]            # [T, half]
    cos, sin = np.cos(angle), np.sin(angle)
    for head in range(num_heads):
        base = head * head_dim
        a = x[:, base:base + half]
        b = x[:, base + half:base + 2 * half]
        out[:, base:base + half] = a * cos - b * sin
        out[:, base + half:base + 2 * half] = b * cos + a * sin
    return out


def softmax_rows(scores):
    """exp(s - max) / sum per row (src/minimax.rs:33-40)."""
    m = np.max(scores, axis=-1, keepdims=True)
    e = np.exp(scores - m)
    return e / np.sum(e, axis=-1, keepdims=True)


def causal_attention(q, k, v, num_heads, num_kv_heads, head_dim, scale, window=None, rows=None):
    """Per query head h with kv = h // (nh / nkv): scores = q_h k_kv^T * scale, -1e30 where j > i,
    softmax, times v_kv (src/minimax.rs:141-154).  ``window`` (not in the reference's MiniMax) hides keys
    with j <= i - window.  ``rows``: compute these query rows only (q then holds just them; k and v hold every
    position), for sequences too long for the square of scores."""
    T = k.shape[0]
    rep = num_heads // num_kv_heads
    i = (np.arange(T) if rows is None else np.asarray(rows))[:, None]
    out = np.zeros((len(i), num_heads * head_dim), dtype=q.dtype)
    j = np.arange(T)[None, :]
    hidden = j > i
    if window is not None:
        hidden = hidden | (j <= i - window)
    for head in range(num_heads):
        kv = head // rep
        qh = q[:, head * head_dim:(head + 1) * head_dim]
        kh = k[:, kv * head_dim:(kv + 1) * head_dim]
        vh = v[:, kv * head_dim:(kv + 1) * head_dim]
        scores = (qh @ kh.T) * q.dtype.type(scale)
        scores[hidden] = -1e30
        out[:, head * head_dim:(head + 1) * head_dim] = softmax_rows(scores) @ vh
    return out


def attention_layer(a, W, prefix, s, positions, rows=None):
    """q/k/v projections without bias, full-width q/k RMSNorm, rotary, attention, output projection
    (src/minimax.rs:135-155).  Linear weights are (out, in) as in the checkpoint.  ``rows``: the output of
    these positions only."""
    q = a @ W[prefix + "self_attn.q_proj.weight"].T
    k = a @ W[prefix + "self_attn.k_proj.weight"].T
    v = a @ W[prefix + "self_attn.v_proj.weight"].T
    if s["qk_norm"]:
        q = rms_norm(q, W[prefix + "self_attn.q_norm.weight"], s["eps"])     # one RMS over all nh*hd
        k = rms_norm(k, W[prefix + "self_attn.k_norm.weight"], s["eps"])     # one RMS over all nkv*hd
    q = rotary(q, s["nh"], s["hd"], s["rotary"], s["theta"], positions)
    k = rotary(k, s["nkv"], s["hd"], s["rotary"], s["theta"], positions)
    if rows is not None:
        q = q[np.asarray(rows)]
    out = causal_attention(q, k, v, s["nh"], s["nkv"], s["hd"], float(s["hd"]) ** -0.5, rows=rows)
    return out @ W[prefix + "self_attn.o_proj.weight"].T


def route(a2, router_weight, choice_bias, top_k, forced_ids=None):
    """sigmoid scores; choice = score + bias; experts in descending choice, ties to the lower id (a stable
    sort); the first top_k; weights = score / sum of picked scores (src/minimax.rs:90-104).
    Returns (ids [T, k] in rank order, weights [T, k], margin [T] between the k-th and the next choice).
    With ``forced_ids`` the choice is given (the weights still come from the scores): this makes the model a
    continuous function of its inputs, for comparisons that must not hinge on a near tie."""
    logits = a2 @ router_weight.T
    score = 1.0 / (1.0 + np.exp(-logits))
    choice = score + choice_bias
    order = np.argsort(-choice, axis=-1, kind="stable")
    ids = order[:, :top_k] if forced_ids is None else np.asarray(forced_ids, dtype=np.int64)
    picked = np.take_along_axis(score, ids, axis=-1)
    weights = picked / np.sum(picked, axis=-1, keepdims=True)
    ranked = np.take_along_axis(choice, order, axis=-1)
    if ranked.shape[1] > top_k:
        margin = ranked[:, top_k - 1] - ranked[:, top_k]
    else:
        margin = np.full(ranked.shape[0], np.inf)
    return ids, weights, margin


def silu(x):
    """x / (1 + exp(-x)) (src/minimax.rs:31)."""
    return x / (1.0 + np.exp(-x))


def expert_swiglu(rows, w_gate, w_up, w_down):
    """silu(r W1^T) * (r W3^T), then W2 (src/minimax.rs:116-120)."""
    return (silu(rows @ w_gate.T) * (rows @ w_up.T)) @ w_down.T


def routed_experts(a2, W, prefix, s, forced_ids=None, return_ids=False):
    """out[t] = sum over the picked experts, in rank order, of weight * expert(a2[t]) (src/minimax.rs:88-126)."""
    moe = prefix + "block_sparse_moe."
    bias = W[moe + "e_score_correction_bias"] if s.get("routing_bias", True) else 0.0
    own_ids, _, margin = route(a2, W[moe + "gate.weight"], bias, s["top_k"])
    ids, weights, _ = route(a2, W[moe + "gate.weight"], bias, s["top_k"], forced_ids)
    out = np.zeros_like(a2)
    for t in range(a2.shape[0]):
        for rank in range(s["top_k"]):
            e = int(ids[t, rank])
            y = expert_swiglu(a2[t:t + 1], W[f"{moe}experts.{e}.w1.weight"], W[f"{moe}experts.{e}.w3.weight"],
                              W[f"{moe}experts.{e}.w2.weight"])
            out[t] += weights[t, rank] * y[0]
    if return_ids:
        return out, margin, own_ids
    return out, margin


# --------------------------------------------------------------------------- whole model

def cast_weights(W, dtype):
    return {k: (v.astype(dtype) if v.dtype.kind == "f" else v) for k, v in W.items()}


def hidden_states(config, W, ids, dtype=np.float64, return_margins=False, forced_routes=None, return_routes=False):
    """All layers on a whole sequence starting at position 0, final norm included (src/minimax.rs:128-160).
    ``forced_routes[layer]`` ([T, k] expert ids) replaces the router's choice in that layer."""
    s = sizes_from_config(config)
    W = cast_weights(W, dtype)
    positions = np.arange(len(ids))
    x = W["model.embed_tokens.weight"][np.asarray(ids, dtype=np.int64)]          # no multiplier, :132
    margins, routes = [], []
    for layer in range(s["layers"]):
        p = f"model.layers.{layer}."
        a = rms_norm(x, W[p + "input_layernorm.weight"], s["eps"])
        x = x + attention_layer(a, W, p, s, positions)
        a2 = rms_norm(x, W[p + "post_attention_layernorm.weight"], s["eps"])
        forced = None if forced_routes is None else forced_routes[layer]
        y, margin, own = routed_experts(a2, W, p, s, forced, return_ids=True)
        margins.append(margin)
        routes.append(own)
        x = x + y
    out = rms_norm(x, W["model.norm.weight"], s["eps"])
    if return_routes:
        return out, np.stack(margins), np.stack(routes)
    return (out, np.stack(margins)) if return_margins else out


def logits_all_positions(config, W, ids, dtype=np.float64):
    """Logits [T, vocab] of every position of a whole sequence.  The reference projects the last row only
    (src/minimax.rs:373-376); every row is the same product."""
    s = sizes_from_config(config)
    xf = hidden_states(config, W, ids, dtype)
    head = W["model.embed_tokens.weight"] if s["tied"] else W["lm_head.weight"]
    return xf @ head.astype(dtype).T


def greedy_pick(logits_row):
    """The largest logit; on an exact tie the last index, as Rust's max_by returns (src/minimax.rs:375)."""
    row = np.asarray(logits_row)
    best = np.max(row)
    return int(np.flatnonzero(row == best)[-1])


def temperature_pick(logits_row, temperature, uniform):
    """Inverse-CDF sample of softmax(logits / temperature) with one uniform number in [0, 1): the first
    index whose cumulative probability exceeds uniform.  (Not in the reference, which is greedy only.)"""
    row = np.asarray(logits_row, dtype=np.float64) / float(temperature)
    p = np.exp(row - np.max(row))
    c = np.cumsum(p)
    idx = int(np.searchsorted(c, uniform * c[-1], side="right"))
    return min(idx, len(row) - 1)


def sampling_floor(logits_row, temperature, top_k=0, top_p=1.0):
    """The smallest logit that may be sampled: the top_k-th largest (top_k > 0), or the one with which the
    probabilities of softmax(logits / temperature), taken in descending order, first add up to top_p
    (top_p < 1), whichever is larger; -inf when neither cuts.  (Not in the reference, which is greedy only.)"""
    row = np.asarray(logits_row, dtype=np.float64)
    ordered = np.sort(row)[::-1]
    floor = -np.inf
    if top_k > 0:
        floor = max(floor, ordered[min(top_k, len(row)) - 1])
    if top_p < 1.0:
        p = np.exp((ordered - ordered[0]) / float(temperature))
        c = np.cumsum(p)
        floor = max(floor, ordered[int(np.searchsorted(c, top_p * c[-1], side="left"))])
    return floor


def top_k_top_p_pick(logits_row, temperature, uniform, top_k=0, top_p=1.0):
    """temperature_pick among the logits at or above sampling_floor; the others have no weight."""
    row = np.asarray(logits_row, dtype=np.float64)
    floor = sampling_floor(row, temperature, top_k, top_p)
    p = np.where(row >= floor, np.exp((row - np.max(row)) / float(temperature)), 0.0)
    c = np.cumsum(p)
    idx = int(np.searchsorted(c, uniform * c[-1], side="right"))
    return min(idx, len(row) - 1)


def generate_greedy(config, W, prompt, max_new_tokens, eos=(), dtype=np.float64):
    """Greedy generation by full recompute, the reference's "naive" side (src/main.rs:3899-3901), with the stop
    rule of its stream loop: a stop token ends the sequence and is not part of the output
    (src/minimax.rs:448-453)."""
    ids = list(prompt)
    out = []
    for _ in range(max_new_tokens):
        nxt = greedy_pick(logits_all_positions(config, W, ids, dtype)[-1])
        if nxt in eos:
            break
        out.append(nxt)
        ids.append(nxt)
    return out
