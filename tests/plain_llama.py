"""A plain, slow Llama written from the reference's formulas.

Whole sequences, no cache, one function per part, PyTorch on the CPU.  It
shares no code with the engine: it reads the config.json dictionary and the
tensors by name itself.  Each function cites the reference file:line whose
arithmetic it restates.  The reference is Rust and cannot be compiled or
imported here (no cargo/rustc in the image), so this file rests on the
formulas alone; `tests/golden/` holds outputs of this file for a fixed tiny
model so that a later change to it shows.

`dtype` is the arithmetic type: float32 restates the reference's CPU backend,
float64 gives an oracle whose own rounding is negligible.
"""
from __future__ import annotations

import math

import torch


def plain_embed(table: torch.Tensor, ids: torch.Tensor, dtype) -> torch.Tensor:
    """x[t,:] = table[ids[t],:]   (src/backend/cpu.rs:370-384)"""
    if int(ids.min()) < 0 or int(ids.max()) >= table.shape[0]:
        raise ValueError("token id out of range")           # src/model.rs:421-428
    return table[ids.long()].to(dtype)


def plain_rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """ms = sum(x^2)/dim; y = x * (1/sqrt(ms+eps)) * w   (src/backend/cpu.rs:388-401)"""
    mean_sq = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    scale = 1.0 / torch.sqrt(mean_sq + eps)
    return x * scale * w.to(x.dtype)


def plain_linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y[t,r] = sum_c W[r,c] x[t,c], no bias   (src/backend/cpu.rs:337-368)"""
    return x @ w.to(x.dtype).t()


def plain_inv_freq(head_dim: int, theta: float, scaling: dict | None) -> torch.Tensor:
    """f_i = theta^(-2i/d)   (src/backend/cpu.rs:76, 146).

    With llama3 scaling each f_i is divided by a per-pair factor, the form the
    reference's split-half rotation takes its divisors in
    (src/backend/cpu.rs:135-156): wavelengths shorter than L/high keep f_i,
    longer than L/low use f_i/factor, the band between is blended linearly in
    L/wavelength.  Computed in float64, stored as float32.
    """
    i = torch.arange(head_dim // 2, dtype=torch.float64)
    f = torch.tensor(float(theta), dtype=torch.float64) ** (-2.0 * i / head_dim)
    if scaling is not None and scaling.get("rope_type", scaling.get("type")) not in (None, "default"):
        factor = float(scaling["factor"])
        low = float(scaling["low_freq_factor"])
        high = float(scaling["high_freq_factor"])
        L = float(scaling["original_max_position_embeddings"])
        out = []
        for fi in f.tolist():
            wavelen = 2.0 * math.pi / fi
            if wavelen < L / high:
                out.append(fi)
            elif wavelen > L / low:
                out.append(fi / factor)
            else:
                s = (L / wavelen - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = torch.tensor(out, dtype=torch.float64)
    return f.to(torch.float32)


def plain_rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor,
               layout: str) -> torch.Tensor:
    """Rotate every head of x [T, heads, D] by angle a = float32(pos) * f_i.

    interleaved: pairs (2i, 2i+1)   (src/backend/cpu.rs:68-84)
    split_half:  pairs (i, i+D/2)   (src/backend/cpu.rs:135-156)
    (x0, x1) <- (x0 cos a - x1 sin a, x0 sin a + x1 cos a).  The angle is a
    float32 product, as in the reference; its sine and cosine are taken in float64.
    """
    T, H, D = x.shape
    half = D // 2
    angle = (positions.to(torch.float32)[:, None] * inv_freq[None, :]).to(torch.float64)  # [T, half]
    cos = torch.cos(angle).to(x.dtype)[:, None, :]
    sin = torch.sin(angle).to(x.dtype)[:, None, :]
    out = torch.empty_like(x)
    if layout == "interleaved":
        x0, x1 = x[..., 0::2], x[..., 1::2]
        out[..., 0::2] = x0 * cos - x1 * sin
        out[..., 1::2] = x0 * sin + x1 * cos
    elif layout == "split_half":
        x0, x1 = x[..., :half], x[..., half:]
        out[..., :half] = x0 * cos - x1 * sin
        out[..., half:] = x0 * sin + x1 * cos
    else:
        raise ValueError(layout)
    return out


def plain_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                    window: int = 0) -> torch.Tensor:
    """Causal grouped-query attention over a whole sequence
    (src/backend/cpu.rs:530-590): query i sees keys [first, i] with
    first = 0, or i+1-window when a window is set; kv head = q head / group;
    s = (q.k) * scale; p = exp(s - max) / sum; o = sum p v.
    q [T, H, D], k and v [T, K, D] -> [T, H*D]."""
    T, H, D = q.shape
    K = k.shape[1]
    group = H // K
    out = torch.zeros(T, H, D, dtype=q.dtype)
    for i in range(T):
        visible = i + 1
        first = 0 if window == 0 else max(0, visible - window)
        for h in range(H):
            kh = h // group
            s = (k[first:visible, kh, :] @ q[i, h, :]) * scale
            p = torch.exp(s - s.max())
            p = p / p.sum()
            out[i, h, :] = p @ v[first:visible, kh, :]
    return out.reshape(T, H * D)


def plain_swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """act = g / (1 + exp(-g)) * u   (src/backend/cpu.rs:447-458)"""
    return gate / (1.0 + torch.exp(-gate)) * up


def plain_forward(config: dict, tensors: dict, ids, dtype=torch.float32) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence starting at position 0.

    Order of operations of src/model/arch/llama.rs:158-246: norm, Q/K/V, rotary
    on q and k (v untouched), attention, output projection, residual; norm,
    gate/up, SwiGLU, down, residual; final norm; output matrix, which is the
    embedding when the model ties them (src/model.rs:175-177).
    """
    ids = torch.as_tensor(ids, dtype=torch.long)
    H = config["num_attention_heads"]
    K = config.get("num_key_value_heads") or H
    D = config.get("head_dim") or config["hidden_size"] // H
    eps = config["rms_norm_eps"]
    layout = config.get("rope_layout", "split_half")
    inv_freq = plain_inv_freq(D, config.get("rope_theta", 10000.0), config.get("rope_scaling"))
    positions = torch.arange(ids.numel())
    scale = 1.0 / math.sqrt(D)

    x = plain_embed(tensors["model.embed_tokens.weight"], ids, dtype)
    T = x.shape[0]
    for i in range(config["num_hidden_layers"]):
        p = f"model.layers.{i}."
        h = plain_rmsnorm(x, tensors[p + "input_layernorm.weight"], eps)
        q = plain_linear(h, tensors[p + "self_attn.q_proj.weight"]).reshape(T, H, D)
        k = plain_linear(h, tensors[p + "self_attn.k_proj.weight"]).reshape(T, K, D)
        v = plain_linear(h, tensors[p + "self_attn.v_proj.weight"]).reshape(T, K, D)
        q = plain_rope(q, positions, inv_freq, layout)
        k = plain_rope(k, positions, inv_freq, layout)
        a = plain_attention(q, k, v, scale)
        x = x + plain_linear(a, tensors[p + "self_attn.o_proj.weight"])
        h = plain_rmsnorm(x, tensors[p + "post_attention_layernorm.weight"], eps)
        act = plain_swiglu(plain_linear(h, tensors[p + "mlp.gate_proj.weight"]),
                           plain_linear(h, tensors[p + "mlp.up_proj.weight"]))
        x = x + plain_linear(act, tensors[p + "mlp.down_proj.weight"])
    h = plain_rmsnorm(x, tensors["model.norm.weight"], eps)
    w_out = tensors["model.embed_tokens.weight"] if config.get("tie_word_embeddings") \
        else tensors["lm_head.weight"]
    return plain_linear(h, w_out)


# ---------------------------------------------------------------- sampling

def plain_argmax(logits) -> int:
    """Index of the largest logit; of equal ones the lowest index wins (the
    engine's rule; the reference's max_by keeps the last, src/sampler.rs:68-74)."""
    best, best_i = None, 0
    for i, l in enumerate(logits):
        if best is None or l > best:
            best, best_i = l, i
    return best_i


def plain_sample(logits, history, u: float, temperature: float, top_p: float = 1.0,
                 min_p: float = 0.0, repetition_penalty: float = 1.0,
                 repetition_window: int = 64) -> int:
    """One token from `logits` given a uniform draw u in [0,1)   (src/sampler.rs:34-61).

    penalty on the last `repetition_window` ids (divide if >0 else multiply,
    :76-86) -> temperature<=0 ? argmax (:43-45) -> /temperature -> softmax
    (:88-93) -> sort descending -> min-p keeps p >= p_max*min_p (:96-103) ->
    top-p keeps the smallest prefix whose sum reaches top_p (:105-119) ->
    first id whose running sum reaches u*total (:121-135).  Arithmetic in
    float32, as the reference does.
    """
    x = torch.as_tensor(logits, dtype=torch.float32).clone()
    if repetition_penalty != 1.0:
        start = max(0, len(history) - repetition_window)
        for tok in history[start:]:
            if 0 <= tok < x.numel():
                x[tok] = x[tok] / repetition_penalty if x[tok] > 0 else x[tok] * repetition_penalty
    if temperature <= 0.0:
        return plain_argmax(x.tolist())
    x = x / temperature
    e = torch.exp(x - x.max())
    p = e / e.sum()
    order = sorted(range(p.numel()), key=lambda i: (-float(p[i]), i))
    ranked = [(i, float(p[i])) for i in order]
    if min_p > 0.0 and ranked:
        thr = torch.tensor(ranked[0][1], dtype=torch.float32) * torch.tensor(min_p, dtype=torch.float32)
        ranked = [(i, q) for i, q in ranked if q >= float(thr)]
    if top_p < 1.0 and ranked:
        cum = torch.tensor(0.0, dtype=torch.float32)
        cutoff = len(ranked)
        for n, (_, q) in enumerate(ranked):
            cum = cum + torch.tensor(q, dtype=torch.float32)
            if float(cum) >= top_p:
                cutoff = n + 1
                break
        ranked = ranked[:max(cutoff, 1)]
    total = torch.tensor(0.0, dtype=torch.float32)
    for _, q in ranked:
        total = total + torch.tensor(q, dtype=torch.float32)
    if float(total) <= 0.0:
        return ranked[0][0]
    target = torch.tensor(u, dtype=torch.float32) * total
    cum = torch.tensor(0.0, dtype=torch.float32)
    for i, q in ranked:
        cum = cum + torch.tensor(q, dtype=torch.float32)
        if float(cum) >= float(target):
            return i
    return ranked[-1][0]


def plain_generate(config: dict, tensors: dict, prompt, max_tokens: int, stop_ids=(),
                   dtype=torch.float32):
    """Greedy generation by re-running the whole sequence for every token
    (loop of src/inference.rs:102-124: a stop token ends the sequence and is not
    emitted; the last sampled token is not fed back)."""
    seq = list(prompt)
    out = []
    for _ in range(max_tokens):
        logits = plain_forward(config, tensors, seq, dtype)[-1]
        if not torch.isfinite(logits).all():
            raise ValueError("nonfinite logits")             # src/inference.rs:111-113
        tok = plain_argmax(logits.tolist())
        if tok in stop_ids:
            break
        out.append(tok)
        seq.append(tok)
    return out
