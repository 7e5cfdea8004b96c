"""A plain, slow Llama decoder: whole sequences, no cache, one function per part.

This file rests on the reference's formulas, not on running its code: the
reference's model code (src/model.cpp) is Windows-only, reads GGUF files only,
and cannot be compiled or imported here.  Each function cites the lines of the
reference it restates.  Nothing here is shared with the library under test: it
reads ``config.json`` keys from a plain dictionary and tensors from a plain
name -> tensor mapping, and computes on the CPU in the dtype it is given
(float64 by default, so that it is the more exact side of every comparison).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch


# ---------------------------------------------------------------------------------------------
# parts
# ---------------------------------------------------------------------------------------------
def embed(ids: Sequence[int], table: torch.Tensor, dtype=torch.float64) -> torch.Tensor:
    """x[t, :] = E[id_t, :]  (src/model.cpp:1381-1383; the reference clamps an
    out-of-range id to [0, V-1], the library rejects it, so ids here are valid)."""
    return table.to(dtype)[torch.as_tensor(list(ids), dtype=torch.long)]


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """ss = sum x^2; s = 1/sqrt(ss/d + eps); y = x * s * w  (src/model.cpp:626-633)."""
    d = x.shape[-1]
    ss = (x * x).sum(-1, keepdim=True)
    s = 1.0 / torch.sqrt(ss / d + eps)
    return x * s * w.to(x.dtype)


def rope_inv_freq(rotary_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """inv_freq[i] = theta^(-2i/n_rot) / rscale / factors[i]  (src/model.cpp:229-237).

    ``rscale`` is the factor of ``linear`` scaling.  ``factors`` are
    per-frequency divisors which the reference reads ready-made from the tensor
    ``rope_freqs.weight`` (src/model.cpp:230, 235); for ``llama3`` scaling they
    follow from the wavelength of each frequency: unchanged below
    orig/high_freq_factor, divided by ``factor`` above orig/low_freq_factor, and
    a linear blend of the two between.  Computed in float64, rounded to float32
    (the precision in which the angles are formed).
    """
    i = torch.arange(rotary_dim // 2, dtype=torch.float64)
    inv = theta ** (-2.0 * i / rotary_dim)
    kind = None if not scaling else scaling.get("rope_type", scaling.get("type"))
    if kind == "linear":
        inv = inv / float(scaling["factor"])
    elif kind == "llama3":
        factor = float(scaling["factor"])
        low = float(scaling["low_freq_factor"])
        high = float(scaling["high_freq_factor"])
        orig = float(scaling["original_max_position_embeddings"])
        wavelen = 2.0 * math.pi / inv
        smooth = (orig / wavelen - low) / (high - low)
        blended = (1.0 - smooth) * inv / factor + smooth * inv
        inv = torch.where(wavelen < orig / high, inv, torch.where(wavelen > orig / low, inv / factor, blended))
    elif kind not in (None, "default"):
        raise ValueError(f"unsupported rope scaling {kind}")
    return inv.to(torch.float32)


def rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, pairing: str = "half") -> torch.Tensor:
    """x: [T, heads, hd].  theta = pos * inv_freq[i] formed in float32, c = cos, s = sin;
    pair (i0, i1) = (i, i + half) when the pairing is half-split, (2i, 2i+1) when
    interleaved; v[i0]' = a c - b s, v[i1]' = a s + b c  (src/model.cpp:635-649, 698-713).
    A model folder with config.json stores q/k rows unpermuted, which is the
    half-split pairing (the reference's ``neox`` flag, src/model.cpp:74, 643)."""
    half = inv_freq.numel()
    ang = positions.to(torch.float32)[:, None] * inv_freq[None, :].to(torch.float32)   # float32 product, as the reference
    c = torch.cos(ang.to(torch.float64)).to(x.dtype)[:, None, :]
    s = torch.sin(ang.to(torch.float64)).to(x.dtype)[:, None, :]
    out = x.clone()
    if pairing == "half":
        a, b = x[..., :half], x[..., half:2 * half]
        out[..., :half] = a * c - b * s
        out[..., half:2 * half] = a * s + b * c
    else:
        a, b = x[..., 0:2 * half:2], x[..., 1:2 * half:2]
        out[..., 0:2 * half:2] = a * c - b * s
        out[..., 1:2 * half:2] = a * s + b * c
    return out


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None,
              window: Optional[int] = None) -> torch.Tensor:
    """q: [T, nh, hd], k/v: [T, nkv, hd] of ONE sequence starting at position 0.
    Per (token t, head h): kv head = h / (nh/nkv); keys j in [j0, t] with
    j0 = t+1-window when a window is set and t+1 > window, else 0 (causal by loop
    bound); s_j = (q . k_j) * scale, scale = 1/sqrt(hd); mx = max s_j;
    p_j = exp(s_j - mx); o = sum (p_j / sum p) v_j   (src/model.cpp:1500-1522)."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    grp = nh // nkv
    if scale is None:
        scale = 1.0 / math.sqrt(hd)
    out = torch.zeros_like(q)
    for t in range(T):
        j0 = t + 1 - window if (window and t + 1 > window) else 0
        for h in range(nh):
            kvh = h // grp
            s = (k[j0:t + 1, kvh] @ q[t, h]) * scale
            p = torch.exp(s - s.max())
            p = p / p.sum()
            out[t, h] = p @ v[j0:t + 1, kvh]
    return out


def silu(x: torch.Tensor) -> torch.Tensor:
    """silu(x) = x / (1 + exp(-x))  (src/model.cpp:1309)."""
    return x / (1.0 + torch.exp(-x))


def gated_mlp(xn: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor) -> torch.Tensor:
    """g = Wg xn, u = Wu xn, h = silu(g) * u, t = Wd h  (src/model.cpp:1559-1563)."""
    dt = xn.dtype
    g = xn @ wg.to(dt).T
    u = xn @ wu.to(dt).T
    return (silu(g) * u) @ wd.to(dt).T


def attention_block(xn: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, cfg: dict, inv_freq: torch.Tensor,
                    positions: torch.Tensor) -> torch.Tensor:
    """q = Wq xn, k = Wk xn, v = Wv xn; rope on q and k; attention; t = Wo att
    (src/model.cpp:1479-1481, 1491-1493, 1500-1531).  Weights are [out, in] and
    y = W x (src/model.cpp:33); head h holds rows [h*hd, (h+1)*hd)."""
    dt = xn.dtype
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    T = xn.shape[0]
    q = (xn @ w[f"{prefix}.q_proj.weight"].to(dt).T).view(T, nh, hd)
    k = (xn @ w[f"{prefix}.k_proj.weight"].to(dt).T).view(T, nkv, hd)
    v = (xn @ w[f"{prefix}.v_proj.weight"].to(dt).T).view(T, nkv, hd)
    q = rope(q, positions, inv_freq)
    k = rope(k, positions, inv_freq)
    # the window applies only where the folder switches it on: the reference runs this architecture without one
    # (src/model.cpp:147 sets a window for other families only)
    att = attention(q, k, v, window=cfg.get("sliding_window") if cfg.get("use_sliding_window") else None)
    return att.reshape(T, nh * hd) @ w[f"{prefix}.o_proj.weight"].to(dt).T


# ---------------------------------------------------------------------------------------------
# whole model
# ---------------------------------------------------------------------------------------------
def normalized_config(cfg: dict) -> dict:
    c = dict(cfg)
    c.setdefault("num_key_value_heads", c["num_attention_heads"])
    c.setdefault("head_dim", c["hidden_size"] // c["num_attention_heads"])
    if c["head_dim"] is None:
        c["head_dim"] = c["hidden_size"] // c["num_attention_heads"]
    c.setdefault("rms_norm_eps", 1e-5)
    c.setdefault("rope_theta", 10000.0)
    c.setdefault("rope_scaling", None)
    c.setdefault("tie_word_embeddings", False)
    return c


def hidden_states(ids: Sequence[int], cfg: dict, w: Dict[str, torch.Tensor], dtype=torch.float64) -> torch.Tensor:
    """The residual stream after the last layer for one whole sequence.  Order per
    layer: norm, attention, x += t, norm, feed-forward, x += t  (src/model.cpp:1460-1565)."""
    cfg = normalized_config(cfg)
    inv_freq = rope_inv_freq(cfg["head_dim"], cfg["rope_theta"], cfg["rope_scaling"])
    x = embed(ids, w["model.embed_tokens.weight"], dtype)
    positions = torch.arange(len(ids))
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}"
        xn = rmsnorm(x, w[f"{p}.input_layernorm.weight"], cfg["rms_norm_eps"])
        x = x + attention_block(xn, w, f"{p}.self_attn", cfg, inv_freq, positions)
        xn = rmsnorm(x, w[f"{p}.post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        x = x + gated_mlp(xn, w[f"{p}.mlp.gate_proj.weight"], w[f"{p}.mlp.up_proj.weight"],
                          w[f"{p}.mlp.down_proj.weight"])
    return x


def logits_whole(ids: Sequence[int], cfg: dict, w: Dict[str, torch.Tensor], dtype=torch.float64) -> torch.Tensor:
    """Logits at every position: final norm, then the output matrix, which is
    the embedding matrix when the model has no output matrix of its own
    (src/model.cpp:132, 1598-1603)."""
    cfg = normalized_config(cfg)
    x = hidden_states(ids, cfg, w, dtype)
    xn = rmsnorm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return xn @ head.to(dtype).T


# ---------------------------------------------------------------------------------------------
# sampling and generation
# ---------------------------------------------------------------------------------------------
def philox_uniform(seed: int, stream: int, counter: int) -> float:
    """Philox-4x32-10 with key (seed lo, seed hi) and counter (counter, stream, 0, 0);
    the top 24 bits of the first output word mapped to (0, 1) as (x + 0.5) / 2^24."""
    M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
    k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    c = [counter & 0xFFFFFFFF, stream & 0xFFFFFFFF, 0, 0]
    for _ in range(10):
        p0, p1 = M0 * c[0], M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k0) & 0xFFFFFFFF, p1 & 0xFFFFFFFF, ((p0 >> 32) ^ c[3] ^ k1) & 0xFFFFFFFF, p0 & 0xFFFFFFFF]
        k0, k1 = (k0 + W0) & 0xFFFFFFFF, (k1 + W1) & 0xFFFFFFFF
    return ((c[0] >> 8) + 0.5) / 16777216.0


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, repetition_penalty: float,
           recent: Sequence[int], u: float) -> int:
    """One token from one row of logits, after src/chat.cpp:124-145:
    each of the recent ids is penalised (l > 0 ? l / pen : l * pen); temperature <= 0
    takes the largest; else the k = clamp(top_k, 1, V) largest are kept, weighted
    exp((l - max) / temp) and normalised, and the shortest prefix in descending order
    whose cumulative probability reaches top_p is kept (the crossing one included).
    The reference then draws r uniform in [0, cum) and walks the kept candidates in
    descending order; the library walks them in vocabulary order with r = u * cum
    (same law, a fixed order that needs no sort), and so does this function.  Ties
    are ordered by ascending id."""
    l = logits.to(torch.float32).clone()
    V = l.numel()
    if repetition_penalty != 1.0:
        for i in (int(r) for r in recent):          # once per occurrence, as the reference
            if 0 <= i < V:
                l[i] = l[i] / repetition_penalty if l[i] > 0 else l[i] * repetition_penalty
    if temperature <= 0:
        return int(torch.argmax(l))          # first of equal maxima
    k = min(V, max(1, top_k))
    order = sorted(range(V), key=lambda i: (-float(l[i]), i))[:k]
    mx = float(l[order[0]])
    p = [math.exp((float(l[i]) - mx) / temperature) for i in order]
    total = sum(p)
    cum, cut = 0.0, len(order)
    for n, pi in enumerate(p):
        cum += pi / total
        if cum >= top_p:
            cut = n + 1
            break
    kept = sorted(order[:cut])
    mass = {i: math.exp((float(l[i]) - mx) / temperature) for i in kept}
    r = u * sum(mass.values())
    acc = 0.0
    for i in kept:
        acc += mass[i]
        if r <= acc:
            return i
    return kept[-1]


def generate(prompt: Sequence[int], cfg: dict, w: Dict[str, torch.Tensor], max_new_tokens: int,
             stop_ids: Sequence[int] = (), temperature: float = 0.0, top_k: int = 40, top_p: float = 0.9,
             repetition_penalty: float = 1.0, seed: int = 0, stream: int = 0, dtype=torch.float64) -> List[int]:
    """The generation loop of src/chat.cpp:443-487 for one sequence, recomputing the
    whole sequence at every step: sample from the last position's logits, stop at a
    stop token (which is not emitted), keep the last 64 generated ids for the
    penalty, stop after ``max_new_tokens``."""
    ids = list(prompt)
    out: List[int] = []
    recent: List[int] = []
    for step in range(max_new_tokens):
        lg = logits_whole(ids, cfg, w, dtype)[-1]
        tok = sample(lg, temperature, top_k, top_p, repetition_penalty, recent, philox_uniform(seed, stream, step))
        if tok in stop_ids:
            break
        out.append(tok)
        ids.append(tok)
        recent = (recent + [tok])[-64:]
    return out
