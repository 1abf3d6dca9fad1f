"""Plain, slow restatement of the Vulanex layer-list family (dnet_b200/core/models/seqmix.py) in float64 on the CPU.

One function per mechanism, whole sequences only: no cache, no page, no carried state, no pooled rows kept anywhere.
Whatever the product computes through portions, batches, pages and slots has to equal what these functions give for
the whole token list.  Notation: T tokens, W width, H heads, G key heads, dk / dv key / value size per head, n the
window's size, P the pooled blocks' size.  Nothing here is imported by the product, and nothing of the product is
imported here.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

F = torch.float64


def lin(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return x @ w.to(F).T


def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(var + eps) * w + b with var = mean((x - mean)^2)"""
    mu = x.mean(-1, keepdim=True)
    var = (x - mu).pow(2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w.to(F) + b.to(F)


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def bigram_rows(tokens: List[int], buckets: int, mul_prev: int, mul_cur: int) -> List[int]:
    """row of the bigram table for every token: a hash of (previous token, token); the extra last row for the first"""
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(buckets if t == 0 else (tokens[t - 1] * mul_prev + tok * mul_cur) % buckets)
    return rows


def input_convolution(h: torch.Tensor, cw: torch.Tensor) -> torch.Tensor:
    """h_t + sum_j cw[:, j] h_(t - taps + 1 + j): tap taps - 1 meets the token itself, tap 0 the oldest; before the
    sequence there are zeros"""
    T = h.shape[0]
    taps = cw.shape[1]
    out = h.clone()
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += cw[:, j].to(F) * h[s]
    return out


def query_temperature(T: int, coef: float, every: int) -> torch.Tensor:
    """the factor on the query at every position: 1 + coef ln(floor((p + 1) / every) + 1)"""
    return torch.tensor([1.0 + coef * math.log((p + 1) // every + 1) for p in range(T)], dtype=F)


def rotary_frequencies(rot: dict) -> Tuple[torch.Tensor, float]:
    """frequencies of the dims/2 pairs and the factor on cos and sin.  With scaling, pairs that turn at least `fast`
    times within the original context keep their frequency, pairs that turn at most `slow` times have it divided by the
    factor, with a linear ramp over the pair index between the two."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return torch.tensor(f, dtype=F), 1.0

    def index_of(turns: float) -> float:       # the (real-valued) pair index that turns this often over the original context
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(sc["fast"])), 0)
    hi = min(math.ceil(index_of(sc["slow"])), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
        out.append(fi / sc["factor"] * ramp + fi * (1.0 - ramp))
    return torch.tensor(out, dtype=F), 0.1 * math.log(sc["factor"]) + 1.0


def rotary_half(x: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, heads, d]: dim i turns with dim i + dims/2 by the angle p f_i; dims from rot.dims up pass"""
    dims = int(rot["dims"])
    f, m = rotary_frequencies(rot)
    T = x.shape[0]
    out = x.clone()
    for p in range(T):
        for i in range(dims // 2):
            c, s = math.cos(p * float(f[i])) * m, math.sin(p * float(f[i])) * m
            u, v = x[p, :, i], x[p, :, i + dims // 2]
            out[p, :, i] = u * c - v * s
            out[p, :, i + dims // 2] = v * c + u * s
    return out


def visible(i: int, size: int, pool: int) -> Tuple[List[int], List[int]]:
    """what the query at position i sees: the tokens j with 0 <= i - j < size (every j <= i without a window), and the
    blocks b of `pool` tokens whose last position b pool + pool - 1 lies at or before i - size"""
    if size <= 0:
        return list(range(i + 1)), []
    toks = [j for j in range(i + 1) if i - j < size]
    blocks = [b for b in range((i + 1) // pool + 1) if b * pool + pool - 1 <= i - size] if pool > 0 else []
    return toks, blocks


def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, size: int = 0, pool: int = 0,
                      sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] -> [T, H, dv], row by row.  A block's key (value) is the mean of its
    tokens' keys (values); tokens and blocks share one softmax, whose denominator also holds exp(sink_h) when the head
    has a sink (a term without key and value, not scaled)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F)
    nb = T // pool if pool > 0 else 0
    kb = torch.stack([k[b * pool:(b + 1) * pool].mean(0) for b in range(nb)]) if nb else k[:0]      # [blocks, G, dk]
    vb = torch.stack([v[b * pool:(b + 1) * pool].mean(0) for b in range(nb)]) if nb else v[:0]
    for i in range(T):
        toks, blocks = visible(i, size, pool)
        for h in range(H):
            g = h // (H // G)
            keys = torch.cat([k[toks, g], kb[blocks, g]])
            vals = torch.cat([v[toks, g], vb[blocks, g]])
            s = keys @ q[i, h] * scale
            m = s.max() if sink is None else torch.maximum(s.max(), sink[h].to(F))
            e = torch.exp(s - m)
            den = e.sum() + (torch.exp(sink[h].to(F) - m) if sink is not None else 0.0)
            out[i, h] = (e / den) @ vals
    return out


def generalized_delta_rule(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, w: torch.Tensor, a: torch.Tensor) -> torch.Tensor:
    """r, k, v, w, a [T, H, d] -> o [T, H, d].  Per head a state S [d, d] from zero; with u = k / sqrt(|k|^2 + 1e-6):
    S <- diag(w) S - (a * u) (u^T S) + k v^T (decay and removal both read the old S), then o = S^T r."""
    T, H, d = k.shape
    o = torch.zeros(T, H, d, dtype=F)
    for h in range(H):
        S = torch.zeros(d, d, dtype=F)
        for t in range(T):
            u = k[t, h] / torch.sqrt(k[t, h].pow(2).sum() + 1e-6)
            along = u @ S                                            # [d]: what every column holds along u
            S = w[t, h][:, None] * S - torch.outer(a[t, h] * u, along) + torch.outer(k[t, h], v[t, h])
            o[t, h] = S.T @ r[t, h]
    return o


def mixer_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mx: dict) -> torch.Tensor:
    """GQA attention without positions whose values are its keys; the query grows with the logarithm of the position"""
    T = h.shape[0]
    H, G, dk = int(mx["heads"]), int(mx.get("kv_heads", mx["heads"])), int(mx["dim"])
    q = lin(h, w[p + "q"]).view(T, H, dk)
    k = lin(h, w[p + "k"]).view(T, G, dk)
    qt = mx.get("q_temp")
    if qt:
        q = q * query_temperature(T, float(qt["coef"]), int(qt["every"]))[:, None, None]
    o = softmax_attention(q, k, k, float(mx["scale"]))
    return lin(o.reshape(T, -1), w[p + "o"])


def left_half(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mx: dict, eps: float) -> torch.Tensor:
    """attention with per-head q / k norms, rotary, a sliding window followed by pooled blocks, and a sink"""
    T = h.shape[0]
    H, G, dk, dv = int(mx["heads"]), int(mx.get("kv_heads", mx["heads"])), int(mx["dim"]), int(mx.get("vdim", mx["dim"]))
    q = unit_rms(lin(h, w[p + "q"]).view(T, H, dk), eps) * w[p + "q.norm"].to(F)
    k = unit_rms(lin(h, w[p + "k"]).view(T, G, dk), eps) * w[p + "k.norm"].to(F)
    v = lin(h, w[p + "v"]).view(T, G, dv)
    if mx.get("rot"):
        q, k = rotary_half(q, mx["rot"]), rotary_half(k, mx["rot"])
    mask = mx.get("mask") or {}
    o = softmax_attention(q, k, v, float(mx["scale"]), int(mask.get("size", 0) or 0), int(mask.get("pool", 0) or 0), w[p + "sink"])
    return lin(o.reshape(T, -1), w[p + "o"])


def right_half(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mx: dict, eps: float) -> torch.Tensor:
    """the generalized delta rule with its decay exp(-e^(-1/2) sigmoid(.)) and removal rate sigmoid(.) per key channel,
    read out through a per-head unit RMS, a weight per channel and a sigmoid gate"""
    T = h.shape[0]
    H, d = int(mx["heads"]), int(mx["dim"])
    r, k, v = (lin(h, w[p + n]).view(T, H, d) for n in "rkv")
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(lin(torch.tanh(lin(h, w[p + "w1"])), w[p + "w2"]) + w[p + "w0"].to(F))).view(T, H, d)
    rate = torch.sigmoid(lin(h, w[p + "a"]) + w[p + "a.b"].to(F)).view(T, H, d)
    o = unit_rms(generalized_delta_rule(r, k, v, decay, rate), eps).reshape(T, -1)
    return lin(o * w[p + "norm"].to(F) * torch.sigmoid(lin(h, w[p + "g"])), w[p + "o"])


def mixer_parallel(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mx: dict, eps: float) -> torch.Tensor:
    """both halves read h; each output is RMS-normed over the width with its own weight, and the mean of the two leaves"""
    left = unit_rms(left_half(h, w, p + "left.", mx["left"], eps), eps) * w[p + "left.out"].to(F)
    right = unit_rms(right_half(h, w, p + "right.", mx["right"], eps), eps) * w[p + "right.out"].to(F)
    return 0.5 * (left + right)


def gated_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return lin(gelu_tanh(lin(h, w[p + "gate"])) * lin(h, w[p + "up"]), w[p + "down"])


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None) -> torch.Tensor:
    """logits [T, V] of a whole sequence; layers_out collects the residual after every layer"""
    w = {k: v.to(F) for k, v in w.items()}
    eps = float((cfg.get("norm") or {}).get("eps", 1e-6))
    taps = int((cfg.get("canon") or {}).get("taps", 0) or 0)
    x = w["embed"][torch.tensor(tokens)]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        x = x + w["bigram"][torch.tensor(bigram_rows(tokens, int(bg["buckets"]), int(bg["mul_prev"]), int(bg["mul_cur"])))]
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        if taps:
            h = input_convolution(h, w[p + "canon1"])
        if L["type"] == "attention":
            x = x + mixer_attention(h, w, p + "mix.", L["mixer"])
        elif L["type"] == "parallel":
            x = x + mixer_parallel(h, w, p + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        if L.get("mlp"):
            h = layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps)
            if taps:
                h = input_convolution(h, w[p + "canon2"])
            x = x + gated_ff(h, w, p + "mlp.")
        if layers_out is not None:
            layers_out.append(x.clone())
    return lin(layer_norm(x, w["final.norm"], w["final.norm.b"], eps), w["embed"]) * float(cfg.get("logit_scale", 1.0))


# -- checkpoints ---------------------------------------------------------------------------------------------------------------
def tensor_shapes(cfg: dict, rank: int = 8) -> Dict[str, Tuple[int, ...]]:
    """every tensor of a checkpoint; `rank` is the inner size of the decay's two-step projection (no config key gives it)"""
    W, V = int(cfg["width"]), int(cfg["vocab"])
    taps = int((cfg.get("canon") or {}).get("taps", 0) or 0)
    out: Dict[str, Tuple[int, ...]] = {"embed": (V, W), "final.norm": (W,), "final.norm.b": (W,)}
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        out["bigram"] = (int(bg["buckets"]) + 1, W)
    for i, L in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", L["mixer"]
        out[p + "norm1"] = out[p + "norm1.b"] = (W,)
        if taps:
            out[p + "canon1"] = (W, taps)
        if L["type"] == "attention":
            H, G, dk = int(mx["heads"]), int(mx.get("kv_heads", mx["heads"])), int(mx["dim"])
            out[p + "mix.q"], out[p + "mix.k"], out[p + "mix.o"] = (H * dk, W), (G * dk, W), (W, H * dk)
        else:
            l, r = mx["left"], mx["right"]
            H, G, dk, dv = int(l["heads"]), int(l.get("kv_heads", l["heads"])), int(l["dim"]), int(l.get("vdim", l["dim"]))
            q = p + "mix.left."
            out[q + "q"], out[q + "k"], out[q + "v"], out[q + "o"] = (H * dk, W), (G * dk, W), (G * dv, W), (W, H * dv)
            out[q + "q.norm"] = out[q + "k.norm"] = (dk,)
            out[q + "sink"] = (H,)
            C = int(r["heads"]) * int(r["dim"])
            q = p + "mix.right."
            for n in "rkvga":
                out[q + n] = (C, W)
            out[q + "a.b"] = out[q + "w0"] = out[q + "norm"] = (C,)
            out[q + "w1"], out[q + "w2"], out[q + "o"] = (rank, W), (C, rank), (W, C)
            out[p + "mix.left.out"] = out[p + "mix.right.out"] = (W,)
        if L.get("mlp"):
            ff = int(L["mlp"]["ff"])
            out[p + "norm2"] = out[p + "norm2.b"] = (W,)
            if taps:
                out[p + "canon2"] = (W, taps)
            out[p + "mlp.gate"] = out[p + "mlp.up"] = (ff, W)
            out[p + "mlp.down"] = (W, ff)
    return out


def random_weights(cfg: dict, seed: int, rank: int = 8) -> Dict[str, torch.Tensor]:
    """fp32 tensors whose values are exact in bf16: matrices ~ N(0, 1/fan_in), norm weights around one, biases, sinks
    and convolution taps of a size that shows when one is left out"""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg, rank).items():
        if name.endswith(".b") or name.endswith(".w0"):
            t = 0.3 * torch.randn(shape, generator=g)
        elif name.endswith(("norm1", "norm2", "final.norm", ".norm", ".out")):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif name.endswith(".sink"):
            t = 0.5 + torch.randn(shape, generator=g)
        elif "canon" in name:
            t = 0.4 * torch.randn(shape, generator=g)
        elif name in ("embed", "bigram"):
            t = torch.randn(shape, generator=g) * (0.5 if name == "bigram" else 1.0)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out
