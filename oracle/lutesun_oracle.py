"""Float64 oracle of the Lutesun family: one plain function per mechanism, whole sequences only, no cache.

It shares nothing with the product path (dnet_b200/core/models/seqmix.py, libdnet_b200_seq): keys and values are
formed per head from the latent of every position and attention is a dense [T, T] table, where the product absorbs
the queries into the latent space and reads one cached row per token.

Notation: T tokens, W width, H heads; a head's query is [dn unrotated; dr rotated] numbers, its value has dv, the
latent has R.  ``eps`` is the model's norm epsilon.

    x0 = embed[tokens] * scale
    x <- x + rms1p(mixer(x));   x <- x + rms1p(ff(x))      (the sublayers read x itself)
    logits = embed . rms1p(x)
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

F64 = torch.float64


# -- norms -----------------------------------------------------------------------------------------------------------
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def rms_one_plus(x, w, eps):
    """weight stored around zero"""
    return unit_rms(x, eps) * (1.0 + w)


def rms_plain(x, w, eps):
    return unit_rms(x, eps) * w


# -- rotary ------------------------------------------------------------------------------------------------------------
def rotary(x: torch.Tensor, pos: torch.Tensor, dims: int, base: float, layout: str) -> torch.Tensor:
    """x [T, ..., d]: the first ``dims`` numbers of the last axis turn by pos * base^(-2i/dims); pair i is
    (2i, 2i+1) for layout 'interleaved' and (i, i + dims/2) for 'half'."""
    if dims == 0:
        return x
    half = dims // 2
    freq = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    ang = pos.to(F64)[:, None] * freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cs, sn = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    ia = torch.arange(half) * 2 if layout == "interleaved" else torch.arange(half)
    ib = ia + 1 if layout == "interleaved" else ia + half
    out = x.clone()
    u, v = x[..., ia], x[..., ib]
    out[..., ia] = u * cs - v * sn
    out[..., ib] = v * cs + u * sn
    return out


# -- masks -------------------------------------------------------------------------------------------------------------
def window_mask(T: int, size: int) -> torch.Tensor:
    """[T, T] bool: query i sees key j when 0 <= i - j < size (size 0: every earlier key)"""
    d = torch.arange(T)[:, None] - torch.arange(T)[None, :]
    return (d >= 0) & ((d < size) if size > 0 else True)


# -- latent attention ----------------------------------------------------------------------------------------------------
def latent_attention(w: Dict[str, torch.Tensor], p: str, L: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    mx = L["mixer"]
    second = L["type"] == "latent_attention_2"
    H, dn, dv, R = mx["heads"], mx["dim"], mx.get("vdim", mx["dim"]), mx["kv_rank"]
    rot = mx.get("rot") or {}
    rdims, base = int(rot.get("dims", 0)), float(rot.get("base", 10000.0))
    dr = int(mx.get("rot_dim", rdims))
    layout = "half" if second else "interleaved"
    T = h.shape[0]
    pos = torch.arange(T)
    if second:
        q = rms_plain(h @ w[p + "mix.dq"].T, w[p + "mix.dq.norm"], eps) @ w[p + "mix.uq"].T
    else:
        q = h @ w[p + "mix.q"].T
    q = q.reshape(T, H, dn + dr)
    down = h @ w[p + "mix.dkv"].T
    lat = rms_plain(down[:, :R], w[p + "mix.dkv.norm"], eps)
    k_rot = rotary(down[:, R:], pos, rdims, base, layout)                     # one part for all heads
    q_rot = rotary(q[:, :, dn:], pos, rdims, base, layout)
    k_un = (lat @ w[p + "mix.uk"].T).reshape(T, H, dn)
    val = (lat @ w[p + "mix.uv"].T).reshape(T, H, dv)
    score = torch.einsum("ihd,jhd->hij", q[:, :, :dn], k_un) + torch.einsum("ihd,jd->hij", q_rot, k_rot)
    score = score * float(mx.get("scale", (dn + dr) ** -0.5))
    vis = window_mask(T, int((mx.get("mask") or {}).get("size", 0)))
    prob = torch.softmax(score.masked_fill(~vis[None], -math.inf), dim=-1)
    out = torch.einsum("hij,jhd->ihd", prob, val)
    if second:
        out = out * torch.sigmoid(h @ w[p + "mix.g"].T)[:, :, None]
    return out.reshape(T, H * dv) @ w[p + "mix.o"].T


# -- feed-forwards ---------------------------------------------------------------------------------------------------------
def relu2_ff(w, p, h):
    return torch.relu(h @ w[p + "mlp.up"].T + w[p + "mlp.up.b"]).pow(2) @ w[p + "mlp.down"].T + w[p + "mlp.down.b"]


def swiglu(h, gate, up, down):
    g = h @ gate.T
    return (g * torch.sigmoid(g) * (h @ up.T)) @ down.T


def scored_router(z: torch.Tensor, corr: Optional[torch.Tensor], top: int, groups: int, keep: int, scale: float) -> Tuple[List[int], List[float]]:
    """one token: logits z over all experts (identity ones included) -> chosen experts and their weights"""
    s = torch.softmax(z, -1)
    c = s + (corr if corr is not None else 0.0)
    n = z.numel()
    allowed = [True] * n
    if groups > 0:
        per = n // groups
        best = [max(float(c[g * per + i]) for i in range(per)) for g in range(groups)]
        order = sorted(range(groups), key=lambda g: (-best[g], g))[:keep]
        allowed = [(e // per) in order for e in range(n)]
    ranked = sorted((e for e in range(n) if allowed[e]), key=lambda e: (-float(c[e]), e))[:top]
    tot = sum(float(s[e]) for e in ranked) + 1e-20
    return ranked, [float(s[e]) / tot * scale for e in ranked]


def routed_ff(w, p, mlp: dict, h: torch.Tensor) -> torch.Tensor:
    r = mlp["router"]
    E, ident = int(r["experts"]), int(r.get("identity", 0) or 0)
    g = r.get("groups") or {}
    out = torch.zeros_like(h)
    z = h @ w[p + "mlp.router"].T
    for t in range(h.shape[0]):
        chosen, weights = scored_router(z[t], w.get(p + "mlp.correction"), int(r["top"]), int(g.get("count", 0) or 0),
                                        int(g.get("keep", g.get("count", 0)) or 0), float(r.get("scale", 1.0)))
        for e, wt in zip(chosen, weights):
            y = h[t] if e >= E else swiglu(h[t], w[f"{p}mlp.e{e}.gate"], w[f"{p}mlp.e{e}.up"], w[f"{p}mlp.e{e}.down"])
            out[t] += wt * y
    if mlp.get("shared"):
        q = p + "mlp.shared."
        out = out + swiglu(h, w[q + "gate"], w[q + "up"], w[q + "down"]) * torch.sigmoid(h @ w[q + "sg"].T)
    return out


# -- the model ---------------------------------------------------------------------------------------------------------------
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens, layers_out: Optional[list] = None) -> torch.Tensor:
    """logits [T, vocab] of a whole sequence; layers_out collects the residual after every layer"""
    w = {k: v.to(F64) for k, v in w.items()}
    eps = float((cfg.get("norm") or {}).get("eps", 1e-6))
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        x = x + rms_one_plus(latent_attention(w, p, L, x, eps), w[p + "norm1"], eps)
        mlp = L.get("mlp")
        if mlp:
            y = relu2_ff(w, p, x) if mlp.get("kind", "dense") == "dense" else routed_ff(w, p, mlp, x)
            x = x + rms_one_plus(y, w[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_one_plus(x, w["final.norm"], eps) @ w["embed"].T


# -- checkpoints ---------------------------------------------------------------------------------------------------------------
def tensor_shapes(cfg: dict) -> Dict[str, Tuple[int, ...]]:
    W, V = int(cfg["width"]), int(cfg["vocab"])
    out: Dict[str, Tuple[int, ...]] = {"embed": (V, W), "final.norm": (W,)}
    for i, L in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", L["mixer"]
        H, dn, dv, R = mx["heads"], mx["dim"], mx.get("vdim", mx["dim"]), mx["kv_rank"]
        dr = int(mx.get("rot_dim", (mx.get("rot") or {}).get("dims", 0)))
        out[p + "norm1"] = (W,)
        if L["type"] == "latent_attention_2":
            out[p + "mix.dq"], out[p + "mix.dq.norm"], out[p + "mix.uq"] = (mx["q_rank"], W), (mx["q_rank"],), (H * (dn + dr), mx["q_rank"])
            out[p + "mix.g"] = (H, W)
        else:
            out[p + "mix.q"] = (H * (dn + dr), W)
        out[p + "mix.dkv"], out[p + "mix.dkv.norm"] = (R + dr, W), (R,)
        out[p + "mix.uk"], out[p + "mix.uv"], out[p + "mix.o"] = (H * dn, R), (H * dv, R), (W, H * dv)
        mlp = L.get("mlp")
        if not mlp:
            continue
        out[p + "norm2"] = (W,)
        if mlp.get("kind", "dense") == "dense":
            F = int(mlp["ff"])
            out[p + "mlp.up"], out[p + "mlp.up.b"], out[p + "mlp.down"], out[p + "mlp.down.b"] = (F, W), (F,), (W, F), (W,)
            continue
        r = mlp["router"]
        n = int(r["experts"]) + int(r.get("identity", 0) or 0)
        F = int(mlp["expert"]["ff"])
        for e in range(int(r["experts"])):
            out[f"{p}mlp.e{e}.gate"] = out[f"{p}mlp.e{e}.up"] = (F, W)
            out[f"{p}mlp.e{e}.down"] = (W, F)
        out[p + "mlp.router"], out[p + "mlp.correction"] = (n, W), (n,)
        if mlp.get("shared"):
            S = int(mlp["shared"]["ff"])
            out[p + "mlp.shared.gate"] = out[p + "mlp.shared.up"] = (S, W)
            out[p + "mlp.shared.down"], out[p + "mlp.shared.sg"] = (W, S), (1, W)
    return out


def random_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """fp32 tensors whose values are exact in bf16: matrices ~ N(0, 1/fan_in), norm weights of the one-plus kind around
    zero, plain norm weights around one, corrections of the size of a score"""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith((".dkv.norm", ".dq.norm")):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif name.endswith(("norm1", "norm2", "final.norm")):
            t = 0.3 * torch.randn(shape, generator=g)
        elif name.endswith(".correction"):
            t = 0.1 * torch.randn(shape, generator=g)
        elif name.endswith(".b"):
            t = 0.3 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        elif name.endswith("mlp.router"):
            t = torch.randn(shape, generator=g) * 2.0 / math.sqrt(shape[-1])
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out
