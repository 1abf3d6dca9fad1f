"""Models given as a list of layers, each a sequence mixer plus an optional gated feed-forward, on
libdnet_b200_seq (include/dnet_b200_seq.h).

The llama-family classes of this package run one request per step and hand a [T, hidden] activation from layer to
layer; the families here run a *ragged batch* per step (portions of prompts beside single decoded tokens of up to
``max_seqs`` live sequences) through all layers, because what a layer carries between tokens is not only a KV page:
a recurrent mixer keeps an fp32 state and the last inputs of its short convolution per sequence, and the residual
is S fp32 streams.  The model owns the page pool and the state slots; ``SeqHandle`` is a sequence's lease on them,
the counterpart of ``KVHandle``.

``SeqMixRingModel`` reads the layer list from the config:

    {"architecture": NAME, "vocab": V, "width": W, "streams": S, "norm": {"eps": e}, "embedding": {"scale": c},
     "layers": [{"type": "attention" | "delta",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "conv",             # both mixers
                           "scale", "rot": {"base", "dims"}, "mask": {"size"},     # attention
                           "kv_from": j},                                          # attention, optional
                 "mlp": {"kind": "dense", "ff": F} | null}, ...]}

Absent keys switch a mechanism off (no ``streams``: plain residual; no ``mask``: plain causal; no ``rot``: no
rotation; no ``conv``: no convolution; no ``kv_from``: own keys and values).

``FilinexRingModel`` reads the same kind of list with other mixers and a routed feed-forward:

    {"architecture": "Filinex", "vocab": V, "width": W, "norm": {"eps": e}, "logit_softcap": c,
     "loop": {"start": a, "stop": b, "times": n},                                  # optional
     "layers": [{"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap"},
                           "right": {"heads", "dim", "vdim", "tau"}, "left_scale", "right_scale"},
                 "mlp": {"kind": "moe", "router": {"experts", "top"}, "expert": {"ff", "limit"},
                         "shared": {"ff", "limit"} | null} | null},
                {"type": "wkv", "mixer": {"heads", "dim"}, "mlp": ...}, ...]}

Sizes the config does not give (the inner size of the two-step decay projections, a wkv layer's value size) are
read from the checkpoint's tensor shapes (``tensor_shapes``), or from the optional keys ``rank`` / ``vdim``.

``LutesunRingModel`` is a list of latent-attention layers with dense or routed feed-forwards:

    {"architecture": "Lutesun", "vocab": V, "width": W, "norm": {"eps": e}, "embedding": {"scale": c},
     "layers": [{"type": "latent_attention" | "latent_attention_2",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank",   # q_rank: the second type only
                           "scale", "rot": {"base", "dims"}, "mask": {"size"}},
                 "mlp": {"kind": "dense", "ff": F}
                      | {"kind": "moe", "router": {"experts", "top", "identity", "scale", "groups": {"count", "keep"}},
                         "expert": {"ff"}, "shared": {"ff"} | null} | null}, ...]}

``VulanexRingModel``: layer norms, a causal convolution on every sublayer's input, a hashed bigram row in the embedding,
attention whose values are its keys beside layers that run windowed attention with pooled blocks next to a generalized
delta rule:

    {"architecture": "Vulanex", "vocab": V, "width": W, "norm": {"eps": e}, "logit_scale": c, "canon": {"taps": n},
     "embedding": {"bigram": {"buckets", "mul_prev", "mul_cur"}},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "q_temp": {"coef", "every"}}, "mlp": ...},
                {"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size", "pool"},
                                    "rot": {"base", "dims", "scaling": {"factor", "original", "fast", "slow"}}},
                           "right": {"heads", "dim"}}, "mlp": ...}, ...]}
"""
from __future__ import annotations

import ctypes as C
import re
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from dnet_b200 import _seqabi
from .base import BaseRingModel, _stream_ptr


_LAYER_KEY = re.compile(r"^l\d+\.")
_EXPERT_KEY = re.compile(r"^mlp\.e(\d+)\.(gate|up|down)$")


class SeqHandle:
    """One live sequence: a state slot of the model and the pages it has taken so far."""

    def __init__(self, model: "SeqMixRingModel", stream=None):
        self.model = model
        slot = C.c_int(-1)
        _seqabi.check(model._lib.dn_seq_open(model._h, _stream_ptr(stream), C.byref(slot)))
        self.slot = int(slot.value)

    @property
    def offset(self) -> int:
        return int(self.model._lib.dn_seq_length(self.model._h, self.slot)) if self.slot >= 0 else 0

    def free(self) -> None:
        if self.slot >= 0 and self.model._h:
            _seqabi.check(self.model._lib.dn_seq_close(self.model._h, self.slot))
        self.slot = -1


def _attention_cfg(lc: _seqabi.LayerCfg, mx: dict, qk_norm, mask: str = "block", rot_layout: str = "interleaved") -> None:
    lc.scale = float(mx.get("scale", float(mx["dim"]) ** -0.5))
    lc.chunk = int((mx.get("mask") or {}).get("size", 0))
    lc.mask_kind = _seqabi.DN_MASK_WINDOW if mask == "window" else _seqabi.DN_MASK_BLOCK
    lc.pool = int((mx.get("mask") or {}).get("pool", 0) or 0) if mask == "window" else 0
    rot = mx.get("rot") or {}
    lc.rot_dims = int(rot.get("dims", 0))
    lc.rot_base = float(rot.get("base", 10000.0))
    lc.rot_layout = _seqabi.DN_ROT_HALF if rot_layout == "half" else _seqabi.DN_ROT_INTERLEAVED
    sc = rot.get("scaling")
    if sc:
        lc.yarn_factor, lc.yarn_original = float(sc["factor"]), float(sc["original"])
        lc.yarn_fast, lc.yarn_slow = float(sc["fast"]), float(sc["slow"])
    qt = mx.get("q_temp")
    if qt:
        lc.qtemp_coef, lc.qtemp_every = float(qt["coef"]), int(qt["every"])
    lc.kv_from = int(mx["kv_from"]) if mx.get("kv_from") is not None else -1
    lc.qk_norm = _seqabi.DN_QKNORM_HEAD if qk_norm == "head" else int(bool(qk_norm))
    lc.softcap = float(mx.get("softcap", 0.0) or 0.0)
    lc.heads, lc.kv_heads = int(mx["heads"]), int(mx.get("kv_heads", mx["heads"]))
    lc.dim, lc.vdim = int(mx["dim"]), int(mx.get("vdim", mx["dim"]))
    lc.conv = int(mx.get("conv", 0) or 0)


def parse_layer_list(cfg: dict, family: Optional[dict] = None,
                     shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> Tuple[_seqabi.SeqCfg, List[_seqabi.LayerCfg]]:
    """config.json of a layer-list family -> the C structs.  Every size and constant comes from the config, or (what
    the config does not give) from a tensor's shape; ``family`` holds what a design fixes (kind of norm, norms after a
    sublayer and on the embedding, whether attention norms q and k, has a sink, gates its heads)."""
    fam = {"norm": "rms", "post_norm": False, "pre_norm": True, "embed_norm": False, "qk_norm": True, "sink": False, "head_gate": False,
           "mask": "block", "ff_act": "geglu", "router": "topk", "expert_act": "cglu", "shared_gate": False}
    fam.update({"v_is_k": False, "rot_layout": "interleaved", "right": "gla", "branch_norm": False})
    fam.update(family or {})
    shapes = shapes or {}

    def per(key: str, kind: str):
        """a family's setting, which may differ by layer type ({type: value}; absent types are off)"""
        v = fam[key]
        return v.get(kind, False) if isinstance(v, dict) else v

    def from_shape(name: str, axis: int, mx: dict, key: str, what: str) -> int:
        if mx.get(key) is not None:
            return int(mx[key])
        if name in shapes:
            return int(shapes[name][axis])
        raise ValueError(f"{what}: the config has no {key!r} and the checkpoint's shape of {name} is not known")

    layers = []
    for i, L in enumerate(cfg["layers"]):
        mx = L["mixer"]
        kind = L["type"]
        lc = _seqabi.LayerCfg()
        lc.kv_from = -1
        if kind == "attention":
            lc.mixer = _seqabi.DN_MIX_ATTENTION
            _attention_cfg(lc, mx, per("qk_norm", kind), fam["mask"], fam["rot_layout"])
            lc.sink, lc.out_gate, lc.v_is_k = int(per("sink", kind)), int(per("head_gate", kind)), int(per("v_is_k", kind))
        elif kind in ("latent_attention", "latent_attention_2"):
            # the second type sends its queries through a normed latent too, pairs rotary dims half apart and gates its heads
            second = kind == "latent_attention_2"
            lc.mixer = _seqabi.DN_MIX_LATENT
            _attention_cfg(lc, {**mx, "kv_heads": 1}, False, fam["mask"])
            lc.rot_part = int(mx.get("rot_dim", lc.rot_dims))
            lc.kv_rank = int(mx["kv_rank"])
            lc.q_rank = from_shape(f"l{i}.mix.dq", 0, mx, "q_rank", f"layer {i}") if second else 0
            lc.rot_layout = _seqabi.DN_ROT_HALF if second else _seqabi.DN_ROT_INTERLEAVED
            lc.out_gate = int(second)
        elif kind == "delta":
            lc.mixer = _seqabi.DN_MIX_DELTA
            lc.heads, lc.kv_heads = int(mx["heads"]), int(mx.get("kv_heads", mx["heads"]))
            lc.dim, lc.vdim = int(mx["dim"]), int(mx.get("vdim", mx["dim"]))
            lc.conv = int(mx.get("conv", 0) or 0)
        elif kind == "parallel":
            lc.mixer = _seqabi.DN_MIX_PARALLEL
            _attention_cfg(lc, mx["left"], per("qk_norm", kind), fam["mask"] if fam["right"] == "gdelta" else "block", fam["rot_layout"])
            lc.sink, lc.out_gate = int(per("sink", kind)), int(per("head_gate", kind))
            r = mx["right"]
            lc.r_heads, lc.r_dim, lc.r_vdim = int(r["heads"]), int(r["dim"]), int(r.get("vdim", r["dim"]))
            if fam["right"] == "gdelta":      # generalized delta rule; the halves' outputs are normed and averaged
                lc.r_kind = _seqabi.DN_RIGHT_GDELTA
                lc.rank = from_shape(f"l{i}.mix.right.w1", 0, r, "rank", f"layer {i}")
                lc.branch_norm = int(fam["branch_norm"])
                lc.left_scale = lc.right_scale = float(fam.get("branch_scale", 1.0))
            else:
                lc.tau = float(r["tau"])
                lc.rank = from_shape(f"l{i}.mix.right.a1", 0, r, "rank", f"layer {i}")
                lc.left_scale, lc.right_scale = float(mx.get("left_scale", 1.0)), float(mx.get("right_scale", 1.0))
        elif kind == "wkv":
            lc.mixer = _seqabi.DN_MIX_WKV
            lc.heads = lc.kv_heads = int(mx["heads"])
            lc.dim = int(mx["dim"])
            if mx.get("vdim") is not None:
                lc.vdim = int(mx["vdim"])
            elif f"l{i}.mix.v" in shapes:
                lc.vdim = int(shapes[f"l{i}.mix.v"][0]) // lc.heads
            else:
                lc.vdim = lc.dim
            lc.rank = from_shape(f"l{i}.mix.w1", 0, mx, "rank", f"layer {i}")
        else:
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        mlp = L.get("mlp")
        if mlp:
            mk = mlp.get("kind", "dense")
            if mk == "dense":
                lc.mlp_kind, lc.ff = _seqabi.DN_MLP_DENSE, int(mlp["ff"])
                lc.ff_act = _seqabi.DN_FF_RELU2 if fam["ff_act"] == "relu2" else _seqabi.DN_FF_GEGLU
            elif mk == "moe":
                lc.mlp_kind = _seqabi.DN_MLP_MOE
                swiglu = fam["expert_act"] == "swiglu"
                lc.expert_act = _seqabi.DN_EXPERT_SWIGLU if swiglu else _seqabi.DN_EXPERT_CGLU
                lc.ff = int(mlp["expert"]["ff"])
                lc.limit = float(mlp["expert"].get("limit", 0.0)) if swiglu else float(mlp["expert"]["limit"])
                r = mlp["router"]
                lc.experts, lc.top = int(r["experts"]), int(r["top"])
                if fam["router"] == "scored":
                    lc.router_kind = _seqabi.DN_ROUTER_SCORED
                    lc.identity = int(r.get("identity", 0) or 0)
                    g = r.get("groups") or {}
                    lc.groups, lc.groups_keep = int(g.get("count", 0) or 0), int(g.get("keep", g.get("count", 0)) or 0)
                    lc.router_scale = float(r.get("scale", 1.0))
                sh = mlp.get("shared")
                if sh:
                    lc.shared_ff = int(sh["ff"])
                    lc.shared_limit = float(sh.get("limit", 0.0)) if swiglu else float(sh["limit"])
                    lc.shared_gate = int(fam["shared_gate"])
            else:
                raise ValueError(f"layer {i}: feed-forward kind {mk!r} unsupported")
        layers.append(lc)
    sc = _seqabi.SeqCfg(width=int(cfg["width"]), vocab=int(cfg["vocab"]), n_layers=len(layers), streams=int(cfg.get("streams", 0) or 0),
                        eps=float((cfg.get("norm") or {}).get("eps", 1e-6)),
                        embed_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)))
    sc.norm_kind = {"dyt": _seqabi.DN_NORM_DYT, "layer": _seqabi.DN_NORM_LAYER}.get(fam["norm"], _seqabi.DN_NORM_RMS)
    sc.canon_taps = int((cfg.get("canon") or {}).get("taps", 0) or 0)
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        sc.bigram_buckets, sc.bigram_mul_prev, sc.bigram_mul_cur = int(bg["buckets"]), int(bg["mul_prev"]), int(bg["mul_cur"])
    sc.logit_scale = float(cfg.get("logit_scale", 1.0))
    sc.post_norm, sc.embed_norm, sc.no_pre_norm = int(fam["post_norm"]), int(fam["embed_norm"]), int(not fam["pre_norm"])
    sc.logit_softcap = float(cfg.get("logit_softcap", 0.0) or 0.0)
    lp = cfg.get("loop")
    if lp:
        sc.loop_start, sc.loop_stop, sc.loop_times = int(lp["start"]), int(lp["stop"]), int(lp["times"])
        if sc.loop_times < 1:
            raise ValueError("loop.times must be at least 1")
    return sc, layers


class SeqMixRingModel(BaseRingModel):
    """A whole layer-list model on one GPU: owns cache pool + state slots, runs ragged-batch steps."""

    model_type: Optional[str] = None
    family: Dict[str, Any] = {}            # what the design fixes (parse_layer_list)
    # checkpoint name of a layer's tensor -> the library's name, per mixer type ("*" for every layer)
    tensor_alias: Dict[str, Dict[str, str]] = {}
    step_kernel_ok = False
    batched_step = True        # ShardRuntime loads it whole and serves it with the `batched` policy over shard.batching.SequenceBatcher

    def __init__(self, model_config: Any, assigned_layers: Optional[List[int]] = None, is_api_layer: bool = False, *,
                 dtype: str = "bfloat16", kv_pool_pages: int = 0, max_seqs: int = 4, max_batch_tokens: int = 2048,
                 tensor_shapes: Optional[Dict[str, Tuple[int, ...]]] = None, **_ignored):
        if is_api_layer and assigned_layers:
            raise RuntimeError("API layer doesn't handle layers")
        self.config = dict(model_config)
        self.model_config = model_config
        sc, layers = parse_layer_list(self.config, self.family, tensor_shapes)
        n = len(layers)
        if assigned_layers is not None and sorted(assigned_layers) != list(range(n)):
            raise ValueError("a layer-list model is served whole by one shard: its layers share pages (kv_from) and fp32 "
                             f"residual streams; assign all {n} layers")
        if dtype in ("bfloat16", "bf16"):
            self.dtype, sc.dtype = torch.bfloat16, _seqabi.DN_SEQ_BF16
        elif dtype in ("float32", "fp32"):
            self.dtype, sc.dtype = torch.float32, _seqabi.DN_SEQ_F32
        else:
            raise ValueError(f"dtype {dtype!r} unsupported (bfloat16 or float32)")
        sc.pool_pages = int(kv_pool_pages) or 64
        sc.max_seqs, sc.max_batch_tokens = int(max_seqs), int(max_batch_tokens)
        self._lib = _seqabi.load()
        self.device = torch.cuda.current_device() if torch.cuda.is_available() else 0
        _seqabi.init(self.device)
        arr = (_seqabi.LayerCfg * n)(*layers)
        h = C.c_void_p()
        _seqabi.check(self._lib.dn_seq_model_create(C.byref(sc), arr, C.byref(h)))
        self._h = h.value
        self._cfg_struct, self._layer_structs = sc, layers
        self.layers = list(range(n))
        self.layer_runs = int(self._lib.dn_seq_layer_runs(self._h))
        self.abs_to_local = {i: i for i in self.layers}
        self.hidden_size, self.vocab_size = int(sc.width), int(sc.vocab)
        self.max_seqs, self.max_batch_tokens, self.pool_pages = int(sc.max_seqs), int(sc.max_batch_tokens), int(sc.pool_pages)
        self._bound: Dict[str, torch.Tensor] = {}

    # -- weights -----------------------------------------------------------------------------
    def expected_tensors(self) -> Dict[str, Tuple[int, ...]]:
        """Checkpoint name -> shape, from the config alone."""
        W, V, S = self.hidden_size, self.vocab_size, int(self._cfg_struct.streams)
        sc = self._cfg_struct
        dyt = sc.norm_kind == _seqabi.DN_NORM_DYT
        lnorm = sc.norm_kind == _seqabi.DN_NORM_LAYER
        out: Dict[str, Tuple[int, ...]] = {"embed": (V, W), "final.norm": (W,)}
        if sc.bigram_buckets > 0:
            out["bigram"] = (sc.bigram_buckets + 1, W)
        if not self.family.get("tied_head"):
            out["head"] = (V, W)

        def norm(name: str) -> None:
            out[name] = (W,)
            if dyt:
                out[name + ".b"], out[name + ".alpha"] = (W,), ()
            if lnorm:
                out[name + ".b"] = (W,)

        norm("final.norm")
        if sc.embed_norm:
            norm("embed.norm")
        if sc.loop_times > 0:
            out["loop.in"] = (W, 2 * W)
        for i, lc in enumerate(self._layer_structs):
            p = f"l{i}."
            att = lc.mixer in (_seqabi.DN_MIX_ATTENTION, _seqabi.DN_MIX_PARALLEL)
            latent = lc.mixer == _seqabi.DN_MIX_LATENT
            cq = (lc.heads if lc.mixer != _seqabi.DN_MIX_DELTA else lc.kv_heads) * lc.dim
            ck, cv = lc.kv_heads * lc.dim, (lc.kv_heads if att else lc.heads) * lc.vdim
            co = lc.heads * lc.vdim
            own = not (att and lc.kv_from >= 0) and not latent
            if not sc.no_pre_norm:
                norm(p + "norm1")
            if sc.canon_taps > 0:
                out[p + "canon1"] = (W, sc.canon_taps)
                if lc.ff > 0:
                    out[p + "canon2"] = (W, sc.canon_taps)
            if sc.post_norm:
                norm(p + "post1")
            out[p + "mix.q"] = (cq, W)
            out[p + "mix.o"] = (W, co)
            if own:
                out[p + "mix.k"], out[p + "mix.v"] = (ck, W), (cv, W)
                if att and lc.v_is_k:
                    del out[p + "mix.v"]
            if latent:
                cq = lc.heads * (lc.dim + lc.rot_part)
                out[p + "mix.q"] = (cq, lc.q_rank if lc.q_rank > 0 else W)
                if lc.q_rank > 0:
                    out[p + "mix.dq"], out[p + "mix.dq.norm"] = (lc.q_rank, W), (lc.q_rank,)
                out[p + "mix.dkv"], out[p + "mix.dkv.norm"] = (lc.kv_rank + lc.rot_part, W), (lc.kv_rank,)
                out[p + "mix.uk"], out[p + "mix.uv"] = (lc.heads * lc.dim, lc.kv_rank), (co, lc.kv_rank)
                if lc.out_gate:
                    out[p + "head_gate"] = (lc.heads, W)
            if lc.conv > 0:
                out[p + "mix.q.conv"] = (cq, lc.conv)
                if own:
                    out[p + "mix.k.conv"], out[p + "mix.v.conv"] = (ck, lc.conv), (cv, lc.conv)
            if att:
                if lc.qk_norm:      # over the whole projection, or per head with one weight for all heads
                    per_head = lc.qk_norm == _seqabi.DN_QKNORM_HEAD
                    out[p + "mix.q.norm"] = (lc.dim,) if per_head else (cq,)
                    if own:
                        out[p + "mix.k.norm"] = (lc.dim,) if per_head else (ck,)
                if lc.sink:
                    out[p + "sink"] = (lc.heads,)
                if lc.out_gate:
                    out[p + "head_gate"] = (lc.heads, W)
            if lc.mixer == _seqabi.DN_MIX_PARALLEL and lc.r_kind == _seqabi.DN_RIGHT_GDELTA:
                rc = lc.r_heads * lc.r_dim
                for q in "qkvga":
                    out[p + "r." + q] = (rc, W)
                out[p + "r.ab"] = out[p + "r.norm"] = out[p + "decay.b"] = (rc,)
                out[p + "decay1"], out[p + "decay2"], out[p + "r.o"] = (lc.rank, W), (rc, lc.rank), (W, rc)
                if lc.branch_norm:
                    out[p + "l.out"] = out[p + "r.out"] = (W,)
            elif lc.mixer == _seqabi.DN_MIX_PARALLEL:
                rc, rv = lc.r_heads * lc.r_dim, lc.r_heads * lc.r_vdim
                out[p + "r.q"] = out[p + "r.k"] = (rc, W)
                out[p + "r.v"] = out[p + "r.g"] = (rv, W)
                out[p + "r.o"], out[p + "r.norm"] = (W, rv), (lc.r_vdim,)
                out[p + "decay1"], out[p + "decay2"], out[p + "decay.b"] = (lc.rank, W), (rc, lc.rank), (rc,)
            elif lc.mixer == _seqabi.DN_MIX_WKV:
                for q in "rkvgw":
                    out[p + "mu." + q] = (W,)
                out[p + "mix.g"], out[p + "mix.norm"] = (co, W), (co,)
                out[p + "decay1"], out[p + "decay2"], out[p + "decay.b"] = (lc.rank, W), (cq, lc.rank), (cq,)
                out[p + "bonus"] = (lc.heads, lc.dim)
            elif lc.mixer == _seqabi.DN_MIX_DELTA:
                out[p + "mix.a"] = out[p + "mix.b"] = (lc.heads, W)
                out[p + "mix.g"] = (co, W)
                out[p + "mix.A_log"] = out[p + "mix.dt_bias"] = (lc.heads,)
                out[p + "mix.norm"] = (lc.vdim,)
            if lc.ff > 0:
                if not sc.no_pre_norm:
                    norm(p + "norm2")
                if sc.post_norm:
                    norm(p + "post2")
                if lc.mlp_kind == _seqabi.DN_MLP_MOE:
                    if lc.router_kind == _seqabi.DN_ROUTER_SCORED:
                        out[p + "router"], out[p + "router.corr"] = (lc.experts + lc.identity, W), (lc.experts + lc.identity,)
                    else:
                        out[p + "router"], out[p + "router.b"] = (lc.experts, W), (lc.experts,)
                    if lc.shared_ff > 0 and lc.shared_gate:
                        out[p + "shared.sg"] = (1, W)
                    for e in range(lc.experts):
                        out[f"{p}mlp.e{e}.gate"] = out[f"{p}mlp.e{e}.up"] = (lc.ff, W)
                        out[f"{p}mlp.e{e}.down"] = (W, lc.ff)
                    if lc.shared_ff > 0:
                        out[p + "shared.gate"] = out[p + "shared.up"] = (lc.shared_ff, W)
                        out[p + "shared.down"] = (W, lc.shared_ff)
                elif lc.ff_act == _seqabi.DN_FF_RELU2:
                    out[p + "mlp.up"], out[p + "mlp.up.b"] = (lc.ff, W), (lc.ff,)
                    out[p + "mlp.down"], out[p + "mlp.down.b"] = (W, lc.ff), (W,)
                else:
                    out[p + "mlp.gate"] = out[p + "mlp.up"] = (lc.ff, W)
                    out[p + "mlp.down"] = (W, lc.ff)
            if S > 0:
                for q in ("hc1", "hc2") if lc.ff > 0 else ("hc1",):
                    out[p + q + ".in"] = out[p + q + ".out"] = (S,)
                    out[p + q + ".mix"] = (S, S)
        return out

    def load_weights(self, file_or_weights, strict: bool = True):
        """Bind tensors by pointer.  Names: the checkpoint's (``l3.mix.q``, ``embed``, ``final.norm``, ``head``) or the
        loader's (``layers.3.mix.q``, ``embed_tokens.weight``, ``norm.weight``, ``lm_head.weight``)."""
        items = file_or_weights.items() if isinstance(file_or_weights, dict) else file_or_weights
        want = self.expected_tensors()
        alias = {"embed_tokens.weight": "embed", "norm.weight": "final.norm", "lm_head.weight": "head"}
        for key, t in items:
            key = key.decode() if isinstance(key, (bytes, bytearray)) else str(key)
            key = key[6:] if key.startswith("model.") else key
            key = alias.get(key, key)
            if key.startswith("layers."):
                _, idx, rest = key.split(".", 2)
                key = f"l{idx}.{rest}"
            if self.tensor_alias and _LAYER_KEY.match(key):
                lname, suffix = key.split(".", 1)
                kind = self.config["layers"][int(lname[1:])]["type"]
                suffix = self.tensor_alias.get(kind, {}).get(suffix, self.tensor_alias.get("*", {}).get(suffix, suffix))
                key = f"{lname}.{suffix}"
            shape = want.get(key)
            if shape is None:
                if strict:
                    raise ValueError(f"unexpected tensor {key}")
                continue
            if shape == () and t.numel() == 1:
                t = t.reshape(())           # a scalar stored as [1]
            if tuple(t.shape) != shape:
                raise ValueError(f"{key}: shape {tuple(t.shape)}, the config asks for {shape}")
            if not t.is_cuda or t.dtype != self.dtype or not t.is_contiguous():
                raise ValueError(f"{key}: expected a contiguous {self.dtype} CUDA tensor")
            if key in _seqabi.MODEL_SLOT:
                _seqabi.check(self._lib.dn_seq_bind(self._h, -1, _seqabi.MODEL_SLOT[key], t.data_ptr()))
            else:
                lname, suffix = key.split(".", 1)
                ex = _EXPERT_KEY.match(suffix)
                if ex:
                    _seqabi.check(self._lib.dn_seq_bind_expert(self._h, int(lname[1:]), int(ex.group(1)), _seqabi.EXPERT_SLOT[ex.group(2)],
                                                               t.data_ptr()))
                else:
                    _seqabi.check(self._lib.dn_seq_bind(self._h, int(lname[1:]), _seqabi.LAYER_SLOT[suffix], t.data_ptr()))
            self._bound[key] = t     # keep the borrowed memory alive
        if self.family.get("tied_head") and "embed" in self._bound:      # logits = embedding table x, the table itself
            _seqabi.check(self._lib.dn_seq_bind(self._h, -1, _seqabi.MODEL_SLOT["head"], self._bound["embed"].data_ptr()))
        return self

    def missing_tensors(self) -> List[str]:
        return sorted(set(self.expected_tensors()) - set(self._bound))

    # -- sequences and the step ----------------------------------------------------------------
    def make_cache(self, max_tokens: int = 0, stream=None) -> SeqHandle:
        return SeqHandle(self, stream)

    @property
    def free_pages(self) -> int:
        return int(self._lib.dn_seq_free_pages(self._h))

    @property
    def free_slots(self) -> int:
        return int(self._lib.dn_seq_free_slots(self._h))

    def step(self, entries: Sequence[Tuple[SeqHandle, Sequence[int]]], want: Sequence[int], stream=None,
             layer_trace: bool = False):
        """One batched step.  entries: (sequence, its next tokens); want: rows of the concatenated tokens whose
        logits are returned as fp32 [len(want), vocab] (None if empty).  With layer_trace also the residual after
        every layer run (a layer inside a loop counts each time), fp32 [layer runs, N, width]."""
        E = len(entries)
        slots = (C.c_int32 * E)(*[h.slot for h, _ in entries])
        counts = (C.c_int32 * E)(*[len(t) for _, t in entries])
        flat = [int(x) for _, t in entries for x in t]
        N = len(flat)
        toks = (C.c_int32 * N)(*flat)
        nw = len(want)
        wr = (C.c_int32 * max(1, nw))(*[int(x) for x in want])
        dev = torch.device("cuda", self.device)
        logits = torch.empty(nw, self.vocab_size, dtype=torch.float32, device=dev) if nw else None
        trace = torch.empty(self.layer_runs, N, self.hidden_size, dtype=torch.float32, device=dev) if layer_trace else None
        _seqabi.check(self._lib.dn_seq_step(self._h, E, slots, counts, toks, nw, wr, logits.data_ptr() if nw else None,
                                            trace.data_ptr() if layer_trace else None, _stream_ptr(stream)))
        return (logits, trace) if layer_trace else logits

    def check(self, stream=None) -> None:
        """Synchronise and raise if a bounded wait inside a kernel ever ran out (results would be invalid)."""
        _seqabi.check(self._lib.dn_seq_check(self._h, _stream_ptr(stream)))

    def profile(self, on: bool) -> None:
        """Switch the per-phase device timers of the step on or off."""
        _seqabi.check(self._lib.dn_seq_profile(self._h, int(bool(on))))

    def set_graphs(self, on: bool) -> None:
        """Decode steps replay a captured CUDA graph (default) or launch their kernels one by one."""
        _seqabi.check(self._lib.dn_seq_set_graphs(self._h, int(bool(on))))

    def profile_read(self, reset: bool = True) -> Dict[str, float]:
        """Milliseconds per phase over the steps run since the last read (synchronises)."""
        ms = (C.c_double * len(_seqabi.PHASES))()
        _seqabi.check(self._lib.dn_seq_profile_read(self._h, ms, int(bool(reset))))
        return {n: float(ms[i]) for i, n in enumerate(_seqabi.PHASES)}

    # -- BaseRingModel surface ---------------------------------------------------------------------
    def _whole(self, *_a, **_k):
        raise NotImplementedError("layer-list models run whole batched steps (SeqMixRingModel.step); the residual between "
                                  "their layers is S fp32 streams, not a [T, hidden] activation of the wire dtype")

    embed = normalize = lm_project = apply_single_layer = _whole

    @property
    def decoding_layers(self):
        return self.layers

    @property
    def head_dim(self) -> Tuple[int, int]:
        lc = self._layer_structs[0]
        return (int(lc.dim), int(lc.vdim))

    @property
    def n_kv_heads(self) -> int:
        return int(self._layer_structs[0].kv_heads)

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    def unload_layers(self, abs_layers: List[int]) -> None:
        raise NotImplementedError("layer-list models stay resident")

    def is_bound(self, abs_layer: int) -> bool:
        return not any(k.startswith(f"l{abs_layer}.") for k in self.missing_tensors())

    def apply_quantization_from_config(self, model_config: Any, model_metadata: Any) -> bool:
        return False

    def destroy(self) -> None:
        if getattr(self, "_h", None):
            self._lib.dn_seq_model_destroy(self._h)
            self._h = None
            self._bound.clear()


class MoputarRingModel(SeqMixRingModel):
    """Moputar: chunk-masked attention layers (some reading an earlier layer's keys and values) interleaved with
    gated delta-rule layers, short convolutions on q / k / v, hyper-connected residual streams."""

    model_type = "moputar"


_NORM_ALIAS = {f"{a}{x}": f"{b}{x}" for a, b in (("norm1b", "post1"), ("norm2b", "post2")) for x in ("", ".b", ".alpha")}
_MOE_ALIAS = {"mlp.router": "router", "mlp.router.b": "router.b", "mlp.shared.gate": "shared.gate", "mlp.shared.up": "shared.up",
              "mlp.shared.down": "shared.down"}


class FilinexRingModel(SeqMixRingModel):
    """Filinex: every norm a dynamic tanh, before and after each sublayer and on the embedding; layers are either a
    parallel mixer (softmax attention with capped scores, a sink and gated heads beside a gated linear attention with
    a decay per key channel) or a wkv mixer (token-shift mixing, decayed state read with a bonus for the current
    token); routed clamped-GLU experts with a shared one; a span of layers that runs several times with the
    embedding fed back in before each pass; capped logits."""

    model_type = "filinex"
    family = {"norm": "dyt", "post_norm": True, "embed_norm": True, "qk_norm": False, "sink": True, "head_gate": True}
    tensor_alias = {
        "*": {**_NORM_ALIAS, **_MOE_ALIAS},
        "parallel": {"mix.left.q": "mix.q", "mix.left.k": "mix.k", "mix.left.v": "mix.v", "mix.left.o": "mix.o", "mix.left.sink": "sink",
                     "mix.left.g": "head_gate", "mix.right.q": "r.q", "mix.right.k": "r.k", "mix.right.v": "r.v", "mix.right.g": "r.g",
                     "mix.right.o": "r.o", "mix.right.norm": "r.norm", "mix.right.a1": "decay1", "mix.right.a2": "decay2",
                     "mix.right.a2.b": "decay.b"},
        "wkv": {"mix.r": "mix.q", "mix.mu.r": "mu.r", "mix.mu.k": "mu.k", "mix.mu.v": "mu.v", "mix.mu.g": "mu.g", "mix.mu.w": "mu.w",
                "mix.w1": "decay1", "mix.w2": "decay2", "mix.w0": "decay.b", "mix.u": "bonus"},
    }


class LutesunRingModel(SeqMixRingModel):
    """Lutesun: latent-attention layers under a sliding window -- the cache keeps one compressed row per token, of which
    every head's keys and values are up-projections; the second layer type also compresses its queries, pairs rotary dims
    half apart and gates its heads --, RMS norms on the sublayers' outputs only, a dense relu-squared feed-forward with
    biases or experts routed by corrected, group-limited softmax scores (identity experts among them) with a gated shared
    expert; scaled embedding whose table is also the output head."""

    model_type = "lutesun"
    family = {"norm": "rms", "post_norm": True, "pre_norm": False, "qk_norm": False, "tied_head": True, "mask": "window",
              "ff_act": "relu2", "router": "scored", "expert_act": "swiglu", "shared_gate": True}
    tensor_alias = {
        "*": {"norm1": "post1", "norm2": "post2", **_MOE_ALIAS, "mlp.correction": "router.corr", "mlp.shared.sg": "shared.sg"},
        "latent_attention_2": {"mix.uq": "mix.q", "mix.g": "head_gate"},
    }


class VulanexRingModel(SeqMixRingModel):
    """Vulanex: layer norms with bias before every sublayer, whose input then passes a short causal convolution over time
    (its last inputs carried per sequence); the embedding adds a row of a hashed (previous token, token) table; layers are
    either GQA attention whose values are its keys, without positions but with a query scale that grows with the logarithm
    of the position, or a parallel mixer -- attention with per-head q / k norms, interpolated rotary frequencies, a
    sliding window behind which blocks of tokens are seen as one mean key / value each, and a sink, beside a generalized
    delta rule with a decay and a removal rate per key channel -- whose two outputs are RMS-normed and averaged; a dense
    gelu-gated feed-forward; the embedding table is the output head and the logits are scaled."""

    model_type = "vulanex"
    family = {"norm": "layer", "tied_head": True, "mask": "window", "rot_layout": "half", "right": "gdelta", "branch_norm": True,
              "branch_scale": 0.5, "qk_norm": {"parallel": "head"}, "sink": {"parallel": True}, "v_is_k": {"attention": True}}
    tensor_alias = {
        "parallel": {"mix.left.q": "mix.q", "mix.left.k": "mix.k", "mix.left.v": "mix.v", "mix.left.o": "mix.o", "mix.left.q.norm": "mix.q.norm",
                     "mix.left.k.norm": "mix.k.norm", "mix.left.sink": "sink", "mix.left.out": "l.out", "mix.right.out": "r.out",
                     "mix.right.r": "r.q", "mix.right.k": "r.k", "mix.right.v": "r.v", "mix.right.g": "r.g", "mix.right.a": "r.a",
                     "mix.right.a.b": "r.ab", "mix.right.w1": "decay1", "mix.right.w2": "decay2", "mix.right.w0": "decay.b",
                     "mix.right.norm": "r.norm", "mix.right.o": "r.o"},
    }
