"""ctypes binding of libdnet_b200_seq.so (include/dnet_b200_seq.h): the batched step of models built from
sequence mixers.  Built in-tree on first use; no CPU fallback -- every call checks its return code."""
from __future__ import annotations

import ctypes as C
import os
import re
from pathlib import Path
from typing import List

from dnet_b200._cabi import DnError

_ROOT = Path(__file__).resolve().parent
HEADER_PATH = _ROOT.parent / "include" / "dnet_b200_seq.h"

DN_SEQ_BF16, DN_SEQ_F32 = 0, 1
DN_MIX_ATTENTION, DN_MIX_DELTA, DN_MIX_PARALLEL, DN_MIX_WKV, DN_MIX_LATENT = 0, 1, 2, 3, 4
DN_MASK_BLOCK, DN_MASK_WINDOW = 0, 1
DN_ROT_INTERLEAVED, DN_ROT_HALF = 0, 1
DN_NORM_RMS, DN_NORM_DYT, DN_NORM_LAYER = 0, 1, 2
DN_QKNORM_NONE, DN_QKNORM_WHOLE, DN_QKNORM_HEAD = 0, 1, 2
DN_RIGHT_GLA, DN_RIGHT_GDELTA = 0, 1
DN_MLP_DENSE, DN_MLP_MOE = 0, 1
DN_FF_GEGLU, DN_FF_RELU2 = 0, 1
DN_ROUTER_TOPK, DN_ROUTER_SCORED = 0, 1
DN_EXPERT_CGLU, DN_EXPERT_SWIGLU = 0, 1
# dn_seq_bind slots, in the header's order
_LAYER_SLOTS = ["norm1", "norm2", "mix.q", "mix.k", "mix.v", "mix.o", "mix.q.conv", "mix.k.conv", "mix.v.conv", "mix.q.norm",
                "mix.k.norm", "mix.a", "mix.b", "mix.g", "mix.A_log", "mix.dt_bias", "mix.norm", "mlp.gate", "mlp.up", "mlp.down",
                "hc1.in", "hc1.out", "hc1.mix", "hc2.in", "hc2.out", "hc2.mix",
                "norm1.b", "norm1.alpha", "norm2.b", "norm2.alpha",
                "post1", "post1.b", "post1.alpha", "post2", "post2.b", "post2.alpha",
                "sink", "head_gate",
                "r.q", "r.k", "r.v", "r.g", "r.o", "r.norm",
                "decay1", "decay2", "decay.b",
                "mu.r", "mu.k", "mu.v", "mu.g", "mu.w", "bonus",
                "router", "router.b", "shared.gate", "shared.up", "shared.down",
                "mix.dq", "mix.dq.norm", "mix.dkv", "mix.dkv.norm", "mix.uk", "mix.uv",
                "mlp.up.b", "mlp.down.b", "router.corr", "shared.sg",
                "canon1", "canon2", "l.out", "r.out", "r.a", "r.ab"]
LAYER_SLOT = {n: i for i, n in enumerate(_LAYER_SLOTS)}
MODEL_SLOT = {"embed": 100, "final.norm": 101, "head": 102, "final.norm.b": 103, "final.norm.alpha": 104,
              "embed.norm": 105, "embed.norm.b": 106, "embed.norm.alpha": 107, "loop.in": 108, "bigram": 109}
EXPERT_SLOT = {"gate": 0, "up": 1, "down": 2}
# phases of a step, in the header's order (dn_seq_profile_read)
PHASES = ["embed", "norm", "proj", "attn_prep", "attn", "delta_prep", "delta_rule", "delta_out", "conv_carry", "out_proj",
          "write_back", "ff_up", "ff_down", "head", "other", "recur_prep", "recur", "recur_out", "router", "moe_up", "moe_down",
          "latent_in", "latent_out", "canon"]


class LayerCfg(C.Structure):
    _fields_ = [("mixer", C.c_int32), ("heads", C.c_int32), ("kv_heads", C.c_int32), ("dim", C.c_int32), ("vdim", C.c_int32),
                ("conv", C.c_int32), ("chunk", C.c_int32), ("rot_dims", C.c_int32), ("rot_base", C.c_float), ("scale", C.c_float),
                ("kv_from", C.c_int32), ("ff", C.c_int32),
                ("qk_norm", C.c_int32), ("softcap", C.c_float), ("sink", C.c_int32), ("out_gate", C.c_int32),
                ("r_heads", C.c_int32), ("r_dim", C.c_int32), ("r_vdim", C.c_int32), ("rank", C.c_int32), ("tau", C.c_float),
                ("left_scale", C.c_float), ("right_scale", C.c_float),
                ("mlp_kind", C.c_int32), ("experts", C.c_int32), ("top", C.c_int32), ("limit", C.c_float),
                ("shared_ff", C.c_int32), ("shared_limit", C.c_float),
                ("mask_kind", C.c_int32), ("rot_layout", C.c_int32), ("kv_rank", C.c_int32), ("q_rank", C.c_int32), ("rot_part", C.c_int32),
                ("ff_act", C.c_int32), ("router_kind", C.c_int32), ("expert_act", C.c_int32), ("identity", C.c_int32),
                ("groups", C.c_int32), ("groups_keep", C.c_int32), ("router_scale", C.c_float), ("shared_gate", C.c_int32),
                ("v_is_k", C.c_int32), ("qtemp_coef", C.c_float), ("qtemp_every", C.c_int32), ("pool", C.c_int32),
                ("yarn_factor", C.c_float), ("yarn_original", C.c_float), ("yarn_fast", C.c_float), ("yarn_slow", C.c_float),
                ("r_kind", C.c_int32), ("branch_norm", C.c_int32)]


class SeqCfg(C.Structure):
    _fields_ = [("width", C.c_int32), ("vocab", C.c_int32), ("n_layers", C.c_int32), ("streams", C.c_int32), ("dtype", C.c_int32),
                ("eps", C.c_float), ("embed_scale", C.c_float), ("pool_pages", C.c_int32), ("max_seqs", C.c_int32),
                ("max_batch_tokens", C.c_int32),
                ("norm_kind", C.c_int32), ("post_norm", C.c_int32), ("embed_norm", C.c_int32), ("logit_softcap", C.c_float),
                ("loop_start", C.c_int32), ("loop_stop", C.c_int32), ("loop_times", C.c_int32), ("no_pre_norm", C.c_int32),
                ("canon_taps", C.c_int32), ("bigram_buckets", C.c_int32), ("bigram_mul_prev", C.c_int32), ("bigram_mul_cur", C.c_int32),
                ("logit_scale", C.c_float)]


def declared_symbols() -> List[str]:
    txt = re.sub(r"/\*.*?\*/", "", HEADER_PATH.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(dn_seq_[a-z0-9_]+)\s*\(", txt)))


_vp, _i = C.c_void_p, C.c_int
_I32P = C.POINTER(C.c_int32)
_PROTOS = {
    "dn_seq_init": (_i, [_i]),
    "dn_seq_last_error": (C.c_char_p, []),
    "dn_seq_launch_count": (C.c_int64, []),
    "dn_seq_model_create": (_i, [C.POINTER(SeqCfg), C.POINTER(LayerCfg), C.POINTER(_vp)]),
    "dn_seq_model_destroy": (_i, [_vp]),
    "dn_seq_bind": (_i, [_vp, _i, _i, _vp]),
    "dn_seq_bind_expert": (_i, [_vp, _i, _i, _i, _vp]),
    "dn_seq_layer_runs": (_i, [_vp]),
    "dn_seq_open": (_i, [_vp, _vp, C.POINTER(_i)]),
    "dn_seq_close": (_i, [_vp, _i]),
    "dn_seq_length": (_i, [_vp, _i]),
    "dn_seq_free_pages": (_i, [_vp]),
    "dn_seq_free_slots": (_i, [_vp]),
    "dn_seq_check": (_i, [_vp, _vp]),
    "dn_seq_profile": (_i, [_vp, _i]),
    "dn_seq_profile_read": (_i, [_vp, C.POINTER(C.c_double), _i]),
    "dn_seq_set_graphs": (_i, [_vp, _i]),
    "dn_seq_step": (_i, [_vp, _i, _I32P, _I32P, _I32P, _i, _I32P, _vp, _vp, _vp]),
}
_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        path = os.environ.get("DNET_B200_SEQ_LIB")
        if not path:
            from dnet_b200 import build as b

            path = str(b.build_seq())
        lib = C.CDLL(path)
        for name, (res, args) in _PROTOS.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(rc: int) -> int:
    if rc < 0:
        raise DnError(rc, load().dn_seq_last_error().decode("utf-8", "replace"))
    return rc


_inited = set()


def init(device: int) -> None:
    if device not in _inited:
        check(load().dn_seq_init(int(device)))
        _inited.add(device)
