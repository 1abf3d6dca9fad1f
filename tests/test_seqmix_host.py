"""Host-side pieces of the layer-list families that need no GPU: config parsing, checkpoint naming, the oracle's
own mechanisms against independent formulations, and the batcher's token loop over a fake model."""
from __future__ import annotations

import math

import pytest
import torch

from oracle import seqmix_oracle as so

CFG = {"architecture": "Moputar", "vocab": 50, "width": 32, "streams": 2, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
       "layers": [
           {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "conv": 3, "scale": 0.3,
                                           "rot": {"base": 777.0, "dims": 4}, "mask": {"size": 11}}, "mlp": {"kind": "dense", "ff": 40}},
           {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "conv": 3, "scale": 0.3, "kv_from": 0,
                                           "rot": {"base": 777.0, "dims": 4}, "mask": {"size": 11}}, "mlp": None},
           {"type": "delta", "mixer": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 16, "conv": 2}, "mlp": None}]}


def test_config_to_structs():
    from dnet_b200 import _seqabi
    from dnet_b200.core.models.seqmix import parse_layer_list

    sc, layers = parse_layer_list(CFG)
    assert (sc.width, sc.vocab, sc.n_layers, sc.streams) == (32, 50, 3, 2)
    assert abs(sc.eps - 1e-5) < 1e-12 and sc.embed_scale == 2.0
    a, b, d = layers
    assert (a.mixer, a.heads, a.kv_heads, a.dim, a.vdim, a.conv, a.chunk, a.rot_dims, a.kv_from, a.ff) == \
        (_seqabi.DN_MIX_ATTENTION, 4, 2, 8, 12, 3, 11, 4, -1, 40)
    assert abs(a.rot_base - 777.0) < 1e-3 and abs(a.scale - 0.3) < 1e-7
    assert b.kv_from == 0 and b.ff == 0
    assert (d.mixer, d.heads, d.kv_heads, d.dim, d.vdim, d.conv, d.ff) == (_seqabi.DN_MIX_DELTA, 2, 1, 8, 16, 2, 0)
    # absent keys switch the mechanism off
    bare = {"vocab": 5, "width": 8, "layers": [{"type": "attention", "mixer": {"heads": 2, "dim": 4}, "mlp": None}]}
    sc, (l0,) = parse_layer_list(bare)
    assert (sc.streams, l0.kv_heads, l0.vdim, l0.conv, l0.chunk, l0.rot_dims, l0.kv_from) == (0, 2, 4, 0, 0, 0, -1)
    assert abs(l0.scale - 0.5) < 1e-7


def test_checkpoint_names_reach_the_registry():
    from dnet_b200.core.models import MoputarRingModel, SeqMixRingModel
    from dnet_b200.utils.model import HostDictSource, get_model_metadata

    w = so.random_weights(CFG, 0)
    md = get_model_metadata(HostDictSource(w, CFG))
    assert md.model_type == "moputar" and md.num_layers == 3
    assert set(md.weight_info[1]) == {"norm1", "mix.q", "mix.q.conv", "mix.q.norm", "mix.o", "hc1.in", "hc1.out", "hc1.mix"}
    assert md.embed_tokens["weight"].shape == (50, 32) and md.norm["weight"].shape == (32,) and md.lm_head["weight"].shape == (50, 32)
    assert MoputarRingModel.model_type == "moputar" and issubclass(MoputarRingModel, SeqMixRingModel)
    assert set(so.tensor_shapes(CFG)) == set(w)


def test_header_and_binding_agree():
    import re

    from dnet_b200 import _seqabi

    assert set(_seqabi.declared_symbols()) == set(_seqabi._PROTOS)
    txt = re.sub(r"/\*.*?\*/", "", _seqabi.HEADER_PATH.read_text(), flags=re.S)
    body = txt.split("DN_SQ_NORM1 = 0", 1)[1].split("DN_SQ_COUNT", 1)[0]
    order = ["DN_SQ_NORM1"] + [n.strip() for n in body.replace("\n", " ").split(",") if n.strip()]
    assert len(order) == len(_seqabi.LAYER_SLOT)
    spell = {"OUT_NORM": "mix.norm", "NORM1": "norm1", "NORM2": "norm2", "GATE": "mlp.gate", "UP": "mlp.up", "DOWN": "mlp.down",
             "HEAD_GATE": "head_gate", "SINK": "sink", "BONUS": "bonus", "DECAY1": "decay1", "DECAY2": "decay2", "DECAY_B": "decay.b",
             "ROUTER": "router", "ROUTER_B": "router.b", "SH_GATE": "shared.gate", "SH_UP": "shared.up", "SH_DOWN": "shared.down",
             "UP_B": "mlp.up.b", "DOWN_B": "mlp.down.b", "ROUTER_CORR": "router.corr", "SH_SG": "shared.sg",
             "CANON1": "canon1", "CANON2": "canon2", "L_OUT": "l.out"}
    for i, name in enumerate(order):
        n = name[len("DN_SQ_"):]
        if n in spell:
            want = spell[n]
        elif n.startswith(("HC", "NORM", "POST", "R_", "MU_")):
            want = n.lower().replace("_", ".", 1)
        else:
            want = "mix." + {"A_LOG": "A_log", "DT_BIAS": "dt_bias"}.get(n, n.lower().replace("_", "."))
        assert _seqabi.LAYER_SLOT[want] == i, (name, want)
    model = [n.strip().split("=")[0].strip() for n in txt.split("DN_SQ_COUNT,", 1)[1].split("}", 1)[0].replace("\n", " ").split(",") if n.strip()]
    assert [_seqabi.MODEL_SLOT[k] for k in ("embed", "final.norm", "head", "final.norm.b", "final.norm.alpha", "embed.norm", "embed.norm.b",
                                           "embed.norm.alpha", "loop.in", "bigram")] == list(range(100, 100 + len(model)))


def _filinex_cfg():
    moe = {"kind": "moe", "router": {"experts": 5, "top": 2}, "expert": {"ff": 24, "limit": 1.5}, "shared": {"ff": 16, "limit": 0.5}}
    return {"architecture": "Filinex", "vocab": 50, "width": 32, "norm": {"eps": 1e-5}, "logit_softcap": 7.0,
            "loop": {"start": 1, "stop": 3, "times": 4},
            "layers": [{"type": "wkv", "mixer": {"heads": 2, "dim": 8}, "mlp": moe},
                       {"type": "parallel", "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "scale": 0.2, "softcap": 20.0},
                                                      "right": {"heads": 3, "dim": 8, "vdim": 4, "tau": 8.0}, "left_scale": 0.7, "right_scale": 0.3},
                        "mlp": {**moe, "shared": None}},
                       {"type": "wkv", "mixer": {"heads": 1, "dim": 16}, "mlp": None}]}


def test_filinex_config_and_checkpoint_names():
    """every tensor of a checkpoint finds its place: the names the oracle writes, through the class's aliases, are
    the names the model expects, with the shapes; sizes the config lacks come from the tensors"""
    from dnet_b200 import _seqabi
    from dnet_b200.core.models import ring_model_class
    from dnet_b200.core.models.seqmix import _LAYER_KEY, parse_layer_list
    from oracle import filinex_oracle as fo

    cfg = _filinex_cfg()
    cls = ring_model_class("filinex")
    shapes = fo.tensor_shapes(cfg, rank=6)
    shapes["l2.mix.v"] = shapes["l2.mix.g"] = (24, 32)       # a value size that differs from the key size
    shapes["l2.mix.norm"], shapes["l2.mix.o"] = (24,), (32, 24)
    sc, layers = parse_layer_list(cfg, cls.family, shapes)
    assert (sc.norm_kind, sc.post_norm, sc.embed_norm) == (_seqabi.DN_NORM_DYT, 1, 1)
    assert (sc.loop_start, sc.loop_stop, sc.loop_times) == (1, 3, 4) and abs(sc.logit_softcap - 7.0) < 1e-6
    assert [l.mixer for l in layers] == [_seqabi.DN_MIX_WKV, _seqabi.DN_MIX_PARALLEL, _seqabi.DN_MIX_WKV]
    assert (layers[0].rank, layers[1].rank, layers[2].vdim) == (6, 6, 24)
    assert (layers[1].sink, layers[1].out_gate, layers[1].qk_norm, layers[1].r_heads, layers[1].shared_ff) == (1, 1, 0, 3, 0)
    assert (layers[0].experts, layers[0].top, layers[0].ff, layers[0].shared_ff, layers[2].ff) == (5, 2, 24, 16, 0)
    with pytest.raises(ValueError):
        parse_layer_list(cfg, cls.family, None)              # the inner size of the decay projection is in no config key
    m = cls.__new__(cls)
    m.config, m._cfg_struct, m._layer_structs, m.hidden_size, m.vocab_size = cfg, sc, layers, sc.width, sc.vocab
    want = m.expected_tensors()
    got = {}
    for key, sh in shapes.items():
        if _LAYER_KEY.match(key):
            lname, suffix = key.split(".", 1)
            kind = cfg["layers"][int(lname[1:])]["type"]
            suffix = cls.tensor_alias.get(kind, {}).get(suffix, cls.tensor_alias["*"].get(suffix, suffix))
            key = f"{lname}.{suffix}"
        got[key] = tuple(sh)
    assert got == {k: tuple(v) for k, v in want.items()}
    for k in want:
        if _LAYER_KEY.match(k) and ".mlp.e" not in k:
            assert k.split(".", 1)[1] in _seqabi.LAYER_SLOT, k


def _lutesun_cfg():
    moe = {"kind": "moe", "router": {"experts": 6, "top": 2, "identity": 2, "scale": 1.5, "groups": {"count": 4, "keep": 3}}, "expert": {"ff": 24},
           "shared": {"ff": 16}}
    mx = {"heads": 3, "dim": 10, "rot_dim": 6, "vdim": 7, "kv_rank": 20, "scale": 0.3, "rot": {"base": 777.0, "dims": 6}, "mask": {"size": 9}}
    return {"architecture": "Lutesun", "vocab": 50, "width": 32, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.25},
            "layers": [{"type": "latent_attention", "mixer": mx, "mlp": {"kind": "dense", "ff": 40}},
                       {"type": "latent_attention_2", "mixer": {**mx, "q_rank": 12, "heads": 2}, "mlp": moe},
                       {"type": "latent_attention", "mixer": {**mx, "mask": None}, "mlp": {**moe, "shared": None, "router": {"experts": 4, "top": 1}}},
                       {"type": "latent_attention_2", "mixer": {k: v for k, v in mx.items() if k != "q_rank"}, "mlp": None}]}


def test_lutesun_config_and_checkpoint_names():
    """every constant of the config lands in the structs, what the design fixes comes from the family, a size the config
    lacks comes from a tensor's shape, and every tensor the oracle writes finds its place through the aliases"""
    from dnet_b200 import _seqabi
    from dnet_b200.core.models import ring_model_class
    from dnet_b200.core.models.seqmix import _LAYER_KEY, parse_layer_list
    from oracle import lutesun_oracle as lo

    cfg = _lutesun_cfg()
    cls = ring_model_class("lutesun")
    with_rank = {**cfg, "layers": cfg["layers"][:3] + [{**cfg["layers"][3], "mixer": {**cfg["layers"][3]["mixer"], "q_rank": 5}}]}
    shapes = lo.tensor_shapes(with_rank)
    with pytest.raises(ValueError):
        parse_layer_list(cfg, cls.family, None)              # the last layer's query latent size is in no config key
    sc, layers = parse_layer_list(cfg, cls.family, shapes)
    assert (sc.norm_kind, sc.post_norm, sc.no_pre_norm, sc.embed_norm, sc.streams) == (_seqabi.DN_NORM_RMS, 1, 1, 0, 0)
    assert abs(sc.embed_scale - 0.25) < 1e-7 and abs(sc.eps - 1e-5) < 1e-9
    assert all(l.mixer == _seqabi.DN_MIX_LATENT and l.kv_heads == 1 and l.kv_rank == 20 and l.rot_part == 6 and l.rot_dims == 6 for l in layers)
    assert [l.q_rank for l in layers] == [0, 12, 0, 5] and [l.out_gate for l in layers] == [0, 1, 0, 1]
    assert [l.rot_layout for l in layers] == [_seqabi.DN_ROT_INTERLEAVED, _seqabi.DN_ROT_HALF] * 2
    assert [l.chunk for l in layers] == [9, 9, 0, 9] and all(l.mask_kind == _seqabi.DN_MASK_WINDOW for l in layers)
    assert (layers[0].mlp_kind, layers[0].ff, layers[0].ff_act) == (_seqabi.DN_MLP_DENSE, 40, _seqabi.DN_FF_RELU2)
    m1 = layers[1]
    assert (m1.mlp_kind, m1.router_kind, m1.expert_act) == (_seqabi.DN_MLP_MOE, _seqabi.DN_ROUTER_SCORED, _seqabi.DN_EXPERT_SWIGLU)
    assert (m1.experts, m1.identity, m1.top, m1.groups, m1.groups_keep, m1.ff, m1.shared_ff, m1.shared_gate) == (6, 2, 2, 4, 3, 24, 16, 1)
    assert abs(m1.router_scale - 1.5) < 1e-7
    m2 = layers[2]
    assert (m2.experts, m2.identity, m2.top, m2.groups, m2.shared_ff, m2.shared_gate) == (4, 0, 1, 0, 0, 0) and abs(m2.router_scale - 1.0) < 1e-7
    assert layers[3].ff == 0
    m = cls.__new__(cls)
    m.config, m._cfg_struct, m._layer_structs, m.hidden_size, m.vocab_size = cfg, sc, layers, sc.width, sc.vocab
    want = m.expected_tensors()
    assert "head" not in want                                # the embedding table is the head
    got = {}
    for key, sh in shapes.items():
        if _LAYER_KEY.match(key):
            lname, suffix = key.split(".", 1)
            kind = cfg["layers"][int(lname[1:])]["type"]
            suffix = cls.tensor_alias.get(kind, {}).get(suffix, cls.tensor_alias["*"].get(suffix, suffix))
            key = f"{lname}.{suffix}"
        got[key] = tuple(sh)
    assert got == {k: tuple(v) for k, v in want.items()}
    for k in want:
        if _LAYER_KEY.match(k) and ".mlp.e" not in k:
            assert k.split(".", 1)[1] in _seqabi.LAYER_SLOT, k


def test_lutesun_oracle_by_hand():
    """the oracle's pieces on numbers small enough to follow"""
    from oracle import lutesun_oracle as lo

    z = torch.log(torch.tensor([0.05, 0.30, 0.10, 0.25, 0.20, 0.10], dtype=torch.float64))
    corr = torch.tensor([0.0, 0.0, 0.5, 0.0, 0.0, 0.0], dtype=torch.float64)
    # groups (0,1) (2,3) (4,5): best corrected scores 0.30, 0.60, 0.20 -> keep the first two; choices 2 (0.60) and 1 (0.30)
    ch, wt = lo.scored_router(z, corr, top=2, groups=3, keep=2, scale=2.0)
    assert ch == [2, 1]
    assert abs(wt[0] - 2.0 * 0.10 / 0.40) < 1e-12 and abs(wt[1] - 2.0 * 0.30 / 0.40) < 1e-12
    ch, _ = lo.scored_router(z, None, top=3, groups=3, keep=1, scale=1.0)         # only group 0 is left: 1, 0, then nothing else
    assert ch == [1, 0]
    ch, _ = lo.scored_router(z, -corr * 10, top=2, groups=0, keep=0, scale=1.0)   # a negative choice score still beats a dropped one
    assert ch == [1, 3]
    # window: a query sees itself and size - 1 tokens before it
    vis = lo.window_mask(6, 3)
    assert vis[4].tolist() == [False, False, True, True, True, False] and vis[1].tolist() == [True, True, False, False, False, False]
    assert lo.window_mask(4, 0).tolist() == torch.ones(4, 4).tril().bool().tolist() and lo.window_mask(3, 1).tolist() == torch.eye(3).bool().tolist()
    # rotary: both layouts keep lengths, leave the tail alone, and make scores depend on the distance only; they pair differently
    z = torch.randn(5, 2, 6, dtype=torch.float64)
    for layout in ("interleaved", "half"):
        r = lo.rotary(z, torch.arange(5), 4, 100.0, layout)
        assert torch.equal(r[..., 4:], z[..., 4:]) and torch.allclose(r[0], z[0]) and torch.allclose(r.pow(2).sum(-1), z.pow(2).sum(-1))
        q, k = torch.randn(1, 4, dtype=torch.float64), torch.randn(1, 4, dtype=torch.float64)
        s = [float((lo.rotary(q, torch.tensor([a]), 4, 100.0, layout) * lo.rotary(k, torch.tensor([a - 3]), 4, 100.0, layout)).sum()) for a in (3, 50)]
        assert abs(s[0] - s[1]) < 1e-9
    e0 = torch.tensor([[1.0, 0.0, 0.0, 0.0]], dtype=torch.float64)
    quarter = torch.tensor([1])      # frequency 1 on pair 0: position 1 turns it by one radian
    a, b = lo.rotary(e0, quarter, 4, 100.0, "interleaved")[0], lo.rotary(e0, quarter, 4, 100.0, "half")[0]
    assert abs(float(a[1]) - math.sin(1.0)) < 1e-12 and abs(float(b[2]) - math.sin(1.0)) < 1e-12 and float(a[2]) == 0.0 and float(b[1]) == 0.0
    # norms: the one-plus weight is stored around zero
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    assert torch.allclose(lo.rms_one_plus(x, torch.zeros(2, dtype=torch.float64), 0.0), lo.rms_plain(x, torch.ones(2, dtype=torch.float64), 0.0))
    assert torch.allclose(lo.unit_rms(x, 0.0), x / math.sqrt(12.5))


def test_filinex_oracle_recurrences_by_hand():
    from oracle import filinex_oracle as fo

    one = torch.ones(2, 1, dtype=torch.float64)
    v = torch.tensor([[1.0], [10.0]], dtype=torch.float64)
    half = torch.full((2, 1), 0.5, dtype=torch.float64)
    # read after the write: o_1 = 0.5 * 1 + 10
    assert torch.allclose(fo.decayed_outer_recurrence(one, one, v, half, None)[:, 0], torch.tensor([1.0, 10.5], dtype=torch.float64))
    # read before it, the current token through the bonus: o_0 = 3 * 1, o_1 = 1 + 3 * 10
    bonus = torch.tensor([3.0], dtype=torch.float64)
    assert torch.allclose(fo.decayed_outer_recurrence(one, one, v, half, bonus)[:, 0], torch.tensor([3.0, 31.0], dtype=torch.float64))
    # a sink as large as the only score halves the weight of the only key
    q = k = torch.ones(1, 1, 1, dtype=torch.float64)
    val = torch.full((1, 1, 1), 8.0, dtype=torch.float64)
    assert torch.allclose(fo.sink_attention(q, k, val, 2.0, 0.0, torch.tensor([2.0])), torch.full((1, 1, 1), 4.0, dtype=torch.float64))
    # the cap bounds the scaled score: with cap 1 a score of 100 counts as 1
    assert torch.allclose(fo.sink_attention(q, k, val, 100.0, 1.0, torch.tensor([1.0])), torch.full((1, 1, 1), 4.0, dtype=torch.float64), atol=1e-9)


def test_oracle_conv_is_a_causal_depthwise_fir():
    g = torch.Generator().manual_seed(0)
    u, w = torch.randn(9, 5, generator=g, dtype=torch.float64), torch.randn(5, 3, generator=g, dtype=torch.float64)
    ref = torch.nn.functional.conv1d(torch.nn.functional.pad(u.T[None], (2, 0)), w[:, None, :], groups=5)[0].T
    assert torch.allclose(so.short_conv(u, w), ref, atol=1e-12)
    assert torch.equal(so.short_conv(u, None), u)


def test_oracle_delta_rule_writes_and_reads_back():
    # with no decay and beta = 1 an orthonormal key's value is stored exactly and replaced exactly
    k = torch.eye(4, dtype=torch.float64)[[0, 1, 0]]
    v = torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]], dtype=torch.float64)
    o = so.delta_rule(k, k, v, torch.ones(3, dtype=torch.float64), torch.ones(3, dtype=torch.float64))
    assert torch.allclose(o, v)
    # decay scales what was stored before the current write
    o = so.delta_rule(torch.eye(4, dtype=torch.float64)[[0, 0]], k[:2], v[:2], torch.zeros(2, dtype=torch.float64).add(1.0),
                      torch.tensor([1.0, 0.5], dtype=torch.float64))
    assert torch.allclose(o[1], 0.5 * v[0])


def test_oracle_block_mask_and_rotation():
    ok = so.visible(7, 3)
    assert ok[5].tolist() == [False, False, False, True, True, True, False] and ok[3].tolist() == [False] * 3 + [True] + [False] * 3
    assert so.visible(4, 0).tolist() == torch.ones(4, 4).tril().bool().tolist()
    z = torch.randn(5, 2, 6, dtype=torch.float64)
    r = so.rotate_pairs(z, torch.arange(5), 4, 100.0)
    assert torch.equal(r[..., 4:], z[..., 4:]) and torch.allclose(r[0], z[0])
    assert torch.allclose(r.pow(2).sum(-1), z.pow(2).sum(-1))
    # scores depend on the distance only
    q, k = torch.randn(1, 1, 4, dtype=torch.float64), torch.randn(1, 1, 4, dtype=torch.float64)
    s = [float((so.rotate_pairs(q, torch.tensor([a]), 4, 100.0) * so.rotate_pairs(k, torch.tensor([a - 3]), 4, 100.0)).sum()) for a in (3, 50)]
    assert abs(s[0] - s[1]) < 1e-9


class _FakeHandle:
    def __init__(self, m):
        self.m, self.offset, self.slot = m, 0, m.slots.pop()

    def free(self):
        self.m.slots.append(self.slot)
        self.m.pages += (self.offset + 63) // 64


class _FakeModel:
    """counts tokens; its 'logits' make the greedy token (last token + 1) mod vocab"""
    max_batch_tokens, vocab_size, pool_pages = 32, 17, 6

    def __init__(self):
        self.slots, self.pages, self.steps = [1, 0], 6, []

    free_slots = property(lambda s: len(s.slots))
    free_pages = property(lambda s: s.pages)

    def make_cache(self, stream=None):
        return _FakeHandle(self)

    def step(self, entries, want, stream=None, layer_trace=False):
        rows = []
        for h, t in entries:
            self.pages -= (h.offset + len(t) + 63) // 64 - (h.offset + 63) // 64
            h.offset += len(t)
            rows += list(t)
        self.steps.append([len(t) for _, t in entries])
        assert sum(self.steps[-1]) <= self.max_batch_tokens and self.pages >= 0
        out = torch.zeros(len(want), self.vocab_size)
        for i, r in enumerate(want):
            out[i, (rows[r] + 1) % self.vocab_size] = 1.0
        return out


def test_token_loop_schedules_decodes_beside_prompt_portions(monkeypatch):
    from dnet_b200.shard import batching

    class _S:
        def synchronize(self): pass
        def wait_stream(self, s): pass

    import contextlib
    monkeypatch.setattr(batching.torch.cuda, "stream", lambda s: contextlib.nullcontext())
    monkeypatch.setattr(batching.torch.cuda, "current_stream", lambda: _S())
    m = _FakeModel()
    eng = batching.SequenceBatcher(m, stream=_S(), step_tokens=16)
    reqs = [batching.GenRequest("a", [1, 2, 3], 4), batching.GenRequest("b", list(range(40)), 3), batching.GenRequest("c", [9] * 70, 2)]
    out = eng.generate(reqs)
    assert out == {"a": [4, 5, 6, 7], "b": [6, 7, 8], "c": [10, 11]}
    assert all(sum(s) <= 16 for s in m.steps)
    assert any(len(s) == 2 and 1 in s and max(s) > 1 for s in m.steps)      # a decode token beside a prompt portion
    assert m.free_slots == 2 and m.free_pages == 6                             # everything was handed back


def _vulanex_cfg():
    rot = {"base": 777.0, "dims": 6, "scaling": {"factor": 4.0, "original": 32, "fast": 2.0, "slow": 0.5}}
    left = {"heads": 4, "kv_heads": 2, "dim": 10, "vdim": 7, "scale": 0.3, "mask": {"size": 9, "pool": 4}, "rot": rot}
    att = {"heads": 6, "kv_heads": 3, "dim": 5, "vdim": 5, "scale": 0.4, "q_temp": {"coef": 0.25, "every": 16}}
    return {"architecture": "Vulanex", "vocab": 50, "width": 32, "norm": {"eps": 1e-5}, "logit_scale": 0.75, "canon": {"taps": 3},
            "embedding": {"bigram": {"buckets": 11, "mul_prev": 5, "mul_cur": 3}},
            "layers": [{"type": "parallel", "mixer": {"left": left, "right": {"heads": 3, "dim": 6}}, "mlp": {"kind": "dense", "ff": 40}},
                       {"type": "attention", "mixer": att, "mlp": None},
                       {"type": "parallel", "mixer": {"left": {**left, "mask": None, "rot": None}, "right": {"heads": 1, "dim": 12}}, "mlp": None},
                       {"type": "attention", "mixer": {k: v for k, v in att.items() if k != "q_temp"}, "mlp": {"kind": "dense", "ff": 24}}]}


def test_vulanex_config_and_checkpoint_names():
    """every constant of the config lands in the structs, what the design fixes comes from the family, the decay's inner
    size comes from a tensor's shape, and every tensor the oracle writes finds its place through the aliases"""
    from dnet_b200 import _seqabi
    from dnet_b200.core.models import ring_model_class
    from dnet_b200.core.models.seqmix import _LAYER_KEY, parse_layer_list
    from oracle import vulanex_oracle as vo

    cfg = _vulanex_cfg()
    cls = ring_model_class("vulanex")
    shapes = vo.tensor_shapes(cfg, rank=5)
    with pytest.raises(ValueError):
        parse_layer_list(cfg, cls.family, None)              # the decay's inner size is in no config key
    sc, layers = parse_layer_list(cfg, cls.family, shapes)
    assert (sc.norm_kind, sc.post_norm, sc.no_pre_norm, sc.embed_norm, sc.streams) == (_seqabi.DN_NORM_LAYER, 0, 0, 0, 0)
    assert (sc.canon_taps, sc.bigram_buckets, sc.bigram_mul_prev, sc.bigram_mul_cur) == (3, 11, 5, 3)
    assert abs(sc.logit_scale - 0.75) < 1e-7 and abs(sc.eps - 1e-5) < 1e-9 and abs(sc.embed_scale - 1.0) < 1e-7
    assert [l.mixer for l in layers] == [_seqabi.DN_MIX_PARALLEL, _seqabi.DN_MIX_ATTENTION] * 2
    p0, a1, p2, a3 = layers
    assert (p0.heads, p0.kv_heads, p0.dim, p0.vdim, p0.chunk, p0.pool, p0.mask_kind) == (4, 2, 10, 7, 9, 4, _seqabi.DN_MASK_WINDOW)
    assert (p0.rot_dims, p0.rot_layout, p0.qk_norm, p0.sink, p0.v_is_k) == (6, _seqabi.DN_ROT_HALF, _seqabi.DN_QKNORM_HEAD, 1, 0)
    assert (p0.yarn_factor, p0.yarn_original, p0.yarn_fast, p0.yarn_slow) == (4.0, 32.0, 2.0, 0.5) and abs(p0.rot_base - 777.0) < 1e-3
    assert (p0.r_kind, p0.r_heads, p0.r_dim, p0.r_vdim, p0.rank, p0.branch_norm) == (_seqabi.DN_RIGHT_GDELTA, 3, 6, 6, 5, 1)
    assert p0.left_scale == 0.5 and p0.right_scale == 0.5 and p0.ff == 40 and p0.qtemp_every == 0
    assert (p2.chunk, p2.pool, p2.rot_dims, p2.yarn_factor, p2.r_heads, p2.r_dim, p2.ff) == (0, 0, 0, 0.0, 1, 12, 0)
    assert (a1.heads, a1.kv_heads, a1.dim, a1.vdim, a1.v_is_k, a1.qk_norm, a1.sink, a1.rot_dims, a1.chunk, a1.pool) == (6, 3, 5, 5, 1, 0, 0, 0, 0, 0)
    assert abs(a1.qtemp_coef - 0.25) < 1e-7 and a1.qtemp_every == 16 and abs(a1.scale - 0.4) < 1e-7 and a1.ff == 0
    assert a3.qtemp_every == 0 and a3.ff == 24
    m = cls.__new__(cls)
    m.config, m._cfg_struct, m._layer_structs, m.hidden_size, m.vocab_size = cfg, sc, layers, sc.width, sc.vocab
    want = m.expected_tensors()
    assert "head" not in want and "l1.mix.v" not in want      # the embedding table is the head; the values are the keys
    assert "l1.canon2" not in want and "l0.canon2" in want    # no feed-forward, no convolution before it
    got = {}
    for key, sh in shapes.items():
        if _LAYER_KEY.match(key):
            lname, suffix = key.split(".", 1)
            kind = cfg["layers"][int(lname[1:])]["type"]
            suffix = cls.tensor_alias.get(kind, {}).get(suffix, cls.tensor_alias.get("*", {}).get(suffix, suffix))
            key = f"{lname}.{suffix}"
        got[key] = tuple(sh)
    assert got == {k: tuple(v) for k, v in want.items()}
    for k in want:
        if _LAYER_KEY.match(k):
            assert k.split(".", 1)[1] in _seqabi.LAYER_SLOT, k


def test_vulanex_oracle_by_hand():
    """the oracle's pieces on numbers small enough to follow"""
    from oracle import vulanex_oracle as vo

    D = torch.float64
    # bigram rows: the extra row for the first token, then the hash of (previous, current)
    assert vo.bigram_rows([4, 9, 4], 11, 5, 3) == [11, (4 * 5 + 9 * 3) % 11, (9 * 5 + 4 * 3) % 11]
    # the convolution: tap taps - 1 meets the token itself, tap 0 the oldest, zeros before the sequence
    h = torch.tensor([[1.0], [10.0], [100.0]], dtype=D)
    cw = torch.tensor([[0.5, 2.0, 3.0]], dtype=D)
    assert torch.allclose(vo.input_convolution(h, cw)[:, 0], torch.tensor([1 + 3.0, 10 + 2.0 + 30.0, 100 + 0.5 + 20.0 + 300.0], dtype=D))
    # the query's factor steps up where floor((p + 1) / every) does
    f = vo.query_temperature(9, 2.0, 4)
    assert f[:3].tolist() == [1.0] * 3 and abs(float(f[3]) - (1 + 2 * math.log(2))) < 1e-12 and abs(float(f[7]) - (1 + 2 * math.log(3))) < 1e-12
    # visibility: a window of 3 with blocks of 2: position 6 sees tokens 4, 5, 6 and the blocks that end at or before 3
    assert vo.visible(6, 3, 2) == ([4, 5, 6], [0, 1]) and vo.visible(5, 3, 2) == ([3, 4, 5], [0]) and vo.visible(2, 3, 2) == ([0, 1, 2], [])
    assert vo.visible(4, 0, 0) == ([0, 1, 2, 3, 4], []) and vo.visible(4, 2, 0) == ([3, 4], [])
    # a block's key and value are means; a sink as large as the only score halves the only key's weight
    q = torch.zeros(3, 1, 1, dtype=D)
    k = torch.zeros(3, 1, 1, dtype=D)
    v = torch.tensor([[[2.0]], [[6.0]], [[100.0]]], dtype=D)
    o = vo.softmax_attention(q, k, v, 1.0, size=1, pool=2)          # position 2: itself and block 0 (mean value 4), equal scores
    assert abs(float(o[2, 0, 0]) - 52.0) < 1e-12 and float(o[1, 0, 0]) == 6.0
    o = vo.softmax_attention(q[:1], k[:1], v[:1], 1.0, sink=torch.tensor([0.0], dtype=D))
    assert abs(float(o[0, 0, 0]) - 1.0) < 1e-12
    # frequencies: without scaling base^(-2i/dims); with it fast pairs keep theirs, slow ones are divided by the factor
    f, m = vo.rotary_frequencies({"base": 100.0, "dims": 4})
    assert torch.allclose(f, torch.tensor([1.0, 0.1], dtype=D)) and m == 1.0
    f, m = vo.rotary_frequencies({"base": 10000.0, "dims": 8, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}})
    plain = torch.tensor([10000.0 ** (-2 * i / 8) for i in range(4)], dtype=D)
    assert float(f[0]) == 1.0 and abs(float(f[3]) - float(plain[3]) / 4.0) < 1e-15 and abs(m - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    assert all(float(plain[i]) / 4.0 - 1e-15 <= float(f[i]) <= float(plain[i]) + 1e-15 for i in range(4))
    # rotation by halves: dim i pairs with dim i + dims / 2; scores depend on the distance only
    e0 = torch.tensor([[[1.0, 0.0, 0.0, 0.0, 7.0]]] * 2, dtype=D)
    r = vo.rotary_half(e0, {"base": 100.0, "dims": 4})
    assert abs(float(r[1, 0, 2]) - math.sin(1.0)) < 1e-12 and float(r[1, 0, 1]) == 0.0 and float(r[1, 0, 4]) == 7.0 and torch.equal(r[0], e0[0])
    # the delta rule: no decay (w = 1), full removal (a = 1): an orthonormal key's value is stored and replaced exactly
    k = torch.eye(4, dtype=D)[[0, 1, 0]][:, None, :]
    v = torch.tensor([[1.0, 2.0, 0.0, 0.0], [3.0, 4.0, 0.0, 0.0], [5.0, 6.0, 0.0, 0.0]], dtype=D)[:, None, :]
    one = torch.ones(3, 1, 4, dtype=D)
    o = vo.generalized_delta_rule(k, k, v, one, one)
    assert torch.allclose(o, v, atol=1e-5)
    # no removal (a = 0), decay 1/2: the value written two tokens ago is read back at a quarter beside the new one
    o = vo.generalized_delta_rule(k, k, v, 0.5 * one, 0.0 * one)
    assert torch.allclose(o[2, 0], 0.25 * v[0, 0] + v[2, 0], atol=1e-5)
    # the decay's range: exp(-e^(-1/2) sigmoid(.)) lies between exp(-e^(-1/2)) and 1
    assert abs(math.exp(-math.exp(-0.5)) - 0.5452) < 1e-3
    # layer norm with the variance of the deviations
    x = torch.tensor([[1.0, 3.0]], dtype=D)
    assert torch.allclose(vo.layer_norm(x, torch.tensor([2.0, 2.0]), torch.tensor([0.5, 0.5]), 0.0), torch.tensor([[-1.5, 2.5]], dtype=D))
