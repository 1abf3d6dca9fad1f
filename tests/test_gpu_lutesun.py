"""The Lutesun family (core/models/seqmix.py LutesunRingModel, shard/batching.py, libdnet_b200_seq) against the float64
oracle (oracle/lutesun_oracle.py): every mechanism alone with the residual after each layer, then portions, batches,
page and slot reuse, keys at the edges of the sliding window and far away with scores made to stand out, long decoding
and greedy generation through the batcher's token loop.  fp32 runs are held to 2e-4 of the logits' spread row by row;
bf16 runs to 4e-2 of the spread over all rows together, on weights whose routers are decisive (a choice of experts that
bf16 rounding flips changes a row by far more than rounding does, and says nothing about the kernels)."""
from __future__ import annotations

import copy

import pytest
import torch

from oracle import lutesun_oracle as lo

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-4, "bfloat16": 4e-2}

DENSE = {"kind": "dense", "ff": 72}
MOE = {"kind": "moe", "router": {"experts": 6, "top": 2, "identity": 2, "scale": 1.75, "groups": {"count": 4, "keep": 2}},
       "expert": {"ff": 40}, "shared": {"ff": 24}}


def lat(mlp=None, second=False, **kw):
    mx = {"heads": 3, "dim": 24, "rot_dim": 8, "vdim": 16, "kv_rank": 40, "scale": 0.2, "rot": {"base": 5000.0, "dims": 8}, "mask": {"size": 21}}
    if second:
        mx["q_rank"] = 28
    mx.update(kw)
    if "rot_dim" in kw and "rot" not in kw:
        mx["rot"] = {"base": 5000.0, "dims": kw["rot_dim"]}
    return {"type": "latent_attention_2" if second else "latent_attention", "mixer": mx, "mlp": mlp}


def config(layers, width=48, vocab=96, eps=1e-5, scale=0.7):
    return {"architecture": "Lutesun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale}, "layers": layers}


FULL = config([lat(DENSE), lat(MOE, second=True), lat(None, heads=2, dim=8, kv_rank=24), lat(MOE, mask={"size": 70}),
               lat({**MOE, "shared": None}, second=True, heads=1, rot={"base": 100.0, "dims": 8})])


class Rig:
    """a model + batcher on the GPU and the oracle's view of the same weights"""

    def __init__(self, cfg, dtype="float32", seed=1, max_tokens=1024, max_seqs=4, max_batch_tokens=512, weights=None):
        from dnet_b200.shard.batching import SequenceBatcher, load_model
        from dnet_b200.utils.model import HostDictSource

        self.cfg, self.dtype = cfg, dtype
        self.w = weights if weights is not None else lo.random_weights(cfg, seed)
        if dtype == "bfloat16":
            self.w = decisive(self.w)
        self.model = load_model(HostDictSource({k: v.to(torch.bfloat16) for k, v in self.w.items()}, cfg), dtype, max_tokens=max_tokens,
                                max_seqs=max_seqs, max_batch_tokens=max_batch_tokens)
        self.eng = SequenceBatcher(self.model)

    def oracle(self, tokens, layers_out=None):
        return lo.forward(self.cfg, self.w, tokens, layers_out)

    def close(self):
        self.eng.close()
        self.model.destroy()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


def err(got: torch.Tensor, ref: torch.Tensor) -> float:
    """worst row of: rms of the difference (mean removed) over the rms spread of the reference row"""
    d = got.double().cpu() - ref.double()
    d = d - d.mean(-1, keepdim=True)
    r = ref.double() - ref.double().mean(-1, keepdim=True)
    return float((d.pow(2).mean(-1).sqrt() / r.pow(2).mean(-1).sqrt().clamp_min(1e-9)).max())


def err16(got: torch.Tensor, ref: torch.Tensor) -> float:
    """rms of the difference (row means removed) over the rms spread of the reference, all rows together"""
    d = got.double().cpu() - ref.double()
    d = d - d.mean(-1, keepdim=True)
    r = ref.double() - ref.double().mean(-1, keepdim=True)
    return float(d.pow(2).mean().sqrt() / r.pow(2).mean().sqrt())


def decisive(w):
    """corrections far apart: the same experts win at every token, whatever the rounding (the weights still come from
    the scores)"""
    w = dict(w)
    for k in w:
        if k.endswith("mlp.correction"):
            n = w[k].numel()
            w[k] = (3.0 * torch.arange(n).roll(n // 3)).to(torch.float32)
    return w


def toks(n, vocab=96, seed=0):
    g = torch.Generator().manual_seed(4000 + seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def run_schedule(rig: Rig, tokens, cuts, rid="r"):
    """feed tokens in portions of the given sizes (the rest one by one); logits of every position"""
    out, at = [], 0
    for c in list(cuts) + [1] * len(tokens):
        if at >= len(tokens):
            break
        part = tokens[at:at + c]
        out.append(rig.eng.step([(rid, part, list(range(len(part))))]))
        at += len(part)
    rig.eng.finish(rid)
    return torch.cat(out)


# -- each mechanism alone -----------------------------------------------------------------------------------------------
def moe(**kw):
    m = copy.deepcopy(MOE)
    for k, v in kw.items():
        if k in ("shared", "expert"):
            m[k] = v
        else:
            m["router"][k] = v
    return m


MECHANISMS = {
    "latent": config([lat()]),
    "latent_second": config([lat(second=True)]),
    "latent_one_head": config([lat(heads=1, dim=32, vdim=40)]),
    "latent_odd_sizes": config([lat(heads=3, dim=10, rot_dim=6, vdim=7, kv_rank=21), lat(second=True, heads=2, dim=5, rot_dim=2, vdim=9, kv_rank=13, q_rank=11)]),
    "latent_equal_sizes": config([lat(heads=2, dim=16, rot_dim=16, vdim=16, kv_rank=16), lat(second=True, heads=2, dim=16, rot_dim=16, vdim=16, kv_rank=16, q_rank=16)]),
    "latent_no_rotated_part": config([lat(rot_dim=0, rot=None)]),
    "latent_partly_turning": config([lat(rot_dim=12, rot={"base": 300.0, "dims": 4}), lat(second=True, rot_dim=12, rot={"base": 300.0, "dims": 6})]),
    "latent_wide_latent": config([lat(heads=2, dim=8, kv_rank=288, vdim=24), lat(second=True, heads=2, dim=8, kv_rank=512, vdim=8)]),
    "latent_large_heads": config([lat(heads=2, dim=160, rot_dim=64, vdim=136, kv_rank=96)], width=64),
    "window_of_one": config([lat(mask={"size": 1}), lat(second=True, mask={"size": 2})]),
    "window_wider_than_the_prompt": config([lat(mask={"size": 4000})]),
    "no_window": config([lat(mask=None), lat(second=True, mask=None)]),
    "window_of_a_page": config([lat(mask={"size": 64}), lat(second=True, mask={"size": 65}), lat(mask={"size": 63})]),
    "dense": config([lat(DENSE)]),
    "dense_wide": config([lat({"kind": "dense", "ff": 200})]),
    "moe": config([lat(MOE)]),
    "moe_top_1": config([lat(moe(top=1))]),
    "moe_every_expert": config([lat(moe(experts=3, identity=1, top=4, groups={"count": 2, "keep": 2}))]),
    "moe_no_identity": config([lat(moe(identity=0, groups={"count": 3, "keep": 1}))]),
    "moe_identity_only_group": config([lat(moe(experts=6, identity=3, top=3, groups={"count": 3, "keep": 2}))]),
    "moe_no_groups": config([lat(moe(groups=None))]),
    "moe_one_group_kept_of_many": config([lat(moe(experts=14, identity=2, top=2, groups={"count": 8, "keep": 1}))]),
    "moe_no_shared": config([lat(moe(shared=None))]),
    "moe_many_experts": config([lat(moe(experts=37, identity=3, top=5, groups={"count": 5, "keep": 3}, expert={"ff": 8}))]),
    "moe_scale_one": config([lat(moe(scale=1.0))]),
    "embedding_scale_one": config([lat(DENSE)], scale=1.0),
    "every_kind_of_layer": FULL,
}


@pytest.mark.parametrize("name", sorted(MECHANISMS))
def test_mechanism_alone_fp32(name):
    cfg = MECHANISMS[name]
    t = toks(150, seed=3)
    with Rig(cfg, "float32", seed=sum(map(ord, name))) as rig:
        layers = []
        ref = rig.oracle(t, layers)
        got, trace = rig.eng.step([("a", t, list(range(len(t))))], layer_trace=True)
        assert trace.shape[0] == len(layers)
        for i, l in enumerate(layers):
            assert err(trace[i], l) < TOL["float32"], f"{name}: residual after layer {i}"
        assert err(got, ref) < TOL["float32"]
        assert err(run_schedule(rig, t[:70], [30, 7, 2]), ref[:70]) < TOL["float32"], f"{name}: portions and decoding"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_model_whole_prompt(dtype):
    t = toks(200, seed=5)
    with Rig(FULL, dtype) as rig:
        got = rig.eng.step([("a", t, list(range(len(t))))])
        assert (err16 if dtype == "bfloat16" else err)(got, rig.oracle(t)) < TOL[dtype]


# -- sizes --------------------------------------------------------------------------------------------------------------
def test_sizes_on_the_tensor_core_products():
    """width and projection sizes in multiples of 64: bf16 prompt portions take the tcgen05 products and the MMA attention"""
    m = {"kind": "moe", "router": {"experts": 8, "top": 2, "identity": 2, "scale": 2.0, "groups": {"count": 5, "keep": 3}}, "expert": {"ff": 128},
         "shared": {"ff": 192}}
    cfg = config([lat({"kind": "dense", "ff": 256}, heads=4, dim=64, rot_dim=32, vdim=32, kv_rank=96, mask={"size": 100}),
                  lat(m, second=True, heads=8, dim=32, rot_dim=32, vdim=64, kv_rank=64, q_rank=64, mask={"size": 33})], width=128, vocab=192)
    t = toks(300, vocab=192, seed=6)
    with Rig(cfg, "bfloat16") as rig:
        ref = rig.oracle(t)
        assert err16(rig.eng.step([("a", t, list(range(len(t))))]), ref) < TOL["bfloat16"]
        rig.eng.finish("a")
        assert err16(run_schedule(rig, t, [130, 17, 64, 2, 70]), ref) < TOL["bfloat16"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_allow_no_wide_loads(dtype):
    """width, head, latent, expert and vocabulary sizes that are multiples of neither 4 nor 8: the scalar forms of every kernel"""
    m = {"kind": "moe", "router": {"experts": 5, "top": 3, "identity": 1, "scale": 0.9, "groups": {"count": 2, "keep": 1}}, "expert": {"ff": 30}, "shared": {"ff": 45}}
    cfg = config([lat(m, heads=3, dim=7, rot_dim=6, vdim=5, kv_rank=11, mask={"size": 19}),
                  lat({"kind": "dense", "ff": 35}, second=True, heads=2, dim=9, rot_dim=10, vdim=3, kv_rank=17, q_rank=9, mask={"size": 80})], width=50, vocab=77)
    t = toks(120, vocab=77, seed=160)
    with Rig(cfg, dtype) as rig:
        ref = rig.oracle(t)
        e = err16 if dtype == "bfloat16" else err
        assert e(run_schedule(rig, t, [120]), ref) < TOL[dtype]
        assert e(run_schedule(rig, t, [70, 2, 20]), ref) < TOL[dtype]


LAYER_SIZED = {
    # width 384: expert width 96 has no TMA descriptor, the others do
    "w384": config([lat({"kind": "dense", "ff": 640}, heads=6, dim=64, rot_dim=32, vdim=64, kv_rank=128, mask={"size": 90}),
                    lat({"kind": "moe", "router": {"experts": 8, "top": 3, "identity": 0, "scale": 0.8, "groups": {"count": 4, "keep": 2}}, "expert": {"ff": 96},
                         "shared": {"ff": 160}}, second=True, heads=12, dim=32, rot_dim=16, vdim=48, kv_rank=64, q_rank=192, mask={"size": 128}),
                    lat(None, heads=4, dim=48, rot_dim=16, vdim=80, kv_rank=256, mask={"size": 40})], width=384, vocab=640),
    # width 512, 32 experts in 8 groups, latent of 320 (the wider value accumulators of the decode kernel)
    "w512": config([lat({"kind": "moe", "router": {"experts": 30, "top": 4, "identity": 2, "scale": 1.0, "groups": {"count": 8, "keep": 4}}, "expert": {"ff": 128},
                         "shared": None}, heads=8, dim=64, rot_dim=64, vdim=64, kv_rank=320, mask={"size": 300}),
                    lat({"kind": "dense", "ff": 1024}, second=True, heads=8, dim=64, rot_dim=32, vdim=32, kv_rank=128, q_rank=256, mask={"size": 64}),
                    lat({"kind": "moe", "router": {"experts": 16, "top": 3, "identity": 0, "scale": 1.5}, "expert": {"ff": 64}, "shared": {"ff": 192}},
                        heads=16, dim=32, rot_dim=32, vdim=32, kv_rank=64, mask={"size": 17})], width=512, vocab=1000),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(LAYER_SIZED))
def test_layer_sized_models(name, dtype):
    cfg = LAYER_SIZED[name]
    V = cfg["vocab"]
    t = toks(210, vocab=V, seed=300)
    w = decisive(lo.random_weights(cfg, 301))
    with Rig(cfg, dtype, weights=w) as rig:
        ref = lo.forward(cfg, w, t)
        e = err16 if dtype == "bfloat16" else err
        whole = run_schedule(rig, t, [len(t)])
        assert e(whole, ref) < TOL[dtype]
        cut = run_schedule(rig, t, [100, 2, 64, 17, 5])
        assert e(cut, ref) < TOL[dtype]
        rig.eng.step([("a", t[:100], [])])
        rig.eng.step([("b", t[:37], [])])
        lg = rig.eng.step([("a", t[100:130], list(range(30))), ("b", t[37:38], [0])])      # a portion beside a decoded token
        assert e(lg[:30], ref[100:130]) < TOL[dtype] and e(lg[30:], ref[37:38]) < 2 * TOL[dtype]
        if dtype == "bfloat16":       # and the schedules agree with each other far better than with the oracle
            assert err16(cut, whole.cpu()) < 0.5 * TOL[dtype] and err16(lg[:30], whole[100:130].cpu()) < 0.5 * TOL[dtype]


# -- schedules ----------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_against_token_by_token(dtype):
    t = toks(90, seed=7)
    with Rig(FULL, dtype) as rig:
        ref = rig.oracle(t)
        e = err16 if dtype == "bfloat16" else err
        assert e(run_schedule(rig, t, []), ref) < TOL[dtype]              # every token alone, from the first
        assert e(run_schedule(rig, t, [50]), ref) < TOL[dtype]            # a prompt, then decoding


@pytest.mark.parametrize("cuts", [[2, 2, 2, 3, 5, 64, 1, 2, 40], [39, 2, 41, 2, 63, 1, 64], [128, 2], [1, 1, 1, 2, 200], [20, 1, 21, 22, 2, 19]])
def test_portions_of_any_size(cuts):
    t = toks(230, seed=11)
    with Rig(FULL, "float32") as rig:
        assert err(run_schedule(rig, t, cuts), rig.oracle(t)) < TOL["float32"]


def test_results_do_not_depend_on_the_cut_beyond_rounding():
    t = toks(130, seed=13)
    with Rig(FULL, "bfloat16") as rig:
        a = run_schedule(rig, t, [130])
        b = run_schedule(rig, t, [3, 61, 2, 30])
        assert err16(b, a.cpu()) < 2e-2


def test_unequal_requests_in_one_batch_equal_each_alone():
    lens = [5, 77, 140, 33]
    seqs = [toks(n, seed=20 + i) for i, n in enumerate(lens)]
    with Rig(FULL, "float32") as rig:
        refs = [rig.oracle(s) for s in seqs]
        at = [0] * 4
        portions = [[2, 3], [40, 2, 35], [64, 64, 12], [1] * 33]
        got = [[] for _ in seqs]
        step = 0
        while any(at[i] < lens[i] for i in range(4)):
            entries = []
            for i in range(4):
                if at[i] < lens[i] and (step + i) % 3 != 2:              # requests sit out some steps
                    n = portions[i][0] if portions[i] else 1
                    portions[i] = portions[i][1:]
                    part = seqs[i][at[i]:at[i] + n]
                    entries.append((f"q{i}", part, list(range(len(part)))))
                    at[i] += len(part)
            step += 1
            if not entries:
                continue
            lg = rig.eng.step(entries)
            row = 0
            for rid, part, _ in entries:
                got[int(rid[1:])].append(lg[row:row + len(part)])
                row += len(part)
        for i in range(4):
            assert err(torch.cat(got[i]), refs[i]) < TOL["float32"], f"request {i}"


def test_pages_and_slots_are_reused():
    """a pool of 4 pages and 2 slots serves 6 requests two at a time; a request that does not fit is refused without
    disturbing the live ones, and a page's old rows never show in its next user's window"""
    from dnet_b200._cabi import DnError

    with Rig(FULL, "float32", max_tokens=256, max_seqs=2, max_batch_tokens=256) as rig:
        for rnd in range(3):
            a, b = toks(100 + rnd, seed=30 + rnd), toks(120 - rnd, seed=40 + rnd)
            la = rig.eng.step([("a", a[:70], []), ("b", b[:3], [])])
            assert la is None
            la = rig.eng.step([("a", a[70:], list(range(len(a) - 70))), ("b", b[3:], list(range(len(b) - 3)))])
            assert err(la[:len(a) - 70], rig.oracle(a)[70:]) < TOL["float32"]
            assert err(la[len(a) - 70:], rig.oracle(b)[3:]) < TOL["float32"]
            assert rig.model.free_pages == 0 and rig.model.free_slots == 0
            with pytest.raises(DnError):
                rig.eng.step([("a", toks(60), [])])                        # a fifth page does not exist
            with pytest.raises(DnError):
                rig.eng.step([("c", [1], [])])                            # nor a third slot
            rig.eng.live.pop("c", None)
            rig.eng.finish("a")
            rig.eng.finish("b")
            assert rig.model.free_pages == 4 and rig.model.free_slots == 2


# -- keys at the window's edges and far away, with scores made to stand out ---------------------------------------------------
def edge_setup(window: int, second: bool = False, n: int = 260, marks=(0, 40, 64, 104, 127, 170)):
    """One latent-attention layer in which a query finds, among everything it sees, the one token whose input points the
    other way.  The first `dim` rows of the key/value latent are minus the first head's unrotated query rows and that head's key
    up-projection copies them, so its unrotated key is minus its query over the latent's root mean square: a token scores
    about -|q|^2 against itself and +|q|^2 against a token with the opposite input.  Token 63's embedding is minus
    token 62's.  Token 63 stands at every position of `marks` and token 62 at mark + window - 1 (it just sees the 63) and
    at mark + window (it just does not); all other tokens are below 62."""
    dn, R = 32, 40
    cfg = config([lat(second=second, heads=2, dim=dn, rot_dim=8, vdim=16, kv_rank=R, scale=0.5, mask={"size": window})], vocab=64, scale=1.0)
    w = lo.random_weights(cfg, 70 + window)
    e = w["embed"].clone()
    e[63] = -e[62]
    w["embed"] = e
    if second:      # the query latent as wide as the input and an identity: q = W_uq rmsnorm(h)
        cfg["layers"][0]["mixer"]["q_rank"] = cfg["width"]
        w = {k: v for k, v in w.items() if not k.startswith("l0.mix.dq") and k != "l0.mix.uq"}
        g = torch.Generator().manual_seed(5)
        w["l0.mix.dq"] = torch.eye(cfg["width"])
        w["l0.mix.dq.norm"] = torch.ones(cfg["width"])
        w["l0.mix.uq"] = (torch.randn(2 * (dn + 8), cfg["width"], generator=g) / cfg["width"] ** 0.5).to(torch.bfloat16).float()
    qw = w["l0.mix.uq" if second else "l0.mix.q"]
    dkv = w["l0.mix.dkv"].clone()
    dkv[:dn] = -qw[:dn]
    w["l0.mix.dkv"] = dkv
    w["l0.mix.dkv.norm"] = torch.ones(R)
    uk = w["l0.mix.uk"].clone()
    uk[:dn] = 0.0
    uk[:dn, :dn] = torch.eye(dn)
    w["l0.mix.uk"] = uk
    g = torch.Generator().manual_seed(71 + window)
    t = torch.randint(0, 62, (n,), generator=g).tolist()
    rows = []
    for m in marks:
        t[m] = 63
    for m in marks:
        for p in (m + window - 1, m + window):
            if p < n and t[p] != 63:
                t[p] = 62
                rows.append(p)
    return cfg, w, t, sorted(set(rows))


def with_window(cfg, size):
    c = copy.deepcopy(cfg)
    c["layers"][0]["mixer"]["mask"]["size"] = size
    return c


@pytest.mark.parametrize("second", [False, True])
@pytest.mark.parametrize("window", [24, 64, 65])
def test_keys_just_inside_and_just_outside_the_window(window, second):
    """marks at the sequence's start (the first tokens a window keeps and loses), in the middle of pages and where the
    window's edge falls on a page border; a window that is one token off in either direction changes those rows by far
    more than the tolerance.  In prompts (cut at, before and after the edges) and decoded one by one, fp32 and bf16."""
    cfg, w, t, rows = edge_setup(window, second)
    ref = lo.forward(cfg, w, t)
    for off in (-1, 1):
        assert err(lo.forward(with_window(cfg, window + off), w, t)[rows], ref[rows]) > 100 * TOL["float32"]
    first = rows[0]
    for dtype in ("float32", "bfloat16"):
        e = err16 if dtype == "bfloat16" else err
        with Rig(cfg, dtype, weights=w) as rig:
            got = run_schedule(rig, t, [len(t)])
            assert e(got, ref) < TOL[dtype] and e(got[rows], ref[rows]) < TOL[dtype]
            got = run_schedule(rig, t, [first, 2, window - 1, 2, window, 17, 2, 64])      # portions that start and end at the edges
            assert e(got, ref) < TOL[dtype] and e(got[rows], ref[rows]) < TOL[dtype]
            got = run_schedule(rig, t, [max(1, first - 3)])                               # every edge row decoded alone
            assert e(got, ref) < TOL[dtype] and e(got[rows], ref[rows]) < TOL[dtype]


def test_far_key_among_hundreds():
    """a window of 1,000: the marked token at position 3 is seen from 700 positions on, through the prompt kernels and
    through decode rows split over several blocks"""
    cfg, w, t, _ = edge_setup(1000, n=706, marks=(3,))
    for p in range(700, 706):
        t[p] = 62
    ref = lo.forward(cfg, w, t)
    t_without = list(t)
    t_without[3] = 5
    assert err(lo.forward(cfg, w, t_without)[-6:], ref[-6:]) > 100 * TOL["float32"]       # the far key matters
    with Rig(cfg, "float32", weights=w, max_batch_tokens=1024) as rig:
        assert err(run_schedule(rig, t, [len(t)]), ref) < TOL["float32"]
        assert err(run_schedule(rig, t, [300, 2, 250, 148]), ref) < TOL["float32"]        # the last six decoded one by one
    with Rig(cfg, "bfloat16", weights=w, max_batch_tokens=1024) as rig:
        assert err16(run_schedule(rig, t, [300, 2, 250, 148])[-6:], ref[-6:]) < TOL["bfloat16"]
        assert err16(run_schedule(rig, t, [len(t)])[-6:], ref[-6:]) < TOL["bfloat16"]


def test_long_rows_split_over_blocks_in_decoding():
    """decoding past 512 and 1024 visible keys under a window of 1,100, and past the window: a row's attention is computed
    by 2 and 3 blocks and joined"""
    cfg = config([lat(heads=2, dim=16, vdim=40, kv_rank=72, scale=0.4, mask={"size": 1100})])
    t = toks(1300, seed=165)
    with Rig(cfg, "float32", max_tokens=1344, max_batch_tokens=1344) as rig:
        ref = rig.oracle(t)
        for first, n in ((508, 8), (1020, 8), (1096, 8), (1290, 8)):
            lg = run_schedule(rig, t[:first + n], [first])
            assert err(lg[first:], ref[first:first + n]) < TOL["float32"]


@pytest.mark.parametrize("heads", [17, 20, 64, 70])
def test_many_heads_in_decoding(heads):
    """bf16 decode steps put the heads of a token into the rows of one MMA tile: more than 16 heads fill several row
    groups, more than 64 several blocks; beside it the same model in prompts and in fp32"""
    cfg = config([lat(heads=heads, dim=8, rot_dim=8, vdim=8, kv_rank=24, mask={"size": 150}),
                  lat(DENSE, second=True, heads=heads, dim=8, rot_dim=8, vdim=8, kv_rank=16, q_rank=32, mask={"size": 70})])
    t = toks(200, seed=170 + heads)
    for dtype in ("bfloat16", "float32"):
        with Rig(cfg, dtype, seed=heads) as rig:
            ref = rig.oracle(t)
            e = err16 if dtype == "bfloat16" else err
            assert e(run_schedule(rig, t, [140]), ref) < TOL[dtype]
            a, b = t[:90], t[5:130]                                          # two sequences decoding side by side
            rig.eng.step([("a", a[:80], []), ("b", b[:120], [])])
            got = [rig.eng.step([("a", [a[80 + i]], [0]), ("b", [b[120 + i]], [0])]) for i in range(5)]
            ga, gb = torch.cat([g[:1] for g in got]), torch.cat([g[1:] for g in got])
            assert e(ga, rig.oracle(a[:85])[80:]) < TOL[dtype] and e(gb, rig.oracle(b[:125])[120:]) < TOL[dtype]


def test_first_tokens_of_a_sequence():
    with Rig(FULL, "float32") as rig:
        for n in (1, 2, 3, 4):
            t = toks(n, seed=80 + n)
            assert err(run_schedule(rig, t, [n]), rig.oracle(t)) < TOL["float32"]
            assert err(run_schedule(rig, t, []), rig.oracle(t)) < TOL["float32"]


def test_long_decoding():
    t = toks(300, seed=90)
    with Rig(FULL, "float32") as rig:
        assert err(run_schedule(rig, t, [20]), rig.oracle(t)) < TOL["float32"]


def test_a_step_larger_than_the_batch_buffer_is_cut_inside():
    t = toks(300, seed=95)
    with Rig(FULL, "float32", max_batch_tokens=64) as rig:
        got = rig.eng.step([("a", t[:290], [0, 63, 64, 289]), ("b", t[:70], [69])])
        ref = rig.oracle(t)
        assert err(got[:4], ref[[0, 63, 64, 289]]) < TOL["float32"]
        assert err(got[4:], ref[[69]]) < TOL["float32"]


def test_graph_replay_equals_launch_by_launch_decoding():
    t = toks(60, seed=97)
    with Rig(FULL, "bfloat16") as rig:
        a = run_schedule(rig, t, [20])
        rig.model.set_graphs(False)
        b = run_schedule(rig, t, [20])
        assert torch.equal(a, b)


# -- the token loop, the command lines, the runtime ----------------------------------------------------------------------------
def greedy_agrees(cfg, w, prompt, got, margin=1e-3):
    seq = list(prompt)
    for tok in got:
        lg = lo.forward(cfg, w, seq)[-1]
        top2 = torch.topk(lg, 2).values
        if float(top2[0] - top2[1]) > margin:           # a near tie may fall either way
            assert tok == int(lg.argmax()), f"at length {len(seq)}"
        seq.append(tok)


def test_greedy_generation_through_the_batcher():
    from dnet_b200.shard.batching import GenRequest

    with Rig(FULL, "float32", max_tokens=320, max_seqs=2) as rig:
        rig.eng.step_tokens = 48
        reqs = [GenRequest(f"g{i}", toks(n, seed=100 + i), max_new_tokens=m) for i, (n, m) in enumerate([(30, 6), (100, 4), (3, 9), (65, 5)])]
        out = rig.eng.generate(reqs)
        assert rig.model.free_slots == 2 and rig.model.free_pages == 5
        for r in reqs:
            greedy_agrees(FULL, rig.w, r.prompt, out[r.id])


def test_command_lines_on_a_checkpoint_folder(tmp_path):
    """bin/trace_run and bin/generate on a folder with config.json and model.safetensors: the class is picked by the
    config's architecture; the checkpoint has no head tensor (the embedding table is the head)"""
    import json
    import os
    import struct
    import subprocess
    import sys

    import numpy as np

    cfg = config([lat(MOE, second=True), lat(DENSE)])
    del cfg["layers"][0]["mixer"]["q_rank"]              # the size then comes from the tensor's shape
    w = lo.random_weights({**cfg, "layers": [lat(MOE, second=True), lat(DENSE)]}, 110)
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(cfg))
    header, blobs, at = {}, [], 0
    for k, v in w.items():
        raw = v.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes()
        header[k] = {"dtype": "BF16", "shape": list(v.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    hj = json.dumps(header).encode()
    (folder / "model.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
    full = {**cfg, "layers": [lat(MOE, second=True), lat(DENSE)]}
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    t = toks(70, seed=111)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": t[:50], "want": [49]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": t[50:52], "want": [0, 1]}, {"id": "b", "tokens": t[:9], "want": [8]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": t[52:], "want": [17]}], "end": ["a"]}]
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "192"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    ref = lo.forward(full, w, t)
    got = [torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4")).view(-1, cfg["vocab"]) for i in range(3)]
    assert err(got[0], ref[[49]]) < TOL["float32"]
    assert err(got[1], torch.cat([ref[[50, 51]], lo.forward(full, w, t[:9])[[8]]])) < TOL["float32"]
    assert err(got[2], ref[[69]]) < TOL["float32"]
    reqs = [{"id": "x", "prompt": t[:40], "max_new_tokens": 5}, {"id": "y", "prompt": t[:7], "max_new_tokens": 3}]
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "generate"), "--model", str(folder), "--dtype", "float32", "--max-tokens", "192",
                        "--step-tokens", "16"], input="\n".join(json.dumps(r) for r in reqs) + "\n", capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    outs = {o["id"]: o["tokens"] for o in map(json.loads, p.stdout.strip().splitlines())}
    for r in reqs:
        assert len(outs[r["id"]]) == r["max_new_tokens"]
        greedy_agrees(full, w, r["prompt"], outs[r["id"]])


def test_served_by_the_shard_runtime():
    """load_model_core finds the class by the config's architecture and serves it with the batched policy: frames of
    tokens in, sampled tokens out, chunked prompts, slots and pages returned at release"""
    import queue

    from dnet_b200.shard.models import ShardLoadModelRequest
    from dnet_b200.shard.policies.batched import BatchedStepPolicy
    from dnet_b200.shard.runtime import ShardRuntime
    from dnet_b200.utils.model import HostDictSource
    from tests.helpers import ring_generate, token_message

    w = decisive(lo.random_weights(FULL, 21))
    n = len(FULL["layers"])
    rt = ShardRuntime(shard_id="s0", queue_size=64)
    rt.kv_cache_config.max_tokens = 256
    src = HostDictSource({k: v.to(torch.bfloat16) for k, v in w.items()}, FULL)
    rt.load_model_core(ShardLoadModelRequest(model_path=src, total_layers=n, layers=list(range(n)), window_size=n, residency_size=n, kv_bits="fp16"))
    try:
        assert isinstance(rt.policy, BatchedStepPolicy)
        a, b = toks(45, seed=180), toks(70, seed=181)
        out_a = [t for t, _, _ in ring_generate([rt], "na", a, 5)]
        greedy_agrees(FULL, w, a, out_a, margin=5e-2 * float(lo.forward(FULL, w, a)[-1].std()))
        for part in (b[:30], b[30:64]):
            rt.policy.process(token_message(rt, "nb", part, more=True))
            with pytest.raises(queue.Empty):
                rt.activation_send_queue.get_nowait()
        out_b = [t for t, _, _ in ring_generate([rt], "nb", b[64:], 4)]
        greedy_agrees(FULL, w, b, out_b, margin=5e-2 * float(lo.forward(FULL, w, b)[-1].std()))
        rt.release_nonce("na")
        rt.release_nonce_deferred("nb")
        assert rt.model.free_pages == rt.model.pool_pages
    finally:
        assert rt.unload_model_core().success
