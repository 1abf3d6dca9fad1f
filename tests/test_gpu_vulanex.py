"""The Vulanex family (core/models/seqmix.py VulanexRingModel, shard/batching.py, libdnet_b200_seq) against the float64
oracle (oracle/vulanex_oracle.py): every mechanism alone with the residual after each layer, then portions, batches,
page and slot reuse, keys at the edges of the sliding window and of the pooled blocks and far away with scores made to
stand out, states that must not survive a slot, long decoding and greedy generation through the batcher's token loop.
fp32 runs are held to 2e-4 of the logits' spread row by row; bf16 runs to 4e-2 of the spread over all rows together."""
from __future__ import annotations

import copy

import pytest
import torch

from oracle import vulanex_oracle as vo

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-4, "bfloat16": 4e-2}

DENSE = {"kind": "dense", "ff": 72}
ROT = {"base": 5000.0, "dims": 8, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}
BIGRAM = {"buckets": 53, "mul_prev": 31, "mul_cur": 5}


def att(mlp=None, **kw):
    mx = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 16, "scale": 0.3, "q_temp": {"coef": 0.7, "every": 9}}
    mx.update(kw)
    mx["vdim"] = mx["dim"]
    return {"type": "attention", "mixer": mx, "mlp": mlp}


def par(mlp=None, right=None, **kw):
    left = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.25, "mask": {"size": 21, "pool": 5}, "rot": copy.deepcopy(ROT)}
    left.update(kw)
    return {"type": "parallel", "mixer": {"left": left, "right": {"heads": 3, "dim": 8, **(right or {})}}, "mlp": mlp}


def config(layers, width=48, vocab=96, eps=1e-5, taps=3, bigram=BIGRAM, logit_scale=0.7):
    cfg = {"architecture": "Vulanex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if taps:
        cfg["canon"] = {"taps": taps}
    if bigram:
        cfg["embedding"] = {"bigram": dict(bigram)}
    if logit_scale is not None:
        cfg["logit_scale"] = logit_scale
    return cfg


FULL = config([par(DENSE), att(DENSE), att(None, heads=2, kv_heads=1, dim=8, q_temp=None), par(DENSE, mask={"size": 70, "pool": 16}),
               par(None, right={"heads": 1, "dim": 24}, heads=3, kv_heads=3, dim=8, vdim=8, rot={"base": 100.0, "dims": 4})])


class Rig:
    """a model + batcher on the GPU and the oracle's view of the same weights"""

    def __init__(self, cfg, dtype="float32", seed=1, max_tokens=1024, max_seqs=4, max_batch_tokens=512, weights=None, rank=8):
        from dnet_b200.shard.batching import SequenceBatcher, load_model
        from dnet_b200.utils.model import HostDictSource

        self.cfg, self.dtype = cfg, dtype
        self.w = weights if weights is not None else vo.random_weights(cfg, seed, rank)
        self.model = load_model(HostDictSource({k: v.to(torch.bfloat16) for k, v in self.w.items()}, cfg), dtype, max_tokens=max_tokens,
                                max_seqs=max_seqs, max_batch_tokens=max_batch_tokens)
        self.eng = SequenceBatcher(self.model)

    def oracle(self, tokens, layers_out=None):
        return vo.forward(self.cfg, self.w, tokens, layers_out)

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


def toks(n, vocab=96, seed=0):
    g = torch.Generator().manual_seed(7000 + seed)
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
def bare(layers, **kw):
    """no input convolution, no bigram row, logits unscaled: the layer's own mechanism only"""
    return config(layers, **{"taps": 0, "bigram": None, "logit_scale": None, **kw})


MECHANISMS = {
    "attention": bare([att()]),
    "attention_no_query_temperature": bare([att(q_temp=None)]),
    "attention_temperature_every_token": bare([att(q_temp={"coef": 0.25, "every": 1})]),
    "attention_temperature_rarely": bare([att(q_temp={"coef": 3.0, "every": 64}), att(q_temp={"coef": 1.5, "every": 100})]),
    "attention_one_head": bare([att(heads=1, kv_heads=1, dim=32)]),
    "attention_as_many_key_heads": bare([att(heads=3, kv_heads=3, dim=8)]),
    "attention_one_key_head": bare([att(heads=6, kv_heads=1, dim=24)]),
    "attention_odd_sizes": bare([att(heads=3, kv_heads=1, dim=7), att(heads=2, kv_heads=2, dim=10)]),
    "attention_large_heads": bare([att(heads=2, kv_heads=1, dim=128, scale=0.05), att(heads=1, kv_heads=1, dim=200, scale=0.05)], width=64),
    "parallel": bare([par()]),
    "parallel_no_rotation": bare([par(rot=None)]),
    "parallel_plain_frequencies": bare([par(rot={"base": 300.0, "dims": 16})]),
    "parallel_partly_turning": bare([par(rot={"base": 300.0, "dims": 4}), par(dim=24, rot={**ROT, "dims": 12})]),
    "parallel_scaling_ramps": bare([par(dim=32, rot={"base": 10000.0, "dims": 32, "scaling": {"factor": 8.0, "original": 40, "fast": 4.0, "slow": 0.5}}),
                                    par(rot={"base": 50.0, "dims": 16, "scaling": {"factor": 1.5, "original": 1000, "fast": 100.0, "slow": 90.0}})]),
    "parallel_one_head": bare([par(heads=1, kv_heads=1, dim=32, vdim=40, right={"heads": 1, "dim": 16})]),
    "parallel_odd_sizes": bare([par(heads=3, kv_heads=1, dim=10, vdim=7, rot={"base": 77.0, "dims": 6}, right={"heads": 5, "dim": 6})]),
    "parallel_equal_sizes": bare([par(heads=2, kv_heads=2, dim=24, vdim=24, rot={**ROT, "dims": 24}, right={"heads": 2, "dim": 24})]),
    "parallel_large_heads": bare([par(heads=2, kv_heads=1, dim=128, vdim=128, scale=0.1, right={"heads": 1, "dim": 128})], width=64),
    "delta_rule_wide": bare([par(right={"heads": 1, "dim": 160})]),
    "delta_rule_many_small_heads": bare([par(right={"heads": 11, "dim": 4})]),
    # as many (head, 16 columns) pairs as the GPU has SMs and more: the recurrence then takes more rows a lane and 16 columns a block
    "delta_rule_150_heads": bare([par(right={"heads": 150, "dim": 8})]),
    "delta_rule_40_heads_of_64": bare([par(right={"heads": 40, "dim": 64})]),
    "delta_rule_19_heads_of_128": bare([par(right={"heads": 19, "dim": 128}), par(right={"heads": 10, "dim": 256})]),
    "window_of_one": bare([par(mask={"size": 1, "pool": 3}), par(mask={"size": 2, "pool": 1})]),
    "window_of_a_page": bare([par(mask={"size": 64, "pool": 8}), par(mask={"size": 65, "pool": 7}), par(mask={"size": 63, "pool": 64})]),
    "window_wider_than_the_prompt": bare([par(mask={"size": 4000, "pool": 4})]),
    "no_window": bare([par(mask=None)]),
    "window_without_blocks": bare([par(mask={"size": 17}), par(mask={"size": 30, "pool": 0})]),
    "blocks_of_one": bare([par(mask={"size": 9, "pool": 1})]),
    "blocks_wider_than_the_window": bare([par(mask={"size": 6, "pool": 20}), par(mask={"size": 10, "pool": 10})]),
    "blocks_wider_than_a_page": bare([par(mask={"size": 11, "pool": 100}), par(mask={"size": 3, "pool": 65})]),
    "blocks_that_divide_a_page": bare([par(mask={"size": 16, "pool": 16}), par(mask={"size": 5, "pool": 32})]),
    "convolution": config([att(), par(DENSE)], taps=4, bigram=None, logit_scale=None),
    "convolution_of_one_tap": config([par(DENSE), att(DENSE)], taps=1, bigram=None, logit_scale=None),
    "convolution_of_two_taps": config([att(DENSE)], taps=2, bigram=None, logit_scale=None),
    "convolution_of_nine_taps": config([att(DENSE), par()], taps=9, bigram=None, logit_scale=None),
    "bigram": config([att()], taps=0, logit_scale=None),
    "bigram_one_bucket": config([att()], taps=0, bigram={"buckets": 1, "mul_prev": 1, "mul_cur": 1}, logit_scale=None),
    "bigram_large_multipliers": config([att()], taps=0, bigram={"buckets": 1021, "mul_prev": 1000003, "mul_cur": 999983}, logit_scale=None),
    "feed_forward": bare([att(DENSE)]),
    "feed_forward_wide": bare([par({"kind": "dense", "ff": 200})]),
    "logit_scale": bare([att()], logit_scale=0.125),
    "parallel_layers_first": config([par(DENSE), par(None), att(DENSE)]),
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
        rig.eng.finish("a")
        assert err(run_schedule(rig, t[:100], [30, 7, 2, 41]), ref[:100]) < TOL["float32"], f"{name}: portions and decoding"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_model_whole_prompt(dtype):
    t = toks(200, seed=5)
    with Rig(FULL, dtype) as rig:
        got = rig.eng.step([("a", t, list(range(len(t))))])
        assert (err16 if dtype == "bfloat16" else err)(got, rig.oracle(t)) < TOL[dtype]


# -- sizes --------------------------------------------------------------------------------------------------------------
def test_sizes_on_the_tensor_core_products():
    """width and projection sizes in multiples of 64: bf16 prompt portions take the tcgen05 products and the MMA attention
    tiles (token pages and pooled rows)"""
    cfg = config([att({"kind": "dense", "ff": 256}, heads=4, kv_heads=2, dim=64, scale=0.1, q_temp={"coef": 0.5, "every": 50}),
                  par({"kind": "dense", "ff": 192}, heads=8, kv_heads=2, dim=32, vdim=64, mask={"size": 33, "pool": 6},
                      rot={**ROT, "dims": 32}, right={"heads": 2, "dim": 64})], width=128, vocab=192, taps=4)
    t = toks(300, vocab=192, seed=6)
    with Rig(cfg, "bfloat16", rank=64) as rig:
        ref = rig.oracle(t)
        assert err16(rig.eng.step([("a", t, list(range(len(t))))]), ref) < TOL["bfloat16"]
        rig.eng.finish("a")
        assert err16(run_schedule(rig, t, [130, 17, 64, 2, 70]), ref) < TOL["bfloat16"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_allow_no_wide_loads(dtype):
    """width, head, feed-forward and vocabulary sizes that are multiples of neither 4 nor 8: the scalar forms of every kernel"""
    cfg = config([par({"kind": "dense", "ff": 35}, heads=3, kv_heads=1, dim=7, vdim=5, mask={"size": 19, "pool": 3}, rot={"base": 900.0, "dims": 6},
                      right={"heads": 3, "dim": 9}),
                  att({"kind": "dense", "ff": 30}, heads=2, kv_heads=2, dim=9)], width=50, vocab=77, taps=3, bigram={"buckets": 7, "mul_prev": 3, "mul_cur": 2})
    t = toks(120, vocab=77, seed=160)
    with Rig(cfg, dtype, rank=5) as rig:
        ref = rig.oracle(t)
        e = err16 if dtype == "bfloat16" else err
        assert e(run_schedule(rig, t, [120]), ref) < TOL[dtype]
        assert e(run_schedule(rig, t, [70, 2, 20]), ref) < TOL[dtype]


LAYER_SIZED = {
    # width 384: the delta rule's channels (5 x 48 = 240) and its decay rank 24 have no TMA descriptor, the others do
    "w384": (config([att({"kind": "dense", "ff": 640}, heads=6, kv_heads=2, dim=64, scale=0.11, q_temp={"coef": 0.4, "every": 32}),
                     par({"kind": "dense", "ff": 512}, heads=12, kv_heads=4, dim=32, vdim=48, mask={"size": 90, "pool": 12}, rot={**ROT, "dims": 16},
                         right={"heads": 5, "dim": 48}),
                     par(None, heads=4, kv_heads=1, dim=96, vdim=64, scale=0.1, mask={"size": 40, "pool": 64}, rot={"base": 1e5, "dims": 96},
                         right={"heads": 6, "dim": 64})], width=384, vocab=640, taps=4), 24),
    # width 512, head sizes of 128, one key head, a window over several pages
    "w512": (config([par({"kind": "dense", "ff": 1024}, heads=4, kv_heads=1, dim=128, vdim=128, scale=0.09, mask={"size": 150, "pool": 20},
                         rot={"base": 250000.0, "dims": 64, "scaling": {"factor": 2.0, "original": 128, "fast": 16.0, "slow": 1.0}},
                         right={"heads": 4, "dim": 128}),
                     att({"kind": "dense", "ff": 768}, heads=8, kv_heads=1, dim=128, scale=0.08, q_temp={"coef": 0.5, "every": 64}),
                     att(None, heads=16, kv_heads=4, dim=32, scale=0.17)], width=512, vocab=1000, taps=2,
                    bigram={"buckets": 4093, "mul_prev": 257, "mul_cur": 3}), 64),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(LAYER_SIZED))
def test_layer_sized_models(name, dtype):
    cfg, rank = LAYER_SIZED[name]
    V = cfg["vocab"]
    t = toks(210, vocab=V, seed=300)
    w = vo.random_weights(cfg, 301, rank)
    with Rig(cfg, dtype, weights=w) as rig:
        ref = vo.forward(cfg, w, t)
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
    disturbing the live ones; a page's old rows and pooled rows, a slot's old state, carried rows and last token never
    show in its next user"""
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
            la = rig.eng.step([("a", [7], [0])])                           # the refused steps changed nothing of "a": not its last token either
            assert err(la, rig.oracle(a + [7])[-1:]) < TOL["float32"]
            rig.eng.finish("a")
            rig.eng.finish("b")
            assert rig.model.free_pages == 4 and rig.model.free_slots == 2


# -- keys at the window's and the blocks' edges and far away, with scores made to stand out --------------------------------------
def edge_setup(size: int, pool: int, token_marks=(0, 40, 64, 104, 127, 170)):
    """One parallel layer in which a query finds, among everything it sees, the token whose input points the other way.
    The key projection is minus the first head's query rows, q / k norm weights are one and the layer norm has no
    bias, so that head's key is minus its query: a token scores about -dim * scale against itself and +dim * scale against a
    token with the opposite input (rotation touches a quarter of the dims).  Token 63's embedding is minus token 62's.
    Token 63 stands at every position of `token_marks`, and token 62 at mark + size - 1 (it just sees the 63) and at
    mark + size (it just does not).  Further on, whole blocks hold 63s except for their last token, and token 62
    stands where such a block is first seen pooled, and one position before, where the 63s have left the window and the
    block is not seen yet.  All other tokens are below 62."""
    dk = 32
    cfg = bare([par(heads=2, kv_heads=1, dim=dk, vdim=16, scale=0.5, mask={"size": size, "pool": pool}, rot={**ROT, "dims": 8},
                    right={"heads": 2, "dim": 8})], vocab=64)
    w = vo.random_weights(cfg, 70 + size)
    e = w["embed"].clone()
    e[63] = -e[62]
    w["embed"] = e
    w["l0.norm1.b"] = torch.zeros_like(w["l0.norm1.b"])
    w["l0.mix.left.k"] = -w["l0.mix.left.q"][:dk].clone()
    w["l0.mix.left.q.norm"] = torch.ones(dk)
    w["l0.mix.left.k.norm"] = torch.ones(dk)
    # marked blocks lie more than a window apart: where one is first seen pooled, no 63 stands in the window itself
    first_block = (max(token_marks) + size + pool) // pool + 1 if pool > 1 else 0
    block_marks = [first_block + ((size + pool) // pool + 2) * i for i in range(3)] if pool > 1 else []
    n = (block_marks[-1] + 1) * pool + size + 8 if block_marks else max(token_marks) + size + 8
    g = torch.Generator().manual_seed(71 + size)
    t = torch.randint(0, 62, (n,), generator=g).tolist()
    for m in token_marks:
        t[m] = 63
    for b in block_marks:
        for p in range(b * pool, b * pool + pool - 1):
            t[p] = 63
    rows = []
    for p in [m + d for m in token_marks for d in (size - 1, size)] + [b * pool + pool - 1 + size - d for b in block_marks for d in (0, 1)]:
        if p < n and t[p] != 63:
            t[p] = 62
            rows.append(p)
    return cfg, w, t, sorted(set(rows))


def shifted_visibility(d_tokens: int, d_blocks: int):
    """the oracle's rule with the window's edge moved for the tokens, and the blocks' edge moved separately"""
    def visible(i, size, pool):
        toks_ = [j for j in range(i + 1) if i - j < size + d_tokens]
        blocks = [b for b in range((i + 1) // pool + 1) if b * pool + pool - 1 <= i - size + d_blocks] if pool > 0 else []
        return toks_, blocks
    return visible


@pytest.mark.parametrize("size,pool", [(24, 5), (64, 16), (65, 12), (40, 64), (30, 0)])
def test_keys_just_inside_and_just_outside_the_window_and_the_blocks(size, pool, monkeypatch):
    """marks at the sequence's start (the first tokens a window keeps and loses), in the middle of pages and where an
    edge falls on a page border; a window or a block rule that is one token off in either direction changes the marked
    rows by far more than the tolerance.  In prompts (cut at, before and after the edges) and decoded one by one, fp32 and bf16."""
    cfg, w, t, rows = edge_setup(size, pool)
    ref = vo.forward(cfg, w, t)
    for dt, db in ((-1, 0), (1, 0)) + (((0, -1), (0, 1)) if pool else ()):
        monkeypatch.setattr(vo, "visible", shifted_visibility(dt, db))
        assert err(vo.forward(cfg, w, t)[rows], ref[rows]) > 100 * TOL["float32"], (dt, db)
        monkeypatch.undo()
    first = rows[0]
    for dtype in ("float32", "bfloat16"):
        e = err16 if dtype == "bfloat16" else err
        with Rig(cfg, dtype, weights=w, max_tokens=1024, max_batch_tokens=1024) as rig:
            got = run_schedule(rig, t, [len(t)])
            assert e(got, ref) < TOL[dtype] and e(got[rows], ref[rows]) < TOL[dtype]
            got = run_schedule(rig, t, [first, 2, size - 1, 2, size, 17, 2, 64, max(pool, 2), 2, 100, 3, len(t)])      # portions that start and end at the edges
            assert e(got, ref) < TOL[dtype] and e(got[rows], ref[rows]) < TOL[dtype]
            got = run_schedule(rig, t, [max(1, first - 3)])                               # every edge row decoded alone
            assert e(got, ref) < TOL[dtype] and e(got[rows], ref[rows]) < TOL[dtype]


def far_setup(n: int, layer):
    """as edge_setup, for a key far back: token 63 stands at position 3 only and the last six tokens are 62s"""
    cfg = bare([layer], vocab=64)
    w = vo.random_weights(cfg, 170)
    e = w["embed"].clone()
    e[63] = -e[62]
    w["embed"] = e
    w["l0.norm1.b"] = torch.zeros_like(w["l0.norm1.b"])
    g = torch.Generator().manual_seed(171)
    t = torch.randint(0, 62, (n,), generator=g).tolist()
    t[3] = 63
    for p in range(n - 6, n):
        t[p] = 62
    return cfg, w, t


def test_far_key_among_hundreds_in_plain_attention():
    """attention whose values are its keys: the marked token at position 3 is seen from 700 positions on, through the
    prompt kernels and through decode rows split over several blocks"""
    dk = 32
    cfg, w, t = far_setup(706, att(heads=2, kv_heads=1, dim=dk, scale=0.5, q_temp={"coef": 0.5, "every": 64}))
    w["l0.mix.k"] = -w["l0.mix.q"][:dk].clone()
    ref = vo.forward(cfg, w, t)
    t_without = list(t)
    t_without[3] = 5
    assert err(vo.forward(cfg, w, t_without)[-6:], ref[-6:]) > 100 * TOL["float32"]       # the far key matters
    with Rig(cfg, "float32", weights=w, max_batch_tokens=1024) as rig:
        assert err(run_schedule(rig, t, [len(t)]), ref) < TOL["float32"]
        assert err(run_schedule(rig, t, [300, 2, 250, 148]), ref) < TOL["float32"]        # the last six decoded one by one
    with Rig(cfg, "bfloat16", weights=w, max_batch_tokens=1024) as rig:
        assert err16(run_schedule(rig, t, [300, 2, 250, 148])[-6:], ref[-6:]) < TOL["bfloat16"]
        assert err16(run_schedule(rig, t, [len(t)])[-6:], ref[-6:]) < TOL["bfloat16"]


def test_far_key_through_a_pooled_block():
    """a window of 50 behind which blocks of two tokens are pooled: the marked tokens at positions 2 and 3 are seen 700 positions
    on only as block 1, among 320 other blocks"""
    dk = 32
    cfg, w, t = far_setup(706, par(heads=2, kv_heads=1, dim=dk, vdim=16, scale=0.5, mask={"size": 50, "pool": 2}, rot=None, right={"heads": 2, "dim": 8}))
    w["l0.mix.left.k"] = -w["l0.mix.left.q"][:dk].clone()
    w["l0.mix.left.q.norm"] = torch.ones(dk)
    w["l0.mix.left.k.norm"] = torch.ones(dk)
    t[2] = 63                                                                            # block 1 = positions 2 and 3
    ref = vo.forward(cfg, w, t)
    t_without = list(t)
    t_without[2] = t_without[3] = 5
    assert err(vo.forward(cfg, w, t_without)[-6:], ref[-6:]) > 100 * TOL["float32"]
    with Rig(cfg, "float32", weights=w, max_batch_tokens=1024) as rig:
        assert err(run_schedule(rig, t, [len(t)]), ref) < TOL["float32"]
        assert err(run_schedule(rig, t, [300, 2, 250, 148]), ref) < TOL["float32"]
    with Rig(cfg, "bfloat16", weights=w, max_batch_tokens=1024) as rig:
        assert err16(run_schedule(rig, t, [300, 2, 250, 148])[-6:], ref[-6:]) < TOL["bfloat16"]
        assert err16(run_schedule(rig, t, [len(t)])[-6:], ref[-6:]) < TOL["bfloat16"]


def test_a_sink_as_large_as_the_best_score():
    """sinks of the size of the marked score: leaving the sink out (or scaling it) changes every row"""
    cfg, w, t, rows = edge_setup(24, 5)
    w["l0.mix.left.sink"] = torch.tensor([14.0, 3.0])
    ref = vo.forward(cfg, w, t)
    w0 = dict(w)
    w0["l0.mix.left.sink"] = torch.tensor([-30.0, -30.0])
    assert err(vo.forward(cfg, w0, t)[rows], ref[rows]) > 100 * TOL["float32"]
    w0["l0.mix.left.sink"] = torch.tensor([14.0, 3.0]) * cfg["layers"][0]["mixer"]["left"]["scale"]
    assert err(vo.forward(cfg, w0, t)[rows], ref[rows]) > 100 * TOL["float32"]
    for dtype in ("float32", "bfloat16"):
        e = err16 if dtype == "bfloat16" else err
        with Rig(cfg, dtype, weights=w) as rig:
            assert e(run_schedule(rig, t, [len(t)]), ref) < TOL[dtype]
            assert e(run_schedule(rig, t, [100, 2, 33]), ref) < TOL[dtype]


def test_long_rows_split_over_blocks_in_decoding():
    """decoding past 512 and 1024 visible keys (plain attention), and past a window of 600 with 70 blocks behind it: a row's
    attention is computed by several blocks and joined"""
    cfg = bare([att(heads=2, kv_heads=1, dim=16, scale=0.4, q_temp={"coef": 0.5, "every": 100}),
                par(heads=2, kv_heads=2, dim=16, vdim=40, scale=0.4, mask={"size": 600, "pool": 10})])
    t = toks(1300, seed=165)
    with Rig(cfg, "float32", max_tokens=1344, max_batch_tokens=1344) as rig:
        ref = rig.oracle(t)
        for first, n in ((508, 8), (1020, 8), (596, 8), (1290, 8)):
            lg = run_schedule(rig, t[:first + n], [first])
            assert err(lg[first:], ref[first:first + n]) < TOL["float32"]


def test_a_slow_decay_shows_a_lost_state():
    """a decay close to one and a small removal rate: the recurrent state carries the first tokens to the end, so a state
    that is dropped, zeroed or taken from another slot between portions changes the last rows"""
    cfg = bare([par(right={"heads": 2, "dim": 16})])
    w = vo.random_weights(cfg, 55)
    w["l0.mix.right.w0"] = torch.full_like(w["l0.mix.right.w0"], -9.0)
    w["l0.mix.right.a.b"] = torch.full_like(w["l0.mix.right.a.b"], -6.0)
    w["l0.mix.right.w2"] = torch.zeros_like(w["l0.mix.right.w2"])
    t = toks(200, seed=56)
    ref = vo.forward(cfg, w, t)
    other = list(t)
    other[:20] = toks(20, seed=57)
    assert err(vo.forward(cfg, w, other)[-5:], ref[-5:]) > 20 * TOL["float32"]           # the first tokens still matter at the end
    with Rig(cfg, "float32", weights=w) as rig:
        rig.eng.step([("x", toks(90, seed=58), [])])                                     # a neighbour with a state of its own
        assert err(run_schedule(rig, t, [20, 2, 90, 1, 64]), ref) < TOL["float32"]
        rig.eng.finish("x")
        assert err(run_schedule(rig, t, [150]), ref) < TOL["float32"]                    # in the slot "x" left behind


def test_first_tokens_of_a_sequence():
    """the first token takes the bigram table's extra row and convolves with zeros; so does the first token of the next
    user of its slot"""
    with Rig(FULL, "float32") as rig:
        for n in (1, 2, 3, 4, 6):
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
        lg = vo.forward(cfg, w, seq)[-1]
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
    config's architecture; the checkpoint has no head tensor (the embedding table is the head) and the decay's inner
    size comes from its tensor's shape"""
    import json
    import os
    import struct
    import subprocess
    import sys

    import numpy as np

    cfg = config([par(DENSE), att(DENSE)])
    w = vo.random_weights(cfg, 110, rank=5)
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
    ref = vo.forward(cfg, w, t)
    got = [torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4")).view(-1, cfg["vocab"]) for i in range(3)]
    assert err(got[0], ref[[49]]) < TOL["float32"]
    assert err(got[1], torch.cat([ref[[50, 51]], vo.forward(cfg, w, t[:9])[[8]]])) < TOL["float32"]
    assert err(got[2], ref[[69]]) < TOL["float32"]
    reqs = [{"id": "x", "prompt": t[:40], "max_new_tokens": 5}, {"id": "y", "prompt": t[:7], "max_new_tokens": 3}]
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "generate"), "--model", str(folder), "--dtype", "float32", "--max-tokens", "192",
                        "--step-tokens", "16"], input="\n".join(json.dumps(r) for r in reqs) + "\n", capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    outs = {o["id"]: o["tokens"] for o in map(json.loads, p.stdout.strip().splitlines())}
    for r in reqs:
        assert len(outs[r["id"]]) == r["max_new_tokens"]
        greedy_agrees(cfg, w, r["prompt"], outs[r["id"]])


def test_served_by_the_shard_runtime():
    """load_model_core finds the class by the config's architecture and serves it with the batched policy: frames of
    tokens in, sampled tokens out, chunked prompts, slots and pages returned at release"""
    import queue

    from dnet_b200.shard.models import ShardLoadModelRequest
    from dnet_b200.shard.policies.batched import BatchedStepPolicy
    from dnet_b200.shard.runtime import ShardRuntime
    from dnet_b200.utils.model import HostDictSource
    from tests.helpers import ring_generate, token_message

    w = vo.random_weights(FULL, 21)
    n = len(FULL["layers"])
    rt = ShardRuntime(shard_id="s0", queue_size=64)
    rt.kv_cache_config.max_tokens = 256
    src = HostDictSource({k: v.to(torch.bfloat16) for k, v in w.items()}, FULL)
    rt.load_model_core(ShardLoadModelRequest(model_path=src, total_layers=n, layers=list(range(n)), window_size=n, residency_size=n, kv_bits="fp16"))
    try:
        assert isinstance(rt.policy, BatchedStepPolicy)
        a, b = toks(45, seed=180), toks(70, seed=181)
        out_a = [t for t, _, _ in ring_generate([rt], "na", a, 5)]
        greedy_agrees(FULL, w, a, out_a, margin=5e-2 * float(vo.forward(FULL, w, a)[-1].std()))
        for part in (b[:30], b[30:64]):
            rt.policy.process(token_message(rt, "nb", part, more=True))
            with pytest.raises(queue.Empty):
                rt.activation_send_queue.get_nowait()
        out_b = [t for t, _, _ in ring_generate([rt], "nb", b[64:], 4)]
        greedy_agrees(FULL, w, b, out_b, margin=5e-2 * float(vo.forward(FULL, w, b)[-1].std()))
        rt.release_nonce("na")
        rt.release_nonce_deferred("nb")
        assert rt.model.free_pages == rt.model.pool_pages
    finally:
        assert rt.unload_model_core().success
