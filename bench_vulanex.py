"""bench_vulanex.py -- `bench.py --config vulanex`: prefill and decode throughput of the Vulanex family (attention whose
values are its keys; a parallel mixer of windowed attention with pooled blocks and a sink beside a generalized delta
rule; layer norms, input convolutions on every sublayer, a hashed bigram row; a dense gelu-gated feed-forward) beside
Moputar, the closest family of this framework (same library, same ragged-batch step, GQA attention, a delta rule with an
fp32 state, the same gated feed-forward), at equal width, heads, layers and feed-forward width.  Random weights,
synthetic tokens, one GPU.

Per size: prefill (one P-token prompt in one step), decode of one and of four sequences at the end of a P-token
context, and the device time of every phase of the step (the library's phase timers) with its algorithmic FLOPs or
bytes and the fraction of the measured peak, for both families.
"""
from __future__ import annotations

from bench_seqmix import HD, SIZES, VOCAB, _Flusher, _rand, _roofline, _run_moputar, _timed, moputar_algorithmic

WINDOW, POOL, RANK, TAPS, RDIM, BUCKETS = 1024, 16, 64, 4, 64, 50021


def vulanex_config(sz: dict) -> dict:
    """6 layers, attention and parallel in turn.  Heads of 128; the left half under a window of 1,024 positions with blocks
    of 16 behind it, rotary on half of each head with scaled frequencies; the right half W / 64 heads of 64 (as many
    channels as the model is wide)."""
    W, H, G, ff = sz["width"], sz["heads"], sz["kv_heads"], sz["ff"]
    mlp = {"kind": "dense", "ff": ff}
    att = {"type": "attention", "mlp": mlp,
           "mixer": {"heads": H, "kv_heads": G, "dim": HD, "vdim": HD, "scale": HD ** -0.5, "q_temp": {"coef": 0.1, "every": 256}}}
    par = {"type": "parallel", "mlp": mlp,
           "mixer": {"left": {"heads": H, "kv_heads": G, "dim": HD, "vdim": HD, "scale": HD ** -0.5, "mask": {"size": WINDOW, "pool": POOL},
                              "rot": {"base": 10000.0, "dims": HD // 2, "scaling": {"factor": 4.0, "original": 2048, "fast": 32.0, "slow": 1.0}}},
                     "right": {"heads": W // RDIM, "dim": RDIM, "rank": RANK}}}
    return {"architecture": "Vulanex", "vocab": VOCAB, "width": W, "norm": {"eps": 1e-5}, "logit_scale": 0.5, "canon": {"taps": TAPS},
            "embedding": {"bigram": {"buckets": BUCKETS, "mul_prev": 8191, "mul_cur": 131}}, "layers": [att, par] * 3}


def vulanex_weights(model, g, dev):
    import torch

    items = []
    for name, shape in model.expected_tensors().items():
        leaf = name.split(".", 1)[-1]
        if leaf in ("norm1", "norm2", "mix.q.norm", "mix.k.norm", "r.norm", "l.out", "r.out") or name == "final.norm":
            t = torch.ones(shape, dtype=torch.bfloat16, device=dev)
        elif leaf.endswith(".b") or leaf in ("sink", "r.ab", "decay.b") or name == "final.norm.b":
            t = _rand(shape, g, 0.1, dev)
        elif leaf.startswith("canon"):
            t = _rand(shape, g, 0.2, dev)
        elif name in ("embed", "bigram"):
            t = _rand(shape, g, 1.0 if name == "embed" else 0.3, dev)
        else:
            t = _rand(shape, g, shape[-1] ** -0.5, dev)
        items.append((name, t))
    return items


def vulanex_algorithmic(cfg: dict, N: int, ctx0: int, n_seqs: int) -> dict:
    """FLOPs and the bytes that must move per phase, for a step of n_seqs entries x (N / n_seqs) tokens whose
    sequences already hold ctx0 tokens each; summed over the layers."""
    W = cfg["width"]
    f = {k: 0.0 for k in ("proj", "attn", "recur", "out_proj", "ff_up", "ff_down")}
    by = dict(f)
    per = N // n_seqs
    for L in cfg["layers"]:
        if L["type"] == "attention":
            mx = L["mixer"]
            H, G, dk = mx["heads"], mx["kv_heads"], mx["dim"]
            cols, co = H * dk + G * dk, H * dk
            vis = sum(p + 1 for p in range(ctx0, ctx0 + per)) * n_seqs
            f["attn"] += 4.0 * dk * H * vis
            by["attn"] += 2.0 * n_seqs * (ctx0 + per) * G * dk + 4.0 * N * H * dk          # one row a token: it is key and value
            inner = 0
        else:
            a, r = L["mixer"]["left"], L["mixer"]["right"]
            H, G, dk, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            win, pool = a["mask"]["size"], a["mask"]["pool"]
            C, d = r["heads"] * r["dim"], r["dim"]
            cols, co = H * dk + G * (dk + dv) + 5 * C + RANK, H * dv + C
            inner = RANK * C
            vis = sum(min(p + 1, win) + max(0, p - win + 1) // pool for p in range(ctx0, ctx0 + per)) * n_seqs
            f["attn"] += 2.0 * (dk + dv) * H * vis
            last = ctx0 + per - 1
            by["attn"] += 2.0 * n_seqs * (min(ctx0 + per, win + per) + max(0, last - win + 1) // pool) * G * (dk + dv) + 2.0 * N * H * (dk + dv)
            f["recur"] += 9.0 * d * d * r["heads"] * N          # u.s, w s, - a u (u.s), + k v, s.r per state element
            by["recur"] += 8.0 * n_seqs * r["heads"] * d * d + 4.0 * N * 7 * C
        f["proj"] += 2.0 * N * (W * cols + inner)
        by["proj"] += 2.0 * (W * cols + inner)
        f["out_proj"] += 2.0 * N * co * W
        by["out_proj"] += 2.0 * co * W
        ff = L["mlp"]["ff"]
        f["ff_up"] += 4.0 * N * W * ff
        by["ff_up"] += 4.0 * W * ff
        f["ff_down"] += 2.0 * N * W * ff
        by["ff_down"] += 2.0 * W * ff
    return {"flops": f, "bytes": by}


def _run_vulanex(sz: dict, args, P: int, flush, dev) -> dict:
    import torch

    from dnet_b200.core.models import get_ring_model

    cfg = vulanex_config(sz)
    pages = 4 * ((P + 64 + 63) // 64)
    model = get_ring_model("vulanex", cfg, assigned_layers=list(range(len(cfg["layers"]))), dtype="bfloat16", kv_pool_pages=pages,
                           max_seqs=4, max_batch_tokens=max(P, 64))
    g = torch.Generator(device=dev).manual_seed(7)
    model.load_weights(vulanex_weights(model, g, dev), strict=True)
    assert not model.missing_tensors()
    prompt = torch.randint(0, VOCAB, (P,), generator=torch.Generator().manual_seed(11)).tolist()
    K, Wm = args.steps, args.warmup
    live = []
    st = torch.cuda.current_stream()

    def fresh(n):
        for h in live:
            h.free()
        live.clear()
        live.extend(model.make_cache(stream=st) for _ in range(n))

    res = {"config": {"layers": [l["type"] for l in cfg["layers"]], "window": WINDOW, "pool": POOL, "taps": TAPS, "right_dim": RDIM, "rank": RANK}}
    t = _timed(lambda: model.step([(live[0], prompt)], [P - 1], stream=st), lambda: fresh(1), K, Wm, flush)
    res["prefill"] = {"ms": t, "tok_s": P / t * 1e3}
    fresh(1)
    model.profile(True)
    model.step([(live[0], prompt)], [P - 1], stream=st)
    res["prefill"]["phases_ms"] = model.profile_read(reset=True)
    model.profile(False)
    for n_seq in (1, 4):
        ctx = (P if n_seq == 1 else P // 4) - 1
        fresh(n_seq)
        model.step([(h, prompt[:ctx]) for h in live], [], stream=st)
        toks = [[int(prompt[(i * 7 + 3) % P])] for i in range(n_seq)]
        want = list(range(n_seq))
        t = _timed(lambda: model.step([(h, toks[i]) for i, h in enumerate(live)], want, stream=st), lambda: None, K, Wm, flush)
        key = "decode_bs%d" % n_seq
        res[key] = {"ms": t, "tok_s": n_seq / t * 1e3, "context": ctx}
        model.profile(True)
        for _ in range(4):
            flush()
            model.step([(h, toks[i]) for i, h in enumerate(live)], want, stream=st)
        ph = model.profile_read(reset=True)
        model.profile(False)
        res[key]["phases_ms"] = {k: v / 4 for k, v in ph.items()}
    model.check(st)
    fresh(0)
    launches = int(model._lib.dn_seq_launch_count())
    model.destroy()
    res["cfg"] = cfg
    res["launches"] = launches
    return res


def run_vulanex(args, rank: int, local_rank: int, world: int) -> None:
    import time

    import torch

    import bench as B
    import bench_seqmix as BS
    from bench import ClockSampler, log

    if world != 1:
        raise SystemExit("--config vulanex runs on one GPU")
    dev = torch.device("cuda", local_rank)
    P = int(args.seqmix_prompt)
    gbs, peak_src = B.peaks()
    tf = B.tensor_peak_tf()
    props = torch.cuda.get_device_properties(dev)
    f32_tf = props.multi_processor_count * 128 * 2 * 1.965e9 / 1e12
    flush = _Flusher(dev)
    side = torch.cuda.Stream(device=dev)
    sampler = ClockSampler(local_rank)
    sampler.start()
    tw0 = time.perf_counter()
    BS.FP32_PHASES = ("recur", "delta_rule")
    sizes, launches = {}, 0
    for name in args.seqmix_sizes.split(","):
        sz = SIZES[name]
        with torch.cuda.stream(side):
            vu = _run_vulanex(sz, args, P, flush, dev)
            mo = _run_moputar(sz, args, P, flush, dev)
        side.synchronize()
        launches += vu.pop("launches") + mo.pop("launches")
        vcfg, mcfg = vu.pop("cfg"), mo.pop("cfg")
        for key in ("prefill", "decode_bs1", "decode_bs4"):
            n_seq = 4 if key.endswith("4") else 1
            N, ctx0 = (P, 0) if key == "prefill" else (n_seq, vu[key]["context"])
            vu[key]["roofline"] = _roofline(vu[key]["phases_ms"], vulanex_algorithmic(vcfg, N, ctx0, n_seq), tf, gbs, f32_tf)
            mo[key]["roofline"] = _roofline(mo[key]["phases_ms"], moputar_algorithmic(mcfg, N, ctx0, n_seq), tf, gbs, f32_tf)
            vu[key]["vs_moputar"] = round(vu[key]["tok_s"] / mo[key]["tok_s"], 4)
            log(f"{name} {key}: vulanex {vu[key]['ms']:.3f} ms ({vu[key]['tok_s']:,.0f} tok/s), moputar {mo[key]['ms']:.3f} ms ({mo[key]['tok_s']:,.0f} tok/s)")
            log("   vulanex " + ", ".join(f"{k} {v['ms']:.3f}ms/{v['frac']:.3f}" for k, v in vu[key]["roofline"].items()))
            log("   moputar " + ", ".join(f"{k} {v['ms']:.3f}ms/{v['frac']:.3f}" for k, v in mo[key]["roofline"].items()))
            log("   vulanex phases " + ", ".join(f"{k} {v:.3f}" for k, v in vu[key]["phases_ms"].items() if v > 0))
        sizes[name] = {"dims": sz, "vulanex": vu, "moputar": mo}
    tw1 = time.perf_counter()
    head = sizes[args.seqmix_sizes.split(",")[-1]]
    out = {"metric": "prefill tok/s Vulanex (layer-list family) beside Moputar at equal size, one prompt in one step",
           "value": head["vulanex"]["prefill"]["tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
           "ms_per_step": head["vulanex"]["prefill"]["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
           "data": "synthetic",
           "config": {"model": "Vulanex, random weights", "prompt_len": P, "sizes": args.seqmix_sizes,
                      "timing": "CUDA events around each step, a 256 MB buffer written between steps (L2 flush)",
                      "peaks": {"bf16_tflops": tf, "hbm_gbs": gbs, "source": peak_src, "fp32_tflops_nominal": round(f32_tf, 1)}},
           "gpu_launches": launches, "sizes": sizes, "clocks": sampler.summary(tw0, tw1)}
    sampler.stop()
    B.emit(out)
