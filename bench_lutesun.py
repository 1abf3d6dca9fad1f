"""bench_lutesun.py -- `bench.py --config lutesun`: prefill and decode throughput of the Lutesun family (latent attention
under a sliding window, RMS norms on the sublayers' outputs, a dense relu-squared feed-forward or experts routed by
corrected group-limited scores with a gated shared expert) beside Filinex, the closest family of this framework (same
library, same ragged-batch step, gated attention heads, routed experts with a shared one), at equal width, heads, layer
runs and active feed-forward width.  Random weights, synthetic tokens, one GPU.

Per size: prefill (one P-token prompt in one step), decode of one and of four sequences at the end of a P-token
context, and the device time of every phase of the step (the library's phase timers) with its algorithmic FLOPs or
bytes and the fraction of the measured peak, for both families.
"""
from __future__ import annotations

from bench_filinex import _run_filinex, filinex_algorithmic
from bench_seqmix import HD, SIZES, VOCAB, _Flusher, _rand, _roofline, _timed

EXPERTS, IDENTITY, TOP = 16, 4, 2
ROT, KV_RANK, WINDOW = 64, 512, 1024


def lutesun_config(sz: dict) -> dict:
    """6 layers: the first with the dense feed-forward, one of the routed ones with the second mixer type.  Heads of 128
    unrotated + 64 rotated query dims and 128 value dims over a latent of 512 (a cached row of 576 numbers a token
    and layer); active feed-forward width = top x expert width + shared width = the dense width of the size."""
    W, H, ff = sz["width"], sz["heads"], sz["ff"]
    moe = {"kind": "moe", "router": {"experts": EXPERTS, "top": TOP, "identity": IDENTITY, "scale": 2.0, "groups": {"count": 4, "keep": 2}},
           "expert": {"ff": ff // 4}, "shared": {"ff": ff // 2}}
    mx = {"heads": H, "dim": HD, "rot_dim": ROT, "vdim": HD, "kv_rank": KV_RANK, "scale": (HD + ROT) ** -0.5, "rot": {"base": 10000.0, "dims": ROT},
          "mask": {"size": WINDOW}}
    one = {"type": "latent_attention", "mixer": mx, "mlp": moe}
    two = {"type": "latent_attention_2", "mixer": {**mx, "q_rank": max(256, W // 2)}, "mlp": moe}
    return {"architecture": "Lutesun", "vocab": VOCAB, "width": W, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "layers": [{**one, "mlp": {"kind": "dense", "ff": ff}}, one, one, two, one, one]}


def lutesun_weights(model, g, dev):
    import torch

    items = []
    for name, shape in model.expected_tensors().items():
        leaf = name.split(".", 1)[-1]
        if leaf in ("post1", "post2") or name == "final.norm":
            t = torch.zeros(shape, dtype=torch.bfloat16, device=dev)
        elif leaf.endswith(".norm"):
            t = torch.ones(shape, dtype=torch.bfloat16, device=dev)
        elif leaf.endswith(".b") or leaf == "router.corr":
            t = _rand(shape, g, 0.05, dev)
        elif name == "embed":
            t = _rand(shape, g, 1.0, dev)
        else:
            t = _rand(shape, g, shape[-1] ** -0.5, dev)
        items.append((name, t))
    return items


def lutesun_algorithmic(cfg: dict, N: int, ctx0: int, n_seqs: int) -> dict:
    """FLOPs and the bytes that must move per phase, for a step of n_seqs entries x (N / n_seqs) tokens whose
    sequences already hold ctx0 tokens each; summed over the layers.  Attention is counted in the form the kernels
    compute: H heads over one cached row of R + rot numbers a token, values = its first R."""
    W = cfg["width"]
    keys = ("proj", "latent_in", "attn", "latent_out", "out_proj", "moe_up", "moe_down", "ff_up", "ff_down")
    f = {k: 0.0 for k in keys}
    by = dict(f)
    per = N // n_seqs
    for L in cfg["layers"]:
        mx = L["mixer"]
        H, dn, dr, dv, R = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
        qr = mx.get("q_rank", 0) if L["type"] == "latent_attention_2" else 0
        gate = H if L["type"] == "latent_attention_2" else 0
        cq = H * (dn + dr)
        wq = (W * qr + qr * cq) if qr else W * cq
        f["proj"] += 2.0 * N * (wq + W * (R + dr + gate))
        by["proj"] += 2.0 * (wq + W * (R + dr + gate))
        f["latent_in"] += 2.0 * N * H * dn * R
        by["latent_in"] += 2.0 * H * dn * R + 2.0 * N * (cq + H * (R + dr))
        win = mx["mask"]["size"]
        vis = sum(min(p + 1, win) for p in range(ctx0, ctx0 + per)) * n_seqs
        f["attn"] += 2.0 * (2 * R + dr) * H * vis
        by["attn"] += 2.0 * n_seqs * min(ctx0 + per, win + per) * (R + dr) + 2.0 * N * H * (2 * R + dr)
        f["latent_out"] += 2.0 * N * H * dv * R
        by["latent_out"] += 2.0 * H * dv * R + 2.0 * N * H * (R + dv)
        f["out_proj"] += 2.0 * N * W * H * dv
        by["out_proj"] += 2.0 * W * H * dv
        mlp = L.get("mlp")
        if not mlp:
            continue
        if mlp["kind"] == "dense":
            f["ff_up"] += 2.0 * N * W * mlp["ff"]
            by["ff_up"] += 2.0 * W * mlp["ff"]
            f["ff_down"] += 2.0 * N * W * mlp["ff"]
            by["ff_down"] += 2.0 * W * mlp["ff"]
            continue
        E, top, ef = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["ff"]
        share = E / float(E + mlp["router"].get("identity", 0))      # pairs that land on an expert with matrices, on average
        hit = min(E, N * top)
        f["moe_up"] += 4.0 * N * top * share * W * ef
        by["moe_up"] += 4.0 * hit * W * ef
        f["moe_down"] += 2.0 * N * top * share * W * ef
        by["moe_down"] += 2.0 * hit * W * ef
        if mlp.get("shared"):
            sf = mlp["shared"]["ff"]
            up, down = ("moe_up", "moe_down") if N <= 8 else ("ff_up", "ff_down")
            f[up] += 4.0 * N * W * sf
            by[up] += 4.0 * W * sf
            f[down] += 2.0 * N * W * sf
            by[down] += 2.0 * W * sf
    return {"flops": f, "bytes": by}


def _run_lutesun(sz: dict, args, P: int, flush, dev) -> dict:
    import torch

    from dnet_b200.core.models import get_ring_model

    cfg = lutesun_config(sz)
    pages = 4 * ((P + 64 + 63) // 64)
    model = get_ring_model("lutesun", cfg, assigned_layers=list(range(len(cfg["layers"]))), dtype="bfloat16", kv_pool_pages=pages,
                           max_seqs=4, max_batch_tokens=max(P, 64))
    g = torch.Generator(device=dev).manual_seed(7)
    model.load_weights(lutesun_weights(model, g, dev), strict=True)
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

    res = {"config": {"layers": [l["type"] + ("+dense" if l["mlp"]["kind"] == "dense" else "+moe") for l in cfg["layers"]], "layer_runs": model.layer_runs,
                      "experts": EXPERTS, "identity": IDENTITY, "top": TOP, "kv_rank": KV_RANK, "rot_dim": ROT, "window": WINDOW}}
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


def run_lutesun(args, rank: int, local_rank: int, world: int) -> None:
    import time

    import torch

    import bench as B
    import bench_seqmix as BS
    from bench import ClockSampler, log

    if world != 1:
        raise SystemExit("--config lutesun runs on one GPU")
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
    BS.FP32_PHASES = ("recur",)
    sizes, launches = {}, 0
    for name in args.seqmix_sizes.split(","):
        sz = SIZES[name]
        with torch.cuda.stream(side):
            lu = _run_lutesun(sz, args, P, flush, dev)
            fx = _run_filinex(sz, args, P, flush, dev)
        side.synchronize()
        launches += lu.pop("launches") + fx.pop("launches")
        lcfg, fcfg = lu.pop("cfg"), fx.pop("cfg")
        for key in ("prefill", "decode_bs1", "decode_bs4"):
            n_seq = 4 if key.endswith("4") else 1
            N, ctx0 = (P, 0) if key == "prefill" else (n_seq, lu[key]["context"])
            lu[key]["roofline"] = _roofline(lu[key]["phases_ms"], lutesun_algorithmic(lcfg, N, ctx0, n_seq), tf, gbs, f32_tf)
            fx[key]["roofline"] = _roofline(fx[key]["phases_ms"], filinex_algorithmic(fcfg, N, ctx0, n_seq), tf, gbs, f32_tf)
            lu[key]["vs_filinex"] = round(lu[key]["tok_s"] / fx[key]["tok_s"], 4)
            log(f"{name} {key}: lutesun {lu[key]['ms']:.3f} ms ({lu[key]['tok_s']:,.0f} tok/s), filinex {fx[key]['ms']:.3f} ms ({fx[key]['tok_s']:,.0f} tok/s)")
            log("   lutesun " + ", ".join(f"{k} {v['ms']:.3f}ms/{v['frac']:.3f}" for k, v in lu[key]["roofline"].items()))
            log("   filinex " + ", ".join(f"{k} {v['ms']:.3f}ms/{v['frac']:.3f}" for k, v in fx[key]["roofline"].items()))
            log("   lutesun phases " + ", ".join(f"{k} {v:.3f}" for k, v in lu[key]["phases_ms"].items() if v > 0))
        sizes[name] = {"dims": sz, "lutesun": lu, "filinex": fx}
    tw1 = time.perf_counter()
    head = sizes[args.seqmix_sizes.split(",")[-1]]
    out = {"metric": "prefill tok/s Lutesun (layer-list family) beside Filinex at equal size, one prompt in one step",
           "value": head["lutesun"]["prefill"]["tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
           "ms_per_step": head["lutesun"]["prefill"]["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
           "data": "synthetic",
           "config": {"model": "Lutesun, random weights", "prompt_len": P, "sizes": args.seqmix_sizes,
                      "timing": "CUDA events around each step, a 256 MB buffer written between steps (L2 flush)",
                      "peaks": {"bf16_tflops": tf, "hbm_gbs": gbs, "source": peak_src, "fp32_tflops_nominal": round(f32_tf, 1)}},
           "gpu_launches": launches, "sizes": sizes, "clocks": sampler.summary(tw0, tw1)}
    sampler.stop()
    B.emit(out)
