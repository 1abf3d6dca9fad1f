"""Generate from a layer-list model (Moputar, Filinex, Lutesun) with the continuous-batching token loop.

    bin/generate --model DIR [--dtype bfloat16|float32] [--max-new-tokens N] [--temperature T] [--top-p P] [--top-k K]
                 [--max-tokens N] [--max-seqs S] [--step-tokens B] [--seed X]

Standard input: one request a line, either a JSON list of token ids or {"id": ..., "prompt": [ids], "max_new_tokens": n}.
(The checkpoints of this family carry no tokenizer: prompts and results are token ids.)  All requests are handed to
``SequenceBatcher.generate`` together: it admits as many as state slots and cache pages allow, batches prompt portions
beside decoded tokens, samples with the framework's ``Sampler`` and hands a finished request's slot and pages to the
next one.  Standard output: one JSON object a request, {"id", "tokens"}, in the order of the input.
"""
from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="generate", description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--max-new-tokens", type=int, default=16)
    ap.add_argument("--temperature", type=float, default=0.0, help="0: greedy")
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=-1)
    ap.add_argument("--min-p", type=float, default=0.0)
    ap.add_argument("--max-tokens", type=int, default=8192, help="tokens the cache pool holds (64-token pages)")
    ap.add_argument("--max-seqs", type=int, default=4, help="state slots (live requests)")
    ap.add_argument("--step-tokens", type=int, default=512, help="token budget of a step")
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)

    import torch

    from dnet_b200.core.decoding.config import DecodingConfig
    from dnet_b200.shard.batching import GenRequest, SequenceBatcher, load_model

    dec = DecodingConfig(temperature=a.temperature, top_p=a.top_p, top_k=a.top_k, min_p=a.min_p)
    reqs = []
    for i, line in enumerate(l for l in sys.stdin if l.strip()):
        obj = json.loads(line)
        if isinstance(obj, list):
            obj = {"prompt": obj}
        reqs.append(GenRequest(str(obj.get("id", i)), [int(t) for t in obj["prompt"]],
                               max_new_tokens=int(obj.get("max_new_tokens", a.max_new_tokens)), decoding=dec,
                               stop_ids=tuple(int(t) for t in obj.get("stop_ids", ()))))
    if not reqs:
        return 0
    model = load_model(a.model, a.dtype, max_tokens=a.max_tokens, max_seqs=a.max_seqs,
                       max_batch_tokens=max(64, min(a.max_tokens, a.step_tokens)))
    eng = SequenceBatcher(model, step_tokens=a.step_tokens)
    gen = torch.Generator(device="cuda").manual_seed(a.seed) if a.temperature > 0 else None
    try:
        out = eng.generate(reqs, generator=gen)
        model.check(eng.stream)
    finally:
        eng.close()
        model.destroy()
    for r in reqs:
        sys.stdout.write(json.dumps({"id": r.id, "tokens": out[r.id]}) + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
