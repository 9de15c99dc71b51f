"""Command-line front door of the CUDA decode backend: the `generate` arm of the reference CLI
(crates/gpt-rs-cli/src/main.rs:451-510, 630-726) with `--backend cuda` semantics, working on token ids
(the tokenizer is outside this backend).

    python gpt.rs_b200/cli.py generate --checkpoint model.gptrschk --prompt-ids 464,2068,286 --max-tokens 64
    python gpt.rs_b200/cli.py inspect  --checkpoint model.gptrschk
    python gpt.rs_b200/cli.py export-random --out tiny.gptrschk --kind gpt --config '{"vocab_size":64,...}'

`generate` prints the generated ids (one line, comma separated) on stdout and the reference's timing
report on stderr: total tokens/s, the steady-state rate without the first token, and the wall time.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import sys
import time
from pathlib import Path


def _package():
    """The package directory is not a valid module name; register it as `gptrs_b200`."""
    if "gptrs_b200" not in sys.modules:
        here = Path(__file__).resolve().parent
        spec = importlib.util.spec_from_file_location("gptrs_b200", here / "__init__.py", submodule_search_locations=[str(here)])
        mod = importlib.util.module_from_spec(spec)
        sys.modules["gptrs_b200"] = mod
        spec.loader.exec_module(mod)
    return sys.modules["gptrs_b200"]


def _ids(args) -> list[int]:
    text = args.prompt_ids if args.prompt_ids is not None else Path(args.prompt_file).read_text()
    ids = [int(t) for t in text.replace(",", " ").split()]
    if not ids:
        raise SystemExit("prompt produced an empty token sequence")
    return ids


def cmd_generate(args) -> int:
    _package()
    from gptrs_b200 import checkpoint as ck
    from gptrs_b200 import model as gm
    prompt = _ids(args)
    mode = {"f32": gm.MODE_F32, "w4a16": gm.MODE_W4A16, "w8a16": gm.MODE_W8A16}[args.weight_mode]
    if args.top_k is not None and args.top_k < 1:
        raise SystemExit("--top-k must be at least 1")
    reader = ck.CheckpointReader(args.checkpoint)
    ctx_cap = int(reader.model_config["config"]["context_length"])
    need = len(prompt) + args.max_tokens
    if need > ctx_cap:
        raise SystemExit(f"prompt + max-tokens = {need} exceeds the model's context_length {ctx_cap}")
    kw = dict(max_seqs=1, max_tokens=min(max(len(prompt), 16), 1024), max_logit_rows=1, use_pdl=1)
    if mode != gm.MODE_F32:
        pages = (need + 15) // 16 + 1
        kw.update(kv_pages=pages + 4, max_pages_per_seq=pages)
    t_load = time.perf_counter()
    model = ck.load_model(args.checkpoint, weight_mode=mode, **kw)
    load_s = time.perf_counter() - t_load
    wall0 = time.perf_counter()
    model.reset_sequence(0)
    t0 = time.perf_counter()
    out: list[int] = []
    if args.temperature > 0:
        model.set_top_k(args.top_k)  # kept on the device, unlike the reference's host-only top-k (inference/sampler.rs:74-81)
        n = len(prompt)
        _, first = model.forward_with_decode_cache(prompt, [0] * n, list(range(n)), [n - 1], want_logits=False,
                                                   temperature=args.temperature, seed=args.seed)
        out.append(int(first[0]))
        first_s = time.perf_counter() - t0
        for i in range(1, args.max_tokens):
            _, tok = model.forward_with_decode_cache([out[-1]], [0], [n + i - 1], [0], want_logits=False,
                                                     temperature=args.temperature, seed=args.seed + i)
            out.append(int(tok[0]))
    else:
        _, first = model.prefill(0, prompt)
        out.append(first)
        first_s = time.perf_counter() - t0
        if args.max_tokens > 1:
            gen = gm.Generator(model, [first], use_graph=not args.no_graph)
            for _ in range(args.max_tokens - 1):
                out.append(int(gen.step()[0]))
    model_s = time.perf_counter() - t0
    print(",".join(str(t) for t in out))
    emitted = len(out)
    print(f"Loaded {args.checkpoint} ({reader.kind}, {len(reader.entries)} tensors) in {load_s:.2f}s", file=sys.stderr)
    print(f"Generated {emitted} tokens in {model_s:.2f}s ({emitted / max(model_s, 1e-9):.2f} tokens/sec)", file=sys.stderr)
    if emitted > 1:
        print(f"Decode steady-state (excluding first token): {(emitted - 1) / max(model_s - first_s, 1e-9):.2f} tokens/sec", file=sys.stderr)
    print(f"Wall time including decode/output: {time.perf_counter() - wall0:.2f}s", file=sys.stderr)
    return 0


def cmd_inspect(args) -> int:
    _package()
    from gptrs_b200 import checkpoint as ck
    r = ck.CheckpointReader(args.checkpoint)
    print(json.dumps(r.model_config))
    names = {ck.TAG_F32: "f32", ck.TAG_F16: "f16", ck.TAG_BF16: "bf16", ck.TAG_I32: "i32"}
    for e in r.entries:
        print(f"{e.name}\t{names[e.dtype_tag]}\t{list(e.dims)}\t{e.byte_len} B\tbase_id={e.base_id:#034x}")
    return 0


def cmd_export_random(args) -> int:
    """A checkpoint of N(0, std) weights (norm gains 1, biases 0) for a given config: stands in for
    pretrained weights where none can be downloaded."""
    _package()
    import numpy as np
    from gptrs_b200 import checkpoint as ck
    config = json.loads(args.config)
    cfg, _ = ck.engine_config({"kind": args.kind, "config": config})
    rng = np.random.default_rng(args.seed)
    tensors = {}
    for name, shape in cfg.param_shapes().items():
        if name.endswith("gamma"):
            tensors[name] = np.ones(shape, np.float32)
        elif name.endswith("beta") or ".b_" in name:
            tensors[name] = np.zeros(shape, np.float32)
        else:
            tensors[name] = (rng.standard_normal(size=shape, dtype=np.float32) * np.float32(args.std))
    ck.save(args.out, args.kind, config, tensors)
    print(f"wrote {args.out}: {len(tensors)} tensors", file=sys.stderr)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="gptrs-cuda", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate", help="greedy / temperature decode from a GPTRSCHK checkpoint")
    g.add_argument("--checkpoint", required=True)
    src = g.add_mutually_exclusive_group(required=True)
    src.add_argument("--prompt-ids", help="comma or space separated token ids")
    src.add_argument("--prompt-file", help="text file with token ids")
    g.add_argument("--max-tokens", type=int, default=64)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-k", type=int, default=None)
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--weight-mode", default="f32", choices=["f32", "w4a16", "w8a16"],
                   help="w4a16 / w8a16 quantise the linear weights on the device while loading (ministral kind)")
    g.add_argument("--no-graph", action="store_true", help="launch kernels one by one instead of replaying a CUDA graph")
    g.set_defaults(fn=cmd_generate)
    i = sub.add_parser("inspect", help="print the config and tensor index of a checkpoint")
    i.add_argument("--checkpoint", required=True)
    i.set_defaults(fn=cmd_inspect)
    x = sub.add_parser("export-random", help="write a checkpoint with random weights for a config")
    x.add_argument("--out", required=True)
    x.add_argument("--kind", required=True, choices=["gpt", "ministral"])
    x.add_argument("--config", required=True, help="the model's config JSON object")
    x.add_argument("--seed", type=int, default=0)
    x.add_argument("--std", type=float, default=0.02)
    x.set_defaults(fn=cmd_export_random)
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
