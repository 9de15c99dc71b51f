"""Writes tests/golden/tiny_gpt.gptrschk with the gpt.rs repository's OWN Python checkpoint writer
(scripts/gptrs_eval/checkpoint.py), so that the reader and writer of this build are pinned against a
file the reference produced. Needs the gpt.rs sources; run once, commit the output.

    python tests/golden/make_checkpoint_fixture.py /path/to/gpt.rs
"""
import importlib.util
import sys
from pathlib import Path

import numpy as np

CONFIG = {"vocab_size": 64, "context_length": 32, "embed_dim": 32, "num_layers": 2, "num_heads": 4, "mlp_ratio": 4, "dropout": 0.0}


def tensors(seed: int = 11) -> dict:
    """GPT parameters in the reference's names and [in, out] layouts (crates/gpt-rs/src/model/gpt.rs:222-291)."""
    rng = np.random.default_rng(seed)
    d, v, ctx, mlp = CONFIG["embed_dim"], CONFIG["vocab_size"], CONFIG["context_length"], CONFIG["embed_dim"] * CONFIG["mlp_ratio"]
    n = lambda *s: (rng.standard_normal(size=s) * 0.5).astype(np.float32)  # noqa: E731
    out = {"tok_embeddings.weight": n(v, d), "pos_embeddings": n(ctx, d), "final_ln.gamma": 1 + n(d) * 0.1, "final_ln.beta": n(d) * 0.1,
           "lm_head": n(d, v)}
    for l in range(CONFIG["num_layers"]):
        b = f"blocks.{l}"
        out.update({f"{b}.ln_1.gamma": 1 + n(d) * 0.1, f"{b}.ln_1.beta": n(d) * 0.1, f"{b}.ln_2.gamma": 1 + n(d) * 0.1,
                    f"{b}.ln_2.beta": n(d) * 0.1, f"{b}.attention.w_qkv": n(d, 3 * d), f"{b}.attention.b_qkv": n(3 * d) * 0.1,
                    f"{b}.attention.w_out": n(d, d), f"{b}.attention.b_out": n(d) * 0.1, f"{b}.feed_forward.w_in": n(d, mlp),
                    f"{b}.feed_forward.b_in": n(mlp) * 0.1, f"{b}.feed_forward.w_out": n(mlp, d), f"{b}.feed_forward.b_out": n(d) * 0.1})
    return {k: np.ascontiguousarray(a, dtype=np.float32) for k, a in out.items()}


if __name__ == "__main__":
    ref = Path(sys.argv[1]) / "scripts" / "gptrs_eval" / "checkpoint.py"
    spec = importlib.util.spec_from_file_location("ref_checkpoint", ref)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    dst = Path(__file__).resolve().parent / "tiny_gpt.gptrschk"
    mod.save(dst, kind="gpt", config=CONFIG, tensors=tensors())
    print(dst, dst.stat().st_size, "bytes")
