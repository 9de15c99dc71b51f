"""Checkpoint -> GPU model -> tokens, through load_model and the CLI front door, against the CPU oracle."""
import importlib.util
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

entry.load_package()
from gptrs_b200 import checkpoint as ck  # noqa: E402
from gptrs_b200 import model as gm  # noqa: E402
from oracle import models_ref as mr  # noqa: E402

pytestmark = pytest.mark.gpu
GOLDEN = ROOT / "tests" / "golden"
FIXTURE = GOLDEN / "tiny_gpt.gptrschk"


def _cli():
    spec = importlib.util.spec_from_file_location("gptrs_cli", ROOT / "gpt.rs_b200" / "cli.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _oracle_for_fixture():
    spec = importlib.util.spec_from_file_location("make_checkpoint_fixture", GOLDEN / "make_checkpoint_fixture.py")
    fx = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(fx)
    c = fx.CONFIG
    cfg = mr.Cfg("gpt", n_layers=c["num_layers"], d_model=c["embed_dim"], n_q=c["num_heads"], n_kv=c["num_heads"],
                 hd=c["embed_dim"] // c["num_heads"], d_mlp=c["embed_dim"] * c["mlp_ratio"], vocab=c["vocab_size"], ctx=c["context_length"])
    return mr.RefModel(cfg, fx.tensors())


def test_load_model_from_reference_written_checkpoint(cuda):
    ref = _oracle_for_fixture()
    prompt = [3, 1, 4, 1, 5]
    want_ids, want_logits = ref.generate_greedy(prompt, 12, return_logits=True)
    m = ck.load_model(FIXTURE, max_seqs=1, max_tokens=8, max_logit_rows=8)
    lg, first = m.prefill(0, prompt, want_logits=True)
    assert float(np.max(np.abs(lg - want_logits[0]))) <= 1e-4
    assert gm.generate_tokens(m, prompt, 12) == want_ids
    # a second load into the same namespace finds every derived layout in the memo
    before = m.stats()["memo_hits"]
    m2 = ck.load_model(FIXTURE, namespace=m.namespace, max_seqs=1, max_tokens=8, max_logit_rows=8)
    assert gm.generate_tokens(m2, prompt, 12) == want_ids
    assert m2.stats()["memo_hits"] >= before


def test_cli_generate_and_inspect(cuda, capsys):
    ref = _oracle_for_fixture()
    want_ids, _ = ref.generate_greedy([7, 8, 9], 10, return_logits=True)
    cli = _cli()
    assert cli.main(["generate", "--checkpoint", str(FIXTURE), "--prompt-ids", "7,8,9", "--max-tokens", "10"]) == 0
    out = capsys.readouterr()
    assert [int(t) for t in out.out.strip().split(",")] == want_ids
    assert "tokens/sec" in out.err and "Decode steady-state" in out.err
    assert cli.main(["inspect", "--checkpoint", str(FIXTURE)]) == 0
    text = capsys.readouterr().out
    assert "tok_embeddings.weight" in text and '"kind": "gpt"' in text
    with pytest.raises(SystemExit):
        cli.main(["generate", "--checkpoint", str(FIXTURE), "--prompt-ids", "1", "--top-k", "0"])
    capsys.readouterr()
    # top-k 1 leaves only the largest logit, so a temperature draw is the greedy id
    assert cli.main(["generate", "--checkpoint", str(FIXTURE), "--prompt-ids", "7,8,9", "--max-tokens", "10",
                     "--temperature", "0.8", "--top-k", "1", "--seed", "3"]) == 0
    assert [int(t) for t in capsys.readouterr().out.strip().split(",")] == want_ids


def test_cli_random_ministral_checkpoint_quantised(cuda, tmp_path, capsys):
    """export-random -> generate with W4A16 weights: same ids as the oracle on exactly dequantised weights."""
    cli = _cli()
    conf = {"vocab_size": 512, "context_length": 128, "embed_dim": 256, "num_layers": 2, "num_heads": 4, "num_kv_heads": 2,
            "head_dim": 128, "mlp_hidden_dim": 512, "rms_norm_eps": 1e-5, "rope_theta": 1e6, "rotary_dim": 128}
    import json
    path = tmp_path / "mini.gptrschk"
    assert cli.main(["export-random", "--out", str(path), "--kind", "ministral", "--config", json.dumps(conf), "--std", "0.05", "--seed", "3"]) == 0
    r = ck.CheckpointReader(path)
    params = {e.name: r.get(e.name) for e in r.entries}
    cfg = mr.Cfg("ministral", n_layers=2, d_model=256, n_q=4, n_kv=2, hd=128, d_mlp=512, vocab=512, ctx=128, rot=128)
    ref = mr.RefModel(cfg, mr.quantised_params(cfg, params, "w4"))
    prompt = list(range(5, 29))
    want_ids, _ = ref.generate_greedy(prompt, 6, return_logits=True)
    capsys.readouterr()
    assert cli.main(["generate", "--checkpoint", str(path), "--prompt-ids", " ".join(map(str, prompt)), "--max-tokens", "6",
                     "--weight-mode", "w4a16"]) == 0
    got = [int(t) for t in capsys.readouterr().out.strip().split(",")]
    # bf16 activations against an f32 oracle: the greedy ids agree wherever the oracle's top-2 margin is clear
    assert got[0] == want_ids[0]
    assert len(got) == 6
