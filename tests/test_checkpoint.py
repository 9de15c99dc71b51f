"""GPTRSCHK reader / writer and the rope-table restatement (CPU). The fixture tests/golden/tiny_gpt.gptrschk
was written by the gpt.rs repository's own Python exporter (tests/golden/make_checkpoint_fixture.py)."""
import importlib.util
import struct
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

entry.load_package()
from gptrs_b200 import BackendError  # noqa: E402
from gptrs_b200 import checkpoint as ck  # noqa: E402
from gptrs_b200 import model as gm  # noqa: E402

GOLDEN = ROOT / "tests" / "golden"
FIXTURE = GOLDEN / "tiny_gpt.gptrschk"


def _fixture_module():
    spec = importlib.util.spec_from_file_location("make_checkpoint_fixture", GOLDEN / "make_checkpoint_fixture.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reader_parses_the_reference_written_file():
    fx = _fixture_module()
    r = ck.CheckpointReader(FIXTURE)
    assert r.kind == "gpt" and r.model_config["config"] == fx.CONFIG
    want = fx.tensors()
    assert [e.name for e in r.entries] == sorted(want)
    cfg, scaling = ck.engine_config(r.model_config)
    assert scaling is None and set(cfg.param_shapes()) == set(want)
    for name, shape in cfg.param_shapes().items():
        got = r.get(name)
        assert got.dtype == np.float32 and tuple(got.shape) == tuple(shape)
        assert np.array_equal(got, want[name])
        e = r.entries[r.by_name[name]]
        assert e.base_id == gm.base_param_id(name)
        assert np.array_equal(r.get_by_base_id(e.base_id), want[name])


def test_writer_is_byte_identical_to_the_reference_writer(tmp_path):
    fx = _fixture_module()
    out = tmp_path / "mine.gptrschk"
    ck.save(out, "gpt", fx.CONFIG, fx.tensors())
    assert out.read_bytes() == FIXTURE.read_bytes()


def test_stored_base_ids_are_validated(tmp_path):
    fx = _fixture_module()
    t = {k: v for k, v in fx.tensors().items() if k.startswith("final_ln")}
    good = tmp_path / "ids.gptrschk"
    ck.save(good, "gpt", fx.CONFIG, t, store_base_ids=True)
    r = ck.CheckpointReader(good)
    assert [e.base_id for e in r.entries] == [gm.base_param_id(n) for n in sorted(t)]
    raw = bytearray(good.read_bytes())
    nb = b"final_ln.beta"
    at = raw.index(nb) + len(nb)
    raw[at] ^= 0xFF  # first byte of the stored id of the first tensor
    bad = tmp_path / "bad.gptrschk"
    bad.write_bytes(bytes(raw))
    with pytest.raises(BackendError, match="base_id mismatch"):
        ck.CheckpointReader(bad)


def test_half_precision_payloads_widen_to_f32(tmp_path):
    rng = np.random.default_rng(0)
    w = rng.standard_normal(size=(5, 7)).astype(np.float32)
    p = tmp_path / "h.gptrschk"
    ck.save(p, "gpt", {}, {"a": w, "b": w, "c": np.arange(6, dtype=np.int32).reshape(2, 3)}, dtype_tags={"a": ck.TAG_F16, "b": ck.TAG_BF16})
    r = ck.CheckpointReader(p)
    assert np.array_equal(r.get("a"), w.astype(np.float16).astype(np.float32))
    import torch
    assert np.array_equal(r.get("b"), torch.from_numpy(w).to(torch.bfloat16).to(torch.float32).numpy())
    assert r.get("c").dtype == np.int32 and r.get("c").tolist() == [[0, 1, 2], [3, 4, 5]]


def test_malformed_files_are_rejected(tmp_path):
    data = FIXTURE.read_bytes()
    cases = {"magic": b"GPTRSXXX" + data[8:], "version": data[:8] + struct.pack("<I", 3) + data[12:]}
    for label, blob in cases.items():
        p = tmp_path / f"{label}.bin"
        p.write_bytes(blob)
        with pytest.raises(BackendError):
            ck.CheckpointReader(p)
    short = tmp_path / "short.bin"
    short.write_bytes(data[:-100])
    r = ck.CheckpointReader(short)  # the index is intact; the last payload is not
    with pytest.raises(BackendError, match="outside the file"):
        r.get(r.entries[-1].name)
    with pytest.raises(BackendError, match="not found"):
        r.get("no.such.tensor")
    # unknown dtype tag
    fx = _fixture_module()
    p = tmp_path / "tag.bin"
    ck.save(p, "gpt", fx.CONFIG, {"x": np.zeros(4, np.float32)})
    raw = bytearray(p.read_bytes())
    at = raw.index(b"x" + bytes(16)) + 1 + 16 + 4 + 8  # name, stored id, rank, one dim
    raw[at:at + 4] = struct.pack("<I", 9)
    p.write_bytes(bytes(raw))
    with pytest.raises(BackendError, match="unknown dtype tag"):
        ck.CheckpointReader(p)


def test_rope_tables():
    from oracle import functional_ref as fr
    cos, sin = ck.rope_tables(64, 1e6, 40)
    want_cos, want_sin = fr.rotary_cos_sin(0, 40, 64, 1e6)
    assert np.allclose(cos, want_cos, rtol=0, atol=2e-6) and np.allclose(sin, want_sin, rtol=0, atol=2e-6)
    # linear scaling by f is the unscaled table sampled at position / f
    c2, s2 = ck.rope_tables(64, 1e4, 9, {"kind": "linear", "factor": 2.0})
    c1, s1 = ck.rope_tables(64, 1e4, 5)
    assert np.allclose(c2[::2], c1, atol=1e-6) and np.allclose(s2[::2], s1, atol=1e-6)
    # yarn: factor 1 changes nothing; a larger factor keeps the fastest pair, slows the slowest by the
    # factor, and scales the magnitude by 0.1 ln(factor) + 1
    y1 = ck.rope_tables(64, 1e4, 16, {"kind": "yarn", "factor": 1.0, "original_max_position_embeddings": 4096})
    base = ck.rope_tables(64, 1e4, 16)
    assert np.allclose(y1[0], base[0], atol=1e-6) and np.allclose(y1[1], base[1], atol=1e-6)
    yc, ys = ck.rope_tables(64, 1e4, 16, {"kind": "yarn", "factor": 4.0, "original_max_position_embeddings": 4096})
    mag = np.float32(0.1 * np.log(4.0) + 1.0)
    assert np.allclose(yc[:, 0], base[0][:, 0] * mag, atol=1e-5)
    slow = np.float32(1e4) ** np.float32(-62.0 / 64.0) / np.float32(4.0)
    assert np.allclose(ys[:, 31], np.sin(np.arange(16, dtype=np.float32) * slow) * mag, atol=1e-6)
    with pytest.raises(BackendError):
        ck.rope_tables(63, 1e4, 4)
    with pytest.raises(BackendError):
        ck.rope_tables(64, 1e4, 4, {"kind": "yarn", "factor": 2.0})  # no original length, no context length


def test_cli_export_random_and_inspect_need_no_gpu(tmp_path, capsys):
    spec = importlib.util.spec_from_file_location("gptrs_cli", ROOT / "gpt.rs_b200" / "cli.py")
    cli = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(cli)
    import json
    conf = {"vocab_size": 96, "context_length": 64, "embed_dim": 128, "num_layers": 2, "num_heads": 2, "num_kv_heads": 1,
            "head_dim": 64, "mlp_hidden_dim": 256, "rms_norm_eps": 1e-5, "rope_theta": 1e4, "rotary_dim": 64,
            "rope_scaling": {"kind": "linear", "factor": 2.0}}
    out = tmp_path / "m.gptrschk"
    assert cli.main(["export-random", "--out", str(out), "--kind", "ministral", "--config", json.dumps(conf), "--seed", "5"]) == 0
    r = ck.CheckpointReader(out)
    cfg, scaling = ck.engine_config(r.model_config)
    assert scaling == {"kind": "linear", "factor": 2.0}
    assert cfg.n_kv_heads == 1 and cfg.head_dim == 64 and cfg.d_mlp == 256
    assert set(cfg.param_shapes()) == {e.name for e in r.entries}
    assert np.array_equal(r.get("final_norm.gamma"), np.ones(128, np.float32))
    capsys.readouterr()
    assert cli.main(["inspect", "--checkpoint", str(out)]) == 0
    text = capsys.readouterr().out
    assert "blocks.1.feed_forward.w_down" in text and '"kind": "ministral"' in text
