"""Host logic of LoadedModel.prefill_many: how the rows of several prompts are packed into forward passes."""
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
import __graft_entry__ as _entry  # noqa: E402

_entry.load_package()
from gptrs_b200 import model as gm  # noqa: E402


class _Recorder(gm.LoadedModel):
    """LoadedModel with the two engine calls prefill_many makes replaced by a recorder."""

    def __init__(self, config):  # no engine handle
        self.config = config
        self._h = None
        self.lens = {}
        self.passes = []

    def __del__(self):
        pass

    def sequence_length(self, slot=0):
        return self.lens.get(slot, 0)

    def forward_with_decode_cache(self, tokens, slots, positions, logit_rows=(), want_logits=True, temperature=0.0, seed=0):
        self.passes.append((list(tokens), list(slots), list(positions), list(logit_rows)))
        for s, p in zip(slots, positions):
            assert p == self.lens.get(s, 0), "rows of a sequence arrive in order, without gaps"
            self.lens[s] = p + 1
        return None, np.array([tokens[r] + 1000 for r in logit_rows], dtype=np.int32)  # "sampled" = last token + 1000


def _cfg(n_q=32, n_kv=8, max_tokens=64, max_logit_rows=0, max_seqs=8):
    return gm.ModelConfig(gm.KIND_MINISTRAL, 1, 128, n_q, n_kv, 4, 128, 1000, 4096, max_seqs=max_seqs, max_tokens=max_tokens,
                          max_logit_rows=max_logit_rows)


@pytest.mark.parametrize("lens,chunk", [((64, 64, 64), 48), ((5, 33, 17, 64, 8, 40), 32), ((1, 1, 1, 1), 64), ((200,), 64), ((4, 4, 4, 4, 4), 64)])
def test_rows_are_packed_in_order_and_every_prompt_gets_its_id(lens, chunk):
    m = _Recorder(_cfg())
    rng = np.random.default_rng(sum(lens))
    prompts = [rng.integers(0, 1000, size=n) for n in lens]
    first = m.prefill_many(list(range(len(lens))), prompts, chunk=chunk)
    assert first == [int(p[-1]) + 1000 for p in prompts]
    assert [m.lens[s] for s in range(len(lens))] == list(lens)
    flat = [t for p in m.passes for t in p[0]]
    assert flat == [int(t) for p in prompts for t in p]            # nothing dropped, duplicated or reordered
    align = 16 // (32 // 8)
    for tok, sl, pos, rows in m.passes:
        assert 0 < len(tok) <= chunk
        for i in range(len(tok)):                                   # aligned groups of rows share a sequence
            assert sl[i] == sl[i - i % align]


def test_full_passes_span_prompt_boundaries():
    m = _Recorder(_cfg(max_tokens=48))
    m.prefill_many([0, 1, 2], [np.arange(64)] * 3, chunk=48)
    assert [len(p[0]) for p in m.passes] == [48, 48, 48, 48]       # 192 rows = four full passes
    assert m.passes[1][1][:16] == [0] * 16 and m.passes[1][1][16:] == [1] * 32
    assert [p[3] for p in m.passes] == [[], [15], [31], [47]]


def test_logit_row_limit_and_continuation():
    m = _Recorder(_cfg(max_tokens=64, max_logit_rows=2, max_seqs=8))
    first = m.prefill_many([0, 1, 2, 3, 4], [np.arange(4) + 10 * i for i in range(5)], chunk=64)
    assert first == [1003, 1013, 1023, 1033, 1043] and max(len(p[3]) for p in m.passes) <= 2
    # a second prompt appended to a slot continues at its length
    m.prefill_many([1], [np.arange(6)], chunk=64)
    assert m.passes[-1][2] == list(range(4, 10))


def test_passes_for_the_tensor_core_attention_are_always_full():
    """Heads of 128 on the paged bf16 path with passes of at least two 256-row tiles: the engine's tensor-core prefill
    attention serves a tile that holds two sequences, so no pass is cut at a sequence boundary."""
    cfg = gm.ModelConfig(gm.KIND_MINISTRAL, 1, 128, 32, 8, 128, 128, 1000, 4096, max_seqs=8, max_tokens=256, max_logit_rows=8,
                         weight_mode=gm.MODE_W4A16)
    m = _Recorder(cfg)
    lens = (301, 77, 190, 255, 13)
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, 1000, size=n) for n in lens]
    first = m.prefill_many(list(range(len(lens))), prompts, chunk=256)
    assert first == [int(p[-1]) + 1000 for p in prompts]
    assert [len(p[0]) for p in m.passes] == [256, 256, 256, sum(lens) - 3 * 256]
    assert [t for p in m.passes for t in p[0]] == [int(t) for p in prompts for t in p]
