"""The description of a captured prompt step, without a GPU: how tokens, sequences, wanted rows and query blocks
are padded (engine/step.py, StepDescription.write_prompts), and how shapes and picking kinds are bucketed
(engine/graphs.py)."""
import types

import numpy as np
import pytest


class _FakeCache:
    max_seqs = 9

    def __init__(self, tables):
        self.tables = tables

    def page_table_rows(self, slots, group):
        return [self.tables[s] for s in slots]


def _description(n_tokens, n_seqs, n_want, width, sizes, tables):
    from stratum_b200.engine.step import StepDescription
    engine = types.SimpleNamespace(cache=_FakeCache(tables), kv_groups=[0],
                                   runtime=types.SimpleNamespace(device="cpu"))
    return StepDescription(engine, n_tokens, n_seqs, n_want, width, qblock_sizes=sizes)


def test_prompts_padded_in_tokens_sequences_and_blocks():
    d = _description(16, 4, 4, 2, (4, 8), {5: [7, 3], 2: [1]})
    d.write_prompts([5, 2], [6, 3], [[5], [0, 2]])
    d.write_tokens([[10, 11, 12, 13, 14, 15], [20, 21, 22]], [64, 0])
    v = d.views
    assert v["seq"].tolist() == [0] * 6 + [1] * 3 + [-1] * 7           # tokens beyond the step's belong to no sequence
    assert v["start"].tolist() == [0, 6, 9, 9, 9]                       # sequences beyond the step's bring no token
    assert v["slot"].tolist() == [5, 2, 9, 9]                           # ... and have the spare state row
    assert v["want"].tolist() == [5, 6, 8, 0]                           # surplus wanted rows point at row 0
    assert v["ids"].tolist() == [10, 11, 12, 13, 14, 15, 20, 21, 22] + [0] * 7
    assert v["pos"].tolist() == [64, 65, 66, 67, 68, 69, 0, 1, 2] + [0] * 7
    assert v["len"].tolist() == [70, 3, 0, 0]
    assert v["tables"].reshape(4, 2).tolist() == [[7, 3], [1, -1], [-1, -1], [-1, -1]]
    # query blocks of 4 tokens: 6 -> 4 + 2, 3 -> 3; the list has room for 16 / 4 + 4 entries, the rest are empty
    qb4 = v["qb4"].reshape(3, 8)
    assert qb4[0].tolist() == [0, 0, 1, -1, -1, -1, -1, -1]
    assert qb4[1].tolist() == [0, 4, 6, 0, 0, 0, 0, 0]
    assert qb4[2].tolist() == [4, 2, 3, 0, 0, 0, 0, 0]
    qb8 = v["qb8"].reshape(3, 6)
    assert qb8[:, :2].tolist() == [[0, 1], [0, 6], [6, 3]] and qb8[0, 2:].tolist() == [-1] * 4
    assert d.n_new == [6, 3, 0, 0] and d.single is False
    # the same description serves the next step of its shape: nothing of the step before is left
    d.write_prompts([2], [2], [[1]])
    d.write_tokens([[30, 31]], [3])
    assert v["seq"].tolist() == [0, 0] + [-1] * 14 and v["want"].tolist() == [1, 0, 0, 0]
    assert v["tables"].reshape(4, 2).tolist() == [[1, -1], [-1, -1], [-1, -1], [-1, -1]]
    assert v["qb4"].reshape(3, 8)[0].tolist() == [0] + [-1] * 7 and v["len"].tolist() == [5, 0, 0, 0]


def test_a_step_too_large_for_its_description_is_refused():
    from stratum_b200.engine.step import StepError
    d = _description(8, 2, 2, 1, (4,), {0: [0], 1: [1], 2: [2]})
    with pytest.raises(StepError, match="9 tokens"):
        d.write_prompts([0, 1], [5, 4], [[0], [0]])
    with pytest.raises(StepError, match="3 sequences"):
        d.write_prompts([0, 1, 2], [1, 1, 1], [[0], [0], [0]])
    with pytest.raises(StepError, match="3 wanted"):
        d.write_prompts([0, 1], [2, 2], [[0, 1], [0]])


def test_shapes_and_picking_kinds():
    from stratum_b200.engine.graphs import (PICK_DRAW, PICK_FILTERED_MANY_ROWS, PICK_GREEDY, padded_rows, padded_seqs,
                                            padded_tokens, pick_kind, width_bucket)
    assert [padded_tokens(n, 1024) for n in (1, 64, 65, 512, 513, 1024, 1025)] == [64, 64, 128, 512, 640, 1024, None]
    assert [padded_seqs(n) for n in (1, 2, 3, 8, 9, 64)] == [1, 2, 4, 8, 16, 64]
    assert [padded_rows(n) for n in (1, 7, 8, 9, 17, 64)] == [1, 7, 8, 16, 24, 64]
    assert [width_bucket(n) for n in (1, 2, 3, 33, 64)] == [1, 2, 4, 64, 64]
    assert pick_kind(8, 0.0, 50, 0.9) == PICK_GREEDY and pick_kind(64, -1.0, 0, 1.0) == PICK_GREEDY
    assert pick_kind(8, 0.7, 0, 1.0) == PICK_DRAW and pick_kind(64, 0.7, 0, 1.0) == PICK_DRAW
    assert pick_kind(32, 0.7, 50, 1.0) == PICK_DRAW               # up to 32 rows the 32-block kernel filters too
    assert pick_kind(40, 0.7, 50, 1.0) == PICK_FILTERED_MANY_ROWS and pick_kind(64, 0.7, 0, 0.9) == PICK_FILTERED_MANY_ROWS
