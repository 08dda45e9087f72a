"""How a step is packed, on the host: tokens of the requests one after the other, positions from where each
request stands, the rows whose logits are wanted, padded block tables per cache group, and what is refused."""
import numpy as np
import pytest
import torch

from prelude_b200.engine.batch import StepItem, build_step_batch, pack_items


def test_a_mixed_step():
    items = [StepItem("a", [5, 6, 7], 10, [0, 2]), StepItem("b", [9], 41, [0]), StepItem("c", [1, 2], 0, [])]
    q_lens, q_start, kv_len, cu_q, tokens, positions, rows = pack_items(items, vocab_size=50, max_positions=64)
    assert q_lens.tolist() == [3, 1, 2] and q_start.tolist() == [10, 41, 0] and kv_len.tolist() == [13, 42, 2]
    assert cu_q.tolist() == [0, 3, 4, 6] and tokens.tolist() == [5, 6, 7, 9, 1, 2]
    assert positions.tolist() == [10, 11, 12, 41, 0, 1] and positions.dtype == np.int32
    assert rows.tolist() == [0, 2, 3]                              # in the order of the requests and of their wanted places
    batch = build_step_batch(items, {0: [[3, 4], [7, 8, 9, 1, 2, 0], [5]], 1: [[-1, 6], [2], [0]]}, [2, 0, 1],
                             torch.device("cpu"), 50, 64)
    assert batch.n_tokens == 6 and batch.n_seqs == 3 and not batch.decode_only and batch.n_real == 6
    assert batch.token_ids.tolist() == [5, 6, 7, 9, 1, 2] and batch.positions.tolist() == [10, 11, 12, 41, 0, 1]
    assert batch.token_seq.tolist() == [0, 0, 0, 1, 2, 2] and batch.state_slots.tolist() == [2, 0, 1]
    assert batch.cu_q.tolist() == [0, 3, 4, 6] and batch.kv_len.tolist() == [13, 42, 2] and batch.logit_rows.tolist() == [0, 2, 3]
    assert batch.block_tables[0].tolist() == [[3, 4, -1, -1, -1, -1], [7, 8, 9, 1, 2, 0], [5, -1, -1, -1, -1, -1]]
    assert batch.block_tables[1].tolist() == [[-1, 6], [2, -1], [0, -1]]          # every group has its own width
    assert int(batch.status) == 0 and batch.max_q_len == 3 and batch.max_kv_len == 42
    # one buffer under all of it: a step's inputs travel in one copy
    base = batch.token_ids.untyped_storage().data_ptr()
    assert all(t.untyped_storage().data_ptr() == base for t in (batch.positions, batch.cu_q, batch.block_tables[1], batch.status))


def test_a_decode_step_and_a_workspace():
    items = [StepItem(i, [i + 1], 7 * i, [0]) for i in range(4)]
    batch = build_step_batch(items, {0: [[i] for i in range(4)]}, list(range(4)), torch.device("cpu"), 10, 100, min_table_width=3)
    assert batch.decode_only and batch.block_tables[0].shape == (4, 3) and batch.logit_rows.tolist() == [0, 1, 2, 3]
    a = batch.workspace("q", (4, 2, 8), torch.float32)
    assert batch.workspace("q", (4, 2, 8), torch.float32) is a and batch.workspace("q", (4, 2, 8), torch.bfloat16) is not a


@pytest.mark.parametrize("items,match", [
    ([], "at least one request"),
    ([StepItem("a", [], 0, [])], "at least one token"),
    ([StepItem("a", [1, 2], 63, [])], "positions"),
    ([StepItem("a", [1], -1, [])], "positions"),
    ([StepItem("a", [1, 50], 0, [])], "token ids"),
    ([StepItem("a", [-1], 0, [])], "token ids"),
    ([StepItem("a", [1, 2], 0, [2])], "wanted place"),
    ([StepItem("a", [1, 2], 0, [-1])], "wanted place"),
])
def test_refusals(items, match):
    with pytest.raises(ValueError, match=match):
        pack_items(items, vocab_size=50, max_positions=64)


def test_one_slot_per_request():
    with pytest.raises(ValueError, match="state slot"):
        build_step_batch([StepItem("a", [1], 0, [0])], {0: [[0]]}, [0, 1], torch.device("cpu"), 10, 10)
