"""The packed arrays of a step (host side): flat token rows, per-request arrays, the order in which
the attention launches take the requests, padding of fixed-size batches."""
import torch

from tffinfer_b200.engine.batch import StepEntry, batch_from_device
from host_twin import build_step_batch, pack_step


def _batch(lens_new, lens_old, page=4):
    entries = [StepEntry(i, [7] * n, [n - 1]) for i, n in enumerate(lens_new)]
    tables, k = [], 0
    for n, o in zip(lens_new, lens_old):
        b = -(-(n + o) // page)
        tables.append(list(range(k, k + b)))
        k += b
    return entries, tables


def test_flat_rows_positions_and_wanted_rows():
    entries, tables = _batch([3, 1, 5], [0, 9, 2])
    b = build_step_batch(entries, [0, 9, 2], [0, 1, 2], [tables], "cpu")
    assert b.num_tokens == 9 and b.num_requests == 3 and b.max_q_len == 5 and b.max_kv_len == 10
    assert b.q_start.tolist() == [0, 3, 4, 9]
    assert b.positions.tolist() == [0, 1, 2, 9, 2, 3, 4, 5, 6]
    assert b.tok_req.tolist() == [0, 0, 0, 1, 2, 2, 2, 2, 2]
    assert b.kv_len.tolist() == [3, 10, 7]
    assert b.logit_rows.tolist() == [2, 3, 8]
    assert not b.all_decode
    assert b.block_tables[0][1].tolist()[:3] == tables[1]


def test_requests_are_ordered_by_new_tokens_then_longest_context_first():
    # decoded tokens (one new token) of contexts 50, 400, 7 and 120 beside portions of 30 and 12 tokens
    new, old = [1, 30, 1, 1, 12, 1], [49, 5, 399, 6, 100, 119]
    entries, tables = _batch(new, old)
    b = build_step_batch(entries, old, list(range(6)), [tables], "cpu")
    order = b.req_order.tolist()
    assert order == [2, 5, 0, 3, 4, 1]
    assert b.h_sorted_q_lens.tolist() == [1, 1, 1, 1, 12, 30]
    assert b.h_sorted_kv_lens.tolist() == [400, 120, 50, 7, 112, 35]


def test_padding_requests_of_a_fixed_size_batch_do_not_count_as_context():
    new, old = [1, 1, 1], [10, 300, 40]
    entries, tables = _batch(new, old)
    arr, layout, info = pack_step(entries, old, [0, 1, 2], [tables], pad_requests=8, widths=(80,),
                                  dummy_pages=[999], dummy_slot=5)
    b = batch_from_device(torch.from_numpy(arr), layout, info)
    assert b.num_requests == 8 and b.real_requests == 3 and b.all_decode
    kv = b.h_sorted_kv_lens
    assert sorted(kv.tolist(), reverse=True)[:3] == [301, 41, 11] and int(kv.sum()) == 353
    # the padding rows write to the spare page and slot
    assert b.block_tables[0][3:].unique().tolist() == [999]
    assert b.slots.tolist()[3:] == [5] * 5
