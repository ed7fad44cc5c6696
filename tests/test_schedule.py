"""The varlen scheduler's work list: index math of the builder (host version of the same rule the
device kernel applies), checked against a plain Python restatement."""

import pytest
import torch

from nanobrain_b200 import _lib, build, schedule
from nanobrain_b200 import workloads as W


@pytest.fixture(scope="module", autouse=True)
def _built():
    build.build()


def expected_items(lengths_own, lengths_other, total_own=None):
    """Items ordered by decreasing cost (128-row steps on the other side), full tiles of all
    sequences first, ragged last tiles after them, sequences ascending inside one cost class. Rows
    past the last sequence form one more sequence with nothing on the other side (cost 0)."""
    pad = 0 if total_own is None else total_own - sum(lengths_own)
    lengths_own, lengths_other = list(lengths_own) + [pad], list(lengths_other) + [0]
    cost = [(lo + 127) // 128 for lo in lengths_other]
    order = sorted(range(len(lengths_own)), key=lambda i: (-cost[i], i))
    full = [(i, t) for i in order for t in range(lengths_own[i] // 128)]
    ragged = [(i, lengths_own[i] // 128) for i in order if lengths_own[i] % 128]
    return full + ragged


def host_list(lq, lk, side, max_q=None, max_k=None, total_q=None, total_k=None):
    lq_t, lk_t = torch.tensor(lq), torch.tensor(lk)
    cu_q, cu_k = W.cu_seqlens_from_lengths(lq_t), W.cu_seqlens_from_lengths(lk_t)
    return schedule.work_list_host(cu_q, cu_k, max_q or max(lq + [1]), max_k or max(lk + [1]),
                                   total_q if total_q is not None else sum(lq),
                                   total_k if total_k is not None else sum(lk), side)


@pytest.mark.parametrize("lengths", [
    [820], [128], [1], [127, 129, 256, 1, 0, 700], [200] * 30 + [2000], [0, 0, 5],
    W.draw_lengths(W.WORKLOADS["vitb_encoder_varlen"]).tolist(),
    W.draw_lengths(W.WORKLOADS["vitl_encoder_varlen"]).tolist(),
])
def test_self_attention_list_matches_the_rule(lengths):
    for side in (0, 1):
        items = host_list(lengths, lengths, side)
        assert items.shape == (sum(lengths) // 128 + len(lengths) + 1, 8)
        assert schedule.decode(items) == expected_items(lengths, lengths)


def test_every_tile_appears_exactly_once_and_padding_is_marked():
    lengths = [300, 5, 129, 1024, 0, 64]
    items = host_list(lengths, lengths, 0)
    got = schedule.decode(items)
    want = {(i, t) for i, l in enumerate(lengths) for t in range((l + 127) // 128)}
    assert len(got) == len(want) and set(got) == want
    assert int((items[:, 0] < 0).sum()) == items.shape[0] - len(want)
    assert bool((items[len(want):, 0] < 0).all())  # unused entries sit at the end
    # every entry carries its sequence's offsets and lengths
    cu = [0]
    for l in lengths:
        cu.append(cu[-1] + l)
    for seq, tile, ob, ol, xb, xl, _, _ in items[:len(want)].tolist():
        assert (ob, ol, xb, xl) == (cu[seq], lengths[seq], cu[seq], lengths[seq]) and tile * 128 < ol


def test_cross_attention_cost_is_the_other_side():
    lq, lk = [130, 5, 64], [3, 900, 129]
    # forward: items are query tiles, ordered by the number of key tiles of their sequence
    assert schedule.decode(host_list(lq, lk, 0)) == expected_items(lq, lk)
    # backward: items are key tiles, ordered by the number of query tiles
    assert schedule.decode(host_list(lq, lk, 1)) == expected_items(lk, lq)


def test_longest_sequences_come_first_and_ragged_tiles_last():
    lengths = [200] * 30 + [2000]
    got = schedule.decode(host_list(lengths, lengths, 1))
    assert got[:15] == [(30, t) for t in range(15)]           # the 2000-token sequence's full tiles
    assert got[15:45] == [(i, 0) for i in range(30)]          # then the full tiles of the short ones
    assert got[45] == (30, 15)                                # ragged tiles: the long sequence's first
    assert got[46:] == [(i, 1) for i in range(30)]


def test_invalid_packings_are_refused():
    lengths = [100, 200]
    with pytest.raises(RuntimeError):   # a sequence longer than max_seqlen
        host_list(lengths, lengths, 0, max_q=150, max_k=200)
    with pytest.raises(RuntimeError):   # last offset beyond the token count
        host_list(lengths, lengths, 0, total_q=299)
    cu_bad = torch.tensor([0, 200, 100], dtype=torch.int32)  # decreasing offsets
    with pytest.raises(RuntimeError):
        schedule.work_list_host(cu_bad, cu_bad, 200, 200, 300, 300, 1)


def test_rows_past_the_last_sequence_become_items_without_a_partner():
    # Packing into a buffer of fixed capacity leaves unused rows at the end; they are listed as
    # sequence index `batch` so that the kernels write zeros there.
    lengths = [100, 200]
    got = schedule.decode(host_list(lengths, lengths, 0, total_q=4096, total_k=4096))
    assert got == expected_items(lengths, lengths, total_own=4096)
    pad_items = [it for it in got if it[0] == 2]
    assert pad_items == [(2, t) for t in range((4096 - 300 + 127) // 128)]
    assert got.index(pad_items[0]) > got.index((1, 0))
