"""Loader behaviour list (names follow the reference's data/loader/tests/{loader,strategy,
pack_concat,pack_document_mask,pack_single,pack_errors,json,shuffle,reconstruct}.rs), against
the C++ module. A plain-Python packer written from the rules is the second opinion on random
document lists."""
import json
import random

import pytest

from prometheus_b200 import native

L = native.loader


def kind_of(fn, *a, **k):
    with pytest.raises(native.NativeError) as e:
        fn(*a, **k)
    return e.value.kind


def P(strategy="concat_eos", n=4, eos=True, pad=0, **kw):
    return L.Packing("p", n, strategy, eos, pad, **kw)


def toks(seqs):
    return [s.tokens for s in seqs]


# ------------------------------------------------------------------ concat_eos
def test_two_docs_eos_between_pads_tail():
    got = L.pack([[5, 6], [7]], P(n=4), 1)
    assert [(s.tokens, s.mask) for s in got] == [([5, 6, 1, 7], [1, 1, 1, 1])]      # none after the last
    got = L.pack([[5, 6], [7, 8, 9]], P(n=4), 1)
    assert [(s.tokens, s.mask) for s in got] == [([5, 6, 1, 7], [1, 1, 1, 1]), ([8, 9, 0, 0], [1, 1, 0, 0])]


def test_two_docs_without_eos_and_single_doc_gets_no_eos_inside():
    assert toks(L.pack([[5, 6], [7]], P(n=4, eos=False), 1)) == [[5, 6, 7, 0]]
    first = L.pack([[5, 6, 7]], P(n=4), 1)[0]
    assert first.tokens[:3] == [5, 6, 7] and first.mask[:3] == [1, 1, 1]


def test_long_doc_splits_and_exact_multiple_has_no_pad():
    got = L.pack([[1, 2, 3, 4, 5, 6, 7, 8]], P(n=4, eos=False), 9)
    assert toks(got) == [[1, 2, 3, 4], [5, 6, 7, 8]] and all(s.mask == [1] * 4 for s in got)


def test_seq_len_one_emits_one_sequence_per_token():
    assert toks(L.pack([[3, 4, 5]], P(n=1, eos=False), 9)) == [[3], [4], [5]]


def test_empty_docs_in_the_list():
    with_eos = L.pack([[1], [], [2]], P(n=8), 9)
    stream = [t for s in with_eos for t, m in zip(s.tokens, s.mask) if m]
    assert stream[:4] == [1, 9, 9, 2]                     # the empty document still gets its separator
    assert L.pack([[], []], P(n=4, eos=False), 9) == []                   # nothing to emit
    only_eos = L.pack([[], []], P(n=4, eos=True), 9)
    assert [(s.tokens, s.mask) for s in only_eos] == [([9, 0, 0, 0], [1, 0, 0, 0])]


def test_pad_id_may_equal_a_real_token_and_the_mask_tells_them_apart():
    s = L.pack([[0, 0, 0]], P(n=4, eos=False, pad=0), 9)[0]
    assert s.tokens == [0, 0, 0, 0] and s.mask == [1, 1, 1, 0]


def test_drop_short_below_is_ignored_for_concat_and_order_is_kept():
    docs = [[1], [2, 3], [4]]
    a = L.pack(docs, P(n=8, eos=False, drop_short_below=2), 9)
    assert [t for s in a for t, m in zip(s.tokens, s.mask) if m] == [1, 2, 3, 4]


# --------------------------------------------------------------- document_mask
def test_document_mask_ids_track_documents_and_eos_belongs_to_the_document_it_closes():
    s = L.pack([[10, 11], [20]], P("document_mask", 5), 9)[0]
    assert s.tokens[:4] == [10, 11, 9, 20] and s.document_ids[:4] == [0, 0, 0, 1]


def test_document_mask_pad_positions_use_document_id_zero_and_split_docs_keep_their_id():
    got = L.pack([[1], [2, 3, 4, 5, 6]], P("document_mask", 4, eos=False), 9)
    assert toks(got) == [[1, 2, 3, 4], [5, 6, 0, 0]]
    assert [s.document_ids for s in got] == [[0, 1, 1, 1], [1, 1, 0, 0]] and got[1].mask == [1, 1, 0, 0]


def test_document_mask_empty_middle_document_still_advances_ids():
    s = L.pack([[1], [], [2]], P("document_mask", 8, eos=False), 9)[0]
    assert s.tokens[:2] == [1, 2] and s.document_ids[:2] == [0, 2]


def test_document_mask_tokens_and_mask_equal_concat():
    rng = random.Random(0)
    for _ in range(30):
        docs = [[rng.randrange(10, 99) for _ in range(rng.randrange(0, 7))] for _ in range(rng.randrange(1, 6))]
        if not any(docs):
            continue
        for eos in (True, False):
            a = L.pack(docs, P("concat_eos", 5, eos), 1)
            b = L.pack(docs, P("document_mask", 5, eos), 1)
            assert [(s.tokens, s.mask) for s in a] == [(s.tokens, s.mask) for s in b]
            assert all(s.document_ids is None for s in a) and all(len(s.document_ids) == 5 for s in b)


# ------------------------------------------------------------- single_document
def test_single_document_pads_truncates_and_ignores_eos_settings():
    got = L.pack([[1, 2], [3, 4, 5, 6, 7, 8]], P("single_document", 4, eos=True, pad=7), 99)
    assert [(s.tokens, s.mask) for s in got] == [([1, 2, 7, 7], [1, 1, 0, 0]), ([3, 4, 5, 6], [1, 1, 1, 1])]


def test_single_document_drop_threshold_keeps_equal_and_order():
    got = L.pack([[1], [2, 3], [4], [5, 6, 7]], P("single_document", 3, drop_short_below=2), 0)
    assert toks(got) == [[2, 3, 0], [5, 6, 7]]


def test_single_document_without_threshold_keeps_an_empty_doc_as_all_pad():
    for kw in ({}, {"drop_short_below": 0}):
        s = L.pack([[]], P("single_document", 3, pad=5, **kw), 0)[0]
        assert s.tokens == [5, 5, 5] and s.mask == [0, 0, 0]


def test_single_document_all_dropped_is_an_error():
    assert kind_of(L.pack, [[1], [2]], P("single_document", 3, drop_short_below=2), 0) == "DroppedShort"


# ---------------------------------------------------------------------- errors
@pytest.mark.parametrize("strategy", ["concat_eos", "document_mask", "single_document"])
def test_empty_doc_list_and_zero_length_for_every_strategy(strategy):
    assert kind_of(L.pack, [], P(strategy, 4), 0) == "Empty"
    assert kind_of(L.pack, [], P(strategy, 4, drop_short_below=2), 0) == "Empty"
    assert kind_of(L.pack, [[1]], P(strategy, 0), 0) == "BadSequenceLength"
    assert kind_of(L.pack, [], P(strategy, 0), 0) == "BadSequenceLength"        # checked before emptiness


def test_unknown_strategy_name():
    assert kind_of(L.Packing, "x", 4, "zigzag") == "UnknownStrategy"


# ------------------------------------------------------------------------ json
def test_packing_json_round_trips_every_strategy_and_rejects_foreign_documents():
    for strategy in ("concat_eos", "document_mask", "single_document"):
        p = P(strategy, 16, eos=False, pad=3, drop_short_below=4)
        back = L.Packing.from_json(p.to_json())
        assert (back.strategy, back.sequence_length, back.eos_between_docs, back.pad_id, back.drop_short_below) == \
            (strategy, 16, False, 3, 4)
        d = json.loads(p.to_json())
        assert d["schema_id"] == "prometheus.packing" and d["schema_version"] == 1
    assert "drop_short_below" not in P().to_json()
    good = json.loads(P().to_json())
    for bad in (dict(good, schema_id="other"), dict(good, strategy="spiral")):
        with pytest.raises(native.NativeError):
            L.Packing.from_json(json.dumps(bad))
    with pytest.raises(native.NativeError):
        L.Packing.from_json("null")


def test_loader_state_json_envelope_round_trip_and_rejections():
    st = L.LoaderState()
    st.epoch, st.shard_offset, st.step, st.consumed_token_count, st.shuffle_seed = 2, 5, 9, 4096, 77
    d = json.loads(st.to_json())
    assert d["schema_id"] == "prometheus.loader_state" and d["schema_version"] == 1 and d["epoch"] == 2
    assert L.LoaderState.from_json(st.to_json()) == st
    with pytest.raises(native.NativeError):
        L.LoaderState.from_json(json.dumps(dict(d, schema_id="other")))
    with pytest.raises(native.NativeError):
        L.LoaderState.from_json("null")


# --------------------------------------------------------------------- shuffle
def test_shuffle_is_a_deterministic_permutation_that_depends_on_seed_and_epoch():
    assert L.shuffle_order(0, 1, 0) == [] and L.shuffle_order(1, 99, 3) == [0]
    for n in (2, 3, 17, 256):
        o = L.shuffle_order(n, 5, 0)
        assert sorted(o) == list(range(n)) and o == L.shuffle_order(n, 5, 0)
    base = L.shuffle_order(64, 5, 0)
    assert base != L.shuffle_order(64, 6, 0) and base != L.shuffle_order(64, 5, 1) and base != list(range(64))


# ---------------------------------------------------------------------- loader
def seqs(n, length=2):
    return [L.PackedSequence([i] * length, [1] * length) for i in range(n)]


def test_new_state_starts_at_origin_and_batches_follow_the_shuffle():
    ld = L.Loader(seqs(5), P(n=2), 3, "mix")
    st = ld.state()
    assert (st.epoch, st.shard_index, st.shard_offset, st.step, st.consumed_token_count) == (0, 0, 0, 0, 0)
    assert st.shuffle_seed == 3 and st.data_mix_hash == "mix"
    b = ld.next_batch(2)
    assert [t[0] for t in b.tokens] == L.shuffle_order(5, 3, 0)[:2] and len(b.mask) == 2
    assert (b.state.step, b.state.shard_offset, b.state.consumed_token_count) == (1, 2, 4)


def test_epoch_wrap_between_and_inside_batches():
    ld = L.Loader(seqs(3), P(n=2), 8, "m")
    first = [t[0] for t in ld.next_batch(3).tokens]
    assert first == L.shuffle_order(3, 8, 0) and ld.state().epoch in (0, 1)
    nxt = [t[0] for t in ld.next_batch(2).tokens]
    assert nxt == L.shuffle_order(3, 8, 1)[:2] and ld.state().epoch == 1
    big = L.Loader(seqs(3), P(n=2), 8, "m").next_batch(7)                 # wraps twice inside one batch
    want = L.shuffle_order(3, 8, 0) + L.shuffle_order(3, 8, 1) + L.shuffle_order(3, 8, 2)
    assert [t[0] for t in big.tokens] == want[:7] and big.state.epoch == 2 and big.state.shard_offset == 1


def test_two_loaders_with_the_same_seed_agree_and_from_state_resumes():
    a, b = L.Loader(seqs(9), P(n=2), 4, "m"), L.Loader(seqs(9), P(n=2), 4, "m")
    assert [a.next_batch(4).tokens for _ in range(3)] == [b.next_batch(4).tokens for _ in range(3)]
    saved = a.state()
    resumed = L.Loader.from_state(seqs(9), P(n=2), saved)
    assert resumed.next_batch(5).tokens == b.next_batch(5).tokens


def test_empty_corpus_is_exhausted_on_the_first_batch():
    assert kind_of(L.Loader([], P(n=2), 0, "").next_batch, 1) == "Exhausted"
    assert kind_of(L.Loader.from_state([], P(n=2), L.LoaderState()).next_batch, 1) == "Exhausted"
    assert kind_of(L.reconstruct, [], P(n=2), L.LoaderState(), 1) == "Exhausted"


# ----------------------------------------------------------------- reconstruct
@pytest.mark.parametrize("batch", [1, 2, 5])
def test_reconstruct_matches_every_step_and_after_a_wrap(batch):
    ld = L.Loader(seqs(7), P(n=2), 21, "m")
    for _ in range(8):                                                   # several epochs at batch 5
        before = ld.state()
        got = ld.next_batch(batch)
        again = L.reconstruct(seqs(7), P(n=2), before, batch)
        assert again.tokens == got.tokens and again.mask == got.mask and again.state == got.state


# -------------------------------------------------- second opinion on the packer
def _py_pack(docs, n, eos_between, pad, eos):
    stream, ids = [], []
    for i, d in enumerate(docs):
        stream += d
        ids += [i] * len(d)
        if eos_between and i + 1 < len(docs):
            stream.append(eos)
            ids.append(i)
    out = []
    for off in range(0, len(stream), n):
        chunk, cid = stream[off:off + n], ids[off:off + n]
        fill = n - len(chunk)
        out.append((chunk + [pad] * fill, [1] * len(chunk) + [0] * fill, cid + [0] * fill))
    return out


def test_packer_agrees_with_a_python_packer_on_random_docs():
    rng = random.Random(4)
    for _ in range(60):
        docs = [[rng.randrange(2, 50) for _ in range(rng.randrange(0, 9))] for _ in range(rng.randrange(1, 7))]
        n, eos_between = rng.randrange(1, 7), rng.random() < 0.5
        want = _py_pack(docs, n, eos_between, 0, 1)
        if not want:
            continue
        got = L.pack(docs, P("document_mask", n, eos_between), 1)
        assert [(s.tokens, s.mask, s.document_ids) for s in got] == want, (docs, n, eos_between)
