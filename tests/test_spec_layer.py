import json
import os

import numpy as np
import pytest
from conftest import reference_path
import torch

from fbamtrain_b200.data import (ArrayRecording, DatasetCursorCommitter, DatasetCursorSnapshot,
                                 RecordingDatasetIterator, StreamTokenizationContext, SyntheticBatchSource,
                                 SyntheticRecording, consume_next_token, prepare_cell_states)
from fbamtrain_b200.data.iterator import DatasetIteratorState
from fbamtrain_b200.rng import SplitMix64
from fbamtrain_b200.tokenizer import Tokenizer
from fbamtrain_b200.utils import safetensors_io as st
from fbamtrain_b200.utils.testing import assert_similar


def test_splitmix64_known_vectors():
    # First outputs of SplitMix64 seeded with 0 and with 1234567 (published test vectors of the algorithm).
    r = SplitMix64(0)
    assert [r.randu64() for _ in range(3)] == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F]
    r = SplitMix64(1234567)
    assert [r.randu64() for _ in range(2)] == [6457827717110365317, 3203168211198807973]
    r = SplitMix64(42)
    v = [r.randint(3, 10) for _ in range(100)]
    assert min(v) >= 3 and max(v) < 10
    with pytest.raises(ValueError):
        r.randint(5, 5)


def test_tokenizer_sort_trie_and_longest_match(tmp_path):
    lines = ["# FBAM_TOK v1.0\n", '"a"\n', '"ab"\n', '"\\u001b[A"\n', '"b"\n', "\n", '"abc"\n']
    p = tmp_path / "tok.txt"
    p.write_text("".join(lines), encoding="utf-8")
    tok = Tokenizer.from_file(str(p))
    # stable sort by length, longest first: "\x1b[A", "abc" (len 3), "ab", then "a", "b" in file order
    assert tok.tokens == ["\x1b[A", "abc", "ab", "a", "b"]
    h = tok.new_handle()
    h.add_char(ord("a"))
    assert h.current_token_id() == 3 and h.has_continuation()
    h.add_char(ord("b"))
    assert h.current_token_id() == 2
    h.add_char(ord("x"))
    assert h.is_dead() and h.current_token_id() is None
    h.reset()
    assert not h.is_dead()
    assert [t for t, _ in tok.encode_longest_match("abcabz\x1b[Ab")] == [1, 2, 0, 4]
    with pytest.raises(ValueError, match="header"):
        Tokenizer.from_lines(["# WRONG\n"])
    with pytest.raises(ValueError, match="line 2"):
        Tokenizer.from_lines(["# FBAM_TOK v1.0\n", "not json\n"])


def test_reference_tokenizer_file_if_present():
    path = reference_path("working_dir", "tokenizer.txt")
    if not os.path.exists(path):
        pytest.skip("reference tree not mounted")
    tok = Tokenizer.from_file(path)
    assert len(tok) == 20351
    lens = [len(t) for t in tok.tokens]
    assert lens == sorted(lens, reverse=True)


def test_token_stream_consumption_pairs_token_with_start_frame():
    tok = Tokenizer(["abc", "ab", "a", "b", "c"])
    cells = np.zeros((5, 2, 3, 3), dtype=np.uint32)
    rec = ArrayRecording(cells, ["a", "b", "", "ca", "z"])
    ctx = StreamTokenizationContext(rec, tok, 0)
    out = []
    while True:
        r = consume_next_token(ctx)
        if r is None:
            break
        out.append(r)
    # "a","b","c" spread over frames 0,1,3 form the longest token "abc" which started on frame 0
    assert out == [(0, 0), (2, 3)]


def test_prepare_cell_states_clamps_codepoints():
    frame = np.array([[[300, 0x112233, 0xFF445566], [5, 1, 2]]], dtype=np.uint32)
    cs = prepare_cell_states(frame, 256)
    assert cs.tolist() == [[255, 0x112233, 0x445566], [5, 1, 2]]


def test_synthetic_recording_resamples_five_percent():
    rec = SyntheticRecording(24, 80, 6, seed=0, cell_vocab=256)
    a, _ = rec.frame(0)
    b, _ = rec.frame(1)
    changed = (a.reshape(-1, 3) != b.reshape(-1, 3)).any(-1).sum()
    assert 0 < changed <= round(0.05 * 24 * 80)
    src = SyntheticBatchSource(8, 16, 512, 64, seed=3, pin=False)
    cells, tg = src.next_batch(2, 5)
    assert cells.shape == (2, 5, 128, 3) and tg.shape == (2, 5)
    assert int(cells[..., 0].max()) < 512 and int(tg.max()) < 64
    frac = (cells[:, 1:, :, 0] != cells[:, :-1, :, 0]).float().mean()
    assert frac <= 0.05 + 1e-6


def _recs(n=3):
    return [SyntheticRecording(4, 6, 40 + 7 * i, seed=i) for i in range(n)]


def test_iterator_sampling_matches_rng_contract_and_restores():
    it = RecordingDatasetIterator(None, batch_size=4, sequence_length=16, seed=99, recordings=_recs())
    rng = SplitMix64(99)
    totals = [40, 47, 54]
    b1 = it.next_batch()
    exp_idx, exp_start = [], []
    for _ in range(4):
        i = rng.randint(0, 3)
        exp_idx.append(i)
        exp_start.append(rng.randint(0, max(0, totals[i] - 16) + 1))
    assert b1.indices == exp_idx and b1.start_positions == exp_start
    state = it.checkpoint()              # describes the *prepared* (next) batch
    cursor = it.cursor_checkpoint()      # RNG after the batch handed out
    b2 = it.next_batch()
    assert state.prepared_indices == b2.indices and state.prepared_start_positions == b2.start_positions
    b3 = it.next_batch()
    it.restore(state)
    r2 = it.next_batch()
    r3 = it.next_batch()
    assert (r2.indices, r2.start_positions) == (b2.indices, b2.start_positions)
    assert (r3.indices, r3.start_positions) == (b3.indices, b3.start_positions)
    it.restore(DatasetIteratorState(rng_state=cursor.rng_state, batch_size=4))  # RNG-only form
    c2 = it.next_batch()
    assert (c2.indices, c2.start_positions) == (b2.indices, b2.start_positions)
    with pytest.raises(RuntimeError, match="batch size"):
        it.restore(DatasetIteratorState(rng_state=1, batch_size=5))
    it.close()


def test_iterator_reads_directory_sorted(tmp_path):
    for i, name in enumerate(["b", "a", "c"]):
        r = SyntheticRecording(2, 3, 10, seed=i)
        ArrayRecording(np.stack([r.frame(t)[0] for t in range(10)]), [r.frame(t)[1] for t in range(10)]).save(
            str(tmp_path / f"{name}.fbrec.npz"))
    it = RecordingDatasetIterator(str(tmp_path), 2, 4, seed=1)
    assert [os.path.basename(p) for p in it._paths] == ["a.fbrec.npz", "b.fbrec.npz", "c.fbrec.npz"]
    it.close()
    with pytest.raises(RuntimeError):
        RecordingDatasetIterator(str(tmp_path / "nope"), 2, 4, seed=1)


def test_cursor_durable_roundtrip(tmp_path):
    path = str(tmp_path / "ck" / "cursor.json")
    assert DatasetCursorCommitter.load(path) is None
    c = DatasetCursorCommitter(path)
    for s in range(20):
        c.commit(DatasetCursorSnapshot(s, 2 ** 63 + s, 8, 1024))
    assert c.flush()
    c.close()
    snap = DatasetCursorCommitter.load(path)
    assert snap == DatasetCursorSnapshot(19, 2 ** 63 + 19, 8, 1024)
    d = json.load(open(path))
    assert d["version"] == 1 and set(d) == {"version", "step_count", "rng_state", "batch_size", "sequence_length"}
    assert not os.path.exists(path + ".tmp")


def test_safetensors_roundtrip_and_validation(tmp_path):
    tensors = {"a": torch.randn(3, 4), "b": torch.randn(5).to(torch.bfloat16), "c": torch.randn(2, 2).half(),
               "u64": torch.tensor([2 ** 63 + 1], dtype=torch.uint64), "u32": torch.tensor([1, 2], dtype=torch.uint32),
               "empty": torch.zeros(0, dtype=torch.uint32)}
    p = str(tmp_path / "x.safetensors")
    st.save_file(tensors, p)
    back = st.load_file(p)
    assert set(back) == set(tensors)
    for k in tensors:
        assert back[k].dtype == tensors[k].dtype and back[k].shape == tensors[k].shape
        assert torch.equal(back[k].view(torch.uint8), tensors[k].view(torch.uint8))
    header, _ = st.read_header(p)
    assert header["u64"]["dtype"] == "U64" and header["b"]["dtype"] == "BF16"
    with pytest.raises(ValueError):
        st.load_inplace(p, {"a": torch.zeros(4, 3)})
    dst = {"a": torch.zeros(3, 4)}
    st.load_inplace(p, dst)
    assert torch.equal(dst["a"], tensors["a"])


def test_assert_similar_rules():
    e = torch.tensor([1.0, 2.0]).bfloat16()
    a = torch.tensor([1.0078125, 2.0]).bfloat16()  # one bf16 ulp above 1.0
    assert_similar(e, a, 1e-6)
    with pytest.raises(AssertionError):
        assert_similar(e.float(), a.float(), 1e-6)
    with pytest.raises(AssertionError, match="non-finite"):
        assert_similar(torch.tensor([float("nan")]), torch.tensor([0.0]), 1.0)
    with pytest.raises(AssertionError, match="shape"):
        assert_similar(torch.zeros(2), torch.zeros(3), 1.0)


def test_flop_accounting_separates_recomputation():
    from fbamtrain_b200.utils import flops
    flops.reset()
    flops.add(10.0)
    with flops.not_useful():
        flops.add(5.0)
        with flops.not_useful():
            flops.add(1.0)
    flops.add(2.0)
    assert flops.snapshot() == (18.0, 12.0)
    flops.reset()
    assert flops.snapshot() == (0.0, 0.0)


def test_backend_preference_environment(monkeypatch):
    import torch
    from fbamtrain_b200.ops import dispatch
    monkeypatch.setenv("FBAMTRAIN_PREFER_MHA_BACKEND", "torch")
    dispatch._read_preferences()
    assert dispatch._prefer == {"gemm": "native", "conv2d": "native", "mha": "torch"}
    q = torch.randn(1, 4, 2, 8)
    dispatch.attention(q, q, q, True)
    assert dispatch.last_backend("mha") == "torch"           # CPU tensors never take the native path
    monkeypatch.setenv("FBAMTRAIN_PREFER_GEMM_BACKEND", "cutlass")
    with pytest.raises(ValueError, match="GEMM_BACKEND"):
        dispatch._read_preferences()
    monkeypatch.delenv("FBAMTRAIN_PREFER_GEMM_BACKEND")
    monkeypatch.delenv("FBAMTRAIN_PREFER_MHA_BACKEND")
    dispatch._read_preferences()


def test_tuning_table_parse_lookup_and_recording(tmp_path, monkeypatch):
    import json
    from fbamtrain_b200.ops import tuning
    key = tuning.gemm_key(8192, 4096, 1024, False, True)
    assert key == "gemm m8192 n4096 k1024 NT"
    ckey = tuning.conv_key(1024, 24, 80, 128, 256, 9, 2, 1)
    doc = {"device": "x", "entries": {key: {"best": {"bm": 256, "bn": 128, "two_cta": False}, "ms": 0.1},
                                      ckey: {"best": {"tile_rows": 128, "two_cta": False}, "ms": 0.2}}}
    path = tmp_path / "tuning.json"
    path.write_text(json.dumps(doc))
    assert tuning.lookup(key) is None                                  # no table configured
    monkeypatch.setenv("FBAMTRAIN_TUNING_FILE", str(path))
    assert tuning.lookup(key) == {"bm": 256, "bn": 128, "two_cta": False}
    assert tuning.lookup(ckey) == {"tile_rows": 128, "two_cta": False}
    assert tuning.lookup("gemm m1 n1 k1 NN") is None
    with tuning.recording() as seen:
        tuning.lookup(key, {"m": 8192})
        tuning.lookup(key, {"m": 1})                                   # first sighting wins
        tuning.lookup("gemm m2 n2 k2 NN", {"m": 2})
    assert seen == {key: {"m": 8192}, "gemm m2 n2 k2 NN": {"m": 2}}
    monkeypatch.delenv("FBAMTRAIN_TUNING_FILE")
    assert tuning.lookup(key) is None
    tuning.set_table({key: {"bm": 128}})
    try:
        assert tuning.lookup(key) == {"bm": 128}
    finally:
        tuning.set_table(None)
    for bad in ({"entries": {key: {"best": {"bm": 100}}}}, {"entries": {key: {"best": {"tile_rows": 128}}}},
                {"entries": {key: {"best": {"two_cta": 1}}}}, {"entries": {"lstm x": {"best": {}}}}, {"entries": {key: {}}},
                {}):
        with pytest.raises(ValueError):
            tuning.parse(bad)
    cands = tuning.gemm_candidates(8192, 4096)
    assert {"bm": 256, "bn": 256, "two_cta": True} in cands and {"bm": 128, "bn": 128, "two_cta": False} in cands
    assert all(not c["two_cta"] for c in tuning.gemm_candidates(8192, 64))
    assert all(c.get("bn", 0) <= 128 for c in tuning.conv_candidates(64))
    for c in cands + tuning.conv_candidates(512):
        tuning._validate(key if "bm" in c else ckey, c)                 # every candidate is a legal table entry


def test_step_plan_records_launches_phases_and_flops():
    import threading
    from fbamtrain_b200.ops import native as nv
    from fbamtrain_b200.utils import flops, plan
    from fbamtrain_b200.utils.nvtx import gputx_range
    nv.check(0, "fbam_before")                                         # outside a recording: no effect
    with plan.record() as p:
        with gputx_range("fbamtrain::frame_head_fwd"):
            nv.check(0, "fbam_gemm")
            flops.add(2e9)
            with flops.not_useful():
                nv.check(0, "fbam_conv")
                flops.add(1e9)

        def backward_thread():
            nv.check(0, "fbam_gemm")
            flops.add(4e9)
        t = threading.Thread(target=backward_thread)
        t.start()
        t.join()
        nv.check(0, "fbam_adamw")
        with pytest.raises(RuntimeError):
            with plan.record():
                pass
    assert plan.active() is None
    assert [(e.name, e.phase, e.backward, e.flops, e.useful_flops) for e in p.entries] == [
        ("fbam_gemm", "fbamtrain::frame_head_fwd", False, 2e9, 2e9),
        ("fbam_conv", "fbamtrain::frame_head_fwd", False, 1e9, 0.0),
        ("fbam_gemm", "", True, 4e9, 4e9),
        ("fbam_adamw", "", False, 0.0, 0.0)]
    assert p.total_flops() == 7e9 and p.total_useful_flops() == 6e9
    assert p.by("name")["fbam_gemm"] == (2, 6e9)
    text = p.listing()
    assert text.startswith("# 4 launches") and "(recompute)" in text and "fbamtrain::frame_head_fwd" in text


def test_kernel_library_layout_matches_the_binding():
    """Loading the kernel library compares the compiled layout of its parameter struct with the ctypes mirror."""
    from fbamtrain_b200.ops import native as nv
    if not nv.available():
        pytest.skip("kernel library not built")
    nv.lib()                                            # raises on a mismatch
    got = (nv.C.c_longlong * 8)()
    nv.lib().fbam_gemm_params_layout(got)
    assert got[0] == nv.C.sizeof(nv.GemmParams) and got[7] == nv.C.sizeof(nv.ConvGeom)


def test_prefetching_source_keeps_order_and_reports_errors():
    from fbamtrain_b200.data import PrefetchingSource, SyntheticBatchSource
    direct = SyntheticBatchSource(8, 16, 256, 32, seed=4, pin=False)
    want = [direct.next_batch(2, 8) for _ in range(4)]
    pre = PrefetchingSource(SyntheticBatchSource(8, 16, 256, 32, seed=4, pin=False), 2, 8)
    got = [pre.next_batch(2, 8) for _ in range(4)]
    pre.close()
    for (c0, t0), (c1, t1) in zip(want, got):
        assert torch.equal(c0, c1) and torch.equal(t0, t1)
    with pytest.raises(ValueError):
        pre.next_batch(3, 8)

    class Broken:
        def next_batch(self, batch, seq):
            raise OSError("no data")
    bad = PrefetchingSource(Broken(), 1, 1)
    with pytest.raises(OSError, match="no data"):
        bad.next_batch(1, 1)
    bad.close()


def test_launch_rules_for_split_k_and_fused_parity_classes():
    """Pure launch rules (no GPU): which weight gradients are split over K, and when the four parity classes of a
    strided data gradient share one launch."""
    from fbamtrain_b200.ops import native_ops as no
    # small output, long K: divided so that the tiles fill the machine; large outputs and short K are left alone
    assert no.weight_grad_splits(1024, 1024, 8192) == 8
    assert no.weight_grad_splits(3072, 1024, 8192) == 3
    assert no.weight_grad_splits(4096, 4096, 8192) == 0
    assert no.weight_grad_splits(1024, 1024, 2048) == 0
    taps = {1: [(0, 0)], 2: [(0, 0), (0, 1)], 4: [(0, 0), (0, 1), (1, 0), (1, 1)]}
    parts = [(taps[1], None, (12, 40), (0, 0)), (taps[2], None, (12, 40), (0, 1)), (taps[2], None, (12, 40), (1, 0)),
             (taps[4], None, (12, 40), (1, 1))]
    assert no._fuse_dgrad_classes(parts, 1024, 256, 2)                     # the benchmark model's second layer
    assert not no._fuse_dgrad_classes(parts, 1024, 128, 2)                 # too few output channels for CTA pairs
    assert not no._fuse_dgrad_classes(parts, 16, 256, 2)                   # too few tiles
    odd = [(taps[1], None, (12, 41), (0, 0))] + parts[1:]
    assert not no._fuse_dgrad_classes(odd, 1024, 256, 2)                   # classes on different grids
