"""Property tests (hypothesis) of the spec layer: the native runtime against the Python definitions on generated
inputs — tokenizer longest-match, SplitMix64 draws, safetensors files."""
import json

import numpy as np
import torch
from hypothesis import given, settings, strategies as st

from fbamtrain_b200 import rng as pyrng
from fbamtrain_b200 import runtime as rt
from fbamtrain_b200.tokenizer import Tokenizer
from fbamtrain_b200.utils import safetensors_io as stio

ALPHABET = "ab\x1bé日\U0001F600\"\\\n "


@settings(max_examples=40, deadline=None)
@given(tokens=st.lists(st.text(alphabet=ALPHABET, min_size=1, max_size=4), min_size=1, max_size=12, unique=True),
       text=st.text(alphabet=ALPHABET + "z", max_size=60))
def test_native_and_python_tokenizers_agree(tmp_path_factory, tokens, text):
    path = str(tmp_path_factory.mktemp("tok") / "tok.txt")
    with open(path, "w", encoding="utf-8") as f:
        f.write("# FBAM_TOK v1.0\n")
        for t in tokens:
            f.write(json.dumps(t) + "\n")
    py, nat = Tokenizer.from_file(path), rt.NativeTokenizer(path)
    assert [nat.token(i) for i in range(len(nat))] == py.tokens
    got, want = nat.encode_longest_match(text), py.encode_longest_match(text)
    assert got == want
    # every emitted token is really at its start position and no longer token of the vocabulary starts there
    for tok_id, start in want:
        tok = py.tokens[tok_id]
        assert text[start:start + len(tok)] == tok
        assert not any(len(o) > len(tok) and text.startswith(o, start) for o in py.tokens)


@settings(max_examples=30, deadline=None)
@given(seed=st.integers(min_value=0, max_value=2 ** 64 - 1), low=st.integers(-1000, 1000),
       span=st.integers(1, 10 ** 6), n=st.integers(1, 50))
def test_native_and_python_splitmix_agree(seed, low, span, n):
    a, b = pyrng.SplitMix64(seed), rt.NativeSplitMix64(seed)
    for _ in range(n):
        assert a.randint(low, low + span) == b.randint(low, low + span)
    assert a.state == b.state


_DTYPES = [torch.float32, torch.float16, torch.bfloat16]


@settings(max_examples=25, deadline=None)
@given(shapes=st.lists(st.lists(st.integers(0, 5), min_size=0, max_size=3), min_size=1, max_size=5),
       dtype_ix=st.lists(st.integers(0, 2), min_size=5, max_size=5), seed=st.integers(0, 10 ** 6))
def test_safetensors_files_cross_read(tmp_path_factory, shapes, dtype_ix, seed):
    """Python writer → native reader → native writer → Python reader reproduces every tensor bit for bit, and the
    native file comparer finds no difference between the two files."""
    gen = torch.Generator().manual_seed(seed)
    tensors = {}
    for i, shape in enumerate(shapes):
        tensors[f"t/{i}"] = torch.randn(tuple(shape), generator=gen).to(_DTYPES[dtype_ix[i]])
    d = tmp_path_factory.mktemp("st")
    p_py, p_nat = str(d / "py.safetensors"), str(d / "nat.safetensors")
    stio.save_file(tensors, p_py)
    native_view = rt.st_read(p_py)
    assert set(native_view) == set(tensors)
    rt.st_write(p_nat, native_view)
    back = stio.load_file(p_nat)
    for k, v in tensors.items():
        assert back[k].dtype == v.dtype and tuple(back[k].shape) == tuple(v.shape)
        if v.numel():
            assert torch.equal(back[k].reshape(-1).view(torch.uint8), v.reshape(-1).view(torch.uint8))
    assert rt.tenscmp(p_py, p_nat, 0.0)[0] == 0


@settings(max_examples=30, deadline=None)
@given(shapes=st.lists(st.lists(st.integers(1, 7), min_size=1, max_size=3), min_size=1, max_size=8),
       kinds=st.lists(st.integers(0, 1), min_size=8, max_size=8), multiple=st.sampled_from([1, 2, 6, 12, 840]))
def test_flat_groups_pack_aligned_and_keep_values(shapes, kinds, multiple):
    """Packing parameters into flat buckets keeps their values, aliases them into the bucket, aligns every slot to
    256 bytes, pads the bucket to the shard multiple and leaves no two slots overlapping."""
    from fbamtrain_b200.utils.flat import ALIGN_BYTES, build_groups
    dts = [torch.float32, torch.bfloat16]
    named = [(f"p{i}", torch.nn.Parameter(torch.randn(tuple(s)).to(dts[kinds[i]]))) for i, s in enumerate(shapes)]
    before = {n: p.detach().clone() for n, p in named}
    groups = build_groups("scope", named, multiple)
    assert sum(len(g.named_params) for g in groups) == len(named)
    for g in groups:
        esize = torch.empty((), dtype=g.dtype).element_size()
        assert (g.numel * esize) % (ALIGN_BYTES * multiple) == 0
        spans = []
        for n, p in g.named_params:
            o = g.offsets[n]
            assert (o * esize) % ALIGN_BYTES == 0
            assert torch.equal(p.detach(), before[n])
            assert p.data_ptr() == g.data.data_ptr() + o * esize          # the parameter lives in the bucket
            assert p.grad.data_ptr() == g.grad.data_ptr() + o * esize
            spans.append((o, o + p.numel()))
        spans.sort()
        assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:])) and spans[-1][1] <= g.numel
        g.data.zero_()
        assert all(float(p.detach().float().abs().sum()) == 0.0 for _, p in g.named_params)


@settings(max_examples=60, deadline=None)
@given(tokens=st.lists(st.text(alphabet="abc", min_size=1, max_size=4), min_size=1, max_size=8, unique=True),
       keys=st.lists(st.text(alphabet="abcd", max_size=4), min_size=1, max_size=12))
def test_token_stream_consumption_equals_greedy_longest_match_over_frames(tokens, keys):
    """Keystrokes typed over several frames are consumed as the greedy longest-match tokenization of their
    concatenation; every token is paired with the frame on which its first keystroke was typed; keystrokes that
    start no token are skipped."""
    from fbamtrain_b200.data.frames import StreamTokenizationContext, consume_next_token
    from fbamtrain_b200.data.recording import ArrayRecording
    tok = Tokenizer(tokens)
    rec = ArrayRecording(np.zeros((len(keys), 1, 1, 3), dtype=np.uint32), keys)
    ctx = StreamTokenizationContext(rec, tok, 0)
    got = []
    while True:
        r = consume_next_token(ctx)
        if r is None:
            break
        got.append(r)
    text = "".join(keys)
    frame_of = [f for f, k in enumerate(keys) for _ in k]
    want, i = [], 0
    while i < len(text):
        best = max((t for t in tok.tokens if text.startswith(t, i)), key=len, default=None)
        if best is None:
            i += 1
            continue
        want.append((tok.tokens.index(best), frame_of[i]))
        i += len(best)
    assert got == want


@settings(max_examples=25, deadline=None)
@given(tokens=st.lists(st.text(alphabet="abcé", min_size=1, max_size=3), min_size=1, max_size=6, unique=True),
       keys=st.lists(st.text(alphabet="abcdé", max_size=3), min_size=3, max_size=20),
       seq=st.integers(1, 9), start_frac=st.floats(0, 1), seed=st.integers(0, 1000))
def test_native_batch_loader_equals_python_assembly(tmp_path_factory, tokens, keys, seq, start_frac, seed):
    """Raw recordings gathered by the native loader give the same cells and targets as the per-frame Python path
    (tokens paired with the frame of their first keystroke, code points clamped, exhausted streams zero-padded)."""
    from fbamtrain_b200.data.iterator import Batch
    from fbamtrain_b200.data.recording import ArrayRecording, RawRecording, write_raw_recording
    from fbamtrain_b200.train import build_batch_from_recordings
    rng = np.random.default_rng(seed)
    d = tmp_path_factory.mktemp("rec")
    rows, cols, max_cp, vocab = 2, 3, 50, 5
    recs, paths = [], []
    for r in range(2):
        ks = keys if r == 0 else keys[::-1]
        cells = rng.integers(0, 80, size=(len(ks), rows, cols, 3), dtype=np.uint32)
        path = str(d / f"r{r}.fbrec")
        write_raw_recording(path, cells, ks)
        raw = RawRecording(path)
        assert raw.total_frames() == len(ks) and raw.frame(1)[1] == ks[1]
        assert np.array_equal(raw.frame(len(ks) - 1)[0], cells[-1])
        recs.append(ArrayRecording(cells, ks))
        paths.append(path)
    tok = Tokenizer(tokens)
    start = int(start_frac * (len(keys) - 1))
    indices, starts = [0, 1, 0], [start, 0, len(keys) - 1]
    want_cells, want_targets = build_batch_from_recordings(Batch([recs[i] for i in indices], indices, starts), tok,
                                                           seq, rows, cols, vocab, max_cp)
    loader = rt.NativeBatchLoader(paths, tok.tokens, max_cp, vocab, threads=3)
    got_cells = torch.full((3, seq, rows * cols, 3), -7, dtype=torch.int32)
    got_targets = torch.full((3, seq), -7, dtype=torch.int64)
    loader.fill(indices, starts, seq, got_cells, got_targets)
    loader.close()
    assert torch.equal(got_targets, want_targets)
    assert torch.equal(got_cells, want_cells)
