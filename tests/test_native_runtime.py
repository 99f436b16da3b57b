"""The C++ host runtime against the Python implementations of the same components."""
import json
import os
import socket
import threading

import numpy as np
import pytest
from conftest import reference_path
import torch

from fbamtrain_b200 import runtime as rt
from fbamtrain_b200.rng import SplitMix64
from fbamtrain_b200.tokenizer import Tokenizer
from fbamtrain_b200.utils import safetensors_io as st


def test_native_rng_matches_python_and_draws_batches():
    a, b = rt.NativeSplitMix64(42), SplitMix64(42)
    assert [a.randu64() for _ in range(5)] == [b.randu64() for _ in range(5)]
    assert [a.randint(3, 1000) for _ in range(5)] == [b.randint(3, 1000) for _ in range(5)]
    assert a.state == b.state
    totals = [40, 47, 54]
    idx, start = a.draw_batch(totals, 16, 6)
    exp_i, exp_s = [], []
    for _ in range(6):
        i = b.randint(0, 3)
        exp_i.append(i)
        exp_s.append(b.randint(0, max(0, totals[i] - 16) + 1))
    assert (idx, start) == (exp_i, exp_s) and a.state == b.state


def test_native_tokenizer_matches_python(tmp_path):
    toks = ["a", "ab", "abc", "\x1b[A", "é", "日本", "b", "\U0001F600x", "\"q\\", "\n"]
    path = str(tmp_path / "tok.txt")
    with open(path, "w", encoding="utf-8") as f:
        f.write("# FBAM_TOK v1.0\n")
        for t in toks:
            f.write(json.dumps(t) + "\n")        # ensure_ascii: exercises \\uXXXX and surrogate pairs
        f.write("\n")
    py, nat = Tokenizer.from_file(path), rt.NativeTokenizer(path)
    assert len(nat) == len(py)
    assert [nat.token(i) for i in range(len(nat))] == py.tokens
    text = "abcabé日本zz\x1b[Ab\U0001F600x\"q\\\n"
    assert nat.encode_longest_match(text) == py.encode_longest_match(text)
    with open(path, "w") as f:
        f.write("# nope\n")
    with pytest.raises(ValueError, match="header"):
        rt.NativeTokenizer(path)


def test_reference_tokenizer_file_natively_if_present():
    path = reference_path("working_dir", "tokenizer.txt")
    if not os.path.exists(path):
        pytest.skip("reference tree not mounted")
    nat, py = rt.NativeTokenizer(path), Tokenizer.from_file(path)
    assert len(nat) == len(py) == 20351
    for i in (0, 1, 100, 5000, 20350):
        assert nat.token(i) == py.tokens[i]


def test_native_safetensors_interop_and_tenscmp(tmp_path):
    tensors = {"w": torch.randn(5, 7), "h": torch.randn(3, 2).bfloat16(), "s": torch.tensor([9], dtype=torch.uint64),
               "e": torch.zeros(0, dtype=torch.uint32)}
    p1 = str(tmp_path / "py.safetensors")
    st.save_file(tensors, p1)
    got = rt.st_read(p1)                                    # native reader on a Python-written file
    assert set(got) == set(tensors)
    assert got["w"][0] == "F32" and np.array_equal(got["w"][1], tensors["w"].numpy())
    assert got["h"][0] == "BF16" and np.array_equal(got["h"][1], tensors["h"].view(torch.int16).numpy().view(np.uint16))
    p2 = str(tmp_path / "native.safetensors")
    rt.st_write(p2, got)                                    # native writer, Python reader
    back = st.load_file(p2)
    for k, v in tensors.items():
        assert back[k].dtype == v.dtype and torch.equal(back[k].view(torch.uint8), v.view(torch.uint8))
    bad, report = rt.tenscmp(p1, p2, 0.0)
    assert bad == 0 and report == ""
    tensors["w"] = tensors["w"] + 0.5
    del tensors["e"]
    st.save_file(tensors, p1)
    bad, report = rt.tenscmp(p1, p2, 0.3)
    assert bad == 2 and "w: max |a-b|" in report and "missing in first file" in report
    assert rt.tenscmp(p1, p2, 0.6)[0] == 1


def test_native_cursor_writer(tmp_path):
    path = str(tmp_path / "c" / "cursor.json")
    c = rt.NativeCursorCommitter(path)
    for s in range(50):
        c.commit(s, 2 ** 63 + s, 8, 1024)
    assert c.flush()
    c.close()
    d = json.load(open(path))
    assert d == {"version": 1, "step_count": 49, "rng_state": 2 ** 63 + 49, "batch_size": 8, "sequence_length": 1024}
    from fbamtrain_b200.data import DatasetCursorCommitter
    assert DatasetCursorCommitter.load(path).step_count == 49          # the Python loader reads the native file


def test_native_rendezvous_and_interop_with_python():
    from fbamtrain_b200.parallel import rendezvous as rdv
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    blob = bytes(range(128))
    out = {}
    th = threading.Thread(target=lambda: rt.rdv_serve("127.0.0.1", port, 3, blob, 20))
    th.start()
    t2 = threading.Thread(target=lambda: out.__setitem__("py", rdv.fetch_blob("127.0.0.1", port, 2)))
    t2.start()
    out["native"] = rt.rdv_fetch("127.0.0.1", port, 1)
    t2.join(20)
    th.join(20)
    assert out["native"] == blob and out["py"] == blob


def test_native_membership_master_protocol():
    """Wire-level check of the native membership service: connect, heartbeat, a two-peer vote, a step gate that
    reports a newcomer, leave."""
    import json
    import socket
    import threading
    from fbamtrain_b200.parallel.ftccl import NativeMembershipMaster
    master = NativeMembershipMaster(heartbeat_timeout_s=5.0).start()
    try:
        def rpc(sock, obj):
            sock.sendall((json.dumps(obj) + "\n").encode())
            buf = b""
            while not buf.endswith(b"\n"):
                buf += sock.recv(4096)
            return json.loads(buf)

        a = socket.create_connection(("127.0.0.1", master.port))
        b = socket.create_connection(("127.0.0.1", master.port))
        ua = rpc(a, {"op": "connect", "peer_group": 0, "ip": "127.0.0.1"})["uid"]
        ub = rpc(b, {"op": "connect", "peer_group": 1, "ip": "127.0.0.1"})["uid"]
        assert rpc(a, {"op": "heartbeat"}) == {"epoch": 0, "pending": 2, "world": 0, "ok": True}
        out = {}
        t = threading.Thread(target=lambda: out.update(b=rpc(b, {"op": "vote", "free_port": 7002, "min_world": 2,
                                                                 "timeout": 20})))
        t.start()
        ra = rpc(a, {"op": "vote", "free_port": 7001, "min_world": 2, "timeout": 20})
        t.join(30)
        assert ra["ok"] and out["b"]["ok"] and ra["epoch"] == out["b"]["epoch"] == 1 and ra["world"] == 2
        assert ra["ranks"] == {str(ua): 0, str(ub): 1} and ra["store"] == {"ip": "127.0.0.1", "port": 7001}
        assert ra["groups"] == {str(ua): 0, str(ub): 1}
        assert master.snapshot() == {"epoch": 1, "accepted": [ua, ub], "pending": []}
        # both members reach the gate of step 3: aligned
        t = threading.Thread(target=lambda: out.update(g=rpc(b, {"op": "gate", "step": 3, "epoch": 1, "world": 2,
                                                                 "timeout": 10})))
        t.start()
        ga = rpc(a, {"op": "gate", "step": 3, "epoch": 1, "world": 2, "timeout": 10})
        t.join(20)
        assert ga["aligned"] and out["g"]["aligned"]
        # a newcomer waits for admission: the gate sends the members to a new vote instead
        c = socket.create_connection(("127.0.0.1", master.port))
        rpc(c, {"op": "connect", "peer_group": 0, "ip": "127.0.0.1"})
        ga = rpc(a, {"op": "gate", "step": 4, "epoch": 1, "world": 2, "timeout": 10})
        assert ga["ok"] and not ga["aligned"] and ga["pending"] == 1
        assert rpc(b, {"op": "leave"}) == {"ok": True}
        assert rpc(a, {"op": "heartbeat"})["world"] == 1
        for s in (a, b, c):
            s.close()
    finally:
        master.interrupt()


def test_native_synthetic_generator_is_reproducible_and_follows_the_recipe():
    """The threaded generator: the same ``(seed, call)`` gives the same batch whatever the thread count, about
    ``resample`` of the cells change between consecutive frames, and every field stays inside its range."""
    from fbamtrain_b200.data import SyntheticBatchSource
    from fbamtrain_b200.data.synthetic import ANSI_PALETTE
    n, k = 8 * 16, 6
    outs = []
    for threads in (1, 3):
        cells = torch.empty((3, 12, n, 3), dtype=torch.int32)
        tg = torch.empty((3, 12), dtype=torch.int64)
        rt.synth_fill(5, 2, n, 300, 16, k, 40, ANSI_PALETTE, cells, tg, threads=threads)
        outs.append((cells, tg))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    cells, tg = outs[0]
    u = cells.numpy().view(np.uint32)
    assert u[..., 0].max() < 300 and 0 <= tg.min() and tg.max() < 40
    assert set(np.unique(u[..., 1])) <= set(np.asarray(ANSI_PALETTE, dtype=np.uint32))
    changed = (u[:, 1:] != u[:, :-1]).any(-1).sum(-1)           # cells that differ between consecutive frames
    assert changed.max() <= k and changed.mean() > k / 2
    src = SyntheticBatchSource(8, 16, 300, 40, seed=5, pin=False, native=True)
    a0, a1 = src.next_batch(3, 12), src.next_batch(3, 12)
    assert not torch.equal(a0[0], a1[0])                        # the call number advances the stream
    again = SyntheticBatchSource(8, 16, 300, 40, seed=5, pin=False, native=True)
    assert torch.equal(again.next_batch(3, 12)[0], a0[0])
