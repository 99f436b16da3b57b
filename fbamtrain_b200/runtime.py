"""ctypes binding of the native host runtime (``lib/libfbam_runtime.so``, sources in ``csrc/runtime``).

The native library holds the pieces the reference implements in C++ outside its tensor library: SplitMix64
dataset RNG and batch drawing, the ``FBAM_TOK v1.0`` trie tokenizer, a safetensors reader / durable writer /
file comparer, the durable dataset-cursor writer thread, the TCP rendezvous, and the membership master of the
fault-tolerant collective layer.  The pure-Python modules
(``rng``, ``tokenizer``, ``utils.safetensors_io``, ``data.cursor``, ``parallel.rendezvous``) implement the same
behaviour and are used as oracles in the tests; callers may use either.  (reference: ``src/random.cpp``,
``src/tokenizer.cpp``, ``tensorlib/src/safe_tensors.cpp``, ``src/dataset_cursor.cpp``, ``src/rdvz.cpp``,
``src/dataset_iterator.cpp``, ``src/tenscmp.cpp:12-79``.)
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, List, Optional, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libfbam_runtime.so")
_lib: Optional[C.CDLL] = None


class RuntimeError_(RuntimeError):
    pass


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not available():
            from . import build
            build.build_runtime()
        L = C.CDLL(LIB_PATH)
        L.fbam_rt_last_error.restype = C.c_char_p
        L.fbam_tok_from_list.restype = C.c_void_p
        L.fbam_tok_from_list.argtypes = [C.c_void_p, C.c_int64]
        L.fbam_tok_free.argtypes = [C.c_void_p]
        L.fbam_synth_fill.argtypes = [C.c_uint64, C.c_uint64, C.c_int64, C.c_int64, C.c_int64, C.c_uint32, C.c_uint32,
                                      C.c_int64, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        L.fbam_tok_max_len.restype = C.c_int64
        L.fbam_tok_max_len.argtypes = [C.c_void_p]
        L.fbam_loader_open.restype = C.c_void_p
        L.fbam_loader_open.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_uint32, C.c_int64, C.c_int]
        L.fbam_loader_close.argtypes = [C.c_void_p]
        L.fbam_loader_frames.restype = C.c_int64
        L.fbam_loader_frames.argtypes = [C.c_void_p, C.c_int64]
        L.fbam_loader_rows.argtypes = [C.c_void_p]
        L.fbam_loader_cols.argtypes = [C.c_void_p]
        L.fbam_loader_fill.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]
        L.fbam_master_start.restype = C.c_void_p
        L.fbam_master_start.argtypes = [C.c_char_p, C.c_int, C.c_double, C.POINTER(C.c_int)]
        L.fbam_master_stop.argtypes = [C.c_void_p]
        L.fbam_master_snapshot.restype = C.c_int
        L.fbam_master_snapshot.argtypes = [C.c_void_p, C.c_char_p, C.c_int]
        L.fbam_splitmix_next.restype = C.c_uint64
        L.fbam_splitmix_next.argtypes = [C.POINTER(C.c_uint64)]
        L.fbam_splitmix_randint.restype = C.c_int64
        L.fbam_splitmix_randint.argtypes = [C.POINTER(C.c_uint64), C.c_int64, C.c_int64]
        L.fbam_dataset_draw.argtypes = [C.POINTER(C.c_uint64), C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p,
                                        C.c_void_p]
        L.fbam_tok_load.restype = C.c_void_p
        L.fbam_tok_load.argtypes = [C.c_char_p]
        L.fbam_tok_free.argtypes = [C.c_void_p]
        L.fbam_tok_size.restype = C.c_int64
        L.fbam_tok_size.argtypes = [C.c_void_p]
        L.fbam_tok_token.restype = C.c_int64
        L.fbam_tok_token.argtypes = [C.c_void_p, C.c_int64, C.c_char_p, C.c_int64]
        L.fbam_tok_encode.restype = C.c_int64
        L.fbam_tok_encode.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64]
        L.fbam_st_open.restype = C.c_void_p
        L.fbam_st_open.argtypes = [C.c_char_p]
        L.fbam_st_close.argtypes = [C.c_void_p]
        for name in ("count", "ndim", "dim", "nbytes"):
            getattr(L, "fbam_st_" + name).restype = C.c_int64
        L.fbam_st_count.argtypes = [C.c_void_p]
        L.fbam_st_ndim.argtypes = [C.c_void_p, C.c_int64]
        L.fbam_st_dim.argtypes = [C.c_void_p, C.c_int64, C.c_int64]
        L.fbam_st_nbytes.argtypes = [C.c_void_p, C.c_int64]
        L.fbam_st_name.restype = C.c_char_p
        L.fbam_st_name.argtypes = [C.c_void_p, C.c_int64]
        L.fbam_st_dtype.restype = C.c_char_p
        L.fbam_st_dtype.argtypes = [C.c_void_p, C.c_int64]
        L.fbam_st_read.argtypes = [C.c_void_p, C.c_int64, C.c_void_p]
        L.fbam_tenscmp.restype = C.c_int64
        L.fbam_tenscmp.argtypes = [C.c_char_p, C.c_char_p, C.c_double, C.c_char_p, C.c_int64]
        L.fbam_cursor_create.restype = C.c_void_p
        L.fbam_cursor_create.argtypes = [C.c_char_p]
        L.fbam_cursor_commit.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64]
        L.fbam_cursor_flush.argtypes = [C.c_void_p, C.c_int]
        L.fbam_cursor_destroy.argtypes = [C.c_void_p]
        L.fbam_rdv_serve.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_char_p, C.c_int]
        L.fbam_rdv_fetch.argtypes = [C.c_char_p, C.c_int, C.c_uint32, C.c_char_p, C.c_int]
        _lib = L
    return _lib


def _err() -> str:
    return (lib().fbam_rt_last_error() or b"").decode("utf-8", "replace")


# -- RNG ---------------------------------------------------------------------------------------
class NativeSplitMix64:
    def __init__(self, seed: int = 0):
        self._state = C.c_uint64(seed & ((1 << 64) - 1))

    @property
    def state(self) -> int:
        return int(self._state.value)

    @state.setter
    def state(self, v: int) -> None:
        self._state.value = v & ((1 << 64) - 1)

    def randu64(self) -> int:
        return int(lib().fbam_splitmix_next(C.byref(self._state)))

    def randint(self, low: int, high: int) -> int:
        if high <= low:
            raise ValueError("high must be > low")
        return int(lib().fbam_splitmix_randint(C.byref(self._state), low, high))

    def draw_batch(self, total_frames: List[int], seq_len: int, batch: int) -> Tuple[List[int], List[int]]:
        tf = np.asarray(total_frames, dtype=np.int64)
        idx = np.empty(batch, dtype=np.uint32)
        start = np.empty(batch, dtype=np.uint64)
        lib().fbam_dataset_draw(C.byref(self._state), tf.ctypes.data, len(tf), seq_len, batch, idx.ctypes.data,
                                start.ctypes.data)
        return [int(i) for i in idx], [int(s) for s in start]


# -- tokenizer -----------------------------------------------------------------------------------
class NativeTokenizer:
    def __init__(self, path: str):
        self._h = lib().fbam_tok_load(path.encode())
        if not self._h:
            raise ValueError(_err())

    def __len__(self) -> int:
        return int(lib().fbam_tok_size(self._h))

    def token(self, idx: int) -> str:
        n = lib().fbam_tok_token(self._h, idx, None, 0)
        buf = C.create_string_buffer(int(n) + 1)
        lib().fbam_tok_token(self._h, idx, buf, n)
        return buf.raw[:n].decode("utf-8")

    def encode_longest_match(self, text: str) -> List[Tuple[int, int]]:
        cps = np.fromiter((ord(c) for c in text), dtype=np.uint32, count=len(text))
        ids = np.empty(max(1, len(text)), dtype=np.int64)
        starts = np.empty(max(1, len(text)), dtype=np.int64)
        n = int(lib().fbam_tok_encode(self._h, cps.ctypes.data, len(cps), ids.ctypes.data, starts.ctypes.data,
                                      len(ids)))
        return [(int(ids[i]), int(starts[i])) for i in range(n)]

    def close(self) -> None:
        if self._h:
            lib().fbam_tok_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass


# -- safetensors ---------------------------------------------------------------------------------
_NP = {"F32": np.float32, "F16": np.float16, "BF16": np.uint16, "U32": np.uint32, "U64": np.uint64, "I32": np.int32,
       "I64": np.int64, "U8": np.uint8, "BOOL": np.uint8, "F64": np.float64, "I8": np.int8}


def st_read(path: str) -> Dict[str, Tuple[str, np.ndarray]]:
    """name → (safetensors dtype tag, array).  BF16 comes back as raw ``uint16`` words."""
    h = lib().fbam_st_open(path.encode())
    if not h:
        raise ValueError(_err())
    try:
        out = {}
        for i in range(int(lib().fbam_st_count(h))):
            name = lib().fbam_st_name(h, i).decode()
            tag = lib().fbam_st_dtype(h, i).decode()
            shape = [int(lib().fbam_st_dim(h, i, d)) for d in range(int(lib().fbam_st_ndim(h, i)))]
            arr = np.empty(shape, dtype=_NP[tag])
            if arr.size and lib().fbam_st_read(h, i, arr.ctypes.data) != 0:
                raise ValueError(_err())
            out[name] = (tag, arr)
        return out
    finally:
        lib().fbam_st_close(h)


def st_write(path: str, tensors: Dict[str, Tuple[str, np.ndarray]]) -> None:
    names = list(tensors)
    n = len(names)
    # (np.ascontiguousarray would turn a 0-d array into shape (1,))
    arrs = [np.require(tensors[k][1], requirements="C") for k in names]
    c_names = (C.c_char_p * n)(*[k.encode() for k in names])
    c_dtypes = (C.c_char_p * n)(*[tensors[k][0].encode() for k in names])
    ndims = (C.c_int64 * n)(*[a.ndim for a in arrs])
    flat_shapes = [d for a in arrs for d in a.shape]
    shapes = (C.c_int64 * max(1, len(flat_shapes)))(*flat_shapes)
    ptrs = (C.c_void_p * n)(*[a.ctypes.data for a in arrs])
    nbytes = (C.c_int64 * n)(*[a.nbytes for a in arrs])
    lib().fbam_st_write.argtypes = [C.c_char_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_void_p]
    if lib().fbam_st_write(path.encode(), n, c_names, c_dtypes, ndims, shapes, ptrs, nbytes) != 0:
        raise ValueError(_err())


def tenscmp(path_a: str, path_b: str, threshold: float) -> Tuple[int, str]:
    buf = C.create_string_buffer(1 << 16)
    bad = int(lib().fbam_tenscmp(path_a.encode(), path_b.encode(), threshold, buf, len(buf)))
    if bad < 0:
        raise ValueError(_err())
    return bad, buf.value.decode("utf-8", "replace")


# -- cursor --------------------------------------------------------------------------------------
class NativeCursorCommitter:
    def __init__(self, path: str):
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        self._h = lib().fbam_cursor_create(path.encode())

    def commit(self, step: int, rng_state: int, batch: int, seq: int) -> None:
        lib().fbam_cursor_commit(self._h, step, rng_state & ((1 << 64) - 1), batch, seq)

    def flush(self, timeout_s: float = 10.0) -> bool:
        return lib().fbam_cursor_flush(self._h, int(timeout_s * 1000)) == 0

    def close(self) -> None:
        if self._h:
            lib().fbam_cursor_destroy(self._h)
            self._h = None


# -- rendezvous ----------------------------------------------------------------------------------
def rdv_serve(ip: str, port: int, world: int, blob: bytes, timeout_s: float = 60.0) -> None:
    if len(blob) != 128:
        raise ValueError("blob must be 128 bytes")
    rc = lib().fbam_rdv_serve(ip.encode(), port, world, blob, int(timeout_s * 1000))
    if rc != 0:
        raise RuntimeError_(_err())


def rdv_fetch(ip: str, port: int, rank: int, timeout_s: float = 60.0) -> bytes:
    buf = C.create_string_buffer(128)
    rc = lib().fbam_rdv_fetch(ip.encode(), port, rank, buf, int(timeout_s * 1000))
    if rc != 0:
        raise RuntimeError_(_err())
    return buf.raw


# -- batch loader --------------------------------------------------------------------------------
class NativeBatchLoader:
    """Gathers batches from raw ``.fbrec`` recordings with worker threads (``csrc/runtime/loader.cpp``).
    ``tokens`` is the tokenizer's vocabulary with ids = list positions; ``fill`` writes into caller-provided (pinned) tensors and
    releases the interpreter lock while it runs, so a prefetch thread really overlaps with the training step."""

    def __init__(self, paths: List[str], tokens: List[str], max_code_point: int, vocab: int, threads: int = 0):
        if any("\0" in t for t in tokens):
            raise ValueError("tokens containing NUL cannot be passed to the native loader")
        tok_arr = (C.c_char_p * len(tokens))(*[t.encode("utf-8") for t in tokens])
        self._tok_handle = lib().fbam_tok_from_list(tok_arr, len(tokens))
        if not self._tok_handle:
            raise ValueError(_err())
        arr = (C.c_char_p * len(paths))(*[p.encode() for p in paths])
        threads = threads or min(16, max(1, (os.cpu_count() or 2) // 2))
        self._h = lib().fbam_loader_open(arr, len(paths), self._tok_handle, max_code_point, vocab, threads)
        if not self._h:
            raise ValueError(_err())
        self.rows, self.cols = int(lib().fbam_loader_rows(self._h)), int(lib().fbam_loader_cols(self._h))
        self.frames = [int(lib().fbam_loader_frames(self._h, i)) for i in range(len(paths))]

    def fill(self, indices, starts, seq: int, out_cells, out_targets) -> None:
        """``out_cells`` int32 ``(B, seq, rows*cols, 3)`` and ``out_targets`` int64 ``(B, seq)`` host tensors."""
        b = len(indices)
        idx = np.asarray(indices, dtype=np.uint32)
        st = np.asarray(starts, dtype=np.uint64)
        if tuple(out_cells.shape) != (b, seq, self.rows * self.cols, 3) or tuple(out_targets.shape) != (b, seq):
            raise ValueError("output tensors have the wrong shape")
        if not out_cells.is_contiguous() or not out_targets.is_contiguous():
            raise ValueError("output tensors must be contiguous")
        if lib().fbam_loader_fill(self._h, idx.ctypes.data, st.ctypes.data, b, seq, out_cells.data_ptr(),
                                  out_targets.data_ptr()) != 0:
            raise ValueError(_err())

    def close(self) -> None:
        if self._h:
            lib().fbam_loader_close(self._h)
            self._h = None
        if getattr(self, "_tok_handle", None):
            lib().fbam_tok_free(self._tok_handle)
            self._tok_handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass


def synth_fill(seed: int, call: int, cells_per_frame: int, cell_vocab: int, attr_ids: int, k: int, action_vocab: int,
               palette16, out_cells, out_targets, threads: int = 0) -> None:
    """Fills ``out_cells`` int32 ``(B, T, P, 3)`` and ``out_targets`` int64 ``(B, T)`` with a seeded synthetic batch
    (``csrc/runtime/loader.cpp``: ``fbam_synth_fill``)."""
    b, t = int(out_cells.shape[0]), int(out_cells.shape[1])
    pal = np.ascontiguousarray(palette16, dtype=np.uint32)
    if pal.size != 16 or not out_cells.is_contiguous() or not out_targets.is_contiguous():
        raise ValueError("need a 16-entry palette and contiguous outputs")
    threads = threads or min(16, max(1, (os.cpu_count() or 2) // 2))
    if lib().fbam_synth_fill(seed & ((1 << 64) - 1), call, cells_per_frame, b, t, cell_vocab, attr_ids, k, action_vocab,
                             pal.ctypes.data, out_cells.data_ptr(), out_targets.data_ptr(), threads) != 0:
        raise ValueError("invalid arguments for the synthetic batch generator")
