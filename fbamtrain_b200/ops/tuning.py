"""Per-shape tile configurations for the tensor-core launchers.

The launchers pick tile shapes by rule (``native_ops.gemm`` / ``conv_pass``).  A tuning table overrides the rule
for the shapes it lists: ``python -m fbamtrain_b200.autotune`` measures the candidates of every GEMM / convolution
shape a model launches on the GPU at hand and writes the winners to a JSON file; ``FBAMTRAIN_TUNING_FILE=<file>``
makes the launchers use it.  The reference keeps the same kind of table per architecture, produced by its
autotune drivers (reference: ``kernel_gen/kernel_gen/pysrc/autotune_matmul.py``,
``kernel_gen/kernel_gen/kernels/cutlass_codegen/configs/output_configs/autotune_constants_sm100.json``).

File format::

    {"device": "NVIDIA B200", "entries": {"gemm m8192 n4096 k1024 NN": {"best": {"bm": 256, "bn": 256,
      "two_cta": true}, "ms": 0.071, "candidates": [{"config": {...}, "ms": 0.075}, ...]}, ...}}

Only ``best`` is read by the launchers.  Keys of a configuration — GEMM: ``bm`` (128 / 256), ``bn`` (128 / 256),
``two_cta`` (bool), ``max_ctas``; convolution: ``tile_rows`` (128 / 256), ``bn``, ``two_cta``.  Missing keys keep
the launcher's rule.
"""
from __future__ import annotations

import contextlib
import json
import os
from typing import Dict, Iterator, List, Optional

_GEMM_KEYS = ("bm", "bn", "two_cta", "max_ctas")
_CONV_KEYS = ("tile_rows", "bn", "two_cta")

_table: Optional[Dict[str, dict]] = None
_loaded_from: Optional[str] = None
_recording: Optional[Dict[str, dict]] = None


def gemm_key(m: int, n: int, k: int, a_mn: bool, b_mn: bool) -> str:
    return f"gemm m{m} n{n} k{k} {'T' if a_mn else 'N'}{'T' if b_mn else 'N'}"


def conv_key(batch: int, grid_h: int, grid_w: int, c: int, n_out: int, taps: int, in_mul: int, out_mul: int) -> str:
    return f"conv b{batch} g{grid_h}x{grid_w} c{c} n{n_out} taps{taps} in_mul{in_mul} out_mul{out_mul}"


def _validate(key: str, cfg: dict) -> dict:
    allowed = _GEMM_KEYS if key.startswith("gemm ") else _CONV_KEYS if key.startswith("conv ") else None
    if allowed is None:
        raise ValueError(f"tuning table: unknown entry kind '{key}'")
    for name, value in cfg.items():
        if name not in allowed:
            raise ValueError(f"tuning table: '{name}' is not a configuration key of '{key}' (allowed: {allowed})")
        if name == "two_cta":
            if not isinstance(value, bool):
                raise ValueError(f"tuning table: two_cta of '{key}' must be true or false")
        elif not isinstance(value, int) or isinstance(value, bool) or value < 0:
            raise ValueError(f"tuning table: {name} of '{key}' must be a non-negative integer")
    for name in ("bm", "bn", "tile_rows"):
        if cfg.get(name, 0) not in (0, 128, 256):
            raise ValueError(f"tuning table: {name} of '{key}' must be 128 or 256")
    return dict(cfg)


def parse(document: dict) -> Dict[str, dict]:
    """``{key: best configuration}`` from a parsed tuning file; raises ``ValueError`` on anything malformed."""
    entries = document.get("entries")
    if not isinstance(entries, dict):
        raise ValueError("tuning table: no 'entries' object")
    out = {}
    for key, entry in entries.items():
        if not isinstance(entry, dict) or not isinstance(entry.get("best"), dict):
            raise ValueError(f"tuning table: entry '{key}' has no 'best' configuration")
        out[key] = _validate(key, entry["best"])
    return out


def set_table(table: Optional[Dict[str, dict]]) -> None:
    """Install a table directly (``None``: back to the environment's file, or to none)."""
    global _table, _loaded_from
    _table = None if table is None else {k: _validate(k, v) for k, v in table.items()}
    _loaded_from = None if table is None else "<set_table>"


def _current() -> Optional[Dict[str, dict]]:
    global _table, _loaded_from
    path = os.environ.get("FBAMTRAIN_TUNING_FILE", "")
    if _loaded_from == "<set_table>":
        return _table
    if not path:
        _table, _loaded_from = None, None
        return None
    if _loaded_from != path:
        with open(path) as f:
            _table = parse(json.load(f))
        _loaded_from = path
    return _table


def lookup(key: str, shape: Optional[dict] = None) -> Optional[dict]:
    """The tuned configuration for ``key`` (None: use the launcher's rule).  While :func:`recording` is active the
    key and ``shape`` (what the tuner needs to rebuild the launch) are noted as well."""
    if _recording is not None and key not in _recording:
        _recording[key] = dict(shape or {})
    table = _current()
    return None if table is None else table.get(key)


@contextlib.contextmanager
def recording() -> Iterator[Dict[str, dict]]:
    """Collects ``{key: shape}`` of every tunable launch made inside the block."""
    global _recording
    previous, _recording = _recording, {}
    try:
        yield _recording
    finally:
        _recording = previous


def gemm_candidates(m: int, n: int) -> List[dict]:
    """Tile configurations worth measuring for an ``m x n`` output."""
    out: List[dict] = []
    for bm in (128, 256):
        for bn in (128, 256):
            if bn > max(128, n) or bm > max(128, m):
                continue
            out.append({"bm": bm, "bn": bn, "two_cta": False})
    if n >= 256 and n % 16 == 0 and m > 128:
        out.append({"bm": 256, "bn": 256, "two_cta": True})
    return out


def conv_candidates(n_out: int) -> List[dict]:
    out = [{"tile_rows": 128, "bn": bn, "two_cta": False} for bn in (128, 256) if bn <= max(128, n_out)]
    if n_out >= 128:
        out += [{"tile_rows": 256, "bn": bn, "two_cta": False} for bn in (128, 256) if bn <= max(128, n_out)]
    if n_out >= 256:
        out.append({"bn": 256, "two_cta": True})
    return out
