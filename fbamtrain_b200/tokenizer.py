"""``FBAM_TOK v1.0`` action tokenizer: a trie over Unicode code points.

File format (reference: ``src/tokenizer.cpp:79-124``): first line is the literal header
``# FBAM_TOK v1.0``; every following non-empty line is one JSON string literal, the token text.
Tokens are stable-sorted by length (in code points), longest first, and a token's id is its index
after that sort.  ``TokenizerHandle`` walks the trie one code point at a time and is the primitive
used for longest-match extraction of action tokens from recorded keystrokes
(reference: ``include/tokenizer.h:14-62``, ``src/main.cpp:1912-1981``).

A native implementation of the same trie lives in ``csrc/runtime/runtime.cpp`` (``fbam_tok_*``); when the runtime
library is built, :func:`Tokenizer.encode_longest_match` dispatches to it.
"""
from __future__ import annotations

import json
from typing import Dict, List, Optional, Sequence, Tuple

HEADER = "# FBAM_TOK v1.0"


class _Node:
    __slots__ = ("children", "token_id")

    def __init__(self) -> None:
        self.children: Dict[int, "_Node"] = {}
        self.token_id: Optional[int] = None


class TokenizerHandle:
    """Incremental matcher.  Dead once a code point has no edge from the current node."""

    def __init__(self, tokenizer: "Tokenizer"):
        self._tok = tokenizer
        self._node: Optional[_Node] = tokenizer._root

    def add_char(self, ch: int) -> None:
        if self._node is None:
            return
        self._node = self._node.children.get(ch)

    def current_token_id(self) -> Optional[int]:
        return None if self._node is None else self._node.token_id

    def is_dead(self) -> bool:
        return self._node is None

    def has_continuation(self) -> bool:
        return self._node is not None and bool(self._node.children)

    def reset(self) -> None:
        self._node = self._tok._root


class Tokenizer:
    def __init__(self, tokens: Sequence[str]):
        self._tokens: List[str] = list(tokens)
        self._root = _Node()
        for idx, tok in enumerate(self._tokens):
            node = self._root
            for ch in tok:
                node = node.children.setdefault(ord(ch), _Node())
            node.token_id = idx  # a duplicated token keeps the later index, like the reference

    @staticmethod
    def from_lines(lines: Sequence[str], origin: str = "<memory>") -> "Tokenizer":
        if not lines:
            raise ValueError(f"Tokenizer file is empty: {origin}")
        if lines[0].rstrip("\r\n") != HEADER:
            raise ValueError(f"Invalid tokenizer header in file {origin}: {lines[0].rstrip()}")
        tokens: List[str] = []
        for line_no, line in enumerate(lines[1:], start=2):
            line = line.rstrip("\r\n")
            if not line:
                continue
            try:
                tok = json.loads(line)
                if not isinstance(tok, str):
                    raise TypeError("token is not a JSON string")
            except Exception as ex:  # noqa: BLE001 - message carries the line number
                raise ValueError(f"Failed to parse token on line {line_no} in {origin}: {ex}") from ex
            tokens.append(tok)
        tokens.sort(key=len, reverse=True)  # list.sort is stable
        return Tokenizer(tokens)

    @staticmethod
    def from_file(path: str) -> "Tokenizer":
        try:
            with open(path, "r", encoding="utf-8", newline="\n") as f:
                lines = f.readlines()
        except OSError as ex:
            raise ValueError(f"Failed to open tokenizer file: {path}") from ex
        return Tokenizer.from_lines(lines, path)

    def save(self, path: str) -> None:
        with open(path, "w", encoding="utf-8", newline="\n") as f:
            f.write(HEADER + "\n")
            for t in self._tokens:
                f.write(json.dumps(t) + "\n")

    def new_handle(self) -> TokenizerHandle:
        return TokenizerHandle(self)

    @property
    def tokens(self) -> List[str]:
        return self._tokens

    def __len__(self) -> int:
        return len(self._tokens)

    def encode_longest_match(self, text: str) -> List[Tuple[int, int]]:
        """Greedy longest-match tokenization.  Returns ``(token_id, start_offset)`` pairs; code points
        that start no token are skipped."""
        out: List[Tuple[int, int]] = []
        i, n = 0, len(text)
        while i < n:
            node, best, best_len, j = self._root, None, 0, i
            while j < n:
                node = node.children.get(ord(text[j]))
                if node is None:
                    break
                j += 1
                if node.token_id is not None:
                    best, best_len = node.token_id, j - i
            if best is None:
                i += 1
            else:
                out.append((best, i))
                i += best_len
        return out
