"""Byte-level BPE tokenizer (rust-nn src/tokenizer.rs): `BpeTokenizer`, `MergeScoring`.

The work happens in the C++ runtime (csrc/io/tokenizer.cpp): pre-tokenisation, training with
incremental pair counts, heap-ordered encoding, batch encoding on a thread pool. This module keeps
the reference's API and its text save format (`# scoring=...`, `# merges=N`, one `left right` pair
per line, optional `# specials` section).
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Sequence, Tuple

import numpy as np

from . import _native as nv

_P, _LL, _I = C.c_void_p, C.c_longlong, C.c_int
nv.register_sigs({
    "b200_bpe_train": [_P, _LL, _I, _I, C.c_double, _P, _LL],
    "b200_bpe_create": [_P, _LL],
    "b200_bpe_free": [_P],
    "b200_bpe_add_special": [_P, _P, _LL],
    "b200_bpe_vocab_size": [_P],
    "b200_bpe_id_bytes": [_P, C.c_uint, _P, _LL],
    "b200_bpe_encode": [_P, _P, _LL, _P, _LL, _P, _P],
    "b200_bpe_count": [_P, _P, _LL],
    "b200_bpe_encode_batch": [_P, _P, _P, _LL, _P, _LL, _P, _I],
    "b200_bpe_decode": [_P, _P, _LL, _P, _LL],
    "b200_bpe_pretokenize": [_P, _LL, _P, _LL],
})


def _lib():
    lib = nv.host()
    for name in ("b200_bpe_train", "b200_bpe_id_bytes", "b200_bpe_encode", "b200_bpe_count", "b200_bpe_encode_batch", "b200_bpe_decode",
                 "b200_bpe_pretokenize"):
        getattr(lib, name).restype = C.c_longlong
    lib.b200_bpe_create.restype = C.c_void_p
    lib.b200_bpe_free.restype = None
    return lib


class MergeScoring:
    """`Frequency` (count), `PMI` (count / (count_l * count_r)), `Hybrid(alpha)`
    (alpha * ln(count + 1) + (1 - alpha) * ln(pmi + 1))."""

    def __init__(self, kind: str = "Frequency", alpha: float = 0.5):
        self.kind, self.alpha = kind, alpha

    def __repr__(self):
        return f"Hybrid {{ alpha: {self.alpha} }}" if self.kind == "Hybrid" else self.kind

    def __eq__(self, other):
        return isinstance(other, MergeScoring) and (self.kind, self.alpha if self.kind == "Hybrid" else 0) == \
            (other.kind, other.alpha if other.kind == "Hybrid" else 0)

    @staticmethod
    def Hybrid(alpha: float) -> "MergeScoring":
        return MergeScoring("Hybrid", alpha)

    @property
    def code(self) -> int:
        return {"Frequency": 0, "PMI": 1, "Hybrid": 2}[self.kind]


MergeScoring.Frequency = MergeScoring("Frequency")
MergeScoring.PMI = MergeScoring("PMI")


def _bytes_arr(b: bytes):
    return (C.c_ubyte * max(len(b), 1)).from_buffer_copy(b if b else b"\0")


def pre_tokenize(text) -> List[Tuple[int, bytes]]:
    """(start, chunk) pairs of the regex-free pre-tokeniser (src/tokenizer.rs:447-485)."""
    b = text.encode("utf-8") if isinstance(text, str) else bytes(text)
    out = np.empty(2 * max(len(b), 1), dtype=np.uint32)
    n = _lib().b200_bpe_pretokenize(_bytes_arr(b), len(b), out.ctypes.data, len(b))
    return [(int(out[2 * i]), b[out[2 * i]:out[2 * i + 1]]) for i in range(n)]


class BpeTokenizer:
    def __init__(self, merges: Sequence[Tuple[int, int]], scoring: MergeScoring = None):
        self._lib = _lib()
        self.merges: List[Tuple[int, int]] = [(int(l), int(r)) for l, r in merges]
        arr = np.asarray(self.merges, dtype=np.uint32).reshape(-1)
        self._h = self._lib.b200_bpe_create(arr.ctypes.data if arr.size else None, len(self.merges))
        self.scoring = scoring or MergeScoring.Frequency
        self.special: Dict[str, int] = {}

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                self._lib.b200_bpe_free(self._h); self._h = None
        except Exception:
            pass

    # ---- construction
    @staticmethod
    def from_merges(merges: Sequence[Tuple[int, int]]) -> "BpeTokenizer":
        return BpeTokenizer(merges)

    @staticmethod
    def train(corpus: str, vocab_size: int, scoring: MergeScoring = None) -> "BpeTokenizer":
        if vocab_size < 256:
            raise ValueError("vocab_size must be >= 256 (base bytes)")
        scoring = scoring or MergeScoring.Frequency
        b = corpus.encode("utf-8")
        cap = vocab_size - 256
        out = np.zeros(2 * max(cap, 1), dtype=np.uint32)
        n = _lib().b200_bpe_train(_bytes_arr(b), len(b), vocab_size, scoring.code, float(scoring.alpha), out.ctypes.data, cap)
        if n < 0:
            raise ValueError("tokenizer training failed")
        return BpeTokenizer([(int(out[2 * i]), int(out[2 * i + 1])) for i in range(n)], scoring)

    def add_special(self, text: str) -> int:
        if text in self.special:
            return self.special[text]
        b = text.encode("utf-8")
        tid = self._lib.b200_bpe_add_special(self._h, _bytes_arr(b), len(b))
        self.special[text] = tid
        return tid

    # ---- queries
    @property
    def vocab_size(self) -> int:
        return self._lib.b200_bpe_vocab_size(self._h)

    def len(self) -> int:
        return self.vocab_size

    def __len__(self) -> int:
        return self.vocab_size

    def is_empty(self) -> bool:
        return not self.merges and not self.special

    def id_to_bytes(self, tid: int) -> bytes:
        buf = (C.c_ubyte * 256)()
        n = self._lib.b200_bpe_id_bytes(self._h, tid, buf, 256)
        if n > 256:
            buf = (C.c_ubyte * n)()
            self._lib.b200_bpe_id_bytes(self._h, tid, buf, n)
        return bytes(buf[:n])

    # ---- encode / decode
    def _encode(self, text: str, offsets: bool):
        b = text.encode("utf-8")
        cap = len(b) + 8
        ids = np.empty(cap, dtype=np.uint32)
        st = np.empty(cap, dtype=np.uint32) if offsets else None
        en = np.empty(cap, dtype=np.uint32) if offsets else None
        n = self._lib.b200_bpe_encode(self._h, _bytes_arr(b), len(b), ids.ctypes.data, cap, st.ctypes.data if offsets else None,
                                      en.ctypes.data if offsets else None)
        return (ids[:n], st[:n], en[:n]) if offsets else ids[:n]

    def encode(self, text: str) -> List[int]:
        return self._encode(text, False).tolist()

    def encode_with_offsets(self, text: str) -> List[Tuple[int, range]]:
        ids, st, en = self._encode(text, True)
        return [(int(i), range(int(a), int(b))) for i, a, b in zip(ids, st, en)]

    def decode_bytes(self, ids: Sequence[int]) -> bytes:
        arr = np.asarray(list(ids), dtype=np.uint32)
        cap = max(int(arr.size) * 8, 16)
        out = np.empty(cap, dtype=np.uint8)
        n = self._lib.b200_bpe_decode(self._h, arr.ctypes.data if arr.size else None, arr.size, out.ctypes.data, cap)
        if n > cap:
            out = np.empty(n, dtype=np.uint8)
            self._lib.b200_bpe_decode(self._h, arr.ctypes.data, arr.size, out.ctypes.data, n)
        return out[:n].tobytes()

    def decode(self, ids: Sequence[int]) -> str:
        return self.decode_bytes(ids).decode("utf-8", errors="replace")

    def encode_batch(self, texts: Sequence[str], threads: int = 0) -> List[List[int]]:
        blobs = [t.encode("utf-8") for t in texts]
        n = len(blobs)
        if n == 0:
            return []
        off = np.zeros(n + 1, dtype=np.int64)
        off[1:] = np.cumsum([len(b) for b in blobs])
        joined = b"".join(blobs)
        cap = len(joined) + 8
        ids = np.empty(cap, dtype=np.uint32)
        id_off = np.zeros(n + 1, dtype=np.int64)
        total = self._lib.b200_bpe_encode_batch(self._h, _bytes_arr(joined), off.ctypes.data, n, ids.ctypes.data, cap, id_off.ctypes.data, threads)
        if total < 0:
            raise RuntimeError("encode_batch: output buffer too small")
        return [ids[id_off[i]:id_off[i + 1]].tolist() for i in range(n)]

    def decode_batch(self, batch: Sequence[Sequence[int]]) -> List[str]:
        return [self.decode(ids) for ids in batch]

    def count_tokens(self, text: str) -> int:
        b = text.encode("utf-8")
        return int(self._lib.b200_bpe_count(self._h, _bytes_arr(b), len(b)))

    def compression_ratio(self, text: str) -> float:
        return self.count_tokens(text) / max(len(text), 1)

    # ---- persistence
    def save(self) -> str:
        lines = [f"# scoring={self.scoring!r}", f"# merges={len(self.merges)}"] + [f"{l} {r}" for l, r in self.merges]
        if self.special:
            lines.append("# specials")
            lines += [f"{tid} {text}".replace("\n", "\\n") for text, tid in sorted(self.special.items(), key=lambda kv: kv[1])]
        return "\n".join(lines) + "\n"

    @staticmethod
    def load(text: str) -> "BpeTokenizer":
        merges, specials, scoring, in_sp = [], [], MergeScoring.Frequency, False
        for line in text.splitlines():
            line = line.strip()
            if not line:
                continue
            if line.startswith("# scoring="):
                rest = line[len("# scoring="):]
                scoring = MergeScoring.PMI if rest == "PMI" else MergeScoring.Hybrid(0.5) if rest.startswith("Hybrid") else MergeScoring.Frequency
                continue
            if line == "# specials":
                in_sp = True
                continue
            if line.startswith("#"):
                continue
            if in_sp:
                parts = line.split(" ", 1)
                specials.append(parts[1].replace("\\n", "\n") if len(parts) > 1 else "")
            else:
                parts = line.split()
                l = int(parts[0]) if parts and parts[0].isdigit() else 0
                r = int(parts[1]) if len(parts) > 1 and parts[1].isdigit() else 0
                merges.append((l, r))
        tok = BpeTokenizer(merges, scoring)
        for s in specials:
            tok.add_special(s)
        return tok
