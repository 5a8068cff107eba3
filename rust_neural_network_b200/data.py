"""Datasets and loaders (rust-nn src/data.rs): `Column`, `Dataset`, `load_csv` / `load_tsv` /
`load_jsonl`, `make_classification` / `make_regression`, `DatasetBuilder`, `Credentials`,
`DatasetListing`, `format_listings`, and the Hugging Face / Kaggle clients.

The text parsers are the C++ runtime's (csrc/io/parsers.cpp); float columns are numpy arrays so
`to_tensor` is one stack + one pinned host-to-device copy. The remote clients
(`load_huggingface`, `load_kaggle`, `search_*`) keep the reference's cache layout
(`~/.cache/rust-nn/datasets/<dataset>_<split>.json`) and are served from that cache; without a
cached copy and without network access they raise `DataError` with the reference's message shape.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
import json
import os
import urllib.error
import urllib.parse
import urllib.request
from typing import Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from . import _native as nv
from .error import RustNnError

_P, _LL, _I = C.c_void_p, C.c_longlong, C.c_int
nv.register_sigs({
    "b200_table_parse_delimited": [C.c_char_p, _LL, C.c_char],
    "b200_table_parse_jsonl": [C.c_char_p, _LL],
    "b200_table_free": [_P],
    "b200_table_error": [_P, _P, _LL],
    "b200_table_ncols": [_P],
    "b200_table_col_len": [_P, _I],
    "b200_table_col_is_float": [_P, _I],
    "b200_table_col_name": [_P, _I, _P, _LL],
    "b200_table_col_floats": [_P, _I, _P],
    "b200_table_col_text": [_P, _I, _P, _LL, _P],
})


class DataError(RustNnError):
    pass


def _lib():
    lib = nv.host()
    lib.b200_table_parse_delimited.restype = C.c_void_p
    lib.b200_table_parse_jsonl.restype = C.c_void_p
    lib.b200_table_free.restype = None
    lib.b200_table_col_floats.restype = None
    for n in ("b200_table_error", "b200_table_col_len", "b200_table_col_name", "b200_table_col_text"):
        getattr(lib, n).restype = C.c_longlong
    return lib


class Column:
    """`Float` (numpy float32) or `Text` (list of str)."""

    def __init__(self, data):
        if isinstance(data, np.ndarray) or (len(data) > 0 and not isinstance(data[0], str)) or (len(data) == 0 and not isinstance(data, list)):
            self.data = np.asarray(data, dtype=np.float32)
            self.numeric = True
        else:
            self.data = list(data)
            self.numeric = False

    @staticmethod
    def Float(v) -> "Column":
        c = Column.__new__(Column); c.data = np.asarray(v, dtype=np.float32); c.numeric = True
        return c

    @staticmethod
    def Text(v) -> "Column":
        c = Column.__new__(Column); c.data = [str(s) for s in v]; c.numeric = False
        return c

    def len(self) -> int:
        return len(self.data)

    def __len__(self) -> int:
        return len(self.data)

    def is_numeric(self) -> bool:
        return self.numeric

    def is_empty(self) -> bool:
        return len(self.data) == 0


class Dataset:
    def __init__(self, source: str = ""):
        self.columns: Dict[str, Column] = {}
        self.num_rows = 0
        self.source = source

    @staticmethod
    def new(source: str) -> "Dataset":
        return Dataset(source)

    def add_float_column(self, name: str, data) -> None:
        col = Column.Float(data)
        self.num_rows = max(self.num_rows, len(col))
        self.columns[name] = col

    def add_text_column(self, name: str, data) -> None:
        col = Column.Text(data)
        self.num_rows = max(self.num_rows, len(col))
        self.columns[name] = col

    def get_float(self, name: str) -> Optional[np.ndarray]:
        c = self.columns.get(name)
        return c.data if c is not None and c.numeric else None

    def get_text(self, name: str) -> Optional[List[str]]:
        c = self.columns.get(name)
        return c.data if c is not None and not c.numeric else None

    def to_tensor(self, column_names: Sequence[str], device=None) -> torch.Tensor:
        """[num_rows, len(column_names)] fp32; missing columns / short columns read as 0."""
        out = np.zeros((self.num_rows, len(column_names)), dtype=np.float32)
        for j, name in enumerate(column_names):
            f = self.get_float(name)
            if f is not None:
                n = min(len(f), self.num_rows)
                out[:n, j] = f[:n]
        t = torch.from_numpy(out)
        if device is not None and torch.device(device).type == "cuda":
            return t.pin_memory().to(device, non_blocking=True)
        return t

    def to_token_tensor(self, column_name: str, tokenizer, max_len: int, device=None, dtype=torch.float32) -> torch.Tensor:
        """[rows, max_len] token ids, zero padded / truncated (fp32 as the reference; pass `dtype=torch.int64` for ids)."""
        text = self.get_text(column_name) or []
        out = np.zeros((len(text), max_len), dtype=np.int64)
        for i, ids in enumerate(tokenizer.encode_batch(text) if text else []):
            n = min(len(ids), max_len)
            out[i, :n] = ids[:n]
        t = torch.from_numpy(out).to(dtype)
        return t.to(device) if device is not None else t

    def summary(self) -> str:
        names = sorted(self.columns)
        info = [f"  {n}: {'f32' if self.columns[n].numeric else 'str'}[{len(self.columns[n])}]" for n in names]
        return f"Dataset (source: {self.source})\n  rows: {self.num_rows}\n  columns ({len(names)}):\n" + "\n".join(info)

    def _slice(self, source: str, a: int, b: int) -> "Dataset":
        d = Dataset(source)
        d.num_rows = max(b - a, 0)
        for name, col in self.columns.items():
            if col.numeric:
                d.add_float_column(name, col.data[a:b].copy())
            else:
                d.add_text_column(name, col.data[a:b])
        d.num_rows = max(b - a, 0)
        return d

    def head(self, n: int) -> "Dataset":
        return self._slice(self.source, 0, min(n, self.num_rows))

    def train_test_split(self, ratio: float) -> Tuple["Dataset", "Dataset"]:
        split = int(self.num_rows * ratio)
        return self._slice(f"{self.source} (train)", 0, split), self._slice(f"{self.source} (test)", split, self.num_rows)


# ------------------------------------------------------------------ parsers
def _table_to_dataset(h, source: str) -> Dataset:
    lib = _lib()
    try:
        err = (C.c_char * 256)()
        n = lib.b200_table_error(h, err, 256)
        if n:
            raise DataError(err.raw[:n].decode())
        ds = Dataset(source)
        for c in range(lib.b200_table_ncols(h)):
            nb = (C.c_char * 4096)()
            ln = lib.b200_table_col_name(h, c, nb, 4096)
            name = nb.raw[:ln].decode("utf-8", errors="replace")
            rows = lib.b200_table_col_len(h, c)
            if lib.b200_table_col_is_float(h, c):
                arr = np.empty(rows, dtype=np.float32)
                lib.b200_table_col_floats(h, c, arr.ctypes.data)
                ds.add_float_column(name, arr)
            else:
                total = lib.b200_table_col_text(h, c, None, 0, None)
                buf = np.empty(max(total, 1), dtype=np.uint8)
                off = np.zeros(rows + 1, dtype=np.int64)
                lib.b200_table_col_text(h, c, buf.ctypes.data, max(total, 1), off.ctypes.data)
                raw = buf.tobytes()
                ds.add_text_column(name, [raw[off[i]:off[i + 1]].decode("utf-8", errors="replace") for i in range(rows)])
        return ds
    finally:
        lib.b200_table_free(h)


def parse_delimited(content: str, delimiter: str) -> Dataset:
    b = content.encode("utf-8")
    return _table_to_dataset(_lib().b200_table_parse_delimited(b, len(b), delimiter.encode()), "csv")


def parse_jsonl(content: str) -> Dataset:
    b = content.encode("utf-8")
    return _table_to_dataset(_lib().b200_table_parse_jsonl(b, len(b)), "jsonl")


def _read(path: str) -> str:
    try:
        with open(path, "r", encoding="utf-8") as f:
            return f.read()
    except OSError as e:
        raise DataError(f"Failed to read {path}: {e}") from e


def load_csv(path: str) -> Dataset:
    return parse_delimited(_read(path), ",")


def load_tsv(path: str) -> Dataset:
    return parse_delimited(_read(path), "\t")


def load_jsonl(path: str) -> Dataset:
    return parse_jsonl(_read(path))


def parse_csv_line(line: str, delimiter: str = ",") -> List[str]:
    fields, cur, q = [], [], False
    for ch in line:
        if ch == '"':
            q = not q
        elif ch == delimiter and not q:
            fields.append("".join(cur)); cur = []
        else:
            cur.append(ch)
    fields.append("".join(cur))
    return fields


def parse_simple_json_object(line: str) -> List[Tuple[str, str]]:
    ds = parse_jsonl(line)
    out = []
    for name, col in ds.columns.items():
        v = col.data[0]
        out.append((name, v if isinstance(v, str) else repr(float(v)).rstrip("0").rstrip(".") if float(v) != int(v) else str(int(v))))
    return out


def split_json_objects(body: str) -> List[str]:
    objs, depth, start = [], 0, None
    for i, ch in enumerate(body):
        if ch == "{":
            if depth == 0:
                start = i
            depth += 1
        elif ch == "}":
            depth -= 1
            if depth == 0 and start is not None:
                objs.append(body[start:i + 1]); start = None
    return objs


def base64_encode(text: str) -> str:
    import base64
    return base64.b64encode(text.encode("utf-8")).decode("ascii")


# ------------------------------------------------------------------ synthetic data
def make_classification(n_samples: int, n_features: int, n_classes: int, seed: Optional[int] = None) -> Dataset:
    """Class c has feature j centred at 0.8 c + 0.05 j with uniform noise of width 0.6; label = i mod classes."""
    rng = np.random.default_rng(seed)
    cls = np.arange(n_samples) % max(n_classes, 1)
    ds = Dataset("synthetic")
    for j in range(n_features):
        ds.add_float_column(f"f{j}", (cls * 0.8 + j * 0.05 + (rng.random(n_samples, dtype=np.float32) - 0.5) * 0.6).astype(np.float32))
    ds.add_float_column("label", cls.astype(np.float32))
    return ds


def make_regression(n_samples: int, n_features: int, seed: Optional[int] = None) -> Dataset:
    """x ~ U(-1,1)^d, y = x . w + U(-0.05, 0.05) with w ~ U(-1,1)^d."""
    rng = np.random.default_rng(seed)
    w = rng.random(n_features, dtype=np.float32) * 2 - 1
    x = rng.random((n_samples, n_features), dtype=np.float32) * 2 - 1
    y = x @ w + (rng.random(n_samples, dtype=np.float32) - 0.5) * 0.1
    ds = Dataset("synthetic")
    for j in range(n_features):
        ds.add_float_column(f"f{j}", x[:, j].copy())
    ds.add_float_column("target", y.astype(np.float32))
    return ds


# ------------------------------------------------------------------ builder
class DatasetBuilder:
    def __init__(self, name: str):
        self.name = name
        self.float_columns: Dict[str, List[float]] = {}
        self.text_columns: Dict[str, List[str]] = {}
        self.num_rows = 0

    @staticmethod
    def new(name: str) -> "DatasetBuilder":
        return DatasetBuilder(name)

    def add_float_row(self, features: Sequence[float], label: float) -> "DatasetBuilder":
        for i, v in enumerate(features):
            self.float_columns.setdefault(f"f{i}", []).append(float(v))
        self.float_columns.setdefault("label", []).append(float(label))
        self.num_rows += 1
        return self

    def add_text_row(self, text: str, label: str) -> "DatasetBuilder":
        self.text_columns.setdefault("text", []).append(text)
        self.text_columns.setdefault("label", []).append(label)
        self.num_rows += 1
        return self

    def add_float_column(self, name: str, data) -> "DatasetBuilder":
        self.num_rows = max(self.num_rows, len(data))
        self.float_columns[name] = [float(v) for v in data]
        return self

    def add_text_column(self, name: str, data) -> "DatasetBuilder":
        self.num_rows = max(self.num_rows, len(data))
        self.text_columns[name] = list(data)
        return self

    def build(self) -> Dataset:
        ds = Dataset(self.name)
        ds.num_rows = self.num_rows
        for n, d in self.float_columns.items():
            ds.add_float_column(n, d)
        for n, d in self.text_columns.items():
            ds.add_text_column(n, d)
        return ds

    def build_csv(self, path: str) -> None:
        headers = list(self.float_columns) + list(self.text_columns)
        lines = [",".join(headers)]
        for r in range(self.num_rows):
            fields = []
            for h in headers:
                if h in self.float_columns:
                    col = self.float_columns[h]
                    v = col[r] if r < len(col) else 0.0
                    fields.append(str(int(v)) if float(v).is_integer() else repr(float(v)))
                else:
                    col = self.text_columns[h]
                    fields.append('"' + (col[r] if r < len(col) else "") + '"')
            lines.append(",".join(fields))
        with open(path, "w", encoding="utf-8") as f:
            f.write("\n".join(lines) + "\n")


# ------------------------------------------------------------------ credentials and remote catalogues
@dataclasses.dataclass
class Credentials:
    hf_token: Optional[str] = None
    kaggle_username: Optional[str] = None
    kaggle_key: Optional[str] = None

    @staticmethod
    def new() -> "Credentials":
        return Credentials()

    @staticmethod
    def from_env() -> "Credentials":
        e = os.environ
        return Credentials(e.get("HF_TOKEN") or e.get("HUGGING_FACE_HUB_TOKEN"), e.get("KAGGLE_USERNAME"), e.get("KAGGLE_KEY"))

    def with_hf_token(self, token: str) -> "Credentials":
        self.hf_token = token
        return self

    def with_kaggle(self, username: str, key: str) -> "Credentials":
        self.kaggle_username, self.kaggle_key = username, key
        return self

    def has_hf(self) -> bool:
        return self.hf_token is not None

    def has_kaggle(self) -> bool:
        return self.kaggle_username is not None and self.kaggle_key is not None

    @staticmethod
    def _path() -> str:
        return os.path.join(os.environ.get("HOME", "."), ".rust-nn", "credentials.toml")

    def save(self) -> None:
        p = self._path()
        os.makedirs(os.path.dirname(p), exist_ok=True)
        s = ""
        if self.hf_token is not None:
            s += f'[huggingface]\ntoken = "{self.hf_token}"\n'
        if self.has_kaggle():
            s += f'[kaggle]\nusername = "{self.kaggle_username}"\nkey = "{self.kaggle_key}"\n'
        fd = os.open(p, os.O_WRONLY | os.O_CREAT | os.O_TRUNC, 0o600)
        with os.fdopen(fd, "w") as f:
            f.write(s)

    @staticmethod
    def load() -> "Credentials":
        c = Credentials.from_env()                       # environment variables take priority
        try:
            with open(Credentials._path()) as f:
                section = ""
                for line in f:
                    line = line.strip()
                    if line.startswith("[") and line.endswith("]"):
                        section = line[1:-1]
                    elif "=" in line:
                        k, v = line.split("=", 1)
                        k, v = k.strip(), v.strip().strip('"')
                        if (section, k) == ("huggingface", "token") and c.hf_token is None:
                            c.hf_token = v
                        elif (section, k) == ("kaggle", "username") and c.kaggle_username is None:
                            c.kaggle_username = v
                        elif (section, k) == ("kaggle", "key") and c.kaggle_key is None:
                            c.kaggle_key = v
        except OSError:
            pass
        return c


@dataclasses.dataclass
class DatasetListing:
    id: str
    description: str = ""
    downloads: int = 0
    tags: List[str] = dataclasses.field(default_factory=list)


def format_listings(listings: Sequence[DatasetListing]) -> str:
    if not listings:
        return "No datasets found."
    out = f"Found {len(listings)} datasets:\n\n"
    for i, d in enumerate(listings):
        out += f"  {i + 1}. {d.id}\n"
        if d.description:
            out += f"     {d.description[:80]}...\n"
        if d.downloads > 0:
            out += f"     Downloads: {d.downloads}\n"
        out += "\n"
    return out


HF_BASE = "https://datasets-server.huggingface.co"


def cache_dir() -> str:
    return os.path.join(os.environ.get("HOME", "."), ".cache", "rust-nn", "datasets")


def _http_get(url: str, headers: Dict[str, str], timeout: float = 20.0) -> str:
    try:
        req = urllib.request.Request(url, headers=headers)
        with urllib.request.urlopen(req, timeout=timeout) as r:
            return r.read().decode("utf-8", errors="replace")
    except (urllib.error.URLError, OSError, ValueError) as e:
        raise DataError(f"HTTP request failed: {e}") from e


def dataset_to_cache_json(ds: Dataset) -> str:
    cols = {n: (c.data.tolist() if c.numeric else c.data) for n, c in ds.columns.items()}
    return json.dumps({"num_rows": ds.num_rows, "float_columns": {n: v for n, v in cols.items() if ds.columns[n].numeric},
                       "text_columns": {n: v for n, v in cols.items() if not ds.columns[n].numeric}})


def dataset_from_cache_json(text: str, source: str) -> Dataset:
    try:
        obj = json.loads(text)
    except json.JSONDecodeError as e:
        raise DataError(f"corrupt dataset cache: {e}") from e
    ds = Dataset(source)
    for n, v in obj.get("float_columns", {}).items():
        ds.add_float_column(n, v)
    for n, v in obj.get("text_columns", {}).items():
        ds.add_text_column(n, v)
    ds.num_rows = max(ds.num_rows, int(obj.get("num_rows", 0)))
    return ds


def extract_rows_from_hf_json(body: str) -> List[Dict[str, str]]:
    """Rows of a datasets-server `/rows` reply: every `"row": {...}` object, values as strings."""
    try:
        obj = json.loads(body)
        return [{k: (v if isinstance(v, str) else json.dumps(v)) for k, v in r.get("row", {}).items()} for r in obj.get("rows", [])]
    except (json.JSONDecodeError, AttributeError):
        return []


def load_huggingface(dataset: str, split: str = "train", max_rows: int = 100, creds: Optional[Credentials] = None) -> Dataset:
    cache = os.path.join(cache_dir(), f"{dataset.replace('/', '_')}_{split}.json")
    if os.path.exists(cache):
        with open(cache) as f:
            return dataset_from_cache_json(f.read(), f"hf:{dataset}")
    headers = {"Authorization": f"Bearer {creds.hf_token}"} if creds is not None and creds.has_hf() else {}
    url = f"{HF_BASE}/rows?dataset={urllib.parse.quote(dataset, safe='')}&config=default&split={split}&offset=0&length={min(max_rows, 100)}"
    rows = extract_rows_from_hf_json(_http_get(url, headers))
    if not rows:
        raise DataError(f"no rows returned for dataset '{dataset}'")
    ds = Dataset(f"hf:{dataset}")
    for k in rows[0]:
        vals = [r.get(k, "") for r in rows]
        try:
            ds.add_float_column(k, [float(v) for v in vals])
        except ValueError:
            ds.add_text_column(k, vals)
    os.makedirs(cache_dir(), exist_ok=True)
    with open(cache, "w") as f:
        f.write(dataset_to_cache_json(ds))
    return ds


def load_huggingface_auth(dataset: str, split: str, max_rows: int, creds: Credentials) -> Dataset:
    return load_huggingface(dataset, split, max_rows, creds)


def load_kaggle(dataset: str, file: str, creds: Optional[Credentials] = None) -> Dataset:
    creds = creds or Credentials.load()
    cached = os.path.join(cache_dir(), "kaggle", dataset.replace("/", "_"), file)
    if os.path.exists(cached):
        return load_csv(cached)
    if not creds.has_kaggle():
        raise DataError("Kaggle credentials missing: set KAGGLE_USERNAME and KAGGLE_KEY")
    auth = base64_encode(f"{creds.kaggle_username}:{creds.kaggle_key}")
    _http_get(f"https://www.kaggle.com/api/v1/datasets/download/{dataset}/{file}", {"Authorization": f"Basic {auth}"})
    raise DataError(f"Kaggle dataset downloaded but needs ZIP extraction for '{file}'. Extract manually and use load_csv() on the extracted file.")


def load_kaggle_auth(dataset: str, file: str, creds: Credentials) -> Dataset:
    return load_kaggle(dataset, file, creds)


def search_huggingface(query: str, limit: int, creds: Optional[Credentials] = None) -> List[DatasetListing]:
    headers = {"Authorization": f"Bearer {creds.hf_token}"} if creds is not None and creds.has_hf() else {}
    body = _http_get(f"https://huggingface.co/api/datasets?search={urllib.parse.quote(query)}&limit={limit}", headers)
    out = []
    for o in split_json_objects(body):
        try:
            d = json.loads(o)
            out.append(DatasetListing(d.get("id", ""), d.get("description", "") or "", int(d.get("downloads", 0) or 0), list(d.get("tags", []) or [])))
        except (json.JSONDecodeError, TypeError, ValueError):
            continue
    return out[:limit]


def search_kaggle(query: str, limit: int, creds: Optional[Credentials] = None) -> List[DatasetListing]:
    creds = creds or Credentials.load()
    if not creds.has_kaggle():
        raise DataError("Kaggle credentials missing: set KAGGLE_USERNAME and KAGGLE_KEY")
    auth = base64_encode(f"{creds.kaggle_username}:{creds.kaggle_key}")
    body = _http_get(f"https://www.kaggle.com/api/v1/datasets/list?search={urllib.parse.quote(query)}", {"Authorization": f"Basic {auth}"})
    out = []
    for o in split_json_objects(body):
        try:
            d = json.loads(o)
            out.append(DatasetListing(d.get("ref", ""), d.get("title", "") or "", int(d.get("downloadCount", 0) or 0), []))
        except (json.JSONDecodeError, TypeError, ValueError):
            continue
    return out[:limit]
