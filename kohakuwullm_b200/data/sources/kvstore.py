"""A single-file key-value store and the record sources built on it.

The reference keeps its corpora and caption / tag databases in ``kohakuvault`` stores
(src/kohakuwullm/data/sources/vault.py:42-314, corpus.py:18-168). That package is not part of this framework, so
the same contract is carried by a store of its own:

``KVWriter`` / ``KVFile``  one file = a data region of values followed by an index of (key, offset, length, kind)
    sorted by key and a 24-byte footer. Keys are bytes; values are bytes, UTF-8 text or JSON documents. Reading
    maps the file, looks the key up by binary search and decodes lazily; handles are per process (a forked loader
    worker reopens the file instead of sharing a descriptor).
``VaultCorpusRecords``     text or conversation corpora: shards ``<root>/<name>/*.kv`` whose keys are sequential
    big-endian int64 ids. The shard sizes seen at construction are the SNAPSHOT a resumed run must find again.
``TagRecords``             image-board style metadata keyed by post id, optionally joined with a caption store
    keyed by image path; yields one normalised record shape (tags per category, rating, score -> quality word,
    size, year, short / long caption) that the TIPO renderer consumes.
"""

from __future__ import annotations

import json
import mmap
import os
import struct
from bisect import bisect_right
from typing import Iterator, Sequence

from kohakuwullm_b200.registry import DATASET

MAGIC = b"KWUKV1\x00\x00"
KIND_BYTES, KIND_TEXT, KIND_JSON = 0, 1, 2
_FOOTER = struct.Struct("<QQ8s")      # index offset, number of keys, magic


class KVWriter:
    """``with KVWriter(path) as w: w.put(key, value)``. Keys may arrive in any order; a repeated key keeps the
    last value. Nothing is readable before ``close``."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path + ".tmp", "wb")
        self._f.write(MAGIC)
        self._index: dict[bytes, tuple[int, int, int]] = {}

    def put(self, key: bytes | str | int, value) -> None:
        key = encode_key(key)
        if isinstance(value, (bytes, bytearray, memoryview)):
            kind, raw = KIND_BYTES, bytes(value)
        elif isinstance(value, str):
            kind, raw = KIND_TEXT, value.encode("utf-8")
        else:
            kind, raw = KIND_JSON, json.dumps(value, ensure_ascii=False, separators=(",", ":")).encode("utf-8")
        self._index[key] = (self._f.tell(), len(raw), kind)
        self._f.write(raw)

    def close(self) -> None:
        if self._f is None:
            return
        start = self._f.tell()
        for key in sorted(self._index):
            off, length, kind = self._index[key]
            self._f.write(struct.pack("<HQIB", len(key), off, length, kind))
            self._f.write(key)
        self._f.write(_FOOTER.pack(start, len(self._index), MAGIC))
        self._f.close()
        self._f = None
        os.replace(self.path + ".tmp", self.path)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def encode_key(key: bytes | str | int) -> bytes:
    if isinstance(key, int):
        return struct.pack(">q", key)          # sequential ids sort numerically as bytes
    return key.encode("utf-8") if isinstance(key, str) else bytes(key)


class KVFile:
    def __init__(self, path: str):
        self.path = path
        self._pid = -1
        self._map = None
        self._keys: list[bytes] = []
        self._where: list[tuple[int, int, int]] = []
        self._open()

    def _open(self) -> None:
        with open(self.path, "rb") as f:
            self._map = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        m = self._map
        if len(m) < len(MAGIC) + _FOOTER.size or m[:8] != MAGIC:
            raise ValueError(f"{self.path} is not a key-value store of this framework (or was cut short)")
        start, count, magic = _FOOTER.unpack(m[-_FOOTER.size:])
        if magic != MAGIC or start > len(m):
            raise ValueError(f"{self.path}: damaged footer")
        if not self._keys:
            pos = start
            for _ in range(count):
                klen, off, length, kind = struct.unpack_from("<HQIB", m, pos)
                pos += 15
                self._keys.append(bytes(m[pos:pos + klen]))
                self._where.append((off, length, kind))
                pos += klen
        self._pid = os.getpid()

    def _mapped(self):
        if self._pid != os.getpid():       # forked: a mapping of one's own
            self._open()
        return self._map

    def __len__(self) -> int:
        return len(self._keys)

    def keys(self) -> list[bytes]:
        return self._keys

    def get(self, key, default=None):
        key = encode_key(key)
        i = bisect_right(self._keys, key) - 1
        if i < 0 or self._keys[i] != key:
            return default
        return self.value_at(i)

    def value_at(self, i: int):
        off, length, kind = self._where[i]
        raw = self._mapped()[off:off + length]
        if kind == KIND_BYTES:
            return bytes(raw)
        text = bytes(raw).decode("utf-8")
        return text if kind == KIND_TEXT else json.loads(text)

    def items(self) -> Iterator[tuple[bytes, object]]:
        for i, k in enumerate(self._keys):
            yield k, self.value_at(i)

    def __getstate__(self):
        return {"path": self.path}

    def __setstate__(self, state):
        self.__init__(state["path"])


def shard_paths(name: str, root: str) -> list[str]:
    d = os.path.join(root, name)
    return sorted(os.path.join(d, f) for f in os.listdir(d) if f.endswith(".kv"))


@DATASET.register("vault_corpus")
class VaultCorpusRecords:
    """``schema="text"``: values are document text -> ``{"text": ...}``; ``schema="json"``: values are JSON
    documents (``{"messages": [...]}`` for conversations), returned as they are."""

    def __init__(self, corpus: str, root: str, schema: str = "text", snapshot: Sequence[int] | None = None, **_unused):
        if schema not in ("text", "json"):
            raise ValueError(f"schema must be 'text' or 'json', not {schema!r}")
        name = corpus
        self.name, self.root, self.schema = name, root, schema
        self.shards = [KVFile(p) for p in shard_paths(name, root)]
        if not self.shards:
            raise FileNotFoundError(f"no .kv shards under {os.path.join(root, name)}")
        sizes = [len(s) for s in self.shards]
        if snapshot is not None and list(snapshot) != sizes:
            raise ValueError(f"corpus {name!r} changed since the run started: shard sizes {sizes}, snapshot {list(snapshot)}")
        self._starts = [0]
        for n in sizes:
            self._starts.append(self._starts[-1] + n)

    def snapshot(self) -> list[int]:
        return [len(s) for s in self.shards]

    def __len__(self) -> int:
        return self._starts[-1]

    def __getitem__(self, i: int):
        if not 0 <= i < len(self):
            raise IndexError(i)
        s = bisect_right(self._starts, i) - 1
        value = self.shards[s].value_at(i - self._starts[s])
        if self.schema == "text":
            return {"text": value if isinstance(value, str) else bytes(value).decode("utf-8", "replace"), "source": self.name}
        if isinstance(value, (str, bytes, bytearray)):
            value = json.loads(value)          # a store whose writer kept the documents as JSON text
        return value


TAG_CATEGORIES = ("general", "artist", "character", "copyright", "meta")
# score -> quality word; here and not baked into the stored records, so it stays a knob
QUALITY_THRESHOLDS = ((150, "masterpiece"), (100, "best quality"), (75, "great quality"), (50, "good quality"),
                      (25, "normal quality"), (10, "below average quality"), (0, "low quality"))


def quality_of(score: int | None) -> str | None:
    if score is None:
        return None
    for low, word in QUALITY_THRESHOLDS:
        if score >= low:
            return word
    return "worst quality"


@DATASET.register("tag_records")
class TagRecords:
    """Ground-truth post metadata (``meta`` store keyed by the 8-digit post id), optionally joined with a caption
    store keyed by image path (``caption_key`` formats the path from the id). ``image_only`` keeps posts whose
    metadata says ``has_image``. A post without a caption is tag-only data, not a missing record."""

    def __init__(self, meta: str, captions: str | None = None, caption_key: str = "{id}.webp", ids: Sequence[int] | None = None,
                 image_only: bool = False, source: str = "danbooru", **_unused):
        self.meta = KVFile(meta)
        self.cap = KVFile(captions) if captions and os.path.exists(captions) else None
        self.caption_key, self.source = caption_key, source
        self.ids = [int(i) for i in ids] if ids is not None else [int(k.decode()) for k in self.meta.keys()]
        if image_only:
            self.ids = [i for i in self.ids if (self.meta.get(f"{i:08d}") or {}).get("has_image")]

    def __len__(self) -> int:
        return len(self.ids)

    def get(self, post_id: int) -> dict | None:
        m = self.meta.get(f"{int(post_id):08d}")
        if m is None:
            return None
        rec = {"source": self.source, "id": m.get("id", post_id), "key": f"{int(post_id):08d}", "short": None, "long": None,
               "title": None}
        for cat in TAG_CATEGORIES:
            rec[cat] = list(m.get(cat) or [])
        rec["tags"] = rec["general"] + rec["character"] + rec["copyright"]
        rec["rating"] = m.get("rating")
        rec["score"] = m.get("score")
        rec["quality"] = quality_of(m.get("score"))
        for k in ("width", "height", "year"):
            rec[k] = m.get(k)
        if rec["width"] and rec["height"]:
            rec["aspect_ratio"] = round(rec["width"] / rec["height"], 2)
        if rec["artist"]:
            rec["artist"] = ", ".join(rec["artist"])
        rec["characters"] = ", ".join(rec["character"]) or None
        if self.cap is not None:
            c = self.cap.get(self.caption_key.format(id=int(post_id)))
            if c:
                rec["short"], rec["long"], rec["title"] = c.get("brief") or None, c.get("description") or None, c.get("title") or None
                rec["caption"], rec["short_caption"] = rec["long"] or "", rec["short"] or ""
        return rec

    def __getitem__(self, index: int) -> dict | None:
        return self.get(self.ids[index])
