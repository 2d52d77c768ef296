"""Record sources. A source is a random-access sequence of raw records (``len``, ``[i]``) that is safe to
use from forked loader workers (file handles are opened lazily per process).

``CorpusRecords``  sharded text corpora: a directory of ``*.jsonl`` / ``*.txt`` shards plus a
                   ``manifest.json`` that pins the snapshot (shard names, record counts, byte offsets),
                   so a resumed run reads exactly the corpus it started on.
``ListRecords``    in-memory records (tests, small fine-tuning sets).
``PathKeyedRecords`` records stored one JSON file per key under a root directory (caption / tag
                   datasets keyed by image path).
The reference reads these through the ``kohakuvault`` store (src/kohakuwullm/data/sources/vault.py:42-314,
corpus.py:18-168); that package is not available here, so plain files carry the same contract.
"""

from __future__ import annotations

import json
import os
from bisect import bisect_right
from typing import Sequence

from kohakuwullm_b200.registry import DATASET


@DATASET.register("list")
class ListRecords:
    def __init__(self, records: Sequence, **_unused):
        self.records = list(records)

    def __len__(self):
        return len(self.records)

    def __getitem__(self, i):
        return self.records[i]


@DATASET.register("corpus")
class CorpusRecords:
    MANIFEST = "manifest.json"

    def __init__(self, root: str, text_field: str = "text", rebuild_manifest: bool = False, **_unused):
        self.root, self.text_field = root, text_field
        path = os.path.join(root, self.MANIFEST)
        if rebuild_manifest or not os.path.exists(path):
            self.manifest = self.build_manifest(root)
            with open(path, "w") as f:
                json.dump(self.manifest, f)
        else:
            with open(path) as f:
                self.manifest = json.load(f)
        self._starts = [0]
        for shard in self.manifest["shards"]:
            self._starts.append(self._starts[-1] + shard["records"])
        self._handles: dict[tuple[int, int], object] = {}

    @staticmethod
    def build_manifest(root: str) -> dict:
        shards = []
        for name in sorted(os.listdir(root)):
            if not name.endswith((".jsonl", ".txt")):
                continue
            offsets, pos = [], 0
            with open(os.path.join(root, name), "rb") as f:
                for line in f:
                    if line.strip():
                        offsets.append(pos)
                    pos += len(line)
            shards.append({"name": name, "records": len(offsets), "offsets": offsets, "bytes": pos})
        return {"version": 1, "shards": shards}

    def __len__(self):
        return self._starts[-1]

    def _file(self, shard_index: int):
        key = (os.getpid(), shard_index)  # one handle per process: fork-safe
        if key not in self._handles:
            self._handles[key] = open(os.path.join(self.root, self.manifest["shards"][shard_index]["name"]), "rb")
        return self._handles[key]

    def __getitem__(self, i: int):
        if not 0 <= i < len(self):
            raise IndexError(i)
        s = bisect_right(self._starts, i) - 1
        shard = self.manifest["shards"][s]
        f = self._file(s)
        f.seek(shard["offsets"][i - self._starts[s]])
        line = f.readline().decode("utf-8", errors="replace").rstrip("\n")
        if shard["name"].endswith(".jsonl"):
            return json.loads(line)
        return {self.text_field: line}

    def __getstate__(self):
        state = self.__dict__.copy()
        state["_handles"] = {}
        return state


@DATASET.register("path_keyed")
class PathKeyedRecords:
    def __init__(self, root: str, index: str = "index.json", **_unused):
        self.root = root
        with open(os.path.join(root, index)) as f:
            self.keys = json.load(f)

    def __len__(self):
        return len(self.keys)

    def __getitem__(self, i):
        key = self.keys[i]
        with open(os.path.join(self.root, key + ".json")) as f:
            rec = json.load(f)
        rec.setdefault("key", key)
        return rec
