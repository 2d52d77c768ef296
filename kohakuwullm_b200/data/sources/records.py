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
            # several ranks may get here at once: each builds the (identical) manifest for itself and publishes it
            # with an atomic rename, so no reader ever sees a half-written file
            self.manifest = self.build_manifest(root)
            tmp = f"{path}.{os.getpid()}.tmp"
            with open(tmp, "w") as f:
                json.dump(self.manifest, f)
            os.replace(tmp, path)
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


@DATASET.register("mixture")
class MixtureRecords:
    """Several sources as one random-access sequence, each repeated ``repeat`` times (the mixture weights of a
    run). ``sources``: a list of ``{"records": <spec or instance>, "repeat": 1.0, "source": "tag"}``. An integer
    part of ``repeat`` gives whole copies; a fractional part gives a fixed pseudo-random subset of that share
    (a Feistel permutation of the source, seeded, so the subset does not depend on the epoch or the rank).
    Dict records get a ``"source"`` field (kept if they already have one): the per-source renderer keys on it."""

    def __init__(self, sources, seed: int = 0, **_unused):
        from kohakuwullm_b200.data.loader.permute import FeistelPermutation, splitmix64
        from kohakuwullm_b200.registry import build

        self.parts = []
        self._starts = [0]
        for i, spec in enumerate(sources):
            spec = dict(spec)
            recs = spec.pop("records")
            if isinstance(recs, (str, dict)):
                recs = build(recs, DATASET)
            repeat = float(spec.pop("repeat", 1.0))
            tag = spec.pop("source", None) or getattr(recs, "name", None) or f"source{i}"
            n = len(recs)
            total = int(n * repeat + 1e-9)
            perm = FeistelPermutation(n, splitmix64(seed * 1000003 + i)) if (total % n and n > 1) else None
            self.parts.append((recs, n, total, perm, tag))
            self._starts.append(self._starts[-1] + total)

    def __len__(self) -> int:
        return self._starts[-1]

    def __getitem__(self, i: int):
        if not 0 <= i < len(self):
            raise IndexError(i)
        s = bisect_right(self._starts, i) - 1
        recs, n, total, perm, tag = self.parts[s]
        j = i - self._starts[s]
        whole = (total // n) * n
        local = j % n if j < whole else perm(j - whole)       # the fractional tail: a fixed subset
        rec = recs[local]
        if isinstance(rec, dict) and "source" not in rec:
            rec = dict(rec, source=tag)
        return rec

    def composition(self) -> dict:
        """Records per source after repetition (what the mixture really is)."""
        return {tag: total for _, _, total, _, tag in self.parts}


@DATASET.register("split")
class SplitRecords:
    """The training or the validation part of a source: record ``i`` is validation when a hash of ``(seed, i)``
    falls under ``fraction`` (the split does not depend on epoch, rank or world size)."""

    def __init__(self, records, fraction: float, part: str = "train", seed: int = 0, **_unused):
        from kohakuwullm_b200.data.loader.permute import is_validation
        from kohakuwullm_b200.registry import build

        if part not in ("train", "val"):
            raise ValueError(f"part must be 'train' or 'val', not {part!r}")
        self.records = build(records, DATASET) if isinstance(records, (str, dict)) else records
        want_val = part == "val"
        self.index = [i for i in range(len(self.records)) if is_validation(i, fraction, seed) == want_val]

    def __len__(self) -> int:
        return len(self.index)

    def __getitem__(self, i: int):
        return self.records[self.index[i]]
