"""The caption corpora of the prompt-optimisation recipes, shared by the configs of this folder.

Two kinds of source, both under ``CAPTION_ROOT`` (override with ``KWU_CAPTION_ROOT``): tag-list posts in key-value
stores (``<name>/meta.kv`` + ``<name>/captions.kv``, read by ``tag_records``) and caption-only sets as jsonl shards
(``<name>/``, read by ``corpus``). The tag-heavy sources repeat because the renderer draws a different task, length
bucket and tag order on every pass: a repeat is a re-render, not a duplicate.
"""

import os

CAPTION_ROOT = os.environ.get("KWU_CAPTION_ROOT", "data/captions")

TAGGED = {"danbooru": 3, "danbooru_tagger": 2}
CAPTIONED = {"coyo11m": 1, "laion_coco": 1, "cc12m": 1, "nozomi": 1}


def caption_sources(names=None):
    out = []
    for name, repeat in {**TAGGED, **CAPTIONED}.items():
        if names and name not in names:
            continue
        root = os.path.join(CAPTION_ROOT, name)
        if name in TAGGED:
            records = {"name": "tag_records", "meta": os.path.join(root, "meta.kv"),
                       "captions": os.path.join(root, "captions.kv"), "source": name}
        else:
            records = {"name": "corpus", "root": root, "text_field": "caption"}
        out.append({"records": records, "repeat": repeat, "source": name})
    return out
