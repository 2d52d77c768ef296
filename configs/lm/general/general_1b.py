"""General-language + prompt-optimisation pretraining of Kohaku-MoE-1B: 400k steps of 262144 tokens (~105 B tokens),
8 pipeline stages on one node.

    torchrun --nproc-per-node 8 -m kohakuwullm_b200.cli.train_lm_pipe --config configs/lm/general/general_1b.py
    # ten steps without data or network:
    python -m kohakuwullm_b200.cli.train_lm_pipe --config configs/lm/general/general_1b.py \
        --set MAX_STEPS=10 --set CKPT_EVERY=0 --set SAMPLE_INTERVAL=0 --set SOURCES=[] --set DATA="'synthetic'"

Mixture weights come from ``python -m kohakuwullm_b200.cli.data_tools mixture`` at a 4096-token context; the question
/ answer and chat sources render as ChatML with the user turns masked, so roughly a tenth of the run carries turn
structure. Each source names its own renderer through the per-source renderer; text roots are under ``KWU_TEXT_ROOT``
(default ``data/text``), caption roots under ``KWU_CAPTION_ROOT``.
"""

import os
import runpy

_text_root = os.environ.get("KWU_TEXT_ROOT", "data/text")
_cap = runpy.run_path(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "tipo", "_sources.py"))

_TEXT = [            # (corpus, repeat, renderer)
    ("en/web-hq", 1.000, "plain"),
    ("en/web-hq-synthetic", 0.270, "plain"),
    ("en/web-mhq", 1.000, "plain"),
    ("ja/web-edu", 0.560, "plain"),
    ("zh-tw/pdfs", 0.576, "plain"),
    ("zh-tw/web", 1.000, "plain"),
    ("zh-tw/wiki", 1.000, "plain"),
    ("zh-tw/forum", 1.000, "plain"),
    ("ko/web", 0.130, "plain"),
    ("en/web-hq-qa", 0.966, "qa_chatml"),
    ("stem/specialized", 1.000, "qa_chatml"),
    ("sft/chat", 1.000, "chat"),
]

SOURCES = [{"records": {"name": "vault_corpus", "root": _text_root, "corpus": name,
                        "schema": "json" if kind in ("chat", "qa_chatml") else "text"}, "repeat": repeat, "source": name}
           for name, repeat, kind in _TEXT] + _cap["caption_sources"](("danbooru", "coyo11m", "laion_coco"))
RENDERER = {"name": "per_source", "default": "plain",
            "renderers": {**{name: kind for name, _, kind in _TEXT},
                          **{name: "tipo" for name in ("danbooru", "coyo11m", "laion_coco")}}}
TOKENIZER = "models/tokenizer"
CTX_MAX = 4096

PRESET = "Kohaku-MoE-1B"
ARCH_OVERRIDES = {"max_position": 4096, "rope_theta": 100000.0, "qk_norm": True, "tie_embeddings": False, "mxfp8": True}
AUX_LOSS_WEIGHT = 0.0
ROUTER_Z_LOSS_WEIGHT = 0.0

GPUS = 8
MICRO_TOKENS = 8192
NUM_MICROBATCHES = 32
SCHEDULE = "1f1b"
AUTOTUNE = True

OPTIMIZER = "muon"
OPTIMIZER_KWARGS = {"muon_lr": 2e-3, "embed_lr": 2e-3}
LR = 5e-4
WEIGHT_DECAY = 0.1
MAX_GRAD_NORM = 1.0
MAX_STEPS = 400_000
WARMUP_STEPS = 2000
# inverse-square-root decay for nine tenths of the run, then a cosine tail from wherever that ended
LR_SCHEDULE = {"phases": [{"mode": "power", "end": 0.9, "s0": 2500, "b": -0.5, "warmup": None},
                          {"mode": "cosine", "end": 1.0, "min_value": 0.01}], "end": None}
SEED = 20090220

RUN_NAME = "general-1b-400k"
WANDB_PROJECT = "kohakuwullm-b200"
LOG_INTERVAL = 20
CKPT_DIR = "out/ckpt/general-1b-400k"
CKPT_EVERY = 2000
SAMPLE_INTERVAL = 2000
SAMPLE_PROMPTS = [("story", "Once upon a time"), ("qa", "<|im_start|>user\nWhy is the sky blue?<|im_end|>\n<|im_start|>assistant\n")]
SAMPLE_TOKENS = 256
SAMPLE_TEMPERATURE = 1.0
SAMPLE_TOP_P = 1.0
