from kohakuwullm_b200.models.backbone import LMBackbone, build_block  # noqa: F401
from kohakuwullm_b200.models.block import DecoderBlock  # noqa: F401
from kohakuwullm_b200.models.cache import KVCache  # noqa: F401
from kohakuwullm_b200.models.head import LMHead  # noqa: F401
from kohakuwullm_b200.models.presets import KOHAKU_LADDER, PRESETS, LMArchConfig, get_preset  # noqa: F401
from kohakuwullm_b200.models.seqinfo import SeqInfo  # noqa: F401
