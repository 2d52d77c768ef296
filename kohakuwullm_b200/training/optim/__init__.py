from kohakuwullm_b200.training.optim.adamw16 import AdamW16  # noqa: F401
from kohakuwullm_b200.training.optim.build import build_optimizer, group_parameters  # noqa: F401
from kohakuwullm_b200.training.optim.fused_adamw import FlatAdamW  # noqa: F401
from kohakuwullm_b200.training.optim.lowbit import KEEP_FP32_DEFAULT, cast_parameters_  # noqa: F401
from kohakuwullm_b200.training.optim.lowbit_optim import StochasticAdamW  # noqa: F401
from kohakuwullm_b200.training.optim.muon import MuonW, newton_schulz  # noqa: F401
from kohakuwullm_b200.training.optim.torch_fused import FusedAdamW  # noqa: F401
