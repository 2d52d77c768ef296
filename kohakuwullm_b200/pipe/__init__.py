"""``kohakuwullm_b200.pipe`` — the architecture-free pipeline engine (the role of ``kohakuwupipe``):
stage planning, schedules, step loop, loss scaling, callbacks and portable checkpoints."""

from kohakuwullm_b200.pipe.callbacks import Checkpoint, LossLog, ProgressBar, Throughput  # noqa: F401
from kohakuwullm_b200.pipe.checkpoint import gather_state_dict, load, save  # noqa: F401
from kohakuwullm_b200.pipe.distributed import PipelineRanks, init_pipeline, shutdown  # noqa: F401
from kohakuwullm_b200.pipe.hooks import Callback, CallbackList  # noqa: F401
from kohakuwullm_b200.pipe.module import PipelineModule  # noqa: F401
from kohakuwullm_b200.pipe.plan import (  # noqa: F401
    StagePlan, describe, partition, partition_v, plan_from_layers, plan_stages,
)
from kohakuwullm_b200.pipe.scaler import PipelineGradScaler  # noqa: F401
from kohakuwullm_b200.pipe.schedules import SCHEDULES  # noqa: F401
from kohakuwullm_b200.pipe.streams import GradCarrier, accumulate, accumulator, reduce_accumulator, split_streams  # noqa: F401
from kohakuwullm_b200.pipe.trainer import PipelineLoop, PipelineTrainer, StepOutput  # noqa: F401
from kohakuwullm_b200.utils.logging import configure, get_logger  # noqa: F401
