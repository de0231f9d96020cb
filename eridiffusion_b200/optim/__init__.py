from .arena import ParamArena  # noqa: F401
from .adamw8bit import AdamW8bit, quantize_m, quantize_v, dequantize_m, dequantize_v  # noqa: F401
from .optimizers import (AdamWArena, Lion, Adafactor, Prodigy, RAdamScheduleFree,  # noqa: F401
                         CPUOffloadedAdamW, MultiOptimizer, create_optimizer, clip_grad_norm_,
                         split_weight_decay)
from .schedulers import LRSchedule, ChainedSchedule, ReduceLROnPlateau, GradScaler, EMA, EMAContext  # noqa: F401
