from .language import LanguageTrainer, TokenRows  # noqa: F401
from .lm_trainer import (AdamW, ArrayTokens, LanguageModelTrainer, LanguageTrainerBuilder, LmBackend, LmParamInfo,  # noqa: F401
                         LmStepResult, NanOptions, ParamGroupPolicy, ParamGroupRule, ShardTokens, SpikeOptions, StepRecord,
                         SyntheticTokens, TokenSource, TrainSummary)
from .loggers import (ConsoleLogger, CsvLogger, JsonlLogger, TensorBoardLogger, WandbOfflineLogger,  # noqa: F401
                      read_tensorboard_scalars)
from .schedule import ConstantLr, InverseSqrt, LinearLr, LrSchedule, WarmupCosine, WSD  # noqa: F401
from .trainer import EpochStats, LossScaler, Trainer, TrainerBuilder  # noqa: F401
from . import callbacks  # noqa: F401
from .distributed import (DataParallelStep, DataParallelTrainer, LoopProfile, all_reduce_mean,  # noqa: F401
                          allreduce_mean_gradients, broadcast_parameters)
