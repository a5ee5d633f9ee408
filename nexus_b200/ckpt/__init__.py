from .checkpoint import (CheckpointError, CheckpointManager, CheckpointOptions, LoadedCheckpoint,  # noqa: F401
                         TrainerState, trailer_hex)
