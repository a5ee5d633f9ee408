from .checkpoint import CheckpointError, CheckpointManager, CheckpointOptions, LoadedCheckpoint  # noqa: F401
