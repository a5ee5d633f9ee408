from .config import (LmConfig, RopeScaling, apply_overrides, count_active_parameters, count_parameters,  # noqa: F401
                     from_json, preset, preset_names, to_json, validate)
from .model import AdamW, KvCache, LanguageModel, build  # noqa: F401
from .rope import RopeCache, alibi_slopes, apply_rope, rope_inv_freq  # noqa: F401
