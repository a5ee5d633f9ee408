from . import functional  # noqa: F401
from .graph import MERGE_ADD, MERGE_CONCAT, MERGE_SINGLE, Graph  # noqa: F401
from .modules import *  # noqa: F401,F403
from .modules import GELU, KIND, Mish, Module, SiLU, make_activation, make_one, register_activation, swish  # noqa: F401
