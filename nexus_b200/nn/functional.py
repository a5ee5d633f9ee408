"""`nn.functional`: stateless forms of the catalog operators (all routed through the fused ops)."""
from torch.nn.functional import (avg_pool2d, conv1d, conv2d, conv3d, elu, gelu, leaky_relu, max_pool2d, mish,  # noqa: F401
                                 relu, sigmoid, silu, softplus, tanh)

from ..fused.ops import (attention, cross_entropy, cross_entropy_shifted, dropout_philox, embedding_pos,  # noqa: F401
                         fused_layernorm as layer_norm, fused_linear as linear, fused_softmax as softmax, rms_norm)
