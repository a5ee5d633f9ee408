from .moe import MoEFFN, Routing, Spec, moe_forward, quantize_experts, reference, route  # noqa: F401
