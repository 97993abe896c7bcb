"""B200 (sm_100a) Mixture-of-Experts layer behind the reference's MoELayer interface."""
from .moe_layer import MoELayer, MoeError, launch_count  # noqa: F401
