"""illatio-b200: sm_100a kernels for illatio's quantized matvec / MoE expert path."""
from .blocks import Q8_0, Q4_K, Q6_K, Q2_K, IQ2_XXS  # noqa: F401
