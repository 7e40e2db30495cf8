"""boltops_b200: B200-native fused-MoE hot path behind the BoltOPs operator API.

``boltops_b200.fused_moe`` mirrors ``boltops.fused_moe`` (``fused_experts``,
``moe_activation``, ``normalize_moe_activation``, ``moe_activation_output_size``).
All device work is hand-written sm_100a CUDA in ``libboltops_b200.so`` reached
through a C ABI (``include/boltops_b200.h``); there is no CPU fallback.
"""

__version__ = "0.1.0"
