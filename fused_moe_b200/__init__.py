"""B200-native DeepSeek-V3 FP8 block-scale fused MoE layer: ``fused_moe_b200.kernel.kernel`` is the drop-in for the
reference's ``solution/python/kernel.py::kernel``; everything on the device runs in libb200moe.so (include/b200moe.h)."""
