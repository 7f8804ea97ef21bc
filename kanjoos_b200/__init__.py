"""kanjoos_b200 -- B200-native quantized (GGUF Q4_K) MoE expert path behind the
Kanjoos device/kernel API. The compute lives in the CUDA library built from
kanjoos_b200/csrc (C-ABI declared in include/knj_device.h); this package is the
host-side mirror used by tests and the benchmark."""
__all__ = ["synth"]
