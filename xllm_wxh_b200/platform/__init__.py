"""Host-platform helpers: NUMA placement of the rank processes, CUDA stream pool.

Counterpart of the reference's `xllm/core/platform` (numa_utils.h:34-52, stream.h, device.h) for a box of B200s."""
