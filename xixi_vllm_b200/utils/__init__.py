"""Support utilities: CLI helpers, metrics, device timers, NVTX ranges."""
