"""Peer-memory communication: symmetric buffers over NVLink and the fused compute+collective kernels."""
