"""Utilities: logging, metrics, safetensors IO, tensor comparison, MFU, NVTX ranges, debug switches."""
