"""Small helpers shared by the package: Chrome-trace spans and NVTX ranges."""
