"""Engine-agnostic connector halves, the RPC clients, the transfer layer and the vLLM adapter."""
