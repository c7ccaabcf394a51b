"""The native serving engines (CUDA and oracle), the model runner, and the engine loop."""
