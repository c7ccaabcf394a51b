"""Llama-3 configuration, weights and the plain PyTorch forward used as the numerical oracle."""
