"""Model-level integration: structural patching of torch modules that carry MLX INT4 weights."""
