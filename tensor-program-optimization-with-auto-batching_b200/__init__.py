"""B200-native multi-LoRA decode path (host side)."""
