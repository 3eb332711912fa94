"""Placeholder package kept for layout parity (the reference's landmark/render/memory_manager is empty)."""
