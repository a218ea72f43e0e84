"""Multimodal path: canvases and salted placeholders (front-end side), vision towers, row injection (engine side)."""
