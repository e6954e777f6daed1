"""Launch, timing and monitoring helpers."""
