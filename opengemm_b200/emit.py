"""Standalone kernel emitter (placeholder until the emitter lands)."""


def emit_kernel(*args, **kwargs):
    raise NotImplementedError("emit_kernel is not built yet")
