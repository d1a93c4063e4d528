"""Operation factories of opset13: the operations that exist in that set, each in the version it has there."""
from .opset import export_versioned as _export

_export(globals(), 13)
