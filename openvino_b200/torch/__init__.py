"""``import openvino_b200.torch`` registers the ``torch.compile`` backends "openvino_b200" and (when the name is free)
"openvino", like ``import openvino.torch`` does in the reference (src/bindings/python/src/openvino/torch/__init__.py)."""
from ..frontend import torchdynamo as _dynamo

_dynamo.register()
