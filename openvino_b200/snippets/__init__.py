"""Snippets: groups of element-wise operations (with Softmax / reductions over the innermost axis) become one
``Subgraph`` operation each, lowered to a linear IR with an explicit loop structure and emitted as one CUDA kernel for
sm_100a (built with nvcc when the model is compiled, cached by the hash of the kernel text) or run by a NumPy executor
on the host.

* ``tokenizer.tokenize(model)``   - graph pass that forms the Subgraph nodes;
* ``lowered.lower(body, kinds)``  - linear IR, stages / loops, register assignment;
* ``emit_cuda.CudaKernel``        - kernel text, build, launch;
* ``emit_numpy.run_numpy``        - host executor of the same linear IR;
* ``runtime.run_subgraph``        - what the CUDA device calls for a Subgraph node.

The CUDA device tokenises when ``SNIPPETS_MODE`` is ``ENABLE`` (default ``DISABLE``). Reference: src/common/snippets.
"""
from .tokenizer import SnippetBody, body_of, classify, ensure_registered, tokenize   # noqa: F401
from .lowered import LinearIR, lower   # noqa: F401
