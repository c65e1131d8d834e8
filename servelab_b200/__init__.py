"""servelab_b200: a single-GPU inference engine for NVIDIA B200 (sm_100a).

Everything between a request's tokens and its next token: typed configuration
and an architecture registry (``config``), weights by tensor name
(``weights``), layers composed from registered parts (``parts``, ``models``), a
paged key/value cache with per-request state slots (``cache``), one step
function, a continuous-batching scheduler and the ``LLMEngine`` entry point
(``engine``), device sampling (``sampling``) and the hand-written CUDA kernels
(``csrc``, called through ``ops``).
"""

__version__ = "0.1.0"
