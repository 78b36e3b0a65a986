"""A small, whole decoder-model library for one NVIDIA B200: configuration, weights, layers built
from parts, a block cache with a slot per sequence, one step function, a generation loop, sampling and
trace replay, running on hand-written sm_100a CUDA kernels.

Entry points, in the manner of ``fms.models.get_model`` and ``fms.utils.generation.generate``
(fms/models/__init__.py:298-503, fms/utils/generation.py:182-369)::

    from fms_b200.models import get_model
    from fms_b200.utils.generation import generate
"""

__version__ = "0.1.0"
