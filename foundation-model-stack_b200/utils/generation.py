"""``from fms_b200.utils.generation import generate, pad_input_ids`` — the reference's import path
(fms/utils/generation.py)."""
from ..engine.generation import (generate, generate_batch, pad_input_ids, plan_batches, trim_prefix,
                                 truncate_after_eos)

__all__ = ["generate", "generate_batch", "pad_input_ids", "plan_batches", "trim_prefix", "truncate_after_eos"]
