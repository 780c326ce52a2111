"""numpy struct dtypes of the original (pre device-resident) write / query rings
(src/chaoscontrol/episodic/payload_dtypes.py:29-67); kept for tools and tests that
still speak that contract."""
from __future__ import annotations

import numpy as np

__all__ = ["make_write_payload_dtype", "make_query_candidate_dtype"]


def make_write_payload_dtype(*, span_length: int, key_rep_dim: int) -> np.dtype:
    if span_length <= 0:
        raise ValueError(f"span_length must be positive; got {span_length}")
    if key_rep_dim <= 0:
        raise ValueError(f"key_rep_dim must be positive; got {key_rep_dim}")
    return np.dtype([("key_fp", np.int64), ("key_rep", np.float32, (key_rep_dim,)),
                     ("value_tok_ids", np.int64, (span_length,)), ("value_anchor_id", np.int64)])


def make_query_candidate_dtype(*, key_rep_dim: int) -> np.dtype:
    if key_rep_dim <= 0:
        raise ValueError(f"key_rep_dim must be positive; got {key_rep_dim}")
    return np.dtype([("batch_index", np.int64), ("position", np.int64), ("pressure", np.float32),
                     ("residual", np.float32, (key_rep_dim,))])
