"""Import location kept for callers of the reference layout
(src/chaoscontrol/optim/episodic_writer.py); the functions live in ``episodic.writer``."""
from ..episodic.writer import *  # noqa: F401,F403
from ..episodic.writer import (_next_admission_trace_seq, _reserve_admission_trace_seq,  # noqa: F401
                               _reset_admission_trace_seq)
