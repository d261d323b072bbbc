"""The trace builders and the reader of results that the replay tests use: the package's own
(``infinicore_infer_b200.traces``), which ``bin/trace_make`` and ``bin/trace_compare`` serve from the command line."""
from infinicore_infer_b200.traces import (by_position, compare, mixed, peak_tokens, portions, read_results,  # noqa: F401
                                          staggered_plan, tail_decode, whole)
