"""CPU restatement of the reference algorithms on the FlashMask hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in ``flashmask_b200`` imports this package;
it is the checker used by ``tests/``, by the smoke run and by the CPU-baseline
leg of ``bench.py``.  It is written in numpy / torch (CPU, fp32) and each
function cites the reference file:line it restates.

Pinning: ``tests/golden/make_golden.py`` imports the reference's own dense-mask
attention (tests/torch/attention_ref.py) and mask expander
(tests/common/startend_row_indices.py) and stores their outputs;
``tests/test_oracle_golden.py`` checks this restatement against those vectors.
The IPO partition solver is pinned against the reference's own header compiled
into ``oracle/_ref`` (see ``oracle/Makefile``).  LSE values, the tile
classification bit patterns and the heap partition are not covered by any
stored vector of the reference ("parity unpinned" for those three: the
restatements here are the pins).
"""
from .attention import (dense_bias, attention_forward, attention_forward_backward,  # noqa: F401
                        block_logit_ref, visible_block, candidate_columns, attention_rows, attention_columns)
from .tiles import (nblk_pad, scan_max_min, valid_block_count, classify_tiles,  # noqa: F401
                    TILE_SKIP, TILE_PARTIAL, TILE_FULL)
