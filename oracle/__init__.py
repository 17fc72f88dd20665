"""CPU oracle for the OmniKV decode-time selection path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package may import this
package: it is the checker that the CUDA path is compared against (tests, the
smoke check and the CPU-baseline leg of the benchmark), never the thing that
is shipped or measured as the product.

Parity status: the selector, the layer plan and the cache flow are PINNED --
``tests/golden/make_golden.py`` runs the reference's own
``select_tokens_by_attn_universal``, ``OmniKVMultiStageCache`` and
``WOPackCache`` (and ``OmniKVLazyCache.set_out_idx`` for the lazy re-gather rule) on seeded inputs and the committed fixtures hold their
outputs; ``tests/test_oracle_golden.py`` checks this restatement against
them.  The attention arithmetic itself (softmax(q K^T / sqrt(d)) V) and the
decoder wrapper are third-party code in the reference (transformers 4.41.2,
flash-attn), absent from its tree: there the oracle is the mathematical
definition in fp32 and parity is UNPINNED.
"""
from .omnikv_oracle import (  # noqa: F401
    apply_rope,
    dense_attention,
    layer_plan,
    rope_cos_sin,
    score_last,
    score_window,
    select_tokens_by_attn_universal,
    selector_k_rule,
    sparse_attention,
    topk_ascending,
    OracleMultiStageCache,
    OracleWOPackCache,
    OracleLazyRule,
    OracleLazyMultiStageCache,
    idx_iou_score,
)
