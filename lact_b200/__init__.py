"""lact_b200: B200 (sm_100a) kernels for LaCT's large-chunk fast-weight TTT step, behind the
reference's own Python call signatures.  Importing the package does not load the CUDA library;
the first op does, and fails loudly if it has not been built (`python -m lact_b200.build`)."""
from .ops import (  # noqa: F401
    ar_fast_weight_swish_glu_weight_norm_mini_batch,
    ar_fast_weight_swish_glu_weight_norm_mini_batch_inference,
    ar_fast_weight_swish_glu_weight_norm_mini_batch_inference_with_momentum,
    ar_fast_weight_swish_glu_weight_norm_mini_batch_with_momentum,
    bidirectional_lact_swiglu,
    block_causal_lact_swiglu,
    bmm_bf16,
    fast_weight_swish_glu_weight_norm_mini_batch_apply,
    fused_lact_swiglu_ffn_fast_weight_grads,
    fused_prenorm_update_with_momentum_and_l2_norm,
    fused_swiglu_ffn_fwd,
    l2_norm,
    l2_norm_add_fused,
    minimal_block_causal_lact_swiglu,
    postnorm_block_causal_lact_swiglu_fused_kernel_triton,
    prenorm_block_causal_lact_swiglu,
    prenorm_block_causal_lact_swiglu_fused_kernel_triton,
    scan,
    zeropower_via_newtonschulz5,
)
from .program import TTTOperator  # noqa: F401
from ._lib import LactError, synchronize_and_check  # noqa: F401
