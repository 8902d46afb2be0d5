"""B200 (sm_100a) implementation of the NAtSL token-level hybrid attention hot path.

Python mirrors of the reference's op and layer interfaces over a C-ABI CUDA library:

    from neuralattentionsearchlinear_b200 import nats_mixed_attn_gdn, nats_mixed_attn_mamba
"""
from .nats_util import SelectionTables, build_selection_tables  # noqa: F401
from .mixed_attn_gdn import (  # noqa: F401
    nats_mixed_attn_gdn,
    nats_mixed_attn_gdn_chunk_inference,
    nats_mixed_attn_gdn_recurrent,
)
from .mixed_attn_mamba import (  # noqa: F401
    nats_mixed_attn_mamba,
    nats_mixed_attn_mamba_chunk_inference,
    nats_mixed_attn_mamba_recurrent,
)
from .cache import NAtSCache, NAtSLayerCache  # noqa: F401

from .natsl_attn_gdn import NeuralAttentionSearchLinearAttnGDN  # noqa: F401
from .natsl_attn_mamba2 import NeuralAttentionSearchLinearAttnMamba  # noqa: F401

__version__ = "0.1.0"
