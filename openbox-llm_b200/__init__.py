"""NSA attention hot path of openbox-llm on B200: C-ABI CUDA library + reference-shaped host API."""
from ._lib import LIB_PATH, NsaError, lib  # noqa: F401
from .ops import (MODE_COMPRESS, MODE_COMPRESS_STRIDED, MODE_WINDOW, SelectionAttnTriton, _RangeAttn,  # noqa: F401
                  block_compress, block_mean_pool, build_block_to_query_csr,
                  compression_attn_triton, gate_combine, get_dq_accumulator, get_impl, nsa_attention,
                  nsa_fused_forward, range_attn_backward, range_attn_forward,
                  select_blocks, selection_attn_triton, selection_backward_triton, selection_forward_triton,
                  set_dq_accumulator, set_impl, set_option, tc_supported, topn_blocks, window_attn_triton)
