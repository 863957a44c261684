from ._ffi import KernelError
from .basic import (PAGE, embed, add_rmsnorm, rope_kv_write, swiglu, gemm_simt, split_k_for_simt, attention_generic, argmax, sample, set_sample_cached, advance_decode, gather_tokens,
                    attention_decode, attention_decode_supported, attention_decode_scratch, DECODE_CHUNK,
                    attention_prefill, attention_prefill_supported, PREFILL_TILE,
                    attention_decode_warps, decode_splits, decode_pages,
                    attention_prefill_tc, attention_prefill_tc_supported, PREFILL_TC_TILE)
from .basic import (relu2, add_row, branch_norm_add, head_norm_kv_write, gemm_simt_grouped, retention_prepare,
                    retention_scan, retention_gate, retention_chunked, RETENTION_CHUNK, moe_route, moe_sort, moe_combine, moe_gather, MOE_TILE_SMALL, MOE_TILE_LARGE, MOE_TILE_TC)
from .basic import (embed_positions, round_rows, clamped_glu, sigmoid_gate, key_span, gla_prepare, gla_scan, MOE_SCORINGS)
from .basic import (dyt_rows, scaled_add, softcap_, gated_scan, gated_chunked, mlstm_prepare, mlstm_gates, conv_silu, mamba_gates, mamba_finish)
from .basic import (weighted_add, stretch_norm, delta_prepare, delta_scan)
from ._ffi import launch_count
from . import tensor_core
