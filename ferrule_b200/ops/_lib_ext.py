"""Declarations for the optional entry-point groups of the native library (collectives,
quantised GEMMs, DeepSeek-V4 operators, host runtime).  Each group is declared only if
its symbols are present, so a partial build still loads."""
from __future__ import annotations

import ctypes as C


def _has(lib, name: str) -> bool:
    try:
        getattr(lib, name)
        return True
    except AttributeError:
        return False


def declare(lib) -> None:
    vp, i, ll, f, ull = C.c_void_p, C.c_int, C.c_longlong, C.c_float, C.c_ulonglong
    table = {
        # comm.cu
        "fb_ipc_handle_bytes": ([], i),
        "fb_ipc_alloc": ([C.POINTER(vp), ll, vp], i),
        "fb_ipc_open": ([vp, C.POINTER(vp)], i),
        "fb_ipc_close": ([vp], i),
        "fb_ipc_free": ([vp], i),
        "fb_moe_reduce_allreduce": ([vp, i, i, vp, i, i, vp, ll, vp, ll, i, i, i, i, i, C.POINTER(vp),
                                     C.POINTER(vp), vp, i, ull, vp, vp], i),
        "fb_moe_reduce_allreduce_mc": ([vp, i, i, vp, i, i, vp, ll, vp, ll, i, i, i, i, i, C.POINTER(vp),
                                        C.POINTER(vp), vp, i, ull, vp, vp, vp], i),
        "fb_argmax_allgather": ([vp, vp, i, i, i, i, i, C.POINTER(vp), C.POINTER(vp), vp, ull, vp, vp], i),
        "fb_flag_wait_probe": ([vp, i, ull, vp, vp, vp], i),
        "fb_peer_pingpong": ([vp, vp, i, i, ull, vp, vp, vp], i),
        # elementwise.cu (fused variants)
        "fb_router_plan_fused": ([vp, ll, vp, i, vp, vp, vp, i, i, i, i, i, i, i, f, vp, vp, i, i, i, i,
                                  vp, vp, vp, vp, vp, vp, i, vp, vp, vp, vp, vp], i),
        "fb_argmax_chunked": ([vp, ll, i, i, i, vp, vp, vp, vp, vp, vp], i),
        "fb_router_append": ([vp, ll, vp, i, vp, vp, vp, i, i, i, i, i, i, i, f, vp, vp, i, i, i, i, vp, vp, vp, vp, vp, ll,
                              vp, vp], i),
        "fb_norm_router_append": ([vp, ll, vp, ll, vp, vp, ll, vp, ll, f, vp, i, vp, vp, vp, i, i, i, i, i, i, i, f, vp, vp,
                                   i, i, i, i, vp, vp, vp, vp, vp, ll, vp, vp], i),
        "fb_router_append_q": ([vp, ll, vp, ll, vp, vp, ll, vp, ll, f, vp, i, vp, vp, vp, i, i, i, i, i, i, i, f, vp, vp,
                                i, i, i, i, vp, vp, vp, vp, vp, ll, vp, ll, vp, ll, vp, ll, vp, ll, i, vp, vp], i),
        "fb_moe_reduce_norm": ([vp, i, i, vp, i, i, vp, ll, vp, ll, i, i, vp, vp, ll, f, vp], i),
        "fb_l2_prefetch": ([vp, ll, vp], i),
        "fb_decode_advance": ([vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, vp], i),
        # comm_mm.cu
        "fb_mm_collective": ([vp, ll, i, i, vp, i, i, vp, ll, vp, ll, i, i, i, vp, vp, ll, f, vp, vp, ll, ll, ll, vp, i, i,
                              ull, vp, vp], i),
        # data_movers.cu
        "fb_mv_fill": ([vp, ll, i, i, vp], i),
        "fb_mv_pack_pairs": ([vp, vp, vp, i, vp], i),
        "fb_mv_index_fill": ([vp, ll, i, i, i, i, vp, vp, vp, ll, vp], i),
        "fb_mv_move_rows": ([vp, ll, ll, vp, ll, vp, i, i, i, vp, vp], i),
        "fb_mv_scatter_add": ([vp, ll, i, vp, ll, vp, i, i, vp, vp], i),
        "fb_mv_saxpy": ([vp, vp, f, ll, vp], i),
        "fb_mv_ring_to_logical": ([vp, ll, i, i, i, vp, vp, vp, vp, ll, vp], i),
        "fb_mv_paged_row_scatter": ([vp, ll, i, vp, i, i, i, vp, vp, vp, ll, i, vp, vp], i),
        # quant.cu
        "fb_quant_fp8_rows": ([vp, ll, vp, ll, vp, ll, i, i, i, vp], i),
        "fb_dequant_fp8_block": ([vp, vp, vp, i, i, i, vp], i),
        "fb_quant_mxfp4_rows": ([vp, ll, vp, vp, i, i, vp], i),
        "fb_dequant_mxfp4": ([vp, vp, vp, i, i, vp], i),
        "fb_hadamard_rows": ([vp, ll, i, i, vp], i),
        # expert_table.cu
        "fb_expert_table_apply": ([vp, vp, vp, vp, i, i, i, vp, vp], i),
        "fb_expert_table_resolve": ([vp, vp, vp, i, vp, i, vp, vp], i),
        # v4_ops.cu
        "fb_hc_pre": ([vp, vp, vp, vp, vp, i, vp, i, i, i, i, f, f, i, vp], i),
        "fb_hc_pre_split": ([vp, vp, vp, vp, vp, i, vp, i, i, i, i, f, f, i, i, vp, vp, vp], i),
        "fb_hc_post": ([vp, vp, vp, vp, i, i, i, vp], i),
        "fb_compressor_pool": ([vp, vp, ll, vp, vp, ll, i, i, i, i, i, i, i, vp], i),
        "fb_rope_rows": ([vp, ll, ll, i, i, i, i, vp, vp, vp, i, i, vp, vp], i),
        "fb_indexer_scores": ([vp, vp, ll, vp, vp, ll, i, i, i, i, vp], i),
        "fb_indexer_topk": ([vp, ll, vp, i, i, vp, ll, i, vp], i),
        "fb_indexer_reduce": ([vp, ll, vp, vp, ll, i, i, i, vp], i),
        "fb_markov_step": ([vp, vp, vp, i, i, i, vp, vp, vp, vp, vp, vp, vp, vp], i),
        "fb_hc_mean_scatter": ([vp, vp, ll, i, i, i, i, vp], i),
    }
    for name, (args, res) in table.items():
        if _has(lib, name):
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = res
