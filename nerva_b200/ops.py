"""Per-operator entry points of libnerva_b200.so (host buffers in, host buffers out)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import ffi


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed: {ffi.last_error() or 'rejected arguments'}")


def projection(weight_bits: np.ndarray, x_bits: np.ndarray, rows: int, cols: int, tokens: int = 1,
               warmup: int = 0, iterations: int = 1):
    """y[m][n] = sum_k W[n][k] x[m][k]; bf16 bits in, fp32 out.  Returns (y, avg_ns)."""
    w = np.ascontiguousarray(weight_bits, dtype=np.uint16)
    x = np.ascontiguousarray(x_bits, dtype=np.uint16)
    assert w.size == rows * cols and x.size == tokens * cols
    y = np.empty((tokens, rows), dtype=np.float32)
    ns = C.c_uint64(0)
    _check(ffi.lib().nerva_b200_projection(w.ctypes.data, x.ctypes.data, y.ctypes.data, rows, cols, tokens,
                                           warmup, iterations, C.byref(ns)), "projection")
    return y, ns.value


def projection_sustained(weight_bits: np.ndarray, x_bits: np.ndarray, rows: int, cols: int, tokens: int = 1,
                         copies: int = 2, warmup: int = 4, iterations: int = 20):
    """The same projection over `copies` device copies of the matrix (together larger than the L2),
    launched back to back with programmatic dependent launch.  Returns (y, ns per launch)."""
    w = np.ascontiguousarray(weight_bits, dtype=np.uint16)
    x = np.ascontiguousarray(x_bits, dtype=np.uint16)
    assert w.size == rows * cols and x.size == tokens * cols
    y = np.empty((tokens, rows), dtype=np.float32)
    ns = C.c_uint64(0)
    _check(ffi.lib().nerva_b200_projection_sustained(w.ctypes.data, x.ctypes.data, y.ctypes.data, rows, cols, tokens,
                                                     copies, warmup, iterations, C.byref(ns)), "projection_sustained")
    return y, ns.value


def gqa_decode_attention(q: np.ndarray, key_pages: np.ndarray, value_pages: np.ndarray, page_table: np.ndarray,
                         batch: int, context: int, heads: int, kv_heads: int, head_dim: int,
                         warmup: int = 0, iterations: int = 1):
    """Paged GQA decode attention for `batch` sequences.  Returns (out f32 [batch, heads*d], avg_ns)."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    k = np.ascontiguousarray(key_pages, dtype=np.uint16)
    v = np.ascontiguousarray(value_pages, dtype=np.uint16)
    t = np.ascontiguousarray(page_table, dtype=np.uint32)
    pages = (context + 15) // 16
    assert q.size == batch * heads * head_dim
    assert k.size == v.size == batch * pages * 16 * kv_heads * head_dim and t.size == batch * pages
    out = np.empty((batch, heads * head_dim), dtype=np.float32)
    ns = C.c_uint64(0)
    _check(ffi.lib().nerva_b200_gqa_decode_attention(q.ctypes.data, k.ctypes.data, v.ctypes.data, t.ctypes.data,
                                                     out.ctypes.data, batch, context, heads, kv_heads, head_dim,
                                                     warmup, iterations, C.byref(ns)), "gqa_decode_attention")
    return out, ns.value


def gqa_decode_attention_sustained(q: np.ndarray, key_pages: np.ndarray, value_pages: np.ndarray,
                                   page_table: np.ndarray, batch: int, context: int, heads: int, kv_heads: int,
                                   head_dim: int, copies: int = 2, warmup: int = 4, iterations: int = 20):
    """The same attention over `copies` device copies of the cache (the caches of that many layers,
    together larger than the L2), launched back to back.  Returns (out, ns per launch)."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    k = np.ascontiguousarray(key_pages, dtype=np.uint16)
    v = np.ascontiguousarray(value_pages, dtype=np.uint16)
    t = np.ascontiguousarray(page_table, dtype=np.uint32)
    out = np.empty((batch, heads * head_dim), dtype=np.float32)
    ns = C.c_uint64(0)
    _check(ffi.lib().nerva_b200_gqa_decode_attention_sustained(
        q.ctypes.data, k.ctypes.data, v.ctypes.data, t.ctypes.data, out.ctypes.data, batch, context, heads, kv_heads,
        head_dim, copies, warmup, iterations, C.byref(ns)), "gqa_decode_attention_sustained")
    return out, ns.value


def gqa_decode_attention_static_scratch(q_ptr: int, key_pages_ptr: int, value_pages_ptr: int, page_table_ptr: int,
                                        out_ptr: int, batch: int, context: int, heads: int, kv_heads: int,
                                        head_dim: int, stream: int = 0) -> None:
    """The same attention on DEVICE addresses, with the split partials in the library's fixed
    device array: the call allocates nothing and returns when `stream` has finished the work.
    Calls on one device share that array; do not overlap them."""
    _check(ffi.lib().nerva_b200_gqa_decode_attention_static_scratch(
        q_ptr, key_pages_ptr, value_pages_ptr, page_table_ptr, out_ptr, batch, context, heads, kv_heads,
        head_dim, stream), "gqa_decode_attention_static_scratch")


def greedy_argmax(logits: np.ndarray) -> int:
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    token = C.c_uint32(0)
    _check(ffi.lib().nerva_b200_greedy_argmax(logits.ctypes.data, logits.size, C.byref(token)), "greedy_argmax")
    return token.value


def sample_token(logits: np.ndarray, position: int, temperature: float, top_p: float, top_k: int, seed: int) -> int:
    """One token with the decode step's seeded temperature / top-k / top-p sampler."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    token = C.c_uint32(0)
    _check(ffi.lib().nerva_b200_sample_token(logits.ctypes.data, logits.size, position, temperature, top_p, top_k,
                                             seed, C.byref(token)), "sample_token")
    return token.value


def projection_bench(rows: int, cols: int, iterations: int = 20, warmup: int = 5, block_tokens: int = 0,
                     dtype: int = 1):
    req = ffi.ProjectionBenchRequest(dtype=dtype, rows=rows, cols=cols, iterations=iterations,
                                     warmup_iterations=warmup, block_tokens=block_tokens)
    out = ffi.ProjectionBenchResult()
    rc = ffi.lib().nerva_cuda_projection_bench(C.byref(req), C.byref(out))
    return rc, out


ROUTER_V3_GROUPED_SIGMOID, ROUTER_V4_SQRTSOFTPLUS, ROUTER_V4_HASH = 1, 2, 3


def deepseek_router_route(kind: int, logits, top_k: int, bias=None, num_groups: int = 0, top_k_groups: int = 0,
                          norm_topk_prob: bool = True, routed_scaling_factor: float = 1.0, hash_route_table=None,
                          route_token: int = 0):
    """Expert ids and weights of one token (reference: deepseek_router_route_* of
    crates/nerva-cuda/src/deepseek/router.rs).  Returns (return code, ids, weights, result struct)."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    bias_arr = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    table = None if hash_route_table is None else np.ascontiguousarray(hash_route_table, dtype=np.uint32)
    ids = np.zeros(top_k, dtype=np.uint32)
    weights = np.zeros(top_k, dtype=np.float32)
    req = ffi.structs["NervaCudaDeepSeekRouterRouteRequest"](
        router_kind=kind, num_experts=logits.size, num_groups=num_groups, top_k_groups=top_k_groups, top_k=top_k,
        norm_topk_prob=int(norm_topk_prob), route_token=route_token, routed_scaling_factor=routed_scaling_factor,
        logits=logits.ctypes.data, correction_bias=None if bias_arr is None else bias_arr.ctypes.data,
        hash_route_table=None if table is None else table.ctypes.data,
        hash_route_table_len=0 if table is None else table.size, expert_ids=ids.ctypes.data,
        weights=weights.ctypes.data)
    out = ffi.structs["NervaCudaDeepSeekRouterRouteResult"]()
    rc = ffi.lib().nerva_cuda_deepseek_router_route(C.byref(req), C.byref(out))
    return rc, ids, weights, out


def deepseek_mla_decode(q_nope, q_pe, kv_c, k_pe, w_uk, w_uv, heads: int, tokens: int, kv_lora_rank: int,
                        qk_nope_head_dim: int, qk_rope_head_dim: int, v_head_dim: int, softmax_scale: float):
    """Absorbed multi-head latent attention decode of one token (fp32 host arrays).
    Returns (return code, out [heads * v_head_dim], result struct)."""
    arrays = [np.ascontiguousarray(a, dtype=np.float32) for a in (q_nope, q_pe, kv_c, k_pe, w_uk, w_uv)]
    out_values = np.zeros(heads * v_head_dim, dtype=np.float32)
    req = ffi.structs["NervaCudaDeepSeekMlaDecodeRequest"](
        heads=heads, tokens=tokens, kv_lora_rank=kv_lora_rank, qk_nope_head_dim=qk_nope_head_dim,
        qk_rope_head_dim=qk_rope_head_dim, v_head_dim=v_head_dim, softmax_scale=softmax_scale,
        q_nope=arrays[0].ctypes.data, q_pe=arrays[1].ctypes.data, kv_c=arrays[2].ctypes.data,
        k_pe=arrays[3].ctypes.data, w_uk=arrays[4].ctypes.data, w_uv=arrays[5].ctypes.data,
        output=out_values.ctypes.data)
    out = ffi.structs["NervaCudaDeepSeekMlaDecodeResult"]()
    rc = ffi.lib().nerva_cuda_deepseek_mla_decode(C.byref(req), C.byref(out))
    return rc, out_values, out


def deepseek_moe_forward(x, expert_ids, expert_weights, w_gate, w_up, w_down, hidden: int, intermediate: int,
                         num_experts: int, clamp_swiglu: bool = False, swiglu_limit: float = 0.0):
    """fp32 expert MLP of one token over already routed experts.  Returns (return code, out, result)."""
    x, w_gate, w_up, w_down, ew = [np.ascontiguousarray(a, dtype=np.float32)
                                   for a in (x, w_gate, w_up, w_down, expert_weights)]
    ids = np.ascontiguousarray(expert_ids, dtype=np.uint32)
    out_values = np.zeros(hidden, dtype=np.float32)
    req = ffi.structs["NervaCudaDeepSeekMoeForwardRequest"](
        hidden_size=hidden, intermediate_size=intermediate, num_experts=num_experts, top_k=ids.size,
        clamp_swiglu=int(clamp_swiglu), swiglu_limit=swiglu_limit, input=x.ctypes.data, expert_ids=ids.ctypes.data,
        expert_weights=ew.ctypes.data, w_gate=w_gate.ctypes.data, w_up=w_up.ctypes.data, w_down=w_down.ctypes.data,
        output=out_values.ctypes.data)
    out = ffi.structs["NervaCudaDeepSeekMoeForwardResult"]()
    rc = ffi.lib().nerva_cuda_deepseek_moe_forward(C.byref(req), C.byref(out))
    return rc, out_values, out


def synth_normal_bf16(seed: int, tensor_id: int, count: int, std: float) -> np.ndarray:
    """Multi-threaded native twin of nerva_b200.synth.normal_bf16 (same bits)."""
    out = np.empty(count, dtype=np.uint16)
    ffi.lib().nerva_b200_synth_normal_bf16(seed, tensor_id, count, std, out.ctypes.data)
    return out


def synth_normal_bf16_block(seed: int, tensor_id: int, full_cols: int, row_begin: int, rows: int, col_begin: int,
                            cols: int, std: float) -> np.ndarray:
    """rows x cols block of the generator's row-major tensor with full_cols columns (flattened)."""
    out = np.empty(rows * cols, dtype=np.uint16)
    ffi.lib().nerva_b200_synth_normal_bf16_block(seed, tensor_id, full_cols, row_begin, rows, col_begin, cols, std,
                                                 out.ctypes.data)
    return out


def plan_layout(cfg, layers, layer_index: int = 0):
    req = ffi.LayoutPlanRequest(hidden=cfg.hidden, heads=cfg.heads, kv_heads=cfg.kv_heads, head_dim=cfg.head_dim,
                                intermediate=cfg.intermediate, vocab_size=cfg.vocab, layer_count=cfg.layers,
                                layer_index=layer_index, layers=C.cast(layers, C.c_void_p))
    out = ffi.LayoutPlanResult()
    rc = ffi.lib().nerva_cuda_hf_decode_sequence_plan_layout(C.byref(req), C.byref(out))
    return rc, out
